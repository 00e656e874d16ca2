"""GPU tests of the runtime layer: custom kernels through the driver API, CUDA-graph replay engine, device pool."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_custom_kernel_compile_and_launch(tmp_path):
    from rustorch_b200 import gpu as G
    mgr = G.CustomKernelManager(G.DeviceType.Cuda(0), cache_dir=str(tmp_path))
    cfg = G.KernelConfig("saxpy", 'extern "C" __global__ void saxpy(float* y, const float* x, long long n, float a)'
                                  "{ long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; if (i < n) y[i] += a * x[i]; }")
    n = 100003
    x, y = torch.randn(n, device="cuda"), torch.randn(n, device="cuda")
    ref = y + 2.5 * x
    mgr.execute_kernel(cfg, ((n + 255) // 256, 1, 1), [y, x, n, 2.5])
    torch.cuda.synchronize()
    assert torch.allclose(y, ref, atol=1e-6) and mgr.get_kernel_stats("saxpy").launches == 1


def test_runtime_engine_replays_cuda_graph():
    from rustorch_b200 import execution as E
    eng = E.RuntimeEngine(use_cuda_graphs=True, warmup_runs=1)
    f = lambda a, b: torch.relu(a @ b) + 1
    a, b = torch.randn(64, 64, device="cuda"), torch.randn(64, 64, device="cuda")
    outs = []
    for i in range(4):
        ai = a + i
        outs.append((eng.execute("f", f, ai, b).clone(), f(ai, b)))
    assert all(torch.allclose(o, r, atol=1e-4) for o, r in outs) and eng.metrics.graph_replays >= 2


def test_device_pool_and_validator_on_gpu():
    from rustorch_b200 import gpu as G
    pool = G.GpuMemoryPool(G.DeviceType.Cuda(0), 1 << 24)
    t = pool.zeros((1024, 1024), torch.bfloat16)
    assert t.is_cuda and t.data_ptr() % 256 == 0 and pool.stats()["in_use"] == 2 << 20
    pool.deallocate(t)
    res = G.GpuValidator(1e-4).validate_all_devices()
    assert all(r.passed for r in res), G.GpuValidator().generate_report(res)
    ctx = G.GpuContext(G.DeviceType.Cuda(0), pool_bytes=1 << 20)
    assert ctx.stream_count() == 4 and ctx.properties()["sms"] > 0
