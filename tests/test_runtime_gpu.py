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


def test_bounded_device_wait_expires_and_context_survives():
    """A device-side wait on a flag that nothing sets gives up after its limit: the kernel returns, the status word
    holds the peer-timeout code, ``check_status`` raises ``KernelTimeout`` and clears the word, and the next launch on
    the same context works.  Nothing faults or hangs; the limit is a few milliseconds.  (The reference's barrier
    returns an error after its timeout the same way, src/gpu/sync_primitives.rs:109-158.)"""
    import time
    from rustorch_b200 import _native
    from rustorch_b200.error import KernelTimeout
    C = _native.load(required=True)
    _native.check_status()
    # two "ranks" whose end-of-step flags both live on this GPU; rank 0 waits for rank 1's flag of epoch 1
    flags = torch.zeros(64, dtype=torch.int32, device="cuda")
    t0 = time.perf_counter()
    C.ddp_wait_end(flags.data_ptr(), 1, 2, 0, 1, 0.005, torch.cuda.current_device())
    torch.cuda.synchronize()
    assert time.perf_counter() - t0 < 2.0
    assert int(C.read_status(torch.cuda.current_device())) == 104
    # the word is cleared by the read; arm it again to see the Python exception
    C.ddp_wait_end(flags.data_ptr(), 1, 2, 0, 1, 0.005, torch.cuda.current_device())
    with pytest.raises(KernelTimeout):
        _native.check_status()
    _native.check_status()                      # cleared
    # the flag set: the same wait returns at once, and ordinary kernels still run on this context
    flags[1] = 1
    C.ddp_wait_end(flags.data_ptr(), 1, 2, 0, 1, 0.005, torch.cuda.current_device())
    _native.check_status()
    from rustorch_b200.ops import kernels as K
    a = torch.randn(256, 128, device="cuda").bfloat16()
    b = torch.randn(192, 128, device="cuda").bfloat16()
    out = K.gemm(a, b)
    assert torch.allclose(out.float(), a.float() @ b.float().T, atol=0.5, rtol=5e-2)
    _native.check_status()


def test_bucket_step_wait_expires_and_counter_rearms():
    """The fused data-parallel bucket kernel launched as rank 0 of 2 with both ranks' buffers on this GPU and no peer
    to raise the start flag: every CTA's wait runs out, the update is skipped, the completion counter still returns
    to zero, and a world-size-1 launch afterwards updates the parameters."""
    from rustorch_b200 import _native
    from rustorch_b200.error import KernelTimeout
    C = _native.load(required=True)
    _native.check_status()
    n = 4096
    grad = torch.ones(n, device="cuda")
    lp = torch.zeros(n, dtype=torch.bfloat16, device="cuda")
    flags = torch.zeros(64, dtype=torch.int32, device="cuda")
    master, m, v = torch.ones(n, device="cuda"), torch.zeros(n, device="cuda"), torch.zeros(n, device="cuda")
    done = torch.zeros(1, dtype=torch.int32, device="cuda")
    gp, lpp, fp = [grad.data_ptr()] * 2, [lp.data_ptr()] * 2, [flags.data_ptr()] * 2
    C.ddp_bucket_step(gp, lpp, fp, master, m, v, done, 0, n // 2, 0, 1, 0, 2, 0.005, 0.1, 0.9, 0.999, 1e-8, 0.0,
                      0.1, 0.001, 0.5, 8, 0, False, True, 0, 0)
    with pytest.raises(KernelTimeout):
        _native.check_status()
    assert int(done.item()) == 0                       # re-armed although every CTA timed out
    assert float(master.min()) == 1.0 and float(grad.min()) == 1.0   # update skipped
    C.ddp_bucket_step(gp[:1], lpp[:1], fp[:1], master, m, v, done, 0, n, 0, 2, 0, 2, 0.005, 0.1, 0.9, 0.999, 1e-8,
                      0.0, 0.1, 0.001, 1.0, 8, 0, False, True, 0, 0)
    _native.check_status()
    assert float(master.max()) < 1.0 and float(grad.abs().max()) == 0.0
    assert torch.equal(lp.float(), master.bfloat16().float())
