"""Custom GPU kernels: CUDA C compiled at run time (NVRTC) for the device at hand and launched on torch tensors, and a
fixed-shape function replayed as a CUDA graph.  Needs a CUDA device; without one it says so and stops."""
import _path  # noqa: F401
import sys

import torch

if not torch.cuda.is_available():
    print("no CUDA device: this example needs one")
    sys.exit(0)

from rustorch_b200 import execution as E, gpu as G

mgr = G.CustomKernelManager(G.DeviceType.Cuda(0))
cfg = G.KernelConfig("saxpy", 'extern "C" __global__ void saxpy(float* y, const float* x, long long n, float a)'
                              "{ long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; if (i < n) y[i] += a * x[i]; }")
n = 1 << 20
x, y = torch.randn(n, device="cuda"), torch.randn(n, device="cuda")
ref = y + 2.5 * x
mgr.execute_kernel(cfg, ((n + 255) // 256, 1, 1), [y, x, n, 2.5])
torch.cuda.synchronize()
print("saxpy kernel: max error %.2e, launches %d" % (float((y - ref).abs().max()), mgr.get_kernel_stats("saxpy").launches))
eng = E.RuntimeEngine(use_cuda_graphs=True, warmup_runs=1)
f = lambda a, b: torch.relu(a @ b) + 1      # noqa: E731
a, b = torch.randn(256, 256, device="cuda"), torch.randn(256, 256, device="cuda")
for i in range(5):
    out = eng.execute("f", f, a + i, b)
print("graph replays:", eng.metrics.graph_replays, " result matches eager:", bool(torch.allclose(out, f(a + 4, b), atol=1e-3)))
