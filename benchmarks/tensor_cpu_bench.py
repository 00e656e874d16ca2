"""CPU micro-benchmarks of the tensor / autograd / linalg façade against the figures the reference publishes
(docs/guides/performance.md:30-59, README.md:300-312, docs/reports/benchmarks.md:21-74 of the reference).

  python benchmarks/tensor_cpu_bench.py

Wall clock (``time.perf_counter``), best of 5 batches; one JSON line per measurement with the published value beside
it where the reference has one.  Runs through ``rustorch_b200.Tensor`` / ``Variable`` and the package's layers.
"""
from __future__ import annotations

import json
import os
import sys
import time

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def best_time(fn, inner: int, batches: int = 5) -> float:
    fn()
    best = float("inf")
    for _ in range(batches):
        t0 = time.perf_counter()
        for _ in range(inner):
            fn()
        best = min(best, (time.perf_counter() - t0) / inner)
    return best


def emit(name: str, seconds: float, published=None, unit: str = "us", **extra):
    out = {"bench": name, "time_us": round(seconds * 1e6, 3)}
    out.update(extra)
    if published is not None:
        out["published"] = published
        out["published_unit"] = unit
    print(json.dumps(out), flush=True)


def main():
    import rustorch_b200 as rt
    from rustorch_b200 import distributions, nn
    torch.manual_seed(0)
    T = rt.Tensor

    # tensor creation / elementwise / reductions (docs/reports/benchmarks.md:21-25)
    emit("tensor_create_1000", best_time(lambda: T.zeros([1000]), 2000), 0.076)
    emit("tensor_create_1000x1000", best_time(lambda: T.zeros([1000, 1000]), 50), 147.2)
    a, b = T.randn([100, 100]), T.randn([100, 100])
    emit("add_100x100", best_time(lambda: a + b, 2000), 29.4)
    emit("matmul_100x100", best_time(lambda: a.matmul(b), 1000), 1030.0)
    emit("transpose_100x100", best_time(lambda: a.transpose(), 5000), 5.81)
    big = T.randn([1000, 1000])
    s = best_time(lambda: big.sum(), 200)
    emit("sum_1000x1000", s, None, elements_per_s=round(1e6 / s))

    # matmul GFLOPS (docs/guides/performance.md:56-59: 0.71-0.77 GFLOPS)
    for n in (64, 128, 256, 512):
        x, y = T.randn([n, n]), T.randn([n, n])
        t = best_time(lambda: x.matmul(y), max(5, 20000 // n))
        emit(f"matmul_{n}x{n}", t, {64: 0.77, 128: 0.76, 256: 0.76, 512: 0.71}[n], unit="GFLOPS", gflops=round(2 * n ** 3 / t / 1e9, 2))

    # autograd (docs/reports/benchmarks.md:33-37)
    def backward_small():
        v = rt.Variable(torch.randn(10, 10), requires_grad=True)
        (v * v).sum().backward()
    emit("variable_backward_10x10", best_time(backward_small, 1000), 1.94)

    def backward_matmul():
        v = rt.Variable(torch.randn(100, 100), requires_grad=True)
        w = rt.Variable(torch.randn(100, 100), requires_grad=True)
        v.matmul(w).sum().backward()
    emit("matmul_grad_100x100", best_time(backward_matmul, 300), 1060.0)

    # linear algebra (docs/guides/performance.md:41-43; docs/reports/benchmarks.md:53-56)
    for n, pub in ((4, (100.0, 6.0, 67.0)), (8, (1000.0, 24.0, 165.0)), (16, (7000.0, 107.0, 473.0))):
        m = T.randn([n, n])
        sym = m + m.transpose()
        emit(f"svd_{n}x{n}", best_time(lambda: m.svd(), 300), pub[0])
        emit(f"qr_{n}x{n}", best_time(lambda: m.qr(), 300), pub[1])
        emit(f"eigh_{n}x{n}", best_time(lambda: sym.eigh(), 300), pub[2])
    m64 = T.randn([64, 64])
    emit("svd_64x64", best_time(lambda: m64.svd(), 20), 76800.0)

    # FFT 8-64 samples (README.md:310: 10-312 us)
    for n, pub in ((8, 10.0), (64, 312.0)):
        sig = T.randn([n])
        emit(f"fft_{n}", best_time(lambda: sig.fft(), 2000), pub)

    # distributions (docs/reports/benchmarks.md:70-74)
    normal = distributions.Normal(torch.tensor(0.0), torch.tensor(1.0))
    emit("normal_sample_100", best_time(lambda: normal.sample([100]), 2000), 1.12)
    emit("normal_sample_10000", best_time(lambda: normal.sample([10000]), 500), 100.0)
    xs = torch.randn(100)
    emit("normal_log_prob_100", best_time(lambda: normal.log_prob(xs), 2000), 0.315)

    # layer construction (docs/reports/benchmarks.md:43-46) and inference (docs/guides/performance.md:56-58)
    emit("conv2d_layer_create", best_time(lambda: nn.Conv2d(16, 32, 3), 200), 573.5)
    emit("conv1d_layer_create", best_time(lambda: nn.Conv1d(16, 32, 3), 200), 161.3)
    net = nn.Sequential(nn.Linear(784, 256), nn.ReLU(), nn.Linear(256, 128), nn.ReLU(), nn.Linear(128, 10))
    for bs, pub in ((32, 59.86), (64, 29.35), (128, 15.09)):
        inp = torch.randn(bs, 784)
        with torch.no_grad():
            t = best_time(lambda: net(inp), 300)
        emit(f"nn_inference_batch{bs}", t, pub, unit="inferences/s", inferences_per_s=round(1.0 / t, 1))


if __name__ == "__main__":
    main()
