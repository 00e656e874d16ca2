"""Optimizer step throughput on the CPU, the one family of numbers the reference publishes for its optimizers
(README.md:300-302, docs/guides/performance.md:15-18: Adamax 33 632, RAdam 21 939 / 28 891, NAdam 18 976 / 30 245,
L-BFGS 15 678 steps/s).  Same protocol as its quick benchmark (src/optim/benchmarks.rs:348-376): one parameter tensor
of 1000 elements, synthetic gradients, 10 warm-up steps, 100 timed steps, lr 1e-3.

    python benchmarks/optimizer_cpu_bench.py [--numel 1000] [--steps 100] [--repeats 5]
"""
import argparse
import json
import os
import sys
import time

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from rustorch_b200 import optim  # noqa: E402

PUBLISHED = {"Adamax": 33632.0, "RAdam": 28891.0, "NAdam": 30245.0, "LBFGS": 15678.0}


def run(name: str, numel: int, steps: int, warmup: int) -> float:
    torch.manual_seed(0)
    p = torch.nn.Parameter(torch.randn(numel))
    cls = getattr(optim, name)
    opt = cls([p], lr=1e-3)
    grads = [torch.randn(numel) * 0.01 for _ in range(16)]

    data = p.data

    def one(i):                          # the reference's call: step(&param, &grad)
        opt.step_tensor(data, grads[i % 16])

    for i in range(warmup):
        one(i)
    t0 = time.perf_counter()
    for i in range(steps):
        one(i)
    return steps / (time.perf_counter() - t0)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--numel", type=int, default=1000)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--repeats", type=int, default=5)
    a = ap.parse_args()
    torch.set_num_threads(1)
    for name in ("Adamax", "RAdam", "NAdam", "LBFGS", "Adam", "AdamW", "SGD"):
        best = max(run(name, a.numel, a.steps, a.warmup) for _ in range(a.repeats))
        out = {"optimizer": name, "steps_per_s": round(best, 1), "numel": a.numel, "steps": a.steps, "device": "cpu"}
        if name in PUBLISHED:
            out["published_steps_per_s"] = PUBLISHED[name]
            out["vs_published"] = round(best / PUBLISHED[name], 2)
        print(json.dumps(out), flush=True)


if __name__ == "__main__":
    main()
