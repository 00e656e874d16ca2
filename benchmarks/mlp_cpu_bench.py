"""MLP classifier on CPU, single process, fp32 (BASELINE config 1): 784 -> 256 -> 128 -> 10 with ReLU, batch 64, inputs
N(0,1), labels uniform in [0, 10), cross-entropy, Adam lr 1e-3, 100 steps, seed 0, Kaiming-uniform init.

  python benchmarks/mlp_cpu_bench.py [--steps 100] [--warmup 3] [--impl ours|library]

Runs through the framework's public Python-binding surface (``rustorch.Linear / ReLU / CrossEntropyLoss / Adam``) and
prints one JSON line: steps/s and the final loss.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "library"], help="library: the same model from stock torch.nn / torch.optim")
    a = ap.parse_args()
    if a.impl == "ours":
        import rustorch as rt
        rt.set_seed(0)
        model = rt.Sequential(rt.Linear(784, 256), rt.ReLU(), rt.Linear(256, 128), rt.ReLU(), rt.Linear(128, 10))
        opt = rt.Adam(model.parameters(), lr=1e-3)
        loss_fn = rt.CrossEntropyLoss()
    else:
        torch.manual_seed(0)
        nn = torch.nn
        model = nn.Sequential(nn.Linear(784, 256), nn.ReLU(), nn.Linear(256, 128), nn.ReLU(), nn.Linear(128, 10))
        opt = torch.optim.Adam(model.parameters(), lr=1e-3)
        loss_fn = nn.CrossEntropyLoss()
    g = torch.Generator().manual_seed(0)
    x = torch.randn(64, 784, generator=g)
    y = torch.randint(0, 10, (64,), generator=g)

    def step():
        opt.zero_grad()
        loss = loss_fn(model(x), y)
        loss.backward()
        opt.step()
        return float(loss.detach())

    first = step()
    for _ in range(a.warmup - 1):
        step()
    t0 = time.perf_counter()
    for _ in range(a.steps):
        last = step()
    dt = time.perf_counter() - t0
    print(json.dumps({"metric": "mlp_cpu_steps_per_s", "value": round(a.steps / dt, 1), "unit": "steps/s", "steps": a.steps,
                      "ms_per_step": round(dt / a.steps * 1e3, 4), "first_loss": round(first, 4), "final_loss": round(last, 4),
                      "dtype": "fp32", "device": "cpu", "impl": a.impl, "threads": torch.get_num_threads(),
                      "config": "MLP 784-256-128-10 ReLU, batch 64, Adam lr 1e-3, seed 0"}))


if __name__ == "__main__":
    main()
