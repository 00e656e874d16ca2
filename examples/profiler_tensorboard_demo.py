"""Profiler report + Chrome trace, and scalars written to a TensorBoard event file."""
import _path  # noqa: F401
import os
import tempfile

import torch

from rustorch_b200 import profiler, tensorboard

profiler.enable_profiler()
with profiler.profile("matmul_chain"):
    a = torch.randn(256, 256)
    for _ in range(10):
        with profiler.profile("matmul"):
            a = torch.tanh(a @ a) * 0.1
profiler.print_profiler_report()
with tempfile.TemporaryDirectory() as d:
    trace = os.path.join(d, "trace.json")
    profiler.export_chrome_trace(trace)
    print("chrome trace bytes:", os.path.getsize(trace))
    w = tensorboard.SummaryWriter(os.path.join(d, "runs"))
    for step in range(20):
        w.add_scalar("loss", 1.0 / (step + 1), step)
    w.close()
    files = [f for _, _, fs in os.walk(os.path.join(d, "runs")) for f in fs]
    print("event files:", files)
profiler.disable_profiler()
