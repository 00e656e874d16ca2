"""Data validation and debugging tools: rule-based validation with a quality grade, outlier detection, streaming drift
detection, structured logging with alert rules, allocation tracking and the debug report."""
import _path  # noqa: F401
import os
import tempfile

import torch

from rustorch_b200 import debug, validation as V

torch.manual_seed(0)
fw = V.DataValidationFramework()
fw.engine.add_rule(V.range_rule(-5, 5)).add_rule(V.shape_rule([None, 4]))
good = torch.randn(200, 4).clamp(-4, 4)
res = fw.validate_tensor(good, valid_range=(-5, 5))
print("clean batch: passed", res.passed, " grade", V.QualityMetrics.grade(res.metrics["score"]))
bad = good.clone()
bad[0, 0], bad[1, 1] = float("nan"), 100.0
r2 = fw.validate_tensor(bad)
print("dirty batch: passed", r2.passed, " rules hit:", sorted({i.rule for i in r2.issues}))
print(fw.validate_tensor(bad, fmt="markdown").splitlines()[0])
x = torch.cat([torch.randn(1000), torch.tensor([40.0])])
det = V.AnomalyDetector()
print("outliers by z-score:", det.zscore(x).tolist(), " by IQR (count):", len(det.iqr(x).tolist()))
stream = V.RealTimeValidator()
for _ in range(20):
    stream.feed(torch.randn(256))
print("drift detected after a mean shift:", any(i.rule == "drift" for i in stream.feed(torch.randn(256) + 5).issues))

log = os.path.join(tempfile.mkdtemp(), "log.jsonl")
f = debug.DebugFramework(level="info", file=log, json_format=True)
f.log("info", "train", "step done", step=3, loss=0.41)
f.log("error", "cuda", "out of memory while allocating 2 GiB")
f.analyzer.add_pattern("oom", r"out of memory")
with f.profile("forward"):
    torch.randn(256, 256) @ torch.randn(256, 256)
h = f.track_allocation(300 << 20, "activations")
rep = f.generate_debug_report()
print("log lines:", sum(1 for _ in open(log)), " counts:", rep["log_counts"], " large allocations:", [a["tag"] for a in rep["memory"]["large"]])
f.memory.track_deallocation(h)
print("profile:", {k: v["calls"] for k, v in rep["profile"].items()}, " tensor summary:", debug.DebugUtils.tensor_summary(torch.tensor([1.0, float("nan")])))
