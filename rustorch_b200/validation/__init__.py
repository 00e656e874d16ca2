"""Data validation: rule engine, anomaly detection, consistency checks, quality metrics and reports, streaming
validator (src/validation/mod.rs, core.rs, anomaly_detector.rs, consistency_checker.rs, quality_metrics.rs,
quality_reporter.rs, real_time_validator.rs).  Statistics are computed with tensor ops on the tensor's own
device, so validating a CUDA tensor does not copy it to the host.
"""
from __future__ import annotations

import json
import time
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence

import torch


@dataclass
class ValidationIssue:
    rule: str
    severity: str          # info | warning | error | critical
    message: str


@dataclass
class ValidationResult:
    passed: bool
    issues: List[ValidationIssue] = field(default_factory=list)
    metrics: Dict[str, float] = field(default_factory=dict)


class ValidationRule:
    """A named check ``tensor -> error message or None`` with a severity (src/validation/core.rs)."""

    def __init__(self, name: str, check: Callable[[torch.Tensor], Optional[str]], severity: str = "error"):
        self.name, self.check, self.severity = name, check, severity


def no_nan_rule() -> ValidationRule:
    return ValidationRule("no_nan", lambda t: f"{int(torch.isnan(t).sum())} NaN values" if t.is_floating_point() and bool(torch.isnan(t).any()) else None, "critical")


def finite_rule() -> ValidationRule:
    return ValidationRule("finite", lambda t: "non-finite values" if t.is_floating_point() and not bool(torch.isfinite(t).all()) else None, "critical")


def range_rule(lo: float, hi: float) -> ValidationRule:
    def check(t):
        if t.numel() == 0:
            return None
        mn, mx = float(t.min()), float(t.max())
        return f"values in [{mn:.4g}, {mx:.4g}] outside [{lo}, {hi}]" if mn < lo or mx > hi else None
    return ValidationRule("range", check)


def shape_rule(shape: Sequence[Optional[int]]) -> ValidationRule:
    def check(t):
        ok = t.dim() == len(shape) and all(s is None or s == d for s, d in zip(shape, t.shape))
        return None if ok else f"shape {tuple(t.shape)} does not match schema {tuple(shape)}"
    return ValidationRule("shape", check)


def dtype_rule(dtype: torch.dtype) -> ValidationRule:
    return ValidationRule("dtype", lambda t: None if t.dtype == dtype else f"dtype {t.dtype} != {dtype}")


class ValidationEngine:
    def __init__(self, rules: Optional[List[ValidationRule]] = None):
        self.rules = rules if rules is not None else [no_nan_rule(), finite_rule()]

    def add_rule(self, r: ValidationRule) -> "ValidationEngine":
        self.rules.append(r)
        return self

    def validate(self, t: torch.Tensor) -> ValidationResult:
        issues = []
        for r in self.rules:
            msg = r.check(t)
            if msg:
                issues.append(ValidationIssue(r.name, r.severity, msg))
        return ValidationResult(not any(i.severity in ("error", "critical") for i in issues), issues)


class AnomalyDetector:
    """z-score and IQR outlier detection; returns indices into the flattened tensor."""

    def __init__(self, z_threshold: float = 3.0, iqr_factor: float = 1.5):
        self.z, self.k = z_threshold, iqr_factor

    def zscore(self, t: torch.Tensor) -> torch.Tensor:
        f = t.detach().float().reshape(-1)
        sd = f.std(unbiased=False)
        if float(sd) == 0:
            return torch.empty(0, dtype=torch.long, device=t.device)
        return torch.nonzero(((f - f.mean()) / sd).abs() > self.z).reshape(-1)

    def iqr(self, t: torch.Tensor) -> torch.Tensor:
        f = t.detach().float().reshape(-1)
        q = torch.quantile(f, torch.tensor([0.25, 0.75], device=f.device))
        span = (q[1] - q[0]) * self.k
        return torch.nonzero((f < q[0] - span) | (f > q[1] + span)).reshape(-1)

    def detect(self, t: torch.Tensor, method: str = "zscore") -> Dict[str, object]:
        idx = self.zscore(t) if method == "zscore" else self.iqr(t)
        return {"method": method, "count": int(idx.numel()), "indices": idx, "fraction": idx.numel() / max(1, t.numel())}


class ConsistencyChecker:
    def check_shapes(self, tensors: Dict[str, torch.Tensor], dim: int = 0) -> List[str]:
        sizes = {k: v.shape[dim] for k, v in tensors.items()}
        return [] if len(set(sizes.values())) <= 1 else [f"inconsistent size along dim {dim}: {sizes}"]

    def check_dtypes(self, tensors: Dict[str, torch.Tensor]) -> List[str]:
        d = {k: v.dtype for k, v in tensors.items()}
        return [] if len(set(d.values())) <= 1 else [f"mixed dtypes: {d}"]

    def check_devices(self, tensors: Dict[str, torch.Tensor]) -> List[str]:
        d = {k: str(v.device) for k, v in tensors.items()}
        return [] if len(set(d.values())) <= 1 else [f"mixed devices: {d}"]

    def check_replicas(self, a: torch.Tensor, b: torch.Tensor, tol: float = 0.0) -> List[str]:
        diff = float((a.float() - b.float()).abs().max()) if a.numel() else 0.0
        return [] if diff <= tol else [f"replicas differ by {diff:.3e} (tolerance {tol})"]


class QualityMetrics:
    """Completeness (finite share), validity (in-range share), uniqueness, consistency (no outliers) -> score and
    letter grade."""

    def compute(self, t: torch.Tensor, valid_range: Optional[tuple] = None) -> Dict[str, float]:
        f = t.detach().float().reshape(-1)
        n = max(1, f.numel())
        finite = torch.isfinite(f)
        comp = float(finite.sum()) / n
        ff = f[finite]
        val = float(((ff >= valid_range[0]) & (ff <= valid_range[1])).sum()) / n if valid_range else comp
        uniq = float(torch.unique(ff).numel()) / max(1, ff.numel())
        cons = 1.0 - AnomalyDetector().detect(ff)["fraction"] if ff.numel() > 1 else 1.0
        score = 0.35 * comp + 0.3 * val + 0.1 * uniq + 0.25 * cons
        return {"completeness": comp, "validity": val, "uniqueness": uniq, "consistency": cons, "score": score}

    @staticmethod
    def grade(score: float) -> str:
        return "A" if score >= 0.9 else "B" if score >= 0.8 else "C" if score >= 0.7 else "D" if score >= 0.6 else "F"


class QualityReporter:
    def render(self, metrics: Dict[str, float], issues: List[ValidationIssue], fmt: str = "text") -> str:
        grade = QualityMetrics.grade(metrics.get("score", 0.0))
        if fmt == "json":
            return json.dumps({"grade": grade, "metrics": metrics, "issues": [i.__dict__ for i in issues]})
        rows = [(k, f"{v:.4f}") for k, v in metrics.items()]
        if fmt == "markdown":
            out = [f"# Data quality report — grade {grade}", "", "| metric | value |", "|---|---|"] + [f"| {k} | {v} |" for k, v in rows]
            out += ["", "## Issues"] + ([f"- **{i.severity}** `{i.rule}`: {i.message}" for i in issues] or ["none"])
            return "\n".join(out)
        if fmt == "html":
            body = "".join(f"<tr><td>{k}</td><td>{v}</td></tr>" for k, v in rows)
            iss = "".join(f"<li><b>{i.severity}</b> {i.rule}: {i.message}</li>" for i in issues)
            return f"<html><body><h1>Data quality report: grade {grade}</h1><table>{body}</table><ul>{iss}</ul></body></html>"
        out = [f"Data quality report: grade {grade}"] + [f"  {k:<14}{v}" for k, v in rows]
        out += [f"  [{i.severity}] {i.rule}: {i.message}" for i in issues]
        return "\n".join(out)


class RealTimeValidator:
    """Streaming validation: running statistics (Welford) plus per-batch rule checks; flags batches whose mean
    drifts more than ``drift_sigmas`` standard errors from the running mean."""

    def __init__(self, engine: Optional[ValidationEngine] = None, drift_sigmas: float = 6.0):
        self.engine = engine or ValidationEngine()
        self.n, self.mean, self.m2 = 0, 0.0, 0.0
        self.drift_sigmas = drift_sigmas
        self.history: List[ValidationResult] = []

    def feed(self, batch: torch.Tensor) -> ValidationResult:
        res = self.engine.validate(batch)
        f = batch.detach().float()
        bm, bn = float(f.mean()), f.numel()
        if self.n > 1000 and bn > 0:
            var = self.m2 / (self.n - 1)
            se = (var / bn) ** 0.5
            if se > 0 and abs(bm - self.mean) > self.drift_sigmas * se:
                res.issues.append(ValidationIssue("drift", "warning", f"batch mean {bm:.4g} vs running {self.mean:.4g}"))
        if bn and res.passed:
            bv = float(f.var(unbiased=False)) * bn
            tot = self.n + bn
            delta = bm - self.mean
            self.m2 += bv + delta * delta * self.n * bn / tot
            self.mean += delta * bn / tot
            self.n = tot
        res.metrics.update(running_mean=self.mean, seen=float(self.n))
        self.history.append(res)
        return res


class DataValidationFramework:
    def __init__(self):
        self.engine = ValidationEngine()
        self.anomaly = AnomalyDetector()
        self.consistency = ConsistencyChecker()
        self.quality = QualityMetrics()
        self.reporter = QualityReporter()

    def validate_tensor(self, t: torch.Tensor, valid_range: Optional[tuple] = None, fmt: Optional[str] = None):
        res = self.engine.validate(t)
        res.metrics = self.quality.compute(t, valid_range)
        res.metrics["anomalies"] = float(self.anomaly.detect(t[torch.isfinite(t)] if t.is_floating_point() else t)["count"])
        return self.reporter.render(res.metrics, res.issues, fmt) if fmt else res
