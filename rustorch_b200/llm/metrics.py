"""Inference metrics: time to first token, tokens per second, memory vs model size, with the
reference's targets for a 7B model (TTFT < 200 ms, > 20 tok/s, memory < 1.5x model size;
example-cli/src/metrics/mod.rs:92-112) and text / JSON / Markdown reporters (metrics/reporter.rs:47-176)."""
from __future__ import annotations

import json
import time
from dataclasses import asdict, dataclass, field
from typing import Dict, List, Optional


class InferenceTimer:
    def __init__(self):
        self.t_start = self.t_first = self.t_end = None
        self.n_tokens = 0

    def start(self) -> None:
        self.t_start, self.t_first, self.n_tokens = time.perf_counter(), None, 0

    def token(self) -> None:
        now = time.perf_counter()
        if self.t_first is None:
            self.t_first = now
        self.n_tokens += 1
        self.t_end = now

    def ttft_ms(self) -> float:
        return (self.t_first - self.t_start) * 1e3 if self.t_first else 0.0

    def tokens_per_s(self) -> float:
        if self.n_tokens < 2 or self.t_end is None:
            return 0.0
        return (self.n_tokens - 1) / max(self.t_end - self.t_first, 1e-9)


@dataclass
class PerformanceTargets:
    ttft_ms: float = 200.0
    tokens_per_s: float = 20.0
    memory_ratio: float = 1.5


@dataclass
class InferenceMetrics:
    ttft_ms: float = 0.0
    tokens_per_s: float = 0.0
    total_tokens: int = 0
    memory_bytes: int = 0
    model_bytes: int = 0

    def memory_ratio(self) -> float:
        return self.memory_bytes / self.model_bytes if self.model_bytes else 0.0


class MetricsCollector:
    def __init__(self, targets: Optional[PerformanceTargets] = None):
        self.targets = targets or PerformanceTargets()
        self.runs: List[InferenceMetrics] = []

    def record(self, m: InferenceMetrics) -> None:
        self.runs.append(m)

    def summary(self) -> Dict[str, float]:
        if not self.runs:
            return {}
        n = len(self.runs)
        return {"runs": n, "ttft_ms": sum(r.ttft_ms for r in self.runs) / n,
                "tokens_per_s": sum(r.tokens_per_s for r in self.runs) / n,
                "total_tokens": sum(r.total_tokens for r in self.runs),
                "memory_ratio": max(r.memory_ratio() for r in self.runs)}

    def meets_targets(self) -> Dict[str, bool]:
        s = self.summary()
        if not s:
            return {}
        return {"ttft": s["ttft_ms"] < self.targets.ttft_ms, "throughput": s["tokens_per_s"] > self.targets.tokens_per_s,
                "memory": s["memory_ratio"] == 0 or s["memory_ratio"] < self.targets.memory_ratio}


class MetricsReporter:
    def __init__(self, collector: MetricsCollector):
        self.c = collector

    def text(self) -> str:
        s, ok = self.c.summary(), self.c.meets_targets()
        if not s:
            return "no runs recorded"
        mark = lambda b: "ok" if b else "MISSED"  # noqa: E731
        return (f"TTFT {s['ttft_ms']:.1f} ms [{mark(ok['ttft'])}]  throughput {s['tokens_per_s']:.1f} tok/s "
                f"[{mark(ok['throughput'])}]  memory x{s['memory_ratio']:.2f} [{mark(ok['memory'])}]  runs {s['runs']}")

    def json(self) -> str:
        return json.dumps({"summary": self.c.summary(), "targets": asdict(self.c.targets), "met": self.c.meets_targets()})

    def markdown(self) -> str:
        s, ok = self.c.summary(), self.c.meets_targets()
        rows = ["| metric | value | target | met |", "|---|---|---|---|"]
        if s:
            rows += [f"| TTFT (ms) | {s['ttft_ms']:.1f} | < {self.c.targets.ttft_ms} | {ok['ttft']} |",
                     f"| tokens/s | {s['tokens_per_s']:.1f} | > {self.c.targets.tokens_per_s} | {ok['throughput']} |",
                     f"| memory / model | {s['memory_ratio']:.2f} | < {self.c.targets.memory_ratio} | {ok['memory']} |"]
        return "\n".join(rows)
