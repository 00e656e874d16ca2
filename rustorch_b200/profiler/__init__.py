"""Profiler: nested timed scopes, CUDA-event kernel timing, memory tracking, Chrome-trace export, metrics with
Prometheus text export, system sampling, alerts, trend analysis and a benchmark suite
(src/profiler/mod.rs:58-968, core.rs:12-631, timeline.rs:11-252, metrics_collector.rs:12-604,
kernel_profiler.rs:12-302, benchmark_suite.rs:12-643).

The reference measures host wall-clock only and its ``CudaEvent`` is a host timer
(kernel_profiler.rs:280-302).  Here a scope on a CUDA device is bracketed by real ``cudaEvent``s on the
current stream, so ``device_ms`` is time on the GPU and ``host_ms`` the wall clock.
"""
from __future__ import annotations

import contextlib
import json
import math
import os
import statistics
import threading
import time
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional

import torch


@dataclass
class ProfilerConfig:
    level: str = "standard"           # disabled | basic | standard | comprehensive
    enable_memory: bool = True
    enable_gpu: bool = True
    enable_system: bool = False
    sampling_rate_hz: float = 10.0
    export_chrome_trace: bool = False
    export_json: bool = False
    enable_nvtx: bool = True          # every profiled scope is also an NVTX range (visible in Nsight timelines)


class _Nvtx:
    """NVTX range push / pop through ``torch.cuda.nvtx`` (a few nanoseconds when no profiler is attached).  ``depth``
    counts the ranges this process has open; where the NVTX library cannot be reached the calls only keep the count."""

    def __init__(self):
        self.depth = 0
        self.pushed = 0
        try:
            from torch.cuda import nvtx as _n
            self._n = _n
        except Exception:  # noqa: BLE001
            self._n = None

    def push(self, name: str) -> None:
        self.depth += 1
        self.pushed += 1
        if self._n is not None:
            try:
                self._n.range_push(name)
            except Exception:  # noqa: BLE001  (no NVTX library on this machine)
                self._n = None

    def pop(self) -> None:
        self.depth = max(0, self.depth - 1)
        if self._n is not None:
            try:
                self._n.range_pop()
            except Exception:  # noqa: BLE001
                self._n = None

    def mark(self, name: str) -> None:
        if self._n is not None:
            try:
                self._n.mark(name)
            except Exception:  # noqa: BLE001
                self._n = None


nvtx = _Nvtx()


@contextlib.contextmanager
def nvtx_range(name: str):
    """``with nvtx_range("attn_fwd"): ...`` marks the enclosed host span (and the kernels launched in it) for Nsight."""
    nvtx.push(name)
    try:
        yield
    finally:
        nvtx.pop()


@dataclass
class ProfileEvent:
    name: str
    category: str
    start_us: float
    host_us: float
    depth: int
    tid: int
    device_ms: Optional[float] = None
    args: Dict[str, object] = field(default_factory=dict)


class Timeline:
    """Ordered events -> Chrome trace (``{"traceEvents": [{name, cat, ph: "X", ts, dur, pid, tid, args}]}``)."""

    def __init__(self):
        self.events: List[ProfileEvent] = []

    def add(self, e: ProfileEvent) -> None:
        self.events.append(e)

    def to_chrome_trace(self) -> dict:
        ev = []
        for e in self.events:
            args = dict(e.args)
            if e.device_ms is not None:
                args["device_ms"] = e.device_ms
            ev.append({"name": e.name, "cat": e.category, "ph": "X", "ts": e.start_us, "dur": e.host_us,
                       "pid": os.getpid(), "tid": e.tid, "args": args})
        return {"traceEvents": ev, "displayTimeUnit": "ms"}

    def export_chrome_trace(self, path: str) -> None:
        with open(path, "w") as f:
            json.dump(self.to_chrome_trace(), f)

    def flame_graph(self) -> Dict[str, float]:
        """Folded stacks ``"a;b;c" -> microseconds`` from the nesting depth of the events."""
        out: Dict[str, float] = {}
        stack: List[str] = []
        for e in sorted(self.events, key=lambda x: x.start_us):
            stack = stack[: e.depth] + [e.name]
            k = ";".join(stack)
            out[k] = out.get(k, 0.0) + e.host_us
        return out


class MemoryProfiler:
    def __init__(self):
        self.samples: List[Dict[str, float]] = []
        self.allocations: Dict[str, int] = {}

    def snapshot(self, tag: str = "") -> Dict[str, float]:
        s = {"tag": tag, "t": time.time()}
        if torch.cuda.is_available():
            s.update(cuda_allocated=torch.cuda.memory_allocated(), cuda_reserved=torch.cuda.memory_reserved(),
                     cuda_peak=torch.cuda.max_memory_allocated())
        try:
            import psutil
            s["rss"] = psutil.Process().memory_info().rss
        except Exception:  # noqa: BLE001
            pass
        self.samples.append(s)
        return s

    def record_allocation(self, name: str, nbytes: int) -> None:
        self.allocations[name] = self.allocations.get(name, 0) + nbytes

    def record_deallocation(self, name: str, nbytes: int) -> None:
        self.allocations[name] = self.allocations.get(name, 0) - nbytes

    def leaks(self) -> Dict[str, int]:
        return {k: v for k, v in self.allocations.items() if v > 0}

    def peak(self, key: str = "cuda_allocated") -> float:
        return max((s.get(key, 0) for s in self.samples), default=0)


class KernelProfiler:
    """Times callables on the device with CUDA events (host clock on CPU)."""

    def __init__(self):
        self.records: Dict[str, List[float]] = {}

    def time(self, name: str, fn: Callable, warmup: int = 1, iters: int = 3) -> float:
        cuda = torch.cuda.is_available()
        for _ in range(warmup):
            fn()
        ts = []
        for _ in range(iters):
            if cuda:
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                torch.cuda.synchronize()
                e0.record()
                fn()
                e1.record()
                torch.cuda.synchronize()
                ts.append(e0.elapsed_time(e1))
            else:
                t0 = time.perf_counter()
                fn()
                ts.append((time.perf_counter() - t0) * 1e3)
        self.records.setdefault(name, []).extend(ts)
        return min(ts)

    def summary(self) -> Dict[str, Dict[str, float]]:
        return {k: {"calls": len(v), "min_ms": min(v), "mean_ms": sum(v) / len(v), "max_ms": max(v)} for k, v in self.records.items()}


class MetricsCollector:
    """Counters, gauges and histograms with Prometheus text exposition."""

    def __init__(self, namespace: str = "rustorch"):
        self.ns = namespace
        self.counters: Dict[str, float] = {}
        self.gauges: Dict[str, float] = {}
        self.histograms: Dict[str, List[float]] = {}
        self._lock = threading.Lock()

    def inc(self, name: str, v: float = 1.0) -> None:
        with self._lock:
            self.counters[name] = self.counters.get(name, 0.0) + v

    def set_gauge(self, name: str, v: float) -> None:
        with self._lock:
            self.gauges[name] = v

    def observe(self, name: str, v: float) -> None:
        with self._lock:
            self.histograms.setdefault(name, []).append(v)

    def export_prometheus(self, buckets=(0.001, 0.01, 0.1, 1.0, 10.0)) -> str:
        lines = []
        for k, v in sorted(self.counters.items()):
            lines += [f"# TYPE {self.ns}_{k} counter", f"{self.ns}_{k} {v}"]
        for k, v in sorted(self.gauges.items()):
            lines += [f"# TYPE {self.ns}_{k} gauge", f"{self.ns}_{k} {v}"]
        for k, vals in sorted(self.histograms.items()):
            lines.append(f"# TYPE {self.ns}_{k} histogram")
            for b in buckets:
                lines.append(f'{self.ns}_{k}_bucket{{le="{b}"}} {sum(1 for x in vals if x <= b)}')
            lines += [f'{self.ns}_{k}_bucket{{le="+Inf"}} {len(vals)}', f"{self.ns}_{k}_sum {sum(vals)}", f"{self.ns}_{k}_count {len(vals)}"]
        return "\n".join(lines) + "\n"

    def export_json(self) -> str:
        return json.dumps({"counters": self.counters, "gauges": self.gauges,
                           "histograms": {k: {"count": len(v), "mean": sum(v) / len(v)} for k, v in self.histograms.items() if v}})


class SystemProfiler:
    def sample(self) -> Dict[str, float]:
        s: Dict[str, float] = {"t": time.time()}
        try:
            import psutil
            s["cpu_percent"] = psutil.cpu_percent(None)
            s["mem_percent"] = psutil.virtual_memory().percent
        except Exception:  # noqa: BLE001
            pass
        if torch.cuda.is_available():
            free, total = torch.cuda.mem_get_info()
            s["gpu_mem_used"] = total - free
        return s


class RealTimeMonitor:
    """Threshold alerts on sampled values: ``add_rule("loss", lambda v: v > 10, "loss exploded")``."""

    def __init__(self):
        self.rules: List[tuple] = []
        self.alerts: List[Dict[str, object]] = []

    def add_rule(self, metric: str, predicate: Callable[[float], bool], message: str) -> None:
        self.rules.append((metric, predicate, message))

    def feed(self, metric: str, value: float) -> List[str]:
        fired = []
        for m, pred, msg in self.rules:
            if m == metric and pred(value):
                self.alerts.append({"metric": metric, "value": value, "message": msg, "t": time.time()})
                fired.append(msg)
        return fired


class PerformanceAnalyzer:
    """Trend (least-squares slope) and simple recommendations from event statistics."""

    @staticmethod
    def trend(values: List[float]) -> float:
        n = len(values)
        if n < 2:
            return 0.0
        mx, my = (n - 1) / 2, sum(values) / n
        den = sum((i - mx) ** 2 for i in range(n))
        return sum((i - mx) * (v - my) for i, v in enumerate(values)) / den

    @staticmethod
    def recommendations(stats: Dict[str, Dict[str, float]]) -> List[str]:
        recs = []
        total = sum(s["total_ms"] for s in stats.values()) or 1.0
        for name, s in sorted(stats.items(), key=lambda kv: -kv[1]["total_ms"]):
            share = s["total_ms"] / total
            if share > 0.5:
                recs.append(f"'{name}' takes {share:.0%} of the profiled time: optimise it first")
            if s["calls"] > 1000 and s["mean_ms"] < 0.02:
                recs.append(f"'{name}' is launched {s['calls']} times at {s['mean_ms'] * 1e3:.1f} us each: fuse or capture in a CUDA graph")
        return recs


class Profiler:
    def __init__(self, config: Optional[ProfilerConfig] = None):
        self.config = config or ProfilerConfig()
        self.enabled = False
        self.timeline = Timeline()
        self.memory = MemoryProfiler()
        self.kernels = KernelProfiler()
        self.metrics = MetricsCollector()
        self._depth = threading.local()
        self._t0 = time.perf_counter()

    def enable(self) -> None:
        self.enabled = True

    def disable(self) -> None:
        self.enabled = False

    def clear(self) -> None:
        self.timeline = Timeline()
        self._recorded: Dict[str, List[float]] = {}

    # the Python binding's manual form (src/python/utils.rs:249-272): durations handed in by the caller
    def record(self, name: str, duration: float) -> None:
        if self.enabled:
            self.__dict__.setdefault("_recorded", {}).setdefault(name, []).append(float(duration))

    def get_stats(self) -> Dict[str, Dict[str, float]]:
        """count / total / mean / min / max per name over ``record``ed durations and profiled scopes (seconds)."""
        series: Dict[str, List[float]] = {k: list(v) for k, v in self.__dict__.get("_recorded", {}).items()}
        for e in self.timeline.events:
            series.setdefault(e.name, []).append(e.host_us / 1e6)
        return {k: {"count": float(len(v)), "total": sum(v), "mean": sum(v) / len(v), "min": min(v), "max": max(v)}
                for k, v in series.items() if v}

    @contextlib.contextmanager
    def profile(self, name: str, category: str = "op", **args):
        if not self.enabled:
            yield
            return
        depth = getattr(self._depth, "v", 0)
        self._depth.v = depth + 1
        use_nvtx = self.config.enable_nvtx
        if use_nvtx:
            nvtx.push(f"{category}:{name}")
        use_gpu = self.config.enable_gpu and torch.cuda.is_available()
        if use_gpu:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
        t0 = time.perf_counter()
        try:
            yield
        finally:
            dt = time.perf_counter() - t0
            dev = None
            if use_gpu:
                e1.record()
                e1.synchronize()
                dev = e0.elapsed_time(e1)
            if use_nvtx:
                nvtx.pop()
            self._depth.v = depth
            self.timeline.add(ProfileEvent(name, category, (t0 - self._t0) * 1e6, dt * 1e6, depth, threading.get_ident() % 100000, dev, args))

    def stats(self) -> Dict[str, Dict[str, float]]:
        out: Dict[str, Dict[str, float]] = {}
        for e in self.timeline.events:
            s = out.setdefault(e.name, {"calls": 0, "total_ms": 0.0, "device_ms": 0.0})
            s["calls"] += 1
            s["total_ms"] += e.host_us / 1e3
            s["device_ms"] += e.device_ms or 0.0
        for s in out.values():
            s["mean_ms"] = s["total_ms"] / s["calls"]
        return out

    def report(self) -> str:
        rows = [f"{'name':<32}{'calls':>8}{'total ms':>12}{'mean ms':>12}{'device ms':>12}"]
        for k, s in sorted(self.stats().items(), key=lambda kv: -kv[1]["total_ms"]):
            rows.append(f"{k:<32}{s['calls']:>8}{s['total_ms']:>12.3f}{s['mean_ms']:>12.3f}{s['device_ms']:>12.3f}")
        return "\n".join(rows)

    def export_chrome_trace(self, path: str) -> None:
        self.timeline.export_chrome_trace(path)


# global profiler + reference-style free functions
PROFILER = Profiler()


def enable_profiler() -> None:
    PROFILER.enable()


def disable_profiler() -> None:
    PROFILER.disable()


def profile(name: str, category: str = "op", **args):
    """``with profile("forward"): ...`` — the ``profile!`` macro / ``ProfileContext`` guard."""
    return PROFILER.profile(name, category, **args)


ProfileContext = profile


def print_profiler_report() -> str:
    r = PROFILER.report()
    print(r)
    return r


def export_chrome_trace(path: str) -> None:
    PROFILER.export_chrome_trace(path)


def clear_profiler() -> None:
    PROFILER.clear()


# ------------------------------------------------------------------ benchmark suite
@dataclass
class BenchmarkResult:
    name: str
    iters: int
    mean_ms: float
    median_ms: float
    std_ms: float
    min_ms: float
    max_ms: float
    throughput: Optional[float] = None


class AdvancedBenchmarkSuite:
    """Warm-up + repeated timing with statistics and JSON export."""

    def __init__(self, warmup: int = 3, iters: int = 10):
        self.warmup, self.iters = warmup, iters
        self.results: List[BenchmarkResult] = []

    def run(self, name: str, fn: Callable, items_per_iter: Optional[float] = None) -> BenchmarkResult:
        kp = KernelProfiler()
        for _ in range(self.warmup):
            fn()
        ts = [kp.time(name, fn, warmup=0, iters=1) for _ in range(self.iters)]
        mean = sum(ts) / len(ts)
        r = BenchmarkResult(name, len(ts), mean, statistics.median(ts), statistics.pstdev(ts), min(ts), max(ts),
                            items_per_iter / (mean / 1e3) if items_per_iter else None)
        self.results.append(r)
        return r

    def to_json(self) -> str:
        return json.dumps([r.__dict__ for r in self.results])
