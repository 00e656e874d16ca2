"""Debug framework: structured logger, scoped profiler, allocation tracker, log analyser with alert rules,
and system utilities (src/debug/mod.rs, logger.rs, profiler.rs, memory_tracker.rs, log_analyzer.rs, utils.rs).
"""
from __future__ import annotations

import json
import os
import platform
import re
import sys
import threading
import time
import traceback
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional

import torch

LEVELS = {"trace": 0, "debug": 1, "info": 2, "warn": 3, "error": 4, "critical": 5}


@dataclass
class LogEntry:
    t: float
    level: str
    component: str
    message: str
    fields: Dict[str, object] = field(default_factory=dict)

    def to_json(self) -> str:
        return json.dumps({"timestamp": self.t, "level": self.level, "component": self.component,
                           "message": self.message, **self.fields})

    def to_text(self) -> str:
        ts = time.strftime("%H:%M:%S", time.localtime(self.t))
        extra = " ".join(f"{k}={v}" for k, v in self.fields.items())
        return f"[{ts}] {self.level.upper():<8} {self.component}: {self.message}{' ' + extra if extra else ''}"


class Logger:
    """Levels, console / file / JSON sinks and component filters."""

    def __init__(self, level: str = "info", console: bool = False, file: Optional[str] = None, json_format: bool = False,
                 components: Optional[List[str]] = None, max_entries: int = 10000):
        self.level, self.console, self.file, self.json_format = level, console, file, json_format
        self.components = set(components) if components else None
        self.entries: List[LogEntry] = []
        self.max_entries = max_entries
        self._lock = threading.Lock()

    def log(self, level: str, component: str, message: str, **fields) -> Optional[LogEntry]:
        if LEVELS[level] < LEVELS[self.level] or (self.components is not None and component not in self.components):
            return None
        e = LogEntry(time.time(), level, component, message, fields)
        line = e.to_json() if self.json_format else e.to_text()
        with self._lock:
            self.entries.append(e)
            if len(self.entries) > self.max_entries:
                del self.entries[: len(self.entries) - self.max_entries]
            if self.console:
                print(line, file=sys.stderr)
            if self.file:
                with open(self.file, "a") as f:
                    f.write(line + "\n")
        return e

    def debug(self, c, m, **f):
        return self.log("debug", c, m, **f)

    def info(self, c, m, **f):
        return self.log("info", c, m, **f)

    def warn(self, c, m, **f):
        return self.log("warn", c, m, **f)

    def error(self, c, m, **f):
        return self.log("error", c, m, **f)


class ProfileScope:
    """Times the enclosed block into a ``DebugProfiler`` (src/debug/profiler.rs)."""

    def __init__(self, profiler: "DebugProfiler", name: str):
        self.p, self.name = profiler, name

    def __enter__(self):
        self.t0 = time.perf_counter()
        return self

    def __exit__(self, *exc):
        self.p.record(self.name, time.perf_counter() - self.t0)
        return False


class DebugProfiler:
    def __init__(self):
        self.samples: Dict[str, List[float]] = {}

    def scope(self, name: str) -> ProfileScope:
        return ProfileScope(self, name)

    def record(self, name: str, seconds: float) -> None:
        self.samples.setdefault(name, []).append(seconds)

    def summary(self) -> Dict[str, Dict[str, float]]:
        return {k: {"calls": len(v), "total_s": sum(v), "mean_s": sum(v) / len(v), "max_s": max(v)} for k, v in self.samples.items()}

    def bottlenecks(self, share: float = 0.3) -> List[str]:
        tot = sum(sum(v) for v in self.samples.values()) or 1.0
        return [k for k, v in self.samples.items() if sum(v) / tot >= share]


class MemoryTracker:
    """Named allocation bookkeeping with leak heuristics (live for longer than ``leak_age_s``) and large-allocation
    reporting."""

    def __init__(self, large_threshold: int = 100 << 20, leak_age_s: float = 300.0):
        self.live: Dict[int, tuple] = {}
        self.large_threshold, self.leak_age_s = large_threshold, leak_age_s
        self.total_allocated = self.total_freed = self.peak = self.current = 0
        self._next = 0

    def track_allocation(self, nbytes: int, tag: str = "") -> int:
        self._next += 1
        self.live[self._next] = (nbytes, tag, time.time())
        self.total_allocated += nbytes
        self.current += nbytes
        self.peak = max(self.peak, self.current)
        return self._next

    def track_deallocation(self, handle: int) -> None:
        nbytes, _, _ = self.live.pop(handle)
        self.total_freed += nbytes
        self.current -= nbytes

    def track_tensor(self, t: torch.Tensor, tag: str = "") -> int:
        return self.track_allocation(t.numel() * t.element_size(), tag)

    def potential_leaks(self, now: Optional[float] = None) -> List[dict]:
        now = now or time.time()
        return [{"handle": h, "bytes": n, "tag": tag, "age_s": now - t} for h, (n, tag, t) in self.live.items() if now - t > self.leak_age_s]

    def large_allocations(self) -> List[dict]:
        return [{"handle": h, "bytes": n, "tag": tag} for h, (n, tag, _) in self.live.items() if n >= self.large_threshold]

    def report(self) -> dict:
        return {"current": self.current, "peak": self.peak, "allocated": self.total_allocated, "freed": self.total_freed,
                "live": len(self.live), "leaks": self.potential_leaks(), "large": self.large_allocations()}


@dataclass
class AlertRule:
    name: str
    pattern: str
    threshold: int = 1
    window_s: float = 60.0
    cooldown_s: float = 60.0
    last_fired: float = 0.0


class LogAnalyzer:
    """Regex patterns over log entries; alert rules fire when a pattern matches ``threshold`` times inside
    ``window_s`` and then stay quiet for ``cooldown_s``."""

    def __init__(self):
        self.patterns: Dict[str, re.Pattern] = {}
        self.rules: List[AlertRule] = []

    def add_pattern(self, name: str, regex: str) -> None:
        self.patterns[name] = re.compile(regex)

    def add_rule(self, rule: AlertRule) -> None:
        self.rules.append(rule)
        self.patterns.setdefault(rule.name, re.compile(rule.pattern))

    def analyze(self, entries: List[LogEntry]) -> Dict[str, int]:
        counts = {k: 0 for k in self.patterns}
        for e in entries:
            for k, p in self.patterns.items():
                if p.search(e.message):
                    counts[k] += 1
        counts["errors"] = sum(1 for e in entries if LEVELS[e.level] >= LEVELS["error"])
        return counts

    def check_alerts(self, entries: List[LogEntry], now: Optional[float] = None) -> List[str]:
        now = now or time.time()
        fired = []
        for r in self.rules:
            if now - r.last_fired < r.cooldown_s:
                continue
            p = self.patterns[r.name]
            n = sum(1 for e in entries if now - e.t <= r.window_s and p.search(e.message))
            if n >= r.threshold:
                r.last_fired = now
                fired.append(r.name)
        return fired


class DebugUtils:
    @staticmethod
    def system_info() -> dict:
        info = {"python": sys.version.split()[0], "platform": platform.platform(), "torch": torch.__version__,
                "cpus": os.cpu_count(), "cuda": torch.cuda.is_available()}
        if torch.cuda.is_available():
            p = torch.cuda.get_device_properties(0)
            info.update(gpu=p.name, sms=p.multi_processor_count, gpu_mem=p.total_memory, cc=f"{p.major}.{p.minor}")
        return info

    @staticmethod
    def stack_trace() -> str:
        return "".join(traceback.format_stack()[:-1])

    @staticmethod
    def perf_timer() -> Callable[[], float]:
        t0 = time.perf_counter()
        return lambda: time.perf_counter() - t0

    @staticmethod
    def tensor_summary(t: torch.Tensor) -> dict:
        f = t.detach().float()
        return {"shape": list(t.shape), "dtype": str(t.dtype), "device": str(t.device), "min": f.min().item() if f.numel() else None,
                "max": f.max().item() if f.numel() else None, "mean": f.mean().item() if f.numel() else None,
                "nan": int(torch.isnan(f).sum()), "inf": int(torch.isinf(f).sum())}


class DebugFramework:
    def __init__(self, level: str = "debug", **logger_kw):
        self.logger = Logger(level, **logger_kw)
        self.profiler = DebugProfiler()
        self.memory = MemoryTracker()
        self.analyzer = LogAnalyzer()

    def log(self, level: str, component: str, message: str, **fields):
        return self.logger.log(level, component, message, **fields)

    def profile(self, name: str) -> ProfileScope:
        return self.profiler.scope(name)

    def track_allocation(self, nbytes: int, tag: str = "") -> int:
        return self.memory.track_allocation(nbytes, tag)

    def generate_debug_report(self) -> dict:
        return {"system": DebugUtils.system_info(), "profile": self.profiler.summary(), "memory": self.memory.report(),
                "log_counts": self.analyzer.analyze(self.logger.entries), "entries": len(self.logger.entries)}
