"""Memory management: arena-backed tensor pool, deduplicating pool with garbage collection, analytics (leaks,
hot spots), pressure monitoring and optimisation advice
(src/memory/mod.rs, enhanced_pool.rs, analytics.rs, pressure_monitor.rs, optimizer.rs).

``MemoryPool`` reserves ONE buffer on its device (HBM on a B200: sized in GB, not in per-tensor ``cudaMalloc``
calls) and carves tensors out of it with the native best-fit/coalescing arena allocator, so steady-state
allocation never reaches the driver and never synchronises the device.
"""
from __future__ import annotations

import hashlib
import time
import weakref
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from .. import _native


class PoolExhausted(MemoryError):
    """Raised when a bounded memory pool cannot serve an allocation."""


class MemoryPool:
    def __init__(self, capacity_bytes: int, device="cpu", alignment: int = 256):
        self.device = torch.device(device)
        self.buffer = torch.empty(capacity_bytes, dtype=torch.uint8, device=self.device)
        self.arena = _native.host().Arena(capacity_bytes, alignment)
        self._live: Dict[int, int] = {}          # data_ptr -> offset

    def allocate(self, shape: Sequence[int], dtype: torch.dtype = torch.float32) -> torch.Tensor:
        n = 1
        for s in shape:
            n *= int(s)
        nbytes = n * torch.empty(0, dtype=dtype).element_size()
        off = self.arena.allocate(nbytes)
        if off < 0:
            st = self.arena.stats()
            raise PoolExhausted(f"pool exhausted: need {nbytes} B, largest free range {st['largest_free']} B "
                                f"of {st['capacity'] - st['in_use']} B free (fragmentation {st['fragmentation']:.2f})")
        size = max(nbytes, 1)
        t = self.buffer[off:off + size].view(dtype).view(*shape) if n else self.buffer[off:off].view(dtype).view(*shape)
        self._live[self.buffer.data_ptr() + off] = off
        return t

    def zeros(self, shape, dtype=torch.float32) -> torch.Tensor:
        return self.allocate(shape, dtype).zero_()

    def _key(self, t: torch.Tensor) -> int:
        return t.data_ptr() if t.numel() else -1

    def deallocate(self, t: torch.Tensor) -> None:
        off = self._live.pop(t.data_ptr(), None)
        if off is None:
            raise ValueError("tensor does not belong to this pool (or was already released)")
        self.arena.release(off)

    def reset(self) -> None:
        self.arena.reset()
        self._live.clear()

    def stats(self) -> dict:
        return dict(self.arena.stats())

    def owns(self, t: torch.Tensor) -> bool:
        return t.data_ptr() in self._live


class EnhancedMemoryPool(MemoryPool):
    """Adds content deduplication (identical read-only tensors share one block, reference counted) and a
    garbage collector that frees blocks whose tensors have been dropped without ``deallocate``."""

    def __init__(self, capacity_bytes: int, device="cpu", alignment: int = 256):
        super().__init__(capacity_bytes, device, alignment)
        self._dedup: Dict[str, Tuple[torch.Tensor, int]] = {}      # digest -> (tensor, refcount)
        self._weak: Dict[int, weakref.ref] = {}
        self.dedup_hits = 0

    def allocate(self, shape, dtype=torch.float32) -> torch.Tensor:
        t = super().allocate(shape, dtype)
        self._weak[t.data_ptr()] = weakref.ref(t)
        return t

    def intern(self, src: torch.Tensor) -> torch.Tensor:
        """Pool-resident read-only copy of ``src``; equal contents are stored once."""
        key = hashlib.sha256(src.detach().cpu().contiguous().reshape(-1).view(torch.uint8).numpy().tobytes()
                             + str((src.dtype, tuple(src.shape))).encode()).hexdigest()
        if key in self._dedup:
            t, rc = self._dedup[key]
            self._dedup[key] = (t, rc + 1)
            self.dedup_hits += 1
            return t
        t = self.allocate(src.shape, src.dtype)
        t.copy_(src)
        self._dedup[key] = (t, 1)
        return t

    def release_interned(self, t: torch.Tensor) -> None:
        for k, (u, rc) in list(self._dedup.items()):
            if u.data_ptr() == t.data_ptr():
                if rc > 1:
                    self._dedup[k] = (u, rc - 1)
                else:
                    del self._dedup[k]
                    self.deallocate(u)
                return
        raise ValueError("tensor was not interned in this pool")

    def garbage_collect(self) -> int:
        """Free blocks whose tensor objects no longer exist.  Returns the number of blocks reclaimed."""
        interned = {t.data_ptr() for t, _ in self._dedup.values()}
        n = 0
        for ptr, ref in list(self._weak.items()):
            if ref() is None and ptr in self._live and ptr not in interned:
                self.arena.release(self._live.pop(ptr))
                del self._weak[ptr]
                n += 1
        return n


@dataclass
class AllocationRecord:
    tag: str
    nbytes: int
    t_alloc: float
    t_free: Optional[float] = None


class MemoryAnalytics:
    """Allocation history -> leaks (never freed and old), hot spots (tags by bytes and count), timeline."""

    def __init__(self):
        self.records: Dict[int, AllocationRecord] = {}
        self._next = 0

    def on_alloc(self, nbytes: int, tag: str = "", now: Optional[float] = None) -> int:
        self._next += 1
        self.records[self._next] = AllocationRecord(tag, nbytes, now if now is not None else time.time())
        return self._next

    def on_free(self, handle: int, now: Optional[float] = None) -> None:
        self.records[handle].t_free = now if now is not None else time.time()

    def leaks(self, older_than_s: float = 60.0, now: Optional[float] = None) -> List[AllocationRecord]:
        now = now if now is not None else time.time()
        return [r for r in self.records.values() if r.t_free is None and now - r.t_alloc > older_than_s]

    def hotspots(self, top: int = 5) -> List[Tuple[str, int, int]]:
        agg: Dict[str, List[int]] = {}
        for r in self.records.values():
            a = agg.setdefault(r.tag, [0, 0])
            a[0] += r.nbytes
            a[1] += 1
        return sorted(((k, v[0], v[1]) for k, v in agg.items()), key=lambda x: -x[1])[:top]

    def peak_live_bytes(self) -> int:
        ev = []
        for r in self.records.values():
            ev.append((r.t_alloc, r.nbytes))
            if r.t_free is not None:
                ev.append((r.t_free, -r.nbytes))
        cur = peak = 0
        for _, d in sorted(ev):
            cur += d
            peak = max(peak, cur)
        return peak

    def mean_lifetime_s(self) -> float:
        ls = [r.t_free - r.t_alloc for r in self.records.values() if r.t_free is not None]
        return sum(ls) / len(ls) if ls else 0.0


class AdaptivePressureMonitor:
    """Classifies memory pressure from utilisation samples with thresholds that adapt to the observed
    baseline (exponential average), and predicts time to exhaustion from the recent slope."""

    LEVELS = ("low", "medium", "high", "critical")

    def __init__(self, thresholds=(0.6, 0.8, 0.93), adapt: float = 0.05):
        self.thresholds, self.adapt = list(thresholds), adapt
        self.baseline: Optional[float] = None
        self.samples: List[Tuple[float, float]] = []

    def sample_device(self, device=None) -> float:
        if torch.cuda.is_available():
            free, total = torch.cuda.mem_get_info(device)
            return self.feed(1.0 - free / total)
        import psutil
        return self.feed(psutil.virtual_memory().percent / 100.0)

    def feed(self, utilisation: float, now: Optional[float] = None) -> float:
        now = now if now is not None else time.time()
        self.samples.append((now, utilisation))
        self.samples = self.samples[-256:]
        self.baseline = utilisation if self.baseline is None else (1 - self.adapt) * self.baseline + self.adapt * utilisation
        return utilisation

    def level(self) -> str:
        if not self.samples:
            return "low"
        u = self.samples[-1][1]
        shift = max(0.0, (self.baseline or 0.0) - 0.5) * 0.2        # a busy steady state raises the alarm levels a little
        idx = sum(u >= min(0.99, t + shift) for t in self.thresholds)
        return self.LEVELS[idx]

    def seconds_to_exhaustion(self) -> Optional[float]:
        if len(self.samples) < 2:
            return None
        (t0, u0), (t1, u1) = self.samples[max(0, len(self.samples) - 16)], self.samples[-1]
        slope = (u1 - u0) / (t1 - t0) if t1 > t0 else 0.0
        return (1.0 - u1) / slope if slope > 1e-9 else None


class MemoryOptimizer:
    """Advice from pool statistics and analytics."""

    @staticmethod
    def recommend(pool_stats: dict, analytics: Optional[MemoryAnalytics] = None) -> List[str]:
        recs = []
        if pool_stats.get("n_fail", 0):
            recs.append(f"{pool_stats['n_fail']} allocations failed: grow the pool or release temporaries earlier")
        if pool_stats.get("fragmentation", 0.0) > 0.5 and pool_stats.get("free_ranges", 0) > 8:
            recs.append("free space is fragmented: allocate long-lived tensors first or reset the pool between phases")
        cap = pool_stats.get("capacity", 0)
        if cap and pool_stats.get("peak", 0) < 0.5 * cap:
            recs.append(f"peak use is {pool_stats['peak'] / cap:.0%} of the pool: it can shrink")
        if analytics:
            for tag, nbytes, count in analytics.hotspots(3):
                if count > 1000 and nbytes / max(1, count) < 4096:
                    recs.append(f"'{tag}' makes {count} tiny allocations: batch them into one buffer")
            if analytics.leaks():
                recs.append(f"{len(analytics.leaks())} allocations older than a minute were never freed")
        return recs or ["no action needed"]

    @staticmethod
    def plan_activation_memory(graph_plan) -> Tuple[List[int], int, int]:
        """``(offsets, arena_bytes, naive_bytes)`` of a native ``ExecutionPlan``: buffers with disjoint lifetimes
        share space."""
        offsets, (total, naive) = graph_plan.memory_plan(256)
        return list(offsets), total, naive
