"""Asynchronous gradient synchronisation with priorities, bucket manager and gradient compression
(src/distributed/async_gradient.rs:26-661, src/distributed/performance.rs:19-382).

A worker thread drains a priority queue of gradient tensors and all-reduces (averages) them; callers
``submit_gradient`` and later ``wait_for_completion`` / ``sync_all`` with timeouts.  Compression
(top-k with error feedback, uniform quantisation) really drops / rounds values — the reference's
top-k is the identity (async_gradient.rs) — and is applied before communication.
"""
from __future__ import annotations

import enum
import itertools
import queue
import threading
import time
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

import torch

from . import api


class Priority(enum.IntEnum):
    """Scheduling priority of a gradient synchronisation request (src/distributed/async_gradient.rs)."""

    LOW = 0
    NORMAL = 1
    HIGH = 2
    CRITICAL = 3


@dataclass
class AsyncConfig:
    max_queue: int = 1024
    timeout_s: float = 30.0
    compression: Optional[str] = None      # None | "topk" | "quantization"
    compression_ratio: float = 0.01
    quantization_bits: int = 8
    error_feedback: bool = True


# ---------------------------------------------------------------- compression
class TopKCompressor:
    """Keep the ``ratio`` largest-magnitude entries; the rest accumulate as residual (error feedback)."""

    def __init__(self, ratio: float = 0.01, error_feedback: bool = True):
        self.ratio, self.error_feedback = ratio, error_feedback
        self.residual: Dict[int, torch.Tensor] = {}

    def compress(self, g: torch.Tensor, key: int = 0) -> Tuple[torch.Tensor, torch.Tensor, torch.Size]:
        flat = g.reshape(-1).clone()
        if self.error_feedback and key in self.residual:
            flat += self.residual[key]
        k = max(1, int(flat.numel() * self.ratio))
        _, idx = flat.abs().topk(k)
        vals = flat[idx]
        if self.error_feedback:
            r = flat.clone()
            r[idx] = 0
            self.residual[key] = r
        return vals, idx, g.shape

    @staticmethod
    def decompress(vals: torch.Tensor, idx: torch.Tensor, shape: torch.Size) -> torch.Tensor:
        out = torch.zeros(int(torch.tensor(shape).prod()) if len(shape) else 1, dtype=vals.dtype, device=vals.device)
        out[idx] = vals
        return out.view(shape)


class QuantizationCompressor:
    """Uniform symmetric quantisation to ``bits`` bits with a per-tensor scale."""

    def __init__(self, bits: int = 8):
        self.bits = bits
        self.qmax = 2 ** (bits - 1) - 1

    def compress(self, g: torch.Tensor) -> Tuple[torch.Tensor, float]:
        scale = float(g.abs().max().clamp_min(1e-12)) / self.qmax
        return torch.clamp(torch.round(g / scale), -self.qmax, self.qmax).to(torch.int8 if self.bits <= 8 else torch.int16), scale

    @staticmethod
    def decompress(q: torch.Tensor, scale: float, dtype=torch.float32) -> torch.Tensor:
        return q.to(dtype) * scale


class GradientCompressor:
    """Front end used by the synchroniser: ``compress_decompress`` returns what the receiver would see."""

    def __init__(self, kind: Optional[str] = None, ratio: float = 0.01, bits: int = 8, error_feedback: bool = True):
        self.kind = kind
        self.topk = TopKCompressor(ratio, error_feedback)
        self.quant = QuantizationCompressor(bits)

    def compress_decompress(self, g: torch.Tensor, key: int = 0) -> torch.Tensor:
        if self.kind in (None, "none"):
            return g
        if self.kind == "topk":
            return TopKCompressor.decompress(*self.topk.compress(g, key)).to(g.dtype)
        if self.kind in ("quantization", "quant"):
            q, s = self.quant.compress(g)
            return QuantizationCompressor.decompress(q, s, g.dtype)
        raise ValueError(f"unknown compression '{self.kind}'")

    def compression_factor(self, g: torch.Tensor) -> float:
        if self.kind == "topk":
            return 1.0 / max(self.topk.ratio * 2, 1e-9)   # value + index per kept entry
        if self.kind in ("quantization", "quant"):
            return g.element_size() * 8 / self.quant.bits
        return 1.0


# ------------------------------------------------------------- bucket manager
class GradientBucketManager:
    """Packs submitted gradients into buckets of ``bucket_size_mb`` (25 MB default) for fewer, larger messages."""

    def __init__(self, bucket_size_mb: float = 25.0):
        self.cap = int(bucket_size_mb * 1024 * 1024)
        self.buckets: List[List[Tuple[str, torch.Tensor]]] = [[]]
        self._bytes = 0

    def add_gradient(self, name: str, g: torch.Tensor) -> Optional[int]:
        """Returns the index of a bucket that just became full (ready to send), else None."""
        nbytes = g.numel() * g.element_size()
        ready = None
        if self.buckets[-1] and self._bytes + nbytes > self.cap:
            ready = len(self.buckets) - 1
            self.buckets.append([])
            self._bytes = 0
        self.buckets[-1].append((name, g))
        self._bytes += nbytes
        return ready

    def flush(self) -> List[List[Tuple[str, torch.Tensor]]]:
        out = [b for b in self.buckets if b]
        self.buckets, self._bytes = [[]], 0
        return out


# --------------------------------------------------------------- synchroniser
class AsyncGradientSynchronizer:
    def __init__(self, config: Optional[AsyncConfig] = None, group: Optional[api.ProcessGroup] = None):
        self.config = config or AsyncConfig()
        self.group = group
        self._q: "queue.PriorityQueue" = queue.PriorityQueue(self.config.max_queue)
        self._ids = itertools.count(1)          # itertools.count is safe under the GIL
        self._done: Dict[int, threading.Event] = {}
        self._errors: Dict[int, BaseException] = {}
        self._lock = threading.Lock()
        self._stop = threading.Event()
        self.compressor = GradientCompressor(self.config.compression, self.config.compression_ratio,
                                             self.config.quantization_bits, self.config.error_feedback)
        self.completed = 0
        self._worker = threading.Thread(target=self._run, daemon=True)
        self._worker.start()

    def _run(self) -> None:
        while not self._stop.is_set():
            try:
                _, rid, tensor = self._q.get(timeout=0.05)
            except queue.Empty:
                continue
            try:
                if self.config.compression:
                    tensor.copy_(self.compressor.compress_decompress(tensor, key=tensor.data_ptr()))
                api.all_reduce(tensor, api.ReduceOp.AVERAGE, self.group)
            except BaseException as e:  # noqa: BLE001
                self._errors[rid] = e
            with self._lock:
                self.completed += 1
                ev = self._done.get(rid)
            if ev:
                ev.set()

    def submit_gradient(self, tensor: torch.Tensor, priority: Priority = Priority.NORMAL) -> int:
        rid = next(self._ids)
        with self._lock:
            self._done[rid] = threading.Event()
        self._q.put((-int(priority), rid, tensor), timeout=self.config.timeout_s)
        return rid

    def check_completions(self) -> List[int]:
        with self._lock:
            return [r for r, e in self._done.items() if e.is_set()]

    def wait_for_completion(self, request_id: int, timeout: Optional[float] = None) -> None:
        ev = self._done.get(request_id)
        if ev is None:
            raise KeyError(f"unknown request {request_id}")
        if not ev.wait(self.config.timeout_s if timeout is None else timeout):
            raise TimeoutError(f"gradient sync request {request_id} timed out")
        with self._lock:
            self._done.pop(request_id, None)
        err = self._errors.pop(request_id, None)
        if err:
            raise err

    def sync_all(self, timeout: Optional[float] = None) -> None:
        deadline = time.monotonic() + (self.config.timeout_s if timeout is None else timeout)
        for rid in list(self._done):
            self.wait_for_completion(rid, max(0.0, deadline - time.monotonic()))

    def shutdown(self) -> None:
        self._stop.set()
        self._worker.join(timeout=2)


class TensorMemoryPool:
    """Reuses communication staging tensors by (shape, dtype, device)."""

    def __init__(self, max_per_key: int = 8):
        self.max_per_key = max_per_key
        self._free: Dict[tuple, List[torch.Tensor]] = {}
        self.hits = self.misses = 0

    def acquire(self, shape, dtype=torch.float32, device="cpu") -> torch.Tensor:
        key = (tuple(shape), dtype, str(device))
        lst = self._free.get(key)
        if lst:
            self.hits += 1
            return lst.pop()
        self.misses += 1
        return torch.empty(tuple(shape), dtype=dtype, device=device)

    def release(self, t: torch.Tensor) -> None:
        key = (tuple(t.shape), t.dtype, str(t.device))
        lst = self._free.setdefault(key, [])
        if len(lst) < self.max_per_key:
            lst.append(t)


class CommunicationScheduler:
    """Collects pending ops and issues them in batches (largest first) to amortise launch latency."""

    def __init__(self, batch_size: int = 8):
        self.batch_size = batch_size
        self.pending: List[Tuple[str, torch.Tensor]] = []
        self.issued = 0

    def schedule(self, op: str, tensor: torch.Tensor) -> None:
        self.pending.append((op, tensor))
        if len(self.pending) >= self.batch_size:
            self.flush()

    def flush(self, group: Optional[api.ProcessGroup] = None) -> int:
        n = len(self.pending)
        for op, t in sorted(self.pending, key=lambda x: -x[1].numel()):
            if op == "all_reduce":
                api.all_reduce(t, api.ReduceOp.SUM, group)
            elif op == "average":
                api.all_reduce(t, api.ReduceOp.AVERAGE, group)
            elif op == "broadcast":
                api.broadcast(t, 0, group)
            else:
                raise ValueError(f"unknown op '{op}'")
        self.pending.clear()
        self.issued += n
        return n
