"""``torch.distributed``-style process-group API with the reference's names (src/distributed/api.rs:20-392,
src/distributed/mod.rs:62-347).

The reference parses the init method and environment and then does nothing (its collectives are
no-ops, src/distributed/common.rs:15-56).  Here every call is real: rendezvous through a TCP store
from ``tcp://host:port`` or ``MASTER_ADDR / MASTER_PORT / RANK / WORLD_SIZE``, NCCL among GPU
ranks (NVLink / NVSwitch) and Gloo among CPU ranks.  ``ReduceOp.Average`` is supported on both.
"""
from __future__ import annotations

import datetime
import enum
import os
import time
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

import torch
import torch.distributed as dist


class DistributedBackend(enum.Enum):
    NCCL = "nccl"
    GLOO = "gloo"
    MPI = "mpi"
    TCP = "tcp"   # served by gloo's TCP transport

    @staticmethod
    def parse(v) -> "DistributedBackend":
        if isinstance(v, DistributedBackend):
            return v
        return DistributedBackend(str(v).lower())


class ReduceOp(enum.Enum):
    """Reduction of a collective; ``AVERAGE`` is a sum followed by a division by the group size (src/distributed/mod.rs)."""

    SUM = "sum"
    PRODUCT = "product"
    MIN = "min"
    MAX = "max"
    AVERAGE = "average"


_TORCH_OP = {ReduceOp.SUM: dist.ReduceOp.SUM, ReduceOp.PRODUCT: dist.ReduceOp.PRODUCT,
             ReduceOp.MIN: dist.ReduceOp.MIN, ReduceOp.MAX: dist.ReduceOp.MAX}


@dataclass
class ProcessGroup:
    rank: int
    world_size: int
    backend: DistributedBackend
    master_addr: str
    master_port: int
    handle: object = None   # torch.distributed group (None = default group)

    def ranks(self) -> List[int]:
        return dist.get_process_group_ranks(self.handle) if self.handle is not None else list(range(self.world_size))


@dataclass
class CommunicationStats:
    calls: Dict[str, int] = field(default_factory=dict)
    bytes: Dict[str, int] = field(default_factory=dict)
    seconds: Dict[str, float] = field(default_factory=dict)

    def record(self, op: str, nbytes: int, dt: float) -> None:
        self.calls[op] = self.calls.get(op, 0) + 1
        self.bytes[op] = self.bytes.get(op, 0) + nbytes
        self.seconds[op] = self.seconds.get(op, 0.0) + dt

    def total_bytes(self) -> int:
        return sum(self.bytes.values())


_state: Dict[str, object] = {"group": None, "stats": CommunicationStats()}


def _parse_init_method(init_method: Optional[str]):
    if init_method and init_method.startswith("tcp://"):
        host, port = init_method[len("tcp://"):].rsplit(":", 1)
        return host, int(port)
    if init_method in (None, "env://"):
        return os.environ.get("MASTER_ADDR", "127.0.0.1"), int(os.environ.get("MASTER_PORT", "29500"))
    raise ValueError(f"unsupported init_method '{init_method}' (use tcp://host:port or env://)")


def init_process_group(backend="nccl", init_method: Optional[str] = None, world_size: Optional[int] = None,
                       rank: Optional[int] = None, timeout: Optional[float] = None) -> ProcessGroup:
    """Join the job.  ``timeout`` (seconds) bounds rendezvous and every later collective."""
    be = DistributedBackend.parse(backend)
    if be is DistributedBackend.MPI:
        raise RuntimeError("MPI backend is not available in this build")
    host, port = _parse_init_method(init_method)
    world_size = int(os.environ.get("WORLD_SIZE", "1")) if world_size is None else world_size
    rank = int(os.environ.get("RANK", "0")) if rank is None else rank
    torch_backend = "nccl" if be is DistributedBackend.NCCL else "gloo"
    if torch_backend == "nccl" and not torch.cuda.is_available():
        raise RuntimeError("NCCL backend requested but no CUDA device is available")
    kw = {}
    if timeout is not None:
        kw["timeout"] = datetime.timedelta(seconds=float(timeout))
    if torch_backend == "nccl":
        local = int(os.environ.get("LOCAL_RANK", rank % max(1, torch.cuda.device_count())))
        torch.cuda.set_device(local)
        kw["device_id"] = torch.device("cuda", local)
    if not dist.is_initialized():
        dist.init_process_group(torch_backend, init_method=f"tcp://{host}:{port}", world_size=world_size,
                                rank=rank, **kw)
    pg = ProcessGroup(rank, world_size, be, host, port)
    _state["group"] = pg
    return pg


init_distributed = init_process_group


def destroy_process_group() -> None:
    if dist.is_initialized():
        dist.destroy_process_group()
    _state["group"] = None


finalize = cleanup_distributed = destroy_process_group


def is_available() -> bool:
    return dist.is_available()


def is_initialized() -> bool:
    return dist.is_initialized() and _state["group"] is not None


def get_rank() -> int:
    return dist.get_rank() if dist.is_initialized() else 0


def get_world_size() -> int:
    return dist.get_world_size() if dist.is_initialized() else 1


def is_master() -> bool:
    return get_rank() == 0


def get_process_group() -> Optional[ProcessGroup]:
    return _state["group"]


def new_group(ranks: Sequence[int], timeout: Optional[float] = None, backend=None) -> ProcessGroup:
    base: ProcessGroup = _state["group"]
    kw = {}
    if timeout is not None:
        kw["timeout"] = datetime.timedelta(seconds=float(timeout))
    if backend is not None:
        be = DistributedBackend.parse(backend)
        kw["backend"] = "nccl" if be is DistributedBackend.NCCL else "gloo"
    h = dist.new_group(list(ranks), **kw)
    r = dist.get_rank()
    return ProcessGroup(list(ranks).index(r) if r in ranks else -1, len(ranks), base.backend, base.master_addr,
                        base.master_port, h)


class DistributedRequest:
    """Handle of an asynchronous collective: ``wait()`` / ``is_completed()``."""

    def __init__(self, work, post=None):
        self._work, self._post, self._done = work, post, work is None

    def wait(self, timeout: Optional[float] = None) -> bool:
        if not self._done:
            if timeout is not None:
                self._work.wait(datetime.timedelta(seconds=timeout))
            else:
                self._work.wait()
            if self._post:
                self._post()
            self._done = True
        return True

    def is_completed(self) -> bool:
        return self._done or self._work.is_completed()


def _t(x) -> torch.Tensor:
    return getattr(x, "data", x) if not isinstance(x, torch.Tensor) else x


def _h(group: Optional[ProcessGroup]):
    return None if group is None else group.handle


def _timed(op: str, nbytes: int, t0: float) -> None:
    _state["stats"].record(op, nbytes, time.perf_counter() - t0)


def all_reduce(tensor, op: ReduceOp = ReduceOp.SUM, group: Optional[ProcessGroup] = None, async_op: bool = False):
    """In place.  ``Average`` = sum followed by division by the group size."""
    t = _t(tensor)
    if not dist.is_initialized() or get_world_size() == 1:
        return DistributedRequest(None) if async_op else None
    t0 = time.perf_counter()
    n = dist.get_world_size(_h(group))
    avg = op is ReduceOp.AVERAGE
    work = dist.all_reduce(t, _TORCH_OP[ReduceOp.SUM if avg else op], group=_h(group), async_op=async_op)
    post = (lambda: t.div_(n)) if avg else None
    if async_op:
        return DistributedRequest(work, post)
    if post:
        post()
    _timed("all_reduce", t.numel() * t.element_size(), t0)
    return None


def all_gather(tensor, group: Optional[ProcessGroup] = None) -> List[torch.Tensor]:
    t = _t(tensor).contiguous()
    if not dist.is_initialized() or get_world_size() == 1:
        return [t.clone()]
    t0 = time.perf_counter()
    outs = [torch.empty_like(t) for _ in range(dist.get_world_size(_h(group)))]
    dist.all_gather(outs, t, group=_h(group))
    _timed("all_gather", t.numel() * t.element_size() * len(outs), t0)
    return outs


def broadcast(tensor, src: int = 0, group: Optional[ProcessGroup] = None, async_op: bool = False):
    t = _t(tensor)
    if not dist.is_initialized() or get_world_size() == 1:
        return DistributedRequest(None) if async_op else None
    t0 = time.perf_counter()
    w = dist.broadcast(t, src, group=_h(group), async_op=async_op)
    if async_op:
        return DistributedRequest(w)
    _timed("broadcast", t.numel() * t.element_size(), t0)


def reduce(tensor, dst: int = 0, op: ReduceOp = ReduceOp.SUM, group: Optional[ProcessGroup] = None):
    t = _t(tensor)
    if not dist.is_initialized() or get_world_size() == 1:
        return None
    avg = op is ReduceOp.AVERAGE
    dist.reduce(t, dst, _TORCH_OP[ReduceOp.SUM if avg else op], group=_h(group))
    if avg and dist.get_rank() == dst:
        t.div_(dist.get_world_size(_h(group)))


def scatter(tensor, scatter_list: Optional[List] = None, src: int = 0, group: Optional[ProcessGroup] = None):
    t = _t(tensor)
    if not dist.is_initialized() or get_world_size() == 1:
        if scatter_list:
            t.copy_(_t(scatter_list[0]))
        return None
    sl = [_t(x).contiguous() for x in scatter_list] if (scatter_list and dist.get_rank() == src) else None
    if dist.get_backend(_h(group)) == "nccl" and sl is None:
        sl = None
    dist.scatter(t, sl, src, group=_h(group))


def gather(tensor, dst: int = 0, group: Optional[ProcessGroup] = None) -> Optional[List[torch.Tensor]]:
    t = _t(tensor).contiguous()
    if not dist.is_initialized() or get_world_size() == 1:
        return [t.clone()]
    n = dist.get_world_size(_h(group))
    outs = [torch.empty_like(t) for _ in range(n)] if dist.get_rank() == dst else None
    dist.gather(t, outs, dst, group=_h(group))
    return outs


def reduce_scatter(output, input_list: List, op: ReduceOp = ReduceOp.SUM, group: Optional[ProcessGroup] = None):
    o = _t(output)
    if not dist.is_initialized() or get_world_size() == 1:
        o.copy_(_t(input_list[0]))
        return None
    avg = op is ReduceOp.AVERAGE
    ins = [_t(x).contiguous() for x in input_list]
    if dist.get_backend(_h(group)) == "gloo":   # gloo has no reduce_scatter: all_reduce each slot
        r = dist.get_rank(_h(group))
        for i, x in enumerate(ins):
            y = x.clone()
            dist.all_reduce(y, _TORCH_OP[ReduceOp.SUM if avg else op], group=_h(group))
            if i == r:
                o.copy_(y)
    else:
        dist.reduce_scatter(o, ins, _TORCH_OP[ReduceOp.SUM if avg else op], group=_h(group))
    if avg:
        o.div_(dist.get_world_size(_h(group)))


def all_to_all(outputs: List, inputs: List, group: Optional[ProcessGroup] = None) -> None:
    outs, ins = [_t(x) for x in outputs], [_t(x).contiguous() for x in inputs]
    if not dist.is_initialized() or get_world_size() == 1:
        outs[0].copy_(ins[0])
        return
    if dist.get_backend(_h(group)) == "gloo":   # emulate with pairwise send/recv
        r, n = dist.get_rank(_h(group)), dist.get_world_size(_h(group))
        outs[r].copy_(ins[r])
        reqs = []
        for p in range(n):
            if p != r:
                reqs.append(dist.isend(ins[p], p, group=_h(group)))
                reqs.append(dist.irecv(outs[p], p, group=_h(group)))
        for q in reqs:
            q.wait()
    else:
        dist.all_to_all(outs, ins, group=_h(group))


def barrier(group: Optional[ProcessGroup] = None) -> None:
    if dist.is_initialized() and get_world_size() > 1:
        dist.barrier(group=_h(group))


def send(tensor, dst: int, group: Optional[ProcessGroup] = None, tag: int = 0) -> None:
    dist.send(_t(tensor).contiguous(), dst, group=_h(group), tag=tag)


def isend(tensor, dst: int, group: Optional[ProcessGroup] = None, tag: int = 0) -> DistributedRequest:
    """Non-blocking send; keep the returned request (and the tensor) alive until ``wait()``."""
    return DistributedRequest(dist.isend(_t(tensor).contiguous(), dst, group=_h(group), tag=tag))


def irecv(tensor, src: int, group: Optional[ProcessGroup] = None, tag: int = 0) -> DistributedRequest:
    return DistributedRequest(dist.irecv(_t(tensor), src, group=_h(group), tag=tag))


def recv(tensor, src: int, group: Optional[ProcessGroup] = None, tag: int = 0) -> None:
    dist.recv(_t(tensor), src, group=_h(group), tag=tag)


class monitoring:
    """``monitoring::get_communication_stats`` (src/distributed/api.rs:324-359)."""

    @staticmethod
    def get_communication_stats() -> CommunicationStats:
        return _state["stats"]

    @staticmethod
    def reset() -> None:
        _state["stats"] = CommunicationStats()
