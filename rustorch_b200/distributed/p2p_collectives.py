"""All-reduce / all-gather / reduce-scatter / broadcast as single kernels over NVLink peer memory
(csrc/collective/p2p_collectives.cu).

``P2PCollectives`` owns symmetric input / result / flag buffers sized for ``max_numel`` elements of one dtype.  The
call epoch is a device word that the kernel itself advances, so these calls can be captured in a CUDA graph and
replayed (the tensor-parallel decode step of the LLM runtime does exactly that).  With one rank they degenerate to
copies.  NCCL equivalents live in ``rustorch_b200.distributed.api``; the reference's versions are host loops
(src/gpu/multi_gpu.rs:583-940).
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

from .. import _native

ONE_SHOT, TWO_SHOT, ALL_GATHER, REDUCE_SCATTER, BROADCAST = range(5)


class P2PCollectives:
    def __init__(self, max_numel: int, dtype: torch.dtype = torch.bfloat16, device=None, group=None, timeout_s: float = 20.0,
                 one_shot_max_bytes: int = 512 * 1024):
        if dist.is_available() and dist.is_initialized():
            self.group = group or dist.group.WORLD
            self.world, self.rank = dist.get_world_size(self.group), dist.get_rank(self.group)
        else:
            self.group, self.world, self.rank = None, 1, 0
        self.device = torch.device(device if device is not None else ("cuda", torch.cuda.current_device()))
        self.dtype, self.timeout_s, self.one_shot_max_bytes = dtype, timeout_s, one_shot_max_bytes
        vec = 4 if dtype == torch.float32 else 8
        self.unit = vec * self.world
        self.max_numel = -(-max_numel // self.unit) * self.unit
        from .tp_fused import _symm
        self.inp, self.in_ptrs, self._h1 = _symm(self.max_numel, dtype, self.device, self.group, self.world)
        self.res, self.res_ptrs, self._h2 = _symm(self.max_numel, dtype, self.device, self.group, self.world)
        self.flags, self.flag_ptrs, self._h3 = _symm(max(16, 3 * self.world), torch.int32, self.device, self.group, self.world)
        self.epoch_dev = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.barrier = torch.zeros(2, dtype=torch.int32, device=self.device)

    def reset(self) -> None:
        """Re-arms the object after a call reported a timeout (a peer that never arrived).  A kernel that gave up
        can leave its grid-barrier count, the call epoch and the peers' flag words out of step with the other
        ranks, so every rank of the group calls this together: it clears the three, then meets at a host barrier
        so that nobody launches against flags that a slower rank is still clearing."""
        torch.cuda.synchronize(self.device)
        if self.world > 1:
            dist.barrier(self.group)                      # no rank clears while a peer's kernel still writes flags
        self.barrier.zero_()
        self.epoch_dev.zero_()
        self.flags.zero_()
        torch.cuda.synchronize(self.device)
        if self.world > 1:
            dist.barrier(self.group)

    def _pad(self, n: int, unit: int) -> int:
        return -(-n // unit) * unit

    def _stage(self, t: torch.Tensor, padded: int) -> None:
        flat = t.reshape(-1)
        self.inp[: flat.numel()].copy_(flat)
        if padded > flat.numel():
            self.inp[flat.numel():padded].zero_()

    def _launch(self, mode: int, out: torch.Tensor, numel: int, root: int = 0) -> None:
        _native.load(required=True).p2p_collective(mode, self.in_ptrs, self.res_ptrs, self.flag_ptrs, out, numel, self.epoch_dev,
                                                   self.barrier, self.rank, root, self.timeout_s)

    def all_reduce(self, t: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Sum over ranks.  Small messages take the one-shot kernel, large ones the two-shot kernel."""
        n = t.numel()
        assert t.dtype == self.dtype and n <= self.max_numel
        two = n * t.element_size() > self.one_shot_max_bytes and self.world > 1
        padded = self._pad(n, self.unit if two else self.unit // self.world)
        self._stage(t, padded)
        buf = torch.empty(padded, dtype=self.dtype, device=self.device)
        self._launch(TWO_SHOT if two else ONE_SHOT, buf, padded)
        res = buf[:n].view(t.shape)
        if out is not None:
            out.copy_(res)
            return out
        return res

    def all_reduce_(self, t: torch.Tensor) -> torch.Tensor:
        return self.all_reduce(t, out=t)

    def all_gather(self, t: torch.Tensor) -> torch.Tensor:
        """-> ``[world, *t.shape]``."""
        n = t.numel()
        padded = self._pad(n, self.unit // self.world)
        assert t.dtype == self.dtype and padded <= self.max_numel
        self._stage(t, padded)
        buf = torch.empty(self.world, padded, dtype=self.dtype, device=self.device)
        self._launch(ALL_GATHER, buf, padded)
        return buf[:, :n].reshape(self.world, *t.shape)

    def reduce_scatter(self, t: torch.Tensor) -> torch.Tensor:
        """``t``: ``[world * k]`` (flattened) on every rank -> this rank's summed chunk ``[k]``."""
        n = t.numel()
        if n % self.unit:
            raise ValueError(f"reduce_scatter needs a length that is a multiple of {self.unit}")
        assert t.dtype == self.dtype and n <= self.max_numel
        self._stage(t, n)
        out = torch.empty(n // self.world, dtype=self.dtype, device=self.device)
        self._launch(REDUCE_SCATTER, out, n)
        return out

    def broadcast(self, t: torch.Tensor, src: int = 0) -> torch.Tensor:
        n = t.numel()
        padded = self._pad(n, self.unit // self.world)
        assert t.dtype == self.dtype and padded <= self.max_numel
        if self.rank == src:
            self._stage(t, padded)
        buf = torch.empty(padded, dtype=self.dtype, device=self.device)
        self._launch(BROADCAST, buf, padded, src)
        res = buf[:n].view(t.shape)
        t.copy_(res)
        return t


class AllReduceResidualNorm:
    """``x += all_reduce(partial)`` and ``h = rmsnorm(x) * w`` as one kernel (csrc/collective/ar_residual_norm.cu):
    the epilogue of a row-parallel projection in tensor-parallel decoding.  The peers' partial sums arrive as
    self-validating data in triple-buffered receive slots, so a call costs one NVLink store latency; the call counter
    is device-resident, so the launch can be captured in a CUDA graph.  ``cap_numel`` bounds ``rows * d`` per call."""

    def __init__(self, cap_numel: int, dtype: torch.dtype = torch.float16, device=None, group=None, timeout_s: float = 20.0):
        if dtype not in (torch.float16, torch.bfloat16):
            raise ValueError("fp16 or bf16 activations")
        if dist.is_available() and dist.is_initialized():
            self.group = group or dist.group.WORLD
            self.world, self.rank = dist.get_world_size(self.group), dist.get_rank(self.group)
        else:
            self.group, self.world, self.rank = None, 1, 0
        self.device = torch.device(device if device is not None else ("cuda", torch.cuda.current_device()))
        self.dtype, self.timeout_s = dtype, timeout_s
        self.cap_numel = -(-cap_numel // 8) * 8
        from .tp_fused import _symm
        self.buf, self.buf_ptrs, self._h = _symm(3 * self.world * self.cap_numel, dtype, self.device, self.group, self.world)
        self.buf.view(torch.int16).fill_(-32768)          # 0x8000 in every lane: "not arrived"
        self.state = torch.zeros(8, dtype=torch.int32, device=self.device)
        torch.cuda.synchronize(self.device)
        if self.world > 1:
            dist.barrier(self.group)                      # nobody pushes before every rank's slots are armed

    def fits(self, rows: int, d: int) -> bool:
        return rows * d <= self.cap_numel and d % 8 == 0 and d <= 16384

    def __call__(self, partial: torch.Tensor, x: torch.Tensor, norm_weight: Optional[torch.Tensor] = None, eps: float = 1e-5,
                 h: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
        """Updates ``x`` in place; returns the normalised activations when ``norm_weight`` is given."""
        if norm_weight is not None and h is None:
            h = torch.empty_like(x)
        _native.load(required=True).ar_residual_norm(self.buf_ptrs, self.cap_numel, partial, x, norm_weight, h, self.state,
                                                     self.rank, eps, self.timeout_s)
        return h
