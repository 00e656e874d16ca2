"""Context parallelism: ring attention over sequence shards.

Every rank of the group holds one contiguous slice of the sequence (``[B, T / W, H, D]`` of q, k and v).  The key /
value slices travel once around the ring; at every hop a rank attends its own queries to the slice it currently
holds (the flash-attention kernel on CUDA, which also returns the row log-sum-exp) and folds the partial result into
its running output with log-sum-exp weights, while the next slice is already on its way (``isend`` / ``irecv`` on a
side stream).  Causal masking works on whole slices: a slice from a later rank is skipped, the rank's own slice is
causal inside, earlier slices are attended in full.  The backward pass is a second trip around the ring in which
the dK / dV accumulators travel with their slice and arrive home after the last hop; it recomputes the
probabilities from the saved global log-sum-exp, exactly as single-GPU flash attention does.

This is the long-sequence companion of the tensor + sequence parallel layers in ``model_parallel.py`` /
``tp_fused.py``: activations, not only weights, are split along the sequence, so the per-GPU attention memory is
``O(T / W)`` in the sequence length.  The reference has no counterpart (its attention materialises the full
``[T, T]`` score matrix on one device, src/nn/attention.rs:92-157); the sequence split follows the contiguous-block
convention of its ``DistributedSampler`` (src/distributed/mod.rs).
"""
from __future__ import annotations

import math
from typing import List, Optional, Tuple

import torch
import torch.distributed as dist

from .. import _native

__all__ = ["ring_attention", "RingAttention", "shard_sequence", "gather_sequence", "RingAttentionFn"]


# --------------------------------------------------------------------------- one (query slice, key slice) block
def _native_block_ok(q: torch.Tensor, k: torch.Tensor) -> bool:
    return (q.is_cuda and q.dtype == torch.bfloat16 and q.shape[-1] in (64, 128) and _native.available()
            and q.shape[2] % k.shape[2] == 0)


def _ct(t: torch.Tensor) -> torch.dtype:
    """Accumulation dtype of the eager path: fp32, or fp64 for fp64 inputs."""
    return torch.float64 if t.dtype == torch.float64 else torch.float32


def _expand_kv(t: torch.Tensor, H: int) -> torch.Tensor:
    return t if t.shape[2] == H else t.repeat_interleave(H // t.shape[2], dim=2)


def _block_forward(q, k, v, causal: bool, scale: float) -> Tuple[torch.Tensor, torch.Tensor]:
    """``(o [B, Tq, H, D] fp32, lse [B, H, Tq] fp32)`` of softmax(q k^T scale) v for one pair of slices."""
    if _native_block_ok(q, k):
        from ..ops import kernels as K
        o, lse = K.attention_fwd(q, k, v, causal, scale)
        return o.float(), lse                                                    # natural-log units
    H, ct = q.shape[2], _ct(q)
    qf, kf, vf = q.to(ct).transpose(1, 2), _expand_kv(k, H).to(ct).transpose(1, 2), _expand_kv(v, H).to(ct).transpose(1, 2)
    s = (qf @ kf.transpose(-1, -2)) * scale                                     # [B, H, Tq, Tk]
    if causal:
        Tq, Tk = s.shape[-2:]
        s = s.masked_fill(torch.ones(Tq, Tk, dtype=torch.bool, device=s.device).triu(1 + Tk - Tq), float("-inf"))
    lse = torch.logsumexp(s, dim=-1)
    o = torch.exp(s - lse.unsqueeze(-1)) @ vf
    return o.transpose(1, 2).contiguous(), lse


def _block_backward(q, k, v, o, lse, d_o, causal: bool, scale: float):
    """Gradients of one block given the GLOBAL output ``o`` and log-sum-exp ``lse`` of the query rows: the block's
    probabilities are ``exp(s - lse)``, which already carry the normalisation over all slices."""
    if _native_block_ok(q, k):
        from ..ops import kernels as K
        dq, dk, dv = K.attention_bwd(q, k, v, o.to(q.dtype), d_o.to(q.dtype), lse, causal, scale)
        return dq.float(), dk.float(), dv.float()
    H, Hkv, ct = q.shape[2], k.shape[2], _ct(q)
    qf, kf, vf = q.to(ct).transpose(1, 2), _expand_kv(k, H).to(ct).transpose(1, 2), _expand_kv(v, H).to(ct).transpose(1, 2)
    of, dof = o.to(ct).transpose(1, 2), d_o.to(ct).transpose(1, 2)
    s = (qf @ kf.transpose(-1, -2)) * scale
    if causal:
        Tq, Tk = s.shape[-2:]
        s = s.masked_fill(torch.ones(Tq, Tk, dtype=torch.bool, device=s.device).triu(1 + Tk - Tq), float("-inf"))
    p = torch.exp(s - lse.unsqueeze(-1))
    dv = p.transpose(-1, -2) @ dof
    dp = dof @ vf.transpose(-1, -2)
    delta = (dof * of).sum(-1, keepdim=True)
    ds = p * (dp - delta) * scale
    dq = ds @ kf
    dk = ds.transpose(-1, -2) @ qf
    if Hkv != H:                                                                 # grouped queries share a kv head
        B, _, Tk, D = dk.shape
        dk = dk.view(B, Hkv, H // Hkv, Tk, D).sum(2)
        dv = dv.view(B, Hkv, H // Hkv, Tk, D).sum(2)
    return dq.transpose(1, 2).contiguous(), dk.transpose(1, 2).contiguous(), dv.transpose(1, 2).contiguous()


# --------------------------------------------------------------------------- the ring
class _Ring:
    """Sends tensors to the next rank and receives from the previous one, on a side stream when on CUDA so that the
    hop overlaps the block that is being computed."""

    def __init__(self, group):
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        ranks = dist.get_process_group_ranks(group) if group is not None else list(range(self.world))
        self.next = ranks[(self.rank + 1) % self.world]
        self.prev = ranks[(self.rank - 1) % self.world]
        self._stream = None

    def start(self, tensors: List[torch.Tensor]):
        recv = [torch.empty_like(t) for t in tensors]
        if self.world == 1:
            return recv, None, tensors
        cuda = tensors[0].is_cuda
        if cuda:
            if self._stream is None:
                self._stream = torch.cuda.Stream(device=tensors[0].device)
            self._stream.wait_stream(torch.cuda.current_stream(tensors[0].device))
        ops = []
        for t, r in zip(tensors, recv):
            ops.append(dist.P2POp(dist.isend, t.contiguous(), self.next, self.group))
            ops.append(dist.P2POp(dist.irecv, r, self.prev, self.group))
        if cuda:
            with torch.cuda.stream(self._stream):
                reqs = dist.batch_isend_irecv(ops)
        else:
            reqs = dist.batch_isend_irecv(ops)
        return recv, reqs, tensors

    def finish(self, handle):
        recv, reqs, sent = handle
        if reqs is None:
            return sent
        for r in reqs:
            r.wait()
        if recv[0].is_cuda:
            torch.cuda.current_stream(recv[0].device).wait_stream(self._stream)
        return recv


def _merge(o, lse, o_b, lse_b):
    """Fold a block's (output, log-sum-exp) into the running pair."""
    if o is None:
        return o_b, lse_b
    new = torch.logaddexp(lse, lse_b)
    w_old = torch.exp(lse - new).transpose(1, 2).unsqueeze(-1)                   # [B, Tq, H, 1]
    w_new = torch.exp(lse_b - new).transpose(1, 2).unsqueeze(-1)
    return o * w_old + o_b * w_new, new


class RingAttentionFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, causal: bool, scale: float, group):
        ring = _Ring(group)
        W, r = ring.world, ring.rank
        o, lse = None, None
        kb, vb = k, v
        for hop in range(W):
            src = (r - hop) % W                                                  # owner of the slice held now
            handle = ring.start([kb, vb]) if hop + 1 < W else None
            if not (causal and src > r):
                o_b, lse_b = _block_forward(q, kb, vb, causal and src == r, scale)
                o, lse = _merge(o, lse, o_b, lse_b)
            if handle is not None:
                kb, vb = ring.finish(handle)
        ctx.save_for_backward(q, k, v, o.to(q.dtype), lse)
        ctx.causal, ctx.scale, ctx.group = causal, scale, group
        return o.to(q.dtype)

    @staticmethod
    def backward(ctx, d_o):
        q, k, v, o, lse = ctx.saved_tensors
        causal, scale = ctx.causal, ctx.scale
        ring = _Ring(ctx.group)
        W, r = ring.world, ring.rank
        ct = _ct(q)
        dq = torch.zeros(q.shape, dtype=ct, device=q.device)
        kb, vb = k, v
        dkb = torch.zeros(k.shape, dtype=ct, device=k.device)                    # travel with their slice
        dvb = torch.zeros(v.shape, dtype=ct, device=v.device)
        for hop in range(W):
            src = (r - hop) % W
            if not (causal and src > r):
                dq_b, dk_b, dv_b = _block_backward(q, kb, vb, o, lse, d_o, causal and src == r, scale)
                dq += dq_b
                dkb += dk_b
                dvb += dv_b
            # after the last hop the accumulators are back at the slice's owner
            kb, vb, dkb, dvb = ring.finish(ring.start([kb, vb, dkb, dvb]))
        return dq.to(q.dtype), dkb.to(k.dtype), dvb.to(v.dtype), None, None, None


def ring_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, causal: bool = False, scale: Optional[float] = None,
                   group=None) -> torch.Tensor:
    """Attention over the full sequence for sequence-sharded ``q / k / v [B, T_local, H(kv), D]``; rank ``i`` of
    ``group`` holds tokens ``[i T_local, (i + 1) T_local)``.  Differentiable."""
    scale = (1.0 / math.sqrt(q.shape[-1])) if scale is None else float(scale)
    return RingAttentionFn.apply(q, k, v, bool(causal), scale, group)


class RingAttention(torch.nn.Module):
    """Module form of :func:`ring_attention` (no parameters)."""

    def __init__(self, causal: bool = False, scale: Optional[float] = None, group=None):
        super().__init__()
        self.causal, self.scale, self.group = causal, scale, group

    def forward(self, q, k, v):
        return ring_attention(q, k, v, self.causal, self.scale, self.group)


def shard_sequence(x: torch.Tensor, dim: int = 1, group=None) -> torch.Tensor:
    """This rank's contiguous slice of ``x`` along ``dim`` (the length must divide by the group size)."""
    W, r = dist.get_world_size(group), dist.get_rank(group)
    if x.shape[dim] % W:
        raise ValueError(f"sequence length {x.shape[dim]} does not divide into {W} ranks")
    n = x.shape[dim] // W
    return x.narrow(dim, r * n, n).contiguous()


def gather_sequence(x: torch.Tensor, dim: int = 1, group=None) -> torch.Tensor:
    """All ranks' slices concatenated along ``dim`` (not differentiable: for outputs and tests)."""
    W = dist.get_world_size(group)
    parts = [torch.empty_like(x) for _ in range(W)]
    dist.all_gather(parts, x.contiguous(), group=group)
    return torch.cat(parts, dim=dim)
