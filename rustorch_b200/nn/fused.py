"""Fused transformer sub-blocks as autograd Functions over the native sm_100a kernels.

Each Function covers one residual branch (pre-norm -> projections -> residual add) so that
* the residual add rides in a GEMM epilogue on the way forward,
* the upstream residual gradient is added inside the norm backward kernel,
* GELU / dGELU ride in GEMM epilogues,
* weight gradients are accumulated by the wgrad GEMM straight into the fp32 ``main_grad``
  buffer of the parameter (when it has one), which the fused optimizer consumes and zeroes.

Parameters without a ``main_grad`` attribute get an ordinary returned gradient instead, so the
Functions also work with stock optimizers.

The reference builds the same blocks from separate host loops without any backward for
attention/norm/activation layers (src/nn/transformer_phase6.rs:922-976,
src/models/transformer_models.rs:760-796).
"""
from __future__ import annotations

import math
import os
from typing import Optional

import torch

from ..ops import kernels as K

_sm_count_cache = {}


def _num_sms(device=None) -> int:
    """SM count of ``device`` (the current CUDA device by default), read once per device; 148 where there is no GPU."""
    if not torch.cuda.is_available():
        return 148
    idx = torch.cuda.current_device() if device is None or device.index is None else device.index
    n = _sm_count_cache.get(idx)
    if n is None:
        n = _sm_count_cache[idx] = int(torch.cuda.get_device_properties(idx).multi_processor_count)
    return n

# Called at the end of every fused backward with the parameters whose gradients that backward has
# finished accumulating AND whose values it no longer reads.  The data-parallel wrapper uses it to
# launch a gradient bucket as soon as the bucket is complete (overlap with the rest of backward).
grad_ready_hook = None


# Weight- and bias-gradient kernels that accumulate straight into ``main_grad`` have no consumer inside backward, so
# they run on a side stream: the input-gradient GEMM of the same layer (and whatever follows it) proceeds on the main
# stream meanwhile and the CTAs of one persistent GEMM fill the SMs the other leaves idle in its last wave.  Every
# backward joins the side stream before it reports its parameters ready (RUSTORCH_WGRAD_STREAM=0: one stream).
_SIDE_ON = os.environ.get("RUSTORCH_WGRAD_STREAM", "1") != "0"
_side_streams = {}
_side_used = {}
_side_keep = {}   # tensors the side stream still reads: released after the join, never through record_stream (a host
                  # that runs many steps ahead would otherwise leave the allocator with blocks it cannot reuse yet)


def _side_run(device: torch.device, fn, *inputs) -> None:
    if not _SIDE_ON or device.type != "cuda":
        fn()
        return
    idx = device.index if device.index is not None else torch.cuda.current_device()
    side = _side_streams.get(idx)
    if side is None:
        side = _side_streams[idx] = torch.cuda.Stream(device=idx)
    side.wait_stream(torch.cuda.current_stream(idx))      # the inputs were produced on the main stream
    with torch.cuda.stream(side):
        fn()
    _side_keep.setdefault(idx, []).extend(inputs)          # their memory must outlive the side stream's reads
    _side_used[idx] = True


def _side_hold(device: torch.device, *tensors) -> None:
    idx = device.index if device.index is not None else torch.cuda.current_device()
    _side_keep.setdefault(idx, []).extend(t for t in tensors if t is not None)


def _side_handle(device: torch.device, direct: bool) -> int:
    """Raw handle of the side stream for kernels that order themselves after the main stream with an event (the second
    stage of the norm backward); 0 when the gradients are returned to autograd instead of accumulated in place."""
    if not (_SIDE_ON and direct and device.type == "cuda"):
        return 0
    idx = device.index if device.index is not None else torch.cuda.current_device()
    side = _side_streams.get(idx)
    if side is None:
        side = _side_streams[idx] = torch.cuda.Stream(device=idx)
    _side_used[idx] = True
    return side.cuda_stream


def _ln_bwd(dh, x2, ln_w, mean, rstd, wg, bg, dres, direct: bool):
    """LayerNorm backward; when the parameter gradients are accumulated in place their reduction runs on the side
    stream (nothing in backward reads them)."""
    h = _side_handle(dh.device, direct)
    if not h:
        return K.layer_norm_bwd(dh, x2, ln_w, mean, rstd, wg, bg, dres=dres)
    dx, partial = K.layer_norm_bwd(dh, x2, ln_w, mean, rstd, wg, bg, dres=dres, reduce_stream=h)
    _side_hold(dh.device, partial)
    return dx


def _side_join() -> None:
    for idx, used in _side_used.items():
        if used:
            torch.cuda.current_stream(idx).wait_stream(_side_streams[idx])
            _side_used[idx] = False
            _side_keep.get(idx, []).clear()                # freed on the main stream, after its wait on the side stream


def _notify(*params):
    _side_join()
    if grad_ready_hook is not None:
        grad_ready_hook([p for p in params if p is not None])


def _split_k_for(tiles: int, k_blocks: int, device=None) -> int:
    """Split the contraction so that tiles x splits fill ONE wave of the persistent GEMM (measured on the GPT-2 weight
    gradient shapes: 3072 x 768 x 16384 takes 67.6 us with 2 splits = 144 work units, 77.8 us with 8, 84 us with 9; every
    extra split adds a pass of fp32 atomics over the output)."""
    sms = _num_sms(device)
    if tiles >= sms:
        return 1
    return max(1, min(sms // max(tiles, 1), max(1, k_blocks // 8)))


def wgrad_into(dy2d: torch.Tensor, x2d: torch.Tensor, param: torch.Tensor, alpha_dev: Optional[torch.Tensor] = None):
    """dW[out,in] (+)= dy2d^T @ x2d (times the device scalar ``alpha_dev`` when given).  Returns None if
    accumulated into ``param.main_grad``."""
    n_out, n_in = dy2d.shape[1], x2d.shape[1]
    tiles = -(-n_out // 128) * -(-n_in // 256)
    sk = _split_k_for(tiles, -(-dy2d.shape[0] // 64), dy2d.device)
    mg = getattr(param, "main_grad", None)
    if mg is not None:
        extra = (alpha_dev,) if alpha_dev is not None else ()
        _side_run(dy2d.device, lambda: K.gemm(dy2d, x2d, a_mn=True, b_mn=True, out=mg.view(n_out, n_in), accumulate=True,
                                               split_k=sk, alpha_dev=alpha_dev), dy2d, x2d, *extra)
        return None
    g = K.gemm(dy2d, x2d, a_mn=True, b_mn=True, out_dtype=torch.float32, accumulate=True, split_k=sk,
               alpha_dev=alpha_dev)
    return g.to(param.dtype)


def bgrad_into(dy2d: torch.Tensor, param: Optional[torch.Tensor]):
    if param is None:
        return None
    mg = getattr(param, "main_grad", None)
    if mg is not None:
        _side_run(dy2d.device, lambda: K.colsum_accum(dy2d, mg), dy2d)
        return None
    g = torch.zeros(dy2d.shape[1], dtype=torch.float32, device=dy2d.device)
    K.colsum_accum(dy2d, g)
    return g.to(param.dtype)


def _norm_grad_bufs(w, b):
    """fp32 accumulation targets for dgamma/dbeta and whether they are the main_grad views."""
    wg = getattr(w, "main_grad", None)
    direct = wg is not None
    if not direct:
        wg = torch.zeros(w.numel(), dtype=torch.float32, device=w.device)
    bg = None
    if b is not None:
        bg = getattr(b, "main_grad", None) if direct else torch.zeros(
            b.numel(), dtype=torch.float32, device=b.device)
    return wg, bg, direct


class AttnBlockFn(torch.autograd.Function):
    """y = x + proj(attention(qkv(norm(x))))  (pre-LayerNorm, fused QKV projection)."""

    @staticmethod
    def forward(ctx, x, ln_w, ln_b, w_qkv, b_qkv, w_proj, b_proj, n_head: int, eps: float,
                causal: bool, residual: bool = True):
        B, T, C = x.shape
        D = C // n_head
        x2 = x.reshape(B * T, C)
        h, mean, rstd = K.layer_norm_fwd(x2, ln_w, ln_b, eps)
        qkv = K.gemm(h, w_qkv, bias=b_qkv)                       # [B*T, 3C]
        qkv5 = qkv.view(B, T, 3, n_head, D)
        o, lse = K.attention_fwd(qkv5[:, :, 0], qkv5[:, :, 1], qkv5[:, :, 2], causal)
        o2 = o.view(B * T, C)
        # residual=False returns the branch alone (the caller applies dropout to it before the residual add)
        y = K.gemm(o2, w_proj, bias=b_proj, aux=x2, epilogue=K.EPI_RESIDUAL) if residual else K.gemm(o2, w_proj, bias=b_proj)
        ctx.save_for_backward(x2, ln_w, ln_b, w_qkv, b_qkv, w_proj, b_proj, mean, rstd, h, qkv, o, lse)
        ctx.meta = (B, T, C, n_head, causal, residual)
        return y.view(B, T, C)

    @staticmethod
    def backward(ctx, dy):
        x2, ln_w, ln_b, w_qkv, b_qkv, w_proj, b_proj, mean, rstd, h, qkv, o, lse = ctx.saved_tensors
        B, T, C, n_head, causal, residual = ctx.meta
        D = C // n_head
        dy2 = dy.contiguous().view(B * T, C)
        o2 = o.view(B * T, C)
        g_wproj = wgrad_into(dy2, o2, w_proj)
        g_bproj = bgrad_into(dy2, b_proj)
        do = K.gemm(dy2, w_proj, b_mn=True)                      # [B*T, C]
        qkv5 = qkv.view(B, T, 3, n_head, D)
        dqkv = torch.empty_like(qkv)
        dqkv5 = dqkv.view(B, T, 3, n_head, D)
        K.attention_bwd(qkv5[:, :, 0], qkv5[:, :, 1], qkv5[:, :, 2], o, do.view(B, T, n_head, D), lse,
                        causal, dq=dqkv5[:, :, 0], dk=dqkv5[:, :, 1], dv=dqkv5[:, :, 2])
        g_wqkv = wgrad_into(dqkv, h, w_qkv)
        g_bqkv = bgrad_into(dqkv, b_qkv)
        dh = K.gemm(dqkv, w_qkv, b_mn=True)                      # [B*T, C]
        wg, bg, direct = _norm_grad_bufs(ln_w, ln_b)
        dx = _ln_bwd(dh, x2, ln_w, mean, rstd, wg, bg, dy2 if residual else None, direct)
        g_lnw = None if direct else wg.to(ln_w.dtype)
        g_lnb = None if (direct or ln_b is None) else bg.to(ln_b.dtype)
        _notify(w_proj, b_proj, w_qkv, b_qkv, ln_w, ln_b)
        return (dx.view(B, T, C), g_lnw, g_lnb, g_wqkv, g_bqkv, g_wproj, g_bproj, None, None, None, None)


class MLPBlockFn(torch.autograd.Function):
    """y = x + fc2(gelu(fc1(norm(x))))  (tanh GELU as in the reference, src/nn/activation.rs:206-217)."""

    @staticmethod
    def forward(ctx, x, ln_w, ln_b, w1, b1, w2, b2, eps: float, residual: bool = True):
        B, T, C = x.shape
        x2 = x.reshape(B * T, C)
        h, mean, rstd = K.layer_norm_fwd(x2, ln_w, ln_b, eps)
        pre = torch.empty((B * T, w1.shape[0]), dtype=torch.bfloat16, device=x.device)
        act = K.gemm(h, w1, bias=b1, aux=pre, epilogue=K.EPI_GELU_DUAL)
        y = K.gemm(act, w2, bias=b2, aux=x2, epilogue=K.EPI_RESIDUAL) if residual else K.gemm(act, w2, bias=b2)
        ctx.save_for_backward(x2, ln_w, ln_b, w1, b1, w2, b2, mean, rstd, h, pre, act)
        ctx.meta = (B, T, C, residual)
        return y.view(B, T, C)

    @staticmethod
    def backward(ctx, dy):
        x2, ln_w, ln_b, w1, b1, w2, b2, mean, rstd, h, pre, act = ctx.saved_tensors
        B, T, C, residual = ctx.meta
        dy2 = dy.contiguous().view(B * T, C)
        g_w2 = wgrad_into(dy2, act, w2)
        g_b2 = bgrad_into(dy2, b2)
        dpre = K.gemm(dy2, w2, b_mn=True, aux=pre, epilogue=K.EPI_DGELU)   # [B*T, 4C]
        g_w1 = wgrad_into(dpre, h, w1)
        g_b1 = bgrad_into(dpre, b1)
        dh = K.gemm(dpre, w1, b_mn=True)
        wg, bg, direct = _norm_grad_bufs(ln_w, ln_b)
        dx = _ln_bwd(dh, x2, ln_w, mean, rstd, wg, bg, dy2 if residual else None, direct)
        g_lnw = None if direct else wg.to(ln_w.dtype)
        g_lnb = None if (direct or ln_b is None) else bg.to(ln_b.dtype)
        _notify(w2, b2, w1, b1, ln_w, ln_b)
        return (dx.view(B, T, C), g_lnw, g_lnb, g_w1, g_b1, g_w2, g_b2, None, None)


class EmbeddingFn(torch.autograd.Function):
    """x[b,t] = wte[idx[b,t]] + wpe[t]."""

    @staticmethod
    def forward(ctx, idx, wte, wpe):
        B, T = idx.shape
        out = K.embedding_fwd(idx, wte, wpe, T)
        ctx.save_for_backward(idx, wte, wpe)
        return out

    @staticmethod
    def backward(ctx, dout):
        idx, wte, wpe = ctx.saved_tensors
        T = idx.shape[1]
        direct = getattr(wte, "main_grad", None) is not None
        if direct:
            dwte = wte.main_grad.view(wte.shape)
            dwpe = wpe.main_grad.view(wpe.shape) if wpe is not None else None
        else:
            dwte = torch.zeros(wte.shape, dtype=torch.float32, device=wte.device)
            dwpe = torch.zeros(wpe.shape, dtype=torch.float32, device=wte.device) if wpe is not None else None
        K.embedding_bwd(idx, dout, dwte, dwpe, T, wte.shape[0])
        _notify(wte, wpe)
        if direct:
            return None, None, None
        return None, dwte.to(wte.dtype), (dwpe.to(wpe.dtype) if wpe is not None else None)


class LMHeadLossFn(torch.autograd.Function):
    """loss = mean over the non-ignored rows of CE(lm_head(norm(x)), targets); logits stay bf16 and become their
    own (unscaled) gradient ``softmax - onehot`` in the forward pass.

    ``w_head`` is ``[vocab_padded, C]`` (rows >= ``vocab`` are padding that receives zero
    gradient); padding keeps logits rows 16-byte aligned for vector access.  The factor
    ``dloss / n_valid`` (upstream gradient over the number of rows that are not ``ignore_index``, the
    normalisation of ``F.cross_entropy``) never visits the host: it is a one-element device tensor that
    the weight- and input-gradient GEMMs multiply into their epilogues, so ``(2 * loss).backward()``
    and a loss scaler give exact gradients.
    """

    @staticmethod
    def forward(ctx, x, ln_w, ln_b, w_head, targets, vocab: int, eps: float, ignore_index: int):
        B, T, C = x.shape
        x2 = x.reshape(B * T, C)
        h, mean, rstd = K.layer_norm_fwd(x2, ln_w, ln_b, eps)
        logits = K.gemm(h, w_head)                                # [B*T, Vp]
        tgt = targets.reshape(-1)
        losses = K.cross_entropy_(logits, tgt, vocab, 1.0, ignore_index)   # rows == ignore_index: zero loss, zero gradient
        inv_valid = (tgt != ignore_index).sum().clamp_(min=1).to(torch.float32).reciprocal_().view(1)
        loss = K.reduce_all(losses, "sum")[0] * inv_valid[0]
        ctx.save_for_backward(x2, ln_w, ln_b, w_head, mean, rstd, h, logits, inv_valid)
        ctx.meta = (B, T, C)
        return loss

    @staticmethod
    def backward(ctx, dloss):
        x2, ln_w, ln_b, w_head, mean, rstd, h, dlogits, inv_valid = ctx.saved_tensors
        B, T, C = ctx.meta
        factor = (inv_valid * dloss.to(torch.float32)).view(1)    # device scalar, folded into both GEMM epilogues
        g_head = wgrad_into(dlogits, h, w_head, alpha_dev=factor)
        dh = K.gemm(dlogits, w_head, b_mn=True, alpha_dev=factor)
        wg, bg, direct = _norm_grad_bufs(ln_w, ln_b)
        dx = _ln_bwd(dh, x2, ln_w, mean, rstd, wg, bg, None, direct)
        g_lnw = None if direct else wg.to(ln_w.dtype)
        g_lnb = None if (direct or ln_b is None) else bg.to(ln_b.dtype)
        _notify(w_head, ln_w, ln_b)
        return dx.view(B, T, C), g_lnw, g_lnb, g_head, None, None, None, None


class LinearFn(torch.autograd.Function):
    """y = x W^T + b on the tcgen05 GEMM (forward, dgrad and wgrad without transposed copies)."""

    @staticmethod
    def forward(ctx, x, w, b):
        x2 = x.reshape(-1, x.shape[-1])
        y = K.gemm(x2, w, bias=b)
        ctx.save_for_backward(x2, w, b)
        ctx.xshape = x.shape
        return y.view(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, w, b = ctx.saved_tensors
        dy2 = dy.contiguous().view(-1, w.shape[0])
        gw = wgrad_into(dy2, x2, w) if ctx.needs_input_grad[1] else None
        gb = bgrad_into(dy2, b) if (b is not None and ctx.needs_input_grad[2]) else None
        dx = K.gemm(dy2, w, b_mn=True).view(ctx.xshape) if ctx.needs_input_grad[0] else None
        _notify(w, b)
        return dx, gw, gb


class LayerNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, b, eps):
        x2 = x.reshape(-1, w.numel())
        y, mean, rstd = K.layer_norm_fwd(x2, w, b, eps)
        ctx.save_for_backward(x2, w, b, mean, rstd)
        ctx.xshape = x.shape
        return y.view(x.shape)

    @staticmethod
    def backward(ctx, dy):
        x2, w, b, mean, rstd = ctx.saved_tensors
        wg, bg, direct = _norm_grad_bufs(w, b)
        dx = K.layer_norm_bwd(dy.contiguous().view(x2.shape), x2, w, mean, rstd, wg, bg)
        _notify(w, b)
        return (dx.view(ctx.xshape), None if direct else wg.to(w.dtype),
                None if (direct or b is None) else bg.to(b.dtype), None)


class RMSNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, eps):
        x2 = x.reshape(-1, w.numel())
        y, rstd = K.rms_norm_fwd(x2, w, eps)
        ctx.save_for_backward(x2, w, rstd)
        ctx.xshape = x.shape
        return y.view(x.shape)

    @staticmethod
    def backward(ctx, dy):
        x2, w, rstd = ctx.saved_tensors
        wg, _, direct = _norm_grad_bufs(w, None)
        dx = K.rms_norm_bwd(dy.contiguous().view(x2.shape), x2, w, rstd, wg)
        _notify(w)
        return dx.view(ctx.xshape), None if direct else wg.to(w.dtype), None


class FlashAttentionFn(torch.autograd.Function):
    """softmax(q k^T * scale [+ causal mask]) v with q [B,T,H,D], k/v [B,T,Hkv,D]."""

    @staticmethod
    def forward(ctx, q, k, v, causal: bool, scale: Optional[float]):
        scale = 1.0 / math.sqrt(q.shape[-1]) if scale is None else scale
        o, lse = K.attention_fwd(q, k, v, causal, scale)
        ctx.save_for_backward(q, k, v, o, lse)
        ctx.meta = (causal, scale)
        return o

    @staticmethod
    def backward(ctx, do):
        q, k, v, o, lse = ctx.saved_tensors
        causal, scale = ctx.meta
        dq, dk, dv = K.attention_bwd(q, k, v, o, do.contiguous(), lse, causal, scale)
        return dq, dk, dv, None, None


class BmmNTFn(torch.autograd.Function):
    """``c[b] = alpha * a[b] @ bt[b]^T`` with a [b, M, K], bt [b, N, K] on the batched tcgen05 GEMM."""

    @staticmethod
    def forward(ctx, a, bt, alpha: float):
        a, bt = a.contiguous(), bt.contiguous()
        ctx.save_for_backward(a, bt)
        ctx.alpha = alpha
        return K.gemm(a, bt, alpha=alpha)

    @staticmethod
    def backward(ctx, dc):
        a, bt = ctx.saved_tensors
        dc = dc.contiguous()
        da = K.gemm(dc, bt, b_mn=True, alpha=ctx.alpha) if ctx.needs_input_grad[0] else None            # dc [M,N] @ bt [N,K]
        dbt = K.gemm(dc, a, a_mn=True, b_mn=True, alpha=ctx.alpha) if ctx.needs_input_grad[1] else None  # dc^T [N,M] @ a [M,K]
        return da, dbt, None


class BmmNNFn(torch.autograd.Function):
    """``c[b] = a[b] @ b[b]`` with a [b, M, K], b [b, K, N] on the batched tcgen05 GEMM (no transposed copies)."""

    @staticmethod
    def forward(ctx, a, b):
        a, b = a.contiguous(), b.contiguous()
        ctx.save_for_backward(a, b)
        return K.gemm(a, b, b_mn=True)

    @staticmethod
    def backward(ctx, dc):
        a, b = ctx.saved_tensors
        dc = dc.contiguous()
        da = K.gemm(dc, b) if ctx.needs_input_grad[0] else None                                 # dc [M,N] . b [K,N]^T
        db = K.gemm(a, dc, a_mn=True, b_mn=True) if ctx.needs_input_grad[1] else None           # a^T [K,M] @ dc [M,N]
        return da, db


def materialized_attention(q, k, v, bias: Optional[torch.Tensor], p_drop: float, scale: Optional[float] = None):
    """Attention with an explicit probability matrix, for the cases the flash kernels do not take (additive masks,
    key-padding masks, dropout on the probabilities, returning the weights): batched tcgen05 GEMM for ``q k^T``, the
    native row-softmax and Philox dropout kernels, and a second batched GEMM for ``p v``.  q [B, Tq, H, D], k / v
    [B, Tk, H, D] bf16, ``bias`` broadcastable to [B, H, Tq, Tk] (0 = keep, large negative = masked).
    Returns ``(o [B, Tq, H, D], probabilities [B, H, Tq, Tk])``.  Tq, Tk and D must be multiples of 8."""
    from ..ops import elementwise as E
    from ..ops.pool import dropout as native_dropout
    B, Tq, H, D = q.shape
    Tk = k.shape[1]
    scale = 1.0 / math.sqrt(D) if scale is None else scale
    qb = q.transpose(1, 2).reshape(B * H, Tq, D)
    kb = k.transpose(1, 2).reshape(B * H, Tk, D)
    vb = v.transpose(1, 2).reshape(B * H, Tk, D)
    s = BmmNTFn.apply(qb, kb, scale)                                         # [BH, Tq, Tk]
    if bias is not None:
        s = E.add(s, bias.to(s.dtype).expand(B, H, Tq, Tk).reshape(B * H, Tq, Tk).contiguous())
    w = E.softmax(s, -1)
    wd = native_dropout(w, p_drop, True) if p_drop > 0.0 else w
    o = BmmNNFn.apply(wd, vb)                                                # [BH, Tq, D]
    return o.view(B, H, Tq, D).transpose(1, 2), w.view(B, H, Tq, Tk)


def _split_bf16(t: torch.Tensor):
    """fp32 ``t`` as ``hi + lo`` with both parts in bf16 (16 mantissa bits between them; tf32 keeps 10)."""
    hi = t.to(torch.bfloat16)
    lo = (t - hi.float()).to(torch.bfloat16)
    return hi, lo


def _gemm3(a, b, a_mn, b_mn, out):
    """``out (fp32) = a @ b`` for fp32 operands on the bf16 tensor cores: ``a_hi b_hi + a_hi b_lo + a_lo b_hi`` with
    fp32 accumulation (the dropped ``a_lo b_lo`` term is ~2^-16 of the product)."""
    ah, al = _split_bf16(a)
    bh, bl = _split_bf16(b)
    K.gemm(ah, bh, a_mn=a_mn, b_mn=b_mn, out=out)
    K.gemm(ah, bl, a_mn=a_mn, b_mn=b_mn, out=out, accumulate=True)
    K.gemm(al, bh, a_mn=a_mn, b_mn=b_mn, out=out, accumulate=True)
    return out


class LinearF32Fn(torch.autograd.Function):
    """``y = x W^T + b`` for fp32 tensors on the tcgen05 GEMM: every operand is split into two bf16 parts and the
    product is three bf16 GEMMs accumulated in fp32 (relative error ~2e-5, below tf32's ~5e-4); forward, input
    gradient and weight gradient read the same row-major tensors.  The reference's fp32 matmul is one cuBLAS SGEMM
    (src/gpu/cuda_enhanced.rs:122-159)."""

    @staticmethod
    def forward(ctx, x, w, b):
        x2 = x.reshape(-1, x.shape[-1]).contiguous()
        y = torch.empty((x2.shape[0], w.shape[0]), dtype=torch.float32, device=x.device)
        _gemm3(x2, w, False, False, y)
        if b is not None:
            y += b
        ctx.save_for_backward(x2, w)
        ctx.meta = (x.shape, b is not None)
        return y.view(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, w = ctx.saved_tensors
        xshape, has_b = ctx.meta
        dy2 = dy.reshape(-1, w.shape[0]).contiguous()
        dx = gw = gb = None
        if ctx.needs_input_grad[0]:
            dx = _gemm3(dy2, w, False, True, torch.empty_like(x2)).view(xshape)
        if ctx.needs_input_grad[1]:
            gw = _gemm3(dy2, x2, True, True, torch.empty_like(w))
        if has_b and ctx.needs_input_grad[2]:
            gb = dy2.sum(0)
        return dx, gw, gb


class LinearF16Fn(torch.autograd.Function):
    """``y = x W^T + b`` for fp16 tensors on the tcgen05 GEMM: fp16 operands, fp32 accumulation and output, cast back
    to fp16 (forward, input gradient and weight gradient read the same row-major tensors; no transposed copies)."""

    @staticmethod
    def forward(ctx, x, w, b):
        x2 = x.reshape(-1, x.shape[-1]).contiguous()
        y = K.gemm(x2, w, out_dtype=torch.float32)
        if b is not None:
            y = y + b.float()
        ctx.save_for_backward(x2, w)
        ctx.meta = (x.shape, b is not None)
        return y.to(torch.float16).view(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, w = ctx.saved_tensors
        xshape, has_b = ctx.meta
        dy2 = dy.reshape(-1, w.shape[0]).contiguous()
        dx = K.gemm(dy2, w, b_mn=True, out_dtype=torch.float32).to(torch.float16).view(xshape) if ctx.needs_input_grad[0] else None
        gw = K.gemm(dy2, x2, a_mn=True, b_mn=True, out_dtype=torch.float32).to(torch.float16) if ctx.needs_input_grad[1] else None
        gb = dy2.float().sum(0).to(torch.float16) if (has_b and ctx.needs_input_grad[2]) else None
        return dx, gw, gb
