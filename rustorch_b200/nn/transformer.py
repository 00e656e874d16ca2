"""Multi-head attention and the Transformer encoder / decoder stack.

Signatures follow the reference's exported "phase 6" transformer
(src/nn/transformer_phase6.rs:84-94,157-219,868-880,1067-1079,1298-1312) and the older
attention module (src/nn/attention.rs:92-157): ``MultiheadAttention(embed_dim, num_heads,
dropout=0, bias=True, kdim, vdim, batch_first=True)`` with fused ``in_proj`` (3E) + ``out_proj``
and ``forward(query, key, value, key_padding_mask, need_weights=True, attn_mask,
average_attn_weights=True) -> (out, weights | None)``.  Mask convention: value 0 / False =
masked out (the reference adds -1e9 there, :469-481).

The reference's batch matmul returns a constant 0.1 tensor (:378-418) and its older module
softmaxes over the whole tensor (src/nn/attention.rs:362-384); this implementation computes
real attention.  With bf16 CUDA inputs, no explicit masks (or a causal mask), no dropout and
``need_weights=False`` it runs the hand-written tcgen05 flash-attention kernels; with masks, a key-padding mask,
dropout on the probabilities or ``need_weights=True`` it runs the same math with an explicit probability matrix on
the batched tcgen05 GEMM and the native softmax / dropout kernels (``fused.materialized_attention``).  Only CPU
tensors and other dtypes take the PyTorch expression.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from . import fused
from .layers import LayerNorm, Linear, gelu


class MultiheadAttention(nn.Module):
    def __init__(self, embed_dim: int, num_heads: int, dropout: float = 0.0, bias: bool = True,
                 kdim: Optional[int] = None, vdim: Optional[int] = None, batch_first: bool = True,
                 device=None, dtype=None):
        super().__init__()
        if embed_dim % num_heads != 0:
            raise ValueError("embed_dim must be divisible by num_heads")
        self.embed_dim, self.num_heads, self.head_dim = embed_dim, num_heads, embed_dim // num_heads
        self.dropout, self.batch_first = dropout, batch_first
        self.kdim, self.vdim = kdim or embed_dim, vdim or embed_dim
        self._same_dims = self.kdim == embed_dim and self.vdim == embed_dim
        kw = dict(device=device, dtype=dtype)
        if self._same_dims:
            self.in_proj = Linear(embed_dim, 3 * embed_dim, bias, **kw)
        else:
            self.w_q = Linear(embed_dim, embed_dim, bias, **kw)
            self.w_k = Linear(self.kdim, embed_dim, bias, **kw)
            self.w_v = Linear(self.vdim, embed_dim, bias, **kw)
        self.out_proj = Linear(embed_dim, embed_dim, bias, **kw)

    def split_qkv(self, x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
        """Fused projection of one tensor into q, k, v ``[B, T, E]`` each."""
        return self.in_proj(x).chunk(3, dim=-1)

    def _project(self, query, key, value):
        if self._same_dims:
            if key is query and value is query:
                return self.split_qkv(query)
            E = self.embed_dim
            w, b = self.in_proj.weight, self.in_proj.bias
            bs = (None, None, None) if b is None else (b[:E], b[E:2 * E], b[2 * E:])
            return (F.linear(query, w[:E], bs[0]), F.linear(key, w[E:2 * E], bs[1]), F.linear(value, w[2 * E:], bs[2]))
        return self.w_q(query), self.w_k(key), self.w_v(value)

    @staticmethod
    def _mask_bias(attn_mask, key_padding_mask, is_causal: bool, B: int, Tq: int, Tk: int, like: torch.Tensor):
        """Additive bias [*, *, Tq, Tk] from the masks (reference convention: 0 / False = masked out, -1e9 added there)."""
        bias = None
        if attn_mask is not None:
            bias = torch.zeros(attn_mask.shape, dtype=like.dtype, device=like.device).masked_fill(attn_mask == 0, -1e9)
            while bias.dim() < 4:
                bias = bias.unsqueeze(0)
        if key_padding_mask is not None:
            kp = torch.zeros(B, 1, 1, Tk, dtype=like.dtype, device=like.device).masked_fill(
                (key_padding_mask == 0).view(B, 1, 1, Tk), -1e9)
            bias = kp if bias is None else bias + kp
        if is_causal:
            causal = torch.ones(Tq, Tk, dtype=torch.bool, device=like.device).tril(Tk - Tq)
            cb = torch.zeros(Tq, Tk, dtype=like.dtype, device=like.device).masked_fill(~causal, -1e9)
            bias = cb if bias is None else bias + cb
        return bias

    def forward(self, query, key=None, value=None, key_padding_mask: Optional[torch.Tensor] = None,
                need_weights: bool = True, attn_mask: Optional[torch.Tensor] = None,
                average_attn_weights: bool = True, is_causal: bool = False):
        key = query if key is None else key
        value = key if value is None else value
        if not self.batch_first:
            query, key, value = (t.transpose(0, 1) for t in (query, key, value))
        B, Tq, _ = query.shape
        Tk = key.shape[1]
        H, D = self.num_heads, self.head_dim
        q, k, v = self._project(query, key, value)
        q, k, v = q.reshape(B, Tq, H, D), k.reshape(B, Tk, H, D), v.reshape(B, Tk, H, D)
        p_drop = self.dropout if self.training else 0.0
        native = (q.is_cuda and q.dtype == torch.bfloat16 and not need_weights and key_padding_mask is None
                  and attn_mask is None and p_drop == 0.0 and D in (64, 128))
        weights = None
        own = (q.is_cuda and q.dtype == torch.bfloat16 and D % 8 == 0 and Tq % 8 == 0 and Tk % 8 == 0
               and fused.K._native.available())
        if native:
            o = fused.FlashAttentionFn.apply(q.contiguous(), k.contiguous(), v.contiguous(), is_causal, None)
        elif own:
            bias = self._mask_bias(attn_mask, key_padding_mask, is_causal, B, Tq, Tk, q)
            o, w = fused.materialized_attention(q, k, v, bias, p_drop)
            if need_weights:
                weights = w.mean(1) if average_attn_weights else w
        else:
            qh, kh, vh = (t.transpose(1, 2) for t in (q, k, v))            # [B,H,T,D]
            bias = None
            if attn_mask is not None:
                # reference convention for every mask dtype: 0 / False = masked out, anything else = keep
                bias = torch.zeros(attn_mask.shape, dtype=qh.dtype, device=qh.device).masked_fill(attn_mask == 0, -1e9)
                while bias.dim() < 4:
                    bias = bias.unsqueeze(0)
            if key_padding_mask is not None:
                kp = torch.zeros(B, 1, 1, Tk, dtype=qh.dtype, device=qh.device).masked_fill(
                    (key_padding_mask == 0).view(B, 1, 1, Tk), -1e9)
                bias = kp if bias is None else bias + kp
            if is_causal:
                causal = torch.ones(Tq, Tk, dtype=torch.bool, device=qh.device).tril(Tk - Tq)
                cb = torch.zeros(Tq, Tk, dtype=qh.dtype, device=qh.device).masked_fill(~causal, -1e9)
                bias = cb if bias is None else bias + cb
            if need_weights:
                s = (qh @ kh.transpose(-1, -2)) / math.sqrt(D)
                if bias is not None:
                    s = s + bias
                w = torch.softmax(s, dim=-1)
                w = F.dropout(w, p_drop)
                o = (w @ vh).transpose(1, 2)
                weights = w.mean(1) if average_attn_weights else w
            else:
                o = F.scaled_dot_product_attention(qh, kh, vh, attn_mask=bias, dropout_p=p_drop).transpose(1, 2)
        out = self.out_proj(o.reshape(B, Tq, self.embed_dim))
        if not self.batch_first:
            out = out.transpose(0, 1)
        return out, weights


class SelfAttention(MultiheadAttention):
    """``forward(x, mask)`` convenience (src/nn/attention.rs:466)."""

    def forward(self, x, attn_mask=None, key_padding_mask=None, need_weights: bool = False, is_causal: bool = False, **kw):
        return super().forward(x, x, x, key_padding_mask, need_weights, attn_mask, is_causal=is_causal)


class CrossAttention(MultiheadAttention):
    """``forward(query, context, mask)`` (src/nn/attention.rs:500)."""

    def forward(self, query, context, attn_mask=None, key_padding_mask=None, need_weights: bool = False, **kw):
        return super().forward(query, context, context, key_padding_mask, need_weights, attn_mask)


def _act(name):
    if callable(name):
        return name
    return {"relu": F.relu, "gelu": gelu}[name.lower()]


class TransformerEncoderLayer(nn.Module):
    """``(d_model, nhead, dim_feedforward=2048, dropout=0.1, activation="relu"|"gelu", layer_norm_eps=1e-5,
    batch_first=True, norm_first=False)``; post-norm by default like the reference (:922-976)."""

    def __init__(self, d_model: int, nhead: int, dim_feedforward: int = 2048, dropout: float = 0.1,
                 activation="relu", layer_norm_eps: float = 1e-5, batch_first: bool = True,
                 norm_first: bool = False, device=None, dtype=None):
        super().__init__()
        kw = dict(device=device, dtype=dtype)
        self.self_attn = MultiheadAttention(d_model, nhead, dropout, batch_first=batch_first, **kw)
        self.linear1 = Linear(d_model, dim_feedforward, **kw)
        self.linear2 = Linear(dim_feedforward, d_model, **kw)
        self.norm1 = LayerNorm(d_model, layer_norm_eps, **kw)
        self.norm2 = LayerNorm(d_model, layer_norm_eps, **kw)
        self.dropout = nn.Dropout(dropout)
        self.activation = _act(activation)
        self.norm_first = norm_first

    def _sa(self, x, mask, kpm, causal):
        return self.dropout(self.self_attn(x, x, x, kpm, False, mask, is_causal=causal)[0])

    def _ff(self, x):
        return self.dropout(self.linear2(self.dropout(self.activation(self.linear1(x)))))

    def forward(self, src, src_mask=None, src_key_padding_mask=None, is_causal: bool = False):
        x = src
        if self.norm_first:
            x = x + self._sa(self.norm1(x), src_mask, src_key_padding_mask, is_causal)
            x = x + self._ff(self.norm2(x))
        else:
            x = self.norm1(x + self._sa(x, src_mask, src_key_padding_mask, is_causal))
            x = self.norm2(x + self._ff(x))
        return x


class TransformerDecoderLayer(nn.Module):
    """Self-attention, cross-attention over ``memory``, feed-forward (:1067-1079)."""

    def __init__(self, d_model: int, nhead: int, dim_feedforward: int = 2048, dropout: float = 0.1,
                 activation="relu", layer_norm_eps: float = 1e-5, batch_first: bool = True,
                 norm_first: bool = False, device=None, dtype=None):
        super().__init__()
        kw = dict(device=device, dtype=dtype)
        self.self_attn = MultiheadAttention(d_model, nhead, dropout, batch_first=batch_first, **kw)
        self.multihead_attn = MultiheadAttention(d_model, nhead, dropout, batch_first=batch_first, **kw)
        self.linear1 = Linear(d_model, dim_feedforward, **kw)
        self.linear2 = Linear(dim_feedforward, d_model, **kw)
        self.norm1 = LayerNorm(d_model, layer_norm_eps, **kw)
        self.norm2 = LayerNorm(d_model, layer_norm_eps, **kw)
        self.norm3 = LayerNorm(d_model, layer_norm_eps, **kw)
        self.dropout = nn.Dropout(dropout)
        self.activation = _act(activation)
        self.norm_first = norm_first

    def forward(self, tgt, memory, tgt_mask=None, memory_mask=None, tgt_key_padding_mask=None,
                memory_key_padding_mask=None, tgt_is_causal: bool = False):
        x = tgt
        sa = lambda h: self.dropout(self.self_attn(h, h, h, tgt_key_padding_mask, False, tgt_mask, is_causal=tgt_is_causal)[0])  # noqa: E731
        ca = lambda h: self.dropout(self.multihead_attn(h, memory, memory, memory_key_padding_mask, False, memory_mask)[0])  # noqa: E731
        ff = lambda h: self.dropout(self.linear2(self.dropout(self.activation(self.linear1(h)))))  # noqa: E731
        if self.norm_first:
            x = x + sa(self.norm1(x))
            x = x + ca(self.norm2(x))
            x = x + ff(self.norm3(x))
        else:
            x = self.norm1(x + sa(x))
            x = self.norm2(x + ca(x))
            x = self.norm3(x + ff(x))
        return x


class TransformerEncoder(nn.Module):
    def __init__(self, encoder_layer_fn, num_layers: int, norm: Optional[nn.Module] = None):
        super().__init__()
        self.layers = nn.ModuleList([encoder_layer_fn() for _ in range(num_layers)])
        self.norm = norm

    def forward(self, src, mask=None, src_key_padding_mask=None, is_causal: bool = False):
        x = src
        for l in self.layers:
            x = l(x, mask, src_key_padding_mask, is_causal)
        return self.norm(x) if self.norm is not None else x


class TransformerDecoder(nn.Module):
    def __init__(self, decoder_layer_fn, num_layers: int, norm: Optional[nn.Module] = None):
        super().__init__()
        self.layers = nn.ModuleList([decoder_layer_fn() for _ in range(num_layers)])
        self.norm = norm

    def forward(self, tgt, memory, tgt_mask=None, memory_mask=None, tgt_key_padding_mask=None,
                memory_key_padding_mask=None, tgt_is_causal: bool = False):
        x = tgt
        for l in self.layers:
            x = l(x, memory, tgt_mask, memory_mask, tgt_key_padding_mask, memory_key_padding_mask, tgt_is_causal)
        return self.norm(x) if self.norm is not None else x


class Transformer(nn.Module):
    """``(d_model=512, nhead=8, num_encoder_layers=6, num_decoder_layers=6, dim_feedforward=2048,
    dropout=0.1, activation, custom_encoder, custom_decoder, layer_norm_eps, batch_first, norm_first)``
    with ``forward / encode / decode`` (:1298-1312,1402-1507)."""

    def __init__(self, d_model: int = 512, nhead: int = 8, num_encoder_layers: int = 6, num_decoder_layers: int = 6,
                 dim_feedforward: int = 2048, dropout: float = 0.1, activation="relu", custom_encoder=None,
                 custom_decoder=None, layer_norm_eps: float = 1e-5, batch_first: bool = True,
                 norm_first: bool = False, device=None, dtype=None):
        super().__init__()
        kw = dict(device=device, dtype=dtype)
        mk_e = lambda: TransformerEncoderLayer(d_model, nhead, dim_feedforward, dropout, activation, layer_norm_eps,  # noqa: E731
                                               batch_first, norm_first, **kw)
        mk_d = lambda: TransformerDecoderLayer(d_model, nhead, dim_feedforward, dropout, activation, layer_norm_eps,  # noqa: E731
                                               batch_first, norm_first, **kw)
        self.encoder = custom_encoder or TransformerEncoder(mk_e, num_encoder_layers, LayerNorm(d_model, layer_norm_eps, **kw))
        self.decoder = custom_decoder or TransformerDecoder(mk_d, num_decoder_layers, LayerNorm(d_model, layer_norm_eps, **kw))
        self.d_model, self.nhead = d_model, nhead

    def encode(self, src, src_mask=None, src_key_padding_mask=None):
        return self.encoder(src, src_mask, src_key_padding_mask)

    def decode(self, tgt, memory, tgt_mask=None, memory_mask=None, tgt_key_padding_mask=None,
               memory_key_padding_mask=None):
        return self.decoder(tgt, memory, tgt_mask, memory_mask, tgt_key_padding_mask, memory_key_padding_mask)

    def forward(self, src, tgt, src_mask=None, tgt_mask=None, memory_mask=None, src_key_padding_mask=None,
                tgt_key_padding_mask=None, memory_key_padding_mask=None):
        memory = self.encode(src, src_mask, src_key_padding_mask)
        return self.decode(tgt, memory, tgt_mask, memory_mask, tgt_key_padding_mask, memory_key_padding_mask)

    @staticmethod
    def generate_square_subsequent_mask(size: int, device=None) -> torch.Tensor:
        """Lower-triangular 1/0 mask (1 = may attend)."""
        return torch.ones(size, size, device=device).tril()


from .._interop import accept_wrappers as _accept_wrappers  # noqa: E402

_accept_wrappers(globals())       # forward() of the layers above also takes this package's Tensor / Variable
