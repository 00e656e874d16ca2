"""Llama-family decoder for training: RMSNorm, rotary embeddings, grouped-query attention, SwiGLU MLP
(the model family of the reference's CLI runtime, example-cli/src/model/transformer.rs:9-270, there
forward-only and stubbed; here a trainable module).

On CUDA with bf16 parameters the block runs on the native kernels: RMSNorm forward/backward, tcgen05 GEMMs
for the projections, tcgen05 flash attention with GQA, elementwise SiLU-gate.  With ``tp_group`` set, the model
is tensor- and sequence-parallel in the Megatron layout: tokens are sharded over ranks between blocks, ``wqkv``
and ``w_gate_up`` are column-parallel (one fused all-gather -> GEMM kernel each), ``wo`` and ``w_down`` are
row-parallel (one fused GEMM -> reduce-scatter kernel each); the fused layers live in
``rustorch_b200.distributed.tp_fused``.  Elsewhere (CPU, fp32) the same math runs through PyTorch ops.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..nn import fused
from ..ops import elementwise as ew


@dataclass
class LlamaTrainConfig:
    vocab_size: int = 32000
    n_layer: int = 32
    n_embd: int = 4096
    n_head: int = 32
    n_head_kv: int = 32
    n_ff: int = 11008
    max_seq_len: int = 4096
    rope_theta: float = 10000.0
    rms_eps: float = 1e-5
    init_std: float = 0.02
    rope_scaling: Optional[dict] = None          # Hugging Face ``rope_scaling`` entry: linear or llama3 (see scale_rope_frequencies)

    @property
    def head_dim(self) -> int:
        return self.n_embd // self.n_head

    @staticmethod
    def llama_7b() -> "LlamaTrainConfig":
        return LlamaTrainConfig()

    @staticmethod
    def llama3_8b() -> "LlamaTrainConfig":
        return LlamaTrainConfig(vocab_size=128256, n_head_kv=8, n_ff=14336, max_seq_len=8192, rope_theta=500000.0)

    @staticmethod
    def tiny(**kw) -> "LlamaTrainConfig":
        base = dict(vocab_size=512, n_layer=2, n_embd=256, n_head=4, n_head_kv=2, n_ff=512, max_seq_len=256)
        base.update(kw)
        return LlamaTrainConfig(**base)


def scale_rope_frequencies(inv: torch.Tensor, scaling: Optional[dict]) -> torch.Tensor:
    """Long-context variants of the rotation frequencies.  ``{"rope_type": "linear", "factor": f}`` divides every
    frequency by ``f``; ``"llama3"`` (Llama 3.1 onwards) divides only the low frequencies (wavelength above
    ``original_max_position_embeddings / low_freq_factor``), leaves the high ones (wavelength below
    ``original / high_freq_factor``) and blends in between; ``{"rope_type": "factors", "factors": [...]}`` divides
    frequency ``i`` by ``factors[i]`` (the ``rope_freqs.weight`` tensor of GGUF files)."""
    if not scaling:
        return inv
    kind = str(scaling.get("rope_type", scaling.get("type", "default"))).lower()
    if kind in ("default", "none"):
        return inv
    if kind == "factors":
        div = torch.as_tensor(scaling["factors"], dtype=inv.dtype, device=inv.device)
        if div.shape != inv.shape:
            raise ValueError(f"rope frequency factors: {tuple(div.shape)} for {tuple(inv.shape)} frequencies")
        return inv / div
    factor = float(scaling["factor"])
    if kind == "linear":
        return inv / factor
    if kind != "llama3":
        raise ValueError(f"rope scaling {kind!r} is not implemented (linear, llama3 and per-frequency factors are)")
    lo, hi = float(scaling.get("low_freq_factor", 1.0)), float(scaling.get("high_freq_factor", 4.0))
    old = float(scaling["original_max_position_embeddings"])
    wavelen = 2 * math.pi / inv
    scaled = torch.where(wavelen > old / lo, inv / factor, inv)
    smooth = (old / wavelen - lo) / (hi - lo)
    blended = (1 - smooth) * scaled / factor + smooth * scaled
    medium = ~(wavelen < old / hi) & ~(wavelen > old / lo)
    return torch.where(medium, blended, scaled)


def rope_tables(T: int, D: int, theta: float, device, dtype=torch.float32, scaling: Optional[dict] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    inv = scale_rope_frequencies(theta ** (-torch.arange(0, D, 2, device=device, dtype=torch.float32) / D), scaling)
    ang = torch.arange(T, device=device, dtype=torch.float32)[:, None] * inv[None, :]
    return ang.cos().to(dtype), ang.sin().to(dtype)


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """``x [B, T, H, D]``, half-split pairs ``(i, i + D/2)`` (the HuggingFace Llama convention)."""
    half = x.shape[-1] // 2
    a, b = x[..., :half], x[..., half:]
    c, s = cos[None, : x.shape[1], None, :], sin[None, : x.shape[1], None, :]
    return torch.cat([a * c - b * s, a * s + b * c], -1).to(x.dtype)


class _RopeSplit(torch.autograd.Function):
    """qkv ``[B*T, (H + 2 Hkv) D]`` -> rotated q ``[B, T, H, D]``, rotated k and v ``[B, T, Hkv, D]`` in one kernel
    (csrc/nn/llama_ops.cu); backward packs the three gradients back with the inverse rotation."""

    @staticmethod
    def forward(ctx, qkv, cos, sin, B, T, H, Hkv, D):
        from .. import _native
        C = _native.load(required=True)
        qkv = qkv.contiguous()
        q = torch.empty((B, T, H, D), dtype=qkv.dtype, device=qkv.device)
        k = torch.empty((B, T, Hkv, D), dtype=qkv.dtype, device=qkv.device)
        v = torch.empty_like(k)
        C.rope_split(qkv, q, k, v, cos, sin, T, False)
        ctx.save_for_backward(cos, sin)
        ctx.geom = (B, T, H, Hkv, D)
        return q, k, v

    @staticmethod
    def backward(ctx, dq, dk, dv):
        from .. import _native
        C = _native.load(required=True)
        cos, sin = ctx.saved_tensors
        B, T, H, Hkv, D = ctx.geom
        dqkv = torch.empty((B * T, (H + 2 * Hkv) * D), dtype=dq.dtype, device=dq.device)
        C.rope_split(dqkv, dq.contiguous(), dk.contiguous(), dv.contiguous(), cos, sin, T, True)
        return dqkv, None, None, None, None, None, None, None


class _SwiGLU(torch.autograd.Function):
    """``silu(gu[:, :F]) * gu[:, F:]`` forward and backward as one kernel each (csrc/nn/llama_ops.cu)."""

    @staticmethod
    def forward(ctx, gu):
        from .. import _native
        C = _native.load(required=True)
        gu = gu.contiguous()
        act = torch.empty((gu.shape[0], gu.shape[1] // 2), dtype=gu.dtype, device=gu.device)
        C.swiglu(gu, None, act, False)
        ctx.save_for_backward(gu)
        return act

    @staticmethod
    def backward(ctx, dact):
        from .. import _native
        C = _native.load(required=True)
        (gu,) = ctx.saved_tensors
        dgu = torch.empty_like(gu)
        C.swiglu(gu, dact.contiguous(), dgu, True)
        return dgu


# True: every op of the model runs on stock PyTorch kernels (cuBLAS, SDPA, ATen elementwise, NCCL collectives): the
# baseline arm of benchmarks/llama_tp_bench.py.  The default is the native path.
LIBRARY_MODE = False
# True: every block is recomputed in backward (activation checkpointing), for models whose activations do not fit.
CHECKPOINT_BLOCKS = False


def _native_ok(x: torch.Tensor) -> bool:
    return x.is_cuda and x.dtype == torch.bfloat16 and not LIBRARY_MODE


def _rms(x, w, eps):
    if _native_ok(x):
        return fused.RMSNormFn.apply(x, w, eps)
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * w.float()).to(x.dtype)


def _linear(x2, w):
    return fused.LinearFn.apply(x2, w, None) if _native_ok(x2) else x2 @ w.t()


def _attention(q, k, v):
    if _native_ok(q) and q.shape[-1] in (64, 128):
        return fused.FlashAttentionFn.apply(q, k, v, True, None)
    if q.is_cuda and q.shape[2] != k.shape[2]:
        return F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), is_causal=True,
                                              enable_gqa=True).transpose(1, 2)
    g = q.shape[2] // k.shape[2]
    kk, vv = k.repeat_interleave(g, 2), v.repeat_interleave(g, 2)
    return F.scaled_dot_product_attention(q.transpose(1, 2), kk.transpose(1, 2), vv.transpose(1, 2), is_causal=True).transpose(1, 2)


class LlamaBlock(nn.Module):
    def shard_spec(self) -> dict:
        """How the fused projections are cut over tensor-parallel ranks (``training.sharded``): q | k | v and gate | up
        are sharded part by part, so a rank holds the concatenation of its slice of every part."""
        from ..training.sharded import ShardSpec
        c = self.cfg
        D = c.head_dim
        dot = ".weight" if self.tp else ""
        return {"wqkv" + dot: ShardSpec(0, [c.n_head * D, c.n_head_kv * D, c.n_head_kv * D]),
                "w_gate_up" + dot: ShardSpec(0, [c.n_ff, c.n_ff]),
                "wo" + dot: ShardSpec(1), "w_down" + dot: ShardSpec(1)}

    def __init__(self, cfg: LlamaTrainConfig, device=None, dtype=None, tp_group=None, rows_per_rank: int = 0):
        super().__init__()
        self.cfg = cfg
        kw = dict(device=device, dtype=dtype)
        D, H, Hkv = cfg.head_dim, cfg.n_head, cfg.n_head_kv
        self.tp = tp_group is not None
        self.attn_norm = nn.Parameter(torch.ones(cfg.n_embd, **kw))
        self.ffn_norm = nn.Parameter(torch.ones(cfg.n_embd, **kw))
        if self.tp:
            import torch.distributed as dist
            if LIBRARY_MODE:
                from ..distributed.tp_library import LibraryColumnParallelLinear as FusedColumnParallelLinear
                from ..distributed.tp_library import LibraryRowParallelLinear as FusedRowParallelLinear
            else:
                from ..distributed.tp_fused import FusedColumnParallelLinear, FusedRowParallelLinear
            W = dist.get_world_size(tp_group)
            if H % W or Hkv % W or cfg.n_ff % W:
                raise ValueError("heads, kv heads and n_ff must divide by the tensor-parallel world size")
            self.h_local, self.hkv_local, self.ff_local = H // W, Hkv // W, cfg.n_ff // W
            self.wqkv = FusedColumnParallelLinear(cfg.n_embd, (H + 2 * Hkv) * D, rows_per_rank, False, tp_group, device, cfg.init_std)
            self.wo = FusedRowParallelLinear(H * D, cfg.n_embd, rows_per_rank, False, tp_group, device, cfg.init_std / math.sqrt(2 * cfg.n_layer))
            self.w_gate_up = FusedColumnParallelLinear(cfg.n_embd, 2 * cfg.n_ff, rows_per_rank, False, tp_group, device, cfg.init_std)
            self.w_down = FusedRowParallelLinear(cfg.n_ff, cfg.n_embd, rows_per_rank, False, tp_group, device, cfg.init_std / math.sqrt(2 * cfg.n_layer))
        else:
            self.h_local, self.hkv_local, self.ff_local = H, Hkv, cfg.n_ff
            self.wqkv = nn.Parameter(torch.randn((H + 2 * Hkv) * D, cfg.n_embd, **kw) * cfg.init_std)
            self.wo = nn.Parameter(torch.randn(cfg.n_embd, H * D, **kw) * cfg.init_std / math.sqrt(2 * cfg.n_layer))
            self.w_gate_up = nn.Parameter(torch.randn(2 * cfg.n_ff, cfg.n_embd, **kw) * cfg.init_std)
            self.w_down = nn.Parameter(torch.randn(cfg.n_embd, cfg.n_ff, **kw) * cfg.init_std / math.sqrt(2 * cfg.n_layer))

    def forward(self, x: torch.Tensor, cos, sin, B: int, T: int) -> torch.Tensor:
        """``x``: ``[B*T, d]`` (or this rank's rows of it under tensor parallelism)."""
        c = self.cfg
        D, H, Hkv = c.head_dim, self.h_local, self.hkv_local
        h = _rms(x, self.attn_norm, c.rms_eps)
        qkv = self.wqkv(h) if self.tp else _linear(h, self.wqkv)                    # [B*T, (H + 2 Hkv) D] (all tokens)
        if _native_ok(qkv) and D % 16 == 0 and cos.dtype == torch.float32:
            q, k, v = _RopeSplit.apply(qkv, cos, sin, B, T, H, Hkv, D)
        else:
            qkv = qkv.view(B, T, H + 2 * Hkv, D)
            q, k, v = qkv[:, :, :H], qkv[:, :, H:H + Hkv], qkv[:, :, H + Hkv:].contiguous()
            q, k = apply_rope(q, cos, sin), apply_rope(k, cos, sin)
        att = _attention(q, k, v).reshape(B * T, H * D)
        x = x + (self.wo(att) if self.tp else _linear(att, self.wo))
        h = _rms(x, self.ffn_norm, c.rms_eps)
        gu = self.w_gate_up(h) if self.tp else _linear(h, self.w_gate_up)           # [B*T, 2 ff_local]: gate | up
        if _native_ok(gu) and self.ff_local % 8 == 0:
            act = _SwiGLU.apply(gu)
        elif LIBRARY_MODE:
            act = F.silu(gu[:, : self.ff_local]) * gu[:, self.ff_local:]
        else:
            act = ew.mul(ew.unary("silu", gu[:, : self.ff_local].contiguous()), gu[:, self.ff_local:].contiguous())
        return x + (self.w_down(act) if self.tp else _linear(act, self.w_down))


class LlamaModel(nn.Module):
    """``forward(idx [B, T], targets) -> (logits or None, loss)``.  Under tensor parallelism every rank receives the
    same ``idx``; the returned loss is this rank's share of the global mean (sum it over ranks for reporting)."""

    def __init__(self, cfg: LlamaTrainConfig, device=None, dtype=None, tp_group=None, batch: int = 0, seq_len: int = 0):
        super().__init__()
        self.cfg, self.tp_group = cfg, tp_group
        kw = dict(device=device, dtype=dtype)
        self.world, self.rank, rows = 1, 0, 0
        if tp_group is not None:
            import torch.distributed as dist
            self.world, self.rank = dist.get_world_size(tp_group), dist.get_rank(tp_group)
            if batch * seq_len % (128 * self.world):
                raise ValueError("batch * seq_len must be a multiple of 128 * world size for the fused TP kernels")
            rows = batch * seq_len // self.world
        self.tok_emb = nn.Parameter(torch.randn(cfg.vocab_size, cfg.n_embd, **kw) * cfg.init_std)
        self.blocks = nn.ModuleList([LlamaBlock(cfg, device, dtype, tp_group, rows) for _ in range(cfg.n_layer)])
        self.out_norm = nn.Parameter(torch.ones(cfg.n_embd, **kw))
        self.lm_head = nn.Parameter(torch.randn(cfg.vocab_size, cfg.n_embd, **kw) * cfg.init_std)
        self._rope = None

    def num_parameters(self) -> int:
        return sum(p.numel() for p in self.parameters())

    @classmethod
    def from_hf(cls, directory: str, device=None, dtype=None) -> "LlamaModel":
        """A single-rank model with the weights of a Hugging Face Llama checkpoint directory (``config.json`` +
        safetensors, sharded or not), e.g. to fine-tune it.  Same head layout (rotate-half RoPE) as those checkpoints, so
        the tensors are copied as they are: q | k | v stacked into ``wqkv``, gate | up into ``w_gate_up``."""
        from ..formats.safetensors import HuggingFaceCheckpoint, hf_rope_settings
        with HuggingFaceCheckpoint(directory) as ck:
            c = ck.config
            if any(k.endswith(".bias") for k in ck.keys()):
                raise ValueError(f"{directory}: projection biases are outside this model")
            theta, scaling = hf_rope_settings(c)
            if scaling:
                scale_rope_frequencies(torch.ones(1), scaling)               # refuses the kinds that are not implemented
            n_head = int(c["num_attention_heads"])
            cfg = LlamaTrainConfig(vocab_size=int(c["vocab_size"]), n_layer=int(c["num_hidden_layers"]), n_embd=int(c["hidden_size"]),
                                   n_head=n_head, n_head_kv=int(c.get("num_key_value_heads") or n_head), n_ff=int(c["intermediate_size"]),
                                   max_seq_len=int(c.get("max_position_embeddings", 4096)), rope_theta=theta,
                                   rms_eps=float(c.get("rms_norm_eps", 1e-5)), rope_scaling=scaling)
            model = cls(cfg, device=device, dtype=dtype)
            get = lambda n: ck.get(n).to(device=device, dtype=dtype or torch.float32)      # noqa: E731
            with torch.no_grad():
                model.tok_emb.copy_(get("model.embed_tokens.weight"))
                model.out_norm.copy_(get("model.norm.weight"))
                model.lm_head.copy_(get("lm_head.weight" if "lm_head.weight" in ck else "model.embed_tokens.weight"))
                for i, b in enumerate(model.blocks):
                    p = f"model.layers.{i}."
                    b.wqkv.copy_(torch.cat([get(p + f"self_attn.{n}_proj.weight") for n in ("q", "k", "v")], 0))
                    b.wo.copy_(get(p + "self_attn.o_proj.weight"))
                    b.w_gate_up.copy_(torch.cat([get(p + "mlp.gate_proj.weight"), get(p + "mlp.up_proj.weight")], 0))
                    b.w_down.copy_(get(p + "mlp.down_proj.weight"))
                    b.attn_norm.copy_(get(p + "input_layernorm.weight"))
                    b.ffn_norm.copy_(get(p + "post_attention_layernorm.weight"))
        return model

    def forward(self, idx: torch.Tensor, targets: Optional[torch.Tensor] = None):
        B, T = idx.shape
        c = self.cfg
        if self._rope is None or self._rope[0].shape[0] < T or self._rope[0].device != idx.device:
            self._rope = rope_tables(max(T, c.max_seq_len), c.head_dim, c.rope_theta, idx.device, scaling=c.rope_scaling)
        cos, sin = self._rope
        flat = idx.reshape(-1)
        lo, hi = 0, B * T
        if self.world > 1:
            n = B * T // self.world
            lo, hi = self.rank * n, (self.rank + 1) * n
        x = self.tok_emb[flat[lo:hi]]
        for blk in self.blocks:
            if CHECKPOINT_BLOCKS and torch.is_grad_enabled():
                from torch.utils.checkpoint import checkpoint
                x = checkpoint(blk, x, cos, sin, B, T, use_reentrant=False)   # keep only the block inputs
            else:
                x = blk(x, cos, sin, B, T)
        x = _rms(x, self.out_norm, c.rms_eps)
        logits = _linear(x, self.lm_head)
        if targets is None:
            return logits.view(-1, c.vocab_size), None
        # under tensor parallelism each rank owns 1/W of the tokens: its loss term is scaled so that the terms of all
        # ranks add up to the global mean (gradients of sharded weights are then exact, see sync_replicated_grads)
        loss = F.cross_entropy(logits.float(), targets.reshape(-1)[lo:hi]) / self.world
        return logits, loss

    def save_hf(self, directory: str, dtype: torch.dtype = torch.float32) -> None:
        """Writes a Hugging Face Llama checkpoint directory (``config.json`` + ``model.safetensors``) from a single-rank
        model: the inverse of :meth:`from_hf`, readable by ``transformers`` and by ``llm.hf_to_gguf``."""
        import json
        import os
        from ..formats.safetensors import save_safetensors
        if self.world > 1:
            raise ValueError("gather a tensor-parallel model to one rank before saving it")
        c = self.cfg
        H, Hkv, D = c.n_head, c.n_head_kv, c.head_dim
        cast = lambda t: t.detach().to("cpu", dtype).contiguous()      # noqa: E731
        sd = {"model.embed_tokens.weight": cast(self.tok_emb), "model.norm.weight": cast(self.out_norm), "lm_head.weight": cast(self.lm_head)}
        for i, b in enumerate(self.blocks):
            p = f"model.layers.{i}."
            q, k, v = b.wqkv.split([H * D, Hkv * D, Hkv * D], 0)
            gate, up = b.w_gate_up.split([c.n_ff, c.n_ff], 0)
            sd.update({p + "self_attn.q_proj.weight": cast(q), p + "self_attn.k_proj.weight": cast(k), p + "self_attn.v_proj.weight": cast(v),
                       p + "self_attn.o_proj.weight": cast(b.wo), p + "mlp.gate_proj.weight": cast(gate), p + "mlp.up_proj.weight": cast(up),
                       p + "mlp.down_proj.weight": cast(b.w_down), p + "input_layernorm.weight": cast(b.attn_norm),
                       p + "post_attention_layernorm.weight": cast(b.ffn_norm)})
        os.makedirs(directory, exist_ok=True)
        save_safetensors(sd, os.path.join(directory, "model.safetensors"), {"format": "pt"})
        name = {torch.float32: "float32", torch.bfloat16: "bfloat16", torch.float16: "float16"}[dtype]
        with open(os.path.join(directory, "config.json"), "w") as f:
            json.dump({"architectures": ["LlamaForCausalLM"], "model_type": "llama", "vocab_size": c.vocab_size, "hidden_size": c.n_embd,
                       "intermediate_size": c.n_ff, "num_hidden_layers": c.n_layer, "num_attention_heads": H, "num_key_value_heads": Hkv,
                       "hidden_act": "silu", "max_position_embeddings": c.max_seq_len, "rms_norm_eps": c.rms_eps, "rope_theta": c.rope_theta,
                       "rope_scaling": c.rope_scaling,
                       "rope_parameters": {"rope_theta": c.rope_theta, **(c.rope_scaling or {"rope_type": "default"})},
                       "tie_word_embeddings": False, "attention_bias": False, "mlp_bias": False, "torch_dtype": name}, f, indent=2)

    def replicated_parameters(self):
        """Parameters every rank holds in full (embeddings, head, norm weights): their gradients are partial sums
        over this rank's tokens."""
        yield self.tok_emb
        yield self.lm_head
        yield self.out_norm
        for b in self.blocks:
            yield b.attn_norm
            yield b.ffn_norm

    def sync_replicated_grads(self) -> None:
        """Sum the gradients of the replicated parameters over the tensor-parallel group (call after backward)."""
        if self.world == 1:
            return
        import torch.distributed as dist
        small = [p.grad for p in self.replicated_parameters() if p.grad is not None and p.grad.numel() < (1 << 20)]
        if small:
            flat = torch.cat([g.reshape(-1).float() for g in small])
            dist.all_reduce(flat, group=self.tp_group)
            o = 0
            for g in small:
                g.copy_(flat[o:o + g.numel()].view_as(g))
                o += g.numel()
        for p in self.replicated_parameters():
            if p.grad is not None and p.grad.numel() >= (1 << 20):
                dist.all_reduce(p.grad, group=self.tp_group)

    @torch.no_grad()
    def load_from_unsharded(self, full: "LlamaModel") -> None:
        """Copy (and shard) the weights of a single-rank model with the same config: used by tests and for resharding."""
        W, r = self.world, self.rank
        self.tok_emb.copy_(full.tok_emb); self.out_norm.copy_(full.out_norm); self.lm_head.copy_(full.lm_head)
        c = self.cfg
        D, H, Hkv = c.head_dim, c.n_head, c.n_head_kv
        for mine, ref in zip(self.blocks, full.blocks):
            mine.attn_norm.copy_(ref.attn_norm); mine.ffn_norm.copy_(ref.ffn_norm)
            if not mine.tp:
                for n in ("wqkv", "wo", "w_gate_up", "w_down"):
                    getattr(mine, n).copy_(getattr(ref, n))
                continue
            hl, kl, fl = H // W, Hkv // W, c.n_ff // W
            q, k, v = ref.wqkv[: H * D], ref.wqkv[H * D:(H + Hkv) * D], ref.wqkv[(H + Hkv) * D:]
            mine.wqkv.weight.copy_(torch.cat([q[r * hl * D:(r + 1) * hl * D], k[r * kl * D:(r + 1) * kl * D], v[r * kl * D:(r + 1) * kl * D]]))
            mine.wo.weight.copy_(ref.wo[:, r * hl * D:(r + 1) * hl * D])
            g, u = ref.w_gate_up[: c.n_ff], ref.w_gate_up[c.n_ff:]
            mine.w_gate_up.weight.copy_(torch.cat([g[r * fl:(r + 1) * fl], u[r * fl:(r + 1) * fl]]))
            mine.w_down.weight.copy_(ref.w_down[:, r * fl:(r + 1) * fl])
