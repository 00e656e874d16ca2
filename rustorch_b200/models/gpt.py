"""GPT-2 style decoder-only language model.

Config defaults follow the reference's ``GPTConfig`` (vocab 50257, n_positions 1024, n_embd 768,
n_layer 12, n_head 12, dropout 0.1; src/models/transformer_models.rs:727-738) and its structure
(token embedding + learned positional embedding + N blocks + final LayerNorm + a separate
``lm_head`` Linear, :760-796).  Where the reference is stubbed or wrong the standard GPT-2
semantics are used instead: causal self-attention (the reference passes no mask, :846-848),
pre-LayerNorm blocks, tanh-GELU MLP, and a working attention (the reference's batch matmul
returns a constant, src/nn/transformer_phase6.rs:378-418).

On CUDA with bf16 parameters the forward/backward runs on the fused native blocks of
:mod:`rustorch_b200.nn.fused`; :meth:`GPT.forward_reference` is the plain PyTorch restatement
used as the CPU path and as the numerics oracle in tests.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, asdict
from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..nn import fused


@dataclass
class GPTConfig:
    vocab_size: int = 50257
    n_positions: int = 1024
    n_embd: int = 768
    n_layer: int = 12
    n_head: int = 12
    dropout: float = 0.1
    layer_norm_eps: float = 1e-5
    tie_weights: bool = False
    init_std: float = 0.02

    @property
    def padded_vocab(self) -> int:
        return -(-self.vocab_size // 64) * 64

    @staticmethod
    def gpt2_small(**kw) -> "GPTConfig":
        return GPTConfig(**kw)

    @staticmethod
    def gpt2_medium(**kw) -> "GPTConfig":
        return GPTConfig(n_embd=1024, n_layer=24, n_head=16, **kw)

    def to_dict(self) -> dict:
        return asdict(self)


class GPTBlock(nn.Module):
    """Parameters of one transformer block of the fused GPT model (the block's arithmetic lives in ``nn.fused``)."""

    def __init__(self, cfg: GPTConfig, device=None, dtype=None):
        super().__init__()
        C = cfg.n_embd
        kw = dict(device=device, dtype=dtype)
        self.ln1_w = nn.Parameter(torch.ones(C, **kw))
        self.ln1_b = nn.Parameter(torch.zeros(C, **kw))
        self.w_qkv = nn.Parameter(torch.empty(3 * C, C, **kw))
        self.b_qkv = nn.Parameter(torch.zeros(3 * C, **kw))
        self.w_proj = nn.Parameter(torch.empty(C, C, **kw))
        self.b_proj = nn.Parameter(torch.zeros(C, **kw))
        self.ln2_w = nn.Parameter(torch.ones(C, **kw))
        self.ln2_b = nn.Parameter(torch.zeros(C, **kw))
        self.w_fc = nn.Parameter(torch.empty(4 * C, C, **kw))
        self.b_fc = nn.Parameter(torch.zeros(4 * C, **kw))
        self.w_fc2 = nn.Parameter(torch.empty(C, 4 * C, **kw))
        self.b_fc2 = nn.Parameter(torch.zeros(C, **kw))


class GPT(nn.Module):
    def __init__(self, cfg: GPTConfig, device=None, dtype=torch.float32, seed: Optional[int] = None):
        super().__init__()
        self.cfg = cfg
        C, Vp = cfg.n_embd, cfg.padded_vocab
        kw = dict(device=device, dtype=dtype)
        self.wte = nn.Parameter(torch.empty(Vp, C, **kw))
        self.wpe = nn.Parameter(torch.empty(cfg.n_positions, C, **kw))
        self.blocks = nn.ModuleList([GPTBlock(cfg, device, dtype) for _ in range(cfg.n_layer)])
        self.lnf_w = nn.Parameter(torch.ones(C, **kw))
        self.lnf_b = nn.Parameter(torch.zeros(C, **kw))
        if cfg.tie_weights:
            self.lm_head = self.wte
            self.wte._grad_contribs = 2  # embedding backward + lm_head backward
        else:
            self.lm_head = nn.Parameter(torch.empty(Vp, C, **kw))
        self.reset_parameters(seed)

    # ------------------------------------------------------------------ init
    def reset_parameters(self, seed: Optional[int] = None) -> None:
        g = None
        if seed is not None:
            g = torch.Generator(device="cpu")
            g.manual_seed(seed)
        std = self.cfg.init_std

        def normal_(p: torch.Tensor, rows: Optional[int] = None):
            w = torch.empty(p.shape, dtype=torch.float32).normal_(0.0, std, generator=g)
            if rows is not None:
                w[rows:] = 0
            with torch.no_grad():
                p.copy_(w)
            if p.dtype != torch.float32:
                p._fp32_init = w.to(p.device)  # lets FlatParams seed exact fp32 master weights

        normal_(self.wte, self.cfg.vocab_size)
        normal_(self.wpe)
        if not self.cfg.tie_weights:
            normal_(self.lm_head, self.cfg.vocab_size)
        for b in self.blocks:
            for w in (b.w_qkv, b.w_proj, b.w_fc, b.w_fc2):
                normal_(w)

    @classmethod
    def from_hf(cls, directory: str, device=None, dtype=torch.float32) -> "GPT":
        """A model with the weights of a Hugging Face GPT-2 checkpoint directory (``config.json`` + safetensors).  GPT-2
        stores its projections as ``Conv1D`` weights ``[in, out]``; they are transposed into the ``[out, in]`` layout of
        this model.  The embedding is padded with zero rows to the model's vocabulary multiple and tied to the head, as
        GPT-2's is."""
        from ..formats.safetensors import HuggingFaceCheckpoint
        with HuggingFaceCheckpoint(directory) as ck:
            c = ck.config
            if c.get("activation_function", "gelu_new") not in ("gelu_new", "gelu_pytorch_tanh"):
                raise ValueError(f"{directory}: activation {c['activation_function']!r}; this model computes the tanh form of GELU")
            pre = "transformer." if any(k.startswith("transformer.") for k in ck.keys()) else ""
            cfg = GPTConfig(vocab_size=int(c["vocab_size"]), n_positions=int(c.get("n_positions", 1024)), n_embd=int(c["n_embd"]),
                            n_layer=int(c["n_layer"]), n_head=int(c["n_head"]), dropout=float(c.get("resid_pdrop", 0.1)),
                            layer_norm_eps=float(c.get("layer_norm_epsilon", 1e-5)), tie_weights=True)
            model = cls(cfg, device=device, dtype=dtype)
            get = lambda n: ck.get(pre + n).to(device=device, dtype=dtype)      # noqa: E731
            with torch.no_grad():
                model.wte.zero_()
                model.wte[: cfg.vocab_size].copy_(get("wte.weight"))
                model.wpe.copy_(get("wpe.weight"))
                model.lnf_w.copy_(get("ln_f.weight"))
                model.lnf_b.copy_(get("ln_f.bias"))
                for i, b in enumerate(model.blocks):
                    h = f"h.{i}."
                    for ours, theirs in (("ln1", "ln_1"), ("ln2", "ln_2")):
                        getattr(b, ours + "_w").copy_(get(h + theirs + ".weight"))
                        getattr(b, ours + "_b").copy_(get(h + theirs + ".bias"))
                    for ours, theirs in (("qkv", "attn.c_attn"), ("proj", "attn.c_proj"), ("fc", "mlp.c_fc"), ("fc2", "mlp.c_proj")):
                        getattr(b, "w_" + ours).copy_(get(h + theirs + ".weight").t())
                        getattr(b, "b_" + ours).copy_(get(h + theirs + ".bias"))
        return model

    def save_hf(self, directory: str) -> None:
        """Writes a Hugging Face GPT-2 checkpoint directory (``config.json`` + ``model.safetensors``): projections go back to
        the ``Conv1D`` layout ``[in, out]``, the vocabulary padding is dropped.  An untied head has no place in that
        format, so the model must tie ``lm_head`` to ``wte``."""
        import json
        import os
        from ..formats.safetensors import save_safetensors
        if not self.cfg.tie_weights:
            raise ValueError("the GPT-2 checkpoint format ties the head to the embedding; this model does not")
        c = self.cfg
        cast = lambda t: t.detach().float().cpu().contiguous()      # noqa: E731
        sd = {"transformer.wte.weight": cast(self.wte[: c.vocab_size]), "transformer.wpe.weight": cast(self.wpe),
              "transformer.ln_f.weight": cast(self.lnf_w), "transformer.ln_f.bias": cast(self.lnf_b)}
        for i, b in enumerate(self.blocks):
            h = f"transformer.h.{i}."
            for ours, theirs in (("ln1", "ln_1"), ("ln2", "ln_2")):
                sd[h + theirs + ".weight"], sd[h + theirs + ".bias"] = cast(getattr(b, ours + "_w")), cast(getattr(b, ours + "_b"))
            for ours, theirs in (("qkv", "attn.c_attn"), ("proj", "attn.c_proj"), ("fc", "mlp.c_fc"), ("fc2", "mlp.c_proj")):
                sd[h + theirs + ".weight"], sd[h + theirs + ".bias"] = cast(getattr(b, "w_" + ours).t()), cast(getattr(b, "b_" + ours))
        os.makedirs(directory, exist_ok=True)
        save_safetensors(sd, os.path.join(directory, "model.safetensors"), {"format": "pt"})
        with open(os.path.join(directory, "config.json"), "w") as f:
            json.dump({"architectures": ["GPT2LMHeadModel"], "model_type": "gpt2", "vocab_size": c.vocab_size, "n_positions": c.n_positions,
                       "n_embd": c.n_embd, "n_layer": c.n_layer, "n_head": c.n_head, "activation_function": "gelu_new",
                       "resid_pdrop": c.dropout, "embd_pdrop": c.dropout, "attn_pdrop": c.dropout, "layer_norm_epsilon": c.layer_norm_eps,
                       "tie_word_embeddings": True}, f, indent=2)

    def num_parameters(self, count_padding: bool = False) -> int:
        n = sum(p.numel() for p in self.parameters())
        if not count_padding:
            pad = (self.cfg.padded_vocab - self.cfg.vocab_size) * self.cfg.n_embd
            n -= pad * (1 if self.cfg.tie_weights else 2)
        return n

    def flops_per_token(self, seq_len: int) -> float:
        """Training FLOPs per token (fwd+bwd = 3x forward): 6*N_matmul + 12*L*C*T (causal halves
        the attention term)."""
        c = self.cfg
        n_mat = c.n_layer * 12 * c.n_embd * c.n_embd + c.vocab_size * c.n_embd
        return 6.0 * n_mat + 6.0 * c.n_layer * c.n_embd * seq_len

    # --------------------------------------------------------------- forward
    def _native_ok(self, idx: torch.Tensor) -> bool:
        return idx.is_cuda and self.wte.dtype == torch.bfloat16

    def forward(self, idx: torch.Tensor, targets: Optional[torch.Tensor] = None):
        if not self._native_ok(idx):
            return self.forward_reference(idx, targets)
        c = self.cfg
        B, T = idx.shape
        assert T <= c.n_positions, "sequence longer than n_positions"
        x = fused.EmbeddingFn.apply(idx, self.wte, self.wpe)
        p_drop = c.dropout if self.training else 0.0
        if p_drop > 0.0:
            # Dropout (reference default 0.1, src/models/transformer_models.rs:727-738) on the embeddings and on both
            # residual branches: the blocks return their branch alone, the Philox dropout kernel (mask regenerated in
            # backward) and the elementwise add kernel finish ``x + dropout(branch)``.  The flash kernel has no dropout
            # on the attention probabilities.
            from ..ops import elementwise as E
            from ..ops.pool import dropout as native_dropout
            x = native_dropout(x, p_drop, True)
            for b in self.blocks:
                br = fused.AttnBlockFn.apply(x, b.ln1_w, b.ln1_b, b.w_qkv, b.b_qkv, b.w_proj, b.b_proj,
                                             c.n_head, c.layer_norm_eps, True, False)
                x = E.add(x, native_dropout(br, p_drop, True))
                br = fused.MLPBlockFn.apply(x, b.ln2_w, b.ln2_b, b.w_fc, b.b_fc, b.w_fc2, b.b_fc2,
                                            c.layer_norm_eps, False)
                x = E.add(x, native_dropout(br, p_drop, True))
        else:
            for b in self.blocks:
                x = fused.AttnBlockFn.apply(x, b.ln1_w, b.ln1_b, b.w_qkv, b.b_qkv, b.w_proj, b.b_proj,
                                            c.n_head, c.layer_norm_eps, True)
                x = fused.MLPBlockFn.apply(x, b.ln2_w, b.ln2_b, b.w_fc, b.b_fc, b.w_fc2, b.b_fc2,
                                           c.layer_norm_eps)
        if targets is not None:
            return fused.LMHeadLossFn.apply(x, self.lnf_w, self.lnf_b, self.lm_head, targets,
                                            c.vocab_size, c.layer_norm_eps, -100)
        h = fused.LayerNormFn.apply(x, self.lnf_w, self.lnf_b, c.layer_norm_eps)
        logits = fused.LinearFn.apply(h, self.lm_head, None)
        return logits[..., :c.vocab_size]

    def forward_reference(self, idx: torch.Tensor, targets: Optional[torch.Tensor] = None):
        """Plain PyTorch restatement (any device / dtype)."""
        c = self.cfg
        B, T = idx.shape
        H, D = c.n_head, c.n_embd // c.n_head
        eps = c.layer_norm_eps
        x = self.wte[idx] + self.wpe[:T]
        p_drop = c.dropout if self.training else 0.0
        x = F.dropout(x, p_drop)
        for b in self.blocks:
            h = F.layer_norm(x, (c.n_embd,), b.ln1_w, b.ln1_b, eps)
            qkv = F.linear(h, b.w_qkv, b.b_qkv).view(B, T, 3, H, D)
            q, k, v = (qkv[:, :, i].transpose(1, 2) for i in range(3))
            att = F.scaled_dot_product_attention(q, k, v, is_causal=True, dropout_p=p_drop)
            att = att.transpose(1, 2).reshape(B, T, c.n_embd)
            x = x + F.dropout(F.linear(att, b.w_proj, b.b_proj), p_drop)
            h = F.layer_norm(x, (c.n_embd,), b.ln2_w, b.ln2_b, eps)
            h = F.gelu(F.linear(h, b.w_fc, b.b_fc), approximate="tanh")
            x = x + F.dropout(F.linear(h, b.w_fc2, b.b_fc2), p_drop)
        x = F.layer_norm(x, (c.n_embd,), self.lnf_w, self.lnf_b, eps)
        logits = F.linear(x, self.lm_head)[..., :c.vocab_size]
        if targets is None:
            return logits
        return F.cross_entropy(logits.float().view(-1, c.vocab_size), targets.reshape(-1))

    @torch.no_grad()
    def forward_cached(self, idx: torch.Tensor, cache: Optional[list] = None):
        """Incremental inference: ``idx [B, t]`` are the tokens after the ones that ``cache`` already holds (``None`` to
        start).  Returns ``(logits [B, t, vocab], cache)``; the cache is one ``(k, v)`` pair ``[B, H, T, D]`` per block,
        so a decode step costs one row of attention per block instead of the whole window again."""
        c = self.cfg
        B, t = idx.shape
        H, D = c.n_head, c.n_embd // c.n_head
        eps = c.layer_norm_eps
        past = 0 if not cache else cache[0][0].shape[2]
        if past + t > c.n_positions:
            raise ValueError(f"{past} cached + {t} new tokens exceed the {c.n_positions} learned positions")
        x = self.wte[idx] + self.wpe[past: past + t]
        out_cache = []
        for li, b in enumerate(self.blocks):
            h = F.layer_norm(x, (c.n_embd,), b.ln1_w, b.ln1_b, eps)
            qkv = F.linear(h, b.w_qkv, b.b_qkv).view(B, t, 3, H, D)
            q, k, v = (qkv[:, :, i].transpose(1, 2) for i in range(3))
            if cache:
                k, v = torch.cat([cache[li][0], k], 2), torch.cat([cache[li][1], v], 2)
            out_cache.append((k, v))
            if past == 0:
                att = F.scaled_dot_product_attention(q, k, v, is_causal=t > 1)
            else:                                        # new row i sees the cached tokens and new rows 0 .. i
                mask = torch.ones(t, past + t, dtype=torch.bool, device=idx.device).tril(past)
                att = F.scaled_dot_product_attention(q, k, v, attn_mask=mask)
            x = x + F.linear(att.transpose(1, 2).reshape(B, t, c.n_embd), b.w_proj, b.b_proj)
            h = F.layer_norm(x, (c.n_embd,), b.ln2_w, b.ln2_b, eps)
            x = x + F.linear(F.gelu(F.linear(h, b.w_fc, b.b_fc), approximate="tanh"), b.w_fc2, b.b_fc2)
        x = F.layer_norm(x, (c.n_embd,), self.lnf_w, self.lnf_b, eps)
        return F.linear(x, self.lm_head)[..., :c.vocab_size], out_cache

    @torch.no_grad()
    def generate(self, idx: torch.Tensor, max_new_tokens: int, temperature: float = 1.0,
                 top_k: Optional[int] = None) -> torch.Tensor:
        for _ in range(max_new_tokens):
            ctx = idx[:, -self.cfg.n_positions:]
            logits = self(ctx)[:, -1].float()
            if temperature <= 0:
                nxt = logits.argmax(-1, keepdim=True)
            else:
                logits = logits / temperature
                if top_k is not None:
                    kth = torch.topk(logits, min(top_k, logits.shape[-1])).values[:, [-1]]
                    logits = logits.masked_fill(logits < kth, float("-inf"))
                nxt = torch.multinomial(F.softmax(logits, -1), 1)
            idx = torch.cat([idx, nxt], dim=1)
        return idx


def gpt2_small(**kw) -> GPT:
    cfg_keys = set(GPTConfig.__dataclass_fields__)
    cfg = GPTConfig(**{k: v for k, v in kw.items() if k in cfg_keys})
    return GPT(cfg, **{k: v for k, v in kw.items() if k not in cfg_keys})


def gpt2_medium(**kw) -> GPT:
    cfg_keys = set(GPTConfig.__dataclass_fields__)
    cfg = GPTConfig.gpt2_medium(**{k: v for k, v in kw.items() if k in cfg_keys})
    return GPT(cfg, **{k: v for k, v in kw.items() if k not in cfg_keys})
