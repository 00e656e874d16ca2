"""Llama-family inference runtime: GGUF weights (Q4_0 / Q8_0 kept quantised), fp16 activations, KV cache,
prefill + token-by-token decode, optional tensor parallelism.

This is the working version of what the reference's CLI sketches: its ``load_gguf`` is a TODO that returns
a dummy model (example-cli/src/model/loader.rs:55-59), its generation loop re-runs the whole sequence for
every token without a KV cache (model/inference.rs:135-192) and its tensor loader never decodes quantised
blocks (model/formats/tensor_loader.rs:103-122).

Per token and layer: RMSNorm -> fused QKV dequant-GEMV -> RoPE + cache append -> cached attention ->
output projection (+residual) -> RMSNorm -> gate/up dequant-GEMV -> SwiGLU -> down projection (+residual).
Tensor parallel (``tp_world > 1``): Q/K/V/gate/up are split by output rows (heads), ``attn_output`` and
``ffn_down`` by input columns; the two partial sums per layer are all-reduced.
"""
from __future__ import annotations

import math
import time
from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

import torch
import torch.distributed as dist

from .. import _native
from ..formats import gguf
from .quant import QuantLinear


@dataclass
class LlamaConfig:
    vocab_size: int = 32000
    n_layer: int = 32
    n_embd: int = 4096
    n_head: int = 32
    n_head_kv: int = 32
    n_ff: int = 11008
    rope_theta: float = 10000.0
    rms_eps: float = 1e-5
    context_length: int = 2048
    rope_interleaved: bool = True
    rope_scaling: Optional[dict] = None          # Hugging Face ``rope_scaling`` entry (linear / llama3); None: plain RoPE

    @property
    def head_dim(self) -> int:
        return self.n_embd // self.n_head

    @staticmethod
    def llama_7b() -> "LlamaConfig":
        return LlamaConfig()

    @staticmethod
    def llama3_8b() -> "LlamaConfig":
        return LlamaConfig(vocab_size=128256, n_head_kv=8, n_ff=14336, rope_theta=500000.0, context_length=8192)

    def num_parameters(self) -> int:
        d, hd = self.n_embd, self.head_dim
        per = d * (self.n_head * hd) + 2 * d * (self.n_head_kv * hd) + (self.n_head * hd) * d + 3 * d * self.n_ff
        return self.n_layer * per + 2 * self.vocab_size * d


class KVCache:
    """fp16 key/value cache ``[B, Hkv_local, T_max, D]`` per layer with per-sequence lengths."""

    def __init__(self, n_layer: int, batch: int, n_head_kv: int, max_len: int, head_dim: int, device, dtype=torch.float16):
        self.k = [torch.zeros(batch, n_head_kv, max_len, head_dim, dtype=dtype, device=device) for _ in range(n_layer)]
        self.v = [torch.zeros(batch, n_head_kv, max_len, head_dim, dtype=dtype, device=device) for _ in range(n_layer)]
        self.lengths = [0] * batch
        self.max_len = max_len

    def seq_len(self, b: int = 0) -> int:
        return self.lengths[b]

    def clear(self) -> None:
        self.lengths = [0] * len(self.lengths)

    def nbytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self.k + self.v)


class _DecodeGraph:
    """Static device tensors and the captured graph of one decode step."""
    tok = pos = seq = step = out = logits = graph = None


class _Layer:
    __slots__ = ("attn_norm", "wqkv", "wo", "ffn_norm", "w_gate_up", "w_down", "qkv_bias")


class LlamaRuntime:
    def __init__(self, cfg: LlamaConfig, device="cuda", tp_rank: int = 0, tp_world: int = 1, tp_group=None):
        self.cfg, self.device = cfg, torch.device(device)
        self.tp_rank, self.tp_world, self.tp_group = tp_rank, tp_world, tp_group
        if cfg.n_head % tp_world or cfg.n_head_kv % tp_world or (cfg.n_ff // 32) % tp_world:
            raise ValueError("heads and n_ff/32 must be divisible by the tensor-parallel size")
        self.h_local, self.hkv_local = cfg.n_head // tp_world, cfg.n_head_kv // tp_world
        self.ff_local = cfg.n_ff // tp_world
        self.layers: List[_Layer] = []
        self.tok_emb: Optional[torch.Tensor] = None        # fp16 [V, d]
        self.out_norm: Optional[torch.Tensor] = None
        self.lm_head: Optional[QuantLinear] = None
        self.act_dtype = torch.float16 if self.device.type == "cuda" else torch.float32
        self._graph = None
        self._p2p = None
        self._ar_norm = None

    # ---------------------------------------------------------------- loading
    def _shard_attn_rows(self, q: QuantLinear, heads: int) -> QuantLinear:
        return q if self.tp_world == 1 else q.shard_rows(self.tp_rank, self.tp_world)

    @staticmethod
    def _cat_rows(parts: List[QuantLinear]) -> QuantLinear:
        new = object.__new__(QuantLinear)
        p0 = parts[0]
        new.ggml_type, new.q8, new.device, new.in_features = p0.ggml_type, p0.q8, p0.device, p0.in_features
        if p0.blocks is not None:
            new.blocks = torch.cat([p.blocks for p in parts], 0)
            new.qs = new.scales = None
            new.out_features = new.blocks.shape[0]
        else:
            new.blocks = None
            new.qs, new.scales = torch.cat([p.qs for p in parts], 0), torch.cat([p.scales for p in parts], 0)
            new.out_features = new.scales.shape[0]
        return new

    def _assemble_layer(self, wq, wk, wv, wo, wg, wu, wd, attn_norm, ffn_norm, qkv_bias=None) -> _Layer:
        """``qkv_bias``: the three bias vectors of the q / k / v projections (Qwen2-style checkpoints), or None."""
        r, w = self.tp_rank, self.tp_world
        L = _Layer()
        L.qkv_bias = None
        if qkv_bias is not None:
            parts = [b.float().chunk(w)[r] if w > 1 else b.float() for b in qkv_bias]      # rows are sharded like the weights
            L.qkv_bias = torch.cat(parts).to(self.device, self.act_dtype)
        if w > 1:
            wq, wk, wv = wq.shard_rows(r, w), wk.shard_rows(r, w), wv.shard_rows(r, w)
            wg, wu = wg.shard_rows(r, w), wu.shard_rows(r, w)
            wo, wd = wo.shard_cols(r, w), wd.shard_cols(r, w)
        L.wqkv = self._cat_rows([wq, wk, wv])
        L.w_gate_up = self._cat_rows([wg, wu])
        L.wo, L.w_down = wo, wd
        L.attn_norm, L.ffn_norm = attn_norm.to(self.device, self.act_dtype), ffn_norm.to(self.device, self.act_dtype)
        return L

    @classmethod
    def from_gguf(cls, path: str, device="cuda", tp_rank: int = 0, tp_world: int = 1, tp_group=None) -> "LlamaRuntime":
        with gguf.GGUFFile(path) as g:
            mc = g.model_config()
            cfg = LlamaConfig(vocab_size=int(mc["vocab_size"]), n_layer=int(mc["n_layer"]), n_embd=int(mc["n_embd"]),
                              n_head=int(mc["n_head"]), n_head_kv=int(mc["n_head_kv"]), n_ff=int(mc["n_ff"]),
                              rope_theta=float(mc["rope_theta"]), rms_eps=float(mc["rms_eps"]),
                              context_length=int(mc["context_length"]))
            need = ["token_embd.weight", "output_norm.weight"] + [f"blk.{i}.{t}.weight" for i in range(cfg.n_layer) for t in (
                "attn_q", "attn_k", "attn_v", "attn_output", "ffn_gate", "ffn_up", "ffn_down", "attn_norm", "ffn_norm")]
            absent = [n for n in need if n not in g.tensors]
            qkv_b = ("attn_q.bias", "attn_k.bias", "attn_v.bias")
            biased = all(f"blk.0.{b}" in g.tensors for b in qkv_b)
            extra = sorted({n.split(".", 2)[-1] for n in g.tensors if n.startswith("blk.") and n.endswith(".bias")
                            and not (biased and n.split(".", 2)[-1] in qkv_b)}
                           | {n.split(".", 2)[-1] for n in g.tensors if "_exps." in n or "ffn_gate_inp" in n})
            if absent or extra:
                what = (f"missing {absent[:4]}{'...' if len(absent) > 4 else ''}" if absent else "") + \
                       (("; " if absent else "") + f"tensors this runtime does not execute: {extra[:6]}" if extra else "")
                raise ValueError(f"{path}: architecture '{mc['architecture']}' is not a Llama-style decoder this runtime runs ({what})")
            window = g.metadata.get(f"{mc['architecture']}.attention.sliding_window")
            if window and 0 < int(window) < cfg.context_length:
                cfg.context_length = int(window)                  # full attention equals windowed attention up to one window
            scaling = g.metadata.get(f"{mc['architecture']}.rope.scaling.type")
            if "rope_freqs.weight" in g.tensors:
                # per-frequency divisors (how Llama 3.1 files carry their long-context scaling)
                cfg.rope_scaling = {"rope_type": "factors", "factors": [float(v) for v in g.load_tensor("rope_freqs.weight").float().flatten()]}
                if len(cfg.rope_scaling["factors"]) != cfg.head_dim // 2:
                    raise ValueError(f"{path}: rope_freqs.weight has {len(cfg.rope_scaling['factors'])} entries for head size {cfg.head_dim}")
            elif scaling == "linear":
                cfg.rope_scaling = {"rope_type": "linear", "factor": float(g.metadata.get(f"{mc['architecture']}.rope.scaling.factor", 1.0))}
            elif scaling not in (None, "none"):
                # ignoring the factors would change the logits at every position
                raise ValueError(f"{path}: RoPE frequency scaling '{scaling}' is not implemented by this runtime (linear and rope_freqs.weight are)")
            # Llama-architecture files rotate adjacent pairs (their q / k rows were re-ordered by the converter); the Qwen
            # family and the other "neox" architectures rotate the two halves of a head
            cfg.rope_interleaved = str(mc["architecture"]).lower() not in ("qwen", "qwen2", "phi3", "gemma", "stablelm", "falcon")
            rt = cls(cfg, device, tp_rank, tp_world, tp_group)

            def ql(name: str) -> QuantLinear:
                info = g.tensors[name]
                if info.ggml_type in (gguf.GGMLType.Q4_0, gguf.GGMLType.Q8_0):
                    blocks, _ = g.load_quantized(name)
                    return QuantLinear(blocks, info.ggml_type, rt.device)
                return QuantLinear.from_float(g.load_tensor(name), gguf.GGMLType.Q8_0, rt.device)

            for i in range(cfg.n_layer):
                p = f"blk.{i}."
                rt.layers.append(rt._assemble_layer(ql(p + "attn_q.weight"), ql(p + "attn_k.weight"), ql(p + "attn_v.weight"),
                                                    ql(p + "attn_output.weight"), ql(p + "ffn_gate.weight"), ql(p + "ffn_up.weight"),
                                                    ql(p + "ffn_down.weight"), g.load_tensor(p + "attn_norm.weight"),
                                                    g.load_tensor(p + "ffn_norm.weight"),
                                                    [g.load_tensor(p + b) for b in qkv_b] if biased else None))
            rt.tok_emb = g.load_tensor("token_embd.weight").to(rt.device, rt.act_dtype)
            rt.out_norm = g.load_tensor("output_norm.weight").to(rt.device, rt.act_dtype)
            head_name = "output.weight" if "output.weight" in g.tensors else "token_embd.weight"
            rt.lm_head = ql(head_name)
        return rt

    @classmethod
    def from_hf(cls, directory: str, device="cuda", ggml_type=gguf.GGMLType.Q8_0, tp_rank: int = 0, tp_world: int = 1,
                tp_group=None) -> "LlamaRuntime":
        """A Hugging Face Llama-style checkpoint directory (``config.json`` + safetensors, sharded or not).  Every linear
        is quantised to ``ggml_type`` (Q8_0 or Q4_0) as it is read, one tensor at a time, so a bf16 checkpoint never
        sits in memory whole.  These checkpoints rotate the two halves of a head (``rotate_half``), not adjacent pairs
        as GGUF files do, hence ``rope_interleaved=False``."""
        from ..formats.safetensors import HuggingFaceCheckpoint, hf_attention_window, hf_rope_settings
        with HuggingFaceCheckpoint(directory) as ck:
            c = ck.config
            theta, scaling = hf_rope_settings(c)
            arch = (c.get("architectures") or [c.get("model_type", "?")])[0]
            try:
                n_head = int(c["num_attention_heads"])
                cfg = LlamaConfig(vocab_size=int(c["vocab_size"]), n_layer=int(c["num_hidden_layers"]), n_embd=int(c["hidden_size"]),
                                  n_head=n_head, n_head_kv=int(c.get("num_key_value_heads") or n_head), n_ff=int(c["intermediate_size"]),
                                  rope_theta=theta, rms_eps=float(c.get("rms_norm_eps", 1e-5)),
                                  context_length=int(c.get("max_position_embeddings", 2048)))
            except KeyError as e:
                raise ValueError(f"{directory}: config.json lacks {e.args[0]!r}") from None
            if c.get("head_dim") not in (None, cfg.n_embd // cfg.n_head):
                raise ValueError(f"{directory}: head_dim {c['head_dim']} differs from hidden_size / num_attention_heads")
            if scaling:
                from ..models.llama import scale_rope_frequencies
                scale_rope_frequencies(torch.ones(1), scaling)         # refuses the kinds that are not implemented
                cfg.rope_scaling = dict(scaling)
            cfg.rope_interleaved = False
            lay = lambda i, t: f"model.layers.{i}.{t}.weight"      # noqa: E731
            parts = ("self_attn.q_proj", "self_attn.k_proj", "self_attn.v_proj", "self_attn.o_proj", "mlp.gate_proj", "mlp.up_proj",
                     "mlp.down_proj", "input_layernorm", "post_attention_layernorm")
            need = ["model.embed_tokens.weight", "model.norm.weight"] + [lay(i, t) for i in range(cfg.n_layer) for t in parts]
            absent = [n for n in need if n not in ck]
            qkv_b = ("self_attn.q_proj.bias", "self_attn.k_proj.bias", "self_attn.v_proj.bias")
            biased = all(f"model.layers.0.{b}" in ck for b in qkv_b)
            extra = sorted({n.split(".", 3)[-1] for n in ck.keys() if n.startswith("model.layers.") and n.endswith(".bias")
                            and not (biased and n.split(".", 3)[-1] in qkv_b)}
                           | {n.split(".", 3)[-1] for n in ck.keys() if ".experts." in n or "block_sparse_moe" in n})
            window = hf_attention_window(c)
            if window is not None and window < cfg.context_length:
                # attention here always sees the whole cache; within one window's length that is what the model computes,
                # so the context is limited to the window instead of attending further back than the model was trained to
                cfg.context_length = window
            if absent or extra:
                what = (f"missing {absent[:4]}{'...' if len(absent) > 4 else ''}" if absent else "") + \
                       (("; " if absent else "") + f"tensors this runtime does not execute: {extra[:6]}" if extra else "")
                raise ValueError(f"{directory}: '{arch}' is not a Llama-style decoder this runtime runs ({what})")
            rt = cls(cfg, device, tp_rank, tp_world, tp_group)
            ql = lambda name: QuantLinear.from_float(ck.get(name).float(), ggml_type, rt.device)      # noqa: E731
            for i in range(cfg.n_layer):
                rt.layers.append(rt._assemble_layer(*(ql(lay(i, t)) for t in parts[:7]), ck.get(lay(i, parts[7])).float(),
                                                    ck.get(lay(i, parts[8])).float(),
                                                    [ck.get(f"model.layers.{i}.{b}") for b in qkv_b] if biased else None))
            rt.tok_emb = ck.get("model.embed_tokens.weight").to(rt.device, rt.act_dtype)
            rt.out_norm = ck.get("model.norm.weight").to(rt.device, rt.act_dtype)
            rt.lm_head = ql("lm_head.weight" if "lm_head.weight" in ck else "model.embed_tokens.weight")
        return rt

    @classmethod
    def random_init(cls, cfg: LlamaConfig, device="cuda", ggml_type=gguf.GGMLType.Q4_0, tp_rank: int = 0, tp_world: int = 1,
                    tp_group=None, seed: int = 0, std: float = 0.02) -> "LlamaRuntime":
        """Synthetic weights of the right shapes and statistics, built directly in quantised form."""
        rt = cls(cfg, device, tp_rank, tp_world, tp_group)
        d, hd = cfg.n_embd, cfg.head_dim
        mk = lambda o, i, s: QuantLinear.random(o, i, ggml_type, std, rt.device, seed * 1000 + s)  # noqa: E731
        for li in range(cfg.n_layer):
            s = li * 10
            rt.layers.append(rt._assemble_layer(mk(cfg.n_head * hd, d, s), mk(cfg.n_head_kv * hd, d, s + 1),
                                                mk(cfg.n_head_kv * hd, d, s + 2), mk(d, cfg.n_head * hd, s + 3),
                                                mk(cfg.n_ff, d, s + 4), mk(cfg.n_ff, d, s + 5), mk(d, cfg.n_ff, s + 6),
                                                torch.ones(d), torch.ones(d)))
        g = torch.Generator(device=rt.device).manual_seed(seed)
        rt.tok_emb = (torch.randn(cfg.vocab_size, d, device=rt.device, generator=g) * std).to(rt.act_dtype)
        rt.out_norm = torch.ones(d, device=rt.device, dtype=rt.act_dtype)
        rt.lm_head = mk(cfg.vocab_size, d, 999999)
        return rt

    def weight_bytes(self) -> int:
        n = self.lm_head.nbytes() + self.tok_emb.numel() * self.tok_emb.element_size()
        for L in self.layers:
            n += L.wqkv.nbytes() + L.wo.nbytes() + L.w_gate_up.nbytes() + L.w_down.nbytes()
        return n

    def new_cache(self, batch: int, max_len: Optional[int] = None) -> KVCache:
        return KVCache(self.cfg.n_layer, batch, self.hkv_local, max_len or self.cfg.context_length, self.cfg.head_dim,
                       self.device, self.act_dtype)

    # ---------------------------------------------------------------- forward
    def _all_reduce(self, x: torch.Tensor) -> torch.Tensor:
        """Sum of the row-parallel partial outputs over the TP ranks: the one-shot peer-memory kernel for decode-sized
        activations (it is graph-capturable and has a fraction of NCCL's latency), NCCL for anything larger."""
        if self.tp_world == 1:
            return x
        if x.is_cuda and x.numel() * x.element_size() <= (1 << 20):
            if self._p2p is None:
                from ..distributed.p2p_collectives import P2PCollectives
                self._p2p = P2PCollectives(1 << 19, x.dtype, self.device, self.tp_group, one_shot_max_bytes=1 << 20)
            return self._p2p.all_reduce(x)
        dist.all_reduce(x, group=self.tp_group)
        return x

    def _fused_epilogue(self, n: int, x: torch.Tensor):
        """The all-reduce + residual + RMSNorm kernel, when this step's activations fit its receive buffers."""
        if self.tp_world == 1 or not x.is_cuda or x.dtype not in (torch.float16, torch.bfloat16):
            return None
        if self._ar_norm is None:
            from ..distributed.p2p_collectives import AllReduceResidualNorm
            self._ar_norm = AllReduceResidualNorm(512 * self.cfg.n_embd, x.dtype, self.device, self.tp_group)
        return self._ar_norm if self._ar_norm.fits(n, x.shape[1]) and x.is_contiguous() else None

    def _rmsnorm(self, x, w):
        if self.device.type == "cuda":
            y = torch.empty_like(x)
            _native.load(required=True).rmsnorm_f16(x, w, y, self.cfg.rms_eps)
            return y
        xf = x.float()
        return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + self.cfg.rms_eps) * w.float()).to(x.dtype)

    def _inv_freq(self, D: int, device) -> torch.Tensor:
        """Rotation frequencies of the ``D // 2`` pairs, with the checkpoint's frequency scaling applied."""
        cached = getattr(self, "_inv_freq_cache", None)
        if cached is None or cached.shape[0] != D // 2 or cached.device != torch.device(device):
            cached = self.cfg.rope_theta ** (-torch.arange(D // 2, device=device, dtype=torch.float32) * 2.0 / D)
            if self.cfg.rope_scaling:
                from ..models.llama import scale_rope_frequencies
                cached = scale_rope_frequencies(cached, self.cfg.rope_scaling)
            self._inv_freq_cache = cached
        return cached

    def _rope_reference(self, t: torch.Tensor, pos: torch.Tensor) -> torch.Tensor:
        D = t.shape[-1]
        half = D // 2
        inv = self._inv_freq(D, t.device)
        ang = pos.float()[:, None, None] * inv
        cs, sn = ang.cos(), ang.sin()
        tf = t.float()
        if self.cfg.rope_interleaved:
            a, b = tf[..., 0::2], tf[..., 1::2]
            out = torch.stack([a * cs - b * sn, a * sn + b * cs], -1).flatten(-2)
        else:
            a, b = tf[..., :half], tf[..., half:]
            out = torch.cat([a * cs - b * sn, a * sn + b * cs], -1)
        return out.to(t.dtype)

    def forward_tokens(self, tokens: torch.Tensor, pos: torch.Tensor, seq: torch.Tensor, cache: KVCache,
                       last_only: Optional[torch.Tensor] = None, max_kv: Optional[int] = None,
                       prefill_bt: Optional[Tuple[int, int]] = None) -> torch.Tensor:
        """``tokens / pos / seq``: ``[n_tok]`` (token id, position in its sequence, sequence index).  The new
        keys/values are appended to ``cache`` and every token attends to positions ``0 .. pos`` of its own
        sequence.  Returns fp32 logits ``[n_tok or len(last_only), vocab]``."""
        cfg = self.cfg
        C = _native.load(required=True) if self.device.type == "cuda" else None
        n = tokens.shape[0]
        H, Hkv, D = self.h_local, self.hkv_local, cfg.head_dim
        x = self.tok_emb[tokens]                                       # [n, d]
        pos32, seq32 = pos.to(torch.int32), seq.to(torch.int32)
        kv_len = pos32 + 1
        if max_kv is None:          # upper bound of kv_len known to the host (avoids a device sync)
            max_kv = cache.max_len
        scale = 1.0 / math.sqrt(D)
        fused_ar = self._fused_epilogue(n, x)
        h = None
        flash_bt, flash_lse = None, None
        if (prefill_bt is not None and C is not None and D in (64, 128) and self.act_dtype == torch.float16 and prefill_bt[1] >= 16
                and prefill_bt[0] * prefill_bt[1] == n):
            flash_bt = prefill_bt
            flash_lse = torch.empty((prefill_bt[0], H, prefill_bt[1]), dtype=torch.float32, device=self.device)
        # decode-sized steps on one GPU: each projection is one kernel with the RMSNorm as its prologue and the
        # residual add / SwiGLU as its epilogue (QuantLinear.fused)
        fuse = C is not None and self.tp_world == 1 and 1 <= n <= QuantLinear.FUSED_MAX_ROWS and x.dtype == torch.float16
        for li, L in enumerate(self.layers):
            rope_done = False
            if fuse:
                if (cfg.rope_interleaved and QuantLinear.ROPE_FUSED and L.qkv_bias is None and L.wqkv.in_features % 64 == 0
                        and (H + 2 * Hkv) * D % 4 == 0 and not cfg.rope_scaling):
                    # rotary embedding and the cache append ride in the projection's epilogue
                    qkv = L.wqkv.fused(x, norm_w=L.attn_norm, eps=cfg.rms_eps,
                                       rope=dict(pos=pos32, seq=seq32, cache_k=cache.k[li], cache_v=cache.v[li], n_head=H,
                                                 theta=cfg.rope_theta))
                    rope_done = True
                else:
                    qkv = L.wqkv.fused(x, norm_w=L.attn_norm, eps=cfg.rms_eps)
            else:
                if h is None:
                    h = self._rmsnorm(x, L.attn_norm)
                qkv = L.wqkv(h)                                            # [n, (H + 2 Hkv) D]
            if L.qkv_bias is not None:
                qkv = qkv + L.qkv_bias.to(qkv.dtype)
            q = qkv[:, : H * D].view(n, H, D)
            k = qkv[:, H * D: (H + Hkv) * D].view(n, Hkv, D)
            v = qkv[:, (H + Hkv) * D:].view(n, Hkv, D)
            if C is not None:
                if cfg.rope_scaling:
                    # scaled frequencies: the rotation kernels derive theta^(-2i/D) themselves, so these checkpoints
                    # rotate with the frequency table in tensor ops and append to the cache by index
                    q, k = self._rope_reference(q, pos), self._rope_reference(k, pos)
                    cache.k[li][seq.long(), :, pos.long()] = k
                    cache.v[li][seq.long(), :, pos.long()] = v
                elif not rope_done:
                    C.rope_kv(q, k, v, cache.k[li], cache.v[li], pos32, seq32, cfg.rope_theta, cfg.rope_interleaved)
                att = torch.empty((n, H, D), dtype=q.dtype, device=q.device)
                if flash_bt is not None:
                    # prompt processing: causal attention among the new tokens on the tcgen05 flash kernel (fp16 I/O),
                    # reading the rotated q / k and v straight from the fused projection output
                    Bp, Tp = flash_bt
                    C.attn_fwd(q.unflatten(0, (Bp, Tp)), k.unflatten(0, (Bp, Tp)), v.unflatten(0, (Bp, Tp)),
                               att.view(Bp, Tp, H, D), flash_lse, True, scale)
                else:
                    C.attn_cache(q, cache.k[li], cache.v[li], att, kv_len, seq32, max_kv, scale)
            else:
                q, k = self._rope_reference(q, pos), self._rope_reference(k, pos)
                cache.k[li][seq, :, pos] = k
                cache.v[li][seq, :, pos] = v
                att = torch.empty_like(q)
                for t in range(n):
                    Lk = int(pos[t]) + 1
                    kk = cache.k[li][int(seq[t]), :, :Lk].float().repeat_interleave(H // Hkv, 0)   # [H, Lk, D]
                    vv = cache.v[li][int(seq[t]), :, :Lk].float().repeat_interleave(H // Hkv, 0)
                    p = torch.softmax((kk @ q[t].float().unsqueeze(-1)).squeeze(-1) * scale, -1)   # [H, Lk]
                    att[t] = (p.unsqueeze(1) @ vv).squeeze(1).to(att.dtype)
            att2 = att.reshape(n, H * D)
            if fuse:
                # wo / down (no prologue, short rows of work per SM) are faster on the K-sliced GEMV kernel
                x = L.wo(att2, residual=x)
                act = L.w_gate_up.fused(x, norm_w=L.ffn_norm, eps=cfg.rms_eps, swiglu=True)
                x = L.w_down(act, residual=x)
                continue
            if self.tp_world == 1:
                x = L.wo(att2, residual=x)
                h = self._rmsnorm(x, L.ffn_norm)
            elif fused_ar is not None:           # x += sum over ranks; h = norm(x): one kernel
                h = fused_ar(L.wo(att2), x, L.ffn_norm, cfg.rms_eps)
            else:
                x = x + self._all_reduce(L.wo(att2))
                h = self._rmsnorm(x, L.ffn_norm)
            if C is not None and n <= QuantLinear.FUSED_MAX_ROWS and h.dtype == torch.float16:
                act = L.w_gate_up.fused(h, swiglu=True)                # gate/up GEMV + SwiGLU in one kernel
            else:
                gu = L.w_gate_up(h)                                    # [n, 2 ff_local]
                if C is not None:
                    act = torch.empty((n, self.ff_local), dtype=gu.dtype, device=gu.device)
                    C.silu_mul(gu[:, : self.ff_local], gu[:, self.ff_local:], act)
                else:
                    act = torch.nn.functional.silu(gu[:, : self.ff_local].float()).to(gu.dtype) * gu[:, self.ff_local:]
            h = None
            if self.tp_world == 1:
                x = L.w_down(act, residual=x)
            elif fused_ar is not None:
                last = li + 1 == len(self.layers)
                if last and last_only is not None:
                    fused_ar(L.w_down(act), x)
                else:
                    h = fused_ar(L.w_down(act), x, self.out_norm if last else self.layers[li + 1].attn_norm, cfg.rms_eps)
            else:
                x = x + self._all_reduce(L.w_down(act))
        if last_only is not None:
            x = x[last_only]
        if fuse and last_only is None:
            return self.lm_head.fused(x, norm_w=self.out_norm, eps=cfg.rms_eps).float()
        if h is None:
            h = self._rmsnorm(x, self.out_norm)
        return self.lm_head(h).float()

    # --------------------------------------------------------------- generate
    @torch.no_grad()
    def prefill(self, prompts: torch.Tensor, cache: KVCache) -> torch.Tensor:
        """``prompts [B, T]`` (equal lengths) -> logits of the last position ``[B, vocab]``."""
        B, T = prompts.shape
        dev = self.device
        tokens = prompts.reshape(-1).to(dev)
        pos = torch.arange(T, device=dev).repeat(B)
        seq = torch.arange(B, device=dev).repeat_interleave(T)
        last = torch.arange(B, device=dev) * T + (T - 1)
        logits = self.forward_tokens(tokens, pos, seq, cache, last_only=last, max_kv=T, prefill_bt=(B, T))
        cache.lengths = [T] * B
        return logits

    @torch.no_grad()
    def decode_step(self, tokens: torch.Tensor, cache: KVCache) -> torch.Tensor:
        """One new token per sequence: ``tokens [B]`` -> logits ``[B, vocab]``."""
        B = tokens.shape[0]
        dev = self.device
        pos = torch.tensor(cache.lengths, device=dev)
        seq = torch.arange(B, device=dev)
        logits = self.forward_tokens(tokens.to(dev), pos, seq, cache, max_kv=max(cache.lengths) + 1)
        cache.lengths = [l + 1 for l in cache.lengths]
        return logits

    # ----------------------------------------------------------- CUDA-graph decode
    @torch.no_grad()
    def capture_decode_graph(self, cache: KVCache, batch: int) -> "_DecodeGraph":
        """Captures one greedy decode step (all layers, lm_head, argmax, position increment) into a CUDA
        graph whose inputs live on the device: a step is then one graph launch, and the ~10 launches per
        layer no longer pay host latency.  Positions and the current tokens are device tensors that the graph
        itself advances, so replaying it N times generates N tokens without any host round trip."""
        dev = self.device
        g = _DecodeGraph()
        g.tok = torch.zeros(batch, dtype=torch.long, device=dev)
        g.pos = torch.zeros(batch, dtype=torch.int32, device=dev)
        g.seq = torch.arange(batch, dtype=torch.int32, device=dev)
        g.step = torch.zeros(1, dtype=torch.long, device=dev)
        g.out = torch.zeros(batch, cache.max_len, dtype=torch.long, device=dev)

        def body():
            logits = self.forward_tokens(g.tok, g.pos, g.seq, cache, max_kv=cache.max_len)
            nxt = logits.argmax(-1)
            g.out.scatter_(1, g.step.view(1, 1).expand(batch, 1), nxt.view(batch, 1))
            g.tok.copy_(nxt)
            g.pos.add_(1)
            g.step.add_(1)
            return logits

        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):                     # warm-up outside capture (lazy inits, scratch growth)
            body()
        torch.cuda.current_stream(dev).wait_stream(side)
        torch.cuda.synchronize(dev)
        g.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g.graph):
            g.logits = body()
        return g

    @torch.no_grad()
    def generate_graph(self, prompts: torch.Tensor, max_new_tokens: int, cache: Optional[KVCache] = None
                       ) -> Tuple[torch.Tensor, Dict[str, float]]:
        """Greedy generation with the decode loop replayed from a CUDA graph (single process or TP ranks that
        all call it together).  Same outputs as ``generate`` without a sampler."""
        B, T = prompts.shape
        cache = cache or self.new_cache(B, T + max_new_tokens)
        dev = self.device
        g = self.capture_decode_graph(cache, B)           # the warm-up/capture writes only at position 0.. (reset below)
        torch.cuda.synchronize(dev)
        t0 = time.perf_counter()
        logits = self.prefill(prompts, cache)
        nxt = logits.argmax(-1)
        g.tok.copy_(nxt)
        g.pos.fill_(T)
        g.step.zero_()
        torch.cuda.synchronize(dev)
        ttft = time.perf_counter() - t0
        t1 = time.perf_counter()
        steps = max_new_tokens - 1
        for _ in range(steps):
            g.graph.replay()
        torch.cuda.synchronize(dev)
        dt = time.perf_counter() - t1
        cache.lengths = [T + steps] * B
        toks = torch.cat([prompts.to(dev), nxt.view(B, 1), g.out[:, :steps]], 1)
        return toks, {"ttft_s": ttft, "decode_tokens_per_s": B * steps / dt if dt > 0 and steps else 0.0,
                      "decode_steps": steps, "batch": B}

    @torch.no_grad()
    def generate(self, prompts: torch.Tensor, max_new_tokens: int, sampler=None, eos_token: Optional[int] = None,
                 cache: Optional[KVCache] = None) -> Tuple[torch.Tensor, Dict[str, float]]:
        """Greedy (or ``sampler(logits) -> tokens``) generation.  Returns tokens ``[B, T + new]`` and timing:
        ``ttft_s`` (prefill + first token) and ``decode_tokens_per_s``."""
        B, T = prompts.shape
        cache = cache or self.new_cache(B, T + max_new_tokens)
        sync = (lambda: torch.cuda.synchronize(self.device)) if self.device.type == "cuda" else (lambda: None)
        sync()
        t0 = time.perf_counter()
        logits = self.prefill(prompts, cache)
        nxt = sampler(logits) if sampler else logits.argmax(-1)
        sync()
        ttft = time.perf_counter() - t0
        out = [prompts.to(self.device), nxt.view(B, 1)]
        t1 = time.perf_counter()
        steps = 0
        for _ in range(max_new_tokens - 1):
            logits = self.decode_step(nxt, cache)
            nxt = sampler(logits) if sampler else logits.argmax(-1)
            out.append(nxt.view(B, 1))
            steps += 1
            if eos_token is not None and bool((nxt == eos_token).all()):
                break
        sync()
        dt = time.perf_counter() - t1
        return torch.cat(out, 1), {"ttft_s": ttft, "decode_tokens_per_s": B * steps / dt if dt > 0 and steps else 0.0,
                                   "decode_steps": steps, "batch": B}
