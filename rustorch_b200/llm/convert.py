"""Hugging Face Llama checkpoint directory -> GGUF file.

The two layouts differ in one thing besides the names: a GGUF Llama file rotates adjacent pairs of a head's dimensions
(RoPE on ``(x[2i], x[2i+1])``), a Hugging Face checkpoint the two halves (``rotate_half``), so the rows of the query and
key projections are re-ordered head by head (half-split order -> interleaved order).  With that permutation both
layouts give the same logits, which the tests check against ``transformers``' own forward pass.
"""
from __future__ import annotations

import os
from typing import Dict, Optional, Tuple

import torch

from ..formats import gguf
from ..formats.safetensors import HuggingFaceCheckpoint, hf_attention_window, hf_rope_settings

_LAYER = {"self_attn.q_proj": "attn_q", "self_attn.k_proj": "attn_k", "self_attn.v_proj": "attn_v", "self_attn.o_proj": "attn_output",
          "mlp.gate_proj": "ffn_gate", "mlp.up_proj": "ffn_up", "mlp.down_proj": "ffn_down", "input_layernorm": "attn_norm",
          "post_attention_layernorm": "ffn_norm"}


def interleave_rope_rows(w: torch.Tensor, n_head: int) -> torch.Tensor:
    """Rows of a q / k projection from half-split order (dimension ``i`` pairs with ``i + D/2``) to interleaved order
    (``2i`` pairs with ``2i + 1``), head by head."""
    d = w.shape[0] // n_head
    return w.reshape(n_head, 2, d // 2, *w.shape[1:]).transpose(1, 2).reshape(w.shape)


def sentencepiece_metadata(model_path: str) -> Dict[str, object]:
    """``tokenizer.ggml.*`` entries (pieces, scores, piece types, special ids) of a SentencePiece ``.model`` file, so that the
    written GGUF file carries its own tokenizer."""
    import sentencepiece as spm
    sp = spm.SentencePieceProcessor(model_file=model_path)
    n = sp.get_piece_size()

    def kind(i: int) -> int:                               # GGUF token types: 1 normal, 2 unknown, 3 control, 5 unused, 6 byte
        return 2 if sp.is_unknown(i) else 3 if sp.is_control(i) else 5 if sp.is_unused(i) else 6 if sp.is_byte(i) else 1
    md: Dict[str, object] = {"tokenizer.ggml.model": "llama", "tokenizer.ggml.tokens": [sp.id_to_piece(i) for i in range(n)],
                             "tokenizer.ggml.scores": [float(sp.get_score(i)) for i in range(n)],
                             "tokenizer.ggml.token_type": [kind(i) for i in range(n)]}
    for key, val in (("bos_token_id", sp.bos_id()), ("eos_token_id", sp.eos_id()), ("unknown_token_id", sp.unk_id()), ("padding_token_id", sp.pad_id())):
        if val is not None and val >= 0:
            md[f"tokenizer.ggml.{key}"] = int(val)
    return md


def hf_to_gguf(directory: str, path: str, ggml_type: gguf.GGMLType = gguf.GGMLType.Q8_0, name: Optional[str] = None) -> Dict[str, int]:
    """Writes ``path`` from the checkpoint in ``directory``: matrices as ``ggml_type`` (F32, F16, Q8_0 or Q4_0), norms and,
    for quantised types, the embedding table as F32 / F16.  Returns ``{"tensors": n, "bytes": size}``."""
    ty = gguf.GGMLType(ggml_type)
    with HuggingFaceCheckpoint(directory) as ck:
        c = ck.config
        # Qwen2 files keep the half-split rotation (the "neox" RoPE of GGUF readers) and carry q / k / v biases; Llama and
        # Mistral files are written under the "llama" architecture with re-ordered q / k rows
        a = "qwen2" if str(c.get("model_type", "")).lower() == "qwen2" else "llama"
        theta, scaling = hf_rope_settings(c)
        try:
            n_layer, n_head = int(c["num_hidden_layers"]), int(c["num_attention_heads"])
            n_kv = int(c.get("num_key_value_heads") or n_head)
            md = {"general.architecture": a, "general.name": name or os.path.basename(os.path.normpath(directory)),
                  f"{a}.block_count": n_layer, f"{a}.embedding_length": int(c["hidden_size"]),
                  f"{a}.feed_forward_length": int(c["intermediate_size"]), f"{a}.attention.head_count": n_head,
                  f"{a}.attention.head_count_kv": n_kv, f"{a}.rope.freq_base": theta,
                  f"{a}.attention.layer_norm_rms_epsilon": float(c.get("rms_norm_eps", 1e-5)),
                  f"{a}.context_length": int(c.get("max_position_embeddings", 2048)), f"{a}.vocab_size": int(c["vocab_size"])}
        except KeyError as e:
            raise ValueError(f"{directory}: config.json lacks {e.args[0]!r}") from None
        window = hf_attention_window(c)
        if window is not None:                             # readers of the file attend over the whole context: one window at most
            md[f"{a}.context_length"] = min(int(md[f"{a}.context_length"]), window)
            md[f"{a}.attention.sliding_window"] = window
        rope_freqs = None
        if scaling:
            kind = str(scaling.get("rope_type", scaling.get("type", ""))).lower()
            if kind == "linear":
                md[f"{a}.rope.scaling.type"], md[f"{a}.rope.scaling.factor"] = "linear", float(scaling["factor"])
            else:
                # other kinds travel as per-frequency divisors: plain frequency / scaled frequency
                from ..models.llama import scale_rope_frequencies
                hd = int(c.get("head_dim") or int(c["hidden_size"]) // n_head)
                inv = theta ** (-torch.arange(0, hd, 2, dtype=torch.float32) / hd)
                rope_freqs = inv / scale_rope_frequencies(inv, scaling)
                if "original_max_position_embeddings" in scaling:
                    md[f"{a}.rope.scaling.original_context_length"] = int(scaling["original_max_position_embeddings"])
        qkv_bias = {"self_attn.q_proj.bias": "attn_q.bias", "self_attn.k_proj.bias": "attn_k.bias", "self_attn.v_proj.bias": "attn_v.bias"}
        other = [k for k in ck.keys() if k.endswith(".bias") and k.split(".", 3)[-1] not in qkv_bias]
        if other:
            raise ValueError(f"{directory}: biases outside the q / k / v projections ({other[:3]}) are not a decoder this format path writes")
        emb_ty = gguf.GGMLType.F16 if ty in (gguf.GGMLType.Q8_0, gguf.GGMLType.Q4_0, gguf.GGMLType.F16) else gguf.GGMLType.F32

        def enc(w: torch.Tensor, t: gguf.GGMLType):
            """Encoded at once, so that the checkpoint is held in its written size, not in fp32."""
            return gguf.RawTensor(tuple(w.shape), gguf.encode_tensor(w, t)), t
        tensors: Dict[str, Tuple[object, gguf.GGMLType]] = {
            "token_embd.weight": enc(ck.get("model.embed_tokens.weight").float(), emb_ty),
            "output_norm.weight": enc(ck.get("model.norm.weight").float(), gguf.GGMLType.F32)}
        if "lm_head.weight" in ck:
            tensors["output.weight"] = enc(ck.get("lm_head.weight").float(), ty)
        if rope_freqs is not None:
            tensors["rope_freqs.weight"] = enc(rope_freqs, gguf.GGMLType.F32)
        for i in range(n_layer):
            for src, dst in _LAYER.items():
                w = ck.get(f"model.layers.{i}.{src}.weight").float()
                if a == "llama" and dst == "attn_q":
                    w = interleave_rope_rows(w, n_head)
                elif a == "llama" and dst == "attn_k":
                    w = interleave_rope_rows(w, n_kv)
                tensors[f"blk.{i}.{dst}.weight"] = enc(w, gguf.GGMLType.F32 if dst.endswith("norm") else ty)
            for src, dst in qkv_bias.items():
                key = f"model.layers.{i}.{src}"
                if key in ck:
                    b = ck.get(key).float()
                    if a == "llama":                       # a biased Llama: the bias follows its rows
                        b = interleave_rope_rows(b.unsqueeze(1), n_head if dst == "attn_q.bias" else n_kv).squeeze(1) if dst != "attn_v.bias" else b
                    tensors[f"blk.{i}.{dst}"] = enc(b, gguf.GGMLType.F32)
    spm_path, json_path = os.path.join(directory, "tokenizer.model"), os.path.join(directory, "tokenizer.json")
    tokenizer = None
    if os.path.exists(spm_path):
        md.update(sentencepiece_metadata(spm_path))
        tokenizer = "llama"
    elif os.path.exists(json_path):
        from ..cli.tokenizer import BPETokenizer
        try:
            md.update(BPETokenizer.from_tokenizer_json(json_path).gguf_metadata())
            tokenizer = "gpt2"
        except ValueError:                                 # not byte-level BPE: the file is written without a tokenizer
            pass
    gguf.write_gguf(path, md, tensors)
    return {"tensors": len(tensors), "bytes": os.path.getsize(path), "tokenizer": tokenizer is not None, "tokenizer_model": tokenizer}
