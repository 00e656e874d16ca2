"""Model loading and text generation for the CLI (example-cli/src/model/loader.rs:6-156, model/inference.rs:58-331).

``ModelLoader.from_file`` dispatches on the file type: GGUF files become a quantised ``LlamaRuntime`` with their
embedded tokenizer; safetensors / RusTorch / torch checkpoints of the in-repo GPT architecture are loaded into
``GPT``; ``dummy`` gives the reference's echo model.  ``InferenceEngine.generate`` streams tokens: prefill once,
then one decode step per token against the KV cache (the reference re-runs the whole sequence per token).
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Callable, Iterator, List, Optional

import torch

from ..formats import gguf as gguf_fmt
from ..formats.safetensors import detect_format
from ..llm import InferenceTimer, LlamaRuntime, Sampler, SamplingConfig
from .session import GenerationConfig
from .tokenizer import ByteTokenizer, Tokenizer, load_tokenizer


@dataclass
class ModelMetadata:
    name: str
    format: str
    vocab_size: int = 0
    hidden_size: int = 0
    num_layers: int = 0
    num_heads: int = 0
    context_length: int = 0
    chat_template: str = "plain"


class _GPTAdapter:
    """Gives the training-time ``GPT`` module the prefill / decode interface.  Decode steps run against per-block key /
    value tensors (``GPT.forward_cached``); when the learned positions run out, the window slides: the newest half of
    the tokens is prefilled again at positions 0 ... and decoding goes on from there."""

    def __init__(self, model, device):
        self.model, self.device = model.to(device).eval(), torch.device(device)
        self.tokens: Optional[torch.Tensor] = None
        self.kv = None

    def new_cache(self, batch: int, max_len: int):
        self.tokens, self.kv = None, None
        return self

    @torch.no_grad()
    def prefill(self, prompts: torch.Tensor, cache) -> torch.Tensor:
        ctx = self.model.cfg.n_positions
        self.tokens = prompts.to(self.device)[:, -ctx:]
        logits, self.kv = self.model.forward_cached(self.tokens)
        return logits[:, -1].float()

    @torch.no_grad()
    def decode_step(self, tokens: torch.Tensor, cache) -> torch.Tensor:
        new = tokens.view(-1, 1).to(self.device)
        self.tokens = torch.cat([self.tokens, new], 1)
        ctx = self.model.cfg.n_positions
        if self.tokens.shape[1] > ctx:                   # positions are learned and absolute: re-base the window
            self.tokens = self.tokens[:, -(ctx // 2):]
            logits, self.kv = self.model.forward_cached(self.tokens)
        else:
            logits, self.kv = self.model.forward_cached(new, self.kv)
        return logits[:, -1].float()


class ModelLoader:
    @staticmethod
    def from_file(path: str, device: str = "cpu", tokenizer_path: Optional[str] = None):
        """-> ``(runtime, tokenizer, ModelMetadata)``; ``ModelMetadata.chat_template`` names the chat layout that the
        file's tokenizer points to."""
        rt, tok, meta = ModelLoader._from_file(path, device, tokenizer_path)
        if path != "dummy" and meta.chat_template == "plain":
            from .session import detect_chat_template
            meta.chat_template = detect_chat_template(tok)
        return rt, tok, meta

    @staticmethod
    def _from_file(path: str, device: str = "cpu", tokenizer_path: Optional[str] = None):
        if path == "dummy":
            return None, ByteTokenizer(), ModelMetadata("dummy", "dummy", 258)
        if not os.path.exists(path):
            raise FileNotFoundError(path)
        fmt = detect_format(path)
        name = os.path.basename(path)
        if fmt == "gguf":
            with gguf_fmt.GGUFFile(path) as g:
                tok = load_tokenizer(tokenizer_path, g)
                mc = g.model_config()
                from .session import detect_chat_template
                template = detect_chat_template(tok, g.metadata)
            rt = LlamaRuntime.from_gguf(path, device)
            meta = ModelMetadata(name, "gguf", rt.cfg.vocab_size, rt.cfg.n_embd, rt.cfg.n_layer, rt.cfg.n_head, rt.cfg.context_length, template)
            if isinstance(tok, ByteTokenizer):
                tok = ByteTokenizer(rt.cfg.vocab_size)
            return rt, tok, meta
        if fmt == "huggingface":
            import json as _json
            cfg_path = os.path.join(path, "config.json")
            hf = _json.load(open(cfg_path)) if os.path.exists(cfg_path) else {}
            if str(hf.get("model_type", "")).lower() in ("llama", "mistral", "qwen2") or any(
                    k in a for a in hf.get("architectures", []) for k in ("Llama", "Mistral", "Qwen2ForCausalLM")):
                rt = LlamaRuntime.from_hf(path, device)
                tok = load_tokenizer(tokenizer_path or path, vocab_size=rt.cfg.vocab_size)
                meta = ModelMetadata(os.path.basename(os.path.normpath(path)), "huggingface", rt.cfg.vocab_size, rt.cfg.n_embd, rt.cfg.n_layer,
                                     rt.cfg.n_head, rt.cfg.context_length)
                return rt, tok, meta
            if str(hf.get("model_type", "")).lower() == "gpt2" or any("GPT2" in a for a in hf.get("architectures", [])):
                from ..models.gpt import GPT
                model = GPT.from_hf(path)
                tok = load_tokenizer(tokenizer_path or path, vocab_size=model.cfg.vocab_size)
                meta = ModelMetadata(os.path.basename(os.path.normpath(path)), "huggingface", model.cfg.vocab_size, model.cfg.n_embd,
                                     model.cfg.n_layer, model.cfg.n_head, model.cfg.n_positions)
                return _GPTAdapter(model, device), tok, meta
        if fmt in ("safetensors", "mlx", "rustorch", "torch", "pth", "huggingface", "json"):
            from ..models.gpt import GPT, GPTConfig
            from ..models.high_level import load_state_dict_file
            sd = load_state_dict_file(path)
            if "wte" not in sd or "wpe" not in sd or "blocks.0.w_qkv" not in sd:
                raise ValueError(f"{name}: not a GPT checkpoint of this framework (wte / wpe / blocks.N.w_qkv expected)")
            n_layer = 1 + max(int(k.split(".")[1]) for k in sd if k.startswith("blocks."))
            n_embd = sd["wpe"].shape[1]
            vocab = int(sd.get("vocab_size", torch.tensor(sd["wte"].shape[0])))
            cfg = GPTConfig(vocab_size=vocab, n_positions=sd["wpe"].shape[0], n_embd=n_embd, n_layer=n_layer,
                            n_head=max(1, n_embd // 64), dropout=0.0, tie_weights="lm_head" not in sd)
            if cfg.padded_vocab != sd["wte"].shape[0]:
                cfg.vocab_size = sd["wte"].shape[0]
            model = GPT(cfg)
            model.load_state_dict(sd, strict=False)
            meta = ModelMetadata(name, fmt, cfg.vocab_size, n_embd, n_layer, cfg.n_head, cfg.n_positions)
            return _GPTAdapter(model, device), load_tokenizer(tokenizer_path, vocab_size=cfg.vocab_size), meta
        raise ValueError(f"{name}: unsupported model format '{fmt}'")


class InferenceEngine:
    def __init__(self, runtime=None, tokenizer: Optional[Tokenizer] = None, generation: Optional[GenerationConfig] = None,
                 device: str = "cpu", seed: Optional[int] = None):
        self.runtime, self.tokenizer = runtime, tokenizer or ByteTokenizer()
        self.generation = generation or GenerationConfig()
        self.device, self.seed = device, seed
        self.timer = InferenceTimer()
        self.last_token_count = 0
        self.stop_ids: set = set()                    # ids besides the tokenizer's eos that end a reply

    def set_stop_tokens(self, names) -> None:
        """Ends replies at the named marker tokens too (those that the tokenizer knows)."""
        added = getattr(self.tokenizer, "added", None) or {}
        self.stop_ids = {added[n] for n in names if n in added}

    def is_loaded(self) -> bool:
        return self.runtime is not None

    def _sampler(self) -> Sampler:
        g = self.generation
        return Sampler(SamplingConfig(temperature=g.temperature, top_k=g.top_k, top_p=g.top_p, repetition_penalty=g.repetition_penalty,
                                      seed=self.seed), device=self.device)

    def stream(self, prompt: str) -> Iterator[str]:
        """Yields decoded text pieces as tokens are produced."""
        if self.runtime is None:                      # the reference's dummy model: echo
            reply = f"[no model loaded] You said: {prompt.strip().splitlines()[-1] if prompt.strip() else ''}"
            self.last_token_count = len(reply.split())
            yield reply
            return
        ids = self.tokenizer.encode(prompt)
        vocab = getattr(getattr(self.runtime, "cfg", None), "vocab_size", 0) or 0
        if vocab and ids and max(ids) >= vocab:
            raise ValueError(f"the tokenizer produced id {max(ids)} but the model's vocabulary has {vocab} entries: "
                             "pass --tokenizer <file> with the tokenizer that belongs to this model")
        ctx = getattr(getattr(self.runtime, "cfg", None), "context_length", 0) or 0
        budget = self.generation.max_tokens
        if ctx and len(ids) + budget > ctx:
            ids = ids[-max(1, ctx - budget):]
        sampler = self._sampler()
        self.timer.start()
        cache = self.runtime.new_cache(1, len(ids) + budget + 1)
        logits = self.runtime.prefill(torch.tensor([ids], dtype=torch.long), cache)
        out: List[int] = []
        emitted = ""
        for _ in range(budget):
            tok = int(sampler(logits.cpu() if logits.device.type != self.device else logits)[0])
            self.timer.token()
            if tok == self.tokenizer.eos_id or tok in self.stop_ids:
                break
            out.append(tok)
            text = self.tokenizer.decode(out)
            if not text.endswith("�"):           # hold back incomplete UTF-8 sequences
                yield text[len(emitted):]
                emitted = text
            logits = self.runtime.decode_step(torch.tensor([tok], dtype=torch.long), cache)
        self.last_token_count = len(out)

    def generate(self, prompt: str, on_token: Optional[Callable[[str], None]] = None) -> str:
        parts = []
        for piece in self.stream(prompt):
            parts.append(piece)
            if on_token:
                on_token(piece)
        return "".join(parts)

    def stats(self) -> dict:
        return {"tokens": self.last_token_count, "ttft_ms": self.timer.ttft_ms(), "tokens_per_s": self.timer.tokens_per_s()}
