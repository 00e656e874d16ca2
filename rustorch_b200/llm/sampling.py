"""Token sampling: temperature, top-k, top-p (nucleus), repetition penalty, multinomial draw
(example-cli/src/model/sampling.rs:8-300; the reference's ``sample_token`` is a placeholder returning
``vocab/2`` and its repetition penalty is a TODO)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Sequence

import torch


@dataclass
class SamplingConfig:
    temperature: float = 1.0
    top_k: int = 0            # 0 = disabled
    top_p: float = 1.0        # 1.0 = disabled
    repetition_penalty: float = 1.0
    seed: Optional[int] = None

    def validate(self) -> None:
        if self.temperature < 0:
            raise ValueError("temperature must be >= 0")
        if self.top_k < 0:
            raise ValueError("top_k must be >= 0")
        if not 0.0 < self.top_p <= 1.0:
            raise ValueError("top_p must be in (0, 1]")
        if self.repetition_penalty <= 0:
            raise ValueError("repetition_penalty must be > 0")

    @staticmethod
    def greedy() -> "SamplingConfig":
        return SamplingConfig(temperature=0.0)


def softmax(logits: torch.Tensor) -> torch.Tensor:
    return torch.softmax(logits.float(), -1)


def apply_repetition_penalty(logits: torch.Tensor, history: torch.Tensor, penalty: float) -> torch.Tensor:
    """Divide positive / multiply negative logits of already generated tokens by ``penalty``."""
    if penalty == 1.0 or history.numel() == 0:
        return logits
    out = logits.clone()
    g = out.gather(-1, history)
    out.scatter_(-1, history, torch.where(g > 0, g / penalty, g * penalty))
    return out


def apply_top_k_to_probs(probs: torch.Tensor, k: int) -> torch.Tensor:
    if k <= 0 or k >= probs.shape[-1]:
        return probs
    kth = probs.topk(k, -1).values[..., -1:]
    p = torch.where(probs < kth, torch.zeros_like(probs), probs)
    return p / p.sum(-1, keepdim=True)


def apply_top_p_to_probs(probs: torch.Tensor, top_p: float) -> torch.Tensor:
    if top_p >= 1.0:
        return probs
    sp, si = probs.sort(-1, descending=True)
    cum = sp.cumsum(-1)
    keep = cum - sp < top_p                   # always keeps the most probable token
    sp = torch.where(keep, sp, torch.zeros_like(sp))
    p = torch.zeros_like(probs).scatter_(-1, si, sp)
    return p / p.sum(-1, keepdim=True)


def multinomial_sample(probs: torch.Tensor, generator: Optional[torch.Generator] = None) -> torch.Tensor:
    return torch.multinomial(probs, 1, generator=generator).squeeze(-1)


class Sampler:
    """Callable ``logits [B, V] -> tokens [B]`` carrying the configuration and the generated history."""

    def __init__(self, config: Optional[SamplingConfig] = None, device=None):
        self.config = config or SamplingConfig()
        self.config.validate()
        self.history: Optional[torch.Tensor] = None
        self._gen = None
        if self.config.seed is not None:
            self._gen = torch.Generator(device=device or "cpu").manual_seed(self.config.seed)

    def __call__(self, logits: torch.Tensor) -> torch.Tensor:
        c = self.config
        logits = logits.float()
        if self.history is not None:
            logits = apply_repetition_penalty(logits, self.history, c.repetition_penalty)
        if c.temperature == 0.0:
            tok = logits.argmax(-1)
        else:
            probs = softmax(logits / c.temperature)
            probs = apply_top_p_to_probs(apply_top_k_to_probs(probs, c.top_k), c.top_p)
            gen = self._gen if (self._gen is not None and self._gen.device == probs.device) else None
            tok = multinomial_sample(probs, gen)
        t = tok.view(-1, 1)
        self.history = t if self.history is None else torch.cat([self.history, t], 1)
        return tok

    def reset(self) -> None:
        self.history = None


def sample_token(logits: torch.Tensor, config: Optional[SamplingConfig] = None) -> int:
    return int(Sampler(config)(logits.view(1, -1))[0])
