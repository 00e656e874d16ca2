"""Command-line arguments (example-cli/src/cli/args.rs:12-320): same flags, defaults and sub-commands."""
from __future__ import annotations

import argparse
from dataclasses import dataclass
from enum import Enum
from typing import List, Optional


class Backend(Enum):
    CPU = "cpu"
    CUDA = "cuda"
    METAL = "metal"
    OPENCL = "opencl"
    HYBRID = "hybrid"
    HYBRID_F32 = "hybrid-f32"

    def available(self) -> bool:
        import torch
        return self is Backend.CPU or (self is Backend.CUDA and torch.cuda.is_available())

    def device(self) -> str:
        """Back-ends that do not exist on this platform resolve to the best available one."""
        import torch
        return "cuda" if (self is not Backend.CPU and torch.cuda.is_available()) else "cpu"


@dataclass
class CliArgs:
    model: Optional[str] = None
    backend: Backend = Backend.CPU
    config: Optional[str] = None
    log_level: str = "info"
    max_tokens: int = 512
    temperature: float = 0.7
    top_p: float = 0.9
    top_k: int = 40
    system_prompt: Optional[str] = None
    chat_template: Optional[str] = None
    save_history: Optional[str] = None
    load_history: Optional[str] = None
    no_progress: bool = False
    tokenizer: Optional[str] = None
    prompt: Optional[str] = None          # one-shot mode: answer and exit
    command: Optional[str] = None         # download | list
    target: Optional[str] = None
    output_dir: Optional[str] = None
    revision: Optional[str] = None
    token: Optional[str] = None
    force: bool = False

    def validate(self) -> None:
        if not 0.0 <= self.temperature <= 2.0:
            raise ValueError("temperature must be between 0.0 and 2.0")
        if not 0.0 <= self.top_p <= 1.0:
            raise ValueError("top-p must be between 0.0 and 1.0")
        if self.top_k < 1:
            raise ValueError("top-k must be at least 1")
        if self.max_tokens < 1:
            raise ValueError("max-tokens must be at least 1")


def build_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(prog="rustorch-cli", description="Interactive CLI for local LLM inference")
    p.add_argument("-m", "--model", help="path to a model file (GGUF, safetensors, MLX, .pt)")
    p.add_argument("-b", "--backend", default="cpu", choices=[b.value for b in Backend])
    p.add_argument("-c", "--config", help="TOML configuration file")
    p.add_argument("--log-level", default="info", choices=["trace", "debug", "info", "warn", "error"])
    p.add_argument("--max-tokens", type=int, default=None)
    p.add_argument("--temperature", type=float, default=None)
    p.add_argument("--top-p", type=float, default=None)
    p.add_argument("--top-k", type=int, default=None)
    p.add_argument("--system-prompt")
    p.add_argument("--save-history")
    p.add_argument("--load-history")
    p.add_argument("--no-progress", action="store_true")
    p.add_argument("--tokenizer", help="tokenizer file (sentencepiece .model); GGUF files carry their own")
    p.add_argument("--prompt", help="answer one prompt and exit")
    p.add_argument("--chat-template", default=None, choices=["auto", "plain", "llama3", "chatml", "llama2"],
                   help="chat layout of the prompt (auto: from the model's tokenizer)")
    sub = p.add_subparsers(dest="command")
    d = sub.add_parser("download", help="download a model: hf:<org>/<repo>[:file] or ollama:<name>[:tag]")
    d.add_argument("target")
    d.add_argument("--output-dir")
    d.add_argument("--revision")
    d.add_argument("--token")
    d.add_argument("--force", action="store_true")
    l = sub.add_parser("list", help="list downloaded models of a source (hf | ollama | all)")
    l.add_argument("target", nargs="?", default="all")
    return p


def parse_args(argv: Optional[List[str]] = None, config=None) -> CliArgs:
    """CLI flags override the configuration file, which overrides the defaults."""
    ns = build_parser().parse_args(argv)
    a = CliArgs(model=ns.model, backend=Backend(ns.backend), config=ns.config, log_level=ns.log_level, system_prompt=ns.system_prompt,
                save_history=ns.save_history, load_history=ns.load_history, no_progress=ns.no_progress, tokenizer=ns.tokenizer,
                prompt=ns.prompt, chat_template=ns.chat_template, command=ns.command, target=getattr(ns, "target", None), output_dir=getattr(ns, "output_dir", None),
                revision=getattr(ns, "revision", None), token=getattr(ns, "token", None), force=getattr(ns, "force", False))
    if config is None and ns.config:
        from .config import Config
        config = Config.load(ns.config)
    g = config.generation if config is not None else None
    a.max_tokens = ns.max_tokens if ns.max_tokens is not None else (g.max_tokens if g else 512)
    a.temperature = ns.temperature if ns.temperature is not None else (g.temperature if g else 0.7)
    a.top_p = ns.top_p if ns.top_p is not None else (g.top_p if g else 0.9)
    a.top_k = ns.top_k if ns.top_k is not None else (g.top_k if g else 40)
    if config is not None:
        if a.model is None:
            a.model = config.model.default
        if ns.backend == "cpu" and config.backend.default != "cpu":
            a.backend = Backend(config.backend.default)
    a.validate()
    return a
