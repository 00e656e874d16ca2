"""TOML configuration ``~/.rustorch/config.toml`` (example-cli/src/utils/config.rs:11-261): sections
``[model] [generation] [backend] [session] [ui]`` with the reference's defaults.  Priority: CLI > file > defaults."""
from __future__ import annotations

import os
import tomllib
from dataclasses import asdict, dataclass, field
from typing import Optional


@dataclass
class ModelConfig:
    default: Optional[str] = None
    cache_dir: str = "~/.rustorch/models"


@dataclass
class GenerationSection:
    max_tokens: int = 512
    temperature: float = 0.7
    top_p: float = 0.9
    top_k: int = 40


@dataclass
class BackendConfig:
    default: str = "cpu"
    fallback: str = "cpu"


@dataclass
class SessionConfig:
    auto_save: bool = True
    history_file: str = "~/.rustorch/history"
    max_history: int = 1000


@dataclass
class UiConfig:
    color: bool = True
    stream: bool = True
    show_metrics: bool = False


def _toml_value(v) -> str:
    if isinstance(v, bool):
        return "true" if v else "false"
    if isinstance(v, (int, float)):
        return repr(v)
    return '"' + str(v).replace("\\", "\\\\").replace('"', '\\"') + '"'


@dataclass
class Config:
    model: ModelConfig = field(default_factory=ModelConfig)
    generation: GenerationSection = field(default_factory=GenerationSection)
    backend: BackendConfig = field(default_factory=BackendConfig)
    session: SessionConfig = field(default_factory=SessionConfig)
    ui: UiConfig = field(default_factory=UiConfig)

    @staticmethod
    def default_path() -> str:
        return os.path.join(os.path.expanduser("~"), ".rustorch", "config.toml")

    @classmethod
    def load(cls, path: Optional[str] = None) -> "Config":
        path = path or cls.default_path()
        with open(path, "rb") as f:
            doc = tomllib.load(f)
        c = cls()
        for section, obj in (("model", c.model), ("generation", c.generation), ("backend", c.backend), ("session", c.session), ("ui", c.ui)):
            for k, v in doc.get(section, {}).items():
                if not hasattr(obj, k):
                    raise ValueError(f"unknown key [{section}].{k}")
                setattr(obj, k, v)
        c.validate()
        return c

    @classmethod
    def load_or_default(cls, path: Optional[str] = None) -> "Config":
        try:
            return cls.load(path)
        except FileNotFoundError:
            return cls()

    def validate(self) -> None:
        g = self.generation
        if not 0.0 <= g.temperature <= 2.0 or not 0.0 <= g.top_p <= 1.0 or g.top_k < 1 or g.max_tokens < 1:
            raise ValueError("invalid [generation] values")

    def to_toml(self) -> str:
        out = []
        for name, section in asdict(self).items():
            out.append(f"[{name}]")
            out += [f"{k} = {_toml_value(v)}" for k, v in section.items() if v is not None]
            out.append("")
        return "\n".join(out)

    def save(self, path: Optional[str] = None) -> str:
        path = path or self.default_path()
        os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
        with open(path, "w") as f:
            f.write(self.to_toml())
        return path

    @staticmethod
    def expand(path: str) -> str:
        return os.path.expanduser(path)
