"""The small helper classes of the reference's Python binding that have no other home
(src/python/utils.rs, training.rs, distributed.rs:114-428, data.rs): ``Device``, ``Config``, ``ModelSerializer``,
``ModelComparator``, ``Transform(s)``, ``DistributedConfig`` and the ``init_distributed`` family (real here: they
drive ``torch.distributed``; the reference's print and return)."""
from __future__ import annotations

import os
import platform
import random
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence

import numpy as np
import torch


class Device:
    """``Device("cpu")``, ``Device("cuda", 1)``, ``Device.cuda(0)``; ``metal`` is accepted as a name and reports
    unavailable."""

    def __init__(self, kind: str = "cpu", index: int = 0):
        kind = kind.lower()
        if ":" in kind:
            kind, idx = kind.split(":")
            index = int(idx)
        if kind not in ("cpu", "cuda", "metal"):
            raise ValueError(f"unknown device type '{kind}'")
        self.type, self.index = kind, index

    @classmethod
    def cpu(cls) -> "Device":
        return cls("cpu")

    @classmethod
    def cuda(cls, index: int = 0) -> "Device":
        return cls("cuda", index)

    @classmethod
    def metal(cls, index: int = 0) -> "Device":
        return cls("metal", index)

    def is_available(self) -> bool:
        return self.type == "cpu" or (self.type == "cuda" and torch.cuda.is_available() and self.index < torch.cuda.device_count())

    def torch(self) -> torch.device:
        if self.type == "metal":
            raise RuntimeError("Metal devices do not exist on this platform")
        return torch.device(self.type, self.index) if self.type == "cuda" else torch.device("cpu")

    def __repr__(self) -> str:
        return f"Device({self.type}:{self.index})" if self.type != "cpu" else "Device(cpu)"

    def __eq__(self, other) -> bool:
        return isinstance(other, Device) and (self.type, self.index) == (other.type, other.index)


class Config:
    """String-keyed settings with typed getters and environment override (``RUSTORCH_<KEY>``)."""

    # the binding's defaults (src/python/utils.rs:166-174)
    DEFAULTS = {"device": "cpu", "dtype": "float32", "backend": "native", "num_threads": "4", "memory_limit": "1024"}

    def __init__(self, **values):
        self._v: Dict[str, object] = {**self.DEFAULTS, **values}

    def set(self, key: str, value) -> None:
        self._v[key] = value

    def get(self, key: str, default=None):
        env = os.environ.get("RUSTORCH_" + key.upper())
        if env is not None:
            return env
        return self._v.get(key, default)

    def get_int(self, key: str, default: int = 0) -> int:
        return int(self.get(key, default))

    def get_float(self, key: str, default: float = 0.0) -> float:
        return float(self.get(key, default))

    def get_bool(self, key: str, default: bool = False) -> bool:
        v = self.get(key, default)
        return v if isinstance(v, bool) else str(v).lower() in ("1", "true", "yes", "on")

    def to_dict(self) -> Dict[str, object]:
        return dict(self._v)

    def all(self) -> Dict[str, object]:
        return dict(self._v)

    def load_from_file(self, path: str) -> None:
        """``key=value`` lines; blank lines and ``#`` comments are skipped (src/python/utils.rs:185-206)."""
        if not os.path.exists(path):
            raise FileNotFoundError(f"Configuration file not found: {path}")
        with open(path) as f:
            for line in f:
                line = line.strip()
                if not line or line.startswith("#") or "=" not in line:
                    continue
                k, v = line.split("=", 1)
                self._v[k.strip()] = v.strip()

    def save_to_file(self, path: str) -> None:
        with open(path, "w") as f:
            f.write("# RusTorch Configuration\n# Auto-generated configuration file\n\n")
            for k in sorted(self._v):
                f.write(f"{k}={self._v[k]}\n")

    def reset(self) -> None:
        self._v = dict(self.DEFAULTS)

    def __repr__(self) -> str:
        return f"Config(settings={len(self._v)})"


def set_seed(seed: int) -> None:
    random.seed(seed)
    np.random.seed(seed % (1 << 32))
    torch.manual_seed(seed)
    if torch.cuda.is_available():
        torch.cuda.manual_seed_all(seed)


def cuda_is_available() -> bool:
    return torch.cuda.is_available()


def get_system_info() -> Dict[str, object]:
    info = {"platform": platform.platform(), "python": platform.python_version(), "torch": torch.__version__,
            "cpu_count": os.cpu_count(), "cuda_available": torch.cuda.is_available(), "cuda_devices": []}
    if torch.cuda.is_available():
        for i in range(torch.cuda.device_count()):
            p = torch.cuda.get_device_properties(i)
            info["cuda_devices"].append({"index": i, "name": p.name, "memory_gb": round(p.total_memory / 2 ** 30, 1),
                                         "sms": p.multi_processor_count, "capability": f"{p.major}.{p.minor}"})
    from . import _native
    info["native_kernels"] = _native.available()
    return info


class ModelSerializer:
    @staticmethod
    def save(model: torch.nn.Module, path: str, fmt: str = "rustorch") -> None:
        from .models.high_level import ModelSaver, SerializationFormat
        ModelSaver.save(model, path, SerializationFormat(fmt) if not isinstance(fmt, SerializationFormat) else fmt)

    @staticmethod
    def load(model, path: Optional[str] = None, strict: bool = True):
        """``load(model, path)`` fills ``model``; the binding's ``load(path)`` (src/python/utils.rs:38-48) returns the
        tensors of the file as a dictionary, since a path alone does not say which architecture to build."""
        from .models.high_level import ModelLoader, load_state_dict_file
        if path is None and isinstance(model, (str, os.PathLike)):
            return load_state_dict_file(str(model))
        return ModelLoader.load(model, path, strict)

    @staticmethod
    def get_model_info(path: str) -> Dict[str, object]:
        """``exists`` / ``path`` / ``size`` (bytes) and, for a readable checkpoint, its format, tensor count and
        parameter count (src/python/utils.rs:50-69)."""
        if not os.path.exists(path):
            return {"exists": False}
        info: Dict[str, object] = {"exists": True, "path": path, "size": os.path.getsize(path)}
        try:
            from .formats import detect_format
            from .models.high_level import load_state_dict_file
            info["format"] = str(getattr(detect_format(path), "value", detect_format(path)))
            sd = load_state_dict_file(path)
            info["tensors"] = len(sd)
            info["parameters"] = int(sum(v.numel() for v in sd.values() if isinstance(v, torch.Tensor)))
        except Exception as e:  # noqa: BLE001  (an unreadable file still has a size)
            info["error"] = f"{type(e).__name__}: {e}"
        return info

    @staticmethod
    def export(model: torch.nn.Module, path: str, format: Optional[str] = None) -> None:
        """``format``: ``rustorch`` (default), ``safetensors``, ``pytorch`` / ``pth``, ``json`` (src/python/utils.rs:71-100)."""
        from .models.high_level import ModelSaver, SerializationFormat
        name = {"pth": "pytorch", "pt": "pytorch", "torch": "pytorch", None: "rustorch"}.get(format, format)
        try:
            fmt = SerializationFormat(name)
        except ValueError:
            raise ValueError(f"Unsupported export format: {format}") from None
        ModelSaver.save(model, path, fmt)


class ModelComparator:
    """Parameter-wise and output-wise comparison of two models."""

    @staticmethod
    def get_stats(model: torch.nn.Module) -> Dict[str, object]:
        """Name, layer count, layer-kind histogram and parameter count (src/python/utils.rs:131-157)."""
        layers = list(getattr(model, "layers", None) or [m for m in model.children()])
        kinds: Dict[str, int] = {}
        for l in layers:
            n = type(l).__name__
            kind = ("dense" if n in ("Dense", "Linear") else "convolutional" if "Conv" in n else "dropout" if "Dropout" in n else "other")
            kinds[f"{kind}_layers"] = kinds.get(f"{kind}_layers", 0) + 1
        return {"name": getattr(model, "name", type(model).__name__), "num_layers": len(layers),
                "compiled": bool(getattr(model, "compiled", False)),
                "parameters": sum(p.numel() for p in model.parameters()), **kinds}

    @staticmethod
    def compare(model1: torch.nn.Module, model2: torch.nn.Module) -> Dict[str, object]:
        """Structure of two models side by side (src/python/utils.rs:113-129) plus whether their parameters agree."""
        a, b = ModelComparator.get_stats(model1), ModelComparator.get_stats(model2)
        sig = lambda m: [(type(l).__name__, tuple(tuple(p.shape) for p in l.parameters()))   # noqa: E731
                         for l in (getattr(m, "layers", None) or m.children())]
        same_layers = sig(model1) == sig(model2)
        return {"model1_name": a["name"], "model2_name": b["name"], "model1_layers": a["num_layers"], "model2_layers": b["num_layers"],
                "model1_compiled": a["compiled"], "model2_compiled": b["compiled"], "layers_identical": same_layers,
                "compilation_identical": a["compiled"] == b["compiled"],
                "parameters_identical": same_layers and ModelComparator.compare_parameters(model1, model2)["identical"]}

    @staticmethod
    def compare_parameters(a: torch.nn.Module, b: torch.nn.Module, atol: float = 0.0) -> Dict[str, object]:
        sa, sb = a.state_dict(), b.state_dict()
        missing = sorted(set(sa) ^ set(sb))
        diffs = {k: float((sa[k].float() - sb[k].float()).abs().max()) for k in sa if k in sb and sa[k].shape == sb[k].shape}
        shape_mismatch = [k for k in sa if k in sb and sa[k].shape != sb[k].shape]
        return {"identical": not missing and not shape_mismatch and all(v <= atol for v in diffs.values()), "missing": missing,
                "shape_mismatch": shape_mismatch, "max_abs_diff": max(diffs.values(), default=0.0), "per_parameter": diffs}

    @staticmethod
    def compare_outputs(a: torch.nn.Module, b: torch.nn.Module, x: torch.Tensor) -> Dict[str, float]:
        with torch.no_grad():
            ya, yb = a(x).float(), b(x).float()
        d = (ya - yb).abs()
        return {"max_abs_diff": float(d.max()), "mean_abs_diff": float(d.mean()),
                "cosine": float(torch.nn.functional.cosine_similarity(ya.flatten(), yb.flatten(), dim=0))}


class Transform:
    """A named image transform of the Python binding (src/python/data.rs)."""

    def __init__(self, fn: Callable[[torch.Tensor], torch.Tensor], name: str = "transform"):
        self.fn, self.name = fn, name

    def __call__(self, x):
        return self.fn(x)


class Transforms:
    """Factory with the binding's names: ``normalize resize random_crop random_horizontal_flip compose``."""

    @staticmethod
    def normalize(mean: Sequence[float], std: Sequence[float]) -> Transform:
        from .vision import Normalize
        return Transform(Normalize(mean, std), "normalize")

    @staticmethod
    def resize(size) -> Transform:
        from .vision import Resize
        return Transform(Resize(size), "resize")

    @staticmethod
    def random_crop(size, padding: int = 0) -> Transform:
        from .vision import RandomCrop
        return Transform(RandomCrop(size, padding), "random_crop")

    @staticmethod
    def random_horizontal_flip(p: float = 0.5) -> Transform:
        from .vision import RandomHorizontalFlip
        return Transform(RandomHorizontalFlip(p), "random_horizontal_flip")

    @staticmethod
    def compose(ts: Sequence[Callable]) -> Transform:
        from .vision import Compose
        return Transform(Compose(ts), "compose")


@dataclass
class DistributedConfig:
    backend: str = "nccl"
    init_method: str = "env://"
    world_size: int = 1
    rank: int = 0
    timeout_s: float = 1800.0
    master_addr: str = "127.0.0.1"
    master_port: int = 29500


def init_distributed(config: Optional[DistributedConfig] = None) -> None:
    from .distributed import api
    c = config or DistributedConfig(backend="nccl" if torch.cuda.is_available() else "gloo",
                                    world_size=int(os.environ.get("WORLD_SIZE", "1")), rank=int(os.environ.get("RANK", "0")))
    os.environ.setdefault("MASTER_ADDR", c.master_addr)
    os.environ.setdefault("MASTER_PORT", str(c.master_port))
    api.init_process_group(c.backend, c.init_method, c.world_size, c.rank, c.timeout_s)


class DistributedBackend:
    """The binding's back-end object (src/python/distributed.rs:169-297): holds the back-end name and drives the
    process group and the basic collectives.  ``DistributedBackend("nccl")``; the enumeration of back-end kinds is
    ``rustorch_b200.distributed.DistributedBackend``.  Collectives accept ``torch.Tensor``, ``Tensor`` or
    ``Variable`` and work in place on the wrapped tensor, returning their argument."""

    def __init__(self, backend_type: Optional[str] = None):
        from .distributed.api import DistributedBackend as Kind
        self.backend_type = Kind.parse(backend_type or ("nccl" if torch.cuda.is_available() else "gloo")).value

    @property
    def value(self) -> str:
        return self.backend_type

    def init_process_group(self, config: Optional[DistributedConfig] = None) -> None:
        c = config or DistributedConfig(backend=self.backend_type, world_size=int(os.environ.get("WORLD_SIZE", "1")),
                                        rank=int(os.environ.get("RANK", "0")))
        if c.backend != self.backend_type:
            c = DistributedConfig(**{**c.__dict__, "backend": self.backend_type})
        init_distributed(c)

    def destroy_process_group(self) -> None:
        cleanup_distributed()

    def is_initialized(self) -> bool:
        from .distributed import api
        return api.is_initialized()

    def barrier(self) -> None:
        from .distributed import api
        api.barrier()

    @staticmethod
    def _raw(t) -> torch.Tensor:
        if isinstance(t, torch.Tensor):
            return t
        from .autograd import Variable
        return t.tensor if isinstance(t, Variable) else t.data

    def all_reduce(self, tensor, op: str = "sum"):
        from .distributed import api
        api.all_reduce(self._raw(tensor), api.ReduceOp(op))
        return tensor

    def all_gather(self, tensor) -> list:
        from .distributed import api
        return api.all_gather(self._raw(tensor))

    def broadcast(self, tensor, src: int = 0):
        from .distributed import api
        api.broadcast(self._raw(tensor), src)
        return tensor

    def __repr__(self) -> str:
        return f"DistributedBackend(backend='{self.backend_type}', initialized={self.is_initialized()})"


def cleanup_distributed() -> None:
    from .distributed import api
    api.destroy_process_group()
