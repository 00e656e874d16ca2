"""Loader / saver objects with the reference's names (src/formats/safetensors.rs:66-176, example-cli/src/model/
formats/gguf.rs, safetensors.rs:11-136, tensor_loader.rs:103-122, model/loader.rs:6-156, src/formats/onnx.rs:50-231).

The reference's CLI never wires these in (``load_gguf`` returns a dummy model); here they read real files.
"""
from __future__ import annotations

import os
from typing import Any, Dict, Iterator, List, Optional, Tuple

import torch

from . import gguf as _gguf
from . import safetensors as _st


class SafetensorsLoader:
    """mmap-backed reader: ``tensor_names() / tensor(name) / tensors() / metadata()``."""

    def __init__(self, path: str, device: str = "cpu"):
        self.path, self.device = path, device
        self._header, self._data_off = _st.read_safetensors_header(path)
        self._cache: Optional[Dict[str, torch.Tensor]] = None

    @classmethod
    def from_file(cls, path: str, device: str = "cpu") -> "SafetensorsLoader":
        return cls(path, device)

    def tensor_names(self) -> List[str]:
        return [k for k in self._header if k != "__metadata__"]

    def metadata(self) -> Dict[str, str]:
        return dict(self._header.get("__metadata__", {}))

    def tensor_info(self, name: str) -> Dict[str, Any]:
        return dict(self._header[name])

    def tensors(self) -> Dict[str, torch.Tensor]:
        if self._cache is None:
            self._cache = _st.load_safetensors(self.path, self.device)
        return self._cache

    def tensor(self, name: str) -> torch.Tensor:
        return self.tensors()[name]

    def __iter__(self) -> Iterator[Tuple[str, torch.Tensor]]:
        return iter(self.tensors().items())


class SafetensorsSaver:
    """Collects tensors and writes one file (8-byte padded header, sorted names)."""

    def __init__(self, metadata: Optional[Dict[str, str]] = None):
        self._tensors: Dict[str, torch.Tensor] = {}
        self._metadata = dict(metadata or {})

    def add_tensor(self, name: str, tensor: torch.Tensor) -> "SafetensorsSaver":
        self._tensors[name] = tensor.detach()
        return self

    def add_metadata(self, key: str, value: str) -> "SafetensorsSaver":
        self._metadata[key] = str(value)
        return self

    def save_to_file(self, path: str) -> None:
        _st.save_safetensors(self._tensors, path, self._metadata or None)

    save = save_to_file


Saver = SafetensorsSaver


class GGUFLoader:
    """``metadata / tensor_names / tensor_info / load_tensor / load_quantized / model_params`` over one GGUF file."""

    def __init__(self, path: str):
        self.file = _gguf.GGUFFile(path)

    @classmethod
    def from_file(cls, path: str) -> "GGUFLoader":
        return cls(path)

    def metadata(self) -> Dict[str, Any]:
        return self.file.metadata

    def tensor_names(self) -> List[str]:
        return list(self.file.tensors)

    def tensor_info(self, name: str) -> "_gguf.GGUFTensorInfo":
        return self.file.tensors[name]

    def architecture(self) -> str:
        return self.file.architecture()

    def model_params(self) -> Dict[str, Any]:
        """vocab_size, hidden_size, num_layers, num_heads, context_length ... from the ``<arch>.*`` keys."""
        return self.file.model_config()

    def load_tensor(self, name: str, dtype: torch.dtype = torch.float32) -> torch.Tensor:
        return self.file.load_tensor(name, dtype)

    def load_quantized(self, name: str):
        return self.file.load_quantized(name)

    def close(self) -> None:
        self.file.close()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()


class TensorLoader:
    """Format-agnostic front end: picks the reader from the file (GGUF, safetensors, RUSTORCH container, PyTorch zip,
    JSON) and returns dequantised fp32 tensors by name."""

    def __init__(self, path: str, device: str = "cpu"):
        self.path, self.device = path, device
        self.format = "gguf" if path.endswith(".gguf") else _st.detect_format(path)
        self._gguf = GGUFLoader(path) if self.format == "gguf" else None
        self._tensors: Optional[Dict[str, torch.Tensor]] = None

    def _load_all(self) -> Dict[str, torch.Tensor]:
        if self._tensors is None:
            if self._gguf is not None:
                self._tensors = {n: self._gguf.load_tensor(n).to(self.device) for n in self._gguf.tensor_names()}
            elif self.format == "safetensors":
                self._tensors = _st.load_safetensors(self.path, self.device)
            elif self.format in ("pth", "pytorch"):
                self._tensors = _st.load_pth(self.path)
            elif self.format == "json":
                self._tensors = _st.load_json_state_dict(self.path)[0]
            elif os.path.isdir(self.path):
                self._tensors = _st.load_huggingface(self.path, self.device)[0]
            else:
                from . import rustorch_bin
                self._tensors = rustorch_bin.load_state_dict(self.path) if hasattr(rustorch_bin, "load_state_dict") else {}
        return self._tensors

    def tensor_names(self) -> List[str]:
        return self._gguf.tensor_names() if self._gguf is not None else list(self._load_all())

    def load_tensor(self, name: str) -> torch.Tensor:
        if self._gguf is not None:
            return self._gguf.load_tensor(name).to(self.device)
        return self._load_all()[name]

    def load_all(self) -> Dict[str, torch.Tensor]:
        return self._load_all()
