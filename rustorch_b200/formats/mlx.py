"""MLX model files (``.mlx`` / MLX-exported weights).

An MLX weight file has the safetensors framing: an 8-byte little-endian header length, a JSON header that maps
tensor names to ``{"dtype", "shape", "data_offsets"}`` (offsets relative to the end of the header) plus an
optional ``"__metadata__"`` object, then the raw little-endian tensor bytes.  The reference reads exactly that
(example-cli/src/model/formats/mlx.rs:12-144): dtypes ``F32 / F16 / I32 / I64`` (also spelled ``float32`` ...),
every tensor widened to f64, and the model description taken from ``__metadata__`` with Llama-7B defaults
(vocab 32000, hidden 4096, 32 layers, 32 heads, context 2048) when a key is missing.

Here tensors keep their stored dtype (``BF16`` is read as well, which MLX exports and the reference rejects),
metadata values may be JSON numbers or numeric strings (safetensors metadata is string-valued), and a corrupt
header or an offset past the end of the file raises :class:`ModelFormatError` instead of slicing garbage.
"""
from __future__ import annotations

import json
import os
import struct
from dataclasses import dataclass
from typing import Dict, Optional, Tuple

import numpy as np
import torch

from ..error import ModelFormatError

_DTYPES = {
    "F32": (np.dtype("<f4"), torch.float32), "FLOAT32": (np.dtype("<f4"), torch.float32),
    "F16": (np.dtype("<f2"), torch.float16), "FLOAT16": (np.dtype("<f2"), torch.float16),
    "I32": (np.dtype("<i4"), torch.int32), "INT32": (np.dtype("<i4"), torch.int32),
    "I64": (np.dtype("<i8"), torch.int64), "INT64": (np.dtype("<i8"), torch.int64),
    "BF16": (np.dtype("<u2"), torch.bfloat16), "BFLOAT16": (np.dtype("<u2"), torch.bfloat16),
    "U8": (np.dtype("u1"), torch.uint8), "UINT8": (np.dtype("u1"), torch.uint8),
}
_NAMES = {torch.float32: "F32", torch.float16: "F16", torch.int32: "I32", torch.int64: "I64", torch.bfloat16: "BF16",
          torch.uint8: "U8"}


@dataclass
class MLXModelMetadata:
    """The reference's ``ModelMetadata`` for an MLX file (mlx.rs:146-181)."""
    name: str = "mlx_model"
    format: str = "mlx"
    vocab_size: int = 32000
    hidden_size: int = 4096
    num_layers: int = 32
    num_heads: int = 32
    context_length: int = 2048


def _meta_int(meta: dict, key: str, default: int) -> int:
    v = meta.get(key, default)
    try:
        return int(v)
    except (TypeError, ValueError):
        return default


def extract_metadata(header: dict) -> MLXModelMetadata:
    meta = header.get("__metadata__") if isinstance(header, dict) else None
    meta = meta if isinstance(meta, dict) else {}
    return MLXModelMetadata(
        vocab_size=_meta_int(meta, "vocab_size", 32000), hidden_size=_meta_int(meta, "hidden_size", 4096),
        num_layers=_meta_int(meta, "num_hidden_layers", 32), num_heads=_meta_int(meta, "num_attention_heads", 32),
        context_length=_meta_int(meta, "max_position_embeddings", 2048))


def parse_tensor(data: bytes, shape, dtype: str) -> torch.Tensor:
    key = dtype.upper()
    if key not in _DTYPES:
        raise ModelFormatError(f"unsupported MLX dtype: {dtype}")
    np_dt, t_dt = _DTYPES[key]
    n = int(np.prod(shape)) if len(shape) else 1
    if len(data) != n * np_dt.itemsize:
        raise ModelFormatError(f"MLX tensor of shape {list(shape)} and dtype {dtype} needs {n * np_dt.itemsize} bytes, got {len(data)}")
    arr = np.frombuffer(data, dtype=np_dt).copy()
    t = torch.from_numpy(arr)
    if t_dt == torch.bfloat16:
        t = t.view(torch.int16).view(torch.bfloat16)
    return t.reshape(tuple(int(s) for s in shape))


class MLXLoader:
    """``MLXLoader.load(path) -> (tensors, metadata)``."""

    @staticmethod
    def read_header(path: str) -> Tuple[dict, int]:
        size = os.path.getsize(path)
        if size < 8:
            raise ModelFormatError(f"MLX file too small: {size} bytes")
        with open(path, "rb") as f:
            (n,) = struct.unpack("<Q", f.read(8))
            if 8 + n > size:
                raise ModelFormatError(f"MLX file corrupted: metadata size {n} exceeds file size {size}")
            raw = f.read(n)
        try:
            header = json.loads(raw)
        except ValueError as e:
            raise ModelFormatError(f"failed to parse MLX metadata: {e}") from e
        if not isinstance(header, dict):
            raise ModelFormatError("invalid MLX metadata format")
        return header, 8 + n

    @staticmethod
    def load(path: str, device: str = "cpu", dtype: Optional[torch.dtype] = None) -> Tuple[Dict[str, torch.Tensor], MLXModelMetadata]:
        header, data_start = MLXLoader.read_header(path)
        size = os.path.getsize(path)
        tensors: Dict[str, torch.Tensor] = {}
        with open(path, "rb") as f:
            for name, meta in header.items():
                if name == "__metadata__":
                    continue
                for k in ("dtype", "shape", "data_offsets"):
                    if not isinstance(meta, dict) or k not in meta:
                        raise ModelFormatError(f"missing {k} for tensor {name}")
                start, end = (int(x) for x in meta["data_offsets"])
                if start < 0 or end < start or data_start + end > size:
                    raise ModelFormatError(f"tensor {name}: data offsets [{start}, {end}) outside the file")
                f.seek(data_start + start)
                t = parse_tensor(f.read(end - start), meta["shape"], meta["dtype"])
                if dtype is not None and t.is_floating_point():
                    t = t.to(dtype)
                tensors[name] = t.to(device)
        md = extract_metadata(header)
        md.name = os.path.basename(path)
        return tensors, md


def save_mlx(path: str, tensors: Dict[str, torch.Tensor], metadata: Optional[dict] = None) -> None:
    """Write tensors in the layout :class:`MLXLoader` reads (used for export and by the tests)."""
    header: dict = {}
    if metadata:
        header["__metadata__"] = {k: (v if isinstance(v, (int, float)) else str(v)) for k, v in metadata.items()}
    blobs, off = [], 0
    for name, t in tensors.items():
        t = t.detach().cpu().contiguous()
        if t.dtype not in _NAMES:
            t = t.float()
        raw = (t.view(torch.int16) if t.dtype == torch.bfloat16 else t).numpy().tobytes()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + len(raw)]}
        blobs.append(raw)
        off += len(raw)
    hj = json.dumps(header, separators=(",", ":")).encode()
    hj += b" " * (-len(hj) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for b in blobs:
            f.write(b)


load_mlx = MLXLoader.load
