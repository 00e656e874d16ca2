"""safetensors, the "PyTorch" formats of the reference, and the HuggingFace directory layout.

* safetensors: u64-LE header length · JSON ``{name: {dtype, shape, data_offsets:[begin,end]}}`` · raw
  little-endian data.  The reference's hand-rolled writer emits F32/F64 only and does not pad the header
  (src/serialization/formats.rs:117-245); files written here follow the published spec (header padded with
  spaces to 8 bytes, optional ``__metadata__``, BF16/F16/I*/U8/BOOL too) and the reader accepts both.
  Loading memory-maps the file so tensors are views until moved.
* ``save_pth`` / ``load_pth``: the reference's own ``"PYTORCH1"`` binary (u32 n · [u32 name_len · name · u32 ndim ·
  u64 dims · u64 bytes · data], formats.rs:44-83).  A real torch pickle/zip file is detected by its magic and
  loaded with ``torch.load(weights_only=True)`` (the reference errors out there, :20-40).
* JSON state dict ``{tensors: {name: {shape, data, dtype}}, metadata}`` (src/formats/pytorch.rs:16-96).
* HuggingFace directory: ``model.safetensors`` + ``config.json`` (formats.rs:249-294).
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from typing import Dict, Optional, Tuple

import numpy as np
import torch

_ST_DTYPES = {
    "F64": torch.float64, "F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16,
    "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8, "U8": torch.uint8,
    "BOOL": torch.bool,
}
_ST_NAMES = {v: k for k, v in _ST_DTYPES.items()}


def save_safetensors(tensors: Dict[str, torch.Tensor], path: str, metadata: Optional[Dict[str, str]] = None) -> None:
    header, blobs, off = {}, [], 0
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    for name in sorted(tensors):
        t = tensors[name].detach().contiguous().cpu()
        if t.dtype not in _ST_NAMES:
            raise TypeError(f"dtype {t.dtype} of '{name}' cannot be stored in safetensors")
        raw = t.reshape(-1).view(torch.uint8).numpy().tobytes() if t.numel() else b""
        header[name] = {"dtype": _ST_NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + len(raw)]}
        blobs.append(raw)
        off += len(raw)
    hj = json.dumps(header, separators=(",", ":")).encode()
    hj += b" " * ((8 - len(hj) % 8) % 8)
    os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for b in blobs:
            f.write(b)


def read_safetensors_header(path: str) -> Tuple[dict, int]:
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        if n > 100 * 1024 * 1024:
            raise ValueError("safetensors header larger than 100 MB")
        return json.loads(f.read(n).decode()), 8 + n


def load_safetensors(path: str, device: str = "cpu", use_mmap: bool = True) -> Dict[str, torch.Tensor]:
    header, base = read_safetensors_header(path)
    out: Dict[str, torch.Tensor] = {}
    with open(path, "rb") as f:
        buf = mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_READ) if use_mmap and os.path.getsize(path) > 0 else f.read()
    for name, info in header.items():
        if name == "__metadata__":
            continue
        dt = _ST_DTYPES[info["dtype"]]
        b, e = info["data_offsets"]
        n = e - b
        if n == 0:
            out[name] = torch.empty(info["shape"], dtype=dt)
            continue
        arr = np.frombuffer(buf, dtype=np.uint8, count=n, offset=base + b)
        t = torch.from_numpy(arr.copy() if not use_mmap else arr).view(dt).reshape(info["shape"])
        out[name] = t.to(device) if device != "cpu" else (t.clone() if use_mmap else t)
    return out


class SafetensorsFile:
    """One safetensors file read tensor by tensor from a memory map: ``keys()``, ``shape(name)``, ``get(name)`` (a copy,
    so the file can be closed).  For checkpoints that are too large to materialise whole."""

    def __init__(self, path: str):
        self.path = path
        self.header, self._base = read_safetensors_header(path)
        self._f = open(path, "rb")
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ) if os.path.getsize(path) > 0 else b""

    def keys(self):
        return [k for k in self.header if k != "__metadata__"]

    def __contains__(self, name: str) -> bool:
        return name in self.header and name != "__metadata__"

    def shape(self, name: str) -> Tuple[int, ...]:
        return tuple(self.header[name]["shape"])

    def get(self, name: str) -> torch.Tensor:
        info = self.header[name]
        b, e = info["data_offsets"]
        dt = _ST_DTYPES[info["dtype"]]
        if e == b:
            return torch.empty(info["shape"], dtype=dt)
        arr = np.frombuffer(self._mm, dtype=np.uint8, count=e - b, offset=self._base + b).copy()
        return torch.from_numpy(arr).view(dt).reshape(info["shape"])

    def close(self) -> None:
        if not isinstance(self._mm, bytes):
            self._mm.close()
        self._f.close()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()
        return False


def hf_rope_settings(config: dict) -> Tuple[float, Optional[dict]]:
    """``(rope_theta, rope_scaling or None)`` of a Hugging Face ``config.json``.  Older files carry ``rope_theta`` and
    ``rope_scaling`` at the top level; newer ones one ``rope_parameters`` entry that holds the base, the type and the
    scaling factors together."""
    rp = config.get("rope_parameters")
    if isinstance(rp, dict):
        theta = float(rp.get("rope_theta", config.get("rope_theta", 10000.0)))
        kind = str(rp.get("rope_type", rp.get("type", "default"))).lower()
        scaling = None if kind in ("default", "none") else {k: v for k, v in rp.items() if k != "rope_theta"}
        return theta, scaling
    sc = config.get("rope_scaling") or None
    if isinstance(sc, dict) and str(sc.get("rope_type", sc.get("type", "default"))).lower() in ("default", "none"):
        sc = None
    return float(config.get("rope_theta", 10000.0)), sc


def hf_attention_window(config: dict) -> Optional[int]:
    """Width of the sliding attention window that a Hugging Face config switches on, or None.  Mistral-style configs
    switch it on by giving ``sliding_window`` a value; Qwen2-style ones carry a value but use it only with
    ``use_sliding_window``."""
    width = config.get("sliding_window")
    if not width:
        return None
    default_on = str(config.get("model_type", "")).lower() not in ("qwen2", "qwen2_moe", "qwen3")
    return int(width) if config.get("use_sliding_window", default_on) else None


class HuggingFaceCheckpoint:
    """A Hugging Face model directory: ``config.json`` plus ``model.safetensors`` or the shards named by
    ``model.safetensors.index.json``; tensors are fetched one at a time from whichever shard holds them."""

    def __init__(self, directory: str):
        self.directory = directory
        cp = os.path.join(directory, "config.json")
        self.config: dict = {}
        if os.path.exists(cp):
            with open(cp) as f:
                self.config = json.load(f)
        idx = os.path.join(directory, "model.safetensors.index.json")
        if os.path.exists(idx):
            with open(idx) as f:
                self.weight_map: Dict[str, str] = dict(json.load(f)["weight_map"])
        else:
            single = os.path.join(directory, "model.safetensors")
            if not os.path.exists(single):
                raise FileNotFoundError(f"{directory}: neither model.safetensors nor model.safetensors.index.json")
            with SafetensorsFile(single) as f:
                self.weight_map = {k: "model.safetensors" for k in f.keys()}
        self._open: Dict[str, SafetensorsFile] = {}

    def keys(self):
        return list(self.weight_map)

    def __contains__(self, name: str) -> bool:
        return name in self.weight_map

    def _file(self, name: str) -> SafetensorsFile:
        shard = self.weight_map[name]
        if shard not in self._open:
            self._open[shard] = SafetensorsFile(os.path.join(self.directory, shard))
        return self._open[shard]

    def shape(self, name: str) -> Tuple[int, ...]:
        return self._file(name).shape(name)

    def get(self, name: str) -> torch.Tensor:
        return self._file(name).get(name)

    def close(self) -> None:
        for f in self._open.values():
            f.close()
        self._open.clear()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()
        return False


def safetensors_metadata(path: str) -> Dict[str, str]:
    return read_safetensors_header(path)[0].get("__metadata__", {})


# ------------------------------------------------------------- "PYTORCH1" binary
_PTH_MAGIC = b"PYTORCH1"


def save_pth(tensors: Dict[str, torch.Tensor], path: str) -> None:
    os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
    with open(path, "wb") as f:
        f.write(_PTH_MAGIC)
        f.write(struct.pack("<I", len(tensors)))
        for name, t in tensors.items():
            nb = name.encode()
            arr = t.detach().float().cpu().contiguous().numpy().astype("<f4")
            f.write(struct.pack("<I", len(nb)) + nb + struct.pack("<I", arr.ndim))
            for d in arr.shape:
                f.write(struct.pack("<Q", d))
            raw = arr.tobytes()
            f.write(struct.pack("<Q", len(raw)) + raw)


def load_pth(path: str) -> Dict[str, torch.Tensor]:
    with open(path, "rb") as f:
        head = f.read(8)
        if head == _PTH_MAGIC:
            (n,) = struct.unpack("<I", f.read(4))
            out = {}
            for _ in range(n):
                (nl,) = struct.unpack("<I", f.read(4))
                name = f.read(nl).decode()
                (nd,) = struct.unpack("<I", f.read(4))
                shape = struct.unpack(f"<{nd}Q", f.read(8 * nd)) if nd else ()
                (nb,) = struct.unpack("<Q", f.read(8))
                out[name] = torch.from_numpy(np.frombuffer(f.read(nb), dtype="<f4").reshape(shape).copy())
            return out
    if head[:2] == b"PK" or head[:1] == b"\x80":          # torch zip archive / legacy pickle
        sd = torch.load(path, map_location="cpu", weights_only=True)
        if isinstance(sd, dict) and "state_dict" in sd and isinstance(sd["state_dict"], dict):
            sd = sd["state_dict"]
        return {k: v for k, v in sd.items() if isinstance(v, torch.Tensor)}
    raise ValueError(f"{path}: not a PYTORCH1 file, torch zip archive or pickle")


def save_torch_state_dict(module_or_dict, path: str) -> None:
    sd = module_or_dict.state_dict() if hasattr(module_or_dict, "state_dict") else module_or_dict
    torch.save({k: v.detach().cpu() for k, v in sd.items()}, path)


# ----------------------------------------------------------------- JSON state dict
def save_json_state_dict(tensors: Dict[str, torch.Tensor], path: str, metadata: Optional[dict] = None) -> None:
    doc = {"tensors": {k: {"shape": list(v.shape), "data": v.detach().double().reshape(-1).tolist(),
                           "dtype": str(v.dtype).replace("torch.", "")} for k, v in tensors.items()},
           "metadata": metadata or {}}
    with open(path, "w") as f:
        json.dump(doc, f)


def load_json_state_dict(path: str) -> Tuple[Dict[str, torch.Tensor], dict]:
    with open(path) as f:
        doc = json.load(f)
    out = {}
    for k, v in doc["tensors"].items():
        dt = getattr(torch, v.get("dtype", "float32"), torch.float32)
        out[k] = torch.tensor(v["data"], dtype=torch.float64).to(dt).reshape(v["shape"])
    return out, doc.get("metadata", {})


def map_pytorch_name(name: str) -> str:
    """PyTorch -> RusTorch parameter naming (src/formats/pytorch.rs:220-229): ``running_mean`` etc. stay,
    ``gamma`` / ``beta`` become ``weight`` / ``bias``."""
    return name.replace(".gamma", ".weight").replace(".beta", ".bias")


# --------------------------------------------------------------- HuggingFace dir
def save_huggingface(tensors: Dict[str, torch.Tensor], directory: str, config: Optional[dict] = None) -> None:
    os.makedirs(directory, exist_ok=True)
    save_safetensors(tensors, os.path.join(directory, "model.safetensors"), {"format": "pt"})
    with open(os.path.join(directory, "config.json"), "w") as f:
        json.dump(config or {}, f, indent=2)


def load_huggingface(directory: str, device: str = "cpu") -> Tuple[Dict[str, torch.Tensor], dict]:
    cfg = {}
    cp = os.path.join(directory, "config.json")
    if os.path.exists(cp):
        with open(cp) as f:
            cfg = json.load(f)
    tensors: Dict[str, torch.Tensor] = {}
    idx = os.path.join(directory, "model.safetensors.index.json")
    if os.path.exists(idx):                                # sharded checkpoint
        with open(idx) as f:
            shards = sorted(set(json.load(f)["weight_map"].values()))
        for s in shards:
            tensors.update(load_safetensors(os.path.join(directory, s), device))
    else:
        tensors = load_safetensors(os.path.join(directory, "model.safetensors"), device)
    return tensors, cfg


def detect_format(path: str) -> str:
    """``rustorch | gguf | safetensors | mlx | pth | torch | json | onnx | unknown`` from magic bytes / extension."""
    if os.path.isdir(path):
        return "huggingface" if os.path.exists(os.path.join(path, "config.json")) else "unknown"
    with open(path, "rb") as f:
        head = f.read(16)
    if head[:8] == b"RUSTORCH":
        return "rustorch"
    if head[:4] == b"GGUF":
        return "gguf"
    if head[:8] == _PTH_MAGIC:
        return "pth"
    if head[:2] == b"PK" or head[:1] == b"\x80":
        return "torch"
    ext = os.path.splitext(path)[1].lower()
    if ext == ".mlx":
        return "mlx"
    if ext == ".safetensors":
        return "safetensors"
    if ext == ".json":
        return "json"
    if ext == ".onnx":
        return "onnx"
    if len(head) >= 9 and head[8:9] == b"{":
        return "safetensors"
    return "unknown"
