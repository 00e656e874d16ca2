"""Reader / writer of RusTorch's native binary container, byte-compatible with the reference.

File = ``b"RUSTORCH"`` (8) · u64-LE header length · bincode ``FileHeader`` · payload
(src/serialization/model_io.rs:18-113).  ``FileHeader { magic: [u8; 8], version: String, object_type: String,
metadata: HashMap<String, String>, checksum: u64 }`` (src/serialization/core.rs:129-168) in bincode 1.x default
encoding: fixed array raw, strings and maps with u64-LE lengths, integers little endian.  ``checksum`` is CRC-64
with the reflected polynomial 0xC96C5795D7870F42, initial value and final XOR all-ones (core.rs:255-269) over
the payload.  Payloads:

* ``tensor``            u32 ndim · u64 dims[] · u64 byte_len · raw little-endian data (model_io.rs:796-929)
* ``state_dict``        u64 json_len · JSON ModelMetadata · u32 n · [u32 name_len · name · u64 len · tensor]* ·
                        u32 n_buffers · [...]* (model_io.rs:118-392)
* ``model_checkpoint``  u64 epoch · u64 step · u64 len · state_dict · optimizer_state map · scheduler_state map
                        (u32 n, [u32 klen · key · u64 vlen · bytes]) · metrics map (u32 n, [u32 klen · key · f64]) ·
                        u64 timestamp (model_io.rs:483-792)
* ``autograd.Variable`` u8 requires_grad · u64 len · tensor · u8 has_grad · [u64 len · tensor]
                        (src/autograd/mod.rs:508-658)

The element type is not stored in a tensor payload (the reference is generic over f32 / f64 and trusts the
caller); readers here take ``dtype`` (default f32) and fall back to f64 when the byte length says so.
"""
from __future__ import annotations

import json
import os
import struct
import time
from typing import Dict, Optional, Tuple

import numpy as np
import torch

MAGIC = b"RUSTORCH"
VERSION = "1.0.0"
_POLY = 0xC96C5795D7870F42
_MASK = 0xFFFFFFFFFFFFFFFF


def _make_table():
    t = []
    for b in range(256):
        c = b
        for _ in range(8):
            c = (c >> 1) ^ _POLY if c & 1 else c >> 1
        t.append(c)
    return t


_TABLE = _make_table()


def crc64(data: bytes) -> int:
    """CRC-64/XZ, bit-identical to the reference's ``compute_checksum``."""
    crc = _MASK
    tbl = _TABLE
    for b in data:
        crc = tbl[(crc ^ b) & 0xFF] ^ (crc >> 8)
    return crc ^ _MASK


def crc64_fast(data) -> int:
    """Same value through the native library's table-driven C++ loop when it is loadable (checkpoints are
    gigabytes; the Python loop above manages only a few MB/s), else the Python loop."""
    try:
        from .. import _native
        mod = _native.load(required=False)
        if mod is not None and hasattr(mod, "crc64"):
            return int(mod.crc64(bytes(data) if not isinstance(data, (bytes, bytearray)) else data))
    except Exception:  # noqa: BLE001
        pass
    return crc64(bytes(data))


# ------------------------------------------------------------------ bincode header
def _bstr(s: str) -> bytes:
    b = s.encode()
    return struct.pack("<Q", len(b)) + b


def encode_header(object_type: str, metadata: Dict[str, str], checksum: int) -> bytes:
    out = MAGIC + _bstr(VERSION) + _bstr(object_type) + struct.pack("<Q", len(metadata))
    for k, v in metadata.items():
        out += _bstr(k) + _bstr(str(v))
    return out + struct.pack("<Q", checksum)


def decode_header(b: bytes) -> Tuple[str, str, Dict[str, str], int]:
    if b[:8] != MAGIC:
        raise ValueError("Invalid file magic")
    off = 8

    def rstr():
        nonlocal off
        (n,) = struct.unpack_from("<Q", b, off)
        off += 8
        s = b[off:off + n].decode()
        off += n
        return s

    version, object_type = rstr(), rstr()
    (n,) = struct.unpack_from("<Q", b, off)
    off += 8
    meta = {}
    for _ in range(n):
        k = rstr()
        meta[k] = rstr()
    (checksum,) = struct.unpack_from("<Q", b, off)
    return version, object_type, meta, checksum


def write_container(path: str, object_type: str, metadata: Dict[str, str], payload: bytes) -> None:
    d = os.path.dirname(os.path.abspath(path))
    os.makedirs(d, exist_ok=True)
    header = encode_header(object_type, metadata, crc64_fast(payload))
    with open(path, "wb") as f:
        f.write(MAGIC)
        f.write(struct.pack("<Q", len(header)))
        f.write(header)
        f.write(payload)


def read_container(path: str, expected_type: Optional[str] = None) -> Tuple[str, Dict[str, str], bytes]:
    with open(path, "rb") as f:
        if f.read(8) != MAGIC:
            raise ValueError("Invalid RusTorch file format")
        (hlen,) = struct.unpack("<Q", f.read(8))
        version, object_type, meta, checksum = decode_header(f.read(hlen))
        payload = f.read()
    if not version.startswith("1."):
        raise ValueError(f"unsupported version {version} (expected 1.x)")
    if expected_type is not None and object_type != expected_type:
        raise TypeError(f"type mismatch: expected {expected_type}, found {object_type}")
    if crc64_fast(payload) != checksum:
        raise IOError("Checksum mismatch")
    return object_type, meta, payload


def is_rustorch_file(path: str) -> bool:
    try:
        with open(path, "rb") as f:
            return f.read(8) == MAGIC
    except OSError:
        return False


# ------------------------------------------------------------------------- tensors
_NP = {"f32": np.dtype("<f4"), "f64": np.dtype("<f8")}


def _rust_dtype(t: torch.Tensor) -> str:
    return "f64" if t.dtype == torch.float64 else "f32"


def encode_tensor(t: torch.Tensor) -> bytes:
    kind = _rust_dtype(t)
    arr = t.detach().to(torch.float64 if kind == "f64" else torch.float32).cpu().contiguous().numpy().astype(_NP[kind])
    raw = arr.tobytes()
    return struct.pack("<I", arr.ndim) + b"".join(struct.pack("<Q", d) for d in arr.shape) + struct.pack("<Q", len(raw)) + raw


def decode_tensor(b: bytes, off: int = 0, dtype: Optional[str] = None) -> Tuple[torch.Tensor, int]:
    (nd,) = struct.unpack_from("<I", b, off)
    off += 4
    shape = struct.unpack_from(f"<{nd}Q", b, off) if nd else ()
    off += 8 * nd
    (nbytes,) = struct.unpack_from("<Q", b, off)
    off += 8
    n = int(np.prod(shape)) if nd else 1
    kind = dtype or ("f64" if n and nbytes == 8 * n else "f32")
    arr = np.frombuffer(b, dtype=_NP[kind], count=nbytes // _NP[kind].itemsize, offset=off).reshape(shape)
    return torch.from_numpy(arr.copy()), off + nbytes


def save_tensor(t: torch.Tensor, path: str) -> None:
    meta = {"shape": str(list(t.shape)), "dtype": _rust_dtype(t), "device": "cpu", "numel": str(t.numel())}
    write_container(path, "tensor", meta, encode_tensor(t))


def load_tensor(path: str, dtype: Optional[str] = None) -> torch.Tensor:
    _, meta, payload = read_container(path, "tensor")
    return decode_tensor(payload, 0, dtype or meta.get("dtype"))[0]


# ---------------------------------------------------------------------- state dict
def _tensor_meta(t: torch.Tensor, offset: int, size: int) -> dict:
    return {"shape": list(t.shape), "dtype": _rust_dtype(t), "device": "cpu",
            "requires_grad": bool(t.requires_grad), "data_offset": offset, "data_size": size}


def encode_state_dict(params: Dict[str, torch.Tensor], buffers: Optional[Dict[str, torch.Tensor]] = None,
                      model_type: str = "model", config: Optional[Dict[str, str]] = None,
                      training_state: bool = False) -> bytes:
    buffers = buffers or {}
    blobs_p = {k: encode_tensor(v) for k, v in params.items()}
    blobs_b = {k: encode_tensor(v) for k, v in buffers.items()}
    off, pm, bm = 0, {}, {}
    for k, v in params.items():
        pm[k] = _tensor_meta(v, off, len(blobs_p[k]))
        off += len(blobs_p[k])
    for k, v in buffers.items():
        bm[k] = _tensor_meta(v, off, len(blobs_b[k]))
        off += len(blobs_b[k])
    meta = json.dumps({"model_type": model_type, "parameters": pm, "buffers": bm,
                       "config": {k: str(v) for k, v in (config or {}).items()},
                       "training_state": training_state}, separators=(",", ":")).encode()
    out = [struct.pack("<Q", len(meta)), meta]
    for blobs in (blobs_p, blobs_b):
        out.append(struct.pack("<I", len(blobs)))
        for k, blob in blobs.items():
            kb = k.encode()
            out += [struct.pack("<I", len(kb)), kb, struct.pack("<Q", len(blob)), blob]
    return b"".join(out)


def decode_state_dict(b: bytes, off: int = 0) -> Tuple[Dict[str, torch.Tensor], Dict[str, torch.Tensor], dict, int]:
    (mlen,) = struct.unpack_from("<Q", b, off)
    off += 8
    meta = json.loads(b[off:off + mlen].decode()) if mlen else {}
    off += mlen
    groups = []
    for which in ("parameters", "buffers"):
        (n,) = struct.unpack_from("<I", b, off)
        off += 4
        d = {}
        for _ in range(n):
            (kl,) = struct.unpack_from("<I", b, off)
            off += 4
            name = b[off:off + kl].decode()
            off += kl
            (tl,) = struct.unpack_from("<Q", b, off)
            off += 8
            dt = meta.get(which, {}).get(name, {}).get("dtype")
            d[name], _ = decode_tensor(b, off, dt if dt in _NP else None)
            off += tl
        groups.append(d)
    return groups[0], groups[1], meta, off


def save_state_dict(params: Dict[str, torch.Tensor], path: str, buffers: Optional[Dict[str, torch.Tensor]] = None,
                    model_type: str = "model", config: Optional[Dict[str, str]] = None, training_state: bool = False) -> None:
    payload = encode_state_dict(params, buffers, model_type, config, training_state)
    meta = {"model_type": model_type, "num_parameters": str(len(params)), "num_buffers": str(len(buffers or {})),
            "training_state": str(training_state).lower()}
    write_container(path, "state_dict", meta, payload)


def load_state_dict(path: str) -> Tuple[Dict[str, torch.Tensor], Dict[str, torch.Tensor], dict]:
    _, _, payload = read_container(path, "state_dict")
    p, b, meta, _ = decode_state_dict(payload)
    return p, b, meta


def save_module(module: torch.nn.Module, path: str, model_type: Optional[str] = None, config: Optional[dict] = None) -> None:
    params = {k: v.detach() for k, v in module.named_parameters()}
    buffers = {k: v.detach() for k, v in module.named_buffers()}
    save_state_dict(params, path, buffers, model_type or type(module).__name__, config, module.training)


def load_module(module: torch.nn.Module, path: str, strict: bool = True) -> dict:
    p, b, meta = load_state_dict(path)
    sd = {**p, **b}
    own = module.state_dict()
    # tensors the module has yet to create (layers built from their first input) pass through as stored; with
    # ``strict`` a name the module does not know is an error, not something to drop silently
    cast = {k: (v.to(own[k].dtype).reshape(own[k].shape) if k in own else v) for k, v in sd.items() if k in own or strict}
    module.load_state_dict(cast, strict=strict)
    return meta


# ---------------------------------------------------------------------- checkpoint
def _enc_map_bytes(m: Dict[str, bytes]) -> bytes:
    out = [struct.pack("<I", len(m))]
    for k, v in m.items():
        kb = k.encode()
        out += [struct.pack("<I", len(kb)), kb, struct.pack("<Q", len(v)), v]
    return b"".join(out)


def _dec_map_bytes(b: bytes, off: int) -> Tuple[Dict[str, bytes], int]:
    (n,) = struct.unpack_from("<I", b, off)
    off += 4
    m = {}
    for _ in range(n):
        (kl,) = struct.unpack_from("<I", b, off)
        off += 4
        k = b[off:off + kl].decode()
        off += kl
        (vl,) = struct.unpack_from("<Q", b, off)
        off += 8
        m[k] = b[off:off + vl]
        off += vl
    return m, off


def save_checkpoint(path: str, epoch: int, step: int, params: Dict[str, torch.Tensor],
                    buffers: Optional[Dict[str, torch.Tensor]] = None, optimizer_state: Optional[Dict[str, bytes]] = None,
                    scheduler_state: Optional[Dict[str, bytes]] = None, metrics: Optional[Dict[str, float]] = None,
                    model_type: str = "model", timestamp: Optional[int] = None) -> None:
    """``optimizer_state`` / ``scheduler_state`` values are opaque byte strings (e.g. an encoded tensor
    from :func:`encode_tensor` per moment buffer, or JSON)."""
    sd = encode_state_dict(params, buffers, model_type)
    metrics = metrics or {}
    out = [struct.pack("<QQQ", epoch, step, len(sd)), sd, _enc_map_bytes(optimizer_state or {}),
           _enc_map_bytes(scheduler_state or {}), struct.pack("<I", len(metrics))]
    for k, v in metrics.items():
        kb = k.encode()
        out += [struct.pack("<I", len(kb)), kb, struct.pack("<d", float(v))]
    out.append(struct.pack("<Q", int(time.time()) if timestamp is None else timestamp))
    meta = {"epoch": str(epoch), "step": str(step), "num_metrics": str(len(metrics))}
    write_container(path, "model_checkpoint", meta, b"".join(out))


def load_checkpoint(path: str) -> dict:
    _, _, b = read_container(path, "model_checkpoint")
    epoch, step, sdl = struct.unpack_from("<QQQ", b, 0)
    off = 24
    params, buffers, meta, _ = decode_state_dict(b, off)
    off += sdl
    opt, off = _dec_map_bytes(b, off)
    sch, off = _dec_map_bytes(b, off)
    (n,) = struct.unpack_from("<I", b, off)
    off += 4
    metrics = {}
    for _ in range(n):
        (kl,) = struct.unpack_from("<I", b, off)
        off += 4
        k = b[off:off + kl].decode()
        off += kl
        (metrics[k],) = struct.unpack_from("<d", b, off)
        off += 8
    (ts,) = struct.unpack_from("<Q", b, off)
    return {"epoch": epoch, "step": step, "parameters": params, "buffers": buffers, "metadata": meta,
            "optimizer_state": opt, "scheduler_state": sch, "metrics": metrics, "timestamp": ts}


# ------------------------------------------------------------------------ variable
def save_variable(t: torch.Tensor, path: str) -> None:
    data = encode_tensor(t.detach())
    out = [struct.pack("<B", int(t.requires_grad)), struct.pack("<Q", len(data)), data]
    if t.grad is not None:
        g = encode_tensor(t.grad)
        out += [struct.pack("<B", 1), struct.pack("<Q", len(g)), g]
    else:
        out.append(struct.pack("<B", 0))
    write_container(path, "autograd.Variable", {"requires_grad": str(t.requires_grad).lower()}, b"".join(out))


def load_variable(path: str) -> torch.Tensor:
    _, _, b = read_container(path, "autograd.Variable")
    rg = b[0] != 0
    (n,) = struct.unpack_from("<Q", b, 1)
    t, _ = decode_tensor(b, 9)
    off = 9 + n
    t.requires_grad_(rg)
    if b[off]:
        g, _ = decode_tensor(b, off + 9)
        t.grad = g
    return t
