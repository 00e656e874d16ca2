"""GGUF reader / writer and the Q4_0 / Q8_0 block codecs.

Container (v3): magic ``0x46554747`` ("GGUF"), u32 version, u64 tensor_count, u64 kv_count, key-value section
(value types 0-12 incl. arrays), tensor infos (name · u32 n_dims · u64 dims (innermost first) · u32 ggml type ·
u64 offset), then tensor data starting at the next multiple of ``general.alignment`` (default 32); a tensor's
bytes are at ``data_start + info.offset``.  Same constants as the reference parser
(example-cli/src/model/formats/gguf.rs:10-145,157-301), which stops at the metadata: its tensor loader seeks to
``info.offset`` without the data-section base and "dequantises" with a placeholder formula
(tensor_loader.rs:83-122).  Here the data is read (memory-mapped) and decoded for real.

Blocks of 32 weights:
* Q4_0 (18 B): f16 ``d`` + 16 bytes; weight j = ((qs[j] & 0xF) - 8) * d, weight j+16 = ((qs[j] >> 4) - 8) * d.
  Quantise: ``m`` = the value with the largest magnitude, ``d = m / -8``, ``q = min(15, floor(x/d + 8.5))``.
* Q8_0 (34 B): f16 ``d`` + 32 int8; ``x = q * d``, ``d = max|x| / 127``.
"""
from __future__ import annotations

import enum
import mmap
import os
import struct
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple

import numpy as np
import torch

GGUF_MAGIC = 0x46554747
GGUF_VERSION = 3
DEFAULT_ALIGNMENT = 32


class GGMLType(enum.IntEnum):
    """Tensor storage types of GGUF files with their block sizes (F32, F16, Q4_0, Q8_0, ...)."""

    F32 = 0
    F16 = 1
    Q4_0 = 2
    Q4_1 = 3
    Q5_0 = 6
    Q5_1 = 7
    Q8_0 = 8
    Q8_1 = 9
    Q2_K = 10
    Q3_K = 11
    Q4_K = 12
    Q5_K = 13
    Q6_K = 14
    Q8_K = 15
    I8 = 16
    I16 = 17
    I32 = 18
    BF16 = 30


# (block elements, block bytes)
_BLOCK = {GGMLType.F32: (1, 4), GGMLType.F16: (1, 2), GGMLType.BF16: (1, 2), GGMLType.Q4_0: (32, 18),
          GGMLType.Q4_1: (32, 20), GGMLType.Q5_0: (32, 22), GGMLType.Q5_1: (32, 24), GGMLType.Q8_0: (32, 34),
          GGMLType.Q8_1: (32, 36), GGMLType.I8: (1, 1), GGMLType.I16: (1, 2), GGMLType.I32: (1, 4),
          # K-quants: super-blocks of 256 weights
          GGMLType.Q2_K: (256, 84), GGMLType.Q3_K: (256, 110), GGMLType.Q4_K: (256, 144), GGMLType.Q5_K: (256, 176),
          GGMLType.Q6_K: (256, 210), GGMLType.Q8_K: (256, 292)}


class GGUFValueType(enum.IntEnum):
    """Type tags of GGUF metadata values."""

    UINT8 = 0
    INT8 = 1
    UINT16 = 2
    INT16 = 3
    UINT32 = 4
    INT32 = 5
    FLOAT32 = 6
    BOOL = 7
    STRING = 8
    ARRAY = 9
    UINT64 = 10
    INT64 = 11
    FLOAT64 = 12


_SCALAR = {0: "<B", 1: "<b", 2: "<H", 3: "<h", 4: "<I", 5: "<i", 6: "<f", 7: "<?", 10: "<Q", 11: "<q", 12: "<d"}


@dataclass
class GGUFTensorInfo:
    name: str
    dims: Tuple[int, ...]        # innermost first (ne[0] = in_features for a weight matrix)
    ggml_type: GGMLType
    offset: int                  # relative to the data section

    @property
    def shape(self) -> Tuple[int, ...]:
        """Row-major (torch) shape: reversed dims."""
        return tuple(reversed(self.dims))

    @property
    def numel(self) -> int:
        n = 1
        for d in self.dims:
            n *= d
        return n

    @property
    def nbytes(self) -> int:
        be, bb = _BLOCK[self.ggml_type]
        return self.numel // be * bb


# ---------------------------------------------------------------- block codecs
def quantize_q4_0(x: np.ndarray) -> np.ndarray:
    """fp32 ``[..., K]`` (K % 32 == 0) -> uint8 ``[..., K/32, 18]``."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    assert x.shape[-1] % 32 == 0, "last dim must be a multiple of 32"
    b = x.reshape(*x.shape[:-1], -1, 32)
    idx = np.abs(b).argmax(-1)[..., None]
    m = np.take_along_axis(b, idx, -1)
    d = (m / -8.0).astype(np.float32)
    dh = d.astype(np.float16)
    inv = np.where(d != 0, 1.0 / np.where(d != 0, d, 1), 0.0).astype(np.float32)
    q = np.minimum(15, np.floor(b * inv + 8.5)).astype(np.int32).clip(0, 15).astype(np.uint8)
    qs = (q[..., :16] | (q[..., 16:] << 4)).astype(np.uint8)
    out = np.empty((*b.shape[:-1], 18), dtype=np.uint8)
    out[..., :2] = dh.view(np.uint8).reshape(*b.shape[:-1], 2)
    out[..., 2:] = qs
    return out


def dequantize_q4_0(blocks: np.ndarray) -> np.ndarray:
    """uint8 ``[..., nb, 18]`` -> fp32 ``[..., nb*32]``."""
    blocks = np.ascontiguousarray(blocks, dtype=np.uint8)
    d = blocks[..., :2].copy().view(np.float16).astype(np.float32)          # [..., nb, 1]
    qs = blocks[..., 2:]
    lo = (qs & 0x0F).astype(np.int8) - 8
    hi = (qs >> 4).astype(np.int8) - 8
    w = np.concatenate([lo, hi], -1).astype(np.float32) * d
    return w.reshape(*blocks.shape[:-2], -1)


def quantize_q8_0(x: np.ndarray) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    assert x.shape[-1] % 32 == 0
    b = x.reshape(*x.shape[:-1], -1, 32)
    d = (np.abs(b).max(-1, keepdims=True) / 127.0).astype(np.float32)
    inv = np.where(d != 0, 1.0 / np.where(d != 0, d, 1), 0.0)
    q = np.rint(b * inv).clip(-127, 127).astype(np.int8)
    out = np.empty((*b.shape[:-1], 34), dtype=np.uint8)
    out[..., :2] = d.astype(np.float16).view(np.uint8).reshape(*b.shape[:-1], 2)
    out[..., 2:] = q.view(np.uint8)
    return out


def dequantize_q8_0(blocks: np.ndarray) -> np.ndarray:
    blocks = np.ascontiguousarray(blocks, dtype=np.uint8)
    d = blocks[..., :2].copy().view(np.float16).astype(np.float32)
    q = blocks[..., 2:].view(np.int8).astype(np.float32)
    return (q * d).reshape(*blocks.shape[:-2], -1)


# Decoders of the other GGML block types.  They only ever run at load time (a tensor in one of these types is expanded
# and, for the runtime's linears, re-encoded as Q8_0, which holds 4- to 6-bit sources without visible loss), so they are
# NumPy: every function takes ``uint8 [nb, block_bytes]`` and returns ``fp32 [nb, block_elements]``.
def _f16(col: np.ndarray) -> np.ndarray:
    """Two byte columns -> fp32 ``[nb, 1]``."""
    return np.ascontiguousarray(col).view(np.float16).astype(np.float32).reshape(-1, 1)


def _nibbles(qs: np.ndarray) -> np.ndarray:
    """``[nb, n]`` bytes -> ``[nb, 2n]``: all low nibbles, then all high nibbles (the 32-weight block layout)."""
    return np.concatenate([qs & 0x0F, qs >> 4], -1)


def _high_bits(qh: np.ndarray) -> np.ndarray:
    """Four bytes (little-endian u32) -> ``[nb, 32]`` bits, bit ``i`` for weight ``i``."""
    word = np.ascontiguousarray(qh).view("<u4").reshape(-1, 1)
    return ((word >> np.arange(32, dtype=np.uint32)) & 1).astype(np.uint8)


def dequantize_q4_1(b: np.ndarray) -> np.ndarray:
    return _nibbles(b[:, 4:20]).astype(np.float32) * _f16(b[:, 0:2]) + _f16(b[:, 2:4])


def dequantize_q5_0(b: np.ndarray) -> np.ndarray:
    q = (_nibbles(b[:, 6:22]) | (_high_bits(b[:, 2:6]) << 4)).astype(np.int16) - 16
    return q.astype(np.float32) * _f16(b[:, 0:2])


def dequantize_q5_1(b: np.ndarray) -> np.ndarray:
    q = _nibbles(b[:, 8:24]) | (_high_bits(b[:, 4:8]) << 4)
    return q.astype(np.float32) * _f16(b[:, 0:2]) + _f16(b[:, 2:4])


def dequantize_q8_1(b: np.ndarray) -> np.ndarray:
    return np.ascontiguousarray(b[:, 4:36]).view(np.int8).astype(np.float32) * _f16(b[:, 0:2])


def _per16(v: np.ndarray) -> np.ndarray:
    """``[nb, 16]`` values, one per run of 16 weights -> ``[nb, 256]``."""
    return np.repeat(v, 16, axis=-1)


def _two_bit_planes(qs: np.ndarray) -> np.ndarray:
    """``[nb, 64]`` bytes of 2-bit codes -> ``[nb, 256]``: per 32-byte half, shifts 0, 2, 4, 6 in turn over its 32 bytes."""
    q = qs.reshape(-1, 2, 1, 32)
    sh = np.array([0, 2, 4, 6], dtype=np.uint8).reshape(1, 1, 4, 1)
    return ((q >> sh) & 3).reshape(-1, 256)


def dequantize_q2_k(b: np.ndarray) -> np.ndarray:
    sc = b[:, 0:16]
    d, dmin = _f16(b[:, 80:82]), _f16(b[:, 82:84])
    return d * _per16((sc & 0x0F).astype(np.float32)) * _two_bit_planes(b[:, 16:80]).astype(np.float32) - dmin * _per16((sc >> 4).astype(np.float32))


def _q3k_scales(raw: np.ndarray) -> np.ndarray:
    """12 bytes -> sixteen 6-bit scales (still biased by 32): low 4 bits from the first 8 bytes, high 2 bits from the last 4."""
    a = np.ascontiguousarray(raw).view("<u4").reshape(-1, 3).astype(np.uint32)
    k1, k2 = np.uint32(0x03030303), np.uint32(0x0F0F0F0F)
    a0, a1, t = a[:, 0], a[:, 1], a[:, 2]
    out = np.stack([(a0 & k2) | ((t & k1) << 4), (a1 & k2) | (((t >> 2) & k1) << 4),
                    ((a0 >> 4) & k2) | (((t >> 4) & k1) << 4), ((a1 >> 4) & k2) | (((t >> 6) & k1) << 4)], -1).astype("<u4")
    return np.ascontiguousarray(out).view(np.uint8).reshape(-1, 16)


def dequantize_q3_k(b: np.ndarray) -> np.ndarray:
    hm, d = b[:, 0:32], _f16(b[:, 108:110])
    low = _two_bit_planes(b[:, 32:96]).astype(np.int16)                      # order: half, shift, byte
    bit = np.arange(8, dtype=np.uint8).reshape(1, 8, 1)                         # plane (half * 4 + shift) tests bit of that index
    high = ((hm.reshape(-1, 1, 32) >> bit) & 1).reshape(-1, 256).astype(np.int16)
    q = low - 4 * (1 - high)
    sc = _q3k_scales(b[:, 96:108]).astype(np.int16) - 32
    return d * _per16(sc.astype(np.float32)) * q.astype(np.float32)


def _k4_scales(raw: np.ndarray):
    """12 bytes -> eight 6-bit scales and eight 6-bit minima of a Q4_K / Q5_K super-block."""
    q = raw.astype(np.uint8)
    sc = np.concatenate([q[:, 0:4] & 63, (q[:, 8:12] & 0x0F) | ((q[:, 0:4] >> 6) << 4)], -1)
    mn = np.concatenate([q[:, 4:8] & 63, (q[:, 8:12] >> 4) | ((q[:, 4:8] >> 6) << 4)], -1)
    return sc.astype(np.float32), mn.astype(np.float32)


def _per32(v: np.ndarray) -> np.ndarray:
    return np.repeat(v, 32, axis=-1)


def _k4_codes(qs: np.ndarray) -> np.ndarray:
    """``[nb, 128]`` bytes -> ``[nb, 256]``: per 32-byte chunk its low nibbles, then its high nibbles."""
    q = qs.reshape(-1, 4, 1, 32)
    return np.concatenate([q & 0x0F, q >> 4], 2).reshape(-1, 256)


def dequantize_q4_k(b: np.ndarray) -> np.ndarray:
    sc, mn = _k4_scales(b[:, 4:16])
    return _f16(b[:, 0:2]) * _per32(sc) * _k4_codes(b[:, 16:144]).astype(np.float32) - _f16(b[:, 2:4]) * _per32(mn)


def dequantize_q5_k(b: np.ndarray) -> np.ndarray:
    sc, mn = _k4_scales(b[:, 4:16])
    bit = np.arange(8, dtype=np.uint8).reshape(1, 8, 1)                         # run r of 32 weights takes bit r of qh
    high = ((b[:, 16:48].reshape(-1, 1, 32) >> bit) & 1).reshape(-1, 256)
    q = _k4_codes(b[:, 48:176]) | (high.astype(np.uint8) << 4)
    return _f16(b[:, 0:2]) * _per32(sc) * q.astype(np.float32) - _f16(b[:, 2:4]) * _per32(mn)


def dequantize_q6_k(b: np.ndarray) -> np.ndarray:
    ql = b[:, 0:128].reshape(-1, 2, 2, 32)                                      # half, which 32-byte row, byte
    qh = b[:, 128:192].reshape(-1, 2, 1, 32)
    low = np.concatenate([ql & 0x0F, ql >> 4], 2)                               # [nb, 2, 4, 32]: rows lo(0..31), lo(32..63), hi(0..31), hi(32..63)
    sh = np.array([0, 2, 4, 6], dtype=np.uint8).reshape(1, 1, 4, 1)
    q = (low | (((qh >> sh) & 3) << 4)).astype(np.int16) - 32
    sc = np.ascontiguousarray(b[:, 192:208]).view(np.int8).astype(np.float32)  # one per 16 weights, in output order
    return _f16(b[:, 208:210]) * _per16(sc) * q.reshape(-1, 256).astype(np.float32)


def dequantize_q8_k(b: np.ndarray) -> np.ndarray:
    d = np.ascontiguousarray(b[:, 0:4]).view("<f4").reshape(-1, 1)
    return np.ascontiguousarray(b[:, 4:260]).view(np.int8).astype(np.float32) * d


_DECODERS = {GGMLType.Q4_1: dequantize_q4_1, GGMLType.Q5_0: dequantize_q5_0, GGMLType.Q5_1: dequantize_q5_1, GGMLType.Q8_1: dequantize_q8_1,
             GGMLType.Q2_K: dequantize_q2_k, GGMLType.Q3_K: dequantize_q3_k, GGMLType.Q4_K: dequantize_q4_k, GGMLType.Q5_K: dequantize_q5_k,
             GGMLType.Q6_K: dequantize_q6_k, GGMLType.Q8_K: dequantize_q8_k}


def dequantize(raw: np.ndarray, ggml_type: GGMLType, shape: Tuple[int, ...]) -> np.ndarray:
    t = GGMLType(ggml_type)
    if t is GGMLType.F32:
        return raw.view(np.float32).reshape(shape)
    if t is GGMLType.F16:
        return raw.view(np.float16).astype(np.float32).reshape(shape)
    if t is GGMLType.BF16:
        return (raw.view(np.uint16).astype(np.uint32) << 16).view(np.float32).reshape(shape)
    if t is GGMLType.Q4_0:
        return dequantize_q4_0(raw.reshape(-1, 18)).reshape(shape)
    if t is GGMLType.Q8_0:
        return dequantize_q8_0(raw.reshape(-1, 34)).reshape(shape)
    if t in (GGMLType.I8, GGMLType.I16, GGMLType.I32):
        return raw.view({GGMLType.I8: np.int8, GGMLType.I16: np.int16, GGMLType.I32: np.int32}[t]).reshape(shape)
    if t in _DECODERS:
        return _DECODERS[t](np.ascontiguousarray(raw, dtype=np.uint8).reshape(-1, _BLOCK[t][1])).reshape(shape)
    raise NotImplementedError(f"dequantisation of {t.name} is not implemented")


# ------------------------------------------------------------------------ reader
class GGUFFile:
    def __init__(self, path: str):
        self.path = path
        self.metadata: Dict[str, Any] = {}
        self.tensors: Dict[str, GGUFTensorInfo] = {}
        self._f = open(path, "rb")
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)
        self._off = 0
        self._parse()

    # primitive readers
    def _rd(self, fmt: str):
        v = struct.unpack_from(fmt, self._mm, self._off)
        self._off += struct.calcsize(fmt)
        return v[0]

    def _rstr(self) -> str:
        n = self._rd("<Q")
        s = self._mm[self._off:self._off + n].decode("utf-8", "replace")
        self._off += n
        return s

    def _rval(self, t: int):
        if t in _SCALAR:
            return self._rd(_SCALAR[t])
        if t == GGUFValueType.STRING:
            return self._rstr()
        if t == GGUFValueType.ARRAY:
            et = self._rd("<I")
            n = self._rd("<Q")
            if et in _SCALAR and et != GGUFValueType.BOOL:
                fmt = _SCALAR[et][1]
                arr = np.frombuffer(self._mm, dtype=np.dtype("<" + fmt), count=n, offset=self._off)
                self._off += arr.nbytes
                return arr.tolist()
            return [self._rval(et) for _ in range(n)]
        raise ValueError(f"unknown GGUF value type {t}")

    def _parse(self) -> None:
        magic = self._rd("<I")
        if magic != GGUF_MAGIC:
            raise ValueError(f"{self.path}: not a GGUF file (magic {magic:#x})")
        self.version = self._rd("<I")
        if self.version not in (2, 3):
            raise ValueError(f"unsupported GGUF version {self.version}")
        n_tensors, n_kv = self._rd("<Q"), self._rd("<Q")
        for _ in range(n_kv):
            k = self._rstr()
            self.metadata[k] = self._rval(self._rd("<I"))
        for _ in range(n_tensors):
            name = self._rstr()
            nd = self._rd("<I")
            dims = tuple(self._rd("<Q") for _ in range(nd))
            ty = GGMLType(self._rd("<I"))
            off = self._rd("<Q")
            self.tensors[name] = GGUFTensorInfo(name, dims, ty, off)
        self.alignment = int(self.metadata.get("general.alignment", DEFAULT_ALIGNMENT))
        self.data_start = -(-self._off // self.alignment) * self.alignment

    # tensor access
    def raw(self, name: str) -> np.ndarray:
        """The tensor's bytes as a read-only uint8 view of the mapped file."""
        info = self.tensors[name]
        return np.frombuffer(self._mm, dtype=np.uint8, count=info.nbytes, offset=self.data_start + info.offset)

    def load_tensor(self, name: str, dtype: torch.dtype = torch.float32) -> torch.Tensor:
        info = self.tensors[name]
        return torch.from_numpy(np.array(dequantize(self.raw(name), info.ggml_type, info.shape), copy=True)).to(dtype)

    def load_quantized(self, name: str) -> Tuple[torch.Tensor, GGUFTensorInfo]:
        """Block bytes ``[rows, K/32, block_bytes]`` (uint8) for Q4_0 / Q8_0 weights, kept quantised for the
        dequant-fused kernels."""
        info = self.tensors[name]
        be, bb = _BLOCK[info.ggml_type]
        rows = info.numel // info.dims[0]
        arr = self.raw(name).reshape(rows, info.dims[0] // be, bb)
        return torch.from_numpy(arr.copy()), info

    def architecture(self) -> str:
        return str(self.metadata.get("general.architecture", "llama"))

    def model_config(self) -> Dict[str, Any]:
        """The Llama-family hyper-parameters under their conventional GGUF keys."""
        a, m = self.architecture(), self.metadata
        g = lambda k, d=None: m.get(f"{a}.{k}", d)  # noqa: E731
        n_head = g("attention.head_count", 32)
        return {"architecture": a, "n_layer": g("block_count"), "n_embd": g("embedding_length"),
                "n_ff": g("feed_forward_length"), "n_head": n_head, "n_head_kv": g("attention.head_count_kv", n_head),
                "rope_theta": g("rope.freq_base", 10000.0), "rms_eps": g("attention.layer_norm_rms_epsilon", 1e-5),
                "context_length": g("context_length", 2048),
                "vocab_size": m.get(f"{a}.vocab_size") or (len(m["tokenizer.ggml.tokens"]) if "tokenizer.ggml.tokens" in m
                                                          else (self.tensors["token_embd.weight"].dims[1] if "token_embd.weight" in self.tensors else None))}

    def close(self) -> None:
        try:
            self._mm.close()
        except BufferError:      # a caller still holds a view from raw(); the mapping goes with it
            pass
        self._f.close()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()
        return False


# ------------------------------------------------------------------------ writer
def _wstr(s: str) -> bytes:
    b = s.encode()
    return struct.pack("<Q", len(b)) + b


def _wval(v) -> bytes:
    if isinstance(v, bool):
        return struct.pack("<I?", GGUFValueType.BOOL, v)
    if isinstance(v, int):
        return struct.pack("<Iq", GGUFValueType.INT64, v) if v < 0 or v >= 2 ** 32 else struct.pack("<II", GGUFValueType.UINT32, v)
    if isinstance(v, float):
        return struct.pack("<If", GGUFValueType.FLOAT32, v)
    if isinstance(v, str):
        return struct.pack("<I", GGUFValueType.STRING) + _wstr(v)
    if isinstance(v, (list, tuple)):
        if all(isinstance(x, str) for x in v):
            return struct.pack("<IIQ", GGUFValueType.ARRAY, GGUFValueType.STRING, len(v)) + b"".join(_wstr(x) for x in v)
        if all(isinstance(x, int) and not isinstance(x, bool) for x in v):
            return struct.pack("<IIQ", GGUFValueType.ARRAY, GGUFValueType.INT32, len(v)) + np.asarray(v, "<i4").tobytes()
        return struct.pack("<IIQ", GGUFValueType.ARRAY, GGUFValueType.FLOAT32, len(v)) + np.asarray(v, "<f4").tobytes()
    raise TypeError(f"cannot store {type(v)} in GGUF metadata")


@dataclass
class RawTensor:
    """Blocks that are encoded already (any GGML type): ``shape`` in torch layout ``[out, in]`` and the block bytes in
    row-major order.  ``write_gguf`` stores them as they are."""
    shape: Tuple[int, ...]
    data: bytes

    def check(self, ggml_type: GGMLType) -> None:
        be, bb = _BLOCK[GGMLType(ggml_type)]
        n = int(np.prod(self.shape))
        if self.shape[-1] % be or len(self.data) != n // be * bb:
            raise ValueError(f"{len(self.data)} bytes do not hold a {tuple(self.shape)} tensor of {GGMLType(ggml_type).name} blocks")


def encode_tensor(t, ggml_type: GGMLType) -> bytes:
    ty = GGMLType(ggml_type)
    if isinstance(t, RawTensor):
        t.check(ty)
        return bytes(t.data)
    x = t.detach().float().cpu().numpy()
    if ty is GGMLType.F32:
        return x.astype("<f4").tobytes()
    if ty is GGMLType.F16:
        return x.astype("<f2").tobytes()
    if ty is GGMLType.Q4_0:
        return quantize_q4_0(x).tobytes()
    if ty is GGMLType.Q8_0:
        return quantize_q8_0(x).tobytes()
    raise NotImplementedError(f"encoding {ty.name} is not implemented: pass blocks that are encoded already as a RawTensor")


def write_gguf(path: str, metadata: Dict[str, Any], tensors: Dict[str, Tuple[torch.Tensor, GGMLType]],
               alignment: int = DEFAULT_ALIGNMENT) -> None:
    """``tensors[name] = (tensor in torch layout [out, in], ggml type)``; the tensor may be a :class:`RawTensor`."""
    md = dict(metadata)
    md.setdefault("general.alignment", alignment)
    head = struct.pack("<IIQQ", GGUF_MAGIC, GGUF_VERSION, len(tensors), len(md))
    kv = b"".join(_wstr(k) + _wval(v) for k, v in md.items())
    infos, blobs, off = [], [], 0
    for name, (t, ty) in tensors.items():
        blob = encode_tensor(t, ty)
        dims = tuple(reversed(t.shape))
        infos.append(_wstr(name) + struct.pack("<I", len(dims)) + b"".join(struct.pack("<Q", d) for d in dims)
                     + struct.pack("<IQ", int(ty), off))
        pad = (-len(blob)) % alignment
        blobs.append(blob + b"\0" * pad)
        off += len(blob) + pad
    pre = head + kv + b"".join(infos)
    pre += b"\0" * ((-len(pre)) % alignment)
    os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
    with open(path, "wb") as f:
        f.write(pre)
        for b in blobs:
            f.write(b)
