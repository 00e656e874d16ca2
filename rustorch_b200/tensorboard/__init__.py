"""TensorBoard ``SummaryWriter`` that writes real TFRecord event files
(src/tensorboard/mod.rs:19-330, summary.rs:10-190, event_writer.rs:13-90).

The reference serialises events as JSON lines (event_writer.rs:37-82), which TensorBoard cannot read.  This
writer emits the ``tensorflow.Event`` protobuf wire format by hand (no protobuf dependency) framed as
TFRecords: ``u64 length · masked crc32c(length) · payload · masked crc32c(payload)``, so the files open in
stock TensorBoard.  ``read_events`` parses them back for tests and tooling.
"""
from __future__ import annotations

import os
import socket
import struct
import time
import zlib
from dataclasses import dataclass, field
from typing import Dict, Iterator, List, Optional, Sequence, Tuple

import numpy as np
import torch

# ----------------------------------------------------------------------------- crc32c (Castagnoli), table-driven
_CRC_TABLE = []
for _i in range(256):
    _c = _i
    for _ in range(8):
        _c = (_c >> 1) ^ 0x82F63B78 if _c & 1 else _c >> 1
    _CRC_TABLE.append(_c)


def crc32c(data: bytes) -> int:
    c = 0xFFFFFFFF
    for b in data:
        c = _CRC_TABLE[(c ^ b) & 0xFF] ^ (c >> 8)
    return c ^ 0xFFFFFFFF


def masked_crc32c(data: bytes) -> int:
    c = crc32c(data)
    return (((c >> 15) | (c << 17)) + 0xA282EAD8) & 0xFFFFFFFF


# ----------------------------------------------------------------------------- protobuf wire helpers
def _varint(n: int) -> bytes:
    out = bytearray()
    n &= (1 << 64) - 1
    while True:
        b = n & 0x7F
        n >>= 7
        if n:
            out.append(b | 0x80)
        else:
            out.append(b)
            return bytes(out)


def _key(fieldno: int, wt: int) -> bytes:
    return _varint((fieldno << 3) | wt)


def _f_varint(no: int, v: int) -> bytes:
    return _key(no, 0) + _varint(v)


def _f_double(no: int, v: float) -> bytes:
    return _key(no, 1) + struct.pack("<d", v)


def _f_float(no: int, v: float) -> bytes:
    return _key(no, 5) + struct.pack("<f", v)


def _f_bytes(no: int, b: bytes) -> bytes:
    return _key(no, 2) + _varint(len(b)) + b


def _f_packed_doubles(no: int, vs: Sequence[float]) -> bytes:
    return _f_bytes(no, struct.pack(f"<{len(vs)}d", *vs))


def _summary_value(tag: str, body: bytes, plugin: Optional[str] = None) -> bytes:
    v = _f_bytes(1, tag.encode())
    if plugin:                                   # SummaryMetadata{plugin_data{plugin_name}}
        v += _f_bytes(9, _f_bytes(1, _f_bytes(1, plugin.encode())))
    return _f_bytes(1, v + body)                 # Summary.value (repeated, field 1)


def _event(step: int, wall: float, summary: Optional[bytes] = None, file_version: Optional[str] = None,
           graph_def: Optional[bytes] = None) -> bytes:
    e = _f_double(1, wall) + _f_varint(2, step)
    if file_version is not None:
        e += _f_bytes(3, file_version.encode())
    if graph_def is not None:
        e += _f_bytes(4, graph_def)
    if summary is not None:
        e += _f_bytes(5, summary)
    return e


@dataclass
class ImageData:
    """``data``: HxWxC uint8 (C in 1, 3, 4)."""
    data: np.ndarray
    height: int = 0
    width: int = 0
    channels: int = 0

    def __post_init__(self):
        self.data = np.asarray(self.data, dtype=np.uint8)
        if self.data.ndim == 2:
            self.data = self.data[:, :, None]
        self.height, self.width, self.channels = self.data.shape


@dataclass
class NodeDef:
    name: str
    op: str
    inputs: List[str] = field(default_factory=list)
    attrs: Dict[str, str] = field(default_factory=dict)


@dataclass
class GraphDef:
    nodes: List[NodeDef] = field(default_factory=list)

    def serialize(self) -> bytes:
        out = b""
        for n in self.nodes:                      # GraphDef.node = 1; NodeDef{name=1, op=2, input=3}
            body = _f_bytes(1, n.name.encode()) + _f_bytes(2, n.op.encode())
            for i in n.inputs:
                body += _f_bytes(3, i.encode())
            out += _f_bytes(1, body)
        return out


def encode_png(img: np.ndarray) -> bytes:
    """Minimal PNG encoder (8-bit grey / grey+alpha / RGB / RGBA, filter 0, zlib)."""
    h, w, c = img.shape
    ctype = {1: 0, 2: 4, 3: 2, 4: 6}[c]
    raw = b"".join(b"\x00" + img[y].tobytes() for y in range(h))

    def chunk(tag: bytes, data: bytes) -> bytes:
        return struct.pack(">I", len(data)) + tag + data + struct.pack(">I", zlib.crc32(tag + data) & 0xFFFFFFFF)
    return (b"\x89PNG\r\n\x1a\n" + chunk(b"IHDR", struct.pack(">IIBBBBB", w, h, 8, ctype, 0, 0, 0))
            + chunk(b"IDAT", zlib.compress(raw, 6)) + chunk(b"IEND", b""))


class EventWriter:
    def __init__(self, log_dir: str, suffix: str = ""):
        os.makedirs(log_dir, exist_ok=True)
        self.path = os.path.join(log_dir, f"events.out.tfevents.{int(time.time())}.{socket.gethostname()}.{os.getpid()}{suffix}")
        self._f = open(self.path, "wb")
        self.write_event(_event(0, time.time(), file_version="brain.Event:2"))

    def write_event(self, payload: bytes) -> None:
        hdr = struct.pack("<Q", len(payload))
        self._f.write(hdr + struct.pack("<I", masked_crc32c(hdr)) + payload + struct.pack("<I", masked_crc32c(payload)))

    def write_summary(self, summary: bytes, step: int, wall: Optional[float] = None) -> None:
        self.write_event(_event(step, wall or time.time(), summary=summary))

    def flush(self) -> None:
        self._f.flush()

    def close(self) -> None:
        if not self._f.closed:
            self._f.flush()
            self._f.close()


class SummaryWriter:
    def __init__(self, log_dir: str = "runs/default", flush_every: int = 100):
        self.log_dir = log_dir
        self.writer = EventWriter(log_dir)
        self.global_step = 0
        self._pending, self._flush_every = 0, flush_every

    def _s(self, step: Optional[int]) -> int:
        return self.global_step if step is None else int(step)

    def _emit(self, summary: bytes, step: Optional[int]) -> None:
        self.writer.write_summary(summary, self._s(step))
        self._pending += 1
        if self._pending >= self._flush_every:
            self.flush()

    def add_scalar(self, tag: str, value, step: Optional[int] = None) -> None:
        self._emit(_summary_value(tag, _f_float(2, float(value))), step)

    def add_scalars(self, main_tag: str, values: Dict[str, float], step: Optional[int] = None) -> None:
        for k, v in values.items():
            self.add_scalar(f"{main_tag}/{k}", v, step)

    def add_histogram(self, tag: str, values, step: Optional[int] = None, bins: int = 30) -> None:
        v = torch.as_tensor(values).detach().double().reshape(-1).cpu().numpy()
        if v.size == 0:
            return
        counts, edges = np.histogram(v, bins=bins)
        histo = (_f_double(1, float(v.min())) + _f_double(2, float(v.max())) + _f_double(3, float(v.size))
                 + _f_double(4, float(v.sum())) + _f_double(5, float((v * v).sum()))
                 + _f_packed_doubles(6, edges[1:].tolist()) + _f_packed_doubles(7, counts.astype(float).tolist()))
        self._emit(_summary_value(tag, _f_bytes(5, histo)), step)

    def add_image(self, tag: str, image, step: Optional[int] = None) -> None:
        if not isinstance(image, ImageData):
            t = torch.as_tensor(image).detach().cpu()
            if t.is_floating_point():
                t = (t.clamp(0, 1) * 255).round().to(torch.uint8)
            if t.dim() == 3 and t.shape[0] in (1, 3, 4) and t.shape[2] not in (1, 3, 4):
                t = t.permute(1, 2, 0)                                   # CHW -> HWC
            image = ImageData(t.contiguous().numpy())
        img = (_f_varint(1, image.height) + _f_varint(2, image.width) + _f_varint(3, image.channels)
               + _f_bytes(4, encode_png(image.data)))
        self._emit(_summary_value(tag, _f_bytes(4, img)), step)

    def add_text(self, tag: str, text: str, step: Optional[int] = None) -> None:
        # TensorProto{dtype=DT_STRING(7), tensor_shape{dim{size=1}}, string_val}
        tensor = _f_varint(1, 7) + _f_bytes(2, _f_bytes(2, _f_varint(1, 1))) + _f_bytes(8, text.encode())
        self._emit(_summary_value(tag, _f_bytes(8, tensor), plugin="text"), step)

    def add_graph(self, graph) -> None:
        if isinstance(graph, torch.nn.Module):
            graph = graph_from_module(graph)
        self.writer.write_event(_event(0, time.time(), graph_def=graph.serialize()))

    def add_embedding(self, mat, metadata: Optional[Sequence[str]] = None, tag: str = "default", step: Optional[int] = None) -> str:
        """Writes ``tensors.tsv`` / ``metadata.tsv`` + ``projector_config.pbtxt`` (the projector plugin's layout)."""
        sub = os.path.join(self.log_dir, f"{self._s(step):05d}", tag)
        os.makedirs(sub, exist_ok=True)
        m = torch.as_tensor(mat).detach().float().cpu().numpy()
        np.savetxt(os.path.join(sub, "tensors.tsv"), m, delimiter="\t", fmt="%.6g")
        if metadata is not None:
            with open(os.path.join(sub, "metadata.tsv"), "w") as f:
                f.write("\n".join(str(x) for x in metadata) + "\n")
        rel = os.path.relpath(sub, self.log_dir)
        with open(os.path.join(self.log_dir, "projector_config.pbtxt"), "a") as f:
            f.write(f'embeddings {{\n  tensor_name: "{tag}:{self._s(step):05d}"\n  tensor_path: "{rel}/tensors.tsv"\n'
                    + (f'  metadata_path: "{rel}/metadata.tsv"\n' if metadata is not None else "") + "}\n")
        return sub

    def add_pr_curve(self, tag: str, labels, predictions, step: Optional[int] = None, num_thresholds: int = 127) -> None:
        y = torch.as_tensor(labels).bool().reshape(-1).cpu().numpy()
        p = torch.as_tensor(predictions).float().reshape(-1).cpu().numpy()
        th = np.linspace(0, 1, num_thresholds)
        tp = np.array([(p >= t)[y].sum() for t in th], dtype=np.float32)
        fp = np.array([(p >= t)[~y].sum() for t in th], dtype=np.float32)
        fn, tn = y.sum() - tp, (~y).sum() - fp
        prec = tp / np.maximum(tp + fp, 1e-7)
        rec = tp / np.maximum(tp + fn, 1e-7)
        data = np.stack([tp, fp, tn, fn, prec, rec]).astype("<f4")
        shape = _f_bytes(2, _f_varint(1, 6)) + _f_bytes(2, _f_varint(1, num_thresholds))
        tensor = _f_varint(1, 1) + _f_bytes(2, shape) + _f_bytes(4, data.tobytes())       # DT_FLOAT, tensor_content
        self._emit(_summary_value(tag, _f_bytes(8, tensor), plugin="pr_curves"), step)

    def add_audio(self, tag: str, audio, sample_rate: int = 44100, step: Optional[int] = None) -> None:
        a = torch.as_tensor(audio).detach().float().reshape(-1).clamp(-1, 1).cpu().numpy()
        pcm = (a * 32767).astype("<i2").tobytes()
        wav = (b"RIFF" + struct.pack("<I", 36 + len(pcm)) + b"WAVEfmt " + struct.pack("<IHHIIHH", 16, 1, 1, sample_rate, sample_rate * 2, 2, 16)
               + b"data" + struct.pack("<I", len(pcm)) + pcm)
        body = (_f_float(1, float(sample_rate)) + _f_varint(2, 1) + _f_varint(3, len(a)) + _f_bytes(4, wav) + _f_bytes(5, b"audio/wav"))
        self._emit(_summary_value(tag, _f_bytes(6, body)), step)

    def step(self) -> None:
        self.global_step += 1

    def flush(self) -> None:
        self.writer.flush()
        self._pending = 0

    def close(self) -> None:
        self.writer.close()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()
        return False


def graph_from_module(module: torch.nn.Module) -> GraphDef:
    g = GraphDef()
    prev = "input"
    g.nodes.append(NodeDef("input", "Placeholder"))
    for name, m in module.named_modules():
        if name and not list(m.children()):
            g.nodes.append(NodeDef(name.replace(".", "/"), type(m).__name__, [prev]))
            prev = name.replace(".", "/")
    return g


def create_writer(base_dir: Optional[str] = None) -> SummaryWriter:
    return SummaryWriter(os.path.join(base_dir or "runs", time.strftime("%Y%m%d-%H%M%S")))


def log_scalar(writer: SummaryWriter, tag: str, value: float) -> None:
    writer.add_scalar(tag, value)


# ----------------------------------------------------------------------------- reader
def _read_varint(b: bytes, i: int) -> Tuple[int, int]:
    n = s = 0
    while True:
        c = b[i]
        i += 1
        n |= (c & 0x7F) << s
        s += 7
        if not c & 0x80:
            return n, i


def parse_message(b: bytes) -> List[Tuple[int, int, object]]:
    """Flat decode of one protobuf message: ``[(field, wire_type, value)]`` (bytes for length-delimited)."""
    out, i = [], 0
    while i < len(b):
        k, i = _read_varint(b, i)
        no, wt = k >> 3, k & 7
        if wt == 0:
            v, i = _read_varint(b, i)
        elif wt == 1:
            v, i = struct.unpack_from("<d", b, i)[0], i + 8
        elif wt == 5:
            v, i = struct.unpack_from("<f", b, i)[0], i + 4
        elif wt == 2:
            n, i = _read_varint(b, i)
            v, i = b[i:i + n], i + n
        else:
            raise ValueError(f"unsupported wire type {wt}")
        out.append((no, wt, v))
    return out


def read_records(path: str) -> Iterator[bytes]:
    with open(path, "rb") as f:
        while True:
            hdr = f.read(8)
            if len(hdr) < 8:
                return
            (n,) = struct.unpack("<Q", hdr)
            (hcrc,) = struct.unpack("<I", f.read(4))
            if hcrc != masked_crc32c(hdr):
                raise ValueError("corrupt TFRecord length checksum")
            payload = f.read(n)
            (pcrc,) = struct.unpack("<I", f.read(4))
            if pcrc != masked_crc32c(payload):
                raise ValueError("corrupt TFRecord payload checksum")
            yield payload


def read_events(path: str) -> List[dict]:
    """``[{step, wall_time, file_version?, graph?, values: [{tag, simple_value?, kind}]}]``."""
    evs = []
    for rec in read_records(path):
        e: dict = {"step": 0, "values": []}
        for no, _, v in parse_message(rec):
            if no == 1:
                e["wall_time"] = v
            elif no == 2:
                e["step"] = v
            elif no == 3:
                e["file_version"] = v.decode()
            elif no == 4:
                e["graph"] = v
            elif no == 5:
                for sno, _, sv in parse_message(v):
                    if sno != 1:
                        continue
                    val: dict = {}
                    for fno, _, fv in parse_message(sv):
                        if fno == 1:
                            val["tag"] = fv.decode()
                        elif fno == 2:
                            val.update(kind="scalar", simple_value=fv)
                        elif fno == 4:
                            val.update(kind="image", image=fv)
                        elif fno == 5:
                            val.update(kind="histogram", histo=fv)
                        elif fno == 6:
                            val.update(kind="audio", audio=fv)
                        elif fno == 8:
                            val.update(kind="tensor", tensor=fv)
                    e["values"].append(val)
        evs.append(e)
    return evs
