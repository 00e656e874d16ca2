"""Model import: format detection / compatibility, importers for PyTorch (zip / pickle / PYTORCH1), safetensors,
RusTorch, GGUF and ONNX files, and conversion of an imported model into a runnable module
(src/model_import/mod.rs:25-330, formats.rs:8-420, pytorch.rs:153-565, onnx.rs:162-448).

The ONNX importer parses the protobuf wire format directly (graph nodes, initialisers with raw or typed data)
and can execute the common feed-forward subset (Gemm / MatMul / Add / Relu / Sigmoid / Tanh / Softmax /
Flatten / Reshape / Conv / BatchNormalization / MaxPool / GlobalAveragePool) with torch ops on any device;
the reference delegates execution to the ``ort`` crate (src/formats/onnx.rs:50-231).
"""
from __future__ import annotations

import os
import struct
from dataclasses import dataclass, field
from enum import Enum
from typing import Callable, Dict, List, Optional, Tuple

import numpy as np
import torch
import torch.nn as nn
import torch.nn.functional as F

from ..formats import gguf as gguf_fmt
from ..formats import safetensors as st
from ..tensorboard import parse_message


class ModelFormat(Enum):
    PYTORCH = "pytorch"
    ONNX = "onnx"
    SAFETENSORS = "safetensors"
    RUSTORCH = "rustorch"
    GGUF = "gguf"
    TENSORFLOW = "tensorflow"
    HUGGINGFACE = "huggingface"

    @classmethod
    def from_extension(cls, ext: str) -> Optional["ModelFormat"]:
        return {"pt": cls.PYTORCH, "pth": cls.PYTORCH, "bin": cls.PYTORCH, "onnx": cls.ONNX, "safetensors": cls.SAFETENSORS,
                "rustorch": cls.RUSTORCH, "rtch": cls.RUSTORCH, "gguf": cls.GGUF, "pb": cls.TENSORFLOW}.get(ext.lower().lstrip("."))

    def extensions(self) -> List[str]:
        return {"pytorch": ["pt", "pth", "bin"], "onnx": ["onnx"], "safetensors": ["safetensors"], "rustorch": ["rustorch", "rtch"],
                "gguf": ["gguf"], "tensorflow": ["pb"], "huggingface": []}[self.value]

    def supports_feature(self, f: "FormatFeature") -> bool:
        table = {
            "pytorch": {FormatFeature.WEIGHTS, FormatFeature.OPTIMIZER_STATE, FormatFeature.METADATA},
            "onnx": {FormatFeature.WEIGHTS, FormatFeature.GRAPH, FormatFeature.METADATA},
            "safetensors": {FormatFeature.WEIGHTS, FormatFeature.METADATA, FormatFeature.MEMORY_MAPPING},
            "rustorch": {FormatFeature.WEIGHTS, FormatFeature.OPTIMIZER_STATE, FormatFeature.METADATA, FormatFeature.CHECKSUM},
            "gguf": {FormatFeature.WEIGHTS, FormatFeature.METADATA, FormatFeature.QUANTIZATION, FormatFeature.MEMORY_MAPPING},
            "tensorflow": {FormatFeature.WEIGHTS, FormatFeature.GRAPH},
            "huggingface": {FormatFeature.WEIGHTS, FormatFeature.METADATA, FormatFeature.MEMORY_MAPPING},
        }
        return f in table[self.value]

    def description(self) -> str:
        return {"pytorch": "PyTorch checkpoint (zip archive, legacy pickle or PYTORCH1 binary)", "onnx": "ONNX protobuf graph",
                "safetensors": "safetensors (JSON header + raw tensors)", "rustorch": "RusTorch binary container (CRC-64 checked)",
                "gguf": "GGUF (llama.cpp) with quantised blocks", "tensorflow": "TensorFlow frozen graph",
                "huggingface": "HuggingFace directory (config.json + model.safetensors)"}[self.value]


class FormatFeature(Enum):
    """Capabilities a model file format may have (metadata, quantisation, streaming ...)."""

    WEIGHTS = "weights"
    GRAPH = "graph"
    OPTIMIZER_STATE = "optimizer_state"
    METADATA = "metadata"
    QUANTIZATION = "quantization"
    MEMORY_MAPPING = "memory_mapping"
    CHECKSUM = "checksum"


class CompressionType(Enum):
    """Compression of an exported model file (src/model_import/formats.rs)."""

    NONE = "none"
    GZIP = "gzip"
    ZSTD = "zstd"


class DeploymentTarget(Enum):
    """Where an exported model is meant to run."""

    SERVER = "server"
    MOBILE = "mobile"
    EDGE = "edge"
    WEB = "web"


class FormatCompatibility:
    """Conversion matrix: 1.0 lossless, 0 impossible; paths go through safetensors when no direct edge exists."""

    def __init__(self):
        F_ = ModelFormat
        w = [F_.PYTORCH, F_.SAFETENSORS, F_.RUSTORCH, F_.HUGGINGFACE]
        self.matrix: Dict[Tuple[ModelFormat, ModelFormat], float] = {(a, b): 1.0 for a in w for b in w}
        self.matrix.update({(F_.GGUF, b): 0.9 for b in w})            # dequantised on the way
        self.matrix.update({(a, F_.GGUF): 0.8 for a in w})            # quantised on the way
        self.matrix.update({(F_.ONNX, b): 0.7 for b in w})            # weights only; graph is re-created
        self.matrix[(F_.GGUF, F_.GGUF)] = self.matrix[(F_.ONNX, F_.ONNX)] = 1.0

    def get_compatibility(self, a: ModelFormat, b: ModelFormat) -> float:
        return self.matrix.get((a, b), 0.0)

    def get_conversion_path(self, a: ModelFormat, b: ModelFormat) -> List[ModelFormat]:
        if self.get_compatibility(a, b) > 0:
            return [a, b] if a != b else [a]
        mid = ModelFormat.SAFETENSORS
        if self.get_compatibility(a, mid) > 0 and self.get_compatibility(mid, b) > 0:
            return [a, mid, b]
        return []


@dataclass
class OptimizationProfile:
    target: DeploymentTarget
    dtype: torch.dtype
    quantize: Optional[str]
    max_batch: int

    @staticmethod
    def server() -> "OptimizationProfile":
        return OptimizationProfile(DeploymentTarget.SERVER, torch.bfloat16, None, 256)

    @staticmethod
    def mobile() -> "OptimizationProfile":
        return OptimizationProfile(DeploymentTarget.MOBILE, torch.float16, "int8", 1)

    @staticmethod
    def edge() -> "OptimizationProfile":
        return OptimizationProfile(DeploymentTarget.EDGE, torch.float16, "int4", 1)

    @staticmethod
    def web() -> "OptimizationProfile":
        return OptimizationProfile(DeploymentTarget.WEB, torch.float32, "int8", 1)


class FormatValidator:
    @staticmethod
    def get_format_confidence(data: bytes) -> Dict[ModelFormat, float]:
        c: Dict[ModelFormat, float] = {}
        if data[:8] == b"RUSTORCH":
            c[ModelFormat.RUSTORCH] = 1.0
        if data[:4] == b"GGUF":
            c[ModelFormat.GGUF] = 1.0
        if data[:2] == b"PK" or data[:8] == b"PYTORCH1":
            c[ModelFormat.PYTORCH] = 0.95
        elif data[:1] == b"\x80":
            c[ModelFormat.PYTORCH] = 0.7
        if len(data) > 9 and data[8:9] == b"{" and struct.unpack("<Q", data[:8])[0] < (100 << 20):
            c[ModelFormat.SAFETENSORS] = 0.9
        if data[:1] == b"\x08" and len(data) > 2:          # ModelProto.ir_version (field 1, varint)
            c[ModelFormat.ONNX] = 0.6
        return c

    @staticmethod
    def validate_format(data: bytes, expected: ModelFormat) -> bool:
        return FormatValidator.get_format_confidence(data).get(expected, 0.0) >= 0.5


# ------------------------------------------------------------------------------ imported model
@dataclass
class TensorSpec:
    name: str
    shape: Tuple[int, ...]
    dtype: str


@dataclass
class LayerInfo:
    name: str
    layer_type: str
    inputs: List[str] = field(default_factory=list)
    outputs: List[str] = field(default_factory=list)
    attributes: Dict[str, object] = field(default_factory=dict)


@dataclass
class ModelMetadata:
    name: str
    format: ModelFormat
    version: str = ""
    producer: str = ""
    extra: Dict[str, object] = field(default_factory=dict)


@dataclass
class ModelArchitecture:
    inputs: List[TensorSpec] = field(default_factory=list)
    outputs: List[TensorSpec] = field(default_factory=list)
    parameter_count: int = 0


@dataclass
class ImportedModel:
    metadata: ModelMetadata
    weights: Dict[str, torch.Tensor]
    layers: List[LayerInfo] = field(default_factory=list)
    architecture: ModelArchitecture = field(default_factory=ModelArchitecture)

    def state_dict(self) -> Dict[str, torch.Tensor]:
        return self.weights


# ------------------------------------------------------------------------------ ONNX
_ONNX_DT = {1: np.float32, 2: np.uint8, 3: np.int8, 5: np.int16, 6: np.int32, 7: np.int64, 9: np.bool_, 10: np.float16, 11: np.float64}


def _onnx_tensor(buf: bytes) -> Tuple[str, torch.Tensor]:
    dims, dt, name, raw = [], 1, "", None
    floats, ints, int64s, doubles = [], [], [], []
    for no, wt, v in parse_message(buf):
        if no == 1:
            dims += list(np.frombuffer(v, dtype=np.uint8)) if False else ([v] if wt == 0 else _packed_varints(v))
        elif no == 2:
            dt = v
        elif no == 8:
            name = v.decode()
        elif no == 9:
            raw = v
        elif no == 4:
            floats += [v] if wt == 5 else list(np.frombuffer(v, dtype="<f4"))
        elif no == 5:
            ints += [v] if wt == 0 else _packed_varints(v)
        elif no == 7:
            int64s += [v] if wt == 0 else _packed_varints(v)
        elif no == 10:
            doubles += [v] if wt == 1 else list(np.frombuffer(v, dtype="<f8"))
    npdt = _ONNX_DT.get(dt)
    if npdt is None:
        raise ValueError(f"unsupported ONNX tensor data type {dt}")
    if raw is not None:
        arr = np.frombuffer(raw, dtype=np.dtype(npdt).newbyteorder("<")).copy()
    else:
        src = floats if dt == 1 else doubles if dt == 11 else int64s if dt == 7 else ints
        arr = np.array([_signed(x) if isinstance(x, int) else x for x in src], dtype=npdt)
    return name, torch.from_numpy(arr.reshape([int(d) for d in dims]) if dims else arr.reshape(()))


def _signed(v: int) -> int:
    return v - (1 << 64) if v >= (1 << 63) else v


def _packed_varints(b: bytes) -> List[int]:
    out, i = [], 0
    while i < len(b):
        n = s = 0
        while True:
            c = b[i]
            i += 1
            n |= (c & 0x7F) << s
            s += 7
            if not c & 0x80:
                break
        out.append(_signed(n))
    return out


def _onnx_attr(buf: bytes) -> Tuple[str, object]:
    name, val, ints, floats = "", None, [], []
    for no, wt, v in parse_message(buf):
        if no == 1:
            name = v.decode()
        elif no == 2:
            val = v                                  # float (wire type 5)
        elif no == 3:
            val = _signed(v)
        elif no == 4:
            val = v.decode(errors="replace")
        elif no == 5:
            val = _onnx_tensor(v)[1]
        elif no == 7:
            floats += [v] if wt == 5 else list(np.frombuffer(v, dtype="<f4"))
        elif no == 8:
            ints += [_signed(v)] if wt == 0 else _packed_varints(v)
    if ints:
        val = ints
    elif floats:
        val = floats
    return name, val


def parse_onnx(data: bytes) -> ImportedModel:
    model = parse_message(data)
    graph = next((v for no, _, v in model if no == 7), None)
    if graph is None:
        raise ValueError("not an ONNX model: no graph")
    producer = next((v.decode() for no, _, v in model if no == 2), "")
    ir = next((v for no, _, v in model if no == 1), 0)
    weights: Dict[str, torch.Tensor] = {}
    layers: List[LayerInfo] = []
    inputs, outputs, gname = [], [], ""
    for no, _, v in parse_message(graph):
        if no == 1:                                   # NodeProto
            ins, outs, op, name, attrs = [], [], "", "", {}
            for fno, _, fv in parse_message(v):
                if fno == 1:
                    ins.append(fv.decode())
                elif fno == 2:
                    outs.append(fv.decode())
                elif fno == 3:
                    name = fv.decode()
                elif fno == 4:
                    op = fv.decode()
                elif fno == 5:
                    k, a = _onnx_attr(fv)
                    attrs[k] = a
            layers.append(LayerInfo(name or f"{op}_{len(layers)}", op, ins, outs, attrs))
        elif no == 2:
            gname = v.decode()
        elif no == 5:
            n, t = _onnx_tensor(v)
            weights[n] = t
        elif no in (11, 12):                          # ValueInfoProto: name only
            nm = next((fv.decode() for fno, _, fv in parse_message(v) if fno == 1), "")
            (inputs if no == 11 else outputs).append(TensorSpec(nm, (), ""))
    arch = ModelArchitecture([i for i in inputs if i.name not in weights], outputs, sum(t.numel() for t in weights.values()))
    return ImportedModel(ModelMetadata(gname or "onnx_model", ModelFormat.ONNX, str(ir), producer), weights, layers, arch)


class OnnxModule(nn.Module):
    """Executes an imported ONNX graph (feed-forward subset) with torch ops."""

    def __init__(self, model: ImportedModel):
        super().__init__()
        self.model = model
        self.params = nn.ParameterDict({self._key(k): nn.Parameter(v.clone(), requires_grad=v.is_floating_point()) for k, v in model.weights.items()})

    @staticmethod
    def _key(name: str) -> str:
        return name.replace(".", "__dot__").replace("/", "__sl__").replace(":", "__c__")

    def forward(self, *inputs: torch.Tensor) -> torch.Tensor:
        env: Dict[str, torch.Tensor] = {k: self.params[self._key(k)] for k in self.model.weights}
        for spec, t in zip(self.model.architecture.inputs, inputs):
            env[spec.name] = t
        for L in self.model.layers:
            x = [env[i] if i else None for i in L.inputs]
            a, op = L.attributes, L.layer_type
            if op == "Gemm":
                A = x[0].t() if a.get("transA") else x[0]
                B = x[1].t() if a.get("transB") else x[1]
                y = a.get("alpha", 1.0) * (A @ B)
                if len(x) > 2 and x[2] is not None:
                    y = y + a.get("beta", 1.0) * x[2]
            elif op == "MatMul":
                y = x[0] @ x[1]
            elif op in ("Add", "Sub", "Mul", "Div"):
                y = {"Add": torch.add, "Sub": torch.sub, "Mul": torch.mul, "Div": torch.div}[op](x[0], x[1])
            elif op in ("Relu", "Sigmoid", "Tanh"):
                y = {"Relu": torch.relu, "Sigmoid": torch.sigmoid, "Tanh": torch.tanh}[op](x[0])
            elif op == "Softmax":
                y = torch.softmax(x[0], a.get("axis", -1))
            elif op == "Flatten":
                y = torch.flatten(x[0], a.get("axis", 1))
            elif op == "Reshape":
                y = x[0].reshape([int(v) for v in x[1].tolist()])
            elif op == "Conv":
                pads = a.get("pads", [0, 0, 0, 0])
                y = F.conv2d(x[0], x[1], x[2] if len(x) > 2 else None, tuple(a.get("strides", [1, 1])), (pads[0], pads[1]),
                             tuple(a.get("dilations", [1, 1])), a.get("group", 1))
            elif op == "BatchNormalization":
                y = F.batch_norm(x[0], x[3], x[4], x[1], x[2], False, 0.0, a.get("epsilon", 1e-5))
            elif op == "MaxPool":
                pads = a.get("pads", [0, 0, 0, 0])
                y = F.max_pool2d(x[0], tuple(a["kernel_shape"]), tuple(a.get("strides", a["kernel_shape"])), (pads[0], pads[1]))
            elif op == "GlobalAveragePool":
                y = x[0].mean((2, 3), keepdim=True)
            elif op == "Identity":
                y = x[0]
            else:
                raise NotImplementedError(f"ONNX operator '{op}' is not supported by the importer")
            env[L.outputs[0]] = y
        return env[self.model.architecture.outputs[0].name if self.model.architecture.outputs else self.model.layers[-1].outputs[0]]


# ------------------------------------------------------------------------------ importer
class ModelImporter:
    PRETRAINED = {"resnet18": ("cnn", "resnet18"), "resnet34": ("cnn", "resnet34"), "resnet50": ("cnn", "resnet50"),
                  "gpt2": ("gpt", {}), "bert-base-uncased": ("bert", "base")}

    def __init__(self):
        self.cache_dir = os.path.join(os.path.expanduser("~"), ".rustorch", "import_cache")
        self.progress: Optional[Callable[[int, Optional[int]], None]] = None

    def with_cache_dir(self, d: str) -> "ModelImporter":
        self.cache_dir = d
        return self

    def with_progress_callback(self, cb) -> "ModelImporter":
        self.progress = cb
        return self

    def import_from_file(self, path: str) -> ImportedModel:
        if not os.path.exists(path):
            raise FileNotFoundError(path)
        kind = st.detect_format(path)
        name = os.path.basename(path)
        if kind == "onnx" or (kind == "unknown" and path.endswith(".onnx")):
            with open(path, "rb") as f:
                m = parse_onnx(f.read())
            m.metadata.name = name
            return m
        if kind == "gguf":
            with gguf_fmt.GGUFFile(path) as g:
                w = {n: g.load_tensor(n) for n in g.tensors}
                md = ModelMetadata(name, ModelFormat.GGUF, str(g.metadata.get("general.file_type", "")), "gguf",
                                   {k: v for k, v in g.metadata.items() if not k.startswith("tokenizer.ggml.")})
            return self._finish(md, w)
        fmt = {"safetensors": ModelFormat.SAFETENSORS, "rustorch": ModelFormat.RUSTORCH, "torch": ModelFormat.PYTORCH,
               "pth": ModelFormat.PYTORCH, "json": ModelFormat.PYTORCH, "huggingface": ModelFormat.HUGGINGFACE}.get(kind)
        if fmt is None:
            raise ValueError(f"{name}: unrecognised model format")
        from ..models.high_level import load_state_dict_file
        return self._finish(ModelMetadata(name, fmt), load_state_dict_file(path))

    def _finish(self, md: ModelMetadata, weights: Dict[str, torch.Tensor]) -> ImportedModel:
        from ..convert import ModelParser
        layers = [LayerInfo(l.name, l.layer_type, attributes=dict(l.params)) for l in ModelParser().parse(weights).layers]
        return ImportedModel(md, weights, layers, ModelArchitecture(parameter_count=sum(t.numel() for t in weights.values())))

    def import_from_url(self, url: str) -> ImportedModel:
        from ..cli.download import _stream
        dest = os.path.join(self.cache_dir, os.path.basename(url.split("?")[0]) or "model.bin")
        return self.import_from_file(_stream(url, dest, {}, self.progress, False))

    def import_pretrained(self, model_name: str) -> ImportedModel:
        """Architecture with fresh weights when the named checkpoint is not in the cache (nothing is fetched implicitly)."""
        if model_name not in self.PRETRAINED:
            raise KeyError(f"unknown pretrained model '{model_name}'; known: {sorted(self.PRETRAINED)}")
        for ext in ("safetensors", "rustorch", "pt"):
            p = os.path.join(self.cache_dir, f"{model_name}.{ext}")
            if os.path.exists(p):
                return self.import_from_file(p)
        family, arg = self.PRETRAINED[model_name]
        if family == "cnn":
            from ..models import cnn
            module = getattr(cnn, arg)()
        elif family == "gpt":
            from ..models.gpt import GPT, GPTConfig
            module = GPT(GPTConfig())
        else:
            from ..models.sequence import bert_base_uncased
            module = bert_base_uncased()
        md = ModelMetadata(model_name, ModelFormat.RUSTORCH, extra={"pretrained": False, "note": "randomly initialised architecture"})
        return self._finish(md, {k: v.detach() for k, v in module.state_dict().items()})

    def to_module(self, model: ImportedModel) -> nn.Module:
        if model.metadata.format is ModelFormat.ONNX:
            return OnnxModule(model)
        from ..convert import SimplePyTorchConverter
        return SimplePyTorchConverter.convert(model.weights).to_module()


def import_model(path: str) -> ImportedModel:
    return ModelImporter().import_from_file(path)


def import_pretrained(name: str) -> ImportedModel:
    return ModelImporter().import_pretrained(name)
