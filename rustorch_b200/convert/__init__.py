"""State-dict to model conversion: layer inference from parameter names and shapes, execution ordering,
transformer / CNN component extraction, layer factories, shape simulation, and validation / benchmarking of a
converted model against its source (src/convert/pytorch_to_rustorch_simplified.rs:13-300, model_parser.rs,
complex_architectures.rs:13-420, layer_integration.rs:11-560, validation_benchmark.rs:12-540).
"""
from __future__ import annotations

import re
import time
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence, Tuple

import torch
import torch.nn as nn


class SimpleConversionError(ValueError):
    """Raised when a PyTorch layer has no counterpart in the simplified converter (src/convert/pytorch_to_rustorch_simplified.rs)."""


@dataclass
class SimpleLayerDescription:
    name: str
    layer_type: str                       # Linear | Conv2d | Conv1d | BatchNorm | LayerNorm | Embedding | Unknown
    params: Dict[str, object] = field(default_factory=dict)
    tensors: Dict[str, torch.Tensor] = field(default_factory=dict)

    def parameter_count(self) -> int:
        return sum(t.numel() for k, t in self.tensors.items() if k in ("weight", "bias"))


LayerDescription = SimpleLayerDescription


def _natural_key(name: str):
    return [int(p) if p.isdigit() else p for p in re.split(r"(\d+)", name)]


def _infer(name: str, t: Dict[str, torch.Tensor]) -> SimpleLayerDescription:
    w = t.get("weight")
    if "running_mean" in t or "running_var" in t:
        return SimpleLayerDescription(name, "BatchNorm", {"num_features": t["running_mean"].numel()}, t)
    if w is None:
        return SimpleLayerDescription(name, "Unknown", {}, t)
    if w.dim() == 4:
        return SimpleLayerDescription(name, "Conv2d", {"out_channels": w.shape[0], "in_channels": w.shape[1], "kernel_size": tuple(w.shape[2:]),
                                                        "bias": "bias" in t}, t)
    if w.dim() == 3:
        return SimpleLayerDescription(name, "Conv1d", {"out_channels": w.shape[0], "in_channels": w.shape[1], "kernel_size": w.shape[2],
                                                        "bias": "bias" in t}, t)
    if w.dim() == 2:
        low = name.lower()
        if "bias" not in t and any(k in low for k in ("emb", "wte", "wpe", "token", "position")):
            return SimpleLayerDescription(name, "Embedding", {"num_embeddings": w.shape[0], "embedding_dim": w.shape[1]}, t)
        return SimpleLayerDescription(name, "Linear", {"out_features": w.shape[0], "in_features": w.shape[1], "bias": "bias" in t}, t)
    if w.dim() == 1:
        return SimpleLayerDescription(name, "LayerNorm", {"normalized_shape": w.shape[0], "bias": "bias" in t}, t)
    return SimpleLayerDescription(name, "Unknown", {}, t)


@dataclass
class ModelGraph:
    layers: List[SimpleLayerDescription]
    execution_order: List[str]
    edges: List[Tuple[str, str]]

    def layer(self, name: str) -> Optional[SimpleLayerDescription]:
        return next((l for l in self.layers if l.name == name), None)


class ModelParser:
    """Groups ``prefix.{weight,bias,running_*}`` entries into layers, orders them by their position in the state
    dict (natural order of numeric components as tie-break) and links consecutive layers whose sizes chain."""

    def parse(self, state_dict: Dict[str, torch.Tensor]) -> ModelGraph:
        groups: Dict[str, Dict[str, torch.Tensor]] = {}
        for k, v in state_dict.items():
            prefix, _, leaf = k.rpartition(".")
            if leaf == "num_batches_tracked":
                continue
            groups.setdefault(prefix, {})[leaf] = v
        layers = [_infer(name, t) for name, t in groups.items()]
        order = [l.name for l in layers]
        edges = []
        for a, b in zip(layers, layers[1:]):
            out_a = a.params.get("out_features") or a.params.get("out_channels") or a.params.get("num_features") or a.params.get("embedding_dim")
            in_b = b.params.get("in_features") or b.params.get("in_channels") or b.params.get("num_features") or b.params.get("normalized_shape")
            if out_a is not None and in_b is not None and (out_a == in_b or (a.layer_type.startswith("Conv") and b.layer_type == "Linear" and in_b % out_a == 0)):
                edges.append((a.name, b.name))
        return ModelGraph(layers, order, edges)


class SimplifiedPyTorchModel:
    def __init__(self, graph: ModelGraph):
        self.graph = graph
        self.layers: Dict[str, SimpleLayerDescription] = {l.name: l for l in graph.layers}
        self.execution_order = graph.execution_order
        self.total_parameters = sum(l.parameter_count() for l in graph.layers)

    def get_layer(self, name: str) -> Optional[SimpleLayerDescription]:
        return self.layers.get(name)

    def layer_names(self) -> List[str]:
        return list(self.execution_order)

    def summary(self) -> str:
        rows = [f"{'layer':<40}{'type':<12}{'params':>12}"]
        rows += [f"{n:<40}{self.layers[n].layer_type:<12}{self.layers[n].parameter_count():>12,}" for n in self.execution_order]
        rows.append(f"total parameters: {self.total_parameters:,}")
        return "\n".join(rows)

    def print_summary(self) -> None:
        print(self.summary())

    def simulate_forward(self, input_shape: Sequence[int]) -> List[int]:
        """Shape propagation through Linear / Conv2d / BatchNorm / LayerNorm layers in execution order (stride 1, no
        padding for convolutions; a flatten is inserted before the first Linear after a convolution)."""
        shape = list(input_shape)
        for n in self.execution_order:
            shape = LayerFactory.wrap(self.layers[n]).simulate_forward(shape)
        return shape

    def to_module(self, activation: Callable[[], nn.Module] = nn.ReLU) -> nn.Sequential:
        """A sequential model with the converted weights and ``activation`` between weighted layers."""
        mods: List[nn.Module] = []
        prev_conv = False
        weighted = [n for n in self.execution_order if self.layers[n].layer_type in ("Linear", "Conv2d", "Conv1d")]
        for n in self.execution_order:
            l = self.layers[n]
            if l.layer_type == "Linear" and prev_conv:
                mods.append(nn.Flatten())
            m = LayerFactory.create(l)
            if m is None:
                continue
            mods.append(m)
            if l.layer_type in ("Linear", "Conv2d", "Conv1d") and n != weighted[-1]:
                mods.append(activation())
            prev_conv = l.layer_type.startswith("Conv") or (prev_conv and l.layer_type == "BatchNorm")
        return nn.Sequential(*mods)


class SimplePyTorchConverter:
    @staticmethod
    def convert(state_dict: Dict[str, torch.Tensor]) -> SimplifiedPyTorchModel:
        if not state_dict:
            raise SimpleConversionError("empty state dict")
        if not all(isinstance(v, torch.Tensor) for v in state_dict.values()):
            raise SimpleConversionError("state dict values must be tensors")
        return SimplifiedPyTorchModel(ModelParser().parse(state_dict))


# ------------------------------------------------------------------------------ layer factory / wrappers
class _Wrapper:
    def __init__(self, desc: SimpleLayerDescription):
        self.desc = desc

    def parameter_count(self) -> int:
        return self.desc.parameter_count()


class LinearLayerWrapper(_Wrapper):
    def input_shape(self) -> List[int]:
        return [self.desc.params["in_features"]]

    def output_shape(self) -> List[int]:
        return [self.desc.params["out_features"]]

    def simulate_forward(self, shape: Sequence[int]) -> List[int]:
        fin = self.desc.params["in_features"]
        if shape[-1] != fin:
            flat = 1
            for s in shape[1:]:
                flat *= s
            if flat != fin:
                raise SimpleConversionError(f"{self.desc.name}: expected {fin} input features, got shape {list(shape)}")
            shape = [shape[0], flat]
        return list(shape[:-1]) + [self.desc.params["out_features"]]


class Conv2dLayerWrapper(_Wrapper):
    def simulate_forward(self, shape: Sequence[int], stride: int = 1, padding: int = 0) -> List[int]:
        p = self.desc.params
        if len(shape) != 4 or shape[1] != p["in_channels"]:
            raise SimpleConversionError(f"{self.desc.name}: expected [N, {p['in_channels']}, H, W], got {list(shape)}")
        kh, kw = p["kernel_size"]
        return [shape[0], p["out_channels"], (shape[2] + 2 * padding - kh) // stride + 1, (shape[3] + 2 * padding - kw) // stride + 1]


class BatchNorm2dLayerWrapper(_Wrapper):
    def simulate_forward(self, shape: Sequence[int]) -> List[int]:
        if shape[1] != self.desc.params["num_features"]:
            raise SimpleConversionError(f"{self.desc.name}: channel mismatch")
        return list(shape)


class _Passthrough(_Wrapper):
    def simulate_forward(self, shape: Sequence[int]) -> List[int]:
        return list(shape)


class LayerFactory:
    @staticmethod
    def wrap(desc: SimpleLayerDescription) -> _Wrapper:
        return {"Linear": LinearLayerWrapper, "Conv2d": Conv2dLayerWrapper, "BatchNorm": BatchNorm2dLayerWrapper}.get(desc.layer_type, _Passthrough)(desc)

    @staticmethod
    def create_linear(desc: SimpleLayerDescription) -> nn.Linear:
        m = nn.Linear(desc.params["in_features"], desc.params["out_features"], bias=desc.params["bias"])
        with torch.no_grad():
            m.weight.copy_(desc.tensors["weight"])
            if m.bias is not None:
                m.bias.copy_(desc.tensors["bias"])
        return m

    @staticmethod
    def create_conv2d(desc: SimpleLayerDescription, stride=1, padding=0) -> nn.Conv2d:
        p = desc.params
        m = nn.Conv2d(p["in_channels"], p["out_channels"], p["kernel_size"], stride, padding, bias=p["bias"])
        with torch.no_grad():
            m.weight.copy_(desc.tensors["weight"])
            if m.bias is not None:
                m.bias.copy_(desc.tensors["bias"])
        return m

    @staticmethod
    def create_batch_norm2d(desc: SimpleLayerDescription) -> nn.BatchNorm2d:
        m = nn.BatchNorm2d(desc.params["num_features"], affine="weight" in desc.tensors)
        m.load_state_dict({k: v for k, v in desc.tensors.items()}, strict=False)
        return m

    @staticmethod
    def create(desc: SimpleLayerDescription) -> Optional[nn.Module]:
        t = desc.layer_type
        if t == "Linear":
            return LayerFactory.create_linear(desc)
        if t == "Conv2d":
            return LayerFactory.create_conv2d(desc)
        if t == "BatchNorm":
            return LayerFactory.create_batch_norm2d(desc)
        if t == "LayerNorm":
            m = nn.LayerNorm(desc.params["normalized_shape"], elementwise_affine=True, bias=desc.params["bias"])
            m.load_state_dict(desc.tensors, strict=False)
            return m
        if t == "Embedding":
            return nn.Embedding.from_pretrained(desc.tensors["weight"].clone(), freeze=False)
        return None


class IntegratedModelRunner:
    def __init__(self):
        self.wrappers: List[_Wrapper] = []

    def add_linear_layer(self, w: LinearLayerWrapper) -> None:
        self.wrappers.append(w)

    def add_conv_layer(self, w: Conv2dLayerWrapper) -> None:
        self.wrappers.append(w)

    def add_batch_norm_layer(self, w: BatchNorm2dLayerWrapper) -> None:
        self.wrappers.append(w)

    def total_parameters(self) -> int:
        return sum(w.parameter_count() for w in self.wrappers)

    def simulate_forward(self, input_shape: Sequence[int]) -> List[int]:
        s = list(input_shape)
        for w in self.wrappers:
            s = w.simulate_forward(s)
        return s

    def summary(self) -> str:
        return "\n".join(f"{w.desc.name}: {w.desc.layer_type} ({w.parameter_count():,} params)" for w in self.wrappers)


def convert_to_integrated_model(model: SimplifiedPyTorchModel) -> IntegratedModelRunner:
    r = IntegratedModelRunner()
    for n in model.execution_order:
        r.wrappers.append(LayerFactory.wrap(model.layers[n]))
    return r


# ------------------------------------------------------------------------------ complex architectures
@dataclass
class MultiheadAttentionInfo:
    name: str
    embed_dim: int
    fused_qkv: bool


@dataclass
class FeedForwardInfo:
    name: str
    d_model: int
    d_ff: int


@dataclass
class TransformerComponents:
    num_layers: int = 0
    attention: List[MultiheadAttentionInfo] = field(default_factory=list)
    feed_forward: List[FeedForwardInfo] = field(default_factory=list)
    layer_norms: List[str] = field(default_factory=list)
    token_embedding: Optional[Tuple[int, int]] = None       # (vocab, dim)
    position_embedding: Optional[Tuple[int, int]] = None


@dataclass
class CNNComponents:
    conv_layers: List[Tuple[str, int, int, Tuple[int, int]]] = field(default_factory=list)   # name, in, out, kernel
    batch_norms: List[str] = field(default_factory=list)
    classifier: Optional[Tuple[str, int, int]] = None


class ComplexArchitectureParser:
    @staticmethod
    def parse_transformer(state_dict: Dict[str, torch.Tensor]) -> TransformerComponents:
        g = ModelParser().parse(state_dict)
        c = TransformerComponents()
        blocks = set()
        for l in g.layers:
            low = l.name.lower()
            m = re.search(r"(?:layers?|h|blocks?|blk)\.(\d+)\.", low)
            if m:
                blocks.add(int(m.group(1)))
            if l.layer_type == "Linear":
                o, i = l.params["out_features"], l.params["in_features"]
                if any(k in low for k in ("attn", "attention")) and ("qkv" in low or "c_attn" in low or "in_proj" in low or o == 3 * i):
                    c.attention.append(MultiheadAttentionInfo(l.name, i, True))
                elif any(k in low for k in ("q_proj", "query", "attn_q", ".wq")):
                    c.attention.append(MultiheadAttentionInfo(l.name, i, False))
                elif o > i and any(k in low for k in ("mlp", "ffn", "fc", "intermediate", "feed_forward", "linear1", "c_fc")):
                    c.feed_forward.append(FeedForwardInfo(l.name, i, o))
            elif l.layer_type == "LayerNorm":
                c.layer_norms.append(l.name)
            elif l.layer_type == "Embedding":
                shape = (l.params["num_embeddings"], l.params["embedding_dim"])
                if any(k in low for k in ("pos", "wpe")):
                    c.position_embedding = shape
                elif c.token_embedding is None:
                    c.token_embedding = shape
        c.num_layers = len(blocks)
        return c

    @staticmethod
    def parse_cnn(state_dict: Dict[str, torch.Tensor]) -> CNNComponents:
        g = ModelParser().parse(state_dict)
        c = CNNComponents()
        for l in g.layers:
            if l.layer_type == "Conv2d":
                c.conv_layers.append((l.name, l.params["in_channels"], l.params["out_channels"], tuple(l.params["kernel_size"])))
            elif l.layer_type == "BatchNorm":
                c.batch_norms.append(l.name)
            elif l.layer_type == "Linear":
                c.classifier = (l.name, l.params["in_features"], l.params["out_features"])
        return c


# ------------------------------------------------------------------------------ validation / benchmark
@dataclass
class AccuracyMetrics:
    max_abs_error: float
    mean_abs_error: float
    relative_error: float
    passed: bool


@dataclass
class PerformanceMetrics:
    mean_ms: float
    min_ms: float
    throughput_per_s: float


@dataclass
class MemoryMetrics:
    parameter_bytes: int
    activation_bytes_estimate: int


@dataclass
class ValidationResults:
    accuracy: AccuracyMetrics
    performance: PerformanceMetrics
    memory: MemoryMetrics


class ModelValidator:
    @staticmethod
    def validate_accuracy(converted: nn.Module, reference: Callable, inputs: torch.Tensor, tolerance: float = 1e-5) -> AccuracyMetrics:
        with torch.no_grad():
            a, b = converted(inputs).float(), reference(inputs).float()
        d = (a - b).abs()
        rel = float(d.max() / b.abs().max().clamp_min(1e-12))
        return AccuracyMetrics(float(d.max()), float(d.mean()), rel, rel <= tolerance)

    @staticmethod
    def benchmark_performance(fn: Callable, inputs: torch.Tensor, iters: int = 10, warmup: int = 2) -> PerformanceMetrics:
        sync = torch.cuda.synchronize if inputs.is_cuda else (lambda: None)
        with torch.no_grad():
            for _ in range(warmup):
                fn(inputs)
            ts = []
            for _ in range(iters):
                sync()
                t0 = time.perf_counter()
                fn(inputs)
                sync()
                ts.append((time.perf_counter() - t0) * 1e3)
        mean = sum(ts) / len(ts)
        return PerformanceMetrics(mean, min(ts), inputs.shape[0] / (mean / 1e3))

    @staticmethod
    def estimate_memory_usage(model: nn.Module, input_shape: Sequence[int], dtype_bytes: int = 4) -> MemoryMetrics:
        pb = sum(p.numel() * p.element_size() for p in model.parameters())
        n = 1
        for s in input_shape:
            n *= s
        return MemoryMetrics(pb, n * dtype_bytes * (1 + sum(1 for _ in model.modules())))

    @staticmethod
    def comprehensive_validation(converted: nn.Module, reference: Callable, inputs: torch.Tensor, tolerance: float = 1e-5) -> ValidationResults:
        return ValidationResults(ModelValidator.validate_accuracy(converted, reference, inputs, tolerance),
                                 ModelValidator.benchmark_performance(converted, inputs, 5, 1),
                                 ModelValidator.estimate_memory_usage(converted, inputs.shape))

    @staticmethod
    def generate_report(r: ValidationResults) -> str:
        return (f"accuracy: max |err| {r.accuracy.max_abs_error:.3e}, relative {r.accuracy.relative_error:.3e} "
                f"({'PASS' if r.accuracy.passed else 'FAIL'})\nperformance: {r.performance.mean_ms:.3f} ms/iter, "
                f"{r.performance.throughput_per_s:.1f} samples/s\nmemory: {r.memory.parameter_bytes / 1e6:.2f} MB parameters")
