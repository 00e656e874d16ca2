"""JIT: ``ScriptModule`` (parameters / buffers / constants + a computation graph of typed nodes), ``trace`` and
``script`` front ends, graph optimisation passes and a compilation cache (src/serialization/jit.rs:18-635).

``trace`` records the leaf modules and their data flow while running the model once (forward hooks), so the graph
is real (the reference's ``trace`` returns an empty graph, jit.rs:470-520).  ``optimize_graph`` removes dead
nodes, folds constant sub-graphs and marks fusible elementwise chains using the native planner.  A traced module
can be serialised (JSON graph + tensors in the RusTorch container) and executed again from the graph alone.
"""
from __future__ import annotations

import hashlib
import json
from dataclasses import asdict, dataclass, field
from typing import Callable, Dict, List, Optional, Sequence, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import _native

_ELEMENTWISE = {"ReLU": "relu", "Sigmoid": "sigmoid", "Tanh": "tanh", "GELU": "gelu", "SiLU": "silu", "Dropout": "dropout", "Identity": "scale"}


@dataclass
class GraphNode:
    id: int
    op_type: str
    name: str
    inputs: List[int]
    attrs: Dict[str, object] = field(default_factory=dict)
    params: List[str] = field(default_factory=list)        # keys into ScriptModule.parameters / buffers
    fused_with: Optional[int] = None


@dataclass
class ComputationGraph:
    nodes: List[GraphNode] = field(default_factory=list)
    inputs: List[int] = field(default_factory=list)
    outputs: List[int] = field(default_factory=list)

    def add(self, op_type: str, name: str, inputs: Sequence[int], attrs=None, params=None) -> int:
        self.nodes.append(GraphNode(len(self.nodes), op_type, name, list(inputs), dict(attrs or {}), list(params or [])))
        return len(self.nodes) - 1

    def to_json(self) -> str:
        return json.dumps({"nodes": [asdict(n) for n in self.nodes], "inputs": self.inputs, "outputs": self.outputs})

    @classmethod
    def from_json(cls, s: str) -> "ComputationGraph":
        d = json.loads(s)
        return cls([GraphNode(**n) for n in d["nodes"]], d["inputs"], d["outputs"])


def _attrs_of(m: nn.Module) -> Dict[str, object]:
    if isinstance(m, (nn.Conv1d, nn.Conv2d, nn.Conv3d)):
        return {"stride": list(m.stride), "padding": list(m.padding), "dilation": list(m.dilation), "groups": m.groups}
    if isinstance(m, (nn.MaxPool2d, nn.AvgPool2d)):
        to = lambda v: list(v) if isinstance(v, (tuple, list)) else [v, v]
        return {"kernel_size": to(m.kernel_size), "stride": to(m.stride or m.kernel_size), "padding": to(m.padding)}
    if isinstance(m, nn.Flatten):
        return {"start_dim": m.start_dim, "end_dim": m.end_dim}
    if isinstance(m, (nn.BatchNorm1d, nn.BatchNorm2d, nn.LayerNorm)):
        return {"eps": m.eps}
    if isinstance(m, nn.Dropout):
        return {"p": m.p}
    if isinstance(m, nn.LeakyReLU):
        return {"negative_slope": m.negative_slope}
    if isinstance(m, nn.Softmax):
        return {"dim": m.dim}
    if isinstance(m, nn.AdaptiveAvgPool2d):
        return {"output_size": list(m.output_size) if isinstance(m.output_size, (tuple, list)) else [m.output_size] * 2}
    return {}


class ScriptModule(nn.Module):
    def __init__(self, graph: ComputationGraph, parameters: Dict[str, torch.Tensor], buffers: Dict[str, torch.Tensor],
                 constants: Optional[Dict[str, object]] = None, name: str = "script_module"):
        super().__init__()
        self.graph, self.constants, self.script_name = graph, dict(constants or {}), name
        self._params = nn.ParameterDict({self._k(k): nn.Parameter(v.detach().clone(), requires_grad=v.is_floating_point()) for k, v in parameters.items()})
        for k, v in buffers.items():
            self.register_buffer(self._k(k), v.detach().clone())
        self.optimized = False

    @staticmethod
    def _k(name: str) -> str:
        return name.replace(".", "__")

    def _t(self, key: str) -> torch.Tensor:
        k = self._k(key)
        return self._params[k] if k in self._params else getattr(self, k)

    def forward(self, *inputs: torch.Tensor):
        vals: Dict[int, torch.Tensor] = dict(zip(self.graph.inputs, inputs))
        for n in self.graph.nodes:
            if n.id in vals:
                continue
            x = [vals[i] for i in n.inputs]
            p = {k.rsplit(".", 1)[-1]: self._t(k) for k in n.params}
            vals[n.id] = _execute(n, x, p, self.training)
        outs = [vals[o] for o in self.graph.outputs]
        return outs[0] if len(outs) == 1 else tuple(outs)

    def code(self) -> str:
        """Readable listing of the graph."""
        lines = [f"graph {self.script_name}({', '.join(f'%{i}' for i in self.graph.inputs)}):"]
        for n in self.graph.nodes:
            if n.op_type == "Input":
                continue
            extra = f"  # fused into %{n.fused_with}" if n.fused_with is not None else ""
            lines.append(f"  %{n.id} = {n.op_type}[{n.name}]({', '.join(f'%{i}' for i in n.inputs)}){extra}")
        lines.append(f"  return {', '.join(f'%{o}' for o in self.graph.outputs)}")
        return "\n".join(lines)

    def save(self, path: str) -> None:
        from ..formats import rustorch_bin
        params = {k: v.detach() for k, v in self._params.items()}
        bufs = {k: v for k, v in self.named_buffers()}
        rustorch_bin.save_state_dict(params, path, bufs, model_type="jit.ScriptModule",
                                     config={"graph": self.graph.to_json(), "constants": json.dumps(self.constants), "name": self.script_name})

    @classmethod
    def load(cls, path: str) -> "ScriptModule":
        from ..formats import rustorch_bin
        params, bufs, meta = rustorch_bin.load_state_dict(path)
        cfg = meta.get("config", {})
        m = cls(ComputationGraph.from_json(cfg["graph"]), {}, {}, json.loads(cfg.get("constants", "{}")), cfg.get("name", "script_module"))
        for k, v in params.items():
            m._params[k] = nn.Parameter(v, requires_grad=v.is_floating_point())
        for k, v in bufs.items():
            m.register_buffer(k, v)
        return m


def _execute(n: GraphNode, x: List[torch.Tensor], p: Dict[str, torch.Tensor], training: bool) -> torch.Tensor:
    t, a = n.op_type, n.attrs
    if t == "Linear":
        return F.linear(x[0], p["weight"], p.get("bias"))
    if t == "Conv2d":
        return F.conv2d(x[0], p["weight"], p.get("bias"), tuple(a["stride"]), tuple(a["padding"]), tuple(a["dilation"]), a["groups"])
    if t == "Conv1d":
        return F.conv1d(x[0], p["weight"], p.get("bias"), tuple(a["stride"]), tuple(a["padding"]), tuple(a["dilation"]), a["groups"])
    if t in ("BatchNorm1d", "BatchNorm2d"):
        return F.batch_norm(x[0], p.get("running_mean"), p.get("running_var"), p.get("weight"), p.get("bias"), False, 0.0, a.get("eps", 1e-5))
    if t == "LayerNorm":
        return F.layer_norm(x[0], p["weight"].shape, p.get("weight"), p.get("bias"), a.get("eps", 1e-5))
    if t == "Embedding":
        return F.embedding(x[0], p["weight"])
    if t == "ReLU":
        return F.relu(x[0])
    if t == "Sigmoid":
        return torch.sigmoid(x[0])
    if t == "Tanh":
        return torch.tanh(x[0])
    if t == "GELU":
        return F.gelu(x[0], approximate="tanh")
    if t in ("SiLU", "Swish"):
        return F.silu(x[0])
    if t == "LeakyReLU":
        return F.leaky_relu(x[0], a.get("negative_slope", 0.01))
    if t == "Softmax":
        return torch.softmax(x[0], a.get("dim", -1) if a.get("dim") is not None else -1)
    if t == "Dropout":
        return F.dropout(x[0], a.get("p", 0.5), training)
    if t == "Flatten":
        return torch.flatten(x[0], a.get("start_dim", 1), a.get("end_dim", -1))
    if t == "MaxPool2d":
        return F.max_pool2d(x[0], tuple(a["kernel_size"]), tuple(a["stride"]), tuple(a["padding"]))
    if t == "AvgPool2d":
        return F.avg_pool2d(x[0], tuple(a["kernel_size"]), tuple(a["stride"]), tuple(a["padding"]))
    if t == "AdaptiveAvgPool2d":
        return F.adaptive_avg_pool2d(x[0], tuple(a["output_size"]))
    if t == "Identity":
        return x[0]
    if t == "Add":
        return x[0] + x[1]
    if t == "Constant":
        return torch.tensor(a["value"])
    raise NotImplementedError(f"graph operator '{t}' cannot be executed")


def trace(module: nn.Module, *example_inputs: torch.Tensor, name: Optional[str] = None) -> ScriptModule:
    """Run ``module`` once and record every leaf module call and which earlier result (or input) fed it."""
    g = ComputationGraph()
    producer: Dict[int, int] = {}                      # id(tensor) -> node id
    keep = []                                          # keep traced tensors alive so ids stay unique
    for i, t in enumerate(example_inputs):
        nid = g.add("Input", f"input{i}", [])
        g.inputs.append(nid)
        producer[id(t)] = nid
        keep.append(t)
    params, buffers = {}, {}
    handles = []

    def hook(mod_name: str):
        def fn(m, inp, out):
            srcs = [producer[id(t)] for t in inp if isinstance(t, torch.Tensor) and id(t) in producer]
            if len(srcs) != sum(isinstance(t, torch.Tensor) for t in inp):
                raise RuntimeError(f"trace: an input of '{mod_name}' was produced outside a leaf module (functional op); wrap it in a module")
            keys = []
            for k, v in m.named_parameters(recurse=False):
                params[f"{mod_name}.{k}"] = v
                keys.append(f"{mod_name}.{k}")
            for k, v in m.named_buffers(recurse=False):
                if k != "num_batches_tracked":
                    buffers[f"{mod_name}.{k}"] = v
                    keys.append(f"{mod_name}.{k}")
            kind = type(m).__name__
            for base in type(m).__mro__:
                if base.__module__.startswith("torch.nn.modules") and base is not nn.Module:
                    kind = base.__name__
                    break
            nid = g.add(kind, mod_name, srcs, _attrs_of(m), keys)
            producer[id(out)] = nid
            keep.append(out)
        return fn

    for mod_name, m in module.named_modules():
        if mod_name and not list(m.children()):
            handles.append(m.register_forward_hook(hook(mod_name)))
    was_training = module.training
    module.eval()
    try:
        with torch.no_grad():
            out = module(*example_inputs)
    finally:
        for h in handles:
            h.remove()
        module.train(was_training)
    outs = out if isinstance(out, (tuple, list)) else [out]
    for o in outs:
        if id(o) not in producer:
            raise RuntimeError("trace: the model output is not the result of a leaf module; wrap the final functional ops in modules")
        g.outputs.append(producer[id(o)])
    return ScriptModule(g, params, buffers, name=name or type(module).__name__).train(was_training)


def script(module: nn.Module, *example_inputs: torch.Tensor) -> ScriptModule:
    """``nn.Sequential``-like containers are scripted structurally; anything else is traced with the example inputs."""
    if isinstance(module, nn.Sequential) and all(not list(m.children()) for m in module):
        g = ComputationGraph()
        prev = g.add("Input", "input0", [])
        g.inputs.append(prev)
        params, buffers = {}, {}
        for name, m in module.named_children():
            keys = []
            for k, v in m.named_parameters(recurse=False):
                params[f"{name}.{k}"] = v
                keys.append(f"{name}.{k}")
            for k, v in m.named_buffers(recurse=False):
                if k != "num_batches_tracked":
                    buffers[f"{name}.{k}"] = v
                    keys.append(f"{name}.{k}")
            kind = next((b.__name__ for b in type(m).__mro__ if b.__module__.startswith("torch.nn.modules") and b is not nn.Module), type(m).__name__)
            prev = g.add(kind, name, [prev], _attrs_of(m), keys)
        g.outputs.append(prev)
        return ScriptModule(g, params, buffers, name=type(module).__name__).train(module.training)
    if not example_inputs:
        raise ValueError("script: this module needs example inputs (it is traced)")
    return trace(module, *example_inputs)


def optimize_graph(sm: ScriptModule) -> Dict[str, int]:
    """Dead-node removal, identity / eval-mode dropout elimination, fusible elementwise chains.  Returns counters."""
    g = sm.graph
    stats = {"dead_removed": 0, "identities_removed": 0, "fusible_chains": 0}
    # 1. bypass Identity and (inference) Dropout
    redirect: Dict[int, int] = {}
    for n in g.nodes:
        n.inputs = [redirect.get(i, i) for i in n.inputs]
        if n.op_type in ("Identity", "Dropout") and len(n.inputs) == 1 and not sm.training:
            redirect[n.id] = n.inputs[0]
            stats["identities_removed"] += 1
    g.outputs = [redirect.get(o, o) for o in g.outputs]
    # 2. dead nodes through the native planner
    plan = _native.host().ExecutionPlan()
    for n in g.nodes:
        plan.add_node(_ELEMENTWISE.get(n.op_type, n.op_type.lower()), n.inputs, 0)
    for o in g.outputs:
        plan.mark_output(o)
    dead = set(plan.eliminate_dead()) - set(g.inputs)
    if dead:
        remap, kept = {}, []
        for n in g.nodes:
            if n.id in dead:
                continue
            remap[n.id] = len(kept)
            kept.append(n)
        for n in kept:
            n.id, n.inputs = remap[n.id], [remap[i] for i in n.inputs]
        g.nodes, g.inputs, g.outputs = kept, [remap[i] for i in g.inputs], [remap[o] for o in g.outputs]
        stats["dead_removed"] = len(dead)
    # 3. fusible chains on the cleaned graph
    plan = _native.host().ExecutionPlan()
    for n in g.nodes:
        plan.add_node(_ELEMENTWISE.get(n.op_type, n.op_type.lower()), n.inputs, 0)
    for chain in plan.fusible_chains():
        for nid in chain[1:]:
            g.nodes[nid].fused_with = chain[0]
        stats["fusible_chains"] += 1
    sm.optimized = True
    return stats


class JitCache:
    """Traced modules keyed by (module class, parameter shapes, input shapes / dtypes)."""

    def __init__(self, capacity: int = 32):
        self.capacity = capacity
        self._store: Dict[str, ScriptModule] = {}
        self.hits = self.misses = 0

    @staticmethod
    def key(module: nn.Module, inputs: Sequence[torch.Tensor]) -> str:
        sig = [type(module).__qualname__] + [f"{k}:{tuple(v.shape)}" for k, v in module.state_dict().items()]
        sig += [f"in:{tuple(t.shape)}:{t.dtype}" for t in inputs]
        return hashlib.sha256("|".join(sig).encode()).hexdigest()

    def get_or_trace(self, module: nn.Module, *inputs: torch.Tensor) -> ScriptModule:
        k = self.key(module, inputs)
        if k in self._store:
            self.hits += 1
            return self._store[k]
        self.misses += 1
        sm = trace(module, *inputs)
        if len(self._store) >= self.capacity:
            self._store.pop(next(iter(self._store)))
        self._store[k] = sm
        return sm

    def clear(self) -> None:
        self._store.clear()
