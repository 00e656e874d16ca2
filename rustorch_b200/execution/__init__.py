"""Dynamic execution: op graphs built at run time, planned natively (ordering, levels, dead-node removal,
liveness-based memory plan, elementwise chains) and executed with result caching; ``RuntimeEngine`` adds
warm-up, profiling and CUDA-graph replay of a planned graph
(src/execution/dynamic.rs:16-539, runtime.rs:14-486).

Instead of a tracing compiler, a planned graph whose shapes are fixed is captured once into a CUDA graph
and replayed: launch overhead disappears without changing any kernel.
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from enum import Enum
from typing import Callable, Dict, List, Optional, Sequence, Tuple

import torch
import torch.nn.functional as F

from .. import _native


class DynamicOp(Enum):
    """Operation kinds of the dynamic execution graph (src/execution/dynamic.rs)."""

    INPUT = "input"
    MATMUL = "matmul"
    ADD = "add"
    MUL = "mul"
    RELU = "relu"
    SIGMOID = "sigmoid"
    CONV2D = "conv2d"
    LINEAR = "linear"
    BATCH_NORM = "batch_norm"
    DROPOUT = "dropout"
    RESHAPE = "reshape"
    CUSTOM = "custom"


@dataclass
class DynamicNode:
    id: int
    op: DynamicOp
    inputs: List[int]
    attrs: Dict[str, object] = field(default_factory=dict)
    fn: Optional[Callable] = None          # CUSTOM ops
    value: Optional[torch.Tensor] = None   # INPUT nodes / cached results


def _apply(node: DynamicNode, xs: List[torch.Tensor]) -> torch.Tensor:
    from ..ops import elementwise as ew
    op, a = node.op, node.attrs
    if op is DynamicOp.MATMUL:
        return xs[0] @ xs[1]
    if op is DynamicOp.ADD:
        return ew.add(xs[0], xs[1]) if xs[0].shape == xs[1].shape else xs[0] + xs[1]
    if op is DynamicOp.MUL:
        return ew.mul(xs[0], xs[1]) if xs[0].shape == xs[1].shape else xs[0] * xs[1]
    if op is DynamicOp.RELU:
        return ew.unary("relu", xs[0])
    if op is DynamicOp.SIGMOID:
        return ew.unary("sigmoid", xs[0])
    if op is DynamicOp.CONV2D:
        return F.conv2d(xs[0], xs[1], xs[2] if len(xs) > 2 else None, a.get("stride", 1), a.get("padding", 0))
    if op is DynamicOp.LINEAR:
        return F.linear(xs[0], xs[1], xs[2] if len(xs) > 2 else None)
    if op is DynamicOp.BATCH_NORM:
        from ..ops.batchnorm import batch_norm
        return batch_norm(xs[0], None, None, xs[1] if len(xs) > 1 else None, xs[2] if len(xs) > 2 else None, True, 0.1, a.get("eps", 1e-5))
    if op is DynamicOp.DROPOUT:
        return F.dropout(xs[0], a.get("p", 0.5), a.get("training", False))
    if op is DynamicOp.RESHAPE:
        return xs[0].reshape(a["shape"])
    if op is DynamicOp.CUSTOM:
        return node.fn(*xs)
    raise ValueError(f"cannot execute {op}")


class DynamicExecutionContext:
    """Graph under construction + native plan + cached node results."""

    def __init__(self):
        self.nodes: List[DynamicNode] = []
        self.plan = _native.host().ExecutionPlan()
        self.cache_hits = self.executions = 0
        self._dirty: set = set()

    def add_input(self, value: torch.Tensor) -> int:
        return self._add(DynamicNode(len(self.nodes), DynamicOp.INPUT, [], value=value), value.numel() * value.element_size())

    def add_op(self, op: DynamicOp, inputs: Sequence[int], fn: Optional[Callable] = None, out_bytes: int = 0, **attrs) -> int:
        if op is DynamicOp.CUSTOM and fn is None:
            raise ValueError("CUSTOM ops need a callable")
        return self._add(DynamicNode(len(self.nodes), op, list(inputs), attrs, fn), out_bytes)

    def _add(self, node: DynamicNode, out_bytes: int) -> int:
        nid = self.plan.add_node(node.op.value, node.inputs, int(out_bytes))
        assert nid == node.id
        self.nodes.append(node)
        return nid

    def set_input(self, node_id: int, value: torch.Tensor) -> None:
        """Replace an input: every result that depends on it is invalidated."""
        n = self.nodes[node_id]
        if n.op is not DynamicOp.INPUT:
            raise ValueError("not an input node")
        n.value = value
        stale = {node_id}
        for m in self.nodes[node_id + 1:]:
            if any(i in stale for i in m.inputs):
                stale.add(m.id)
                m.value = None

    def execute(self, node_id: int) -> torch.Tensor:
        """Evaluate ``node_id``; nodes that no path to it needs are not run, cached results are reused."""
        order = [i for i in self.plan.topo_order() if i <= node_id]
        needed, stack = set(), [node_id]
        while stack:
            v = stack.pop()
            if v not in needed:
                needed.add(v)
                stack.extend(self.nodes[v].inputs)
        for i in order:
            n = self.nodes[i]
            if i not in needed:
                continue
            if n.value is not None:
                if n.op is not DynamicOp.INPUT:
                    self.cache_hits += 1
                continue
            n.value = _apply(n, [self.nodes[j].value for j in n.inputs])
            self.executions += 1
        return self.nodes[node_id].value

    def clear_cache(self) -> None:
        for n in self.nodes:
            if n.op is not DynamicOp.INPUT:
                n.value = None

    # -- planning views
    def execution_plan(self) -> List[int]:
        return list(self.plan.topo_order())

    def parallel_levels(self) -> List[List[int]]:
        return [list(l) for l in self.plan.levels()]

    def memory_plan(self) -> Dict[str, object]:
        offsets, (total, naive) = self.plan.memory_plan(256)
        return {"offsets": list(offsets), "arena_bytes": total, "naive_bytes": naive}

    def fusible_chains(self) -> List[List[int]]:
        return [list(c) for c in self.plan.fusible_chains()]

    def dead_nodes(self, outputs: Sequence[int]) -> List[int]:
        p = _native.host().ExecutionPlan()
        for n in self.nodes:
            p.add_node(n.op.value, n.inputs, 0)
        for o in outputs:
            p.mark_output(o)
        return list(p.eliminate_dead())


class GraphBuilder:
    """Fluent construction: ``b.input(x); h = b.linear(x_id, w, bias); y = b.relu(h)``."""

    def __init__(self, ctx: Optional[DynamicExecutionContext] = None):
        self.ctx = ctx or DynamicExecutionContext()

    def input(self, t: torch.Tensor) -> int:
        return self.ctx.add_input(t)

    def _bytes(self, *shape, like: int) -> int:
        n = 1
        for s in shape:
            n *= s
        return n * self.ctx.nodes[like].value.element_size() if self.ctx.nodes[like].value is not None else 0

    def linear(self, x: int, weight: torch.Tensor, bias: Optional[torch.Tensor] = None) -> int:
        ins = [x, self.input(weight)] + ([self.input(bias)] if bias is not None else [])
        return self.ctx.add_op(DynamicOp.LINEAR, ins)

    def conv2d(self, x: int, weight: torch.Tensor, bias: Optional[torch.Tensor] = None, stride: int = 1, padding: int = 0) -> int:
        ins = [x, self.input(weight)] + ([self.input(bias)] if bias is not None else [])
        return self.ctx.add_op(DynamicOp.CONV2D, ins, stride=stride, padding=padding)

    def relu(self, x: int) -> int:
        return self.ctx.add_op(DynamicOp.RELU, [x])

    def sigmoid(self, x: int) -> int:
        return self.ctx.add_op(DynamicOp.SIGMOID, [x])

    def add(self, a: int, b: int) -> int:
        return self.ctx.add_op(DynamicOp.ADD, [a, b])

    def mul(self, a: int, b: int) -> int:
        return self.ctx.add_op(DynamicOp.MUL, [a, b])

    def matmul(self, a: int, b: int) -> int:
        return self.ctx.add_op(DynamicOp.MATMUL, [a, b])

    def reshape(self, x: int, shape: Sequence[int]) -> int:
        return self.ctx.add_op(DynamicOp.RESHAPE, [x], shape=tuple(shape))

    def custom(self, fn: Callable, *inputs: int) -> int:
        return self.ctx.add_op(DynamicOp.CUSTOM, list(inputs), fn=fn)

    def build(self) -> DynamicExecutionContext:
        return self.ctx


@dataclass
class RuntimeMetrics:
    executions: int = 0
    total_ms: float = 0.0
    cache_hits: int = 0
    cache_misses: int = 0
    graph_replays: int = 0

    @property
    def avg_ms(self) -> float:
        return self.total_ms / self.executions if self.executions else 0.0

    @property
    def cache_hit_rate(self) -> float:
        t = self.cache_hits + self.cache_misses
        return self.cache_hits / t if t else 0.0


class RuntimeEngine:
    """Executes callables keyed by a signature (op name + input shapes/dtypes).  The first call of a key runs
    eagerly (warm-up); from then on, on CUDA, the call is captured into a CUDA graph and replayed with the new
    inputs copied into the captured buffers."""

    def __init__(self, use_cuda_graphs: bool = True, warmup_runs: int = 1):
        self.metrics = RuntimeMetrics()
        self.use_cuda_graphs = use_cuda_graphs and torch.cuda.is_available()
        self.warmup_runs = warmup_runs
        self._seen: Dict[tuple, int] = {}
        self._graphs: Dict[tuple, Tuple[object, List[torch.Tensor], object]] = {}
        self.profile: Dict[str, List[float]] = {}

    @staticmethod
    def _key(name: str, inputs: Sequence[torch.Tensor]) -> tuple:
        return (name,) + tuple((tuple(t.shape), t.dtype, str(t.device)) for t in inputs)

    def execute(self, name: str, fn: Callable, *inputs: torch.Tensor):
        key = self._key(name, inputs)
        t0 = time.perf_counter()
        n = self._seen.get(key, 0)
        self._seen[key] = n + 1
        cuda = self.use_cuda_graphs and all(t.is_cuda for t in inputs) and len(inputs) > 0
        if key in self._graphs:
            g, static_in, static_out = self._graphs[key]
            for s, t in zip(static_in, inputs):
                s.copy_(t)
            g.replay()
            out = static_out
            self.metrics.cache_hits += 1
            self.metrics.graph_replays += 1
        else:
            self.metrics.cache_misses += 1 if n == 0 else 0
            self.metrics.cache_hits += 1 if n > 0 else 0
            if cuda and n >= self.warmup_runs:
                static_in = [t.clone() for t in inputs]
                side = torch.cuda.Stream()
                side.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(side):
                    fn(*static_in)
                torch.cuda.current_stream().wait_stream(side)
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g):
                    static_out = fn(*static_in)
                self._graphs[key] = (g, static_in, static_out)
                g.replay()
                out = static_out
            else:
                out = fn(*inputs)
        if inputs and inputs[0].is_cuda:
            torch.cuda.synchronize()
        ms = (time.perf_counter() - t0) * 1e3
        self.metrics.executions += 1
        self.metrics.total_ms += ms
        self.profile.setdefault(name, []).append(ms)
        return out

    def warmup(self, name: str, fn: Callable, *inputs: torch.Tensor, runs: int = 3) -> None:
        for _ in range(runs):
            self.execute(name, fn, *inputs)

    def profile_report(self) -> Dict[str, Dict[str, float]]:
        return {k: {"calls": len(v), "mean_ms": sum(v) / len(v), "min_ms": min(v), "first_ms": v[0]} for k, v in self.profile.items()}

    def run_graph(self, ctx: DynamicExecutionContext, output: int) -> torch.Tensor:
        return self.execute(f"graph:{id(ctx)}:{output}", lambda: ctx.execute(output))
