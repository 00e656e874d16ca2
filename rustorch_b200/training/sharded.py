"""Sharded (per tensor-parallel rank) checkpoints with a merge / reshard tool, and asynchronous saves from pinned host
staging.

The reference keeps whole-model checkpoints only (``ModelCheckpoint`` / ``CheckpointManager``, src/serialization/
model_io.rs:483-792, src/training/checkpoint.rs:14-461) because its tensor parallelism never shards a real model
(src/distributed/model_parallel.rs:429-503).  Here every rank of a tensor-parallel group writes its own safetensors
shard; ``index.json`` records how each tensor was cut, so the shards can be merged into one state dict, or re-cut for
another world size, without the model code.

  python -m rustorch_b200.training.sharded merge <directory> <out.safetensors>
"""
from __future__ import annotations

import json
import os
import sys
import threading
from dataclasses import asdict, dataclass
from typing import Dict, List, Optional

import torch

from ..formats import load_safetensors, save_safetensors


@dataclass
class ShardSpec:
    """How a tensor is cut over the ranks: along ``dim``; ``segments`` (sizes along ``dim`` in the FULL tensor) for fused
    weights whose parts are sharded one by one (q | k | v, gate | up): a rank then holds the concatenation of its slice
    of every segment.  A tensor without a spec is replicated."""
    dim: int
    segments: Optional[List[int]] = None


Spec = Dict[str, Optional[ShardSpec]]


def shard_tensor(full: torch.Tensor, spec: Optional[ShardSpec], rank: int, world: int) -> torch.Tensor:
    if spec is None or world == 1:
        return full
    segs = spec.segments or [full.shape[spec.dim]]
    if sum(segs) != full.shape[spec.dim]:
        raise ValueError(f"segments {segs} do not cover dimension {spec.dim} of shape {tuple(full.shape)}")
    parts, start = [], 0
    for n in segs:
        if n % world:
            raise ValueError(f"segment of {n} rows does not divide over {world} ranks")
        k = n // world
        parts.append(full.narrow(spec.dim, start + rank * k, k))
        start += n
    return torch.cat(parts, spec.dim).contiguous()


def merge_tensors(parts: List[torch.Tensor], spec: Optional[ShardSpec], name: str = "") -> torch.Tensor:
    if spec is None or len(parts) == 1:
        for p in parts[1:]:
            if not torch.equal(p, parts[0]):
                raise ValueError(f"replicated tensor '{name}' differs between ranks")
        return parts[0]
    world = len(parts)
    segs = spec.segments or [parts[0].shape[spec.dim] * world]
    out, start = [], 0
    for n in segs:
        k = n // world
        out.extend(p.narrow(spec.dim, start, k) for p in parts)
        start += k
    return torch.cat(out, spec.dim).contiguous()


def infer_spec(module: torch.nn.Module) -> Spec:
    """Shard specs from the layer types: column-parallel weights (and biases) are cut along dim 0, row-parallel weights
    along dim 1; a module may add or override entries through a ``shard_spec()`` method (fused q|k|v weights)."""
    from ..distributed.model_parallel import ColumnParallelLinear, RowParallelLinear
    from ..distributed.tp_fused import FusedColumnParallelLinear, FusedRowParallelLinear
    spec: Spec = {}
    for prefix, m in module.named_modules():
        dot = prefix + "." if prefix else ""
        if isinstance(m, (ColumnParallelLinear, FusedColumnParallelLinear)):
            spec[dot + "weight"] = ShardSpec(0)
            if getattr(m, "bias", None) is not None:
                spec[dot + "bias"] = ShardSpec(0)
        elif isinstance(m, (RowParallelLinear, FusedRowParallelLinear)):
            spec[dot + "weight"] = ShardSpec(1)
    for prefix, m in module.named_modules():
        fn = getattr(m, "shard_spec", None)
        if callable(fn):
            dot = prefix + "." if prefix else ""
            spec.update({dot + k: v for k, v in fn().items()})
    return spec


def _shard_name(rank: int, world: int) -> str:
    return f"shard-{rank:05d}-of-{world:05d}.safetensors"


def save_sharded(state: Dict[str, torch.Tensor], directory: str, rank: int, world: int, spec: Spec,
                 metadata: Optional[Dict[str, str]] = None) -> str:
    """Write this rank's shard; rank 0 also writes ``index.json``.  ``state`` holds the rank's LOCAL tensors."""
    os.makedirs(directory, exist_ok=True)
    path = os.path.join(directory, _shard_name(rank, world))
    save_safetensors({k: v.detach().cpu() for k, v in state.items()}, path,
                     dict(metadata or {}, rank=str(rank), world=str(world)))
    if rank == 0:
        index = {"world": world, "format": "rustorch_b200.sharded.v1",
                 "tensors": {k: (asdict(spec[k]) if spec.get(k) is not None else None) for k in state}}
        tmp = os.path.join(directory, "index.json.tmp")
        with open(tmp, "w") as f:
            json.dump(index, f, indent=1)
        os.replace(tmp, os.path.join(directory, "index.json"))
    return path


def read_index(directory: str) -> dict:
    with open(os.path.join(directory, "index.json")) as f:
        return json.load(f)


def merge_sharded(directory: str) -> Dict[str, torch.Tensor]:
    """All shards of ``directory`` as one unsharded state dict."""
    index = read_index(directory)
    world = int(index["world"])
    shards = [load_safetensors(os.path.join(directory, _shard_name(r, world))) for r in range(world)]
    out = {}
    for name, s in index["tensors"].items():
        spec = ShardSpec(**s) if s is not None else None
        out[name] = merge_tensors([sh[name] for sh in shards], spec, name)
    return out


def load_sharded(directory: str, rank: int, world: int) -> Dict[str, torch.Tensor]:
    """The local state of ``rank`` in a group of ``world`` ranks; re-cuts the tensors when the checkpoint was written by
    a group of another size."""
    index = read_index(directory)
    if int(index["world"]) == world:
        return load_safetensors(os.path.join(directory, _shard_name(rank, world)))
    full = merge_sharded(directory)
    return {k: shard_tensor(v, ShardSpec(**index["tensors"][k]) if index["tensors"][k] is not None else None, rank, world)
            for k, v in full.items()}


class AsyncCheckpointer:
    """Saves a state dict without stalling the training loop: tensors are copied into reusable pinned host buffers
    (on a side CUDA stream when they live on a GPU), and a worker thread writes the safetensors file from there."""

    def __init__(self):
        self._staging: Dict[str, torch.Tensor] = {}
        self._thread: Optional[threading.Thread] = None
        self._error: Optional[BaseException] = None
        self._stream = torch.cuda.Stream() if torch.cuda.is_available() else None
        self.saved: List[str] = []

    def _stage(self, name: str, t: torch.Tensor) -> torch.Tensor:
        buf = self._staging.get(name)
        if buf is None or buf.shape != t.shape or buf.dtype != t.dtype:
            buf = torch.empty(t.shape, dtype=t.dtype, pin_memory=torch.cuda.is_available())
            self._staging[name] = buf
        buf.copy_(t.detach(), non_blocking=t.is_cuda)
        return buf

    def save(self, state: Dict[str, torch.Tensor], path: str, metadata: Optional[Dict[str, str]] = None) -> None:
        self.wait()                                           # one save in flight: the staging buffers are reused
        event = None
        if self._stream is not None and any(t.is_cuda for t in state.values()):
            self._stream.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(self._stream):
                staged = {k: self._stage(k, v) for k, v in state.items()}
                event = torch.cuda.Event()
                event.record(self._stream)
        else:
            staged = {k: self._stage(k, v) for k, v in state.items()}

        def work():
            try:
                if event is not None:
                    event.synchronize()
                tmp = path + ".tmp"
                save_safetensors(staged, tmp, metadata)
                os.replace(tmp, path)
                self.saved.append(path)
            except BaseException as e:                        # surfaced by wait()
                self._error = e

        self._thread = threading.Thread(target=work, name="async-checkpoint", daemon=True)
        self._thread.start()

    def wait(self) -> None:
        if self._thread is not None:
            self._thread.join()
            self._thread = None
        if self._error is not None:
            err, self._error = self._error, None
            raise err


def main(argv: Optional[List[str]] = None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    if len(argv) != 3 or argv[0] != "merge":
        print("usage: python -m rustorch_b200.training.sharded merge <directory> <out.safetensors>")
        return 2
    merged = merge_sharded(argv[1])
    save_safetensors(merged, argv[2], {"merged_from": os.path.abspath(argv[1])})
    print(f"merged {len(merged)} tensors from {read_index(argv[1])['world']} shards into {argv[2]}")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
