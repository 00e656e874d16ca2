"""Sparse tensors (COO / CSR), sparse ops, pruning, sparse layers, analysis / validation / IO
(src/sparse/mod.rs:28-420, pruning.rs:15-560, sparse_layers.rs:16-600, utils.rs:13-600, gpu_ops.rs).

``SparseTensor`` keeps indices and values as device tensors and multiplies through ``torch.sparse`` (cuSPARSE
SpMV / SpMM on CUDA), so a pruned layer runs on the GPU without densifying.  Pruning masks are computed with
``kthvalue`` / ``topk`` on the device.
"""
from __future__ import annotations

import struct
import time
from dataclasses import dataclass, field
from enum import Enum
from typing import Dict, List, Optional, Sequence, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F


class SparseFormat(Enum):
    """COO or CSR storage of a sparse tensor (src/sparse/mod.rs)."""

    COO = "coo"
    CSR = "csr"


class SparseTensor:
    """2-D (CSR or COO) or N-D (COO) sparse tensor."""

    def __init__(self, fmt: SparseFormat, shape: Sequence[int], values: torch.Tensor, indices: Optional[torch.Tensor] = None,
                 crow: Optional[torch.Tensor] = None, col: Optional[torch.Tensor] = None):
        self.format, self.shape, self.values = fmt, tuple(shape), values
        self.indices, self.crow, self.col = indices, crow, col

    # -- constructors
    @classmethod
    def from_coo(cls, indices: torch.Tensor, values: torch.Tensor, shape: Sequence[int]) -> "SparseTensor":
        indices = torch.as_tensor(indices, dtype=torch.long, device=values.device)
        if indices.dim() != 2 or indices.shape[0] != len(shape) or indices.shape[1] != values.numel():
            raise ValueError("COO indices must be [ndim, nnz]")
        for d, n in enumerate(shape):
            if indices.numel() and (int(indices[d].min()) < 0 or int(indices[d].max()) >= n):
                raise IndexError(f"index out of range along dim {d}")
        return cls(SparseFormat.COO, shape, values, indices=indices)

    @classmethod
    def from_csr(cls, crow: torch.Tensor, col: torch.Tensor, values: torch.Tensor, shape: Sequence[int]) -> "SparseTensor":
        crow = torch.as_tensor(crow, dtype=torch.long, device=values.device)
        col = torch.as_tensor(col, dtype=torch.long, device=values.device)
        if len(shape) != 2 or crow.numel() != shape[0] + 1 or int(crow[-1]) != values.numel() or col.numel() != values.numel():
            raise ValueError("CSR needs a 2-D shape, rows + 1 row pointers and one column index per value")
        return cls(SparseFormat.CSR, shape, values, crow=crow, col=col)

    @classmethod
    def from_dense(cls, dense: torch.Tensor, threshold: float = 0.0) -> "SparseTensor":
        mask = dense.abs() > threshold
        idx = mask.nonzero().t().contiguous()
        return cls(SparseFormat.COO, dense.shape, dense[mask], indices=idx)

    # -- properties
    @property
    def nnz(self) -> int:
        return self.values.numel()

    @property
    def device(self):
        return self.values.device

    def dense_size(self) -> int:
        n = 1
        for s in self.shape:
            n *= s
        return n

    def sparsity(self) -> float:
        return 1.0 - self.nnz / max(1, self.dense_size())

    def memory_usage(self) -> int:
        idx = self.indices.numel() * 8 if self.format is SparseFormat.COO else (self.crow.numel() + self.col.numel()) * 8
        return self.values.numel() * self.values.element_size() + idx

    # -- conversions
    def to_coo(self) -> "SparseTensor":
        if self.format is SparseFormat.COO:
            return self
        counts = self.crow[1:] - self.crow[:-1]
        rows = torch.repeat_interleave(torch.arange(self.shape[0], device=self.device), counts)
        return SparseTensor(SparseFormat.COO, self.shape, self.values, indices=torch.stack([rows, self.col]))

    def to_csr(self) -> "SparseTensor":
        if self.format is SparseFormat.CSR:
            return self
        if len(self.shape) != 2:
            raise ValueError("CSR is defined for matrices")
        order = torch.argsort(self.indices[0] * self.shape[1] + self.indices[1])
        rows, cols, vals = self.indices[0][order], self.indices[1][order], self.values[order]
        crow = torch.zeros(self.shape[0] + 1, dtype=torch.long, device=self.device)
        crow[1:] = torch.cumsum(torch.bincount(rows, minlength=self.shape[0]), 0)
        return SparseTensor(SparseFormat.CSR, self.shape, vals, crow=crow, col=cols)

    def to_dense(self) -> torch.Tensor:
        c = self.to_coo()
        out = torch.zeros(self.shape, dtype=self.values.dtype, device=self.device)
        out.index_put_(tuple(c.indices), c.values, accumulate=True)
        return out

    def to_torch(self) -> torch.Tensor:
        if self.format is SparseFormat.CSR:
            return torch.sparse_csr_tensor(self.crow, self.col, self.values, self.shape)
        return torch.sparse_coo_tensor(self.indices, self.values, self.shape).coalesce()

    def to(self, device) -> "SparseTensor":
        mv = lambda t: None if t is None else t.to(device)
        return SparseTensor(self.format, self.shape, self.values.to(device), mv(self.indices), mv(self.crow), mv(self.col))

    # -- ops (the SparseOps trait)
    def spmv(self, v: torch.Tensor) -> torch.Tensor:
        if len(self.shape) != 2 or v.dim() != 1 or v.shape[0] != self.shape[1]:
            raise ValueError("spmv: matrix [m, n] times vector [n]")
        if self._native(v):
            return self._native_spmm(v.unsqueeze(1)).squeeze(1)
        return (self.to_torch() @ v.unsqueeze(1)).squeeze(1)

    def _native(self, dense: torch.Tensor) -> bool:
        from .. import _native
        return (dense.is_cuda and self.values.is_cuda and self.values.dtype == torch.float32 and dense.dtype == torch.float32
                and not dense.requires_grad and _native.available())

    def _native_spmm(self, dense: torch.Tensor) -> torch.Tensor:
        """CSR x dense on the warp-per-row kernel (csrc/nn/rnn_amp_sparse.cu)."""
        from .. import _native
        c = self if self.format is SparseFormat.CSR else self.to_csr()
        y = torch.empty((self.shape[0], dense.shape[1]), dtype=torch.float32, device=dense.device)
        _native.load(required=True).csr_spmm(c.crow.to(torch.int64).contiguous(), c.col.to(torch.int64).contiguous(),
                                             c.values.contiguous(), dense.contiguous(), y)
        return y

    def spmm(self, dense: torch.Tensor) -> torch.Tensor:
        if len(self.shape) != 2 or dense.shape[0] != self.shape[1]:
            raise ValueError("spmm: matrix [m, n] times dense [n, k]")
        if dense.dim() == 2 and self._native(dense):
            return self._native_spmm(dense)
        return self.to_torch() @ dense

    def add(self, other: "SparseTensor") -> "SparseTensor":
        if self.shape != other.shape:
            raise ValueError("shape mismatch")
        a, b = self.to_coo(), other.to_coo()
        t = torch.sparse_coo_tensor(torch.cat([a.indices, b.indices], 1), torch.cat([a.values, b.values]), self.shape).coalesce()
        return SparseTensor(SparseFormat.COO, self.shape, t.values(), indices=t.indices())

    def mul_scalar(self, s: float) -> "SparseTensor":
        return SparseTensor(self.format, self.shape, self.values * s, self.indices, self.crow, self.col)

    def transpose(self) -> "SparseTensor":
        c = self.to_coo()
        return SparseTensor(SparseFormat.COO, self.shape[::-1], c.values, indices=c.indices.flip(0))


SparseOps = SparseTensor


# ------------------------------------------------------------------------------ pruning
class PruningStrategy(Enum):
    """Criterion of the sparse module's pruners (src/sparse/pruning.rs)."""

    MAGNITUDE = "magnitude"
    RANDOM = "random"
    STRUCTURED = "structured"
    GRADIENT = "gradient"
    FISHER = "fisher"


class StructuredGranularity(Enum):
    """Rows, columns or blocks as the unit of structured pruning."""

    ROW = "row"           # output neurons
    COLUMN = "column"     # input features
    CHANNEL = "channel"   # conv filters
    BLOCK = "block"       # n x n blocks


@dataclass
class PruningConfig:
    strategy: PruningStrategy = PruningStrategy.MAGNITUDE
    target_sparsity: float = 0.5
    granularity: StructuredGranularity = StructuredGranularity.ROW
    block_size: int = 4


@dataclass
class PruningSchedule:
    """Polynomial (cubic) ramp from ``initial`` to ``final`` sparsity between ``begin`` and ``end`` steps."""
    initial_sparsity: float = 0.0
    final_sparsity: float = 0.9
    begin_step: int = 0
    end_step: int = 1000
    frequency: int = 100
    step_count: int = 0

    def current_sparsity(self) -> float:
        if self.step_count <= self.begin_step:
            return self.initial_sparsity
        if self.step_count >= self.end_step:
            return self.final_sparsity
        p = (self.step_count - self.begin_step) / (self.end_step - self.begin_step)
        return self.final_sparsity + (self.initial_sparsity - self.final_sparsity) * (1 - p) ** 3

    def step(self) -> None:
        self.step_count += 1

    def should_prune(self) -> bool:
        return self.begin_step <= self.step_count <= self.end_step and (self.step_count - self.begin_step) % self.frequency == 0


def _mask_smallest(score: torch.Tensor, sparsity: float) -> torch.Tensor:
    k = int(score.numel() * sparsity)
    if k <= 0:
        return torch.ones_like(score, dtype=torch.bool)
    if k >= score.numel():
        return torch.zeros_like(score, dtype=torch.bool)
    thr = torch.kthvalue(score.reshape(-1).float(), k).values
    mask = score > thr
    short = score.numel() - k - int(mask.sum())              # ties at the threshold: keep just enough of them
    if short > 0:
        ties = (score == thr).reshape(-1).nonzero().reshape(-1)[:short]
        mask.reshape(-1)[ties] = True
    return mask


class MagnitudePruner:
    def __init__(self, sparsity: float = 0.5):
        self.sparsity = sparsity

    def mask(self, t: torch.Tensor) -> torch.Tensor:
        return _mask_smallest(t.detach().abs(), self.sparsity)

    def prune(self, t: torch.Tensor) -> torch.Tensor:
        return t * self.mask(t)


class StructuredPruner:
    def __init__(self, sparsity: float = 0.5, granularity: StructuredGranularity = StructuredGranularity.ROW, block_size: int = 4):
        self.sparsity, self.granularity, self.block = sparsity, granularity, block_size

    def mask(self, w: torch.Tensor) -> torch.Tensor:
        g = self.granularity
        if g in (StructuredGranularity.ROW, StructuredGranularity.CHANNEL):
            keep = _mask_smallest(w.detach().reshape(w.shape[0], -1).norm(dim=1), self.sparsity)
            return keep.view(-1, *([1] * (w.dim() - 1))).expand_as(w)
        if g is StructuredGranularity.COLUMN:
            keep = _mask_smallest(w.detach().transpose(0, 1).reshape(w.shape[1], -1).norm(dim=1), self.sparsity)
            return keep.view(1, -1, *([1] * (w.dim() - 2))).expand_as(w)
        b = self.block
        if w.dim() != 2 or w.shape[0] % b or w.shape[1] % b:
            raise ValueError("block pruning needs a matrix whose sides are multiples of the block size")
        blocks = w.detach().reshape(w.shape[0] // b, b, w.shape[1] // b, b).permute(0, 2, 1, 3).reshape(w.shape[0] // b, w.shape[1] // b, -1)
        keep = _mask_smallest(blocks.norm(dim=-1), self.sparsity)
        return keep.repeat_interleave(b, 0).repeat_interleave(b, 1)

    def prune_linear_weights(self, w: torch.Tensor) -> torch.Tensor:
        return w * self.mask(w)


class FisherPruner:
    """Importance = running mean of squared gradients x squared weight (diagonal Fisher information)."""

    def __init__(self, sparsity: float = 0.5, decay: float = 0.9):
        self.sparsity, self.decay = sparsity, decay
        self.fisher: Dict[str, torch.Tensor] = {}

    def update_fisher(self, name: str, grad: torch.Tensor) -> None:
        g2 = grad.detach().float() ** 2
        self.fisher[name] = g2 if name not in self.fisher else self.decay * self.fisher[name] + (1 - self.decay) * g2

    def prune_with_fisher(self, name: str, t: torch.Tensor) -> torch.Tensor:
        if name not in self.fisher:
            raise KeyError(f"no Fisher information for '{name}'")
        return t * _mask_smallest(self.fisher[name] * t.detach().float() ** 2, self.sparsity)


class ModelPruner:
    def __init__(self, config: Optional[PruningConfig] = None, schedule: Optional[PruningSchedule] = None):
        self.config, self.schedule = config or PruningConfig(), schedule
        self.importance: Dict[str, torch.Tensor] = {}
        self.masks: Dict[str, torch.Tensor] = {}

    def update_importance_scores(self, name: str, grad: torch.Tensor) -> None:
        s = grad.detach().abs().float()
        self.importance[name] = s if name not in self.importance else 0.9 * self.importance[name] + 0.1 * s

    def _mask(self, name: str, t: torch.Tensor, sparsity: float) -> torch.Tensor:
        st = self.config.strategy
        if st is PruningStrategy.MAGNITUDE:
            return MagnitudePruner(sparsity).mask(t)
        if st is PruningStrategy.RANDOM:
            return _mask_smallest(torch.rand_like(t, dtype=torch.float32), sparsity)
        if st is PruningStrategy.STRUCTURED:
            return StructuredPruner(sparsity, self.config.granularity, self.config.block_size).mask(t)
        score = self.importance.get(name)
        if score is None:
            return MagnitudePruner(sparsity).mask(t)
        return _mask_smallest(score * (t.detach().abs().float() if st is PruningStrategy.GRADIENT else t.detach().float() ** 2), sparsity)

    def prune_tensor(self, t: torch.Tensor, name: str = "") -> SparseTensor:
        sp = self.schedule.current_sparsity() if self.schedule else self.config.target_sparsity
        return SparseTensor.from_dense(t.detach() * self._mask(name, t, sp))

    def prune_model(self, model: nn.Module, min_dim: int = 2) -> Dict[str, float]:
        """Zero the pruned weights in place (weight matrices / filters only) and remember the masks."""
        sp = self.schedule.current_sparsity() if self.schedule else self.config.target_sparsity
        report = {}
        with torch.no_grad():
            for name, p in model.named_parameters():
                if p.dim() >= min_dim:
                    m = self._mask(name, p, sp)
                    p.mul_(m)
                    self.masks[name] = m
                    report[name] = 1.0 - float(m.float().mean())
        return report

    def apply_masks(self, model: nn.Module) -> None:
        """Re-apply the stored masks (call after each optimiser step to keep pruned weights at zero)."""
        with torch.no_grad():
            for name, p in model.named_parameters():
                if name in self.masks:
                    p.mul_(self.masks[name])


# ------------------------------------------------------------------------------ layers
class SparseLinear(nn.Module):
    """Linear layer whose weight is stored as CSR values (trainable) with a fixed pattern."""

    def __init__(self, in_features: int, out_features: int, sparsity: float = 0.9, bias: bool = True):
        super().__init__()
        self.in_features, self.out_features = in_features, out_features
        w = torch.empty(out_features, in_features)
        nn.init.kaiming_uniform_(w, a=5 ** 0.5)
        self._set_pattern(w * _mask_smallest(torch.rand_like(w), sparsity))
        self.bias = nn.Parameter(torch.zeros(out_features)) if bias else None

    def _set_pattern(self, dense: torch.Tensor) -> None:
        csr = SparseTensor.from_dense(dense).to_csr()
        self.values = nn.Parameter(csr.values.clone())
        self.register_buffer("crow", csr.crow, persistent=True)
        self.register_buffer("col", csr.col, persistent=True)

    @classmethod
    def from_dense(cls, linear: nn.Linear, sparsity: float) -> "SparseLinear":
        m = cls.__new__(cls)
        nn.Module.__init__(m)
        m.in_features, m.out_features = linear.in_features, linear.out_features
        m._set_pattern(MagnitudePruner(sparsity).prune(linear.weight.detach()))
        m.bias = nn.Parameter(linear.bias.detach().clone()) if linear.bias is not None else None
        return m

    with_pruning = from_dense

    def weight(self) -> SparseTensor:
        return SparseTensor(SparseFormat.CSR, (self.out_features, self.in_features), self.values, crow=self.crow, col=self.col)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        rows = torch.repeat_interleave(torch.arange(self.out_features, device=self.values.device), self.crow[1:] - self.crow[:-1])
        w = torch.sparse_coo_tensor(torch.stack([rows, self.col]), self.values, (self.out_features, self.in_features))
        y = torch.sparse.mm(w, x.reshape(-1, self.in_features).t()).t()          # differentiable w.r.t. values and x
        y = y.reshape(*x.shape[:-1], self.out_features)
        return y + self.bias if self.bias is not None else y

    def prune_weights(self, new_sparsity: float) -> None:
        self._set_pattern(MagnitudePruner(new_sparsity).prune(self.weight().to_dense().detach()))

    def sparsity(self) -> float:
        return 1.0 - self.values.numel() / (self.in_features * self.out_features)

    def memory_efficiency(self) -> float:
        return self.weight().memory_usage() / (self.in_features * self.out_features * self.values.element_size())


class SparseConv2d(nn.Module):
    """Conv2d with a pruning mask (filter- or weight-level); the masked weight feeds the dense convolution."""

    def __init__(self, in_ch: int, out_ch: int, kernel_size, stride=1, padding=0, sparsity: float = 0.5, structured: bool = False):
        super().__init__()
        self.conv = nn.Conv2d(in_ch, out_ch, kernel_size, stride, padding)
        pr = StructuredPruner(sparsity, StructuredGranularity.CHANNEL) if structured else MagnitudePruner(sparsity)
        self.register_buffer("mask", pr.mask(self.conv.weight.detach()).clone())

    @classmethod
    def from_dense(cls, conv: nn.Conv2d, sparsity: float, structured: bool = False) -> "SparseConv2d":
        m = cls(conv.in_channels, conv.out_channels, conv.kernel_size, conv.stride, conv.padding, sparsity, structured)
        m.conv.load_state_dict(conv.state_dict())
        pr = StructuredPruner(sparsity, StructuredGranularity.CHANNEL) if structured else MagnitudePruner(sparsity)
        m.mask = pr.mask(m.conv.weight.detach()).clone()
        return m

    def forward(self, x):
        return F.conv2d(x, self.conv.weight * self.mask, self.conv.bias, self.conv.stride, self.conv.padding)

    def filter_sparsity(self) -> List[float]:
        return (1.0 - self.mask.float().reshape(self.mask.shape[0], -1).mean(1)).tolist()


class SparseEmbedding(nn.Module):
    """Embedding whose gradient is a sparse tensor (only the looked-up rows)."""

    def __init__(self, num_embeddings: int, embedding_dim: int):
        super().__init__()
        self.emb = nn.Embedding(num_embeddings, embedding_dim, sparse=True)

    def forward(self, idx):
        return self.emb(idx)


class SparseAttention(nn.Module):
    """Multi-head attention restricted to a sparse pattern ``mask [T, T]`` (a ``SparseTensor`` or bool tensor)."""

    def __init__(self, embed_dim: int, num_heads: int):
        super().__init__()
        self.h, self.d = num_heads, embed_dim // num_heads
        self.qkv = nn.Linear(embed_dim, 3 * embed_dim)
        self.out = nn.Linear(embed_dim, embed_dim)
        self.mask: Optional[torch.Tensor] = None

    def set_attention_mask(self, mask) -> None:
        self.mask = (mask.to_dense() != 0) if isinstance(mask, SparseTensor) else mask.bool()

    @staticmethod
    def local_window_mask(T: int, window: int) -> torch.Tensor:
        i = torch.arange(T)
        return (i[:, None] - i[None, :]).abs() <= window

    def forward(self, x):
        B, T, E = x.shape
        q, k, v = self.qkv(x).view(B, T, 3, self.h, self.d).permute(2, 0, 3, 1, 4)
        m = self.mask.to(x.device) if self.mask is not None else None
        y = F.scaled_dot_product_attention(q, k, v, attn_mask=m)
        return self.out(y.transpose(1, 2).reshape(B, T, E))

    def attention_stats(self) -> Optional[Tuple[float, int]]:
        if self.mask is None:
            return None
        return 1.0 - float(self.mask.float().mean()), int(self.mask.sum())


class SparseTransformerBlock(nn.Module):
    def __init__(self, embed_dim: int, num_heads: int, ff_dim: int, sparsity: float = 0.8, window: Optional[int] = None, seq_len: int = 0):
        super().__init__()
        self.attn = SparseAttention(embed_dim, num_heads)
        if window is not None and seq_len:
            self.attn.set_attention_mask(SparseAttention.local_window_mask(seq_len, window))
        self.n1, self.n2 = nn.LayerNorm(embed_dim), nn.LayerNorm(embed_dim)
        self.ff1, self.ff2 = SparseLinear(embed_dim, ff_dim, sparsity), SparseLinear(ff_dim, embed_dim, sparsity)

    def forward(self, x):
        x = x + self.attn(self.n1(x))
        return x + self.ff2(F.gelu(self.ff1(self.n2(x))))

    def sparsity_report(self) -> Dict[str, float]:
        r = {"ff1": self.ff1.sparsity(), "ff2": self.ff2.sparsity()}
        st = self.attn.attention_stats()
        if st:
            r["attention"] = st[0]
        return r


# ------------------------------------------------------------------------------ analysis / validation / IO
@dataclass
class SparsePatternAnalysis:
    nnz: int
    sparsity: float
    row_nnz_mean: float
    row_nnz_max: int
    empty_rows: int
    bandwidth: int
    diagonal_fraction: float

    def report(self) -> str:
        return (f"nnz={self.nnz} sparsity={self.sparsity:.4f} row nnz mean={self.row_nnz_mean:.2f} max={self.row_nnz_max} "
                f"empty rows={self.empty_rows} bandwidth={self.bandwidth} diagonal fraction={self.diagonal_fraction:.3f}")

    def optimization_recommendations(self) -> List[str]:
        recs = []
        if self.sparsity < 0.7:
            recs.append("sparsity below 70%: a dense GEMM on the tensor cores is likely faster")
        if self.row_nnz_max > 8 * max(1.0, self.row_nnz_mean):
            recs.append("row lengths are very uneven: prefer COO (or split long rows) for load balance")
        if self.empty_rows:
            recs.append(f"{self.empty_rows} empty rows: structured pruning could drop them from the layer")
        if self.diagonal_fraction > 0.5:
            recs.append("mostly (block-)diagonal: a banded / block format fits")
        return recs or ["CSR is a good fit"]


class SparseAnalyzer:
    @staticmethod
    def analyze_pattern(t: SparseTensor) -> SparsePatternAnalysis:
        c = t.to_coo()
        rows, cols = c.indices[0], c.indices[1]
        counts = torch.bincount(rows, minlength=t.shape[0])
        band = int((rows - cols).abs().max()) if t.nnz else 0
        return SparsePatternAnalysis(t.nnz, t.sparsity(), float(counts.float().mean()), int(counts.max()) if t.nnz else 0,
                                     int((counts == 0).sum()), band, float((rows == cols).float().mean()) if t.nnz else 0.0)

    @staticmethod
    def suggest_optimal_format(t: SparseTensor, row_access: bool = True) -> SparseFormat:
        return SparseFormat.CSR if row_access and len(t.shape) == 2 else SparseFormat.COO


class SparseValidator:
    @staticmethod
    def validate(t: SparseTensor) -> None:
        if t.format is SparseFormat.COO:
            if t.indices.shape != (len(t.shape), t.nnz):
                raise ValueError("COO index shape mismatch")
            for d, n in enumerate(t.shape):
                if t.nnz and (int(t.indices[d].min()) < 0 or int(t.indices[d].max()) >= n):
                    raise ValueError(f"COO index out of bounds along dim {d}")
        else:
            if int(t.crow[0]) != 0 or int(t.crow[-1]) != t.nnz or bool((t.crow[1:] < t.crow[:-1]).any()):
                raise ValueError("CSR row pointers must start at 0, end at nnz and be non-decreasing")
            if t.nnz and (int(t.col.min()) < 0 or int(t.col.max()) >= t.shape[1]):
                raise ValueError("CSR column index out of bounds")
        if not bool(torch.isfinite(t.values).all()):
            raise ValueError("non-finite values")


class SparseConverter:
    @staticmethod
    def convert(t: SparseTensor, fmt: SparseFormat) -> SparseTensor:
        return t.to_csr() if fmt is SparseFormat.CSR else t.to_coo()

    @staticmethod
    def batch_convert(ts: Sequence[SparseTensor], fmt: SparseFormat) -> List[SparseTensor]:
        return [SparseConverter.convert(t, fmt) for t in ts]


class SparseIO:
    """``"RTSP"`` · u8 format · u32 ndim · u64 dims · u64 nnz · int64 indices (COO) or crow+col (CSR) · fp32 values."""

    @staticmethod
    def save_binary(t: SparseTensor, path: str) -> None:
        with open(path, "wb") as f:
            f.write(b"RTSP" + struct.pack("<BI", 0 if t.format is SparseFormat.COO else 1, len(t.shape)))
            f.write(struct.pack(f"<{len(t.shape)}Q", *t.shape) + struct.pack("<Q", t.nnz))
            parts = [t.indices] if t.format is SparseFormat.COO else [t.crow, t.col]
            for p in parts:
                f.write(p.cpu().contiguous().numpy().astype("<i8").tobytes())
            f.write(t.values.detach().float().cpu().numpy().astype("<f4").tobytes())

    @staticmethod
    def load_binary(path: str) -> SparseTensor:
        import numpy as np
        with open(path, "rb") as f:
            if f.read(4) != b"RTSP":
                raise ValueError("not a sparse tensor file")
            fmt, nd = struct.unpack("<BI", f.read(5))
            shape = struct.unpack(f"<{nd}Q", f.read(8 * nd))
            (nnz,) = struct.unpack("<Q", f.read(8))
            rd = lambda n: torch.from_numpy(np.frombuffer(f.read(8 * n), dtype="<i8").copy())
            if fmt == 0:
                idx = rd(nd * nnz).reshape(nd, nnz)
                vals = torch.from_numpy(np.frombuffer(f.read(4 * nnz), dtype="<f4").copy())
                return SparseTensor.from_coo(idx, vals, shape)
            crow, col = rd(shape[0] + 1), rd(nnz)
            vals = torch.from_numpy(np.frombuffer(f.read(4 * nnz), dtype="<f4").copy())
            return SparseTensor.from_csr(crow, col, vals, shape)


@dataclass
class BenchmarkResult:
    name: str
    sparse_ms: float
    dense_ms: float

    @property
    def speedup(self) -> float:
        return self.dense_ms / self.sparse_ms if self.sparse_ms > 0 else 0.0


class SparseBenchmark:
    def __init__(self, iters: int = 10):
        self.iters = iters
        self.results: List[BenchmarkResult] = []

    def _time(self, fn) -> float:
        fn()
        sync = torch.cuda.synchronize if torch.cuda.is_available() else (lambda: None)
        sync()
        t0 = time.perf_counter()
        for _ in range(self.iters):
            fn()
        sync()
        return (time.perf_counter() - t0) / self.iters * 1e3

    def benchmark_spmv(self, t: SparseTensor, v: torch.Tensor) -> BenchmarkResult:
        return self.compare_with_dense(t, v.unsqueeze(1), "spmv")

    def compare_with_dense(self, t: SparseTensor, dense_rhs: torch.Tensor, name: str = "spmm") -> BenchmarkResult:
        sp, dn = t.to_csr().to_torch(), t.to_dense()
        r = BenchmarkResult(name, self._time(lambda: sp @ dense_rhs), self._time(lambda: dn @ dense_rhs))
        self.results.append(r)
        return r

    def report(self) -> str:
        return "\n".join(f"{r.name}: sparse {r.sparse_ms:.3f} ms, dense {r.dense_ms:.3f} ms, speedup {r.speedup:.2f}x" for r in self.results)
