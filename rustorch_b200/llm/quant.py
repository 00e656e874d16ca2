"""Quantised linear layers for the LLM runtime (GGUF Q4_0 / Q8_0 weights kept quantised on the device).

``QuantLinear`` stores the repacked nibbles / int8 values and the fp16 block scales and multiplies fp16
activations through the dequant-fused GEMV kernel (csrc/quant/q_gemv.cu).  On a machine without CUDA the
same object dequantises to fp32 and uses a plain matmul, which is also the oracle in the tests.
"""
from __future__ import annotations

import os

from typing import Optional, Tuple

import numpy as np
import torch

from .. import _native
from ..formats import gguf


class QuantLinear:
    def __init__(self, blocks: torch.Tensor, ggml_type: gguf.GGMLType, device=None):
        """``blocks``: uint8 ``[out_features, in_features / 32, 18 | 34]`` as stored in a GGUF file."""
        self.ggml_type = gguf.GGMLType(ggml_type)
        if self.ggml_type not in (gguf.GGMLType.Q4_0, gguf.GGMLType.Q8_0):
            raise ValueError("QuantLinear supports Q4_0 and Q8_0")
        self.q8 = self.ggml_type is gguf.GGMLType.Q8_0
        self.out_features, nb, bb = blocks.shape
        assert bb == (34 if self.q8 else 18), "block byte size does not match the type"
        self.in_features = nb * 32
        dev = torch.device(device) if device is not None else blocks.device
        self.device = dev
        if dev.type == "cuda":
            C = _native.load(required=True)
            b = blocks.to(dev).contiguous()
            self.scales = torch.empty((self.out_features, nb), dtype=torch.float16, device=dev)
            self.qs = torch.empty((self.out_features, nb, 32 if self.q8 else 16), dtype=torch.int8 if self.q8 else torch.uint8,
                                  device=dev)
            C.repack_quant(b, self.qs, self.scales, self.q8)
            self.blocks = None
        else:
            self.blocks = blocks.contiguous()
            self.qs = self.scales = None

    # ------------------------------------------------------------ constructors
    @classmethod
    def from_float(cls, weight: torch.Tensor, ggml_type: gguf.GGMLType = gguf.GGMLType.Q4_0, device=None) -> "QuantLinear":
        w = weight.detach().float().cpu().numpy()
        q = gguf.quantize_q8_0(w) if gguf.GGMLType(ggml_type) is gguf.GGMLType.Q8_0 else gguf.quantize_q4_0(w)
        return cls(torch.from_numpy(q), ggml_type, device or weight.device)

    @classmethod
    def random(cls, out_features: int, in_features: int, ggml_type: gguf.GGMLType = gguf.GGMLType.Q4_0, std: float = 0.02,
               device="cpu", seed: int = 0) -> "QuantLinear":
        """Synthetic quantised weights, statistically like quantising N(0, std) (random nibbles + the scale
        that maps the extreme code to ~3.3 sigma), generated directly in block form on the target device."""
        dev = torch.device(device)
        g = torch.Generator(device=dev).manual_seed(seed)
        nb = in_features // 32
        q8 = gguf.GGMLType(ggml_type) is gguf.GGMLType.Q8_0
        bb = 34 if q8 else 18
        blocks = torch.randint(0, 256, (out_features, nb, bb), dtype=torch.uint8, device=dev, generator=g)
        d = (torch.rand(out_features, nb, device=dev, generator=g) * 0.2 + 0.9) * (std * 3.3 / (127 if q8 else 8))
        blocks[..., :2] = d.to(torch.float16).view(torch.uint8).reshape(out_features, nb, 2)
        return cls(blocks, ggml_type, dev)

    # ------------------------------------------------------------------ compute
    # From this many activation rows on, expanding the weights (0.56 B read + 2 B written + 2 B re-read per
    # weight) costs less than re-streaming the quantised matrix once per 8 rows through the GEMV kernel.
    GEMM_MIN_ROWS = 64
    # Between these row counts the dequant-fused tcgen05 GEMM reads the quantised weights once for all rows
    # (the GEMV kernel's per-row arithmetic makes it slower from 5 rows on, and it re-reads the weights for every
    # 8 rows; the two-pass path moves 4.5 B per weight).
    TC_MIN_ROWS, TC_MAX_ROWS = 5, 256
    # 0: expanded weights in tensor memory (default); 1: staged in shared memory (RUSTORCH_QGEMM_PATH overrides)
    TC_PATH = int(os.environ.get("RUSTORCH_QGEMM_PATH", "0"))
    _scratch_buf = {}
    _tc_scratch = {}

    def _tc_buffers(self, rows: int):
        """Split-K scratch of the fused GEMM: fp32 partial sums (grown on demand) and zeroed per-tile counters that
        every call leaves zeroed; shared by all layers of a device (kernels on one stream run in order)."""
        C = _native.load(required=True)
        need, ncnt, splits = C.q_gemm_tc_scratch(rows, self.out_features, self.in_features, self.q8)
        if splits == 1:
            return None, None
        key = (self.device.type, self.device.index)
        part, cnt = QuantLinear._tc_scratch.get(key, (None, None))
        if part is None or part.numel() < need or cnt.numel() < ncnt:
            part = torch.empty(max(need, 1 << 22), dtype=torch.float32, device=self.device)
            cnt = torch.zeros(max(ncnt, 4096), dtype=torch.int32, device=self.device)
            QuantLinear._tc_scratch[key] = (part, cnt)
        return part, cnt

    def _scratch(self, numel: int) -> torch.Tensor:
        """One fp16 expansion buffer per device, grown to the largest matrix seen (kernels on one stream run in
        order, so consecutive layers can share it)."""
        key = (self.device.type, self.device.index)
        buf = QuantLinear._scratch_buf.get(key)
        if buf is None or buf.numel() < numel:
            buf = torch.empty(numel, dtype=torch.float16, device=self.device)
            QuantLinear._scratch_buf[key] = buf
        return buf[:numel]

    def dequantize(self) -> torch.Tensor:
        """fp32 ``[out, in]`` weights (decoded from the stored representation)."""
        if self.blocks is not None:
            arr = self.blocks.numpy()
            w = gguf.dequantize_q8_0(arr) if self.q8 else gguf.dequantize_q4_0(arr)
            return torch.from_numpy(w)
        d = self.scales.float().unsqueeze(-1)
        if self.q8:
            return (self.qs.float() * d).reshape(self.out_features, self.in_features)
        words = self.qs.view(torch.int32).to(torch.int64) & 0xFFFFFFFF            # [N, nb, 4]
        out = torch.empty(self.out_features, self.in_features // 32, 32, dtype=torch.float32, device=self.device)
        for e in range(8):
            shift = 16 + 4 * (e >> 1) if e & 1 else 4 * (e >> 1)
            out[..., e::8] = (((words >> shift) & 0xF).float() - 8.0)
        # out[..., e::8] picks positions e, 8+e, 16+e, 24+e = word index 0..3 at element e  ->  weight 8*i + e
        return (out * d).reshape(self.out_features, self.in_features)

    def __call__(self, x: torch.Tensor, residual: Optional[torch.Tensor] = None) -> torch.Tensor:
        """``x [..., in]`` -> ``[..., out]`` (fp16 on CUDA)."""
        shp = x.shape[:-1]
        x2 = x.reshape(-1, self.in_features)
        if self.device.type == "cuda":
            C = _native.load(required=True)
            x2 = x2.to(torch.float16).contiguous()
            r = residual.reshape(-1, self.out_features) if residual is not None else None
            if self.TC_MIN_ROWS <= x2.shape[0] <= self.TC_MAX_ROWS:
                y = torch.empty((x2.shape[0], self.out_features), dtype=torch.float16, device=self.device)
                part, cnt = self._tc_buffers(x2.shape[0])
                C.q_gemm_tc(self.qs, self.scales, x2, y, None, r, self.q8, part, cnt, self.TC_PATH)
            elif x2.shape[0] >= self.GEMM_MIN_ROWS:
                # prefill / large batch: expand once to fp16 scratch, then the tcgen05 GEMM (fp32 accumulate + output)
                w = self._scratch(self.out_features * self.in_features).view(self.out_features, self.in_features)
                C.dequant_f16(self.qs, self.scales, w, self.q8)
                acc = torch.empty((x2.shape[0], self.out_features), dtype=torch.float32, device=self.device)
                C.gemm(x2, False, w, False, acc, None, None, 0, 1.0, False, 1, 0)
                if r is not None:
                    acc += r
                y = acc.to(torch.float16)
            else:
                y = torch.empty((x2.shape[0], self.out_features), dtype=torch.float16, device=self.device)
                C.q_gemv(self.qs, self.scales, x2, y, None, r, self.q8)
        else:
            y = x2.float() @ self.dequantize().t()
            if residual is not None:
                y = y + residual.reshape(-1, self.out_features).float()
            y = y.to(x.dtype)
        return y.reshape(*shp, self.out_features)

    FUSED_MAX_ROWS = 4 if os.environ.get("RUSTORCH_DECODE_FUSED", "1") != "0" else 0

    PREFETCH_NEXT = os.environ.get("RUSTORCH_DECODE_PREFETCH", "1") != "0"
    # rotary embedding + cache append in the q | k | v projection's epilogue: one launch per layer less, but measured
    # slower (571.7 against 587.8 tokens/s at batch 1: the rotation runs on one lane per warp at the kernel's tail), so
    # it is opt-in
    ROPE_FUSED = os.environ.get("RUSTORCH_DECODE_ROPE_FUSED", "0") == "1"

    def fused(self, x: torch.Tensor, norm_w: Optional[torch.Tensor] = None, eps: float = 1e-5,
              residual: Optional[torch.Tensor] = None, swiglu: bool = False,
              prefetch: Optional["QuantLinear"] = None, rope: Optional[dict] = None) -> torch.Tensor:
        """``epilogue(W @ rmsnorm(x))`` for ``x [n, in]``: ``norm_w`` applies RMSNorm to ``x`` first, ``residual`` is
        added to the result, ``swiglu`` treats the rows of ``W`` as ``[gate; up]`` and returns ``silu(gate) * up``
        (``out_features / 2`` columns).  Up to ``FUSED_MAX_ROWS`` rows on CUDA this is ONE kernel (decode steps);
        otherwise the same arithmetic through the separate kernels.  ``prefetch``: the projection that runs next; the
        kernel asks the L2 for its weights while it works, so HBM keeps streaming across the kernel boundary.  ``rope``
        (one-kernel path only): ``dict(pos, seq, cache_k, cache_v, n_head, theta)`` for a fused q | k | v projection."""
        n = x.shape[0]
        if (self.device.type == "cuda" and 1 <= n <= self.FUSED_MAX_ROWS and x.dtype == torch.float16
                and self.in_features % 64 == 0):
            C = _native.load(required=True)
            x2 = x if x.stride(-1) == 1 else x.contiguous()
            y = torch.empty((n, self.out_features // 2 if swiglu else self.out_features), dtype=torch.float16, device=self.device)
            pq = ps = None
            if prefetch is not None and self.PREFETCH_NEXT and prefetch.qs is not None:
                pq, ps = prefetch.qs, prefetch.scales        # the kernel pulls the next projection's weights towards L2
            if rope is not None:
                # [q; k; v] projection: rotate q and k by the tokens' positions and append k, v to the cache in the
                # kernel's epilogue (interleaved pairs only; the caller checks that)
                C.q_gemv_fused(self.qs, self.scales, x2, y, norm_w, float(eps), None, self.q8, False, pq, ps,
                               rope["pos"], rope["seq"], rope["cache_k"], rope["cache_v"], int(rope["n_head"]), float(rope["theta"]))
            else:
                C.q_gemv_fused(self.qs, self.scales, x2, y, norm_w, float(eps), residual, self.q8, swiglu, pq, ps)
            return y
        h = x
        if norm_w is not None:
            if self.device.type == "cuda":
                h = torch.empty_like(x)
                _native.load(required=True).rmsnorm_f16(x, norm_w, h, float(eps))
            else:
                xf = x.float()
                h = (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * norm_w.float()).to(x.dtype)
        y = self(h, residual=residual)
        if swiglu:
            ff = self.out_features // 2
            if self.device.type == "cuda":
                act = torch.empty((n, ff), dtype=y.dtype, device=y.device)
                _native.load(required=True).silu_mul(y[:, :ff], y[:, ff:], act)
                return act
            return torch.nn.functional.silu(y[:, :ff].float()).to(y.dtype) * y[:, ff:]
        return y

    def nbytes(self) -> int:
        return self.out_features * (self.in_features // 32) * (34 if self.q8 else 18)

    def shard_rows(self, rank: int, world: int) -> "QuantLinear":
        """Column-parallel shard: a contiguous slice of output rows."""
        n = self.out_features // world
        return self._slice(slice(rank * n, (rank + 1) * n), slice(None))

    def shard_cols(self, rank: int, world: int) -> "QuantLinear":
        """Row-parallel shard: a contiguous slice of input blocks."""
        nb = self.in_features // 32 // world
        return self._slice(slice(None), slice(rank * nb, (rank + 1) * nb))

    def _slice(self, rows, blks) -> "QuantLinear":
        new = object.__new__(QuantLinear)
        new.ggml_type, new.q8, new.device = self.ggml_type, self.q8, self.device
        if self.blocks is not None:
            new.blocks = self.blocks[rows, blks].contiguous()
            new.qs = new.scales = None
            new.out_features, nb = new.blocks.shape[0], new.blocks.shape[1]
        else:
            new.blocks = None
            new.qs, new.scales = self.qs[rows, blks].contiguous(), self.scales[rows, blks].contiguous()
            new.out_features, nb = new.scales.shape
        new.in_features = nb * 32
        return new
