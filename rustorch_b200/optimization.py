"""Hardware- and platform-dependent tuning hints (src/optimization/*: ``HardwareOptimizer`` caps / tile sizes /
layout, ``PlatformOptimizer``, ``SimdOptimizer``).

The reference tunes CPU SIMD widths and cache tiles.  Here the same objects describe the B200 the process runs on
(SM count, shared memory, L2, TMEM) and derive the tile and grid choices the native kernels use, so that user code can
size its own launches consistently; on a CPU-only host they fall back to the CPU figures.
"""
from __future__ import annotations

import os
import platform
from dataclasses import dataclass, field
from typing import Dict, Tuple

import torch


@dataclass
class HardwareCapabilities:
    device: str
    sms: int = 0
    smem_per_block: int = 0
    l2_bytes: int = 0
    tmem_columns: int = 0
    memory_bytes: int = 0
    cpu_threads: int = 1
    simd: Dict[str, bool] = field(default_factory=dict)


class SimdOptimizer:
    """Vector widths: 16-byte accesses on the device (8 x 16-bit / 4 x 32-bit), host SIMD flags from cpuinfo."""

    def __init__(self):
        self.flags: Dict[str, bool] = {}
        try:
            import cpuinfo
            f = set(cpuinfo.get_cpu_info().get("flags", []))
            self.flags = {"sse2": "sse2" in f, "avx2": "avx2" in f, "avx512f": "avx512f" in f, "fma": "fma" in f, "neon": "neon" in f}
        except Exception:  # noqa: BLE001
            pass

    def vector_width(self, dtype: torch.dtype, device: str = "cuda") -> int:
        size = torch.empty((), dtype=dtype).element_size()
        if device == "cuda":
            return 16 // size
        lanes = 64 if self.flags.get("avx512f") else 32 if self.flags.get("avx2") else 16
        return lanes // size

    def is_aligned(self, t: torch.Tensor) -> bool:
        return t.data_ptr() % 16 == 0 and (t.numel() * t.element_size()) % 16 == 0


class PlatformOptimizer:
    def __init__(self):
        self.os, self.arch = platform.system().lower(), platform.machine().lower()
        self.cpu_threads = os.cpu_count() or 1

    def optimal_thread_count(self, work_items: int) -> int:
        return max(1, min(self.cpu_threads, work_items))

    def pinned_memory_recommended(self) -> bool:
        return torch.cuda.is_available()

    def features(self) -> Dict[str, object]:
        return {"os": self.os, "arch": self.arch, "cpu_threads": self.cpu_threads, "cuda": torch.cuda.is_available()}


class HardwareOptimizer:
    def __init__(self, device_index: int = 0):
        self.simd, self.platform = SimdOptimizer(), PlatformOptimizer()
        if torch.cuda.is_available():
            p = torch.cuda.get_device_properties(device_index)
            blackwell = p.major >= 10
            self.caps = HardwareCapabilities(p.name, p.multi_processor_count, getattr(p, "shared_memory_per_block_optin", 227 * 1024),
                                             getattr(p, "L2_cache_size", 0), 512 if blackwell else 0, p.total_memory,
                                             self.platform.cpu_threads, self.simd.flags)
        else:
            self.caps = HardwareCapabilities("cpu", cpu_threads=self.platform.cpu_threads, simd=self.simd.flags)

    def gemm_tile(self, M: int, N: int, K: int) -> Tuple[int, int, int]:
        """(BLOCK_M, BLOCK_N, BLOCK_K) of the tcgen05 GEMM for a shape: 128 x 256 x 64, 128-wide N for narrow outputs."""
        return 128, (128 if N <= 128 else 256), 64

    def persistent_grid(self, tiles: int, ctas_per_sm: int = 1) -> int:
        """One CTA (or ``ctas_per_sm``) per SM, never more CTAs than tiles."""
        return max(1, min(tiles, max(1, self.caps.sms) * ctas_per_sm))

    def elementwise_grid(self, numel: int, vec: int = 8, threads: int = 256) -> int:
        work = -(-numel // (vec * threads))
        return max(1, min(work, 8 * max(1, self.caps.sms)))

    def preferred_layout(self, op: str) -> str:
        return "channels_last" if op in ("conv2d", "batch_norm", "pool2d") else "contiguous"

    def exceeds_l2(self, nbytes: int) -> bool:
        return self.caps.l2_bytes > 0 and nbytes > self.caps.l2_bytes

    def report(self) -> str:
        c = self.caps
        return (f"{c.device}: {c.sms} SMs, {c.smem_per_block // 1024} KB smem/block, L2 {c.l2_bytes // 2 ** 20} MB, "
                f"TMEM {c.tmem_columns} columns, {c.memory_bytes // 2 ** 30} GB; host {c.cpu_threads} threads {self.simd.flags}")
