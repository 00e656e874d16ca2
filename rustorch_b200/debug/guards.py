"""Canary-guarded buffers: a tensor carved out of a larger allocation with guard regions of a known byte pattern
before and after it; ``check()`` finds writes that ran past either end.  Meant for workspaces, staging and symmetric
buffers handed to kernels in tests (the CUDA sanitizers are not always available), on CPU and GPU alike.

The reference relies on Rust's bounds checks plus miri / valgrind in its nightly CI (.github/workflows/nightly.yml:79-99)
and has no device-side guard.
"""
from __future__ import annotations

import contextlib
from typing import Iterator, List, Sequence

import torch

from ..error import MemoryError_

_PATTERN = 0xA5


class GuardedTensor:
    """``GuardedTensor((rows, cols), torch.bfloat16, "cuda").tensor`` is an ordinary contiguous tensor; the bytes around
    it are watched."""

    def __init__(self, shape: Sequence[int], dtype: torch.dtype = torch.float32, device="cpu", guard_bytes: int = 256,
                 fill: float = 0.0):
        self.guard_bytes = int(guard_bytes)
        if self.guard_bytes % 16:
            raise ValueError("guard size must keep 16-byte alignment")
        itemsize = torch.empty((), dtype=dtype).element_size()
        numel = 1
        for s in shape:
            numel *= int(s)
        self.nbytes = numel * itemsize
        pad = (-self.nbytes) % 16                                   # keep the trailing guard 16-byte aligned too
        self._raw = torch.full((self.guard_bytes + self.nbytes + pad + self.guard_bytes,), _PATTERN, dtype=torch.uint8, device=device)
        self._pad = pad
        self.tensor = self._raw[self.guard_bytes:self.guard_bytes + self.nbytes].view(dtype).view(*shape)
        self.tensor.fill_(fill)

    def violations(self) -> List[int]:
        """Byte offsets relative to the start of the tensor (negative: before it) whose guard value changed."""
        head = self._raw[:self.guard_bytes]
        tail = self._raw[self.guard_bytes + self.nbytes:]
        bad = [int(i) - self.guard_bytes for i in torch.nonzero(head != _PATTERN).flatten().tolist()]
        bad += [self.nbytes + int(i) for i in torch.nonzero(tail != _PATTERN).flatten().tolist()]
        return bad

    def check(self, what: str = "buffer") -> None:
        bad = self.violations()
        if bad:
            raise MemoryError_(f"{what}: {len(bad)} guard byte(s) overwritten, first at offset {bad[0]} "
                               f"(tensor spans 0..{self.nbytes - 1})", offsets=bad[:16])


@contextlib.contextmanager
def guard_scope(*buffers: GuardedTensor) -> Iterator[Sequence[GuardedTensor]]:
    """Checks every buffer when the block ends (after a device synchronise when any of them lives on a GPU)."""
    yield buffers
    if any(b.tensor.is_cuda for b in buffers):
        torch.cuda.synchronize()
    for i, b in enumerate(buffers):
        b.check(f"guarded buffer {i}")
