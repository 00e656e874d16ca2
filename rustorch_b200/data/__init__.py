"""Datasets, samplers and the batch loader (src/data/dataset.rs:15-215, src/data/dataloader.rs:17-115,
src/data/sampler.rs:12-314).

``DataLoader(dataset, sampler, batch_size)`` with ``next_batch() / reset() / is_empty()`` as in the
reference, plus Python iteration.  ``with_options`` adds ``num_workers`` (threaded prefetch),
``pin_memory`` (batches land in pinned host memory ready for an async host-to-device copy) and
``drop_last``.
"""
from __future__ import annotations

import threading
from typing import Callable, Iterator, List, Optional, Sequence, Tuple

import torch

from .._interop import IntValue


# ------------------------------------------------------------------- datasets
class Dataset:
    def __len__(self) -> int:
        raise NotImplementedError

    def __getitem__(self, index: int):
        raise NotImplementedError

    def len(self) -> int:
        return len(self)

    def get_item(self, index: int):
        return self[index]

    def is_empty(self) -> bool:
        return len(self) == 0


class IterableDataset:
    """A dataset that is only iterated, not indexed (src/data/dataset.rs)."""

    def __iter__(self):
        raise NotImplementedError


class TensorDataset(Dataset):
    """Tuples of rows from equally long tensors."""

    def __init__(self, *tensors):
        if len(tensors) == 1 and isinstance(tensors[0], (list, tuple)):
            tensors = tuple(tensors[0])
        tensors = tuple(getattr(t, "data", t) if not isinstance(t, torch.Tensor) else t for t in tensors)
        if not tensors:
            raise ValueError("TensorDataset needs at least one tensor")
        n = tensors[0].shape[0]
        if any(t.shape[0] != n for t in tensors):
            raise ValueError("all tensors must have the same first dimension")
        self.tensors = tensors

    @classmethod
    def from_features_targets(cls, features, targets) -> "TensorDataset":
        return cls(features, targets)

    @classmethod
    def from_tensors(cls, tensors) -> "TensorDataset":
        return cls(*tensors)

    def __len__(self):
        return self.tensors[0].shape[0]

    def __getitem__(self, i):
        if not -len(self) <= i < len(self):
            raise IndexError(f"index {i} outside a dataset of {len(self)}")
        return tuple(t[i] for t in self.tensors)

    def get_batch(self, indices: Sequence[int]):
        """One entry per tensor of the dataset, each the rows ``indices`` stacked (src/python/data.rs get_batch)."""
        idx = torch.as_tensor(list(indices), dtype=torch.long)
        return tuple(t[idx.to(t.device)] for t in self.tensors)

    # first / last tensor under the names of the Python binding; attribute or call (src/python/data.rs)
    @property
    def data(self):
        from ..tensor import Tensor
        return Tensor(self.tensors[0])

    @property
    def targets(self):
        from ..tensor import Tensor
        return Tensor(self.tensors[-1])


class ConcatDataset(Dataset):
    """Several datasets end to end (src/data/dataset.rs)."""

    def __init__(self, datasets: Sequence[Dataset]):
        self.datasets = list(datasets)
        self.offsets = []
        n = 0
        for d in self.datasets:
            self.offsets.append(n)
            n += len(d)
        self._len = n

    def __len__(self):
        return self._len

    def __getitem__(self, i):
        if i < 0 or i >= self._len:
            raise IndexError(i)
        for d, off in zip(reversed(self.datasets), reversed(self.offsets)):
            if i >= off:
                return d[i - off]
        raise IndexError(i)


# ------------------------------------------------------------------- samplers
class Sampler:
    def sample(self) -> Optional[int]:
        raise NotImplementedError

    def reset(self) -> None:
        raise NotImplementedError

    def __len__(self) -> int:
        raise NotImplementedError

    def is_empty(self) -> bool:
        return len(self) == 0

    def __iter__(self) -> Iterator[int]:
        self.reset()
        while True:
            i = self.sample()
            if i is None:
                return
            yield i


class _ListSampler(Sampler):
    def __init__(self):
        self._order: List[int] = []
        self._pos = 0

    def _make_order(self) -> List[int]:
        raise NotImplementedError

    def reset(self):
        self._order = self._make_order()
        self._pos = 0

    def sample(self):
        if not self._order and self._pos == 0:
            self.reset()
        if self._pos >= len(self._order):
            return None
        i = self._order[self._pos]
        self._pos += 1
        return i

    def __len__(self):
        return len(self._make_order()) if not self._order else len(self._order)


class SequentialSampler(_ListSampler):
    """Indices ``0 .. len - 1`` in order (src/data/sampler.rs:33-60)."""

    def __init__(self, data_len: int):
        super().__init__()
        self.data_len = data_len

    def _make_order(self):
        return list(range(self.data_len))


class RandomSampler(_ListSampler):
    """``RandomSampler(len)``, ``with_replacement(len, n)``, ``with_seed(len, seed)``."""

    def __init__(self, data_len: int, replacement: bool = False, num_samples: Optional[int] = None,
                 seed: Optional[int] = None):
        super().__init__()
        self.data_len, self.replacement = data_len, replacement
        self.num_samples = num_samples if num_samples is not None else data_len
        self._gen = torch.Generator()
        if seed is not None:
            self._gen.manual_seed(seed)

    with_replacement = classmethod(lambda cls, n, num_samples: cls(n, True, num_samples))
    with_seed = classmethod(lambda cls, n, seed: cls(n, seed=seed))

    def _make_order(self):
        if self.replacement:
            return torch.randint(0, self.data_len, (self.num_samples,), generator=self._gen).tolist()
        return torch.randperm(self.data_len, generator=self._gen)[: self.num_samples].tolist()

    def __len__(self):
        return self.num_samples


class SubsetRandomSampler(_ListSampler):
    """A random permutation of the given indices (src/data/sampler.rs)."""

    def __init__(self, indices: Sequence[int], seed: Optional[int] = None):
        super().__init__()
        self.indices = list(indices)
        self._gen = torch.Generator()
        if seed is not None:
            self._gen.manual_seed(seed)

    def _make_order(self):
        return [self.indices[i] for i in torch.randperm(len(self.indices), generator=self._gen).tolist()]

    def __len__(self):
        return len(self.indices)


class WeightedRandomSampler(_ListSampler):
    """``num_samples`` indices drawn in proportion to ``weights``, with or without replacement (src/data/sampler.rs)."""

    def __init__(self, weights: Sequence[float], num_samples: int, replacement: bool = True, seed: Optional[int] = None):
        super().__init__()
        self.weights = torch.as_tensor(weights, dtype=torch.double)
        if (self.weights < 0).any() or float(self.weights.sum()) <= 0:
            raise ValueError("weights must be non-negative with a positive sum")
        self.num_samples, self.replacement = num_samples, replacement
        self._gen = torch.Generator()
        if seed is not None:
            self._gen.manual_seed(seed)

    def _make_order(self):
        return torch.multinomial(self.weights, self.num_samples, self.replacement, generator=self._gen).tolist()

    def __len__(self):
        return self.num_samples


class BatchSampler:
    """Groups another sampler's indices into lists of ``batch_size``."""

    def __init__(self, sampler: Sampler, batch_size: int, drop_last: bool = False):
        if batch_size <= 0:
            raise ValueError("batch_size must be positive")
        self.sampler, self.batch_size, self.drop_last = sampler, batch_size, drop_last

    def __iter__(self):
        batch = []
        for i in self.sampler:
            batch.append(i)
            if len(batch) == self.batch_size:
                yield batch
                batch = []
        if batch and not self.drop_last:
            yield batch

    def __len__(self):
        n = len(self.sampler)
        return n // self.batch_size if self.drop_last else -(-n // self.batch_size)


# --------------------------------------------------------------------- loader
def default_collate(items: List):
    first = items[0]
    if isinstance(first, torch.Tensor):
        return torch.stack(items)
    if isinstance(first, (tuple, list)):
        return type(first)(default_collate([it[k] for it in items]) for k in range(len(first)))
    if isinstance(first, dict):
        return {k: default_collate([it[k] for it in items]) for k in first}
    return torch.as_tensor(items)


def _pin(x):
    if isinstance(x, torch.Tensor):
        return x.pin_memory() if torch.cuda.is_available() and not x.is_cuda else x
    if isinstance(x, (tuple, list)):
        return type(x)(_pin(v) for v in x)
    if isinstance(x, dict):
        return {k: _pin(v) for k, v in x.items()}
    return x


class DataLoader:
    def __init__(self, dataset: Dataset, sampler: Optional[Sampler] = None, batch_size: int = 1,
                 drop_last: bool = False, num_workers: int = 0, pin_memory: bool = False,
                 collate_fn: Callable = default_collate, shuffle: bool = False, prefetch: int = 2):
        self.dataset = dataset
        self.sampler = sampler or (RandomSampler(len(dataset)) if shuffle else SequentialSampler(len(dataset)))
        if int(batch_size) <= 0:
            raise ValueError("batch_size must be positive")
        self._batch_size, self.drop_last = int(batch_size), drop_last
        self.num_workers, self.pin_memory, self.collate_fn, self.prefetch = num_workers, pin_memory, collate_fn, prefetch
        self._it: Optional[Iterator] = None
        self._served = 0

    @property
    def batch_size(self) -> int:
        """Attribute, or ``loader.batch_size()`` as in the Python binding."""
        return IntValue(self._batch_size)

    @batch_size.setter
    def batch_size(self, n: int) -> None:
        self._batch_size = int(n)

    @classmethod
    def with_options(cls, dataset, sampler, batch_size, drop_last=False, num_workers=0, pin_memory=False,
                     collate_fn=default_collate) -> "DataLoader":
        return cls(dataset, sampler, batch_size, drop_last, num_workers, pin_memory, collate_fn)

    def _load(self, idx: List[int]):
        b = self.collate_fn([self.dataset[i] for i in idx])
        return _pin(b) if self.pin_memory else b

    def _batches(self):
        for idx in BatchSampler(self.sampler, self.batch_size, self.drop_last):
            yield idx

    def __iter__(self):
        if self.num_workers <= 0:
            for idx in self._batches():
                yield self._load(idx)
            return
        # threaded prefetch that preserves batch order; the workers stay at most ``prefetch * num_workers`` batches
        # ahead of the consumer, and stop when the consumer abandons the iterator
        window = max(1, self.prefetch) * self.num_workers
        index_list = list(self._batches())
        results = {}
        cond = threading.Condition()
        state = {"next": 0, "consumed": 0, "stop": False, "error": None}

        def worker():
            while True:
                with cond:
                    while not state["stop"] and state["next"] < len(index_list) and state["next"] - state["consumed"] >= window:
                        cond.wait()
                    if state["stop"] or state["next"] >= len(index_list):
                        return
                    j = state["next"]
                    state["next"] += 1
                try:
                    b = self._load(index_list[j])
                except BaseException as e:  # noqa: BLE001  (handed to the consumer, which re-raises it)
                    with cond:
                        state["error"], state["stop"] = e, True
                        cond.notify_all()
                    return
                with cond:
                    results[j] = b
                    cond.notify_all()

        threads = [threading.Thread(target=worker, daemon=True) for _ in range(self.num_workers)]
        for t in threads:
            t.start()
        try:
            for j in range(len(index_list)):
                with cond:
                    while j not in results and state["error"] is None:
                        cond.wait()
                    if state["error"] is not None:
                        raise state["error"]
                    b = results.pop(j)
                    state["consumed"] = j + 1
                    cond.notify_all()
                yield b
        finally:
            with cond:
                state["stop"] = True
                cond.notify_all()

    def __len__(self):
        return len(BatchSampler(self.sampler, self.batch_size, self.drop_last))

    # reference-style stepping API
    def next_batch(self):
        if self._it is None:
            self._it = iter(self)
            self._served = 0
        try:
            b = next(self._it)
            self._served += 1
            return b
        except StopIteration:
            self._it = None
            return None

    def reset(self) -> None:
        self._it = None
        self._served = 0

    def num_batches(self) -> int:
        return len(self)

    def current_batch_index(self) -> int:
        """Batches handed out by ``next_batch`` since the last ``reset``."""
        return self._served

    def has_next(self) -> bool:
        return self._served < len(self)

    def is_empty(self) -> bool:
        return len(self.dataset) == 0


__all__ = ["Dataset", "IterableDataset", "TensorDataset", "ConcatDataset", "Sampler", "SequentialSampler",
           "RandomSampler", "SubsetRandomSampler", "WeightedRandomSampler", "BatchSampler", "DataLoader",
           "default_collate"]
