"""Datasets, samplers and loaders: batching, shuffling with a seed, weighted and subset sampling, the distributed
sampler's shards, worker threads with a bounded prefetch window."""
import _path  # noqa: F401
import time

import torch

import rustorch as rt
from rustorch_b200 import data as D
from rustorch_b200.distributed import DistributedSampler

ds = rt.TensorDataset(torch.arange(20.0).view(10, 2), torch.arange(10))
print("sequential batches:", [b[1].tolist() for b in rt.DataLoader(ds, batch_size=4)])
print("seeded shuffle    :", [b[1].tolist() for b in rt.DataLoader(ds, D.RandomSampler(len(ds), seed=3), batch_size=4)])
print("drop_last         :", [b[1].tolist() for b in rt.DataLoader(ds, batch_size=4, drop_last=True)])
print("subset [1, 3, 5]  :", sorted(D.SubsetRandomSampler([1, 3, 5])))
w = D.WeightedRandomSampler([0.0] * 9 + [1.0], 5, True)
print("all weight on item 9:", list(w))
for rank in range(2):
    s = DistributedSampler(10, 2, rank, seed=0)
    s.set_epoch(1)
    print(f"rank {rank} of 2 sees", s.get_indices())
loader = rt.DataLoader(ds, batch_size=3)
while loader.has_next():
    batch = loader.next_batch()
print("stepping API served", loader.current_batch_index(), "of", loader.num_batches(), "batches; last has", batch[0].shape[0], "rows")


class Slow(rt.Dataset):
    def __len__(self):
        return 32

    def __getitem__(self, i):
        time.sleep(0.01)
        return torch.tensor([float(i)])


for workers in (0, 4):
    t0 = time.time()
    n = sum(b.shape[0] for b in rt.DataLoader(Slow(), batch_size=4, num_workers=workers))
    print(f"{n} slow samples with {workers} workers: {time.time() - t0:.2f} s")
