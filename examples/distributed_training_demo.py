"""Data-parallel training step.  Launch with
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 examples/distributed_training_demo.py
(gloo on CPU, NCCL on GPUs).  Without a launcher it runs as a single rank."""
import _path  # noqa: F401
import os

import torch
import torch.distributed as dist

from rustorch_b200 import nn, optim
from rustorch_b200 import distributed as rdist

world = int(os.environ.get("WORLD_SIZE", "1"))
rank = int(os.environ.get("RANK", "0"))
cuda = torch.cuda.is_available()
if world > 1:
    dist.init_process_group("nccl" if cuda else "gloo")
dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0"))) if cuda else torch.device("cpu")
if cuda:
    torch.cuda.set_device(dev)
torch.manual_seed(0)                                    # same initial weights on every rank
model = nn.Sequential(nn.Linear(32, 64), nn.ReLU(), nn.Linear(64, 4)).to(dev)
ddp = rdist.DistributedDataParallel(model) if world > 1 else model
opt = optim.SGD(model.parameters(), lr=0.1)
g = torch.Generator().manual_seed(100 + rank)           # a different shard of data per rank
x, y = torch.randn(64, 32, generator=g).to(dev), torch.randn(64, 4, generator=g).to(dev)
for step in range(5):
    opt.zero_grad()
    loss = torch.nn.functional.mse_loss(ddp(x), y)
    loss.backward()
    if world > 1 and hasattr(ddp, "sync_gradients"):
        ddp.sync_gradients()
    opt.step()
    if rank == 0:
        print(f"step {step}: loss {float(loss):.4f}")
if world > 1:
    w0 = model[0].weight.detach().clone()
    dist.broadcast(w0, 0)
    assert torch.allclose(w0, model[0].weight.detach()), "ranks diverged"
    if rank == 0:
        print("weights identical on all ranks")
    dist.destroy_process_group()
