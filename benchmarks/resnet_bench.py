"""ResNet-18 image classifier, data-parallel bf16 training (BASELINE config 2).

  python benchmarks/resnet_bench.py --steps 10 --warmup 3 [--batch 256] [--impl ours|library]
  python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P benchmarks/resnet_bench.py ...

Input 3x224x224 i.i.d. N(0,1), labels uniform in [0, 1000), per-GPU batch 256, SGD momentum 0.9 lr 0.1 wd 1e-4.
``ours``: channels-last bf16 model on this framework's kernels: implicit-GEMM tcgen05 convolutions (forward, weight
gradient, stride-1 input gradient; the 3-channel stem and the strided input gradients use the library), BatchNorm
(+ residual + ReLU fused), fused flat SGD; on more than one GPU the fused data-parallel bucket kernel (reduce + SGD
momentum + parameter broadcast over peer memory, overlapped with backward).  ``library``: the same topology from stock ``torch.nn``
modules + ``torch.optim.SGD`` + PyTorch DDP.  Prints one JSON line: images/s of the whole job, device time,
max over ranks.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


class _StockBlock(nn.Module):
    def __init__(self, i, o, stride):
        super().__init__()
        self.c1, self.b1 = nn.Conv2d(i, o, 3, stride, 1, bias=False), nn.BatchNorm2d(o)
        self.c2, self.b2 = nn.Conv2d(o, o, 3, 1, 1, bias=False), nn.BatchNorm2d(o)
        self.down = None if stride == 1 and i == o else nn.Sequential(nn.Conv2d(i, o, 1, stride, bias=False), nn.BatchNorm2d(o))

    def forward(self, x):
        idt = x if self.down is None else self.down(x)
        return F.relu(self.b2(self.c2(F.relu(self.b1(self.c1(x))))) + idt)


def stock_resnet18(num_classes=1000) -> nn.Module:
    """The same topology from stock ``torch.nn`` modules (cuDNN convolutions and BatchNorm): the library arm."""
    layers, i = [nn.Conv2d(3, 64, 7, 2, 3, bias=False), nn.BatchNorm2d(64), nn.ReLU(), nn.MaxPool2d(3, 2, 1)], 64
    for o, stride in ((64, 1), (64, 1), (128, 2), (128, 1), (256, 2), (256, 1), (512, 2), (512, 1)):
        layers.append(_StockBlock(i, o, stride))
        i = o
    return nn.Sequential(*layers, nn.AdaptiveAvgPool2d(1), nn.Flatten(), nn.Linear(512, num_classes))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--batch", type=int, default=256)
    ap.add_argument("--impl", default="ours", choices=["ours", "library"])
    a = ap.parse_args()
    rank, world, local = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1)), int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    from rustorch_b200 import _native
    from rustorch_b200.models import cnn
    from rustorch_b200.utils.clocks import ClockSampler
    torch.manual_seed(0)
    model = (cnn.resnet18(1000) if a.impl == "ours" else stock_resnet18(1000)).to(dev).to(memory_format=torch.channels_last)
    x = torch.randn(a.batch, 3, 224, 224, device=dev).to(torch.bfloat16).contiguous(memory_format=torch.channels_last)
    y = torch.randint(0, 1000, (a.batch,), device=dev)
    if a.impl == "ours":
        model = model.to(torch.bfloat16)
        from rustorch_b200.optim.flat import FlatParams, FusedSGD
        if world > 1:
            # one fused kernel per 25 MB bucket: reduce over NVLink (NVLS where available) + SGD momentum + parameter
            # broadcast, launched from gradient hooks while backward is still running
            from rustorch_b200.distributed.fused_allreduce import FusedDDPSGD
            ddp = FusedDDPSGD(model, lr=0.1, momentum=0.9, weight_decay=1e-4, bucket_cap_mb=25.0,
                              decay_filter=lambda n, p: p.dim() > 1)

            def step():
                out = model(x)
                loss = F.cross_entropy(out.float(), y)
                loss.backward()
                ddp.step()
                return loss
        else:
            flat = FlatParams(model, decay_filter=lambda n, p: p.dim() > 1)
            opt = FusedSGD(flat, lr=0.1, momentum=0.9, weight_decay=1e-4)

            def step():
                out = model(x)
                loss = F.cross_entropy(out.float(), y)
                loss.backward()
                flat.collect_autograd_grads()
                opt.step()
                return loss
    else:
        model = model.to(torch.bfloat16)
        opt = torch.optim.SGD(model.parameters(), lr=0.1, momentum=0.9, weight_decay=1e-4)
        net = nn.parallel.DistributedDataParallel(model, device_ids=[local], bucket_cap_mb=25) if world > 1 else model

        def step():
            opt.zero_grad(set_to_none=True)
            loss = F.cross_entropy(net(x).float(), y)
            loss.backward()
            opt.step()
            return loss

    for _ in range(a.warmup):
        step()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    l0 = _native.launch_count()
    sampler = ClockSampler(local, 0.05)
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(a.steps):
        loss = step()
    e1.record()
    torch.cuda.synchronize()
    clocks = sampler.stop()
    t = torch.tensor([e0.elapsed_time(e1)], device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t) / a.steps
    _native.check_status()
    out = {"metric": "train_images_per_s", "value": round(a.batch * world / (ms / 1e3), 1), "unit": "images/s", "n_gpus": world,
           "steps": a.steps, "warmup": a.warmup, "ms_per_step": round(ms, 3), "higher_is_better": True, "scaling": "weak", "dtype": "bf16",
           "impl": a.impl, "data": "synthetic N(0,1) images, random-init weights",
           "config": {"model": "resnet18 (channels-last)", "per_gpu_batch": a.batch, "image": "3x224x224", "optimizer": "SGD m0.9 lr0.1 wd1e-4",
                      "parallelism": f"dp{world}", "convolutions": "implicit-GEMM tcgen05; stem as im2col + tcgen05 GEMM" if a.impl == "ours" else "cuDNN"},
           "clocks": clocks, "gpu_launches": _native.launch_count() - l0, "final_loss": round(float(loss), 4)}
    if rank == 0:
        print(json.dumps(out), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
