"""Llama-style 8B decoder, tensor + sequence parallel bf16 training step (BASELINE config 4).

  python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
      benchmarks/llama_tp_bench.py --steps 5 --warmup 3 [--layers 32] [--seqs 8] [--seq-len 4096]

Every rank gets the same global batch (``--seqs`` sequences of ``--seq-len`` uniform random token ids); the model
is sharded over the N ranks with the fused all-gather->GEMM / GEMM->reduce-scatter kernels.
AdamW through the fused
flat optimizer.  Prints one JSON line (tokens/s of the whole job, device time, max over ranks).  ``--layers`` below 32
is for bring-up and is marked ``"reduced": true`` in the output.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--layers", type=int, default=32)
    ap.add_argument("--seqs", type=int, default=8)
    ap.add_argument("--seq-len", type=int, default=4096)
    ap.add_argument("--vocab", type=int, default=128256)
    ap.add_argument("--impl", default="ours", choices=["ours", "library"],
                    help="library: the same model and sharding on NCCL collectives + cuBLAS + SDPA + torch.optim.AdamW(fused=True)")
    ap.add_argument("--checkpoint", action="store_true", help="recompute each block in backward (activation checkpointing)")
    a = ap.parse_args()
    rank, world, local = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1)), int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    from rustorch_b200 import _native
    from rustorch_b200.models import llama as llama_mod
    from rustorch_b200.models.llama import LlamaModel, LlamaTrainConfig
    llama_mod.LIBRARY_MODE = a.impl == "library"
    llama_mod.CHECKPOINT_BLOCKS = a.checkpoint
    from rustorch_b200.optim.flat import FlatParams, FusedAdamW
    from rustorch_b200.utils.clocks import ClockSampler
    cfg = LlamaTrainConfig.llama3_8b()
    cfg.n_layer, cfg.vocab_size, cfg.max_seq_len = a.layers, a.vocab, a.seq_len
    torch.manual_seed(0)
    model = LlamaModel(cfg, device=dev, dtype=torch.bfloat16, tp_group=dist.group.WORLD if world > 1 else None, batch=a.seqs,
                       seq_len=a.seq_len)
    if a.impl == "library":
        opt = torch.optim.AdamW(model.parameters(), lr=3e-4, betas=(0.9, 0.95), weight_decay=0.1, fused=True)
    else:
        flat = FlatParams(model)
        opt = FusedAdamW(flat, lr=3e-4, betas=(0.9, 0.95), weight_decay=0.1)
    g = torch.Generator().manual_seed(1)
    idx = torch.randint(0, a.vocab, (a.seqs, a.seq_len), generator=g).to(dev)
    tgt = idx.roll(-1, 1)

    def step():
        _, loss = model(idx, tgt)
        loss.backward()
        model.sync_replicated_grads()
        opt.step()
        if a.impl == "library":
            opt.zero_grad(set_to_none=True)
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
    tokens = a.seqs * a.seq_len
    d, dkv, ff = 4096, 1024, 14336
    n_params = a.layers * (2 * d * d + 2 * d * dkv + 3 * d * ff + 2 * d) + 2 * a.vocab * d + d
    out = {"metric": "train_tokens_per_s", "value": round(tokens / (ms / 1e3), 1), "unit": "tokens/s", "n_gpus": world, "steps": a.steps,
           "warmup": a.warmup, "ms_per_step": round(ms, 3), "higher_is_better": True, "scaling": "strong", "dtype": "bf16", "impl": a.impl, "activation_checkpointing": bool(a.checkpoint),
           "data": "synthetic uniform random tokens, random-init weights", "reduced": a.layers != 32,
           "config": {"model": f"llama-8B style ({a.layers}L, d4096, 32q/8kv heads, SwiGLU 14336, vocab {a.vocab})", "global_batch": a.seqs,
                      "seq_len": a.seq_len, "parallelism": f"tp{world}+sp", "params": n_params},
           "clocks": clocks, "gpu_launches": _native.launch_count() - l0, "final_loss": round(float(loss.detach()), 4)}
    if rank == 0:
        print(json.dumps(out), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
