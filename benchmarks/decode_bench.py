#!/usr/bin/env python
"""GGUF-layout Llama decode benchmark: Q4_0 weights, fp16 activations / KV cache, greedy decoding.

    python benchmarks/decode_bench.py [--batch 1] [--prompt 512] [--new 256] [--model 7b]
    python -m torch.distributed.run --nproc-per-node N ... benchmarks/decode_bench.py --tp N

Weights are random Q4_0 blocks of the 7B Llama shape (32 layers, d 4096, 32 heads, FFN 11008, vocab 32000),
prompts are uniform random tokens.  Reports prefill time (TTFT) and decode tokens/s, device-timed with CUDA
events (max over ranks), and the fraction of the HBM roofline for batch 1 (weight bytes per token / time).
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--prompt", type=int, default=512)
    ap.add_argument("--new", type=int, default=256)
    ap.add_argument("--layers", type=int, default=32)
    ap.add_argument("--tp", type=int, default=1)
    ap.add_argument("--eager", action="store_true", help="launch every kernel from the host instead of replaying a CUDA graph")
    a = ap.parse_args()
    import torch.distributed as dist
    from rustorch_b200 import _native
    from rustorch_b200.llm import LlamaConfig, LlamaRuntime

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    cfg = LlamaConfig(n_layer=a.layers)
    rt = LlamaRuntime.random_init(cfg, dev, tp_rank=rank, tp_world=world, seed=0)
    B, T, N = a.batch, a.prompt, a.new
    gen = torch.Generator().manual_seed(0)
    prompts = torch.randint(0, cfg.vocab_size, (B, T), generator=gen).to(dev)
    cache = rt.new_cache(B, T + N + 8)
    # warm-up
    lg = rt.prefill(prompts, cache)
    for _ in range(3):
        lg = rt.decode_step(lg.argmax(-1), cache)
    launches_per_step = 0
    graph = None
    if not a.eager:
        lc0 = _native.launch_count()
        graph = rt.capture_decode_graph(cache, B)     # one decode step (all layers + lm_head + argmax) as a CUDA graph
        launches_per_step = (_native.launch_count() - lc0) // 2      # warm-up pass + captured pass
    cache.clear()
    torch.cuda.synchronize()
    e = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
    l0 = _native.launch_count()
    e[0].record()
    logits = rt.prefill(prompts, cache)
    nxt = logits.argmax(-1)
    e[1].record()
    if a.eager:
        for _ in range(N - 1):
            nxt = rt.decode_step(nxt, cache).argmax(-1)
    else:
        graph.tok.copy_(nxt)
        graph.pos.fill_(T)
        graph.step.zero_()
        for _ in range(N - 1):
            graph.graph.replay()
    e[2].record()
    torch.cuda.synchronize()
    t = torch.tensor([e[0].elapsed_time(e[1]), e[1].elapsed_time(e[2])], device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ttft_ms, dec_ms = float(t[0]), float(t[1])
    _native.check_status()
    tok_s = B * (N - 1) / (dec_ms / 1e3)
    peaks = os.path.join(ROOT, "MEASURED_PEAKS.json")
    hbm = json.load(open(peaks))["hbm_gbs"] * 1e9 if os.path.exists(peaks) else 6.65e12
    per_tok_s = dec_ms / 1e3 / (N - 1)
    out = {"metric": "gguf_q4_0_decode_tokens_per_s", "value": round(tok_s, 1), "unit": "tokens/s", "n_gpus": world,
           "batch": B, "prompt": T, "new_tokens": N, "ttft_ms": round(ttft_ms, 2), "ms_per_token": round(per_tok_s * 1e3, 4),
           "weight_bytes_per_rank": rt.weight_bytes(),
           "hbm_roofline_frac": round(rt.weight_bytes() / per_tok_s / hbm, 3),
           "gpu_launches": _native.launch_count() - l0 + launches_per_step * (N - 1 if graph else 0), "layers": a.layers,
           "decode_loop": "eager" if a.eager else "cuda_graph",
           "config": "llama-7b shape, Q4_0 random weights, fp16 KV cache, greedy", "parallelism": f"tp{world}"}
    if rank == 0:
        print(json.dumps(out), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
