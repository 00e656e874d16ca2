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
import torch.nn.functional as F

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


class _LibraryDecoder:
    """The same model on stock PyTorch kernels: the quantised weights expanded once to dense fp16 (what a runtime
    without quantised kernels has to do), cuBLAS matmuls, SDPA over the whole cache with a validity mask, eager RoPE /
    RMSNorm / SwiGLU, greedy argmax; one decode step captured in a CUDA graph like ours.  Single GPU."""

    def __init__(self, rt, batch: int, max_len: int):
        cfg = rt.cfg
        self.cfg, self.dev = cfg, rt.device
        self.H, self.Hkv, self.D = cfg.n_head, cfg.n_head_kv, cfg.head_dim
        dense = lambda q: q.dequantize().half()  # noqa: E731
        self.layers = [(dense(L.wqkv), dense(L.wo), dense(L.w_gate_up), dense(L.w_down), L.attn_norm, L.ffn_norm) for L in rt.layers]
        self.tok_emb, self.out_norm, self.lm_head = rt.tok_emb, rt.out_norm, dense(rt.lm_head)
        self.k = torch.zeros(cfg.n_layer, batch, self.Hkv, max_len, self.D, dtype=torch.float16, device=self.dev)
        self.v = torch.zeros_like(self.k)
        half = self.D // 2
        self.inv = cfg.rope_theta ** (-torch.arange(half, device=self.dev, dtype=torch.float32) * 2.0 / self.D)
        self.max_len = max_len

    def weight_bytes(self) -> int:
        return sum(w.numel() * 2 for L in self.layers for w in L[:4]) + self.lm_head.numel() * 2

    def _norm(self, x, w):
        xf = x.float()
        return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + self.cfg.rms_eps) * w.float()).half()

    def _rope(self, t, pos):                       # t [B, T, h, D], pos [B, T]
        ang = pos.float()[..., None, None] * self.inv
        cs, sn = ang.cos(), ang.sin()
        tf = t.float()
        if self.cfg.rope_interleaved:
            a, b = tf[..., 0::2], tf[..., 1::2]
            return torch.stack([a * cs - b * sn, a * sn + b * cs], -1).flatten(-2).half()
        hd = self.D // 2
        a, b = tf[..., :hd], tf[..., hd:]
        return torch.cat([a * cs - b * sn, a * sn + b * cs], -1).half()

    def forward(self, tokens, pos, prefill: bool):
        """tokens / pos [B, T] (T = prompt length, or 1 for a decode step) -> logits of the last position [B, vocab]."""
        B, T = tokens.shape
        H, Hkv, D = self.H, self.Hkv, self.D
        x = self.tok_emb[tokens]
        bidx = torch.arange(B, device=self.dev)[:, None].expand(B, T)
        for li, (wqkv, wo, wgu, wd, n1, n2) in enumerate(self.layers):
            qkv = self._norm(x, n1) @ wqkv.t()
            q, k, v = qkv.split([H * D, Hkv * D, Hkv * D], -1)
            q, k = self._rope(q.view(B, T, H, D), pos), self._rope(k.view(B, T, Hkv, D), pos)
            self.k[li][bidx, :, pos] = k                                   # [B, T, Hkv, D] rows at (b, :, pos)
            self.v[li][bidx, :, pos] = v.view(B, T, Hkv, D)
            if prefill:
                att = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.view(B, T, Hkv, D).transpose(1, 2),
                                                     is_causal=True, enable_gqa=Hkv != H)
            else:
                mask = (torch.arange(self.max_len, device=self.dev)[None, :] <= pos[:, :1])[:, None, None, :]
                att = F.scaled_dot_product_attention(q.transpose(1, 2), self.k[li], self.v[li], attn_mask=mask, enable_gqa=Hkv != H)
            x = x + att.transpose(1, 2).reshape(B, T, H * D) @ wo.t()
            gu = self._norm(x, n2) @ wgu.t()
            g, u = gu.chunk(2, -1)
            x = x + (F.silu(g) * u) @ wd.t()
        return (self._norm(x[:, -1], self.out_norm) @ self.lm_head.t()).float()


def run_library(a, rt, prompts):
    """Times the stock-PyTorch arm with the same protocol: prefill + first token = TTFT, then N - 1 graph replays."""
    B, T, N = a.batch, a.prompt, a.new
    dev = rt.device
    lib = _LibraryDecoder(rt, B, T + N + 8)
    pos0 = torch.arange(T, device=dev)[None, :].expand(B, T).contiguous()
    tok = torch.zeros(B, 1, dtype=torch.long, device=dev)
    pos = torch.full((B, 1), T, dtype=torch.long, device=dev)

    def step():
        nxt = lib.forward(tok, pos, False).argmax(-1)
        tok.copy_(nxt[:, None])
        pos.add_(1)

    lib.forward(prompts, pos0, True)
    side = torch.cuda.Stream(device=dev)
    side.wait_stream(torch.cuda.current_stream(dev))
    with torch.cuda.stream(side):
        step()
    torch.cuda.current_stream(dev).wait_stream(side)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        step()
    e = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
    torch.cuda.synchronize()
    e[0].record()
    nxt = lib.forward(prompts, pos0, True).argmax(-1)
    e[1].record()
    tok.copy_(nxt[:, None])
    pos.fill_(T)
    for _ in range(N - 1):
        g.replay()
    e[2].record()
    torch.cuda.synchronize()
    return e[0].elapsed_time(e[1]), e[1].elapsed_time(e[2]), lib.weight_bytes()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--prompt", type=int, default=512)
    ap.add_argument("--new", type=int, default=256)
    ap.add_argument("--layers", type=int, default=32)
    ap.add_argument("--tp", type=int, default=1)
    ap.add_argument("--eager", action="store_true", help="launch every kernel from the host instead of replaying a CUDA graph")
    ap.add_argument("--impl", default="ours", choices=["ours", "library"],
                    help="library: dense fp16 weights on cuBLAS + SDPA + eager elementwise ops, CUDA-graph loop (one GPU)")
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
    if a.impl == "library":
        assert world == 1, "the library arm is single-GPU"
        ttft_ms, dec_ms, wbytes = run_library(a, rt, prompts)
        per_tok_s = dec_ms / 1e3 / (N - 1)
        peaks = os.path.join(ROOT, "MEASURED_PEAKS.json")
        hbm = json.load(open(peaks))["hbm_gbs"] * 1e9 if os.path.exists(peaks) else 6.65e12
        print(json.dumps({"metric": "gguf_q4_0_decode_tokens_per_s", "value": round(B * (N - 1) / (dec_ms / 1e3), 1), "unit": "tokens/s",
                          "n_gpus": 1, "batch": B, "prompt": T, "new_tokens": N, "ttft_ms": round(ttft_ms, 2),
                          "ms_per_token": round(per_tok_s * 1e3, 4), "weight_bytes_per_rank": wbytes,
                          "hbm_roofline_frac": round(wbytes / per_tok_s / hbm, 3), "layers": a.layers, "decode_loop": "cuda_graph",
                          "impl": "library", "config": "llama-7b shape, the Q4_0 weights expanded to dense fp16, fp16 KV cache, greedy",
                          "parallelism": "tp1"}), flush=True)
        return
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
