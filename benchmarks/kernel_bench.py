#!/usr/bin/env python
"""Per-kernel micro-benchmarks with roofline fractions against the measured peaks.

    python benchmarks/kernel_bench.py --op gemm --m 16384 --n 3072 --k 768 [--layout nt|nn|tn]
    python benchmarks/kernel_bench.py --op attn_fwd --batch 16 --heads 12 --seq 1024 --dim 64
    python benchmarks/kernel_bench.py --op all

Timing hygiene: >= 3 warm-up launches, CUDA events on the launching stream, an L2 flush (write
of a 256 MB buffer) between timed iterations, best and median of ``--iters`` reported.  Peaks are
read from ``MEASURED_PEAKS.json`` at the repo root when present ("of measured"), else the
documented fallback 6.65 TB/s / 1.59 PFLOP/s ("of fallback").
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from rustorch_b200.ops import kernels as K  # noqa: E402


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return d["hbm_gbs"] * 1e9, d["bf16_tflops"] * 1e12, "measured"
    return 6.65e12, 1.59e15, "fallback"


_flush = None


def flush_l2():
    global _flush
    if _flush is None:
        _flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device="cuda")
    _flush.fill_(1)


def time_op(fn, iters, warmup=3, flush=True):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        if flush:
            flush_l2()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1) * 1e-3)
    return min(ts), statistics.median(ts)


def bf(*shape):
    return (torch.randn(*shape, device="cuda") * 0.5).to(torch.bfloat16)


def report(name, best, med, flops=None, bytes_=None, extra=""):
    bw, fl, src = peaks()
    out = {"op": name, "best_us": round(best * 1e6, 2), "median_us": round(med * 1e6, 2)}
    if flops:
        out["tflops"] = round(flops / best / 1e12, 1)
        out[f"frac_of_{src}_bf16_peak"] = round(flops / best / fl, 3)
    if bytes_:
        out["gbs"] = round(bytes_ / best / 1e9, 1)
        out[f"frac_of_{src}_hbm_peak"] = round(bytes_ / best / bw, 3)
    if extra:
        out["note"] = extra
    print(json.dumps(out), flush=True)
    return out


def bench_gemm(a):
    M, N, Kd = a.m, a.n, a.k
    lay = a.layout
    if lay == "nt":      # forward: x[M,K] @ W[N,K]^T
        A, B, kw = bf(M, Kd), bf(N, Kd), {}
    elif lay == "nn":    # dgrad: dy[M,K] @ W[K,N]
        A, B, kw = bf(M, Kd), bf(Kd, N), {"b_mn": True}
    else:                # wgrad: dy[K,M]^T @ x[K,N]
        A, B, kw = bf(Kd, M), bf(Kd, N), {"a_mn": True, "b_mn": True}
    if a.split_k > 1 or a.accumulate:
        out = torch.zeros(M, N, dtype=torch.float32, device="cuda")
        fn = lambda: K.gemm(A, B, out=out, accumulate=True, split_k=a.split_k, block_n=a.block_n, **kw)
        obytes = 4
    else:
        out = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
        fn = lambda: K.gemm(A, B, out=out, block_n=a.block_n, **kw)
        obytes = 2
    best, med = time_op(fn, a.iters)
    ours = report(f"gemm_{lay}_{M}x{N}x{Kd}_sk{a.split_k}", best, med, flops=2.0 * M * N * Kd,
                  bytes_=2.0 * (M * Kd + N * Kd) + obytes * M * N)
    if a.compare:
        Af = A.t() if kw.get("a_mn") else A
        Bf = B if kw.get("b_mn") else B.t()
        best, med = time_op(lambda: torch.matmul(Af, Bf), a.iters)
        report(f"cublas_{lay}_{M}x{N}x{Kd}", best, med, flops=2.0 * M * N * Kd, extra="library baseline")
    return ours


def bench_attn(a, bwd):
    B, H, T, D = a.batch, a.heads, a.seq, a.dim
    Hkv = a.kv_heads or H
    q, k, v = bf(B, T, H, D), bf(B, T, Hkv, D), bf(B, T, Hkv, D)
    causal = not a.non_causal
    fl = 4.0 * B * H * T * T * D * (0.5 if causal else 1.0)
    if not bwd:
        best, med = time_op(lambda: K.attention_fwd(q, k, v, causal), a.iters)
        report(f"attn_fwd_b{B}h{H}t{T}d{D}", best, med, flops=fl)
        if a.compare:
            qt, kt, vt = (x.transpose(1, 2) for x in (q, k, v))
            f = lambda: torch.nn.functional.scaled_dot_product_attention(qt, kt, vt, is_causal=causal,
                                                                         enable_gqa=Hkv != H)
            best, med = time_op(f, a.iters)
            report(f"sdpa_fwd_b{B}h{H}t{T}d{D}", best, med, flops=fl, extra="library baseline")
    else:
        o, lse = K.attention_fwd(q, k, v, causal)
        do = bf(B, T, H, D)
        best, med = time_op(lambda: K.attention_bwd(q, k, v, o, do, lse, causal), a.iters)
        report(f"attn_bwd_b{B}h{H}t{T}d{D}", best, med, flops=2.5 * fl,
               extra="flops counted as 2.5x forward (algorithmic); includes the delta and dQ-conversion kernels")
        if a.compare:
            qt, kt, vt = (x.transpose(1, 2).detach().requires_grad_(True) for x in (q, k, v))
            ot = torch.nn.functional.scaled_dot_product_attention(qt, kt, vt, is_causal=causal, enable_gqa=Hkv != H)
            dot = do.transpose(1, 2)
            f = lambda: torch.autograd.grad(ot, (qt, kt, vt), dot, retain_graph=True)
            best, med = time_op(f, a.iters)
            report(f"sdpa_bwd_b{B}h{H}t{T}d{D}", best, med, flops=2.5 * fl, extra="library baseline (backward only)")


def bench_norm(a):
    rows, C = a.m, a.n
    x, w, b = bf(rows, C), bf(C), bf(C)
    best, med = time_op(lambda: K.layer_norm_fwd(x, w, b, 1e-5), a.iters)
    report(f"layernorm_fwd_{rows}x{C}", best, med, bytes_=4.0 * rows * C)
    y, mean, rstd = K.layer_norm_fwd(x, w, b, 1e-5)
    dg, db = torch.zeros(C, device="cuda"), torch.zeros(C, device="cuda")
    dy = bf(rows, C)
    best, med = time_op(lambda: K.layer_norm_bwd(dy, x, w, mean, rstd, dg, db, dres=dy), a.iters)
    report(f"layernorm_bwd_{rows}x{C}", best, med, bytes_=6.0 * rows * C)


def bench_adamw(a):
    n = a.m * a.n
    p, g, m, v = (torch.randn(n, device="cuda") for _ in range(4))
    v.abs_()
    lp = torch.empty(n, dtype=torch.bfloat16, device="cuda")
    fn = lambda: K.fused_optim_step(p, g, m, v, lp, mode=K.OPT_ADAMW, lr=1e-3, beta1=0.9, beta2=0.95,
                                    eps=1e-8, weight_decay=0.1, bias_corr1=0.1, bias_corr2=0.05)
    best, med = time_op(fn, a.iters)
    report(f"fused_adamw_{n}", best, med, bytes_=34.0 * n)


def bench_ce(a):
    rows, V = a.m, a.n
    ld = -(-V // 64) * 64
    logits = bf(rows, ld)
    tgt = torch.randint(0, V, (rows,), device="cuda")
    best, med = time_op(lambda: K.cross_entropy_(logits, tgt, V, 1.0 / rows), a.iters)
    report(f"cross_entropy_{rows}x{V}", best, med, bytes_=4.0 * rows * ld)


def bench_bn(a):
    """BatchNorm2d (+ ReLU) training forward and backward at the ResNet-18 activation shapes, batch 256, channels-last
    bf16.  Bytes: forward reads x twice and writes y; backward reads x, dy and y twice and writes dx."""
    from rustorch_b200.ops.batchnorm import batch_norm
    for (C, H) in [(64, 112), (64, 56), (128, 28), (256, 14), (512, 7)]:
        x = bf(256, C, H, H).contiguous(memory_format=torch.channels_last).requires_grad_(True)
        w = torch.ones(C, device="cuda", requires_grad=True)
        b = torch.zeros(C, device="cuda", requires_grad=True)
        rm, rv = torch.zeros(C, device="cuda"), torch.ones(C, device="cuda")
        dy = torch.randn_like(x)
        nbytes = 2.0 * x.numel()
        best, med = time_op(lambda: batch_norm(x, rm, rv, w, b, True, 0.1, 1e-5, None, True), a.iters)
        report(f"bn_relu_fwd_256x{C}x{H}x{H}", best, med, bytes_=3.0 * nbytes)
        y = batch_norm(x, rm, rv, w, b, True, 0.1, 1e-5, None, True)
        best, med = time_op(lambda: torch.autograd.grad(y, (x, w, b), dy, retain_graph=True), a.iters)
        report(f"bn_relu_bwd_256x{C}x{H}x{H}", best, med, bytes_=7.0 * nbytes)
        del x, y, dy


def bench_qgemv(a):
    """Q4_0 dequant-fused GEMV at the llama-7B decode shapes, register-fed vs bulk-copy-fed kernel.  Each timed
    region walks enough distinct weight matrices (> 300 MB) that none of them is served from L2."""
    from rustorch_b200 import _native
    from rustorch_b200.formats import gguf
    from rustorch_b200.llm import QuantLinear
    C = _native.load(required=True)
    shapes = [(12288, 4096), (4096, 4096), (22016, 4096), (4096, 11008), (32000, 4096)]
    rows = (1, 4)
    if getattr(a, "qshape", ""):
        shapes, rows = [tuple(int(v) for v in a.qshape.split(","))], (1,)
    for (N, Kd) in shapes:
        nbytes = N * Kd // 32 * 18
        copies = max(2, -(-300_000_000 // nbytes))
        mats = [QuantLinear.random(N, Kd, gguf.GGMLType.Q4_0, 0.02, "cuda", seed=i) for i in range(copies)]
        for M in rows:
            x = (torch.randn(M, Kd, device="cuda") * 0.5).half()
            y = torch.empty(M, N, device="cuda", dtype=torch.half)
            for reg in (True, False):
                def run():
                    for q in mats:
                        C.q_gemv(q.qs, q.scales, x, y, None, None, False, path=1 if reg else 2)
                best, med = time_op(run, a.iters, flush=False)
                report(f"q4_gemv_{'register' if reg else 'bulk'}_m{M}_{N}x{Kd}", best / copies, med / copies, bytes_=float(nbytes),
                       extra=f"mean over {copies} distinct matrices per timed region")
            # the decode kernel: RMSNorm prologue + int8-activation dp4a GEMV (+ SwiGLU epilogue on the gate/up shape)
            nw = torch.ones(Kd, device="cuda", dtype=torch.half)
            sw = N == 22016
            yf = torch.empty(M, N // 2 if sw else N, device="cuda", dtype=torch.half)

            def run_fused():
                for q in mats:
                    C.q_gemv_fused(q.qs, q.scales, x, yf, nw, 1e-5, None, False, sw)
            best, med = time_op(run_fused, a.iters, flush=False)
            report(f"q4_gemv_fused_norm{'_swiglu' if sw else ''}_m{M}_{N}x{Kd}", best / copies, med / copies, bytes_=float(nbytes),
                   extra=f"mean over {copies} distinct matrices per timed region")
        del mats


def bench_qgemm(a):
    """Q4_0 weights times 16 / 32 / 128 activation rows at the llama-7B shapes: dequant-fused tcgen05 GEMM against the
    GEMV kernel (one pass over the weights per 8 rows) and the two-pass path (expand to fp16, then the dense GEMM).
    Distinct matrices per timed region keep the weights out of L2."""
    from rustorch_b200 import _native
    from rustorch_b200.formats import gguf
    from rustorch_b200.llm import QuantLinear
    C = _native.load(required=True)
    for (N, Kd) in [(12288, 4096), (4096, 4096), (22016, 4096), (4096, 11008)]:
        nbytes = N * Kd // 32 * 18
        copies = max(2, -(-300_000_000 // nbytes))
        mats = [QuantLinear.random(N, Kd, gguf.GGMLType.Q4_0, 0.02, "cuda", seed=i) for i in range(copies)]
        for M in (16, 32, 128):
            x = (torch.randn(M, Kd, device="cuda") * 0.5).half()
            y = torch.empty(M, N, device="cuda", dtype=torch.half)
            part, cnt = mats[0]._tc_buffers(M)

            def run_tc():
                for q in mats:
                    C.q_gemm_tc(q.qs, q.scales, x, y, None, None, False, part, cnt, 0)

            def run_tc_smem():
                for q in mats:
                    C.q_gemm_tc(q.qs, q.scales, x, y, None, None, False, part, cnt, 1)

            def run_gemv():
                for q in mats:
                    for m0 in range(0, M, 8):
                        C.q_gemv(q.qs, q.scales, x[m0:m0 + 8], y[m0:m0 + 8], None, None, False)
            best, med = time_op(run_tc, a.iters, flush=False)
            report(f"q4_gemm_tc_m{M}_{N}x{Kd}", best / copies, med / copies, bytes_=float(nbytes), flops=2.0 * M * N * Kd,
                   extra=f"mean over {copies} distinct matrices per timed region")
            best, med = time_op(run_tc_smem, a.iters, flush=False)
            report(f"q4_gemm_tc_smemA_m{M}_{N}x{Kd}", best / copies, med / copies, bytes_=float(nbytes), flops=2.0 * M * N * Kd,
                   extra="operand A staged in shared memory")
            if M <= 16:
                best, med = time_op(run_gemv, a.iters, flush=False)
                report(f"q4_gemv_x{M // 8}_m{M}_{N}x{Kd}", best / copies, med / copies, bytes_=float(nbytes), extra="GEMV kernel, 8 rows per pass")
        del mats


def bench_conv(a):
    """ResNet-18 body convolutions at batch 256 (channels-last bf16): implicit-GEMM kernels vs cuDNN."""
    import torch.nn.functional as F
    from rustorch_b200.ops.conv import Conv2dFn
    for (N, Cin, H, W, Cout, k, s, p) in [(256, 64, 56, 56, 64, 3, 1, 1), (256, 128, 28, 28, 128, 3, 1, 1), (256, 256, 14, 14, 256, 3, 1, 1),
                                          (256, 512, 7, 7, 512, 3, 1, 1), (256, 64, 56, 56, 128, 3, 2, 1)]:
        x = torch.randn(N, Cin, H, W, device="cuda").bfloat16().contiguous(memory_format=torch.channels_last)
        w = (torch.randn(Cout, Cin, k, k, device="cuda") * 0.05).bfloat16().contiguous(memory_format=torch.channels_last)
        OH, OW = (H + 2 * p - k) // s + 1, (W + 2 * p - k) // s + 1
        flops = 2.0 * N * OH * OW * Cout * Cin * k * k
        tag = f"{N}x{Cin}x{H}x{W}_to{Cout}_k{k}s{s}"
        best, med = time_op(lambda: Conv2dFn.apply(x, w, None, s, p), a.iters)
        report(f"conv_fwd_{tag}", best, med, flops=flops)
        best, med = time_op(lambda: F.conv2d(x, w, None, s, p), a.iters)
        report(f"cudnn_fwd_{tag}", best, med, flops=flops, extra="library baseline")
        xg, wg = x.clone().requires_grad_(True), w.clone().requires_grad_(True)
        y = Conv2dFn.apply(xg, wg, None, s, p)
        g = torch.randn_like(y)
        best, med = time_op(lambda: torch.autograd.grad(y, (xg, wg), g, retain_graph=True), a.iters)
        report(f"conv_bwd_{tag}", best, med, flops=2 * flops, extra="dgrad + wgrad" + ("" if s == 1 else " (dgrad through the library)"))
        xl, wl = x.clone().requires_grad_(True), w.clone().requires_grad_(True)
        yl = F.conv2d(xl, wl, None, s, p)
        best, med = time_op(lambda: torch.autograd.grad(yl, (xl, wl), g, retain_graph=True), a.iters)
        report(f"cudnn_bwd_{tag}", best, med, flops=2 * flops, extra="library baseline")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--op", default="all")
    ap.add_argument("--m", type=int, default=16384)
    ap.add_argument("--n", type=int, default=3072)
    ap.add_argument("--k", type=int, default=768)
    ap.add_argument("--layout", default="nt", choices=["nt", "nn", "tn"])
    ap.add_argument("--split-k", type=int, default=1)
    ap.add_argument("--accumulate", action="store_true")
    ap.add_argument("--block-n", type=int, default=0)
    ap.add_argument("--batch", type=int, default=16)
    ap.add_argument("--heads", type=int, default=12)
    ap.add_argument("--kv-heads", type=int, default=0)
    ap.add_argument("--seq", type=int, default=1024)
    ap.add_argument("--dim", type=int, default=64)
    ap.add_argument("--non-causal", action="store_true")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--compare", action="store_true", help="also time the stock PyTorch op")
    ap.add_argument("--qshape", default="", help="qgemv: only this N,K (e.g. 12288,4096), one activation row: a small case for a profiler capture")
    a = ap.parse_args()
    torch.cuda.set_device(0)
    if a.op == "gemm":
        bench_gemm(a)
    elif a.op == "attn_fwd":
        bench_attn(a, False)
    elif a.op == "attn_bwd":
        bench_attn(a, True)
    elif a.op == "norm":
        bench_norm(a)
    elif a.op == "adamw":
        bench_adamw(a)
    elif a.op == "bn":
        bench_bn(a)
    elif a.op == "ce":
        bench_ce(a)
    elif a.op == "qgemv":
        bench_qgemv(a)
    elif a.op == "conv":
        bench_conv(a)
    elif a.op == "qgemm":
        bench_qgemm(a)
    elif a.op == "all":
        a.compare = True
        for (m, n, k, lay, sk) in [(8192, 8192, 8192, "nt", 1), (16384, 2304, 768, "nt", 1),
                                   (16384, 3072, 768, "nt", 1), (16384, 768, 3072, "nt", 1),
                                   (16384, 768, 768, "nt", 1), (16384, 50304, 768, "nt", 1),
                                   (16384, 768, 3072, "nn", 1), (16384, 3072, 768, "nn", 1),
                                   (16384, 768, 50304, "nn", 1),
                                   (3072, 768, 16384, "tn", 2), (768, 3072, 16384, "tn", 2),
                                   (2304, 768, 16384, "tn", 2), (50304, 768, 16384, "tn", 1)]:
            a.m, a.n, a.k, a.layout, a.split_k = m, n, k, lay, sk
            a.accumulate = lay == "tn"
            bench_gemm(a)
        bench_attn(a, False)
        bench_attn(a, True)
        sv = (a.batch, a.heads, a.kv_heads, a.seq, a.dim)
        a.batch, a.heads, a.kv_heads, a.seq, a.dim = 2, 32, 8, 4096, 128      # the Llama-8B attention shape (GQA 32 / 8)
        bench_attn(a, False)
        bench_attn(a, True)
        a.batch, a.heads, a.kv_heads, a.seq, a.dim = sv
        a.m, a.n = 16384, 768
        bench_norm(a)
        a.m, a.n = 16384, 50257
        bench_ce(a)
        a.m, a.n = 16384, 10000
        bench_adamw(a)
    else:
        raise SystemExit(f"unknown op {a.op}")
    from rustorch_b200 import _native
    _native.check_status()


if __name__ == "__main__":
    main()
