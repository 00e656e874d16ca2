"""Launches every hand-written kernel of the framework ONCE on a mid-size case (inputs larger than L2 where the
kernel is bandwidth bound, a few hundred MB on the device at any time), so that a single profiler pass over this
script yields one record per kernel.  Without a profiler it prints the launch count and exits.

    python benchmarks/ncu_suite.py [--only gemm,attn,...]

Cases are independent; device memory is released between them.
"""
import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from rustorch_b200 import _native  # noqa: E402
from rustorch_b200.ops import kernels as K  # noqa: E402


def bf(*shape):
    return (torch.randn(*shape, device="cuda") * 0.5).to(torch.bfloat16)


def case_gemm():
    a, b = bf(8192, 2048), bf(8192, 2048)
    K.gemm(a, b)                                                  # forward layout, 8192 x 8192 x 2048
    dy, x = bf(8192, 3072), bf(8192, 768)
    out = torch.zeros(3072, 768, device="cuda")
    K.gemm(dy, x, a_mn=True, b_mn=True, out=out, accumulate=True, split_k=8)   # weight-gradient layout, split-K atomics


def case_attn():
    B, H, T, D = 16, 12, 1024, 64
    q, k, v, do = bf(B, T, H, D), bf(B, T, H, D), bf(B, T, H, D), bf(B, T, H, D)
    o, lse = K.attention_fwd(q, k, v, True)
    K.attention_bwd(q, k, v, o, do, lse, True)


def case_norm():
    rows, C = 65536, 1024                                          # 134 MB per tensor
    x, w, b, dy = bf(rows, C), bf(C), bf(C), bf(rows, C)
    y, mean, rstd = K.layer_norm_fwd(x, w, b, 1e-5)
    dg, db = torch.zeros(C, device="cuda"), torch.zeros(C, device="cuda")
    K.layer_norm_bwd(dy, x, w, mean, rstd, dg, db, dres=dy)
    y, rstd = K.rms_norm_fwd(x, w, 1e-5)
    K.rms_norm_bwd(dy, x, w, rstd, dg)
    del x, dy, y
    xw, ww, dyw = bf(16384, 4096), bf(4096), bf(16384, 4096)       # wide rows (Llama-8B width): CTA-per-row backward
    yw, rstdw = K.rms_norm_fwd(xw, ww, 1e-5)
    K.rms_norm_bwd(dyw, xw, ww, rstdw, torch.zeros(4096, device="cuda"))


def case_optim():
    n = 1 << 26                                                    # 67 M parameters, 1.2 GB of state
    p, g, m, v = (torch.randn(n, device="cuda") for _ in range(4))
    v.abs_()
    lp = torch.empty(n, dtype=torch.bfloat16, device="cuda")
    K.fused_optim_step(p, g, m, v, lp, mode=K.OPT_ADAMW, lr=1e-3, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1,
                       bias_corr1=0.1, bias_corr2=0.05)


def case_loss_embedding():
    rows, V = 8192, 50257
    ld = -(-V // 64) * 64
    logits = bf(rows, ld)
    tgt = torch.randint(0, V, (rows,), device="cuda")
    K.cross_entropy_(logits, tgt, V, 1.0 / rows)
    del logits
    T, C = 1024, 768
    idx = torch.randint(0, V, (rows,), device="cuda")
    wte, wpe = bf(V, C), bf(T, C)
    out = K.embedding_fwd(idx, wte, wpe, T)
    dwte, dwpe = torch.zeros(V, C, device="cuda"), torch.zeros(T, C, device="cuda")
    K.embedding_bwd(idx, out, dwte, dwpe, T, V)
    K.colsum_accum(bf(65536, 768), torch.zeros(768, device="cuda"))
    K.reduce_all(torch.randn(1 << 26, device="cuda"), "sum")


def case_elementwise():
    from rustorch_b200.ops import elementwise as E
    x, y = bf(1 << 27), bf(1 << 27)                                # 268 MB each
    E.add(x, y)
    E.unary("gelu", x)
    z = bf(131072, 1024)
    E.softmax(z, -1)
    E.log_softmax(bf(8192, 16384), -1)
    E.reduce_last(z, "var")


def case_batchnorm():
    from rustorch_b200.ops.batchnorm import batch_norm
    x = bf(256, 64, 56, 56).contiguous(memory_format=torch.channels_last).requires_grad_(True)
    w, b = torch.ones(64, device="cuda", requires_grad=True), torch.zeros(64, device="cuda", requires_grad=True)
    rm, rv = torch.zeros(64, device="cuda"), torch.ones(64, device="cuda")
    res = bf(256, 64, 56, 56).contiguous(memory_format=torch.channels_last)
    y = batch_norm(x, rm, rv, w, b, training=True, residual=res, relu=True)
    y.backward(torch.ones_like(y))


def case_conv():
    from rustorch_b200.ops.conv import Conv2dFn
    x = bf(256, 128, 28, 28).contiguous(memory_format=torch.channels_last).requires_grad_(True)
    w = (bf(128, 128, 3, 3) * 0.1).contiguous(memory_format=torch.channels_last).requires_grad_(True)
    y = Conv2dFn.apply(x, w, None, 1, 1)
    y.backward(torch.ones_like(y))                                # input gradient (forward kernel) + weight gradient
    del x, w, y
    # 64-channel 3 x 3 layer: resident-halo forward / input gradient, three-tap weight gradient
    x = bf(256, 64, 56, 56).contiguous(memory_format=torch.channels_last).requires_grad_(True)
    w = (bf(64, 64, 3, 3) * 0.1).contiguous(memory_format=torch.channels_last).requires_grad_(True)
    y = Conv2dFn.apply(x, w, None, 1, (1, 1))
    y.backward(torch.ones_like(y))
    del x, w, y
    # strided layer: input gradient as parity-class convolutions scattered into dx
    x = bf(256, 64, 56, 56).contiguous(memory_format=torch.channels_last).requires_grad_(True)
    w = (bf(128, 64, 3, 3) * 0.1).contiguous(memory_format=torch.channels_last).requires_grad_(True)
    y = Conv2dFn.apply(x, w, None, 2, (1, 1))
    y.backward(torch.ones_like(y))
    del x, w, y
    # stem: patch matrix + tcgen05 GEMM
    from rustorch_b200.ops.conv import conv2d
    x = bf(256, 3, 224, 224).contiguous(memory_format=torch.channels_last)
    w = (bf(64, 3, 7, 7) * 0.1).contiguous(memory_format=torch.channels_last).requires_grad_(True)
    y = conv2d(x, w, None, 2, 3)
    y.backward(torch.ones_like(y))


def case_pool_groupnorm_rnn():
    from rustorch_b200.ops import pool
    from rustorch_b200.ops.groupnorm import group_norm
    from rustorch_b200.ops.rnn import lstm_gates
    x = bf(256, 64, 112, 112).contiguous(memory_format=torch.channels_last).requires_grad_(True)
    y = pool.max_pool2d(x, 3, 2, 1)
    y.backward(torch.ones_like(y))
    z = pool.adaptive_avg_pool2d(bf(256, 512, 7, 7).contiguous(memory_format=torch.channels_last), 1)
    pool.dropout(bf(1 << 27), 0.1, True)
    del x, y, z
    g = bf(64, 256, 56, 56).requires_grad_(True)
    wg, bg = torch.ones(256, device="cuda", requires_grad=True), torch.zeros(256, device="cuda", requires_grad=True)
    o = group_norm(g, 32, wg, bg)
    o.backward(torch.ones_like(o))
    gates, c0 = bf(65536, 4 * 1024).requires_grad_(True), bf(65536, 1024)
    h, c = lstm_gates(gates, c0)
    (h.sum() + c.sum()).backward()


def case_quant_decode():
    from rustorch_b200.formats import gguf
    from rustorch_b200.llm import LlamaConfig, LlamaRuntime, QuantLinear
    C = _native.load(required=True)
    for qt in (gguf.GGMLType.Q4_0, gguf.GGMLType.Q8_0):
        q = QuantLinear.random(22016, 4096, qt, 0.02, "cuda", seed=1)
        for M in (1, 4):
            x = (torch.randn(M, 4096, device="cuda") * 0.5).half()
            yv = torch.empty(M, 22016, device="cuda", dtype=torch.half)
            C.q_gemv(q.qs, q.scales, x, yv, None, None, qt == gguf.GGMLType.Q8_0, path=1)
            if M == 4:
                C.q_gemv(q.qs, q.scales, x, yv, None, None, qt == gguf.GGMLType.Q8_0, path=2)
            # decode projection in one kernel: RMSNorm prologue + dp4a GEMV + SwiGLU epilogue (rows as [gate; up])
            q.fused(x, norm_w=torch.ones(4096, device="cuda", dtype=torch.half), eps=1e-5, swiglu=True)
        q((torch.randn(32, 4096, device="cuda") * 0.5).half())     # dequant-fused tcgen05 GEMM (batched decode), A from TMEM
        if qt == gguf.GGMLType.Q4_0:
            part, cnt = q._tc_buffers(32)                          # the shared-memory-A variant of the same GEMM
            x32 = (torch.randn(32, 4096, device="cuda") * 0.5).half()
            C.q_gemm_tc(q.qs, q.scales, x32, torch.empty(32, 22016, device="cuda", dtype=torch.half), None, None, False, part, cnt, path=1)
        q((torch.randn(512, 4096, device="cuda") * 0.5).half())    # dequantise + tcgen05 GEMM (prefill path)
    cfg = LlamaConfig(n_layer=1)
    rt = LlamaRuntime.random_init(cfg, "cuda", seed=0)
    cache = rt.new_cache(4, 1024)
    lg = rt.prefill(torch.randint(0, cfg.vocab_size, (4, 512)).cuda(), cache)
    rt.decode_step(lg.argmax(-1), cache)                           # rmsnorm, rope + cache append, split attention, SwiGLU


def case_collectives_single_rank():
    """World of one: the kernels run their full protocol (flags, barriers, staging) against their own buffers."""
    from rustorch_b200.distributed.p2p_collectives import AllReduceResidualNorm, P2PCollectives
    from rustorch_b200.distributed.tp_fused import AllGatherGemm, GemmReduceScatter
    ag = AllGatherGemm(2048, 4096, "cuda")
    w = bf(11008, 4096)
    ag(w, x=bf(2048, 4096))
    rs = GemmReduceScatter(2048, 4096, "cuda")
    rs(bf(2048, 11008), bf(4096, 11008))
    pc = P2PCollectives(1 << 24, torch.bfloat16, "cuda")
    pc.all_reduce(bf(1 << 24))
    arn = AllReduceResidualNorm(32 * 4096, torch.float16, "cuda")
    part, xx = torch.randn(32, 4096, device="cuda").half(), torch.randn(32, 4096, device="cuda").half()
    arn(part, xx, torch.ones(4096, device="cuda").half(), 1e-5)
    from rustorch_b200.distributed.fused_allreduce import FusedDDPAdamW
    m = torch.nn.Linear(4096, 4096, bias=False, device="cuda").to(torch.bfloat16)
    opt = FusedDDPAdamW(m, lr=1e-3, overlap=False)
    m(torch.randn(8, 4096, device="cuda").bfloat16()).sum().backward()
    opt.step()


CASES = {"gemm": case_gemm, "attn": case_attn, "norm": case_norm, "optim": case_optim, "loss": case_loss_embedding,
         "elementwise": case_elementwise, "batchnorm": case_batchnorm, "conv": case_conv, "pool_gn_rnn": case_pool_groupnorm_rnn,
         "quant": case_quant_decode,
         "collectives": case_collectives_single_rank}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--only", default="")
    a = ap.parse_args()
    torch.cuda.set_device(0)
    names = [n for n in a.only.split(",") if n] or list(CASES)
    l0 = _native.launch_count()
    for n in names:
        CASES[n]()
        torch.cuda.synchronize()
        _native.check_status()
        torch.cuda.empty_cache()
        print(f"{n}: ok, {_native.launch_count() - l0} launches so far, {torch.cuda.max_memory_allocated() / 2 ** 30:.2f} GiB peak", flush=True)


if __name__ == "__main__":
    main()
