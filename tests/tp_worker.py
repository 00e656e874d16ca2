"""torchrun worker: fused tensor-parallel linears on W GPUs vs the unsharded fp32 model.  Writes rank<r>.json."""
import json
import os
import sys
import time

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def rel(a, b):
    return float((a.float() - b.float()).abs().max() / b.float().abs().max().clamp_min(1e-6))


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    from rustorch_b200 import _native
    from rustorch_b200.distributed.tp_fused import AllGatherGemm, FusedColumnParallelLinear, FusedRowParallelLinear, GemmReduceScatter
    res = {}
    rows, d, ff = int(os.environ.get("TP_ROWS", "512")), int(os.environ.get("TP_D", "1024")), int(os.environ.get("TP_FF", "4096"))
    g = torch.Generator().manual_seed(0)                              # identical full tensors on every rank
    X = (torch.randn(world * rows, d, generator=g) * 0.5).bfloat16().to(dev)
    Wc = (torch.randn(ff, d, generator=g) * 0.05).bfloat16().to(dev)
    Wr = (torch.randn(d, ff, generator=g) * 0.05).bfloat16().to(dev)
    bc = torch.randn(ff, generator=g).bfloat16().to(dev)
    br = torch.randn(d, generator=g).bfloat16().to(dev)
    G = torch.randn(world * rows, d, generator=g).bfloat16().to(dev)
    ffl = ff // world
    # ---- raw ops, several epochs
    ag = AllGatherGemm(rows, d, dev)
    rs = GemmReduceScatter(rows, d, dev)
    worst_ag = worst_rs = 0.0
    for it in range(3):
        Xi = (X * (1 + it)).bfloat16()
        y = ag(Wc[rank * ffl:(rank + 1) * ffl], bc[rank * ffl:(rank + 1) * ffl], x=Xi[rank * rows:(rank + 1) * rows])
        ref = Xi.float() @ Wc[rank * ffl:(rank + 1) * ffl].float().t() + bc[rank * ffl:(rank + 1) * ffl].float()
        worst_ag = max(worst_ag, rel(y, ref))
        assert torch.equal(ag.gather, Xi)
        H = torch.nn.functional.gelu(Xi.float() @ Wc.float().t() + bc.float(), approximate="tanh").bfloat16()
        resid = Xi[rank * rows:(rank + 1) * rows].contiguous() if it == 1 else None      # fused residual on one of the epochs
        out = rs(H[:, rank * ffl:(rank + 1) * ffl].contiguous(), Wr[:, rank * ffl:(rank + 1) * ffl].contiguous(), br, residual=resid)
        ref2 = (H.float() @ Wr.float().t() + br.float())[rank * rows:(rank + 1) * rows]
        if resid is not None:
            ref2 = ref2 + resid.float()
        worst_rs = max(worst_rs, rel(out, ref2))
    res["ag_rel"], res["rs_rel"] = worst_ag, worst_rs
    # ---- layers with autograd
    col = FusedColumnParallelLinear(d, ff, rows, device=dev)
    row = FusedRowParallelLinear(ff, d, rows, device=dev)
    with torch.no_grad():
        col.weight.copy_(Wc[rank * ffl:(rank + 1) * ffl]); col.bias.copy_(bc[rank * ffl:(rank + 1) * ffl])
        row.weight.copy_(Wr[:, rank * ffl:(rank + 1) * ffl]); row.bias.copy_(br)
    xs = X[rank * rows:(rank + 1) * rows].clone().requires_grad_(True)
    y = row(torch.nn.functional.gelu(col(xs), approximate="tanh"))
    y.backward(G[rank * rows:(rank + 1) * rows])
    Xr = X.float().requires_grad_(True)
    wc, wr, bcf, brf = (t.float().requires_grad_(True) for t in (Wc, Wr, bc, br))
    yr = torch.nn.functional.gelu(Xr @ wc.t() + bcf, approximate="tanh") @ wr.t() + brf
    yr.backward(G.float())
    res["y_rel"] = rel(y, yr[rank * rows:(rank + 1) * rows])
    res["dx_rel"] = rel(xs.grad, Xr.grad[rank * rows:(rank + 1) * rows])
    res["dwc_rel"] = rel(col.weight.grad, wc.grad[rank * ffl:(rank + 1) * ffl])
    res["dwr_rel"] = rel(row.weight.grad, wr.grad[:, rank * ffl:(rank + 1) * ffl])
    res["dbr_rel"] = rel(row.bias.grad, brf.grad)
    # ---- the library arm (NCCL + cuBLAS) of the same two layers: the benchmark baseline must compute the same thing
    from rustorch_b200.distributed.tp_library import LibraryColumnParallelLinear, LibraryRowParallelLinear
    lcol = LibraryColumnParallelLinear(d, ff, rows, device=dev)
    lrow = LibraryRowParallelLinear(ff, d, rows, device=dev)
    with torch.no_grad():
        lcol.weight.copy_(Wc[rank * ffl:(rank + 1) * ffl]); lrow.weight.copy_(Wr[:, rank * ffl:(rank + 1) * ffl])
    xl = X[rank * rows:(rank + 1) * rows].clone().requires_grad_(True)
    yl = lrow(torch.nn.functional.gelu(lcol(xl), approximate="tanh"))
    yl.backward(G[rank * rows:(rank + 1) * rows])
    Xq = X.float().requires_grad_(True)
    wq, wq2 = Wc.float().requires_grad_(True), Wr.float().requires_grad_(True)
    yq = torch.nn.functional.gelu(Xq @ wq.t(), approximate="tanh") @ wq2.t()
    yq.backward(G.float())
    res["lib_y_rel"] = rel(yl, yq[rank * rows:(rank + 1) * rows])
    res["lib_dx_rel"] = rel(xl.grad, Xq.grad[rank * rows:(rank + 1) * rows])
    res["lib_dw_rel"] = max(rel(lcol.weight.grad, wq.grad[rank * ffl:(rank + 1) * ffl]), rel(lrow.weight.grad, wq2.grad[:, rank * ffl:(rank + 1) * ffl]))
    # ---- peer-memory collectives against NCCL
    from rustorch_b200.distributed.p2p_collectives import P2PCollectives
    pc = P2PCollectives(1 << 22, torch.bfloat16, dev)
    gq = torch.Generator().manual_seed(100 + rank)
    worst = 0.0
    for n_el in (4096, 1 << 20, 3 * (1 << 20) + 8 * world * 5):
        v = torch.randn(n_el, generator=gq).bfloat16().to(dev)
        ref = v.float().clone()
        dist.all_reduce(ref)
        worst = max(worst, rel(pc.all_reduce(v), ref))
        gathered = pc.all_gather(v)
        lst = [torch.empty_like(v) for _ in range(world)]
        dist.all_gather(lst, v)
        assert all(torch.equal(gathered[r], lst[r]) for r in range(world))
        if n_el % (8 * world) == 0:
            rs_ref = ref.view(world, -1)[rank]
            worst = max(worst, rel(pc.reduce_scatter(v), rs_ref))
        b = v.clone()
        pc.broadcast(b, src=world - 1)
        bref = v.clone()
        dist.broadcast(bref, world - 1)
        assert torch.equal(b, bref)
    res["p2p_coll_rel"] = worst
    small = torch.randn(4096, device=dev).bfloat16()
    # ---- all-reduce + residual + RMSNorm kernel: varying row counts, more calls than receive slots, then a CUDA graph
    from rustorch_b200.distributed.p2p_collectives import AllReduceResidualNorm
    worst_x = worst_h = 0.0
    for dt_ in (torch.float16, torch.bfloat16):
        arn = AllReduceResidualNorm(64 * 1024, dt_, dev)
        wn = (torch.rand(1024, generator=gq) + 0.5).to(dt_).to(dev)
        dist.broadcast(wn, 0)
        for call, nr in enumerate((1, 32, 3, 64, 1, 1, 7)):
            part = torch.randn(nr, 1024, generator=gq).to(dt_).to(dev)
            if call == 2:
                part[0, :16] = -0.0                      # the sentinel value itself must survive as a zero
            x0 = torch.randn(nr, 1024, generator=torch.Generator().manual_seed(call)).to(dt_).to(dev)
            tot = part.float().clone()
            dist.all_reduce(tot)
            x_ref = (x0.float() + tot).to(dt_).float()
            h_ref = x_ref * torch.rsqrt(x_ref.pow(2).mean(-1, keepdim=True) + 1e-5) * wn.float()
            x1 = x0.clone()
            hh = arn(part, x1, wn, 1e-5) if call % 2 == 0 else (arn(part, x1), None)[1]
            worst_x = max(worst_x, rel(x1, x_ref))
            if hh is not None:
                worst_h = max(worst_h, rel(hh, h_ref))
            gat = [torch.empty_like(x1) for _ in range(world)]
            dist.all_gather(gat, x1)
            assert all(torch.equal(gat[0], g_) for g_ in gat), "ranks disagree on the residual stream"
        # graph replay: the call counter is device state
        part = torch.randn(4, 1024, generator=gq).to(dt_).to(dev)
        xg = torch.zeros(4, 1024, dtype=dt_, device=dev)
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            arn(part, xg)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        gr = torch.cuda.CUDAGraph()
        with torch.cuda.graph(gr):
            arn(part, xg)
        for _ in range(5):
            gr.replay()
        torch.cuda.synchronize()
        tot = part.float().clone()
        dist.all_reduce(tot)
        ref7 = torch.zeros(4, 1024, device=dev)
        for _ in range(6):
            ref7 = (ref7 + tot).to(dt_).float()
        worst_x = max(worst_x, rel(xg, ref7))
    res["arn_x_rel"], res["arn_h_rel"] = worst_x, worst_h
    # ---- quantised Llama runtime: tensor-parallel prefill + CUDA-graph decode against the unsharded runtime
    from rustorch_b200.llm import LlamaConfig, LlamaRuntime
    qh = max(4, world)                                   # heads (and KV heads beyond two ranks) must split over the ranks
    qcfg = LlamaConfig(vocab_size=256, n_layer=2, n_embd=64 * qh, n_head=qh, n_head_kv=qh if world > 2 else 2, n_ff=256 * qh, context_length=128)
    rt_full = LlamaRuntime.random_init(qcfg, dev, seed=5, std=0.08)
    rt_tp = LlamaRuntime.random_init(qcfg, dev, tp_rank=rank, tp_world=world, tp_group=dist.group.WORLD, seed=5, std=0.08)
    prompt = torch.randint(0, 256, (2, 70), generator=torch.Generator().manual_seed(1))
    c1, c2 = rt_full.new_cache(2, 96), rt_tp.new_cache(2, 96)
    res["dec_prefill_rel"] = rel(rt_tp.prefill(prompt, c2), rt_full.prefill(prompt, c1))
    tok_full, _ = rt_full.generate_graph(prompt, 12)
    tok_tp, _ = rt_tp.generate_graph(prompt, 12)
    res["dec_tokens_equal"] = float((tok_full == tok_tp).float().mean())
    # ---- Llama block stack, tensor + sequence parallel, against the unsharded model
    from rustorch_b200.models.llama import LlamaModel, LlamaTrainConfig
    torch.manual_seed(7)
    th = max(4, world)
    cfg = LlamaTrainConfig.tiny(n_layer=2, n_embd=64 * th, n_head=th, n_head_kv=max(2, world), n_ff=128 * th, vocab_size=512)
    Bq, Tq = 2, 64 * world
    full = LlamaModel(cfg, device=dev, dtype=torch.bfloat16)
    for p_ in full.parameters():
        dist.broadcast(p_.data, 0)
    tpm = LlamaModel(cfg, device=dev, dtype=torch.bfloat16, tp_group=dist.group.WORLD, batch=Bq, seq_len=Tq)
    tpm.load_from_unsharded(full)
    gi = torch.Generator().manual_seed(3)
    idx = torch.randint(0, 512, (Bq, Tq), generator=gi).to(dev)
    tgt = idx.roll(-1, 1)
    _, loss_tp = tpm(idx, tgt)
    loss_tp.backward()
    tpm.sync_replicated_grads()
    _, loss_full = full(idx, tgt)
    loss_full.backward()
    lt = loss_tp.detach().clone()
    dist.all_reduce(lt)
    res["llama_loss_tp"], res["llama_loss_full"] = float(lt), float(loss_full)
    ffl2 = cfg.n_ff // world
    res["llama_dw_rel"] = rel(tpm.blocks[0].w_down.weight.grad, full.blocks[0].w_down.grad[:, rank * ffl2:(rank + 1) * ffl2])
    res["llama_dnorm_rel"] = rel(tpm.blocks[1].attn_norm.grad, full.blocks[1].attn_norm.grad)
    res["llama_dhead_rel"] = rel(tpm.lm_head.grad, full.lm_head.grad)
    # ---- timing against NCCL + library GEMM (device time, max over ranks)
    def timed(fn, iters=10):
        for _ in range(3):
            fn()
        torch.cuda.synchronize(); dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            fn()
        e1.record(); torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / iters], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t)
    xsh, wcl = X[rank * rows:(rank + 1) * rows].contiguous(), Wc[rank * ffl:(rank + 1) * ffl].contiguous()
    full = torch.empty(world * rows, d, dtype=torch.bfloat16, device=dev)
    def nccl_ag():
        dist.all_gather_into_tensor(full, xsh)
        return full @ wcl.t()
    hl, wrl = torch.randn(world * rows, ffl, device=dev).bfloat16(), Wr[:, rank * ffl:(rank + 1) * ffl].contiguous()
    outb = torch.empty(rows, d, dtype=torch.bfloat16, device=dev)
    def nccl_rs():
        dist.reduce_scatter_tensor(outb, hl @ wrl.t())
        return outb
    res["ar_8kb_p2p_us"] = timed(lambda: pc.all_reduce(small), 50) * 1e3
    res["ar_8kb_nccl_us"] = timed(lambda: dist.all_reduce(small), 50) * 1e3
    arn = AllReduceResidualNorm(32 * 4096, torch.float16, dev)
    for nr in (1, 32):
        part = torch.randn(nr, 4096, device=dev).half()
        xx = torch.zeros(nr, 4096, device=dev).half()
        wn = torch.ones(4096, device=dev).half()
        hb = torch.empty_like(xx)
        res[f"arn_{nr}x4096_us"] = timed(lambda: arn(part, xx, wn, 1e-5, hb), 50) * 1e3
    big_ar = torch.randn(1 << 22, device=dev).bfloat16()
    res["ar_8mb_p2p_us"] = timed(lambda: pc.all_reduce(big_ar), 20) * 1e3
    res["ar_8mb_nccl_us"] = timed(lambda: dist.all_reduce(big_ar), 20) * 1e3
    res["ag_fused_ms"] = timed(lambda: ag(wcl, None, x=None))
    res["ag_nccl_ms"] = timed(nccl_ag)
    res["rs_fused_ms"] = timed(lambda: rs(hl, wrl))
    res["rs_nccl_ms"] = timed(nccl_rs)
    res["shape"] = {"rows_per_rank": rows, "d": d, "ff": ff, "world": world}
    _native.check_status()
    with open(os.path.join(os.environ["TP_RESULT_DIR"], f"rank{rank}.json"), "w") as f:
        json.dump(res, f)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
