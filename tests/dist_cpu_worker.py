"""Gloo worker for the CPU multi-process tests (spawned by test_distributed_cpu.py)."""
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from rustorch_b200 import distributed as D  # noqa: E402
from rustorch_b200 import optim  # noqa: E402


def main():
    case = sys.argv[1]
    out = {}
    pg = D.init_process_group("gloo", timeout=60)
    r, W = pg.rank, pg.world_size
    if case == "collectives":
        t = torch.tensor([1.0, 2.0, 3.0, 4.0]) + 4.0 * r
        D.all_reduce(t, D.ReduceOp.AVERAGE)
        out["avg"] = t.tolist()
        g = D.all_gather(torch.tensor([float(r)]))
        out["gather"] = [float(x) for x in g]
        b = torch.tensor([float(r + 7)])
        D.broadcast(b, 0)
        out["bcast"] = float(b)
        o = torch.zeros(2)
        D.reduce_scatter(o, [torch.ones(2) * (r + 1) for _ in range(W)])
        out["rs"] = o.tolist()
        outs = [torch.zeros(1) for _ in range(W)]
        D.all_to_all(outs, [torch.tensor([float(10 * r + p)]) for p in range(W)])
        out["a2a"] = [float(x) for x in outs]
        req = D.all_reduce(torch.ones(3), async_op=True)
        req.wait()
        out["async_done"] = req.is_completed()
        out["stats_calls"] = D.monitoring.get_communication_stats().calls.get("all_reduce", 0)
    elif case == "ring_attention":
        from rustorch_b200.distributed.context_parallel import gather_sequence, ring_attention, shard_sequence
        g = torch.Generator().manual_seed(5)
        B, T, H, Hkv, Dh = 2, 8 * W, 4, 2, 16
        q = torch.randn(B, T, H, Dh, generator=g, dtype=torch.float64)
        k = torch.randn(B, T, Hkv, Dh, generator=g, dtype=torch.float64)
        v = torch.randn(B, T, Hkv, Dh, generator=g, dtype=torch.float64)
        go = torch.randn(B, T, H, Dh, generator=g, dtype=torch.float64)
        for causal in (False, True):
            # oracle: full attention on every rank
            qf, kf, vf = (t.clone().requires_grad_(True) for t in (q, k, v))
            s = (qf.transpose(1, 2) @ kf.repeat_interleave(H // Hkv, 2).transpose(1, 2).transpose(-1, -2)) / Dh ** 0.5
            if causal:
                s = s.masked_fill(torch.ones(T, T, dtype=torch.bool).triu(1), float("-inf"))
            ref = (torch.softmax(s, -1) @ vf.repeat_interleave(H // Hkv, 2).transpose(1, 2)).transpose(1, 2)
            ref.backward(go)
            ql, kl, vl = (shard_sequence(t).requires_grad_(True) for t in (q, k, v))
            att = ring_attention(ql, kl, vl, causal=causal)
            att.backward(shard_sequence(go))
            tag = "causal" if causal else "full"
            out[f"{tag}_fwd"] = float((gather_sequence(att.detach()) - ref.detach()).abs().max())
            out[f"{tag}_dq"] = float((gather_sequence(ql.grad) - qf.grad).abs().max())
            out[f"{tag}_dk"] = float((gather_sequence(kl.grad) - kf.grad).abs().max())
            out[f"{tag}_dv"] = float((gather_sequence(vl.grad) - vf.grad).abs().max())
    elif case == "backends":
        be = D.BackendFactory.create_backend(D.DistributedBackend.GLOO, optimizations=D.BackendOptimizations(bucket_size_mb=1))
        ts = [torch.full((n,), float(r + 1)) for n in (3, 300_000, 5)]
        be.all_reduce_bucketed(ts)
        out["bucketed"] = [float(t[0]) for t in ts]
        out["name"] = be.name
        rep = D.MultiGpuValidator().validate_distributed(torch.device("cpu"))
        out["valid"], out["err"] = rep.collectives_ok, rep.max_error
        x = torch.ones(1000)
        sb = D.MultiGpuValidator().benchmark(lambda: x.mul(2.0), lambda: be.all_reduce(x.clone()), 10, iters=2)
        out["bench_world"], out["overhead_ok"] = sb.world_size, 0.0 <= sb.comm_overhead <= 1.0
        comm = D.NCCLCommunicator(0, r, W, num_streams=0)
        out["comm_sum"] = float(comm.all_reduce(torch.tensor([1.0]))[0])
    elif case == "ddp":
        torch.manual_seed(0)
        model = torch.nn.Sequential(torch.nn.Linear(8, 16), torch.nn.ReLU(), torch.nn.Linear(16, 4))
        ddp = D.DistributedDataParallel(model, bucket_cap_mb=0.0005)
        ref = torch.nn.Sequential(torch.nn.Linear(8, 16), torch.nn.ReLU(), torch.nn.Linear(16, 4))
        ref.load_state_dict(model.state_dict())
        g = torch.Generator().manual_seed(1)
        X, Y = torch.randn(W * 4, 8, generator=g), torch.randn(W * 4, 4, generator=g)
        opt, ropt = torch.optim.SGD(model.parameters(), 0.1), torch.optim.SGD(ref.parameters(), 0.1)
        for _ in range(3):
            opt.zero_grad()
            torch.nn.functional.mse_loss(ddp(X[r * 4:(r + 1) * 4]), Y[r * 4:(r + 1) * 4]).backward()
            ddp.sync_gradients()
            opt.step()
            ropt.zero_grad()
            torch.nn.functional.mse_loss(ref(X), Y).backward()
            ropt.step()
        out["max_diff"] = max(float((a - b).abs().max()) for a, b in zip(model.parameters(), ref.parameters()))
        out["n_buckets"] = len(ddp.buckets)
    elif case == "tp":
        torch.manual_seed(0)
        full1, full2 = torch.randn(16, 8) * 0.1, torch.randn(8, 16) * 0.1
        tp = D.TensorParallel(W, r)
        col = D.ColumnParallelLinear(8, 16, tp, bias=False)
        row = D.RowParallelLinear(16, 8, tp, bias=False)
        with torch.no_grad():
            col.weight.copy_(D.TensorParallel(W, r, 0).split_tensor(full1))
            row.weight.copy_(D.TensorParallel(W, r, 1).split_tensor(full2))
        x = torch.randn(3, 8, generator=torch.Generator().manual_seed(2), requires_grad=True)
        y = row(torch.relu(col(x)))
        y.sum().backward()
        xr = x.detach().clone().requires_grad_(True)
        yr = torch.relu(xr @ full1.t()) @ full2.t()
        yr.sum().backward()
        out["fwd"] = float((y - yr).abs().max())
        out["bwd"] = float((x.grad - xr.grad).abs().max())
        out["gathered"] = list(tp.gather_tensors(col(x.detach())).shape)
    elif case == "pp":
        torch.manual_seed(0)
        l1, l2 = torch.nn.Linear(4, 6), torch.nn.Linear(6, 2)
        cfg = D.PipelineConfig(num_micro_batches=4, num_stages=2)
        g = torch.Generator().manual_seed(3)
        X, Y = torch.randn(8, 4, generator=g), torch.randn(8, 2, generator=g)
        xs, ys = list(X.chunk(4)), list(Y.chunk(4))
        stage = D.PipelineStage(l1 if r == 0 else l2, r, cfg)
        losses = stage.run(xs if r == 0 else None, torch.nn.functional.mse_loss, ys if r == 1 else None,
                           act_shape=(2, 6))
        ref1, ref2 = torch.nn.Linear(4, 6), torch.nn.Linear(6, 2)
        ref1.load_state_dict(l1.state_dict()) if r == 0 else None
        mine = l1 if r == 0 else l2
        # reference: both layers are seeded identically on both ranks (same manual_seed above)
        torch.manual_seed(0)
        a, b = torch.nn.Linear(4, 6), torch.nn.Linear(6, 2)
        sum(torch.nn.functional.mse_loss(b(a(x)), y) / 4 for x, y in zip(xs, ys)).backward()
        refm = a if r == 0 else b
        out["grad_diff"] = float((mine.weight.grad - refm.weight.grad).abs().max())
        out["n_losses"] = len(losses)
    elif case == "ep":
        torch.manual_seed(0)
        experts_all = [torch.nn.Linear(4, 4) for _ in range(W)]
        ep = D.ExpertParallel(W, 1, r, [experts_all[r]], d_model=4, top_k=1)
        torch.manual_seed(5)
        gate = torch.nn.Linear(4, W, bias=False)
        ep.gate.load_state_dict(gate.state_dict())
        x = torch.randn(6, 4, generator=torch.Generator().manual_seed(10 + r))
        with torch.no_grad():
            y = ep.route_tokens(x)
            idx = (x @ gate.weight.t()).argmax(-1)
            ref = torch.stack([experts_all[int(e)](t) for t, e in zip(x, idx)])
        out["diff"] = float((y - ref).abs().max())
    elif case == "dist_optim":
        torch.manual_seed(0)
        m = torch.nn.Linear(4, 2)
        for p in m.parameters():
            D.broadcast(p.data, 0)
        kind = sys.argv[2]
        strat = {"sync": D.SyncStrategy.Synchronous(), "local": D.SyncStrategy.LocalSGD(2),
                 "compressed": D.SyncStrategy.Compressed(0.5), "async": D.SyncStrategy.Asynchronous()}[kind]
        do = D.DistributedOptimizer(torch.optim.SGD(m.parameters(), 0.1), strat, bucket_size_mb=0.0001)
        for s in range(2):
            do.zero_grad()
            (m(torch.ones(1, 4) * (r + 1)).sum()).backward()
            do.step()
        ws = D.all_gather(m.weight.data.reshape(-1))
        out["replicas_equal"] = all(torch.allclose(ws[0], w, atol=1e-6) for w in ws)
    elif case == "fused_ddp_resume":
        # host emulation of the fused data-parallel step: ownership, gathered state dict, resume, other optimizers
        from rustorch_b200.distributed.fused_allreduce import FusedDDP
        kind = sys.argv[2]

        def make():
            torch.manual_seed(0)
            return torch.nn.Sequential(torch.nn.Linear(8, 32), torch.nn.Tanh(), torch.nn.Linear(32, 4)).to(torch.bfloat16)

        def run_step(model, ddp, it):
            g = torch.Generator().manual_seed(100 + it * W + r)
            x, y = torch.randn(4, 8, generator=g).bfloat16(), torch.randn(4, 4, generator=g).bfloat16()
            loss = ((model(x) - y).float() ** 2).mean()
            loss.backward()
            ddp.step()

        kw = dict(optimizer=kind, lr=0.05, weight_decay=0.01, bucket_cap_mb=0.0005)
        if kind == "sgd":
            kw.update(momentum=0.9, decay_all=True)
        m1 = make()
        d1 = FusedDDP(m1, **kw)
        for it in range(3):
            run_step(m1, d1, it)
        sd = d1.state_dict()
        out["n_buckets"] = d1.n_buckets
        # moments outside this rank's slices are stale locally but complete in the gathered dictionary
        if d1.m is not None:
            out["local_m_is_partial"] = bool((d1.m != sd["exp_avg"]).any())
        run_step(m1, d1, 3)
        want = d1.gather_master().clone()
        d1.close()
        m2 = make()
        d2 = FusedDDP(m2, **kw)
        d2.load_state_dict(sd)
        out["lp_restored"] = float((d2.flat.lp.float() - sd["master"].bfloat16().float()).abs().max())
        run_step(m2, d2, 3)
        out["resume_diff"] = float((d2.gather_master() - want).abs().max())
        out["step"] = d2.step_count
        # single-process oracle: same global batch through a plain fp32-master update
        d2.close()
    elif case == "leave":
        # rank W-1 leaves between steps; the others learn it from the store heartbeat before their next collective
        import torch.distributed as dist
        store = dist.distributed_c10d._get_default_store()
        hb = D.StoreHeartbeat(store, r, W, timeout=1.0)
        hb.beat()
        D.barrier()
        if r == W - 1:
            out["left"] = True
        else:
            import time
            time.sleep(1.5)
            hb.beat()
            out["dead"] = hb.dead_ranks()
    with open(os.path.join(os.environ["RESULT_DIR"], f"{case}_{r}.json"), "w") as f:
        json.dump(out, f)
    if case != "leave":
        D.barrier()
        D.destroy_process_group()


if __name__ == "__main__":
    main()
