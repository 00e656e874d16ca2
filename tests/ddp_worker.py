"""Worker for the multi-GPU data-parallel tests (launched by torch.distributed.run).

Every rank trains the same tiny GPT on its own batches with the fused peer-memory bucket kernel
and, in the same process, replays the job as one big-batch single-GPU run (gradients of all
ranks' batches averaged) with the plain fused AdamW.  Writes one JSON file per rank into $DDP_RESULT_DIR.
"""
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    mode = sys.argv[1] if len(sys.argv) > 1 else "fused"
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    from rustorch_b200 import _native
    from rustorch_b200.models.gpt import GPT, GPTConfig
    from rustorch_b200.optim.flat import FlatParams, FusedAdamW, FusedSGD
    from rustorch_b200.distributed.fused_allreduce import FusedDDPAdamW, FusedDDPSGD
    from rustorch_b200.distributed.ddp_flat import FlatDDP

    cfg = GPTConfig(vocab_size=512, n_positions=128, n_embd=256, n_layer=2, n_head=4, dropout=0.0)
    steps, B, T = 6, 4, 128
    gen = torch.Generator().manual_seed(7)
    data = torch.randint(0, cfg.vocab_size, (steps, world, B, T + 1), generator=gen).to(dev)
    sgd = mode.endswith("_sgd")
    hp = dict(lr=0.05, momentum=0.9, weight_decay=1e-4) if sgd else dict(lr=1e-3, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)

    # --- single-GPU big-batch replay (oracle)
    ref = GPT(cfg, device=dev, dtype=torch.bfloat16, seed=3)
    rflat = FlatParams(ref)
    init = rflat.master.clone()
    ropt = FusedSGD(rflat, **hp) if sgd else FusedAdamW(rflat, **hp)
    ropt.grad_scale = 1.0 / world
    ref_losses = []
    for s in range(steps):
        tot = 0.0
        for r in range(world):
            b = data[s, r]
            loss = ref(b[:, :-1], b[:, 1:])
            loss.backward()
            tot += float(loss)
        ropt.step()
        ref_losses.append(tot / world)
    ref_master = rflat.named_views(rflat.master)

    # --- data-parallel run
    model = GPT(cfg, device=dev, dtype=torch.bfloat16, seed=3)
    losses = []
    nvls_used = False
    rollback = None
    if mode == "public":
        # the public wrapper in fused mode: forward through the wrapper, step() instead of sync_gradients + optimizer
        from rustorch_b200.distributed.ddp import DistributedDataParallel
        wrap = DistributedDataParallel(model, bucket_cap_mb=1.0, fused_optimizer=dict(optimizer="adamw", timeout_s=10.0, **hp))
        for s in range(steps):
            b = data[s, rank]
            loss = wrap(b[:, :-1], b[:, 1:])
            loss.backward()
            wrap.step()
            losses.append(float(loss))
        _native.check_status()
        got = wrap.fused.flat.named_views(wrap.fused.gather_master())
        n_buckets = wrap.fused.n_buckets
        nvls_used = wrap.fused.nvls
        wrap.fused.close()
    elif mode.startswith("fused"):
        # "fused" / "fused_sgd": plain peer loads and stores; "fused_nvls" / "fused_nvls_sgd": multimem through the switch
        kw = dict(bucket_cap_mb=1.0, timeout_s=10.0, use_nvls="nvls" in mode, **hp)
        ddp = FusedDDPSGD(model, **kw) if sgd else FusedDDPAdamW(model, **kw)
        nvls_used = ddp.nvls
        for s in range(steps):
            b = data[s, rank]
            loss = model(b[:, :-1], b[:, 1:])
            loss.backward()
            ddp.step()
            losses.append(float(loss))
        _native.check_status()
        full = ddp.gather_master()
        got = ddp.flat.named_views(full)
        n_buckets = ddp.n_buckets
        if mode in ("fused", "fused_sgd"):
            # roll back in place: two more steps, restore the state from before them (the step count, which the
            # cross-rank flag words carry, goes back by two), repeat the same two steps
            sd = ddp.state_dict()

            def two_steps():
                for s in (0, 1):
                    b = data[s, rank]
                    model(b[:, :-1], b[:, 1:]).backward()
                    ddp.step()
                _native.check_status()
                return ddp.gather_master().clone()

            first = two_steps()
            ddp.load_state_dict(sd)
            second = two_steps()
            moved = (first - full).abs().mean().clamp_min(1e-12)
            rollback = float((second - first).abs().mean() / moved)
        ddp.close()
    else:
        flat = FlatParams(model)
        opt = FusedAdamW(flat, **hp)
        opt.grad_scale = 1.0 / world
        nddp = FlatDDP(flat, bucket_cap_mb=1.0)
        nddp.broadcast_parameters()
        for s in range(steps):
            b = data[s, rank]
            loss = model(b[:, :-1], b[:, 1:])
            loss.backward()
            nddp.sync_gradients()
            opt.step()
            losses.append(float(loss))
        got = flat.named_views(flat.master)
        n_buckets = len(nddp.buckets)

    # averaged loss across ranks must follow the big-batch run
    lt = torch.tensor(losses, device=dev)
    dist.all_reduce(lt)
    lt /= world
    init_v = rflat.named_views(init)
    worst, per_name = 0.0, []
    for name in ref_master:
        upd = (ref_master[name] - init_v[name]).abs().mean().clamp_min(1e-12)
        diff = (got[name].to(dev) - ref_master[name]).abs().mean()
        worst = max(worst, float(diff / upd))
        per_name.append((round(float(diff / upd), 4), name))
    per_name.sort(reverse=True)
    out = {"rank": rank, "world": world, "mode": mode, "n_buckets": n_buckets,
           "loss_ddp": [round(float(x), 4) for x in lt], "loss_ref": [round(x, 4) for x in ref_losses],
           "worst_rel_update_diff": round(worst, 4), "nvls": nvls_used, "worst_params": per_name[:6],
           "rollback_rel_diff": rollback}
    # one file per rank: lines printed by several ranks to a shared pipe can interleave
    with open(os.path.join(os.environ["DDP_RESULT_DIR"], f"rank{rank}.json"), "w") as f:
        json.dump(out, f)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
