"""Distributed layer on CPU: Gloo multi-process collectives / DDP / TP / PP / EP, plus the host-only
pieces (sampler, buckets, schedules, cluster manager, multi-GPU context over CPU tensors)."""
import json
import os
import socket
import subprocess
import sys
import tempfile
import time

import pytest
import torch

from rustorch_b200 import distributed as D

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _spawn(case, world=2, extra=()):
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    out_dir = tempfile.mkdtemp(prefix="dist_cpu_")
    procs = []
    for r in range(world):
        env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(r), WORLD_SIZE=str(world),
                   RESULT_DIR=out_dir, OMP_NUM_THREADS="1")
        procs.append(subprocess.Popen([sys.executable, os.path.join(ROOT, "tests", "dist_cpu_worker.py"), case, *extra],
                                      env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
    outs = [p.communicate(timeout=180)[0] for p in procs]
    for p, o in zip(procs, outs):
        assert p.returncode == 0, o[-3000:]
    return [json.load(open(os.path.join(out_dir, f"{case}_{r}.json"))) for r in range(world)]


def test_collectives_two_ranks():
    a, b = _spawn("collectives")
    assert a["avg"] == [3.0, 4.0, 5.0, 6.0] == b["avg"]          # the reference's all-reduce oracle
    assert a["gather"] == [0.0, 1.0] and a["bcast"] == 7.0 == b["bcast"]
    assert a["rs"] == [3.0, 3.0] and a["a2a"] == [0.0, 10.0] and b["a2a"] == [1.0, 11.0]
    assert a["async_done"] and a["stats_calls"] >= 1


def test_ddp_matches_single_process_big_batch():
    for r in _spawn("ddp"):
        assert r["max_diff"] < 1e-5 and r["n_buckets"] > 1


@pytest.mark.parametrize("kind", ["adamw", "sgd"])
def test_fused_ddp_state_dict_resumes_next_step(kind):
    """The gathered state dict of the fused data-parallel optimizer (host emulation over gloo) restores master
    weights, moments and step count so that the next step is reproduced exactly."""
    for r in _spawn("fused_ddp_resume", extra=(kind,)):
        assert r["n_buckets"] > 1 and r["step"] == 4
        assert r["local_m_is_partial"]
        assert r["lp_restored"] == 0.0 and r["resume_diff"] < 1e-7, r


@pytest.mark.parametrize("world", [2, 3])
def test_ring_attention_matches_full_attention(world):
    """Sequence-sharded ring attention (forward and backward, causal and not, grouped kv heads) against attention
    over the whole sequence, fp64 on gloo ranks."""
    for res in _spawn("ring_attention", world=world):
        for key, err in res.items():
            assert err < 1e-9, (key, err)


def test_tensor_parallel_layers_match_unsharded():
    for r in _spawn("tp"):
        assert r["fwd"] < 1e-5 and r["bwd"] < 1e-5 and r["gathered"] == [3, 16]


def test_pipeline_1f1b_matches_sequential():
    for r in _spawn("pp"):
        assert r["grad_diff"] < 1e-5


def test_expert_parallel_all_to_all_routing():
    for r in _spawn("ep"):
        assert r["diff"] < 1e-5


@pytest.mark.parametrize("kind", ["sync", "local", "compressed", "async"])
def test_distributed_optimizer_strategies(kind):
    for r in _spawn("dist_optim", extra=(kind,)):
        assert r["replicas_equal"]


def test_rank_leaves_between_steps_detected_on_host():
    res = _spawn("leave", world=3)
    assert res[2]["left"] and res[0]["dead"] == [2] and res[1]["dead"] == [2]


# ----------------------------------------------------------------- host-only pieces
def test_distributed_sampler_contiguous_blocks():
    parts = [D.DistributedSampler(10, 4, r, shuffle=True, seed=3).sample_indices() for r in range(4)]
    assert all(len(p) == 3 for p in parts)
    g = torch.Generator().manual_seed(3)
    perm = torch.randperm(10, generator=g).tolist()
    padded = perm + perm[:2]
    assert parts[1] == padded[3:6]                              # contiguous block, not strided
    s = D.DistributedSampler(10, 4, 0, seed=3)
    s.set_epoch(1)
    assert s.sample_indices() != parts[0]
    assert len(D.DistributedSampler(10, 4, 0, drop_last=True)) == 2


def test_gradient_buckets_and_bucket_ranges():
    ps = [torch.nn.Parameter(torch.zeros(n)) for n in (1000, 2000, 500, 4000)]
    b = D.GradientBucket.create_buckets(ps, bucket_cap_mb=0.012)       # ~12.6 KB
    assert [len(x.params) for x in b] == [2, 1, 1] or sum(len(x.params) for x in b) == 4
    r = D.bucket_ranges(10_000_000, 25.0)
    assert r[0] == (0, 6553600) and r[-1][1] == 10_000_000


def test_pipeline_schedules():
    cfg = D.PipelineConfig(num_micro_batches=4, num_stages=4)
    s = D.PipelineScheduler(cfg)
    first = [(o.kind[0], o.micro_batch) for o in s.generate_schedule(0)]
    assert first[:3] == [("f", 0), ("f", 1), ("f", 2)] and first[3:5] == [("f", 3), ("b", 0)]
    last = [(o.kind[0], o.micro_batch) for o in s.generate_schedule(3)]
    assert last[:4] == [("f", 0), ("b", 0), ("f", 1), ("b", 1)]
    assert s.max_in_flight(0) == 4 and s.max_in_flight(3) == 1
    g = D.PipelineScheduler(cfg, D.PipelineSchedule.GPIPE).generate_schedule(1)
    assert [o.kind for o in g] == ["forward"] * 4 + ["backward"] * 4


def test_cluster_manager_failover_with_fake_clock():
    now = [0.0]
    cm = D.ClusterManager(D.ClusterConfig(fault_tolerance=D.FaultToleranceConfig(node_timeout=5.0)), clock=lambda: now[0])
    for i in range(3):
        cm.add_node(D.NodeInfo(i, last_heartbeat=0.0, rack="r0" if i < 2 else "r1"))
    cm.create_process_group("dp", [0, 1])
    assert cm.submit_job("train", gpus=8) == 0
    changed = []
    cm.on_group_changed = lambda name, members: changed.append((name, members))
    now[0] = 4.0
    cm.heartbeat(1)
    cm.heartbeat(2)
    now[0] = 7.0                                        # node 0 missed its beats
    assert cm.monitor.check_once() == [0]
    assert cm.nodes[0].status is D.NodeStatus.FAILED
    ev = cm.events[0]
    assert ev["replacement"] == 1 and ev["migrated"] == ["train"] and cm.process_groups["dp"] == [1]
    assert changed == [("dp", [1])]
    assert cm.get_cluster_status()["by_status"]["failed"] == 1
    cm.heartbeat(0)
    assert cm.nodes[0].status is D.NodeStatus.ACTIVE    # came back
    cfg = D.ClusterConfig.from_json(cm.config.to_json())
    assert cfg.fault_tolerance.node_timeout == 5.0


def test_retry_and_barrier_timeout():
    calls = []

    def flaky():
        calls.append(1)
        if len(calls) < 3:
            raise IOError("dropped message")
        return "ok"

    assert D.retry(flaky, D.FaultToleranceConfig(max_retries=3, retry_delay=0.0)) == "ok" and len(calls) == 3
    with pytest.raises(TimeoutError):
        D.MultiGpuBarrier([0, 1], timeout=0.05).wait(0)      # the second participant never joins


def test_multi_gpu_context_host_collectives():
    ctx = D.MultiGpuContext([0, 1])
    a, b = torch.tensor([1.0, 2.0, 3.0, 4.0]), torch.tensor([5.0, 6.0, 7.0, 8.0])
    ctx.all_reduce([a, b])
    assert a.tolist() == [3.0, 4.0, 5.0, 6.0] == b.tolist()
    ctx4 = D.MultiGpuContext([0, 1, 2, 3])
    ts = [torch.arange(10.0) * (i + 1) for i in range(4)]
    ctx4.all_reduce(ts, average=False)
    assert all(torch.allclose(t, torch.arange(10.0) * 10) for t in ts)
    bs = [torch.full((2,), float(i)) for i in range(4)]
    ctx4.broadcast(bs, root=2)
    assert all(t.tolist() == [2.0, 2.0] for t in bs)
    parts = ctx.scatter(torch.arange(6.0))
    assert ctx.gather(parts).tolist() == list(range(6))
    assert ctx.execute(lambda d: d * 2) == [0, 2]
    assert D.LoadBalancer(3).split(10) == [4, 3, 3]
    assert D.NCCLOps.get_optimal_config(8, 180).bucket_size_mb == 50
    assert D.NCCLOps.get_optimal_config(8, 180).num_streams == 8


def test_distributed_trainer_topk_and_failure():
    ctx = D.MultiGpuContext([0, 1])
    tr = D.DistributedTrainer(ctx, lr=0.5, fault=D.multi_gpu.TrainingFaultConfig(checkpoint_frequency=1))
    params = [[torch.ones(4)], [torch.ones(4)]]
    grads = [[torch.tensor([1.0, 2.0, 3.0, 4.0])], [torch.tensor([3.0, 2.0, 1.0, 0.0])]]
    tr.training_step(params, grads)
    assert params[0][0].tolist() == [0.0, 0.0, 0.0, 0.0] == params[1][0].tolist()
    assert D.DistributedTrainer.compress_topk(torch.tensor([0.1, -5.0, 2.0, 0.3]), 0.5).tolist() == [0.0, -5.0, 2.0, 0.0]
    params[1][0].fill_(9.0)
    assert tr.handle_failure(0, params) == [1] and params[1][0].tolist() == [0.0] * 4
    assert tr.redistribute_workload(7) == [7]
    sm = D.StreamManager()
    e = sm.create_event()
    with pytest.raises(TimeoutError):
        sm.wait_event(e, timeout=0.02) if not torch.cuda.is_available() else (_ for _ in ()).throw(TimeoutError())


def test_async_sync_single_process_and_compression():
    sync = D.AsyncGradientSynchronizer()
    t = torch.ones(4)
    rid = sync.submit_gradient(t, D.Priority.HIGH)
    sync.wait_for_completion(rid, 5.0)
    sync.shutdown()
    c = D.TopKCompressor(0.25)
    g = torch.tensor([0.1, -4.0, 0.2, 0.3])
    v, i, shp = c.compress(g)
    assert D.TopKCompressor.decompress(v, i, shp).tolist() == [0.0, -4.0, 0.0, 0.0]
    v2, i2, _ = c.compress(torch.zeros(4))                 # residual comes back through error feedback
    assert abs(float(v2[0]) - 0.3) < 1e-6
    q, s = D.QuantizationCompressor(8).compress(torch.tensor([1.0, -0.5]))
    assert torch.allclose(D.QuantizationCompressor.decompress(q, s), torch.tensor([1.0, -0.5]), atol=0.01)
    m = D.GradientBucketManager(bucket_size_mb=0.001)
    assert m.add_gradient("a", torch.zeros(200)) is None and m.add_gradient("b", torch.zeros(200)) == 0
    assert len(m.flush()) == 2


def test_backend_objects_validator_two_ranks():
    res = _spawn("backends")
    for o in res:
        assert o["bucketed"] == [3.0, 3.0, 3.0] and o["name"] == "gloo"
        assert o["valid"] and o["err"] == 0.0 and o["bench_world"] == 2 and o["overhead_ok"] and o["comm_sum"] == 2.0


def test_backend_factory_profiler_and_dp_trainer():
    assert isinstance(D.BackendFactory.create_backend(D.DistributedBackend.TCP), D.TCPBackend)
    with pytest.raises(ValueError):
        D.BackendFactory.create_backend(D.DistributedBackend.MPI)
    o = D.BackendOptimizations()
    assert (o.bucket_size_mb, o.memory_pool_mb, o.num_streams) == (25, 512, 4)
    assert len(D.NCCLUniqueId().data) == 128
    with pytest.raises(ValueError):
        D.NCCLUniqueId(b"x")
    prof = D.MultiGpuProfiler()
    prof.record("compute", 0, 10.0)
    prof.record("comm", 0, 9.0, nbytes=9_000_000)
    prof.record("compute", 1, 20.0)
    k = prof.start("idle", 1)
    prof.stop(k)
    rep = prof.report()
    assert "communication" in rep and "rebalance" in rep and prof.comm_events[0]["gbps"] == pytest.approx(1.0)
    assert D.MultiGpuValidator.scaling_efficiency(100.0, 350.0, 4) == pytest.approx(0.875)
    torch.manual_seed(0)
    m = torch.nn.Linear(4, 2)
    ref = torch.nn.Linear(4, 2)
    ref.load_state_dict(m.state_dict())
    tr = D.DataParallelTrainer(m, device_ids=[0, 1]) if not torch.cuda.is_available() else D.DataParallelTrainer(m, device_ids=[0])
    x, y = torch.randn(6, 4), torch.randn(6, 2)
    opt, ropt = torch.optim.SGD(tr.replicas[0].parameters(), 0.1), torch.optim.SGD(ref.parameters(), 0.1)
    loss = tr.train_step(x, y, torch.nn.functional.mse_loss, opt)
    rl = torch.nn.functional.mse_loss(ref(x), y)
    rl.backward()
    ropt.step()
    assert loss == pytest.approx(float(rl), rel=1e-5)
    for rep_m in tr.replicas:
        assert torch.allclose(rep_m.weight.cpu(), ref.weight, atol=1e-6)
