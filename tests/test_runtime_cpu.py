"""CPU tests: native host runtime (arena, planner), memory pools, gpu device layer, dynamic execution."""
import pytest
import torch

from rustorch_b200 import _native, execution as E, gpu as G, memory as M


def test_arena_best_fit_coalescing_and_stats():
    A = _native.host().Arena(4096, 256)
    a, b, c = A.allocate(100), A.allocate(300), A.allocate(256)
    assert (a, b, c) == (0, 256, 768) and A.size_of(b) == 512
    A.release(b)
    assert A.allocate(600) == 1024            # does not fit the 512-byte hole
    assert A.allocate(512) == 256             # best fit reuses the hole exactly
    A.release(a)
    A.release(256)
    st = A.stats()
    assert st["free_ranges"] == 2 and st["live_blocks"] == 2 and st["peak"] >= st["in_use"]
    assert A.allocate(1 << 20) == -1 and A.stats()["n_fail"] == 1
    with pytest.raises(ValueError):
        A.release(12345)
    A.reset()
    assert A.stats()["in_use"] == 0 and A.allocate(4096) == 0
    with pytest.raises(ValueError):
        _native.host().Arena(100, 3)


def test_arena_random_stress_never_overlaps():
    import random
    rnd = random.Random(0)
    A = _native.host().Arena(1 << 16, 64)
    live = {}
    for _ in range(2000):
        if live and rnd.random() < 0.45:
            off = rnd.choice(list(live))
            A.release(off)
            del live[off]
        else:
            n = rnd.randint(1, 3000)
            off = A.allocate(n)
            if off >= 0:
                size = A.size_of(off)
                assert size >= n and off % 64 == 0
                for o, s in live.items():
                    assert off + size <= o or o + s <= off
                live[off] = size
    assert A.stats()["in_use"] == sum(live.values())
    for off in list(live):
        A.release(off)
    st = A.stats()
    assert st["in_use"] == 0 and st["free_ranges"] == 1 and st["largest_free"] == 1 << 16


def test_planner_order_levels_memory_dead_chains():
    P = _native.host().ExecutionPlan()
    x = P.add_node("input", [], 1000)
    w = P.add_node("input", [], 4000)
    h = P.add_node("linear", [x, w], 2000)
    r = P.add_node("relu", [h], 2000)
    e = P.add_node("exp", [r], 2000)
    unused = P.add_node("sigmoid", [h], 2000)
    y = P.add_node("matmul", [e, w], 500)
    P.mark_output(y)
    assert list(P.topo_order()) == [0, 1, 2, 3, 4, 5, 6]
    assert [sorted(l) for l in P.levels()] == [[0, 1], [2], [3, 5], [4], [6]]
    assert list(P.eliminate_dead()) == [unused]
    offsets, (total, naive) = P.memory_plan(256)
    assert total < naive and all(o >= 0 for o in offsets)
    # buffers alive at the same time never overlap
    order = list(P.topo_order())
    last = {i: i for i in order}
    for i in order:
        for j in P.node(i).inputs:
            last[j] = max(last[j], i)
    last[y] = 99
    size = lambda i: -(-P.node(i).out_bytes // 256) * 256
    for i in order:
        for j in order:
            if i < j and not (last[i] < j or last[j] < i):
                assert offsets[i] + size(i) <= offsets[j] or offsets[j] + size(j) <= offsets[i], (i, j)
    assert [list(c) for c in P.fusible_chains()] == [[3, 4]]
    with pytest.raises(ValueError):
        P.add_node("add", [42], 0)


def test_memory_pools_and_analytics():
    p = M.EnhancedMemoryPool(1 << 16)
    a = p.allocate((16, 16))
    b = p.zeros((100,), torch.float16)
    assert p.owns(a) and a.shape == (16, 16) and float(b.sum()) == 0 and p.stats()["live_blocks"] == 2
    a.fill_(3.0)
    assert float(b.float().sum()) == 0                   # blocks do not alias
    p.deallocate(a)
    with pytest.raises(ValueError):
        p.deallocate(a)
    c, d = p.intern(torch.arange(10.0)), p.intern(torch.arange(10.0))
    assert c.data_ptr() == d.data_ptr() and p.dedup_hits == 1
    p.release_interned(c)
    p.release_interned(d)
    del b
    assert p.garbage_collect() == 1 and p.stats()["in_use"] == 0
    with pytest.raises(M.PoolExhausted):
        p.allocate((1 << 20,))
    an = M.MemoryAnalytics()
    h1 = an.on_alloc(1000, "act", now=0.0)
    an.on_alloc(5000, "weights", now=1.0)
    an.on_free(h1, now=2.0)
    assert an.peak_live_bytes() == 6000 and an.mean_lifetime_s() == 2.0 and an.hotspots(1)[0][0] == "weights"
    assert len(an.leaks(older_than_s=10, now=100.0)) == 1
    mon = M.AdaptivePressureMonitor()
    for i, u in enumerate([0.3, 0.5, 0.7, 0.9]):
        mon.feed(u, now=float(i))
    assert mon.level() in ("high", "critical") and 0 < mon.seconds_to_exhaustion() < 1
    assert any("failed" in r for r in M.MemoryOptimizer.recommend(p.stats()))


def test_device_layer_cpu():
    mgr = G.get_device_manager()
    assert G.DeviceType.Cpu() in mgr.available_devices() and not G.DeviceType.Metal().is_available()
    with pytest.raises(G.DeviceNotAvailable):
        mgr.set_device(G.DeviceType.Metal())
    G.set_device(G.DeviceType.Cpu())
    assert G.current_device() == G.DeviceType.Cpu() and mgr.current_context().stream_count() == 0
    cache = G.DeviceCache(ttl_s=100)
    assert cache.is_device_available(G.DeviceType.Cpu()) and cache.is_device_available(G.DeviceType.Cpu())
    assert cache.get_stats() == {"entries": 1, "hits": 1, "misses": 1}
    sel = G.SmartDeviceSelector([G.DeviceType.Cpu(), G.DeviceType.Cuda(0)])
    small = G.OperationProfile(G.OperationType.MATMUL, [8, 8])
    big = G.OperationProfile(G.OperationType.MATMUL, [1024, 1024])
    assert sel.select_device(small) == G.DeviceType.Cpu() and sel.select_device(big) == G.DeviceType.Cuda(0)
    assert sel.get_fallback_chain(big)[0] == G.DeviceType.Cuda(0) and big.memory_footprint() == 4 << 20
    hy = G.HybridExecutor(sel)

    def run(dev):
        if dev.type == "cuda":
            raise RuntimeError("no gpu here")
        return "cpu result"
    assert hy.execute(big, run) == "cpu result" and hy.fallbacks == 1
    po = G.PerformanceOptimizer()
    po.feed({"temperature_c": 90})
    assert po.strategy() == "throttle" and po.recommendations()
    res = G.GpuValidator(1e-4).validate_all_devices()
    assert all(r.passed for r in res if r.device == "cpu") and "passed" in G.GpuValidator().generate_report(res)
    ex = G.UnifiedKernelExecutor(G.DeviceType.Cpu())
    out = ex.execute(G.KernelOp.ADD, torch.ones(4), torch.ones(4))
    assert out.tolist() == [2.0] * 4 and ex.get_metrics().launches == 1
    ks = G.KernelSelector()
    ks.add_executor(ex)
    assert float(ks.execute(G.KernelOp.SUM, torch.arange(5.0))) == 10.0
    xfer = G.DataTransfer(G.DeviceType.Cpu())
    assert torch.equal(xfer.to_host(xfer.to_device(torch.arange(3.0))), torch.arange(3.0)) and xfer.bytes_h2d == 12


def test_custom_kernel_manager_compiles_for_sm100a(tmp_path):
    mgr = G.CustomKernelManager(G.DeviceType.Cpu(), cache_dir=str(tmp_path))
    cfg = G.KernelConfig("saxpy", 'extern "C" __global__ void saxpy(float* y, const float* x, long long n, float a)'
                                  "{ long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; if (i < n) y[i] += a * x[i]; }")
    cubin = mgr.compile_kernel(cfg)
    assert cubin.endswith(".cubin") and mgr.get_kernel_stats("saxpy").compile_ms > 0
    mgr.compile_kernel(cfg)
    assert mgr.get_kernel_stats("saxpy").cache_hit
    with pytest.raises(RuntimeError):
        mgr.compile_kernel(G.KernelConfig("bad", "this is not CUDA"))
    with pytest.raises(G.DeviceNotAvailable):
        mgr.execute_kernel(cfg, (1, 1, 1), [])


def test_dynamic_graph_and_runtime_engine():
    torch.manual_seed(0)
    b = E.GraphBuilder()
    x0 = torch.randn(4, 8)
    w, bias = torch.randn(16, 8), torch.randn(16)
    x = b.input(x0)
    h = b.relu(b.linear(x, w, bias))
    s = b.sigmoid(h)
    side = b.custom(lambda t: t * 100, h)              # not needed for `out`
    out = b.add(s, h)
    ctx = b.build()
    ref = torch.sigmoid(torch.relu(x0 @ w.t() + bias)) + torch.relu(x0 @ w.t() + bias)
    assert torch.allclose(ctx.execute(out), ref, atol=1e-6)
    assert ctx.nodes[side].value is None and ctx.executions == 4
    ctx.execute(out)
    assert ctx.cache_hits >= 1 and ctx.executions == 4
    ctx.set_input(x, x0 * 2)
    assert torch.allclose(ctx.execute(out), torch.sigmoid(torch.relu(2 * x0 @ w.t() + bias)) + torch.relu(2 * x0 @ w.t() + bias), atol=1e-5)
    assert side in ctx.dead_nodes([out]) and ctx.execution_plan() == list(range(len(ctx.nodes)))
    assert len(ctx.parallel_levels()) >= 4 and "arena_bytes" in ctx.memory_plan()
    eng = E.RuntimeEngine()
    f = lambda a: torch.relu(a) + 1
    for _ in range(3):
        y = eng.execute("f", f, x0)
    assert torch.equal(y, torch.relu(x0) + 1) and eng.metrics.executions == 3 and eng.metrics.cache_hit_rate == pytest.approx(2 / 3)
    assert eng.profile_report()["f"]["calls"] == 3
    with pytest.raises(ValueError):
        ctx.add_op(E.DynamicOp.CUSTOM, [x])


def test_bounds_checked_build_mode_compiles(tmp_path):
    """The checked build (-DRT_BOUNDS_CHECK) turns RT_GUARD into real index checks; it must keep compiling for sm_100a.
    One translation unit that uses the macro is enough to catch a broken guard expression."""
    import shutil
    import subprocess
    from pathlib import Path
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(nvcc).exists():
        import pytest
        pytest.skip("no nvcc")
    root = Path(__file__).resolve().parents[1]
    src = root / "csrc" / "conv" / "unfold_nd.cu"
    assert "RT_GUARD" in src.read_text()
    for flags in ([], ["-DRT_BOUNDS_CHECK"]):
        r = subprocess.run([nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-std=c++17", "--expt-relaxed-constexpr", *flags,
                            f"-I{root / 'csrc'}", "-c", str(src), "-o", str(tmp_path / "u.o")], capture_output=True, text=True)
        assert r.returncode == 0, r.stderr[-2000:]
