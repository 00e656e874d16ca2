"""CPU tests: profiler, debug, validation, tensorboard, special functions, distributions."""
import json
import math
import os

import numpy as np
import pytest
import torch

from rustorch_b200 import debug, distributions as D, profiler, special, tensorboard as tb, validation as V


# ------------------------------------------------------------------ profiler
def test_profiler_scopes_and_chrome_trace(tmp_path):
    p = profiler.Profiler()
    p.enable()
    with p.profile("outer"):
        with p.profile("inner", category="kernel", n=3):
            torch.randn(64, 64) @ torch.randn(64, 64)
    st = p.stats()
    assert st["outer"]["calls"] == 1 and st["inner"]["total_ms"] <= st["outer"]["total_ms"]
    path = tmp_path / "trace.json"
    p.export_chrome_trace(str(path))
    doc = json.loads(path.read_text())
    assert {e["name"] for e in doc["traceEvents"]} == {"outer", "inner"}
    assert all(e["ph"] == "X" and e["dur"] >= 0 for e in doc["traceEvents"])
    assert "outer;inner" in p.timeline.flame_graph()
    assert "inner" in p.report()


def test_profiler_disabled_is_noop_and_global_api():
    profiler.clear_profiler()
    profiler.disable_profiler()
    with profiler.profile("x"):
        pass
    assert not profiler.PROFILER.timeline.events
    profiler.enable_profiler()
    with profiler.profile("x"):
        pass
    profiler.disable_profiler()
    assert len(profiler.PROFILER.timeline.events) == 1


def test_metrics_prometheus_export():
    m = profiler.MetricsCollector("rt")
    m.inc("steps")
    m.inc("steps", 2)
    m.set_gauge("loss", 0.5)
    for v in (0.005, 0.05, 5.0):
        m.observe("latency", v)
    text = m.export_prometheus()
    assert "# TYPE rt_steps counter\nrt_steps 3.0" in text
    assert "rt_loss 0.5" in text
    assert 'rt_latency_bucket{le="0.01"} 1' in text and 'rt_latency_bucket{le="+Inf"} 3' in text
    assert "rt_latency_count 3" in text


def test_monitor_analyzer_benchmark():
    mon = profiler.RealTimeMonitor()
    mon.add_rule("loss", lambda v: v > 10, "loss exploded")
    assert mon.feed("loss", 1.0) == [] and mon.feed("loss", 11.0) == ["loss exploded"]
    assert profiler.PerformanceAnalyzer.trend([1, 2, 3, 4]) == pytest.approx(1.0)
    recs = profiler.PerformanceAnalyzer.recommendations({"a": {"total_ms": 90, "calls": 1, "mean_ms": 90}, "b": {"total_ms": 10, "calls": 1, "mean_ms": 10}})
    assert any("'a'" in r for r in recs)
    suite = profiler.AdvancedBenchmarkSuite(warmup=1, iters=3)
    r = suite.run("mm", lambda: torch.randn(32, 32) @ torch.randn(32, 32), items_per_iter=1.0)
    assert r.iters == 3 and r.min_ms <= r.median_ms <= r.max_ms and json.loads(suite.to_json())[0]["name"] == "mm"


# ------------------------------------------------------------------ debug
def test_debug_framework(tmp_path):
    f = debug.DebugFramework(level="info", file=str(tmp_path / "log.jsonl"), json_format=True)
    assert f.log("debug", "core", "hidden") is None
    f.log("info", "core", "step done", step=3)
    f.log("error", "cuda", "out of memory while allocating")
    lines = (tmp_path / "log.jsonl").read_text().strip().splitlines()
    assert len(lines) == 2 and json.loads(lines[0])["step"] == 3
    with f.profile("work"):
        sum(range(1000))
    h = f.track_allocation(200 << 20, "big")
    f.analyzer.add_pattern("oom", r"out of memory")
    rep = f.generate_debug_report()
    assert rep["log_counts"]["oom"] == 1 and rep["log_counts"]["errors"] == 1
    assert rep["memory"]["large"][0]["tag"] == "big" and rep["profile"]["work"]["calls"] == 1
    f.memory.track_deallocation(h)
    assert f.memory.current == 0 and f.memory.peak == 200 << 20


def test_log_analyzer_alert_cooldown():
    lg = debug.Logger("info")
    an = debug.LogAnalyzer()
    an.add_rule(debug.AlertRule("nan", r"NaN", threshold=2, window_s=60, cooldown_s=30))
    lg.info("t", "NaN in grad")
    assert an.check_alerts(lg.entries) == []
    lg.info("t", "NaN in loss")
    assert an.check_alerts(lg.entries) == ["nan"]
    assert an.check_alerts(lg.entries) == []          # cooling down
    s = debug.DebugUtils.tensor_summary(torch.tensor([1.0, float("nan")]))
    assert s["nan"] == 1 and "torch" in debug.DebugUtils.system_info()


# ------------------------------------------------------------------ validation
def test_validation_rules_and_quality():
    fw = V.DataValidationFramework()
    fw.engine.add_rule(V.range_rule(-5, 5)).add_rule(V.shape_rule([None, 4]))
    good = torch.randn(100, 4).clamp(-4, 4)
    res = fw.validate_tensor(good, valid_range=(-5, 5))
    assert res.passed and res.metrics["completeness"] == 1.0 and V.QualityMetrics.grade(res.metrics["score"]) in "AB"
    bad = good.clone()
    bad[0, 0] = float("nan")
    bad[1, 1] = 100.0
    r2 = fw.validate_tensor(bad)
    assert not r2.passed and {i.rule for i in r2.issues} >= {"no_nan", "finite"}
    for fmt in ("text", "json", "markdown", "html"):
        out = fw.validate_tensor(bad, fmt=fmt)
        assert "grade" in out.lower()


def test_anomaly_consistency_streaming():
    x = torch.cat([torch.randn(1000), torch.tensor([50.0])])
    det = V.AnomalyDetector()
    assert 1000 in det.zscore(x).tolist() and 1000 in det.iqr(x).tolist()
    cc = V.ConsistencyChecker()
    assert cc.check_shapes({"x": torch.zeros(4, 2), "y": torch.zeros(4)}) == []
    assert cc.check_shapes({"x": torch.zeros(4, 2), "y": torch.zeros(5)})
    assert cc.check_replicas(torch.ones(3), torch.ones(3)) == [] and cc.check_replicas(torch.ones(3), torch.zeros(3))
    rt = V.RealTimeValidator()
    for _ in range(20):
        assert rt.feed(torch.randn(256)).passed
    drift = rt.feed(torch.randn(256) + 5)
    assert any(i.rule == "drift" for i in drift.issues)
    assert not rt.feed(torch.tensor([float("inf")])).passed


# ------------------------------------------------------------------ tensorboard
def test_crc32c_known_vectors():
    assert tb.crc32c(b"123456789") == 0xE3069283
    assert tb.crc32c(b"") == 0


def test_summary_writer_roundtrip(tmp_path):
    with tb.SummaryWriter(str(tmp_path)) as w:
        w.add_scalar("loss", 0.25, 1)
        w.add_scalar("loss", 0.125, 2)
        w.add_histogram("w", torch.randn(1000), 2)
        w.add_image("img", torch.rand(3, 8, 8), 2)
        w.add_text("note", "hello", 2)
        w.add_pr_curve("pr", torch.tensor([1, 0, 1, 1]), torch.tensor([0.9, 0.2, 0.6, 0.4]), 2)
        w.add_audio("a", torch.sin(torch.linspace(0, 100, 800)), 8000, 2)
        w.add_graph(torch.nn.Sequential(torch.nn.Linear(2, 2), torch.nn.ReLU()))
        w.add_embedding(torch.randn(5, 3), ["a", "b", "c", "d", "e"], "emb", 2)
        path = w.writer.path
    evs = tb.read_events(path)
    assert evs[0]["file_version"] == "brain.Event:2"
    scal = [(e["step"], v["simple_value"]) for e in evs for v in e["values"] if v.get("kind") == "scalar"]
    assert scal == [(1, 0.25), (2, 0.125)]
    kinds = [v.get("kind") for e in evs for v in e["values"]]
    assert {"histogram", "image", "tensor", "audio"} <= set(kinds)
    assert any("graph" in e for e in evs)
    img = next(v["image"] for e in evs for v in e["values"] if v.get("kind") == "image")
    fields = {no: val for no, _, val in tb.parse_message(img)}
    assert fields[1] == 8 and fields[2] == 8 and fields[3] == 3 and fields[4][:8] == b"\x89PNG\r\n\x1a\n"
    assert os.path.exists(tmp_path / "projector_config.pbtxt")
    # a flipped byte is detected by the record checksum
    raw = bytearray(open(path, "rb").read())
    raw[30] ^= 0xFF
    bad = tmp_path / "bad.tfevents"
    bad.write_bytes(bytes(raw))
    with pytest.raises(ValueError):
        tb.read_events(str(bad))


# ------------------------------------------------------------------ special
def test_special_against_scipy():
    sp = pytest.importorskip("scipy.special")
    x = torch.tensor([0.3, 1.5, 4.2, 9.7, 25.0], dtype=torch.float64)
    for n in (0, 1, 2, 5, 12):
        np.testing.assert_allclose(special.bessel_j(n, x).numpy(), sp.jv(n, x.numpy()), rtol=1e-7, atol=1e-10)
        np.testing.assert_allclose(special.bessel_y(n, x).numpy(), sp.yv(n, x.numpy()), rtol=1e-7)
        np.testing.assert_allclose(special.bessel_i(n, x).numpy(), sp.iv(n, x.numpy()), rtol=1e-7)
        np.testing.assert_allclose(special.bessel_k(n, x).numpy(), sp.kv(n, x.numpy()), rtol=1e-7)
    np.testing.assert_allclose(special.bessel_j(3, -x).numpy(), sp.jv(3, -x.numpy()), rtol=1e-7, atol=1e-10)
    g = torch.tensor([-2.5, -0.5, 0.5, 3.0, 7.5], dtype=torch.float64)
    np.testing.assert_allclose(special.gamma(g).numpy(), sp.gamma(g.numpy()), rtol=1e-10)
    np.testing.assert_allclose(special.digamma(g.abs()).numpy(), sp.digamma(g.abs().numpy()), rtol=1e-10)
    np.testing.assert_allclose(special.beta(2.5, 1.5).item(), sp.beta(2.5, 1.5), rtol=1e-10)
    e = torch.tensor([-0.9, -0.1, 0.0, 0.5, 0.99], dtype=torch.float64)
    np.testing.assert_allclose(special.erfinv(e).numpy(), sp.erfinv(e.numpy()), rtol=1e-9, atol=1e-12)
    np.testing.assert_allclose(special.erfcinv(1 - e).numpy(), sp.erfcinv(1 - e.numpy()), rtol=1e-9, atol=1e-12)
    np.testing.assert_allclose(special.erfcx(x).numpy(), sp.erfcx(x.numpy()), rtol=1e-10)
    with pytest.raises(ValueError):
        special.erfinv(torch.tensor(1.5))


def test_special_scalar_helpers():
    assert special.factorial(5) == 120 and special.double_factorial(7) == 105 and special.binomial_coefficient(10, 3) == 120
    assert special.pochhammer(2.0, 3) == 24 and special.harmonic_number(4) == pytest.approx(25 / 12)
    assert special.bernoulli_number(2) == pytest.approx(1 / 6) and special.bernoulli_number(4) == pytest.approx(-1 / 30)
    assert special.bernoulli_number(3) == 0 and special.bernoulli_number(1) == -0.5
    assert special.is_integer(3.0000000000001) and special.signum(-2.0) == -1


# ------------------------------------------------------------------ distributions
@pytest.mark.parametrize("ours,theirs", [
    (lambda: D.Normal(torch.tensor([0.5, -1.0]), torch.tensor([1.5, 0.3])), lambda: torch.distributions.Normal(torch.tensor([0.5, -1.0]), torch.tensor([1.5, 0.3]))),
    (lambda: D.Uniform(torch.tensor([0.0, -1.0]), torch.tensor([2.0, 3.0])), lambda: torch.distributions.Uniform(torch.tensor([0.0, -1.0]), torch.tensor([2.0, 3.0]))),
    (lambda: D.Exponential(torch.tensor([0.5, 2.0])), lambda: torch.distributions.Exponential(torch.tensor([0.5, 2.0]))),
    (lambda: D.Gamma(torch.tensor([2.0, 0.7]), torch.tensor([1.5, 3.0])), lambda: torch.distributions.Gamma(torch.tensor([2.0, 0.7]), torch.tensor([1.5, 3.0]))),
    (lambda: D.Beta(torch.tensor([2.0, 0.7]), torch.tensor([1.5, 3.0])), lambda: torch.distributions.Beta(torch.tensor([2.0, 0.7]), torch.tensor([1.5, 3.0]))),
])
def test_continuous_distributions_match_torch(ours, theirs):
    a, b = ours(), theirs()
    v = torch.tensor([0.4, 0.6])
    torch.testing.assert_close(a.log_prob(v), b.log_prob(v))
    torch.testing.assert_close(a.entropy(), b.entropy())
    torch.testing.assert_close(a.mean, b.mean)
    torch.testing.assert_close(a.variance, b.variance)
    s = a.sample((20000,))
    assert s.shape == (20000, 2)
    torch.testing.assert_close(s.mean(0), b.mean, rtol=0.1, atol=0.05)
    try:
        torch.testing.assert_close(a.cdf(v), b.cdf(v), rtol=1e-4, atol=1e-5)
    except NotImplementedError:
        pass


def test_beta_gamma_cdf_against_scipy():
    st = pytest.importorskip("scipy.stats")
    x = torch.tensor([0.05, 0.3, 0.5, 0.9])
    np.testing.assert_allclose(D.Beta(2.5, 0.8).cdf(x).numpy(), st.beta(2.5, 0.8).cdf(x.numpy()), rtol=1e-5)
    np.testing.assert_allclose(D.Gamma(2.5, 2.0).cdf(x).numpy(), st.gamma(2.5, scale=0.5).cdf(x.numpy()), rtol=1e-5)
    n = D.Normal.standard()
    torch.testing.assert_close(n.icdf(n.cdf(torch.tensor([-1.2, 0.3]))), torch.tensor([-1.2, 0.3]), rtol=1e-4, atol=1e-5)


def test_discrete_distributions_and_validation():
    b = D.Bernoulli(probs=torch.tensor([0.2, 0.9]))
    tb_ = torch.distributions.Bernoulli(probs=torch.tensor([0.2, 0.9]))
    v = torch.tensor([1.0, 0.0])
    torch.testing.assert_close(b.log_prob(v), tb_.log_prob(v))
    torch.testing.assert_close(b.entropy(), tb_.entropy())
    assert b.sample((1000,)).mean(0)[1] > 0.8
    c = D.Categorical(probs=torch.tensor([[1.0, 1.0, 2.0], [0.0, 3.0, 1.0]]))
    tc = torch.distributions.Categorical(probs=torch.tensor([[1.0, 1.0, 2.0], [0.0, 3.0, 1.0]]))
    torch.testing.assert_close(c.entropy(), tc.entropy())
    s = c.sample((5000,))
    assert s.shape == (5000, 2) and (s[:, 1] != 0).all()
    torch.testing.assert_close(c.log_prob(torch.tensor([2, 1])), tc.log_prob(torch.tensor([2, 1])))
    with pytest.raises(ValueError):
        D.Normal(0.0, -1.0)
    assert D.Normal(0.0, -1.0, validate_args=False) is not None
    assert "gamma" in D.available_distributions() and D.get_distribution("Beta") is D.Beta
    loc = torch.tensor(0.0, requires_grad=True)
    D.Normal(loc, 1.0).rsample((8,)).sum().backward()
    assert loc.grad.item() == 8


def test_profiler_scopes_are_nvtx_ranges():
    """Every profiled scope pushes / pops one NVTX range (balanced, also when the body raises); ``nvtx_range`` is the
    stand-alone form."""
    from rustorch_b200 import profiler as P
    prof = P.Profiler(P.ProfilerConfig(enable_gpu=False))
    prof.enable()
    before = P.nvtx.pushed
    with prof.profile("outer"):
        assert P.nvtx.depth == 1
        with prof.profile("inner", category="kernel"):
            assert P.nvtx.depth == 2
    assert P.nvtx.depth == 0 and P.nvtx.pushed == before + 2
    with pytest.raises(ValueError):
        with P.nvtx_range("boom"):
            raise ValueError("x")
    assert P.nvtx.depth == 0
    quiet = P.Profiler(P.ProfilerConfig(enable_gpu=False, enable_nvtx=False))
    quiet.enable()
    n = P.nvtx.pushed
    with quiet.profile("silent"):
        pass
    assert P.nvtx.pushed == n
