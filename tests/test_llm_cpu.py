"""LLM runtime on CPU: quantised linear, sampling, metrics, GGUF -> runtime -> generation."""
import pytest
import torch

from rustorch_b200.formats import gguf
from rustorch_b200 import llm


def test_quant_linear_cpu_matches_dequantised_matmul():
    w = torch.randn(24, 64) * 0.05
    for ty in (gguf.GGMLType.Q4_0, gguf.GGMLType.Q8_0):
        q = llm.QuantLinear.from_float(w, ty)
        x = torch.randn(3, 64)
        assert torch.allclose(q(x), x @ q.dequantize().t(), atol=1e-5)
        tol = float(w.abs().max()) / 8 * 1.05 if ty is gguf.GGMLType.Q4_0 else float(w.abs().max()) / 127 * 0.6
        assert float((q.dequantize() - w).abs().max()) < tol
        r0, r1 = q.shard_rows(0, 2), q.shard_rows(1, 2)
        assert torch.allclose(torch.cat([r0(x), r1(x)], -1), q(x), atol=1e-5)
        c0, c1 = q.shard_cols(0, 2), q.shard_cols(1, 2)
        assert torch.allclose(c0(x[:, :32]) + c1(x[:, 32:]), q(x), atol=1e-5)


def test_sampling():
    logits = torch.tensor([[1.0, 3.0, 2.0, -1.0]])
    assert llm.sample_token(logits[0], llm.SamplingConfig.greedy()) == 1
    p = llm.softmax(logits)
    pk = llm.apply_top_k_to_probs(p, 2)
    assert float(pk[0, 0]) == 0.0 and abs(float(pk.sum()) - 1) < 1e-6
    pp = llm.apply_top_p_to_probs(p, 0.5)
    assert int((pp > 0).sum()) == 1 and int(pp.argmax()) == 1
    pen = llm.apply_repetition_penalty(logits, torch.tensor([[1]]), 2.0)
    assert float(pen[0, 1]) == 1.5
    s = llm.Sampler(llm.SamplingConfig(temperature=0.7, top_k=3, top_p=0.9, seed=0))
    toks = [int(s(logits)[0]) for _ in range(20)]
    assert set(toks) <= {0, 1, 2} and s.history.shape == (1, 20)
    with pytest.raises(ValueError):
        llm.SamplingConfig(top_p=0.0).validate()


def test_metrics_and_targets():
    t = llm.InferenceTimer()
    t.start()
    for _ in range(3):
        t.token()
    assert t.ttft_ms() >= 0 and t.tokens_per_s() > 0
    c = llm.MetricsCollector()
    c.record(llm.InferenceMetrics(ttft_ms=50, tokens_per_s=100, total_tokens=10, memory_bytes=5, model_bytes=4))
    assert c.meets_targets() == {"ttft": True, "throughput": True, "memory": True}
    rep = llm.MetricsReporter(c)
    assert "tok/s" in rep.text() and "| TTFT" in rep.markdown() and "summary" in rep.json()


def _tiny_gguf(path):
    cfg = llm.LlamaConfig(vocab_size=64, n_layer=2, n_embd=64, n_head=4, n_head_kv=2, n_ff=128, context_length=64)
    g = torch.Generator().manual_seed(0)
    rnd = lambda *s: torch.randn(*s, generator=g) * 0.05  # noqa: E731
    hd = cfg.head_dim
    tensors = {"token_embd.weight": (rnd(64, 64), gguf.GGMLType.F16), "output_norm.weight": (torch.ones(64), gguf.GGMLType.F32),
               "output.weight": (rnd(64, 64), gguf.GGMLType.Q8_0)}
    for i in range(cfg.n_layer):
        p = f"blk.{i}."
        tensors.update({p + "attn_q.weight": (rnd(4 * hd, 64), gguf.GGMLType.Q4_0), p + "attn_k.weight": (rnd(2 * hd, 64), gguf.GGMLType.Q4_0),
                        p + "attn_v.weight": (rnd(2 * hd, 64), gguf.GGMLType.Q4_0), p + "attn_output.weight": (rnd(64, 64), gguf.GGMLType.Q4_0),
                        p + "ffn_gate.weight": (rnd(128, 64), gguf.GGMLType.Q4_0), p + "ffn_up.weight": (rnd(128, 64), gguf.GGMLType.Q4_0),
                        p + "ffn_down.weight": (rnd(64, 128), gguf.GGMLType.Q4_0), p + "attn_norm.weight": (torch.ones(64), gguf.GGMLType.F32),
                        p + "ffn_norm.weight": (torch.ones(64), gguf.GGMLType.F32)})
    md = {"general.architecture": "llama", "llama.block_count": 2, "llama.embedding_length": 64, "llama.feed_forward_length": 128,
          "llama.attention.head_count": 4, "llama.attention.head_count_kv": 2, "llama.rope.freq_base": 10000.0,
          "llama.attention.layer_norm_rms_epsilon": 1e-5, "llama.context_length": 64, "llama.vocab_size": 64}
    gguf.write_gguf(path, md, tensors)
    return cfg


def test_gguf_runtime_cache_equals_full_recompute(tmp_path):
    p = str(tmp_path / "tiny.gguf")
    _tiny_gguf(p)
    rt = llm.LlamaRuntime.from_gguf(p, device="cpu")
    assert rt.cfg.n_head_kv == 2 and len(rt.layers) == 2
    prompt = torch.randint(0, 64, (2, 5), generator=torch.Generator().manual_seed(1))
    out, stats = rt.generate(prompt, 4)
    assert out.shape == (2, 9) and stats["decode_steps"] == 3
    # decoding with the cache must equal running the whole prefix again (what the reference does every step)
    cache = rt.new_cache(2, 16)
    logits_full = rt.prefill(out[:, :8], cache)
    assert torch.equal(logits_full.argmax(-1), out[:, 8])
    # tensor-parallel shards sum to the unsharded result
    r0 = llm.LlamaRuntime.from_gguf(p, device="cpu", tp_rank=0, tp_world=2)
    assert r0.h_local == 2 and r0.hkv_local == 1 and r0.layers[0].wo.in_features == 32


def test_quant_linear_fused_projection_fallback_on_cpu():
    """``QuantLinear.fused`` (RMSNorm prologue, residual or SwiGLU epilogue) away from the one-kernel CUDA path is the
    same arithmetic through separate ops: checked against plain fp32 math on the dequantised weights."""
    from rustorch_b200.formats import gguf
    from rustorch_b200.llm import QuantLinear
    torch.manual_seed(0)
    q = QuantLinear.random(64, 128, gguf.GGMLType.Q4_0, 0.05, "cpu", seed=4)
    W = q.dequantize()
    x = torch.randn(3, 128)
    nw = 1.0 + 0.1 * torch.randn(128)
    res = torch.randn(3, 64)
    h = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-5) * nw
    y = q.fused(x, norm_w=nw, eps=1e-5, residual=res)
    assert torch.allclose(y, h @ W.t() + res, atol=1e-4, rtol=1e-4)
    act = q.fused(x, norm_w=nw, eps=1e-5, swiglu=True)
    t = h @ W.t()
    assert act.shape == (3, 32)
    assert torch.allclose(act, torch.nn.functional.silu(t[:, :32]) * t[:, 32:], atol=1e-4, rtol=1e-4)
    assert torch.allclose(q.fused(x), x @ W.t(), atol=1e-4, rtol=1e-4)


def test_from_gguf_names_what_it_cannot_run(tmp_path):
    """Files of other decoder families fail with a message that says which tensors are the problem, not with a KeyError
    or, worse, by ignoring biases."""
    p = str(tmp_path / "t.gguf")
    _tiny_gguf(p)
    with gguf.GGUFFile(p) as g:
        md = dict(g.metadata)
        tensors = {n: (g.load_tensor(n), gguf.GGMLType.F32) for n in g.tensors}
    biased = dict(tensors)
    biased["blk.0.attn_q.bias"] = (torch.zeros(64), gguf.GGMLType.F32)
    pb = str(tmp_path / "biased.gguf")
    gguf.write_gguf(pb, md, biased)
    with pytest.raises(ValueError, match="attn_q.bias"):
        llm.LlamaRuntime.from_gguf(pb, device="cpu")
    lacking = {k: v for k, v in tensors.items() if "ffn_gate" not in k}
    pl = str(tmp_path / "lacking.gguf")
    gguf.write_gguf(pl, md, lacking)
    with pytest.raises(ValueError, match="missing"):
        llm.LlamaRuntime.from_gguf(pl, device="cpu")
