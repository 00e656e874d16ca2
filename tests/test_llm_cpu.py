"""LLM runtime on CPU: quantised linear, sampling, metrics, GGUF -> runtime -> generation."""
import os

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


def test_from_hf_matches_transformers_llama(tmp_path):
    """A Hugging Face Llama checkpoint directory runs on the quantised runtime and agrees with ``transformers``' own
    forward pass (grouped-query attention, rotate-half RoPE, RMSNorm epsilon, untied head) up to Q8_0 rounding."""
    tf = pytest.importorskip("transformers")
    torch.manual_seed(0)
    hc = tf.LlamaConfig(vocab_size=96, hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                        num_key_value_heads=2, max_position_embeddings=64, rms_norm_eps=1e-5, rope_theta=50000.0, tie_word_embeddings=False)
    ref = tf.LlamaForCausalLM(hc).eval()
    d = str(tmp_path / "hf")
    ref.save_pretrained(d, safe_serialization=True)
    rt = llm.LlamaRuntime.from_hf(d, device="cpu")
    assert not rt.cfg.rope_interleaved and rt.cfg.n_head_kv == 2 and len(rt.layers) == 2
    assert rt.cfg.rope_theta == 50000.0              # whichever layout this transformers version writes the base in
    prompt = torch.randint(0, 96, (2, 9), generator=torch.Generator().manual_seed(1))
    with torch.no_grad():
        want = ref(prompt).logits[:, -1]
    cache = rt.new_cache(2, 16)
    got = rt.prefill(prompt, cache)
    assert float((want - got).abs().max()) < 0.03 * float(want.abs().max()) and torch.equal(want.argmax(-1), got.argmax(-1))
    nxt = want.argmax(-1)
    with torch.no_grad():
        want2 = ref(torch.cat([prompt, nxt[:, None]], 1)).logits[:, -1]
    assert float((want2 - rt.decode_step(nxt, cache)).abs().max()) < 0.03 * float(want2.abs().max())
    # 4-bit on load, tied head, and the sharded layout (index file naming two shards)
    from rustorch_b200.formats.safetensors import HuggingFaceCheckpoint, load_safetensors, save_safetensors
    import json
    q4 = llm.LlamaRuntime.from_hf(d, device="cpu", ggml_type=gguf.GGMLType.Q4_0)
    assert q4.layers[0].wqkv.ggml_type is gguf.GGMLType.Q4_0 and torch.isfinite(q4.prefill(prompt, q4.new_cache(2, 16))).all()
    sd = load_safetensors(os.path.join(d, "model.safetensors"))
    sd.pop("lm_head.weight")
    names = sorted(sd)
    sh = str(tmp_path / "sharded")
    os.makedirs(sh)
    save_safetensors({k: sd[k] for k in names[::2]}, os.path.join(sh, "model-00001-of-00002.safetensors"))
    save_safetensors({k: sd[k] for k in names[1::2]}, os.path.join(sh, "model-00002-of-00002.safetensors"))
    json.dump({"weight_map": {k: f"model-0000{1 + i % 2}-of-00002.safetensors" for i, k in enumerate(names)}}, open(os.path.join(sh, "model.safetensors.index.json"), "w"))
    json.dump({**json.load(open(os.path.join(d, "config.json"))), "tie_word_embeddings": True}, open(os.path.join(sh, "config.json"), "w"))
    with HuggingFaceCheckpoint(sh) as ck:
        assert len(ck.keys()) == len(names) and ck.shape("model.embed_tokens.weight") == (96, 64)
    tied = llm.LlamaRuntime.from_hf(sh, device="cpu")
    assert tied.lm_head.out_features == 96 and torch.isfinite(tied.prefill(prompt, tied.new_cache(2, 16))).all()
    # other families are refused by name
    cfg = json.load(open(os.path.join(d, "config.json")))
    bad = str(tmp_path / "bad")
    os.makedirs(bad)
    json.dump(cfg, open(os.path.join(bad, "config.json"), "w"))
    full = load_safetensors(os.path.join(d, "model.safetensors"))
    full["model.layers.0.self_attn.q_proj.bias"] = torch.zeros(64)
    save_safetensors(full, os.path.join(bad, "model.safetensors"))
    with pytest.raises(ValueError, match="q_proj.bias"):
        llm.LlamaRuntime.from_hf(bad, device="cpu")
    json.dump({**cfg, "rope_scaling": {"type": "yarn", "factor": 2.0}, "rope_parameters": None}, open(os.path.join(d, "config.json"), "w"))
    with pytest.raises(ValueError, match="yarn"):
        llm.LlamaRuntime.from_hf(d, device="cpu")
    json.dump({**cfg, "rope_parameters": {"rope_type": "longrope", "factor": 8.0, "rope_theta": 1e4}}, open(os.path.join(d, "config.json"), "w"))
    with pytest.raises(ValueError, match="longrope"):
        llm.LlamaRuntime.from_hf(d, device="cpu")


def test_runtime_applies_rope_scaling_from_hf_and_gguf(tmp_path):
    """Long-context checkpoints (llama3 and linear frequency scaling): the serving runtime on the Hugging Face directory
    and on the GGUF file converted from it rotates with ``transformers``' frequencies and agrees on the logits."""
    tf = pytest.importorskip("transformers")
    prompt = torch.randint(0, 96, (1, 90), generator=torch.Generator().manual_seed(2))
    for rs in ({"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0, "original_max_position_embeddings": 32},
               {"rope_type": "linear", "factor": 4.0}):
        torch.manual_seed(0)
        hc = tf.LlamaConfig(vocab_size=96, hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                            num_key_value_heads=2, max_position_embeddings=128, rope_theta=50000.0, rope_scaling=rs, tie_word_embeddings=False)
        ref = tf.LlamaForCausalLM(hc).eval()
        d = str(tmp_path / f"hf_{rs['rope_type']}")
        ref.save_pretrained(d, safe_serialization=True)
        out = str(tmp_path / f"{rs['rope_type']}.gguf")
        info = llm.hf_to_gguf(d, out, gguf.GGMLType.Q8_0)
        assert info["tensors"] == 3 + 9 * 2 + (rs["rope_type"] == "llama3")
        with torch.no_grad():
            want = ref(prompt).logits[:, -1]
            nxt = want.argmax(-1)
            want2 = ref(torch.cat([prompt, nxt[:, None]], 1)).logits[:, -1]
        for rt in (llm.LlamaRuntime.from_hf(d, device="cpu"), llm.LlamaRuntime.from_gguf(out, device="cpu")):
            assert rt.cfg.rope_scaling["rope_type"] in (rs["rope_type"], "factors")
            cache = rt.new_cache(1, 96)
            got = rt.prefill(prompt, cache)
            err = float((want - got).abs().max()) / float(want.abs().max())
            assert err < 0.03 and float((want2 - rt.decode_step(nxt, cache)).abs().max()) < 0.03 * float(want2.abs().max())
            # at random initialisation attention is near uniform and Q8_0 rounding is as large as the effect of the
            # scaling on the logits, so the frequencies themselves are compared with the library's
            assert torch.allclose(rt._inv_freq(16, "cpu"), ref.model.rotary_emb.inv_freq.float(), rtol=1e-5, atol=0)
            assert not torch.allclose(rt._inv_freq(16, "cpu"), 50000.0 ** (-torch.arange(8.0) / 8), rtol=1e-2)


def test_hf_rope_settings_reads_both_config_layouts():
    from rustorch_b200.formats.safetensors import hf_rope_settings
    assert hf_rope_settings({}) == (10000.0, None)
    assert hf_rope_settings({"rope_theta": 5e5, "rope_scaling": None}) == (5e5, None)
    assert hf_rope_settings({"rope_theta": 5e5, "rope_scaling": {"type": "linear", "factor": 2.0}}) == (5e5, {"type": "linear", "factor": 2.0})
    assert hf_rope_settings({"rope_parameters": {"rope_theta": 1e6, "rope_type": "default"}}) == (1e6, None)
    th, sc = hf_rope_settings({"rope_theta": 1.0, "rope_parameters": {"rope_theta": 5e5, "rope_type": "llama3", "factor": 8.0}})
    assert th == 5e5 and sc == {"rope_type": "llama3", "factor": 8.0}


def test_hf_to_gguf_keeps_the_logits(tmp_path):
    """The converter's row permutation of q / k turns rotate-half checkpoints into interleaved-RoPE GGUF files: the
    runtime on the written file agrees with ``transformers`` on the original checkpoint."""
    tf = pytest.importorskip("transformers")
    torch.manual_seed(0)
    hc = tf.LlamaConfig(vocab_size=96, hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                        num_key_value_heads=2, max_position_embeddings=64, rms_norm_eps=1e-5, rope_theta=50000.0, tie_word_embeddings=False)
    ref = tf.LlamaForCausalLM(hc).eval()
    d = str(tmp_path / "hf")
    ref.save_pretrained(d, safe_serialization=True)
    prompt = torch.randint(0, 96, (2, 9), generator=torch.Generator().manual_seed(1))
    with torch.no_grad():
        want = ref(prompt).logits[:, -1]
    for ty, tol in ((gguf.GGMLType.F32, 0.03), (gguf.GGMLType.Q8_0, 0.03), (gguf.GGMLType.Q4_0, 0.4)):      # the runtime holds F32 matrices as Q8_0
        out = str(tmp_path / f"{ty.name}.gguf")
        info = llm.hf_to_gguf(d, out, ty)
        assert info["tensors"] == 3 + 9 * 2 and info["bytes"] == os.path.getsize(out)
        rt = llm.LlamaRuntime.from_gguf(out, device="cpu")
        assert rt.cfg.rope_interleaved and rt.cfg.rope_theta == 50000.0
        got = rt.prefill(prompt, rt.new_cache(2, 16))
        assert float((want - got).abs().max()) < tol * float(want.abs().max()), ty
    w = torch.arange(16.0).view(8, 2)                                # two heads of four rows: halves (0, 1 | 2, 3) -> pairs (0, 2, 1, 3)
    assert llm.interleave_rope_rows(w, 2)[:, 0].tolist() == [0.0, 4.0, 2.0, 6.0, 8.0, 12.0, 10.0, 14.0]


def test_hf_to_gguf_embeds_the_sentencepiece_tokenizer(tmp_path):
    """With a ``tokenizer.model`` beside the weights the written GGUF file carries the vocabulary, and the CLI's GGUF
    tokenizer then splits text like SentencePiece does."""
    tf = pytest.importorskip("transformers")
    spm = pytest.importorskip("sentencepiece")
    from rustorch_b200.cli.tokenizer import GGUFTokenizer
    d = str(tmp_path / "hf")
    os.makedirs(d)
    corpus = str(tmp_path / "corpus.txt")
    words = "the quick brown fox jumps over the lazy dog and runs far away from here with great speed every single day".split()
    g = torch.Generator().manual_seed(0)
    with open(corpus, "w") as f:
        for _ in range(400):
            f.write(" ".join(words[int(i)] for i in torch.randint(0, len(words), (8,), generator=g)) + "\n")
    spm.SentencePieceTrainer.train(input=corpus, model_prefix=os.path.join(d, "tokenizer"), vocab_size=340, model_type="bpe", byte_fallback=True,
                                   character_coverage=1.0, bos_id=1, eos_id=2, unk_id=0, minloglevel=2)
    sp = spm.SentencePieceProcessor(model_file=os.path.join(d, "tokenizer.model"))
    n = sp.get_piece_size()
    torch.manual_seed(0)
    hc = tf.LlamaConfig(vocab_size=n, hidden_size=64, intermediate_size=128, num_hidden_layers=1, num_attention_heads=4, num_key_value_heads=2,
                        max_position_embeddings=64)
    tf.LlamaForCausalLM(hc).save_pretrained(d, safe_serialization=True)
    out = str(tmp_path / "m.gguf")
    info = llm.hf_to_gguf(d, out, gguf.GGMLType.Q8_0)
    assert info["tokenizer"]
    with gguf.GGUFFile(out) as f:
        assert len(f.metadata["tokenizer.ggml.tokens"]) == n and f.metadata["tokenizer.ggml.bos_token_id"] == 1
        tok = GGUFTokenizer.from_gguf(f)
    for text in ("the quick brown fox", "lazy dog runs far away", "zebra!"):
        ids = tok.encode(text, add_bos=False)
        assert ids == sp.encode(text) and tok.decode(ids).strip() == text


def test_hf_to_gguf_embeds_a_byte_level_bpe_tokenizer(tmp_path):
    """A directory whose only tokenizer file is ``tokenizer.json`` (Llama 3, Qwen2): the GGUF file carries it as a ``gpt2``
    tokenizer, and the CLI's loader, given the file alone, tokenizes like the ``tokenizers`` library and generates."""
    tf = pytest.importorskip("transformers")
    tk = pytest.importorskip("tokenizers")
    from tokenizers import Regex, decoders, models, pre_tokenizers, processors, trainers
    from rustorch_b200.cli.engine import InferenceEngine, ModelLoader
    from rustorch_b200.cli.session import GenerationConfig
    d = str(tmp_path / "hf")
    os.makedirs(d)
    tok = tk.Tokenizer(models.BPE(ignore_merges=True))
    pat = r"(?i:'s|'t|'re|'ve|'m|'ll|'d)|[^\r\n\p{L}\p{N}]?\p{L}+|\p{N}{1,3}| ?[^\s\p{L}\p{N}]+[\r\n]*|\s*[\r\n]+|\s+(?!\S)|\s+"
    tok.pre_tokenizer = pre_tokenizers.Sequence([pre_tokenizers.Split(Regex(pat), behavior="isolated"),
                                                 pre_tokenizers.ByteLevel(add_prefix_space=False, use_regex=False)])
    tok.decoder = decoders.ByteLevel()
    tok.train_from_iterator(["the quick brown fox jumps over the lazy dog 1234 times, doesn't it?\n"] * 50, trainers.BpeTrainer(
        vocab_size=330, special_tokens=["<|begin_of_text|>", "<|eot_id|>"], initial_alphabet=pre_tokenizers.ByteLevel.alphabet()))
    tok.post_processor = processors.TemplateProcessing(single="<|begin_of_text|> $A", special_tokens=[("<|begin_of_text|>", 0)])
    tok.save(os.path.join(d, "tokenizer.json"))
    import json
    json.dump({"eos_token": "<|eot_id|>"}, open(os.path.join(d, "tokenizer_config.json"), "w"))
    n = tok.get_vocab_size()
    torch.manual_seed(0)
    tf.LlamaForCausalLM(tf.LlamaConfig(vocab_size=n, hidden_size=64, intermediate_size=128, num_hidden_layers=1, num_attention_heads=4,
                                       num_key_value_heads=2, max_position_embeddings=64)).save_pretrained(d, safe_serialization=True)
    out = str(tmp_path / "m.gguf")
    info = llm.hf_to_gguf(d, out, gguf.GGMLType.Q8_0)
    assert info["tokenizer"] and info["tokenizer_model"] == "gpt2"
    rt, carried, meta = ModelLoader.from_file(out, "cpu")
    assert carried.vocab_size == n == meta.vocab_size and carried.bos_id == 0 and carried.eos_id == 1
    for text in ("the quick brown fox", "doesn't it? 123456", "<|eot_id|>lazy dog\n"):
        assert carried.encode(text) == tok.encode(text).ids
    eng = InferenceEngine(rt, carried, GenerationConfig(max_tokens=5, temperature=0.0), "cpu", seed=0)
    assert isinstance(eng.generate("the quick"), str) and eng.last_token_count <= 5
    # the directory itself is served with the same tokenizer
    rt2, tok2, _ = ModelLoader.from_file(d, "cpu")
    assert tok2.encode("the quick brown fox") == tok.encode("the quick brown fox").ids


def test_qwen2_style_checkpoints_with_qkv_biases(tmp_path):
    """q / k / v biases and the half-split rotation of the Qwen2 family: the runtime on the Hugging Face directory and on
    the GGUF file written from it agrees with ``transformers``' Qwen2."""
    tf = pytest.importorskip("transformers")
    torch.manual_seed(0)
    hc = tf.Qwen2Config(vocab_size=96, hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                        max_position_embeddings=64, rms_norm_eps=1e-6, rope_theta=1000000.0, tie_word_embeddings=True, use_sliding_window=False)
    ref = tf.Qwen2ForCausalLM(hc).eval()
    with torch.no_grad():
        for n, p in ref.named_parameters():
            if n.endswith("bias"):
                p.normal_(0, 0.2)
    d = str(tmp_path / "qwen")
    ref.save_pretrained(d, safe_serialization=True)
    prompt = torch.randint(0, 96, (2, 9), generator=torch.Generator().manual_seed(1))
    with torch.no_grad():
        want = ref(prompt).logits[:, -1]
        nxt = want.argmax(-1)
        want2 = ref(torch.cat([prompt, nxt[:, None]], 1)).logits[:, -1]
    out = str(tmp_path / "qwen.gguf")
    assert llm.hf_to_gguf(d, out, gguf.GGMLType.Q8_0)["tensors"] == 2 + 12 * 2          # tied head: no output.weight
    for rt in (llm.LlamaRuntime.from_hf(d, device="cpu"), llm.LlamaRuntime.from_gguf(out, device="cpu")):
        assert not rt.cfg.rope_interleaved and rt.layers[0].qkv_bias.shape == (4 * 16 + 2 * 2 * 16,) and rt.cfg.rope_theta == 1e6
        cache = rt.new_cache(2, 16)
        got = rt.prefill(prompt, cache)
        assert float((want - got).abs().max()) < 0.03 * float(want.abs().max())
        assert float((want2 - rt.decode_step(nxt, cache)).abs().max()) < 0.03 * float(want2.abs().max())
    half = llm.LlamaRuntime.from_hf(d, device="cpu", tp_rank=1, tp_world=2)               # bias rows are sharded with the weight rows
    assert half.layers[0].qkv_bias.shape == (2 * 16 + 2 * 16,)
    full = llm.LlamaRuntime.from_hf(d, device="cpu").layers[0].qkv_bias
    assert torch.equal(half.layers[0].qkv_bias, torch.cat([full[32:64], full[64 + 16:64 + 32], full[96 + 16:128]]))


def test_from_gguf_rope_frequency_scaling_kinds(tmp_path):
    p = str(tmp_path / "t.gguf")
    _tiny_gguf(p)
    with gguf.GGUFFile(p) as g:
        md = dict(g.metadata)
        tensors = {n: (g.load_tensor(n), gguf.GGMLType.F32) for n in g.tensors}
    tensors["rope_freqs.weight"] = (torch.ones(5), gguf.GGMLType.F32)
    gguf.write_gguf(p, md, tensors)
    with pytest.raises(ValueError, match="rope_freqs.weight has 5 entries"):
        llm.LlamaRuntime.from_gguf(p, device="cpu")
    del tensors["rope_freqs.weight"]
    gguf.write_gguf(p, {**md, "llama.rope.scaling.type": "yarn"}, tensors)
    with pytest.raises(ValueError, match="yarn"):
        llm.LlamaRuntime.from_gguf(p, device="cpu")
    gguf.write_gguf(p, {**md, "llama.rope.scaling.type": "linear", "llama.rope.scaling.factor": 2.0}, tensors)
    assert llm.LlamaRuntime.from_gguf(p, device="cpu").cfg.rope_scaling == {"rope_type": "linear", "factor": 2.0}


def test_sliding_window_checkpoints_limit_the_context(tmp_path):
    """A Mistral-style config switches a sliding attention window on by naming its width: the runtime (which attends over
    its whole cache) takes the window as its context length, from the directory and from the converted GGUF file, and
    agrees with ``transformers`` inside it.  Qwen2-style configs carry a width that is off unless ``use_sliding_window``."""
    tf = pytest.importorskip("transformers")
    from rustorch_b200.formats.safetensors import hf_attention_window
    assert hf_attention_window({"model_type": "mistral", "sliding_window": 4096}) == 4096
    assert hf_attention_window({"model_type": "mistral", "sliding_window": None}) is None
    assert hf_attention_window({"model_type": "qwen2", "sliding_window": 4096}) is None
    assert hf_attention_window({"model_type": "qwen2", "sliding_window": 4096, "use_sliding_window": True}) == 4096
    torch.manual_seed(0)
    hc = tf.MistralConfig(vocab_size=96, hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                          max_position_embeddings=128, sliding_window=24, tie_word_embeddings=False)
    ref = tf.MistralForCausalLM(hc).eval()
    d = str(tmp_path / "mistral")
    ref.save_pretrained(d, safe_serialization=True)
    out = str(tmp_path / "mistral.gguf")
    llm.hf_to_gguf(d, out, gguf.GGMLType.Q8_0)
    prompt = torch.randint(0, 96, (1, 20), generator=torch.Generator().manual_seed(1))
    with torch.no_grad():
        want = ref(prompt).logits[:, -1]
    for rt in (llm.LlamaRuntime.from_hf(d, device="cpu"), llm.LlamaRuntime.from_gguf(out, device="cpu")):
        assert rt.cfg.context_length == 24
        got = rt.prefill(prompt, rt.new_cache(1, 24))
        assert float((want - got).abs().max()) < 0.03 * float(want.abs().max())
