"""Model zoo on CPU: shapes, the fixed ResNet semantics, Keras-style fit, save/load in every format."""
import pytest
import torch

from rustorch_b200 import models as M
from rustorch_b200 import nn


def test_resnet18_structure_and_residual():
    m = M.resnet18(10)
    assert M.count_parameters(m) == 11181642          # torchvision's resnet18 with 10 classes
    x = torch.randn(2, 3, 64, 64)
    assert m(x).shape == (2, 10)
    blk = M.BasicBlock(8, 8)
    with torch.no_grad():
        for p in blk.parameters():
            p.zero_()
    blk.eval()
    y = blk(torch.ones(1, 8, 4, 4))
    assert torch.allclose(y, torch.ones(1, 8, 4, 4))   # zero branch => output is the identity path (the add exists)
    assert M.ResNetBuilder().depth(34).num_classes(5).build()(x).shape == (2, 5)
    assert M.resnet50(7)(x).shape == (2, 7)
    with pytest.raises(ValueError):
        M.ResNetBuilder().depth(19)


def test_cnn_rnn_seq2seq_bert_transformer_shapes():
    c = M.CNNBuilder().input_shape(1, 28, 28).conv_channels([8, 16]).fc_sizes([32]).num_classes(10).batch_norm().build()
    assert c(torch.randn(3, 1, 28, 28)).shape == (3, 10)
    tok = torch.randint(0, 50, (4, 9))
    assert M.RNNModel(50, 16, 32, 3)(tok).shape == (4, 3)
    assert M.LSTMModel(50, 16, 32, 3, 2, True, 0.1)(tok).shape == (4, 3)
    s2s = M.Seq2SeqModel(50, 60, 16, 32)
    assert s2s(tok, torch.randint(0, 60, (4, 5))).shape == (4, 5, 60)
    assert s2s.generate(tok, bos=1, max_len=6).shape == (4, 6)
    cfg = M.BERTConfig(vocab_size=100, hidden_size=32, num_hidden_layers=2, num_attention_heads=4, intermediate_size=64,
                       max_position_embeddings=16)
    bert = M.BERT(cfg, num_labels=3)
    mask = torch.ones(4, 9)
    mask[:, -2:] = 0
    seq, pooled = bert(tok, attention_mask=mask)
    assert seq.shape == (4, 9, 32) and pooled.shape == (4, 32) and bert.classify(tok).shape == (4, 3)
    assert bert.masked_lm_logits(tok).shape == (4, 9, 100)
    assert M.BERTConfig.bert_large_uncased().num_hidden_layers == 24
    tm = M.TransformerModelBuilder().vocab_size(50).d_model(32).nhead(4).num_layers(2).dim_feedforward(64).causal(True).build()
    assert tm(tok).shape == (4, 9, 50)
    assert M.gpt2_medium is not None and M.GPTConfig.gpt2_medium().n_layer == 24


def test_keras_style_fit_evaluate_predict():
    torch.manual_seed(0)
    X = torch.randn(200, 4)
    y = (X.sum(1) > 0).long()
    model = M.ModelBuilder().linear(4, 16).relu().linear(16, 2).build().compile("adam", "cross_entropy", ["accuracy"], lr=0.05)
    hist = model.fit(X, y, epochs=15, batch_size=32, validation_split=0.2, seed=0)
    assert hist.loss[-1] < hist.loss[0] and hist.metrics["accuracy"][-1] > 0.9 and len(hist.val_loss) == 15
    assert model.evaluate(X, y)["accuracy"] > 0.9 and model.predict(X[:5]).shape == (5, 2)
    assert "Total params: 114" in model.summary() and model.mode() is M.ModelMode.EVAL
    eng = M.InferenceEngine(model)
    eng.predict_batch([X[:3], X[3:7]])
    assert eng.stats()["n"] == 2


@pytest.mark.parametrize("fmt,ext", [(M.SerializationFormat.RUSTORCH, "rt"), (M.SerializationFormat.SAFETENSORS, "safetensors"),
                                     (M.SerializationFormat.PYTORCH, "pt"), (M.SerializationFormat.JSON, "json")])
def test_save_load_every_format(tmp_path, fmt, ext):
    a = nn.Sequential(nn.Linear(4, 3), nn.BatchNorm1d(3))
    b = nn.Sequential(nn.Linear(4, 3), nn.BatchNorm1d(3))
    p = str(tmp_path / f"m.{ext}")
    M.ModelSaver.save(a, p, fmt)
    M.ModelLoader.load(b, p)
    assert torch.allclose(a[0].weight, b[0].weight)
    assert M.ModelInfo.of(a, p).size_bytes > 0


def test_checkpoint_with_optimizer_moments(tmp_path):
    m = nn.Linear(3, 2)
    o = torch.optim.Adam(m.parameters(), 0.1)
    m(torch.ones(1, 3)).sum().backward()
    o.step()
    p = str(tmp_path / "ck.rt")
    M.ModelSaver.save_checkpoint(m, o, p, epoch=2, step=7, metrics={"loss": 0.5})
    m2 = nn.Linear(3, 2)
    o2 = torch.optim.Adam(m2.parameters(), 0.1)
    ck = M.ModelLoader.load_checkpoint(m2, o2, p)
    assert ck["epoch"] == 2 and ck["metrics"]["loss"] == 0.5 and torch.equal(m.weight, m2.weight)
    st = list(o2.state_dict()["state"].values())
    assert st and "exp_avg" in st[0]


def test_llama_training_model_cpu():
    from rustorch_b200.models.llama import LlamaModel, LlamaTrainConfig, apply_rope, rope_tables
    torch.manual_seed(0)
    cfg = LlamaTrainConfig.tiny(n_layer=2, n_embd=64, n_head=4, n_head_kv=2, n_ff=128, vocab_size=97)
    m = LlamaModel(cfg)
    idx = torch.randint(0, 97, (2, 16))
    logits, loss = m(idx, idx.roll(-1, 1))
    assert logits.shape == (32, 97) and 3.5 < float(loss) < 6.0
    loss.backward()
    assert all(p.grad is not None and torch.isfinite(p.grad).all() for p in m.parameters())
    opt = torch.optim.AdamW(m.parameters(), lr=3e-3)
    first = float(loss)
    for _ in range(20):
        opt.zero_grad()
        _, l = m(idx, idx.roll(-1, 1))
        l.backward()
        opt.step()
    assert float(l) < first * 0.7
    # rotary embedding: norm preserving, position 0 is the identity, relative property q_m . k_n depends on m - n
    cos, sin = rope_tables(8, 16, 10000.0, "cpu")
    x = torch.randn(1, 8, 1, 16)
    r = apply_rope(x, cos, sin)
    assert torch.allclose(r.norm(dim=-1), x.norm(dim=-1), atol=1e-5) and torch.allclose(r[:, 0], x[:, 0])
    q = torch.randn(16)
    k = torch.randn(16)
    qs = apply_rope(q.expand(1, 8, 1, 16), cos, sin)[0, :, 0]
    ks = apply_rope(k.expand(1, 8, 1, 16), cos, sin)[0, :, 0]
    assert torch.allclose(qs[5] @ ks[3], qs[4] @ ks[2], atol=1e-4)
    assert LlamaTrainConfig.llama3_8b().n_head_kv == 8 and m.num_parameters() > 0


def test_load_checkpoint_rejects_a_checkpoint_of_another_model(tmp_path):
    a, b = torch.nn.Linear(4, 2), torch.nn.Sequential(torch.nn.Linear(4, 2))
    oa = torch.optim.SGD(a.parameters(), 0.1)
    p = str(tmp_path / "a.ckpt")
    M.ModelSaver.save_checkpoint(a, oa, p, epoch=1, step=2, metrics={"loss": 1.0})
    with pytest.raises(RuntimeError):
        M.ModelLoader.load_checkpoint(b, None, p)                    # names differ: nothing would have been restored
    before = b[0].weight.detach().clone()
    M.ModelLoader.load_checkpoint(b, None, p, strict=False)
    assert torch.equal(b[0].weight, before)
    a2 = torch.nn.Linear(4, 2)
    ck = M.ModelLoader.load_checkpoint(a2, None, p)
    assert torch.equal(a2.weight, a.weight) and ck["epoch"] == 1


def test_metrics_summary():
    """src/models/mod.rs:118-152 plus a real computation from predictions (macro averages)."""
    m = M.Metrics.from_predictions(torch.tensor([[2., 1.], [0., 3.], [1., 0.], [0., 1.]]), torch.tensor([0, 1, 1, 1]), 0.3)
    assert m.accuracy == 0.75 and m.precision == 0.75 and m.recall == pytest.approx(5 / 6) and m.f1_score == pytest.approx(2 * 0.75 * (5 / 6) / (0.75 + 5 / 6))
    assert m.loss == 0.3 and M.Metrics.new().accuracy == 0.0 and M.Metrics.with_values(1, 0.9, 0.8, 0.85, 0.1).recall == 0.8
    ids = M.Metrics.from_predictions(torch.tensor([0, 2, 2]), torch.tensor([0, 1, 2]), num_classes=3)
    assert ids.accuracy == pytest.approx(2 / 3) and ids.precision == pytest.approx((1 + 0 + 0.5) / 3) and ids.recall == pytest.approx((1 + 0 + 1) / 3)


def test_llama_training_model_matches_transformers(tmp_path):
    """``LlamaModel.from_hf`` copies a Hugging Face checkpoint; logits, loss and gradients equal ``transformers``' Llama
    (grouped-query attention, rotate-half RoPE, SwiGLU, RMSNorm) in fp32 on CPU."""
    tf = pytest.importorskip("transformers")
    from rustorch_b200.models.llama import LlamaModel
    torch.manual_seed(0)
    hc = tf.LlamaConfig(vocab_size=96, hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                        num_key_value_heads=2, max_position_embeddings=64, rms_norm_eps=1e-5, rope_theta=10000.0, tie_word_embeddings=False)
    ref = tf.LlamaForCausalLM(hc)
    d = str(tmp_path / "hf")
    ref.save_pretrained(d, safe_serialization=True)
    m = LlamaModel.from_hf(d)
    assert m.cfg.n_head_kv == 2 and m.num_parameters() == sum(p.numel() for p in ref.parameters())
    idx, tgt = torch.randint(0, 96, (2, 12)), torch.randint(0, 96, (2, 12))
    logits, loss = m(idx, tgt)
    want = ref(idx).logits.view(-1, 96)
    want_loss = torch.nn.functional.cross_entropy(want, tgt.view(-1))
    assert torch.allclose(logits, want, atol=1e-5) and float(loss.detach()) == pytest.approx(float(want_loss.detach()), rel=1e-6)
    loss.backward()
    want_loss.backward()
    l0 = ref.model.layers[0]
    qkv = torch.cat([l0.self_attn.q_proj.weight.grad, l0.self_attn.k_proj.weight.grad, l0.self_attn.v_proj.weight.grad], 0)
    gu = torch.cat([l0.mlp.gate_proj.weight.grad, l0.mlp.up_proj.weight.grad], 0)
    assert torch.allclose(m.blocks[0].wqkv.grad, qkv, atol=1e-6) and torch.allclose(m.blocks[0].w_gate_up.grad, gu, atol=1e-6)
    assert torch.allclose(m.tok_emb.grad, ref.model.embed_tokens.weight.grad, atol=1e-6)
    assert torch.allclose(m.blocks[1].attn_norm.grad, ref.model.layers[1].input_layernorm.weight.grad, atol=1e-6)


def test_bert_matches_transformers(tmp_path):
    """``BERT.from_hf``: embeddings, post-norm encoder (erf GELU), pooler and the padding mask agree with ``transformers``'
    BertModel."""
    tf = pytest.importorskip("transformers")
    torch.manual_seed(0)
    hc = tf.BertConfig(vocab_size=120, hidden_size=64, num_hidden_layers=2, num_attention_heads=4, intermediate_size=128,
                       max_position_embeddings=40, hidden_dropout_prob=0.0, attention_probs_dropout_prob=0.0)
    ref = tf.BertModel(hc).eval()
    with torch.no_grad():
        for p in ref.parameters():
            if p.dim() == 1:
                p.add_(torch.randn_like(p) * 0.1)
    d = str(tmp_path / "bert")
    ref.save_pretrained(d, safe_serialization=True)
    m = M.BERT.from_hf(d).eval()
    ids, tt = torch.randint(0, 120, (2, 10)), torch.randint(0, 2, (2, 10))
    mask = torch.ones(2, 10, dtype=torch.long)
    mask[1, 7:] = 0
    with torch.no_grad():
        want = ref(ids, token_type_ids=tt)
        seq, pooled = m(ids, tt)
        assert torch.allclose(seq, want.last_hidden_state, atol=2e-5) and torch.allclose(pooled, want.pooler_output, atol=2e-5)
        wm = ref(ids, token_type_ids=tt, attention_mask=mask)
        sm, pm = m(ids, tt, attention_mask=mask)
        assert torch.allclose(sm[0], wm.last_hidden_state[0], atol=2e-5) and torch.allclose(sm[1, :7], wm.last_hidden_state[1, :7], atol=2e-5)
        assert torch.allclose(pm, wm.pooler_output, atol=2e-5) and not torch.allclose(sm[1, :7], seq[1, :7], atol=1e-4)
    assert m.masked_lm_logits(ids).shape == (2, 10, 120) and m.classify(ids).shape == (2, 2)


def test_llama_from_hf_applies_rope_base_and_scaling(tmp_path):
    """The RoPE base and the llama3 / linear frequency scaling of a Hugging Face config reach the training model: logits
    agree with ``transformers`` at positions where the unscaled tables are measurably off, and ``save_hf`` keeps them."""
    tf = pytest.importorskip("transformers")
    from rustorch_b200.models.llama import LlamaModel, scale_rope_frequencies
    idx = torch.randint(0, 96, (2, 100), generator=torch.Generator().manual_seed(3))
    for rs in ({"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0, "original_max_position_embeddings": 32},
               {"rope_type": "linear", "factor": 2.0}, None):
        torch.manual_seed(0)
        hc = tf.LlamaConfig(vocab_size=96, hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                            num_key_value_heads=2, max_position_embeddings=128, rope_theta=50000.0, rope_scaling=rs, tie_word_embeddings=False)
        ref = tf.LlamaForCausalLM(hc).eval()
        d = str(tmp_path / f"hf_{rs['rope_type'] if rs else 'plain'}")
        ref.save_pretrained(d, safe_serialization=True)
        m = LlamaModel.from_hf(d).eval()
        assert m.cfg.rope_theta == 50000.0 and (m.cfg.rope_scaling or {}).get("rope_type") == (rs or {}).get("rope_type")
        with torch.no_grad():
            want = ref(idx).logits.view(-1, 96)
            assert float((want - m(idx)[0]).abs().max()) < 2e-5
            if rs:
                m.cfg.rope_scaling, m._rope = None, None
                assert float((want - m(idx)[0]).abs().max()) > 1e-3      # the scaling is what made them agree
                m.cfg.rope_scaling, m._rope = rs, None
        out = str(tmp_path / f"out_{rs['rope_type'] if rs else 'plain'}")
        m.save_hf(out)
        with torch.no_grad():
            assert torch.allclose(tf.LlamaForCausalLM.from_pretrained(out).eval()(idx).logits.view(-1, 96), want, atol=2e-5)
    with pytest.raises(ValueError, match="yarn"):
        scale_rope_frequencies(torch.ones(4), {"rope_type": "yarn", "factor": 2.0})


def test_save_hf_is_read_back_by_transformers(tmp_path):
    """Fine-tuning loop closed: a model of this package written with ``save_hf`` loads in ``transformers`` and gives the
    same logits; ``from_hf`` of the written directory reproduces the parameters."""
    tf = pytest.importorskip("transformers")
    from rustorch_b200.models.gpt import GPT, GPTConfig
    from rustorch_b200.models.llama import LlamaModel, LlamaTrainConfig
    torch.manual_seed(0)
    lm = LlamaModel(LlamaTrainConfig.tiny(vocab_size=96, n_embd=64, n_ff=128, max_seq_len=64))
    with torch.no_grad():
        for b in lm.blocks:
            b.attn_norm.add_(torch.randn_like(b.attn_norm) * 0.1)
    d = str(tmp_path / "llama")
    lm.save_hf(d)
    ref = tf.LlamaForCausalLM.from_pretrained(d).eval()
    idx = torch.randint(0, 96, (2, 10))
    with torch.no_grad():
        assert torch.allclose(lm(idx)[0], ref(idx).logits.view(-1, 96), atol=1e-5)
    back = LlamaModel.from_hf(d)
    assert all(torch.equal(a, b) for a, b in zip(lm.parameters(), back.parameters()))
    g = GPT(GPTConfig(vocab_size=100, n_positions=32, n_embd=64, n_layer=2, n_head=4, dropout=0.0, tie_weights=True), seed=0).eval()
    with torch.no_grad():
        for b in g.blocks:
            b.b_qkv.normal_(0, 0.1)
            b.ln2_b.normal_(0, 0.1)
    d2 = str(tmp_path / "gpt2")
    g.save_hf(d2)
    ref2 = tf.GPT2LMHeadModel.from_pretrained(d2).eval()
    ids = torch.randint(0, 100, (2, 12))
    with torch.no_grad():
        assert torch.allclose(g.forward_reference(ids), ref2(ids).logits, atol=1e-5)
    assert all(torch.equal(a, b) for a, b in zip(g.parameters(), GPT.from_hf(d2).parameters()))
    with pytest.raises(ValueError, match="ties the head"):
        GPT(GPTConfig(vocab_size=100, n_positions=32, n_embd=64, n_layer=1, n_head=4), seed=0).save_hf(str(tmp_path / "untied"))


def test_metrics_against_sklearn():
    sk = pytest.importorskip("sklearn.metrics")
    g = torch.Generator().manual_seed(0)
    y = torch.randint(0, 5, (400,), generator=g)
    pred = torch.where(torch.rand(400, generator=g) < 0.7, y, torch.randint(0, 5, (400,), generator=g))
    m = M.Metrics.from_predictions(pred, y, num_classes=5)
    p, r, _f, _ = sk.precision_recall_fscore_support(y.numpy(), pred.numpy(), average="macro", zero_division=0)
    assert m.accuracy == pytest.approx(sk.accuracy_score(y.numpy(), pred.numpy())) and m.precision == pytest.approx(p) and m.recall == pytest.approx(r)
    assert m.f1_score == pytest.approx(2 * p * r / (p + r))           # harmonic mean of the macro averages (src/models/mod.rs keeps one f1 field)


def test_resnet_takes_torchvision_weights(tmp_path):
    """``ResNet.from_torchvision``: same tensors, same logits as the torchvision model, in eval and in training mode
    (batch statistics), for basic-block and bottleneck depths; from the module, the state dict or a saved file."""
    tv = pytest.importorskip("torchvision")
    from rustorch_b200.models.cnn import ResNet
    x = torch.randn(2, 3, 64, 64, generator=torch.Generator().manual_seed(0))
    for name in ("resnet18", "resnet50"):
        torch.manual_seed(0)
        ref = getattr(tv.models, name)(num_classes=10)
        with torch.no_grad():
            for m in ref.modules():
                if isinstance(m, torch.nn.BatchNorm2d):
                    m.running_mean.normal_(0, 0.1)
                    m.running_var.uniform_(0.5, 1.5)
                    m.weight.uniform_(0.5, 1.5)
        mine = ResNet.from_torchvision(ref)
        assert sum(p.numel() for p in mine.parameters()) == sum(p.numel() for p in ref.parameters())
        with torch.no_grad():
            assert torch.allclose(ref.eval()(x), mine.eval()(x), atol=1e-5)
            assert torch.allclose(ref.train()(x), mine.train()(x), atol=1e-5)
    path = str(tmp_path / "r18.pth")
    ref18 = tv.models.resnet18(num_classes=7)
    torch.save({"state_dict": {"module." + k: v for k, v in ref18.state_dict().items()}}, path)     # a DataParallel-style checkpoint
    assert ResNet.from_torchvision(path).fc.out_features == 7
    with pytest.raises(ValueError, match="wide and grouped"):
        ResNet.from_torchvision(tv.models.wide_resnet50_2(num_classes=3).state_dict())
    with pytest.raises(ValueError, match="not a torchvision ResNet"):
        ResNet.from_torchvision({"a": torch.zeros(1)})


def test_gpt_forward_cached_equals_the_full_forward():
    """Prefill + decode steps (one token, then three at once) against the key / value cache reproduce the logits of the
    whole-sequence forward; the CLI adapter built on it slides its window when the learned positions run out."""
    from rustorch_b200.cli.engine import _GPTAdapter
    from rustorch_b200.models.gpt import GPT, GPTConfig
    g = GPT(GPTConfig(vocab_size=100, n_positions=16, n_embd=64, n_layer=2, n_head=4, dropout=0.0, tie_weights=True), seed=0).eval()
    with torch.no_grad():
        for b in g.blocks:
            b.b_qkv.normal_(0, 0.1)
    ids = torch.randint(0, 100, (2, 12), generator=torch.Generator().manual_seed(0))
    with torch.no_grad():
        want = g.forward_reference(ids)
        l0, kv = g.forward_cached(ids[:, :8])
        l1, kv = g.forward_cached(ids[:, 8:9], kv)
        l2, kv = g.forward_cached(ids[:, 9:12], kv)
    assert torch.allclose(torch.cat([l0, l1, l2], 1), want, atol=1e-5) and kv[0][0].shape == (2, 4, 12, 16)
    with pytest.raises(ValueError, match="learned positions"):
        g.forward_cached(ids[:, :6], kv)
    ad = _GPTAdapter(g, "cpu")
    logits = ad.prefill(ids[:1], ad.new_cache(1, 64))
    assert torch.allclose(logits, want[:1, -1], atol=1e-5)
    seq = ids[:1]
    for step in range(8):                                # crosses the 16 learned positions at the fifth step
        nxt = logits.argmax(-1)
        seq = torch.cat([seq, nxt[:, None]], 1)
        logits = ad.decode_step(nxt, ad)
        window = seq if seq.shape[1] <= 16 else ad.tokens
        with torch.no_grad():
            assert torch.allclose(logits, g.forward_reference(window)[:, -1], atol=1e-5), step
    assert ad.tokens.shape[1] <= 16 and torch.equal(ad.tokens, seq[:, -ad.tokens.shape[1]:])
