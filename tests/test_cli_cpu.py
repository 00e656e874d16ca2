"""CPU tests of the CLI: arguments, configuration, commands, session, tokenizers, download logic, REPL end to end."""
import json
import os

import pytest
import torch

from rustorch_b200 import cli
from rustorch_b200.formats import gguf


def test_args_defaults_overrides_and_validation(tmp_path):
    a = cli.parse_args([])
    assert (a.max_tokens, a.temperature, a.top_p, a.top_k, a.backend) == (512, 0.7, 0.9, 40, cli.Backend.CPU)
    cfg = tmp_path / "c.toml"
    cfg.write_text('[generation]\nmax_tokens = 64\ntemperature = 0.2\n[model]\ndefault = "m.gguf"\n[backend]\ndefault = "cuda"\n')
    a = cli.parse_args(["--config", str(cfg), "--temperature", "1.5"])
    assert a.max_tokens == 64 and a.temperature == 1.5 and a.model == "m.gguf" and a.backend is cli.Backend.CUDA
    with pytest.raises(ValueError):
        cli.parse_args(["--temperature", "3"])
    with pytest.raises(ValueError):
        cli.parse_args(["--top-k", "0"])
    d = cli.parse_args(["download", "hf:org/repo", "--force"])
    assert d.command == "download" and d.target == "hf:org/repo" and d.force
    assert cli.Backend.METAL.available() is False and cli.Backend.METAL.device() in ("cpu", "cuda")


def test_config_roundtrip_and_errors(tmp_path):
    c = cli.Config()
    c.generation.top_k = 7
    c.model.default = 'a "quoted" path'
    p = c.save(str(tmp_path / "cfg" / "config.toml"))
    back = cli.Config.load(p)
    assert back.generation.top_k == 7 and back.model.default == 'a "quoted" path' and back.session.max_history == 1000
    assert cli.Config.load_or_default(str(tmp_path / "missing.toml")).generation.max_tokens == 512
    (tmp_path / "bad.toml").write_text("[generation]\nbogus = 1\n")
    with pytest.raises(ValueError):
        cli.Config.load(str(tmp_path / "bad.toml"))


def test_command_parsing():
    K = cli.CommandKind
    for text, kind in (("/exit", K.EXIT), ("/quit", K.EXIT), ("/q", K.EXIT), ("/help", K.HELP), ("/?", K.HELP), ("/cls", K.CLEAR),
                       ("/stats", K.STATS), ("/config", K.CONFIG)):
        assert cli.Command.parse(text).kind is kind
    assert cli.Command.parse("/save x.json").arg == "x.json" and cli.Command.parse("/save").arg is None
    assert cli.Command.parse("/system You are helpful").arg == "You are helpful"
    assert cli.Command.parse("/nope").kind is K.UNKNOWN
    for bad in ("/backend", "/system", "/load", "/model"):
        with pytest.raises(ValueError):
            cli.Command.parse(bad)
    assert not cli.Command.is_command("hello")


def test_session_history_save_load(tmp_path):
    s = cli.SessionManager(cli.GenerationConfig(max_tokens=8), "cpu", "m", max_history=3)
    s.set_system_prompt("Be brief.")
    for i in range(3):
        s.add_user_message(f"q{i}")
        s.add_assistant_message(f"a{i}")
    assert s.message_count() == 3 and s.get_messages()[0].content == "a1"       # capped
    assert s.build_prompt().startswith("Be brief.\n") and s.build_prompt().endswith("Assistant:")
    p = str(tmp_path / "h.json")
    s.save_history(p)
    t = cli.SessionManager()
    t.load_history(p)
    assert [m.content for m in t.get_messages()] == ["a1", "q2", "a2"] and t.system_prompt() == "Be brief."
    assert json.load(open(p))["generation"]["max_tokens"] == 8 and s.total_tokens() == 3
    with pytest.raises(ValueError):
        cli.SessionManager(cli.GenerationConfig(temperature=9))


def test_tokenizers():
    bt = cli.ByteTokenizer()
    ids = bt.encode("héllo")
    assert ids[0] == bt.bos_id and bt.decode(ids) == "héllo"
    toks = ["<unk>", "<s>", "</s>"] + [f"<0x{b:02X}>" for b in range(256)] + ["▁", "h", "e", "l", "o", "▁h", "he", "ll", "▁he", "llo", "▁hello", "w", "▁w"]
    scores = [0.0] * 259 + [-1, -2, -2, -2, -2, -3, -3, -3, -4, -5, -6, -2, -3]
    types = [2, 3, 3] + [6] * 256 + [1] * 13
    gt = cli.GGUFTokenizer(toks, [-s if s > 0 else s for s in scores], types)
    # higher score merges first; the full word exists so it becomes one token
    ids = gt.encode("hello")
    assert ids[0] == 1 and gt.decode(ids) == "hello"
    assert gt.decode(gt.encode("hello wé")) == "hello wé"                      # byte fallback for é
    assert any(259 <= i for i in gt.encode("hello", add_bos=False))


def test_download_identifiers_and_offline_logic(tmp_path):
    i = cli.ModelIdentifier.parse("hf:TheBloke/Llama-2-7B-GGUF:llama-2-7b.Q4_0.gguf")
    assert i.source is cli.ModelSource.HUGGINGFACE and i.repo_id == "TheBloke/Llama-2-7B-GGUF" and i.filename.endswith("Q4_0.gguf")
    o = cli.ModelIdentifier.parse("ollama:llama2:7b")
    assert o.source is cli.ModelSource.OLLAMA and o.repo_id == "llama2" and o.revision == "7b"
    for bad in ("llama", "s3:x/y", "hf:norepo", "hf:"):
        with pytest.raises(ValueError):
            cli.ModelIdentifier.parse(bad)
    hf = cli.HuggingFaceClient(token="t")
    assert hf.file_url("a/b", "f.gguf", "dev") == "https://huggingface.co/a/b/resolve/dev/f.gguf" and hf._headers()["Authorization"] == "Bearer t"
    from rustorch_b200.cli.download import ModelFile
    files = [ModelFile("README.md"), ModelFile("m.Q8_0.gguf"), ModelFile("m.Q4_0.gguf")]
    assert hf.recommend_gguf(files, ["Q4_0", "Q8_0"]).filename == "m.Q4_0.gguf" and len(hf.find_gguf_files(files)) == 2
    assert cli.OllamaClient().manifest_url("llama2", "7b") == "https://registry.ollama.ai/v2/library/llama2/manifests/7b"
    assert cli.OllamaClient.model_layer({"layers": [{"mediaType": "application/vnd.ollama.image.model", "digest": "sha256:x"}]})["digest"] == "sha256:x"
    mgr = cli.ModelDownloadManager(str(tmp_path))
    d = mgr.target_dir(i)
    os.makedirs(d)
    open(os.path.join(d, "llama-2-7b.Q4_0.gguf"), "wb").close()
    assert mgr.list_models() == ["hf:TheBloke/Llama-2-7B-GGUF:llama-2-7b.Q4_0.gguf"] and mgr.list_models(cli.ModelSource.OLLAMA) == []


def _tiny_gguf(path):
    torch.manual_seed(0)
    V, d, ff, L, H = 300, 64, 128, 2, 2
    toks = ["<unk>", "<s>", "</s>"] + [f"<0x{b:02X}>" for b in range(256)] + ["▁", "a", "b", "▁a", "ab"] + [f"t{i}" for i in range(V - 264)]
    md = {"general.architecture": "llama", "llama.block_count": L, "llama.embedding_length": d, "llama.feed_forward_length": ff,
          "llama.attention.head_count": H, "llama.attention.head_count_kv": H, "llama.context_length": 64,
          "llama.attention.layer_norm_rms_epsilon": 1e-5, "llama.rope.freq_base": 10000.0,
          "tokenizer.ggml.model": "llama", "tokenizer.ggml.tokens": toks, "tokenizer.ggml.scores": [0.0] * V,
          "tokenizer.ggml.token_type": [2, 3, 3] + [6] * 256 + [1] * (V - 259),
          "tokenizer.ggml.bos_token_id": 1, "tokenizer.ggml.eos_token_id": 2}
    Q = gguf.GGMLType.Q8_0
    t = {"token_embd.weight": (torch.randn(V, d) * 0.1, gguf.GGMLType.F32), "output_norm.weight": (torch.ones(d), gguf.GGMLType.F32),
         "output.weight": (torch.randn(V, d) * 0.1, Q)}
    for i in range(L):
        p = f"blk.{i}."
        for n, shp in (("attn_q", (d, d)), ("attn_k", (d, d)), ("attn_v", (d, d)), ("attn_output", (d, d)), ("ffn_gate", (ff, d)),
                       ("ffn_up", (ff, d)), ("ffn_down", (d, ff))):
            t[p + n + ".weight"] = (torch.randn(*shp) * 0.1, Q)
        t[p + "attn_norm.weight"] = (torch.ones(d), gguf.GGMLType.F32)
        t[p + "ffn_norm.weight"] = (torch.ones(d), gguf.GGMLType.F32)
    gguf.write_gguf(path, md, t)


def test_repl_end_to_end_with_gguf_model(tmp_path):
    model = str(tmp_path / "tiny.gguf")
    _tiny_gguf(model)
    hist = str(tmp_path / "hist.json")
    lines = iter(["/help", "/system Be terse.", "ab a", "/stats", "/config", f"/save {hist}", "/clear", "/bogus", "/backend metal", "/exit"])
    buf = []
    rc = cli.main(["--model", model, "--max-tokens", "6", "--temperature", "0"], read=lambda _: next(lines), out=buf.append)
    text = "".join(buf)
    assert rc == 0 and "Commands:" in text and "Assistant: " in text and "tokens generated: " in text and "Goodbye!" in text
    assert "Unknown command '/bogus'" in text and "not available" in text and "model: tiny.gguf" in text
    doc = json.load(open(hist))
    assert [m["role"] for m in doc["messages"]] == ["user", "assistant"] and doc["system_prompt"] == "Be terse."
    # deterministic at temperature 0: one-shot mode gives the same reply as the REPL turn
    buf2 = []
    assert cli.main(["--model", model, "--max-tokens", "6", "--temperature", "0", "--system-prompt", "Be terse.", "--prompt", "ab a"], out=buf2.append) == 0
    assert doc["messages"][1]["content"] == "".join(buf2).split("Assistant: ", 1)[1].strip()


def test_dummy_model_and_list_command(tmp_path):
    buf = []
    assert cli.main(["--prompt", "hi there"], out=buf.append) == 0 and "You said: " in "".join(buf)
    buf = []
    assert cli.main(["list", "hf"], out=buf.append) == 0
    buf = []
    assert cli.main(["--model", str(tmp_path / "nope.gguf"), "--prompt", "x"], out=buf.append) == 1 and "cannot load model" in "".join(buf)
    assert cli.main(["download", "ftp:x"], out=buf.append) == 2


def test_repl_survives_a_failed_generation(tmp_path):
    """A model without an embedded tokenizer and a prompt whose byte-level ids exceed its vocabulary: the turn is
    reported and dropped, the session goes on (the reference's REPL prints the error and continues,
    example-cli/src/cli/repl.rs)."""
    import sys
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    from test_llm_cpu import _tiny_gguf as plain_gguf                # no tokenizer metadata, vocabulary of 64
    model = str(tmp_path / "plain.gguf")
    plain_gguf(model)
    lines = iter(["hello there", "/stats", "/exit"])
    buf = []
    rc = cli.main(["--model", model, "--backend", "cpu", "--max-tokens", "4"], read=lambda _: next(lines), out=buf.append)
    text = "".join(buf)
    assert rc == 0 and "error: ValueError: the tokenizer produced id" in text and "--tokenizer" in text
    assert "messages: 0" in text and "Goodbye!" in text             # the failed turn left no half conversation behind
    one = []
    assert cli.main(["--model", model, "--backend", "cpu", "--prompt", "hello"], out=one.append) == 1 and "error:" in "".join(one)


def test_cli_runs_a_hugging_face_llama_directory(tmp_path):
    tf = pytest.importorskip("transformers")
    torch.manual_seed(0)
    hc = tf.LlamaConfig(vocab_size=300, hidden_size=64, intermediate_size=128, num_hidden_layers=1, num_attention_heads=4,
                        num_key_value_heads=2, max_position_embeddings=128, tie_word_embeddings=True)
    d = str(tmp_path / "hf-llama")
    tf.LlamaForCausalLM(hc).save_pretrained(d, safe_serialization=True)
    buf = []
    assert cli.main(["--model", d, "--backend", "cpu", "--max-tokens", "4", "--temperature", "0", "--prompt", "hi"], out=buf.append) == 0
    assert "Assistant: " in "".join(buf) and "error" not in "".join(buf)
    lines = iter(["/config", "/exit"])
    buf2 = []
    cli.main(["--model", d, "--backend", "cpu"], read=lambda _: next(lines), out=buf2.append)
    assert "model: hf-llama" in "".join(buf2)


def _tiny_bpe_files(directory):
    """vocab.json + merges.txt of a byte-level BPE trained on a few sentences (60 merges)."""
    import collections
    import regex
    from rustorch_b200.cli.tokenizer import BPETokenizer, _byte_alphabet
    text = "Hello world! The quick brown fox jumps over the lazy dog. It's 2024, isn't it?  Naïve café — 東京 \n\n tabs\tand   spaces. " * 3
    tab = _byte_alphabet()
    words = collections.Counter("".join(tab[b] for b in w.encode()) for w in regex.compile(BPETokenizer._PATTERN).findall(text))
    vocab = {tab[b]: b for b in range(256)}
    vocab = {c: i for i, c in enumerate(tab[b] for b in range(256))}
    merges, seqs = [], {w: list(w) for w in words}
    for _ in range(60):
        pairs = collections.Counter()
        for w, s in seqs.items():
            for a, b in zip(s, s[1:]):
                pairs[(a, b)] += words[w]
        (a, b), _n = pairs.most_common(1)[0]
        merges.append((a, b))
        vocab[a + b] = len(vocab)
        for w, s in seqs.items():
            out, i = [], 0
            while i < len(s):
                if i < len(s) - 1 and s[i] == a and s[i + 1] == b:
                    out.append(a + b)
                    i += 2
                else:
                    out.append(s[i])
                    i += 1
            seqs[w] = out
    vocab["<|endoftext|>"] = len(vocab)
    os.makedirs(directory, exist_ok=True)
    json.dump(vocab, open(os.path.join(directory, "vocab.json"), "w", encoding="utf-8"), ensure_ascii=False)
    open(os.path.join(directory, "merges.txt"), "w", encoding="utf-8").write("#version: 0.2\n" + "\n".join(" ".join(m) for m in merges) + "\n")
    return text, len(vocab)


def test_bpe_tokenizer_matches_transformers(tmp_path):
    tf = pytest.importorskip("transformers")
    from rustorch_b200.cli.tokenizer import BPETokenizer, load_tokenizer
    d = str(tmp_path / "tok")
    text, n = _tiny_bpe_files(d)
    ours = load_tokenizer(d)
    assert isinstance(ours, BPETokenizer) and ours.vocab_size == n and ours.eos_id == n - 1 and ours.bos_id is None
    hf = tf.GPT2Tokenizer(os.path.join(d, "vocab.json"), os.path.join(d, "merges.txt"))
    for t in (text, "isn't it lazy?", "  leading and trailing  ", "unseen ZZZ qqq 東 ☃", ""):
        ids = ours.encode(t)
        assert ids == hf.encode(t) and ours.decode(ids) == t
    assert len(ours.encode("the lazy dog")) < len("the lazy dog")        # merges really apply
    bad = dict(ours.vocab)
    del bad[next(k for k in bad if len(k) > 1 and k.startswith("Ġ"))]
    with pytest.raises(ValueError, match="not in the vocabulary"):
        BPETokenizer(bad, list(ours.rank)).encode(text)


def test_cli_runs_a_hugging_face_gpt2_directory(tmp_path):
    """``config.json`` + safetensors + vocab.json / merges.txt of a GPT-2 checkpoint: weights load into the GPT model
    (logits equal ``transformers``'), the BPE tokenizer is picked up, one prompt is answered."""
    tf = pytest.importorskip("transformers")
    from rustorch_b200.models.gpt import GPT
    d = str(tmp_path / "gpt2-tiny")
    _, n = _tiny_bpe_files(d)
    torch.manual_seed(0)
    hc = tf.GPT2Config(vocab_size=n, n_positions=64, n_embd=64, n_layer=2, n_head=4, resid_pdrop=0.0, embd_pdrop=0.0, attn_pdrop=0.0)
    ref = tf.GPT2LMHeadModel(hc).eval()
    with torch.no_grad():
        for p in ref.parameters():
            if p.dim() == 1:
                p.add_(torch.randn_like(p) * 0.1)                     # non-trivial biases and norm parameters
    ref.save_pretrained(d, safe_serialization=True)
    m = GPT.from_hf(d).eval()
    idx = torch.randint(0, n, (2, 16))
    with torch.no_grad():
        want = ref(idx).logits
    got = m.forward_reference(idx)
    assert m.cfg.tie_weights and got.shape == want.shape and torch.allclose(got, want, atol=1e-5)
    assert float(m.wte[n:].abs().sum()) == 0.0                         # padding rows of the vocabulary stay zero
    buf = []
    assert cli.main(["--model", d, "--backend", "cpu", "--max-tokens", "5", "--temperature", "0", "--prompt", "The quick brown"], out=buf.append) == 0
    assert "Assistant: " in "".join(buf) and "error" not in "".join(buf)


def test_tokenizer_json_byte_level_bpe_matches_the_tokenizers_library(tmp_path):
    """``tokenizer.json`` (the only tokenizer file of Llama 3 / Qwen2 directories): vocabulary, merges, the split pattern,
    ``ignore_merges``, added tokens inside the text and the prepended start marker give the ids of the ``tokenizers``
    library, for the GPT-2 layout and for the Split + ByteLevel layout."""
    tk = pytest.importorskip("tokenizers")
    import json
    from tokenizers import Regex, decoders, models, pre_tokenizers, processors, trainers
    from rustorch_b200.cli.tokenizer import BPETokenizer, load_tokenizer
    corpus = ["The quick brown fox jumps over the lazy dog. " * 3, "Ünïcödé tëxt with 12345 numbers and 日本語 too!",
              "don't you're they'll  spaces   and\nnewlines\n\n", "def f(x):\n    return x + 1  # code"] * 20
    texts = ["Hello world, the fox don't jump 1234567!", "  leading spaces and\n\nnewlines ", "日本語 mixed Ünï",
             "<|begin_of_text|>system<|eot_id|>hi there", ""]
    for style in ("gpt2", "llama3"):
        tok = tk.Tokenizer(models.BPE(ignore_merges=(style == "llama3")))
        if style == "gpt2":
            tok.pre_tokenizer = pre_tokenizers.ByteLevel(add_prefix_space=False, use_regex=True)
        else:
            pat = r"(?i:'s|'t|'re|'ve|'m|'ll|'d)|[^\r\n\p{L}\p{N}]?\p{L}+|\p{N}{1,3}| ?[^\s\p{L}\p{N}]+[\r\n]*|\s*[\r\n]+|\s+(?!\S)|\s+"
            tok.pre_tokenizer = pre_tokenizers.Sequence([pre_tokenizers.Split(Regex(pat), behavior="isolated"),
                                                         pre_tokenizers.ByteLevel(add_prefix_space=False, use_regex=False)])
        tok.decoder = decoders.ByteLevel()
        tok.train_from_iterator(corpus, trainers.BpeTrainer(vocab_size=400, special_tokens=["<|begin_of_text|>", "<|eot_id|>"],
                                                            initial_alphabet=pre_tokenizers.ByteLevel.alphabet()))
        if style == "llama3":
            tok.post_processor = processors.Sequence([processors.ByteLevel(trim_offsets=False), processors.TemplateProcessing(
                single="<|begin_of_text|> $A", special_tokens=[("<|begin_of_text|>", tok.token_to_id("<|begin_of_text|>"))])])
        d = tmp_path / style
        d.mkdir()
        tok.save(str(d / "tokenizer.json"))
        json.dump({"eos_token": {"content": "<|eot_id|>"}}, open(d / "tokenizer_config.json", "w"))
        mine = load_tokenizer(str(d))
        assert isinstance(mine, BPETokenizer) and mine.vocab_size == tok.get_vocab_size() and mine.eos_id == tok.token_to_id("<|eot_id|>")
        assert mine.bos_id == (tok.token_to_id("<|begin_of_text|>") if style == "llama3" else None)
        for t in texts:
            want = tok.encode(t).ids
            got = mine.encode(t)
            assert got == want, (style, t)
            assert mine.decode(got) == tok.decode(want)
        assert mine.decode(mine.encode("a<|eot_id|>b"), skip_special=False).endswith("a<|eot_id|>b")
        assert mine.encode("hi", add_bos=False) == tok.encode("hi", add_special_tokens=False).ids
        # the same tokenizer carried by a GGUF file (tokenizer.ggml.model = gpt2: tokens, merges, token types, pre name)
        from rustorch_b200.formats import gguf
        md = mine.gguf_metadata()
        assert md["tokenizer.ggml.model"] == "gpt2" and md["tokenizer.ggml.pre"] == ("llama-bpe" if style == "llama3" else "gpt-2")
        gp = str(tmp_path / f"{style}.gguf")
        gguf.write_gguf(gp, {"general.architecture": "llama", **md}, {"w": (torch.zeros(4), gguf.GGMLType.F32)})
        with gguf.GGUFFile(gp) as g:
            carried = load_tokenizer(None, g)
            g.metadata.pop("tokenizer.rustorch.pattern")          # a file from another writer: the pattern comes from the pre name
            g.metadata.pop("tokenizer.rustorch.ignore_merges")
            foreign = load_tokenizer(None, g)
            g.metadata["tokenizer.ggml.pre"] = "some-new-model"
            with pytest.raises(ValueError, match="some-new-model"):
                load_tokenizer(None, g)
        for t in texts:
            assert carried.encode(t) == tok.encode(t).ids and carried.decode(carried.encode(t)) == tok.decode(tok.encode(t).ids)
            if "'" not in t:                                       # the two spellings of the contraction rule differ on case only
                assert foreign.encode(t) == tok.encode(t).ids, (style, t)
        assert isinstance(carried, BPETokenizer) and carried.eos_id == mine.eos_id and carried.bos_id == mine.bos_id
    sp = tmp_path / "unigram"
    sp.mkdir()
    json.dump({"model": {"type": "Unigram"}}, open(sp / "tokenizer.json", "w"))
    with pytest.raises(ValueError, match="Unigram"):
        load_tokenizer(str(sp))
    json.dump({"model": {"type": "BPE", "vocab": {}, "merges": []}, "pre_tokenizer": {"type": "Metaspace"}}, open(sp / "tokenizer.json", "w"))
    with pytest.raises(ValueError, match="not byte-level"):
        load_tokenizer(str(sp))


def test_chat_templates_detection_and_turn_end_tokens():
    """Prompt layouts of the model families, chosen from what the model's tokenizer carries; replies end at the family's
    turn-end marker as well as at the tokenizer's eos."""
    from rustorch_b200.cli.engine import InferenceEngine
    from rustorch_b200.cli.session import TURN_END_TOKENS, GenerationConfig, SessionManager, detect_chat_template
    from rustorch_b200.cli.tokenizer import BPETokenizer, GGUFTokenizer
    s = SessionManager()
    s.set_system_prompt("Be brief.")
    s.add_user_message("Hi")
    s.add_assistant_message("Hello!")
    s.add_user_message("Bye")
    assert s.build_prompt() == "Be brief.\nUser: Hi\nAssistant: Hello!\nUser: Bye\nAssistant:"
    s.set_chat_template("llama3")
    assert s.build_prompt() == ("<|start_header_id|>system<|end_header_id|>\n\nBe brief.<|eot_id|><|start_header_id|>user<|end_header_id|>\n\nHi<|eot_id|>"
                                "<|start_header_id|>assistant<|end_header_id|>\n\nHello!<|eot_id|><|start_header_id|>user<|end_header_id|>\n\nBye<|eot_id|>"
                                "<|start_header_id|>assistant<|end_header_id|>\n\n")
    s.set_chat_template("chatml")
    assert s.build_prompt() == ("<|im_start|>system\nBe brief.<|im_end|>\n<|im_start|>user\nHi<|im_end|>\n<|im_start|>assistant\nHello!<|im_end|>\n"
                                "<|im_start|>user\nBye<|im_end|>\n<|im_start|>assistant\n")
    s.set_chat_template("llama2")
    assert s.build_prompt() == "[INST] <<SYS>>\nBe brief.\n<</SYS>>\n\nHi [/INST] Hello! </s><s>[INST] Bye [/INST]"
    with pytest.raises(ValueError, match="not one of"):
        s.set_chat_template("vicuna")
    alphabet = {c: i for i, c in enumerate("abcdefgh ĠĊ")}
    l3 = BPETokenizer(alphabet, [], None, None, {"<|start_header_id|>": 20, "<|end_header_id|>": 21, "<|eot_id|>": 22})
    cm = BPETokenizer(alphabet, [], None, None, {"<|im_start|>": 20, "<|im_end|>": 21})
    assert detect_chat_template(l3) == "llama3" and detect_chat_template(cm) == "chatml" and detect_chat_template(BPETokenizer(alphabet, [])) == "plain"
    assert detect_chat_template(None, {"tokenizer.chat_template": "{% for m in messages %}[INST] {{ m }} [/INST]{% endfor %}"}) == "llama2"
    assert detect_chat_template(None, {"tokenizer.chat_template": "...<|im_start|>..."}) == "chatml"
    # control tokens written out in a prompt become their ids in the SentencePiece-style GGUF tokenizer too
    gt = GGUFTokenizer(["<unk>", "<s>", "</s>", "▁a", "▁b", "a", "b", "▁"], [0, 0, 0, -1, -2, -3, -4, -5], [2, 3, 3, 1, 1, 1, 1, 1])
    assert gt.encode("a </s><s>b", add_bos=True) == [1, 3, 7, 2, 1, 4] and gt.encode("a b", add_bos=False) == [3, 4]

    class OneShot:                                   # a runtime that always proposes the same next token
        class cfg:
            vocab_size, context_length = 32, 64

        def __init__(self, tok):
            self.tok = tok

        def new_cache(self, b, n):
            return None

        def prefill(self, prompts, cache):
            out = torch.full((1, 32), -1e4)
            out[0, self.tok] = 0.0
            return out
        decode_step = prefill
    eng = InferenceEngine(OneShot(22), l3, GenerationConfig(max_tokens=6, temperature=0.0), "cpu")
    eng.generate("ab")
    assert eng.last_token_count == 6                 # nothing says that 22 ends a turn
    eng.set_stop_tokens(TURN_END_TOKENS["llama3"])
    eng.generate("ab")
    assert eng.stop_ids == {22} and eng.last_token_count == 0


def test_template_command_switches_the_prompt_layout():
    from rustorch_b200.cli.engine import InferenceEngine
    from rustorch_b200.cli.repl import Repl
    from rustorch_b200.cli.session import SessionManager
    out = []
    repl = Repl(SessionManager(), InferenceEngine(), out=out.append, stream=False)
    repl.apply_chat_template("chatml")                       # what a loaded model pointed to
    repl.handle_line("/template")
    assert out[-1] == "chat template: chatml (auto)\n"
    repl.handle_line("/template llama3")
    assert out[-1] == "chat template: llama3\n" and repl.session.build_prompt().endswith("<|start_header_id|>assistant<|end_header_id|>\n\n")
    repl.handle_line("/template vicuna")
    assert out[-1].startswith("error:") and repl.session.chat_template == "llama3"
    repl.handle_line("/template auto")
    assert out[-1] == "chat template: chatml (auto)\n"
    repl.handle_line("/help")
    assert "/template" in out[-1]
