"""CPU tests: model import (incl. an ONNX file built by hand), convert, model hub, JIT."""
import io
import os
import struct

import numpy as np
import pytest
import torch
import torch.nn as nn

from rustorch_b200 import convert as C, jit as J, model_hub as H, model_import as MI
from rustorch_b200.formats import save_safetensors
from rustorch_b200.tensorboard import _f_bytes, _f_float, _f_varint


# -- a tiny ONNX writer for the test (the framework itself only reads ONNX)
def _tensor(name, arr):
    b = b"".join(_f_varint(1, d) for d in arr.shape) + _f_varint(2, 1) + _f_bytes(8, name.encode()) + _f_bytes(9, arr.astype("<f4").tobytes())
    return b


def _node(op, ins, outs, attrs=()):
    b = b"".join(_f_bytes(1, i.encode()) for i in ins) + b"".join(_f_bytes(2, o.encode()) for o in outs) + _f_bytes(4, op.encode())
    for k, v in attrs:
        a = _f_bytes(1, k.encode()) + (_f_varint(3, v) + _f_varint(20, 2) if isinstance(v, int) else _f_float(2, v) + _f_varint(20, 1))
        b += _f_bytes(5, a)
    return b


def _onnx_mlp(w1, b1, w2, b2):
    g = (_f_bytes(1, _node("Gemm", ["x", "w1", "b1"], ["h"], [("transB", 1), ("alpha", 1.0)])) + _f_bytes(1, _node("Relu", ["h"], ["r"]))
         + _f_bytes(1, _node("Gemm", ["r", "w2", "b2"], ["y"], [("transB", 1)])) + _f_bytes(2, b"mlp")
         + _f_bytes(5, _tensor("w1", w1)) + _f_bytes(5, _tensor("b1", b1)) + _f_bytes(5, _tensor("w2", w2)) + _f_bytes(5, _tensor("b2", b2))
         + _f_bytes(11, _f_bytes(1, b"x")) + _f_bytes(11, _f_bytes(1, b"w1")) + _f_bytes(12, _f_bytes(1, b"y")))
    return _f_varint(1, 8) + _f_bytes(2, b"test-writer") + _f_bytes(7, g)


def test_onnx_import_and_execution(tmp_path):
    rng = np.random.default_rng(0)
    w1, b1, w2, b2 = rng.normal(size=(6, 4)), rng.normal(size=6), rng.normal(size=(3, 6)), rng.normal(size=3)
    p = tmp_path / "m.onnx"
    p.write_bytes(_onnx_mlp(w1, b1, w2, b2))
    m = MI.import_model(str(p))
    assert m.metadata.format is MI.ModelFormat.ONNX and m.metadata.producer == "test-writer" and [l.layer_type for l in m.layers] == ["Gemm", "Relu", "Gemm"]
    assert [i.name for i in m.architecture.inputs] == ["x"] and m.architecture.parameter_count == 24 + 6 + 18 + 3
    mod = MI.ModelImporter().to_module(m)
    x = torch.randn(5, 4)
    ref = torch.relu(x @ torch.tensor(w1, dtype=torch.float32).t() + torch.tensor(b1, dtype=torch.float32)) @ torch.tensor(w2, dtype=torch.float32).t() + torch.tensor(b2, dtype=torch.float32)
    assert torch.allclose(mod(x), ref, atol=1e-5)


def test_format_tables_and_detection(tmp_path):
    F = MI.ModelFormat
    assert F.from_extension(".pth") is F.PYTORCH and F.from_extension("gguf") is F.GGUF and F.from_extension("xyz") is None
    assert F.GGUF.supports_feature(MI.FormatFeature.QUANTIZATION) and not F.ONNX.supports_feature(MI.FormatFeature.OPTIMIZER_STATE)
    fc = MI.FormatCompatibility()
    assert fc.get_compatibility(F.PYTORCH, F.SAFETENSORS) == 1.0 and fc.get_conversion_path(F.ONNX, F.GGUF) == [F.ONNX, F.SAFETENSORS, F.GGUF]
    assert fc.get_conversion_path(F.TENSORFLOW, F.GGUF) == []
    assert MI.FormatValidator.validate_format(b"GGUF\x03\x00\x00\x00", F.GGUF) and not MI.FormatValidator.validate_format(b"GGUF", F.ONNX)
    assert MI.OptimizationProfile.edge().quantize == "int4"
    sd = {"fc1.weight": torch.randn(8, 4), "fc1.bias": torch.randn(8), "fc2.weight": torch.randn(2, 8), "fc2.bias": torch.randn(2)}
    save_safetensors(sd, str(tmp_path / "m.safetensors"))
    m = MI.import_model(str(tmp_path / "m.safetensors"))
    assert m.metadata.format is F.SAFETENSORS and [l.layer_type for l in m.layers] == ["Linear", "Linear"]
    mod = MI.ModelImporter().to_module(m)
    x = torch.randn(3, 4)
    assert torch.allclose(mod(x), torch.relu(x @ sd["fc1.weight"].t() + sd["fc1.bias"]) @ sd["fc2.weight"].t() + sd["fc2.bias"], atol=1e-5)
    pre = MI.ModelImporter().with_cache_dir(str(tmp_path)).import_pretrained("resnet18")
    assert pre.architecture.parameter_count > 11_000_000 and pre.metadata.extra["pretrained"] is False
    with pytest.raises(KeyError):
        MI.import_pretrained("nope")


def test_convert_parser_simulation_and_architectures():
    cnn = nn.Sequential(nn.Conv2d(3, 8, 3), nn.BatchNorm2d(8), nn.ReLU(), nn.Conv2d(8, 4, 3), nn.Flatten(), nn.Linear(4 * 4 * 4, 10))
    model = C.SimplePyTorchConverter.convert(cnn.state_dict())
    assert [model.layers[n].layer_type for n in model.layer_names()] == ["Conv2d", "BatchNorm", "Conv2d", "Linear"]
    assert model.simulate_forward([2, 3, 8, 8]) == [2, 10] and model.total_parameters == sum(p.numel() for p in cnn.parameters())
    with pytest.raises(C.SimpleConversionError):
        model.simulate_forward([2, 5, 8, 8])
    rebuilt = model.to_module().eval()
    x = torch.randn(2, 3, 8, 8)
    ref = nn.Sequential(cnn[0], cnn[1], nn.ReLU(), cnn[3], nn.ReLU(), cnn[4], cnn[5]).eval()
    assert torch.allclose(rebuilt(x), ref(x), atol=1e-5)
    res = C.ModelValidator.comprehensive_validation(rebuilt, ref, x, 1e-4)
    assert res.accuracy.passed and "PASS" in C.ModelValidator.generate_report(res)
    assert convert_ok(model)
    sd = {"transformer.wte.weight": torch.zeros(64, 32), "transformer.wpe.weight": torch.zeros(16, 32)}
    for i in range(2):
        h = f"transformer.h.{i}."
        sd.update({h + "ln_1.weight": torch.ones(32), h + "ln_1.bias": torch.zeros(32), h + "attn.c_attn.weight": torch.zeros(96, 32),
                   h + "attn.c_attn.bias": torch.zeros(96), h + "attn.c_proj.weight": torch.zeros(32, 32), h + "attn.c_proj.bias": torch.zeros(32),
                   h + "mlp.c_fc.weight": torch.zeros(128, 32), h + "mlp.c_fc.bias": torch.zeros(128),
                   h + "mlp.c_proj.weight": torch.zeros(32, 128), h + "mlp.c_proj.bias": torch.zeros(32)})
    tc = C.ComplexArchitectureParser.parse_transformer(sd)
    assert tc.num_layers == 2 and len(tc.attention) == 2 and tc.feed_forward[0].d_ff == 128 and tc.token_embedding == (64, 32) and tc.position_embedding == (16, 32)
    cc = C.ComplexArchitectureParser.parse_cnn(cnn.state_dict())
    assert len(cc.conv_layers) == 2 and cc.classifier[2] == 10
    with pytest.raises(C.SimpleConversionError):
        C.SimplePyTorchConverter.convert({})


def convert_ok(model):
    r = C.convert_to_integrated_model(model)
    return r.total_parameters() == model.total_parameters and r.simulate_forward([1, 3, 8, 8]) == [1, 10] and "Conv2d" in r.summary()


def test_model_hub_cache_lru_download_retry_verify(tmp_path):
    blob = os.urandom(3000)
    calls = {"n": 0}

    def opener(url, offset):
        calls["n"] += 1
        data = blob[offset:]
        if calls["n"] == 1:
            data = data[:1000]                    # connection drops after 1000 bytes: the retry resumes
        return io.BytesIO(data), len(blob)
    dl = H.ModelDownloader(max_retries=3, opener=opener)
    seen = []
    dest = dl.download("http://x/model.bin", str(tmp_path / "dl" / "model.bin"), seen.append)
    assert open(dest, "rb").read() == blob and calls["n"] == 2 and seen[-1].percentage() == 100.0 and "MB" in seen[-1].format_size()
    with pytest.raises(H.DownloadError):
        H.ModelDownloader(max_retries=2, opener=lambda u, o: (_ for _ in ()).throw(IOError("offline"))).download("http://x", str(tmp_path / "f"))
    import hashlib
    assert H.ModelVerifier.verify(dest, hashlib.sha256(blob).hexdigest()) and not H.ModelVerifier.verify(dest, "00")
    assert len(H.ModelVerifier.checksum(dest, "crc32")) == 8 and len(H.ModelVerifier.checksum(dest, "md5")) == 32
    cache = H.ModelCache(str(tmp_path / "cache"), H.CacheConfig(max_size_bytes=7000, max_entries=10))
    for i, name in enumerate(["a", "b", "c"]):
        cache.cache_model(name, dest, now=float(i))
    assert cache.list_cached_models() == ["b", "c"] and cache.stats() == (2, 6000)          # 'a' was least recently used
    assert cache.get_model_path("b") and H.ModelCache(str(tmp_path / "cache")).list_cached_models() == ["b", "c"]
    assert cache.remove_model("b") and not cache.remove_model("b")
    hub = H.ModelHub(str(tmp_path / "hub"), H.ModelDownloader(opener=lambda u, o: (io.BytesIO(blob[o:]), len(blob))))
    assert "gpt2" in hub.list_models() and hub.registry.search("bert")[0].architecture == "bert" and hub.registry.search(tag="vision")
    hub.registry.register_model(H.ModelInfo("toy", "http://x/toy.bin", "mlp", sha256=hashlib.sha256(blob).hexdigest(), file_format="bin"))
    p1 = hub.download_model("toy")
    assert hub.download_model("toy") == p1
    hub.registry.register_model(H.ModelInfo("bad", "http://x/bad.bin", "mlp", sha256="ff", file_format="bin"))
    with pytest.raises(H.DownloadError):
        hub.download_model("bad")


def test_jit_trace_script_optimize_save(tmp_path):
    torch.manual_seed(0)
    net = nn.Sequential(nn.Conv2d(1, 4, 3, padding=1), nn.BatchNorm2d(4), nn.ReLU(), nn.Dropout(0.5), nn.Identity(), nn.Sigmoid(),
                        nn.AdaptiveAvgPool2d(2), nn.Flatten(), nn.Linear(16, 3)).eval()
    x = torch.randn(2, 1, 6, 6)
    sm = J.trace(net, x)
    assert [n.op_type for n in sm.graph.nodes][:4] == ["Input", "Conv2d", "BatchNorm2d", "ReLU"] and torch.allclose(sm(x), net(x), atol=1e-6)
    sm.eval()
    stats = J.optimize_graph(sm)
    assert stats["identities_removed"] == 2 and stats["dead_removed"] == 2 and stats["fusible_chains"] == 1
    assert torch.allclose(sm(x), net(x), atol=1e-6) and "fused into" in sm.code()
    sm.save(str(tmp_path / "m.jit"))
    back = J.ScriptModule.load(str(tmp_path / "m.jit")).eval()
    assert torch.allclose(back(x), net(x), atol=1e-6)
    s2 = J.script(nn.Sequential(nn.Linear(4, 4), nn.Tanh()))
    assert len(s2.graph.nodes) == 3

    class Res(nn.Module):
        def __init__(self):
            super().__init__()
            self.a, self.act = nn.Linear(4, 4), nn.ReLU()

        def forward(self, t):
            return self.act(self.a(t)) + t
    with pytest.raises(RuntimeError):
        J.trace(Res(), torch.randn(2, 4))                 # functional add at the output is reported, not mis-traced
    cache = J.JitCache()
    m = nn.Sequential(nn.Linear(4, 2))
    a = cache.get_or_trace(m, torch.randn(1, 4))
    assert cache.get_or_trace(m, torch.randn(1, 4)) is a and (cache.hits, cache.misses) == (1, 1)
    assert cache.get_or_trace(m, torch.randn(3, 4)) is not a
