"""File formats: RUSTORCH container (byte layout + CRC-64), safetensors, PYTORCH1, JSON, HF dir, GGUF + Q4_0/Q8_0."""
import json
import os
import struct

import numpy as np
import pytest
import torch

from rustorch_b200.formats import gguf, rustorch_bin as rb
from rustorch_b200 import formats as F
from rustorch_b200.tensor import Tensor


def test_crc64_known_vector_and_native_agree():
    assert rb.crc64(b"123456789") == 0x995DC9BBDF1939FA        # CRC-64/XZ check value
    d = os.urandom(4099)
    assert rb.crc64(d) == rb.crc64_fast(d)


def test_tensor_container_byte_layout(tmp_path):
    p = str(tmp_path / "t.rustorch")
    t = torch.arange(6, dtype=torch.float32).reshape(2, 3)
    rb.save_tensor(t, p)
    raw = open(p, "rb").read()
    assert raw[:8] == b"RUSTORCH"
    (hlen,) = struct.unpack_from("<Q", raw, 8)
    header = raw[16:16 + hlen]
    assert header[:8] == b"RUSTORCH"                                             # bincode [u8; 8]: raw bytes
    assert struct.unpack_from("<Q", header, 8)[0] == 5 and header[16:21] == b"1.0.0"  # String: u64 len + bytes
    assert struct.unpack_from("<Q", header, 21)[0] == 6 and header[29:35] == b"tensor"
    payload = raw[16 + hlen:]
    assert struct.unpack_from("<I", payload, 0)[0] == 2                          # ndim
    assert struct.unpack_from("<QQ", payload, 4) == (2, 3)                       # dims
    assert struct.unpack_from("<Q", payload, 20)[0] == 24                        # byte length
    assert np.frombuffer(payload, "<f4", 6, 28).tolist() == [0, 1, 2, 3, 4, 5]
    assert struct.unpack_from("<Q", header, hlen - 8)[0] == rb.crc64(payload)    # checksum is the last field
    assert torch.equal(rb.load_tensor(p), t)
    assert torch.equal(Tensor.load(p).data, t)


def test_corruption_type_and_version_checks(tmp_path):
    p = str(tmp_path / "t.bin")
    rb.save_tensor(torch.ones(4), p)
    raw = bytearray(open(p, "rb").read())
    raw[-1] ^= 0xFF
    open(p, "wb").write(raw)
    with pytest.raises(IOError, match="Checksum"):
        rb.load_tensor(p)
    rb.save_tensor(torch.ones(4), p)
    with pytest.raises(TypeError):
        rb.load_state_dict(p)
    open(p, "wb").write(b"NOTRUSTO" + b"\0" * 32)
    with pytest.raises(ValueError):
        rb.read_container(p)


def test_state_dict_and_checkpoint_roundtrip(tmp_path):
    m = torch.nn.Sequential(torch.nn.Linear(4, 3), torch.nn.BatchNorm1d(3))
    p = str(tmp_path / "m.rustorch")
    rb.save_module(m, p, config={"hidden": 3})
    params, buffers, meta = rb.load_state_dict(p)
    assert set(params) == {"0.weight", "0.bias", "1.weight", "1.bias"} and "1.running_mean" in buffers
    assert meta["parameters"]["0.weight"]["shape"] == [3, 4] and meta["config"]["hidden"] == "3"
    m2 = torch.nn.Sequential(torch.nn.Linear(4, 3), torch.nn.BatchNorm1d(3))
    rb.load_module(m2, p)
    assert torch.equal(m2[0].weight, m[0].weight)
    c = str(tmp_path / "ck.rustorch")
    mom = rb.encode_tensor(torch.full((3, 4), 0.5))
    rb.save_checkpoint(c, 3, 1200, params, buffers, {"0.weight.exp_avg": mom, "hyper": json.dumps({"lr": 0.1}).encode()},
                       {"last_epoch": b"3"}, {"loss": 0.25, "acc": 0.9}, timestamp=42)
    ck = rb.load_checkpoint(c)
    assert (ck["epoch"], ck["step"], ck["timestamp"]) == (3, 1200, 42) and ck["metrics"] == {"loss": 0.25, "acc": 0.9}
    assert torch.equal(rb.decode_tensor(ck["optimizer_state"]["0.weight.exp_avg"])[0], torch.full((3, 4), 0.5))
    assert torch.equal(ck["parameters"]["0.weight"], m[0].weight.detach())
    v = torch.ones(3, requires_grad=True)
    v.grad = torch.full((3,), 2.0)
    rb.save_variable(v, str(tmp_path / "v.bin"))
    v2 = rb.load_variable(str(tmp_path / "v.bin"))
    assert v2.requires_grad and torch.equal(v2.grad, v.grad)
    d = torch.ones(2, dtype=torch.float64)
    rb.save_tensor(d, str(tmp_path / "d.bin"))
    assert rb.load_tensor(str(tmp_path / "d.bin")).dtype == torch.float64


def test_safetensors_spec_and_reference_style(tmp_path):
    p = str(tmp_path / "m.safetensors")
    ts = {"a": torch.randn(3, 4), "b": torch.randn(5).to(torch.bfloat16), "c": torch.arange(4)}
    F.save_safetensors(ts, p, {"format": "pt"})
    raw = open(p, "rb").read()
    (n,) = struct.unpack_from("<Q", raw, 0)
    assert n % 8 == 0 and json.loads(raw[8:8 + n])["a"]["dtype"] == "F32"
    back = F.load_safetensors(p)
    assert all(torch.equal(back[k], ts[k]) for k in ts) and back["b"].dtype == torch.bfloat16
    # a file as the reference writes it: unpadded header, F64 entry, no metadata
    hdr = json.dumps({"w": {"dtype": "F64", "shape": [2], "data_offsets": [0, 16]}}).encode()
    q = str(tmp_path / "ref.safetensors")
    open(q, "wb").write(struct.pack("<Q", len(hdr)) + hdr + np.array([1.5, -2.0], "<f8").tobytes())
    assert F.load_safetensors(q)["w"].tolist() == [1.5, -2.0]
    assert F.detect_format(p) == "safetensors"


def test_pth_json_and_hf_dir(tmp_path):
    ts = {"layer.weight": torch.randn(2, 3), "layer.bias": torch.zeros(2)}
    p = str(tmp_path / "m.pth")
    F.save_pth(ts, p)
    assert open(p, "rb").read(8) == b"PYTORCH1" and torch.equal(F.load_pth(p)["layer.weight"], ts["layer.weight"])
    tp = str(tmp_path / "real.pt")
    F.save_torch_state_dict(ts, tp)
    assert torch.equal(F.load_pth(tp)["layer.bias"], ts["layer.bias"]) and F.detect_format(tp) == "torch"
    j = str(tmp_path / "m.json")
    F.save_json_state_dict(ts, j, {"arch": "mlp"})
    back, meta = F.load_json_state_dict(j)
    assert torch.allclose(back["layer.weight"], ts["layer.weight"]) and meta["arch"] == "mlp"
    d = str(tmp_path / "hf")
    F.save_huggingface(ts, d, {"hidden_size": 3})
    b2, cfg = F.load_huggingface(d)
    assert cfg["hidden_size"] == 3 and torch.equal(b2["layer.bias"], ts["layer.bias"]) and F.detect_format(d) == "huggingface"


def test_q4_0_q8_0_codecs():
    rng = np.random.default_rng(0)
    x = rng.normal(0, 0.02, (8, 64)).astype(np.float32)
    q4 = gguf.quantize_q4_0(x)
    assert q4.shape == (8, 2, 18) and q4.dtype == np.uint8
    y = gguf.dequantize_q4_0(q4)
    blk = x.reshape(8, 2, 32)
    assert np.abs(y - x).max() <= np.abs(blk).max() / 8 * 1.01 + 1e-6          # one step: the code range -8..7 clips the far side
    # the element of largest magnitude maps to code 0 (value -8 * d) exactly up to f16 rounding of d
    i = np.abs(blk[0, 0]).argmax()
    assert abs(y.reshape(8, 2, 32)[0, 0, i] - blk[0, 0, i]) < abs(blk[0, 0, i]) * 2e-3
    # manual decode of one block following the layout
    b0 = q4[0, 0]
    d = b0[:2].copy().view(np.float16).astype(np.float32)[0]
    assert np.allclose(((b0[2:] & 0xF).astype(np.int32) - 8) * d, y[0, :16]) and np.allclose(((b0[2:] >> 4).astype(np.int32) - 8) * d, y[0, 16:32])
    q8 = gguf.quantize_q8_0(x)
    assert q8.shape == (8, 2, 34) and np.abs(gguf.dequantize_q8_0(q8) - x).max() <= np.abs(x).max() / 127 * 0.51 + 1e-6
    assert np.all(gguf.dequantize_q4_0(gguf.quantize_q4_0(np.zeros((1, 32), np.float32))) == 0)


def test_gguf_write_read_roundtrip(tmp_path):
    p = str(tmp_path / "m.gguf")
    w = torch.randn(16, 64) * 0.02
    emb = torch.randn(10, 64)
    md = {"general.architecture": "llama", "llama.block_count": 2, "llama.embedding_length": 64,
          "llama.attention.head_count": 4, "llama.rope.freq_base": 10000.0, "tokenizer.ggml.tokens": ["a", "b", "c"],
          "general.name": "tiny"}
    gguf.write_gguf(p, md, {"blk.0.attn_q.weight": (w, gguf.GGMLType.Q4_0), "token_embd.weight": (emb, gguf.GGMLType.F16),
                            "blk.0.ffn_up.weight": (w, gguf.GGMLType.Q8_0), "output_norm.weight": (torch.ones(64), gguf.GGMLType.F32)})
    raw = open(p, "rb").read()
    assert struct.unpack_from("<II", raw, 0) == (0x46554747, 3)
    with gguf.GGUFFile(p) as g:
        assert g.metadata["general.name"] == "tiny" and g.metadata["tokenizer.ggml.tokens"] == ["a", "b", "c"]
        assert g.data_start % 32 == 0
        info = g.tensors["blk.0.attn_q.weight"]
        assert info.dims == (64, 16) and info.shape == (16, 64) and info.nbytes == 16 * 2 * 18
        ref = torch.from_numpy(gguf.dequantize_q4_0(gguf.quantize_q4_0(w.numpy())))
        assert torch.equal(g.load_tensor("blk.0.attn_q.weight"), ref)
        assert torch.allclose(g.load_tensor("token_embd.weight"), emb, atol=2e-3)
        assert torch.equal(g.load_tensor("output_norm.weight"), torch.ones(64))
        blocks, _ = g.load_quantized("blk.0.ffn_up.weight")
        assert blocks.shape == (16, 2, 34)
        cfg = g.model_config()
        assert cfg["n_layer"] == 2 and cfg["n_head_kv"] == 4 and cfg["vocab_size"] == 3
    assert F.detect_format(p) == "gguf"


def test_mlx_loader_roundtrip_metadata_and_errors(tmp_path):
    """MLX weight files (example-cli/src/model/formats/mlx.rs:12-144): 8-byte header length, JSON header, raw data."""
    import json
    import struct
    from rustorch_b200.error import ModelFormatError
    from rustorch_b200.formats import detect_format
    from rustorch_b200.formats.mlx import MLXLoader, extract_metadata, parse_tensor, save_mlx
    # the reference's own unit vectors: [1.0, 2.0, 3.0] as little-endian f32, and Llama-7B defaults for empty metadata
    t = parse_tensor(bytes([0, 0, 128, 63, 0, 0, 0, 64, 0, 0, 64, 64]), [3], "F32")
    assert t.tolist() == [1.0, 2.0, 3.0]
    md = extract_metadata({})
    assert (md.vocab_size, md.hidden_size, md.num_layers, md.num_heads, md.context_length) == (32000, 4096, 32, 32, 2048)
    tensors = {"a.weight": torch.randn(3, 5), "b": torch.arange(6, dtype=torch.int64).reshape(2, 3),
               "h": torch.randn(4).half(), "i": torch.tensor([1, -2], dtype=torch.int32), "bf": torch.randn(2, 2).bfloat16()}
    path = str(tmp_path / "model.mlx")
    save_mlx(path, tensors, {"vocab_size": 1234, "hidden_size": "64", "num_hidden_layers": 2})
    assert detect_format(path) == "mlx"
    got, md = MLXLoader.load(path)
    assert set(got) == set(tensors)
    for k, v in tensors.items():
        assert got[k].dtype == v.dtype and torch.equal(got[k], v), k
    assert (md.vocab_size, md.hidden_size, md.num_layers, md.num_heads, md.format) == (1234, 64, 2, 32, "mlx")
    # hand-built file with the long dtype spelling the reference accepts
    hdr = json.dumps({"w": {"dtype": "float32", "shape": [2], "data_offsets": [0, 8]}}).encode()
    p2 = str(tmp_path / "hand.mlx")
    with open(p2, "wb") as f:
        f.write(struct.pack("<Q", len(hdr)) + hdr + struct.pack("<2f", 0.5, -1.5))
    assert MLXLoader.load(p2)[0]["w"].tolist() == [0.5, -1.5]
    # corrupt: header longer than the file; unknown dtype; offsets outside the data
    p3 = str(tmp_path / "bad.mlx")
    with open(p3, "wb") as f:
        f.write(struct.pack("<Q", 1 << 20) + b"{}")
    with pytest.raises(ModelFormatError):
        MLXLoader.load(p3)
    with pytest.raises(ModelFormatError):
        parse_tensor(b"\0" * 4, [1], "C64")
    hdr = json.dumps({"w": {"dtype": "F32", "shape": [4], "data_offsets": [0, 16]}}).encode()
    with open(p3, "wb") as f:
        f.write(struct.pack("<Q", len(hdr)) + hdr + b"\0" * 8)
    with pytest.raises(ModelFormatError):
        MLXLoader.load(p3)
    # the generic state-dict reader goes through the same loader
    from rustorch_b200.models.high_level import load_state_dict_file
    assert torch.equal(load_state_dict_file(path)["a.weight"], tensors["a.weight"])


# ------------------------------------------------------------------ the other GGML block types
def _rand_blocks(rng, nb, nbytes, f16_cols=(), f32_cols=()):
    b = rng.integers(0, 256, (nb, nbytes), dtype=np.uint8)
    for c in f16_cols:
        b[:, c:c + 2] = (rng.standard_normal(nb) * 0.1).astype(np.float16).view(np.uint8).reshape(nb, 2)
    for c in f32_cols:
        b[:, c:c + 4] = (rng.standard_normal(nb) * 0.1).astype(np.float32).view(np.uint8).reshape(nb, 4)
    return b


_BLOCK_CASES = {"Q4_1": (20, (0, 2)), "Q5_0": (22, (0,)), "Q5_1": (24, (0, 2)), "Q2_K": (84, (80, 82)), "Q3_K": (110, (108,)),
                "Q4_K": (144, (0, 2)), "Q5_K": (176, (0, 2)), "Q6_K": (210, (208,))}


@pytest.mark.parametrize("name", sorted(_BLOCK_CASES))
def test_block_decoders_match_the_gguf_package(name):
    """Random block bytes (finite scales) decode to the same floats as the ``gguf`` package's reference decoders."""
    ref_pkg = pytest.importorskip("gguf")
    from gguf import quants
    from rustorch_b200.formats import gguf as ours
    nbytes, cols = _BLOCK_CASES[name]
    b = _rand_blocks(np.random.default_rng(1), 96, nbytes, cols)
    want = quants.dequantize(b, getattr(ref_pkg.GGMLQuantizationType, name))
    got = ours.dequantize(b.reshape(-1), getattr(ours.GGMLType, name), want.shape)
    assert got.dtype == np.float32 and np.array_equal(got, want)


def test_block_decoders_against_scalar_loops():
    """Q4_K, Q6_K, Q8_1 and Q8_K written out weight by weight from the format's definition (no package needed)."""
    from rustorch_b200.formats import gguf as ours
    rng = np.random.default_rng(2)
    h = lambda two: float(np.frombuffer(bytes(two), dtype=np.float16)[0])      # noqa: E731
    # Q4_K: d, dmin, 12 scale bytes, 128 code bytes; chunk c of 64 weights = low nibbles then high nibbles of 32 bytes
    b = _rand_blocks(rng, 3, 144, (0, 2))
    want = np.zeros((3, 256), dtype=np.float32)
    for n in range(3):
        d, dmin, sc, qs = h(b[n, 0:2]), h(b[n, 2:4]), b[n, 4:16].astype(int), b[n, 16:144].astype(int)

        def scale_min(j):
            if j < 4:
                return sc[j] & 63, sc[j + 4] & 63
            return (sc[j + 4] & 0xF) | ((sc[j - 4] >> 6) << 4), (sc[j + 4] >> 4) | ((sc[j] >> 6) << 4)
        for c in range(4):
            (s1, m1), (s2, m2) = scale_min(2 * c), scale_min(2 * c + 1)
            for l in range(32):
                want[n, c * 64 + l] = np.float32(d) * np.float32(s1) * np.float32(qs[c * 32 + l] & 0xF) - np.float32(dmin) * np.float32(m1)
                want[n, c * 64 + 32 + l] = np.float32(d) * np.float32(s2) * np.float32(qs[c * 32 + l] >> 4) - np.float32(dmin) * np.float32(m2)
    assert np.allclose(ours.dequantize(b.reshape(-1), ours.GGMLType.Q4_K, (3, 256)), want, rtol=1e-6, atol=1e-6)
    # Q6_K: 128 low-nibble bytes, 64 bytes of 2-bit highs, 16 int8 scales, d
    b = _rand_blocks(rng, 2, 210, (208,))
    want = np.zeros((2, 256), dtype=np.float32)
    for n in range(2):
        ql, qh, sc, d = b[n, 0:128].astype(int), b[n, 128:192].astype(int), b[n, 192:208].view(np.int8).astype(int), h(b[n, 208:210])
        for half in range(2):
            for l in range(32):
                i = l // 16
                qv = [(ql[half * 64 + l] & 0xF) | (((qh[half * 32 + l] >> 0) & 3) << 4), (ql[half * 64 + l + 32] & 0xF) | (((qh[half * 32 + l] >> 2) & 3) << 4),
                      (ql[half * 64 + l] >> 4) | (((qh[half * 32 + l] >> 4) & 3) << 4), (ql[half * 64 + l + 32] >> 4) | (((qh[half * 32 + l] >> 6) & 3) << 4)]
                for k in range(4):
                    want[n, half * 128 + k * 32 + l] = np.float32(d) * np.float32(sc[half * 8 + i + 2 * k]) * np.float32(qv[k] - 32)
    assert np.allclose(ours.dequantize(b.reshape(-1), ours.GGMLType.Q6_K, (2, 256)), want, rtol=1e-6, atol=1e-6)
    b = _rand_blocks(rng, 4, 36, (0, 2))
    want = b[:, 4:36].copy().view(np.int8).astype(np.float32) * b[:, 0:2].copy().view(np.float16).astype(np.float32)
    assert np.array_equal(ours.dequantize(b.reshape(-1), ours.GGMLType.Q8_1, (4, 32)), want)
    b = _rand_blocks(rng, 2, 292, (), (0,))
    want = b[:, 4:260].copy().view(np.int8).astype(np.float32) * b[:, 0:4].copy().view(np.float32)
    assert np.array_equal(ours.dequantize(b.reshape(-1), ours.GGMLType.Q8_K, (2, 256)), want)
    with pytest.raises(ValueError):
        ours.RawTensor((2, 256), b"x" * 10).check(ours.GGMLType.Q4_K)


def test_runtime_loads_a_k_quant_file(tmp_path):
    """A Llama GGUF whose linears are Q4_K / Q6_K / Q5_0 blocks: tensor sizes and offsets follow the 256-weight block
    sizes, the runtime expands and re-encodes the linears, and its logits equal those of a runtime built from the same
    weights stored as F32."""
    from rustorch_b200 import llm
    from rustorch_b200.formats import gguf as ours
    rng = np.random.default_rng(3)
    d_model, n_ff, vocab, hd = 256, 512, 64, 64

    def blocks(ty, out_f, in_f):
        nbytes, cols = _BLOCK_CASES[ty]
        b = _rand_blocks(rng, out_f * in_f // ours._BLOCK[getattr(ours.GGMLType, ty)][0], nbytes, cols)
        for c in cols:                                                # small block scales: weights of order 0.01 - 0.1
            b[:, c:c + 2] = (rng.standard_normal(len(b)) * (0.002 if ty == "Q5_0" else 4e-5)).astype(np.float16).view(np.uint8).reshape(len(b), 2)
        return ours.RawTensor((out_f, in_f), b.tobytes())
    quant = {"token_embd.weight": (torch.randn(vocab, d_model) * 0.05, ours.GGMLType.F16), "output_norm.weight": (torch.ones(d_model), ours.GGMLType.F32),
             "output.weight": (blocks("Q6_K", vocab, d_model), ours.GGMLType.Q6_K)}
    p = "blk.0."
    quant.update({p + "attn_q.weight": (blocks("Q4_K", 4 * hd, d_model), ours.GGMLType.Q4_K), p + "attn_k.weight": (blocks("Q4_K", 2 * hd, d_model), ours.GGMLType.Q4_K),
                  p + "attn_v.weight": (blocks("Q6_K", 2 * hd, d_model), ours.GGMLType.Q6_K), p + "attn_output.weight": (blocks("Q5_0", d_model, 4 * hd), ours.GGMLType.Q5_0),
                  p + "ffn_gate.weight": (blocks("Q4_K", n_ff, d_model), ours.GGMLType.Q4_K), p + "ffn_up.weight": (blocks("Q4_K", n_ff, d_model), ours.GGMLType.Q4_K),
                  p + "ffn_down.weight": (blocks("Q6_K", d_model, n_ff), ours.GGMLType.Q6_K), p + "attn_norm.weight": (torch.ones(d_model), ours.GGMLType.F32),
                  p + "ffn_norm.weight": (torch.ones(d_model), ours.GGMLType.F32)})
    md = {"general.architecture": "llama", "llama.block_count": 1, "llama.embedding_length": d_model, "llama.feed_forward_length": n_ff,
          "llama.attention.head_count": 4, "llama.attention.head_count_kv": 2, "llama.rope.freq_base": 10000.0,
          "llama.attention.layer_norm_rms_epsilon": 1e-5, "llama.context_length": 64, "llama.vocab_size": vocab}
    qpath, fpath = str(tmp_path / "k.gguf"), str(tmp_path / "f32.gguf")
    ours.write_gguf(qpath, md, quant)
    with ours.GGUFFile(qpath) as g:
        assert g.tensors[p + "attn_q.weight"].ggml_type == ours.GGMLType.Q4_K and g.tensors[p + "attn_q.weight"].nbytes == 4 * hd * d_model // 256 * 144
        dense = {k: (g.load_tensor(k), ours.GGMLType.F32 if k.endswith("weight") and "norm" not in k and "token_embd" not in k else quant[k][1])
                 for k in quant}
        w = dense[p + "ffn_down.weight"][0]
        assert w.shape == (d_model, n_ff) and torch.isfinite(w).all() and 0.001 < float(w.std()) < 1.0, float(w.std())
    dense["token_embd.weight"] = quant["token_embd.weight"]
    ours.write_gguf(fpath, md, dense)
    rq, rf = llm.LlamaRuntime.from_gguf(qpath, device="cpu"), llm.LlamaRuntime.from_gguf(fpath, device="cpu")
    prompt = torch.randint(0, vocab, (1, 6), generator=torch.Generator().manual_seed(0))
    lq, lf = rq.prefill(prompt, rq.new_cache(1, 16)), rf.prefill(prompt, rf.new_cache(1, 16))
    assert torch.isfinite(lq).all() and torch.allclose(lq, lf, atol=1e-5)
