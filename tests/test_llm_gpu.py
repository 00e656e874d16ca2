"""Dequant-fused GEMV, fp16 decode kernels and the Llama runtime on the GPU vs fp32 references."""
import math

import pytest
import torch

from conftest import rel_err

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("q8", [False, True])
@pytest.mark.parametrize("M,N,K", [(1, 4096, 4096), (3, 1001, 11008), (8, 256, 64), (20, 512, 4096)])
def test_q_gemv_matches_dequantised_matmul(q8, M, N, K):
    from rustorch_b200.formats import gguf
    from rustorch_b200.llm import QuantLinear
    ty = gguf.GGMLType.Q8_0 if q8 else gguf.GGMLType.Q4_0
    q = QuantLinear.random(N, K, ty, 0.02, "cuda", seed=1)
    x = (torch.randn(M, K, device="cuda") * 0.5).half()
    res = (torch.randn(M, N, device="cuda")).half()
    y = q(x, residual=res)
    ref = x.float() @ q.dequantize().t() + res.float()
    assert rel_err(y, ref) < 6e-3


def test_repack_roundtrip_from_gguf_blocks():
    from rustorch_b200.formats import gguf
    from rustorch_b200.llm import QuantLinear
    w = torch.randn(64, 256) * 0.02
    for ty, fn in ((gguf.GGMLType.Q4_0, gguf.quantize_q4_0), (gguf.GGMLType.Q8_0, gguf.quantize_q8_0)):
        blocks = torch.from_numpy(fn(w.numpy()))
        cpu = QuantLinear(blocks, ty, "cpu").dequantize()
        gpu = QuantLinear(blocks, ty, "cuda").dequantize().cpu()
        assert torch.equal(cpu, gpu)


def test_decode_kernels_vs_reference():
    from rustorch_b200 import _native
    C = _native.load(required=True)
    torch.manual_seed(0)
    x = torch.randn(5, 512, device="cuda").half()
    w = torch.rand(512, device="cuda").half()
    y = torch.empty_like(x)
    C.rmsnorm_f16(x, w, y, 1e-5)
    ref = x.float() * torch.rsqrt(x.float().pow(2).mean(-1, keepdim=True) + 1e-5) * w.float()
    assert rel_err(y, ref) < 2e-3
    g, u = torch.randn(4, 64, device="cuda").half(), torch.randn(4, 64, device="cuda").half()
    o = torch.empty_like(g)
    C.silu_mul(g, u, o)
    assert rel_err(o, torch.nn.functional.silu(g.float()) * u.float()) < 2e-3


@pytest.mark.parametrize("gqa", [False, True])
def test_runtime_gpu_matches_cpu_path(gqa):
    from rustorch_b200.llm import LlamaConfig, LlamaRuntime
    cfg = LlamaConfig(vocab_size=128, n_layer=2, n_embd=256, n_head=4, n_head_kv=2 if gqa else 4, n_ff=512, context_length=64)
    gpu = LlamaRuntime.random_init(cfg, "cuda", seed=3, std=0.05)
    cpu = LlamaRuntime(cfg, "cpu")
    # copy the synthetic weights into a CPU runtime through their dequantised form
    from rustorch_b200.formats import gguf
    from rustorch_b200.llm import QuantLinear

    class _Dense:
        def __init__(self, w):
            self.w = w
            self.out_features, self.in_features = w.shape

        def __call__(self, x, residual=None):
            y = x.float() @ self.w.t()
            return (y + residual.float() if residual is not None else y).to(x.dtype)

    for L in gpu.layers:
        n = type(L)()
        n.wqkv, n.wo = _Dense(L.wqkv.dequantize().cpu()), _Dense(L.wo.dequantize().cpu())
        n.w_gate_up, n.w_down = _Dense(L.w_gate_up.dequantize().cpu()), _Dense(L.w_down.dequantize().cpu())
        n.attn_norm, n.ffn_norm = L.attn_norm.float().cpu(), L.ffn_norm.float().cpu()
        cpu.layers.append(n)
    cpu.tok_emb, cpu.out_norm = gpu.tok_emb.float().cpu(), gpu.out_norm.float().cpu()
    cpu.lm_head = _Dense(gpu.lm_head.dequantize().cpu())
    prompt = torch.randint(0, 128, (2, 9), generator=torch.Generator().manual_seed(0))
    cg, cc = gpu.new_cache(2, 32), cpu.new_cache(2, 32)
    lg, lc = gpu.prefill(prompt, cg), cpu.prefill(prompt, cc)
    assert rel_err(lg.cpu(), lc) < 3e-2
    nxt = lc.argmax(-1)
    lg2, lc2 = gpu.decode_step(nxt.cuda(), cg), cpu.decode_step(nxt, cc)
    assert rel_err(lg2.cpu(), lc2) < 3e-2
    assert rel_err(cg.k[1][:, :, :10].float().cpu(), cc.k[1][:, :, :10]) < 2e-2
    out, stats = gpu.generate(prompt, 6)
    assert out.shape == (2, 15) and stats["decode_tokens_per_s"] > 0


@pytest.mark.parametrize("D,H,Hkv", [(128, 8, 2), (64, 4, 4), (128, 16, 2), (256, 2, 1), (96, 4, 4)])
def test_cached_attention_split_kv_vs_reference(D, H, Hkv):
    """Split-KV decode attention (several key slices + merge) and the generic fallback (D = 96)."""
    from rustorch_b200 import _native
    C = _native.load(required=True)
    torch.manual_seed(1)
    B, T_max = 3, 1024
    ck = torch.randn(B, Hkv, T_max, D, device="cuda").half()
    cv = torch.randn(B, Hkv, T_max, D, device="cuda").half()
    kv_len = torch.tensor([700, 1, 130, 64, 1024], dtype=torch.int32, device="cuda")
    seq = torch.tensor([0, 1, 2, 1, 0], dtype=torch.int32, device="cuda")
    n = kv_len.numel()
    qkv = torch.randn(n, (H + 3) * D, device="cuda").half()          # q is a strided view, as in the runtime
    q = qkv[:, : H * D].view(n, H, D)
    out = torch.empty(n, H, D, device="cuda", dtype=torch.half)
    scale = 1.0 / math.sqrt(D)
    C.attn_cache(q, ck, cv, out, kv_len, seq, T_max, scale)
    for t in range(n):
        L, s = int(kv_len[t]), int(seq[t])
        k = ck[s, :, :L].float().repeat_interleave(H // Hkv, 0)
        v = cv[s, :, :L].float().repeat_interleave(H // Hkv, 0)
        p = torch.softmax((k @ q[t].float().unsqueeze(-1)).squeeze(-1) * scale, -1)
        ref = (p.unsqueeze(1) @ v).squeeze(1)
        assert rel_err(out[t], ref) < 3e-3, (t, L)


@pytest.mark.parametrize("q8", [False, True])
def test_quant_linear_gemm_path_for_many_rows(q8):
    """From 64 rows on the weights are expanded to fp16 and multiplied on the tcgen05 GEMM."""
    from rustorch_b200.formats import gguf
    from rustorch_b200.llm import QuantLinear
    q = QuantLinear.random(1000, 1024, gguf.GGMLType.Q8_0 if q8 else gguf.GGMLType.Q4_0, 0.02, "cuda", seed=2)
    x = (torch.randn(200, 1024, device="cuda") * 0.5).half()
    res = torch.randn(200, 1000, device="cuda").half()
    assert x.shape[0] >= QuantLinear.GEMM_MIN_ROWS
    y = q(x, residual=res)
    ref = x.float() @ q.dequantize().t() + res.float()
    assert rel_err(y, ref) < 3e-3
    from rustorch_b200 import _native
    _native.check_status()


def test_graph_decode_matches_eager_decode():
    from rustorch_b200.llm import LlamaConfig, LlamaRuntime
    cfg = LlamaConfig(vocab_size=256, n_layer=2, n_embd=256, n_head=4, n_head_kv=2, n_ff=512, context_length=128)
    rt_ = LlamaRuntime.random_init(cfg, "cuda", seed=5, std=0.08)
    prompt = torch.randint(0, 256, (2, 70), generator=torch.Generator().manual_seed(1))
    a, _ = rt_.generate(prompt, 12)
    b, stats = rt_.generate_graph(prompt, 12)
    assert torch.equal(a, b) and stats["decode_steps"] == 11


@pytest.mark.parametrize("q8", [False, True])
@pytest.mark.parametrize("M,N,K", [(1, 4096, 4096), (2, 1001, 11008), (4, 70, 256), (7, 515, 2048)])
def test_q_gemv_register_and_bulk_paths_agree(q8, M, N, K):
    """The bulk-copy (shared-memory ring) kernel and the register-fed kernel compute the same product."""
    from rustorch_b200 import _native
    from rustorch_b200.formats import gguf
    from rustorch_b200.llm import QuantLinear
    C = _native.load(required=True)
    q = QuantLinear.random(N, K, gguf.GGMLType.Q8_0 if q8 else gguf.GGMLType.Q4_0, 0.02, "cuda", seed=4)
    x = (torch.randn(M, K, device="cuda") * 0.5).half()
    ya, yb = torch.empty(M, N, device="cuda", dtype=torch.half), torch.empty(M, N, device="cuda", dtype=torch.half)
    C.q_gemv(q.qs, q.scales, x, ya, None, None, q.q8, path=2)
    C.q_gemv(q.qs, q.scales, x, yb, None, None, q.q8, path=1)
    ref = x.float() @ q.dequantize().t()
    assert rel_err(ya, ref) < 6e-3 and rel_err(yb, ref) < 6e-3
    _native.check_status()


@pytest.mark.parametrize("q8", [False, True])
@pytest.mark.parametrize("M,N,K", [(9, 1000, 1024), (16, 4096, 4096), (32, 515, 5504), (100, 384, 2752), (256, 1024, 4096),
                                   (33, 128, 32), (64, 22016, 4096)])
def test_q_gemm_tensor_core_matches_reference(q8, M, N, K):
    """Dequant-fused tcgen05 GEMM (weights read once for all rows) against x @ dequant(W)^T + residual; covers ragged N,
    K that is not a multiple of the raw tile, every padded row count and the split-K reduction."""
    from rustorch_b200 import _native
    from rustorch_b200.formats import gguf
    from rustorch_b200.llm import QuantLinear
    q = QuantLinear.random(N, K, gguf.GGMLType.Q8_0 if q8 else gguf.GGMLType.Q4_0, 0.05, "cuda", seed=M + N)
    x = (torch.randn(M, K, device="cuda") * 0.5).half()
    res = torch.randn(M, N, device="cuda").half()
    assert QuantLinear.TC_MIN_ROWS <= M <= QuantLinear.TC_MAX_ROWS
    ref = x.float() @ q.dequantize().t().to("cuda") + res.float()
    try:
        for path in (0, 1):                           # operand A in tensor memory / staged in shared memory
            QuantLinear.TC_PATH = path
            for _ in range(2):                        # second call: the tile counters were left at zero
                y = q(x, residual=res)
                assert rel_err(y, ref) < 3e-3, path
            y2 = q(x)
            assert rel_err(y2, ref - res.float()) < 3e-3, path
    finally:
        QuantLinear.TC_PATH = 0
    _native.check_status()


@pytest.mark.parametrize("D,H,Hkv", [(64, 4, 2), (128, 8, 2)])
def test_flash_attention_fp16_io_on_packed_qkv(D, H, Hkv):
    """The prefill path: fp16 q / k / v read as strided views of one packed projection output."""
    from rustorch_b200 import _native
    C = _native.load(required=True)
    B, T = 2, 200
    qkv = (torch.randn(B * T, (H + 2 * Hkv) * D, device="cuda") * 0.7).half()
    q = qkv[:, : H * D].view(B * T, H, D).unflatten(0, (B, T))
    k = qkv[:, H * D: (H + Hkv) * D].view(B * T, Hkv, D).unflatten(0, (B, T))
    v = qkv[:, (H + Hkv) * D:].view(B * T, Hkv, D).unflatten(0, (B, T))
    out = torch.empty((B, T, H, D), dtype=torch.half, device="cuda")
    lse = torch.empty((B, H, T), dtype=torch.float32, device="cuda")
    scale = D ** -0.5
    C.attn_fwd(q, k, v, out, lse, True, scale)
    g = H // Hkv
    qf, kf, vf = q.float().transpose(1, 2), k.float().repeat_interleave(g, 2).transpose(1, 2), v.float().repeat_interleave(g, 2).transpose(1, 2)
    s = (qf @ kf.transpose(-1, -2)) * scale
    s = s.masked_fill(torch.ones(T, T, device="cuda", dtype=torch.bool).triu(1), float("-inf"))
    ref = (torch.softmax(s, -1) @ vf).transpose(1, 2)
    assert rel_err(out, ref) < 4e-3
    assert rel_err(lse, torch.logsumexp(s, -1)) < 1e-3
    _native.check_status()


def test_prefill_flash_path_matches_cached_attention_path():
    from rustorch_b200.llm import LlamaConfig, LlamaRuntime
    cfg = LlamaConfig(vocab_size=256, n_layer=2, n_embd=256, n_head=4, n_head_kv=2, n_ff=512, context_length=128)
    rt_ = LlamaRuntime.random_init(cfg, "cuda", seed=5, std=0.08)
    prompt = torch.randint(0, 256, (2, 70), generator=torch.Generator().manual_seed(1)).cuda()
    c1, c2 = rt_.new_cache(2, 96), rt_.new_cache(2, 96)
    a = rt_.prefill(prompt, c1)                                               # flash kernel
    pos = torch.arange(70, device="cuda").repeat(2)
    seq = torch.arange(2, device="cuda").repeat_interleave(70)
    last = torch.arange(2, device="cuda") * 70 + 69
    b = rt_.forward_tokens(prompt.reshape(-1), pos, seq, c2, last_only=last, max_kv=70)   # per-token cached attention
    assert rel_err(a, b) < 5e-3
    assert rel_err(c1.k[0], c2.k[0]) < 1e-6                      # layer 0: same inputs, same rotation
    assert all(rel_err(x, y) < 5e-3 for x, y in zip(c1.k, c2.k))   # later layers see the other kernel's rounding


@pytest.mark.parametrize("q8", [False, True])
@pytest.mark.parametrize("M,N,K", [(1, 4096, 4096), (2, 1002, 11008), (4, 250, 832), (3, 64, 64), (1, 38, 128)])
def test_fused_decode_projection_matches_fp32_reference(q8, M, N, K):
    """RMSNorm prologue + dequant-fused GEMV + residual / SwiGLU epilogue in one kernel vs fp32 math on the
    dequantised weights (ragged N, K that is not a multiple of the lanes' stride, 1..4 rows).  The kernel
    quantises the activations to int8 per 32-element block (max |h| / 127), which bounds its error at ~0.4 % of a
    typical output; the tolerances are set for that."""
    from rustorch_b200 import _native
    from rustorch_b200.formats import gguf
    from rustorch_b200.llm import QuantLinear
    ty = gguf.GGMLType.Q8_0 if q8 else gguf.GGMLType.Q4_0
    q = QuantLinear.random(N, K, ty, 0.02, "cuda", seed=2)
    W = q.dequantize()
    x = (torch.randn(M, K, device="cuda") * 0.7).half()
    nw = (1.0 + 0.1 * torch.randn(K, device="cuda")).half()
    res = torch.randn(M, N, device="cuda").half()
    eps = 1e-5
    xf = x.float()
    h = (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * nw.float()).half().float()
    n0 = _native.launch_count()
    y = q.fused(x, norm_w=nw, eps=eps, residual=res)
    assert _native.launch_count() == n0 + 1                      # one kernel
    tol = 8e-3 if K >= 512 else 2e-2
    assert rel_err(y, h @ W.t() + res.float()) < tol
    y2 = q.fused(x)                                              # no prologue, no epilogue
    assert rel_err(y2, xf @ W.t()) < tol
    ff = N // 2
    act = q.fused(x, norm_w=nw, eps=eps, swiglu=True)
    t = h @ W.t()
    ref = torch.nn.functional.silu(t[:, :ff].half().float()) * t[:, ff:].half().float()
    # with K = 128 only four int8 blocks average the activation rounding out
    assert act.shape == (M, ff) and rel_err(act, ref) < (1e-2 if K >= 512 else 2.5e-2)
    _native.check_status()


def test_fused_decode_projection_falls_back_beyond_four_rows():
    from rustorch_b200.formats import gguf
    from rustorch_b200.llm import QuantLinear
    q = QuantLinear.random(512, 256, gguf.GGMLType.Q4_0, 0.02, "cuda", seed=3)
    x = (torch.randn(6, 256, device="cuda") * 0.7).half()
    nw = torch.ones(256, device="cuda").half()
    xf = x.float()
    h = (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-5)).half().float()
    t = h @ q.dequantize().t()
    ref = torch.nn.functional.silu(t[:, :256].half().float()) * t[:, 256:].half().float()
    assert rel_err(q.fused(x, norm_w=nw, eps=1e-5, swiglu=True), ref) < 8e-3


def test_cache_position_past_the_end_is_reported_not_written():
    """Positions and sequence numbers come from device data (a replayed decode graph advances them itself): a token
    past the end of the cache must turn into an IndexOutOfBounds error with the cache untouched, never a write
    outside it, and the device stays usable."""
    from rustorch_b200 import _native
    from rustorch_b200.error import IndexOutOfBounds
    C = _native.load(required=True)
    H, Hkv, D, T_max = 4, 2, 64, 16
    q = torch.randn(1, H, D, device="cuda").half()
    k = torch.randn(1, Hkv, D, device="cuda").half()
    v = torch.randn(1, Hkv, D, device="cuda").half()
    ck = torch.zeros(2, Hkv, T_max, D, device="cuda", dtype=torch.half)
    cv = torch.zeros_like(ck)
    seq = torch.zeros(1, device="cuda", dtype=torch.int32)
    for bad_pos, bad_seq in ((T_max, 0), (-1, 0), (3, 2)):
        pos = torch.full((1,), bad_pos, device="cuda", dtype=torch.int32)
        seq.fill_(bad_seq)
        C.rope_kv(q.clone(), k.clone(), v, ck, cv, pos, seq, 10000.0, True)
        with pytest.raises(IndexOutOfBounds):
            _native.check_status()
        assert float(ck.abs().max()) == 0.0 and float(cv.abs().max()) == 0.0
    # attention over a claimed length beyond the cache: reported, result finite
    out = torch.empty(1, H, D, device="cuda", dtype=torch.half)
    seq.fill_(0)
    C.attn_cache(q, ck, cv, out, torch.full((1,), T_max + 5, device="cuda", dtype=torch.int32), seq, T_max, 0.125)
    with pytest.raises(IndexOutOfBounds):
        _native.check_status()
    assert torch.isfinite(out.float()).all()
    # a valid step still works afterwards
    pos = torch.full((1,), 3, device="cuda", dtype=torch.int32)
    C.rope_kv(q.clone(), k.clone(), v, ck, cv, pos, seq, 10000.0, True)
    _native.check_status()
    assert float(ck[0, :, 3].abs().max()) > 0.0


@pytest.mark.parametrize("q8", [False, True])
@pytest.mark.parametrize("M,H,Hkv,D", [(1, 4, 4, 64), (3, 8, 2, 128), (4, 2, 1, 32)])
def test_fused_qkv_projection_with_rotary_epilogue_matches_separate_kernels(q8, M, H, Hkv, D):
    """q | k | v projection with the rotary embedding and the cache append in its epilogue against the projection
    kernel followed by the stand-alone rotary / append kernel: same outputs, same cache contents."""
    from rustorch_b200 import _native
    from rustorch_b200.formats import gguf
    from rustorch_b200.llm import QuantLinear
    C = _native.load(required=True)
    K, T_max, B = 256, 24, 5
    ty = gguf.GGMLType.Q8_0 if q8 else gguf.GGMLType.Q4_0
    lin = QuantLinear.random((H + 2 * Hkv) * D, K, ty, 0.05, "cuda", seed=6)
    x = (torch.randn(M, K, device="cuda") * 0.7).half()
    nw = (1.0 + 0.1 * torch.randn(K, device="cuda")).half()
    pos = torch.tensor([5, 0, 23, 11][:M], device="cuda", dtype=torch.int32)
    seq = torch.tensor([4, 1, 0, 2][:M], device="cuda", dtype=torch.int32)
    # separate kernels
    y_ref = lin.fused(x, norm_w=nw, eps=1e-5)
    ck_ref = torch.zeros(B, Hkv, T_max, D, device="cuda", dtype=torch.half)
    cv_ref = torch.zeros_like(ck_ref)
    q = y_ref[:, : H * D].view(M, H, D)
    k = y_ref[:, H * D: (H + Hkv) * D].view(M, Hkv, D)
    v = y_ref[:, (H + Hkv) * D:].view(M, Hkv, D)
    C.rope_kv(q, k, v, ck_ref, cv_ref, pos, seq, 10000.0, True)
    # one kernel
    ck, cv = torch.zeros_like(ck_ref), torch.zeros_like(cv_ref)
    n0 = _native.launch_count()
    y = lin.fused(x, norm_w=nw, eps=1e-5, rope=dict(pos=pos, seq=seq, cache_k=ck, cache_v=cv, n_head=H, theta=10000.0))
    assert _native.launch_count() == n0 + 1
    _native.check_status()
    assert torch.equal(y, y_ref)
    assert torch.equal(ck, ck_ref) and torch.equal(cv, cv_ref)
    assert float(ck.abs().max()) > 0 and float(cv.abs().max()) > 0
