"""CPU tests: sparse tensors, pruning, sparse layers, analysis / IO."""
import pytest
import torch

from rustorch_b200 import sparse as S


def _rand_sparse(m=12, n=9, density=0.3, seed=0):
    g = torch.Generator().manual_seed(seed)
    d = torch.randn(m, n, generator=g) * (torch.rand(m, n, generator=g) < density)
    return d, S.SparseTensor.from_dense(d)


def test_formats_conversions_and_ops():
    d, sp = _rand_sparse()
    assert sp.format is S.SparseFormat.COO and sp.nnz == int((d != 0).sum()) and abs(sp.sparsity() - (1 - sp.nnz / d.numel())) < 1e-9
    csr = sp.to_csr()
    assert torch.equal(csr.to_dense(), d) and torch.equal(csr.to_coo().to_dense(), d)
    S.SparseValidator.validate(sp), S.SparseValidator.validate(csr)
    v, B = torch.randn(9), torch.randn(9, 4)
    assert torch.allclose(sp.spmv(v), d @ v, atol=1e-5) and torch.allclose(csr.spmv(v), d @ v, atol=1e-5)
    assert torch.allclose(csr.spmm(B), d @ B, atol=1e-5)
    d2, sp2 = _rand_sparse(seed=1)
    assert torch.allclose(sp.add(sp2).to_dense(), d + d2, atol=1e-6)
    assert torch.equal(sp.transpose().to_dense(), d.t()) and torch.allclose(sp.mul_scalar(2).to_dense(), 2 * d)
    assert sp.memory_usage() < d.numel() * 4 * 3
    with pytest.raises(ValueError):
        S.SparseTensor.from_coo(torch.zeros(2, 3, dtype=torch.long), torch.ones(2), (4, 4))
    with pytest.raises(IndexError):
        S.SparseTensor.from_coo(torch.tensor([[5], [0]]), torch.ones(1), (4, 4))
    with pytest.raises(ValueError):
        S.SparseTensor.from_csr(torch.tensor([0, 1]), torch.tensor([0]), torch.ones(1), (3, 3))


def test_pruners_hit_target_sparsity():
    w = torch.randn(32, 64)
    for sp in (0.25, 0.5, 0.9):
        p = S.MagnitudePruner(sp).prune(w)
        assert abs(float((p == 0).float().mean()) - sp) < 0.01
        assert p.abs()[p != 0].min() >= w.abs().flatten().kthvalue(int(w.numel() * sp)).values
    rows = S.StructuredPruner(0.5, S.StructuredGranularity.ROW).prune_linear_weights(w)
    assert int((rows.abs().sum(1) == 0).sum()) == 16
    cols = S.StructuredPruner(0.25, S.StructuredGranularity.COLUMN).prune_linear_weights(w)
    assert int((cols.abs().sum(0) == 0).sum()) == 16
    blk = S.StructuredPruner(0.5, S.StructuredGranularity.BLOCK, 4).prune_linear_weights(w)
    zb = (blk.reshape(8, 4, 16, 4).abs().sum((1, 3)) == 0).sum()
    assert int(zb) == 64
    fp = S.FisherPruner(0.5)
    fp.update_fisher("w", torch.randn(32, 64))
    assert abs(float((fp.prune_with_fisher("w", w) == 0).float().mean()) - 0.5) < 0.01
    ties = S.MagnitudePruner(0.5).prune(torch.ones(10))
    assert int((ties == 0).sum()) == 5


def test_schedule_and_model_pruner():
    sch = S.PruningSchedule(0.0, 0.8, begin_step=0, end_step=100, frequency=10)
    vals = []
    for _ in range(120):
        vals.append(sch.current_sparsity())
        sch.step()
    assert vals[0] == 0 and abs(vals[-1] - 0.8) < 1e-9 and all(b >= a - 1e-12 for a, b in zip(vals, vals[1:]))
    model = torch.nn.Sequential(torch.nn.Linear(16, 32), torch.nn.ReLU(), torch.nn.Linear(32, 4))
    pr = S.ModelPruner(S.PruningConfig(target_sparsity=0.75))
    rep = pr.prune_model(model)
    assert set(rep) == {"0.weight", "2.weight"} and all(abs(v - 0.75) < 0.02 for v in rep.values())
    opt = torch.optim.SGD(model.parameters(), lr=0.1)
    model(torch.randn(8, 16)).sum().backward()
    opt.step()
    pr.apply_masks(model)
    assert abs(float((model[0].weight == 0).float().mean()) - 0.75) < 0.02
    st = pr.prune_tensor(torch.randn(10, 10))
    assert isinstance(st, S.SparseTensor) and abs(st.sparsity() - 0.75) < 0.02


def test_sparse_layers_forward_backward():
    torch.manual_seed(0)
    lin = torch.nn.Linear(20, 12)
    sl = S.SparseLinear.from_dense(lin, 0.7)
    x = torch.randn(5, 20, requires_grad=True)
    y = sl(x)
    ref = x @ sl.weight().to_dense().t() + lin.bias
    assert torch.allclose(y, ref, atol=1e-5) and abs(sl.sparsity() - 0.7) < 0.02
    y.sum().backward()
    assert sl.values.grad is not None and sl.values.grad.shape == sl.values.shape and x.grad is not None
    sl.prune_weights(0.9)
    assert abs(sl.sparsity() - 0.9) < 0.02 and sl(x).shape == (5, 12)
    conv = S.SparseConv2d(3, 8, 3, padding=1, sparsity=0.5, structured=True)
    assert conv(torch.randn(2, 3, 6, 6)).shape == (2, 8, 6, 6) and sum(1 for s in conv.filter_sparsity() if s == 1.0) == 4
    blk = S.SparseTransformerBlock(16, 4, 32, sparsity=0.5, window=2, seq_len=10)
    out = blk(torch.randn(2, 10, 16))
    assert out.shape == (2, 10, 16) and set(blk.sparsity_report()) == {"ff1", "ff2", "attention"}
    emb = S.SparseEmbedding(50, 8)
    emb(torch.tensor([1, 2, 2])).sum().backward()
    assert emb.emb.weight.grad.is_sparse


def test_analysis_io_benchmark(tmp_path):
    d, sp = _rand_sparse(20, 20, 0.1)
    an = S.SparseAnalyzer.analyze_pattern(sp)
    assert an.nnz == sp.nnz and "nnz=" in an.report() and an.optimization_recommendations()
    assert S.SparseAnalyzer.suggest_optimal_format(sp) is S.SparseFormat.CSR
    for t in (sp, sp.to_csr()):
        S.SparseIO.save_binary(t, str(tmp_path / "t.bin"))
        back = S.SparseIO.load_binary(str(tmp_path / "t.bin"))
        assert back.format is t.format and torch.allclose(back.to_dense(), d)
    assert [t.format for t in S.SparseConverter.batch_convert([sp, sp], S.SparseFormat.CSR)] == [S.SparseFormat.CSR] * 2
    bad = S.SparseTensor(S.SparseFormat.CSR, (3, 3), torch.ones(2), crow=torch.tensor([0, 2, 1, 2]), col=torch.tensor([0, 1]))
    with pytest.raises(ValueError):
        S.SparseValidator.validate(bad)
    bm = S.SparseBenchmark(iters=2)
    r = bm.benchmark_spmv(sp, torch.randn(20))
    assert r.sparse_ms > 0 and "speedup" in bm.report()
