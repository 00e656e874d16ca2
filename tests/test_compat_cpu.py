"""Named pieces of the reference surface: errors, parallel traits, hardware hints, hybrid f32, loaders, devices."""
import os

import pytest
import torch

import rustorch_b200 as rt


def test_error_hierarchy_and_helpers():
    from rustorch_b200 import error as E
    with pytest.raises(E.TensorOp) as ei:
        raise E.RusTorchError.shape_mismatch([2, 3], [3, 2])
    assert ei.value.kind == "ShapeMismatch" and "expected [2, 3]" in str(ei.value)
    assert issubclass(E.KernelTimeout, E.GpuError) and issubclass(E.GpuError, rt.RusTorchError)
    assert E.check_status_to_error(0) is None and isinstance(E.check_status_to_error(104), E.KernelTimeout)
    assert isinstance(E.check_status_to_error(201), E.IndexOutOfBounds)


def test_parallel_traits_and_context():
    from rustorch_b200 import parallel as P
    a, b = torch.randn(6, 4, 5), torch.randn(6, 5, 3)
    assert torch.allclose(P.batch_matmul_parallel(a, b), torch.bmm(a, b))
    n = P.batch_normalize_parallel(torch.randn(4, 10))
    assert n.mean(1).abs().max() < 1e-5 and (n.var(1, unbiased=False) - 1).abs().max() < 1e-3
    with P.ParallelContext(P.ParallelConfig(strategy=P.ParallelStrategy.FORCE_PARALLEL, chunk_size=2)) as ctx:
        assert torch.equal(ctx.map_chunks(lambda t: t * 3, torch.ones(7, 2)), torch.full((7, 2), 3.0))
    pt = rt.ParallelTensor(a)
    assert pt.matmul(b).data.shape == (6, 4, 3) and abs(float(pt.sum()) - float(a.sum())) < 1e-3
    assert not P.ParallelConfig(strategy=P.ParallelStrategy.SEQUENTIAL).should_parallelize(10 ** 9)
    assert P.kaiming_init((64, 32)).std() < 1.0 and P.DistributedSampler is not None


def test_hardware_optimizer_and_backends():
    h = rt.HardwareOptimizer()
    assert h.gemm_tile(4096, 4096, 4096) == (128, 256, 64) and h.gemm_tile(64, 100, 64)[1] == 128
    assert h.persistent_grid(10) <= 10 and h.preferred_layout("conv2d") == "channels_last"
    assert rt.SimdOptimizer().vector_width(torch.bfloat16) == 8
    from rustorch_b200.gpu import devices as D
    cpu = D.CpuBackend()
    assert torch.equal(cpu.add(torch.ones(2), torch.ones(2)), torch.full((2,), 2.0)) and "threads" in cpu.capabilities()
    assert isinstance(D.BackendManager(D.SelectionStrategy.CPU_ONLY).select(), D.CpuBackend)
    ex = D.KernelExecutor(D.CpuDevice())
    assert torch.allclose(ex.execute("matmul", torch.eye(3), torch.ones(3, 2)), torch.ones(3, 2))
    from rustorch_b200.gpu import DeviceNotAvailable
    for cls in (D.MetalKernelExecutor, D.OpenClKernelExecutor, D.CoreMLHybrid):
        with pytest.raises(DeviceNotAvailable):
            cls()


def test_adam_utils_and_lbfgs_memory_match_torch():
    from rustorch_b200.compat import AdamConfig, AdamState, AdamUtils, LBFGSMemory, LineSearchMethod
    p = torch.nn.Parameter(torch.tensor([1.0, -2.0, 3.0]))
    ref = p.detach().clone()
    opt = torch.optim.Adam([p], lr=0.1)
    st, cfg = AdamState(), AdamConfig(lr=0.1)
    for _ in range(3):
        g = torch.tensor([0.5, -1.0, 2.0])
        p.grad = g.clone()
        opt.step()
        AdamUtils.step(ref, g, st, cfg)
    assert torch.allclose(ref, p.detach(), atol=1e-6)
    mem = LBFGSMemory(4)
    A = torch.diag(torch.tensor([1.0, 4.0, 9.0]))          # quadratic: after n updates the direction is Newton's
    x = torch.zeros(3)
    for _ in range(6):
        g = A @ x - torch.ones(3)
        d = mem.direction(g)
        x_new = x + d * (0.1 if len(mem) == 0 else 1.0)
        mem.update(x_new - x, A @ x_new - torch.ones(3) - g)
        x = x_new
    assert torch.allclose(x, torch.tensor([1.0, 0.25, 1 / 9]), atol=1e-3)
    assert LineSearchMethod.STRONG_WOLFE.torch_name() == "strong_wolfe"


def test_shape_builder_lazy_expand_safe_numeric_window_int4():
    from rustorch_b200 import compat as C
    assert C.ShapeBuilder(torch.zeros(2, 3)).unsqueeze(0).expand(4, -1, -1).flatten(1).shape() == (4, 6)
    lz = C.LazyExpandedTensor(torch.arange(3.0).view(1, 3), (5, 3))
    assert lz.memory_saved() == 12 * 4 and lz.materialize().is_contiguous() and float(lz[4, 2]) == 2.0
    with pytest.raises(rt.RusTorchError):
        C.SafeTensor(torch.tensor([1e38])) * 1e10
    with pytest.raises(rt.RusTorchError):
        C.SafeNumeric.safe_cast(torch.tensor([70000.0]), torch.float16)
    with pytest.raises(rt.RusTorchError):
        C.TypedTensor(torch.zeros(3), 2)
    assert torch.allclose(C.WindowType.HAMMING.apply(torch.ones(8)), torch.hamming_window(8, periodic=False))
    v = torch.tensor([-8, 7, 0, -1, 5])
    assert torch.equal(C.Int4.unpack(C.Int4.pack(v), 5), v.to(torch.int8))
    assert C.ZeroCopyOps.shares_storage(torch.zeros(4, 4), torch.zeros(1)) is False
    t = torch.arange(12.0).view(3, 4)
    assert C.ZeroCopyOps.shares_storage(t, C.ZeroCopyOps.slice_view(t, 1, 1, 3))
    assert C.TensorIterOps.fold(t, 0.0, lambda a, c: a + float(c.sum()), chunk=5) == 66.0
    pc = C.ProfilerCore()
    pc.start_session("s"); pc.start_timer("a"); pc.stop_timer("a")
    assert pc.end_session()["timers"]["a"] and pc.summary()["a"]["count"] == 1


def test_hybrid_f32_tensor_variable_trainer(tmp_path):
    from rustorch_b200 import hybrid_f32 as H
    a = H.F32Tensor.from_vec([1, 2, 3, 4], [2, 2])
    assert (a @ a).to_vec() == [7.0, 10.0, 15.0, 22.0] and a.transpose().to_vec() == [1.0, 3.0, 2.0, 4.0]
    v = H.F32Variable(a, True)
    (v * v).sum().backward()
    assert v.grad().to_vec() == [2.0, 4.0, 6.0, 8.0]
    torch.manual_seed(0)
    m = torch.nn.Sequential(H.F32Linear(4, 8), torch.nn.ReLU(), H.F32Linear(8, 1))
    X = torch.randn(64, 4)
    Y = X.sum(1, keepdim=True)
    data = [(X[i:i + 16], Y[i:i + 16]) for i in range(0, 64, 16)]
    cfg = H.F32TrainerConfig(epochs=40, learning_rate=0.05, early_stopping_patience=8, scheduler="cosine", checkpoint_dir=str(tmp_path))
    tr = H.F32Trainer(m, torch.nn.functional.mse_loss, cfg, device="cpu")
    hist = tr.fit(data, data)
    assert hist["train_loss"][-1] < 0.2 * hist["train_loss"][0] and os.path.exists(tmp_path / "best.pt")
    assert tr.load_checkpoint(str(tmp_path / "best.pt")) >= 0


def test_loader_objects_round_trip(tmp_path):
    from rustorch_b200.formats import gguf
    from rustorch_b200.formats.loaders import GGUFLoader, SafetensorsLoader, SafetensorsSaver, TensorLoader
    p = str(tmp_path / "m.safetensors")
    w = {"a.weight": torch.randn(3, 4), "b": torch.arange(5.0)}
    sv = SafetensorsSaver({"format": "pt"})
    for k, t in w.items():
        sv.add_tensor(k, t)
    sv.save_to_file(p)
    ld = SafetensorsLoader.from_file(p)
    assert sorted(ld.tensor_names()) == sorted(w) and ld.metadata()["format"] == "pt" and torch.equal(ld.tensor("b"), w["b"])
    assert torch.equal(TensorLoader(p).load_tensor("a.weight"), w["a.weight"])
    g = str(tmp_path / "m.gguf")
    gguf.write_gguf(g, {"general.architecture": "llama", "llama.block_count": 2}, {"t": (torch.randn(4, 64), gguf.GGMLType.Q8_0)})
    with GGUFLoader(g) as gl:
        assert gl.architecture() == "llama" and gl.tensor_names() == ["t"] and gl.load_tensor("t").shape == (4, 64)
    assert TensorLoader(g).tensor_names() == ["t"]


def test_misc_named_pieces():
    from rustorch_b200 import compat as C
    g = C.GPTModel(50, 32, 1, 2, 16)
    out = g(torch.randint(0, 50, (2, 8)))
    assert out.shape == (2, 8, 50) and torch.equal(out, C.GPTModel(50, 32, 1, 2, 16)(torch.randint(0, 50, (2, 8), generator=None)) * 0 + out)
    x, w = torch.randn(4, 3, requires_grad=True), torch.randn(2, 3, requires_grad=True)
    C.LinearBackward.apply(x, w, None).sum().backward()
    assert torch.allclose(w.grad, x.detach().sum(0).expand(2, 3))
    assert C.DistributedState.get()["world_size"] == 1 and not C.DistributedState.is_initialized()
    cell = torch.nn.GRUCell(3, 4)
    ys, h = C.RecurrentOps.run_cell(lambda xt, s: cell(xt, s), torch.randn(5, 2, 3))
    assert ys.shape == (5, 2, 4) and torch.equal(ys[-1], h)
    assert C.AllocationStrategy.PINNED.allocate((4,)).shape == (4,)


def test_gpu_trait_methods_and_linalg_helpers_on_cpu():
    from rustorch_b200 import tensor as T
    from rustorch_b200.parallel import GpuParallelOp
    a = rt.tensor([[1.0, 2.0], [3.0, 4.0]])
    assert a.gpu_matmul(a).data.cpu().tolist() == [[7.0, 10.0], [15.0, 22.0]] and a.gpu_sum() == 10.0 and a.gpu_max() == 4.0
    assert a.gpu_matvec(rt.tensor([1.0, 1.0])).data.cpu().tolist() == [3.0, 7.0]
    assert a.topk_util(1)[0].data.cpu().flatten().tolist() == [2.0, 4.0] and abs(a.quantile_util(0.5) - 2.5) < 1e-6
    assert T.select_optimal_device(4) == "cpu" and T.multithreaded_matmul(a, a, 2).data.shape == (2, 2)
    assert T.memory_optimized((3, 3)).data.sum() == 0
    assert float(GpuParallelOp().gpu_var(torch.tensor([1.0, 3.0]))) == 1.0


def test_guarded_tensor_detects_overrun():
    import pytest
    import torch
    from rustorch_b200.debug.guards import GuardedTensor, guard_scope
    from rustorch_b200.error import RusTorchError
    g = GuardedTensor((5, 7), torch.bfloat16)
    assert g.tensor.shape == (5, 7) and g.tensor.is_contiguous() and g.tensor.data_ptr() % 16 == 0
    with guard_scope(g):
        g.tensor.fill_(3.0)                               # in bounds: nothing to report
    past_end = torch.as_strided(g.tensor, (36,), (1,))    # one element more than the 35 the tensor has
    past_end[35] = 1.0
    assert g.violations() and g.violations()[0] == 70
    with pytest.raises(RusTorchError):
        g.check("workspace")
    h = GuardedTensor((16,), torch.float32)
    torch.as_strided(h.tensor, (1,), (1,), storage_offset=h.tensor.storage_offset() - 1)[0] = 2.0
    assert h.violations()[0] == -4


def test_python_module_surface_of_the_reference():
    """Names of the reference's Python module (src/python/mod.rs:51-115) resolve on ``import rustorch``."""
    import rustorch as rt
    names = ("Tensor Variable Linear Conv2d MaxPool2d BatchNorm1d BatchNorm2d Dropout Flatten ReLU Sigmoid Tanh MSELoss "
             "CrossEntropyLoss SGD Adam tensor zeros ones no_grad enable_grad grad Device relu sigmoid tanh softmax gelu leaky_relu "
             "swish elu selu mish StepLR ExponentialLR TensorDataset DataLoader Transform Transforms normalize resize random_crop "
             "random_horizontal_flip Trainer TrainerConfig TrainingHistory Model ModelBuilder ModelSerializer ModelComparator Config "
             "Profiler get_system_info set_seed cuda_is_available DistributedDataParallel DistributedConfig DistributedBackend "
             "DistributedSampler init_distributed get_world_size get_rank is_master cleanup_distributed Plotter ModelVisualizer "
             "TensorStats Sequential Module Parameter").split()
    missing = [n for n in names if not hasattr(rt, n)]
    assert not missing, missing
    import torch
    x = torch.tensor([-1.0, 0.5])
    assert torch.equal(rt.relu(x), torch.tensor([0.0, 0.5])) and abs(float(rt.softmax(x).sum()) - 1.0) < 1e-6


def test_compat_extra_objects(tmp_path):
    import torch
    import rustorch_b200 as rt
    a, b = torch.randn(3, 4, requires_grad=True), torch.randn(4, 5, requires_grad=True)
    g = torch.randn(3, 5)
    (a @ b).backward(g)
    ga, gb = rt.MatMulBackward(a.detach(), b.detach()).apply(g)
    assert torch.allclose(ga, a.grad) and torch.allclose(gb, b.grad)
    x, y = torch.randn(3, 4), torch.randn(1, 4)
    gx, gy = rt.MulBackward(x, y).apply(torch.ones(3, 4))
    assert gx.shape == x.shape and gy.shape == y.shape and torch.allclose(gy, x.sum(0, keepdim=True))
    assert torch.allclose(rt.MeanBackward(x).apply(torch.tensor(1.0))[0], torch.full_like(x, 1 / 12))
    # state dicts
    m = torch.nn.Sequential(torch.nn.Linear(4, 3), torch.nn.BatchNorm1d(3))
    sd = rt.StateDict.from_module(m)
    assert "1.running_mean" in sd.buffers and sd.tensor_metadata()["0.weight"].shape == [3, 4]
    path = str(tmp_path / "sd.rustorch")
    sd.save(path)
    back = rt.StateDict.load(path)
    assert torch.equal(back.parameters["0.weight"], sd.parameters["0.weight"]) and torch.equal(back.buffers["1.running_var"], sd.buffers["1.running_var"])
    msd = rt.ModelStateDict.from_module(m)
    assert torch.allclose(msd.to_tensors()["0.bias"], m[0].bias.detach())
    # generic Adam family
    p = torch.nn.Parameter(torch.ones(4))
    opt = rt.GenericAdamOptimizer([p], rt.AdamVariant.RADAM, lr=0.1)
    p.grad = torch.ones(4)
    opt.step()
    assert type(opt).__name__ == "RAdam" and float(p.detach().sum()) < 4.0
    assert abs(rt.CommonOps.bias_correction(0.9, 2) - 0.19) < 1e-12
    # gradient compression
    grad = torch.randn(1000)
    topk = rt.GradientCompression.TOP_K.compressor(ratio=0.1).compress_decompress(grad)
    assert int((topk != 0).sum()) == 100 and torch.equal(topk[topk != 0], grad[topk != 0])
    q = rt.GradientCompression.QUANTIZATION.compressor(bits=8).compress_decompress(grad)
    assert float((q - grad).abs().max()) < float(grad.abs().max()) / 100
    assert int((rt.GradientCompression.RANDOM.compressor(ratio=0.05).compress_decompress(grad) != 0).sum()) == 50
    # device helpers on CPU
    buf = rt.GpuBuffer.from_host([1.0, 2.0, 3.0], device="cpu")
    assert len(buf) == 3 and not buf.is_cuda() and buf.to_host().tolist() == [1.0, 2.0, 3.0]
    assert torch.allclose(rt.CudaBlas.gemm(x, y.t().contiguous()), x @ y.t())
    dense = torch.tensor([[1.0, 0.0, 2.0], [0.0, 3.0, 0.0]])
    csr = dense.to_sparse_csr()
    v = torch.tensor([1.0, 1.0, 1.0])
    assert torch.allclose(rt.CudaSparseOps.spmv(csr.crow_indices(), csr.col_indices(), csr.values(), v, 2), dense @ v)
    assert torch.equal(rt.GpuActivation.relu(torch.tensor([-1.0, 2.0])), torch.tensor([0.0, 2.0]))
    assert rt.GpuBatchMatrixExecutor("cpu").batch_matmul(torch.randn(2, 3, 4), torch.randn(2, 4, 5)).shape == (2, 3, 5)
    mgr = rt.CommunicationManager()
    mgr.schedule(rt.CommunicationOp.ALL_REDUCE, torch.ones(2))
    assert mgr.execute_all()[0].tolist() == [1.0, 1.0] and mgr.completed == 1


def test_named_call_sites_of_the_reference(tmp_path):
    import torch
    import rustorch_b200 as rt
    from rustorch_b200 import quantization, vision
    from rustorch_b200.distributed import multi_gpu as mg
    ts = [torch.full((8,), float(i + 1)) for i in range(4)]
    assert all(torch.allclose(t, torch.full((8,), 10.0)) for t in mg.p2p_all_reduce([t.clone() for t in ts]))
    assert all(torch.allclose(t, torch.full((8,), 2.5)) for t in mg.host_staged_all_reduce([t.clone() for t in ts]))
    assert all(torch.allclose(t, torch.full((8,), 2.5)) for t in mg.NCCLOps.all_reduce_multi_gpu([t.clone() for t in ts]))
    assert torch.equal(mg.nccl_all_reduce(torch.ones(3)), torch.ones(3))                  # no process group: identity
    assert len(mg.NCCLOps.init_multi_gpu([0]).device_ids) == 1
    grid = vision.make_grid(torch.rand(5, 3, 4, 4), nrow=3, padding=1)
    assert grid.shape == (3, 2 * 5 + 1, 3 * 5 + 1)
    png = str(tmp_path / "g.png")
    vision.save_image(torch.rand(5, 3, 4, 4), png, nrow=3, padding=1)
    assert open(png, "rb").read(4)[1:] == b"PNG"
    assert rt.get_compute_capability() == (0, 0) or rt.get_compute_capability()[0] >= 7
    q, k, v = (torch.randn(1, 2, 5, 8) for _ in range(3))
    ref = torch.softmax(q @ k.transpose(-1, -2) / 8 ** 0.5, -1) @ v
    assert torch.allclose(rt.execute_attention(q, k, v), ref, atol=1e-5)
    assert hasattr(quantization, "qmatmul_cuda") and hasattr(quantization, "qconv2d_cuda")
    assert rt.GpuBatchMatrixExecutor("cpu").cuda_batch_matmul(torch.randn(2, 3, 4), torch.randn(2, 4, 5)).shape == (2, 3, 5)
