"""Tensor façade, dtype and autograd surface (CPU)."""
import math

import numpy as np
import pytest
import torch

from rustorch_b200.autograd import (ComputationGraph, AddFunction, MulFunction, MatMulFunction, SumFunction,
                                    GradCheckConfig, GradientFlowAnalyzer, GradientFlowVisualizer, Variable,
                                    grad, gradcheck, hessian, hvp, jacobian, no_grad)
from rustorch_b200.dtype import DType, parse_dtype
from rustorch_b200.tensor import Device, Tensor, tensor


def test_constructors_and_accessors():
    t = Tensor.from_vec([1, 2, 3, 4, 5, 6], [2, 3])
    assert t.shape() == (2, 3) and t.ndim() == 2 and t.numel() == 6
    assert t.get([1, 2]) == 6.0
    t.set([0, 0], 9.0)
    assert t.as_slice()[0] == 9.0
    assert Tensor.zeros([2, 2]).sum().item() == 0 and Tensor.ones([2, 2]).sum().item() == 4
    assert Tensor.full([3], 2.5).mean().item() == 2.5
    assert Tensor.eye(3).trace() == 3.0
    assert Tensor.arange(5).shape() == (5,) and Tensor.linspace(0, 1, 11).shape() == (11,)
    with pytest.raises(ValueError):
        Tensor.from_vec([1, 2, 3], [2, 2])
    assert str(Device.cuda(1)) == "cuda:1" and str(t.device()) == "cpu"


def test_arithmetic_matmul_broadcast():
    a = tensor([[1.0, 2.0], [3.0, 4.0]])
    b = tensor([[5.0, 6.0], [7.0, 8.0]])
    assert (a + b).as_slice() == [6, 8, 10, 12]
    assert (a * 2.0).as_slice() == [2, 4, 6, 8]
    assert a.matmul(b).as_slice() == [19, 22, 43, 50]
    assert (a @ tensor([1.0, 1.0])).as_slice() == [3, 7]
    assert a.transpose().as_slice() == [1, 3, 2, 4]
    assert abs(a.det() + 2.0) < 1e-5
    assert (a + tensor([10.0, 20.0])).as_slice() == [11, 22, 13, 24]
    assert a.maximum(tensor([[2.0, 2.0], [2.0, 2.0]])).as_slice() == [2, 2, 3, 4]


def test_math_reductions_shape_ops():
    x = tensor([[1.0, -2.0, 3.0], [4.0, 5.0, -6.0]])
    assert x.abs().sum().item() == 21
    assert x.argmax() == 4 and x.argmin() == 5
    assert x.sum_axis(0).as_slice() == [5, 3, -3]
    assert x.clamp(-1, 1).as_slice() == [1, -1, 1, 1, 1, -1]
    assert x.flatten().shape() == (6,) and x.unsqueeze(0).shape() == (1, 2, 3)
    assert x.flip([1]).as_slice()[:3] == [3, -2, 1]
    assert Tensor.stack([x, x]).shape() == (2, 2, 3) and Tensor.concatenate([x, x], 1).shape() == (2, 6)
    v, i = x.topk(2, dim=1)
    assert v.as_slice() == [3, 1, 5, 4]
    assert abs(tensor([1.0, 2.0, 3.0, 4.0]).var_unbiased().item() - 1.6666666) < 1e-5
    assert tensor([0.5]).gamma().as_slice()[0] == pytest.approx(math.sqrt(math.pi), rel=1e-5)
    assert tensor([1.0, float("nan")]).has_nan() and not tensor([1.0]).has_inf()
    assert x.exp().shape() == (2, 3)  # falls through to torch
    assert x.map(lambda v: v * 2).as_slice() == [2, -4, 6, 8, 10, -12]


def test_linalg_and_fft():
    a = tensor([[4.0, 1.0], [1.0, 3.0]])
    u, s, v = a.svd()
    rec = u.data @ torch.diag(s.data) @ v.data.t()
    assert torch.allclose(rec, a.data, atol=1e-5)
    q, r = a.qr()
    assert torch.allclose(q.data @ r.data, a.data, atol=1e-5)
    assert torch.allclose(a.inverse().data @ a.data, torch.eye(2), atol=1e-5)
    L = a.cholesky()
    assert torch.allclose(L.data @ L.data.t(), a.data, atol=1e-5)
    sig = Tensor.arange(8)
    assert torch.allclose(sig.fft().ifft().data.real, sig.data, atol=1e-5)
    assert sig.apply_window("hamming").shape() == (8,)


def test_dtype():
    assert parse_dtype("float32") is DType.F32 and DType.BF16.size() == 2
    assert DType.F16.promote(DType.F32) is DType.F32
    assert DType.I32.is_int() and DType.C64.is_complex()
    with pytest.raises(ValueError):
        parse_dtype("q7")


def test_variable_backward_and_hooks():
    x = Variable(tensor([[1.0, 2.0], [3.0, 4.0]]), requires_grad=True)
    w = Variable(tensor([[0.5], [0.25]]), requires_grad=True)
    y = (x.matmul(w) * 2.0).sum()
    y.backward()
    assert x.grad().as_slice() == [1.0, 0.5, 1.0, 0.5]
    assert w.grad().as_slice() == [8.0, 12.0]
    x.zero_grad()
    assert x.grad is None
    with no_grad():
        z = x * 2.0
    assert not z.requires_grad()
    (gx,) = grad([(x * x).sum()], [x])
    assert gx.as_slice() == [2, 4, 6, 8]
    assert x.exp().shape() == (2, 2)


def test_gradcheck_and_higher_order():
    f = lambda v: (v * v * v).sum()
    assert gradcheck(f, [tensor([1.0, 2.0])], GradCheckConfig(eps=1e-6, atol=1e-4, rtol=1e-3))
    H = hessian(f, tensor([1.0, 2.0]))
    assert torch.allclose(H.data, torch.tensor([[6.0, 0.0], [0.0, 12.0]]), atol=1e-2)
    J = jacobian(lambda v: v * v, tensor([1.0, 3.0]))
    assert torch.allclose(J.data, torch.tensor([[2.0, 0.0], [0.0, 6.0]]), atol=1e-3)
    hv = hvp(f, tensor([1.0, 2.0]), tensor([1.0, 1.0]))
    assert torch.allclose(hv.data, torch.tensor([6.0, 12.0]), atol=1e-2)


def test_computation_graph_topological_backward():
    g = ComputationGraph()
    a = g.add_leaf(torch.tensor([[1.0, 2.0]]))
    b = g.add_leaf(torch.tensor([[3.0], [4.0]]))
    c = g.add_node(MatMulFunction(), [a, b])
    d = g.add_node(MulFunction(), [c, c])       # shared sub-graph: c used twice
    e = g.add_node(SumFunction(), [d])
    g.backward(e)
    assert g.value(e).item() == 121.0
    assert g.grad(a).as_slice() == [66.0, 88.0]
    assert g.topological_sort().index(c) < g.topological_sort().index(d)


def test_gradient_flow_tools(tmp_path):
    x = Variable(tensor([1.0, 2.0]), requires_grad=True)
    y = (x * x).sum()
    dot = GradientFlowVisualizer().to_dot(y)
    assert "digraph" in dot and "MulBackward" in dot
    lin = torch.nn.Linear(2, 1)
    lin(torch.ones(1, 2)).sum().backward()
    an = GradientFlowAnalyzer()
    an.record(lin.named_parameters())
    assert "weight" in an.history and an.issues() == {}


def test_tensor_shape_device_and_predicate_helpers():
    """src/tensor/core.rs:436-445, ops/shape_operations.rs, ops/advanced_shape.rs, ops/utils.rs:28-140."""
    from rustorch_b200.tensor import Tensor
    t = Tensor(torch.arange(24.0).view(2, 3, 4))
    assert t.resolve_dim(-1) == 2 and t.resolve_dim(0) == 0
    with pytest.raises(IndexError):
        t.resolve_dim(3)
    assert t.to_cpu().device_type() == "cpu" and not t.is_on_gpu() and t.batch_size() == 2 and t.as_ptr() == t.data.data_ptr()
    assert t.with_device("cpu").shape == (2, 3, 4) and t.clone_to_device("cpu").as_ptr() != t.as_ptr()
    md = t.get_metadata()
    assert md == {"shape": "[2, 3, 4]", "dtype": "float32", "device": "cpu", "numel": "24", "requires_grad": "false"}
    g = Tensor(torch.ones(3), requires_grad=True)
    (g.data * 2).sum().backward()
    c = g.clone_with_grad()
    assert c.requires_grad and torch.equal(c.data.grad, g.data.grad) and c.data.grad is not g.data.grad
    assert t.can_broadcast_with(Tensor(torch.ones(3, 1))) and t.can_broadcast_with(Tensor(torch.ones(4)))
    assert not t.can_broadcast_with(Tensor(torch.ones(3)))
    u = Tensor(torch.zeros(1, 3, 1))
    assert u.squeeze_dim(0).shape == (3, 1) and u.squeeze_dim(-1).shape == (1, 3) and u.squeeze_all().shape == (3,)
    with pytest.raises(ValueError):
        u.squeeze_dim(1)
    assert Tensor(torch.zeros(3)).unsqueeze_multiple([0, 2]).shape == (1, 3, 1) and Tensor(torch.zeros(3)).expand_dims(1).shape == (3, 1)
    with pytest.raises(IndexError):
        Tensor(torch.zeros(3)).unsqueeze_multiple([3])
    assert t.flatten_from(1).shape == (2, 12) and t.flatten_range(0, 1).shape == (6, 4) and t.flatten_view().shape == (24,)
    with pytest.raises(IndexError):
        t.flatten_range(2, 1)
    o = t.flatten_owned()
    assert o.as_ptr() != t.as_ptr() and t.flatten_view().as_ptr() == t.as_ptr()
    v = Tensor(torch.zeros(2, 1))
    sh = v.expand_shared([2, 5])
    assert sh.data.stride() == (1, 0) and v.expand_owned([2, 5]).data.is_contiguous() and sh.materialize().data.is_contiguous()
    assert Tensor(torch.zeros(2, 3)).repeat_advanced([2, 1, 2]).shape == (2, 2, 6)
    with pytest.raises(ValueError):
        Tensor(torch.zeros(2, 3)).repeat_advanced([2])
    r = Tensor([1.0, 2.0, 3.0, 4.0])
    assert r.roll_1d(1, 0).as_slice() == [4.0, 1.0, 2.0, 3.0] and r.repeat_interleave_scalar(2, 0).shape == (8,)
    assert Tensor(torch.arange(6.0).view(2, 3)).roll_1d(1).as_slice() == [5.0, 0.0, 1.0, 2.0, 3.0, 4.0]
    m = Tensor(torch.arange(6.0).view(2, 3))
    m.unsqueeze_inplace(0)
    assert m.shape == (1, 2, 3)
    m.squeeze_inplace()
    m.flatten_inplace()
    assert m.shape == (6,)
    assert r.std_unbiased() == pytest.approx(1.2909944, rel=1e-6) and r.quantile_advanced(0.5) == 2.5
    with pytest.raises(ValueError):
        r.quantile_advanced(1.5)
    z = Tensor(torch.tensor([[0.0, 1.0, 2.0], [0.0, 0.0, 3.0]]))
    assert z.count_nonzero_axis(0).as_slice() == [0.0, 1.0, 2.0] and z.count_nonzero_axis(-1).as_slice() == [2.0, 1.0]
    q, rr = Tensor(torch.randn(4, 3)).qr_basic()
    assert q.shape == (4, 3) and rr.shape == (3, 3)
    w, _ = Tensor(torch.eye(3) * 2).symeig_basic()
    assert w.as_slice() == [2.0, 2.0, 2.0]
    assert Tensor(torch.eye(2)).matmul_hybrid(Tensor([[1.0, 2.0], [3.0, 4.0]])).as_slice() == [1.0, 2.0, 3.0, 4.0]
    # predicates: a whole-tensor mask function or an element-wise Python predicate
    assert r.count_where(lambda x: x > 2) == 2 and r.count_where(lambda x: 1.5 < x < 3.5) == 2
    assert r.find_first(lambda x: x > 2) == 2 and r.find_first(lambda x: x > 9) is None and r.find_all(lambda x: x % 2 == 0) == [1, 3]
    assert r.replace_where(lambda x: x > 2, 0.0).as_slice() == [1.0, 2.0, 0.0, 0.0]
    assert r.map_with_index(lambda i, x: x * i).as_slice() == [0.0, 2.0, 6.0, 12.0]
    k = r.clone_tensor()
    k.map_inplace(lambda x: x + 1)
    assert k.as_slice() == [2.0, 3.0, 4.0, 5.0] and r.as_slice() == [1.0, 2.0, 3.0, 4.0]


def test_wrapper_protocols_numpy_iteration_comparison():
    import numpy as np
    import rustorch as rt
    a = rt.tensor([[1.0, 2.0], [3.0, 4.0]])
    assert np.asarray(a).dtype == np.float32 and np.asarray(a).shape == (2, 2) and np.asarray(a, dtype=np.float64).dtype == np.float64
    assert np.asarray(rt.Variable(a)).tolist() == [[1.0, 2.0], [3.0, 4.0]]
    assert (a != rt.tensor([[1.0, 0.0], [3.0, 0.0]])).data.tolist() == [[False, True], [False, True]]
    assert [r.as_slice() for r in a] == [[1.0, 2.0], [3.0, 4.0]] and len({a: 1}) == 1
    with pytest.raises(TypeError):
        iter(rt.tensor(3.0).reshape([]))
    v = rt.Variable(a, requires_grad=True)
    assert len(v) == 2 and isinstance(v[0], rt.Variable)
    v[1].sum().backward()
    assert v.grad.as_slice() == [0.0, 0.0, 1.0, 1.0]
    assert isinstance(torch.ones(2, 2) + a, rt.Tensor) and isinstance(torch.ones(2, 2) * v, rt.Variable)


def test_gradient_context_and_anomaly_guard():
    """src/autograd/context.rs:10-155: the two thread-local flags, their guards, and what anomaly detection does."""
    from rustorch_b200 import autograd as A
    ctx = A.GradientContext.current()
    assert ctx.grad_enabled and not ctx.anomaly_detection and "grad_enabled=True" in repr(ctx)
    with A.NoGradGuard():
        assert not ctx.grad_enabled
        with A.EnableGradGuard():
            assert A.is_grad_enabled()
        assert not A.is_grad_enabled()
    ctx.grad_enabled = False
    assert not torch.is_grad_enabled()
    ctx.grad_enabled = True
    x = torch.tensor([0.0], requires_grad=True)
    torch.sqrt(x).sum().backward()                                    # silently produces inf without the guard
    assert torch.isinf(x.grad).all()
    with A.AnomalyDetectionGuard():
        assert A.is_anomaly_detection_enabled() and ctx.anomaly_detection
        y = torch.tensor([0.0], requires_grad=True)
        with pytest.raises(RuntimeError, match="nan"):
            (torch.sqrt(y) * 0.0).sum().backward()                    # 0 * inf = nan in the backward pass
    assert not A.is_anomaly_detection_enabled()
    A.set_anomaly_detection(True)
    assert ctx.anomaly_detection
    A.set_anomaly_detection(False)
