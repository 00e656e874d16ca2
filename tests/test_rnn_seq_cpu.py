"""Whole-sequence RNN / LSTM / GRU (rustorch_b200/ops/rnn_seq.py) against torch.nn on the CPU: forward values, final
states and every gradient, for multi-layer, bidirectional, batch_first, with and without bias and initial state."""
import pytest
import torch

from rustorch_b200 import nn as rnn


def _pair(kind, **kw):
    torch.manual_seed(0)
    ours = getattr(rnn, kind)(10, 12, **kw).double()
    ref = getattr(torch.nn, kind)(10, 12, **kw).double()
    assert set(ours.state_dict()) == set(ref.state_dict())
    ref.load_state_dict(ours.state_dict())
    return ours, ref


CASES = [dict(), dict(num_layers=2, bidirectional=True), dict(batch_first=True, bias=False), dict(num_layers=3, bidirectional=True, batch_first=True)]


@pytest.mark.parametrize("kind", ["LSTM", "GRU", "RNN"])
@pytest.mark.parametrize("kw", CASES)
@pytest.mark.parametrize("with_state", [False, True])
def test_sequence_layers_match_torch(kind, kw, with_state):
    ours, ref = _pair(kind, **kw)
    g = torch.Generator().manual_seed(1)
    B, T = 3, 7
    x = torch.randn((B, T, 10) if kw.get("batch_first") else (T, B, 10), generator=g, dtype=torch.float64)
    n = kw.get("num_layers", 1) * (2 if kw.get("bidirectional") else 1)
    hx = None
    if with_state:
        h0 = torch.randn(n, B, 12, generator=g, dtype=torch.float64)
        hx = (h0, torch.randn(n, B, 12, generator=g, dtype=torch.float64)) if kind == "LSTM" else h0
    xs = [x.clone().requires_grad_(True) for _ in range(2)]
    hxs = []
    for _ in range(2):
        if hx is None:
            hxs.append(None)
        elif kind == "LSTM":
            hxs.append(tuple(t.clone().requires_grad_(True) for t in hx))
        else:
            hxs.append(hx.clone().requires_grad_(True))
    o1, s1 = ours(xs[0], hxs[0])
    o2, s2 = ref(xs[1], hxs[1])
    torch.testing.assert_close(o1, o2, rtol=1e-9, atol=1e-10)
    s1 = s1 if isinstance(s1, tuple) else (s1,)
    s2 = s2 if isinstance(s2, tuple) else (s2,)
    for a, b in zip(s1, s2):
        torch.testing.assert_close(a, b, rtol=1e-9, atol=1e-10)
    w = torch.randn(o1.shape, generator=g, dtype=torch.float64)
    ws = [torch.randn(a.shape, generator=g, dtype=torch.float64) for a in s1]
    (o1 * w).sum().add(sum((a * b).sum() for a, b in zip(s1, ws))).backward()
    (o2 * w).sum().add(sum((a * b).sum() for a, b in zip(s2, ws))).backward()
    torch.testing.assert_close(xs[0].grad, xs[1].grad, rtol=1e-8, atol=1e-10)
    for (k, p), (_, q) in zip(sorted(ours.named_parameters()), sorted(ref.named_parameters())):
        torch.testing.assert_close(p.grad, q.grad, rtol=1e-8, atol=1e-10, msg=lambda m, k=k: f"{k}: {m}")
    if hx is not None:
        a = hxs[0] if isinstance(hxs[0], tuple) else (hxs[0],)
        b = hxs[1] if isinstance(hxs[1], tuple) else (hxs[1],)
        for u, v in zip(a, b):
            torch.testing.assert_close(u.grad, v.grad, rtol=1e-8, atol=1e-10)


def test_relu_rnn_unbatched_and_state_dict_loads_from_torch():
    torch.manual_seed(3)
    ref = torch.nn.RNN(10, 12, nonlinearity="relu")
    ours = rnn.RNN(10, 12, nonlinearity="relu")
    ours.load_state_dict(ref.state_dict())
    x = torch.randn(5, 10)
    o1, h1 = ours(x)
    o2, h2 = ref(x)
    torch.testing.assert_close(o1, o2, rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(h1, h2, rtol=1e-5, atol=1e-6)
    lstm = rnn.LSTM(4, 6, num_layers=2, dropout=0.5)
    lstm.eval()
    a, _ = lstm(torch.ones(3, 2, 4))
    b, _ = lstm(torch.ones(3, 2, 4))
    assert torch.equal(a, b) and lstm.init_state(2)[0].shape == (2, 2, 6)
    assert not isinstance(lstm, torch.nn.LSTM)          # this package's own layer, not the cuDNN module
