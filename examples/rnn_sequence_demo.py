"""Recurrent layers: an LSTM that learns to sum a sequence, a bidirectional GRU tagger's shapes, and one LSTM step
written out with the cell-level helpers."""
import _path  # noqa: F401

import torch

from rustorch_b200 import nn

torch.manual_seed(0)


class Summer(torch.nn.Module):
    def __init__(self):
        super().__init__()
        self.rnn = nn.LSTM(1, 24, batch_first=True)
        self.head = nn.Linear(24, 1)

    def forward(self, x):
        out, (h, c) = self.rnn(x)
        return self.head(h[-1])


net = Summer()
opt = torch.optim.Adam(net.parameters(), 0.01)
for step in range(800):
    x = torch.rand(64, 10, 1)
    opt.zero_grad()
    loss = torch.nn.functional.mse_loss(net(x), x.sum(1))
    loss.backward()
    opt.step()
test = torch.rand(4, 10, 1)
print("LSTM sums sequences: predicted", [round(v, 2) for v in net(test).flatten().tolist()], "true", [round(v, 2) for v in test.sum(1).flatten().tolist()])
gru = nn.GRU(8, 16, num_layers=2, batch_first=True, bidirectional=True)
out, h = gru(torch.randn(3, 7, 8))
print("2-layer bidirectional GRU: outputs", tuple(out.shape), "final states", tuple(h.shape))
cell = nn.LSTMCell(4, 6)
x, h0, c0 = torch.randn(2, 4), torch.zeros(2, 6), torch.zeros(2, 6)
gates = nn.RecurrentOps.linear_transform(x, cell.weight_ih, cell.bias_ih) + nn.RecurrentOps.linear_transform(h0, cell.weight_hh, cell.bias_hh)
i, f, g, o = (nn.RecurrentOps.slice_gates(gates, k, 6) for k in range(4))
c1 = torch.sigmoid(f) * c0 + torch.sigmoid(i) * torch.tanh(g)
h1 = torch.sigmoid(o) * torch.tanh(c1)
hr, cr = cell(x, (h0, c0))
print("cell written out with RecurrentOps equals LSTMCell:", bool(torch.allclose(h1, hr, atol=1e-6) and torch.allclose(c1, cr, atol=1e-6)))
