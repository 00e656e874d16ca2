"""Embedding tables: lookup, padding index, frozen tables, learned and sinusoidal positions."""
import _path  # noqa: F401

import torch

from rustorch_b200 import nn

torch.manual_seed(0)
emb = nn.Embedding(10, 4, padding_idx=0)
ids = torch.tensor([[1, 2, 0], [3, 0, 0]])
out = emb(ids)
print("lookup", tuple(out.shape), " padding rows are zero:", bool((out[ids == 0] == 0).all()))
out.sum().backward()
print("rows with gradient:", emb.weight.grad.abs().sum(1).nonzero().flatten().tolist(), "(the padding row 0 gets none)")
frozen = nn.Embedding(10, 4, freeze=True)
print("frozen table requires_grad:", frozen.weight.requires_grad)
pos = nn.PositionalEmbedding(16, 4)
sin = nn.SinusoidalPositionalEncoding(16, 4)
x = torch.zeros(2, 5, 4)
print("learned positions:", tuple(pos(x).shape), " sinusoidal row 1:", [round(v, 3) for v in sin(x)[0, 1].tolist()])
pe = nn.PositionalEncoding(4, max_len=32)
print("PositionalEncoding adds to the input:", bool(torch.allclose(pe(x)[0, 0], torch.tensor([0.0, 1.0, 0.0, 1.0]))))
