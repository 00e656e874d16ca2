"""GPT-2-style language model: a few AdamW steps on random tokens, then greedy generation.  On a B200 the blocks run
on the fused tcgen05 kernels (GEMM + bias/GELU epilogues, flash attention, fused LayerNorm and cross-entropy)."""
import _path  # noqa: F401
import torch

from rustorch_b200 import optim
from rustorch_b200.models.gpt import GPT, GPTConfig

dev = "cuda" if torch.cuda.is_available() else "cpu"
torch.manual_seed(0)
cfg = GPTConfig(vocab_size=512, n_positions=128, n_embd=128, n_layer=2, n_head=4, dropout=0.0)
model = GPT(cfg).to(dev)
if dev == "cuda":
    model = model.to(torch.bfloat16)
opt = optim.AdamW(model.parameters(), lr=3e-3, betas=(0.9, 0.95), weight_decay=0.1)
tokens = torch.randint(0, cfg.vocab_size, (8, 128), device=dev)
for step in range(10):
    opt.zero_grad()
    out = model(tokens, tokens.roll(-1, 1))
    loss = out[1] if isinstance(out, tuple) else out
    loss.backward()
    opt.step()
    print(f"step {step}: loss {float(loss):.4f}")
model.eval()
with torch.no_grad():
    print("generated:", model.generate(tokens[:1, :8], 8, temperature=0.0)[0].tolist())
