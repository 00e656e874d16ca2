"""Train a small Llama-style model, write it as a Hugging Face checkpoint, convert that to a quantised GGUF file and serve
it with the decode runtime: the training model and the runtime are two implementations of the same network, so the
runtime's greedy continuation follows the pattern the model was trained on."""
import _path  # noqa: F401
import os
import tempfile

import torch

from rustorch_b200 import llm
from rustorch_b200.formats import gguf
from rustorch_b200.models.llama import LlamaModel, LlamaTrainConfig

torch.manual_seed(0)
cfg = LlamaTrainConfig.tiny(vocab_size=64, n_layer=2, n_embd=64, n_head=4, n_head_kv=2, n_ff=128, max_seq_len=64)
model = LlamaModel(cfg)
opt = torch.optim.AdamW(model.parameters(), lr=3e-3)
period = 7


def batch(n=32, T=24):
    start = torch.randint(0, cfg.vocab_size, (n, 1))
    seq = (start + torch.arange(T + 1)[None, :] * period) % cfg.vocab_size      # token t+1 = token t + 7 (mod 64)
    return seq[:, :-1], seq[:, 1:]


for step in range(300):
    x, y = batch()
    _, loss = model(x, y)
    opt.zero_grad()
    loss.backward()
    opt.step()
    if step % 100 == 99:
        print(f"step {step + 1}: loss {float(loss.detach()):.4f}")
out = tempfile.mkdtemp()
hf_dir, gguf_path = os.path.join(out, "hf"), os.path.join(out, "model.q8_0.gguf")
model.save_hf(hf_dir)
info = llm.hf_to_gguf(hf_dir, gguf_path, gguf.GGMLType.Q8_0)
print("checkpoint:", sorted(os.listdir(hf_dir)), "-> GGUF with", info["tensors"], "tensors,", info["bytes"], "bytes")
device = "cuda" if torch.cuda.is_available() else "cpu"
rt = llm.LlamaRuntime.from_gguf(gguf_path, device=device)
prompt = torch.tensor([[3, 10, 17, 24]], device=device)
tokens, stats = rt.generate(prompt, 8)
want = [(24 + period * (i + 1)) % cfg.vocab_size for i in range(8)]
print("prompt", prompt[0].tolist(), "-> generated", tokens[0, 4:].tolist(), "(pattern:", want, ")")
print("decode: %.0f tokens/s on %s" % (stats["decode_tokens_per_s"], device))
