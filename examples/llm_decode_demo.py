"""The LLM runtime end to end on a toy model: write a GGUF file with Q4_0 / Q8_0 blocks, load it (weights stay
quantised), prefill + cached decode, sampling settings, throughput metrics.  On a GPU the same calls run the
dequant-fused kernels and replay one CUDA graph per token."""
import _path  # noqa: F401
import os
import tempfile

import torch

from rustorch_b200 import llm
from rustorch_b200.formats import gguf

cfg = llm.LlamaConfig(vocab_size=96, n_layer=2, n_embd=64, n_head=4, n_head_kv=2, n_ff=128, context_length=128)
g = torch.Generator().manual_seed(0)
rnd = lambda *s: torch.randn(*s, generator=g) * 0.05      # noqa: E731
hd = cfg.head_dim
tensors = {"token_embd.weight": (rnd(96, 64), gguf.GGMLType.F16), "output_norm.weight": (torch.ones(64), gguf.GGMLType.F32),
           "output.weight": (rnd(96, 64), gguf.GGMLType.Q8_0)}
for i in range(cfg.n_layer):
    p = f"blk.{i}."
    tensors.update({p + "attn_q.weight": (rnd(4 * hd, 64), gguf.GGMLType.Q4_0), p + "attn_k.weight": (rnd(2 * hd, 64), gguf.GGMLType.Q4_0),
                    p + "attn_v.weight": (rnd(2 * hd, 64), gguf.GGMLType.Q4_0), p + "attn_output.weight": (rnd(64, 64), gguf.GGMLType.Q4_0),
                    p + "ffn_gate.weight": (rnd(128, 64), gguf.GGMLType.Q4_0), p + "ffn_up.weight": (rnd(128, 64), gguf.GGMLType.Q4_0),
                    p + "ffn_down.weight": (rnd(64, 128), gguf.GGMLType.Q4_0), p + "attn_norm.weight": (torch.ones(64), gguf.GGMLType.F32),
                    p + "ffn_norm.weight": (torch.ones(64), gguf.GGMLType.F32)})
md = {"general.architecture": "llama", "llama.block_count": 2, "llama.embedding_length": 64, "llama.feed_forward_length": 128,
      "llama.attention.head_count": 4, "llama.attention.head_count_kv": 2, "llama.rope.freq_base": 10000.0,
      "llama.attention.layer_norm_rms_epsilon": 1e-5, "llama.context_length": 128, "llama.vocab_size": 96}
path = os.path.join(tempfile.mkdtemp(), "toy.gguf")
gguf.write_gguf(path, md, tensors)
device = "cuda" if torch.cuda.is_available() else "cpu"
rt = llm.LlamaRuntime.from_gguf(path, device=device)
print(f"loaded {os.path.getsize(path)} bytes: {len(rt.layers)} layers, {rt.cfg.n_head} heads ({rt.cfg.n_head_kv} kv), device {device}")
prompt = torch.randint(0, 96, (1, 12), generator=g).to(device)
greedy, stats = rt.generate(prompt, 16)
print("greedy continuation:", greedy[0, 12:].tolist())
print("stats:", {k: (round(v, 2) if isinstance(v, float) else v) for k, v in stats.items()})
cache = rt.new_cache(1, 64)
logits = rt.prefill(greedy[:, :20], cache)
print("cached decode equals recomputing the prefix:", int(logits.argmax(-1)) == int(greedy[0, 20]))
sampler = llm.Sampler(llm.SamplingConfig(temperature=0.8, top_k=20, top_p=0.95, seed=1))
print("sampled tokens:", [int(sampler(logits.float().cpu())[0]) for _ in range(8)])
