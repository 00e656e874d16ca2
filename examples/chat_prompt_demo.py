"""Chat plumbing of the command-line program without a model file: a byte-level BPE tokenizer built in memory, the
prompt layouts of the model families, detection of the layout from the tokenizer's marker tokens, turn-end stop tokens,
and key / value cached decoding of a small GPT through the same engine the program uses."""
import _path  # noqa: F401
import torch

from rustorch_b200.cli.engine import InferenceEngine, _GPTAdapter
from rustorch_b200.cli.session import TURN_END_TOKENS, GenerationConfig, SessionManager, detect_chat_template
from rustorch_b200.cli.tokenizer import BPETokenizer, _byte_alphabet
from rustorch_b200.models.gpt import GPT, GPTConfig

# ---- a tokenizer: the 256 byte symbols, two merges, and the markers of the ChatML layout as added tokens
alphabet = _byte_alphabet()
vocab = {ch: i for i, ch in enumerate(alphabet[b] for b in range(256))}
space = alphabet[ord(" ")]
merges = [("h", "i"), (space, "t"), (space + "t", "h")]
for a, b in merges:
    vocab[a + b] = len(vocab)
added = {"<|im_start|>": len(vocab), "<|im_end|>": len(vocab) + 1}
tok = BPETokenizer(vocab, merges, eos_token="<|im_end|>", added_tokens=added)
ids = tok.encode("hi there<|im_end|>")
print("ids:", ids, "->", repr(tok.decode(ids)), "| with markers:", repr(tok.decode(ids, skip_special=False)))
assert tok.decode(ids) == "hi there" and ids[-1] == added["<|im_end|>"] and ids[0] == vocab["hi"]

# ---- the same conversation in the four layouts
session = SessionManager()
session.set_system_prompt("Answer in one word.")
session.add_user_message("Capital of France?")
session.add_assistant_message("Paris")
session.add_user_message("Of Italy?")
for name in ("plain", "llama3", "chatml", "llama2"):
    session.set_chat_template(name)
    print(f"--- {name}\n{session.build_prompt()}")
layout = detect_chat_template(tok)
print("layout that this tokenizer points to:", layout)
assert layout == "chatml"
session.set_chat_template(layout)

# ---- generation through the program's engine: a small random GPT, cached decode, stop at the turn-end marker
model = GPT(GPTConfig(vocab_size=tok.vocab_size, n_positions=128, n_embd=64, n_layer=2, n_head=4, dropout=0.0), seed=0)
engine = InferenceEngine(_GPTAdapter(model, "cpu"), tok, GenerationConfig(max_tokens=12, temperature=0.8, top_k=40), "cpu", seed=0)
engine.set_stop_tokens(TURN_END_TOKENS[layout])
reply = engine.generate(session.build_prompt())
print(f"reply of the untrained model ({engine.last_token_count} tokens):", repr(reply))
with torch.no_grad():
    full = model.forward_reference(torch.tensor([tok.encode("hi there")]))
step, _ = model.forward_cached(torch.tensor([tok.encode("hi there")]))
assert torch.allclose(full, step, atol=1e-5)
print("cached and whole-sequence logits agree:", float((full - step).abs().max()))
