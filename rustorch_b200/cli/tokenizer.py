"""Tokenizers for the CLI (example-cli/src/tokenizer/wrapper.rs:8-96 wraps the HF ``tokenizers`` crate or a dummy).

* ``GGUFTokenizer``: the SentencePiece-style vocabulary embedded in a GGUF file (``tokenizer.ggml.tokens`` /
  ``scores`` / ``token_type``): text is split into UTF-8 characters (spaces become U+2581), adjacent pieces are
  merged best-score-first while the merged piece exists in the vocabulary, unknown characters fall back to
  ``<0xXX>`` byte tokens.
* ``SentencePieceTokenizer``: a ``.model`` file through the ``sentencepiece`` package.
* ``ByteTokenizer``: 256 byte tokens + BOS/EOS, for models without a vocabulary (and for tests).
"""
from __future__ import annotations

import heapq
from typing import Dict, List, Optional, Sequence


class Tokenizer:
    bos_id: Optional[int] = None
    eos_id: Optional[int] = None

    def encode(self, text: str, add_bos: bool = True) -> List[int]:
        raise NotImplementedError

    def decode(self, ids: Sequence[int]) -> str:
        raise NotImplementedError

    @property
    def vocab_size(self) -> int:
        raise NotImplementedError


class ByteTokenizer(Tokenizer):
    def __init__(self, vocab_size: int = 258):
        self._n = max(258, vocab_size)
        self.bos_id, self.eos_id = 256, 257

    def encode(self, text, add_bos=True):
        return ([self.bos_id] if add_bos else []) + list(text.encode("utf-8"))

    def decode(self, ids):
        return bytes(i for i in ids if 0 <= i < 256).decode("utf-8", errors="replace")

    @property
    def vocab_size(self):
        return self._n


class GGUFTokenizer(Tokenizer):
    SPACE = "▁"

    def __init__(self, tokens: Sequence[str], scores: Optional[Sequence[float]] = None, token_types: Optional[Sequence[int]] = None,
                 bos_id: Optional[int] = 1, eos_id: Optional[int] = 2, unk_id: int = 0, add_space_prefix: bool = True):
        self.tokens = list(tokens)
        self.scores = list(scores) if scores is not None else [0.0] * len(self.tokens)
        self.types = list(token_types) if token_types is not None else [1] * len(self.tokens)
        self.index: Dict[str, int] = {}
        for i, t in enumerate(self.tokens):
            self.index.setdefault(t, i)
        self.bos_id, self.eos_id, self.unk_id, self.add_space_prefix = bos_id, eos_id, unk_id, add_space_prefix
        self.byte_ids = {b: self.index[f"<0x{b:02X}>"] for b in range(256) if f"<0x{b:02X}>" in self.index}

    @classmethod
    def from_gguf(cls, gguf_file) -> "GGUFTokenizer":
        md = gguf_file.metadata
        toks = md.get("tokenizer.ggml.tokens")
        if toks is None:
            raise KeyError("the GGUF file has no tokenizer.ggml.tokens")
        return cls(toks, md.get("tokenizer.ggml.scores"), md.get("tokenizer.ggml.token_type"),
                   md.get("tokenizer.ggml.bos_token_id", 1), md.get("tokenizer.ggml.eos_token_id", 2),
                   md.get("tokenizer.ggml.unknown_token_id", 0), bool(md.get("tokenizer.ggml.add_space_prefix", True)))

    @property
    def vocab_size(self):
        return len(self.tokens)

    def encode(self, text, add_bos=True):
        if self.add_space_prefix and text and not text.startswith(" "):
            text = " " + text
        pieces = list(text.replace(" ", self.SPACE))
        n = len(pieces)
        nxt, prv, alive = list(range(1, n + 1)), list(range(-1, n - 1)), [True] * n
        heap = []

        def push(i):
            j = nxt[i]
            if j < n and alive[i] and alive[j]:
                m = pieces[i] + pieces[j]
                k = self.index.get(m)
                if k is not None:
                    heapq.heappush(heap, (-self.scores[k], i, m))
        for i in range(n - 1):
            push(i)
        while heap:
            _, i, m = heapq.heappop(heap)
            j = nxt[i]
            if not alive[i] or j >= n or not alive[j] or pieces[i] + pieces[j] != m:
                continue                                     # stale entry
            pieces[i], alive[j] = m, False
            nxt[i] = nxt[j]
            if nxt[j] < n:
                prv[nxt[j]] = i
            if prv[i] >= 0:
                push(prv[i])
            push(i)
        ids = [self.bos_id] if add_bos and self.bos_id is not None else []
        for i in range(n):
            if not alive[i]:
                continue
            k = self.index.get(pieces[i])
            if k is not None:
                ids.append(k)
            else:
                bs = pieces[i].encode("utf-8")
                ids += [self.byte_ids[b] for b in bs] if all(b in self.byte_ids for b in bs) else [self.unk_id]
        return ids

    def decode(self, ids):
        out = bytearray()
        for i in ids:
            if i in (self.bos_id, self.eos_id) or not 0 <= i < len(self.tokens):
                continue
            t = self.tokens[i]
            if len(t) == 6 and t.startswith("<0x") and t.endswith(">"):
                out.append(int(t[3:5], 16))
            elif self.types[i] == 3:                        # control token
                continue
            else:
                out += t.replace(self.SPACE, " ").encode("utf-8")
        s = out.decode("utf-8", errors="replace")
        return s[1:] if self.add_space_prefix and s.startswith(" ") else s


class SentencePieceTokenizer(Tokenizer):
    def __init__(self, path: str):
        import sentencepiece as spm
        self.sp = spm.SentencePieceProcessor(model_file=path)
        self.bos_id, self.eos_id = self.sp.bos_id(), self.sp.eos_id()

    def encode(self, text, add_bos=True):
        ids = self.sp.encode(text)
        return ([self.bos_id] if add_bos and self.bos_id >= 0 else []) + ids

    def decode(self, ids):
        return self.sp.decode([i for i in ids if i not in (self.bos_id, self.eos_id)])

    @property
    def vocab_size(self):
        return self.sp.get_piece_size()


def load_tokenizer(path: Optional[str] = None, gguf_file=None, vocab_size: int = 258) -> Tokenizer:
    if path and path.endswith(".model"):
        return SentencePieceTokenizer(path)
    if gguf_file is not None and "tokenizer.ggml.tokens" in gguf_file.metadata:
        return GGUFTokenizer.from_gguf(gguf_file)
    return ByteTokenizer(vocab_size)
