"""Tokenizers for the CLI (example-cli/src/tokenizer/wrapper.rs:8-96 wraps the HF ``tokenizers`` crate or a dummy).

* ``GGUFTokenizer``: the SentencePiece-style vocabulary embedded in a GGUF file (``tokenizer.ggml.tokens`` /
  ``scores`` / ``token_type``): text is split into UTF-8 characters (spaces become U+2581), adjacent pieces are
  merged best-score-first while the merged piece exists in the vocabulary, unknown characters fall back to
  ``<0xXX>`` byte tokens.
* ``SentencePieceTokenizer``: a ``.model`` file through the ``sentencepiece`` package.
* ``BPETokenizer``: byte-level BPE from ``vocab.json`` + ``merges.txt`` (the GPT-2 family's files in a Hugging Face
  directory): text is cut by the GPT-2 pre-tokenisation pattern, every piece's UTF-8 bytes are mapped to printable
  characters and merged in the order of the merge table.
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


def _byte_alphabet() -> Dict[int, str]:
    """The byte -> printable character table of byte-level BPE: printable Latin-1 bytes stand for themselves, the rest
    are moved to code points from 256 upwards."""
    keep = list(range(ord("!"), ord("~") + 1)) + list(range(0xA1, 0xAD)) + list(range(0xAE, 0x100))
    table, extra = {}, 0
    for b in range(256):
        if b in keep:
            table[b] = chr(b)
        else:
            table[b] = chr(256 + extra)
            extra += 1
    return table


class BPETokenizer(Tokenizer):
    _PATTERN = r"""'s|'t|'re|'ve|'m|'ll|'d| ?\p{L}+| ?\p{N}+| ?[^\s\p{L}\p{N}]+|\s+(?!\S)|\s+"""

    def __init__(self, vocab: Dict[str, int], merges: Sequence[Sequence[str]], eos_token: str = "<|endoftext|>"):
        import regex
        self.vocab = dict(vocab)
        self.inverse = {i: t for t, i in self.vocab.items()}
        self.rank = {tuple(m): r for r, m in enumerate(merges)}
        self.to_char = _byte_alphabet()
        self.to_byte = {c: b for b, c in self.to_char.items()}
        self._split = regex.compile(self._PATTERN)
        self._cache: Dict[str, List[str]] = {}
        self.eos_id = self.vocab.get(eos_token)
        self.bos_id = None                                   # the GPT-2 family starts a text without a marker

    @classmethod
    def from_files(cls, vocab_path: str, merges_path: str) -> "BPETokenizer":
        import json
        with open(vocab_path, encoding="utf-8") as f:
            vocab = json.load(f)
        with open(merges_path, encoding="utf-8") as f:
            merges = [tuple(line.split()) for line in f.read().split("\n") if line and not line.startswith("#version") and len(line.split()) == 2]
        return cls(vocab, merges)

    @property
    def vocab_size(self):
        return len(self.vocab)

    def _merge(self, word: str) -> List[str]:
        hit = self._cache.get(word)
        if hit is not None:
            return hit
        parts = list(word)
        while len(parts) > 1:
            best, at = None, -1
            for i in range(len(parts) - 1):
                r = self.rank.get((parts[i], parts[i + 1]))
                if r is not None and (best is None or r < best):
                    best, at = r, i
            if best is None:
                break
            a, b = parts[at], parts[at + 1]
            out, i = [], 0
            while i < len(parts):                            # merge every occurrence of the best pair, left to right
                if i < len(parts) - 1 and parts[i] == a and parts[i + 1] == b:
                    out.append(a + b)
                    i += 2
                else:
                    out.append(parts[i])
                    i += 1
            parts = out
        self._cache[word] = parts
        return parts

    def encode(self, text, add_bos=True):
        ids: List[int] = []
        for piece in self._split.findall(text):
            word = "".join(self.to_char[b] for b in piece.encode("utf-8"))
            for tok in self._merge(word):
                if tok not in self.vocab:
                    raise ValueError(f"token {tok!r} is not in the vocabulary: vocab.json and merges.txt do not belong together")
                ids.append(self.vocab[tok])
        return ids

    def decode(self, ids):
        chars = "".join(self.inverse.get(int(i), "") for i in ids)
        return bytes(self.to_byte[c] for c in chars if c in self.to_byte).decode("utf-8", errors="replace")


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
    """``path``: a SentencePiece ``.model`` file, a ``vocab.json`` (its ``merges.txt`` beside it) or a directory that
    holds one of the two."""
    import os
    if path and os.path.isdir(path):
        for cand in ("tokenizer.model", "vocab.json"):
            if os.path.exists(os.path.join(path, cand)):
                path = os.path.join(path, cand)
                break
        else:
            path = None
    if path and path.endswith("vocab.json"):
        return BPETokenizer.from_files(path, os.path.join(os.path.dirname(path), "merges.txt"))
    if path and path.endswith(".model"):
        return SentencePieceTokenizer(path)
    if gguf_file is not None and "tokenizer.ggml.tokens" in gguf_file.metadata:
        return GGUFTokenizer.from_gguf(gguf_file)
    return ByteTokenizer(vocab_size)
