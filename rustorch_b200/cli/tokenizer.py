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
        # control tokens (<s>, </s>, chat markers) written out in a prompt stand for their ids
        self.added = {t: i for i, t in enumerate(self.tokens) if self.types[i] == 3 and len(t) > 2 and self.index.get(t) == i}

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
        hits = [t for t in self.added if t in text] if self.added else []
        if hits:
            import re
            ids = [self.bos_id] if add_bos and self.bos_id is not None else []
            for chunk in re.split("(" + "|".join(re.escape(t) for t in sorted(hits, key=len, reverse=True)) + ")", text):
                if chunk in self.added:
                    ids.append(self.added[chunk])
                elif chunk:
                    ids += self._encode_plain(chunk, False)
            return ids
        return self._encode_plain(text, add_bos)

    def _encode_plain(self, text, add_bos):
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

    def __init__(self, vocab: Dict[str, int], merges: Sequence[Sequence[str]], eos_token: str = "<|endoftext|>",
                 pattern: Optional[str] = None, added_tokens: Optional[Dict[str, int]] = None, bos_token: Optional[str] = None,
                 ignore_merges: bool = False):
        import regex
        self.vocab = dict(vocab)
        self.added = dict(added_tokens or {})                # matched in the raw text ahead of the split, never merged
        self.inverse = {i: t for t, i in self.vocab.items()}
        self.added_inverse = {i: t for t, i in self.added.items()}
        self.rank = {tuple(m): r for r, m in enumerate(merges)}
        self.to_char = _byte_alphabet()
        self.to_byte = {c: b for b, c in self.to_char.items()}
        self._split = regex.compile(pattern or self._PATTERN)
        self._added_split = (regex.compile("(" + "|".join(regex.escape(t) for t in sorted(self.added, key=len, reverse=True)) + ")")
                             if self.added else None)
        self.ignore_merges = ignore_merges
        self._cache: Dict[str, List[str]] = {}
        self.eos_id = self.added.get(eos_token, self.vocab.get(eos_token))
        # the GPT-2 family starts a text without a marker; files whose post-processor prepends one name it here
        self.bos_id = self.added.get(bos_token, self.vocab.get(bos_token)) if bos_token else None

    @classmethod
    def from_files(cls, vocab_path: str, merges_path: str) -> "BPETokenizer":
        import json
        with open(vocab_path, encoding="utf-8") as f:
            vocab = json.load(f)
        with open(merges_path, encoding="utf-8") as f:
            merges = [tuple(line.split()) for line in f.read().split("\n") if line and not line.startswith("#version") and len(line.split()) == 2]
        return cls(vocab, merges)

    # split patterns by the ``tokenizer.ggml.pre`` name of GGUF files
    _APOS = "(?:'[sS]|'[tT]|'[rR][eE]|'[vV][eE]|'[mM]|'[lL][lL]|'[dD])"
    _TAIL = r"| ?[^\s\p{L}\p{N}]+[\r\n]*|\s*[\r\n]+|\s+(?!\S)|\s+"
    PRE_PATTERNS = {"llama-bpe": _APOS + r"|[^\r\n\p{L}\p{N}]?\p{L}+|\p{N}{1,3}" + _TAIL, "qwen2": _APOS + r"|[^\r\n\p{L}\p{N}]?\p{L}+|\p{N}" + _TAIL,
                    "gpt-2": _PATTERN, "default": _PATTERN}
    PRE_PATTERNS["llama3"] = PRE_PATTERNS["llama-v3"] = PRE_PATTERNS["llama-bpe"]

    @classmethod
    def from_gguf(cls, gguf_file) -> "BPETokenizer":
        """GGUF files whose ``tokenizer.ggml.model`` is ``gpt2`` (Llama 3, Qwen2, GPT-2 ...): the token list in the
        byte-level alphabet, ``tokenizer.ggml.merges``, control / user-defined token types as added tokens, and the split
        pattern that ``tokenizer.ggml.pre`` names."""
        md = gguf_file.metadata
        toks, merges = md.get("tokenizer.ggml.tokens"), md.get("tokenizer.ggml.merges")
        if toks is None or merges is None:
            raise KeyError("the GGUF file has no tokenizer.ggml.tokens / tokenizer.ggml.merges")
        types = md.get("tokenizer.ggml.token_type") or [1] * len(toks)
        vocab = {t: i for i, t in enumerate(toks)}
        added = {t: i for i, (t, ty) in enumerate(zip(toks, types)) if int(ty) in (3, 4)}      # control, user-defined
        pre = str(md.get("tokenizer.ggml.pre", "default"))
        pattern = md.get("tokenizer.rustorch.pattern") or cls.PRE_PATTERNS.get(pre)
        if pattern is None:
            raise ValueError(f"tokenizer.ggml.pre = '{pre}': no split pattern is known for this pre-tokenizer "
                             f"(known: {sorted(cls.PRE_PATTERNS)}); pass --tokenizer with the model's tokenizer.json")
        eos, bos = md.get("tokenizer.ggml.eos_token_id"), md.get("tokenizer.ggml.bos_token_id")
        add_bos = bool(md.get("tokenizer.ggml.add_bos_token", pre in ("llama-bpe", "llama3", "llama-v3")))
        self = cls(vocab, [tuple(m.split(" ")) for m in merges], None, pattern, added, None, bool(md.get("tokenizer.rustorch.ignore_merges", pre in ("llama-bpe", "llama3", "llama-v3"))))
        self.eos_id = int(eos) if eos is not None else None
        self.bos_id = int(bos) if (bos is not None and add_bos) else None
        return self

    def gguf_metadata(self, pre: Optional[str] = None) -> Dict[str, object]:
        """``tokenizer.ggml.*`` entries that describe this tokenizer (what ``from_gguf`` reads back)."""
        size = self.vocab_size
        toks = [self.added_inverse.get(i, self.inverse.get(i, f"[PAD{i}]")) for i in range(size)]
        types = [3 if i in self.added_inverse else (1 if i in self.inverse else 5) for i in range(size)]      # control / normal / unused
        by_rank = sorted(self.rank.items(), key=lambda kv: kv[1])
        pattern = self._split.pattern
        if pre is None:                               # the name other GGUF readers pick their pattern by
            pre = ("llama-bpe" if r"\p{N}{1,3}" in pattern else "qwen2" if r"|\p{N}|" in pattern else
                   "gpt-2" if pattern == self._PATTERN else "default")
        md: Dict[str, object] = {"tokenizer.ggml.model": "gpt2", "tokenizer.ggml.pre": pre, "tokenizer.ggml.tokens": toks,
                                 "tokenizer.ggml.token_type": types, "tokenizer.ggml.merges": [f"{a} {b}" for (a, b), _ in by_rank],
                                 "tokenizer.ggml.add_bos_token": self.bos_id is not None,
                                 "tokenizer.rustorch.pattern": pattern, "tokenizer.rustorch.ignore_merges": self.ignore_merges}
        if self.bos_id is not None:
            md["tokenizer.ggml.bos_token_id"] = int(self.bos_id)
        if self.eos_id is not None:
            md["tokenizer.ggml.eos_token_id"] = int(self.eos_id)
        return md

    @classmethod
    def from_tokenizer_json(cls, path: str) -> "BPETokenizer":
        """The single-file ``tokenizer.json`` of the ``tokenizers`` library, for byte-level BPE models (GPT-2, Llama 3,
        Qwen2, Mistral-Nemo...): vocabulary and merges, the split pattern of the pre-tokenizer, added / special tokens,
        and the start-of-text marker that the post-processor prepends.  ``eos`` comes from ``tokenizer_config.json``
        beside the file when there is one."""
        import json
        import os
        with open(path, encoding="utf-8") as f:
            tj = json.load(f)
        model = tj.get("model") or {}
        if model.get("type") != "BPE":
            raise ValueError(f"{path}: tokenizer model type {model.get('type')!r}; byte-level BPE is what this reader handles")

        def steps(node):
            if not node:
                return []
            if node.get("type") == "Sequence":
                return [s for sub in node.get("pretokenizers", node.get("processors", [])) for s in steps(sub)]
            return [node]
        pre = steps(tj.get("pre_tokenizer"))
        if not any(p.get("type") == "ByteLevel" for p in pre):
            raise ValueError(f"{path}: the pre-tokenizer is not byte-level ({[p.get('type') for p in pre]}); "
                             "for SentencePiece-style vocabularies pass the tokenizer.model file")
        pattern = None
        for p in pre:
            if p.get("type") == "Split" and isinstance(p.get("pattern"), dict) and "Regex" in p["pattern"]:
                pattern = p["pattern"]["Regex"]
        merges = [tuple(m.split(" ")) if isinstance(m, str) else tuple(m) for m in model.get("merges", [])]
        added = {t["content"]: int(t["id"]) for t in tj.get("added_tokens", [])}
        bos = None
        for p in steps(tj.get("post_processor")):
            single = p.get("single") or []
            if p.get("type") == "TemplateProcessing" and single and "SpecialToken" in single[0]:
                bos = single[0]["SpecialToken"]["id"]
        eos = "<|endoftext|>"
        cfg_path = os.path.join(os.path.dirname(path), "tokenizer_config.json")
        if os.path.exists(cfg_path):
            with open(cfg_path, encoding="utf-8") as f:
                tc = json.load(f)
            e = tc.get("eos_token")
            eos = (e.get("content") if isinstance(e, dict) else e) or eos
            b = tc.get("bos_token")
            if bos is None and tc.get("add_bos_token") and b:
                bos = b.get("content") if isinstance(b, dict) else b
        return cls(model.get("vocab", {}), merges, eos, pattern, added, bos, bool(model.get("ignore_merges", False)))

    @property
    def vocab_size(self):
        return max(len(self.vocab), 1 + max(self.added.values(), default=-1), 1 + max(self.vocab.values(), default=-1))

    def _merge(self, word: str) -> List[str]:
        hit = self._cache.get(word)
        if hit is not None:
            return hit
        if self.ignore_merges and word in self.vocab:
            self._cache[word] = [word]
            return [word]
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
        ids: List[int] = [self.bos_id] if (add_bos and self.bos_id is not None) else []
        for chunk in (self._added_split.split(text) if self._added_split else [text]):
            if not chunk:
                continue
            if chunk in self.added:
                ids.append(self.added[chunk])
                continue
            for piece in self._split.findall(chunk):
                word = "".join(self.to_char[b] for b in piece.encode("utf-8"))
                for tok in self._merge(word):
                    if tok not in self.vocab:
                        raise ValueError(f"token {tok!r} is not in the vocabulary: the vocabulary and the merges do not belong together")
                    ids.append(self.vocab[tok])
        return ids

    def decode(self, ids, skip_special: bool = True):
        out, run = [], []

        def flush():
            if run:
                out.append(bytes(self.to_byte[c] for c in "".join(run) if c in self.to_byte).decode("utf-8", errors="replace"))
                run.clear()
        for i in ids:
            i = int(i)
            if i in self.added_inverse:
                if not skip_special:
                    flush()
                    out.append(self.added_inverse[i])
                continue
            run.append(self.inverse.get(i, ""))
        flush()
        return "".join(out)


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
    """``path``: a SentencePiece ``.model`` file, a ``vocab.json`` (its ``merges.txt`` beside it), a byte-level BPE
    ``tokenizer.json``, or a directory that holds one of the three."""
    import os
    if path and os.path.isdir(path):
        for cand in ("tokenizer.model", "vocab.json", "tokenizer.json"):
            if os.path.exists(os.path.join(path, cand)):
                path = os.path.join(path, cand)
                break
        else:
            path = None
    if path and path.endswith("vocab.json"):
        return BPETokenizer.from_files(path, os.path.join(os.path.dirname(path), "merges.txt"))
    if path and path.endswith("tokenizer.json"):
        return BPETokenizer.from_tokenizer_json(path)
    if path and path.endswith(".model"):
        return SentencePieceTokenizer(path)
    if gguf_file is not None and "tokenizer.ggml.tokens" in gguf_file.metadata:
        if str(gguf_file.metadata.get("tokenizer.ggml.model", "llama")) == "gpt2":
            return BPETokenizer.from_gguf(gguf_file)
        return GGUFTokenizer.from_gguf(gguf_file)
    return ByteTokenizer(vocab_size)
