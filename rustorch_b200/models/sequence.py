"""Sequence models: ``RNNModel``, ``LSTMModel``, ``Seq2SeqModel`` (src/models/rnn.rs:15-949), ``BERT`` and the
generic ``TransformerModel`` with their configs / builders (src/models/transformer_models.rs:18-670,931-1219).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..nn.layers import Embedding, LayerNorm, Linear, PositionalEncoding
from ..nn.transformer import TransformerEncoder, TransformerEncoderLayer


class RNNModel(nn.Module):
    """embedding -> (bi)RNN/LSTM/GRU -> classifier on the last time step."""

    def __init__(self, vocab_size: int, embedding_dim: int, hidden_size: int, num_classes: int, num_layers: int = 1,
                 bidirectional: bool = False, dropout: float = 0.0, cell: str = "rnn"):
        super().__init__()
        self.embedding = Embedding(vocab_size, embedding_dim)
        rnn_cls = {"rnn": nn.RNN, "lstm": nn.LSTM, "gru": nn.GRU}[cell.lower()]
        self.rnn = rnn_cls(embedding_dim, hidden_size, num_layers, batch_first=True, bidirectional=bidirectional,
                           dropout=dropout if num_layers > 1 else 0.0)
        self.dropout = nn.Dropout(dropout)
        self.classifier = Linear(hidden_size * (2 if bidirectional else 1), num_classes)

    def forward(self, tokens: torch.Tensor) -> torch.Tensor:
        out, _ = self.rnn(self.embedding(tokens))
        return self.classifier(self.dropout(out[:, -1]))


class LSTMModel(RNNModel):
    """Embedding + LSTM stack + classifier head (src/models/rnn.rs)."""

    def __init__(self, vocab_size, embedding_dim, hidden_size, num_classes, num_layers=1, bidirectional=False, dropout=0.0):
        super().__init__(vocab_size, embedding_dim, hidden_size, num_classes, num_layers, bidirectional, dropout, "lstm")


class Seq2SeqModel(nn.Module):
    """LSTM encoder -> LSTM decoder with teacher forcing; ``generate`` decodes greedily."""

    def __init__(self, src_vocab: int, tgt_vocab: int, embedding_dim: int, hidden_size: int, num_layers: int = 1,
                 dropout: float = 0.0):
        super().__init__()
        self.src_emb, self.tgt_emb = Embedding(src_vocab, embedding_dim), Embedding(tgt_vocab, embedding_dim)
        self.encoder = nn.LSTM(embedding_dim, hidden_size, num_layers, batch_first=True, dropout=dropout if num_layers > 1 else 0.0)
        self.decoder = nn.LSTM(embedding_dim, hidden_size, num_layers, batch_first=True, dropout=dropout if num_layers > 1 else 0.0)
        self.out = Linear(hidden_size, tgt_vocab)

    def forward(self, src: torch.Tensor, tgt: torch.Tensor) -> torch.Tensor:
        _, state = self.encoder(self.src_emb(src))
        dec, _ = self.decoder(self.tgt_emb(tgt), state)
        return self.out(dec)

    @torch.no_grad()
    def generate(self, src: torch.Tensor, bos: int, max_len: int = 32, eos: Optional[int] = None) -> torch.Tensor:
        _, state = self.encoder(self.src_emb(src))
        tok = torch.full((src.shape[0], 1), bos, dtype=torch.long, device=src.device)
        outs = []
        for _ in range(max_len):
            dec, state = self.decoder(self.tgt_emb(tok), state)
            tok = self.out(dec[:, -1:]).argmax(-1)
            outs.append(tok)
            if eos is not None and bool((tok == eos).all()):
                break
        return torch.cat(outs, 1)


class _Builder:
    _cls = None

    def __init__(self):
        self._kw = {}

    def __getattr__(self, name):
        if name.startswith("_"):
            raise AttributeError(name)

        def setter(v):
            self._kw[name] = v
            return self
        return setter

    def build(self):
        return type(self)._cls(**self._kw)


class RNNModelBuilder(_Builder):
    """Fluent builder of :class:`RNNModel`."""

    _cls = RNNModel


class LSTMModelBuilder(_Builder):
    """Fluent builder of :class:`LSTMModel`."""

    _cls = LSTMModel


class Seq2SeqModelBuilder(_Builder):
    """Fluent builder of :class:`Seq2SeqModel`."""

    _cls = Seq2SeqModel


# ----------------------------------------------------------------------------- BERT
@dataclass
class BERTConfig:
    vocab_size: int = 30522
    hidden_size: int = 768
    num_hidden_layers: int = 12
    num_attention_heads: int = 12
    intermediate_size: int = 3072
    max_position_embeddings: int = 512
    type_vocab_size: int = 2
    hidden_dropout_prob: float = 0.1
    layer_norm_eps: float = 1e-12

    @staticmethod
    def bert_base_uncased() -> "BERTConfig":
        return BERTConfig()

    @staticmethod
    def bert_large_uncased() -> "BERTConfig":
        return BERTConfig(hidden_size=1024, num_hidden_layers=24, num_attention_heads=16, intermediate_size=4096)


class BERTEmbeddings(nn.Module):
    def __init__(self, c: BERTConfig):
        super().__init__()
        self.word = Embedding(c.vocab_size, c.hidden_size)
        self.position = Embedding(c.max_position_embeddings, c.hidden_size)
        self.token_type = Embedding(c.type_vocab_size, c.hidden_size)
        self.norm = LayerNorm(c.hidden_size, c.layer_norm_eps)
        self.dropout = nn.Dropout(c.hidden_dropout_prob)

    def forward(self, input_ids, token_type_ids=None):
        T = input_ids.shape[1]
        pos = torch.arange(T, device=input_ids.device).unsqueeze(0)
        tt = torch.zeros_like(input_ids) if token_type_ids is None else token_type_ids
        return self.dropout(self.norm(self.word(input_ids) + self.position(pos) + self.token_type(tt)))


class BERT(nn.Module):
    """Bidirectional encoder with pooler, masked-LM head and sequence-classification head."""

    def __init__(self, config: Optional[BERTConfig] = None, num_labels: int = 2):
        super().__init__()
        c = self.config = config or BERTConfig()
        self.embeddings = BERTEmbeddings(c)
        self.encoder = TransformerEncoder(
            lambda: TransformerEncoderLayer(c.hidden_size, c.num_attention_heads, c.intermediate_size, c.hidden_dropout_prob,
                                            "gelu", c.layer_norm_eps), c.num_hidden_layers)
        self.pooler = Linear(c.hidden_size, c.hidden_size)
        self.mlm_head = Linear(c.hidden_size, c.vocab_size)
        self.classifier = Linear(c.hidden_size, num_labels)

    def forward(self, input_ids, token_type_ids=None, attention_mask=None) -> Tuple[torch.Tensor, torch.Tensor]:
        """Returns ``(sequence_output [B,T,H], pooled_output [B,H])``; ``attention_mask``: 1 = token, 0 = padding."""
        h = self.encoder(self.embeddings(input_ids, token_type_ids), src_key_padding_mask=attention_mask)
        return h, torch.tanh(self.pooler(h[:, 0]))

    @classmethod
    def from_hf(cls, directory: str, num_labels: int = 2) -> "BERT":
        """The encoder, embeddings and pooler of a Hugging Face BERT checkpoint directory (``config.json`` +
        safetensors).  Query / key / value projections are stacked into the attention's input projection; the
        masked-LM and classification heads keep their fresh initialisation unless the checkpoint has a decoder bias
        and tied decoder (``cls.predictions``), which only the full pre-training head has."""
        from ..formats.safetensors import HuggingFaceCheckpoint
        with HuggingFaceCheckpoint(directory) as ck:
            c = ck.config
            if c.get("hidden_act", "gelu") != "gelu" or c.get("position_embedding_type", "absolute") != "absolute":
                raise ValueError(f"{directory}: only absolute positions and the erf form of GELU are implemented")
            cfg = BERTConfig(vocab_size=int(c["vocab_size"]), hidden_size=int(c["hidden_size"]), num_hidden_layers=int(c["num_hidden_layers"]),
                             num_attention_heads=int(c["num_attention_heads"]), intermediate_size=int(c["intermediate_size"]),
                             max_position_embeddings=int(c.get("max_position_embeddings", 512)), type_vocab_size=int(c.get("type_vocab_size", 2)),
                             hidden_dropout_prob=float(c.get("hidden_dropout_prob", 0.1)), layer_norm_eps=float(c.get("layer_norm_eps", 1e-12)))
            model = cls(cfg, num_labels)
            pre = "bert." if any(k.startswith("bert.") for k in ck.keys()) else ""
            get = lambda n: ck.get(pre + n).float()      # noqa: E731

            def lin(dst, src):
                dst.weight.copy_(get(src + ".weight"))
                dst.bias.copy_(get(src + ".bias"))
            with torch.no_grad():
                e = model.embeddings
                e.word.weight.copy_(get("embeddings.word_embeddings.weight"))
                e.position.weight.copy_(get("embeddings.position_embeddings.weight"))
                e.token_type.weight.copy_(get("embeddings.token_type_embeddings.weight"))
                lin(e.norm, "embeddings.LayerNorm")
                for i, layer in enumerate(model.encoder.layers):
                    p = f"encoder.layer.{i}."
                    att = layer.self_attn
                    att.in_proj.weight.copy_(torch.cat([get(p + f"attention.self.{n}.weight") for n in ("query", "key", "value")], 0))
                    att.in_proj.bias.copy_(torch.cat([get(p + f"attention.self.{n}.bias") for n in ("query", "key", "value")], 0))
                    lin(att.out_proj, p + "attention.output.dense")
                    lin(layer.norm1, p + "attention.output.LayerNorm")
                    lin(layer.linear1, p + "intermediate.dense")
                    lin(layer.linear2, p + "output.dense")
                    lin(layer.norm2, p + "output.LayerNorm")
                if pre + "pooler.dense.weight" in ck:
                    lin(model.pooler, "pooler.dense")
        return model

    def masked_lm_logits(self, input_ids, **kw) -> torch.Tensor:
        return self.mlm_head(self.forward(input_ids, **kw)[0])

    def classify(self, input_ids, **kw) -> torch.Tensor:
        return self.classifier(self.forward(input_ids, **kw)[1])


class BERTBuilder(_Builder):
    def build(self) -> BERT:
        labels = self._kw.pop("num_labels", 2)
        return BERT(BERTConfig(**self._kw), labels)


def bert_base_uncased(**kw) -> BERT:
    return BERT(BERTConfig.bert_base_uncased(), **kw)


def bert_large_uncased(**kw) -> BERT:
    return BERT(BERTConfig.bert_large_uncased(), **kw)


# ----------------------------------------------------------------- generic transformer
class TransformerModel(nn.Module):
    """Token embedding + sinusoidal positions + encoder stack + output projection."""

    def __init__(self, vocab_size: int, d_model: int = 512, nhead: int = 8, num_layers: int = 6, dim_feedforward: int = 2048,
                 dropout: float = 0.1, max_len: int = 5000, num_classes: Optional[int] = None, causal: bool = False):
        super().__init__()
        self.embedding = Embedding(vocab_size, d_model)
        self.pos = PositionalEncoding(d_model, max_len, dropout)
        self.encoder = TransformerEncoder(lambda: TransformerEncoderLayer(d_model, nhead, dim_feedforward, dropout, "gelu"),
                                          num_layers, LayerNorm(d_model))
        self.head = Linear(d_model, num_classes if num_classes is not None else vocab_size)
        self.causal, self.pool = causal, num_classes is not None
        self.d_model = d_model

    def forward(self, tokens: torch.Tensor, key_padding_mask=None) -> torch.Tensor:
        x = self.pos(self.embedding(tokens) * (self.d_model ** 0.5))
        x = self.encoder(x, src_key_padding_mask=key_padding_mask, is_causal=self.causal)
        return self.head(x.mean(1) if self.pool else x)


class TransformerModelBuilder(_Builder):
    """Fluent builder of :class:`TransformerModel`."""

    _cls = TransformerModel
