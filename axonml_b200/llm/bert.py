"""BERT encoder with sequence-classification and masked-LM heads (crates/axonml-llm/src/bert.rs).
Post-LN blocks, learned position + token-type embeddings, GELU FFN."""
from __future__ import annotations

import torch

from .. import nn
from ..ops.attention import sdpa
from .config import BertConfig
from ._api import ModelApi
from .hf_loader import LoadStateDict


class BertEmbeddings(nn.Module):
    def __init__(self, cfg: BertConfig):
        super().__init__()
        self.word_embeddings = nn.Embedding(cfg.vocab_size, cfg.hidden_size)
        self.position_embeddings = nn.Embedding(cfg.max_position_embeddings, cfg.hidden_size)
        self.token_type_embeddings = nn.Embedding(cfg.type_vocab_size, cfg.hidden_size)
        self.LayerNorm = nn.LayerNorm(cfg.hidden_size, cfg.layer_norm_eps)
        self.dropout = nn.Dropout(cfg.hidden_dropout_prob)

    def forward(self, ids, token_type_ids=None):
        B, S = ids.shape
        pos = torch.arange(S, device=ids.device).unsqueeze(0).expand(B, S)
        tt = token_type_ids if token_type_ids is not None else torch.zeros_like(ids)
        e = self.word_embeddings(ids) + self.position_embeddings(pos) + self.token_type_embeddings(tt)
        return self.dropout(self.LayerNorm(e))


class BertLayer(nn.Module):
    def __init__(self, cfg: BertConfig):
        super().__init__()
        H = cfg.hidden_size
        self.h, self.hd = cfg.num_attention_heads, cfg.head_dim()
        self.query, self.key, self.value = nn.Linear(H, H), nn.Linear(H, H), nn.Linear(H, H)
        self.attn_out = nn.Linear(H, H)
        self.attn_norm = nn.LayerNorm(H, cfg.layer_norm_eps)
        self.intermediate = nn.Linear(H, cfg.intermediate_size, activation="gelu")
        self.output = nn.Linear(cfg.intermediate_size, H)
        self.out_norm = nn.LayerNorm(H, cfg.layer_norm_eps)
        self.dropout = nn.Dropout(cfg.hidden_dropout_prob)

    def forward(self, x, attention_mask=None):
        B, S, H = x.shape
        q = self.query(x).view(B, S, self.h, self.hd)
        k = self.key(x).view(B, S, self.h, self.hd)
        v = self.value(x).view(B, S, self.h, self.hd)
        mask = None
        if attention_mask is not None:
            mask = attention_mask.bool()[:, None, None, :]
        a = sdpa(q, k, v, mask=mask).reshape(B, S, H)
        x = self.attn_norm(x + self.dropout(self.attn_out(a)))
        return self.out_norm(x + self.dropout(self.output(self.intermediate(x))))


class BertPooler(nn.Module):
    """tanh(dense(hidden state of the first token)) (bert.rs:29-60)."""

    def __init__(self, hidden_size: int):
        super().__init__()
        self.dense = nn.Linear(hidden_size, hidden_size, activation="tanh")

    @classmethod
    def new(cls, hidden_size: int): return cls(hidden_size)

    def forward(self, hidden_states):
        return self.dense(hidden_states[:, 0])


class BertPredictionHeadTransform(nn.Module):
    """dense -> activation -> LayerNorm in front of the vocabulary projection (bert.rs:260-300)."""

    def __init__(self, hidden_size: int, layer_norm_eps: float = 1e-12, activation: str = "gelu"):
        super().__init__()
        act = {"gelu": "gelu", "relu": "relu", "silu": "silu", "swish": "silu", "tanh": "tanh"}[activation]
        self.dense = nn.Linear(hidden_size, hidden_size, activation=act)
        self.layer_norm = nn.LayerNorm(hidden_size, layer_norm_eps)
        self.activation = activation

    @classmethod
    def new(cls, hidden_size, layer_norm_eps, activation): return cls(hidden_size, layer_norm_eps, activation)

    def forward(self, x):
        return self.layer_norm(self.dense(x))


class BertLMPredictionHead(nn.Module):
    """Transform followed by the projection onto the vocabulary (bert.rs:251-258).  With
    ``tied_weight`` (the word-embedding matrix) the head owns only the output bias, as in the
    published checkpoints; without it the head has a ``decoder`` Linear of its own."""

    def __init__(self, hidden_size: int, vocab_size: int, layer_norm_eps: float = 1e-12, activation: str = "gelu", tied_weight=None):
        super().__init__()
        self.transform = BertPredictionHeadTransform(hidden_size, layer_norm_eps, activation)
        self._tied = [tied_weight] if tied_weight is not None else None          # in a list: not registered a second time
        if tied_weight is None:
            self.decoder = nn.Linear(hidden_size, vocab_size)
        else:
            self.bias = nn.Parameter(torch.zeros(vocab_size))

    def forward(self, x):
        h = self.transform(x)
        if self._tied is None:
            return self.decoder(h)
        return torch.nn.functional.linear(h, self._tied[0].to(h.dtype), self.bias.to(h.dtype))


def _bert_config_from_json(j: dict) -> BertConfig:
    d = BertConfig()
    g = lambda k, cast: cast(j.get(k, getattr(d, k)))
    return BertConfig(vocab_size=g("vocab_size", int), hidden_size=g("hidden_size", int), num_hidden_layers=g("num_hidden_layers", int),
                      num_attention_heads=g("num_attention_heads", int), intermediate_size=g("intermediate_size", int),
                      max_position_embeddings=g("max_position_embeddings", int), type_vocab_size=g("type_vocab_size", int),
                      layer_norm_eps=g("layer_norm_eps", float), hidden_dropout_prob=g("hidden_dropout_prob", float),
                      attention_probs_dropout_prob=g("attention_probs_dropout_prob", float))


class Bert(nn.Module, LoadStateDict, ModelApi):
    ARCH = "bert"
    _config_from_json = staticmethod(_bert_config_from_json)

    def __init__(self, cfg: BertConfig, add_pooler: bool = True):
        super().__init__()
        self.cfg = cfg
        self.embeddings = BertEmbeddings(cfg)
        self.layers = nn.ModuleList([BertLayer(cfg) for _ in range(cfg.num_hidden_layers)])
        self.pooler = BertPooler(cfg.hidden_size) if add_pooler else None

    @classmethod
    def new(cls, cfg): return cls(cfg)

    @classmethod
    def with_pooler(cls, cfg, add_pooler: bool = True):
        """Encoder with (``True``) or without the pooling layer over the first token (bert.rs ``with_pooler``)."""
        return cls(cfg, add_pooler)

    def encode(self, ids, token_type_ids=None, attention_mask=None):
        """Hidden states [batch, seq, hidden] of the last layer."""
        h = self.embeddings(ids, token_type_ids)
        for l in self.layers:
            h = l(h, attention_mask)
        return h

    def forward(self, ids, token_type_ids=None, attention_mask=None):
        h = self.encode(ids, token_type_ids, attention_mask)
        return h, (self.pooler(h) if self.pooler is not None else None)

    def forward_with_pooling(self, ids, token_type_ids=None, attention_mask=None):
        """``(hidden states, pooled first-token vector)``; an encoder built without a pooler raises."""
        if self.pooler is None:
            raise ValueError("this encoder was built without a pooler")
        return self.forward(ids, token_type_ids, attention_mask)

    def forward_ids(self, ids, token_type_ids=None, attention_mask=None):
        """Hidden states for integer (or float-typed) token ids."""
        ids = torch.as_tensor(ids)
        return self.encode((ids.unsqueeze(0) if ids.dim() == 1 else ids).long(), token_type_ids, attention_mask)


class BertForSequenceClassification(nn.Module, LoadStateDict, ModelApi):
    ARCH = "bert"
    _config_from_json = staticmethod(_bert_config_from_json)

    def __init__(self, cfg: BertConfig, num_labels: int = 2):
        super().__init__()
        self.cfg = cfg
        self.bert, self.dropout = Bert(cfg), nn.Dropout(cfg.hidden_dropout_prob)
        self.classifier = nn.Linear(cfg.hidden_size, num_labels)

    def forward(self, ids, token_type_ids=None, attention_mask=None):
        return self.classifier(self.dropout(self.bert(ids, token_type_ids, attention_mask)[1]))

    forward_classification = forward


class BertForMaskedLM(nn.Module, LoadStateDict, ModelApi):
    ARCH = "bert"
    _config_from_json = staticmethod(_bert_config_from_json)

    def __init__(self, cfg: BertConfig):
        super().__init__()
        self.cfg = cfg
        self.bert = Bert(cfg)
        self.cls = BertLMPredictionHead(cfg.hidden_size, cfg.vocab_size, cfg.layer_norm_eps, getattr(cfg, "hidden_act", "gelu"),
                                        tied_weight=self.bert.embeddings.word_embeddings.weight)

    def forward(self, ids, token_type_ids=None, attention_mask=None):
        return self.cls(self.bert(ids, token_type_ids, attention_mask)[0])

    forward_mlm = forward


_BERT_RENAMES = (("attention.self.query", "query"), ("attention.self.key", "key"), ("attention.self.value", "value"),
                 ("attention.output.dense", "attn_out"), ("attention.output.LayerNorm", "attn_norm"),
                 ("intermediate.dense", "intermediate"), ("output.dense", "output"), ("output.LayerNorm", "out_norm"))


def map_bert_weights(sd: dict, prefix: str = "") -> dict:
    """Names of a published BERT checkpoint -> the names of ``Bert`` (``prefix=""``) or of the
    task models that hold it as ``.bert`` (``prefix="bert."``).  ``encoder.layer.N.attention.self.
    query`` becomes ``layers.N.query`` and so on; the masked-LM head ``cls.predictions.*`` becomes
    ``cls.*``; the tied ``cls.predictions.decoder.weight`` and the position-id buffer are dropped;
    old checkpoints' ``gamma`` / ``beta`` are read as ``weight`` / ``bias``."""
    out = {}
    for k, v in sd.items():
        if k.endswith("position_ids") or k == "cls.predictions.decoder.weight" or k == "cls.predictions.decoder.bias":
            continue
        k = k.replace(".gamma", ".weight").replace(".beta", ".bias")
        if k.startswith("cls.predictions."):
            k = "cls." + k[len("cls.predictions."):].replace("transform.LayerNorm", "transform.layer_norm")
            out[k] = v
            continue
        if k.startswith(("classifier.", "cls.seq_relationship")):
            out[k] = v
            continue
        k = k.removeprefix("bert.")
        if k.startswith("encoder.layer."):
            k = "layers." + k[len("encoder.layer."):]
            for old, new in _BERT_RENAMES:
                k = k.replace("." + old + ".", "." + new + ".")
        out[prefix + k] = v
    return out
