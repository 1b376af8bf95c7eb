"""BERT encoder with sequence-classification and masked-LM heads (crates/axonml-llm/src/bert.rs).
Post-LN blocks, learned position + token-type embeddings, GELU FFN."""
from __future__ import annotations

import torch

from .. import nn
from ..ops.attention import sdpa
from .config import BertConfig
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


class Bert(nn.Module, LoadStateDict):
    def __init__(self, cfg: BertConfig):
        super().__init__()
        self.cfg = cfg
        self.embeddings = BertEmbeddings(cfg)
        self.layers = nn.ModuleList([BertLayer(cfg) for _ in range(cfg.num_hidden_layers)])
        self.pooler = nn.Linear(cfg.hidden_size, cfg.hidden_size, activation="tanh")

    @classmethod
    def new(cls, cfg): return cls(cfg)

    def forward(self, ids, token_type_ids=None, attention_mask=None):
        h = self.embeddings(ids, token_type_ids)
        for l in self.layers:
            h = l(h, attention_mask)
        return h, self.pooler(h[:, 0])


class BertForSequenceClassification(nn.Module):
    def __init__(self, cfg: BertConfig, num_labels: int = 2):
        super().__init__()
        self.bert, self.dropout = Bert(cfg), nn.Dropout(cfg.hidden_dropout_prob)
        self.classifier = nn.Linear(cfg.hidden_size, num_labels)

    def forward(self, ids, token_type_ids=None, attention_mask=None):
        return self.classifier(self.dropout(self.bert(ids, token_type_ids, attention_mask)[1]))


class BertForMaskedLM(nn.Module):
    def __init__(self, cfg: BertConfig):
        super().__init__()
        self.bert = Bert(cfg)
        self.transform = nn.Linear(cfg.hidden_size, cfg.hidden_size, activation="gelu")
        self.norm = nn.LayerNorm(cfg.hidden_size, cfg.layer_norm_eps)
        self.decoder_bias = nn.Parameter(torch.zeros(cfg.vocab_size))

    def forward(self, ids, token_type_ids=None, attention_mask=None):
        h = self.norm(self.transform(self.bert(ids, token_type_ids, attention_mask)[0]))
        return torch.nn.functional.linear(h, self.bert.embeddings.word_embeddings.weight.to(h.dtype), self.decoder_bias.to(h.dtype))
