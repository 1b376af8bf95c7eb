"""Vocabulary (crates/axonml-text/src/vocab.rs:31-231)."""
from __future__ import annotations

import collections

import torch

PAD, UNK, BOS, EOS, MASK = "<pad>", "<unk>", "<bos>", "<eos>", "<mask>"


class Vocab:
    def __init__(self):
        self.token_to_idx: dict = {}
        self.idx_to_token: list = []
        self.unk_index = None

    @classmethod
    def new(cls): return cls()

    @classmethod
    def with_special_tokens(cls):
        v = cls()
        for t in (PAD, UNK, BOS, EOS, MASK):
            v.add_token(t)
        v.unk_index = v.token_to_idx[UNK]
        return v

    @classmethod
    def from_tokens(cls, tokens, min_freq: int = 1, specials: bool = True):
        v = cls.with_special_tokens() if specials else cls()
        for t, c in collections.Counter(tokens).most_common():
            if c >= min_freq:
                v.add_token(t)
        return v

    @classmethod
    def from_text(cls, text: str, tokenizer=None, min_freq: int = 1):
        """``from_text(corpus, 1)`` (the reference's ``Vocab::from_text(text, min_freq)``) or
        ``from_text(corpus, tokenizer, min_freq)``."""
        if isinstance(tokenizer, int):
            tokenizer, min_freq = None, tokenizer
        toks = tokenizer(text) if tokenizer else text.split()
        return cls.from_tokens(toks, min_freq)

    def add_token(self, token: str) -> int:
        if token not in self.token_to_idx:
            self.token_to_idx[token] = len(self.idx_to_token)
            self.idx_to_token.append(token)
        return self.token_to_idx[token]

    def add_special_tokens(self, tokens) -> None:
        for t in tokens:
            self.add_token(t)

    def set_unk_token(self, token: str) -> None:
        """Adds ``token`` (if new) and makes it what unknown words map to."""
        self.unk_index = self.add_token(token)
        self.unk_token = token

    def set_pad_token(self, token: str) -> None:
        self.add_token(token)
        self.pad_token = token

    def tokens(self) -> list: return list(self.idx_to_token)
    def is_empty(self) -> bool: return not self.idx_to_token
    def len(self) -> int: return len(self.idx_to_token)
    def __len__(self) -> int: return len(self.idx_to_token)
    def contains(self, token: str) -> bool: return token in self.token_to_idx
    def token_to_index(self, token: str):
        return self.token_to_idx.get(token, self.unk_index)
    def index_to_token(self, idx: int):
        return self.idx_to_token[idx] if 0 <= idx < len(self.idx_to_token) else None
    def encode(self, tokens) -> list: return [self.token_to_index(t) for t in tokens]
    def decode(self, indices) -> list: return [self.index_to_token(int(i)) for i in indices]
    def encode_tensor(self, tokens) -> torch.Tensor: return torch.tensor(self.encode(tokens), dtype=torch.long)
    def pad_index(self): return self.token_to_idx.get(getattr(self, "pad_token", PAD))
    def unk_index_(self): return self.unk_index
    def bos_index(self): return self.token_to_idx.get(BOS)
    def eos_index(self): return self.token_to_idx.get(EOS)
