"""Text datasets (crates/axonml-text/src/datasets/mod.rs:18-317): TextDataset,
LanguageModelDataset, SyntheticSentimentDataset, SyntheticSeq2SeqDataset."""
from __future__ import annotations

import torch

from ..data.dataset import Dataset
from .vocab import Vocab


class TextDataset(Dataset):
    def __init__(self, texts, labels, vocab: Vocab, tokenizer, max_len: int):
        self.texts, self.labels, self.vocab, self.tokenizer, self.max_len = list(texts), list(labels), vocab, tokenizer, max_len

    @classmethod
    def new(cls, texts, labels, vocab, tokenizer, max_len): return cls(texts, labels, vocab, tokenizer, max_len)

    @classmethod
    def from_samples(cls, samples, tokenizer, min_freq: int = 1, max_length: int = 64):
        """Dataset from ``(text, label)`` pairs: the vocabulary holds the special tokens and then
        every token seen at least ``min_freq`` times, most frequent first (ties alphabetically)."""
        import collections
        freq = collections.Counter(t for text, _ in samples for t in tokenizer(text))
        vocab = Vocab.with_special_tokens()
        for tok, _ in sorted(((t, c) for t, c in freq.items() if c >= min_freq), key=lambda tc: (-tc[1], tc[0])):
            vocab.add_token(tok)
        return cls([t for t, _ in samples], [l for _, l in samples], vocab, tokenizer, max_length)

    def len(self) -> int: return len(self.texts)
    def num_classes(self) -> int: return (max(self.labels) + 1) if self.labels else 0
    def max_length(self) -> int: return self.max_len

    def get(self, i: int):
        ids = self.vocab.encode(self.tokenizer(self.texts[i]))[: self.max_len]
        ids += [self.vocab.pad_index() or 0] * (self.max_len - len(ids))
        return torch.tensor(ids, dtype=torch.long), torch.tensor(self.labels[i], dtype=torch.long)


class LanguageModelDataset(Dataset):
    """Sliding windows over a token stream: input = tokens[i:i+L], target = tokens[i+1:i+L+1]."""

    def __init__(self, tokens, seq_len: int, stride: int | None = None):
        self.tokens = torch.as_tensor(tokens, dtype=torch.long)
        self.seq_len, self.stride = seq_len, stride or seq_len

    @classmethod
    def from_text(cls, text: str, vocab: Vocab, tokenizer, seq_len: int):
        ds = cls(vocab.encode(tokenizer(text)), seq_len)
        ds._vocab = vocab
        return ds

    def vocab(self):
        """The vocabulary the token stream was encoded with (``None`` for a dataset built from ids)."""
        return getattr(self, "_vocab", None)

    def len(self) -> int: return max(0, (self.tokens.numel() - self.seq_len - 1) // self.stride + 1)

    def get(self, i: int):
        s = i * self.stride
        return self.tokens[s:s + self.seq_len], self.tokens[s + 1:s + self.seq_len + 1]


class SyntheticSentimentDataset(Dataset):
    """Random token sequences whose label is decided by which of two disjoint token ranges dominates."""

    def __init__(self, num_samples: int = 1000, seq_len: int = 32, vocab_size: int = 1000, seed: int = 42):
        g = torch.Generator().manual_seed(seed)
        self.labels = torch.randint(0, 2, (num_samples,), generator=g)
        half = vocab_size // 2
        base = torch.randint(0, half, (num_samples, seq_len), generator=g)
        self.data = base + self.labels[:, None] * half * (torch.rand(num_samples, seq_len, generator=g) < 0.7)

    @classmethod
    def new(cls, num_samples, seq_len, vocab_size): return cls(num_samples, seq_len, vocab_size)
    # sizes of the reference's presets (datasets/mod.rs:234-248)
    @classmethod
    def small(cls): return cls(100, 32, 1000)
    @classmethod
    def train(cls): return cls(10000, 64, 10000)
    @classmethod
    def test(cls): return cls(2000, 64, 10000)
    def len(self) -> int: return self.data.shape[0]
    def get(self, i): return self.data[i], self.labels[i]


class SyntheticSeq2SeqDataset(Dataset):
    """Source = random tokens, target = the reversed (or copied) source."""

    def __init__(self, num_samples: int = 1000, seq_len: int = 16, vocab_size: int = 100, task: str = "reverse", seed: int = 42):
        g = torch.Generator().manual_seed(seed)
        self.src = torch.randint(2, vocab_size, (num_samples, seq_len), generator=g)
        self.tgt = self.src.flip(1) if task == "reverse" else self.src.clone()

    @classmethod
    def reverse_task(cls, n, seq_len, vocab_size): return cls(n, seq_len, vocab_size, "reverse")
    @classmethod
    def copy_task(cls, n, seq_len, vocab_size): return cls(n, seq_len, vocab_size, "copy")
    def len(self) -> int: return self.src.shape[0]
    def get(self, i): return self.src[i], self.tgt[i]
