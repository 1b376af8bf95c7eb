"""Tokenizers (crates/axonml-text/src/tokenizer.rs:16-384): Whitespace, Char, WordPunct, NGram,
BasicBPE (trainable merges) and Unigram."""
from __future__ import annotations

import collections
import re


class Tokenizer:
    def tokenize(self, text: str) -> list: raise NotImplementedError
    def __call__(self, text: str) -> list: return self.tokenize(text)


class WhitespaceTokenizer(Tokenizer):
    def __init__(self, lowercase: bool = False): self._lowercase = lowercase
    @classmethod
    def new(cls): return cls()
    @classmethod
    def lowercase(cls):
        """Tokenizer that lower-cases its input first."""
        return cls(True)
    def tokenize(self, text): return (text.lower() if self._lowercase else text).split()


class CharTokenizer(Tokenizer):
    def __init__(self, include_whitespace: bool = True): self.include_whitespace = include_whitespace
    @classmethod
    def new(cls): return cls()
    @classmethod
    def no_whitespace(cls):
        """Tokenizer that drops blanks instead of emitting them as tokens."""
        return cls(False)
    def tokenize(self, text): return [c for c in text if self.include_whitespace or not c.isspace()]


class WordPunctTokenizer(Tokenizer):
    def __init__(self, lowercase: bool = False): self._lowercase = lowercase
    @classmethod
    def new(cls): return cls()
    @classmethod
    def lowercase(cls): return cls(True)
    def tokenize(self, text): return re.findall(r"\w+|[^\w\s]", text.lower() if self._lowercase else text)


class NGramTokenizer(Tokenizer):
    def __init__(self, n: int, char_level: bool = False): self.n, self.char_level = n, char_level
    @classmethod
    def word_ngrams(cls, n): return cls(n, False)
    @classmethod
    def char_ngrams(cls, n): return cls(n, True)
    def tokenize(self, text):
        units = list(text) if self.char_level else text.split()
        sep = "" if self.char_level else " "
        return [sep.join(units[i:i + self.n]) for i in range(max(0, len(units) - self.n + 1))]


class BasicBPETokenizer(Tokenizer):
    """Byte-pair encoding trained on a corpus: start from characters (+ ``</w>`` end-of-word marker)
    and repeatedly merge the most frequent adjacent pair."""

    def __init__(self):
        self.merges: list = []
        self.vocab: dict = {}

    @classmethod
    def new(cls): return cls()

    def train(self, corpus, num_merges: int) -> None:
        words = collections.Counter()
        for line in ([corpus] if isinstance(corpus, str) else corpus):
            for w in line.split():
                words[tuple(w) + ("</w>",)] += 1
        for _ in range(num_merges):
            pairs = collections.Counter()
            for w, c in words.items():
                for a, b in zip(w, w[1:]):
                    pairs[(a, b)] += c
            if not pairs:
                break
            best = max(pairs, key=lambda p: (pairs[p], p))
            self.merges.append(best)
            new = collections.Counter()
            for w, c in words.items():
                new[self._merge(w, best)] += c
            words = new
        toks = {t for w in words for t in w}
        self.vocab = {t: i for i, t in enumerate(sorted(toks))}

    def get_vocab(self) -> list:
        """The learned symbols in index order."""
        return sorted(self.vocab, key=self.vocab.get)

    @staticmethod
    def _merge(w, pair):
        out, i = [], 0
        while i < len(w):
            if i + 1 < len(w) and (w[i], w[i + 1]) == pair:
                out.append(w[i] + w[i + 1])
                i += 2
            else:
                out.append(w[i])
                i += 1
        return tuple(out)

    def tokenize(self, text):
        out = []
        for w in text.split():
            sym = tuple(w) + ("</w>",)
            for m in self.merges:
                sym = self._merge(sym, m)
            out.extend(sym)
        return out


class UnigramTokenizer(Tokenizer):
    """Greedy longest-match segmentation over a scored vocabulary."""

    def __init__(self, vocab: dict | None = None): self.vocab = dict(vocab or {})
    @classmethod
    def new(cls, vocab): return cls(vocab)
    @classmethod
    def from_tokens(cls, tokens):
        """Vocabulary of the given pieces, all with the same score."""
        return cls({t: 1.0 for t in tokens})

    def train(self, corpus, vocab_size: int) -> None:
        c = collections.Counter()
        for line in ([corpus] if isinstance(corpus, str) else corpus):
            for w in line.split():
                for i in range(len(w)):
                    for j in range(i + 1, min(len(w), i + 8) + 1):
                        c[w[i:j]] += 1
        singles = {k: v for k, v in c.items() if len(k) == 1}
        multi = dict(collections.Counter({k: v * len(k) for k, v in c.items() if len(k) > 1}).most_common(max(0, vocab_size - len(singles))))
        total = sum(singles.values()) + sum(multi.values()) or 1
        import math
        self.vocab = {k: math.log(v / total) for k, v in {**singles, **multi}.items()}

    def tokenize(self, text):
        out = []
        for w in text.split():
            i = 0
            while i < len(w):
                for j in range(min(len(w), i + 16), i, -1):
                    if w[i:j] in self.vocab or j == i + 1:
                        out.append(w[i:j])
                        i = j
                        break
        return out
