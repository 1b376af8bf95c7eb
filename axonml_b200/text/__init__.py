"""Text processing (crates/axonml-text)."""
from .datasets import LanguageModelDataset, SyntheticSentimentDataset, SyntheticSeq2SeqDataset, TextDataset
from .tokenizer import (BasicBPETokenizer, CharTokenizer, NGramTokenizer, Tokenizer, UnigramTokenizer,
                        WhitespaceTokenizer, WordPunctTokenizer)
from .vocab import BOS, EOS, MASK, PAD, UNK, Vocab
