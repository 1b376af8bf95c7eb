"""Text processing (crates/axonml-text)."""
from .datasets import LanguageModelDataset, SyntheticSentimentDataset, SyntheticSeq2SeqDataset, TextDataset
from .tokenizer import (BasicBPETokenizer, CharTokenizer, NGramTokenizer, Tokenizer, UnigramTokenizer,
                        WhitespaceTokenizer, WordPunctTokenizer)
from .vocab import BOS, EOS, MASK, PAD, UNK, Vocab

# the reference's constant names (crates/axonml-text/src/vocab.rs:15-23)
BOS_TOKEN, EOS_TOKEN, MASK_TOKEN, PAD_TOKEN, UNK_TOKEN = BOS, EOS, MASK, PAD, UNK
