"""Language models and generation (crates/axonml-llm)."""
from .attention import FlashAttention, KVCache, LayerKVCache, scaled_dot_product_attention
from .config import BertConfig, GPT2Config, LLaMAConfig, MistralConfig, PhiConfig
from .generation import BeamSearch, GenerationConfig, TextGenerator
from .gpt2 import GPT2, CausalSelfAttention, FeedForward, GPT2Embedding, GPT2LMHead, TransformerBlock
from .llama import (LLaMA, LLaMAAttention, LLaMADecoderLayer, LLaMAForCausalLM, LLaMAMLP,
                    RotaryEmbedding)
from .bert import Bert, BertForMaskedLM, BertForSequenceClassification
from .hf_loader import (HFLoader, HFTokenizer, LoadStateDict, map_gpt2_weights, map_llama_weights,
                        map_llama_weights_alt)
from .mistral_phi import Mistral, MistralForCausalLM, Phi, PhiForCausalLM
