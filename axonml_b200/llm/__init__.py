"""Language models and generation (crates/axonml-llm)."""
from ..nn import RMSNorm
from . import error, hub
from .attention import FlashAttention, FlashAttentionConfig, KVCache, LayerKVCache, scaled_dot_product_attention
from .config import BertConfig, GPT2Config, LLaMAConfig, MistralConfig, PhiConfig
from .embedding import BertEmbedding, PositionalEmbedding, SinusoidalPositionalEncoding, TokenEmbedding
from .error import LLMError
from .generation import Beam, BeamSearch, GenerationConfig, TextGenerator
from .gpt2 import GPT2, CausalSelfAttention, FeedForward, GPT2Embedding, GPT2LMHead, TransformerBlock
from .llama import (LLaMA, LLaMAAttention, LLaMADecoderLayer, LLaMAForCausalLM, LLaMAMLP,
                    RotaryEmbedding)
from .bert import (Bert, BertForMaskedLM, BertForSequenceClassification, BertLMPredictionHead, BertPooler,
                   BertPredictionHeadTransform, map_bert_weights)
from .hf_loader import (HFLoader, HFTokenizer, LLaMAWeightMapper, LoadResult, LoadStateDict, MistralWeightMapper, PhiWeightMapper,
                        SpecialTokens, TensorInfo, WeightMapper, load_llama_from_hf,
                        load_mistral_from_hf, load_with_mapping, map_axonml_to_hf, map_gpt2_weights, map_hf_to_axonml,
                        map_llama_weights, map_llama_weights_alt)
from .hub import PretrainedLLM, llm_registry
from .hub import download_weights as download_llm_weights
from .mistral_phi import (Mistral, MistralAttention, MistralDecoderLayer, MistralForCausalLM, MistralMLP, Phi, PhiAttention,
                          PhiDecoderLayer, PhiForCausalLM, PhiMLP)
from .transformer import (MultiHeadSelfAttention, TransformerConfig, TransformerDecoder, TransformerDecoderBlock,
                          TransformerEncoder, TransformerEncoderBlock)
