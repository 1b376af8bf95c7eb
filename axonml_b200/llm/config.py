"""Model configurations with the reference's presets (crates/axonml-llm/src/config.rs:147-275 for
GPT-2 and BERT, llama.rs:29-121 for LLaMA, mistral.rs:40-93, phi.rs) plus the two architectures
named by the benchmark configurations: ``GPT2Config.gpt_1_3b()`` (24 x 2048, 16 heads, FFN 8192,
ctx 2048) and ``LLaMAConfig.llama3_8b()``."""
from __future__ import annotations

import dataclasses


@dataclasses.dataclass
class GPT2Config:
    vocab_size: int = 50257
    n_ctx: int = 1024
    n_embd: int = 768
    n_layer: int = 12
    n_head: int = 12
    dropout: float = 0.1
    attn_dropout: float = 0.1
    resid_dropout: float = 0.1
    layer_norm_eps: float = 1e-5
    activation: str = "gelu"
    bos_token_id: int = 50256
    eos_token_id: int = 50256

    @classmethod
    def small(cls): return cls()
    @classmethod
    def medium(cls): return cls(n_embd=1024, n_layer=24, n_head=16)
    @classmethod
    def large(cls): return cls(n_embd=1280, n_layer=36, n_head=20)
    @classmethod
    def xl(cls): return cls(n_embd=1600, n_layer=48, n_head=25)
    @classmethod
    def tiny(cls): return cls(vocab_size=1000, n_ctx=128, n_embd=128, n_layer=2, n_head=2,
                              bos_token_id=0, eos_token_id=0)

    @classmethod
    def gpt_1_3b(cls):
        """24 layers, d_model 2048, 16 heads of 128, FFN 8192 GELU, learned positions, ctx 2048."""
        return cls(n_ctx=2048, n_embd=2048, n_layer=24, n_head=16, dropout=0.0, attn_dropout=0.0,
                   resid_dropout=0.0)

    def head_dim(self) -> int: return self.n_embd // self.n_head
    def intermediate_size(self) -> int: return 4 * self.n_embd

    def padded_vocab(self, multiple: int = 128) -> int:
        return (self.vocab_size + multiple - 1) // multiple * multiple


@dataclasses.dataclass
class LLaMAConfig:
    vocab_size: int = 32000
    hidden_size: int = 4096
    intermediate_size: int = 11008
    num_hidden_layers: int = 32
    num_attention_heads: int = 32
    num_key_value_heads: int = 32
    max_position_embeddings: int = 4096
    rms_norm_eps: float = 1e-5
    rope_theta: float = 10000.0
    attention_dropout: float = 0.0
    hidden_dropout: float = 0.0

    @classmethod
    def llama2_7b(cls): return cls()
    @classmethod
    def llama2_13b(cls): return cls(hidden_size=5120, intermediate_size=13824, num_hidden_layers=40,
                                    num_attention_heads=40, num_key_value_heads=40)
    @classmethod
    def llama3_8b(cls): return cls(vocab_size=128256, intermediate_size=14336, num_key_value_heads=8,
                                   max_position_embeddings=8192, rope_theta=500000.0)
    @classmethod
    def tiny(cls): return cls(vocab_size=1000, hidden_size=128, intermediate_size=256,
                              num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                              max_position_embeddings=128)

    def head_dim(self) -> int: return self.hidden_size // self.num_attention_heads
    def num_kv_groups(self) -> int: return self.num_attention_heads // self.num_key_value_heads


@dataclasses.dataclass
class MistralConfig(LLaMAConfig):
    sliding_window: int | None = 4096

    @classmethod
    def mistral_7b(cls): return cls(vocab_size=32000, intermediate_size=14336, num_key_value_heads=8,
                                    max_position_embeddings=32768, rope_theta=10000.0, sliding_window=4096)
    @classmethod
    def mistral_7b_instruct(cls):
        """Mistral-7B-Instruct v0.2: the 7B architecture without a sliding window and with rope theta 1e6."""
        return cls(vocab_size=32000, intermediate_size=14336, num_key_value_heads=8, max_position_embeddings=32768, rope_theta=1e6,
                   sliding_window=None)

    @classmethod
    def mixtral_8x7b(cls): return cls(vocab_size=32000, intermediate_size=14336, num_key_value_heads=8,
                                      max_position_embeddings=32768, rope_theta=1e6, sliding_window=None)
    @classmethod
    def tiny(cls): return cls(vocab_size=1000, hidden_size=128, intermediate_size=256, num_hidden_layers=2,
                              num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=128,
                              sliding_window=32)


@dataclasses.dataclass
class PhiConfig:
    vocab_size: int = 51200
    hidden_size: int = 2560
    intermediate_size: int = 10240
    num_hidden_layers: int = 32
    num_attention_heads: int = 32
    num_key_value_heads: int = 32
    max_position_embeddings: int = 2048
    layer_norm_eps: float = 1e-5
    rope_theta: float = 10000.0
    partial_rotary_factor: float = 0.4
    parallel_attn: bool = True

    @classmethod
    def phi1(cls): return cls(hidden_size=2048, intermediate_size=8192, num_hidden_layers=24,
                              partial_rotary_factor=0.5)
    @classmethod
    def phi2(cls): return cls()
    @classmethod
    def phi3_mini(cls): return cls(vocab_size=32064, hidden_size=3072, intermediate_size=8192,
                                   max_position_embeddings=4096, partial_rotary_factor=1.0, parallel_attn=False)
    @classmethod
    def tiny(cls): return cls(vocab_size=1000, hidden_size=128, intermediate_size=256, num_hidden_layers=2,
                              num_attention_heads=4, num_key_value_heads=4, max_position_embeddings=128)

    def head_dim(self) -> int: return self.hidden_size // self.num_attention_heads

    def rotary_dim(self) -> int:
        """Leading features of each head that are rotated (an even number)."""
        return int(self.head_dim() * self.partial_rotary_factor) // 2 * 2


@dataclasses.dataclass
class BertConfig:
    vocab_size: int = 30522
    hidden_size: int = 768
    num_hidden_layers: int = 12
    num_attention_heads: int = 12
    intermediate_size: int = 3072
    hidden_dropout_prob: float = 0.1
    attention_probs_dropout_prob: float = 0.1
    max_position_embeddings: int = 512
    type_vocab_size: int = 2
    layer_norm_eps: float = 1e-12

    @classmethod
    def base(cls): return cls()
    @classmethod
    def large(cls): return cls(hidden_size=1024, num_hidden_layers=24, num_attention_heads=16, intermediate_size=4096)
    @classmethod
    def tiny(cls): return cls(vocab_size=1000, hidden_size=128, num_hidden_layers=2, num_attention_heads=2,
                              intermediate_size=256, max_position_embeddings=128)

    def head_dim(self) -> int: return self.hidden_size // self.num_attention_heads
