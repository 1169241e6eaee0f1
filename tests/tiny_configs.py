"""The tests' own small configurations: two Llama shapes that differ in every size and option."""
from __future__ import annotations

# 2 layers, 4 query heads over 2 kv heads of 16, untied head, theta 1e4, eps 1e-5
TINY_A = dict(
    architectures=["LlamaForCausalLM"], model_type="llama", hidden_size=64, intermediate_size=176, num_hidden_layers=2,
    num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=128, vocab_size=256, rms_norm_eps=1e-5,
    rope_theta=10000.0, tie_word_embeddings=False, hidden_act="silu", attention_bias=False, bos_token_id=1,
    eos_token_id=2, torch_dtype="bfloat16",
)
SEED_A = 0

# 3 layers, 6 query heads over 2 kv heads of 32, tied head, theta 5e5, eps 1e-6, sizes that are no power of two
TINY_B = dict(
    architectures=["LlamaForCausalLM"], model_type="llama", hidden_size=192, intermediate_size=512, num_hidden_layers=3,
    num_attention_heads=6, num_key_value_heads=2, max_position_embeddings=256, vocab_size=384, rms_norm_eps=1e-6,
    rope_theta=500000.0, tie_word_embeddings=True, hidden_act="silu", attention_bias=False, bos_token_id=1,
    eos_token_id=2, torch_dtype="bfloat16",
)
SEED_B = 2

# 1 layer, 3 query heads = 3 kv heads of 48 (explicit head_dim, not hidden / heads), odd vocabulary and widths
TINY_C = dict(
    architectures=["LlamaForCausalLM"], model_type="llama", hidden_size=80, intermediate_size=112, num_hidden_layers=1,
    num_attention_heads=3, num_key_value_heads=3, head_dim=48, max_position_embeddings=320, vocab_size=131,
    rms_norm_eps=1e-4, rope_theta=777.0, tie_word_embeddings=False, hidden_act="silu", attention_bias=False,
    bos_token_id=None, eos_token_id=None, torch_dtype="bfloat16",
)
SEED_C = 5

# 2 layers, 8 query heads over 2 kv heads of 128 (the head size of the larger Llama checkpoints), long context
TINY_D = dict(
    architectures=["LlamaForCausalLM"], model_type="llama", hidden_size=320, intermediate_size=200, num_hidden_layers=2,
    num_attention_heads=8, num_key_value_heads=2, head_dim=128, max_position_embeddings=1100, vocab_size=517,
    rms_norm_eps=1e-5, rope_theta=500000.0, tie_word_embeddings=False, hidden_act="silu", attention_bias=False,
    bos_token_id=1, eos_token_id=2, torch_dtype="bfloat16",
)
SEED_D = 7

# 2 layers, 6 query heads over 3 kv heads of 64 (the head size of the 1.1B model), widths that are no power of two
TINY_E = dict(
    architectures=["LlamaForCausalLM"], model_type="llama", hidden_size=200, intermediate_size=304, num_hidden_layers=2,
    num_attention_heads=6, num_key_value_heads=3, head_dim=64, max_position_embeddings=700, vocab_size=333,
    rms_norm_eps=1e-5, rope_theta=10000.0, tie_word_embeddings=False, hidden_act="silu", attention_bias=False,
    bos_token_id=1, eos_token_id=2, torch_dtype="bfloat16",
)
SEED_E = 11

ALL = {"a": (TINY_A, SEED_A), "b": (TINY_B, SEED_B), "c": (TINY_C, SEED_C), "d": (TINY_D, SEED_D), "e": (TINY_E, SEED_E)}
