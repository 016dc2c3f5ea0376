"""The tiny configurations the tests run: they differ in every size and option."""
import os

import torch

from leone_b200.config.qwen3 import Qwen3Config
from leone_b200.weights.random_init import write_random_model

TINY_A = dict(architectures=["Qwen3ForCausalLM"], num_hidden_layers=2, hidden_size=64,
              num_attention_heads=4, num_key_value_heads=2, head_dim=16, intermediate_size=128,
              vocab_size=256, rope_theta=10000.0, rms_norm_eps=1e-6, max_position_embeddings=128,
              tie_word_embeddings=True, eos_token_id=255)
TINY_B = dict(architectures=["Qwen3ForCausalLM"], num_hidden_layers=3, hidden_size=96,
              num_attention_heads=6, num_key_value_heads=3, head_dim=32, intermediate_size=224,
              vocab_size=384, rope_theta=1000000.0, rms_norm_eps=1e-5, max_position_embeddings=256,
              tie_word_embeddings=False)
# Sizes that are no power of two anywhere, one KV head per 5 query heads, head size 48,
# long enough positions for the replay tests.
TINY_C = dict(architectures=["Qwen3ForCausalLM"], num_hidden_layers=2, hidden_size=80,
              num_attention_heads=5, num_key_value_heads=1, head_dim=48, intermediate_size=176,
              vocab_size=331, rope_theta=50000.0, rms_norm_eps=3e-6, max_position_embeddings=512,
              tie_word_embeddings=False)
# Head size 64 (the smallest that the tensor-memory prompt attention and the fused decode
# preparation take), three query heads per KV head (does not divide a block's 128 rows).
TINY_D = dict(architectures=["Qwen3ForCausalLM"], num_hidden_layers=2, hidden_size=192,
              num_attention_heads=6, num_key_value_heads=2, head_dim=64, intermediate_size=320,
              vocab_size=500, rope_theta=200000.0, rms_norm_eps=2e-6, max_position_embeddings=256,
              tie_word_embeddings=True)
PAGE_TOKENS = {"A": 4, "B": 8, "C": 16, "D": 16}
CONFIGS = {"A": TINY_A, "B": TINY_B, "C": TINY_C, "D": TINY_D}


def tiny_config(which):
    return Qwen3Config.from_dict(CONFIGS[which])


def make_folder(tmp_path, which, seed=1234, store_dtype=torch.float32):
    folder = os.path.join(str(tmp_path), f"tiny_{which}_{seed}")
    if not os.path.isdir(folder):
        write_random_model(tiny_config(which), folder, seed, store_dtype)
    return folder
