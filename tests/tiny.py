"""Tiny configurations of the architecture for the tests, and helpers that
write them as model folders with random weights.

A and B are the two tiny models of the benchmark description (with longer
position ranges so that long decoding fits); C adds what they lack: a sliding
window on some layers, one key/value head for five query heads, and sizes that
are neither powers of two nor multiples of 64.  Between them every size and
option differs: layers, widths, head counts and groups, head size,
intermediate size, vocabulary, theta, eps, tied or not, biases or not, window.
"""
from __future__ import annotations

import torch

from nncpu_b200.config import config_from_dict
from nncpu_b200.weights import write_model_folder

TINY = {
    "A": dict(architectures=["Qwen3ForCausalLM"], num_hidden_layers=2, hidden_size=64, num_attention_heads=4,
              num_key_value_heads=2, head_dim=16, intermediate_size=192, vocab_size=256, rope_theta=10000.0,
              rms_norm_eps=1e-6, tie_word_embeddings=True, attention_bias=False, max_position_embeddings=1024,
              eos_token_id=255),
    "B": dict(architectures=["Qwen3ForCausalLM"], num_hidden_layers=3, hidden_size=96, num_attention_heads=8,
              num_key_value_heads=2, head_dim=32, intermediate_size=160, vocab_size=384, rope_theta=1000000.0,
              rms_norm_eps=1e-5, tie_word_embeddings=False, attention_bias=True, max_position_embeddings=2048,
              eos_token_id=[382, 383]),
    "C": dict(architectures=["Qwen3ForCausalLM"], num_hidden_layers=4, hidden_size=80, num_attention_heads=5,
              num_key_value_heads=1, head_dim=48, intermediate_size=136, vocab_size=307, rope_theta=500000.0,
              rms_norm_eps=3e-6, tie_word_embeddings=False, attention_bias=False, max_position_embeddings=4096,
              use_sliding_window=True, sliding_window=40,
              layer_types=["sliding_attention", "full_attention", "sliding_attention", "full_attention"]),
    # head sizes the tensor-core attention kernels take: 64 with two heads per key/value head, and 128 with
    # eight heads on one key/value head and a window on the first layer
    "D": dict(architectures=["Qwen3ForCausalLM"], num_hidden_layers=2, hidden_size=128, num_attention_heads=4,
              num_key_value_heads=2, head_dim=64, intermediate_size=320, vocab_size=520, rope_theta=10000.0,
              rms_norm_eps=1e-6, tie_word_embeddings=True, attention_bias=False, max_position_embeddings=2048),
    "E": dict(architectures=["Qwen3ForCausalLM"], num_hidden_layers=2, hidden_size=192, num_attention_heads=8,
              num_key_value_heads=1, head_dim=128, intermediate_size=256, vocab_size=333, rope_theta=1000000.0,
              rms_norm_eps=1e-5, tie_word_embeddings=False, attention_bias=True, max_position_embeddings=2048,
              use_sliding_window=True, sliding_window=100, layer_types=["sliding_attention", "full_attention"]),
    # what the prompt kernels want: head size 128, even head counts (two heads of a block share a key/value
    # head; the q/k/v epilogue takes two heads a tile), a window longer than a 128-row tile on one layer
    "G": dict(architectures=["Qwen3ForCausalLM"], num_hidden_layers=2, hidden_size=256, num_attention_heads=4,
              num_key_value_heads=2, head_dim=128, intermediate_size=384, vocab_size=410, rope_theta=1000000.0,
              rms_norm_eps=1e-6, tie_word_embeddings=False, attention_bias=False, max_position_embeddings=4096,
              use_sliding_window=True, sliding_window=200, layer_types=["full_attention", "sliding_attention"]),
    # sizes that keep every fast path out: a width that is no multiple of 8, as many key/value heads as heads
    "F": dict(architectures=["Qwen3ForCausalLM"], num_hidden_layers=1, hidden_size=100, num_attention_heads=5,
              num_key_value_heads=5, head_dim=16, intermediate_size=90, vocab_size=257, rope_theta=20000.0,
              rms_norm_eps=2e-6, tie_word_embeddings=False, attention_bias=True, max_position_embeddings=512),
}


def tiny_config(name: str, **overrides):
    return config_from_dict(dict(TINY[name], **overrides))


def make_folder(path, name: str, seed: int = 0, store_dtype=torch.float32, vector_dtype=None, **overrides):
    """Writes tiny model ``name`` under ``path`` and returns the folder."""
    return write_model_folder(path, tiny_config(name, **overrides), seed, store_dtype, vector_dtype)
