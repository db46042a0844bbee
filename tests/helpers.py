"""Tiny configurations and small utilities shared by the tests."""
import random

import torch

import citlali_b200 as cb

# Three tiny Qwen3 configurations that differ in every size and option: layers, width, head
# counts and group size, head size (16 / 32 / 48), intermediate size, vocabulary (two of them
# no power of two), rotary base, eps, tied or untied head, longest sequence.
TINY = {
    "A": dict(architectures=["Qwen3ForCausalLM"], num_hidden_layers=2, hidden_size=64, num_attention_heads=4,
              num_key_value_heads=2, head_dim=16, intermediate_size=192, vocab_size=512, rope_theta=1e6,
              rms_norm_eps=1e-6, tie_word_embeddings=True, max_position_embeddings=128, hidden_act="silu",
              attention_bias=False),
    "B": dict(architectures=["Qwen3ForCausalLM"], num_hidden_layers=3, hidden_size=96, num_attention_heads=8,
              num_key_value_heads=2, head_dim=32, intermediate_size=160, vocab_size=1000, rope_theta=1e4,
              rms_norm_eps=1e-5, tie_word_embeddings=False, max_position_embeddings=256, hidden_act="silu",
              attention_bias=False),
    "C": dict(architectures=["Qwen3ForCausalLM"], num_hidden_layers=2, hidden_size=120, num_attention_heads=6,
              num_key_value_heads=3, head_dim=48, intermediate_size=208, vocab_size=777, rope_theta=5e5,
              rms_norm_eps=3e-6, tie_word_embeddings=False, max_position_embeddings=1024, hidden_act="silu",
              attention_bias=False, eos_token_id=[5, 9]),
    # the benchmark's head geometry (head size 128, four query heads per key/value head) at a small width,
    # with sequences long enough for the prompt-sized kernels: many 64-key tiles, more than 128 rows
    "D": dict(architectures=["Qwen3ForCausalLM"], num_hidden_layers=2, hidden_size=256, num_attention_heads=8,
              num_key_value_heads=2, head_dim=128, intermediate_size=768, vocab_size=1536, rope_theta=1e6,
              rms_norm_eps=1e-6, tie_word_embeddings=False, max_position_embeddings=2048, hidden_act="silu",
              attention_bias=False),
}
SEEDS = {"A": 11, "B": 23, "C": 37, "D": 41}


def tiny_config(name):
    return cb.config_from_dict(dict(TINY[name]))


def make_model_dir(path, name, stored="float32", seed=None):
    cb.write_random_model(path, tiny_config(name), SEEDS[name] if seed is None else seed, dtype=stored)
    return path


def random_tokens(vocab, count, seed):
    rng = random.Random(seed)
    return [rng.randrange(vocab) for _ in range(count)]


def read_f32(path, vocab):
    import numpy as np
    return torch.from_numpy(np.fromfile(path, dtype="<f4").reshape(-1, vocab).copy())
