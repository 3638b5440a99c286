"""Tiny configurations of the architecture for tests, and helpers shared by test files.

The three differ in every size and option: head counts and grouping (GQA, MQA, MHA
with a head size that is not hidden/heads), widths and vocabularies that are no power
of two, layer counts, eps, theta, rope scaling (none / llama3 with all three branches
hit / linear), tied or untied head, norm weights 1 or scattered.
"""
import json
import random

import torch

TINY_A = dict(
    architectures=["LlamaForCausalLM"], model_type="llama",
    num_hidden_layers=2, hidden_size=64, num_attention_heads=4, num_key_value_heads=2, head_dim=16,
    intermediate_size=192, vocab_size=256, rope_theta=10000.0, rope_scaling=None,
    tie_word_embeddings=True, rms_norm_eps=1e-5, max_position_embeddings=128)
TINY_A_INIT = dict(seed=11, norm_std=0.0)

TINY_B = dict(
    architectures=["LlamaForCausalLM"], model_type="llama",
    num_hidden_layers=3, hidden_size=96, num_attention_heads=3, num_key_value_heads=1, head_dim=32,
    intermediate_size=256, vocab_size=384, rope_theta=500000.0,
    rope_scaling=dict(rope_type="llama3", factor=32.0, low_freq_factor=1.0, high_freq_factor=4.0,
                      original_max_position_embeddings=64),
    tie_word_embeddings=False, rms_norm_eps=1e-6, max_position_embeddings=512)
TINY_B_INIT = dict(seed=23, norm_std=0.1)

# MHA, head_dim 48 although hidden / heads = 24, odd vocabulary and widths
TINY_C = dict(
    architectures=["LlamaForCausalLM"], model_type="llama",
    num_hidden_layers=1, hidden_size=72, num_attention_heads=3, num_key_value_heads=3, head_dim=48,
    intermediate_size=136, vocab_size=333, rope_theta=1000.0,
    rope_scaling=dict(rope_type="linear", factor=2.0),
    tie_word_embeddings=False, rms_norm_eps=1e-4, max_position_embeddings=256)
TINY_C_INIT = dict(seed=5, norm_std=0.2)

# head size 80 (a step of 16 that is neither 64 nor 128), an intermediate size that no fused epilogue takes,
# a hidden size that is no multiple of 64, more kv groups
TINY_D = dict(
    architectures=["LlamaForCausalLM"], model_type="llama",
    num_hidden_layers=2, hidden_size=200, num_attention_heads=6, num_key_value_heads=2, head_dim=80,
    intermediate_size=120, vocab_size=1000, rope_theta=250000.0, rope_scaling=None,
    tie_word_embeddings=True, rms_norm_eps=3e-6, max_position_embeddings=1024)
TINY_D_INIT = dict(seed=77, norm_std=0.05)

# head size 64 with an odd head count and one kv head, a width that no tile divides: every layer of a decode
# step of this one (and of F) runs inside the one-kernel decode path
TINY_E = dict(
    architectures=["LlamaForCausalLM"], model_type="llama",
    num_hidden_layers=3, hidden_size=208, num_attention_heads=3, num_key_value_heads=1, head_dim=64,
    intermediate_size=320, vocab_size=777, rope_theta=50000.0,
    rope_scaling=dict(rope_type="llama3", factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0,
                      original_max_position_embeddings=128),
    tie_word_embeddings=True, rms_norm_eps=2e-5, max_position_embeddings=1024)
TINY_E_INIT = dict(seed=31, norm_std=0.1)

# head size 128, two kv groups, a width above one weight tile's 512 columns plus a ragged rest
TINY_F = dict(
    architectures=["LlamaForCausalLM"], model_type="llama",
    num_hidden_layers=2, hidden_size=592, num_attention_heads=4, num_key_value_heads=2, head_dim=128,
    intermediate_size=1152, vocab_size=515, rope_theta=10000.0, rope_scaling=None,
    tie_word_embeddings=False, rms_norm_eps=1e-5, max_position_embeddings=1024)
TINY_F_INIT = dict(seed=41, norm_std=0.05)

TINIES = {"A": (TINY_A, TINY_A_INIT), "B": (TINY_B, TINY_B_INIT), "C": (TINY_C, TINY_C_INIT),
          "D": (TINY_D, TINY_D_INIT), "E": (TINY_E, TINY_E_INIT), "F": (TINY_F, TINY_F_INIT)}


def make_folder(cfg_dict, init, folder, std=0.02):
    """A model folder written by the library's random-weights mode."""
    from spissa_b200 import write_random_model
    from spissa_b200.config import config_from_dict
    cfg = config_from_dict(cfg_dict)
    write_random_model(cfg, folder, seed=init["seed"], std=std, norm_std=init["norm_std"])
    return folder


def random_prompt(vocab, n, seed):
    rng = random.Random(seed)
    return [rng.randrange(vocab) for _ in range(n)]


def rel_err(got: torch.Tensor, ref: torch.Tensor) -> float:
    """max |got − ref| over max |ref|, in float64."""
    got = got.detach().double().cpu()
    ref = ref.detach().double().cpu()
    return float((got - ref).abs().max() / ref.abs().max().clamp_min(1e-30))


# Allowed distance from the float64 plain implementation, as a fraction of the largest
# logit. float32: products of a few hundred terms accumulate about 1e-6. bfloat16:
# activations are rounded to 8 bits of mantissa (2^-9 relative) between kernels.
TOL = {"float32": 5e-6, "bfloat16": 1e-2}
