"""The tiny configurations the tests run on, and helpers to make model folders from them.

A and B differ in every size and option: layer pattern and count, width, head counts and
grouping, head size, taps, feed-forward width, vocabulary, eps, rope bases, rope factors,
window, tied or own head, output gate.  C is B with the post-norms off and the gate on.
L has a window larger than one cache page and a pattern that makes the ring wrap.
"""
import os

TINY_A = dict(
    architecture="lfm3", vocab_size=256, hidden_size=64, intermediate_size=176, num_hidden_layers=4,
    layer_types=["conv", "sliding_attention", "conv", "full_attention"],
    num_attention_heads=4, num_key_value_heads=2, head_dim=16, conv_L_cache=3, sliding_window=16,
    rope_theta=10000.0, norm_eps=1e-5, tie_word_embeddings=True, max_position_embeddings=1024,
    eos_token_id=7, post_norm=True, attn_output_gate=True)
RANDOM_A = dict(std=0.02, norm_weights="random", rope_factors="ones")

TINY_B = dict(
    architecture="lfm3", vocab_size=384, hidden_size=96, intermediate_size=272, num_hidden_layers=6,
    layer_types=["conv", "conv", "full_attention", "conv", "sliding_attention", "full_attention"],
    num_attention_heads=4, num_key_value_heads=1, head_dim=24, conv_L_cache=4, sliding_window=8,
    rope_theta=1000000.0, rope_theta_sliding=10000.0, norm_eps=1e-6, tie_word_embeddings=False,
    max_position_embeddings=2048, eos_token_id=[3, 11], post_norm=True, attn_output_gate=False)
RANDOM_B = dict(std=0.05, norm_weights="random", rope_factors="uniform")

TINY_C = dict(TINY_B, post_norm=False, attn_output_gate=True)

TINY_L = dict(
    architecture="lfm3", vocab_size=300, hidden_size=80, intermediate_size=200, num_hidden_layers=3,
    layer_types=["sliding_attention", "conv", "full_attention"],
    num_attention_heads=5, num_key_value_heads=5, head_dim=32, conv_L_cache=2, sliding_window=70,
    rope_theta=50000.0, rope_theta_sliding=777.0, norm_eps=1e-5, tie_word_embeddings=True,
    max_position_embeddings=4096, post_norm=True, attn_output_gate=True)
RANDOM_L = dict(std=0.05, norm_weights="random", rope_factors="uniform")

# R runs its layers in an order of its own: layer 1 (sliding attention) three times, layer 2 last
TINY_R = dict(TINY_A, layer_order=[0, 1, 1, 3, 2, 1], eos_token_id=[])

ALL = {"A": (TINY_A, RANDOM_A), "B": (TINY_B, RANDOM_B), "C": (TINY_C, RANDOM_B), "L": (TINY_L, RANDOM_L),
       "R": (TINY_R, RANDOM_B)}


def make_folder(tmp, name, seed=0):
    """Write the named tiny model into `tmp/name` and return the path."""
    from catena_models_b200.weights.random_init import write_random_model

    config, rnd = ALL[name]
    return write_random_model(os.path.join(str(tmp), name), config, seed, **rnd)


def random_prompt(n, vocab, seed):
    import torch

    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()
