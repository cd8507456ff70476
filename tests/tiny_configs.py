"""Tiny configurations of the architecture for tests.  They differ in every size and
option: head counts and groups, head size, widths that are no power of two, number of
layers, vocabulary, the norms' eps, the rotary base, tied or untied output matrix, number
of MTP heads, page size, window, layer order."""
from __future__ import annotations

import os
import tempfile

import torch

TINY_A = dict(architecture="gqa_mtp_transformer", vocab_size=256, hidden_size=64, num_layers=2, num_heads=4,
              num_kv_heads=2, head_dim=16, ffn_hidden=192, rms_norm_eps=1e-5, rope_theta=10000.0,
              max_context=128, tie_word_embeddings=True, num_mtp_heads=1)
TINY_A_PAGE = 16

TINY_B = dict(architecture="gqa_mtp_transformer", vocab_size=512, hidden_size=128, num_layers=3, num_heads=4,
              num_kv_heads=1, head_dim=32, ffn_hidden=352, rms_norm_eps=1e-6, rope_theta=500000.0,
              max_context=256, tie_word_embeddings=False, num_mtp_heads=2)
TINY_B_PAGE = 8

# odd sizes: width 120 with 6 heads of 48 (so H*hd != width), 3 query heads per kv head,
# vocabulary 301, a window of 24 keys on all layers but layer 0, layer 1 run twice
TINY_C = dict(architecture="gqa_mtp_transformer", vocab_size=301, hidden_size=120, num_layers=2, num_heads=6,
              num_kv_heads=2, head_dim=48, ffn_hidden=200, rms_norm_eps=3e-6, rope_theta=25000.0,
              max_context=192, tie_word_embeddings=True, num_mtp_heads=1, sliding_window=24,
              full_attention_layers=[0], layer_order=[0, 1, 1])
TINY_C_PAGE = 4

# a layer that reads another layer's keys and values
TINY_D = dict(architecture="gqa_mtp_transformer", vocab_size=200, hidden_size=48, num_layers=3, num_heads=3,
              num_kv_heads=3, head_dim=16, ffn_hidden=80, rms_norm_eps=1e-5, rope_theta=10000.0,
              max_context=96, tie_word_embeddings=False, num_mtp_heads=0, layer_order=[0, 1, 2],
              cache_source=[None, None, 1])
TINY_D_PAGE = 16

# heads of 64 (the smaller of the two head sizes that the tcgen05 attention kernel takes), 3 query heads per kv
# head, pages of 32, a window of 100 keys on the second layer: prompts of more than 64 tokens run that kernel
TINY_E = dict(architecture="gqa_mtp_transformer", vocab_size=777, hidden_size=192, num_layers=2, num_heads=6,
              num_kv_heads=2, head_dim=64, ffn_hidden=320, rms_norm_eps=1e-5, rope_theta=50000.0, max_context=512,
              tie_word_embeddings=False, num_mtp_heads=1, sliding_window=100, full_attention_layers=[0])
TINY_E_PAGE = 32

# a windowed layer whose cache a later layer reads (with the same window: pages behind it are given back while
# both still run), the first layer unwindowed, 5 query heads on one kv head, pages of 8
TINY_F = dict(architecture="gqa_mtp_transformer", vocab_size=190, hidden_size=80, num_layers=3, num_heads=5,
              num_kv_heads=1, head_dim=16, ffn_hidden=136, rms_norm_eps=2e-6, rope_theta=30000.0,
              max_context=160, tie_word_embeddings=True, num_mtp_heads=1, sliding_window=19,
              full_attention_layers=[0, 3], layer_order=[0, 1, 2], cache_source=[None, None, 1])
TINY_F_PAGE = 8

# a context long enough to decode across the 512-, 1024- and 2048-key bounds that decode graphs are keyed by
TINY_G = dict(architecture="gqa_mtp_transformer", vocab_size=320, hidden_size=96, num_layers=2, num_heads=4,
              num_kv_heads=2, head_dim=64, ffn_hidden=160, rms_norm_eps=1e-6, rope_theta=100000.0,
              max_context=2304, tie_word_embeddings=True, num_mtp_heads=1)
TINY_G_PAGE = 16

# the layer sizes of the upstream 0.9B model (Config/config.py:11-23), two layers and one MTP head of them
WIDE = dict(architecture="gqa_mtp_transformer", vocab_size=49152, hidden_size=1536, num_layers=2, num_heads=12,
            num_kv_heads=3, head_dim=128, ffn_hidden=4096, rms_norm_eps=2e-8, rope_theta=10000.0, max_context=4096,
            tie_word_embeddings=True, num_mtp_heads=1)
WIDE_PAGE = 16

ALL = {"A": (TINY_A, TINY_A_PAGE, 0), "B": (TINY_B, TINY_B_PAGE, 1), "C": (TINY_C, TINY_C_PAGE, 2),
       "D": (TINY_D, TINY_D_PAGE, 3), "E": (TINY_E, TINY_E_PAGE, 5), "F": (TINY_F, TINY_F_PAGE, 6), "G": (TINY_G, TINY_G_PAGE, 7),
       "WIDE": (WIDE, WIDE_PAGE, 4)}


def make_model_folder(cfg_dict: dict, seed: int, folder: str, std: float = 0.02) -> str:
    """Write config.json + model.safetensors with the engine's random-weights mode."""
    from tiny_inference_server_b200.registry import config_from_dict
    from tiny_inference_server_b200.weights import write_random_model

    cfg = config_from_dict(dict(cfg_dict))
    return write_random_model(folder, cfg, seed, std=std)


def random_prompts(vocab: int, lengths, seed: int):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, vocab, (n,), generator=g).tolist() for n in lengths]
