"""Shared fixtures: two tiny Qwen3 configurations that differ in every size
and option, their model folders with random weights (written to a temporary
folder, never committed), and the tolerances the comparisons use."""
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

# Tiny A: tied head, head_dim 16, group 2, theta 1e4, eps 1e-6.
TINY_A = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", hidden_act="silu",
              num_hidden_layers=2, hidden_size=64, num_attention_heads=4, num_key_value_heads=2,
              head_dim=16, intermediate_size=128, vocab_size=256, rope_theta=10000.0,
              rms_norm_eps=1e-6, tie_word_embeddings=True, max_position_embeddings=128)
# Tiny B: untied head, head_dim 32 with heads * head_dim != hidden, group 3,
# sizes that are no power of two, theta 1e6, eps 1e-5.
TINY_B = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", hidden_act="silu",
              num_hidden_layers=3, hidden_size=96, num_attention_heads=6, num_key_value_heads=2,
              head_dim=32, intermediate_size=224, vocab_size=384, rope_theta=1000000.0,
              rms_norm_eps=1e-5, tie_word_embeddings=False, max_position_embeddings=256)
# Tiny C: head_dim 48 (a step of 16, no power of two), one key/value head,
# odd vocabulary, more layers, long context for the decoding tests.
TINY_C = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", hidden_act="silu",
              num_hidden_layers=4, hidden_size=80, num_attention_heads=3, num_key_value_heads=1,
              head_dim=48, intermediate_size=136, vocab_size=331, rope_theta=50000.0,
              rms_norm_eps=3e-6, tie_word_embeddings=False, max_position_embeddings=1024)
# Tiny D: head_dim 64 with three query heads per key/value head: the head
# layout the split-key decode kernel takes.
TINY_D = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", hidden_act="silu",
              num_hidden_layers=2, hidden_size=128, num_attention_heads=6, num_key_value_heads=2,
              head_dim=64, intermediate_size=192, vocab_size=500, rope_theta=100000.0,
              rms_norm_eps=1e-6, tie_word_embeddings=True, max_position_embeddings=768)
TINY = {"A": (TINY_A, 0, 4), "B": (TINY_B, 1, 8), "C": (TINY_C, 2, 16), "D": (TINY_D, 3, 16)}  # config, seed, page size

# Stated tolerances on logits (tiny models: |logit| stays below about 2).
# float32: the engine against the float64 plain implementation; measured
# errors are below 1e-6. bfloat16: against the plain implementation that rounds
# activations where the engine stores them, and against the unrounded one.
TOL_F32 = 2e-5
TOL_BF16_VS_ROUNDED = 1.5e-2
TOL_BF16_VS_EXACT = 3e-2
# However the work is cut or batched: float32 kernels keep one order of
# additions per output, so the bound is rounding of the matrix products only.
TOL_CUTS_F32 = 2e-6
TOL_CUTS_BF16 = 1.5e-2


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200)")


@pytest.fixture(scope="session")
def model_folders(tmp_path_factory):
    """name -> (folder, config dict, tensors as float64 numpy, page size)."""
    import plain_qwen3 as plain
    from metallix_b200 import Qwen3Config, write_model_folder
    out = {}
    for name, (raw, seed, page) in TINY.items():
        folder = str(tmp_path_factory.mktemp(f"tiny_{name}"))
        # bfloat16 matrices with float32 norm weights: both engines and the
        # plain implementation then use exactly the same values.
        write_model_folder(folder, Qwen3Config.from_dict(raw), seed, dtype="bfloat16",
                           norm_dtype="float32")
        config, tensors = plain.read_model(folder)
        out[name] = (folder, config, tensors, page)
    return out


def random_ids(seed, count, vocab):
    return np.random.default_rng(seed).integers(0, vocab, size=count).tolist()
