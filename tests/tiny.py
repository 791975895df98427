"""The tiny configurations of the test suite: they differ in every size and option."""
import json
import tempfile
from pathlib import Path

import torch

# A: tied head, head_dim 16, group 2, H * hd == D, theta 1e4, eps 1e-6, no window
TINY_A = dict(model_type="qwen3", architectures=["Qwen3ForCausalLM"], hidden_size=64, num_hidden_layers=2,
              num_attention_heads=4, num_key_value_heads=2, head_dim=16, intermediate_size=128, vocab_size=256,
              rope_theta=10000.0, rms_norm_eps=1e-6, tie_word_embeddings=True, attention_bias=False,
              use_sliding_window=False, max_position_embeddings=128, hidden_act="silu")
# B: untied head, head_dim 32, group 4, H * hd = 256 != D = 96, F = 200, V = 1000, theta 1e6, eps 1e-5
TINY_B = dict(model_type="qwen3", architectures=["Qwen3ForCausalLM"], hidden_size=96, num_hidden_layers=3,
              num_attention_heads=8, num_key_value_heads=2, head_dim=32, intermediate_size=200, vocab_size=1000,
              rope_theta=1000000.0, rms_norm_eps=1e-5, tie_word_embeddings=False, attention_bias=False,
              use_sliding_window=False, max_position_embeddings=512, hidden_act="silu")
# C: a window from layer 1 on, biases, head_dim 48 (no power of two), group 3, partial rotary, linear rope scaling
TINY_C = dict(model_type="qwen3", architectures=["Qwen3ForCausalLM"], hidden_size=72, num_hidden_layers=4,
              num_attention_heads=6, num_key_value_heads=2, head_dim=48, intermediate_size=176, vocab_size=517,
              rope_theta=50000.0, rms_norm_eps=3e-6, tie_word_embeddings=False, attention_bias=True,
              use_sliding_window=True, sliding_window=40, max_window_layers=1, max_position_embeddings=1024,
              partial_rotary_factor=0.5, rope_scaling={"rope_type": "linear", "factor": 2.0}, hidden_act="silu")

# D: head_dim 64 (the size the tensor-core prefill attention takes), a window on every layer but the first two
TINY_D = dict(model_type="qwen3", architectures=["Qwen3ForCausalLM"], hidden_size=136, num_hidden_layers=3,
              num_attention_heads=6, num_key_value_heads=3, head_dim=64, intermediate_size=264, vocab_size=333,
              rope_theta=20000.0, rms_norm_eps=2e-6, tie_word_embeddings=True, attention_bias=False,
              use_sliding_window=True, sliding_window=70, max_window_layers=2, max_position_embeddings=2048,
              hidden_act="silu")

# E: head_dim 128 (the size of the tcgen05 attention kernels and of the staged decode kernel), group 2, a window on
# the last layer only, widths that are no powers of two
TINY_E = dict(model_type="qwen3", architectures=["Qwen3ForCausalLM"], hidden_size=168, num_hidden_layers=3,
              num_attention_heads=4, num_key_value_heads=2, head_dim=128, intermediate_size=312, vocab_size=421,
              rope_theta=500000.0, rms_norm_eps=1e-6, tie_word_embeddings=False, attention_bias=False,
              use_sliding_window=True, sliding_window=150, max_window_layers=2, max_position_embeddings=4096,
              hidden_act="silu")

CONFIGS = {"A": TINY_A, "B": TINY_B, "C": TINY_C, "D": TINY_D, "E": TINY_E}


def make_model_folder(config: dict, seed: int, where=None, vector_dtype=None) -> Path:
    """A temporary model folder with random weights; never inside the repository."""
    from jllm_serve_b200.weights import write_model_folder
    d = Path(where or tempfile.mkdtemp(prefix="jllm_tiny_"))
    return write_model_folder(config, seed, d, torch.bfloat16, vector_dtype)


def random_tokens(n: int, vocab: int, seed: int) -> list:
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


def random_config(seed: int) -> dict:
    """A configuration drawn from everything the architecture's keys allow at tiny sizes: head sizes in steps of 16 up
    to 256, any number of heads and groups (also odd ones), widths and vocabularies that are no powers of two, with and
    without window, biases, tied head, linear or yarn scaling, partial rotary."""
    import random
    rng = random.Random(seed)
    kv_heads = rng.choice([1, 2, 3, 4, 5])
    layers = rng.randint(1, 4)
    cfg = dict(model_type="qwen3", architectures=["Qwen3ForCausalLM"], hidden_size=8 * rng.randint(4, 40),
               num_hidden_layers=layers, num_attention_heads=kv_heads * rng.choice([1, 2, 3, 4, 5, 7, 8]),
               num_key_value_heads=kv_heads, head_dim=rng.choice([16, 32, 48, 64, 80, 96, 112, 128, 128, 160, 256]),
               intermediate_size=8 * rng.randint(5, 60), vocab_size=rng.randint(50, 1500),
               rope_theta=float(rng.choice([1e4, 5e4, 1e6])), rms_norm_eps=rng.choice([1e-6, 1e-5, 3e-6]),
               tie_word_embeddings=rng.random() < 0.5, attention_bias=rng.random() < 0.4, use_sliding_window=False,
               max_position_embeddings=1024, hidden_act="silu")
    if rng.random() < 0.5:
        cfg.update(use_sliding_window=True, sliding_window=rng.randint(5, 200), max_window_layers=rng.randint(0, layers))
    scaling = rng.random()
    if scaling < 0.2:
        cfg["rope_scaling"] = {"rope_type": "linear", "factor": rng.choice([2.0, 4.0])}
    elif scaling < 0.4:
        cfg["rope_scaling"] = {"rope_type": "yarn", "factor": rng.choice([2.0, 4.0]),
                               "original_max_position_embeddings": 256}
    if rng.random() < 0.25:
        cfg["partial_rotary_factor"] = rng.choice([0.25, 0.5])
    return cfg
