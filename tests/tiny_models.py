"""The two tiny Llama configurations the tests run on, and helpers to make model folders.

They differ in every size and option: layers, width, heads and grouping, head size, feed-forward
width (176 is no multiple of 64), vocabulary, rope theta and scaling, eps, tied or untied head,
positions, gain initialisation.
"""
from __future__ import annotations

import random

import torch

TINY_A = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "num_hidden_layers": 2, "hidden_size": 64, "num_attention_heads": 4, "num_key_value_heads": 2,
    "head_dim": 16, "intermediate_size": 176, "vocab_size": 256,
    "rope_theta": 10000.0, "rope_scaling": None, "rms_norm_eps": 1e-5,
    "tie_word_embeddings": True, "max_position_embeddings": 128, "hidden_act": "silu",
    "eos_token_id": 2, "bos_token_id": 1,
}
TINY_A_PROMPTS = (5, 11, 17)
TINY_A_DECODE = 8

TINY_B = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "num_hidden_layers": 3, "hidden_size": 192, "num_attention_heads": 6, "num_key_value_heads": 6,
    "head_dim": 32, "intermediate_size": 512, "vocab_size": 384,
    "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0,
                     "high_freq_factor": 4.0, "original_max_position_embeddings": 64},
    "rms_norm_eps": 1e-6, "tie_word_embeddings": False, "max_position_embeddings": 256,
    "hidden_act": "silu", "eos_token_id": [7, 9],
}
TINY_B_PROMPTS = (1, 9, 33, 70)
TINY_B_DECODE = 12

# A third shape for kernels that want head_dim 64 and a 4:1 grouping.
TINY_C = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "num_hidden_layers": 2, "hidden_size": 320, "num_attention_heads": 8, "num_key_value_heads": 2,
    "head_dim": 64, "intermediate_size": 720, "vocab_size": 1000,
    "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0,
                     "high_freq_factor": 4.0, "original_max_position_embeddings": 128},
    "rms_norm_eps": 1e-5, "tie_word_embeddings": False, "max_position_embeddings": 1024,
    "hidden_act": "silu",
}

# A fourth with the benchmark model's head size (128) and grouping (4:1): the head size that the
# tcgen05 prefill kernel and the decode kernel's own rotation are written for.
TINY_D = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "num_hidden_layers": 2, "hidden_size": 512, "num_attention_heads": 4, "num_key_value_heads": 1,
    "head_dim": 128, "intermediate_size": 1376, "vocab_size": 512,
    "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0,
                     "high_freq_factor": 4.0, "original_max_position_embeddings": 128},
    "rms_norm_eps": 1e-5, "tie_word_embeddings": False, "max_position_embeddings": 1024,
    "hidden_act": "silu",
}

CONFIGS = {"A": TINY_A, "B": TINY_B, "C": TINY_C, "D": TINY_D}
GAIN_INIT = {"A": ("one_plus_uniform", 0.1), "B": ("ones",), "C": ("one_plus_uniform", 0.1), "D": ("one_plus_uniform", 0.1)}


def make_folder(tmp_path, which, seed=0, dtype=torch.float32):
    """Write the tiny model's folder with the package's random-weights mode."""
    from dotllm_b200.config import config_from_dict
    from dotllm_b200.models.llama import build_llama_spec
    from dotllm_b200.weights import write_random_model
    cfg = config_from_dict(CONFIGS[which])
    folder = tmp_path / f"tiny_{which}_{seed}_{str(dtype).split('.')[-1]}"
    write_random_model(folder, cfg, seed, dtype=dtype,
                       spec_builder=lambda c: build_llama_spec(c, GAIN_INIT[which]))
    return folder


def random_tokens(n, vocab, seed):
    rng = random.Random(seed)
    return [rng.randrange(vocab) for _ in range(n)]
