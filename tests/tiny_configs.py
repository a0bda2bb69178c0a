"""The tiny configurations the tests run: Llama shapes that differ in every size and option (A and B
are the two named by the baseline; C and D have the head sizes 64 and 128 of the 1B and the 3B / 8B
shapes, for which the tensor-core attention kernels are built)."""
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

TINY_A = {   # grouped heads 4:2, tied head, plain RoPE, float32 weights
    "architectures": ["LlamaForCausalLM"], "model_type": "llama", "hidden_act": "silu",
    "hidden_size": 64, "intermediate_size": 128, "num_hidden_layers": 2, "num_attention_heads": 4,
    "num_key_value_heads": 2, "head_dim": 16, "vocab_size": 256, "max_position_embeddings": 128,
    "rope_theta": 10000.0, "rope_scaling": None, "rms_norm_eps": 1e-5, "tie_word_embeddings": True,
}

TINY_B = {   # one key/value head for 3 query heads, untied head, llama3-scaled RoPE, sizes that are no power of two
    "architectures": ["LlamaForCausalLM"], "model_type": "llama", "hidden_act": "silu",
    "hidden_size": 96, "intermediate_size": 160, "num_hidden_layers": 3, "num_attention_heads": 3,
    "num_key_value_heads": 1, "head_dim": 32, "vocab_size": 384, "max_position_embeddings": 256,
    "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 64},
    "rms_norm_eps": 1e-6, "tie_word_embeddings": False,
}

# How each tiny model's weights are drawn (weights.write_random_model arguments).
WEIGHTS_A = {"seed": 11, "dtype": "float32", "std": 0.02, "norm_mean": 1.0, "norm_std": 0.01}
WEIGHTS_B = {"seed": 23, "dtype": "bfloat16", "std": 0.02, "norm_mean": 1.0, "norm_std": 0.02}
# Larger weights give peaked attention and distinct logits, so a wrong key, a wrong position or a
# stale page changes the result visibly (with N(0, 0.02) every softmax is nearly uniform).
SHARP_A = dict(WEIGHTS_A, seed=12, std=0.2, norm_std=0.1)
SHARP_B = dict(WEIGHTS_B, seed=24, std=0.2, norm_std=0.1)


def make_model_dir(config, weights, out_dir):
    from geneinfer_b200.weights import write_random_model
    return write_random_model(config, weights["seed"], out_dir, weights["dtype"], std=weights["std"],
                              norm_mean=weights["norm_mean"], norm_std=weights["norm_std"])


def random_tokens(n, vocab, seed):
    import numpy as np
    return [int(t) for t in np.random.default_rng(seed).integers(0, vocab, size=n)]

TINY_C = {   # head size 64 (the tcgen05 prefill attention and the fused gate/up product are built for it), 6:2 heads
    "architectures": ["LlamaForCausalLM"], "model_type": "llama", "hidden_act": "silu",
    "hidden_size": 192, "intermediate_size": 264, "num_hidden_layers": 2, "num_attention_heads": 6,
    "num_key_value_heads": 2, "head_dim": 64, "vocab_size": 500, "max_position_embeddings": 512,
    "rope_theta": 100000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 128},
    "rms_norm_eps": 1e-5, "tie_word_embeddings": True,
}
SHARP_C = {"seed": 31, "dtype": "bfloat16", "std": 0.12, "norm_mean": 1.0, "norm_std": 0.1}

TINY_D = {   # head size 128 as in the 3B and 8B shapes, 4:2 heads, untied head, three layers
    "architectures": ["LlamaForCausalLM"], "model_type": "llama", "hidden_act": "silu",
    "hidden_size": 256, "intermediate_size": 328, "num_hidden_layers": 3, "num_attention_heads": 4,
    "num_key_value_heads": 2, "head_dim": 128, "vocab_size": 333, "max_position_embeddings": 384,
    "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 96},
    "rms_norm_eps": 2e-6, "tie_word_embeddings": False,
}
SHARP_D = {"seed": 41, "dtype": "bfloat16", "std": 0.1, "norm_mean": 1.0, "norm_std": 0.1}

WIDE_W = {   # the Llama-3.2-1B widths, heads, vocabulary and RoPE scaling with two of its sixteen layers
    "architectures": ["LlamaForCausalLM"], "model_type": "llama", "hidden_act": "silu",
    "hidden_size": 2048, "intermediate_size": 8192, "num_hidden_layers": 2, "num_attention_heads": 32,
    "num_key_value_heads": 8, "head_dim": 64, "vocab_size": 128256, "max_position_embeddings": 8192,
    "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 8192},
    "rms_norm_eps": 1e-5, "tie_word_embeddings": True,
}
SHARP_W = {"seed": 51, "dtype": "bfloat16", "std": 0.05, "norm_mean": 1.0, "norm_std": 0.1}

WIDE_W3 = dict(WIDE_W, hidden_size=3072, num_attention_heads=24, head_dim=128, num_hidden_layers=1)   # the Llama-3.2-3B widths, one layer
SHARP_W3 = {"seed": 52, "dtype": "bfloat16", "std": 0.04, "norm_mean": 1.0, "norm_std": 0.1}
