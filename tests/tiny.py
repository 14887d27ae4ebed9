"""The tests' own small configurations.  They differ in every size and option: head counts
and groups, head size, sizes that are no power of two, number of layers, vocabulary, the
norms' eps, rope theta, tied or untied head, stored precision, and the window."""

import json
import os

import torch

CONFIGS = {
    # 2 layers, head_dim * heads == hidden, tied, float32 weights, all keys
    "a": dict(vocab_size=256, hidden_size=64, intermediate_size=128, num_hidden_layers=2,
              num_attention_heads=4, num_key_value_heads=2, head_dim=16, rms_norm_eps=1e-6, rope_theta=10000.0,
              tie_word_embeddings=True, max_position_embeddings=4096, seed=0, stored="float32"),
    # 3 layers, one kv head for 8 query heads, q projection wider than hidden, untied
    "b": dict(vocab_size=512, hidden_size=96, intermediate_size=160, num_hidden_layers=3,
              num_attention_heads=8, num_key_value_heads=1, head_dim=32, rms_norm_eps=1e-5, rope_theta=1000000.0,
              tie_word_embeddings=False, max_position_embeddings=4096, seed=1, stored="float32"),
    # 4 layers, nothing a power of two, head size 48, a window of 24 keys on layers 1 and 3,
    # weights stored in bfloat16
    "c": dict(vocab_size=300, hidden_size=80, intermediate_size=112, num_hidden_layers=4,
              num_attention_heads=6, num_key_value_heads=3, head_dim=48, rms_norm_eps=3e-6, rope_theta=500000.0,
              tie_word_embeddings=False, max_position_embeddings=2048, sliding_window=24, use_sliding_window=True,
              layer_types=["full_attention", "sliding_attention", "full_attention", "sliding_attention"],
              seed=2, stored="bfloat16"),
    # 2 layers, head size 64 (tensor-core attention kernels), groups of 2, window 70 (crosses a page) on layer 0
    "d": dict(vocab_size=1000, hidden_size=128, intermediate_size=192, num_hidden_layers=2,
              num_attention_heads=4, num_key_value_heads=2, head_dim=64, rms_norm_eps=1e-6, rope_theta=5000000.0,
              tie_word_embeddings=True, max_position_embeddings=8192, sliding_window=70, use_sliding_window=True,
              layer_types=["sliding_attention", "full_attention"], seed=3, stored="bfloat16"),
}


def config_json(name):
    data = {k: v for k, v in CONFIGS[name].items() if k not in ("seed", "stored")}
    data["architectures"] = ["Qwen3ForCausalLM"]
    data["model_type"] = "qwen3"
    data["hidden_act"] = "silu"
    data["attention_bias"] = False
    data["rope_scaling"] = None
    data["torch_dtype"] = CONFIGS[name]["stored"]
    return data


def write_model(folder, name, gain_std=0.1):
    """Writes the folder with the library's random-weights mode."""
    from thing_htn_2026_b200.config import config_from_dict
    from thing_htn_2026_b200.weights import write_random_model
    config = config_from_dict(config_json(name))
    dtype = {"float32": torch.float32, "bfloat16": torch.bfloat16}[CONFIGS[name]["stored"]]
    write_random_model(folder, config, CONFIGS[name]["seed"], dtype=dtype, gain_std=gain_std)
    # keep exactly the keys of config_json (the library's writer adds defaults)
    with open(os.path.join(folder, "config.json"), "w") as handle:
        json.dump(config_json(name), handle, indent=1)
    return folder


def tokens(name, length, seed):
    g = torch.Generator().manual_seed(1000 + seed)
    return torch.randint(0, CONFIGS[name]["vocab_size"], (length,), generator=g).tolist()


def tokens_for_dir(model_dir, length):
    """Tokens for the configuration whose folder this is (folders are named by configuration)."""
    return tokens(os.path.basename(os.path.normpath(model_dir)), length, 999)
