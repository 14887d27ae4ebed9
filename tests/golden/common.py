"""The tiny model and inputs that the golden outputs were made with.  Everything comes from
seeded CPU generators, so the test can rebuild exactly what the script fed to the
reference."""

import torch

CONFIG = dict(vocab_size=256, hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
              num_key_value_heads=2, head_dim=16, rms_norm_eps=1e-6, rope_theta=10000.0, tie_word_embeddings=True)
BATCH, PROMPT, STEPS = 3, 9, 8


def weights(seed=0):
    """name -> float32 tensor; matrices N(0, 0.02), norm gains 1 + N(0, 0.1); all values are
    rounded to bfloat16 so that the float32 and bfloat16 runs use the same numbers."""
    g = torch.Generator().manual_seed(seed)
    c = CONFIG
    H, I, V, D = c["hidden_size"], c["intermediate_size"], c["vocab_size"], c["head_dim"]
    Nq, Nkv = c["num_attention_heads"], c["num_key_value_heads"]

    def matrix(*shape):
        return (torch.randn(shape, generator=g) * 0.02).to(torch.bfloat16).float()

    def gain(n):
        return (1 + 0.1 * torch.randn(n, generator=g)).to(torch.bfloat16).float()

    out = {"model.embed_tokens.weight": matrix(V, H)}
    for i in range(c["num_hidden_layers"]):
        p = f"model.layers.{i}."
        out[p + "input_layernorm.weight"] = gain(H)
        out[p + "self_attn.q_proj.weight"] = matrix(Nq * D, H)
        out[p + "self_attn.k_proj.weight"] = matrix(Nkv * D, H)
        out[p + "self_attn.v_proj.weight"] = matrix(Nkv * D, H)
        out[p + "self_attn.o_proj.weight"] = matrix(H, Nq * D)
        out[p + "self_attn.q_norm.weight"] = gain(D)
        out[p + "self_attn.k_norm.weight"] = gain(D)
        out[p + "post_attention_layernorm.weight"] = gain(H)
        out[p + "mlp.gate_proj.weight"] = matrix(I, H)
        out[p + "mlp.up_proj.weight"] = matrix(I, H)
        out[p + "mlp.down_proj.weight"] = matrix(H, I)
    out["model.norm.weight"] = gain(H)
    return out


def prompts(seed=1):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, CONFIG["vocab_size"], (BATCH, PROMPT), generator=g)
