"""Plain, slow Qwen3 dense forward: whole sequences, no cache, one function per part.

This file is the oracle of the tests.  It is written from the reference's formulas
(each function cites file:line under the reference project) and shares no code with
the library: it parses config.json itself, reads safetensors itself, and runs one
sequence at a time on the CPU with torch tensor arithmetic only.

``dtype`` is the activation dtype.  With ``torch.float32`` every rounding below is the
identity.  With ``torch.bfloat16`` values are rounded where the reference rounds them
(engine/kernels/torch_ref.py:16-29); all arithmetic in between is float32.

Differences from the reference, on purpose:
* logits are returned in float32 without a final rounding (the reference's LM head
  stores bfloat16, engine/engine.py:1120, and never returns logits);
* a sliding window (the reference has none, OPTIMIZATION_GUIDE.md:36): query at
  position p sees keys j with p - window < j <= p.

It rests on the reference's formulas; tests/golden/ holds outputs of the reference's
own CPU code (its torch twins and its step functions) that this file is compared with.
"""

from __future__ import annotations

import json
import math
import os
import struct

import numpy as np
import torch

# --------------------------------------------------------------------------- files


def read_config(model_dir):
    """The keys the reference reads (engine/engine.py:128-141) plus tie and window keys."""
    with open(os.path.join(model_dir, "config.json")) as handle:
        raw = json.load(handle)
    heads = raw["num_attention_heads"]
    layers = raw["num_hidden_layers"]
    window = raw.get("sliding_window")
    if not raw.get("use_sliding_window", False) and "layer_types" not in raw:
        window = None
    types = raw.get("layer_types")
    if types is None:
        first = raw.get("max_window_layers", layers)
        types = ["sliding_attention" if (window is not None and i >= first) else "full_attention"
                 for i in range(layers)]
    return {
        "H": raw["hidden_size"], "I": raw["intermediate_size"], "V": raw["vocab_size"], "L": layers,
        "Nq": heads, "Nkv": raw.get("num_key_value_heads", heads),
        "D": raw.get("head_dim") or raw["hidden_size"] // heads,
        "eps": float(raw["rms_norm_eps"]), "theta": float(raw["rope_theta"]),
        "tied": bool(raw.get("tie_word_embeddings", False)),
        "windows": [window if t == "sliding_attention" else None for t in types],
    }


def read_safetensors(path):
    """8-byte header length, JSON header, raw data.  Returns name -> float32/int tensor."""
    kinds = {"F32": ("<f4", None), "F16": ("<f2", None), "BF16": ("<u2", "bf16"), "F64": ("<f8", None),
             "I64": ("<i8", None), "I32": ("<i4", None)}
    with open(path, "rb") as handle:
        blob = handle.read()
    (n,) = struct.unpack("<Q", blob[:8])
    header = json.loads(blob[8:8 + n])
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        np_kind, special = kinds[info["dtype"]]
        b, e = info["data_offsets"]
        arr = np.frombuffer(blob, dtype=np_kind, count=(e - b) // np.dtype(np_kind).itemsize, offset=8 + n + b)
        if special == "bf16":
            arr = (arr.astype(np.uint32) << 16).view(np.float32)
        t = torch.from_numpy(np.array(arr)).reshape(info["shape"])
        out[name] = t.float() if t.is_floating_point() else t
    return out


# --------------------------------------------------------------------------- parts


def rms_norm(x, w, eps, dtype):
    """y = w * round(x * rsqrt(mean(x^2) + eps)); the normalised value is rounded BEFORE
    the gain, the product once more.  engine/kernels/torch_ref.py:47-58."""
    xf = x.float()
    variance = xf.pow(2).mean(-1, keepdim=True)
    normed = (xf * torch.rsqrt(variance + eps)).to(dtype)
    return (w.float() * normed.float()).to(dtype)


def add_residual(h, d, dtype):
    """h = round(h + d), the sum in float32.  engine/kernels/torch_ref.py:61-68."""
    return (h.float() + d.float()).to(dtype)


def linear(x, w, dtype):
    """x @ w^T, w is [out, in]; float32 accumulation, one rounding of the result.
    engine/engine.py:341-350 (F.linear), OPTIMIZATION_GUIDE.md:117."""
    return (x.float() @ w.float().t()).to(dtype)


def rope_cos_sin(positions, head_dim, theta, dtype):
    """inv_freq[i] = 1 / theta^(2i/D); angle = position * inv_freq in float32;
    tables are cat(angle, angle), rounded to the activation dtype.
    engine/engine.py:238-247."""
    inv_freq = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.int64).float() / head_dim))
    angle = positions.float()[:, None] * inv_freq[None, :]
    emb = torch.cat((angle, angle), dim=-1)
    return emb.cos().to(dtype), emb.sin().to(dtype)


def apply_rope(x, cos, sin, dtype):
    """out = round(round(x*cos) + round(rotate_half(x)*sin)), rotate_half(x) =
    cat(-x[D/2:], x[:D/2]).  x [S, heads, D]; cos, sin [S, D].
    engine/kernels/torch_ref.py:94-104."""
    xf = x.float()
    half = xf.shape[-1] // 2
    rotated = torch.cat((-xf[..., half:], xf[..., :half]), dim=-1)
    p1 = (xf * cos.float()[:, None, :]).to(dtype)
    p2 = (rotated * sin.float()[:, None, :]).to(dtype)
    return (p1.float() + p2.float()).to(dtype)


def attention(q, k, v, scale, window, dtype):
    """Causal grouped-query attention of one whole sequence.

    q [S, Nq, D], k and v [S, Nkv, D]; query head h reads kv head h // (Nq // Nkv).
    scores = (q . k) * scale in float32; e = exp(s - rowmax); the un-normalised e is
    rounded to the activation dtype before the value product, the float32 row sum
    divides at the end, the result is rounded once.
    engine/kernels/torch_ref.py:168-227 (mask :207-208, softmax :222-225,
    head mapping :199-200)."""
    S, Nq, D = q.shape
    Nkv = k.shape[1]
    G = Nq // Nkv
    qf = q.float().permute(1, 0, 2)                                   # [Nq, S, D]
    kf = k.float().permute(1, 0, 2).repeat_interleave(G, dim=0)       # [Nq, S, D]
    vf = v.float().permute(1, 0, 2).repeat_interleave(G, dim=0)
    scores = torch.matmul(qf, kf.transpose(-1, -2)) * scale           # [Nq, S, S]
    i = torch.arange(S)[:, None]
    j = torch.arange(S)[None, :]
    visible = j <= i
    if window is not None:
        visible = visible & (j > i - window)
    scores = scores.masked_fill(~visible[None], float("-inf"))
    mx = scores.amax(dim=-1, keepdim=True)
    e = torch.exp(scores - mx)
    l = e.sum(dim=-1, keepdim=True)
    out = torch.matmul(e.to(dtype).float(), vf) / l                   # [Nq, S, D]
    return out.permute(1, 0, 2).to(dtype).reshape(S, Nq * D)


def swiglu(gate, up, dtype):
    """round(round(g / (1 + exp(-g))) * u).  engine/kernels/torch_ref.py:74-88."""
    g = gate.float()
    s = (g / (1.0 + torch.exp(-g))).to(dtype)
    return (s.float() * up.float()).to(dtype)


def attention_block(n, w, cfg, layer, positions, dtype):
    """q/k/v projections, per-head RMSNorm of q and k, RoPE, attention, output projection.
    engine/engine.py:1108-1114; engine/kernels/torch_ref.py:141-152."""
    p = f"model.layers.{layer}.self_attn."
    S = n.shape[0]
    Nq, Nkv, D = cfg["Nq"], cfg["Nkv"], cfg["D"]
    q = linear(n, w[p + "q_proj.weight"], dtype).reshape(S, Nq, D)
    k = linear(n, w[p + "k_proj.weight"], dtype).reshape(S, Nkv, D)
    v = linear(n, w[p + "v_proj.weight"], dtype).reshape(S, Nkv, D)
    q = rms_norm(q, w[p + "q_norm.weight"], cfg["eps"], dtype)
    k = rms_norm(k, w[p + "k_norm.weight"], cfg["eps"], dtype)
    cos, sin = rope_cos_sin(positions, D, cfg["theta"], dtype)
    q = apply_rope(q, cos, sin, dtype)
    k = apply_rope(k, cos, sin, dtype)
    a = attention(q, k, v, D ** -0.5, cfg["windows"][layer], dtype)
    return linear(a, w[p + "o_proj.weight"], dtype)


def mlp_block(n, w, layer, dtype):
    """down(silu(gate(n)) * up(n)).  engine/engine.py:1116-1118."""
    p = f"model.layers.{layer}.mlp."
    g = linear(n, w[p + "gate_proj.weight"], dtype)
    u = linear(n, w[p + "up_proj.weight"], dtype)
    return linear(swiglu(g, u, dtype), w[p + "down_proj.weight"], dtype)


def held(weights, dtype):
    """Precision in which weights are held: matrices in the activation dtype; vectors
    (norm gains) keep the stored values (a gain stored in 32 bits stays in 32 bits)."""
    return {k: (v.to(dtype) if v.is_floating_point() and v.dim() >= 2 else v) for k, v in weights.items()}


def hidden_states(weights, cfg, tokens, dtype):
    """Embedding and all decoder layers; returns the residual stream after the last
    layer, [S, H].  Pre-norm block with the residual outside each branch:
    a = x + attn(norm1(x)); y = a + mlp(norm2(a)).
    engine/engine.py:1101-1118; OPTIMIZATION_GUIDE.md:57-70."""
    w = held(weights, dtype)
    ids = torch.as_tensor(tokens, dtype=torch.int64)
    positions = torch.arange(ids.shape[0])
    h = w["model.embed_tokens.weight"][ids]
    for layer in range(cfg["L"]):
        p = f"model.layers.{layer}."
        n = rms_norm(h, w[p + "input_layernorm.weight"], cfg["eps"], dtype)
        h = add_residual(h, attention_block(n, w, cfg, layer, positions, dtype), dtype)
        n = rms_norm(h, w[p + "post_attention_layernorm.weight"], cfg["eps"], dtype)
        h = add_residual(h, mlp_block(n, w, layer, dtype), dtype)
    return h


def logits(weights, cfg, tokens, dtype=torch.float32):
    """Final norm and LM head at every position: float32 [S, V].
    engine/engine.py:1119-1120; tied head uses the embedding (:225-226)."""
    h = hidden_states(weights, cfg, tokens, dtype)
    n = rms_norm(h, weights["model.norm.weight"], cfg["eps"], dtype)
    head = weights["model.embed_tokens.weight" if cfg["tied"] else "lm_head.weight"].to(dtype)
    return n.float() @ head.float().t()


def model_logits(model_dir, tokens, dtype=torch.float32):
    cfg = read_config(model_dir)
    weights = read_safetensors(os.path.join(model_dir, "model.safetensors"))
    return logits(weights, cfg, tokens, dtype)


# --------------------------------------------------------------------------- token choice


def greedy(row):
    """argmax, lowest index on exact ties.  engine/engine.py:1121; OPTIMIZATION_GUIDE.md:213."""
    row = np.asarray(row, dtype=np.float32)
    return int(np.flatnonzero(row == row.max())[0])


_PHILOX_M0, _PHILOX_M1 = 0xD2511F53, 0xCD9E8D57
_PHILOX_W0, _PHILOX_W1 = 0x9E3779B9, 0xBB67AE85


def philox4x32(counter, key):
    """Philox-4x32 with 10 rounds (Salmon et al., 2011).  counter: four uint64 arrays
    holding 32-bit words; key: two ints.  Returns four uint64 arrays of 32-bit words."""
    c0, c1, c2, c3 = [np.asarray(c, dtype=np.uint64) for c in counter]
    k0, k1 = key[0] & 0xFFFFFFFF, key[1] & 0xFFFFFFFF
    mask = np.uint64(0xFFFFFFFF)
    for _ in range(10):
        p0 = np.uint64(_PHILOX_M0) * c0
        p1 = np.uint64(_PHILOX_M1) * c2
        hi0, lo0 = p0 >> np.uint64(32), p0 & mask
        hi1, lo1 = p1 >> np.uint64(32), p1 & mask
        c0, c1, c2, c3 = (hi1 ^ c1 ^ np.uint64(k0)), lo1, (hi0 ^ c3 ^ np.uint64(k1)), lo0
        k0 = (k0 + _PHILOX_W0) & 0xFFFFFFFF
        k1 = (k1 + _PHILOX_W1) & 0xFFFFFFFF
    return c0, c1, c2, c3


def gumbel_noise(vocab, seed, stream, step):
    """One float32 Gumbel variate per vocabulary entry.  Entry i uses word i % 4 of
    Philox(counter = (i // 4, step, stream, 0), key = (seed low, seed high));
    u = ((word >> 9) + 0.5) * 2^-23; noise = -log(-log(u))."""
    blocks = np.arange((vocab + 3) // 4, dtype=np.uint64)
    zeros = np.zeros_like(blocks)
    words = philox4x32((blocks, zeros + np.uint64(step & 0xFFFFFFFF), zeros + np.uint64(stream & 0xFFFFFFFF), zeros),
                       (seed & 0xFFFFFFFF, (seed >> 32) & 0xFFFFFFFF))
    x = np.stack(words, axis=1).reshape(-1)[:vocab]
    u = ((x >> np.uint64(9)).astype(np.float32) + np.float32(0.5)) * np.float32(2.0 ** -23)
    return -np.log(-np.log(u, dtype=np.float32), dtype=np.float32)


def sample(row, temperature, seed, stream, step):
    """Temperature sampling by the Gumbel-max rule: argmax(logits / T + noise) is a draw
    from softmax(logits / T).  temperature 0 is greedy."""
    if temperature == 0:
        return greedy(row)
    row = np.asarray(row, dtype=np.float32)
    scored = row / np.float32(temperature) + gumbel_noise(row.shape[0], seed, stream, step)
    return int(np.flatnonzero(scored == scored.max())[0])
