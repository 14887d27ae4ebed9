"""The plain implementation itself: against outputs of the reference's own CPU code
(tests/golden/reference_outputs.json, made by tests/golden/make_golden.py), and its parts
against hand-checkable cases."""

import json
import os

import numpy as np
import torch

from golden import common
from plain import qwen3_plain as plain

HERE = os.path.dirname(os.path.abspath(__file__))


def golden():
    with open(os.path.join(HERE, "golden", "reference_outputs.json")) as handle:
        return json.load(handle)


def plain_cfg():
    c = common.CONFIG
    return {"H": c["hidden_size"], "I": c["intermediate_size"], "V": c["vocab_size"], "L": c["num_hidden_layers"],
            "Nq": c["num_attention_heads"], "Nkv": c["num_key_value_heads"], "D": c["head_dim"],
            "eps": c["rms_norm_eps"], "theta": c["rope_theta"], "tied": True,
            "windows": [None] * c["num_hidden_layers"]}


def teacher_forced(dtype, tokens):
    """Plain logits at the places that chose each generated token: [B, STEPS, V]."""
    weights, cfg, prompts = common.weights(), plain_cfg(), common.prompts()
    out = []
    for b in range(common.BATCH):
        generated = [step[b] for step in tokens]
        full = prompts[b].tolist() + generated[:-1]
        logits = plain.logits(weights, cfg, full, dtype)
        out.append(logits[common.PROMPT - 1:].numpy())
    return np.stack(out)


def test_float32_matches_the_reference():
    ref = golden()["float32"]
    got = teacher_forced(torch.float32, ref["tokens"])
    want = np.array(ref["logits"], dtype=np.float32)
    assert got.shape == want.shape
    assert np.abs(got - want).max() <= 2e-5
    assert got.argmax(-1).T.tolist() == ref["tokens"]


def test_bfloat16_matches_the_reference():
    """Same rounding points as the reference's bfloat16 code; what remains is the order of
    float32 sums inside products and the reference's rounding of its logits to bfloat16."""
    ref = golden()["bfloat16"]
    got = teacher_forced(torch.bfloat16, ref["tokens"])
    want = np.array(ref["logits"], dtype=np.float32)
    exact = teacher_forced(torch.float32, ref["tokens"])
    noise = np.abs(got - exact).max()
    assert np.abs(got - want).max() <= noise + 2.0 ** -8 * np.abs(want).max()
    chosen = np.take_along_axis(got, np.array(ref["tokens"]).T[:, :, None], axis=-1)[..., 0]
    assert (got.max(-1) - chosen).max() <= 2 * noise, "the reference's tokens are (near-)argmax of the plain logits"


def test_rms_norm_rounds_before_the_gain():
    x = torch.tensor([[1.0, 2.0, 3.0, 4.0]])
    w = torch.tensor([1.5, 1.0, 1.0, 1.0])
    rstd = 1 / np.sqrt(7.5 + 1e-6)
    assert torch.allclose(plain.rms_norm(x, w, 1e-6, torch.float32), torch.tensor([[1.5, 2.0, 3.0, 4.0]]) * rstd)
    got = plain.rms_norm(x.bfloat16(), w.bfloat16(), 1e-6, torch.bfloat16)
    normed = (x * rstd).bfloat16()
    assert torch.equal(got, (w * normed.float()).bfloat16())


def test_rope_rotates_halves():
    d = 8
    cos, sin = plain.rope_cos_sin(torch.tensor([0, 3]), d, 10000.0, torch.float32)
    x = torch.arange(1.0, 2 * d + 1).reshape(2, 1, d)
    out = plain.apply_rope(x, cos, sin, torch.float32)
    assert torch.equal(out[0], x[0])                       # position 0: no rotation
    i = 1
    angle = 3 * 10000.0 ** (-2 * i / d)
    a, b = x[1, 0, i], x[1, 0, i + d // 2]
    assert abs(out[1, 0, i] - (a * np.cos(angle) - b * np.sin(angle))) < 1e-5
    assert abs(out[1, 0, i + d // 2] - (b * np.cos(angle) + a * np.sin(angle))) < 1e-5


def test_attention_is_causal_grouped_and_windowed():
    torch.manual_seed(0)
    S, Nq, Nkv, D = 6, 4, 2, 8
    q, k, v = torch.randn(S, Nq, D), torch.randn(S, Nkv, D), torch.randn(S, Nkv, D)
    out = plain.attention(q, k, v, D ** -0.5, None, torch.float32).reshape(S, Nq, D)
    assert torch.allclose(out[0], v[0].repeat_interleave(2, dim=0))      # first row sees one key
    row, head = 4, 3
    scores = (k[:row + 1, head // 2] @ q[row, head]) * D ** -0.5
    want = torch.softmax(scores, 0) @ v[:row + 1, head // 2]
    assert torch.allclose(out[row, head], want, atol=1e-6)
    windowed = plain.attention(q, k, v, D ** -0.5, 2, torch.float32).reshape(S, Nq, D)
    scores = (k[row - 1:row + 1, head // 2] @ q[row, head]) * D ** -0.5   # keys row-1 and row only
    want = torch.softmax(scores, 0) @ v[row - 1:row + 1, head // 2]
    assert torch.allclose(windowed[row, head], want, atol=1e-6)


def test_philox_known_answers():
    """Vectors of the Random123 distribution for philox4x32-10."""
    cases = [((0, 0, 0, 0), (0, 0), (0x6627e8d5, 0xe169c58d, 0xbc57ac4c, 0x9b00dbd8)),
             ((0xffffffff,) * 4, (0xffffffff, 0xffffffff), (0x408f276d, 0x41c83b0e, 0xa20bc7c6, 0x6d5451fd)),
             ((0x243f6a88, 0x85a308d3, 0x13198a2e, 0x03707344), (0xa4093822, 0x299f31d0),
              (0xd16cfe09, 0x94fdcceb, 0x5001e420, 0x24126ea1))]
    for counter, key, want in cases:
        got = plain.philox4x32([[c] for c in counter], key)
        assert tuple(int(x[0]) for x in got) == want


def test_sampling():
    row = np.array([0.0, 3.0, 3.0, -1.0], dtype=np.float32)
    assert plain.greedy(row) == 1                                       # lowest index on ties
    assert plain.sample(row, 0.0, 5, 0, 0) == 1
    draws = [plain.sample(row, 1.0, 7, 0, step) for step in range(2000)]
    freq = np.bincount(draws, minlength=4) / 2000
    want = np.exp(row) / np.exp(row).sum()
    assert np.abs(freq - want).max() < 0.04
    assert draws == [plain.sample(row, 1.0, 7, 0, step) for step in range(2000)]       # reproducible
    assert draws != [plain.sample(row, 1.0, 7, 1, step) for step in range(2000)]       # stream matters
    noise = plain.gumbel_noise(1000, 3, 2, 1)
    assert np.isfinite(noise).all() and noise.dtype == np.float32
