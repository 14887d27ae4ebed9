"""Two more parts that live only in this test and are registered from it: a feed-forward with
routing (one expert per row, chosen by a float32 router) and another position encoding
(position interpolation over a part of the head, with its own angle tables).  A
configuration puts them into different layers beside the library's attention and SwiGLU;
the model is built from a folder, stepped whole, token by token and in unequal batches on
reused slots, and compared with the same model written out plainly.  No file of the
library changes for it."""

import json
import os

import numpy as np
import pytest
import torch

import harness
from plain import qwen3_plain as plain

pytestmark = pytest.mark.gpu

HEAD_DIM, ROTARY_DIM, N_HEADS, N_KV = 32, 16, 3, 1
FACTOR, BASE = 4.0, 777.0
WINDOW = 16


def define_routed_toy():
    from dataclasses import dataclass

    from thing_htn_2026_b200 import ops
    from thing_htn_2026_b200.config import register_architecture
    from thing_htn_2026_b200.config.base import LayerSpec, ModelConfig, ModelPlan, PartSpec, ScheduleEntry
    from thing_htn_2026_b200.config.registry import _decoder_model, known_architectures
    from thing_htn_2026_b200.parts import register_part
    from thing_htn_2026_b200.weights import MATRIX, TensorSpec

    @register_part("position", "toy_interpolated")
    class InterpolatedRotary:
        """Angles (p / factor) * base^(-2i / rotary_dim) over the first rotary_dim values of a head."""

        @classmethod
        def tensor_specs(cls, spec):
            return []

        def __init__(self, spec, rt):
            self.rotary_dim, self.factor, self.base = spec.params["rotary_dim"], spec.params["factor"], spec.params["base"]
            self.device = rt.device
            self._tables = None

        def ensure(self, n_positions):
            if self._tables is not None and self._tables.cos.shape[0] >= n_positions:
                return
            i = torch.arange(0, self.rotary_dim, 2, dtype=torch.float32, device=self.device)
            inv_freq = self.base ** (-i / self.rotary_dim)
            angle = (torch.arange(n_positions, dtype=torch.float32, device=self.device) / self.factor)[:, None] * inv_freq
            self._tables = ops.RotaryTables(angle.cos().contiguous(), angle.sin().contiguous(), self.rotary_dim)

        def tables(self):
            return self._tables

    @register_part("ffn", "toy_routed")
    class RoutedFFN:
        """Each row goes through the one expert its float32 router score picks (lowest index
        on ties); an expert is down(relu(up(x)))."""

        @classmethod
        def tensor_specs(cls, spec):
            h, e, m = spec.params["hidden_size"], spec.params["n_experts"], spec.params["expert_size"]
            return [TensorSpec(spec.tensors["router"], (e, h), MATRIX), TensorSpec(spec.tensors["up"], (e * m, h), MATRIX),
                    TensorSpec(spec.tensors["down"], (e * h, m), MATRIX)]

        def __init__(self, spec, rt):
            self.h, self.e, self.m = spec.params["hidden_size"], spec.params["n_experts"], spec.params["expert_size"]
            self.router = rt.tensor(spec, "router")
            self.up = rt.tensor(spec, "up").reshape(self.e, self.m, self.h)
            self.down = rt.tensor(spec, "down").reshape(self.e, self.h, self.m)

        def forward(self, x, ctx):
            choice = (x.float() @ self.router.float().t()).argmax(dim=-1)          # a row decides for itself
            mid = torch.relu(torch.einsum("rh,rmh->rm", x.float(), self.up.float()[choice]))
            return torch.einsum("rm,rhm->rh", mid, self.down.float()[choice]).to(x.dtype)

    @dataclass(frozen=True)
    class RoutedToyConfig(ModelConfig):
        vocab_size: int
        hidden_size: int
        n_experts: int
        architecture = "RoutedToyForCausalLM"

        @classmethod
        def from_dict(cls, data):
            return cls(data["vocab_size"], data["hidden_size"], data["n_experts"])

        def to_dict(self):
            return {"architectures": [self.architecture], "vocab_size": self.vocab_size,
                    "hidden_size": self.hidden_size, "n_experts": self.n_experts}

        def plan(self):
            h = self.hidden_size

            def norm(name):
                return PartSpec("rmsnorm", {"size": h, "eps": 1e-5}, {"weight": name})

            def attention(i, position, window):
                return PartSpec("attention", {"hidden_size": h, "n_heads": N_HEADS, "n_kv_heads": N_KV, "head_dim": HEAD_DIM,
                                              "scale": HEAD_DIM ** -0.5, "window": window, "qk_norm_eps": 1e-5,
                                              "position": position},
                                {k: f"l{i}.{k}" for k in ("q_proj", "k_proj", "v_proj", "o_proj", "q_norm", "k_norm")})

            interpolated = PartSpec("toy_interpolated", {"rotary_dim": ROTARY_DIM, "factor": FACTOR, "base": BASE})
            rope = PartSpec("rope", {"head_dim": HEAD_DIM, "theta": 10000.0})
            swiglu = PartSpec("swiglu", {"hidden_size": h, "intermediate_size": 3 * h},
                              {k: f"l0.{k}" for k in ("gate_proj", "up_proj", "down_proj")})
            routed = PartSpec("toy_routed", {"hidden_size": h, "n_experts": self.n_experts, "expert_size": 2 * h},
                              {k: f"l1.{k}" for k in ("router", "up", "down")})
            layers = (LayerSpec.of("pre_norm", mixer=attention(0, interpolated, None), ffn=swiglu, norm_mixer=norm("l0.n1"), norm_ffn=norm("l0.n2")),
                      LayerSpec.of("pre_norm", mixer=attention(1, rope, WINDOW), ffn=routed, norm_mixer=norm("l1.n1"), norm_ffn=norm("l1.n2")))
            return ModelPlan(h, self.vocab_size,
                             PartSpec("embedding", {"vocab_size": self.vocab_size, "hidden_size": h}, {"weight": "emb"}),
                             layers, (ScheduleEntry(0, 0), ScheduleEntry(1, 1)), norm("final"),
                             PartSpec("lm_head", {"vocab_size": self.vocab_size, "hidden_size": h, "tied": False},
                                      {"weight": "head"}), 1024)

    if "RoutedToyForCausalLM" not in known_architectures():
        register_architecture("RoutedToyForCausalLM", RoutedToyConfig, _decoder_model)
    return RoutedToyConfig


def routed_toy_plain_logits(folder, tokens):
    """The same model written out plainly: whole sequence, float32, no cache."""
    w = plain.read_safetensors(os.path.join(folder, "model.safetensors"))
    cfg = json.load(open(os.path.join(folder, "config.json")))
    f32 = torch.float32
    S = len(tokens)
    positions = torch.arange(S)
    h = w["emb"][torch.tensor(tokens)]

    def rotate(x, cos, sin, rotary_dim):
        """rotate-half over the first rotary_dim values of every head; the rest passes."""
        head, rest = x[..., :rotary_dim], x[..., rotary_dim:]
        full_cos, full_sin = torch.cat((cos, cos), dim=-1), torch.cat((sin, sin), dim=-1)
        return torch.cat((plain.apply_rope(head, full_cos, full_sin, f32), rest), dim=-1)

    def attention(n, i, cos, sin, rotary_dim, window):
        q = plain.linear(n, w[f"l{i}.q_proj"], f32).reshape(S, N_HEADS, HEAD_DIM)
        k = plain.linear(n, w[f"l{i}.k_proj"], f32).reshape(S, N_KV, HEAD_DIM)
        v = plain.linear(n, w[f"l{i}.v_proj"], f32).reshape(S, N_KV, HEAD_DIM)
        q = rotate(plain.rms_norm(q, w[f"l{i}.q_norm"], 1e-5, f32), cos, sin, rotary_dim)
        k = rotate(plain.rms_norm(k, w[f"l{i}.k_norm"], 1e-5, f32), cos, sin, rotary_dim)
        a = plain.attention(q, k, v, HEAD_DIM ** -0.5, window, f32).reshape(S, N_HEADS * HEAD_DIM)
        return plain.linear(a, w[f"l{i}.o_proj"], f32)

    # layer 0: interpolated partial rotation, all keys, SwiGLU
    i2 = torch.arange(0, ROTARY_DIM, 2, dtype=torch.float32)
    angle = (positions.float() / FACTOR)[:, None] * BASE ** (-i2 / ROTARY_DIM)
    n = plain.rms_norm(h, w["l0.n1"], 1e-5, f32)
    h = h + attention(n, 0, angle.cos(), angle.sin(), ROTARY_DIM, None)
    n = plain.rms_norm(h, w["l0.n2"], 1e-5, f32)
    g, u = plain.linear(n, w["l0.gate_proj"], f32), plain.linear(n, w["l0.up_proj"], f32)
    h = h + plain.linear(plain.swiglu(g, u, f32), w["l0.down_proj"], f32)

    # layer 1: plain rotation over the whole head, a window, routed experts
    cos, sin = plain.rope_cos_sin(positions, HEAD_DIM, 10000.0, f32)
    n = plain.rms_norm(h, w["l1.n1"], 1e-5, f32)
    h = h + attention(n, 1, cos[:, :HEAD_DIM // 2], sin[:, :HEAD_DIM // 2], HEAD_DIM, WINDOW)
    n = plain.rms_norm(h, w["l1.n2"], 1e-5, f32)
    hidden, experts = cfg["hidden_size"], cfg["n_experts"]
    up = w["l1.up"].reshape(experts, 2 * hidden, hidden)
    down = w["l1.down"].reshape(experts, hidden, 2 * hidden)
    out = torch.empty_like(n)
    choices = []
    for r in range(S):
        e = int((n[r] @ w["l1.router"].t()).argmax())
        choices.append(e)
        out[r] = down[e] @ torch.relu(up[e] @ n[r])
    h = h + out
    return (plain.rms_norm(h, w["final"], 1e-5, f32) @ w["head"].t()).numpy(), choices


def test_routed_feed_forward_and_another_position_encoding(tmp_path):
    Config = define_routed_toy()
    from thing_htn_2026_b200.weights import write_random_model
    folder = write_random_model(str(tmp_path / "routed"), Config(101, 40, 3), seed=11, gain_std=0.1)
    requests = {f"r{i}": torch.randint(0, 101, (n,), generator=torch.Generator().manual_seed(40 + i)).tolist()
                for i, n in enumerate([25, 6, 41, 70])}
    whole = harness.replay(folder, "float32", harness.trace_whole(requests), str(tmp_path / "w"))
    tail = harness.replay(folder, "float32", harness.trace_tail(requests, 8), str(tmp_path / "t"))
    batches = [{k: requests[k] for k in ("r0", "r1")}, {k: requests[k] for k in ("r2", "r3")}]
    mixed = harness.replay(folder, "float32", harness.trace_batches(batches, {"r0": 5, "r1": 6, "r2": 1, "r3": 64}),
                           str(tmp_path / "b"), max_tokens=192)
    used = set()
    for name, toks in requests.items():
        want, choices = routed_toy_plain_logits(folder, toks)
        used.update(choices)
        for what, got in (("whole", whole), ("tail", tail), ("batches", mixed)):
            assert np.abs(got[name] - want).max() <= 1e-4, f"{what} {name}: {np.abs(got[name] - want).max():.2e}"
    assert len(used) > 1, "the random router sends every row to the same expert: the test shows nothing"


# ----------------------------------------------------------------------------- other block arrangements


def define_sandwich_toy():
    """Two block arrangements that live only in this test: one with a third norm (behind the
    mixer) whose gain is stored as ``w`` of ``1 + w`` and drawn by an initializer registered
    here, and one that has no feed-forward at all."""
    from dataclasses import dataclass

    from thing_htn_2026_b200 import ops
    from thing_htn_2026_b200.config import register_architecture
    from thing_htn_2026_b200.config.base import LayerSpec, ModelConfig, ModelPlan, PartSpec, ScheduleEntry
    from thing_htn_2026_b200.config.registry import _decoder_model, known_architectures
    from thing_htn_2026_b200.parts import Block, register_part
    from thing_htn_2026_b200.weights import GAIN, INITIALIZERS, TensorSpec, register_initializer

    if "toy_around_zero" not in INITIALIZERS:
        register_initializer("toy_around_zero", lambda t, gen, matrix_std, gain_std: t.normal_(0.0, gain_std, generator=gen))

    @register_part("norm", "toy_one_plus_rmsnorm")
    class OnePlusRMSNorm:
        @classmethod
        def tensor_specs(cls, spec):
            return [TensorSpec(spec.tensors["weight"], (spec.params["size"],), GAIN, init="toy_around_zero")]

        def __init__(self, spec, rt):
            self.eps = spec.params["eps"]
            self.gain = (1.0 + rt.tensor(spec, "weight").float()).to(rt.tensor(spec, "weight").dtype)

        def forward(self, x):
            return ops.rmsnorm(x, self.gain, self.eps)

        def add_forward(self, h, d):
            return ops.add_rmsnorm(h, d, self.gain, self.eps)

    @register_part("block", "toy_sandwich")
    class SandwichBlock(Block):
        MEMBERS = {"norm_mixer": "norm", "mixer": "mixer", "norm_after": "norm", "norm_ffn": "norm", "ffn": "ffn"}

        def forward(self, h, d, ctx, entry):
            n = self.norm_mixer.forward(h) if d is None else self.norm_mixer.add_forward(h, d)
            a = self.norm_after.forward(self.mixer.forward(n, ctx, entry))
            n = self.norm_ffn.add_forward(h, a)
            return h, self.ffn.forward(n, ctx)

    @register_part("block", "toy_mixer_only")
    class MixerOnlyBlock(Block):
        MEMBERS = {"norm_mixer": "norm", "mixer": "mixer"}

        def forward(self, h, d, ctx, entry):
            n = self.norm_mixer.forward(h) if d is None else self.norm_mixer.add_forward(h, d)
            return h, self.mixer.forward(n, ctx, entry)

    @dataclass(frozen=True)
    class SandwichToyConfig(ModelConfig):
        vocab_size: int
        hidden_size: int
        architecture = "SandwichToyForCausalLM"

        @classmethod
        def from_dict(cls, data):
            return cls(data["vocab_size"], data["hidden_size"])

        def to_dict(self):
            return {"architectures": [self.architecture], "vocab_size": self.vocab_size, "hidden_size": self.hidden_size}

        def plan(self):
            h = self.hidden_size

            def norm(name):
                return PartSpec("rmsnorm", {"size": h, "eps": 1e-5}, {"weight": name})

            def attention(i):
                return PartSpec("attention", {"hidden_size": h, "n_heads": N_HEADS, "n_kv_heads": N_KV, "head_dim": HEAD_DIM,
                                              "scale": HEAD_DIM ** -0.5, "window": None, "qk_norm_eps": None,
                                              "position": PartSpec("rope", {"head_dim": HEAD_DIM, "theta": 10000.0})},
                                {k: f"l{i}.{k}" for k in ("q_proj", "k_proj", "v_proj", "o_proj", "q_norm", "k_norm")})

            layers = (
                LayerSpec.of("toy_sandwich", mixer=attention(0), norm_mixer=norm("l0.n1"), norm_ffn=norm("l0.n2"),
                             norm_after=PartSpec("toy_one_plus_rmsnorm", {"size": h, "eps": 1e-5}, {"weight": "l0.after"}),
                             ffn=PartSpec("swiglu", {"hidden_size": h, "intermediate_size": 2 * h},
                                          {k: f"l0.{k}" for k in ("gate_proj", "up_proj", "down_proj")})),
                LayerSpec.of("toy_mixer_only", mixer=attention(1), norm_mixer=norm("l1.n1")),
            )
            return ModelPlan(h, self.vocab_size,
                             PartSpec("embedding", {"vocab_size": self.vocab_size, "hidden_size": h}, {"weight": "emb"}),
                             layers, (ScheduleEntry(0, 0), ScheduleEntry(1, 1)), norm("final"),
                             PartSpec("lm_head", {"vocab_size": self.vocab_size, "hidden_size": h, "tied": False},
                                      {"weight": "head"}), 1024, ignored_tensors=("*.running_stat",))

    if "SandwichToyForCausalLM" not in known_architectures():
        register_architecture("SandwichToyForCausalLM", SandwichToyConfig, _decoder_model)
    return SandwichToyConfig


def sandwich_toy_plain_logits(folder, tokens):
    w = plain.read_safetensors(os.path.join(folder, "model.safetensors"))
    f32 = torch.float32
    S = len(tokens)
    cos, sin = plain.rope_cos_sin(torch.arange(S), HEAD_DIM, 10000.0, f32)
    h = w["emb"][torch.tensor(tokens)]

    def attention(n, i):
        q = plain.linear(n, w[f"l{i}.q_proj"], f32).reshape(S, N_HEADS, HEAD_DIM)
        k = plain.linear(n, w[f"l{i}.k_proj"], f32).reshape(S, N_KV, HEAD_DIM)
        v = plain.linear(n, w[f"l{i}.v_proj"], f32).reshape(S, N_KV, HEAD_DIM)
        q, k = plain.apply_rope(q, cos, sin, f32), plain.apply_rope(k, cos, sin, f32)
        a = plain.attention(q, k, v, HEAD_DIM ** -0.5, None, f32).reshape(S, N_HEADS * HEAD_DIM)
        return plain.linear(a, w[f"l{i}.o_proj"], f32)

    a = attention(plain.rms_norm(h, w["l0.n1"], 1e-5, f32), 0)
    h = h + plain.rms_norm(a, 1.0 + w["l0.after"], 1e-5, f32)
    n = plain.rms_norm(h, w["l0.n2"], 1e-5, f32)
    g, u = plain.linear(n, w["l0.gate_proj"], f32), plain.linear(n, w["l0.up_proj"], f32)
    h = h + plain.linear(plain.swiglu(g, u, f32), w["l0.down_proj"], f32)
    h = h + attention(plain.rms_norm(h, w["l1.n1"], 1e-5, f32), 1)
    return (plain.rms_norm(h, w["final"], 1e-5, f32) @ w["head"].t()).numpy()


def test_blocks_with_a_third_norm_and_without_a_feed_forward(tmp_path):
    """The model above sees blocks only: these two arrangements, their tensors (one with an
    initializer of its own), their cache needs and the buffer their checkpoint carries are
    all the test's; no file of the library changes."""
    Config = define_sandwich_toy()
    from thing_htn_2026_b200.weights import Checkpoint, write_random_model, write_safetensors
    folder = write_random_model(str(tmp_path / "sandwich"), Config(90, 48), seed=5, gain_std=0.1)
    stored = Checkpoint(folder)
    tensors = {name: stored.read(name) for name in stored.names()}
    assert abs(tensors["l0.after"].mean().item()) < 0.05 and abs(tensors["l0.n1"].mean().item() - 1) < 0.05
    assert not any(name.startswith("l1.gate") or name.startswith("l1.n2") for name in tensors)
    tensors["l0.mixer.running_stat"] = torch.ones(3)           # a buffer the plan says to pass over
    write_safetensors(os.path.join(folder, "model.safetensors"), tensors)
    requests = {f"r{i}": torch.randint(0, 90, (n,), generator=torch.Generator().manual_seed(60 + i)).tolist()
                for i, n in enumerate([25, 6, 41, 70])}
    whole = harness.replay(folder, "float32", harness.trace_whole(requests), str(tmp_path / "w"))
    tail = harness.replay(folder, "float32", harness.trace_tail(requests, 8), str(tmp_path / "t"))
    batches = [{k: requests[k] for k in ("r0", "r1")}, {k: requests[k] for k in ("r2", "r3")}]
    mixed = harness.replay(folder, "float32", harness.trace_batches(batches, {"r0": 5, "r1": 6, "r2": 1, "r3": 64}),
                           str(tmp_path / "b"), max_tokens=192)
    for name, toks in requests.items():
        want = sandwich_toy_plain_logits(folder, toks)
        for what, got in (("whole", whole), ("tail", tail), ("batches", mixed)):
            assert np.abs(got[name] - want).max() <= 1e-4, f"{what} {name}: {np.abs(got[name] - want).max():.2e}"
