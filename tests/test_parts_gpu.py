"""Each part alone (norm, position encoding, feed-forward, mixer, block, embedding and head)
against the plain implementation; the order of layers as data (a layer named twice, a
layer reading another layer's cache); and a toy mixer with per-sequence state of its own,
defined here, registered, built and stepped without touching the library's files."""

import json
import os

import numpy as np
import pytest
import torch

import harness
import tiny
from plain import qwen3_plain as plain

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DTYPES = [torch.float32, torch.bfloat16]


def rand(shape, dtype, seed, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).to(dtype)


def close(got, want, dtype, what):
    got, want = got.float().cpu(), want.float().cpu()
    if dtype == torch.float32:
        err = (got - want).abs().max().item()
        assert err <= 3e-5 * max(1.0, want.abs().max().item()), f"{what}: float32 differs by {err:.3e}"
    else:
        bad = (got - want).abs() > 1e-2 + want.abs() / 64         # engine/engine.py:425-429
        assert not bad.any(), f"{what}: {int(bad.sum())} of {bad.numel()} bfloat16 values out of tolerance"


def runtime(dtype, tensors):
    from thing_htn_2026_b200.parts import Runtime
    return Runtime(dtype, torch.device(DEV), {k: v.to(DEV) for k, v in tensors.items()})


def step_context(cache, slots, counts):
    """A StepContext for ``counts[i]`` new tokens of ``slots[i]`` (pages mapped, rows made)."""
    from thing_htn_2026_b200 import ops
    from thing_htn_2026_b200.parts import StepContext
    cache.prepare(slots, counts)
    cu = [0]
    for c in counts:
        cu.append(cu[-1] + c)
    cu_dev = torch.tensor(cu, dtype=torch.int32, device=DEV)
    slots_dev = torch.tensor(slots, dtype=torch.int32, device=DEV)
    rows = ops.step_rows(cu_dev, slots_dev, cache.seq_lens, cu[-1], max(counts))
    inputs = {}
    if max(counts) > 1:
        # what the attention part asks of the step function for steps of several rows
        size = ops.ROW_TILE()
        r0, rn = ops.row_tiles_of(counts, [cache.length(s) for s in slots], size)
        inputs = {f"row_tiles/{size}/row0": torch.tensor(r0, dtype=torch.int32, device=DEV),
                  f"row_tiles/{size}/rows": torch.tensor(rn, dtype=torch.int32, device=DEV)}
    return StepContext(rows=rows, cache=cache, err=ops.new_error_word(DEV), inputs=inputs), cu


def finish_step(cache, ctx, slots, counts):
    from thing_htn_2026_b200 import ops
    ops.advance(cache.seq_lens, ctx.rows.slots, ctx.rows.cu_seqlens)
    cache.commit(slots, counts)
    assert int(ctx.err.item()) == 0


@pytest.mark.parametrize("dtype", DTYPES)
def test_norm_part(dtype):
    from thing_htn_2026_b200.config.base import PartSpec
    from thing_htn_2026_b200.parts import part_class
    w = (1 + 0.2 * torch.randn(200, generator=torch.Generator().manual_seed(1))).to(dtype)
    part = part_class("norm", "rmsnorm")(PartSpec("rmsnorm", {"size": 200, "eps": 1e-5}, {"weight": "g"}),
                                         runtime(dtype, {"g": w}))
    x, d = rand((7, 200), dtype, 2), rand((7, 200), dtype, 3)
    close(part.forward(x.to(DEV)), plain.rms_norm(x, w, 1e-5, dtype), dtype, "norm")
    h = x.clone().to(DEV)
    y = part.add_forward(h, d.to(DEV))
    assert torch.equal(h.cpu(), plain.add_residual(x, d, dtype))
    close(y, plain.rms_norm(plain.add_residual(x, d, dtype), w, 1e-5, dtype), dtype, "add + norm")


@pytest.mark.parametrize("dtype", DTYPES)
def test_feed_forward_part(dtype):
    from thing_htn_2026_b200.config.base import PartSpec
    from thing_htn_2026_b200.parts import part_class
    hidden, inter = 72, 200
    tensors = {"g": rand((inter, hidden), dtype, 4, 0.1), "u": rand((inter, hidden), dtype, 5, 0.1),
               "d": rand((hidden, inter), dtype, 6, 0.1)}
    spec = PartSpec("swiglu", {"hidden_size": hidden, "intermediate_size": inter},
                    {"gate_proj": "g", "up_proj": "u", "down_proj": "d"})
    part = part_class("ffn", "swiglu")(spec, runtime(dtype, tensors))
    assert [s.shape for s in part.tensor_specs(spec)] == [(inter, hidden), (inter, hidden), (hidden, inter)]
    x = rand((9, hidden), dtype, 7)
    weights = {"model.layers.0.mlp.gate_proj.weight": tensors["g"], "model.layers.0.mlp.up_proj.weight": tensors["u"],
               "model.layers.0.mlp.down_proj.weight": tensors["d"]}
    from thing_htn_2026_b200 import ops
    got = part.forward(x.to(DEV), None)
    close(got, plain.mlp_block(x, weights, 0, dtype), dtype, "feed-forward")


@pytest.mark.parametrize("dtype", DTYPES)
def test_embedding_and_head_parts(dtype):
    from thing_htn_2026_b200 import ops
    from thing_htn_2026_b200.config.base import PartSpec
    from thing_htn_2026_b200.parts import part_class
    table = rand((333, 40), dtype, 8)
    rt = runtime(dtype, {"e": table})
    emb = part_class("embedding", "embedding")(PartSpec("embedding", {"vocab_size": 333, "hidden_size": 40},
                                                        {"weight": "e"}), rt)
    head = part_class("head", "lm_head")(PartSpec("lm_head", {"vocab_size": 333, "hidden_size": 40, "tied": True},
                                                  {"weight": "e"}), rt)
    assert head.weight.data_ptr() == emb.table.data_ptr()           # tied: one tensor
    tokens = torch.tensor([0, 332, 5, 5], dtype=torch.int32, device=DEV)
    x = emb.forward(tokens, ops.new_error_word(DEV))
    assert torch.equal(x.cpu(), table[tokens.cpu().long()])
    logits = head.forward(x)
    assert logits.dtype == torch.float32
    want = x.cpu().float() @ table.float().t()
    assert (logits.cpu() - want).abs().max() <= (3e-5 if dtype == torch.float32 else 1e-2)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("n_q,n_kv,D,window", [(4, 2, 16, None), (6, 3, 48, 20), (4, 2, 64, 70), (8, 1, 128, None)])
def test_attention_part_and_block(dtype, n_q, n_kv, D, window):
    """The mixer alone, then a whole pre-norm block, over a prompt step and single-token
    steps, against the plain layer on the whole sequence."""
    from thing_htn_2026_b200.cache import SequenceCache
    from thing_htn_2026_b200.config.base import PartSpec, ScheduleEntry
    from thing_htn_2026_b200.parts import part_class
    hidden, inter, eps, theta = 80, 112, 1e-5, 54321.0
    names = {"q_proj": "q", "k_proj": "k", "v_proj": "v", "o_proj": "o", "q_norm": "qn", "k_norm": "kn"}
    tensors = {"q": rand((n_q * D, hidden), dtype, 10, 0.1), "k": rand((n_kv * D, hidden), dtype, 11, 0.1),
               "v": rand((n_kv * D, hidden), dtype, 12, 0.1), "o": rand((hidden, n_q * D), dtype, 13, 0.1),
               "qn": (1 + rand((D,), torch.float32, 14, 0.1)).to(dtype), "kn": (1 + rand((D,), torch.float32, 15, 0.1)).to(dtype),
               "n1": (1 + rand((hidden,), torch.float32, 16, 0.1)).to(dtype), "n2": (1 + rand((hidden,), torch.float32, 17, 0.1)).to(dtype),
               "g": rand((inter, hidden), dtype, 18, 0.1), "u": rand((inter, hidden), dtype, 19, 0.1),
               "d": rand((hidden, inter), dtype, 20, 0.1)}
    position = PartSpec("rope", {"head_dim": D, "rotary_dim": D, "theta": theta})
    mixer_spec = PartSpec("attention", {"hidden_size": hidden, "n_heads": n_q, "n_kv_heads": n_kv, "head_dim": D,
                                        "scale": D ** -0.5, "window": window, "qk_norm_eps": eps, "position": position},
                          names)
    rt = runtime(dtype, tensors)
    # the block builds its own members from the specs among its parameters
    block = part_class("block", "pre_norm")(PartSpec("pre_norm", {
        "mixer": mixer_spec,
        "ffn": PartSpec("swiglu", {"hidden_size": hidden, "intermediate_size": inter},
                        {"gate_proj": "g", "up_proj": "u", "down_proj": "d"}),
        "norm_mixer": PartSpec("rmsnorm", {"size": hidden, "eps": eps}, {"weight": "n1"}),
        "norm_ffn": PartSpec("rmsnorm", {"size": hidden, "eps": eps}, {"weight": "n2"}),
    }), rt)
    mixer = block.mixer
    assert block.cache_need() == mixer.cache_need()
    assert {s.name for s in type(block).tensor_specs(PartSpec("pre_norm", {"mixer": mixer_spec}))} == set(names.values())
    for part in rt.shared.values():
        part.ensure(512)

    from thing_htn_2026_b200 import ops
    lengths = [150, 9]
    xs = [rand((n, hidden), dtype, 30 + i) for i, n in enumerate(lengths)]
    w = {"model.layers.0.self_attn." + k + ".weight": tensors[v] for k, v in names.items()}
    w.update({"model.layers.0.mlp.gate_proj.weight": tensors["g"], "model.layers.0.mlp.up_proj.weight": tensors["u"],
              "model.layers.0.mlp.down_proj.weight": tensors["d"]})
    cfg = {"Nq": n_q, "Nkv": n_kv, "D": D, "eps": eps, "theta": theta, "windows": [window]}

    for use_block in (False, True):
        cache = SequenceCache([mixer.cache_need()], max_tokens=512, dtype=dtype, device=DEV, max_slots=4)
        slots = cache.open(2)
        entry = ScheduleEntry(layer=0, cache=0)
        got = [[], []]
        # a prompt step of unequal lengths, then three single-token steps
        heads = [n - 3 for n in lengths]
        plan = [heads] + [[1, 1]] * 3
        done = [0, 0]
        for counts in plan:
            ctx, cu = step_context(cache, slots, counts)
            x = torch.cat([xs[i][done[i]:done[i] + c] for i, c in enumerate(counts)]).to(DEV)
            if use_block:
                h, d = block.forward(x.clone(), None, ctx, entry)
                out = plain.add_residual(h.cpu(), d.cpu(), dtype)
            else:
                out = mixer.forward(x, ctx, entry).cpu()
            for i, c in enumerate(counts):
                got[i].append(out[cu[i]:cu[i] + c])
                done[i] += c
            finish_step(cache, ctx, slots, counts)
        def plain_layer(x, dt):
            positions = torch.arange(x.shape[0])
            if not use_block:
                return plain.attention_block(x.to(dt), w, cfg, 0, positions, dt)
            nrm = plain.rms_norm(x.to(dt), tensors["n1"], eps, dt)
            h = plain.add_residual(x.to(dt), plain.attention_block(nrm, w, cfg, 0, positions, dt), dt)
            return plain.add_residual(h, plain.mlp_block(plain.rms_norm(h, tensors["n2"], eps, dt), w, 0, dt), dt)

        for i, n in enumerate(lengths):
            what = f"{'block' if use_block else 'mixer'} sequence {i}"
            want = plain_layer(xs[i], dtype)
            result = torch.cat(got[i])
            if dtype == torch.float32:
                close(result, want, dtype, what)
            else:
                # A chain of a dozen rounded operations.  The engine rounds where the plain
                # implementation rounds, but sums in another order, which flips a rounding
                # now and then; a flip is carried through the norm and the products like any
                # other rounding error, and a flip of the last rounding is one bfloat16 step of
                # that value.  So: no element is farther from the plain bfloat16 result than
                # bfloat16's own noise on this input (the distance of the plain bfloat16 result
                # from the plain float32 result) plus one step of its own size; and on the
                # whole the two are much closer than that noise.
                exact = plain_layer(xs[i], torch.float32)
                noise = (want.float() - exact).abs()
                err = (result.float() - want.float()).abs()
                step = torch.exp2(torch.floor(torch.log2(want.float().abs().clamp_min(1e-30))) - 7)
                worst = (err - step).max().item()
                assert worst <= noise.max().item(), f"{what}: {worst:.3e} beyond a rounding step, noise {noise.max():.3e}"
                assert err.pow(2).mean().sqrt() <= noise.pow(2).mean().sqrt(), f"{what}: rms error above the noise"
        cache.close(slots)
        cache.check()


# ----------------------------------------------------------------------------- a toy architecture


def define_toy():
    """A mixer with per-sequence state of fixed size (an exponential moving sum of a
    projection of its inputs), a configuration that mixes it with attention layer by layer,
    names one layer twice and lets one attention layer read another's cache.  Nothing of it
    lives in the library."""
    from dataclasses import dataclass

    from thing_htn_2026_b200.cache import StateSpec
    from thing_htn_2026_b200.config import register_architecture
    from thing_htn_2026_b200.config.base import LayerSpec, ModelConfig, ModelPlan, PartSpec, ScheduleEntry
    from thing_htn_2026_b200.config.registry import known_architectures
    from thing_htn_2026_b200.parts import register_part
    from thing_htn_2026_b200.weights import MATRIX, TensorSpec

    @register_part("mixer", "toy_decay")
    class DecayMixer:
        @classmethod
        def tensor_specs(cls, spec):
            h = spec.params["hidden_size"]
            return [TensorSpec(spec.tensors["proj"], (h, h), MATRIX)]

        def __init__(self, spec, rt):
            self.hidden, self.decay = spec.params["hidden_size"], spec.params["decay"]
            self.proj = rt.tensor(spec, "proj")

        def cache_need(self):
            return StateSpec((self.hidden,), torch.float32)

        def forward(self, x, ctx, entry):
            state = ctx.cache.state_view(entry.cache)             # [max_slots, hidden] float32
            cu = ctx.rows.cu_seqlens.tolist()
            slots = ctx.rows.slots.tolist()
            z = (x.float() @ self.proj.float().t())
            out = torch.empty_like(z)
            for b, slot in enumerate(slots):
                s = state[slot]
                for r in range(cu[b], cu[b + 1]):
                    s = self.decay * s + z[r]
                    out[r] = s
                state[slot] = s
            return out.to(x.dtype)

    @dataclass(frozen=True)
    class ToyConfig(ModelConfig):
        vocab_size: int
        hidden_size: int
        decay: float
        architecture = "ToyForCausalLM"

        @classmethod
        def from_dict(cls, data):
            return cls(data["vocab_size"], data["hidden_size"], data["decay"])

        def to_dict(self):
            return {"architectures": [self.architecture], "vocab_size": self.vocab_size,
                    "hidden_size": self.hidden_size, "decay": self.decay}

        def plan(self):
            h = self.hidden_size

            def norm(name):
                return PartSpec("rmsnorm", {"size": h, "eps": 1e-6}, {"weight": name})

            def ffn(i):
                return PartSpec("swiglu", {"hidden_size": h, "intermediate_size": 2 * h},
                                {k: f"l{i}.{k}" for k in ("gate_proj", "up_proj", "down_proj")})

            attention = PartSpec("attention", {"hidden_size": h, "n_heads": 2, "n_kv_heads": 1, "head_dim": 16,
                                               "scale": 0.25, "window": None, "qk_norm_eps": None, "position": None},
                                 {k: f"l0.{k}" for k in ("q_proj", "k_proj", "v_proj", "o_proj", "q_norm", "k_norm")})
            toy = PartSpec("toy_decay", {"hidden_size": h, "decay": self.decay}, {"proj": "l1.proj"})
            layers = (LayerSpec.of("pre_norm", mixer=attention, ffn=ffn(0), norm_mixer=norm("l0.n1"), norm_ffn=norm("l0.n2")),
                      LayerSpec.of("pre_norm", mixer=toy, ffn=ffn(1), norm_mixer=norm("l1.n1"), norm_ffn=norm("l1.n2")))
            # attention (writes cache 0), toy (state 1), attention again with the same weights
            # reading cache 0, toy again with a state of its own (2)
            schedule = (ScheduleEntry(0, 0), ScheduleEntry(1, 1), ScheduleEntry(0, 0, writes_cache=False),
                        ScheduleEntry(1, 2))
            return ModelPlan(h, self.vocab_size,
                             PartSpec("embedding", {"vocab_size": self.vocab_size, "hidden_size": h}, {"weight": "emb"}),
                             layers, schedule, norm("final"),
                             PartSpec("lm_head", {"vocab_size": self.vocab_size, "hidden_size": h, "tied": True},
                                      {"weight": "emb"}), 1024)

    if "ToyForCausalLM" not in known_architectures():
        from thing_htn_2026_b200.config.registry import _decoder_model
        register_architecture("ToyForCausalLM", ToyConfig, _decoder_model)
    return ToyConfig


def toy_plain_logits(folder, tokens):
    """The toy model written out plainly, whole sequence, float32."""
    w = plain.read_safetensors(os.path.join(folder, "model.safetensors"))
    cfg = json.load(open(os.path.join(folder, "config.json")))
    f32 = torch.float32
    h = w["emb"][torch.tensor(tokens)]
    S = len(tokens)

    def attn(n):
        q = plain.linear(n, w["l0.q_proj"], f32).reshape(S, 2, 16)
        k = plain.linear(n, w["l0.k_proj"], f32).reshape(S, 1, 16)
        v = plain.linear(n, w["l0.v_proj"], f32).reshape(S, 1, 16)
        return k, v, plain.linear(plain.attention(q, k, v, 0.25, None, f32), w["l0.o_proj"], f32)

    def attn_reading(n, k, v):
        q = plain.linear(n, w["l0.q_proj"], f32).reshape(S, 2, 16)
        return plain.linear(plain.attention(q, k, v, 0.25, None, f32), w["l0.o_proj"], f32)

    def toy(n):
        z = n @ w["l1.proj"].t()
        out, s = [], torch.zeros(z.shape[1])
        for r in range(S):
            s = cfg["decay"] * s + z[r]
            out.append(s)
        return torch.stack(out)

    def mlp(n, i):
        g, u = plain.linear(n, w[f"l{i}.gate_proj"], f32), plain.linear(n, w[f"l{i}.up_proj"], f32)
        return plain.linear(plain.swiglu(g, u, f32), w[f"l{i}.down_proj"], f32)

    kept = {}
    for which, layer in ((0, 0), (1, 1), (2, 0), (3, 1)):
        n = plain.rms_norm(h, w[f"l{layer}.n1"], 1e-6, f32)
        if which == 0:
            kept["k"], kept["v"], a = attn(n)
        elif which == 2:
            a = attn_reading(n, kept["k"], kept["v"])
        else:
            a = toy(n)
        h = h + a
        h = h + mlp(plain.rms_norm(h, w[f"l{layer}.n2"], 1e-6, f32), layer)
    return (plain.rms_norm(h, w["final"], 1e-6, f32) @ w["emb"].t()).numpy()


def test_toy_mixer_with_state_of_its_own(tmp_path):
    ToyConfig = define_toy()
    from thing_htn_2026_b200.weights import write_random_model
    folder = write_random_model(str(tmp_path / "toy"), ToyConfig(97, 48, 0.5), seed=5, gain_std=0.1)
    requests = {f"r{i}": torch.randint(0, 97, (n,), generator=torch.Generator().manual_seed(i)).tolist()
                for i, n in enumerate([20, 7, 33, 70])}
    # whole; token by token; unequal batches one after another on reused slots
    whole = harness.replay(folder, "float32", harness.trace_whole(requests), str(tmp_path / "w"))
    tail = harness.replay(folder, "float32", harness.trace_tail(requests, 6), str(tmp_path / "t"))
    batches = [{k: requests[k] for k in ("r0", "r1")}, {k: requests[k] for k in ("r2", "r3")}]
    mixed = harness.replay(folder, "float32", harness.trace_batches(batches, {"r0": 3, "r1": 7, "r2": 1, "r3": 64}),
                           str(tmp_path / "b"), max_tokens=192)
    for name, toks in requests.items():
        want = toy_plain_logits(folder, toks)
        for what, got in (("whole", whole), ("tail", tail), ("batches", mixed)):
            assert np.abs(got[name] - want).max() <= 1e-4, f"{what} {name}"
