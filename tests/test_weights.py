"""Weights: the safetensors reader and writer, loading by tensor name with one error that
lists everything wrong, precision rules, and the random-weights mode."""

import json
import os
import struct

import pytest
import torch

import tiny
from plain import qwen3_plain as plain
from thing_htn_2026_b200.config import config_from_dict
from thing_htn_2026_b200.models.decoder import tensor_specs_of_plan
from thing_htn_2026_b200.weights import (GAIN, MATRIX, Checkpoint, SafetensorsError, TensorSpec,
                                         UndeclaredTensorsWarning, WeightError,
                                         held_dtype, load_tensors, random_tensors_cpu, write_random_model,
                                         write_safetensors)

CPU = torch.device("cpu")


def specs_of(name):
    return tensor_specs_of_plan(config_from_dict(tiny.config_json(name)).plan())


def test_expected_tensor_names_and_shapes():
    specs = {s.name: s for s in specs_of("b")}
    assert specs["model.embed_tokens.weight"].shape == (512, 96)
    assert specs["model.layers.2.self_attn.q_proj.weight"].shape == (256, 96)     # 8 heads x 32, hidden 96
    assert specs["model.layers.0.self_attn.k_proj.weight"].shape == (32, 96)
    assert specs["model.layers.0.self_attn.o_proj.weight"].shape == (96, 256)
    assert specs["model.layers.1.self_attn.q_norm.weight"].shape == (32,)
    assert specs["model.layers.1.mlp.gate_proj.weight"].shape == (160, 96)
    assert specs["model.layers.1.mlp.down_proj.weight"].shape == (96, 160)
    assert specs["lm_head.weight"].shape == (512, 96)
    assert specs["model.norm.weight"].role == GAIN
    assert "lm_head.weight" not in {s.name for s in specs_of("a")}                 # tied


def test_round_trip_all_dtypes(tmp_path):
    tensors = {
        "f32": torch.randn(3, 5), "bf16": torch.randn(7).bfloat16(), "f16": torch.randn(2, 2).half(),
        "i64": torch.arange(6).reshape(2, 3), "i32": torch.arange(4, dtype=torch.int32), "scalar": torch.tensor(2.5),
    }
    path = str(tmp_path / "model.safetensors")
    write_safetensors(path, tensors, metadata={"format": "pt"})
    ckpt = Checkpoint(str(tmp_path))
    assert set(ckpt.names()) == set(tensors)
    for name, want in tensors.items():
        got = ckpt.read(name)
        assert got.dtype == want.dtype and got.shape == want.shape and torch.equal(got, want)
    # the plain implementation's own reader agrees
    other = plain.read_safetensors(path)
    assert torch.equal(other["bf16"], tensors["bf16"].float())


def test_loads_and_keeps_precisions(tiny_models):
    for dtype in (torch.float32, torch.bfloat16):
        got = load_tensors(tiny_models["a"], specs_of("a"), dtype, CPU)       # stored in float32
        assert got["model.embed_tokens.weight"].dtype == dtype
        assert got["model.norm.weight"].dtype == torch.float32                # a stored 32-bit vector stays 32-bit
        got = load_tensors(tiny_models["c"], specs_of("c"), dtype, CPU)       # stored in bfloat16
        assert got["model.layers.0.mlp.up_proj.weight"].dtype == dtype
        assert got["model.norm.weight"].dtype == dtype
    assert held_dtype(torch.int64, "table", torch.bfloat16) == torch.int32


def test_one_error_lists_everything(tmp_path, tiny_models):
    good = Checkpoint(tiny_models["b"])
    tensors = {name: good.read(name) for name in good.names()}
    del tensors["model.layers.1.mlp.up_proj.weight"]
    del tensors["lm_head.weight"]
    tensors["model.layers.0.self_attn.q_proj.weight"] = torch.zeros(96, 256)
    tensors["model.layers.7.extra.weight"] = torch.zeros(1)
    os.makedirs(tmp_path / "m")
    write_safetensors(str(tmp_path / "m" / "model.safetensors"), tensors)
    with pytest.raises(WeightError) as info:
        load_tensors(str(tmp_path / "m"), specs_of("b"), torch.float32, CPU)
    error = info.value
    assert error.missing == ["model.layers.1.mlp.up_proj.weight", "lm_head.weight"]
    assert error.unexpected == ["model.layers.7.extra.weight"]
    assert error.wrong == [("model.layers.0.self_attn.q_proj.weight", (96, 256), (256, 96))]
    text = str(error)
    for needle in ("missing tensors (2)", "unexpected tensors (1)", "wrong shapes (1)", "file [96, 256], model [256, 96]"):
        assert needle in text


def hand_written_folder(tmp_path, source, change):
    """A folder that this library did not write: the tensors of ``source``, changed by hand."""
    good = Checkpoint(source)
    tensors = {name: good.read(name) for name in good.names()}
    change(tensors)
    write_safetensors(str(tmp_path / "model.safetensors"), tensors)
    return str(tmp_path)


def test_tied_head_needs_no_head_tensor_and_accepts_a_stored_copy(tmp_path, tiny_models, recwarn):
    plan = config_from_dict(tiny.config_json("a")).plan()
    assert "lm_head.weight" not in Checkpoint(tiny_models["a"]).names()

    def add_copy(tensors):
        tensors["lm_head.weight"] = tensors["model.embed_tokens.weight"].clone()

    folder = hand_written_folder(tmp_path, tiny_models["a"], add_copy)
    got = load_tensors(folder, specs_of("a"), torch.float32, CPU, ignored=plan.ignored_tensors, strict=True)
    assert "lm_head.weight" not in got and not recwarn.list      # an equal copy: accepted in silence, even strictly


def test_a_stored_head_that_differs_from_the_tied_embedding_is_reported(tmp_path, tiny_models):
    def add_other(tensors):
        tensors["lm_head.weight"] = tensors["model.embed_tokens.weight"] + 1.0

    folder = hand_written_folder(tmp_path, tiny_models["a"], add_other)
    with pytest.warns(UndeclaredTensorsWarning, match="lm_head.weight is stored beside model.embed_tokens.weight"):
        got = load_tensors(folder, specs_of("a"), torch.float32, CPU)
    assert torch.equal(got["model.embed_tokens.weight"], Checkpoint(tiny_models["a"]).read("model.embed_tokens.weight"))

    def add_misshapen(tensors):
        tensors["lm_head.weight"] = torch.zeros(3, 3)

    (tmp_path / "b").mkdir()
    folder = hand_written_folder(tmp_path / "b", tiny_models["a"], add_misshapen)
    with pytest.raises(WeightError, match="wrong shapes"):
        load_tensors(folder, specs_of("a"), torch.float32, CPU)


def test_undeclared_tensors_warn_once_and_buffers_pass_in_silence(tmp_path, tiny_models, recwarn):
    plan = config_from_dict(tiny.config_json("b")).plan()

    def add_extras(tensors):
        tensors["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.ones(16)     # a writer's buffer
        tensors["model.layers.7.extra.weight"] = torch.zeros(1)
        tensors["adapter.scale"] = torch.zeros(2)

    folder = hand_written_folder(tmp_path, tiny_models["b"], add_extras)
    with pytest.warns(UndeclaredTensorsWarning) as caught:
        got = load_tensors(folder, specs_of("b"), torch.float32, CPU, ignored=plan.ignored_tensors)
    assert len(caught) == 1
    text = str(caught[0].message)
    assert "2 tensors that no part of the model reads" in text
    assert "model.layers.7.extra.weight" in text and "adapter.scale" in text and "inv_freq" not in text
    assert set(got) == {s.name for s in specs_of("b")}
    with pytest.raises(WeightError, match=r"unexpected tensors \(2\)"):
        load_tensors(folder, specs_of("b"), torch.float32, CPU, ignored=plan.ignored_tensors, strict=True)


def test_initializer_rules_by_name():
    from thing_htn_2026_b200.weights import INITIALIZERS, register_initializer
    from thing_htn_2026_b200.weights.random_init import _draw
    g = torch.Generator().manual_seed(3)
    bias = _draw(TensorSpec("b", (64,), GAIN, init="zeros"), g, "cpu", 0.02, 0.1, torch.float32)
    assert bias.abs().max() == 0                                   # a role's default can be overridden per tensor
    if "test_small_gain" not in INITIALIZERS:
        register_initializer("test_small_gain", lambda t, gen, matrix_std, gain_std: t.normal_(0, gain_std, generator=gen))
    w = _draw(TensorSpec("w", (4096,), GAIN, init="test_small_gain"), g, "cpu", 0.02, 0.1, torch.float32)
    assert abs(w.mean().item()) < 0.02 and 0.05 < w.std().item() < 0.15      # a gain stored as w of (1 + w)
    with pytest.raises(KeyError, match="no initializer named"):
        _draw(TensorSpec("x", (2,), MATRIX, init="nope"), g, "cpu", 0.02, 0.1, torch.float32)


def test_broken_files(tmp_path):
    with pytest.raises(SafetensorsError, match="neither"):
        Checkpoint(str(tmp_path))
    path = tmp_path / "model.safetensors"
    path.write_bytes(b"\x01\x02")
    with pytest.raises(SafetensorsError, match="truncated"):
        Checkpoint(str(tmp_path))
    path.write_bytes(struct.pack("<Q", 1000) + b"{}")
    with pytest.raises(SafetensorsError, match="exceeds file size"):
        Checkpoint(str(tmp_path))
    path.write_bytes(struct.pack("<Q", 5) + b"{nope")
    with pytest.raises(SafetensorsError, match="not valid JSON"):
        Checkpoint(str(tmp_path))
    header = json.dumps({"w": {"dtype": "F32", "shape": [4], "data_offsets": [0, 16]}}).encode()
    path.write_bytes(struct.pack("<Q", len(header)) + header + b"\x00" * 8)
    with pytest.raises(SafetensorsError, match="truncated"):
        Checkpoint(str(tmp_path))
    header = json.dumps({"w": {"dtype": "F32", "shape": [4], "data_offsets": [0, 12]}}).encode()
    path.write_bytes(struct.pack("<Q", len(header)) + header + b"\x00" * 12)
    with pytest.raises(SafetensorsError, match="needs 16 bytes"):
        Checkpoint(str(tmp_path))
    header = json.dumps({"w": {"dtype": "Q4", "shape": [4], "data_offsets": [0, 4]}}).encode()
    path.write_bytes(struct.pack("<Q", len(header)) + header + b"\x00" * 4)
    with pytest.raises(SafetensorsError, match="unknown dtype"):
        Checkpoint(str(tmp_path))


def test_sharded_folder(tmp_path, tiny_models):
    good = Checkpoint(tiny_models["a"])
    names = list(good.names())
    half = len(names) // 2
    write_safetensors(str(tmp_path / "one.safetensors"), {n: good.read(n) for n in names[:half]})
    write_safetensors(str(tmp_path / "two.safetensors"), {n: good.read(n) for n in names[half:]})
    index = {"weight_map": {n: ("one.safetensors" if i < half else "two.safetensors") for i, n in enumerate(names)}}
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps(index))
    got = load_tensors(str(tmp_path), specs_of("a"), torch.float32, CPU)
    assert torch.equal(got[names[-1]], good.read(names[-1]).float())


def test_random_weights_mode(tmp_path):
    config = config_from_dict(tiny.config_json("b"))
    folder = write_random_model(str(tmp_path / "m"), config, seed=1)
    assert sorted(os.listdir(folder)) == ["config.json", "model.safetensors"]
    again = random_tensors_cpu(config, seed=1)
    other = random_tensors_cpu(config, seed=2)
    ckpt = Checkpoint(folder)
    for spec in specs_of("b"):
        stored = ckpt.read(spec.name)
        assert stored.shape == spec.shape and stored.dtype == torch.float32
        assert torch.equal(stored, again[spec.name]) and not torch.equal(stored, other[spec.name])
    matrix = ckpt.read("model.embed_tokens.weight")
    gain = ckpt.read("model.layers.0.input_layernorm.weight")
    assert abs(matrix.std().item() - 0.02) < 2e-3 and abs(matrix.mean().item()) < 2e-3
    assert abs(gain.mean().item() - 1.0) < 0.05 and 0.05 < gain.std().item() < 0.2
    assert config_from_dict(json.load(open(os.path.join(folder, "config.json")))) == config
