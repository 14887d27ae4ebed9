"""Configuration: typed reading of config.json keys, validation, the registry, the plan."""

import json

import pytest

import tiny
from thing_htn_2026_b200.config import (ConfigError, Qwen3Config, config_from_dict, known_architectures,
                                        load_config, register_architecture)
from thing_htn_2026_b200.config.base import LayerSpec, ModelPlan, PartSpec, ScheduleEntry


def test_reads_every_size_from_config_json():
    for name in tiny.CONFIGS:
        raw = tiny.config_json(name)
        cfg = config_from_dict(raw)
        assert isinstance(cfg, Qwen3Config)
        for key in ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads",
                    "num_key_value_heads", "head_dim", "rms_norm_eps", "rope_theta", "tie_word_embeddings"):
            assert getattr(cfg, key) == raw[key], key


def test_head_dim_defaults_and_is_independent():
    raw = tiny.config_json("a")
    del raw["head_dim"]
    assert config_from_dict(raw).head_dim == raw["hidden_size"] // raw["num_attention_heads"]
    raw["head_dim"] = 48                     # wider than hidden / heads, as in the 4B model
    cfg = config_from_dict(raw)
    assert cfg.head_dim == 48
    q = cfg.plan().layers[0].part("mixer")
    assert q.params["head_dim"] == 48 and q.params["scale"] == 48 ** -0.5


def test_plan_carries_sizes_names_and_windows():
    cfg = config_from_dict(tiny.config_json("c"))
    plan = cfg.plan()
    assert len(plan.layers) == 4 and [e.layer for e in plan.schedule] == [0, 1, 2, 3]
    assert [l.part("mixer").params["window"] for l in plan.layers] == [None, 24, None, 24]
    layer = plan.layers[2]
    assert layer.part("mixer").tensors["q_proj"] == "model.layers.2.self_attn.q_proj.weight"
    assert layer.part("ffn").tensors["down_proj"] == "model.layers.2.mlp.down_proj.weight"
    assert layer.part("norm_mixer").params == {"size": 80, "eps": 3e-6}
    assert plan.head.tensors["weight"] == "lm_head.weight"
    tied = config_from_dict(tiny.config_json("a")).plan()
    assert tied.head.tensors["weight"] == "model.embed_tokens.weight"
    assert layer.part("mixer").params["position"].params["theta"] == 500000.0


def test_window_keys():
    raw = tiny.config_json("a")
    raw.update(sliding_window=16, use_sliding_window=False)
    assert config_from_dict(raw).sliding_window is None
    raw.update(use_sliding_window=True, max_window_layers=1)
    cfg = config_from_dict(raw)
    assert cfg.layer_types == ("full_attention", "sliding_attention")
    raw2 = tiny.config_json("a")
    raw2["layer_types"] = ["sliding_attention", "full_attention"]
    with pytest.raises(ConfigError, match="sliding_window is null"):
        config_from_dict(raw2)


@pytest.mark.parametrize("change,match", [
    ({"num_key_value_heads": 3}, "not a multiple"),
    ({"head_dim": 15}, "must be even"),
    ({"hidden_act": "gelu"}, "hidden_act"),
    ({"attention_bias": True}, "attention_bias"),
    ({"rope_scaling": {"rope_type": "yarn", "factor": 4.0}}, "rope_scaling"),
    ({"rms_norm_eps": 0.0}, "rms_norm_eps"),
    ({"vocab_size": None}, "vocab_size"),
    ({"hidden_size": "64"}, "hidden_size"),
    ({"layer_types": ["full_attention"]}, "layer_types"),
    ({"architectures": ["LlamaForCausalLM"]}, "not registered"),
    ({"architectures": []}, "architectures"),
])
def test_refuses_what_it_cannot_run(change, match):
    raw = tiny.config_json("a")
    raw.update(change)
    with pytest.raises(ConfigError, match=match):
        config_from_dict(raw)


def test_rope_parameters_spelling():
    raw = tiny.config_json("a")
    del raw["rope_theta"]
    raw["rope_parameters"] = {"rope_type": "default", "rope_theta": 12345.0}
    assert config_from_dict(raw).rope_theta == 12345.0
    del raw["rope_parameters"]
    with pytest.raises(ConfigError, match="rope_theta"):
        config_from_dict(raw)


def test_load_config_errors(tmp_path):
    with pytest.raises(ConfigError, match="not found"):
        load_config(str(tmp_path))
    (tmp_path / "config.json").write_text("{ not json")
    with pytest.raises(ConfigError, match="not valid JSON"):
        load_config(str(tmp_path))
    (tmp_path / "config.json").write_text(json.dumps(tiny.config_json("b")))
    assert load_config(str(tmp_path)).hidden_size == 96


def test_round_trip_through_to_dict():
    for name in tiny.CONFIGS:
        cfg = config_from_dict(tiny.config_json(name))
        assert config_from_dict(cfg.to_dict()) == cfg


def test_registry():
    assert "Qwen3ForCausalLM" in known_architectures()
    with pytest.raises(ValueError, match="already registered"):
        register_architecture("Qwen3ForCausalLM", Qwen3Config, lambda: object)


def test_schedule_rules():
    part = PartSpec("x")
    layer = LayerSpec.of("pre_norm", mixer=part, ffn=part, norm_mixer=part, norm_ffn=part)

    def plan(schedule):
        return ModelPlan(8, 8, part, (layer, layer), tuple(schedule), part, part, 64)

    shared = plan([ScheduleEntry(0, 0), ScheduleEntry(1, 0, writes_cache=False), ScheduleEntry(0, 1)])
    assert shared.n_cache_entries == 2          # a layer named twice, a layer reading another's cache
    with pytest.raises(ConfigError, match="both write"):
        plan([ScheduleEntry(0, 0), ScheduleEntry(1, 0)])
    with pytest.raises(ConfigError, match="before any entry has written"):
        plan([ScheduleEntry(0, 0, writes_cache=False), ScheduleEntry(1, 0)])
    with pytest.raises(ConfigError, match="names layer"):
        plan([ScheduleEntry(2, 0)])
