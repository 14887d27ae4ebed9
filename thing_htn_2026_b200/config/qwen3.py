"""Typed configuration of the Qwen3 dense decoder (``Qwen3ForCausalLM``).

Keys and their meaning follow the reference's reader (engine/engine.py:128-141):
``hidden_size``, ``intermediate_size``, ``vocab_size``, ``num_hidden_layers``,
``num_attention_heads``, ``num_key_value_heads``, ``head_dim`` (default
``hidden_size // num_attention_heads`` and otherwise independent of both),
``rms_norm_eps``, ``rope_theta``; a non-null ``rope_scaling`` is refused there
(engine/engine.py:140-141) and here.  The attention scale is ``head_dim ** -0.5``
(engine/engine.py:139).  The reference never reads ``tie_word_embeddings`` (it
finds the tie by pointer equality after loading, engine/engine.py:225-226); a
loader that reads tensors by name needs the key itself.

The window keys (``sliding_window``, ``use_sliding_window``, ``max_window_layers``,
``layer_types``) select, layer by layer, attention over all keys or over the last
``sliding_window`` keys.  The pinned checkpoint of the reference has none
(OPTIMIZATION_GUIDE.md:36), which is the default.
"""

from __future__ import annotations

from dataclasses import dataclass, field, fields
from typing import Any, Mapping, Optional, Tuple

from .base import (ConfigError, LayerSpec, ModelConfig, ModelPlan, PartSpec,
                   ScheduleEntry, require)

FULL = "full_attention"
SLIDING = "sliding_attention"


@dataclass(frozen=True)
class Qwen3Config(ModelConfig):
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    rms_norm_eps: float
    rope_theta: float
    tie_word_embeddings: bool = False
    max_position_embeddings: int = 32768
    sliding_window: Optional[int] = None
    layer_types: Tuple[str, ...] = ()
    hidden_act: str = "silu"
    attention_bias: bool = False
    bos_token_id: Optional[int] = None
    eos_token_id: Optional[int] = None
    torch_dtype: str = "bfloat16"

    architecture = "Qwen3ForCausalLM"

    # ------------------------------------------------------------------ reading

    @classmethod
    def from_dict(cls, data: Mapping[str, Any]) -> "Qwen3Config":
        hidden = require(data, "hidden_size", int)
        heads = require(data, "num_attention_heads", int)
        kv_heads = data.get("num_key_value_heads")
        if kv_heads is None:
            kv_heads = heads
        layers = require(data, "num_hidden_layers", int)
        head_dim = data.get("head_dim")
        if head_dim is None:
            if hidden % heads:
                raise ConfigError(
                    f"config.json: 'head_dim' is absent and hidden_size {hidden} is not a multiple of "
                    f"num_attention_heads {heads}")
            head_dim = hidden // heads

        rope = data.get("rope_parameters")
        theta = data.get("rope_theta")
        if isinstance(rope, Mapping):
            kind = rope.get("rope_type", rope.get("type", "default"))
            if kind not in (None, "default"):
                raise ConfigError(f"config.json: rope_parameters.rope_type '{kind}' is not supported (only 'default')")
            theta = rope.get("rope_theta", theta)
        if data.get("rope_scaling") is not None:
            scaling = data["rope_scaling"]
            kind = scaling.get("rope_type", scaling.get("type")) if isinstance(scaling, Mapping) else scaling
            if kind not in (None, "default"):
                raise ConfigError(f"config.json: rope_scaling {scaling!r} is not supported (must be null)")
        if theta is None:
            raise ConfigError("config.json: required key 'rope_theta' is missing")

        window = data.get("sliding_window")
        if not data.get("use_sliding_window", False) and "layer_types" not in data:
            window = None
        types = data.get("layer_types")
        if types is None:
            first_sliding = data.get("max_window_layers", layers)
            types = [SLIDING if (window is not None and i >= first_sliding) else FULL for i in range(layers)]
        if window is None and any(t == SLIDING for t in types):
            raise ConfigError("config.json: layer_types names sliding_attention but sliding_window is null")

        eos = data.get("eos_token_id")
        if isinstance(eos, list):
            eos = eos[0] if eos else None

        config = cls(
            vocab_size=require(data, "vocab_size", int),
            hidden_size=hidden,
            intermediate_size=require(data, "intermediate_size", int),
            num_hidden_layers=layers,
            num_attention_heads=heads,
            num_key_value_heads=int(kv_heads),
            head_dim=int(head_dim),
            rms_norm_eps=require(data, "rms_norm_eps", float),
            rope_theta=float(theta),
            tie_word_embeddings=bool(data.get("tie_word_embeddings", False)),
            max_position_embeddings=int(data.get("max_position_embeddings", 32768)),
            sliding_window=None if window is None else int(window),
            layer_types=tuple(types),
            hidden_act=str(data.get("hidden_act", "silu")),
            attention_bias=bool(data.get("attention_bias", False)),
            bos_token_id=data.get("bos_token_id"),
            eos_token_id=eos,
            torch_dtype=str(data.get("torch_dtype", data.get("dtype", "bfloat16"))),
        )
        config.validate()
        return config

    def validate(self) -> None:
        for f in ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
                  "num_attention_heads", "num_key_value_heads", "head_dim", "max_position_embeddings"):
            if int(getattr(self, f)) <= 0:
                raise ConfigError(f"config.json: '{f}' must be positive, got {getattr(self, f)}")
        if self.num_attention_heads % self.num_key_value_heads:
            raise ConfigError(
                f"config.json: num_attention_heads {self.num_attention_heads} is not a multiple of "
                f"num_key_value_heads {self.num_key_value_heads}")
        if self.head_dim % 2:
            raise ConfigError(f"config.json: head_dim {self.head_dim} must be even (rotate-half RoPE)")
        if not self.rms_norm_eps > 0:
            raise ConfigError(f"config.json: rms_norm_eps must be positive, got {self.rms_norm_eps}")
        if not self.rope_theta > 0:
            raise ConfigError(f"config.json: rope_theta must be positive, got {self.rope_theta}")
        if self.hidden_act != "silu":
            raise ConfigError(f"config.json: hidden_act '{self.hidden_act}' is not supported (only 'silu')")
        if self.attention_bias:
            raise ConfigError("config.json: attention_bias=true is not supported (Qwen3 has no linear biases)")
        if len(self.layer_types) != self.num_hidden_layers:
            raise ConfigError(
                f"config.json: layer_types has {len(self.layer_types)} entries for "
                f"{self.num_hidden_layers} layers")
        for t in self.layer_types:
            if t not in (FULL, SLIDING):
                raise ConfigError(f"config.json: unknown layer type '{t}'")
        if self.sliding_window is not None and self.sliding_window <= 0:
            raise ConfigError(f"config.json: sliding_window must be positive, got {self.sliding_window}")

    def to_dict(self) -> dict:
        out = {"architectures": [self.architecture], "model_type": "qwen3"}
        for f in fields(self):
            value = getattr(self, f.name)
            out[f.name] = list(value) if isinstance(value, tuple) else value
        out["use_sliding_window"] = self.sliding_window is not None
        out["rope_scaling"] = None
        return out

    # ------------------------------------------------------------------ the plan

    def plan(self) -> ModelPlan:
        eps = self.rms_norm_eps
        hidden, head_dim = self.hidden_size, self.head_dim
        position = PartSpec("rope", {"head_dim": head_dim, "rotary_dim": head_dim, "theta": self.rope_theta})
        layers = []
        for i, kind in enumerate(self.layer_types):
            prefix = f"model.layers.{i}"
            mixer = PartSpec(
                "attention",
                {
                    "hidden_size": hidden,
                    "n_heads": self.num_attention_heads,
                    "n_kv_heads": self.num_key_value_heads,
                    "head_dim": head_dim,
                    "scale": head_dim ** -0.5,
                    "window": self.sliding_window if kind == SLIDING else None,
                    "qk_norm_eps": eps,
                    "position": position,
                },
                {
                    "q_proj": f"{prefix}.self_attn.q_proj.weight",
                    "k_proj": f"{prefix}.self_attn.k_proj.weight",
                    "v_proj": f"{prefix}.self_attn.v_proj.weight",
                    "o_proj": f"{prefix}.self_attn.o_proj.weight",
                    "q_norm": f"{prefix}.self_attn.q_norm.weight",
                    "k_norm": f"{prefix}.self_attn.k_norm.weight",
                },
            )
            ffn = PartSpec(
                "swiglu",
                {"hidden_size": hidden, "intermediate_size": self.intermediate_size},
                {
                    "gate_proj": f"{prefix}.mlp.gate_proj.weight",
                    "up_proj": f"{prefix}.mlp.up_proj.weight",
                    "down_proj": f"{prefix}.mlp.down_proj.weight",
                },
            )
            layers.append(LayerSpec.of(
                "pre_norm",
                mixer=mixer,
                ffn=ffn,
                norm_mixer=PartSpec("rmsnorm", {"size": hidden, "eps": eps},
                                    {"weight": f"{prefix}.input_layernorm.weight"}),
                norm_ffn=PartSpec("rmsnorm", {"size": hidden, "eps": eps},
                                  {"weight": f"{prefix}.post_attention_layernorm.weight"}),
            ))
        embed_name = "model.embed_tokens.weight"
        return ModelPlan(
            hidden_size=hidden,
            vocab_size=self.vocab_size,
            embedding=PartSpec("embedding", {"vocab_size": self.vocab_size, "hidden_size": hidden},
                               {"weight": embed_name}),
            layers=tuple(layers),
            schedule=tuple(ScheduleEntry(layer=i, cache=i) for i in range(len(layers))),
            final_norm=PartSpec("rmsnorm", {"size": hidden, "eps": eps}, {"weight": "model.norm.weight"}),
            head=PartSpec("lm_head",
                          {"vocab_size": self.vocab_size, "hidden_size": hidden,
                           "tied": self.tie_word_embeddings},
                          # A tied head reads the embedding table; some writers store the head a
                          # second time under its own name, which the loader then compares.
                          {"weight": embed_name, "stored_copy": "lm_head.weight"} if self.tie_word_embeddings
                          else {"weight": "lm_head.weight"}),
            max_positions=self.max_position_embeddings,
            ignored_tensors=("*.rotary_emb.inv_freq",),
        )
