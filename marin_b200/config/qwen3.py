"""Configuration of the Qwen3 dense decoder (``Qwen3ForCausalLM``).

Keys, defaults and refusals follow the reference's parser
(crates/model/src/qwen3/config.rs:24-46 keys, :79-123 defaults, :159-196 validation,
:198-222 refused variants).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any, Dict, Optional

from .base import ConfigError, ModelConfig, eos_ids, optional, require


@dataclass
class Qwen3Config(ModelConfig):
    intermediate_size: int = 0
    num_hidden_layers: int = 0
    num_attention_heads: int = 0
    num_key_value_heads: int = 0
    head_dim: int = 0
    rms_norm_eps: float = 0.0
    rope_theta: float = 0.0
    tie_word_embeddings: bool = False
    eos_from_generation_config: bool = False

    ARCHITECTURE = "Qwen3ForCausalLM"
    MODEL_TYPE = "qwen3"

    @property
    def q_dim(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_dim(self) -> int:
        return self.num_key_value_heads * self.head_dim

    def parameter_count(self) -> int:
        """Weight count implied by the sizes (config.rs:138-157)."""
        h, i, d = self.hidden_size, self.intermediate_size, self.head_dim
        q, kv = self.q_dim, self.kv_dim
        per_layer = h * (q + 2 * kv + q) + 3 * h * i + 2 * h + 2 * d
        embeddings = self.vocab_size * h
        head = 0 if self.tie_word_embeddings else embeddings
        return per_layer * self.num_hidden_layers + embeddings + head + h

    @classmethod
    def from_dict(cls, raw: Dict[str, Any], generation: Optional[Dict[str, Any]] = None) -> "Qwen3Config":
        model_type = optional(raw, "model_type", str)
        archs = raw.get("architectures") or []
        if model_type is None and cls.ARCHITECTURE in archs:
            model_type = cls.MODEL_TYPE
        if model_type != cls.MODEL_TYPE:
            raise ConfigError(f"config.json: model_type `{model_type}` is not `{cls.MODEL_TYPE}`")
        _reject_unsupported(raw)
        rope_theta = optional(raw, "rope_theta", float)
        if rope_theta is None:
            params = raw.get("rope_parameters")
            if isinstance(params, dict):
                rope_theta = optional(params, "rope_theta", float)
        if rope_theta is None:
            raise ConfigError("config.json: `rope_theta` is missing")
        heads = require(raw, "num_attention_heads", int)
        kv_heads = optional(raw, "num_key_value_heads", int, heads)
        hidden = require(raw, "hidden_size", int)
        head_dim = optional(raw, "head_dim", int)
        if head_dim is None:
            head_dim = hidden // heads if heads > 0 else 0
        gen_eos = None
        if generation is not None and generation.get("eos_token_id") is not None:
            gen_eos = eos_ids(generation["eos_token_id"])
        cfg = cls(
            architecture=cls.ARCHITECTURE,
            model_type=cls.MODEL_TYPE,
            vocab_size=require(raw, "vocab_size", int),
            hidden_size=hidden,
            max_position_embeddings=require(raw, "max_position_embeddings", int),
            eos_token_ids=gen_eos if gen_eos is not None else eos_ids(raw.get("eos_token_id")),
            raw=dict(raw),
            intermediate_size=require(raw, "intermediate_size", int),
            num_hidden_layers=require(raw, "num_hidden_layers", int),
            num_attention_heads=heads,
            num_key_value_heads=kv_heads,
            head_dim=head_dim,
            rms_norm_eps=require(raw, "rms_norm_eps", float),
            rope_theta=rope_theta,
            tie_word_embeddings=bool(raw.get("tie_word_embeddings", False)),
            eos_from_generation_config=gen_eos is not None,
        )
        cfg.validate()
        return cfg

    def validate(self) -> None:
        positive = [
            ("hidden_size", self.hidden_size),
            ("intermediate_size", self.intermediate_size),
            ("num_hidden_layers", self.num_hidden_layers),
            ("num_attention_heads", self.num_attention_heads),
            ("num_key_value_heads", self.num_key_value_heads),
            ("head_dim", self.head_dim),
            ("vocab_size", self.vocab_size),
            ("max_position_embeddings", self.max_position_embeddings),
        ]
        for name, value in positive:
            if value <= 0:
                raise ConfigError(f"config.json: `{name}` must be above 0, got {value}")
        if self.num_attention_heads % self.num_key_value_heads != 0:
            raise ConfigError(
                f"config.json: {self.num_attention_heads} attention heads cannot be shared evenly by "
                f"{self.num_key_value_heads} key/value heads"
            )
        if self.head_dim % 2 != 0:
            raise ConfigError(f"config.json: head_dim {self.head_dim} must be even for rotary embeddings")
        if not math.isfinite(self.rms_norm_eps) or self.rms_norm_eps < 0:
            raise ConfigError("config.json: `rms_norm_eps` must be a finite number >= 0")
        if not math.isfinite(self.rope_theta) or self.rope_theta <= 0:
            raise ConfigError("config.json: `rope_theta` must be a finite number above 0")

    def to_json_dict(self) -> Dict[str, Any]:
        return {
            "architectures": [self.ARCHITECTURE],
            "model_type": self.MODEL_TYPE,
            "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "vocab_size": self.vocab_size,
            "max_position_embeddings": self.max_position_embeddings,
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "hidden_act": "silu",
            "tie_word_embeddings": self.tie_word_embeddings,
            "attention_bias": False,
            "use_sliding_window": False,
            "eos_token_id": self.eos_token_ids[0] if len(self.eos_token_ids) == 1 else (self.eos_token_ids or None),
        }


def _reject_unsupported(raw: Dict[str, Any]) -> None:
    if raw.get("attention_bias", False):
        raise ConfigError("config.json: unsupported variant: attention_bias=true")
    if raw.get("use_sliding_window", False):
        raise ConfigError("config.json: unsupported variant: sliding window attention")
    if raw.get("rope_scaling") is not None:
        raise ConfigError("config.json: unsupported variant: rope_scaling (long-context rope variants)")
    params = raw.get("rope_parameters")
    if isinstance(params, dict):
        kind = params.get("rope_type")
        if kind is not None and kind != "default":
            raise ConfigError(f"config.json: unsupported variant: rope type `{kind}`")
    act = raw.get("hidden_act")
    if act is not None and act != "silu":
        raise ConfigError(f"config.json: unsupported variant: activation `{act}` (only silu)")
