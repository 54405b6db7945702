"""Qwen3 dense decoder as data: every layer is a pre-norm block of grouped-query attention
(per-head q/k RMSNorm, rotary positions) and a SwiGLU feed-forward
(crates/model/src/qwen3/layer.rs:39-105; tensor names crates/model/src/qwen3/weights.rs:103-130).
"""
from __future__ import annotations

from ..config.qwen3 import Qwen3Config
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry
from .registry import register_architecture


def build_spec(cfg: Qwen3Config) -> ModelSpec:
    norm = PartSpec("rmsnorm", {"dim": cfg.hidden_size, "eps": cfg.rms_norm_eps})
    layers = []
    for n in range(cfg.num_hidden_layers):
        mixer = PartSpec("gqa_attention", {
            "hidden": cfg.hidden_size,
            "heads": cfg.num_attention_heads,
            "kv_heads": cfg.num_key_value_heads,
            "head_dim": cfg.head_dim,
            "qk_norm": True,
            "norm_eps": cfg.rms_norm_eps,
            "window": None,
            "position": PartSpec("rope", {"head_dim": cfg.head_dim, "theta": cfg.rope_theta}),
        })
        ffn = PartSpec("swiglu", {"hidden": cfg.hidden_size, "intermediate": cfg.intermediate_size})
        layers.append(LayerSpec(
            block="prenorm", norm=norm, mixer=mixer, feedforward=ffn, prefix=f"model.layers.{n}",
            names={"norm1": "input_layernorm", "mixer": "self_attn",
                   "norm2": "post_attention_layernorm", "feedforward": "mlp"},
        ))
    return ModelSpec(
        hidden_size=cfg.hidden_size,
        vocab_size=cfg.vocab_size,
        embedding=PartSpec("token_table", {"vocab": cfg.vocab_size, "hidden": cfg.hidden_size,
                                           "name": "model.embed_tokens"}),
        final_norm=PartSpec("rmsnorm", {"dim": cfg.hidden_size, "eps": cfg.rms_norm_eps, "name": "model.norm"}),
        head=PartSpec("linear", {"vocab": cfg.vocab_size, "hidden": cfg.hidden_size, "name": "lm_head",
                                 "tied": cfg.tie_word_embeddings}),
        layers=layers,
        schedule=[ScheduleEntry(n) for n in range(cfg.num_hidden_layers)],
        ignorable=("lm_head.weight",) if cfg.tie_word_embeddings else (),
    )


register_architecture(Qwen3Config.ARCHITECTURE, Qwen3Config.MODEL_TYPE, Qwen3Config, build_spec)
