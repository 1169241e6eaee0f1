"""The Llama dense decoder as data: its configuration turned into a ModelSpec.

Pre-RMSNorm blocks of grouped-query attention with rotary positions and a
SiLU-gated feed-forward, a final RMSNorm and an untied or tied output head
(src/model.cpp:80-234, tensor names src/model_config.cpp:78-97).  This file only
names parts and sizes; every formula lives in the parts.
"""
from __future__ import annotations

from .llama_config import LlamaConfig
from ..config.registry import Architecture, register_architecture
from ..parts.spec import LayerSpec, ModelSpec, OrderEntry, PartSpec


def build_llama_spec(config: LlamaConfig) -> ModelSpec:
    norm = PartSpec("rmsnorm", {"size": config.hidden_size, "eps": config.rms_norm_eps})
    mixer = PartSpec(
        "attention",
        {
            "hidden_size": config.hidden_size,
            "num_heads": config.num_attention_heads,
            "num_kv_heads": config.num_key_value_heads,
            "head_dim": config.head_dim,
            "window": 0,
            "scale": None,
            "position": PartSpec("rotary", {"rotary_dim": config.head_dim, "theta": config.rope_theta}),
        },
    )
    feed_forward = PartSpec(
        "gated_mlp",
        {"hidden_size": config.hidden_size, "intermediate_size": config.intermediate_size, "activation": config.hidden_act},
    )
    block = PartSpec(
        "pre_norm_residual",
        {
            "mixer_norm": norm, "mixer_norm_name": "input_layernorm",
            "mixer": mixer, "mixer_name": "self_attn",
            "feed_forward_norm": norm, "feed_forward_norm_name": "post_attention_layernorm",
            "feed_forward": feed_forward, "feed_forward_name": "mlp",
        },
    )
    layers = tuple(LayerSpec(f"model.layers.{i}", block) for i in range(config.num_hidden_layers))
    order = tuple(OrderEntry(layer=i, cache=i) for i in range(config.num_hidden_layers))
    spec = ModelSpec(
        architecture="LlamaForCausalLM",
        hidden_size=config.hidden_size,
        vocab_size=config.vocab_size,
        max_positions=config.max_position_embeddings,
        embedding=PartSpec("token_embedding", {"vocab_size": config.vocab_size, "hidden_size": config.hidden_size, "name": "model.embed_tokens"}),
        layers=layers,
        order=order,
        final_norm=PartSpec("rmsnorm", {"size": config.hidden_size, "eps": config.rms_norm_eps, "name": "model.norm"}),
        head=PartSpec(
            "linear_head",
            {
                "vocab_size": config.vocab_size, "hidden_size": config.hidden_size, "name": "lm_head",
                "tied_to": "model.embed_tokens" if config.tie_word_embeddings else None,
            },
        ),
    )
    spec.validate()
    return spec


LLAMA = Architecture(name="LlamaForCausalLM", config_class=LlamaConfig, build_spec=build_llama_spec, model_types=("llama",))
register_architecture(LLAMA, replace=True)
