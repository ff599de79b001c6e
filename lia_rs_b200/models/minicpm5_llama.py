"""MiniCPM5 Llama: a pre-norm Llama decoder (RMSNorm, grouped-query attention with rotary
positions, SwiGLU) with MiniCPM's three scalars.  This file only translates a `LlamaConfig` into
a `ModelSpec`; checkpoint names are the reference's (src/inference/huggingface/minicpm5.rs:31-68).
"""
from __future__ import annotations

from ..config import LlamaConfig, register_architecture
from ..parts import LayerSpec, PartSpec
from .decoder import ModelSpec


def build_llama(config: LlamaConfig) -> ModelSpec:
    norm = PartSpec("rmsnorm", {"hidden": config.hidden_size, "eps": config.rms_norm_eps})
    position = PartSpec("rotary", {"theta": config.rope_theta, "rotary_dim": config.head_dim})
    layers = []
    for i in range(config.num_hidden_layers):
        mixer = PartSpec("gqa_attention", {
            "hidden": config.hidden_size, "heads": config.num_attention_heads,
            "kv_heads": config.num_key_value_heads, "head_dim": config.head_dim,
            "window": config.window_of_layer(i), "position": position})
        feed_forward = PartSpec("swiglu", {"hidden": config.hidden_size,
                                           "intermediate": config.intermediate_size})
        layers.append(LayerSpec(mixer=mixer, feed_forward=feed_forward, norm=norm, arrangement="prenorm",
                                residual_scale=config.residual_scale))
    return ModelSpec(
        hidden_size=config.hidden_size, vocab_size=config.vocab_size,
        max_positions=config.max_position_embeddings, layers=layers, final_norm=norm,
        embedding_scale=config.embedding_scale, logit_scale=config.logit_scale,
        head_name=None if config.tie_word_embeddings else "lm_head.weight",
        eos_token_ids=tuple(config.eos_token_id))


register_architecture(("LlamaForCausalLM", "llama", "MiniCPMForCausalLM", "minicpm"), LlamaConfig, build_llama)
