"""The Llama 3 dense decoder as a plan of parts.

What the reference runs for `model_type == "llama"`
(crates/model-runtime/src/execute.rs:3-249 with Mixer::Attention{qn:None,kn:None}
and FeedForward::Dense; tensor names crates/model-format/src/mlx/names.rs:9-57):
every layer is pre-norm attention with rotary positions followed by a
SiLU-gated feed-forward, all layers alike, run once each in order, each with a
cache entry of its own.
"""
from __future__ import annotations

from ..config.llama import LlamaConfig
from ..parts.base import LayerSpec, ModelPlan, PartSpec, ScheduleEntry
from ..registry import register_architecture


def llama_plan(config: LlamaConfig) -> ModelPlan:
    scaling = config.rope_scaling
    position = PartSpec("rope", dict(
        head_dim=config.head_dim, rotary_dim=config.rotary_dim, theta=config.rope_theta,
        scaling=scaling.kind, factor=scaling.factor, low_freq_factor=scaling.low_freq_factor,
        high_freq_factor=scaling.high_freq_factor,
        original_max_position_embeddings=scaling.original_max_position_embeddings,
        adjacent_pairs=config.rope_adjacent_pairs))
    layers = []
    for i in range(config.num_hidden_layers):
        p = f"model.layers.{i}."
        norm = dict(size=config.hidden_size, eps=config.rms_norm_eps)
        layers.append(LayerSpec(
            block="pre_norm",
            mixer=PartSpec("attention", dict(
                hidden_size=config.hidden_size, num_heads=config.num_attention_heads,
                num_kv_heads=config.num_key_value_heads, head_dim=config.head_dim,
                position=position, window=None), prefix=p + "self_attn."),
            feed_forward=PartSpec("gated_mlp", dict(
                hidden_size=config.hidden_size, intermediate_size=config.intermediate_size,
                activation="silu"), prefix=p + "mlp."),
            mixer_norm=PartSpec("rms_norm", norm, prefix=p + "input_layernorm."),
            feed_forward_norm=PartSpec("rms_norm", norm, prefix=p + "post_attention_layernorm."),
        ))
    tied = config.tie_word_embeddings
    return ModelPlan(
        hidden_size=config.hidden_size, vocab_size=config.vocab_size,
        max_positions=config.max_position_embeddings,
        embedding_name="model.embed_tokens.weight",
        layers=tuple(layers),
        schedule=tuple(ScheduleEntry(layer=i, cache=i) for i in range(config.num_hidden_layers)),
        final_norm=PartSpec("rms_norm", dict(size=config.hidden_size, eps=config.rms_norm_eps),
                            prefix="model.norm."),
        head_name=None if tied else "lm_head.weight",
        # explicit tying ignores a saved head (crates/model-format/src/mlx/mod.rs:44-48)
        ignored_names=("lm_head.weight",) if tied else (),
        stop_token_ids=tuple(config.eos_token_ids),
    )


register_architecture("LlamaForCausalLM", LlamaConfig, llama_plan, model_types=("llama",))
