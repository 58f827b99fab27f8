"""Qwen3 dense (`Qwen3ForCausalLM`) as a ModelSpec.

Per layer: pre-norm block; grouped-query attention with per-head RMSNorm of q and k before
rotary encoding over the full head; dense SwiGLU; RMSNorm everywhere with one eps; no biases;
head tied to the embedding or not (atomserve/model.py:292-385). Tensor names are the
checkpoint's (atomserve/loader.py:108-128). Layers from `max_window_layers` on attend through
a sliding window when the configuration enables one.
"""

from __future__ import annotations

from atomserve_b200.config.model_config import Qwen3Config
from atomserve_b200.config.registry import register_architecture
from atomserve_b200.parts.spec import LayerCall, LayerSpec, ModelSpec, PartSpec


def build_spec(c: Qwen3Config) -> ModelSpec:
    layers = []
    for i in range(c.num_hidden_layers):
        p = f"model.layers.{i}."
        layers.append(
            LayerSpec(
                block="pre_norm",
                mixer=PartSpec(
                    "gqa_attention",
                    dict(
                        num_heads=c.num_attention_heads,
                        num_kv_heads=c.num_key_value_heads,
                        head_dim=c.head_dim,
                        qk_norm_eps=c.rms_norm_eps,
                        position=PartSpec("rotary", dict(head_dim=c.head_dim, theta=c.rope_theta)),
                        window=c.window_of_layer(i),
                    ),
                    p + "self_attn.",
                ),
                feed_forward=PartSpec("swiglu", dict(intermediate_size=c.intermediate_size), p + "mlp."),
                mixer_norm=PartSpec("rms_norm", dict(eps=c.rms_norm_eps), p + "input_layernorm."),
                feed_forward_norm=PartSpec("rms_norm", dict(eps=c.rms_norm_eps), p + "post_attention_layernorm."),
            )
        )
    return ModelSpec(
        hidden_size=c.hidden_size,
        vocab_size=c.vocab_size,
        max_positions=c.max_position_embeddings,
        embedding=PartSpec("token_embedding", dict(vocab_size=c.vocab_size), "model.embed_tokens."),
        layers=tuple(layers),
        schedule=tuple(LayerCall(i) for i in range(c.num_hidden_layers)),
        final_norm=PartSpec("rms_norm", dict(eps=c.rms_norm_eps), "model.norm."),
        head=PartSpec("lm_head", dict(vocab_size=c.vocab_size, tied=c.tie_word_embeddings), "lm_head."),
        # a tied checkpoint may still ship a copy of the head; the configuration decides
        ignored_tensors=("lm_head.weight",) if c.tie_word_embeddings else (),
    )


register_architecture(Qwen3Config.architecture, Qwen3Config, build_spec)
