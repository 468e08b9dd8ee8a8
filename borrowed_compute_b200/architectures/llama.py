"""The Llama dense decoder as a layout of parts.

Every layer is the same pre-norm block of grouped-query attention with rotary positions
and a SwiGLU feed-forward, and the layers run once each in order
(crates/bc-infer/src/model.rs:1-15, 320-346).  Tensor names are those of published
safetensors checkpoints; shapes are [out, in] as in the reference (model.rs:184-201).
"""

from __future__ import annotations

from ..config.llama import LlamaConfig
from ..parts.base import LayerSpec, ModelSpec, PartSpec, RunSpec
from .registry import register_architecture


def llama_model_spec(cfg: LlamaConfig) -> ModelSpec:
    position = {
        "kind": "rotary",
        "head_dim": cfg.head_dim,
        "theta": cfg.rope_theta,
        "pairing": cfg.rope_pairing,
        "scaling": None if cfg.rope_scaling is None else cfg.rope_scaling.to_dict(),
        "max_positions": cfg.max_position_embeddings,
    }
    layers = []
    for l in range(cfg.num_hidden_layers):
        p = f"model.layers.{l}."
        layers.append(LayerSpec(
            "prenorm",
            norm1=PartSpec("rmsnorm", {"size": cfg.hidden_size, "eps": cfg.rms_norm_eps}, p + "input_layernorm."),
            mixer=PartSpec("gqa_attention", {
                "hidden_size": cfg.hidden_size, "heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads,
                "head_dim": cfg.head_dim, "position": position,
            }, p + "self_attn."),
            norm2=PartSpec("rmsnorm", {"size": cfg.hidden_size, "eps": cfg.rms_norm_eps}, p + "post_attention_layernorm."),
            feed_forward=PartSpec("swiglu", {"hidden_size": cfg.hidden_size, "intermediate_size": cfg.intermediate_size}, p + "mlp."),
        ))
    return ModelSpec(
        hidden_size=cfg.hidden_size,
        vocab_size=cfg.vocab_size,
        max_positions=cfg.max_position_embeddings,
        embedding=PartSpec("token_embedding", {"vocab_size": cfg.vocab_size, "hidden_size": cfg.hidden_size}, "model.embed_tokens."),
        layers=tuple(layers),
        schedule=tuple(RunSpec(l) for l in range(cfg.num_hidden_layers)),
        final_norm=PartSpec("rmsnorm", {"size": cfg.hidden_size, "eps": cfg.rms_norm_eps}, "model.norm."),
        head=PartSpec("linear_head", {"vocab_size": cfg.vocab_size, "hidden_size": cfg.hidden_size,
                                      "tied": cfg.tie_word_embeddings}, "lm_head."),
        stop_ids=tuple(cfg.eos_token_ids),
    )


register_architecture("LlamaForCausalLM", LlamaConfig.from_dict, llama_model_spec)
