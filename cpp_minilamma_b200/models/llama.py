"""The dense Llama decoder as data: `LlamaConfig` -> `ModelSpec`.

Every layer is a pre-norm block of grouped-query attention with rotary encoding and a
SwiGLU feed-forward (src/forward.cc:385-414), between a token embedding and a final
RMSNorm + lm_head (src/forward.cc:415-424).  Tensor names are those of a Llama model
folder; the reference's own names for the same tensors (src/load.cc:386-406) are
`token_embedding`, `layers.N.{attention_norm,wq,wk,wv,wo,ffn_norm,w_gate,w_up,w_down}`,
`final_norm`, `lm_head`.
"""
from __future__ import annotations

from ..config.base import register_architecture
from ..config.llama import LlamaConfig
from ..parts.base import LayerSpec, ModelSpec, PartSpec, ScheduleEntry


def build_llama_spec(config: LlamaConfig) -> ModelSpec:
    position = PartSpec("rotary", {
        "head_dim": config.head_dim,
        "theta": config.rope_theta,
        "scaling": config.rope_scaling.to_dict() if config.rope_scaling else None,
        "interleaved": config.rope_interleaved,
    })
    layers = []
    for i in range(config.num_hidden_layers):
        prefix = f"model.layers.{i}."
        layers.append(LayerSpec(
            block=PartSpec("pre_norm"),
            mixer=PartSpec("attention", {
                "n_heads": config.num_attention_heads,
                "n_kv_heads": config.num_key_value_heads,
                "head_dim": config.head_dim,
                "window": 0,
                "position": position,
                "qkv_bias": config.attention_bias,
                "o_bias": config.attention_bias,
                "names": {p: f"{prefix}self_attn.{p}_proj" for p in ("q", "k", "v", "o")},
            }),
            feed_forward=PartSpec("swiglu", {
                "intermediate": config.intermediate_size,
                "names": {p: f"{prefix}mlp.{p}_proj" for p in ("gate", "up", "down")},
            }),
            norms={
                "input": PartSpec("rms_norm", {"width": config.hidden_size, "eps": config.rms_norm_eps,
                                               "name": prefix + "input_layernorm.weight"}),
                "post_mixer": PartSpec("rms_norm", {"width": config.hidden_size, "eps": config.rms_norm_eps,
                                                    "name": prefix + "post_attention_layernorm.weight"}),
            }))
    embed_name = "model.embed_tokens.weight"
    return ModelSpec(
        hidden_size=config.hidden_size,
        vocab_size=config.vocab_size,
        max_positions=config.max_position_embeddings,
        embedding=PartSpec("token_embedding", {"vocab": config.vocab_size, "name": embed_name}),
        layers=layers,
        schedule=[ScheduleEntry(i) for i in range(config.num_hidden_layers)],
        final_norm=PartSpec("rms_norm", {"width": config.hidden_size, "eps": config.rms_norm_eps,
                                         "name": "model.norm.weight"}),
        lm_head=PartSpec("linear_head", {"vocab": config.vocab_size, "name": "lm_head.weight",
                                         "tied_to": embed_name if config.tie_word_embeddings else None}),
        stop_token_ids=list(config.eos_token_ids),
    )


register_architecture("LlamaForCausalLM", LlamaConfig, build_llama_spec)
