"""The Llama dense decoder as a model description.

Layer structure and checkpoint names follow the reference's graph builder
(infernum-llama/src/graph_builder.rs:220-363 for the names, :451-507 for one
layer, :529-536 for the final norm, row selection and head):

    model.embed_tokens.weight
    model.layers.N.input_layernorm.weight
    model.layers.N.self_attn.{q,k,v,o}_proj.weight
    model.layers.N.post_attention_layernorm.weight
    model.layers.N.mlp.{gate,up,down}_proj.weight
    model.norm.weight
    lm_head.weight        (absent or ignored when tie_word_embeddings)

Every size and constant below comes from the typed configuration.
"""

from __future__ import annotations

from ..config.llama import LlamaConfig
from ..parts.base import LayerSpec, ModelSpec, PartSpec, ScheduleItem
from ..registry import register_architecture

EMBED = "model.embed_tokens.weight"


def build_llama_spec(cfg: LlamaConfig) -> ModelSpec:
    rope = {
        "kind": "rotary",
        "params": {
            "head_dim": cfg.head_dim,
            "theta": cfg.rope_theta,
            "scaling": cfg.rope_scaling.to_dict() if cfg.rope_scaling else None,
        },
    }
    layers = []
    for n in range(cfg.num_hidden_layers):
        p = f"model.layers.{n}."
        norm = lambda name: PartSpec("rmsnorm", {  # noqa: E731
            "hidden_size": cfg.hidden_size, "eps": cfg.rms_norm_eps, "weight": p + name})
        layers.append(LayerSpec(
            block="prenorm",
            name=p,
            parts={
                "norm1": norm("input_layernorm.weight"),
                "mixer": PartSpec("attention", {
                    "hidden_size": cfg.hidden_size,
                    "num_heads": cfg.num_attention_heads,
                    "num_kv_heads": cfg.num_key_value_heads,
                    "head_dim": cfg.head_dim,
                    "position": rope,
                    "window": 0,
                    "prefix": p + "self_attn.",
                }),
                "norm2": norm("post_attention_layernorm.weight"),
                "ffn": PartSpec("swiglu", {
                    "hidden_size": cfg.hidden_size,
                    "intermediate_size": cfg.intermediate_size,
                    "prefix": p + "mlp.",
                }),
            },
        ))
    head = {"vocab_size": cfg.vocab_size, "hidden_size": cfg.hidden_size,
            "weight": "lm_head.weight"}
    if cfg.tie_word_embeddings:
        head["tied_to"] = EMBED
    else:
        head["fallback"] = EMBED
    return ModelSpec(
        hidden_size=cfg.hidden_size,
        vocab_size=cfg.vocab_size,
        embedding=PartSpec("token_embedding", {
            "vocab_size": cfg.vocab_size, "hidden_size": cfg.hidden_size, "weight": EMBED}),
        layers=tuple(layers),
        schedule=tuple(ScheduleItem(n) for n in range(cfg.num_hidden_layers)),
        final_norm=PartSpec("rmsnorm", {
            "hidden_size": cfg.hidden_size, "eps": cfg.rms_norm_eps, "weight": "model.norm.weight"}),
        lm_head=PartSpec("linear_head", head),
        max_position=cfg.max_position_embeddings,
        eos_token_id=cfg.eos_token_id,
        bos_token_id=cfg.bos_token_id,
        ignorable=("lm_head.weight", "*.rotary_emb.inv_freq") if cfg.tie_word_embeddings
        else ("*.rotary_emb.inv_freq",),
    )


register_architecture("llama", LlamaConfig.from_dict, build_llama_spec)
