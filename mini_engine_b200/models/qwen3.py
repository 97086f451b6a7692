"""Qwen3 dense (``Qwen3ForCausalLM``) laid out as parts.

Every layer is: RMSNorm -> grouped-query attention with per-head q/k RMSNorm and RoPE ->
residual -> RMSNorm -> SwiGLU MLP -> residual; all layers attend to every earlier key; the
head is tied to the embedding when the configuration says so
(src/mini_engine/model.py:93-195 of YuvGev00/mini-engine).  Tensor names are the
checkpoint's own (the eleven per-layer names and three global ones).  Every number below
comes from the typed configuration.
"""

from __future__ import annotations

from mini_engine_b200.config.model_spec import LayerSpec, ModelSpec, OrderEntry, PartSpec
from mini_engine_b200.config.qwen3 import Qwen3Config
from mini_engine_b200.config.registry import Architecture, register_architecture


def qwen3_spec(cfg: Qwen3Config) -> ModelSpec:
    rope = PartSpec("rope", {"head_dim": cfg.head_dim, "theta": cfg.rope_theta})
    layers = []
    for index in range(cfg.num_hidden_layers):
        layers.append(
            LayerSpec(
                prefix=f"model.layers.{index}.",
                block="prenorm",
                mixer=PartSpec(
                    "gqa_attention",
                    {
                        "num_heads": cfg.num_attention_heads,
                        "kv_heads": cfg.num_key_value_heads,
                        "head_dim": cfg.head_dim,
                        "qk_norm_eps": cfg.rms_norm_eps,
                        "position_encoding": rope,
                        "window": None,
                        "names": {
                            "q": "self_attn.q_proj.weight",
                            "k": "self_attn.k_proj.weight",
                            "v": "self_attn.v_proj.weight",
                            "o": "self_attn.o_proj.weight",
                            "q_norm": "self_attn.q_norm.weight",
                            "k_norm": "self_attn.k_norm.weight",
                        },
                    },
                ),
                feed_forward=PartSpec(
                    "gated_mlp",
                    {
                        "intermediate_size": cfg.intermediate_size,
                        "activation": "silu",
                        "names": {
                            "gate": "mlp.gate_proj.weight",
                            "up": "mlp.up_proj.weight",
                            "down": "mlp.down_proj.weight",
                        },
                    },
                ),
                mixer_norm=PartSpec("rmsnorm", {"name": "input_layernorm.weight", "eps": cfg.rms_norm_eps}),
                feed_forward_norm=PartSpec(
                    "rmsnorm", {"name": "post_attention_layernorm.weight", "eps": cfg.rms_norm_eps}
                ),
            )
        )
    return ModelSpec(
        vocab_size=cfg.vocab_size,
        hidden_size=cfg.hidden_size,
        embedding=PartSpec("token_embedding", {"weight": "model.embed_tokens.weight"}),
        layers=tuple(layers),
        order=tuple(OrderEntry(i) for i in range(cfg.num_hidden_layers)),
        final_norm=PartSpec("rmsnorm", {"name": "model.norm.weight", "eps": cfg.rms_norm_eps}),
        head=PartSpec(
            "linear_head",
            {
                "weight": "lm_head.weight",
                "tied_to": "model.embed_tokens.weight" if cfg.tie_word_embeddings else None,
            },
        ),
    )


register_architecture(
    Architecture(
        name=Qwen3Config.architecture,
        read_config=Qwen3Config.from_folder,
        build_spec=qwen3_spec,
        config_type=Qwen3Config,
    )
)
