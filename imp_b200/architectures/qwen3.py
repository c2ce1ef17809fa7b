"""The Qwen3 dense decoder as a plan of parts.

Pre-norm blocks of grouped-query attention (per-head RMSNorm on q and k before
the rotary encoding, no bias, head size independent of the width) and a SwiGLU
feed-forward; final RMSNorm; output head tied to the embedding or its own
(the reference's forward pass for this family: src/graph/executor_forward.cu:
2701-3140; tensor names: src/model/safetensors_loader.cpp:366-401 and, for the
q/k norms that binder lacks, the GGUF twins at src/model/gguf_loader.cpp:387-388).
Everything here is data: the part kinds, their sizes from the configuration and
the checkpoint's tensor names.
"""
from __future__ import annotations

from ..config.model_config import Qwen3Config
from ..config.registry import register_architecture
from ..parts.plan import LayerSpec, ModelPlan, PartSpec


def qwen3_plan(cfg: Qwen3Config) -> ModelPlan:
    d = cfg.hidden_size
    rotary = PartSpec("rotary", {"head_dim": cfg.head_dim, "theta": cfg.rope_theta,
                                 "max_positions": cfg.max_position_embeddings})
    layers = []
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}."
        attn = PartSpec(
            "gqa_attention",
            {"hidden_size": d, "num_heads": cfg.num_attention_heads, "num_kv_heads": cfg.num_key_value_heads,
             "head_dim": cfg.head_dim, "window": cfg.window_of_layer(i), "qk_norm": True,
             "qk_norm_eps": cfg.rms_norm_eps, "position": rotary},
            {"q_proj": p + "self_attn.q_proj.weight", "k_proj": p + "self_attn.k_proj.weight",
             "v_proj": p + "self_attn.v_proj.weight", "o_proj": p + "self_attn.o_proj.weight",
             "q_norm": p + "self_attn.q_norm.weight", "k_norm": p + "self_attn.k_norm.weight"})
        ffn = PartSpec(
            "swiglu", {"hidden_size": d, "intermediate_size": cfg.intermediate_size},
            {"gate_proj": p + "mlp.gate_proj.weight", "up_proj": p + "mlp.up_proj.weight",
             "down_proj": p + "mlp.down_proj.weight"})
        norm1 = PartSpec("rmsnorm", {"size": d, "eps": cfg.rms_norm_eps}, {"weight": p + "input_layernorm.weight"})
        norm2 = PartSpec("rmsnorm", {"size": d, "eps": cfg.rms_norm_eps},
                         {"weight": p + "post_attention_layernorm.weight"})
        layers.append(LayerSpec(mixer=attn, feed_forward=ffn, mixer_norm=norm1, ffn_norm=norm2, block="prenorm"))
    head_name = "model.embed_tokens.weight" if cfg.tie_word_embeddings else "lm_head.weight"
    return ModelPlan(
        architecture=cfg.architecture,
        hidden_size=d,
        vocab_size=cfg.vocab_size,
        embedding=PartSpec("token_embedding", {"vocab_size": cfg.vocab_size, "hidden_size": d},
                           {"weight": "model.embed_tokens.weight"}),
        layers=layers,
        final_norm=PartSpec("rmsnorm", {"size": d, "eps": cfg.rms_norm_eps}, {"weight": "model.norm.weight"}),
        head=PartSpec("linear_head", {"vocab_size": cfg.vocab_size, "hidden_size": d}, {"weight": head_name}),
        max_positions=cfg.max_position_embeddings,
    )


register_architecture("Qwen3ForCausalLM", Qwen3Config, qwen3_plan, replace=True)
