"""Qwen3 dense (``Qwen3ForCausalLM``) as a list of parts.

Every layer: RMSNorm -> GQA attention with per-head RMSNorm of q and k and neox RoPE over the whole
head at ``rope_theta`` -> RMSNorm -> SwiGLU MLP; final RMSNorm; tied or untied head
(models/qwen3/src/model.rs:129-315,427-496; tensor names listed at model.rs:5-6).
"""
from __future__ import annotations

from ..config.model_config import Qwen3Config
from ..config.registry import register_architecture
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry


def qwen3_spec(cfg: Qwen3Config) -> ModelSpec:
    position = PartSpec("rope_neox", {"head_dim": cfg.head_dim, "theta": cfg.rope_theta,
                                      "max_positions": cfg.max_position_embeddings})
    layers = []
    for l in range(cfg.num_hidden_layers):
        layers.append(LayerSpec(
            prefix=f"model.layers.{l}.",
            block="prenorm_residual",
            mixer=PartSpec("gqa_attention", {
                "num_heads": cfg.num_attention_heads, "num_kv_heads": cfg.num_key_value_heads,
                "head_dim": cfg.head_dim, "qk_norm": True, "eps": cfg.rms_norm_eps, "position": position,
                "q_proj": "self_attn.q_proj.weight", "k_proj": "self_attn.k_proj.weight",
                "v_proj": "self_attn.v_proj.weight", "o_proj": "self_attn.o_proj.weight",
                "q_norm": "self_attn.q_norm.weight", "k_norm": "self_attn.k_norm.weight"}),
            mixer_norm=PartSpec("rmsnorm", {"size": cfg.hidden_size, "eps": cfg.rms_norm_eps,
                                            "weight": "input_layernorm.weight"}),
            feed_forward=PartSpec("swiglu", {
                "intermediate_size": cfg.intermediate_size, "gate_proj": "mlp.gate_proj.weight",
                "up_proj": "mlp.up_proj.weight", "down_proj": "mlp.down_proj.weight"}),
            feed_forward_norm=PartSpec("rmsnorm", {"size": cfg.hidden_size, "eps": cfg.rms_norm_eps,
                                                   "weight": "post_attention_layernorm.weight"}),
        ))
    return ModelSpec(
        architecture=cfg.architecture,
        hidden_size=cfg.hidden_size,
        vocab_size=cfg.vocab_size,
        max_positions=cfg.max_position_embeddings,
        embedding_tensor="model.embed_tokens.weight",
        layers=tuple(layers),
        schedule=tuple(ScheduleEntry(l) for l in range(cfg.num_hidden_layers)),
        final_norm=PartSpec("rmsnorm", {"size": cfg.hidden_size, "eps": cfg.rms_norm_eps,
                                        "weight": "model.norm.weight"}),
        lm_head_tensor="lm_head.weight",
        tie_word_embeddings=cfg.tie_word_embeddings,
        eos_token_ids=cfg.eos_token_ids,
    )


register_architecture("Qwen3ForCausalLM", Qwen3Config.from_dict, qwen3_spec)
