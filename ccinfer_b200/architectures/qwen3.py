"""Qwen3 dense (``Qwen3ForCausalLM``) put together from the parts.

Layer structure and tensor names as in 7QiC/ccInfer's only model
(src/model/qwen3/qwen3_model.cpp:141-426, src/model/qwen3/qwen3_weights.cpp:74-152):
pre-norm blocks of grouped-query attention with per-head q/k RMSNorm and
rotate-half RoPE, and a SwiGLU feed-forward; final norm; tied or untied head.
"""
from __future__ import annotations

from ..config.qwen3 import Qwen3Config
from ..engine.plan import ModelPlan, RunEntry
from ..parts import (GroupedQueryAttention, OutputHead, PreNormBlock, RMSNorm, RotaryHalf, SwiGLU,
                     TokenEmbedding)


def build_plan(cfg: Qwen3Config) -> ModelPlan:
    D = cfg.hidden_size
    layers = []
    for l in range(cfg.num_hidden_layers):
        p = f"model.layers.{l}."
        attn = GroupedQueryAttention(
            hidden=D, num_heads=cfg.num_attention_heads, num_kv_heads=cfg.num_key_value_heads,
            head_dim=cfg.head_dim, position=RotaryHalf(cfg.head_dim, cfg.rope_theta),
            names={"q": p + "self_attn.q_proj.weight", "k": p + "self_attn.k_proj.weight",
                   "v": p + "self_attn.v_proj.weight", "o": p + "self_attn.o_proj.weight",
                   "q_norm": p + "self_attn.q_norm.weight", "k_norm": p + "self_attn.k_norm.weight"},
            qk_norm_eps=cfg.rms_norm_eps, window=cfg.layer_window(l))
        ffn = SwiGLU(D, cfg.intermediate_size,
                     names={"gate": p + "mlp.gate_proj.weight", "up": p + "mlp.up_proj.weight",
                            "down": p + "mlp.down_proj.weight"})
        layers.append(PreNormBlock(RMSNorm(D, cfg.rms_norm_eps, p + "input_layernorm.weight"), attn,
                                   RMSNorm(D, cfg.rms_norm_eps, p + "post_attention_layernorm.weight"), ffn))
    head_name = "model.embed_tokens.weight" if cfg.tie_word_embeddings else "lm_head.weight"
    return ModelPlan(
        embedding=TokenEmbedding(cfg.vocab_size, D, "model.embed_tokens.weight"),
        layers=layers,
        order=[RunEntry(l) for l in range(cfg.num_hidden_layers)],
        final_norm=RMSNorm(D, cfg.rms_norm_eps, "model.norm.weight"),
        head=OutputHead(D, cfg.vocab_size, head_name),
        vocab_size=cfg.vocab_size,
        max_position=cfg.max_position_embeddings)
