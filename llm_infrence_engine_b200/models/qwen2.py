"""The dense Qwen2 decoder, put together from parts (src/miniserve/model.py:168-237).

Every layer is a pre-norm block of grouped-query attention (QKV bias, rotary positions) and a
SwiGLU feed-forward between RMS norms; the output head shares the embedding's table when
``tie_word_embeddings`` is set. Tensor names are the checkpoint's own (model.py:3-5).
"""
from __future__ import annotations

from ..config.model_config import Qwen2Config
from ..parts import GatedMLP, OutputHead, PagedAttention, PreNormBlock, RMSNorm, RotaryEncoding, TokenEmbedding
from .registry import register_architecture
from .spec import ModelSpec, sequential


def build_qwen2(cfg: Qwen2Config) -> ModelSpec:
    rotary = RotaryEncoding(cfg.head_dim, cfg.rope_theta)
    embedding = TokenEmbedding(cfg.vocab_size, cfg.hidden_size, "model.embed_tokens.weight")
    layers = []
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}"
        layers.append(PreNormBlock(
            RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, f"{p}.input_layernorm.weight"),
            PagedAttention(cfg.hidden_size, cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim, rotary,
                           f"{p}.self_attn", bias=cfg.attention_bias, window=cfg.layer_window(i)),
            RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, f"{p}.post_attention_layernorm.weight"),
            GatedMLP(cfg.hidden_size, cfg.intermediate_size, f"{p}.mlp", cfg.hidden_act),
        ))
    return ModelSpec(
        config=cfg,
        embedding=embedding,
        layers=layers,
        schedule=sequential(cfg.num_hidden_layers),
        final_norm=RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, "model.norm.weight"),
        head=OutputHead(cfg.vocab_size, cfg.hidden_size, "lm_head.weight",
                        tied_to=embedding if cfg.tie_word_embeddings else None),
    )


register_architecture("Qwen2ForCausalLM", Qwen2Config, build_qwen2)
