"""Llama 3 dense, assembled from parts (tamnd/fastmlx compute/models/llama.go).

Tensor names are the checkpoint's (llama.go:164-201).  The builder chooses each layer's
parts from the configuration, layer by layer; for this architecture every layer gets the
same kinds, but nothing below depends on that.
"""
from __future__ import annotations

from .. import registry
from ..config.llama import LlamaConfig
from ..parts import (Embedding, GQAAttention, LMHead, Model, PreNormBlock, RMSNorm, RotaryEmbedding, Run,
                     SwiGLU)


def build_llama(cfg: LlamaConfig) -> Model:
    d = cfg.hidden_size
    embed = Embedding(cfg.vocab_size, d, "model.embed_tokens")
    layers = []
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}"
        rope = RotaryEmbedding(cfg.head_dim, cfg.rope_theta, cfg.rope_scaling, cfg.rope_traditional)
        mixer = GQAAttention(d, cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim, rope,
                             f"{p}.self_attn", bias=cfg.attention_bias, scale=cfg.scale)
        ffn = SwiGLU(d, cfg.intermediate_size, f"{p}.mlp", bias=cfg.mlp_bias)
        layers.append(PreNormBlock(mixer, ffn,
                                   RMSNorm(d, cfg.rms_norm_eps, f"{p}.input_layernorm"),
                                   RMSNorm(d, cfg.rms_norm_eps, f"{p}.post_attention_layernorm")))
    head = LMHead(cfg.vocab_size, d, None, tied=embed) if cfg.tie_word_embeddings \
        else LMHead(cfg.vocab_size, d, "lm_head")
    drop = ["self_attn.rotary_emb.inv_freq"] + (["lm_head.weight"] if cfg.tie_word_embeddings else [])
    return Model(embed, layers, RMSNorm(d, cfg.rms_norm_eps, "model.norm"), head,
                 schedule=[Run(i) for i in range(len(layers))], drop=drop,
                 vocab_size=cfg.vocab_size, max_positions=cfg.max_position_embeddings,
                 eos_token_ids=cfg.eos_token_ids)


registry.register(["llama", "LlamaForCausalLM"], LlamaConfig.from_dict, build_llama, replace=True)
