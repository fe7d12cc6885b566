"""LFM2 (`Lfm2ForCausalLM`): short-convolution and grouped-query-attention layers interleaved as
`layer_types` says, each followed by a SwiGLU feed-forward, RMSNorm before both
(reference arch `lfm2`, src/model.zig:29, layer binding src/model.zig:591-786).

Tensor names are the Hugging Face names of the architecture; the reference's own names are the
GGUF ones (src/model.zig:593-600, 632-636, 712-776): token_embd -> model.embed_tokens,
token_embd_norm -> model.embedding_norm (the final norm, src/model.zig:599-600),
blk.i.attn_norm -> operator_norm, blk.i.ffn_norm -> ffn_norm,
blk.i.shortconv.{in_proj,conv,out_proj} -> conv.{in_proj,conv,out_proj},
blk.i.attn_{q,k,v,output} -> self_attn.{q,k,v,out}_proj, attn_{q,k}_norm -> {q,k}_layernorm,
ffn_{gate,up,down} -> feed_forward.{w1,w3,w2}, output -> lm_head.
"""
from __future__ import annotations

from ..config.lfm2 import LAYER_CONV, LAYER_FULL, LAYER_WINDOW, Lfm2Config
from ..config.registry import register_architecture
from ..parts import GqaAttention, LMHead, PreNormBlock, RMSNorm, RotaryEncoding, ShortConv, SwiGLU, TokenEmbedding
from .model import Model


def build_lfm2(cfg: Lfm2Config) -> Model:
    D = cfg.hidden_size
    embedding = TokenEmbedding(cfg.vocab_size, D, "model.embed_tokens.weight")
    rope = RotaryEncoding(cfg.head_dim, cfg.rope_theta)          # one table for all layers, src/model.zig:808-819
    layers = []
    for i, kind in enumerate(cfg.layer_types):
        p = f"model.layers.{i}."
        if kind == LAYER_CONV:
            mixer = ShortConv(D, cfg.conv_L_cache, p + "conv.in_proj.weight", p + "conv.conv.weight",
                              p + "conv.out_proj.weight",
                              conv_bias_name=p + "conv.conv.bias" if cfg.conv_bias else None,
                              in_bias_name=p + "conv.in_proj.bias" if cfg.conv_bias else None,
                              out_bias_name=p + "conv.out_proj.bias" if cfg.conv_bias else None)
        elif kind in (LAYER_FULL, LAYER_WINDOW):
            a = p + "self_attn."
            mixer = GqaAttention(D, cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim,
                                 a + "q_proj.weight", a + "k_proj.weight", a + "v_proj.weight", a + "out_proj.weight",
                                 q_norm_name=a + "q_layernorm.weight", k_norm_name=a + "k_layernorm.weight",
                                 norm_eps=cfg.norm_eps, position=rope,
                                 window=cfg.sliding_window if kind == LAYER_WINDOW else 0)
        else:  # unreachable after Lfm2Config.validate
            raise ValueError(f"layer kind {kind!r}")
        ffn = SwiGLU(D, cfg.ffn_dim, p + "feed_forward.w1.weight", p + "feed_forward.w3.weight",
                     p + "feed_forward.w2.weight")
        layers.append(PreNormBlock(RMSNorm(D, cfg.norm_eps, p + "operator_norm.weight"), mixer,
                                   RMSNorm(D, cfg.norm_eps, p + "ffn_norm.weight"), ffn))
    final_norm = RMSNorm(D, cfg.norm_eps, "model.embedding_norm.weight")
    tied = cfg.tie_word_embeddings
    head = LMHead(cfg.vocab_size, D, None if tied else "lm_head.weight", embedding)
    return Model(cfg, embedding, layers, final_norm, head,
                 ignorable_weights=("lm_head.weight",) if tied else ())


register_architecture("Lfm2ForCausalLM", Lfm2Config, build_lfm2)
