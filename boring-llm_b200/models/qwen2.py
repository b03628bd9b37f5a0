"""The dense Qwen2 decoder as a list of parts, and its checkpoint tensor names.

Layer shape follows the reference's plain layer for GGUF arch `qwen2` (src/model.br:1297-1358):
pre-norm RMSNorm, grouped-query attention with bias on q/k/v only, NEOX rotary positions
(`rope_style_for_arch`, src/model.br:328-330), SwiGLU without biases, sequential residuals, a final
RMSNorm, and an output head that is the embedding when tied (src/model.br:686-690).
Checkpoint names are the public ones of this architecture's safetensors files; the reference's GGUF
names (src/model.br:614-690) are given beside them.
"""
from __future__ import annotations

from ..config import Qwen2Config, register_architecture
from ..parts import (DecoderModel, Embedding, GQAAttention, OutputHead, PreNormBlock, RMSNorm,
                     RotaryTable, SwiGLU)


def build_qwen2(cfg: Qwen2Config) -> DecoderModel:
    d, H, KV, dh = cfg.hidden_size, cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
    embedding = Embedding(cfg.vocab_size, d, {"table": "model.embed_tokens.weight"})      # token_embd.weight
    blocks = []
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}."
        window = cfg.layer_windows[i] if cfg.layer_windows else 0
        mixer = GQAAttention(
            d, H, KV, dh, RotaryTable(dh, cfg.rope_theta),
            {"wq": p + "self_attn.q_proj.weight", "bq": p + "self_attn.q_proj.bias",        # blk.i.attn_q.*
             "wk": p + "self_attn.k_proj.weight", "bk": p + "self_attn.k_proj.bias",        # blk.i.attn_k.*
             "wv": p + "self_attn.v_proj.weight", "bv": p + "self_attn.v_proj.bias",        # blk.i.attn_v.*
             "wo": p + "self_attn.o_proj.weight"},                                          # blk.i.attn_output.weight
            qkv_bias=cfg.attention_bias, window=window)
        ffn = SwiGLU(d, cfg.intermediate_size,
                     {"w_gate": p + "mlp.gate_proj.weight", "w_up": p + "mlp.up_proj.weight",   # blk.i.ffn_gate / ffn_up
                      "w_down": p + "mlp.down_proj.weight"})                                   # blk.i.ffn_down
        blocks.append(PreNormBlock(
            RMSNorm(d, cfg.rms_norm_eps, {"weight": p + "input_layernorm.weight"}),             # blk.i.attn_norm
            mixer,
            RMSNorm(d, cfg.rms_norm_eps, {"weight": p + "post_attention_layernorm.weight"}),    # blk.i.ffn_norm
            ffn))
    final_norm = RMSNorm(d, cfg.rms_norm_eps, {"weight": "model.norm.weight"})                  # output_norm.weight
    if cfg.tie_word_embeddings:
        head = OutputHead(cfg.vocab_size, d, {}, tied_to=embedding)
        ignorable = ("lm_head.weight",)       # some files store the shared matrix a second time
    else:
        head = OutputHead(cfg.vocab_size, d, {"weight": "lm_head.weight"})                      # output.weight
        ignorable = ()
    return DecoderModel(embedding, blocks, final_norm, head, ignorable_tensors=ignorable)


register_architecture(Qwen2Config.ARCHITECTURES + Qwen2Config.MODEL_TYPES, Qwen2Config, build_qwen2)
