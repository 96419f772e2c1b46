"""Gemma 2 put together from parts.

Composition (reference: crates/kf-arch/src/archs/gemma2.rs:32-46): embedding scaled by
sqrt(width); per layer a sandwich block of (1+w) RMS norms around grouped-query attention
(rotary positions, softcapped scores, a sliding window on the layers the configuration
marks) and a gated GELU feed-forward; final (1+w) RMS norm, output matrix tied to the
embedding unless the file carries `lm_head.weight`, softcapped logits.
Tensor names are the ones Gemma 2 safetensors files use.
"""
from __future__ import annotations

import torch

from ..config.gemma2 import Gemma2Config
from ..parts import (DecoderModel, Embedding, GatedFfn, LmHead, PagedAttention, RmsNorm, Rope, SandwichBlock)
from ..weights.store import TensorSpec, WeightStore

NORM_STD = 0.1
MATRIX_STD = 0.02


def tensor_specs(cfg: Gemma2Config) -> list[TensorSpec]:
    """Every tensor a Gemma 2 file holds for `cfg`, with the spread random weights are drawn with."""
    H, I = cfg.hidden_size, cfg.intermediate_size
    specs = [TensorSpec("model.embed_tokens.weight", (cfg.vocab_size, H), MATRIX_STD)]
    for l in range(cfg.num_hidden_layers):
        p = f"model.layers.{l}."
        specs += [
            TensorSpec(p + "input_layernorm.weight", (H,), NORM_STD, "norm"),
            TensorSpec(p + "self_attn.q_proj.weight", (cfg.q_size, H), MATRIX_STD),
            TensorSpec(p + "self_attn.k_proj.weight", (cfg.kv_size, H), MATRIX_STD),
            TensorSpec(p + "self_attn.v_proj.weight", (cfg.kv_size, H), MATRIX_STD),
            TensorSpec(p + "self_attn.o_proj.weight", (H, cfg.q_size), MATRIX_STD),
            TensorSpec(p + "post_attention_layernorm.weight", (H,), NORM_STD, "norm"),
            TensorSpec(p + "pre_feedforward_layernorm.weight", (H,), NORM_STD, "norm"),
            TensorSpec(p + "mlp.gate_proj.weight", (I, H), MATRIX_STD),
            TensorSpec(p + "mlp.up_proj.weight", (I, H), MATRIX_STD),
            TensorSpec(p + "mlp.down_proj.weight", (H, I), MATRIX_STD),
            TensorSpec(p + "post_feedforward_layernorm.weight", (H,), NORM_STD, "norm"),
        ]
    specs.append(TensorSpec("model.norm.weight", (H,), NORM_STD, "norm"))
    if not cfg.tie_word_embeddings:
        specs.append(TensorSpec("lm_head.weight", (cfg.vocab_size, H), MATRIX_STD))
    return specs


def _stack(parts: list[torch.Tensor]) -> torch.Tensor:
    if any(p.numel() == 0 for p in parts) or len({p.dtype for p in parts}) != 1:
        return torch.empty(0)                       # a fault already recorded by the store
    return torch.cat(parts, dim=0).contiguous()


def build(cfg: Gemma2Config, w: WeightStore) -> DecoderModel:
    H, I = cfg.hidden_size, cfg.intermediate_size
    table = w.take("model.embed_tokens.weight", (cfg.vocab_size, H))
    embedding = Embedding(table, scale=cfg.embedding_scale)
    rope = Rope(cfg.head_dim, cfg.rope_theta, w.device)

    def rms(name: str) -> RmsNorm:
        return RmsNorm(w.take(name, (H,)), cfg.rms_norm_eps, plus_one=True)

    layers = []
    for l in range(cfg.num_hidden_layers):
        p = f"model.layers.{l}."
        wqkv = _stack([w.take(p + "self_attn.q_proj.weight", (cfg.q_size, H)),
                       w.take(p + "self_attn.k_proj.weight", (cfg.kv_size, H)),
                       w.take(p + "self_attn.v_proj.weight", (cfg.kv_size, H))])
        wo = w.take(p + "self_attn.o_proj.weight", (H, cfg.q_size))
        w.release(p + "self_attn.q_proj.weight", p + "self_attn.k_proj.weight", p + "self_attn.v_proj.weight")
        w_gate_up = _stack([w.take(p + "mlp.gate_proj.weight", (I, H)), w.take(p + "mlp.up_proj.weight", (I, H))])
        w_down = w.take(p + "mlp.down_proj.weight", (H, I))
        w.release(p + "mlp.gate_proj.weight", p + "mlp.up_proj.weight")
        norms = [rms(p + n) for n in ("input_layernorm.weight", "post_attention_layernorm.weight",
                                      "pre_feedforward_layernorm.weight", "post_feedforward_layernorm.weight")]
        if w.faulty:                                # keep claiming tensors so the error lists everything; build nothing
            continue
        mixer = PagedAttention(wqkv, wo, n_heads=cfg.num_attention_heads, n_kv_heads=cfg.num_key_value_heads,
                               head_dim=cfg.head_dim, scale=cfg.attention_scale,
                               softcap=cfg.attn_logit_softcapping, window=cfg.window_of(l), position=rope)
        ffn = GatedFfn(w_gate_up, w_down, cfg.activation)
        layers.append(SandwichBlock(norms[0], mixer, norms[1], norms[2], ffn, norms[3]))
    final_norm = rms("model.norm.weight")
    out = w.take_optional("lm_head.weight", (cfg.vocab_size, H))
    if out is None:
        if not cfg.tie_word_embeddings:
            w.take("lm_head.weight", (cfg.vocab_size, H))     # records it as missing
        out = table
    w.finish()
    head = LmHead(final_norm, out, softcap=cfg.final_logit_softcapping)
    return DecoderModel(embedding, layers, head, name=cfg.architecture)
