"""A plain, slow Gemma 2: whole sequences, no cache, one function per part.

This file rests on the reference's formulas only (nickheyer/kungfu; file:line cited at each
function).  The reference's own model code is Rust with crates.io dependencies and no Rust toolchain or
network exists where this was written, so it could not be compiled or imported for a golden
comparison.  Nothing here shares code with the engine under `kungfu_b200/`: tensors are read from a
dictionary by their file names and every step is ordinary torch arithmetic on the CPU, in float64 by
default so that it can serve as ground truth for both the 32-bit and the bfloat16 engine paths.
"""
from __future__ import annotations

import math

import torch


def embed(table: torch.Tensor, tokens: torch.Tensor, hidden: int, dtype) -> torch.Tensor:
    """x = E[token] * sqrt(hidden), the factor rounded to 32-bit first.
    crates/kf-layers/src/basic.rs:35-36, crates/kf-arch/src/archs/gemma2.rs:34."""
    scale = torch.tensor(math.sqrt(hidden), dtype=torch.float32).to(dtype)
    return table.to(dtype)[tokens] * scale


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """y = x / sqrt(mean(x^2) + eps) * (1 + w).
    crates/kf-backend-cuda/src/kernels/norm.cu:4-14 (the reference multiplies by the stored vector; Gemma 2
    safetensors store w and use 1 + w)."""
    inv = torch.rsqrt(x.pow(2).mean(dim=-1, keepdim=True) + eps)
    return x * inv * (1.0 + w.to(x.dtype))


def rope_angles(positions: torch.Tensor, head_dim: int, base: float, dtype) -> tuple[torch.Tensor, torch.Tensor]:
    """angle[p, i] = p * base^(-2i/d) for i < d/2.  crates/kf-backend-cpu/src/rope.rs:57-108,
    crates/kf-backend-cuda/src/exec.rs:1412-1426 (inverse frequencies held as 32-bit numbers)."""
    i = torch.arange(head_dim // 2, dtype=torch.float64)
    inv_freq = (base ** (-2.0 * i / head_dim)).to(torch.float32).to(dtype)
    ang = positions.to(dtype)[:, None] * inv_freq.to(positions.device)[None, :]
    return torch.cos(ang), torch.sin(ang)


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """x: [T, heads, d]; pairs (i, i + d/2): x'_i = x_i cos - x_{i+d/2} sin; x'_{i+d/2} = x_i sin + x_{i+d/2} cos.
    crates/kf-backend-cuda/src/kernels/rope.cu:16-37 (NeoX pairing, gemma2.rs:19)."""
    half = x.shape[-1] // 2
    a, b = x[..., :half], x[..., half:]
    c, s = cos[:, None, :], sin[:, None, :]
    return torch.cat([a * c - b * s, a * s + b * c], dim=-1)


def softcap(x: torch.Tensor, cap: float) -> torch.Tensor:
    """cap * tanh(x / cap); cap 0 leaves x.  crates/kf-backend-cuda/src/kernels/elementwise.cu:38-40."""
    return cap * torch.tanh(x / cap) if cap > 0 else x


def visible(n: int, window: int | None) -> torch.Tensor:
    """mask[p, j]: key j is seen from position p iff j <= p and (no window or p - j < window).
    crates/kf-backend-cpu/src/attention.rs:33-45."""
    p = torch.arange(n)[:, None]
    j = torch.arange(n)[None, :]
    m = j <= p
    if window is not None:
        m &= (p - j) < window
    return m


def rounded(x: torch.Tensor, to) -> torch.Tensor:
    """x as it is after being stored in element type `to` (None: unchanged).  The reference rounds activations to the
    weights' companion type before a product and keeps the cache in 16 bits (crates/kf-quant/src/lib.rs:154-175,
    crates/kf-backend-cpu/src/lib.rs:95-110); with `to=torch.bfloat16` this file rounds at the same places as an
    engine that computes in bfloat16: product inputs, and queries, keys and values as attention reads them."""
    return x if to is None else x.to(to).to(x.dtype)


def attention(x, wq, wk, wv, wo, *, n_heads, n_kv_heads, head_dim, scale, cap, window, base, rounding=None, probe=None):
    """Grouped-query attention over the whole sequence.  crates/kf-layers/src/attention.rs:118-150,211-283;
    scores, cap, mask and softmax crates/kf-backend-cpu/src/attention.rs:79-147; head h reads kv head
    h / (n_heads / n_kv_heads) (:79,92).  `probe`: a list that receives the scores before the cap (visible ones)."""
    T = x.shape[0]
    dt = x.dtype
    q = (x @ wq.to(dt).T).view(T, n_heads, head_dim)
    k = (x @ wk.to(dt).T).view(T, n_kv_heads, head_dim)
    v = (x @ wv.to(dt).T).view(T, n_kv_heads, head_dim)
    cos, sin = rope_angles(torch.arange(T, device=x.device), head_dim, base, dt)
    q, k = rounded(apply_rope(q, cos, sin), rounding), rounded(apply_rope(k, cos, sin), rounding)
    v = rounded(v, rounding)
    group = n_heads // n_kv_heads
    mask = visible(T, window).to(x.device)
    out = torch.empty(T, n_heads, head_dim, dtype=dt, device=x.device)
    for h in range(n_heads):
        kh, vh = k[:, h // group], v[:, h // group]
        raw = (q[:, h] @ kh.T) * scale
        if probe is not None:
            probe.append(raw[mask])
        s = softcap(raw, cap)
        s = s.masked_fill(~mask, float("-inf"))
        if rounding is None:
            out[:, h] = torch.softmax(s, dim=-1) @ vh
        else:
            # an engine that multiplies the softmax weights with the values on 16-bit tensor cores rounds the weights
            # e^(s - max) too (the sum that divides them stays exact); the reference does so as well
            # (crates/kf-backend-cuda/src/kernels/flash.cu:193-199)
            e = torch.exp(s - s.max(dim=-1, keepdim=True).values)
            out[:, h] = (rounded(e, rounding) @ vh) / e.sum(dim=-1, keepdim=True)
    return rounded(out.reshape(T, n_heads * head_dim), rounding) @ wo.to(dt).T


def gelu_tanh(x: torch.Tensor) -> torch.Tensor:
    """0.5 x (1 + tanh(sqrt(2/pi) (x + 0.044715 x^3))).  crates/kf-backend-cuda/src/kernels/common.cuh:95."""
    return 0.5 * x * (1.0 + torch.tanh(0.7978845608028654 * (x + 0.044715 * x.pow(3))))


def activation(name: str, x: torch.Tensor) -> torch.Tensor:
    if name in ("gelu_pytorch_tanh", "gelu_tanh"):
        return gelu_tanh(x)
    if name == "gelu":
        return 0.5 * x * (1.0 + torch.erf(x / math.sqrt(2.0)))
    if name == "silu":
        return x * torch.sigmoid(x)
    raise ValueError(name)


def feed_forward(x, w_gate, w_up, w_down, act: str, rounding=None) -> torch.Tensor:
    """y = (act(x Wgate^T) * (x Wup^T)) Wdown^T.  crates/kf-layers/src/ffn.rs:24-47."""
    dt = x.dtype
    return rounded(activation(act, x @ w_gate.to(dt).T) * (x @ w_up.to(dt).T), rounding) @ w_down.to(dt).T


def is_sliding(cfg: dict, layer: int) -> bool:
    """Even layers slide, odd layers see everything, unless `layer_types` says otherwise.
    crates/kf-arch/src/hparams.rs:541-554 with period 2 (gemma2.rs:23)."""
    types = cfg.get("layer_types")
    if types is not None:
        return types[layer] == "sliding_attention"
    return layer % 2 == 0


def forward(cfg: dict, tensors: dict, tokens, dtype=torch.float64, rounding=None, probe: dict | None = None,
            device="cpu") -> torch.Tensor:
    """Logits [T, vocab] for the whole token sequence.  `cfg` is the config.json dictionary, `tensors` maps
    file names to tensors.  Block arrangement: crates/kf-layers/src/basic.rs:241-253 and gemma2.rs:39-41:
      h = x + post_attn_norm(attn(input_norm(x)));  out = h + post_ffn_norm(ffn(pre_ffn_norm(h)))
    Head: final norm, tied output matrix, final cap (crates/kf-layers/src/model.rs:155-175).
    `rounding`: see `rounded`.  `probe`: a dictionary that receives 'scores' (per layer, the visible scores before the
    cap) and 'logits' (before the cap).  `device`: where the arithmetic runs (tensors are moved there as they are used)."""
    tokens = torch.as_tensor(tokens, dtype=torch.long, device=device)
    H = cfg["hidden_size"]
    eps = cfg["rms_norm_eps"]
    nh, nkv = cfg["num_attention_heads"], cfg.get("num_key_value_heads", cfg["num_attention_heads"])
    d = cfg.get("head_dim", H // nh)
    scale = 1.0 / math.sqrt(cfg.get("query_pre_attn_scalar", d))
    act = cfg.get("hidden_activation") or cfg.get("hidden_act") or "gelu_pytorch_tanh"

    def t(name):
        return tensors[name].to(device)
    x = embed(t("model.embed_tokens.weight"), tokens, H, dtype)
    for l in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{l}."
        n = rounded(rms_norm(x, t(p + "input_layernorm.weight"), eps), rounding)
        scores = [] if probe is not None else None
        a = attention(n, t(p + "self_attn.q_proj.weight"), t(p + "self_attn.k_proj.weight"),
                      t(p + "self_attn.v_proj.weight"), t(p + "self_attn.o_proj.weight"),
                      n_heads=nh, n_kv_heads=nkv, head_dim=d, scale=scale,
                      cap=cfg.get("attn_logit_softcapping", 50.0) or 0.0,
                      window=(cfg.get("sliding_window", 4096) or None) if is_sliding(cfg, l) else None,
                      base=cfg.get("rope_theta", 10000.0), rounding=rounding, probe=scores)
        if probe is not None:
            probe.setdefault("scores", []).append(torch.cat([s.reshape(-1) for s in scores]).cpu())
        x = x + rms_norm(a, t(p + "post_attention_layernorm.weight"), eps)
        n = rounded(rms_norm(x, t(p + "pre_feedforward_layernorm.weight"), eps), rounding)
        f = feed_forward(n, t(p + "mlp.gate_proj.weight"), t(p + "mlp.up_proj.weight"),
                         t(p + "mlp.down_proj.weight"), act, rounding)
        x = x + rms_norm(f, t(p + "post_feedforward_layernorm.weight"), eps)
    n = rounded(rms_norm(x, t("model.norm.weight"), eps), rounding)
    out = t("lm_head.weight") if "lm_head.weight" in tensors else t("model.embed_tokens.weight")
    logits = n @ out.to(dtype).T
    if probe is not None:
        probe["logits"] = logits.cpu()
    return softcap(logits, cfg.get("final_logit_softcapping", 30.0) or 0.0).cpu()


def greedy(cfg: dict, tensors: dict, prompt, n_new: int, dtype=torch.float64) -> list[int]:
    """Greedy continuation by recomputing the whole sequence each step; first maximum wins
    (crates/kf-engine/src/sampler.rs:219-227)."""
    ids = list(prompt)
    out = []
    for _ in range(n_new):
        nxt = int(torch.argmax(forward(cfg, tensors, ids, dtype)[-1]))
        out.append(nxt)
        ids.append(nxt)
    return out
