"""CPU restatement (numpy, f32) of one decode step of the reference's Qwen3 decoder, for the
parity tests of the device decode step. Test infrastructure: nothing in the product imports it.

Follows, in the reference tree:
  crates/nn-qwen3/src/layers.rs:40-47      SwiGLU MLP: down(silu(gate(x)) * up(x))
  crates/nn-qwen3/src/layers.rs:94-167     attention: q/k/v, per-head QK-norm, half-split RoPE,
                                           cache append, repeat_kv, sdpa with scale 1/sqrt(head_dim), o
  crates/nn-qwen3/src/layers.rs:205-226    pre-norm residual layer
  crates/nn-core/src/layers/rms_norm.rs:87-100           x / sqrt(mean(x^2) + eps) * w
  crates/nn-core/src/layers/attention/rope.rs:78-106     inv_freq in f32, angle = (pos * inv_freq in f64) -> f32
  crates/nn-core/src/layers/attention/rope_half_split.rs:98-134   y1 = x1 cos - x2 sin, y2 = x1 sin + x2 cos
  crates/nn-core/src/layers/attention/sdpa.rs:59-71      softmax(q k^T * scale) v
  crates/nn-core/src/dyn_tensor/ops/math.rs:140          silu(x) = x / (1 + exp(-x))
  crates/nn-core/src/layers/generation/autoregressive_sampling.rs:14-21   argmax, last of equal maxima
Weights are given dequantized (f32 [n, k]); the quantized decode itself is pinned elsewhere.

`act_bf16=True` rounds the four vectors per layer that feed a product (the normed hidden state
twice, the attention output, silu(gate) * up) and the final normed state to bf16 (round to nearest
even) before the product, and leaves everything else in f32: the rounding points of a decoder
whose products take bf16 activations.
"""
from __future__ import annotations

import numpy as np

F = np.float32


def bf16_round(x):
    """f32 -> nearest bf16 (ties to even) -> f32."""
    u = np.ascontiguousarray(x, dtype=F).view(np.uint32)
    r = ((u >> np.uint32(16)) & np.uint32(1)) + np.uint32(0x7FFF)
    return ((u + r) & np.uint32(0xFFFF0000)).view(F)


def rms_norm(x, w, eps):
    x = x.astype(F)
    ms = np.mean(x * x, axis=-1, keepdims=True, dtype=F)
    return (x / np.sqrt(ms + F(eps))) * w


def rope_tables(head_dim: int, max_seq: int, theta: float):
    half = head_dim // 2
    inv = np.array([1.0 / theta ** (2 * i / head_dim) for i in range(half)], dtype=np.float64).astype(F)
    ang = (np.arange(max_seq, dtype=np.float64)[:, None] * inv.astype(np.float64)[None, :]).astype(F)
    return np.cos(ang).astype(F), np.sin(ang).astype(F)


def rotate(x, cos, sin):
    half = x.shape[-1] // 2
    x1, x2 = x[..., :half], x[..., half:]
    return np.concatenate([x1 * cos - x2 * sin, x1 * sin + x2 * cos], axis=-1).astype(F)


def argmax_last(v) -> int:
    v = np.asarray(v)
    return int(len(v) - 1 - np.argmax(v[::-1]))


def step(model: dict, token: int, pos: int, kcache: np.ndarray, vcache: np.ndarray, act_bf16: bool = False):
    """model: cfg (dict), embed [vocab, hidden] f32, layers (list of dicts with q k v o gate up down
    in_norm post_norm q_norm k_norm), final_norm, lm_head. kcache / vcache: [layers, kv_heads,
    max_seq, head_dim] f32, updated in place at `pos`. Returns (logits f32 [vocab], next token)."""
    c = model["cfg"]
    nh, nkv, hd, eps = c["n_heads"], c["n_kv_heads"], c["head_dim"], c["rms_eps"]
    cos, sin = model["rope"]
    h = model["embed"][token].astype(F)
    scale = F(1.0 / np.sqrt(float(hd)))
    act = bf16_round if act_bf16 else (lambda a: a)
    for li, L in enumerate(model["layers"]):
        x = act(rms_norm(h, L["in_norm"], eps))
        q = (L["q"] @ x).reshape(nh, hd)
        k = (L["k"] @ x).reshape(nkv, hd)
        v = (L["v"] @ x).reshape(nkv, hd)
        q = rotate(rms_norm(q, L["q_norm"], eps), cos[pos], sin[pos])
        k = rotate(rms_norm(k, L["k_norm"], eps), cos[pos], sin[pos])
        kcache[li, :, pos, :] = k
        vcache[li, :, pos, :] = v
        out = np.empty((nh, hd), F)
        for head in range(nh):
            kv = head // (nh // nkv)
            s = (kcache[li, kv, : pos + 1, :] @ q[head]) * scale
            p = np.exp(s - s.max(), dtype=F)
            p = p / p.sum(dtype=F)
            out[head] = p @ vcache[li, kv, : pos + 1, :]
        h = h + L["o"] @ act(out.reshape(-1))
        x = act(rms_norm(h, L["post_norm"], eps))
        g = L["gate"] @ x
        u = L["up"] @ x
        with np.errstate(over="ignore"):   # exp(-g) may reach +inf, which gives the correct limit 0
            h = h + L["down"] @ act((g / (F(1.0) + np.exp(-g, dtype=F))) * u)
    logits = (model["lm_head"] @ act(rms_norm(h, model["final_norm"], eps))).astype(F)
    return logits, argmax_last(logits)
