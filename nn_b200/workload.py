"""The benchmark workload: the Q4_K projection sweep over Qwen3-8B layer shapes.

Shapes come from the callers that fix them in the reference
(crates/nn-qwen3/src/layers.rs:26-47,65-92: q/o hidden->hidden, k/v hidden->kv,
gate/up hidden->ffn, down ffn->hidden) with the Qwen3-8B sizes of the benchmark
configuration (hidden 4096, 32 query / 8 KV heads x 128, FFN 12288, 36 layers).
Weights are synthetic with the configured distributions and are drawn on the device.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np

from .formats import QuantFormat, algorithmic_bytes, weight_nbytes

HIDDEN = 4096
KV_DIM = 1024
FFN = 12288
LAYERS = 36

# (name, N, K) in the order a decoder layer issues them
PROJECTIONS = (
    ("q_proj", HIDDEN, HIDDEN),
    ("k_proj", KV_DIM, HIDDEN),
    ("v_proj", KV_DIM, HIDDEN),
    ("o_proj", HIDDEN, HIDDEN),
    ("gate_proj", FFN, HIDDEN),
    ("up_proj", FFN, HIDDEN),
    ("down_proj", HIDDEN, FFN),
)

# launch groups of one layer: products that share their input go out in one call
GROUPS = (("q_proj", "k_proj", "v_proj"), ("o_proj",), ("gate_proj", "up_proj"), ("down_proj",))

# tensor-parallel split axis of each projection: 0 = rows (column-parallel, no exchange),
# 1 = K blocks (row-parallel, outputs summed across ranks)
TP_AXIS = {"q_proj": 0, "k_proj": 0, "v_proj": 0, "o_proj": 1, "gate_proj": 0, "up_proj": 0, "down_proj": 1}


@dataclass
class LayerBytes:
    weights: int
    algorithmic: int


def layer_bytes(m: int, x_bytes: int = 2, y_bytes: int = 2, world: int = 1) -> LayerBytes:
    wsum = 0
    asum = 0
    for _, n, k in PROJECTIONS:
        wb, sb = weight_nbytes(QuantFormat.Q4_K, n, k)
        wsum += wb + sb
        asum += algorithmic_bytes(QuantFormat.Q4_K, m, n, k, x_bytes, y_bytes)
    return LayerBytes(wsum // world, asum // world)


def gen_q4_k_device(torch, gen, n: int, k: int, scale: float = 0.01):
    """Q4_K blocks drawn on the device: d, dmin = f16(|N(0,1)|*scale), all scale and quant
    bytes uniform (every 6-bit scale / min uniform in 0..63, every nibble uniform in 0..15)."""
    nb = n * (k // 256)
    dev = gen.device
    out = torch.randint(0, 256, (nb, 144), dtype=torch.uint8, device=dev, generator=gen)
    d = (torch.randn(nb, 2, device=dev, generator=gen).abs() * scale).to(torch.float16)
    out[:, 0:4] = d.view(torch.uint8).reshape(nb, 4)
    return out.reshape(-1)


def gen_q8_0_device(torch, gen, n: int, k: int, scale: float = 0.02):
    """Q8_0 blocks drawn on the device: d = f16(|N(0,1)|*scale), quants uniform over all bytes
    (the configured range is [-127, 127]; -128 appears with probability 1/256)."""
    nb = n * (k // 32)
    dev = gen.device
    out = torch.randint(0, 256, (nb, 34), dtype=torch.uint8, device=dev, generator=gen)
    d = (torch.randn(nb, 1, device=dev, generator=gen).abs() * scale).to(torch.float16)
    out[:, 0:2] = d.view(torch.uint8).reshape(nb, 2)
    return out.reshape(-1)


def gen_q6_k_device(torch, gen, n: int, k: int, scale: float = 0.01):
    """Q6_K blocks drawn on the device: d = f16(|N(0,1)|*scale), int8 scales and six-bit quants
    uniform."""
    nb = n * (k // 256)
    dev = gen.device
    out = torch.randint(0, 256, (nb, 210), dtype=torch.uint8, device=dev, generator=gen)
    d = (torch.randn(nb, 1, device=dev, generator=gen).abs() * scale).to(torch.float16)
    out[:, 208:210] = d.view(torch.uint8).reshape(nb, 2)
    return out.reshape(-1)


def gen_q4_k_host(seed: int, n: int, k: int) -> np.ndarray:
    from .formats import gen_q4_k
    return gen_q4_k(seed, n, k)
