"""Block geometry of the quantized weight formats and seeded synthetic inputs.

Geometry follows the reference's tables: ``GgufDType::{block_size,type_size}``
(crates/nn-gguf/src/dequant.rs:84-114), ``QuantType::{block_size,block_bytes}``
(crates/nn-core/src/dyn_tensor/quantized.rs:58-76) and the MXFP4 block constants
(crates/nn-core/src/layers/quantized/mxfp4.rs:42-48).

The generators produce raw block bytes with the value distributions of the
benchmark configurations (scales |N(0,1)|*c as f16, integer codes uniform over
their range). They are driven by a SplitMix64 counter stream -- the same mixing
function as the reference's shared test generator
(crates/nn-core/src/test_prng.rs:18-23) -- so the bytes depend only on the seed,
not on the numpy version.
"""
from __future__ import annotations

import enum
from dataclasses import dataclass

import numpy as np


class QuantFormat(enum.IntEnum):
    """Format codes; the integer values are the ``nnq_format`` codes of include/nnq.h."""

    Q4_0 = 0
    Q4_1 = 1
    Q8_0 = 2
    Q4_K = 3        # nn-gguf element order and scale packing
    Q4_K_GGML = 4   # nn-core BlockQ4K element order and scale packing
    Q6_K = 5
    MXFP4_CORE = 6    # 17-byte interleaved blocks, low nibble = even element
    MXFP4_SPLIT = 7   # packed[N][K/2] + exps[N][K/32], low nibble = even element
    MXFP4_GPTOSS = 8  # data[n/2] + scales[n/32], high nibble = even element
    Q5_0 = 9          # nn-gguf decoders without a tiled layout: dequantization, row kernel and
    Q5_1 = 10         # tensor-core product only
    Q2_K = 11
    Q3_K = 12
    Q5_K = 13
    F32_DENSE = 14    # unquantized weights behind the same entry points: "blocks" of 32 values
    BF16_DENSE = 15


@dataclass(frozen=True)
class BlockGeometry:
    elems: int        # weights per block
    bytes: int        # bytes per block in the main buffer
    scale_bytes: int  # bytes per block in the separate scale buffer (MXFP4 split layouts)


GEOMETRY = {
    QuantFormat.Q4_0: BlockGeometry(32, 18, 0),
    QuantFormat.Q4_1: BlockGeometry(32, 20, 0),
    QuantFormat.Q8_0: BlockGeometry(32, 34, 0),
    QuantFormat.Q4_K: BlockGeometry(256, 144, 0),
    QuantFormat.Q4_K_GGML: BlockGeometry(256, 144, 0),
    QuantFormat.Q6_K: BlockGeometry(256, 210, 0),
    QuantFormat.MXFP4_CORE: BlockGeometry(32, 17, 0),
    QuantFormat.MXFP4_SPLIT: BlockGeometry(32, 16, 1),
    QuantFormat.MXFP4_GPTOSS: BlockGeometry(32, 16, 1),
    QuantFormat.Q5_0: BlockGeometry(32, 22, 0),
    QuantFormat.Q5_1: BlockGeometry(32, 24, 0),
    QuantFormat.Q2_K: BlockGeometry(256, 84, 0),
    QuantFormat.Q3_K: BlockGeometry(256, 110, 0),
    QuantFormat.Q5_K: BlockGeometry(256, 176, 0),
    QuantFormat.F32_DENSE: BlockGeometry(32, 128, 0),
    QuantFormat.BF16_DENSE: BlockGeometry(32, 64, 0),
}


def weight_nbytes(fmt: QuantFormat, n: int, k: int) -> tuple[int, int]:
    """(main buffer bytes, scale buffer bytes) of an [n, k] weight, blocks along k."""
    g = GEOMETRY[QuantFormat(fmt)]
    if k % g.elems:
        raise ValueError(f"in_features {k} is not a multiple of the {QuantFormat(fmt).name} block ({g.elems})")
    blocks = n * (k // g.elems)
    return blocks * g.bytes, blocks * g.scale_bytes


def algorithmic_bytes(fmt: QuantFormat, m: int, n: int, k: int, x_bytes: int, y_bytes: int) -> int:
    """Weights once in their file-format bytes, activations and outputs once."""
    wb, sb = weight_nbytes(fmt, n, k)
    return wb + sb + m * k * x_bytes + m * n * y_bytes


# --------------------------------------------------------------------------- #
# SplitMix64 counter stream
# --------------------------------------------------------------------------- #

_GOLDEN = np.uint64(0x9E3779B97F4A7C15)


def splitmix64(z: np.ndarray) -> np.ndarray:
    """Vectorised SplitMix64 finaliser (crates/nn-core/src/test_prng.rs:18-23)."""
    z = z.astype(np.uint64, copy=True)
    with np.errstate(over="ignore"):
        z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
        z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
    return z ^ (z >> np.uint64(31))


class Stream:
    """Deterministic stream: value i of a draw is splitmix64(seed + (offset+i)*golden)."""

    def __init__(self, seed: int):
        self.seed = np.uint64(seed & 0xFFFFFFFFFFFFFFFF)
        self.offset = 0

    def u64(self, count: int) -> np.ndarray:
        idx = np.arange(self.offset, self.offset + count, dtype=np.uint64)
        self.offset += count
        with np.errstate(over="ignore"):
            return splitmix64(self.seed + idx * _GOLDEN)

    def uniform(self, count: int) -> np.ndarray:
        """f64 in [0, 1) with 53 random bits."""
        return (self.u64(count) >> np.uint64(11)).astype(np.float64) * (1.0 / (1 << 53))

    def integers(self, count: int, lo: int, hi: int) -> np.ndarray:
        """Integers uniform in [lo, hi] (inclusive)."""
        span = hi - lo + 1
        return (self.u64(count) % np.uint64(span)).astype(np.int64) + lo

    def normal(self, count: int) -> np.ndarray:
        """Standard normals by Box-Muller on the same stream."""
        half = (count + 1) // 2
        u1 = 1.0 - self.uniform(half)          # (0, 1]
        u2 = self.uniform(half)
        r = np.sqrt(-2.0 * np.log(u1))
        out = np.concatenate([r * np.cos(2 * np.pi * u2), r * np.sin(2 * np.pi * u2)])
        return out[:count]


def _f16_bytes(v: np.ndarray) -> np.ndarray:
    return v.astype(np.float16).view(np.uint8).reshape(-1, 2)


# --------------------------------------------------------------------------- #
# synthetic weights (raw block bytes)
# --------------------------------------------------------------------------- #

def gen_q8_0(seed: int, n: int, k: int, scale: float = 0.02) -> np.ndarray:
    """d = f16(|N(0,1)|*scale), q uniform in [-127, 127]."""
    s = Stream(seed)
    nb = n * (k // 32)
    out = np.empty((nb, 34), np.uint8)
    out[:, 0:2] = _f16_bytes(np.abs(s.normal(nb)) * scale)
    out[:, 2:] = s.integers(nb * 32, -127, 127).astype(np.int8).view(np.uint8).reshape(nb, 32)
    return out.reshape(-1)


def gen_q4_0(seed: int, n: int, k: int, scale: float = 0.02) -> np.ndarray:
    s = Stream(seed)
    nb = n * (k // 32)
    out = np.empty((nb, 18), np.uint8)
    out[:, 0:2] = _f16_bytes(np.abs(s.normal(nb)) * scale)
    out[:, 2:] = s.integers(nb * 16, 0, 255).astype(np.uint8).reshape(nb, 16)
    return out.reshape(-1)


def gen_q4_1(seed: int, n: int, k: int, scale: float = 0.02) -> np.ndarray:
    s = Stream(seed)
    nb = n * (k // 32)
    out = np.empty((nb, 20), np.uint8)
    out[:, 0:2] = _f16_bytes(np.abs(s.normal(nb)) * scale)
    out[:, 2:4] = _f16_bytes(s.normal(nb) * scale)
    out[:, 4:] = s.integers(nb * 16, 0, 255).astype(np.uint8).reshape(nb, 16)
    return out.reshape(-1)


def gen_q4_k(seed: int, n: int, k: int, scale: float = 0.01) -> np.ndarray:
    """d, dmin = f16(|N(0,1)|*scale); 8 (sc, min) uniform 0..63; 256 nibbles uniform.

    Every bit of the 12 scale bytes and of the 128 quant bytes is uniform, which makes
    all 16 six-bit fields uniform in 0..63 under both the nn-gguf and the GGML packing.
    """
    s = Stream(seed)
    nb = n * (k // 256)
    out = np.empty((nb, 144), np.uint8)
    out[:, 0:2] = _f16_bytes(np.abs(s.normal(nb)) * scale)
    out[:, 2:4] = _f16_bytes(np.abs(s.normal(nb)) * scale)
    out[:, 4:16] = s.integers(nb * 12, 0, 255).astype(np.uint8).reshape(nb, 12)
    out[:, 16:] = s.integers(nb * 128, 0, 255).astype(np.uint8).reshape(nb, 128)
    return out.reshape(-1)


def gen_q6_k(seed: int, n: int, k: int, scale: float = 0.01) -> np.ndarray:
    """d = f16(|N(0,1)|*scale); 16 int8 scales uniform -128..127; q6 uniform 0..63."""
    s = Stream(seed)
    nb = n * (k // 256)
    out = np.empty((nb, 210), np.uint8)
    out[:, 0:192] = s.integers(nb * 192, 0, 255).astype(np.uint8).reshape(nb, 192)
    out[:, 192:208] = s.integers(nb * 16, -128, 127).astype(np.int8).view(np.uint8).reshape(nb, 16)
    out[:, 208:210] = _f16_bytes(np.abs(s.normal(nb)) * scale)
    return out.reshape(-1)


def gen_uniform_blocks(fmt: "QuantFormat", seed: int, n: int, k: int, scale: float = 0.01) -> np.ndarray:
    """Q5_0 / Q5_1 / Q2_K / Q3_K / Q5_K blocks: every code, high-bit and packed-scale byte uniform in
    0..255, the f16 super-block scales |N(0,1)| * scale (Q5_1's minimum signed)."""
    fmt = QuantFormat(fmt)
    g = GEOMETRY[fmt]
    s = Stream(seed)
    nb = n * (k // g.elems)
    out = s.integers(nb * g.bytes, 0, 255).astype(np.uint8).reshape(nb, g.bytes)
    f16_at = {QuantFormat.Q5_0: [(0, False)], QuantFormat.Q5_1: [(0, False), (2, True)],
              QuantFormat.Q2_K: [(80, False), (82, False)], QuantFormat.Q3_K: [(108, False)],
              QuantFormat.Q5_K: [(0, False), (2, False)]}[fmt]
    for off, signed in f16_at:
        v = s.normal(nb) * scale
        out[:, off:off + 2] = _f16_bytes(v if signed else np.abs(v))
    return out.reshape(-1)


def gen_mxfp4(seed: int, n: int, k: int, e_lo: int = 119, e_hi: int = 127):
    """Codes uniform over the 16 E2M1 values, exponent byte uniform in [e_lo, e_hi].

    Returns (codes[n, k/2] uint8, exps[n, k/32] uint8): nibble payload and E8M0 bytes;
    the three MXFP4 layouts are different arrangements of these two arrays.
    """
    s = Stream(seed)
    nb = n * (k // 32)
    codes = s.integers(nb * 16, 0, 255).astype(np.uint8).reshape(n, k // 2)
    exps = s.integers(nb, e_lo, e_hi).astype(np.uint8).reshape(n, k // 32)
    return codes, exps


def mxfp4_core_bytes(codes: np.ndarray, exps: np.ndarray) -> np.ndarray:
    """Interleave into 17-byte [exp][16 packed] blocks (nn-core Mxfp4Block)."""
    nb = exps.size
    out = np.empty((nb, 17), np.uint8)
    out[:, 0] = exps.reshape(-1)
    out[:, 1:] = codes.reshape(nb, 16)
    return out.reshape(-1)


def gen_weight(fmt: QuantFormat, seed: int, n: int, k: int):
    """(main bytes, scale bytes or None) for any format, benchmark distributions."""
    fmt = QuantFormat(fmt)
    if fmt in (QuantFormat.F32_DENSE, QuantFormat.BF16_DENSE):
        # unquantized weights ~ N(0, 0.02), the distribution the benchmark configures for dense parts
        v = (Stream(seed).normal(n * k) * 0.02).astype(np.float32)
        if fmt == QuantFormat.F32_DENSE:
            return v.view(np.uint8).copy(), None
        return to_bf16_bits(v).astype(np.uint16).view(np.uint8).copy(), None
    if fmt == QuantFormat.Q8_0:
        return gen_q8_0(seed, n, k), None
    if fmt == QuantFormat.Q4_0:
        return gen_q4_0(seed, n, k), None
    if fmt == QuantFormat.Q4_1:
        return gen_q4_1(seed, n, k), None
    if fmt in (QuantFormat.Q4_K, QuantFormat.Q4_K_GGML):
        return gen_q4_k(seed, n, k), None
    if fmt == QuantFormat.Q6_K:
        return gen_q6_k(seed, n, k), None
    if fmt >= QuantFormat.Q5_0:
        return gen_uniform_blocks(fmt, seed, n, k), None
    codes, exps = gen_mxfp4(seed, n, k)
    if fmt == QuantFormat.MXFP4_CORE:
        return mxfp4_core_bytes(codes, exps), None
    return codes.reshape(-1).copy(), exps.reshape(-1).copy()


# --------------------------------------------------------------------------- #
# activations
# --------------------------------------------------------------------------- #

def to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even f32 -> bf16, returned as uint16 bit patterns."""
    u = np.ascontiguousarray(x, np.float32).view(np.uint32)
    rounded = u + np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1))
    return (rounded >> np.uint32(16)).astype(np.uint16)


def bf16_bits_to_f32(b: np.ndarray) -> np.ndarray:
    return (b.astype(np.uint32) << np.uint32(16)).view(np.float32)


def gen_activations(seed: int, m: int, k: int, bf16: bool) -> np.ndarray:
    """x ~ N(0,1) as f32 [m, k]; with bf16=True the values are bf16-representable."""
    x = Stream(seed).normal(m * k).astype(np.float32).reshape(m, k)
    if bf16:
        x = bf16_bits_to_f32(to_bf16_bits(x)).reshape(m, k)
    return x
