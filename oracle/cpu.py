"""ctypes front end of the CPU oracle (oracle/nnq_oracle.c).

Test infrastructure only: imported by tests/, by the smoke check and by the
benchmark's CPU-baseline leg. The product package never imports it.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "libnnq_oracle.so")
_lib = None

_u8p = ctypes.POINTER(ctypes.c_uint8)
_f32p = ctypes.POINTER(ctypes.c_float)
_f64p = ctypes.POINTER(ctypes.c_double)
_i32p = ctypes.POINTER(ctypes.c_int)


def build(force: bool = False) -> str:
    src = os.path.join(_HERE, "nnq_oracle.c")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.run(["make", "-C", _HERE, "-B" if force else "-s"], check=True,
                       stdout=subprocess.DEVNULL)
    return _SO


def lib():
    global _lib
    if _lib is None:
        build()   # no-op when the library is newer than its source
        _lib = ctypes.CDLL(_SO)
        _lib.orc_f16_to_f32.restype = ctypes.c_float
        _lib.orc_f16_to_f32.argtypes = [ctypes.c_uint16]
        for name in ("orc_dequant_q4_0", "orc_dequant_q4_1", "orc_dequant_q8_0", "orc_dequant_q4_k",
                     "orc_dequant_q4_k_ggml", "orc_dequant_q6_k", "orc_dequant_q5_0", "orc_dequant_q5_1",
                     "orc_dequant_q2_k", "orc_dequant_q3_k", "orc_dequant_q5_k"):
            f = getattr(_lib, name)
            f.restype = ctypes.c_size_t
            f.argtypes = [_u8p, ctypes.c_size_t, ctypes.c_size_t, _f32p]
        _lib.orc_f32_to_f16.restype = ctypes.c_uint16
        _lib.orc_f32_to_f16.argtypes = [ctypes.c_float]
        _lib.orc_quantize_q4_k_ggml.restype = ctypes.c_longlong
        _lib.orc_quantize_q4_k_ggml.argtypes = [_f32p, ctypes.c_size_t, _u8p]
        _lib.orc_quantize_mxfp4_core.restype = ctypes.c_longlong
        _lib.orc_quantize_mxfp4_core.argtypes = [_f32p, ctypes.c_size_t, _u8p]
        _lib.orc_quantize_mxfp4_gptoss.restype = ctypes.c_longlong
        _lib.orc_quantize_mxfp4_gptoss.argtypes = [_f32p, ctypes.c_size_t, _u8p, _u8p]
        _lib.orc_int8_quantize_per_channel.restype = ctypes.c_int
        _lib.orc_int8_quantize_per_channel.argtypes = [_f32p, ctypes.c_size_t, ctypes.c_size_t, ctypes.c_int, _u8p, _f32p, _i32p]
        _lib.orc_int8_dequantize_per_channel.argtypes = [_u8p, _f32p, _i32p, ctypes.c_size_t, ctypes.c_size_t, _f32p]
        _u32p = ctypes.POINTER(ctypes.c_uint32)
        sz = ctypes.c_size_t
        _lib.orc_group_quantize.restype = ctypes.c_int
        _lib.orc_group_quantize.argtypes = [_f32p, sz, sz, ctypes.c_int, sz, ctypes.c_int, _u8p, _f32p, _i32p]
        _lib.orc_group_dequantize.argtypes = [_u8p, _f32p, _i32p, sz, sz, ctypes.c_int, sz, _f32p]
        _lib.orc_gptq_unpack_qweight.argtypes = [_u32p, sz, sz, _f32p]
        _lib.orc_gptq_unpack_qzeros.argtypes = [_u32p, sz, sz, _f32p]
        _lib.orc_gptq_dequantize.restype = ctypes.c_int
        _lib.orc_gptq_dequantize.argtypes = [_f32p, _f32p, _f32p, sz, sz, sz, sz, _f32p]
        _lib.orc_gptq_load_weight.restype = ctypes.c_int
        _lib.orc_gptq_load_weight.argtypes = [_u32p, _f32p, _u32p, sz, sz, sz, sz, _f32p]
        _lib.orc_mxfp4_core_scale.restype = ctypes.c_float
        _lib.orc_mxfp4_core_scale.argtypes = [ctypes.c_uint8]
        _lib.orc_mxfp4_gptoss_scale.restype = ctypes.c_float
        _lib.orc_mxfp4_gptoss_scale.argtypes = [ctypes.c_uint8]
        _lib.orc_dequant_mxfp4_core.argtypes = [_u8p, ctypes.c_size_t, _f32p]
        _lib.orc_dequant_mxfp4_gptoss.argtypes = [_u8p, _u8p, ctypes.c_size_t, _f32p]
        _lib.orc_dequant_mxfp4_split.argtypes = [_u8p, _u8p, ctypes.c_size_t, ctypes.c_size_t, _f32p]
        _lib.orc_mxfp4_split_linear.argtypes = [_f32p, _u8p, _u8p, _f32p, _f32p, ctypes.c_size_t,
                                                ctypes.c_size_t, ctypes.c_size_t]
        _lib.orc_quantized_linear.restype = ctypes.c_int
        _lib.orc_quantized_linear.argtypes = [ctypes.c_int, _f32p, _u8p, _f32p, _f32p,
                                              ctypes.c_size_t, ctypes.c_size_t, ctypes.c_size_t]
        _lib.orc_linear_f32.argtypes = [_f32p, _f32p, _f32p, _f32p] + [ctypes.c_size_t] * 3
        _lib.orc_linear_f64.argtypes = [_f32p, _f32p, _f32p, _f64p] + [ctypes.c_size_t] * 3
        _lib.orc_linear_abs.argtypes = [_f32p, _f32p, _f64p] + [ctypes.c_size_t] * 3
        _lib.orc_nncpu_linear.argtypes = [_f32p, _f32p, _f32p, _f32p] + [ctypes.c_size_t] * 3 + [ctypes.c_int]
        _lib.orc_have_avx2.restype = ctypes.c_int
        _lib.orc_cpu_forward.restype = ctypes.c_int
        _lib.orc_cpu_forward.argtypes = [ctypes.c_int, _u8p, ctypes.c_size_t, _f32p, _f32p, _f32p, _f32p,
                                         ctypes.c_size_t, ctypes.c_size_t, ctypes.c_size_t, ctypes.c_int]
        _lib.orc_moe_route.argtypes = [_f32p, ctypes.c_int, ctypes.c_int, _i32p, _f32p]
        _lib.orc_moe_forward.argtypes = [_f32p, ctypes.c_size_t, ctypes.c_size_t, ctypes.c_size_t,
                                         ctypes.c_int, ctypes.c_int, _f32p, _f32p, _f32p, _f32p, _f32p,
                                         _f32p, ctypes.c_float, _f32p, _i32p, _f32p]
    return _lib


def _u8(a):
    a = np.ascontiguousarray(a, np.uint8)
    return a, a.ctypes.data_as(_u8p)


def _f32(a):
    if a is None:
        return None, None
    a = np.ascontiguousarray(a, np.float32)
    return a, a.ctypes.data_as(_f32p)


_DEQ = {0: "orc_dequant_q4_0", 1: "orc_dequant_q4_1", 2: "orc_dequant_q8_0", 3: "orc_dequant_q4_k",
        4: "orc_dequant_q4_k_ggml", 5: "orc_dequant_q6_k", 9: "orc_dequant_q5_0", 10: "orc_dequant_q5_1",
        11: "orc_dequant_q2_k", 12: "orc_dequant_q3_k", 13: "orc_dequant_q5_k"}


class ValueOutOfRange(ValueError):
    """The reference's TensorError::ValueOutOfRange (a non-finite input to an encoder)."""


def quantize(fmt: int, values):
    """f32 -> blocks with the reference's encoders: format 4 = BlockQ4K::quantize, 6 = nn-core
    quantize_tensor, 8 = nn-gptoss Mxfp4Tensor::quantize. Returns (bytes, scale bytes or None);
    the tail block is padded with zeros as the reference pads it."""
    fmt = int(fmt)
    v, vp = _f32(np.asarray(values, np.float32).reshape(-1))
    if fmt == 4:
        out = np.zeros((v.size + 255) // 256 * 144, np.uint8)
        rc = lib().orc_quantize_q4_k_ggml(vp, v.size, out.ctypes.data_as(_u8p))
        sc = None
    elif fmt == 6:
        out = np.zeros((v.size + 31) // 32 * 17, np.uint8)
        rc = lib().orc_quantize_mxfp4_core(vp, v.size, out.ctypes.data_as(_u8p))
        sc = None
    elif fmt == 8:
        nb = (v.size + 31) // 32
        out, sc = np.zeros(nb * 16, np.uint8), np.zeros(nb, np.uint8)
        rc = lib().orc_quantize_mxfp4_gptoss(vp, v.size, out.ctypes.data_as(_u8p), sc.ctypes.data_as(_u8p))
    else:
        raise ValueError("the reference has encoders for formats 4, 6 and 8 only")
    if rc < 0:
        raise ValueOutOfRange("non-finite value")
    return out, sc


def int8_quantize_per_channel(w, mode: int):
    """(q uint8 [n, k], scale f32 [n], zero_point i32 [n]) of an f32 [n, k] weight; mode 0 symmetric, 1 asymmetric."""
    w = np.ascontiguousarray(w, np.float32)
    n, k = w.shape
    q, sc, zp = np.zeros((n, k), np.uint8), np.zeros(n, np.float32), np.zeros(n, np.int32)
    rc = lib().orc_int8_quantize_per_channel(w.ctypes.data_as(_f32p), n, k, int(mode), q.ctypes.data_as(_u8p),
                                             sc.ctypes.data_as(_f32p), zp.ctypes.data_as(_i32p))
    if rc != 0:
        raise ValueOutOfRange("non-finite weight value")
    return q, sc, zp


def int8_dequantize_per_channel(q, scale, zp) -> np.ndarray:
    q = np.ascontiguousarray(q, np.uint8)
    scale = np.ascontiguousarray(scale, np.float32)
    zp = np.ascontiguousarray(zp, np.int32)
    n, k = q.shape
    out = np.zeros((n, k), np.float32)
    lib().orc_int8_dequantize_per_channel(q.ctypes.data_as(_u8p), scale.ctypes.data_as(_f32p), zp.ctypes.data_as(_i32p), n, k,
                                          out.ctypes.data_as(_f32p))
    return out


class ShapeMismatch(ValueError):
    """The reference's TensorError::ShapeMismatch / DataLengthMismatch."""


def group_quantize(w, bits: int, group_size: int, symmetric: bool = True):
    """quantize_per_group: (packed codes uint8, scale f32 [n * groups], zero_point i32 [n * groups])."""
    w = np.ascontiguousarray(w, np.float32)
    n, k = w.shape
    gpr = k // group_size if group_size else 0
    q = np.zeros(n * k if bits == 8 else (n * k + 1) // 2, np.uint8)
    sc, zp = np.zeros(n * gpr, np.float32), np.zeros(n * gpr, np.int32)
    rc = lib().orc_group_quantize(w.ctypes.data_as(_f32p), n, k, int(bits), int(group_size), int(bool(symmetric)),
                                  q.ctypes.data_as(_u8p), sc.ctypes.data_as(_f32p), zp.ctypes.data_as(_i32p))
    if rc in (-1, -2):
        raise ValueOutOfRange("non-finite weight value" if rc == -1 else "group_size must be > 0")
    if rc == -3:
        raise ShapeMismatch("group_size does not divide in_features")
    return q, sc, zp


def group_dequantize(q, scale, zp, n: int, k: int, bits: int, group_size: int) -> np.ndarray:
    q = np.ascontiguousarray(q, np.uint8)
    scale = np.ascontiguousarray(scale, np.float32)
    zp = np.ascontiguousarray(zp, np.int32)
    out = np.zeros((n, k), np.float32)
    lib().orc_group_dequantize(q.ctypes.data_as(_u8p), scale.ctypes.data_as(_f32p), zp.ctypes.data_as(_i32p), n, k,
                               int(bits), int(group_size), out.ctypes.data_as(_f32p))
    return out


def _u32(a):
    a = np.ascontiguousarray(a, np.uint32)
    return a, a.ctypes.data_as(ctypes.POINTER(ctypes.c_uint32))


def gptq_unpack_qweight(packed) -> np.ndarray:
    packed, pp = _u32(packed)
    rows, cols = packed.shape
    out = np.zeros((rows * 8, cols), np.float32)
    lib().orc_gptq_unpack_qweight(pp, rows, cols, out.ctypes.data_as(_f32p))
    return out


def gptq_unpack_qzeros(packed) -> np.ndarray:
    packed, pp = _u32(packed)
    groups, cols = packed.shape
    out = np.zeros((groups, cols * 8), np.float32)
    lib().orc_gptq_unpack_qzeros(pp, groups, cols, out.ctypes.data_as(_f32p))
    return out


def gptq_dequantize(q, scales, zeros, group_size: int) -> np.ndarray:
    q, qp = _f32(q)
    scales, sp = _f32(scales)
    zeros, zp = _f32(zeros)
    k, n = q.shape
    if scales.shape[1] != n or zeros.shape != scales.shape:
        raise ShapeMismatch("scales / zeros shape")
    out = np.zeros((k, n), np.float32)
    if lib().orc_gptq_dequantize(qp, sp, zp, k, n, scales.shape[0], int(group_size), out.ctypes.data_as(_f32p)) != 0:
        raise ShapeMismatch("group count")
    return out


def gptq_load_weight(qweight, scales, qzeros, group_size: int) -> np.ndarray:
    """f32 [n, k] weight of load_gptq_linear / load_awq_linear."""
    qweight, qp = _u32(qweight)
    scales, sp = _f32(scales)
    qzeros, zp = _u32(qzeros)
    k, n = qweight.shape[0] * 8, qweight.shape[1]
    out = np.zeros((n, k), np.float32)
    if lib().orc_gptq_load_weight(qp, sp, zp, n, k, scales.shape[0], int(group_size), out.ctypes.data_as(_f32p)) != 0:
        raise ShapeMismatch("group count")
    return out


def mxfp4_core_scale(e: int) -> float:
    return float(lib().orc_mxfp4_core_scale(int(e)))


def mxfp4_gptoss_scale(e: int) -> float:
    return float(lib().orc_mxfp4_gptoss_scale(int(e)))


def f32_to_f16(v: float) -> int:
    return int(lib().orc_f32_to_f16(float(v)))


def f16_to_f32(bits: int) -> float:
    return float(lib().orc_f16_to_f32(int(bits) & 0xFFFF))


def dequantize(fmt: int, data, num_elements: int, scales=None) -> np.ndarray:
    """Dequantize raw blocks of any supported format to f32 (flat)."""
    fmt = int(fmt)
    data, dp = _u8(data)
    if fmt == 14:     # unquantized f32: the bytes are the values
        return data[: num_elements * 4].view(np.float32).copy()
    if fmt == 15:     # unquantized bf16: exact widening
        return (data[: num_elements * 2].view(np.uint16).astype(np.uint32) << np.uint32(16)).view(np.float32)
    if fmt in _DEQ:
        out = np.zeros(num_elements, np.float32)
        n = getattr(lib(), _DEQ[fmt])(dp, data.size, num_elements, out.ctypes.data_as(_f32p))
        return out[:n]
    nblocks = num_elements // 32
    out = np.zeros(nblocks * 32, np.float32)
    if fmt == 6:
        lib().orc_dequant_mxfp4_core(dp, nblocks, out.ctypes.data_as(_f32p))
    elif fmt == 7:
        sc, sp = _u8(scales)
        lib().orc_dequant_mxfp4_split(dp, sp, 1, nblocks * 32, out.ctypes.data_as(_f32p))
    elif fmt == 8:
        sc, sp = _u8(scales)
        lib().orc_dequant_mxfp4_gptoss(dp, sp, nblocks, out.ctypes.data_as(_f32p))
    else:
        raise ValueError(f"unknown format {fmt}")
    return out


def mxfp4_split_linear(a, packed, exps, bias, m, k, n) -> np.ndarray:
    a, ap = _f32(a)
    packed, pp = _u8(packed)
    exps, ep = _u8(exps)
    bias, bp = _f32(bias)
    c = np.zeros((m, n), np.float32)
    lib().orc_mxfp4_split_linear(ap, pp, ep, bp, c.ctypes.data_as(_f32p), m, k, n)
    return c


def quantized_linear(fmt: int, x, w, bias, rows: int, n: int, k: int) -> np.ndarray:
    """nn-core fused Q4_0/Q8_0 product (block-wise accumulation order)."""
    x, xp = _f32(x)
    w, wp = _u8(w)
    bias, bp = _f32(bias)
    y = np.zeros((rows, n), np.float32)
    rc = lib().orc_quantized_linear(int(fmt), xp, wp, bp, y.ctypes.data_as(_f32p), rows, n, k)
    if rc != 0:
        raise ValueError("fused product exists only for Q4_0 and Q8_0")
    return y


def linear_f32(x, w, bias, m, n, k) -> np.ndarray:
    x, xp = _f32(x)
    w, wp = _f32(w)
    bias, bp = _f32(bias)
    y = np.zeros((m, n), np.float32)
    lib().orc_linear_f32(xp, wp, bp, y.ctypes.data_as(_f32p), m, n, k)
    return y


def linear_f64(x, w, bias, m, n, k) -> np.ndarray:
    x, xp = _f32(x)
    w, wp = _f32(w)
    bias, bp = _f32(bias)
    y = np.zeros((m, n), np.float64)
    lib().orc_linear_f64(xp, wp, bp, y.ctypes.data_as(_f64p), m, n, k)
    return y


def linear_abs(x, w, m, n, k) -> np.ndarray:
    x, xp = _f32(x)
    w, wp = _f32(w)
    y = np.zeros((m, n), np.float64)
    lib().orc_linear_abs(xp, wp, y.ctypes.data_as(_f64p), m, n, k)
    return y


def nncpu_linear(x, w, bias, m, n, k, threads=1) -> np.ndarray:
    x, xp = _f32(x)
    w, wp = _f32(w)
    bias, bp = _f32(bias)
    y = np.zeros((m, n), np.float32)
    lib().orc_nncpu_linear(xp, wp, bp, y.ctypes.data_as(_f32p), m, n, k, threads)
    return y


def cpu_forward(fmt: int, w, x, bias, m, n, k, threads=1, scratch=None) -> np.ndarray:
    """Dequantize-then-product, the cost of one reference QLinear::forward."""
    w, wp = _u8(w)
    x, xp = _f32(x)
    bias, bp = _f32(bias)
    if scratch is None:
        scratch = np.empty(n * k, np.float32)
    y = np.zeros((m, n), np.float32)
    rc = lib().orc_cpu_forward(int(fmt), wp, w.size, xp, bp, y.ctypes.data_as(_f32p),
                               scratch.ctypes.data_as(_f32p), m, n, k, threads)
    if rc != 0:
        raise ValueError("cpu_forward: unsupported format or short buffer")
    return y


def moe_route(logits, top_k):
    logits, lp = _f32(logits)
    idx = np.zeros(top_k, np.int32)
    w = np.zeros(top_k, np.float32)
    lib().orc_moe_route(lp, logits.size, top_k, idx.ctypes.data_as(_i32p), w.ctypes.data_as(_f32p))
    return idx, w


def moe_forward(x, router_w, router_b, w_gu, b_gu, w_d, b_d, top_k, limit):
    """x [T,H]; router_w [E,H]; w_gu [E,H,2I]; w_d [E,I,H] (all dequantized f32)."""
    x, xp = _f32(x)
    t, h = x.shape
    e = router_w.shape[0]
    inter = w_gu.shape[2] // 2
    rw, rwp = _f32(router_w)
    rb, rbp = _f32(router_b)
    wg, wgp = _f32(w_gu)
    bg, bgp = _f32(b_gu)
    wd, wdp = _f32(w_d)
    bd, bdp = _f32(b_d)
    y = np.zeros((t, h), np.float32)
    idx = np.zeros((t, top_k), np.int32)
    wt = np.zeros((t, top_k), np.float32)
    lib().orc_moe_forward(xp, t, h, inter, e, top_k, rwp, rbp, wgp, bgp, wdp, bdp,
                          ctypes.c_float(limit), y.ctypes.data_as(_f32p), idx.ctypes.data_as(_i32p),
                          wt.ctypes.data_as(_f32p))
    return y, idx, wt
