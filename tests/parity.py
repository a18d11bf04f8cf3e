"""Shared helpers of the GPU parity tests: reference values from the CPU oracle and the
error measures the tolerances are written against."""
import numpy as np

from nn_b200 import formats as F
from nn_b200.formats import QuantFormat as Q
from oracle import cpu as orc

# north-star tolerances: f32 accumulation / bf16 tensor-core operands
TOL_F32_ACC = 2e-3
TOL_BF16_MMA = 1e-2


def oracle_dequant(fmt, w, scales, n, k):
    return orc.dequantize(fmt, w, n * k, scales).reshape(n, k)


def oracle_linear(fmt, w, scales, x, bias, n, k):
    """Reference result: dequantize (bit-exact decoders) then sequential f32 product, as
    DynTensor::matmul on the dequantized weight; plus the f64 value and the |x||w| scale."""
    m = x.shape[0]
    deq = oracle_dequant(fmt, w, scales, n, k)
    y32 = orc.linear_f32(x, deq, bias, m, n, k)
    y64 = orc.linear_f64(x, deq, bias, m, n, k)
    mag = orc.linear_abs(x, deq, m, n, k)
    if bias is not None:
        mag = mag + np.abs(bias.astype(np.float64))[None, :]
    return y32, y64, mag


def max_rel_err(y, ref):
    """max |y - ref| over the largest |ref|: the 'max relative error' of the tolerance. One scale
    for the whole output, so it says little about small elements next to large ones: every bar in
    these tests is asserted on this measure AND on max_scaled_err, the element-wise one."""
    denom = float(np.max(np.abs(ref))) or 1.0
    return float(np.max(np.abs(y.astype(np.float64) - ref.astype(np.float64)))) / denom


def max_scaled_err(y, ref64, mag):
    """Element-wise error relative to sum_k |x_k w_k| (the forward-error scale of a dot)."""
    return float(np.max(np.abs(y.astype(np.float64) - ref64) / np.maximum(mag, 1e-30)))


def assert_close(y, y32, y64, mag, tol=TOL_F32_ACC):
    assert np.all(np.isfinite(y))
    assert max_rel_err(y, y32) <= tol, ("max relative error", max_rel_err(y, y32))
    assert max_scaled_err(y, y64, mag) <= tol, ("scaled error", max_scaled_err(y, y64, mag))
