"""Pins the oracle's INT4 / INT8 per-group and GPTQ / AWQ restatements to the reference's own
tests, restated: crates/nn-core/src/layers/quantized/weight_quant_tests.rs:14-410 and
crates/nn-core/src/layers/quantized/gptq_awq_tests.rs (known packed words, dequantize formula,
load -> forward end to end). No GPU needed."""
import numpy as np
import pytest

from oracle import cpu as orc

f32 = np.float32


def _ramp(n=512, lo=-1.0, hi=1.0):
    return (np.arange(n, dtype=f32) / f32(n - 1) * f32(hi - lo) + f32(lo)).astype(f32).reshape(4, n // 4)


def _rt(w, bits, g, symmetric=True):
    w = np.asarray(w, f32)
    q, sc, zp = orc.group_quantize(w, bits, g, symmetric)
    return orc.group_dequantize(q, sc, zp, w.shape[0], w.shape[1], bits, g), q, sc, zp


def test_zeros_give_zero_scales_and_values():
    out, q, sc, zp = _rt(np.zeros((4, 128)), 4, 128)
    assert sc.shape == (4,) and zp.shape == (4,) and np.all(sc == 0) and np.all(out == 0) and np.all(q == 0)


@pytest.mark.parametrize("bits,g,sym,tol", [(4, 128, True, 0.10), (4, 32, True, 0.10), (8, 128, True, 0.02),
                                            (4, 128, False, 0.2)])
def test_round_trip_bounds_on_a_ramp(bits, g, sym, tol):
    w = _ramp()
    out, q, sc, zp = _rt(w, bits, g, sym)
    assert sc.shape == (4 * (128 // g),)
    assert np.max(np.abs(out - w)) < tol
    if sym:
        assert np.all(zp == 0)
        # scale = max|w| / 7 or 127 per group
        qmax = f32(7.0 if bits == 4 else 127.0)
        want = np.abs(w).reshape(-1, g).max(axis=1) / qmax
        assert np.array_equal(sc, want.astype(f32))


def test_int8_is_at_least_as_close_as_int4():
    w = np.clip(np.sin(np.arange(512, dtype=f32)) * f32(0.5), -0.5, 0.5).astype(f32).reshape(4, 128)
    e4 = np.max(np.abs(_rt(w, 4, 128)[0] - w))
    e8 = np.max(np.abs(_rt(w, 8, 128)[0] - w))
    assert e8 <= e4


def test_constant_and_negative_only_groups():
    out, q, sc, zp = _rt(np.full((4, 128), 0.5), 4, 128)
    assert np.max(np.abs(out - 0.5)) < 0.01
    w = (-(np.arange(512, dtype=f32) / f32(511.0)) * f32(0.5)).reshape(4, 128)
    assert np.max(np.abs(_rt(w, 4, 128)[0] - w)) < 0.2


def test_error_cases():
    w = np.zeros((4, 128), f32)
    w[1, 7] = np.nan
    with pytest.raises(orc.ValueOutOfRange):
        orc.group_quantize(w, 4, 128)
    w[1, 7] = np.inf
    with pytest.raises(orc.ValueOutOfRange):
        orc.group_quantize(w, 8, 128)
    with pytest.raises(orc.ShapeMismatch):
        orc.group_quantize(np.zeros((4, 100), f32), 4, 128)
    with pytest.raises(orc.ValueOutOfRange):
        orc.group_quantize(np.zeros((4, 128), f32), 4, 0)


def test_nibble_packing_is_low_then_high_and_sign_extended():
    # every pair of codes in [-8, 7] survives pack -> unpack (the reference's exhaustive proof harness)
    codes = np.array([(lo, hi) for lo in range(-8, 8) for hi in range(-8, 8)], np.int8).reshape(-1)
    packed = ((codes[0::2] & 0x0F).astype(np.uint8) | ((codes[1::2] & 0x0F).astype(np.uint8) << 4)).astype(np.uint8)
    n = codes.size
    out = orc.group_dequantize(packed, np.ones(1, f32), np.zeros(1, np.int32), 1, n, 4, n)
    assert np.array_equal(out.reshape(-1), codes.astype(f32))
    # and the encoder produces that packing: scale 1 (max |w| = 7), the codes are the values
    w = np.array([[7, -7, 3, -8 + 1, 0, 1, -1, 5]], f32)
    q, sc, zp = orc.group_quantize(w, 4, 8)
    assert sc[0] == f32(1.0)
    assert list(q) == [(7 & 15) | ((-7 & 15) << 4), (3 & 15) | ((-7 & 15) << 4), 0 | (1 << 4), (-1 & 15) | (5 << 4)]


def test_asymmetric_parameters():
    w = np.array([[-1.0, 0.0, 1.0, 3.0]], f32)
    q, sc, zp = orc.group_quantize(w, 8, 4, symmetric=False)
    assert sc[0] == f32(4.0) / f32(255.0)
    assert zp[0] == int(np.round(f32(-128.0) - f32(-1.0) / sc[0]))
    assert q.view(np.int8)[0] == -128 and q.view(np.int8)[3] == 127
    q, sc, zp = orc.group_quantize(w, 4, 4, symmetric=False)
    assert sc[0] == f32(4.0) / f32(15.0) and zp[0] == int(np.round(f32(-8.0) - f32(-1.0) / sc[0]))


def test_quantized_matmul_close_to_float():
    w = ((np.arange(512) % 17).astype(f32) / f32(16.0) * f32(0.3) - f32(0.15)).reshape(4, 128)
    x = np.ones((2, 128), f32)
    ref = x @ w.T
    for bits, tol in ((4, 2.0), (8, 0.5)):
        deq = _rt(w, bits, 128)[0]
        y = orc.linear_f32(x, deq, None, 2, 4, 128)
        assert y.shape == (2, 4) and np.max(np.abs(y - ref)) < tol


def _pack8(vals):
    p = 0
    for i, v in enumerate(vals):
        p |= (int(v) & 0xF) << (4 * i)
    return p


def test_gptq_unpack_known_words():
    out = orc.gptq_unpack_qweight(np.array([[_pack8([1, 2, 3, 4, 5, 6, 7, 8])]], np.uint32))
    assert out.shape == (8, 1) and list(out[:, 0]) == [1, 2, 3, 4, 5, 6, 7, 8]
    assert np.all(orc.gptq_unpack_qweight(np.array([[0]], np.uint32)) == 0)
    assert np.all(orc.gptq_unpack_qweight(np.array([[0xFFFFFFFF]], np.uint32)) == 15)
    two = orc.gptq_unpack_qweight(np.array([[_pack8(range(8)), _pack8(range(8, 16))]], np.uint32))
    assert two.shape == (8, 2) and list(two[:, 0]) == list(range(8)) and list(two[:, 1]) == list(range(8, 16))
    # AWQ shares the packing
    awq = orc.gptq_unpack_qweight(np.array([[_pack8([3, 7, 11, 15, 0, 4, 8, 12])]], np.uint32))
    assert list(awq[:, 0]) == [3, 7, 11, 15, 0, 4, 8, 12]
    z = orc.gptq_unpack_qzeros(np.array([[_pack8([8] * 8)]], np.uint32))
    assert z.shape == (1, 8) and np.all(z == 8)


def test_gptq_dequantize_formula():
    q = np.full((8, 8), 8.0, f32)
    out = orc.gptq_dequantize(q, np.full((1, 8), 0.1, f32), np.full((1, 8), 8.0, f32), 8)
    assert out.shape == (8, 8) and np.all(np.abs(out) < 1e-6)
    out = orc.gptq_dequantize(np.full((8, 8), 10.0, f32), np.full((1, 8), 0.5, f32), np.full((1, 8), 8.0, f32), 8)
    assert np.all(np.abs(out - 1.0) < 1e-6)
    with pytest.raises(orc.ShapeMismatch):
        orc.gptq_dequantize(np.zeros((16, 8), f32), np.ones((1, 8), f32), np.zeros((1, 8), f32), 8)


@pytest.mark.parametrize("rows,g,qv,zv,scale,want", [(1, 8, 10, 8, 0.5, 8.0), (16, 128, 5, 0, 1.0, 640.0)])
def test_gptq_load_then_forward(rows, g, qv, zv, scale, want):
    qweight = np.full((rows, 8), _pack8([qv] * 8), np.uint32)
    scales = np.full((1, 8), scale, f32)
    qzeros = np.array([[_pack8([zv] * 8)]], np.uint32)
    w = orc.gptq_load_weight(qweight, scales, qzeros, g)
    assert w.shape == (8, rows * 8)
    y = orc.linear_f32(np.ones((1, rows * 8), f32), w, None, 1, 8, rows * 8)
    assert np.all(np.abs(y - want) < 1e-2)


def test_gptq_load_equals_unpack_dequantize_transpose():
    rng = np.random.default_rng(5)
    k, n, g = 64, 24, 16
    qweight = rng.integers(0, 2 ** 32, size=(k // 8, n), dtype=np.uint64).astype(np.uint32)
    qzeros = rng.integers(0, 2 ** 32, size=(k // g, n // 8), dtype=np.uint64).astype(np.uint32)
    scales = rng.standard_normal((k // g, n)).astype(f32)
    want = orc.gptq_dequantize(orc.gptq_unpack_qweight(qweight), scales, orc.gptq_unpack_qzeros(qzeros), g).T
    assert np.array_equal(orc.gptq_load_weight(qweight, scales, qzeros, g), want)
