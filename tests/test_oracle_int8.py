"""Pins the oracle's INT8 per-channel restatement to the reference's tests
(crates/nn-core/src/layers/quantized/int8_tests.rs:14-160), restated. No GPU needed."""
import numpy as np
import pytest

from oracle import cpu as orc

f32 = np.float32


def _rt(w, mode):
    q, sc, zp = orc.int8_quantize_per_channel(np.asarray(w, f32), mode)
    return orc.int8_dequantize_per_channel(q, sc, zp), q, sc, zp


def test_zeros():
    out, q, sc, zp = _rt(np.zeros((4, 8)), 0)
    assert q.shape == (4, 8) and q.dtype == np.uint8 and np.all(sc == 0) and np.all(zp == 0) and np.all(out == 0)


@pytest.mark.parametrize("mode,data,tol", [
    (0, (np.arange(64) / 31.0) * 2.0 - 1.0, 0.02), (0, (np.arange(64) / 63.0) * 0.5, 0.01),
    (1, (np.arange(64) / 63.0) * 2.0 - 1.0, 0.02)])
def test_round_trip_bounds(mode, data, tol):
    w = data.astype(f32).reshape(4, 16)
    out, q, sc, zp = _rt(w, mode)
    assert np.max(np.abs(out - w)) < tol
    if mode == 0:
        assert np.all(zp == 0)


def test_constant_channels():
    out, q, sc, zp = _rt(np.full((3, 8), 0.5), 0)
    assert np.max(np.abs(out - 0.5)) < 0.01 and np.all(q.view(np.int8) == 127)
    out, q, sc, zp = _rt(np.full((3, 8), 0.5), 1)      # asymmetric: range 0 -> scale 0, codes 0
    assert np.all(sc == 0) and np.all(zp == 0) and np.all(q == 0) and np.all(out == 0)


def test_asymmetric_parameters():
    w = np.array([[-1.0, 0.0, 1.0, 3.0]], f32)
    out, q, sc, zp = _rt(w, 1)
    assert sc[0] == f32(4.0) / f32(255.0)
    assert zp[0] == int(np.round(f32(-128.0) - f32(-1.0) / sc[0]))
    assert q.view(np.int8)[0, 0] == -128 and q.view(np.int8)[0, 3] == 127


@pytest.mark.parametrize("bad", [np.nan, np.inf, -np.inf])
def test_non_finite_is_an_error(bad):
    w = np.array([[0.0, 1.0, bad, 0.5], [0.0, 1.0, 0.0, 0.5]], f32)
    for mode in (0, 1):
        with pytest.raises(orc.ValueOutOfRange):
            orc.int8_quantize_per_channel(w, mode)


def test_dequantize_formula_with_wide_zero_points():
    q = np.arange(256, dtype=np.uint8).reshape(2, 128)
    sc = np.array([0.25, 3.0e-3], f32)
    zp = np.array([-7, 100_000_000], np.int32)
    out = orc.int8_dequantize_per_channel(q, sc, zp)
    want = (q.view(np.int8).astype(f32) - zp.astype(f32)[:, None]) * sc[:, None]
    assert np.array_equal(out, want)
