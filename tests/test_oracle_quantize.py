"""Pins the oracle's f32 -> block encoders to the reference's own tests, restated:
BlockQ4K::quantize round trips and error cases (crates/nn-core/src/layers/quantized/linear_tests.rs:34-100,
301-330), nn-core MXFP4 (mxfp4_tests.rs:10-160,168-236,259-365) and nn-gptoss MXFP4
(crates/nn-gptoss/src/quantize.rs:292-318,344-372,398-405). No GPU needed."""
import numpy as np
import pytest

from nn_b200 import formats as F
from nn_b200.formats import QuantFormat as Q
from oracle import cpu as orc

f32 = np.float32


def _rt(fmt, v):
    v = np.asarray(v, f32)
    blocks, sc = orc.quantize(fmt, v)
    g = F.GEOMETRY[fmt]
    nb = (v.size + g.elems - 1) // g.elems
    assert blocks.size == nb * g.bytes and (sc is None or sc.size == nb)
    return orc.dequantize(fmt, blocks, nb * g.elems, sc)[:v.size], blocks, sc


def test_f32_to_f16_is_round_to_nearest_even():
    s = F.Stream(7)
    x = (s.normal(4000) * 10.0 ** s.integers(4000, -9, 5)).astype(f32)
    edge = np.array([0.0, -0.0, 65504.0, 65519.996, 65520.0, 1e-8, 5.9604645e-8, 2.9802322e-8, 2.98023224e-8 * 1.0000001,
                     6.1035156e-5, 6.0975552e-5, np.inf, -np.inf, 1.0009765625, 1.00048828125, 1.00146484375], f32)
    with np.errstate(over="ignore"):
        for v in np.concatenate([x, edge]):
            assert orc.f32_to_f16(v) == int(np.array(v, f32).astype(np.float16).view(np.uint16)), v


@pytest.mark.parametrize("values,tol", [(np.zeros(256), 0.01), (np.arange(256) / 255.0, 0.1),
                                        (np.arange(256) / 127.5 - 1.0, 0.2), (np.full(256, 0.5), 0.1)])
def test_q4_k_round_trips_within_the_reference_bounds(values, tol):
    out, blocks, _ = _rt(Q.Q4_K_GGML, values)
    assert np.max(np.abs(out - values.astype(f32))) < tol


def test_q4_k_error_and_degenerate_cases():
    v = np.full(256, 0.5, f32)
    v[128] = np.nan
    with pytest.raises(orc.ValueOutOfRange):
        orc.quantize(Q.Q4_K_GGML, v)
    for bad in (np.inf, -np.inf):
        v[128] = bad
        with pytest.raises(orc.ValueOutOfRange):
            orc.quantize(Q.Q4_K_GGML, v)
    v = np.full(256, -1.0, f32)    # clustered at the minimum: sumlx = 0 must not divide by zero
    v[0] = 0.0
    out, _, _ = _rt(Q.Q4_K_GGML, v)
    assert np.all(np.isfinite(out))
    # all-negative constant sub-blocks: scale 0, minimum -c; reproduced exactly up to the f16 minimum
    out, blocks, _ = _rt(Q.Q4_K_GGML, np.full(256, -0.75, f32))
    assert np.allclose(out, -0.75, atol=2e-3)
    # from_linear pads the flat buffer with zeros to whole blocks (linear.rs:318-336)
    w = (F.Stream(3).normal(300) * 0.1).astype(f32)
    blocks, _ = orc.quantize(Q.Q4_K_GGML, w)
    padded, _ = orc.quantize(Q.Q4_K_GGML, np.concatenate([w, np.zeros(212, f32)]))
    assert blocks.size == 2 * 144 and np.array_equal(blocks, padded)


def test_q4_k_quantizer_beats_rounding_noise_on_weights():
    w = (F.Stream(11).normal(64 * 1024) * 0.05).astype(f32)
    out, blocks, _ = _rt(Q.Q4_K_GGML, w)
    # 4-bit levels over each sub-block's range: rms error well under a tenth of the weights' rms
    assert np.sqrt(np.mean((out - w) ** 2)) < 0.1 * np.sqrt(np.mean(w ** 2))
    # packed fields stay in range and decode to the same values under nn-core's decoder only
    assert not np.array_equal(orc.dequantize(Q.Q4_K, blocks, w.size), out)


def test_mxfp4_core_cases():
    out, blocks, _ = _rt(Q.MXFP4_CORE, np.zeros(32))
    assert np.all(out == 0.0) and blocks[0] == 0 and not blocks[1:].any()
    # the eight magnitudes and their negatives are exact at scale 1 (max 6 -> shared exponent 127)
    mags = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0], f32)
    v = np.concatenate([mags, -mags, np.zeros(16, f32)])
    out, blocks, _ = _rt(Q.MXFP4_CORE, v)
    assert blocks[0] == 127 and np.array_equal(out, v)
    # max |v| = 1 -> ceil(log2(1/6)) + 127 = 125
    v = np.zeros(32, f32)
    v[0], v[1] = 1.0, -1.0
    _, blocks, _ = _rt(Q.MXFP4_CORE, v)
    assert blocks[0] == 125 and 6.0 * orc.mxfp4_core_scale(125) >= 1.0
    # signs survive; errors stay below half the largest step of the block's scale
    v = np.array([(1 if i % 2 == 0 else -1) * (i + 1) * 0.5 for i in range(32)], f32)
    out, blocks, _ = _rt(Q.MXFP4_CORE, v)
    assert np.all(np.sign(out[v > 0]) >= 0) and np.all(np.sign(out[v < 0]) <= 0)
    assert np.max(np.abs(out - v)) <= orc.mxfp4_core_scale(int(blocks[0])) * 1.0 + 1e-6
    for bad in (np.nan, np.inf, -np.inf):
        v2 = v.copy()
        v2[5] = bad
        with pytest.raises(orc.ValueOutOfRange):
            orc.quantize(Q.MXFP4_CORE, v2)
    # tensors: 64 -> 2 blocks, 50 -> 2 blocks (zero padded), 1 -> 1 block, 0 -> none
    for n, nb in ((64, 2), (50, 2), (1, 1), (0, 0)):
        blocks, _ = orc.quantize(Q.MXFP4_CORE, np.linspace(-1, 1, n, dtype=f32))
        assert blocks.size == nb * 17
    # near the top of the f32 range: ceil(log2(2e38 / 6)) + 127 = 252 (the clamp at 254 is never reached)
    out, blocks, _ = _rt(Q.MXFP4_CORE, np.full(32, 2.0e38, f32))
    assert blocks[0] == 252 and np.all(np.isfinite(out))


def test_mxfp4_gptoss_cases():
    v = np.array([0.0, 1.0, -1.0, 2.0, -2.0, 3.0, -3.0, 4.0], f32)
    out, data, sc = _rt(Q.MXFP4_GPTOSS, v)
    assert np.max(np.abs(out - v)) < 1e-6 and sc.size == 1 and data.size == 16
    assert sc[0] == 127 and data[0] == 0x02       # max 4 = 2^2 -> 129 - 2; element 0 in the HIGH nibble
    v = ((np.arange(64) - 32.0) * 0.1).astype(f32)
    out, data, sc = _rt(Q.MXFP4_GPTOSS, v)
    for b in range(2):
        seg = slice(32 * b, 32 * b + 32)
        assert np.max(np.abs(out[seg] - v[seg])) <= orc.mxfp4_gptoss_scale(int(sc[b])) * 1.0 + 1e-6
    out, _, _ = _rt(Q.MXFP4_GPTOSS, np.zeros(64))
    assert np.all(out == 0.0)
    out, _, _ = _rt(Q.MXFP4_GPTOSS, np.array([1000.0, -500.0, 250.0, -125.0], f32))
    assert np.all(np.isfinite(out))
    out, data, sc = _rt(Q.MXFP4_GPTOSS, np.arange(50, dtype=f32))
    assert out.size == 50 and sc.size == 2
    out, _, sc = _rt(Q.MXFP4_GPTOSS, np.full(32, np.finfo(f32).tiny / 100.0, f32))
    assert sc[0] == 0 and np.all(np.abs(out) < 1e-30)
    # non-finite values are skipped in the maximum and encode as zero (no error in this encoder)
    v = np.ones(32, f32)
    v[3], v[4] = np.nan, np.inf
    out, _, sc = _rt(Q.MXFP4_GPTOSS, v)
    assert sc[0] == 125 and out[3] == 0.0 and out[4] == 0.0 and out[0] == 1.0
