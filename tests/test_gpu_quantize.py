"""Device encoders (nnq_quantize through the C ABI) against the oracle's restatements of
BlockQ4K::quantize, nn-core quantize_tensor and nn-gptoss Mxfp4Tensor::quantize: identical bytes
on seeded weights, on the reference tests' inputs, on rounding edge cases, ragged tails and
empty inputs; error behaviour; QLinear.from_linear end to end."""
import numpy as np
import pytest

torch = pytest.importorskip("torch")

from nn_b200 import api
from nn_b200 import formats as F
from nn_b200.formats import QuantFormat as Q
from oracle import cpu as orc

pytestmark = pytest.mark.gpu
f32 = np.float32
ENC = [Q.Q4_K_GGML, Q.MXFP4_CORE, Q.MXFP4_GPTOSS]


def _same(fmt, v):
    v = np.asarray(v, f32)
    try:
        want, want_sc = orc.quantize(fmt, v)
    except orc.ValueOutOfRange:      # e.g. Q4_K on values whose f16 super-block scale overflows
        with pytest.raises(api.ValueOutOfRange):
            api.quantize(torch.from_numpy(v), fmt)
        return None, None
    got, got_sc = api.quantize(torch.from_numpy(v), fmt)
    got = got.cpu().numpy()
    bad = np.nonzero(got != want)[0]
    assert bad.size == 0, (fmt.name, bad[:8], got[bad[:8]], want[bad[:8]])
    if want_sc is not None:
        assert np.array_equal(got_sc.cpu().numpy(), want_sc)
    return want, want_sc


@pytest.mark.parametrize("fmt", ENC)
@pytest.mark.parametrize("n,scale", [(256, 1.0), (4096, 0.02), (1 << 20, 0.05), (1000, 3.0), (33, 1e-3), (1, 1.0)])
def test_encoders_are_byte_identical_on_seeded_weights(fmt, n, scale):
    v = (F.Stream(n + int(fmt)).normal(n) * scale).astype(f32)
    _same(fmt, v)


@pytest.mark.parametrize("fmt", ENC)
def test_reference_test_inputs(fmt):
    cases = [np.zeros(256), np.arange(256) / 255.0, np.arange(256) / 127.5 - 1.0, np.full(256, 0.5), np.full(256, -0.75),
             np.concatenate([[0.0], np.full(255, -1.0)]), (np.arange(64) - 32.0) * 0.1, np.arange(50.0),
             [0.0, 1.0, -1.0, 2.0, -2.0, 3.0, -3.0, 4.0], [1000.0, -500.0, 250.0, -125.0],
             np.full(32, np.finfo(f32).tiny / 100.0), [(1 if i % 2 == 0 else -1) * (i + 1) * 0.5 for i in range(32)],
             np.full(32, 2.0e38), np.abs(F.Stream(5).normal(512)) + 0.1]
    for c in cases:
        _same(fmt, c)


@pytest.mark.parametrize("fmt", ENC)
def test_rounding_edges(fmt):
    s = F.Stream(91)
    # block maxima on and next to powers of two and 6 * 2^e, over a wide exponent range; ties between
    # neighbouring magnitudes; signed zeros; subnormals
    compared = 0
    for e in list(range(-140, 128, 7)) + [-126, -127, -1, 0, 1]:
        blocks = []
        for m in (1.0, 1.5, 6.0 / 4.0, 1.25, 1.75):
            top = f32(m) * f32(2.0) ** f32(e) if e > -127 else f32(m * 2.0 ** -126) * f32(2.0 ** (e + 126))
            if not np.isfinite(top) or top > 3.0e38:
                continue
            for t in (top, np.nextafter(f32(top), f32(np.inf)), np.nextafter(f32(top), f32(0))):
                if not np.isfinite(t):
                    continue
                b = (s.uniform(32) * 2 - 1).astype(f32) * f32(t)
                b[0] = t
                b[1] = -t * f32(0.5)
                b[2:10] = (f32(t) / f32(6.0)) * np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 0.125], f32)
                b[10], b[11] = 0.0, -0.0
                assert np.all(np.isfinite(b))
                blocks.append(b)
        if blocks:   # per exponent, so that a range the reference rejects (Q4_K: f16 scale overflow) stays local
            compared += _same(fmt, np.concatenate(blocks))[0] is not None
    # nn-core's Q4_K encoder rejects blocks whose f16 super-block scale overflows (inf * 0 reaches nearest_int);
    # there the device must raise too, which _same checked
    assert compared >= (24 if fmt == Q.Q4_K_GGML else 44)


def test_q4_k_sub_block_patterns():
    s = F.Stream(17)
    parts = []
    for kind in range(12):
        b = (s.normal(256) * 0.1).astype(f32)
        if kind == 1:
            b = np.abs(b)                      # all positive: minima are zero
        elif kind == 2:
            b = -np.abs(b)                     # all negative
        elif kind == 3:
            b[:32] = 0.25                      # constant positive sub-block
        elif kind == 4:
            b[32:64] = -0.25                   # constant negative sub-block
        elif kind == 5:
            b[:] = 0.0
            b[7] = 1e-30
        elif kind == 6:
            b *= f32(1e20)
        elif kind == 7:
            b *= f32(1e-25)
        elif kind == 8:
            b[64:96] = np.where(np.arange(32) % 2 == 0, -1.0, -1.0 + 1e-6)   # clustered at the minimum
        elif kind == 9:
            b = np.round(b * 40) / 40          # many exact ties
        elif kind == 10:
            b[:128] = 0.0
        elif kind == 11:
            b = (s.uniform(256) * 15).astype(f32)
        parts.append(b.astype(f32))
    for part in parts:
        _same(Q.Q4_K_GGML, part)
    blocks, _ = _same(Q.Q4_K_GGML, np.concatenate(parts[:6] + parts[7:]))
    out = orc.dequantize(Q.Q4_K_GGML, blocks, 11 * 256)
    assert blocks is not None and np.all(np.isfinite(out[:11 * 256]))


@pytest.mark.parametrize("fmt", ENC)
def test_empty_input(fmt):
    out, sc = api.quantize(torch.zeros(0), fmt)
    assert out.numel() == 0 and (sc is None or sc.numel() == 0)


def test_non_finite_inputs():
    v = np.full(512, 0.5, f32)
    for bad in (np.nan, np.inf, -np.inf):
        v[300] = bad
        for fmt in (Q.Q4_K_GGML, Q.MXFP4_CORE):
            with pytest.raises(api.ValueOutOfRange):
                api.quantize(torch.from_numpy(v), fmt)
        _same(Q.MXFP4_GPTOSS, v)    # this encoder skips them
    v[300] = 0.5
    _same(Q.Q4_K_GGML, v)           # the error state does not stick
    # a NaN the Q4_K reference never looks at: constant negative sub-block, so the block's levels stay zero
    v = np.full(256, -1.0, f32)
    v[5] = np.nan
    try:
        want, _ = orc.quantize(Q.Q4_K_GGML, v)
    except orc.ValueOutOfRange:
        with pytest.raises(api.ValueOutOfRange):
            api.quantize(torch.from_numpy(v), Q.Q4_K_GGML)
    else:
        _same(Q.Q4_K_GGML, v)


def test_formats_without_an_encoder_are_refused():
    for fmt in (Q.Q8_0, Q.Q4_K, Q.Q6_K, Q.MXFP4_SPLIT):
        with pytest.raises(api.Unsupported):
            api.quantize(torch.ones(256), fmt)


def test_qlinear_from_linear_end_to_end():
    n, k, m = 96, 1024, 5
    s = F.Stream(23)
    w = (s.normal(n * k) * 0.05).astype(f32).reshape(n, k)
    x = s.normal(m * k).astype(f32).reshape(m, k)
    bias = torch.from_numpy(s.normal(n).astype(f32)).cuda()
    layer = api.QLinear.from_linear(torch.from_numpy(w), bias)
    assert layer.is_quantized() and layer.weight.dims() == (n, k)
    blocks, _ = orc.quantize(Q.Q4_K_GGML, w)
    wq = orc.dequantize(Q.Q4_K_GGML, blocks, n * k).reshape(n, k)
    deq, _ = layer.dequantize()
    assert np.array_equal(deq.cpu().numpy(), wq)             # same blocks, same decoder
    y = layer(torch.from_numpy(x).cuda()).cpu().numpy()
    want = orc.linear_f64(x, wq, bias.cpu().numpy(), m, n, k)
    assert np.max(np.abs(y - want)) <= 2e-3 * max(1.0, np.max(np.abs(want)))
    # and close to the unquantized layer, as the reference's forward test asks (4-bit noise)
    dense = x.astype(np.float64) @ w.T.astype(np.float64) + bias.cpu().numpy()
    assert np.sqrt(np.mean((y - dense) ** 2)) < 0.1 * np.sqrt(np.mean(dense ** 2))
    with pytest.raises(api.Unsupported):
        api.QLinear.from_linear(torch.ones(4, 100))
