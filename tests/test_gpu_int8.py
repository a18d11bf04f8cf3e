"""INT8 per-channel (W8A16) on the device through the C ABI against the oracle's restatement of
quantize_per_channel / dequantize_per_channel / Int8Linear::forward: identical codes and
parameters, bit-identical dequantization, products within the f32-accumulation tolerance."""
import numpy as np
import pytest

torch = pytest.importorskip("torch")

from nn_b200 import api, int8
from nn_b200 import formats as F
from oracle import cpu as orc

pytestmark = pytest.mark.gpu
f32 = np.float32
TOL = 2e-3   # f32 accumulation, relative to sum |w||x|


def _weights(seed, n, k, kind=0):
    s = F.Stream(seed)
    w = (s.normal(n * k) * 0.05).astype(f32).reshape(n, k)
    if kind == 1:
        w += f32(0.3)                 # asymmetric rows: zero points far from 0
    if kind == 2 and n > 2:
        w[1] = 0.0                    # a zero row and a constant row
        w[2] = 0.125
    return w


@pytest.mark.parametrize("mode", [int8.SYMMETRIC, int8.ASYMMETRIC])
@pytest.mark.parametrize("n,k,kind", [(4, 8, 0), (33, 100, 1), (64, 4096, 0), (7, 1, 2), (300, 1024, 2), (1, 12288, 1)])
def test_quantize_and_dequantize_are_identical(mode, n, k, kind):
    w = _weights(n * 31 + k + mode, n, k, kind)
    q0, sc0, zp0 = orc.int8_quantize_per_channel(w, mode)
    q, p = int8.quantize_per_channel(torch.from_numpy(w), mode)
    assert np.array_equal(p.scale.cpu().numpy().view(np.uint32), sc0.view(np.uint32))
    assert np.array_equal(p.zero_point.cpu().numpy(), zp0)
    assert np.array_equal(q.cpu().numpy(), q0)
    d = int8.dequantize_per_channel(q, p).cpu().numpy()
    assert np.array_equal(d.view(np.uint32), orc.int8_dequantize_per_channel(q0, sc0, zp0).view(np.uint32))


def test_reference_test_inputs():
    cases = [(0, np.zeros((4, 8))), (0, ((np.arange(64) / 31.0) * 2 - 1).reshape(4, 16)), (0, ((np.arange(64) / 63.0) * 0.5).reshape(4, 16)),
             (0, np.full((3, 8), 0.5)), (1, np.full((3, 8), 0.5)), (1, ((np.arange(64) / 63.0) * 2 - 1).reshape(4, 16))]
    for mode, w in cases:
        w = w.astype(f32)
        q0, sc0, zp0 = orc.int8_quantize_per_channel(w, mode)
        q, p = int8.quantize_per_channel(torch.from_numpy(w), mode)
        assert np.array_equal(q.cpu().numpy(), q0) and np.array_equal(p.scale.cpu().numpy(), sc0)
        assert np.array_equal(p.zero_point.cpu().numpy(), zp0)


@pytest.mark.parametrize("bad", [np.nan, np.inf, -np.inf])
def test_non_finite_weight_is_refused(bad):
    w = np.array([[0.0, 1.0, bad, 0.5], [0.0, 1.0, 0.0, 0.5]], f32)
    with pytest.raises(api.ValueOutOfRange):
        int8.quantize_per_channel(torch.from_numpy(w), int8.SYMMETRIC)
    q, p = int8.quantize_per_channel(torch.from_numpy(np.nan_to_num(w, posinf=1.0, neginf=-1.0)), int8.SYMMETRIC)   # state does not stick
    assert q.shape == (2, 4)


def test_wide_zero_point_dequantizes_like_the_reference():
    q = torch.arange(256, dtype=torch.uint8).reshape(2, 128).cuda()
    p = int8.Int8QuantParams(torch.tensor([0.25, 3.0e-3], dtype=torch.float32).cuda(),
                             torch.tensor([-7, 100_000_000], dtype=torch.int32).cuda())
    d = int8.dequantize_per_channel(q, p).cpu().numpy()
    want = orc.int8_dequantize_per_channel(q.cpu().numpy(), p.scale.cpu().numpy(), p.zero_point.cpu().numpy())
    assert np.array_equal(d.view(np.uint32), want.view(np.uint32))
    layer = int8.Int8Linear(q, p)
    x = torch.from_numpy(F.Stream(3).normal(128).astype(f32)).cuda()
    y = layer(x).cpu().numpy()
    ref = orc.linear_f64(x.cpu().numpy()[None], want, None, 1, 2, 128)[0]
    mag = orc.linear_abs(x.cpu().numpy()[None], want, 1, 2, 128)[0]
    assert np.all(np.abs(y - ref) <= TOL * mag)


@pytest.mark.parametrize("mode", [int8.SYMMETRIC, int8.ASYMMETRIC])
@pytest.mark.parametrize("m,x_bf16", [(1, False), (1, True), (2, False), (3, True), (8, False), (13, True), (20, False)])
@pytest.mark.parametrize("n,k", [(64, 4096), (200, 1024), (33, 100), (5, 7), (1030, 2304)])
def test_linear_matches_dequantize_then_product(mode, m, x_bf16, n, k):
    w = _weights(n + 3 * k + m, n, k, 1 if mode else 0)
    s = F.Stream(n * k + m)
    x = s.normal(m * k).astype(f32).reshape(m, k)
    bias = s.normal(n).astype(f32)
    layer = int8.Int8Linear.from_linear(torch.from_numpy(w), torch.from_numpy(bias), mode)
    xt = torch.from_numpy(x).cuda()
    if x_bf16:
        xt = xt.to(torch.bfloat16)
        x = xt.float().cpu().numpy()
    y = layer(xt).cpu().numpy()
    q0, sc0, zp0 = orc.int8_quantize_per_channel(w, mode)
    wq = orc.int8_dequantize_per_channel(q0, sc0, zp0)
    ref = orc.linear_f64(x, wq, bias, m, n, k)
    mag = orc.linear_abs(x, wq, m, n, k) + np.abs(bias)[None]
    assert y.shape == (m, n) and np.all(np.abs(y - ref) <= TOL * mag + 1e-6)


def test_layer_interface_and_errors():
    n, k = 48, 256
    w = _weights(9, n, k)
    layer = int8.Int8Linear.from_linear(torch.from_numpy(w))
    assert (layer.out_features, layer.in_features) == (n, k)
    assert layer.memory_bytes() == n * k + 5 * n and abs(layer.compression_ratio() - n * k * 4 / (n * k + 5 * n)) < 1e-9
    x = torch.ones(2, 3, k).cuda()
    assert layer(x).shape == (2, 3, n)
    assert layer(x, out_dtype=torch.bfloat16).dtype == torch.bfloat16
    with pytest.raises(api.ShapeMismatch):
        layer(torch.ones(2, k + 1).cuda())
    q, p = int8.quantize_per_channel(torch.from_numpy(w), int8.SYMMETRIC)
    with pytest.raises(api.DataLengthMismatch):
        int8.Int8Linear(q, int8.Int8QuantParams(p.scale[:-1], p.zero_point))
    with pytest.raises(api.DataLengthMismatch):
        int8.dequantize_per_channel(q, int8.Int8QuantParams(p.scale, p.zero_point[:-1]))
    with pytest.raises(api.ShapeMismatch):
        int8.Int8Linear(q, p, torch.ones(n + 1).cuda())
    wd, _ = layer.dequantize()
    assert float((wd.cpu() - torch.from_numpy(w)).abs().max()) <= float(p.scale.max()) * 0.5 + 1e-7
