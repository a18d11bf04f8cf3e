"""INT4 / INT8 per-group weights and GPTQ / AWQ packed weights on the GPU against the oracle:
codes, scales, zero points and decoded weights bit for bit; products within the f32 bar on the
streaming kernels and within the bf16 bar on the tensor-core path. The reference's own cases
(weight_quant_tests.rs, gptq_awq_tests.rs) run through the mirror of its API."""
import numpy as np
import pytest

torch = pytest.importorskip("torch")

from nn_b200 import api, gptq
from nn_b200 import weight_quant as wq
from oracle import cpu as orc
from tests import parity as P

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
f32 = np.float32


def _weights(seed, n, k, kind="normal"):
    rng = np.random.default_rng(seed)
    if kind == "normal":
        return (rng.standard_normal((n, k)) * 0.05).astype(f32)
    if kind == "shifted":      # far from zero: large asymmetric zero points
        return (rng.random((n, k)) * 0.01 + 3.0).astype(f32)
    return (np.arange(n * k, dtype=f32) / f32(n * k - 1) * f32(2.0) - f32(1.0)).reshape(n, k)


def _cfg(bits, g, sym=True):
    return wq.QuantizationConfig(wq.QuantDtype.Int4 if bits == 4 else wq.QuantDtype.Int8, g, sym)


@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("sym", [True, False])
@pytest.mark.parametrize("n,k,g,kind", [(4, 128, 128, "ramp"), (4, 128, 32, "ramp"), (64, 1024, 128, "normal"),
                                        (3, 96, 8, "normal"), (3, 5, 5, "normal"), (7, 33, 11, "shifted"),
                                        (16, 512, 64, "shifted"), (1, 4096, 256, "normal")])
def test_quantize_and_dequantize_match_the_oracle_bit_for_bit(bits, sym, n, k, g, kind):
    w = _weights(n * 31 + k, n, k, kind)
    w[0, : min(g, k)] = 0.0 if kind == "normal" else w[0, 0]     # an all-zero (or constant) group: scale 0
    q_ref, sc_ref, zp_ref = orc.group_quantize(w, bits, g, sym)
    qt = wq.quantize_per_group(torch.from_numpy(w), _cfg(bits, g, sym))
    assert np.array_equal(qt.quantized_data.cpu().numpy(), q_ref)
    assert np.array_equal(qt.scales.cpu().numpy().view(np.uint32), sc_ref.view(np.uint32))
    assert np.array_equal(qt.zero_points.cpu().numpy(), zp_ref)
    want = orc.group_dequantize(q_ref, sc_ref, zp_ref, n, k, bits, g)
    got = wq.dequantize(qt).cpu().numpy()
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    # the resident operand decodes to the same bits
    got2 = qt.device_weight().dequantize().cpu().numpy()
    assert np.array_equal(got2.view(np.uint32), want.view(np.uint32))
    qt.release()


def test_reference_round_trip_cases():
    ramp = _weights(0, 4, 128, "ramp")
    for bits, g, sym, tol in ((4, 128, True, 0.10), (4, 32, True, 0.10), (8, 128, True, 0.02), (4, 128, False, 0.2)):
        qt = wq.quantize_per_group(torch.from_numpy(ramp), _cfg(bits, g, sym))
        assert qt.shape == [4, 128] and qt.scales.numel() == 4 * (128 // g) and qt.zero_points.numel() == 4 * (128 // g)
        assert float((wq.dequantize(qt).cpu() - torch.from_numpy(ramp)).abs().max()) < tol
    z = wq.quantize_per_group(torch.zeros(4, 128), wq.QuantizationConfig.int4(128))
    assert bool((z.scales == 0).all()) and bool((wq.dequantize(z) == 0).all())
    c = wq.quantize_per_group(torch.full((4, 128), 0.5), wq.QuantizationConfig.int4(128))
    assert float((wq.dequantize(c) - 0.5).abs().max()) < 0.01
    i4 = wq.quantize_per_group(torch.from_numpy(ramp), wq.QuantizationConfig.int4(128))
    i8 = wq.quantize_per_group(torch.from_numpy(ramp), wq.QuantizationConfig.int8(128))
    assert i4.memory_bytes() < i8.memory_bytes() and i4.compression_ratio() > 4.0 and i8.compression_ratio() > 3.0
    assert wq.QuantizationConfig().dtype == wq.QuantDtype.Int4 and wq.QuantizationConfig().group_size == 128
    assert wq.QuantDtype.Int4.bits() == 4 and wq.QuantDtype.Int8.bits() == 8


def test_quantize_error_cases():
    w = torch.zeros(4, 128)
    w[2, 5] = float("nan")
    with pytest.raises(api.ValueOutOfRange):
        wq.quantize_per_group(w, wq.QuantizationConfig.int4(128))
    w[2, 5] = float("inf")
    with pytest.raises(api.ValueOutOfRange):
        wq.quantize_per_group(w, wq.QuantizationConfig.int8(128))
    with pytest.raises(api.ShapeMismatch):
        wq.quantize_per_group(torch.zeros(4, 100), wq.QuantizationConfig.int4(128))
    with pytest.raises(api.ValueOutOfRange):
        wq.quantize_per_group(torch.zeros(4, 128), wq.QuantizationConfig.int4(0))
    qt = wq.quantize_per_group(torch.zeros(4, 128), wq.QuantizationConfig.int4(128))
    with pytest.raises(api.ShapeMismatch):
        wq.quantized_matmul(torch.ones(2, 64, device=DEV), qt)
    api.gpu_backend().device_status()


def _check_product(got, x, deq, bias, m, n, k, tensor_path):
    y32 = orc.linear_f32(x, deq, bias, m, n, k)
    y64 = orc.linear_f64(x, deq, bias, m, n, k)
    mag = orc.linear_abs(x, deq, m, n, k)
    if bias is not None:
        mag = mag + np.abs(bias)[None, :]
    if tensor_path:
        assert np.all(np.isfinite(got))
        assert P.max_scaled_err(got, y64, mag) <= P.TOL_BF16_MMA
    else:
        P.assert_close(got, y32, y64, mag)


@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("m,x_bf16", [(1, False), (1, True), (2, True), (3, False), (4, True), (7, False), (16, True)])
@pytest.mark.parametrize("n,k,g,sym", [(200, 2048, 128, True), (67, 1024, 32, False), (1030, 4096, 64, True), (9, 32, 8, False)])
def test_quantized_matmul_streaming_kernel(bits, m, x_bf16, n, k, g, sym):
    w = _weights(n + k + bits, n, k)
    qt = wq.quantize_per_group(torch.from_numpy(w), _cfg(bits, g, sym))
    assert qt.device_weight().streaming
    x = (np.random.default_rng(m).standard_normal((m, k))).astype(f32)
    xt = torch.from_numpy(x).to(DEV)
    if x_bf16:
        xt = xt.to(torch.bfloat16)
        x = xt.float().cpu().numpy()
    y = wq.quantized_matmul(xt, qt)
    torch.cuda.synchronize()
    qt.backend.device_status()
    deq = orc.group_dequantize(*orc.group_quantize(w, bits, g, sym), n, k, bits, g)
    _check_product(y.cpu().numpy(), x, deq, None, m, n, k, False)
    qt.release()


@pytest.mark.parametrize("bits,n,k,g,sym,kind", [(4, 9, 40, 5, True, "normal"), (8, 5, 33, 11, False, "normal"), (4, 3, 5, 5, False, "normal"),
                                                 (4, 16, 512, 64, False, "shifted"), (8, 16, 512, 64, False, "shifted")])
def test_quantized_matmul_elementwise_kernel(bits, n, k, g, sym, kind):
    """Group sizes and widths off the 8-weight grid, rows that straddle bytes, and zero points too
    wide for the mantissa trick take the element-wise kernel."""
    w = _weights(5, n, k, kind)
    if kind == "shifted":
        w = w + f32(1.0e4)        # zero points beyond 4e6
    qt = wq.quantize_per_group(torch.from_numpy(w), _cfg(bits, g, sym))
    assert not qt.device_weight().streaming
    for m in (1, 3):
        x = np.random.default_rng(m).standard_normal((m, k)).astype(f32)
        y = wq.quantized_matmul(torch.from_numpy(x).to(DEV), qt)
        torch.cuda.synchronize()
        qt.backend.device_status()
        deq = orc.group_dequantize(*orc.group_quantize(w, bits, g, sym), n, k, bits, g)
        _check_product(y.cpu().numpy(), x, deq, None, m, n, k, False)
    qt.release()


@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("m,x_bf16,y_bf16", [(17, True, False), (64, False, False), (300, True, True), (1000, True, False)])
def test_quantized_matmul_large_batches_take_the_tensor_cores(bits, m, x_bf16, y_bf16):
    n, k, g = 520, 1024, 128
    w = _weights(m, n, k)
    qt = wq.quantize_per_group(torch.from_numpy(w), _cfg(bits, g, False))
    x = np.random.default_rng(m).standard_normal((m, k)).astype(f32)
    xt = torch.from_numpy(x).to(DEV)
    if x_bf16:
        xt = xt.to(torch.bfloat16)
        x = xt.float().cpu().numpy()
    y = wq.quantized_matmul(xt, qt, out_dtype=torch.bfloat16 if y_bf16 else torch.float32)
    torch.cuda.synchronize()
    qt.backend.device_status()
    deq = orc.group_dequantize(*orc.group_quantize(w, bits, g, False), n, k, bits, g)
    _check_product(y.float().cpu().numpy(), x, deq, None, m, n, k, True)
    qt.release()


def test_reference_matmul_cases():
    w = ((np.arange(512) % 17).astype(f32) / f32(16.0) * f32(0.3) - f32(0.15)).reshape(4, 128)
    x = torch.ones(2, 128, device=DEV)
    ref = np.ones((2, 128), f32) @ w.T
    for cfg, tol in ((wq.QuantizationConfig.int4(128), 2.0), (wq.QuantizationConfig.int8(128), 0.5)):
        y = wq.quantized_matmul(x, wq.quantize_per_group(torch.from_numpy(w), cfg))
        assert tuple(y.shape) == (2, 4) and np.max(np.abs(y.cpu().numpy() - ref)) < tol
    qt = wq.quantize_per_group(torch.full((4, 128), 0.1), wq.QuantizationConfig.int4(128))
    assert tuple(wq.quantized_matmul(torch.ones(2, 3, 128, device=DEV), qt).shape) == (2, 3, 4)


def _pack8(vals):
    p = 0
    for i, v in enumerate(vals):
        p |= (int(v) & 0xF) << (4 * i)
    return p


def _words(a):
    return torch.from_numpy(np.asarray(a, np.uint32).view(np.int32))


def test_gptq_unpack_and_dequantize_reference_cases():
    out = gptq.unpack_gptq_qweight(_words([[_pack8([1, 2, 3, 4, 5, 6, 7, 8])]]))
    assert tuple(out.shape) == (8, 1) and out.dtype == torch.float32 and out[:, 0].tolist() == [1, 2, 3, 4, 5, 6, 7, 8]
    assert bool((gptq.unpack_gptq_qweight(_words([[0]])) == 0).all())
    assert bool((gptq.unpack_gptq_qweight(_words([[0xFFFFFFFF]])) == 15).all())
    two = gptq.unpack_gptq_qweight(_words([[_pack8(range(8)), _pack8(range(8, 16))]]))
    assert tuple(two.shape) == (8, 2) and two[:, 0].tolist() == list(range(8)) and two[:, 1].tolist() == list(range(8, 16))
    assert gptq.unpack_awq_qweight(_words([[_pack8([3, 7, 11, 15, 0, 4, 8, 12])]]))[:, 0].tolist() == [3, 7, 11, 15, 0, 4, 8, 12]
    z = gptq.unpack_gptq_qzeros(_words([[_pack8([8] * 8)]]))
    assert tuple(z.shape) == (1, 8) and bool((z == 8).all())
    d = gptq.dequantize_gptq(torch.full((8, 8), 8.0), torch.full((1, 8), 0.1), torch.full((1, 8), 8.0), 8)
    assert tuple(d.shape) == (8, 8) and float(d.abs().max()) < 1e-6
    d = gptq.dequantize_gptq(torch.full((8, 8), 10.0), torch.full((1, 8), 0.5), torch.full((1, 8), 8.0), 8)
    assert float((d - 1.0).abs().max()) < 1e-6
    with pytest.raises(api.DataLengthMismatch):
        gptq.dequantize_gptq(torch.zeros(16, 8), torch.ones(1, 8), torch.zeros(1, 8), 8)
    # random words against the oracle, bit for bit
    rng = np.random.default_rng(3)
    qw = rng.integers(0, 2 ** 32, size=(12, 40), dtype=np.uint64).astype(np.uint32)
    assert np.array_equal(gptq.unpack_gptq_qweight(_words(qw)).cpu().numpy(), orc.gptq_unpack_qweight(qw))
    assert np.array_equal(gptq.unpack_gptq_qzeros(_words(qw)).cpu().numpy(), orc.gptq_unpack_qzeros(qw))


def test_gptq_linear_from_a_dense_weight_reference_cases():
    lin = gptq.GptqLinear(torch.eye(16, 8), None, gptq.GptqFormat())
    assert tuple(lin(torch.ones(2, 8, device=DEV)).shape) == (2, 16)
    lin = gptq.GptqLinear(torch.eye(4), torch.full((4,), 10.0))
    assert np.allclose(lin(torch.tensor([[1.0, 2.0, 3.0, 4.0]], device=DEV)).cpu().numpy(), [[11.0, 12.0, 13.0, 14.0]], atol=1e-5)
    lin = gptq.GptqLinear(torch.full((4, 8), 0.1))
    assert tuple(lin(torch.ones(2, 3, 8, device=DEV)).shape) == (2, 3, 4)
    with pytest.raises(api.ShapeMismatch):
        lin(torch.ones(2, 7, device=DEV))
    with pytest.raises(api.ShapeMismatch):
        gptq.GptqLinear(torch.eye(4), torch.zeros(5))


@pytest.mark.parametrize("loader", [gptq.load_gptq_linear, gptq.load_awq_linear])
@pytest.mark.parametrize("rows,g,qv,zv,scale,want", [(1, 8, 10, 8, 0.5, 8.0), (4, 32, 10, 8, 0.5, 32.0), (16, 128, 5, 0, 1.0, 640.0)])
def test_load_then_forward_reference_cases(loader, rows, g, qv, zv, scale, want):
    qweight = _words(np.full((rows, 8), _pack8([qv] * 8), np.uint32))
    lin = loader(qweight, torch.full((1, 8), scale), _words([[_pack8([zv] * 8)]]), None, g)
    assert lin.out_features == 8 and lin.in_features == rows * 8 and lin.format.group_size == g
    y = lin(torch.ones(1, rows * 8, device=DEV))
    assert float((y - want).abs().max()) < 1e-2
    lin.release()


@pytest.mark.parametrize("k,n,g", [(256, 64, 64), (4096, 512, 128), (1024, 72, 32), (24, 8, 5), (40, 16, 8), (2048, 200, 128)])
def test_gptq_packed_weight_and_product_match_the_oracle(k, n, g):
    rng = np.random.default_rng(k + n)
    groups = (k + g - 1) // g
    qweight = rng.integers(0, 2 ** 32, size=(k // 8, n), dtype=np.uint64).astype(np.uint32)
    qzeros = rng.integers(0, 2 ** 32, size=(groups, n // 8), dtype=np.uint64).astype(np.uint32)
    scales = (rng.random((groups, n)) * 0.02 + 0.001).astype(f32)
    bias = rng.standard_normal(n).astype(f32)
    lin = gptq.load_gptq_linear(_words(qweight), torch.from_numpy(scales), _words(qzeros), torch.from_numpy(bias), g)
    w_ref = orc.gptq_load_weight(qweight, scales, qzeros, g)
    assert np.array_equal(lin.weight().cpu().numpy().view(np.uint32), w_ref.view(np.uint32))
    for m, x_bf16 in ((1, False), (1, True), (5, True), (16, False), (40, True), (300, True)):
        x = rng.standard_normal((m, k)).astype(f32)
        xt = torch.from_numpy(x).to(DEV)
        if x_bf16:
            xt = xt.to(torch.bfloat16)
            x = xt.float().cpu().numpy()
        y = lin(xt)
        torch.cuda.synchronize()
        lin.backend.device_status()
        _check_product(y.cpu().numpy(), x, w_ref, bias, m, n, k, tensor_path=(m > 16 and k % 64 == 0))
    lin.release()


def test_gptq_shape_errors():
    with pytest.raises(api.DataLengthMismatch):     # two groups of scales for one group of in-features
        gptq.load_gptq_linear(_words(np.zeros((1, 8), np.uint32)), torch.ones(2, 8), _words(np.zeros((2, 1), np.uint32)), None, 8)
    with pytest.raises(api.ShapeMismatch):
        gptq.load_gptq_linear(_words(np.zeros((1, 8), np.uint32)), torch.ones(1, 16), _words(np.zeros((1, 1), np.uint32)), None, 8)
    with pytest.raises(api.RankMismatch):
        gptq.unpack_gptq_qweight(_words(np.zeros(8, np.uint32)))
