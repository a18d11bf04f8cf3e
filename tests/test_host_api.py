"""Host-side mirror of the reference's op API: validation and error behaviour that is
decided before any device work (crates/nn-core/src/dyn_tensor/quantized_tests.rs size
validation; quantized_matmul_tests.rs:205-270 error cases). Runs without a GPU."""
import numpy as np
import pytest

from nn_b200 import api
from nn_b200 import formats as F
from nn_b200.formats import QuantFormat as Q


def test_from_quantized_rejects_partial_block():
    with pytest.raises(api.InvalidShape):
        api.from_quantized(np.zeros(34, np.uint8), Q.Q8_0, [1, 31])
    with pytest.raises(api.InvalidShape):
        api.from_quantized(np.zeros(144, np.uint8), Q.Q4_K, [1, 255])


def test_from_quantized_rejects_wrong_byte_length():
    with pytest.raises(api.DataLengthMismatch):
        api.from_quantized(np.zeros(33, np.uint8), Q.Q8_0, [1, 32])
    with pytest.raises(api.DataLengthMismatch):
        api.from_quantized(np.zeros(2 * 18 + 1, np.uint8), Q.Q4_0, [2, 32])
    with pytest.raises(api.DataLengthMismatch):  # split MXFP4 needs its exponent bytes
        api.from_quantized(np.zeros(16, np.uint8), Q.MXFP4_SPLIT, [1, 32])


def test_from_quantized_accepts_empty_and_reports_shape():
    t = api.from_quantized(b"", Q.Q8_0, [0, 32])
    assert t.is_quantized() and t.dims() == (0, 32) and t.rank() == 2
    w, _ = F.gen_weight(Q.Q4_K, 1, 4, 512)
    t = api.from_quantized(w, Q.Q4_K, [4, 512])
    assert t.dims() == (4, 512)


def test_matmul_rejects_non_quantized_weight():
    x = np.ones((1, 32), np.float32)
    with pytest.raises(api.NotQuantized):
        api.quantized_matmul_q8_0(x, np.ones((2, 32), np.float32))
    with pytest.raises(api.Unsupported):
        api.quantized_linear(x, np.ones((2, 32), np.float32))


def test_matmul_rejects_wrong_quant_type():
    w, _ = F.gen_weight(Q.Q8_0, 1, 2, 32)
    t = api.from_quantized(w, Q.Q8_0, [2, 32])
    with pytest.raises(api.WrongQuantType):
        api.quantized_matmul_q4_0(np.ones((1, 32), np.float32), t)


def test_matmul_rejects_non_2d_weight():
    w, _ = F.gen_weight(Q.Q8_0, 1, 4, 32)
    t = api.from_quantized(w, Q.Q8_0, [2, 2, 32])
    with pytest.raises(api.WeightRank):
        api.quantized_matmul_q8_0(np.ones((1, 32), np.float32), t)


def test_errors_are_unsupported_subclasses():
    # QuantizedMatmulError converts into TensorError::Unsupported
    for e in (api.NotQuantized, api.WrongQuantType, api.ShapeMismatch, api.WeightRank, api.BiasMismatch):
        assert issubclass(e, api.Unsupported) and issubclass(e, api.TensorError)


def test_generators_are_deterministic_and_sized():
    for fmt in Q:
        a, sa = F.gen_weight(fmt, 42, 4, 512)
        b, sb = F.gen_weight(fmt, 42, 4, 512)
        assert np.array_equal(a, b)
        nb, ns = F.weight_nbytes(fmt, 4, 512)
        assert a.size == nb and (sa.size if sa is not None else 0) == ns
    x = F.gen_activations(9, 3, 64, bf16=True)
    assert np.array_equal(F.bf16_bits_to_f32(F.to_bf16_bits(x)).reshape(3, 64), x)
    assert abs(float(F.Stream(1).normal(100000).std()) - 1.0) < 0.02


def test_algorithmic_bytes_table():
    # Q4_K 4096->4096, M=1, bf16 in/out: 9 437 184 + 8 192 + 8 192
    assert F.algorithmic_bytes(Q.Q4_K, 1, 4096, 4096, 2, 2) == 9453568
    assert F.algorithmic_bytes(Q.Q8_0, 1, 4096, 4096, 4, 4) == 17858560
    assert F.algorithmic_bytes(Q.Q4_K, 1, 12288, 4096, 2, 2) == 28344320
