"""GPU dequantization is bit-identical to the oracle (memcmp of f32), through the C ABI:
the reference's known-answer blocks, seeded random tensors of every format, short
buffers, and special scale values."""
import ctypes

import numpy as np
import pytest

torch = pytest.importorskip("torch")

from nn_b200 import api
from nn_b200 import formats as F
from nn_b200.formats import QuantFormat as Q
from oracle import cpu as orc

pytestmark = pytest.mark.gpu


def _same_bits(a: np.ndarray, b: np.ndarray):
    a = np.ascontiguousarray(a, np.float32).reshape(-1)
    b = np.ascontiguousarray(b, np.float32).reshape(-1)
    assert a.size == b.size
    bad = np.nonzero(a.view(np.uint32) != b.view(np.uint32))[0]
    assert bad.size == 0, (bad[:8], a[bad[:8]], b[bad[:8]])


def _raw_dequant(fmt, data, scales, num_elements):
    b = api.gpu_backend()
    dev = torch.device("cuda", b.device)
    src = torch.from_numpy(np.ascontiguousarray(data)).to(dev)
    sc = torch.from_numpy(np.ascontiguousarray(scales)).to(dev) if scales is not None else None
    out = torch.full((max(num_elements, 1),), float("nan"), dtype=torch.float32, device=dev)
    n = ctypes.c_int64(-1)
    b.check(b._lib.nnq_dequantize_raw(b._ctx, int(fmt), src.data_ptr() if src.numel() else None, src.numel(),
                                      sc.data_ptr() if sc is not None else None,
                                      sc.numel() if sc is not None else 0, num_elements, out.data_ptr(),
                                      ctypes.byref(n), None))
    torch.cuda.synchronize()
    return out.cpu().numpy(), n.value


def test_known_answer_blocks(golden):
    for case in golden["dequant"]:
        fmt = Q[case["fmt"]]
        data = np.frombuffer(bytes.fromhex(case["bytes"]), np.uint8)
        scales = np.frombuffer(bytes.fromhex(case["scales"]), np.uint8) if case["scales"] else None
        out, n = _raw_dequant(fmt, data, scales, case["num_elements"])
        assert n == case["num_elements"], case["name"]
        for seg in case["expect"]:
            got = out[seg["start"]:seg["end"]]
            if seg["tol"] == 0.0:
                assert np.all(got == np.float32(seg["value"])), case["name"]
            else:
                assert np.all(np.abs(got - seg["value"]) < seg["tol"]), case["name"]
        _same_bits(out[:n], orc.dequantize(fmt, data, case["num_elements"], scales))


@pytest.mark.parametrize("fmt", list(Q))
@pytest.mark.parametrize("n,k", [(1, 256), (3, 512), (48, 4096), (17, 1280)])
def test_weight_dequant_bit_exact(fmt, n, k):
    w, sc = F.gen_weight(fmt, 0x5EED + int(fmt), n, k)
    t = api.from_quantized(w, fmt, [n, k], sc)
    got = t.dequantize().cpu().numpy()
    _same_bits(got, orc.dequantize(fmt, w, n * k, sc))
    t.release()


@pytest.mark.parametrize("fmt", [Q.Q8_0, Q.Q4_K, Q.Q6_K])
def test_full_size_tensor_bit_exact(fmt):
    # one Qwen3-8B projection at full size: q_proj 4096 x 4096
    n = k = 4096
    w, sc = F.gen_weight(fmt, 77, n, k)
    t = api.from_quantized(w, fmt, [n, k], sc)
    got = t.dequantize().cpu().numpy()
    _same_bits(got, orc.dequantize(fmt, w, n * k, sc))
    t.release()


def test_short_buffer_decodes_whole_blocks_only():
    # crates/nn-gguf/src/dequant.rs:123-139
    data = F.gen_q4_k(3, 1, 1024)
    out, n = _raw_dequant(Q.Q4_K, data[:2 * 144 + 100], None, 1024)
    assert n == 512
    _same_bits(out[:512], orc.dequantize(Q.Q4_K, data[:288], 512))
    assert np.all(np.isnan(out[512:]))  # nothing written past the decoded blocks
    out, n = _raw_dequant(Q.Q8_0, F.gen_q8_0(4, 1, 64)[:33], None, 64)
    assert n == 0
    out, n = _raw_dequant(Q.Q6_K, np.zeros(0, np.uint8), None, 0)
    assert n == 0


def test_special_scales():
    # f16 subnormal / inf / nan scales widen exactly; MXFP4 exponent 0, 254, 255
    blk = np.zeros((4, 34), np.uint8)
    for i, bits in enumerate((0x0001, 0x03FF, 0x7C00, 0xFC00)):
        blk[i, 0] = bits & 0xFF
        blk[i, 1] = bits >> 8
        blk[i, 2:] = np.arange(32, dtype=np.uint8) - 16
    out, _ = _raw_dequant(Q.Q8_0, blk.reshape(-1), None, 128)
    ref = orc.dequantize(Q.Q8_0, blk.reshape(-1), 128)
    assert np.array_equal(np.isnan(out), np.isnan(ref))
    ok = ~np.isnan(ref)
    _same_bits(out[ok], ref[ok])
    codes = np.tile(np.arange(16, dtype=np.uint8) | (np.arange(16, dtype=np.uint8)[::-1] << 4), 3).reshape(3, 16)
    exps = np.array([0, 254, 255], np.uint8).reshape(3, 1)
    core = F.mxfp4_core_bytes(codes, exps)
    for fmt, data, sc in ((Q.MXFP4_CORE, core, None), (Q.MXFP4_SPLIT, codes.reshape(-1), exps.reshape(-1)),
                          (Q.MXFP4_GPTOSS, codes.reshape(-1), exps.reshape(-1))):
        out, _ = _raw_dequant(fmt, data, sc, 96)
        ref = orc.dequantize(fmt, data, 96, sc)
        nan = np.isnan(ref)  # 0 * inf
        assert np.array_equal(np.isnan(out), nan)
        _same_bits(out[~nan], ref[~nan])


def test_dequantize_then_checksum_is_linear_in_blocks():
    # size-independent property: decoding a concatenation equals concatenating decodes
    a = F.gen_q6_k(10, 2, 512)
    b = F.gen_q6_k(11, 3, 512)
    ab, _ = _raw_dequant(Q.Q6_K, np.concatenate([a, b]), None, 5 * 512)
    oa, _ = _raw_dequant(Q.Q6_K, a, None, 2 * 512)
    ob, _ = _raw_dequant(Q.Q6_K, b, None, 3 * 512)
    _same_bits(ab, np.concatenate([oa, ob]))
