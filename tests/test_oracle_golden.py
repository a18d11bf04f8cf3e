"""Pins the CPU oracle against the reference's own known-answer tests (fixture:
tests/golden/known_answers.json, written by tests/golden/make_golden.py) and against
closed-form properties of the formats. No GPU needed."""
import numpy as np
import pytest

from nn_b200 import formats as F
from nn_b200.formats import QuantFormat as Q
from oracle import cpu as orc


def _check_segments(out, expect):
    for seg in expect:
        got = out[seg["start"]:seg["end"]]
        assert got.size == seg["end"] - seg["start"]
        if seg["tol"] == 0.0:
            assert np.all(got == np.float32(seg["value"])), (seg, got[:4])
        else:
            assert np.all(np.abs(got - seg["value"]) < seg["tol"]), (seg, got[:4])


def test_dequant_known_answers(golden):
    for case in golden["dequant"]:
        fmt = Q[case["fmt"]]
        data = np.frombuffer(bytes.fromhex(case["bytes"]), np.uint8)
        scales = np.frombuffer(bytes.fromhex(case["scales"]), np.uint8) if case["scales"] else None
        out = orc.dequantize(fmt, data, case["num_elements"], scales)
        assert out.size == case["num_elements"], case["name"]
        _check_segments(out, case["expect"])


def test_fused_matmul_known_answers(golden):
    for case in golden["matmul"]:
        fmt = Q[case["fmt"]]
        w = np.frombuffer(bytes.fromhex(case["bytes"]), np.uint8)
        x = np.array(case["x"], np.float32)
        bias = np.array(case["bias"], np.float32) if case["bias"] else None
        y = orc.quantized_linear(fmt, x, w, bias, x.shape[0], case["n"], case["k"])
        assert np.all(np.abs(y - np.array(case["expect"], np.float32)) < case["tol"]), case["name"]


def test_f16_widening_exact():
    # every binary16 pattern widens exactly as numpy's IEEE conversion does
    bits = np.arange(65536, dtype=np.uint16)
    want = bits.view(np.float16).astype(np.float32)
    got = np.array([orc.f16_to_f32(int(b)) for b in bits[::7]], np.float32)
    w = want[::7]
    nan = np.isnan(w)
    assert np.array_equal(np.isnan(got), nan)
    assert np.array_equal(got[~nan].view(np.uint32), w[~nan].view(np.uint32))


def test_short_buffer_clamps_block_count():
    # crates/nn-gguf/src/dequant.rs:123-139: a short buffer decodes only whole blocks present
    data = F.gen_q4_k(1, 1, 512)
    out = orc.dequantize(Q.Q4_K, data[:144 + 10], 512)
    assert out.size == 256
    assert np.array_equal(out, orc.dequantize(Q.Q4_K, data[:144], 256))


def _numpy_q4_k(data):
    """Independent numpy transcription of the nn-gguf Q4_K formulas."""
    blk = data.reshape(-1, 144)
    d = blk[:, 0:2].copy().view(np.float16).astype(np.float32)[:, 0]
    dmin = blk[:, 2:4].copy().view(np.float16).astype(np.float32)[:, 0]
    S = blk[:, 4:16].astype(np.uint32)
    out = np.zeros((blk.shape[0], 256), np.float32)
    for j in range(8):
        sc = ((S[:, j // 2] >> (4 * (j % 2))) & 15) | (((S[:, 8 + j // 4] >> (2 * (j % 4))) & 3) << 4)
        mn = ((S[:, 4 + j // 2] >> (4 * (j % 2))) & 15) | (((S[:, 10 + j // 4] >> (2 * (j % 4))) & 3) << 4)
        s = d * sc.astype(np.float32)
        m = dmin * mn.astype(np.float32)
        q = blk[:, 16 + 16 * j:32 + 16 * j]
        out[:, 32 * j:32 * j + 32:2] = s[:, None] * (q & 15).astype(np.float32) - m[:, None]
        out[:, 32 * j + 1:32 * j + 32:2] = s[:, None] * (q >> 4).astype(np.float32) - m[:, None]
    return out.reshape(-1)


def _numpy_q6_k(data):
    blk = data.reshape(-1, 210)
    d = blk[:, 208:210].copy().view(np.float16).astype(np.float32)[:, 0]
    sc = blk[:, 192:208].view(np.int8).astype(np.float32)
    idx = np.arange(256)
    lo4 = (blk[:, idx // 2] >> (4 * (idx % 2))) & 15
    hi2 = (blk[:, 128 + idx // 4] >> (2 * (idx % 4))) & 3
    q6 = (lo4 | (hi2 << 4)).astype(np.int32) - 32
    return ((d[:, None] * sc[:, idx // 16]) * q6.astype(np.float32)).reshape(-1)


def test_q4_k_matches_numpy_transcription():
    data = F.gen_q4_k(0x5EED, 8, 1024)
    a = orc.dequantize(Q.Q4_K, data, 8 * 1024)
    assert np.array_equal(a.view(np.uint32), _numpy_q4_k(data).view(np.uint32))


def test_q6_k_matches_numpy_transcription():
    data = F.gen_q6_k(0x5EED, 8, 1024)
    a = orc.dequantize(Q.Q6_K, data, 8 * 1024)
    assert np.array_equal(a.view(np.uint32), _numpy_q6_k(data).view(np.uint32))


def _h(blk, off):
    return blk[:, off:off + 2].copy().view(np.float16).astype(np.float32)[:, 0][:, None]


def _numpy_flat(fmt, data):
    """Independent numpy transcriptions (flat element index) of the Q5_0 / Q5_1 / Q2_K / Q3_K / Q5_K
    formulas of crates/nn-gguf/src/dequant.rs:241-316,476-684, every operation rounded to f32."""
    f = np.float32
    if fmt in (Q.Q5_0, Q.Q5_1):
        hdr = 2 if fmt == Q.Q5_0 else 4
        blk = data.reshape(-1, hdr + 20)
        idx = np.arange(32)
        qh = blk[:, hdr:hdr + 4].copy().view("<u4")
        q = ((blk[:, hdr + 4 + idx // 2] >> (4 * (idx % 2))) & 15) | (((qh >> idx) & 1) << 4).astype(np.uint8)
        if fmt == Q.Q5_0:
            return (_h(blk, 0) * (q.astype(np.int32) - 16).astype(f)).reshape(-1)
        return (_h(blk, 0) * q.astype(f) + _h(blk, 2)).reshape(-1)
    idx = np.arange(256)
    if fmt == Q.Q2_K:
        blk = data.reshape(-1, 84)
        sc = (blk[:, idx // 16] & 15).astype(f)
        mn = (blk[:, idx // 16] >> 4).astype(f)
        q = ((blk[:, 16 + idx // 4] >> (2 * (idx % 4))) & 3).astype(f)
        return ((_h(blk, 80) * sc) * q - _h(blk, 82) * mn).reshape(-1)
    if fmt == Q.Q3_K:
        blk = data.reshape(-1, 110)
        k = idx // 16
        lo4 = (blk[:, 96 + k // 2] >> (4 * (k % 2))) & 15
        hi2 = (blk[:, 104 + k // 4] >> (2 * (k % 4))) & 3
        sc = ((lo4 | (hi2 << 4)).astype(np.int32) - 32).astype(f)
        q = ((blk[:, 32 + idx // 4] >> (2 * (idx % 4))) & 3) | (((blk[:, idx // 8] >> (idx % 8)) & 1) << 2)
        return ((_h(blk, 108) * sc) * (q.astype(np.int32) - 4).astype(f)).reshape(-1)
    blk = data.reshape(-1, 176)
    S = blk[:, 4:16]
    j = idx // 32
    sc = ((S[:, j // 2] >> (4 * (j % 2))) & 15) | (((S[:, 8 + j // 4] >> (2 * (j % 4))) & 3) << 4)
    mn = ((S[:, 4 + j // 2] >> (4 * (j % 2))) & 15) | (((S[:, 10 + j // 4] >> (2 * (j % 4))) & 3) << 4)
    q = ((blk[:, 48 + idx // 2] >> (4 * (idx % 2))) & 15) | (((blk[:, 16 + idx // 8] >> (idx % 8)) & 1) << 4)
    return ((_h(blk, 0) * sc.astype(f)) * q.astype(f) - _h(blk, 2) * mn.astype(f)).reshape(-1)


@pytest.mark.parametrize("fmt", [Q.Q5_0, Q.Q5_1, Q.Q2_K, Q.Q3_K, Q.Q5_K])
def test_flat_index_formats_match_numpy_transcription(fmt):
    data, _ = F.gen_weight(fmt, 0x5EED + int(fmt), 8, 1024)
    assert data.size == 8 * 1024 // F.GEOMETRY[fmt].elems * F.GEOMETRY[fmt].bytes
    a = orc.dequantize(fmt, data, 8 * 1024)
    assert a.size == 8 * 1024 and np.all(np.isfinite(a))
    assert np.array_equal(a.view(np.uint32), _numpy_flat(fmt, data).view(np.uint32))
    # a short buffer decodes only its whole blocks (validate_dequant_input, dequant.rs:123-139)
    g = F.GEOMETRY[fmt]
    short = orc.dequantize(fmt, data[:3 * g.bytes + 5], 8 * 1024)
    assert short.size == 3 * g.elems and np.array_equal(short, a[:3 * g.elems])


def test_q4_k_ggml_variant_differs_only_in_order_and_packing():
    # A block whose 12 scale bytes hold 6-bit values below 16 in bytes 0..7 and zero in
    # bytes 8..11 decodes, under the GGML packing, to sc_j = S[j], m_j = S[j+4] for j<4
    # (crates/nn-core/src/layers/quantized/linear.rs:166-176).
    b = np.zeros(144, np.uint8)
    b[0:2] = np.frombuffer(np.float16(1.0).tobytes(), np.uint8)
    b[2:4] = np.frombuffer(np.float16(0.5).tobytes(), np.uint8)
    b[4:8] = [1, 2, 3, 4]
    b[8:12] = [5, 6, 7, 8]
    b[16:144] = 0x21  # low nibble 1, high nibble 2
    out = orc.dequantize(Q.Q4_K_GGML, b, 256)
    # group g: first 32 use (sc,m)_{2g} with low nibbles, next 32 use (sc,m)_{2g+1} with high nibbles
    assert np.all(out[0:32] == 1.0 * 1 * 1 - 0.5 * 5)
    assert np.all(out[32:64] == 1.0 * 2 * 2 - 0.5 * 6)
    assert np.all(out[64:96] == 1.0 * 3 * 1 - 0.5 * 7)
    assert np.all(out[96:128] == 1.0 * 4 * 2 - 0.5 * 8)
    assert np.all(out[128:] == 0.0)


def test_mxfp4_exponent_zero_rules():
    # nn-core: 2^-127 (f32 subnormal); nn-gptoss: 2^-126 (crates/nn-gptoss/src/quantize.rs:84-90)
    assert orc.lib().orc_mxfp4_core_scale(0) == np.float32(2.0 ** -127)
    assert orc.lib().orc_mxfp4_gptoss_scale(0) == np.float32(2.0 ** -126)
    for e in range(1, 255):
        assert orc.lib().orc_mxfp4_core_scale(e) == orc.lib().orc_mxfp4_gptoss_scale(e) == np.float32(2.0 ** (e - 127))


def test_mxfp4_layouts_agree_in_benchmark_exponent_range():
    codes, exps = F.gen_mxfp4(7, 4, 256)
    core = orc.dequantize(Q.MXFP4_CORE, F.mxfp4_core_bytes(codes, exps), 4 * 256)
    split = orc.dequantize(Q.MXFP4_SPLIT, codes, 4 * 256, exps)
    assert np.array_equal(core.view(np.uint32), split.view(np.uint32))
    # the nn-gptoss layout reads the same bytes with the nibbles of each byte swapped
    swapped = ((codes << 4) | (codes >> 4)).astype(np.uint8)
    gpt = orc.dequantize(Q.MXFP4_GPTOSS, swapped, 4 * 256, exps)
    assert np.array_equal(core.view(np.uint32), gpt.view(np.uint32))


@pytest.mark.parametrize("fmt", [Q.Q4_0, Q.Q8_0])
def test_fused_product_close_to_dequant_then_matmul(fmt):
    # crates/nn-core/src/dyn_tensor/quantized_matmul_tests.rs:421-491: within 1e-3 absolute
    n, k, m = 16, 256, 3
    w, _ = F.gen_weight(fmt, 11, n, k)
    x = F.gen_activations(12, m, k, bf16=False)
    fused = orc.quantized_linear(fmt, x, w, None, m, n, k)
    deq = orc.dequantize(fmt, w, n * k).reshape(n, k)
    ref = orc.linear_f32(x, deq, None, m, n, k)
    assert np.max(np.abs(fused - ref)) < 1e-3


def test_nncpu_dot_close_to_sequential():
    n, k, m = 32, 4096, 2
    w = F.Stream(3).normal(n * k).astype(np.float32).reshape(n, k) * 0.02
    x = F.gen_activations(4, m, k, bf16=False)
    a = orc.nncpu_linear(x, w, None, m, n, k, threads=2)
    b = orc.linear_f64(x, w, None, m, n, k)
    scale = orc.linear_abs(x, w, m, n, k)
    assert np.max(np.abs(a - b) / scale) < 1e-6


def test_cpu_forward_equals_dequant_then_nncpu():
    n, k, m = 32, 512, 1
    w = F.gen_q4_k(5, n, k)
    x = F.gen_activations(6, m, k, bf16=True)
    y = orc.cpu_forward(Q.Q4_K, w, x, None, m, n, k, threads=2)
    deq = orc.dequantize(Q.Q4_K, w, n * k).reshape(n, k)
    assert np.array_equal(y, orc.nncpu_linear(x, deq, None, m, n, k))


def test_moe_route_orders_and_renormalises():
    logits = np.array([0.1, 2.0, -1.0, 1.5, 0.7, 0.3], np.float32)
    idx, w = orc.moe_route(logits, 3)
    assert list(idx) == [1, 3, 4]
    p = np.exp(logits - logits.max())
    p /= p.sum()
    want = p[[1, 3, 4]] / p[[1, 3, 4]].sum()
    assert np.allclose(w, want, rtol=1e-6)
    assert abs(w.sum() - 1.0) < 1e-6
