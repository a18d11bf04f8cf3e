"""GPU product parity against the oracle, through the C ABI: every format, skinny and
ragged M, f32 / bf16 activations and outputs, bias, batch call, host entry point, shards.
Tolerance: max relative error 2e-3 (f32 accumulation), the bar the task sets."""
import numpy as np
import pytest

torch = pytest.importorskip("torch")

from nn_b200 import api
from nn_b200 import formats as F
from nn_b200.formats import QuantFormat as Q
from oracle import cpu as orc
from tests import parity as P

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


def _run(fmt, n, k, m, x_bf16, y_bf16, with_bias, seed=1, path=api.PATH_AUTO):
    w, sc = F.gen_weight(fmt, seed, n, k)
    x = F.gen_activations(seed + 1, m, k, bf16=x_bf16)
    bias = (F.Stream(seed + 2).normal(n) * 0.5).astype(np.float32) if with_bias else None
    t = api.from_quantized(w, fmt, [n, k], sc)
    t.backend.set_path(path)
    try:
        xt = torch.from_numpy(x).to(DEV)
        if x_bf16:
            xt = xt.to(torch.bfloat16)
        bt = torch.from_numpy(bias).to(DEV) if with_bias else None
        y = api.quantized_linear(xt, t, bt, out_dtype=torch.bfloat16 if y_bf16 else torch.float32)
        torch.cuda.synchronize()
        t.backend.device_status()
    finally:
        t.backend.set_path(api.PATH_AUTO)
    y32, y64, mag = P.oracle_linear(fmt, w, sc, x, bias, n, k)
    got = y.float().cpu().numpy()
    tiled = (fmt in (Q.Q4_K, Q.Q4_K_GGML, Q.Q8_0, Q.Q6_K, Q.Q4_0, Q.Q4_1) and k % 256 == 0) or (
        fmt in (Q.MXFP4_CORE, Q.MXFP4_SPLIT) and (k % 256 == 0 or k % 192 == 0))
    skinny = tiled and 1 <= m <= 16 and (x_bf16 or m <= 8 or (m == 1 and fmt in (Q.Q4_K, Q.Q4_K_GGML)))
    tensor_path = path == api.PATH_TENSOR or (
        path == api.PATH_AUTO and not skinny and k % 64 == 0 and (m > 16 or (m >= 5 and x_bf16)))
    if tensor_path:
        # weights (and f32 activations) are rounded to bf16 for the tensor cores: 1e-2 bar
        assert np.all(np.isfinite(got))
        assert P.max_rel_err(got, y32) <= P.TOL_BF16_MMA, P.max_rel_err(got, y32)
        assert P.max_scaled_err(got, y64, mag) <= P.TOL_BF16_MMA
    elif y_bf16:
        # output rounding to bf16 adds half an ulp (2^-9 relative) on top of the f32 bar
        assert P.max_rel_err(got, y32) <= P.TOL_F32_ACC + 2.0 ** -9
        ref_b = F.bf16_bits_to_f32(F.to_bf16_bits(y32)).reshape(y32.shape)
        ulp = np.maximum(np.abs(ref_b), 1e-30) * 2.0 ** -7
        assert np.all(np.abs(got - ref_b) <= ulp + P.TOL_F32_ACC * mag)
    else:
        P.assert_close(got, y32, y64, mag)
    t.release()
    return got


@pytest.mark.parametrize("fmt", [Q.Q4_K, Q.Q4_K_GGML])
@pytest.mark.parametrize("m", [2, 3, 7, 8, 9, 16])
@pytest.mark.parametrize("n,k", [(200, 2048), (64, 4096), (1030, 2304)])
def test_token_column_skinny_kernel(fmt, m, n, k):
    """2..16 tokens of bf16 activations on the tiled Q4_K layout: ragged row tiles, token counts
    on both sides of the 8-column boundary, K not a multiple of 8 super-blocks per warp."""
    _run(fmt, n, k, m, x_bf16=True, y_bf16=(m % 2 == 0), with_bias=(m % 3 == 0), seed=300 + m, path=api.PATH_SKINNY)


@pytest.mark.parametrize("fmt", [Q.Q8_0, Q.Q6_K, Q.Q4_K, Q.Q4_0, Q.Q4_1])
@pytest.mark.parametrize("m,x_bf16", [(1, True), (1, False), (2, True), (5, False), (8, True), (8, False), (9, True), (16, True)])
@pytest.mark.parametrize("n,k", [(200, 2048), (64, 4096), (1030, 2304), (40, 512)])
def test_token_column_kernel_formats(fmt, m, x_bf16, n, k):
    """Q8_0 / Q6_K / Q4_K tiles, bf16 and f32 activations (the latter as two bf16 terms), ragged
    row tiles, K smaller than the 8-way warp split."""
    if fmt == Q.Q4_K and m == 1:
        pytest.skip("M = 1 Q4_K has its own kernel")
    _run(fmt, n, k, m, x_bf16=x_bf16, y_bf16=(m % 2 == 0), with_bias=(m % 3 == 2), seed=400 + m, path=api.PATH_SKINNY)


@pytest.mark.parametrize("fmt", [Q.MXFP4_CORE, Q.MXFP4_SPLIT])
@pytest.mark.parametrize("m,x_bf16", [(1, True), (1, False), (4, False), (8, True), (13, True)])
@pytest.mark.parametrize("n,k", [(200, 2048), (90, 2880), (33, 576), (40, 512)])
def test_token_column_kernel_mxfp4(fmt, m, x_bf16, n, k):
    """MXFP4 tiles with eight blocks per tile row, and with six (K = 2880 and 576 are multiples
    of 192 but not of 256, as the gpt-oss expert width)."""
    _run(fmt, n, k, m, x_bf16=x_bf16, y_bf16=(m % 2 == 0), with_bias=(m == 4), seed=500 + m, path=api.PATH_SKINNY)


def test_q8_0_gemv_reference_config():
    """The reference's own CPU-runnable case: Q8_0 4096 x 4096, x f32 [1, 4096], y f32."""
    _run(Q.Q8_0, 4096, 4096, 1, x_bf16=False, y_bf16=False, with_bias=False, seed=0x5EED)


@pytest.mark.parametrize("fmt", list(Q))
@pytest.mark.parametrize("m", [1, 2, 5, 8, 16])
def test_skinny_m_all_formats(fmt, m):
    _run(fmt, 64, 1024, m, x_bf16=True, y_bf16=False, with_bias=False, seed=10 + m)


@pytest.mark.parametrize("fmt", list(Q))
def test_generic_path_all_formats(fmt):
    _run(fmt, 40, 512, 3, x_bf16=False, y_bf16=False, with_bias=True, seed=5, path=api.PATH_GENERIC)


@pytest.mark.parametrize("fmt", [Q.Q8_0, Q.Q4_K, Q.Q6_K, Q.MXFP4_SPLIT])
@pytest.mark.parametrize("x_bf16,y_bf16", [(False, False), (True, True), (False, True)])
def test_dtypes_and_bias(fmt, x_bf16, y_bf16):
    _run(fmt, 128, 2048, 4, x_bf16, y_bf16, with_bias=True, seed=21)


@pytest.mark.parametrize("n,k", [(1, 256), (7, 256), (33, 768), (250, 1280), (4096, 4096)])
def test_q4_k_ragged_shapes(n, k):
    _run(Q.Q4_K, n, k, 1, x_bf16=True, y_bf16=False, with_bias=False, seed=n)


@pytest.mark.parametrize("m", [17, 33, 130])
def test_q4_k_larger_m(m):
    _run(Q.Q4_K, 96, 1024, m, x_bf16=True, y_bf16=False, with_bias=False, seed=m)


@pytest.mark.parametrize("fmt", list(Q))
def test_tensor_path_all_formats(fmt):
    _run(fmt, 200, 512, 150, x_bf16=True, y_bf16=False, with_bias=True, seed=71, path=api.PATH_TENSOR)


@pytest.mark.parametrize("m,n,k", [(1, 128, 64), (128, 128, 256), (129, 130, 320), (300, 72, 1024), (512, 256, 2048),
                                   (700, 384, 512)])
@pytest.mark.parametrize("x_bf16,y_bf16", [(True, True), (False, False)])
def test_tensor_path_shapes(m, n, k, x_bf16, y_bf16):
    _run(Q.Q8_0, n, k, m, x_bf16, y_bf16, with_bias=False, seed=m + n, path=api.PATH_TENSOR)


def test_tensor_path_is_exact_on_bf16_representable_weights():
    # Q8_0 with power-of-two scales and small codes decodes to bf16-exact weights, bf16 x: the
    # only difference from the oracle is the f32 summation order
    n, k, m = 128, 512, 128
    blk = np.zeros((n * k // 32, 34), np.uint8)
    blk[:, 0:2] = np.frombuffer(np.float16(0.25).tobytes(), np.uint8)
    blk[:, 2:] = (F.Stream(5).integers(n * k, -8, 7)).astype(np.int8).view(np.uint8).reshape(-1, 32)
    w = blk.reshape(-1)
    x = F.gen_activations(6, m, k, bf16=True)
    t = api.from_quantized(w, Q.Q8_0, [n, k])
    t.backend.set_path(api.PATH_TENSOR)
    try:
        y = api.quantized_matmul(torch.from_numpy(x).to(DEV).to(torch.bfloat16), t, out_dtype=torch.float32)
        torch.cuda.synchronize()
        t.backend.device_status()
    finally:
        t.backend.set_path(api.PATH_AUTO)
    y32, y64, mag = P.oracle_linear(Q.Q8_0, w, None, x, None, n, k)
    P.assert_close(y.cpu().numpy(), y32, y64, mag, tol=1e-5)
    t.release()


def test_config2_q4_k_m128_and_m512():
    # benchmark configuration 2 at the prefill sizes: q_proj 4096 -> 4096
    _run(Q.Q4_K, 4096, 4096, 128, x_bf16=True, y_bf16=True, with_bias=False, seed=0x5EF0)
    _run(Q.Q4_K, 4096, 4096, 512, x_bf16=True, y_bf16=True, with_bias=False, seed=0x5EF1)


def test_config1_q8_0_gemv_4096():
    # benchmark configuration 1: W 4096x4096 Q8_0, x f32 [1,4096], y f32 [1,4096]
    _run(Q.Q8_0, 4096, 4096, 1, x_bf16=False, y_bf16=False, with_bias=False, seed=0x5EED)


@pytest.mark.parametrize("n,k", [(1024, 4096), (4096, 12288), (12288, 4096)])
def test_config2_q4_k_projection_shapes_m1(n, k):
    _run(Q.Q4_K, n, k, 1, x_bf16=True, y_bf16=True, with_bias=False, seed=0x5EEE)


def test_config2_q4_k_m16():
    _run(Q.Q4_K, 4096, 4096, 16, x_bf16=True, y_bf16=True, with_bias=False, seed=0x5EEF)


def test_known_answer_products(golden):
    for case in golden["matmul"]:
        fmt = Q[case["fmt"]]
        w = np.frombuffer(bytes.fromhex(case["bytes"]), np.uint8)
        x = torch.tensor(case["x"], dtype=torch.float32, device=DEV)
        t = api.from_quantized(w, fmt, [case["n"], case["k"]])
        bias = torch.tensor(case["bias"], dtype=torch.float32, device=DEV) if case["bias"] else None
        y = api.quantized_linear(x, t, bias).cpu().numpy()
        assert np.all(np.abs(y - np.array(case["expect"], np.float32)) < case["tol"]), case["name"]
        t.release()


def test_batched_leading_dims():
    # input [2, 3, K] -> [2, 3, N] (crates/nn-core/src/dyn_tensor/quantized_matmul_tests.rs:274-317)
    n, k = 24, 256
    w, _ = F.gen_weight(Q.Q8_0, 3, n, k)
    x = F.gen_activations(4, 6, k, bf16=False)
    t = api.from_quantized(w, Q.Q8_0, [n, k])
    y = api.quantized_matmul_q8_0(torch.from_numpy(x.reshape(2, 3, k)).to(DEV), t)
    assert tuple(y.shape) == (2, 3, n)
    y32, y64, mag = P.oracle_linear(Q.Q8_0, w, None, x, None, n, k)
    P.assert_close(y.cpu().numpy().reshape(6, n), y32, y64, mag)
    t.release()


def test_error_cases_on_device():
    n, k = 8, 64
    w, _ = F.gen_weight(Q.Q8_0, 3, n, k)
    t = api.from_quantized(w, Q.Q8_0, [n, k])
    with pytest.raises(api.ShapeMismatch):
        api.quantized_matmul_q8_0(torch.zeros(2, 32, device=DEV), t)
    with pytest.raises(api.RankMismatch):
        api.quantized_matmul_q8_0(torch.zeros(64, device=DEV), t)
    with pytest.raises(api.BiasMismatch):
        api.quantized_linear(torch.zeros(1, 64, device=DEV), t, torch.zeros(n + 1, device=DEV))
    # the context is still usable afterwards
    y = api.quantized_matmul_q8_0(torch.zeros(1, 64, device=DEV), t)
    assert float(y.abs().max()) == 0.0
    t.release()


def test_empty_inputs():
    w, _ = F.gen_weight(Q.Q4_K, 3, 4, 256)
    t = api.from_quantized(w, Q.Q4_K, [4, 256])
    y = api.quantized_matmul(torch.zeros(0, 256, device=DEV), t)
    assert tuple(y.shape) == (0, 4)
    t.release()
    t0 = api.from_quantized(b"", Q.Q8_0, [0, 32])
    y = api.quantized_matmul(torch.zeros(3, 32, device=DEV), t0)
    assert tuple(y.shape) == (3, 0)
    t0.release()


def test_host_entry_point_matches_device_entry_point():
    n, k, m = 64, 512, 2
    w, _ = F.gen_weight(Q.Q4_K, 8, n, k)
    x = F.gen_activations(9, m, k, bf16=False)
    bias = (F.Stream(10).normal(n)).astype(np.float32)
    t = api.from_quantized(w, Q.Q4_K, [n, k])
    y_host = api.quantized_linear(x, t, bias)
    assert isinstance(y_host, np.ndarray)
    y_dev = api.quantized_linear(torch.from_numpy(x).to(DEV), t, torch.from_numpy(bias).to(DEV)).cpu().numpy()
    assert np.array_equal(y_host, y_dev)
    t.release()


def test_batch_call_matches_single_calls():
    k, m = 1024, 1
    shapes = [(256, k), (64, k), (64, k)]
    ws = []
    for i, (n, kk) in enumerate(shapes):
        w, _ = F.gen_weight(Q.Q4_K, 30 + i, n, kk)
        ws.append(api.from_quantized(w, Q.Q4_K, [n, kk]))
    x = torch.from_numpy(F.gen_activations(40, m, k, bf16=True)).to(DEV).to(torch.bfloat16)
    ys = api.linear_batch([x, x, x], ws, out_dtype=torch.float32)
    for y, w in zip(ys, ws):
        single = api.quantized_matmul(x, w, out_dtype=torch.float32)
        # the k-chunking (hence the f32 summation order) depends on the size of the launch
        assert float((y - single).abs().max()) <= 1e-5 * float(single.abs().max())
        w.release()


def test_batch_host_entry_point_matches_device_calls():
    """nnq_linear_batch_host: shared and distinct host activations, a bias, mixed shapes."""
    k = 2048
    shapes = [(256, k), (64, k), (130, 4096)]
    ws = []
    for i, (n, kk) in enumerate(shapes):
        w, _ = F.gen_weight(Q.Q4_K, 90 + i, n, kk)
        ws.append(api.from_quantized(w, Q.Q4_K, [n, kk]))
    xa = F.gen_activations(95, 1, k, bf16=True)
    xb = F.gen_activations(96, 1, 4096, bf16=True)
    bias = (F.Stream(97).normal(64) * 0.5).astype(np.float32)
    ys = api.linear_batch([xa, xa, xb], ws, biases=[None, bias, None])
    for y, w, x, bb in zip(ys, ws, (xa, xa, xb), (None, bias, None)):
        assert isinstance(y, np.ndarray)
        want = api.quantized_linear(torch.from_numpy(x).to(DEV), w, torch.from_numpy(bb).to(DEV) if bb is not None else None)
        assert float(np.max(np.abs(y - want.cpu().numpy()))) <= 1e-5 * float(want.abs().max())
        w.release()


@pytest.mark.parametrize("m", [4, 12])
def test_batch_call_token_column_kernel(m):
    # three projections sharing their activations go out as one launch of the token-column kernel
    k = 2048
    shapes = [(256, k), (72, k), (64, k)]
    ws = []
    for i, (n, kk) in enumerate(shapes):
        w, _ = F.gen_weight(Q.Q4_K, 60 + i, n, kk)
        ws.append(api.from_quantized(w, Q.Q4_K, [n, kk]))
    x = torch.from_numpy(F.gen_activations(70, m, k, bf16=True)).to(DEV).to(torch.bfloat16)
    ys = api.linear_batch([x, x, x], ws, out_dtype=torch.float32)
    for y, w in zip(ys, ws):
        single = api.quantized_matmul(x, w, out_dtype=torch.float32)
        assert y.shape == single.shape
        assert float((y - single).abs().max()) <= 1e-5 * float(single.abs().max())
        w.release()


@pytest.mark.parametrize("fmt", [Q.Q4_K, Q.Q8_0, Q.MXFP4_SPLIT])
def test_tensor_parallel_shards_reassemble(fmt):
    # column-parallel shards concatenate; row-parallel shard outputs sum (what an
    # all-reduce would do) -- size-independent linearity property
    n, k, world = 64, 2048, 4
    w, sc = F.gen_weight(fmt, 50, n, k)
    x = F.gen_activations(51, 2, k, bf16=False)
    full = api.from_quantized(w, fmt, [n, k], sc)
    xt = torch.from_numpy(x).to(DEV)
    y_full = api.quantized_matmul(xt, full)
    cols = [api.quantized_matmul(xt, full.shard(0, r, world)) for r in range(world)]
    assert torch.equal(torch.cat(cols, dim=-1), y_full)
    ks = k // world
    rows = [api.quantized_matmul(xt[:, r * ks:(r + 1) * ks].contiguous(), full.shard(1, r, world))
            for r in range(world)]
    y_sum = torch.stack(rows).sum(0)
    y32, y64, mag = P.oracle_linear(fmt, w, sc, x, None, n, k)
    P.assert_close(y_sum.cpu().numpy(), y32, y64, mag)
    with pytest.raises(api.InvalidShape):
        full.shard(0, 0, 7)
    full.release()


@pytest.mark.parametrize("fmt,k,world", [(Q.Q4_K, 25600, 8), (Q.Q6_K, 1280, 4), (Q.Q8_0, 96, 2)])
def test_uneven_row_parallel_shards(fmt, k, world):
    """K that does not divide by the ranks: 100 super-blocks over 8 ranks (13 / 12, the Qwen3-32B
    down projection), 5 over 4, three Q8_0 blocks over 2. Every shard holds exactly the bytes the
    host partition selects, and the shard products sum to the full product."""
    from nn_b200 import tp
    n = 48
    w, sc = F.gen_weight(fmt, 70, n, k)
    x = F.gen_activations(71, 1, k, bf16=True)
    full = api.from_quantized(w, fmt, [n, k], sc)
    xt = torch.from_numpy(x).to(DEV).to(torch.bfloat16)
    parts = []
    widths = set()
    for rank in range(world):
        sh = full.shard(1, rank, world)
        ns, ks = tp.shard_shape(fmt, n, k, 1, world, rank)
        assert sh.dims() == (ns, ks)
        widths.add(ks)
        ws, ss = tp.shard_bytes(fmt, w, sc, n, k, 1, rank, world)
        ref = orc.dequantize(fmt, ws, ns * ks, ss).reshape(ns, ks)
        assert np.array_equal(sh.dequantize().cpu().numpy().view(np.uint32), ref.view(np.uint32))
        cols = tp.input_slice(k, 1, rank, world, fmt)
        parts.append(api.quantized_linear(xt[:, cols].contiguous(), sh, None, out_dtype=torch.float32))
        sh.release()
    assert len(widths) == 2                      # the split really is uneven
    y32, y64, mag = P.oracle_linear(fmt, w, sc, x, None, n, k)
    P.assert_close(torch.stack(parts).sum(0).cpu().numpy(), y32, y64, mag)
    full.release()


@pytest.mark.parametrize("fmt", [Q.Q4_K, Q.Q6_K, Q.MXFP4_SPLIT])
@pytest.mark.parametrize("axis", [0, 1])
def test_device_shard_equals_host_partition(fmt, axis):
    # nnq_weight_create_shard keeps exactly the bytes nn_b200.tp.shard_bytes selects
    from nn_b200 import tp
    from oracle import cpu as orc
    n, k, world = 32, 2048, 4
    w, sc = F.gen_weight(fmt, 60, n, k)
    full = api.from_quantized(w, fmt, [n, k], sc)
    for rank in range(world):
        sh = full.shard(axis, rank, world)
        ws, ss = tp.shard_bytes(fmt, w, sc, n, k, axis, rank, world)
        ns, ks = tp.shard_shape(fmt, n, k, axis, world, rank)
        assert sh.dims() == (ns, ks)
        ref = orc.dequantize(fmt, ws, ns * ks, ss).reshape(ns, ks)
        got = sh.dequantize().cpu().numpy()
        assert np.array_equal(got.view(np.uint32), ref.view(np.uint32))
        sh.release()
    full.release()


@pytest.mark.parametrize("scale", [3.0e5, 1.0e-7, 1.0e30])
@pytest.mark.parametrize("x_bf16", [True, False])
def test_q4_k_activation_range(scale, x_bf16):
    # the skinny kernel feeds fp16 to the tensor cores after an exact power-of-two prescale:
    # very large and very small activations must come out as accurately as ordinary ones
    n, k = 64, 1024
    w, _ = F.gen_weight(Q.Q4_K, 90, n, k)
    x = (F.gen_activations(91, 1, k, bf16=True) * np.float32(scale)).astype(np.float32)
    if x_bf16:
        x = F.bf16_bits_to_f32(F.to_bf16_bits(x)).reshape(1, k)
    t = api.from_quantized(w, Q.Q4_K, [n, k])
    xt = torch.from_numpy(x).to(DEV)
    if x_bf16:
        xt = xt.to(torch.bfloat16)
    y = api.quantized_matmul(xt, t, out_dtype=torch.float32).cpu().numpy()
    t.backend.device_status()
    y32, y64, mag = P.oracle_linear(Q.Q4_K, w, None, x, None, n, k)
    P.assert_close(y, y32, y64, mag)
    t.release()


# --------------------------------------------------------------------------- #
# Qwen3-32B layer shapes (hidden 5120, FFN 25600, 64 query / 8 key-value heads x 128)
# --------------------------------------------------------------------------- #

QWEN3_32B_SHAPES = [(1024, 5120), (5120, 8192), (5120, 25600)]   # k/v, o, down: K = 20, 32, 100 super-blocks


@pytest.mark.parametrize("fmt", [Q.Q4_K, Q.Q6_K])
@pytest.mark.parametrize("n,k", QWEN3_32B_SHAPES)
def test_qwen3_32b_shapes_prefill_and_decode(fmt, n, k):
    """The large-prefill configuration's own shapes: Q6_K rows of K = 5120 / 25600 are only 8-byte
    aligned (210-byte blocks), K = 25600 is 100 super-blocks. M = 4096 runs the tensor-core path
    (bf16 operands: 1e-2), M = 1 the streaming kernels (f32 accumulation: 2e-3). The weights are
    drawn on the device and dequantized by the oracle; at M = 4096 the oracle product is formed for
    a seeded sample of 12 token rows (every output column of those rows is checked)."""
    from nn_b200 import workload as W
    b = api.gpu_backend()
    gen = torch.Generator(device=DEV)
    gen.manual_seed(3200 + n + k)
    raw = (W.gen_q4_k_device if fmt == Q.Q4_K else W.gen_q6_k_device)(torch, gen, n, k)
    w = api.DeviceWeight.from_device(b, fmt, raw, n, k)
    deq = orc.dequantize(fmt, raw.cpu().numpy(), n * k).reshape(n, k)
    assert np.array_equal(w.dequantize().cpu().numpy().view(np.uint32), deq.view(np.uint32))   # bit-exact decode
    # prefill: 4096 tokens of bf16 activations
    m = 4096
    x = torch.randn(m, k, device=DEV, generator=gen).to(torch.bfloat16)
    y = api.quantized_linear(x, w, None, out_dtype=torch.float32)
    torch.cuda.synchronize()
    b.device_status()
    rows = np.sort(F.Stream(n + k).integers(12, 0, m - 1))
    xs = x[torch.from_numpy(rows).to(DEV)].float().cpu().numpy()
    y32 = orc.linear_f32(xs, deq, None, len(rows), n, k)
    y64 = orc.linear_f64(xs, deq, None, len(rows), n, k)
    mag = orc.linear_abs(xs, deq, len(rows), n, k)
    got = y[torch.from_numpy(rows).to(DEV)].cpu().numpy()
    assert np.all(np.isfinite(got))
    assert P.max_rel_err(got, y32) <= P.TOL_BF16_MMA, P.max_rel_err(got, y32)
    assert P.max_scaled_err(got, y64, mag) <= P.TOL_BF16_MMA
    # decode: one token, bf16 and f32 activations, all rows
    for x_bf16 in (True, False):
        x1 = torch.randn(1, k, device=DEV, generator=gen)
        if x_bf16:
            x1 = x1.to(torch.bfloat16)
        y1 = api.quantized_linear(x1, w, None, out_dtype=torch.float32)
        torch.cuda.synchronize()
        b.device_status()
        xh = x1.float().cpu().numpy()
        r32 = orc.linear_f32(xh, deq, None, 1, n, k)
        r64 = orc.linear_f64(xh, deq, None, 1, n, k)
        rmag = orc.linear_abs(xh, deq, 1, n, k)
        P.assert_close(y1.cpu().numpy(), r32, r64, rmag)
    w.release()


@pytest.mark.parametrize("fmt", [Q.Q4_K, Q.Q8_0, Q.Q6_K, Q.MXFP4_SPLIT, Q.Q5_K, Q.F32_DENSE, Q.BF16_DENSE])
@pytest.mark.parametrize("m,n,k", [(256, 200, 512), (300, 520, 1024), (1000, 72, 2304)])
def test_large_batch_takes_the_decode_once_path(fmt, m, n, k):
    """From 256 rows of bf16 activations on (Q8_0: 384, Q4_K: 513 -- their fused decode is the faster
    one below that, so the smaller cases here run it with two accumulators per CTA and K split over
    CTAs), the weight is decoded to bf16 once and a plain TMA + tcgen05 product follows: ragged M and
    N tiles, K a multiple of 64, bias, both outputs."""
    _run(fmt, n, k, m, x_bf16=True, y_bf16=(m == 300), with_bias=(m != 256), seed=900 + m)


def test_unquantized_weights_are_bit_exact_at_one_token():
    """An f32 [n, k] weight behind the same entry point (the dense branch of the reference's
    Linear): the M = 1 product accumulates in f32, so the f32 bar applies, and the decode of a
    bf16 weight returns exactly the stored values."""
    n, k = 96, 1024
    for fmt in (Q.F32_DENSE, Q.BF16_DENSE):
        w, _ = F.gen_weight(fmt, 11, n, k)
        t = api.from_quantized(w, fmt, [n, k])
        deq = t.dequantize().cpu().numpy()
        assert np.array_equal(deq.view(np.uint32), orc.dequantize(fmt, w, n * k).reshape(n, k).view(np.uint32))
        t.release()
        _run(fmt, n, k, 1, x_bf16=False, y_bf16=False, with_bias=True, seed=12)


def test_failed_staging_growth_leaves_the_context_usable():
    """A host call whose staging buffers cannot be allocated returns OutOfMemory before it touches
    the caller's buffers, and the next host call reallocates and gives the right answer."""
    n, k = 64, 512
    w, _ = F.gen_weight(Q.Q4_K, 18, n, k)
    t = api.from_quantized(w, Q.Q4_K, [n, k])
    x = F.gen_activations(19, 2, k, bf16=False)
    want = api.quantized_linear(x, t, None)
    b = t.backend
    y = np.zeros((2, n), np.float32)
    for _ in range(2):
        # 2^36 rows of 512 floats: the pinned allocation is refused; only the sizes are read before that
        st = b._lib.nnq_linear_host(b._ctx, t.handle(), x.ctypes.data, api.F32, 1 << 36, None, y.ctypes.data, api.F32)
        with pytest.raises(api.BackendFailure) as e:
            b.check(st)
        assert e.value.kind in ("OutOfMemory", "DispatchFailed")   # the runtime's word for an impossible size
        got = api.quantized_linear(x, t, None)
        assert np.array_equal(got, want)
    t.release()


@pytest.mark.parametrize("fmt", [Q.Q4_K, Q.Q4_K_GGML, Q.Q6_K, Q.Q8_0, Q.Q4_0, Q.Q5_K])
@pytest.mark.parametrize("n,k", [(96, 256), (300, 1280)])
def test_fused_decode_tensor_path_multiplies_the_rounded_decoded_weights(fmt, n, k):
    """128 rows of activations take the product with the decode fused in (Q4_K: raw blocks through a
    shared-memory ring, K of 1280 = five super-blocks: a last chunk of one, split over CTAs). With
    unit vectors as activations it returns the weights its tensor-core operand held: the oracle's
    decode rounded to bf16, bit for bit. The 128 columns probed are spread over K."""
    w, sc = F.gen_weight(fmt, 67, n, k)
    t = api.from_quantized(w, fmt, [n, k], sc)
    cols = np.unique(np.concatenate([np.arange(0, k, max(1, k // 100)), [k - 1, k - 2, 255, 256 % k]]))[:128]
    x = torch.zeros(128, k, device=DEV, dtype=torch.bfloat16)
    x[torch.arange(len(cols)), torch.from_numpy(cols)] = 1.0
    y = api.quantized_linear(x, t, None, out_dtype=torch.float32)
    torch.cuda.synchronize()
    t.backend.device_status()
    deq = orc.dequantize(fmt, w, n * k, sc).reshape(n, k)
    want = F.bf16_bits_to_f32(F.to_bf16_bits(deq)).reshape(n, k)[:, cols]
    got = y.cpu().numpy()[: len(cols)].T
    normal = (want == 0) | (np.abs(want) >= 2.0 ** -126)   # the tensor cores flush subnormal operands
    assert np.array_equal(got[normal], want[normal])
    t.release()


@pytest.mark.parametrize("fmt", [Q.Q8_0, Q.Q4_0])
def test_fused_decode_tensor_path_k_not_a_multiple_of_256(fmt):
    """K = 320: Q8_0 rows are then not whole 16-byte units and the product loads its blocks from global
    memory instead of the shared-memory ring; same exactness."""
    test_fused_decode_tensor_path_multiplies_the_rounded_decoded_weights(fmt, 200, 320)


@pytest.mark.parametrize("fmt", [Q.Q4_K, Q.Q6_K, Q.Q8_0, Q.MXFP4_SPLIT, Q.MXFP4_CORE, Q.MXFP4_GPTOSS, Q.BF16_DENSE])
def test_decode_once_path_multiplies_the_rounded_decoded_weights(fmt):
    """With the identity (and rows of zeros below it: 640 rows, so that the decode-once path runs for
    every format) as activations the product returns the bf16 weights the GEMM was fed: they must be
    the oracle's decoded weights rounded to bf16, bit for bit -- including MXFP4 blocks with extreme
    scale exponents, which the direct-to-bf16 decode hands to the f32 decoder (exponent 0) or that sit
    at the top of its own range."""
    n, k = 96, 256
    w, sc = F.gen_weight(fmt, 61, n, k)
    if fmt == Q.MXFP4_SPLIT or fmt == Q.MXFP4_GPTOSS:
        sc = np.array(sc, copy=True)
        sc[:6] = [0, 1, 3, 250, 251, 252]
    elif fmt == Q.MXFP4_CORE:
        w = np.array(w, copy=True)
        w.reshape(-1, 17)[:6, 0] = [0, 1, 3, 250, 251, 252]
    t = api.from_quantized(w, fmt, [n, k], sc)
    x = torch.zeros(640, k, device=DEV, dtype=torch.bfloat16)
    x[:k] = torch.eye(k, device=DEV, dtype=torch.bfloat16)
    y = api.quantized_linear(x, t, None, out_dtype=torch.float32)     # rows [0, k) = W^T
    torch.cuda.synchronize()
    t.backend.device_status()
    deq = orc.dequantize(fmt, w, n * k, sc).reshape(n, k)
    with np.errstate(over="ignore"):
        want = F.bf16_bits_to_f32(F.to_bf16_bits(deq)).reshape(n, k)
    got = y.cpu().numpy()[:k].T
    # values compared as numbers (a sum of products with zeros does not keep the sign of a zero weight);
    # weights below the normal range are left out: the tensor cores flush subnormal operands to zero
    check = np.isfinite(want) & ((want == 0) | (np.abs(want) >= 2.0 ** -126))
    assert np.array_equal(got[check], want[check])
    assert np.all(np.abs(got[~check & np.isfinite(want)]) <= 2.0 ** -126)
    t.release()
