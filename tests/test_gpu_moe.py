"""GPU MoE block against the oracle's restatement of the reference's moe_forward
(crates/nn-gptoss/src/quantized_model.rs:99-194), through the C ABI. Router logits are
continuous (no ties), as the reference's unstable top-k requires."""
import numpy as np
import pytest

torch = pytest.importorskip("torch")

from nn_b200 import api, moe
from nn_b200 import formats as F
from nn_b200.formats import QuantFormat as Q
from oracle import cpu as orc

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _gen(fmt, seed, n, k, fast):
    """Raw blocks with the benchmark distributions; fast=True draws the MXFP4 payload (codes uniform
    over all bytes, E8M0 exponent uniform in [-8, 0]) with numpy's PCG64 instead of the SplitMix64
    counter stream, which takes a minute per full-size expert tensor."""
    if not fast:
        return F.gen_weight(fmt, seed, n, k)
    assert fmt in (Q.MXFP4_GPTOSS, Q.MXFP4_SPLIT)
    rng = np.random.default_rng(seed)
    codes = rng.integers(0, 256, size=n * (k // 2), dtype=np.uint8)
    exps = rng.integers(119, 128, size=n * (k // 32), dtype=np.uint8)
    return codes, exps


def _make(layout, fmt, E, H, I, seed, fast=False):
    s = F.Stream(seed)
    router_w = (s.normal(E * H) * 0.5).astype(np.float32).reshape(E, H)
    router_b = (s.normal(E) * 0.1).astype(np.float32)
    b_gu = (s.normal(E * 2 * I) * 0.1).astype(np.float32).reshape(E, 2 * I)
    b_d = (s.normal(E * H) * 0.1).astype(np.float32).reshape(E, H)
    if layout == moe.LAYOUT_KN_GPTOSS:
        # flat nn-gptoss tensors [E, H, 2I] and [E, I, H]: blocks of 32 along the last axis
        gu, gus = _gen(Q.MXFP4_GPTOSS, seed + 1, E * H, 2 * I, fast)
        dn, dns = _gen(Q.MXFP4_GPTOSS, seed + 2, E * I, H, fast)
        w_gu = orc.dequantize(Q.MXFP4_GPTOSS, gu, E * H * 2 * I, gus).reshape(E, H, 2 * I)
        w_d = orc.dequantize(Q.MXFP4_GPTOSS, dn, E * I * H, dns).reshape(E, I, H)
    else:
        gu, gus = _gen(fmt, seed + 1, E * 2 * I, H, fast)
        dn, dns = _gen(fmt, seed + 2, E * H, I, fast)
        w_gu = orc.dequantize(fmt, gu, E * 2 * I * H, gus).reshape(E, 2 * I, H).transpose(0, 2, 1).copy()
        w_d = orc.dequantize(fmt, dn, E * H * I, dns).reshape(E, H, I).transpose(0, 2, 1).copy()
    return router_w, router_b, gu, gus, b_gu, dn, dns, b_d, w_gu, w_d


@pytest.mark.parametrize("layout,fmt", [(moe.LAYOUT_KN_GPTOSS, Q.MXFP4_GPTOSS), (moe.LAYOUT_NK, Q.MXFP4_SPLIT),
                                        (moe.LAYOUT_NK, Q.Q4_K), (moe.LAYOUT_NK, Q.Q5_K), (moe.LAYOUT_NK, Q.Q3_K),
                                        (moe.LAYOUT_NK, Q.BF16_DENSE), (moe.LAYOUT_NK, Q.F32_DENSE)])
@pytest.mark.parametrize("T", [1, 7, 64])
def test_moe_forward_matches_oracle(layout, fmt, T):
    E, H, I, k, limit = 8, 256, 256, 4, 7.0
    rw, rb, gu, gus, bgu, dn, dns, bd, w_gu, w_d = _make(layout, fmt, E, H, I, 100 + T)
    x = F.gen_activations(7 + T, T, H, bf16=True)
    blk = moe.MoeBlock(E, H, I, k, limit, rw, rb, layout, fmt, gu, gus, bgu, dn, dns, bd)
    xt = torch.from_numpy(x).to(DEV)
    idx, wt = blk.route(xt)
    y = blk(xt).cpu().numpy()
    torch.cuda.synchronize()
    y_ref, idx_ref, wt_ref = orc.moe_forward(x, rw, rb, w_gu, bgu, w_d, bd, k, limit)
    assert np.array_equal(idx.cpu().numpy(), idx_ref)
    assert np.allclose(wt.cpu().numpy(), wt_ref, rtol=1e-5, atol=1e-7)
    assert np.all(np.isfinite(y))
    err = np.max(np.abs(y - y_ref)) / np.max(np.abs(y_ref))
    assert err <= 2e-3, err
    # bf16 activations give the same result as their f32 widening
    y16 = blk(xt.to(torch.bfloat16)).cpu().numpy()
    assert np.array_equal(y16, y)
    blk.release()


@pytest.mark.parametrize("fmt", [Q.MXFP4_SPLIT, Q.Q4_K, Q.Q4_K_GGML, Q.Q8_0, Q.BF16_DENSE])
def test_prefill_sized_batch_takes_the_tensor_core_path(fmt):
    """From 32 routed rows per expert on, [N, K] experts run the grouped tcgen05 products (bf16
    operands: the 1e-2 bar of the tensor path); ragged expert loads, rows not a multiple of 128."""
    # 8 experts, top-4. 70 tokens: 35 routed rows per expert; 150: 75; 333: 166; 1024: 512. The product
    # with the decode fused in serves Q4_K (either element order) up to 127 rows per expert and Q8_0 up
    # to 383 (the raw-block ring of the 128- and 256-row tiles); everything else is decoded to bf16
    # once and multiplied by the plain grouped GEMM. (Q6_K experts are not in this list: the generator's
    # Q6_K weights reach +-4000 and the block's outputs 2e6 after the clamp; the bf16 operands then
    # measure 1.3e-2 of the largest output at 70 tokens, just above this test's bar.)
    for T in (70, 150, 333, 1024):
        _prefill_case(fmt, T)


@pytest.mark.parametrize("T", [70, 333, 1024])
def test_prefill_sized_batch_of_kn_gptoss_experts(T):
    """nn-gptoss [E, K, N] experts at prefill size: a transposing decode into the bf16 scratch, then the
    grouped GEMM with SwiGLU in the epilogue of the gate / up product (same numerics as [N, K] MXFP4)."""
    _prefill_case(Q.MXFP4_GPTOSS, T, moe.LAYOUT_KN_GPTOSS)


def _prefill_case(fmt, T, layout=moe.LAYOUT_NK):
    E, H, I, k = 8, 256, 256, 4
    rw, rb, gu, gus, bgu, dn, dns, bd, w_gu, w_d = _make(layout, fmt, E, H, I, 77)
    x = F.gen_activations(78, T, H, bf16=True)
    blk = moe.MoeBlock(E, H, I, k, 7.0, rw, rb, layout, fmt, gu, gus, bgu, dn, dns, bd)
    y = blk(torch.from_numpy(x).to(DEV)).cpu().numpy()
    blk.backend.device_status()
    y_ref, _, _ = orc.moe_forward(x, rw, rb, w_gu, bgu, w_d, bd, k, 7.0)
    assert np.all(np.isfinite(y))
    assert np.max(np.abs(y - y_ref)) / np.max(np.abs(y_ref)) <= 1e-2
    blk.release()


@pytest.mark.parametrize("layout,fmt,T", [(moe.LAYOUT_KN_GPTOSS, Q.MXFP4_GPTOSS, 5), (moe.LAYOUT_NK, Q.MXFP4_SPLIT, 5),
                                          (moe.LAYOUT_NK, Q.MXFP4_SPLIT, 23)])
def test_gptoss_shape_decode_batch(layout, fmt, T):
    # gpt-oss-20b expert geometry (hidden = inter = 2880, not a multiple of 128 or 256), fewer experts
    E, H, I, k = 4, 2880, 2880, 2
    rw, rb, gu, gus, bgu, dn, dns, bd, w_gu, w_d = _make(layout, fmt, E, H, I, 9)
    x = F.gen_activations(3, T, H, bf16=True)
    blk = moe.MoeBlock(E, H, I, k, 7.0, rw, rb, layout, fmt, gu, gus, bgu, dn, dns, bd)
    y = blk(torch.from_numpy(x).to(DEV)).cpu().numpy()
    y_ref, _, _ = orc.moe_forward(x, rw, rb, w_gu, bgu, w_d, bd, k, 7.0)
    assert np.max(np.abs(y - y_ref)) / np.max(np.abs(y_ref)) <= 2e-3
    blk.release()


def test_moe_argument_errors():
    E, H, I = 4, 64, 64
    rw, rb, gu, gus, bgu, dn, dns, bd, _, _ = _make(moe.LAYOUT_NK, Q.Q8_0, E, H, I, 5)
    with pytest.raises(api.DataLengthMismatch):
        moe.MoeBlock(E, H, I, 2, 7.0, rw, rb, moe.LAYOUT_NK, Q.Q8_0, gu[:-1], gus, bgu, dn, dns, bd)
    with pytest.raises(api.WrongQuantType):
        moe.MoeBlock(E, H, I, 2, 7.0, rw, rb, moe.LAYOUT_KN_GPTOSS, Q.Q8_0, gu, gus, bgu, dn, dns, bd)
    with pytest.raises(api.InvalidArgument):
        moe.MoeBlock(E, H, I, 9, 7.0, rw, rb, moe.LAYOUT_NK, Q.Q8_0, gu, gus, bgu, dn, dns, bd)
    blk = moe.MoeBlock(E, H, I, 2, 7.0, rw, rb, moe.LAYOUT_NK, Q.Q8_0, gu, gus, bgu, dn, dns, bd)
    with pytest.raises(api.ShapeMismatch):
        blk(torch.zeros(3, H + 1, device=DEV))
    assert tuple(blk(torch.zeros(0, H, device=DEV)).shape) == (0, H)
    blk.release()


@pytest.mark.parametrize("layout,fmt", [(moe.LAYOUT_KN_GPTOSS, Q.MXFP4_GPTOSS), (moe.LAYOUT_NK, Q.MXFP4_SPLIT)])
def test_expert_parallel_shards_sum_to_full_block(layout, fmt):
    # expert parallelism with replicated activations: every "rank" holds E / p experts; the sum of
    # the shard outputs (what the all-reduce forms) equals the full block
    E, H, I, k, T, world = 8, 256, 256, 4, 33, 4
    rw, rb, gu, gus, bgu, dn, dns, bd, w_gu, w_d = _make(layout, fmt, E, H, I, 300)
    x = F.gen_activations(301, T, H, bf16=True)
    xt = torch.from_numpy(x).to(DEV)
    full = moe.MoeBlock(E, H, I, k, 7.0, rw, rb, layout, fmt, gu, gus, bgu, dn, dns, bd)
    y_full = full(xt)
    ec = E // world
    gu2 = np.asarray(gu).reshape(E, -1)
    dn2 = np.asarray(dn).reshape(E, -1)
    gus2 = np.asarray(gus).reshape(E, -1)
    dns2 = np.asarray(dns).reshape(E, -1)
    total = torch.zeros_like(y_full)
    for r in range(world):
        sl = slice(r * ec, (r + 1) * ec)
        shard = moe.MoeBlock(E, H, I, k, 7.0, rw, rb, layout, fmt, gu2[sl], gus2[sl], bgu[sl], dn2[sl], dns2[sl],
                             bd[sl], expert_range=(r * ec, ec))
        idx_s, wt_s = shard.route(xt)
        idx_f, wt_f = full.route(xt)
        assert torch.equal(idx_s, idx_f) and torch.equal(wt_s, wt_f)   # routing is replicated
        total += shard(xt)
        shard.release()
    torch.cuda.synchronize()
    err = float((total - y_full).abs().max() / y_full.abs().max())
    assert err <= 1e-5, err
    y_ref, _, _ = orc.moe_forward(x, rw, rb, w_gu, bgu, w_d, bd, k, 7.0)
    assert np.max(np.abs(total.cpu().numpy() - y_ref)) / np.max(np.abs(y_ref)) <= 2e-3
    full.release()


@pytest.mark.parametrize("layout,fmt", [(moe.LAYOUT_KN_GPTOSS, Q.MXFP4_GPTOSS), (moe.LAYOUT_NK, Q.MXFP4_SPLIT), (moe.LAYOUT_NK, Q.Q4_K)])
def test_expert_parallel_token_dispatch_on_one_device(layout, fmt):
    """The device-side pieces of expert parallelism with token dispatch (gather by destination,
    experts over supplied routing, weighted combine) with the all-to-all played by hand: four
    "ranks" on one GPU hold 8 / 4 experts each and ragged shares of the tokens."""
    E, H, I, k, world = 8, 256, 256, 4, 4
    shares = [10, 9, 11, 7]
    T = sum(shares)
    rw, rb, gu, gus, bgu, dn, dns, bd, w_gu, w_d = _make(layout, fmt, E, H, I, 500)
    x = F.gen_activations(501, T, H, bf16=True)
    xt = torch.from_numpy(x).to(DEV)
    full = moe.MoeBlock(E, H, I, k, 7.0, rw, rb, layout, fmt, gu, gus, bgu, dn, dns, bd)
    y_full = full(xt)
    ec = E // world
    rs = lambda a: None if a is None else np.asarray(a).reshape(E, -1)
    gu2, dn2, gus2, dns2 = rs(gu), rs(dn), rs(gus), rs(dns)
    shards = []
    for r in range(world):
        sl = slice(r * ec, (r + 1) * ec)
        shards.append(moe.MoeBlock(E, H, I, k, 7.0, rw, rb, layout, fmt, gu2[sl], None if gus2 is None else gus2[sl], bgu[sl],
                                   dn2[sl], None if dns2 is None else dns2[sl], bd[sl], expert_range=(r * ec, ec)))
    b = full.backend
    xs = torch.split(xt, shares)
    plans, sends = [], []
    for r in range(world):
        idx, wt = shards[r].route(xs[r])
        order, send_experts, src_token, send_counts, pos = moe.dispatch_plan(idx, E, world)
        rows = moe.gather_rows(b, xs[r], src_token)
        counts = send_counts.cpu().tolist()
        plans.append((idx, wt, pos, counts))
        sends.append((torch.split(rows, counts), torch.split(send_experts, counts)))
    # "all-to-all": destination d receives, from every source in rank order, the slice meant for it
    outs = []
    for d in range(world):
        recv_rows = torch.cat([sends[r][0][d] for r in range(world)])
        recv_experts = torch.cat([sends[r][1][d] for r in range(world)])
        assert bool(((recv_experts // ec) == d).all())
        ones = torch.ones(recv_rows.shape[0], device=DEV)
        out = shards[d].forward_routed(recv_rows, recv_experts, ones, 1)
        outs.append(torch.split(out, [plans[r][3][d] for r in range(world)]))
    ys = []
    for r in range(world):
        back = torch.cat([outs[d][r] for d in range(world)])     # this rank's rows, in its sorted order
        idx, wt, pos, _ = plans[r]
        ys.append(moe.combine_rows(b, back, idx, wt, pos))
    y = torch.cat(ys)
    torch.cuda.synchronize()
    b.device_status()
    assert float((y - y_full).abs().max() / y_full.abs().max()) <= 1e-5
    y_ref, _, _ = orc.moe_forward(x, rw, rb, w_gu, bgu, w_d, bd, k, 7.0)
    assert np.max(np.abs(y.cpu().numpy() - y_ref)) / np.max(np.abs(y_ref)) <= 2e-3
    for s_ in shards:
        s_.release()
    full.release()


def _ep_worker(rank, world, port, out):
    import os

    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        dev = f"cuda:{rank}"
        E, H, I, k = 8, 256, 256, 4
        layout, fmt = moe.LAYOUT_NK, Q.MXFP4_SPLIT
        rw, rb, gu, gus, bgu, dn, dns, bd, w_gu, w_d = _make(layout, fmt, E, H, I, 700)
        shares = [13, 20][:world] if world == 2 else [9] * world
        x = F.gen_activations(701, sum(shares), H, bf16=True)
        b = api.Backend(rank)
        ec = E // world
        sl = slice(rank * ec, (rank + 1) * ec)
        rs = lambda a: np.asarray(a).reshape(E, -1)
        shard = moe.MoeBlock(E, H, I, k, 7.0, rw, rb, layout, fmt, rs(gu)[sl], rs(gus)[sl], bgu[sl], rs(dn)[sl], rs(dns)[sl], bd[sl],
                             backend=b, expert_range=(rank * ec, ec))
        ep = moe.ExpertParallelMoe(shard, rank, world)
        lo = sum(shares[:rank])
        y = ep(torch.from_numpy(x[lo:lo + shares[rank]]).to(dev)).cpu().numpy()
        torch.cuda.synchronize()
        b.device_status()
        y_ref, _, _ = orc.moe_forward(x[lo:lo + shares[rank]], rw, rb, w_gu, bgu, w_d, bd, k, 7.0)
        ok = bool(np.max(np.abs(y - y_ref)) / np.max(np.abs(y_ref)) <= 2e-3)
        oks = [None] * world
        dist.all_gather_object(oks, ok)
        if rank == 0:
            np.save(out, np.array([1 if all(oks) else 0]))
        dist.barrier()
        shard.release()
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_expert_parallel_all_to_all_two_gpus(tmp_path):
    import socket

    import torch.multiprocessing as mp
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    out = str(tmp_path / "ok.npy")
    mp.spawn(_ep_worker, args=(2, port, out), nprocs=2, join=True)
    assert int(np.load(out)[0]) == 1


# --------------------------------------------------------------------------- #
# gpt-oss-20b geometry: 32 experts, top-4, hidden = inter = 2880
# --------------------------------------------------------------------------- #

_GPTOSS = {}


def _gptoss_block(layout, fmt):
    """Weights of the full-size block are expensive to draw and to dequantize on the CPU: built
    once per layout and shared by the decode-sized and the prefill-sized case."""
    key = (layout, int(fmt))
    if key not in _GPTOSS:
        E, H, I, k = 32, 2880, 2880, 4
        made = _make(layout, fmt, E, H, I, 4242, fast=True)
        rw, rb, gu, gus, bgu, dn, dns, bd, w_gu, w_d = made
        blk = moe.MoeBlock(E, H, I, k, 7.0, rw, rb, layout, fmt, gu, gus, bgu, dn, dns, bd)
        _GPTOSS[key] = (blk, rw, rb, bgu, bd, w_gu, w_d)
    return _GPTOSS[key]


@pytest.mark.parametrize("layout,fmt", [(moe.LAYOUT_KN_GPTOSS, Q.MXFP4_GPTOSS), (moe.LAYOUT_NK, Q.MXFP4_SPLIT)])
@pytest.mark.parametrize("T", [64, 4096])
def test_gptoss_20b_geometry(layout, fmt, T):
    """The benchmark configuration itself (32 experts, top-4, 2880 x 2880 experts): every token of
    the 64-token decode batch, and a seeded sample of 24 tokens of the 4096-token prefill batch
    (a token's output depends on no other token, so the oracle runs on the sample alone).
    64 tokens stay on the f32-accumulating kernels (2e-3); 4096 tokens give 512 routed rows per
    expert, which both layouts run on the tensor cores with bf16 operands (1e-2)."""
    blk, rw, rb, bgu, bd, w_gu, w_d = _gptoss_block(layout, fmt)
    H, k = 2880, 4
    x = F.gen_activations(900 + T, T, H, bf16=True)
    xt = torch.from_numpy(x).to(DEV)
    y = blk(xt)
    idx, wt = blk.route(xt)
    torch.cuda.synchronize()
    blk.backend.device_status()
    sample = np.arange(T) if T <= 64 else np.sort(F.Stream(31).integers(24, 0, T - 1))
    y_ref, idx_ref, wt_ref = orc.moe_forward(x[sample], rw, rb, w_gu, bgu, w_d, bd, k, 7.0)
    got = y.cpu().numpy()[sample]
    assert np.array_equal(idx.cpu().numpy()[sample], idx_ref)
    # router logits over 2880 terms reach +-100: a rounding difference of 1e-4 in a logit moves a
    # small softmax weight by 1e-4 of itself, so the weights are compared to 2e-3 of themselves
    assert np.allclose(wt.cpu().numpy()[sample], wt_ref, rtol=2e-3, atol=1e-7)
    assert np.all(np.isfinite(got))
    tol = 1e-2 if T > 64 else 2e-3
    err = np.max(np.abs(got - y_ref)) / np.max(np.abs(y_ref))
    assert err <= tol, err
    # per-token bound as well: one scale per token instead of one for the whole batch
    per_tok = np.max(np.abs(got - y_ref), axis=1) / np.max(np.abs(y_ref), axis=1)
    assert np.all(per_tok <= 2 * tol), per_tok.max()


def test_gptoss_20b_release():
    """Frees the shared full-size blocks (kept last in this file)."""
    for blk, *_ in _GPTOSS.values():
        blk.release()
    _GPTOSS.clear()
