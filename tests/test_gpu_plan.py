"""Compiled product plan (one persistent kernel for a sequence of one-token products) against the
CPU oracle and against the same products issued one by one, through the C ABI.
Tolerance: max relative error 2e-3 (f32 accumulation; the products themselves are exact)."""
import ctypes

import numpy as np
import pytest

torch = pytest.importorskip("torch")

from nn_b200 import api, plan
from nn_b200 import formats as F
from nn_b200.formats import QuantFormat as Q
from tests import parity as P

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


def _weights(shapes, seed, fmt=Q.Q4_K):
    out = []
    for i, (n, k) in enumerate(shapes):
        w, sc = F.gen_weight(fmt, seed + i, n, k)
        out.append((w, api.from_quantized(w, fmt, [n, k], sc)))
    return out


def _check(got, fmt, w, x, bias, n, k, y_bf16=False):
    y32, y64, mag = P.oracle_linear(fmt, w, None, x, bias, n, k)
    got = got.float().cpu().numpy().reshape(1, n)
    if y_bf16:
        assert P.max_rel_err(got, y32) <= P.TOL_F32_ACC + 2.0 ** -9
    else:
        P.assert_close(got, y32, y64, mag)


@pytest.mark.parametrize("x_bf16", [True, False])
@pytest.mark.parametrize("fmt", [Q.Q4_K, Q.Q4_K_GGML])
def test_independent_groups_match_the_oracle(fmt, x_bf16):
    """Groups of 1..3 products with ragged row counts, K from 1 to 12 super-blocks: fewer tiles
    than CTAs, row tiles that straddle CTAs, tails of 16-row tiles, a bias."""
    shapes = [[(200, 2048), (64, 2048), (1030, 2048)], [(40, 256)], [(4100, 512), (17, 512)], [(333, 3072)]]
    b = api.gpu_backend()
    xdt = torch.bfloat16 if x_bf16 else torch.float32
    pl = plan.ProductPlan(b, xdt, torch.float32)
    keep = []
    for gi, group in enumerate(shapes):
        ws = _weights(group, 1000 + 10 * gi, fmt)
        k = group[0][1]
        x = F.gen_activations(77 + gi, 1, k, bf16=x_bf16)
        xt = torch.from_numpy(x).to(DEV).to(xdt)
        ys = [torch.full((n,), float("nan"), device=DEV) for n, _ in group]
        bias = (F.Stream(5 + gi).normal(group[0][0]) * 0.5).astype(np.float32) if gi == 1 else None
        bt = [torch.from_numpy(bias).to(DEV)] + [None] * (len(group) - 1) if bias is not None else None
        pl.add([t for _, t in ws], xt, ys, bt)
        keep.append((group, ws, x, ys, bias))
    pl.finalize()
    info = pl.info()
    assert info["groups"] == len(shapes) and info["ctas"] >= 1 and info["stages"] >= 2
    for rep in range(2):   # the counters only count up: a second run must give the same result
        pl.run()
        torch.cuda.synchronize()
        b.device_status()
        for group, ws, x, ys, bias in keep:
            for j, (n, k) in enumerate(group):
                _check(ys[j], fmt, ws[j][0], x, bias if j == 0 else None, n, k)
        if rep == 0:
            first = [[y.clone() for y in ys] for _, _, _, ys, _ in keep]
            for _, _, _, ys, _ in keep:
                for y in ys:
                    y.fill_(float("nan"))
    for a, (_, _, _, ys, _) in zip(first, keep):   # fixed summation order: identical bits
        for u, v in zip(a, ys):
            assert torch.equal(u, v)
    pl.release()
    for _, ws, _, _, _ in keep:
        for _, t in ws:
            t.release()


def test_chained_groups_see_their_producers():
    """Every group reads what the one before wrote (as o reads attention, down reads gate/up):
    the plan must give what the same products give when launched one after another."""
    b = api.gpu_backend()
    dims = [1024, 2048, 512, 4096, 256, 768]
    ws = _weights([(dims[i + 1], dims[i]) for i in range(len(dims) - 1)], 2000)
    x0 = torch.from_numpy(F.gen_activations(3, 1, dims[0], bf16=True)).to(DEV).to(torch.bfloat16).reshape(-1)
    bufs = [x0] + [torch.zeros(d, dtype=torch.bfloat16, device=DEV) for d in dims[1:]]
    pl = plan.ProductPlan(b, torch.bfloat16, torch.bfloat16)
    for i, (_, t) in enumerate(ws):
        pl.add([t], bufs[i], [bufs[i + 1]])
    pl.finalize()
    assert [pl.dependency(g) for g in range(len(ws))] == [-1, 0, 1, 2, 3]
    # reference: separate launches; values are rescaled between the products so that the chain
    # neither overflows nor vanishes -- here the plan and the separate launches see the same bits
    ref = [x0]
    for i, (_, t) in enumerate(ws):
        ref.append(api.quantized_linear(ref[-1].reshape(1, -1), t, None, out_dtype=torch.bfloat16).reshape(-1))
    torch.cuda.synchronize()
    for rep in range(3):
        for bf in bufs[1:]:
            bf.zero_()
        pl.run()
        torch.cuda.synchronize()
        b.device_status()
        for i in range(1, len(dims)):
            got, want = bufs[i].float(), ref[i].float()
            assert torch.isfinite(got).all()
            scale = want.abs().max().item() or 1.0
            # bf16 outputs feed the next product: allow one bf16 ulp of the largest value per stage
            assert (got - want).abs().max().item() <= scale * (2.0 ** -7) * i, (i, rep)
    pl.release()
    for _, t in ws:
        t.release()


def test_dependency_analysis_and_graph_replay():
    b = api.gpu_backend()
    ws = _weights([(512, 1024), (512, 1024), (1024, 512), (256, 1024)], 3000)
    xa = torch.from_numpy(F.gen_activations(9, 1, 1024, bf16=True)).to(DEV).to(torch.bfloat16).reshape(-1)
    ya, yb = torch.zeros(512, device=DEV), torch.zeros(512, device=DEV)
    xm = torch.from_numpy(F.gen_activations(10, 1, 512, bf16=True)).to(DEV).to(torch.bfloat16).reshape(-1)
    yc, yd = torch.zeros(1024, device=DEV), torch.zeros(256, device=DEV)
    pl = plan.ProductPlan(b, torch.bfloat16, torch.float32, analyze_deps=True)
    pl.add([ws[0][1], ws[1][1]], xa, [ya, yb])      # 0
    pl.add([ws[2][1]], xm, [yc])                    # 1: touches nothing of group 0
    pl.add([ws[3][1]], xa, [yd])                    # 2: reads xa only
    pl.add([ws[0][1]], xa, [ya])                    # 3: rewrites ya (written by group 0)
    pl.finalize()
    assert [pl.dependency(g) for g in range(4)] == [-1, -1, -1, 0]
    stream = torch.cuda.Stream(device=DEV)
    with torch.cuda.stream(stream):
        pl.run(stream)
        stream.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=stream):
            pl.run(torch.cuda.current_stream())
        for y in (ya, yb, yc, yd):
            y.fill_(float("nan"))
        g.replay()
        g.replay()
        stream.synchronize()
    b.device_status()
    xa_h, xm_h = xa.float().cpu().numpy().reshape(1, -1), xm.float().cpu().numpy().reshape(1, -1)
    _check(ya, Q.Q4_K, ws[0][0], xa_h, None, 512, 1024)
    _check(yb, Q.Q4_K, ws[1][0], xa_h, None, 512, 1024)
    _check(yc, Q.Q4_K, ws[2][0], xm_h, None, 1024, 512)
    _check(yd, Q.Q4_K, ws[3][0], xa_h, None, 256, 1024)
    pl.release()
    for _, t in ws:
        t.release()


def test_layer_shapes_match_separate_launches():
    """Two Qwen3-8B layers' worth of groups (q/k/v, o, gate/up, down at full size): sampled rows
    against the oracle, all rows against the library's separate launches."""
    b = api.gpu_backend()
    gen = torch.Generator(device=DEV)
    gen.manual_seed(11)
    from nn_b200 import workload as W
    pl = plan.ProductPlan(b, torch.bfloat16, torch.float32)
    layers = []
    for li in range(2):
        lw, xs, ys = {}, {}, {}
        for name, n, k in W.PROJECTIONS:
            raw = W.gen_q4_k_device(torch, gen, n, k)
            lw[name] = (api.DeviceWeight.from_device(b, Q.Q4_K, raw, n, k), raw)
        for group in W.GROUPS:
            k = lw[group[0]][0].shape[1]
            x = torch.randn(k, device=DEV, generator=gen).to(torch.bfloat16)
            for name in group:
                xs[name] = x
                ys[name] = torch.zeros(lw[name][0].shape[0], device=DEV)
            pl.add([lw[n_][0] for n_ in group], x, [ys[n_] for n_ in group])
        layers.append((lw, xs, ys))
    pl.finalize()
    pl.run()
    torch.cuda.synchronize()
    b.device_status()
    rows = np.array([0, 1, 15, 16, 17, 255, 256, 1000, 1023])
    for lw, xs, ys in layers:
        for name, n, k in W.PROJECTIONS:
            w, raw = lw[name]
            want = api.quantized_linear(xs[name].reshape(1, -1), w, None, out_dtype=torch.float32).reshape(-1)
            torch.cuda.synchronize()
            scale = want.abs().max().item()
            assert (ys[name] - want).abs().max().item() <= P.TOL_F32_ACC * scale, name
            # oracle on a sample of rows (dequantize those rows' blocks only)
            rs = rows[rows < n]
            blocks = raw.reshape(n, (k // 256) * 144)[torch.from_numpy(rs).to(DEV)].cpu().numpy().reshape(-1)
            x = xs[name].float().cpu().numpy().reshape(1, -1)
            y32, y64, mag = P.oracle_linear(Q.Q4_K, blocks, None, x, None, len(rs), k)
            got = ys[name][torch.from_numpy(rs).to(DEV)].cpu().numpy().reshape(1, -1)
            P.assert_close(got, y32, y64, mag)
    pl.release()
    for lw, _, _ in layers:
        for w, _ in lw.values():
            w.release()


def test_plan_rejects_what_it_cannot_run():
    b = api.gpu_backend()
    (w8, t8), = _weights([(64, 512)], 1, Q.Q8_0)
    (w4, t4), (w4b, t4b) = _weights([(64, 512), (64, 768)], 2)
    x = torch.zeros(512, dtype=torch.bfloat16, device=DEV)
    y = torch.zeros(64, device=DEV)
    pl = plan.ProductPlan(b, torch.bfloat16, torch.float32)
    with pytest.raises(api.Unsupported):
        pl.add([t8], x, [y])
    with pytest.raises(api.ShapeMismatch):
        pl.add([t4, t4b], x, [y, y])
    with pytest.raises(api.InvalidArgument):
        pl.finalize()          # empty
    with pytest.raises(api.InvalidArgument):
        pl.run()               # not finalized
    pl.add([t4], x, [y])
    pl.finalize()
    with pytest.raises(api.InvalidArgument):
        pl.add([t4], x, [y])   # finalized
    pl.run()
    torch.cuda.synchronize()
    b.device_status()
    pl.release()
    for t in (t8, t4, t4b):
        t.release()


def test_exchanged_groups_world_one_and_mixed_with_other_exchanges():
    """Row-parallel groups whose partial sums go through a communicator's slots inside the kernel,
    on one rank: same values as the plain products, the communicator's sequence number advances by
    the number of exchanged groups per run, and plain all-reduces on the same communicator still
    line up afterwards."""
    from nn_b200 import comm
    b = api.gpu_backend()
    shapes = [(520, 2048), (200, 1024), (1030, 512)]
    c = comm.PeerComm(b, 0, 1, max_bytes=max(n for n, _ in shapes) * 8)
    pl = plan.ProductPlan(b, torch.bfloat16, torch.float32)
    keep = []
    for i, (n, k) in enumerate(shapes):
        (w, t), = _weights([(n, k)], 2000 + i)
        x = F.gen_activations(300 + i, 1, k, bf16=True)
        xt = torch.from_numpy(x).to(DEV).to(torch.bfloat16)
        y = torch.full((n,), float("nan"), device=DEV)
        bias = torch.from_numpy((F.Stream(9 + i).normal(n) * 0.5).astype(np.float32)).to(DEV) if i == 1 else None
        if i == 2:
            pl.add([t], xt, [y])                 # a plain group between exchanged ones
        else:
            pl.add_reduced(c, t, xt, y, bias)
        keep.append((w, t, x, y, bias, n, k))
    pl.finalize()
    for rep in range(3):
        pl.run()
        z = torch.full((64,), 2.0, device=DEV)
        c.all_reduce(z)                          # shares the sequence number with the plan's exchanges
        torch.cuda.synchronize()
        b.device_status()
        assert bool((z == 2.0).all())
        for w, t, x, y, bias, n, k in keep:
            _check(y, Q.Q4_K, w, x, bias.cpu().numpy() if bias is not None else None, n, k)
            y.fill_(float("nan"))
    pl.release()
    c.release()
    for _, t, *_ in keep:
        t.release()
