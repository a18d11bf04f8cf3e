"""One-shot peer all-reduce: world 1 on any box, world 2 as child processes when two GPUs are
visible (plain peer loads/stores only)."""
import os
import socket

import numpy as np
import pytest

torch = pytest.importorskip("torch")

from nn_b200 import api, comm

pytestmark = pytest.mark.gpu


def test_world_one_is_identity_and_sized():
    b = api.gpu_backend()
    c = comm.PeerComm(b, 0, 1, max_bytes=4096)
    for dt in (torch.float32, torch.bfloat16):
        x = torch.randn(1000, device="cuda:0").to(dt)
        want = x.clone()
        for _ in range(3):   # repeated calls advance the device-side sequence number
            c.all_reduce(x)
        torch.cuda.synchronize()
        b.device_status()
        assert torch.equal(x, want)
    with pytest.raises(api.Unsupported):
        c.all_reduce(torch.zeros(2000, device="cuda:0"))
    c.release()
    # messages from 32 KB on take the multi-CTA kernel (several CTAs, 16-byte units, a ragged last run)
    big = comm.PeerComm(b, 0, 1, max_bytes=3 << 20)
    for dt, n in ((torch.float32, 8192), (torch.float32, 700_004), (torch.bfloat16, 1_000_008), (torch.float32, 8193)):
        x = torch.randn(n, device="cuda:0").to(dt)
        want = x.clone()
        for _ in range(3):
            big.all_reduce(x)
        big.all_reduce(torch.ones(16, device="cuda:0"))    # the small kernel shares the sequence number
        torch.cuda.synchronize()
        b.device_status()
        assert torch.equal(x, want)
    big.release()


def test_fused_linear_world_one_matches_plain_product():
    """The product kernel with the all-reduce tail, on one rank: partial sums go through the slot
    and the last CTA writes the outputs; mixed with plain all-reduces on the same communicator."""
    from nn_b200 import formats as F
    from nn_b200.formats import QuantFormat as Q
    b = api.gpu_backend()
    n, k = 1000, 4096
    c = comm.PeerComm(b, 0, 1, max_bytes=n * 8)
    w, _ = F.gen_weight(Q.Q4_K, 77, n, k)
    wt = api.from_quantized(w, Q.Q4_K, [n, k])
    bias = torch.randn(n, device="cuda:0")
    for it, dt in enumerate((torch.bfloat16, torch.float32, torch.bfloat16)):
        x = torch.from_numpy(F.gen_activations(80 + it, 1, k, bf16=True)).to("cuda:0").to(dt)
        want = api.quantized_linear(x, wt, bias, out_dtype=torch.float32)
        got = c.linear(x, wt, bias, out_dtype=torch.float32)
        torch.cuda.synchronize()
        b.device_status()
        assert float((got - want).abs().max()) <= 1e-5 * float(want.abs().max())
        c.all_reduce(torch.ones(16, device="cuda:0"))   # shares the sequence number with the fused call
    # small K: fewer than 8 super-blocks, the warps of a CTA work on several row tiles
    for kk in (256, 1024):
        w3, _ = F.gen_weight(Q.Q4_K, 78, 200, kk)
        wt3 = api.from_quantized(w3, Q.Q4_K, [200, kk])
        x3 = torch.from_numpy(F.gen_activations(91, 1, kk, bf16=True)).to("cuda:0").to(torch.bfloat16)
        got = c.linear(x3, wt3, None)
        want = api.quantized_linear(x3, wt3, None, out_dtype=torch.float32)
        torch.cuda.synchronize()
        b.device_status()
        assert float((got - want).abs().max()) <= 1e-5 * float(want.abs().max())
        wt3.release()
    # a shape the fused kernel does not cover falls back to product + all-reduce
    x2 = torch.from_numpy(F.gen_activations(90, 3, k, bf16=True)).to("cuda:0").to(torch.bfloat16)
    c2 = comm.PeerComm(b, 0, 1, max_bytes=3 * n * 4)
    got = c2.linear(x2, wt, bias)
    want = api.quantized_linear(x2, wt, bias, out_dtype=torch.float32)
    torch.cuda.synchronize()
    assert float((got - want).abs().max()) <= 1e-5 * float(want.abs().max())
    c.release()
    c2.release()
    wt.release()


def test_a_peer_that_never_arrives_ends_in_a_timeout_status():
    """Failure made on the host: rank 0 of a two-rank world whose rank 1 never calls. Both
    communicators live in this process on one device (rank 1's buffer is plain local memory that
    nobody writes), the wait bound is short, and nothing faults: the kernel returns, the status
    word reads Timeout once and is clear afterwards, and a healthy communicator still works."""
    b = api.gpu_backend()
    c0 = comm.PeerComm(b, 0, 2, max_bytes=4096, exchange_handles=False)
    c1 = comm.PeerComm(b, 1, 2, max_bytes=4096, exchange_handles=False)
    bufs = [c0.local_buffer(), c1.local_buffer()]
    c0.open_local_peers(bufs)
    c1.open_local_peers(bufs)
    c0.set_spin_limit(2000)
    x = torch.ones(256, device="cuda:0")
    c0.all_reduce(x)                      # rank 1 never publishes: the bounded wait runs out
    torch.cuda.synchronize()
    with pytest.raises(api.BackendFailure) as e:
        b.device_status()
    assert e.value.kind == "Timeout"
    b.device_status()                     # cleared by the read
    # the multi-CTA form of the all-reduce gives up the same way, and leaves its counters usable
    cb0 = comm.PeerComm(b, 0, 2, max_bytes=1 << 20, exchange_handles=False)
    cb1 = comm.PeerComm(b, 1, 2, max_bytes=1 << 20, exchange_handles=False)
    bb = [cb0.local_buffer(), cb1.local_buffer()]
    cb0.open_local_peers(bb)
    cb1.open_local_peers(bb)
    cb0.set_spin_limit(2000)
    for _ in range(2):
        cb0.all_reduce(torch.ones(100_000, device="cuda:0"))
        torch.cuda.synchronize()
        with pytest.raises(api.BackendFailure) as e:
            b.device_status()
        assert e.value.kind == "Timeout"
    cb0.release()
    cb1.release()
    # the fused product + exchange kernel gives up the same way
    from nn_b200 import formats as F
    from nn_b200.formats import QuantFormat as Q
    n, k = 320, 2048
    w, _ = F.gen_weight(Q.Q4_K, 3, n, k)
    wt = api.from_quantized(w, Q.Q4_K, [n, k])
    xs = torch.from_numpy(F.gen_activations(4, 1, k, bf16=True)).to("cuda:0").to(torch.bfloat16)
    c0.linear(xs, wt, None)
    torch.cuda.synchronize()
    with pytest.raises(api.BackendFailure) as e:
        b.device_status()
    assert e.value.kind == "Timeout"
    # a healthy world-1 communicator on the same context is unaffected
    c = comm.PeerComm(b, 0, 1, max_bytes=4096)
    y = torch.arange(100, device="cuda:0", dtype=torch.float32)
    c.all_reduce(y)
    torch.cuda.synchronize()
    b.device_status()
    assert torch.equal(y, torch.arange(100, device="cuda:0", dtype=torch.float32))
    want = api.quantized_linear(xs, wt, None, out_dtype=torch.float32)
    c2 = comm.PeerComm(b, 0, 1, max_bytes=n * 8)
    got = c2.linear(xs, wt, None)
    torch.cuda.synchronize()
    b.device_status()
    assert float((got - want).abs().max()) <= 1e-5 * float(want.abs().max())
    for cc in (c, c2, c0, c1):
        cc.release()
    wt.release()


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, out):
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        b = api.Backend(rank)
        c = comm.PeerComm(b, rank, world, max_bytes=1 << 21)
        dev = torch.device("cuda", rank)
        ok = True
        for it in range(20):
            g = torch.Generator().manual_seed(100 + it)
            parts = [torch.randn(4096, generator=g) for _ in range(world)]
            x = parts[rank].to(dev)
            c.all_reduce(x)
            want = parts[0].clone()
            for r in range(1, world):
                want += parts[r]
            torch.cuda.synchronize()
            ok = ok and torch.equal(x.cpu(), want)
        b.device_status()
        # large messages (multi-CTA kernel), f32 and bf16, alternating with small ones
        for it, (dt, n) in enumerate(((torch.float32, 300_000), (torch.bfloat16, 500_000), (torch.float32, 524_288))):
            g = torch.Generator().manual_seed(500 + it)
            parts = [torch.randn(n, generator=g).to(dt) for _ in range(world)]
            x = parts[rank].to(dev)
            c.all_reduce(x)
            want = parts[0].float().clone()
            for r in range(1, world):
                want += parts[r].float()
            torch.cuda.synchronize()
            ok = ok and torch.equal(x.cpu(), want.to(dt))
            z = torch.full((64,), float(rank + 1), device=dev)
            c.all_reduce(z)
            torch.cuda.synchronize()
            ok = ok and bool((z == float(world * (world + 1) // 2)).all())
        b.device_status()
        # row-parallel product fused with its all-reduce against the unsharded product
        from nn_b200 import formats as F
        from nn_b200.formats import QuantFormat as Q
        n, k = 520, 8192
        w, _ = F.gen_weight(Q.Q4_K, 5, n, k)
        full = api.QuantizedTensor(w, Q.Q4_K, [n, k], None, b)
        shard = full.shard(1, rank, world)
        bias = torch.from_numpy((F.Stream(6).normal(n) * 0.5).astype(np.float32)).to(dev)
        for it in range(6):
            x = torch.from_numpy(F.gen_activations(200 + it, 1, k, bf16=True)).to(dev).to(torch.bfloat16)
            ks = k // world
            got = c.linear(x[:, rank * ks:(rank + 1) * ks].contiguous(), shard, bias)
            want = api.quantized_linear(x, full, bias, out_dtype=torch.float32)
            torch.cuda.synchronize()
            ok = ok and float((got - want).abs().max()) <= 1e-4 * float(want.abs().max())
            # identical bits on every rank
            sums = [None] * world
            dist.all_gather_object(sums, got.cpu().numpy().tobytes())
            ok = ok and all(s_ == sums[0] for s_ in sums)
            # fused exchanges and plain all-reduces alternate on one communicator
            z = torch.full((64,), float(rank + 1), device=dev)
            c.all_reduce(z)
            torch.cuda.synchronize()
            ok = ok and bool((z == float(world * (world + 1) // 2)).all())
        b.device_status()
        # the same exchange inside a compiled plan: two row-parallel groups and a plain one per run
        from nn_b200 import plan
        pl = plan.ProductPlan(b, torch.bfloat16, torch.float32)
        cases = []
        for i, (pn, pk) in enumerate(((520, 8192), (260, 4096))):
            pw, _ = F.gen_weight(Q.Q4_K, 40 + i, pn, pk)
            pfull = api.QuantizedTensor(pw, Q.Q4_K, [pn, pk], None, b)
            pshard = pfull.shard(1, rank, world)
            px = torch.from_numpy(F.gen_activations(300 + i, 1, pk, bf16=True)).to(dev).to(torch.bfloat16)
            pks = pk // world
            pxs = px[:, rank * pks:(rank + 1) * pks].contiguous()
            py = torch.full((pn,), float("nan"), device=dev)
            pl.add_reduced(c, pshard, pxs, py)
            cases.append((pfull, pshard, px, pxs, py))
        pl.finalize()
        for it in range(3):
            pl.run()
            z = torch.full((64,), float(rank + 1), device=dev)
            c.all_reduce(z)
            torch.cuda.synchronize()
            ok = ok and bool((z == float(world * (world + 1) // 2)).all())
            for pfull, pshard, px, pxs, py in cases:
                want = api.quantized_linear(px, pfull, None, out_dtype=torch.float32).reshape(-1)
                torch.cuda.synchronize()
                ok = ok and float((py - want).abs().max()) <= 1e-4 * float(want.abs().max())
                sums = [None] * world
                dist.all_gather_object(sums, py.cpu().numpy().tobytes())
                ok = ok and all(s_ == sums[0] for s_ in sums)
                py.fill_(float("nan"))
        b.device_status()
        pl.release()
        oks = [None] * world
        dist.all_gather_object(oks, bool(ok))     # a wrong result on any rank fails the test
        if rank == 0:
            np.save(out, np.array([1 if all(oks) else 0]))
        dist.barrier()
        c.release()
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_world_two_sums_in_rank_order(tmp_path):
    import torch.multiprocessing as mp
    out = str(tmp_path / "ok.npy")
    mp.spawn(_worker, args=(2, _free_port(), out), nprocs=2, join=True)
    assert int(np.load(out)[0]) == 1
