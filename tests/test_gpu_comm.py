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
        c = comm.PeerComm(b, rank, world, max_bytes=1 << 15)
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
        if rank == 0:
            np.save(out, np.array([1 if ok else 0]))
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
