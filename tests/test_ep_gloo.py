"""Expert-parallel token dispatch on CPU ranks (gloo, world_size 2): the index arithmetic of
nn_b200.moe.dispatch_plan and the two all-to-all exchanges around it, with a stand-in for the
expert computation. What comes back must equal the single-device rule: per token, the outputs of
its experts weighted and added in expert-index order."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from nn_b200 import moe

E, K, H = 8, 2, 4


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _expert(rows, experts):
    """Stand-in for an expert MLP: depends on the row and on the expert that receives it."""
    e = experts.to(torch.float32)[:, None]
    return rows * (e + 1.0) + e


def _exchange(rows, send_counts, recv_counts):
    out = torch.empty((int(sum(recv_counts)),) + tuple(rows.shape[1:]), dtype=rows.dtype)
    dist.all_to_all_single(out, rows.contiguous(), list(recv_counts), list(send_counts))
    return out


def _worker(rank, world, port, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = torch.Generator().manual_seed(100 + rank)
        t = 5 + 2 * rank                                   # ragged: the ranks hold different token counts
        x = torch.randn(t, H, generator=g)
        idx = torch.stack([torch.randperm(E, generator=g)[:K] for _ in range(t)]).to(torch.int32)
        wt = torch.rand(t, K, generator=g)
        order, send_experts, src_token, send_counts, pos = moe.dispatch_plan(idx, E, world)
        per_rank = E // world
        # sorted by expert, hence by destination; stable inside an expert
        assert torch.all(send_experts[1:] >= send_experts[:-1])
        assert int(send_counts.sum()) == t * K
        recv_counts = torch.empty_like(send_counts)
        dist.all_to_all_single(recv_counts, send_counts)
        sc, rc = send_counts.tolist(), recv_counts.tolist()
        recv_rows = _exchange(x[src_token.to(torch.int64)], sc, rc)
        recv_experts = _exchange(send_experts, sc, rc)
        # every received assignment belongs to an expert this rank holds
        assert torch.all((recv_experts // per_rank) == rank)
        back = _exchange(_expert(recv_rows, recv_experts), rc, sc)
        # combine: expert-index order per token
        y = torch.zeros(t, H)
        for tok in range(t):
            for slot in sorted(range(K), key=lambda s_: int(idx[tok, s_])):
                y[tok] += wt[tok, slot] * back[int(pos[tok, slot])]
        want = torch.zeros(t, H)
        for tok in range(t):
            for slot in sorted(range(K), key=lambda s_: int(idx[tok, s_])):
                e = idx[tok, slot].reshape(1)
                want[tok] += wt[tok, slot] * _expert(x[tok:tok + 1], e)[0]
        ok = torch.equal(y, want)
        oks = [None] * world
        dist.all_gather_object(oks, bool(ok))
        if rank == 0:
            np.save(out, np.array([1 if all(oks) else 0]))
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_dispatch_exchange_combine_equals_single_device_rule(tmp_path):
    out = str(tmp_path / "ok.npy")
    mp.spawn(_worker, args=(2, _free_port(), out), nprocs=2, join=True)
    assert int(np.load(out)[0]) == 1


def test_dispatch_plan_is_a_stable_sort_by_expert():
    idx = torch.tensor([[3, 0], [0, 7], [3, 1]], dtype=torch.int32)
    order, send_experts, src_token, send_counts, pos = moe.dispatch_plan(idx, 8, 4)
    assert send_experts.tolist() == [0, 0, 1, 3, 3, 7]
    assert order.tolist() == [1, 2, 5, 0, 4, 3]          # flat order inside an expert
    assert src_token.tolist() == [0, 1, 2, 0, 2, 1]
    assert send_counts.tolist() == [3, 2, 0, 1]          # experts 0-1, 2-3, 4-5, 6-7
    assert pos.tolist() == [[3, 0], [1, 5], [4, 2]]
