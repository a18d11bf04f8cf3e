"""Tensor-parallel partition + collective plan on CPU ranks (gloo, world_size 2): every rank
computes its shard's product with the oracle, the collective of the plan (all-gather for
column-parallel, all-reduce for row-parallel) must reproduce the single-device product."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from nn_b200 import formats as F
from nn_b200 import tp
from nn_b200.formats import QuantFormat as Q
from oracle import cpu as orc


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, fmt, n, k, m, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        w, sc = F.gen_weight(fmt, 50, n, k)       # same bytes on every rank
        x = F.gen_activations(51, m, k, bf16=False)
        res = {}
        for axis in (tp.COLUMN, tp.ROW):
            ws, ss = tp.shard_bytes(fmt, w, sc, n, k, axis, rank, world)
            ns, ks = tp.shard_shape(fmt, n, k, axis, world)
            xs = np.ascontiguousarray(x[:, tp.input_slice(k, axis, rank, world)])
            deq = orc.dequantize(fmt, ws, ns * ks, ss).reshape(ns, ks)
            y = torch.from_numpy(orc.linear_f32(xs, deq, None, m, ns, ks))
            if axis == tp.COLUMN:
                parts = [torch.empty_like(y) for _ in range(world)]
                dist.all_gather(parts, y)
                res[axis] = torch.cat(parts, dim=-1).numpy()
            else:
                dist.all_reduce(y)
                res[axis] = y.numpy()
        if rank == 0:
            np.savez(out, col=res[tp.COLUMN], row=res[tp.ROW])
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("fmt", [Q.Q4_K, Q.Q8_0, Q.MXFP4_SPLIT])
def test_shards_plus_collective_equal_single_device(fmt, tmp_path):
    n, k, m, world = 32, 1024, 2, 2
    out = str(tmp_path / "res.npz")
    mp.spawn(_worker, args=(world, _free_port(), fmt, n, k, m, out), nprocs=world, join=True)
    w, sc = F.gen_weight(fmt, 50, n, k)
    x = F.gen_activations(51, m, k, bf16=False)
    deq = orc.dequantize(fmt, w, n * k, sc).reshape(n, k)
    full = orc.linear_f32(x, deq, None, m, n, k)
    res = np.load(out)
    assert np.array_equal(res["col"], full)              # same arithmetic, just concatenated
    scale = orc.linear_abs(x, deq, m, n, k)
    assert np.max(np.abs(res["row"] - full) / scale) < 1e-6   # two partial sums instead of one


def test_shard_geometry_and_errors():
    assert tp.shard_shape(Q.Q4_K, 4096, 12288, tp.ROW, 8) == (4096, 1536)
    assert tp.shard_shape(Q.Q4_K, 12288, 4096, tp.COLUMN, 8) == (1536, 4096)
    # Qwen3-32B down_proj: 25600 = 100 super-blocks splits evenly for 2 and 4 ranks only
    assert tp.shard_shape(Q.Q4_K, 5120, 25600, tp.ROW, 4) == (5120, 6400)
    with pytest.raises(ValueError):
        tp.shard_shape(Q.Q4_K, 5120, 25600, tp.ROW, 8)
    with pytest.raises(ValueError):
        tp.shard_shape(Q.Q8_0, 10, 64, tp.COLUMN, 4)
    w, _ = F.gen_weight(Q.Q8_0, 1, 4, 128)
    parts = [tp.shard_bytes(Q.Q8_0, w, None, 4, 128, tp.ROW, r, 2)[0] for r in range(2)]
    full = w.reshape(4, 4, 34)
    assert np.array_equal(parts[0].reshape(4, 2, 34), full[:, :2])
    assert np.array_equal(parts[1].reshape(4, 2, 34), full[:, 2:])
