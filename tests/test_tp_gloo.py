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
            ns, ks = tp.shard_shape(fmt, n, k, axis, world, rank)
            xs = np.ascontiguousarray(x[:, tp.input_slice(k, axis, rank, world, fmt)])
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


@pytest.mark.parametrize("fmt,k", [(Q.Q4_K, 1024), (Q.Q8_0, 1024), (Q.MXFP4_SPLIT, 1024), (Q.Q4_K, 768), (Q.Q8_0, 96)])
def test_shards_plus_collective_equal_single_device(fmt, k, tmp_path):
    """K = 768 (three super-blocks) and K = 96 (three Q8_0 blocks) split unevenly over two ranks."""
    n, m, world = 32, 2, 2
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
    # Qwen3-32B down_proj: 25600 = 100 super-blocks: even for 2 and 4 ranks, 13 / 12 super-blocks for 8
    assert tp.shard_shape(Q.Q4_K, 5120, 25600, tp.ROW, 4) == (5120, 6400)
    ks = [tp.shard_shape(Q.Q4_K, 5120, 25600, tp.ROW, 8, r)[1] for r in range(8)]
    assert sorted(set(ks)) == [12 * 256, 13 * 256] and sum(ks) == 25600
    sl = [tp.input_slice(25600, tp.ROW, r, 8, Q.Q4_K) for r in range(8)]
    assert sl[0].start == 0 and sl[-1].stop == 25600 and all(sl[i].stop == sl[i + 1].start for i in range(7))
    # 32-weight blocks keep 256-weight units when K allows, so that every shard keeps a tiled layout
    assert tp.shard_shape(Q.Q8_0, 8, 768, tp.ROW, 2, 0) == (8, 256) and tp.shard_shape(Q.Q8_0, 8, 768, tp.ROW, 2, 1) == (8, 512)
    with pytest.raises(ValueError):
        tp.shard_shape(Q.Q4_K, 16, 256, tp.ROW, 2)
    with pytest.raises(ValueError):
        tp.shard_shape(Q.Q8_0, 10, 64, tp.COLUMN, 4)
    w, _ = F.gen_weight(Q.Q8_0, 1, 4, 128)
    parts = [tp.shard_bytes(Q.Q8_0, w, None, 4, 128, tp.ROW, r, 2)[0] for r in range(2)]
    full = w.reshape(4, 4, 34)
    assert np.array_equal(parts[0].reshape(4, 2, 34), full[:, :2])
    assert np.array_equal(parts[1].reshape(4, 2, 34), full[:, 2:])
