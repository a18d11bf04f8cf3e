"""Tensor-parallel partitioning of quantized weights (host logic).

The reference runs on one device; the split follows the Megatron scheme for the shapes its
callers fix (crates/nn-qwen3/src/layers.rs:26-47,65-92): q/k/v and gate/up are split by rows
(column-parallel, input replicated, outputs concatenated), o_proj and down_proj by whole
quantization blocks along K (row-parallel, inputs split, outputs summed with an all-reduce).
Blocks never cross a row, so both splits are plain byte ranges of the raw tensor; the same
arithmetic is implemented on the device side by nnq_weight_create_shard.
"""
from __future__ import annotations

import numpy as np

from .formats import GEOMETRY, QuantFormat

COLUMN, ROW = 0, 1


def shard_shape(fmt, n: int, k: int, axis: int, world: int) -> tuple[int, int]:
    g = GEOMETRY[QuantFormat(fmt)]
    if axis == COLUMN:
        if n % world:
            raise ValueError(f"out_features {n} not divisible by {world} ranks")
        return n // world, k
    kb = k // g.elems
    if kb % world:
        raise ValueError(f"{kb} blocks per row not divisible by {world} ranks")
    return n, (kb // world) * g.elems


def shard_bytes(fmt, raw: np.ndarray, scales, n: int, k: int, axis: int, rank: int, world: int):
    """(main bytes, scale bytes or None) of one rank's shard of an [n, k] weight."""
    g = GEOMETRY[QuantFormat(fmt)]
    kb = k // g.elems
    ns, ks = shard_shape(fmt, n, k, axis, world)
    main = np.ascontiguousarray(raw, np.uint8).reshape(n, kb * g.bytes)
    sc = None if scales is None else np.ascontiguousarray(scales, np.uint8).reshape(n, kb * g.scale_bytes)
    if axis == COLUMN:
        rows = slice(rank * ns, (rank + 1) * ns)
        return main[rows].reshape(-1).copy(), (None if sc is None else sc[rows].reshape(-1).copy())
    kbs = kb // world
    cols = slice(rank * kbs * g.bytes, (rank + 1) * kbs * g.bytes)
    scols = slice(rank * kbs * g.scale_bytes, (rank + 1) * kbs * g.scale_bytes)
    return main[:, cols].reshape(-1).copy(), (None if sc is None else sc[:, scols].reshape(-1).copy())


def input_slice(k: int, axis: int, rank: int, world: int) -> slice:
    """Columns of the activation a rank multiplies: all of them for a column-parallel weight,
    its K range for a row-parallel one."""
    if axis == COLUMN:
        return slice(0, k)
    return slice(rank * (k // world), (rank + 1) * (k // world))


def combine(outputs, axis: int):
    """What the collective does with the per-rank outputs: concatenate (all-gather) for
    column-parallel, sum (all-reduce) for row-parallel."""
    if axis == COLUMN:
        return np.concatenate(outputs, axis=-1)
    return np.sum(np.stack(outputs), axis=0)
