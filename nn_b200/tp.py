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


def k_range(fmt, k: int, rank: int, world: int) -> tuple[int, int]:
    """Blocks [b0, b1) of every row that `rank` keeps of a row-parallel weight: K is dealt out in
    units of 256 weights when it is a multiple of 256 (every shard keeps a tiled layout), else of
    one block; rank r takes units [r * U / world, (r + 1) * U / world), so shards may differ by one
    unit (same arithmetic as nnq_weight_create_shard)."""
    g = GEOMETRY[QuantFormat(fmt)]
    kb = k // g.elems
    per_unit = 256 // g.elems if (k % 256 == 0 and 256 % g.elems == 0) else 1
    units = kb // per_unit
    if units < world:
        raise ValueError(f"{units} units of K cannot be split over {world} ranks")
    return (rank * units // world) * per_unit, ((rank + 1) * units // world) * per_unit


def shard_shape(fmt, n: int, k: int, axis: int, world: int, rank: int = 0) -> tuple[int, int]:
    g = GEOMETRY[QuantFormat(fmt)]
    if axis == COLUMN:
        if n % world:
            raise ValueError(f"out_features {n} not divisible by {world} ranks")
        return n // world, k
    b0, b1 = k_range(fmt, k, rank, world)
    return n, (b1 - b0) * g.elems


def shard_bytes(fmt, raw: np.ndarray, scales, n: int, k: int, axis: int, rank: int, world: int):
    """(main bytes, scale bytes or None) of one rank's shard of an [n, k] weight."""
    g = GEOMETRY[QuantFormat(fmt)]
    kb = k // g.elems
    ns, ks = shard_shape(fmt, n, k, axis, world, rank)
    main = np.ascontiguousarray(raw, np.uint8).reshape(n, kb * g.bytes)
    sc = None if scales is None else np.ascontiguousarray(scales, np.uint8).reshape(n, kb * g.scale_bytes)
    if axis == COLUMN:
        rows = slice(rank * ns, (rank + 1) * ns)
        return main[rows].reshape(-1).copy(), (None if sc is None else sc[rows].reshape(-1).copy())
    b0, b1 = k_range(fmt, k, rank, world)
    cols = slice(b0 * g.bytes, b1 * g.bytes)
    scols = slice(b0 * g.scale_bytes, b1 * g.scale_bytes)
    return main[:, cols].reshape(-1).copy(), (None if sc is None else sc[:, scols].reshape(-1).copy())


def input_slice(k: int, axis: int, rank: int, world: int, fmt=None) -> slice:
    """Columns of the activation a rank multiplies: all of them for a column-parallel weight,
    its K range for a row-parallel one (`fmt` gives the block size; without it K is assumed to
    split evenly)."""
    if axis == COLUMN:
        return slice(0, k)
    if fmt is None:
        return slice(rank * (k // world), (rank + 1) * (k // world))
    g = GEOMETRY[QuantFormat(fmt)]
    b0, b1 = k_range(fmt, k, rank, world)
    return slice(b0 * g.elems, b1 * g.elems)


def combine(outputs, axis: int):
    """What the collective does with the per-rank outputs: concatenate (all-gather) for
    column-parallel, sum (all-reduce) for row-parallel."""
    if axis == COLUMN:
        return np.concatenate(outputs, axis=-1)
    return np.sum(np.stack(outputs), axis=0)
