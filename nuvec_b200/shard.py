"""Sharding of quantized weights across ranks and the layouts of the joined products.

Rows (N-sharding).  The reference shards a projection by slicing rows of the packed weights, scales
and biases (`Projection::rows`, crates/nuvec-lm/src/model/shard.rs:80-106) and joins N-sharded
outputs with an all_gather that concatenates along axis 0
(crates/nuvec-core/src/distributed.rs:695-700, crates/nuvec-lm/src/model.rs:3336-3346).  Each rank's
product [M, N/g] lands in slot `rank` of a [g, M, N/g] buffer; `unshard` turns that buffer into the
[M, N] result.  A fused projection (q|k|v, gate|up) is split segment by segment, so that every rank
holds its share of every segment (`parts`, shard.rs:34-45, used by `Mlp::shard` :241-256 and the
attention :266-330).

Columns (K-sharding).  The layer that consumes an N-sharded output is sharded along its input
columns in whole quantization groups (`Projection::cols`, shard.rs:108-145) and its partial products
are summed across ranks (`ShardedToAllLinear`, crates/nuvec-nn/src/sharded.rs:137-202).

Experts.  The benchmark's mixture-of-experts configuration shards along experts (the reference shards
experts along their intermediate axis instead, shard.rs:230-239): rank r owns experts
[r E/g, (r+1) E/g) and, because the gathered rows are sorted by expert, a contiguous slice of them.
"""
from __future__ import annotations

from typing import Sequence

import numpy as np


def row_range(n: int, world: int, rank: int) -> tuple[int, int]:
    """Rows [lo, hi) of an N-row matrix owned by `rank`; N must divide evenly (as the reference
    requires of sharded dimensions, crates/nuvec-nn/src/sharded.rs:84-106)."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"rank {rank} of {world}")
    if n % world != 0:
        raise ValueError(f"{n} rows do not divide over {world} ranks")
    per = n // world
    return rank * per, (rank + 1) * per


def parts(segments: Sequence[int], world: int, rank: int) -> list[tuple[int, int]]:
    """Rank `rank`'s part [r len/n, (r+1) len/n) of each segment, in segment order (shard.rs:34-45)."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"rank {rank} of {world}")
    out, at = [], 0
    for length in segments:
        if length % world != 0:
            raise ValueError(f"a segment of {length} rows does not divide over {world} ranks")
        out.append((at + rank * length // world, at + (rank + 1) * length // world))
        at += length
    return out


def shard_rows(a: np.ndarray, world: int, rank: int, segments: Sequence[int] | None = None) -> np.ndarray:
    """The rank's rows of an array whose second-to-last axis is the weight-row axis; with `segments`
    (the row counts of the fused projections, summing to the axis) its part of every segment."""
    n = a.shape[-2]
    if segments is None:
        segments = [n]
    if sum(segments) != n:
        raise ValueError(f"segments {list(segments)} do not add up to {n} rows")
    pieces = [a[..., lo:hi, :] for lo, hi in parts(segments, world, rank)]
    return np.ascontiguousarray(pieces[0] if len(pieces) == 1 else np.concatenate(pieces, axis=-2))


def unshard(gathered: np.ndarray, segments: Sequence[int] | None = None) -> np.ndarray:
    """[g, M, N/g] (slot r = rank r's columns) -> [M, N]; with `segments` the ranks' parts go back
    to their places inside each segment."""
    g, m, per = gathered.shape
    if segments is None:
        return np.ascontiguousarray(np.transpose(gathered, (1, 0, 2)).reshape(m, g * per))
    if sum(segments) != g * per:
        raise ValueError(f"segments {list(segments)} do not add up to {g * per} columns")
    out = np.empty((m, g * per), gathered.dtype)
    at_local = 0
    for (lo0, _), length in zip(parts(segments, g, 0), segments):
        share = length // g
        for r in range(g):
            out[:, lo0 + r * share:lo0 + (r + 1) * share] = gathered[r, :, at_local:at_local + share]
        at_local += share
    return out


def col_range(k: int, group_size: int, world: int, rank: int) -> tuple[int, int]:
    """Input columns [lo, hi) owned by `rank` when a layer is sharded along K: whole quantization
    groups only (`Projection::cols`, shard.rs:108-145)."""
    lo, hi = row_range(k, world, rank)
    if (hi - lo) % group_size != 0:
        raise ValueError(f"{k} columns over {world} ranks do not split into whole groups of {group_size}")
    return lo, hi


def shard_cols(codes: np.ndarray, scales: np.ndarray, biases, bits: int, group_size: int, world: int, rank: int):
    """The rank's columns of a quantized matrix: packed words, scales and biases sliced consistently."""
    k = codes.shape[-1] * 32 // bits
    lo, hi = col_range(k, group_size, world, rank)
    if (lo * bits) % 32 != 0 or (hi * bits) % 32 != 0:
        raise ValueError("the column range does not fall on packed-word boundaries")
    c = np.ascontiguousarray(codes[..., lo * bits // 32:hi * bits // 32])
    s = np.ascontiguousarray(scales[..., lo // group_size:hi // group_size])
    b = None if biases is None else np.ascontiguousarray(biases[..., lo // group_size:hi // group_size])
    return c, s, b


def expert_range(experts: int, world: int, rank: int) -> tuple[int, int]:
    """Experts [lo, hi) owned by `rank` (expert-sharded mixture of experts)."""
    return row_range(experts, world, rank)


def expert_rows(sorted_ids: np.ndarray, experts: int, world: int, rank: int) -> tuple[int, int]:
    """Gathered rows [first, last) of a list sorted by expert that belong to `rank`'s experts: the slice
    between the sorted offsets (crates/nuvec-core/src/kernels.rs:875-892) of its first expert and of
    the next rank's first expert."""
    lo, hi = expert_range(experts, world, rank)
    ids = np.asarray(sorted_ids)
    return int(np.searchsorted(ids, lo, side="left")), int(np.searchsorted(ids, hi, side="left"))
