"""Row sharding of quantized weights across ranks and the layout of the gathered product.

The reference shards a projection by slicing rows of the packed weights, scales and biases
(`Projection::rows`, crates/nuvec-lm/src/model/shard.rs:80-106) and joins N-sharded outputs with
an all_gather that concatenates along axis 0 (crates/nuvec-core/src/distributed.rs:695-700,
crates/nuvec-lm/src/model.rs:3336-3346).  Each rank's product [M, N/g] lands in slot `rank` of a
[g, M, N/g] buffer; `unshard` turns that buffer into the [M, N] result.
"""
from __future__ import annotations

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


def shard_rows(a: np.ndarray, world: int, rank: int) -> np.ndarray:
    """The rank's slice of an array whose second-to-last axis is the weight-row axis."""
    lo, hi = row_range(a.shape[-2], world, rank)
    return np.ascontiguousarray(a[..., lo:hi, :])


def unshard(gathered: np.ndarray) -> np.ndarray:
    """[g, M, N/g] (slot r = rank r's columns) -> [M, N]."""
    g, m, per = gathered.shape
    return np.ascontiguousarray(np.transpose(gathered, (1, 0, 2)).reshape(m, g * per))


def expert_range(experts: int, world: int, rank: int) -> tuple[int, int]:
    """Experts [lo, hi) owned by `rank` (expert-sharded mixture of experts)."""
    return row_range(experts, world, rank)
