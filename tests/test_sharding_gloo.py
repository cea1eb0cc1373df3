"""N-sharded products joined by an all_gather, on two CPU ranks (gloo).

Each rank multiplies its row slice with the CPU oracle, the slices are gathered, and the
result must equal the unsharded product bit for bit (every output column depends only on its
own weight row, so sharding along N changes no arithmetic).
"""
import os
import socket
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank(rank, world, port, out):
    sys.path[:0] = [str(ROOT), str(ROOT / "tests")]
    import torch
    import torch.distributed as dist

    import oracle
    from nuvec_b200 import shard

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        rng = np.random.default_rng(0)  # every rank draws the same tensors
        N, K, M = 96, 256, 3
        w = oracle.from_f32((rng.standard_normal((N, K)) * 0.02).astype(np.float32), oracle.BF16)
        codes, scales, biases = oracle.quantize(w, oracle.BF16, oracle.AFFINE, 64, 4)
        x = oracle.from_f32(rng.standard_normal((M, K)).astype(np.float32), oracle.BF16)
        full = oracle.quantized_matmul(x, codes, scales, biases, oracle.BF16)
        mine = oracle.quantized_matmul(x, shard.shard_rows(codes, world, rank), shard.shard_rows(scales, world, rank),
                                       shard.shard_rows(biases, world, rank), oracle.BF16)
        slots = [torch.zeros(mine.shape, dtype=torch.int32) for _ in range(world)]
        dist.all_gather(slots, torch.from_numpy(mine.astype(np.int32)))
        joined = shard.unshard(np.stack([s.numpy().astype(np.uint16) for s in slots]))
        ok = bool(np.array_equal(joined, full))
        # expert sharding: the ranks' row ranges of a sorted index list are disjoint and cover it
        rhs = np.sort(rng.integers(0, 8, 64)).astype(np.uint32)
        lo, hi = shard.expert_range(8, world, rank)
        offs = oracle.sorted_offsets(rhs, 9 if False else 8)
        first = int(offs[lo])
        last = int(offs[hi]) if hi < 8 else len(rhs)
        counts = [torch.zeros(1, dtype=torch.int64) for _ in range(world)]
        dist.all_gather(counts, torch.tensor([last - first]))
        ok = ok and sum(int(c) for c in counts) == len(rhs) and bool(np.all((rhs[first:last] >= lo) & (rhs[first:last] < hi)))
        out.put((rank, ok))
    finally:
        dist.destroy_process_group()


def test_n_sharded_product_equals_the_unsharded_one():
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_rank, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    results = [out.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert sorted(results) == [(0, True), (1, True)]


def test_row_ranges():
    from nuvec_b200 import shard
    assert [shard.row_range(24576, 8, r) for r in (0, 7)] == [(0, 3072), (21504, 24576)]
    assert shard.expert_range(128, 8, 3) == (48, 64)
    with pytest.raises(ValueError):
        shard.row_range(10, 4, 0)
    g = np.arange(2 * 3 * 4).reshape(2, 3, 4)
    assert shard.unshard(g)[1].tolist() == [4, 5, 6, 7, 16, 17, 18, 19]
