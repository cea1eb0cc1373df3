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


def test_segment_aware_split_keeps_every_rank_in_every_segment():
    # q|k|v of a Qwen3-8B layer: 4096 + 1024 + 1024 rows; the reference gives every rank its share of
    # each segment (shard.rs:34-45), not a flat slice of the fused matrix
    from nuvec_b200 import shard
    import oracle
    segs = [4096, 1024, 1024]
    assert shard.parts(segs, 8, 3) == [(1536, 2048), (4096 + 384, 4096 + 512), (5120 + 384, 5120 + 512)]
    assert shard.parts([12288, 12288], 2, 1) == [(6144, 12288), (18432, 24576)]
    with pytest.raises(ValueError):
        shard.parts([10, 6], 4, 0)
    rng = np.random.default_rng(1)
    segs, K, M, g = [64, 32, 32], 256, 2, 4
    N = sum(segs)
    w = oracle.from_f32((rng.standard_normal((N, K)) * 0.02).astype(np.float32), oracle.BF16)
    c, s, b = oracle.quantize(w, oracle.BF16, oracle.AFFINE, 64, 4)
    x = oracle.from_f32(rng.standard_normal((M, K)).astype(np.float32), oracle.BF16)
    full = oracle.quantized_matmul(x, c, s, b, oracle.BF16)
    slots = np.stack([oracle.quantized_matmul(x, shard.shard_rows(c, g, r, segs), shard.shard_rows(s, g, r, segs),
                                              shard.shard_rows(b, g, r, segs), oracle.BF16) for r in range(g)])
    assert np.array_equal(shard.unshard(slots, segs), full)
    assert not np.array_equal(shard.unshard(slots), full)   # a flat reading of the slots mixes the segments


def test_column_shards_sum_to_the_whole_product():
    from nuvec_b200 import shard
    import oracle
    rng = np.random.default_rng(2)
    N, K, M, g = 48, 512, 3, 4
    w = (rng.standard_normal((N, K)) * 0.02).astype(np.float32)
    c, s, b = oracle.quantize(w, oracle.F32, oracle.AFFINE, 64, 4)
    x = rng.standard_normal((M, K)).astype(np.float32)
    full = oracle.quantized_matmul(x, c, s, b, oracle.F32)
    total = np.zeros_like(full, dtype=np.float64)
    for r in range(g):
        lo, hi = shard.col_range(K, 64, g, r)
        cr, sr, br = shard.shard_cols(c, s, b, 4, 64, g, r)
        total += oracle.quantized_matmul(np.ascontiguousarray(x[:, lo:hi]), cr, sr, br, oracle.F32)
    assert np.allclose(total, full, rtol=1e-5, atol=1e-6)
    with pytest.raises(ValueError):
        shard.col_range(192, 64, 2, 0)   # 96 columns per rank are not whole groups of 64


def test_expert_rows_partition_the_sorted_list():
    from nuvec_b200 import shard
    import oracle
    rng = np.random.default_rng(3)
    E, g = 128, 8
    ids = np.sort(np.concatenate([rng.permutation(E)[:8] for _ in range(512)])).astype(np.uint32)
    offs = oracle.sorted_offsets(ids, E)
    at = 0
    for r in range(g):
        first, last = shard.expert_rows(ids, E, g, r)
        lo, hi = shard.expert_range(E, g, r)
        assert first == at and first == int(offs[lo]) and last == (int(offs[hi]) if hi < E else len(ids))
        assert np.all((ids[first:last] >= lo) & (ids[first:last] < hi))
        at = last
    assert at == len(ids)


def test_row_ranges():
    from nuvec_b200 import shard
    assert [shard.row_range(24576, 8, r) for r in (0, 7)] == [(0, 3072), (21504, 24576)]
    assert shard.expert_range(128, 8, 3) == (48, 64)
    with pytest.raises(ValueError):
        shard.row_range(10, 4, 0)
    g = np.arange(2 * 3 * 4).reshape(2, 3, 4)
    assert shard.unshard(g)[1].tolist() == [4, 5, 6, 7, 16, 17, 18, 19]
