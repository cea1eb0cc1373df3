"""Two ranks, one process per GPU: the fused collectives against the oracle and NCCL-free.

The parent computes the whole product with the oracle; each child takes its shard of the weights
(rows for the gather, columns for the all-sum), runs the fused product and returns what its own
region / output holds.  Skipped on a box with a single GPU."""
import ctypes as C
import multiprocessing as mp

import numpy as np
import pytest

import oracle

pytestmark = pytest.mark.gpu

SHAPES = [(1, 1024, 4096), (4, 512, 2048), (8, 256, 1024), (1, 6144, 4096)]
ROUNDS = 3


def _child(rank, world, cases, conn):
    try:
        import nuvec_b200 as nv
        from nuvec_b200 import _ffi
        lib = _ffi.lib()
        dev = nv.Device.shared(rank)
        quant = nv.Quant.affine(64, 4)
        qc = quant._c()
        # offsets: per case a gather footprint, then an all-sum footprint
        at, offs = 4096, []
        for M, N, K, *_ in cases:
            g = at
            at += lib.nvc_gather_footprint(world, M, N // world)
            a = at
            at += lib.nvc_all_sum_footprint(world, M, N)
            offs.append((g, a))
        region, handle = C.c_void_p(), (C.c_uint8 * 64)()
        assert lib.nvc_symm_alloc(dev._h, at, C.byref(region), handle) == 0, _ffi.last_error()
        conn.send(bytes(handle))
        handles = conn.recv()
        bases = (C.c_void_p * world)()
        for r in range(world):
            if r == rank:
                bases[r] = region.value
            else:
                hb = (C.c_uint8 * 64).from_buffer_copy(handles[r])
                ptr = C.c_void_p()
                assert lib.nvc_symm_open(dev._h, hb, C.byref(ptr)) == 0, _ffi.last_error()
                bases[r] = ptr.value
        group = C.c_void_p()
        assert lib.nvc_peer_group_create(dev._h, rank, world, bases, at, C.byref(group)) == 0, _ffi.last_error()
        up = lambda a, dt: dev.array(np.ascontiguousarray(a), dt)
        dev_cases = []
        for M, N, K, x, c, s, b in cases:
            nl, kl = N // world, K // world
            rows = slice(rank * nl, (rank + 1) * nl)
            row_shard = (up(c[rows], nv.U32), up(s[rows], nv.BF16), up(b[rows], nv.BF16))
            col_shard = (up(c[:, rank * kl // 8:(rank + 1) * kl // 8], nv.U32), up(s[:, rank * kl // 64:(rank + 1) * kl // 64], nv.BF16),
                         up(b[:, rank * kl // 64:(rank + 1) * kl // 64], nv.BF16))
            dev_cases.append((M, N, K, up(x, nv.BF16), up(x[:, rank * kl:(rank + 1) * kl], nv.BF16), row_shard, col_shard,
                              dev.empty((M, N), nv.BF16)))
        out = []
        for rnd in range(ROUNDS):
            for (M, N, K, x, xk, rs, cs, y), (g, a) in zip(dev_cases, offs):
                rc = lib.nvc_quantized_matmul_gather(dev._h, group, C.byref(qc), x.ptr, rs[0].ptr, rs[1].ptr, rs[2].ptr,
                                                     M, N // world, K, g)
                assert rc == 0, _ffi.last_error()
                rc = lib.nvc_quantized_matmul_all_sum(dev._h, group, C.byref(qc), xk.ptr, cs[0].ptr, cs[1].ptr, cs[2].ptr,
                                                      M, N, K // world, y.ptr, a)
                assert rc == 0, _ffi.last_error()
            assert lib.nvc_synchronize(dev._h) == 0, _ffi.last_error()
        for (M, N, K, x, xk, rs, cs, y), (g, a) in zip(dev_cases, offs):
            gathered = np.empty((world, M, N // world), np.uint16)
            assert lib.nvc_memcpy_d2h(dev._h, gathered.ctypes.data_as(C.c_void_p), C.c_void_p(region.value + g), gathered.nbytes) == 0
            out.append((gathered, y.to_numpy().view(np.uint16)))
        conn.send(("ok", out))
        conn.recv()  # leave together: nobody unmaps a region a peer may still write
    except Exception as e:  # pragma: no cover - reported to the parent
        import traceback
        conn.send(("error", traceback.format_exc()))


def test_two_ranks_gather_and_all_sum_against_the_oracle():
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    from test_gpu_parity import assert_product_tight
    world = 2
    rng = np.random.default_rng(7)
    cases = []
    for M, N, K in SHAPES:
        w = oracle.from_f32((rng.standard_normal((N, K)) * 0.02).astype(np.float32), oracle.BF16)
        c, s, b = oracle.quantize(w, oracle.BF16, oracle.AFFINE, 64, 4)
        x = oracle.from_f32(rng.standard_normal((M, K)).astype(np.float32), oracle.BF16)
        cases.append((M, N, K, x, c, s, b))
    ctx = mp.get_context("spawn")
    pipes, procs = [], []
    for r in range(world):
        parent, child = ctx.Pipe()
        pr = ctx.Process(target=_child, args=(r, world, cases, child))
        pr.start()
        pipes.append(parent)
        procs.append(pr)
    try:
        handles = []
        for p in pipes:
            assert p.poll(120), "a rank did not report its region"
            handles.append(p.recv())
        assert all(isinstance(h, bytes) for h in handles), handles
        for p in pipes:
            p.send(handles)
        results = []
        for p in pipes:
            assert p.poll(180), "a rank did not finish"
            status, payload = p.recv()
            assert status == "ok", payload
            results.append(payload)
        for i, (M, N, K, x, c, s, b) in enumerate(cases):
            want = oracle.quantized_matmul(x, c, s, b, oracle.BF16)
            nl = N // world
            for r in range(world):
                gathered, y = results[r][i]
                # the gather moves bits: every rank holds the oracle-checked slices of all ranks
                full = np.concatenate([gathered[k] for k in range(world)], axis=1)
                assert_product_tight(full, want, oracle.BF16, f"gather case {i} rank {r}")
                assert np.array_equal(gathered, results[0][i][0]), f"gathered buffers differ between ranks (case {i})"
                # the all-sum adds float32 partials in rank order: within one output rounding of the
                # oracle, and the same bits on every rank
                assert_product_tight(y, want, oracle.BF16, f"all-sum case {i} rank {r}")
                assert np.array_equal(y, results[0][i][1]), f"all-sum results differ between ranks (case {i})"
    finally:
        for p in pipes:
            try:
                p.send("bye")
            except Exception:
                pass
        for pr in procs:
            pr.join(30)
            if pr.is_alive():
                pr.kill()


def _comm_child(rank, world, conn):
    try:
        import nuvec_b200 as nv
        from nuvec_b200 import _ffi
        lib = _ffi.lib()
        dev = nv.Device.shared(rank)
        if rank == 0:
            ident = (C.c_uint8 * 128)()
            assert lib.nvc_comm_unique_id(ident) == 0, _ffi.last_error()
            conn.send(bytes(ident))
        ident = (C.c_uint8 * 128).from_buffer_copy(conn.recv())
        comm = C.c_void_p()
        assert lib.nvc_comm_init_timeout(dev._h, rank, world, ident, 120000, C.byref(comm)) == 0, _ffi.last_error()
        assert lib.nvc_comm_rank(comm) == rank and lib.nvc_comm_size(comm) == world
        base = np.arange(1000, dtype=np.float32) * (1 if rank == 0 else -1) + rank
        out = {}
        for name, op in (("sum", 0), ("max", 1), ("min", 2)):
            buf = dev.array(base.copy(), nv.F32)
            assert lib.nvc_all_reduce(comm, op, nv.F32, buf.ptr, base.size) == 0, _ffi.last_error()
            out[name] = buf.to_numpy()
        # ring exchange: send to the next rank, receive from the previous one
        nxt, prv = (rank + 1) % world, (rank - 1) % world
        src = dev.array(np.full(4096, rank + 1, np.uint8), nv.U8)
        dst = dev.array(np.zeros(4096, np.uint8), nv.U8)
        if rank % 2 == 0:
            assert lib.nvc_send(comm, src.ptr, 4096, nxt) == 0, _ffi.last_error()
            assert lib.nvc_recv(comm, dst.ptr, 4096, prv) == 0, _ffi.last_error()
        else:
            assert lib.nvc_recv(comm, dst.ptr, 4096, prv) == 0, _ffi.last_error()
            assert lib.nvc_send(comm, src.ptr, 4096, nxt) == 0, _ffi.last_error()
        out["recv"] = dst.to_numpy()
        gathered = dev.array(np.zeros(world * 8, np.uint8), nv.U8)
        mine = dev.array(np.full(8, 10 + rank, np.uint8), nv.U8)
        assert lib.nvc_all_gather(comm, mine.ptr, gathered.ptr, 8) == 0, _ffi.last_error()
        out["gather"] = gathered.to_numpy()
        assert lib.nvc_comm_health(comm) == 0, _ffi.last_error()
        conn.send(("ok", out))
        conn.recv()
        lib.nvc_comm_destroy(comm)
    except Exception:  # pragma: no cover - reported to the parent
        import traceback
        conn.send(("error", traceback.format_exc()))


def test_two_ranks_nccl_communicator_reduce_ops_send_recv():
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    world = 2
    ctx = mp.get_context("spawn")
    pipes, procs = [], []
    for r in range(world):
        parent, child = ctx.Pipe()
        pr = ctx.Process(target=_comm_child, args=(r, world, child))
        pr.start()
        pipes.append(parent)
        procs.append(pr)
    try:
        assert pipes[0].poll(120)
        ident = pipes[0].recv()
        assert isinstance(ident, bytes), ident
        for p in pipes:
            p.send(ident)
        results = []
        for p in pipes:
            assert p.poll(180), "a rank did not finish"
            status, payload = p.recv()
            assert status == "ok", payload
            results.append(payload)
        a = np.arange(1000, dtype=np.float32)
        b = -a + 1
        for r in range(world):
            assert np.array_equal(results[r]["sum"], a + b)
            assert np.array_equal(results[r]["max"], np.maximum(a, b))
            assert np.array_equal(results[r]["min"], np.minimum(a, b))
            assert np.all(results[r]["recv"] == ((r - 1) % world) + 1)
            assert results[r]["gather"].tolist() == [10] * 8 + [11] * 8
    finally:
        for p in pipes:
            try:
                p.send("bye")
            except Exception:
                pass
        for pr in procs:
            pr.join(30)
            if pr.is_alive():
                pr.kill()
