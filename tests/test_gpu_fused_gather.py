"""The products fused with their collective (nvc_quantized_matmul_gather, nvc_quantized_matmul_all_sum)
on one GPU: a peer group of a single rank exercises the kernel's whole protocol -- the sequence
count, the packets, the stores into the gathered buffer of the region -- against the plain product;
a group whose second region is more memory of the same GPU shows the bounded wait giving up.  The
multi-rank cases need one process per GPU: tests/test_gpu_multi_rank.py."""
import ctypes as C

import numpy as np
import pytest

import oracle

pytestmark = pytest.mark.gpu


def test_single_rank_group_matches_the_plain_product():
    import nuvec_b200 as nv
    from nuvec_b200 import _ffi
    lib = _ffi.lib()
    dev = nv.Device.shared(0)
    rng = np.random.default_rng(3)
    quant = nv.Quant.affine(64, 4)
    qc = quant._c()
    shapes = [(1, 6144, 4096), (4, 1024, 2048), (8, 4096, 4096), (1, 40, 2880 // 64 * 64)]
    RES = 4096
    offsets, at = [], RES
    for M, N, K in shapes:
        offsets.append(at)
        at += lib.nvc_gather_footprint(1, M, N)
    region, handle = C.c_void_p(), (C.c_uint8 * 64)()
    assert lib.nvc_symm_alloc(dev._h, at, C.byref(region), handle) == 0, _ffi.last_error()
    bases = (C.c_void_p * 1)(region.value)
    group = C.c_void_p()
    assert lib.nvc_peer_group_create(dev._h, 0, 1, bases, at, C.byref(group)) == 0, _ffi.last_error()
    try:
        cases = []
        for M, N, K in shapes:
            w = oracle.from_f32((rng.standard_normal((N, K)) * 0.02).astype(np.float32), oracle.BF16)
            q = nv.quantize(dev.array(w, nv.BF16), quant)
            x = dev.array(oracle.from_f32(rng.standard_normal((M, K)).astype(np.float32), oracle.BF16), nv.BF16)
            cases.append((M, N, K, q, x, nv.quantized_matmul(x, q).to_numpy()))
        for rounds in range(3):  # the sequence count and the flags advance from call to call
            for (M, N, K, q, x, want), off in zip(cases, offsets):
                rc = lib.nvc_quantized_matmul_gather(dev._h, group, C.byref(qc), x.ptr, q.weight.ptr, q.scales.ptr,
                                                     q.biases.ptr, M, N, K, off)
                assert rc == 0, _ffi.last_error()
            dev.synchronize()
            for (M, N, K, q, x, want), off in zip(cases, offsets):
                got = np.empty((M, N), np.uint16)
                assert lib.nvc_memcpy_d2h(dev._h, got.ctypes.data_as(C.c_void_p), C.c_void_p(region.value + off), got.nbytes) == 0
                assert np.array_equal(got, want.view(np.uint16).reshape(M, N))
        # the all-sum of a single rank is the plain product: one float32 partial, rounded once
        scratch = offsets[0]
        for M, N, K, q, x, want in cases:
            if lib.nvc_all_sum_footprint(1, M, N) > at - scratch:
                continue
            y = dev.empty((M, N), nv.BF16)
            rc = lib.nvc_quantized_matmul_all_sum(dev._h, group, C.byref(qc), x.ptr, q.weight.ptr, q.scales.ptr,
                                                  q.biases.ptr, M, N, K, y.ptr, scratch)
            assert rc == 0, _ffi.last_error()
            assert np.array_equal(y.to_numpy(), want)
        rounds_done = 3 * len(shapes) + sum(1 for M, N, K, *_ in cases if lib.nvc_all_sum_footprint(1, M, N) <= at - scratch)
        head = np.empty(18, np.uint32)
        assert lib.nvc_memcpy_d2h(dev._h, head.ctypes.data_as(C.c_void_p), region, head.nbytes) == 0
        assert head[0] == rounds_done and head[16] == rounds_done and head[17] == 0
    finally:
        lib.nvc_peer_group_destroy(group)
        lib.nvc_symm_free(dev._h, region)


def test_gather_arguments_are_checked():
    import nuvec_b200 as nv
    from nuvec_b200 import _ffi
    lib = _ffi.lib()
    dev = nv.Device.shared(0)
    region, handle = C.c_void_p(), (C.c_uint8 * 64)()
    assert lib.nvc_symm_alloc(dev._h, 100, C.byref(region), handle) == _ffi.ERR_INVALID_ARGUMENT
    bases = (C.c_void_p * 1)(None)
    group = C.c_void_p()
    assert lib.nvc_peer_group_create(dev._h, 0, 1, bases, 1 << 20, C.byref(group)) == _ffi.ERR_INVALID_ARGUMENT
    assert lib.nvc_peer_group_create(dev._h, 2, 2, bases, 1 << 20, C.byref(group)) == _ffi.ERR_INVALID_ARGUMENT
    # offsets and footprints are checked against the region's size before anything is launched
    import numpy as np
    quant = nv.Quant.affine(64, 4)
    qc = quant._c()
    M, N, K = 1, 256, 1024
    size = 4096 + lib.nvc_gather_footprint(1, M, N)
    assert lib.nvc_symm_alloc(dev._h, size, C.byref(region), handle) == 0, _ffi.last_error()
    bases = (C.c_void_p * 1)(region.value)
    assert lib.nvc_peer_group_create(dev._h, 0, 1, bases, 100, C.byref(group)) == _ffi.ERR_INVALID_ARGUMENT
    assert lib.nvc_peer_group_create(dev._h, 0, 1, bases, size, C.byref(group)) == 0, _ffi.last_error()
    try:
        rng = np.random.default_rng(0)
        q = nv.quantize(dev.array(oracle.from_f32((rng.standard_normal((N, K)) * 0.02).astype(np.float32), oracle.BF16), nv.BF16), quant)
        x = dev.array(oracle.from_f32(rng.standard_normal((M, K)).astype(np.float32), oracle.BF16), nv.BF16)
        args = (dev._h, group, C.byref(qc), x.ptr, q.weight.ptr, q.scales.ptr, q.biases.ptr, M, N, K)
        assert lib.nvc_quantized_matmul_gather(*args, 4096 + 256) == _ffi.ERR_INVALID_ARGUMENT   # past the end of the region
        assert "does not fit" in _ffi.last_error()
        assert lib.nvc_quantized_matmul_gather(*args, 2048) == _ffi.ERR_INVALID_ARGUMENT         # inside the reserved head
        assert lib.nvc_quantized_matmul_gather(*args, 4096 + 8) == _ffi.ERR_INVALID_ARGUMENT     # not a multiple of 256
        inside = C.c_void_p(region.value + 4096)   # activations that overlap the product's own buffers
        assert lib.nvc_quantized_matmul_gather(dev._h, group, C.byref(qc), inside, q.weight.ptr, q.scales.ptr, q.biases.ptr,
                                               M, N, K, 4096) == _ffi.ERR_INVALID_ARGUMENT
        y = dev.empty((M, N), nv.BF16)
        assert lib.nvc_quantized_matmul_all_sum(*args, y.ptr, 4096 + 4096) == _ffi.ERR_INVALID_ARGUMENT
        assert lib.nvc_quantized_matmul_gather(*args, 4096) == 0, _ffi.last_error()
        assert lib.nvc_synchronize(dev._h) == 0
    finally:
        lib.nvc_peer_group_destroy(group)
        lib.nvc_symm_free(dev._h, region)


def test_a_rank_that_never_shows_up_ends_the_wait_with_an_error():
    """Failure detection without a fault: a group of two ranks whose second region is just more
    memory of this GPU -- nobody ever raises rank 1's flag.  The kernel's bounded wait runs out
    (about a second), the kernel returns, nvc_synchronize reports the failure, and the device
    stays usable."""
    import nuvec_b200 as nv
    from nuvec_b200 import _ffi
    lib = _ffi.lib()
    dev = nv.Device.shared(0)
    rng = np.random.default_rng(4)
    quant = nv.Quant.affine(64, 4)
    qc = quant._c()
    M, N, K = 1, 256, 1024
    size = 4096 + lib.nvc_gather_footprint(2, M, N)
    r0, r1, h = C.c_void_p(), C.c_void_p(), (C.c_uint8 * 64)()
    assert lib.nvc_symm_alloc(dev._h, size, C.byref(r0), h) == 0, _ffi.last_error()
    assert lib.nvc_symm_alloc(dev._h, size, C.byref(r1), h) == 0, _ffi.last_error()
    bases = (C.c_void_p * 2)(r0.value, r1.value)
    group = C.c_void_p()
    assert lib.nvc_peer_group_create(dev._h, 0, 2, bases, size, C.byref(group)) == 0, _ffi.last_error()
    try:
        w = oracle.from_f32((rng.standard_normal((N, K)) * 0.02).astype(np.float32), oracle.BF16)
        q = nv.quantize(dev.array(w, nv.BF16), quant)
        x = dev.array(oracle.from_f32(rng.standard_normal((M, K)).astype(np.float32), oracle.BF16), nv.BF16)
        want = nv.quantized_matmul(x, q).to_numpy()
        rc = lib.nvc_quantized_matmul_gather(dev._h, group, C.byref(qc), x.ptr, q.weight.ptr, q.scales.ptr,
                                             q.biases.ptr, M, N, K, 4096)
        assert rc == 0, _ffi.last_error()
        assert lib.nvc_synchronize(dev._h) == _ffi.ERR_DRIVER
        assert "gave up waiting" in _ffi.last_error()
        # this rank's slice did reach its own gathered buffer, and its packets the other region, before the wait gave up
        got = np.empty((M, N), np.uint16)
        assert lib.nvc_memcpy_d2h(dev._h, got.ctypes.data_as(C.c_void_p), C.c_void_p(r0.value + 4096), got.nbytes) == 0
        assert np.array_equal(got, want.view(np.uint16).reshape(M, N))
        packets = np.empty((M * N, 2), np.uint32)
        area = 4096 + (2 * M * N * 2 + 255) // 256 * 256 + 2 * M * N * 8   # sequence number 1: the odd half, rank 0's slots first
        assert lib.nvc_memcpy_d2h(dev._h, packets.ctypes.data_as(C.c_void_p), C.c_void_p(r1.value + area), packets.nbytes) == 0
        assert np.all(packets[:, 1] == 1) and np.array_equal(packets[:, 0].astype(np.uint16), want.view(np.uint16).reshape(-1))
        # and the device goes on working
        assert lib.nvc_synchronize(dev._h) == 0
        assert np.array_equal(nv.quantized_matmul(x, q).to_numpy(), want)
    finally:
        lib.nvc_peer_group_destroy(group)
        lib.nvc_symm_free(dev._h, r0)
        lib.nvc_symm_free(dev._h, r1)
