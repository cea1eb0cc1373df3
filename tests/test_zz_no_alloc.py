"""The entry point that allocates nothing, against the ordinary one (through the C ABI).

`nvc_quantized_matmul_noalloc` serves callers that hold a fixed device-memory reservation while
they run -- a serving loop under a memory budget, a plugin inside a runtime that owns the
allocator -- and so cannot let a library call cudaMalloc behind their back.  Its scratch is a
fixed array inside the library; everything else is the same kernel, so the two entry points must
agree bit for bit.  Two calls in a row check that what the first call leaves in the shared array
does not disturb the second.  The file sorts last so that a run stopping at the first failure
has already run every other test.
"""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def test_noalloc_entry_point_matches_the_pooled_one_twice_in_a_row():
    import nuvec_b200 as nv
    from nuvec_b200 import _ffi

    dev, lib = nv.Device.shared(0), _ffi.lib()
    rng = np.random.default_rng(42)
    quant = nv.Quant.affine(64, 4)
    qc = quant._c()
    # (the third product has the height of a vocabulary projection: the fixed array serves any N)
    for call, (M, N, K) in enumerate([(1, 4096, 4096), (5, 1000, 2048), (1, 151936, 1024)]):
        w = nv.f32_to_bf16((rng.standard_normal((N, K)) * 0.02).astype(np.float32))
        x = dev.array(nv.f32_to_bf16(rng.standard_normal((M, K)).astype(np.float32)), nv.BF16)
        q = nv.quantize(dev.array(w, nv.BF16), quant)
        want = nv.quantized_matmul(x, q).to_numpy()
        before = dev.memory()["allocations"]
        y = dev.empty((M, N), nv.BF16)
        after_output = dev.memory()["allocations"]
        rc = lib.nvc_quantized_matmul_noalloc(dev._h, C.byref(qc), x.ptr, q.weight.ptr, q.scales.ptr, q.biases.ptr,
                                              M, N, K, y.ptr)
        assert rc == 0, _ffi.last_error()
        got = y.to_numpy()
        assert np.array_equal(got, want), f"call {call}: {np.count_nonzero(got != want)} of {got.size} values differ"
        # the pool saw no allocation from the call itself (the output buffer is the caller's)
        assert dev.memory()["allocations"] == after_output >= before


def test_noalloc_entry_point_rejects_what_its_fixed_scratch_cannot_hold():
    import nuvec_b200 as nv
    from nuvec_b200 import _ffi

    dev, lib = nv.Device.shared(0), _ffi.lib()
    qc = nv.Quant.affine(64, 4)._c()
    one = dev.empty((16,), nv.U32)
    # 9 rows of x are beyond the few-row kernel; 19 tiles of 512 iterations spread over every
    # multiprocessor can each be cut into 130 parts, which is more partial tiles than the array holds
    for M, N, K, words in [(9, 64, 64, "no-alloc"), (1, 304, 65536, "fixed scratch")]:
        rc = lib.nvc_quantized_matmul_noalloc(dev._h, C.byref(qc), one.ptr, one.ptr, one.ptr, one.ptr, M, N, K, one.ptr)
        assert rc == _ffi.ERR_UNSUPPORTED, (M, N, K, rc)
        assert words in _ffi.last_error(), _ffi.last_error()
