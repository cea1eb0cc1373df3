"""The NCCL communicator's host-side failure handling, on one GPU and without any GPU fault: a rank
that never joins ends `nvc_comm_init_timeout` with an error after the limit (the half-built
communicator is aborted), and the device stays usable.  Collectives between live ranks are covered
by tests/test_gpu_multi_rank.py."""
import ctypes as C
import time

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def test_comm_init_gives_up_when_a_rank_never_joins():
    import nuvec_b200 as nv
    from nuvec_b200 import _ffi
    lib = _ffi.lib()
    dev = nv.Device.shared(0)
    ident = (C.c_uint8 * 128)()
    assert lib.nvc_comm_unique_id(ident) == 0, _ffi.last_error()
    comm = C.c_void_p()
    t0 = time.perf_counter()
    rc = lib.nvc_comm_init_timeout(dev._h, 0, 2, ident, 2500, C.byref(comm))   # rank 1 never calls
    dt = time.perf_counter() - t0
    assert rc == _ffi.ERR_COMM, _ffi.last_error()
    assert "gave up" in _ffi.last_error() and comm.value is None
    assert 2.0 <= dt < 30.0, dt
    # a communicator of one rank still comes up, and the device goes on working
    assert lib.nvc_comm_unique_id(ident) == 0
    assert lib.nvc_comm_init_timeout(dev._h, 0, 1, ident, 60000, C.byref(comm)) == 0, _ffi.last_error()
    buf = dev.array(np.arange(16, dtype=np.float32), nv.F32)
    assert lib.nvc_all_reduce(comm, 1, nv.F32, buf.ptr, 16) == 0, _ffi.last_error()   # max over one rank
    assert lib.nvc_all_reduce(comm, 7, nv.F32, buf.ptr, 16) == _ffi.ERR_INVALID_ARGUMENT
    assert lib.nvc_send(comm, buf.ptr, 16, 0) == _ffi.ERR_INVALID_ARGUMENT              # no peer to send to
    assert np.array_equal(buf.to_numpy(), np.arange(16, dtype=np.float32))
    assert lib.nvc_comm_destroy(comm) == 0
