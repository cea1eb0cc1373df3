"""Host-side logic and the C-ABI surface, without a GPU."""
import re
from pathlib import Path

import numpy as np
import pytest

import nuvec_b200 as nv
from nuvec_b200 import _ffi

ROOT = Path(__file__).resolve().parent.parent


def test_library_loads_and_exports_every_declared_symbol():
    header = (ROOT / "include" / "nuvec_cuda.h").read_text()
    declared = set(re.findall(r"\b(nvc_[a-z0-9_]+)\s*\(", header))
    declared -= {"nvc_alloc"} - set(_ffi.SIGNATURES)  # nothing excluded: keep the set as parsed
    assert declared, "no declarations parsed"
    lib = _ffi.lib()
    missing = [name for name in sorted(declared) if not hasattr(lib, name)]
    assert not missing, f"libnuvec_cuda.so lacks {missing}"
    assert declared == set(_ffi.SIGNATURES), declared ^ set(_ffi.SIGNATURES)
    assert b"sm_100a" in lib.nvc_version()


def test_no_device_is_an_error_not_a_fallback():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a device is present")
    with pytest.raises(nv.NoDevice):
        nv.Device(0)


def test_quant_checked_follows_the_reference_rules():
    assert nv.Quant() == nv.Quant.affine(64, 4)
    assert nv.Quant.new(nv.QuantMode.MXFP4) == nv.Quant(nv.QuantMode.MXFP4, 32, 4)
    assert nv.Quant.new(nv.QuantMode.NVFP4) == nv.Quant(nv.QuantMode.NVFP4, 16, 4)
    assert nv.Quant.new(nv.QuantMode.MXFP8) == nv.Quant(nv.QuantMode.MXFP8, 32, 8)
    for g in (32, 64, 128):
        for b in (1, 2, 3, 4, 5, 6, 8):
            assert nv.Quant.affine(g, b).checked("t") == (g, b)
    for bad in (nv.Quant.affine(48, 4), nv.Quant.affine(64, 7), nv.Quant.affine(64, 0),
                nv.Quant(nv.QuantMode.MXFP4, 64, 4), nv.Quant(nv.QuantMode.NVFP4, 16, 8),
                nv.Quant(nv.QuantMode.MXFP8, 32, 4)):
        with pytest.raises(nv.InvalidArgument):
            bad.checked("t")
    with pytest.raises(nv.InvalidArgument):
        nv.QuantMode.parse("int4")
    assert nv.QuantMode.parse("nvfp4") is nv.QuantMode.NVFP4


def test_grouped_rule():
    # crates/nuvec-core/src/quantized.rs:724-731
    assert nv.GatherQmm.groups(4096, 128) and nv.GatherQmm.groups(4096, 32) and nv.GatherQmm.groups(16, 4)
    assert not nv.GatherQmm.groups(8, 128) and not nv.GatherQmm.groups(15, 1) and not nv.GatherQmm.groups(64, 32)
    assert nv.GatherQmm().transpose and not nv.GatherQmm().sorted_indices


def test_bf16_helpers_round_to_nearest_even():
    x = np.array([1.0, 1.0 + 2.0 ** -8, 1.0 + 3 * 2.0 ** -8, -2.5, 0.0, np.inf], np.float32)
    assert nv.f32_to_bf16(x).tolist() == [0x3F80, 0x3F80, 0x3F82, 0xC020, 0, 0x7F80]
    assert np.array_equal(nv.bf16_to_f32(nv.f32_to_bf16(x))[[0, 3, 4, 5]], x[[0, 3, 4, 5]])


def test_pool_size_classes_match_the_reference():
    # crates/nuvec-gpu/src/cuda/memory.rs:54-60 restated for the documentation of nvc_alloc.
    def size_class(n):
        if n <= 8:
            return 8
        if n < 16 << 10:
            return 1 << (n - 1).bit_length()
        page = 16 << 10
        return (n + page - 1) // page * page
    assert [size_class(n) for n in (1, 8, 9, 1000, 16383, 16384, 16385, 100000)] == \
        [8, 8, 16, 1024, 16384, 16384, 32768, 114688]
