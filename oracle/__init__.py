"""ctypes front end of the CPU oracle.  TEST INFRASTRUCTURE ONLY.

Only the tests, ``__graft_entry__.smoke`` and the CPU-baseline legs of ``bench.py`` may import
this package; the product package ``nuvec_b200`` never does.

Arrays are numpy.  float16 and bfloat16 data travel as ``uint16`` bit patterns together with
an explicit dtype code (``F16``/``BF16``/``F32``, nuvec's DType numbering).
"""
from __future__ import annotations

import ctypes
import hashlib
import subprocess
from pathlib import Path

import numpy as np

U8, U32, F16, BF16, F32 = 1, 3, 9, 10, 11
AFFINE, MXFP4, MXFP8, NVFP4 = 0, 1, 2, 3
MODES = {"affine": AFFINE, "mxfp4": MXFP4, "mxfp8": MXFP8, "nvfp4": NVFP4}

_HERE = Path(__file__).resolve().parent
_LIB = None


def build(force: bool = False) -> Path:
    """Compiles the oracle with gcc if the shared object is missing or stale."""
    so = _HERE / "libnuvec_oracle.so"
    srcs = [_HERE / "nuvec_oracle.c", _HERE / "nuvec_oracle.h"]
    # The object is compiled with -march=native: rebuild when it was made on another CPU.
    stamp, host = _HERE / "libnuvec_oracle.so.host", _host_id()
    stale = (not so.exists() or not stamp.exists() or stamp.read_text() != host
             or any(s.stat().st_mtime > so.stat().st_mtime for s in srcs))
    if force or stale:
        subprocess.run(["make", "-C", str(_HERE), "-B", "libnuvec_oracle.so"], check=True,
                       capture_output=True)
        stamp.write_text(host)
    return so


def _host_id() -> str:
    try:
        for line in open("/proc/cpuinfo"):
            if line.startswith("flags"):
                return hashlib.sha1(line.encode()).hexdigest()
    except OSError:
        pass
    return "unknown"


def lib():
    global _LIB
    if _LIB is None:
        _LIB = ctypes.CDLL(str(build()))
        _LIB.orc_last_error.restype = ctypes.c_char_p
        for name in ("orc_e4m3_to_f32", "orc_e2m1_to_f32", "orc_e8m0_to_f32",
                     "orc_mx_scale_round_up", "orc_bf16_to_f32", "orc_f16_to_f32"):
            getattr(_LIB, name).restype = ctypes.c_float
        for name in ("orc_e4m3_from_f32", "orc_e2m1_from_f32", "orc_e8m0_from_f32"):
            getattr(_LIB, name).restype = ctypes.c_uint8
            getattr(_LIB, name).argtypes = [ctypes.c_float]
        for name in ("orc_e4m3_to_f32", "orc_e2m1_to_f32", "orc_e8m0_to_f32"):
            getattr(_LIB, name).argtypes = [ctypes.c_uint8]
        _LIB.orc_mx_scale_round_up.argtypes = [ctypes.c_float]
        _LIB.orc_f32_to_bf16.restype = ctypes.c_uint16
        _LIB.orc_f32_to_bf16.argtypes = [ctypes.c_float]
        _LIB.orc_f64_to_f16.restype = ctypes.c_uint16
        _LIB.orc_f64_to_f16.argtypes = [ctypes.c_double]
    return _LIB


class OracleError(ValueError):
    pass


def _check(rc):
    if rc != 0:
        raise OracleError(lib().orc_last_error().decode())


def _ptr(a):
    return None if a is None else a.ctypes.data_as(ctypes.c_void_p)


def _c(a, dtype=None):
    if a is None:
        return None
    return np.ascontiguousarray(a, dtype=dtype)


def _sz(n):
    return ctypes.c_size_t(int(n))


def store_dtype(code):
    """numpy storage dtype for a float dtype code."""
    return np.float32 if code == F32 else np.uint16


def to_f32(a, code):
    """Widens an array stored as `code` to float32 (exact)."""
    a = np.asarray(a)
    if code == F32:
        return a.astype(np.float32, copy=False)
    if code == F16:
        return a.view(np.float16).astype(np.float32)
    return (a.astype(np.uint32) << 16).view(np.float32)


def from_f32(a, code):
    """Rounds float32 to `code` (nearest even), returning the storage array."""
    a = np.ascontiguousarray(a, dtype=np.float32)
    if code == F32:
        return a
    if code == F16:
        return a.astype(np.float16).view(np.uint16)
    u = a.view(np.uint32)
    nan = (u & 0x7FFFFFFF) > 0x7F800000
    r = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)
    return np.where(nan, ((u >> 16) | 0x40).astype(np.uint16), r)


def quantize(w, dtype, mode=AFFINE, group_size=64, bits=4, global_scale=None):
    """w: [..., cols] stored as `dtype`.  Returns (codes u32, scales, biases|None)."""
    w = _c(w)
    cols = w.shape[-1]
    rows = w.size // cols if cols else 0
    codes = np.zeros(w.shape[:-1] + (cols * bits // 32,), np.uint32)
    gshape = w.shape[:-1] + (cols // group_size if group_size else 0,)
    if mode == AFFINE:
        scales = np.zeros(gshape, store_dtype(dtype))
        biases = np.zeros(gshape, store_dtype(dtype))
    else:
        scales, biases = np.zeros(gshape, np.uint8), None
    g = None if global_scale is None else _c(np.asarray(global_scale, np.float32).reshape(1))
    _check(lib().orc_quantize(mode, group_size, bits, dtype, _ptr(w), _sz(rows), _sz(cols),
                              _ptr(g), _ptr(codes), _ptr(scales), _ptr(biases)))
    return codes, scales, biases


def dequantize(codes, scales, biases, dtype, mode=AFFINE, group_size=64, bits=4,
               global_scale=None, fused=False):
    codes, scales, biases = _c(codes, np.uint32), _c(scales), _c(biases)
    cols = codes.shape[-1] * 32 // bits
    rows = codes.size // codes.shape[-1] if codes.shape[-1] else 0
    out = np.zeros(codes.shape[:-1] + (cols,), store_dtype(dtype))
    g = None if global_scale is None else _c(np.asarray(global_scale, np.float32).reshape(1))
    _check(lib().orc_dequantize(mode, group_size, bits, dtype, _ptr(codes), _ptr(scales),
                                _ptr(biases), _ptr(g), _sz(rows), _sz(cols), _ptr(out),
                                int(fused)))
    return out


def sorted_offsets(indices, groups):
    idx = _c(indices, np.uint32).reshape(-1)
    out = np.zeros(groups, np.int32)
    _check(lib().orc_sorted_offsets(_ptr(idx), _sz(idx.size), _sz(groups), _ptr(out)))
    return out


def quantized_matmul(x, codes, scales, biases, dtype, mode=AFFINE, group_size=64, bits=4,
                     transpose=True, global_scale=None, parallel_dequant=True):
    """2-D product: x [M, K] (storage of `dtype`) with one quantized matrix."""
    x, codes, scales, biases = _c(x), _c(codes, np.uint32), _c(scales), _c(biases)
    M, K = x.shape
    N = codes.shape[0] if transpose else codes.shape[1] * 32 // bits
    y = np.zeros((M, N), store_dtype(dtype))
    g = None if global_scale is None else _c(np.asarray(global_scale, np.float32).reshape(1))
    _check(lib().orc_quantized_matmul(mode, group_size, bits, dtype, int(transpose), _ptr(x),
                                      _ptr(codes), _ptr(scales), _ptr(biases), _ptr(g), _sz(M),
                                      _sz(N), _sz(K), _ptr(y), int(parallel_dequant)))
    return y


def gather_qmm(x, codes, scales, biases, lhs, rhs, dtype, mode=AFFINE, group_size=64, bits=4,
               transpose=True, global_scale=None, parallel_dequant=True):
    """x [B, M, K]; codes [E, rows, words]; lhs/rhs flat u32 index lists of equal length."""
    x, codes, scales, biases = _c(x), _c(codes, np.uint32), _c(scales), _c(biases)
    lhs, rhs = _c(lhs, np.uint32).reshape(-1), _c(rhs, np.uint32).reshape(-1)
    _, M, K = x.shape
    E = codes.shape[0]
    N = codes.shape[1] if transpose else codes.shape[2] * 32 // bits
    y = np.zeros((rhs.size, M, N), store_dtype(dtype))
    g = None if global_scale is None else _c(np.asarray(global_scale, np.float32).reshape(-1))
    _check(lib().orc_gather_qmm(mode, group_size, bits, dtype, int(transpose), _ptr(x),
                                _ptr(codes), _ptr(scales), _ptr(biases), _ptr(g), _ptr(lhs),
                                _ptr(rhs), _sz(rhs.size), _sz(M), _sz(N), _sz(K), _sz(E),
                                _ptr(y), int(parallel_dequant)))
    return y


def moe_route(probs, dtype, k, normalize=True):
    """probs [..., E] stored as `dtype` -> (indices uint32 [..., k], scores [..., k])."""
    probs = _c(probs)
    e = probs.shape[-1]
    rows = probs.size // e if e else 0
    idx = np.zeros(probs.shape[:-1] + (k,), np.uint32)
    scores = np.zeros(probs.shape[:-1] + (k,), store_dtype(dtype))
    _check(lib().orc_moe_route(dtype, _ptr(probs), _sz(rows), _sz(e), _sz(k), int(normalize), _ptr(idx), _ptr(scores)))
    return idx, scores


def weighted_sum(x, w, dtype):
    """x [..., k, D], w [..., k] -> [..., D]."""
    x, w = _c(x), _c(w)
    k, d = x.shape[-2], x.shape[-1]
    rows = x.size // (k * d) if k * d else 0
    out = np.zeros(x.shape[:-2] + (d,), store_dtype(dtype))
    _check(lib().orc_weighted_sum(dtype, _ptr(x), _ptr(w), _sz(rows), _sz(k), _sz(d), _ptr(out)))
    return out


def expert_bias_add(y, bias, indices, dtype):
    """y [rows, n] + bias[indices] ([experts, n]); returns a new array."""
    out = np.array(_c(y), copy=True)
    bias, idx = _c(bias), _c(indices, np.uint32).reshape(-1)
    n = out.shape[-1]
    rows = out.size // n if n else 0
    _check(lib().orc_expert_bias_add(dtype, _ptr(out), _ptr(bias), _ptr(idx), _sz(rows), _sz(n), _sz(bias.shape[0])))
    return out


def moe_sort(indices, experts):
    """indices [..., k] -> (order, restore, tokens, sorted) uint32 [pairs] and offsets int32 [experts]."""
    idx = _c(indices, np.uint32)
    k = idx.shape[-1]
    flat = idx.reshape(-1)
    n = flat.size
    order, restore, tokens, srt = (np.zeros(n, np.uint32) for _ in range(4))
    offsets = np.zeros(experts, np.int32)
    _check(lib().orc_moe_sort(_ptr(flat), _sz(n), _sz(k), _sz(experts), _ptr(order), _ptr(restore), _ptr(tokens), _ptr(srt), _ptr(offsets)))
    return order, restore, tokens, srt, offsets


def swiglu(gate, up, dtype, oai=False, alpha=1.702, limit=7.0):
    """silu(gate) * up, or gpt-oss's clamped form; arrays of one shape stored as `dtype`."""
    gate, up = _c(gate), _c(up)
    out = np.zeros(gate.shape, store_dtype(dtype))
    _check(lib().orc_swiglu(dtype, int(oai), _ptr(gate), _ptr(up), ctypes.c_float(alpha), ctypes.c_float(limit), _sz(gate.size), _ptr(out)))
    return out


def rms_norm(x, dtype, weight=None, eps=1e-5, residual=None):
    """rms_norm over the last axis; with `residual` returns (x + residual, its rms_norm)."""
    x = _c(x)
    d = x.shape[-1]
    rows = x.size // d if d else 0
    y = np.zeros(x.shape, store_dtype(dtype))
    h = np.zeros(x.shape, store_dtype(dtype)) if residual is not None else None
    res = None if residual is None else _c(residual)
    w = None if weight is None else _c(weight)
    _check(lib().orc_rms_norm(dtype, _ptr(x), _ptr(res), _ptr(w), ctypes.c_float(eps), _sz(rows), _sz(d), _ptr(h), _ptr(y)))
    return y if residual is None else (h, y)


def threads() -> int:
    return int(lib().orc_threads())


def set_threads(n: int) -> None:
    """Threads for the parallel parts from now on (overrides an inherited OMP_NUM_THREADS)."""
    lib().orc_set_threads(int(n))
