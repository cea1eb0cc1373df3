"""Host-side mirror of nuvec's quantized operations over the CUDA backend.

Same names, argument meaning and error behaviour as the reference's op layer
(crates/nuvec-core/src/ops.rs:967-1078 and quantized.rs): ``quantize``, ``dequantize``,
``quantized_matmul``, ``gather_qmm``, the types ``QuantMode``, ``Quant``, ``Quantized`` and
``GatherQmm``.  Every computation runs in libnuvec_cuda.so; this module only checks shapes,
promotes dtypes, broadcasts batches and marshals pointers, as the reference's Rust layer does
before it reaches a backend.
"""
from __future__ import annotations

import ctypes as C
import enum
from dataclasses import dataclass, replace
from typing import Optional, Sequence

import numpy as np

from . import _ffi
from ._ffi import BF16, F16, F32, I32, U8, U32

__all__ = ["Device", "Array", "QuantMode", "Quant", "Quantized", "GatherQmm", "quantize", "dequantize",
           "quantized_matmul", "gather_qmm", "sorted_offsets", "moe_route", "weighted_sum", "expert_bias_add", "moe_sort", "take_rows", "swiglu", "swiglu_oai", "quantized_embedding", "rms_norm", "add_rms_norm", "quantized_attention", "fake_quant", "gather_qqmm", "qqmm", "qqmm_prepare_scales", "NuvecError", "InvalidArgument",
           "UnsupportedError", "OutOfMemory", "NoDevice", "BackendError", "CommError",
           "f32_to_bf16", "bf16_to_f32"]


# ── errors (crates/nuvec-core/src/error.rs:17-42) ──────────────────────────────────────────
class NuvecError(Exception):
    pass


class InvalidArgument(NuvecError, ValueError):
    pass


class UnsupportedError(NuvecError):
    pass


class OutOfMemory(NuvecError, MemoryError):
    pass


class NoDevice(NuvecError):
    pass


class BackendError(NuvecError):
    pass


class CommError(NuvecError):
    pass


_ERRORS = {_ffi.ERR_INVALID_ARGUMENT: InvalidArgument, _ffi.ERR_UNSUPPORTED: UnsupportedError,
           _ffi.ERR_OUT_OF_MEMORY: OutOfMemory, _ffi.ERR_NO_DEVICE: NoDevice,
           _ffi.ERR_DRIVER: BackendError, _ffi.ERR_COMM: CommError}


def _check(status: int):
    if status != _ffi.OK:
        raise _ERRORS.get(status, BackendError)(_ffi.last_error())


# ── dtypes ─────────────────────────────────────────────────────────────────────────────────
_ITEMSIZE = {U8: 1, U32: 4, I32: 4, F16: 2, BF16: 2, F32: 4}
_NP = {U8: np.uint8, U32: np.uint32, I32: np.int32, F16: np.float16, BF16: np.uint16, F32: np.float32}
_FLOATS = (F16, BF16, F32)
DTYPE_NAMES = {U8: "uint8", U32: "uint32", I32: "int32", F16: "float16", BF16: "bfloat16", F32: "float32"}


def f32_to_bf16(a) -> np.ndarray:
    """float32 -> bfloat16 bit patterns (uint16), round to nearest even."""
    a = np.ascontiguousarray(a, dtype=np.float32)
    u = a.view(np.uint32)
    nan = (u & 0x7FFFFFFF) > 0x7F800000
    r = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)
    return np.where(nan, ((u >> 16) | 0x40).astype(np.uint16), r)


def bf16_to_f32(a) -> np.ndarray:
    return (np.asarray(a, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def promote_types(a: int, b: int) -> int:
    """The common float dtype of two float dtypes (MLX's promotion: unequal halves -> f32)."""
    if a == b:
        return a
    return F32


# ── device and arrays ──────────────────────────────────────────────────────────────────────
class Device:
    """One GPU with its stream and pool (crates/nuvec-gpu/src/cuda/device.rs:77-227)."""

    _shared = {}

    def __init__(self, ordinal: int = 0):
        h = C.c_void_p()
        _check(_ffi.lib().nvc_device_open(ordinal, C.byref(h)))
        self._h, self.ordinal = h, ordinal

    @classmethod
    def shared(cls, ordinal: int = 0) -> "Device":
        if ordinal not in cls._shared:
            cls._shared[ordinal] = cls(ordinal)
        return cls._shared[ordinal]

    def close(self):
        if self._h:
            _check(_ffi.lib().nvc_device_close(self._h))
            self._h = None
            Device._shared.pop(self.ordinal, None)

    def info(self) -> dict:
        i = _ffi.Info()
        _check(_ffi.lib().nvc_device_info(self._h, C.byref(i)))
        return {"name": i.name.decode(), "compute_capability": (i.cc_major, i.cc_minor),
                "multiprocessors": i.multiprocessors, "driver_version": i.driver_version,
                "total_memory": i.total_memory, "l2_bytes": i.l2_bytes}

    def synchronize(self):
        _check(_ffi.lib().nvc_synchronize(self._h))

    def set_stream(self, cuda_stream: Optional[int]):
        _check(_ffi.lib().nvc_device_set_stream(self._h, C.c_void_p(cuda_stream or 0)))

    @property
    def launches(self) -> int:
        return int(_ffi.lib().nvc_launch_count(self._h))

    def memory(self) -> dict:
        s = _ffi.MemStats()
        _check(_ffi.lib().nvc_mem_stats_get(self._h, C.byref(s)))
        return {k: int(getattr(s, k)) for k, _ in _ffi.MemStats._fields_}

    def set_memory_limit(self, n: int):
        _check(_ffi.lib().nvc_set_memory_limit(self._h, n))

    def set_cache_limit(self, n: int):
        _check(_ffi.lib().nvc_set_cache_limit(self._h, n))

    def clear_cache(self):
        _check(_ffi.lib().nvc_clear_cache(self._h))

    def reset_peak(self):
        _check(_ffi.lib().nvc_reset_peak(self._h))

    def row_exact(self):
        """``with dev.row_exact():`` crate::with_row_exact (crates/nuvec-core/src/lib.rs:175-186): products of up to 8
        rows built inside give each row the bits of its one-row product."""
        dev = self

        class _RowExact:
            def __enter__(self):
                self.before = _ffi.lib().nvc_row_exact(dev._h)
                _check(_ffi.lib().nvc_set_row_exact(dev._h, 1))

            def __exit__(self, *exc):
                _check(_ffi.lib().nvc_set_row_exact(dev._h, self.before))
                return False
        return _RowExact()

    # arrays
    def empty(self, shape: Sequence[int], dtype: int) -> "Array":
        return Array(self, tuple(int(d) for d in shape), dtype)

    def array(self, data, dtype: Optional[int] = None) -> "Array":
        """Uploads a numpy array.  bfloat16 travels as uint16 bit patterns with dtype=BF16."""
        data = np.asarray(data)
        if dtype is None:
            dtype = {np.dtype(np.float32): F32, np.dtype(np.float16): F16, np.dtype(np.uint32): U32,
                     np.dtype(np.uint8): U8, np.dtype(np.int32): I32}.get(data.dtype)
            if dtype is None:
                raise InvalidArgument(f"cannot infer a device dtype for numpy {data.dtype}; pass dtype=")
        host = np.ascontiguousarray(data, dtype=_NP[dtype] if dtype != F16 else np.float16)
        out = self.empty(host.shape, dtype)
        if host.nbytes:
            _check(_ffi.lib().nvc_memcpy_h2d(self._h, out.ptr, host.ctypes.data_as(C.c_void_p), host.nbytes))
            self.synchronize()  # the numpy buffer may be pageable and go away
        return out

    def event(self) -> "Event":
        return Event(self)

    def record(self, fn) -> "Graph":
        """Records the stream work `fn()` enqueues (run it once beforehand so scratch exists)
        and returns a replayable graph -- the analogue of one committed command buffer."""
        _check(_ffi.lib().nvc_graph_begin(self._h))
        try:
            fn()
        finally:
            h = C.c_void_p()
            status = _ffi.lib().nvc_graph_end(self._h, C.byref(h))
        _check(status)
        return Graph(self, h)


class Graph:
    def __init__(self, dev: Device, h):
        self._dev, self._h = dev, h

    def launch(self):
        _check(_ffi.lib().nvc_graph_launch(self._dev._h, self._h))

    def __del__(self):
        try:
            if self._h:
                _ffi.lib().nvc_graph_destroy(self._h)
                self._h = None
        except Exception:
            pass


class Event:
    def __init__(self, dev: Device):
        h = C.c_void_p()
        _check(_ffi.lib().nvc_event_create(dev._h, C.byref(h)))
        self._h, self._dev = h, dev

    def record(self):
        _check(_ffi.lib().nvc_event_record(self._dev._h, self._h))
        return self

    def synchronize(self):
        _check(_ffi.lib().nvc_event_synchronize(self._h))

    def elapsed_ms(self, later: "Event") -> float:
        out = C.c_float()
        _check(_ffi.lib().nvc_event_elapsed_ms(self._h, later._h, C.byref(out)))
        return float(out.value)

    def __del__(self):
        try:
            if self._h:
                _ffi.lib().nvc_event_destroy(self._h)
                self._h = None
        except Exception:
            pass


class Array:
    """A dense row-major device buffer with a shape and a dtype code.

    `view` arrays share another array's storage at a byte offset (sliced weights, rows of x).
    """

    def __init__(self, dev: Device, shape, dtype: int, _base: "Array" = None, _offset: int = 0):
        self.dev, self.shape, self.dtype = dev, tuple(shape), dtype
        self._base, self._offset = _base, _offset
        if _base is None:
            p = C.c_void_p()
            _check(_ffi.lib().nvc_alloc(dev._h, max(self.nbytes, 1), C.byref(p)))
            self._ptr = p.value
        else:
            self._ptr = None

    @property
    def ptr(self) -> C.c_void_p:
        base = self._ptr if self._base is None else self._base.ptr.value
        return C.c_void_p(base + self._offset)

    @property
    def size(self) -> int:
        n = 1
        for d in self.shape:
            n *= d
        return n

    @property
    def ndim(self) -> int:
        return len(self.shape)

    @property
    def itemsize(self) -> int:
        return _ITEMSIZE[self.dtype]

    @property
    def nbytes(self) -> int:
        return self.size * self.itemsize

    def reshape(self, *shape) -> "Array":
        shape = tuple(shape[0]) if len(shape) == 1 and isinstance(shape[0], (tuple, list)) else tuple(shape)
        if -1 in shape:
            known = -int(np.prod(shape))
            shape = tuple(self.size // known if d == -1 else d for d in shape)
        assert int(np.prod(shape)) == self.size, (shape, self.shape)
        root = self if self._base is None else self._base
        return Array(self.dev, shape, self.dtype, _base=root, _offset=self._offset)

    def __getitem__(self, index) -> "Array":
        """Leading-axis integer or slice (a contiguous view)."""
        inner = int(np.prod(self.shape[1:])) if self.ndim > 1 else 1
        root = self if self._base is None else self._base
        if isinstance(index, slice):
            start, stop, step = index.indices(self.shape[0])
            assert step == 1
            return Array(self.dev, (max(stop - start, 0),) + self.shape[1:], self.dtype, _base=root,
                         _offset=self._offset + start * inner * self.itemsize)
        i = int(index) % self.shape[0]
        return Array(self.dev, self.shape[1:], self.dtype, _base=root,
                     _offset=self._offset + i * inner * self.itemsize)

    def to_numpy(self) -> np.ndarray:
        host = np.empty(self.shape, dtype=_NP[self.dtype])
        if host.nbytes:
            _check(_ffi.lib().nvc_memcpy_d2h(self.dev._h, host.ctypes.data_as(C.c_void_p), self.ptr, host.nbytes))
        return host

    def to_f32(self) -> np.ndarray:
        host = self.to_numpy()
        return bf16_to_f32(host) if self.dtype == BF16 else host.astype(np.float32)

    def astype(self, dtype: int) -> "Array":
        """dtype conversion of float arrays (round to nearest even), done through the host: it
        only runs where the reference promotes mismatched operand dtypes."""
        if dtype == self.dtype:
            return self
        f = self.to_f32()
        if dtype == BF16:
            return self.dev.array(f32_to_bf16(f), BF16)
        return self.dev.array(f.astype(_NP[dtype]), dtype)

    def copy_from(self, other: "Array"):
        assert other.nbytes == self.nbytes
        _check(_ffi.lib().nvc_memcpy_d2d(self.dev._h, self.ptr, other.ptr, self.nbytes))

    def __del__(self):
        try:
            if self._base is None and self._ptr and self.dev._h:
                _ffi.lib().nvc_free(self.dev._h, C.c_void_p(self._ptr))
                self._ptr = None
        except Exception:
            pass


# ── quantization descriptors (crates/nuvec-core/src/quantized.rs:24-168, 195-359) ──────────
class QuantMode(enum.Enum):
    AFFINE = "affine"
    MXFP4 = "mxfp4"
    MXFP8 = "mxfp8"
    NVFP4 = "nvfp4"

    @classmethod
    def parse(cls, s: str) -> "QuantMode":
        try:
            return cls(s)
        except ValueError:
            raise InvalidArgument(f"invalid quantization mode '{s}' (affine, mxfp4, mxfp8 or nvfp4)") from None

    @property
    def code(self) -> int:
        return {"affine": 0, "mxfp4": 1, "mxfp8": 2, "nvfp4": 3}[self.value]

    def defaults(self):
        return {"affine": (64, 4), "mxfp4": (32, 4), "mxfp8": (32, 8), "nvfp4": (16, 4)}[self.value]


@dataclass(frozen=True)
class Quant:
    mode: QuantMode = QuantMode.AFFINE
    group_size: int = 64
    bits: int = 4

    @classmethod
    def new(cls, mode: QuantMode) -> "Quant":
        g, b = mode.defaults()
        return cls(mode, g, b)

    @classmethod
    def affine(cls, group_size: int, bits: int) -> "Quant":
        return cls(QuantMode.AFFINE, group_size, bits)

    def with_group_size(self, g: int) -> "Quant":
        return replace(self, group_size=g)

    def with_bits(self, b: int) -> "Quant":
        return replace(self, bits=b)

    def checked(self, op: str):
        """quantized.rs:137-167"""
        g, b = self.group_size, self.bits
        if self.mode == QuantMode.AFFINE:
            if g not in (32, 64, 128):
                raise InvalidArgument(f"{op}: group size {g} is not supported (32, 64 or 128)")
            if b not in (1, 2, 3, 4, 5, 6, 8):
                raise InvalidArgument(f"{op}: {b} bits are not supported (1, 2, 3, 4, 5, 6 or 8)")
        else:
            eg, eb = self.mode.defaults()
            if g != eg:
                raise InvalidArgument(f"{op}: {self.mode.value} quantization requires group size {eg} but got {g}")
            if b != eb:
                raise InvalidArgument(f"{op}: {self.mode.value} quantization requires bits to be {eb} but got {b}")
        return g, b

    def _c(self) -> _ffi.Quant:
        return _ffi.Quant(self.mode.code, self.group_size, self.bits)


@dataclass
class Quantized:
    """Packed codes (uint32), one scale per group, affine biases, an optional NVFP4 global
    scale and how they were quantized (quantized.rs:195-278)."""
    weight: Array
    scales: Array
    biases: Optional[Array] = None
    quant: Quant = Quant()
    global_scale: Optional[Array] = None

    def with_global_scale(self, g: Array) -> "Quantized":
        return replace(self, global_scale=g)

    def dequantize(self, dtype: Optional[int] = None) -> Array:
        return dequantize(self, dtype)


@dataclass(frozen=True)
class GatherQmm:
    """Options of gather_qmm (quantized.rs:318-359)."""
    transpose: bool = True
    sorted_indices: bool = False

    @staticmethod
    def groups(rows: int, experts: int) -> bool:
        """quantized.rs:724-731: the grouped kernel needs 16 rows and 4 per expert."""
        return rows >= 16 and rows // max(experts, 1) >= 4

    def with_transpose(self, t: bool) -> "GatherQmm":
        return replace(self, transpose=t)

    def with_sorted_indices(self, s: bool) -> "GatherQmm":
        return replace(self, sorted_indices=s)


def _check_groups(op: str, mode: QuantMode, scales: Array, biases: Optional[Array]):
    """quantized.rs:363-379"""
    if mode == QuantMode.AFFINE:
        if biases is None:
            raise InvalidArgument(f"{op}: biases must be provided for affine quantization")
        return
    if biases is not None:
        raise InvalidArgument(f"{op}: biases must be null for quantization mode '{mode.value}'")
    if scales.dtype != U8:
        raise InvalidArgument(f"{op}: scale type must be uint8 but received type {DTYPE_NAMES[scales.dtype]}")


def _check_global(op: str, quant: Quant, g: Optional[Array], experts_shape=None):
    if g is None:
        return
    if quant.mode != QuantMode.NVFP4:
        raise InvalidArgument(f"{op}: a global scale is only supported for nvfp4, got {quant.mode.value}")
    if experts_shape is None:
        if g.size != 1 or g.dtype != F32:
            raise InvalidArgument(f"{op}: the global scale must be one float32 value, got "
                                  f"{DTYPE_NAMES[g.dtype]} {list(g.shape)}")
    else:
        if g.dtype != F32:
            raise InvalidArgument(f"{op}: global scale must have dtype float32 but got {DTYPE_NAMES[g.dtype]}")
        if tuple(g.shape) != tuple(experts_shape):
            raise InvalidArgument(f"{op}: global scale must have one entry per expert with shape "
                                  f"{list(experts_shape)} but got {list(g.shape)}")


def _ptr(a: Optional[Array]):
    return None if a is None else a.ptr


def _columns(op: str, w: Array, scales: Array, biases: Optional[Array], quant: Quant) -> int:
    """Values per row of packed codes after the reference's checks (primitive.rs:1405-1460)."""
    g, b = quant.checked(op)
    if w.dtype != U32 or w.ndim < 2:
        raise InvalidArgument(f"{op}: the packed weights must be uint32 with at least 2 dimensions, got "
                              f"{DTYPE_NAMES[w.dtype]} {list(w.shape)}")
    cols = w.shape[-1] * 32 // b
    want = w.shape[:-1] + (cols // g,)
    if cols % g != 0 or tuple(scales.shape) != want or (biases is not None and tuple(biases.shape) != want):
        raise InvalidArgument(f"{op}: scales{'/biases' if biases is not None else ''} of shape {list(scales.shape)} "
                              f"do not match weights {list(w.shape)} with group size {g} and {b} bits")
    return cols


# ── operations ─────────────────────────────────────────────────────────────────────────────
def quantize(w: Array, quant=Quant(), global_scale: Optional[Array] = None) -> Quantized:
    """ops::quantize (ops.rs:967-1009): quantizes the last axis of `w`."""
    if isinstance(quant, QuantMode):
        quant = Quant.new(quant)
    g, b = quant.checked("quantize")
    _check_global("quantize", quant, global_scale)
    if w.dtype not in _FLOATS:
        raise UnsupportedError(f"quantize: unsupported dtype {DTYPE_NAMES[w.dtype]}")
    if w.ndim < 2 or w.shape[-1] % g != 0:
        raise InvalidArgument(f"quantize: needs at least 2 dimensions with the last divisible by the group size "
                              f"{g}, got shape {list(w.shape)}")
    cols = w.shape[-1]
    rows = w.size // cols if cols else 0
    dev = w.dev
    codes = dev.empty(w.shape[:-1] + (cols * b // 32,), U32)
    gshape = w.shape[:-1] + (cols // g,)
    affine = quant.mode == QuantMode.AFFINE
    scales = dev.empty(gshape, w.dtype if affine else U8)
    biases = dev.empty(gshape, w.dtype) if affine else None
    q = quant._c()
    _check(_ffi.lib().nvc_quantize(dev._h, C.byref(q), w.dtype, w.ptr, rows, cols, _ptr(global_scale), codes.ptr,
                                   scales.ptr, _ptr(biases)))
    return Quantized(codes, scales, biases, quant, global_scale)


def dequantize(q: Quantized, dtype: Optional[int] = None, fused: bool = False) -> Array:
    """ops::dequantize (ops.rs:1014-1027; quantized.rs:401-444).  `fused` selects the single
    rounding of the reference's Metal kernel instead of its CPU result."""
    quant = q.quant
    quant.checked("dequantize")
    _check_groups("dequantize", quant.mode, q.scales, q.biases)
    if dtype is not None and dtype not in _FLOATS:
        raise InvalidArgument(f"dequantize: only real floating types are supported but the output dtype is "
                              f"{DTYPE_NAMES.get(dtype, dtype)}")
    _check_global("dequantize", quant, q.global_scale)
    cols = _columns("dequantize", q.weight, q.scales, q.biases, quant)
    rows = q.weight.size // q.weight.shape[-1] if q.weight.shape[-1] else 0
    dev = q.weight.dev
    affine = quant.mode == QuantMode.AFFINE
    if affine and q.scales.dtype != q.biases.dtype:
        raise InvalidArgument("dequantize: scales and biases must share a dtype")
    kernel_dtype = q.scales.dtype if affine else (dtype if dtype is not None else BF16)
    out = dev.empty(q.weight.shape[:-1] + (cols,), kernel_dtype)
    c = quant._c()
    _check(_ffi.lib().nvc_dequantize(dev._h, C.byref(c), kernel_dtype, q.weight.ptr, q.scales.ptr, _ptr(q.biases),
                                     _ptr(q.global_scale), rows, cols, out.ptr, int(fused)))
    if affine and dtype is not None and dtype != kernel_dtype:
        return out.astype(dtype)
    return out


def sorted_offsets(indices: Array, groups: int) -> Array:
    """Primitive::SortedOffsets (quantized.rs:772-782)."""
    if indices.dtype != U32:
        raise InvalidArgument("sorted_offsets: indices must be uint32")
    out = indices.dev.empty((groups,), I32)
    _check(_ffi.lib().nvc_sorted_offsets(indices.dev._h, indices.ptr, indices.size, groups, out.ptr))
    return out


def moe_route(probs: Array, k: int, normalize: bool = True):
    """fast::moe_route (fast/imp.rs:2652-2672): (indices uint32 [..., k], scores [..., k]) of the k
    largest probabilities along the last axis, in the stable ascending order of a sort."""
    if probs.dtype not in _FLOATS:
        raise InvalidArgument(f"moe_route: probabilities must be floating point, got {DTYPE_NAMES.get(probs.dtype, probs.dtype)}")
    e = probs.shape[-1] if probs.ndim else 0
    if not 1 <= k <= e:
        raise InvalidArgument(f"moe_route: k must be in 1..={e} for probabilities of shape {list(probs.shape)}")
    rows = probs.size // e
    lead = tuple(probs.shape[:-1])
    idx = probs.dev.empty(lead + (k,), U32)
    scores = probs.dev.empty(lead + (k,), probs.dtype)
    _check(_ffi.lib().nvc_moe_route(probs.dev._h, probs.dtype, probs.ptr, rows, e, k, int(normalize), idx.ptr, scores.ptr))
    return idx, scores


def weighted_sum(x: Array, w: Array) -> Array:
    """fast::weighted_sum (fast/imp.rs:2731-2747): x [..., k, D] times w [..., k], summed over k."""
    if x.ndim < 2 or tuple(w.shape) != tuple(x.shape[:-1]):
        raise InvalidArgument(f"weighted_sum: x must be [..., k, D] and w [..., k], got {list(x.shape)} and {list(w.shape)}")
    if x.dtype not in _FLOATS or w.dtype != x.dtype:
        raise UnsupportedError("weighted_sum: x and w must share one floating-point dtype")
    k, d = x.shape[-2], x.shape[-1]
    rows = x.size // (k * d) if k * d else 0
    out = x.dev.empty(tuple(x.shape[:-2]) + (d,), x.dtype)
    _check(_ffi.lib().nvc_weighted_sum(x.dev._h, x.dtype, x.ptr, w.ptr, rows, k, d, out.ptr))
    return out


def expert_bias_add(y: Array, bias: Array, indices: Array) -> Array:
    """The bias of SwitchProjection::forward (crates/nuvec-lm/src/model.rs:2139-2143): y [rows, ..., n] plus
    bias[indices] ([experts, n], uint32 indices [rows]), in place; returns y."""
    if bias.ndim != 2 or y.ndim < 2 or y.shape[-1] != bias.shape[1]:
        raise InvalidArgument(f"expert_bias_add: y [..., n] and bias [experts, n] expected, got {list(y.shape)} and {list(bias.shape)}")
    if y.dtype not in _FLOATS or bias.dtype != y.dtype:
        raise UnsupportedError("expert_bias_add: y and bias must share one floating-point dtype")
    n = y.shape[-1]
    rows = y.size // n if n else 0
    if indices.dtype != U32 or indices.size != rows:
        raise InvalidArgument(f"expert_bias_add: {rows} uint32 indices expected, got {indices.size}")
    _check(_ffi.lib().nvc_expert_bias_add(y.dev._h, y.dtype, y.ptr, bias.ptr, indices.ptr, rows, n, bias.shape[0]))
    return y


def moe_sort(indices: Array, experts: int):
    """The bookkeeping of SwitchGlu::forward (crates/nuvec-lm/src/model.rs:2199-2210) for expert indices
    [..., k] (uint32): (order, restore, tokens, sorted, offsets) -- the stable argsort of the flattened
    indices, its inverse, each sorted pair's token and expert (uint32 [pairs]) and the experts' first
    rows (int32 [experts])."""
    if indices.dtype != U32 or indices.ndim < 1:
        raise InvalidArgument("moe_sort: uint32 indices [..., k] expected")
    k = indices.shape[-1]
    pairs = indices.size
    if k < 1:
        raise InvalidArgument("moe_sort: k must be at least 1")
    dev = indices.dev
    order, restore, tokens, srt = (dev.empty((pairs,), U32) for _ in range(4))
    offsets = dev.empty((experts,), I32)
    _check(_ffi.lib().nvc_moe_sort(dev._h, indices.ptr, pairs, k, experts, order.ptr, restore.ptr, tokens.ptr, srt.ptr, offsets.ptr))
    return order, restore, tokens, srt, offsets


def take_rows(src: Array, indices: Array) -> Array:
    """take(src, indices, 0) of whole rows: out[i] = src[indices[i]] (indices past the end take the last row)."""
    if src.ndim < 1 or indices.dtype != U32:
        raise InvalidArgument("take_rows: an array of rows and uint32 indices expected")
    rows = src.shape[0]
    row_bytes = (src.size // rows if rows else 0) * src.itemsize
    out = src.dev.empty((indices.size,) + tuple(src.shape[1:]), src.dtype)
    _check(_ffi.lib().nvc_take_rows(src.dev._h, src.ptr, rows, row_bytes, indices.ptr, indices.size, out.ptr))
    return out


def quantized_embedding(q: Quantized, ids: Array) -> Array:
    """QuantizedEmbedding::forward (crates/nuvec-nn/src/layers.rs:246-255): the ids' rows of a quantized table
    [vocab, cols], dequantized: shape ids.shape + (cols,), the scales' dtype (bfloat16 for the fp modes)."""
    quant = q.quant
    quant.checked("quantized_embedding")
    if q.weight.ndim != 2 or ids.dtype != U32:
        raise InvalidArgument("quantized_embedding: a 2-D quantized table and uint32 ids expected")
    if q.global_scale is not None:
        raise UnsupportedError("quantized_embedding: tables with a global scale are not supported")
    _check_groups("quantized_embedding", quant.mode, q.scales, q.biases)
    cols = _columns("quantized_embedding", q.weight, q.scales, q.biases, quant)
    affine = quant.mode == QuantMode.AFFINE
    dtype = q.scales.dtype if affine else BF16
    dev = q.weight.dev
    out = dev.empty(tuple(ids.shape) + (cols,), dtype)
    c = quant._c()
    _check(_ffi.lib().nvc_quantized_embedding(dev._h, C.byref(c), dtype, q.weight.ptr, q.scales.ptr, _ptr(q.biases),
                                              q.weight.shape[0], cols, ids.ptr, ids.size, out.ptr))
    return out


def qqmm_prepare_scales(q: Quantized) -> Array:
    """The weight's scales laid out once the way the tensor core reads them (for qqmm(..., prepared=...))."""
    c = q.quant._c()
    N, K = q.weight.shape[0], q.weight.shape[1] * 8
    nbytes = _ffi.lib().nvc_qqmm_scales_bytes(C.byref(c), N, K)
    if nbytes == 0:
        raise UnsupportedError("qqmm_prepare_scales: nvfp4 or mxfp4 weights expected")
    out = q.weight.dev.empty((nbytes,), U8)
    _check(_ffi.lib().nvc_qqmm_prepare_scales(q.weight.dev._h, C.byref(c), q.scales.ptr, N, K, out.ptr))
    return out


def fake_quant(x: Array, quant: Quant, global_scale: Optional[Array] = None) -> Array:
    """x through its quantization in a floating-point mode: the values its codes represent, in x's dtype
    (products.rs:306-315, MLX's fp_quantize_dequantize)."""
    quant.checked("qqmm")
    if quant.mode == QuantMode.AFFINE:
        raise InvalidArgument("qqmm: needs a floating-point mode (mxfp4, mxfp8 or nvfp4)")
    if x.dtype not in (F16, BF16, F32) or x.ndim < 1 or x.shape[-1] % quant.group_size != 0:
        raise InvalidArgument(f"qqmm: a float activation [..., K] with K a multiple of {quant.group_size} expected, got {list(x.shape)}")
    if global_scale is not None:
        _check_global("qqmm", quant, global_scale)
    K = x.shape[-1]
    out = x.dev.empty(x.shape, x.dtype)
    c = quant._c()
    _check(_ffi.lib().nvc_quantize_dequantize(x.dev._h, C.byref(c), x.dtype, x.ptr, x.size // K if K else 0, K, _ptr(global_scale), out.ptr))
    return out


def _qq_scales(name: str, q: Quantized, global_scale_x: Optional[Array]):
    """MLX's rule (products.rs:317-335): nvfp4 global scales for both operands or neither."""
    if (global_scale_x is None) != (q.global_scale is None):
        raise InvalidArgument(f"{name}: for nvfp4, give global scales for both the activations and the weight, or neither")


def gather_qqmm(x: Array, q: Quantized, lhs_indices: Optional[Array] = None, rhs_indices: Optional[Array] = None,
                sorted_indices: bool = False, global_scale_x: Optional[Array] = None) -> Array:
    """MLX's gather_qqmm (products.rs:437-463): gather_qmm of the quantized activations with quantized experts
    (w [E, N, K]), transposed.  The activations go through fake_quant, the product is the exact gather_qmm."""
    name = "gather_qqmm"
    _qq_scales(name, q, global_scale_x)
    if q.quant.mode == QuantMode.AFFINE:
        raise InvalidArgument(f"{name}: needs a floating-point mode (mxfp4, mxfp8 or nvfp4)")
    if q.global_scale is not None and q.global_scale.size == 1 and q.weight.ndim > 2:
        # MLX broadcasts the weight's one global scale to every expert
        experts = tuple(q.weight.shape[:-2])
        host = np.broadcast_to(q.global_scale.to_numpy().reshape(()), experts)
        q = q.with_global_scale(x.dev.array(np.ascontiguousarray(host), F32))
    xq = fake_quant(x, q.quant, global_scale_x)
    return gather_qmm(xq, q, lhs_indices, rhs_indices, GatherQmm(True, sorted_indices))


def qqmm(x: Array, q: Quantized, prepared: Optional[Array] = None, global_scale_x: Optional[Array] = None) -> Array:
    """MLX's qqmm (crates/nuvec-core/src/products.rs:337-352): x through its own quantization in q's mode, times
    the quantized weight transposed.  NVFP4 (without a global scale) or MXFP4 weights, bfloat16 x [..., K]."""
    quant = q.quant
    quant.checked("qqmm")
    if quant.mode == QuantMode.AFFINE:
        raise InvalidArgument("qqmm: needs a floating-point mode (mxfp4, mxfp8 or nvfp4)")
    _qq_scales("qqmm", q, global_scale_x)
    if quant.mode not in (QuantMode.NVFP4, QuantMode.MXFP4) or q.global_scale is not None or x.dtype != BF16:
        # the reference's definition, step by step (products.rs:337-352): x through its quantization, then the exact
        # quantized product (mxfp8, nvfp4 global scales, other activation types)
        return quantized_matmul(fake_quant(x, quant, global_scale_x), q, True)
    if x.dtype != BF16 or x.ndim < 1 or q.weight.ndim != 2:
        raise UnsupportedError("qqmm: bfloat16 activations [..., K] and a 2-D quantized weight expected")
    K = x.shape[-1]
    N = q.weight.shape[0]
    if q.weight.shape[1] * 8 != K:
        raise InvalidArgument(f"qqmm: shapes {list(x.shape)} and {list(q.weight.shape)} do not match")
    M = x.size // K if K else 0
    out = x.dev.empty(tuple(x.shape[:-1]) + (N,), BF16)
    c = quant._c()
    if prepared is not None:
        _check(_ffi.lib().nvc_qqmm_prepared(x.dev._h, C.byref(c), BF16, x.ptr, q.weight.ptr, prepared.ptr, M, N, K, out.ptr))
    else:
        _check(_ffi.lib().nvc_qqmm(x.dev._h, C.byref(c), BF16, x.ptr, q.weight.ptr, q.scales.ptr, M, N, K, out.ptr))
    return out


def quantized_attention(q: Array, k: Quantized, v: Quantized, scale: float, sinks: Optional[Array] = None,
                        length: Optional[int] = None, causal: bool = False) -> Array:
    """fast::quantized_attention (crates/nuvec-core/src/fast.rs:694-722): q [B, Hq, L, D] over affine-quantized keys
    and values (codes [B, Hkv, S, D * bits / 32], scales and biases [B, Hkv, S, D / group_size]), no mask (every query
    row attends to all the keys), optional per-head sinks [Hq].  ``length`` attends to the first ``length`` keys of a
    longer cache (the reference's cache views, ``k.weight.i((.., .., ..length))``).  The head sizes, bit widths, group
    sizes and head ratios of the reference's kernel (fast/imp.rs:3944-3993); up to 64 query rows, one pass over the
    cache each.  ``causal``: query row l stands at position S - L + l and attends to the keys up to it."""
    if k.quant != v.quant or k.quant.mode != QuantMode.AFFINE:
        raise InvalidArgument("quantized_attention: keys and values need one affine quantization")
    if k.biases is None or v.biases is None:
        raise InvalidArgument("quantized_attention: affine biases missing")
    if q.ndim != 4 or k.weight.ndim != 4 or v.weight.ndim != 4:
        raise InvalidArgument("quantized_attention: queries, keys and values must be 4-D")
    quant = k.quant
    gs, bits = quant.checked("quantized_attention")
    B, Hq, L, D = q.shape
    Bk, Hkv, cap, words = k.weight.shape
    S = cap if length is None else int(length)
    groups = D // gs if gs else 0
    side_ok = all(t.weight.shape == (B, Hkv, cap, words) and t.weight.dtype == U32 and words * 32 == D * bits
                  and t.scales.shape == (B, Hkv, cap, groups) and t.biases.shape == t.scales.shape
                  and t.scales.dtype == q.dtype and t.biases.dtype == q.dtype for t in (k, v))
    if not side_ok or not 0 <= S <= cap:
        raise InvalidArgument(f"quantized_attention: cache of shape {list(k.weight.shape)} / {list(v.weight.shape)} does not "
                              f"match queries {list(q.shape)}")
    if sinks is not None and (sinks.shape != (Hq,) or sinks.dtype != q.dtype):
        raise InvalidArgument(f"quantized_attention: sinks must be [{Hq}] of the queries' dtype")
    out = q.dev.empty((B, Hq, L, D), q.dtype)
    c = quant._c()
    _check(_ffi.lib().nvc_quantized_attention(q.dev._h, C.byref(c), q.dtype, q.ptr, k.weight.ptr, k.scales.ptr, k.biases.ptr,
                                              v.weight.ptr, v.scales.ptr, v.biases.ptr, _ptr(sinks), B, Hq, Hkv, L, S, D, cap,
                                              float(scale), int(bool(causal)), out.ptr))
    return out


def _norm_args(name, x: Array, weight):
    if x.ndim < 1 or x.dtype not in _FLOATS:
        raise InvalidArgument(f"{name}: a floating-point input with at least one dimension expected")
    d = x.shape[-1]
    if weight is not None and (weight.dtype != x.dtype or tuple(weight.shape) != (d,)):
        raise InvalidArgument(f"{name}: the weight must be [{d}] of the input's dtype")
    return d, (x.size // d if d else 0)


def rms_norm(x: Array, weight: Optional[Array] = None, eps: float = 1e-5) -> Array:
    """fast::rms_norm (crates/nuvec-core/src/fast/imp.rs:358-378) over the last axis."""
    d, rows = _norm_args("rms_norm", x, weight)
    y = x.dev.empty(tuple(x.shape), x.dtype)
    _check(_ffi.lib().nvc_rms_norm(x.dev._h, x.dtype, x.ptr, _ptr(weight), eps, rows, d, y.ptr))
    return y


def add_rms_norm(x: Array, residual: Array, weight: Optional[Array] = None, eps: float = 1e-5):
    """fast::add_rms_norm (fast/imp.rs:381-412): (x + residual, rms_norm of that)."""
    d, rows = _norm_args("add_rms_norm", x, weight)
    if tuple(residual.shape) != tuple(x.shape) or residual.dtype != x.dtype:
        raise InvalidArgument("add_rms_norm: x and the residual must share shape and dtype")
    h, y = x.dev.empty(tuple(x.shape), x.dtype), x.dev.empty(tuple(x.shape), x.dtype)
    _check(_ffi.lib().nvc_add_rms_norm(x.dev._h, x.dtype, x.ptr, residual.ptr, _ptr(weight), eps, rows, d, h.ptr, y.ptr))
    return h, y


def _glu(name, gate: Array, up: Array, call):
    if tuple(gate.shape) != tuple(up.shape) or gate.dtype not in _FLOATS or up.dtype != gate.dtype:
        raise InvalidArgument(f"{name}: gate and up must share one shape and one floating-point dtype")
    out = gate.dev.empty(tuple(gate.shape), gate.dtype)
    _check(call(out))
    return out


def swiglu(gate: Array, up: Array) -> Array:
    """nuvec_nn::swiglu (crates/nuvec-nn/src/lib.rs:513): silu(gate) * up."""
    return _glu("swiglu", gate, up, lambda out: _ffi.lib().nvc_swiglu(gate.dev._h, gate.dtype, gate.ptr, up.ptr, gate.size, out.ptr))


def swiglu_oai(gate: Array, up: Array, alpha: float = 1.702, limit: float = 7.0) -> Array:
    """nuvec_nn::swiglu_oai (crates/nuvec-nn/src/lib.rs:564): gpt-oss's clamped SwiGLU."""
    return _glu("swiglu_oai", gate, up,
                lambda out: _ffi.lib().nvc_swiglu_oai(gate.dev._h, gate.dtype, gate.ptr, up.ptr, alpha, limit, gate.size, out.ptr))


def _promote(op: str, x: Array, q: Quantized):
    """quantized.rs:491-503: affine promotes x, scales and biases to one float dtype."""
    if q.biases is not None:
        dtype = promote_types(promote_types(x.dtype, q.scales.dtype), q.biases.dtype)
    else:
        dtype = x.dtype
    if dtype not in _FLOATS:
        raise UnsupportedError(f"{op}: unsupported dtype {DTYPE_NAMES.get(dtype, dtype)}")
    x = x.astype(dtype)
    scales, biases = q.scales, q.biases
    if biases is not None:
        scales, biases = scales.astype(dtype), biases.astype(dtype)
    return dtype, x, scales, biases


def quantized_matmul(x: Array, q: Quantized, transpose: bool = True) -> Array:
    """ops::quantized_matmul (ops.rs:1031-1046; quantized.rs:453-537): `x @ dequantize(w).T`
    (or without the transpose).  A 1-D x is a row vector; batch dimensions broadcast."""
    quant = q.quant
    g, b = quant.checked("quantized_matmul")
    _check_groups("quantized_matmul", quant.mode, q.scales, q.biases)
    w = q.weight
    gscale = q.global_scale
    if gscale is not None and (w.ndim > 2 or x.ndim > 2 or not transpose):
        # quantized.rs:481-490: dequantize in x's dtype, then an ordinary product.
        raise UnsupportedError("quantized_matmul: an nvfp4 global scale with batches or untransposed weights "
                               "takes the reference's dense matmul, which this backend does not provide")
    _check_global("quantized_matmul", quant, gscale)
    if x.dtype not in _FLOATS:
        raise UnsupportedError(f"quantized_matmul: unsupported dtype {DTYPE_NAMES.get(x.dtype, x.dtype)}")
    dtype, x, scales, biases = _promote("quantized_matmul", x, q)
    cols = _columns("quantized_matmul", w, scales, biases, quant)
    rows = w.shape[-2]
    inner, outer = (cols, rows) if transpose else (rows, cols)
    vector = x.ndim == 1
    if x.ndim == 0 or x.shape[-1] != inner:
        raise InvalidArgument(f"quantized_matmul: shapes {list(x.shape)} and {list(w.shape)} do not match")
    if vector:
        x = x.reshape(1, x.shape[0])
    M, K = x.shape[-2], x.shape[-1]
    N = outer
    bx, bw = x.shape[:-2], w.shape[:-2]
    try:
        batch = tuple(np.broadcast_shapes(bx, bw)) if bw else bx
    except ValueError:
        raise InvalidArgument(f"quantized_matmul: batch dimensions {list(bx)} and {list(bw)} do not broadcast") from None
    dev = x.dev
    out = dev.empty(batch + (M, N), dtype)
    nb = int(np.prod(batch)) if batch else 1
    c = quant._c()
    lib = _ffi.lib()

    def call(xa, wa, sa, ba, ya, count, xs, ws, ss):
        _check(lib.nvc_quantized_matmul(dev._h, C.byref(c), dtype, int(transpose), xa, wa, sa, ba, _ptr(gscale),
                                        M, N, K, K, count, xs, ws, ss, ya))

    x_mat, w_mat, s_mat = M * K, w.shape[-2] * w.shape[-1], scales.shape[-2] * scales.shape[-1]
    if not bw:
        call(x.ptr, w.ptr, scales.ptr, _ptr(biases), out.ptr, nb, x_mat, 0, 0)
    elif tuple(bx) == tuple(bw):
        call(x.ptr, w.ptr, scales.ptr, _ptr(biases), out.ptr, nb, x_mat, w_mat, s_mat)
    else:
        # General broadcasting: one call per output batch with the operands' own batch index.
        xi = np.broadcast_to(np.arange(int(np.prod(bx)) if bx else 1).reshape(bx or (1,)), batch).reshape(-1)
        wi = np.broadcast_to(np.arange(int(np.prod(bw))).reshape(bw), batch).reshape(-1)
        isz = _ITEMSIZE[dtype]
        ssz = isz if biases is not None else 1
        for i in range(nb):
            off = lambda a, n, size: C.c_void_p(a.ptr.value + int(n) * size)
            call(off(x, xi[i], x_mat * isz), off(w, wi[i], w_mat * 4), off(scales, wi[i], s_mat * ssz),
                 None if biases is None else off(biases, wi[i], s_mat * ssz), off(out, i, M * N * isz), 1, 0, 0, 0)
    return out.reshape(N) if vector and not batch else (out.reshape(batch + (N,)) if vector else out)


def gather_qmm(x: Array, q: Quantized, lhs_indices: Optional[Array] = None, rhs_indices: Optional[Array] = None,
               options: GatherQmm = GatherQmm(), offsets: Optional[Array] = None) -> Array:
    """ops::gather_qmm (ops.rs:1050-1078; quantized.rs:589-673): output batch i is
    ``x[lhs[i]] @ dequantize(w)[rhs[i]].T`` over the flattened batch dimensions."""
    quant = q.quant
    quant.checked("gather_qmm")
    if lhs_indices is None and rhs_indices is None:
        return quantized_matmul(x, q, options.transpose)
    _check_groups("gather_qmm", quant.mode, q.scales, q.biases)
    w = q.weight
    if x.ndim < 2 or w.ndim < 2 or (q.biases is not None and q.scales.shape != q.biases.shape):
        raise InvalidArgument(f"gather_qmm: x must be [..., M, K] and w [..., N, K'], got {list(x.shape)} and "
                              f"{list(w.shape)}")
    if q.global_scale is not None:
        if quant.mode != QuantMode.NVFP4:
            raise InvalidArgument("gather_qmm: global scale is only supported for 'nvfp4' quantization mode")
        _check_global("gather_qmm", quant, q.global_scale, experts_shape=w.shape[:-2])
    for name, idx in (("lhs", lhs_indices), ("rhs", rhs_indices)):
        if idx is not None and idx.dtype not in (U32, I32):
            raise InvalidArgument("gather_qmm: indices must be integers")
    dtype, x, scales, biases = _promote("gather_qmm", x, q)
    cols = _columns("gather_qmm", w, scales, biases, quant)
    rows_w = w.shape[-2]
    inner, N = (cols, rows_w) if options.transpose else (rows_w, cols)
    M, K = x.shape[-2], x.shape[-1]
    if K != inner:
        raise InvalidArgument(f"gather_qmm: shapes {list(x.shape)} and {list(w.shape)} do not match")
    x_batches = int(np.prod(x.shape[:-2])) if x.ndim > 2 else 1
    experts = int(np.prod(w.shape[:-2])) if w.ndim > 2 else 1
    dev = x.dev
    # Indices broadcast together; either defaults to every batch of its operand in order
    # (quantized.rs:739-767).  Explicit broadcasting is materialised on the host.
    lshape = tuple(lhs_indices.shape) if lhs_indices is not None else tuple(x.shape[:-2])
    rshape = tuple(rhs_indices.shape) if rhs_indices is not None else tuple(w.shape[:-2])
    try:
        ishape = tuple(np.broadcast_shapes(lshape, rshape))
    except ValueError:
        raise InvalidArgument(f"gather_qmm: index shapes {list(lshape)} and {list(rshape)} do not broadcast") from None
    rows = int(np.prod(ishape)) if ishape else 1

    def flat(idx, default_n, shape):
        if idx is not None and tuple(idx.shape) == ishape:
            return idx
        host = idx.to_numpy().astype(np.uint32) if idx is not None else np.arange(default_n, dtype=np.uint32).reshape(shape)
        return dev.array(np.ascontiguousarray(np.broadcast_to(host, ishape)), U32)

    lhs_default = lhs_indices is None and lshape == ishape
    lhs = None if lhs_default else flat(lhs_indices, x_batches, lshape)
    rhs = flat(rhs_indices, experts, rshape)
    out = dev.empty(ishape + (M, N), dtype)
    c = quant._c()
    _check(_ffi.lib().nvc_gather_qmm(dev._h, C.byref(c), dtype, int(options.transpose), x.ptr, w.ptr, scales.ptr,
                                     _ptr(biases), _ptr(q.global_scale), _ptr(lhs), rhs.ptr, _ptr(offsets),
                                     int(options.sorted_indices), rows, x_batches, M, N, K, experts, out.ptr))
    return out
