"""ctypes binding of libnuvec_cuda.so (include/nuvec_cuda.h).

The library is the product: importing this module fails loudly when the shared object is
missing or does not load -- there is no CPU fallback.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "libnuvec_cuda.so"

OK = 0
ERR_INVALID_ARGUMENT, ERR_UNSUPPORTED, ERR_OUT_OF_MEMORY, ERR_NO_DEVICE, ERR_DRIVER, ERR_COMM = -1, -2, -3, -4, -5, -6
U8, U32, I32, F16, BF16, F32 = 1, 3, 7, 9, 10, 11
AFFINE, MXFP4, MXFP8, NVFP4 = 0, 1, 2, 3


class Quant(C.Structure):
    _fields_ = [("mode", C.c_int32), ("group_size", C.c_int32), ("bits", C.c_int32)]


class HostProduct(C.Structure):
    """nvc_host_product: one entry of nvc_quantized_matmul_host_batch."""
    _fields_ = [("quant", Quant), ("dtype", C.c_int32), ("transpose", C.c_int32), ("host_x", C.c_void_p),
                ("w", C.c_void_p), ("scales", C.c_void_p), ("biases", C.c_void_p), ("global_scale", C.c_void_p),
                ("M", C.c_int64), ("N", C.c_int64), ("K", C.c_int64), ("host_y", C.c_void_p)]


class Info(C.Structure):
    _fields_ = [("name", C.c_char * 128), ("cc_major", C.c_int32), ("cc_minor", C.c_int32),
                ("multiprocessors", C.c_int32), ("driver_version", C.c_int32),
                ("total_memory", C.c_uint64), ("l2_bytes", C.c_uint64)]


class MemStats(C.Structure):
    _fields_ = [("active", C.c_uint64), ("cached", C.c_uint64), ("peak", C.c_uint64),
                ("limit", C.c_uint64), ("cache_limit", C.c_uint64), ("allocations", C.c_uint64)]


P, I32T, I64T, SZ = C.c_void_p, C.c_int32, C.c_int64, C.c_size_t
QP = C.POINTER(Quant)
PP = C.POINTER(C.c_void_p)

# name -> (restype, argtypes); every symbol include/nuvec_cuda.h declares.
SIGNATURES = {
    "nvc_last_error": (None, [C.c_char_p, SZ]),
    "nvc_version": (C.c_char_p, []),
    "nvc_device_open": (I32T, [I32T, C.POINTER(P)]),
    "nvc_device_close": (I32T, [P]),
    "nvc_device_info": (I32T, [P, C.POINTER(Info)]),
    "nvc_synchronize": (I32T, [P]),
    "nvc_device_set_stream": (I32T, [P, P]),
    "nvc_device_stream": (P, [P]),
    "nvc_launch_count": (C.c_uint64, [P]),
    "nvc_alloc": (I32T, [P, SZ, C.POINTER(P)]),
    "nvc_free": (I32T, [P, P]),
    "nvc_memcpy_h2d": (I32T, [P, P, P, SZ]),
    "nvc_memcpy_d2h": (I32T, [P, P, P, SZ]),
    "nvc_memcpy_d2d": (I32T, [P, P, P, SZ]),
    "nvc_memset": (I32T, [P, P, C.c_int, SZ]),
    "nvc_host_alloc": (I32T, [SZ, C.POINTER(P)]),
    "nvc_host_free": (I32T, [P]),
    "nvc_mem_stats_get": (I32T, [P, C.POINTER(MemStats)]),
    "nvc_set_memory_limit": (I32T, [P, C.c_uint64]),
    "nvc_set_cache_limit": (I32T, [P, C.c_uint64]),
    "nvc_clear_cache": (I32T, [P]),
    "nvc_reset_peak": (I32T, [P]),
    "nvc_event_create": (I32T, [P, C.POINTER(P)]),
    "nvc_event_destroy": (I32T, [P]),
    "nvc_event_record": (I32T, [P, P]),
    "nvc_event_synchronize": (I32T, [P]),
    "nvc_event_elapsed_ms": (I32T, [P, P, C.POINTER(C.c_float)]),
    "nvc_graph_begin": (I32T, [P]),
    "nvc_graph_end": (I32T, [P, C.POINTER(P)]),
    "nvc_graph_launch": (I32T, [P, P]),
    "nvc_graph_destroy": (I32T, [P]),
    "nvc_quantize": (I32T, [P, QP, I32T, P, I64T, I64T, P, P, P, P]),
    "nvc_dequantize": (I32T, [P, QP, I32T, P, P, P, P, I64T, I64T, P, I32T]),
    "nvc_quantized_matmul": (I32T, [P, QP, I32T, I32T, P, P, P, P, P, I64T, I64T, I64T, I64T, I64T,
                                    I64T, I64T, I64T, P]),
    "nvc_sorted_offsets": (I32T, [P, P, I64T, I64T, P]),
    "nvc_gather_qmm": (I32T, [P, QP, I32T, I32T, P, P, P, P, P, P, P, P, I32T, I64T, I64T, I64T, I64T,
                              I64T, I64T, P]),
    "nvc_moe_route": (I32T, [P, I32T, P, I64T, I64T, I64T, I32T, P, P]),
    "nvc_weighted_sum": (I32T, [P, I32T, P, P, I64T, I64T, I64T, P]),
    "nvc_expert_bias_add": (I32T, [P, I32T, P, P, P, I64T, I64T, I64T]),
    "nvc_moe_sort": (I32T, [P, P, I64T, I64T, I64T, P, P, P, P, P]),
    "nvc_take_rows": (I32T, [P, P, I64T, I64T, P, I64T, P]),
    "nvc_quantized_embedding": (I32T, [P, QP, I32T, P, P, P, I64T, I64T, P, I64T, P]),
    "nvc_qqmm": (I32T, [P, QP, I32T, P, P, P, I64T, I64T, I64T, P]),
    "nvc_qqmm_scales_bytes": (SZ, [QP, I64T, I64T]),
    "nvc_qqmm_prepare_scales": (I32T, [P, QP, P, I64T, I64T, P]),
    "nvc_qqmm_prepared": (I32T, [P, QP, I32T, P, P, P, I64T, I64T, I64T, P]),
    "nvc_convert_packed": (I32T, [P, I32T, I32T, I32T, I32T, P, P, P, I64T, I64T, P, P, P]),
    "nvc_quantized_attention": (I32T, [P, QP, I32T, P, P, P, P, P, P, P, P, I64T, I64T, I64T, I64T, I64T, I64T, I64T, C.c_float, I32T, P]),
    "nvc_quantize_dequantize": (I32T, [P, QP, I32T, P, I64T, I64T, P, P]),
    "nvc_set_row_exact": (I32T, [P, I32T]),
    "nvc_row_exact": (I32T, [P]),
    "nvc_take_strided": (I32T, [P, P, I64T, I64T, I64T, I64T, I64T, P]),
    "nvc_rms_norm": (I32T, [P, I32T, P, P, C.c_float, I64T, I64T, P]),
    "nvc_add_rms_norm": (I32T, [P, I32T, P, P, P, C.c_float, I64T, I64T, P, P]),
    "nvc_swiglu": (I32T, [P, I32T, P, P, I64T, P]),
    "nvc_swiglu_oai": (I32T, [P, I32T, P, P, C.c_float, C.c_float, I64T, P]),
    "nvc_quantized_matmul_host": (I32T, [P, QP, I32T, I32T, P, P, P, P, P, I64T, I64T, I64T, P]),
    "nvc_quantized_matmul_host_async": (I32T, [P, QP, I32T, I32T, P, P, P, P, P, I64T, I64T, I64T, P]),
    "nvc_quantized_matmul_host_batch": (I32T, [P, C.POINTER(HostProduct), SZ]),
    "nvc_quantized_matmul_noalloc": (I32T, [P, QP, P, P, P, P, I64T, I64T, I64T, P]),
    "nvc_comm_unique_id": (I32T, [P]),
    "nvc_comm_init": (I32T, [P, I32T, I32T, P, C.POINTER(P)]),
    "nvc_comm_init_timeout": (I32T, [P, I32T, I32T, P, I64T, C.POINTER(P)]),
    "nvc_all_reduce": (I32T, [P, I32T, I32T, P, SZ]),
    "nvc_send": (I32T, [P, P, SZ, I32T]),
    "nvc_recv": (I32T, [P, P, SZ, I32T]),
    "nvc_comm_rank": (I32T, [P]),
    "nvc_comm_size": (I32T, [P]),
    "nvc_all_gather": (I32T, [P, P, P, SZ]),
    "nvc_all_reduce_sum": (I32T, [P, I32T, P, SZ]),
    "nvc_comm_health": (I32T, [P]),
    "nvc_comm_abort": (I32T, [P]),
    "nvc_comm_destroy": (I32T, [P]),
    "nvc_symm_alloc": (I32T, [P, SZ, PP, P]),
    "nvc_symm_open": (I32T, [P, P, PP]),
    "nvc_symm_close": (I32T, [P, P]),
    "nvc_symm_free": (I32T, [P, P]),
    "nvc_peer_group_create": (I32T, [P, I32T, I32T, PP, SZ, PP]),
    "nvc_peer_group_destroy": (I32T, [P]),
    "nvc_gather_footprint": (SZ, [I32T, I64T, I64T]),
    "nvc_all_sum_footprint": (SZ, [I32T, I64T, I64T]),
    "nvc_quantized_matmul_gather": (I32T, [P, P, QP, P, P, P, P, I64T, I64T, I64T, SZ]),
    "nvc_quantized_matmul_all_sum": (I32T, [P, P, QP, P, P, P, P, I64T, I64T, I64T, P, SZ]),
}

_lib = None


def lib():
    """The loaded library, with every signature set.  Raises if it is not built."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise ImportError(f"{LIB_PATH} is missing: build it with `python -m nuvec_b200.build` "
                              "(there is no CPU fallback)")
        handle = C.CDLL(str(LIB_PATH))
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)  # AttributeError if the export is missing
            fn.restype, fn.argtypes = res, args
        _lib = handle
    return _lib


def last_error() -> str:
    buf = C.create_string_buffer(512)
    lib().nvc_last_error(buf, 512)
    return buf.value.decode(errors="replace")
