"""The CUDA path wrapped as a replay backend (see replay.OracleBackend for the interface).

Everything goes through nuvec_b200's public operations, i.e. through the C ABI.
"""
from __future__ import annotations

import numpy as np

import nuvec_b200 as nv
import oracle

MODE = {oracle.AFFINE: nv.QuantMode.AFFINE, oracle.MXFP4: nv.QuantMode.MXFP4,
        oracle.MXFP8: nv.QuantMode.MXFP8, oracle.NVFP4: nv.QuantMode.NVFP4}


def host(a: nv.Array, dtype=None):
    """Device array -> the oracle's storage convention (uint16 bit patterns for the halves)."""
    h = a.to_numpy()
    return h.view(np.uint16) if a.dtype == nv.F16 else h


class CudaBackend:
    name = "cuda"

    def __init__(self, dev=None):
        self.dev = dev or nv.Device.shared(0)

    def up(self, a, dtype):
        a = np.ascontiguousarray(a)
        if dtype == nv.F16:
            a = a.view(np.float16)
        return self.dev.array(a, dtype)

    def quantized(self, codes, scales, biases, dtype, mode, gs, bits, g=None):
        affine = mode == oracle.AFFINE
        return nv.Quantized(self.up(codes, nv.U32), self.up(scales, dtype if affine else nv.U8),
                            self.up(biases, dtype) if biases is not None else None,
                            nv.Quant(MODE[mode], gs, bits),
                            None if g is None else self.up(np.asarray(g, np.float32), nv.F32))

    def quantize(self, w, dtype, mode, gs, bits, global_scale=None):
        g = None if global_scale is None else self.up(np.asarray(global_scale, np.float32).reshape(1), nv.F32)
        q = nv.quantize(self.up(w, dtype), nv.Quant(MODE[mode], gs, bits), g)
        return host(q.weight), host(q.scales), None if q.biases is None else host(q.biases)

    def dequantize(self, codes, scales, biases, dtype, mode, gs, bits, global_scale=None, fused=False):
        g = None if global_scale is None else np.asarray(global_scale, np.float32).reshape(1)
        q = self.quantized(codes, scales, biases, dtype, mode, gs, bits, g)
        return host(nv.dequantize(q, None if mode == oracle.AFFINE else dtype, fused=fused))

    def quantized_matmul(self, x, codes, scales, biases, dtype, mode, gs, bits, transpose, global_scale=None):
        g = None if global_scale is None else np.asarray(global_scale, np.float32).reshape(1)
        q = self.quantized(codes, scales, biases, dtype, mode, gs, bits, g)
        return host(nv.quantized_matmul(self.up(x, dtype), q, transpose))

    def gather_qmm(self, x, codes, scales, biases, lhs, rhs, dtype, mode, gs, bits, transpose,
                   global_scale=None, sorted_indices=False):
        g = None if global_scale is None else np.asarray(global_scale, np.float32)
        q = self.quantized(codes, scales, biases, dtype, mode, gs, bits, g)
        li = None if lhs is None else self.up(np.asarray(lhs).astype(np.uint32), nv.U32)
        ri = None if rhs is None else self.up(np.asarray(rhs).astype(np.uint32), nv.U32)
        return host(nv.gather_qmm(self.up(x, dtype), q, li, ri, nv.GatherQmm(transpose, sorted_indices)))
