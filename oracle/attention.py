"""CPU restatement of fast::quantized_attention.  TEST INFRASTRUCTURE ONLY.

``dense``     attention over the dequantized cache in float32/float64: the yardstick of the reference's own
              test (crates/nuvec-core/tests/quantized.rs:1964-2031: `scaled_dot_product_attention` of the float32
              queries over `dequantize(F32)` of keys and values, with the sinks in float32).
``composed``  the reference's CPU path, mlx-lm's composition (crates/nuvec-core/src/fast/imp.rs:3996-4035): the
              queries times the scale (rounded to their type), grouped by key head; `quantized_matmul` with the
              keys; the sinks' column; a precise softmax (float32 inside, rounded to the type);
              `quantized_matmul` with the values, untransposed.

Pinned by the `*_l1_*` records of the reference's fixture crates/nuvec-lm/tests/fixtures/kv_quant_attention.safetensors
(mlx-lm's outputs; tests/golden/make_attention_golden.py copies them), within the float tolerance the reference
itself allows off the GPU they were recorded on.
"""
from __future__ import annotations

import numpy as np

from . import AFFINE, from_f32, quantized_matmul, to_f32


def _dense_cache(codes, scales, biases, dtype, gs, bits):
    """float32 scale * code + bias of a cache [B, H, S, D * bits / 32] (codes packed low bits first)."""
    B, H, S, W = codes.shape
    D = W * 32 // bits
    flat = np.ascontiguousarray(codes).reshape(-1, W)
    bitstream = np.unpackbits(flat.view(np.uint8), axis=1, bitorder="little").reshape(len(flat), D, bits)
    values = (bitstream.astype(np.uint32) << np.arange(bits, dtype=np.uint32)).sum(axis=2).astype(np.float32)
    s32 = np.repeat(to_f32(scales, dtype).reshape(len(flat), -1), gs, axis=1)
    b32 = np.repeat(to_f32(biases, dtype).reshape(len(flat), -1), gs, axis=1)
    return (s32 * values + b32).astype(np.float32).reshape(B, H, S, D)


def dense(q, k, v, dtype, gs, bits, scale, sinks=None, causal=False):
    """q [B, Hq, L, D] of dtype; k, v = (codes, scales, biases) with [B, Hkv, S, ...]; returns float64 [B, Hq, L, D]."""
    q32 = to_f32(q, dtype).astype(np.float64)
    kd = _dense_cache(*k, dtype, gs, bits).astype(np.float64)
    vd = _dense_cache(*v, dtype, gs, bits).astype(np.float64)
    B, Hq, L, D = q32.shape
    rep = Hq // kd.shape[1]
    out = np.zeros((B, Hq, L, D))
    for b in range(B):
        for h in range(Hq):
            s = (q32[b, h] * np.float64(np.float32(scale))) @ kd[b, h // rep].T          # [L, S]
            if causal:  # row l stands at position S - L + l
                S_ = s.shape[1]
                s = np.where(np.arange(S_)[None, :] <= (S_ - L + np.arange(L))[:, None], s, -np.inf)
            if sinks is not None:
                s = np.concatenate([s, np.full((L, 1), float(to_f32(sinks, dtype)[h]))], axis=1)
            m = s.max(axis=1, keepdims=True) if s.shape[1] else np.zeros((L, 1))
            e = np.exp(s - m)
            p = e / e.sum(axis=1, keepdims=True) if s.shape[1] else e
            if sinks is not None:
                p = p[:, :-1]
            out[b, h] = p @ vd[b, h // rep]
    return out


def composed(q, k, v, dtype, gs, bits, scale, sinks=None):
    """fast/imp.rs:3996-4035 with the oracle's products; returns an array of dtype [B, Hq, L, D]."""
    B, Hq, L, D = q.shape
    Hkv, S = k[0].shape[1], k[0].shape[2]
    rep = Hq // Hkv
    qs = from_f32((to_f32(q, dtype) * np.float32(scale)).astype(np.float32), dtype)
    out = np.zeros((B, Hq, L, D), dtype=qs.dtype)
    for b in range(B):
        for hk in range(Hkv):
            x = np.ascontiguousarray(qs[b, hk * rep:(hk + 1) * rep].reshape(rep * L, D))
            scores = quantized_matmul(x, k[0][b, hk], k[1][b, hk], k[2][b, hk], dtype, AFFINE, gs, bits)          # [rep * L, S]
            s32 = to_f32(scores, dtype).reshape(rep, L, S)
            if sinks is not None:
                col = to_f32(sinks, dtype)[hk * rep:(hk + 1) * rep].reshape(rep, 1, 1)
                s32 = np.concatenate([s32, np.broadcast_to(col, (rep, L, 1))], axis=2)
            m = s32.max(axis=2, keepdims=True)
            e = np.exp((s32 - m).astype(np.float32))
            p = from_f32((e / e.sum(axis=2, keepdims=True, dtype=np.float32)).astype(np.float32), dtype)
            if sinks is not None:
                p = p[:, :, :S]
            y = quantized_matmul(np.ascontiguousarray(p.reshape(rep * L, S)), v[0][b, hk], v[1][b, hk], v[2][b, hk], dtype, AFFINE, gs, bits,
                                 transpose=False)
            out[b, hk * rep:(hk + 1) * rep] = y.reshape(rep, L, D)
    return out
