"""CPU restatement of the reference's checkpoint-format adapters.  TEST INFRASTRUCTURE ONLY.

What the reference does to quantized tensors between a checkpoint file and the product kernels
(crates/nuvec-lm/src/quant.rs and lib.rs), in plain numpy loops over small cases:

  * ``mxfp4_from_hf_blocks``  (quant.rs:9-34)    gpt-oss ``*_blocks`` -> MLX packed codes
  * ``split_interleaved``     (lib.rs:414-420)   every other entry along an axis (gate / up rows)
  * ``sanitize_gpt_oss``      (lib.rs:403-459)   the expert tensors of a Hugging Face gpt-oss file
  * ``convert_packed``        (quant.rs:36-199)  one AWQ / GPTQ layer -> MLX affine layout
  * ``infer_quant``           (lib.rs:461-480)   the quantization a layer's tensors were packed with
  * ``read_safetensors``                         the file format itself (header length, JSON, raw bytes)

float16 / bfloat16 data are ``uint16`` bit patterns with a dtype code, as in the rest of the oracle.
Pinned by the reference's own examples (the doc tests of quant.rs) and by its fixture pair
gpt_oss_hf_mxfp4 / gpt_oss_mxfp4, which hold the same experts in both layouts
(tests/golden/make_checkpoint_golden.py extracts them).
"""
from __future__ import annotations

import json
import struct

import numpy as np

from . import AFFINE, BF16, F16, F32, MXFP4, MXFP8, NVFP4, from_f32, to_f32

AWQ, GPTQ_V1, GPTQ_V2 = 0, 1, 2
# quant.rs:36-38: value c of a group of eight outputs sits in nibble AWQ_ORDER[c]
AWQ_ORDER = (0, 4, 1, 5, 2, 6, 3, 7)

_ST_DTYPES = {"U8": np.uint8, "I8": np.int8, "U16": np.uint16, "I16": np.int16, "U32": np.uint32, "I32": np.int32,
              "U64": np.uint64, "I64": np.int64, "F16": np.uint16, "BF16": np.uint16, "F32": np.float32, "F64": np.float64,
              "BOOL": np.bool_}


def read_safetensors(path):
    """name -> (safetensors dtype string, numpy array; F16 / BF16 as uint16 bit patterns)."""
    raw = open(path, "rb").read()
    (n,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + n])
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        lo, hi = info["data_offsets"]
        a = np.frombuffer(raw[8 + n + lo:8 + n + hi], dtype=_ST_DTYPES[info["dtype"]]).reshape(info["shape"])
        out[name] = (info["dtype"], a)
    return out


def mxfp4_from_hf_blocks(blocks):
    """uint8 [..., K / 32, 16] -> uint32 [..., K / 8]: the bytes reinterpreted (quant.rs:24-34)."""
    codes = np.ascontiguousarray(blocks).view(np.uint32)
    if codes.ndim < 2:
        return codes
    return codes.reshape(codes.shape[:-2] + (codes.shape[-2] * codes.shape[-1],))


def split_interleaved(v, first, axis):
    """v[..., first::2, ...] along axis (lib.rs:416-420)."""
    index = [slice(None)] * v.ndim
    index[axis] = slice(first, None, 2)
    return np.ascontiguousarray(v[tuple(index)])


def sanitize_gpt_oss(weights):
    """lib.rs:409-459 for the quantized and bias entries: name -> array in, name -> array out."""
    if any("experts.gate_proj." in k for k in weights):
        return dict(weights)
    out = {}
    for k, v in weights.items():
        if k.endswith("gate_up_proj_bias"):
            p = k[:-len("gate_up_proj_bias")]
            out[p + "gate_proj.bias"] = split_interleaved(v, 0, -1)
            out[p + "up_proj.bias"] = split_interleaved(v, 1, -1)
        elif k.endswith("down_proj_bias"):
            out[k[:-len("down_proj_bias")] + "down_proj.bias"] = v
        elif k.endswith("gate_up_proj_blocks"):
            p, codes = k[:-len("gate_up_proj_blocks")], mxfp4_from_hf_blocks(v)
            out[p + "gate_proj.weight"] = split_interleaved(codes, 0, -2)
            out[p + "up_proj.weight"] = split_interleaved(codes, 1, -2)
        elif k.endswith("gate_up_proj_scales"):
            p = k[:-len("gate_up_proj_scales")]
            out[p + "gate_proj.scales"] = split_interleaved(v, 0, -2)
            out[p + "up_proj.scales"] = split_interleaved(v, 1, -2)
        elif k.endswith("down_proj_blocks"):
            out[k[:-len("down_proj_blocks")] + "down_proj.weight"] = mxfp4_from_hf_blocks(v)
        elif k.endswith("down_proj_scales"):
            out[k[:-len("down_proj_scales")] + "down_proj.scales"] = v
        else:
            out[k] = v
    return out


def convert_packed(qweight, qzeros, scales, scale_dtype, fmt, bits, group_size, g_idx=None):
    """One layer of quant.rs:66-199.  qweight int32 [inputs, outputs / per_word] (AWQ) or
    [inputs / per_word, outputs] (GPTQ); qzeros int32 [groups, outputs / per_word] or None; scales
    [groups, outputs] in scale_dtype.  Returns (codes uint32 [outputs, inputs / per_word], scales
    [outputs, groups], biases [outputs, groups]), the last two in scale_dtype."""
    per_word, mask = 32 // bits, (1 << bits) - 1
    words = np.asarray(qweight).astype(np.int32).view(np.uint32)
    rows, cols = words.shape
    inputs, outputs = (rows, cols * per_word) if fmt == AWQ else (rows * per_word, cols)
    groups = -(-inputs // group_size)
    if inputs % group_size != 0 or tuple(scales.shape) != (groups, outputs):
        raise ValueError(f"{inputs} inputs and scales {scales.shape} do not match groups of {group_size}")
    if g_idx is not None:
        ids = np.asarray(g_idx).astype(np.int64)
        if len(ids) != inputs or np.any(ids != np.arange(inputs) // group_size):
            raise ValueError("g_idx reorders the inputs (activation reordering), which MLX's grouping cannot express")

    def code(i, o):
        if fmt == AWQ:
            return (int(words[i, o // per_word]) >> (4 * AWQ_ORDER[o % per_word])) & mask
        return (int(words[i // per_word, o]) >> (bits * (i % per_word))) & mask

    packed = np.zeros((outputs, inputs // per_word), np.uint32)
    for o in range(outputs):
        for i in range(inputs):
            packed[o, i // per_word] |= np.uint32(code(i, o) << (bits * (i % per_word)))
    if qzeros is None:
        zeros = np.full((groups, outputs), float(1 << (bits - 1)), np.float32)
    else:
        zw = np.asarray(qzeros).astype(np.int32).view(np.uint32)
        if zw.shape != (groups, -(-outputs // per_word)):
            raise ValueError(f"qzeros {zw.shape} for {groups} groups of {outputs} outputs")
        offset = 1 if fmt == GPTQ_V1 else 0
        zeros = np.zeros((groups, outputs), np.float32)
        for g in range(groups):
            for o in range(outputs):
                shift = 4 * AWQ_ORDER[o % per_word] if fmt == AWQ else bits * (o % per_word)
                zeros[g, o] = ((int(zw[g, o // per_word]) >> shift) & mask) + offset
    # -zero in float32 times the scales in float32, rounded to the scales' dtype; both [out, groups]
    biases = from_f32(np.ascontiguousarray((np.negative(zeros) * to_f32(scales, scale_dtype)).astype(np.float32).T), scale_dtype)
    return packed, np.ascontiguousarray(np.asarray(scales).T), biases


def infer_quant(weight_shape, scales_is_u8, scales_shape, default):
    """lib.rs:465-480.  default and the result are (mode, group_size, bits)."""
    if not scales_is_u8:
        return default if default[0] == AFFINE else (AFFINE, 64, 4)
    packed, groups = (weight_shape[-1] if weight_shape else 0), max(scales_shape[-1] if scales_shape else 0, 1)
    ratio = packed // groups
    if ratio == 2:
        return (NVFP4, 16, 4)
    if ratio == 8:
        return (MXFP8, 32, 8)
    return (MXFP4, 32, 4)
