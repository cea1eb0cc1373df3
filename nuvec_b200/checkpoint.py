"""Quantized checkpoints -> device-resident ``Quantized`` weights.

The part of the reference's loader that stands between a checkpoint file and the quantized products
(crates/nuvec-lm/src/lib.rs:225-480, crates/nuvec-lm/src/quant.rs, the tensor names of
crates/nuvec-core/src/quantized.rs:292-303), with the same names and argument meaning:

  * ``SafeTensors``            the file format: 8-byte header length, JSON header, raw little-endian data;
                               memory-mapped, a tensor's bytes go to the device as they are
  * ``mxfp4_from_hf_blocks``   gpt-oss ``*_blocks`` (uint8 [..., K / 32, 16]) as MLX codes (uint32 [..., K / 8]):
                               a reinterpretation of the same device bytes (quant.rs:9-34)
  * ``sanitize_gpt_oss``       Hugging Face gpt-oss experts -> ``experts.{gate,up,down}_proj.{weight,scales,bias}``,
                               the interleaved gate / up rows taken apart on the device (lib.rs:403-459)
  * ``convert_packed``         AutoAWQ / GPTQ layers -> MLX's affine layout on the device (quant.rs:36-199,
                               ``nvc_convert_packed``); the other float tensors in the scales' dtype
  * ``packed_format``          config.json's ``quantization_config`` -> (format, Quant) (config.rs:1115-1190)
  * ``infer_quant``            the quantization a layer's tensors were packed with (lib.rs:461-480)
  * ``load_quantized``         all of it: a file -> {layer path: Quantized}, optionally with the weight scales
                               laid out once for the block-scaled product (``qqmm_prepare_scales``)

Everything that touches tensor data runs in libnuvec_cuda.so; this module parses, names and checks.
"""
from __future__ import annotations

import json
import mmap
import struct
from pathlib import Path
from typing import Dict, Optional, Tuple

import numpy as np

from . import ops
from ._ffi import BF16, F16, F32, I32, U8, U32
from .ops import Array, Device, InvalidArgument, Quant, QuantMode, Quantized, UnsupportedError

AWQ, GPTQ_V1, GPTQ_V2 = 0, 1, 2  # NVC_PACKED_*

_DEVICE_DTYPE = {"U8": U8, "U32": U32, "I32": I32, "F16": F16, "BF16": BF16, "F32": F32}
_HOST_DTYPE = {"BOOL": np.bool_, "U8": np.uint8, "I8": np.int8, "U16": np.uint16, "I16": np.int16, "U32": np.uint32,
               "I32": np.int32, "U64": np.uint64, "I64": np.int64, "F16": np.float16, "BF16": np.uint16,
               "F32": np.float32, "F64": np.float64}


class SafeTensors:
    """A memory-mapped safetensors file.  ``numpy(name)`` is a view of the mapping (bfloat16 as uint16
    bit patterns); ``upload(dev, name)`` copies the tensor's bytes to the device unchanged."""

    def __init__(self, path):
        self.path = Path(path)
        self._file = open(self.path, "rb")
        size = self.path.stat().st_size
        if size < 8:
            raise InvalidArgument(f"{self.path}: not a safetensors file ({size} bytes)")
        self._map = mmap.mmap(self._file.fileno(), 0, access=mmap.ACCESS_READ)
        (n,) = struct.unpack("<Q", self._map[:8])
        if n > size - 8:
            raise InvalidArgument(f"{self.path}: header of {n} bytes in a file of {size}")
        try:
            header = json.loads(self._map[8:8 + n])
        except ValueError as e:
            raise InvalidArgument(f"{self.path}: header is not JSON ({e})") from None
        self.metadata = header.pop("__metadata__", None) or {}
        self._base = 8 + n
        self._entries = {}
        for name, info in header.items():
            lo, hi = info["data_offsets"]
            dtype, shape = info["dtype"], tuple(int(d) for d in info["shape"])
            if dtype not in _HOST_DTYPE:
                raise UnsupportedError(f"{self.path}: {name} has dtype {dtype}")
            want = int(np.prod(shape, dtype=np.int64)) * np.dtype(_HOST_DTYPE[dtype]).itemsize
            if lo < 0 or hi < lo or self._base + hi > size or hi - lo != want:
                raise InvalidArgument(f"{self.path}: {name} spans bytes {lo}..{hi} for {dtype} {list(shape)}")
            self._entries[name] = (dtype, shape, lo, hi)

    def keys(self):
        return self._entries.keys()

    def __contains__(self, name):
        return name in self._entries

    def info(self, name) -> Tuple[str, Tuple[int, ...]]:
        dtype, shape, _, _ = self._entries[name]
        return dtype, shape

    def numpy(self, name) -> np.ndarray:
        dtype, shape, lo, hi = self._entries[name]
        return np.frombuffer(self._map, dtype=_HOST_DTYPE[dtype], count=int(np.prod(shape, dtype=np.int64)),
                             offset=self._base + lo).reshape(shape)

    def upload(self, dev: Device, name) -> Array:
        dtype, _ = self.info(name)
        if dtype not in _DEVICE_DTYPE:
            raise UnsupportedError(f"{self.path}: {name} ({dtype}) has no device dtype")
        return dev.array(self.numpy(name), _DEVICE_DTYPE[dtype])

    def close(self):
        try:
            self._map.close()
        except BufferError:  # numpy views of the mapping are still alive: it goes with the last of them
            pass
        self._file.close()


# ── gpt-oss (Hugging Face layout) ────────────────────────────────────────────────────────────
def mxfp4_from_hf_blocks(blocks: Array) -> Array:
    """uint8 [..., K / 32, 16] -> uint32 [..., K / 8], the same device bytes (quant.rs:24-34)."""
    if blocks.dtype != U8 or blocks.ndim < 2 or blocks.shape[-1] % 4 != 0:
        raise InvalidArgument(f"mxfp4_from_hf_blocks: uint8 blocks expected, got {list(blocks.shape)}")
    root = blocks if blocks._base is None else blocks._base
    shape = blocks.shape[:-2] + (blocks.shape[-2] * blocks.shape[-1] // 4,)
    return Array(blocks.dev, shape, U32, _base=root, _offset=blocks._offset)


def split_interleaved(v: Array, first: int, axis: int) -> Array:
    """``v[..., first::2, ...]`` along ``axis`` (-1 or -2), on the device (lib.rs:414-420)."""
    if axis not in (-1, -2) or v.ndim < -axis:
        raise InvalidArgument(f"split_interleaved: axis {axis} of {list(v.shape)}")
    n = v.shape[axis]
    inner = 1 if axis == -1 else v.shape[-1]
    outer = v.size // (n * inner) if n * inner else 0
    shape = list(v.shape)
    shape[axis] = len(range(first, n, 2))
    out = v.dev.empty(tuple(shape), v.dtype)
    from . import _ffi
    ops._check(_ffi.lib().nvc_take_strided(v.dev._h, v.ptr, outer, n, inner * v.itemsize, first, 2, out.ptr))
    return out


def sanitize_gpt_oss(weights: Dict[str, Array]) -> Dict[str, Array]:
    """lib.rs:409-459 for the experts' quantized tensors and biases.  (The full-precision layout of the same
    experts, which the reference transposes, is outside the quantized path.)"""
    if any("experts.gate_proj." in k for k in weights):
        return dict(weights)  # converted already
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
        elif k.endswith("experts.gate_up_proj") or k.endswith("experts.down_proj"):
            raise UnsupportedError(f"{k}: full-precision gpt-oss experts are not on the quantized path")
        else:
            out[k] = v
    return out


# ── AWQ / GPTQ ───────────────────────────────────────────────────────────────────────────────
def packed_format(quantization_config: Optional[dict]) -> Optional[Tuple[int, Quant]]:
    """config.json's ``quantization_config`` of a Hugging Face AWQ / GPTQ checkpoint -> (format, Quant), None
    for anything this loader leaves alone (config.rs:1115-1190)."""
    q = quantization_config
    if not q:
        return None
    method = q.get("quant_method", "")
    if method not in ("awq", "gptq"):
        return None
    bits, group = int(q.get("bits", 4) or 4), int(q.get("group_size", 128) or 128)
    if group not in (32, 64, 128):
        raise InvalidArgument(f"{method}: group size {group} (MLX's affine kernels take 32, 64 or 128)")
    if method == "awq":
        version = q.get("version", "gemm") or "gemm"
        if version.lower() != "gemm" or bits != 4:
            raise InvalidArgument(f"awq: version {version!r} with {bits} bits (4-bit GEMM checkpoints load)")
        return AWQ, Quant.affine(group, 4)
    if bits not in (4, 8):
        raise InvalidArgument(f"gptq: {bits} bits (4 and 8 load)")
    if q.get("desc_act") is True:
        raise InvalidArgument("gptq: activation reordering (`desc_act`) is not supported; use a checkpoint quantized without it")
    v1 = (q.get("checkpoint_format") or "gptq") != "gptq_v2"
    return (GPTQ_V1 if v1 else GPTQ_V2), Quant.affine(group, bits)


def convert_packed_layer(dev: Device, fmt: int, quant: Quant, qweight: Array, scales: Array, qzeros: Optional[Array] = None,
                         g_idx: Optional[np.ndarray] = None, prefix: str = "") -> Quantized:
    """One ``{prefix}.qweight/.qzeros/.scales[/.g_idx]`` -> MLX's affine ``Quantized`` (quant.rs:84-193)."""
    if quant.mode != QuantMode.AFFINE:
        raise InvalidArgument(f"{prefix}: AWQ and GPTQ layers are affine")
    bits, group = quant.bits, quant.group_size
    per_word = 32 // bits
    if qweight.ndim != 2:
        raise InvalidArgument(f"{prefix}: a 2-D packed tensor, got {list(qweight.shape)}")
    rows, cols = qweight.shape
    inputs, outputs = (rows, cols * per_word) if fmt == AWQ else (rows * per_word, cols)
    groups = -(-inputs // group)
    if inputs % group != 0 or tuple(scales.shape) != (groups, outputs):
        raise InvalidArgument(f"{prefix}: {inputs} inputs and scales {list(scales.shape)} do not match groups of {group}")
    if g_idx is not None:
        ids = np.asarray(g_idx).astype(np.int64).reshape(-1)
        if len(ids) != inputs or np.any(ids != np.arange(inputs) // group):
            raise InvalidArgument(f"{prefix}: g_idx reorders the inputs (activation reordering), which MLX's grouping cannot express")
    if qzeros is not None and tuple(qzeros.shape) != (groups, -(-outputs // per_word)):
        raise InvalidArgument(f"{prefix}: qzeros {list(qzeros.shape)} for {groups} groups of {outputs} outputs")
    if qweight.dtype not in (I32, U32) or (qzeros is not None and qzeros.dtype not in (I32, U32)):
        raise InvalidArgument(f"{prefix}: int32 qweight and qzeros expected")
    codes = dev.empty((outputs, inputs // per_word), U32)
    s_out, b_out = dev.empty((outputs, groups), scales.dtype), dev.empty((outputs, groups), scales.dtype)
    from . import _ffi
    ops._check(_ffi.lib().nvc_convert_packed(dev._h, fmt, bits, group, scales.dtype, qweight.ptr, ops._ptr(qzeros), scales.ptr,
                                             inputs, outputs, codes.ptr, s_out.ptr, b_out.ptr))
    return Quantized(codes, s_out, b_out, quant)


def infer_quant(weight: Array, scales: Array, default: Quant) -> Quant:
    """lib.rs:465-480: uint8 scales mean a floating-point mode, told apart by the packed words per group."""
    if scales.dtype != U8:
        return default if default.mode == QuantMode.AFFINE else Quant()
    packed = weight.shape[-1] if weight.ndim else 0
    groups = max(scales.shape[-1] if scales.ndim else 0, 1)
    ratio = packed // groups
    if ratio == 2:
        return Quant.new(QuantMode.NVFP4)
    if ratio == 8:
        return Quant.new(QuantMode.MXFP8)
    return Quant.new(QuantMode.MXFP4)


# ── a whole file ─────────────────────────────────────────────────────────────────────────────
def load_quantized(dev: Device, path, default: Quant = Quant(), quantization_config: Optional[dict] = None,
                   prepare_qqmm: bool = False):
    """Every quantized layer of a safetensors file as {layer path: Quantized}; the remaining tensors that have
    a device dtype as {name: Array}.

    MLX files carry ``{path}.weight`` (uint32), ``.scales`` and, for affine, ``.biases``
    (quantized.rs:292-303); Hugging Face gpt-oss files their ``*_blocks`` / ``*_scales``; AWQ / GPTQ files
    ``.qweight`` / ``.qzeros`` / ``.scales`` (with ``quantization_config`` of the model's config.json).
    With ``prepare_qqmm`` the NVFP4 / MXFP4 layers also get their scales in the tensor core's layout
    (returned as a third dict, {layer path: Array}) for ``qqmm(x, q, prepared=...)``."""
    st = SafeTensors(path)
    try:
        packed = packed_format(quantization_config)
        layers: Dict[str, Quantized] = {}
        used = set()
        if packed is not None:
            fmt, quant = packed
            for name in [k for k in st.keys() if k.endswith(".qweight")]:
                prefix = name[:-len(".qweight")]
                if prefix + ".scales" not in st:
                    raise InvalidArgument(f"{prefix}: qweight without scales")
                zeros = st.upload(dev, prefix + ".qzeros") if prefix + ".qzeros" in st else None
                g_idx = st.numpy(prefix + ".g_idx") if prefix + ".g_idx" in st else None
                layers[prefix] = convert_packed_layer(dev, fmt, quant, st.upload(dev, name), st.upload(dev, prefix + ".scales"),
                                                      zeros, g_idx, prefix)
                used.update(prefix + s for s in (".qweight", ".qzeros", ".scales", ".g_idx"))
        rest = {k: st.upload(dev, k) for k in st.keys() if k not in used and st.info(k)[0] in _DEVICE_DTYPE}
        if any(k.endswith("_blocks") for k in rest):
            rest = sanitize_gpt_oss(rest)
        for name in [k for k in rest if k.endswith(".scales")]:
            prefix = name[:-len(".scales")]
            weight = rest.get(prefix + ".weight")
            if weight is None or weight.dtype != U32:
                continue
            scales, biases = rest[name], rest.get(prefix + ".biases")
            quant = infer_quant(weight, scales, default)
            if quant.mode == QuantMode.AFFINE and biases is None:
                raise InvalidArgument(f"{prefix}: affine weight without biases")
            layers[prefix] = Quantized(weight, scales, biases if quant.mode == QuantMode.AFFINE else None, quant)
            for s in (".weight", ".scales", ".biases"):
                rest.pop(prefix + s, None)
        if packed is not None:
            # as mlx-lm leaves an AWQ model: every other float tensor in the scales' dtype (quant.rs:186-194)
            dtypes = {q.scales.dtype for q in layers.values()}
            if len(dtypes) == 1:
                (dtype,) = dtypes
                rest = {k: (v.astype(dtype) if v.dtype in (F16, BF16, F32) and v.dtype != dtype else v) for k, v in rest.items()}
        if not prepare_qqmm:
            return layers, rest
        prepared = {p: ops.qqmm_prepare_scales(q) for p, q in layers.items()
                    if q.quant.mode in (QuantMode.NVFP4, QuantMode.MXFP4) and q.weight.ndim == 2 and q.global_scale is None}
        return layers, rest, prepared
    finally:
        dev.synchronize()
        st.close()
