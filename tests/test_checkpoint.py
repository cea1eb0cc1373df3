"""Checkpoint formats in front of the quantized products (crates/nuvec-lm/src/quant.rs, lib.rs:403-480).

Without a GPU: the oracle's restatement against the reference's own examples (the doc tests of quant.rs)
and against its fixture pair gpt_oss_hf_mxfp4 / gpt_oss_mxfp4 (tests/golden/checkpoint_gpt_oss_*.safetensors,
the same experts in Hugging Face's and in MLX's layout), and the host logic of the loader.
With a GPU: the device conversions against the oracle bit for bit, and the loader end to end.
"""
import json
import struct
from pathlib import Path

import numpy as np
import pytest

import oracle
from oracle import checkpoint as ock

GOLDEN = Path(__file__).resolve().parent / "golden"


def write_safetensors(path, tensors):
    """name -> (dtype string, numpy array)."""
    header, blobs, at = {}, [], 0
    for name, (dtype, a) in tensors.items():
        data = np.ascontiguousarray(a).tobytes()
        header[name] = {"dtype": dtype, "shape": list(a.shape), "data_offsets": [at, at + len(data)]}
        blobs.append(data)
        at += len(data)
    text = json.dumps(header).encode()
    Path(path).write_bytes(struct.pack("<Q", len(text)) + text + b"".join(blobs))


# ── oracle against the reference's examples and fixtures (CPU) ───────────────────────────────
def test_blocks_example_of_the_reference():
    # quant.rs:15-22: [[[[1,0,0,0, 2,0,0,0, 3,0,0,0, 4,0,0,0]]]] -> shape [1, 1, 4], values 1 2 3 4
    blocks = np.array([[[[1, 0, 0, 0, 2, 0, 0, 0, 3, 0, 0, 0, 4, 0, 0, 0]]]], np.uint8)
    codes = ock.mxfp4_from_hf_blocks(blocks)
    assert codes.shape == (1, 1, 4) and codes.dtype == np.uint32 and codes.reshape(-1).tolist() == [1, 2, 3, 4]


def test_gptq_example_of_the_reference():
    # quant.rs:51-65: GPTQ v2, 4-bit, 32 inputs (one group), one output: codes 0..16 twice down the inputs,
    # zero 8, scale 0.5 -> dequantized ((i % 16) - 8) * 0.5
    words = np.array([[sum((((r * 8 + k) % 16) << (4 * k)) for k in range(8))] for r in range(4)], np.uint32).view(np.int32)
    scales = np.array([[0.5]], np.float32).astype(np.float16).view(np.uint16)
    codes, s, b = ock.convert_packed(words, np.array([[8]], np.int32), scales, oracle.F16, ock.GPTQ_V2, 4, 32)
    dense = oracle.to_f32(oracle.dequantize(codes, s, b, oracle.F16, oracle.AFFINE, 32, 4), oracle.F16).reshape(-1)
    assert dense.tolist() == [((i % 16) - 8) * 0.5 for i in range(32)]


def test_gptq_v1_stores_zero_minus_one_and_missing_zeros_are_symmetric():
    rng = np.random.default_rng(1)
    words = rng.integers(0, 2 ** 32, (8, 16), dtype=np.uint32).view(np.int32)      # 64 inputs, 16 outputs
    scales = oracle.from_f32(rng.uniform(0.01, 0.1, (1, 16)).astype(np.float32), oracle.BF16)
    zeros = rng.integers(0, 2 ** 32, (1, 2), dtype=np.uint32)
    _, _, b2 = ock.convert_packed(words, zeros.view(np.int32), scales, oracle.BF16, ock.GPTQ_V2, 4, 64)
    _, _, b1 = ock.convert_packed(words, zeros.view(np.int32), scales, oracle.BF16, ock.GPTQ_V1, 4, 64)
    _, _, bs = ock.convert_packed(words, None, scales, oracle.BF16, ock.GPTQ_V2, 4, 64)
    z = np.array([[(int(zeros[0, o // 8]) >> (4 * (o % 8))) & 15 for o in range(16)]], np.float32)
    s32 = oracle.to_f32(scales, oracle.BF16)
    assert np.array_equal(b2, oracle.from_f32((-z * s32).T.copy(), oracle.BF16))
    assert np.array_equal(b1, oracle.from_f32((-(z + 1) * s32).T.copy(), oracle.BF16))
    assert np.array_equal(bs, oracle.from_f32((-8.0 * s32).T.copy(), oracle.BF16))


def test_awq_order_round_trip():
    # AutoAWQ packs output c of a group of eight into nibble AWQ_ORDER[c] (quant.rs:36-38): packing known
    # codes that way and converting gives them back, input-major.
    rng = np.random.default_rng(2)
    inputs, outputs = 64, 24
    codes = rng.integers(0, 16, (inputs, outputs), dtype=np.uint32)
    words = np.zeros((inputs, outputs // 8), np.uint32)
    for o in range(outputs):
        words[:, o // 8] |= codes[:, o] << np.uint32(4 * ock.AWQ_ORDER[o % 8])
    scales = np.ones((1, outputs), np.float32)
    packed, _, _ = ock.convert_packed(words.view(np.int32), None, scales, oracle.F32, ock.AWQ, 4, 64)
    back = np.array([[(int(packed[o, i // 8]) >> (4 * (i % 8))) & 15 for i in range(inputs)] for o in range(outputs)])
    assert np.array_equal(back, codes.T)


def test_g_idx_must_be_the_identity_grouping():
    words = np.zeros((8, 8), np.int32)
    scales = np.ones((2, 8), np.float32)
    ock.convert_packed(words, None, scales, oracle.F32, ock.GPTQ_V2, 4, 32, g_idx=np.arange(64) // 32)
    with pytest.raises(ValueError, match="reorders"):
        ock.convert_packed(words, None, scales, oracle.F32, ock.GPTQ_V2, 4, 32, g_idx=(np.arange(64) // 32)[::-1])
    with pytest.raises(ValueError, match="do not match"):
        ock.convert_packed(words, None, np.ones((1, 8), np.float32), oracle.F32, ock.GPTQ_V2, 4, 32)


def test_gpt_oss_fixture_pair_of_the_reference():
    hf = {k: v[1] for k, v in ock.read_safetensors(GOLDEN / "checkpoint_gpt_oss_hf.safetensors").items()}
    mlx = {k: v[1] for k, v in ock.read_safetensors(GOLDEN / "checkpoint_gpt_oss_mlx.safetensors").items()}
    got = ock.sanitize_gpt_oss(hf)
    assert sorted(got) == sorted(mlx)
    for name in mlx:
        assert got[name].shape == mlx[name].shape and np.array_equal(got[name], mlx[name]), name
    assert ock.sanitize_gpt_oss(mlx).keys() == mlx.keys()          # converted already: untouched


def test_infer_quant():
    affine = (oracle.AFFINE, 32, 8)
    assert ock.infer_quant((64, 8), False, (64, 1), affine) == affine
    assert ock.infer_quant((64, 8), False, (64, 1), (oracle.MXFP4, 32, 4)) == (oracle.AFFINE, 64, 4)
    assert ock.infer_quant((8, 64, 8), True, (8, 64, 2), affine) == (oracle.MXFP4, 32, 4)
    assert ock.infer_quant((64, 8), True, (64, 4), affine) == (oracle.NVFP4, 16, 4)
    assert ock.infer_quant((64, 16), True, (64, 2), affine) == (oracle.MXFP8, 32, 8)


# ── host logic of the loader (CPU: no device calls) ──────────────────────────────────────────
def test_safetensors_reader(tmp_path):
    from nuvec_b200 import checkpoint as ck
    rng = np.random.default_rng(0)
    tensors = {"a.weight": ("U32", rng.integers(0, 2 ** 32, (3, 5), dtype=np.uint32)),
               "a.scales": ("BF16", rng.integers(0, 2 ** 16, (3, 2), dtype=np.uint16)),
               "b": ("F16", rng.standard_normal((7,)).astype(np.float16)),
               "g": ("I64", np.arange(9, dtype=np.int64)), "empty": ("F32", np.zeros((0, 4), np.float32))}
    write_safetensors(tmp_path / "t.safetensors", tensors)
    st = ck.SafeTensors(tmp_path / "t.safetensors")
    assert sorted(st.keys()) == sorted(tensors)
    for name, (dtype, a) in tensors.items():
        assert st.info(name) == (dtype, a.shape)
        assert np.array_equal(st.numpy(name), a)
    st.close()
    (tmp_path / "bad.safetensors").write_bytes(struct.pack("<Q", 1000) + b"{}")
    with pytest.raises(ck.InvalidArgument):
        ck.SafeTensors(tmp_path / "bad.safetensors")
    header = json.dumps({"x": {"dtype": "F32", "shape": [4], "data_offsets": [0, 8]}}).encode()
    (tmp_path / "short.safetensors").write_bytes(struct.pack("<Q", len(header)) + header + b"\0" * 8)
    with pytest.raises(ck.InvalidArgument):
        ck.SafeTensors(tmp_path / "short.safetensors")


def test_packed_format_of_a_config():
    from nuvec_b200 import checkpoint as ck
    import nuvec_b200 as nv
    assert ck.packed_format(None) is None and ck.packed_format({"quant_method": "mxfp4"}) is None
    assert ck.packed_format({"bits": 4, "group_size": 64, "quant_method": "awq", "version": "gemm"}) == (ck.AWQ, nv.Quant.affine(64, 4))
    assert ck.packed_format({"bits": 4, "quant_method": "gptq"}) == (ck.GPTQ_V1, nv.Quant.affine(128, 4))
    assert ck.packed_format({"bits": 8, "group_size": 32, "quant_method": "gptq", "checkpoint_format": "gptq_v2"}) == (ck.GPTQ_V2, nv.Quant.affine(32, 8))
    for bad in ({"quant_method": "awq", "bits": 8}, {"quant_method": "awq", "version": "gemv"}, {"quant_method": "gptq", "bits": 3},
                {"quant_method": "gptq", "desc_act": True}, {"quant_method": "gptq", "group_size": 48}):
        with pytest.raises(ck.InvalidArgument):
            ck.packed_format(bad)


# ── device conversions and the loader (GPU) ──────────────────────────────────────────────────
def _dev():
    import nuvec_b200 as nv
    return nv, nv.Device.shared(0)


@pytest.mark.gpu
@pytest.mark.parametrize("fmt,bits,group,inputs,outputs,zeros", [
    ("awq", 4, 64, 128, 64, True), ("awq", 4, 128, 4096, 1024, True), ("awq", 4, 32, 96, 40, False),
    ("gptq1", 4, 64, 128, 72, True), ("gptq2", 8, 32, 160, 100, True), ("gptq2", 4, 128, 2048, 1000, False),
    ("gptq2", 2, 64, 256, 48, True)])
@pytest.mark.parametrize("dt", ["f16", "bf16", "f32"])
def test_convert_packed_on_the_device(fmt, bits, group, inputs, outputs, zeros, dt):
    from nuvec_b200 import checkpoint as ck
    nv, dev = _dev()
    code = {"awq": ock.AWQ, "gptq1": ock.GPTQ_V1, "gptq2": ock.GPTQ_V2}[fmt]
    dtype = {"f16": oracle.F16, "bf16": oracle.BF16, "f32": oracle.F32}[dt]
    per_word = 32 // bits
    rng = np.random.default_rng(inputs + outputs + bits)
    shape = (inputs, outputs // per_word) if code == ock.AWQ else (inputs // per_word, outputs)
    small = inputs * outputs <= 1 << 16      # the oracle's loops are Python: full check on the small cases
    qweight = rng.integers(0, 2 ** 32, shape, dtype=np.uint32).view(np.int32)
    groups = inputs // group
    qzeros = rng.integers(0, 2 ** 32, (groups, -(-outputs // per_word)), dtype=np.uint32).view(np.int32) if zeros else None
    scales = oracle.from_f32(rng.uniform(-0.1, 0.1, (groups, outputs)).astype(np.float32), dtype)
    sc = scales.view(np.float16) if dtype == oracle.F16 else scales
    q = ck.convert_packed_layer(dev, code, nv.Quant.affine(group, bits), dev.array(qweight, nv.I32), dev.array(sc, dtype),
                                dev.array(qzeros, nv.I32) if zeros else None, np.arange(inputs) // group, "layer")
    got_codes, got_s, got_b = q.weight.to_numpy(), q.scales.to_numpy().view(np.uint16 if dtype != oracle.F32 else np.float32), \
        q.biases.to_numpy().view(np.uint16 if dtype != oracle.F32 else np.float32)
    if small:
        want_codes, want_s, want_b = ock.convert_packed(qweight, qzeros, scales, dtype, code, bits, group)
    else:  # vectorised restatement of the same definition, itself checked against the loops on the small cases
        want_codes, want_s, want_b = _convert_packed_vectorised(qweight, qzeros, scales, dtype, code, bits, group)
    assert np.array_equal(got_codes, want_codes)
    assert np.array_equal(got_s, want_s.view(got_s.dtype))
    assert np.array_equal(got_b.view(np.uint8), np.ascontiguousarray(want_b).view(np.uint8))
    if small:
        v = _convert_packed_vectorised(qweight, qzeros, scales, dtype, code, bits, group)
        assert np.array_equal(v[0], want_codes) and np.array_equal(np.ascontiguousarray(v[2]).view(np.uint8), np.ascontiguousarray(want_b).view(np.uint8))


def _convert_packed_vectorised(qweight, qzeros, scales, dtype, fmt, bits, group):
    per_word, mask = 32 // bits, (1 << bits) - 1
    words = qweight.view(np.uint32)
    if fmt == ock.AWQ:
        order = np.array(ock.AWQ_ORDER)
        inputs, outputs = words.shape[0], words.shape[1] * 8
        codes = (words[:, :, None] >> (4 * order)[None, None, :].astype(np.uint32)) & mask      # [i, col, c]
        codes = codes.reshape(inputs, outputs)
    else:
        inputs, outputs = words.shape[0] * per_word, words.shape[1]
        codes = (words[:, None, :] >> (bits * np.arange(per_word, dtype=np.uint32))[None, :, None]) & mask  # [w, k, o]
        codes = codes.reshape(inputs, outputs)
    t = codes.T.reshape(outputs, inputs // per_word, per_word).astype(np.uint64)
    packed = (t << (bits * np.arange(per_word, dtype=np.uint64))[None, None, :]).sum(axis=2).astype(np.uint32)
    groups = inputs // group
    if qzeros is None:
        z = np.full((groups, outputs), float(1 << (bits - 1)), np.float32)
    else:
        zw = qzeros.view(np.uint32)
        o = np.arange(outputs)
        shift = (4 * np.array(ock.AWQ_ORDER)[o % per_word]) if fmt == ock.AWQ else bits * (o % per_word)
        z = ((zw[:, o // per_word] >> shift.astype(np.uint32)[None, :]) & mask).astype(np.float32) + (1 if fmt == ock.GPTQ_V1 else 0)
    biases = oracle.from_f32(np.ascontiguousarray((np.negative(z) * oracle.to_f32(scales, dtype)).astype(np.float32).T), dtype)
    return packed, np.ascontiguousarray(scales.T), biases


@pytest.mark.gpu
def test_convert_packed_rejects_what_the_reference_rejects():
    from nuvec_b200 import checkpoint as ck
    nv, dev = _dev()
    qw, sc = dev.array(np.zeros((8, 8), np.int32), nv.I32), dev.array(np.ones((2, 8), np.float32), nv.F32)
    quant = nv.Quant.affine(32, 4)
    with pytest.raises(nv.InvalidArgument, match="reorders"):
        ck.convert_packed_layer(dev, ck.GPTQ_V2, quant, qw, sc, None, (np.arange(64) // 32)[::-1], "l")
    with pytest.raises(nv.InvalidArgument, match="do not match"):
        ck.convert_packed_layer(dev, ck.GPTQ_V2, quant, qw, dev.array(np.ones((1, 8), np.float32), nv.F32), None, None, "l")
    with pytest.raises(nv.InvalidArgument, match="qzeros"):
        ck.convert_packed_layer(dev, ck.GPTQ_V2, quant, qw, sc, dev.array(np.zeros((2, 2), np.int32), nv.I32), None, "l")


@pytest.mark.gpu
def test_gpt_oss_checkpoint_loads_as_the_reference_converts_it():
    # The reference's fixture pair: the Hugging Face file through the loader must give the tensors of the MLX
    # file bit for bit, and the layers must multiply like the oracle's product of the MLX tensors.
    from nuvec_b200 import checkpoint as ck
    nv, dev = _dev()
    layers, rest = ck.load_quantized(dev, GOLDEN / "checkpoint_gpt_oss_hf.safetensors")
    mlx = {k: v[1] for k, v in ock.read_safetensors(GOLDEN / "checkpoint_gpt_oss_mlx.safetensors").items()}
    assert sorted(layers) == sorted({k[:-len(".weight")] for k in mlx if k.endswith(".weight")})
    for prefix, q in layers.items():
        assert q.quant == nv.Quant.new(nv.QuantMode.MXFP4) and q.biases is None
        assert np.array_equal(q.weight.to_numpy(), mlx[prefix + ".weight"]), prefix
        assert np.array_equal(q.scales.to_numpy(), mlx[prefix + ".scales"]), prefix
        assert np.array_equal(rest[prefix + ".bias"].to_numpy(), mlx[prefix + ".bias"]), prefix
    # one expert's product through the loaded weight
    prefix = sorted(layers)[0]
    q = layers[prefix]
    rng = np.random.default_rng(0)
    K = q.weight.shape[-1] * 8
    x = oracle.from_f32(rng.standard_normal((3, K)).astype(np.float32), oracle.BF16)
    one = nv.Quantized(q.weight[2], q.scales[2], None, q.quant)
    got = nv.quantized_matmul(dev.array(x, nv.BF16), one).to_numpy()
    want = oracle.quantized_matmul(x, mlx[prefix + ".weight"][2], mlx[prefix + ".scales"][2], None, oracle.BF16, oracle.MXFP4, 32, 4)
    assert np.array_equal(got, want)
    # an MLX file loads as it is
    layers2, _ = ck.load_quantized(dev, GOLDEN / "checkpoint_gpt_oss_mlx.safetensors")
    for prefix, q in layers2.items():
        assert np.array_equal(q.weight.to_numpy(), mlx[prefix + ".weight"])


@pytest.mark.gpu
def test_awq_and_gptq_files_load_and_multiply(tmp_path):
    from nuvec_b200 import checkpoint as ck
    nv, dev = _dev()
    rng = np.random.default_rng(5)
    for method, cfg, code, bits, group in (("awq", {"quant_method": "awq", "bits": 4, "group_size": 64, "version": "gemm"}, ock.AWQ, 4, 64),
                                           ("gptq", {"quant_method": "gptq", "bits": 8, "group_size": 32, "checkpoint_format": "gptq_v2"}, ock.GPTQ_V2, 8, 32)):
        inputs, outputs, per_word = 128, 64, 32 // bits
        shape = (inputs, outputs // per_word) if code == ock.AWQ else (inputs // per_word, outputs)
        qweight = rng.integers(0, 2 ** 32, shape, dtype=np.uint32).view(np.int32)
        qzeros = rng.integers(0, 2 ** 32, (inputs // group, outputs // per_word), dtype=np.uint32).view(np.int32)
        scales = rng.uniform(0.001, 0.01, (inputs // group, outputs)).astype(np.float16)
        tensors = {"m.l.qweight": ("I32", qweight), "m.l.qzeros": ("I32", qzeros), "m.l.scales": ("F16", scales),
                   "m.norm.weight": ("F32", rng.standard_normal((inputs,)).astype(np.float32))}
        if code != ock.AWQ:
            tensors["m.l.g_idx"] = ("I32", (np.arange(inputs) // group).astype(np.int32))
        write_safetensors(tmp_path / f"{method}.safetensors", tensors)
        layers, rest = ck.load_quantized(dev, tmp_path / f"{method}.safetensors", quantization_config=cfg)
        assert list(layers) == ["m.l"] and rest["m.norm.weight"].dtype == nv.F16        # other floats follow the scales' dtype
        want_codes, want_s, want_b = ock.convert_packed(qweight, qzeros, scales.view(np.uint16), oracle.F16, code, bits, group)
        q = layers["m.l"]
        assert np.array_equal(q.weight.to_numpy(), want_codes)
        assert np.array_equal(q.biases.to_numpy().view(np.uint16), want_b)
        x = rng.standard_normal((2, inputs)).astype(np.float16)
        got = nv.quantized_matmul(dev.array(x, nv.F16), q).to_numpy().view(np.uint16)
        want = oracle.quantized_matmul(x.view(np.uint16), want_codes, want_s, want_b, oracle.F16, oracle.AFFINE, group, bits)
        err = np.abs(oracle.to_f32(got, oracle.F16) - oracle.to_f32(want, oracle.F16))
        assert np.all(err <= 1e-2 * np.abs(oracle.to_f32(want, oracle.F16)).max(axis=1, keepdims=True))


@pytest.mark.gpu
def test_loader_prepares_the_scales_of_the_block_scaled_product(tmp_path):
    from nuvec_b200 import checkpoint as ck
    nv, dev = _dev()
    rng = np.random.default_rng(9)
    N, K = 256, 512
    w = oracle.from_f32((rng.standard_normal((N, K)) * 0.05).astype(np.float32), oracle.BF16)
    codes, scales, _ = oracle.quantize(w, oracle.BF16, oracle.NVFP4, 16, 4)
    write_safetensors(tmp_path / "m.safetensors", {"p.weight": ("U32", codes), "p.scales": ("U8", scales)})
    layers, _, prepared = ck.load_quantized(dev, tmp_path / "m.safetensors", prepare_qqmm=True)
    q = layers["p"]
    assert q.quant == nv.Quant.new(nv.QuantMode.NVFP4) and "p" in prepared
    x = dev.array(oracle.from_f32(rng.standard_normal((130, K)).astype(np.float32), oracle.BF16), nv.BF16)
    assert np.array_equal(nv.qqmm(x, q, prepared=prepared["p"]).to_numpy(), nv.qqmm(x, q).to_numpy())
