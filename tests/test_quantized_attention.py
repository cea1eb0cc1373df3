"""fast::quantized_attention (crates/nuvec-core/src/fast.rs:694-722): decode attention over a quantized KV cache.

The bound is the reference's own (crates/nuvec-core/tests/quantized.rs:1964-2031): against attention over the
dequantized cache in float32, |got - want| <= tol * max(1, max |want|) with tol 2e-5 (float32), 5e-3 (float16),
3e-2 (bfloat16), over its grid of head sizes, bits, group sizes, head counts, lengths, sinks and cache views.
Golden records: mlx-lm's outputs from the reference's fixture (tests/golden/kv_quant_attention_l1.safetensors).
"""
from pathlib import Path

import numpy as np
import pytest

import oracle
from oracle import attention as oat
from oracle import checkpoint as ock

GOLDEN = Path(__file__).resolve().parent / "golden" / "kv_quant_attention_l1.safetensors"
TOL = {oracle.F32: 2e-5, oracle.F16: 5e-3, oracle.BF16: 3e-2}
DT = {"f32": oracle.F32, "f16": oracle.F16, "bf16": oracle.BF16}


def close(got, want, tol, name):
    scale = max(1.0, float(np.abs(want).max()) if want.size else 1.0)
    err = np.abs(np.asarray(got, np.float64) - want)
    assert err.max(initial=0.0) <= tol * scale, f"{name}: {err.max()} over {tol * scale}"


def make_cache(rng, B, Hkv, cap, D, dtype, gs, bits):
    w = oracle.from_f32(rng.standard_normal((B * Hkv * cap, D)).astype(np.float32), dtype)
    codes, scales, biases = oracle.quantize(w, dtype, oracle.AFFINE, gs, bits)
    return tuple(a.reshape(B, Hkv, cap, -1) for a in (codes, scales, biases))


def golden_cases():
    t = ock.read_safetensors(GOLDEN)
    for dt in ("f32", "bf16"):
        for bits in (8, 4):
            tag = f"{dt}_b{bits}_l1_"
            get = lambda k: t[tag + k][1]
            yield tag, DT[dt], bits, get("q"), (get("k0"), get("k1"), get("k2")), (get("v0"), get("v1"), get("v2")), get("out")


# ── the oracle against the reference's records and its own yardstick (CPU) ───────────────────
def test_oracle_against_the_records_of_mlx_lm():
    for tag, dtype, bits, q, k, v, out in golden_cases():
        want = oracle.to_f32(out, dtype).astype(np.float64)
        # (the reference allows 1e-2 for its composition off the recorded GPU, 1e-5 / 2e-2 for its kernel)
        tol = 1e-5 if dtype == oracle.F32 else 2e-2
        got = oracle.to_f32(oat.composed(q, k, v, dtype, 32, bits, 0.125), dtype)
        assert np.abs(got - want).max() < tol, tag
        assert np.abs(oat.dense(q, k, v, dtype, 32, bits, 0.125) - want).max() < tol, tag


@pytest.mark.parametrize("dt", ["f32", "f16", "bf16"])
def test_composition_is_within_the_bound_of_the_dense_attention(dt):
    dtype = DT[dt]
    rng = np.random.default_rng(3)
    for D, bits, gs, Hq, Hkv, S, sinks in ((128, 4, 64, 8, 2, 37, True), (64, 8, 32, 4, 1, 50, False), (128, 3, 128, 4, 4, 21, True)):
        k, v = make_cache(rng, 1, Hkv, S, D, dtype, gs, bits), make_cache(rng, 1, Hkv, S, D, dtype, gs, bits)
        q = oracle.from_f32(rng.standard_normal((1, Hq, 1, D)).astype(np.float32), dtype)
        sink = oracle.from_f32(rng.standard_normal(Hq).astype(np.float32), dtype) if sinks else None
        scale = 1.0 / np.sqrt(D)
        want = oat.dense(q, k, v, dtype, gs, bits, scale, sink)
        close(oracle.to_f32(oat.composed(q, k, v, dtype, gs, bits, scale, sink), dtype), want, TOL[dtype], f"{dt} d{D} b{bits}")


# ── the device kernel (GPU) ──────────────────────────────────────────────────────────────────
def _upload(nv, dev, arrays, dtype):
    code = {oracle.F32: nv.F32, oracle.F16: nv.F16, oracle.BF16: nv.BF16}[dtype]
    out = []
    for a in arrays:
        if a.dtype == np.uint32:
            out.append(dev.array(a, nv.U32))
        else:
            out.append(dev.array(a.view(np.float16) if dtype == oracle.F16 else a, code))
    return out


def _run(nv, dev, q, k, v, dtype, gs, bits, scale, sinks, length):
    code = {oracle.F32: nv.F32, oracle.F16: nv.F16, oracle.BF16: nv.BF16}[dtype]
    quant = nv.Quant.affine(gs, bits)
    kq = nv.Quantized(*_upload(nv, dev, k, dtype), quant)
    vq = nv.Quantized(*_upload(nv, dev, v, dtype), quant)
    (qd,) = _upload(nv, dev, [q], dtype)
    sd = _upload(nv, dev, [sinks], dtype)[0] if sinks is not None else None
    out = nv.quantized_attention(qd, kq, vq, scale, sd, length=length).to_numpy()
    return oracle.to_f32(out.view(np.uint16) if dtype == oracle.F16 else out, dtype)


@pytest.mark.gpu
def test_kernel_against_the_records_of_mlx_lm():
    import nuvec_b200 as nv
    dev = nv.Device.shared(0)
    for tag, dtype, bits, q, k, v, out in golden_cases():
        got = _run(nv, dev, q, k, v, dtype, 32, bits, 0.125, None, None)
        tol = 1e-5 if dtype == oracle.F32 else 2e-2          # the reference's bounds for its kernel against these records
        assert np.abs(got - oracle.to_f32(out, dtype)).max() < tol, tag


@pytest.mark.gpu
@pytest.mark.parametrize("dt", ["f32", "f16", "bf16"])
@pytest.mark.parametrize("D,bits,gs", [(128, 8, 64), (128, 4, 64), (64, 8, 32), (128, 4, 128), (64, 4, 64), (128, 3, 64), (64, 3, 32),
                                       (128, 3, 128)])
def test_kernel_equals_the_dequantized_attention(dt, D, bits, gs):
    import nuvec_b200 as nv
    dev = nv.Device.shared(0)
    dtype = DT[dt]
    rng = np.random.default_rng(17 + D + bits + gs)
    for Hq, Hkv, S, sinks in ((4, 1, 1, False), (8, 2, 37, True), (32, 8, 300, False), (4, 4, 2100, True), (16, 2, 9000, True),
                              (8, 1, 777, False), (2, 2, 128, False), (8, 1, 129, True), (4, 2, 130, True), (16, 8, 257, False)):
        cap = S + 50
        k, v = make_cache(rng, 1, Hkv, cap, D, dtype, gs, bits), make_cache(rng, 1, Hkv, cap, D, dtype, gs, bits)
        q = oracle.from_f32(rng.standard_normal((1, Hq, 1, D)).astype(np.float32), dtype)
        sink = oracle.from_f32(rng.standard_normal(Hq).astype(np.float32), dtype) if sinks else None
        scale = 1.0 / np.sqrt(D)
        got = _run(nv, dev, q, k, v, dtype, gs, bits, scale, sink, S)
        cut = lambda t: tuple(np.ascontiguousarray(a[:, :, :S]) for a in t)
        want = oat.dense(q, cut(k), cut(v), dtype, gs, bits, scale, sink)
        close(got, want, TOL[dtype], f"{dt} d{D} b{bits} gs{gs} hq{Hq} hkv{Hkv} s{S} sinks {sinks}")


@pytest.mark.gpu
def test_batches_empty_caches_and_refusals():
    import nuvec_b200 as nv
    dev = nv.Device.shared(0)
    rng = np.random.default_rng(5)
    dtype, D, gs, bits = oracle.BF16, 128, 64, 4
    k, v = make_cache(rng, 3, 2, 70, D, dtype, gs, bits), make_cache(rng, 3, 2, 70, D, dtype, gs, bits)
    q = oracle.from_f32(rng.standard_normal((3, 8, 1, D)).astype(np.float32), dtype)
    got = _run(nv, dev, q, k, v, dtype, gs, bits, 0.1, None, None)
    close(got, oat.dense(q, k, v, dtype, gs, bits, 0.1), TOL[dtype], "batch of 3")
    sink = oracle.from_f32(rng.standard_normal(8).astype(np.float32), dtype)
    assert not _run(nv, dev, q, k, v, dtype, gs, bits, 0.1, sink, 0).any()          # no keys: zeros
    quant = nv.Quant.affine(gs, bits)
    kq, vq = nv.Quantized(*_upload(nv, dev, k, dtype), quant), nv.Quantized(*_upload(nv, dev, v, dtype), quant)
    (qd,) = _upload(nv, dev, [q], dtype)
    with pytest.raises(nv.InvalidArgument, match="one affine quantization"):
        nv.quantized_attention(qd, kq, nv.Quantized(vq.weight, vq.scales, vq.biases, nv.Quant.affine(gs, 8)), 0.1)
    # several query rows per head, no mask: every row over all the keys (the reference's (8, 2, 37, 3) case and a longer one)
    for Hq, Hkv, S, L in ((8, 2, 37, 3), (4, 4, 700, 5)):
        k2, v2 = make_cache(rng, 2, Hkv, S, D, dtype, gs, bits), make_cache(rng, 2, Hkv, S, D, dtype, gs, bits)
        q2 = oracle.from_f32(rng.standard_normal((2, Hq, L, D)).astype(np.float32), dtype)
        got2 = _run(nv, dev, q2, k2, v2, dtype, gs, bits, 0.1, None, None)
        close(got2, oat.dense(q2, k2, v2, dtype, gs, bits, 0.1), TOL[dtype], f"{L} query rows")
    # causal: row l at position S - L + l (a prefill of L tokens over a cache that already holds their keys)
    for Hq, Hkv, S, L, sinks in ((8, 2, 37, 6, False), (4, 1, 300, 4, True), (4, 4, 3, 5, False)):
        k2, v2 = make_cache(rng, 1, Hkv, S, D, dtype, gs, bits), make_cache(rng, 1, Hkv, S, D, dtype, gs, bits)
        q2 = oracle.from_f32(rng.standard_normal((1, Hq, L, D)).astype(np.float32), dtype)
        sk = oracle.from_f32(rng.standard_normal(Hq).astype(np.float32), dtype) if sinks else None
        quant2 = nv.Quant.affine(gs, bits)
        kq2, vq2 = nv.Quantized(*_upload(nv, dev, k2, dtype), quant2), nv.Quantized(*_upload(nv, dev, v2, dtype), quant2)
        sd = _upload(nv, dev, [sk], dtype)[0] if sinks else None
        got2 = oracle.to_f32(nv.quantized_attention(_upload(nv, dev, [q2], dtype)[0], kq2, vq2, 0.1, sd, causal=True).to_numpy(), dtype)
        want2 = oat.dense(q2, k2, v2, dtype, gs, bits, 0.1, sk, causal=True)
        want2 = np.nan_to_num(want2)          # rows before the first key (S < L) attend to nothing: zeros
        close(got2, want2, TOL[dtype], f"causal S{S} L{L}")
    with pytest.raises(nv.UnsupportedError, match="query rows"):
        nv.quantized_attention(dev.array(np.zeros((3, 8, 65, D), np.uint16), nv.BF16), kq, vq, 0.1)
    with pytest.raises(nv.InvalidArgument, match="sinks"):
        nv.quantized_attention(qd, kq, vq, 0.1, dev.array(np.zeros(4, np.uint16), nv.BF16))
    k6 = make_cache(rng, 1, 1, 8, D, dtype, gs, 6)
    q1 = _upload(nv, dev, [q[:1, :1]], dtype)[0]
    six = nv.Quantized(*_upload(nv, dev, k6, dtype), nv.Quant.affine(gs, 6))
    with pytest.raises(nv.UnsupportedError):
        nv.quantized_attention(q1, six, six, 0.1)


@pytest.mark.gpu
def test_attention_inside_a_recorded_step():
    # the splits' partial results live in the handle's scratch block, so a call whose shape ran once before can be
    # recorded with the rest of a decode step and replayed
    import ctypes as C
    import nuvec_b200 as nv
    from nuvec_b200 import _ffi
    dev = nv.Device.shared(0)
    rng = np.random.default_rng(11)
    dtype, D, gs, bits, Hq, Hkv, S = oracle.BF16, 128, 64, 4, 8, 2, 900
    k, v = make_cache(rng, 1, Hkv, S, D, dtype, gs, bits), make_cache(rng, 1, Hkv, S, D, dtype, gs, bits)
    q = oracle.from_f32(rng.standard_normal((1, Hq, 1, D)).astype(np.float32), dtype)
    quant = nv.Quant.affine(gs, bits)
    kq, vq = nv.Quantized(*_upload(nv, dev, k, dtype), quant), nv.Quantized(*_upload(nv, dev, v, dtype), quant)
    (qd,) = _upload(nv, dev, [q], dtype)
    direct = nv.quantized_attention(qd, kq, vq, 0.1).to_numpy()
    out = dev.empty((1, Hq, 1, D), nv.BF16)
    c = quant._c()

    def call():
        assert _ffi.lib().nvc_quantized_attention(dev._h, C.byref(c), nv.BF16, qd.ptr, kq.weight.ptr, kq.scales.ptr, kq.biases.ptr,
                                                  vq.weight.ptr, vq.scales.ptr, vq.biases.ptr, None, 1, Hq, Hkv, 1, S, D, S, 0.1, 0,
                                                  out.ptr) == 0, _ffi.last_error()
    graph = dev.record(call)
    for _ in range(2):
        graph.launch()
    dev.synchronize()
    assert np.array_equal(out.to_numpy(), direct)
