"""Known-answer tests of the oracle's codecs.

The expected values are the reference's own tables (crates/nuvec-core/src/fp8.rs:135-233,
recorded from MLX 0.32.4) and the documented rules of the reference's bit packing and
`sorted_offsets` (crates/nuvec-core/src/kernels.rs:749-756, 875-892).
"""
import math

import numpy as np
import pytest

import oracle

L = oracle.lib()


def test_e4m3_encode_probes():
    values = [0.1, 1.0, 448.0, 500.0, -3.3, 1e-4, 0.0, -0.0, math.inf, -math.inf, math.nan,
              2.0 ** -9, 2.0 ** -10, 0.0029296875, 464.0, 465.0, 1.0625, 1.1875]
    expected = [29, 56, 126, 126, 197, 0, 0, 128, 126, 254, 126, 1, 0, 2, 126, 126, 56, 58]
    assert [L.orc_e4m3_from_f32(v) for v in values] == expected


def test_e4m3_decode_and_round_trip():
    for code, value in [(0, 0.0), (1, 0.001953125), (7, 0.013671875), (8, 0.015625), (56, 1.0),
                        (126, 448.0), (128, -0.0), (254, -448.0)]:
        v = L.orc_e4m3_to_f32(code)
        assert v == value and math.copysign(1, v) == math.copysign(1, value)
    assert math.isnan(L.orc_e4m3_to_f32(0x7F)) and math.isnan(L.orc_e4m3_to_f32(0xFF))
    for code in range(256):
        if code & 0x7F != 0x7F:
            assert L.orc_e4m3_from_f32(L.orc_e4m3_to_f32(code)) == code


def test_e2m1_round_trips_and_ties():
    values = [0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0]
    for code, v in enumerate(values):
        assert L.orc_e2m1_to_f32(code) == v
        assert L.orc_e2m1_to_f32(code | 8) == -v
    for code in range(16):
        assert L.orc_e2m1_from_f32(L.orc_e2m1_to_f32(code)) == code
    for x, code in [(0.25, 0), (0.75, 2), (1.25, 2), (1.75, 4), (2.5, 4), (3.5, 6), (5.0, 6), (7.0, 7)]:
        assert L.orc_e2m1_from_f32(x) == code
    assert L.orc_e2m1_from_f32(-0.0) == 0x8
    assert L.orc_e2m1_from_f32(math.nan) == 0x7


def test_e8m0_rounds_and_clamps():
    assert L.orc_e8m0_from_f32(1.0) == 127
    assert L.orc_e8m0_from_f32(0.25) == 125
    assert L.orc_e8m0_from_f32(0.0) == 0
    assert L.orc_e8m0_from_f32(-1.0) == 0
    assert L.orc_e8m0_from_f32(math.inf) == 0xFF
    assert L.orc_e8m0_from_f32(math.nan) == 0xFF
    tiny = float(np.array([0x400000], np.uint32).view(np.float32)[0])
    assert L.orc_e8m0_to_f32(0) == tiny
    assert L.orc_e8m0_to_f32(0xFF) == math.inf
    assert L.orc_mx_scale_round_up(1.0 / 6.0) == 0.25
    assert L.orc_mx_scale_round_up(0.0) == tiny
    assert L.orc_mx_scale_round_up(0.5) == 0.5


def test_bf16_rounding_is_nearest_even():
    rng = np.random.default_rng(0)
    x = rng.standard_normal(4096).astype(np.float32)
    got = oracle.from_f32(x, oracle.BF16)
    ref = np.array([L.orc_f32_to_bf16(float(v)) for v in x], np.uint16)
    assert np.array_equal(got, ref)
    # ties: 1 + 2^-8 is halfway between 1 and 1 + 2^-7 -> even (1.0); 1 + 3*2^-8 -> 1 + 2^-6
    assert L.orc_f32_to_bf16(1.0 + 2.0 ** -8) == 0x3F80
    assert L.orc_f32_to_bf16(1.0 + 3 * 2.0 ** -8) == 0x3F82


def test_f16_single_rounding_from_double():
    assert L.orc_f64_to_f16(65504.0) == 0x7BFF
    assert L.orc_f64_to_f16(65520.0) == 0x7C00
    assert L.orc_f64_to_f16(2.0 ** -24) == 0x0001
    assert L.orc_f64_to_f16(2.0 ** -25) == 0x0000          # tie to even
    assert L.orc_f64_to_f16(2.0 ** -25 * 1.0000001) == 0x0001
    x = np.random.default_rng(1).standard_normal(2048) * 100
    ref = x.astype(np.float16).view(np.uint16)
    got = np.array([L.orc_f64_to_f16(float(v)) for v in x], np.uint16)
    assert np.array_equal(got, ref)


@pytest.mark.parametrize("bits", [1, 2, 3, 4, 5, 6, 8])
def test_packing_is_a_little_endian_bit_stream(bits):
    # Quantize a ramp whose codes are known: with lo=0, hi=2^bits-1 the codes are the values.
    n = (1 << bits) - 1
    gs = 32
    row = (np.arange(gs) % (n + 1)).astype(np.float32)
    row[0], row[-1] = 0.0, float(n)
    w = np.tile(row, (2, 2))
    codes, scales, biases = oracle.quantize(w, oracle.F32, oracle.AFFINE, gs, bits)
    stream = np.unpackbits(codes.view(np.uint8).reshape(2, -1), axis=1, bitorder="little")
    vals = stream.reshape(2, -1, bits) @ (1 << np.arange(bits))
    deq = oracle.dequantize(codes, scales, biases, oracle.F32, oracle.AFFINE, gs, bits)
    # codes decode back to the ramp (scale may be negative: bias is the larger-magnitude edge)
    assert np.allclose(deq, w, atol=1e-5)
    s, b = scales.repeat(gs, axis=1), biases.repeat(gs, axis=1)
    assert np.allclose(vals * s + b, w, atol=1e-5)


def test_sorted_offsets_is_a_partition_point():
    idx = np.array([0, 0, 2, 2, 2, 5, 7, 7], np.uint32)
    assert oracle.sorted_offsets(idx, 9).tolist() == [0, 2, 2, 5, 5, 5, 6, 6, 8]
    assert oracle.sorted_offsets(np.zeros(0, np.uint32), 3).tolist() == [0, 0, 0]


def test_invalid_quant_is_rejected():
    w = np.zeros((2, 64), np.float32)
    with pytest.raises(oracle.OracleError):
        oracle.quantize(w, oracle.F32, oracle.AFFINE, 48, 4)
    with pytest.raises(oracle.OracleError):
        oracle.quantize(w, oracle.F32, oracle.AFFINE, 64, 7)
    with pytest.raises(oracle.OracleError):
        oracle.quantize(w, oracle.F32, oracle.MXFP4, 64, 4)
    with pytest.raises(oracle.OracleError):
        oracle.quantize(w, oracle.F32, oracle.NVFP4, 16, 8)


def test_few_row_products_do_not_depend_on_the_row_count():
    # few_rows.rs:1-10: a row of an M-row product has the bits of the same row alone.
    rng = np.random.default_rng(3)
    w = oracle.from_f32(rng.standard_normal((40, 256)).astype(np.float32) * 0.02, oracle.BF16)
    codes, scales, biases = oracle.quantize(w, oracle.BF16, oracle.AFFINE, 64, 4)
    x = oracle.from_f32(rng.standard_normal((16, 256)).astype(np.float32), oracle.BF16)
    full = oracle.quantized_matmul(x, codes, scales, biases, oracle.BF16)
    for m in (1, 5, 16):
        part = oracle.quantized_matmul(x[:m], codes, scales, biases, oracle.BF16)
        assert np.array_equal(part, full[:m])


@pytest.mark.parametrize("nan_bits", [0x7FC00000, 0x7F800001, 0xFF800001, 0xFFC00000])
def test_a_nan_of_either_kind_is_ignored_by_the_group_extremes(nan_bits):
    # kernels.rs:935 (and :785-790 for affine) fold with f32::max / f32::min, which return the other
    # operand for a NaN, quiet or signalling; the C library's fmaxf does not for a signalling one.
    w = np.linspace(-1.0, 3.0, 64, dtype=np.float32).reshape(1, 64)
    poisoned = w.copy()
    poisoned.view(np.uint32)[0, 5] = nan_bits
    for mode, gs, bits in ((oracle.MXFP4, 32, 4), (oracle.NVFP4, 16, 4), (oracle.MXFP8, 32, 8)):
        _, s0, _ = oracle.quantize(w, oracle.F32, mode, gs, bits)
        _, s1, _ = oracle.quantize(poisoned, oracle.F32, mode, gs, bits)
        assert np.array_equal(s0, s1)
    clean = w.copy()
    clean[0, 5] = clean[0, 6]                                # an interior value: the extremes stay
    _, s0, b0 = oracle.quantize(clean, oracle.F32, oracle.AFFINE, 64, 4)
    _, s1, b1 = oracle.quantize(poisoned, oracle.F32, oracle.AFFINE, 64, 4)
    assert np.array_equal(s0.view(np.uint8), s1.view(np.uint8)) and np.array_equal(b0.view(np.uint8), b1.view(np.uint8))
