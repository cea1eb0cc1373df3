"""CUDA path vs the CPU oracle on seeded inputs (bit-exact where the path is integer/byte or
rounding-specified; within 1e-2 * ||row||_inf for products, the bound the task states)."""
import numpy as np
import pytest

import oracle

pytestmark = pytest.mark.gpu

DT = {"bf16": oracle.BF16, "f16": oracle.F16, "f32": oracle.F32}


@pytest.fixture(scope="module")
def be():
    from cuda_backend import CudaBackend
    return CudaBackend()


def rand(rng, shape, dtype, scale=1.0):
    return oracle.from_f32((rng.standard_normal(shape) * scale).astype(np.float32), dtype)


def assert_product_close(got, want, dtype, what=""):
    g, w = oracle.to_f32(got, dtype).astype(np.float64), oracle.to_f32(want, dtype).astype(np.float64)
    assert g.shape == w.shape
    g2, w2 = g.reshape(-1, g.shape[-1]), w.reshape(-1, w.shape[-1])
    bound = 1e-2 * np.abs(w2).max(axis=1, keepdims=True)   # 1e-2 * ||row||_inf
    err = np.abs(g2 - w2)
    assert np.all(err <= bound + 1e-30), f"{what}: max err {err.max():.4g}, worst ratio {(err / (bound + 1e-30)).max():.3f}"


def assert_product_tight(got, want, dtype, what=""):
    """For kernels whose operands equal the oracle's dequantized weights bit for bit: only the
    float32 summation order differs, so results agree to one rounding of the output dtype."""
    g, w = oracle.to_f32(got, dtype).astype(np.float64), oracle.to_f32(want, dtype).astype(np.float64)
    ulp = {oracle.BF16: 2.0 ** -7, oracle.F16: 2.0 ** -10, oracle.F32: 2.0 ** -22}[dtype]
    rowmax = np.abs(w).reshape(-1, w.shape[-1]).max(axis=1, keepdims=True).reshape(w.shape[:-1] + (1,))
    lim = ulp * np.abs(w) + 2e-5 * rowmax
    err = np.abs(g - w)
    assert np.all(err <= lim), f"{what}: max err {err.max():.4g}, worst ratio {(err / lim).max():.3f}"


AFFINE = [(b, g) for b in (1, 2, 3, 4, 5, 6, 8) for g in (32, 64, 128)]


@pytest.mark.parametrize("bits,gs", AFFINE)
@pytest.mark.parametrize("dt", ["bf16", "f16", "f32"])
def test_quantize_dequantize_bit_exact(be, bits, gs, dt):
    dtype = DT[dt]
    rng = np.random.default_rng(bits * 1000 + gs)
    w = rand(rng, (37, 4 * gs), dtype, 0.02)
    c0, s0, b0 = oracle.quantize(w, dtype, oracle.AFFINE, gs, bits)
    c1, s1, b1 = be.quantize(w, dtype, oracle.AFFINE, gs, bits)
    assert np.array_equal(c0, c1) and np.array_equal(s0, s1) and np.array_equal(b0, b1)
    for fused in (False, True):
        d0 = oracle.dequantize(c0, s0, b0, dtype, oracle.AFFINE, gs, bits, fused=fused)
        d1 = be.dequantize(c0, s0, b0, dtype, oracle.AFFINE, gs, bits, fused=fused)
        assert np.array_equal(d0, d1), f"fused={fused}"


@pytest.mark.parametrize("mode,gs,bits", [(oracle.MXFP4, 32, 4), (oracle.MXFP8, 32, 8), (oracle.NVFP4, 16, 4)])
@pytest.mark.parametrize("dt", ["bf16", "f16", "f32"])
def test_fp_quantize_dequantize_bit_exact(be, mode, gs, bits, dt):
    dtype = DT[dt]
    rng = np.random.default_rng(mode * 10 + dtype)
    w = rand(rng, (19, 8 * gs), dtype, 0.5)
    w.reshape(-1)[:5] = oracle.from_f32(np.array([0.0, -0.0, 1e-30, 7.0, -448.0], np.float32), dtype)
    for g in ([None] if mode != oracle.NVFP4 else [None, 3.5]):
        c0, s0, _ = oracle.quantize(w, dtype, mode, gs, bits, g)
        c1, s1, _ = be.quantize(w, dtype, mode, gs, bits, g)
        assert np.array_equal(c0, c1) and np.array_equal(s0, s1), f"global={g}"
        for out in (oracle.BF16, oracle.F16, oracle.F32):
            d0 = oracle.dequantize(c0, s0, None, out, mode, gs, bits, g)
            d1 = be.dequantize(c0, s0, None, out, mode, gs, bits, g)
            assert np.array_equal(d0.view(np.uint8), d1.view(np.uint8)), f"global={g} out={out}"


@pytest.mark.parametrize("mode,gs", [(oracle.MXFP4, 32), (oracle.NVFP4, 16)])
def test_fp4_quantize_every_bfloat16_pattern(be, mode, gs):
    # The 4-bit codes come from the hardware's conversion instruction: every bfloat16 bit pattern
    # (NaNs, infinities, both zeros, subnormals, every tie of the E2M1 grid) goes through it under
    # several group scales and must give the oracle's code.  The first value of a group fixes the
    # scale (6 * 2^k decodes to exactly 2^k), the others sweep the patterns.
    patterns = np.arange(65536, dtype=np.uint32).astype(np.uint16)
    per = gs - 1
    pad = (-len(patterns)) % per
    sweep = np.concatenate([patterns, np.zeros(pad, np.uint16)]).reshape(-1, per)
    for k in (-3, 0, 5) if mode == oracle.NVFP4 else (-120, -3, 0, 40):
        lead = oracle.from_f32(np.full((len(sweep), 1), 6.0 * 2.0 ** k, np.float32), oracle.BF16)
        w = np.concatenate([lead.view(np.uint16).reshape(-1, 1), sweep], axis=1).view(lead.dtype)
        c0, s0, _ = oracle.quantize(w, oracle.BF16, mode, gs, 4)
        c1, s1, _ = be.quantize(w, oracle.BF16, mode, gs, 4)
        bad = np.nonzero(s0.reshape(-1) != s1.reshape(-1))[0]
        assert len(bad) == 0, f"scales, k={k}: group {bad[0]} oracle {s0.reshape(-1)[bad[0]]} device {s1.reshape(-1)[bad[0]]} values {[hex(v) for v in w[bad[0]]]}"
        bad = np.nonzero((c0.view(np.uint8).reshape(len(w), -1) != c1.view(np.uint8).reshape(len(w), -1)).any(axis=1))[0]
        assert len(bad) == 0, (f"codes, k={k}: group {bad[0]} oracle {c0.view(np.uint8).reshape(len(w), -1)[bad[0]]} "
                               f"device {c1.view(np.uint8).reshape(len(w), -1)[bad[0]]} values {[hex(v) for v in w[bad[0]]]}")


def test_dequantize_full_size_checksum(be):
    # The headline decode matrix (4096 x 4096, 4 bits, groups of 64): bit-exact at full size.
    rng = np.random.default_rng(0)
    w = rand(rng, (4096, 4096), oracle.BF16, 0.02)
    c, s, b = oracle.quantize(w, oracle.BF16, oracle.AFFINE, 64, 4)
    c1, s1, b1 = be.quantize(w, oracle.BF16, oracle.AFFINE, 64, 4)
    assert np.array_equal(c, c1) and np.array_equal(s, s1) and np.array_equal(b, b1)
    d0 = oracle.dequantize(c, s, b, oracle.BF16, oracle.AFFINE, 64, 4)
    d1 = be.dequantize(c, s, b, oracle.BF16, oracle.AFFINE, 64, 4)
    assert np.array_equal(d0, d1)


@pytest.mark.parametrize("bits,gs", AFFINE)
@pytest.mark.parametrize("M", [1, 3, 8])
def test_qmv_affine_bf16(be, bits, gs, M):
    rng = np.random.default_rng(bits * 100 + gs + M)
    N, K = 72, 1024
    w = rand(rng, (N, K), oracle.BF16, 0.02)
    c, s, b = oracle.quantize(w, oracle.BF16, oracle.AFFINE, gs, bits)
    x = rand(rng, (M, K), oracle.BF16)
    want = oracle.quantized_matmul(x, c, s, b, oracle.BF16, oracle.AFFINE, gs, bits)
    got = be.quantized_matmul(x, c, s, b, oracle.BF16, oracle.AFFINE, gs, bits, True)
    assert_product_close(got, want, oracle.BF16, f"b{bits} g{gs} M{M}")
    assert_product_tight(got, want, oracle.BF16, f"b{bits} g{gs} M{M}")


@pytest.mark.parametrize("N,K", [(4096, 4096), (6144, 4096), (4096, 12288), (512, 12288), (768, 2048), (2048, 768),
                                 (40, 2880), (17, 64), (4096, 128)])
@pytest.mark.parametrize("M", [1, 4, 8])
def test_qmv_shapes_b4_g64(be, N, K, M):
    rng = np.random.default_rng(N + K + M)
    w = rand(rng, (N, K), oracle.BF16, 0.02)
    c, s, b = oracle.quantize(w, oracle.BF16, oracle.AFFINE, 64, 4)
    x = rand(rng, (M, K), oracle.BF16)
    want = oracle.quantized_matmul(x, c, s, b, oracle.BF16)
    got = be.quantized_matmul(x, c, s, b, oracle.BF16, oracle.AFFINE, 64, 4, True)
    assert_product_close(got, want, oracle.BF16, f"N{N} K{K} M{M}")
    assert_product_tight(got, want, oracle.BF16, f"N{N} K{K} M{M}")


@pytest.mark.parametrize("bits,gs", [(4, 64), (2, 64), (3, 64), (6, 64), (8, 64), (3, 32), (6, 128)])
def test_qmv_one_hot_rows_return_the_dequantized_weights(be, bits, gs):
    # x = unit vectors: y[m, n] is exactly dequantize(w)[n, k_m] rounded to bf16 -- a
    # size-independent check that no k-slot is permuted or dropped in the fast kernel
    # (3- and 6-bit codes straddle words and come out of funnel shifts).
    rng = np.random.default_rng(5 + bits)
    N, K = 64, 512
    w = rand(rng, (N, K), oracle.BF16, 0.02)
    c, s, b = oracle.quantize(w, oracle.BF16, oracle.AFFINE, gs, bits)
    dense = oracle.to_f32(oracle.dequantize(c, s, b, oracle.BF16, oracle.AFFINE, gs, bits), oracle.BF16)
    ks = rng.permutation(K)[:64]
    for k0 in range(0, 64, 8):
        x = np.zeros((8, K), np.float32)
        for i in range(8):
            x[i, ks[k0 + i]] = 1.0
        got = oracle.to_f32(be.quantized_matmul(oracle.from_f32(x, oracle.BF16), c, s, b, oracle.BF16,
                                                oracle.AFFINE, gs, bits, True), oracle.BF16)
        want = dense[:, ks[k0:k0 + 8]].T
        assert np.array_equal(got, want)


@pytest.mark.parametrize("dt", ["f16", "f32"])
@pytest.mark.parametrize("transpose", [True, False])
def test_generic_product_other_dtypes(be, dt, transpose):
    dtype = DT[dt]
    rng = np.random.default_rng(11)
    N, K, M = 96, 256, 5
    w = rand(rng, (N, K) if transpose else (K, N), dtype, 0.05)
    c, s, b = oracle.quantize(w, dtype, oracle.AFFINE, 32, 6)
    x = rand(rng, (M, K), dtype)
    want = oracle.quantized_matmul(x, c, s, b, dtype, oracle.AFFINE, 32, 6, transpose)
    got = be.quantized_matmul(x, c, s, b, dtype, oracle.AFFINE, 32, 6, transpose)
    assert_product_close(got, want, dtype)


@pytest.mark.parametrize("mode,gs", [(oracle.MXFP4, 32), (oracle.NVFP4, 16)])
@pytest.mark.parametrize("M", [1, 4])
def test_fp_product(be, mode, gs, M):
    rng = np.random.default_rng(mode + M)
    N, K = 80, 2880
    w = rand(rng, (N, K), oracle.BF16, 0.02)
    c, s, _ = oracle.quantize(w, oracle.BF16, mode, gs, 4)
    x = rand(rng, (M, K), oracle.BF16)
    want = oracle.quantized_matmul(x, c, s, None, oracle.BF16, mode, gs, 4)
    got = be.quantized_matmul(x, c, s, None, oracle.BF16, mode, gs, 4, True)
    assert_product_close(got, want, oracle.BF16)


@pytest.mark.parametrize("mode,gs", [(oracle.MXFP4, 32), (oracle.NVFP4, 16)])
@pytest.mark.parametrize("N,K", [(80, 2880), (256, 4096), (48, 512)])
def test_fp_few_rows_tight_and_unit_rows_bit_for_bit(be, mode, gs, N, K):
    # the few-row kernel decodes E2M1 x scale exactly: products agree to one output rounding and
    # unit-vector rows return the oracle's float32 decode (rounded to bfloat16) bit for bit
    rng = np.random.default_rng(mode + N)
    w = rand(rng, (N, K), oracle.BF16, 0.02)
    w.reshape(-1)[:4] = oracle.from_f32(np.array([0.0, 0.011, -0.5, 3.0], np.float32), oracle.BF16)
    c, s, _ = oracle.quantize(w, oracle.BF16, mode, gs, 4)
    for M in (1, 5, 8):
        x = rand(rng, (M, K), oracle.BF16)
        want = oracle.quantized_matmul(x, c, s, None, oracle.BF16, mode, gs, 4)
        got = be.quantized_matmul(x, c, s, None, oracle.BF16, mode, gs, 4, True)
        assert_product_tight(got, want, oracle.BF16, f"M{M}")
    dense = oracle.to_f32(oracle.dequantize(c, s, None, oracle.F32, mode, gs, 4), oracle.F32)
    ks = rng.permutation(K)[:8]
    xu = np.zeros((8, K), np.float32)
    xu[np.arange(8), ks] = 1.0
    got = oracle.to_f32(be.quantized_matmul(oracle.from_f32(xu, oracle.BF16), c, s, None, oracle.BF16, mode, gs, 4, True), oracle.BF16)
    assert np.array_equal(got, dense[:, ks].T)


def test_sorted_offsets(be):
    import nuvec_b200 as nv
    rng = np.random.default_rng(2)
    idx = np.sort(rng.integers(0, 128, 4096)).astype(np.uint32)
    got = nv.sorted_offsets(be.up(idx, nv.U32), 128).to_numpy()
    assert np.array_equal(got, oracle.sorted_offsets(idx, 128))
    assert nv.sorted_offsets(be.up(np.zeros(0, np.uint32), nv.U32), 3).to_numpy().tolist() == [0, 0, 0]


@pytest.mark.parametrize("T,E,topk,N,K", [(1, 128, 8, 768, 2048), (1, 128, 8, 2048, 768), (6, 16, 4, 96, 256)])
def test_gather_rows_affine(be, T, E, topk, N, K):
    rng = np.random.default_rng(T + E)
    Ee = min(E, 16)  # keep the oracle's expert tensors small; ids are drawn from these
    w = rand(rng, (Ee, N, K), oracle.BF16, 0.02)
    c, s, b = oracle.quantize(w, oracle.BF16, oracle.AFFINE, 64, 4)
    ids = np.concatenate([rng.permutation(Ee)[:topk] for _ in range(T)]).astype(np.uint32)
    order = np.argsort(ids, kind="stable")
    rhs = ids[order]
    x = rand(rng, (T, K), oracle.BF16)
    rows = np.repeat(np.arange(T), topk)[order]
    xr = x[rows][:, None, :]
    want = oracle.gather_qmm(xr, c, s, b, np.arange(len(rhs)), rhs, oracle.BF16)
    got = be.gather_qmm(xr, c, s, b, None, rhs, oracle.BF16, oracle.AFFINE, 64, 4, True, None, True)
    assert_product_close(got, want, oracle.BF16)


def test_empty_operands_are_no_ops(be):
    import nuvec_b200 as nv
    rng = np.random.default_rng(0)
    w = rand(rng, (8, 64), oracle.BF16, 0.02)
    c, s, b = oracle.quantize(w, oracle.BF16, oracle.AFFINE, 64, 4)
    q = be.quantized(c, s, b, oracle.BF16, oracle.AFFINE, 64, 4)
    out = nv.quantized_matmul(be.dev.empty((0, 64), nv.BF16), q)
    assert out.shape == (0, 8)
    q0 = be.quantized(c[:0], s[:0], b[:0], oracle.BF16, oracle.AFFINE, 64, 4)
    out = nv.quantized_matmul(be.up(rand(rng, (3, 64), oracle.BF16), nv.BF16), q0)
    assert out.shape == (3, 0)


def test_invalid_arguments_raise(be):
    import nuvec_b200 as nv
    rng = np.random.default_rng(0)
    w = rand(rng, (8, 64), oracle.BF16, 0.02)
    c, s, b = oracle.quantize(w, oracle.BF16, oracle.AFFINE, 64, 4)
    x = be.up(rand(rng, (2, 64), oracle.BF16), nv.BF16)
    with pytest.raises(nv.InvalidArgument):
        nv.quantized_matmul(x, nv.Quantized(be.up(c, nv.U32), be.up(s, nv.BF16), None, nv.Quant.affine(64, 4)))
    with pytest.raises(nv.InvalidArgument):
        nv.quantized_matmul(x, be.quantized(c, s, b, oracle.BF16, oracle.AFFINE, 48, 4))
    with pytest.raises(nv.InvalidArgument):
        nv.quantized_matmul(be.up(rand(rng, (2, 32), oracle.BF16), nv.BF16), be.quantized(c, s, b, oracle.BF16, oracle.AFFINE, 64, 4))
    with pytest.raises(nv.InvalidArgument):
        nv.quantize(be.up(rand(rng, (8, 48), oracle.BF16), nv.BF16), nv.Quant.affine(64, 4))
    with pytest.raises(nv.InvalidArgument):
        nv.quantize(be.up(rand(rng, (8, 64), oracle.BF16), nv.BF16), nv.Quant(nv.QuantMode.MXFP4, 64, 4))


def test_pool_reuses_blocks_and_reports_stats(be):
    import nuvec_b200 as nv
    dev = be.dev
    dev.synchronize()
    before = dev.memory()
    a = dev.empty((1 << 20,), nv.F32)
    mid = dev.memory()
    assert mid["active"] >= before["active"] + (4 << 20)
    ptr = a.ptr.value
    del a
    after = dev.memory()
    assert after["active"] == before["active"] and after["cached"] >= 4 << 20
    b = dev.empty((1 << 20,), nv.F32)
    assert b.ptr.value == ptr and dev.memory()["allocations"] == mid["allocations"]


@pytest.mark.parametrize("bits,gs", [(3, 64), (6, 32)])
@pytest.mark.parametrize("M", [9, 20, 67])
def test_many_rows_of_3_and_6_bit_weights_go_eight_at_a_time(be, bits, gs, M):
    # no tensor-core decode for these widths: the few-row kernel takes the rows in blocks of eight
    rng = np.random.default_rng(bits + M)
    N, K = 200, 1024
    w = rand(rng, (N, K), oracle.BF16, 0.02)
    c, s, b = oracle.quantize(w, oracle.BF16, oracle.AFFINE, gs, bits)
    x = rand(rng, (M, K), oracle.BF16)
    want = oracle.quantized_matmul(x, c, s, b, oracle.BF16, oracle.AFFINE, gs, bits)
    got = be.quantized_matmul(x, c, s, b, oracle.BF16, oracle.AFFINE, gs, bits, True)
    assert_product_close(got, want, oracle.BF16)
    assert_product_tight(got, want, oracle.BF16)


# ── many-row products on the tensor-core kernel ────────────────────────────────────────────
@pytest.mark.parametrize("bits,gs", [(4, 64), (4, 32), (4, 128), (8, 64), (8, 32), (2, 64), (2, 128)])
@pytest.mark.parametrize("M,N,K", [(17, 128, 64), (64, 200, 256), (200, 384, 512), (300, 136, 2880 // 45 * 45)])
def test_qmm_affine_bf16(be, bits, gs, M, N, K):
    K = max(K // gs * gs, gs)
    if K % 64:
        K = (K // 64 + 1) * 64
    rng = np.random.default_rng(bits * 7 + gs + M)
    w = rand(rng, (N, K), oracle.BF16, 0.02)
    c, s, b = oracle.quantize(w, oracle.BF16, oracle.AFFINE, gs, bits)
    x = rand(rng, (M, K), oracle.BF16)
    want = oracle.quantized_matmul(x, c, s, b, oracle.BF16, oracle.AFFINE, gs, bits)
    got = be.quantized_matmul(x, c, s, b, oracle.BF16, oracle.AFFINE, gs, bits, True)
    assert_product_close(got, want, oracle.BF16, f"b{bits} g{gs} M{M} N{N} K{K}")
    assert_product_tight(got, want, oracle.BF16, f"b{bits} g{gs} M{M} N{N} K{K}")


@pytest.mark.parametrize("bits,gs", [(4, 64), (8, 64), (2, 64), (4, 32)])
def test_qmm_unit_rows_return_the_dequantized_weights_bit_for_bit(be, bits, gs):
    # x = 192 unit vectors: y[m, :] must equal column k_m of dequantize(w) exactly (products with
    # 1.0 and sums with zeros are exact), which pins the tensor-core operands to the oracle's
    # dequantized matrix bit for bit.
    rng = np.random.default_rng(bits)
    N, K, M = 256, 512, 192
    w = rand(rng, (N, K), oracle.BF16, 0.02)
    c, s, b = oracle.quantize(w, oracle.BF16, oracle.AFFINE, gs, bits)
    dense = oracle.dequantize(c, s, b, oracle.BF16, oracle.AFFINE, gs, bits)
    ks = rng.permutation(K)[:M]
    x = np.zeros((M, K), np.float32)
    x[np.arange(M), ks] = 1.0
    got = be.quantized_matmul(oracle.from_f32(x, oracle.BF16), c, s, b, oracle.BF16, oracle.AFFINE, gs, bits, True)
    assert np.array_equal(got, dense[:, ks].T)


@pytest.mark.parametrize("bits,gs,K", [(4, 64, 2048), (8, 64, 2048), (2, 64, 2048), (8, 32, 2880 // 64 * 64), (4, 128, 1920)])
def test_qmm_unit_rows_through_a_long_persistent_run(be, bits, gs, K):
    # More tiles than multiprocessors and many k-blocks per tile: every block of the persistent
    # kernel walks several tiles, the activation / weight / packed-slab rings wrap many times and
    # each dequantizer group meets slabs that hold none of its blocks.  Unit-vector rows make any
    # stale or overwritten stage visible as a bit difference, at a size no product oracle is needed for.
    rng = np.random.default_rng(bits + K)
    N, M = 2560, 1600
    w = rand(rng, (N, K), oracle.BF16, 0.02)
    c, s, b = oracle.quantize(w, oracle.BF16, oracle.AFFINE, gs, bits)
    dense = oracle.dequantize(c, s, b, oracle.BF16, oracle.AFFINE, gs, bits)
    ks = rng.integers(0, K, M)
    x = np.zeros((M, K), np.float32)
    x[np.arange(M), ks] = 1.0
    xb = oracle.from_f32(x, oracle.BF16)
    for _ in range(2):  # twice: the second launch starts on warm caches and different timing
        got = be.quantized_matmul(xb, c, s, b, oracle.BF16, oracle.AFFINE, gs, bits, True)
        assert np.array_equal(got, dense[:, ks].T)


@pytest.mark.parametrize("bits,M,N,K", [(4, 40, 256, 8192), (8, 12, 384, 4096), (2, 300, 128, 4096), (4, 8, 4096, 12288)])
def test_qmm_tiles_cut_along_k(be, bits, M, N, K):
    # Fewer tiles than multiprocessors: every tile is cut along K, the parts meet in scratch and
    # the block that arrives last adds them.  Random rows within the product bound; unit rows bit
    # for bit (a sum with a single non-zero part is exact whatever the cut).
    rng = np.random.default_rng(bits + M)
    w = rand(rng, (N, K), oracle.BF16, 0.02)
    c, s, b = oracle.quantize(w, oracle.BF16, oracle.AFFINE, 64, bits)
    x = rand(rng, (M, K), oracle.BF16)
    if M == 8:  # the few-row kernel refuses this shape (its activations do not fit shared memory)
        Ns = 256
        want = oracle.quantized_matmul(x, c[:Ns], s[:Ns], b[:Ns], oracle.BF16, oracle.AFFINE, 64, bits)
        got = be.quantized_matmul(x, c, s, b, oracle.BF16, oracle.AFFINE, 64, bits, True)[:, :Ns]
    else:
        want = oracle.quantized_matmul(x, c, s, b, oracle.BF16, oracle.AFFINE, 64, bits)
        got = be.quantized_matmul(x, c, s, b, oracle.BF16, oracle.AFFINE, 64, bits, True)
    assert_product_close(got, want, oracle.BF16)
    assert_product_tight(got, want, oracle.BF16)
    dense = oracle.dequantize(c, s, b, oracle.BF16, oracle.AFFINE, 64, bits)
    ks = rng.integers(0, K, M)
    xu = np.zeros((M, K), np.float32)
    xu[np.arange(M), ks] = 1.0
    for _ in range(2):
        got = be.quantized_matmul(oracle.from_f32(xu, oracle.BF16), c, s, b, oracle.BF16, oracle.AFFINE, 64, bits, True)
        assert np.array_equal(got, dense[:, ks].T)


@pytest.mark.parametrize("mode,gs", [(oracle.MXFP4, 32), (oracle.NVFP4, 16)])
@pytest.mark.parametrize("M,N,K", [(40, 128, 128), (130, 200, 2880)])
def test_qmm_fp4(be, mode, gs, M, N, K):
    rng = np.random.default_rng(mode + M)
    w = rand(rng, (N, K), oracle.BF16, 0.02)
    w.reshape(-1)[:4] = oracle.from_f32(np.array([0.0, 0.011, -0.5, 3.0], np.float32), oracle.BF16)
    c, s, _ = oracle.quantize(w, oracle.BF16, mode, gs, 4)
    x = rand(rng, (M, K), oracle.BF16)
    want = oracle.quantized_matmul(x, c, s, None, oracle.BF16, mode, gs, 4)
    got = be.quantized_matmul(x, c, s, None, oracle.BF16, mode, gs, 4, True)
    assert_product_tight(got, want, oracle.BF16)
    # unit rows: the operands are the oracle's float32 decode exactly
    dense = oracle.to_f32(oracle.dequantize(c, s, None, oracle.F32, mode, gs, 4), oracle.F32)
    ks = rng.permutation(K)[:64]
    xu = np.zeros((64, K), np.float32)
    xu[np.arange(64), ks] = 1.0
    got = oracle.to_f32(be.quantized_matmul(oracle.from_f32(xu, oracle.BF16), c, s, None, oracle.BF16, mode, gs, 4, True), oracle.BF16)
    assert np.array_equal(got, dense[:, ks].T)


@pytest.mark.parametrize("M", [1, 3, 8])
@pytest.mark.parametrize("N,K", [(72, 1024), (160, 2880), (33, 96)])
def test_qmv_mxfp8(be, M, N, K):
    # MXFP8 weights (E4M3 codes, E8M0 scale per 32) on the few-row kernel: within one output rounding of the
    # oracle, and unit rows return the oracle's float32 decode bit for bit
    rng = np.random.default_rng(M + N + K)
    w = rand(rng, (N, K), oracle.BF16, 0.02)
    w.reshape(-1)[:6] = oracle.from_f32(np.array([0.0, -0.0, 1e-4, -0.5, 3.0, 1e-7], np.float32), oracle.BF16)
    c, s, _ = oracle.quantize(w, oracle.BF16, oracle.MXFP8, 32, 8)
    x = rand(rng, (M, K), oracle.BF16)
    want = oracle.quantized_matmul(x, c, s, None, oracle.BF16, oracle.MXFP8, 32, 8)
    got = be.quantized_matmul(x, c, s, None, oracle.BF16, oracle.MXFP8, 32, 8, True)
    assert_product_tight(got, want, oracle.BF16, f"M{M} N{N} K{K}")
    dense = oracle.to_f32(oracle.dequantize(c, s, None, oracle.F32, oracle.MXFP8, 32, 8), oracle.F32)
    ks = rng.permutation(K)[:8]
    xu = np.zeros((8, K), np.float32)
    xu[np.arange(8), ks] = 1.0
    got = oracle.to_f32(be.quantized_matmul(oracle.from_f32(xu, oracle.BF16), c, s, None, oracle.BF16, oracle.MXFP8, 32, 8, True), oracle.BF16)
    assert np.array_equal(got, dense[:, ks].T)


@pytest.mark.parametrize("M,N,K", [(40, 128, 128), (130, 200, 2880), (300, 512, 1024)])
def test_qmm_mxfp8(be, M, N, K):
    # 9+ rows of MXFP8 weights on the tensor-core kernel: within one output rounding of the oracle; unit rows return the
    # oracle's float32 decode bit for bit
    rng = np.random.default_rng(M + N)
    w = rand(rng, (N, K), oracle.BF16, 0.02)
    w.reshape(-1)[:4] = oracle.from_f32(np.array([0.0, 1e-4, -0.5, 3.0], np.float32), oracle.BF16)
    c, s, _ = oracle.quantize(w, oracle.BF16, oracle.MXFP8, 32, 8)
    x = rand(rng, (M, K), oracle.BF16)
    want = oracle.quantized_matmul(x, c, s, None, oracle.BF16, oracle.MXFP8, 32, 8)
    got = be.quantized_matmul(x, c, s, None, oracle.BF16, oracle.MXFP8, 32, 8, True)
    assert_product_tight(got, want, oracle.BF16)
    dense = oracle.to_f32(oracle.dequantize(c, s, None, oracle.F32, oracle.MXFP8, 32, 8), oracle.F32)
    ks = rng.permutation(K)[:64]
    xu = np.zeros((64, K), np.float32)
    xu[np.arange(64), ks] = 1.0
    got = oracle.to_f32(be.quantized_matmul(oracle.from_f32(xu, oracle.BF16), c, s, None, oracle.BF16, oracle.MXFP8, 32, 8, True), oracle.BF16)
    assert np.array_equal(got, dense[:, ks].T)


def test_qmm_mxfp8_every_code(be):
    codes = np.array([v for v in range(256) if v & 0x7F != 0x7F], np.uint8)
    K = 256
    rows = np.resize(codes, (128, K))
    for r in range(128):
        rows[r] = np.roll(rows[r], 5 * r)
    c = np.ascontiguousarray(rows).view(np.uint32)
    s = np.random.default_rng(1).integers(110, 140, (128, K // 32), dtype=np.uint8)
    dense = oracle.to_f32(oracle.dequantize(c, s, None, oracle.F32, oracle.MXFP8, 32, 8), oracle.F32)
    xu = np.eye(K, dtype=np.float32)                       # 256 unit rows: the tensor-core kernel
    got = oracle.to_f32(be.quantized_matmul(oracle.from_f32(xu, oracle.BF16), c, s, None, oracle.BF16, oracle.MXFP8, 32, 8, True), oracle.BF16)
    assert np.array_equal(got, dense.T)


def test_qmv_mxfp8_every_code(be):
    # every E4M3 code the quantizer can write (all but the two NaN codes), subnormals included, under several
    # scales: the kernel's operand is the oracle's decode
    codes = np.array([v for v in range(256) if v & 0x7F != 0x7F], np.uint8)
    K = 256
    rows = np.resize(codes, (64, K))
    for r in range(64):
        rows[r] = np.roll(rows[r], 7 * r)
    c = np.ascontiguousarray(rows).view(np.uint32)
    rng = np.random.default_rng(0)
    s = rng.integers(110, 140, (64, K // 32), dtype=np.uint8)
    dense = oracle.to_f32(oracle.dequantize(c, s, None, oracle.F32, oracle.MXFP8, 32, 8), oracle.F32)
    for k0 in range(0, K, 8):
        xu = np.zeros((8, K), np.float32)
        xu[np.arange(8), np.arange(k0, k0 + 8)] = 1.0
        got = oracle.to_f32(be.quantized_matmul(oracle.from_f32(xu, oracle.BF16), c, s, None, oracle.BF16, oracle.MXFP8, 32, 8, True), oracle.BF16)
        assert np.array_equal(got, dense[:, k0:k0 + 8].T), k0


def moe_case(rng, T, E, topk, N, K, mode=oracle.AFFINE, gs=64, bits=4):
    w = rand(rng, (E, N, K), oracle.BF16, 0.02)
    c, s, b = oracle.quantize(w, oracle.BF16, mode, gs, bits)
    ids = np.concatenate([rng.permutation(E)[:topk] for _ in range(T)]).astype(np.uint32)
    order = np.argsort(ids, kind="stable")
    rhs = ids[order]
    x = rand(rng, (T, K), oracle.BF16)
    xr = x[np.repeat(np.arange(T), topk)[order]][:, None, :]
    return c, s, b, rhs, np.ascontiguousarray(xr)


@pytest.mark.parametrize("T,E,topk,N,K", [(64, 16, 4, 256, 512), (100, 8, 2, 136, 256), (512, 128, 8, 768, 2048)])
def test_gather_grouped_affine(be, T, E, topk, N, K):
    rng = np.random.default_rng(T + E)
    c, s, b, rhs, xr = moe_case(rng, T, E, topk, N, K)
    want = oracle.gather_qmm(xr, c, s, b, np.arange(len(rhs)), rhs, oracle.BF16)
    got = be.gather_qmm(xr, c, s, b, None, rhs, oracle.BF16, oracle.AFFINE, 64, 4, True, None, True)
    assert_product_tight(got, want, oracle.BF16)


@pytest.mark.parametrize("mode,gs", [(oracle.MXFP4, 32), (oracle.NVFP4, 16)])
def test_gather_grouped_fp4(be, mode, gs):
    rng = np.random.default_rng(mode)
    T, E, topk, N, K = 96, 8, 4, 192, 2880
    c, s, _, rhs, xr = moe_case(rng, T, E, topk, N, K, mode, gs, 4)
    for g in ([None] if mode != oracle.NVFP4 else [None, (rng.random(E) * 4 + 0.5).astype(np.float32)]):
        want = oracle.gather_qmm(xr, c, s, None, np.arange(len(rhs)), rhs, oracle.BF16, mode, gs, 4, True, g)
        got = be.gather_qmm(xr, c, s, None, None, rhs, oracle.BF16, mode, gs, 4, True, g, True)
        assert_product_tight(got, want, oracle.BF16, f"global={g is not None}")


@pytest.mark.parametrize("T", [1, 96])
def test_gather_mxfp8(be, T):
    # MXFP8 experts: one token (per-row gather on the few-row kernel) and 96 tokens (sorted rows, grouped, tensor-core kernel)
    rng = np.random.default_rng(T)
    E, topk, N, K = 8, 4, 192, 1024
    c, s, _, rhs, xr = moe_case(rng, T, E, topk, N, K, oracle.MXFP8, 32, 8)
    want = oracle.gather_qmm(xr, c, s, None, np.arange(len(rhs)), rhs, oracle.BF16, oracle.MXFP8, 32, 8, True, None)
    got = be.gather_qmm(xr, c, s, None, None, rhs, oracle.BF16, oracle.MXFP8, 32, 8, True, None, True)
    assert_product_tight(got, want, oracle.BF16)


@pytest.mark.parametrize("mode,gs", [(oracle.MXFP4, 32), (oracle.NVFP4, 16)])
@pytest.mark.parametrize("sorted_rows", [True, False])
def test_gather_few_rows_fp4(be, mode, gs, sorted_rows):
    # one decode token of a gpt-oss-shaped layer: 4 rows, one expert each -> the few-row kernel
    # with per-row expert indices (and the per-expert nvfp4 global scale)
    rng = np.random.default_rng(mode + sorted_rows)
    T, E, topk, N, K = 1, 32, 4, 160, 2880
    c, s, _, rhs, xr = moe_case(rng, T, E, topk, N, K, mode, gs, 4)
    if not sorted_rows:
        perm = rng.permutation(len(rhs))
        rhs, xr = rhs[perm], xr[perm]
    for g in ([None] if mode != oracle.NVFP4 else [None, (rng.random(E) * 4 + 0.5).astype(np.float32)]):
        want = oracle.gather_qmm(xr, c, s, None, np.arange(len(rhs)), rhs, oracle.BF16, mode, gs, 4, True, g)
        got = be.gather_qmm(xr, c, s, None, None, rhs, oracle.BF16, mode, gs, 4, True, g, sorted_rows)
        assert_product_tight(got, want, oracle.BF16, f"global={g is not None}")


@pytest.mark.parametrize("M,N,K", [(1, 4096, 4096), (8, 512, 1024), (600, 512, 1024)])
def test_host_operand_entry_point_matches_the_device_one(be, M, N, K):
    # nvc_quantized_matmul_host: x and y in host memory (small results come back through the
    # pinned block's device mapping, large ones by a copy) -- same bits as the device-resident call
    import ctypes as C
    import nuvec_b200 as nv
    from nuvec_b200 import _ffi
    rng = np.random.default_rng(M + N)
    dev = nv.Device.shared(0)
    quant = nv.Quant.affine(64, 4)
    q = nv.quantize(dev.array(rand(rng, (N, K), oracle.BF16, 0.02), nv.BF16), quant)
    xh = np.ascontiguousarray(rand(rng, (M, K), oracle.BF16))
    want = nv.quantized_matmul(dev.array(xh, nv.BF16), q).to_numpy()
    got = np.zeros((M, N), np.uint16)
    qc = quant._c()
    for _ in range(2):
        rc = _ffi.lib().nvc_quantized_matmul_host(dev._h, C.byref(qc), nv.BF16, 1, xh.ctypes.data_as(C.c_void_p), q.weight.ptr,
                                                  q.scales.ptr, q.biases.ptr, None, M, N, K, got.ctypes.data_as(C.c_void_p))
        assert rc == 0, _ffi.last_error()
        assert np.array_equal(got, want.view(np.uint16).reshape(M, N))
        got[:] = 0


def test_asynchronous_host_entry_point_delivers_at_synchronize(be):
    # nvc_quantized_matmul_host_async: products are issued back to back, nothing waits, and one
    # nvc_synchronize delivers every pending result -- the same bits as the device-resident call
    import ctypes as C
    import nuvec_b200 as nv
    from nuvec_b200 import _ffi
    lib = _ffi.lib()
    rng = np.random.default_rng(31)
    dev = nv.Device.shared(0)
    quant = nv.Quant.affine(64, 4)
    qc = quant._c()
    cases = []
    for M, N, K in [(1, 4096, 4096), (8, 512, 1024), (1, 24576, 4096), (300, 512, 1024), (1, 64, 128)]:
        q = nv.quantize(dev.array(rand(rng, (N, K), oracle.BF16, 0.02), nv.BF16), quant)
        xh = np.ascontiguousarray(rand(rng, (M, K), oracle.BF16))
        want = nv.quantized_matmul(dev.array(xh, nv.BF16), q).to_numpy().view(np.uint16).reshape(M, N)
        cases.append((M, N, K, q, xh, want, np.zeros((M, N), np.uint16)))
    for rounds in range(3):
        for M, N, K, q, xh, want, got in cases:
            got[:] = 0
            x_call = xh.copy()
            rc = lib.nvc_quantized_matmul_host_async(dev._h, C.byref(qc), nv.BF16, 1, x_call.ctypes.data_as(C.c_void_p),
                                                     q.weight.ptr, q.scales.ptr, q.biases.ptr, None, M, N, K,
                                                     got.ctypes.data_as(C.c_void_p))
            assert rc == 0, _ffi.last_error()
            x_call[:] = 0  # the activations may be reused as soon as the call returns
        dev.synchronize()
        for M, N, K, q, xh, want, got in cases:
            assert np.array_equal(got, want), (M, N, K)
    # the same products as one list (nvc_quantized_matmul_host_batch)
    items = (_ffi.HostProduct * len(cases))()
    for it, (M, N, K, q, xh, want, got) in zip(items, cases):
        got[:] = 0
        it.quant, it.dtype, it.transpose = qc, nv.BF16, 1
        it.host_x, it.host_y = xh.ctypes.data, got.ctypes.data
        it.w, it.scales, it.biases, it.global_scale = q.weight.ptr.value, q.scales.ptr.value, q.biases.ptr.value, None
        it.M, it.N, it.K = M, N, K
    assert lib.nvc_quantized_matmul_host_batch(dev._h, items, len(items)) == 0, _ffi.last_error()
    dev.synchronize()
    for M, N, K, q, xh, want, got in cases:
        assert np.array_equal(got, want), (M, N, K)
    # The same list again and again, as a decode loop sends it: the second call records its copy and
    # kernels, later calls replay the recording.  New activations in the same host buffers every
    # time; every result must be the product of the activations of ITS call.
    originals = [xh.copy() for _, _, _, _, xh, _, _ in cases]
    for step in range(4):
        fresh = []
        for M, N, K, q, xh, want, got in cases:
            xh[:] = rand(rng, (M, K), oracle.BF16)
            fresh.append(nv.quantized_matmul(dev.array(xh, nv.BF16), q).to_numpy().view(np.uint16).reshape(M, N))
            got[:] = 0
        dev.synchronize()
        assert lib.nvc_quantized_matmul_host_batch(dev._h, items, len(items)) == 0, _ffi.last_error()
        dev.synchronize()
        for (M, N, K, q, xh, want, got), ref in zip(cases, fresh):
            assert np.array_equal(got, ref), (step, M, N, K)
    # a different list afterwards drops the recording
    assert lib.nvc_quantized_matmul_host_batch(dev._h, items, len(items) - 1) == 0, _ffi.last_error()
    dev.synchronize()
    for (M, N, K, q, xh, want, got), ref in zip(cases[:-1], fresh[:-1]):
        assert np.array_equal(got, ref), (M, N, K)
    for (M, N, K, q, xh, want, got), x0 in zip(cases, originals):
        xh[:] = x0  # the rest of the test uses the first activations and their products again
    # more pending work than the staging blocks hold: the call flushes by itself
    M, N, K, q, xh, want, _ = cases[2]
    outs = [np.zeros((M, N), np.uint16) for _ in range(40)]
    big = [np.zeros((300, 512), np.uint16) for _ in range(200)]
    Mb, Nb, Kb, qb, xb, wantb, _ = cases[3]
    for o in big:
        assert lib.nvc_quantized_matmul_host_async(dev._h, C.byref(qc), nv.BF16, 1, xb.ctypes.data_as(C.c_void_p), qb.weight.ptr,
                                                   qb.scales.ptr, qb.biases.ptr, None, Mb, Nb, Kb, o.ctypes.data_as(C.c_void_p)) == 0
    dev.synchronize()
    assert all(np.array_equal(o, wantb) for o in big)


def test_quantized_embedding_is_take_then_dequantize(be):
    # QuantizedEmbedding::forward (crates/nuvec-nn/src/layers.rs:246-255): the ids' rows of the packed table,
    # its scales and biases, dequantized -- bit for bit the oracle's dequantize of the rows numpy takes;
    # ids past the end take the last row
    import nuvec_b200 as nv
    dev = nv.Device.shared(0)
    rng = np.random.default_rng(77)
    vocab, cols = 1000, 512
    ids = rng.integers(0, vocab, (3, 37)).astype(np.uint32)
    ids[0, :3] = [vocab - 1, vocab, vocab + 50]
    picked = np.minimum(ids, vocab - 1)
    for bits, gs in [(4, 64), (3, 32), (8, 128), (6, 64), (2, 64)]:
        quant = nv.Quant.affine(gs, bits)
        w = rand(rng, (vocab, cols), oracle.BF16, 0.05)
        codes, scales, biases = oracle.quantize(w, oracle.BF16, oracle.AFFINE, gs, bits)
        q = nv.Quantized(dev.array(codes, nv.U32), dev.array(scales, nv.BF16), dev.array(biases, nv.BF16), quant)
        got = nv.quantized_embedding(q, dev.array(ids, nv.U32)).to_numpy().view(np.uint16)
        want = oracle.dequantize(codes[picked], scales[picked], biases[picked], oracle.BF16, oracle.AFFINE, gs, bits)
        assert got.shape == (3, 37, cols) and np.array_equal(got, want), (bits, gs)
    for mode, name, gs in [(oracle.MXFP4, "mxfp4", 32), (oracle.NVFP4, "nvfp4", 16), (oracle.MXFP8, "mxfp8", 32)]:
        bits = 8 if mode == oracle.MXFP8 else 4
        quant = nv.Quant(nv.QuantMode(name), gs, bits)
        w = rand(rng, (vocab, cols), oracle.BF16, 0.05)
        codes, scales, _ = oracle.quantize(w, oracle.BF16, mode, gs, bits)
        q = nv.Quantized(dev.array(codes, nv.U32), dev.array(scales, nv.U8), None, quant)
        got = nv.quantized_embedding(q, dev.array(ids, nv.U32)).to_numpy().view(np.uint16)
        want = oracle.dequantize(codes[picked], scales[picked], None, oracle.BF16, mode, gs, bits)
        assert np.array_equal(got, want), name


@pytest.mark.parametrize("mode", ["nvfp4", "mxfp4"])
@pytest.mark.parametrize("M,N,K", [(128, 128, 256), (64, 256, 512), (1, 128, 64), (300, 384, 1024), (96, 256, 2880),
                                   (513, 1000, 320), (2048, 1024, 4096)])
def test_qqmm_on_the_block_scaled_tensor_core_path(be, M, N, K, mode):
    # MLX's qqmm (crates/nuvec-core/src/products.rs:337-352): x through its own NVFP4 quantization, then the
    # ordinary quantized product.  The kernel feeds both operands to tcgen05.mma.kind::mxf4nvf4.block_scale
    # as 4-bit codes with their scales; every block's scaled sum is exact in float32, so the result
    # agrees with the oracle's float32 product of the two dequantized operands within one output rounding.
    import nuvec_b200 as nv
    dev = nv.Device.shared(0)
    rng = np.random.default_rng(M * 7 + N * 3 + K)
    omode, gs, bits = (oracle.NVFP4, 16, 4) if mode == "nvfp4" else (oracle.MXFP4, 32, 4)
    w = rand(rng, (N, K), oracle.BF16, 0.05)
    wc, ws, _ = oracle.quantize(w, oracle.BF16, omode, gs, bits)
    x = rand(rng, (M, K), oracle.BF16)
    xc, xs, _ = oracle.quantize(x, oracle.BF16, omode, gs, bits)
    xhat = oracle.dequantize(xc, xs, None, oracle.BF16, omode, gs, bits)   # fake_quant(x)
    want = oracle.quantized_matmul(xhat, wc, ws, None, oracle.BF16, omode, gs, bits)
    q = nv.Quantized(dev.array(wc, nv.U32), dev.array(ws, nv.U8), None, nv.Quant(nv.QuantMode(mode), gs, bits))
    got = nv.qqmm(dev.array(x, nv.BF16), q).to_numpy().view(np.uint16)
    assert_product_tight(got, want, oracle.BF16, f"qqmm {mode} {M}x{N}x{K}")
    # the same with the weight's scales laid out beforehand: the same bits
    again = nv.qqmm(dev.array(x, nv.BF16), q, nv.qqmm_prepare_scales(q)).to_numpy().view(np.uint16)
    assert np.array_equal(again, got)
    # and it is NOT the product of the unquantized activations: the activation rounding is the operation
    plain = oracle.quantized_matmul(x, wc, ws, None, oracle.BF16, omode, gs, bits)
    if K >= 256 and M > 1:
        assert np.abs(oracle.to_f32(got, oracle.BF16) - oracle.to_f32(plain, oracle.BF16)).max() > 0


@pytest.mark.parametrize("mode,gs,bits,N,K", [(oracle.AFFINE, 64, 4, 264, 4096), (oracle.AFFINE, 64, 4, 512, 12288),
                                               (oracle.AFFINE, 32, 3, 96, 1024), (oracle.AFFINE, 128, 8, 4096, 4096),
                                               (oracle.MXFP4, 32, 4, 160, 2880), (oracle.MXFP8, 32, 8, 136, 2048)])
def test_row_exact_products_give_each_row_its_one_row_bits(be, mode, gs, bits, N, K):
    # crate::with_row_exact (crates/nuvec-core/src/lib.rs:160-193; the reference's tests/few_rows.rs): up to 8 rows,
    # each with the bits of the same row multiplied alone -- also where 8 rows do not fit the few-row kernel together
    # (K = 12288) and with several batches
    import nuvec_b200 as nv
    dev = nv.Device.shared(0)
    rng = np.random.default_rng(N + K + bits)
    w = rand(rng, (N, K), oracle.BF16, 0.02)
    c, s, b = oracle.quantize(w, oracle.BF16, mode, gs, bits)
    x = rand(rng, (8, K), oracle.BF16)
    with dev.row_exact():
        alone = [be.quantized_matmul(x[i:i + 1], c, s, b, oracle.BF16, mode, gs, bits, True) for i in range(8)]
        for M in (2, 3, 5, 8):
            got = be.quantized_matmul(x[:M], c, s, b, oracle.BF16, mode, gs, bits, True)
            for i in range(M):
                assert np.array_equal(got[i:i + 1], alone[i]), f"M={M} row {i}"
    # the one-row product itself is the same inside and outside the mode
    assert np.array_equal(be.quantized_matmul(x[:1], c, s, b, oracle.BF16, mode, gs, bits, True), alone[0])
    want = oracle.quantized_matmul(x, c, s, b, oracle.BF16, mode, gs, bits)
    assert_product_tight(np.concatenate(alone), want, oracle.BF16)


def test_row_exact_gathers_give_each_row_its_one_row_bits(be):
    # 5 tokens x 4 experts = 20 sorted rows: outside the mode they take the grouped kernel (16+ rows, 4 per expert),
    # inside it every row is its own product and has the bits of that row gathered alone
    import nuvec_b200 as nv
    dev = nv.Device.shared(0)
    rng = np.random.default_rng(77)
    T, E, topk, N, K = 5, 4, 4, 256, 1024
    c, s, b, rhs, xr = moe_case(rng, T, E, topk, N, K)
    with dev.row_exact():
        got = be.gather_qmm(xr, c, s, b, None, rhs, oracle.BF16, oracle.AFFINE, 64, 4, True, None, True)
        for i in (0, 7, 19):
            one = be.gather_qmm(xr[i:i + 1], c, s, b, None, rhs[i:i + 1], oracle.BF16, oracle.AFFINE, 64, 4, True, None, True)
            assert np.array_equal(got[i:i + 1], one), i
    want = oracle.gather_qmm(xr, c, s, b, np.arange(len(rhs)), rhs, oracle.BF16, oracle.AFFINE, 64, 4, True, None)
    assert_product_tight(got, want, oracle.BF16)


@pytest.mark.parametrize("mode,gs,bits", [(oracle.MXFP4, 32, 4), (oracle.NVFP4, 16, 4), (oracle.MXFP8, 32, 8)])
@pytest.mark.parametrize("dt", ["bf16", "f16", "f32"])
def test_fake_quant_is_quantize_then_dequantize(be, mode, gs, bits, dt):
    # FastOp::QuantizeDequantize (crates/nuvec-core/src/products.rs:306-315): the activation side of qqmm / gather_qqmm
    import nuvec_b200 as nv
    dev = nv.Device.shared(0)
    dtype = DT[dt]
    rng = np.random.default_rng(mode * 7 + dtype)
    x = rand(rng, (13, 4 * gs), dtype, 1.0)
    x.reshape(-1)[:4] = oracle.from_f32(np.array([0.0, -0.0, 1e-30, 500.0], np.float32), dtype)
    code = {oracle.BF16: nv.BF16, oracle.F16: nv.F16, oracle.F32: nv.F32}[dtype]
    for g in ([None] if mode != oracle.NVFP4 else [None, 2.5]):
        c, s, _ = oracle.quantize(x, dtype, mode, gs, bits, g)
        want = oracle.dequantize(c, s, None, dtype, mode, gs, bits, g)
        gd = None if g is None else dev.array(np.array([g], np.float32), nv.F32)
        xd = dev.array(x.view(np.float16) if dtype == oracle.F16 else x, code)
        got = nv.fake_quant(xd, nv.Quant(be_mode(mode), gs, bits), gd).to_numpy()
        assert np.array_equal(got.view(np.uint8), np.ascontiguousarray(want).view(np.uint8)), f"global={g}"


def be_mode(mode):
    import nuvec_b200 as nv
    return {oracle.MXFP4: nv.QuantMode.MXFP4, oracle.NVFP4: nv.QuantMode.NVFP4, oracle.MXFP8: nv.QuantMode.MXFP8,
            oracle.AFFINE: nv.QuantMode.AFFINE}[mode]


@pytest.mark.parametrize("mode,gs,bits,scaled", [(oracle.MXFP4, 32, 4, False), (oracle.NVFP4, 16, 4, False), (oracle.NVFP4, 16, 4, True),
                                                 (oracle.MXFP8, 32, 8, False)])
def test_gather_qqmm_and_qqmm_with_global_scales(be, mode, gs, bits, scaled):
    # MLX's gather_qqmm (products.rs:437-463) and qqmm with nvfp4 global scales (:317-352): the activations through
    # their quantization (with their global scale), then the ordinary gathered / plain quantized product
    import nuvec_b200 as nv
    dev = nv.Device.shared(0)
    rng = np.random.default_rng(mode + scaled)
    T, E, topk, N, K = 6, 8, 2, 96, 256
    w = rand(rng, (E, N, K), oracle.BF16, 0.05)
    gw, gx = (3.0, 1.5) if scaled else (None, None)
    c, s, _ = oracle.quantize(w.reshape(E * N, K), oracle.BF16, mode, gs, bits, gw)
    c, s = c.reshape(E, N, -1), s.reshape(E, N, -1)
    x = rand(rng, (T, K), oracle.BF16)
    rhs = np.sort(rng.integers(0, E, T * topk)).astype(np.uint32)
    xr = np.repeat(x, topk, axis=0).reshape(T * topk, 1, K)
    xc, xs, _ = oracle.quantize(xr.reshape(-1, K), oracle.BF16, mode, gs, bits, gx)
    xhat = oracle.dequantize(xc, xs, None, oracle.BF16, mode, gs, bits, gx).reshape(T * topk, 1, K)
    gexp = None if gw is None else np.full(E, gw, np.float32)
    want = oracle.gather_qmm(xhat, c, s, None, np.arange(len(rhs)), rhs, oracle.BF16, mode, gs, bits, True, gexp)
    q = nv.Quantized(dev.array(c, nv.U32), dev.array(s, nv.U8), None, nv.Quant(be_mode(mode), gs, bits),
                     None if gw is None else dev.array(np.array([gw], np.float32), nv.F32))
    gxd = None if gx is None else dev.array(np.array([gx], np.float32), nv.F32)
    got = nv.gather_qqmm(dev.array(xr, nv.BF16), q, None, dev.array(rhs, nv.U32), True, gxd).to_numpy()
    assert_product_tight(got.reshape(want.shape), want, oracle.BF16, "gather_qqmm")
    # qqmm on one expert's matrix, with the global scales
    one = nv.Quantized(q.weight[3], q.scales[3], None, q.quant, q.global_scale)
    got2 = nv.qqmm(dev.array(x, nv.BF16), one, None, gxd).to_numpy()
    xc2, xs2, _ = oracle.quantize(x, oracle.BF16, mode, gs, bits, gx)
    xhat2 = oracle.dequantize(xc2, xs2, None, oracle.BF16, mode, gs, bits, gx)
    want2 = oracle.quantized_matmul(xhat2, c[3], s[3], None, oracle.BF16, mode, gs, bits, True, gw)
    assert_product_tight(got2, want2, oracle.BF16, "qqmm")
    if scaled:
        with pytest.raises(nv.InvalidArgument, match="both"):
            nv.qqmm(dev.array(x, nv.BF16), one)
