"""The benchmark definition's own configurations at their full size, CUDA path against the oracle.

Sizes (the metric's configurations): Qwen3-8B prefill 2048 x 12288 x 4096 at 4 and 8 bits, the fused
gate+up decode product (N = 24576) at 1, 4 and 8 rows, the Qwen3-30B-A3B expert products with 128
experts and 512 tokens (both projections), the gpt-oss-shaped MXFP4 / NVFP4 expert products with 32
experts and 1024 tokens (N = 5760 and 2880, K = 2880), and a persistent tensor-core run of more
tiles than multiprocessors at every token-tile width.

At these sizes the oracle is only affordable on a part of the output, so every case combines
  * unit-vector activations over the whole output: y[m, :] is then column k_m of the dequantized
    matrix and must equal the oracle's `dequantize` bit for bit (size-independent: it needs no
    product oracle and catches any permuted, dropped or stale k-slot), and
  * random activations checked against the oracle's product on a subset of output rows / gathered
    rows, within one output rounding (the kernels' operands are exact; only the float32
    summation order differs) and therefore far inside the stated 1e-2 * ||row||_inf.
Weights are random codes with scales and biases in the range quantizing N(0, 0.02) weights gives;
the oracle and the kernel consume the same arrays.
"""
import numpy as np
import pytest

import oracle
from test_gpu_parity import assert_product_close, assert_product_tight, rand

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def be():
    from cuda_backend import CudaBackend
    return CudaBackend()


def affine_weights(rng, shape_nk, bits, gs=64):
    """Random codes; scales / biases as quantizing N(0, 0.02) weights gives them."""
    *lead, N, K = shape_nk
    c = rng.integers(0, 2 ** 32, (*lead, N, K * bits // 32), dtype=np.uint32)
    levels = float(2 ** bits - 1)
    s = oracle.from_f32((rng.random((*lead, N, K // gs), dtype=np.float32) * 0.06 + 0.03) / levels, oracle.BF16)
    b = oracle.from_f32(-(rng.random((*lead, N, K // gs), dtype=np.float32) * 0.04 + 0.02), oracle.BF16)
    return c, s, b


def fp4_weights(rng, shape_nk, mode):
    *lead, N, K = shape_nk
    gs = 32 if mode == oracle.MXFP4 else 16
    c = rng.integers(0, 2 ** 32, (*lead, N, K // 8), dtype=np.uint32)
    if mode == oracle.MXFP4:
        s = rng.integers(117, 123, (*lead, N, K // gs), dtype=np.uint8)      # E8M0: 2^-10 .. 2^-5
    else:
        s = rng.integers(0x08, 0x30, (*lead, N, K // gs), dtype=np.uint8)    # E4M3: 2^-6 .. ~0.03 (positive)
    return c, s, gs


def unit_rows(rng, M, K):
    ks = rng.integers(0, K, M)
    x = np.zeros((M, K), np.float32)
    x[np.arange(M), ks] = 1.0
    return oracle.from_f32(x, oracle.BF16), ks


@pytest.mark.parametrize("bits", [4, 8])
def test_prefill_2048x12288x4096(be, bits):
    rng = np.random.default_rng(300 + bits)
    M, N, K = 2048, 12288, 4096
    c, s, b = affine_weights(rng, (N, K), bits)
    dense = oracle.dequantize(c, s, b, oracle.BF16, oracle.AFFINE, 64, bits)
    xu, ks = unit_rows(rng, M, K)
    got = be.quantized_matmul(xu, c, s, b, oracle.BF16, oracle.AFFINE, 64, bits, True)
    assert np.array_equal(got, dense[:, ks].T)
    x = rand(rng, (M, K), oracle.BF16)
    got = be.quantized_matmul(x, c, s, b, oracle.BF16, oracle.AFFINE, 64, bits, True)
    rows = np.sort(rng.permutation(N)[:192])
    want = oracle.quantized_matmul(x, c[rows], s[rows], b[rows], oracle.BF16, oracle.AFFINE, 64, bits)
    assert_product_close(got[:, rows], want, oracle.BF16)
    assert_product_tight(got[:, rows], want, oracle.BF16)


def test_decode_gate_up_24576(be):
    rng = np.random.default_rng(24576)
    N, K = 24576, 4096
    c, s, b = affine_weights(rng, (N, K), 4)
    for M in (1, 4, 8):
        x = rand(rng, (M, K), oracle.BF16)
        want = oracle.quantized_matmul(x, c, s, b, oracle.BF16)
        got = be.quantized_matmul(x, c, s, b, oracle.BF16, oracle.AFFINE, 64, 4, True)
        assert_product_close(got, want, oracle.BF16, f"M{M}")
        assert_product_tight(got, want, oracle.BF16, f"M{M}")
    dense = oracle.dequantize(c, s, b, oracle.BF16)
    xu, ks = unit_rows(rng, 8, K)
    got = be.quantized_matmul(xu, c, s, b, oracle.BF16, oracle.AFFINE, 64, 4, True)
    assert np.array_equal(got, dense[:, ks].T)


def sorted_routing(rng, T, E, topk):
    ids = np.concatenate([rng.permutation(E)[:topk] for _ in range(T)]).astype(np.uint32)
    order = np.argsort(ids, kind="stable")
    return ids[order], np.repeat(np.arange(T), topk)[order]


def check_grouped(be, rng, c, s, b, mode, gs, rhs, xr, subset, g=None):
    """Whole grouped product on the device; the oracle on `subset` gathered rows."""
    got = be.gather_qmm(xr, c, s, b, None, rhs, oracle.BF16, mode, gs, 4, True, g, True)
    want = oracle.gather_qmm(np.ascontiguousarray(xr[subset]), c, s, b, np.arange(len(subset)), rhs[subset],
                             oracle.BF16, mode, gs, 4, True, g)
    assert_product_close(got[subset], want, oracle.BF16)
    assert_product_tight(got[subset], want, oracle.BF16)
    return got


@pytest.mark.parametrize("N,K", [(768, 2048), (1536, 2048), (2048, 768)])
def test_moe_128_experts_512_tokens(be, N, K):
    # gate / up, fused gate+up and down of a Qwen3-30B-A3B layer: 4096 gathered rows, 32 per expert
    rng = np.random.default_rng(N + K)
    T, E, topk = 512, 128, 8
    c, s, b = affine_weights(rng, (E, N, K), 4)
    rhs, tok = sorted_routing(rng, T, E, topk)
    x = rand(rng, (T, K), oracle.BF16)
    xr = np.ascontiguousarray(x[tok][:, None, :])
    subset = np.sort(rng.permutation(len(rhs))[:48])
    check_grouped(be, rng, c, s, b, oracle.AFFINE, 64, rhs, xr, subset)
    # unit rows: every gathered row returns a column of its own expert's dequantized matrix
    xu, ks = unit_rows(rng, len(rhs), K)
    got = be.gather_qmm(xu[:, None, :], c, s, b, None, rhs, oracle.BF16, oracle.AFFINE, 64, 4, True, None, True)
    for e in range(0, E, 9):  # expert by expert (bounded host memory and time)
        dense = oracle.dequantize(c[e], s[e], b[e], oracle.BF16)
        sel = np.nonzero(rhs == e)[0]
        assert np.array_equal(got[sel, 0, :], dense[:, ks[sel]].T), f"expert {e}"


@pytest.mark.parametrize("mode", [oracle.MXFP4, oracle.NVFP4])
@pytest.mark.parametrize("N", [5760, 2880])
def test_moe_32_experts_1024_tokens_fp4(be, mode, N):
    # gpt-oss-20b-shaped layer: 4096 gathered rows, 128 per expert, K = 2880 (45 groups of 64)
    rng = np.random.default_rng(mode * 7 + N)
    T, E, topk, K = 1024, 32, 4, 2880
    c, s, gs = fp4_weights(rng, (E, N, K), mode)
    rhs, tok = sorted_routing(rng, T, E, topk)
    x = rand(rng, (T, K), oracle.BF16)
    xr = np.ascontiguousarray(x[tok][:, None, :])
    subset = np.sort(rng.permutation(len(rhs))[:12])
    g = None if mode == oracle.MXFP4 else (rng.random(E) * 4 + 0.5).astype(np.float32)
    check_grouped(be, rng, c, s, None, mode, gs, rhs, xr, subset, g)
    if g is not None:  # the same product without the per-expert scale
        check_grouped(be, rng, c, s, None, mode, gs, rhs, xr, subset[:4], None)
    # unit rows against the float32 decode, expert by expert (bounded host memory)
    xu, ks = unit_rows(rng, len(rhs), K)
    got = oracle.to_f32(be.gather_qmm(xu[:, None, :], c, s, None, None, rhs, oracle.BF16, mode, gs, 4, True, None, True),
                        oracle.BF16)[:, 0, :]
    for e in range(0, E, 5):
        dense = oracle.to_f32(oracle.dequantize(c[e], s[e], None, oracle.F32, mode, gs, 4), oracle.F32)
        sel = np.nonzero(rhs == e)[0]
        assert np.array_equal(got[sel], dense[:, ks[sel]].T), f"expert {e}"


@pytest.mark.parametrize("mode", [oracle.MXFP4, oracle.NVFP4])
def test_moe_32_experts_one_token_fp4(be, mode):
    rng = np.random.default_rng(mode + 99)
    E, topk, N, K = 32, 4, 5760, 2880
    c, s, gs = fp4_weights(rng, (E, N, K), mode)
    rhs, tok = sorted_routing(rng, 1, E, topk)
    x = rand(rng, (1, K), oracle.BF16)
    xr = np.ascontiguousarray(x[tok][:, None, :])
    want = oracle.gather_qmm(xr, c, s, None, np.arange(len(rhs)), rhs, oracle.BF16, mode, gs, 4)
    got = be.gather_qmm(xr, c, s, None, None, rhs, oracle.BF16, mode, gs, 4, True, None, True)
    assert_product_tight(got, want, oracle.BF16)


@pytest.mark.parametrize("bits,gs,K", [(4, 64, 2048), (8, 64, 2048), (2, 64, 2048), (4, 128, 1920), (8, 32, 1024)])
def test_qmm_persistent_run_of_more_tiles_than_multiprocessors(be, bits, gs, K):
    # 4096 tokens x 2560 weight rows: 16 x 20 = 320 tiles of 256 tokens (22 x 20 = 440 of 192) on
    # 148 multiprocessors, i.e. two whole waves plus a K-split tail at every token-tile width.
    # Unit-vector rows make any stale or overwritten pipeline stage a bit difference.
    rng = np.random.default_rng(bits * 31 + K)
    M, N = 4096, 2560
    c, s, b = affine_weights(rng, (N, K), bits, gs)
    dense = oracle.dequantize(c, s, b, oracle.BF16, oracle.AFFINE, gs, bits)
    xu, ks = unit_rows(rng, M, K)
    for _ in range(2):  # twice: the second launch starts on warm caches and different timing
        got = be.quantized_matmul(xu, c, s, b, oracle.BF16, oracle.AFFINE, gs, bits, True)
        assert np.array_equal(got, dense[:, ks].T)
    x = rand(rng, (M, K), oracle.BF16)
    got = be.quantized_matmul(x, c, s, b, oracle.BF16, oracle.AFFINE, gs, bits, True)
    rows = np.sort(rng.permutation(N)[:64])
    want = oracle.quantized_matmul(x, c[rows], s[rows], b[rows], oracle.BF16, oracle.AFFINE, gs, bits)
    assert_product_tight(got[:, rows], want, oracle.BF16)


def test_gather_indices_past_the_end_select_the_last_batch(be):
    # The reference casts gather indices to u32 and its `take` clamps indices past the end
    # (crates/nuvec-core/src/quantized.rs:756, crates/nuvec-core/src/kernels.rs:120-129): so does every route here.
    rng = np.random.default_rng(77)
    E, N, K = 6, 96, 256
    c, s, b = affine_weights(rng, (E, N, K), 4)
    x = rand(rng, (5, 1, K), oracle.BF16)
    rhs = np.array([0, 5, 6, 1000, 0xFFFFFFFF, 2], np.uint32)
    lhs = np.array([0, 4, 5, 77, 1, 0xFFFFFFFF], np.uint32)
    want = oracle.gather_qmm(x, c, s, b, np.minimum(lhs, 4), np.minimum(rhs, E - 1), oracle.BF16)
    got = be.gather_qmm(x, c, s, b, lhs, rhs, oracle.BF16, oracle.AFFINE, 64, 4, True, None, False)
    assert_product_tight(got, want, oracle.BF16)
    # f32 operands take the generic kernel
    xf = oracle.to_f32(x, oracle.BF16)
    sf, bf = oracle.to_f32(s, oracle.BF16), oracle.to_f32(b, oracle.BF16)
    want = oracle.gather_qmm(xf, c, sf, bf, np.minimum(lhs, 4), np.minimum(rhs, E - 1), oracle.F32)
    got = be.gather_qmm(xf, c, sf, bf, lhs, rhs, oracle.F32, oracle.AFFINE, 64, 4, True, None, False)
    assert_product_close(got, want, oracle.F32)


def test_block_pairs_switched_on():
    # The tensor-core kernel's block pairs (tcgen05.mma.cta_group::2) are off by default and the
    # switch is read once per process: the prefill and persistent-run cases of this file run again
    # in a child process with NUVEC_QMM_PAIRS=1.
    import os
    import subprocess
    import sys
    env = dict(os.environ, NUVEC_QMM_PAIRS="1")
    here = os.path.dirname(os.path.abspath(__file__))
    out = subprocess.run([sys.executable, "-m", "pytest", os.path.join(here, "test_gpu_configs.py"), "-x", "-q", "-m", "gpu",
                          "-k", "prefill or persistent"], env=env, cwd=os.path.dirname(here), capture_output=True, text=True,
                         timeout=1200)
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-2000:]
    assert " passed" in out.stdout, out.stdout[-500:]
