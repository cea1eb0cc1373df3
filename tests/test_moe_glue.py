"""The router's top-k selection and the weighted expert sum: the CPU oracle against a plain numpy
statement of the compositions (CPU), and the CUDA kernels against the oracle bit for bit (GPU).
Cases follow the reference's own test (crates/nuvec-core/tests/fast.rs:841-925): router
probabilities with and without ties, k from 1 to all experts, every float dtype, NaN last."""
import numpy as np
import pytest

import oracle

DT = {"f32": oracle.F32, "f16": oracle.F16, "bf16": oracle.BF16}
CASES = [(3, 8, (1, 2, 8)), (5, 60, (4, 8)), (4, 128, (1, 8, 10, 128)), (2, 512, (8, 22))]


def probabilities(rng, rows, e, dtype, ties):
    z = rng.standard_normal((rows, e)).astype(np.float32)
    p = np.exp(z - z.max(-1, keepdims=True))
    p /= p.sum(-1, keepdims=True)
    if ties:  # a few values (none 0) repeated across experts
        levels = 4.0 * e
        p = (np.floor(p * levels) + 1.0) / levels
    return oracle.from_f32(p.astype(np.float32), dtype)


@pytest.mark.parametrize("dt", list(DT))
def test_oracle_moe_route_is_a_stable_sort_take_and_renormalisation(dt):
    dtype = DT[dt]
    rng = np.random.default_rng(0x72)
    for rows, e, ks in CASES:
        for ties in (False, True):
            p = probabilities(rng, rows, e, dtype, ties)
            pf = oracle.to_f32(p, dtype)
            order = np.argsort(pf, axis=-1, kind="stable")
            for k in ks:
                idx, scores = oracle.moe_route(p, dtype, k, False)
                assert np.array_equal(idx, order[:, e - k:])
                assert np.array_equal(scores, np.take_along_axis(p, order[:, e - k:], -1))
                idx, scores = oracle.moe_route(p, dtype, k, True)
                assert np.array_equal(idx, order[:, e - k:])
                top = np.take_along_axis(pf, order[:, e - k:], -1).astype(np.float64)
                total = oracle.to_f32(oracle.from_f32(top.sum(-1, keepdims=True).astype(np.float32), dtype), dtype)
                want = oracle.from_f32((top.astype(np.float32) / total).astype(np.float32), dtype)
                got = oracle.to_f32(scores, dtype)
                # (the float64 sum of at most 128 such values is exact; so is its one rounding)
                assert np.allclose(got, oracle.to_f32(want, dtype), rtol=2.0 ** -7 if dt == "bf16" else 2.0 ** -10, atol=0)
    # NaN sorts last
    p = np.array([[0.1, np.nan, 0.3, 0.2]], np.float32)
    idx, _ = oracle.moe_route(p, oracle.F32, 2, False)
    assert idx.tolist() == [[2, 1]]
    with pytest.raises(oracle.OracleError):
        oracle.moe_route(p, oracle.F32, 5, False)


@pytest.mark.parametrize("dt", list(DT))
def test_oracle_weighted_sum(dt):
    dtype = DT[dt]
    rng = np.random.default_rng(5)
    for rows, k, d in [(3, 8, 16), (7, 4, 1), (2, 1, 5), (4, 10, 33)]:
        x = oracle.from_f32(rng.standard_normal((rows, k, d)).astype(np.float32), dtype)
        w = oracle.from_f32(rng.random((rows, k)).astype(np.float32), dtype)
        got = oracle.to_f32(oracle.weighted_sum(x, w, dtype), dtype)
        prod = oracle.to_f32(oracle.from_f32(oracle.to_f32(x, dtype) * oracle.to_f32(w, dtype)[..., None], dtype), dtype)
        want = oracle.to_f32(oracle.from_f32(prod.astype(np.float64).sum(-2).astype(np.float32), dtype), dtype)
        tol = {"f32": 1e-6, "f16": 2.0 ** -10, "bf16": 2.0 ** -7}[dt]
        assert np.allclose(got, want, rtol=tol, atol=tol * 1e-3)


@pytest.mark.gpu
@pytest.mark.parametrize("dt", list(DT))
def test_cuda_moe_route_matches_the_oracle_bit_for_bit(dt):
    import nuvec_b200 as nv
    dtype = DT[dt]
    code = {"f32": nv.F32, "f16": nv.F16, "bf16": nv.BF16}[dt]
    dev = nv.Device.shared(0)
    rng = np.random.default_rng(0x73)
    up = lambda a: dev.array(a.view(np.float16) if dt == "f16" else a, code)
    bits = lambda a: a.to_numpy().view(np.uint16 if dt != "f32" else np.uint32)
    for rows, e, ks in CASES + [(512, 128, (8,)), (1024, 32, (4,)), (2, 1024, (64,))]:
        for ties in (False, True):
            p = probabilities(rng, rows, e, dtype, ties)
            for k in ks:
                for normalize in (False, True):
                    want_idx, want_scores = oracle.moe_route(p, dtype, k, normalize)
                    idx, scores = nv.moe_route(up(p), k, normalize)
                    assert np.array_equal(idx.to_numpy(), want_idx), (rows, e, k, ties, normalize)
                    assert np.array_equal(bits(scores), want_scores.view(bits(scores).dtype)), (rows, e, k, ties, normalize)
    p = np.array([[0.1, np.nan, 0.3, 0.2]], np.float32)
    idx, _ = nv.moe_route(dev.array(p, nv.F32), 2, False)
    assert idx.to_numpy().tolist() == [[2, 1]]
    # batched leading axes, as a model's [B, L, E]
    p = probabilities(rng, 6, 16, dtype, False).reshape(2, 3, 16)
    idx, scores = nv.moe_route(up(p), 4, True)
    assert idx.shape == (2, 3, 4) and np.array_equal(idx.to_numpy(), oracle.moe_route(p, dtype, 4, True)[0])
    with pytest.raises(nv.InvalidArgument):
        nv.moe_route(up(p), 17, True)


@pytest.mark.gpu
@pytest.mark.parametrize("dt", list(DT))
def test_cuda_weighted_sum_matches_the_oracle_bit_for_bit(dt):
    import nuvec_b200 as nv
    dtype = DT[dt]
    code = {"f32": nv.F32, "f16": nv.F16, "bf16": nv.BF16}[dt]
    dev = nv.Device.shared(0)
    rng = np.random.default_rng(9)
    up = lambda a: dev.array(a.view(np.float16) if dt == "f16" else a, code)
    for rows, k, d in [(3, 8, 16), (7, 4, 1), (2, 1, 5), (4, 10, 33), (512, 8, 2048), (1024, 4, 2880)]:
        x = oracle.from_f32(rng.standard_normal((rows, k, d)).astype(np.float32), dtype)
        w = oracle.from_f32(rng.random((rows, k)).astype(np.float32), dtype)
        want = oracle.weighted_sum(x, w, dtype)
        got = nv.weighted_sum(up(x), up(w)).to_numpy()
        assert np.array_equal(got.view(want.dtype) if dt != "f16" else got.view(np.uint16), want), (rows, k, d)
    with pytest.raises(nv.InvalidArgument):
        nv.weighted_sum(up(x), up(w[:, :2]))


@pytest.mark.parametrize("dt", list(DT))
def test_oracle_expert_bias_add(dt):
    # y + bias.take(indices, 0): the add in the array's type (float32 arithmetic, one rounding),
    # indices past the end clamped to the last expert
    dtype = DT[dt]
    rng = np.random.default_rng(11)
    for rows, n, e in [(5, 16, 4), (9, 33, 7), (1, 1, 1)]:
        y = oracle.from_f32(rng.standard_normal((rows, n)).astype(np.float32), dtype)
        b = oracle.from_f32(rng.standard_normal((e, n)).astype(np.float32), dtype)
        idx = rng.integers(0, e + 2, rows).astype(np.uint32)
        got = oracle.expert_bias_add(y, b, idx, dtype)
        want = oracle.from_f32(oracle.to_f32(y, dtype) + oracle.to_f32(b, dtype)[np.minimum(idx, e - 1)], dtype)
        assert np.array_equal(got.view(want.dtype), want), (rows, n, e)
        assert np.array_equal(y.view(want.dtype), oracle.from_f32(oracle.to_f32(y, dtype), dtype).view(want.dtype))  # the input is left alone


@pytest.mark.gpu
@pytest.mark.parametrize("dt", list(DT))
def test_cuda_expert_bias_add_matches_the_oracle_bit_for_bit(dt):
    import nuvec_b200 as nv
    dtype = DT[dt]
    code = {"f32": nv.F32, "f16": nv.F16, "bf16": nv.BF16}[dt]
    dev = nv.Device.shared(0)
    rng = np.random.default_rng(12)
    up = lambda a: dev.array(a.view(np.float16) if dt == "f16" else a, code)
    # the expert products' own shapes: 4096 gathered rows of 2880 (32 experts) and of 2048 (128 experts)
    for rows, n, e in [(5, 16, 4), (9, 33, 7), (4096, 2880, 32), (4096, 2048, 128), (8, 1536, 128)]:
        y = oracle.from_f32(rng.standard_normal((rows, n)).astype(np.float32), dtype)
        b = oracle.from_f32(rng.standard_normal((e, n)).astype(np.float32), dtype)
        idx = np.sort(rng.integers(0, e + (2 if rows < 100 else 0), rows)).astype(np.uint32)
        want = oracle.expert_bias_add(y, b, idx, dtype)
        got = nv.expert_bias_add(up(y), up(b), dev.array(idx, nv.U32)).to_numpy()
        assert np.array_equal(got.view(np.uint16) if dt != "f32" else got.view(np.uint32),
                              want.view(np.uint16) if dt != "f32" else want.view(np.uint32)), (rows, n, e)
    with pytest.raises(nv.InvalidArgument):
        nv.expert_bias_add(up(y), up(b[:, :5]), dev.array(idx, nv.U32))


def expert_choices(rng, tokens, experts, k):
    """k distinct experts per token, as a router's top-k gives them."""
    return np.stack([rng.permutation(experts)[:k] for _ in range(tokens)]).astype(np.uint32)


def test_oracle_moe_sort_is_the_stable_argsort_and_its_inverse():
    rng = np.random.default_rng(21)
    for tokens, experts, k in [(1, 8, 2), (7, 16, 4), (512, 128, 8), (1024, 32, 4), (3, 5, 5)]:
        idx = expert_choices(rng, tokens, experts, k)
        order, restore, toks, srt, offsets = oracle.moe_sort(idx, experts)
        flat = idx.reshape(-1)
        want = np.argsort(flat, kind="stable").astype(np.uint32)
        assert np.array_equal(order, want)
        assert np.array_equal(restore, np.argsort(want, kind="stable").astype(np.uint32))
        assert np.array_equal(toks, want // k) and np.array_equal(srt, flat[want])
        assert np.array_equal(offsets, oracle.sorted_offsets(srt, experts))
    with pytest.raises(oracle.OracleError):
        oracle.moe_sort(np.array([[9]], np.uint32), 4)


@pytest.mark.gpu
def test_cuda_moe_sort_and_take_rows_match_the_oracle():
    import nuvec_b200 as nv
    dev = nv.Device.shared(0)
    rng = np.random.default_rng(22)
    for tokens, experts, k in [(1, 8, 2), (7, 16, 4), (512, 128, 8), (1024, 32, 4), (3, 5, 5), (8192, 128, 8), (300, 1024, 3)]:
        idx = expert_choices(rng, tokens, experts, k)
        want = oracle.moe_sort(idx, experts)
        got = nv.moe_sort(dev.array(idx, nv.U32), experts)
        for name, g, w in zip(("order", "restore", "tokens", "sorted", "offsets"), got, want):
            assert np.array_equal(g.to_numpy(), w), (name, tokens, experts, k)
        # the layer's two row gathers: activations by sorted pair, results back into pair order
        d = 96
        x = oracle.from_f32(rng.standard_normal((tokens, d)).astype(np.float32), oracle.BF16)
        rows = nv.take_rows(dev.array(x, nv.BF16), got[2]).to_numpy().view(np.uint16)
        assert np.array_equal(rows, x[want[2]])
        back = nv.take_rows(dev.array(rows, nv.BF16), got[1]).to_numpy().view(np.uint16)
        assert np.array_equal(back, x[np.arange(tokens * k) // k])
    # rows of a width that is no multiple of 16 bytes, and an index past the end
    src = rng.integers(0, 255, (5, 7), dtype=np.uint8)
    out = nv.take_rows(dev.array(src, nv.U8), dev.array(np.array([4, 0, 9, 2], np.uint32), nv.U32)).to_numpy()
    assert np.array_equal(out, src[[4, 0, 4, 2]])
    with pytest.raises(nv.UnsupportedError):
        nv.moe_sort(dev.array(np.zeros((2, 2), np.uint32), nv.U32), 2000)


def glu_inputs(rng, n, dtype):
    gate = rng.standard_normal(n).astype(np.float32) * 3.0
    up = rng.standard_normal(n).astype(np.float32) * 3.0
    gate[:8] = [0.0, -0.0, 20.0, -20.0, 90.0, -90.0, 7.0, np.nan]
    up[:8] = [1.0, 1.0, 9.0, -9.0, 1.0, 1.0, np.nan, 1.0]
    return oracle.from_f32(gate, dtype), oracle.from_f32(up, dtype)


@pytest.mark.parametrize("dt", list(DT))
def test_oracle_swiglu_is_the_composition_op_by_op(dt):
    dtype = DT[dt]
    rng = np.random.default_rng(31)
    gate, up = glu_inputs(rng, 4096, dtype)
    g, x = oracle.to_f32(gate, dtype), oracle.to_f32(up, dtype)
    rnd = lambda v: oracle.to_f32(oracle.from_f32(v.astype(np.float32), dtype), dtype)
    with np.errstate(over="ignore", invalid="ignore"):
        def sigmoid(v):
            y = (np.float32(1) / (np.float32(1) + np.exp(np.abs(v), dtype=np.float32))).astype(np.float32)
            return np.where(v < 0, y, np.float32(1) - y).astype(np.float32)
        want = rnd(rnd(g * rnd(sigmoid(g))) * x)
        got = oracle.to_f32(oracle.swiglu(gate, up, dtype), dtype)
        tol = {"f32": 1e-6, "f16": 2.0 ** -10, "bf16": 2.0 ** -7}[dt]
        assert np.allclose(got, want, rtol=tol, atol=1e-30, equal_nan=True)
        # the clamped form: limits reached on both sides, NaN kept
        alpha, limit = rnd(np.float32(1.702)), rnd(np.float32(7.0))
        gc = np.where(np.isnan(g), np.nan, np.minimum(g, limit)).astype(np.float32)
        xc = np.where(np.isnan(x), np.nan, np.clip(x, -limit, limit)).astype(np.float32)
        want = rnd(rnd(xc + np.float32(1)) * rnd(gc * rnd(sigmoid(rnd(alpha * gc)))))
        got = oracle.to_f32(oracle.swiglu(gate, up, dtype, oai=True), dtype)
        assert np.allclose(got, want, rtol=tol, atol=1e-30, equal_nan=True)


@pytest.mark.gpu
@pytest.mark.parametrize("dt", list(DT))
def test_cuda_swiglu_matches_the_oracle(dt):
    # every step but the exponential is an IEEE operation: results equal the oracle's bit for bit
    # except where the device's and the host's expf differ in their last bit AND the sigmoid's
    # rounding to the array's type falls the other way -- the sigmoid is then one unit in the last
    # place off, and the two roundings behind it can make that two (measured: 2 of 3.1 M float16
    # elements); float32 shows the exponentials' difference directly (a few units)
    import nuvec_b200 as nv
    dtype = DT[dt]
    code = {"f32": nv.F32, "f16": nv.F16, "bf16": nv.BF16}[dt]
    dev = nv.Device.shared(0)
    rng = np.random.default_rng(32)
    up_ = lambda a: dev.array(a.view(np.float16) if dt == "f16" else a, code)
    for n in (4096 * 768, 1000):
        gate, up = glu_inputs(rng, n, dtype)
        for oai in (False, True):
            want = oracle.swiglu(gate, up, dtype, oai=oai)
            got = (nv.swiglu_oai(up_(gate), up_(up)) if oai else nv.swiglu(up_(gate), up_(up))).to_numpy()
            g32, w32 = oracle.to_f32(got.view(want.dtype) if dt != "f16" else got.view(np.uint16), dtype), oracle.to_f32(want, dtype)
            same = (g32 == w32) | (np.isnan(g32) & np.isnan(w32))
            if dt == "f32":
                assert np.allclose(g32, w32, rtol=4e-7, atol=1e-37, equal_nan=True), (n, oai)
            else:
                assert same.mean() > 0.9995, (n, oai, float(same.mean()))
                # (units in the last place: relative for normal numbers, 2^-24 among float16's subnormals)
                ulp = np.maximum(np.abs(w32) * (2.0 ** -10 if dt == "f16" else 2.0 ** -7), 2.0 ** -24 if dt == "f16" else 2.0 ** -133)
                bad = ~(same | (np.abs(g32 - w32) <= 2.0 * ulp))
                assert not bad.any(), (n, oai, int(bad.sum()), g32[bad][:4], w32[bad][:4])
    with pytest.raises(nv.InvalidArgument):
        nv.swiglu(up_(gate), up_(up[:5]))


@pytest.mark.parametrize("dt", list(DT))
def test_oracle_rms_norm(dt):
    dtype = DT[dt]
    rng = np.random.default_rng(41)
    for rows, d in [(3, 64), (2, 4096), (5, 37), (1, 8), (4, 5)]:
        x = oracle.from_f32(rng.standard_normal((rows, d)).astype(np.float32) * 2.0, dtype)
        w = oracle.from_f32(rng.standard_normal(d).astype(np.float32), dtype)
        res = oracle.from_f32(rng.standard_normal((rows, d)).astype(np.float32), dtype)
        xf = oracle.to_f32(x, dtype)
        rnd = lambda v: oracle.to_f32(oracle.from_f32(v.astype(np.float32), dtype), dtype)
        def norm(v):
            n = np.float32(1) / np.sqrt((v.astype(np.float64) ** 2).mean(-1, keepdims=True).astype(np.float32) + np.float32(1e-5))
            return rnd(rnd(v * n.astype(np.float32)) * oracle.to_f32(w, dtype))
        tol = {"f32": 2e-6, "f16": 2.0 ** -9, "bf16": 2.0 ** -6}[dt]
        got = oracle.to_f32(oracle.rms_norm(x, dtype, w), dtype)
        assert np.allclose(got, norm(xf), rtol=tol, atol=tol * 1e-2), (rows, d)
        h, y = oracle.rms_norm(x, dtype, w, residual=res)
        hf = rnd(xf + oracle.to_f32(res, dtype))
        assert np.array_equal(oracle.to_f32(h, dtype), hf)
        assert np.allclose(oracle.to_f32(y, dtype), norm(hf), rtol=tol, atol=tol * 1e-2), (rows, d)
        # without a weight: the scaled input, rounded once
        got = oracle.to_f32(oracle.rms_norm(x, dtype), dtype)
        n = np.float32(1) / np.sqrt((xf.astype(np.float64) ** 2).mean(-1, keepdims=True).astype(np.float32) + np.float32(1e-5))
        assert np.allclose(got, rnd(xf * n), rtol=tol, atol=tol * 1e-2)


@pytest.mark.gpu
@pytest.mark.parametrize("dt", list(DT))
def test_cuda_rms_norm_matches_the_oracle_bit_for_bit(dt):
    import nuvec_b200 as nv
    dtype = DT[dt]
    code = {"f32": nv.F32, "f16": nv.F16, "bf16": nv.BF16}[dt]
    dev = nv.Device.shared(0)
    rng = np.random.default_rng(42)
    up_ = lambda a: dev.array(a.view(np.float16) if dt == "f16" else a, code)
    bits = lambda a: a.view(np.uint32) if dt == "f32" else a.view(np.uint16)
    for rows, d in [(3, 64), (1, 4096), (5, 37), (1, 8), (4, 5), (512, 2048), (64, 12288), (2, 40000)]:
        x = oracle.from_f32(rng.standard_normal((rows, d)).astype(np.float32) * 2.0, dtype)
        w = oracle.from_f32(rng.standard_normal(d).astype(np.float32), dtype)
        res = oracle.from_f32(rng.standard_normal((rows, d)).astype(np.float32), dtype)
        want = oracle.rms_norm(x, dtype, w, eps=1e-6)
        got = nv.rms_norm(up_(x), up_(w), 1e-6).to_numpy()
        assert np.array_equal(bits(got), bits(want)), (rows, d)
        assert np.array_equal(bits(nv.rms_norm(up_(x)).to_numpy()), bits(oracle.rms_norm(x, dtype))), (rows, d)
        wh, wy = oracle.rms_norm(x, dtype, w, eps=1e-6, residual=res)
        gh, gy = nv.add_rms_norm(up_(x), up_(res), up_(w), 1e-6)
        assert np.array_equal(bits(gh.to_numpy()), bits(wh)) and np.array_equal(bits(gy.to_numpy()), bits(wy)), (rows, d)
    with pytest.raises(nv.UnsupportedError):
        nv.rms_norm(dev.empty((1, 60000), code))


@pytest.mark.gpu
@pytest.mark.parametrize("tokens", [3, 96])
def test_a_mixture_of_experts_layer_end_to_end(tokens):
    # The layer as nuvec-lm runs it (MoeMlp / SwitchGlu::forward, crates/nuvec-lm/src/model.rs:2160-2210):
    # router top-k, sort by expert, the activations by sorted pair, gate and up products, SwiGLU, down
    # product, the experts' biases, back into pair order, weighted sum -- every step on the device, against
    # the same steps through the oracle.  3 tokens take the per-row gather, 96 the sorted, grouped one.
    import nuvec_b200 as nv
    dev = nv.Device.shared(0)
    rng = np.random.default_rng(50 + tokens)
    E, k, D, I, gs, bits = 8, 2, 128, 192, 64, 4
    quant = nv.Quant.affine(gs, bits)
    bf = lambda a: oracle.from_f32(np.asarray(a, np.float32), oracle.BF16)
    x = bf(rng.standard_normal((tokens, D)))
    logits = rng.standard_normal((tokens, E)).astype(np.float32)
    probs = np.exp(logits - logits.max(-1, keepdims=True))
    probs = bf(probs / probs.sum(-1, keepdims=True))
    experts = {}
    for name, n_out, n_in in (("gate", I, D), ("up", I, D), ("down", D, I)):
        w = bf(rng.standard_normal((E, n_out, n_in)) * 0.05)
        experts[name] = oracle.quantize(w, oracle.BF16, oracle.AFFINE, gs, bits)
    bias = bf(rng.standard_normal((E, D)) * 0.1)

    # the oracle's layer
    idx, scores = oracle.moe_route(probs, oracle.BF16, k, True)
    order, restore, toks, srt, offsets = oracle.moe_sort(idx, E)
    rows = x[toks][:, None, :]                                  # [pairs, 1, D]
    lhs = np.arange(tokens * k, dtype=np.uint32)
    prod = lambda name, a: oracle.gather_qmm(a, *experts[name], lhs, srt, oracle.BF16, oracle.AFFINE, gs, bits)
    h = oracle.swiglu(prod("gate", rows), prod("up", rows), oracle.BF16)
    y = oracle.expert_bias_add(prod("down", h).reshape(tokens * k, D), bias, srt, oracle.BF16)
    want = oracle.weighted_sum(y[restore].reshape(tokens, k, D), scores, oracle.BF16)

    # the same on the device
    up = lambda a, code=nv.BF16: dev.array(a, code)
    q = {name: nv.Quantized(up(c, nv.U32), up(s), up(b), quant) for name, (c, s, b) in experts.items()}
    d_idx, d_scores = nv.moe_route(up(probs), k, True)
    d_order, d_restore, d_toks, d_srt, d_offsets = nv.moe_sort(d_idx, E)
    assert np.array_equal(d_srt.to_numpy(), srt) and np.array_equal(d_restore.to_numpy(), restore)
    d_rows = nv.take_rows(up(x), d_toks).reshape((tokens * k, 1, D))
    opts = nv.GatherQmm().with_sorted_indices(True)
    dprod = lambda name, a: nv.gather_qmm(a, q[name], None, d_srt, opts, d_offsets)
    d_h = nv.swiglu(dprod("gate", d_rows), dprod("up", d_rows))
    d_y = nv.expert_bias_add(dprod("down", d_h).reshape((tokens * k, D)), up(bias), d_srt)
    got = nv.weighted_sum(nv.take_rows(d_y, d_restore).reshape((tokens, k, D)), d_scores).to_numpy().view(np.uint16)

    g32, w32 = oracle.to_f32(got, oracle.BF16), oracle.to_f32(want, oracle.BF16)
    # products agree within one output rounding; three of them in a row, an activation and a
    # weighted sum in between: a few bfloat16 units of the row's largest magnitude
    bound = 4.0 * 2.0 ** -7 * np.abs(w32).max(-1, keepdims=True)
    assert np.all(np.abs(g32 - w32) <= bound), float((np.abs(g32 - w32) / bound).max())
    assert (g32 == w32).mean() > 0.5
