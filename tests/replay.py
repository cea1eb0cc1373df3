"""Replays the reference's recorded cases through a backend (the oracle or the CUDA path).

A backend offers ``quantize``, ``dequantize``, ``quantized_matmul`` and ``gather_qmm`` with the
signatures of :class:`OracleBackend`.  The comparison rules are the reference's own:
crates/nuvec-core/tests/common/fixture.rs:1300-1317 for the CPU recording and
crates/nuvec-core/tests/mlx.rs:127-146 for the Metal recording.
"""
from __future__ import annotations

import numpy as np

import oracle
from golden_cases import Case

EPS = {oracle.F16: 2.0 ** -10, oracle.BF16: 2.0 ** -7, oracle.F32: float(np.finfo(np.float32).eps)}


def quant_of(case: Case):
    mode = oracle.MODES[case.p("mode", "affine")]
    gs, bits = {oracle.AFFINE: (64, 4), oracle.MXFP4: (32, 4), oracle.MXFP8: (32, 8),
                oracle.NVFP4: (16, 4)}[mode]
    return mode, int(case.p("group_size", gs)), int(case.p("bits", bits))


class OracleBackend:
    """The CPU oracle, with the batch broadcasting the reference's op layer performs
    (crates/nuvec-core/src/quantized.rs:504-521) done here in numpy."""

    name = "oracle"

    def quantize(self, w, dtype, mode, gs, bits, global_scale=None):
        return oracle.quantize(w, dtype, mode, gs, bits, global_scale)

    def dequantize(self, codes, scales, biases, dtype, mode, gs, bits, global_scale=None,
                   fused=False):
        return oracle.dequantize(codes, scales, biases, dtype, mode, gs, bits, global_scale, fused)

    def quantized_matmul(self, x, codes, scales, biases, dtype, mode, gs, bits, transpose):
        vector = x.ndim == 1
        if vector:
            x = x[None, :]
        bx, bw = x.shape[:-2], codes.shape[:-2]
        batch = np.broadcast_shapes(bx, bw) if bw else bx
        N = codes.shape[-2] if transpose else codes.shape[-1] * 32 // bits
        xb = np.broadcast_to(x, batch + x.shape[-2:]).reshape((-1,) + x.shape[-2:])

        def full(a):
            if a is None:
                return None
            if not bw:
                return np.broadcast_to(a, (xb.shape[0],) + a.shape)
            return np.broadcast_to(a, batch + a.shape[-2:]).reshape((-1,) + a.shape[-2:])

        cb, sb, bb = full(codes), full(scales), full(biases)
        out = np.stack([
            oracle.quantized_matmul(xb[i], cb[i], sb[i], None if bb is None else bb[i], dtype,
                                    mode, gs, bits, transpose)
            for i in range(xb.shape[0])]) if xb.shape[0] else np.zeros((0, x.shape[-2], N), oracle.store_dtype(dtype))
        out = out.reshape(batch + (x.shape[-2], N))
        return out[0] if vector else out

    def gather_qmm(self, x, codes, scales, biases, lhs, rhs, dtype, mode, gs, bits, transpose,
                   global_scale=None, sorted_indices=False):
        M, K = x.shape[-2:]
        xf = x.reshape((-1, M, K))
        cf = codes.reshape((-1,) + codes.shape[-2:])
        sf = scales.reshape((-1,) + scales.shape[-2:])
        bf = None if biases is None else biases.reshape((-1,) + biases.shape[-2:])
        if lhs is None:
            lhs = np.arange(xf.shape[0], dtype=np.uint32).reshape(x.shape[:-2])
        if rhs is None:
            rhs = np.arange(cf.shape[0], dtype=np.uint32).reshape(codes.shape[:-2])
        lhs, rhs = np.broadcast_arrays(np.asarray(lhs), np.asarray(rhs))
        y = oracle.gather_qmm(xf, cf, sf, bf, lhs.reshape(-1), rhs.reshape(-1), dtype, mode, gs,
                              bits, transpose, global_scale)
        return y.reshape(lhs.shape + y.shape[-2:])


def _f64(t_or_arr, dtype):
    return oracle.to_f32(t_or_arr, dtype).astype(np.float64)


def run_case(case: Case, be):
    """Runs one recorded case; returns the list of outputs (numpy storage arrays)."""
    mode, gs, bits = quant_of(case)
    xs = case.inputs
    if case.op == "quantize":
        w, dt = xs[0].data, xs[0].dtype
        if case.p("pre") == "t":
            w = np.ascontiguousarray(np.swapaxes(w, -1, -2))
        elif case.p("pre") == "r":
            w = np.ascontiguousarray(w[..., ::-1])
        g = xs[1].data if case.p("gs") == "1" else None
        codes, scales, biases = be.quantize(w, dt, mode, gs, bits, g)
        return [codes, scales] + ([biases] if biases is not None else [])
    if case.op == "dequantize":
        if mode == oracle.AFFINE:
            dt = xs[1].dtype
            fused = case.name.startswith("gpu:")  # the Metal recording rounds once
            return [be.dequantize(xs[0].data, xs[1].data, xs[2].data, dt, mode, gs, bits,
                                  fused=fused)]
        dt = int(case.p("dtype", "10"))
        g = xs[2].data if case.p("gs") == "1" else None
        return [be.dequantize(xs[0].data, xs[1].data, None, dt, mode, gs, bits, g)]
    if case.op == "quantized_matmul":
        b = xs[3].data if len(xs) > 3 else None
        return [be.quantized_matmul(xs[0].data, xs[1].data, xs[2].data, b, xs[0].dtype, mode, gs,
                                    bits, case.p("transpose") == "1")]
    if case.op == "gather_qmm":
        rest = list(xs[3:])
        g = rest.pop(0).data if case.p("gs") == "1" else None
        lhs = rest.pop(0).data if "l" in case.p("idx") else None
        rhs = rest.pop(0).data if "r" in case.p("idx") else None
        return [be.gather_qmm(xs[0].data, xs[1].data, xs[2].data, None, lhs, rhs, xs[0].dtype,
                              mode, gs, bits, case.p("transpose") == "1", g,
                              case.p("sorted") == "1")]
    raise ValueError(case.op)


def exact_ops(case: Case) -> bool:
    return case.op in ("quantize", "dequantize")


def check_case(case: Case, be):
    """Raises AssertionError when the backend's outputs leave the reference's bounds."""
    got = run_case(case, be)
    assert len(got) == len(case.outputs), case.name
    for g, e in zip(got, case.outputs):
        g = np.asarray(g)
        assert g.shape == e.data.shape, (case.name, g.shape, e.data.shape)
        if exact_ops(case):
            if e.dtype in EPS:  # compare bit patterns, NaNs included
                same = g.view(np.uint8).tobytes() == e.data.view(np.uint8).tobytes()
                if not same:
                    gv, ev = _f64(g, e.dtype), _f64(e.data, e.dtype)
                    bad = np.flatnonzero(~((gv == ev) | (np.isnan(gv) & np.isnan(ev))).reshape(-1)
                                         | (g.reshape(-1).view(e.data.dtype) != e.data.reshape(-1)))
                    raise AssertionError(f"{case.name}: {bad.size} of {g.size} values differ, "
                                         f"first at {bad[0]}: {gv.reshape(-1)[bad[0]]} vs "
                                         f"{ev.reshape(-1)[bad[0]]}")
            else:
                assert np.array_equal(g, e.data), f"{case.name}: integer output differs"
            continue
        gv, ev = _f64(g, e.dtype), _f64(e.data, e.dtype)
        if case.name.startswith("cpu:"):
            # fixture.rs:1309-1317
            mode, gs, bits = quant_of(case)
            bound = lambda t: max(1.0, float(np.abs(_f64(t.data, t.dtype)).max(initial=0.0)))
            k = case.inputs[0].data.shape[-1]
            w = bound(case.inputs[2]) * ((1 << bits) - 1) + bound(case.inputs[3])
            tol = 4.0 * (k + 1.0) * EPS[e.dtype] * bound(case.inputs[0]) * w
            err = np.abs(gv - ev)
            assert np.all((err <= tol) | (gv == ev)), f"{case.name}: max err {err.max()} > {tol}"
        else:
            # mlx.rs:127-146
            atol, rtol = {oracle.F32: (1e-5, 1e-4), oracle.F16: (1e-3, 5e-3)}.get(e.dtype, (1e-2, 4e-2))
            scale = max(1.0, float(np.abs(ev).max(initial=0.0)))
            err = np.abs(gv - ev)
            lim = atol * scale + rtol * np.abs(ev)
            assert np.all(err <= lim), f"{case.name}: max excess {(err - lim).max()}"
