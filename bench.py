#!/usr/bin/env python3
"""Benchmark of the quantized-matmul path: decode (qmv, weight GB/s) and prefill (qmm, TFLOP/s).

    python bench.py --gpus N --steps K --warmup W [--impl reference] [--workload decode|prefill]

One "step" of the default workload is one decode token through the quantized projections of a
Qwen3-8B-shaped model (36 layers x {qkv, o, gate+up, down}, affine 4-bit, groups of 64, M = 1):
144 few-row products streaming 3.9 GB of packed weights, far more than L2, so every launch
reads its weights from HBM.  On N GPUs each projection is split along its output rows; every
rank multiplies its slice and the slices are joined by an all-gather (NCCL) on the same stream.

The JSON line printed by rank 0 carries:
  value       whole-job weight GB/s with inputs resident in HBM (device-timed, max over ranks)
  roofline    the qmv kernel against the measured HBM copy bandwidth
  e2e         the same metric through the host-operand entry point (pinned H2D of x, D2H of y
              inside the timed region)
  cpu_baseline  the CPU port of the reference's path, timed on this host on a bounded sample
  also        the prefill product (M = 2048, K = 4096, N = 12288) in TFLOP/s with its roofline

`--impl reference` times the reference's CPU algorithm (the oracle port; the reference itself
is Rust and cannot be built with this toolchain) on the same workload, one layer per step.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import statistics
import subprocess
import sys
import threading
import time
import zlib
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

# Qwen3-8B projection shapes (N out, K in): qkv, o, gate+up, down.
PROJECTIONS = [("qkv", 6144, 4096), ("o", 4096, 4096), ("gate_up", 24576, 4096), ("down", 4096, 12288)]
# Rows of the fused projections' segments (q | k | v with 32 query and 8 key/value heads of 128; gate | up):
# a rank of an N-sharded step holds its share of every segment (nuvec_b200.shard.parts).
SEGMENTS = {"qkv": [4096, 1024, 1024], "o": [4096], "gate_up": [12288, 12288], "down": [4096]}
LAYERS = 36
GS, BITS = 64, 4
PREFILL = (2048, 12288, 4096)  # M, N, K
# DRAM bytes (read + write) of one launch of the few-row kernel on each projection at M = 1, from an
# ncu capture of three launches per shape on distinct weight copies (profiles/qmv_dram_traffic_decode.md):
# within 0.6 % of the algorithmic bytes, i.e. every weight byte crosses HBM once.
NCU_DRAM_BYTES = {"qkv": 14.24e6, "o": 9.52e6, "gate_up": 56.84e6, "down": 28.41e6}


def qmv_bytes(M, N, K, bits=BITS, gs=GS, s=4):
    """Algorithmic bytes of one few-row product: packed weights + scales/biases + x + y."""
    return N * K * bits // 8 + N * (K // gs) * s + M * K * 2 + M * N * 2


def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons through NVML while the timed region runs (a thread
    polling every few milliseconds, so that even a timed region of tens of milliseconds is seen);
    falls back to an nvidia-smi loop when the NVML binding is missing."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    NAMES = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]

    def __init__(self, index: int):
        self.index, self.rows, self.proc, self.nvml, self.thread = index, [], None, None, None
        self.running = False

    def start(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            self.handle = pynvml.nvmlDeviceGetHandleByIndex(self.index)
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM))
            self.nvml = pynvml
            self.running = True
            self.thread = threading.Thread(target=self._poll, daemon=True)
            self.thread.start()
            return
        except Exception:
            self.nvml = None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                                          "-i", str(self.index), "-lms", "100"], stdout=subprocess.PIPE, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _poll(self):
        n = self.nvml
        bits = {"hw_slowdown": n.nvmlClocksEventReasonHwSlowdown, "hw_thermal_slowdown": n.nvmlClocksEventReasonHwThermalSlowdown,
                "sw_thermal_slowdown": n.nvmlClocksEventReasonSwThermalSlowdown, "sw_power_cap": n.nvmlClocksEventReasonSwPowerCap}
        while self.running:
            try:
                mhz = float(n.nvmlDeviceGetClockInfo(self.handle, n.NVML_CLOCK_SM))
                get = getattr(n, "nvmlDeviceGetCurrentClocksEventReasons", None) or n.nvmlDeviceGetCurrentClocksThrottleReasons
                mask = int(get(self.handle))
                self.rows.append([str(mhz), str(self.max_mhz)] +
                                 ["Active" if mask & bits[k] else "Not Active" for k in self.NAMES])
            except Exception:
                pass
            time.sleep(0.004)

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self) -> dict:
        if self.nvml is not None:
            self.running = False
            self.thread.join(timeout=1.0)
        elif self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        else:
            time.sleep(0.15)
            self.proc.terminate()
        mhz = [float(r[0]) for r in self.rows if r and r[0].replace(".", "").isdigit()]
        mx = [float(r[1]) for r in self.rows if len(r) > 1 and r[1].replace(".", "").isdigit()]
        reasons = sorted({n for r in self.rows if len(r) >= 6 for n, v in zip(self.NAMES, r[2:6]) if v.lower() == "active"})
        return {"sm_mhz": statistics.median(mhz) if mhz else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(mhz), "source": "nvml" if self.nvml is not None else "nvidia-smi"}


# ── CPU arm: the oracle port of the reference's CPU path ────────────────────────────────────
def cpu_layer_inputs(seed=0):
    import oracle
    rng = np.random.default_rng(seed)
    out = []
    for name, N, K in PROJECTIONS:
        w = oracle.from_f32((rng.standard_normal((N, K), dtype=np.float32) * 0.02), oracle.BF16)
        codes, scales, biases = oracle.quantize(w, oracle.BF16, oracle.AFFINE, GS, BITS)
        x = oracle.from_f32(rng.standard_normal((1, K), dtype=np.float32), oracle.BF16)
        out.append((name, N, K, x, codes, scales, biases))
    return out


def use_all_host_threads():
    """The CPU arm runs on every core of this host, whatever OMP_NUM_THREADS the launcher exported
    (torchrun sets it to 1); returns the thread count used."""
    import oracle
    oracle.set_threads(os.cpu_count() or 1)
    return oracle.threads()


def time_cpu_layer(inputs, reps, parallel_dequant=False):
    """Seconds per layer (4 projections, M = 1) through the oracle's quantized_matmul: the
    reference's serial dequantize (kernels.rs:852-856) by default, all threads with
    `parallel_dequant`; the few-row product runs over all threads either way."""
    import oracle
    best = float("inf")
    for _ in range(reps):
        t0 = time.perf_counter()
        for _, _, _, x, codes, scales, biases in inputs:
            oracle.quantized_matmul(x, codes, scales, biases, oracle.BF16, oracle.AFFINE, GS, BITS, True,
                                    parallel_dequant=parallel_dequant)
        best = min(best, time.perf_counter() - t0)
    return best


def reference_arm(args):
    """`--impl reference`: the reference's CPU algorithm on this host (rank 0 only)."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    threads = use_all_host_threads()
    inputs = cpu_layer_inputs()
    layer_bytes = sum(qmv_bytes(1, N, K) for _, N, K in PROJECTIONS)
    # A step of this arm is the bounded sample it really runs: one layer of the token (a whole token
    # is 36 such layers and would take minutes on the CPU).  `ms_per_step` is the measured time of
    # that sample; `value` is a rate, so it compares with the GPU arm's directly.
    for _ in range(max(args.warmup, 0)):
        time_cpu_layer(inputs, 1)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        time_cpu_layer(inputs, 1)
    dt = (time.perf_counter() - t0) / max(args.steps, 1)
    value = layer_bytes / dt / 1e9
    par = layer_bytes / time_cpu_layer(inputs, 1, parallel_dequant=True) / 1e9
    sample = ("one layer (qkv, o, gate+up, down at M=1) per step: 1/36 of the GPU arm's step; serial dequantize as "
              "the reference (kernels.rs:852-856), few-row product over all threads")
    config = dict(workload_config(args.gpus), sample=sample)
    line = {"impl": "reference", "metric": "quantized_matmul weight GB/s (M=1)", "value": value, "unit": "GB/s",
            "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": config,
            "cpu_baseline": {"value": value, "unit": "GB/s", "cores": threads, "kind": "port", "sample": sample,
                             "host_cores": os.cpu_count(), "value_parallel_dequantize": par,
                             "note": "value_parallel_dequantize: the same layer with the dequantize spread over all "
                                     "threads, which the reference does not do"},
            "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line))


def workload_config(gpus):
    return {"workload": "qwen3-8b decode projections, M=1, affine 4-bit g64, 36 layers x (qkv 4096->6144, o 4096->4096, "
                        "gate+up 4096->24576, down 12288->4096)",
            "parallelism": f"N-sharded x{gpus} (each rank its share of every q|k|v and gate|up segment) + all_gather" if gpus > 1 else "single GPU",
            "l2": "inputs larger than L2 (3.9 GB of weights per step, 108 MB per layer)",
            "weights": "one seeded layer (W ~ N(0, 0.02) -> bf16 -> nuvec quantize) replicated into 36 distinct buffers"}


# ── parity of what is timed, checked on the bench's own arrays before any timing ────────────
def product_error(got, want):
    """Worst |got - want| / (1e-2 * ||row||_inf) over the rows of a bfloat16 product (<= 1 passes)."""
    import oracle
    g = oracle.to_f32(got, oracle.BF16).astype(np.float64)
    w = oracle.to_f32(want, oracle.BF16).astype(np.float64)
    bound = 1e-2 * np.abs(w).max(axis=1, keepdims=True) + 1e-30
    return float((np.abs(g - w) / bound).max())


def check_products(nv, lib, dev, qc, cases, what):
    """Every case (name, M, q, x): random rows against the oracle's product within the stated
    1e-2 * ||row||_inf, on all output rows when M <= 8 and on a subset otherwise, and unit-vector
    rows bit for bit against the oracle's dequantize.  Raises SystemExit on the first difference."""
    import oracle
    rng = np.random.default_rng(4242)
    worst = 0.0
    for name, M, q, x in cases:
        n, K = q.weight.shape[0], x.shape[-1]
        c = q.weight.to_numpy()
        s = q.scales.to_numpy().view(np.uint16)
        b = q.biases.to_numpy().view(np.uint16)
        xh = x.to_numpy().view(np.uint16).reshape(M, K)
        y = dev.empty((M, n), nv.BF16)

        def run(xa):
            rc = lib.nvc_quantized_matmul(dev._h, C.byref(qc), nv.BF16, 1, xa.ptr, q.weight.ptr, q.scales.ptr,
                                          q.biases.ptr, None, M, n, K, K, 1, 0, 0, 0, y.ptr)
            assert rc == 0
            return y.to_numpy().view(np.uint16).reshape(M, n)

        got = run(x)
        rows = np.arange(n) if M <= 8 else np.sort(rng.permutation(n)[:128])
        want = oracle.quantized_matmul(xh, c[rows], s[rows], b[rows], oracle.BF16, oracle.AFFINE, GS, BITS)
        err = product_error(got[:, rows], want)
        worst = max(worst, err)
        if not err <= 1.0:
            raise SystemExit(f"parity check failed: {what} {name}: error {err:.3f} x the bound 1e-2*||row||_inf")
        ks = rng.integers(0, K, M)
        xu = np.zeros((M, K), np.float32)
        xu[np.arange(M), ks] = 1.0
        got = run(dev.array(nv.f32_to_bf16(xu), nv.BF16))
        rows = np.sort(rng.permutation(n)[:min(n, 512)])
        dense = oracle.dequantize(c[rows], s[rows], b[rows], oracle.BF16, oracle.AFFINE, GS, BITS)
        if not np.array_equal(got[:, rows], dense[:, ks].T):
            raise SystemExit(f"parity check failed: {what} {name}: unit-vector rows differ from the oracle's dequantize")
    return worst


# ── GPU arm ────────────────────────────────────────────────────────────────────────────────
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=LAYERS)
    ap.add_argument("--rows", type=int, default=1, help="rows of x per decode product (M)")
    ap.add_argument("--no-prefill", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-check", action="store_true", help="skip the parity check that precedes the timing")
    ap.add_argument("--sweep", action="store_true", help="time every single-GPU configuration of the benchmark definition and print one JSON object")
    ap.add_argument("--no-graph", action="store_true", help="launch every product from the host instead of replaying a recorded step")
    ap.add_argument("--one", default=None, metavar="M,N,K,BITS,COPIES",
                    help="profiling driver: one product shape on COPIES distinct weight sets, each launched twice "
                         "(prints the device time per launch); what the ncu commands under profiles/ run")
    ap.add_argument("--attention", action="store_true",
                    help="diagnostic: decode attention over a quantized KV cache at the reference's benchmark shapes "
                         "(32 query / 8 key heads of 128, groups of 64, 8 and 4 bits, 1K-64K keys)")
    ap.add_argument("--checkpoint", action="store_true",
                    help="diagnostic: device time of the checkpoint-format conversions (AWQ / GPTQ layer, gpt-oss gate/up split) "
                         "at the sizes of the configurations, against the bytes they read and write")
    ap.add_argument("--qqmm", default=None, metavar="M,N,K,COPIES",
                    help="the NVFP4 x NVFP4 product on the block-scaled tensor-core path (nvc_qqmm: activations "
                         "quantized on the way) next to the exact product of the same weights with bfloat16 activations")
    ap.add_argument("--timeline", type=int, default=0, metavar="LAYERS",
                    help="diagnostic: replay a recorded decode step of LAYERS layers on the timeline build of the "
                         "library (python -m nuvec_b200.build --timeline) and print where each product's time goes")
    ap.add_argument("--workload", default="decode", choices=["decode", "moe"],
                    help="moe: the expert-sharded mixture-of-experts products (gather_qmm) on --gpus ranks")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm(args)

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus and world > 1:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")

    import nuvec_b200 as nv
    from nuvec_b200 import _ffi, shard
    if args.timeline:
        from nuvec_b200 import build as nvbuild
        if not nvbuild.TIMELINE_LIB.exists():
            raise SystemExit("build the timeline library first: python -m nuvec_b200.build --timeline")
        _ffi.LIB_PATH = nvbuild.TIMELINE_LIB

    dist = None
    if world > 1:
        import torch
        import torch.distributed as dist
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    dev = nv.Device.shared(local)
    lib = _ffi.lib()
    peaks = measured_peaks()
    if args.sweep:
        if world > 1:
            raise SystemExit("--sweep runs on one GPU")
        print(json.dumps({"sweep": config_sweep(nv, _ffi, dev, peaks), "peaks": peaks}))
        return
    if args.one:
        return one_shape(args, nv, _ffi, dev)
    if args.attention:
        return attention_shapes(nv, dev, peaks)
    if args.checkpoint:
        return checkpoint_conversions(nv, dev, peaks)
    if args.qqmm:
        return qqmm_shape(args, nv, _ffi, dev, peaks)
    if args.timeline:
        return timeline(args, nv, _ffi, dev)
    if args.workload == "moe":
        return moe_bench(args, nv, _ffi, shard, dev, dist, rank, world, peaks)
    M = args.rows

    # ── weights: one seeded layer, quantized on the device, replicated into distinct buffers ──
    rng = np.random.default_rng(0)
    quant = nv.Quant.affine(GS, BITS)
    layers = []
    base = []
    for name, N, K in PROJECTIONS:
        assert N % world == 0
        n_local = N // world
        w = shard.shard_rows(rng.standard_normal((N, K), dtype=np.float32) * 0.02, world, rank, SEGMENTS[name])
        q = nv.quantize(dev.array(nv.f32_to_bf16(w), nv.BF16), quant)
        x = dev.array(nv.f32_to_bf16(rng.standard_normal((M, K), dtype=np.float32)), nv.BF16)
        base.append((name, N, K, n_local, q, x))
    dev.synchronize()
    for layer in range(args.layers):
        projs = []
        for name, N, K, n_local, q, x in base:
            if layer == 0:
                ql = q
            else:
                ql = nv.Quantized(dev.empty(q.weight.shape, nv.U32), dev.empty(q.scales.shape, nv.BF16),
                                  dev.empty(q.biases.shape, nv.BF16), quant)
                ql.weight.copy_from(q.weight), ql.scales.copy_from(q.scales), ql.biases.copy_from(q.biases)
            # [world, M, n_local] gather buffer; this rank's product lands in its own slot.
            y = dev.empty((world, M, n_local), nv.BF16)
            projs.append((name, N, K, n_local, ql, x, y))
        layers.append(projs)
    dev.synchronize()

    qc = quant._c()
    # What the timed region runs, checked first (rank 0's slices): abort instead of timing wrong results.
    parity = None
    if rank == 0 and not args.no_check:
        worst = check_products(nv, lib, dev, qc, [(name, M, q, x) for name, N, K, n_local, q, x in base], "decode")
        parity = {"status": "ok", "worst_error_over_bound": worst,
                  "what": "the step's four products on this rank's arrays: all rows against the oracle within "
                          "1e-2*||row||_inf, unit-vector rows bit for bit against the oracle's dequantize"}

    comm = None
    if world > 1:
        import torch
        ident = torch.zeros(128, dtype=torch.uint8, device="cuda")
        if rank == 0:
            buf = (C.c_uint8 * 128)()
            assert lib.nvc_comm_unique_id(buf) == 0, _ffi.last_error()
            ident = torch.tensor(list(buf), dtype=torch.uint8, device="cuda")
        dist.broadcast(ident, 0)
        idb = (C.c_uint8 * 128)(*ident.cpu().tolist())
        h = C.c_void_p()
        assert lib.nvc_comm_init(dev._h, rank, world, idb, C.byref(h)) == 0, _ffi.last_error()
        comm = h

    # ── fused product + gather over peer stores (the multi-GPU headline; NCCL stays as the check) ──
    fused = None
    if world > 1:
        try:
            RES = 4096
            offsets, at = [], RES
            for projs in layers:
                row = []
                for name, N, K, n_local, q, x, y in projs:
                    row.append(at)
                    at += lib.nvc_gather_footprint(world, M, n_local)
                offsets.append(row)
            # packet areas of the K-sharded products of the paired layout (o and down), one pair per layer
            sum_offsets = []
            for projs in layers:
                row = {}
                for name, N, K, n_local, q, x, y in projs:
                    if name in ("o", "down"):
                        row[name] = at
                        at += lib.nvc_all_sum_footprint(world, M, N)
                sum_offsets.append(row)
            region, handle = C.c_void_p(), (C.c_uint8 * 64)()
            assert lib.nvc_symm_alloc(dev._h, at, C.byref(region), handle) == 0, _ffi.last_error()
            handles = [None] * world
            dist.all_gather_object(handles, bytes(handle))
            bases = (C.c_void_p * world)()
            for r in range(world):
                if r == rank:
                    bases[r] = region.value
                else:
                    hb = (C.c_uint8 * 64).from_buffer_copy(handles[r])
                    ptr = C.c_void_p()
                    assert lib.nvc_symm_open(dev._h, hb, C.byref(ptr)) == 0, _ffi.last_error()
                    bases[r] = ptr.value
            group = C.c_void_p()
            assert lib.nvc_peer_group_create(dev._h, rank, world, bases, at, C.byref(group)) == 0, _ffi.last_error()
            fused = {"region": region, "group": group, "offsets": offsets, "sum_offsets": sum_offsets, "bytes": at}
        except Exception as e:  # no peer access on this box: the NCCL path still runs
            fused = None
            if rank == 0:
                print(f"fused gather unavailable: {e}", file=sys.stderr)

    # Paired layout (the reference's own tensor-parallel pairing, crates/nuvec-nn/src/sharded.rs:84-202,
    # crates/nuvec-lm/src/model/shard.rs:108-145): qkv and gate+up stay N-sharded and feed K-sharded o and down,
    # whose partial products are summed across ranks -- two collectives per layer instead of four.
    paired = None
    if fused is not None:
        prng = np.random.default_rng(0)
        pbase = {}
        for name, N, K in PROJECTIONS:
            wfull = prng.standard_normal((N, K), dtype=np.float32) * 0.02
            prng.standard_normal((M, K), dtype=np.float32)  # keep the stream aligned with the weights drawn above
            if name in ("o", "down"):
                kl = K // world
                qk = nv.quantize(dev.array(nv.f32_to_bf16(np.ascontiguousarray(wfull[:, rank * kl:(rank + 1) * kl])), nv.BF16), quant)
                xk = dev.array(nv.f32_to_bf16(prng.standard_normal((M, kl), dtype=np.float32)), nv.BF16)
                pbase[name] = (qk, xk, kl)
        paired = []
        for layer in range(args.layers):
            row = {}
            for name, (qk, xk, kl) in pbase.items():
                ql = nv.Quantized(dev.empty(qk.weight.shape, nv.U32), dev.empty(qk.scales.shape, nv.BF16),
                                  dev.empty(qk.biases.shape, nv.BF16), quant)
                ql.weight.copy_from(qk.weight), ql.scales.copy_from(qk.scales), ql.biases.copy_from(qk.biases)
                N = qk.weight.shape[0]
                row[name] = (ql, xk, kl, dev.empty((M, N), nv.BF16))
            paired.append(row)
        dev.synchronize()

    def step_paired():
        for projs, sums, row in zip(layers, fused["sum_offsets"], paired):
            for name, N, K, n_local, q, x, y in projs:
                if name in row:
                    ql, xk, kl, yk = row[name]
                    rc = lib.nvc_quantized_matmul_all_sum(dev._h, fused["group"], C.byref(qc), xk.ptr, ql.weight.ptr, ql.scales.ptr,
                                                          ql.biases.ptr, M, N, kl, yk.ptr, sums[name])
                else:  # N-sharded, its slice stays on this rank
                    slot = C.c_void_p(y.ptr.value + rank * M * n_local * 2)
                    rc = lib.nvc_quantized_matmul(dev._h, C.byref(qc), nv.BF16, 1, x.ptr, q.weight.ptr, q.scales.ptr,
                                                  q.biases.ptr, None, M, n_local, K, K, 1, 0, 0, 0, slot)
                assert rc == 0, _ffi.last_error()

    def step_fused():
        for projs, offs in zip(layers, fused["offsets"]):
            for (name, N, K, n_local, q, x, y), off in zip(projs, offs):
                rc = lib.nvc_quantized_matmul_gather(dev._h, fused["group"], C.byref(qc), x.ptr, q.weight.ptr, q.scales.ptr,
                                                     q.biases.ptr, M, n_local, K, off)
                assert rc == 0, _ffi.last_error()

    def step(gather=True):
        for projs in layers:
            for name, N, K, n_local, q, x, y in projs:
                slot = C.c_void_p(y.ptr.value + rank * M * n_local * 2)
                rc = lib.nvc_quantized_matmul(dev._h, C.byref(qc), nv.BF16, 1, x.ptr, q.weight.ptr, q.scales.ptr,
                                              q.biases.ptr, None, M, n_local, K, K, 1, 0, 0, 0, slot)
                assert rc == 0, _ffi.last_error()
                if comm is not None and gather:
                    rc = lib.nvc_all_gather(comm, slot, y.ptr, M * n_local * 2)
                    assert rc == 0, _ffi.last_error()

    def barrier():
        dev.synchronize()
        if dist is not None:
            import torch
            dist.barrier()
            torch.cuda.synchronize()

    def timed(fn, steps):
        barrier()
        e0, e1 = dev.event(), dev.event()
        l0 = dev.launches
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        e1.synchronize()
        barrier()
        ms = e0.elapsed_ms(e1)
        if dist is not None:
            import torch
            t = torch.tensor([ms], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms, dev.launches - l0

    # The step is recorded once and replayed: 144 launches of a few microseconds each would
    # otherwise be bound by the host's launch rate, not by the GPU.
    step()
    graph = dev.record(step) if not args.no_graph else None
    run = graph.launch if graph is not None else step
    for _ in range(args.warmup):
        run()
    nccl_ms = None
    fused_check = None
    if fused is not None:
        # The NCCL variant is timed first (it is also what the fused result is checked against).
        nccl_ms, _ = timed(run, args.steps)
        step_fused()
        dev.synchronize()
        # every rank's region must hold exactly what all_gather delivered
        bad = 0
        for projs, offs in zip(layers[-1:], fused["offsets"][-1:]):
            for (name, N, K, n_local, q, x, y), off in zip(projs, offs):
                got = np.empty((world, M, n_local), np.uint16)
                assert lib.nvc_memcpy_d2h(dev._h, got.ctypes.data_as(C.c_void_p), C.c_void_p(fused["region"].value + off), got.nbytes) == 0
                bad += int(np.count_nonzero(got != y.to_numpy().view(np.uint16).reshape(got.shape)))
        import torch
        t = torch.tensor([bad], device="cuda")
        dist.all_reduce(t)
        fused_check = "ok" if int(t.item()) == 0 else f"{int(t.item())} elements differ from the all_gather result"
        graph_f = dev.record(step_fused) if not args.no_graph else None
        run = graph_f.launch if graph_f is not None else step_fused
        for _ in range(args.warmup):
            run()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    ms, launches = timed(run, args.steps)
    clocks = sampler.stop() if rank == 0 else None
    paired_ms = paired_check = None
    if paired is not None:
        step_paired()
        dev.synchronize()
        # every rank must hold the same bits, and they must be the sum of the ranks' partial products
        bad = 0
        for name, (ql, xk, kl, yk) in paired[-1].items():
            mine = yk.to_numpy().view(np.uint16).astype(np.int64)
            t = torch.tensor(mine, device="cuda")
            lo, hi = t.clone(), t.clone()
            dist.all_reduce(lo, op=dist.ReduceOp.MIN)
            dist.all_reduce(hi, op=dist.ReduceOp.MAX)
            bad += int((lo != hi).sum().item())
            part = nv.quantized_matmul(xk, ql)  # this rank's partial product, rounded to bfloat16
            pf = torch.tensor(nv.bf16_to_f32(part.to_numpy()), device="cuda")
            dist.all_reduce(pf)
            got = torch.tensor(nv.bf16_to_f32(yk.to_numpy()), device="cuda")
            tol = 2e-2 * pf.abs().max()  # partials rounded to bfloat16 before this check's own sum
            bad += int(((got - pf).abs() > tol).sum().item())
        paired_check = "ok" if bad == 0 else f"{bad} elements differ"
        graph_p = dev.record(step_paired) if not args.no_graph else None
        run_p = graph_p.launch if graph_p is not None else step_paired
        for _ in range(args.warmup):
            run_p()
        paired_ms, _ = timed(run_p, args.steps)
    if world > 1:
        step(gather=False)
        graph_k = dev.record(lambda: step(gather=False)) if not args.no_graph else None
        ms_kernel_only, _ = timed(graph_k.launch if graph_k is not None else (lambda: step(gather=False)), args.steps)
    else:
        ms_kernel_only = ms

    step_bytes = args.layers * sum(qmv_bytes(M, N, K) for _, N, K in PROJECTIONS)  # whole job, all ranks
    fused_ms = None
    if fused is not None:
        # Both gathers were timed over the same steps; the headline is the faster one, the other
        # is reported beside it.
        fused_ms = ms
        if fused_check != "ok" or nccl_ms < fused_ms:
            ms = nccl_ms
    per_step_ms = ms / args.steps
    value = step_bytes / (per_step_ms * 1e-3) / 1e9
    n_kernels = args.layers * len(PROJECTIONS)
    # Dominant kernel: the few-row product.  Per launch on this rank: the rank's share of bytes.
    launch_bytes = step_bytes / world / n_kernels
    launch_s = (ms_kernel_only / args.steps) * 1e-3 / n_kernels
    achieved = launch_bytes / launch_s / 1e9
    # ncu's DRAM bytes per launch, averaged over the step's four shapes; a rank of an N-sharded step
    # streams 1/N of every matrix (traffic is proportional to the rows a launch covers)
    traffic = sum(NCU_DRAM_BYTES.values()) / len(NCU_DRAM_BYTES) / world if M == 1 else None
    roofline = {"kernel": "qmv_affine_kernel", "bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"],
                "unit": "GB/s", "frac": achieved / peaks["hbm_gbs"], "traffic": traffic,
                "traffic_note": "dram__bytes_read.sum + dram__bytes_write.sum per launch from one ncu capture per shape "
                                "(profiles/qmv_dram_traffic_decode.md), averaged over the four shapes" +
                                ("" if world == 1 else f", scaled by 1/{world} for this rank's row slice"),
                "peak_source": peaks["source"],
                "avg_launch_us": launch_s * 1e6, "algorithmic_bytes_per_launch": launch_bytes}

    line = {"metric": "quantized_matmul weight GB/s (M=1)", "value": value, "unit": "GB/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": per_step_ms, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": dict(workload_config(world), launch="recorded step replayed (CUDA graph)" if graph is not None else "host launches"),
            "roofline": roofline, "gpu_launches": launches, "clocks": clocks}
    if parity is not None:
        line["parity_check"] = parity["status"]
        line["parity"] = parity
    if world > 1:
        line["kernel_only"] = {"value": step_bytes / (ms_kernel_only / args.steps * 1e-3) / 1e9, "unit": "GB/s",
                               "note": "same step without any gather after the products"}
        if fused is not None:
            if ms == fused_ms:
                line["config"]["parallelism"] = (f"N-sharded x{world}; every product sends its slice into all ranks' gathered "
                                                 "buffers (NVLink peer stores) and flags completion: no collective call")
            line["fused_gather_check"] = fused_check
            line["fused_gather"] = {"value": step_bytes / (fused_ms / args.steps * 1e-3) / 1e9, "unit": "GB/s",
                                    "note": "nvc_quantized_matmul_gather: peer stores + flags inside the product kernel"}
            line["nccl_gather"] = {"value": step_bytes / (nccl_ms / args.steps * 1e-3) / 1e9, "unit": "GB/s",
                                   "note": "nvc_quantized_matmul followed by ncclAllGather"}
            line["config"]["value_is"] = "the faster of fused_gather and nccl_gather (both all-gather layouts, timed over the same steps)"
        if paired_ms is not None:
            line["paired_layout"] = {"value": step_bytes / (paired_ms / args.steps * 1e-3) / 1e9, "unit": "GB/s",
                                     "ms_per_step": paired_ms / args.steps, "check": paired_check,
                                     "note": "the reference's tensor-parallel pairing: N-sharded qkv and gate+up feed K-sharded "
                                             "o and down (nvc_quantized_matmul_all_sum): 72 collectives per step instead of 144"}

    # ── end to end through the host-operand entry point (rank-local x in, y out) ─────────────
    if not args.no_e2e:
        hx = {K: np.ascontiguousarray(nv.f32_to_bf16(rng.standard_normal((M, K), dtype=np.float32))) for _, _, K in PROJECTIONS}

        hy = {(li, name): np.empty((M, n_local), np.uint16) for li, projs in enumerate(layers)
              for name, N, K, n_local, q, x, y in projs}

        items = (_ffi.HostProduct * (len(layers) * len(PROJECTIONS)))()
        i = 0
        for li, projs in enumerate(layers):
            for name, N, K, n_local, q, x, y in projs:
                it = items[i]
                it.quant, it.dtype, it.transpose = qc, nv.BF16, 1
                it.host_x, it.host_y = hx[K].ctypes.data, hy[(li, name)].ctypes.data
                it.w, it.scales, it.biases, it.global_scale = q.weight.ptr.value, q.scales.ptr.value, q.biases.ptr.value, None
                it.M, it.N, it.K = M, n_local, K
                i += 1

        def step_host():
            # the whole token through the host-operand call: every product's activations come from host
            # memory and its result goes back to host memory; the step's products are issued as one
            # list (what an evaluator walking the step's nodes does) and the step waits once
            assert lib.nvc_quantized_matmul_host_batch(dev._h, items, len(items)) == 0, _ffi.last_error()
            assert lib.nvc_synchronize(dev._h) == 0, _ffi.last_error()

        step_host()
        barrier()
        t0 = time.perf_counter()
        e2e_steps = max(3, args.steps // 4)
        for _ in range(e2e_steps):
            step_host()
        barrier()
        wall = (time.perf_counter() - t0) / e2e_steps
        if dist is not None:
            import torch
            t = torch.tensor([wall], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            wall = float(t.item())
        line["e2e"] = {"value": step_bytes / wall / 1e9, "unit": "GB/s",
                       "h2d_bytes_per_step": args.layers * sum(M * K * 2 for _, _, K in PROJECTIONS),
                       "d2h_bytes_per_step": args.layers * sum(M * (N // world) * 2 for _, N, _ in PROJECTIONS),
                       "ms_per_step": wall * 1e3,
                       "note": "nvc_quantized_matmul_host_batch: the step's 144 products as one list of host-operand products (x from "
                               "host memory through a pinned block and an H2D copy, y stored by the kernel into the pinned "
                               "block over PCIe), one nvc_synchronize per step delivers the results into host memory; weights resident"}
        # the results that came back through host memory are the ones the device-resident step computes
        if rank == 0 and not args.no_check:
            name, N, K, n_local, q, x, y = layers[0][0]
            ref = nv.quantized_matmul(dev.array(hx[K], nv.BF16), q).to_numpy().view(np.uint16).reshape(M, n_local)
            if not np.array_equal(ref, hy[(0, name)]):
                raise SystemExit("parity check failed: host-operand result differs from the device-resident product")

    # ── prefill product on tcgen05 (rank 0's view; N-sharded like the decode products) ───────
    if not args.no_prefill:
        line["also"] = [prefill_bench(nv, _ffi, dev, peaks, rank, world, timed, barrier, not args.no_check)]

    # ── the same prefill shape with both operands NVFP4 on the block-scaled path (one GPU) ─────
    if not args.no_prefill and world == 1:
        line["also"].append(qqmm_leg(nv, _ffi, dev, peaks, not args.no_check))

    # ── CPU baseline on this host's cores (rank 0, bounded sample) ───────────────────────────
    if rank == 0 and world == 1 and not args.no_cpu:
        threads = use_all_host_threads()
        inputs = cpu_layer_inputs()
        secs = time_cpu_layer(inputs, 3)
        secs_par = time_cpu_layer(inputs, 2, parallel_dequant=True)
        layer_bytes = sum(qmv_bytes(1, N, K) for _, N, K in PROJECTIONS)
        line["cpu_baseline"] = {"value": layer_bytes / secs / 1e9, "unit": "GB/s", "cores": threads,
                                "kind": "port", "host_cores": os.cpu_count(),
                                "sample": "one layer (4 products, M=1), best of 3; serial dequantize as the reference, "
                                          "few-row product over all threads", "seconds_per_layer": secs,
                                "value_parallel_dequantize": layer_bytes / secs_par / 1e9,
                                "note": "value_parallel_dequantize: the same layer with the dequantize spread over all "
                                        "threads, which the reference does not do"}
    if rank == 0:
        print(json.dumps(line), flush=True)
    # Multi-rank runs leave without tearing down: the ranks meet at a barrier and exit.  (Destroying
    # the recorded steps and the two NCCL instances of this process in the interpreter's teardown
    # was observed to block; the work is complete and its results are printed at this point.)
    dev.synchronize()
    if world > 1:
        dist.barrier()
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(0)


# ── profiling driver (--one) ─────────────────────────────────────────────────────────────────
def one_shape(args, nv, _ffi, dev):
    """One product shape on several distinct weight sets (random codes, scales and biases in the range
    quantizing N(0, 0.02) weights gives), every set launched twice: launches COPIES + 1 .. 2 COPIES run
    on weights that left L2 long ago.  Used under ncu with -k / -s / -c."""
    M, N, K, bits, copies = (int(v) for v in args.one.split(","))
    lib = _ffi.lib()
    rng = np.random.default_rng(0)
    quant = nv.Quant.affine(GS, bits)
    qc = quant._c()
    codes = rng.integers(0, 2 ** 32, (N, K * bits // 32), dtype=np.uint32)
    sc = nv.f32_to_bf16((rng.random((N, K // GS), dtype=np.float32) * 0.06 + 0.03) / float(2 ** bits - 1))
    bi = nv.f32_to_bf16(-(rng.random((N, K // GS), dtype=np.float32) * 0.04 + 0.02))
    x = dev.array(nv.f32_to_bf16(rng.standard_normal((M, K), dtype=np.float32)), nv.BF16)
    sets = [(dev.array(codes, nv.U32), dev.array(sc, nv.BF16), dev.array(bi, nv.BF16), dev.empty((M, N), nv.BF16))
            for _ in range(copies)]
    dev.synchronize()
    e0, e1 = dev.event(), dev.event()
    for rnd in range(2):
        if rnd == 1:
            e0.record()
        for c, s, b, y in sets:
            rc = lib.nvc_quantized_matmul(dev._h, C.byref(qc), nv.BF16, 1, x.ptr, c.ptr, s.ptr, b.ptr, None, M, N, K, K, 1, 0, 0, 0, y.ptr)
            assert rc == 0, _ffi.last_error()
    e1.record()
    e1.synchronize()
    out = {"one": args.one, "launches": 2 * copies, "us_per_launch": e0.elapsed_ms(e1) * 1e3 / copies,
           "bytes_per_launch": qmv_bytes(M, N, K, bits)}
    if args.timeline and M > 8:
        # the timeline build of the tensor-core kernel: cycles per role of blocks 0 and 1 in the last launch
        # (total, then the role's waits in program order)
        buf = (C.c_longlong * (2 * 8 * 6))()
        lib.nvc_debug_qmm_timing.restype = C.c_int32
        assert lib.nvc_debug_qmm_timing(buf) == 0
        t = np.frombuffer(buf, dtype=np.int64).reshape(2, 8, 6)
        roles = ["activation producer", "mma issuer", "watcher", "dequantizers 0", "dequantizers 1", "dequantizers 2",
                 "dequantizers 3", "epilogue"]
        out["role_cycles"] = {f"block {b}": {r: t[b, i].tolist() for i, r in enumerate(roles)} for b in range(2)}
    print(json.dumps(out))


# ── NVFP4 x NVFP4 on the block-scaled path (--qqmm) ─────────────────────────────────────────
def qqmm_shape(args, nv, _ffi, dev, peaks):
    """nvc_qqmm (quantize x, lay out the scales, block-scaled MMA) and, beside it, nvc_quantized_matmul of
    the same NVFP4 weights with bfloat16 activations (weights dequantized exactly into tensor memory), on
    COPIES distinct weight sets; device time per product from CUDA events."""
    M, N, K, copies = (int(v) for v in args.qqmm.split(","))
    lib = _ffi.lib()
    rng = np.random.default_rng(0)
    quant = nv.Quant(nv.QuantMode("nvfp4"), 16, 4)
    qc = quant._c()
    codes = rng.integers(0, 2 ** 32, (N, K // 8), dtype=np.uint32)
    scales = rng.integers(0x08, 0x30, (N, K // 16), dtype=np.uint8)
    x = dev.array(nv.f32_to_bf16(rng.standard_normal((M, K), dtype=np.float32)), nv.BF16)
    sets = [(dev.array(codes, nv.U32), dev.array(scales, nv.U8), dev.empty((M, N), nv.BF16)) for _ in range(copies)]
    dev.synchronize()

    def timed(call):
        e0, e1 = dev.event(), dev.event()
        for rnd in range(3):
            if rnd == 1:
                e0.record()
            for c, s, y in sets:
                assert call(c, s, y) == 0, _ffi.last_error()
        e1.record()
        e1.synchronize()
        return e0.elapsed_ms(e1) * 1e3 / (2 * copies)
    us_qq = timed(lambda c, s, y: lib.nvc_qqmm(dev._h, C.byref(qc), nv.BF16, x.ptr, c.ptr, s.ptr, M, N, K, y.ptr))
    lib.nvc_qqmm_scales_bytes.restype = C.c_size_t
    laid = []
    for c, sc, y in sets:
        buf = dev.empty((lib.nvc_qqmm_scales_bytes(C.byref(qc), N, K),), nv.U8)
        assert lib.nvc_qqmm_prepare_scales(dev._h, C.byref(qc), sc.ptr, N, K, buf.ptr) == 0, _ffi.last_error()
        laid.append(buf)
    by_codes = {c.ptr.value: b for (c, _, _), b in zip(sets, laid)}
    us_prep = timed(lambda c, s, y: lib.nvc_qqmm_prepared(dev._h, C.byref(qc), nv.BF16, x.ptr, c.ptr, by_codes[c.ptr.value].ptr, M, N, K, y.ptr))
    us_exact = timed(lambda c, s, y: lib.nvc_quantized_matmul(dev._h, C.byref(qc), nv.BF16, 1, x.ptr, c.ptr, s.ptr, None, None,
                                                              M, N, K, K, 1, 0, 0, 0, y.ptr))
    flops = 2.0 * M * N * K
    if args.timeline:
        # the timeline build: cycles of block (0, 0) of the last launch, per role
        buf = (C.c_longlong * 12)()
        lib.nvc_debug_qqmm_timing.restype = C.c_int32
        assert lib.nvc_debug_qqmm_timing(buf) == 0
        t = np.array(list(buf)).reshape(3, 4)
        print(json.dumps({"qqmm_role_cycles": {r: {"start": int(t[i, 0]), "end": int(t[i, 1]), "in_waits": int(t[i, 2])}
                                               for i, r in enumerate(["producer", "mma issuer", "epilogue"])}}))
    print(json.dumps({"qqmm": args.qqmm, "us_qqmm": us_qq, "TFLOP/s_qqmm": flops / us_qq / 1e6,
                      "us_qqmm_prepared_scales": us_prep, "TFLOP/s_qqmm_prepared_scales": flops / us_prep / 1e6,
                      "us_exact_bf16_activations": us_exact, "TFLOP/s_exact": flops / us_exact / 1e6,
                      "frac_of_measured_bf16_burst_qqmm": flops / us_qq / 1e6 / peaks["bf16_tflops"],
                      "note": "qqmm includes the quantization of x and the layout of both scale arrays"}))


# ── decode attention over a quantized cache (--attention) ────────────────────────────────────
def _ffi_lib():
    from nuvec_b200 import _ffi
    return _ffi.lib()


def attention_shapes(nv, dev, peaks):
    """nvc_quantized_attention at the shapes of the reference's benchmark (crates/nuvec-core/benches/kv_attention.rs):
    one query row, 32 query and 8 key heads of size 128, groups of 64, 8- and 4-bit caches of 1K to 64K keys; 32
    independent calls (distinct queries) recorded as one step and replayed, device time per call against the cache
    bytes it has to read."""
    rng = np.random.default_rng(0)
    Hq, Hkv, D, gs, calls = 32, 8, 128, 64, 32
    rows = []
    for bits in (8, 4):
        quant = nv.Quant.affine(gs, bits)
        for S in (1024, 4096, 16384, 32768, 65536):
            def side():
                return nv.Quantized(dev.array(rng.integers(0, 2 ** 32, (1, Hkv, S, D * bits // 32), dtype=np.uint32), nv.U32),
                                    dev.array(nv.f32_to_bf16(rng.uniform(0.01, 0.05, (1, Hkv, S, D // gs)).astype(np.float32)), nv.BF16),
                                    dev.array(nv.f32_to_bf16(rng.uniform(-0.4, -0.1, (1, Hkv, S, D // gs)).astype(np.float32)), nv.BF16), quant)
            k, v = side(), side()
            qs = [dev.array(nv.f32_to_bf16(rng.standard_normal((1, Hq, 1, D)).astype(np.float32)), nv.BF16) for _ in range(calls)]
            scale = D ** -0.5
            for q in qs[:4]:
                nv.quantized_attention(q, k, v, scale)
            # the 32 calls as one recorded step (the reference evaluates its 32 calls together), replayed three times
            lib, c = _ffi_lib(), quant._c()
            outs = [dev.empty((1, Hq, 1, D), nv.BF16) for _ in range(calls)]

            def step():
                for q, o in zip(qs, outs):
                    assert lib.nvc_quantized_attention(dev._h, C.byref(c), nv.BF16, q.ptr, k.weight.ptr, k.scales.ptr, k.biases.ptr,
                                                       v.weight.ptr, v.scales.ptr, v.biases.ptr, None, 1, Hq, Hkv, 1, S, D, S, scale, 0,
                                                       o.ptr) == 0
            graph = dev.record(step)
            graph.launch()
            e0, e1 = dev.event(), dev.event()
            e0.record()
            for _ in range(3):
                graph.launch()
            e1.record()
            e1.synchronize()
            us = e0.elapsed_ms(e1) * 1e3 / (3 * calls)
            cache = 2 * (k.weight.nbytes + k.scales.nbytes + k.biases.nbytes)
            rows.append({"bits": bits, "keys": S, "us": us, "cache_GB/s": cache / us / 1e3, "frac_of_measured_hbm": cache / us / 1e3 / peaks["hbm_gbs"],
                         "cache_MB": cache / 1e6})
    print(json.dumps({"quantized_attention": rows, "shape": "1 x 32 query / 8 key heads x 128, groups of 64, bfloat16",
                      "note": "caches up to 16K keys (q8) / 32K keys (q4) fit the 126 MB L2 and are re-read from it by the 32 calls"}))


# ── checkpoint-format conversions (--checkpoint) ───────────────────────────────────────────────
def checkpoint_conversions(nv, dev, peaks):
    """Device time of nvc_convert_packed for one AWQ and one GPTQ layer of the dense configuration's gate+up
    projection (4096 -> 24576, 4-bit, groups of 128) and of the gate / up split of a gpt-oss layer's MXFP4
    experts (32 experts x 5760 rows x 2880), each against the bytes it has to read and write."""
    from nuvec_b200 import checkpoint as ck
    rng = np.random.default_rng(0)
    rows = []

    def timed(fn, reps=10):
        fn()
        e0, e1 = dev.event(), dev.event()
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        e1.synchronize()
        return e0.elapsed_ms(e1) * 1e3 / reps

    inputs, outputs, group = 4096, 24576, 128
    scales = dev.array(rng.uniform(0.001, 0.01, (inputs // group, outputs)).astype(np.float16), nv.F16)
    zeros = dev.array(rng.integers(0, 2 ** 31, (inputs // group, outputs // 8), dtype=np.int32), nv.I32)
    quant = nv.Quant.affine(group, 4)
    for name, fmt, shape in (("awq", ck.AWQ, (inputs, outputs // 8)), ("gptq", ck.GPTQ_V2, (inputs // 8, outputs))):
        qw = dev.array(rng.integers(0, 2 ** 31, shape, dtype=np.int32), nv.I32)
        us = timed(lambda: ck.convert_packed_layer(dev, fmt, quant, qw, scales, zeros, None, name))
        moved = 2 * qw.nbytes + 3 * scales.nbytes + zeros.nbytes
        rows.append({"conversion": f"{name} 4-bit g128 layer {inputs} -> {outputs}", "us": us, "GB/s": moved / us / 1e3,
                     "frac_of_measured_hbm": moved / us / 1e3 / peaks["hbm_gbs"]})
    E, R, K = 32, 5760, 2880
    blocks = dev.array(rng.integers(0, 256, (E, R, K // 32, 16), dtype=np.uint8), nv.U8)
    sc = dev.array(rng.integers(100, 140, (E, R, K // 32), dtype=np.uint8), nv.U8)
    us = timed(lambda: ck.sanitize_gpt_oss({"l.experts.gate_up_proj_blocks": blocks, "l.experts.gate_up_proj_scales": sc}), reps=5)
    moved = 2 * (blocks.nbytes + sc.nbytes)
    rows.append({"conversion": f"gpt-oss gate/up split, {E} experts x {R} rows x {K} (blocks + scales)", "us": us,
                 "GB/s": moved / us / 1e3, "frac_of_measured_hbm": moved / us / 1e3 / peaks["hbm_gbs"],
                 "note": "four nvc_take_strided calls"})
    print(json.dumps({"checkpoint_conversions": rows}))


# ── where a decode product's time goes (--timeline) ──────────────────────────────────────────
def timeline(args, nv, _ffi, dev):
    """Replays a recorded step of args.timeline layers on the library built with -DNUVEC_TIMELINE,
    whose few-row kernel records %globaltimer (minimum and maximum over its blocks) at: block start,
    before / after the dependency wait, activations staged, a warp's last iteration, block end.  All
    figures are relative to the end of the previous product's last block.  The stamps themselves cost
    time (the products run ~30 % longer than in the plain build): read proportions, not absolutes."""
    lib = _ffi.lib()
    lib.nvc_debug_timeline_read.restype = C.c_int32
    lib.nvc_debug_timeline_read.argtypes = [C.c_void_p, C.c_int32]
    lib.nvc_debug_timeline_reset.restype = C.c_int32
    rng = np.random.default_rng(0)
    quant = nv.Quant.affine(GS, BITS)
    qc = quant._c()
    M = args.rows
    prods = []
    for _ in range(args.timeline):
        for name, N, K in PROJECTIONS:
            codes = dev.array(rng.integers(0, 2 ** 32, (N, K * BITS // 32), dtype=np.uint32), nv.U32)
            sc = dev.array(nv.f32_to_bf16(rng.random((N, K // GS), dtype=np.float32) * 0.004 + 0.001), nv.BF16)
            bi = dev.array(nv.f32_to_bf16(-rng.random((N, K // GS), dtype=np.float32) * 0.04), nv.BF16)
            x = dev.array(nv.f32_to_bf16(rng.standard_normal((M, K), dtype=np.float32)), nv.BF16)
            prods.append((name, N, K, codes, sc, bi, x, dev.empty((M, N), nv.BF16)))

    def step():
        for name, N, K, c, s, b, x, y in prods:
            rc = lib.nvc_quantized_matmul(dev._h, C.byref(qc), nv.BF16, 1, x.ptr, c.ptr, s.ptr, b.ptr, None, M, N, K, K, 1, 0, 0, 0, y.ptr)
            assert rc == 0, _ffi.last_error()
    step()
    graph = dev.record(step)
    for _ in range(3):
        graph.launch()
    dev.synchronize()
    assert lib.nvc_debug_timeline_reset() == 0
    graph.launch()
    dev.synchronize()
    n = len(prods)
    buf = (C.c_ulonglong * (12 * n))()
    got = lib.nvc_debug_timeline_read(buf, n)
    assert got == n, f"{got} launches recorded, {n} expected"
    a = np.frombuffer(buf, dtype=np.uint64).reshape(n, 12).astype(np.int64) / 1000.0   # microseconds
    per = {}
    for i in range(1, n):
        start, _, pre_wait_max, wait_ret_max, staged_max, loop_first, loop_last, end_last = \
            a[i, 0], a[i, 1], a[i, 3], a[i, 5], a[i, 7], a[i, 8], a[i, 9], a[i, 11]
        prev_end = a[i - 1, 11]
        per.setdefault(prods[i][0], []).append([
            start - prev_end,            # first block starts (negative: while the previous product runs)
            pre_wait_max - prev_end,     # last block has issued its first weight copies and reaches the wait
            wait_ret_max - prev_end,     # last block's wait returns
            staged_max - wait_ret_max,   # activations staged
            loop_first - staged_max,     # first warp finishes its iterations
            loop_last - staged_max,      # last warp finishes its iterations
            end_last - loop_last,        # partial sums met, results stored
            end_last - prev_end])        # the product's share of the step
    keys = ["first_block_start", "last_block_at_wait", "last_wait_returns", "stage_activations",
            "first_warp_done", "last_warp_done", "tail", "period"]
    out = {name: {k: round(float(v), 2) for k, v in zip(keys, np.median(np.array(rows), axis=0))} for name, rows in per.items()}
    print(json.dumps({"timeline_us": out, "layers": args.timeline, "rows": M,
                      "relative_to": "end of the previous product's last block (median over layers)"}))


# ── expert-sharded mixture of experts (gather_qmm), --workload moe ───────────────────────────
MOE_CONFIGS = [
    # name, experts, top-k, tokens, (projection, N, K) list, quantization
    ("qwen3-30b-a3b", 128, 8, (1, 512), [("gate_up", 1536, 2048), ("down", 2048, 768)], ("affine", 64, 4)),
    ("gpt-oss-20b mxfp4", 32, 4, (1, 1024), [("gate_up", 5760, 2880), ("down", 2880, 2880)], ("mxfp4", 32, 4)),
    ("gpt-oss-20b nvfp4", 32, 4, (1, 1024), [("gate_up", 5760, 2880), ("down", 2880, 2880)], ("nvfp4", 16, 4)),
]


def moe_glue_rows(nv, dev):
    """The layer's glue around the expert products at the same configurations (one GPU): router top-k,
    the sort's bookkeeping, the two row gathers, the experts' bias, the weighted sum.  Device time per
    call (CUDA events over a recorded run of 20 calls) and the bytes each call has to move."""
    rng = np.random.default_rng(3)
    out = []
    for cname, E, topk, tokens, projs, _ in MOE_CONFIGS[:2]:
        D = projs[0][2]  # the model width: K of the first projection
        T = tokens[1]
        probs = rng.random((T, E), dtype=np.float32)
        probs /= probs.sum(-1, keepdims=True)
        p = dev.array(nv.f32_to_bf16(probs), nv.BF16)
        idx, scores = nv.moe_route(p, topk, True)
        order, restore, toks, srt, offsets = nv.moe_sort(idx, E)
        x = dev.array(nv.f32_to_bf16(rng.standard_normal((T, D), dtype=np.float32)), nv.BF16)
        rows = nv.take_rows(x, toks)
        bias = dev.array(nv.f32_to_bf16(rng.standard_normal((E, D), dtype=np.float32)), nv.BF16)
        y4 = dev.array(nv.f32_to_bf16(rng.standard_normal((T, topk, D), dtype=np.float32)), nv.BF16)
        inter = projs[1][2]  # the experts' intermediate width: K of the down projection
        gate = dev.array(nv.f32_to_bf16(rng.standard_normal((T * topk, inter), dtype=np.float32)), nv.BF16)
        upp = dev.array(nv.f32_to_bf16(rng.standard_normal((T * topk, inter), dtype=np.float32)), nv.BF16)
        glu = (lambda: nv.swiglu_oai(gate, upp)) if "gpt-oss" in cname else (lambda: nv.swiglu(gate, upp))
        wnorm = dev.array(nv.f32_to_bf16(rng.standard_normal(D, dtype=np.float32)), nv.BF16)
        calls = [
            ("add_rms_norm (in front of the layer)", lambda: nv.add_rms_norm(x, x, wnorm, 1e-6), T * D * 2 * 4 + D * 2),
            ("moe_route", lambda: nv.moe_route(p, topk, True), T * E * 2 + T * topk * 6),
            ("moe_sort", lambda: nv.moe_sort(idx, E), T * topk * 4 * 5 + E * 4),
            ("take_rows (activations by sorted pair)", lambda: nv.take_rows(x, toks), T * topk * D * 2 * 2),
            ("swiglu_oai" if "gpt-oss" in cname else "swiglu", glu, T * topk * inter * 2 * 3),
            ("expert_bias_add", lambda: nv.expert_bias_add(rows, bias, srt), T * topk * D * 2 * 3),
            ("take_rows (results back into pair order)", lambda: nv.take_rows(rows, restore), T * topk * D * 2 * 2),
            ("weighted_sum", lambda: nv.weighted_sum(y4, scores), T * topk * D * 2 + T * D * 2 + T * topk * 2),
        ]
        for name, call, nbytes in calls:
            call()
            dev.synchronize()

            def run():
                for _ in range(20):
                    call()
            g = dev.record(run)
            g.launch()
            dev.synchronize()
            e0, e1 = dev.event(), dev.event()
            e0.record()
            for _ in range(3):
                g.launch()
            e1.record()
            e1.synchronize()
            us = e0.elapsed_ms(e1) * 1e3 / 60
            out.append({"config": cname, "tokens": T, "kernel": name, "us": us, "GB/s": nbytes / us / 1e3})
    return out


def moe_bench(args, nv, _ffi, shard, dev, dist, rank, world, peaks):
    """Every rank owns experts [r E/g, (r+1) E/g) and, the gathered rows being sorted by expert, a
    contiguous slice of them (from the sorted offsets); it multiplies that slice with its own experts
    (nvc_gather_qmm) and the ranks' disjoint row ranges are joined by a padded all_gather.  Before any
    timing, rank 0 multiplies the whole list with all experts on its own GPU and the joined result
    must agree with it row for row (same kernel, same operands: bit for bit unless a tile is cut
    along K differently, in which case within one output rounding)."""
    lib = _ffi.lib()
    comm = None
    if world > 1:
        import torch
        ident = torch.zeros(128, dtype=torch.uint8, device="cuda")
        if rank == 0:
            buf = (C.c_uint8 * 128)()
            assert lib.nvc_comm_unique_id(buf) == 0, _ffi.last_error()
            ident = torch.tensor(list(buf), dtype=torch.uint8, device="cuda")
        dist.broadcast(ident, 0)
        idb = (C.c_uint8 * 128)(*ident.cpu().tolist())
        comm = C.c_void_p()
        assert lib.nvc_comm_init(dev._h, rank, world, idb, C.byref(comm)) == 0, _ffi.last_error()
    rows_out = []
    for cname, E, topk, tokens, projs, (mode, gs, bits) in MOE_CONFIGS:
        quant = nv.Quant(nv.QuantMode(mode), gs, bits)
        lo, hi = shard.expert_range(E, world, rank)
        for pname, N, K in projs:
            rng = np.random.default_rng(zlib.crc32(f"{cname}/{pname}".encode()))
            # random codes with scales in the range quantizing N(0, 0.02) weights gives; every rank
            # draws the same experts, keeps its own (rank 0 keeps all of them for the check)
            words = K * bits // 32
            codes = rng.integers(0, 2 ** 32, (E, N, words), dtype=np.uint32)
            if mode == "affine":
                sc = nv.f32_to_bf16((rng.random((E, N, K // gs), dtype=np.float32) * 0.06 + 0.03) / 15.0)
                bi = nv.f32_to_bf16(-(rng.random((E, N, K // gs), dtype=np.float32) * 0.04 + 0.02))
                sdt = nv.BF16
            else:
                sc = rng.integers(117, 123, (E, N, K // gs), dtype=np.uint8) if mode == "mxfp4" else \
                    rng.integers(0x08, 0x30, (E, N, K // gs), dtype=np.uint8)
                bi, sdt = None, nv.U8

            def on_device(e0, e1):
                return nv.Quantized(dev.array(np.ascontiguousarray(codes[e0:e1]), nv.U32), dev.array(np.ascontiguousarray(sc[e0:e1]), sdt),
                                    None if bi is None else dev.array(np.ascontiguousarray(bi[e0:e1]), nv.BF16), quant)
            mine = on_device(lo, hi)
            copies = [mine]
            per_rank_bytes = (hi - lo) * N * (words * 4 + (K // gs) * (4 if mode == "affine" else 1))
            while len(copies) * per_rank_bytes < 300e6 and len(copies) < 16:  # distinct copies: more than L2 per rank
                copies.append(on_device(lo, hi))
            full = on_device(0, E) if rank == 0 and world > 1 else None
            for T in tokens:
                ids = np.concatenate([rng.permutation(E)[:topk] for _ in range(T)]).astype(np.uint32)
                order = np.argsort(ids, kind="stable")
                sid = ids[order]
                xh = nv.f32_to_bf16(rng.standard_normal((T, K), dtype=np.float32))
                xs = np.ascontiguousarray(xh[order // topk]).reshape(T * topk, 1, K)
                bounds = [shard.expert_rows(sid, E, world, r) for r in range(world)]
                first, last = bounds[rank]
                mrows = max(1, max(b - a for a, b in bounds))
                x_local = dev.array(np.ascontiguousarray(xs[first:last]) if last > first else np.zeros((1, 1, K), np.uint16), nv.BF16)
                rhs_local = dev.array((sid[first:last] - lo).astype(np.uint32) if last > first else np.zeros(1, np.uint32), nv.U32)
                n_local = last - first
                gathered = dev.empty((world, mrows, N), nv.BF16)
                lib.nvc_memset(dev._h, gathered.ptr, 0, gathered.nbytes)
                slot = C.c_void_p(gathered.ptr.value + rank * mrows * N * 2)
                qc = quant._c()
                opts = nv.GatherQmm(transpose=True, sorted_indices=True)
                state = {"i": 0}

                def product():
                    q = copies[state["i"] % len(copies)]
                    state["i"] += 1
                    if n_local > 0:
                        rc = lib.nvc_gather_qmm(dev._h, C.byref(qc), nv.BF16, 1, x_local.ptr, q.weight.ptr, q.scales.ptr,
                                                None if q.biases is None else q.biases.ptr, None, None, rhs_local.ptr, None, 1,
                                                n_local, n_local, 1, N, K, hi - lo, slot)
                        assert rc == 0, _ffi.last_error()
                    if comm is not None:
                        assert lib.nvc_all_gather(comm, slot, gathered.ptr, mrows * N * 2) == 0, _ffi.last_error()

                product()
                dev.synchronize()
                check = None
                if world > 1:
                    got = gathered.to_numpy().view(np.uint16)
                    joined = np.concatenate([got[r, :b - a] for r, (a, b) in enumerate(bounds)], axis=0)
                    if rank == 0:
                        want = nv.gather_qmm(dev.array(xs, nv.BF16), full, None, dev.array(sid, nv.U32), opts).to_numpy()
                        want = want.view(np.uint16).reshape(T * topk, N)
                        if np.array_equal(joined, want):
                            check = "ok (bit for bit)"
                        else:
                            g32, w32 = nv.bf16_to_f32(joined).astype(np.float64), nv.bf16_to_f32(want).astype(np.float64)
                            lim = 2.0 ** -7 * np.abs(w32) + 2e-5 * np.abs(w32).max(axis=1, keepdims=True)
                            check = "ok (within one output rounding)" if np.all(np.abs(g32 - w32) <= lim) else "FAILED"
                        if check == "FAILED":
                            raise SystemExit(f"parity check failed: expert-sharded {cname} {pname} T={T} differs from the single-GPU product")
                reps = 5 if T > 1 else 20

                def step():
                    for _ in range(len(copies)):
                        product()
                step()
                g = dev.record(step)
                for _ in range(3):
                    g.launch()
                dev.synchronize()
                if dist is not None:
                    dist.barrier()
                e0, e1 = dev.event(), dev.event()
                e0.record()
                for _ in range(reps):
                    g.launch()
                e1.record()
                e1.synchronize()
                us = e0.elapsed_ms(e1) * 1e3 / reps / len(copies)
                if dist is not None:
                    import torch
                    t = torch.tensor([us], device="cuda")
                    dist.all_reduce(t, op=dist.ReduceOp.MAX)
                    us = float(t.item())
                touched = len(np.unique(ids))
                wbytes = touched * N * (words * 4 + (K // gs) * (4 if mode == "affine" else 1))
                flops = 2.0 * T * topk * N * K
                rows_out.append({"config": cname, "projection": pname, "tokens": T, "rows": T * topk, "experts": E, "N": N, "K": K,
                                 "quant": f"{mode} b{bits} g{gs}", "n_gpus": world, "experts_per_gpu": hi - lo,
                                 "rows_per_rank": [b - a for a, b in bounds], "us_per_product": us,
                                 "weight_GB/s": wbytes / us / 1e3, "TFLOP/s": flops / us / 1e6, "check": check,
                                 "includes": "gather_qmm on the rank's row slice" + (" + padded ncclAllGather of the row slices" if world > 1 else "")})
    glue = moe_glue_rows(nv, dev) if world == 1 else None
    if rank == 0:
        print(json.dumps({"workload": "moe", "metric": "gather_qmm, expert-sharded", "n_gpus": world, "data": "synthetic",
                          "scaling": "strong", "rows": rows_out, "glue": glue, "peaks": peaks}), flush=True)
    dev.synchronize()
    if world > 1:
        dist.barrier()
        sys.stdout.flush()
        os._exit(0)


# ── the other configurations of the benchmark definition, one line each (--sweep) ────────────
def config_sweep(nv, _ffi, dev, peaks):
    """Times every single-GPU configuration the benchmark definition lists (decode projections
    at M = 1, 4, 8; prefill at M = 2048 / 8192 and 4 / 8 bits; the two mixture-of-experts shapes
    through gather_qmm with sorted indices) and returns one row per product.  Device time only
    (CUDA events around replays of a recorded step); parity of the same shapes is what the GPU
    tests check."""
    lib = _ffi.lib()
    rng = np.random.default_rng(0)
    rows = []

    def time_fn(fn, reps):
        fn()
        g = dev.record(fn)
        for _ in range(3):
            g.launch()
        dev.synchronize()
        e0, e1 = dev.event(), dev.event()
        e0.record()
        for _ in range(reps):
            g.launch()
        e1.record()
        e1.synchronize()
        return e0.elapsed_ms(e1) * 1e3 / reps  # us per replay

    def quantized(shape, quant):
        """Random weights ~ N(0, 0.02) quantized on the device, expert by expert (bounded host memory)."""
        lead = shape[:-2]
        n = int(np.prod(lead)) if lead else 1
        parts = []
        for _ in range(n):
            w = nv.f32_to_bf16(rng.standard_normal(shape[-2:], dtype=np.float32) * 0.02)
            parts.append(nv.quantize(dev.array(w, nv.BF16), quant))
        if not lead:
            return parts[0]
        def stack(get, dtype):
            first = get(parts[0])
            out = dev.empty(tuple(lead) + tuple(first.shape), dtype)
            per = first.nbytes
            for i, q in enumerate(parts):
                lib.nvc_memcpy_d2d(dev._h, C.c_void_p(out.ptr.value + i * per), get(q).ptr, per)
            return out
        sdt = parts[0].scales.dtype
        return nv.Quantized(stack(lambda q: q.weight, nv.U32), stack(lambda q: q.scales, sdt),
                            None if parts[0].biases is None else stack(lambda q: q.biases, sdt), quant)

    def dense(tag, M, N, K, quant, copies, reps):
        q0 = quantized((N, K), quant)
        x = dev.array(nv.f32_to_bf16(rng.standard_normal((M, K), dtype=np.float32)), nv.BF16)
        sets = [q0]
        for _ in range(copies - 1):
            q = nv.Quantized(dev.empty(q0.weight.shape, nv.U32), dev.empty(q0.scales.shape, q0.scales.dtype),
                             None if q0.biases is None else dev.empty(q0.biases.shape, q0.biases.dtype), quant)
            q.weight.copy_from(q0.weight), q.scales.copy_from(q0.scales)
            if q0.biases is not None:
                q.biases.copy_from(q0.biases)
            sets.append(q)
        ys = [dev.empty((M, N), nv.BF16) for _ in sets]
        qc = quant._c()
        def step():
            for q, y in zip(sets, ys):
                rc = lib.nvc_quantized_matmul(dev._h, C.byref(qc), nv.BF16, 1, x.ptr, q.weight.ptr, q.scales.ptr,
                                              None if q.biases is None else q.biases.ptr, None, M, N, K, K, 1, 0, 0, 0, y.ptr)
                assert rc == 0, _ffi.last_error()
        us = time_fn(step, reps) / copies
        bits, gs = quant.bits, quant.group_size
        sbytes = 4 if quant.mode == nv.QuantMode.AFFINE else 1
        nbytes = N * K * bits / 8 + N * (K // gs) * sbytes + M * K * 2 + M * N * 2
        flops = 2.0 * M * N * K
        row = {"config": tag, "M": M, "N": N, "K": K, "quant": f"{quant.mode.name.lower()} b{bits} g{gs}", "us": us,
               "GB/s": nbytes / us / 1e3, "TFLOP/s": flops / us / 1e6}
        if M <= 8:
            row["frac"], row["of"] = row["GB/s"] / peaks["hbm_gbs"], "measured HBM copy"
        else:
            row["frac"], row["of"] = row["TFLOP/s"] / peaks["bf16_tflops"], "measured bf16 burst"
        rows.append(row)

    a4 = nv.Quant.affine(GS, BITS)
    dense("C1 qmv", 1, 4096, 4096, a4, 64, 20)
    for bits in (2, 3, 6, 8):  # 3- and 6-bit codes straddle words: three-word units in the few-row kernel
        dense(f"C1 qmv b{bits}", 1, 4096, 4096, nv.Quant.affine(GS, bits), 64, 10)
    for M in (1, 4, 8):
        for name, N, K in PROJECTIONS:
            dense(f"C2 {name}", M, N, K, a4, max(2, int(600e6 // (N * K // 2))), 20)
    for M in (2048, 8192):
        for bits in (4, 8):
            dense("C3 prefill", M, 12288, 4096, nv.Quant.affine(GS, bits), 3, 5)

    def moe(tag, T, E, topk, N, K, quant, reps):
        q = quantized((E, N, K), quant)
        ids = np.concatenate([rng.permutation(E)[:topk] for _ in range(T)]).astype(np.uint32)
        order = np.argsort(ids, kind="stable")
        rhs = dev.array(ids[order], nv.U32)
        xh = nv.f32_to_bf16(rng.standard_normal((T, K), dtype=np.float32))
        x = dev.array(np.ascontiguousarray(xh[order // topk]).reshape(T * topk, 1, K), nv.BF16)
        opts = nv.GatherQmm(transpose=True, sorted_indices=True)
        keep = []
        def step():
            keep.clear()
            keep.append(nv.gather_qmm(x, q, None, rhs, opts))
        us = time_fn(step, reps)
        bits, gs = quant.bits, quant.group_size
        sbytes = 4 if quant.mode == nv.QuantMode.AFFINE else 1
        touched = len(np.unique(ids))
        nbytes = touched * (N * K * bits / 8 + N * (K // gs) * sbytes) + T * topk * (K + N) * 2
        flops = 2.0 * T * topk * N * K
        rows.append({"config": tag, "M": f"{T}x{topk}", "N": N, "K": K, "quant": f"{quant.mode.name.lower()} b{bits} g{gs}, {E} experts",
                     "us": us, "GB/s": nbytes / us / 1e3, "TFLOP/s": flops / us / 1e6,
                     "frac": (nbytes / us / 1e3) / peaks["hbm_gbs"] if T == 1 else (flops / us / 1e6) / peaks["bf16_tflops"],
                     "of": "measured HBM copy (experts touched)" if T == 1 else "measured bf16 burst"})

    for T in (1, 512):
        moe("C4 moe gate+up", T, 128, 8, 1536, 2048, a4, 10)
        moe("C4 moe down", T, 128, 8, 2048, 768, a4, 10)
    for quant in (nv.Quant.new(nv.QuantMode.MXFP4), nv.Quant.new(nv.QuantMode.NVFP4)):
        for T in (1, 1024):
            moe("C5 moe gate+up", T, 32, 4, 5760, 2880, quant, 10)
            moe("C5 moe down", T, 32, 4, 2880, 2880, quant, 10)
    return rows



def qqmm_leg(nv, _ffi, dev, peaks, check=True):
    """MLX's qqmm at the prefill shape: weights quantized to NVFP4 with the reference's quantize, x quantized
    on the way by nvc_qqmm, the product on tcgen05.mma.kind::mxf4nvf4.block_scale.  Checked against the
    oracle's product of the two dequantized operands on 64 weight rows before it is timed."""
    M, N, K = PREFILL
    rng = np.random.default_rng(2)
    quant = nv.Quant(nv.QuantMode("nvfp4"), 16, 4)
    w = nv.f32_to_bf16(rng.standard_normal((N, K), dtype=np.float32) * 0.02)
    q0 = nv.quantize(dev.array(w, nv.BF16), quant)
    xh = nv.f32_to_bf16(rng.standard_normal((M, K), dtype=np.float32))
    x = dev.array(xh, nv.BF16)
    copies = 4
    sets = []
    for i in range(copies):
        c, sc = dev.empty(q0.weight.shape, nv.U32), dev.empty(q0.scales.shape, nv.U8)
        c.copy_from(q0.weight), sc.copy_from(q0.scales)
        sets.append((nv.Quantized(c, sc, None, quant), dev.empty((M, N), nv.BF16)))
    lib = _ffi.lib()
    qc = quant._c()

    def run(qw, y):
        rc = lib.nvc_qqmm(dev._h, C.byref(qc), nv.BF16, x.ptr, qw.weight.ptr, qw.scales.ptr, M, N, K, y.ptr)
        assert rc == 0, _ffi.last_error()
    parity = None
    if check:
        import oracle
        rows, toks = 64, 256
        run(*sets[0])
        got = nv.bf16_to_f32(sets[0][1].to_numpy().view(np.uint16)[:toks, :rows])
        wc, ws = q0.weight.to_numpy()[:rows], q0.scales.to_numpy()[:rows]
        xc, xs, _ = oracle.quantize(xh[:toks], oracle.BF16, oracle.NVFP4, 16, 4)
        xhat = oracle.dequantize(xc, xs, None, oracle.BF16, oracle.NVFP4, 16, 4)
        want = nv.bf16_to_f32(oracle.quantized_matmul(xhat, wc, ws, None, oracle.BF16, oracle.NVFP4, 16, 4))
        bound = 1e-2 * np.abs(want).max(-1, keepdims=True)
        worst = float((np.abs(got - want) / bound).max())
        if worst > 1.0:
            raise SystemExit(f"parity check failed: qqmm differs from the oracle ({worst:.3f} of the bound)")
        parity = {"status": "ok", "worst_error_over_bound": worst,
                  "what": f"{toks} token rows x {rows} weight rows against the oracle's product of the dequantized operands"}
    for qw, y in sets:
        run(qw, y)
    dev.synchronize()
    e0, e1 = dev.event(), dev.event()
    reps = 5
    e0.record()
    for _ in range(reps):
        for qw, y in sets:
            run(qw, y)
    e1.record()
    e1.synchronize()
    ms = e0.elapsed_ms(e1) / (reps * copies)
    tf = 2.0 * M * N * K / (ms * 1e-3) / 1e12
    return {"workload": f"qqmm M={M} K={K} N={N}: NVFP4 x NVFP4 (activations quantized on the way), block-scaled MMA",
            "metric": "qqmm TFLOP/s (M=2048)", "value": tf, "unit": "TFLOP/s", "ms_per_product": ms,
            "gpu_launches": reps * copies * 4, "parity_check": "ok" if parity else "skipped", "parity": parity,
            "roofline": {"kernel": "qqmm_kernel", "bound": "tensor", "achieved": tf, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                         "frac": tf / peaks["bf16_tflops"], "traffic": None,
                         "peak_source": peaks["source"] + " (bf16 burst: no measured 4-bit peak exists; nominal dense fp4 is 4x the bf16 figure)"}}


def prefill_bench(nv, _ffi, dev, peaks, rank, world, timed, barrier, check=True):
    M, N, K = PREFILL
    n_local = N // world
    rng = np.random.default_rng(1)
    quant = nv.Quant.affine(GS, BITS)
    w = (rng.standard_normal((N, K), dtype=np.float32) * 0.02)[rank * n_local:(rank + 1) * n_local]
    copies = 4  # 4 x (25 MB + x 16 MB + y 50 MB) per rank at N=1: larger than L2
    qs = []
    q0 = nv.quantize(dev.array(nv.f32_to_bf16(w), nv.BF16), quant)
    x0 = dev.array(nv.f32_to_bf16(rng.standard_normal((M, K), dtype=np.float32)), nv.BF16)
    for i in range(copies):
        q = nv.Quantized(dev.empty(q0.weight.shape, nv.U32), dev.empty(q0.scales.shape, nv.BF16),
                         dev.empty(q0.biases.shape, nv.BF16), quant)
        q.weight.copy_from(q0.weight), q.scales.copy_from(q0.scales), q.biases.copy_from(q0.biases)
        x = dev.empty(x0.shape, nv.BF16)
        x.copy_from(x0)
        qs.append((q, x, dev.empty((M, n_local), nv.BF16)))
    lib, qc = _ffi.lib(), quant._c()

    def step():
        for q, x, y in qs:
            rc = lib.nvc_quantized_matmul(dev._h, C.byref(qc), nv.BF16, 1, x.ptr, q.weight.ptr, q.scales.ptr,
                                          q.biases.ptr, None, M, n_local, K, K, 1, 0, 0, 0, y.ptr)
            assert rc == 0, _ffi.last_error()

    if rank == 0 and check:
        worst = check_products(nv, lib, dev, qc, [("prefill", M, qs[0][0], qs[0][1])], "prefill")
        checked = {"status": "ok", "worst_error_over_bound": worst,
                   "what": "128 output columns against the oracle within 1e-2*||row||_inf, 2048 unit-vector rows bit for "
                           "bit against the oracle's dequantize on 512 weight rows"}
    else:
        checked = None
    for _ in range(3):
        step()
    steps = 10
    ms, launches = timed(step, steps)
    flops = 2.0 * M * N * K * copies  # whole job
    tf = flops / (ms / steps * 1e-3) / 1e12
    per_launch = 2.0 * M * n_local * K / ((ms / steps) * 1e-3 / copies) / 1e12
    return {"workload": f"prefill qmm M={M} K={K} N={N} affine 4-bit g64", "metric": "quantized_matmul TFLOP/s (M=2048)",
            "value": tf, "unit": "TFLOP/s", "ms_per_product": ms / steps / copies, "gpu_launches": launches,
            "parity_check": None if checked is None else checked["status"], "parity": checked,
            "roofline": {"kernel": "qmm kernel", "bound": "tensor", "achieved": per_launch, "peak": peaks["bf16_tflops"],
                         "unit": "TFLOP/s", "frac": per_launch / peaks["bf16_tflops"], "traffic": None,
                         "peak_source": peaks["source"] + " (burst)"}}


if __name__ == "__main__":
    main()
