#!/usr/bin/env python3
"""Selects the quantized-path cases from the reference's recorded MLX fixtures.

Reads the two fixture files the reference's own tests replay
(crates/nuvec-core/tests/fixtures/mlx.bin and mlx_gpu.bin; container format described at
crates/nuvec-core/tests/common/fixture.rs:1-6) and writes the subset that pins this
repository's path -- quantize, dequantize, quantized_matmul, gather_qmm -- to
tests/golden/mlx_quant.bin.gz in the same container format, so the tests can run where the
reference tree is not mounted.  The records are copied byte for byte; nothing is recomputed.

Usage: python tests/golden/extract_golden.py /path/to/reference
"""
import gzip
import struct
import sys
from pathlib import Path

OPS = {"quantize", "dequantize", "quantized_matmul", "gather_qmm"}
# Per-case size caps keep the committed file small: every quantize/dequantize case is kept,
# products are kept up to these byte counts (bfloat16 is the path's working dtype, so it gets
# the larger allowance).
CAP_BF16 = 110_000
CAP_OTHER = 40_000
CAP_CPU_FILE = 70_000


def records(blob):
    """Yields (name, spelled_op, record_bytes, in_dtypes, total_tensor_bytes) per case."""
    assert blob[:8] == b"BSMXFIX1"
    pos = 8
    (n,) = struct.unpack_from("<H", blob, pos)
    meta = blob[pos + 2:pos + 2 + n].decode()
    pos += 2 + n
    (count,) = struct.unpack_from("<I", blob, pos)
    pos += 4
    out = []
    for _ in range(count):
        start = pos
        strs = []
        for _ in range(2):
            (n,) = struct.unpack_from("<H", blob, pos)
            strs.append(blob[pos + 2:pos + 2 + n].decode())
            pos += 2 + n
        dtypes, total = [], 0
        for _side in range(2):
            k = blob[pos]
            pos += 1
            for _ in range(k):
                dt, nd = blob[pos], blob[pos + 1]
                pos += 2 + 8 * nd
                (nbytes,) = struct.unpack_from("<Q", blob, pos)
                pos += 8 + nbytes
                dtypes.append(dt)
                total += nbytes
        out.append((strs[0], strs[1], blob[start:pos], dtypes, total))
    assert pos == len(blob)
    return meta, out


def keep(name, spelled, dtypes, total, cpu_file):
    op = spelled.split("|")[0]
    if op not in OPS:
        return False
    if op in ("quantize", "dequantize"):
        return True
    if "mode=mxfp8" in spelled:
        return total <= 16_000
    if cpu_file:
        return total <= CAP_CPU_FILE
    bf16 = dtypes[0] == 10
    return total <= (CAP_BF16 if bf16 else CAP_OTHER)


def main(ref):
    fixtures = Path(ref) / "crates/nuvec-core/tests/fixtures"
    chosen, metas = [], []
    for fname in ("mlx.bin", "mlx_gpu.bin"):
        meta, recs = records((fixtures / fname).read_bytes())
        metas.append(f"{fname}: {meta}")
        tag = "cpu" if fname == "mlx.bin" else "gpu"
        for name, spelled, rec, dtypes, total in recs:
            if keep(name, spelled, dtypes, total, tag == "cpu"):
                # Prefix the case name with the file it came from: the two recordings pin
                # different roundings (MLX CPU vs MLX Metal).
                new_name = f"{tag}:{name}".encode()
                (n0,) = struct.unpack_from("<H", rec, 0)
                chosen.append(struct.pack("<H", len(new_name)) + new_name + rec[2 + n0:])
    meta = (" ; ".join(metas)).encode()
    blob = b"BSMXFIX1" + struct.pack("<H", len(meta)) + meta + struct.pack("<I", len(chosen))
    blob += b"".join(chosen)
    out = Path(__file__).with_name("mlx_quant.bin.gz")
    with gzip.GzipFile(out, "wb", compresslevel=9, mtime=0) as f:
        f.write(blob)
    print(f"{len(chosen)} cases, {len(blob)} bytes raw, {out.stat().st_size} bytes gz")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: extract_golden.py <path of the nuvec checkout>")
    main(sys.argv[1])
