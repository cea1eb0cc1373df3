"""Makes tests/golden/kv_quant_attention_l1.safetensors: the one-query-row records of the reference's fixture
crates/nuvec-lm/tests/fixtures/kv_quant_attention.safetensors (mlx-lm's quantized attention: float32 and bfloat16,
8 and 4 bits in groups of 32, 4 query heads over 2 key heads of size 64, 40 keys, scale 0.125; queries `q`, keys
`k0 k1 k2` and values `v0 v1 v2` as codes, scales, biases, and mlx-lm's output `out`).

    python tests/golden/make_attention_golden.py /path/to/reference
"""
import json
import struct
import sys
from pathlib import Path


def main():
    src = Path(sys.argv[1]) / "crates/nuvec-lm/tests/fixtures/kv_quant_attention.safetensors"
    raw = src.read_bytes()
    (n,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + n])
    keep = sorted(k for k in header if "_l1_" in k)
    out_header, blobs, at = {}, [], 0
    for k in keep:
        lo, hi = header[k]["data_offsets"]
        data = raw[8 + n + lo:8 + n + hi]
        out_header[k] = {"dtype": header[k]["dtype"], "shape": header[k]["shape"], "data_offsets": [at, at + len(data)]}
        blobs.append(data)
        at += len(data)
    text = json.dumps(out_header, separators=(",", ":")).encode()
    text += b" " * (-len(text) % 8)
    dst = Path(__file__).resolve().parent / "kv_quant_attention_l1.safetensors"
    dst.write_bytes(struct.pack("<Q", len(text)) + text + b"".join(blobs))
    print(len(keep), "tensors", at, "bytes")


if __name__ == "__main__":
    main()
