"""Makes tests/golden/checkpoint_gpt_oss_{hf,mlx}.safetensors from the reference's fixture pair.

The reference's tests hold the same tiny gpt-oss model twice: as Hugging Face writes it (MXFP4 experts as
`*_blocks` / `*_scales`, gate and up rows interleaved) in crates/nuvec-lm/tests/fixtures/gpt_oss_hf_mxfp4
and as mlx-lm converts it (`experts.{gate,up,down}_proj.{weight,scales,bias}`) in .../gpt_oss_mxfp4.  The
expert tensors of both files are copied here (every layer), so the adapters can be checked bit for bit
against what the reference's loader must produce.  Run from the repository root, with the reference
checkout beside it:

    python tests/golden/make_checkpoint_golden.py /path/to/reference
"""
import json
import struct
import sys
from pathlib import Path


def read(path):
    raw = Path(path).read_bytes()
    (n,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + n])
    return {k: (v["dtype"], v["shape"], raw[8 + n + v["data_offsets"][0]:8 + n + v["data_offsets"][1]])
            for k, v in header.items() if k != "__metadata__"}


def write(path, tensors):
    header, blobs, at = {}, [], 0
    for name in sorted(tensors):
        dtype, shape, data = tensors[name]
        header[name] = {"dtype": dtype, "shape": shape, "data_offsets": [at, at + len(data)]}
        blobs.append(data)
        at += len(data)
    text = json.dumps(header, separators=(",", ":")).encode()
    text += b" " * (-len(text) % 8)
    Path(path).write_bytes(struct.pack("<Q", len(text)) + text + b"".join(blobs))


def main():
    fixtures = Path(sys.argv[1]) / "crates/nuvec-lm/tests/fixtures"
    here = Path(__file__).resolve().parent
    for kind, folder in (("hf", "gpt_oss_hf_mxfp4"), ("mlx", "gpt_oss_mxfp4")):
        tensors = {k: v for k, v in read(fixtures / folder / "model.safetensors").items() if ".mlp.experts." in k}
        write(here / f"checkpoint_gpt_oss_{kind}.safetensors", tensors)
        print(kind, len(tensors), "tensors", sum(len(v[2]) for v in tensors.values()), "bytes")


if __name__ == "__main__":
    main()
