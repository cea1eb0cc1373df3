"""Reader for tests/golden/mlx_quant.bin.gz (the reference's recorded MLX vectors).

Container format (crates/nuvec-core/tests/common/fixture.rs:1-6), little-endian:
``magic | meta:str | count:u32 | case*``; ``case := name:str op:str n_in:u8 tensor* n_out:u8
tensor*``; ``tensor := dtype:u8 ndim:u8 dims:u64* nbytes:u64 data``; ``str := len:u16 utf8``.
The op string is ``name|key=value|...``.
"""
from __future__ import annotations

import gzip
import struct
from dataclasses import dataclass, field
from functools import lru_cache
from pathlib import Path

import numpy as np

# nuvec's DType order -> numpy storage dtype (float16/bfloat16 as uint16 bit patterns).
_NP = {0: np.bool_, 1: np.uint8, 2: np.uint16, 3: np.uint32, 4: np.uint64, 5: np.int8,
       6: np.int16, 7: np.int32, 8: np.int64, 9: np.uint16, 10: np.uint16, 11: np.float32,
       12: np.float64}


@dataclass
class Tensor:
    dtype: int
    data: np.ndarray


@dataclass
class Case:
    name: str
    op: str
    params: dict = field(default_factory=dict)
    inputs: list = field(default_factory=list)
    outputs: list = field(default_factory=list)

    def p(self, key, default=""):
        return self.params.get(key, default)


@lru_cache(maxsize=1)
def load():
    blob = gzip.open(Path(__file__).parent / "golden" / "mlx_quant.bin.gz").read()
    assert blob[:8] == b"BSMXFIX1"
    pos = 8

    def take(fmt):
        nonlocal pos
        v = struct.unpack_from(fmt, blob, pos)[0]
        pos += struct.calcsize(fmt)
        return v

    def string():
        nonlocal pos
        n = take("<H")
        s = blob[pos:pos + n].decode()
        pos += n
        return s

    def tensor():
        nonlocal pos
        dt, nd = take("<B"), take("<B")
        shape = [take("<Q") for _ in range(nd)]
        n = take("<Q")
        arr = np.frombuffer(blob, dtype=_NP[dt], count=n // np.dtype(_NP[dt]).itemsize,
                            offset=pos).reshape(shape)
        pos += n
        return Tensor(dt, arr)

    meta = string()
    cases = []
    for _ in range(take("<I")):
        name, spelled = string(), string()
        parts = spelled.split("|")
        case = Case(name, parts[0], dict(kv.split("=", 1) for kv in parts[1:]))
        case.inputs = [tensor() for _ in range(take("<B"))]
        case.outputs = [tensor() for _ in range(take("<B"))]
        cases.append(case)
    assert pos == len(blob)
    return meta, cases


def cases(op=None, source=None):
    out = load()[1]
    if op is not None:
        out = [c for c in out if c.op == op]
    if source is not None:
        out = [c for c in out if c.name.startswith(source + ":")]
    return out
