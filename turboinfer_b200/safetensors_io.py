"""Reader and writer of safetensors files: an 8-byte little-endian header length, that many bytes of JSON
(name -> dtype, shape, data_offsets), then the raw little-endian data.  numpy only."""
from __future__ import annotations

import json
import struct
from typing import Dict

import numpy as np

from .seq import Bf16Array, bf16_bits

_NP = {"F32": np.float32, "F16": np.float16, "I32": np.int32, "I64": np.int64, "F64": np.float64, "U8": np.uint8, "I8": np.int8}


def read_safetensors(path: str) -> Dict[str, object]:
    """name -> numpy array, or Bf16Array (raw bits + shape) for BF16 tensors, which numpy has no type for."""
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n))
        data = f.read()
    out: Dict[str, object] = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        a, b = info["data_offsets"]
        raw = memoryview(data)[a:b]
        shape = tuple(int(s) for s in info["shape"])
        if info["dtype"] == "BF16":
            out[name] = Bf16Array(np.frombuffer(raw, dtype="<u2"), shape)
        elif info["dtype"] in _NP:
            out[name] = np.frombuffer(raw, dtype=np.dtype(_NP[info["dtype"]]).newbyteorder("<")).reshape(shape)
        else:
            raise ValueError(f"{path}: tensor {name} has unsupported dtype {info['dtype']}")
    return out


def write_safetensors(path: str, tensors: Dict[str, np.ndarray], bf16: bool = True) -> None:
    """Floating tensors are written as BF16 (rounded to nearest even) when `bf16`, else F32; integer tensors as I32."""
    header, blobs, off = {}, [], 0
    for name, t in tensors.items():
        a = np.asarray(t)
        if np.issubdtype(a.dtype, np.integer):
            raw, dt = np.ascontiguousarray(a, dtype="<i4").tobytes(), "I32"
        elif bf16:
            raw, dt = bf16_bits(a.astype(np.float32)).astype("<u2").tobytes(), "BF16"
        else:
            raw, dt = np.ascontiguousarray(a, dtype="<f4").tobytes(), "F32"
        header[name] = {"dtype": dt, "shape": list(a.shape), "data_offsets": [off, off + len(raw)]}
        blobs.append(raw)
        off += len(raw)
    hj = json.dumps(header, separators=(",", ":")).encode()
    hj += b" " * (-len(hj) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for b in blobs:
            f.write(b)
