"""safetensors container: reader (mmap) and writer.

The file is an 8-byte little-endian header length, that many bytes of JSON (``name -> {dtype, shape, data_offsets}``, offsets
relative to the end of the header) and the tensor bytes.  The reader hands out zero-copy ``uint8`` views, like ``gguf.GGUFFile``
does for GGUF tensors; the writer exists because no real checkpoints are available offline and tests and benchmarks run on
seeded synthetic weights.  The reference has no counterpart (it reads GGUF only).
"""
from __future__ import annotations

import json
import mmap
import struct

import numpy as np

DTYPE_BYTES = {"BF16": 2, "F16": 2, "F32": 4, "I32": 4, "I64": 8, "U8": 1}


class SafetensorsFile:
    def __init__(self, path: str):
        self.path = path
        self._f = open(path, "rb")
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)
        if len(self._mm) < 8:
            raise ValueError(f"{path}: too short for a safetensors header")
        (n,) = struct.unpack_from("<Q", self._mm, 0)
        if 8 + n > len(self._mm):
            raise ValueError(f"{path}: header length {n} exceeds the file")
        head = json.loads(bytes(self._mm[8:8 + n]).decode("utf-8"))
        self.metadata = head.pop("__metadata__", {})
        self.base = 8 + n
        self.infos: dict[str, tuple[str, tuple[int, ...], int, int]] = {}
        for name, m in head.items():
            dt, shape = m["dtype"], tuple(int(d) for d in m["shape"])
            lo, hi = (int(v) for v in m["data_offsets"])
            if dt not in DTYPE_BYTES:
                raise ValueError(f"{path}: tensor {name} has unsupported dtype {dt}")
            if hi - lo != int(np.prod(shape, dtype=np.int64)) * DTYPE_BYTES[dt] or self.base + hi > len(self._mm) or lo < 0:
                raise ValueError(f"{path}: tensor {name}: offsets {lo}..{hi} do not fit shape {shape} of {dt}")
            self.infos[name] = (dt, shape, lo, hi)

    def tensor_bytes(self, name: str) -> np.ndarray:
        _, _, lo, hi = self.infos[name]
        return np.frombuffer(self._mm, dtype=np.uint8, count=hi - lo, offset=self.base + lo)

    def close(self):
        self._mm.close()
        self._f.close()


def bf16_bits(x: np.ndarray) -> np.ndarray:
    """float32 -> bfloat16 bit patterns, round to nearest even."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)


def bf16_to_f32(bits: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(bits, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def write_safetensors(path: str, tensors: dict, metadata: dict | None = None) -> None:
    """``tensors[name] = (dtype string, shape, bytes-like)``."""
    head, blobs, off = {}, [], 0
    if metadata:
        head["__metadata__"] = metadata
    for name, (dt, shape, raw) in tensors.items():
        b = np.ascontiguousarray(raw).view(np.uint8).reshape(-1).tobytes()
        head[name] = {"dtype": dt, "shape": [int(d) for d in shape], "data_offsets": [off, off + len(b)]}
        blobs.append(b)
        off += len(b)
    hj = json.dumps(head, separators=(",", ":")).encode("utf-8")
    hj += b" " * (-len(hj) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for b in blobs:
            f.write(b)
