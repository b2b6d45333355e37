"""Writes GGUF v3 files for the tests (an independent statement of the layout the reader parses:
ggml's docs/gguf.md, version 3)."""
from __future__ import annotations

import struct

import numpy as np

U8, I8, U16, I16, U32, I32, F32, BOOL, STRING, ARRAY, U64, I64, F64 = range(13)
_FMT = {U8: "<B", I8: "<b", U16: "<H", I16: "<h", U32: "<I", I32: "<i", F32: "<f", BOOL: "<B", U64: "<Q", I64: "<q",
        F64: "<d"}


def string(s) -> bytes:
    raw = s if isinstance(s, bytes) else s.encode()
    return struct.pack("<Q", len(raw)) + raw


def value(kind: int, v) -> bytes:
    """The encoded value (without its type word). Arrays are `(element kind, [values])`."""
    if kind == STRING:
        return string(v)
    if kind == ARRAY:
        element, items = v
        return struct.pack("<IQ", element, len(items)) + b"".join(value(element, x) for x in items)
    return struct.pack(_FMT[kind], v)


def file(metadata, tensors, alignment: int = 32, version: int = 3, offsets=None) -> bytes:
    """metadata: [(key, kind, value)]; tensors: [(name, dims, ggml type id, bytes)]; `offsets` overrides
    the offsets written in the tensor descriptions (to write a file that is wrong)."""
    pad = lambda n: -n % alignment
    out = b"GGUF" + struct.pack("<IQQ", version, len(tensors), len(metadata))
    for key, kind, v in metadata:
        out += string(key) + struct.pack("<I", kind) + (v if isinstance(v, bytes) and kind != STRING else value(kind, v))
    data = b""
    for i, (name, dims, kind, raw) in enumerate(tensors):
        out += string(name) + struct.pack("<I", len(dims)) + b"".join(struct.pack("<Q", d) for d in dims)
        out += struct.pack("<IQ", kind, len(data) if offsets is None else offsets[i])
        raw = np.ascontiguousarray(raw).tobytes() if isinstance(raw, np.ndarray) else bytes(raw)
        data += raw + b"\0" * pad(len(raw))
    out += b"\0" * pad(len(out))
    return out + data
