"""`Gguf` of loadngo's `weights` crate (weights/src/gguf.rs) over the library's reader.

The parsing is libcuda_compute.so's (`cc_gguf_*`); this file only gives it the reference's names:
`Gguf.parse(prefix, file_len)`, `open(path)`, `gguf.tensor(name)`, `gguf.get(key)`, and the error
variants of `GgufError` (gguf.rs:147-163).
"""
from __future__ import annotations

import ctypes
from ctypes import byref, c_double, c_int, c_int64, c_uint64, c_void_p
from dataclasses import dataclass

import numpy as np

from . import compute


class GgufError(Exception):
    """`GgufError` (weights/src/gguf.rs:147-163)."""
    code = 0


class Magic(GgufError):
    code = 1


class Version(GgufError):
    code = 2


class Truncated(GgufError):
    code = 3


class ValueType(GgufError):
    code = 4


class Utf8(GgufError):
    code = 5


class Invalid(GgufError):
    code = 6


class Read(GgufError):
    code = 7


_ERRORS = {c.code: c for c in (Magic, Version, Truncated, ValueType, Utf8, Invalid, Read)}

F32, F16, Q8_0, BF16, MXFP4 = 0, 1, 8, 30, 39   # `GgmlType`, by ggml number (gguf.rs:103-113)
ARRAY, STRING, BOOL = 9, 8, 7


def _check(code: int) -> None:
    if code != 0:
        raise _ERRORS.get(code, GgufError)(compute.lib().cc_last_error().decode())


@dataclass
class Tensor:
    """`Tensor` (gguf.rs:127-145)."""
    name: str
    dims: list          # the first varies fastest
    ggml_type: int
    offset: int         # absolute in the file
    len: int | None     # None for an element type that is not sized

    def numel(self) -> int:
        n = 1
        for d in self.dims:
            n *= d
        return n


class Gguf:
    """A parsed header (`Gguf`, gguf.rs:165-391)."""

    def __init__(self, handle: int):
        self._h = handle
        L = compute.lib()
        self.version = L.cc_gguf_version(handle)
        self.alignment = L.cc_gguf_alignment(handle)
        self.data_offset = L.cc_gguf_data_offset(handle)
        self.tensors = []
        raw = compute.GgufTensor()
        for i in range(L.cc_gguf_tensor_count(handle)):
            _check(L.cc_gguf_tensor_at(handle, i, byref(raw)))
            self.tensors.append(Tensor(raw.name.decode(), [int(d) for d in raw.dims[: raw.n_dims]], raw.ggml_type,
                                       raw.offset, None if raw.len == 2 ** 64 - 1 else raw.len))

    @classmethod
    def parse(cls, prefix: bytes, file_len: int) -> "Gguf":
        """`Gguf::parse` (gguf.rs:258-351). `Truncated` means the header needs more of the file."""
        buf = (ctypes.c_uint8 * max(len(prefix), 1)).from_buffer_copy(bytes(prefix) or b"\0")
        h = c_void_p()
        _check(compute.lib().cc_gguf_parse(ctypes.addressof(buf), len(prefix), file_len, byref(h)))
        return cls(h.value)

    def keys(self) -> list:
        L = compute.lib()
        return [L.cc_gguf_metadata_key(self._h, i).decode() for i in range(L.cc_gguf_metadata_count(self._h))]

    def tensor(self, name: str) -> Tensor | None:
        i = compute.lib().cc_gguf_find_tensor(self._h, name.encode())
        return None if i < 0 else self.tensors[i]

    def _scalar(self, key: bytes, kind: int, index: int):
        L = compute.lib()
        if kind in (0, 2, 4, 10):
            v = c_uint64()
            return int(v.value) if L.cc_gguf_get_u64(self._h, key, index, byref(v)) else None
        if kind in (1, 3, 5, 11):
            v = c_int64()
            return int(v.value) if L.cc_gguf_get_i64(self._h, key, index, byref(v)) else None
        if kind in (6, 12):
            v = c_double()
            return float(v.value) if L.cc_gguf_get_f64(self._h, key, index, byref(v)) else None
        if kind == BOOL:
            v = c_int()
            return bool(v.value) if L.cc_gguf_get_bool(self._h, key, index, byref(v)) else None
        if kind == STRING:
            p, n = c_void_p(), c_uint64()
            if not L.cc_gguf_get_str(self._h, key, index, byref(p), byref(n)):
                return None
            return ctypes.string_at(p.value, n.value).decode() if n.value else ""
        return None

    def get(self, key: str):
        """`Gguf::get` (gguf.rs:388-390): the value as a Python int, float, bool, str or list; None
        when the key is absent."""
        L, k = compute.lib(), key.encode()
        kind = L.cc_gguf_value_type(self._h, k)
        if kind < 0:
            return None
        if kind == ARRAY:
            element = L.cc_gguf_array_type(self._h, k)
            return [self._scalar(k, element, i) for i in range(L.cc_gguf_array_len(self._h, k))]
        return self._scalar(k, kind, -1)

    def value_type(self, key: str) -> int:
        return compute.lib().cc_gguf_value_type(self._h, key.encode())

    def read(self, tensor: Tensor) -> np.ndarray:
        """The tensor's bytes, from a header opened with `open` (the reference's
        `FileReader::read_ranges`, used at gpt-oss/src/model.rs:291-309)."""
        if tensor.len is None:
            raise Invalid(f"{tensor.name}: unsupported type")
        out = np.empty(tensor.len, np.uint8)
        _check(compute.lib().cc_gguf_read(self._h, tensor.offset, tensor.len, out.ctypes.data))
        return out

    def close(self) -> None:
        if self._h:
            compute.lib().cc_gguf_free(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def open(path: str, first_read: int = 0) -> Gguf:  # noqa: A001 - the reference's name
    """`gguf::open` (gguf.rs:405-408): parses the header, reading it in pieces of `first_read`
    bytes (16 MiB when 0) doubled until it fits; the handle serves the tensor bytes afterwards."""
    h = c_void_p()
    _check(compute.lib().cc_gguf_open(str(path).encode(), first_read, byref(h)))
    return Gguf(h.value)
