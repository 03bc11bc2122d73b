"""MFQ container reader over the C ABI (mirrors ``MfqFile`` of the reference runtime,
cpp_runtime/mfq_decode.cpp:1294-1527, and ``open_mmap`` of mfq/formats/io.py:782-831)."""

from __future__ import annotations

import ctypes as C
import json

from . import _capi
from ._capi import check, lib


class MfqFile:
    """Record table of one ``.mfq`` file (or shard set); blobs are views into the mapping."""

    def __init__(self, path: str | None = None, *, image: bytes | None = None):
        self._h = C.c_void_p()
        if (path is None) == (image is None):
            raise ValueError("give exactly one of path / image")
        if path is not None:
            check(lib.mfqb_file_open(str(path).encode(), C.byref(self._h)))
        else:
            addr, n, keep = _capi.buffer_address(image)
            check(lib.mfqb_file_open_memory(addr, n, C.byref(self._h)))
        ver, arch, nx, nr = C.c_uint32(), C.c_char_p(), C.c_int(), C.c_int()
        check(lib.mfqb_file_header(self._h, C.byref(ver), C.byref(arch), C.byref(nx), C.byref(nr)))
        self.version = ver.value
        self.arch = arch.value.decode()
        self.extra = {}
        for i in range(nx.value):
            k, v = C.c_char_p(), C.c_char_p()
            check(lib.mfqb_file_extra(self._h, i, C.byref(k), C.byref(v)))
            self.extra[k.value.decode()] = json.loads(v.value.decode())
        self.records = []
        for i in range(nr.value):
            name, dtype, nb = C.c_char_p(), C.c_char_p(), C.c_uint64()
            check(lib.mfqb_file_record(self._h, i, C.byref(name), C.byref(dtype), C.byref(nb)))
            self.records.append((name.value.decode(), dtype.value.decode(), nb.value))

    def names(self):
        return [r[0] for r in self.records]

    def find(self, name: str) -> int:
        idx = C.c_int()
        check(lib.mfqb_file_find(self._h, name.encode(), C.byref(idx)))
        return idx.value

    def dtype(self, name: str) -> str:
        return self.records[self._index(name)][1]

    def _index(self, name: str) -> int:
        i = self.find(name)
        if i < 0:
            raise KeyError(name)
        return i

    def blob(self, name: str) -> bytes:
        p, n = C.c_void_p(), C.c_uint64()
        check(lib.mfqb_file_blob(self._h, self._index(name), C.byref(p), C.byref(n)))
        return C.string_at(p.value, n.value)

    def close(self) -> None:
        if self._h:
            lib.mfqb_file_close(self._h)
            self._h = C.c_void_p()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
