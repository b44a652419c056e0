"""`.fvecs` / `.ivecs` readers (src/vector/io.rs:7-42) over the C ABI."""
from __future__ import annotations

import ctypes as C

import numpy as np

from ._lib import check, lib


def _read(fn, path: str, limit, dtype) -> np.ndarray:
    out, n, dim = C.c_void_p(), C.c_size_t(0), C.c_size_t(0)
    check(fn(str(path).encode(), int(limit or 0), C.byref(out), C.byref(n), C.byref(dim)))
    try:
        buf = (C.c_uint8 * (n.value * dim.value * 4)).from_address(out.value)
        return np.frombuffer(buf, dtype=dtype).reshape(n.value, dim.value).copy()
    finally:
        lib().fv_free(out)


def read_fvecs(path, limit=None) -> np.ndarray:
    """Up to `limit` vectors as an (n, dim) float32 array."""
    return _read(lib().fv_read_fvecs, path, limit, "<f4")


def read_ivecs(path, limit=None) -> np.ndarray:
    """Up to `limit` rows of integers (e.g. ground-truth neighbour ids) as an (n, dim) uint32 array."""
    return _read(lib().fv_read_ivecs, path, limit, "<u4")
