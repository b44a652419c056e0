"""ctypes front end of the CPU oracle (``ferro_oracle.cpp``).

TEST INFRASTRUCTURE ONLY: imported by ``tests/``, by the smoke check and by the
CPU-baseline leg of the benchmark.  The shipped library never loads it.

The classes mirror the reference's Rust types (``FlatIndex``, ``IvfPq``, ``Hnsw``
in src/vector/) closely enough that a parity test reads like the reference's own
tests/vector.rs.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "libferro_oracle.so")

L2, INNER_PRODUCT = 0, 1

NEIGHBOR = np.dtype([("id", "<u4"), ("distance", "<f4")])


def build(force: bool = False) -> str:
    src = os.path.join(_HERE, "ferro_oracle.cpp")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "-s", "-B"])
    return _SO


_lib = None


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(_SO):
            build()
        L = C.CDLL(_SO)
        vp, sz, u64, f32p, u32p, i = C.c_void_p, C.c_size_t, C.c_uint64, C.c_void_p, C.c_void_p, C.c_int
        sig = {
            "orc_has_avx2": (i, []),
            "orc_rng_new": (vp, [u64]),
            "orc_rng_free": (None, [vp]),
            "orc_rng_next": (u64, [vp]),
            "orc_rng_below": (u64, [vp, u64]),
            "orc_rng_uniform": (C.c_double, [vp]),
            "orc_rng_normal": (C.c_double, [vp]),
            "orc_testdata": (None, [sz, sz, u64, f32p]),
            "orc_datagen": (None, [i, u64, sz, sz, sz, sz, i, f32p]),
            "orc_l2sq": (C.c_float, [f32p, f32p, sz]),
            "orc_dot": (C.c_float, [f32p, f32p, sz]),
            "orc_l2sq_scalar": (C.c_float, [f32p, f32p, sz]),
            "orc_dot_scalar": (C.c_float, [f32p, f32p, sz]),
            "orc_distance": (C.c_float, [i, f32p, f32p, sz]),
            "orc_padded": (sz, [sz]),
            "orc_normalize": (None, [f32p, sz, sz]),
            "orc_topk": (sz, [f32p, sz, sz, vp]),
            "orc_recall": (C.c_double, [vp, u32p, u32p, sz, sz, sz]),
            "orc_flat_new": (vp, [i, sz]),
            "orc_flat_free": (None, [vp]),
            "orc_flat_add": (None, [vp, f32p, sz]),
            "orc_flat_len": (sz, [vp]),
            "orc_flat_search_batch": (None, [vp, f32p, sz, sz, i, vp, u32p]),
            "orc_kmeans_assign": (None, [f32p, sz, f32p, sz, sz, i, u32p]),
            "orc_kmeans_train": (i, [f32p, sz, sz, sz, sz, u64, i, f32p]),
            "orc_kmeans_nearest": (C.c_float, [f32p, f32p, sz, sz, u32p]),
            "orc_ivfpq_train": (vp, [i, sz, f32p, sz, sz, sz, sz, i, u64, i]),
            "orc_ivfpq_free": (None, [vp]),
            "orc_ivfpq_add": (None, [vp, f32p, sz, i]),
            "orc_ivfpq_len": (sz, [vp]),
            "orc_ivfpq_bytes_per_vector": (sz, [vp]),
            "orc_ivfpq_has_tables": (i, [vp]),
            "orc_ivfpq_search_batch": (u64, [vp, f32p, sz, sz, sz, sz, i, vp, u32p]),
            "orc_ivfpq_save": (sz, [vp, vp, sz]),
            "orc_ivfpq_load": (vp, [vp, sz, C.c_char_p, sz]),
            "orc_hnsw_build": (vp, [i, sz, f32p, sz, sz, sz, u64, i]),
            "orc_hnsw_build_batched": (vp, [i, sz, f32p, sz, sz, sz, u64, sz, sz]),
            "orc_hnsw_free": (None, [vp]),
            "orc_hnsw_len": (sz, [vp]),
            "orc_hnsw_reachable": (sz, [vp]),
            "orc_hnsw_mean_degree": (C.c_double, [vp]),
            "orc_hnsw_search_batch": (None, [vp, f32p, sz, sz, sz, i, vp, u32p, vp]),
            "orc_hnsw_save": (sz, [vp, vp, sz]),
            "orc_hnsw_load": (vp, [vp, sz, C.c_char_p, sz]),
        }
        for name, (res, args) in sig.items():
            fn = getattr(L, name)
            fn.restype = res
            fn.argtypes = args
        _lib = L
    return _lib


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


def _p(a: np.ndarray):
    return a.ctypes.data_as(C.c_void_p)


def cores() -> int:
    return len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)


class Rng:
    """src/rng.rs:7-45."""

    def __init__(self, seed: int):
        self._h = lib().orc_rng_new(seed)

    def __del__(self):
        if getattr(self, "_h", None):
            lib().orc_rng_free(self._h)
            self._h = None

    def next_u64(self) -> int:
        return lib().orc_rng_next(self._h)

    def below(self, n: int) -> int:
        return lib().orc_rng_below(self._h, n)

    def uniform(self) -> float:
        return lib().orc_rng_uniform(self._h)

    def normal(self) -> float:
        return lib().orc_rng_normal(self._h)


def testdata(n: int, dim: int, seed: int) -> np.ndarray:
    """The generator of tests/vector.rs:11-24."""
    out = np.empty((n, dim), dtype=np.float32)
    lib().orc_testdata(n, dim, seed, _p(out))
    return out


def datagen(kind: int, seed: int, n: int, dim: int, clusters: int, first_row: int = 0, threads: int | None = None) -> np.ndarray:
    """The benchmark's seeded Gaussian-mixture rows (kind 0: SIFT-like integers, kind 1: unit-length embeddings):
    the same bytes the product library's fv_datagen gives."""
    out = np.empty((n, dim), dtype=np.float32)
    lib().orc_datagen(kind, seed, first_row, n, dim, clusters, threads or cores(), _p(out))
    return out


def l2sq(a, b) -> float:
    a, b = _f32(a), _f32(b)
    return lib().orc_l2sq(_p(a), _p(b), a.size)


def dot(a, b) -> float:
    a, b = _f32(a), _f32(b)
    return lib().orc_dot(_p(a), _p(b), a.size)


def distance(metric: int, a, b) -> float:
    a, b = _f32(a), _f32(b)
    return lib().orc_distance(metric, _p(a), _p(b), a.size)


def normalize(data: np.ndarray) -> np.ndarray:
    data = _f32(data).copy()
    n, dim = data.shape
    lib().orc_normalize(_p(data), n, dim)
    return data


def topk(distances, k: int) -> np.ndarray:
    d = _f32(distances)
    out = np.zeros(k, dtype=NEIGHBOR)
    c = lib().orc_topk(_p(d), d.size, k, _p(out))
    return out[:c]


def recall(found: np.ndarray, counts: np.ndarray, truth: np.ndarray, k: int) -> float:
    """src/vector/mod.rs:145-152; `found` is (nq, k) NEIGHBOR, `truth` (nq, >=k) ids."""
    found = np.ascontiguousarray(found)
    counts = np.ascontiguousarray(counts, dtype=np.uint32)
    truth = np.ascontiguousarray(truth, dtype=np.uint32)
    return lib().orc_recall(_p(found), _p(counts), _p(truth), truth.shape[1], found.shape[0], k)


def _results(nq: int, k: int):
    return np.zeros((nq, k), dtype=NEIGHBOR), np.zeros(nq, dtype=np.uint32)


class FlatIndex:
    """src/vector/flat.rs."""

    def __init__(self, metric: int, dim: int):
        self.metric, self.dim = metric, dim
        self._h = lib().orc_flat_new(metric, dim)

    def __del__(self):
        if getattr(self, "_h", None):
            lib().orc_flat_free(self._h)
            self._h = None

    def add(self, vectors):
        v = _f32(vectors).reshape(-1, self.dim)
        lib().orc_flat_add(self._h, _p(v), v.shape[0])

    def __len__(self):
        return lib().orc_flat_len(self._h)

    def search_batch(self, queries, k: int, threads: int | None = None):
        q = _f32(queries).reshape(-1, self.dim)
        out, counts = _results(q.shape[0], k)
        lib().orc_flat_search_batch(self._h, _p(q), q.shape[0], k, threads or cores(), _p(out), _p(counts))
        return out, counts


def kmeans_train(data, k: int, iters: int, seed: int, threads: int | None = None) -> np.ndarray:
    d = _f32(data)
    n, dim = d.shape
    cen = np.empty((k, dim), dtype=np.float32)
    rc = lib().orc_kmeans_train(_p(d), n, dim, k, iters, seed, threads or cores(), _p(cen))
    if rc:
        raise ValueError(f"need at least {k} training vectors, got {n}")
    return cen


def kmeans_assign(data, centroids, threads: int | None = None) -> np.ndarray:
    d, c = _f32(data), _f32(centroids)
    out = np.empty(d.shape[0], dtype=np.uint32)
    lib().orc_kmeans_assign(_p(d), d.shape[0], _p(c), c.shape[0], d.shape[1], threads or cores(), _p(out))
    return out


def kmeans_nearest(x, centroids):
    x, c = _f32(x), _f32(centroids)
    which = C.c_uint32(0)
    d = lib().orc_kmeans_nearest(_p(x), _p(c), c.shape[0], c.shape[1], C.byref(which))
    return which.value, d


class IvfPq:
    """src/vector/ivfpq.rs."""

    def __init__(self, handle, dim: int):
        self._h, self.dim = handle, dim

    def __del__(self):
        if getattr(self, "_h", None):
            lib().orc_ivfpq_free(self._h)
            self._h = None

    @staticmethod
    def train(metric: int, dim: int, sample, nlist: int, m: int, iters: int, keep_vectors: bool, seed: int,
              threads: int | None = None) -> "IvfPq":
        s = _f32(sample).reshape(-1, dim)
        h = lib().orc_ivfpq_train(metric, dim, _p(s), s.shape[0], nlist, m, iters, int(keep_vectors), seed,
                                  threads or cores())
        if not h:
            raise ValueError("bad IVF-PQ parameters")
        return IvfPq(h, dim)

    def add(self, vectors, threads: int | None = None):
        v = _f32(vectors).reshape(-1, self.dim)
        lib().orc_ivfpq_add(self._h, _p(v), v.shape[0], threads or cores())

    def __len__(self):
        return lib().orc_ivfpq_len(self._h)

    def bytes_per_vector(self) -> int:
        return lib().orc_ivfpq_bytes_per_vector(self._h)

    def has_tables(self) -> bool:
        return bool(lib().orc_ivfpq_has_tables(self._h))

    def search_batch(self, queries, k: int, nprobe: int, refine: int, threads: int | None = None,
                     want_rows: bool = False):
        q = _f32(queries).reshape(-1, self.dim)
        out, counts = _results(q.shape[0], k)
        rows = lib().orc_ivfpq_search_batch(self._h, _p(q), q.shape[0], k, nprobe, refine, threads or cores(),
                                            _p(out), _p(counts))
        return (out, counts, rows) if want_rows else (out, counts)

    def save(self) -> bytes:
        n = lib().orc_ivfpq_save(self._h, None, 0)
        buf = np.empty(n, dtype=np.uint8)
        lib().orc_ivfpq_save(self._h, _p(buf), n)
        return buf.tobytes()

    @staticmethod
    def load(data: bytes) -> "IvfPq":
        buf = np.frombuffer(data, dtype=np.uint8)
        err = C.create_string_buffer(256)
        h = lib().orc_ivfpq_load(_p(buf), buf.size, err, 256)
        if not h:
            raise ValueError(err.value.decode())
        dim = int(np.frombuffer(data[12:16], dtype="<u4")[0])
        return IvfPq(h, dim)


class Hnsw:
    """src/vector/hnsw.rs."""

    def __init__(self, handle, dim: int):
        self._h, self.dim = handle, dim

    def __del__(self):
        if getattr(self, "_h", None):
            lib().orc_hnsw_free(self._h)
            self._h = None

    @staticmethod
    def build(metric: int, dim: int, vectors, m: int = 16, ef_construction: int = 200, seed: int = 1,
              threads: int = 1) -> "Hnsw":
        """`threads=1` is the only deterministic build (hnsw.rs:117-127 races by design)."""
        v = _f32(vectors).reshape(-1, dim)
        return Hnsw(lib().orc_hnsw_build(metric, dim, _p(v), v.shape[0], m, ef_construction, seed, threads), dim)

    @staticmethod
    def build_batched(metric: int, dim: int, vectors, m: int = 16, ef_construction: int = 200, seed: int = 1,
                      max_batch: int = 8192, divisor: int = 32) -> "Hnsw":
        """The batch-synchronous order of the construction (what the product's GPU build runs); deterministic."""
        v = _f32(vectors).reshape(-1, dim)
        return Hnsw(lib().orc_hnsw_build_batched(metric, dim, _p(v), v.shape[0], m, ef_construction, seed, max_batch,
                                                 divisor), dim)

    def __len__(self):
        return lib().orc_hnsw_len(self._h)

    def reachable(self) -> int:
        return lib().orc_hnsw_reachable(self._h)

    def mean_degree(self) -> float:
        return lib().orc_hnsw_mean_degree(self._h)

    def search_batch(self, queries, k: int, ef: int, threads: int | None = None, want_work: bool = False):
        q = _f32(queries).reshape(-1, self.dim)
        out, counts = _results(q.shape[0], k)
        work = np.zeros(2, dtype=np.uint64)
        lib().orc_hnsw_search_batch(self._h, _p(q), q.shape[0], k, ef, threads or cores(), _p(out), _p(counts),
                                    _p(work))
        return (out, counts, work) if want_work else (out, counts)

    def save(self) -> bytes:
        n = lib().orc_hnsw_save(self._h, None, 0)
        buf = np.empty(n, dtype=np.uint8)
        lib().orc_hnsw_save(self._h, _p(buf), n)
        return buf.tobytes()

    @staticmethod
    def load(data: bytes) -> "Hnsw":
        buf = np.frombuffer(data, dtype=np.uint8)
        err = C.create_string_buffer(256)
        h = lib().orc_hnsw_load(_p(buf), buf.size, err, 256)
        if not h:
            raise ValueError(err.value.decode())
        dim = int(np.frombuffer(data[12:16], dtype="<u4")[0])
        return Hnsw(h, dim)
