"""Python mirror of the reference's `ferrolm::vector` API over the C ABI.

Names and argument meaning follow src/vector/{mod,flat,ivfpq,hnsw}.rs:
`FlatIndex(metric, dim).add(...)/.search_batch(pool, q, k)`,
`IvfPq.train(pool, metric, dim, sample, params)/.add/.search_batch(pool, q, k, nprobe, refine)`,
`Hnsw.build(pool, metric, dim, vectors, params)/.search_batch(pool, q, k, ef)`,
with a `Context` (one GPU + stream + scratch) where the reference takes a `&Pool`.

Host arrays (numpy) go through the copying entry points; CUDA tensors go through
the `_dev` entry points and results stay on the device.  All computation happens
in libferrovec.so; this module only marshals pointers.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import numpy as np

from . import _lib
from ._lib import FerrovecError, check, fv_hnsw_params, fv_ivfpq_params, fv_stats, lib

NEIGHBOR = np.dtype([("id", "<u4"), ("distance", "<f4")])


class Metric:
    """src/vector/mod.rs:20-49."""

    L2 = 0
    InnerProduct = 1


def padded(dim: int) -> int:
    return lib().fv_padded(dim)


def normalize(data: np.ndarray) -> np.ndarray:
    """Scales each row to unit length (src/vector/mod.rs:132-141); returns a new array."""
    out = np.ascontiguousarray(data, dtype=np.float32).copy()
    n, dim = out.shape
    check(lib().fv_normalize(out.ctypes.data_as(C.c_void_p), n, dim))
    return out


def recall(found: np.ndarray, counts: np.ndarray, truth: np.ndarray, k: int) -> float:
    """src/vector/mod.rs:145-152."""
    found = np.ascontiguousarray(found)
    counts = np.ascontiguousarray(counts, dtype=np.uint32)
    truth = np.ascontiguousarray(truth, dtype=np.uint32)
    return lib().fv_recall(found.ctypes.data_as(C.c_void_p), counts.ctypes.data_as(C.c_void_p),
                           truth.ctypes.data_as(C.c_void_p), truth.shape[1], found.shape[0], k)


def datagen(kind: int, seed: int, n: int, dim: int, clusters: int, first_row: int = 0, threads: int = 0) -> np.ndarray:
    """Seeded Gaussian-mixture rows (kind 0: SIFT-like integers in [0,255]; kind 1: unit-length embeddings)."""
    out = np.empty((n, dim), dtype=np.float32)
    check(lib().fv_datagen(kind, seed, first_row, n, dim, clusters, threads, out.ctypes.data_as(C.c_void_p)))
    return out


def datagen_dev(ctx, seed: int, n: int, dim: int, clusters: int, first_row: int = 0):
    """datagen kind 0 computed on the GPU into a new device tensor (for bases too large for the host cores)."""
    import torch

    out = torch.empty((n, dim), dtype=torch.float32, device=f"cuda:{ctx.device}")
    torch.cuda.current_stream(out.device).synchronize()
    check(lib().fv_datagen_dev(ctx._h, seed, first_row, n, dim, clusters, out.data_ptr()))
    return out


def comm_unique_id() -> bytes:
    """The 128-byte id of a new group of contexts; rank 0 makes it, every rank passes it to Context.comm_init."""
    buf = (C.c_uint8 * 128)()
    check(lib().fv_comm_unique_id(buf))
    return bytes(buf)


def _is_cuda_tensor(x) -> bool:
    return hasattr(x, "is_cuda") and bool(x.is_cuda)


def _host_f32(x) -> np.ndarray:
    return np.ascontiguousarray(x, dtype=np.float32)


class Context:
    """One GPU, one stream and the scratch arena searches reuse: the stand-in for `&Pool`."""

    def __init__(self, device: int = 0):
        h = C.c_void_p()
        check(lib().fv_ctx_create(device, C.byref(h)))
        self._h = h
        self.device = device

    def close(self):
        if getattr(self, "_h", None):
            lib().fv_ctx_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def sync(self):
        check(lib().fv_ctx_sync(self._h))

    def set_timing(self, on: bool):
        check(lib().fv_ctx_set_timing(self._h, int(on)))

    def stats(self) -> dict:
        s = fv_stats()
        check(lib().fv_ctx_stats(self._h, C.byref(s)))
        return {"launches": s.launches, "uncertified": s.uncertified, "rows_scanned": s.rows_scanned,
                "dist_evals": s.dist_evals, "expansions": s.expansions, "regrown": s.regrown,
                "stage_ms": list(s.stage_ms), "rows_list_scan": s.rows_list_scan}

    def stream_handle(self) -> int:
        return lib().fv_ctx_stream(self._h) or 0

    def comm_init(self, group_id: bytes, nranks: int, rank: int):
        """Joins the group `group_id` (collective: returns when every rank has called it)."""
        buf = (C.c_uint8 * 128).from_buffer_copy(group_id)
        check(lib().fv_ctx_comm_init(self._h, buf, nranks, rank))

    @property
    def comm_rank(self) -> int:
        return lib().fv_ctx_comm_rank(self._h)

    @property
    def comm_size(self) -> int:
        return lib().fv_ctx_comm_size(self._h)

    # ---- merging per-shard results (device tensors)
    def merge_topk(self, parts, part_counts, k_out: int):
        """parts: (nparts, nq, k_in) structured as int32 pairs on the device; returns (nq, k_out) and counts."""
        import torch

        nparts, nq, k_in = parts.shape[0], parts.shape[1], parts.shape[2]
        out = torch.empty((nq, k_out, 2), dtype=torch.int32, device=parts.device)
        counts = torch.empty((nq,), dtype=torch.int32, device=parts.device)
        torch.cuda.current_stream(parts.device).synchronize()
        check(lib().fv_merge_topk_dev(self._h, parts.data_ptr(),
                                      part_counts.data_ptr() if part_counts is not None else None, nparts, nq, k_in,
                                      k_out, out.data_ptr(), counts.data_ptr()))
        return out, counts

    def merge_refine(self, adc_parts, exact_parts, part_counts, k: int):
        import torch

        nparts, nq, keep = adc_parts.shape[0], adc_parts.shape[1], adc_parts.shape[2]
        out = torch.empty((nq, k, 2), dtype=torch.int32, device=adc_parts.device)
        counts = torch.empty((nq,), dtype=torch.int32, device=adc_parts.device)
        torch.cuda.current_stream(adc_parts.device).synchronize()
        check(lib().fv_merge_refine_dev(self._h, adc_parts.data_ptr(), exact_parts.data_ptr(),
                                        part_counts.data_ptr() if part_counts is not None else None, nparts, nq, keep,
                                        k, out.data_ptr(), counts.data_ptr()))
        return out, counts


def merge_topk_static(parts, part_counts, k_out: int, out, counts):
    """Shard merge that allocates nothing, for callers that cannot: the outputs are passed in (`out` is an
    (nq, k_out, 2) int32 device tensor, `counts` (nq,) int32) and the scratch is a fixed array inside the
    library.  Limits: nq * k_out <= 262144, k_out <= 1024; calls that overlap on one GPU race on that array."""
    import torch

    nparts, nq, k_in = parts.shape[0], parts.shape[1], parts.shape[2]
    dev = parts.device.index if parts.device.index is not None else torch.cuda.current_device()
    stream = torch.cuda.current_stream(parts.device)
    check(lib().fv_merge_topk_static_dev(dev, stream.cuda_stream, parts.data_ptr(),
                                         part_counts.data_ptr() if part_counts is not None else None, nparts, nq,
                                         k_in, k_out, out.data_ptr(), counts.data_ptr()))
    return out, counts


def neighbors_from_tensor(t) -> np.ndarray:
    """(nq, k, 2) int32 device tensor -> (nq, k) NEIGHBOR array on the host."""
    a = t.cpu().numpy()
    return np.ascontiguousarray(a).view(NEIGHBOR).reshape(a.shape[0], a.shape[1])


def _search(fn, handle, queries, dim: int, k: int, extra: tuple, fn_dev):
    """Common marshalling of a search_batch call; returns (neighbours, counts)."""
    if _is_cuda_tensor(queries):
        import torch

        q = queries.contiguous().view(-1, dim)
        assert q.dtype == torch.float32
        nq = q.shape[0]
        out = torch.empty((nq, k, 2), dtype=torch.int32, device=q.device)
        counts = torch.empty((nq,), dtype=torch.int32, device=q.device)
        torch.cuda.current_stream(q.device).synchronize()  # the library runs on its own stream
        check(fn_dev(handle, q.data_ptr(), nq, k, *extra, out.data_ptr(), counts.data_ptr()))
        return out, counts
    q = _host_f32(queries).reshape(-1, dim)
    nq = q.shape[0]
    out = np.empty((nq, k), dtype=NEIGHBOR)
    counts = np.zeros(nq, dtype=np.uint32)
    check(fn(handle, q.ctypes.data_as(C.c_void_p), nq, k, *extra, out.ctypes.data_as(C.c_void_p),
             counts.ctypes.data_as(C.c_void_p)))
    return out, counts


class FlatIndex:
    """Exact search (src/vector/flat.rs)."""

    def __init__(self, ctx: Context, metric: int, dim: int):
        self.ctx, self.metric, self.dim = ctx, metric, dim
        h = C.c_void_p()
        check(lib().fv_flat_new(ctx._h, metric, dim, C.byref(h)))
        self._h = h

    def close(self):
        if getattr(self, "_h", None):
            lib().fv_flat_free(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def add(self, vectors):
        if _is_cuda_tensor(vectors):
            import torch

            v = vectors.contiguous().view(-1, self.dim)
            torch.cuda.current_stream(v.device).synchronize()
            check(lib().fv_flat_add_dev(self._h, v.data_ptr(), v.shape[0]))
        else:
            v = _host_f32(vectors).reshape(-1, self.dim)
            check(lib().fv_flat_add(self._h, v.ctypes.data_as(C.c_void_p), v.shape[0]))

    def __len__(self) -> int:
        return lib().fv_flat_len(self._h)

    def is_empty(self) -> bool:
        return len(self) == 0

    def vector(self, id: int) -> np.ndarray:
        out = np.empty(padded(self.dim), dtype=np.float32)
        check(lib().fv_flat_vector(self._h, id, out.ctypes.data_as(C.c_void_p)))
        return out

    def set_id_base(self, base: int):
        check(lib().fv_flat_set_id_base(self._h, base))

    def set_mode(self, mode: int):
        """0 automatic, 1 tensor-core front end + exact re-rank, 2 full-precision scan."""
        check(lib().fv_flat_set_mode(self._h, mode))

    def search(self, query, k: int) -> np.ndarray:
        out, counts = self.search_batch(_host_f32(query).reshape(1, self.dim), k)
        return out[0, : counts[0]]

    def search_batch(self, queries, k: int):
        return _search(lib().fv_flat_search_batch, self._h, queries, self.dim, k, (), lib().fv_flat_search_batch_dev)

    def search_sharded(self, queries, k: int):
        """Collective search over the row shards of the context's group (CUDA tensor, the same on every rank)."""
        return _search(None, self._h, queries, self.dim, k, (), lib().fv_flat_search_sharded_dev)


@dataclass
class IvfPqParams:
    """src/vector/ivfpq.rs:18-27."""

    nlist: int
    m: int
    iters: int
    keep_vectors: bool
    seed: int


class IvfPq:
    """src/vector/ivfpq.rs."""

    def __init__(self, ctx: Context, handle, dim: int):
        self.ctx, self._h, self.dim = ctx, handle, dim

    def close(self):
        if getattr(self, "_h", None):
            lib().fv_ivfpq_free(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    @staticmethod
    def train(ctx: Context, metric: int, dim: int, sample, p: IvfPqParams) -> "IvfPq":
        s = _host_f32(sample).reshape(-1, dim)
        cp = fv_ivfpq_params(p.nlist, p.m, p.iters, int(p.keep_vectors), p.seed)
        h = C.c_void_p()
        check(lib().fv_ivfpq_train(ctx._h, metric, dim, s.ctypes.data_as(C.c_void_p), s.shape[0], C.byref(cp),
                                   C.byref(h)))
        return IvfPq(ctx, h, dim)

    def add(self, vectors):
        if _is_cuda_tensor(vectors):
            import torch

            v = vectors.contiguous().view(-1, self.dim)
            torch.cuda.current_stream(v.device).synchronize()
            check(lib().fv_ivfpq_add_dev(self._h, v.data_ptr(), v.shape[0]))
            return
        v = _host_f32(vectors).reshape(-1, self.dim)
        check(lib().fv_ivfpq_add(self._h, v.ctypes.data_as(C.c_void_p), v.shape[0]))

    def set_id_base(self, base: int):
        check(lib().fv_ivfpq_set_id_base(self._h, base))

    def set_shard(self, rank: int, world: int):
        """Keep and scan only the inverted lists l with l % world == rank (give every shard the same rows)."""
        check(lib().fv_ivfpq_set_shard(self._h, rank, world))

    def set_scan_mode(self, mode: int):
        """0 chosen by size, 1 one block per query, 2 the list-major table scan, 3 the list-major tensor-core pass,
        4 that pass with its bounds from the per-query kernel (2 to 4 whenever the index allows it)."""
        check(lib().fv_ivfpq_set_scan_mode(self._h, mode))

    def set_candidate_slots(self, slots: int):
        """Candidate slots per query of the list-major scan (0 = default); overflowing queries are re-run."""
        check(lib().fv_ivfpq_set_candidate_slots(self._h, slots))

    def set_survivor_slots(self, slots: int):
        """Survivor pool entries per CTA of the tensor-core pass (0 = default); queries that lose survivors are re-run."""
        check(lib().fv_ivfpq_set_survivor_slots(self._h, slots))

    def __len__(self) -> int:
        return lib().fv_ivfpq_len(self._h)

    def bytes_per_vector(self) -> int:
        return lib().fv_ivfpq_bytes_per_vector(self._h)

    def search(self, query, k: int, nprobe: int, refine: int) -> np.ndarray:
        out, counts = self.search_batch(_host_f32(query).reshape(1, self.dim), k, nprobe, refine)
        return out[0, : counts[0]]

    def search_batch(self, queries, k: int, nprobe: int, refine: int, cells=None):
        """`cells`: the keys `coarse` returned for these queries (CUDA tensors only), to skip the coarse step."""
        if cells is not None:
            import torch

            q = queries.contiguous().view(-1, self.dim)
            nq = q.shape[0]
            assert cells.is_cuda and cells.dtype == torch.int64 and cells.is_contiguous() and cells.shape[0] == nq
            out = torch.empty((nq, k, 2), dtype=torch.int32, device=q.device)
            counts = torch.empty((nq,), dtype=torch.int32, device=q.device)
            torch.cuda.current_stream(q.device).synchronize()
            check(lib().fv_ivfpq_search_batch_cells_dev(self._h, q.data_ptr(), nq, k, nprobe, refine, cells.data_ptr(),
                                                        out.data_ptr(), counts.data_ptr()))
            return out, counts
        return _search(lib().fv_ivfpq_search_batch, self._h, queries, self.dim, k, (nprobe, refine),
                       lib().fv_ivfpq_search_batch_dev)

    def search_sharded(self, queries, k: int, nprobe: int, refine: int):
        """Collective search over the list shards of the context's group (CUDA tensor, the same on every rank)."""
        return _search(None, self._h, queries, self.dim, k, (nprobe, refine), lib().fv_ivfpq_search_sharded_dev)

    def coarse(self, queries, nprobe: int):
        """The probed cells of every query (CUDA tensor in, (nq, min(nprobe, nlist)) int64 keys out): the coarse step
        of a search on its own, so that list shards can split it by queries and exchange the keys."""
        import torch

        q = queries.contiguous().view(-1, self.dim)
        nq = q.shape[0]
        cells = torch.empty((nq, min(nprobe, lib().fv_ivfpq_nlist(self._h))), dtype=torch.int64, device=q.device)
        torch.cuda.current_stream(q.device).synchronize()
        check(lib().fv_ivfpq_coarse_dev(self._h, q.data_ptr(), nq, nprobe, cells.data_ptr()))
        return cells

    def search_candidates(self, queries, keep: int, nprobe: int, cells=None):
        """Per-shard half of a re-ranked search: best `keep` by compressed distance plus exact distances."""
        import torch

        q = queries.contiguous().view(-1, self.dim)
        nq = q.shape[0]
        adc = torch.empty((nq, keep, 2), dtype=torch.int32, device=q.device)
        exact = torch.empty((nq, keep), dtype=torch.float32, device=q.device)
        counts = torch.empty((nq,), dtype=torch.int32, device=q.device)
        torch.cuda.current_stream(q.device).synchronize()
        if cells is not None:
            assert cells.is_cuda and cells.dtype == torch.int64 and cells.is_contiguous() and cells.shape[0] == nq
            check(lib().fv_ivfpq_search_candidates_cells_dev(self._h, q.data_ptr(), nq, keep, nprobe, cells.data_ptr(),
                                                             adc.data_ptr(), exact.data_ptr(), counts.data_ptr()))
        else:
            check(lib().fv_ivfpq_search_candidates_dev(self._h, q.data_ptr(), nq, keep, nprobe, adc.data_ptr(),
                                                       exact.data_ptr(), counts.data_ptr()))
        return adc, exact, counts

    def save(self) -> bytes:
        n = lib().fv_ivfpq_save_size(self._h)
        buf = np.empty(n, dtype=np.uint8)
        w = C.c_size_t(0)
        check(lib().fv_ivfpq_save(self._h, buf.ctypes.data_as(C.c_void_p), n, C.byref(w)))
        return buf[: w.value].tobytes()

    @staticmethod
    def load(ctx: Context, data: bytes) -> "IvfPq":
        buf = np.frombuffer(data, dtype=np.uint8)
        h = C.c_void_p()
        check(lib().fv_ivfpq_load(ctx._h, buf.ctypes.data_as(C.c_void_p), buf.size, C.byref(h)))
        return IvfPq(ctx, h, int(lib().fv_ivfpq_dim(h)))


@dataclass
class HnswParams:
    """src/vector/hnsw.rs:24-40."""

    m: int = 16
    ef_construction: int = 200
    seed: int = 1


class Hnsw:
    """src/vector/hnsw.rs."""

    def __init__(self, ctx: Context, handle, dim: int):
        self.ctx, self._h, self.dim = ctx, handle, dim

    def close(self):
        if getattr(self, "_h", None):
            lib().fv_hnsw_free(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    @staticmethod
    def build(ctx: Context, metric: int, dim: int, vectors, p: HnswParams = HnswParams(), threads: int = 1) -> "Hnsw":
        v = _host_f32(vectors).reshape(-1, dim)
        cp = fv_hnsw_params(p.m, p.ef_construction, p.seed)
        h = C.c_void_p()
        check(lib().fv_hnsw_build(ctx._h, metric, dim, v.ctypes.data_as(C.c_void_p), v.shape[0], C.byref(cp), threads,
                                  C.byref(h)))
        return Hnsw(ctx, h, dim)

    @staticmethod
    def build_batched(ctx: Context, metric: int, dim: int, vectors, p: HnswParams = HnswParams(), max_batch: int = 8192,
                      divisor: int = 32) -> "Hnsw":
        """The construction (hnsw.rs:85-129, :244-320) on the GPU, in id order in batches of at most `max_batch` nodes
        and at most 1/`divisor` of the nodes already in.  Deterministic; `max_batch=1` gives the graph of the
        reference's single-thread build byte for byte."""
        v = _host_f32(vectors).reshape(-1, dim)
        cp = fv_hnsw_params(p.m, p.ef_construction, p.seed)
        h = C.c_void_p()
        check(lib().fv_hnsw_build_batched(ctx._h, metric, dim, v.ctypes.data_as(C.c_void_p), v.shape[0], C.byref(cp),
                                          max_batch, divisor, C.byref(h)))
        return Hnsw(ctx, h, dim)

    def __len__(self) -> int:
        return lib().fv_hnsw_len(self._h)

    def reachable(self) -> int:
        return lib().fv_hnsw_reachable(self._h)

    def mean_degree(self) -> float:
        return lib().fv_hnsw_mean_degree(self._h)

    def search(self, query, k: int, ef: int) -> np.ndarray:
        out, counts = self.search_batch(_host_f32(query).reshape(1, self.dim), k, ef)
        return out[0, : counts[0]]

    def search_batch(self, queries, k: int, ef: int):
        return _search(lib().fv_hnsw_search_batch, self._h, queries, self.dim, k, (ef,),
                       lib().fv_hnsw_search_batch_dev)

    def save(self) -> bytes:
        n = lib().fv_hnsw_save_size(self._h)
        buf = np.empty(n, dtype=np.uint8)
        w = C.c_size_t(0)
        check(lib().fv_hnsw_save(self._h, buf.ctypes.data_as(C.c_void_p), n, C.byref(w)))
        return buf[: w.value].tobytes()

    @staticmethod
    def load(ctx: Context, data: bytes) -> "Hnsw":
        buf = np.frombuffer(data, dtype=np.uint8)
        h = C.c_void_p()
        check(lib().fv_hnsw_load(ctx._h, buf.ctypes.data_as(C.c_void_p), buf.size, C.byref(h)))
        return Hnsw(ctx, h, int(lib().fv_hnsw_dim(h)))


def kmeans_train(ctx: Context, data, k: int, iters: int, seed: int) -> np.ndarray:
    """src/vector/kmeans.rs:39-90."""
    d = _host_f32(data)
    n, dim = d.shape
    cen = np.empty((k, dim), dtype=np.float32)
    check(lib().fv_kmeans_train(ctx._h, d.ctypes.data_as(C.c_void_p), n, dim, k, iters, seed,
                                cen.ctypes.data_as(C.c_void_p)))
    return cen


def kmeans_assign(ctx: Context, data, centroids) -> np.ndarray:
    """src/vector/kmeans.rs:22-35."""
    d, c = _host_f32(data), _host_f32(centroids)
    out = np.empty(d.shape[0], dtype=np.uint32)
    check(lib().fv_kmeans_assign(ctx._h, d.ctypes.data_as(C.c_void_p), d.shape[0], c.ctypes.data_as(C.c_void_p),
                                 c.shape[0], d.shape[1], out.ctypes.data_as(C.c_void_p)))
    return out


__all__ = ["Metric", "Context", "FlatIndex", "IvfPq", "IvfPqParams", "Hnsw", "HnswParams", "NEIGHBOR", "padded",
           "normalize", "recall", "datagen", "datagen_dev", "kmeans_train", "kmeans_assign", "neighbors_from_tensor",
           "merge_topk_static", "comm_unique_id", "FerrovecError"]
