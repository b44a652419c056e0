"""Loader of libferrovec.so (the C ABI of include/ferrovec.h).

There is no Python or CPU implementation behind this module: if the shared
library is missing or cannot be loaded, importing fails with the reason.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

_HERE = os.path.dirname(os.path.abspath(__file__))
SO_PATH = os.path.join(_HERE, "libferrovec.so")
CSRC = os.path.join(_HERE, "csrc")


def build(force: bool = False, verbose: bool = False) -> str:
    """Compiles the CUDA sources for sm_100a into ferrolm_b200/libferrovec.so (needs nvcc, no GPU)."""
    cmd = ["make", "-C", CSRC, "-j", str(min(8, os.cpu_count() or 1))]
    if force:
        cmd.append("-B")
    r = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or r.returncode != 0:
        print(r.stdout)
        print(r.stderr)
    if r.returncode != 0:
        raise RuntimeError("building libferrovec.so failed")
    return SO_PATH


class fv_neighbor(C.Structure):
    _fields_ = [("id", C.c_uint32), ("distance", C.c_float)]


class fv_stats(C.Structure):
    _fields_ = [
        ("launches", C.c_uint64),
        ("uncertified", C.c_uint64),
        ("rows_scanned", C.c_uint64),
        ("dist_evals", C.c_uint64),
        ("expansions", C.c_uint64),
        ("regrown", C.c_uint64),
        ("stage_ms", C.c_float * 8),
        ("rows_list_scan", C.c_uint64),
    ]


class fv_ivfpq_params(C.Structure):
    _fields_ = [("nlist", C.c_size_t), ("m", C.c_size_t), ("iters", C.c_size_t), ("keep_vectors", C.c_int),
                ("seed", C.c_uint64)]


class fv_hnsw_params(C.Structure):
    _fields_ = [("m", C.c_size_t), ("ef_construction", C.c_size_t), ("seed", C.c_uint64)]


_vp, _sz, _i, _u32, _u64 = C.c_void_p, C.c_size_t, C.c_int, C.c_uint32, C.c_uint64
_pp = C.POINTER(C.c_void_p)

# every symbol include/ferrovec.h declares: name -> (restype, argtypes)
SIGNATURES = {
    "fv_last_error": (C.c_char_p, []),
    "fv_version": (C.c_char_p, []),
    "fv_ctx_create": (_i, [_i, _pp]),
    "fv_ctx_destroy": (None, [_vp]),
    "fv_ctx_device": (_i, [_vp]),
    "fv_ctx_sync": (_i, [_vp]),
    "fv_ctx_stream": (_vp, [_vp]),
    "fv_ctx_stats": (_i, [_vp, C.POINTER(fv_stats)]),
    "fv_ctx_set_timing": (_i, [_vp, _i]),
    "fv_flat_new": (_i, [_vp, _i, _u32, _pp]),
    "fv_flat_free": (None, [_vp]),
    "fv_flat_add": (_i, [_vp, _vp, _sz]),
    "fv_flat_add_dev": (_i, [_vp, _vp, _sz]),
    "fv_flat_len": (_sz, [_vp]),
    "fv_flat_vector": (_i, [_vp, _u32, _vp]),
    "fv_flat_search": (_i, [_vp, _vp, _sz, _vp, _vp]),
    "fv_flat_search_batch": (_i, [_vp, _vp, _sz, _sz, _vp, _vp]),
    "fv_flat_search_batch_dev": (_i, [_vp, _vp, _sz, _sz, _vp, _vp]),
    "fv_flat_set_id_base": (_i, [_vp, _u32]),
    "fv_flat_set_mode": (_i, [_vp, _i]),
    "fv_kmeans_assign": (_i, [_vp, _vp, _sz, _vp, _sz, _sz, _vp]),
    "fv_kmeans_train": (_i, [_vp, _vp, _sz, _sz, _sz, _sz, _u64, _vp]),
    "fv_ivfpq_train": (_i, [_vp, _i, _u32, _vp, _sz, C.POINTER(fv_ivfpq_params), _pp]),
    "fv_ivfpq_free": (None, [_vp]),
    "fv_ivfpq_add": (_i, [_vp, _vp, _sz]),
    "fv_ivfpq_add_dev": (_i, [_vp, _vp, _sz]),
    "fv_ivfpq_len": (_sz, [_vp]),
    "fv_ivfpq_bytes_per_vector": (_sz, [_vp]),
    "fv_ivfpq_search": (_i, [_vp, _vp, _sz, _sz, _sz, _vp, _vp]),
    "fv_ivfpq_search_batch": (_i, [_vp, _vp, _sz, _sz, _sz, _sz, _vp, _vp]),
    "fv_ivfpq_search_batch_dev": (_i, [_vp, _vp, _sz, _sz, _sz, _sz, _vp, _vp]),
    "fv_ivfpq_set_id_base": (_i, [_vp, _u32]),
    "fv_ivfpq_set_shard": (_i, [_vp, _i, _i]),
    "fv_ivfpq_search_candidates_dev": (_i, [_vp, _vp, _sz, _sz, _sz, _vp, _vp, _vp]),
    "fv_ivfpq_nlist": (_sz, [_vp]),
    "fv_ivfpq_dim": (_u32, [_vp]),
    "fv_ivfpq_metric": (_i, [_vp]),
    "fv_hnsw_dim": (_u32, [_vp]),
    "fv_hnsw_metric": (_i, [_vp]),
    "fv_ivfpq_set_scan_mode": (_i, [_vp, _i]),
    "fv_ivfpq_set_candidate_slots": (_i, [_vp, _sz]),
    "fv_ivfpq_set_survivor_slots": (_i, [_vp, _sz]),
    "fv_debug_bounds_build": (_i, []),
    "fv_debug_tc_fault": (_i, [C.c_longlong, _i]),
    "fv_ivfpq_coarse_dev": (_i, [_vp, _vp, _sz, _sz, _vp]),
    "fv_ivfpq_search_batch_cells_dev": (_i, [_vp, _vp, _sz, _sz, _sz, _sz, _vp, _vp, _vp]),
    "fv_ivfpq_search_candidates_cells_dev": (_i, [_vp, _vp, _sz, _sz, _sz, _vp, _vp, _vp, _vp]),
    "fv_ivfpq_save_size": (_sz, [_vp]),
    "fv_ivfpq_save": (_i, [_vp, _vp, _sz, C.POINTER(_sz)]),
    "fv_ivfpq_load": (_i, [_vp, _vp, _sz, _pp]),
    "fv_hnsw_build": (_i, [_vp, _i, _u32, _vp, _sz, C.POINTER(fv_hnsw_params), _i, _pp]),
    "fv_hnsw_build_batched": (_i, [_vp, _i, _u32, _vp, _sz, C.POINTER(fv_hnsw_params), _sz, _sz, _pp]),
    "fv_hnsw_free": (None, [_vp]),
    "fv_hnsw_len": (_sz, [_vp]),
    "fv_hnsw_reachable": (_sz, [_vp]),
    "fv_hnsw_mean_degree": (C.c_double, [_vp]),
    "fv_hnsw_search": (_i, [_vp, _vp, _sz, _sz, _vp, _vp]),
    "fv_hnsw_search_batch": (_i, [_vp, _vp, _sz, _sz, _sz, _vp, _vp]),
    "fv_hnsw_search_batch_dev": (_i, [_vp, _vp, _sz, _sz, _sz, _vp, _vp]),
    "fv_hnsw_save_size": (_sz, [_vp]),
    "fv_hnsw_save": (_i, [_vp, _vp, _sz, C.POINTER(_sz)]),
    "fv_hnsw_load": (_i, [_vp, _vp, _sz, _pp]),
    "fv_padded": (_sz, [_sz]),
    "fv_normalize": (_i, [_vp, _sz, _sz]),
    "fv_recall": (C.c_double, [_vp, _vp, _vp, _sz, _sz, _sz]),
    "fv_comm_unique_id": (_i, [_vp]),
    "fv_ctx_comm_init": (_i, [_vp, _vp, _i, _i]),
    "fv_ctx_comm_rank": (_i, [_vp]),
    "fv_ctx_comm_size": (_i, [_vp]),
    "fv_flat_search_sharded_dev": (_i, [_vp, _vp, _sz, _sz, _vp, _vp]),
    "fv_ivfpq_search_sharded_dev": (_i, [_vp, _vp, _sz, _sz, _sz, _sz, _vp, _vp]),
    "fv_merge_topk_dev": (_i, [_vp, _vp, _vp, _sz, _sz, _sz, _sz, _vp, _vp]),
    "fv_merge_refine_dev": (_i, [_vp, _vp, _vp, _vp, _sz, _sz, _sz, _sz, _vp, _vp]),
    "fv_merge_topk_static_dev": (_i, [_i, _vp, _vp, _vp, _sz, _sz, _sz, _sz, _vp, _vp]),
    "fv_datagen": (_i, [_i, _u64, _sz, _sz, _sz, _sz, _i, _vp]),
    "fv_read_fvecs": (_i, [C.c_char_p, _sz, _pp, C.POINTER(_sz), C.POINTER(_sz)]),
    "fv_read_ivecs": (_i, [C.c_char_p, _sz, _pp, C.POINTER(_sz), C.POINTER(_sz)]),
    "fv_free": (None, [_vp]),
    "fv_datagen_dev": (_i, [_vp, _u64, _sz, _sz, _sz, _sz, _vp]),
}

_lib = None


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(SO_PATH):
            raise ImportError(
                f"{SO_PATH} is missing: build it with `python -c 'import __graft_entry__ as g; g.build()'` "
                "(nvcc, sm_100a). There is no fallback implementation.")
        L = C.CDLL(SO_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(L, name)  # AttributeError here means the .so is stale
            fn.restype = res
            fn.argtypes = args
        _lib = L
    return _lib


class FerrovecError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"ferrovec status {status}: {message}")
        self.status = status


FV_OK, FV_ERR_ARG, FV_ERR_FILE, FV_ERR_CUDA, FV_ERR_TIMEOUT, FV_ERR_OVERFLOW, FV_ERR_UNSUPPORTED, FV_ERR_NOMEM, FV_ERR_COMM = range(9)


def check(status: int):
    if status != 0:
        raise FerrovecError(status, lib().fv_last_error().decode(errors="replace"))
