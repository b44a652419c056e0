//! `extern "C"` declarations for libferrovec (include/ferrovec.h) and the two helpers every wrapper uses.
#![allow(dead_code)]
use std::ffi::CStr;
use std::os::raw::{c_char, c_int, c_void};
use std::sync::OnceLock;

#[repr(C)]
#[derive(Clone, Copy, Default)]
pub struct FvNeighbor {
    pub id: u32,
    pub distance: f32,
} // = vector::Neighbor (mod.rs:52-56)

#[repr(C)]
pub struct FvIvfPqParams {
    pub nlist: usize,
    pub m: usize,
    pub iters: usize,
    pub keep_vectors: c_int,
    pub seed: u64,
}

#[repr(C)]
pub struct FvHnswParams {
    pub m: usize,
    pub ef_construction: usize,
    pub seed: u64,
}

pub const FV_OK: c_int = 0;
pub const FV_ERR_FILE: c_int = 2;

extern "C" {
    pub fn fv_last_error() -> *const c_char;
    pub fn fv_ctx_create(device: c_int, out: *mut *mut c_void) -> c_int;
    pub fn fv_ctx_destroy(ctx: *mut c_void);
    // FlatIndex (flat.rs)
    pub fn fv_flat_new(ctx: *mut c_void, metric: c_int, dim: u32, out: *mut *mut c_void) -> c_int;
    pub fn fv_flat_free(ix: *mut c_void);
    pub fn fv_flat_add(ix: *mut c_void, vectors: *const f32, n: usize) -> c_int;
    pub fn fv_flat_len(ix: *const c_void) -> usize;
    pub fn fv_flat_vector(ix: *const c_void, id: u32, out_padded: *mut f32) -> c_int;
    pub fn fv_flat_search_batch(ix: *mut c_void, q: *const f32, nq: usize, k: usize, out: *mut FvNeighbor, counts: *mut u32) -> c_int;
    // IvfPq (ivfpq.rs)
    pub fn fv_ivfpq_train(ctx: *mut c_void, metric: c_int, dim: u32, sample: *const f32, n: usize, p: *const FvIvfPqParams, out: *mut *mut c_void) -> c_int;
    pub fn fv_ivfpq_free(ix: *mut c_void);
    pub fn fv_ivfpq_add(ix: *mut c_void, vectors: *const f32, n: usize) -> c_int;
    pub fn fv_ivfpq_len(ix: *const c_void) -> usize;
    pub fn fv_ivfpq_bytes_per_vector(ix: *const c_void) -> usize;
    pub fn fv_ivfpq_nlist(ix: *const c_void) -> usize;
    pub fn fv_ivfpq_search_batch(ix: *mut c_void, q: *const f32, nq: usize, k: usize, nprobe: usize, refine: usize, out: *mut FvNeighbor, counts: *mut u32) -> c_int;
    pub fn fv_ivfpq_save_size(ix: *const c_void) -> usize;
    pub fn fv_ivfpq_save(ix: *const c_void, buf: *mut u8, cap: usize, written: *mut usize) -> c_int;
    pub fn fv_ivfpq_load(ctx: *mut c_void, bytes: *const u8, len: usize, out: *mut *mut c_void) -> c_int;
    pub fn fv_ivfpq_metric(ix: *const c_void) -> c_int;
    pub fn fv_ivfpq_dim(ix: *const c_void) -> u32;
    // Hnsw (hnsw.rs)
    pub fn fv_hnsw_build(ctx: *mut c_void, metric: c_int, dim: u32, vectors: *const f32, n: usize, p: *const FvHnswParams, threads: c_int, out: *mut *mut c_void) -> c_int;
    pub fn fv_hnsw_build_batched(ctx: *mut c_void, metric: c_int, dim: u32, vectors: *const f32, n: usize, p: *const FvHnswParams, max_batch: usize, divisor: usize, out: *mut *mut c_void) -> c_int;
    pub fn fv_hnsw_free(ix: *mut c_void);
    pub fn fv_hnsw_len(ix: *const c_void) -> usize;
    pub fn fv_hnsw_reachable(ix: *const c_void) -> usize;
    pub fn fv_hnsw_mean_degree(ix: *const c_void) -> f64;
    pub fn fv_hnsw_search_batch(ix: *mut c_void, q: *const f32, nq: usize, k: usize, ef: usize, out: *mut FvNeighbor, counts: *mut u32) -> c_int;
    pub fn fv_hnsw_save_size(ix: *const c_void) -> usize;
    pub fn fv_hnsw_save(ix: *const c_void, buf: *mut u8, cap: usize, written: *mut usize) -> c_int;
    pub fn fv_hnsw_load(ctx: *mut c_void, bytes: *const u8, len: usize, out: *mut *mut c_void) -> c_int;
    pub fn fv_hnsw_metric(ix: *const c_void) -> c_int;
    pub fn fv_hnsw_dim(ix: *const c_void) -> u32;
    // a group of GPUs (one context per rank) and the collective searches over a sharded index
    pub fn fv_comm_unique_id(id128: *mut u8) -> c_int;
    pub fn fv_ctx_comm_init(ctx: *mut c_void, id128: *const u8, nranks: c_int, rank: c_int) -> c_int;
    pub fn fv_flat_set_id_base(ix: *mut c_void, id_base: u32) -> c_int;
    pub fn fv_ivfpq_set_shard(ix: *mut c_void, rank: c_int, world: c_int) -> c_int;
    pub fn fv_flat_search_sharded_dev(ix: *mut c_void, d_queries: *const f32, nq: usize, k: usize, d_out: *mut FvNeighbor, d_counts: *mut u32) -> c_int;
    pub fn fv_ivfpq_search_sharded_dev(ix: *mut c_void, d_queries: *const f32, nq: usize, k: usize, nprobe: usize, refine: usize, d_out: *mut FvNeighbor, d_counts: *mut u32) -> c_int;
}

/// The last error of this thread, as the library words it.
pub fn last_error() -> String {
    unsafe { CStr::from_ptr(fv_last_error()) }.to_string_lossy().into_owned()
}

/// Panics with the library's message on any failure, as the reference panics on its own precondition failures
/// (Cargo.toml: panic = "abort").
pub fn check(status: c_int) {
    if status != FV_OK {
        panic!("ferrovec: {}", last_error());
    }
}

struct Ctx(*mut c_void);
unsafe impl Send for Ctx {}
unsafe impl Sync for Ctx {} // the library serialises callers of one context on a mutex

/// The process-wide GPU context (device FERROVEC_DEVICE, default 0).  The library has no CPU path: without an
/// sm_100 device this panics with its message.
pub fn gpu_ctx() -> *mut c_void {
    static CTX: OnceLock<Ctx> = OnceLock::new();
    CTX.get_or_init(|| {
        let dev = std::env::var("FERROVEC_DEVICE").ok().and_then(|s| s.parse().ok()).unwrap_or(0);
        let mut h = std::ptr::null_mut();
        check(unsafe { fv_ctx_create(dev, &mut h) });
        Ctx(h)
    })
    .0
}

/// (out, counts) of a batch call -> the reference's Vec<Vec<Neighbor>>.
pub fn collect(out: &[FvNeighbor], counts: &[u32], k: usize) -> Vec<Vec<super::Neighbor>> {
    counts
        .iter()
        .enumerate()
        .map(|(i, &c)| out[i * k..i * k + c as usize].iter().map(|n| super::Neighbor { id: n.id, distance: n.distance }).collect())
        .collect()
}
