//! `src/vector/hnsw.rs` over libferrovec: the graph is built by the library, on the GPU in batches (`build`, what a
//! pool of many threads is to the reference: nodes in flight that do not see one another, but with a result that
//! does not depend on timing) or on the host cores (`build_on_host`: the reference's algorithm on `pool.threads()`
//! threads; one thread gives the reference's single-thread graph byte for byte), and searched on the GPU, one warp
//! per query.  Public surface as in the reference (hnsw.rs:24-466).
use super::ffi;
use super::{Metric, Neighbor};
use crate::pool::Pool;
use std::os::raw::c_void;

#[derive(Clone, Copy, Debug)]
pub struct HnswParams {
    /// links per node above layer 0 (layer 0 keeps 2m)
    pub m: usize,
    pub ef_construction: usize,
    pub seed: u64,
}

impl Default for HnswParams {
    fn default() -> Self {
        HnswParams { m: 16, ef_construction: 200, seed: 1 }
    }
}

pub struct Hnsw {
    pub metric: Metric,
    pub dim: usize,
    h: *mut c_void,
}

unsafe impl Send for Hnsw {}
unsafe impl Sync for Hnsw {}

impl Hnsw {
    fn wrap(h: *mut c_void) -> Hnsw {
        let metric = Metric::from_code(unsafe { ffi::fv_hnsw_metric(h) } as u8).expect("metric code");
        Hnsw { metric, dim: unsafe { ffi::fv_hnsw_dim(h) } as usize, h }
    }

    /// hnsw.rs:85.  A pool of one thread asks for the deterministic single-thread graph and gets it (batches of one
    /// node); any other pool gets batches of up to 8192 nodes and 1/32 of the graph.
    pub fn build(pool: &Pool, metric: Metric, dim: usize, vectors: &[f32], p: HnswParams) -> Hnsw {
        let fp = ffi::FvHnswParams { m: p.m, ef_construction: p.ef_construction, seed: p.seed };
        let (max_batch, divisor) = if pool.threads() == 1 { (1, 1) } else { (8192, 32) };
        let mut h = std::ptr::null_mut();
        ffi::check(unsafe {
            ffi::fv_hnsw_build_batched(ffi::gpu_ctx(), metric.code() as i32, dim as u32, vectors.as_ptr(), vectors.len() / dim, &fp, max_batch, divisor, &mut h)
        });
        Hnsw::wrap(h)
    }

    /// The same construction on the host cores, with the reference's locks and its timing-dependent result.
    pub fn build_on_host(pool: &Pool, metric: Metric, dim: usize, vectors: &[f32], p: HnswParams) -> Hnsw {
        let fp = ffi::FvHnswParams { m: p.m, ef_construction: p.ef_construction, seed: p.seed };
        let mut h = std::ptr::null_mut();
        ffi::check(unsafe {
            ffi::fv_hnsw_build(ffi::gpu_ctx(), metric.code() as i32, dim as u32, vectors.as_ptr(), vectors.len() / dim, &fp, pool.threads() as i32, &mut h)
        });
        Hnsw::wrap(h)
    }

    pub fn len(&self) -> usize {
        unsafe { ffi::fv_hnsw_len(self.h) }
    }

    pub fn is_empty(&self) -> bool {
        self.len() == 0
    }

    pub fn search(&self, query: &[f32], k: usize, ef: usize) -> Vec<Neighbor> {
        self.batch(query, k, ef).pop().unwrap_or_default()
    }

    pub fn search_batch(&self, _pool: &Pool, queries: &[f32], k: usize, ef: usize) -> Vec<Vec<Neighbor>> {
        self.batch(queries, k, ef)
    }

    fn batch(&self, queries: &[f32], k: usize, ef: usize) -> Vec<Vec<Neighbor>> {
        let nq = queries.len() / self.dim;
        let mut out = vec![ffi::FvNeighbor::default(); nq * k];
        let mut counts = vec![0u32; nq];
        ffi::check(unsafe { ffi::fv_hnsw_search_batch(self.h, queries.as_ptr(), nq, k, ef, out.as_mut_ptr(), counts.as_mut_ptr()) });
        ffi::collect(&out, &counts, k)
    }

    pub fn reachable(&self) -> usize {
        unsafe { ffi::fv_hnsw_reachable(self.h) }
    }

    pub fn mean_degree(&self) -> f64 {
        unsafe { ffi::fv_hnsw_mean_degree(self.h) }
    }

    pub fn save(&self) -> Vec<u8> {
        let mut buf = vec![0u8; unsafe { ffi::fv_hnsw_save_size(self.h) }];
        let mut written = 0usize;
        ffi::check(unsafe { ffi::fv_hnsw_save(self.h, buf.as_mut_ptr(), buf.len(), &mut written) });
        buf.truncate(written);
        buf
    }

    /// Errors carry the reference's messages ("not an HNSW index file", "index file is truncated", ...).
    pub fn load(bytes: &[u8]) -> Result<Hnsw, String> {
        let mut h = std::ptr::null_mut();
        match unsafe { ffi::fv_hnsw_load(ffi::gpu_ctx(), bytes.as_ptr(), bytes.len(), &mut h) } {
            ffi::FV_OK => Ok(Hnsw::wrap(h)),
            ffi::FV_ERR_FILE => Err(ffi::last_error()),
            _ => panic!("ferrovec: {}", ffi::last_error()),
        }
    }
}

impl Drop for Hnsw {
    fn drop(&mut self) {
        unsafe { ffi::fv_hnsw_free(self.h) }
    }
}
