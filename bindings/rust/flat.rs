//! `src/vector/flat.rs` over libferrovec: exact search on the GPU.  Public surface as in the reference
//! (flat.rs:7-66).  The rows live in device memory; a padded host copy is kept only for `vector()`, which hands
//! out a slice as the reference does.
use super::ffi;
use super::{pad, padded, Metric, Neighbor};
use crate::pool::Pool;
use std::os::raw::c_void;

pub struct FlatIndex {
    pub metric: Metric,
    pub dim: usize,
    h: *mut c_void,
    data: Vec<f32>, // rows padded to padded(dim), as FlatIndex::data in the reference (flat.rs:10-12)
}

// The library serialises the callers of one context; search takes &self as in the reference.
unsafe impl Send for FlatIndex {}
unsafe impl Sync for FlatIndex {}

impl FlatIndex {
    pub fn new(metric: Metric, dim: usize) -> FlatIndex {
        let mut h = std::ptr::null_mut();
        ffi::check(unsafe { ffi::fv_flat_new(ffi::gpu_ctx(), metric.code() as i32, dim as u32, &mut h) });
        FlatIndex { metric, dim, h, data: Vec::new() }
    }

    pub fn add(&mut self, vectors: &[f32]) {
        assert_eq!(vectors.len() % self.dim, 0); // flat.rs:25
        ffi::check(unsafe { ffi::fv_flat_add(self.h, vectors.as_ptr(), vectors.len() / self.dim) });
        self.data.extend_from_slice(&pad(vectors, self.dim));
    }

    pub fn len(&self) -> usize {
        unsafe { ffi::fv_flat_len(self.h) }
    }

    pub fn is_empty(&self) -> bool {
        self.len() == 0
    }

    pub fn vector(&self, id: u32) -> &[f32] {
        let pd = padded(self.dim);
        &self.data[id as usize * pd..(id as usize + 1) * pd]
    }

    pub fn search(&self, query: &[f32], k: usize) -> Vec<Neighbor> {
        self.batch(query, k).pop().unwrap_or_default()
    }

    /// `pool` is accepted for signature compatibility; the batch is one GPU call.
    pub fn search_batch(&self, _pool: &Pool, queries: &[f32], k: usize) -> Vec<Vec<Neighbor>> {
        self.batch(queries, k)
    }

    fn batch(&self, queries: &[f32], k: usize) -> Vec<Vec<Neighbor>> {
        let nq = queries.len() / self.dim;
        let mut out = vec![ffi::FvNeighbor::default(); nq * k];
        let mut counts = vec![0u32; nq];
        ffi::check(unsafe { ffi::fv_flat_search_batch(self.h, queries.as_ptr(), nq, k, out.as_mut_ptr(), counts.as_mut_ptr()) });
        ffi::collect(&out, &counts, k)
    }
}

impl Drop for FlatIndex {
    fn drop(&mut self) {
        unsafe { ffi::fv_flat_free(self.h) }
    }
}
