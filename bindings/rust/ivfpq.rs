//! `src/vector/ivfpq.rs` over libferrovec: IVF-PQ training, adding, searching and the FLIVFPQ1 file on the GPU.
//! Public surface as in the reference (ivfpq.rs:18-390).  Index files are byte-compatible with the reference's
//! both ways; an index trained here is byte-identical to one the reference trains with the same seed.
use super::ffi;
use super::{Metric, Neighbor};
use crate::pool::Pool;
use std::os::raw::c_void;

#[derive(Clone, Copy, Debug)]
pub struct IvfPqParams {
    pub nlist: usize,
    /// sub-quantizers; dim must be divisible by it
    pub m: usize,
    pub iters: usize,
    /// keep the raw vectors for exact re-ranking
    pub keep_vectors: bool,
    pub seed: u64,
}

pub struct IvfPq {
    pub metric: Metric,
    pub dim: usize,
    nlist: usize,
    h: *mut c_void,
}

unsafe impl Send for IvfPq {}
unsafe impl Sync for IvfPq {}

impl IvfPq {
    fn wrap(h: *mut c_void) -> IvfPq {
        let metric = Metric::from_code(unsafe { ffi::fv_ivfpq_metric(h) } as u8).expect("metric code");
        IvfPq { metric, dim: unsafe { ffi::fv_ivfpq_dim(h) } as usize, nlist: unsafe { ffi::fv_ivfpq_nlist(h) }, h }
    }

    /// `pool` is accepted for signature compatibility: k-means assignment and PQ training run on the GPU.
    pub fn train(_pool: &Pool, metric: Metric, dim: usize, sample: &[f32], p: IvfPqParams) -> IvfPq {
        let fp = ffi::FvIvfPqParams { nlist: p.nlist, m: p.m, iters: p.iters, keep_vectors: p.keep_vectors as i32, seed: p.seed };
        let mut h = std::ptr::null_mut();
        ffi::check(unsafe { ffi::fv_ivfpq_train(ffi::gpu_ctx(), metric.code() as i32, dim as u32, sample.as_ptr(), sample.len() / dim, &fp, &mut h) });
        IvfPq::wrap(h)
    }

    pub fn len(&self) -> usize {
        unsafe { ffi::fv_ivfpq_len(self.h) }
    }

    pub fn is_empty(&self) -> bool {
        self.len() == 0
    }

    pub fn bytes_per_vector(&self) -> usize {
        unsafe { ffi::fv_ivfpq_bytes_per_vector(self.h) }
    }

    pub fn add(&mut self, _pool: &Pool, vectors: &[f32]) {
        assert_eq!(vectors.len() % self.dim, 0);
        ffi::check(unsafe { ffi::fv_ivfpq_add(self.h, vectors.as_ptr(), vectors.len() / self.dim) });
    }

    pub fn search(&self, query: &[f32], k: usize, nprobe: usize, refine: usize) -> Vec<Neighbor> {
        self.batch(query, k, nprobe, refine).pop().unwrap_or_default()
    }

    pub fn search_batch(&self, _pool: &Pool, queries: &[f32], k: usize, nprobe: usize, refine: usize) -> Vec<Vec<Neighbor>> {
        self.batch(queries, k, nprobe, refine)
    }

    fn batch(&self, queries: &[f32], k: usize, nprobe: usize, refine: usize) -> Vec<Vec<Neighbor>> {
        let nq = queries.len() / self.dim;
        let mut out = vec![ffi::FvNeighbor::default(); nq * k];
        let mut counts = vec![0u32; nq];
        ffi::check(unsafe {
            ffi::fv_ivfpq_search_batch(self.h, queries.as_ptr(), nq, k, nprobe, refine, out.as_mut_ptr(), counts.as_mut_ptr())
        });
        ffi::collect(&out, &counts, k)
    }

    pub fn save(&self) -> Vec<u8> {
        let mut buf = vec![0u8; unsafe { ffi::fv_ivfpq_save_size(self.h) }];
        let mut written = 0usize;
        ffi::check(unsafe { ffi::fv_ivfpq_save(self.h, buf.as_mut_ptr(), buf.len(), &mut written) });
        buf.truncate(written);
        buf
    }

    /// Errors carry the reference's messages ("not an IVF-PQ index file", "index file is truncated", ...).
    pub fn load(bytes: &[u8]) -> Result<IvfPq, String> {
        let mut h = std::ptr::null_mut();
        match unsafe { ffi::fv_ivfpq_load(ffi::gpu_ctx(), bytes.as_ptr(), bytes.len(), &mut h) } {
            ffi::FV_OK => Ok(IvfPq::wrap(h)),
            ffi::FV_ERR_FILE => Err(ffi::last_error()),
            _ => panic!("ferrovec: {}", ffi::last_error()),
        }
    }
}

impl Drop for IvfPq {
    fn drop(&mut self) {
        unsafe { ffi::fv_ivfpq_free(self.h) }
    }
}
