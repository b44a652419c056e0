// Host-side internals shared by the translation units of libferrovec.
#pragma once

#include <cuda_runtime.h>

#include <cstring>
#include <memory>
#include <mutex>
#include <string>
#include <vector>

#include "common.cuh"

// A growable device allocation (raw bytes).
struct DevBuf {
  void* p = nullptr;
  size_t cap = 0;
  ~DevBuf() { release(); }
  DevBuf() = default;
  DevBuf(const DevBuf&) = delete;
  DevBuf& operator=(const DevBuf&) = delete;
  void release() {
    if (p) cudaFree(p);
    p = nullptr;
    cap = 0;
  }
  // Makes room for `bytes`; contents are NOT kept.
  int reserve(size_t bytes) {
    if (bytes <= cap) return FV_OK;
    release();
    size_t want = bytes + bytes / 8 + 256;
    cudaError_t e = cudaMalloc(&p, want);
    if (e != cudaSuccess) {
      p = nullptr;
      (void)cudaGetLastError();
      return fv::fail(FV_ERR_NOMEM, "cudaMalloc of " + std::to_string(want) + " bytes: " + cudaGetErrorString(e));
    }
    cap = want;
    return FV_OK;
  }
  // Makes room for `bytes`, keeping the first `keep` bytes.
  int grow(size_t bytes, size_t keep, cudaStream_t s) {
    if (bytes <= cap) return FV_OK;
    size_t want = bytes > 2 * cap ? bytes : 2 * cap;
    void* np = nullptr;
    cudaError_t e = cudaMalloc(&np, want);
    if (e != cudaSuccess && want > bytes) {
      (void)cudaGetLastError();
      want = bytes;
      e = cudaMalloc(&np, want);
    }
    if (e != cudaSuccess) {
      (void)cudaGetLastError();
      return fv::fail(FV_ERR_NOMEM, "cudaMalloc of " + std::to_string(want) + " bytes: " + cudaGetErrorString(e));
    }
    if (keep && p) {
      e = cudaMemcpyAsync(np, p, keep, cudaMemcpyDeviceToDevice, s);
      if (e == cudaSuccess) e = cudaStreamSynchronize(s);
      if (e != cudaSuccess) {
        cudaFree(np);
        return fv::fail(FV_ERR_CUDA, std::string("device copy while growing: ") + cudaGetErrorString(e));
      }
    }
    if (p) cudaFree(p);
    p = np;
    cap = want;
    return FV_OK;
  }
  template <class T>
  T* as() const {
    return static_cast<T*>(p);
  }
};

enum { FV_NSCRATCH = 18, FV_NSTAGE = 8 };

struct fv_ctx {
  // Every entry point that uses the stream, the scratch arena, the events or the counters holds this lock for the
  // whole call (fv::CtxGuard): the reference's search methods take &self and its index types are Sync
  // (hnsw.rs:42-77, flat.rs:56-66), so several host threads may search indexes of one context at once; here
  // their calls run one after the other.  Recursive because the host-pointer entry points call their _dev twins.
  std::recursive_mutex mu;
  int device = 0;
  cudaStream_t stream = nullptr;
  int sm_count = 0;
  size_t smem_optin = 0;
  DevBuf scratch[FV_NSCRATCH];  // reused between calls; indices are private to each search routine
  fv_stats stats{};
  bool timing = false;
  cudaEvent_t ev[FV_NSTAGE + 1] = {};
  int ev_used = 0;
  int* d_flags = nullptr;  // small device word array for error / overflow flags
  bool stage_outer = false;  // an enclosing call owns the stage table: nested searches leave it alone
  // the group this context belongs to (fv_ctx_comm_init): one rank per GPU, NCCL over NVLink for the one exchange step
  void* comm = nullptr;      // ncclComm_t
  int comm_rank = 0, comm_size = 1;
  int refs = 0;            // indexes alive on this context
  bool closing = false;    // fv_ctx_destroy was called while indexes were alive
};

namespace fv {

// RAII: makes the context's device current for the duration of a call.
struct DeviceGuard {
  int prev = -1;
  bool ok = true;
  explicit DeviceGuard(int dev) {
    if (cudaGetDevice(&prev) != cudaSuccess) prev = -1;
    if (prev != dev) ok = cudaSetDevice(dev) == cudaSuccess;
  }
  ~DeviceGuard() {
    if (prev >= 0) cudaSetDevice(prev);
  }
};

// Held by an entry point for its whole duration: the context's lock, then its device made current.
struct CtxGuard {
  std::unique_lock<std::recursive_mutex> lk;
  DeviceGuard dg;
  bool ok;
  explicit CtxGuard(fv_ctx* ctx) : lk(ctx->mu), dg(ctx->device), ok(dg.ok) {}
};

// Indexes keep their context alive: destruction is deferred until the last one is freed.
void ctx_retain(fv_ctx* ctx);
void ctx_release(fv_ctx* ctx);

// stage timing helpers (no-ops unless ctx->timing)
void stage_begin(fv_ctx* ctx);
void stage_mark(fv_ctx* ctx);  // closes the current stage
void stage_end(fv_ctx* ctx);   // after the stream is synchronised: fills stats.stage_ms

// A call that runs several searches under one stage table (the sharded searches): begins the table, keeps the nested
// calls from restarting or marking it, and closes it when the call returns (the stream is synchronised by then).
struct StageScope {
  fv_ctx* ctx;
  explicit StageScope(fv_ctx* c) : ctx(c) {
    stage_begin(c);
    c->stage_outer = true;
  }
  ~StageScope() {
    ctx->stage_outer = false;
    stage_end(ctx);
  }
};
void stage_mark_outer(fv_ctx* ctx);  // the enclosing call's own marks

// ---- exchange between the ranks of the context's group (comm.cu): every rank contributes `bytes` and receives
// all contributions, rank-major, on the context's stream.
// Debug build (FV_BOUNDS): FV_ERR_OVERFLOW if a checked gather index of that file's kernels was out of range since
// the last call; always FV_OK in the normal build.  Call after the stream has been synchronized.
int bounds_report_ivfpq_scan();
int bounds_report_hnsw();
int bounds_report_hnsw_build();

int comm_all_gather(fv_ctx* ctx, const void* d_send, void* d_recv, size_t bytes);
void comm_destroy(fv_ctx* ctx);

// merge of per-shard result lists (flat.cu): nparts blocks of nq * k_in neighbours -> the k_out best per query.
// part_stride: neighbours between the starts of two blocks (0: nq * k_in, the blocks are adjacent)
int merge_topk_impl(fv_ctx* ctx, const fv_neighbor* d_parts, const uint32_t* d_part_counts, size_t nparts, size_t nq,
                    size_t k_in, size_t k_out, fv_neighbor* d_out, uint32_t* d_counts, size_t part_stride = 0);

// ---- the full-precision scan (flat.cu): for every query the L best rows by (distance, id).
// d_out_keys: nq * L keys, ascending, FV_EMPTY_KEY padded.  `prefilter_inf`: a distance must be
// < +inf to enter (flat.rs:45); off for the coarse quantizer, where every cell is pushed (ivfpq.rs:213).
// `d_query_ids` (optional) selects a subset of the query rows: query i is d_queries[d_query_ids[i]].
int exact_scan(fv_ctx* ctx, int metric, const float* d_rows, size_t n, int pd, const float* d_queries,
               size_t q_stride, const uint32_t* d_query_ids, size_t nq, int L, bool prefilter_inf,
               uint32_t id_base, u64* d_out_keys, int scratch_slot);

// keys -> fv_neighbor rows and counts.  in: nq * L keys (ascending), out: nq * k neighbours.
int keys_to_neighbors(fv_ctx* ctx, const u64* d_keys, size_t nq, int L, int k, fv_neighbor* d_out,
                      uint32_t* d_counts, const uint32_t* d_query_ids = nullptr);

// ---- tensor-core front end of exact search (gemm_topk.cu): 16-bit operand copy of a row set, searched with the
// sampled-bound GEMM, exact re-rank and certificate; result keys are those of the full-precision chain.
struct TcSide;
void tc_free(TcSide* tc);
int tc_append(fv_ctx* ctx, TcSide** tc, int metric, const float* d_rows_new, size_t n_old, size_t n_new, int pd);
// `prefilter_inf`: what the full-precision scan that re-runs uncertified queries is told (see exact_scan).
int tc_search(fv_ctx* ctx, TcSide* tc, int metric, const float* d_rows, size_t n, int pd, const float* d_queries,
              size_t nq, int k, uint32_t id_base, u64* d_out_keys, bool mark_stages, bool prefilter_inf);
bool tc_usable(const TcSide* tc, size_t n, size_t nq, int k);

// ---- the same kernel in task mode, for callers that bring their own operand rows and work table (the IVF-PQ scan).
struct TcInfo {
  int Kp;            // operand row length (padded dimension rounded up to 64)
  bool bf16;         // operand type (else fp16)
  size_t n;          // rows of the side
  float max_norm2, min_v, max_v;
  bool not_finite;
};
void tc_info(const TcSide* tc, TcInfo* out);
// Device word that a bounded wait inside the kernel sets when it runs out.  tc_list_pass does not clear it: a caller
// that launches several passes clears it once (cudaMemsetAsync on the context's stream) and reads it after the last.
int* tc_error_word(TcSide* tc);
// Scores the tile_rows (256 or 128) operand rows of every task against its run of side rows: d_tasks[t] = {first operand row, first side
// row (a multiple of 8), units of 256 side rows, valid side rows}.  Every (operand row, side row) whose score
// ||b||^2 - 2<a, b> (L2; -<a, b> for inner product, operand rows being pre-scaled) is below d_thr[operand row] goes to
// the survivor pool as (operand row << 32 | side row relative to the task's first): CTA c of *grid_out fills
// d_pool[c * pool_cap ..] and writes its count (which may exceed pool_cap: overflow) to d_pool_cnt[c]; a survivor
// that does not fit is dropped and d_dropped[d_row_owner[operand row]] set to 1.  The CTAs draw the tasks in table
// order from the counter *d_next_task (which this call zeroes): sort the table longest first.  Asynchronous.
// Minima variant (d_minima != null): no survivors; instead, for the first d_task_rows[t] operand rows of task t, the
// smallest score of every 32 side rows (rows beyond the task's valid ones as +inf) goes to
// d_minima[d_task_moff[t] + (operand row in the task * units + unit) * 8 + side row in the unit / 32]; a task with
// d_task_moff[t] == 0xFFFFFFFF writes nothing.  d_thr and the pool are not used then.
int tc_list_pass(fv_ctx* ctx, TcSide* tc, int metric, const uint16_t* d_A, size_t a_rows, const float* d_thr,
                 const uint4* d_tasks, const uint32_t* d_ntasks, unsigned int* d_next_task, u64* d_pool, unsigned int* d_pool_cnt,
                 unsigned int pool_cap, const uint32_t* d_row_owner, uint32_t* d_dropped, int* grid_out, int tile_rows = 256,
                 float* d_minima = nullptr, const uint32_t* d_task_moff = nullptr, const uint32_t* d_task_rows = nullptr);

// pads rows of `dim` floats to `pd` on the device (host or device source)
int upload_padded(fv_ctx* ctx, const float* src, bool src_is_device, size_t n, size_t dim, size_t pd, float* d_dst);

}  // namespace fv
