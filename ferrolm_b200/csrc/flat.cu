// FlatIndex (src/vector/flat.rs) and the full-precision scan that every index shares.
//
// exact_scan_kernel evaluates the reference's distance chain (src/kernels.rs:200-231) for
// (query, row) pairs and keeps, per query, the L smallest (distance, id) keys.  A warp owns
// QT queries (in shared memory) and walks rows 32 at a time, one row per lane, so the rows a
// warp sees have ascending ids and the strict pre-filter of flat.rs:45 is the lexicographic
// order.  All warps of a block sweep the same rows.  TILE: the block first copies the 32 rows of a step into shared
// memory with coalesced loads (row stride pd + 4 floats: a lane's 16-byte reads of its own row then fall on
// different banks within every quarter-warp); without it every lane streams its row from global memory, 32 cache
// lines per load instruction, and the L1 data pipe -- not the FMAs -- sets the pace (measured: 78 % of its peak
// on the coarse step of an IVF-PQ search).
#include <algorithm>

#include "internal.h"

namespace fv {

template <int QT, bool IS_L2, bool TILE>
__global__ void __launch_bounds__(128)
    exact_scan_kernel(const float* __restrict__ rows, size_t n, int pd, const float* __restrict__ queries,
                      size_t q_stride, const uint32_t* __restrict__ qids, size_t nq, int L, int prefilter_inf,
                      uint32_t id_base, size_t rows_per_split, u64* __restrict__ parts, u64* __restrict__ dense,
                      size_t dense_stride) {
  unsigned char* smem_raw = dyn_smem();
  const int W = blockDim.x >> 5;
  const int w = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  float* sq = reinterpret_cast<float*>(smem_raw);                               // [W*QT][pd]
  u64* lists = reinterpret_cast<u64*>(smem_raw + size_t(W) * QT * pd * sizeof(float));  // [W*QT][L]
  const int tstride = pd + 4;
  float* tile = reinterpret_cast<float*>(smem_raw + ((size_t(W) * QT * (size_t(pd) * 4 + size_t(L) * 8) + 15) & ~size_t(15)));  // TILE: [32][pd + 4]

  const size_t q0 = (size_t(blockIdx.x) * W + w) * QT;  // first query of this warp
  const int nqw = q0 < nq ? int(min(size_t(QT), nq - q0)) : 0;
  float* myq = sq + size_t(w) * QT * pd;
  u64* mylists = lists + size_t(w) * QT * L;
  for (int qi = 0; qi < QT; ++qi) {
    if (qi < nqw) {
      const size_t src = qids ? size_t(qids[q0 + qi]) : (q0 + qi);
      for (int c = lane; c < pd; c += 32) myq[qi * pd + c] = queries[src * q_stride + c];
    } else {
      for (int c = lane; c < pd; c += 32) myq[qi * pd + c] = 0.f;
    }
    warp_list_init(mylists + qi * L, L);
  }
  __syncwarp();
  if (!TILE && nqw == 0) return;  // (with TILE a warp without queries still helps to copy the rows)

  const size_t r_begin = size_t(blockIdx.y) * rows_per_split;
  const size_t r_end = min(n, r_begin + rows_per_split);
  u64 bound[QT];
#pragma unroll
  for (int qi = 0; qi < QT; ++qi) bound[qi] = FV_EMPTY_KEY;

  // TILE: two buffers; the copy of the next 32 rows (asynchronous, 16 bytes per request, rows past the end filled
  // with zeros) is in flight while the current 32 are worked on
  const int tile_floats = 32 * tstride;
  auto stage_rows = [&](size_t r0, float* dst) {
    const int q4 = pd >> 2;
    for (int i = threadIdx.x; i < 32 * q4; i += blockDim.x) {
      const int tr = i / q4, c4 = i - tr * q4;
      const bool in = r0 + tr < r_end;
      const float4* src = reinterpret_cast<const float4*>(rows + (in ? r0 + tr : r_begin) * size_t(pd)) + c4;
      const uint32_t d = uint32_t(__cvta_generic_to_shared(dst + tr * tstride + c4 * 4));
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(in ? 16 : 0) : "memory");
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  if (TILE && r_begin < r_end) stage_rows(r_begin, tile);
  int buf = 0;
  for (size_t r0 = r_begin; r0 < r_end; r0 += 32, buf ^= 1) {
    const size_t row = r0 + lane;
    const bool valid = row < r_end;
    const float* cur_tile = tile + buf * tile_floats;
    if (TILE) {
      if (r0 + 32 < r_end) {
        stage_rows(r0 + 32, tile + (buf ^ 1) * tile_floats);  // (its last readers passed the barrier below one step ago)
        asm volatile("cp.async.wait_group 1;" ::: "memory");
      } else {
        asm volatile("cp.async.wait_group 0;" ::: "memory");
      }
      __syncthreads();  // this step's rows have landed, for every thread's copies
    }
    if (!TILE || nqw > 0) {
    const float4* b4 = TILE ? reinterpret_cast<const float4*>(cur_tile + lane * tstride)
                            : reinterpret_cast<const float4*>(rows + (valid ? row : r_begin) * size_t(pd));
    float acc[QT][8];
#pragma unroll
    for (int qi = 0; qi < QT; ++qi)
#pragma unroll
      for (int l = 0; l < 8; ++l) acc[qi][l] = 0.f;
#pragma unroll 2
    for (int c = 0; c < pd / 8; ++c) {
      const float4 b0 = TILE ? b4[2 * c] : __ldg(b4 + 2 * c), b1 = TILE ? b4[2 * c + 1] : __ldg(b4 + 2 * c + 1);
#pragma unroll
      for (int qi = 0; qi < QT; ++qi) {
        const float4* a4 = reinterpret_cast<const float4*>(myq + qi * pd) + 2 * c;
        dist_step8<IS_L2>(acc[qi], a4[0], a4[1], b0, b1);
      }
    }
#pragma unroll
    for (int qi = 0; qi < QT; ++qi) {
      if (qi < nqw) {
        float d = hsum8(acc[qi]);
        if (!IS_L2) d = -d;
        u64 key = make_key(d, id_base + uint32_t(row));
        if (!valid || (prefilter_inf && !(d < INFINITY))) key = FV_EMPTY_KEY;
        if (dense) {  // every key is kept: the selection happens in block_select_kernel
          if (valid) dense[(q0 + qi) * dense_stride + row] = key;
        } else {
          bound[qi] = warp_list_offer(mylists + qi * L, L, key, bound[qi]);
        }
      }
    }
    }
    if (TILE) __syncthreads();  // everybody is done with this buffer before the step after next refills it
  }
  __syncwarp();
  if (dense || nqw == 0) return;
  const int P = gridDim.y;
  for (int qi = 0; qi < nqw; ++qi) {
    u64* dst = parts + ((q0 + qi) * size_t(P) + blockIdx.y) * size_t(L);
    for (int e = lane; e < L; e += 32) dst[e] = mylists[qi * L + e];
  }
}

// One block per query: the L smallest of n keys (n <= npow2, a power of two), by sorting them in shared memory.
__global__ void __launch_bounds__(256) block_select_kernel(const u64* __restrict__ dense, size_t stride, int n, int npow2,
                                                           int L, u64* __restrict__ out) {
  u64* buf = reinterpret_cast<u64*>(dyn_smem());
  const size_t q = blockIdx.x;
  for (int i = threadIdx.x; i < npow2; i += blockDim.x) buf[i] = i < n ? dense[q * stride + i] : FV_EMPTY_KEY;
  __syncthreads();
  block_sort(buf, npow2);
  for (int e = threadIdx.x; e < L; e += blockDim.x) out[q * size_t(L) + e] = e < npow2 ? buf[e] : FV_EMPTY_KEY;
}

// One warp per query: the L smallest of n <= 32 * NPL keys without sorting them all.  A lane keeps the distance words
// of rows lane, lane + 32, ... in registers; 32 bisection steps on that word find the L-th smallest distance T;
// the rows below T and the first ties at T (rows are in id order) are gathered and only those L keys are sorted.
template <int NPL>
__global__ void __launch_bounds__(128) warp_select_kernel(const u64* __restrict__ dense, size_t stride, int n, int L,
                                                          int Lpow2, size_t nq, u64* __restrict__ out) {
  u64* buf = reinterpret_cast<u64*>(dyn_smem()) + size_t(threadIdx.x >> 5) * Lpow2;
  const int lane = threadIdx.x & 31;
  const size_t q = blockIdx.x * size_t(blockDim.x >> 5) + (threadIdx.x >> 5);
  if (q >= nq) return;
  const u64* src = dense + q * stride;
  uint32_t h[NPL];
#pragma unroll
  for (int j = 0; j < NPL; ++j) {
    const int r = j * 32 + lane;
    h[j] = r < n ? uint32_t(src[r] >> 32) : 0xFFFFFFFFu;
  }
  // Bisection between the smallest and the largest word.  It may stop at any value with exactly L words at or below
  // it: that value separates the same rows as the L-th smallest word itself (the selection below takes every row
  // below T and as many rows at T as are still wanted, which is then all of them).
  uint32_t lo = 0xFFFFFFFFu, hi = 0;
#pragma unroll
  for (int j = 0; j < NPL; ++j) {
    lo = min(lo, h[j]);
    if (j * 32 + lane < n) hi = max(hi, h[j]);
  }
  lo = __reduce_min_sync(FV_FULL, lo);
  hi = __reduce_max_sync(FV_FULL, hi);
  if (n < L) hi = 0xFFFFFFFFu;  // fewer rows than wanted: the filler value is the L-th smallest
  while (lo < hi) {
    const uint32_t mid = lo + ((hi - lo) >> 1);
    int c = 0;
#pragma unroll
    for (int j = 0; j < NPL; ++j) c += h[j] <= mid ? 1 : 0;
    c = __reduce_add_sync(FV_FULL, c);
    if (c == L) {
      lo = mid;
      break;
    }
    if (c > L) hi = mid;
    else lo = mid + 1;
  }
  const uint32_t T = lo;
  int below = 0;
#pragma unroll
  for (int j = 0; j < NPL; ++j) below += h[j] < T ? 1 : 0;
  below = __reduce_add_sync(FV_FULL, below);
  const int ties_wanted = L - below;  // >= 1 by the choice of T (or rows ran out: then T is the filler value)
  for (int e = lane; e < Lpow2; e += 32) buf[e] = FV_EMPTY_KEY;
  __syncwarp();
  int pos = 0, ties = 0;  // the same in every lane
#pragma unroll
  for (int j = 0; j < NPL; ++j) {
    const int r = j * 32 + lane;
    const unsigned tmask = __ballot_sync(FV_FULL, h[j] == T);
    const int my_tie = ties + __popc(tmask & ((1u << lane) - 1u));
    const bool take = h[j] < T || (h[j] == T && my_tie < ties_wanted);
    const unsigned smask = __ballot_sync(FV_FULL, take);
    if (take && r < n) buf[pos + __popc(smask & ((1u << lane) - 1u))] = src[r];
    pos += __popc(smask);
    ties += __popc(tmask);
  }
  __syncwarp();
  // sort the L gathered keys (bitonic over Lpow2, one warp)
  for (int k = 2; k <= Lpow2; k <<= 1) {
    for (int j = k >> 1; j > 0; j >>= 1) {
      for (int t = lane; t < (Lpow2 >> 1); t += 32) {
        const int i = ((t & ~(j - 1)) << 1) | (t & (j - 1));
        const u64 x = buf[i], y = buf[i | j];
        if ((x > y) == ((i & k) == 0)) {
          buf[i] = y;
          buf[i | j] = x;
        }
      }
      __syncwarp();
    }
  }
  for (int e = lane; e < L; e += 32) out[q * size_t(L) + e] = buf[e];
}

// One warp per query: the L smallest of P sorted partial lists.
__global__ void merge_keys_kernel(const u64* __restrict__ parts, int P, int Lin, size_t nq, int Lout,
                                  u64* __restrict__ out) {
  unsigned char* smem_raw = dyn_smem();
  const int w = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const size_t q = size_t(blockIdx.x) * (blockDim.x >> 5) + w;
  if (q >= nq) return;
  u64* list = reinterpret_cast<u64*>(smem_raw) + size_t(w) * Lout;
  warp_list_init(list, Lout);
  u64 bound = FV_EMPTY_KEY;
  const u64* src = parts + q * size_t(P) * Lin;
  const int total = P * Lin;
  for (int i0 = 0; i0 < total; i0 += 32) {
    const int i = i0 + lane;
    const u64 key = i < total ? src[i] : FV_EMPTY_KEY;
    bound = warp_list_offer(list, Lout, key, bound);
  }
  __syncwarp();
  for (int e = lane; e < Lout; e += 32) out[q * size_t(Lout) + e] = list[e];
}

__global__ void keys_to_neighbors_kernel(const u64* __restrict__ keys, size_t nq, int L, int k,
                                         fv_neighbor* __restrict__ out, uint32_t* __restrict__ counts,
                                         const uint32_t* __restrict__ qids) {
  const size_t q = blockIdx.x * size_t(blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (q >= nq) return;
  const size_t dst = qids ? size_t(qids[q]) : q;
  int cnt = 0;
  for (int e0 = 0; e0 < k; e0 += 32) {
    const int e = e0 + lane;
    u64 key = (e < k && e < L) ? keys[q * size_t(L) + e] : FV_EMPTY_KEY;
    if (e < k) {
      fv_neighbor nb;
      if (key == FV_EMPTY_KEY) {
        nb.id = 0xFFFFFFFFu;
        nb.distance = INFINITY;
      } else {
        nb.id = key_id(key);
        nb.distance = key_distance(key);
      }
      out[dst * size_t(k) + e] = nb;
    }
    cnt += __popc(__ballot_sync(FV_FULL, key != FV_EMPTY_KEY));
  }
  if (lane == 0 && counts) counts[dst] = uint32_t(cnt);
}

int keys_to_neighbors(fv_ctx* ctx, const u64* d_keys, size_t nq, int L, int k, fv_neighbor* d_out, uint32_t* d_counts,
                      const uint32_t* d_query_ids) {
  if (nq == 0) return FV_OK;
  const int wpb = 8;
  keys_to_neighbors_kernel<<<unsigned((nq + wpb - 1) / wpb), wpb * 32, 0, ctx->stream>>>(d_keys, nq, L, k, d_out,
                                                                                         d_counts, d_query_ids);
  ctx->stats.launches++;
  FV_CUDA(cudaGetLastError());
  return FV_OK;
}

template <int QT>
static int launch_scan(fv_ctx* ctx, bool is_l2, dim3 grid, int threads, size_t smem, const float* rows, size_t n, int pd,
                       const float* q, size_t q_stride, const uint32_t* qids, size_t nq, int L, bool prefilter,
                       uint32_t id_base, size_t rps, u64* parts, u64* dense = nullptr, size_t dense_stride = 0) {
  // the row tile goes behind the queries and lists when the shared memory of an SM still holds four such blocks
  const size_t tile_bytes = 2 * size_t(32) * (size_t(pd) + 4) * sizeof(float);  // two buffers
  const size_t with_tile = ((smem + 15) & ~size_t(15)) + tile_bytes;
  // (only for full blocks: a single warp that scans a long run of rows for a few queries streams them faster itself)
  const bool tiled = with_tile <= 72 * 1024 && threads >= 128;
  auto k = is_l2 ? (tiled ? exact_scan_kernel<QT, true, true> : exact_scan_kernel<QT, true, false>)
                 : (tiled ? exact_scan_kernel<QT, false, true> : exact_scan_kernel<QT, false, false>);
  if (tiled) smem = with_tile;
  if (smem > 40 * 1024) FV_CUDA(cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)));
  k<<<grid, threads, smem, ctx->stream>>>(rows, n, pd, q, q_stride, qids, nq, L, prefilter ? 1 : 0, id_base, rps, parts,
                                          dense, dense_stride);
  ctx->stats.launches++;
  FV_CUDA(cudaGetLastError());
  return FV_OK;
}

int exact_scan(fv_ctx* ctx, int metric, const float* d_rows, size_t n, int pd, const float* d_queries, size_t q_stride,
               const uint32_t* d_query_ids, size_t nq, int L, bool prefilter_inf, uint32_t id_base, u64* d_out_keys,
               int scratch_slot) {
  if (nq == 0) return FV_OK;
  if (L < 1 || L > 4096) return fail(FV_ERR_UNSUPPORTED, "top-k list length must be in 1..4096");
  const size_t budget = std::min<size_t>(ctx->smem_optin, 200 * 1024);
  // choose queries per warp (QT) and warps per block (W) so that queries + lists fit in shared memory
  int QT = 8, W = 4;
  auto need = [&](int qt, int w) { return size_t(w) * qt * (size_t(pd) * 4 + size_t(L) * 8); };
  if (nq <= 64) QT = 2;  // few queries: spread them over warps instead of queueing eight behind one
  while (need(QT, W) > budget && W > 1) W >>= 1;
  if (need(QT, W) > budget) QT = 2;
  if (need(QT, W) > budget)
    return fail(FV_ERR_UNSUPPORTED, "dimension and k too large for the shared-memory budget of the scan");
  // Long lists over few rows (the coarse quantizer: 64 of 1024 cells): keeping a sorted list per query costs more
  // than the distances.  Write every key instead and let one block per query sort them.
  if (L >= 32 && n <= 4096 && nq >= 64 && !d_query_ids) {
    int npow2 = 32;
    while (size_t(npow2) < n) npow2 <<= 1;
    FV_TRY(ctx->scratch[scratch_slot].reserve(nq * n * sizeof(u64)));
    u64* dense = ctx->scratch[scratch_slot].as<u64>();
    const int w4 = 4;
    const size_t groups = (nq + size_t(QT) * w4 - 1) / (size_t(QT) * w4);
    size_t S = std::max<size_t>(1, std::min<size_t>(n / 128, (size_t(ctx->sm_count) * 8 + groups - 1) / groups));
    size_t rps = ((n + S - 1) / S + 31) / 32 * 32;
    S = (n + rps - 1) / rps;
    const dim3 grid(static_cast<unsigned>(groups), static_cast<unsigned>(S));
    const size_t smem = size_t(w4) * QT * (size_t(pd) * 4 + 8);
    if (QT == 8)
      FV_TRY(launch_scan<8>(ctx, metric == FV_L2, grid, w4 * 32, smem, d_rows, n, pd, d_queries, q_stride, nullptr, nq, 1,
                            prefilter_inf, id_base, rps, nullptr, dense, n));
    else
      FV_TRY(launch_scan<2>(ctx, metric == FV_L2, grid, w4 * 32, smem, d_rows, n, pd, d_queries, q_stride, nullptr, nq, 1,
                            prefilter_inf, id_base, rps, nullptr, dense, n));
    if (n <= 2048 && L <= 256) {
      int lp = 32;
      while (lp < L) lp <<= 1;
      const unsigned blocks = unsigned((nq + 3) / 4);
      if (n <= 1024)
        warp_select_kernel<32><<<blocks, 128, size_t(4) * lp * 8, ctx->stream>>>(dense, n, int(n), L, lp, nq, d_out_keys);
      else
        warp_select_kernel<64><<<blocks, 128, size_t(4) * lp * 8, ctx->stream>>>(dense, n, int(n), L, lp, nq, d_out_keys);
    } else {
      block_select_kernel<<<unsigned(nq), 256, size_t(npow2) * 8, ctx->stream>>>(dense, n, int(n), npow2, L, d_out_keys);
    }
    ctx->stats.launches++;
    FV_CUDA(cudaGetLastError());
    return FV_OK;
  }
  const size_t qgroups = (nq + size_t(QT) * W - 1) / (size_t(QT) * W);
  while (W > 1 && nq <= size_t(QT) * (W / 2)) W >>= 1;  // do not launch warps without queries
  // split the rows when there are too few query groups to fill the GPU
  size_t S = 1;
  // aim at about 32 resident warps per SM: each lane streams its own row, so the loads need that many in flight
  const size_t target = size_t(ctx->sm_count) * std::max(4, 32 / W);
  if (qgroups < target) S = (target + qgroups - 1) / qgroups;
  // (a handful of queries over a few thousand rows -- the re-run of the uncertified queries of a coarse step -- is
  // all latency: 128-row splits give the SMs something to do)
  const size_t max_split = std::max<size_t>(1, n / (nq <= 64 ? 128 : 1024));
  S = std::min(S, max_split);
  S = std::min<size_t>(S, 4096);
  size_t rps = (n + S - 1) / S;
  rps = (rps + 31) / 32 * 32;
  if (rps == 0) rps = 32;
  S = std::max<size_t>(1, (n + rps - 1) / rps);
  u64* parts = d_out_keys;
  if (S > 1) {
    FV_TRY(ctx->scratch[scratch_slot].reserve(nq * S * size_t(L) * sizeof(u64)));
    parts = ctx->scratch[scratch_slot].as<u64>();
  }
  dim3 grid(unsigned((nq + size_t(QT) * W - 1) / (size_t(QT) * W)), unsigned(S));
  const size_t smem = need(QT, W);
  if (QT == 8)
    FV_TRY(launch_scan<8>(ctx, metric == FV_L2, grid, W * 32, smem, d_rows, n, pd, d_queries, q_stride, d_query_ids, nq,
                          L, prefilter_inf, id_base, rps, parts));
  else
    FV_TRY(launch_scan<2>(ctx, metric == FV_L2, grid, W * 32, smem, d_rows, n, pd, d_queries, q_stride, d_query_ids, nq,
                          L, prefilter_inf, id_base, rps, parts));
  if (S > 1) {
    int wpb = 4;
    while (wpb > 1 && size_t(wpb) * L * 8 > 96 * 1024) wpb >>= 1;
    const size_t msmem = size_t(wpb) * L * 8;
    if (msmem > 40 * 1024)
      FV_CUDA(cudaFuncSetAttribute(merge_keys_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(msmem)));
    merge_keys_kernel<<<unsigned((nq + wpb - 1) / wpb), wpb * 32, msmem, ctx->stream>>>(parts, int(S), L, nq, L,
                                                                                         d_out_keys);
    ctx->stats.launches++;
    FV_CUDA(cudaGetLastError());
  }
  return FV_OK;
}

}  // namespace fv

// ------------------------------------------------------------------------------------------------
// FlatIndex
struct fv_flat {
  fv_ctx* ctx;
  int metric;
  uint32_t dim, pd;
  size_t n = 0;
  DevBuf data;  // n * pd f32
  uint32_t id_base = 0;
  int mode = 0;
  fv::TcSide* tc = nullptr;  // tensor-core front end state (gemm_topk.cu)
};


extern "C" {

int fv_flat_new(fv_ctx* ctx, int metric, uint32_t dim, fv_flat** out) {
  if (!ctx || !out || dim == 0 || (metric != FV_L2 && metric != FV_INNER_PRODUCT))
    return fv::fail(FV_ERR_ARG, "fv_flat_new: bad argument");
  auto* ix = new fv_flat();
  ix->ctx = ctx;
  ix->metric = metric;
  ix->dim = dim;
  ix->pd = uint32_t(fv::padded(dim));
  fv::ctx_retain(ctx);
  *out = ix;
  return FV_OK;
}

void fv_flat_free(fv_flat* ix) {
  if (!ix) return;
  fv_ctx* ctx = ix->ctx;
  {
    fv::CtxGuard g(ctx);
    cudaStreamSynchronize(ctx->stream);
    fv::tc_free(ix->tc);
    delete ix;
  }
  fv::ctx_release(ctx);  // may destroy the context: its lock is no longer held
}

static int flat_add_impl(fv_flat* ix, const float* v, size_t n, bool dev) {
  if (!ix || (!v && n)) return fv::fail(FV_ERR_ARG, "fv_flat_add: null argument");
  if (n == 0) return FV_OK;
  if (uint64_t(ix->id_base) + ix->n + n > 0xFFFFFFF0ull)
    return fv::fail(FV_ERR_UNSUPPORTED, "row ids (id base + rows) would pass 2^32 - 16");
  fv_ctx* ctx = ix->ctx;
  fv::CtxGuard g(ctx);
  const size_t row = size_t(ix->pd) * sizeof(float);
  FV_TRY(ix->data.grow((ix->n + n) * row, ix->n * row, ctx->stream));
  float* dst = ix->data.as<float>() + ix->n * size_t(ix->pd);
  FV_TRY(fv::upload_padded(ctx, v, dev, n, ix->dim, ix->pd, dst));
  FV_TRY(fv::tc_append(ctx, &ix->tc, ix->metric, dst, ix->n, n, int(ix->pd)));
  FV_CUDA(cudaStreamSynchronize(ctx->stream));
  ix->n += n;
  return FV_OK;
}

int fv_flat_add(fv_flat* ix, const float* vectors, size_t n) { return flat_add_impl(ix, vectors, n, false); }
int fv_flat_add_dev(fv_flat* ix, const float* d_vectors, size_t n) { return flat_add_impl(ix, d_vectors, n, true); }

size_t fv_flat_len(const fv_flat* ix) { return ix ? ix->n : 0; }

int fv_flat_vector(const fv_flat* ix, uint32_t id, float* out_padded) {
  if (!ix || !out_padded || id >= ix->n) return fv::fail(FV_ERR_ARG, "fv_flat_vector: bad argument");
  fv::CtxGuard g(ix->ctx);
  FV_CUDA(cudaMemcpy(out_padded, ix->data.as<float>() + size_t(id) * ix->pd, size_t(ix->pd) * sizeof(float),
                     cudaMemcpyDeviceToHost));
  return FV_OK;
}

int fv_flat_set_id_base(fv_flat* ix, uint32_t id_base) {
  if (!ix) return fv::fail(FV_ERR_ARG, "null index");
  if (ix->n) return fv::fail(FV_ERR_ARG, "id base must be set before the first add");
  ix->id_base = id_base;
  return FV_OK;
}

int fv_flat_set_mode(fv_flat* ix, int mode) {
  if (!ix || mode < 0 || mode > 2) return fv::fail(FV_ERR_ARG, "fv_flat_set_mode: mode must be 0, 1 or 2");
  ix->mode = mode;
  return FV_OK;
}

// scratch slots: 0 padded queries, 1 final keys, 2 scan partials, 3.. tensor-core path
int fv_flat_search_batch_dev(fv_flat* ix, const float* d_queries, size_t nq, size_t k, fv_neighbor* d_out,
                             uint32_t* d_counts) {
  if (!ix || (nq && (!d_queries || !d_out))) return fv::fail(FV_ERR_ARG, "fv_flat_search_batch: null argument");
  if (k == 0) return fv::fail(FV_ERR_ARG, "k must be at least 1");
  if (k > 4096) return fv::fail(FV_ERR_UNSUPPORTED, "k above 4096 is not supported");
  if (nq == 0) return FV_OK;
  fv_ctx* ctx = ix->ctx;
  fv::CtxGuard g(ctx);
  ctx->stats = fv_stats{};
  fv::stage_begin(ctx);
  const int pd = int(ix->pd);
  const float* q = d_queries;
  if (ix->pd != ix->dim) {
    FV_TRY(ctx->scratch[0].reserve(nq * size_t(pd) * sizeof(float)));
    FV_TRY(fv::upload_padded(ctx, d_queries, true, nq, ix->dim, ix->pd, ctx->scratch[0].as<float>()));
    q = ctx->scratch[0].as<float>();
  }
  const int L = int(k);
  FV_TRY(ctx->scratch[1].reserve(nq * size_t(L) * sizeof(u64)));
  u64* keys = ctx->scratch[1].as<u64>();
  const bool want_tc = ix->mode == 1 || (ix->mode == 0 && fv::tc_usable(ix->tc, ix->n, nq, L));
  if (want_tc) {
    if (!fv::tc_usable(ix->tc, ix->n, nq, L))
      return fv::fail(FV_ERR_UNSUPPORTED, "tensor-core search needs k <= 32, at least 4096 rows and a padded dimension of at most 384");
    FV_TRY(fv::tc_search(ctx, ix->tc, ix->metric, ix->data.as<float>(), ix->n, pd, q, nq, L, ix->id_base, keys, true, true));
  } else {
    FV_TRY(fv::exact_scan(ctx, ix->metric, ix->data.as<float>(), ix->n, pd, q, size_t(pd), nullptr, nq, L, true,
                          ix->id_base, keys, 2));
    fv::stage_mark(ctx);
  }
  FV_TRY(fv::keys_to_neighbors(ctx, keys, nq, L, int(k), d_out, d_counts));
  fv::stage_mark(ctx);
  FV_CUDA(cudaStreamSynchronize(ctx->stream));
  fv::stage_end(ctx);
  return FV_OK;
}

int fv_flat_search_batch(fv_flat* ix, const float* queries, size_t nq, size_t k, fv_neighbor* out, uint32_t* counts) {
  if (!ix || (nq && (!queries || !out))) return fv::fail(FV_ERR_ARG, "fv_flat_search_batch: null argument");
  if (nq == 0) return FV_OK;
  fv_ctx* ctx = ix->ctx;
  fv::CtxGuard g(ctx);
  const size_t qbytes = nq * size_t(ix->dim) * sizeof(float);
  const size_t obytes = nq * k * sizeof(fv_neighbor);
  FV_TRY(ctx->scratch[10].reserve(qbytes));
  FV_TRY(ctx->scratch[11].reserve(obytes + nq * sizeof(uint32_t)));
  float* dq = ctx->scratch[10].as<float>();
  fv_neighbor* dout = ctx->scratch[11].as<fv_neighbor>();
  uint32_t* dc = reinterpret_cast<uint32_t*>(ctx->scratch[11].as<unsigned char>() + obytes);
  FV_CUDA(cudaMemcpyAsync(dq, queries, qbytes, cudaMemcpyHostToDevice, ctx->stream));
  FV_TRY(fv_flat_search_batch_dev(ix, dq, nq, k, dout, dc));
  FV_CUDA(cudaMemcpyAsync(out, dout, obytes, cudaMemcpyDeviceToHost, ctx->stream));
  if (counts) FV_CUDA(cudaMemcpyAsync(counts, dc, nq * sizeof(uint32_t), cudaMemcpyDeviceToHost, ctx->stream));
  FV_CUDA(cudaStreamSynchronize(ctx->stream));
  return FV_OK;
}

int fv_flat_search(fv_flat* ix, const float* query, size_t k, fv_neighbor* out, uint32_t* count) {
  return fv_flat_search_batch(ix, query, 1, k, out, count);
}

// Merging per-shard results: the k_out best of nparts * k_in candidates per query.
namespace fv {
__global__ void merge_parts_kernel(const fv_neighbor* __restrict__ parts, const uint32_t* __restrict__ part_counts,
                                   int nparts, size_t nq, int k_in, int k_out, size_t part_stride, u64* __restrict__ out) {
  unsigned char* smem_raw = dyn_smem();
  const int w = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const size_t q = size_t(blockIdx.x) * (blockDim.x >> 5) + w;
  if (q >= nq) return;
  u64* list = reinterpret_cast<u64*>(smem_raw) + size_t(w) * k_out;
  warp_list_init(list, k_out);
  u64 bound = FV_EMPTY_KEY;
  for (int p = 0; p < nparts; ++p) {
    const int cnt = part_counts ? int(min(part_counts[size_t(p) * nq + q], uint32_t(k_in))) : k_in;
    const fv_neighbor* src = parts + size_t(p) * part_stride + q * size_t(k_in);
    for (int i0 = 0; i0 < cnt; i0 += 32) {
      const int i = i0 + lane;
      u64 key = FV_EMPTY_KEY;
      if (i < cnt) {
        const fv_neighbor nb = src[i];
        if (nb.id != 0xFFFFFFFFu) key = make_key(nb.distance, nb.id);
      }
      bound = warp_list_offer(list, k_out, key, bound);
    }
  }
  __syncwarp();
  for (int e = lane; e < k_out; e += 32) out[q * size_t(k_out) + e] = list[e];
}
}  // namespace fv

extern "C++" {
namespace fv {
int merge_topk_impl(fv_ctx* ctx, const fv_neighbor* d_parts, const uint32_t* d_part_counts, size_t nparts, size_t nq,
                    size_t k_in, size_t k_out, fv_neighbor* d_out, uint32_t* d_counts, size_t part_stride) {
  if (part_stride == 0) part_stride = nq * k_in;
  FV_TRY(ctx->scratch[1].reserve(nq * k_out * sizeof(u64)));
  u64* keys = ctx->scratch[1].as<u64>();
  int wpb = 4;
  while (wpb > 1 && size_t(wpb) * k_out * 8 > 96 * 1024) wpb >>= 1;
  const size_t smem = size_t(wpb) * k_out * 8;
  if (smem > 40 * 1024)
    FV_CUDA(cudaFuncSetAttribute(merge_parts_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)));
  merge_parts_kernel<<<unsigned((nq + wpb - 1) / wpb), wpb * 32, smem, ctx->stream>>>(d_parts, d_part_counts, int(nparts), nq,
                                                                                     int(k_in), int(k_out), part_stride, keys);
  ctx->stats.launches++;
  FV_CUDA(cudaGetLastError());
  return keys_to_neighbors(ctx, keys, nq, int(k_out), int(k_out), d_out, d_counts);
}
}  // namespace fv
}  // extern "C++"

int fv_merge_topk_dev(fv_ctx* ctx, const fv_neighbor* d_parts, const uint32_t* d_part_counts, size_t nparts, size_t nq,
                      size_t k_in, size_t k_out, fv_neighbor* d_out, uint32_t* d_counts) {
  if (!ctx || !d_parts || !d_out || nparts == 0 || k_in == 0 || k_out == 0)
    return fv::fail(FV_ERR_ARG, "fv_merge_topk_dev: bad argument");
  if (k_out > 4096) return fv::fail(FV_ERR_UNSUPPORTED, "k above 4096 is not supported");
  if (nq == 0) return FV_OK;
  fv::CtxGuard g(ctx);
  FV_TRY(fv::merge_topk_impl(ctx, d_parts, d_part_counts, nparts, nq, k_in, k_out, d_out, d_counts));
  FV_CUDA(cudaStreamSynchronize(ctx->stream));
  return FV_OK;
}

// Search over row shards, one per rank of the context's communicator: the local search (ids carry the shard's id
// base), one exchange of the per-shard result lists, the merge.  Every rank ends up with the full result.
// Stages (fv_stats.stage_ms): 0 the local search, 1 the exchange, 2 the merge.
int fv_flat_search_sharded_dev(fv_flat* ix, const float* d_queries, size_t nq, size_t k, fv_neighbor* d_out,
                               uint32_t* d_counts) {
  if (!ix || (nq && (!d_queries || !d_out))) return fv::fail(FV_ERR_ARG, "fv_flat_search_sharded: null argument");
  fv_ctx* ctx = ix->ctx;
  fv::CtxGuard g(ctx);
  const int world = ctx->comm_size;
  if (world <= 1) return fv_flat_search_batch_dev(ix, d_queries, nq, k, d_out, d_counts);
  if (nq == 0) return FV_OK;
  if (k == 0 || k > 4096) return fv::fail(FV_ERR_ARG, "k must be in 1..4096");
  fv::StageScope scope(ctx);
  const size_t blk = nq * k * sizeof(fv_neighbor);
  FV_TRY(ctx->scratch[10].reserve(blk));
  FV_TRY(ctx->scratch[11].reserve(nq * sizeof(uint32_t)));
  fv_neighbor* mine = ctx->scratch[10].as<fv_neighbor>();
  FV_TRY(fv_flat_search_batch_dev(ix, d_queries, nq, k, mine, ctx->scratch[11].as<uint32_t>()));
  fv::stage_mark_outer(ctx);  // 0
  FV_TRY(ctx->scratch[15].reserve(size_t(world) * blk));
  FV_TRY(fv::comm_all_gather(ctx, mine, ctx->scratch[15].p, blk));  // unused slots carry the id 0xFFFFFFFF: no counts needed
  fv::stage_mark_outer(ctx);  // 1
  FV_TRY(fv::merge_topk_impl(ctx, ctx->scratch[15].as<fv_neighbor>(), nullptr, size_t(world), nq, k, k, d_out, d_counts));
  fv::stage_mark_outer(ctx);  // 2
  FV_CUDA(cudaStreamSynchronize(ctx->stream));
  return FV_OK;
}

}  // extern "C"
