// IvfPq (src/vector/ivfpq.rs) and k-means (src/vector/kmeans.rs).
//
// Device layout: the inverted lists are one CSR -- list_off[nlist+1] row offsets, codes
// (rows * m bytes) and ids (rows * u32) grouped by list in the reference's insertion order
// (ivfpq.rs:183-187) -- plus centroids, codebooks, the precomputed L2 tables (ivfpq.rs:108-126)
// and, when kept, the raw vectors in id order.
//
// Build side: the nearest-centroid searches of k-means and `add` run on the GPU with the
// reference's distance chain (so the argmin is bit-identical); the f64 centroid sums stay on the
// host in data order (kmeans.rs:55-71), as does the stable filing of rows into lists.
#include <algorithm>
#include <cmath>
#include <cstdlib>
#include <numeric>

#include "ivfpq_scan.h"

namespace fv {

static const size_t KSUB = 256;
static const size_t MAX_PRE = size_t(64) << 20;  // ivfpq.rs:52

// ------------------------------------------------------------------------------------------------
// host rng, as src/rng.rs:7-24 (k-means initialisation draws rows with `below`)
struct HostRng {
  uint64_t s;
  explicit HostRng(uint64_t seed) : s((seed * 0x9E3779B97F4A7C15ull) | 1ull) {}
  uint64_t next() {
    s ^= s >> 12;
    s ^= s << 25;
    s ^= s >> 27;
    return s * 0x2545F4914F6CDD1Dull;
  }
  uint64_t below(uint64_t n) { return next() % n; }
};

__global__ void keys_to_ids_kernel(const u64* __restrict__ keys, size_t n, uint32_t* __restrict__ out) {
  for (size_t i = blockIdx.x * size_t(blockDim.x) + threadIdx.x; i < n; i += size_t(gridDim.x) * blockDim.x) {
    const u64 k = keys[i];
    out[i] = k == FV_EMPTY_KEY ? 0u : key_id(k);  // no finite distance: the reference keeps cluster 0 (kmeans.rs:11)
  }
}

// Nearest centroid of every row of d_data (n x dim, dim a multiple of 8), first minimum on ties.
// scratch slots used: 2 (scan partials), 3 (keys)
static int assign_dev(fv_ctx* ctx, int metric, bool prefilter, const float* d_data, size_t n, const float* d_cen,
                      size_t k, size_t dim, uint32_t* d_out) {
  const size_t CH = size_t(1) << 22;
  for (size_t b = 0; b < n; b += CH) {
    const size_t c = std::min(CH, n - b);
    FV_TRY(ctx->scratch[3].reserve(c * sizeof(u64)));
    u64* keys = ctx->scratch[3].as<u64>();
    FV_TRY(exact_scan(ctx, metric, d_cen, k, int(dim), d_data + b * dim, dim, nullptr, c, 1, prefilter, 0, keys, 2));
    keys_to_ids_kernel<<<ctx->sm_count * 4, 256, 0, ctx->stream>>>(keys, c, d_out + b);
    ctx->stats.launches++;
    FV_CUDA(cudaGetLastError());
  }
  return FV_OK;
}

// kmeans.rs:39-90 with the assignment step on the GPU.  h_data / d_data: the same n x dim rows.
static int kmeans_train_impl(fv_ctx* ctx, const float* h_data, const float* d_data, size_t n, size_t dim, size_t k,
                             size_t iters, uint64_t seed, std::vector<float>& cen) {
  if (n < k) return fail(FV_ERR_ARG, "need at least " + std::to_string(k) + " training vectors, got " + std::to_string(n));
  if (dim % 8 != 0) return fail(FV_ERR_ARG, "k-means dimension must be a multiple of 8");
  HostRng rng(seed);
  std::vector<size_t> idx(n);
  std::iota(idx.begin(), idx.end(), size_t(0));
  for (size_t i = 0; i < k; i++) {
    size_t j = i + size_t(rng.below(uint64_t(n - i)));
    std::swap(idx[i], idx[j]);
  }
  cen.resize(k * dim);
  for (size_t c = 0; c < k; c++) std::memcpy(&cen[c * dim], h_data + idx[c] * dim, dim * sizeof(float));
  DevBuf d_cen, d_assign;
  FV_TRY(d_cen.reserve(k * dim * sizeof(float)));
  FV_TRY(d_assign.reserve(n * sizeof(uint32_t)));
  std::vector<uint32_t> a(n);
  std::vector<double> sums(k * dim);
  std::vector<size_t> counts(k);
  for (size_t it = 0; it < iters; it++) {
    FV_CUDA(cudaMemcpyAsync(d_cen.p, cen.data(), k * dim * sizeof(float), cudaMemcpyHostToDevice, ctx->stream));
    FV_TRY(assign_dev(ctx, FV_L2, true, d_data, n, d_cen.as<float>(), k, dim, d_assign.as<uint32_t>()));
    FV_CUDA(cudaMemcpyAsync(a.data(), d_assign.p, n * sizeof(uint32_t), cudaMemcpyDeviceToHost, ctx->stream));
    FV_CUDA(cudaStreamSynchronize(ctx->stream));
    std::fill(sums.begin(), sums.end(), 0.0);
    std::fill(counts.begin(), counts.end(), size_t(0));
    for (size_t i = 0; i < n; i++) {
      const size_t c = a[i];
      counts[c]++;
      double* s = &sums[c * dim];
      const float* v = h_data + i * dim;
      for (size_t d = 0; d < dim; d++) s[d] += double(v[d]);
    }
    for (size_t c = 0; c < k; c++)
      if (counts[c] > 0)
        for (size_t d = 0; d < dim; d++) cen[c * dim + d] = float(sums[c * dim + d] / double(counts[c]));
    for (size_t c = 0; c < k; c++) {
      if (counts[c] == 0) {
        size_t big = 0;  // the LAST largest cluster (Iterator::max_by_key, kmeans.rs:77)
        for (size_t j = 0; j < k; j++)
          if (counts[j] >= counts[big]) big = j;
        for (size_t d = 0; d < dim; d++) {
          const float v = cen[big * dim + d];
          const float e = 1e-4f * (1.0f + std::fabs(v));
          cen[c * dim + d] = v + e;
          cen[big * dim + d] = v - e;
        }
        counts[c] = counts[big] / 2;
        counts[big] -= counts[c];
      }
    }
  }
  return FV_OK;
}

// ------------------------------------------------------------------------------------------------
// device kernels of the index

// ivfpq.rs:108-126: pre[l][j][c] = sum_t (w*w + 2*w*c_j), a plain left-to-right f32 sum from -0.0.
__global__ void pre_tables_kernel(const float* __restrict__ centroids, const float* __restrict__ codebooks, int pd,
                                  int m, int dsub, size_t nlist, float* __restrict__ pre) {
  const size_t total = nlist * size_t(m) * KSUB;
  for (size_t i = blockIdx.x * size_t(blockDim.x) + threadIdx.x; i < total; i += size_t(gridDim.x) * blockDim.x) {
    const size_t l = i / (size_t(m) * KSUB);
    const int jc = int(i - l * size_t(m) * KSUB);
    const int j = jc >> 8;
    const float* w = codebooks + size_t(jc) * dsub;
    const float* cj = centroids + l * size_t(pd) + size_t(j) * dsub;
    float s = -0.0f;
    for (int t = 0; t < dsub; ++t) {
      const float a = w[t], b = cj[t];
      const float term = __fadd_rn(__fmul_rn(a, a), __fmul_rn(__fmul_rn(2.0f, a), b));
      s = __fadd_rn(s, term);
    }
    pre[i] = s;
  }
}

// ivfpq.rs:141-158: one thread per (row, sub-quantizer); first minimum over the 256 codewords of
// sum_t (r-w)*(r-w), with the residual r = x - centroid formed in f32 first (ivfpq.rs:174-176).
template <int DSUB>
__global__ void encode_kernel(const float* __restrict__ x, const uint32_t* __restrict__ assign,
                              const float* __restrict__ centroids, const float* __restrict__ codebooks, size_t n, int pd,
                              int m, int dsub_rt, uint8_t* __restrict__ codes) {
  const int dsub = DSUB > 0 ? DSUB : dsub_rt;
  const size_t total = n * size_t(m);
  for (size_t i = blockIdx.x * size_t(blockDim.x) + threadIdx.x; i < total; i += size_t(gridDim.x) * blockDim.x) {
    const size_t row = i / m;
    const int j = int(i - row * m);
    const float* xv = x + row * size_t(pd) + size_t(j) * dsub;
    const float* cv = centroids + size_t(assign[row]) * pd + size_t(j) * dsub;
    const float* cb = codebooks + size_t(j) * KSUB * dsub;
    float r[DSUB > 0 ? DSUB : 1];
    if (DSUB > 0) {
#pragma unroll
      for (int t = 0; t < DSUB; ++t) r[t] = __fsub_rn(xv[t], cv[t]);
    }
    int best = 0;
    float bd = INFINITY;
    for (int c = 0; c < int(KSUB); ++c) {
      const float* w = cb + size_t(c) * dsub;
      float s = -0.0f;
      if (DSUB > 0) {
#pragma unroll
        for (int t = 0; t < DSUB; ++t) {
          const float d = __fsub_rn(r[t], __ldg(w + t));
          s = __fadd_rn(s, __fmul_rn(d, d));
        }
      } else {
        for (int t = 0; t < dsub; ++t) {
          const float d = __fsub_rn(__fsub_rn(xv[t], cv[t]), __ldg(w + t));
          s = __fadd_rn(s, __fmul_rn(d, d));
        }
      }
      if (s < bd) {
        bd = s;
        best = c;
      }
    }
    codes[i] = uint8_t(best);
  }
}

// moves the rows of the old CSR to their places in the new one
__global__ void move_lists_kernel(const uint32_t* __restrict__ old_off, const uint32_t* __restrict__ new_off, int m,
                                  const uint8_t* __restrict__ old_codes, const uint32_t* __restrict__ old_ids,
                                  uint8_t* __restrict__ new_codes, uint32_t* __restrict__ new_ids) {
  const size_t l = blockIdx.x;
  const size_t o0 = old_off[l], o1 = old_off[l + 1], n0 = new_off[l];
  for (size_t r = threadIdx.x; r < o1 - o0; r += blockDim.x) new_ids[n0 + r] = old_ids[o0 + r];
  const size_t bytes = (o1 - o0) * size_t(m);
  for (size_t b = threadIdx.x; b < bytes; b += blockDim.x) new_codes[n0 * size_t(m) + b] = old_codes[o0 * size_t(m) + b];
}

__global__ void scatter_rows_kernel(const uint32_t* __restrict__ dest, const uint8_t* __restrict__ codes, size_t n,
                                    int m, uint32_t first_id, const uint32_t* __restrict__ row_ids,
                                    uint8_t* __restrict__ new_codes, uint32_t* __restrict__ new_ids) {
  for (size_t i = blockIdx.x * size_t(blockDim.x) + threadIdx.x; i < n; i += size_t(gridDim.x) * blockDim.x) {
    const size_t d = dest[i];
    new_ids[d] = row_ids ? row_ids[i] : first_id + uint32_t(i);
    for (int j = 0; j < m; ++j) new_codes[d * size_t(m) + j] = codes[i * size_t(m) + j];
  }
}

// list-sharded add: keeps the rows a shard owns (row sel[s] of the chunk), with their global ids
__global__ void gather_owned_kernel(const float* __restrict__ x, const uint32_t* __restrict__ assign,
                                    const uint32_t* __restrict__ sel, size_t ns, int pd, uint32_t first_id,
                                    float* __restrict__ xs, uint32_t* __restrict__ assign_s, uint32_t* __restrict__ ids_s) {
  const int lane = threadIdx.x & 31;
  const size_t s = blockIdx.x * size_t(blockDim.x >> 5) + (threadIdx.x >> 5);
  if (s >= ns) return;
  const size_t i = sel[s];
  const float4* a = reinterpret_cast<const float4*>(x + i * size_t(pd));
  float4* b = reinterpret_cast<float4*>(xs + s * size_t(pd));
  for (int c = lane; c < pd / 4; c += 32) b[c] = a[c];
  if (lane == 0) {
    assign_s[s] = assign[i];
    ids_s[s] = first_id + uint32_t(i);
  }
}

}  // namespace fv

// ------------------------------------------------------------------------------------------------
struct fv_ivfpq {
  fv_ctx* ctx = nullptr;
  ~fv_ivfpq() {
    fv::tc_free(ctc);
    fv::tc_free(recon);
    roff8.release();
    centroids.release(); codebooks.release(); pre.release(); list_off.release(); owned_ids.release();
    codes.release(); ids.release(); vectors.release(); codes_t.release(); off16.release();
    if (ctx) fv::ctx_release(ctx);
  }
  int metric = 0;
  uint32_t dim = 0, pd = 0;
  size_t nlist = 0, m = 0, dsub = 0;
  bool keep = false;
  uint32_t id_base = 0;
  size_t count = 0;   // rows stored here
  size_t seen = 0;    // rows passed to add (equals count unless the index is list-sharded)
  int shard_rank = 0, shard_world = 1;
  DevBuf owned_ids;   // list-sharded: ids of the kept vectors, ascending
  fv::TcSide* ctc = nullptr;  // 16-bit copy of the centroids for the tensor-core coarse search
  std::vector<float> h_centroids, h_codebooks;
  std::vector<uint32_t> h_off;  // nlist + 1
  DevBuf centroids, codebooks, pre, list_off, codes, ids, vectors;
  bool has_pre = false;
  DevBuf codes_t, off16;  // m = 16: the sub-quantizer-major copy of the codes the list-major scan reads
  bool has_codes_t = false;
  fv::TcSide* recon = nullptr;  // 16-bit reconstruction of every row for the tensor-core pass, built on first use
  DevBuf roff8;
  bool recon_valid = false;     // false after an add: rebuilt by the next search that wants it
  float cen_norm2_max = 0.f, code_norm2_max = 0.f;
  int scan_mode = 0;      // 0 pick by size, 1 one block per query, 2 list-major table scan, 3 list-major tensor-core pass
  int cand_slots = 0;     // list-major scan: candidate slots per query (0 = default)
  size_t survivor_slots = 0;  // tensor-core pass: survivor pool entries per CTA (0 = default)
};

namespace fv {

static int upload_quantizers(fv_ivfpq* ix) {
  fv_ctx* ctx = ix->ctx;
  FV_TRY(ix->centroids.reserve(ix->h_centroids.size() * sizeof(float) + 16));
  FV_TRY(ix->codebooks.reserve(ix->h_codebooks.size() * sizeof(float) + 16));
  FV_CUDA(cudaMemcpyAsync(ix->centroids.p, ix->h_centroids.data(), ix->h_centroids.size() * sizeof(float),
                          cudaMemcpyHostToDevice, ctx->stream));
  FV_CUDA(cudaMemcpyAsync(ix->codebooks.p, ix->h_codebooks.data(), ix->h_codebooks.size() * sizeof(float),
                          cudaMemcpyHostToDevice, ctx->stream));
  // ivfpq.rs:108-112: tables only for L2 and only up to MAX_PRE entries
  const size_t size = ix->nlist * ix->m * KSUB;
  ix->has_pre = false;
  if (ix->metric == FV_L2 && size <= MAX_PRE && size > 0) {
    FV_TRY(ix->pre.reserve(size * sizeof(float)));
    pre_tables_kernel<<<ctx->sm_count * 8, 256, 0, ctx->stream>>>(ix->centroids.as<float>(), ix->codebooks.as<float>(),
                                                                  int(ix->pd), int(ix->m), int(ix->dsub), ix->nlist,
                                                                  ix->pre.as<float>());
    ctx->stats.launches++;
    FV_CUDA(cudaGetLastError());
    ix->has_pre = true;
  }
  // bounds the tensor-core pass's error margin needs: the largest centroid, the largest sum of codewords
  ix->cen_norm2_max = 0.f;
  for (size_t l = 0; l < ix->nlist; ++l) {
    double s = 0.0;
    for (size_t d = 0; d < ix->pd; ++d) s += double(ix->h_centroids[l * ix->pd + d]) * ix->h_centroids[l * ix->pd + d];
    ix->cen_norm2_max = std::max(ix->cen_norm2_max, float(s * 1.000001));
  }
  ix->code_norm2_max = 0.f;
  for (size_t j = 0; j < ix->m; ++j) {
    double best = 0.0;
    for (size_t c = 0; c < KSUB; ++c) {
      double s = 0.0;
      for (size_t t = 0; t < ix->dsub; ++t) {
        const double w = ix->h_codebooks[(j * KSUB + c) * ix->dsub + t];
        s += w * w;
      }
      best = std::max(best, s);
    }
    ix->code_norm2_max += float(best * 1.000001);
  }
  // coarse search as a small GEMM when there are enough cells (ivfpq.rs:211-220 at batch scale)
  tc_free(ix->ctc);
  ix->ctc = nullptr;
  if (ix->nlist >= 4096) FV_TRY(tc_append(ctx, &ix->ctc, ix->metric, ix->centroids.as<float>(), 0, ix->nlist, int(ix->pd)));
  FV_CUDA(cudaStreamSynchronize(ctx->stream));
  return FV_OK;
}

static int upload_offsets(fv_ivfpq* ix) {
  FV_TRY(ix->list_off.reserve((ix->nlist + 1) * sizeof(uint32_t)));
  FV_CUDA(cudaMemcpyAsync(ix->list_off.p, ix->h_off.data(), (ix->nlist + 1) * sizeof(uint32_t), cudaMemcpyHostToDevice,
                          ix->ctx->stream));
  return FV_OK;
}

// after the lists changed: the second copy of the codes (m = 16 only)
static int refresh_transposed(fv_ivfpq* ix) {
  ix->has_codes_t = false;
  ix->recon_valid = false;
  if (ix->m != 16) return FV_OK;
  FV_TRY(build_transposed_codes(ix->ctx, ix->h_off.data(), ix->nlist, ix->list_off.as<uint32_t>(), ix->codes.as<uint8_t>(),
                                &ix->codes_t, &ix->off16));
  ix->has_codes_t = true;
  return FV_OK;
}

static int launch_encode(fv_ctx* ctx, const fv_ivfpq* ix, const float* d_x, const uint32_t* d_assign, size_t n,
                         uint8_t* d_codes) {
  const int threads = 128;
  const unsigned blocks = unsigned(std::min<size_t>((n * ix->m + threads - 1) / threads, size_t(ctx->sm_count) * 32));
  const float* cen = ix->centroids.as<float>();
  const float* cb = ix->codebooks.as<float>();
  const int pd = int(ix->pd), m = int(ix->m), dsub = int(ix->dsub);
  switch (dsub) {
    case 4: encode_kernel<4><<<blocks, threads, 0, ctx->stream>>>(d_x, d_assign, cen, cb, n, pd, m, dsub, d_codes); break;
    case 8: encode_kernel<8><<<blocks, threads, 0, ctx->stream>>>(d_x, d_assign, cen, cb, n, pd, m, dsub, d_codes); break;
    case 16: encode_kernel<16><<<blocks, threads, 0, ctx->stream>>>(d_x, d_assign, cen, cb, n, pd, m, dsub, d_codes); break;
    default: encode_kernel<0><<<blocks, threads, 0, ctx->stream>>>(d_x, d_assign, cen, cb, n, pd, m, dsub, d_codes); break;
  }
  ctx->stats.launches++;
  FV_CUDA(cudaGetLastError());
  return FV_OK;
}

}  // namespace fv

extern "C" {

int fv_kmeans_assign(fv_ctx* ctx, const float* data, size_t n, const float* centroids, size_t k, size_t dim,
                     uint32_t* out) {
  if (!ctx || !data || !centroids || !out || k == 0 || dim == 0 || dim % 8 != 0)
    return fv::fail(FV_ERR_ARG, "fv_kmeans_assign: bad argument (dim must be a multiple of 8)");
  fv::CtxGuard g(ctx);
  DevBuf d_data, d_cen, d_out;
  FV_TRY(d_data.reserve(n * dim * sizeof(float)));
  FV_TRY(d_cen.reserve(k * dim * sizeof(float)));
  FV_TRY(d_out.reserve(n * sizeof(uint32_t)));
  FV_CUDA(cudaMemcpyAsync(d_data.p, data, n * dim * sizeof(float), cudaMemcpyHostToDevice, ctx->stream));
  FV_CUDA(cudaMemcpyAsync(d_cen.p, centroids, k * dim * sizeof(float), cudaMemcpyHostToDevice, ctx->stream));
  FV_TRY(fv::assign_dev(ctx, FV_L2, true, d_data.as<float>(), n, d_cen.as<float>(), k, dim, d_out.as<uint32_t>()));
  FV_CUDA(cudaMemcpyAsync(out, d_out.p, n * sizeof(uint32_t), cudaMemcpyDeviceToHost, ctx->stream));
  FV_CUDA(cudaStreamSynchronize(ctx->stream));
  return FV_OK;
}

int fv_kmeans_train(fv_ctx* ctx, const float* data, size_t n, size_t dim, size_t k, size_t iters, uint64_t seed,
                    float* centroids_out) {
  if (!ctx || !data || !centroids_out || k == 0 || dim == 0) return fv::fail(FV_ERR_ARG, "fv_kmeans_train: bad argument");
  fv::CtxGuard g(ctx);
  DevBuf d_data;
  FV_TRY(d_data.reserve(n * dim * sizeof(float)));
  FV_CUDA(cudaMemcpyAsync(d_data.p, data, n * dim * sizeof(float), cudaMemcpyHostToDevice, ctx->stream));
  std::vector<float> cen;
  FV_TRY(fv::kmeans_train_impl(ctx, data, d_data.as<float>(), n, dim, k, iters, seed, cen));
  std::memcpy(centroids_out, cen.data(), cen.size() * sizeof(float));
  return FV_OK;
}

int fv_ivfpq_train(fv_ctx* ctx, int metric, uint32_t dim, const float* sample, size_t n, const fv_ivfpq_params* p,
                   fv_ivfpq** out) {
  if (!ctx || !sample || !p || !out || dim == 0 || (metric != FV_L2 && metric != FV_INNER_PRODUCT))
    return fv::fail(FV_ERR_ARG, "fv_ivfpq_train: bad argument");
  const size_t pd = fv::padded(dim);
  if (p->m == 0 || pd % p->m != 0)
    return fv::fail(FV_ERR_ARG, "padded dimension " + std::to_string(pd) + " must be a multiple of m = " + std::to_string(p->m));
  if (p->nlist == 0 || n < p->nlist)
    return fv::fail(FV_ERR_ARG, "need at least " + std::to_string(p->nlist) + " training vectors, got " + std::to_string(n));
  if (p->m * fv::KSUB * 8 + 2 * pd * 4 > 190 * 1024) return fv::fail(FV_ERR_UNSUPPORTED, "m above 92 is not supported");
  fv::CtxGuard g(ctx);
  ctx->stats = fv_stats{};
  auto ix = std::unique_ptr<fv_ivfpq>(new fv_ivfpq());
  ix->ctx = ctx;
  fv::ctx_retain(ctx);
  ix->metric = metric;
  ix->dim = dim;
  ix->pd = uint32_t(pd);
  ix->nlist = p->nlist;
  ix->m = p->m;
  ix->dsub = pd / p->m;
  ix->keep = p->keep_vectors != 0;
  // x = pad(sample) on both sides
  std::vector<float> x(n * pd, 0.f);
  for (size_t i = 0; i < n; i++) std::memcpy(&x[i * pd], sample + i * size_t(dim), size_t(dim) * sizeof(float));
  DevBuf d_x, d_assign;
  FV_TRY(d_x.reserve(n * pd * sizeof(float)));
  FV_TRY(d_assign.reserve(n * sizeof(uint32_t)));
  FV_CUDA(cudaMemcpyAsync(d_x.p, x.data(), n * pd * sizeof(float), cudaMemcpyHostToDevice, ctx->stream));
  FV_TRY(fv::kmeans_train_impl(ctx, x.data(), d_x.as<float>(), n, pd, p->nlist, p->iters, p->seed, ix->h_centroids));
  // ivfpq.rs:62: assignment against the final centroids, then residuals
  DevBuf d_cen;
  FV_TRY(d_cen.reserve(ix->h_centroids.size() * sizeof(float)));
  FV_CUDA(cudaMemcpyAsync(d_cen.p, ix->h_centroids.data(), ix->h_centroids.size() * sizeof(float), cudaMemcpyHostToDevice,
                          ctx->stream));
  FV_TRY(fv::assign_dev(ctx, FV_L2, true, d_x.as<float>(), n, d_cen.as<float>(), p->nlist, pd, d_assign.as<uint32_t>()));
  std::vector<uint32_t> assign(n);
  FV_CUDA(cudaMemcpyAsync(assign.data(), d_assign.p, n * sizeof(uint32_t), cudaMemcpyDeviceToHost, ctx->stream));
  FV_CUDA(cudaStreamSynchronize(ctx->stream));
  for (size_t i = 0; i < n; i++) {
    const float* c = &ix->h_centroids[size_t(assign[i]) * pd];
    float* r = &x[i * pd];
    for (size_t d = 0; d < pd; d++) r[d] = r[d] - c[d];
  }
  const size_t dsub = ix->dsub, ksub = std::min(fv::KSUB, n);
  ix->h_codebooks.assign(p->m * fv::KSUB * dsub, 0.f);
  const size_t ps = fv::padded(dsub);  // sub-vectors are padded when dsub is not a multiple of 8 (ivfpq.rs:80-87)
  std::vector<float> sub(n * ps);
  DevBuf d_sub;
  FV_TRY(d_sub.reserve(n * ps * sizeof(float)));
  for (size_t j = 0; j < p->m; j++) {
    std::fill(sub.begin(), sub.end(), 0.f);
    for (size_t i = 0; i < n; i++) std::memcpy(&sub[i * ps], &x[i * pd + j * dsub], dsub * sizeof(float));
    FV_CUDA(cudaMemcpyAsync(d_sub.p, sub.data(), n * ps * sizeof(float), cudaMemcpyHostToDevice, ctx->stream));
    std::vector<float> cb;
    FV_TRY(fv::kmeans_train_impl(ctx, sub.data(), d_sub.as<float>(), n, ps, ksub, p->iters, p->seed + 1 + j, cb));
    for (size_t r = 0; r < ksub; r++)
      std::memcpy(&ix->h_codebooks[(j * fv::KSUB + r) * dsub], &cb[r * ps], dsub * sizeof(float));
  }
  ix->h_off.assign(ix->nlist + 1, 0);
  FV_TRY(fv::upload_quantizers(ix.get()));
  FV_TRY(fv::upload_offsets(ix.get()));
  FV_TRY(ix->codes.reserve(16));
  FV_TRY(fv::refresh_transposed(ix.get()));
  FV_CUDA(cudaStreamSynchronize(ctx->stream));
  *out = ix.release();
  return FV_OK;
}

void fv_ivfpq_free(fv_ivfpq* ix) {
  if (!ix) return;
  fv_ctx* ctx = ix->ctx;
  {
    fv::CtxGuard g(ctx);
    cudaStreamSynchronize(ctx->stream);
    ix->ctx = nullptr;  // the destructor must not drop the reference while the lock is held
    delete ix;
  }
  fv::ctx_release(ctx);  // may destroy the context
}

size_t fv_ivfpq_len(const fv_ivfpq* ix) { return ix ? ix->count : 0; }
size_t fv_ivfpq_bytes_per_vector(const fv_ivfpq* ix) { return ix ? ix->m + 4 : 0; }

int fv_ivfpq_set_id_base(fv_ivfpq* ix, uint32_t id_base) {
  if (!ix) return fv::fail(FV_ERR_ARG, "null index");
  if (ix->count) return fv::fail(FV_ERR_ARG, "id base must be set before the first add");
  ix->id_base = id_base;
  return FV_OK;
}

int fv_ivfpq_set_shard(fv_ivfpq* ix, int rank, int world) {
  if (!ix || world < 1 || rank < 0 || rank >= world) return fv::fail(FV_ERR_ARG, "fv_ivfpq_set_shard: bad rank or world");
  if (ix->seen) return fv::fail(FV_ERR_ARG, "the shard must be set before the first add");
  ix->shard_rank = rank;
  ix->shard_world = world;
  return FV_OK;
}

// ivfpq.rs:161-192
static int ivfpq_add_impl(fv_ivfpq* ix, const float* vectors, size_t n_total, bool src_is_device) {
  if (!ix || (!vectors && n_total)) return fv::fail(FV_ERR_ARG, "fv_ivfpq_add: null argument");
  fv_ctx* ctx = ix->ctx;
  fv::CtxGuard g(ctx);
  const size_t pd = ix->pd, m = ix->m;
  const size_t CH = size_t(1) << 22;
  for (size_t b0 = 0; b0 < n_total; b0 += CH) {
    size_t n = std::min(CH, n_total - b0);
    // ids are id_base + running count; 0xFFFFFFFF marks an unused result slot and must stay out of reach
    if (uint64_t(ix->id_base) + ix->seen + n > 0xFFFFFFF0ull)
      return fv::fail(FV_ERR_UNSUPPORTED, "row ids (id base + rows) would pass 2^32 - 16");
    const float* src = vectors + b0 * size_t(ix->dim);
    DevBuf d_x_tmp, d_assign, d_codes, d_dest, d_sel, d_xs, d_assign_s, d_ids_s;
    FV_TRY(d_x_tmp.reserve(n * pd * sizeof(float)));
    float* d_x = d_x_tmp.as<float>();
    FV_TRY(fv::upload_padded(ctx, src, src_is_device, n, ix->dim, pd, d_x));
    FV_TRY(d_assign.reserve(n * sizeof(uint32_t)));
    // ivfpq.rs:194-204: L2 -> nearest centroid; inner product -> the best cell, every cell pushed
    FV_TRY(fv::assign_dev(ctx, ix->metric, ix->metric == FV_L2, d_x, n, ix->centroids.as<float>(), ix->nlist, pd,
                          d_assign.as<uint32_t>()));
    std::vector<uint32_t> assign_all(n);
    FV_CUDA(cudaMemcpyAsync(assign_all.data(), d_assign.p, n * sizeof(uint32_t), cudaMemcpyDeviceToHost, ctx->stream));
    FV_CUDA(cudaStreamSynchronize(ctx->stream));
    // list-sharded: keep only the rows whose list this shard owns; ids still count every row given to add
    const size_t n_chunk = n;
    const uint32_t first_id = ix->id_base + uint32_t(ix->seen);
    const uint32_t* d_row_ids = nullptr;
    uint32_t* d_assign_use = d_assign.as<uint32_t>();
    std::vector<uint32_t> assign;
    if (ix->shard_world > 1) {
      std::vector<uint32_t> sel;
      for (size_t i = 0; i < n; i++)
        if (int(assign_all[i] % uint32_t(ix->shard_world)) == ix->shard_rank) {
          sel.push_back(uint32_t(i));
          assign.push_back(assign_all[i]);
        }
      n = sel.size();
      FV_TRY(d_sel.reserve(n * sizeof(uint32_t) + 16));
      FV_TRY(d_xs.reserve(n * pd * sizeof(float) + 16));
      FV_TRY(d_assign_s.reserve(n * sizeof(uint32_t) + 16));
      FV_TRY(d_ids_s.reserve(n * sizeof(uint32_t) + 16));
      if (n) {
        FV_CUDA(cudaMemcpyAsync(d_sel.p, sel.data(), n * sizeof(uint32_t), cudaMemcpyHostToDevice, ctx->stream));
        fv::gather_owned_kernel<<<unsigned((n + 7) / 8), 256, 0, ctx->stream>>>(
            d_x, d_assign.as<uint32_t>(), d_sel.as<uint32_t>(), n, int(pd), first_id, d_xs.as<float>(),
            d_assign_s.as<uint32_t>(), d_ids_s.as<uint32_t>());
        ctx->stats.launches++;
        FV_CUDA(cudaGetLastError());
        FV_CUDA(cudaStreamSynchronize(ctx->stream));
      }
      d_x = d_xs.as<float>();
      d_assign_use = d_assign_s.as<uint32_t>();
      d_row_ids = d_ids_s.as<uint32_t>();
      FV_TRY(ix->owned_ids.grow((ix->count + n) * sizeof(uint32_t) + 16, ix->count * sizeof(uint32_t), ctx->stream));
      if (n)
        FV_CUDA(cudaMemcpyAsync(ix->owned_ids.as<uint32_t>() + ix->count, d_row_ids, n * sizeof(uint32_t),
                                cudaMemcpyDeviceToDevice, ctx->stream));
    } else {
      assign.swap(assign_all);
    }
    if (ix->keep) {
      FV_TRY(ix->vectors.grow((ix->count + n) * pd * sizeof(float) + 16, ix->count * pd * sizeof(float), ctx->stream));
      if (n)
        FV_CUDA(cudaMemcpyAsync(ix->vectors.as<float>() + ix->count * pd, d_x, n * pd * sizeof(float),
                                cudaMemcpyDeviceToDevice, ctx->stream));
    }
    FV_TRY(d_codes.reserve(n * m + 16));
    FV_TRY(d_dest.reserve(n * sizeof(uint32_t) + 16));
    if (n) FV_TRY(fv::launch_encode(ctx, ix, d_x, d_assign_use, n, d_codes.as<uint8_t>()));
    // file the rows into their lists in input order (a stable counting sort on the host)
    std::vector<uint32_t> add_cnt(ix->nlist, 0), new_off(ix->nlist + 1, 0), dest(n);
    for (size_t i = 0; i < n; i++) add_cnt[assign[i]]++;
    for (size_t l = 0; l < ix->nlist; l++) new_off[l + 1] = new_off[l] + (ix->h_off[l + 1] - ix->h_off[l]) + add_cnt[l];
    std::vector<uint32_t> cursor(ix->nlist);
    for (size_t l = 0; l < ix->nlist; l++) cursor[l] = new_off[l] + (ix->h_off[l + 1] - ix->h_off[l]);
    for (size_t i = 0; i < n; i++) dest[i] = cursor[assign[i]]++;
    DevBuf new_codes, new_ids, d_new_off;
    FV_TRY(new_codes.reserve((ix->count + n) * m + 16));
    FV_TRY(new_ids.reserve((ix->count + n) * sizeof(uint32_t)));
    FV_TRY(d_new_off.reserve((ix->nlist + 1) * sizeof(uint32_t)));
    FV_CUDA(cudaMemcpyAsync(d_new_off.p, new_off.data(), (ix->nlist + 1) * sizeof(uint32_t), cudaMemcpyHostToDevice,
                            ctx->stream));
    if (n) FV_CUDA(cudaMemcpyAsync(d_dest.p, dest.data(), n * sizeof(uint32_t), cudaMemcpyHostToDevice, ctx->stream));
    if (ix->count) {
      fv::move_lists_kernel<<<unsigned(ix->nlist), 128, 0, ctx->stream>>>(
          ix->list_off.as<uint32_t>(), d_new_off.as<uint32_t>(), int(m), ix->codes.as<uint8_t>(), ix->ids.as<uint32_t>(),
          new_codes.as<uint8_t>(), new_ids.as<uint32_t>());
      ctx->stats.launches++;
      FV_CUDA(cudaGetLastError());
    }
    fv::scatter_rows_kernel<<<ctx->sm_count * 4, 256, 0, ctx->stream>>>(
        d_dest.as<uint32_t>(), d_codes.as<uint8_t>(), n, int(m), first_id, d_row_ids, new_codes.as<uint8_t>(),
        new_ids.as<uint32_t>());
    ctx->stats.launches++;
    FV_CUDA(cudaGetLastError());
    FV_CUDA(cudaStreamSynchronize(ctx->stream));
    std::swap(ix->codes.p, new_codes.p);
    std::swap(ix->codes.cap, new_codes.cap);
    std::swap(ix->ids.p, new_ids.p);
    std::swap(ix->ids.cap, new_ids.cap);
    ix->h_off = new_off;
    FV_TRY(fv::upload_offsets(ix));
    FV_CUDA(cudaStreamSynchronize(ctx->stream));
    ix->count += n;
    ix->seen += n_chunk;
  }
  FV_TRY(fv::refresh_transposed(ix));
  return FV_OK;
}

int fv_ivfpq_add(fv_ivfpq* ix, const float* vectors, size_t n) { return ivfpq_add_impl(ix, vectors, n, false); }
int fv_ivfpq_add_dev(fv_ivfpq* ix, const float* d_vectors, size_t n) { return ivfpq_add_impl(ix, d_vectors, n, true); }

// scratch slots: 0 padded queries, 1 final keys, 2 scan partials, 4 cells, 5 per-query tables (after the coarse search is done with it)
// `cells_in`: the probed cells of every query if the caller already has them (nq x min(nprobe, nlist) keys from
// fv_ivfpq_coarse_dev), else null.  `cells_only`: stop after the coarse search and leave the keys there.
static int ivfpq_search_impl(fv_ivfpq* ix, const float* d_queries, size_t nq, size_t k, size_t nprobe, size_t refine,
                             bool candidates, fv_neighbor* d_out, uint32_t* d_counts, fv_neighbor* d_adc, float* d_exact,
                             const uint64_t* cells_in = nullptr, uint64_t* cells_only = nullptr) {
  fv_ctx* ctx = ix->ctx;
  if (k == 0) return fv::fail(FV_ERR_ARG, "k must be at least 1");
  if (nprobe == 0) return fv::fail(FV_ERR_ARG, "nprobe must be at least 1");
  if (nq == 0) return FV_OK;
  const bool rerank = refine > 0 && ix->keep;
  const size_t keep = candidates ? k : (rerank ? k * refine : k);  // ivfpq.rs:228-232
  const size_t kout = candidates ? keep : k;
  if (keep > 4096 || std::min(nprobe, ix->nlist) > 4096)
    return fv::fail(FV_ERR_UNSUPPORTED, "k * refine and nprobe above 4096 are not supported");
  if (candidates && !ix->keep) return fv::fail(FV_ERR_ARG, "candidate output needs an index that keeps its vectors");
  ctx->stats = fv_stats{};
  fv::stage_begin(ctx);
  const int pd = int(ix->pd);
  const float* q = d_queries;
  if (ix->pd != ix->dim) {
    FV_TRY(ctx->scratch[0].reserve(nq * size_t(pd) * sizeof(float)));
    FV_TRY(fv::upload_padded(ctx, d_queries, true, nq, ix->dim, ix->pd, ctx->scratch[0].as<float>()));
    q = ctx->scratch[0].as<float>();
  }
  const int np = int(std::min(nprobe, ix->nlist));
  const u64* cells = reinterpret_cast<const u64*>(cells_in);
  if (!cells_in) {
    u64* dst = reinterpret_cast<u64*>(cells_only);
    if (!dst) {
      FV_TRY(ctx->scratch[4].reserve(nq * size_t(np) * sizeof(u64)));
      dst = ctx->scratch[4].as<u64>();
    }
    // ivfpq.rs:211-220: every cell is pushed, no pre-filter
    if (nq >= 256 && fv::tc_usable(ix->ctc, ix->nlist, nq, np))
      FV_TRY(fv::tc_search(ctx, ix->ctc, ix->metric, ix->centroids.as<float>(), ix->nlist, pd, q, nq, np, 0, dst, false, false));
    else
      FV_TRY(fv::exact_scan(ctx, ix->metric, ix->centroids.as<float>(), ix->nlist, pd, q, size_t(pd), nullptr, nq, np,
                            false, 0, dst, 2));
    cells = dst;
  }
  fv::stage_mark(ctx);
  if (cells_only) {
    FV_CUDA(cudaStreamSynchronize(ctx->stream));
    fv::stage_end(ctx);
    return FV_OK;
  }
  FV_TRY(ctx->scratch[1].reserve(nq * kout * sizeof(u64)));
  fv::ScanIndex si{};
  si.centroids = ix->centroids.as<float>();
  si.codebooks = ix->codebooks.as<float>();
  si.pre = ix->has_pre ? ix->pre.as<float>() : nullptr;
  si.list_off = ix->list_off.as<uint32_t>();
  si.codes = ix->codes.as<uint8_t>();
  si.ids = ix->ids.as<uint32_t>();
  si.vectors = ix->keep ? ix->vectors.as<float>() : nullptr;
  si.owned_ids = ix->shard_world > 1 ? ix->owned_ids.as<uint32_t>() : nullptr;
  si.owned_n = uint32_t(ix->count);
  si.shard_rank = ix->shard_rank;
  si.shard_world = ix->shard_world;
  si.metric = ix->metric;
  si.pd = pd;
  si.m = int(ix->m);
  si.dsub = int(ix->dsub);
  si.nlist = ix->nlist;
  si.id_base = ix->id_base;
  si.codes_t = ix->has_codes_t ? ix->codes_t.as<uint8_t>() : nullptr;
  si.off16 = ix->has_codes_t ? ix->off16.as<uint32_t>() : nullptr;
  // the reconstruction the tensor-core pass needs: built by the first search that may take that path
  const bool separable = ix->metric == FV_INNER_PRODUCT || ix->has_pre;
  if (ix->has_codes_t && separable && ix->pd <= 128 && ix->count > 0 && keep <= 1024 && !ix->recon_valid &&
      fv::ivfpq_wants_tensor(ix->scan_mode, nq, size_t(np), ix->nlist, ix->shard_world)) {
    FV_TRY(fv::build_reconstruction(ctx, ix->metric, pd, int(ix->m), int(ix->dsub), ix->h_off.data(), ix->nlist,
                                    ix->list_off.as<uint32_t>(), ix->codes.as<uint8_t>(), ix->centroids.as<float>(),
                                    ix->codebooks.as<float>(), &ix->recon, &ix->roff8));
    ix->recon_valid = true;
  }
  si.recon = ix->recon_valid ? ix->recon : nullptr;
  si.roff8 = ix->recon_valid && ix->recon ? ix->roff8.as<uint32_t>() : nullptr;
  si.cen_norm2_max = ix->cen_norm2_max;
  si.code_norm2_max = ix->code_norm2_max;
  si.max_list_rows = 0;
  for (size_t l = 0; l < ix->nlist; ++l) si.max_list_rows = std::max(si.max_list_rows, ix->h_off[l + 1] - ix->h_off[l]);
  si.nrows = ix->h_off[ix->nlist];
  si.survivor_slots = ix->survivor_slots;
  fv::ScanOut so{};
  so.keys = ctx->scratch[1].as<u64>();
  so.adc = d_adc;
  so.exact = d_exact;
  so.counts = d_counts;
  FV_TRY(fv::ivfpq_scan(ctx, si, q, nq, cells, np, int(keep), int(k), rerank, candidates, ix->scan_mode, ix->cand_slots, so));
  if (!candidates) FV_TRY(fv::keys_to_neighbors(ctx, so.keys, nq, int(k), int(k), d_out, d_counts));
  fv::stage_mark(ctx);
  FV_CUDA(cudaStreamSynchronize(ctx->stream));
  fv::stage_end(ctx);
  return fv::bounds_report_ivfpq_scan();
}

int fv_ivfpq_search_batch_dev(fv_ivfpq* ix, const float* d_queries, size_t nq, size_t k, size_t nprobe, size_t refine,
                              fv_neighbor* d_out, uint32_t* d_counts) {
  if (!ix || (nq && (!d_queries || !d_out))) return fv::fail(FV_ERR_ARG, "fv_ivfpq_search_batch: null argument");
  fv::CtxGuard g(ix->ctx);
  return ivfpq_search_impl(ix, d_queries, nq, k, nprobe, refine, false, d_out, d_counts, nullptr, nullptr);
}

size_t fv_ivfpq_nlist(const fv_ivfpq* ix) { return ix ? ix->nlist : 0; }
uint32_t fv_ivfpq_dim(const fv_ivfpq* ix) { return ix ? uint32_t(ix->dim) : 0; }
int fv_ivfpq_metric(const fv_ivfpq* ix) { return ix ? ix->metric : -1; }

int fv_ivfpq_set_candidate_slots(fv_ivfpq* ix, size_t slots) {
  if (!ix || slots > 4096) return fv::fail(FV_ERR_ARG, "fv_ivfpq_set_candidate_slots: at most 4096 slots");
  ix->cand_slots = int(slots);
  return FV_OK;
}

int fv_ivfpq_set_survivor_slots(fv_ivfpq* ix, size_t slots) {
  if (!ix || slots > (size_t(1) << 21)) return fv::fail(FV_ERR_ARG, "fv_ivfpq_set_survivor_slots: at most 2^21 slots");
  ix->survivor_slots = slots;
  return FV_OK;
}

int fv_ivfpq_set_scan_mode(fv_ivfpq* ix, int mode) {
  if (!ix || mode < 0 || mode > 4) return fv::fail(FV_ERR_ARG, "fv_ivfpq_set_scan_mode: mode must be 0, 1, 2, 3 or 4");
  ix->scan_mode = mode;
  return FV_OK;
}

int fv_ivfpq_coarse_dev(fv_ivfpq* ix, const float* d_queries, size_t nq, size_t nprobe, uint64_t* d_cells) {
  if (!ix || (nq && (!d_queries || !d_cells))) return fv::fail(FV_ERR_ARG, "fv_ivfpq_coarse: null argument");
  fv::CtxGuard g(ix->ctx);
  return ivfpq_search_impl(ix, d_queries, nq, 1, nprobe, 0, false, nullptr, nullptr, nullptr, nullptr, nullptr, d_cells);
}

int fv_ivfpq_search_batch_cells_dev(fv_ivfpq* ix, const float* d_queries, size_t nq, size_t k, size_t nprobe,
                                    size_t refine, const uint64_t* d_cells, fv_neighbor* d_out, uint32_t* d_counts) {
  if (!ix || (nq && (!d_queries || !d_out || !d_cells)))
    return fv::fail(FV_ERR_ARG, "fv_ivfpq_search_batch_cells: null argument");
  fv::CtxGuard g(ix->ctx);
  return ivfpq_search_impl(ix, d_queries, nq, k, nprobe, refine, false, d_out, d_counts, nullptr, nullptr, d_cells);
}

int fv_ivfpq_search_candidates_cells_dev(fv_ivfpq* ix, const float* d_queries, size_t nq, size_t keep, size_t nprobe,
                                         const uint64_t* d_cells, fv_neighbor* d_adc, float* d_exact,
                                         uint32_t* d_counts) {
  if (!ix || (nq && (!d_queries || !d_adc || !d_exact || !d_counts || !d_cells)))
    return fv::fail(FV_ERR_ARG, "fv_ivfpq_search_candidates_cells: null argument");
  fv::CtxGuard g(ix->ctx);
  return ivfpq_search_impl(ix, d_queries, nq, keep, nprobe, 1, true, nullptr, d_counts, d_adc, d_exact, d_cells);
}

int fv_ivfpq_search_candidates_dev(fv_ivfpq* ix, const float* d_queries, size_t nq, size_t keep, size_t nprobe,
                                   fv_neighbor* d_adc, float* d_exact, uint32_t* d_counts) {
  if (!ix || (nq && (!d_queries || !d_adc || !d_exact || !d_counts)))
    return fv::fail(FV_ERR_ARG, "fv_ivfpq_search_candidates: null argument");
  fv::CtxGuard g(ix->ctx);
  return ivfpq_search_impl(ix, d_queries, nq, keep, nprobe, 1, true, nullptr, d_counts, d_adc, d_exact);
}

int fv_ivfpq_search_batch(fv_ivfpq* ix, const float* queries, size_t nq, size_t k, size_t nprobe, size_t refine,
                          fv_neighbor* out, uint32_t* counts) {
  if (!ix || (nq && (!queries || !out))) return fv::fail(FV_ERR_ARG, "fv_ivfpq_search_batch: null argument");
  if (nq == 0) return FV_OK;
  fv_ctx* ctx = ix->ctx;
  fv::CtxGuard g(ctx);
  const size_t qbytes = nq * size_t(ix->dim) * sizeof(float), obytes = nq * k * sizeof(fv_neighbor);
  FV_TRY(ctx->scratch[10].reserve(qbytes));
  FV_TRY(ctx->scratch[11].reserve(obytes + nq * sizeof(uint32_t)));
  float* dq = ctx->scratch[10].as<float>();
  fv_neighbor* dout = ctx->scratch[11].as<fv_neighbor>();
  uint32_t* dc = reinterpret_cast<uint32_t*>(ctx->scratch[11].as<unsigned char>() + obytes);
  FV_CUDA(cudaMemcpyAsync(dq, queries, qbytes, cudaMemcpyHostToDevice, ctx->stream));
  FV_TRY(ivfpq_search_impl(ix, dq, nq, k, nprobe, refine, false, dout, dc, nullptr, nullptr));
  FV_CUDA(cudaMemcpyAsync(out, dout, obytes, cudaMemcpyDeviceToHost, ctx->stream));
  if (counts) FV_CUDA(cudaMemcpyAsync(counts, dc, nq * sizeof(uint32_t), cudaMemcpyDeviceToHost, ctx->stream));
  FV_CUDA(cudaStreamSynchronize(ctx->stream));
  return FV_OK;
}

int fv_ivfpq_search(fv_ivfpq* ix, const float* query, size_t k, size_t nprobe, size_t refine, fv_neighbor* out,
                    uint32_t* count) {
  return fv_ivfpq_search_batch(ix, query, 1, k, nprobe, refine, out, count);
}

// ---- FLIVFPQ1 files (ivfpq.rs:332-390, io.rs:45-116)
size_t fv_ivfpq_save_size(const fv_ivfpq* ix) {
  if (!ix) return 0;
  size_t s = 8 + 5 * 4;
  s += 8 + ix->h_centroids.size() * 4;
  s += 8 + ix->h_codebooks.size() * 4;
  s += ix->nlist * 16 + ix->count * 4 + ix->count * ix->m;
  s += 8 + (ix->keep ? ix->count * size_t(ix->pd) * 4 : 0);
  s += 4;
  return s;
}

int fv_ivfpq_save(const fv_ivfpq* ix, uint8_t* buf, size_t cap, size_t* written) {
  if (!ix || !buf) return fv::fail(FV_ERR_ARG, "fv_ivfpq_save: null argument");
  if (ix->shard_world > 1) return fv::fail(FV_ERR_UNSUPPORTED, "a list-sharded index holds part of the rows and cannot be saved as one file");
  // The file has no field for an id base, and a loaded index finds the kept vector of id i in row i.
  if (ix->id_base != 0) return fv::fail(FV_ERR_UNSUPPORTED, "a row shard (id base != 0) cannot be saved: the file format has no id base");
  const size_t need = fv_ivfpq_save_size(ix);
  if (cap < need) return fv::fail(FV_ERR_ARG, "fv_ivfpq_save: buffer too small");
  fv::CtxGuard g(ix->ctx);
  std::vector<uint32_t> ids(ix->count);
  std::vector<uint8_t> codes(ix->count * ix->m);
  if (ix->count) {
    FV_CUDA(cudaMemcpy(ids.data(), ix->ids.p, ix->count * 4, cudaMemcpyDeviceToHost));
    FV_CUDA(cudaMemcpy(codes.data(), ix->codes.p, ix->count * ix->m, cudaMemcpyDeviceToHost));
  }
  uint8_t* w = buf;
  auto raw = [&](const void* p, size_t n) {
    std::memcpy(w, p, n);
    w += n;
  };
  auto u32 = [&](uint32_t v) { raw(&v, 4); };
  auto u64w = [&](uint64_t v) { raw(&v, 8); };
  raw("FLIVFPQ1", 8);
  u32(uint32_t(ix->metric));
  u32(ix->dim);
  u32(uint32_t(ix->nlist));
  u32(uint32_t(ix->m));
  u32(uint32_t(ix->count));
  u64w(ix->h_centroids.size());
  raw(ix->h_centroids.data(), ix->h_centroids.size() * 4);
  u64w(ix->h_codebooks.size());
  raw(ix->h_codebooks.data(), ix->h_codebooks.size() * 4);
  for (size_t l = 0; l < ix->nlist; l++) {
    const size_t o = ix->h_off[l], c = ix->h_off[l + 1] - o;
    u64w(c);
    raw(ids.data() + o, c * 4);
    u64w(c * ix->m);
    raw(codes.data() + o * ix->m, c * ix->m);
  }
  if (ix->keep) {
    const size_t nf = ix->count * size_t(ix->pd);
    u64w(nf);
    if (nf) FV_CUDA(cudaMemcpy(w, ix->vectors.p, nf * 4, cudaMemcpyDeviceToHost));
    w += nf * 4;
  } else {
    u64w(0);
  }
  u32(ix->keep ? 1u : 0u);
  if (written) *written = size_t(w - buf);
  return FV_OK;
}

int fv_ivfpq_load(fv_ctx* ctx, const uint8_t* bytes, size_t len, fv_ivfpq** out) {
  if (!ctx || !bytes || !out) return fv::fail(FV_ERR_ARG, "fv_ivfpq_load: null argument");
  if (len < 8 || std::memcmp(bytes, "FLIVFPQ1", 8) != 0) return fv::fail(FV_ERR_FILE, "not an IVF-PQ index file");
  size_t i = 8;
  bool ok = true;
  auto take = [&](size_t n) -> const uint8_t* {
    if (!ok || n > len - i) {
      ok = false;
      return nullptr;
    }
    const uint8_t* p = bytes + i;
    i += n;
    return p;
  };
  auto u32 = [&]() {
    uint32_t v = 0;
    if (auto p = take(4)) std::memcpy(&v, p, 4);
    return v;
  };
  auto u64r = [&]() {
    uint64_t v = 0;
    if (auto p = take(8)) std::memcpy(&v, p, 8);
    return v;
  };
  auto span = [&](size_t elem, size_t* count) -> const uint8_t* {
    uint64_t n = u64r();
    if (!ok || n > (len - i) / elem) {
      ok = false;
      return nullptr;
    }
    *count = size_t(n);
    return take(size_t(n) * elem);
  };
  const char* trunc = "index file is truncated";
  auto ix = std::unique_ptr<fv_ivfpq>(new fv_ivfpq());
  ix->ctx = ctx;
  fv::ctx_retain(ctx);
  const uint32_t mc = u32();
  ix->dim = u32();
  ix->nlist = u32();
  ix->m = u32();
  ix->count = u32();
  ix->seen = ix->count;
  if (!ok) return fv::fail(FV_ERR_FILE, trunc);
  if ((mc & 0xFF) > 1) return fv::fail(FV_ERR_FILE, "bad metric");
  ix->metric = int(mc & 0xFF);
  size_t nc = 0, nb = 0;
  const uint8_t* pc = span(4, &nc);
  const uint8_t* pb = span(4, &nb);
  if (!ok) return fv::fail(FV_ERR_FILE, trunc);
  ix->h_centroids.resize(nc);
  std::memcpy(ix->h_centroids.data(), pc, nc * 4);
  ix->h_codebooks.resize(nb);
  std::memcpy(ix->h_codebooks.data(), pb, nb * 4);
  ix->pd = uint32_t(fv::padded(ix->dim));
  if (ix->m == 0 || ix->dim == 0 || ix->pd % ix->m != 0 || nc != ix->nlist * size_t(ix->pd) ||
      nb != ix->m * fv::KSUB * (ix->pd / ix->m))
    return fv::fail(FV_ERR_FILE, "index file sizes do not match");
  ix->dsub = ix->pd / ix->m;
  std::vector<uint32_t> ids;
  std::vector<uint8_t> codes;
  ix->h_off.assign(ix->nlist + 1, 0);
  for (size_t l = 0; l < ix->nlist; l++) {
    size_t ni = 0, ncb = 0;
    const uint8_t* pi = span(4, &ni);
    const uint8_t* pcd = span(1, &ncb);
    if (!ok) return fv::fail(FV_ERR_FILE, trunc);
    if (ncb != ni * ix->m) return fv::fail(FV_ERR_FILE, "index file sizes do not match");
    const size_t o = ids.size();
    ids.resize(o + ni);
    std::memcpy(ids.data() + o, pi, ni * 4);
    codes.insert(codes.end(), pcd, pcd + ncb);
    ix->h_off[l + 1] = uint32_t(ids.size());
  }
  size_t nv = 0;
  const uint8_t* pv = span(4, &nv);
  const bool has = u32() == 1;
  if (!ok) return fv::fail(FV_ERR_FILE, trunc);
  if (ids.size() != ix->count || (has && nv != ix->count * size_t(ix->pd)))
    return fv::fail(FV_ERR_FILE, "index file sizes do not match");
  ix->keep = has;
  // With kept vectors the search re-ranks candidate `id` from row `id` of them (ivfpq.rs:289 indexes the same way and
  // panics on a bad id): a damaged file must not send the kernel out of bounds.
  if (has)
    for (uint32_t id : ids)
      if (id >= ix->count) return fv::fail(FV_ERR_FILE, "index file holds a row id beyond its row count");
  fv::CtxGuard g(ctx);
  FV_TRY(fv::upload_quantizers(ix.get()));
  FV_TRY(fv::upload_offsets(ix.get()));
  FV_TRY(ix->ids.reserve(ix->count * 4 + 16));
  FV_TRY(ix->codes.reserve(ix->count * ix->m + 16));
  if (ix->count) {
    FV_CUDA(cudaMemcpyAsync(ix->ids.p, ids.data(), ix->count * 4, cudaMemcpyHostToDevice, ctx->stream));
    FV_CUDA(cudaMemcpyAsync(ix->codes.p, codes.data(), ix->count * ix->m, cudaMemcpyHostToDevice, ctx->stream));
  }
  if (has && nv) {
    FV_TRY(ix->vectors.reserve(nv * 4));
    FV_CUDA(cudaMemcpyAsync(ix->vectors.p, pv, nv * 4, cudaMemcpyHostToDevice, ctx->stream));
  }
  FV_CUDA(cudaStreamSynchronize(ctx->stream));
  FV_TRY(fv::refresh_transposed(ix.get()));
  // A loaded index reports the ids stored in the file; rows of the kept vectors are indexed by id.
  ix->id_base = 0;
  *out = ix.release();
  return FV_OK;
}

// Cross-shard re-ranking: global best `keep` by compressed distance, then the k best of those by exact distance.
namespace fv {
// Part p's candidates of query q start at adc[p * adc_stride + q * keep] and exact[p * exact_stride + q * keep].
__global__ void merge_refine_kernel(const fv_neighbor* __restrict__ adc, const float* __restrict__ exact,
                                    const uint32_t* __restrict__ part_counts, int nparts, size_t nq, int keep, int k,
                                    size_t adc_stride, size_t exact_stride, u64* __restrict__ out) {
  unsigned char* smem_raw = dyn_smem();
  const int lane = threadIdx.x & 31;
  const size_t q = blockIdx.x;
  u64* list = reinterpret_cast<u64*>(smem_raw);  // keep: (adc, id) keys
  u64* fin = list + keep;                        // k
  // the position of a candidate in its shard's block rides along in a side table keyed by id: since ids are
  // unique across shards, re-find the exact distance by scanning the shard blocks after the cut.
  warp_list_init(list, keep);
  warp_list_init(fin, k);
  u64 bound = FV_EMPTY_KEY;
  for (int p = 0; p < nparts; ++p) {
    const int cnt = part_counts ? int(min(part_counts[size_t(p) * nq + q], uint32_t(keep))) : keep;
    const fv_neighbor* src = adc + size_t(p) * adc_stride + q * size_t(keep);
    for (int i0 = 0; i0 < cnt; i0 += 32) {
      const int i = i0 + lane;
      u64 key = FV_EMPTY_KEY;
      if (i < cnt && src[i].id != 0xFFFFFFFFu) key = make_key(src[i].distance, src[i].id);
      bound = warp_list_offer(list, keep, key, bound);
    }
  }
  __syncwarp();
  const u64 cut = list[keep - 1];  // candidates with key <= cut survive
  u64 b2 = FV_EMPTY_KEY;
  for (int p = 0; p < nparts; ++p) {
    const int cnt = part_counts ? int(min(part_counts[size_t(p) * nq + q], uint32_t(keep))) : keep;
    const size_t base = size_t(p) * adc_stride + q * size_t(keep), ebase = size_t(p) * exact_stride + q * size_t(keep);
    for (int i0 = 0; i0 < cnt; i0 += 32) {
      const int i = i0 + lane;
      u64 key = FV_EMPTY_KEY;
      if (i < cnt && adc[base + i].id != 0xFFFFFFFFu) {
        const u64 ak = make_key(adc[base + i].distance, adc[base + i].id);
        if (ak <= cut) key = make_key(exact[ebase + i], adc[base + i].id);
      }
      b2 = warp_list_offer(fin, k, key, b2);
    }
  }
  __syncwarp();
  for (int e = lane; e < k; e += 32) out[q * size_t(k) + e] = fin[e];
}

// The same for at most 32 * NPL candidates per query, without sorted insertion: a lane keeps its share of the
// (compressed distance, id) keys in registers, 64 bisection steps find the keep-th smallest key (ids are unique, so
// keys are), and only the survivors' exact keys are offered to the k-long result list.  One warp per query.
extern "C++" {
template <int NPL>
__global__ void __launch_bounds__(128) merge_refine_select_kernel(const fv_neighbor* __restrict__ adc,
                                                                  const float* __restrict__ exact,
                                                                  const uint32_t* __restrict__ part_counts, int nparts,
                                                                  size_t nq, int keep, int k, size_t adc_stride,
                                                                  size_t exact_stride, u64* __restrict__ out) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  const size_t q = blockIdx.x * size_t(blockDim.x >> 5) + w;
  if (q >= nq) return;
  u64* fin = reinterpret_cast<u64*>(dyn_smem()) + size_t(w) * k;
  const int total = nparts * keep;
  u64 key[NPL];
  int nvalid = 0;
#pragma unroll
  for (int j = 0; j < NPL; ++j) {
    const int e = j * 32 + lane;
    key[j] = FV_EMPTY_KEY;
    if (e < total) {
      const int p = e / keep, i = e - p * keep;
      const int cnt = part_counts ? int(min(part_counts[size_t(p) * nq + q], uint32_t(keep))) : keep;
      const fv_neighbor nb = adc[size_t(p) * adc_stride + q * size_t(keep) + i];
      if (i < cnt && nb.id != 0xFFFFFFFFu) {
        key[j] = make_key(nb.distance, nb.id);
        nvalid++;
      }
    }
  }
  nvalid = __reduce_add_sync(FV_FULL, nvalid);
  const int want = min(keep, nvalid);
  u64 lo = 0, hi = FV_EMPTY_KEY - 1;  // the smallest T with at least `want` keys <= T
  while (lo < hi) {
    const u64 mid = lo + ((hi - lo) >> 1);
    int c = 0;
#pragma unroll
    for (int j = 0; j < NPL; ++j) c += key[j] <= mid ? 1 : 0;
    c = __reduce_add_sync(FV_FULL, c);
    if (c >= want) hi = mid;
    else lo = mid + 1;
  }
  const u64 cut = want > 0 ? lo : 0;
  warp_list_init(fin, k);
  u64 b2 = FV_EMPTY_KEY;
#pragma unroll
  for (int j = 0; j < NPL; ++j) {
    const int e = j * 32 + lane;
    u64 ek = FV_EMPTY_KEY;
    if (want > 0 && key[j] <= cut) {
      const int p = e / keep, i = e - p * keep;
      ek = make_key(exact[size_t(p) * exact_stride + q * size_t(keep) + i], key_id(key[j]));
    }
    if (__any_sync(FV_FULL, ek != FV_EMPTY_KEY)) b2 = warp_list_offer(fin, k, ek, b2);
  }
  __syncwarp();
  for (int e = lane; e < k; e += 32) out[q * size_t(k) + e] = fin[e];
}
}  // extern "C++"
}  // namespace fv

// merge of the per-shard candidates (see merge_refine_kernel for the strides); keys to scratch slot 1, then neighbours
static int merge_refine_impl(fv_ctx* ctx, const fv_neighbor* d_adc_parts, const float* d_exact_parts,
                             const uint32_t* d_part_counts, size_t nparts, size_t nq, size_t keep, size_t k,
                             size_t adc_stride, size_t exact_stride, fv_neighbor* d_out, uint32_t* d_counts) {
  FV_TRY(ctx->scratch[1].reserve(nq * k * sizeof(u64)));
  u64* keys = ctx->scratch[1].as<u64>();
  const size_t smem = (keep + k) * sizeof(u64);
  if (smem > 40 * 1024)
    FV_CUDA(cudaFuncSetAttribute(fv::merge_refine_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)));
  if (nparts * keep <= 1024 && k <= 256) {
    const unsigned blocks = unsigned((nq + 3) / 4);
    const size_t sm = 4 * k * sizeof(u64);
    if (nparts * keep <= 256)
      fv::merge_refine_select_kernel<8><<<blocks, 128, sm, ctx->stream>>>(d_adc_parts, d_exact_parts, d_part_counts,
                                                                         int(nparts), nq, int(keep), int(k), adc_stride,
                                                                         exact_stride, keys);
    else
      fv::merge_refine_select_kernel<32><<<blocks, 128, sm, ctx->stream>>>(d_adc_parts, d_exact_parts, d_part_counts,
                                                                          int(nparts), nq, int(keep), int(k), adc_stride,
                                                                          exact_stride, keys);
  } else {
    fv::merge_refine_kernel<<<unsigned(nq), 32, smem, ctx->stream>>>(d_adc_parts, d_exact_parts, d_part_counts,
                                                                    int(nparts), nq, int(keep), int(k), adc_stride,
                                                                    exact_stride, keys);
  }
  ctx->stats.launches++;
  FV_CUDA(cudaGetLastError());
  FV_TRY(fv::keys_to_neighbors(ctx, keys, nq, int(k), int(k), d_out, d_counts));
  return FV_OK;
}

int fv_merge_refine_dev(fv_ctx* ctx, const fv_neighbor* d_adc_parts, const float* d_exact_parts,
                        const uint32_t* d_part_counts, size_t nparts, size_t nq, size_t keep, size_t k,
                        fv_neighbor* d_out, uint32_t* d_counts) {
  if (!ctx || !d_adc_parts || !d_exact_parts || !d_out || nparts == 0 || keep == 0 || k == 0)
    return fv::fail(FV_ERR_ARG, "fv_merge_refine_dev: bad argument");
  if (keep > 4096 || k > 4096) return fv::fail(FV_ERR_UNSUPPORTED, "k * refine above 4096 is not supported");
  if (nq == 0) return FV_OK;
  fv::CtxGuard g(ctx);
  FV_TRY(merge_refine_impl(ctx, d_adc_parts, d_exact_parts, d_part_counts, nparts, nq, keep, k, nq * keep, nq * keep, d_out,
                           d_counts));
  FV_CUDA(cudaStreamSynchronize(ctx->stream));
  return FV_OK;
}

// ---- search over list shards, one per rank of the context's communicator: coarse cells by query slices (exchanged),
// the local scan, one exchange of the per-shard candidates, the merge.  Every rank ends up with the full result.
// Stages (fv_stats.stage_ms): 0 coarse cells of this rank's query slice, 1 their exchange, 2 the local search up to
// its candidates (bound pass, bucketing, scan, re-score, sort, re-rank), 3 the candidate exchange, 4 the merge.
// Sharded search on a grid with more than one query slice.  Rank (slice s, list shard l) searches query slice s on
// its lists; with L > 1 the L shards of a slice exchange their candidates (one all-gather over the whole group, each
// rank reading the blocks of its slice) and merge them as the reference cuts (ivfpq.rs:285-296); the finished slices
// are then gathered so that every rank holds the whole result.  Called with the context locked and its stage table
// open (stages: 0 and 1 empty, 2 local search, 3 candidate exchange, 4 merge, result exchange and unpacking).
// The gathered result blocks (per slice: per x k neighbours, then per counts; the blocks of a slice's L shards are
// adjacent and equal) laid out as the caller's arrays, in one launch.
__global__ void unpack_slices_kernel(const unsigned char* __restrict__ all, size_t rblk, int L, size_t per, size_t k,
                                     size_t nq, fv_neighbor* __restrict__ out, uint32_t* __restrict__ counts) {
  const size_t total = nq * k;
  for (size_t i = blockIdx.x * size_t(blockDim.x) + threadIdx.x; i < total + nq; i += size_t(gridDim.x) * blockDim.x) {
    if (i < total) {
      const size_t q = i / k, s = q / per;
      const fv_neighbor* src = reinterpret_cast<const fv_neighbor*>(all + s * size_t(L) * rblk);
      out[i] = src[(q - s * per) * k + (i - q * k)];
    } else if (counts) {
      const size_t q = i - total, s = q / per;
      const uint32_t* src = reinterpret_cast<const uint32_t*>(all + s * size_t(L) * rblk + per * k * sizeof(fv_neighbor));
      counts[q] = src[q - s * per];
    }
  }
}

static int search_grid(fv_ivfpq* ix, const float* d_queries, size_t nq, size_t k, size_t nprobe, size_t refine,
                       fv_neighbor* d_out, uint32_t* d_counts, int L) {
  fv_ctx* ctx = ix->ctx;
  const int world = ctx->comm_size, rank = ctx->comm_rank;
  const int Q = world / L, slice = rank / L;
  const size_t per = (nq + size_t(Q) - 1) / size_t(Q);
  const size_t lo = std::min(nq, size_t(slice) * per), hi = std::min(nq, lo + per), ns = hi - lo;
  const float* q = d_queries + lo * size_t(ix->dim);
  fv::stage_mark_outer(ctx);  // 0
  fv::stage_mark_outer(ctx);  // 1
  // the finished slice: per x k neighbours, then per counts
  const size_t rblk = (per * k * sizeof(fv_neighbor) + per * sizeof(uint32_t) + 15) & ~size_t(15);
  FV_TRY(ctx->scratch[16].reserve(rblk));  // slots 16 and 17 belong to this function: the slice's result lives across the local search
  unsigned char* res = ctx->scratch[16].as<unsigned char>();
  fv_neighbor* res_nb = reinterpret_cast<fv_neighbor*>(res);
  uint32_t* res_cnt = reinterpret_cast<uint32_t*>(res + per * k * sizeof(fv_neighbor));
  const bool rerank = refine > 0 && ix->keep;
  if (L == 1) {
    if (ns) FV_TRY(ivfpq_search_impl(ix, q, ns, k, nprobe, refine, false, res_nb, res_cnt, nullptr, nullptr));
    fv::stage_mark_outer(ctx);  // 2
    fv::stage_mark_outer(ctx);  // 3
  } else if (rerank) {
    const size_t keep = k * refine;
    const size_t blk = (per * keep * 12 + 15) & ~size_t(15);
    FV_TRY(ctx->scratch[10].reserve(blk));
    unsigned char* send = ctx->scratch[10].as<unsigned char>();
    fv_neighbor* adc = reinterpret_cast<fv_neighbor*>(send);
    float* exact = reinterpret_cast<float*>(send + per * keep * sizeof(fv_neighbor));
    FV_TRY(ctx->scratch[11].reserve(per * sizeof(uint32_t)));
    if (ns) FV_TRY(ivfpq_search_impl(ix, q, ns, keep, nprobe, 1, true, nullptr, ctx->scratch[11].as<uint32_t>(), adc, exact, nullptr));
    fv::stage_mark_outer(ctx);  // 2
    FV_TRY(ctx->scratch[15].reserve(size_t(world) * blk));
    unsigned char* recv = ctx->scratch[15].as<unsigned char>();
    FV_TRY(fv::comm_all_gather(ctx, send, recv, blk));
    fv::stage_mark_outer(ctx);  // 3
    const unsigned char* mine = recv + size_t(slice) * size_t(L) * blk;  // the L blocks of this slice are adjacent
    if (ns)
      FV_TRY(merge_refine_impl(ctx, reinterpret_cast<const fv_neighbor*>(mine),
                               reinterpret_cast<const float*>(mine + per * keep * sizeof(fv_neighbor)), nullptr, size_t(L), ns, keep,
                               k, blk / sizeof(fv_neighbor), blk / sizeof(float), res_nb, res_cnt));
  } else {
    const size_t blk = (per * k * sizeof(fv_neighbor) + 15) & ~size_t(15);
    FV_TRY(ctx->scratch[10].reserve(blk));
    FV_TRY(ctx->scratch[11].reserve(per * sizeof(uint32_t)));
    fv_neighbor* part = ctx->scratch[10].as<fv_neighbor>();
    if (ns) FV_TRY(ivfpq_search_impl(ix, q, ns, k, nprobe, 0, false, part, ctx->scratch[11].as<uint32_t>(), nullptr, nullptr, nullptr));
    fv::stage_mark_outer(ctx);  // 2
    FV_TRY(ctx->scratch[15].reserve(size_t(world) * blk));
    FV_TRY(fv::comm_all_gather(ctx, part, ctx->scratch[15].p, blk));
    fv::stage_mark_outer(ctx);  // 3
    const fv_neighbor* mine = reinterpret_cast<const fv_neighbor*>(ctx->scratch[15].as<unsigned char>() + size_t(slice) * size_t(L) * blk);
    if (ns) FV_TRY(fv::merge_topk_impl(ctx, mine, nullptr, size_t(L), ns, k, k, res_nb, res_cnt, blk / sizeof(fv_neighbor)));
  }
  // every rank gets every slice (the L shards of a slice hold the same one: shard 0's is taken)
  FV_TRY(ctx->scratch[17].reserve(size_t(world) * rblk));
  unsigned char* all = ctx->scratch[17].as<unsigned char>();
  FV_TRY(fv::comm_all_gather(ctx, res, all, rblk));
  {
    const size_t items = nq * k + nq;
    const unsigned blocks = unsigned(std::min<size_t>((items + 255) / 256, size_t(ctx->sm_count) * 8));
    unpack_slices_kernel<<<blocks, 256, 0, ctx->stream>>>(all, rblk, L, per, k, nq, d_out, d_counts);
    ctx->stats.launches++;
    FV_CUDA(cudaGetLastError());
  }
  fv::stage_mark_outer(ctx);  // 4
  FV_CUDA(cudaStreamSynchronize(ctx->stream));
  return FV_OK;
}

int fv_ivfpq_search_sharded_dev(fv_ivfpq* ix, const float* d_queries, size_t nq, size_t k, size_t nprobe, size_t refine,
                                fv_neighbor* d_out, uint32_t* d_counts) {
  if (!ix || (nq && (!d_queries || !d_out))) return fv::fail(FV_ERR_ARG, "fv_ivfpq_search_sharded: null argument");
  fv_ctx* ctx = ix->ctx;
  fv::CtxGuard g(ctx);
  const int world = ctx->comm_size, rank = ctx->comm_rank;
  if (world <= 1) return ivfpq_search_impl(ix, d_queries, nq, k, nprobe, refine, false, d_out, d_counts, nullptr, nullptr);
  // The group is a grid of L list shards x Q query slices, rank = slice * L + list shard: L is the number of shards
  // the index was built for (1: every rank holds all lists), Q = group size / L.
  const int L = std::max(1, ix->shard_world);
  if (world % L != 0 || ix->shard_rank != rank % L)
    return fv::fail(FV_ERR_ARG, "the index's shard (fv_ivfpq_set_shard) does not fit the context's group: its shard count must "
                                "divide the group size and its shard number equal rank % shard count");
  if (nq == 0) return FV_OK;
  if (k == 0 || nprobe == 0) return fv::fail(FV_ERR_ARG, "k and nprobe must be at least 1");
  const size_t np = std::min(nprobe, ix->nlist);
  fv::StageScope scope(ctx);  // one stage table for the whole call: the inner searches do not restart it
  if (world / L > 1) return search_grid(ix, d_queries, nq, k, nprobe, refine, d_out, d_counts, L);
  // every shard needs the probed cells of all queries: rank r computes those of query slice r
  const size_t per = (nq + size_t(world) - 1) / size_t(world);
  const size_t lo = std::min(nq, size_t(rank) * per), hi = std::min(nq, lo + per);
  const uint64_t* cells = nullptr;
  if (nq >= 256 * size_t(world)) {
    FV_TRY(ctx->scratch[13].reserve(per * np * sizeof(u64)));
    u64* mine = ctx->scratch[13].as<u64>();
    if (hi > lo)
      FV_TRY(ivfpq_search_impl(ix, d_queries + lo * size_t(ix->dim), hi - lo, 1, nprobe, 0, false, nullptr, nullptr, nullptr,
                               nullptr, nullptr, reinterpret_cast<uint64_t*>(mine)));
    if (hi - lo < per) FV_CUDA(cudaMemsetAsync(mine + (hi - lo) * np, 0xFF, (per - (hi - lo)) * np * sizeof(u64), ctx->stream));
    fv::stage_mark_outer(ctx);  // 0
    FV_TRY(ctx->scratch[14].reserve(size_t(world) * per * np * sizeof(u64)));
    u64* all = ctx->scratch[14].as<u64>();
    FV_TRY(fv::comm_all_gather(ctx, mine, all, per * np * sizeof(u64)));
    // the gathered keys are needed until the local search has bucketed them; it uses slot 14 itself only on the
    // tensor-core path, after the pairs are built -- so they move to a slot of their own
    FV_TRY(ctx->scratch[4].reserve(nq * np * sizeof(u64)));
    FV_CUDA(cudaMemcpyAsync(ctx->scratch[4].p, all, nq * np * sizeof(u64), cudaMemcpyDeviceToDevice, ctx->stream));
    cells = ctx->scratch[4].as<uint64_t>();
    fv::stage_mark_outer(ctx);  // 1
  } else {
    fv::stage_mark_outer(ctx);  // 0 (the local search does its own coarse step)
    fv::stage_mark_outer(ctx);  // 1
  }
  const bool rerank = refine > 0 && ix->keep;
  if (rerank) {
    // a shard may not cut to k on its own: the global cut by compressed distance comes first (ivfpq.rs:285-296).
    // One record block per rank: its candidates (id, compressed distance), then their exact distances.
    const size_t keep = k * refine;
    const size_t blk = (nq * keep * 12 + 15) & ~size_t(15);
    FV_TRY(ctx->scratch[10].reserve(blk));
    unsigned char* send = ctx->scratch[10].as<unsigned char>();
    fv_neighbor* adc = reinterpret_cast<fv_neighbor*>(send);
    float* exact = reinterpret_cast<float*>(send + nq * keep * sizeof(fv_neighbor));
    FV_TRY(ctx->scratch[11].reserve(nq * sizeof(uint32_t)));
    FV_TRY(ivfpq_search_impl(ix, d_queries, nq, keep, nprobe, 1, true, nullptr, ctx->scratch[11].as<uint32_t>(), adc, exact, cells));
    fv::stage_mark_outer(ctx);  // 2
    FV_TRY(ctx->scratch[15].reserve(size_t(world) * blk));
    unsigned char* recv = ctx->scratch[15].as<unsigned char>();
    FV_TRY(fv::comm_all_gather(ctx, send, recv, blk));
    fv::stage_mark_outer(ctx);  // 3
    FV_TRY(merge_refine_impl(ctx, reinterpret_cast<const fv_neighbor*>(recv),
                             reinterpret_cast<const float*>(recv + nq * keep * sizeof(fv_neighbor)), nullptr, size_t(world), nq,
                             keep, k, blk / sizeof(fv_neighbor), blk / sizeof(float), d_out, d_counts));
  } else {
    const size_t blk = nq * k * sizeof(fv_neighbor);
    FV_TRY(ctx->scratch[10].reserve(blk));
    FV_TRY(ctx->scratch[11].reserve(nq * sizeof(uint32_t)));
    fv_neighbor* mine = ctx->scratch[10].as<fv_neighbor>();
    FV_TRY(ivfpq_search_impl(ix, d_queries, nq, k, nprobe, 0, false, mine, ctx->scratch[11].as<uint32_t>(), nullptr, nullptr, cells));
    fv::stage_mark_outer(ctx);  // 2
    FV_TRY(ctx->scratch[15].reserve(size_t(world) * blk));
    FV_TRY(fv::comm_all_gather(ctx, mine, ctx->scratch[15].p, blk));
    fv::stage_mark_outer(ctx);  // 3
    FV_TRY(fv::merge_topk_impl(ctx, ctx->scratch[15].as<fv_neighbor>(), nullptr, size_t(world), nq, k, k, d_out, d_counts));
  }
  fv::stage_mark_outer(ctx);  // 4
  FV_CUDA(cudaStreamSynchronize(ctx->stream));
  return FV_OK;
}

}  // extern "C"
