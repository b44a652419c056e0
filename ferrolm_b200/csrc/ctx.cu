// Context, error reporting and the small host-side helpers of src/vector/mod.rs.
#include <cmath>
#include <mutex>
#include <thread>
#include <unordered_set>

#include "internal.h"

namespace fv {

static thread_local std::string g_error;

void set_error(const std::string& msg) { g_error = msg; }
int fail(int status, const std::string& msg) {
  g_error = msg;
  return status;
}

static std::mutex g_ctx_mutex;
}  // namespace fv
static void ctx_destroy_now(fv_ctx* ctx);
namespace fv {
void ctx_retain(fv_ctx* ctx) {
  std::lock_guard<std::mutex> g(g_ctx_mutex);
  ctx->refs++;
}
void ctx_release(fv_ctx* ctx) {
  std::lock_guard<std::mutex> g(g_ctx_mutex);
  if (--ctx->refs == 0 && ctx->closing) ctx_destroy_now(ctx);
}

void stage_mark_outer(fv_ctx* ctx) {
  if (!ctx->timing || ctx->ev_used == 0 || ctx->ev_used > FV_NSTAGE) return;
  cudaEventRecord(ctx->ev[ctx->ev_used], ctx->stream);
  ctx->ev_used++;
}
void stage_begin(fv_ctx* ctx) {
  if (ctx->stage_outer) return;
  ctx->ev_used = 0;
  for (int i = 0; i < FV_NSTAGE; i++) ctx->stats.stage_ms[i] = 0.f;
  if (!ctx->timing) return;
  cudaEventRecord(ctx->ev[0], ctx->stream);
  ctx->ev_used = 1;
}
void stage_mark(fv_ctx* ctx) {
  if (ctx->stage_outer || !ctx->timing || ctx->ev_used == 0 || ctx->ev_used > FV_NSTAGE) return;
  cudaEventRecord(ctx->ev[ctx->ev_used], ctx->stream);
  ctx->ev_used++;
}
void stage_end(fv_ctx* ctx) {
  if (ctx->stage_outer || !ctx->timing) return;
  for (int i = 0; i < FV_NSTAGE; i++) ctx->stats.stage_ms[i] = 0.f;
  for (int i = 1; i < ctx->ev_used; i++) {
    float ms = 0.f;
    if (cudaEventElapsedTime(&ms, ctx->ev[i - 1], ctx->ev[i]) == cudaSuccess) ctx->stats.stage_ms[i - 1] = ms;
  }
}

__global__ void pad_rows_kernel(const float* __restrict__ src, float* __restrict__ dst, size_t n, int dim, int pd) {
  size_t total = n * size_t(pd);
  for (size_t i = blockIdx.x * size_t(blockDim.x) + threadIdx.x; i < total; i += size_t(gridDim.x) * blockDim.x) {
    size_t r = i / pd;
    int c = int(i - r * pd);
    dst[i] = c < dim ? src[r * dim + c] : 0.f;
  }
}

int upload_padded(fv_ctx* ctx, const float* src, bool src_is_device, size_t n, size_t dim, size_t pd, float* d_dst) {
  if (n == 0) return FV_OK;
  if (pd == dim) {
    FV_CUDA(cudaMemcpyAsync(d_dst, src, n * dim * sizeof(float),
                            src_is_device ? cudaMemcpyDeviceToDevice : cudaMemcpyHostToDevice, ctx->stream));
    return FV_OK;
  }
  if (src_is_device) {
    pad_rows_kernel<<<ctx->sm_count * 4, 256, 0, ctx->stream>>>(src, d_dst, n, int(dim), int(pd));
    ctx->stats.launches++;
    FV_CUDA(cudaGetLastError());
    return FV_OK;
  }
  FV_CUDA(cudaMemsetAsync(d_dst, 0, n * pd * sizeof(float), ctx->stream));
  FV_CUDA(cudaMemcpy2DAsync(d_dst, pd * sizeof(float), src, dim * sizeof(float), dim * sizeof(float), n,
                            cudaMemcpyHostToDevice, ctx->stream));
  return FV_OK;
}

}  // namespace fv

static void ctx_destroy_now(fv_ctx* ctx) {
  fv::DeviceGuard g(ctx->device);
  cudaStreamSynchronize(ctx->stream);
  fv::comm_destroy(ctx);
  for (auto& b : ctx->scratch) b.release();
  for (auto& ev : ctx->ev)
    if (ev) cudaEventDestroy(ev);
  if (ctx->d_flags) cudaFree(ctx->d_flags);
  cudaStreamDestroy(ctx->stream);
  delete ctx;
}

extern "C" {

const char* fv_last_error(void) { return fv::g_error.c_str(); }
const char* fv_version(void) { return "ferrovec 0.1 (sm_100a)"; }

int fv_ctx_create(int device, fv_ctx** out) {
  if (!out) return fv::fail(FV_ERR_ARG, "fv_ctx_create: out is null");
  *out = nullptr;
  int count = 0;
  cudaError_t e = cudaGetDeviceCount(&count);
  if (e != cudaSuccess || count == 0) {
    (void)cudaGetLastError();
    return fv::fail(FV_ERR_CUDA, std::string("no CUDA device: ") + (e != cudaSuccess ? cudaGetErrorString(e) : "count is 0") +
                                     " (this library has no CPU path)");
  }
  if (device < 0 || device >= count) return fv::fail(FV_ERR_ARG, "fv_ctx_create: no such device");
  cudaDeviceProp prop;
  FV_CUDA(cudaGetDeviceProperties(&prop, device));
  if (prop.major != 10)
    return fv::fail(FV_ERR_CUDA, std::string("device ") + prop.name + " is sm_" + std::to_string(prop.major) +
                                     std::to_string(prop.minor) + "; this library is built for sm_100a only");
  fv::DeviceGuard g(device);
  if (!g.ok) return fv::fail(FV_ERR_CUDA, "cudaSetDevice failed");
  auto* ctx = new fv_ctx();
  ctx->device = device;
  ctx->sm_count = prop.multiProcessorCount;
  ctx->smem_optin = prop.sharedMemPerBlockOptin;
  if (cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking) != cudaSuccess) {
    delete ctx;
    return fv::fail(FV_ERR_CUDA, "cudaStreamCreate failed");
  }
  for (auto& ev : ctx->ev) cudaEventCreate(&ev);
  if (cudaMalloc(&ctx->d_flags, 64 * sizeof(int)) != cudaSuccess) {
    cudaStreamDestroy(ctx->stream);
    delete ctx;
    return fv::fail(FV_ERR_NOMEM, "cudaMalloc failed");
  }
  cudaMemset(ctx->d_flags, 0, 64 * sizeof(int));
  *out = ctx;
  return FV_OK;
}

void fv_ctx_destroy(fv_ctx* ctx) {
  if (!ctx) return;
  std::lock_guard<std::mutex> g(fv::g_ctx_mutex);
  if (ctx->refs > 0) {
    ctx->closing = true;  // freed with the last index
    return;
  }
  ctx_destroy_now(ctx);
}

int fv_ctx_device(const fv_ctx* ctx) { return ctx ? ctx->device : -1; }

int fv_ctx_sync(fv_ctx* ctx) {
  if (!ctx) return fv::fail(FV_ERR_ARG, "null context");
  fv::CtxGuard g(ctx);
  FV_CUDA(cudaStreamSynchronize(ctx->stream));
  return FV_OK;
}

void* fv_ctx_stream(fv_ctx* ctx) { return ctx ? (void*)ctx->stream : nullptr; }

int fv_ctx_stats(const fv_ctx* ctx, fv_stats* out) {
  if (!ctx || !out) return fv::fail(FV_ERR_ARG, "null argument");
  std::lock_guard<std::recursive_mutex> lk(const_cast<fv_ctx*>(ctx)->mu);
  *out = ctx->stats;
  return FV_OK;
}

int fv_ctx_set_timing(fv_ctx* ctx, int on) {
  if (!ctx) return fv::fail(FV_ERR_ARG, "null context");
  std::lock_guard<std::recursive_mutex> lk(ctx->mu);
  ctx->timing = on != 0;
  return FV_OK;
}

size_t fv_padded(size_t dim) { return fv::padded(dim); }

// src/vector/mod.rs:132-141: sequential sum of squares (no fusing), sqrt, divide.
int fv_normalize(float* data, size_t n, size_t dim) {
  if (!data && n) return fv::fail(FV_ERR_ARG, "null data");
  for (size_t i = 0; i < n; i++) {
    float* v = data + i * dim;
    volatile float s = -0.0f;  // volatile: keeps the compiler from fusing or reassociating the sum
    for (size_t d = 0; d < dim; d++) {
      volatile float sq = v[d] * v[d];
      s = s + sq;
    }
    float nn = std::sqrt(s);
    if (nn > 0.0f)
      for (size_t d = 0; d < dim; d++) v[d] /= nn;
  }
  return FV_OK;
}

// src/vector/mod.rs:145-152
double fv_recall(const fv_neighbor* found, const uint32_t* counts, const uint32_t* truth, size_t truth_stride,
                 size_t nq, size_t k) {
  size_t hit = 0;
  for (size_t i = 0; i < nq; i++) {
    std::unordered_set<uint32_t> want;
    for (size_t t = 0; t < k && t < truth_stride; t++) want.insert(truth[i * truth_stride + t]);
    size_t c = counts ? (counts[i] < k ? counts[i] : k) : k;
    for (size_t j = 0; j < c; j++) hit += want.count(found[i * k + j].id);
  }
  return nq && k ? double(hit) / double(nq * k) : 0.0;
}

// Seeded Gaussian-mixture rows; row i is a function of (seed, i) only.
namespace {
struct XorShift {  // xorshift64* as in src/rng.rs:7-45
  uint64_t s;
  explicit XorShift(uint64_t seed) : s((seed * 0x9E3779B97F4A7C15ull) | 1ull) {}
  uint64_t next() {
    s ^= s >> 12;
    s ^= s << 25;
    s ^= s >> 27;
    return s * 0x2545F4914F6CDD1Dull;
  }
  double uniform() { return double(next() >> 11) / double(1ull << 53); }
  double normal() {
    double u = 1.0 - uniform();
    double v = uniform();
    return std::sqrt(-2.0 * std::log(u)) * std::cos(6.283185307179586476925286766559 * v);
  }
};
}  // namespace

int fv_datagen(int kind, uint64_t seed, size_t first_row, size_t n, size_t dim, size_t clusters, int threads,
               float* out) {
  if (!out || dim == 0 || clusters == 0 || (kind != 0 && kind != 1)) return fv::fail(FV_ERR_ARG, "fv_datagen: bad argument");
  std::vector<float> centres(clusters * dim);
  {
    XorShift c(seed * 1000003ull + 17);
    for (auto& v : centres) v = kind == 0 ? float(c.uniform() * 255.0) : float(c.normal()) * 3.0f;
  }
  int nt = threads > 0 ? threads : int(std::thread::hardware_concurrency());
  if (nt < 1) nt = 1;
  auto work = [&](int t) {
    for (size_t i = size_t(t); i < n; i += size_t(nt)) {
      size_t row = first_row + i;
      XorShift r(seed ^ ((row + 1) * 0xD1B54A32D192ED03ull));
      r.next();
      size_t c = size_t(r.next() % clusters);
      float* o = out + i * dim;
      if (kind == 0) {
        for (size_t d = 0; d < dim; d++) {
          float v = centres[c * dim + d] + float(r.normal()) * 30.0f;
          v = std::nearbyint(v);
          o[d] = v < 0.f ? 0.f : (v > 255.f ? 255.f : v);
        }
      } else {
        double ss = 0.0;
        for (size_t d = 0; d < dim; d++) {
          o[d] = centres[c * dim + d] + float(r.normal());
          ss += double(o[d]) * double(o[d]);
        }
        float inv = ss > 0 ? float(1.0 / std::sqrt(ss)) : 0.f;
        for (size_t d = 0; d < dim; d++) o[d] *= inv;
      }
    }
  };
  std::vector<std::thread> th;
  for (int t = 1; t < nt; t++) th.emplace_back(work, t);
  work(0);
  for (auto& t : th) t.join();
  return FV_OK;
}

}  // extern "C"

// ---- .fvecs / .ivecs files (src/vector/io.rs:7-42): per record a little-endian i32 dimension, then that many
// 4-byte values.  The buffer handed back is malloc'ed; release it with fv_free.
#include <cstdio>
#include <cstdlib>

static int read_vecs(const char* path, size_t limit, void** out, size_t* n, size_t* dim) {
  if (!path || !out || !n || !dim) return fv::fail(FV_ERR_ARG, "read_vecs: null argument");
  *out = nullptr;
  *n = *dim = 0;
  FILE* f = std::fopen(path, "rb");
  if (!f) return fv::fail(FV_ERR_FILE, std::string(path) + ": cannot open");
  std::fseek(f, 0, SEEK_END);
  const long long size = std::ftell(f);
  std::fseek(f, 0, SEEK_SET);
  if (size < 4) {
    std::fclose(f);
    return fv::fail(FV_ERR_FILE, std::string(path) + ": empty");
  }
  int32_t d = 0;
  if (std::fread(&d, 4, 1, f) != 1) d = 0;
  const size_t rec = 4 + 4 * size_t(d > 0 ? d : 0);
  if (d <= 0 || size_t(size) % rec != 0) {
    std::fclose(f);
    return fv::fail(FV_ERR_FILE, std::string(path) + ": not a vecs file of dimension " + std::to_string(d));
  }
  size_t rows = size_t(size) / rec;
  if (limit && limit < rows) rows = limit;
  unsigned char* buf = static_cast<unsigned char*>(std::malloc(rows * size_t(d) * 4 + 4));
  std::vector<unsigned char> line(rec);
  std::fseek(f, 0, SEEK_SET);
  for (size_t r = 0; r < rows; r++) {
    if (std::fread(line.data(), 1, rec, f) != rec) {
      std::free(buf);
      std::fclose(f);
      return fv::fail(FV_ERR_FILE, std::string(path) + ": short read");
    }
    int32_t dr;
    std::memcpy(&dr, line.data(), 4);
    if (dr != d) {
      std::free(buf);
      std::fclose(f);
      return fv::fail(FV_ERR_FILE, std::string(path) + ": record " + std::to_string(r) + " has a different dimension");
    }
    std::memcpy(buf + r * size_t(d) * 4, line.data() + 4, size_t(d) * 4);
  }
  std::fclose(f);
  *out = buf;
  *n = rows;
  *dim = size_t(d);
  return FV_OK;
}

extern "C" {
int fv_read_fvecs(const char* path, size_t limit, float** out, size_t* n, size_t* dim) {
  return read_vecs(path, limit, reinterpret_cast<void**>(out), n, dim);
}
int fv_read_ivecs(const char* path, size_t limit, uint32_t** out, size_t* n, size_t* dim) {
  return read_vecs(path, limit, reinterpret_cast<void**>(out), n, dim);
}
void fv_free(void* p) { std::free(p); }
}

// ---- the same generator on the device (kind 0 only), for bases too large to generate on the host cores.
// Same streams and formulas as fv_datagen; the device's double-precision log/cos may differ from the host
// library's in the last bit, so a value that lands within rounding of x.5 can round the other way: use one
// generator or the other for a given experiment, not both.
namespace fv {
__global__ void datagen_kernel(uint64_t seed, size_t first_row, size_t n, int dim, size_t clusters,
                               const float* __restrict__ centres, float* __restrict__ out) {
  for (size_t i = blockIdx.x * size_t(blockDim.x) + threadIdx.x; i < n; i += size_t(gridDim.x) * blockDim.x) {
    const size_t row = first_row + i;
    uint64_t s = ((seed ^ ((row + 1) * 0xD1B54A32D192ED03ull)) * 0x9E3779B97F4A7C15ull) | 1ull;
    auto next = [&]() {
      s ^= s >> 12;
      s ^= s << 25;
      s ^= s >> 27;
      return s * 0x2545F4914F6CDD1Dull;
    };
    next();
    const size_t c = size_t(next() % clusters);
    for (int d = 0; d < dim; d++) {
      const double u = 1.0 - double(next() >> 11) / 9007199254740992.0;
      const double v = double(next() >> 11) / 9007199254740992.0;
      const double nrm = sqrt(-2.0 * log(u)) * cos(6.283185307179586476925286766559 * v);
      float x = centres[c * dim + d] + float(nrm) * 30.0f;
      x = nearbyintf(x);
      out[i * size_t(dim) + d] = x < 0.f ? 0.f : (x > 255.f ? 255.f : x);
    }
  }
}
}  // namespace fv

extern "C" int fv_datagen_dev(fv_ctx* ctx, uint64_t seed, size_t first_row, size_t n, size_t dim, size_t clusters,
                              float* d_out) {
  if (!ctx || !d_out || dim == 0 || clusters == 0) return fv::fail(FV_ERR_ARG, "fv_datagen_dev: bad argument");
  if (n == 0) return FV_OK;
  std::vector<float> centres(clusters * dim);
  {
    XorShift c(seed * 1000003ull + 17);
    for (auto& v : centres) v = float(c.uniform() * 255.0);
  }
  fv::CtxGuard g(ctx);
  DevBuf d_cen;
  FV_TRY(d_cen.reserve(centres.size() * sizeof(float)));
  FV_CUDA(cudaMemcpyAsync(d_cen.p, centres.data(), centres.size() * sizeof(float), cudaMemcpyHostToDevice, ctx->stream));
  fv::datagen_kernel<<<ctx->sm_count * 8, 128, 0, ctx->stream>>>(seed, first_row, n, int(dim), clusters, d_cen.as<float>(),
                                                                d_out);
  FV_CUDA(cudaGetLastError());
  FV_CUDA(cudaStreamSynchronize(ctx->stream));
  return FV_OK;
}
