// Shared device helpers: order-preserving (distance, id) keys, the warp-owned
// sorted list used for every top-k, and the reference's exact distance chains.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include <string>

#include "../../include/ferrovec.h"

typedef unsigned long long u64;

namespace fv {

// ---------------------------------------------------------------------------------------------
// host-side error plumbing
void set_error(const std::string& msg);
int fail(int status, const std::string& msg);

inline const char* base_name(const char* path) {  // the file's name without its directories, for error messages
  const char* b = path;
  for (const char* c = path; *c; ++c)
    if (*c == '/') b = c + 1;
  return b;
}

#define FV_CUDA(expr)                                                                          \
  do {                                                                                         \
    cudaError_t _e = (expr);                                                                   \
    if (_e != cudaSuccess)                                                                     \
      return fv::fail(FV_ERR_CUDA, std::string(#expr) + " (" + fv::base_name(__FILE__) + ":" +  \
                                       std::to_string(__LINE__) + "): " + cudaGetErrorString(_e)); \
  } while (0)

#define FV_TRY(expr)            \
  do {                          \
    int _s = (expr);            \
    if (_s != FV_OK) return _s; \
  } while (0)

inline size_t padded(size_t dim) { return (dim + 7) / 8 * 8; }

// ---------------------------------------------------------------------------------------------
// keys.  Neighbours are ordered by f32::total_cmp on the distance, then by id
// (src/vector/mod.rs:60-64).  Mapping the float's bits to an unsigned integer that
// sorts the same way and putting the id below it turns that order into one u64 compare.
#define FV_EMPTY_KEY 0xFFFFFFFFFFFFFFFFull

__host__ __device__ __forceinline__ uint32_t order_bits(float f) {
#ifdef __CUDA_ARCH__
  uint32_t b = __float_as_uint(f);
#else
  uint32_t b;
  memcpy(&b, &f, 4);
#endif
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
__host__ __device__ __forceinline__ float order_bits_to_float(uint32_t k) {
  uint32_t b = (k & 0x80000000u) ? (k & 0x7FFFFFFFu) : ~k;
#ifdef __CUDA_ARCH__
  return __uint_as_float(b);
#else
  float f;
  memcpy(&f, &b, 4);
  return f;
#endif
}
__host__ __device__ __forceinline__ u64 make_key(float d, uint32_t id) {
  return (u64(order_bits(d)) << 32) | u64(id);
}
__host__ __device__ __forceinline__ float key_distance(u64 k) { return order_bits_to_float(uint32_t(k >> 32)); }
__host__ __device__ __forceinline__ uint32_t key_id(u64 k) { return uint32_t(k & 0xFFFFFFFFull); }

// Debug build (make EXTRA=-DFV_BOUNDS): the indices kernels gather through (probed cells, list offsets, row ids,
// graph links, vector slots, gathered operand rows) are checked against their extents before the access.  A
// violation is recorded in the translation unit's g_bounds words {count, site, index, extent} and the access is
// skipped; at the end of a search the host turns a non-zero count into FV_ERR_OVERFLOW (bounds_report_*).
// FV_BOUNDS_TU(name) goes once into every .cu with checked kernels.
#if defined(FV_BOUNDS) && defined(__CUDACC__)
static __device__ unsigned long long g_bounds[4];
__device__ __forceinline__ bool idx_ok(unsigned long long i, unsigned long long n, int site) {
  if (i < n) return true;
  if (atomicAdd(&g_bounds[0], 1ull) == 0ull) {
    g_bounds[1] = (unsigned long long)site;
    g_bounds[2] = i;
    g_bounds[3] = n;
  }
  return false;
}
#define FV_IDX_OK(i, n, site) fv::idx_ok((unsigned long long)(i), (unsigned long long)(n), site)
#define FV_BOUNDS_TU(name)                                                                                        \
  namespace fv {                                                                                                  \
  int bounds_report_##name() {                                                                                    \
    unsigned long long h[4] = {0, 0, 0, 0};                                                                       \
    if (cudaMemcpyFromSymbol(h, g_bounds, sizeof(h)) != cudaSuccess) return fail(FV_ERR_CUDA, "bounds words");    \
    if (h[0] == 0) return FV_OK;                                                                                  \
    const unsigned long long z[4] = {0, 0, 0, 0};                                                                 \
    cudaMemcpyToSymbol(g_bounds, z, sizeof(z));                                                                   \
    return fail(FV_ERR_OVERFLOW, std::string("bounds check in " #name ": ") + std::to_string(h[0]) +              \
                                     " violation(s); first at site " + std::to_string(h[1]) + ", index " +         \
                                     std::to_string(h[2]) + ", extent " + std::to_string(h[3]));                   \
  }                                                                                                               \
  }
#else
#define FV_IDX_OK(i, n, site) true
#define FV_BOUNDS_TU(name)                          \
  namespace fv {                                    \
  int bounds_report_##name() { return FV_OK; }      \
  }
#endif

#ifdef __CUDACC__
#define FV_FULL 0xFFFFFFFFu

__device__ __forceinline__ int lane_id() { return threadIdx.x & 31; }

// the one dynamic shared-memory array of every kernel
__device__ __forceinline__ unsigned char* dyn_smem() {
  extern __shared__ __align__(1024) unsigned char fv_dyn_smem[];
  return fv_dyn_smem;
}

// Sorts the first `n` keys (a power of two) of `buf` (shared memory) ascending: a bitonic network run by the whole
// block, one barrier per stage.  Called by every thread of the block.
__device__ __forceinline__ void block_sort(u64* buf, int n) {
  for (int k = 2; k <= n; k <<= 1) {
    for (int j = k >> 1; j > 0; j >>= 1) {
      for (int t = threadIdx.x; t < (n >> 1); t += blockDim.x) {
        const int i = ((t & ~(j - 1)) << 1) | (t & (j - 1));  // the lower index of pair t
        const u64 x = buf[i], y = buf[i | j];
        const bool asc = (i & k) == 0;
        if ((x > y) == asc) {
          buf[i] = y;
          buf[i | j] = x;
        }
      }
      __syncthreads();
    }
  }
}

// ---------------------------------------------------------------------------------------------
// A sorted list of L keys (ascending) owned by ONE warp, in shared or global memory.
// All 32 lanes call every function with the same arguments.
__device__ __forceinline__ void warp_list_init(u64* list, int L) {
  for (int e = lane_id(); e < L; e += 32) list[e] = FV_EMPTY_KEY;
  __syncwarp();
}

// Inserts `key` (must be < list[L-1]) and drops the last entry.  Works from the top chunk of
// 32 entries downwards so that every read sees the list as it was before the call.
__device__ __forceinline__ void warp_list_insert(u64* list, int L, u64 key) {
  const int lane = lane_id();
  for (int c = (L - 1) >> 5; c >= 0; --c) {
    const int e = (c << 5) + lane;
    const u64 cur = (e < L) ? list[e] : FV_EMPTY_KEY;
    const u64 prev = (e > 0 && e <= L) ? list[e - 1] : 0ull;
    __syncwarp();
    if (e < L) {
      u64 nv = cur;
      if (!(cur < key)) nv = (e == 0 || prev < key) ? key : prev;
      list[e] = nv;
    }
    const u64 low = __shfl_sync(FV_FULL, cur, 0);
    __syncwarp();
    if (low < key) break;
  }
}

// Offers the candidates held one per lane (key = FV_EMPTY_KEY for "none") to the list, in lane order.
// Returns the list's last key afterwards (the admission bound).
__device__ __forceinline__ u64 warp_list_offer(u64* list, int L, u64 key, u64 bound) {
  unsigned pending = __ballot_sync(FV_FULL, key < bound);
  while (pending) {
    const int src = __ffs(pending) - 1;
    pending &= pending - 1;
    const u64 k = __shfl_sync(FV_FULL, key, src);
    if (k < bound) {
      warp_list_insert(list, L, k);
      bound = list[L - 1];
    }
  }
  return bound;
}

// ---------------------------------------------------------------------------------------------
// The reference's distance arithmetic (src/kernels.rs:192-231): eight lane accumulators, each a
// chain of fused multiply-adds over every eighth element, then the fixed pairwise lane sum.
__device__ __forceinline__ float hsum8(const float* l) {
  return __fadd_rn(__fadd_rn(__fadd_rn(l[0], l[4]), __fadd_rn(l[2], l[6])),
                   __fadd_rn(__fadd_rn(l[1], l[5]), __fadd_rn(l[3], l[7])));
}

template <bool IS_L2>
__device__ __forceinline__ void dist_step8(float* acc, const float4& a0, const float4& a1, const float4& b0,
                                           const float4& b1) {
  if (IS_L2) {
    float d;
    d = __fsub_rn(a0.x, b0.x); acc[0] = __fmaf_rn(d, d, acc[0]);
    d = __fsub_rn(a0.y, b0.y); acc[1] = __fmaf_rn(d, d, acc[1]);
    d = __fsub_rn(a0.z, b0.z); acc[2] = __fmaf_rn(d, d, acc[2]);
    d = __fsub_rn(a0.w, b0.w); acc[3] = __fmaf_rn(d, d, acc[3]);
    d = __fsub_rn(a1.x, b1.x); acc[4] = __fmaf_rn(d, d, acc[4]);
    d = __fsub_rn(a1.y, b1.y); acc[5] = __fmaf_rn(d, d, acc[5]);
    d = __fsub_rn(a1.z, b1.z); acc[6] = __fmaf_rn(d, d, acc[6]);
    d = __fsub_rn(a1.w, b1.w); acc[7] = __fmaf_rn(d, d, acc[7]);
  } else {
    acc[0] = __fmaf_rn(a0.x, b0.x, acc[0]);
    acc[1] = __fmaf_rn(a0.y, b0.y, acc[1]);
    acc[2] = __fmaf_rn(a0.z, b0.z, acc[2]);
    acc[3] = __fmaf_rn(a0.w, b0.w, acc[3]);
    acc[4] = __fmaf_rn(a1.x, b1.x, acc[4]);
    acc[5] = __fmaf_rn(a1.y, b1.y, acc[5]);
    acc[6] = __fmaf_rn(a1.z, b1.z, acc[6]);
    acc[7] = __fmaf_rn(a1.w, b1.w, acc[7]);
  }
}

// Distance between `a` (shared or global, 16-byte aligned, pd floats) and row `b` (global).
template <bool IS_L2>
__device__ __forceinline__ float exact_distance(const float* __restrict__ a, const float* __restrict__ b, int pd) {
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  const float4* a4 = reinterpret_cast<const float4*>(a);
  const float4* b4 = reinterpret_cast<const float4*>(b);
#pragma unroll 4
  for (int c = 0; c < pd / 8; ++c) {
    const float4 b0 = __ldg(b4 + 2 * c), b1 = __ldg(b4 + 2 * c + 1);
    const float4 a0 = a4[2 * c], a1 = a4[2 * c + 1];
    dist_step8<IS_L2>(acc, a0, a1, b0, b1);
  }
  const float s = hsum8(acc);
  return IS_L2 ? s : -s;
}

// Exact distances to FOUR gathered rows at once, for rows fetched by id (a re-rank).  With one row per lane every
// load instruction touches 32 different rows, 16 bytes of each, and a row costs one trip to memory per unrolled group
// of loads.  Here the warp copies four rows into shared memory with asynchronous 16-byte copies (quad_issue: whole
// rows in flight at once, no registers held, coalesced 512 bytes per instruction), and while the next four are on
// their way works on the current ones as 4 rows x 8 chain lanes (quad_compute): lane (r, l) runs chain l of row r --
// elements l, l + 8, ... in order, src/kernels.rs:200-231 -- and the eight lane sums are added in the reference's
// pairwise order, so the result is bit for bit exact_distance's.  Lane i brings the id of candidate i and whether it
// has one; a quad is candidates 4 qd .. 4 qd + 3.  A stage buffer holds 4 * quad_stride(pd) floats, 16-byte aligned.
__host__ __device__ __forceinline__ int quad_stride(int pd) { return ((pd + 31) / 32) * 32 + 8; }  // = 8 mod 32: no bank conflicts

__device__ __forceinline__ void quad_issue(const float* __restrict__ rows, int pd, uint32_t id, bool valid, int qd,
                                           float* stage) {
  const int lane = lane_id();
  const int ts = quad_stride(pd), q4 = pd >> 2;
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    const uint32_t rid = __shfl_sync(FV_FULL, id, 4 * qd + r);
    const bool rv = __shfl_sync(FV_FULL, int(valid), 4 * qd + r) != 0;
    if (rv) {  // (a candidate without a row leaves its part of the stage as it is: its lanes' results are not used)
      const float4* src = reinterpret_cast<const float4*>(rows + size_t(rid) * pd);
      const uint32_t dst = uint32_t(__cvta_generic_to_shared(stage + r * ts));
      for (int c = lane; c < q4; c += 32)
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst + uint32_t(c) * 16u), "l"(src + c) : "memory");
    }
  }
  asm volatile("cp.async.commit_group;" ::: "memory");
}
// waits until at most `pending` of this thread's copy groups are still in flight (0 or 1), then lines the warp up
__device__ __forceinline__ void quad_wait(int pending) {
  if (pending) asm volatile("cp.async.wait_group 1;" ::: "memory");
  else asm volatile("cp.async.wait_group 0;" ::: "memory");
  __syncwarp();
}
// returns, in lanes 4 qd .. 4 qd + 3 of the quad that was staged, the distance of the lane's own candidate (every lane
// gets the distance of row lane & 3)
template <bool IS_L2>
__device__ __forceinline__ float quad_compute(const float* sq, int pd, const float* stage) {
  const int lane = lane_id();
  const int ts = quad_stride(pd);
  const float* b = stage + (lane >> 3) * ts + (lane & 7);
  const float* a = sq + (lane & 7);
  float acc = 0.f;
#pragma unroll 4
  for (int t = 0; t < pd; t += 8) {
    if (IS_L2) {
      const float d = __fsub_rn(a[t], b[t]);
      acc = __fmaf_rn(d, d, acc);
    } else {
      acc = __fmaf_rn(a[t], b[t], acc);
    }
  }
  // hsum8: ((l0 + l4) + (l2 + l6)) + ((l1 + l5) + (l3 + l7)); fadd commutes, so all eight lanes end with that value
  float s = __fadd_rn(acc, __shfl_xor_sync(FV_FULL, acc, 4));
  s = __fadd_rn(s, __shfl_xor_sync(FV_FULL, s, 2));
  s = __fadd_rn(s, __shfl_xor_sync(FV_FULL, s, 1));
  const float mine = __shfl_sync(FV_FULL, s, (lane & 3) * 8);
  __syncwarp();  // the stage may be refilled
  return IS_L2 ? mine : -mine;
}
// The distances of up to 32 candidates (one per lane), quads pipelined through two stage buffers.
template <bool IS_L2>
__device__ __forceinline__ float quad_distances(const float* sq, const float* __restrict__ rows, int pd, uint32_t id,
                                                bool valid, float* stage2) {
  const int lane = lane_id();
  const int qs = 4 * quad_stride(pd);
  unsigned quads = 0;  // bit qd: quad qd has a candidate
  const unsigned act = __ballot_sync(FV_FULL, valid);
  for (int qd = 0; qd < 8; ++qd)
    if ((act >> (4 * qd)) & 0xFu) quads |= 1u << qd;
  float d = INFINITY;
  int buf = 0;
  if (quads) quad_issue(rows, pd, id, valid, __ffs(quads) - 1, stage2);
  while (quads) {
    const int cur = __ffs(quads) - 1;
    quads &= quads - 1;
    if (quads) quad_issue(rows, pd, id, valid, __ffs(quads) - 1, stage2 + (buf ^ 1) * qs);
    quad_wait(quads ? 1 : 0);
    const float dv = quad_compute<IS_L2>(sq, pd, stage2 + buf * qs);
    if ((lane >> 2) == cur) d = dv;
    buf ^= 1;
  }
  return d;
}

__device__ __forceinline__ float exact_distance(int metric, const float* a, const float* b, int pd) {
  return metric == FV_L2 ? exact_distance<true>(a, b, pd) : exact_distance<false>(a, b, pd);
}
#endif  // __CUDACC__

}  // namespace fv
