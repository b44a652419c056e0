// fv_merge_topk_static_dev: the shard merge for callers that must not allocate.
//
// Some hosts of this library run where device allocation is off the table: a latency-critical
// serving loop that has handed all free HBM to its own arena, a component of a framework whose
// allocator owns the device and forbids cudaMalloc beside it, or code that runs after the process
// has fixed its memory budget.  For them every other entry point is unusable, because each one may
// grow the context's scratch arena with cudaMalloc.  This file gives them one call that never
// does: the intermediate keys of the merge live in a fixed array that is part of the library
// image itself.
//
// The price is a size limit and a shared buffer:
//   - nq * k_out may not exceed FV_STATIC_MERGE_MAX_KEYS (2 MiB of keys); larger calls are refused;
//   - every GPU that loads the library carries the array until the process exits;
//   - all calls on one GPU use the same array, which keeps whatever the previous call left.  Nothing
//     in it has to start at zero (each call overwrites the part it reads), but two calls that overlap
//     on the GPU -- different streams, or different threads -- race on it.  Serialise them.
//
// The call is synchronous: it launches two kernels on the caller's stream and waits for that stream,
// so it is refused (FV_ERR_UNSUPPORTED) on a stream that is being captured, and it may not be made
// from a host-function callback (no CUDA call may).
//
// The first call on each device looks up the array's device address (cudaGetSymbolAddress, with that
// device current).  With the CUDA runtime's lazy module loading that first call is also when the
// array and this file's kernels are placed on the device, so make it once at start-up: before any
// stream capture begins, and while the device still has a few MiB that the process has not claimed.
#include <climits>

#include "internal.h"

#define FV_STATIC_MERGE_MAX_KEYS (1u << 18)

namespace fv {

// The scratch itself.  In host code this name is only a handle for the runtime, not a device address.
static __device__ __align__(256) u64 g_static_merge_keys[FV_STATIC_MERGE_MAX_KEYS];

// One warp per query: the k_out best (distance, id) of nparts blocks of k_in candidates, as keys.
__global__ void merge_static_kernel(const fv_neighbor* __restrict__ parts, const uint32_t* __restrict__ part_counts,
                                    int nparts, size_t nq, int k_in, int k_out, u64* __restrict__ keys) {
  unsigned char* smem_raw = dyn_smem();
  const int w = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const size_t q = size_t(blockIdx.x) * (blockDim.x >> 5) + w;
  if (q >= nq) return;
  u64* list = reinterpret_cast<u64*>(smem_raw) + size_t(w) * k_out;
  warp_list_init(list, k_out);
  u64 bound = FV_EMPTY_KEY;
  for (int p = 0; p < nparts; ++p) {
    const int cnt = part_counts ? int(min(part_counts[size_t(p) * nq + q], uint32_t(k_in))) : k_in;
    const fv_neighbor* src = parts + (size_t(p) * nq + q) * size_t(k_in);
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
  for (int e = lane; e < k_out; e += 32) keys[q * size_t(k_out) + e] = list[e];
}

__global__ void static_keys_to_neighbors_kernel(const u64* __restrict__ keys, size_t nq, int k,
                                                fv_neighbor* __restrict__ out, uint32_t* __restrict__ counts) {
  const size_t q = blockIdx.x * size_t(blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (q >= nq) return;
  int cnt = 0;
  for (int e0 = 0; e0 < k; e0 += 32) {
    const int e = e0 + lane;
    const u64 key = e < k ? keys[q * size_t(k) + e] : FV_EMPTY_KEY;
    if (e < k) {
      fv_neighbor nb;
      nb.id = key == FV_EMPTY_KEY ? 0xFFFFFFFFu : key_id(key);
      nb.distance = key == FV_EMPTY_KEY ? INFINITY : key_distance(key);
      out[q * size_t(k) + e] = nb;
    }
    cnt += __popc(__ballot_sync(FV_FULL, key != FV_EMPTY_KEY));
  }
  if (lane == 0 && counts) counts[q] = uint32_t(cnt);
}

// per-device address of the scratch, looked up once
static u64* g_scratch_addr[64] = {};

static int static_scratch(int device, u64** out) {
  if (device < 0 || device >= 64) return fail(FV_ERR_ARG, "device index out of range");
  if (!g_scratch_addr[device]) {
    void* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&p, g_static_merge_keys);  // the device is current here
    if (e != cudaSuccess || !p)
      return fail(FV_ERR_CUDA, std::string("cudaGetSymbolAddress(static merge scratch): ") + cudaGetErrorString(e));
    g_scratch_addr[device] = static_cast<u64*>(p);
  }
  *out = g_scratch_addr[device];
  return FV_OK;
}

}  // namespace fv

extern "C" int fv_merge_topk_static_dev(int device, void* stream, const fv_neighbor* d_parts,
                                        const uint32_t* d_part_counts, size_t nparts, size_t nq, size_t k_in,
                                        size_t k_out, fv_neighbor* d_out, uint32_t* d_counts) {
  if (!d_parts || !d_out || nparts == 0 || k_in == 0 || k_out == 0)
    return fv::fail(FV_ERR_ARG, "fv_merge_topk_static_dev: bad argument");
  if (nq == 0) return FV_OK;
  if (nparts > size_t(INT_MAX) || k_in > size_t(INT_MAX))
    return fv::fail(FV_ERR_UNSUPPORTED, "fv_merge_topk_static_dev: nparts and k_in must fit a 32-bit int");
  if (k_out > 1024) return fv::fail(FV_ERR_UNSUPPORTED, "fv_merge_topk_static_dev: k_out above 1024 is not supported");
  if (nq > FV_STATIC_MERGE_MAX_KEYS / k_out)
    return fv::fail(FV_ERR_UNSUPPORTED,
                    "fv_merge_topk_static_dev: nq * k_out = " + std::to_string(nq * k_out) + " exceeds the static scratch of " +
                        std::to_string(FV_STATIC_MERGE_MAX_KEYS) + " keys; use fv_merge_topk_dev");
  fv::DeviceGuard g(device);
  if (!g.ok) return fv::fail(FV_ERR_CUDA, "cudaSetDevice failed");
  u64* keys = nullptr;
  FV_TRY(fv::static_scratch(device, &keys));
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
  if (cudaStreamIsCapturing(s, &cap) != cudaSuccess) {
    (void)cudaGetLastError();
    return fv::fail(FV_ERR_CUDA, "fv_merge_topk_static_dev: cudaStreamIsCapturing failed");
  }
  if (cap != cudaStreamCaptureStatusNone)
    return fv::fail(FV_ERR_UNSUPPORTED, "fv_merge_topk_static_dev waits for its stream and cannot run on a capturing stream");
  // 4 warps per block; k_out <= 1024 keeps the lists within the default 48 KB of shared memory
  int wpb = 4;
  while (wpb > 1 && size_t(wpb) * k_out * 8 > 48 * 1024) wpb >>= 1;
  const size_t smem = size_t(wpb) * k_out * 8;
  fv::merge_static_kernel<<<unsigned((nq + wpb - 1) / wpb), wpb * 32, smem, s>>>(d_parts, d_part_counts, int(nparts), nq,
                                                                                 int(k_in), int(k_out), keys);
  FV_CUDA(cudaGetLastError());
  fv::static_keys_to_neighbors_kernel<<<unsigned((nq + 7) / 8), 256, 0, s>>>(keys, nq, int(k_out), d_out, d_counts);
  FV_CUDA(cudaGetLastError());
  FV_CUDA(cudaStreamSynchronize(s));
  return FV_OK;
}
