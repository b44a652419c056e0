// What the Hnsw search (hnsw.cu) and the construction on the GPU (hnsw_build.cu) share: the index object, the
// per-warp visited table and the beam's entry format.
#pragma once

#include <memory>
#include <vector>

#include "internal.h"

struct fv_hnsw {
  fv_ctx* ctx = nullptr;
  ~fv_hnsw() {
    d_data.release(); d_links0.release(); d_upper_off.release(); d_upper_flat.release();
    if (ctx) fv::ctx_release(ctx);
  }
  int metric = 0;
  uint32_t dim = 0, pd = 0;
  size_t m = 0, m0 = 0;
  uint32_t ep = 0;
  size_t top = 0;
  // host copies (the file's content)
  std::vector<float> data;
  std::vector<uint8_t> levels;
  std::vector<uint32_t> links0;
  std::vector<std::vector<uint32_t>> upper;  // per node: concatenated (count, ids...) per layer, fixed stride m+1
  // device copies
  DevBuf d_data, d_links0, d_upper_off, d_upper_flat;
  size_t n() const { return levels.size(); }
};

namespace fv {

// An index with its rows padded, its levels drawn (hnsw.rs:88-94) and every link list empty; node 0 is the entry.
int hnsw_new(fv_ctx* ctx, int metric, uint32_t dim, const float* vectors, size_t n, const fv_hnsw_params* p,
             std::unique_ptr<fv_hnsw>& out);
// Copies the host graph to the device in the search kernel's layout; the rows too unless they are there already.
int upload_graph(fv_hnsw* h, bool with_data = true);

// The reference keeps two heaps: an entry pushed out of the result heap stays in the candidate heap, and because its
// loop stops only on a STRICTLY larger distance (hnsw.rs:195-197), such an entry is still expanded if its distance
// equals the worst kept distance when its turn comes.  The beam is one list, so the unexpanded entries it pushes out
// while their distance equals the new worst distance are remembered in a side list of this many ids (all share that
// distance) and take their turn in (distance, id) order; the list is dropped as soon as the worst distance goes down.
static constexpr int TIED_CAP = 64;

#ifdef __CUDACC__
__device__ __forceinline__ uint32_t hash_slot(uint32_t x, int log2slots) { return (x * 2654435761u) >> (32 - log2slots); }

// true if x was not in the table (and is now)
__device__ __forceinline__ bool visit(uint32_t* table, int log2slots, uint32_t x) {
  const uint32_t mask = (1u << log2slots) - 1u;
  uint32_t s = hash_slot(x, log2slots);
  for (uint32_t probe = 0; probe <= mask; ++probe) {
    const uint32_t old = atomicCAS(table + s, 0xFFFFFFFFu, x);
    if (old == 0xFFFFFFFFu) return true;
    if (old == x) return false;
    s = (s + 1) & mask;
  }
  return false;  // full table: cannot happen below the half-full limit
}

// list entry: order bits of the distance (32) | id (31) | expanded (1)
__device__ __forceinline__ u64 beam_key(float d, uint32_t id) { return (u64(order_bits(d)) << 32) | (u64(id) << 1); }
__device__ __forceinline__ uint32_t beam_id(u64 key) { return uint32_t(key >> 1) & 0x7FFFFFFFu; }
__device__ __forceinline__ float beam_distance(u64 key) { return order_bits_to_float(uint32_t(key >> 32)); }
#endif

}  // namespace fv
