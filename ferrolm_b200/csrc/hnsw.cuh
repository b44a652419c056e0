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

// search_layer (hnsw.rs:179-226) by one warp, from the entries best[0..filled) (sorted, at most ef).  `rows(c)` is the
// link block of node c on the searched layer (count, then at most `width` ids; width + 1 words are readable).  The
// reference's pair of heaps is ONE sorted list of ef entries with an "expanded" bit each: a candidate that has been
// evicted from `best` can only be popped after every entry of `best` has been expanded, and then it trips the stop
// test (hnsw.rs:203-205) unless its distance ties the current worst exactly -- see TIED_CAP.  Neighbours of the
// expanded node are evaluated one per lane and offered to the list in stored order, so the admission test
// (hnsw.rs:214) sees the same evolving bound as the sequential loop.  The visited set is an exact open-addressing
// hash table of 2^log2slots words owned by the warp; a search that fills more than half of it stops with `over`.
// On return best[0..filled) is the reference's result, nearest first; n_dist and n_exp have grown by the distances
// evaluated and the nodes expanded.
template <bool IS_L2, class Rows>
__device__ __forceinline__ void beam_search(const float* __restrict__ data, int pd, size_t n, Rows rows, int width,
                                            const float* sq, u64* best, int ef, uint32_t* tied, uint32_t* table,
                                            int log2slots, int& filled, bool& over, bool& tie_lost,
                                            unsigned long long& n_dist, unsigned long long& n_exp) {
  const int lane = lane_id();
  const int slots = 1 << log2slots;
  for (int s = lane * 4; s < slots; s += 128) *reinterpret_cast<uint4*>(table + s) = make_uint4(~0u, ~0u, ~0u, ~0u);
  __syncwarp();
  for (int e = lane; e < filled; e += 32) {
    const u64 b = best[e] & ~1ull;
    best[e] = b;
    visit(table, log2slots, beam_id(b));
  }
  __syncwarp();
  int visited = filled, cursor = 0, ntied = 0;
  over = false;
  for (;;) {
    int pos = -1;
    for (int e0 = cursor & ~31; e0 < filled; e0 += 32) {
      const int e = e0 + lane;
      const bool open = e >= cursor && e < filled && !(best[e] & 1ull);
      const unsigned mk = __ballot_sync(FV_FULL, open);
      if (mk) {
        pos = e0 + __ffs(mk) - 1;
        break;
      }
    }
    uint32_t c = 0;
    if (ntied > 0) {
      uint32_t tmin = 0xFFFFFFFFu;
      for (int t = lane; t < ntied; t += 32) tmin = min(tmin, tied[t]);
      for (int o = 16; o > 0; o >>= 1) tmin = min(tmin, __shfl_xor_sync(FV_FULL, tmin, o));
      const u64 tkey = (best[ef - 1] & 0xFFFFFFFF00000000ull) | (u64(tmin) << 1);
      if (pos < 0 || tkey < best[pos]) {
        __syncwarp();
        for (int t = lane; t < ntied; t += 32)
          if (tied[t] == tmin) tied[t] = tied[ntied - 1];
        __syncwarp();
        ntied--;
        pos = -2;
        c = tmin;
      }
    }
    if (pos == -1) break;
    if (pos >= 0) {
      const u64 ck = best[pos];
      __syncwarp();
      if (lane == 0) best[pos] = ck | 1ull;
      __syncwarp();
      cursor = pos + 1;
      c = beam_id(ck);
    }
    if (!FV_IDX_OK(c, n, 1)) break;
    const uint32_t* row = rows(c);
    // the first 32 links are requested together with the count: one round trip, not two
    // (rows of the searched graph are not written while a search runs: the non-coherent path is safe)
    const uint32_t x_first = lane < width ? __ldg(row + 1 + lane) : 0u;
    const int cnt = min(int(__ldg(row)), width);
    n_exp += 1;
    for (int c0 = 0; c0 < cnt; c0 += 32) {
      const int i = c0 + lane;
      u64 key = FV_EMPTY_KEY;
      bool fresh = false;
      uint32_t x = 0;
      if (i < cnt) {
        x = c0 == 0 ? x_first : __ldg(row + 1 + i);
        fresh = FV_IDX_OK(x, n, 2) && visit(table, log2slots, x);
      }
      const int nfresh = __popc(__ballot_sync(FV_FULL, fresh));
      visited += nfresh;
      n_dist += nfresh;
      if (fresh) {
        // all lines of the row are requested before the dependent FMA chains start, so the gather costs one
        // memory round trip instead of one per unrolled group of loads
        const char* rowp = reinterpret_cast<const char*>(data + size_t(x) * pd);
        for (int b = 0; b < pd * 4; b += 128) asm volatile("prefetch.global.L1 [%0];" ::"l"(rowp + b));
        key = beam_key(exact_distance<IS_L2>(sq, data + size_t(x) * pd, pd), x);
      }
      // offered in stored order: admitted while the list is not full, or on a strictly smaller distance
      u64 bound = best[ef - 1];
      unsigned pending = __ballot_sync(FV_FULL, fresh);
      while (pending) {
        const int src = __ffs(pending) - 1;
        pending &= pending - 1;
        const u64 kk = __shfl_sync(FV_FULL, key, src);
        if ((kk >> 32) < (bound >> 32)) {
          int below = 0;
          for (int e0 = 0; e0 < filled; e0 += 32) {
            const int e = e0 + lane;
            below += __popc(__ballot_sync(FV_FULL, e < filled && best[e] < kk));
          }
          __syncwarp();
          const bool was_full = filled == ef;
          warp_list_insert(best, ef, kk);
          if (filled < ef) filled++;
          if (below < cursor) cursor = below;
          const u64 pushed = bound;
          bound = best[ef - 1];
          if (was_full) {
            if ((bound >> 32) < (pushed >> 32)) {
              ntied = 0;
            } else if (!(pushed & 1ull)) {
              if (ntied < TIED_CAP) {
                __syncwarp();
                if (lane == 0) tied[ntied] = beam_id(pushed);
                __syncwarp();
                ntied++;
              } else {
                tie_lost = true;
              }
            }
          }
        }
      }
    }
    if (visited > (slots >> 1)) {
      over = true;
      break;
    }
  }
  __syncwarp();
}
#endif

}  // namespace fv
