// Hnsw (src/vector/hnsw.rs): batched search on the GPU, one warp per query.
//
// Device layout: data n x pd f32; links0 n x (m0+1) u32 (count, then ids) exactly as the
// reference stores layer 0 (hnsw.rs:50-51, :154-157); the upper layers as one flat u32 array in
// the order of the FLHNSW01 file (per node, per layer: count, ids) with a per-node start offset.
//
// Search of one query (hnsw.rs:323-351): greedy descent on the upper layers, then the best-first
// beam of search_layer (hnsw.rs:179-226) kept as ONE sorted list of ef entries with an "expanded"
// bit per entry.  That is the reference's pair of heaps: a candidate that has been evicted from
// `best` can only be popped after every entry of `best` has been expanded, and then it trips the
// stop test (hnsw.rs:203-205) unless its distance ties the current worst exactly.  Neighbours of
// the expanded node are evaluated one per lane and offered to the list in stored order, so the
// admission test (hnsw.rs:214) sees the same evolving bound as the sequential loop.
//
// The visited set is an exact open-addressing hash table per warp (shared memory when it fits,
// global memory otherwise).  A query that fills more than half of it stops with an overflow mark
// and is re-run by the host with a table four times larger.
#include <algorithm>
#include <atomic>
#include <cmath>
#include <cstdlib>
#include <memory>
#include <mutex>
#include <thread>

#include "hnsw.cuh"

FV_BOUNDS_TU(hnsw)

namespace fv {

struct HnswDev {
  const float* data;
  const uint32_t* links0;
  const uint32_t* upper_off;   // n + 1 offsets into upper_flat
  const uint32_t* upper_flat;
  int pd, m0, metric, top;
  uint32_t ep;
  size_t n;
};

template <bool IS_L2>
__global__ void __launch_bounds__(256, 4)
    hnsw_search_kernel(HnswDev g, const float* __restrict__ queries, const uint32_t* __restrict__ qids, size_t nq, int k,
                       int ef, int log2slots, uint32_t* __restrict__ global_tables, u64* __restrict__ out_keys,
                       uint32_t* __restrict__ overflow, unsigned long long* __restrict__ work,
                       unsigned int* __restrict__ next_query) {
  unsigned char* smem_raw = dyn_smem();
  const int W = blockDim.x >> 5, w = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int slots = 1 << log2slots;
  const size_t list_bytes = ((size_t(ef) * 8 + 15) & ~size_t(15)) + TIED_CAP * 4;
  const size_t per_warp = size_t(g.pd) * 4 + list_bytes + (global_tables ? 0 : size_t(slots) * 4);
  unsigned char* mine = smem_raw + size_t(w) * per_warp;
  float* sq = reinterpret_cast<float*>(mine);
  u64* best = reinterpret_cast<u64*>(mine + size_t(g.pd) * 4);
  uint32_t* tied = reinterpret_cast<uint32_t*>(mine + size_t(g.pd) * 4 + list_bytes - TIED_CAP * 4);
  const size_t gw = size_t(blockIdx.x) * W + w;
  uint32_t* table = global_tables ? global_tables + gw * size_t(slots)
                                  : reinterpret_cast<uint32_t*>(mine + size_t(g.pd) * 4 + list_bytes);
  unsigned long long n_dist = 0, n_exp = 0, n_tie_lost = 0;

  // Queries are drawn from a counter (zero at launch): a batch gives every resident warp two or three of them and
  // they differ in length, so a fixed deal leaves the warps that drew three long ones running alone at the end.
  for (;;) {
    size_t qi = 0;
    if (lane == 0) qi = atomicAdd(next_query, 1u);
    qi = __shfl_sync(FV_FULL, qi, 0);
    if (qi >= nq) break;
    const size_t qsrc = qids ? size_t(qids[qi]) : qi;
    const unsigned long long n_dist0 = n_dist, n_exp0 = n_exp;  // a query that overflows its table is re-run: its work counts once
    for (int c = lane; c < g.pd; c += 32) sq[c] = queries[qsrc * size_t(g.pd) + c];
    for (int s = lane * 4; s < slots; s += 128) *reinterpret_cast<uint4*>(table + s) = make_uint4(~0u, ~0u, ~0u, ~0u);
    warp_list_init(best, ef);

    // entry point and greedy descent (hnsw.rs:329-347)
    uint32_t cur = g.ep;
    float curd = exact_distance<IS_L2>(sq, g.data + size_t(cur) * g.pd, g.pd);
    n_dist += 1;
    for (int layer = g.top; layer >= 1; --layer) {
      bool changed = true;
      while (changed) {
        changed = false;
        size_t p = g.upper_off[cur];
        for (int s = 1; s < layer; ++s) p += 1 + g.upper_flat[p];
        const int cnt = int(g.upper_flat[p]);
        n_exp += 1;
        for (int c0 = 0; c0 < cnt; c0 += 32) {
          const int i = c0 + lane;
          uint32_t x = 0;
          float d = INFINITY;
          if (i < cnt) {
            x = g.upper_flat[p + 1 + i];
            const char* rowp = reinterpret_cast<const char*>(g.data + size_t(x) * g.pd);
            for (int b = 0; b < g.pd * 4; b += 128) asm volatile("prefetch.global.L1 [%0];" ::"l"(rowp + b));
            d = exact_distance<IS_L2>(sq, g.data + size_t(x) * g.pd, g.pd);
          }
          n_dist += __popc(__ballot_sync(FV_FULL, i < cnt));
          // first minimum of the chunk, taken only if strictly below the current distance
          const unsigned better = __ballot_sync(FV_FULL, i < cnt && d < curd);
          if (better) {
            float md = d < curd ? d : INFINITY;
            for (int o = 16; o > 0; o >>= 1) md = fminf(md, __shfl_xor_sync(FV_FULL, md, o));
            const unsigned at = __ballot_sync(FV_FULL, i < cnt && d == md);
            const int src = __ffs(at) - 1;
            cur = __shfl_sync(FV_FULL, x, src);
            curd = md;
            changed = true;
          }
        }
      }
    }

    // layer 0 (hnsw.rs:179-226 with ef = max(ef, k)).  This is beam_search of hnsw.cuh (which the graph construction
    // uses on every layer) written out for one entry point and layer 0's fixed-stride rows: through the shared
    // function this kernel measured 2.3 % slower (7.78 against 7.61 ms per 10,000 queries on 1M nodes).
    warp_list_insert(best, ef, beam_key(curd, cur));
    if (lane == 0) visit(table, log2slots, cur);
    __syncwarp();
    int filled = 1;          // entries of `best` in use
    int visited = 1;
    bool over = false, tie_lost = false;
    int cursor = 0;          // first entry that may be unexpanded
    int ntied = 0;           // pushed-out entries still tied with the worst kept distance
    for (;;) {
      // next unexpanded entry at or after `cursor`
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
        // the smallest id among the tied entries; it goes first if the beam has nothing open or only a larger key
        uint32_t tmin = 0xFFFFFFFFu;
        for (int t = lane; t < ntied; t += 32) tmin = min(tmin, tied[t]);
        for (int o = 16; o > 0; o >>= 1) tmin = min(tmin, __shfl_xor_sync(FV_FULL, tmin, o));
        const u64 tkey = (best[ef - 1] & 0xFFFFFFFF00000000ull) | (u64(tmin) << 1);
        if (pos < 0 || tkey < best[pos]) {
          __syncwarp();
          for (int t = lane; t < ntied; t += 32)
            if (tied[t] == tmin) tied[t] = tied[ntied - 1];  // ids are unique: one match
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
        c = uint32_t(ck >> 1) & 0x7FFFFFFFu;
      }
      if (!FV_IDX_OK(c, g.n, 1)) break;
      const uint32_t* row = g.links0 + size_t(c) * (g.m0 + 1);
      // the first 32 links are requested together with the count: one round trip, not two
      const uint32_t x_first = lane < g.m0 ? __ldg(row + 1 + lane) : 0u;
      const int cnt = int(__ldg(row));
      n_exp += 1;
      for (int c0 = 0; c0 < cnt; c0 += 32) {
        const int i = c0 + lane;
        u64 key = FV_EMPTY_KEY;
        bool fresh = false;
        uint32_t x = 0;
        if (i < cnt) {
          x = c0 == 0 ? x_first : row[1 + i];
          fresh = FV_IDX_OK(x, g.n, 2) && visit(table, log2slots, x);
        }
        const int nfresh = __popc(__ballot_sync(FV_FULL, fresh));
        visited += nfresh;
        n_dist += nfresh;
        if (fresh) {
          // all lines of the row are requested before the dependent FMA chains start, so the gather costs one
          // memory round trip instead of one per unrolled group of loads
          const char* rowp = reinterpret_cast<const char*>(g.data + size_t(x) * g.pd);
          for (int b = 0; b < g.pd * 4; b += 128) asm volatile("prefetch.global.L1 [%0];" ::"l"(rowp + b));
          key = beam_key(exact_distance<IS_L2>(sq, g.data + size_t(x) * g.pd, g.pd), x);
        }
        // offer in stored order: admitted while the list is not full, or on a strictly smaller distance
        u64 bound = best[ef - 1];
        unsigned pending = __ballot_sync(FV_FULL, fresh);
        while (pending) {
          const int src = __ffs(pending) - 1;
          pending &= pending - 1;
          const u64 kk = __shfl_sync(FV_FULL, key, src);
          if ((kk >> 32) < (bound >> 32)) {
            // position of the new entry = number of entries below it
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
            const u64 pushed = bound;  // the entry that fell off the end, if the beam was full
            bound = best[ef - 1];
            if (was_full) {
              if ((bound >> 32) < (pushed >> 32)) {
                ntied = 0;  // the worst distance went down: nothing pushed out so far can tie with it any more
              } else if (!(pushed & 1ull)) {
                if (ntied < TIED_CAP) {
                  __syncwarp();
                  if (lane == 0) tied[ntied] = uint32_t(pushed >> 1) & 0x7FFFFFFFu;
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
    if (tie_lost && !over) n_tie_lost += 1;
    if (over) {
      if (lane == 0) overflow[qi] = 1;
      n_dist = n_dist0;
      n_exp = n_exp0;
    } else {
      if (lane == 0) overflow[qi] = 0;
      for (int e = lane; e < k; e += 32) {
        u64 v = FV_EMPTY_KEY;
        if (e < filled) {
          const u64 b = best[e];
          v = (b & 0xFFFFFFFF00000000ull) | u64(uint32_t(b >> 1) & 0x7FFFFFFFu);
        }
        out_keys[qsrc * size_t(k) + e] = v;
      }
    }
    __syncwarp();
  }
  if (work && lane == 0) {
    atomicAdd(work, n_dist);
    atomicAdd(work + 1, n_exp);
    if (n_tie_lost) atomicAdd(work + 2, n_tie_lost);
  }
}

// ------------------------------------------------------------------------------------------------
// host side distances for construction (src/kernels.rs:200-231; same chains as the device code)
static inline float h_hsum8(const float* l) {
  return ((l[0] + l[4]) + (l[2] + l[6])) + ((l[1] + l[5]) + (l[3] + l[7]));
}
static inline float h_distance(int metric, const float* a, const float* b, size_t n) {
  float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  if (metric == FV_L2) {
    for (size_t i = 0; i + 8 <= n; i += 8)
      for (int l = 0; l < 8; l++) {
        const float d = a[i + l] - b[i + l];
        acc[l] = __builtin_fmaf(d, d, acc[l]);
      }
    return h_hsum8(acc);
  }
  for (size_t i = 0; i + 8 <= n; i += 8)
    for (int l = 0; l < 8; l++) acc[l] = __builtin_fmaf(a[i + l], b[i + l], acc[l]);
  return -h_hsum8(acc);
}

struct HNb {
  uint32_t id;
  float d;
};
static inline bool h_less(const HNb& a, const HNb& b) {
  const uint32_t ka = order_bits(a.d), kb = order_bits(b.d);
  return ka != kb ? ka < kb : a.id < b.id;
}

}  // namespace fv

namespace fv {

// upper[node] holds `level` blocks of (m + 1) u32: count then ids.
static inline uint32_t* upper_block(fv_hnsw* h, uint32_t id, size_t layer) { return &h->upper[id][(layer - 1) * (h->m + 1)]; }

static void flatten_upper(const fv_hnsw* h, std::vector<uint32_t>& off, std::vector<uint32_t>& flat) {
  const size_t n = h->n();
  off.assign(n + 1, 0);
  flat.clear();
  for (size_t i = 0; i < n; i++) {
    off[i] = uint32_t(flat.size());
    for (size_t l = 0; l < h->levels[i]; l++) {
      const uint32_t* b = &h->upper[i][l * (h->m + 1)];
      flat.push_back(b[0]);
      flat.insert(flat.end(), b + 1, b + 1 + b[0]);
    }
  }
  off[n] = uint32_t(flat.size());
}

int upload_graph(fv_hnsw* h, bool with_data) {
  fv_ctx* ctx = h->ctx;
  std::vector<uint32_t> off, flat;
  flatten_upper(h, off, flat);
  if (with_data) FV_TRY(h->d_data.reserve(h->data.size() * 4 + 16));
  FV_TRY(h->d_links0.reserve(h->links0.size() * 4 + 16));
  FV_TRY(h->d_upper_off.reserve(off.size() * 4 + 16));
  FV_TRY(h->d_upper_flat.reserve(flat.size() * 4 + 16));
  if (with_data)
    FV_CUDA(cudaMemcpyAsync(h->d_data.p, h->data.data(), h->data.size() * 4, cudaMemcpyHostToDevice, ctx->stream));
  FV_CUDA(cudaMemcpyAsync(h->d_links0.p, h->links0.data(), h->links0.size() * 4, cudaMemcpyHostToDevice, ctx->stream));
  FV_CUDA(cudaMemcpyAsync(h->d_upper_off.p, off.data(), off.size() * 4, cudaMemcpyHostToDevice, ctx->stream));
  if (!flat.empty())
    FV_CUDA(cudaMemcpyAsync(h->d_upper_flat.p, flat.data(), flat.size() * 4, cudaMemcpyHostToDevice, ctx->stream));
  FV_CUDA(cudaStreamSynchronize(ctx->stream));
  return FV_OK;
}

// ---- construction on the host cores (hnsw.rs:85-129, :230-320)
struct Builder {
  fv_hnsw* h;
  std::unique_ptr<std::mutex[]> locks;
  std::mutex entry_lock;
  const float* vec(uint32_t id) const { return &h->data[size_t(id) * h->pd]; }
  float dist(const float* q, uint32_t id) const { return h_distance(h->metric, q, vec(id), h->pd); }

  void neighbors(uint32_t id, size_t layer, bool locked, std::vector<uint32_t>& out) {
    out.clear();
    std::unique_lock<std::mutex> g;
    if (locked) g = std::unique_lock<std::mutex>(locks[id]);
    const uint32_t* b = layer == 0 ? &h->links0[size_t(id) * (h->m0 + 1)] : upper_block(h, id, layer);
    out.assign(b + 1, b + 1 + b[0]);
  }
  void set_neighbors(uint32_t id, size_t layer, const std::vector<uint32_t>& list) {
    uint32_t* b = layer == 0 ? &h->links0[size_t(id) * (h->m0 + 1)] : upper_block(h, id, layer);
    for (size_t i = 0; i < list.size(); i++) b[1 + i] = list[i];
    b[0] = uint32_t(list.size());
  }

  struct Visited {
    std::vector<uint32_t> v;
    uint32_t stamp = 0;
  };

  std::vector<HNb> search_layer(const float* q, const std::vector<HNb>& entry, size_t ef, size_t layer, Visited& vs) {
    if (vs.v.size() < h->n()) {
      vs.v.assign(h->n(), 0);
      vs.stamp = 0;
    }
    if (++vs.stamp == 0) {
      std::fill(vs.v.begin(), vs.v.end(), 0);
      vs.stamp = 1;
    }
    const uint32_t stamp = vs.stamp;
    auto gt = [](const HNb& a, const HNb& b) { return h_less(b, a); };
    std::vector<HNb> cand, best;  // cand: min-heap, best: max-heap
    for (const HNb& e : entry) {
      vs.v[e.id] = stamp;
      cand.push_back(e);
      std::push_heap(cand.begin(), cand.end(), gt);
      best.push_back(e);
      std::push_heap(best.begin(), best.end(), h_less);
    }
    while (best.size() > ef) {
      std::pop_heap(best.begin(), best.end(), h_less);
      best.pop_back();
    }
    std::vector<uint32_t> nb;
    while (!cand.empty()) {
      std::pop_heap(cand.begin(), cand.end(), gt);
      const HNb c = cand.back();
      cand.pop_back();
      if (best.size() >= ef && c.d > best.front().d) break;
      neighbors(c.id, layer, true, nb);
      for (uint32_t x : nb) {
        if (vs.v[x] == stamp) continue;
        vs.v[x] = stamp;
        const float d = dist(q, x);
        if (best.size() < ef || d < best.front().d) {
          const HNb nn{x, d};
          cand.push_back(nn);
          std::push_heap(cand.begin(), cand.end(), gt);
          best.push_back(nn);
          std::push_heap(best.begin(), best.end(), h_less);
          if (best.size() > ef) {
            std::pop_heap(best.begin(), best.end(), h_less);
            best.pop_back();
          }
        }
      }
    }
    std::sort_heap(best.begin(), best.end(), h_less);
    return best;
  }

  std::vector<uint32_t> select(const std::vector<HNb>& cands, size_t mm) const {
    std::vector<uint32_t> out;
    for (const HNb& c : cands) {
      if (out.size() >= mm) break;
      const float* cv = vec(c.id);
      bool keep = true;
      for (uint32_t s : out)
        if (!(h_distance(h->metric, cv, vec(s), h->pd) > c.d)) {
          keep = false;
          break;
        }
      if (keep) out.push_back(c.id);
    }
    return out;
  }

  void add_links(uint32_t id, size_t layer, const std::vector<uint32_t>& nw, size_t cap) {
    std::lock_guard<std::mutex> g(locks[id]);
    std::vector<uint32_t> list;
    neighbors(id, layer, false, list);
    const size_t before = list.size();
    for (uint32_t x : nw)
      if (x != id && std::find(list.begin(), list.end(), x) == list.end()) list.push_back(x);
    if (list.size() == before) return;
    if (list.size() > cap) {
      std::vector<HNb> c;
      for (uint32_t x : list) c.push_back({x, h_distance(h->metric, vec(id), vec(x), h->pd)});
      std::sort(c.begin(), c.end(), h_less);
      list = select(c, cap);
    }
    set_neighbors(id, layer, list);
  }

  void insert(uint32_t id, size_t ef, Visited& vs) {
    std::vector<float> q(vec(id), vec(id) + h->pd);
    const size_t level = h->levels[id];
    uint32_t e0;
    size_t tp;
    {
      std::lock_guard<std::mutex> g(entry_lock);
      e0 = h->ep;
      tp = h->top;
    }
    HNb cur{e0, dist(q.data(), e0)};
    std::vector<uint32_t> nb;
    for (size_t layer = tp; layer > level; layer--) {
      bool changed = true;
      while (changed) {
        changed = false;
        neighbors(cur.id, layer, true, nb);
        for (uint32_t x : nb) {
          const float d = dist(q.data(), x);
          if (d < cur.d) {
            cur = {x, d};
            changed = true;
          }
        }
      }
    }
    std::vector<HNb> entry{cur};
    for (size_t layer = std::min(level, tp) + 1; layer-- > 0;) {
      auto found = search_layer(q.data(), entry, ef, layer, vs);
      const size_t cap = layer == 0 ? h->m0 : h->m;
      const auto chosen = select(found, cap);
      add_links(id, layer, chosen, cap);
      const std::vector<uint32_t> me{id};
      for (uint32_t x : chosen) add_links(x, layer, me, cap);
      entry = std::move(found);
    }
    if (level > tp) {
      std::lock_guard<std::mutex> g(entry_lock);
      if (level > h->top) {
        h->ep = id;
        h->top = level;
      }
    }
  }
};

// scratch slots: 0 padded queries, 1 keys, 5 overflow flags, 6 retry ids, 7 global tables
static int hnsw_search_dev(fv_hnsw* h, const float* d_queries, size_t nq, size_t k, size_t ef_in, fv_neighbor* d_out,
                           uint32_t* d_counts) {
  fv_ctx* ctx = h->ctx;
  if (k == 0) return fail(FV_ERR_ARG, "k must be at least 1");
  if (nq == 0) return FV_OK;
  ctx->stats = fv_stats{};
  const size_t n = h->n();
  FV_TRY(ctx->scratch[1].reserve(nq * k * sizeof(u64)));
  u64* keys = ctx->scratch[1].as<u64>();
  if (n == 0) {  // hnsw.rs:324-326: an empty index finds nothing
    FV_CUDA(cudaMemsetAsync(keys, 0xFF, nq * k * sizeof(u64), ctx->stream));
    FV_TRY(keys_to_neighbors(ctx, keys, nq, int(k), int(k), d_out, d_counts));
    FV_CUDA(cudaStreamSynchronize(ctx->stream));
    return FV_OK;
  }
  const size_t ef = std::max(ef_in, k);
  if (ef > 4096) return fail(FV_ERR_UNSUPPORTED, "ef above 4096 is not supported");
  if (n > 0x7FFFFFFFull) return fail(FV_ERR_UNSUPPORTED, "more than 2^31 nodes");
  stage_begin(ctx);
  const int pd = int(h->pd);
  const float* q = d_queries;
  if (h->pd != h->dim) {
    FV_TRY(ctx->scratch[0].reserve(nq * size_t(pd) * sizeof(float)));
    FV_TRY(upload_padded(ctx, d_queries, true, nq, h->dim, h->pd, ctx->scratch[0].as<float>()));
    q = ctx->scratch[0].as<float>();
  }
  FV_TRY(ctx->scratch[5].reserve(nq * sizeof(uint32_t)));
  uint32_t* d_over = ctx->scratch[5].as<uint32_t>();
  unsigned long long* d_work = reinterpret_cast<unsigned long long*>(ctx->d_flags + 16);
  FV_CUDA(cudaMemsetAsync(d_work, 0, 3 * sizeof(unsigned long long), ctx->stream));
  HnswDev g{};
  g.data = h->d_data.as<float>();
  g.links0 = h->d_links0.as<uint32_t>();
  g.upper_off = h->d_upper_off.as<uint32_t>();
  g.upper_flat = h->d_upper_flat.as<uint32_t>();
  g.pd = pd;
  g.m0 = int(h->m0);
  g.metric = h->metric;
  g.top = int(h->top);
  g.ep = h->ep;
  g.n = n;
  // visited-table size: room for the nodes a beam of width ef usually touches, doubled
  int log2slots = 11;
  // visited-table size: a beam of width ef evaluates a few dozen nodes per entry kept; start at 48 * ef slots
  // (the table may fill to one half) and let the overflow path quadruple it for the queries that need more
  const char* menv = getenv("FV_HNSW_SLOTS_PER_EF");  // tuning knob
  const size_t per_ef = menv ? size_t(atoi(menv)) : 48;
  while ((size_t(1) << log2slots) < ef * per_ef && log2slots < 26) log2slots++;
  const uint32_t* d_qids = nullptr;
  size_t active = nq;
  std::vector<uint32_t> h_over(nq), retry;
  for (int attempt = 0; attempt < 8; ++attempt) {
    const size_t slots = size_t(1) << log2slots;
    const size_t base_bytes = size_t(pd) * 4 + ((ef * 8 + 15) & ~size_t(15)) + TIED_CAP * 4;
    const size_t budget = std::min<size_t>(ctx->smem_optin, 200 * 1024);
    int W = 8;
    bool use_global = false;
    // Tables in shared memory cap the resident warps (latency-bound kernel); in global memory they are
    // L2-resident and 32 warps fit per SM (64 registers each: the kernel spills about 40 words, which costs less
    // than the eight extra warps bring -- measured 4.85 against 5.30 ms per 10,000 queries with 24 warps of 80
    // registers, and 5.26 ms with 40 warps of 48).
    const char* genv = getenv("FV_HNSW_TABLES");  // tuning knob: "smem" or "global"
    use_global = genv ? genv[0] == 'g' : true;
    if (base_bytes + slots * 4 > budget / 2) use_global = true;
    const size_t per_warp = base_bytes + (use_global ? 0 : slots * 4);
    while (W > 1 && per_warp * W > budget) W >>= 1;
    if (per_warp * W > budget) return fail(FV_ERR_UNSUPPORTED, "dimension and ef too large for shared memory");
    int blocks_per_sm = int(std::max<size_t>(1, std::min<size_t>(budget / (per_warp * W), 32 / W)));
    size_t blocks = std::min<size_t>((active + W - 1) / W, size_t(ctx->sm_count) * blocks_per_sm);
    uint32_t* tables = nullptr;
    if (use_global) {
      FV_TRY(ctx->scratch[7].reserve(blocks * W * slots * 4));
      tables = ctx->scratch[7].as<uint32_t>();
    }
    auto kern = h->metric == FV_L2 ? hnsw_search_kernel<true> : hnsw_search_kernel<false>;
    const size_t smem = per_warp * W;
    if (smem > 40 * 1024) FV_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)));
    unsigned int* d_next = reinterpret_cast<unsigned int*>(ctx->d_flags + 32);
    FV_CUDA(cudaMemsetAsync(d_next, 0, sizeof(unsigned int), ctx->stream));
    kern<<<unsigned(blocks), W * 32, smem, ctx->stream>>>(g, q, d_qids, active, int(k), int(ef), log2slots, tables, keys,
                                                         d_over, d_work, d_next);
    ctx->stats.launches++;
    FV_CUDA(cudaGetLastError());
    FV_CUDA(cudaMemcpyAsync(h_over.data(), d_over, active * sizeof(uint32_t), cudaMemcpyDeviceToHost, ctx->stream));
    FV_CUDA(cudaStreamSynchronize(ctx->stream));
    std::vector<uint32_t> next;
    for (size_t i = 0; i < active; i++)
      if (h_over[i]) next.push_back(d_qids ? retry[i] : uint32_t(i));
    if (next.empty()) {
      active = 0;
      break;
    }
    ctx->stats.regrown += next.size();
    retry = next;
    active = retry.size();
    FV_TRY(ctx->scratch[6].reserve(active * sizeof(uint32_t)));
    FV_CUDA(cudaMemcpyAsync(ctx->scratch[6].p, retry.data(), active * sizeof(uint32_t), cudaMemcpyHostToDevice,
                            ctx->stream));
    d_qids = ctx->scratch[6].as<uint32_t>();
    log2slots = std::min(log2slots + 2, 27);
  }
  if (active) return fail(FV_ERR_OVERFLOW, "visited table overflow after regrowing");
  stage_mark(ctx);
  FV_TRY(keys_to_neighbors(ctx, keys, nq, int(k), int(k), d_out, d_counts));
  unsigned long long wk[3] = {0, 0, 0};
  FV_CUDA(cudaMemcpyAsync(wk, d_work, sizeof(wk), cudaMemcpyDeviceToHost, ctx->stream));
  FV_CUDA(cudaStreamSynchronize(ctx->stream));
  ctx->stats.dist_evals = wk[0];
  ctx->stats.expansions = wk[1];
  ctx->stats.uncertified = wk[2];  // queries whose list of tied, pushed-out entries overflowed (see TIED_CAP)
  stage_end(ctx);
  return bounds_report_hnsw();
}

int hnsw_new(fv_ctx* ctx, int metric, uint32_t dim, const float* vectors, size_t n, const fv_hnsw_params* p,
             std::unique_ptr<fv_hnsw>& out) {
  if (!ctx || !p || (!vectors && n) || dim == 0 || (metric != FV_L2 && metric != FV_INNER_PRODUCT))
    return fail(FV_ERR_ARG, "hnsw build: bad argument");
  if (p->m < 2 || p->m > 64) return fail(FV_ERR_UNSUPPORTED, "m must be in 2..64");
  auto h = std::unique_ptr<fv_hnsw>(new fv_hnsw());
  h->ctx = ctx;
  ctx_retain(ctx);
  h->metric = metric;
  h->dim = dim;
  h->pd = uint32_t(padded(dim));
  h->m = p->m;
  h->m0 = 2 * p->m;
  h->data.assign(n * size_t(h->pd), 0.f);
  for (size_t i = 0; i < n; i++) std::memcpy(&h->data[i * h->pd], vectors + i * size_t(dim), size_t(dim) * sizeof(float));
  // levels: hnsw.rs:88-94, drawn in node order from one generator
  const double ml = 1.0 / std::log(double(p->m));
  uint64_t s = (p->seed * 0x9E3779B97F4A7C15ull) | 1ull;
  h->levels.resize(n);
  for (size_t i = 0; i < n; i++) {
    s ^= s >> 12;
    s ^= s << 25;
    s ^= s >> 27;
    const double u = double((s * 0x2545F4914F6CDD1Dull) >> 11) / double(1ull << 53);
    const double v = -std::log(1.0 - u) * ml;
    const size_t lv = (v != v || v <= 0.0) ? 0 : (v >= 1.8e19 ? size_t(-1) : size_t(v));
    h->levels[i] = uint8_t(std::min<size_t>(lv, 15));
  }
  h->upper.resize(n);
  for (size_t i = 0; i < n; i++) h->upper[i].assign(size_t(h->levels[i]) * (h->m + 1), 0);
  h->links0.assign(n * (h->m0 + 1), 0);
  h->ep = 0;
  h->top = n ? h->levels[0] : 0;
  out = std::move(h);
  return FV_OK;
}

}  // namespace fv

extern "C" {

int fv_hnsw_build(fv_ctx* ctx, int metric, uint32_t dim, const float* vectors, size_t n, const fv_hnsw_params* p,
                  int threads, fv_hnsw** out) {
  if (!out) return fv::fail(FV_ERR_ARG, "fv_hnsw_build: bad argument");
  std::unique_ptr<fv_hnsw> h;
  FV_TRY(fv::hnsw_new(ctx, metric, dim, vectors, n, p, h));
  if (n > 1) {
    fv::Builder b;
    b.h = h.get();
    b.locks.reset(new std::mutex[n]);
    std::atomic<size_t> next{1};
    const int nt = std::max(1, threads);
    auto work = [&]() {
      fv::Builder::Visited vs;
      for (;;) {
        const size_t i = next.fetch_add(1, std::memory_order_relaxed);
        if (i >= n) break;
        b.insert(uint32_t(i), p->ef_construction, vs);
      }
    };
    std::vector<std::thread> th;
    for (int t = 1; t < nt; t++) th.emplace_back(work);
    work();
    for (auto& t : th) t.join();
  }
  fv::CtxGuard g(ctx);
  FV_TRY(fv::upload_graph(h.get()));
  *out = h.release();
  return FV_OK;
}

void fv_hnsw_free(fv_hnsw* ix) {
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

size_t fv_hnsw_len(const fv_hnsw* ix) { return ix ? ix->n() : 0; }
uint32_t fv_hnsw_dim(const fv_hnsw* ix) { return ix ? ix->dim : 0; }
int fv_hnsw_metric(const fv_hnsw* ix) { return ix ? ix->metric : -1; }

size_t fv_hnsw_reachable(const fv_hnsw* ix) {  // hnsw.rs:367-385
  if (!ix || ix->n() == 0) return 0;
  std::vector<char> seen(ix->n(), 0);
  std::vector<uint32_t> stack{ix->ep};
  seen[ix->ep] = 1;
  size_t count = 0;
  while (!stack.empty()) {
    const uint32_t x = stack.back();
    stack.pop_back();
    count++;
    const uint32_t* b = &ix->links0[size_t(x) * (ix->m0 + 1)];
    for (uint32_t i = 0; i < b[0]; i++) {
      const uint32_t y = b[1 + i];
      if (!seen[y]) {
        seen[y] = 1;
        stack.push_back(y);
      }
    }
  }
  return count;
}

double fv_hnsw_mean_degree(const fv_hnsw* ix) {  // hnsw.rs:388-393
  if (!ix) return 0.0;
  uint64_t total = 0;
  for (size_t i = 0; i < ix->n(); i++) total += ix->links0[i * (ix->m0 + 1)];
  return double(total) / double(std::max<size_t>(ix->n(), 1));
}

int fv_hnsw_search_batch_dev(fv_hnsw* ix, const float* d_queries, size_t nq, size_t k, size_t ef, fv_neighbor* d_out,
                             uint32_t* d_counts) {
  if (!ix || (nq && (!d_queries || !d_out))) return fv::fail(FV_ERR_ARG, "fv_hnsw_search_batch: null argument");
  fv::CtxGuard g(ix->ctx);
  return fv::hnsw_search_dev(ix, d_queries, nq, k, ef, d_out, d_counts);
}

int fv_hnsw_search_batch(fv_hnsw* ix, const float* queries, size_t nq, size_t k, size_t ef, fv_neighbor* out,
                         uint32_t* counts) {
  if (!ix || (nq && (!queries || !out))) return fv::fail(FV_ERR_ARG, "fv_hnsw_search_batch: null argument");
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
  FV_TRY(fv::hnsw_search_dev(ix, dq, nq, k, ef, dout, dc));
  FV_CUDA(cudaMemcpyAsync(out, dout, obytes, cudaMemcpyDeviceToHost, ctx->stream));
  if (counts) FV_CUDA(cudaMemcpyAsync(counts, dc, nq * sizeof(uint32_t), cudaMemcpyDeviceToHost, ctx->stream));
  FV_CUDA(cudaStreamSynchronize(ctx->stream));
  return FV_OK;
}

int fv_hnsw_search(fv_hnsw* ix, const float* query, size_t k, size_t ef, fv_neighbor* out, uint32_t* count) {
  return fv_hnsw_search_batch(ix, query, 1, k, ef, out, count);
}

// ---- FLHNSW01 files (hnsw.rs:395-466)
size_t fv_hnsw_save_size(const fv_hnsw* ix) {
  if (!ix) return 0;
  size_t flat = 0;
  for (size_t i = 0; i < ix->n(); i++)
    for (size_t l = 0; l < ix->levels[i]; l++) flat += 1 + ix->upper[i][l * (ix->m + 1)];
  return 8 + 5 * 4 + (8 + ix->levels.size()) + (8 + ix->links0.size() * 4) + (8 + flat * 4) + (8 + ix->data.size() * 4);
}

int fv_hnsw_save(const fv_hnsw* ix, uint8_t* buf, size_t cap, size_t* written) {
  if (!ix || !buf) return fv::fail(FV_ERR_ARG, "fv_hnsw_save: null argument");
  if (cap < fv_hnsw_save_size(ix)) return fv::fail(FV_ERR_ARG, "fv_hnsw_save: buffer too small");
  uint8_t* w = buf;
  auto raw = [&](const void* p, size_t n) {
    if (n) std::memcpy(w, p, n);
    w += n;
  };
  auto u32 = [&](uint32_t v) { raw(&v, 4); };
  auto u64w = [&](uint64_t v) { raw(&v, 8); };
  raw("FLHNSW01", 8);
  u32(uint32_t(ix->metric));
  u32(ix->dim);
  u32(uint32_t(ix->m));
  u32(ix->ep);
  u32(uint32_t(ix->top));
  u64w(ix->levels.size());
  raw(ix->levels.data(), ix->levels.size());
  u64w(ix->links0.size());
  raw(ix->links0.data(), ix->links0.size() * 4);
  std::vector<uint32_t> off, flat;
  fv::flatten_upper(ix, off, flat);
  u64w(flat.size());
  raw(flat.data(), flat.size() * 4);
  u64w(ix->data.size());
  raw(ix->data.data(), ix->data.size() * 4);
  if (written) *written = size_t(w - buf);
  return FV_OK;
}

int fv_hnsw_load(fv_ctx* ctx, const uint8_t* bytes, size_t len, fv_hnsw** out) {
  if (!ctx || !bytes || !out) return fv::fail(FV_ERR_ARG, "fv_hnsw_load: null argument");
  if (len < 8 || std::memcmp(bytes, "FLHNSW01", 8) != 0) return fv::fail(FV_ERR_FILE, "not an HNSW index file");
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
  auto span = [&](size_t elem, size_t* count) -> const uint8_t* {
    uint64_t n = 0;
    if (auto p = take(8)) std::memcpy(&n, p, 8);
    if (!ok || n > (len - i) / elem) {
      ok = false;
      return nullptr;
    }
    *count = size_t(n);
    return take(size_t(n) * elem);
  };
  const char* trunc = "index file is truncated";
  auto h = std::unique_ptr<fv_hnsw>(new fv_hnsw());
  h->ctx = ctx;
  fv::ctx_retain(ctx);
  const uint32_t mc = u32();
  h->dim = u32();
  h->m = u32();
  h->ep = u32();
  h->top = u32();
  if (!ok) return fv::fail(FV_ERR_FILE, trunc);
  if ((mc & 0xFF) > 1) return fv::fail(FV_ERR_FILE, "bad metric");
  h->metric = int(mc & 0xFF);
  size_t nl = 0, nk = 0, nf = 0, nd = 0;
  const uint8_t* pl = span(1, &nl);
  const uint8_t* pk = span(4, &nk);
  const uint8_t* pf = span(4, &nf);
  const uint8_t* pdat = span(4, &nd);
  if (!ok) return fv::fail(FV_ERR_FILE, trunc);
  h->levels.assign(pl, pl + nl);
  std::vector<uint32_t> flat(nf);
  if (nf) std::memcpy(flat.data(), pf, nf * 4);
  const size_t n = nl;
  h->pd = uint32_t(fv::padded(h->dim));
  h->m0 = 2 * h->m;
  if (h->dim == 0 || h->m == 0) return fv::fail(FV_ERR_FILE, "index file sizes do not match");
  h->upper.resize(n);
  size_t at = 0;
  for (size_t node = 0; node < n; node++) {
    h->upper[node].assign(size_t(h->levels[node]) * (h->m + 1), 0);
    for (size_t l = 0; l < h->levels[node]; l++) {
      if (at >= nf) return fv::fail(FV_ERR_FILE, "truncated links");
      const size_t c = flat[at];
      if (at + 1 + c > nf) return fv::fail(FV_ERR_FILE, "truncated links");
      if (c > h->m) return fv::fail(FV_ERR_FILE, "index file sizes do not match");
      uint32_t* b = &h->upper[node][l * (h->m + 1)];
      b[0] = uint32_t(c);
      for (size_t t = 0; t < c; t++) b[1 + t] = flat[at + 1 + t];
      at += 1 + c;
    }
  }
  if (nk != n * (2 * h->m + 1) || nd != n * size_t(h->pd)) return fv::fail(FV_ERR_FILE, "index file sizes do not match");
  h->links0.resize(nk);
  if (nk) std::memcpy(h->links0.data(), pk, nk * 4);
  h->data.resize(nd);
  if (nd) std::memcpy(h->data.data(), pdat, nd * 4);
  // a damaged file must not send the kernel out of bounds
  if (n && (h->ep >= n || h->top > 15 || h->levels[h->ep] < h->top)) return fv::fail(FV_ERR_FILE, "bad entry point");
  for (size_t node = 0; node < n; node++) {
    const uint32_t* b = &h->links0[node * (h->m0 + 1)];
    if (b[0] > h->m0) return fv::fail(FV_ERR_FILE, "bad link count");
    for (uint32_t t = 0; t < b[0]; t++)
      if (b[1 + t] >= n) return fv::fail(FV_ERR_FILE, "link out of range");
    for (size_t l = 0; l < h->levels[node]; l++) {
      const uint32_t* u = &h->upper[node][l * (h->m + 1)];
      for (uint32_t t = 0; t < u[0]; t++)
        if (u[1 + t] >= n || h->levels[u[1 + t]] < l + 1) return fv::fail(FV_ERR_FILE, "link out of range");
    }
  }
  fv::CtxGuard g(ctx);
  FV_TRY(fv::upload_graph(h.get()));
  *out = h.release();
  return FV_OK;
}

}  // extern "C"
