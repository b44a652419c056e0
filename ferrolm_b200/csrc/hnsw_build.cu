// Hnsw construction on the GPU (src/vector/hnsw.rs:85-129 build, :244-290 insert, :230-242 select, :294-320
// add_links), batch-synchronous.
//
// The reference hands nodes out in id order to the pool's threads; what each thread's search sees of the others'
// half-made links depends on timing.  Here nodes go in in id order in BATCHES:
//   1. hnsw_insert_kernel, one warp per node of the batch: the greedy descent and the per-layer search_layer of
//      insert() against the graph as it stood when the batch began (no node of the batch is visible to another),
//      then select() over what was found; the node's own lists are written and one edge (target, layer, source) per
//      chosen neighbour is pushed on a chain headed at (target, layer);
//   2. hnsw_link_kernel, one warp per (target, layer) chain: add_links(target, layer, [source]) for the chain's
//      sources in ascending id, that is in the order a single thread would have reached them.
// Between batches the entry point moves as in hnsw.rs:285-289; a node above the current top layer ends its batch
// before it and goes in alone.  The result does not depend on timing: the same input gives the same graph, and with
// batches of one node it is byte for byte the graph of the reference's single-thread build.
//
// A batch holds at most max_batch nodes and at most 1/divisor of the nodes already in, so that the early graph (the
// backbone every later search walks) is built nearly node by node.
#include <algorithm>
#include <cstring>

#include "hnsw.cuh"

FV_BOUNDS_TU(hnsw_build)

namespace fv {

static constexpr uint32_t NIL = 0xFFFFFFFFu;
static constexpr int BUILD_BLOCKS_PER_SM = 3;  // of 256 threads: 24 warps per SM at up to 80 registers
static constexpr int SRC_CAP = 128;  // sources of one chain sorted in shared memory; longer chains are walked again per source

struct Edge {
  uint32_t tgt, src, blk, next;  // blk: the chain's head slot; next: the edge pushed before this one on the same chain
};

struct BuildDev {
  const float* data;
  uint32_t* links0;         // n x (m0 + 1): count, ids
  uint32_t* up;             // upper layers: blocks of (m + 1) words, per node its layers 1..level
  const uint32_t* up_blk;   // n + 1: first block of each node
  const uint8_t* levels;
  int pd, m, m0;
  uint32_t n;
};

__device__ __forceinline__ uint32_t* link_row(const BuildDev& g, uint32_t x, int layer) {
  return layer == 0 ? g.links0 + size_t(x) * (g.m0 + 1) : g.up + (size_t(g.up_blk[x]) + layer - 1) * (g.m + 1);
}
__device__ __forceinline__ uint32_t head_slot(const BuildDev& g, uint32_t x, int layer) {
  return layer == 0 ? x : g.n + g.up_blk[x] + uint32_t(layer - 1);
}

// select (hnsw.rs:230-242): from candidates sorted nearest first (keys: order bits of the distance above, id at
// `id_shift` below), keep those farther from every kept one than from the base, up to cap.  `sc` stages the
// candidate's row.  Returns the number kept (ids in sel[]).
template <bool IS_L2>
__device__ __forceinline__ int select_links(const BuildDev& g, const u64* cand, int ncand, int id_shift, int cap,
                                            float* sc, uint32_t* sel) {
  const int lane = lane_id();
  int nsel = 0;
  for (int i = 0; i < ncand && nsel < cap; ++i) {
    const u64 ck = cand[i];
    const uint32_t cid = uint32_t((ck & 0xFFFFFFFFull) >> id_shift);
    const float cd = order_bits_to_float(uint32_t(ck >> 32));
    if (!FV_IDX_OK(cid, g.n, 3)) continue;
    bool bad = false;
    if (nsel > 0) {
      __syncwarp();
      for (int c = lane; c < g.pd; c += 32) sc[c] = g.data[size_t(cid) * g.pd + c];
      __syncwarp();
      for (int s0 = 0; s0 < nsel && !bad; s0 += 32) {
        const int s = s0 + lane;
        bool b = false;
        if (s < nsel) b = !(exact_distance<IS_L2>(sc, g.data + size_t(sel[s]) * g.pd, g.pd) > cd);
        bad = __any_sync(FV_FULL, b);
      }
    }
    if (!bad) {
      __syncwarp();
      if (lane == 0) sel[nsel] = cid;
      nsel++;
      __syncwarp();
    }
  }
  return nsel;
}

// flags: [0] visited-table overflows, [1] tie lists that overflowed, [2] edges that did not fit
template <bool IS_L2>
__global__ void __launch_bounds__(256, BUILD_BLOCKS_PER_SM)
    hnsw_insert_kernel(BuildDev g, uint32_t lo, uint32_t hi, uint32_t ep, int top, int ef, int log2slots,
                       uint32_t* __restrict__ tables, Edge* __restrict__ edges, uint32_t* __restrict__ edge_cnt,
                       uint32_t* __restrict__ next_node, uint32_t edge_cap, uint32_t* __restrict__ head,
                       unsigned long long* __restrict__ flags) {
  unsigned char* smem_raw = dyn_smem();
  const int W = blockDim.x >> 5, w = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const size_t list_bytes = (size_t(ef) * 8 + 15) & ~size_t(15);
  const size_t per_warp = size_t(g.pd) * 8 + list_bytes + TIED_CAP * 4 + size_t(g.m0) * 4;
  unsigned char* mine = smem_raw + size_t(w) * per_warp;
  float* sq = reinterpret_cast<float*>(mine);
  float* sc = sq + g.pd;
  u64* best = reinterpret_cast<u64*>(mine + size_t(g.pd) * 8);
  uint32_t* tied = reinterpret_cast<uint32_t*>(mine + size_t(g.pd) * 8 + list_bytes);
  uint32_t* sel = tied + TIED_CAP;
  const uint32_t gw = blockIdx.x * W + w;
  uint32_t* table = tables + (size_t(gw) << log2slots);

  // nodes are drawn from a counter: a search takes anything from a few to a few hundred expansions, and which warp
  // inserts which node changes nothing in the result
  for (;;) {
    uint32_t id = 0;
    if (lane == 0) id = lo + atomicAdd(next_node, 1u);
    id = __shfl_sync(FV_FULL, id, 0);
    if (id >= hi) break;
    const int level = g.levels[id];
    __syncwarp();
    for (int c = lane; c < g.pd; c += 32) sq[c] = g.data[size_t(id) * g.pd + c];
    warp_list_init(best, ef);

    // greedy descent through the layers above the node's own (hnsw.rs:254-268)
    uint32_t cur = ep;
    float curd = exact_distance<IS_L2>(sq, g.data + size_t(cur) * g.pd, g.pd);
    for (int layer = top; layer > level; --layer) {
      bool changed = true;
      while (changed) {
        changed = false;
        const uint32_t* row = link_row(g, cur, layer);
        const int cnt = min(int(row[0]), g.m);
        for (int c0 = 0; c0 < cnt; c0 += 32) {
          const int i = c0 + lane;
          uint32_t x = 0;
          float d = INFINITY;
          const bool on = i < cnt && FV_IDX_OK(row[1 + i], g.n, 4);
          if (on) {
            x = row[1 + i];
            d = exact_distance<IS_L2>(sq, g.data + size_t(x) * g.pd, g.pd);
          }
          const unsigned better = __ballot_sync(FV_FULL, on && d < curd);
          if (better) {
            float md = d < curd ? d : INFINITY;
            for (int o = 16; o > 0; o >>= 1) md = fminf(md, __shfl_xor_sync(FV_FULL, md, o));
            const unsigned at = __ballot_sync(FV_FULL, on && d == md);
            cur = __shfl_sync(FV_FULL, x, __ffs(at) - 1);
            curd = md;
            changed = true;
          }
        }
      }
    }

    warp_list_insert(best, ef, beam_key(curd, cur));
    int filled = 1;
    bool tie_lost = false;
    for (int layer = min(level, top); layer >= 0; --layer) {
      bool over = false;
      unsigned long long n_dist = 0, n_exp = 0;  // (not reported by the build)
      beam_search<IS_L2>(g.data, g.pd, g.n, [&](uint32_t c) { return (const uint32_t*)link_row(g, c, layer); },
                         layer == 0 ? g.m0 : g.m, sq, best, ef, tied, table, log2slots, filled, over, tie_lost, n_dist,
                         n_exp);
      if (over) {
        if (lane == 0) atomicAdd(flags, 1ull);
        break;
      }
      const int cap = layer == 0 ? g.m0 : g.m;
      const int nsel = select_links<IS_L2>(g, best, filled, 1, cap, sc, sel);
      // the node's own list: it is new, so add_links(id, layer, chosen) finds it empty (hnsw.rs:277)
      uint32_t* own = link_row(g, id, layer);
      for (int i = lane; i < nsel; i += 32) own[1 + i] = sel[i];
      uint32_t base = 0;
      if (lane == 0) {
        own[0] = uint32_t(nsel);
        base = atomicAdd(edge_cnt, uint32_t(nsel));
      }
      base = __shfl_sync(FV_FULL, base, 0);
      if (base + uint32_t(nsel) > edge_cap) {
        if (lane == 0) atomicAdd(flags + 2, 1ull);
        break;
      }
      for (int i = lane; i < nsel; i += 32) {
        const uint32_t e = base + uint32_t(i), t = sel[i];
        const uint32_t blk = head_slot(g, t, layer);
        Edge ed;
        ed.tgt = t;
        ed.src = id;
        ed.blk = blk;
        ed.next = atomicExch(head + blk, e);
        edges[e] = ed;
      }
      __syncwarp();
    }
    if (tie_lost && lane == 0) atomicAdd(flags + 1, 1ull);
  }
}

// add_links(target, layer, [source]) (hnsw.rs:294-320) for every edge of the batch.  The warp whose edge was the
// first pushed on its chain (next == NIL) owns the chain's (target, layer).
template <bool IS_L2>
__global__ void __launch_bounds__(256, BUILD_BLOCKS_PER_SM)
    hnsw_link_kernel(BuildDev g, const Edge* __restrict__ edges, const uint32_t* __restrict__ edge_cnt,
                     uint32_t edge_cap, uint32_t* __restrict__ head) {
  unsigned char* smem_raw = dyn_smem();
  const int W = blockDim.x >> 5, w = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int cap_max = g.m0, nc = cap_max + 1;
  const size_t keys_bytes = (size_t(nc) * 8 + 15) & ~size_t(15);
  const size_t per_warp = size_t(g.pd) * 8 + 2 * keys_bytes + size_t(nc + cap_max + 2 * SRC_CAP + 1) * 4;
  unsigned char* mine = smem_raw + size_t(w) * ((per_warp + 15) & ~size_t(15));
  float* sb = reinterpret_cast<float*>(mine);
  float* sc = sb + g.pd;
  u64* keys = reinterpret_cast<u64*>(mine + size_t(g.pd) * 8);
  u64* sorted = reinterpret_cast<u64*>(mine + size_t(g.pd) * 8 + keys_bytes);
  uint32_t* ids = reinterpret_cast<uint32_t*>(mine + size_t(g.pd) * 8 + 2 * keys_bytes);
  uint32_t* sel = ids + nc;
  uint32_t* srcs = sel + cap_max;
  uint32_t* srcs_sorted = srcs + SRC_CAP;
  const uint32_t count = min(*edge_cnt, edge_cap);
  const uint32_t gw = blockIdx.x * W + w, total_warps = gridDim.x * W;

  for (uint32_t e = gw; e < count; e += total_warps) {
    const Edge first = edges[e];
    if (first.next != NIL) continue;
    const uint32_t t = first.tgt;
    if (!FV_IDX_OK(t, g.n, 5)) continue;
    const int layer = first.blk < g.n ? 0 : int(first.blk - g.n - g.up_blk[t]) + 1;
    const int cap = layer == 0 ? g.m0 : g.m;
    uint32_t* row = link_row(g, t, layer);
    __syncwarp();
    // the chain's sources; the walk is bounded by the number of edges
    int k = 0;
    if (lane == 0) {
      uint32_t x = head[first.blk];
      for (uint32_t hop = 0; x != NIL && hop < count; ++hop) {
        if (!FV_IDX_OK(x, count, 6)) break;
        if (k < SRC_CAP) srcs[k] = edges[x].src;
        k++;
        x = edges[x].next;
      }
    }
    k = __shfl_sync(FV_FULL, k, 0);
    __syncwarp();
    if (k <= SRC_CAP) {  // ascending by rank: ids are distinct
      for (int i = lane; i < k; i += 32) {
        const uint32_t v = srcs[i];
        int r = 0;
        for (int j = 0; j < k; ++j) r += srcs[j] < v;
        srcs_sorted[r] = v;
      }
      __syncwarp();
    }
    for (int c = lane; c < g.pd; c += 32) sb[c] = g.data[size_t(t) * g.pd + c];
    // The list is kept in shared memory and every change is written through to the row as set_neighbors does
    // (hnsw.rs:165-175): a shorter list leaves the old ids behind it in the row, and the FLHNSW01 file holds the
    // rows whole, so the words past the count must be the reference's too.
    int cnt = min(int(row[0]), cap);
    for (int i = lane; i < cnt; i += 32) ids[i] = row[1 + i];
    __syncwarp();
    long long last = -1;
    for (int si = 0; si < k; ++si) {
      uint32_t s;
      if (k <= SRC_CAP) {
        s = srcs_sorted[si];
      } else {  // the smallest source above the last one, by another walk
        uint32_t best_s = NIL;
        if (lane == 0) {
          uint32_t x = head[first.blk];
          for (uint32_t hop = 0; x != NIL && hop < count; ++hop) {
            if (!FV_IDX_OK(x, count, 7)) break;
            const uint32_t v = edges[x].src;
            if ((long long)v > last && v < best_s) best_s = v;
            x = edges[x].next;
          }
        }
        s = __shfl_sync(FV_FULL, best_s, 0);
        if (s == NIL) break;
      }
      last = (long long)s;
      // x != id && !list.contains(&x)  (hnsw.rs:299-303)
      bool dup = s == t;
      for (int i0 = 0; i0 < cnt && !dup; i0 += 32) {
        const int i = i0 + lane;
        dup = __any_sync(FV_FULL, i < cnt && ids[i] == s);
      }
      if (dup || !FV_IDX_OK(s, g.n, 8)) continue;
      __syncwarp();
      if (lane == 0) ids[cnt] = s;
      cnt++;
      __syncwarp();
      if (cnt > cap) {
        // distances from the base, sorted by (distance, id), chosen again (hnsw.rs:307-318)
        for (int i = lane; i < cnt; i += 32)
          keys[i] = make_key(exact_distance<IS_L2>(sb, g.data + size_t(ids[i]) * g.pd, g.pd), ids[i]);
        __syncwarp();
        for (int i = lane; i < cnt; i += 32) {
          const u64 v = keys[i];
          int r = 0;
          for (int j = 0; j < cnt; ++j) r += keys[j] < v;
          sorted[r] = v;
        }
        __syncwarp();
        const int nsel = select_links<IS_L2>(g, sorted, cnt, 0, cap, sc, sel);
        for (int i = lane; i < nsel; i += 32) {
          ids[i] = sel[i];
          row[1 + i] = sel[i];
        }
        cnt = nsel;
        __syncwarp();
      } else if (lane == 0) {
        row[cnt] = s;
      }
    }
    if (lane == 0) {
      row[0] = uint32_t(cnt);
      head[first.blk] = NIL;
    }
    __syncwarp();
  }
}

// The next batch: at most max_batch nodes, at most 1/divisor of those already in, cut before a node whose level is
// above the current top layer (such a node goes in alone).
static size_t next_batch(const std::vector<uint8_t>& levels, size_t inserted, size_t top, size_t max_batch,
                         size_t divisor) {
  const size_t n = levels.size();
  size_t b = std::max<size_t>(1, std::min(max_batch, inserted / std::max<size_t>(1, divisor)));
  b = std::min(b, n - inserted);
  if (levels[inserted] > top) return 1;
  for (size_t j = 1; j < b; j++)
    if (levels[inserted + j] > top) return j;
  return b;
}

static int build_on_device(fv_hnsw* h, size_t ef, size_t max_batch, size_t divisor) {
  fv_ctx* ctx = h->ctx;
  const size_t n = h->n(), m = h->m, m0 = h->m0;
  if (n > 0x7FFFFFFFull) return fail(FV_ERR_UNSUPPORTED, "more than 2^31 nodes");
  if (ef == 0 || ef > 4096) return fail(FV_ERR_UNSUPPORTED, "ef_construction must be in 1..4096");
  const int pd = int(h->pd);
  // block offsets of the upper layers; the batches and the edges the largest can push
  std::vector<uint32_t> up_blk(n + 1, 0);
  for (size_t i = 0; i < n; i++) up_blk[i + 1] = up_blk[i] + h->levels[i];
  const size_t nblk = up_blk[n];
  if (n + nblk >= 0xFFFFFFFFull) return fail(FV_ERR_UNSUPPORTED, "too many link lists for 32-bit chain heads");
  size_t edge_cap = 0, widest = 0;
  {
    size_t inserted = 1, top = h->levels[0];
    while (inserted < n) {
      const size_t b = next_batch(h->levels, inserted, top, max_batch, divisor);
      size_t e = 0;
      for (size_t j = 0; j < b; j++) e += m0 + std::min<size_t>(h->levels[inserted + j], top) * m;
      edge_cap = std::max(edge_cap, e);
      widest = std::max(widest, b);
      if (h->levels[inserted] > top) top = h->levels[inserted];
      inserted += b;
    }
  }
  if (edge_cap >= 0xFFFFFFFFull) return fail(FV_ERR_UNSUPPORTED, "batch too large");

  DevBuf d_up, d_up_blk, d_levels, d_head, d_edges, d_tables, d_words;
  FV_TRY(h->d_data.reserve(h->data.size() * 4 + 16));
  FV_TRY(h->d_links0.reserve(h->links0.size() * 4 + 16));
  FV_TRY(d_up.reserve(nblk * (m + 1) * 4 + 16));
  FV_TRY(d_up_blk.reserve((n + 1) * 4));
  FV_TRY(d_levels.reserve(n + 16));
  FV_TRY(d_head.reserve((n + nblk) * 4 + 16));
  FV_TRY(d_edges.reserve((edge_cap + 1) * sizeof(Edge)));
  FV_TRY(d_words.reserve(64));
  uint32_t* d_edge_cnt = d_words.as<uint32_t>();
  uint32_t* d_next_node = d_edge_cnt + 1;
  unsigned long long* d_flags = reinterpret_cast<unsigned long long*>(d_words.as<unsigned char>() + 16);
  cudaStream_t st = ctx->stream;
  FV_CUDA(cudaMemcpyAsync(h->d_data.p, h->data.data(), h->data.size() * 4, cudaMemcpyHostToDevice, st));
  FV_CUDA(cudaMemcpyAsync(d_up_blk.p, up_blk.data(), (n + 1) * 4, cudaMemcpyHostToDevice, st));
  FV_CUDA(cudaMemcpyAsync(d_levels.p, h->levels.data(), n, cudaMemcpyHostToDevice, st));

  BuildDev g{};
  g.data = h->d_data.as<float>();
  g.links0 = h->d_links0.as<uint32_t>();
  g.up = d_up.as<uint32_t>();
  g.up_blk = d_up_blk.as<uint32_t>();
  g.levels = d_levels.as<uint8_t>();
  g.pd = pd;
  g.m = int(m);
  g.m0 = int(m0);
  g.n = uint32_t(n);

  // launch shapes: shared memory per warp, warps per block, resident warps
  const size_t list_bytes = (ef * 8 + 15) & ~size_t(15);
  const size_t ins_warp = size_t(pd) * 8 + list_bytes + TIED_CAP * 4 + m0 * 4;
  const size_t nc = m0 + 1;
  const size_t keys_bytes = (nc * 8 + 15) & ~size_t(15);
  const size_t link_warp = ((size_t(pd) * 8 + 2 * keys_bytes + (nc + m0 + 2 * SRC_CAP + 1) * 4) + 15) & ~size_t(15);
  const size_t budget = std::min<size_t>(ctx->smem_optin, 200 * 1024);
  int W = 8;
  while (W > 1 && std::max(ins_warp, link_warp) * W > budget / BUILD_BLOCKS_PER_SM) W >>= 1;
  if (std::max(ins_warp, link_warp) * W > budget) return fail(FV_ERR_UNSUPPORTED, "dimension and ef_construction too large for shared memory");
  const size_t resident_blocks = size_t(ctx->sm_count) * BUILD_BLOCKS_PER_SM;
  const size_t ins_blocks_max = std::min<size_t>(resident_blocks, (widest + W - 1) / W);
  auto ins = h->metric == FV_L2 ? hnsw_insert_kernel<true> : hnsw_insert_kernel<false>;
  auto lnk = h->metric == FV_L2 ? hnsw_link_kernel<true> : hnsw_link_kernel<false>;
  if (ins_warp * W > 40 * 1024) FV_CUDA(cudaFuncSetAttribute(ins, cudaFuncAttributeMaxDynamicSharedMemorySize, int(ins_warp * W)));
  if (link_warp * W > 40 * 1024) FV_CUDA(cudaFuncSetAttribute(lnk, cudaFuncAttributeMaxDynamicSharedMemorySize, int(link_warp * W)));

  int log2slots = 11;
  while ((size_t(1) << log2slots) < ef * 128 && log2slots < 24) log2slots++;
  for (int attempt = 0; attempt < 3; ++attempt, log2slots += 2) {
    FV_TRY(d_tables.reserve((ins_blocks_max * W << log2slots) * 4 + 16));
    FV_CUDA(cudaMemsetAsync(h->d_links0.p, 0, h->links0.size() * 4, st));
    FV_CUDA(cudaMemsetAsync(d_up.p, 0, nblk * (m + 1) * 4, st));
    FV_CUDA(cudaMemsetAsync(d_head.p, 0xFF, (n + nblk) * 4, st));
    FV_CUDA(cudaMemsetAsync(d_words.p, 0, 64, st));
    size_t inserted = 1, top = h->levels[0];
    uint32_t ep = 0;
    stage_begin(ctx);  // stage 0: uploads and clears; stage 1: the batches
    stage_mark(ctx);
    while (inserted < n) {
      const size_t b = next_batch(h->levels, inserted, top, max_batch, divisor);
      FV_CUDA(cudaMemsetAsync(d_edge_cnt, 0, 8, st));  // and the node counter
      const size_t ins_blocks = std::min<size_t>(ins_blocks_max, (b + W - 1) / W);
      ins<<<unsigned(ins_blocks), W * 32, ins_warp * W, st>>>(g, uint32_t(inserted), uint32_t(inserted + b), ep, int(top),
                                                               int(ef), log2slots, d_tables.as<uint32_t>(),
                                                               d_edges.as<Edge>(), d_edge_cnt, d_next_node, uint32_t(edge_cap),
                                                               d_head.as<uint32_t>(), d_flags);
      FV_CUDA(cudaGetLastError());
      size_t e_max = 0;
      for (size_t j = 0; j < b; j++) e_max += m0 + std::min<size_t>(h->levels[inserted + j], top) * m;
      const size_t lnk_blocks = std::max<size_t>(1, std::min<size_t>(resident_blocks, (e_max + W - 1) / W));
      lnk<<<unsigned(lnk_blocks), W * 32, link_warp * W, st>>>(g, d_edges.as<Edge>(), d_edge_cnt, uint32_t(edge_cap),
                                                              d_head.as<uint32_t>());
      FV_CUDA(cudaGetLastError());
      ctx->stats.launches += 2;
      if (h->levels[inserted] > top) {  // hnsw.rs:285-289
        top = h->levels[inserted];
        ep = uint32_t(inserted);
      }
      inserted += b;
    }
    stage_mark(ctx);
    unsigned long long flags[3] = {0, 0, 0};
    FV_CUDA(cudaMemcpyAsync(flags, d_flags, sizeof(flags), cudaMemcpyDeviceToHost, st));
    FV_CUDA(cudaStreamSynchronize(st));
    stage_end(ctx);
    FV_TRY(bounds_report_hnsw_build());
    if (flags[2]) return fail(FV_ERR_OVERFLOW, "hnsw build: edge buffer overflow");
    if (flags[0]) {
      ctx->stats.regrown += flags[0];
      continue;  // a visited table filled up: again with tables four times larger
    }
    ctx->stats.uncertified = flags[1];  // searches whose list of tied, pushed-out entries overflowed (see TIED_CAP)
    h->ep = ep;
    h->top = top;
    FV_CUDA(cudaMemcpyAsync(h->links0.data(), h->d_links0.p, h->links0.size() * 4, cudaMemcpyDeviceToHost, st));
    std::vector<uint32_t> flat(nblk * (m + 1));
    if (!flat.empty()) FV_CUDA(cudaMemcpyAsync(flat.data(), d_up.p, flat.size() * 4, cudaMemcpyDeviceToHost, st));
    FV_CUDA(cudaStreamSynchronize(st));
    for (size_t i = 0; i < n; i++)
      if (h->levels[i])
        std::memcpy(h->upper[i].data(), &flat[size_t(up_blk[i]) * (m + 1)], size_t(h->levels[i]) * (m + 1) * 4);
    return FV_OK;
  }
  return fail(FV_ERR_OVERFLOW, "hnsw build: visited table overflow after regrowing");
}

}  // namespace fv

extern "C" int fv_hnsw_build_batched(fv_ctx* ctx, int metric, uint32_t dim, const float* vectors, size_t n,
                                     const fv_hnsw_params* p, size_t max_batch, size_t divisor, fv_hnsw** out) {
  if (!out || max_batch == 0 || divisor == 0) return fv::fail(FV_ERR_ARG, "fv_hnsw_build_batched: bad argument");
  std::unique_ptr<fv_hnsw> h;
  FV_TRY(fv::hnsw_new(ctx, metric, dim, vectors, n, p, h));
  fv::CtxGuard g(ctx);
  ctx->stats = fv_stats{};
  if (n > 1) {
    FV_TRY(fv::build_on_device(h.get(), p->ef_construction, max_batch, divisor));
    FV_TRY(fv::upload_graph(h.get(), false));
  } else {
    FV_TRY(fv::upload_graph(h.get()));
  }
  *out = h.release();
  return FV_OK;
}
