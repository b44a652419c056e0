// IvfPq::search (ivfpq.rs:225-297) on the GPU: lookup tables, ADC scan, top-k and the optional exact re-rank.
//
// Two scans produce the same result.
//
//  * ivfpq_scan_kernel: one block per query.  Per probed cell the block builds the cell's table in shared memory and
//    its lanes walk the list's rows (codes differ per lane: the sixteen lookups of a row land in random banks).
//    It serves every index (any m, with or without precomputed tables), small batches and the fallback of the
//    list-major scan.
//
//  * ivfpq_list_scan_kernel: list-major, for m = 16 with the query's table separable from the cell's
//    (lut = pre[l] + qtab[q], ivfpq.rs:256-262, or lut = qtab[q] for inner product, :236-238).  The (query, probe)
//    pairs of a batch are bucketed by list.  A task is (list, up to 1024 of its rows, up to 4 groups of 32 queries
//    that probe it).  The 32 queries of a group sit one per LANE and a warp walks rows: every lane of a lookup
//    reads the same table entry (sub-quantizer j, code c) of its own query, and the group's tables are stored
//    entry-major -- word c * 36 + lane of the slice of sub-quantizer j -- so the 32 reads of a lookup fall into 32
//    different banks: one shared-memory wavefront per 32 lookups instead of the ~2.7 of random codes.  Shared
//    memory holds two such slices (one sub-quantizer each, 36 KB); the scan runs in 16 phases, one per
//    sub-quantizer in the reference's order, and the partial sums of a lane's rows (64 per thread) wait in registers
//    between phases, so every distance is base + lut[0] + ... + lut[15] added in that order: bit-identical to
//    ivfpq.rs:272-276.  The next slices are on their way while a phase runs: cp.async brings the 32 queries' raw
//    table rows (1 KB each) into a staging buffer two phases ahead, and one phase ahead the threads turn them into
//    the entry-major slice (conflict-free reads, + pre[l], conflict-free 16-byte stores), so no phase waits for L2.
//    The code bytes come from a second, sub-quantizer-major copy of the lists: one 16-byte broadcast read serves
//    16 rows of a phase.
//    Candidates.  A BOUND pass runs the same kernel over each query's few nearest probed lists and keeps, per
//    thread, the minimum of every 8 rows; the keep-th smallest of a query's minima is a distance that at least
//    `keep` of its rows reach (every minimum is a different row), hence an upper bound of its keep-th best.  The
//    main pass appends every row at or below that bound to the query's buffer in global memory; a finishing kernel
//    sorts the buffer, keeps the best `keep` and re-ranks.  A query whose buffer overflows is re-run by the
//    per-query kernel.
#include <algorithm>
#include <cmath>
#include <cstdlib>

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "ivfpq_scan.h"

FV_BOUNDS_TU(ivfpq_scan)

extern "C" int fv_debug_bounds_build(void) {
#ifdef FV_BOUNDS
  return 1;
#else
  return 0;
#endif
}

namespace fv {

static const size_t KSUB = 256;

// ------------------------------------------------------------------------------------------------
struct ScanArgs {
  const float* queries;  // nq x pd
  const u64* cells;      // nq x nprobe keys (distance, list), ascending
  const float* centroids;
  const float* codebooks;
  const float* pre;  // may be null
  const float* qtab; // nq x m x 256: per query, -dot(q_j, w) (inner product) or -2 dot(q_j, w) (L2 with tables)
  const uint32_t* list_off;
  const uint8_t* codes;
  const uint32_t* ids;
  const float* vectors;  // may be null
  const uint32_t* owned_ids;  // list-sharded index: ascending ids of the kept vectors (row s of `vectors`); else null
  uint32_t owned_n;
  int shard_rank, shard_world;  // this shard scans the probed lists l with l % world == rank
  int metric, pd, m, dsub, nprobe, keep, k;
  int refine;        // 1: re-rank the kept candidates exactly
  int np;            // producer warps (L2 with precomputed tables)
  int cap;           // keys of the block's candidate buffer (a power of two, >= keep + 2 * threads)
  int candidates;    // 1: write the kept candidates with both distances instead of the final k
  uint32_t id_base;
  u64* out_keys;             // nq x k        (candidates == 0)
  fv_neighbor* out_adc;      // nq x keep     (candidates == 1)
  float* out_exact;          // nq x keep
  uint32_t* out_counts;      // nq
  unsigned long long* rows_scanned;
  const uint32_t* qids;      // block b works on query qids[b] (null: query b)
  uint32_t nlist, nrows, nvec;  // extents (lists, rows in all lists, kept vectors), for the checks of the debug build
  // Bound mode (bound_out != null): only the nearest probed lists are scanned, until they hold row_budget rows, and
  // instead of results the query's keep-th best compressed distance over those rows goes to bound_out[q] as its
  // order bits (0xFFFFFFFF when they hold fewer than keep rows): an upper bound for the list-major passes.
  uint32_t row_budget;
  uint32_t* bound_out;
};

// The query's part of the lookup tables for a whole batch (ivfpq.rs:236-238 inner product, :241-251 L2 with
// precomputed tables): entry (j, e) = -dot(q_j, w_je) or -2 dot(q_j, w_je), the products summed in index order from
// -0.0 as the reference's iterator sum does.  One block per (16 queries, sub-quantizer), one thread per entry: the
// codebook is read once per 16 queries instead of once per query.
template <int DSUB>  // 0: any sub-vector length; otherwise the codebook entry is held in registers
__global__ void __launch_bounds__(256) query_tables_kernel(const float* __restrict__ queries, size_t nq, int pd,
                                                           const float* __restrict__ codebooks, int m, int dsub,
                                                           int is_ip, float* __restrict__ out) {
  unsigned char* smem_raw = dyn_smem();
  float* sqs = reinterpret_cast<float*>(smem_raw);  // [16][dsub]
  const int j = blockIdx.y, e = threadIdx.x;
  const size_t q0 = size_t(blockIdx.x) * 16;
  for (int i = threadIdx.x; i < 16 * dsub; i += blockDim.x) {
    const size_t qi = q0 + i / dsub;
    sqs[i] = qi < nq ? queries[qi * size_t(pd) + j * dsub + (i % dsub)] : 0.f;
  }
  __syncthreads();
  const float* wv = codebooks + (size_t(j) * KSUB + e) * dsub;
  const size_t tab = size_t(m) * KSUB;
  float wr[DSUB > 0 ? DSUB : 1];
  if (DSUB > 0) {
#pragma unroll
    for (int t = 0; t < DSUB; ++t) wr[t] = __ldg(wv + t);
  }
  for (int qi = 0; qi < 16 && q0 + qi < nq; ++qi) {
    float s = -0.0f;
    if (DSUB > 0) {
#pragma unroll
      for (int t = 0; t < DSUB; ++t) s = __fadd_rn(s, __fmul_rn(sqs[qi * DSUB + t], wr[t]));
    } else {
      for (int t = 0; t < dsub; ++t) s = __fadd_rn(s, __fmul_rn(sqs[qi * dsub + t], __ldg(wv + t)));
    }
    out[(q0 + qi) * tab + size_t(j) * KSUB + e] = is_ip ? -s : __fmul_rn(-2.0f, s);
  }
}

// Entry (code byte J) of sub-quantizer J's table.  `w` is the 32-bit word of the code that holds byte J, `lut_s` the
// shared-memory address of the tables (a multiple of 1024): the byte, times 4, is moved into bits 2..9 by one shift,
// masked and OR-ed onto the address by one logic op, and the table's offset J * 1024 rides in the load.
template <int J>
__device__ __forceinline__ float lut_entry(uint32_t w, uint32_t lut_s) {
  const uint32_t sh = (J & 3) == 0 ? (w << 2) : (w >> ((J & 3) * 8 - 2));
  const uint32_t addr = (sh & 0x3FCu) | lut_s;
  float t;
  asm volatile("ld.shared.f32 %0, [%1 + %2];" : "=f"(t) : "r"(addr), "n"(J * 1024));
  return t;
}

// What follows the scan of a query, for both kernels: `cand` holds the query's best a.keep keys by (compressed
// distance, id), ascending, padded with FV_EMPTY_KEY; `rerank` has room for a.keep + a.k keys; `sq` is the padded
// query.  Writes the final k keys, or (candidates mode) the kept candidates with both distances and their count
// (ivfpq.rs:285-296).  Called by every thread of the block.
__device__ __forceinline__ void scan_tail(const ScanArgs& a, size_t q, const u64* cand, u64* rerank, const float* sq) {
  const int W = blockDim.x >> 5, w = threadIdx.x >> 5, lane = threadIdx.x & 31, tid = threadIdx.x;
  if (a.bound_out) {
    if (tid == 0) a.bound_out[q] = cand[a.keep - 1] == FV_EMPTY_KEY ? 0xFFFFFFFFu : uint32_t(cand[a.keep - 1] >> 32);
    return;
  }
  if (!a.refine && !a.candidates) {
    for (int e = tid; e < a.k; e += blockDim.x) a.out_keys[q * size_t(a.k) + e] = e < a.keep ? cand[e] : FV_EMPTY_KEY;
    return;
  }
  // exact distances of the kept candidates
  for (int e = tid; e < a.keep; e += blockDim.x) {
    const u64 c = cand[e];
    u64 rk = FV_EMPTY_KEY;
    float ex = INFINITY;
    if (c != FV_EMPTY_KEY) {
      const uint32_t id = key_id(c);
      size_t slot = size_t(id - a.id_base);
      if (a.owned_ids) {  // position of the id among the ids this shard keeps (ascending)
        uint32_t lo = 0, hi = a.owned_n;
        while (lo < hi) {
          const uint32_t mid = (lo + hi) >> 1;
          if (a.owned_ids[mid] < id) lo = mid + 1;
          else hi = mid;
        }
        slot = lo;
      }
      if (FV_IDX_OK(slot, a.nvec, 3)) {
        ex = exact_distance(a.metric, sq, a.vectors + slot * a.pd, a.pd);
        rk = make_key(ex, id);
      }
    }
    rerank[e] = rk;
    if (a.candidates) {
      fv_neighbor nb;
      nb.id = c == FV_EMPTY_KEY ? 0xFFFFFFFFu : key_id(c);
      nb.distance = c == FV_EMPTY_KEY ? INFINITY : key_distance(c);
      a.out_adc[q * size_t(a.keep) + e] = nb;
      a.out_exact[q * size_t(a.keep) + e] = ex;
    }
  }
  if (a.candidates) {
    if (w == 0) {
      int cnt = 0;
      for (int e0 = 0; e0 < a.keep; e0 += 32)
        cnt += __popc(__ballot_sync(FV_FULL, (e0 + lane) < a.keep && cand[e0 + lane] != FV_EMPTY_KEY));
      if (lane == 0) a.out_counts[q] = uint32_t(cnt);
    }
    return;
  }
  __syncthreads();
  if (w == 1 || W == 1) {  // a second list of k entries behind the re-ranked keys
    u64* fin = rerank + a.keep;
    warp_list_init(fin, a.k);
    u64 b2 = FV_EMPTY_KEY;
    for (int e0 = 0; e0 < a.keep; e0 += 32) {
      const int e = e0 + lane;
      b2 = warp_list_offer(fin, a.k, e < a.keep ? rerank[e] : FV_EMPTY_KEY, b2);
    }
    __syncwarp();
    for (int e = lane; e < a.k; e += 32) a.out_keys[q * size_t(a.k) + e] = fin[e];
  }
}

template <bool M16, int R>
__global__ void __launch_bounds__(256, 4) ivfpq_scan_kernel(ScanArgs a) {
  unsigned char* smem_raw = dyn_smem();
  const int W = blockDim.x >> 5, w = threadIdx.x >> 5, lane = threadIdx.x & 31, tid = threadIdx.x;
  const int tab = a.m * int(KSUB);
  const bool use_pre = a.metric == FV_L2 && a.pre != nullptr;
  // The lookup tables first: their shared-memory addresses are multiples of 1024, so a lookup address is formed by
  // OR.  With precomputed tables there are two: NP producer warps build the next cell's table (pre[l] + the query's
  // own table, both read from L2) while the other warps scan the current cell with the other one, so the L2 round
  // trips of the build are off the scan's critical path and one barrier per cell is enough.
  float* lut0 = reinterpret_cast<float*>(smem_raw);   // tab
  float* lut1 = lut0 + tab;                           // tab (L2 with tables only)
  float* sq = lut1 + (use_pre ? tab : 0);             // pd
  float* srq = sq + a.pd;                             // pd
  // Candidates: ONE unsorted buffer for the block.  A row whose key is below the bound is appended (a shared-memory
  // counter hands out the slots); when the count passes `compact_at`, the block sorts the buffer, keeps the best
  // `keep` and takes the keep-th key as the new bound.  One list per block sees every row, so its bound is the
  // tightest the scan order allows (lists per warp each converged on the best of their own eighth and let 5-8x
  // more rows in).
  u64* lists = reinterpret_cast<u64*>(srq + a.pd);  // cap keys, then keep keys for the re-rank, then k
  u64* rerank = lists + a.cap;
  const size_t q = a.qids ? size_t(a.qids[blockIdx.x]) : size_t(blockIdx.x);
  const int NP = use_pre ? a.np : 0;    // producer warps
  const int WC = W - NP, cw = w - NP;   // consumer warps; this warp's index among them (negative: a producer)
  const float* qtab = a.qtab ? a.qtab + q * size_t(tab) : nullptr;

  for (int c = tid; c < a.pd; c += blockDim.x) sq[c] = a.queries[q * size_t(a.pd) + c];
  __shared__ int shared_count;  // keys in the buffer
  if (tid == 0) shared_count = 0;
  // inner product: the query's own table IS the lookup table (ivfpq.rs:236-238, :307)
  if (a.metric == FV_INNER_PRODUCT)
    for (int i = tid; i < tab / 4; i += blockDim.x)
      reinterpret_cast<float4*>(lut0)[i] = __ldg(reinterpret_cast<const float4*>(qtab) + i);
  __syncthreads();

  u64 bound = FV_EMPTY_KEY;  // the keep-th best key at the last compaction
  // Sorts the buffer, keeps the best `keep`, refreshes the bound.  Every thread calls it at a point where no append
  // is in flight (right after a barrier every appending warp has passed); on return appends may resume at once.
  auto compact = [&]() {
    const int cnt = shared_count;
    int n = 32;
    while (n < cnt) n <<= 1;
    for (int e = cnt + tid; e < n; e += blockDim.x) lists[e] = FV_EMPTY_KEY;
    __syncthreads();
    block_sort(lists, n);
    const int kept = min(cnt, a.keep);
    if (kept == a.keep) bound = lists[a.keep - 1];  // appends go behind it: it stays put
    if (tid == 0) shared_count = kept;
    __syncthreads();
    return kept;
  };
  const int chunk_rows = WC * 32;  // rows the consumers scan per step: the most one step can append
  // Compacting early and often keeps the bound tight (the sort is over the next power of two above the count, so a
  // small buffer sorts fast).  `seen` is the highest count this warp's own appends have produced; the barrier that
  // ends a piece ORs "seen >= compact_at" over the block, so all threads agree on compacting without reading the
  // counter while others may already be appending again.  `cnt_ub` bounds the count from above for sizing a piece.
  const int compact_at = min(a.cap - chunk_rows, 2 * a.keep + 64);
  int seen = 0, cnt_ub = 0, rows_seen = 0;
  auto piece_barrier = [&]() {
    if (__syncthreads_or(seen >= compact_at)) {
      cnt_ub = compact();
      seen = 0;
    } else {
      cnt_ub = compact_at - 1;
    }
  };
  unsigned long long scanned = 0;
  // the next probed cell this block scans (a list-sharded index skips the other shards' lists), or -1
  uint32_t budget_used = 0;  // bound mode: rows of the lists taken so far (the same in every thread)
  auto next_probe = [&](int p) {
    for (++p; p < a.nprobe; ++p) {
      const u64 c = a.cells[q * size_t(a.nprobe) + p];
      if (c == FV_EMPTY_KEY) return -1;
      if (a.shard_world > 1 && int(key_id(c) % uint32_t(a.shard_world)) != a.shard_rank) continue;
      if (!FV_IDX_OK(key_id(c), a.nlist, 1)) continue;
      if (a.row_budget) {
        if (budget_used >= a.row_budget) return -1;
        budget_used += a.list_off[key_id(c) + 1] - a.list_off[key_id(c)];
      }
      return p;
    }
    return -1;
  };
  // table of cell l with precomputed tables (ivfpq.rs:256-262), by `nthr` threads of which this is number `t`
  auto build_pre = [&](float* dst, uint32_t l, int t, int nthr) {
    const float4* pre = reinterpret_cast<const float4*>(a.pre + size_t(l) * tab);
    const float4* qt = reinterpret_cast<const float4*>(qtab);
#pragma unroll 8
    for (int i = t; i < tab / 4; i += nthr) {
      const float4 x = __ldg(pre + i), y = __ldg(qt + i);
      reinterpret_cast<float4*>(dst)[i] =
          make_float4(__fadd_rn(x.x, y.x), __fadd_rn(x.y, y.y), __fadd_rn(x.z, y.z), __fadd_rn(x.w, y.w));
    }
  };

  int p = next_probe(-1);
  int cur = 0;  // which table the scan reads
  if (use_pre && p >= 0) {
    build_pre(lut0, key_id(a.cells[q * size_t(a.nprobe) + p]), tid, int(blockDim.x));
    __syncthreads();
  }
  while (p >= 0) {
    const u64 cell = a.cells[q * size_t(a.nprobe) + p];
    const uint32_t l = key_id(cell);
    const size_t off = a.list_off[l];
    const int len = int(a.list_off[l + 1] - off);
    const int pnext = next_probe(p);
    float* lut = cur ? lut1 : lut0;
    float base;
    if (use_pre) {
      base = key_distance(cell);
      if (cw < 0 && pnext >= 0)  // producers: the next cell's table, into the other buffer
        build_pre(cur ? lut0 : lut1, key_id(a.cells[q * size_t(a.nprobe) + pnext]), tid, NP * 32);
    } else if (a.metric == FV_L2) {  // ivfpq.rs:263-269
      const float* cen = a.centroids + size_t(l) * a.pd;
      for (int c = tid; c < a.pd; c += blockDim.x) srq[c] = __fsub_rn(sq[c], cen[c]);
      __syncthreads();
      for (int i = tid; i < tab; i += blockDim.x) {
        const int j = i >> 8;
        const float* wv = a.codebooks + size_t(i) * a.dsub;
        float s = -0.0f;
        for (int t = 0; t < a.dsub; ++t) {
          const float d = __fsub_rn(srq[j * a.dsub + t], __ldg(wv + t));
          s = __fadd_rn(s, __fmul_rn(d, d));
        }
        lut[i] = s;
      }
      base = 0.0f;
      __syncthreads();
    } else {
      base = key_distance(cell);  // -dot(q, centroid), the same chain as ivfpq.rs:270
    }
    const uint32_t lut_s = uint32_t(__cvta_generic_to_shared(lut));
    if (tid == 0) scanned += len;
    // The list is scanned in pieces that cannot overflow the buffer even if every row is appended; every piece ends
    // with the barrier that decides about compaction (the last one also hands the tables over).
    for (int done = 0; done < len || done == 0;) {
      const u64 eff = bound;
      const uint32_t eff_hi = uint32_t(eff >> 32);
      // The first pieces of a query are short (two steps, then as many rows as were scanned so far): until a bound
      // exists every row is appended, so it pays to sort a few hundred keys early and scan the rest against a bound.
      const int piece = min(((a.cap - cnt_ub) / chunk_rows) * chunk_rows, max(2 * chunk_rows, rows_seen));
      const int end = min(len, done + piece);
      if (cw >= 0) {
        // R rows per lane and step: their 16-step add chains are independent and interleave
        for (int r0 = done + cw * (32 * R); r0 < end; r0 += WC * 32 * R) {
          float d[R];
          bool pass[R];
          uint32_t cws[R][4];
#pragma unroll
          for (int i = 0; i < R; ++i) {
            const int r = r0 + i * 32 + lane;
            d[i] = base;  // ivfpq.rs:273-276: base first, then the m table entries in order
            pass[i] = false;
            if (M16) {
              uint4 cwv = make_uint4(0u, 0u, 0u, 0u);
              if (r < end) cwv = __ldg(reinterpret_cast<const uint4*>(a.codes + (off + r) * 16));
              cws[i][0] = cwv.x;
              cws[i][1] = cwv.y;
              cws[i][2] = cwv.z;
              cws[i][3] = cwv.w;
            }
          }
          if (M16) {
            // byte j of the code, times 4, OR the table's shared address: one shift and one logic op per lookup
#define FV_ADC_STEP(J)                                                              \
  _Pragma("unroll") for (int i = 0; i < R; ++i) d[i] = __fadd_rn(d[i], lut_entry<J>(cws[i][(J) >> 2], lut_s));
            FV_ADC_STEP(0) FV_ADC_STEP(1) FV_ADC_STEP(2) FV_ADC_STEP(3) FV_ADC_STEP(4) FV_ADC_STEP(5)
            FV_ADC_STEP(6) FV_ADC_STEP(7) FV_ADC_STEP(8) FV_ADC_STEP(9) FV_ADC_STEP(10) FV_ADC_STEP(11)
            FV_ADC_STEP(12) FV_ADC_STEP(13) FV_ADC_STEP(14) FV_ADC_STEP(15)
#undef FV_ADC_STEP
          } else {
#pragma unroll
            for (int i = 0; i < R; ++i) {
              const int r = r0 + i * 32 + lane;
              if (r < end) {
                const uint8_t* code = a.codes + (off + r) * size_t(a.m);
                for (int j = 0; j < a.m; ++j) d[i] = __fadd_rn(d[i], lut[j * 256 + code[j]]);
              }
            }
          }
#pragma unroll
          for (int i = 0; i < R; ++i) {
            const int r = r0 + i * 32 + lane;
            // the distance alone decides for almost every row; the id is fetched only when it can matter
            pass[i] = r < end && d[i] < INFINITY && order_bits(d[i]) <= eff_hi;
          }
#pragma unroll
          for (int i = 0; i < R; ++i) {
            if (__any_sync(FV_FULL, pass[i])) {
              const int r = r0 + i * 32 + lane;
              u64 key = FV_EMPTY_KEY;
              if (pass[i] && FV_IDX_OK(off + r, a.nrows, 2)) key = make_key(d[i], __ldg(a.ids + off + r));
              const bool in = key < eff;
              const unsigned hit = __ballot_sync(FV_FULL, in);
              if (hit) {
                int slot = 0;
                if (lane == 0) slot = atomicAdd(&shared_count, __popc(hit));
                slot = __shfl_sync(FV_FULL, slot, 0);
                if (in) lists[slot + __popc(hit & ((1u << lane) - 1u))] = key;
                seen = max(seen, slot + __popc(hit));
              }
            }
          }
        }
      }
      rows_seen += end - done;
      done = end;
      piece_barrier();
      if (len == 0) break;
    }
    p = pnext;
    cur = use_pre ? cur ^ 1 : 0;
  }
  if (tid == 0 && a.rows_scanned) atomicAdd(a.rows_scanned, scanned);

  cnt_ub = compact();  // the best `keep` by (compressed distance, id), ascending, at the front of the buffer
  for (int e = cnt_ub + tid; e < a.keep; e += blockDim.x) lists[e] = FV_EMPTY_KEY;
  __syncthreads();
  scan_tail(a, q, lists, rerank, sq);
}


// ================================================================================================
// The list-major scan.

static constexpr int LS_THREADS = 512;                     // 16 warps, one block per SM
static constexpr int LS_WARPS = LS_THREADS / 32;
static constexpr int LS_NG = 4;                            // row groups (16 rows each) per warp: 64 partial sums per thread
static constexpr int LS_CH = LS_WARPS * LS_NG * 16;        // rows of a list one task covers: 1024
static constexpr int LS_STRIDE = 36;                       // words per table entry: 32 query slots + 4, so that 16-byte stores
                                                           // of eight consecutive entries cover all banks
static constexpr int LS_SLICE = 256 * LS_STRIDE;           // words of one sub-quantizer's entry-major slice
static constexpr int LS_STAGE = 32 * 256;                  // words of one staging buffer: 32 queries x 256 raw entries
static constexpr int LS_GB = 4;                            // query groups per task
static constexpr size_t LS_SMEM = size_t(2 * LS_SLICE + 2 * LS_STAGE) * 4 + size_t(16) * LS_CH;

// How a list of `len` rows probed by `npairs` queries of the batch becomes tasks: equal row chunks of at most LS_CH
// rows (multiples of 16) times blocks of LS_GB query groups.
__host__ __device__ __forceinline__ uint32_t ls_chunks(uint32_t len) { return (len + LS_CH - 1) / LS_CH; }
__host__ __device__ __forceinline__ uint32_t ls_chunk_rows(uint32_t len) {
  const uint32_t n = ls_chunks(len);
  return n ? ((len + n - 1) / n + 15) / 16 * 16 : 0;
}
__host__ __device__ __forceinline__ uint32_t ls_group_blocks(uint32_t npairs) {
  return ((npairs + 31) / 32 + LS_GB - 1) / LS_GB;
}
__host__ __device__ __forceinline__ uint32_t ls_tasks(uint32_t len, uint32_t npairs) {
  return (len && npairs) ? ls_chunks(len) * ls_group_blocks(npairs) : 0u;
}

// counters (u32 words): 0 next task, 1 number of tasks, 2 queries whose buffer overflowed, 3 number of pairs
// 4 queries left to the per-query kernel
enum { LS_C_NEXT = 0, LS_C_TASKS = 1, LS_C_OVER = 2, LS_C_PAIRS = 3, LS_C_RERUN = 4, LS_NCOUNTERS = 8 };

__device__ __forceinline__ void cp_async16(void* dst_smem, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(uint32_t(__cvta_generic_to_shared(dst_smem))), "l"(src)
               : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

struct PairArgs {
  const u64* cells;
  size_t nq;
  int nprobe, shard_rank, shard_world;
  uint32_t nlist;       // lists of the index (the debug build checks the probed cells against it)
  uint32_t min_rows;    // 0: every probed list this shard owns; else only the nearest ones, until they hold this many rows
  const uint32_t* list_off;
  uint32_t* pair_cnt;   // nlist (zeroed): pairs per list
  uint32_t* cursor;     // nlist (zeroed)
  const uint32_t* pair_off;
  uint2* pairs;         // (query, the f32 cell distance as bits)
  uint32_t* slot_of;    // pair_flat_kernel: nq x nprobe, the place of every (query, probe) within its list
};

// One thread per query: its probes counted per list (FILL = false) or filed under their list (FILL = true).
// The order of a list's pairs is whatever the atomics give; results do not depend on it.
template <bool FILL>
__global__ void pair_kernel(PairArgs a) {
  const size_t q = blockIdx.x * size_t(blockDim.x) + threadIdx.x;
  if (q >= a.nq) return;
  uint32_t rows = 0;
  for (int p = 0; p < a.nprobe; ++p) {
    const u64 c = a.cells[q * size_t(a.nprobe) + p];
    if (c == FV_EMPTY_KEY) break;
    const uint32_t l = key_id(c);
    if (a.shard_world > 1 && int(l % uint32_t(a.shard_world)) != a.shard_rank) continue;
    if (!FV_IDX_OK(l, a.nlist, 4)) continue;
    if (a.min_rows) {
      if (rows >= a.min_rows) break;
      rows += a.list_off[l + 1] - a.list_off[l];
    }
    if (FILL) {
      const uint32_t slot = atomicAdd(a.cursor + l, 1u);
      a.pairs[a.pair_off[l] + slot] = make_uint2(uint32_t(q), __float_as_uint(key_distance(c)));
    } else {
      atomicAdd(a.pair_cnt + l, 1u);
    }
  }
}

// The same for ALL probed lists of this shard (no row budget), one thread per (query, probe); the counting pass
// remembers the place its atomic handed out, so the filing pass needs none.  The threads are numbered probe rank
// first (all queries' nearest cell, then all second nearest, ...), so that a list's pairs come out roughly in order of
// probe rank: the pairs that will let many rows through (a query meeting one of its nearest lists) sit together in
// the first operand tiles and warps of a list, and the epilogue warps that hold only far pairs keep to their fast
// path (with the pairs in query order the tensor-core pass measured 0.51 instead of 0.41 ms).
template <bool FILL>
__global__ void pair_flat_kernel(PairArgs a) {
  const size_t i = blockIdx.x * size_t(blockDim.x) + threadIdx.x;
  if (i >= a.nq * size_t(a.nprobe)) return;
  const size_t p = i / a.nq, q = i - p * a.nq;
  const u64 c = a.cells[q * size_t(a.nprobe) + p];
  if (c == FV_EMPTY_KEY) return;
  const uint32_t l = key_id(c);
  if (a.shard_world > 1 && int(l % uint32_t(a.shard_world)) != a.shard_rank) return;
  if (!FV_IDX_OK(l, a.nlist, 4)) return;
  if (FILL) {
    a.pairs[a.pair_off[l] + a.slot_of[i]] = make_uint2(uint32_t(q), __float_as_uint(key_distance(c)));
  } else {
    a.slot_of[i] = atomicAdd(a.pair_cnt + l, 1u);
  }
}

// One block: exclusive prefix sums over the lists of the pair counts and of the task counts.
__global__ void __launch_bounds__(1024) pair_offsets_kernel(const uint32_t* __restrict__ pair_cnt,
                                                            const uint32_t* __restrict__ list_off, size_t nlist,
                                                            uint32_t* __restrict__ pair_off, uint32_t* __restrict__ task_off,
                                                            uint32_t* __restrict__ counters) {
  __shared__ uint32_t sp[1024], st[1024];
  const int tid = threadIdx.x;
  const size_t per = (nlist + 1023) / 1024;
  const size_t l0 = min(nlist, size_t(tid) * per), l1 = min(nlist, l0 + per);
  uint32_t np = 0, nt = 0;
  for (size_t l = l0; l < l1; ++l) {
    np += pair_cnt[l];
    nt += ls_tasks(list_off[l + 1] - list_off[l], pair_cnt[l]);
  }
  sp[tid] = np;
  st[tid] = nt;
  __syncthreads();
  for (int o = 1; o < 1024; o <<= 1) {  // inclusive scan
    const uint32_t a = tid >= o ? sp[tid - o] : 0u, b = tid >= o ? st[tid - o] : 0u;
    __syncthreads();
    sp[tid] += a;
    st[tid] += b;
    __syncthreads();
  }
  uint32_t bp = sp[tid] - np, bt = st[tid] - nt;  // exclusive
  for (size_t l = l0; l < l1; ++l) {
    pair_off[l] = bp;
    task_off[l] = bt;
    bp += pair_cnt[l];
    bt += ls_tasks(list_off[l + 1] - list_off[l], pair_cnt[l]);
  }
  if (tid == 1023) {
    pair_off[nlist] = sp[1023];
    task_off[nlist] = st[1023];
    counters[LS_C_TASKS] = st[1023];
    counters[LS_C_PAIRS] = sp[1023];
  }
}

struct ListScanArgs {
  const float* qtab;           // nq x 16 x 256
  const float* pre;            // nlist x 16 x 256 (HAS_PRE)
  const uint32_t* list_off;
  const uint32_t* off16;
  const uint8_t* codes_t;
  const uint32_t* ids;
  const uint32_t* pair_off;
  const uint32_t* task_off;
  const uint2* pairs;
  uint32_t nlist;
  uint32_t* counters;
  // main pass
  const uint32_t* tau_bits;    // nq: order bits of the query's bound (0xFFFFFFFF: none), rows at or below it are kept
  u64* cand;                   // nq x cap
  uint32_t* cand_cnt;          // nq (zeroed); may pass cap: the query overflowed
  int cap;
  unsigned long long* rows_scanned;
  // bound pass
  float* minima;               // nq x minima_cap
  uint32_t* minima_cnt;        // nq (zeroed)
  int minima_cap;
};

template <bool HAS_PRE, bool BOUND_PASS>
__global__ void __launch_bounds__(LS_THREADS, 1) ivfpq_list_scan_kernel(ListScanArgs a) {
  float* slice = reinterpret_cast<float*>(dyn_smem());                       // [2][LS_SLICE] entry-major tables
  float* stage = slice + 2 * LS_SLICE;                                       // [2][32][256] raw table rows
  uint8_t* codes_s = reinterpret_cast<uint8_t*>(stage + 2 * LS_STAGE);       // [16][LS_CH]
  __shared__ __align__(16) uint32_t s_q[2][32];   // the queries of the current and of the next group, by slot
  __shared__ uint32_t s_mbase[2][32];             // bound pass: where each slot's query puts this chunk's minima
  __shared__ uint32_t s_task[8];
  const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
  const int fc = tid & 255, fh = tid >> 8;        // table building: this thread's entry and its half of the slots
  const uint32_t ntasks = a.counters[LS_C_TASKS];
  unsigned long long scanned = 0;

  for (;;) {
    if (tid == 0) {
      const uint32_t t = atomicAdd(a.counters + LS_C_NEXT, 1u);
      s_task[0] = t;
      if (t < ntasks) {
        uint32_t lo = 0, hi = a.nlist;  // the list l with task_off[l] <= t < task_off[l + 1]
        while (hi - lo > 1) {
          const uint32_t mid = (lo + hi) >> 1;
          if (a.task_off[mid] <= t) lo = mid;
          else hi = mid;
        }
        const uint32_t l = lo, local = t - a.task_off[l];
        const uint32_t npair = a.pair_off[l + 1] - a.pair_off[l];
        const uint32_t len = a.list_off[l + 1] - a.list_off[l];
        const uint32_t ngb = ls_group_blocks(npair);
        s_task[1] = l;
        s_task[2] = (local / ngb) * ls_chunk_rows(len);   // first row of the chunk
        s_task[3] = (local % ngb) * LS_GB;                // first query group
      }
    }
    __syncthreads();
    if (s_task[0] >= ntasks) break;
    const uint32_t l = s_task[1], r0 = s_task[2], g0 = s_task[3];
    const uint32_t pbase = a.pair_off[l], npair = a.pair_off[l + 1] - pbase;
    const uint32_t loff = a.list_off[l], len = a.list_off[l + 1] - loff;
    const int nrows = r0 < len ? int(min(len - r0, ls_chunk_rows(len))) : 0;  // (rounding can leave a last chunk empty)
    const int rows_pad = (nrows + 15) & ~15;
    const int ngroups = int(min(uint32_t(LS_GB), (npair + 31) / 32 - g0));
    const int total_ph = ngroups * 16;
    {  // this chunk's code bytes, sub-quantizer w by warp w
      const uint32_t len16 = a.off16[l + 1] - a.off16[l];
      const uint4* src = reinterpret_cast<const uint4*>(a.codes_t + size_t(a.off16[l]) * 16 + size_t(w) * len16 + r0);
      uint4* dst = reinterpret_cast<uint4*>(codes_s + w * LS_CH);
      for (int v = lane; v < rows_pad / 16; v += 32) dst[v] = __ldg(src + v);
    }
    // the pair of slot `lane` of group g: (query, base distance, slot in use)
    uint32_t q_cur, q_nxt = 0;
    float base_cur, base_nxt = 0.f;
    bool valid_cur, valid_nxt = false;
    auto load_pair = [&](uint32_t g, uint32_t& qo, float& bo, bool& vo) {
      const uint32_t i = g * 32 + lane;
      vo = i < npair;
      const uint2 pr = a.pairs[pbase + (vo ? i : g * 32)];  // an unused slot repeats the group's first query
      qo = pr.x;
      bo = __uint_as_float(pr.y);
    };
    load_pair(g0, q_cur, base_cur, valid_cur);
    if (w == 0) s_q[0][lane] = q_cur;
    __syncthreads();

    // Phase P of the task = (group P / 16, sub-quantizer P % 16).  Its raw table rows travel to staging[P & 1] by
    // cp.async (thread t: 16 bytes of the rows of four queries), issued during phase P - 2 ...
    auto stage_issue = [&](int P) {
      const int fj = P & 15;
      float* dst = stage + (P & 1) * LS_STAGE + (tid & 63) * 4;
      const float* src = a.qtab + fj * 256 + (tid & 63) * 4;
      const uint32_t* sq = s_q[(P >> 4) & 1];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int slot = (tid >> 6) + 8 * i;
        cp_async16(dst + slot * 256, src + size_t(sq[slot]) * 4096);
      }
      cp_async_commit();
    };
    // ... and become quarter `pc` of slice P & 1 during phase P - 1: entry fc of four queries, + pre[l]'s entry
    auto build_slice = [&](int P, int pc, float prev) {
      const float* src = stage + (P & 1) * LS_STAGE + (fh * 16 + pc * 4) * 256 + fc;
      float4 o = make_float4(src[0], src[256], src[512], src[768]);
      if (HAS_PRE) o = make_float4(__fadd_rn(prev, o.x), __fadd_rn(prev, o.y), __fadd_rn(prev, o.z), __fadd_rn(prev, o.w));
      *reinterpret_cast<float4*>(slice + (P & 1) * LS_SLICE + fc * LS_STRIDE + fh * 16 + pc * 4) = o;
    };
    const float* pre_l = HAS_PRE ? a.pre + size_t(l) * 4096 + fc : nullptr;
    stage_issue(0);
    stage_issue(1);
    float prev_nxt = HAS_PRE ? __ldg(pre_l + 256) : 0.f;  // pre[l]'s entry for the slice built during the next phase
    {
      const float prev = HAS_PRE ? __ldg(pre_l) : 0.f;
      cp_async_wait_all();
      __syncthreads();
#pragma unroll
      for (int pc = 0; pc < 4; ++pc) build_slice(0, pc, prev);
    }
    __syncthreads();

    for (int gi = 0; gi < ngroups; ++gi) {
      float acc[LS_NG][16];
#pragma unroll
      for (int g = 0; g < LS_NG; ++g)
#pragma unroll
        for (int i = 0; i < 16; ++i) acc[g][i] = base_cur;  // ivfpq.rs:273: the distance starts at the cell's base
      if (gi + 1 < ngroups) {
        load_pair(g0 + gi + 1, q_nxt, base_nxt, valid_nxt);
        if (w == 0) s_q[(gi + 1) & 1][lane] = q_nxt;  // read from phase 14 on: many barriers away
      }
      if (BOUND_PASS && w == 0 && valid_cur) s_mbase[gi & 1][lane] = atomicAdd(a.minima_cnt + q_cur, uint32_t(rows_pad / 8));
#pragma unroll 1
      for (int j = 0; j < 16; ++j) {
        const int P = gi * 16 + j;
        const bool has1 = P + 1 < total_ph, has2 = P + 2 < total_ph;
        if (has2) stage_issue(P + 2);  // into the staging buffer that slice P was built from, one phase ago
        const float prev = prev_nxt;
        if (HAS_PRE && has2) prev_nxt = __ldg(pre_l + ((j + 2) & 15) * 256);
        const float* tb = slice + (j & 1) * LS_SLICE + lane;
#pragma unroll
        for (int g = 0; g < LS_NG; ++g) {
          const int G = g * LS_WARPS + w;
          if (G * 16 < rows_pad) {
            const uint4 cw = *reinterpret_cast<const uint4*>(codes_s + j * LS_CH + G * 16);
            const uint32_t cws[4] = {cw.x, cw.y, cw.z, cw.w};
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              const uint32_t c = (cws[i >> 2] >> ((i & 3) * 8)) & 0xFFu;
              acc[g][i] = __fadd_rn(acc[g][i], tb[c * LS_STRIDE]);
            }
          }
          if (has1) build_slice(P + 1, g, prev);
        }
        cp_async_wait_all();
        __syncthreads();
      }
      if (BOUND_PASS) {
        // the minimum of every 8 rows (rows beyond the chunk count as +inf), two per thread and row group
        if (valid_cur) {
          const uint32_t mb = s_mbase[gi & 1][lane];
          {
            // every slot below min(count, capacity) gets written: the selection reads exactly those
            float* dst = a.minima + size_t(q_cur) * a.minima_cap + mb;
#pragma unroll
            for (int g = 0; g < LS_NG; ++g) {
              const int G = g * LS_WARPS + w;
              if (G * 16 < rows_pad && mb + uint32_t(G * 2) < uint32_t(a.minima_cap)) {
                float m0 = INFINITY, m1 = INFINITY;
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                  m0 = fminf(m0, (G * 16 + i < nrows) ? acc[g][i] : INFINITY);
                  m1 = fminf(m1, (G * 16 + 8 + i < nrows) ? acc[g][8 + i] : INFINITY);
                }
                *reinterpret_cast<float2*>(dst + G * 2) = make_float2(m0, m1);
              }
            }
          }
        }
      } else {
        // rows at or below the query's bound become candidates
        const uint32_t tbits = a.tau_bits[q_cur];
        const float tau_d = tbits == 0xFFFFFFFFu ? INFINITY : order_bits_to_float(tbits);
        const uint32_t nvalid = min(32u, npair - (g0 + gi) * 32);
        if (tid == 0) scanned += (unsigned long long)nrows * nvalid;
        // a buffer that has run over is not fed any further: the per-query kernel re-runs that query anyway
        if (valid_cur && a.cand_cnt[q_cur] <= uint32_t(a.cap)) {
#pragma unroll
          for (int g = 0; g < LS_NG; ++g) {
            const int G = g * LS_WARPS + w;
            if (G * 16 < nrows) {
              float mn = acc[g][0];
#pragma unroll
              for (int i = 1; i < 16; ++i) mn = fminf(mn, acc[g][i]);
              if (mn <= tau_d) {
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                  const int row = G * 16 + i;
                  const float d = acc[g][i];
                  if (d <= tau_d && d < INFINITY && row < nrows && order_bits(d) <= tbits) {
                    const uint32_t slot = atomicAdd(a.cand_cnt + q_cur, 1u);
                    if (slot < uint32_t(a.cap))
                      a.cand[size_t(q_cur) * a.cap + slot] = make_key(d, __ldg(a.ids + loff + r0 + row));  // (row < len by construction)
                  }
                }
              }
            }
          }
        }
      }
      q_cur = q_nxt;
      base_cur = base_nxt;
      valid_cur = valid_nxt;
    }
  }
  if (!BOUND_PASS && tid == 0 && a.rows_scanned && scanned) atomicAdd(a.rows_scanned, scanned);
}

// One warp per query: the keep-th smallest of the minima its bound pass left, as order bits (0xFFFFFFFF when there
// are fewer than `keep` finite ones).  At least `keep` different rows of the query's probed lists reach it.
__global__ void __launch_bounds__(128) bound_select_kernel(const float* __restrict__ minima,
                                                           const uint32_t* __restrict__ minima_cnt, int minima_cap,
                                                           int keep, size_t nq, uint32_t* __restrict__ tau_bits) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  const size_t q = blockIdx.x * size_t(blockDim.x >> 5) + w;
  if (q >= nq) return;
  uint32_t* v = reinterpret_cast<uint32_t*>(dyn_smem()) + size_t(w) * minima_cap;  // order-bit words
  const int n = int(min(minima_cnt[q], uint32_t(minima_cap)));
  const uint32_t INF_BITS = 0xFF800000u;  // order bits of +inf; NaNs sort above it
  int finite = 0;
  for (int i = lane; i < n; i += 32) {
    const uint32_t b = order_bits(minima[q * size_t(minima_cap) + i]);
    v[i] = b;
    finite += b < INF_BITS ? 1 : 0;
  }
  __syncwarp();
  if (__reduce_add_sync(FV_FULL, finite) < keep) {
    if (lane == 0) tau_bits[q] = 0xFFFFFFFFu;
    return;
  }
  uint32_t lo = 0, hi = INF_BITS - 1;  // the smallest T with at least `keep` values <= T
  while (lo < hi) {
    const uint32_t mid = lo + ((hi - lo) >> 1);
    int c = 0;
    for (int i = lane; i < n; i += 32) c += v[i] <= mid ? 1 : 0;
    if (__reduce_add_sync(FV_FULL, c) >= keep) hi = mid;
    else lo = mid + 1;
  }
  if (lane == 0) tau_bits[q] = lo;
}

// Bound from the tensor-core scores.  The minima variant of the kernel left, per (query, near list) pair, the smallest
// score of every 32 rows; score + add[row] is an upper bound of the compressed distance of the row that attains it.
// One warp per query collects those bounds over its pairs; their keep-th smallest is a distance that at least `keep`
// different rows of the query's probed lists do not exceed.
__global__ void __launch_bounds__(128) tc_bound_select_kernel(const float* __restrict__ minima, const uint4* __restrict__ tasks,
                                                              const uint32_t* __restrict__ tile_task0,
                                                              const uint32_t* __restrict__ task_moff,
                                                              const uint32_t* __restrict__ task_rows,
                                                              const float* __restrict__ add, const uint32_t* __restrict__ q_rows,
                                                              const uint32_t* __restrict__ q_cnt, int q_slots, int vcap,
                                                              int keep, size_t nq, uint32_t* __restrict__ tau_bits,
                                                              int tile_shift) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  const size_t q = blockIdx.x * size_t(blockDim.x >> 5) + w;
  if (q >= nq) return;
  uint32_t* v = reinterpret_cast<uint32_t*>(dyn_smem()) + size_t(w) * vcap;  // order-bit words
  const uint32_t INF_BITS = 0xFF800000u;
  const int np = int(min(q_cnt[q], uint32_t(q_slots)));
  int n = 0, finite = 0;
  uint32_t vmin = 0xFFFFFFFFu, vmax = 0u;  // over the finite bounds
  for (int s0 = 0; s0 < np && n < vcap; s0 += 32) {
    // lane i looks up pair s0 + i (one round of dependent loads for 32 pairs instead of one per pair) ...
    uint32_t my_t0 = 0, my_t1 = 0, my_rt = 0;
    float my_add = 0.f;
    // (the first two tasks of the pair's tile -- most lists are one or two segments long -- are looked up here too:
    // minima offset, or none when the pair's row lies beyond the task's rows, and the count of minima per row)
    uint32_t my_moff[2] = {0xFFFFFFFFu, 0xFFFFFFFFu};
    int my_cnt[2] = {0, 0};
    if (s0 + lane < np) {
      const uint32_t arow = q_rows[q * size_t(q_slots) + s0 + lane];
      my_rt = arow & ((1u << tile_shift) - 1u);
      my_t0 = tile_task0[arow >> tile_shift];
      my_t1 = tile_task0[(arow >> tile_shift) + 1];
      my_add = add[arow];
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        if (my_t0 + u < my_t1) {
          const uint32_t t = my_t0 + u;
          const uint32_t mo = task_moff[t], tr = task_rows[t];
          my_cnt[u] = int(tasks[t].z & 0xFFFFu) * 8;
          my_moff[u] = my_rt < tr ? mo : 0xFFFFFFFFu;
        }
      }
    }
    // ... and the warp copies their minima, one pair and one of its tile's tasks (list segments) after the other
    const int np32 = min(32, np - s0);
    for (int j = 0; j < np32 && n < vcap; ++j) {
      const uint32_t t0 = __shfl_sync(FV_FULL, my_t0, j), t1 = __shfl_sync(FV_FULL, my_t1, j);
      const uint32_t rt = __shfl_sync(FV_FULL, my_rt, j);
      const float ad = __shfl_sync(FV_FULL, my_add, j);
      const uint32_t mo0 = __shfl_sync(FV_FULL, my_moff[0], j), mo1 = __shfl_sync(FV_FULL, my_moff[1], j);
      const int cn0 = __shfl_sync(FV_FULL, my_cnt[0], j), cn1 = __shfl_sync(FV_FULL, my_cnt[1], j);
      for (uint32_t t = t0; t < t1 && n < vcap; ++t) {
        uint32_t moff;
        int cnt;
        if (t - t0 < 2u) {
          moff = t == t0 ? mo0 : mo1;
          cnt = t == t0 ? cn0 : cn1;
          if (moff == 0xFFFFFFFFu) continue;
        } else {
          moff = task_moff[t];
          if (moff == 0xFFFFFFFFu || rt >= task_rows[t]) continue;
          cnt = int(tasks[t].z & 0xFFFFu) * 8;
        }
        const float* src = minima + size_t(moff) + size_t(rt) * cnt;
        const int room = min(cnt, vcap - n);
        for (int i = lane; i < room; i += 32) {
          const uint32_t b = order_bits(__fadd_ru(src[i], ad));  // rounded up: still an upper bound
          v[n + i] = b;
          if (b < INF_BITS) {
            finite += 1;
            vmin = min(vmin, b);
            vmax = max(vmax, b);
          }
        }
        n += room;
      }
    }
  }
  __syncwarp();
  if (__reduce_add_sync(FV_FULL, finite) < keep) {
    if (lane == 0) tau_bits[q] = 0xFFFFFFFFu;
    return;
  }
  // Bisection between the smallest and the largest finite bound; any value with exactly `keep` bounds at or below it
  // will do (it is at least the keep-th smallest and below the next one), so the search stops there.
  uint32_t lo = __reduce_min_sync(FV_FULL, vmin), hi = __reduce_max_sync(FV_FULL, vmax);
  while (lo < hi) {
    const uint32_t mid = lo + ((hi - lo) >> 1);
    int c = 0;
    for (int i = lane; i < n; i += 32) c += v[i] <= mid ? 1 : 0;
    c = __reduce_add_sync(FV_FULL, c);
    if (c == keep) {
      lo = mid;
      break;
    }
    if (c > keep) hi = mid;
    else lo = mid + 1;
  }
  if (lane == 0) tau_bits[q] = lo;
}

struct FinishArgs {
  const u64* cand;
  uint32_t* cand_cnt;
  int cap;
  uint32_t* counters;
  const uint32_t* qids;    // second round: the queries to finish (null: all, block b = query b) ...
  const uint32_t* nqids;   // ... and the device word that says how many there are
  // A query whose buffer ran over (count > cap):
  //   tighten == 1: its stored `cap` candidates still give a valid, tighter bound -- the keep-th smallest of them,
  //                 since that many rows reach it -- which goes to tau_bits[q]; the count is reset, redo[q] is set and
  //                 q is appended to over_ids, so that the survivors of exactly these queries are re-scored against
  //                 the new bound and finished in a second round;
  //   tighten == 0: q is appended to rerun_ids, the queries the per-query kernel takes over.
  // A count of 0xFFFFFFFF marks a query the scan could not handle at all: always to rerun_ids.
  int tighten;
  uint32_t* tau_bits;
  uint32_t* redo;
  uint32_t* over_ids;
  uint32_t* rerun_ids;
  const uint32_t* dropped;  // or null; dropped[q] != 0: the scan lost survivors of q (a full pool): to rerun_ids
};

// One block per query: the best `keep` of the appended candidates, then the common tail.  With f.qids the blocks
// walk that list (*f.nqids entries: a count only the device knows when the kernel is launched) instead of taking
// query blockIdx.x.
__device__ __forceinline__ void finish_block_query(const ScanArgs& a, const FinishArgs& f, size_t q, u64* lists, u64* rerank,
                                                   float* sq) {
  const int tid = threadIdx.x;
  const uint32_t cnt = f.cand_cnt[q];
  if (cnt == 0xFFFFFFFFu || (cnt > uint32_t(f.cap) && !f.tighten) || (f.dropped && f.dropped[q])) {
    if (tid == 0) f.rerun_ids[atomicAdd(f.counters + LS_C_RERUN, 1u)] = uint32_t(q);
    return;
  }
  const int have = int(min(cnt, uint32_t(f.cap)));
  int n = 32;
  while (n < have || n < a.keep) n <<= 1;
  for (int e = tid; e < n; e += blockDim.x) lists[e] = e < have ? f.cand[q * size_t(f.cap) + e] : FV_EMPTY_KEY;
  for (int c = tid; c < a.pd; c += blockDim.x) sq[c] = a.queries[q * size_t(a.pd) + c];
  __syncthreads();
  block_sort(lists, n);
  if (cnt > uint32_t(f.cap)) {  // ran over: a tighter bound from what was stored, and a second round
    if (tid == 0) {
      f.tau_bits[q] = uint32_t(lists[a.keep - 1] >> 32);  // cap >= keep entries are stored
      f.cand_cnt[q] = 0;
      f.redo[q] = 1;
      f.over_ids[atomicAdd(f.counters + LS_C_OVER, 1u)] = uint32_t(q);
    }
    return;
  }
  scan_tail(a, q, lists, rerank, sq);
}

__global__ void __launch_bounds__(256) ivfpq_finish_kernel(ScanArgs a, FinishArgs f, int n2max) {
  u64* lists = reinterpret_cast<u64*>(dyn_smem());  // n2max keys
  u64* rerank = lists + n2max;                      // keep + k
  float* sq = reinterpret_cast<float*>(rerank + a.keep + a.k);
  if (!f.qids) {
    finish_block_query(a, f, blockIdx.x, lists, rerank, sq);
    return;
  }
  const uint32_t n = *f.nqids;
  for (uint32_t i = blockIdx.x; i < n; i += gridDim.x) {
    finish_block_query(a, f, f.qids[i], lists, rerank, sq);
    __syncthreads();  // the shared buffers are reused by the next query
  }
}

// codes (rows x 16, by list) -> sub-quantizer-major copy, lists padded to 16 rows with zero bytes
__global__ void transpose_codes_kernel(const uint32_t* __restrict__ list_off, const uint32_t* __restrict__ off16,
                                       const uint8_t* __restrict__ codes, uint8_t* __restrict__ out) {
  const size_t l = blockIdx.x;
  const uint32_t off = list_off[l], len = list_off[l + 1] - off;
  const uint32_t len16 = off16[l + 1] - off16[l];
  uint8_t* dst = out + size_t(off16[l]) * 16;
  for (uint32_t r = threadIdx.x; r < len16; r += blockDim.x) {
    uint4 cw = make_uint4(0u, 0u, 0u, 0u);
    if (r < len) cw = *reinterpret_cast<const uint4*>(codes + (size_t(off) + r) * 16);
    const uint32_t wds[4] = {cw.x, cw.y, cw.z, cw.w};
#pragma unroll
    for (int j = 0; j < 16; ++j) dst[size_t(j) * len16 + r] = uint8_t((wds[j >> 2] >> ((j & 3) * 8)) & 0xFFu);
  }
}

int build_transposed_codes(fv_ctx* ctx, const uint32_t* h_off, size_t nlist, const uint32_t* d_list_off,
                           const uint8_t* d_codes, DevBuf* codes_t, DevBuf* off16) {
  std::vector<uint32_t> o16(nlist + 1, 0);
  for (size_t l = 0; l < nlist; ++l) {
    const uint64_t next = uint64_t(o16[l]) + ((h_off[l + 1] - h_off[l] + 15u) & ~15u);
    if (next > 0xFFFFFFF0ull) return fail(FV_ERR_UNSUPPORTED, "more than 2^32 padded rows");
    o16[l + 1] = uint32_t(next);
  }
  FV_TRY(off16->reserve((nlist + 1) * sizeof(uint32_t)));
  FV_TRY(codes_t->reserve(size_t(o16[nlist]) * 16 + 16));
  FV_CUDA(cudaMemcpyAsync(off16->p, o16.data(), (nlist + 1) * sizeof(uint32_t), cudaMemcpyHostToDevice, ctx->stream));
  if (o16[nlist]) {
    transpose_codes_kernel<<<unsigned(nlist), 256, 0, ctx->stream>>>(d_list_off, off16->as<uint32_t>(), d_codes,
                                                                    codes_t->as<uint8_t>());
    ctx->stats.launches++;
    FV_CUDA(cudaGetLastError());
  }
  FV_CUDA(cudaStreamSynchronize(ctx->stream));  // o16 leaves scope
  return FV_OK;
}

// ================================================================================================
// The tensor-core pass.  The compressed distance of a row is, up to rounding, the true distance between the query and
// the vector its code stands for: base + sum_j lut[j][code_j] = ||(q - centroid) - codewords||^2 (ivfpq.rs:108-126,
// :256-262), or -<q, centroid> - <q, codewords> for inner product.  So the list-major work -- every query that
// probes a list against every row of the list -- is a GEMM between the queries' residuals q - centroid (one operand
// row per (query, probe) pair; plain q for inner product) and a 16-bit copy of the rows' codewords: the tcgen05
// kernel of exact search in task mode scores 256 pairs x 256 rows per unit and hands back every (pair, row) whose
// score is below the query's bound plus a rigorous error margin.  Working on residuals keeps both operands small
// (a few hundred instead of a few thousand in norm), and with them the 16-bit rounding the margin has to cover.  Only those survivors get the reference's table arithmetic
// (rescore_kernel: base first, then the m table entries in order, each lut entry rounded on its own), and only a
// survivor whose exact compressed distance is at or below the bound becomes a candidate.  The tensor cores decide
// nothing on their own: a row they drop is provably above the bound.

// the residual each stored row's code stands for (its m codewords side by side), f32, list by list; lists start at
// multiples of 8 rows, the filler rows are zero
__global__ void reconstruct_kernel(const uint32_t* __restrict__ list_off, const uint32_t* __restrict__ roff8,
                                   const uint8_t* __restrict__ codes, const float* __restrict__ centroids,
                                   const float* __restrict__ codebooks, int pd, int m, int dsub, float* __restrict__ out) {
  const size_t l = blockIdx.x;
  const uint32_t off = list_off[l], len = list_off[l + 1] - off;
  const uint32_t r0 = roff8[l], len8 = roff8[l + 1] - r0;
  const size_t total = size_t(len8) * pd;
  for (size_t i = threadIdx.x; i < total; i += blockDim.x) {
    const uint32_t r = uint32_t(i / pd);
    const int d = int(i - size_t(r) * pd);
    float v = 0.f;
    if (r < len) {
      const int j = d / dsub, t = d - j * dsub;
      const uint32_t c = codes[(size_t(off) + r) * m + j];
      v = codebooks[(size_t(j) * KSUB + c) * dsub + t];
    }
    out[(size_t(r0) + r) * pd + d] = v;
  }
}

int build_reconstruction(fv_ctx* ctx, int metric, int pd, int m, int dsub, const uint32_t* h_off, size_t nlist,
                         const uint32_t* d_list_off, const uint8_t* d_codes, const float* d_centroids,
                         const float* d_codebooks, TcSide** recon, DevBuf* roff8) {
  tc_free(*recon);
  *recon = nullptr;
  std::vector<uint32_t> o8(nlist + 1, 0);
  for (size_t l = 0; l < nlist; ++l) {
    const uint64_t next = uint64_t(o8[l]) + ((h_off[l + 1] - h_off[l] + 7u) & ~7u);
    if (next > 0x7FFFFF00ull) return FV_OK;  // beyond the kernel's row range: no tensor-core pass for this index
    o8[l + 1] = uint32_t(next);
  }
  const size_t rows = o8[nlist];
  if (rows == 0 || pd > 128) return FV_OK;
  // behind the offsets: the list numbers, longest list first (the order the tasks are dealt in)
  o8.resize(2 * nlist + 1);
  for (size_t l = 0; l < nlist; ++l) o8[nlist + 1 + l] = uint32_t(l);
  std::stable_sort(o8.begin() + nlist + 1, o8.end(),
                   [&](uint32_t x, uint32_t y) { return h_off[x + 1] - h_off[x] > h_off[y + 1] - h_off[y]; });
  FV_TRY(roff8->reserve(o8.size() * sizeof(uint32_t)));
  FV_CUDA(cudaMemcpyAsync(roff8->p, o8.data(), o8.size() * sizeof(uint32_t), cudaMemcpyHostToDevice, ctx->stream));
  DevBuf tmp;
  FV_TRY(tmp.reserve(rows * size_t(pd) * sizeof(float)));
  reconstruct_kernel<<<unsigned(nlist), 256, 0, ctx->stream>>>(d_list_off, roff8->as<uint32_t>(), d_codes, d_centroids,
                                                              d_codebooks, pd, m, dsub, tmp.as<float>());
  ctx->stats.launches++;
  FV_CUDA(cudaGetLastError());
  FV_TRY(tc_append(ctx, recon, metric, tmp.as<float>(), 0, rows, pd));
  FV_CUDA(cudaStreamSynchronize(ctx->stream));  // tmp and o8 leave scope
  return FV_OK;
}

// One block: the tasks of the tensor-core pass.  The n pairs of a list with len rows fill ceil(n / TR) operand tiles
// of TR gathered rows (a_off[l] is the list's first gathered row; TR = 256, or 128 when the lists have few pairs each,
// so that a half-empty tile does not cost a whole tile's multiplications), and every tile meets the list's rows in segments
// of at most TC_SEG_UNITS units of 256 rows: one task per (tile, segment), so that no task is longer than a segment
// and a few very long lists cannot hold up the CTAs that drew them.  A tile's tasks are consecutive;
// tile_task0[tile] is the first (and tile_task0[tiles] the task count).  Lists are walked in `order` (longest
// first), so the long tasks are drawn first.
// A task is {first operand row, first side row of the segment, units in the segment | first unit << 16, list length}.
static constexpr uint32_t TC_SEG_UNITS = 8;

__global__ void __launch_bounds__(1024) tc_tasks_kernel(const uint32_t* __restrict__ pair_off,
                                                        const uint32_t* __restrict__ list_off,
                                                        const uint32_t* __restrict__ roff8,
                                                        const uint32_t* __restrict__ order, size_t nlist,
                                                        uint4* __restrict__ tasks, uint32_t* __restrict__ a_off,
                                                        uint32_t* __restrict__ tile_task0, uint32_t max_tasks,
                                                        uint32_t* __restrict__ ntasks, unsigned long long* __restrict__ rows,
                                                        uint32_t* __restrict__ task_moff, uint32_t* __restrict__ task_rows,
                                                        uint32_t minima_cap, uint32_t TR) {  // TR: rows of an operand tile, 128 or 256
  __shared__ uint32_t st[1024], sl[1024];
  __shared__ unsigned long long sm8[1024];  // minima variant: floats of minima the tasks before a thread's need
  const int tid = threadIdx.x;
  const size_t per = (nlist + 1023) / 1024;
  const size_t l0 = min(nlist, size_t(tid) * per), l1 = min(nlist, l0 + per);
  uint32_t nt = 0, ntl = 0;  // tasks, tiles
  unsigned long long nr = 0, nm = 0;
  for (size_t o = l0; o < l1; ++o) {
    const size_t l = order[o];
    const uint32_t n = pair_off[l + 1] - pair_off[l], len = list_off[l + 1] - list_off[l];
    if (!n || !len) continue;
    const uint32_t tiles = (n + TR - 1u) / TR, units = (len + 255u) / 256u;
    ntl += tiles;
    nt += tiles * ((units + TC_SEG_UNITS - 1) / TC_SEG_UNITS);
    nr += (unsigned long long)n * len;
    nm += (unsigned long long)n * units * 8u;  // 8 minima per pair and unit
  }
  st[tid] = nt;
  sl[tid] = ntl;
  sm8[tid] = nm;
  __syncthreads();
  for (int o = 1; o < 1024; o <<= 1) {
    const uint32_t b = tid >= o ? st[tid - o] : 0u, bl = tid >= o ? sl[tid - o] : 0u;
    const unsigned long long b8 = tid >= o ? sm8[tid - o] : 0ull;
    __syncthreads();
    st[tid] += b;
    sl[tid] += bl;
    sm8[tid] += b8;
    __syncthreads();
  }
  uint32_t bt = st[tid] - nt, bl = sl[tid] - ntl;
  unsigned long long bm = sm8[tid] - nm;
  for (size_t o = l0; o < l1; ++o) {
    const size_t l = order[o];
    const uint32_t len = list_off[l + 1] - list_off[l], n = pair_off[l + 1] - pair_off[l];
    a_off[l] = bl * TR;
    if (!n || !len) continue;
    const uint32_t tiles = (n + TR - 1u) / TR, units = (len + 255u) / 256u;
    const uint32_t nseg = (units + TC_SEG_UNITS - 1) / TC_SEG_UNITS;
    for (uint32_t t = 0; t < tiles; ++t) {
      tile_task0[bl + t] = bt;
      const uint32_t valid = min(TR, n - t * TR);
      for (uint32_t sg = 0; sg < nseg; ++sg, ++bt) {
        if (bt >= max_tasks) continue;  // cannot happen with the caller's sizing; never write past the table
        const uint32_t u0 = sg * TC_SEG_UNITS, un = min(TC_SEG_UNITS, units - u0);
        tasks[bt] = make_uint4((bl + t) * TR, roff8[l] + u0 * 256u, un | (u0 << 16), len);
        if (task_moff) {
          const unsigned long long need = (unsigned long long)valid * un * 8u;
          task_rows[bt] = valid;
          task_moff[bt] = bm + need <= minima_cap ? uint32_t(bm) : 0xFFFFFFFFu;  // beyond the buffer: this task leaves no minima
          bm += need;
        }
      }
    }
    bl += tiles;
  }
  if (tid == 1023) {
    *ntasks = min(st[1023], max_tasks);
    tile_task0[sl[1023]] = min(st[1023], max_tasks);
  }
  if (nr && rows) atomicAdd(rows, nr);
}

struct GatherArgs {
  uint32_t tile_rows;          // rows of an operand tile (128 or 256): a list's rows are padded to whole tiles
  const uint32_t* pair_off;
  const uint32_t* list_off;
  const uint32_t* a_off;
  const uint2* pairs;
  const float* queries;       // nq x pd f32
  const float* centroids;     // nlist x pd
  const uint32_t* tau_bits;   // nq
  uint32_t* cand_cnt;         // nq
  int cap, pd, Kp, is_l2, bf16;
  float kf, bn, cw2, c1;      // Kp; largest codeword-row norm; max ||centroid||^2 + max ||codewords||^2; rounding count of the chain
  uint16_t* qg;               // gathered operand rows
  float* thr;                 // per gathered row
  uint32_t* g_q;
  uint32_t* g_l;
  float* g_base;
  // bound variant (q_rows != null): thr[row] receives what turns a score into an UPPER bound of the compressed
  // distance (||a||^2 + eps, or base + eps), and the row is filed under its query: q_rows[q * q_slots + i]
  uint32_t* q_rows;
  uint32_t* q_cnt;
  int q_slots;
};

__device__ __forceinline__ uint16_t to_operand(float x, int bf16) {
  return bf16 ? __bfloat16_as_ushort(__float2bfloat16_rn(x)) : __half_as_ushort(__float2half_rn(x));
}

// Eight lanes per gathered row, four rows per warp and step (blockIdx.x = list, blockIdx.y strides its rows): writes
// the pair's operand row, -2 (q - centroid) for L2 or -q for inner product in the side's 16-bit type, and turns the
// query's bound into the score threshold of that row.  (One warp per row spent two thirds of its instructions in
// the single lane that works out the margin; with eight lanes per row four margins are worked out side by side.)
// With a = q - centroid (L2) the kernel's score is ||w||^2 - 2 <a, w> for the row's codewords w, and
// |score + ||a||^2 - compressed distance| <= eps, where eps adds up
//   - the 16-bit score against the f32 arithmetic on (a, w): input rounding 2 u |a||w|, fp32 accumulation, the norm
//     step (the margin exact search uses, on the residuals' norms);
//   - the rounding of the reference's own chain (base, precomputed and query tables, the m + 1 additions): c1
//     roundings of at most 2^-24 * 3 (|q|^2 + |c|^2 + |w|^2) each;
//   - the rounding of a itself and of ||a||^2 (summed in any order: 2e-6 ||a||^2 covers it).
// Every row with compressed distance <= bound therefore scores below bound - ||a||^2 + eps.  For inner product the
// score is -<q, w> and the threshold bound - base + eps with base = -<q, centroid> as the reference computed it.
// Queries the tensor cores cannot score (no bound, non-finite or beyond the 16-bit range) are marked for the
// per-query kernel instead.
__global__ void __launch_bounds__(256) tc_gather_kernel(GatherArgs a) {
  const size_t l = blockIdx.x;
  const int w = threadIdx.x >> 5, lane = threadIdx.x & 31, grp = lane >> 3, sub = lane & 7;
  const uint32_t p0 = a.pair_off[l], n = a.pair_off[l + 1] - p0;
  if (n == 0 || a.list_off[l + 1] == a.list_off[l]) return;
  const uint32_t rows = (n + a.tile_rows - 1u) / a.tile_rows * a.tile_rows;
  const uint32_t a0 = a.a_off[l];
  const float* cen = a.centroids + l * size_t(a.pd);
  const float mul = a.is_l2 ? -2.f : -1.f;
  const int e_per = a.Kp >> 3;  // elements of a row per lane: a multiple of 8 (Kp is a multiple of 64)
  for (uint32_t rb = blockIdx.y * 32 + w * 4; rb < rows; rb += gridDim.y * 32) {  // rows is a multiple of 128
    const uint32_t r = rb + grp, arow = a0 + r;
    const bool live = r < n;
    uint2 pr = make_uint2(0u, 0u);
    if (live) pr = a.pairs[p0 + r];
    const uint32_t q = pr.x;
    const float* qv = a.queries + size_t(q) * a.pd;
    uint16_t* dst = a.qg + size_t(arow) * a.Kp;
    float mx = 0.f, a2 = 0.f, q2 = 0.f;
    bool fin = true;
    if (live) {
      for (int e = 0; e < e_per; e += 8) {
        const int c = sub * e_per + e;
        float x[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        if (c < a.pd) {  // pd is a multiple of 8: the whole group of 8 is inside or outside
          const float4 q0 = *reinterpret_cast<const float4*>(qv + c), q1 = *reinterpret_cast<const float4*>(qv + c + 4);
          x[0] = q0.x, x[1] = q0.y, x[2] = q0.z, x[3] = q0.w, x[4] = q1.x, x[5] = q1.y, x[6] = q1.z, x[7] = q1.w;
#pragma unroll
          for (int i = 0; i < 8; ++i) q2 = __fmaf_rn(x[i], x[i], q2);
          if (a.is_l2) {
            const float4 c0 = *reinterpret_cast<const float4*>(cen + c), c1 = *reinterpret_cast<const float4*>(cen + c + 4);
            x[0] = __fsub_rn(x[0], c0.x), x[1] = __fsub_rn(x[1], c0.y), x[2] = __fsub_rn(x[2], c0.z), x[3] = __fsub_rn(x[3], c0.w);
            x[4] = __fsub_rn(x[4], c1.x), x[5] = __fsub_rn(x[5], c1.y), x[6] = __fsub_rn(x[6], c1.z), x[7] = __fsub_rn(x[7], c1.w);
          }
        }
        uint32_t h[4];
#pragma unroll
        for (int i = 0; i < 8; i += 2) {
          mx = fmaxf(mx, fmaxf(fabsf(x[i]), fabsf(x[i + 1])));
          a2 = __fmaf_rn(x[i], x[i], a2);
          a2 = __fmaf_rn(x[i + 1], x[i + 1], a2);
          fin = fin && fabsf(x[i]) <= 3.0e38f && fabsf(x[i + 1]) <= 3.0e38f;
          h[i >> 1] = uint32_t(to_operand(x[i] * mul, a.bf16)) | (uint32_t(to_operand(x[i + 1] * mul, a.bf16)) << 16);
        }
        *reinterpret_cast<uint4*>(dst + c) = make_uint4(h[0], h[1], h[2], h[3]);
      }
    }
    for (int o = 4; o > 0; o >>= 1) {  // over the eight lanes of the row
      mx = fmaxf(mx, __shfl_xor_sync(FV_FULL, mx, o));
      a2 += __shfl_xor_sync(FV_FULL, a2, o);
      q2 += __shfl_xor_sync(FV_FULL, q2, o);
    }
    const unsigned finb = __ballot_sync(FV_FULL, fin);
    fin = ((finb >> (grp * 8)) & 0xFFu) == 0xFFu;
    if (sub != 0) continue;
    if (!live) {
      a.thr[arow] = -INFINITY;  // filler row: never below its threshold
      continue;
    }
    const bool bound_pass = a.q_rows != nullptr;
    const uint32_t tb = bound_pass ? 0u : a.tau_bits[q];
    const bool in_range = fin && (a.bf16 ? mx <= 1.0e38f : mx * (a.is_l2 ? 2.f : 1.f) <= 65504.f);
    const float base = __uint_as_float(pr.y);
    float thr = -INFINITY;
    if (tb != 0xFFFFFFFFu && in_range) {
      const float tau = bound_pass ? 0.f : order_bits_to_float(tb);
      const float u16 = a.bf16 ? 0.00390625f : 0.00048828125f;
      const float an = sqrtf(a2), bn = a.bn, kf = a.kf;
      const float e_dot = (2.f * u16 * (1.f + u16) + kf * 4.7683716e-7f + kf * 1.1920929e-7f) * an * bn +
                          5.9604645e-8f * sqrtf(kf) * (an + bn);
      const float e_norm = (kf + 16.f) * 4.7683716e-7f * bn * bn + 1.1920929e-7f * bn * bn;
      const float e_score = a.is_l2 ? 2.f * e_dot + e_norm + kf * 4.7683716e-7f * (a2 + bn * bn) : e_dot;
      const float e_chain = a.c1 * 5.9604645e-8f * 3.f * (q2 + a.cw2);
      const float e_self = 2.4e-7f * (an + bn) * an + 2.0e-6f * a2;
      const float eps = 1.05f * (e_score + e_chain + e_self) + 1e-30f;
      if (bound_pass) {
        thr = a.is_l2 ? a2 + eps : base + eps;  // score + this >= the row's compressed distance
        if (!(thr == thr)) thr = INFINITY;
      } else {
        thr = a.is_l2 ? (tau - a2) + eps : (tau - base) + eps;
        if (!(thr == thr) || thr == INFINITY) thr = -INFINITY;  // a margin that is not a number: leave it to the other kernel
      }
    } else if (bound_pass) {
      thr = INFINITY;  // no usable scores for this query: its minima say nothing
    }
    if (bound_pass) {
      const uint32_t slot = atomicAdd(a.q_cnt + q, 1u);
      if (slot < uint32_t(a.q_slots)) a.q_rows[size_t(q) * a.q_slots + slot] = arow;
    } else if (thr == -INFINITY) {
      a.cand_cnt[q] = 0xFFFFFFFFu;  // left to the per-query kernel (none of its rows survives)
    }
    a.thr[arow] = thr;
    a.g_q[arow] = q;
    a.g_l[arow] = uint32_t(l);
    a.g_base[arow] = base;
  }
}

struct RescoreArgs {
  const u64* pool;
  const unsigned int* pool_cnt;
  unsigned int pool_cap;
  int npools;
  const uint32_t* g_q;
  const uint32_t* g_l;
  const float* g_base;
  const uint32_t* list_off;
  const uint8_t* codes;
  const uint32_t* ids;
  const float* qtab;
  const float* pre;  // or null (inner product)
  int m;
  const uint32_t* tau_bits;
  u64* cand;
  uint32_t* cand_cnt;
  int cap;
  const uint32_t* only;  // second round: only survivors of queries with only[q] != 0 (null: all)
  const uint32_t* gate;  // second round: the device word that counts its queries; the kernel leaves at once if it is 0
  size_t a_rows;         // extents (gathered operand rows, lists, rows in all lists), for the checks of the debug build
  uint32_t nlist, nrows;
};

// One thread per survivor: the reference's compressed distance (ivfpq.rs:256-262, :272-276), bit for bit; kept if
// at or below the query's bound.
// The pools are very unequal (a CTA that drew the lists of a dense region holds several times the average), so the
// blocks split the concatenation of all pools evenly instead of a pool each.
__global__ void __launch_bounds__(128) rescore_kernel(RescoreArgs a) {
  if (a.gate && *a.gate == 0) return;
  uint32_t* start = reinterpret_cast<uint32_t*>(dyn_smem());  // npools + 1: first global index of every pool
  if (threadIdx.x == 0) {
    uint32_t s = 0;
    for (int c = 0; c < a.npools; ++c) {
      start[c] = s;
      s += min(a.pool_cnt[c], a.pool_cap);
    }
    start[a.npools] = s;
  }
  __syncthreads();
  const uint32_t total = start[a.npools];
  const uint32_t per = ((total + gridDim.x - 1) / gridDim.x + 127u) & ~127u;
  const uint32_t i0 = min(total, blockIdx.x * per), i1 = min(total, i0 + per);
  const size_t tab = size_t(a.m) * KSUB;
  for (uint32_t i = i0 + threadIdx.x; i < i1; i += blockDim.x) {
    int lo = 0, hi = a.npools - 1;  // the pool holding global index i: the last one starting at or before it
    while (lo < hi) {
      const int mid = (lo + hi + 1) >> 1;
      if (start[mid] <= i) lo = mid;
      else hi = mid - 1;
    }
    const u64 e = a.pool[size_t(lo) * a.pool_cap + (i - start[lo])];
    const uint32_t arow = uint32_t(e >> 32), row = uint32_t(e);
    if (!FV_IDX_OK(arow, a.a_rows, 5)) continue;
    const uint32_t q = a.g_q[arow], l = a.g_l[arow];
    if (!FV_IDX_OK(l, a.nlist, 6)) continue;
    if (a.only && !a.only[q]) continue;
    const size_t r = size_t(a.list_off[l]) + row;
    if (!FV_IDX_OK(r, a.nrows, 7)) continue;
    const uint8_t* code = a.codes + r * a.m;
    const float* qt = a.qtab + size_t(q) * tab;
    const float* pt = a.pre ? a.pre + size_t(l) * tab : nullptr;
    float d = a.g_base[arow];
    if (a.m == 16) {  // all 32 table reads in flight before the chain of additions starts
      const uint4 cw = *reinterpret_cast<const uint4*>(code);
      const uint32_t cws[4] = {cw.x, cw.y, cw.z, cw.w};
      float t[16], pv[16];
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        const int cj = int((cws[j >> 2] >> ((j & 3) * 8)) & 0xFFu);
        t[j] = __ldg(qt + j * 256 + cj);
        pv[j] = pt ? __ldg(pt + j * 256 + cj) : 0.f;
      }
#pragma unroll
      for (int j = 0; j < 16; ++j) d = __fadd_rn(d, pt ? __fadd_rn(pv[j], t[j]) : t[j]);
    } else {
      for (int j = 0; j < a.m; ++j) {
        const int cj = code[j];
        float t = __ldg(qt + j * 256 + cj);
        if (pt) t = __fadd_rn(__ldg(pt + j * 256 + cj), t);
        d = __fadd_rn(d, t);
      }
    }
    if (d < INFINITY && order_bits(d) <= a.tau_bits[q]) {
      const uint32_t slot = atomicAdd(a.cand_cnt + q, 1u);
      if (slot < uint32_t(a.cap)) a.cand[size_t(q) * a.cap + slot] = make_key(d, __ldg(a.ids + r));
    }
  }
}

// ------------------------------------------------------------------------------------------------
static int launch_block_scan(fv_ctx* ctx, const ScanArgs& a, size_t nblocks, bool use_pre) {
  const size_t tab = size_t(a.m) * KSUB;
  const size_t smem = (2 * size_t(a.pd) + tab * (use_pre ? 2 : 1)) * sizeof(float) +
                      (size_t(a.cap) + size_t(a.keep) + size_t(a.k)) * sizeof(u64);
  if (smem + 256 > ctx->smem_optin) return fail(FV_ERR_UNSUPPORTED, "m, k * refine too large for shared memory");
  auto kern = a.m == 16 ? ivfpq_scan_kernel<true, 2> : ivfpq_scan_kernel<false, 1>;
  if (smem > 40 * 1024) FV_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)));
  kern<<<unsigned(nblocks), 256, smem, ctx->stream>>>(a);
  ctx->stats.launches++;
  FV_CUDA(cudaGetLastError());
  return FV_OK;
}

// The small arrays of one pass over the pairs, in one allocation; the first `nzero` words must start at zero.
struct PairSet {
  uint32_t *pair_cnt, *cursor, *per_query, *counters, *pair_off, *task_off, *extra, *extra2;  // per_query, extra, extra2: nq words each
  size_t nzero, words;
  static size_t words_for(size_t nlist, size_t nq) {
    return ((2 * nlist + nq + 1) & ~size_t(1)) + LS_NCOUNTERS + 2 * (nlist + 1) + 2 * nq;
  }
  void carve(uint32_t* base, size_t nlist, size_t nq) {
    pair_cnt = base;
    cursor = base + nlist;
    per_query = base + 2 * nlist;
    const size_t o_ctr = (2 * nlist + nq + 1) & ~size_t(1);
    counters = base + o_ctr;
    nzero = o_ctr + LS_NCOUNTERS;
    pair_off = base + nzero;
    task_off = pair_off + nlist + 1;
    extra = task_off + nlist + 1;
    extra2 = extra + nq;
    words = nzero + 2 * (nlist + 1) + 2 * nq;
  }
};

static int bucket_pairs(fv_ctx* ctx, const ScanIndex& ix, const u64* cells, size_t nq, int nprobe, uint32_t min_rows,
                        const PairSet& ps, uint2* pairs, uint32_t* slot_of = nullptr) {
  PairArgs pa{};
  pa.cells = cells;
  pa.nq = nq;
  pa.nprobe = nprobe;
  pa.shard_rank = ix.shard_rank;
  pa.shard_world = ix.shard_world;
  pa.min_rows = min_rows;
  pa.nlist = uint32_t(ix.nlist);
  pa.list_off = ix.list_off;
  pa.pair_cnt = ps.pair_cnt;
  pa.cursor = ps.cursor;
  pa.pair_off = ps.pair_off;
  pa.pairs = pairs;
  pa.slot_of = slot_of;
  if (min_rows == 0 && slot_of) {
    const unsigned fblocks = unsigned((nq * size_t(nprobe) + 255) / 256);
    pair_flat_kernel<false><<<fblocks, 256, 0, ctx->stream>>>(pa);
    pair_offsets_kernel<<<1, 1024, 0, ctx->stream>>>(ps.pair_cnt, ix.list_off, ix.nlist, ps.pair_off, ps.task_off, ps.counters);
    pair_flat_kernel<true><<<fblocks, 256, 0, ctx->stream>>>(pa);
  } else {
    const unsigned qblocks = unsigned((nq + 255) / 256);
    pair_kernel<false><<<qblocks, 256, 0, ctx->stream>>>(pa);
    pair_offsets_kernel<<<1, 1024, 0, ctx->stream>>>(ps.pair_cnt, ix.list_off, ix.nlist, ps.pair_off, ps.task_off, ps.counters);
    pair_kernel<true><<<qblocks, 256, 0, ctx->stream>>>(pa);
  }
  ctx->stats.launches += 3;
  FV_CUDA(cudaGetLastError());
  return FV_OK;
}

bool ivfpq_wants_tensor(int mode, size_t nq, size_t nprobe, size_t nlist, int shard_world) {
  (void)shard_world;  // a list shard sees 1 / world of the pairs on 1 / world of the lists: the same pairs per list
  if (mode == 3 || mode == 4) return nq >= 1;
  if (mode != 0) return false;
  // The tensor-core pass costs about one unit of work per (list, 256-pair tile, 256 rows) whatever the tile holds, the
  // per-query kernel one per (pair, row): measured on 1M x 128 / 1024 lists, the pass wins from about 8 pairs per
  // list (4 pairs per list: 0.50 against 0.46 ms; 78: 0.80 against 1.34 ms), and on 50M x 128 / 16384 lists with 20
  // pairs per list it takes 8.6 ms against 18.7.
  return nq >= 256 && nq * nprobe >= 12 * std::max<size_t>(1, nlist);
}

// Stages (fv_stats.stage_ms) of an IVF-PQ search: 0 coarse cells (marked by the caller); 1 query tables and, on the
// list-major paths, the bound pass; 2 bucketing the (query, probe) pairs by list (tensor-core pass: plus the task
// table and the gathered operand rows); 3 the scan (the per-query kernel, the list-major table kernel, or the
// tensor-core kernel); 4 re-scoring survivors (tensor-core pass); 5 sorting the candidates, re-ranking and any re-run
// of queries by the per-query kernel; 6 keys -> neighbours (marked by the caller).
int ivfpq_scan(fv_ctx* ctx, const ScanIndex& ix, const float* q, size_t nq, const u64* cells, int nprobe, int keep,
               int k, bool refine, bool candidates, int mode, int cand_slots, const ScanOut& out) {
  const bool use_pre = ix.metric == FV_L2 && ix.pre != nullptr;
  const bool separable = use_pre || ix.metric == FV_INNER_PRODUCT;
  const size_t tab = size_t(ix.m) * KSUB;
  unsigned long long* d_rows = reinterpret_cast<unsigned long long*>(ctx->d_flags + 16);  // [0] per-query kernel, [1] list-major
  FV_CUDA(cudaMemsetAsync(d_rows, 0, 2 * sizeof(unsigned long long), ctx->stream));
  const float* qtab = nullptr;
  if (separable) {
    FV_TRY(ctx->scratch[5].reserve(nq * tab * sizeof(float)));
    qtab = ctx->scratch[5].as<float>();
    dim3 grid(unsigned((nq + 15) / 16), unsigned(ix.m));
    auto qk = ix.dsub == 8 ? query_tables_kernel<8> : (ix.dsub == 4 ? query_tables_kernel<4> : query_tables_kernel<0>);
    qk<<<grid, KSUB, 16 * ix.dsub * sizeof(float), ctx->stream>>>(q, nq, ix.pd, ix.codebooks, ix.m, ix.dsub,
                                                                   ix.metric == FV_INNER_PRODUCT ? 1 : 0,
                                                                   ctx->scratch[5].as<float>());
    ctx->stats.launches++;
    FV_CUDA(cudaGetLastError());
  }
  ScanArgs a{};
  a.queries = q;
  a.qtab = qtab;
  a.cells = cells;
  a.centroids = ix.centroids;
  a.codebooks = ix.codebooks;
  a.pre = ix.pre;
  a.list_off = ix.list_off;
  a.codes = ix.codes;
  a.ids = ix.ids;
  a.vectors = ix.vectors;
  a.owned_ids = ix.owned_ids;
  a.owned_n = ix.owned_n;
  a.shard_rank = ix.shard_rank;
  a.shard_world = ix.shard_world;
  a.metric = ix.metric;
  a.pd = ix.pd;
  a.m = ix.m;
  a.dsub = ix.dsub;
  a.nprobe = nprobe;
  a.keep = keep;
  a.k = k;
  a.np = 2;
  a.cap = 2048;
  while (a.cap < keep + 1024) a.cap <<= 1;
  a.refine = refine && !candidates ? 1 : 0;
  a.candidates = candidates ? 1 : 0;
  a.id_base = ix.id_base;
  a.nlist = uint32_t(ix.nlist);
  a.nrows = ix.nrows;
  a.nvec = ix.owned_n;
  a.out_keys = out.keys;
  a.out_adc = out.adc;
  a.out_exact = out.exact;
  a.out_counts = out.counts;
  a.rows_scanned = d_rows;

  // Which scan.  Both list-major paths need m = 16 (the bound pass reads the sub-quantizer-major codes), a table that
  // separates into a list part and a query part, and at most 1024 kept candidates.  The tensor-core pass also needs
  // the reconstructed rows and enough pairs per list (ivfpq_wants_tensor).  The table scan is never chosen
  // automatically (measured no faster than the per-query kernel).
  enum { BLOCK, LIST_TABLE, LIST_TENSOR } path = BLOCK;
  const bool list_ok = ix.m == 16 && ix.codes_t && separable && keep <= 1024;
  const bool tensor_ok = list_ok && ix.recon != nullptr;
  if (mode == 2 && list_ok) path = LIST_TABLE;
  if (tensor_ok && ivfpq_wants_tensor(mode, nq, size_t(nprobe), ix.nlist, ix.shard_world)) path = LIST_TENSOR;
  if (path == BLOCK) {
    stage_mark(ctx);  // 1
    stage_mark(ctx);  // 2 (empty)
    FV_TRY(launch_block_scan(ctx, a, nq, use_pre));
    stage_mark(ctx);  // 3
    stage_mark(ctx);  // 4 (empty)
    stage_mark(ctx);  // 5 (empty)
  } else {
    // candidate slots per query: 2048 (at the benchmark's size one query in twenty finds more than 1024 rows at or
    // below its bound, and any re-run costs the latency of a whole pass of the per-query kernel), fewer when the
    // buffers of a large batch would pass 256 MB
    int cap = 2048;
    while (cap > 256 && nq * size_t(cap) * sizeof(u64) > (size_t(256) << 20)) cap >>= 1;
    if (cand_slots > 0) cap = std::min(cand_slots, 4096);
    // Bound pass: each query's nearest owned lists until they hold 32 * keep rows, i.e. four times `keep` minima
    // (one per 8 rows), and room for twice that plus one long list per query.
    const uint32_t bound_rows = uint32_t(std::max(1024, 32 * keep));
    // The tensor-core bound pass keeps one minimum per 32 rows and looks at three times the rows: the lists a query's
    // best candidates come from are more than its nearest three or four, and a bound that has seen ten of them lets
    // about half as many rows through the main pass (180 against 350 per query at keep = 100) for the same number
    // of minima to select from.
    const uint32_t bound_rows_tc = uint32_t(std::max(3072, 96 * keep));
    size_t mcap = 1024;
    while (mcap < 16384 && mcap < 2 * size_t(bound_rows / 8) + 512) mcap <<= 1;
    PairSet pa_set, pb_set;
    const size_t set_words = (PairSet::words_for(ix.nlist, nq) + 3) & ~size_t(3);
    FV_TRY(ctx->scratch[8].reserve(2 * set_words * sizeof(uint32_t)));
    uint32_t* sm = ctx->scratch[8].as<uint32_t>();
    pa_set.carve(sm, ix.nlist, nq);
    pb_set.carve(sm + set_words, ix.nlist, nq);
    FV_CUDA(cudaMemsetAsync(pa_set.pair_cnt, 0, pa_set.nzero * sizeof(uint32_t), ctx->stream));
    FV_CUDA(cudaMemsetAsync(pb_set.pair_cnt, 0, pb_set.nzero * sizeof(uint32_t), ctx->stream));
    FV_TRY(ctx->scratch[7].reserve(2 * nq * size_t(nprobe) * sizeof(uint2) + nq * size_t(nprobe) * sizeof(uint32_t) + 16));
    FV_TRY(ctx->scratch[9].reserve(nq * size_t(cap) * sizeof(u64)));
    uint2* pairs_a = ctx->scratch[7].as<uint2>();
    uint2* pairs_b = pairs_a + nq * size_t(nprobe);
    uint32_t* slot_of = reinterpret_cast<uint32_t*>(pairs_b + nq * size_t(nprobe));
    uint32_t* tau_bits = pa_set.extra;
    // How the bound is found.  The tensor-core bound pass costs about one unit of work per (touched list, 256 rows)
    // however few of the batch's queries are near that list, plus five small kernels; scanning each query's few
    // nearest lists with the per-query kernel costs one (query, row) evaluation each, at a poor rate (short blocks).
    // Both are estimated from measured rates (1M x 128 / 1024 lists: 0.185 ms on the tensor cores at 1,250 queries,
    // 0.20 and 0.31 ms by the per-query kernel at 1,250 and 2,500; 50M x 128 / 16384 lists, 10,000 queries: 2.5
    // against 1.5 ms) and the cheaper one is taken: the tensor cores unless the lists are long and many.
    bool mini_bound = false;
    if (path == LIST_TENSOR) {
      const double avg_len = double(ix.nrows) / double(std::max<size_t>(1, ix.nlist));
      const double lists_per_query = std::max(1.0, std::ceil(double(bound_rows) / std::max(1.0, avg_len)));
      const double pairs_a_est = double(nq) * std::min(lists_per_query, double(nprobe));
      const size_t owned = std::max<size_t>(1, ix.nlist / size_t(std::max(1, ix.shard_world)));
      const double t_mini = pairs_a_est * avg_len * 5e-5;                                                    // microseconds
      const double t_tc = std::min(double(owned), pairs_a_est) * std::max(1.0, avg_len / 256.0) * 0.025 + 80.0;
      mini_bound = t_mini < t_tc || mode == 4;
    }
    if (mini_bound) {
      ScanArgs b = a;
      b.row_budget = bound_rows;
      b.bound_out = tau_bits;
      b.rows_scanned = nullptr;
      b.refine = 0;
      b.candidates = 0;
      FV_TRY(launch_block_scan(ctx, b, nq, use_pre));
    } else {
      FV_TRY(bucket_pairs(ctx, ix, cells, nq, nprobe, path == LIST_TENSOR ? bound_rows_tc : bound_rows, pa_set, pairs_a));
    }
    ListScanArgs la{};
    la.qtab = qtab;
    la.pre = ix.pre;
    la.list_off = ix.list_off;
    la.off16 = ix.off16;
    la.codes_t = ix.codes_t;
    la.ids = ix.ids;
    la.nlist = uint32_t(ix.nlist);
    auto main_k = use_pre ? ivfpq_list_scan_kernel<true, false> : ivfpq_list_scan_kernel<false, false>;
    // buffers of the tensor-core pass (both its bound pass and its main pass use them, one after the other)
    TcInfo ti{};
    size_t a_rows = 0, max_tasks = 0;
    uint16_t* qg = nullptr;
    float* thr = nullptr;
    uint32_t *g_q = nullptr, *g_l = nullptr, *a_off = nullptr, *ntasks = nullptr, *task_moff = nullptr, *task_rows = nullptr;
    uint32_t* tile_task0 = nullptr;
    uint32_t tr_a = 256u, tr_b = 256u;  // operand tile rows of the bound pass and of the main pass
    float* g_base = nullptr;
    uint4* tasks = nullptr;
    unsigned int* pool_cnt = nullptr;
    unsigned int pool_cap = 0;
    uint32_t* dropped = nullptr;  // per query: the main pass lost survivors of it (a full pool)
    GatherArgs ga{};
    if (path == LIST_TENSOR) {
      tc_info(ix.recon, &ti);
      FV_CUDA(cudaMemsetAsync(tc_error_word(ix.recon), 0, sizeof(int), ctx->stream));  // read after the last pass
      const size_t Kp = size_t(ti.Kp);
      // gathered operand rows: every pair once, every list's rows rounded up to whole 256-row tiles
      a_rows = nq * size_t(nprobe) + 256 * std::min<size_t>(ix.nlist, nq * size_t(nprobe)) + 256;
      const size_t max_tiles = a_rows / 128;  // (tiles of 128 rows at the most)
      const size_t max_units = (size_t(ix.max_list_rows) + 255) / 256;
      max_tasks = max_tiles * std::max<size_t>(1, (max_units + TC_SEG_UNITS - 1) / TC_SEG_UNITS);
      if (max_tasks > 0x7FFFFFF0u) return fail(FV_ERR_UNSUPPORTED, "too many tasks for one tensor-core pass");
      const int q_slots = std::min(nprobe, 64);
      FV_TRY(ctx->scratch[12].reserve(a_rows * Kp * sizeof(uint16_t)));
      FV_TRY(ctx->scratch[13].reserve((a_rows * 4 + nq * size_t(q_slots + 2)) * sizeof(uint32_t) + 64));
      FV_TRY(ctx->scratch[14].reserve(max_tasks * (sizeof(uint4) + 2 * sizeof(uint32_t)) +
                                      (ix.nlist + 8 + size_t(ctx->sm_count) + max_tiles + 2) * sizeof(uint32_t)));
      // per CTA; the fullest pool measured holds four to six times the average
      pool_cap = unsigned(std::min<size_t>(size_t(1) << 21, std::max<size_t>(65536, nq * 4096 / size_t(ctx->sm_count))));
      if (ix.survivor_slots) pool_cap = unsigned(ix.survivor_slots);
      FV_TRY(ctx->scratch[15].reserve(size_t(ctx->sm_count) * pool_cap * sizeof(u64)));
      qg = ctx->scratch[12].as<uint16_t>();
      thr = ctx->scratch[13].as<float>();
      g_q = reinterpret_cast<uint32_t*>(thr + a_rows);
      g_l = g_q + a_rows;
      g_base = reinterpret_cast<float*>(g_l + a_rows);
      uint32_t* q_rows = reinterpret_cast<uint32_t*>(g_base + a_rows);
      uint32_t* q_cnt = q_rows + nq * size_t(q_slots);
      dropped = q_cnt + nq;
      tasks = ctx->scratch[14].as<uint4>();
      task_moff = reinterpret_cast<uint32_t*>(tasks + max_tasks);
      task_rows = task_moff + max_tasks;
      a_off = task_rows + max_tasks;
      ntasks = a_off + ix.nlist;
      pool_cnt = ntasks + 8;
      tile_task0 = pool_cnt + ctx->sm_count;
      ga.list_off = ix.list_off;
      ga.a_off = a_off;
      ga.queries = q;
      ga.centroids = ix.centroids;
      ga.tau_bits = tau_bits;
      ga.cand_cnt = pb_set.per_query;
      ga.cap = cap;
      ga.pd = ix.pd;
      ga.Kp = ti.Kp;
      ga.is_l2 = ix.metric == FV_L2 ? 1 : 0;
      ga.bf16 = ti.bf16 ? 1 : 0;
      ga.kf = float(ti.Kp);
      ga.bn = std::sqrt(ti.max_norm2);
      ga.cw2 = ix.cen_norm2_max + ix.code_norm2_max;
      ga.c1 = 4.f * float(ix.pd / 8 + ix.m + 3 * ix.dsub + 24);
      ga.qg = qg;
      ga.thr = thr;
      ga.g_q = g_q;
      ga.g_l = g_l;
      ga.g_base = g_base;
      // Operand tiles of 128 rows instead of 256 when a list has few pairs: the pass costs a tile's multiplications
      // whatever the tile holds.  Estimated from the averages (pairs per list), per pass.
      const double avg_len = double(ix.nrows) / double(std::max<size_t>(1, ix.nlist));
      const double pairs_b_per_list = double(nq) * double(nprobe) / double(std::max<size_t>(1, ix.nlist));
      const double lists_a = std::min(double(nprobe), std::max(1.0, std::ceil(double(bound_rows_tc) / std::max(1.0, avg_len))));
      const double pairs_a_per_list = double(nq) * lists_a / double(std::max<size_t>(1, ix.nlist));
      const double tr_max = 1000.0;  // 128-row tiles never issue more MMA rows than 256-row ones, only more B-tile reads
      tr_a = pairs_a_per_list <= tr_max ? 128u : 256u;
      tr_b = pairs_b_per_list <= tr_max ? 128u : 256u;
      // ---- the bound pass on the tensor cores: the near pairs' rows scored, the minimum of every 32 kept
      if (!mini_bound) {
      size_t mfloats = std::max<size_t>(size_t(1) << 20, nq * 4096);
      mfloats = std::min<size_t>(mfloats, size_t(1) << 30);
      FV_TRY(ctx->scratch[6].reserve(mfloats * sizeof(float)));
      FV_CUDA(cudaMemsetAsync(q_cnt, 0, nq * sizeof(uint32_t), ctx->stream));
      tc_tasks_kernel<<<1, 1024, 0, ctx->stream>>>(pa_set.pair_off, ix.list_off, ix.roff8, ix.roff8 + ix.nlist + 1, ix.nlist, tasks,
                                                   a_off, tile_task0, uint32_t(max_tasks), ntasks, nullptr, task_moff, task_rows,
                                                   uint32_t(mfloats), tr_a);
      GatherArgs gb = ga;
      gb.tile_rows = tr_a;
      gb.pair_off = pa_set.pair_off;
      gb.pairs = pairs_a;
      gb.q_rows = q_rows;
      gb.q_cnt = q_cnt;
      gb.q_slots = q_slots;
      tc_gather_kernel<<<dim3(unsigned(ix.nlist), 4), 256, 0, ctx->stream>>>(gb);
      ctx->stats.launches += 2;
      FV_CUDA(cudaGetLastError());
      int g0 = 0;
      FV_TRY(tc_list_pass(ctx, ix.recon, ix.metric, qg, a_rows, nullptr, tasks, ntasks, ntasks + 1, nullptr, pool_cnt, 0, nullptr, nullptr, &g0,
                          int(tr_a), ctx->scratch[6].as<float>(), task_moff, task_rows));
      // bounds looked at per query: room for twice the 32-row minima of the rows the bound pass aims at
      int vcap = 2048;
      while (vcap < 16384 && size_t(vcap) < 2 * size_t(bound_rows_tc / 32) + 512) vcap <<= 1;
      const int wpb = vcap <= 4096 ? 4 : 1;  // warps (queries) per block, by the shared memory their bounds take
      const size_t ssmem = size_t(wpb) * vcap * sizeof(uint32_t);
      FV_CUDA(cudaFuncSetAttribute(tc_bound_select_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(ssmem)));
      tc_bound_select_kernel<<<unsigned((nq + wpb - 1) / wpb), wpb * 32, ssmem, ctx->stream>>>(
          ctx->scratch[6].as<float>(), tasks, tile_task0, task_moff, task_rows, thr, q_rows, q_cnt, q_slots, vcap, keep, nq, tau_bits,
          tr_a == 128u ? 7 : 8);
      ctx->stats.launches++;
      FV_CUDA(cudaGetLastError());
      }
    } else {
      la.pair_off = pa_set.pair_off;
      la.task_off = pa_set.task_off;
      la.pairs = pairs_a;
      la.counters = pa_set.counters;
      la.minima = ctx->scratch[6].as<float>();
      la.minima_cnt = pa_set.per_query;
      la.minima_cap = int(mcap);
      FV_TRY(ctx->scratch[6].reserve(nq * mcap * sizeof(float)));
      la.minima = ctx->scratch[6].as<float>();
      auto bound_k = use_pre ? ivfpq_list_scan_kernel<true, true> : ivfpq_list_scan_kernel<false, true>;
      FV_CUDA(cudaFuncSetAttribute(bound_k, cudaFuncAttributeMaxDynamicSharedMemorySize, int(LS_SMEM)));
      bound_k<<<ctx->sm_count, LS_THREADS, LS_SMEM, ctx->stream>>>(la);
      {
        const int wpb = mcap <= 2048 ? 4 : 1;  // warps (queries) per block, by the shared memory their minima take
        const size_t ssmem = size_t(wpb) * mcap * sizeof(uint32_t);
        if (ssmem > 40 * 1024)
          FV_CUDA(cudaFuncSetAttribute(bound_select_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(ssmem)));
        bound_select_kernel<<<unsigned((nq + wpb - 1) / wpb), wpb * 32, ssmem, ctx->stream>>>(la.minima, la.minima_cnt, int(mcap),
                                                                                               keep, nq, tau_bits);
      }
      ctx->stats.launches += 2;
      FV_CUDA(cudaGetLastError());
    }
    stage_mark(ctx);  // 1
    FV_TRY(bucket_pairs(ctx, ix, cells, nq, nprobe, 0, pb_set, pairs_b, slot_of));
    u64* cand = ctx->scratch[9].as<u64>();
    uint32_t* cand_cnt = pb_set.per_query;
    RescoreArgs ra{};
    int tc_grid = 0;
    if (path == LIST_TABLE) {
      stage_mark(ctx);  // 2
      la.pair_off = pb_set.pair_off;
      la.task_off = pb_set.task_off;
      la.pairs = pairs_b;
      la.counters = pb_set.counters;
      la.tau_bits = tau_bits;
      la.cand = cand;
      la.cand_cnt = cand_cnt;
      la.cap = cap;
      la.rows_scanned = d_rows + 1;
      FV_CUDA(cudaFuncSetAttribute(main_k, cudaFuncAttributeMaxDynamicSharedMemorySize, int(LS_SMEM)));
      main_k<<<ctx->sm_count, LS_THREADS, LS_SMEM, ctx->stream>>>(la);
      ctx->stats.launches++;
      FV_CUDA(cudaGetLastError());
      stage_mark(ctx);  // 3
    } else {
      tc_tasks_kernel<<<1, 1024, 0, ctx->stream>>>(pb_set.pair_off, ix.list_off, ix.roff8, ix.roff8 + ix.nlist + 1, ix.nlist, tasks,
                                                   a_off, tile_task0, uint32_t(max_tasks), ntasks, d_rows + 1, nullptr, nullptr, 0u, tr_b);
      ga.tile_rows = tr_b;
      ga.pair_off = pb_set.pair_off;
      ga.pairs = pairs_b;
      tc_gather_kernel<<<dim3(unsigned(ix.nlist), 4), 256, 0, ctx->stream>>>(ga);
      ctx->stats.launches += 2;
      FV_CUDA(cudaGetLastError());
      stage_mark(ctx);  // 2
      FV_CUDA(cudaMemsetAsync(dropped, 0, nq * sizeof(uint32_t), ctx->stream));
      FV_TRY(tc_list_pass(ctx, ix.recon, ix.metric, qg, a_rows, thr, tasks, ntasks, ntasks + 1, ctx->scratch[15].as<u64>(), pool_cnt,
                          pool_cap, g_q, dropped, &tc_grid, int(tr_b)));
      stage_mark(ctx);  // 3
      ra.pool = ctx->scratch[15].as<u64>();
      ra.pool_cnt = pool_cnt;
      ra.pool_cap = pool_cap;
      ra.a_rows = a_rows;
      ra.nlist = uint32_t(ix.nlist);
      ra.nrows = ix.nrows;
      ra.npools = tc_grid;
      ra.g_q = g_q;
      ra.g_l = g_l;
      ra.g_base = g_base;
      ra.list_off = ix.list_off;
      ra.codes = ix.codes;
      ra.ids = ix.ids;
      ra.qtab = qtab;
      ra.pre = use_pre ? ix.pre : nullptr;
      ra.m = ix.m;
      ra.tau_bits = tau_bits;
      ra.cand = cand;
      ra.cand_cnt = cand_cnt;
      ra.cap = cap;
      rescore_kernel<<<unsigned(tc_grid) * 16, 128, size_t(tc_grid + 1) * sizeof(uint32_t), ctx->stream>>>(ra);
      ctx->stats.launches++;
      FV_CUDA(cudaGetLastError());
    }
    stage_mark(ctx);  // 4
    // the bound pass is done with its per-query counters: they become the marks of queries that get a second round
    uint32_t* redo = pa_set.per_query;
    FV_CUDA(cudaMemsetAsync(redo, 0, nq * sizeof(uint32_t), ctx->stream));
    FinishArgs fa{};
    fa.cand = cand;
    fa.cand_cnt = cand_cnt;
    fa.cap = cap;
    fa.counters = pb_set.counters;
    fa.tighten = path == LIST_TENSOR ? 1 : 0;  // the table scan keeps no survivor list to re-score
    fa.tau_bits = tau_bits;
    fa.redo = redo;
    fa.over_ids = pb_set.extra;
    fa.rerun_ids = pb_set.extra2;
    fa.dropped = dropped;
    int n2max = 32;
    while (n2max < cap || n2max < keep) n2max <<= 1;
    const size_t fsmem = (size_t(n2max) + size_t(keep) + size_t(k)) * sizeof(u64) + size_t(ix.pd) * sizeof(float);
    if (fsmem + 256 > ctx->smem_optin) return fail(FV_ERR_UNSUPPORTED, "k * refine too large for shared memory");
    if (fsmem > 40 * 1024)
      FV_CUDA(cudaFuncSetAttribute(ivfpq_finish_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(fsmem)));
    ivfpq_finish_kernel<<<unsigned(nq), 256, fsmem, ctx->stream>>>(a, fa, n2max);
    ctx->stats.launches++;
    FV_CUDA(cudaGetLastError());
    if (path == LIST_TENSOR) {
      // Second round, launched without asking the host: the queries whose buffer ran over (their count is a device
      // word) get their survivors re-scored against the tightened bounds and are finished from the list the first
      // round left.  Both kernels leave at once when there are none.
      ra.only = redo;
      ra.gate = pb_set.counters + LS_C_OVER;
      rescore_kernel<<<unsigned(tc_grid) * 16, 128, size_t(tc_grid + 1) * sizeof(uint32_t), ctx->stream>>>(ra);
      FinishArgs f2 = fa;
      f2.qids = fa.over_ids;
      f2.nqids = pb_set.counters + LS_C_OVER;
      f2.tighten = 0;
      ivfpq_finish_kernel<<<unsigned(std::min<size_t>(nq, size_t(ctx->sm_count) * 4)), 256, fsmem, ctx->stream>>>(a, f2, n2max);
      ctx->stats.launches += 2;
      FV_CUDA(cudaGetLastError());
    }
    // one read-back for the whole scan: counters, pool fill, the kernel's error word, rows scanned
    uint32_t h_ctr[LS_NCOUNTERS] = {};
    std::vector<unsigned int> h_pool(size_t(tc_grid) + 1, 0u);
    unsigned long long rows2[2] = {0, 0};
    FV_CUDA(cudaMemcpyAsync(h_ctr, pb_set.counters, sizeof(h_ctr), cudaMemcpyDeviceToHost, ctx->stream));
    if (tc_grid) {
      FV_CUDA(cudaMemcpyAsync(h_pool.data(), pool_cnt, size_t(tc_grid) * sizeof(unsigned int), cudaMemcpyDeviceToHost, ctx->stream));
      FV_CUDA(cudaMemcpyAsync(&h_pool[tc_grid], tc_error_word(ix.recon), sizeof(int), cudaMemcpyDeviceToHost, ctx->stream));
    }
    FV_CUDA(cudaMemcpyAsync(rows2, d_rows, sizeof(rows2), cudaMemcpyDeviceToHost, ctx->stream));
    FV_CUDA(cudaStreamSynchronize(ctx->stream));
    if (tc_grid && h_pool[tc_grid]) return fail(FV_ERR_TIMEOUT, "a bounded wait inside the tensor-core kernel ran out");
    // survivors of the tensor-core pass: pairs re-scored exactly (a pool that ran over dropped the rest, and the
    // finishing kernel has put the queries they belonged to on the re-run list)
    for (int c = 0; c < tc_grid; ++c) ctx->stats.dist_evals += std::min(h_pool[c], pool_cap);
    const uint32_t n_rerun = h_ctr[LS_C_RERUN];
    if (n_rerun) {  // whatever is left: those queries once more, by the per-query kernel (their rows are counted already)
      ScanArgs r = a;
      r.qids = fa.rerun_ids;
      r.rows_scanned = nullptr;
      FV_TRY(launch_block_scan(ctx, r, n_rerun, use_pre));
    }
    ctx->stats.regrown = h_ctr[LS_C_OVER];
    ctx->stats.uncertified = n_rerun;
    stage_mark(ctx);  // 5
    ctx->stats.rows_scanned = rows2[0] + rows2[1];
    ctx->stats.rows_list_scan = rows2[1];
    return FV_OK;
  }
  unsigned long long rows[2] = {0, 0};
  FV_CUDA(cudaMemcpyAsync(rows, d_rows, sizeof(rows), cudaMemcpyDeviceToHost, ctx->stream));
  FV_CUDA(cudaStreamSynchronize(ctx->stream));
  ctx->stats.rows_scanned = rows[0] + rows[1];
  ctx->stats.rows_list_scan = rows[1];
  return FV_OK;
}

}  // namespace fv
