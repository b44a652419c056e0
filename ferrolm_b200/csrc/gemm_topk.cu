// Tensor-core front end of exact search (flat.rs:40-53 at batch scale).
//
//   scores(q, b) = ||b||^2 - 2 <q, b>      (L2; the per-query constant ||q||^2 is left out)
//                = -<q, b>                 (inner product)
//
// computed as a 16-bit-input, fp32-accumulate GEMM on the 5th-generation tensor cores:
// tcgen05.mma issued by one thread, operands staged in shared memory by TMA with the 128-byte
// swizzle, accumulators in tensor memory.  The accumulator IS the score: the query operand is
// stored pre-multiplied by -2 (or -1), and for L2 one extra k step of 16 adds ||b||^2, split
// into three 16-bit pieces, inside the MMA.  The epilogue reads the accumulators back with
// tcgen05.ld (one query row per thread) and only compares.
//
// Two passes.  A sample pass over 1 base row in 32 keeps, per query, its best few scores in
// registers; the fifth best is that query's bound.  The main pass appends every row scoring below
// the bound to a candidate list.  A third kernel recomputes the reference's exact fp32 distance
// chain (src/kernels.rs:200-231) for those candidates, picks the k best by (distance, id) and
// CERTIFIES the result: a query passes only if every row that was not a candidate is provably
// farther than its k-th result.  Queries that do not pass are re-run by the full-precision scan,
// so the tensor cores never decide a result on their own.
//
// Work split: a unit is (query tile, 256 base rows); see make_tiling for how units become chunks
// and chunks are dealt to the persistent CTAs (one per SM) so that base tiles are shared in L2.
//
// Two tilings share the code:
//   MH = 2: 256 queries per tile, kept in shared memory for a whole chunk (K <= 128);
//           the two 128-row halves use the two accumulator slots, so each B tile is read once
//           from L2 for 256 queries.
//   MH = 1: 128 queries per tile (K <= 384); the two accumulator slots alternate between units.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <algorithm>
#include <atomic>
#include <cmath>

#include "internal.h"

namespace fv {

static constexpr int KP = 16;          // candidate slots per query and segment in the candidate buffer
static constexpr int TILE_N = 256;     // base rows per unit
static constexpr int KBLK = 64;        // k elements per shared-memory block (128 bytes)
static constexpr int A_BLOCK_BYTES = 128 * 128;   // 128 rows x 128 B
static constexpr int B_STAGE_BYTES = TILE_N * 128;
static constexpr int EXT_K = 16;                  // k elements of the norm step: one MMA
static constexpr int A_EXT_BYTES = 128 * EXT_K * 2;     // query side of the norm step
static constexpr int B_EXT_BYTES = TILE_N * EXT_K * 2;  // base side: one 8 KB tile per unit
static constexpr int NEPI = 16;        // epilogue warps: four per tensor-memory lane quadrant
static constexpr int LISTS = NEPI * 32; // per-thread lists of one segment
static constexpr int SCRATCH_BYTES = NEPI * 16 * 32 * 4;  // list mode only; per epilogue warp: 16 columns x 32 rows of scores
static constexpr int NTHREADS = 64 + NEPI * 32;   // warp 0 TMA, warp 1 MMA, warps 2..17 epilogue
static constexpr long long WAIT_LIMIT_CYCLES = 4000000000ll;  // about 2 s; then the kernel gives up

// ------------------------------------------------------------------------------------------------
// PTX wrappers
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return uint32_t(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// What a waiting thread needs to give up: the CTA's abort flag (shared memory) and the launch's limit in cycles.
struct AbortCtl {
  volatile int* flag;
  long long limit;
};

// Bounded wait.  Returns false when the limit ran out or another thread already gave up.
// Every failed probe reads shared memory, and the tensor cores fetch their operands through the same port:
// sixteen warps probing back to back slow the MMAs measurably, so a waiting thread sleeps between probes.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, const AbortCtl& abort_flag, unsigned sleep_ns = 64) {
  if (mbar_try(bar, parity)) return true;
  const long long t0 = clock64();
  for (;;) {
    for (int i = 0; i < 64; ++i) {
      if (sleep_ns) __nanosleep(sleep_ns);
      if (mbar_try(bar, parity)) return true;
    }
    if (*abort_flag.flag) return false;
    if (clock64() - t0 > abort_flag.limit) {
      *abort_flag.flag = 1;
      return false;
    }
  }
}

__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, uint64_t* bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(
          smem_u32(dst)),
      "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y)
      : "memory");
}

__device__ __forceinline__ void bulk_load_1d(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(dst)),
               "l"(src), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tc_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}

__device__ __forceinline__ void tc_mma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                           uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
      "}\n" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// 32 lanes x 32 columns of 32-bit accumulators: thread l of the warp gets lane (base + l), columns c..c+31.
// The load is asynchronous: the registers are valid only after tc_ld_wait on the same array, which takes
// them as in/out operands so that no use can be scheduled ahead of the wait.
__device__ __forceinline__ void tc_ld32_issue(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tc_ld_wait(uint32_t* r) {
  asm volatile("tcgen05.wait::ld.sync.aligned;"
               : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]),
                 "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15]),
                 "+r"(r[16]), "+r"(r[17]), "+r"(r[18]), "+r"(r[19]), "+r"(r[20]), "+r"(r[21]), "+r"(r[22]),
                 "+r"(r[23]), "+r"(r[24]), "+r"(r[25]), "+r"(r[26]), "+r"(r[27]), "+r"(r[28]), "+r"(r[29]),
                 "+r"(r[30]), "+r"(r[31])
               :
               : "memory");
}

// The same for 64 columns.
__device__ __forceinline__ void tc_ld64_issue(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x64.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, "
      "%32, %33, %34, %35, %36, %37, %38, %39, %40, %41, %42, %43, %44, %45, %46, %47, %48, %49, %50, %51, %52, %53, %54, %55, %56, %57, %58, %59, %60, %61, %62, %63}, [%64];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31]), "=r"(r[32]),
        "=r"(r[33]), "=r"(r[34]), "=r"(r[35]), "=r"(r[36]), "=r"(r[37]), "=r"(r[38]), "=r"(r[39]), "=r"(r[40]),
        "=r"(r[41]), "=r"(r[42]), "=r"(r[43]), "=r"(r[44]), "=r"(r[45]), "=r"(r[46]), "=r"(r[47]), "=r"(r[48]),
        "=r"(r[49]), "=r"(r[50]), "=r"(r[51]), "=r"(r[52]), "=r"(r[53]), "=r"(r[54]), "=r"(r[55]), "=r"(r[56]),
        "=r"(r[57]), "=r"(r[58]), "=r"(r[59]), "=r"(r[60]), "=r"(r[61]), "=r"(r[62]), "=r"(r[63])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tc_ld64_wait(uint32_t* r) {
  asm volatile("tcgen05.wait::ld.sync.aligned;"
               : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]), "+r"(r[8]),
                 "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15]), "+r"(r[16]),
                 "+r"(r[17]), "+r"(r[18]), "+r"(r[19]), "+r"(r[20]), "+r"(r[21]), "+r"(r[22]), "+r"(r[23]), "+r"(r[24]),
                 "+r"(r[25]), "+r"(r[26]), "+r"(r[27]), "+r"(r[28]), "+r"(r[29]), "+r"(r[30]), "+r"(r[31]), "+r"(r[32]),
                 "+r"(r[33]), "+r"(r[34]), "+r"(r[35]), "+r"(r[36]), "+r"(r[37]), "+r"(r[38]), "+r"(r[39]), "+r"(r[40]),
                 "+r"(r[41]), "+r"(r[42]), "+r"(r[43]), "+r"(r[44]), "+r"(r[45]), "+r"(r[46]), "+r"(r[47]), "+r"(r[48]),
                 "+r"(r[49]), "+r"(r[50]), "+r"(r[51]), "+r"(r[52]), "+r"(r[53]), "+r"(r[54]), "+r"(r[55]), "+r"(r[56]),
                 "+r"(r[57]), "+r"(r[58]), "+r"(r[59]), "+r"(r[60]), "+r"(r[61]), "+r"(r[62]), "+r"(r[63])
               :
               : "memory");
}

__device__ __forceinline__ float min3(float a, float b, float c) {
  float r;
  asm("min.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
  return r;
}

// Shared-memory matrix descriptor: K-major operand, 128-byte swizzle, rows of 128 bytes, groups of
// 8 rows 1024 bytes apart; bits 46-47 carry the descriptor version of this architecture.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t saddr) {
  uint64_t d = 0;
  d |= uint64_t((saddr & 0x3FFFF) >> 4);  // start address
  d |= uint64_t(1) << 16;                 // leading byte offset (unused with swizzle): 1
  d |= uint64_t(1024 >> 4) << 32;         // stride byte offset
  d |= uint64_t(1) << 46;                 // version
  d |= uint64_t(2) << 61;                 // SWIZZLE_128B
  return d;
}

// The same for a K = 16 operand: rows of 32 bytes with the 32-byte swizzle, groups of 8 rows 256 bytes apart.
__device__ __forceinline__ uint64_t smem_desc_sw32(uint32_t saddr) {
  uint64_t d = 0;
  d |= uint64_t((saddr & 0x3FFFF) >> 4);
  d |= uint64_t(1) << 16;
  d |= uint64_t(256 >> 4) << 32;
  d |= uint64_t(1) << 46;
  d |= uint64_t(6) << 61;                 // SWIZZLE_32B
  return d;
}

// Instruction descriptor of kind::f16: fp32 accumulate, A and B both K-major, M x N tile.
__host__ __device__ constexpr uint32_t make_idesc(int m, int n, bool bf16) {
  return (1u << 4) | ((bf16 ? 1u : 0u) << 7) | ((bf16 ? 1u : 0u) << 10) | (uint32_t(n >> 3) << 17) |
         (uint32_t(m >> 4) << 24);
}

// Ring position (stage index and phase bit), advanced without divisions: each role loop is a single thread on
// the critical path of the tensor pipe, and a 64-bit division per k block is a measurable bubble there.
struct StageCursor {
  int s, n;
  uint32_t phase;
  __device__ StageCursor(int n_) : s(0), n(n_), phase(0) {}
  __device__ __forceinline__ void next() {
    if (++s == n) {
      s = 0;
      phase ^= 1;
    }
  }
};

// ------------------------------------------------------------------------------------------------
struct GemmParams {
  int n, nq;
  int KB;          // 64-wide k blocks
  int NT;          // base tiles of 256 rows
  int MT;          // query tiles of 128 * MH rows
  int cpn;         // base tiles per chunk
  int nchunks;     // MT * parts; chunk g = part * MT + query tile, taken by CTA g % grid as its (g / grid)-th segment
  int segmax;      // segments per CTA
  int nstage;
  int scratch_bytes;  // SCRATCH_BYTES in list mode, 0 in threshold mode
  int has_ext;        // L2: one more k step of 16 adds the row norms inside the MMA
  int ext_ring;       // norm-step tiles (8 KB each) kept in shared memory
  uint32_t aext_c;    // 16-bit pattern of the constant the query side of the norm step holds
  const uint16_t* ext;  // base side of the norm step: 32 bytes per row, padded to whole tiles
  uint32_t idesc;
  u64* cand;           // [grid * segmax][LISTS][KP]  (list mode: output)
  int* err;            // set to 1 when a bounded wait ran out
  long long wait_limit;  // cycles a thread waits on one barrier before the kernel gives up (WAIT_LIMIT_CYCLES)
  int fault_skip_unit;   // test hook, -1 = off: the producer of work item 0 leaves out the loads of this unit of it
  // threshold mode: per-query bounds from the sample pass, and the candidate buffers they fill
  const float* tau;      // [MT * 128 * MH]
  u64* cbuf;             // [grid * segmax][LISTS][ccap] (score, row) keys: one private list per epilogue thread and segment
  unsigned int* ccnt;    // [grid * segmax][LISTS] entries appended (may exceed ccap: overflow)
  int ccap;
  // task mode (TASKS): the work is a table of (A tile, run of B units) pairs instead of the tiling above
  // x: first operand row of the 256-row A tile; y: first B row of the task; z: its B units of 256 rows (low 16 bits)
  // and the number of the first one within the run of B rows the task is a segment of (high 16 bits: survivors and
  // the valid-row test count rows from the start of that run); w: valid B rows of the run
  const uint4* tasks;
  const uint32_t* ntasks;      // device word: number of tasks
  unsigned int* next_task;     // device word, zero at launch: the next task nobody has taken yet
  u64* pool;                   // [grid][pool_cap] survivors: (A row << 32) | B row relative to y
  unsigned int* pool_cnt;      // [grid] entries each CTA produced (may exceed pool_cap: overflow)
  unsigned int pool_cap;
  // A survivor that finds its CTA's pool full is dropped, and the owner of its operand row (row_owner[A row], a
  // query number) is marked in owner_dropped so that the caller can hand that query to another kernel.
  const uint32_t* row_owner;
  uint32_t* owner_dropped;
  // task mode, minima variant (minima != null): instead of survivors, the smallest score of every 32 B rows, for the
  // first task_rows[t] operand rows of task t: minima[task_moff[t] + (row in tile * units + unit) * 8 + column / 32];
  // B rows beyond the task's valid ones count as +inf.  Tasks with task_moff[t] == 0xFFFFFFFF write nothing.
  float* minima;
  const uint32_t* task_moff;
  const uint32_t* task_rows;
};

struct __align__(8) Barriers {
  uint64_t full[8], empty[8];
  uint64_t a_full, a_empty;
  uint64_t tfull[2], tempty[2];
  uint32_t tmem_base;
  int abort_flag;
  unsigned int pool_pos;  // task mode: survivors this CTA has appended
  // task mode: the tasks this CTA has drawn, handed from the producer to the MMA and epilogue warps.  Entry
  // i & 7 holds the i-th draw (a value >= the task count ends the work); tq_full[i & 7] completes once per draw.
  uint64_t tq_full[8];
  unsigned int tq[8];
};

// Epilogue thread -> list index: warp group `sub` (0..3) * 128 + lane quadrant * 32 + lane.  MH = 2: sub & 1 is the
// 128-row half of the query tile, sub >> 1 the half of the 256 columns; MH = 1: sub is the column quarter.
// The li-th list that holds candidates of query row r of its tile:
__host__ __device__ __forceinline__ int list_of_row(int MH, int r, int li) {
  return MH == 2 ? ((r >> 7) + 2 * li) * 128 + (r & 127) : li * 128 + r;
}

// Sampling.  The sample pass scores 1 base row in E; a query's bound is its R-th best sampled score, so about R * E
// rows of the full set score below it (negative binomial) and the k nearest are among them unless R or more of the
// k - 1 nearest rows happen to be sampled: probability P(Binomial(k - 1, 1/E) >= R), kept below 2e-5 by the choice
// of R (5..13: k = 10 takes 5 to 7, k = 32 up to 13 -- with R capped at 7 a quarter of the queries of a k = 32
// search over 16384 rows failed their certificate and went to the full-precision scan).  E follows the base size
// (about sqrt(n / 1000)): the sample pass costs ~ n / E, the re-rank ~ R * E.
static constexpr int SAMPLE_R_MIN = 5, SAMPLE_R_MAX = 13;

static int pick_sample_every(size_t n) {
  int e = 8;
  while (e < 128 && double(e) * double(e) * 2000.0 < double(n)) e <<= 1;  // 1M -> 32, 125k -> 8, 6M -> 64
  return e;
}

static int pick_sample_r(int k, int every) {
  const double p = 1.0 / every;
  for (int r = SAMPLE_R_MIN; r < SAMPLE_R_MAX; ++r) {
    // P(Binomial(k - 1, p) >= r) by summing the lower tail
    double tail = 1.0, term = std::pow(1.0 - p, k - 1);
    for (int i = 0; i < r; ++i) {
      tail -= term;
      term *= double(k - 1 - i) / double(i + 1) * p / (1.0 - p);
    }
    if (tail < 2e-5) return r;
  }
  return SAMPLE_R_MAX;
}

// The R-th smallest score of every query over the lists the sample pass left (+inf when the sample holds fewer rows).
__global__ void sample_tau_kernel(const u64* __restrict__ lists, int MT, int parts, int grid, int segmax, int MH,
                                  int nq_pad, int R, float* __restrict__ tau) {
  const int q = blockIdx.x * blockDim.x + threadIdx.x;
  if (q >= nq_pad) return;
  const int rows_per_tile = 128 * MH;
  const int mt = q / rows_per_tile, r = q - mt * rows_per_tile;
  float best[SAMPLE_R_MAX];
#pragma unroll
  for (int j = 0; j < SAMPLE_R_MAX; ++j) best[j] = INFINITY;
  const int nl = MH == 2 ? 2 : 4;
  for (int part = 0; part < parts; ++part) {
    const int g = part * MT + mt;
    const int c = g % grid, seg = g / grid;
    for (int li = 0; li < nl; ++li) {
      const u64* src = lists + ((size_t(c) * segmax + seg) * LISTS + list_of_row(MH, r, li)) * KP;
#pragma unroll
      for (int j = 0; j < SAMPLE_R_MAX; ++j) {
        const u64 key = j < R ? src[j] : FV_EMPTY_KEY;  // a list holds R + 1 entries; the slots behind are stale
        if (key != FV_EMPTY_KEY) {
          float sc = key_distance(key);
#pragma unroll
          for (int t = 0; t < SAMPLE_R_MAX; ++t) {
            const bool lt = sc < best[t];
            const float tmp = best[t];
            best[t] = lt ? sc : tmp;
            sc = lt ? tmp : sc;
          }
        }
      }
    }
  }
  float out = INFINITY;
#pragma unroll
  for (int t = 0; t < SAMPLE_R_MAX; ++t)
    if (t == R - 1) out = best[t];
  tau[q] = out;
}

template <int MH, int KPT, bool THRESH, bool TASKS = false>
__global__ void __launch_bounds__(NTHREADS, 1)
    gemm_topk_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, GemmParams p) {
  unsigned char* raw = dyn_smem();
  unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(raw) + 1023) & ~uintptr_t(1023));
  unsigned char* sA = base;                                            // [MH][KB] blocks of 16 KB
  unsigned char* sAext = sA + size_t(MH) * p.KB * A_BLOCK_BYTES;       // 4 KB: the constant rows of the norm step
  unsigned char* sB = sAext + A_EXT_BYTES;                             // [nstage] stages of 32 KB
  unsigned char* sE = sB + size_t(p.nstage) * B_STAGE_BYTES;           // [ext_ring] norm-step tiles of 8 KB
  unsigned char* scratch = sE + size_t(p.ext_ring) * B_EXT_BYTES;      // list mode: 16 epilogue warps x 2 KB
  Barriers* bars = reinterpret_cast<Barriers*>(scratch + p.scratch_bytes);
  const AbortCtl abort_flag{&bars->abort_flag, p.wait_limit};

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int i = 0; i < 8; ++i) {
      mbar_init(&bars->full[i], 1);
      mbar_init(&bars->empty[i], 1);
    }
    mbar_init(&bars->a_full, 1);
    mbar_init(&bars->a_empty, 1);
    for (int i = 0; i < 8; ++i) mbar_init(&bars->tq_full[i], 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bars->tfull[i], 1);
      mbar_init(&bars->tempty[i], MH == 2 ? NEPI / 2 : NEPI);
    }
    bars->abort_flag = 0;
    bars->pool_pos = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  // Query side of the norm step: every row is {c, c, c, 0, 0, 0, 0, 0} twice.  Both 16-byte halves of a row are
  // equal, so the 32-byte swizzle (which only exchanges the halves of some rows) leaves the tile as written.
  if (threadIdx.x < A_EXT_BYTES / 16)
    reinterpret_cast<uint4*>(sAext)[threadIdx.x] = make_uint4(p.aext_c | (p.aext_c << 16), p.aext_c, 0u, 0u);
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  if (warp == 1) {  // the MMA warp owns the tensor memory: all 512 columns (one CTA per SM)
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 512;" ::"r"(smem_u32(&bars->tmem_base))
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = bars->tmem_base;
  // Work items.  Plain and threshold mode: chunk g of the tiling, CTA b taking g = b, b + grid, ...
  // Task mode: tasks cost very different amounts (their length, and how many survivors the epilogue has to append),
  // so they are not dealt in advance: the producer draws the next task from a device-wide counter whenever the
  // operand tile is free again, and passes the number on to the MMA and epilogue warps through a small ring in shared
  // memory.  The ring has 8 entries; the producer is at most 3 draws ahead of the slowest reader, because it draws
  // task i + 1 only after every MMA of task i - 1 has completed, by when the epilogue is at work on task i - 2 at
  // the latest (two accumulator slots).  The caller sorts the tasks by decreasing length: longest first.
  const int nwork = TASKS ? int(*p.ntasks) : p.nchunks;
  auto work_of = [&](int seg) -> int {  // consumer side
    if (!TASKS) return int(blockIdx.x) + seg * int(gridDim.x);
    if (!mbar_wait(&bars->tq_full[seg & 7], uint32_t(seg >> 3) & 1, abort_flag)) return 0x7FFFFFFF;
    return int(*reinterpret_cast<volatile unsigned int*>(&bars->tq[seg & 7]));
  };
  auto draw = [&](int seg) -> int {  // producer side
    if (!TASKS) return int(blockIdx.x) + seg * int(gridDim.x);
    const unsigned int g = min(atomicAdd(p.next_task, 1u), 0x7FFFFFFEu);
    bars->tq[seg & 7] = g;
    mbar_arrive(&bars->tq_full[seg & 7]);  // release: the entry is visible to whoever sees this phase complete
    return int(g);
  };

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer
    if (lane == 0) {
      bool ok = true;
      StageCursor st(p.nstage);
      int ring = 0;
      for (int seg = 0, g = draw(0); g < nwork && ok; g = draw(++seg)) {
        int nt0, nt1, a_row0, b_row0 = 0;
        if (TASKS) {
          const uint4 t = p.tasks[g];
          a_row0 = int(t.x);
          b_row0 = int(t.y);
          nt0 = 0;
          nt1 = int(t.z & 0xFFFFu);
        } else {
          const int part = g / p.MT, mt = g - part * p.MT;
          nt0 = part * p.cpn;
          nt1 = min(p.NT, nt0 + p.cpn);
          a_row0 = mt * MH * 128;
        }
        ok = mbar_wait(&bars->a_empty, (seg & 1) ^ 1, abort_flag);
        if (!ok) break;
        mbar_expect_tx(&bars->a_full, uint32_t(MH * p.KB * A_BLOCK_BYTES));
        for (int mh = 0; mh < MH; ++mh)
          for (int kb = 0; kb < p.KB; ++kb)
            tma_load_2d(sA + size_t(mh * p.KB + kb) * A_BLOCK_BYTES, &tmA, &bars->a_full, kb * KBLK, a_row0 + mh * 128);
        for (int nt = nt0; nt < nt1 && ok; ++nt) {
          for (int kb = 0; kb < p.KB; ++kb, st.next()) {
            const int s = st.s;
            ok = mbar_wait(&bars->empty[s], st.phase ^ 1, abort_flag);
            if (!ok) break;
            // The unit's norm-step tile rides on the barrier of its first k block.  Its ring slot is reused
            // ext_ring units later; the stage acquired just above was last read by a unit at most
            // ceil(nstage / KB) back, and the commit that freed it also covers every norm step issued before it.
            const bool with_ext = kb == 0 && p.has_ext;
            // (test hook: the stage is never posted, its consumer waits until the limit and the kernel gives up)
            if (p.fault_skip_unit >= 0 && g == 0 && nt == nt0 + p.fault_skip_unit) continue;
            mbar_expect_tx(&bars->full[s], uint32_t(B_STAGE_BYTES + (with_ext ? B_EXT_BYTES : 0)));
            // first B row of the unit (task mode: a multiple of 8, which keeps the norm tile's swizzle image in step)
            const size_t brow = size_t(b_row0) + size_t(nt) * TILE_N;
            if (with_ext)  // stored as the swizzled shared-memory image: one contiguous 8 KB copy
              bulk_load_1d(sE + size_t(ring) * B_EXT_BYTES, p.ext + brow * EXT_K, B_EXT_BYTES, &bars->full[s]);
            tma_load_2d(sB + size_t(s) * B_STAGE_BYTES, &tmB, &bars->full[s], kb * KBLK, int(brow));
          }
          if (++ring == p.ext_ring) ring = 0;
        }
      }
      // Do not leave while copies may still land in this CTA's shared memory: wait (bounded) until the
      // MMA side has consumed everything that was issued, or until the abort flag says nobody will.
      if (!ok) {
        const long long t0 = clock64();
        while (clock64() - t0 < 2000000) {
        }
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      int job = 0, ring = 0;
      bool ok = true;
      StageCursor st(p.nstage);
      const uint32_t a_base = smem_u32(sA), b_base = smem_u32(sB), e_base = smem_u32(sE);
      const uint64_t aext_desc = smem_desc_sw32(smem_u32(sAext));
      for (int seg = 0, g = work_of(0); g < nwork && ok; g = work_of(++seg)) {
        int nt0, nt1;
        if (TASKS) {
          nt0 = 0;
          nt1 = int(p.tasks[g].z & 0xFFFFu);
        } else {
          const int part = g / p.MT;
          nt0 = part * p.cpn;
          nt1 = min(p.NT, nt0 + p.cpn);
        }
        ok = mbar_wait(&bars->a_full, seg & 1, abort_flag);
        if (!ok) break;
        tc_fence_after();
        for (int nt = nt0; nt < nt1 && ok; ++nt) {
          for (int mh = 0; mh < MH && ok; ++mh, ++job) {
            const int slot = job & 1;
            ok = mbar_wait(&bars->tempty[slot], (uint32_t(job >> 1) & 1) ^ 1, abort_flag);
            if (!ok) break;
            tc_fence_after();
            const uint32_t d_tmem = tmem_base + uint32_t(slot * TILE_N);
            StageCursor sk = st;  // both halves walk the same stages of this unit
            uint32_t acc = 0;     // the first MMA of a job overwrites the accumulator
            for (int kb = 0; kb < p.KB; ++kb, sk.next()) {
              const int s = sk.s;
              if (mh == 0) {
                ok = mbar_wait(&bars->full[s], sk.phase, abort_flag);
                if (!ok) break;
                tc_fence_after();
              }
              if (kb == 0 && p.has_ext) {  // + ||b||^2: always the first step of a job
                tc_mma_f16(d_tmem, aext_desc, smem_desc_sw32(e_base + uint32_t(ring * B_EXT_BYTES)), p.idesc, 0u);
                acc = 1;
              }
              const uint32_t a_addr = a_base + uint32_t((mh * p.KB + kb) * A_BLOCK_BYTES);
              const uint32_t b_addr = b_base + uint32_t(s * B_STAGE_BYTES);
#pragma unroll
              for (int k4 = 0; k4 < KBLK / 16; ++k4)
                tc_mma_f16(d_tmem, smem_desc_sw128(a_addr + k4 * 32), smem_desc_sw128(b_addr + k4 * 32), p.idesc,
                           k4 != 0 ? 1u : acc);
              acc = 1;
              if (mh == MH - 1) tc_commit(&bars->empty[s]);  // the stage is free once these MMAs have read it
            }
            if (!ok) break;
            tc_commit(&bars->tfull[slot]);
          }
          for (int kb = 0; kb < p.KB; ++kb) st.next();
          if (++ring == p.ext_ring) ring = 0;
        }
        if (ok) tc_commit(&bars->a_empty);  // the query tile may be replaced once every MMA above has read it
      }
    }
  } else {
    // ---------------------------------------------------------------- epilogue: 16 warps, one query row per thread
    const int ew = warp - 2;
    const int quad = warp & 3;   // tensor-memory lanes this warp may read: 32 * quad .. +31
    const int sub = ew >> 2;     // warp group 0..3
    const int grp = MH == 2 ? (sub & 1) : 0;  // MH = 2: which 128-row half (= accumulator slot)
    const int e = sub * 128 + quad * 32 + lane;  // list index inside a segment
    const uint32_t lane_addr = uint32_t(quad * 32) << 16;
    // list mode: the KPT best (score, id) of this thread's query row in the current segment, ascending by score;
    // rows arrive in ascending id order, so a strict score compare keeps the (score, id) order
    float sc[KPT];
    uint32_t idv[KPT];
    float thr = INFINITY;
    size_t cslot = 0;        // this thread's list of the current segment
    unsigned int ncand = 0;
    float* sv = reinterpret_cast<float*>(scratch) + size_t(ew) * 512;  // list mode: 16 columns x 32 rows of scores
    int tile_idx = 0;
    bool ok = true;
    constexpr int NCOL = MH == 2 ? TILE_N / 2 : TILE_N / 4;
    const int col0 = MH == 2 ? (sub >> 1) * NCOL : sub * NCOL;
    uint32_t n_rows = uint32_t(p.n);
    uint32_t a_row = 0;  // task mode: this thread's operand row
    uint32_t unit0 = 0;  // task mode: number of the task's first unit within its B run
    float* mdst = nullptr;  // task mode, minima variant: where this thread's minima of the current task go
    for (int seg = 0, g = work_of(0); g < nwork && ok; g = work_of(++seg)) {
      int nt0, nt1, mt = 0;
      if (TASKS) {
        const uint4 t = p.tasks[g];
        nt0 = 0;
        nt1 = int(t.z & 0xFFFFu);
        unit0 = t.z >> 16;
        n_rows = t.w;  // rows of this task's B run; the rest of its last unit belongs to someone else
        a_row = t.x + uint32_t((MH == 2 ? grp * 128 : 0) + quad * 32 + lane);
        if (p.minima) {
          const uint32_t moff = p.task_moff[g];
          const uint32_t rt = a_row - t.x;
          mdst = (moff != 0xFFFFFFFFu && rt < p.task_rows[g]) ? p.minima + size_t(moff) + size_t(rt) * (t.z & 0xFFFFu) * 8 : nullptr;
        }
      } else {
        const int part = g / p.MT;
        mt = g - part * p.MT;
        nt0 = part * p.cpn;
        nt1 = min(p.NT, nt0 + p.cpn);
      }
      cslot = (size_t(blockIdx.x) * p.segmax + seg) * LISTS + e;
      ncand = 0;
      if (THRESH) {  // the bound is fixed: the sample pass's estimate for this query
        thr = TASKS ? (p.minima ? 0.f : p.tau[a_row]) : p.tau[mt * (128 * MH) + (MH == 2 ? grp * 128 : 0) + quad * 32 + lane];
      } else {
        thr = INFINITY;
#pragma unroll
        for (int j = 0; j < KPT; ++j) {
          sc[j] = INFINITY;
          idv[j] = 0xFFFFFFFFu;
        }
      }
      for (int nt = nt0; nt < nt1 && ok; ++nt, ++tile_idx) {
        const int job = MH == 2 ? tile_idx * 2 + grp : tile_idx;
        const int slot = job & 1;
        ok = mbar_wait(&bars->tfull[slot], uint32_t(job >> 1) & 1, abort_flag);
        if (!ok) break;
        tc_fence_after();
        const uint32_t row_base = (unit0 + uint32_t(nt)) * TILE_N + col0;
        const uint32_t t_addr = tmem_base + lane_addr + uint32_t(slot * TILE_N + col0);
        if (THRESH) {
          // Threshold mode.  The accumulator IS the score (the norm step and the scaled query side put
          // ||b||^2 - 2<q,b> there), so a chunk of 64 columns costs a minimum tree and one vote.  Every column
          // below the bound is appended to this thread's private list: a plain store and a register counter.
          // (Issuing the next load before working on this one was tried and ran slower than this plain loop.)
          auto chunk = [&](const uint32_t* r, int c) {
            float g8[8];
#pragma unroll
            for (int gi = 0; gi < 8; ++gi) {
              const uint32_t* q = r + gi * 8;
              const float t0 = min3(__uint_as_float(q[0]), __uint_as_float(q[1]), __uint_as_float(q[2]));
              const float t1 = min3(__uint_as_float(q[3]), __uint_as_float(q[4]), __uint_as_float(q[5]));
              g8[gi] = fminf(min3(t0, t1, __uint_as_float(q[6])), __uint_as_float(q[7]));
            }
            const float m = fminf(min3(g8[0], g8[1], g8[2]), min3(min3(g8[3], g8[4], g8[5]), g8[6], g8[7]));
            if (__any_sync(FV_FULL, m < thr)) {
              u64* cl = p.cbuf + cslot * size_t(p.ccap);
#pragma unroll
              for (int gi = 0; gi < 8; ++gi) {
                if (__any_sync(FV_FULL, g8[gi] < thr)) {
#pragma unroll
                  for (int i = gi * 8; i < gi * 8 + 8; ++i) {
                    const float v = __uint_as_float(r[i]);
                    const uint32_t row = row_base + uint32_t(c + i);
                    if (v < thr && row < n_rows) {
                      if (ncand < unsigned(p.ccap)) cl[ncand] = make_key(v, row);
                      ncand++;
                    }
                  }
                }
              }
            }
          };
          // Task mode.  Survivors are dense where a query meets its own neighbourhood (one row in ten of a near list),
          // so the append must not cost a shared-memory atomic per hit: every thread collects its hits of the chunk
          // as two bit masks, the warp reserves room for all of them with ONE atomic on the CTA's counter, and each
          // thread stores its own.
          auto chunk_tasks = [&](const uint32_t* r, int c) {
            float m = __uint_as_float(r[0]);
#pragma unroll
            for (int i = 1; i < 64; ++i) m = fminf(m, __uint_as_float(r[i]));
            if (!__any_sync(FV_FULL, m < thr)) return;
            uint32_t mk[2] = {0u, 0u};
#pragma unroll
            for (int i = 0; i < 64; ++i)
              if (__uint_as_float(r[i]) < thr && row_base + uint32_t(c + i) < n_rows) mk[i >> 5] |= 1u << (i & 31);
            const int mine = __popc(mk[0]) + __popc(mk[1]);
            int incl = mine;  // inclusive prefix sum over the warp
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
              const int t = __shfl_up_sync(FV_FULL, incl, o);
              if (lane >= o) incl += t;
            }
            const int total = __shfl_sync(FV_FULL, incl, 31);
            if (total == 0) return;
            unsigned int base = 0;
            if (lane == 31) base = atomicAdd(&bars->pool_pos, unsigned(total));
            base = __shfl_sync(FV_FULL, base, 31);
            unsigned int pos = base + unsigned(incl - mine);
            u64* dst = p.pool + size_t(blockIdx.x) * p.pool_cap;
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              uint32_t mm = mk[h];
              while (mm) {
                const int i = __ffs(mm) - 1;
                mm &= mm - 1;
                if (pos < p.pool_cap) dst[pos] = (u64(a_row) << 32) | u64(row_base + uint32_t(c + h * 32 + i));
                ++pos;
              }
            }
            if (mine && pos > p.pool_cap) p.owner_dropped[p.row_owner[a_row]] = 1u;  // some of this row's did not fit
          };
          uint32_t rbuf[64];
#pragma unroll 1
          for (int c = 0; c < NCOL; c += 64) {
            tc_ld64_issue(t_addr + uint32_t(c), rbuf);
            tc_ld64_wait(rbuf);
            if (c + 64 == NCOL) {  // the last load has landed: the MMA may overwrite this accumulator slot
              tc_fence_before();
              __syncwarp();
              if (lane == 0) mbar_arrive(&bars->tempty[slot]);
            }
            if (TASKS) {
              if (p.minima) {
                // minima variant: the smallest score of every 32 columns of this chunk, rows beyond the task's as +inf
                if (mdst) {
                  float g2[2];
                  const bool tail = row_base + uint32_t(c + 63) >= n_rows;
#pragma unroll
                  for (int gi = 0; gi < 2; ++gi) {
                    float m = INFINITY;
#pragma unroll
                    for (int i = gi * 32; i < gi * 32 + 32; ++i) {
                      const float v = __uint_as_float(rbuf[i]);
                      m = fminf(m, (!tail || row_base + uint32_t(c + i) < n_rows) ? v : INFINITY);
                    }
                    g2[gi] = m;
                  }
                  *reinterpret_cast<float2*>(mdst + size_t(nt) * 8 + (col0 + c) / 32) = make_float2(g2[0], g2[1]);
                }
              } else {
                chunk_tasks(rbuf, c);
              }
            } else {
              chunk(rbuf, c);
            }
          }
        } else {
          // List mode.  Common path: the minimum of a chunk against the bound.  Rare path (entered by the whole
          // warp when any of its 32 rows has a column below its bound): the scores are parked in this warp's
          // shared-memory scratch so that they can be indexed, and each row inserts its passing columns, in
          // ascending id order, into its sorted register list.
          uint32_t rbuf[32];
#pragma unroll 1
          for (int c = 0; c < NCOL; c += 32) {
            tc_ld32_issue(t_addr + uint32_t(c), rbuf);
            tc_ld_wait(rbuf);
            float m = INFINITY;
#pragma unroll
            for (int i = 0; i < 32; i += 2) m = min3(m, __uint_as_float(rbuf[i]), __uint_as_float(rbuf[i + 1]));
            if (__any_sync(FV_FULL, m < thr)) {
#pragma unroll
              for (int h = 0; h < 2; ++h) {  // two halves of 16 columns, in id order; the scratch holds one half
                unsigned mask = 0;
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                  const float v = __uint_as_float(rbuf[h * 16 + i]);
                  sv[i * 32 + lane] = v;
                  mask |= (v < thr && row_base + uint32_t(c + h * 16 + i) < n_rows) ? (1u << i) : 0u;
                }
                while (__any_sync(FV_FULL, mask != 0)) {
                  if (mask) {
                    const int i = __ffs(mask) - 1;
                    mask &= mask - 1;
                    const float val = sv[i * 32 + lane];
                    if (val < thr) {
                      float cs = val;
                      uint32_t ci = row_base + uint32_t(c + h * 16 + i);
#pragma unroll
                      for (int j = 0; j < KPT; ++j) {
                        const bool lt = cs < sc[j];
                        const float ts = sc[j];
                        const uint32_t ti = idv[j];
                        sc[j] = lt ? cs : ts;
                        idv[j] = lt ? ci : ti;
                        cs = lt ? ts : cs;
                        ci = lt ? ti : ci;
                      }
                      thr = sc[KPT - 1];
                    }
                  }
                }
              }
            }
          }
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&bars->tempty[slot]);
        }
      }
      if (!ok) break;
      if (THRESH) {
        if (!TASKS) p.ccnt[cslot] = ncand;
      } else {
        u64* dst = p.cand + cslot * KP;
#pragma unroll
        for (int j = 0; j + 1 < KPT; j += 2) {
          const u64 k0 = idv[j] == 0xFFFFFFFFu ? FV_EMPTY_KEY : make_key(sc[j], idv[j]);
          const u64 k1 = idv[j + 1] == 0xFFFFFFFFu ? FV_EMPTY_KEY : make_key(sc[j + 1], idv[j + 1]);
          *reinterpret_cast<ulonglong2*>(dst + j) = make_ulonglong2(k0, k1);
        }
        if (KPT & 1) dst[KPT - 1] = idv[KPT - 1] == 0xFFFFFFFFu ? FV_EMPTY_KEY : make_key(sc[KPT - 1], idv[KPT - 1]);
      }
    }
  }

  // ---------------------------------------------------------------- teardown
  tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0 && *abort_flag.flag) atomicExch(p.err, 1);
  if (TASKS && threadIdx.x == 0) p.pool_cnt[blockIdx.x] = bars->pool_pos;
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 512;" ::"r"(tmem_base) : "memory");
  }
}

// ------------------------------------------------------------------------------------------------
// fp32 rows -> 16-bit operand rows (zero padded to Kp), squared norms and range statistics
struct RangeStats {
  float min_v, max_v;      // over all values seen
  float max_norm2;         // largest squared row norm
  int not_integer;         // some value is not integer-valued
  int not_finite;
};

__device__ __forceinline__ void atomic_min_f(float* a, float v) {
  if (v >= 0) atomicMin(reinterpret_cast<int*>(a), __float_as_int(v));
  else atomicMax(reinterpret_cast<unsigned*>(a), __float_as_uint(v));
}
__device__ __forceinline__ void atomic_max_f(float* a, float v) {
  if (v >= 0) atomicMax(reinterpret_cast<int*>(a), __float_as_int(v));
  else atomicMin(reinterpret_cast<unsigned*>(a), __float_as_uint(v));
}

// one warp per row
template <bool BF16>
__global__ void convert_rows_kernel(const float* __restrict__ src, size_t n, int pd, int Kp, uint16_t* __restrict__ dst,
                                    float* __restrict__ norm2, int is_l2, float mul, RangeStats* __restrict__ st) {
  const int lane = threadIdx.x & 31;
  const size_t row = blockIdx.x * size_t(blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= n) return;
  float s = 0.f, mn = INFINITY, mx = -INFINITY;
  int bad_int = 0, bad_fin = 0;
  for (int c = lane; c < Kp; c += 32) {
    float x = c < pd ? src[row * size_t(pd) + c] : 0.f;
    if (c < pd) {
      s = __fmaf_rn(x, x, s);
      mn = fminf(mn, x);
      mx = fmaxf(mx, x);
      if (x != rintf(x)) bad_int = 1;
      if (!(fabsf(x) <= 3.0e38f)) bad_fin = 1;
    }
    uint16_t h;
    if (BF16) h = __bfloat16_as_ushort(__float2bfloat16_rn(x * mul));
    else h = __half_as_ushort(__float2half_rn(x * mul));
    dst[row * size_t(Kp) + c] = h;
  }
  for (int o = 16; o > 0; o >>= 1) {
    s += __shfl_xor_sync(FV_FULL, s, o);
    mn = fminf(mn, __shfl_xor_sync(FV_FULL, mn, o));
    mx = fmaxf(mx, __shfl_xor_sync(FV_FULL, mx, o));
    bad_int |= __shfl_xor_sync(FV_FULL, bad_int, o);
    bad_fin |= __shfl_xor_sync(FV_FULL, bad_fin, o);
  }
  if (lane == 0) {
    if (norm2) norm2[row] = is_l2 ? s : 0.f;
    atomic_min_f(&st->min_v, mn);
    atomic_max_f(&st->max_v, mx);
    atomic_max_f(&st->max_norm2, s);
    if (bad_int) st->not_integer = 1;
    if (bad_fin) st->not_finite = 1;
  }
}

// Base side of the norm step: ||b||^2 / 2^e as three 16-bit pieces (p0 + p1 + p2, each the rounding of what the
// ones before left), then 13 zeros.  The query side holds 2^e three times, so the MMA adds the norm back exactly
// to 24 bits (fp16: 3 x 11 bits, bf16: 3 x 8).  Rows with a non-finite norm (the padding is +inf) get +inf.
// The array is kept as the shared-memory image of the 32-byte swizzle (the two 16-byte halves of a row trade
// places in rows 4..7 of every 8), so that a tile is one contiguous bulk copy instead of 256 narrow TMA rows.
template <bool BF16>
__global__ void split_norms_kernel(const float* __restrict__ norm2, size_t first, size_t count, float inv_scale,
                                   uint16_t* __restrict__ ext) {
  const size_t i = blockIdx.x * size_t(blockDim.x) + threadIdx.x;
  if (i >= count) return;
  const size_t row = first + i;
  const float t = norm2[row] * inv_scale;
  uint16_t pc[3] = {0, 0, 0};
  if (!(fabsf(t) < INFINITY)) {
    pc[0] = BF16 ? 0x7F80 : 0x7C00;
  } else {
    float r = t;
#pragma unroll
    for (int j = 0; j < 3; ++j) {
      float back;
      if (BF16) {
        const __nv_bfloat16 h = __float2bfloat16_rn(r);
        pc[j] = __bfloat16_as_ushort(h);
        back = __bfloat162float(h);
      } else {
        const __half h = __float2half_rn(r);
        pc[j] = __half_as_ushort(h);
        back = __half2float(h);
      }
      if (!(fabsf(back) < INFINITY)) break;  // beyond the 16-bit range: the row scores +inf and is never a candidate
      r = __fsub_rn(r, back);
    }
  }
  uint4* dst = reinterpret_cast<uint4*>(ext + row * EXT_K);
  const int sw = int(row >> 2) & 1;
  dst[sw] = make_uint4(uint32_t(pc[0]) | (uint32_t(pc[1]) << 16), uint32_t(pc[2]), 0u, 0u);
  dst[sw ^ 1] = make_uint4(0u, 0u, 0u, 0u);
}

__global__ void fill_f32_kernel(float* p, size_t n, float v) {
  for (size_t i = blockIdx.x * size_t(blockDim.x) + threadIdx.x; i < n; i += size_t(gridDim.x) * blockDim.x) p[i] = v;
}

__global__ void init_stats_kernel(RangeStats* st) {
  st->min_v = INFINITY;
  st->max_v = -INFINITY;
  st->max_norm2 = 0.f;
  st->not_integer = 0;
  st->not_finite = 0;
}

// ------------------------------------------------------------------------------------------------
// Exact re-rank and certification: one warp per query.
struct RerankParams {
  const float* tau;       // the bound every candidate was tested against
  const u64* cbuf;        // candidates of the main pass: [grid * segmax][LISTS][ccap]
  const unsigned int* ccnt;
  int ccap, MT, parts, grid, segmax;  // main-pass tiling
  const float* rows;      // n x pd fp32
  const float* queries;   // nq x pd fp32
  const float* qnorm2;    // nq (0 for inner product)
  const RangeStats* bst;  // base statistics
  const RangeStats* qst;  // query statistics
  int n, nq, pd, Kp, k, MH, is_l2, bf16;
  uint32_t id_base;
  u64* out_keys;          // nq x k
  uint32_t* retry_ids;    // queries that did not certify
  unsigned int* retry_count;
};

__global__ void rerank_kernel(RerankParams p) {
  unsigned char* smem_raw = dyn_smem();
  const int W = blockDim.x >> 5, w = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const size_t q = size_t(blockIdx.x) * W + w;
  if (q >= size_t(p.nq)) return;
  float* sq = reinterpret_cast<float*>(smem_raw) + size_t(w) * p.pd;
  u64* list = reinterpret_cast<u64*>(smem_raw + size_t(W) * p.pd * sizeof(float)) + size_t(w) * p.k;
  float* stage = reinterpret_cast<float*>(smem_raw + ((size_t(W) * (size_t(p.pd) * 4 + size_t(p.k) * 8) + 15) & ~size_t(15))) +
                 size_t(w) * 8 * quad_stride(p.pd);  // two stage buffers
  for (int c = lane; c < p.pd; c += 32) sq[c] = p.queries[q * size_t(p.pd) + c];
  warp_list_init(list, p.k);

  // exact-arithmetic regime: integer-valued inputs small enough that every product, partial sum and
  // distance is an integer below 2^24 in both the tensor-core score and the reference's fp32 chain
  const float lo = fminf(p.bst->min_v, p.qst->min_v), hi = fmaxf(p.bst->max_v, p.qst->max_v);
  const float mabs = fmaxf(fabsf(lo), fabsf(hi)), range = hi - lo;
  // the accumulator starts at ||b||^2 <= Kp mabs^2 and then takes the terms -2 q_i b_i: it stays within
  // [-2 Kp mabs^2, Kp mabs^2 + 2 Kp |lo hi|], the upper end only when the values take both signs
  const float negprod = (lo < 0.f && hi > 0.f) ? -lo * hi : 0.f;
  const bool exact_regime = !p.bst->not_integer && !p.qst->not_integer && !p.bst->not_finite && !p.qst->not_finite &&
                            mabs <= (p.bf16 ? 256.f : 2048.f) && float(p.Kp) * mabs * mabs <= 8388608.f &&
                            float(p.Kp) * (mabs * mabs + 2.f * negprod) <= 16777216.f &&
                            float(p.Kp) * range * range < 16777216.f;
  const float qn2 = p.qnorm2[q];
  // error bound of a score against the reference distance (minus ||q||^2 for L2) outside that regime
  const float u16 = p.bf16 ? 0.00390625f : 0.00048828125f;
  const float qn = sqrtf(p.is_l2 ? qn2 : 0.f), bn = sqrtf(p.bst->max_norm2);
  float eps;
  // The query operand of the GEMM is this row times -2 (L2) or -1 in the 16-bit type.  A component that leaves that
  // type's range (fp16: 65504) turns every score of the query into +-inf or NaN, so no row is a candidate and the
  // reasoning below ("a row that is not a candidate scores above the bound") says nothing: such a query is never
  // certified here and goes to the full-precision scan, which returns the reference's k finite neighbours.
  bool q_in_range;
  {
    // inner-product case needs the query norm too; it is recomputed here from the staged query
    float s = 0.f, qmax = 0.f;
    bool fin = true;
    for (int c = lane; c < p.pd; c += 32) {
      s = __fmaf_rn(sq[c], sq[c], s);
      qmax = fmaxf(qmax, fabsf(sq[c]));
      fin = fin && fabsf(sq[c]) <= 3.0e38f;  // false for inf and NaN
    }
    for (int o = 16; o > 0; o >>= 1) {
      s += __shfl_xor_sync(FV_FULL, s, o);
      qmax = fmaxf(qmax, __shfl_xor_sync(FV_FULL, qmax, o));
    }
    fin = __all_sync(FV_FULL, fin);
    const float scale = p.is_l2 ? 2.f : 1.f;
    q_in_range = fin && (p.bf16 ? qmax <= 1.0e38f : qmax * scale <= 65504.f);
    const float qnorm = p.is_l2 ? qn : sqrtf(s);
    const float kf = float(p.Kp);
    const float e_dot = (2.f * u16 * (1.f + u16) + kf * 4.7683716e-7f + kf * 1.1920929e-7f) * qnorm * bn +
                        5.9604645e-8f * sqrtf(kf) * (qnorm + bn);
    // L2: the norm is added inside the MMA (its split loses < 2^-24 of the largest norm, the accumulation
    // about 2^-21 per step of a partial sum that now includes it), then the reference chain's own rounding
    const float e_norm = (kf + 16.f) * 4.7683716e-7f * bn * bn + 1.1920929e-7f * bn * bn;
    eps = p.is_l2 ? 2.f * e_dot + e_norm + kf * 2.3841858e-7f * (qnorm * qnorm + bn * bn) * 2.f : e_dot;
    eps = exact_regime ? 0.f : eps * 1.01f + 1e-30f;
  }

  const int rows_per_tile = 128 * p.MH;
  const int mt = int(q / rows_per_tile), r = int(q % rows_per_tile);
  // every row whose score is below tau is in the buffer; every other row scores >= tau
  const float tau = p.tau[q];
  bool overflow = false;
  bool mismatch = false;  // exact regime only: a score that is not the exact distance
  u64 bound = FV_EMPTY_KEY;
  const int lists_per_seg = p.MH == 2 ? 2 : 4;
  // The candidates of this query sit in parts * lists_per_seg short lists.  32 lists at a time: each lane looks up
  // one list's count, a prefix sum lines the entries up, and the warp walks them 32 per step (a lane finds the
  // list of its entry by bisection over the prefix sums), so every step computes 32 exact distances.
  const int nlist = p.parts * lists_per_seg;
  for (int l0 = 0; l0 < nlist; l0 += 32) {
    const int l = l0 + lane;
    unsigned int cnt = 0;
    unsigned long long slot = 0;
    if (l < nlist) {
      const int part = l / lists_per_seg, li = l - part * lists_per_seg;
      const int g = part * p.MT + mt;
      const int c = g % p.grid, seg_local = g / p.grid;
      slot = (size_t(c) * p.segmax + seg_local) * LISTS + list_of_row(p.MH, r, li);
      cnt = p.ccnt[slot];
      if (cnt > unsigned(p.ccap)) {
        overflow = true;
        cnt = unsigned(p.ccap);
      }
    }
    unsigned int pre = cnt;  // inclusive prefix sum
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const unsigned int v = __shfl_up_sync(FV_FULL, pre, o);
      if (lane >= o) pre += v;
    }
    const unsigned int total = __shfl_sync(FV_FULL, pre, 31);
    for (unsigned int t0 = 0; t0 < total; t0 += 32) {
      const unsigned int x = t0 + lane;
      int j = 0;  // lists whose entries all come before entry x
#pragma unroll
      for (int step = 16; step > 0; step >>= 1) {
        const unsigned int pv = __shfl_sync(FV_FULL, pre, j + step - 1);
        if (pv <= x) j += step;
      }
      const unsigned int pj = __shfl_sync(FV_FULL, pre, j), cj = __shfl_sync(FV_FULL, cnt, j);
      const unsigned long long sj = __shfl_sync(FV_FULL, slot, j);
      u64 key = FV_EMPTY_KEY, ck = 0;
      uint32_t id = 0;
      bool have = false;
      if (x < total) {
        ck = p.cbuf[sj * size_t(p.ccap) + (x - (pj - cj))];
        id = key_id(ck);
        have = id < uint32_t(p.n);
        if (!have) mismatch = true;  // a padded row can only get here through a non-finite score
      }
      // four candidates' rows at a time (asynchronous coalesced gathers, 4 rows x 8 chain lanes)
      const float d = p.is_l2 ? quad_distances<true>(sq, p.rows, p.pd, id, have, stage)
                              : quad_distances<false>(sq, p.rows, p.pd, id, have, stage);
      if (have) {
        if (exact_regime && d != key_distance(ck) + qn2) mismatch = true;
        if (d < INFINITY) key = make_key(d, id + p.id_base);
      }
      bound = warp_list_offer(list, p.k, key, bound);
    }
  }
  __syncwarp();
  mismatch = __any_sync(FV_FULL, mismatch);
  overflow = __any_sync(FV_FULL, overflow);
  const u64 kth = list[p.k - 1];
  bool certified;
  if (overflow || mismatch || !q_in_range || !(tau == tau)) {
    certified = false;
  } else if (tau == INFINITY) {
    certified = true;  // every row with a finite score was a candidate
  } else {
    // the k-th result must be provably nearer than anything that was not a candidate
    certified = kth != FV_EMPTY_KEY && (key_distance(kth) - qn2) + eps < tau;
  }
  for (int e = lane; e < p.k; e += 32) p.out_keys[q * size_t(p.k) + e] = list[e];
  if (!certified && lane == 0) {
    const unsigned int slot = atomicAdd(p.retry_count, 1u);
    p.retry_ids[slot] = uint32_t(q);
  }
}

// rows of the strided sample: sample row i is base row floor(i * n / ns)
__global__ void gather_sample_kernel(const uint16_t* __restrict__ half, const float* __restrict__ norm2, size_t n, int Kp,
                                     size_t ns, uint16_t* __restrict__ samp, float* __restrict__ snorm) {
  const int lane = threadIdx.x & 31;
  const size_t i = blockIdx.x * size_t(blockDim.x >> 5) + (threadIdx.x >> 5);
  if (i >= ns) return;
  const size_t src = size_t((unsigned long long)i * n / ns);
  const uint4* a = reinterpret_cast<const uint4*>(half + src * size_t(Kp));
  uint4* b = reinterpret_cast<uint4*>(samp + i * size_t(Kp));
  for (int c = lane; c < Kp / 8; c += 32) b[c] = a[c];
  if (lane == 0) snorm[i] = norm2[src];
}

__global__ void scatter_keys_kernel(const u64* __restrict__ src, const uint32_t* __restrict__ qids, size_t nsub, int L,
                                    u64* __restrict__ dst) {
  for (size_t i = blockIdx.x * size_t(blockDim.x) + threadIdx.x; i < nsub * L; i += size_t(gridDim.x) * blockDim.x) {
    const size_t s = i / L;
    dst[size_t(qids[s]) * L + (i - s * L)] = src[i];
  }
}

// ------------------------------------------------------------------------------------------------
// host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

// rows x Kp 16-bit matrix, boxes of `box_rows` rows x 64 elements, 128-byte swizzle
static int make_tmap(CUtensorMap* map, bool bf16, void* ptr, size_t rows, int Kp, int box_rows) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return fail(FV_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  cuuint64_t gdim[2] = {cuuint64_t(Kp), cuuint64_t(rows)};
  cuuint64_t gstride[1] = {cuuint64_t(Kp) * 2};
  cuuint32_t box[2] = {cuuint32_t(KBLK), cuuint32_t(box_rows)};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, ptr, gdim, gstride,
                  box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(FV_ERR_CUDA, "cuTensorMapEncodeTiled failed with code " + std::to_string(int(r)));
  return FV_OK;
}

struct TcSide {
  int pd = 0, Kp = 0;
  bool bf16 = false;
  size_t n = 0;            // rows converted
  DevBuf half;             // n_cap x Kp 16-bit
  DevBuf norm2;            // padded to 256, +inf beyond n
  DevBuf stats;            // RangeStats (base), RangeStats (queries), retry counter, error word
  size_t ns = 0;           // rows of the strided sample
  int every = 32;          // 1 row in `every` is sampled
  DevBuf samp, samp_norm2; // the sample's operand rows and norms (+inf padded)
  DevBuf ext, samp_ext;    // norm pieces of the base rows and of the sample (padded like the norms), 32 B per row
  int ext_e = 0;           // the pieces hold ||b||^2 / 2^ext_e
  bool ext_valid = false;
  RangeStats h_stats{};
};

void tc_free(TcSide* tc) { delete tc; }

static inline int round_up(int x, int m) { return (x + m - 1) / m * m; }

static int convert(fv_ctx* ctx, bool bf16, const float* d_src, size_t n, int pd, int Kp, uint16_t* dst, float* norm2,
                   bool is_l2, float mul, RangeStats* st) {
  if (n == 0) return FV_OK;
  const int wpb = 8;
  const unsigned blocks = unsigned((n + wpb - 1) / wpb);
  if (bf16)
    convert_rows_kernel<true><<<blocks, wpb * 32, 0, ctx->stream>>>(d_src, n, pd, Kp, dst, norm2, is_l2 ? 1 : 0, mul, st);
  else
    convert_rows_kernel<false><<<blocks, wpb * 32, 0, ctx->stream>>>(d_src, n, pd, Kp, dst, norm2, is_l2 ? 1 : 0, mul, st);
  ctx->stats.launches++;
  FV_CUDA(cudaGetLastError());
  return FV_OK;
}

static int split_norms(fv_ctx* ctx, bool bf16, const float* norm2, size_t first, size_t count, int e, uint16_t* ext) {
  if (count == 0) return FV_OK;
  const float inv = std::ldexp(1.f, -e);
  const unsigned blocks = unsigned((count + 255) / 256);
  if (bf16) split_norms_kernel<true><<<blocks, 256, 0, ctx->stream>>>(norm2, first, count, inv, ext);
  else split_norms_kernel<false><<<blocks, 256, 0, ctx->stream>>>(norm2, first, count, inv, ext);
  ctx->stats.launches++;
  FV_CUDA(cudaGetLastError());
  return FV_OK;
}

// Called by FlatIndex::add after the fp32 rows are in place.  d_rows_new points at the new rows.
int tc_append(fv_ctx* ctx, TcSide** ptc, int metric, const float* d_rows_new, size_t n_old, size_t n_new, int pd) {
  const int Kp = round_up(pd, KBLK);
  if (Kp > 384) return FV_OK;  // beyond the tilings of this kernel: such an index uses the scan only
  if (!*ptc) {
    *ptc = new TcSide();
    (*ptc)->pd = pd;
    (*ptc)->Kp = Kp;
  }
  TcSide* tc = *ptc;
  const size_t total = n_old + n_new;
  if (!tc->stats.p) {
    FV_TRY(tc->stats.reserve(256));
    init_stats_kernel<<<1, 1, 0, ctx->stream>>>(tc->stats.as<RangeStats>());
    FV_CUDA(cudaGetLastError());
  }
  FV_TRY(tc->half.grow(total * size_t(Kp) * 2 + 1024, n_old * size_t(Kp) * 2, ctx->stream));
  const size_t npad = (total + TILE_N - 1) / TILE_N * TILE_N + TILE_N;
  FV_TRY(tc->norm2.grow(npad * sizeof(float), n_old * sizeof(float), ctx->stream));
  // pick the operand type from the range of the NEW rows first (fp16 unless the values do not fit)
  DevBuf tmp_stats;
  FV_TRY(tmp_stats.reserve(sizeof(RangeStats)));
  init_stats_kernel<<<1, 1, 0, ctx->stream>>>(tmp_stats.as<RangeStats>());
  FV_CUDA(cudaGetLastError());
  uint16_t* dst = tc->half.as<uint16_t>() + n_old * size_t(Kp);
  float* nrm = tc->norm2.as<float>() + n_old;
  FV_TRY(convert(ctx, tc->bf16, d_rows_new, n_new, pd, Kp, dst, nrm, metric == FV_L2, 1.f, tmp_stats.as<RangeStats>()));
  RangeStats hs;
  FV_CUDA(cudaMemcpyAsync(&hs, tmp_stats.p, sizeof(hs), cudaMemcpyDeviceToHost, ctx->stream));
  FV_CUDA(cudaStreamSynchronize(ctx->stream));
  const float mabs = std::max(std::fabs(hs.min_v), std::fabs(hs.max_v));
  // fp16 also needs the largest squared norm within reach of the norm step: 2^15 (query side) x 2^15 (pieces)
  const float max_n2 = std::max(hs.max_norm2, tc->n ? tc->h_stats.max_norm2 : 0.f);
  const bool need_bf16 = !(mabs <= 32768.f) || !(max_n2 <= 1073741824.f);
  bool resplit = false;
  if (need_bf16 && !tc->bf16) {
    resplit = true;
    // values beyond the fp16 range: the whole operand copy becomes bf16.  The caller passes the new rows
    // only, so the old ones are re-read from the fp32 matrix that precedes them in the same allocation.
    tc->bf16 = true;
    const float* all_rows = d_rows_new - n_old * size_t(pd);
    init_stats_kernel<<<1, 1, 0, ctx->stream>>>(tc->stats.as<RangeStats>());
    FV_TRY(convert(ctx, true, all_rows, total, pd, Kp, tc->half.as<uint16_t>(), tc->norm2.as<float>(), metric == FV_L2,
                   1.f, tc->stats.as<RangeStats>()));
    FV_CUDA(cudaMemcpyAsync(&tc->h_stats, tc->stats.p, sizeof(RangeStats), cudaMemcpyDeviceToHost, ctx->stream));
    FV_CUDA(cudaStreamSynchronize(ctx->stream));
  } else {
    // fold the new rows' statistics into the running ones
    FV_CUDA(cudaMemcpyAsync(&tc->h_stats, tc->stats.p, sizeof(RangeStats), cudaMemcpyDeviceToHost, ctx->stream));
    FV_CUDA(cudaStreamSynchronize(ctx->stream));
    RangeStats m = tc->h_stats;
    m.min_v = std::min(m.min_v, hs.min_v);
    m.max_v = std::max(m.max_v, hs.max_v);
    m.max_norm2 = std::max(m.max_norm2, hs.max_norm2);
    m.not_integer |= hs.not_integer;
    m.not_finite |= hs.not_finite;
    FV_CUDA(cudaMemcpyAsync(tc->stats.p, &m, sizeof(m), cudaMemcpyHostToDevice, ctx->stream));
    FV_CUDA(cudaStreamSynchronize(ctx->stream));
    tc->h_stats = m;
  }
  fill_f32_kernel<<<8, 256, 0, ctx->stream>>>(tc->norm2.as<float>() + total, npad - total, INFINITY);
  ctx->stats.launches++;
  FV_CUDA(cudaGetLastError());
  tc->n = total;
  if (metric == FV_L2) {
    // norm pieces: ||b||^2 / 2^e with the largest quotient in (128, 256] when e was chosen, re-split when it outgrows 2^15
    FV_TRY(tc->ext.grow(npad * size_t(EXT_K) * 2, n_old * size_t(EXT_K) * 2, ctx->stream));
    int e = tc->ext_e;
    const float mx = tc->h_stats.max_norm2;
    if (tc->bf16) {
      e = 0;
      if (!tc->ext_valid || tc->ext_e != 0) resplit = true;
    } else if (!tc->ext_valid || !(std::ldexp(mx, -e) <= 32768.f)) {
      int ex = 0;
      if (mx > 0.f && mx < INFINITY) std::frexp(mx, &ex);  // mx in [2^(ex-1), 2^ex)
      e = std::min(15, std::max(-14, ex - 8));
      resplit = true;
    }
    tc->ext_e = e;
    tc->ext_valid = true;
    const size_t first = resplit ? 0 : n_old;
    FV_TRY(split_norms(ctx, tc->bf16, tc->norm2.as<float>(), first, npad - first, e, tc->ext.as<uint16_t>()));
  }
  // the strided sample the threshold of the main pass is estimated from
  tc->every = pick_sample_every(total);
  tc->ns = std::max<size_t>(SAMPLE_R_MAX, total / size_t(tc->every));
  const size_t nspad = (tc->ns + TILE_N - 1) / TILE_N * TILE_N + TILE_N;
  FV_TRY(tc->samp.reserve(tc->ns * size_t(Kp) * 2 + 1024));
  FV_TRY(tc->samp_norm2.reserve(nspad * sizeof(float)));
  gather_sample_kernel<<<unsigned((tc->ns + 7) / 8), 256, 0, ctx->stream>>>(
      tc->half.as<uint16_t>(), tc->norm2.as<float>(), total, Kp, tc->ns, tc->samp.as<uint16_t>(),
      tc->samp_norm2.as<float>());
  fill_f32_kernel<<<8, 256, 0, ctx->stream>>>(tc->samp_norm2.as<float>() + tc->ns, nspad - tc->ns, INFINITY);
  ctx->stats.launches += 2;
  FV_CUDA(cudaGetLastError());
  if (metric == FV_L2) {
    FV_TRY(tc->samp_ext.reserve(nspad * size_t(EXT_K) * 2));
    FV_TRY(split_norms(ctx, tc->bf16, tc->samp_norm2.as<float>(), 0, nspad, tc->ext_e, tc->samp_ext.as<uint16_t>()));
  }
  return FV_OK;
}

bool tc_usable(const TcSide* tc, size_t n, size_t nq, int k) {
  (void)nq;
  return tc && tc->n == n && k <= 32 && n >= 4096 && n <= 0x7FFFFF00ull;
}

// One launch of the GEMM kernel over `rows` operand rows.
//
// Work split.  A unit is (query tile, 256 base rows).  Each query tile's row of units is cut into `parts` chunks of
// `cpn` units; chunk g = part * MT + query tile goes to CTA g % grid as that CTA's (g / grid)-th segment.  The CTAs
// that run side by side therefore hold DIFFERENT query tiles but walk the SAME base tiles at about the same time:
// a base tile is fetched from HBM once and served to the other query tiles from L2 (with a contiguous split of the
// units the 16-bit copy of the base was streamed from HBM once per query tile).  `parts` is the value that minimises
// waves x (chunk length + a fixed cost per chunk).
struct Tiling {
  int KB, MH, MT, NT, grid, segmax, nstage, cpn, parts, nchunks, ext_ring;
  size_t smem;
};

static int make_tiling(fv_ctx* ctx, int Kp, size_t nq, size_t rows, int scratch_bytes, Tiling* t, int force_mh = 0) {
  t->KB = Kp / KBLK;
  t->MH = force_mh ? force_mh : (t->KB <= 2 ? 2 : 1);
  const int rows_per_tile = 128 * t->MH;
  t->MT = int((nq + rows_per_tile - 1) / rows_per_tile);
  t->NT = int((rows + TILE_N - 1) / TILE_N);
  t->grid = int(std::min<long long>(ctx->sm_count, (long long)t->MT * t->NT));
  long long best = -1;
  for (int P = 1; P <= t->NT && P <= 4096; ++P) {
    const int cpn = (t->NT + P - 1) / P;
    const int parts = (t->NT + cpn - 1) / cpn;
    const long long chunks = (long long)t->MT * parts;
    const long long waves = (chunks + t->grid - 1) / t->grid;
    const long long cost = waves * (cpn + 3);
    if (best < 0 || cost < best) {
      best = cost;
      t->cpn = cpn;
      t->parts = parts;
    }
  }
  const long long chunks = (long long)t->MT * t->parts;
  if (chunks > 0x7FFFFFFF) return fail(FV_ERR_UNSUPPORTED, "too many work chunks for the tensor-core tiling");
  t->nchunks = int(chunks);
  t->segmax = int((chunks + t->grid - 1) / t->grid);
  const size_t a_bytes = size_t(t->MH) * t->KB * A_BLOCK_BYTES + A_EXT_BYTES;
  const size_t tail = size_t(scratch_bytes) + sizeof(Barriers) + 64;
  for (t->nstage = 6; t->nstage >= 2; --t->nstage) {
    t->ext_ring = (t->nstage + t->KB - 1) / t->KB + 1;
    t->smem = 1024 + a_bytes + size_t(t->nstage) * B_STAGE_BYTES + size_t(t->ext_ring) * B_EXT_BYTES + tail;
    if (t->smem <= ctx->smem_optin) return FV_OK;
  }
  return fail(FV_ERR_UNSUPPORTED, "not enough shared memory for the tensor-core tiling");
}

template <int KPT, bool THRESH>
static int launch_gemm(fv_ctx* ctx, const Tiling& t, const CUtensorMap& tmA, const CUtensorMap& tmB,
                       const GemmParams& gp) {
  void (*kern)(const CUtensorMap, const CUtensorMap, GemmParams) =
      t.MH == 2 ? gemm_topk_kernel<2, KPT, THRESH> : gemm_topk_kernel<1, KPT, THRESH>;
  FV_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(t.smem)));
  kern<<<t.grid, NTHREADS, t.smem, ctx->stream>>>(tmA, tmB, gp);
  ctx->stats.launches++;
  FV_CUDA(cudaGetLastError());
  return FV_OK;
}

// Test hook (fv_debug_tc_fault): the next launch of the kernel, once, runs with this wait limit and with one unit's
// loads left out, so that the give-up path of the bounded waits can be exercised without any fault on the device.
static std::atomic<long long> g_test_wait_limit{0};
static std::atomic<int> g_test_skip_unit{-1};

static void fill_params(GemmParams* g, const Tiling& t, size_t rows, size_t nq, int scratch_bytes) {
  g->wait_limit = WAIT_LIMIT_CYCLES;
  g->fault_skip_unit = -1;
  const long long test_limit = g_test_wait_limit.exchange(0);
  if (test_limit > 0) {
    g->wait_limit = test_limit;
    g->fault_skip_unit = g_test_skip_unit.exchange(-1);
  }
  g->n = int(rows);
  g->nq = int(nq);
  g->KB = t.KB;
  g->NT = t.NT;
  g->MT = t.MT;
  g->cpn = t.cpn;
  g->nchunks = t.nchunks;
  g->segmax = t.segmax;
  g->nstage = t.nstage;
  g->scratch_bytes = scratch_bytes;
  g->ext_ring = t.ext_ring;
}

// ------------------------------------------------------------------------------------------------
// Task mode for other callers (the IVF-PQ scan): operand rows they prepared, scored against runs of this side's rows.
void tc_info(const TcSide* tc, TcInfo* out) {
  out->Kp = tc->Kp;
  out->bf16 = tc->bf16;
  out->n = tc->n;
  out->max_norm2 = tc->h_stats.max_norm2;
  out->min_v = tc->h_stats.min_v;
  out->max_v = tc->h_stats.max_v;
  out->not_finite = tc->h_stats.not_finite != 0;
}

int* tc_error_word(TcSide* tc) {
  RangeStats* qst = tc->stats.as<RangeStats>() + 1;
  return reinterpret_cast<int*>(reinterpret_cast<unsigned int*>(qst + 1) + 1);
}

int tc_list_pass(fv_ctx* ctx, TcSide* tc, int metric, const uint16_t* d_A, size_t a_rows, const float* d_thr,
                 const uint4* d_tasks, const uint32_t* d_ntasks, unsigned int* d_next_task, u64* d_pool, unsigned int* d_pool_cnt,
                 unsigned int pool_cap, const uint32_t* d_row_owner, uint32_t* d_dropped, int* grid_out, int tile_rows,
                 float* d_minima, const uint32_t* d_task_moff, const uint32_t* d_task_rows) {
  const int Kp = tc->Kp;
  if (Kp > 2 * KBLK) return fail(FV_ERR_UNSUPPORTED, "task mode of the tensor-core kernel covers padded dimensions up to 128");
  if (tile_rows != 128 && tile_rows != 256) return fail(FV_ERR_ARG, "operand tiles have 128 or 256 rows");
  Tiling t{};
  // stages and shared memory for operand tiles of that height; the tiling itself is unused
  FV_TRY(make_tiling(ctx, Kp, 256, size_t(TILE_N) * 1024, 0, &t, tile_rows == 128 ? 1 : 2));
  GemmParams gp{};
  fill_params(&gp, t, tc->n, a_rows, 0);
  gp.nchunks = 0;
  gp.has_ext = metric == FV_L2 ? 1 : 0;
  gp.aext_c = tc->bf16 ? 0x3F80u : uint32_t((tc->ext_e + 15) << 10);
  gp.idesc = make_idesc(128, TILE_N, tc->bf16);
  gp.err = tc_error_word(tc);
  gp.ext = tc->ext.as<uint16_t>();
  gp.tau = d_thr;
  gp.tasks = d_tasks;
  gp.ntasks = d_ntasks;
  gp.next_task = d_next_task;
  gp.pool = d_pool;
  gp.pool_cnt = d_pool_cnt;
  gp.pool_cap = pool_cap;
  gp.row_owner = d_row_owner;
  gp.owner_dropped = d_dropped;
  gp.minima = d_minima;
  gp.task_moff = d_task_moff;
  gp.task_rows = d_task_rows;
  CUtensorMap tmA, tmB;
  FV_TRY(make_tmap(&tmA, tc->bf16, const_cast<uint16_t*>(d_A), a_rows, Kp, 128));
  FV_TRY(make_tmap(&tmB, tc->bf16, tc->half.p, tc->n, Kp, TILE_N));
  FV_CUDA(cudaMemsetAsync(d_next_task, 0, sizeof(unsigned int), ctx->stream));
  void (*kern)(const CUtensorMap, const CUtensorMap, GemmParams) =
      tile_rows == 128 ? gemm_topk_kernel<1, 2, true, true> : gemm_topk_kernel<2, 2, true, true>;
  FV_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(t.smem)));
  kern<<<ctx->sm_count, NTHREADS, t.smem, ctx->stream>>>(tmA, tmB, gp);
  ctx->stats.launches++;
  FV_CUDA(cudaGetLastError());
  *grid_out = ctx->sm_count;
  return FV_OK;
}

// Stages (fv_stats.stage_ms): 0 query conversion, 1 sample pass, 2 main pass, 3 re-rank + certificate, 4 fallback.
// scratch slots: 2 scan partials (fallback), 3 A operand, 5 query norms + bounds + candidate counters, 6 sample lists,
// 7 retry ids, 8 fallback keys, 9 candidate buffers
int tc_search(fv_ctx* ctx, TcSide* tc, int metric, const float* d_rows, size_t n, int pd, const float* d_queries,
              size_t nq, int k, uint32_t id_base, u64* d_out_keys, bool mark_stages, bool prefilter_inf) {
  const int Kp = tc->Kp;
  const bool is_l2 = metric == FV_L2;
  Tiling ts{}, tm{};
  FV_TRY(make_tiling(ctx, Kp, nq, tc->ns, SCRATCH_BYTES, &ts));
  FV_TRY(make_tiling(ctx, Kp, nq, n, 0, &tm));
  const int rows_per_tile = 128 * tm.MH;

  // queries -> 16-bit operand rows scaled by -2 (L2) or -1 (inner product), padded to whole tiles with zeros;
  // norms; statistics
  const size_t nq_pad = size_t(tm.MT) * rows_per_tile;
  FV_TRY(ctx->scratch[3].reserve(nq_pad * size_t(Kp) * 2));
  const size_t nlists = size_t(tm.grid) * tm.segmax * LISTS;
  // Candidate slots per epilogue thread and segment: 256 unless the buffers would pass 2 GB (they are written
  // sparsely: about 160 entries per query in all).  A base stored cluster by cluster puts most of a query's
  // candidates into one or two chunks, so the slots must hold more than the average.
  int ccap = 256;
  while (ccap > 16 && nlists * size_t(ccap) * sizeof(u64) > (size_t(2) << 30)) ccap >>= 1;
  FV_TRY(ctx->scratch[5].reserve(2 * nq_pad * sizeof(float) + nlists * sizeof(unsigned int)));
  FV_TRY(ctx->scratch[6].reserve(size_t(ts.grid) * ts.segmax * LISTS * KP * sizeof(u64)));
  FV_TRY(ctx->scratch[7].reserve(nq * sizeof(uint32_t)));
  FV_TRY(ctx->scratch[9].reserve(nlists * size_t(ccap) * sizeof(u64)));
  uint16_t* dA = ctx->scratch[3].as<uint16_t>();
  float* qn2 = ctx->scratch[5].as<float>();
  float* tau = qn2 + nq_pad;
  unsigned int* ccnt = reinterpret_cast<unsigned int*>(tau + nq_pad);
  RangeStats* bst = tc->stats.as<RangeStats>();
  RangeStats* qst = bst + 1;
  unsigned int* retry_count = reinterpret_cast<unsigned int*>(qst + 1);
  int* err = reinterpret_cast<int*>(retry_count + 1);
  CUtensorMap tmA, tmS, tmB;
  FV_TRY(make_tmap(&tmA, tc->bf16, dA, nq_pad, Kp, 128));
  FV_TRY(make_tmap(&tmS, tc->bf16, tc->samp.p, tc->ns, Kp, TILE_N));
  FV_TRY(make_tmap(&tmB, tc->bf16, tc->half.p, n, Kp, TILE_N));

  init_stats_kernel<<<1, 1, 0, ctx->stream>>>(qst);
  FV_CUDA(cudaMemsetAsync(retry_count, 0, 8, ctx->stream));
  if (nq_pad > nq) FV_CUDA(cudaMemsetAsync(dA + nq * size_t(Kp), 0, (nq_pad - nq) * size_t(Kp) * 2, ctx->stream));
  FV_TRY(convert(ctx, tc->bf16, d_queries, nq, pd, Kp, dA, qn2, is_l2, is_l2 ? -2.f : -1.f, qst));
  if (mark_stages) stage_mark(ctx);

  // sample pass: per query the R (+1) best scores over the sampled rows
  // the epilogue keeps its lists in registers, so their length is a template parameter: R is rounded up to the next
  // instantiated length - 1 (a larger R only loosens the bound)
  int R = pick_sample_r(k, tc->every);
  R = R <= 7 ? R : (R <= 9 ? 9 : 13);
  GemmParams gs{};
  fill_params(&gs, ts, tc->ns, nq, SCRATCH_BYTES);
  gs.has_ext = is_l2 ? 1 : 0;
  gs.aext_c = tc->bf16 ? 0x3F80u : uint32_t((tc->ext_e + 15) << 10);  // 1.0 (bf16) or 2^ext_e (fp16)
  gs.idesc = make_idesc(128, TILE_N, tc->bf16);
  gs.cand = ctx->scratch[6].as<u64>();
  gs.err = err;
  gs.ext = tc->samp_ext.as<uint16_t>();
  if (R == 5) FV_TRY((launch_gemm<6, false>(ctx, ts, tmA, tmS, gs)));
  else if (R == 6) FV_TRY((launch_gemm<7, false>(ctx, ts, tmA, tmS, gs)));
  else if (R == 7) FV_TRY((launch_gemm<8, false>(ctx, ts, tmA, tmS, gs)));
  else if (R == 9) FV_TRY((launch_gemm<10, false>(ctx, ts, tmA, tmS, gs)));
  else FV_TRY((launch_gemm<14, false>(ctx, ts, tmA, tmS, gs)));
  sample_tau_kernel<<<unsigned((nq_pad + 255) / 256), 256, 0, ctx->stream>>>(gs.cand, ts.MT, ts.parts, ts.grid, ts.segmax,
                                                                             ts.MH, int(nq_pad), R, tau);
  ctx->stats.launches++;
  FV_CUDA(cudaGetLastError());
  if (mark_stages) stage_mark(ctx);

  // main pass: every row scoring below the query's sampled bound becomes a candidate
  GemmParams gp = gs;
  fill_params(&gp, tm, n, nq, 0);
  gp.cand = nullptr;
  gp.tau = tau;
  gp.cbuf = ctx->scratch[9].as<u64>();
  gp.ccnt = ccnt;
  gp.ccap = ccap;
  gp.ext = tc->ext.as<uint16_t>();
  FV_TRY((launch_gemm<2, true>(ctx, tm, tmA, tmB, gp)));
  if (mark_stages) stage_mark(ctx);

  RerankParams rp{};
  rp.tau = tau;
  rp.cbuf = gp.cbuf;
  rp.ccnt = gp.ccnt;
  rp.ccap = gp.ccap;
  rp.MT = tm.MT;
  rp.parts = tm.parts;
  rp.grid = tm.grid;
  rp.segmax = tm.segmax;
  rp.rows = d_rows;
  rp.queries = d_queries;
  rp.qnorm2 = qn2;
  rp.bst = bst;
  rp.qst = qst;
  rp.n = int(n);
  rp.nq = int(nq);
  rp.pd = pd;
  rp.Kp = Kp;
  rp.k = k;
  rp.MH = tm.MH;
  rp.is_l2 = metric == FV_L2 ? 1 : 0;
  rp.bf16 = tc->bf16 ? 1 : 0;
  rp.id_base = id_base;
  rp.out_keys = d_out_keys;
  rp.retry_ids = ctx->scratch[7].as<uint32_t>();
  rp.retry_count = retry_count;
  int wpb = 8;
  const size_t rwarp = size_t(pd) * 4 + size_t(k) * 8 + size_t(8 * quad_stride(pd)) * 4;  // query, list, two stages of four rows
  while (wpb > 1 && size_t(wpb) * rwarp + 16 > 72 * 1024) wpb >>= 1;
  const size_t rsmem = ((size_t(wpb) * (size_t(pd) * 4 + size_t(k) * 8) + 15) & ~size_t(15)) + size_t(wpb) * 8 * quad_stride(pd) * 4;
  if (rsmem > 48 * 1024) FV_CUDA(cudaFuncSetAttribute(rerank_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(rsmem)));
  rerank_kernel<<<unsigned((nq + wpb - 1) / wpb), wpb * 32, rsmem, ctx->stream>>>(rp);
  ctx->stats.launches++;
  FV_CUDA(cudaGetLastError());
  if (mark_stages) stage_mark(ctx);

  unsigned int h_words[2] = {0, 0};  // retry count, error word
  FV_CUDA(cudaMemcpyAsync(h_words, retry_count, sizeof(h_words), cudaMemcpyDeviceToHost, ctx->stream));
  FV_CUDA(cudaStreamSynchronize(ctx->stream));
  if (h_words[1]) return fail(FV_ERR_TIMEOUT, "a bounded wait inside the tensor-core kernel ran out");
  ctx->stats.uncertified = h_words[0];
  if (h_words[0]) {
    const size_t nsub = h_words[0];
    FV_TRY(ctx->scratch[8].reserve(nsub * size_t(k) * sizeof(u64)));
    u64* sub = ctx->scratch[8].as<u64>();
    FV_TRY(exact_scan(ctx, metric, d_rows, n, pd, d_queries, size_t(pd), rp.retry_ids, nsub, k, prefilter_inf, id_base, sub, 2));
    scatter_keys_kernel<<<ctx->sm_count, 256, 0, ctx->stream>>>(sub, rp.retry_ids, nsub, k, d_out_keys);
    ctx->stats.launches++;
    FV_CUDA(cudaGetLastError());
  }
  if (mark_stages) stage_mark(ctx);
  return FV_OK;
}

}  // namespace fv

// Test hook: arms the next launch of the tensor-core kernel (once) with a short wait limit, in cycles, and makes the
// producer of work item 0 leave out the loads of unit `skip_unit` of it: the consumer of that stage waits until
// the limit, the kernel sets its error word, frees its tensor memory and returns, and the search that launched it
// fails with FV_ERR_TIMEOUT.  Nothing on the device faults or spins without bound.  (0, -1) disarms.
extern "C" int fv_debug_tc_fault(long long wait_limit_cycles, int skip_unit) {
  if (wait_limit_cycles < 0 || skip_unit < -1) return fv::fail(FV_ERR_ARG, "fv_debug_tc_fault: bad argument");
  fv::g_test_skip_unit.store(skip_unit);
  fv::g_test_wait_limit.store(wait_limit_cycles);
  return FV_OK;
}
