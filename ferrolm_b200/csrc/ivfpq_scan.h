// The search side of IvfPq (ivfpq.rs:225-297) as seen by the index code: what the scan needs to know about an
// index, and the one host routine that runs tables + scan + top-k (+ re-rank) for a query batch.
#pragma once

#include "internal.h"

namespace fv {

// Device view of an index for the duration of one search.
struct ScanIndex {
  const float* centroids;     // nlist x pd
  const float* codebooks;     // m x 256 x dsub
  const float* pre;           // nlist x m x 256 precomputed L2 tables (ivfpq.rs:108-126), or null
  const uint32_t* list_off;   // nlist + 1 row offsets of the lists
  const uint8_t* codes;       // rows x m, grouped by list
  const uint32_t* ids;        // rows, grouped by list
  const float* vectors;       // kept raw vectors in id order, or null
  const uint32_t* owned_ids;  // list-sharded index: ascending ids of the kept vectors (row s of `vectors`); else null
  uint32_t owned_n;
  int shard_rank, shard_world;  // this shard scans the probed lists l with l % world == rank
  int metric, pd, m, dsub;
  size_t nlist;
  uint32_t id_base;
  // m = 16 only: the codes once more, sub-quantizer-major inside every list.  List l starts at byte 16 * off16[l];
  // with len16 = off16[l+1] - off16[l] (the list length rounded up to 16) byte (j, r) sits at j * len16 + r.
  const uint8_t* codes_t;     // or null
  const uint32_t* off16;      // nlist + 1
  // Tensor-core pass: every stored row once more as the vector its code stands for (centroid + codewords), 16-bit,
  // list by list with every list starting at a multiple of 8 rows (roff8[l]); null when not built.
  TcSide* recon;
  const uint32_t* roff8;      // nlist + 1 row offsets, then the nlist list numbers in order of decreasing length
  float cen_norm2_max;        // largest squared centroid norm
  float code_norm2_max;       // sum over sub-quantizers of their largest squared codeword norm
  uint32_t max_list_rows;     // length of the longest list
  uint32_t nrows;             // rows in all lists of this index (list_off[nlist])
  size_t survivor_slots;      // survivor pool entries per CTA of the tensor-core pass (0 = sized from the batch)
};

struct ScanOut {
  u64* keys;             // nq x k final keys                  (candidates == false)
  fv_neighbor* adc;      // nq x keep kept candidates          (candidates == true)
  float* exact;          // nq x keep their exact distances
  uint32_t* counts;      // nq                                 (candidates == true)
};

// mode: 0 = pick by size, 1 = one block per query only, 2 = the list-major table scan whenever the index allows it,
// 3 = the list-major tensor-core pass whenever the index allows it, 4 = the same with the bounds from the per-query
// kernel (the form it takes by itself when the lists are long and many).
// `cells`: nq x nprobe keys (distance, list), ascending.  `keep` = candidates kept by compressed distance;
// `refine`: re-rank them exactly and cut to k.  Marks the context's stages and fills stats.rows_scanned.
// `cand_slots`: candidate slots per query of the list-major scans (0 = default).
// Scratch slots used: 5, 6, 7, 8, 9, 12, 13, 14, 15.
int ivfpq_scan(fv_ctx* ctx, const ScanIndex& ix, const float* d_queries, size_t nq, const u64* d_cells, int nprobe,
               int keep, int k, bool refine, bool candidates, int mode, int cand_slots, const ScanOut& out);

// Whether a search of this size would take the tensor-core pass if the index has what it needs (so that the index
// builds the reconstruction only when it will be used).
bool ivfpq_wants_tensor(int mode, size_t nq, size_t nprobe, size_t nlist, int shard_world);

// Builds the 16-bit reconstruction of every stored row for the tensor-core pass (padded dimension up to 128).
int build_reconstruction(fv_ctx* ctx, int metric, int pd, int m, int dsub, const uint32_t* h_off, size_t nlist,
                         const uint32_t* d_list_off, const uint8_t* d_codes, const float* d_centroids,
                         const float* d_codebooks, TcSide** recon, DevBuf* roff8);

// Builds codes_t / off16 from the row-major lists (m = 16).  h_off: nlist + 1 host offsets.
int build_transposed_codes(fv_ctx* ctx, const uint32_t* h_off, size_t nlist, const uint32_t* d_list_off,
                           const uint8_t* d_codes, DevBuf* codes_t, DevBuf* off16);

}  // namespace fv
