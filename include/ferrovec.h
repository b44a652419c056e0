/* ferrovec.h -- C ABI of the B200 (sm_100a) nearest-neighbour search library.
 *
 * The reference (ferrolm, Rust) has no FFI for this path: src/vector is an
 * in-crate module called directly by src/rag.rs and src/main.rs.  Each entry
 * point below therefore names the Rust method it stands in for, so a Rust
 * `extern "C"` block can bind them one to one and keep the reference's
 * FlatIndex / IvfPq / Hnsw method signatures on top.
 *
 * Conventions
 *   - every function returns an fv_status (0 = ok) unless it returns a size;
 *     fv_last_error() gives the message of the calling thread's last failure;
 *   - vectors are row-major f32 with the caller's unpadded `dim`; the library
 *     pads rows to a multiple of 8 internally (src/vector/mod.rs:113-129);
 *   - results are caller-allocated: `out` holds nq*k fv_neighbor, row i filled
 *     with counts[i] <= k entries in ascending (distance, id) order
 *     (src/vector/mod.rs:60-64) and padded with {0xFFFFFFFF, +inf};
 *   - inner-product distances are NEGATED dots, as in the reference
 *     (src/vector/mod.rs:28-33);
 *   - plain entry points take HOST pointers and copy; the `_dev` twins take
 *     DEVICE pointers of the context's GPU and run on the context's stream
 *     (results are complete when the call returns);
 *   - there is no CPU code path: without a usable GPU every call fails.
 */
#ifndef FERROVEC_H
#define FERROVEC_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* src/vector/mod.rs:52-56 */
typedef struct fv_neighbor {
  uint32_t id;
  float distance;
} fv_neighbor;

/* src/vector/mod.rs:20-49 (Metric::code) */
enum { FV_L2 = 0, FV_INNER_PRODUCT = 1 };

typedef enum fv_status {
  FV_OK = 0,
  FV_ERR_ARG = 1,         /* precondition the reference asserts on (e.g. ivfpq.rs:58, kmeans.rs:41) */
  FV_ERR_FILE = 2,        /* load(): Err(String) in the reference (hnsw.rs:425-452, ivfpq.rs:355-357) */
  FV_ERR_CUDA = 3,        /* a CUDA runtime call failed, or no sm_100 device */
  FV_ERR_TIMEOUT = 4,     /* a bounded device-side wait ran out */
  FV_ERR_OVERFLOW = 5,    /* a device-side work list ran out of room even after regrowing */
  FV_ERR_UNSUPPORTED = 6, /* size beyond a documented limit of this library */
  FV_ERR_NOMEM = 7,
  FV_ERR_COMM = 8         /* NCCL is missing or a collective failed */
} fv_status;

const char* fv_last_error(void);
/* Library version string; also a cheap "is the .so loadable" probe. */
const char* fv_version(void);

/* ---- context: stands in for the `&Pool` argument of every batch call (src/pool.rs:42-106).
 * Holds one device, one stream and the scratch arena that searches reuse. */
typedef struct fv_ctx fv_ctx;
int fv_ctx_create(int device, fv_ctx** out);
void fv_ctx_destroy(fv_ctx* ctx);
int fv_ctx_device(const fv_ctx* ctx);
/* Blocks until everything queued on the context's stream has finished. */
int fv_ctx_sync(fv_ctx* ctx);
/* The context's cudaStream_t, for callers that order their own work against it. */
void* fv_ctx_stream(fv_ctx* ctx);
/* Counters of the last search call on this context (kernel launches, slow-path queries). */
typedef struct fv_stats {
  uint64_t launches;        /* kernels launched by the last call */
  uint64_t uncertified;     /* exact search: queries re-run on the full-precision scan; IVF-PQ: queries whose candidate buffer ran over in the list-major scan and were re-run by the per-query kernel; HNSW: queries whose list of tied, pushed-out entries overflowed (64; ties beyond that may be resolved differently from the reference) */
  uint64_t rows_scanned;    /* IVF-PQ: code rows visited (sum over queries and probes) */
  uint64_t dist_evals;      /* HNSW: distance evaluations; IVF-PQ tensor-core pass: (query, row) pairs that survived the tensor-core scores and were re-scored with the exact table arithmetic */
  uint64_t expansions;      /* HNSW: node expansions */
  uint64_t regrown;         /* HNSW: queries re-run with a larger visited table; IVF-PQ list-major scans: queries whose candidate buffer ran over and that got a second round with a tightened bound */
  float stage_ms[8];        /* per-stage device time of the last call when timing is on */
  uint64_t rows_list_scan;  /* IVF-PQ: the part of rows_scanned that the list-major kernel visited (0: per-query kernel only) */
} fv_stats;
int fv_ctx_stats(const fv_ctx* ctx, fv_stats* out);
/* 1 = record per-stage device times (CUDA events) for fv_ctx_stats; 0 = off (default). */
int fv_ctx_set_timing(fv_ctx* ctx, int on);

/* ---- FlatIndex (src/vector/flat.rs:7-66) */
typedef struct fv_flat fv_flat;
int fv_flat_new(fv_ctx* ctx, int metric, uint32_t dim, fv_flat** out);                /* FlatIndex::new  :15 */
void fv_flat_free(fv_flat* ix);
int fv_flat_add(fv_flat* ix, const float* vectors, size_t n);                         /* add             :24 */
int fv_flat_add_dev(fv_flat* ix, const float* d_vectors, size_t n);
size_t fv_flat_len(const fv_flat* ix);                                                /* len             :28 */
int fv_flat_vector(const fv_flat* ix, uint32_t id, float* out_padded);                /* vector          :36 */
int fv_flat_search(fv_flat* ix, const float* query, size_t k, fv_neighbor* out, uint32_t* count); /* search :40 */
int fv_flat_search_batch(fv_flat* ix, const float* queries, size_t nq, size_t k,      /* search_batch    :56 */
                         fv_neighbor* out, uint32_t* counts);
int fv_flat_search_batch_dev(fv_flat* ix, const float* d_queries, size_t nq, size_t k,
                             fv_neighbor* d_out, uint32_t* d_counts);
/* Row-sharded use: ids reported by this index are local row + id_base. */
int fv_flat_set_id_base(fv_flat* ix, uint32_t id_base);
/* Search strategy: 0 = automatic, 1 = tensor-core front end + exact re-rank, 2 = full-precision scan only.
 * Both return the same neighbours; 2 exists for validation and as the fallback of 1. */
int fv_flat_set_mode(fv_flat* ix, int mode);

/* ---- k-means (src/vector/kmeans.rs:10-90), the build side of IVF-PQ */
int fv_kmeans_assign(fv_ctx* ctx, const float* data, size_t n, const float* centroids, size_t k, size_t dim,
                     uint32_t* out);                                                  /* assign :22 */
int fv_kmeans_train(fv_ctx* ctx, const float* data, size_t n, size_t dim, size_t k, size_t iters, uint64_t seed,
                    float* centroids_out);                                            /* train  :39 */

/* ---- IvfPq (src/vector/ivfpq.rs) */
typedef struct fv_ivfpq fv_ivfpq;
typedef struct fv_ivfpq_params { /* IvfPqParams, ivfpq.rs:18-27 */
  size_t nlist;
  size_t m;
  size_t iters;
  int keep_vectors;
  uint64_t seed;
} fv_ivfpq_params;
int fv_ivfpq_train(fv_ctx* ctx, int metric, uint32_t dim, const float* sample, size_t n,
                   const fv_ivfpq_params* p, fv_ivfpq** out);                          /* train :56 */
void fv_ivfpq_free(fv_ivfpq* ix);
int fv_ivfpq_add(fv_ivfpq* ix, const float* vectors, size_t n);                       /* add   :161 */
int fv_ivfpq_add_dev(fv_ivfpq* ix, const float* d_vectors, size_t n);
size_t fv_ivfpq_len(const fv_ivfpq* ix);                                              /* len   :128 */
size_t fv_ivfpq_bytes_per_vector(const fv_ivfpq* ix);                                 /* bytes_per_vector :137 */
size_t fv_ivfpq_nlist(const fv_ivfpq* ix);                                            /* field nlist :33 */
uint32_t fv_ivfpq_dim(const fv_ivfpq* ix);                                            /* field dim   :31 */
int fv_ivfpq_metric(const fv_ivfpq* ix);                                              /* field metric :30 (fv_metric) */
int fv_ivfpq_search(fv_ivfpq* ix, const float* query, size_t k, size_t nprobe, size_t refine,
                    fv_neighbor* out, uint32_t* count);                               /* search :225 */
int fv_ivfpq_search_batch(fv_ivfpq* ix, const float* queries, size_t nq, size_t k, size_t nprobe, size_t refine,
                          fv_neighbor* out, uint32_t* counts);                        /* search_batch :313 */
int fv_ivfpq_search_batch_dev(fv_ivfpq* ix, const float* d_queries, size_t nq, size_t k, size_t nprobe,
                              size_t refine, fv_neighbor* d_out, uint32_t* d_counts);
/* Row-sharded use.  The shard keeps the rows it is given with ids id_base + running count.  With refine > 0 a
 * shard must not cut to k by itself: this call returns its best `keep` = k*refine candidates by compressed
 * distance (d_adc, ascending) together with their exact distances (d_exact), for fv_merge_refine_dev. */
int fv_ivfpq_set_id_base(fv_ivfpq* ix, uint32_t id_base);
/* Sharding by inverted list, for throughput: shard `rank` of `world` keeps (and scans) only the lists l with
 * l % world == rank.  Every shard is given the same trained quantizers and the SAME rows in the same order
 * (ids count every row passed to add); each keeps its own.  A search then does 1/world of the table builds and
 * code scans; the per-shard results merge exactly as for row shards.  Call before the first add. */
int fv_ivfpq_set_shard(fv_ivfpq* ix, int rank, int world);
int fv_ivfpq_search_candidates_dev(fv_ivfpq* ix, const float* d_queries, size_t nq, size_t keep, size_t nprobe,
                                   fv_neighbor* d_adc, float* d_exact, uint32_t* d_counts);
/* The coarse step on its own (the cell list of search, ivfpq.rs:211-220): for every query the min(nprobe, nlist)
 * nearest cells as keys (order-preserving bits of the f32 distance in the high word, cell number in the low word),
 * ascending, nq x min(nprobe, nlist) keys.  The `_cells` searches take such keys instead of computing them.  With
 * list shards every shard would otherwise repeat the same coarse step for the whole batch: each shard computes
 * the keys of a slice of the queries, the slices are all-gathered, every shard searches with the full set. */
int fv_ivfpq_coarse_dev(fv_ivfpq* ix, const float* d_queries, size_t nq, size_t nprobe, uint64_t* d_cells);
int fv_ivfpq_search_batch_cells_dev(fv_ivfpq* ix, const float* d_queries, size_t nq, size_t k, size_t nprobe,
                                    size_t refine, const uint64_t* d_cells, fv_neighbor* d_out, uint32_t* d_counts);
int fv_ivfpq_search_candidates_cells_dev(fv_ivfpq* ix, const float* d_queries, size_t nq, size_t keep, size_t nprobe,
                                         const uint64_t* d_cells, fv_neighbor* d_adc, float* d_exact,
                                         uint32_t* d_counts);
/* Which scan a search uses: 0 = chosen by batch and index size (default), 1 = one block per query, 2 = the
 * list-major table scan, 3 = the list-major tensor-core pass, 4 = that pass with its bounds from the per-query kernel
 * instead of the tensor cores (2, 3 and 4 whenever the index allows it: m = 16, L2 with precomputed tables or inner
 * product, for 3 and 4 also a padded dimension up to 128; they keep a 16-bit reconstruction of every row,
 * 2 * padded dimension bytes per row, built by the first search that uses it).  All give the same neighbours;
 * 1 to 4 exist for validation and measurement. */
int fv_ivfpq_set_scan_mode(fv_ivfpq* ix, int mode);
/* List-major scan: global-memory candidate slots per query (8 bytes each; 0 = default, 1024 or fewer for very large
 * batches; at most 4096).  A query that finds more rows below its bound than it has slots is re-run by the
 * per-query kernel (counted in fv_stats.uncertified), so a small value trades memory for re-runs, never results. */
int fv_ivfpq_set_candidate_slots(fv_ivfpq* ix, size_t slots);
/* Tensor-core pass: entries (8 bytes each) of the pool every CTA appends its survivors to (0 = default, sized from
 * the batch; at most 2^21).  Survivors that find the pool full are dropped and the queries they belong to re-run by
 * the per-query kernel (fv_stats.uncertified): again memory against re-runs, never results. */
int fv_ivfpq_set_survivor_slots(fv_ivfpq* ix, size_t slots);
/* 1 when the library was built with -DFV_BOUNDS (make EXTRA=-DFV_BOUNDS), the debug build in which the kernels check
 * every index they gather through (probed cells, row ids, vector slots, graph links) against its extent, skip an
 * access that would leave it and make the search return FV_ERR_OVERFLOW with the first offending site, index and
 * extent in fv_last_error; 0 for the normal build, which trusts its inputs (the *_cells_dev entry points in
 * particular take the probed cells from the caller unchecked). */
int fv_debug_bounds_build(void);
/* Test hook for the give-up path of the bounded waits in the tensor-core kernel: arms the NEXT launch of that kernel,
 * once, with a wait limit of wait_limit_cycles and makes one CTA's producer leave out the loads of unit skip_unit of
 * its first work item.  The consumer of that stage waits until the limit, the kernel sets its error word, frees its
 * tensor memory and returns, and the search that launched it fails with FV_ERR_TIMEOUT; the context stays usable.
 * Nothing on the device faults or spins without bound.  (0, -1) disarms.  Not for production callers. */
int fv_debug_tc_fault(long long wait_limit_cycles, int skip_unit);
size_t fv_ivfpq_save_size(const fv_ivfpq* ix);
int fv_ivfpq_save(const fv_ivfpq* ix, uint8_t* buf, size_t cap, size_t* written);      /* save :332 ("FLIVFPQ1") */
int fv_ivfpq_load(fv_ctx* ctx, const uint8_t* bytes, size_t len, fv_ivfpq** out);      /* load :354 */

/* ---- Hnsw (src/vector/hnsw.rs) */
typedef struct fv_hnsw fv_hnsw;
typedef struct fv_hnsw_params { /* HnswParams, hnsw.rs:24-40; defaults m=16, ef_construction=200, seed=1 */
  size_t m;
  size_t ef_construction;
  uint64_t seed;
} fv_hnsw_params;
/* Graph construction runs on the host cores (`threads` of them, as the reference's pool; 1 = deterministic). */
int fv_hnsw_build(fv_ctx* ctx, int metric, uint32_t dim, const float* vectors, size_t n,
                  const fv_hnsw_params* p, int threads, fv_hnsw** out);                /* build :85 */
/* Graph construction on the GPU, batch-synchronous (build :85, insert :244, select :230, add_links :294).  Nodes go in
 * in id order in batches of at most `max_batch` nodes and at most 1/`divisor` of the nodes already in; within a batch
 * every node searches the graph as it stood when the batch began, then the reverse links are made target by target
 * with the sources in ascending id.  The same input always gives the same graph; with max_batch = 1 it is byte for
 * byte the graph of the reference's single-thread build.  A wider batch is what `threads` is to the reference's
 * build: more nodes in flight that do not see one another.  Suggested: max_batch 8192, divisor 32. */
int fv_hnsw_build_batched(fv_ctx* ctx, int metric, uint32_t dim, const float* vectors, size_t n,
                          const fv_hnsw_params* p, size_t max_batch, size_t divisor, fv_hnsw** out);
void fv_hnsw_free(fv_hnsw* ix);
size_t fv_hnsw_len(const fv_hnsw* ix);                                                /* len :131 */
uint32_t fv_hnsw_dim(const fv_hnsw* ix);                                              /* field dim :44 */
int fv_hnsw_metric(const fv_hnsw* ix);                                                /* field metric :43 (fv_metric) */
size_t fv_hnsw_reachable(const fv_hnsw* ix);                                          /* reachable :367 */
double fv_hnsw_mean_degree(const fv_hnsw* ix);                                        /* mean_degree :388 */
int fv_hnsw_search(fv_hnsw* ix, const float* query, size_t k, size_t ef, fv_neighbor* out, uint32_t* count); /* :323 */
int fv_hnsw_search_batch(fv_hnsw* ix, const float* queries, size_t nq, size_t k, size_t ef,
                         fv_neighbor* out, uint32_t* counts);                         /* search_batch :353 */
int fv_hnsw_search_batch_dev(fv_hnsw* ix, const float* d_queries, size_t nq, size_t k, size_t ef,
                             fv_neighbor* d_out, uint32_t* d_counts);
size_t fv_hnsw_save_size(const fv_hnsw* ix);
int fv_hnsw_save(const fv_hnsw* ix, uint8_t* buf, size_t cap, size_t* written);        /* save :395 ("FLHNSW01") */
int fv_hnsw_load(fv_ctx* ctx, const uint8_t* bytes, size_t len, fv_hnsw** out);        /* load :424 */

/* ---- helpers of src/vector/mod.rs */
size_t fv_padded(size_t dim);                                                         /* padded    :113 */
int fv_normalize(float* data, size_t n, size_t dim);                                  /* normalize :132 (host, in place) */
double fv_recall(const fv_neighbor* found, const uint32_t* counts, const uint32_t* truth, size_t truth_stride,
                 size_t nq, size_t k);                                                /* recall    :145 */

/* ---- .fvecs / .ivecs benchmark files (src/vector/io.rs:7-42).  `limit` 0 = all rows.  *out is allocated by the
 * library (rows * dim values, flattened) and released with fv_free.  Errors are FV_ERR_FILE with the reference's
 * messages ("empty", "not a vecs file of dimension D", "record R has a different dimension"). */
int fv_read_fvecs(const char* path, size_t limit, float** out, size_t* n, size_t* dim);      /* read_fvecs :30 */
int fv_read_ivecs(const char* path, size_t limit, uint32_t** out, size_t* n, size_t* dim);   /* read_ivecs :36 */
void fv_free(void* p);

/* ---- searching a sharded index with one rank per GPU (no counterpart in the single-process reference).
 * The base set is split over the ranks -- contiguous row ranges for exact search (fv_flat_set_id_base), inverted
 * lists for IVF-PQ (fv_ivfpq_set_shard) -- and every rank holds a context that belongs to the same group.  Rank 0
 * makes the 128-byte group id with fv_comm_unique_id and hands it to the other ranks by whatever channel the host
 * has (a file, a socket, MPI, its own RPC); then every rank calls fv_ctx_comm_init (collective).  NCCL
 * (libnccl.so.2) is bound at run time, so hosts that never shard do not need it.
 * The *_sharded_dev searches are collective too: every rank calls them with the SAME queries (device pointers);
 * each searches its shard, the per-shard candidates are all-gathered over NVLink on the context's stream and merged
 * by a kernel of this library, and every rank gets the complete result.  HNSW is searched by replicas (one graph;
 * per-shard graphs would change the results): split the query batch over the ranks instead.
 * For IVF-PQ the group is a grid of L list shards x Q query slices, rank = slice * L + shard, where L is the shard
 * count the index was given (fv_ivfpq_set_shard; 1 when it was never called: every rank holds all lists) and
 * Q = group size / L.  A rank searches its slice of the batch on its lists; the L shards of a slice exchange and merge
 * their candidates (nothing to exchange when L = 1), and the finished slices are all-gathered.  L = group size is the
 * plain list-sharded search (for indexes beyond one GPU's memory); L = 1 divides a batch over replicas of an index
 * that fits every GPU, which costs the least per query.
 * fv_stats.stage_ms after a sharded IVF-PQ search: L = group size: 0 coarse step of the rank's query slice, 1 cell
 * exchange, 2 local search, 3 candidate exchange, 4 merge; Q > 1: 0 and 1 empty, 2 local search of the slice,
 * 3 candidate exchange, 4 merge + result exchange + unpacking. */
int fv_comm_unique_id(uint8_t* id128);
int fv_ctx_comm_init(fv_ctx* ctx, const uint8_t* id128, int nranks, int rank);
int fv_ctx_comm_rank(const fv_ctx* ctx);
int fv_ctx_comm_size(const fv_ctx* ctx);
int fv_flat_search_sharded_dev(fv_flat* ix, const float* d_queries, size_t nq, size_t k, fv_neighbor* d_out,
                               uint32_t* d_counts);
int fv_ivfpq_search_sharded_dev(fv_ivfpq* ix, const float* d_queries, size_t nq, size_t k, size_t nprobe, size_t refine,
                                fv_neighbor* d_out, uint32_t* d_counts);

/* ---- merging per-shard results (no counterpart in the single-process reference; the row-sharded layout
 * needs it).  `d_parts` holds nparts blocks of nq*k_in neighbours, `d_part_counts` nparts*nq counts (may be
 * NULL = all k_in); the k_out best by (distance, id) of each query go to d_out. */
int fv_merge_topk_dev(fv_ctx* ctx, const fv_neighbor* d_parts, const uint32_t* d_part_counts, size_t nparts,
                      size_t nq, size_t k_in, size_t k_out, fv_neighbor* d_out, uint32_t* d_counts);
/* IVF-PQ with re-ranking across shards: global best `keep` by compressed distance, then the k best of those
 * by exact distance (ivfpq.rs:285-296 done once over all shards). */
int fv_merge_refine_dev(fv_ctx* ctx, const fv_neighbor* d_adc_parts, const float* d_exact_parts,
                        const uint32_t* d_part_counts, size_t nparts, size_t nq, size_t keep, size_t k,
                        fv_neighbor* d_out, uint32_t* d_counts);

/* The same merge as fv_merge_topk_dev for callers that must not allocate device memory (a serving loop that
 * has given all free HBM to its own arena, a component of a framework whose allocator owns the device, a
 * process past its memory-budget checkpoint).  It has no counterpart in the reference and takes no context:
 * the intermediate keys live in a fixed 2 MiB array inside the library image, so the call performs no
 * cudaMalloc/cudaFree.  Limits: nq * k_out <= 262144 and k_out <= 1024, otherwise FV_ERR_UNSUPPORTED.  All
 * calls on one GPU share that array and it keeps the last call's contents (nothing in it needs clearing), so
 * calls that overlap on the GPU race: serialise them.  The call is synchronous: it runs on `stream` (a
 * cudaStream_t, NULL = default stream) of `device`, waits for it and returns when the result is complete; a
 * capturing stream is refused (FV_ERR_UNSUPPORTED) and it may not be called from a host callback.  The first
 * call on each device resolves the array's address and, with lazy module loading, places the array and the
 * kernels on the device: make it at start-up, before any stream capture and before the process has claimed
 * the last few MiB of that device. */
int fv_merge_topk_static_dev(int device, void* stream, const fv_neighbor* d_parts, const uint32_t* d_part_counts,
                             size_t nparts, size_t nq, size_t k_in, size_t k_out, fv_neighbor* d_out,
                             uint32_t* d_counts);

/* ---- seeded synthetic data for benchmarks and tests: a mixture of `clusters` Gaussians.
 * kind 0: centres uniform in [0,255]^dim, sigma 30, clipped to [0,255] and rounded (SIFT-like integers);
 * kind 1: centres normal*3, sigma 1, rows then scaled to unit length (embedding-like).
 * Row i depends only on (seed, i), so any row range can be generated independently. */
int fv_datagen(int kind, uint64_t seed, size_t first_row, size_t n, size_t dim, size_t clusters, int threads,
               float* out);

/* kind 0 of fv_datagen computed on the GPU into device memory (same streams and formulas; device libm, so a
 * value within rounding of x.5 may round differently: do not mix the two generators within one experiment). */
int fv_datagen_dev(fv_ctx* ctx, uint64_t seed, size_t first_row, size_t n, size_t dim, size_t clusters, float* d_out);

#ifdef __cplusplus
}
#endif
#endif /* FERROVEC_H */
