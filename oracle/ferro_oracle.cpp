// CPU oracle for ferrolm's vector-search path.  TEST INFRASTRUCTURE ONLY.
//
// This file is a plain C++ restatement of the reference's CPU algorithms for
// exact, IVF-PQ and HNSW search (src/vector/{mod,flat,kmeans,ivfpq,hnsw,io}.rs,
// src/kernels.rs:192-231, src/rng.rs).  It exists so that the CUDA library can
// be checked against it and so that the benchmark can time the CPU algorithm on
// the host cores.  Nothing in the shipped library links, loads or calls it.
//
// Parity status: the reference is Rust and no Rust toolchain is available to
// run it, and its own tests hold only three literal known answers for this path
// (src/vector/mod.rs:158-171) plus property thresholds (tests/vector.rs,
// src/vector/kmeans.rs:96-112).  Those are all checked in tests/; beyond them
// PARITY IS UNPINNED: it rests on this restatement following the reference's
// arithmetic order line by line.
//
// Build: g++ -O2 -std=c++17 -mavx2 -mfma -ffp-contract=off -fPIC -shared -pthread
// (-ffp-contract=off matters: only dot/l2sq fuse multiply-add, as in the reference).

#include <algorithm>
#include <atomic>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <functional>
#include <limits>
#include <memory>
#include <mutex>
#include <queue>
#include <string>
#include <thread>
#include <vector>
#if defined(__AVX2__) && defined(__FMA__)
#include <immintrin.h>
#endif

namespace {

// ---------------------------------------------------------------- rng (src/rng.rs:7-45)
struct Rng {
  uint64_t s;
  explicit Rng(uint64_t seed) : s((seed * 0x9E3779B97F4A7C15ull) | 1ull) {}
  uint64_t next_u64() {
    s ^= s >> 12;
    s ^= s << 25;
    s ^= s >> 27;
    return s * 0x2545F4914F6CDD1Dull;
  }
  uint64_t below(uint64_t n) { return next_u64() % n; }
  double uniform() { return double(next_u64() >> 11) / double(1ull << 53); }
  double normal() {
    double u = 1.0 - uniform();
    double v = uniform();
    return std::sqrt(-2.0 * std::log(u)) * std::cos(6.283185307179586476925286766559 * v);
  }
};

// ---------------------------------------------------------------- pool (src/pool.rs:74-118)
// Dynamic hand-out of task indices; each task writes its own output slot, so
// results do not depend on the thread count.
void pool_run(int threads, size_t tasks, const std::function<void(size_t)>& f) {
  if (tasks == 0) return;
  if (threads <= 1 || tasks == 1) {
    for (size_t i = 0; i < tasks; i++) f(i);
    return;
  }
  std::atomic<size_t> next{0};
  auto drain = [&]() {
    for (;;) {
      size_t i = next.fetch_add(1, std::memory_order_relaxed);
      if (i >= tasks) break;
      f(i);
    }
  };
  std::vector<std::thread> w;
  for (int t = 1; t < threads; t++) w.emplace_back(drain);
  drain();
  for (auto& t : w) t.join();
}

// ---------------------------------------------------------------- distances (src/kernels.rs:192-231, :490-515)
inline float hsum8(const float* l) {
  return ((l[0] + l[4]) + (l[2] + l[6])) + ((l[1] + l[5]) + (l[3] + l[7]));
}

inline float dot(const float* a, const float* b, size_t n) {
#if defined(__AVX2__) && defined(__FMA__)
  __m256 acc = _mm256_setzero_ps();
  for (size_t i = 0; i + 8 <= n; i += 8)
    acc = _mm256_fmadd_ps(_mm256_loadu_ps(a + i), _mm256_loadu_ps(b + i), acc);
  float l[8];
  _mm256_storeu_ps(l, acc);
  return hsum8(l);
#else
  float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  for (size_t i = 0; i + 8 <= n; i += 8)
    for (int l = 0; l < 8; l++) acc[l] = std::fmaf(a[i + l], b[i + l], acc[l]);
  return hsum8(acc);
#endif
}

inline float l2sq(const float* a, const float* b, size_t n) {
#if defined(__AVX2__) && defined(__FMA__)
  __m256 acc = _mm256_setzero_ps();
  for (size_t i = 0; i + 8 <= n; i += 8) {
    __m256 d = _mm256_sub_ps(_mm256_loadu_ps(a + i), _mm256_loadu_ps(b + i));
    acc = _mm256_fmadd_ps(d, d, acc);
  }
  float l[8];
  _mm256_storeu_ps(l, acc);
  return hsum8(l);
#else
  float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  for (size_t i = 0; i + 8 <= n; i += 8)
    for (int l = 0; l < 8; l++) {
      float d = a[i + l] - b[i + l];
      acc[l] = std::fmaf(d, d, acc[l]);
    }
  return hsum8(acc);
#endif
}

// scalar twin of the two above, used by the self-check that both paths agree
inline float dot_scalar(const float* a, const float* b, size_t n) {
  float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  for (size_t i = 0; i + 8 <= n; i += 8)
    for (int l = 0; l < 8; l++) acc[l] = std::fmaf(a[i + l], b[i + l], acc[l]);
  return hsum8(acc);
}
inline float l2sq_scalar(const float* a, const float* b, size_t n) {
  float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  for (size_t i = 0; i + 8 <= n; i += 8)
    for (int l = 0; l < 8; l++) {
      float d = a[i + l] - b[i + l];
      acc[l] = std::fmaf(d, d, acc[l]);
    }
  return hsum8(acc);
}

// ---------------------------------------------------------------- mod.rs
enum Metric : int { L2 = 0, InnerProduct = 1 };

inline float metric_distance(int metric, const float* a, const float* b, size_t n) {
  return metric == L2 ? l2sq(a, b, n) : -dot(a, b, n);  // src/vector/mod.rs:28-33
}

struct Neighbor {
  uint32_t id;
  float distance;
};

// f32::total_cmp then id (src/vector/mod.rs:60-64)
inline int32_t total_key(float f) {
  int32_t b;
  std::memcpy(&b, &f, 4);
  b ^= int32_t(uint32_t(b >> 31) >> 1);
  return b;
}
inline bool nb_less(const Neighbor& a, const Neighbor& b) {
  int32_t ka = total_key(a.distance), kb = total_key(b.distance);
  if (ka != kb) return ka < kb;
  return a.id < b.id;
}
struct NbLess {
  bool operator()(const Neighbor& a, const Neighbor& b) const { return nb_less(a, b); }
};
struct NbGreater {
  bool operator()(const Neighbor& a, const Neighbor& b) const { return nb_less(b, a); }
};

// bounded max-heap (src/vector/mod.rs:73-110)
struct TopK {
  size_t k;
  std::vector<Neighbor> heap;  // max-heap under nb_less
  explicit TopK(size_t k_) : k(k_) { heap.reserve(k_ + 1); }
  float bound() const {
    return heap.size() < k ? std::numeric_limits<float>::infinity() : heap.front().distance;
  }
  void push(Neighbor n) {
    if (heap.size() < k) {
      heap.push_back(n);
      std::push_heap(heap.begin(), heap.end(), NbLess());
    } else if (k > 0 && nb_less(n, heap.front())) {
      std::pop_heap(heap.begin(), heap.end(), NbLess());
      heap.back() = n;
      std::push_heap(heap.begin(), heap.end(), NbLess());
    }
  }
  std::vector<Neighbor> into_sorted() {
    std::sort_heap(heap.begin(), heap.end(), NbLess());
    return std::move(heap);
  }
};

inline size_t padded(size_t dim) { return (dim + 7) / 8 * 8; }

std::vector<float> pad(const float* data, size_t n, size_t dim) {
  size_t pd = padded(dim);
  std::vector<float> out(n * pd, 0.0f);
  if (pd == dim) {
    std::memcpy(out.data(), data, n * dim * sizeof(float));
    return out;
  }
  for (size_t i = 0; i < n; i++) std::memcpy(&out[i * pd], &data[i * dim], dim * sizeof(float));
  return out;
}

// Rust's f32 `Sum` folds from -0.0 and adds left to right, without fusing.
inline float seq_sum_start() { return -0.0f; }

void normalize(float* data, size_t n, size_t dim) {  // src/vector/mod.rs:132-141
  for (size_t i = 0; i < n; i++) {
    float* v = data + i * dim;
    float s = seq_sum_start();
    for (size_t d = 0; d < dim; d++) s = s + v[d] * v[d];
    float nn = std::sqrt(s);
    if (nn > 0.0f)
      for (size_t d = 0; d < dim; d++) v[d] /= nn;
  }
}

// ---------------------------------------------------------------- flat.rs
struct Flat {
  int metric;
  size_t dim, pd;
  std::vector<float> data;
  size_t len() const { return data.size() / pd; }
  void add(const float* v, size_t n) {
    auto p = pad(v, n, dim);
    data.insert(data.end(), p.begin(), p.end());
  }
  std::vector<Neighbor> search(const float* query, size_t k) const {  // src/vector/flat.rs:40-53
    auto q = pad(query, 1, dim);
    TopK top(k);
    size_t n = len();
    for (size_t i = 0; i < n; i++) {
      float d = metric_distance(metric, q.data(), &data[i * pd], pd);
      if (d < top.bound()) top.push({uint32_t(i), d});
    }
    return top.into_sorted();
  }
};

// ---------------------------------------------------------------- kmeans.rs
inline std::pair<size_t, float> km_nearest(const float* x, const float* cen, size_t k, size_t dim) {
  size_t bc = 0;
  float bd = std::numeric_limits<float>::infinity();
  for (size_t c = 0; c < k; c++) {
    float d = l2sq(x, cen + c * dim, dim);
    if (d < bd) {
      bc = c;
      bd = d;
    }
  }
  return {bc, bd};
}

std::vector<uint32_t> km_assign(int threads, const float* data, size_t n, const float* cen, size_t k, size_t dim) {
  std::vector<uint32_t> out(n, 0);
  const size_t CHUNK = 256;
  pool_run(threads, (n + CHUNK - 1) / CHUNK, [&](size_t t) {
    for (size_t i = t * CHUNK; i < std::min((t + 1) * CHUNK, n); i++)
      out[i] = uint32_t(km_nearest(data + i * dim, cen, k, dim).first);
  });
  return out;
}

// src/vector/kmeans.rs:39-90
std::vector<float> km_train(int threads, const float* data, size_t n, size_t dim, size_t k, size_t iters,
                            uint64_t seed) {
  Rng rng(seed);
  std::vector<size_t> idx(n);
  for (size_t i = 0; i < n; i++) idx[i] = i;
  for (size_t i = 0; i < k; i++) {
    size_t j = i + size_t(rng.below(uint64_t(n - i)));
    std::swap(idx[i], idx[j]);
  }
  std::vector<float> cen(k * dim);
  for (size_t c = 0; c < k; c++) std::memcpy(&cen[c * dim], data + idx[c] * dim, dim * sizeof(float));
  for (size_t it = 0; it < iters; it++) {
    auto a = km_assign(threads, data, n, cen.data(), k, dim);
    std::vector<double> sums(k * dim, 0.0);
    std::vector<size_t> counts(k, 0);
    for (size_t i = 0; i < n; i++) {
      size_t c = a[i];
      counts[c]++;
      double* s = &sums[c * dim];
      const float* v = data + i * dim;
      for (size_t d = 0; d < dim; d++) s[d] += double(v[d]);
    }
    for (size_t c = 0; c < k; c++)
      if (counts[c] > 0)
        for (size_t d = 0; d < dim; d++) cen[c * dim + d] = float(sums[c * dim + d] / double(counts[c]));
    for (size_t c = 0; c < k; c++) {
      if (counts[c] == 0) {
        // max_by_key returns the LAST maximum
        size_t big = 0;
        for (size_t j = 0; j < k; j++)
          if (counts[j] >= counts[big]) big = j;
        for (size_t d = 0; d < dim; d++) {
          float v = cen[big * dim + d];
          float e = 1e-4f * (1.0f + std::fabs(v));
          cen[c * dim + d] = v + e;
          cen[big * dim + d] = v - e;
        }
        counts[c] = counts[big] / 2;
        counts[big] -= counts[c];
      }
    }
  }
  return cen;
}

// ---------------------------------------------------------------- io.rs writer/reader
struct Writer {
  std::vector<uint8_t> b;
  void raw(const void* p, size_t n) {
    const uint8_t* c = static_cast<const uint8_t*>(p);
    b.insert(b.end(), c, c + n);
  }
  void u32(uint32_t v) { raw(&v, 4); }
  void u64(uint64_t v) { raw(&v, 8); }
  void f32s(const float* v, size_t n) {
    u64(n);
    raw(v, n * 4);
  }
  void u32s(const uint32_t* v, size_t n) {
    u64(n);
    raw(v, n * 4);
  }
  void bytes(const uint8_t* v, size_t n) {
    u64(n);
    raw(v, n);
  }
};

struct Reader {
  const uint8_t* b;
  size_t len, i = 0;
  bool ok = true;
  Reader(const uint8_t* p, size_t n) : b(p), len(n) {}
  const uint8_t* take(size_t n) {
    if (!ok || n > len - i) {
      ok = false;
      return nullptr;
    }
    const uint8_t* s = b + i;
    i += n;
    return s;
  }
  uint32_t u32() {
    auto p = take(4);
    uint32_t v = 0;
    if (p) std::memcpy(&v, p, 4);
    return v;
  }
  uint64_t u64() {
    auto p = take(8);
    uint64_t v = 0;
    if (p) std::memcpy(&v, p, 8);
    return v;
  }
  template <class T>
  std::vector<T> vec() {
    uint64_t n = u64();
    std::vector<T> out;
    if (!ok || n > (len - i) / sizeof(T)) {
      ok = false;
      return out;
    }
    auto p = take(size_t(n) * sizeof(T));
    if (!p) return out;
    out.resize(size_t(n));
    std::memcpy(out.data(), p, size_t(n) * sizeof(T));
    return out;
  }
};

// ---------------------------------------------------------------- ivfpq.rs
const size_t KSUB = 256;
const size_t MAX_PRE = size_t(64) << 20;

struct IvfPq {
  int metric;
  size_t dim, pd, nlist, m, dsub;
  std::vector<float> centroids, codebooks;
  std::vector<std::vector<uint32_t>> ids;
  std::vector<std::vector<uint8_t>> codes;
  bool has_vectors = false;
  std::vector<float> vectors;
  size_t count = 0;
  std::vector<float> pre;

  static float sub_distance(const float* a, const float* b, size_t n) {  // ivfpq.rs:141-143
    float s = seq_sum_start();
    for (size_t t = 0; t < n; t++) {
      float d = a[t] - b[t];
      s = s + d * d;
    }
    return s;
  }

  void with_tables() {  // ivfpq.rs:108-126
    pre.clear();
    size_t size = nlist * m * KSUB;
    if (metric != L2 || size > MAX_PRE) return;
    pre.assign(size, 0.0f);
    for (size_t l = 0; l < nlist; l++) {
      float* t = &pre[l * m * KSUB];
      const float* cen = &centroids[l * pd];
      for (size_t j = 0; j < m; j++) {
        const float* cj = cen + j * dsub;
        const float* cb = &codebooks[j * KSUB * dsub];
        for (size_t c = 0; c < KSUB; c++) {
          const float* w = cb + c * dsub;
          float s = seq_sum_start();
          for (size_t x = 0; x < dsub; x++) {
            float a = w[x], b = cj[x];
            s = s + (a * a + 2.0f * a * b);
          }
          t[j * KSUB + c] = s;
        }
      }
    }
  }

  void encode(const float* resid, uint8_t* out) const {  // ivfpq.rs:145-158
    for (size_t j = 0; j < m; j++) {
      const float* r = resid + j * dsub;
      const float* cb = &codebooks[j * KSUB * dsub];
      uint8_t bc = 0;
      float bd = std::numeric_limits<float>::infinity();
      for (size_t c = 0; c < KSUB; c++) {
        float d = sub_distance(r, cb + c * dsub, dsub);
        if (d < bd) {
          bc = uint8_t(c);
          bd = d;
        }
      }
      out[j] = bc;
    }
  }

  std::vector<Neighbor> nearest_cells(const float* q, size_t nprobe) const {  // ivfpq.rs:211-220
    TopK top(nprobe);
    for (size_t c = 0; c < nlist; c++) top.push({uint32_t(c), metric_distance(metric, q, &centroids[c * pd], pd)});
    return top.into_sorted();
  }

  std::vector<uint32_t> coarse_assign(int threads, const float* x, size_t n) const {  // ivfpq.rs:194-204
    if (metric == L2) return km_assign(threads, x, n, centroids.data(), nlist, pd);
    std::vector<uint32_t> out(n);
    for (size_t i = 0; i < n; i++) out[i] = nearest_cells(x + i * pd, 1)[0].id;
    return out;
  }

  void add(int threads, const float* v, size_t n) {  // ivfpq.rs:161-192
    auto x = pad(v, n, dim);
    auto assign = coarse_assign(threads, x.data(), n);
    std::vector<uint8_t> cds(n * m);
    const size_t CHUNK = 512;
    pool_run(threads, (n + CHUNK - 1) / CHUNK, [&](size_t t) {
      std::vector<float> resid(pd);
      for (size_t i = t * CHUNK; i < std::min((t + 1) * CHUNK, n); i++) {
        const float* c = &centroids[size_t(assign[i]) * pd];
        for (size_t d = 0; d < pd; d++) resid[d] = x[i * pd + d] - c[d];
        encode(resid.data(), &cds[i * m]);
      }
    });
    for (size_t i = 0; i < n; i++) {
      size_t l = assign[i];
      ids[l].push_back(uint32_t(count + i));
      codes[l].insert(codes[l].end(), &cds[i * m], &cds[(i + 1) * m]);
    }
    if (has_vectors) vectors.insert(vectors.end(), x.begin(), x.end());
    count += n;
  }

  void fill_lut(const float* r, float* lut) const {  // ivfpq.rs:300-311
    for (size_t j = 0; j < m; j++) {
      const float* rs = r + j * dsub;
      const float* cb = &codebooks[j * KSUB * dsub];
      for (size_t c = 0; c < KSUB; c++) {
        const float* w = cb + c * dsub;
        if (metric == L2) {
          lut[j * KSUB + c] = sub_distance(rs, w, dsub);
        } else {
          float s = seq_sum_start();
          for (size_t t = 0; t < dsub; t++) s = s + rs[t] * w[t];
          lut[j * KSUB + c] = -s;
        }
      }
    }
  }

  // ivfpq.rs:225-297.  `scanned` (optional) receives the number of code rows visited.
  std::vector<Neighbor> search(const float* query, size_t k, size_t nprobe, size_t refine,
                               uint64_t* scanned = nullptr) const {
    auto q = pad(query, 1, dim);
    auto cells = nearest_cells(q.data(), std::min(nprobe, nlist));
    size_t keep = (refine > 0 && has_vectors) ? k * refine : k;
    TopK top(keep);
    std::vector<float> lut(m * KSUB, 0.0f);
    if (metric == InnerProduct) fill_lut(q.data(), lut.data());
    std::vector<float> rq(pd, 0.0f);
    std::vector<float> qlut;
    if (metric == L2 && !pre.empty()) {
      qlut.assign(m * KSUB, 0.0f);
      for (size_t j = 0; j < m; j++) {
        const float* qj = &q[j * dsub];
        const float* cb = &codebooks[j * KSUB * dsub];
        for (size_t c = 0; c < KSUB; c++) {
          const float* w = cb + c * dsub;
          float s = seq_sum_start();
          for (size_t t = 0; t < dsub; t++) s = s + qj[t] * w[t];
          qlut[j * KSUB + c] = -2.0f * s;
        }
      }
    }
    uint64_t rows = 0;
    for (const Neighbor& cell : cells) {
      size_t l = cell.id;
      const float* cen = &centroids[l * pd];
      float base;
      if (metric == L2 && !qlut.empty()) {
        const float* p = &pre[l * m * KSUB];
        for (size_t i = 0; i < m * KSUB; i++) lut[i] = p[i] + qlut[i];
        base = cell.distance;
      } else if (metric == L2) {
        for (size_t d = 0; d < pd; d++) rq[d] = q[d] - cen[d];
        fill_lut(rq.data(), lut.data());
        base = 0.0f;
      } else {
        base = -dot(q.data(), cen, pd);
      }
      const std::vector<uint8_t>& cl = codes[l];
      size_t nrows = cl.size() / m;
      rows += nrows;
      for (size_t i = 0; i < nrows; i++) {
        const uint8_t* code = &cl[i * m];
        float d = base;
        for (size_t j = 0; j < m; j++) d += lut[j * KSUB + code[j]];
        if (d < top.bound()) top.push({ids[l][i], d});
      }
    }
    if (scanned) *scanned = rows;
    auto cand = top.into_sorted();
    if (has_vectors && refine > 0) {
      TopK exact(k);
      for (const Neighbor& c : cand)
        exact.push({c.id, metric_distance(metric, q.data(), &vectors[size_t(c.id) * pd], pd)});
      return exact.into_sorted();
    }
    if (cand.size() > k) cand.resize(k);
    return cand;
  }

  std::vector<uint8_t> save() const {  // ivfpq.rs:332-352
    Writer w;
    w.raw("FLIVFPQ1", 8);
    w.u32(uint32_t(metric));
    w.u32(uint32_t(dim));
    w.u32(uint32_t(nlist));
    w.u32(uint32_t(m));
    w.u32(uint32_t(count));
    w.f32s(centroids.data(), centroids.size());
    w.f32s(codebooks.data(), codebooks.size());
    for (size_t l = 0; l < nlist; l++) {
      w.u32s(ids[l].data(), ids[l].size());
      w.bytes(codes[l].data(), codes[l].size());
    }
    w.f32s(vectors.data(), has_vectors ? vectors.size() : 0);
    w.u32(has_vectors ? 1u : 0u);
    return std::move(w.b);
  }
};

IvfPq* ivfpq_train(int threads, int metric, size_t dim, const float* sample, size_t n, size_t nlist, size_t m,
                   size_t iters, bool keep, uint64_t seed) {  // ivfpq.rs:56-106
  size_t pd = padded(dim);
  if (m == 0 || pd % m != 0 || n < nlist) return nullptr;
  auto x = pad(sample, n, dim);
  auto* ix = new IvfPq();
  ix->metric = metric;
  ix->dim = dim;
  ix->pd = pd;
  ix->nlist = nlist;
  ix->m = m;
  ix->dsub = pd / m;
  ix->centroids = km_train(threads, x.data(), n, pd, nlist, iters, seed);
  auto assign = km_assign(threads, x.data(), n, ix->centroids.data(), nlist, pd);
  size_t dsub = ix->dsub;
  std::vector<float> resid = x;
  for (size_t i = 0; i < n; i++) {
    const float* c = &ix->centroids[size_t(assign[i]) * pd];
    for (size_t d = 0; d < pd; d++) resid[i * pd + d] -= c[d];
  }
  ix->codebooks.assign(m * KSUB * dsub, 0.0f);
  size_t ksub = std::min(KSUB, n);
  for (size_t j = 0; j < m; j++) {
    std::vector<float> cb;
    if (dsub % 8 == 0) {
      std::vector<float> sub(n * dsub);
      for (size_t i = 0; i < n; i++) std::memcpy(&sub[i * dsub], &resid[i * pd + j * dsub], dsub * sizeof(float));
      cb = km_train(threads, sub.data(), n, dsub, ksub, iters, seed + 1 + j);
    } else {
      size_t ps = padded(dsub);
      std::vector<float> sp(n * ps, 0.0f);
      for (size_t i = 0; i < n; i++) std::memcpy(&sp[i * ps], &resid[i * pd + j * dsub], dsub * sizeof(float));
      auto c = km_train(threads, sp.data(), n, ps, ksub, iters, seed + 1 + j);
      cb.resize(ksub * dsub);
      for (size_t r = 0; r < ksub; r++) std::memcpy(&cb[r * dsub], &c[r * ps], dsub * sizeof(float));
    }
    std::memcpy(&ix->codebooks[j * KSUB * dsub], cb.data(), cb.size() * sizeof(float));
  }
  ix->ids.assign(nlist, {});
  ix->codes.assign(nlist, {});
  ix->has_vectors = keep;
  ix->with_tables();
  return ix;
}

IvfPq* ivfpq_load(const uint8_t* bytes, size_t len, std::string& err) {  // ivfpq.rs:354-390
  if (len < 8 || std::memcmp(bytes, "FLIVFPQ1", 8) != 0) {
    err = "not an IVF-PQ index file";
    return nullptr;
  }
  Reader r(bytes + 8, len - 8);
  uint32_t mc = r.u32();
  auto ix = std::make_unique<IvfPq>();
  ix->dim = r.u32();
  ix->nlist = r.u32();
  ix->m = r.u32();
  ix->count = r.u32();
  if (!r.ok) {
    err = "index file is truncated";
    return nullptr;
  }
  if ((mc & 0xFF) > 1) {
    err = "bad metric";
    return nullptr;
  }
  ix->metric = int(mc & 0xFF);
  ix->centroids = r.vec<float>();
  ix->codebooks = r.vec<float>();
  for (size_t l = 0; l < ix->nlist && r.ok; l++) {
    ix->ids.push_back(r.vec<uint32_t>());
    ix->codes.push_back(r.vec<uint8_t>());
  }
  auto v = r.vec<float>();
  bool has = r.u32() == 1;
  if (!r.ok) {
    err = "index file is truncated";
    return nullptr;
  }
  ix->pd = padded(ix->dim);
  if (ix->m == 0) {
    err = "index file sizes do not match";
    return nullptr;
  }
  ix->dsub = ix->pd / ix->m;
  ix->has_vectors = has;
  if (has) ix->vectors = std::move(v);
  ix->with_tables();
  return ix.release();
}

// ---------------------------------------------------------------- hnsw.rs
struct Hnsw {
  int metric;
  size_t dim, pd, m, m0;
  std::vector<float> data;
  std::vector<uint8_t> levels;
  std::vector<uint32_t> links0;               // n * (m0 + 1): count then ids
  std::vector<std::vector<std::vector<uint32_t>>> upper;  // per node, layers 1..
  std::unique_ptr<std::mutex[]> locks;
  std::mutex entry_lock;
  uint32_t ep = 0;
  size_t top = 0;

  size_t len() const { return levels.size(); }
  const float* vec(uint32_t id) const { return &data[size_t(id) * pd]; }
  float dist(const float* q, uint32_t id) const { return metric_distance(metric, q, vec(id), pd); }

  void neighbors(uint32_t id, size_t layer, bool locked, std::vector<uint32_t>& out) {  // hnsw.rs:151-163
    out.clear();
    std::unique_lock<std::mutex> g;
    if (locked) g = std::unique_lock<std::mutex>(locks[id]);
    if (layer == 0) {
      size_t base = size_t(id) * (m0 + 1);
      size_t c = links0[base];
      out.insert(out.end(), &links0[base + 1], &links0[base + 1 + c]);
    } else {
      out = upper[id][layer - 1];
    }
  }
  void set_neighbors(uint32_t id, size_t layer, const std::vector<uint32_t>& list) {  // hnsw.rs:165-175
    if (layer == 0) {
      size_t base = size_t(id) * (m0 + 1);
      for (size_t i = 0; i < list.size(); i++) links0[base + 1 + i] = list[i];
      links0[base] = uint32_t(list.size());
    } else {
      upper[id][layer - 1] = list;
    }
  }

  struct Visited {
    std::vector<uint32_t> v;
    uint32_t stamp = 0;
  };

  // hnsw.rs:179-226.  n_dist / n_expand count distance evaluations and expansions.
  std::vector<Neighbor> search_layer(const float* q, const std::vector<Neighbor>& entry, size_t ef, size_t layer,
                                     bool locked, Visited& vs, uint64_t* n_dist = nullptr,
                                     uint64_t* n_expand = nullptr) {
    if (vs.v.size() < len()) {
      vs.v.assign(len(), 0);
      vs.stamp = 0;
    }
    vs.stamp += 1;
    if (vs.stamp == 0) {
      std::fill(vs.v.begin(), vs.v.end(), 0);
      vs.stamp = 1;
    }
    uint32_t stamp = vs.stamp;
    std::priority_queue<Neighbor, std::vector<Neighbor>, NbGreater> cand;  // min-heap
    std::priority_queue<Neighbor, std::vector<Neighbor>, NbLess> best;     // max-heap
    for (const Neighbor& e : entry) {
      vs.v[e.id] = stamp;
      cand.push(e);
      best.push(e);
    }
    while (best.size() > ef) best.pop();
    std::vector<uint32_t> nb;
    nb.reserve(m0);
    while (!cand.empty()) {
      Neighbor c = cand.top();
      cand.pop();
      if (best.size() >= ef && c.distance > best.top().distance) break;
      neighbors(c.id, layer, locked, nb);
      if (n_expand) (*n_expand)++;
      for (uint32_t x : nb) {
        if (vs.v[x] == stamp) continue;
        vs.v[x] = stamp;
        float d = dist(q, x);
        if (n_dist) (*n_dist)++;
        if (best.size() < ef || d < best.top().distance) {
          Neighbor n{x, d};
          cand.push(n);
          best.push(n);
          if (best.size() > ef) best.pop();
        }
      }
    }
    std::vector<Neighbor> out;
    out.reserve(best.size());
    while (!best.empty()) {
      out.push_back(best.top());
      best.pop();
    }
    std::reverse(out.begin(), out.end());
    return out;
  }

  std::vector<uint32_t> select(const std::vector<Neighbor>& cands, size_t mm) const {  // hnsw.rs:230-242
    std::vector<uint32_t> out;
    out.reserve(mm);
    for (const Neighbor& c : cands) {
      if (out.size() >= mm) break;
      const float* cv = vec(c.id);
      bool all = true;
      for (uint32_t s : out)
        if (!(metric_distance(metric, cv, vec(s), pd) > c.distance)) {
          all = false;
          break;
        }
      if (all) out.push_back(c.id);
    }
    return out;
  }

  void add_links(uint32_t id, size_t layer, const std::vector<uint32_t>& nw, size_t cap) {  // hnsw.rs:294-320
    std::lock_guard<std::mutex> g(locks[id]);
    std::vector<uint32_t> list;
    neighbors(id, layer, false, list);
    size_t before = list.size();
    for (uint32_t x : nw)
      if (x != id && std::find(list.begin(), list.end(), x) == list.end()) list.push_back(x);
    if (list.size() == before) return;
    if (list.size() > cap) {
      const float* base = vec(id);
      std::vector<Neighbor> c;
      c.reserve(list.size());
      for (uint32_t x : list) c.push_back({x, metric_distance(metric, base, vec(x), pd)});
      std::sort(c.begin(), c.end(), NbLess());
      list = select(c, cap);
    }
    set_neighbors(id, layer, list);
  }

  void insert(uint32_t id, size_t ef, Visited& vs) {  // hnsw.rs:244-290
    std::vector<float> q(vec(id), vec(id) + pd);
    size_t level = levels[id];
    uint32_t e0;
    size_t tp;
    {
      std::lock_guard<std::mutex> g(entry_lock);
      e0 = ep;
      tp = top;
    }
    Neighbor cur{e0, dist(q.data(), e0)};
    std::vector<uint32_t> nb;
    for (size_t layer = tp; layer >= level + 1; layer--) {
      bool changed = true;
      while (changed) {
        changed = false;
        neighbors(cur.id, layer, true, nb);
        for (uint32_t x : nb) {
          float d = dist(q.data(), x);
          if (d < cur.distance) {
            cur = {x, d};
            changed = true;
          }
        }
      }
    }
    std::vector<Neighbor> entry{cur};
    for (size_t layer = std::min(level, tp) + 1; layer-- > 0;) {
      auto found = search_layer(q.data(), entry, ef, layer, true, vs);
      size_t cap = layer == 0 ? m0 : m;
      auto chosen = select(found, cap);
      add_links(id, layer, chosen, cap);
      std::vector<uint32_t> me{id};
      for (uint32_t n : chosen) add_links(n, layer, me, cap);
      entry = std::move(found);
    }
    if (level > tp) {
      std::lock_guard<std::mutex> g(entry_lock);
      if (level > top) {
        ep = id;
        top = level;
      }
    }
  }

  // The first half of insert (hnsw.rs:244-279) for the batch-synchronous build: the descent, the per-layer
  // search_layer and select, and the node's own lists; the reverse links (hnsw.rs:280-282) are only recorded as
  // (target, layer, source), and the entry point is left alone.
  struct PendingLink {
    uint32_t target, layer, source;
  };
  void insert_forward(uint32_t id, size_t ef, Visited& vs, std::vector<PendingLink>& pending) {
    std::vector<float> q(vec(id), vec(id) + pd);
    size_t level = levels[id];
    Neighbor cur{ep, dist(q.data(), ep)};
    std::vector<uint32_t> nb;
    for (size_t layer = top; layer >= level + 1; layer--) {
      bool changed = true;
      while (changed) {
        changed = false;
        neighbors(cur.id, layer, false, nb);
        for (uint32_t x : nb) {
          float d = dist(q.data(), x);
          if (d < cur.distance) {
            cur = {x, d};
            changed = true;
          }
        }
      }
    }
    std::vector<Neighbor> entry{cur};
    for (size_t layer = std::min(level, top) + 1; layer-- > 0;) {
      auto found = search_layer(q.data(), entry, ef, layer, false, vs);
      size_t cap = layer == 0 ? m0 : m;
      auto chosen = select(found, cap);
      add_links(id, layer, chosen, cap);
      for (uint32_t n : chosen) pending.push_back({n, uint32_t(layer), id});
      entry = std::move(found);
    }
  }

  // hnsw.rs:323-351
  std::vector<Neighbor> search(const float* query, size_t k, size_t ef, Visited& vs, uint64_t* n_dist = nullptr,
                               uint64_t* n_expand = nullptr) {
    if (len() == 0) return {};
    auto q = pad(query, 1, dim);
    Neighbor cur{ep, dist(q.data(), ep)};
    if (n_dist) (*n_dist)++;
    std::vector<uint32_t> nb;
    for (size_t layer = top; layer >= 1; layer--) {
      bool changed = true;
      while (changed) {
        changed = false;
        neighbors(cur.id, layer, false, nb);
        if (n_expand) (*n_expand)++;
        for (uint32_t x : nb) {
          float d = dist(q.data(), x);
          if (n_dist) (*n_dist)++;
          if (d < cur.distance) {
            cur = {x, d};
            changed = true;
          }
        }
      }
    }
    auto r = search_layer(q.data(), {cur}, std::max(ef, k), 0, false, vs, n_dist, n_expand);
    if (r.size() > k) r.resize(k);
    return r;
  }

  size_t reachable() {  // hnsw.rs:367-385
    if (len() == 0) return 0;
    std::vector<char> seen(len(), 0);
    std::vector<uint32_t> stack{ep};
    seen[ep] = 1;
    std::vector<uint32_t> nb;
    size_t count = 0;
    while (!stack.empty()) {
      uint32_t x = stack.back();
      stack.pop_back();
      count++;
      neighbors(x, 0, false, nb);
      for (uint32_t y : nb)
        if (!seen[y]) {
          seen[y] = 1;
          stack.push_back(y);
        }
    }
    return count;
  }

  double mean_degree() const {  // hnsw.rs:388-393
    uint64_t total = 0;
    for (size_t i = 0; i < len(); i++) total += links0[i * (m0 + 1)];
    return double(total) / double(std::max<size_t>(len(), 1));
  }

  std::vector<uint8_t> save() const {  // hnsw.rs:395-422
    Writer w;
    w.raw("FLHNSW01", 8);
    w.u32(uint32_t(metric));
    w.u32(uint32_t(dim));
    w.u32(uint32_t(m));
    w.u32(ep);
    w.u32(uint32_t(top));
    w.bytes(levels.data(), levels.size());
    w.u32s(links0.data(), links0.size());
    std::vector<uint32_t> flat;
    for (const auto& u : upper)
      for (const auto& list : u) {
        flat.push_back(uint32_t(list.size()));
        flat.insert(flat.end(), list.begin(), list.end());
      }
    w.u32s(flat.data(), flat.size());
    w.f32s(data.data(), data.size());
    return std::move(w.b);
  }
};

// hnsw.rs:85-112: the rows padded, the levels drawn, every list empty, node 0 the entry point
static Hnsw* hnsw_prepare(int metric, size_t dim, const float* vectors, size_t n, size_t m, uint64_t seed) {
  auto* h = new Hnsw();
  h->metric = metric;
  h->dim = dim;
  h->pd = padded(dim);
  h->m = m;
  h->m0 = 2 * m;
  h->data = pad(vectors, n, dim);
  double ml = 1.0 / std::log(double(m));
  Rng rng(seed);
  h->levels.resize(n);
  for (size_t i = 0; i < n; i++) {
    double v = -std::log(1.0 - rng.uniform()) * ml;
    // Rust `as usize` saturates: NaN -> 0, negative -> 0, huge -> max
    size_t lv = (v != v || v <= 0.0) ? 0 : (v >= 1.8e19 ? SIZE_MAX : size_t(v));
    h->levels[i] = uint8_t(std::min<size_t>(lv, 15));
  }
  h->upper.resize(n);
  for (size_t i = 0; i < n; i++) h->upper[i].assign(h->levels[i], {});
  h->links0.assign(n * (h->m0 + 1), 0);
  h->locks.reset(new std::mutex[std::max<size_t>(n, 1)]);
  h->ep = 0;
  h->top = n ? h->levels[0] : 0;
  return h;
}

Hnsw* hnsw_build(int threads, int metric, size_t dim, const float* vectors, size_t n, size_t m, size_t efc,
                 uint64_t seed) {  // hnsw.rs:85-129
  Hnsw* h = hnsw_prepare(metric, dim, vectors, n, m, seed);
  if (n <= 1) return h;
  std::atomic<size_t> next{1};
  int nt = std::max(threads, 1);
  pool_run(nt, size_t(nt), [&](size_t) {
    Hnsw::Visited vs;
    for (;;) {
      size_t i = next.fetch_add(1, std::memory_order_relaxed);
      if (i >= n) break;
      h->insert(uint32_t(i), efc, vs);
    }
  });
  return h;
}

// The batch-synchronous order of the same construction, as the GPU build of the product runs it: nodes go in in id
// order in batches of at most `max_batch` nodes and at most 1/`divisor` of the nodes already in, a node whose level
// is above the current top layer going in alone.  Within a batch every node runs the first half of insert
// (hnsw.rs:244-279) against the graph as it stood when the batch began; then the reverse links
// (add_links(n, layer, [id]), hnsw.rs:280-282) are made in ascending source id, and the entry point moves
// (hnsw.rs:285-289).  With max_batch = 1 this is hnsw_build with one thread.
Hnsw* hnsw_build_batched(int metric, size_t dim, const float* vectors, size_t n, size_t m, size_t efc, uint64_t seed,
                         size_t max_batch, size_t divisor) {
  Hnsw* h = hnsw_prepare(metric, dim, vectors, n, m, seed);
  if (n <= 1) return h;
  Hnsw::Visited vs;
  std::vector<Hnsw::PendingLink> pending;
  size_t inserted = 1;
  while (inserted < n) {
    size_t b = std::max<size_t>(1, std::min(max_batch, inserted / std::max<size_t>(1, divisor)));
    b = std::min(b, n - inserted);
    if (h->levels[inserted] > h->top) {
      b = 1;
    } else {
      for (size_t j = 1; j < b; j++)
        if (h->levels[inserted + j] > h->top) {
          b = j;
          break;
        }
    }
    pending.clear();
    for (size_t j = 0; j < b; j++) h->insert_forward(uint32_t(inserted + j), efc, vs, pending);
    // pending is in ascending source id already (nodes were taken in id order)
    for (const auto& e : pending) h->add_links(e.target, e.layer, {e.source}, e.layer == 0 ? h->m0 : h->m);
    if (h->levels[inserted] > h->top) {
      h->ep = uint32_t(inserted);
      h->top = h->levels[inserted];
    }
    inserted += b;
  }
  return h;
}

Hnsw* hnsw_load(const uint8_t* bytes, size_t len, std::string& err) {  // hnsw.rs:424-466
  if (len < 8 || std::memcmp(bytes, "FLHNSW01", 8) != 0) {
    err = "not an HNSW index file";
    return nullptr;
  }
  Reader r(bytes + 8, len - 8);
  uint32_t mc = r.u32();
  auto h = std::make_unique<Hnsw>();
  h->dim = r.u32();
  h->m = r.u32();
  h->ep = r.u32();
  h->top = r.u32();
  if (!r.ok) {
    err = "index file is truncated";
    return nullptr;
  }
  if ((mc & 0xFF) > 1) {
    err = "bad metric";
    return nullptr;
  }
  h->metric = int(mc & 0xFF);
  h->levels = r.vec<uint8_t>();
  h->links0 = r.vec<uint32_t>();
  auto flat = r.vec<uint32_t>();
  h->data = r.vec<float>();
  if (!r.ok) {
    err = "index file is truncated";
    return nullptr;
  }
  size_t n = h->levels.size();
  h->upper.resize(n);
  size_t i = 0;
  for (size_t node = 0; node < n; node++) {
    for (size_t l = 0; l < h->levels[node]; l++) {
      if (i >= flat.size()) {
        err = "truncated links";
        return nullptr;
      }
      size_t c = flat[i];
      if (i + 1 + c > flat.size()) {
        err = "truncated links";
        return nullptr;
      }
      h->upper[node].emplace_back(flat.begin() + i + 1, flat.begin() + i + 1 + c);
      i += 1 + c;
    }
  }
  h->pd = padded(h->dim);
  h->m0 = 2 * h->m;
  if (h->links0.size() != n * (2 * h->m + 1) || h->data.size() != n * h->pd) {
    err = "index file sizes do not match";
    return nullptr;
  }
  h->locks.reset(new std::mutex[std::max<size_t>(n, 1)]);
  return h.release();
}

void set_err(char* err, size_t cap, const std::string& s) {
  if (err && cap) {
    std::snprintf(err, cap, "%s", s.c_str());
  }
}

size_t copy_out(const std::vector<uint8_t>& b, uint8_t* buf, size_t cap) {
  if (buf && cap >= b.size()) std::memcpy(buf, b.data(), b.size());
  return b.size();
}

void write_rows(const std::vector<Neighbor>& r, size_t k, Neighbor* out, uint32_t* counts, size_t i) {
  size_t c = std::min(r.size(), k);
  for (size_t j = 0; j < c; j++) out[i * k + j] = r[j];
  for (size_t j = c; j < k; j++) out[i * k + j] = {0xFFFFFFFFu, std::numeric_limits<float>::infinity()};
  counts[i] = uint32_t(c);
}

}  // namespace

// =============================================================== C interface (ctypes)
extern "C" {

struct orc_neighbor {
  uint32_t id;
  float distance;
};
static_assert(sizeof(orc_neighbor) == 8 && sizeof(Neighbor) == 8, "Neighbor is 8 bytes");

int orc_has_avx2() {
#if defined(__AVX2__) && defined(__FMA__)
  return 1;
#else
  return 0;
#endif
}

// ---- rng
void* orc_rng_new(uint64_t seed) { return new Rng(seed); }
void orc_rng_free(void* r) { delete static_cast<Rng*>(r); }
uint64_t orc_rng_next(void* r) { return static_cast<Rng*>(r)->next_u64(); }
uint64_t orc_rng_below(void* r, uint64_t n) { return static_cast<Rng*>(r)->below(n); }
double orc_rng_uniform(void* r) { return static_cast<Rng*>(r)->uniform(); }
double orc_rng_normal(void* r) { return static_cast<Rng*>(r)->normal(); }

// The generator of the reference's integration tests (tests/vector.rs:11-24).
void orc_testdata(size_t n, size_t dim, uint64_t seed, float* out) {
  Rng crng(12345 + dim);
  std::vector<float> centres(50 * dim);
  for (auto& c : centres) c = float(crng.normal()) * 3.0f;
  Rng rng(seed);
  for (size_t i = 0; i < n; i++) {
    size_t c = size_t(rng.below(50));
    for (size_t d = 0; d < dim; d++) out[i * dim + d] = centres[c * dim + d] + float(rng.normal());
  }
}

// The benchmark's stand-in for SIFT1M and for encoder embeddings: a seeded mixture of `clusters` Gaussians whose row i
// depends on (seed, i) only.  kind 0: centres uniform in [0, 255]^dim, sigma 30, rounded and clipped to [0, 255];
// kind 1: centres normal * 3, sigma 1, rows scaled to unit length.  The product library generates the same rows
// (its fv_datagen); this copy lets the CPU arm of the benchmark run without loading that library.
void orc_datagen(int kind, uint64_t seed, size_t first_row, size_t n, size_t dim, size_t clusters, int threads, float* out) {
  std::vector<float> centres(clusters * dim);
  {
    Rng c(seed * 1000003ull + 17);
    for (auto& v : centres) v = kind == 0 ? float(c.uniform() * 255.0) : float(c.normal()) * 3.0f;
  }
  pool_run(threads, n, [&](size_t i) {
    const size_t row = first_row + i;
    Rng r(seed ^ ((row + 1) * 0xD1B54A32D192ED03ull));
    r.next_u64();
    const size_t c = size_t(r.next_u64() % clusters);
    float* o = out + i * dim;
    if (kind == 0) {
      for (size_t d = 0; d < dim; d++) {
        float v = centres[c * dim + d] + float(r.normal()) * 30.0f;
        v = std::nearbyint(v);
        o[d] = v < 0.f ? 0.f : (v > 255.f ? 255.f : v);
      }
    } else {
      double ss = 0.0;
      for (size_t d = 0; d < dim; d++) {
        o[d] = centres[c * dim + d] + float(r.normal());
        ss += double(o[d]) * double(o[d]);
      }
      const float inv = ss > 0 ? float(1.0 / std::sqrt(ss)) : 0.f;
      for (size_t d = 0; d < dim; d++) o[d] *= inv;
    }
  });
}

// ---- primitives
float orc_l2sq(const float* a, const float* b, size_t n) { return l2sq(a, b, n); }
float orc_dot(const float* a, const float* b, size_t n) { return dot(a, b, n); }
float orc_l2sq_scalar(const float* a, const float* b, size_t n) { return l2sq_scalar(a, b, n); }
float orc_dot_scalar(const float* a, const float* b, size_t n) { return dot_scalar(a, b, n); }
float orc_distance(int metric, const float* a, const float* b, size_t n) { return metric_distance(metric, a, b, n); }
size_t orc_padded(size_t dim) { return padded(dim); }
void orc_normalize(float* data, size_t n, size_t dim) { normalize(data, n, dim); }

// TopK over a stream of (id = position, distance) pushes; returns the count written.
size_t orc_topk(const float* distances, size_t n, size_t k, orc_neighbor* out) {
  TopK t(k);
  for (size_t i = 0; i < n; i++) t.push({uint32_t(i), distances[i]});
  auto r = t.into_sorted();
  for (size_t i = 0; i < r.size(); i++) out[i] = {r[i].id, r[i].distance};
  return r.size();
}

double orc_recall(const orc_neighbor* found, const uint32_t* counts, const uint32_t* truth, size_t truth_stride,
                  size_t nq, size_t k) {  // src/vector/mod.rs:145-152
  size_t hit = 0;
  for (size_t i = 0; i < nq; i++) {
    size_t c = std::min<size_t>(counts[i], k);
    for (size_t j = 0; j < c; j++) {
      uint32_t id = found[i * k + j].id;
      for (size_t t = 0; t < std::min(k, truth_stride); t++)
        if (truth[i * truth_stride + t] == id) {
          hit++;
          break;
        }
    }
  }
  return double(hit) / double(nq * k);
}

// ---- flat
void* orc_flat_new(int metric, size_t dim) {
  auto* f = new Flat();
  f->metric = metric;
  f->dim = dim;
  f->pd = padded(dim);
  return f;
}
void orc_flat_free(void* f) { delete static_cast<Flat*>(f); }
void orc_flat_add(void* f, const float* v, size_t n) { static_cast<Flat*>(f)->add(v, n); }
size_t orc_flat_len(void* f) { return static_cast<Flat*>(f)->len(); }
void orc_flat_search_batch(void* fp, const float* q, size_t nq, size_t k, int threads, orc_neighbor* out,
                           uint32_t* counts) {  // src/vector/flat.rs:56-66
  auto* f = static_cast<Flat*>(fp);
  pool_run(threads, nq, [&](size_t i) {
    auto r = f->search(q + i * f->dim, k);
    write_rows(r, k, reinterpret_cast<Neighbor*>(out), counts, i);
  });
}

// ---- kmeans
void orc_kmeans_assign(const float* data, size_t n, const float* cen, size_t k, size_t dim, int threads,
                       uint32_t* out) {
  auto a = km_assign(threads, data, n, cen, k, dim);
  std::memcpy(out, a.data(), n * 4);
}
int orc_kmeans_train(const float* data, size_t n, size_t dim, size_t k, size_t iters, uint64_t seed, int threads,
                     float* cen_out) {
  if (n < k) return 1;
  auto c = km_train(threads, data, n, dim, k, iters, seed);
  std::memcpy(cen_out, c.data(), c.size() * 4);
  return 0;
}
float orc_kmeans_nearest(const float* x, const float* cen, size_t k, size_t dim, uint32_t* which) {
  auto r = km_nearest(x, cen, k, dim);
  *which = uint32_t(r.first);
  return r.second;
}

// ---- ivfpq
void* orc_ivfpq_train(int metric, size_t dim, const float* sample, size_t n, size_t nlist, size_t m, size_t iters,
                      int keep, uint64_t seed, int threads) {
  return ivfpq_train(threads, metric, dim, sample, n, nlist, m, iters, keep != 0, seed);
}
void orc_ivfpq_free(void* p) { delete static_cast<IvfPq*>(p); }
void orc_ivfpq_add(void* p, const float* v, size_t n, int threads) { static_cast<IvfPq*>(p)->add(threads, v, n); }
size_t orc_ivfpq_len(void* p) { return static_cast<IvfPq*>(p)->count; }
size_t orc_ivfpq_bytes_per_vector(void* p) { return static_cast<IvfPq*>(p)->m + 4; }
int orc_ivfpq_has_tables(void* p) { return static_cast<IvfPq*>(p)->pre.empty() ? 0 : 1; }
// Returns the total number of code rows visited over the batch (algorithmic scan work).
uint64_t orc_ivfpq_search_batch(void* p, const float* q, size_t nq, size_t k, size_t nprobe, size_t refine,
                                int threads, orc_neighbor* out, uint32_t* counts) {  // ivfpq.rs:313-330
  auto* ix = static_cast<IvfPq*>(p);
  std::vector<uint64_t> rows(nq, 0);
  pool_run(threads, nq, [&](size_t i) {
    auto r = ix->search(q + i * ix->dim, k, nprobe, refine, &rows[i]);
    write_rows(r, k, reinterpret_cast<Neighbor*>(out), counts, i);
  });
  uint64_t total = 0;
  for (auto r : rows) total += r;
  return total;
}
size_t orc_ivfpq_save(void* p, uint8_t* buf, size_t cap) { return copy_out(static_cast<IvfPq*>(p)->save(), buf, cap); }
void* orc_ivfpq_load(const uint8_t* bytes, size_t len, char* err, size_t errcap) {
  std::string e;
  auto* ix = ivfpq_load(bytes, len, e);
  if (!ix) set_err(err, errcap, e);
  return ix;
}

// ---- hnsw
void* orc_hnsw_build(int metric, size_t dim, const float* v, size_t n, size_t m, size_t efc, uint64_t seed,
                     int threads) {
  return hnsw_build(threads, metric, dim, v, n, m, efc, seed);
}
void* orc_hnsw_build_batched(int metric, size_t dim, const float* v, size_t n, size_t m, size_t efc, uint64_t seed,
                             size_t max_batch, size_t divisor) {
  return hnsw_build_batched(metric, dim, v, n, m, efc, seed, max_batch, divisor);
}
void orc_hnsw_free(void* p) { delete static_cast<Hnsw*>(p); }
size_t orc_hnsw_len(void* p) { return static_cast<Hnsw*>(p)->len(); }
size_t orc_hnsw_reachable(void* p) { return static_cast<Hnsw*>(p)->reachable(); }
double orc_hnsw_mean_degree(void* p) { return static_cast<Hnsw*>(p)->mean_degree(); }
// work[0] += distance evaluations, work[1] += node expansions (for the gather-traffic estimate).
void orc_hnsw_search_batch(void* p, const float* q, size_t nq, size_t k, size_t ef, int threads, orc_neighbor* out,
                           uint32_t* counts, uint64_t* work) {  // hnsw.rs:353-363
  auto* h = static_cast<Hnsw*>(p);
  std::vector<uint64_t> nd(nq, 0), ne(nq, 0);
  int nt = std::max(threads, 1);
  std::atomic<size_t> next{0};
  pool_run(nt, size_t(nt), [&](size_t) {
    Hnsw::Visited vs;  // the reference keeps one stamp array per thread (hnsw.rs:79-81)
    for (;;) {
      size_t i = next.fetch_add(1, std::memory_order_relaxed);
      if (i >= nq) break;
      auto r = h->search(q + i * h->dim, k, ef, vs, &nd[i], &ne[i]);
      write_rows(r, k, reinterpret_cast<Neighbor*>(out), counts, i);
    }
  });
  if (work) {
    for (size_t i = 0; i < nq; i++) {
      work[0] += nd[i];
      work[1] += ne[i];
    }
  }
}
size_t orc_hnsw_save(void* p, uint8_t* buf, size_t cap) { return copy_out(static_cast<Hnsw*>(p)->save(), buf, cap); }
void* orc_hnsw_load(const uint8_t* bytes, size_t len, char* err, size_t errcap) {
  std::string e;
  auto* h = hnsw_load(bytes, len, e);
  if (!h) set_err(err, errcap, e);
  return h;
}

}  // extern "C"
