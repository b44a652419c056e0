"""The reference's own tests for the vector path, run against the CPU oracle.

Each case restates one test of the reference so that the oracle is pinned to
every known answer and property threshold the reference holds for this path:
src/vector/mod.rs:158-171, src/vector/kmeans.rs:96-112, tests/vector.rs:35-125.
"""
import numpy as np
import pytest

L2, IP = 0, 1


def truth(o, metric, dim, base, queries, k):
    flat = o.FlatIndex(metric, dim)
    flat.add(base)
    out, counts = flat.search_batch(queries, k)
    assert (counts == k).all()
    return out["id"].copy()


def test_topk_keeps_the_nearest_in_order(oracle):
    # src/vector/mod.rs:158-171 -- the only literal known answers of the path
    r = oracle.topk([5.0, 1.0, 4.0, 3.0, 2.0, 9.0], 3)
    assert list(r["id"]) == [1, 4, 3]
    assert oracle.distance(L2, np.zeros(8), np.ones(8)) == 8.0
    assert oracle.distance(IP, np.ones(8), np.full(8, 2.0)) == -16.0


def test_avx2_and_scalar_paths_agree_bit_for_bit(oracle):
    # src/kernels.rs:200-231: the portable path runs the same chains as the AVX2 one
    import ctypes as C

    assert oracle.lib().orc_has_avx2() == 1
    rng = np.random.default_rng(0)
    for n in (8, 40, 128, 384):
        for _ in range(50):
            a = rng.standard_normal(n).astype(np.float32) * 100
            b = rng.standard_normal(n).astype(np.float32) * 100
            pa, pb = a.ctypes.data_as(C.c_void_p), b.ctypes.data_as(C.c_void_p)
            L = oracle.lib()
            assert L.orc_l2sq(pa, pb, n) == L.orc_l2sq_scalar(pa, pb, n)
            assert L.orc_dot(pa, pb, n) == L.orc_dot_scalar(pa, pb, n)


def test_rng_matches_its_definition(oracle):
    # src/rng.rs:10-20 restated in Python integers
    mask = (1 << 64) - 1
    s = (7 * 0x9E3779B97F4A7C15 & mask) | 1
    r = oracle.Rng(7)
    for _ in range(20):
        s ^= s >> 12
        s ^= (s << 25) & mask
        s ^= s >> 27
        assert r.next_u64() == (s * 0x2545F4914F6CDD1D) & mask
    u = oracle.Rng(3).uniform()
    assert 0.0 <= u < 1.0


def test_total_order_of_neighbours(oracle):
    # src/vector/mod.rs:60-64: total_cmp then id; -0.0 sorts before +0.0
    r = oracle.topk([0.0, -0.0, 1.0, 1.0, float("inf")], 5)
    assert list(r["id"]) == [1, 0, 2, 3, 4]


def test_kmeans_finds_well_separated_clusters(oracle):
    # src/vector/kmeans.rs:96-112
    rng = oracle.Rng(3)
    centers = np.array([[0.0] * 8, [10.0] * 8, [-10.0] * 8], dtype=np.float32)
    data = np.empty((600, 8), dtype=np.float32)
    for i in range(600):
        for d in range(8):
            data[i, d] = np.float32(centers[i % 3, d]) + np.float32(rng.normal()) * np.float32(0.1)
    cen = oracle.kmeans_train(data, 3, 10, 1, threads=2)
    for c in centers:
        _, d = oracle.kmeans_nearest(c, cen)
        assert d < 0.1


def test_kmeans_is_independent_of_thread_count(oracle):
    data = oracle.testdata(3000, 16, 5)
    a = oracle.kmeans_train(data, 32, 5, 1, threads=1)
    b = oracle.kmeans_train(data, 32, 5, 1, threads=4)
    assert a.tobytes() == b.tobytes()


@pytest.mark.parametrize("metric,dim", [(L2, 40), (IP, 64)])
def test_hnsw_finds_the_nearest_neighbours_and_round_trips(oracle, metric, dim):
    # tests/vector.rs:35-69
    base = oracle.testdata(20_000, dim, 1)
    queries = oracle.testdata(200, dim, 2)
    if metric == IP:
        base, queries = oracle.normalize(base), oracle.normalize(queries)
    t = truth(oracle, metric, dim, base, queries, 10)
    h = oracle.Hnsw.build(metric, dim, base, m=16, ef_construction=100, seed=1, threads=4)
    assert h.mean_degree() > 8.0
    lo, c_lo = h.search_batch(queries, 10, 16)
    hi, c_hi = h.search_batch(queries, 10, 128)
    r_low, r_high = oracle.recall(lo, c_lo, t, 10), oracle.recall(hi, c_hi, t, 10)
    assert r_high >= 0.98
    assert r_high >= r_low
    loaded = oracle.Hnsw.load(h.save())
    a, ca = loaded.search_batch(queries, 10, 64)
    b, cb = h.search_batch(queries, 10, 64)
    assert a.tobytes() == b.tobytes() and (ca == cb).all()
    assert loaded.save() == h.save()


def test_ivfpq_recall_grows_with_probes_and_reranking(oracle):
    # tests/vector.rs:71-98
    dim = 32
    base = oracle.testdata(20_000, dim, 3)
    queries = oracle.testdata(200, dim, 4)
    t = truth(oracle, L2, dim, base, queries, 10)
    ix = oracle.IvfPq.train(L2, dim, base[:10_000], nlist=64, m=8, iters=10, keep_vectors=True, seed=1, threads=4)
    ix.add(base, threads=4)
    assert len(ix) == 20_000
    assert ix.bytes_per_vector() == 12

    def rec(nprobe, refine):
        out, counts = ix.search_batch(queries, 10, nprobe, refine)
        return oracle.recall(out, counts, t, 10)

    r1, r16, r16r = rec(1, 0), rec(16, 0), rec(16, 10)
    assert r16 > r1 and r16r > r16 and r16r > 0.9, (r1, r16, r16r)
    loaded = oracle.IvfPq.load(ix.save())
    a, ca = loaded.search_batch(queries, 10, 8, 5)
    b, cb = ix.search_batch(queries, 10, 8, 5)
    assert a.tobytes() == b.tobytes() and (ca == cb).all()
    assert loaded.save() == ix.save()


def test_ivfpq_build_is_independent_of_thread_count(oracle):
    dim = 16
    base = oracle.testdata(4000, dim, 9)
    a = oracle.IvfPq.train(L2, dim, base[:2000], 16, 4, 4, True, 1, threads=1)
    a.add(base, threads=1)
    b = oracle.IvfPq.train(L2, dim, base[:2000], 16, 4, 4, True, 1, threads=4)
    b.add(base, threads=4)
    assert a.save() == b.save()


def test_parallel_hnsw_build_keeps_the_graph_connected(oracle):
    # tests/vector.rs:104-125
    n, nq, dim = 5000, 200, 384
    rng = oracle.Rng(7)
    common = np.array([np.float32(rng.normal()) * np.float32(3.0) for _ in range(dim)], dtype=np.float32)

    def sample(count):
        v = oracle.testdata(count, dim, rng.next_u64())
        v = (v / np.float32(3.0) + common).astype(np.float32)
        return oracle.normalize(v)

    base, queries = sample(n), sample(nq)
    t = truth(oracle, IP, dim, base, queries, 10)
    h = oracle.Hnsw.build(IP, dim, base, threads=4)
    assert h.reachable() >= n - 2
    out, counts = h.search_batch(queries, 10, 256)
    assert oracle.recall(out, counts, t, 10) >= 0.999


def test_batched_hnsw_build_with_batches_of_one_is_the_single_thread_build(oracle):
    # the batch-synchronous order the GPU construction runs (and is compared with, byte for byte, in the GPU tests) is
    # pinned to the reference's own order where the two must coincide: one node per batch
    dim = 24
    base = oracle.testdata(2500, dim, 5)
    for metric in (oracle.L2, oracle.INNER_PRODUCT):
        v = oracle.normalize(base) if metric == oracle.INNER_PRODUCT else base
        seq = oracle.Hnsw.build(metric, dim, v, m=8, ef_construction=40, seed=3, threads=1)
        one = oracle.Hnsw.build_batched(metric, dim, v, m=8, ef_construction=40, seed=3, max_batch=1, divisor=1)
        assert one.save() == seq.save()
        wide = oracle.Hnsw.build_batched(metric, dim, v, m=8, ef_construction=40, seed=3, max_batch=256, divisor=8)
        again = oracle.Hnsw.build_batched(metric, dim, v, m=8, ef_construction=40, seed=3, max_batch=256, divisor=8)
        assert wide.save() == again.save() and wide.save() != seq.save()
        assert abs(wide.reachable() - seq.reachable()) <= 25 and abs(wide.mean_degree() - seq.mean_degree()) < 0.5


def test_index_files_reject_damage(oracle):
    # src/vector/io.rs:82, hnsw.rs:425-452, ivfpq.rs:355-357
    base = oracle.testdata(300, 8, 1)
    h = oracle.Hnsw.build(L2, 8, base, m=4, ef_construction=20)
    blob = h.save()
    with pytest.raises(ValueError, match="not an HNSW"):
        oracle.Hnsw.load(b"XXXXXXXX" + blob[8:])
    with pytest.raises(ValueError, match="truncated"):
        oracle.Hnsw.load(blob[: len(blob) // 2])
    ix = oracle.IvfPq.train(L2, 8, base, 4, 2, 2, False, 1)
    ix.add(base)
    blob = ix.save()
    with pytest.raises(ValueError, match="not an IVF-PQ"):
        oracle.IvfPq.load(blob[1:])
    with pytest.raises(ValueError, match="truncated"):
        oracle.IvfPq.load(blob[:-3])
