"""GPU parity at the shapes the benchmark configurations name (seeded synthetic data stands in for SIFT1M and for
the encoder's embeddings, which cannot be shipped): the CUDA library through its C ABI against the CPU oracle.

  configuration 0: exact L2, 100,000 x 128 clipped integers from 64 clusters, 1,000 queries, in full;
  configuration 1: exact inner product on unit-length 384-d rows from 1,000 clusters, at 100,000 rows;
  configuration 2: IVF-PQ on 1,000,000 x 128, nlist 1024, m 16, trained on a 100,000-row sample,
                   nprobe in {1, 4, 16, 64} x refine in {0, 10}, a 500-query sample against the oracle
                   on the byte-identical index;
  configuration 3: HNSW M 16, efConstruction 200 on a 200,000-node graph built by the oracle,
                   efSearch in {16, 64, 128, 256}.
"""
import numpy as np
import pytest

from tests.parity import assert_same_neighbours

pytestmark = pytest.mark.gpu

L2, IP = 0, 1


@pytest.fixture(scope="module")
def fv():
    import ferrolm_b200

    return ferrolm_b200


@pytest.fixture(scope="module")
def ctx(fv):
    c = fv.Context(0)
    yield c
    c.close()


@pytest.mark.parametrize("mode", [1, 2])
def test_configuration_0_exact_l2(fv, oracle, ctx, mode):
    n, dim, nq, k = 100_000, 128, 1_000, 10
    base = fv.datagen(0, 1, n, dim, 64)
    queries = fv.datagen(0, 2, nq, dim, 64)
    g = fv.FlatIndex(ctx, L2, dim)
    g.add(base)
    g.set_mode(mode)
    o = oracle.FlatIndex(L2, dim)
    o.add(base)
    got, gc = g.search_batch(queries, k)
    want, wc = o.search_batch(queries, k)
    eq, total = assert_same_neighbours(got, gc, want, wc, f"configuration 0, mode {mode}")
    assert eq == total
    assert got.tobytes() == want.tobytes()  # integer distances tie often: the (distance, id) order must hold too
    if mode == 1:
        assert ctx.stats()["uncertified"] == 0  # integers of this range are scored exactly by the tensor cores


def test_configuration_1_shape_inner_product_on_unit_vectors(fv, oracle, ctx):
    n, dim, nq, k = 100_000, 384, 1_000, 10
    base = fv.datagen(1, 1, n, dim, 1000)
    queries = fv.datagen(1, 2, nq, dim, 1000)
    g = fv.FlatIndex(ctx, IP, dim)
    g.add(base)
    g.set_mode(1)
    o = oracle.FlatIndex(IP, dim)
    o.add(base)
    got, gc = g.search_batch(queries, k)
    want, wc = o.search_batch(queries, k)
    eq, total = assert_same_neighbours(got, gc, want, wc, "configuration 1 shape")
    assert eq == total
    # the only regime where the tensor-core scores carry rounding error: the certificate may send a few queries
    # to the full-precision scan, not many
    assert ctx.stats()["uncertified"] <= nq // 100


@pytest.fixture(scope="module")
def configuration_2(fv, oracle, ctx):
    n, dim = 1_000_000, 128
    base = fv.datagen(0, 1, n, dim, 256)
    learn = fv.datagen(0, 3, 100_000, dim, 256)
    queries = fv.datagen(0, 2, 10_000, dim, 256)
    g = fv.IvfPq.train(ctx, L2, dim, learn, fv.IvfPqParams(1024, 16, 20, True, 1))
    g.add(base)
    o = oracle.IvfPq.load(g.save())  # the same index, byte for byte, on the CPU side
    return g, o, queries


@pytest.mark.parametrize("refine", [0, 10])
@pytest.mark.parametrize("nprobe", [1, 4, 16, 64])
def test_configuration_2_ivfpq_sweep(fv, oracle, configuration_2, nprobe, refine):
    g, o, queries = configuration_2
    k, nsub = 10, 500
    # the whole 10,000-query batch on the GPU (so that the list-major scan sees the benchmark's pairs per list);
    # the first 500 queries against the oracle
    got, gc = g.search_batch(queries, k, nprobe, refine)
    rows_gpu = g.ctx.stats()["rows_scanned"]
    want, wc = o.search_batch(queries[:nsub], k, nprobe, refine)
    eq, total = assert_same_neighbours(got[:nsub], gc[:nsub], want, wc, f"configuration 2 nprobe={nprobe} refine={refine}")
    assert eq == total
    # both scans agree on the full batch, rows and all
    g.set_scan_mode(1)
    try:
        got1, gc1 = g.search_batch(queries, k, nprobe, refine)
        assert g.ctx.stats()["rows_scanned"] == rows_gpu
    finally:
        g.set_scan_mode(0)
    assert got1.tobytes() == got.tobytes() and (gc1 == gc).all()


@pytest.fixture(scope="module")
def configuration_3(fv, oracle, ctx):
    n, dim = 200_000, 128
    base = fv.datagen(0, 1, n, dim, 256)
    queries = fv.datagen(0, 2, 2_000, dim, 256)
    o = oracle.Hnsw.build(L2, dim, base, m=16, ef_construction=200, seed=1, threads=oracle.cores())
    g = fv.Hnsw.load(ctx, o.save())
    return g, o, queries


@pytest.mark.parametrize("ef", [16, 64, 128, 256])
def test_configuration_3_hnsw_sweep(fv, oracle, configuration_3, ef):
    g, o, queries = configuration_3
    got, gc = g.search_batch(queries, 10, ef)
    st = g.ctx.stats()
    want, wc, work = o.search_batch(queries, 10, ef, want_work=True)
    assert_same_neighbours(got, gc, want, wc, f"configuration 3 ef={ef}")
    if st["uncertified"] == 0:  # no query ran out of room for tied entries: the traversal is the oracle's, step by step
        assert st["dist_evals"] == int(work[0]) and st["expansions"] == int(work[1])
