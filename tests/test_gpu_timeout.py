"""The give-up path of the bounded waits inside the tensor-core kernel, exercised without any fault on the device:
a test hook arms the next launch with a short wait limit and makes one producer leave out one stage's loads, so the
consumer of that stage waits on a barrier nothing completes.  The kernel must give up (error word, tensor memory
freed, normal return), the search must fail with FV_ERR_TIMEOUT, and the context must stay usable."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

FV_ERR_TIMEOUT = 4
LIMIT_CYCLES = 20_000_000  # about 10 ms


@pytest.fixture(scope="module")
def fv():
    import ferrolm_b200

    return ferrolm_b200


def arm(skip_unit=0):
    from ferrolm_b200._lib import check, lib

    check(lib().fv_debug_tc_fault(LIMIT_CYCLES, skip_unit))


def test_exact_search_times_out_and_recovers(fv, oracle):
    from ferrolm_b200._lib import FerrovecError

    ctx = fv.Context(0)
    dim, n, nq, k = 128, 30_000, 300, 10
    base = fv.datagen(0, 1, n, dim, 32)
    queries = fv.datagen(0, 2, nq, dim, 32)
    ix = fv.FlatIndex(ctx, 0, dim)
    ix.add(base)
    ix.set_mode(1)  # the tensor-core front end
    o = oracle.FlatIndex(0, dim)
    o.add(base)
    want, wc = o.search_batch(queries, k)
    got, gc = ix.search_batch(queries, k)
    assert got.tobytes() == want.tobytes()
    arm()
    with pytest.raises(FerrovecError) as e:
        ix.search_batch(queries, k)
    assert e.value.status == FV_ERR_TIMEOUT
    # the hook disarmed itself with that launch; same context, same index: the ordinary result
    again, ac = ix.search_batch(queries, k)
    assert again.tobytes() == want.tobytes() and (ac == wc).all()
    ctx.close()


def test_ivfpq_tensor_pass_times_out_and_recovers(fv, oracle):
    from ferrolm_b200._lib import FerrovecError

    ctx = fv.Context(0)
    dim, n, nq, k = 128, 40_000, 700, 10
    base = fv.datagen(0, 1, n, dim, 32)
    queries = fv.datagen(0, 2, nq, dim, 32)
    ix = fv.IvfPq.train(ctx, 0, dim, base[:12_000], fv.IvfPqParams(24, 16, 6, True, 1))
    ix.add(base)
    ix.set_scan_mode(3)
    want, wc = oracle.IvfPq.load(ix.save()).search_batch(queries, k, 16, 10)
    got, gc = ix.search_batch(queries, k, 16, 10)  # also builds what the tensor-core pass needs
    assert np.array_equal(got["id"], want["id"])
    arm()
    with pytest.raises(FerrovecError) as e:
        ix.search_batch(queries, k, 16, 10)
    assert e.value.status == FV_ERR_TIMEOUT
    again, ac = ix.search_batch(queries, k, 16, 10)
    assert again.tobytes() == got.tobytes() and (ac == gc).all()
    ctx.close()
