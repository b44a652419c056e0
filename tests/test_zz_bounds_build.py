"""The debug build of the library (make -C ferrolm_b200/csrc clean && make EXTRA=-DFV_BOUNDS): its kernels check every
index they gather through against its extent, skip an access that would leave it and report FV_ERR_OVERFLOW.
These tests run ONLY against that build (they hand the library probed cells that name lists which do not exist,
which the normal build is entitled to trust); with the normal build they are skipped."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

FV_ERR_OVERFLOW = 5


@pytest.fixture(scope="module")
def fv():
    import ferrolm_b200
    from ferrolm_b200._lib import lib

    if lib().fv_debug_bounds_build() != 1:
        pytest.skip("normal build: the kernels trust their indices (build with EXTRA=-DFV_BOUNDS to run this)")
    return ferrolm_b200


@pytest.mark.parametrize("mode", [1, 3])
def test_a_probed_cell_beyond_the_lists_is_skipped_and_reported(fv, oracle, mode):
    import torch
    from ferrolm_b200._lib import FerrovecError

    ctx = fv.Context(0)
    dim, n, nq, k, nprobe = 128, 30_000, 300, 10, 8
    base = fv.datagen(0, 1, n, dim, 32)
    queries = fv.datagen(0, 2, nq, dim, 32)
    ix = fv.IvfPq.train(ctx, 0, dim, base[:8000], fv.IvfPqParams(24, 16, 5, True, 1))
    ix.add(base)
    ix.set_scan_mode(mode)
    dq = torch.from_numpy(queries).cuda()
    cells = ix.coarse(dq, nprobe)
    good, gc = ix.search_batch(dq, k, nprobe, 4, cells=cells)
    want, wc = oracle.IvfPq.load(ix.save()).search_batch(queries, k, nprobe, 4)
    assert np.array_equal(fv.neighbors_from_tensor(good)["id"], want["id"])
    bad = cells.clone()
    bad[17, 3] = (bad[17, 3] & ~0xFFFFFFFF) | (24 + 5)  # a list number past the last list, same distance word
    with pytest.raises(FerrovecError) as e:
        ix.search_batch(dq, k, nprobe, 4, cells=bad)
    assert e.value.status == FV_ERR_OVERFLOW and "bounds check" in str(e.value)
    # the violation was skipped, not executed: the context is intact and the next search is the ordinary one
    again, ac = ix.search_batch(dq, k, nprobe, 4, cells=cells)
    assert torch.equal(again, good) and torch.equal(ac, gc)
    ctx.close()
