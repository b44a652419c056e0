"""Shared checks of the parity contract: identical neighbour ids except at exact distance
ties, distances within 1e-4 relative (they are expected to be bit-equal), equal counts."""
import numpy as np

REL_TOL = 1e-4  # the stated tolerance for distances


def assert_same_neighbours(got, got_counts, want, want_counts, what=""):
    got_counts = np.asarray(got_counts).astype(np.int64)
    want_counts = np.asarray(want_counts).astype(np.int64)
    assert (got_counts == want_counts).all(), f"{what}: result counts differ"
    nq, k = want.shape
    bit_equal = 0
    total = 0
    for i in range(nq):
        c = int(want_counts[i])
        g, w = got[i, :c], want[i, :c]
        gd, wd = g["distance"], w["distance"]
        scale = np.maximum(np.abs(wd), 1e-30)
        assert (np.abs(gd - wd) <= REL_TOL * scale).all(), f"{what}: query {i} distances differ: {gd} vs {wd}"
        bit_equal += int((gd.view(np.uint32) == wd.view(np.uint32)).sum())
        total += c
        diff = np.nonzero(g["id"] != w["id"])[0]
        for j in diff:
            # a differing id is acceptable only inside a run of exactly equal distances
            d = wd[j]
            assert gd[j] == d, f"{what}: query {i} rank {j}: id {g['id'][j]} vs {w['id'][j]} without a tie"
            tied_w = set(w["id"][wd == d].tolist())
            tied_g = set(g["id"][gd == d].tolist())
            at_cut = (j == c - 1) or wd[c - 1] == d
            assert tied_w == tied_g or at_cut, f"{what}: query {i}: different ids inside a tie that is not at the cut"
    return bit_equal, total
