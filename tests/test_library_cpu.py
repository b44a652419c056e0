"""Checks that need no GPU: the shared library loads, exports every symbol the header
declares, its host-side helpers agree with the oracle, and it refuses to work without a GPU."""
import ctypes as C
import os
import re

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def fv():
    import __graft_entry__ as g

    g.build()
    import ferrolm_b200

    return ferrolm_b200


def test_every_declared_symbol_is_exported(fv):
    from ferrolm_b200 import _lib

    header = open(os.path.join(ROOT, "include", "ferrovec.h")).read()
    header = re.sub(r"/\*.*?\*/", "", header, flags=re.S)  # declarations only, not the comments
    declared = set(re.findall(r"\b(fv_[a-z0-9_]+)\s*\(", header))
    assert declared, "no declarations found"
    L = C.CDLL(_lib.SO_PATH)
    missing = [n for n in sorted(declared) if not hasattr(L, n)]
    assert not missing, missing
    assert declared == set(_lib.SIGNATURES), declared ^ set(_lib.SIGNATURES)
    assert b"sm_100a" in _lib.lib().fv_version()


def test_host_helpers_match_the_oracle(fv, oracle):
    assert [fv.padded(d) for d in (1, 8, 40, 127, 128, 384)] == [8, 8, 40, 128, 128, 384]
    x = oracle.testdata(64, 24, 5)
    assert fv.normalize(x).tobytes() == oracle.normalize(x).tobytes()
    found = np.zeros((2, 3), dtype=fv.NEIGHBOR)
    found["id"] = [[1, 2, 3], [7, 8, 9]]
    truth = np.array([[3, 2, 0, 99], [1, 1, 7, 99]], dtype=np.uint32)
    counts = np.array([3, 3], dtype=np.uint32)
    assert fv.recall(found, counts, truth, 3) == pytest.approx(3 / 6)
    assert fv.recall(found, counts, truth, 3) == oracle.recall(found, counts, truth, 3)


def test_datagen_is_seeded_and_row_addressable(fv):
    a = fv.datagen(0, 1, 1000, 32, 16)
    b = fv.datagen(0, 1, 1000, 32, 16, threads=3)
    assert a.tobytes() == b.tobytes()
    c = fv.datagen(0, 1, 100, 32, 16, first_row=500)
    assert c.tobytes() == a[500:600].tobytes()
    assert a.min() >= 0 and a.max() <= 255 and (a == np.round(a)).all()
    assert fv.datagen(0, 2, 10, 32, 16).tobytes() != a[:10].tobytes()
    e = fv.datagen(1, 1, 100, 48, 7)
    assert np.allclose(np.linalg.norm(e, axis=1), 1.0, atol=1e-5)


def test_the_oracle_generates_the_same_benchmark_rows(fv, oracle):
    # the CPU arm of the benchmark generates its data without loading the product library: same bytes
    for kind, dim, clusters in [(0, 128, 256), (1, 384, 1000), (0, 24, 7)]:
        a = fv.datagen(kind, 5, 3000, dim, clusters, first_row=123)
        b = oracle.datagen(kind, 5, 3000, dim, clusters, first_row=123)
        assert a.tobytes() == b.tobytes()


def test_no_gpu_means_a_loud_failure(fv):
    import torch

    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    with pytest.raises(fv.FerrovecError, match="no CPU path|CUDA"):
        fv.Context(0)
