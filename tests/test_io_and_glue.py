"""`.fvecs/.ivecs` readers (src/vector/io.rs:7-42) and the retrieval glue (src/rag.rs:153-189)."""
import numpy as np
import pytest


def write_vecs(path, rows, dtype):
    with open(path, "wb") as f:
        for r in rows:
            f.write(np.int32(len(r)).tobytes())
            f.write(np.asarray(r, dtype=dtype).tobytes())


def test_fvecs_and_ivecs_readers(tmp_path):
    from ferrolm_b200 import FerrovecError
    from ferrolm_b200.io import read_fvecs, read_ivecs

    rng = np.random.default_rng(0)
    v = rng.standard_normal((7, 5)).astype(np.float32)
    write_vecs(tmp_path / "a.fvecs", v, "<f4")
    assert read_fvecs(tmp_path / "a.fvecs").tobytes() == v.tobytes()
    assert read_fvecs(tmp_path / "a.fvecs", 3).tobytes() == v[:3].tobytes()       # row limit (io.rs:17)
    ids = rng.integers(0, 1 << 31, (4, 10)).astype(np.uint32)
    write_vecs(tmp_path / "t.ivecs", ids, "<u4")
    assert (read_ivecs(tmp_path / "t.ivecs") == ids).all()
    (tmp_path / "empty").write_bytes(b"")
    with pytest.raises(FerrovecError, match="empty"):
        read_fvecs(tmp_path / "empty")
    (tmp_path / "odd").write_bytes(np.int32(3).tobytes() + b"\x00" * 13)
    with pytest.raises(FerrovecError, match="not a vecs file of dimension 3"):
        read_fvecs(tmp_path / "odd")
    write_vecs(tmp_path / "mixed", [[1.0, 2.0, 3.0, 4.0, 5.0]], "<f4")
    with open(tmp_path / "mixed", "ab") as f:      # second record claims 2 dims but the size still divides
        f.write(np.int32(2).tobytes() + b"\x00" * 20)
    with pytest.raises(FerrovecError, match="record 1 has a different dimension"):
        read_fvecs(tmp_path / "mixed")
    with pytest.raises(FerrovecError, match="cannot open"):
        read_fvecs(tmp_path / "missing")


@pytest.mark.gpu
def test_retriever_glue_matches_the_reference_semantics(oracle):
    import ferrolm_b200 as fv
    from ferrolm_b200.rag import Retriever

    ctx = fv.Context(0)
    dim, n_docs = 48, 400
    rng = np.random.default_rng(1)
    per = rng.integers(1, 5, n_docs)                         # passages per document
    passage_doc = np.repeat(np.arange(n_docs), per).astype(np.uint32)
    vecs = oracle.normalize(oracle.testdata(len(passage_doc), dim, 5))
    q = oracle.normalize(oracle.testdata(20, dim, 6))
    r = Retriever(ctx, vecs, passage_doc)
    hits = r.search_vectors(q, 5)
    o = oracle.FlatIndex(oracle.INNER_PRODUCT, dim)
    o.add(vecs)
    want, _ = o.search_batch(q, 5)
    for i in range(len(q)):
        assert [h[0] for h in hits[i]] == [int(x) for x in want[i]["id"]]
        assert [h[1] for h in hits[i]] == [-float(x) for x in want[i]["distance"]]   # cosine = -distance (rag.rs:160)
    docs = r.search_docs(q, 3)
    per_doc = -(-len(passage_doc) // n_docs)
    wide, _ = o.search_batch(q, 3 * min(per_doc, 8))
    for i in range(len(q)):
        seen, exp = set(), []
        for nb in wide[i]:
            d = int(passage_doc[nb["id"]])
            if d not in seen:
                seen.add(d)
                exp.append(d)
        assert [d for d, _ in docs[i]] == exp[:3]
    # with a graph index the same call goes through Hnsw::search_batch with max(ef, k) (rag.rs:155)
    rh = Retriever(ctx, vecs, passage_doc, hnsw=fv.HnswParams(8, 60, 1), ef=64)
    got = rh.search_vectors(q, 5)
    overlap = np.mean([len({h[0] for h in got[i]} & {h[0] for h in hits[i]}) / 5 for i in range(len(q))])
    assert overlap >= 0.95
    assert rh.search_vectors(q, 5, exact=True) == hits


@pytest.mark.gpu
def test_ann_driver_writes_the_reference_jsonl_schema(tmp_path):
    import json

    from ferrolm_b200 import ann

    out = tmp_path / "ann.jsonl"
    ann.main(["--index", "ivfpq", "--n", "20000", "--queries", "200", "--nlist", "64", "--iters", "3", "--nprobe", "4",
              "--refine", "0,4", "--single-thread-queries", "20", "--json", str(out)])
    rows = [json.loads(l) for l in open(out)]
    assert len(rows) == 2
    assert set(rows[0]) == {"engine", "index", "param", "recall10", "qps_1", "qps_n", "threads", "build_s", "n"}
    assert rows[0]["index"] == "ivfpq" and rows[0]["n"] == 20000 and rows[1]["recall10"] >= rows[0]["recall10"]
