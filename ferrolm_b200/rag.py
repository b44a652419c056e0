"""The retrieval step of the reference's RAG pipeline over this library (src/rag.rs:153-189).

`Retriever` there owns an encoder, a `FlatIndex` (inner product) over the passage embeddings and optionally
an `Hnsw`; the encoder is out of scope here, so this mirror starts from the embeddings: `search_vectors` and
`search_docs` with the reference's semantics (scores are cosines = negated distances; a document scores as its
best passage; `k * min(per_doc, 8)` passages are fetched before de-duplication).
"""
from __future__ import annotations

import numpy as np

from .vector import Context, FlatIndex, Hnsw, HnswParams, Metric


class Retriever:
    def __init__(self, ctx: Context, passage_vectors, passage_doc, hnsw: HnswParams | None = None, ef: int = 64,
                 build_threads: int = 0):
        """passage_vectors: (n, dim) unit-length embeddings; passage_doc[i]: the document of passage i
        (non-decreasing, as rag.rs:98-104 builds it)."""
        v = np.ascontiguousarray(passage_vectors, dtype=np.float32)
        self.dim = v.shape[1]
        self.passage_doc = np.asarray(passage_doc, dtype=np.uint32)
        self.flat = FlatIndex(ctx, Metric.InnerProduct, self.dim)      # rag.rs:111-112
        self.flat.add(v)
        # the graph is built on the GPU (deterministic batches) unless host threads are asked for
        self.hnsw = None
        if hnsw:
            self.hnsw = (Hnsw.build(ctx, Metric.InnerProduct, self.dim, v, hnsw, threads=build_threads) if build_threads
                         else Hnsw.build_batched(ctx, Metric.InnerProduct, self.dim, v, hnsw))
        self.ef = ef

    def set_ef(self, ef: int):                                          # rag.rs:145-149
        self.ef = ef

    def docs(self) -> int:                                              # rag.rs:191-193
        return int(self.passage_doc[-1]) + 1 if len(self.passage_doc) else 0

    def search_vectors(self, q, k: int, exact: bool = False):          # rag.rs:153-162
        """Per query a list of (passage, cosine), nearest first."""
        if self.hnsw is not None and not exact:
            out, counts = self.hnsw.search_batch(q, k, max(self.ef, k))
        else:
            out, counts = self.flat.search_batch(q, k)
        return [[(int(n["id"]), -float(n["distance"])) for n in row[:c]] for row, c in zip(out, counts)]

    def search_docs(self, q, k: int, exact: bool = False):             # rag.rs:172-189
        per_doc = max(1, -(-len(self.passage_doc) // max(self.docs(), 1)))
        res = []
        for hits in self.search_vectors(q, k * min(per_doc, 8), exact):
            seen, out = set(), []
            for p, s in hits:
                d = int(self.passage_doc[p])
                if d not in seen:
                    seen.add(d)
                    out.append((d, s))
            res.append(out[:k])
        return res
