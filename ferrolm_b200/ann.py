"""`python -m ferrolm_b200.ann` — the reference's `ferrolm ann` benchmark driver (src/main.rs:445-569) on the GPU.

Same flags and the same JSONL row per setting
({"engine","index","param","recall10","qps_1","qps_n","threads","build_s","n"}), so a SIFT1M run can be laid
beside bench/results/ann.jsonl of the reference.  `qps_n` is the batched search of all queries on one GPU;
`qps_1` (one CPU thread in the reference) is the same search issued one query at a time.
Without --base the seeded synthetic stand-in of the benchmark is generated (--n rows, 128 dimensions).
"""
from __future__ import annotations

import argparse
import json
import time

import numpy as np


def main(argv=None):
    ap = argparse.ArgumentParser(prog="ferrolm_b200.ann")
    ap.add_argument("--index", default="hnsw", choices=["hnsw", "ivfpq", "flat"])
    ap.add_argument("--base")
    ap.add_argument("--query")
    ap.add_argument("--truth")
    ap.add_argument("--learn")
    ap.add_argument("--n", type=int)
    ap.add_argument("--queries", type=int, default=10_000)
    ap.add_argument("--threads", type=int, default=0, help="host threads for the HNSW build (with --host-build)")
    ap.add_argument("--host-build", action="store_true",
                    help="build the HNSW graph on the host threads as the reference does (default: on the GPU, in batches)")
    ap.add_argument("--m", type=int, default=16)
    ap.add_argument("--ef-construction", type=int, default=200)
    ap.add_argument("--ef", default="16,32,64,128,256")
    ap.add_argument("--nlist", type=int, default=1024)
    ap.add_argument("--pq-m", type=int, default=16)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--nprobe", default="1,4,16,64")
    ap.add_argument("--refine", default="0,10")
    ap.add_argument("--single-thread-queries", type=int, default=2000)
    ap.add_argument("--label", default="ferrolm_b200")
    ap.add_argument("--json")
    ap.add_argument("--device", type=int, default=0)
    a = ap.parse_args(argv)

    import os

    import ferrolm_b200 as fv
    from ferrolm_b200.io import read_fvecs, read_ivecs

    ctx = fv.Context(a.device)
    if a.base:
        base = read_fvecs(a.base, a.n)
        queries = read_fvecs(a.query, a.queries)
        learn = read_fvecs(a.learn) if a.learn else base[:100_000]
    else:
        n = a.n or 1_000_000
        base = fv.datagen(0, 1, n, 128, 256)
        queries = fv.datagen(0, 2, a.queries, 128, 256)
        learn = fv.datagen(0, 3, min(100_000, n), 128, 256)
    dim, nq = base.shape[1], queries.shape[0]
    if a.truth:
        truth = read_ivecs(a.truth, nq)
    else:  # exact search of this library (checked against the CPU oracle by the test suite)
        flat = fv.FlatIndex(ctx, fv.Metric.L2, dim)
        flat.add(base)
        truth = flat.search_batch(queries, 10)[0]["id"]
        flat.close()
    threads = a.threads or (os.cpu_count() or 1)
    sub = min(nq, a.single_thread_queries)

    def timed(search):
        search(queries[:64])  # warm-up
        t = time.perf_counter()
        out, counts = search(queries)
        qpsn = nq / (time.perf_counter() - t)
        t = time.perf_counter()
        for i in range(sub):
            search(queries[i:i + 1])
        qps1 = sub / (time.perf_counter() - t)
        return fv.recall(out, counts, truth, 10), qps1, qpsn

    def emit(index, param, r, q1, qn, build):
        print(f"{a.label} {index} {param}: recall@10 {r:.4f}  {q1:.0f} QPS (one query per call)  {qn:.0f} QPS (batched)  "
              f"build {build:.0f} s")
        if a.json:
            with open(a.json, "a") as f:
                f.write(json.dumps({"engine": a.label, "index": index, "param": param, "recall10": round(r, 5),
                                    "qps_1": round(q1, 1), "qps_n": round(qn, 1), "threads": threads,
                                    "build_s": round(build, 1), "n": int(base.shape[0])}) + "\n")

    lst = lambda s: [int(x) for x in str(s).split(",")]
    if a.index == "hnsw":
        t = time.perf_counter()
        hp = fv.HnswParams(a.m, a.ef_construction, 1)
        h = (fv.Hnsw.build(ctx, fv.Metric.L2, dim, base, hp, threads=threads) if a.host_build
             else fv.Hnsw.build_batched(ctx, fv.Metric.L2, dim, base, hp))
        build = time.perf_counter() - t
        print(f"HNSW over {len(h)} vectors built in {build:.0f} s, mean degree {h.mean_degree():.1f}")
        for ef in lst(a.ef):
            r, q1, qn = timed(lambda q: h.search_batch(q, 10, ef))
            emit("hnsw", f"M={a.m} efC={a.ef_construction} ef={ef}", r, q1, qn, build)
    elif a.index == "ivfpq":
        t = time.perf_counter()
        ix = fv.IvfPq.train(ctx, fv.Metric.L2, dim, learn, fv.IvfPqParams(a.nlist, a.pq_m, a.iters, True, 1))
        ix.add(base)
        build = time.perf_counter() - t
        print(f"IVF-PQ over {len(ix)} vectors built in {build:.0f} s, {ix.bytes_per_vector()} bytes per vector")
        for refine in lst(a.refine):
            for nprobe in lst(a.nprobe):
                r, q1, qn = timed(lambda q: ix.search_batch(q, 10, nprobe, refine))
                emit("ivfpq", f"nlist={a.nlist} m={a.pq_m} nprobe={nprobe} refine={refine}", r, q1, qn, build)
    else:
        t = time.perf_counter()
        flat = fv.FlatIndex(ctx, fv.Metric.L2, dim)
        flat.add(base)
        build = time.perf_counter() - t
        r, q1, qn = timed(lambda q: flat.search_batch(q, 10))
        emit("flat", "exact", r, q1, qn, build)


if __name__ == "__main__":
    main()
