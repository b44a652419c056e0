"""The multi-rank host logic on CPU: two gloo ranks, each searching its shard with the CPU oracle, exchange
their candidate lists with the library's gather helper; the merged result must equal the unsharded search.
(The merge kernels themselves are covered on the GPU in test_gpu_parity.py.)"""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _merge(parts, counts, k):
    """(world, nq, kin) structured parts -> k best by (distance, id) per query."""
    world, nq, kin = parts.shape
    out = []
    for q in range(nq):
        cand = [(float(parts[w, q, i]["distance"]), int(parts[w, q, i]["id"])) for w in range(world)
                for i in range(int(counts[w, q]))]
        cand.sort()
        out.append(cand[:k])
    return out


def _worker(rank, world, port, tmp):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from ferrolm_b200.sharding import all_gather_stacked, row_range
    from oracle import oracle as o

    dim, n, nq, k = 24, 3001, 37, 10   # an odd row count: the last shard is shorter
    base, queries = o.testdata(n, dim, 1), o.testdata(nq, dim, 2)
    lo, hi = row_range(rank, world, n)
    # ---- exact search, contiguous row shards
    flat = o.FlatIndex(o.L2, dim)
    flat.add(base[lo:hi])
    out, counts = flat.search_batch(queries, k, threads=1)
    out["id"] += np.uint32(lo)
    parts = all_gather_stacked(torch.from_numpy(out.view(np.int32).reshape(nq, k, 2)), world).numpy()
    parts = np.ascontiguousarray(parts).view(o.NEIGHBOR).reshape(world, nq, k)
    cnts = all_gather_stacked(torch.from_numpy(counts.astype(np.int32)), world).numpy()
    merged = _merge(parts, cnts, k)
    whole = o.FlatIndex(o.L2, dim)
    whole.add(base)
    want, _ = whole.search_batch(queries, k, threads=1)
    for q in range(nq):
        assert [m[1] for m in merged[q]] == [int(x) for x in want[q]["id"]], (rank, q)
    # ---- IVF-PQ with re-ranking: global cut by compressed distance, then by exact distance
    refine, nprobe = 4, 6
    full = o.IvfPq.train(o.L2, dim, base[:1500], 16, 6, 4, True, 1, threads=1)
    blob = full.save()
    full.add(base, threads=1)
    want, wc = full.search_batch(queries, k, nprobe, refine, threads=1)
    shard = o.IvfPq.load(blob)
    shard.add(base[lo:hi], threads=1)
    adc, ac = shard.search_batch(queries, k * refine, nprobe, 0, threads=1)   # best keep by compressed distance
    exact = np.full((nq, k * refine), np.inf, dtype=np.float32)
    for q in range(nq):
        for i in range(int(ac[q])):
            exact[q, i] = o.distance(o.L2, queries[q], base[lo + int(adc[q, i]["id"])])
    adc["id"] += np.uint32(lo)
    g_adc = all_gather_stacked(torch.from_numpy(adc.view(np.int32).reshape(nq, k * refine, 2)), world).numpy()
    g_adc = np.ascontiguousarray(g_adc).view(o.NEIGHBOR).reshape(world, nq, k * refine)
    g_ex = all_gather_stacked(torch.from_numpy(exact), world).numpy()
    g_cnt = all_gather_stacked(torch.from_numpy(ac.astype(np.int32)), world).numpy()
    for q in range(nq):
        cand = [(float(g_adc[w, q, i]["distance"]), int(g_adc[w, q, i]["id"]), float(g_ex[w, q, i]))
                for w in range(world) for i in range(int(g_cnt[w, q]))]
        cand.sort()
        kept = sorted((c[2], c[1]) for c in cand[: k * refine])[:k]
        assert [c[1] for c in kept] == [int(x) for x in want[q]["id"][: int(wc[q])]], (rank, q)
    # ---- work split by query slices (the coarse step of list shards): same rows as the unsplit computation,
    # also when the query count does not divide by the world size
    from ferrolm_b200.sharding import per_query_slices

    calls = []

    def keys(part):
        calls.append(part.shape[0])
        return (part[:, :5] * 1000.0).to(torch.int64)

    tq = torch.from_numpy(queries)
    got = per_query_slices(keys, tq, world)
    assert torch.equal(got, (tq[:, :5] * 1000.0).to(torch.int64))
    assert calls == [row_range(rank, world, nq)[1] - row_range(rank, world, nq)[0]] and sum(calls) < nq
    dist.barrier()
    dist.destroy_process_group()
    open(os.path.join(tmp, f"ok{rank}"), "w").write("ok")


def test_two_rank_sharded_search_on_gloo(tmp_path, oracle):
    import socket

    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    assert os.path.exists(tmp_path / "ok0") and os.path.exists(tmp_path / "ok1")


def test_row_ranges_cover_everything():
    from ferrolm_b200.sharding import row_range

    for n in (0, 1, 7, 1000, 1_000_003):
        for world in (1, 2, 3, 8):
            spans = [row_range(r, world, n) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
