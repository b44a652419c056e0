"""Sharded search through the library's collective entry points on two GPUs (skipped on a box with one):
every rank holds a shard and a context of one group; the exchange (NCCL) and the merge happen inside the C ABI
call.  The merged result must be byte-equal to the search over the unsharded index."""
import os
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, tmp):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    import torch
    import torch.distributed as dist

    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    import ferrolm_b200 as fv
    from ferrolm_b200.sharding import ShardedSearch, init_group, row_range

    ctx = fv.Context(rank)
    init_group(ctx, rank, world)
    assert ctx.comm_size == world and ctx.comm_rank == rank
    dim, n, nq, k = 128, 60_000, 1_000, 10
    base = fv.datagen(0, 1, n, dim, 48)
    queries = fv.datagen(0, 2, nq, dim, 48)
    dq = torch.from_numpy(queries).cuda()
    # ---- exact search over contiguous row ranges
    lo, hi = row_range(rank, world, n)
    shard = fv.FlatIndex(ctx, fv.Metric.L2, dim)
    shard.set_id_base(lo)
    shard.add(base[lo:hi])
    got, gc = ShardedSearch(ctx, shard, "flat", world).search_batch(dq, k)
    whole = fv.FlatIndex(ctx, fv.Metric.L2, dim)
    whole.add(base)
    want, wc = whole.search_batch(dq, k)
    assert torch.equal(got, want) and torch.equal(gc, wc), "exact search over row shards"
    # ---- IVF-PQ over list shards, every scan, with and without re-ranking
    full = fv.IvfPq.train(ctx, fv.Metric.L2, dim, base[:20_000], fv.IvfPqParams(48, 16, 5, True, 1))
    blob = full.save()
    full.add(base)
    part = fv.IvfPq.load(ctx, blob)
    part.set_shard(rank, world)
    part.add(base)
    for mode in (0, 1, 3):
        full.set_scan_mode(mode)
        part.set_scan_mode(mode)
        for nprobe, refine in [(16, 10), (48, 0), (4, 3)]:
            got, gc = ShardedSearch(ctx, part, "ivfpq", world).search_batch(dq, k, nprobe, refine)
            want, wc = full.search_batch(dq, k, nprobe, refine)
            assert torch.equal(got, want) and torch.equal(gc, wc), f"IVF-PQ list shards, mode {mode} nprobe {nprobe} refine {refine}"
    # query slices over replicas (no list shards: L = 1, Q = 2), odd batch sizes included
    for mode in (0, 3):
        full.set_scan_mode(mode)
        for nq_s, nprobe, refine in [(nq, 16, 10), (nq - 1, 48, 0), (1, 4, 3), (3, 8, 0)]:
            got, gc = full.search_sharded(dq[:nq_s].contiguous(), k, nprobe, refine)
            want, wc = full.search_batch(dq[:nq_s].contiguous(), k, nprobe, refine)
            assert torch.equal(got, want) and torch.equal(gc, wc), f"IVF-PQ query slices, mode {mode} nq {nq_s}"
    full.set_scan_mode(0)
    # a small batch: every rank does its own coarse step, no cell exchange
    got, gc = part.search_sharded(dq[:50], k, 8, 4)
    want, wc = full.search_batch(dq[:50], k, 8, 4)
    assert torch.equal(got, want) and torch.equal(gc, wc)
    # the stage table of the collective call: coarse slice, cell exchange, local search, candidate exchange, merge
    ctx.set_timing(True)
    part.search_sharded(dq, k, 16, 10)
    st = ctx.stats()["stage_ms"]
    assert all(x > 0 for x in st[:5]), st
    dist.barrier()
    dist.destroy_process_group()
    open(os.path.join(tmp, f"ok{rank}"), "w").write("ok")


def test_two_gpu_sharded_search_through_the_c_abi(tmp_path):
    import socket

    import torch
    import torch.multiprocessing as mp

    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    assert os.path.exists(tmp_path / "ok0") and os.path.exists(tmp_path / "ok1")
