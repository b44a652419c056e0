"""Host-side plumbing of the multi-GPU layout: one process per GPU.  The base is split over the ranks (contiguous
row ranges for exact search, inverted lists for IVF-PQ), every rank searches its part for the whole query batch,
the per-rank candidate lists are all-gathered and merged.  On GPUs all of that happens inside the library
(fv_*_search_sharded_dev: NCCL on the context's stream, then a merge kernel); this module forms the group and keeps
the small helpers that state the exchange protocol on CPU tensors for the gloo test.  Nothing here computes distances.
"""
from __future__ import annotations


def row_range(rank: int, world: int, n: int) -> tuple[int, int]:
    """Contiguous rows [lo, hi) of rank `rank`: local row + lo is the global id."""
    per = (n + world - 1) // world
    lo = min(n, rank * per)
    return lo, min(n, lo + per)


def all_gather_stacked(t, world: int):
    """(world, *t.shape) tensor holding every rank's `t`, rank-major; works for NCCL (CUDA) and gloo (CPU)."""
    import torch
    import torch.distributed as dist

    t = t.contiguous()
    out = torch.empty((world,) + tuple(t.shape), dtype=t.dtype, device=t.device)
    if t.is_cuda:
        dist.all_gather_into_tensor(out, t)
    else:
        dist.all_gather(list(out.unbind(0)), t)
    return out


def init_group(ctx, rank: int, world: int):
    """Puts `ctx` into the library's group of `world` ranks.  The 128-byte group id is made by rank 0 and travels by
    a `torch.distributed` broadcast (any host channel would do: the library only needs the bytes on every rank)."""
    import numpy as np
    import torch
    import torch.distributed as dist

    from .vector import comm_unique_id

    if world == 1:
        return
    dev = torch.device("cuda", ctx.device) if torch.cuda.is_available() and dist.get_backend() == "nccl" else torch.device("cpu")
    t = torch.zeros(128, dtype=torch.uint8, device=dev)
    if rank == 0:
        t.copy_(torch.from_numpy(np.frombuffer(comm_unique_id(), dtype=np.uint8).copy()))
    dist.broadcast(t, 0)
    ctx.comm_init(bytes(t.cpu().numpy()), world, rank)


class ShardedSearch:
    """search_batch over an index that is split across the ranks of the context's group (`init_group`).

    kind "flat":  `index` is a FlatIndex over this rank's row range (set_id_base(lo) before add).
    kind "ivfpq": `index` is an IvfPq with set_shard(rank, world) that was given all rows.
    The exchange and the merge happen inside the library (NCCL on the context's stream): one collective call.
    """

    def __init__(self, ctx, index, kind: str, world: int):
        self.ctx, self.index, self.kind, self.world = ctx, index, kind, world

    def search_batch(self, queries, k: int, nprobe: int = 0, refine: int = 0):
        ix = self.index
        if self.kind == "flat":
            return ix.search_sharded(queries, k) if self.world > 1 else ix.search_batch(queries, k)
        if self.world == 1:
            return ix.search_batch(queries, k, nprobe, refine)
        return ix.search_sharded(queries, k, nprobe, refine)


def per_query_slices(compute, queries, world: int):
    """`compute(queries[lo:hi])` on this rank's contiguous slice of the query rows, all-gathered: returns what
    `compute(queries)` would, with every rank doing 1/world of the work.  `compute` maps (n, d) -> (n, w) rows."""
    import torch
    import torch.distributed as dist

    nq = queries.shape[0]
    per = (nq + world - 1) // world
    lo, hi = row_range(dist.get_rank(), world, nq)
    mine = compute(queries[lo:hi])
    if hi - lo < per:  # the last slices may be short: pad so that all ranks send the same amount
        pad = torch.zeros((per - (hi - lo), mine.shape[1]), dtype=mine.dtype, device=mine.device)
        mine = torch.cat([mine, pad])
    return all_gather_stacked(mine, world).view(world * per, -1)[:nq].contiguous()
