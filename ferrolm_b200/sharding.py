"""Host-side plumbing of the multi-GPU layout: one process per GPU, `torch.distributed` for the one
exchange step.  The base is split over the ranks (contiguous row ranges for exact search, inverted lists
for IVF-PQ), every rank searches its part for the whole query batch, the per-rank candidate lists are
all-gathered and merged by a kernel of the library.  Nothing here computes distances.
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


class ShardedSearch:
    """search_batch over an index that is split across the ranks of the default process group.

    kind "flat":  `index` is a FlatIndex over this rank's row range (set_id_base(lo) before add).
    kind "ivfpq": `index` is an IvfPq with set_shard(rank, world) that was given all rows.
    """

    def __init__(self, ctx, index, kind: str, world: int):
        self.ctx, self.index, self.kind, self.world = ctx, index, kind, world

    def search_batch(self, queries, k: int, nprobe: int = 0, refine: int = 0):
        ix = self.index
        if self.kind == "flat":
            out, counts = ix.search_batch(queries, k)
            if self.world == 1:
                return out, counts
            return self.ctx.merge_topk(all_gather_stacked(out, self.world), all_gather_stacked(counts, self.world), k)
        if self.world == 1:
            return ix.search_batch(queries, k, nprobe, refine)
        cells = self._coarse_by_query_slices(queries, nprobe)
        if refine > 0:
            # a shard may not cut to k on its own: the global cut by compressed distance comes first
            # (unused candidate slots carry the id 0xFFFFFFFF, so the per-shard counts need not travel)
            adc, exact, _ = ix.search_candidates(queries, k * refine, nprobe, cells)
            return self.ctx.merge_refine(all_gather_stacked(adc, self.world), all_gather_stacked(exact, self.world),
                                         None, k)
        out, counts = ix.search_batch(queries, k, nprobe, 0, cells)
        return self.ctx.merge_topk(all_gather_stacked(out, self.world), all_gather_stacked(counts, self.world), k)

    def _coarse_by_query_slices(self, queries, nprobe: int):
        """Every list shard needs the probed cells of ALL queries; instead of each shard repeating the whole coarse
        search, rank r computes the cells of query slice r and the slices are all-gathered.  None (= let the search
        do its own coarse step) for host arrays and for batches too small to be worth an exchange."""
        if not (hasattr(queries, "is_cuda") and queries.is_cuda):
            return None
        q = queries.contiguous().view(-1, self.index.dim)
        if q.shape[0] < 256 * self.world:
            return None
        return per_query_slices(lambda part: self.index.coarse(part, nprobe), q, self.world)


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
