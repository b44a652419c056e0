"""The allocation-free shard merge (fv_merge_topk_static_dev) against the ordinary one.

It exists for callers that cannot allocate device memory (all HBM already handed to their own
arena, code inside another runtime's callback or replayed section): its scratch is a fixed array
in the library image.  The test calls it through the C ABI twice in a row with different inputs --
the array keeps the first call's contents, so the second call shows that nothing stale leaks --
and demands bit-identical results (the merge is integer/bit work on (distance, id) keys).
Collected last on purpose: a failure here cannot hide the result of any other test.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def make_parts(torch, seed, nparts, nq, k_in):
    g = torch.Generator(device="cpu").manual_seed(seed)
    dist = torch.rand((nparts, nq, k_in), generator=g).sort(dim=2).values
    ids = torch.randperm(nparts * nq * k_in, generator=g).reshape(nparts, nq, k_in).to(torch.int32)
    counts = torch.randint(0, k_in + 1, (nparts, nq), generator=g, dtype=torch.int32)
    parts = torch.stack([ids, dist.view(torch.int32)], dim=3).contiguous()
    return parts.cuda(), counts.cuda()


def test_static_merge_equals_the_allocating_merge_twice_in_a_row():
    import torch

    import ferrolm_b200 as fv

    ctx = fv.Context(0)
    for call, (seed, nparts, nq, k_in, k_out) in enumerate([(1, 4, 3000, 10, 10), (2, 3, 700, 16, 7)]):
        parts, counts = make_parts(torch, seed, nparts, nq, k_in)
        want, want_counts = ctx.merge_topk(parts, counts, k_out)
        out = torch.full((nq, k_out, 2), -7, dtype=torch.int32, device="cuda")
        got_counts = torch.full((nq,), -7, dtype=torch.int32, device="cuda")
        torch.cuda.synchronize()
        if call == 1:
            # the second call finds everything in place: free device memory must not move across it
            # (the first call may load the library's kernels and the array onto the device)
            free_before, _ = torch.cuda.mem_get_info()
        fv.merge_topk_static(parts, counts, k_out, out, got_counts)
        if call == 1:
            free_after, _ = torch.cuda.mem_get_info()
            assert free_after == free_before, "the allocation-free merge changed the free device memory"
        assert torch.equal(out, want), f"call {call}: neighbours differ"
        assert torch.equal(got_counts, want_counts), f"call {call}: counts differ"
        # against an independent statement of the merge on the host
        p, c = parts.cpu().numpy(), counts.cpu().numpy()
        for q in range(0, nq, 97):
            cand = [(np.int32(p[s, q, i, 1]).view(np.float32), int(np.uint32(p[s, q, i, 0])))
                    for s in range(nparts) for i in range(c[s, q])]
            cand.sort()
            ref = cand[:k_out]
            got = fv.neighbors_from_tensor(out[q:q + 1])[0][: len(ref)]
            assert [int(x) for x in got["id"]] == [r[1] for r in ref]
            assert int(got_counts[q]) == len(ref)


def test_static_merge_refuses_what_does_not_fit():
    import torch

    import ferrolm_b200 as fv

    parts, counts = make_parts(torch, 3, 2, 64, 4)
    nq_big = 262144 // 8 + 1
    out = torch.empty((nq_big, 8, 2), dtype=torch.int32, device="cuda")
    cnt = torch.empty((nq_big,), dtype=torch.int32, device="cuda")
    big_parts = torch.zeros((1, nq_big, 8, 2), dtype=torch.int32, device="cuda")
    with pytest.raises(fv.FerrovecError, match="exceeds the static scratch"):
        fv.merge_topk_static(big_parts, None, 8, out, cnt)
