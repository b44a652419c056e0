#!/usr/bin/env python
"""Benchmark of the vector-search hot path: queries/s at recall@10 on N=1M, d=128, k=10.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload ivfpq|flat|hnsw] [--impl reference]

One "step" is one search_batch over a 10,000-query batch (seeded synthetic data with the shape and
value range of SIFT1M, which cannot be shipped: clipped-integer Gaussian mixture).  The default
workload is the IVF-PQ configuration (nlist=1024, M=16x8 bit, trained on a 100,000-row sample,
nprobe=64, refine=10); --workload flat is exact L2 search on the same data, --workload hnsw the
graph index.  With N>1 GPUs (one process per GPU under torchrun) the base rows are sharded
over the ranks (strong scaling: the 1M rows are fixed) -- contiguous row ranges for exact search, inverted
lists for IVF-PQ -- and every step is ONE collective call of the library: each rank searches its part, the
per-rank candidates are all-gathered over NCCL on the library's stream and merged by its kernels.

The line printed by rank 0 carries: `value` (device-resident queries), `e2e` (host queries in pinned
memory, copies inside the timed region), `roofline` of the dominant kernel (algorithmic bytes or
flops per launch over its CUDA-event duration), `cpu_baseline` (the CPU oracle timed on the host
cores on a bounded sample, with the reference's own protocol: all threads, and one thread on the first
2,000 queries), `parity_sample` and `recall_at_10`, the per-stage device times, the sampled GPU clocks and,
at N=1, `also`: the other benchmark configurations at a glance.

--impl reference times the CPU restatement of the reference's algorithm (the reference is Rust and
cannot be built here) on the host cores with all threads, same data and configuration; it loads
nothing of the GPU library.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

N_BASE, DIM, NQ, K = 1_000_000, 128, 10_000, 10
CLUSTERS = 256
IVF = dict(nlist=1024, m=16, iters=20, learn=100_000, nprobe=64, refine=10)
BIG_IVF = dict(nlist=16384, m=16, iters=20, learn=640_000, nprobe=32)  # configs[4]; 39 training rows per list
HNSW = dict(m=16, ef_construction=200, ef=64)
METRIC = "queries/s at recall@10 (N=1M, d=128, k=10)"
IVF_STAGES = ["coarse cells", "query tables + bound pass", "pair bucketing + operand gather", "scan", "re-score of survivors",
              "sort + re-rank", "keys -> neighbours"]
IVF_SHARDED_STAGES = ["coarse cells of the rank's query slice", "cell exchange (NCCL all-gather)",
                      "local search up to the shard's candidates", "candidate exchange (NCCL all-gather)", "merge"]
IVF_GRID_STAGES = ["(no coarse step outside the local search)", "(no cell exchange)", "local search of the rank's query slice", "candidate exchange between the list shards (NCCL all-gather)",
                   "merge + result exchange (NCCL all-gather) + unpacking"]
FLAT_STAGES = ["query conversion", "sample pass", "main pass (tensor cores)", "exact re-rank + certificate",
               "full-precision re-run of uncertified queries", "keys -> neighbours"]
FLAT_SHARDED_STAGES = ["local search", "result exchange (NCCL all-gather)", "merge"]


def peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            p = json.load(f)
        return {"hbm_gbs": float(p["hbm_gbs"]), "tflops": float(p["bf16_tflops"]),
                "tflops_sustained": float(p.get("bf16_tflops_sustained", p["bf16_tflops"])), "source": "measured"}
    except Exception:
        return {"hbm_gbs": 6650.0, "tflops": 1590.0, "tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region runs: ONE process for all the job's GPUs
    (rank 0 starts it; a poller per rank, eight on one host, delays the ranks' launches by different amounts and the
    step waits for the slowest)."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.lines, self.proc, self.thread = index, [], None, None

    def start(self):
        if self.index is None:  # a rank that leaves the sampling to rank 0
            return
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except Exception:
            self.proc = None
            return
        self.thread = threading.Thread(target=lambda: [self.lines.append(l) for l in self.proc.stdout], daemon=True)
        self.thread.start()

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()  # the exact process started above
        try:
            self.proc.wait(timeout=5)
        except Exception:
            pass
        sm, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for l in self.lines:
            f = [x.strip() for x in l.split(",")]
            if len(f) < 6:
                continue
            try:
                sm.append(float(f[0]))
                mx = float(f[1])
            except ValueError:
                continue
            for name, v in zip(names, f[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(sm)}


def workload_config(workload: str, n_gpus: int, nprobe: int, refine: int, list_shards: int = 0) -> dict:
    if n_gpus == 1:
        sharding = "single GPU"
    elif workload == "ivfpq" and list_shards and list_shards < n_gpus:
        sharding = (f"grid of {list_shards} list shard(s) x {n_gpus // list_shards} query slices over {n_gpus} GPUs: a rank searches its "
                    "slice of the batch on its lists; candidates are all-gathered between list shards and merged, finished "
                    "slices all-gathered (NCCL) so that every rank holds the whole result")
    else:
        sharding = (f"{'inverted lists' if workload == 'ivfpq' else 'row ranges'} over {n_gpus} GPUs, per-shard candidates "
                    "all-gathered (NCCL) and merged")
    cfg = {"n": N_BASE, "d": DIM, "nq": NQ, "k": K, "distribution": f"clipped-integer Gaussian mixture, {CLUSTERS} clusters",
           "sharding": sharding,
           "l2_note": "inputs exceed L2: 1M x 128 f32 rows (512 MB), 256 MB of 16-bit codeword rows and 164 MB of query "
                      "tables are re-read each step"}
    if workload == "ivfpq":
        cfg.update({"workload": f"IVF-PQ L2 search, nlist=1024, M=16x8bit, nprobe={nprobe}, refine={refine} (BASELINE configs[2])",
                    "nlist": IVF["nlist"], "m": IVF["m"], "nprobe": nprobe, "refine": refine})
    elif workload == "flat":
        cfg.update({"workload": "exact L2 k-NN, tensor-core front end + exact re-rank (BASELINE configs[0] shape at N=1M)"})
    else:
        cfg.update({"workload": "HNSW L2 search, M=16, efC=200, efSearch=64 (BASELINE configs[3])", **HNSW})
    return cfg


def timed_cpu(search, queries, threads: int, budget_s: float = 10.0):
    """The reference's timing protocol (src/main.rs:496-507): qps_n with all threads over whole passes of the query
    batch (as many as fit the budget), qps_1 with one thread over the first 2,000 queries."""
    t0 = time.perf_counter()
    search(queries, threads)
    one = time.perf_counter() - t0
    passes = int(max(1, min(64, round(budget_s / max(one, 1e-3)))))
    t0 = time.perf_counter()
    for _ in range(passes):
        search(queries, threads)
    dt = time.perf_counter() - t0
    n1 = min(len(queries), 2000)
    t0 = time.perf_counter()
    search(queries[:n1], 1)
    d1 = time.perf_counter() - t0
    return {"qps_n": passes * len(queries) / dt, "qps_1": n1 / d1, "passes": passes, "seconds": dt + d1,
            "single_thread_queries": n1}


# ----------------------------------------------------------------------------------------------- reference arm
def run_reference(args):
    """The CPU restatement of the reference (oracle/), all host threads, same data and configuration.  Nothing of
    the GPU library is imported here."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import oracle

    oracle.build()
    threads = oracle.cores()
    base = oracle.datagen(0, 1, N_BASE, DIM, CLUSTERS)
    queries = oracle.datagen(0, 2, NQ, DIM, CLUSTERS)
    nprobe, refine = args.nprobe or IVF["nprobe"], IVF["refine"] if args.refine is None else args.refine
    t0 = time.perf_counter()
    if args.workload == "ivfpq":
        learn = oracle.datagen(0, 3, IVF["learn"], DIM, CLUSTERS)
        ix = oracle.IvfPq.train(oracle.L2, DIM, learn, IVF["nlist"], IVF["m"], IVF["iters"], True, 1, threads)
        ix.add(base, threads)
        nqs = NQ
        search = lambda q, t: ix.search_batch(q, K, nprobe, refine, t)
        sample = f"all {nqs} queries per step, index built by the CPU oracle"
    elif args.workload == "flat":
        ix = oracle.FlatIndex(oracle.L2, DIM)
        ix.add(base)
        nqs = min(NQ, 64 * max(1, threads // 8))
        search = lambda q, t: ix.search_batch(q, K, t)
        sample = f"first {nqs} of {NQ} queries per step (a full batch is minutes of CPU time)"
    else:
        ix = oracle.Hnsw.build(oracle.L2, DIM, base, HNSW["m"], HNSW["ef_construction"], 1, threads)
        nqs = NQ
        search = lambda q, t: ix.search_batch(q, K, HNSW["ef"], t)
        sample = f"all {nqs} queries per step, graph built by the CPU oracle with {threads} threads"
    build_s = time.perf_counter() - t0
    for _ in range(args.warmup):
        search(queries[:nqs], threads)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        search(queries[:nqs], threads)
    dt = (time.perf_counter() - t0) / args.steps
    qps = nqs / dt
    n1 = min(nqs, 2000)
    t0 = time.perf_counter()
    search(queries[:n1], 1)
    qps_1 = n1 / (time.perf_counter() - t0)
    line = {
        "impl": "reference", "metric": METRIC, "value": qps, "unit": "queries/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        # the configuration of the arm this one is compared with at the same N (the CPU search itself has one layout)
        "config": workload_config(args.workload, int(os.environ.get("WORLD_SIZE", "1")), nprobe, refine,
                                  (args.list_shards or 1) if args.workload == "ivfpq" else 0),
        "cpu_baseline": {"value": qps, "unit": "queries/s", "cores": threads, "kind": "port", "sample": sample,
                         "qps_1": qps_1, "qps_1_note": f"one thread, first {n1} queries (the reference's own protocol)",
                         "build_s": build_s},
        "e2e": {"value": qps, "unit": "queries/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


# ----------------------------------------------------------------------------------------------- GPU arm
def time_gpu(fn, stream, reps: int, warm: int = 3):
    """Mean device time of fn() over `reps` calls, CUDA events on the library's stream."""
    import torch

    for _ in range(warm):
        fn()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(reps):
        fn()
    e1.record(stream)
    stream.synchronize()
    return e0.elapsed_time(e1) / reps


def also_section(fv, oracle, ctx, stream, ix, base, queries, dq, pk, nprobe, refine, threads):
    """The other benchmark configurations at a glance (N=1 only): each entry carries its own time, recall against
    exact search on the same data and, where the oracle is cheap enough, a parity sample."""
    import torch

    out = {}
    nsub = 500
    flat = fv.FlatIndex(ctx, fv.Metric.L2, DIM)
    flat.add(base)
    truth_t, _ = flat.search_batch(dq, K)
    truth = fv.neighbors_from_tensor(truth_t)["id"]

    def rec(res):
        o, c = res
        return fv.recall(fv.neighbors_from_tensor(o), c.cpu().numpy().astype(np.uint32), truth, K)

    # exact search on the same data (recall 1.0 by construction), same timing method
    ms_f = time_gpu(lambda: flat.search_batch(dq, K), stream, 10)
    st = ctx.stats()
    gemm_ms = st["stage_ms"][2]
    tf = 2.0 * NQ * N_BASE * DIM / (gemm_ms * 1e-3) / 1e12
    out["exact_search_same_data"] = {"value": NQ / (ms_f * 1e-3), "unit": "queries/s", "recall_at_10": 1.0, "ms_per_step": ms_f,
                                     "gemm_topk_kernel_ms": gemm_ms, "tensor_tflops": tf, "frac_of_measured_peak": tf / pk["tflops"],
                                     "uncertified": st["uncertified"]}
    del flat
    # the sweep of the reference's driver (src/main.rs:553-565) on this index, with a parity sample each
    oix = oracle.IvfPq.load(ix.save())
    sweep = {}
    for rf in (0, 10):
        for npb in (1, 4, 16, 64):
            ms_s = time_gpu(lambda: ix.search_batch(dq, K, npb, rf), stream, 5, warm=2)
            st = ctx.stats()
            got = ix.search_batch(dq, K, npb, rf)
            want, wc = oix.search_batch(queries[:nsub], K, npb, rf, threads)[:2]
            g = fv.neighbors_from_tensor(got[0])[:nsub]
            sweep[f"nprobe={npb},refine={rf}"] = {
                "value": NQ / (ms_s * 1e-3), "ms_per_step": ms_s, "recall_at_10": rec(got),
                "scan_ms": st["stage_ms"][3], "code_bytes_scanned": st["rows_scanned"] * IVF["m"],
                "parity_sample": {"queries": nsub, "identical_id_rows": int((g["id"] == want["id"]).all(axis=1).sum()),
                                  "bit_equal_distances": bool((g["distance"].view(np.uint32) == want["distance"].view(np.uint32)).all())}}
    out["ivfpq_sweep"] = sweep
    del oix
    # the three scans on the headline configuration
    scans = {}
    for mode, name in ((1, "per_query_kernel"), (2, "list_major_table_scan"), (3, "list_major_tensor_core_pass")):
        ix.set_scan_mode(mode)
        ms_s = time_gpu(lambda: ix.search_batch(dq, K, nprobe, refine), stream, 5, warm=2)
        st = ctx.stats()
        scans[name] = {"ms_per_step": ms_s, "stage_ms": dict(zip(IVF_STAGES, [round(float(x), 4) for x in st["stage_ms"][:7]])),
                       "scan_gbs_of_code_bytes": st["rows_scanned"] * IVF["m"] / (st["stage_ms"][3] * 1e-3) / 1e9}
    ix.set_scan_mode(0)
    out["ivfpq_scans"] = scans
    # HNSW (BASELINE configs[3]) on a 200,000-node graph built on the GPU, efSearch 64
    hn, hq = 200_000, NQ
    t0 = time.perf_counter()
    h = fv.Hnsw.build_batched(ctx, fv.Metric.L2, DIM, base[:hn], fv.HnswParams(HNSW["m"], HNSW["ef_construction"], 1))
    gpu_build_s = time.perf_counter() - t0
    t0 = time.perf_counter()
    oh = oracle.Hnsw.build(oracle.L2, DIM, base[:hn], HNSW["m"], HNSW["ef_construction"], 1, threads)
    cpu_build_s = time.perf_counter() - t0
    cpu_reachable = oh.reachable()
    oh = oracle.Hnsw.load(h.save())  # the oracle searches the graph the GPU built
    dqh = dq[:hq].contiguous()
    fsub = fv.FlatIndex(ctx, fv.Metric.L2, DIM)
    fsub.add(base[:hn])
    ht = fv.neighbors_from_tensor(fsub.search_batch(dqh, K)[0])["id"]
    ms_h = time_gpu(lambda: h.search_batch(dqh, K, HNSW["ef"]), stream, 5, warm=2)
    st = ctx.stats()
    got = h.search_batch(dqh, K, HNSW["ef"])
    want, wc = oh.search_batch(queries[:nsub], K, HNSW["ef"], threads)[:2]
    g = fv.neighbors_from_tensor(got[0])
    alg = st["dist_evals"] * DIM * 4 + st["expansions"] * (2 * HNSW["m"] + 1) * 4
    out["hnsw_ef64_200k_nodes"] = {
        "value": hq / (ms_h * 1e-3), "unit": "queries/s", "ms_per_step": ms_h, "queries": hq,
        "recall_at_10": fv.recall(g, got[1].cpu().numpy().astype(np.uint32), ht, K),
        "gather_gbs": alg / (st["stage_ms"][0] * 1e-3) / 1e9, "frac_of_measured_hbm": alg / (st["stage_ms"][0] * 1e-3) / 1e9 / pk["hbm_gbs"],
        "parity_sample": {"queries": nsub, "identical_id_rows": int((g[:nsub]["id"] == want["id"]).all(axis=1).sum())},
        "graph_build": {"gpu_batched_s": round(gpu_build_s, 3), "reachable": h.reachable(),
                        "cpu_oracle_s": round(cpu_build_s, 3), "cpu_threads": threads, "cpu_reachable": cpu_reachable,
                        "note": "m 16, ef_construction 200; seconds include the host-side padding and copies"}}
    # the reference's ef sweep (src/main.rs:523-524) on the same graph
    sweep = {}
    for ef in (16, 32, 128, 256):
        ms_e = time_gpu(lambda: h.search_batch(dqh, K, ef), stream, 3, warm=1)
        o_e = h.search_batch(dqh, K, ef)
        sweep[f"ef{ef}"] = {"queries_per_s": round(hq / (ms_e * 1e-3)), "ms_per_step": round(ms_e, 3),
                            "recall_at_10": round(float(fv.recall(fv.neighbors_from_tensor(o_e[0]),
                                                                  o_e[1].cpu().numpy().astype(np.uint32), ht, K)), 4)}
    out["hnsw_ef64_200k_nodes"]["ef_sweep"] = sweep
    del h, oh, fsub
    # IVF-PQ on the reference's own test generator (tests/vector.rs:11-24: 50 centres, sigma 1), where the compressed
    # distances rank well: one operating point with a recall that says something
    rn = 1_000_000
    rbase = oracle.testdata(rn, DIM, 1)
    rq = oracle.testdata(NQ, DIM, 2)
    rix = fv.IvfPq.train(ctx, fv.Metric.L2, DIM, rbase[:100_000], fv.IvfPqParams(IVF["nlist"], IVF["m"], IVF["iters"], True, 1))
    rix.add(rbase)
    drq = torch.from_numpy(rq).cuda()
    rflat = fv.FlatIndex(ctx, fv.Metric.L2, DIM)
    rflat.add(rbase)
    rt = fv.neighbors_from_tensor(rflat.search_batch(drq, K)[0])["id"]
    ms_r = time_gpu(lambda: rix.search_batch(drq, K, nprobe, refine), stream, 5, warm=2)
    got = rix.search_batch(drq, K, nprobe, refine)
    out["ivfpq_on_the_reference_test_generator"] = {
        "value": NQ / (ms_r * 1e-3), "unit": "queries/s", "ms_per_step": ms_r, "n": rn,
        "recall_at_10": fv.recall(fv.neighbors_from_tensor(got[0]), got[1].cpu().numpy().astype(np.uint32), rt, K)}
    del rix, rflat, rbase
    # exact inner-product search on unit-length 384-d rows (BASELINE configs[1]: the regime where the tensor-core scores
    # carry rounding error and the certificate decides)
    d1 = 384
    ebase = fv.datagen(1, 1, N_BASE, d1, 1000)
    eq = fv.datagen(1, 2, NQ, d1, 1000)
    eflat = fv.FlatIndex(ctx, fv.Metric.InnerProduct, d1)
    eflat.add(ebase)
    deq = torch.from_numpy(eq).cuda()
    ms_e = time_gpu(lambda: eflat.search_batch(deq, K), stream, 5, warm=2)
    st = ctx.stats()
    got = eflat.search_batch(deq, K)
    ofl = oracle.FlatIndex(oracle.INNER_PRODUCT, d1)
    ofl.add(ebase)
    nse = 64
    want, wc = ofl.search_batch(eq[:nse], K, threads)
    g = fv.neighbors_from_tensor(got[0])[:nse]
    tfe = 2.0 * NQ * N_BASE * d1 / (st["stage_ms"][2] * 1e-3) / 1e12
    out["exact_inner_product_1Mx384"] = {
        "value": NQ / (ms_e * 1e-3), "unit": "queries/s", "ms_per_step": ms_e, "gemm_topk_kernel_ms": st["stage_ms"][2],
        "tensor_tflops": tfe, "frac_of_measured_peak": tfe / pk["tflops"], "uncertified": st["uncertified"],
        "parity_sample": {"queries": nse, "identical_id_rows": int((g["id"] == want["id"]).all(axis=1).sum()),
                          "bit_equal_distances": bool((g["distance"].view(np.uint32) == want["distance"].view(np.uint32)).all())}}
    return out


def run_ours(args):
    import torch
    import torch.distributed as dist

    import ferrolm_b200 as fv

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: this library has no CPU path")
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    ctx = fv.Context(local)
    ctx.set_timing(True)
    stream = torch.cuda.ExternalStream(ctx.stream_handle(), device=local)  # everything runs on the library's stream

    from ferrolm_b200.sharding import ShardedSearch, init_group, row_range

    init_group(ctx, rank, world)  # the library's own NCCL group; torch.distributed only carried the 128-byte id

    t_build = time.perf_counter()
    refine, nprobe = 0, 0
    base, empty_blob = None, None
    list_shards = world  # IVF-PQ: list shards of the grid (the rest of the group are query slices)
    if args.big:
        # BASELINE configs[4]: 50M x 128, 4096 clusters; rows are generated on the GPU in chunks and never
        # exist on the host.  exact search: row ranges; IVF-PQ: nlist=16384, nprobe=32, sharded by list.
        queries = fv.datagen(0, 2, NQ, DIM, CLUSTERS)

        def add_rows(index, r0, r1):
            step_rows = 4_000_000
            for a0 in range(r0, r1, step_rows):
                t = fv.datagen_dev(ctx, 1, min(step_rows, r1 - a0), DIM, CLUSTERS, first_row=a0)
                index.add(t)
                del t

        if args.workload == "ivfpq":
            lo, hi = 0, N_BASE
            learn = fv.datagen_dev(ctx, 3, BIG_IVF["learn"], DIM, CLUSTERS).cpu().numpy()
            ix = fv.IvfPq.train(ctx, fv.Metric.L2, DIM, learn,
                                fv.IvfPqParams(BIG_IVF["nlist"], BIG_IVF["m"], BIG_IVF["iters"], False, 1))
            ix.set_shard(rank, world)
            add_rows(ix, 0, N_BASE)
            ix.set_scan_mode(args.scan_mode)
            refine, nprobe = 0, BIG_IVF["nprobe"]
            searcher = ShardedSearch(ctx, ix, "ivfpq", world)
        elif args.workload == "flat":
            lo, hi = row_range(rank, world, N_BASE)
            ix = fv.FlatIndex(ctx, fv.Metric.L2, DIM)
            ix.set_id_base(lo)
            add_rows(ix, lo, hi)
            searcher = ShardedSearch(ctx, ix, "flat", world)
        else:
            raise SystemExit("--big covers the flat and ivfpq workloads")
    elif args.workload == "ivfpq":
        # sharded by inverted list: every rank trains the same quantizers (deterministic) and is given all rows;
        # it keeps and scans the lists l with l % world == rank
        lo, hi = 0, N_BASE
        base = fv.datagen(0, 1, N_BASE, DIM, CLUSTERS)
        queries = fv.datagen(0, 2, NQ, DIM, CLUSTERS)
        learn = fv.datagen(0, 3, IVF["learn"], DIM, CLUSTERS)
        ix = fv.IvfPq.train(ctx, fv.Metric.L2, DIM, learn, fv.IvfPqParams(IVF["nlist"], IVF["m"], IVF["iters"], True, 1))
        if world > 1 and rank == 0:
            empty_blob = ix.save()  # the trained quantizers, for the unsharded copy the result is checked against
        # the group is a grid: list_shards list shards x (world / list_shards) query slices, rank = slice * L + shard
        list_shards = args.list_shards or 1
        if world % list_shards:
            raise SystemExit("--list-shards must divide the number of GPUs")
        if list_shards > 1:
            ix.set_shard(rank % list_shards, list_shards)
        ix.add(base)
        ix.set_scan_mode(args.scan_mode)
        refine, nprobe = IVF["refine"] if args.refine is None else args.refine, args.nprobe or IVF["nprobe"]
        searcher = ShardedSearch(ctx, ix, "ivfpq", world)
    elif args.workload == "flat":
        lo, hi = row_range(rank, world, N_BASE)  # contiguous row shards
        base = fv.datagen(0, 1, hi - lo, DIM, CLUSTERS, first_row=lo)
        queries = fv.datagen(0, 2, NQ, DIM, CLUSTERS)
        ix = fv.FlatIndex(ctx, fv.Metric.L2, DIM)
        ix.set_id_base(lo)
        ix.add(base)
        searcher = ShardedSearch(ctx, ix, "flat", world)
    else:
        if world > 1:
            raise SystemExit("hnsw: replicas only (one graph); run with --gpus 1")
        lo, hi = 0, N_BASE
        base = fv.datagen(0, 1, N_BASE, DIM, CLUSTERS)
        queries = fv.datagen(0, 2, NQ, DIM, CLUSTERS)
        ix = fv.Hnsw.build_batched(ctx, fv.Metric.L2, DIM, base, fv.HnswParams(HNSW["m"], HNSW["ef_construction"], 1))
        searcher = None
    build_s = time.perf_counter() - t_build

    dq = torch.from_numpy(queries).cuda()
    hq = torch.from_numpy(queries).pin_memory()
    h_out = torch.empty((NQ, K, 2), dtype=torch.int32).pin_memory()
    launches = [0]
    stage_sum = np.zeros(8)
    last = {}

    def step(q):
        """One search_batch of the whole (possibly sharded) index on device-resident queries."""
        with torch.cuda.stream(stream):
            if searcher is None:
                r = ix.search_batch(q, K, HNSW["ef"])
            else:
                r = searcher.search_batch(q, K, nprobe, refine)
        st = ctx.stats()
        launches[0] += st["launches"]
        stage_sum[:] += np.array(st["stage_ms"])
        last.update(st)
        return r[0], r[1]

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-resident timing (value)
    # rank 0 samples every GPU of the job (ranks use GPUs 0..world-1 of the node)
    sampler = ClockSampler(",".join(str(i) for i in range(world)) if rank == 0 else None)
    sampler.start()
    n_warm = max(args.warmup, 3)
    if world > 1 and searcher is not None:
        # NCCL sets its channels up over the first collectives of a group: a few small sharded searches (not steps of
        # the workload) before the warm-up steps, so that the warm-up steps are already steady
        with torch.cuda.stream(stream):
            for _ in range(8):
                searcher.search_batch(dq[:64 * world].contiguous(), K, *((nprobe, refine) if args.workload == "ivfpq" else ()))
        barrier()
    for _ in range(n_warm):
        step(dq)
    barrier()
    launches[0] = 0
    stage_sum[:] = 0
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.profiler.start()  # lets `ncu --profile-from-start off` skip the index build
    ev0.record(stream)
    for _ in range(args.steps):
        out, counts = step(dq)
    ev1.record(stream)
    barrier()
    torch.cuda.profiler.stop()
    ms = ev0.elapsed_time(ev1) / args.steps
    steady_launches = launches[0]
    stages = stage_sum / args.steps
    # ---- end to end: host queries (pinned) in, host results out, every step.  A rank of a query-slice grid reads
    # only its own slice of the batch (fv_ivfpq_search_sharded_dev), so that is what it copies.
    q_lo, q_hi = 0, NQ
    if world > 1 and args.workload == "ivfpq" and list_shards < world:
        slices = world // list_shards
        per = (NQ + slices - 1) // slices
        q_lo = min(NQ, (rank // list_shards) * per)
        q_hi = min(NQ, q_lo + per)
    q_dev = torch.empty_like(dq)

    def upload():
        # on the library's own stream: the search that follows is ordered behind the copy, the host need not wait for it
        with torch.cuda.stream(stream):
            q_dev[q_lo:q_hi].copy_(hq[q_lo:q_hi], non_blocking=True)
        return q_dev

    for _ in range(2):
        o, c = step(upload())
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        q = upload()
        o, c = step(q)
        with torch.cuda.stream(stream):
            h_out.copy_(o, non_blocking=True)
        stream.synchronize()
    barrier()
    e2e_ms = (time.perf_counter() - t0) * 1e3 / args.steps
    clocks = sampler.stop()
    # how the shard's own search splits (the collective call reports a coarser table of its own)
    local_st = None
    if world > 1:
        with torch.cuda.stream(stream):
            if args.workload == "ivfpq":  # the rank's slice of the batch on its lists
                slices = world // list_shards
                per = (NQ + slices - 1) // slices
                s0 = (rank // list_shards) * per
                ix.search_batch(dq[s0:min(NQ, s0 + per)].contiguous(), K, nprobe, refine if list_shards == 1 else 0)
            else:
                ix.search_batch(dq, K)
        local_st = ctx.stats()
        t = torch.tensor([ms, e2e_ms] + [float(x) for x in stages], device=f"cuda:{local}", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, e2e_ms = float(t[0]), float(t[1])
        stages_max = t[2:].cpu().numpy()
    else:
        stages_max = stages
    if rank != 0:
        if world > 1:
            barrier()  # rank 0 may still be checking its result against the unsharded index
            dist.destroy_process_group()
        return

    found = fv.neighbors_from_tensor(out)
    cnt = counts.cpu().numpy().astype(np.uint32)
    if args.big:
        args.no_cpu = True  # the rows never exist on the host; runs at different N are compared by the checksum below
    pk = peaks()
    if args.workload == "ivfpq":
        names = IVF_STAGES if world == 1 else IVF_SHARDED_STAGES if list_shards == world else IVF_GRID_STAGES
    elif args.workload == "flat":
        names = FLAT_SHARDED_STAGES if world > 1 else FLAT_STAGES
    else:
        names = ["beam search", "keys -> neighbours"]
    line = {
        "metric": METRIC, "value": NQ / (ms * 1e-3), "unit": "queries/s",
        "n_gpus": world, "steps": args.steps, "warmup": n_warm, "ms_per_step": ms,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "data": "synthetic",
        "dtype": "f32" if args.workload == "hnsw" else "f16 operands, f32 accumulate, f32 exact re-score",
        "config": workload_config(args.workload, world, nprobe, refine, list_shards),
        "e2e": {"value": NQ / (e2e_ms * 1e-3), "unit": "queries/s", "h2d_bytes_per_step": int((q_hi - q_lo) * DIM * 4),
                "d2h_bytes_per_step": int(h_out.numel() * 4), "ms_per_step": e2e_ms,
                "bytes_note": "per rank: the queries the rank searches in, all results out"},
        "gpu_launches": int(steady_launches), "clocks": clocks, "build_s": build_s,
        "stage_ms": {n: round(float(x), 4) for n, x in zip(names, stages_max)},
        "stage_ms_note": "device time per stage of one step (CUDA events on the library's stream), max over ranks",
    }
    if local_st is not None:
        lnames = IVF_STAGES if args.workload == "ivfpq" else FLAT_STAGES
        line["local_search_stage_ms"] = {n: round(float(x), 4) for n, x in zip(lnames, local_st["stage_ms"])}
    # ---- roofline of the dominant kernel (per launch = per step; durations from CUDA events on the library's stream)
    src = local_st if local_st is not None else last
    if args.workload == "ivfpq":
        kms = float(local_st["stage_ms"][3]) if local_st is not None else float(stages[3])
        rows, rows_list, surv = src["rows_scanned"], src["rows_list_scan"], src["dist_evals"]
        # The dominant kernel is the scan (stage 3).  Its algorithmic work is the code bytes of every (query, probed
        # list) pair: rows * m.  The per-query kernel and the table scan read them as such.  The tensor-core pass
        # does the same work as a GEMM over 16-bit codeword rows that are read once per 256-query tile, not once per
        # pair: the byte figure then measures equivalent scan throughput and can pass the HBM peak; the tensor
        # figures beside it say how busy the tensor cores are.
        tensor = rows_list > 0 and surv > 0
        alg = (rows_list if rows_list else rows) * IVF["m"]
        ach = alg / (kms * 1e-3) / 1e9
        if tensor:
            # The tensor-core pass scores every (pair, row) as a 16-bit GEMM: 2 * rows * d flop of useful work per
            # launch (padding of the 256 x 256 tiles not counted).  The code bytes of a list are not read per pair
            # by this kernel, so its bound is the tensor pipe, not HBM; the equivalent scan rate (code bytes of all
            # pairs / kernel time) is given beside it for comparison with the scanning kernels.
            flops = 2.0 * rows_list * DIM
            tf = flops / (kms * 1e-3) / 1e12
            line["roofline"] = {"kernel": "gemm_topk_kernel (task mode)", "bound": "tensor", "achieved": tf, "peak": pk["tflops"],
                                "unit": "TFLOP/s", "frac": tf / pk["tflops"], "traffic": None, "peak_source": pk["source"],
                                "algorithmic_flops_per_launch": flops, "kernel_ms": kms,
                                "frac_of_sustained_peak": tf / pk["tflops_sustained"],
                                "survivors_rescored": int(surv), "equivalent_scan_gbs": ach,
                                "equivalent_scan_frac_of_hbm_peak": ach / pk["hbm_gbs"], "algorithmic_bytes_per_launch": int(alg),
                                "equivalent_scan_note": "code bytes of all (query, probe) pairs / kernel time: what a kernel that "
                                                        "reads the codes per pair would have to sustain; not DRAM traffic"}
        else:
            line["roofline"] = {"kernel": "ivfpq_list_scan_kernel" if rows_list else "ivfpq_scan_kernel",
                                "bound": "hbm", "achieved": ach, "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": ach / pk["hbm_gbs"],
                                "traffic": None, "peak_source": pk["source"], "algorithmic_bytes_per_launch": int(alg),
                                "kernel_ms": kms}
    elif args.workload == "flat":
        kms = float(src["stage_ms"][2])
        alg = 2.0 * NQ * (hi - lo) * DIM
        ach = alg / (kms * 1e-3) / 1e12
        line["roofline"] = {"kernel": "gemm_topk_kernel", "bound": "tensor", "achieved": ach, "peak": pk["tflops"],
                            "unit": "TFLOP/s", "frac": ach / pk["tflops"], "traffic": None, "peak_source": pk["source"],
                            "algorithmic_flops_per_launch": alg, "kernel_ms": kms,
                            "frac_of_sustained_peak": ach / pk["tflops_sustained"]}
    else:
        kms = float(stages[0])
        alg = last["dist_evals"] * DIM * 4 + last["expansions"] * (2 * HNSW["m"] + 1) * 4
        ach = alg / (kms * 1e-3) / 1e9
        line["roofline"] = {"kernel": "hnsw_search_kernel", "bound": "hbm", "achieved": ach, "peak": pk["hbm_gbs"],
                            "unit": "GB/s", "frac": ach / pk["hbm_gbs"], "traffic": None, "peak_source": pk["source"],
                            "algorithmic_bytes_per_launch": int(alg), "kernel_ms": kms}
    line["result_checksum"] = int(found["id"].astype(np.uint64).sum() % (1 << 61))  # equal across GPU counts
    if args.big:
        line["config"]["workload"] = ("BASELINE configs[4], 50M x 128: " + ("exact L2 k-NN, row ranges" if args.workload == "flat" else
                                     "IVF-PQ nlist=16384 M=16x8bit nprobe=32 refine=0, sharded by list"))
        line["config"]["l2_note"] = "inputs exceed L2 by orders of magnitude"
        if args.workload == "ivfpq":
            line["config"].update({k: BIG_IVF[k] for k in ("nlist", "m", "nprobe")}, refine=0)
    # DRAM traffic of the dominant kernel: from the committed ncu capture of a smaller case, scaled to this launch
    try:
        if args.big:
            raise KeyError("no capture at this size")
        with open(os.path.join(ROOT, "profiles", "ncu_traffic.json")) as f:
            tr = json.load(f)[line["roofline"]["kernel"]]
        nq_local = NQ
        if args.workload == "ivfpq" and world > 1:
            nq_local = (NQ + world // list_shards - 1) // (world // list_shards)
        if "bytes_per_launch" in tr:
            line["roofline"]["traffic"] = tr["bytes_per_launch"] * (hi - lo) / 1_000_000 + tr.get("bytes_per_query", 0.0) * nq_local
        else:
            line["roofline"]["traffic"] = tr["bytes_per_query"] * nq_local / (list_shards if args.workload == "ivfpq" and world > 1 else 1)
        line["roofline"]["traffic_note"] = "ncu dram bytes of a smaller capture, scaled: " + tr["scaling"]
    except Exception:
        pass
    # ---- parity against the CPU oracle, recall against exact search, the CPU baseline: on bounded samples
    if not args.no_cpu:
        from oracle import oracle

        oracle.build()
        threads = oracle.cores()
        nsub = min(NQ, 2000)
        if args.workload == "ivfpq":
            if world > 1 and list_shards == 1:  # every rank holds the whole index: the plain search is the check
                blob = ix.save()
                ref_out, ref_cnt = ix.search_batch(dq, K, nprobe, refine)
                line["sharded_equals_unsharded"] = bool(torch.equal(ref_out, out) and torch.equal(ref_cnt, counts))
            elif world > 1:  # the shards cannot be saved as one file: the same index once more, unsharded, on this rank
                full = fv.IvfPq.load(ctx, empty_blob)
                full.add(base)
                blob = full.save()
                ref_out, ref_cnt = full.search_batch(dq, K, nprobe, refine)
                line["sharded_equals_unsharded"] = bool(torch.equal(ref_out, out) and torch.equal(ref_cnt, counts))
                del full
            else:
                blob = ix.save()
            oix = oracle.IvfPq.load(blob)  # the same trained index, byte for byte
            del blob
            search = lambda q, t: oix.search_batch(q, K, nprobe, refine, t)[:2]
            sample = "same index (loaded from the GPU-built FLIVFPQ1 bytes)"
        elif args.workload == "flat":
            nsub = 64
            full_base = base if world == 1 else fv.datagen(0, 1, N_BASE, DIM, CLUSTERS)
            oix = oracle.FlatIndex(oracle.L2, DIM)
            oix.add(full_base)
            search = lambda q, t: oix.search_batch(q, K, t)[:2]
            sample = "brute force over all rows"
        else:
            oix = oracle.Hnsw.load(ix.save())
            search = lambda q, t: oix.search_batch(q, K, HNSW["ef"], t)[:2]
            sample = "same graph (loaded from the FLHNSW01 bytes)"
        want, wc = search(queries[:nsub], threads)
        same_ids = int((found[:nsub]["id"] == want["id"]).all(axis=1).sum())
        line["parity_sample"] = {"queries": nsub, "identical_id_rows": same_ids,
                                 "bit_equal_distances": bool((found[:nsub]["distance"].view(np.uint32) ==
                                                              want["distance"].view(np.uint32)).all())}
        if world == 1:
            # the timed CPU baseline: about 10 s of CPU work with the reference's protocol
            if args.workload == "flat":
                t0 = time.perf_counter()
                search(queries[:nsub], threads)
                est = nsub / (time.perf_counter() - t0)
                nt = int(min(NQ, max(nsub, est * 10.0)))
                t0 = time.perf_counter()
                search(queries[:nt], threads)
                dt = time.perf_counter() - t0
                n1 = max(8, min(nt, int(est / max(threads, 1) * 3.0)))
                t0 = time.perf_counter()
                search(queries[:n1], 1)
                d1 = time.perf_counter() - t0
                line["cpu_baseline"] = {"value": nt / dt, "unit": "queries/s", "cores": threads, "kind": "port",
                                        "sample": f"first {nt} of {NQ} queries, {sample}", "seconds": dt + d1,
                                        "qps_1": n1 / d1, "qps_1_note": f"one thread, first {n1} queries"}
            else:
                r = timed_cpu(search, queries, threads)
                line["cpu_baseline"] = {"value": r["qps_n"], "unit": "queries/s", "cores": threads, "kind": "port",
                                        "sample": f"{r['passes']} passes over all {NQ} queries, {sample}", "seconds": r["seconds"],
                                        "qps_1": r["qps_1"],
                                        "qps_1_note": f"one thread, first {r['single_thread_queries']} queries (the reference's own protocol, src/main.rs:496-507)"}
        else:
            line["cpu_baseline"] = None
        del oix
        # recall@10 against exact search (GPU exact search, itself checked against the oracle in tests/)
        if args.workload == "flat":
            line["recall_at_10"] = 1.0
        else:
            flat = fv.FlatIndex(ctx, fv.Metric.L2, DIM)
            flat.add(base)
            truth, _ = flat.search_batch(queries[:nsub], K)
            line["recall_at_10"] = fv.recall(found[:nsub], cnt[:nsub], truth["id"], K)
            del flat
        if world == 1 and args.workload == "ivfpq" and not args.no_also and N_BASE == 1_000_000 and NQ == 10_000:
            line["also"] = also_section(fv, oracle, ctx, stream, ix, base, queries, dq, pk, nprobe, refine, threads)
    else:
        line["cpu_baseline"] = None
    print(json.dumps(line), flush=True)
    if world > 1:
        barrier()
        dist.destroy_process_group()


def main():
    global NQ, N_BASE
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="ivfpq", choices=["ivfpq", "flat", "hnsw"])
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU oracle legs (parity sample, recall, CPU baseline, also)")
    ap.add_argument("--no-also", action="store_true", help="skip the other configurations (N=1 only)")
    ap.add_argument("--nq", type=int, default=NQ, help="queries per step (smaller = a profiling-sized case)")
    ap.add_argument("--n", type=int, default=None, help="base rows (smaller = a profiling-sized case)")
    ap.add_argument("--scan-mode", type=int, default=0,
                    help="IVF-PQ scan: 0 automatic, 1 per-query kernel, 2 list-major table scan, 3 list-major tensor-core pass")
    ap.add_argument("--nprobe", type=int, default=0, help="IVF-PQ: probed lists (default: the benchmark's 64)")
    ap.add_argument("--refine", type=int, default=None, help="IVF-PQ: re-rank factor (default: the benchmark's 10)")
    ap.add_argument("--list-shards", type=int, default=0,
                    help="IVF-PQ at N > 1: list shards L of the L x (N / L) grid (default 1: query slices only; N: list shards only)")
    ap.add_argument("--big", action="store_true", help="BASELINE configs[4]: 50M rows, 4096 clusters, sharded")
    args = ap.parse_args()
    global CLUSTERS
    NQ = args.nq
    if args.big:
        N_BASE, CLUSTERS = 50_000_000, 4096
    if args.n:
        N_BASE = args.n
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
