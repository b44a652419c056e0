#!/usr/bin/env python
"""Benchmark of the vector-search hot path: queries/s at recall@10 on N=1M, d=128, k=10.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload ivfpq|flat|hnsw] [--impl reference]

One "step" is one search_batch over a 10,000-query batch (seeded synthetic data with the shape and
value range of SIFT1M, which cannot be shipped: clipped-integer Gaussian mixture).  The default
workload is the IVF-PQ configuration (nlist=1024, M=16x8 bit, trained on a 100,000-row sample,
nprobe=64, refine=10); --workload flat is exact L2 search on the same data, --workload hnsw the
graph index.  With N>1 GPUs (one process per GPU under torchrun) the base rows are sharded
over the ranks (strong scaling: the 1M rows are fixed) -- contiguous row ranges for exact search, inverted
lists for IVF-PQ -- every rank searches its part and the per-rank candidates are all-gathered over NCCL and
merged by a kernel of this library.

The line printed by rank 0 carries: `value` (device-resident queries), `e2e` (host queries in pinned
memory, copies inside the timed region), `roofline` of the dominant kernel (algorithmic bytes or
flops per launch over its CUDA-event duration), `cpu_baseline` (the CPU oracle timed on the host
cores on a bounded sample) and the sampled GPU clocks.

--impl reference times the CPU restatement of the reference's algorithm (the reference is Rust and
cannot be built here) on the host cores with all threads, same data and configuration.
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


def peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            p = json.load(f)
        return {"hbm_gbs": float(p["hbm_gbs"]), "tflops": float(p["bf16_tflops"]),
                "tflops_sustained": float(p.get("bf16_tflops_sustained", p["bf16_tflops"])), "source": "measured"}
    except Exception:
        return {"hbm_gbs": 6650.0, "tflops": 1590.0, "tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons of one GPU with nvidia-smi while a region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.lines, self.proc, self.thread = index, [], None, None

    def start(self):
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


def make_data(rank_rows: tuple[int, int]):
    import ferrolm_b200 as fv

    lo, hi = rank_rows
    base = fv.datagen(0, 1, hi - lo, DIM, CLUSTERS, first_row=lo)
    queries = fv.datagen(0, 2, NQ, DIM, CLUSTERS)
    return base, queries


# ----------------------------------------------------------------------------------------------- reference arm
def run_reference(args):
    """The CPU restatement of the reference (oracle/), all host threads, same data and configuration."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import oracle

    oracle.build()
    import ferrolm_b200 as fv  # host-side data generator only; no GPU call is made on this arm

    threads = oracle.cores()
    base, queries = make_data((0, N_BASE))
    sample = None
    t0 = time.perf_counter()
    if args.workload == "ivfpq":
        learn = fv.datagen(0, 3, IVF["learn"], DIM, CLUSTERS)
        ix = oracle.IvfPq.train(oracle.L2, DIM, learn, IVF["nlist"], IVF["m"], IVF["iters"], True, 1, threads)
        ix.add(base, threads)
        nqs = NQ
        step = lambda: ix.search_batch(queries[:nqs], K, IVF["nprobe"], IVF["refine"], threads)
        sample = f"all {nqs} queries per step, index built by the CPU oracle"
    elif args.workload == "flat":
        ix = oracle.FlatIndex(oracle.L2, DIM)
        ix.add(base)
        nqs = min(NQ, 64 * max(1, threads // 8))
        step = lambda: ix.search_batch(queries[:nqs], K, threads)
        sample = f"first {nqs} of {NQ} queries per step (a full batch is minutes of CPU time)"
    else:
        ix = oracle.Hnsw.build(oracle.L2, DIM, base, HNSW["m"], HNSW["ef_construction"], 1, threads)
        nqs = NQ
        step = lambda: ix.search_batch(queries[:nqs], K, HNSW["ef"], threads)
        sample = f"all {nqs} queries per step, graph built by the CPU oracle with {threads} threads"
    build_s = time.perf_counter() - t0
    for _ in range(args.warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    dt = (time.perf_counter() - t0) / args.steps
    qps = nqs / dt
    line = {
        "impl": "reference", "metric": "queries/s at recall@10 (N=1M, d=128, k=10)", "value": qps, "unit": "queries/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(args.workload, 1),
        "cpu_baseline": {"value": qps, "unit": "queries/s", "cores": threads, "kind": "port", "sample": sample,
                         "build_s": build_s},
        "e2e": {"value": qps, "unit": "queries/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def workload_config(workload: str, n_gpus: int) -> dict:
    cfg = {"n": N_BASE, "d": DIM, "nq": NQ, "k": K, "distribution": f"clipped-integer Gaussian mixture, {CLUSTERS} clusters",
           "sharding": (f"{'inverted lists' if workload == 'ivfpq' else 'row ranges'} over {n_gpus} GPUs, per-shard candidates "
                        "all-gathered (NCCL) and merged") if n_gpus > 1 else "single GPU",
           "l2_note": "inputs exceed L2: 1M x 128 f32 rows (512 MB) plus 16 MB of codes are re-read each step"}
    if workload == "ivfpq":
        cfg.update({"workload": "IVF-PQ L2 search, nlist=1024, M=16x8bit, nprobe=64, refine=10 (BASELINE configs[2])",
                    **{k: IVF[k] for k in ("nlist", "m", "nprobe", "refine")}})
    elif workload == "flat":
        cfg.update({"workload": "exact L2 k-NN, tensor-core front end + exact re-rank (BASELINE configs[0] shape at N=1M)"})
    else:
        cfg.update({"workload": "HNSW L2 search, M=16, efC=200, efSearch=64 (BASELINE configs[3])", **HNSW})
    return cfg


# ----------------------------------------------------------------------------------------------- GPU arm
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

    from ferrolm_b200.sharding import ShardedSearch, row_range

    t_build = time.perf_counter()
    refine, nprobe = 0, 0
    if args.big:
        # BASELINE configs[4]: 50M x 128, 4096 clusters; rows are generated on the GPU in chunks and never
        # exist on the host.  exact search: row ranges; IVF-PQ: nlist=16384, nprobe=32, sharded by list.
        queries = fv.datagen(0, 2, NQ, DIM, CLUSTERS)
        base = None

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
        base, queries = make_data((lo, hi))
        learn = fv.datagen(0, 3, IVF["learn"], DIM, CLUSTERS)
        ix = fv.IvfPq.train(ctx, fv.Metric.L2, DIM, learn, fv.IvfPqParams(IVF["nlist"], IVF["m"], IVF["iters"], True, 1))
        ix.set_shard(rank, world)
        ix.add(base)
        ix.set_scan_mode(args.scan_mode)
        refine, nprobe = IVF["refine"] if args.refine is None else args.refine, args.nprobe or IVF["nprobe"]
        searcher = ShardedSearch(ctx, ix, "ivfpq", world)
    elif args.workload == "flat":
        lo, hi = row_range(rank, world, N_BASE)  # contiguous row shards
        base, queries = make_data((lo, hi))
        ix = fv.FlatIndex(ctx, fv.Metric.L2, DIM)
        ix.set_id_base(lo)
        ix.add(base)
        searcher = ShardedSearch(ctx, ix, "flat", world)
    else:
        if world > 1:
            raise SystemExit("hnsw: replicas only (one graph); run with --gpus 1")
        lo, hi = 0, N_BASE
        base, queries = make_data((lo, hi))
        ix = fv.Hnsw.build(ctx, fv.Metric.L2, DIM, base, fv.HnswParams(HNSW["m"], HNSW["ef_construction"], 1),
                           threads=os.cpu_count() or 1)
        searcher = None
    build_s = time.perf_counter() - t_build

    dq = torch.from_numpy(queries).cuda()
    hq = torch.from_numpy(queries).pin_memory()
    h_out = torch.empty((NQ, K, 2), dtype=torch.int32).pin_memory()
    launches = [0]
    stage_sum = np.zeros(8)
    rows_scanned = [0, 0]
    work = [0, 0]

    def step(q):
        """One search_batch of the whole (possibly sharded) index on device-resident queries."""
        with torch.cuda.stream(stream):
            if searcher is None:
                r = ix.search_batch(q, K, HNSW["ef"])
            else:
                r = searcher.search_batch(q, K, nprobe, refine)
        st = ctx.stats()  # the merge kernels add to the launch count and leave the search's stage times in place
        launches[0] += st["launches"]
        stage_sum[:] += np.array(st["stage_ms"])
        rows_scanned[0], rows_scanned[1] = st["rows_scanned"], st["rows_list_scan"]
        work[0], work[1] = st["dist_evals"], st["expansions"]
        return r[0], r[1]

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-resident timing (value)
    sampler = ClockSampler(local)
    sampler.start()
    for _ in range(max(args.warmup, 3)):
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
    # ---- end to end: host queries (pinned) in, host results out, every step
    for _ in range(2):
        with torch.cuda.stream(stream):
            q = hq.to(f"cuda:{local}", non_blocking=True)
        stream.synchronize()
        o, c = step(q)
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        with torch.cuda.stream(stream):
            q = hq.to(f"cuda:{local}", non_blocking=True)
        stream.synchronize()
        o, c = step(q)
        with torch.cuda.stream(stream):
            h_out.copy_(o, non_blocking=True)
        stream.synchronize()
    barrier()
    e2e_ms = (time.perf_counter() - t0) * 1e3 / args.steps
    clocks = sampler.stop()
    if world > 1:
        t = torch.tensor([ms, e2e_ms], device=f"cuda:{local}", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, e2e_ms = float(t[0]), float(t[1])
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    found = fv.neighbors_from_tensor(out)
    cnt = counts.cpu().numpy().astype(np.uint32)
    if args.big:
        args.no_cpu = True  # the rows never exist on the host; runs at different N are compared by the checksum below
    pk = peaks()
    line = {
        "metric": "queries/s at recall@10 (N=1M, d=128, k=10)", "value": NQ / (ms * 1e-3), "unit": "queries/s",
        "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "data": "synthetic",
        "dtype": "f32" if args.workload != "flat" else "f16 operands, f32 accumulate, f32 exact re-rank",
        "config": workload_config(args.workload, world),
        "e2e": {"value": NQ / (e2e_ms * 1e-3), "unit": "queries/s", "h2d_bytes_per_step": int(hq.numel() * 4),
                "d2h_bytes_per_step": int(h_out.numel() * 4), "ms_per_step": e2e_ms},
        "gpu_launches": int(steady_launches), "clocks": clocks, "build_s": build_s,
        "stage_ms": [round(float(x), 4) for x in stages[:6]],
    }
    # ---- roofline of the dominant kernel (per launch = per step; durations from CUDA events on the library's stream)
    if args.workload == "ivfpq":
        # stages of an IVF-PQ search: 0 coarse cells, 1 query tables + sample pass, 2 pair bucketing, 3 the scan,
        # 4 merge + re-rank, 5 keys -> neighbours.  The dominant kernel is the scan of stage 3: the list-major
        # kernel over the rows it visited (rows_list_scan), or the per-query kernel over all rows.
        kms = float(stages[3])
        list_major = rows_scanned[1] > 0
        alg = (rows_scanned[1] if list_major else rows_scanned[0]) * IVF["m"]  # code bytes that launch has to read
        ach = alg / (kms * 1e-3) / 1e9
        line["roofline"] = {"kernel": "ivfpq_list_scan_kernel" if list_major else "ivfpq_scan_kernel", "bound": "hbm", "achieved": ach, "peak": pk["hbm_gbs"],
                            "unit": "GB/s", "frac": ach / pk["hbm_gbs"], "traffic": None, "peak_source": pk["source"],
                            "algorithmic_bytes_per_launch": int(alg), "kernel_ms": kms}
    elif args.workload == "flat":
        kms = float(stages[2])  # stage 2 = main pass of the tensor-core kernel (0 convert, 1 sample pass, 3 re-rank)
        alg = 2.0 * NQ * (hi - lo) * DIM
        ach = alg / (kms * 1e-3) / 1e12
        line["roofline"] = {"kernel": "gemm_topk_kernel", "bound": "tensor", "achieved": ach, "peak": pk["tflops"],
                            "unit": "TFLOP/s", "frac": ach / pk["tflops"], "traffic": None, "peak_source": pk["source"],
                            "algorithmic_flops_per_launch": alg, "kernel_ms": kms,
                            "frac_of_sustained_peak": ach / pk["tflops_sustained"]}
    else:
        kms = float(stages[0])
        alg = work[0] * DIM * 4 + work[1] * (2 * HNSW["m"] + 1) * 4
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
            tr = json.load(f)[args.workload]
        if args.workload == "flat":
            line["roofline"]["traffic"] = tr["bytes_per_launch"] * (hi - lo) / 1_000_000
        else:
            line["roofline"]["traffic"] = tr["bytes_per_query"] * NQ
        line["roofline"]["traffic_note"] = "ncu dram bytes of a smaller capture, scaled: " + tr["scaling"]
    except Exception:
        pass
    # ---- CPU baseline (the oracle on the host cores) and recall against exact search, on a bounded sample
    if world == 1 and not args.no_cpu:
        from oracle import oracle

        oracle.build()
        threads = oracle.cores()
        nsub = min(NQ, 2000)
        t0 = time.perf_counter()
        if args.workload == "ivfpq":
            oix = oracle.IvfPq.load(ix.save())  # the same trained index, byte for byte
            load_s = time.perf_counter() - t0
            t0 = time.perf_counter()
            want, wc = oix.search_batch(queries[:nsub], K, nprobe, refine, threads)
            sample = f"first {nsub} of {NQ} queries, same index (loaded from the GPU-built FLIVFPQ1 bytes)"
        elif args.workload == "flat":
            nsub = 64
            oix = oracle.FlatIndex(oracle.L2, DIM)
            oix.add(base)
            load_s = time.perf_counter() - t0
            t0 = time.perf_counter()
            want, wc = oix.search_batch(queries[:nsub], K, threads)
            sample = f"first {nsub} of {NQ} queries"
        else:
            oix = oracle.Hnsw.load(ix.save())
            load_s = time.perf_counter() - t0
            t0 = time.perf_counter()
            want, wc = oix.search_batch(queries[:nsub], K, HNSW["ef"], threads)
            sample = f"first {nsub} of {NQ} queries, same graph (loaded from the FLHNSW01 bytes)"
        dt = time.perf_counter() - t0
        # the timed sample: about 10 s of CPU work (whole passes over the query batch, or a longer prefix of it for
        # exact search); the pass above doubles as the parity check and as a rate estimate
        est = nsub / dt
        if args.workload == "flat":
            nt = int(min(NQ, max(nsub, est * 10.0)))
            t0 = time.perf_counter()
            oix.search_batch(queries[:nt], K, threads)
            cpu_dt, cpu_n = time.perf_counter() - t0, nt
            sample = f"first {nt} of {NQ} queries"
        else:
            passes = int(max(1, min(64, round(est * 10.0 / NQ))))
            t0 = time.perf_counter()
            for _ in range(passes):
                if args.workload == "ivfpq":
                    oix.search_batch(queries, K, nprobe, refine, threads)
                else:
                    oix.search_batch(queries, K, HNSW["ef"], threads)
            cpu_dt, cpu_n = time.perf_counter() - t0, passes * NQ
            sample = f"{passes} passes over all {NQ} queries; " + sample.split(", ", 1)[1]
        line["cpu_baseline"] = {"value": cpu_n / cpu_dt, "unit": "queries/s", "cores": threads, "kind": "port",
                                "sample": sample, "seconds": cpu_dt}
        same_ids = int((found[:nsub]["id"] == want["id"]).all(axis=1).sum())
        line["parity_sample"] = {"queries": nsub, "identical_id_rows": same_ids,
                                 "bit_equal_distances": bool((found[:nsub]["distance"].view(np.uint32) ==
                                                              want["distance"].view(np.uint32)).all())}
        # recall@10 against exact search (GPU exact search, itself checked against the oracle in tests/)
        flat = fv.FlatIndex(ctx, fv.Metric.L2, DIM)
        flat.add(base)
        truth, _ = flat.search_batch(queries[:nsub], K)
        line["config"]["recall_at_10"] = fv.recall(found[:nsub], cnt[:nsub], truth["id"], K)
        if args.workload != "flat":
            # for context, exact search (recall 1.0) on the same data and query batch, same timing method
            for _ in range(3):
                flat.search_batch(dq, K)
            ms_f, gemm_ms = [], []
            for _ in range(10):
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record(stream)
                flat.search_batch(dq, K)
                e1.record(stream)
                stream.synchronize()
                ms_f.append(e0.elapsed_time(e1))
                gemm_ms.append(ctx.stats()["stage_ms"][2])
            tf = 2.0 * NQ * N_BASE * DIM / (np.mean(gemm_ms) * 1e-3) / 1e12
            line["also"] = {"exact_search_same_data": {
                "value": NQ / (np.mean(ms_f) * 1e-3), "unit": "queries/s", "recall_at_10": 1.0,
                "ms_per_step": float(np.mean(ms_f)), "gemm_topk_kernel_ms": float(np.mean(gemm_ms)),
                "tensor_tflops": tf, "frac_of_measured_peak": tf / pk["tflops"]}}
    else:
        line["cpu_baseline"] = None
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main():
    global NQ, N_BASE
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="ivfpq", choices=["ivfpq", "flat", "hnsw"])
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--nq", type=int, default=NQ, help="queries per step (smaller = a profiling-sized case)")
    ap.add_argument("--n", type=int, default=None, help="base rows (smaller = a profiling-sized case)")
    ap.add_argument("--scan-mode", type=int, default=0, help="IVF-PQ scan: 0 automatic, 1 per-query kernel, 2 list-major")
    ap.add_argument("--nprobe", type=int, default=0, help="IVF-PQ: probed lists (default: the benchmark's 64)")
    ap.add_argument("--refine", type=int, default=None, help="IVF-PQ: re-rank factor (default: the benchmark's 10)")
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
