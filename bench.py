"""Benchmark of the exact 10-NN search path: QPS on 10,000,000 x 128 uint8 vectors, 10,000 queries, k = 10, L2.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

A step is one search of all queries (every stage: anchor pass, threshold, screen, exact fp64 verification, top-k,
and for N > 1 the all-gather + merge of the per-rank lists); for N > 1 a step repeats that search `--searches-per-step`
times (default 4, stated in `config`), so that the timed region stays long enough for a stable number when a search
takes a few milliseconds. Inputs are seeded synthetic Gaussian-mixture rows with the
shape and value range of the reference's benchmark set (which is not available offline). For N > 1 (launched with
torch.distributed.run, one rank per GPU) the 10 M rows are split into N contiguous shards: total work is fixed
(strong scaling). Rank 0 prints one JSON line.

--impl reference times the reference's fp64 exhaustive CPU check (restated in oracle/) on the host cores over a
bounded sample of the same workload.
"""

import argparse
import json
import os
import sys
import threading
import time

import numpy as np
import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "exact 10-NN QPS, 10Mx128 u8"
# DRAM bytes per stored row of a SCREEN launch: 1.318 GB read + 0.018 GB written, measured by ncu over 10 M rows of 128
# bytes and 10 000 queries (the launch passes every query panel over one chunk of rows while the chunk is in L2, so the
# codes come from DRAM once)
TRAFFIC_PER_ROW = 1.336e9 / 10_000_000
N_BASE, N_QUERIES, DIM, K = 10_000_000, 10_000, 128, 10


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"bf16_burst": p["bf16_tflops"], "bf16_sustained": p["bf16_tflops_sustained"], "hbm_gbs": p["hbm_gbs"],
                "source": "measured"}
    return {"bf16_burst": 1590.0, "bf16_sustained": 1400.0, "hbm_gbs": 6650.0, "source": "fallback"}


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons of one GPU through NVML (read-only) while the timed region runs."""

    def __init__(self, device):
        super().__init__(daemon=True)
        self.device, self.samples, self.reasons, self.max_mhz = device, [], set(), None
        self._halt = threading.Event()
        self.ok = False
        try:
            import pynvml

            self.nv = pynvml
            pynvml.nvmlInit()
            try:
                uuid = str(torch.cuda.get_device_properties(device).uuid)
                self.h = pynvml.nvmlDeviceGetHandleByUUID(("GPU-" + uuid).encode())
            except Exception:
                self.h = pynvml.nvmlDeviceGetHandleByIndex(device)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
            self.ok = True
        except Exception:
            self.ok = False

    def run(self):
        if not self.ok:
            return
        nv = self.nv
        names = {
            getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4): "sw_power_cap",
            getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8): "hw_slowdown",
            getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20): "sw_thermal_slowdown",
            getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40): "hw_thermal_slowdown",
            getattr(nv, "nvmlClocksEventReasonHwPowerBrakeSlowdown", 0x80): "hw_power_brake_slowdown",
        }
        while not self._halt.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                try:
                    mask = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                except Exception:
                    mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for bit, name in names.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(0.05)

    def reset(self):
        """Forgets what was seen so far: called where the timed region begins (the thread is started earlier, during
        the warm-up, because the first NVML queries of a process take long and hold up CUDA calls meanwhile)."""
        self.samples, self.reasons = [], set()

    def stop(self):
        self._halt.set()
        if self.is_alive():
            self.join()
        med = float(np.median(self.samples)) if self.samples else None
        return {"sm_mhz": med, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": len(self.samples)}


def config_of(args):
    """The `config` object of the JSON line; both arms print the same one."""
    per_step = args.searches_per_step or (1 if args.gpus == 1 else 4)
    return {
        "workload": f"{args.n_base}x{DIM} uint8 Gaussian mixture (1000 centres in [20,235], sigma 18), "
                    f"{args.n_queries} queries, k={K}, L2, {args.gpus} row shard(s)",
        "batch": args.batch, "anchor_stride": args.anchor_stride, "searches_per_step": per_step,
        "share_thresholds": bool(args.share_thresholds) and args.gpus > 1,
        # searches of a step that are between search_begin and search_end at once (the host prepares one while the
        # device works on the other); every search is complete and checked like the others
        "searches_in_flight": max(1, min(args.pipeline, 2)) if args.gpus > 1 else 1,
        "l2_policy": "inputs exceed L2: every step streams the whole shard (>= 160 MB) from HBM",
    }


def measure_i8_peak(iters=5):
    """int8 tensor-pipe rate of this GPU with the screen's own tiling: the pass's TMA + tcgen05.mma stream (M128 x
    N256 x K32 instructions, uint8 operands, int32 accumulators in TMEM) with no epilogue, over 2048 queries x 1 M
    rows, best of `iters` (CUDA events around the launch, inside the library). TOP/s."""
    import ctypes

    from libcertex_b200 import _lib

    L, res = _lib.lib(), _lib.resources()
    nq, n, cl = 2048, 1_000_000, 128
    g = torch.Generator(device="cuda").manual_seed(11)
    q = torch.randint(0, 256, (nq, cl), generator=g, device="cuda", dtype=torch.uint8)
    x = torch.randint(0, 256, (n, cl), generator=g, device="cuda", dtype=torch.uint8)
    init = torch.zeros((-(-n // 256) * 256,), dtype=torch.int32, device="cuda")
    dummy = torch.zeros((nq,), dtype=torch.int32, device="cuda")
    ms, best = ctypes.c_float(), None
    for _ in range(iters):
        _lib.check(L.certexB200ScreenRaw(res, q.data_ptr(), nq, x.data_ptr(), n, cl, 0, init.data_ptr(), 2,
                                         dummy.data_ptr(), dummy.data_ptr(), 8, dummy.data_ptr(), dummy.data_ptr(), 1,
                                         ctypes.byref(ms)))
        best = ms.value if best is None else min(best, ms.value)
    return 2.0 * nq * n * cl / (best / 1e3) / 1e12


def cpu_baseline(xb_host, xq_host, target_seconds=15.0):
    """The oracle (a restatement of the reference's fp64 exhaustive check) on all host cores, on the first queries of
    the workload; the sample is sized from a short probe so that it takes roughly `target_seconds`. Also returns the
    sample's answers (number of queries, ids, fp64 scores) for the parity check."""
    from oracle import oracle

    cores = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    t0 = time.perf_counter()
    oracle.knn(xb_host, xq_host[:8], K, "l2", threads=cores)
    probe = time.perf_counter() - t0
    nqs = int(max(8, min(xq_host.shape[0], 8 * target_seconds / max(probe, 1e-3))))
    t0 = time.perf_counter()
    ids, scores = oracle.knn(xb_host, xq_host[:nqs], K, "l2", threads=cores)
    dt = time.perf_counter() - t0
    return {"value": nqs / dt, "unit": "queries/s", "cores": int(oracle.knn.threads_used), "kind": "port",
            "sample": f"first {nqs} of {xq_host.shape[0]} queries against all {xb_host.shape[0]} rows, {dt:.1f} s"}, \
        (np.arange(nqs), ids, scores)


def run_reference(args):
    """CPU arm: rank 0 only; every step is a bounded sample of the workload."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from libcertex_b200 import synthetic
    from oracle import oracle

    dev = "cuda" if torch.cuda.is_available() else "cpu"
    n_base = args.n_base
    xb = synthetic.mixture_u8(n_base, seed=0, device=dev).cpu().numpy()
    xq = synthetic.mixture_u8(args.n_queries, seed=1, device=dev).cpu().numpy()
    cores = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    # every host core, also under a launcher that sets OMP_NUM_THREADS=1 for its ranks (the other ranks do nothing)
    oracle.knn(xb, xq[:4], K, "l2", threads=cores)
    t0 = time.perf_counter()
    oracle.knn(xb, xq[:8], K, "l2", threads=cores)
    per_query = (time.perf_counter() - t0) / 8
    budget = 150.0 / max(args.steps + args.warmup, 1)  # seconds per step so that the whole run takes a few minutes
    nqs = int(max(4, min(args.n_queries, budget / per_query)))
    for _ in range(args.warmup):
        oracle.knn(xb, xq[:nqs], K, "l2", threads=cores)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        oracle.knn(xb, xq[:nqs], K, "l2", threads=cores)
    dt = time.perf_counter() - t0
    qps = nqs * args.steps / dt
    cores = int(oracle.knn.threads_used)
    sample = f"{nqs} of {args.n_queries} queries per step against all {n_base} rows (fp64 exhaustive, OpenMP)"
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": qps, "unit": "queries/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1000 * dt / args.steps, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f64", "data": "synthetic",
        "config": config_of(args),
        "cpu_baseline": {"value": qps, "unit": "queries/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": qps, "unit": "queries/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=40)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--n-base", type=int, default=N_BASE)
    ap.add_argument("--n-queries", type=int, default=N_QUERIES)
    ap.add_argument("--batch", type=int, default=10240, help="queries that share one pass over the stored rows")
    ap.add_argument("--anchor-stride", type=int, default=16)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--searches-per-step", type=int, default=0,
                    help="searches of all queries per step (default: 1 on one GPU, 4 on several)")
    ap.add_argument("--pipeline", type=int, default=2,
                    help="N > 1: searches of a step between search_begin and search_end at once (1 or 2)")
    ap.add_argument("--parity-queries", type=int, default=16, help="queries checked against the CPU oracle at N > 1")
    ap.add_argument("--share-thresholds", type=int, default=1,
                    help="N > 1: the shards screen with the tightest threshold any of them found (one all-reduce per "
                         "batch, the first round of the reference's sharded search); 0: every shard with its own")
    ap.add_argument("--shard-parity", type=int, default=0,
                    help="sets too large for one host copy (the 500 M-row configuration): every rank checks the local "
                         "top-k of this many queries against the CPU oracle over its own shard, streamed in chunks; "
                         "replaces the check over all rows")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.impl == "reference":
        return run_reference(args)

    import torch.distributed as dist

    import libcertex_b200 as certex
    from libcertex_b200 import distributed, synthetic

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    assert world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run"
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))

    n_base, nq = args.n_base, args.n_queries
    per_step = args.searches_per_step or (1 if world == 1 else 4)
    lo, hi = distributed.shard_bounds(n_base, world, rank)
    xb = synthetic.mixture_u8(hi - lo, seed=0, row0=lo)
    xq = synthetic.mixture_u8(nq, seed=1)
    if world > 1:
        index = distributed.DistributedIndex(DIM, anchor_stride=args.anchor_stride,
                                             share_thresholds=bool(args.share_thresholds)).add_shard(xb, lo)
    else:
        index = certex.Index(DIM, anchor_stride=args.anchor_stride)
        index.add(xb)
    search = lambda q, **kw: index.search(q, k=K, batch=args.batch, **kw)  # noqa: E731
    depth = max(1, min(args.pipeline, 2)) if world > 1 else 1

    def run_step(make_queries, done):
        """One step: per_step searches. On several GPUs up to `depth` of them are between search_begin and search_end,
        so that the host prepares a search while the device works on the one before; done(answer) takes every answer."""
        if depth == 1:
            for _ in range(per_step):
                out = search(make_queries())
                done(out)
            return out
        tickets = []
        for _ in range(per_step):
            tickets.append(index.search_begin(make_queries(), k=K, batch=args.batch))
            if len(tickets) == depth:
                out = index.search_end(tickets.pop(0))
                done(out)
        while tickets:
            out = index.search_end(tickets.pop(0))
            done(out)
        return out
    del xb
    torch.cuda.synchronize()
    i8_peak = measure_i8_peak() if rank == 0 else None  # a few ms of the screen's own MMA stream, before the timed region

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps):
        """Device time of `steps` steps of `per_step` calls each (CUDA events on the launching stream), max over ranks,
        in ms."""
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        e0.record()
        for _ in range(steps):
            out = fn()
        e1.record()
        barrier()
        ms = torch.tensor([e0.elapsed_time(e1)], device="cuda")
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item()), out

    # ---- device-resident inputs
    sampler = ClockSampler(local)
    sampler.start()
    # the warm-up steps run exactly what the timed region runs (statistics on, the same events and barriers), so that
    # whatever the process sets up on first use (event pools, NVML) is set up before the clock starts
    with certex.search_stats():
        for _ in range(args.warmup):
            timed(lambda: run_step(lambda: xq, lambda out: None), 1)
    sampler.reset()
    with certex.search_stats() as st:
        ms, (D, I) = timed(lambda: run_step(lambda: xq, lambda out: None), args.steps)
    clocks = sampler.stop()
    n_searches = args.steps * per_step
    qps = nq * n_searches / (ms / 1000)
    # kernels of the library outside the local searches, per sharded search: merge + finish of the merged lists, and the
    # k-th largest of the shards' threshold candidates when thresholds are exchanged (NCCL's own kernels are not counted)
    launches = st.launches + (n_searches if world > 1 else 0) * (3 if args.share_thresholds else 2)

    # ---- end to end through the public API with host buffers: H2D of the queries, search, D2H of ids + distances
    hq = xq.cpu().pin_memory()
    hI = torch.empty((nq, K), dtype=torch.int64).pin_memory()
    hD = torch.empty((nq, K), dtype=torch.float32).pin_memory()

    def copy_back(out):
        hI.copy_(out[1], non_blocking=True)
        hD.copy_(out[0], non_blocking=True)

    def e2e_step():
        return run_step(lambda: hq.to("cuda", non_blocking=True), copy_back)

    for _ in range(2):
        e2e_step()
    ms_e2e, _ = timed(e2e_step, args.steps)
    e2e_qps = nq * n_searches / (ms_e2e / 1000)
    assert torch.equal(hI, I.cpu()), "end-to-end ids differ from the device-resident run"

    # ---- parity, outside the timed regions: the answers of this run against the CPU oracle on all rows
    _, I_all, S_all = search(xq, return_scores=True)
    torch.cuda.synchronize()
    assert torch.equal(I_all, I), "two searches of the same queries returned different ids"

    # ---- per-shard parity for sets that do not fit one host copy: every rank against the oracle over its own rows
    shard_parity = None
    if args.shard_parity > 0:
        from oracle import oracle

        pick_s = np.arange(0, nq, max(1, nq // args.shard_parity))[: args.shard_parity]
        local_index = index.local if world > 1 else index
        _, I_loc, S_loc = local_index.search(xq[torch.from_numpy(pick_s).cuda()].contiguous(), k=K, batch=args.batch,
                                             return_scores=True, id_base=lo)
        cores = max(1, (len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)) // world)
        q_host = xq.cpu().numpy()[pick_s]
        chunk, parts_i, parts_s = 4 * synthetic.CHUNK, [], []
        for off in range(0, hi - lo, chunk):
            rows = synthetic.mixture_u8(min(chunk, hi - lo - off), seed=0, row0=lo + off).cpu().numpy()
            ids_c, sc_c = oracle.knn(rows, q_host, K, "l2", id_base=lo + off, threads=cores)
            parts_i.append(ids_c)
            parts_s.append(sc_c)
        want_i, want_s = oracle.merge(np.stack(parts_i), np.stack(parts_s))
        mine_ok = bool(np.array_equal(I_loc.cpu().numpy(), want_i) and np.array_equal(S_loc.cpu().numpy(), want_s))
        flag = torch.tensor([1 if mine_ok else 0], dtype=torch.int32, device="cuda")
        if world > 1:
            dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        shard_parity = {"queries": int(len(pick_s)), "ranks": world, "every_rank_equal": bool(flag.item()),
                        "against": "CPU oracle over each rank's own shard (streamed in chunks of 4 Mi rows), local ids "
                                   "and fp64 scores bit for bit"}

    if rank == 0:
        pk = peaks()
        shard_rows = hi - lo
        ops = 2.0 * nq * shard_rows * 128  # int8 multiply-adds x 2 of one screen pass set on this rank, per search
        screen_s = st.screen_ms / 1000 / max(n_searches, 1)
        achieved = ops / screen_s / 1e12 if screen_s > 0 else None
        proxy = 2 * pk["bf16_burst"]
        traffic = int(TRAFFIC_PER_ROW * shard_rows * -(-nq // args.batch))  # once per batch of queries
        line = {
            "metric": METRIC, "value": qps, "unit": "queries/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "u8", "data": "synthetic",
            "config": config_of(args),
            "e2e": {"value": e2e_qps, "unit": "queries/s", "h2d_bytes_per_step": int(hq.numel()) * per_step,
                    "d2h_bytes_per_step": int(hI.numel() * 8 + hD.numel() * 4) * per_step,
                    "ms_per_step": ms_e2e / args.steps},
            "gpu_launches": int(launches),
            "clocks": clocks,
            "roofline": {
                "bound": "tensor", "kernel": "screen_i8_kernel (SCREEN pass)", "achieved": achieved, "peak": i8_peak,
                "unit": "TFLOP/s", "frac": None if achieved is None else achieved / i8_peak, "traffic": traffic,
                "peak_measured_i8": i8_peak, "peak_nominal": 4500.0,
                "frac_of_nominal": None if achieved is None else achieved / 4500.0,
                "peak_2x_bf16_burst": proxy,
                "note": "int8 tensor ops (2 x nq x rows x 128) / CUDA-event time of the screen passes on rank 0; peak = "
                        "the int8 rate measured in this run directly before the timed region by the pass's own TMA + "
                        "tcgen05.mma stream without epilogue (M128 x N256 x K32, 2048 queries x 1 M rows, best of 5); "
                        f"peak_2x_bf16_burst = twice the {pk['source']} burst bf16 cuBLAS rate, for comparison only",
                "traffic_note": "DRAM bytes of one SCREEN launch, scaled by rows from the ncu capture of the 10M x 128, "
                                "10000-query launch under profiles/ (codes are read from DRAM once per launch: all "
                                "query panels pass over a chunk of rows while it is in L2)",
                "screen_ms_per_search": st.screen_ms / n_searches, "anchor_ms_per_search": st.anchor_ms / n_searches,
                # device time from the first to the last operation of a search on rank 0 (before the exchange of the
                # shards' lists at N > 1): ms_per_step / searches_per_step minus this is device time not spent in the search
                "span_ms_per_search": st.span_ms / n_searches,
            },
            "stats": {"survivors_per_query": st.survivors / max(st.queries, 1), "dense_queries": st.dense_queries},
        }
        if shard_parity is not None:
            line["parity"] = shard_parity
            print(json.dumps(line))
            ok = shard_parity["every_rank_equal"]
            xb_host = None
        else:
            xb_host = synthetic.mixture_u8(n_base, seed=0).cpu().numpy()
        xq_host = xq.cpu().numpy()
        if xb_host is None:
            pass
        elif world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"], (pick, ids, scores) = cpu_baseline(xb_host, xq_host)
        else:
            from oracle import oracle

            pick = np.arange(0, nq, max(1, nq // max(args.parity_queries, 1)))[: args.parity_queries]
            cores = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
            ids, scores = oracle.knn(xb_host, xq_host[pick], K, "l2", threads=cores)
        if xb_host is not None:
            ids_equal = bool(np.array_equal(I_all[pick].cpu().numpy(), ids))
            scores_equal = bool(np.array_equal(S_all[pick].cpu().numpy(), scores))
            line["parity"] = {"queries": int(len(pick)), "ids_equal": ids_equal, "scores_equal": scores_equal,
                              "against": "CPU oracle (fp64 exhaustive over all rows), ids and fp64 scores bit for bit"}
            print(json.dumps(line))
            ok = ids_equal and scores_equal
    else:
        ok = True
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if not ok:
        sys.exit("parity check failed: the answers differ from the CPU oracle")


if __name__ == "__main__":
    main()
