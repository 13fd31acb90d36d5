"""Times the other benchmark configurations (the headline one is bench.py at the repository root) on one GPU with
seeded synthetic inputs of their shapes, and prints one JSON line per workload with the search counters:

    python -m libcertex_b200.workload_bench --workload labels      # 1 M x 768 float32, cosine, k = 100, 64 labels
    python -m libcertex_b200.workload_bench --workload wide        # the same vectors without labels
    python -m libcertex_b200.workload_bench --workload gaussian    # 100 000 x 128 float32 N(0, 1), k = 10, L2
    python -m libcertex_b200.workload_bench --workload keycache    # 8 KV heads x 131 072 keys x 128, k = 2048

`--n` scales the number of stored vectors (keys per head for keycache). Times are wall clock around the public call
with the stream synchronised on both sides, best of `--iters` after one warm-up call."""

import argparse
import json
import time

import torch

from . import synthetic
from .attention import KeyCache
from .index import Index, search_stats


def _timed(call, iters):
    call()
    best, stats = None, None
    for _ in range(iters):
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        with search_stats() as st:
            call()
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        if best is None or dt < best:
            best, stats = dt, st
    return best, stats


def _line(name, nq, seconds, st, **extra):
    out = {"workload": name, "queries": nq, "ms": round(seconds * 1e3, 3), "qps": round(nq / seconds, 1),
           "survivors_per_query": round(st.survivors / max(st.queries, 1), 1), "dense_queries": st.dense_queries,
           "rescreened": st.rescreened, "routed_slots": st.routed_queries, "launches": st.launches,
           "screen_ms": round(st.screen_ms, 3), "anchor_ms": round(st.anchor_ms, 3)}
    out.update(extra)
    print(json.dumps(out), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--workload", required=True, choices=["labels", "wide", "gaussian", "keycache"])
    ap.add_argument("--n", type=int, default=None)
    ap.add_argument("--nq", type=int, default=None)
    ap.add_argument("--k", type=int, default=None)
    ap.add_argument("--iters", type=int, default=3)
    args = ap.parse_args()

    if args.workload in ("labels", "wide"):
        n, nq, k, dim = args.n or 1_000_000, args.nq or 10_000, args.k or 100, 768
        x = synthetic.clustered_unit_f32(n, dim, seed=0)
        q = synthetic.clustered_unit_f32(nq, dim, seed=1)
        index = Index(dim, metric="cosine")
        if args.workload == "labels":
            g = torch.Generator().manual_seed(3)
            lab = torch.randint(0, 64, (n,), generator=g, dtype=torch.int32).cuda()
            ql = torch.randint(0, 64, (nq,), generator=g, dtype=torch.int32).cuda()
            index.add(x, labels=lab)
            sec, st = _timed(lambda: index.search(q, k=k, labels=ql, batch=10240), args.iters)
            _line("labels", nq, sec, st, n=n, dim=dim, k=k, labels=64)
            # 1 % of the vectors removed and as many added (with a new partition) between query batches
            gone = torch.randperm(n, generator=g)[: n // 100].cuda()
            fresh = synthetic.clustered_unit_f32(n // 100, dim, seed=9)
            fresh_lab = torch.randint(0, 64, (n // 100,), generator=g, dtype=torch.int32).cuda()
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            index.remove(gone)
            index.add(fresh, labels=fresh_lab)
            torch.cuda.synchronize()
            churn = time.perf_counter() - t0
            sec, st = _timed(lambda: index.search(q, k=k, labels=ql, batch=10240), args.iters)
            _line("labels after 1 % churn", nq, sec, st, n=n, dim=dim, k=k, labels=64, churn_ms=round(churn * 1e3, 2))
        else:
            index.add(x)
            sec, st = _timed(lambda: index.search(q, k=k, batch=10240), args.iters)
            _line("wide", nq, sec, st, n=n, dim=dim, k=k)
    elif args.workload == "gaussian":
        n, nq, k = args.n or 100_000, args.nq or 1000, args.k or 10
        xb, xq = synthetic.gaussian_f32(n, nq, 128, seed=0)
        index = Index(128)
        index.add(torch.from_numpy(xb).cuda())
        q = torch.from_numpy(xq).cuda()
        sec, st = _timed(lambda: index.search(q, k=k), args.iters)
        _line("gaussian", nq, sec, st, n=n, dim=128, k=k)
    else:
        n, k = args.n or 131_072, args.k or 2048
        keys = synthetic.keys_with_outliers(8, n, 128, seed=0)
        g = torch.Generator(device="cuda").manual_seed(5)
        q = torch.randn((32, 16, 128), generator=g, device="cuda").to(torch.bfloat16)
        cache = KeyCache(8, 128, k=k).append(keys)
        sec, st = _timed(lambda: cache.topk(q), args.iters)
        _line("keycache", 32 * 16, sec, st, keys_per_head=n, kv_heads=8, k=k)


if __name__ == "__main__":
    main()
