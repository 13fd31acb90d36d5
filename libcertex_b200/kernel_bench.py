"""Times the tensor-core pass alone (the counterpart of the reference's cpp/bench/kernel_bench.cu, which prints the
TFLOPS of its fp16 pass): random uint8 codes, `--mode screen` with a threshold nothing reaches (pure pass cost) or
with `--survivors` kept pairs per query on average, `--mode groupmax`, or the rate probe `--mode rate`: the same
TMA + tcgen05.mma stream with no epilogue, i.e. the tensor-pipe rate this tiling can reach.

    python -m libcertex_b200.kernel_bench --nq 2048 --n 1000000 --iters 5
"""

import argparse
import ctypes

import torch

from . import _lib


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--nq", type=int, default=2048)
    ap.add_argument("--n", type=int, default=1_000_000)
    ap.add_argument("--code-len", type=int, default=128)
    ap.add_argument("--mode", default="screen", choices=["screen", "groupmax", "rate", "groupbound"])
    ap.add_argument("--survivors", type=float, default=0.0, help="average kept pairs per query (screen mode)")
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--trace", type=int, default=0,
                    help="print SM clock stamps of this many units of CTA 0 of the last run (needs the trace build: "
                         "CERTEX_B200_LIB=<...>/lib/libcertex_b200_trace.so)")
    args = ap.parse_args()

    L, res = _lib.lib(), _lib.resources()
    nq, n, cl = args.nq, args.n, args.code_len
    nq_pad, n_pad = -(-nq // 128) * 128, -(-n // 256) * 256
    g = torch.Generator(device="cuda").manual_seed(0)
    q = torch.zeros((nq_pad, cl), dtype=torch.uint8, device="cuda")
    q[:nq] = torch.randint(0, 256, (nq, cl), generator=g, device="cuda", dtype=torch.uint8)
    x = torch.randint(0, 256, (n, cl), generator=g, device="cuda", dtype=torch.uint8)
    init = torch.full((n_pad,), -(1 << 30), dtype=torch.int32, device="cuda")
    for i in range(0, n, 1 << 20):  # chunked: the int64 squares of a large x would not fit
        init[i : i + (1 << 20)][: min(1 << 20, n - i)] = -((x[i : i + (1 << 20)].long() ** 2).sum(1) >> 1).int()
    # rows in the order the engine keeps them: sorted by norm, so that e is almost constant over a chain of 16 rows
    order = torch.argsort(init[:n], descending=True, stable=True)
    x = x[order].contiguous()
    init[:n] = init[:n][order]
    ld = -(-(n_pad // 64) // 8) * 8
    need_gmax = args.mode in ("groupmax", "groupbound") or args.survivors > 0
    gmax = torch.zeros((nq if need_gmax else 1, ld), dtype=torch.int32, device="cuda")
    cap = 4096
    cnt = torch.zeros((nq,), dtype=torch.int32, device="cuda")
    cand = torch.zeros((nq, cap), dtype=torch.int32, device="cuda")
    thr = torch.full((nq,), 2**31 - 1, dtype=torch.int32, device="cuda")
    mode = {"screen": 0, "groupmax": 1, "rate": 2, "groupbound": 3}[args.mode]
    ms = ctypes.c_float()

    def run(m, t):
        cnt.zero_()
        _lib.check(L.certexB200ScreenRaw(res, q.data_ptr(), nq, x.data_ptr(), n, cl, 0, init.data_ptr(), m,
                                         t.data_ptr(), gmax.data_ptr(), ld, cnt.data_ptr(), cand.data_ptr(), cap,
                                         ctypes.byref(ms)))
        return ms.value

    if mode == 0 and args.survivors > 0:
        # threshold = the value that about `survivors` pairs per query reach: from the group maxima of a first pass
        run(1, thr)
        k = max(1, min(int(args.survivors), gmax.shape[1]))
        thr = torch.topk(gmax[:, : n_pad // 64], k, dim=1).values[:, -1].contiguous()
    clocks = []
    try:
        import pynvml

        pynvml.nvmlInit()
        h = pynvml.nvmlDeviceGetHandleByIndex(torch.cuda.current_device())
    except Exception:
        h = None
    trace = None
    if args.trace > 0:
        trace = torch.zeros((args.trace, 12), dtype=torch.int64, device="cuda")
        _lib.check(L.certexB200ScreenTrace(trace.data_ptr(), args.trace))
    times = []
    for _ in range(args.iters):
        times.append(run(mode, thr))
        if h is not None:
            clocks.append(pynvml.nvmlDeviceGetClockInfo(h, pynvml.NVML_CLOCK_SM))
    if trace is not None:
        _lib.check(L.certexB200ScreenTrace(None, 0))
    best = min(times)
    tops = 2.0 * nq * n * cl / (best / 1e3) / 1e12
    units = (nq_pad // 128) * (n_pad // 256)
    print(f"mode={args.mode} nq={nq} n={n} code_len={cl}: best {best:.3f} ms of {args.iters} "
          f"({tops:.1f} int8 TOP/s, {units} units, kept/query {float(cnt.float().mean()):.1f}, "
          f"SM MHz after each run min/max {min(clocks) if clocks else None}/{max(clocks) if clocks else None})")

    if trace is not None:
        t = trace.cpu().numpy()
        t0 = int(t[t > 0].min())
        names = "m_wait m_have m_commit e_wait e_full e_ld e_rel e_done eL_full eL_ld".split()
        print("unit " + " ".join(f"{n:>8s}" for n in names))
        for u in range(args.trace):
            print(f"{u:4d} " + " ".join(f"{int(v) - t0 if v > 0 else -1:8d}" for v in t[u, :10]))


if __name__ == "__main__":
    main()
