"""Kernel-level parity of the tensor-core pass (tcgen05 int8 MMA + fused threshold / group-maximum epilogue) against
an int32 CPU Gram product. Every keep / not-keep decision and every group maximum must match exactly: all inputs of the
test are integers. The shapes include the partial-tile shapes of the reference's kernel tests
(cpp/tests/neighbors/certex_kernels.cu:193-197)."""

import ctypes

import numpy as np
import pytest
import torch

from libcertex_b200 import _lib
from oracle import oracle

pytestmark = pytest.mark.gpu
NEVER = -(1 << 30)

SHAPES = [
    # nq, n, code_len, signed
    (300, 10000, 128, 0),
    (129, 5000, 128, 1),
    (1000, 20011, 256, 0),
    (17, 333, 128, 0),
    (64, 7777, 256, 1),
    (2100, 3000, 128, 0),
    (130, 40000, 256, 0),
    (1, 128, 128, 0),
    (513, 255, 128, 0),
    # rows of more than two K blocks: the K blocks stream through the stage ring
    (300, 6000, 384, 0),
    (129, 3000, 512, 1),
    (50, 2000, 1536, 0),
    (700, 1500, 4096, 1),
]


def _run(mode, q, x, init, thr=None, cap=64, signed=0):
    L = _lib.lib()
    res = _lib.resources()
    nq, n, cl = q.shape[0], x.shape[0], x.shape[1]
    nq_pad, n_pad = -(-nq // 128) * 128, -(-n // 256) * 256
    dq = torch.zeros((nq_pad, cl), dtype=torch.uint8, device="cuda")
    dq[:nq] = torch.from_numpy(q.view(np.uint8)).cuda()
    dx = torch.from_numpy(x.view(np.uint8)).cuda()
    dinit = torch.full((n_pad,), NEVER, dtype=torch.int32, device="cuda")
    dinit[:n] = torch.from_numpy(init).cuda()
    ld = -(-(n_pad // 64) // 8) * 8
    gmax = torch.full((nq, ld), -7, dtype=torch.int32, device="cuda")
    cnt = torch.zeros((nq,), dtype=torch.int32, device="cuda")
    cand = torch.full((nq, cap), -1, dtype=torch.int32, device="cuda")
    dthr = torch.zeros((nq,), dtype=torch.int32, device="cuda") if thr is None else torch.from_numpy(thr).cuda()
    ms = ctypes.c_float()
    _lib.check(L.certexB200ScreenRaw(res, dq.data_ptr(), nq, dx.data_ptr(), n, cl, signed, dinit.data_ptr(), mode,
                                     dthr.data_ptr(), gmax.data_ptr(), ld, cnt.data_ptr(), cand.data_ptr(), cap,
                                     ctypes.byref(ms)))
    torch.cuda.synchronize()
    return gmax.cpu().numpy(), cnt.cpu().numpy(), cand.cpu().numpy(), ms.value


def _data(nq, n, cl, signed, seed):
    rng = np.random.default_rng(seed)
    if signed:
        q = rng.integers(-128, 128, (nq, cl), dtype=np.int8)
        x = rng.integers(-128, 128, (n, cl), dtype=np.int8)
    else:
        q = rng.integers(0, 256, (nq, cl), dtype=np.uint8)
        x = rng.integers(0, 256, (n, cl), dtype=np.uint8)
    xn = (x.astype(np.int64) ** 2).sum(1)
    init = (-(xn >> 1)).astype(np.int32)
    init[rng.random(n) < 0.02] = NEVER  # removed rows
    return q, x, init


@pytest.mark.parametrize("nq,n,cl,signed", SHAPES)
def test_group_maxima_match_int32_gram(nq, n, cl, signed):
    q, x, init = _data(nq, n, cl, signed, seed=nq + n)
    acc = oracle.int_gram(q, x, init)
    n_pad = -(-n // 256) * 256
    full = np.full((nq, n_pad), NEVER, dtype=np.int64)
    full[:, :n] = acc
    want = full.reshape(nq, n_pad // 64, 64).max(2)
    gmax, _, _, _ = _run(1, q, x, init, signed=signed)
    assert np.array_equal(gmax[:, : n_pad // 64], want)


def _kept(q, x, init, thr):
    """What the pass keeps: (q, x) with <q, x> + (largest e of x's chain of 16 rows) >= thr[q]; a superset of the pairs
    at or above the threshold with their own e, equal to it when e is constant over every chain (the engine keeps the
    rows sorted by norm for that)."""
    n = x.shape[0]
    n_pad = -(-n // 16) * 16
    e = np.full(n_pad, NEVER, dtype=np.int64)
    e[:n] = init
    cmax = np.repeat(e.reshape(-1, 16).max(1), 16)[:n]
    gram = oracle.int_gram(q, x, np.zeros(n, dtype=np.int32)).astype(np.int64)
    keep = gram + cmax[None, :] >= thr[:, None].astype(np.int64)
    exact = gram + init[None, :].astype(np.int64) >= thr[:, None].astype(np.int64)
    assert (keep | ~exact).all()
    return keep, exact


@pytest.mark.parametrize("nq,n,cl,signed", SHAPES)
def test_screen_keeps_the_pairs_at_or_above_the_threshold(nq, n, cl, signed):
    q, x, init = _data(nq, n, cl, signed, seed=7 * nq + n)
    order = np.argsort(-init.astype(np.int64), kind="stable")  # rows by norm, removed rows (NEVER) last
    x, init = np.ascontiguousarray(x[order]), init[order]
    acc = oracle.int_gram(q, x, init)
    kth = min(n, 25)
    thr = np.sort(acc, axis=1)[:, -kth].astype(np.int32)  # the 25th largest value: ties included below
    keep, exact = _kept(q, x, init, thr)
    assert keep.sum() <= 1.5 * exact.sum() + 16 * nq  # sorted rows: hardly more than the exact set
    cap = int(keep.sum(1).max())
    _, cnt, cand, _ = _run(0, q, x, init, thr=thr, cap=cap, signed=signed)
    assert np.array_equal(cnt, keep.sum(1))
    for i in range(nq):
        assert np.array_equal(np.sort(cand[i, : cnt[i]]), np.nonzero(keep[i])[0])


def test_overflow_is_counted_and_written_entries_are_valid():
    q, x, init = _data(200, 6000, 128, 0, seed=3)
    acc = oracle.int_gram(q, x, init)
    thr = np.sort(acc, axis=1)[:, -40].astype(np.int32)
    keep, _ = _kept(q, x, init, thr)
    _, cnt, cand, _ = _run(0, q, x, init, thr=thr, cap=8)
    assert np.array_equal(cnt, keep.sum(1)) and (cnt > 8).all()
    for i in range(200):
        assert keep[i, cand[i]].all() and len(set(cand[i].tolist())) == 8


# ---------------------------------------------------------------------------------------------------- float16 codes
def _run_f16(mode, hq, hx, e, thr=None, cap=64):
    """The pass on float16 code rows (code kind 2): e and thr are float32, passed as their bit patterns."""
    L, res = _lib.lib(), _lib.resources()
    nq, n, d = hq.shape[0], hx.shape[0], hx.shape[1]
    cl = -(-(2 * d) // 128) * 128
    nq_pad, n_pad = -(-nq // 128) * 128, -(-n // 256) * 256
    dq = torch.zeros((nq_pad, cl // 2), dtype=torch.float16, device="cuda")
    dq[:nq, :d] = torch.from_numpy(hq).cuda()
    dx = torch.zeros((n, cl // 2), dtype=torch.float16, device="cuda")
    dx[:, :d] = torch.from_numpy(hx).cuda()
    dinit = torch.full((n_pad,), -np.inf, dtype=torch.float32, device="cuda")
    dinit[:n] = torch.from_numpy(e).cuda()
    ld = -(-(n_pad // 64) // 8) * 8
    gmax = torch.zeros((nq, ld), dtype=torch.int32, device="cuda")
    cnt = torch.zeros((nq,), dtype=torch.int32, device="cuda")
    cand = torch.full((nq, cap), -1, dtype=torch.int32, device="cuda")
    dthr = torch.zeros((nq,), dtype=torch.float32, device="cuda") if thr is None else torch.from_numpy(thr).cuda()
    ms = ctypes.c_float()
    _lib.check(L.certexB200ScreenRaw(res, dq.data_ptr(), nq, dx.data_ptr(), n, cl, 2, dinit.data_ptr(), mode,
                                     dthr.data_ptr(), gmax.data_ptr(), ld, cnt.data_ptr(), cand.data_ptr(), cap,
                                     ctypes.byref(ms)))
    torch.cuda.synchronize()
    return gmax.cpu().numpy(), cnt.cpu().numpy(), cand.cpu().numpy()


@pytest.mark.parametrize("d,n,nq", [(96, 6000, 200), (128, 3000, 130), (768, 3000, 140), (2048, 1500, 70)])
def test_float16_pass_stays_inside_its_accumulation_bound(d, n, nq):
    """The soundness of the float screen rests on one inequality: the value the tensor cores return for a pair of
    float16 code rows differs from their exact product by at most gamma |h| |x~| with gamma = (d + 16) 2^-20 (float32
    accumulation of exact float16 products in the order the hardware chooses). The test puts many rows right at every
    query's threshold (copies of the row at the threshold with single coordinates nudged by one float16 step) and
    requires: every pair whose exact value lies above the threshold by more than the bound is kept, and no pair is kept
    whose exact value, taken with the largest e of its chain, lies below it by more than the bound. It also checks the
    group maxima of the threshold stage against the exact maxima within the same bound."""
    rng = np.random.default_rng(d + n)
    hx = (rng.standard_normal((n, d)) * rng.uniform(0.3, 2.0, (n, 1))).astype(np.float16)
    hq = rng.standard_normal((nq, d)).astype(np.float16)
    X, Q = hx.astype(np.float64), hq.astype(np.float64)
    # adversarial rows: for the first queries, the row at rank 20 is copied 12 times with one coordinate moved by one ulp
    base = Q[:, :] @ X.T
    for i in range(min(nq, 40)):
        r = int(np.argsort(-base[i])[20])
        for c in range(12):
            row = hx[r].copy()
            t = int(rng.integers(0, d))
            row[t] = np.nextafter(row[t], np.float16(np.inf if c % 2 else -np.inf), dtype=np.float16)
            hx[int(rng.integers(0, n))] = row
    X = hx.astype(np.float64)
    e32 = (-0.5 * (X * X).sum(1)).astype(np.float32)
    order = np.argsort(-e32, kind="stable")  # rows by norm, as the engine stores them
    hx, X, e32 = np.ascontiguousarray(hx[order]), X[order], e32[order]
    exact = Q @ X.T  # products of float16 values are exact in float64; the sums round far below the bound
    value = exact + e32[None, :].astype(np.float64)
    thr = np.sort(value, axis=1)[:, -21].astype(np.float32)  # the adversarial copies sit around this value
    gamma = (d + 16) * 2.0 ** -20
    bound = gamma * np.sqrt((Q * Q).sum(1))[:, None] * np.sqrt((X * X).sum(1))[None, :]
    bound = bound + 2.0 ** -22 * (np.abs(exact) + np.abs(e32)[None, :] + np.abs(thr)[:, None])  # float32 epilogue sums
    n_pad = -(-n // 16) * 16
    epad = np.full(n_pad, -np.inf)
    epad[:n] = e32
    cmax = np.repeat(epad.reshape(-1, 16).max(1), 16)[:n]
    must = value >= thr[:, None] + bound
    may = exact + cmax[None, :] >= thr[:, None] - bound
    assert (may | ~must).all()
    cap = int(may.sum(1).max()) + 8
    _, cnt, cand = _run_f16(0, hq, hx, e32, thr=thr, cap=cap)
    assert (cnt <= cap).all()
    near = 0
    for i in range(nq):
        got = np.zeros(n, dtype=bool)
        got[cand[i, : cnt[i]]] = True
        assert len(set(cand[i, : cnt[i]].tolist())) == cnt[i]
        assert not (must[i] & ~got).any(), f"query {i}: a pair above the threshold by more than the bound was dropped"
        assert not (got & ~may[i]).any(), f"query {i}: a pair below the threshold by more than the bound was kept"
        near += int((may[i] & ~must[i]).sum())
    assert near >= 10 * min(nq, 40)  # the test did put rows inside the band
    # group maxima of the threshold stage: float keys back to floats, against the exact maxima
    gmax, _, _ = _run_f16(1, hq, hx, e32)
    n256 = -(-n // 256) * 256
    keys = gmax[:, : n256 // 64].astype(np.int64)
    bits = np.where(keys < 0, keys ^ 0x7FFFFFFF, keys).astype(np.int32)
    got_max = bits.view(np.float32).astype(np.float64)
    full_v = np.full((nq, n256), -np.inf)
    full_v[:, :n] = value
    full_b = np.zeros((nq, n256))
    full_b[:, :n] = bound
    want_max = full_v.reshape(nq, -1, 64).max(2)
    slack = full_b.reshape(nq, -1, 64).max(2)
    finite = np.isfinite(want_max)
    assert (np.abs(got_max[finite] - want_max[finite]) <= slack[finite]).all()
    assert (got_max[~finite] == -np.inf).all()


@pytest.mark.parametrize("nq,n,cl,signed", SHAPES)
def test_chained_group_bound_is_reached_by_a_row_of_the_group(nq, n, cl, signed):
    """The threshold stage's cheap variant: per group of 64 rows the maximum over its four chains of 16 rows of (largest
    product of the chain + smallest e of the chain). It must equal that expression exactly (integers), never exceed the
    exact group maximum, and hence be a value that some row of the group reaches."""
    q, x, init = _data(nq, n, cl, signed, seed=3 * nq + n)
    order = np.argsort(-init.astype(np.int64), kind="stable")  # rows by norm, as the engine keeps them
    x, init = np.ascontiguousarray(x[order]), init[order]
    gram = oracle.int_gram(q, x, np.zeros(n, dtype=np.int32)).astype(np.int64)
    n_pad = -(-n // 256) * 256
    acc = np.zeros((nq, n_pad), dtype=np.int64)  # padding rows are zero codes with e = NEVER
    acc[:, :n] = gram
    e = np.full(n_pad, NEVER, dtype=np.int64)
    e[:n] = init
    chain = acc.reshape(nq, n_pad // 16, 16).max(2) + e.reshape(n_pad // 16, 16).min(1)[None, :]
    want = chain.reshape(nq, n_pad // 64, 4).max(2)
    exact = (acc + e[None, :]).reshape(nq, n_pad // 64, 64).max(2)
    assert (want <= exact).all()
    got, _, _, _ = _run(3, q, x, init, signed=signed)
    assert np.array_equal(got[:, : n_pad // 64], want)
