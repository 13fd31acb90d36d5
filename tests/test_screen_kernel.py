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
