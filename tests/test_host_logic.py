"""Host-side logic that needs no GPU: the work split of the tensor-core pass, shard bounds, mask packing, argument
validation of the Python face (the reference's tests/test_api.py covers the same ground for its package)."""

import ctypes

import numpy as np
import pytest
import torch

import libcertex_b200 as certex
from libcertex_b200 import distributed, index as index_mod


@pytest.mark.parametrize(
    "nqt,nt,panel,grid",
    [(79, 78125, 8, 148), (1, 1, 8, 148), (3, 47, 8, 148), (16, 1000, 8, 148), (79, 4883, 8, 148), (256, 10, 1, 148),
     (5, 7, 2, 3), (8, 1, 8, 148), (100, 100, 4, 148), (33, 1234, 8, 7)],
)
def test_plan_segments_covers_every_unit_once(built_library, nqt, nt, panel, grid):
    out = (ctypes.c_int32 * (grid * 16))()
    assert built_library.certexB200PlanSegments(nqt, nt, panel, grid, out) == 1
    segs = np.frombuffer(out, dtype=np.int32).reshape(grid, 4, 4)
    cover = np.zeros((nqt, nt), dtype=np.int32)
    units = []
    for b in range(grid):
        total, ended = 0, False
        for q0, nq_, t0, t1 in segs[b]:
            if t1 <= t0:
                ended = True
                continue
            assert not ended, "segments of a CTA must be contiguous at the front"
            assert 1 <= nq_ <= panel and q0 >= 0 and q0 + nq_ <= nqt and 0 <= t0 < t1 <= nt
            cover[q0 : q0 + nq_, t0:t1] += 1
            total += nq_ * (t1 - t0)
        units.append(total)
    assert (cover == 1).all()
    # balanced: no CTA has more than one panel-row of tiles above the mean
    assert max(units) - nqt * nt / grid <= panel


@pytest.mark.parametrize(
    "runs,panel,grid,max_segs",
    [([(2, 62)] * 64, 2, 148, 64),                      # 64 labels, two query tiles and 62 base tiles each
     ([(1, 3)] * 300 + [(4, 3)], 7, 148, 64),           # many small labels, one with several query tiles
     ([(9, 500), (1, 1), (2, 40)], 2, 148, 64),         # more query tiles than a panel holds
     ([(1, 5)] * 40, 7, 3, 4),                          # few CTAs with few slots: not everything fits one pass
     ([(3, 1000)], 2, 7, 64), ([(1, 1)], 7, 148, 64)],
)
def test_plan_routed_covers_every_unit_of_the_runs_it_takes(built_library, runs, panel, grid, max_segs):
    n = len(runs)
    nqt = (ctypes.c_int32 * n)(*[r[0] for r in runs])
    nt = (ctypes.c_int32 * n)(*[r[1] for r in runs])
    cap = 100000
    segs = (ctypes.c_int32 * (5 * cap))()
    n_segs, done = ctypes.c_int32(), ctypes.c_int32()
    begin = (ctypes.c_int32 * (grid + 1))()
    assert built_library.certexB200PlanRouted(n, nqt, nt, panel, grid, max_segs, segs, cap, ctypes.byref(n_segs), begin,
                                              ctypes.byref(done)) == 1
    done, n_segs = done.value, n_segs.value
    assert 1 <= done <= n and (done == n or grid * max_segs < 10 * n)
    seg = np.frombuffer(segs, dtype=np.int32)[: 5 * n_segs].reshape(n_segs, 5)
    begin = np.frombuffer(begin, dtype=np.int32)
    assert begin[0] == 0 and begin[-1] == n_segs and (np.diff(begin) >= 0).all() and (np.diff(begin) <= max_segs).all()
    q0 = np.concatenate([[0], np.cumsum([r[0] for r in runs])])
    t0 = np.concatenate([[0], np.cumsum([r[1] for r in runs])])
    cover = {}
    for a, w, lo, hi, col0 in seg:
        r = int(np.searchsorted(t0, lo, side="right") - 1)  # the run this segment belongs to
        assert r < done and col0 == t0[r] and 1 <= w <= panel
        assert q0[r] <= a and a + w <= q0[r + 1] and t0[r] <= lo < hi <= t0[r + 1]
        for qt in range(a, a + w):
            for t in range(lo, hi):
                cover[(qt, t)] = cover.get((qt, t), 0) + 1
    want = sum(runs[r][0] * runs[r][1] for r in range(done))
    assert len(cover) == want and all(v == 1 for v in cover.values())
    if done == n:  # balanced: no CTA but the last (which takes what is left) is more than a panel above its share
        units = [sum(int(w) * int(hi - lo) for a, w, lo, hi, _ in seg[begin[b] : begin[b + 1]]) for b in range(grid)]
        assert max(units[:-1], default=0) <= -(-want // grid) + panel


def test_shard_bounds_partition_rows():
    for n, world in [(10_000_000, 8), (1001, 3), (7, 7), (5, 2)]:
        bounds = [distributed.shard_bounds(n, world, r) for r in range(world)]
        assert bounds[0][0] == 0 and bounds[-1][1] == n
        assert all(bounds[r][1] == bounds[r + 1][0] for r in range(world - 1))


def test_rejects_unknown_metric_and_storage():
    with pytest.raises(ValueError):
        certex.Index(8, metric="hamming")
    with pytest.raises(ValueError):
        certex.Index(8, storage="disk")


def test_empty_index():
    idx = certex.Index(8)
    assert idx.ntotal == 0 and idx.info()["width"] is None and idx.dtype is None
    with pytest.raises(ValueError):
        idx.search(torch.zeros(1, 8))


def test_integer_cast_is_checked():
    with pytest.raises(ValueError):
        index_mod._to_dtype(torch.tensor([[0.5, 1.0]]), torch.uint8)
    with pytest.raises(ValueError):
        index_mod._to_dtype(torch.tensor([[300.0, 1.0]]), torch.uint8)
    assert index_mod._to_dtype(torch.tensor([[3.0, 255.0]]), torch.uint8).dtype == torch.uint8


def test_version():
    assert certex.__version__.count(".") == 2


def test_both_bench_arms_name_the_same_configuration():
    """The benchmark's own arm and its CPU reference arm must print one and the same `config` object."""
    import argparse
    import importlib.util
    import os

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    spec = importlib.util.spec_from_file_location("bench_module", os.path.join(root, "bench.py"))
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)
    for gpus in (1, 2, 8):
        args = argparse.Namespace(gpus=gpus, n_base=bench.N_BASE, n_queries=bench.N_QUERIES, batch=10240,
                                  anchor_stride=16, searches_per_step=0, share_thresholds=1, pipeline=2)
        cfg = bench.config_of(args)
        assert cfg == bench.config_of(args)
        assert cfg["searches_per_step"] == (1 if gpus == 1 else 4)
        assert cfg["share_thresholds"] == (gpus > 1)
        assert cfg["searches_in_flight"] == (1 if gpus == 1 else 2)
        assert f"{gpus} row shard(s)" in cfg["workload"] and "10000000x128 uint8" in cfg["workload"]


@pytest.mark.parametrize("nqt,nt,panel,grid,chunk", [(79, 39063, 7, 148, 1024), (79, 4883, 7, 148, 1024), (16, 3907, 7, 148, 1024),
                                                     (3, 47, 7, 148, 16), (1, 500, 7, 148, 64), (33, 1234, 2, 7, 100),
                                                     (79, 2441, 7, 148, 0)])
def test_chunked_plan_covers_every_unit_once_chunk_by_chunk(built_library, nqt, nt, panel, grid, chunk):
    cap = 4 * grid * (nt // max(chunk, 1) + 2)
    segs = (ctypes.c_int32 * (4 * cap))()
    begin = (ctypes.c_int32 * (grid + 1))()
    n = ctypes.c_int32()
    assert built_library.certexB200PlanChunked(nqt, nt, panel, grid, chunk, segs, cap, ctypes.byref(n), begin) == 1
    segs = np.frombuffer(segs, dtype=np.int32).reshape(-1, 4)[: n.value]
    begin = np.frombuffer(begin, dtype=np.int32)
    assert begin[0] == 0 and begin[-1] == n.value and (np.diff(begin) >= 0).all()
    cover = np.zeros((nqt, nt), dtype=np.int32)
    n_panels = -(-nqt // panel)
    step = chunk if (chunk > 0 and n_panels > 1) else nt
    for b in range(grid):
        last_chunk = -1
        for q0, nq_, t0, t1 in segs[begin[b] : begin[b + 1]]:
            assert 1 <= nq_ <= panel and q0 >= 0 and q0 + nq_ <= nqt and 0 <= t0 < t1 <= nt
            assert t0 // step == (t1 - 1) // step, "a segment stays inside one chunk"
            assert t0 // step >= last_chunk, "a CTA takes the chunks in order"
            last_chunk = t0 // step
            cover[q0 : q0 + nq_, t0:t1] += 1
    assert (cover == 1).all()
    # inside every chunk the CTAs get about the same number of units
    for c0 in range(0, nt, step):
        c1 = min(nt, c0 + step)
        units = [sum(nq_ * (min(t1, c1) - max(t0, c0)) for _, nq_, t0, t1 in segs[begin[b] : begin[b + 1]] if t0 < c1 and t1 > c0)
                 for b in range(grid)]
        assert max(units) - nqt * (c1 - c0) / grid <= panel


@pytest.mark.parametrize("kind", ["few labels", "wide range", "negative", "one label", "empty", "extremes"])
def test_queries_are_grouped_by_label_like_a_stable_sort(built_library, kind):
    rng = np.random.default_rng(7)
    if kind == "few labels":
        lab = rng.integers(0, 64, size=10000)
    elif kind == "wide range":
        lab = rng.integers(-2**31, 2**31, size=5000)          # more than 2^20 apart: the radix passes
    elif kind == "negative":
        lab = rng.integers(-5, 5, size=3000)
    elif kind == "one label":
        lab = np.full(100, 42)
    elif kind == "empty":
        lab = np.zeros(0)
    else:
        lab = rng.choice(np.array([-2**31, -1, 0, 1, 2**31 - 1]), size=2000)
    lab = np.ascontiguousarray(lab, dtype=np.int32)
    order = np.full(len(lab), -1, dtype=np.int32)
    p = ctypes.POINTER(ctypes.c_int32)
    assert built_library.certexB200OrderByLabel(lab.ctypes.data_as(p), len(lab), order.ctypes.data_as(p)) == 1
    assert np.array_equal(order, np.argsort(lab, kind="stable").astype(np.int32))
