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
