"""certexB200SearchStatic, the search entry point that allocates nothing on the GPU.

Some callers cannot allocate device memory when they search: a serving process in which another allocator reserved the
whole GPU at start-up (a cudaMalloc inside the search would fail), or a loop whose latency budget has no room for the
device-wide synchronisation an allocation can cause. For them the library keeps the temporaries of its dense search in
a fixed array inside the library image. This test calls that entry point through the C ABI twice in a row (different
queries, different sizes, so the second call runs over what the first left in the array) and requires the same ids and
distances as the regular entry point, cuvsCertexSearch, on an index built from the same vectors, and as the CPU oracle
(ids equal; distances equal to the oracle's fp64 scores brought to the entry point's float32 conventions), so that a
fault shared by both entry points would not pass. It also checks that a request larger than the fixed array, or one
made with another device's resources, is refused with a message. The file sorts last so that a run that stops at the
first failure has already run every other test."""

import ctypes

import numpy as np
import pytest
import torch

from libcertex_b200 import _lib
from oracle import oracle

pytestmark = pytest.mark.gpu
METRIC_NAME = {_lib.L2Expanded: "l2", _lib.InnerProduct: "ip", _lib.CosineExpanded: "cosine"}


def _oracle(x, q, k, metric):
    """ids and float32 distances of the CPU oracle in the conventions of cuvsCertexSearch: squared distance for L2,
    <q, x> for the inner product, 1 - cos for the cosine metric."""
    xh, qh = x.cpu().numpy(), q.cpu().numpy()
    ids, s = oracle.knn(xh, qh, k, METRIC_NAME[metric])
    if metric == _lib.L2Expanded:
        d = s
    elif metric == _lib.CosineExpanded:
        d = s / 2
    else:
        qq = np.zeros(len(qh))
        for t in range(qh.shape[1]):  # the sequential fp64 sum the engine and the oracle use for |q|^2
            qq = qq + qh[:, t].astype(np.float64) * qh[:, t].astype(np.float64)
        d = (qq[:, None] - s) / 2
    return ids, d.astype(np.float32)


def _regular(x, q, k, metric):
    """cuvsCertexSearch on an index built from x (the existing entry point)."""
    L, res = _lib.lib(), _lib.resources()
    ip = ctypes.POINTER(_lib.IndexParams)()
    _lib.check(L.cuvsCertexIndexParamsCreate(ctypes.byref(ip)))
    ip.contents.metric = metric
    index = ctypes.POINTER(_lib.IndexHandle)()
    _lib.check(L.cuvsCertexIndexCreate(ctypes.byref(index)))
    _lib.check(L.cuvsCertexBuild(res, ip, _lib.Tensor(x).ref, index))
    sp = ctypes.POINTER(_lib.SearchParams)()
    _lib.check(L.cuvsCertexSearchParamsCreate(ctypes.byref(sp)))
    nb = torch.empty((q.shape[0], k), dtype=torch.int64, device="cuda")
    ds = torch.empty((q.shape[0], k), dtype=torch.float32, device="cuda")
    _lib.check(L.cuvsCertexSearch(res, sp, index, _lib.Tensor(q).ref, _lib.Tensor(nb).ref, _lib.Tensor(ds).ref,
                                  _lib.Filter(None, _lib.NO_FILTER)))
    _lib.check(L.cuvsStreamSync(res))
    L.cuvsCertexSearchParamsDestroy(sp)
    L.cuvsCertexIndexDestroy(index)
    L.cuvsCertexIndexParamsDestroy(ip)
    return nb, ds


def _static(x, q, k, metric):
    L, res = _lib.lib(), _lib.resources()
    code, bits = _lib._DT[x.dtype]
    nb = torch.full((q.shape[0], k), -7, dtype=torch.int64, device="cuda")
    ds = torch.full((q.shape[0], k), -7.0, dtype=torch.float32, device="cuda")
    status = L.certexB200SearchStatic(res, metric, _lib.DLDataType(code, bits, 1), x.data_ptr(), x.shape[0], q.data_ptr(),
                                      q.shape[0], x.shape[1], k, nb.data_ptr(), ds.data_ptr())
    return status, nb, ds


def test_two_calls_in_a_row_match_the_regular_entry_point():
    g = torch.Generator(device="cuda").manual_seed(0)
    xf = torch.randn((20000, 32), generator=g, device="cuda")
    xf[17] = xf[3]  # equal scores: both entry points must pick the smaller id
    xu = torch.randint(0, 256, (6000, 64), generator=g, device="cuda", dtype=torch.uint8)
    xh = xf.half()
    xi = (torch.randint(0, 256, (6000, 48), generator=g, device="cuda") - 128).to(torch.int8)
    calls = [
        (xf, torch.randn((90, 32), generator=g, device="cuda"), 10, _lib.L2Expanded),
        (xu, torch.randint(0, 256, (300, 64), generator=g, device="cuda", dtype=torch.uint8), 25, _lib.L2Expanded),
        (xf, torch.randn((40, 32), generator=g, device="cuda"), 7, _lib.InnerProduct),
        (xh, torch.randn((50, 32), generator=g, device="cuda").half(), 12, _lib.CosineExpanded),
        (xi, (torch.randint(0, 256, (120, 48), generator=g, device="cuda") - 128).to(torch.int8), 5, _lib.InnerProduct),
        (xf, torch.randn((60, 32), generator=g, device="cuda"), 9, _lib.CosineExpanded),
    ]
    for x, q, k, metric in calls:  # back to back: no other GPU work of the library in between
        status, nb, ds = _static(x, q, k, metric)
        _lib.check(status)
        torch.cuda.synchronize()
        want_nb, want_ds = _regular(x, q, k, metric)
        assert torch.equal(nb, want_nb)
        assert torch.equal(ds, want_ds)
        ids, dist = _oracle(x, q, k, metric)
        assert np.array_equal(nb.cpu().numpy(), ids)
        if metric == _lib.InnerProduct and x.dtype.is_floating_point:
            # <q, x> = (|q|^2 - score) / 2 cancels digits: the float32 value may differ in its last place
            np.testing.assert_allclose(ds.cpu().numpy(), dist, rtol=1e-6, atol=1e-6)
        else:
            assert np.array_equal(ds.cpu().numpy(), dist)


def test_requests_beyond_the_fixed_scratch_are_refused():
    x = torch.zeros((300000, 16), dtype=torch.float32, device="cuda")
    q = torch.zeros((64, 16), dtype=torch.float32, device="cuda")  # 64 * 300000 * 8 bytes of scores > 16 MiB
    status, _, _ = _static(x, q, 5, _lib.L2Expanded)
    assert status == 0
    message = _lib.lib().cuvsGetLastErrorText().decode()
    assert "scratch" in message and str(16 << 20) in message
    odd = torch.zeros((100, 10), dtype=torch.float32, device="cuda")  # rows of 40 bytes: not a multiple of 16
    status, _, _ = _static(odd, odd[:4].contiguous(), 5, _lib.L2Expanded)
    assert status == 0 and "16" in _lib.lib().cuvsGetLastErrorText().decode()
    wide = torch.zeros((64, 8000), dtype=torch.float32, device="cuda")  # more dimensions than a launch takes
    nb = torch.full((4, 5), -7, dtype=torch.int64, device="cuda")
    status = _lib.lib().certexB200SearchStatic(_lib.resources(), _lib.L2Expanded, _lib.DLDataType(_lib.kDLFloat, 32, 1),
                                               wide.data_ptr(), 64, wide.data_ptr(), 4, 8000, 5, nb.data_ptr(),
                                               torch.zeros((4, 5), device="cuda").data_ptr())
    torch.cuda.synchronize()
    assert status == 0 and "dimensions" in _lib.lib().cuvsGetLastErrorText().decode()
    assert bool((nb == -7).all())  # a refused call launches nothing


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_resources_of_another_device_are_refused():
    x = torch.zeros((100, 16), dtype=torch.float32, device="cuda:0")
    res0 = _lib.resources()
    with torch.cuda.device(1):
        nb = torch.zeros((4, 5), dtype=torch.int64, device="cuda:1")
        status = _lib.lib().certexB200SearchStatic(res0, _lib.L2Expanded, _lib.DLDataType(_lib.kDLFloat, 32, 1),
                                                   x.data_ptr(), 100, x.data_ptr(), 4, 16, 5, nb.data_ptr(),
                                                   torch.zeros((4, 5), device="cuda:1").data_ptr())
    assert status == 0 and "device" in _lib.lib().cuvsGetLastErrorText().decode()
