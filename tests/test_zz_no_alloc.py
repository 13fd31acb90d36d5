"""certexB200SearchStatic, the search entry point that allocates nothing on the GPU.

Some callers cannot allocate device memory when they search: a serving process in which another allocator reserved the
whole GPU at start-up (a cudaMalloc inside the search would fail), or a loop whose latency budget has no room for the
device-wide synchronisation an allocation can cause. For them the library keeps the temporaries of its dense search in
a fixed array inside the library image. This test calls that entry point through the C ABI twice in a row (different
queries, different sizes, so the second call runs over what the first left in the array) and requires the same ids and
distances as the regular entry point, cuvsCertexSearch, on an index built from the same vectors. It also checks that a
request larger than the fixed array is refused with a message. The file sorts last so that a run that stops at the
first failure has already run every other test."""

import ctypes

import numpy as np
import pytest
import torch

from libcertex_b200 import _lib

pytestmark = pytest.mark.gpu


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
    calls = [
        (xf, torch.randn((90, 32), generator=g, device="cuda"), 10, _lib.L2Expanded),
        (xu, torch.randint(0, 256, (300, 64), generator=g, device="cuda", dtype=torch.uint8), 25, _lib.L2Expanded),
        (xf, torch.randn((40, 32), generator=g, device="cuda"), 7, _lib.InnerProduct),
    ]
    for x, q, k, metric in calls:  # back to back: no other GPU work of the library in between
        status, nb, ds = _static(x, q, k, metric)
        _lib.check(status)
        torch.cuda.synchronize()
        want_nb, want_ds = _regular(x, q, k, metric)
        assert torch.equal(nb, want_nb)
        assert torch.equal(ds, want_ds)


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
