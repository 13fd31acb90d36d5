"""The C-ABI library: every symbol that include/certex_b200.h declares is exported, parameter objects carry the
reference's defaults, errors surface as CUVS_ERROR with a message and never as a crash (no GPU needed); and on the GPU,
a plain C-style call sequence through ctypes (the reference's c/tests/neighbors/run_certex_c.c:38-101)."""

import ctypes
import os
import re

import numpy as np
import pytest
import torch

from libcertex_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "certex_b200.h")).read()
    return sorted(set(re.findall(r"CERTEX_B200_EXPORT\s+[\w\s\*]+?\b(\w+)\s*\(", text)))


def test_every_declared_symbol_is_exported(built_library):
    names = declared_symbols()
    assert len(names) >= 30 and "cuvsCertexSearch" in names and "certexB200SearchEx" in names
    for name in names:
        assert hasattr(built_library, name), name
    assert sorted(_lib.SYMBOLS) == names


def test_parameter_defaults_match_the_reference(built_library):
    p = ctypes.POINTER(_lib.IndexParams)()
    assert built_library.cuvsCertexIndexParamsCreate(ctypes.byref(p)) == 1
    c = p.contents
    assert (c.metric, c.width, c.anchor_stride, c.pca_sample, c.host_vectors, c.n_lists, c.local_projections,
            c.int8_rows) == (0, 0, 16, 1_000_000, False, 0, False, False) and abs(c.variance - 0.95) < 1e-12
    assert built_library.cuvsCertexIndexParamsDestroy(p) == 1
    s = ctypes.POINTER(_lib.SearchParams)()
    assert built_library.cuvsCertexSearchParamsCreate(ctypes.byref(s)) == 1
    assert (s.contents.anchors, s.contents.batch_size, s.contents.probe_lists) == (128, 2048, 2)
    assert built_library.cuvsCertexSearchParamsDestroy(s) == 1


def test_errors_are_reported_not_raised(built_library):
    L = built_library
    h = ctypes.POINTER(_lib.IndexHandle)()
    assert L.cuvsCertexIndexCreate(ctypes.byref(h)) == 1
    size = ctypes.c_int64(-1)
    assert L.cuvsCertexIndexGetSize(h, ctypes.byref(size)) == 0  # empty handle
    assert b"empty" in L.cuvsGetLastErrorText()
    assert L.cuvsCertexSerialize(None, b"/nonexistent/x", h) == 0
    assert L.cuvsCertexIndexDestroy(h) == 1
    if not torch.cuda.is_available():
        res = ctypes.c_void_p()
        assert L.cuvsResourcesCreate(ctypes.byref(res)) == 0  # no device: an error, not a fallback
        assert L.cuvsGetLastErrorText()


def _build_c_caller(tmp_path):
    """tests/c/exact_search.c compiled as C11 with gcc against the public header and linked to the library."""
    import shutil
    import subprocess

    cuda = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    lib_dir = os.path.join(ROOT, "libcertex_b200", "lib")
    exe = str(tmp_path / "exact_search_c")
    cmd = [shutil.which("gcc") or "gcc", "-std=c11", "-Wall", "-Wextra", "-Werror", "-O1",
           "-I" + os.path.join(ROOT, "include"), "-I" + os.path.join(cuda, "include"),
           os.path.join(ROOT, "tests", "c", "exact_search.c"), "-o", exe, "-L" + lib_dir, "-lcertex_b200",
           "-L" + os.path.join(cuda, "lib64"), "-lcudart", "-lm", "-Wl,-rpath," + lib_dir,
           "-Wl,-rpath," + os.path.join(cuda, "lib64")]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr[-3000:]
    return exe


def _build_cpp_caller(tmp_path):
    """tests/cpp/exact_search.cpp compiled as C++17 with g++ against include/certex_b200.hpp."""
    import shutil
    import subprocess

    cuda = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    lib_dir = os.path.join(ROOT, "libcertex_b200", "lib")
    exe = str(tmp_path / "exact_search_cpp")
    cmd = [shutil.which("g++") or "g++", "-std=c++17", "-Wall", "-Wextra", "-Werror", "-O1",
           "-I" + os.path.join(ROOT, "include"), "-I" + os.path.join(cuda, "include"),
           os.path.join(ROOT, "tests", "cpp", "exact_search.cpp"), "-o", exe, "-L" + lib_dir, "-lcertex_b200",
           "-L" + os.path.join(cuda, "lib64"), "-lcudart", "-Wl,-rpath," + lib_dir,
           "-Wl,-rpath," + os.path.join(cuda, "lib64")]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr[-3000:]
    return exe


def test_header_is_plain_c_and_a_c_caller_links(built_library, tmp_path):
    _build_c_caller(tmp_path)


def test_cpp_header_compiles_and_a_cpp_caller_links(built_library, tmp_path):
    _build_cpp_caller(tmp_path)


@pytest.mark.gpu
def test_cpp_caller_gets_exact_answers(built_library, tmp_path):
    import subprocess

    exe = _build_cpp_caller(tmp_path)
    r = subprocess.run([exe, str(tmp_path / "index.bin")], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and r.stdout.strip() == "ok", (r.returncode, r.stdout[-500:], r.stderr[-2000:])


@pytest.mark.gpu
def test_c_caller_gets_exact_answers(built_library, tmp_path):
    import subprocess

    exe = _build_c_caller(tmp_path)
    r = subprocess.run([exe, str(tmp_path / "index.bin")], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and r.stdout.strip() == "ok", (r.returncode, r.stdout[-500:], r.stderr[-2000:])


@pytest.mark.gpu
def test_plain_c_call_sequence(tmp_path):
    from oracle import oracle

    L = _lib.lib()
    rng = np.random.default_rng(0)
    n, nq, d, k = 20000, 64, 32, 10
    x = rng.standard_normal((n, d)).astype(np.float32)
    q = rng.standard_normal((nq, d)).astype(np.float32)
    res = ctypes.c_void_p()
    _lib.check(L.cuvsResourcesCreate(ctypes.byref(res)))
    dx, dq = torch.from_numpy(x).cuda(), torch.from_numpy(q).cuda()
    nb = torch.empty((nq, k), dtype=torch.int64, device="cuda")
    ds = torch.empty((nq, k), dtype=torch.float32, device="cuda")
    ip = ctypes.POINTER(_lib.IndexParams)()
    _lib.check(L.cuvsCertexIndexParamsCreate(ctypes.byref(ip)))
    ip.contents.width = 16
    index = ctypes.POINTER(_lib.IndexHandle)()
    _lib.check(L.cuvsCertexIndexCreate(ctypes.byref(index)))
    _lib.check(L.cuvsCertexBuild(res, ip, _lib.Tensor(dx).ref, index))
    assert L.cuvsCertexBuild(res, ip, _lib.Tensor(dx).ref, index) == 0  # the handle already holds an index
    size, dim = ctypes.c_int64(), ctypes.c_int64()
    _lib.check(L.cuvsCertexIndexGetSize(index, ctypes.byref(size)))
    _lib.check(L.cuvsCertexIndexGetDim(index, ctypes.byref(dim)))
    assert (size.value, dim.value) == (n, d)
    # save, destroy, reload: the search below runs on the loaded index
    path = str(tmp_path / "c_index.bin").encode()
    _lib.check(L.cuvsCertexSerialize(res, path, index))
    _lib.check(L.cuvsCertexIndexDestroy(index))
    _lib.check(L.cuvsCertexIndexCreate(ctypes.byref(index)))
    _lib.check(L.cuvsCertexDeserialize(res, path, index))
    sp = ctypes.POINTER(_lib.SearchParams)()
    _lib.check(L.cuvsCertexSearchParamsCreate(ctypes.byref(sp)))
    keep = rng.random(n) < 0.5
    from libcertex_b200.index import pack_mask

    words = _lib.Tensor(pack_mask(torch.from_numpy(keep)))
    words.m.dl_tensor.dtype = _lib.DLDataType(_lib.kDLUInt, 32, 1)
    flt = _lib.Filter(ctypes.cast(ctypes.pointer(words.m), ctypes.c_void_p), _lib.BITSET)
    _lib.check(L.cuvsCertexSearch(res, sp, index, _lib.Tensor(dq).ref, _lib.Tensor(nb).ref, _lib.Tensor(ds).ref, flt))
    _lib.check(L.cuvsStreamSync(res))
    ids, scores = oracle.knn(x, q, k, "l2", keep_row=keep.astype(np.uint8))
    assert np.array_equal(nb.cpu().numpy(), ids)
    assert np.allclose(ds.cpu().numpy(), scores, rtol=1e-6)
    # wrong dtype of the queries is an error
    assert L.cuvsCertexSearch(res, sp, index, _lib.Tensor(dq.half()).ref, _lib.Tensor(nb).ref, _lib.Tensor(ds).ref,
                              _lib.Filter(None, _lib.NO_FILTER)) == 0
    assert b"vector type" in L.cuvsGetLastErrorText()
    _lib.check(L.cuvsCertexSearchParamsDestroy(sp))
    _lib.check(L.cuvsCertexIndexDestroy(index))
    _lib.check(L.cuvsCertexIndexParamsDestroy(ip))
    _lib.check(L.cuvsResourcesDestroy(res))
