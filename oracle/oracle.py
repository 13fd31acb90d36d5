"""Python face of the CPU oracle. TEST INFRASTRUCTURE ONLY: the package `libcertex_b200` never imports this module;
tests, the smoke check and the CPU-baseline leg of the benchmark do.

`knn` calls the C restatement (exact_knn.c, compiled to liboracle.so next to this file) of the reference's fp64
exhaustive check (cpp/tests/neighbors/ann_certex.cuh:78-141). `knn_numpy` is an independent restatement of the same
loops in numpy (sequential over the coordinates, vectorised over the pairs, so that every fp64 rounding happens in the
same order as in the C loop); it serves as a cross-check of the C code on small cases.
"""

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "liboracle.so")
_lib = None

DTYPES = {"float32": 0, "float16": 1, "int8": 2, "uint8": 3}
METRICS = {"l2": 0, "ip": 1, "cosine": 2}


def build(force=False):
    """Compile liboracle.so with the Makefile of this directory (gcc, OpenMP)."""
    src = os.path.join(_HERE, "exact_knn.c")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.run(["make", "-C", _HERE, "liboracle.so"], check=True, capture_output=True)
    return _SO


def lib():
    global _lib
    if _lib is None:
        build()
        L = ctypes.CDLL(_SO)
        vp, i64, i32 = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int
        L.oracle_knn.restype = ctypes.c_int
        L.oracle_knn.argtypes = [vp, i64, vp, i64, i64, i32, i32, i32, i64, vp, vp, vp, vp, vp, vp, i32]
        L.oracle_score.restype = ctypes.c_double
        L.oracle_score.argtypes = [vp, vp, i32, i64, i64, i64, i32]
        L.oracle_merge.restype = None
        L.oracle_merge.argtypes = [vp, vp, i32, i64, i32, vp, vp]
        L.oracle_int_gram.restype = None
        L.oracle_int_gram.argtypes = [vp, i64, vp, i64, i64, i64, i64, i32, vp, vp]
        _lib = L
    return _lib


def _ptr(a):
    return None if a is None else a.ctypes.data_as(ctypes.c_void_p)


def _prep(x, q):
    x = np.ascontiguousarray(x)
    q = np.ascontiguousarray(q)
    if x.dtype.name not in DTYPES:
        raise ValueError(f"unsupported dtype {x.dtype}")
    if q.dtype != x.dtype:
        raise ValueError("queries must have the dtype of the vectors")
    return x, q


def knn(x, q, k, metric="l2", keep_row=None, keep_pair=None, row_labels=None, query_labels=None, id_base=0, threads=0):
    """Exact k nearest neighbours of every row of q among the rows of x: (ids int64 [nq,k], scores fp64 [nq,k]),
    ordered by (score, id). Scores: squared distance (l2), |q|^2 - 2<q,x> (ip), 2 - 2cos (cosine)."""
    x, q = _prep(x, q)
    n, d = x.shape
    nq = q.shape[0]
    ids = np.empty((nq, k), dtype=np.int64)
    scores = np.empty((nq, k), dtype=np.float64)
    kr = None if keep_row is None else np.ascontiguousarray(keep_row, dtype=np.uint8)
    kp = None if keep_pair is None else np.ascontiguousarray(keep_pair, dtype=np.uint8)
    rl = None if row_labels is None else np.ascontiguousarray(row_labels, dtype=np.int32)
    ql = None if query_labels is None else np.ascontiguousarray(query_labels, dtype=np.int32)
    used = lib().oracle_knn(
        _ptr(x), n, _ptr(q), nq, d, DTYPES[x.dtype.name], METRICS[metric], k, id_base,
        _ptr(kr), _ptr(kp), _ptr(rl), _ptr(ql), _ptr(ids), _ptr(scores), threads,
    )
    knn.threads_used = used
    return ids, scores


def score(x, q, i, j, metric="l2"):
    x, q = _prep(x, q)
    return lib().oracle_score(_ptr(x), _ptr(q), DTYPES[x.dtype.name], i, j, x.shape[1], METRICS[metric])


def merge(ids, scores):
    """Merge per-shard answers [S, nq, k] by (score, id)."""
    ids = np.ascontiguousarray(ids, dtype=np.int64)
    scores = np.ascontiguousarray(scores, dtype=np.float64)
    S, nq, k = ids.shape
    out_i = np.empty((nq, k), dtype=np.int64)
    out_s = np.empty((nq, k), dtype=np.float64)
    lib().oracle_merge(_ptr(ids), _ptr(scores), S, nq, k, _ptr(out_i), _ptr(out_s))
    return out_i, out_s


def int_gram(q, x, init=None):
    """int32 <q_i, x_j> + init[j] for uint8 or int8 matrices (the integer screening product)."""
    q = np.ascontiguousarray(q)
    x = np.ascontiguousarray(x)
    assert q.dtype == x.dtype and q.dtype in (np.uint8, np.int8)
    acc = np.empty((q.shape[0], x.shape[0]), dtype=np.int32)
    it = None if init is None else np.ascontiguousarray(init, dtype=np.int32)
    lib().oracle_int_gram(_ptr(q), q.shape[0], _ptr(x), x.shape[0], q.shape[1], q.shape[1], x.shape[1],
                          int(q.dtype == np.int8), _ptr(it), _ptr(acc))
    return acc


def scores_numpy(x, q, metric="l2"):
    """All-pairs fp64 scores [nq, n], coordinates accumulated sequentially (same rounding order as exact_score)."""
    xd = np.asarray(x).astype(np.float64)
    qd = np.asarray(q).astype(np.float64)
    nq, n, d = qd.shape[0], xd.shape[0], xd.shape[1]
    if metric == "l2":
        s = np.zeros((nq, n))
        for t in range(d):
            diff = qd[:, t, None] - xd[None, :, t]
            s = s + diff * diff
        return s
    ip = np.zeros((nq, n))
    qq = np.zeros((nq, 1))
    xx = np.zeros((1, n))
    for t in range(d):
        ip = ip + qd[:, t, None] * xd[None, :, t]
        qq = qq + qd[:, t, None] * qd[:, t, None]
        xx = xx + xd[None, :, t] * xd[None, :, t]
    if metric == "ip":
        return qq - 2 * ip
    return 2 - 2 * ip / np.sqrt(np.maximum(qq * xx, 1e-300))


def knn_numpy(x, q, k, metric="l2", keep=None):
    """Small-case restatement: sort all (score, id) pairs. keep: optional bool [nq, n] or [n]."""
    s = scores_numpy(x, q, metric)
    if keep is not None:
        s = np.where(np.broadcast_to(np.asarray(keep, dtype=bool), s.shape), s, np.inf)
    n = s.shape[1]
    order = np.lexsort((np.broadcast_to(np.arange(n), s.shape), s), axis=1)[:, :k]
    sc = np.take_along_axis(s, order, 1)
    ids = np.where(np.isfinite(sc), order, -1).astype(np.int64)
    if ids.shape[1] < k:
        pad = k - ids.shape[1]
        ids = np.pad(ids, ((0, 0), (0, pad)), constant_values=-1)
        sc = np.pad(sc, ((0, 0), (0, pad)), constant_values=np.inf)
    return ids, sc
