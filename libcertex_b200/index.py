"""Python face of the engine with the call surface of the reference's `certex` package
(certex/index.py: `Index` 191-397, `ShardedIndex` 400-457, `search` 460-484, `verify` 487-548, `search_stats` 171-188).

Every call goes through the C ABI (`_lib`), on the current torch CUDA stream; nothing here computes distances itself.
Metrics: "l2" (squared Euclidean distances, ascending), "ip" (inner products, descending), "cosine" (cosine
similarities, descending). Ties between equal exact scores go to the smaller id.
"""

import ctypes
import threading

import numpy as np
import torch

from . import _lib as L

METRICS = ("l2", "cosine", "ip")
_INDEX_DTYPES = (torch.float32, torch.float16, torch.int8, torch.uint8)
_NAMES = {torch.float32: "float32", torch.float16: "float16", torch.int8: "int8", torch.uint8: "uint8"}
_FROM_DL = {(L.kDLFloat, 32): torch.float32, (L.kDLFloat, 16): torch.float16, (L.kDLInt, 8): torch.int8,
            (L.kDLUInt, 8): torch.uint8}


def _need(ok, message):
    if not ok:
        raise ValueError(message)


def _as_torch(x):
    """(torch view of x, kind of the input) for numpy, torch, DLPack and CUDA-array-interface arrays."""
    if isinstance(x, torch.Tensor):
        return x, "torch"
    if isinstance(x, np.ndarray):
        return torch.from_numpy(np.ascontiguousarray(x)), "numpy"
    if hasattr(x, "__dlpack__"):
        return torch.from_dlpack(x), type(x).__module__.split(".")[0]
    if hasattr(x, "__cuda_array_interface__"):
        return torch.as_tensor(x, device="cuda"), type(x).__module__.split(".")[0]
    return torch.from_numpy(np.ascontiguousarray(np.asarray(x))), "numpy"


def _like_input(t, kind):
    if kind == "torch":
        return t
    if kind == "numpy":
        return t.cpu().numpy()
    try:
        import importlib

        return importlib.import_module(kind).from_dlpack(t)
    except (ImportError, AttributeError, TypeError):
        return t


def _to_dtype(t, dtype):
    """t converted to the element type of the index; an integer index takes only values it represents exactly."""
    if t.dtype == dtype:
        return t
    if not dtype.is_floating_point:
        info = torch.iinfo(dtype)
        f = t.double()
        exact = bool(((f == f.round()) & (f >= info.min) & (f <= info.max)).all())
        _need(exact, f"the index holds {dtype} vectors: values must be integers in [{info.min}, {info.max}]")
    return t.to(dtype)


def pack_mask(mask):
    """Boolean mask (flattened row-major) as uint32 filter words: bit j of word i is entry 32 i + j."""
    b = mask.reshape(-1).to(device="cuda", dtype=torch.int64)
    b = torch.nn.functional.pad(b, (0, (-b.numel()) % 32)).view(-1, 32)
    w = (b << torch.arange(32, device=b.device)).sum(1)
    return torch.where(w >= 2**31, w - 2**32, w).to(torch.int32).contiguous()


class search_stats:
    """Counters of the calling thread's searches inside the block: queries, survivors (pairs the screen kept),
    verified (exact scores computed), dense_queries (queries answered without the screen), rescreened (queries screened
    a second time with a tighter threshold), routed_queries (query slots of searches by label screened against their
    label's rows), launches (kernels of the library), and the device time of the tensor-core
    passes: screen_ms, anchor_ms over screen_passes passes, and span_ms, the device time from the first to the last
    operation the screened searches enqueued (what it exceeds the passes by is small kernels and gaps between kernels;
    what a caller's own clock exceeds it by is time the device waited for the host)."""

    def __enter__(self):
        L.check(L.lib().certexB200StatsBegin())
        self.queries = self.survivors = self.verified = self.dense_queries = 0
        self.launches = self.screen_passes = self.rescreened = self.routed_queries = 0
        self.screen_ms = self.anchor_ms = self.span_ms = 0.0
        return self

    def __exit__(self, *exc):
        torch.cuda.current_stream().synchronize()
        out = (ctypes.c_uint64 * 16)()
        L.check(L.lib().certexB200StatsEnd(out))
        self.queries, self.survivors, self.verified, self.dense_queries, self.launches = (int(v) for v in out[:5])
        self.screen_ms, self.anchor_ms, self.screen_passes = out[5] / 1000.0, out[6] / 1000.0, int(out[7])
        self.rescreened, self.routed_queries, self.span_ms = int(out[8]), int(out[9]), out[10] / 1000.0
        return False


class _Core:
    """Owner of one cuvsCertexIndex handle."""

    def __init__(self):
        self.handle = ctypes.POINTER(L.IndexHandle)()
        L.check(L.lib().cuvsCertexIndexCreate(ctypes.byref(self.handle)))

    def __del__(self):
        try:
            if self.handle:
                L.lib().cuvsCertexIndexDestroy(self.handle)
                self.handle = None
        except Exception:
            pass

    def info(self):
        out = L.IndexInfo()
        L.check(L.lib().certexB200IndexGetInfo(self.handle, ctypes.byref(out)))
        return out

    @property
    def dtype(self):
        d = self.handle.contents.dtype
        return _FROM_DL[(d.code, d.bits)]


class Index:
    """Exact k-NN index; every search returns the exact k nearest stored vectors of every query.

    Same constructor as the reference (certex/index.py:220-238). width, n_lists, local_projections and int8_rows
    only tune the reference's speed; they are accepted and have no effect here. partition_labels=True keeps the ids
    grouped by label, so that a search by labels screens and scores only the vectors of the query's label
    ("lazy": renewed only once an eighth of the vectors is newer than the partition). storage="host" is
    accepted; vectors are kept in GPU memory. The vectors keep the element type of the first addition (float32,
    float16, int8, uint8; other types become float32; cosine needs a float type).
    """

    def __init__(self, dim, metric="l2", width="auto", storage="device", capacity=None, anchor_stride=16,
                 partition_labels=True, n_lists=0, local_projections=False, int8_rows=False):
        _need(metric in METRICS, f"metric must be one of {METRICS}, not {metric!r}")
        _need(storage in ("device", "host"), f'storage must be "device" or "host", not {storage!r}')
        self.d, self.metric, self.width, self.storage = dim, metric, width, storage
        self.capacity, self.anchor_stride, self.partition_labels = capacity, anchor_stride, partition_labels
        self.n_lists, self.local_projections, self.int8_rows = n_lists, local_projections, int8_rows
        self.core = None
        self._writer = threading.Lock()

    # ------------------------------------------------------------------ properties
    @property
    def ntotal(self):
        if self.core is None:
            return 0
        i = self.core.info()
        return int(i.size - i.n_removed)

    @property
    def dtype(self):
        return None if self.core is None else self.core.dtype

    def info(self):
        i = None if self.core is None else self.core.info()
        return {
            "metric": self.metric,
            "width": None if i is None else int(i.dim),
            "row_bytes": None if i is None else int(i.row_pitch_bytes),
            "screening_bytes_per_vector": None if i is None else (4 if i.integer_screen else 0),
            "dtype": None if i is None else _NAMES[self.core.dtype],
            "storage": self.storage,
            "ntotal": self.ntotal,
            "integer_screen": None if i is None else bool(i.integer_screen),
            "n_partitioned": 0 if i is None else int(i.n_partitioned),
        }

    # ------------------------------------------------------------------ updates
    def _matrix(self, x, to_device):
        t, kind = _as_torch(x)
        if t.ndim == 1:
            t = t.reshape(1, -1)
        _need(t.ndim == 2 and t.shape[1] == self.d,
              f"expected vectors of dimension {self.d} (a matrix (n, {self.d}) or one vector), got shape {tuple(t.shape)}")
        if to_device or t.is_cuda:
            t = t.cuda()
        if self.core is not None:
            t = _to_dtype(t, self.dtype)
        elif t.dtype not in _INDEX_DTYPES or (self.metric == "cosine" and not t.dtype.is_floating_point):
            t = t.float()
        return t.contiguous(), kind

    def add(self, x, labels=None):
        """Add vectors (optionally one non-negative label each); returns their ids (consecutive, never reused)."""
        X, kind = self._matrix(x, to_device=False)
        lab = None
        if labels is not None:
            lab = _as_torch(labels)[0].reshape(-1).to(device="cuda", dtype=torch.int32).contiguous()
            _need(lab.shape[0] == X.shape[0] and (lab.numel() == 0 or int(lab.min()) >= 0), "one non-negative label per vector")
        lib = L.lib()
        with self._writer:
            labeled = self.core is not None and bool(self.core.info().has_labels)
            if labeled:
                _need(lab is not None, "this index is labeled: add labels with every addition")
            if self.core is not None and lab is not None and not labeled:
                raise ValueError("labels must be given from the first addition on")
            res = L.resources()
            xt = L.Tensor(X)
            if self.core is None:
                p = ctypes.POINTER(L.IndexParams)()
                L.check(lib.cuvsCertexIndexParamsCreate(ctypes.byref(p)))
                try:
                    p.contents.metric = L.METRIC_CODE[self.metric]
                    p.contents.width = 0 if self.width == "auto" else int(self.width)
                    p.contents.anchor_stride = int(self.anchor_stride)
                    p.contents.host_vectors = self.storage == "host"
                    p.contents.n_lists = int(self.n_lists)
                    p.contents.local_projections = bool(self.local_projections)
                    p.contents.int8_rows = bool(self.int8_rows)
                    core = _Core()
                    L.check(lib.cuvsCertexBuild(res, p, xt.ref, core.handle))
                    self.core = core
                finally:
                    lib.cuvsCertexIndexParamsDestroy(p)
                first = 0
                if self.capacity is not None and self.capacity > X.shape[0]:
                    L.check(lib.certexB200IndexReserve(res, self.core.handle, int(self.capacity)))
            else:
                first = int(self.core.info().size)
                L.check(lib.cuvsCertexExtend(res, xt.ref, self.core.handle))
            if lab is not None:
                L.check(lib.cuvsCertexSetLabels(res, L.Tensor(lab).ref, first, self.core.handle))
                # The partition (ids grouped by label and a label-ordered copy of the screen's rows) is renewed with
                # every labeled addition: it costs a sort of the labels and one copy of the code rows.
                # partition_labels="lazy" keeps the reference's rule instead (certex/index.py:306-311): renew once an
                # eighth of the vectors is newer than the partition; until then the newer vectors are scored densely.
                i = self.core.info()
                lazy = self.partition_labels == "lazy"
                if self.partition_labels and (not lazy or 8 * (int(i.size) - int(i.n_partitioned)) > int(i.size)):
                    L.check(lib.cuvsCertexPartitionByLabels(res, self.core.handle))
        return _like_input(torch.arange(first, first + X.shape[0]), kind)

    def set_labels(self, labels, first=0):
        """Labels of the vectors first, first + 1, ... (cuvsCertexSetLabels); relabeling voids the label partition."""
        _need(self.core is not None, "add vectors first")
        lab = _as_torch(labels)[0].reshape(-1).to(device="cuda", dtype=torch.int32).contiguous()
        with self._writer:
            L.check(L.lib().cuvsCertexSetLabels(L.resources(), L.Tensor(lab).ref, int(first), self.core.handle))

    def partition_by_labels(self):
        """Group the ids by label now (cuvsCertexPartitionByLabels); `add` does it by itself as the index grows."""
        _need(self.core is not None, "add vectors first")
        with self._writer:
            L.check(L.lib().cuvsCertexPartitionByLabels(L.resources(), self.core.handle))

    def remove(self, ids):
        """Remove vectors by id; they never appear in later results."""
        _need(self.core is not None, "add vectors first")
        t = _as_torch(ids)[0].reshape(-1).to(device="cuda", dtype=torch.int64).contiguous()
        with self._writer:
            L.check(L.lib().cuvsCertexRemove(L.resources(), L.Tensor(t).ref, self.core.handle))

    # ------------------------------------------------------------------ search
    def search(self, q, k=10, batch=2048, labels=None, filter=None, anchors=128, probe_lists=2, return_scores=False,
               id_base=0):
        """Exact k nearest neighbours of every query: (distances or similarities, ids), best first.

        labels: one per query, neighbours are taken among the vectors of that label. filter: boolean mask over the ids
        (True keeps) or one row of such a mask per query. Missing entries have id -1. return_scores=True appends the
        exact fp64 scores the ranking used (squared distance, |q|^2 - 2<q,x>, or 2 - 2cos)."""
        _need(self.core is not None, "the index is empty: add vectors first")
        single = _as_torch(q)[0].ndim == 1
        Q, kind = self._matrix(q, to_device=True)
        nq = Q.shape[0]
        size = int(self.core.info().size)
        _need(1 <= k <= 2048, f"k must be between 1 and 2048, not {k}")
        _need(k <= size, f"k = {k} exceeds the {size} vectors added to the index")
        I = torch.empty((nq, k), dtype=torch.int64, device="cuda")
        D = torch.empty((nq, k), dtype=torch.float32, device="cuda")
        S = torch.empty((nq, k), dtype=torch.float64, device="cuda") if return_scores else None
        ql = None
        if labels is not None:
            _need(bool(self.core.info().has_labels), "the index has no labels")
            ql = _as_torch(labels)[0].reshape(-1).to(device="cuda", dtype=torch.int32).contiguous()
            _need(ql.shape[0] == nq, "one label per query")
        flt, words = L.Filter(None, L.NO_FILTER), None
        if filter is not None:
            m = _as_torch(filter)[0].to(torch.bool)
            _need(m.shape[-1] == size, "the filter needs one entry per id")
            _need(m.ndim == 1 or (m.ndim == 2 and m.shape[0] == nq), "a mask over the ids, or one row per query")
            words = L.Tensor(pack_mask(m).view(torch.int32))
            words.m.dl_tensor.dtype = L.DLDataType(L.kDLUInt, 32, 1)
            flt = L.Filter(ctypes.cast(ctypes.pointer(words.m), ctypes.c_void_p), L.BITSET if m.ndim == 1 else L.BITMAP)
        if nq > 0:
            lib = L.lib()
            sp = ctypes.POINTER(L.SearchParams)()
            L.check(lib.cuvsCertexSearchParamsCreate(ctypes.byref(sp)))
            try:
                sp.contents.anchors, sp.contents.batch_size, sp.contents.probe_lists = int(anchors), int(batch), int(probe_lists)
                L.check(lib.certexB200SearchEx(
                    L.resources(), sp, self.core.handle, L.Tensor(Q).ref, None if ql is None else L.Tensor(ql).ref,
                    L.Tensor(I).ref, L.Tensor(D).ref, None if S is None else L.Tensor(S).ref, flt, int(id_base)))
            finally:
                lib.cuvsCertexSearchParamsDestroy(sp)
        if self.metric == "cosine":
            D = 1 - D  # similarity from the cosine distance; -inf where an entry is missing
        if single:
            D, I = D[0], I[0]
            S = None if S is None else S[0]
        out = (_like_input(D, kind), _like_input(I, kind))
        return out + (_like_input(S, kind),) if return_scores else out

    # ------------------------------------------------------------------ files
    def save(self, path):
        _need(self.core is not None, "add vectors first")
        L.check(L.lib().cuvsCertexSerialize(L.resources(), str(path).encode(), self.core.handle))

    @classmethod
    def load(cls, path):
        core = _Core()
        L.check(L.lib().cuvsCertexDeserialize(L.resources(), str(path).encode(), core.handle))
        i = core.info()
        idx = cls(int(i.dim), metric=L.METRIC_NAME[int(i.metric)], anchor_stride=int(i.anchor_stride))
        idx.core = core
        return idx

    def _test_mode(self, mode, cap=0):
        L.check(L.lib().certexB200IndexSetTestMode(self.core.handle, mode, cap))


def merge_shards(queries, part_scores, part_ids, metric="l2", return_scores=False):
    """Device merge of per-shard answers [parts, nq, k] by (exact score, id): (distances, ids[, scores])."""
    Q = queries.contiguous()
    P, nq, k = part_ids.shape
    I = torch.empty((nq, k), dtype=torch.int64, device="cuda")
    D = torch.empty((nq, k), dtype=torch.float32, device="cuda")
    S = torch.empty((nq, k), dtype=torch.float64, device="cuda")
    L.check(L.lib().certexB200MergeShards(
        L.resources(), L.METRIC_CODE[metric], L.Tensor(Q).ref, L.Tensor(part_scores.contiguous()).ref,
        L.Tensor(part_ids.contiguous()).ref, L.Tensor(I).ref, L.Tensor(D).ref, L.Tensor(S).ref))
    if metric == "cosine":
        D = 1 - D
    return (D, I, S) if return_scores else (D, I)


class ShardedIndex:
    """Exact k-NN over several GPUs of one process: contiguous row shards, one index per device, shard s owning the
    ids [n s / S, n (s + 1) / S) (the reference's ShardedIndex, certex/index.py:400-457). The library runs one host
    thread per shard, so the GPUs build and search at the same time; every shard computes its exact local top-k and
    the lists are merged by (score, id) on the first device. The vectors and the queries are host arrays; results are
    numpy arrays. For one process per GPU use `DistributedIndex`."""

    def __init__(self, dim, devices, metric="l2", width="auto", storage="device", anchor_stride=16, n_lists=0,
                 local_projections=False):
        _need(metric in METRICS and storage in ("device", "host"), "unknown metric or storage")
        self.d, self.devices, self.metric = dim, list(devices), metric
        self.anchor_stride = anchor_stride
        self._handle, self._dtype, self._n = None, None, 0

    def __del__(self):
        if getattr(self, "_handle", None) is not None:
            L.lib().certexB200ShardedDestroy(self._handle)
            self._handle = None

    def add(self, x):
        _need(self._handle is None, "a sharded index is built by one addition")
        t, _ = _as_torch(x)
        _need(t.ndim == 2 and t.shape[1] == self.d and not t.is_cuda, "a host matrix (n, dim)")
        if t.dtype not in _INDEX_DTYPES or (self.metric == "cosine" and not t.dtype.is_floating_point):
            t = t.float()
        t = t.contiguous()
        params = L.IndexParams(metric=L.METRIC_CODE[self.metric], anchor_stride=self.anchor_stride)
        devices = (ctypes.c_int32 * len(self.devices))(*self.devices)
        handle = ctypes.c_void_p()
        L.check(L.lib().certexB200ShardedBuild(devices, len(self.devices), ctypes.byref(params), L.Tensor(t).ref,
                                               ctypes.byref(handle)))
        self._handle, self._dtype, self._n = handle, t.dtype, t.shape[0]
        return np.arange(self._n)

    @property
    def ntotal(self):
        return self._n

    def search(self, q, k=10, batch=2048, anchors=128, probe_lists=2):
        _need(self._handle is not None, "add vectors first")
        Q = _to_dtype(_as_torch(q)[0].cpu(), self._dtype).contiguous()
        _need(Q.ndim == 2 and Q.shape[1] == self.d, "queries must be a matrix (nq, dim)")
        I = torch.empty((Q.shape[0], k), dtype=torch.int64)
        D = torch.empty((Q.shape[0], k), dtype=torch.float32)
        sp = L.SearchParams(anchors, batch, probe_lists)
        L.check(L.lib().certexB200ShardedSearch(ctypes.byref(sp), self._handle, L.Tensor(Q).ref, L.Tensor(I).ref,
                                                L.Tensor(D).ref))
        if self.metric == "cosine":
            D = 1 - D
        return D.numpy(), I.numpy()


def search(xb, xq=None, k=10, metric="l2", **index_options):
    """The exact k nearest neighbours in one call: (distances or similarities, ids), best first; without xq every
    vector of xb is a query. Results come back in the array type of the queries."""
    X, _ = _as_torch(xb)
    _need(X.ndim == 2, "xb must be a matrix (n, dim)")
    index = Index(dim=X.shape[1], metric=metric, **index_options)
    index.add(X)
    return index.search(xb if xq is None else xq, k=k)


def verify(xb, xq, I, metric="l2", sample=100, seed=0):
    """Fraction of (sampled) queries whose returned ids carry exactly the k smallest exact scores. The check re-derives
    the exact top-k of the sampled queries with the unscreened dense path of the engine (every stored vector scored in
    fp64) and compares the sorted scores of the given ids with it; ties count as exact whichever tied vector was
    returned, ids of -1 count as missing."""
    _need(metric in METRICS, f"metric must be one of {METRICS}, not {metric!r}")
    X, _ = _as_torch(xb)
    Q, _ = _as_torch(xq)
    ids, _ = _as_torch(I)
    if Q.ndim == 1:
        Q, ids = Q.reshape(1, -1), ids.reshape(1, -1)
    _need(X.ndim == 2 and Q.ndim == 2 and Q.shape[1] == X.shape[1], "xb and xq need the same dimension")
    _need(ids.shape[0] == Q.shape[0], "one row of ids per query")
    nq, k = ids.shape
    pick = torch.arange(nq) if sample is None or sample >= nq else torch.randperm(
        nq, generator=torch.Generator().manual_seed(seed))[:sample]
    index = Index(X.shape[1], metric=metric)
    index.add(X)
    Qs = _to_dtype(Q[pick.to(Q.device)].cuda(), index.dtype)
    got = ids[pick.to(ids.device)].cuda().long()
    index._test_mode(1)
    _, _, best = index.search(Qs, k=k, return_scores=True)
    # exact scores of the given ids: search restricted, per query, to exactly those ids
    n = X.shape[0]
    mask = torch.zeros((Qs.shape[0], n), dtype=torch.bool, device="cuda")
    rows = torch.arange(Qs.shape[0], device="cuda")[:, None].expand_as(got)
    valid = got >= 0
    mask[rows[valid], got[valid]] = True
    _, _, mine = index.search(Qs, k=k, filter=mask, return_scores=True)
    tol = 1e-9 * best.abs().amax(1, keepdim=True).clamp_min(1e-30)
    same = ((mine - best).abs() <= tol) | (torch.isinf(mine) & torch.isinf(best))
    return float(same.all(1).float().mean())
