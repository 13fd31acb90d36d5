"""ctypes binding of the C ABI (include/certex_b200.h). Tensors cross the boundary as DLPack `DLManagedTensor`
structures that point at the torch tensor's memory (zero copy); the library borrows them for the duration of the call.

There is no fallback: if the shared library is missing or a GPU call fails, an exception is raised.
"""

import ctypes
import os
import threading

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
# CERTEX_B200_LIB names another build of the same library (the trace build of the tensor-core pass, for profiling)
LIB_PATH = os.environ.get("CERTEX_B200_LIB") or os.path.join(_HERE, "lib", "libcertex_b200.so")

CUVS_SUCCESS = 1
L2Expanded, CosineExpanded, InnerProduct = 0, 2, 6
METRIC_CODE = {"l2": L2Expanded, "cosine": CosineExpanded, "ip": InnerProduct}
METRIC_NAME = {v: k for k, v in METRIC_CODE.items()}
NO_FILTER, BITSET, BITMAP = 0, 1, 2

kDLCPU, kDLCUDA, kDLCUDAHost = 1, 2, 3
kDLInt, kDLUInt, kDLFloat = 0, 1, 2


class DLDevice(ctypes.Structure):
    _fields_ = [("device_type", ctypes.c_int), ("device_id", ctypes.c_int32)]


class DLDataType(ctypes.Structure):
    _fields_ = [("code", ctypes.c_uint8), ("bits", ctypes.c_uint8), ("lanes", ctypes.c_uint16)]


class DLTensor(ctypes.Structure):
    _fields_ = [
        ("data", ctypes.c_void_p),
        ("device", DLDevice),
        ("ndim", ctypes.c_int32),
        ("dtype", DLDataType),
        ("shape", ctypes.POINTER(ctypes.c_int64)),
        ("strides", ctypes.POINTER(ctypes.c_int64)),
        ("byte_offset", ctypes.c_uint64),
    ]


class DLManagedTensor(ctypes.Structure):
    _fields_ = [("dl_tensor", DLTensor), ("manager_ctx", ctypes.c_void_p), ("deleter", ctypes.c_void_p)]


class IndexParams(ctypes.Structure):
    _fields_ = [
        ("metric", ctypes.c_int),
        ("width", ctypes.c_int32),
        ("variance", ctypes.c_double),
        ("anchor_stride", ctypes.c_int32),
        ("pca_sample", ctypes.c_int64),
        ("host_vectors", ctypes.c_bool),
        ("n_lists", ctypes.c_int32),
        ("local_projections", ctypes.c_bool),
        ("int8_rows", ctypes.c_bool),
    ]


class SearchParams(ctypes.Structure):
    _fields_ = [("anchors", ctypes.c_int32), ("batch_size", ctypes.c_int32), ("probe_lists", ctypes.c_int32)]


class IndexHandle(ctypes.Structure):
    _fields_ = [("addr", ctypes.c_void_p), ("dtype", DLDataType)]


class Filter(ctypes.Structure):
    _fields_ = [("addr", ctypes.c_void_p), ("type", ctypes.c_int)]


class IndexInfo(ctypes.Structure):
    _fields_ = [
        ("size", ctypes.c_int64),
        ("dim", ctypes.c_int64),
        ("capacity", ctypes.c_int64),
        ("n_removed", ctypes.c_int64),
        ("metric", ctypes.c_int32),
        ("anchor_stride", ctypes.c_int32),
        ("has_labels", ctypes.c_int32),
        ("integer_screen", ctypes.c_int32),
        ("row_pitch_bytes", ctypes.c_int64),
        ("n_partitioned", ctypes.c_int64),
    ]


_DT = {
    torch.float32: (kDLFloat, 32),
    torch.float16: (kDLFloat, 16),
    torch.float64: (kDLFloat, 64),
    torch.int8: (kDLInt, 8),
    torch.uint8: (kDLUInt, 8),
    torch.int32: (kDLInt, 32),
    torch.int64: (kDLInt, 64),
}

# every symbol include/certex_b200.h declares
SYMBOLS = [
    "cuvsResourcesCreate", "cuvsResourcesDestroy", "cuvsStreamSet", "cuvsStreamGet", "cuvsStreamSync",
    "cuvsGetLastErrorText", "cuvsSetLastErrorText",
    "cuvsCertexIndexParamsCreate", "cuvsCertexIndexParamsDestroy", "cuvsCertexSearchParamsCreate",
    "cuvsCertexSearchParamsDestroy", "cuvsCertexIndexCreate", "cuvsCertexIndexDestroy", "cuvsCertexIndexGetSize",
    "cuvsCertexIndexGetDim", "cuvsCertexBuild", "cuvsCertexExtend", "cuvsCertexRemove", "cuvsCertexSetLabels",
    "cuvsCertexPartitionByLabels", "cuvsCertexSearch", "cuvsCertexSearchWithLabels", "cuvsCertexSerialize",
    "cuvsCertexDeserialize",
    "certexB200SearchEx", "certexB200MergeShards", "certexB200IndexGetInfo", "certexB200IndexReserve",
    "certexB200StatsBegin", "certexB200StatsEnd", "certexB200IndexSetTestMode", "certexB200ScreenRaw",
    "certexB200PlanSegments", "certexB200SearchStatic", "certexB200Version",
    "certexB200SetThresholdHook", "certexB200IndexWillScreen", "certexB200PlanRouted",
    "certexB200ShardedBuild", "certexB200ShardedDestroy", "certexB200ShardedGetSize", "certexB200ShardedSearch",
    "certexB200CommGetUniqueId", "certexB200CommInitRank", "certexB200CommAdopt", "certexB200CommDestroy",
    "certexB200DistributedSearch", "certexB200ScreenTrace", "certexB200PlanChunked",
    "certexB200DistributedSearchBegin", "certexB200DistributedSearchEnd", "certexB200OrderByLabel",
]

# void hook(void* ctx, int32_t* keys, int64_t n, cudaStream_t stream)
ThresholdHook = ctypes.CFUNCTYPE(None, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64, ctypes.c_void_p)

_lib = None
_lock = threading.Lock()
_tls = threading.local()


def lib():
    """The loaded shared library; raises if it has not been built (python -c 'import __graft_entry__ as g; g.build()')."""
    global _lib
    if _lib is None:
        with _lock:
            if _lib is None:
                if not os.path.exists(LIB_PATH):
                    raise RuntimeError(
                        f"{LIB_PATH} is missing: build it with `make -C {os.path.join(_HERE, 'csrc')}`; "
                        "there is no CPU or PyTorch fallback"
                    )
                L = ctypes.CDLL(LIB_PATH)
                P = ctypes.POINTER
                vp, i64 = ctypes.c_void_p, ctypes.c_int64
                mt = P(DLManagedTensor)
                L.cuvsGetLastErrorText.restype = ctypes.c_char_p
                L.certexB200Version.restype = ctypes.c_char_p
                L.cuvsResourcesCreate.argtypes = [P(vp)]
                L.cuvsResourcesDestroy.argtypes = [vp]
                L.cuvsStreamSet.argtypes = [vp, vp]
                L.cuvsStreamGet.argtypes = [vp, P(vp)]
                L.cuvsStreamSync.argtypes = [vp]
                L.cuvsCertexIndexParamsCreate.argtypes = [P(P(IndexParams))]
                L.cuvsCertexIndexParamsDestroy.argtypes = [P(IndexParams)]
                L.cuvsCertexSearchParamsCreate.argtypes = [P(P(SearchParams))]
                L.cuvsCertexSearchParamsDestroy.argtypes = [P(SearchParams)]
                L.cuvsCertexIndexCreate.argtypes = [P(P(IndexHandle))]
                L.cuvsCertexIndexDestroy.argtypes = [P(IndexHandle)]
                L.cuvsCertexIndexGetSize.argtypes = [P(IndexHandle), P(i64)]
                L.cuvsCertexIndexGetDim.argtypes = [P(IndexHandle), P(i64)]
                L.cuvsCertexBuild.argtypes = [vp, P(IndexParams), mt, P(IndexHandle)]
                L.cuvsCertexExtend.argtypes = [vp, mt, P(IndexHandle)]
                L.cuvsCertexRemove.argtypes = [vp, mt, P(IndexHandle)]
                L.cuvsCertexSetLabels.argtypes = [vp, mt, i64, P(IndexHandle)]
                L.cuvsCertexPartitionByLabels.argtypes = [vp, P(IndexHandle)]
                L.cuvsCertexSearch.argtypes = [vp, P(SearchParams), P(IndexHandle), mt, mt, mt, Filter]
                L.cuvsCertexSearchWithLabels.argtypes = [vp, P(SearchParams), P(IndexHandle), mt, mt, mt, mt]
                L.cuvsCertexSerialize.argtypes = [vp, ctypes.c_char_p, P(IndexHandle)]
                L.cuvsCertexDeserialize.argtypes = [vp, ctypes.c_char_p, P(IndexHandle)]
                L.certexB200SearchEx.argtypes = [vp, P(SearchParams), P(IndexHandle), mt, mt, mt, mt, mt, Filter, i64]
                L.certexB200MergeShards.argtypes = [vp, ctypes.c_int, mt, mt, mt, mt, mt, mt]
                L.certexB200IndexGetInfo.argtypes = [P(IndexHandle), P(IndexInfo)]
                L.certexB200IndexReserve.argtypes = [vp, P(IndexHandle), i64]
                L.certexB200StatsBegin.argtypes = []
                L.certexB200StatsEnd.argtypes = [P(ctypes.c_uint64)]
                L.certexB200IndexSetTestMode.argtypes = [P(IndexHandle), ctypes.c_int32, ctypes.c_int32]
                L.certexB200SetThresholdHook.argtypes = [ThresholdHook, vp]
                L.certexB200IndexWillScreen.argtypes = [P(IndexHandle), ctypes.c_int32, P(ctypes.c_int32)]
                L.certexB200ScreenRaw.argtypes = [
                    vp, vp, i64, vp, i64, i64, ctypes.c_int32, vp, ctypes.c_int32, vp, vp, i64, vp, vp,
                    ctypes.c_uint32, P(ctypes.c_float),
                ]
                L.certexB200PlanSegments.argtypes = [ctypes.c_int32] * 4 + [P(ctypes.c_int32)]
                L.certexB200PlanChunked.argtypes = [ctypes.c_int32] * 5 + [P(ctypes.c_int32), ctypes.c_int32,
                                                                           P(ctypes.c_int32), P(ctypes.c_int32)]
                L.certexB200PlanRouted.argtypes = [ctypes.c_int32, P(ctypes.c_int32), P(ctypes.c_int32), ctypes.c_int32,
                                                   ctypes.c_int32, ctypes.c_int32, P(ctypes.c_int32), ctypes.c_int32,
                                                   P(ctypes.c_int32), P(ctypes.c_int32), P(ctypes.c_int32)]
                L.certexB200ShardedBuild.argtypes = [P(ctypes.c_int32), ctypes.c_int32, P(IndexParams), mt, P(vp)]
                L.certexB200ShardedDestroy.argtypes = [vp]
                L.certexB200ShardedGetSize.argtypes = [vp, P(i64)]
                L.certexB200ShardedSearch.argtypes = [P(SearchParams), vp, mt, mt, mt]
                L.certexB200CommGetUniqueId.argtypes = [vp]
                L.certexB200CommInitRank.argtypes = [vp, ctypes.c_int32, ctypes.c_int32, P(vp)]
                L.certexB200CommAdopt.argtypes = [vp, P(vp)]
                L.certexB200CommDestroy.argtypes = [vp]
                L.certexB200DistributedSearch.argtypes = [vp, vp, P(SearchParams), P(IndexHandle), mt, mt, mt, mt, i64,
                                                          ctypes.c_int32]
                L.certexB200DistributedSearchBegin.argtypes = [vp, vp, P(SearchParams), P(IndexHandle), mt, mt, mt, mt, i64,
                                                               ctypes.c_int32, P(vp)]
                L.certexB200DistributedSearchEnd.argtypes = [vp]
                L.certexB200ScreenTrace.argtypes = [vp, ctypes.c_int32]
                L.certexB200OrderByLabel.argtypes = [P(ctypes.c_int32), i64, P(ctypes.c_int32)]
                L.certexB200SearchStatic.argtypes = [vp, ctypes.c_int, DLDataType, vp, i64, vp, i64, i64, ctypes.c_int32, vp, vp]
                _lib = L
    return _lib


class CertexError(RuntimeError):
    pass


def check(status):
    if status != CUVS_SUCCESS:
        text = lib().cuvsGetLastErrorText()
        raise CertexError(text.decode() if text else "certex: unknown error")


class Tensor:
    """A DLManagedTensor that borrows a torch tensor (kept alive by this object)."""

    def __init__(self, t):
        if not t.is_contiguous():
            raise ValueError("tensors must be contiguous")
        self.t = t
        self.shape = (ctypes.c_int64 * max(t.ndim, 1))(*t.shape)
        m = DLManagedTensor()
        m.dl_tensor.data = t.data_ptr()
        if t.is_cuda:
            m.dl_tensor.device = DLDevice(kDLCUDA, t.device.index or 0)
        else:
            m.dl_tensor.device = DLDevice(kDLCUDAHost if t.is_pinned() else kDLCPU, 0)
        m.dl_tensor.ndim = t.ndim
        code, bits = _DT[t.dtype]
        m.dl_tensor.dtype = DLDataType(code, bits, 1)
        m.dl_tensor.shape = ctypes.cast(self.shape, ctypes.POINTER(ctypes.c_int64))
        m.dl_tensor.strides = None
        m.dl_tensor.byte_offset = 0
        m.manager_ctx = None
        m.deleter = None
        self.m = m

    @property
    def ref(self):
        return ctypes.byref(self.m)


def resources():
    """The resources handle of the calling thread for the current CUDA device, bound to torch's current stream."""
    dev = torch.cuda.current_device()
    cache = getattr(_tls, "res", None)
    if cache is None:
        cache = _tls.res = {}
    if dev not in cache:
        h = ctypes.c_void_p()
        check(lib().cuvsResourcesCreate(ctypes.byref(h)))
        cache[dev] = h
    h = cache[dev]
    check(lib().cuvsStreamSet(h, ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)))
    return h
