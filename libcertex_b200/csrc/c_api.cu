// C ABI of the library (include/certex_b200.h): argument checks, DLPack unwrapping and exception translation over
// the engine. Mirrors the reference's c/src/neighbors/certex.cpp, c/src/core/interop.hpp and c/src/core/exceptions.hpp.
#include "../../include/certex_b200.h"

#include "engine.hpp"
#include "screen_i8.cuh"

#include <cuda.h>

#include <algorithm>
#include <exception>
#include <fstream>
#include <memory>
#include <string>
#include <thread>
#include <vector>

namespace {

using namespace certex_b200;

thread_local std::string g_last_error;
thread_local SearchStats g_stats;

template <typename F>
cuvsError_t translate(F&& f)
{
  try {
    f();
    return CUVS_SUCCESS;
  } catch (const std::exception& e) {
    g_last_error = e.what();
  } catch (...) {
    g_last_error = "certex: unknown error";
  }
  return CUVS_ERROR;
}

struct Holder {
  std::unique_ptr<Index> index;
};

Resources& as_res(cuvsResources_t r)
{
  CERTEX_EXPECTS(r != 0, "certex: null resources handle");
  return *reinterpret_cast<Resources*>(r);
}

Holder& as_holder(cuvsCertexIndex_t index)
{
  CERTEX_EXPECTS(index != nullptr && index->addr != 0, "certex: the index is empty (build or deserialize it first)");
  return *reinterpret_cast<Holder*>(index->addr);
}

int metric_of(int m)
{
  switch (m) {
    case L2Expanded: return kL2;
    case InnerProduct: return kIP;
    case CosineExpanded: return kCos;
    default: throw Error("certex: the metric must be L2Expanded, InnerProduct, or CosineExpanded");
  }
}

int metric_back(int m) { return m == kL2 ? L2Expanded : m == kIP ? InnerProduct : CosineExpanded; }

int dtype_of(DLDataType t)
{
  CERTEX_EXPECTS(t.lanes == 1, "certex: the DLPack tensor must have one lane");
  if (t.code == kDLFloat && t.bits == 32) { return kF32; }
  if (t.code == kDLFloat && t.bits == 16) { return kF16; }
  if (t.code == kDLInt && t.bits == 8) { return kI8; }
  if (t.code == kDLUInt && t.bits == 8) { return kU8; }
  throw Error("certex: vectors must be float32, float16, int8, or uint8");
}

bool on_device(const DLTensor& t) { return t.device.device_type == kDLCUDA || t.device.device_type == kDLCUDAManaged; }
bool on_host(const DLTensor& t) { return t.device.device_type == kDLCPU || t.device.device_type == kDLCUDAHost; }

/// Dense row-major tensor of the given rank and element type; returns the data pointer with byte_offset applied.
void* checked(DLManagedTensor* m, int ndim, int code, int bits, bool device, const char* what)
{
  CERTEX_EXPECTS(m != nullptr, std::string("certex: null tensor for ") + what);
  const DLTensor& t = m->dl_tensor;
  CERTEX_EXPECTS(t.ndim == ndim, std::string("certex: ") + what + " has the wrong number of dimensions");
  CERTEX_EXPECTS(t.dtype.lanes == 1 && (code < 0 || (t.dtype.code == code && t.dtype.bits == bits)),
                 std::string("certex: ") + what + " has the wrong data type");
  if (device) {
    CERTEX_EXPECTS(on_device(t), std::string("certex: expected ") + what + " in device memory");
  }
  if (t.strides != nullptr) {
    int64_t expect = 1;
    for (int i = ndim - 1; i >= 0; --i) {
      CERTEX_EXPECTS(t.shape[i] == 1 || t.strides[i] == expect, "certex: the DLPack tensor must be dense and row major");
      expect *= t.shape[i];
    }
  }
  return static_cast<char*>(t.data) + t.byte_offset;
}

Filter filter_of(const cuvsFilter& f, int64_t nq, int64_t size)
{
  Filter out;
  if (f.type == NO_FILTER) { return out; }
  CERTEX_EXPECTS(f.type == BITSET || f.type == BITMAP, "certex: unsupported filter type");
  auto* words_t = reinterpret_cast<DLManagedTensor*>(f.addr);
  out.words     = static_cast<const uint32_t*>(checked(words_t, 1, kDLUInt, 32, true, "the filter words"));
  const int64_t have = words_t->dl_tensor.shape[0];
  // the index may grow between this look at its size and the search's own (taken under its reader lock): the search
  // checks covered_ids against the size it works with
  if (f.type == BITSET) {
    CERTEX_EXPECTS(have * 32 >= size, "certex: the bitset must cover every id of the index");
    out.covered_ids = have * 32;
  } else {
    out.bitmap_cols = size;
    out.covered_ids = size;
    CERTEX_EXPECTS(have * 32 >= nq * size, "certex: the bitmap must hold one row of size() bits per query");
  }
  return out;
}

void search_impl(cuvsResources_t res, cuvsCertexSearchParams_t params, cuvsCertexIndex_t index, DLManagedTensor* queries,
                 DLManagedTensor* query_labels, DLManagedTensor* neighbors, DLManagedTensor* distances,
                 DLManagedTensor* scores, cuvsFilter filter, int64_t id_base)
{
  Resources& r = as_res(res);
  Holder& h    = as_holder(index);
  CERTEX_EXPECTS(params != nullptr, "certex: null search parameters");
  CERTEX_EXPECTS(queries != nullptr && queries->dl_tensor.dtype.code == index->dtype.code &&
                   queries->dl_tensor.dtype.bits == index->dtype.bits,
                 "certex: the queries must have the vector type of the index");
  const void* q = checked(queries, 2, -1, 0, true, "the queries");
  const int64_t nq = queries->dl_tensor.shape[0];
  CERTEX_EXPECTS(queries->dl_tensor.shape[1] == h.index->dim(), "certex: the queries must have the dimension of the index");
  auto* nb = static_cast<int64_t*>(checked(neighbors, 2, kDLInt, 64, true, "the neighbors"));
  auto* ds = static_cast<float*>(checked(distances, 2, kDLFloat, 32, true, "the distances"));
  const int64_t k = neighbors->dl_tensor.shape[1];
  CERTEX_EXPECTS(neighbors->dl_tensor.shape[0] == nq && distances->dl_tensor.shape[0] == nq &&
                   distances->dl_tensor.shape[1] == k,
                 "certex: neighbors and distances must be [n_queries, k]");
  double* sc = nullptr;
  if (scores) {
    sc = static_cast<double*>(checked(scores, 2, kDLFloat, 64, true, "the scores"));
    CERTEX_EXPECTS(scores->dl_tensor.shape[0] == nq && scores->dl_tensor.shape[1] == k, "certex: scores must be [n_queries, k]");
  }
  Filter f = filter_of(filter, nq, h.index->size());
  if (query_labels) {
    f.query_labels = static_cast<const int32_t*>(checked(query_labels, 1, kDLInt, 32, true, "the query labels"));
    CERTEX_EXPECTS(query_labels->dl_tensor.shape[0] == nq, "certex: one label per query");
  }
  SearchParams sp;
  sp.anchors     = params->anchors;
  sp.batch_size  = params->batch_size;
  sp.probe_lists = params->probe_lists;
  CERTEX_EXPECTS(k >= 1 && k <= 2048, "certex: k must be between 1 and 2048");
  h.index->search(r, sp, q, nq, static_cast<int>(k), nb, ds, sc, f, id_base);
}

// ------------------------------------------------------------------------------------------- row shards on several GPUs
/// One row shard: a device, a stream on it and the index of the shard's rows.
struct Shard {
  int device = 0;
  Resources res;
  std::unique_ptr<Index> index;
  int64_t first_id = 0;
  Shard()                        = default;
  Shard(const Shard&)            = delete;
  Shard& operator=(const Shard&) = delete;
  ~Shard()
  {
    int old = 0;
    cudaGetDevice(&old);
    cudaSetDevice(device);
    index.reset();
    if (res.stream) { cudaStreamDestroy(res.stream); }
    cudaSetDevice(old);
  }
};

/// Restores the calling thread's current device when it goes out of scope.
struct DeviceGuard {
  int old = 0;
  DeviceGuard() { CERTEX_CUDA(cudaGetDevice(&old)); }
  ~DeviceGuard() { cudaSetDevice(old); }
};

/// Runs work(s) for every shard on a host thread of its own (the GPUs work at the same time, as in the reference's
/// cpp/src/neighbors/certex/certex_shards.cu:105-135) and rethrows the first failure.
template <typename Work>
void for_each_shard(size_t n_shards, Work&& work)
{
  std::vector<std::exception_ptr> failed(n_shards);
  std::vector<std::thread> threads;
  for (size_t s = 0; s < n_shards; ++s) {
    threads.emplace_back([&, s] {
      try {
        work(s);
      } catch (...) {
        failed[s] = std::current_exception();
      }
    });
  }
  for (auto& t : threads) { t.join(); }
  for (auto& f : failed) {
    if (f) { std::rethrow_exception(f); }
  }
}

/// Device memory of one call from the stream's pool.
struct PoolBuffer {
  void* p = nullptr;
  cudaStream_t stream;
  PoolBuffer(size_t bytes, cudaStream_t s) : stream(s) { CERTEX_CUDA(cudaMallocAsync(&p, std::max<size_t>(bytes, 16), s)); }
  ~PoolBuffer() { cudaFreeAsync(p, stream); }
  PoolBuffer(const PoolBuffer&)            = delete;
  PoolBuffer& operator=(const PoolBuffer&) = delete;
};

const char* prefix_of(int dtype)
{
  switch (dtype) {
    case kF32: return "<f4";
    case kF16: return "<f2";
    case kI8: return "|i1";
    default: return "|u1";
  }
}

}  // namespace

extern "C" {

const char* cuvsGetLastErrorText(void) { return g_last_error.empty() ? nullptr : g_last_error.c_str(); }
void cuvsSetLastErrorText(const char* text) { g_last_error = text ? text : ""; }

cuvsError_t cuvsResourcesCreate(cuvsResources_t* res)
{
  return translate([=] {
    CERTEX_EXPECTS(res != nullptr, "certex: null pointer");
    *res = reinterpret_cast<cuvsResources_t>(new Resources());
  });
}

cuvsError_t cuvsResourcesDestroy(cuvsResources_t res)
{
  return translate([=] { delete reinterpret_cast<Resources*>(res); });
}

cuvsError_t cuvsStreamSet(cuvsResources_t res, void* stream)
{
  return translate([=] { as_res(res).stream = static_cast<cudaStream_t>(stream); });
}

cuvsError_t cuvsStreamGet(cuvsResources_t res, void** stream)
{
  return translate([=] { *stream = as_res(res).stream; });
}

cuvsError_t cuvsStreamSync(cuvsResources_t res)
{
  return translate([=] { as_res(res).sync(); });
}

cuvsError_t cuvsCertexIndexParamsCreate(cuvsCertexIndexParams_t* params)
{
  return translate([=] {
    const IndexParams d;
    *params = new cuvsCertexIndexParams{static_cast<cuvsDistanceType>(metric_back(d.metric)),
                                        d.width,
                                        d.variance,
                                        d.anchor_stride,
                                        d.pca_sample,
                                        d.host_vectors,
                                        d.n_lists,
                                        d.local_projections,
                                        d.int8_rows};
  });
}

cuvsError_t cuvsCertexIndexParamsDestroy(cuvsCertexIndexParams_t params)
{
  return translate([=] { delete params; });
}

cuvsError_t cuvsCertexSearchParamsCreate(cuvsCertexSearchParams_t* params)
{
  return translate([=] {
    const SearchParams d;
    *params = new cuvsCertexSearchParams{d.anchors, d.batch_size, d.probe_lists};
  });
}

cuvsError_t cuvsCertexSearchParamsDestroy(cuvsCertexSearchParams_t params)
{
  return translate([=] { delete params; });
}

cuvsError_t cuvsCertexIndexCreate(cuvsCertexIndex_t* index)
{
  return translate([=] { *index = new cuvsCertexIndex{}; });
}

cuvsError_t cuvsCertexIndexDestroy(cuvsCertexIndex_t index)
{
  return translate([=] {
    if (index == nullptr) { return; }
    if (index->addr != 0) { delete reinterpret_cast<Holder*>(index->addr); }
    delete index;
  });
}

cuvsError_t cuvsCertexIndexGetSize(cuvsCertexIndex_t index, int64_t* size)
{
  return translate([=] { *size = as_holder(index).index->size(); });
}

cuvsError_t cuvsCertexIndexGetDim(cuvsCertexIndex_t index, int64_t* dim)
{
  return translate([=] { *dim = as_holder(index).index->dim(); });
}

cuvsError_t cuvsCertexBuild(cuvsResources_t res, cuvsCertexIndexParams_t params, DLManagedTensor* dataset,
                            cuvsCertexIndex_t index)
{
  return translate([=] {
    Resources& r = as_res(res);
    CERTEX_EXPECTS(index != nullptr && index->addr == 0, "certex: the index handle already holds an index");
    CERTEX_EXPECTS(params != nullptr, "certex: null index parameters");
    const void* x     = checked(dataset, 2, -1, 0, false, "the dataset");
    const DLTensor& t = dataset->dl_tensor;
    CERTEX_EXPECTS(on_device(t) || on_host(t), "certex: the dataset must be in device or host memory");
    const int dtype = dtype_of(t.dtype);
    IndexParams p;
    p.metric            = metric_of(params->metric);
    p.width             = params->width;
    p.variance          = params->variance;
    p.anchor_stride     = params->anchor_stride;
    p.pca_sample        = params->pca_sample;
    p.host_vectors      = params->host_vectors;
    p.n_lists           = params->n_lists;
    p.local_projections = params->local_projections;
    p.int8_rows         = params->int8_rows;
    CERTEX_EXPECTS(t.shape[0] >= 1, "certex: the dataset is empty");
    auto holder   = std::make_unique<Holder>();
    holder->index = std::make_unique<Index>(r, p, dtype, t.shape[1]);
    holder->index->extend(r, x, t.shape[0], on_host(t));
    index->dtype = t.dtype;
    index->addr  = reinterpret_cast<uintptr_t>(holder.release());
  });
}

cuvsError_t cuvsCertexExtend(cuvsResources_t res, DLManagedTensor* new_vectors, cuvsCertexIndex_t index)
{
  return translate([=] {
    Resources& r      = as_res(res);
    Holder& h         = as_holder(index);
    const void* x     = checked(new_vectors, 2, index->dtype.code, index->dtype.bits, false, "the new vectors");
    const DLTensor& t = new_vectors->dl_tensor;
    CERTEX_EXPECTS(on_device(t) || on_host(t), "certex: the vectors must be in device or host memory");
    CERTEX_EXPECTS(t.shape[1] == h.index->dim(), "certex: the new vectors must have the dimension of the index");
    h.index->extend(r, x, t.shape[0], on_host(t));
  });
}

cuvsError_t cuvsCertexRemove(cuvsResources_t res, DLManagedTensor* ids, cuvsCertexIndex_t index)
{
  return translate([=] {
    Resources& r = as_res(res);
    Holder& h    = as_holder(index);
    auto* p      = static_cast<const int64_t*>(checked(ids, 1, kDLInt, 64, true, "the ids"));
    h.index->remove(r, p, ids->dl_tensor.shape[0]);
  });
}

cuvsError_t cuvsCertexSetLabels(cuvsResources_t res, DLManagedTensor* labels, int64_t first, cuvsCertexIndex_t index)
{
  return translate([=] {
    Resources& r = as_res(res);
    Holder& h    = as_holder(index);
    auto* p      = static_cast<const int32_t*>(checked(labels, 1, kDLInt, 32, true, "the labels"));
    h.index->set_labels(r, p, labels->dl_tensor.shape[0], first);
  });
}

cuvsError_t cuvsCertexPartitionByLabels(cuvsResources_t res, cuvsCertexIndex_t index)
{
  return translate([=] {
    Resources& r = as_res(res);
    Holder& h    = as_holder(index);
    h.index->partition_by_labels(r);
  });
}

cuvsError_t cuvsCertexSearch(cuvsResources_t res, cuvsCertexSearchParams_t params, cuvsCertexIndex_t index,
                             DLManagedTensor* queries, DLManagedTensor* neighbors, DLManagedTensor* distances,
                             cuvsFilter filter)
{
  return translate([=] { search_impl(res, params, index, queries, nullptr, neighbors, distances, nullptr, filter, 0); });
}

cuvsError_t cuvsCertexSearchWithLabels(cuvsResources_t res, cuvsCertexSearchParams_t params, cuvsCertexIndex_t index,
                                       DLManagedTensor* queries, DLManagedTensor* query_labels,
                                       DLManagedTensor* neighbors, DLManagedTensor* distances)
{
  return translate([=] {
    CERTEX_EXPECTS(query_labels != nullptr, "certex: null query labels");
    cuvsFilter none{0, NO_FILTER};
    search_impl(res, params, index, queries, query_labels, neighbors, distances, nullptr, none, 0);
  });
}

cuvsError_t certexB200SearchEx(cuvsResources_t res, cuvsCertexSearchParams_t params, cuvsCertexIndex_t index,
                               DLManagedTensor* queries, DLManagedTensor* query_labels, DLManagedTensor* neighbors,
                               DLManagedTensor* distances, DLManagedTensor* scores, cuvsFilter filter, int64_t id_base)
{
  return translate([=] { search_impl(res, params, index, queries, query_labels, neighbors, distances, scores, filter, id_base); });
}

cuvsError_t cuvsCertexSerialize(cuvsResources_t res, const char* filename, cuvsCertexIndex_t index)
{
  return translate([=] {
    Resources& r = as_res(res);
    Holder& h    = as_holder(index);
    std::ofstream os(filename, std::ios::binary);
    CERTEX_EXPECTS(os.good(), "certex: cannot open the index file for writing");
    std::string prefix = prefix_of(h.index->dtype());
    prefix.resize(4, '\0');
    os << prefix;
    h.index->save(r, os);
  });
}

cuvsError_t cuvsCertexDeserialize(cuvsResources_t res, const char* filename, cuvsCertexIndex_t index)
{
  return translate([=] {
    Resources& r = as_res(res);
    CERTEX_EXPECTS(index != nullptr && index->addr == 0, "certex: the index handle already holds an index");
    std::ifstream is(filename, std::ios::binary);
    CERTEX_EXPECTS(is.good(), "certex: cannot open the index file");
    char prefix[4] = {};
    is.read(prefix, 4);
    const std::string d(prefix + 1, 2);
    DLDataType dt{};
    if (d == "f4") {
      dt = {kDLFloat, 32, 1};
    } else if (d == "f2") {
      dt = {kDLFloat, 16, 1};
    } else if (d == "i1") {
      dt = {kDLInt, 8, 1};
    } else if (d == "u1") {
      dt = {kDLUInt, 8, 1};
    } else {
      throw Error("certex: not a CertEx index file");
    }
    auto holder   = std::make_unique<Holder>();
    holder->index = Index::load(r, is, dtype_of(dt));
    index->dtype  = dt;
    index->addr   = reinterpret_cast<uintptr_t>(holder.release());
  });
}

cuvsError_t certexB200MergeShards(cuvsResources_t res, cuvsDistanceType metric, DLManagedTensor* queries,
                                  DLManagedTensor* part_scores, DLManagedTensor* part_ids, DLManagedTensor* neighbors,
                                  DLManagedTensor* distances, DLManagedTensor* scores)
{
  return translate([=] {
    Resources& r     = as_res(res);
    const void* q    = checked(queries, 2, -1, 0, true, "the queries");
    const int dtype  = dtype_of(queries->dl_tensor.dtype);
    auto* ps         = static_cast<const double*>(checked(part_scores, 3, kDLFloat, 64, true, "the shard scores"));
    auto* pi         = static_cast<const int64_t*>(checked(part_ids, 3, kDLInt, 64, true, "the shard ids"));
    auto* nb         = static_cast<int64_t*>(checked(neighbors, 2, kDLInt, 64, true, "the neighbors"));
    auto* ds         = static_cast<float*>(checked(distances, 2, kDLFloat, 32, true, "the distances"));
    double* sc       = scores ? static_cast<double*>(checked(scores, 2, kDLFloat, 64, true, "the scores")) : nullptr;
    const int64_t* s = part_scores->dl_tensor.shape;
    const int64_t nq = queries->dl_tensor.shape[0];
    CERTEX_EXPECTS(s[1] == nq && part_ids->dl_tensor.shape[0] == s[0] && part_ids->dl_tensor.shape[1] == nq &&
                     part_ids->dl_tensor.shape[2] == s[2] && neighbors->dl_tensor.shape[0] == nq &&
                     neighbors->dl_tensor.shape[1] == s[2] && distances->dl_tensor.shape[0] == nq &&
                     distances->dl_tensor.shape[1] == s[2],
                   "certex: shard answers must be [parts, n_queries, k] and the outputs [n_queries, k]");
    merge_shards(r, ps, pi, static_cast<int>(s[0]), static_cast<int>(nq), static_cast<int>(s[2]), q, dtype,
                 queries->dl_tensor.shape[1], metric_of(metric), nb, ds, sc);
  });
}

cuvsError_t certexB200IndexGetInfo(cuvsCertexIndex_t index, certexB200IndexInfo* info)
{
  return translate([=] {
    Holder& h             = as_holder(index);
    info->size            = h.index->size();
    info->dim             = h.index->dim();
    info->capacity        = h.index->capacity();
    info->n_removed       = h.index->n_removed();
    info->metric          = metric_back(h.index->metric());
    info->anchor_stride   = h.index->params().anchor_stride;
    info->has_labels      = h.index->has_labels() ? 1 : 0;
    info->integer_screen  = h.index->int_screen() ? 1 : 0;
    info->row_pitch_bytes = static_cast<int64_t>(h.index->pitch());
    info->n_partitioned   = h.index->n_partitioned();
  });
}

cuvsError_t certexB200IndexReserve(cuvsResources_t res, cuvsCertexIndex_t index, int64_t n_rows)
{
  return translate([=] { as_holder(index).index->reserve(as_res(res), n_rows); });
}

cuvsError_t certexB200StatsBegin(void)
{
  return translate([] {
    g_stats           = SearchStats{};
    Index::stats_sink = &g_stats;
  });
}

cuvsError_t certexB200StatsEnd(uint64_t out[16])
{
  return translate([=] {
    Index::stats_sink = nullptr;
    out[0] = g_stats.queries, out[1] = g_stats.survivors, out[2] = g_stats.verified, out[3] = g_stats.dense_queries;
    out[4] = g_stats.launches;
    out[5] = static_cast<uint64_t>(g_stats.screen_ms * 1000.0);
    out[6] = static_cast<uint64_t>(g_stats.anchor_ms * 1000.0);
    out[7] = g_stats.screen_passes;
    out[8] = g_stats.rescreened;
    out[9] = g_stats.routed_queries;
    out[10] = static_cast<uint64_t>(g_stats.span_ms * 1000.0);
    for (int i = 11; i < 16; ++i) { out[i] = 0; }
  });
}

cuvsError_t certexB200SetThresholdHook(certexB200ThresholdHook hook, void* ctx)
{
  return translate([=] {
    Index::threshold_hook     = reinterpret_cast<Index::ThresholdHook>(hook);
    Index::threshold_hook_ctx = ctx;
  });
}

cuvsError_t certexB200IndexWillScreen(cuvsCertexIndex_t index, int32_t k, int32_t* out)
{
  return translate([=] {
    CERTEX_EXPECTS(out != nullptr, "certex: out is null");
    *out = as_holder(index).index->will_screen(k) ? 1 : 0;
  });
}

cuvsError_t certexB200IndexSetTestMode(cuvsCertexIndex_t index, int32_t mode, int32_t cap)
{
  return translate([=] {
    CERTEX_EXPECTS(mode >= 0 && mode <= 5 && (mode != 2 || cap >= 1) && (mode != 4 || cap >= 0), "certex: unknown test mode");
    as_holder(index).index->set_test_mode(mode, cap);
  });
}

cuvsError_t certexB200ScreenRaw(cuvsResources_t res, const void* q_codes, int64_t nq, const void* x_codes, int64_t n,
                                int64_t code_len, int32_t is_signed, const int32_t* init, int32_t mode,
                                const int32_t* thr, int32_t* gmax, int64_t ld, uint32_t* cnt, int32_t* cand,
                                uint32_t cap, float* elapsed_ms)
{
  return translate([=] {
    Resources& r = as_res(res);
    CERTEX_EXPECTS(code_len >= 128 && code_len <= 4096 && code_len % 128 == 0, "certex: code_len must be a multiple of 128 up to 4096");
    CERTEX_EXPECTS(nq >= 1 && n >= 1 && n < (int64_t(1) << 31) && nq < (int64_t(1) << 24), "certex: sizes out of range");
    CERTEX_EXPECTS(mode >= 0 && mode <= 3, "certex: the mode is 0 (screen), 1 (group maxima), 2 (rate probe) or 3 (chained bound)");
    CERTEX_EXPECTS(is_signed >= 0 && is_signed <= 2, "certex: the code kind is 0 (uint8), 1 (int8) or 2 (float16)");
    screen_raw(r, q_codes, nq, x_codes, n, code_len, is_signed, init, mode, thr, gmax, ld, cnt, cand, cap, elapsed_ms);
  });
}

cuvsError_t certexB200ScreenTrace(void* trace, int32_t units)
{
  return translate([=] {
    CERTEX_EXPECTS(trace == nullptr || screen_trace_compiled(),
                   "certex: this library was built without the trace stamps of the tensor-core pass (make trace)");
    screen_set_trace(static_cast<long long*>(trace), units);
  });
}

cuvsError_t certexB200PlanSegments(int32_t n_query_tiles, int32_t n_base_tiles, int32_t panel_tiles, int32_t grid,
                                   int32_t* out)
{
  return translate([=] { plan_segments_flat(n_query_tiles, n_base_tiles, panel_tiles, grid, out); });
}

cuvsError_t certexB200PlanChunked(int32_t n_query_tiles, int32_t n_base_tiles, int32_t panel_tiles, int32_t grid,
                                  int32_t chunk_tiles, int32_t* segs, int32_t cap_segs, int32_t* n_segs, int32_t* seg_begin)
{
  return translate([=] {
    *n_segs = plan_chunked_flat(n_query_tiles, n_base_tiles, panel_tiles, grid, chunk_tiles, segs, cap_segs, seg_begin);
  });
}

cuvsError_t certexB200OrderByLabel(const int32_t* labels, int64_t n, int32_t* order)
{
  return translate([=] {
    CERTEX_EXPECTS(n >= 0 && (n == 0 || (labels != nullptr && order != nullptr)), "certex: null argument");
    order_by_label_flat(labels, n, order);
  });
}

cuvsError_t certexB200PlanRouted(int32_t n_runs, const int32_t* n_query_tiles, const int32_t* n_base_tiles,
                                 int32_t panel_tiles, int32_t grid, int32_t max_segs, int32_t* segs, int32_t cap_segs,
                                 int32_t* n_segs, int32_t* seg_begin, int32_t* runs_done)
{
  return translate([=] {
    *runs_done = plan_routed_flat(n_runs, n_query_tiles, n_base_tiles, panel_tiles, grid, max_segs, segs, cap_segs, n_segs,
                                  seg_begin);
  });
}

struct certexB200Sharded {
  std::vector<std::unique_ptr<Shard>> shards;
  int dtype   = 0;
  int64_t dim = 0;
  int metric  = kL2;
};

cuvsError_t certexB200ShardedBuild(const int32_t* devices, int32_t n_shards, cuvsCertexIndexParams_t params,
                                   DLManagedTensor* dataset, certexB200ShardedIndex_t* out)
{
  return translate([=] {
    CERTEX_EXPECTS(out != nullptr && devices != nullptr && n_shards >= 1, "certex: one device per shard, at least one");
    CERTEX_EXPECTS(params != nullptr, "certex: null index parameters");
    auto* x           = static_cast<const char*>(checked(dataset, 2, -1, 0, false, "the dataset"));
    const DLTensor& t = dataset->dl_tensor;
    CERTEX_EXPECTS(on_host(t), "certex: a sharded index is built from a host matrix");
    const int dtype  = dtype_of(t.dtype);
    const int64_t n  = t.shape[0], dim = t.shape[1];
    CERTEX_EXPECTS(n >= n_shards, "certex: fewer vectors than shards");
    IndexParams p;
    p.metric        = metric_of(params->metric);
    p.anchor_stride = params->anchor_stride;
    auto sharded    = std::make_unique<certexB200Sharded>();
    sharded->dtype  = dtype;
    sharded->dim    = dim;
    sharded->metric = p.metric;
    sharded->shards.resize(static_cast<size_t>(n_shards));
    const size_t row_bytes = static_cast<size_t>(dim) * (dtype == kF32 ? 4 : dtype == kF16 ? 2 : 1);
    for_each_shard(static_cast<size_t>(n_shards), [&](size_t s) {
      CERTEX_CUDA(cudaSetDevice(devices[s]));
      auto sh    = std::make_unique<Shard>();  // Resources() reads the device that is current now
      sh->device = devices[s];
      CERTEX_CUDA(cudaStreamCreateWithFlags(&sh->res.stream, cudaStreamNonBlocking));
      // shard s owns the ids [n s / S, n (s + 1) / S) (certex_shards.cu:70-75)
      const int64_t lo = n * static_cast<int64_t>(s) / n_shards, hi = n * static_cast<int64_t>(s + 1) / n_shards;
      sh->first_id     = lo;
      sh->index        = std::make_unique<Index>(sh->res, p, dtype, dim);
      sh->index->extend(sh->res, x + static_cast<size_t>(lo) * row_bytes, hi - lo, true);
      sharded->shards[s] = std::move(sh);
    });
    *out = sharded.release();
  });
}

cuvsError_t certexB200ShardedDestroy(certexB200ShardedIndex_t index)
{
  return translate([=] {
    delete index;  // every shard frees its index and its stream on its own device
  });
}

cuvsError_t certexB200ShardedGetSize(certexB200ShardedIndex_t index, int64_t* size)
{
  return translate([=] {
    CERTEX_EXPECTS(index != nullptr && size != nullptr, "certex: null sharded index");
    int64_t n = 0;
    for (auto& sh : index->shards) { n += sh->index->size(); }
    *size = n;
  });
}

cuvsError_t certexB200ShardedSearch(cuvsCertexSearchParams_t params, certexB200ShardedIndex_t index,
                                    DLManagedTensor* queries, DLManagedTensor* neighbors, DLManagedTensor* distances)
{
  return translate([=] {
    CERTEX_EXPECTS(index != nullptr && !index->shards.empty(), "certex: null sharded index");
    CERTEX_EXPECTS(params != nullptr, "certex: null search parameters");
    const void* q = checked(queries, 2, -1, 0, false, "the queries");
    auto* nb      = static_cast<int64_t*>(checked(neighbors, 2, kDLInt, 64, false, "the neighbors"));
    auto* ds      = static_cast<float*>(checked(distances, 2, kDLFloat, 32, false, "the distances"));
    CERTEX_EXPECTS(on_host(queries->dl_tensor) && on_host(neighbors->dl_tensor) && on_host(distances->dl_tensor),
                   "certex: a sharded search takes and returns host matrices");
    CERTEX_EXPECTS(dtype_of(queries->dl_tensor.dtype) == index->dtype && queries->dl_tensor.shape[1] == index->dim,
                   "certex: the queries must have the vector type and the dimension of the index");
    const int64_t nq = queries->dl_tensor.shape[0], k = neighbors->dl_tensor.shape[1];
    CERTEX_EXPECTS(neighbors->dl_tensor.shape[0] == nq && distances->dl_tensor.shape[0] == nq &&
                     distances->dl_tensor.shape[1] == k,
                   "certex: neighbors and distances must be [n_queries, k]");
    CERTEX_EXPECTS(k >= 1 && k <= 2048, "certex: k must be between 1 and 2048");
    for (auto& sh : index->shards) {
      CERTEX_EXPECTS(sh->index->size() >= k, "certex: every shard must hold at least k vectors");  // certex_shards.cu:97-99
    }
    if (nq == 0) { return; }
    SearchParams sp;
    sp.anchors     = params->anchors;
    sp.batch_size  = params->batch_size;
    sp.probe_lists = params->probe_lists;
    const size_t S       = index->shards.size();
    const size_t q_bytes = static_cast<size_t>(nq) * static_cast<size_t>(index->dim) *
                           (index->dtype == kF32 ? 4 : index->dtype == kF16 ? 2 : 1);
    const size_t cells = static_cast<size_t>(nq) * static_cast<size_t>(k);
    std::vector<double> part_scores(S * cells);
    std::vector<int64_t> part_ids(S * cells);
    // every shard: its exact k best with global ids and fp64 scores
    for_each_shard(S, [&](size_t s) {
      Shard& sh = *index->shards[s];
      CERTEX_CUDA(cudaSetDevice(sh.device));
      cudaStream_t st = sh.res.stream;
      PoolBuffer dq(q_bytes, st), ids(cells * 8, st), dist(cells * 4, st), scores(cells * 8, st);
      CERTEX_CUDA(cudaMemcpyAsync(dq.p, q, q_bytes, cudaMemcpyHostToDevice, st));
      sh.index->search(sh.res, sp, dq.p, nq, static_cast<int>(k), static_cast<int64_t*>(ids.p), static_cast<float*>(dist.p),
                       static_cast<double*>(scores.p), Filter{}, sh.first_id);
      CERTEX_CUDA(cudaMemcpyAsync(part_scores.data() + s * cells, scores.p, cells * 8, cudaMemcpyDeviceToHost, st));
      CERTEX_CUDA(cudaMemcpyAsync(part_ids.data() + s * cells, ids.p, cells * 8, cudaMemcpyDeviceToHost, st));
      sh.res.sync();
    });
    // merge by (score, id) on the first shard's device (the reference merges on the host, certex_shards.cu:144-166)
    DeviceGuard guard;
    Shard& first = *index->shards[0];
    CERTEX_CUDA(cudaSetDevice(first.device));
    cudaStream_t st = first.res.stream;
    PoolBuffer dq(q_bytes, st), ps(S * cells * 8, st), pi(S * cells * 8, st), ids(cells * 8, st), dist(cells * 4, st);
    CERTEX_CUDA(cudaMemcpyAsync(dq.p, q, q_bytes, cudaMemcpyHostToDevice, st));
    CERTEX_CUDA(cudaMemcpyAsync(ps.p, part_scores.data(), S * cells * 8, cudaMemcpyHostToDevice, st));
    CERTEX_CUDA(cudaMemcpyAsync(pi.p, part_ids.data(), S * cells * 8, cudaMemcpyHostToDevice, st));
    merge_shards(first.res, static_cast<const double*>(ps.p), static_cast<const int64_t*>(pi.p), static_cast<int>(S),
                 static_cast<int>(nq), static_cast<int>(k), dq.p, index->dtype, index->dim, index->metric,
                 static_cast<int64_t*>(ids.p), static_cast<float*>(dist.p), nullptr);
    CERTEX_CUDA(cudaMemcpyAsync(nb, ids.p, cells * 8, cudaMemcpyDeviceToHost, st));
    CERTEX_CUDA(cudaMemcpyAsync(ds, dist.p, cells * 4, cudaMemcpyDeviceToHost, st));
    first.res.sync();
  });
}

// ------------------------------------------------------------------------------------------- row shards over NCCL ranks
cuvsError_t certexB200CommGetUniqueId(void* id128)
{
  return translate([=] {
    CERTEX_EXPECTS(id128 != nullptr, "certex: null id buffer");
    comm_unique_id(id128);
  });
}

cuvsError_t certexB200CommInitRank(const void* id128, int32_t n_ranks, int32_t rank, certexB200Comm_t* comm)
{
  return translate([=] {
    CERTEX_EXPECTS(comm != nullptr, "certex: null communicator handle");
    *comm = reinterpret_cast<certexB200Comm_t>(comm_create(id128, n_ranks, rank, nullptr));
  });
}

cuvsError_t certexB200CommAdopt(void* nccl_comm, certexB200Comm_t* comm)
{
  return translate([=] {
    CERTEX_EXPECTS(comm != nullptr && nccl_comm != nullptr, "certex: null communicator");
    *comm = reinterpret_cast<certexB200Comm_t>(comm_create(nullptr, 0, 0, nccl_comm));
  });
}

cuvsError_t certexB200CommDestroy(certexB200Comm_t comm)
{
  return translate([=] { comm_destroy(reinterpret_cast<Comm*>(comm)); });
}

cuvsError_t certexB200DistributedSearchBegin(cuvsResources_t res, certexB200Comm_t comm, cuvsCertexSearchParams_t params,
                                             cuvsCertexIndex_t index, DLManagedTensor* queries, DLManagedTensor* neighbors,
                                             DLManagedTensor* distances, DLManagedTensor* scores, int64_t id_base,
                                             int32_t share_thresholds, certexB200PendingSearch_t* pending)
{
  return translate([=] {
    Resources& r = as_res(res);
    Holder& h    = as_holder(index);
    CERTEX_EXPECTS(pending != nullptr, "certex: null pending search");
    *pending = nullptr;
    CERTEX_EXPECTS(comm != nullptr, "certex: null communicator");
    CERTEX_EXPECTS(params != nullptr, "certex: null search parameters");
    CERTEX_EXPECTS(queries != nullptr && queries->dl_tensor.dtype.code == index->dtype.code &&
                     queries->dl_tensor.dtype.bits == index->dtype.bits,
                   "certex: the queries must have the vector type of the index");
    const void* q    = checked(queries, 2, -1, 0, true, "the queries");
    const int64_t nq = queries->dl_tensor.shape[0];
    CERTEX_EXPECTS(queries->dl_tensor.shape[1] == h.index->dim(), "certex: the queries must have the dimension of the index");
    auto* nb        = static_cast<int64_t*>(checked(neighbors, 2, kDLInt, 64, true, "the neighbors"));
    auto* ds        = static_cast<float*>(checked(distances, 2, kDLFloat, 32, true, "the distances"));
    const int64_t k = neighbors->dl_tensor.shape[1];
    CERTEX_EXPECTS(neighbors->dl_tensor.shape[0] == nq && distances->dl_tensor.shape[0] == nq && distances->dl_tensor.shape[1] == k,
                   "certex: neighbors and distances must be [n_queries, k]");
    double* sc = nullptr;
    if (scores) {
      sc = static_cast<double*>(checked(scores, 2, kDLFloat, 64, true, "the scores"));
      CERTEX_EXPECTS(scores->dl_tensor.shape[0] == nq && scores->dl_tensor.shape[1] == k, "certex: scores must be [n_queries, k]");
    }
    CERTEX_EXPECTS(k >= 1 && k <= 2048, "certex: k must be between 1 and 2048");
    CERTEX_EXPECTS(h.index->size() >= k, "certex: every shard must hold at least k vectors");  // certex_shards.cu:97-99
    SearchParams sp;
    sp.anchors     = params->anchors;
    sp.batch_size  = params->batch_size;
    sp.probe_lists = params->probe_lists;
    *pending = reinterpret_cast<certexB200PendingSearch_t>(distributed_search_begin(
      r, *reinterpret_cast<Comm*>(comm), *h.index, sp, q, nq, static_cast<int>(k), nb, ds, sc, id_base, share_thresholds != 0));
  });
}

cuvsError_t certexB200DistributedSearchEnd(certexB200PendingSearch_t pending)
{
  return translate([=] {
    CERTEX_EXPECTS(pending != nullptr, "certex: null pending search");
    distributed_search_end(reinterpret_cast<DistributedPending*>(pending));
  });
}

cuvsError_t certexB200DistributedSearch(cuvsResources_t res, certexB200Comm_t comm, cuvsCertexSearchParams_t params,
                                        cuvsCertexIndex_t index, DLManagedTensor* queries, DLManagedTensor* neighbors,
                                        DLManagedTensor* distances, DLManagedTensor* scores, int64_t id_base,
                                        int32_t share_thresholds)
{
  certexB200PendingSearch_t pending = nullptr;
  if (certexB200DistributedSearchBegin(res, comm, params, index, queries, neighbors, distances, scores, id_base, share_thresholds,
                                       &pending) != CUVS_SUCCESS) {
    return CUVS_ERROR;
  }
  return certexB200DistributedSearchEnd(pending);
}

const char* certexB200Version(void) { return "0.2.0"; }

}  // extern "C"
