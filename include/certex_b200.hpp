// C++ face of libcertex_b200: the names, argument order and meaning of the reference's
// cuvs::neighbors::certex API (cpp/include/cuvs/neighbors/certex.hpp: index_params 43-87, search_params 97-107,
// index<T> 131-423, build 481-511, extend 534-557, set_labels 579-591, partition_by_labels 609-612, remove 632-641,
// search 668-735, serialize / deserialize 764-767; cpp/include/cuvs/neighbors/certex_shards.hpp: sharded_index<T>,
// build_sharded, search), header-only over the C ABI of certex_b200.h.
//
// The reference passes raft::resources and raft mdspan views; this header has no RAFT dependency and declares the two
// small view types it needs (a pointer and extents, the same accessors: data_handle(), extent(i)). A caller that
// already holds raft views converts with  {v.data_handle(), v.extent(0), v.extent(1)}.  Errors are thrown as
// certex_b200::error with the text cuvsGetLastErrorText() would return (the reference throws raft::exception).
#pragma once

#include <cstdint>
#include <stdexcept>
#include <string>
#include <type_traits>
#include <utility>
#include <vector>

#include "certex_b200.h"

namespace certex_b200 {

struct error : std::runtime_error {
  using std::runtime_error::runtime_error;
};

namespace detail {
inline void check(cuvsError_t status)
{
  if (status != CUVS_SUCCESS) { throw error(cuvsGetLastErrorText()); }
}

template <typename T>
constexpr DLDataType dl_type()
{
  using U = std::remove_cv_t<T>;
  static_assert(sizeof(U) == 1 || sizeof(U) == 2 || sizeof(U) == 4 || sizeof(U) == 8, "unsupported element type");
  if constexpr (std::is_same_v<U, float>) {
    return DLDataType{kDLFloat, 32, 1};
  } else if constexpr (std::is_same_v<U, int8_t>) {
    return DLDataType{kDLInt, 8, 1};
  } else if constexpr (std::is_same_v<U, uint8_t>) {
    return DLDataType{kDLUInt, 8, 1};
  } else if constexpr (std::is_same_v<U, int32_t>) {
    return DLDataType{kDLInt, 32, 1};
  } else if constexpr (std::is_same_v<U, uint32_t>) {
    return DLDataType{kDLUInt, 32, 1};
  } else if constexpr (std::is_same_v<U, int64_t>) {
    return DLDataType{kDLInt, 64, 1};
  } else {
    static_assert(sizeof(U) == 2, "use float, a 16-bit float type, int8_t, uint8_t, int32_t, uint32_t or int64_t");
    return DLDataType{kDLFloat, 16, 1};  // __half, or any other 2-byte IEEE half type
  }
}

/// A borrowed DLPack tensor over device (or host) memory; lives for one call.
struct tensor {
  DLManagedTensor t{};
  int64_t shape[2] = {0, 0};
  tensor(const void* data, DLDataType type, int ndim, int64_t n0, int64_t n1, bool on_host)
  {
    shape[0] = n0, shape[1] = n1;
    t.dl_tensor.data               = const_cast<void*>(data);
    t.dl_tensor.device.device_type = on_host ? kDLCPU : kDLCUDA;
    t.dl_tensor.device.device_id   = 0;
    t.dl_tensor.ndim               = ndim;
    t.dl_tensor.dtype              = type;
    t.dl_tensor.shape              = shape;
    t.dl_tensor.strides            = nullptr;
    t.dl_tensor.byte_offset        = 0;
  }
  DLManagedTensor* ptr() { return &t; }
};
}  // namespace detail

/// Stream and device of the calls (the role of raft::resources). The stream is a cudaStream_t passed as void*.
class resources {
 public:
  resources() { detail::check(cuvsResourcesCreate(&handle_)); }
  explicit resources(void* stream) : resources() { set_stream(stream); }
  ~resources() { cuvsResourcesDestroy(handle_); }
  resources(const resources&)            = delete;
  resources& operator=(const resources&) = delete;
  void set_stream(void* stream) const { detail::check(cuvsStreamSet(handle_, stream)); }
  void sync() const { detail::check(cuvsStreamSync(handle_)); }
  cuvsResources_t handle() const { return handle_; }

 private:
  cuvsResources_t handle_ = 0;
};

template <typename T>
struct device_matrix_view {
  T* data      = nullptr;
  int64_t rows = 0, cols = 0;
  T* data_handle() const { return data; }
  int64_t extent(int i) const { return i == 0 ? rows : cols; }
};
template <typename T>
struct device_vector_view {
  T* data   = nullptr;
  int64_t n = 0;
  T* data_handle() const { return data; }
  int64_t extent(int) const { return n; }
};
/// A matrix in host memory (build / extend stream it to the device).
template <typename T>
struct host_matrix_view : device_matrix_view<T> {};

/// certex.hpp:43-87. Every setting returns the same exact neighbours.
struct index_params {
  cuvsDistanceType metric = L2Expanded;
  int width               = 0;
  double variance         = 0.95;
  int anchor_stride       = 16;
  int64_t pca_sample      = 1000000;
  bool host_vectors       = false;
  int n_lists             = 0;
  bool local_projections  = false;
  bool int8_rows          = false;
};

/// certex.hpp:97-107.
struct search_params {
  int anchors     = 128;
  int batch_size  = 2048;
  int probe_lists = 2;
};

/// Filters of a search: none, one bit per id (set = keep), or one row of such bits per query
/// (cuvs::neighbors::filtering::none_sample_filter / bitset_filter / bitmap_filter in the reference's overload).
struct sample_filter {
  cuvsFilterType type   = NO_FILTER;
  const uint32_t* words = nullptr;  // device words, bit j of word i is entry 32 i + j
  int64_t rows = 0, cols = 0;       // bitmap: queries x ids; bitset: 1 x ids
  static sample_filter none() { return {}; }
  static sample_filter bitset(const uint32_t* words, int64_t n_ids) { return {BITSET, words, 1, n_ids}; }
  static sample_filter bitmap(const uint32_t* words, int64_t n_queries, int64_t n_ids) { return {BITMAP, words, n_queries, n_ids}; }
};

/// certex.hpp:131-423: owner of one index; movable, not copyable.
template <typename T>
class index {
 public:
  index() { detail::check(cuvsCertexIndexCreate(&handle_)); }  // empty: to be filled by build() or deserialize()
  ~index()
  {
    if (handle_) { cuvsCertexIndexDestroy(handle_); }
  }
  index(index&& o) noexcept : handle_(std::exchange(o.handle_, nullptr)) {}
  index& operator=(index&& o) noexcept
  {
    if (this != &o) {
      if (handle_) { cuvsCertexIndexDestroy(handle_); }
      handle_ = std::exchange(o.handle_, nullptr);
    }
    return *this;
  }
  index(const index&)            = delete;
  index& operator=(const index&) = delete;

  int64_t size() const { return info().size; }
  int64_t dim() const { return info().dim; }
  int64_t n_removed() const { return info().n_removed; }
  int64_t capacity() const { return info().capacity; }
  int64_t n_partitioned() const { return info().n_partitioned; }
  bool has_labels() const { return info().has_labels != 0; }
  cuvsDistanceType metric() const { return static_cast<cuvsDistanceType>(info().metric); }
  int anchor_stride() const { return info().anchor_stride; }
  void reserve(resources const& res, int64_t n) { detail::check(certexB200IndexReserve(res.handle(), handle_, n)); }
  cuvsCertexIndex_t handle() const { return handle_; }

 private:
  certexB200IndexInfo info() const
  {
    certexB200IndexInfo i{};
    detail::check(certexB200IndexGetInfo(handle_, &i));
    return i;
  }
  cuvsCertexIndex_t handle_ = nullptr;
};

namespace detail {
template <typename T>
index<T> build_impl(resources const& res, index_params const& p, const T* data, int64_t rows, int64_t cols, bool on_host)
{
  cuvsCertexIndexParams_t ip = nullptr;
  check(cuvsCertexIndexParamsCreate(&ip));
  ip->metric            = p.metric;
  ip->width             = p.width;
  ip->variance          = p.variance;
  ip->anchor_stride     = p.anchor_stride;
  ip->pca_sample        = p.pca_sample;
  ip->host_vectors      = p.host_vectors;
  ip->n_lists           = p.n_lists;
  ip->local_projections = p.local_projections;
  ip->int8_rows         = p.int8_rows;
  index<T> idx;
  tensor x(data, dl_type<T>(), 2, rows, cols, on_host);
  const cuvsError_t status = cuvsCertexBuild(res.handle(), ip, x.ptr(), idx.handle());
  cuvsCertexIndexParamsDestroy(ip);
  check(status);
  return idx;
}
}  // namespace detail

/// certex.hpp:481-511: an index over the rows of `dataset` (ids 0 .. n_rows - 1).
template <typename T>
index<std::remove_cv_t<T>> build(resources const& res, index_params const& params, device_matrix_view<T> dataset)
{
  return detail::build_impl<std::remove_cv_t<T>>(res, params, dataset.data, dataset.rows, dataset.cols, false);
}
template <typename T>
index<std::remove_cv_t<T>> build(resources const& res, index_params const& params, host_matrix_view<T> dataset)
{
  return detail::build_impl<std::remove_cv_t<T>>(res, params, dataset.data, dataset.rows, dataset.cols, true);
}

/// certex.hpp:534-557: append vectors; they receive the next consecutive ids.
template <typename T, typename U>
void extend(resources const& res, device_matrix_view<U> new_vectors, index<T>* idx)
{
  static_assert(std::is_same_v<std::remove_cv_t<U>, T>, "the vectors must have the element type of the index");
  detail::tensor x(new_vectors.data, detail::dl_type<T>(), 2, new_vectors.rows, new_vectors.cols, false);
  detail::check(cuvsCertexExtend(res.handle(), x.ptr(), idx->handle()));
}
template <typename T, typename U>
void extend(resources const& res, host_matrix_view<U> new_vectors, index<T>* idx)
{
  static_assert(std::is_same_v<std::remove_cv_t<U>, T>, "the vectors must have the element type of the index");
  detail::tensor x(new_vectors.data, detail::dl_type<T>(), 2, new_vectors.rows, new_vectors.cols, true);
  detail::check(cuvsCertexExtend(res.handle(), x.ptr(), idx->handle()));
}

/// certex.hpp:632-641: remove by id; ids are never reused.
template <typename T>
void remove(resources const& res, device_vector_view<const int64_t> ids, index<T>* idx)
{
  detail::tensor t(ids.data, detail::dl_type<int64_t>(), 1, ids.n, 0, false);
  detail::check(cuvsCertexRemove(res.handle(), t.ptr(), idx->handle()));
}

/// certex.hpp:579-591: labels of the vectors first, first + 1, ...
template <typename T>
void set_labels(resources const& res, device_vector_view<const int32_t> labels, index<T>* idx, int64_t first = 0)
{
  detail::tensor t(labels.data, detail::dl_type<int32_t>(), 1, labels.n, 0, false);
  detail::check(cuvsCertexSetLabels(res.handle(), t.ptr(), first, idx->handle()));
}

/// certex.hpp:609-612.
template <typename T>
void partition_by_labels(resources const& res, index<T>* idx)
{
  detail::check(cuvsCertexPartitionByLabels(res.handle(), idx->handle()));
}

/// certex.hpp:668-699: exact k nearest neighbours, k = neighbors.extent(1); results are on the stream of `res`.
template <typename T, typename U>
void search(resources const& res, search_params const& params, index<T> const& idx, device_matrix_view<U> queries,
            device_matrix_view<int64_t> neighbors, device_matrix_view<float> distances,
            sample_filter const& filter = sample_filter::none())
{
  static_assert(std::is_same_v<std::remove_cv_t<U>, T>, "the queries must have the element type of the index");
  cuvsCertexSearchParams sp{params.anchors, params.batch_size, params.probe_lists};
  detail::tensor q(queries.data, detail::dl_type<T>(), 2, queries.rows, queries.cols, false);
  detail::tensor nb(neighbors.data, detail::dl_type<int64_t>(), 2, neighbors.rows, neighbors.cols, false);
  detail::tensor ds(distances.data, detail::dl_type<float>(), 2, distances.rows, distances.cols, false);
  const bool map = filter.type == BITMAP;
  const int64_t n_words = map ? (filter.rows * filter.cols + 31) / 32 : (filter.cols + 31) / 32;
  detail::tensor words(filter.words, detail::dl_type<uint32_t>(), 1, n_words, 0, false);
  cuvsFilter f;
  f.type = filter.type;
  f.addr = filter.type == NO_FILTER ? 0 : reinterpret_cast<uintptr_t>(words.ptr());
  detail::check(cuvsCertexSearch(res.handle(), &sp, idx.handle(), q.ptr(), nb.ptr(), ds.ptr(), f));
}

/// certex.hpp:714-735: every query searches the vectors of its own label.
template <typename T, typename U>
void search(resources const& res, search_params const& params, index<T> const& idx, device_matrix_view<U> queries,
            device_vector_view<const int32_t> query_labels, device_matrix_view<int64_t> neighbors,
            device_matrix_view<float> distances)
{
  static_assert(std::is_same_v<std::remove_cv_t<U>, T>, "the queries must have the element type of the index");
  cuvsCertexSearchParams sp{params.anchors, params.batch_size, params.probe_lists};
  detail::tensor q(queries.data, detail::dl_type<T>(), 2, queries.rows, queries.cols, false);
  detail::tensor ql(query_labels.data, detail::dl_type<int32_t>(), 1, query_labels.n, 0, false);
  detail::tensor nb(neighbors.data, detail::dl_type<int64_t>(), 2, neighbors.rows, neighbors.cols, false);
  detail::tensor ds(distances.data, detail::dl_type<float>(), 2, distances.rows, distances.cols, false);
  detail::check(cuvsCertexSearchWithLabels(res.handle(), &sp, idx.handle(), q.ptr(), ql.ptr(), nb.ptr(), ds.ptr()));
}

/// certex.hpp:764-767 (file names; the layout of the file is this library's own).
template <typename T>
void serialize(resources const& res, const std::string& filename, index<T> const& idx)
{
  detail::check(cuvsCertexSerialize(res.handle(), filename.c_str(), idx.handle()));
}
template <typename T>
void deserialize(resources const& res, const std::string& filename, index<T>* idx)
{
  *idx = index<T>();
  detail::check(cuvsCertexDeserialize(res.handle(), filename.c_str(), idx->handle()));
}

/// certex_shards.hpp:39-60: contiguous row shards, one index per device; movable, not copyable.
template <typename T>
class sharded_index {
 public:
  sharded_index() = default;
  explicit sharded_index(certexB200ShardedIndex_t h) : handle_(h) {}
  ~sharded_index()
  {
    if (handle_) { certexB200ShardedDestroy(handle_); }
  }
  sharded_index(sharded_index&& o) noexcept : handle_(std::exchange(o.handle_, nullptr)) {}
  sharded_index& operator=(sharded_index&& o) noexcept
  {
    if (this != &o) {
      if (handle_) { certexB200ShardedDestroy(handle_); }
      handle_ = std::exchange(o.handle_, nullptr);
    }
    return *this;
  }
  sharded_index(const sharded_index&)            = delete;
  sharded_index& operator=(const sharded_index&) = delete;
  int64_t size() const
  {
    int64_t n = 0;
    detail::check(certexB200ShardedGetSize(handle_, &n));
    return n;
  }
  certexB200ShardedIndex_t handle() const { return handle_; }

 private:
  certexB200ShardedIndex_t handle_ = nullptr;
};

/// certex_shards.hpp:70-90: one shard per entry of `devices` (a device may appear more than once), built in parallel.
template <typename T>
sharded_index<std::remove_cv_t<T>> build_sharded(std::vector<int> const& devices, index_params const& params,
                                                 host_matrix_view<T> dataset)
{
  cuvsCertexIndexParams ip{};
  ip.metric        = params.metric;
  ip.anchor_stride = params.anchor_stride;
  std::vector<int32_t> dev(devices.begin(), devices.end());
  detail::tensor x(dataset.data, detail::dl_type<T>(), 2, dataset.rows, dataset.cols, true);
  certexB200ShardedIndex_t h = nullptr;
  detail::check(certexB200ShardedBuild(dev.data(), static_cast<int32_t>(dev.size()), &ip, x.ptr(), &h));
  return sharded_index<std::remove_cv_t<T>>(h);
}

/// certex_shards.hpp:104-120: queries, neighbors and distances are host matrices; complete on return.
template <typename T, typename U>
void search(search_params const& params, sharded_index<T> const& idx, host_matrix_view<U> queries,
            host_matrix_view<int64_t> neighbors, host_matrix_view<float> distances)
{
  static_assert(std::is_same_v<std::remove_cv_t<U>, T>, "the queries must have the element type of the index");
  cuvsCertexSearchParams sp{params.anchors, params.batch_size, params.probe_lists};
  detail::tensor q(queries.data, detail::dl_type<T>(), 2, queries.rows, queries.cols, true);
  detail::tensor nb(neighbors.data, detail::dl_type<int64_t>(), 2, neighbors.rows, neighbors.cols, true);
  detail::tensor ds(distances.data, detail::dl_type<float>(), 2, distances.rows, distances.cols, true);
  detail::check(certexB200ShardedSearch(&sp, idx.handle(), q.ptr(), nb.ptr(), ds.ptr()));
}

/// One process per GPU, one row shard per process: the ranks of a communicator answer a search together (local exact
/// top-k, ncclAllGather of the lists, merge by (score, id); certexB200DistributedSearch). The reference's sharded search
/// (certex_shards.hpp:39-60, 104-120) keeps its shards in one process; this is the same search for processes that each
/// own a device. Movable, not copyable.
class communicator {
 public:
  /// 128 bytes that one rank makes and the application sends to the others (an ncclUniqueId).
  static std::vector<uint8_t> unique_id()
  {
    std::vector<uint8_t> id(128);
    detail::check(certexB200CommGetUniqueId(id.data()));
    return id;
  }
  /// Every rank, with its device current.
  communicator(std::vector<uint8_t> const& id, int n_ranks, int rank)
  {
    if (id.size() != 128) { throw error("certex: a communicator id has 128 bytes"); }
    detail::check(certexB200CommInitRank(id.data(), n_ranks, rank, &handle_));
  }
  /// Wraps an ncclComm_t that the application made and keeps.
  explicit communicator(void* nccl_comm) { detail::check(certexB200CommAdopt(nccl_comm, &handle_)); }
  ~communicator()
  {
    if (handle_) { certexB200CommDestroy(handle_); }
  }
  communicator(communicator&& o) noexcept : handle_(std::exchange(o.handle_, nullptr)) {}
  communicator(const communicator&)            = delete;
  communicator& operator=(const communicator&) = delete;
  certexB200Comm_t handle() const { return handle_; }

 private:
  certexB200Comm_t handle_ = nullptr;
};

/// Every rank calls it with the same queries and k; `idx` holds the rank's rows, whose global ids start at first_id.
/// The same merged answer arrives on every rank (device matrices, complete on return). share_thresholds: the ranks
/// agree on thresholds between the anchor pass and the screen (the reference's first round, certex_shards.cu:136-141).
template <typename T, typename U>
void search(resources const& res, communicator const& comm, search_params const& params, index<T> const& idx,
            int64_t first_id, device_matrix_view<U> queries, device_matrix_view<int64_t> neighbors,
            device_matrix_view<float> distances, bool share_thresholds = true)
{
  static_assert(std::is_same_v<std::remove_cv_t<U>, T>, "the queries must have the element type of the index");
  cuvsCertexSearchParams sp{params.anchors, params.batch_size, params.probe_lists};
  detail::tensor q(queries.data, detail::dl_type<T>(), 2, queries.rows, queries.cols, false);
  detail::tensor nb(neighbors.data, detail::dl_type<int64_t>(), 2, neighbors.rows, neighbors.cols, false);
  detail::tensor ds(distances.data, detail::dl_type<float>(), 2, distances.rows, distances.cols, false);
  detail::check(certexB200DistributedSearch(res.handle(), comm.handle(), &sp, idx.handle(), q.ptr(), nb.ptr(), ds.ptr(), nullptr,
                                            first_id, share_thresholds ? 1 : 0));
}

/// A sharded search between search_begin and search_end. Movable, not copyable; it must be ended (search_end) before
/// it is destroyed, in the order the searches were begun.
class pending_search {
 public:
  pending_search() = default;
  explicit pending_search(certexB200PendingSearch_t h) : handle_(h) {}
  pending_search(pending_search&& o) noexcept : handle_(std::exchange(o.handle_, nullptr)) {}
  pending_search& operator=(pending_search&& o) noexcept
  {
    handle_ = std::exchange(o.handle_, nullptr);
    return *this;
  }
  pending_search(const pending_search&)            = delete;
  pending_search& operator=(const pending_search&) = delete;
  certexB200PendingSearch_t release() { return std::exchange(handle_, nullptr); }

 private:
  certexB200PendingSearch_t handle_ = nullptr;
};

/// The sharded search in two calls (certexB200DistributedSearchBegin / End): search_begin enqueues the local search, the
/// exchange and the merge and returns without waiting; search_end waits for that search and leaves the outputs final.
/// Up to two searches may be between the calls per communicator, so that the host prepares one while the device works
/// on the other. Queries and outputs must stay valid and untouched from search_begin to search_end.
template <typename T, typename U>
pending_search search_begin(resources const& res, communicator const& comm, search_params const& params, index<T> const& idx,
                            int64_t first_id, device_matrix_view<U> queries, device_matrix_view<int64_t> neighbors,
                            device_matrix_view<float> distances, bool share_thresholds = true)
{
  static_assert(std::is_same_v<std::remove_cv_t<U>, T>, "the queries must have the element type of the index");
  cuvsCertexSearchParams sp{params.anchors, params.batch_size, params.probe_lists};
  detail::tensor q(queries.data, detail::dl_type<T>(), 2, queries.rows, queries.cols, false);
  detail::tensor nb(neighbors.data, detail::dl_type<int64_t>(), 2, neighbors.rows, neighbors.cols, false);
  detail::tensor ds(distances.data, detail::dl_type<float>(), 2, distances.rows, distances.cols, false);
  certexB200PendingSearch_t h = nullptr;
  detail::check(certexB200DistributedSearchBegin(res.handle(), comm.handle(), &sp, idx.handle(), q.ptr(), nb.ptr(), ds.ptr(),
                                                 nullptr, first_id, share_thresholds ? 1 : 0, &h));
  return pending_search(h);
}

inline void search_end(pending_search& pending)
{
  certexB200PendingSearch_t h = pending.release();
  if (h == nullptr) { throw error("certex: this search was ended already"); }
  detail::check(certexB200DistributedSearchEnd(h));
}

}  // namespace certex_b200
