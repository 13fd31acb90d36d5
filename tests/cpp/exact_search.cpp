// A C++ caller of include/certex_b200.hpp in the shape of the reference's examples/cpp/exact_search.cu: build from a
// host matrix, extend from device memory, remove, search with and without a bitset filter and by label, search three
// row shards, compare with an fp64 loop over all vectors (ties to the smaller id). Prints "ok" and returns 0 when everything agrees.
#include <cuda_runtime_api.h>

#include <algorithm>
#include <cmath>
#include <cstdio>
#include <random>
#include <utility>
#include <vector>

#include "certex_b200.hpp"

namespace cx = certex_b200;

namespace {
constexpr int kN = 30000, kNq = 50, kDim = 40, kK = 8;

template <typename T>
T* to_device(const std::vector<T>& v)
{
  T* p = nullptr;
  if (cudaMalloc(reinterpret_cast<void**>(&p), v.size() * sizeof(T)) != cudaSuccess) { throw cx::error("cudaMalloc failed"); }
  cudaMemcpy(p, v.data(), v.size() * sizeof(T), cudaMemcpyHostToDevice);
  return p;
}

std::vector<std::pair<double, int64_t>> brute(const std::vector<float>& x, const float* q, const std::vector<char>& keep)
{
  std::vector<std::pair<double, int64_t>> all;
  for (int64_t i = 0; i < kN; ++i) {
    if (!keep[i]) { continue; }
    double s = 0;
    for (int t = 0; t < kDim; ++t) {
      const double d = double(q[t]) - double(x[i * kDim + t]);
      s += d * d;
    }
    all.emplace_back(s, i);
  }
  std::sort(all.begin(), all.end());
  all.resize(std::min<size_t>(all.size(), kK));
  return all;
}

bool same(const char* what, const std::vector<float>& x, const std::vector<float>& q, const std::vector<char>* keep_rows,
          const std::vector<int32_t>* lab, const std::vector<int32_t>* qlab, const int64_t* d_ids, const float* d_dist)
{
  std::vector<int64_t> ids(kNq * kK);
  std::vector<float> dist(kNq * kK);
  cudaMemcpy(ids.data(), d_ids, ids.size() * 8, cudaMemcpyDeviceToHost);
  cudaMemcpy(dist.data(), d_dist, dist.size() * 4, cudaMemcpyDeviceToHost);
  for (int i = 0; i < kNq; ++i) {
    std::vector<char> keep(kN, 1);
    for (int r = 0; r < kN; ++r) {
      if (keep_rows && !(*keep_rows)[r]) { keep[r] = 0; }
      if (lab && (*lab)[r] != (*qlab)[i]) { keep[r] = 0; }
    }
    const auto want = brute(x, q.data() + i * kDim, keep);
    for (int j = 0; j < kK; ++j) {
      if (ids[i * kK + j] != want[j].second || dist[i * kK + j] != float(want[j].first)) {
        std::fprintf(stderr, "%s: query %d entry %d: got (%lld, %g), want (%lld, %g)\n", what, i, j,
                     (long long)ids[i * kK + j], dist[i * kK + j], (long long)want[j].second, want[j].first);
        return false;
      }
    }
  }
  return true;
}
}  // namespace

// The entry points for one process per GPU need NCCL ranks to run (tests/test_sharded.py runs them from Python); here
// they are instantiated so that the header's wrappers are compiled and linked: one search, and two searches in flight.
void sharded_over_nccl(cx::resources const& res, cx::communicator const& comm, cx::search_params const& sp,
                       cx::index<float> const& shard, int64_t first_id, cx::device_matrix_view<const float> queries,
                       cx::device_matrix_view<int64_t> n0, cx::device_matrix_view<float> d0,
                       cx::device_matrix_view<int64_t> n1, cx::device_matrix_view<float> d1)
{
  cx::search(res, comm, sp, shard, first_id, queries, n0, d0);
  cx::pending_search a = cx::search_begin(res, comm, sp, shard, first_id, queries, n0, d0);
  cx::pending_search b = cx::search_begin(res, comm, sp, shard, first_id, queries, n1, d1);
  cx::search_end(a);
  cx::search_end(b);
}

int main(int argc, char** argv)
{
  std::mt19937 gen(7);
  std::normal_distribution<float> normal(0.f, 1.f);
  std::vector<float> x(size_t(kN) * kDim), q(size_t(kNq) * kDim);
  for (auto& v : x) { v = normal(gen); }
  for (auto& v : q) { v = normal(gen); }
  std::copy(x.begin() + 3 * kDim, x.begin() + 4 * kDim, x.begin() + 9000 * kDim);  // a duplicate row
  std::copy(x.begin() + 3 * kDim, x.begin() + 4 * kDim, q.begin());
  std::vector<int32_t> lab(kN), qlab(kNq);
  for (auto& l : lab) { l = int32_t(gen() % 3); }
  for (auto& l : qlab) { l = int32_t(gen() % 3); }

  try {
    cx::resources res;
    cx::index_params ip;
    cx::search_params sp;
    // build from the first 20 000 rows in host memory, extend with the rest from device memory
    cx::host_matrix_view<const float> first;
    first.data = x.data(), first.rows = 20000, first.cols = kDim;
    auto index   = cx::build(res, ip, first);
    float* d_x   = to_device(x);
    cx::extend(res, cx::device_matrix_view<const float>{d_x + size_t(20000) * kDim, kN - 20000, kDim}, &index);
    if (index.size() != kN || index.dim() != kDim || index.metric() != L2Expanded) { return 2; }

    float* d_q     = to_device(q);
    int64_t* d_ids = to_device(std::vector<int64_t>(kNq * kK));
    float* d_dist  = to_device(std::vector<float>(kNq * kK));
    const cx::device_matrix_view<const float> queries{d_q, kNq, kDim};
    const cx::device_matrix_view<int64_t> neighbors{d_ids, kNq, kK};
    const cx::device_matrix_view<float> distances{d_dist, kNq, kK};
    cx::search(res, sp, index, queries, neighbors, distances);
    res.sync();
    if (!same("search", x, q, nullptr, nullptr, nullptr, d_ids, d_dist)) { return 3; }

    // remove every 7th id, then a bitset that keeps the even ids
    std::vector<int64_t> gone;
    std::vector<char> keep(kN, 1);
    for (int64_t i = 0; i < kN; i += 7) {
      gone.push_back(i);
      keep[i] = 0;
    }
    int64_t* d_gone = to_device(gone);
    cx::remove(res, cx::device_vector_view<const int64_t>{d_gone, int64_t(gone.size())}, &index);
    if (index.n_removed() != int64_t(gone.size())) { return 4; }
    std::vector<uint32_t> words((kN + 31) / 32, 0);
    for (int i = 0; i < kN; i += 2) { words[i / 32] |= 1u << (i % 32); }
    for (int i = 1; i < kN; i += 2) { keep[i] = 0; }
    uint32_t* d_words = to_device(words);
    cx::search(res, sp, index, queries, neighbors, distances, cx::sample_filter::bitset(d_words, kN));
    res.sync();
    if (!same("filtered search", x, q, &keep, nullptr, nullptr, d_ids, d_dist)) { return 5; }

    // labels: every query among the (not removed) vectors of its label, through the partition
    for (int i = 1; i < kN; i += 2) { keep[i] = (i % 7) != 0; }
    int32_t* d_lab  = to_device(lab);
    int32_t* d_qlab = to_device(qlab);
    cx::set_labels(res, cx::device_vector_view<const int32_t>{d_lab, kN}, &index);
    cx::partition_by_labels(res, &index);
    if (!index.has_labels() || index.n_partitioned() != kN) { return 6; }
    cx::search(res, sp, index, queries, cx::device_vector_view<const int32_t>{d_qlab, kNq}, neighbors, distances);
    res.sync();
    if (!same("search by labels", x, q, &keep, &lab, &qlab, d_ids, d_dist)) { return 7; }

    if (argc > 1) {
      cx::serialize(res, argv[1], index);
      cx::index<float> loaded;
      cx::deserialize(res, argv[1], &loaded);
      cx::search(res, sp, loaded, queries, cx::device_vector_view<const int32_t>{d_qlab, kNq}, neighbors, distances);
      res.sync();
      if (loaded.size() != kN || !same("search by labels after reload", x, q, &keep, &lab, &qlab, d_ids, d_dist)) { return 8; }
    }

    // row shards: three shards on this device, host matrices in and out, merged by (score, id)
    {
      cx::host_matrix_view<const float> all;
      all.data = x.data(), all.rows = kN, all.cols = kDim;
      auto sharded = cx::build_sharded(std::vector<int>{0, 0, 0}, ip, all);
      if (sharded.size() != kN) { return 10; }
      std::vector<int64_t> h_ids(kNq * kK);
      std::vector<float> h_dist(kNq * kK);
      cx::host_matrix_view<const float> hq;
      hq.data = q.data(), hq.rows = kNq, hq.cols = kDim;
      cx::host_matrix_view<int64_t> hn;
      hn.data = h_ids.data(), hn.rows = kNq, hn.cols = kK;
      cx::host_matrix_view<float> hd;
      hd.data = h_dist.data(), hd.rows = kNq, hd.cols = kK;
      cx::search(sp, sharded, hq, hn, hd);
      const std::vector<char> everything(kN, 1);
      for (int i = 0; i < kNq; ++i) {
        const auto want = brute(x, q.data() + i * kDim, everything);
        for (int j = 0; j < kK; ++j) {
          if (h_ids[i * kK + j] != want[j].second || h_dist[i * kK + j] != float(want[j].first)) {
            std::fprintf(stderr, "sharded search: query %d entry %d differs\n", i, j);
            return 11;
          }
        }
      }
    }

    // errors are exceptions with the library's message
    bool threw = false;
    try {
      cx::search(res, sp, index, cx::device_matrix_view<const float>{d_q, kNq, kDim + 1}, neighbors, distances);
    } catch (const cx::error& e) {
      threw = std::string(e.what()).size() > 0;
    }
    if (!threw) { return 9; }
  } catch (const cx::error& e) {
    std::fprintf(stderr, "certex_b200::error: %s\n", e.what());
    return 1;
  }
  std::printf("ok\n");
  return 0;
}
