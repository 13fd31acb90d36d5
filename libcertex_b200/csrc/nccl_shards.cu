// Row shards over several processes, one GPU each: the exchange step of the sharded search over NCCL.
//
// The reference keeps all shards in one process and moves the per-shard lists through host memory
// (cpp/src/neighbors/certex/certex_shards.cu:85-167: one thread per shard, host std::sort of the lists). Here every
// rank owns one shard and one GPU; a search call is, on one stream and without a host round trip in between,
//   local exact top-k of all queries (Index::search_begin)            -> k (fp64 score, int64 global id) per query
//   ncclAllGather of the lists (+ one status word per rank)           -> [ranks, nq, k] on every GPU
//   merge by (score, id) (merge_shards)                               -> the answer, identical on every rank
// and then one wait of the host, which reads every rank's status word: if a rank's candidate lists overflowed (rare)
// it repairs its lists (Index::search_end) and all ranks run the exchange and the merge once more; if a rank failed,
// every rank reports the failure instead of waiting for it. The optional first round of the reference (shards share
// their thresholds, certex_shards.cu:136-141) is an ncclAllReduce(max) over the per-query threshold keys.
//
// NCCL is not linked: the library is found at run time (the copy that the process has already loaded, e.g. the one
// PyTorch brings, else libnccl.so.2 on the loader's path), so libcertex_b200.so loads on machines without NCCL as long
// as these entry points are not called. No kernel reads another GPU's memory; NCCL moves the lists.
#include "../../include/certex_b200.h"

#include "engine.hpp"

#include <dlfcn.h>
#include <nccl.h>

#include <cstring>
#include <map>
#include <mutex>
#include <string>
#include <vector>

namespace certex_b200 {

namespace {

struct NcclApi {
  void* handle = nullptr;
  ncclResult_t (*GetUniqueId)(ncclUniqueId*)                                                            = nullptr;
  ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int)                                     = nullptr;
  ncclResult_t (*CommDestroy)(ncclComm_t)                                                               = nullptr;
  ncclResult_t (*CommCount)(const ncclComm_t, int*)                                                     = nullptr;
  ncclResult_t (*CommUserRank)(const ncclComm_t, int*)                                                  = nullptr;
  ncclResult_t (*AllGather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t)       = nullptr;
  ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
  const char* (*GetErrorString)(ncclResult_t)                                                           = nullptr;
};

const NcclApi& nccl()
{
  static NcclApi api = [] {
    NcclApi a;
    // the copy already in the process first (RTLD_NOLOAD finds it by its soname)
    a.handle = dlopen("libnccl.so.2", RTLD_NOW | RTLD_NOLOAD);
    if (!a.handle) { a.handle = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL); }
    if (!a.handle) { a.handle = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL); }
    CERTEX_EXPECTS(a.handle != nullptr, std::string("certex: NCCL is not available (") + dlerror() + ")");
    auto need = [&](const char* name) {
      void* f = dlsym(a.handle, name);
      CERTEX_EXPECTS(f != nullptr, std::string("certex: the NCCL library lacks ") + name);
      return f;
    };
    a.GetUniqueId    = reinterpret_cast<decltype(a.GetUniqueId)>(need("ncclGetUniqueId"));
    a.CommInitRank   = reinterpret_cast<decltype(a.CommInitRank)>(need("ncclCommInitRank"));
    a.CommDestroy    = reinterpret_cast<decltype(a.CommDestroy)>(need("ncclCommDestroy"));
    a.CommCount      = reinterpret_cast<decltype(a.CommCount)>(need("ncclCommCount"));
    a.CommUserRank   = reinterpret_cast<decltype(a.CommUserRank)>(need("ncclCommUserRank"));
    a.AllGather      = reinterpret_cast<decltype(a.AllGather)>(need("ncclAllGather"));
    a.AllReduce      = reinterpret_cast<decltype(a.AllReduce)>(need("ncclAllReduce"));
    a.GetErrorString = reinterpret_cast<decltype(a.GetErrorString)>(need("ncclGetErrorString"));
    return a;
  }();
  return api;
}

#define CERTEX_NCCL(call)                                                                                        \
  do {                                                                                                           \
    ncclResult_t r_ = (call);                                                                                    \
    if (r_ != ncclSuccess) {                                                                                     \
      throw ::certex_b200::Error(std::string("certex: NCCL error ") + nccl().GetErrorString(r_) + " at " + __FILE__ + \
                                 ":" + std::to_string(__LINE__));                                                \
    }                                                                                                            \
  } while (0)

constexpr unsigned long long kStatusFailed = 8;  // the rank's local search threw: its lists are empty

}  // namespace

/// A communicator over the ranks of one sharded set, with the exchange buffers of its searches (kept between calls).
struct Comm {
  ncclComm_t comm = nullptr;
  bool owned      = false;  // made by certexB200CommInitRank (destroyed with this object) or adopted from the caller
  int n_ranks = 0, rank = 0, device = 0;
  int64_t* send = nullptr;  // [2 nq k + 1]: fp64 scores as bits, global ids, the status word
  int64_t* recv = nullptr;  // [n_ranks, 2 nq k + 1]
  size_t send_words = 0;
  unsigned long long* host_status = nullptr;  // page-locked, [kStatusSlots][n_ranks]: the status words of the searches in flight
  static constexpr int kStatusSlots = 4;
  unsigned long long begun = 0, ended = 0;    // sharded searches begun / ended on this communicator
  unsigned long long send_owner = ~0ull;      // the search whose lists the send buffer holds (in stream order)
  unsigned long long* status_of(unsigned long long seq) const { return host_status + (seq % kStatusSlots) * n_ranks; }
  int32_t* topk_recv = nullptr;               // [n_ranks, nq, k] keys of the threshold exchange, and the rows made of them
  int32_t* topk_rows = nullptr;
  size_t topk_ints   = 0;
  std::map<int, bool> all_screen;             // k -> every rank's search for k neighbours goes through the screen
  int64_t all_screen_size = -1;               // ... decided for this index size
  ~Comm()
  {
    cudaFree(send), cudaFree(recv), cudaFree(topk_recv), cudaFree(topk_rows);
    if (host_status) { cudaFreeHost(host_status); }
    if (owned && comm) { nccl().CommDestroy(comm); }
  }
  void reserve(size_t words)
  {
    if (words <= send_words) { return; }
    cudaFree(send), cudaFree(recv);
    send = recv = nullptr, send_words = 0;
    CERTEX_CUDA(cudaMalloc(&send, words * 8));
    CERTEX_CUDA(cudaMalloc(&recv, words * 8 * static_cast<size_t>(n_ranks)));
    send_words = words;
  }
};

namespace {

void share_topk_hook(void* ctx, const int32_t* topk, int32_t* thr, int64_t n, int k, cudaStream_t stream)
{
  // every rank's k largest keys per query -> the k-th largest of all of them: k rows of the whole set reach it
  auto* c           = static_cast<Comm*>(ctx);
  const size_t mine = static_cast<size_t>(n) * k, rows = static_cast<size_t>(n) * ((static_cast<size_t>(c->n_ranks) * k + 7) / 8 * 8);
  if (mine * c->n_ranks > c->topk_ints || rows > c->topk_ints) {
    cudaFree(c->topk_recv), cudaFree(c->topk_rows);
    c->topk_recv = c->topk_rows = nullptr, c->topk_ints = 0;
    const size_t want = std::max(mine * c->n_ranks, rows);
    CERTEX_CUDA(cudaMalloc(&c->topk_recv, want * 4));
    CERTEX_CUDA(cudaMalloc(&c->topk_rows, want * 4));
    c->topk_ints = want;
  }
  CERTEX_NCCL(nccl().AllGather(topk, c->topk_recv, mine, ncclInt32, c->comm, stream));
  launch_union_kth(c->topk_recv, c->n_ranks, static_cast<int>(n), k, c->topk_rows, thr, stream);
  CERTEX_CUDA(cudaGetLastError());
}

void share_thresholds_hook(void* ctx, int32_t* keys, int64_t n, cudaStream_t stream)
{
  // any k rows of one shard bound the k-th neighbour of the whole set: every rank screens with the tightest bound
  auto* c = static_cast<Comm*>(ctx);
  CERTEX_NCCL(nccl().AllReduce(keys, keys, static_cast<size_t>(n), ncclInt32, ncclMax, c->comm, stream));
}

}  // namespace

void comm_unique_id(void* id128)
{
  static_assert(sizeof(ncclUniqueId) == 128, "the id buffer of the C ABI holds an ncclUniqueId");
  ncclUniqueId id;
  CERTEX_NCCL(nccl().GetUniqueId(&id));
  std::memcpy(id128, &id, sizeof(id));
}

Comm* comm_create(const void* id128, int n_ranks, int rank, void* adopt)
{
  auto c = std::make_unique<Comm>();
  CERTEX_CUDA(cudaGetDevice(&c->device));
  if (adopt) {
    c->comm = static_cast<ncclComm_t>(adopt);
    CERTEX_NCCL(nccl().CommCount(c->comm, &c->n_ranks));
    CERTEX_NCCL(nccl().CommUserRank(c->comm, &c->rank));
  } else {
    CERTEX_EXPECTS(id128 != nullptr && n_ranks >= 1 && rank >= 0 && rank < n_ranks, "certex: a rank in [0, n_ranks) and an id");
    ncclUniqueId id;
    std::memcpy(&id, id128, sizeof(id));
    CERTEX_NCCL(nccl().CommInitRank(&c->comm, n_ranks, id, rank));
    c->owned = true, c->n_ranks = n_ranks, c->rank = rank;
  }
  CERTEX_CUDA(cudaHostAlloc(reinterpret_cast<void**>(&c->host_status), sizeof(unsigned long long) * c->n_ranks * Comm::kStatusSlots, cudaHostAllocDefault));
  return c.release();
}

void comm_destroy(Comm* c) { delete c; }

int comm_ranks(const Comm* c) { return c->n_ranks; }

/// A sharded search between its two calls: the local search in flight and what the second call needs.
struct DistributedPending {
  const Resources* res = nullptr;
  Comm* c              = nullptr;
  const Index* index   = nullptr;
  Index::Pending* pending = nullptr;
  std::exception_ptr failed;
  const void* queries = nullptr;
  int64_t nq = 0, id_base = 0;
  int k = 0;
  int64_t* neighbors = nullptr;
  float* distances   = nullptr;
  double* scores_out = nullptr;
  size_t cells = 0, words = 0;
  unsigned long long seq = 0;   // number of the search on its communicator: they end in the order they began
  cudaEvent_t done = nullptr;   // behind the first exchange
  ~DistributedPending()
  {
    if (done) { cudaEventDestroy(done); }
  }
};

namespace {

// empty lists and the failure flag in this rank's contribution
void fail_lists(const Resources& res, Comm& c, size_t cells)
{
  cudaGetLastError();
  CERTEX_CUDA(cudaMemsetAsync(c.send, 0xff, 2 * cells * 8, res.stream));  // ids -1 (scores: never read)
  CERTEX_CUDA(cudaMemcpyAsync(c.send + 2 * cells, &kStatusFailed, 8, cudaMemcpyHostToDevice, res.stream));
}

// all-gather of the ranks' lists and status words, merge into the caller's outputs, status words to the host
void exchange(DistributedPending& d)
{
  Comm& c = *d.c;
  const Resources& res = *d.res;
  CERTEX_NCCL(nccl().AllGather(c.send, c.recv, d.words, ncclInt64, c.comm, res.stream));
  merge_shards(res, reinterpret_cast<const double*>(c.recv), c.recv + d.cells, c.n_ranks, static_cast<int>(d.nq), d.k, d.queries,
               d.index->dtype(), d.index->dim(), d.index->metric(), d.neighbors, d.distances, d.scores_out,
               static_cast<int64_t>(d.words));
  CERTEX_CUDA(cudaMemcpy2DAsync(c.status_of(d.seq), 8, c.recv + 2 * d.cells, d.words * 8, 8, static_cast<size_t>(c.n_ranks),
                                cudaMemcpyDeviceToHost, res.stream));
}

}  // namespace

DistributedPending* distributed_search_begin(const Resources& res, Comm& c, const Index& index, const SearchParams& sp,
                                             const void* queries, int64_t nq, int k, int64_t* neighbors, float* distances,
                                             double* scores_out, int64_t id_base, bool share_thresholds)
{
  CERTEX_EXPECTS(res.device == c.device, "certex: the communicator was made on another device than these resources");
  CERTEX_EXPECTS(c.begun - c.ended < static_cast<unsigned long long>(Resources::kMaxInFlight),
                 "certex: too many sharded searches in flight on this communicator (end the oldest first)");
  auto d = std::make_unique<DistributedPending>();
  d->res = &res, d->c = &c, d->index = &index, d->queries = queries, d->nq = nq, d->k = k, d->id_base = id_base;
  d->neighbors = neighbors, d->distances = distances, d->scores_out = scores_out;
  d->seq = c.begun;
  if (nq == 0) {
    ++c.begun;
    return d.release();
  }
  const size_t cells = static_cast<size_t>(nq) * k, words = 2 * cells + 1;
  d->cells = cells, d->words = words;
  c.reserve(words);
  auto* send_scores = reinterpret_cast<double*>(c.send);
  int64_t* send_ids = c.send + cells;
  auto* send_status = reinterpret_cast<unsigned long long*>(c.send + 2 * cells);

  if (share_thresholds) {
    // (also on a communicator of one rank, where the exchange returns the rank's own threshold: one code path)
    // the exchange needs every rank to reach it, i.e. to screen: agreed once per k and index size
    if (c.all_screen_size != index.size()) { c.all_screen.clear(), c.all_screen_size = index.size(); }
    if (!c.all_screen.count(k)) {
      int32_t mine = index.will_screen(k) ? 1 : 0, *dev = reinterpret_cast<int32_t*>(c.send);
      res.sync();  // a search in flight may still use the send buffer
      CERTEX_CUDA(cudaMemcpyAsync(dev, &mine, 4, cudaMemcpyHostToDevice, res.stream));
      CERTEX_NCCL(nccl().AllReduce(dev, dev, 1, ncclInt32, ncclMin, c.comm, res.stream));
      CERTEX_CUDA(cudaMemcpyAsync(&mine, dev, 4, cudaMemcpyDeviceToHost, res.stream));
      res.sync();
      c.all_screen[k] = mine != 0;
    }
    share_thresholds = c.all_screen[k];
  } else {
    share_thresholds = false;
  }
  ++c.begun;  // from here on the search takes part in the collectives: it must be ended
  c.send_owner = d->seq;

  // ---- the local exact top-k, written straight into the send buffer (distances: scratch use of the caller's output)
  try {
    if (share_thresholds) {
      Index::threshold_hook = share_thresholds_hook, Index::topk_hook = share_topk_hook, Index::threshold_hook_ctx = &c;
    }
    d->pending = index.search_begin(res, sp, queries, nq, k, send_ids, distances, send_scores, Filter{}, id_base, send_status);
    Index::threshold_hook = nullptr, Index::topk_hook = nullptr, Index::threshold_hook_ctx = nullptr;
  } catch (...) {
    // this rank cannot answer: it still takes part in the exchange, with empty lists and the failure in its status
    // word, so that no rank is left waiting in the collective (a rank that failed inside the threshold exchange cannot
    // be helped this way; NCCL's own timeout ends the others' wait)
    Index::threshold_hook = nullptr, Index::topk_hook = nullptr, Index::threshold_hook_ctx = nullptr;
    d->failed = std::current_exception();
    fail_lists(res, c, cells);
  }
  // the first exchange assumes that no candidate list overflowed; the ranks' status words say whether that held everywhere
  try {
    exchange(*d);
    CERTEX_CUDA(cudaEventCreateWithFlags(&d->done, cudaEventDisableTiming));
    CERTEX_CUDA(cudaEventRecord(d->done, res.stream));
  } catch (...) {
    if (d->pending) {
      try {
        index.search_end(d->pending);
      } catch (...) {
      }
    }
    ++c.ended;
    throw;
  }
  return d.release();
}

void distributed_search_end(DistributedPending* raw)
{
  CERTEX_EXPECTS(raw != nullptr, "certex: no sharded search to end");
  CERTEX_EXPECTS(raw->seq == raw->c->ended, "certex: sharded searches end in the order they began");  // raw stays valid
  std::unique_ptr<DistributedPending> d(raw);
  Comm& c              = *d->c;
  const Resources& res = *d->res;
  ++c.ended;
  if (d->nq == 0) { return; }
  // Whether the send buffer has been reused meanwhile (by a later search that was begun, or by the second round of an
  // earlier one): a second round must then write this search's lists there again, also on a rank that has nothing to
  // repair.
  const bool overtaken = c.send_owner != d->seq;
  bool again = false;
  int failed_rank = -1;
  auto read_status = [&](bool first) {
    const unsigned long long* st = c.status_of(d->seq);
    for (int r = 0; r < c.n_ranks; ++r) {
      if (first && (st[r] & 7ull) != 0) { again = true; }
      if ((st[r] & kStatusFailed) != 0 && failed_rank < 0) { failed_rank = r; }
    }
  };
  try {
    CERTEX_CUDA(cudaEventSynchronize(d->done));  // the one wait of a round: everything before it ran back to back on the device
    read_status(true);
  } catch (...) {
    if (d->pending) {
      try {
        d->index->search_end(d->pending);
      } catch (...) {
      }
    }
    throw;
  }
  std::exception_ptr failed = d->failed;
  if (d->pending) {
    if (overtaken) {
      // the send buffer may even be another allocation by now (a later, larger search): what this search still writes
      // goes to where the second exchange will read it
      Index::search_retarget(d->pending, c.send + d->cells, d->distances, reinterpret_cast<double*>(c.send));
    }
    try {
      // repairs this rank's lists when its own status word was set
      d->index->search_end(d->pending, /*refinish=*/again && failed_rank < 0 && overtaken);
    } catch (...) {
      // only a rank whose status word was set can fail here, so every rank is about to run the second round: this
      // rank takes part in it with the failure in its status word
      failed = std::current_exception();
      fail_lists(res, c, d->cells);
    }
  }
  if (failed_rank < 0 && again) {
    c.send_owner = d->seq;
    if (overtaken && !failed) {
      // the status word in the send buffer is the later search's by now: this rank's lists are in order
      CERTEX_CUDA(cudaMemsetAsync(c.send + 2 * d->cells, 0, 8, res.stream));
    }
    exchange(*d);
    res.sync();
    read_status(false);
  }
  if (failed) { std::rethrow_exception(failed); }
  CERTEX_EXPECTS(failed_rank < 0, "certex: the local search of rank " + std::to_string(failed_rank) + " failed; no answer for this call");
}

void distributed_search(const Resources& res, Comm& c, const Index& index, const SearchParams& sp, const void* queries,
                        int64_t nq, int k, int64_t* neighbors, float* distances, double* scores_out, int64_t id_base,
                        bool share_thresholds)
{
  distributed_search_end(distributed_search_begin(res, c, index, sp, queries, nq, k, neighbors, distances, scores_out, id_base,
                                                  share_thresholds));
}

}  // namespace certex_b200
