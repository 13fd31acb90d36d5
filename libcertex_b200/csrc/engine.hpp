// Host side of the engine: the index container and the search pipeline, mirroring the reference's
// cuvs::neighbors::certex `index<T>`, `build`, `extend`, `remove`, `set_labels` and `search`
// (cpp/include/cuvs/neighbors/certex.hpp:43-741, cpp/src/neighbors/certex/certex.cu:641-843, 1460-1508).
// Plain C++ with raw device pointers; the C ABI (c_api.cpp) is a thin layer over it.
#pragma once

#include <cuda_runtime.h>

#include <cstdint>
#include <functional>
#include <iosfwd>
#include <memory>
#include <mutex>
#include <array>
#include <map>
#include <condition_variable>
#include <mutex>
#include <shared_mutex>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

#include "kernels.cuh"

namespace certex_b200 {

struct Error : std::runtime_error {
  using std::runtime_error::runtime_error;
};

/// Device memory for a call's temporaries could not be had. A search answers it by splitting its queries in halves,
/// like the reference (cpp/src/neighbors/certex/certex.cu:1477-1502).
struct OutOfMemory : Error {
  using Error::Error;
};

#define CERTEX_EXPECTS(cond, msg)                                \
  do {                                                           \
    if (!(cond)) { throw ::certex_b200::Error(std::string(msg)); } \
  } while (0)

#define CERTEX_CUDA(call)                                                                              \
  do {                                                                                                 \
    cudaError_t e_ = (call);                                                                           \
    if (e_ != cudaSuccess) {                                                                           \
      throw ::certex_b200::Error(std::string("certex: CUDA error ") + cudaGetErrorString(e_) + " at " + \
                                 __FILE__ + ":" + std::to_string(__LINE__));                           \
    }                                                                                                  \
  } while (0)

/// Stream and device a call runs on (the role of cuvsResources_t / raft::resources).
struct Resources {
  int device          = 0;
  cudaStream_t stream = nullptr;
  int sm_count        = 0;
  Resources();
  ~Resources();
  Resources(const Resources&)            = delete;
  Resources& operator=(const Resources&) = delete;
  void sync() const;
  /// Searches that may be in flight at once per Resources (search_begin .. search_end).
  static constexpr int kMaxInFlight = 2;
  /// Block `slot` of kPinnedSlots small blocks of page-locked host memory (256 bytes each) that the counters of the
  /// searches in flight are copied to; made on first use.
  static constexpr int kPinnedSlots = 4;
  void* pinned_block(int slot) const;
  /// Sends small host arrays to the device in one copy: `pieces` (pointer, bytes) are packed, 256-byte aligned, into
  /// page-locked memory and copied to `device` (at least upload_bytes(pieces) bytes) on the stream; offsets[i] is where
  /// piece i starts. A copy from pageable memory would make the host wait for the stream once per array.
  static size_t upload_bytes(const std::vector<std::pair<const void*, size_t>>& pieces);
  void upload(const std::vector<std::pair<const void*, size_t>>& pieces, void* device, std::vector<size_t>& offsets) const;

 private:
  mutable void* pinned_ = nullptr;
  mutable void* staging_        = nullptr;  // page-locked, grows; reused once the copy out of it has finished
  mutable size_t staging_bytes_ = 0;
  mutable cudaEvent_t staging_done_ = nullptr;
  friend class Index;
  mutable int searches_in_flight_ = 0;
  mutable unsigned next_slot_     = 0;
};

/// Readers-writer gate of an index. Unlike std::shared_mutex the shared side may be taken again by a thread that holds
/// it already (two searches in flight from one thread): a waiting writer does not hold back new readers.
class ReaderGate {
 public:
  void lock_shared()
  {
    std::unique_lock<std::mutex> l(m_);
    cv_.wait(l, [&] { return !writer_; });
    ++readers_;
  }
  void unlock_shared()
  {
    std::lock_guard<std::mutex> l(m_);
    if (--readers_ == 0) { cv_.notify_all(); }
  }
  void lock()
  {
    std::unique_lock<std::mutex> l(m_);
    cv_.wait(l, [&] { return !writer_ && readers_ == 0; });
    writer_ = true;
  }
  bool try_lock()
  {
    std::lock_guard<std::mutex> l(m_);
    if (writer_ || readers_ != 0) { return false; }
    writer_ = true;
    return true;
  }
  void unlock()
  {
    {
      std::lock_guard<std::mutex> l(m_);
      writer_ = false;
    }
    cv_.notify_all();
  }

 private:
  std::mutex m_;
  std::condition_variable cv_;
  int readers_ = 0;
  bool writer_ = false;
};

/// cuvs::neighbors::certex::index_params (cpp/include/cuvs/neighbors/certex.hpp:43-87). Every setting returns the same
/// exact neighbours. width, variance, pca_sample, n_lists, local_projections and int8_rows steer the reference's
/// projected screening rows; this engine screens 8-bit vectors by their exact integer Gram product and has no
/// projection, so it accepts and ignores them. host_vectors (certex.hpp:56-61) keeps the vectors in page-locked host
/// memory instead of device memory: the screen's code rows stay on the device, the exact stage reads the few candidate
/// rows it needs from the host in place (8-bit indexes: from the code rows, which are the vectors, so a screened search
/// does not touch host memory at all).
struct IndexParams {
  int metric             = kL2;
  int width              = 0;
  double variance        = 0.95;
  int anchor_stride      = 16;
  int64_t pca_sample     = 1000000;
  bool host_vectors      = false;
  int n_lists            = 0;
  bool local_projections = false;
  bool int8_rows         = false;
};

/// cuvs::neighbors::certex::search_params (certex.hpp:97-107).
struct SearchParams {
  int anchors     = 128;
  int batch_size  = 2048;
  int probe_lists = 2;
};

/// Counters of the reference's search_stats (cpp/src/neighbors/certex/detail/kernels.hpp:256-263).
struct SearchStats {
  unsigned long long queries = 0, survivors = 0, verified = 0, dense_queries = 0;
  unsigned long long launches = 0;     // kernels of this library launched by the searches
  double screen_ms = 0, anchor_ms = 0; // device time of the SCREEN and GROUPMAX tensor-core passes (CUDA events)
  double span_ms = 0;                  // device time from the first to the last operation a screened search enqueued
  unsigned long long screen_passes = 0;
  unsigned long long rescreened = 0;   // queries screened a second time with a tighter threshold
  unsigned long long routed_queries = 0;  // query slots of searches by label that went through the routed screen
};

struct LabelRun;  // the queries of one label in a search by labels (engine.cu)

struct Filter {
  const uint32_t* words = nullptr;  // device words, bit j of word i is entry 32 i + j, set = keep
  int64_t bitmap_cols   = 0;        // 0: bitset over the ids; > 0: bitmap [n_queries, bitmap_cols]
  const int32_t* query_labels = nullptr;  // device [n_queries]: search by label
  int64_t covered_ids         = 0;        // ids the words cover (bits of a bitset, columns of a bitmap): checked against
                                          // the index size under the search's reader lock
};

class Index {
 public:
  Index(const Resources& res, const IndexParams& params, int dtype, int64_t dim);
  ~Index();
  Index(const Index&)            = delete;
  Index& operator=(const Index&) = delete;

  /// Appends n rows ([n, dim] dense row-major, device or host memory); they receive the next consecutive ids.
  void extend(const Resources& res, const void* rows, int64_t n, bool on_host);
  void remove(const Resources& res, const int64_t* ids_device, int64_t n_ids);
  void set_labels(const Resources& res, const int32_t* labels_device, int64_t n, int64_t first);
  void reserve(const Resources& res, int64_t n);
  /// Groups the ids by label (the reference's partition_by_labels, cpp/src/neighbors/certex/certex.cu:1542-1606):
  /// searches by label then score only the rows of the query's label, plus the rows added since.
  void partition_by_labels(const Resources& res);

  /**
   * Exact k nearest neighbours of nq queries (device, dense row-major, the index's element type).
   * neighbors int64 [nq, k], distances float [nq, k] (device); scores_out (optional, device fp64 [nq, k]) receives the
   * exact scores the ranking used. id_base is added to every returned id (row shards of a larger set).
   */
  void search(const Resources& res, const SearchParams& sp, const void* queries, int64_t nq, int k, int64_t* neighbors,
              float* distances, double* scores_out, const Filter& filter, int64_t id_base = 0) const;

  /**
   * The same search in two steps, for callers that have more device work to enqueue behind it (the all-gather and the
   * merge of a sharded search) before the host looks at anything. search_begin enqueues the whole search on res.stream,
   * outputs included, and returns without waiting for the device; it assumes that no candidate list overflows, which
   * is what nearly every call sees. status_out (optional, device) receives a non-zero word when the assumption did not
   * hold for this call. search_end waits for the stream, and only then, if a list did overflow, enqueues the repair
   * (second pass or dense scan of the queries concerned) and writes the outputs again; it returns true in that case:
   * whatever the caller derived from the outputs in between must be derived again. Every search_begin needs its
   * search_end on the same thread (it holds the index's reader lock and the call's temporaries); two searches may be in
   * flight per Resources, ended in the order they were begun. search() is search_begin + search_end (plus the halving on allocation failure).
   */
  struct Pending;
  Pending* search_begin(const Resources& res, const SearchParams& sp, const void* queries, int64_t nq, int k,
                        int64_t* neighbors, float* distances, double* scores_out, const Filter& filter, int64_t id_base,
                        unsigned long long* status_out) const;
  /// refinish: write the outputs once more from the kept lists even when nothing was repaired (a caller whose output
  /// buffers were reused in between, as the sharded search's send buffer is by a later search in flight).
  bool search_end(Pending* pending, bool refinish = false) const;
  /// Gives a search in flight other output matrices for what search_end still writes (a repair, refinish): for a
  /// caller whose first outputs have been given away in between.
  static void search_retarget(Pending* pending, int64_t* neighbors, float* distances, double* scores_out);

  int64_t size() const { return size_; }
  int64_t dim() const { return dim_; }
  int64_t capacity() const { return capacity_; }
  int64_t n_removed() const { return n_removed_; }
  int dtype() const { return dtype_; }
  int metric() const { return params_.metric; }
  bool has_labels() const { return has_labels_; }
  int64_t n_partitioned() const { return n_part_; }
  bool int_screen() const { return screen_kind_ != 0 && !code_overflow_; }  // a tensor-core screen is available
  bool host_vectors() const { return host_vectors_; }
  const IndexParams& params() const { return params_; }
  size_t pitch() const { return pitch_; }
  const void* vectors() const { return vectors_; }

  /// Writes / reads the index (parameters, vectors, removed flags, labels) after the 4-byte dtype prefix of a file.
  void save(const Resources& res, std::ostream& os) const;
  /// load() also reads a file written by the reference (format "CERX" version 1): its vectors, removal flags and labels.
  static std::unique_ptr<Index> load(const Resources& res, std::istream& is, int dtype);

  /// Forces a path for tests: 0 = automatic, 1 = always the dense path, 2 = screen with this candidate capacity,
  /// 3 = searches by label score their label's rows densely (no routed screen), 4 = a search call of more than `cap`
  /// queries fails as if the device were out of memory (exercises the halving, on the host, without exhausting a GPU),
  /// 5 = the threshold stage of plain searches computes exact group maxima instead of the chained bound.
  void set_test_mode(int mode, int cap) { test_mode_ = mode, test_cap_ = cap; }

  static thread_local SearchStats* stats_sink;  // counters of the calling thread's searches, when set

  /// Exchange of thresholds between the row shards of one set (the reference's threshold hooks,
  /// cpp/src/neighbors/certex/detail/kernels.hpp:271-277, and the first round of its sharded search,
  /// certex_shards.cu:136-141). Between the anchor pass and the screen of every batch the hook of the calling thread
  /// gets keys [n] on the device: key i is a monotone int32 image of a score that k rows of this shard certainly reach
  /// for query i of the batch (larger = tighter). It may raise keys to what another shard of the same set certainly
  /// reaches (e.g. the maximum over the shards); it must enqueue its work on `stream`. Plain unfiltered searches only.
  using ThresholdHook = void (*)(void* ctx, int32_t* keys, int64_t n, cudaStream_t stream);
  static thread_local ThresholdHook threshold_hook;
  static thread_local void* threshold_hook_ctx;
  /// The wider exchange for small k (k <= kTopkExchangeMaxK), used instead of threshold_hook when set: the hook gets
  /// the k largest keys of every query in this shard, topk [n, k], next to thr [n] (their k-th) and leaves in thr the
  /// k-th largest key over the lists of all shards. Every key is reached by a row of its own shard, so that value is
  /// reached by k rows of the whole set: the threshold a single index over all rows would find, where the maximum of
  /// the shards' own thresholds is only as tight as the best shard's.
  using TopkHook = void (*)(void* ctx, const int32_t* topk, int32_t* thr, int64_t n, int k, cudaStream_t stream);
  static thread_local TopkHook topk_hook;
  static constexpr int kTopkExchangeMaxK = 64;
  /// Whether an unfiltered search for k neighbours goes through the tensor-core screen (and calls the hook).
  bool will_screen(int k) const;

 private:
  static std::unique_ptr<Index> load_reference_file(const Resources& res, std::istream& is, int dtype);
  static std::unique_ptr<Index> from_blocks(const Resources& res, const IndexParams& p, int dtype, int64_t dim, int64_t n,
                                            int64_t n_rem, bool labeled,
                                            const std::function<void(char*, size_t)>& next_block);
  void search_screened(const Resources& res, const uint8_t* qbuf, const float* shift, const void* queries, size_t row_bytes,
                       int q0, int nq, int k, double* best_s, int32_t* best_row, int32_t* ovf_list,
                       unsigned int* ovf_count, unsigned long long* stats, int* err, int anchor_stride, int64_t n,
                       int32_t* thr2, const Admit& adm, std::vector<cudaEvent_t>* events) const;
  void screen_pass(const Resources& res, const uint8_t* qcodes, const int32_t* thr, const void* queries, size_t row_bytes,
                   int q0, int nq, int k, double* best_s, int32_t* best_row, int32_t* ovf_list, unsigned int* ovf_count,
                   unsigned long long* stats, int* err, int64_t n, int32_t* thr2, const float* shift, const Admit& adm,
                   std::vector<cudaEvent_t>* events) const;
  int anchor_stride_for(int64_t n, int k) const;
  void search_dense(const Resources& res, const void* q, size_t qpitch, const int32_t* qsel, int q0, int nqb, int k,
                    const Admit& adm, double* best_s, int32_t* best_row, int64_t n) const;
  /// Search by label over the label partition; returns the (query, row) pairs scored and counts its launches.
  unsigned long long search_by_labels(const Resources& res, const void* q, size_t qpitch, int nq, int k, const Admit& adm,
                                      double* best_s, int32_t* best_row, int64_t n, SearchStats* st) const;
  /// The routed (screened) part of a search by labels for one class of labels; see engine.cu.
  unsigned long long search_routed(const Resources& res, const void* q, size_t qpitch, int k, std::vector<LabelRun>& routed,
                                   bool fine, double* best_s, int32_t* best_row, SearchStats* st,
                                   std::vector<LabelRun>& dense) const;

  IndexParams params_;
  int dtype_;
  int64_t dim_;
  size_t pitch_       = 0;  // bytes per stored row (zero padded: integer types to a multiple of 128, others of 16)
  size_t code_pitch_  = 0;  // bytes per code row of the screen: the vector itself (8-bit types) or its fp16 rounding
  int kb_             = 0;  // 128-byte K blocks per code row
  int screen_kind_    = 0;  // 0: no tensor-core screen (dense path only), 1: 8-bit codes, 2: fp16 codes of float data
  bool code_overflow_ = false;      // a float coordinate did not fit fp16: the index answers by the dense path
  float n1max_ = 0, n2max_ = 0, emax_ = 0;  // fp16 codes: largest |code|, |rounding residual|, |e| over all rows
  unsigned int* maxima_ = nullptr;  // device copy of the three maxima (float bits) and the overflow flag
  int device_         = 0;
  int64_t size_       = 0;
  int64_t capacity_   = 0;
  int64_t n_removed_  = 0;
  bool has_labels_    = false;
  bool host_vectors_  = false;    // vectors_ is page-locked host memory that the GPU reads in place (index_params.host_vectors)
  void* vectors_      = nullptr;  // [capacity, pitch]
  uint8_t* removed_   = nullptr;  // [capacity rounded up to 4]
  int32_t* labels_    = nullptr;  // [capacity], -1 = none
  // label partition: ids 0 .. n_part_ - 1 in (label, id) order; label part_labels_[i] owns entries
  // part_offsets_[i] .. part_offsets_[i + 1] - 1
  int32_t* part_ids_  = nullptr;
  int64_t n_part_     = 0;
  std::vector<int32_t> part_labels_;
  std::vector<int64_t> part_offsets_;
  // label-ordered copy of the screen's rows (made with the partition when the index has a screen): every label's
  // entries in id order, padded to whole tiles of 256 rows; label i starts at tile part_tile0_[i]
  void* lcodes_       = nullptr;  // [n_lrows_, code_pitch_]
  int32_t* linit_     = nullptr;  // [n_lrows_] e (never: padding, removed)
  int32_t* lcmax_     = nullptr;  // [n_lrows_ / 16]
  int32_t* lperm_     = nullptr;  // [n_lrows_] row -> id, -1 padding
  int32_t* linv_      = nullptr;  // [n_part_] id -> row
  int64_t n_lrows_    = 0;
  std::vector<int64_t> part_tile0_;
  // screen: the code rows sorted by squared norm run by run (a run: one appended batch, or several small ones of an
  // L2 index sorted together), and per sorted row
  void* codes_        = nullptr;  // [capacity, pitch] rows in sorted order
  int32_t* perm_      = nullptr;  // [capacity] sorted row -> id
  int32_t* inv_       = nullptr;  // [capacity] id -> sorted row
  int32_t* init_      = nullptr;  // [capacity rounded up to 256] e of the sorted row (kNeverInit: removed / padding)
  double* sqnorm_     = nullptr;  // [capacity] cosine metric, float rows on the device: |x|^2 by id, the verification's own fp64 sum
  int32_t* cmax_      = nullptr;  // [capacity rounded up to 256, / 16] maximum of e over each chain of 16 sorted rows
  // L2 only: the sorted runs [first row, rows) at the end of the index that a later append may still sort again with
  // its own rows; a run of kFrozenRun rows or more stays as it is
  std::vector<std::pair<int64_t, int64_t>> runs_;
  static constexpr int64_t kFrozenRun = 65536;
  int test_mode_      = 0;
  int test_cap_       = 0;
  mutable ReaderGate rw_;  // searches hold it shared per call; size/pointer publication holds it exclusive
  /// Work splits of the tensor-core passes, kept in device memory per shape (query tiles, base tiles, panel, CTAs,
  /// chunk): a search then enqueues no copy from pageable host memory, which would make the host wait for the stream in
  /// the middle of the search.
  struct DevicePlan {
    void* segs = nullptr;  // ScreenSeg[]
    int* begin = nullptr;  // [grid + 1]
  };
  DevicePlan device_plan(int nqt, int nt, int panel_tiles, int grid, int chunk_tiles) const;  // empty: not kept, upload it
  mutable std::mutex plans_mutex_;
  mutable std::map<std::array<int, 5>, DevicePlan> plans_;
  static constexpr size_t kMaxPlans = 64;
  std::mutex writer_;             // serialises extend / remove / set_labels
};

/// Merge of `parts` per-shard answers [parts, nq, k] (fp64 scores, int64 ids, id -1 = missing) by (score, id), the
/// order of the reference's sharded merge (cpp/src/neighbors/certex/certex_shards.cu:144-166).
void merge_shards(const Resources& res, const double* scores, const int64_t* ids, int parts, int nq, int k,
                  const void* queries, int dtype, int64_t dim, int metric, int64_t* neighbors, float* distances,
                  double* scores_out, int64_t part_stride = 0);

/// Row shards over several processes, one GPU each (nccl_shards.cu): a communicator with its exchange buffers, and the
/// sharded search over it. comm_create: from a 128-byte id that one rank made with comm_unique_id and the application
/// sent to the others (ncclCommInitRank on the current device), or adopting an ncclComm_t the application owns.
struct Comm;
void comm_unique_id(void* id128);
Comm* comm_create(const void* id128, int n_ranks, int rank, void* adopt);
void comm_destroy(Comm* c);
int comm_ranks(const Comm* c);
/// Every rank calls it with the same queries, k and parameters: local exact top-k of its shard (ids + id_base),
/// ncclAllGather of the lists, merge by (score, id); the same answer on every rank. Device pointers.
void distributed_search(const Resources& res, Comm& c, const Index& index, const SearchParams& sp, const void* queries,
                        int64_t nq, int k, int64_t* neighbors, float* distances, double* scores_out, int64_t id_base,
                        bool share_thresholds);
/// The same in two calls: begin enqueues the local search, the exchange and the merge and returns without waiting; end
/// waits for that search (not for what was enqueued behind it), and runs the second round if a list had overflowed on
/// some rank. Up to Resources::kMaxInFlight searches may be between their two calls per communicator, so that the
/// host's work for the next search overlaps the device's work for this one; they end in the order they began, and
/// every rank makes the same sequence of calls. Queries and outputs stay valid and untouched until end.
struct DistributedPending;
DistributedPending* distributed_search_begin(const Resources& res, Comm& c, const Index& index, const SearchParams& sp,
                                             const void* queries, int64_t nq, int k, int64_t* neighbors, float* distances,
                                             double* scores_out, int64_t id_base, bool share_thresholds);
void distributed_search_end(DistributedPending* pending);

/// Host-side work split of the tensor-core pass: grid * kMaxSegs segments of 4 ints each.
void plan_segments_flat(int nqt, int nt, int panel_tiles, int grid, int32_t* out);

/// order [n] = the numbers 0 .. n - 1 sorted by labels[i], equal labels in ascending order: how a search by labels
/// groups its queries (test hook).
void order_by_label_flat(const int32_t* labels, int64_t n, int32_t* order);

/// The split the searches use: the same, with the base tiles taken in chunks of `chunk_tiles` (0: one chunk) that every
/// query panel passes over while they are in L2. Segments of 4 ints each, CTA b owns [seg_begin[b], seg_begin[b + 1]);
/// returns their number.
int plan_chunked_flat(int nqt, int nt, int panel_tiles, int grid, int chunk_tiles, int32_t* segs_out, int cap_segs,
                      int32_t* seg_begin);

/// Host-side work split of a routed pass (searches by label): run r pairs n_query_tiles[r] query tiles with its own
/// n_base_tiles[r] base tiles (runs are laid out one after the other in both directions). Writes the segments (5 ints
/// each: first query tile, query tiles, first base tile, end base tile, first base tile of the run), their number and
/// the per-CTA ranges seg_begin [grid + 1]; returns how many runs fit.
int plan_routed_flat(int n_runs, const int32_t* n_query_tiles, const int32_t* n_base_tiles, int panel_tiles, int grid,
                     int max_segs, int32_t* segs_out, int cap_segs, int32_t* n_segs, int32_t* seg_begin);

/// The tensor-core pass alone on caller buffers (see certexB200ScreenRaw in the public header). Synchronises.
void screen_raw(const Resources& res, const void* q_codes, int64_t nq, const void* x_codes, int64_t n, int64_t code_len,
                int code_kind, const int32_t* init, int mode, const int32_t* thr, int32_t* gmax, int64_t ld,
                uint32_t* cnt, int32_t* cand, uint32_t cap, float* elapsed_ms);

}  // namespace certex_b200
