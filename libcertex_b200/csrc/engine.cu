// Index container and search pipeline (host orchestration). See engine.hpp for the reference counterparts.
//
// Search of an 8-bit index (no filter), per batch of queries, all on one stream without a host round trip:
//   1 GROUPMAX pass of the tensor-core kernel over every `stride`-th stored row (the anchors, read in place through a
//     strided TMA map)                                   -> gmax [nq, groups of 128 anchors]
//   2 k-th largest group maximum                          -> thr [nq]   (k distinct rows are at least that close)
//   3 SCREEN pass over all rows, keep iff acc >= thr      -> per-query candidate lists
//   4 exact fp64 scores of the candidates + top-k by (score, id)
// Queries whose candidate list overflowed, searches with a filter or labels, float / half indexes and small indexes
// take the dense path: exact fp64 scores of all rows, then a radix selection. One stream synchronisation per search
// call reads the overflow count.
#include "engine.hpp"

#include "screen_i8.cuh"

#include <cuda.h>

#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <istream>
#include <ostream>
#include <vector>

namespace certex_b200 {

thread_local SearchStats* Index::stats_sink = nullptr;
thread_local Index::ThresholdHook Index::threshold_hook = nullptr;
thread_local void* Index::threshold_hook_ctx = nullptr;
thread_local Index::TopkHook Index::topk_hook = nullptr;

namespace {

constexpr int64_t kTile = kBaseTile;  // stored rows per base tile of the tensor-core pass
constexpr int64_t kQTile = kQueryTile;
constexpr int64_t kMaxCodeBytes = 4096;  // longest code row the tensor-core pass takes (32 K blocks)

inline int64_t round_up(int64_t v, int64_t m) { return (v + m - 1) / m * m; }

// ------------------------------------------------------------------ stream-ordered scratch memory
struct Scratch {
  cudaStream_t stream;
  std::vector<void*> ptrs;
  explicit Scratch(cudaStream_t s) : stream(s) {}
  ~Scratch()
  {
    for (void* p : ptrs) { cudaFreeAsync(p, stream); }
  }
  template <typename T>
  T* get(size_t count)
  {
    void* p             = nullptr;
    const size_t bytes  = std::max<size_t>(count, 1) * sizeof(T);
    const cudaError_t e = cudaMallocAsync(&p, bytes, stream);
    if (e == cudaErrorMemoryAllocation) {
      cudaGetLastError();  // the failed allocation leaves nothing behind: the error is reported, not kept
      throw OutOfMemory("certex: out of device memory (" + std::to_string(bytes) + " bytes of scratch)");
    }
    CERTEX_CUDA(e);
    ptrs.push_back(p);
    return static_cast<T*>(p);
  }
};

// ------------------------------------------------------------------ TMA descriptors
using EncodeTiled = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                 const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                 CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiled encode_tiled()
{
  static EncodeTiled fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q{};
    const cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q);
    if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || p == nullptr) {
      throw Error("certex: the CUDA driver does not provide cuTensorMapEncodeTiled");
    }
    return reinterpret_cast<EncodeTiled>(p);
  }();
  return fn;
}

/// Map over rows of `row_bytes` 8-bit codes, `row_stride` bytes apart; boxes of 128 bytes x box_rows, 128-byte swizzle,
/// rows beyond `rows` read as zeros.
CUtensorMap make_code_map(const void* base, uint64_t row_bytes, uint64_t rows, uint64_t row_stride, uint32_t box_rows)
{
  CUtensorMap m;
  const cuuint64_t dims[2]    = {row_bytes, rows};
  const cuuint64_t strides[1] = {row_stride};
  const cuuint32_t box[2]     = {128, box_rows};
  const cuuint32_t estr[2]    = {1, 1};
  const CUresult r = encode_tiled()(&m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
                                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  CERTEX_EXPECTS(r == CUDA_SUCCESS, "certex: cuTensorMapEncodeTiled failed (" + std::to_string(int(r)) + ")");
  return m;
}

// ------------------------------------------------------------------ work split of the tensor-core pass
struct ScreenShape {
  int panel_tiles;
  int n_stages;
};

ScreenShape shape_for(int kb)
{
  // shared memory: panel_tiles * kb * 16 KB + n_stages * (kb * 32 KB + 1 KB) + 9 KB must stay below 227 KB; rows of
  // more than two K blocks stream their K blocks instead (two query tiles per segment, stages fixed by the kernel)
  return kb == 1 ? ScreenShape{7, 3} : ScreenShape{2, 2};
}

/// 3-D map (bytes of a row, column of a tile, tile) with free byte strides between columns and between tiles; box
/// 128 bytes x 256 columns x 1 tile. The anchors of the threshold stage use it: anchor a = sorted row a * stride, and
/// column c of tile t is anchor c * n_tiles + t (column stride n_tiles * stride rows, tile stride `stride` rows).
CUtensorMap make_tile_map(const void* base, uint64_t row_bytes, uint64_t column_stride, uint64_t tile_stride, uint64_t n_tiles)
{
  CUtensorMap m;
  const cuuint64_t dims[3]    = {row_bytes, static_cast<cuuint64_t>(kBaseTile), n_tiles};
  const cuuint64_t strides[2] = {column_stride, tile_stride};
  const cuuint32_t box[3]     = {128, static_cast<cuuint32_t>(kBaseTile), 1};
  const cuuint32_t estr[3]    = {1, 1, 1};
  const CUresult r = encode_tiled()(&m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(base), dims, strides, box, estr,
                                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  CERTEX_EXPECTS(r == CUDA_SUCCESS, "certex: cuTensorMapEncodeTiled failed (" + std::to_string(int(r)) + ")");
  return m;
}

/// 4-D map of the chained anchor pass: (bytes of a row, anchor of a chain [16], chain of a tile [16], tile). Anchor a
/// is sorted row a * stride; chain i of tile t holds the anchors (i * n_tiles + t) * 16 .. + 15, so a chain is 16
/// neighbours in the norm order (their e is almost one value) and the chains of a tile, and of every group of 64
/// columns, are spread over the whole set. Box 128 bytes x 16 x 16 x 1 = the 256 rows of a tile in shared memory.
CUtensorMap make_chain_map(const void* base, uint64_t row_bytes, uint64_t anchor_stride_bytes, uint64_t n_tiles)
{
  CUtensorMap m;
  const cuuint64_t dims[4]    = {row_bytes, static_cast<cuuint64_t>(kChainRows), static_cast<cuuint64_t>(kBaseTile / kChainRows), n_tiles};
  const cuuint64_t strides[3] = {anchor_stride_bytes, n_tiles * kChainRows * anchor_stride_bytes, kChainRows * anchor_stride_bytes};
  const cuuint32_t box[4]     = {128, static_cast<cuuint32_t>(kChainRows), static_cast<cuuint32_t>(kBaseTile / kChainRows), 1};
  const cuuint32_t estr[4]    = {1, 1, 1, 1};
  const CUresult r = encode_tiled()(&m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, const_cast<void*>(base), dims, strides, box, estr,
                                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  CERTEX_EXPECTS(r == CUDA_SUCCESS, "certex: cuTensorMapEncodeTiled failed (" + std::to_string(int(r)) + ")");
  return m;
}

/// Splits nqt query tiles x nt base tiles over `grid` CTAs: query tiles are grouped into panels of at most
/// `panel_tiles`; the (panel, base tile) items are laid out panel-major and cut into `grid` ranges of equal unit count.
std::vector<ScreenSeg> plan_segments(int nqt, int nt, int panel_tiles, int grid)
{
  std::vector<ScreenSeg> segs(static_cast<size_t>(grid) * kMaxSegs, ScreenSeg{0, 0, 0, 0});
  if (nqt <= 0 || nt <= 0) { return segs; }
  const int n_panels = (nqt + panel_tiles - 1) / panel_tiles;
  std::vector<int64_t> q_lo(n_panels + 1), off(n_panels + 1);
  for (int p = 0; p <= n_panels; ++p) { q_lo[p] = static_cast<int64_t>(p) * nqt / n_panels; }
  off[0] = 0;
  for (int p = 0; p < n_panels; ++p) { off[p + 1] = off[p] + (q_lo[p + 1] - q_lo[p]) * nt; }
  const int64_t total = off[n_panels];
  // position of a unit boundary as (panel, tile)
  auto locate = [&](int64_t u, int& p, int64_t& t) {
    p = 0;
    while (p < n_panels - 1 && u >= off[p + 1]) { ++p; }
    const int64_t w = q_lo[p + 1] - q_lo[p];
    t               = std::min<int64_t>((u - off[p]) / w, nt);
  };
  for (int b = 0; b < grid; ++b) {
    const int64_t u0 = total * b / grid, u1 = total * (b + 1) / grid;
    int p0, p1;
    int64_t t0, t1;
    locate(u0, p0, t0);
    if (b + 1 == grid) {
      p1 = n_panels - 1, t1 = nt;
    } else {
      locate(u1, p1, t1);
    }
    int n = 0;
    for (int p = p0; p <= p1; ++p) {
      const int64_t a = p == p0 ? t0 : 0, e = p == p1 ? t1 : nt;
      if (e > a) {
        CERTEX_EXPECTS(n < kMaxSegs, "certex: internal error: too many query panels for one launch");
        segs[static_cast<size_t>(b) * kMaxSegs + n++] =
          ScreenSeg{static_cast<int>(q_lo[p]), static_cast<int>(q_lo[p + 1] - q_lo[p]), static_cast<int>(a), static_cast<int>(e)};
      }
    }
  }
  return segs;
}

/// The same split, but with the base tiles taken in chunks that stay in L2 while every query panel passes over them:
/// all CTAs work on one chunk at a time (each on its share of the chunk's panel x tile items), then on the next. A
/// stored row then comes from HBM once per pass instead of once per query panel; the price is a reload of the query
/// panel per chunk and CTA. One list of segments with per-CTA ranges (ScreenArgs::seg_begin).
struct ChunkedPlan {
  std::vector<ScreenSeg> segs;
  std::vector<int> begin;  // [grid + 1]
};

ChunkedPlan plan_chunked(int nqt, int nt, int panel_tiles, int grid, int chunk_tiles)
{
  const int n_panels = nqt > 0 ? (nqt + panel_tiles - 1) / panel_tiles : 0;
  if (n_panels <= 1 || chunk_tiles <= 0) { chunk_tiles = std::max(nt, 1); }  // one panel reads every tile once anyway
  std::vector<std::vector<ScreenSeg>> per(static_cast<size_t>(grid));
  for (int c0 = 0; c0 < nt; c0 += chunk_tiles) {
    const int c1 = std::min(nt, c0 + chunk_tiles);
    const std::vector<ScreenSeg> part = plan_segments(nqt, c1 - c0, panel_tiles, grid);
    for (int b = 0; b < grid; ++b) {
      for (int i = 0; i < kMaxSegs; ++i) {
        const ScreenSeg& sg = part[static_cast<size_t>(b) * kMaxSegs + i];
        if (sg.t1 > sg.t0) { per[static_cast<size_t>(b)].push_back(ScreenSeg{sg.q_tile0, sg.n_qtiles, sg.t0 + c0, sg.t1 + c0}); }
      }
    }
  }
  ChunkedPlan plan;
  plan.begin.assign(1, 0);
  for (int b = 0; b < grid; ++b) {
    plan.segs.insert(plan.segs.end(), per[static_cast<size_t>(b)].begin(), per[static_cast<size_t>(b)].end());
    plan.begin.push_back(static_cast<int>(plan.segs.size()));
  }
  if (plan.segs.empty()) { plan.segs.push_back(ScreenSeg{0, 0, 0, 0}); }  // something to allocate and copy
  return plan;
}

/// Base tiles per chunk of plan_chunked: the chunk's code rows take about a quarter of the L2 (126 MB on B200).
/// A plan in the call's scratch memory, copied on the call's stream (from pageable memory: the host waits for the stream).
void upload_plan(Scratch& scratch, const ChunkedPlan& plan, ScreenSeg*& segs, int*& begin)
{
  segs  = scratch.get<ScreenSeg>(plan.segs.size());
  begin = scratch.get<int>(plan.begin.size());
  CERTEX_CUDA(cudaMemcpyAsync(segs, plan.segs.data(), plan.segs.size() * sizeof(ScreenSeg), cudaMemcpyHostToDevice, scratch.stream));
  CERTEX_CUDA(cudaMemcpyAsync(begin, plan.begin.data(), plan.begin.size() * sizeof(int), cudaMemcpyHostToDevice, scratch.stream));
}

int chunk_tiles_for(size_t code_pitch) { return static_cast<int>(std::max<size_t>(64, (size_t(32) << 20) / (kTile * code_pitch))); }

}  // namespace

// ============================================================================================ Resources
Resources::Resources()
{
  CERTEX_CUDA(cudaGetDevice(&device));
  CERTEX_CUDA(cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, device));
  int major = 0;
  CERTEX_CUDA(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device));
  CERTEX_EXPECTS(major == 10, "certex: this library is built for sm_100a (B200) only");
  // keep freed scratch memory in the stream-ordered pool instead of returning it to the driver at every sync
  cudaMemPool_t pool;
  CERTEX_CUDA(cudaDeviceGetDefaultMemPool(&pool, device));
  uint64_t keep = UINT64_MAX;
  CERTEX_CUDA(cudaMemPoolSetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &keep));
}

Resources::~Resources()
{
  if (pinned_) { cudaFreeHost(pinned_); }
  if (staging_) { cudaFreeHost(staging_); }
  if (staging_done_) { cudaEventDestroy(staging_done_); }
}

size_t Resources::upload_bytes(const std::vector<std::pair<const void*, size_t>>& pieces)
{
  size_t total = 0;
  for (const auto& p : pieces) { total = (total + 255) / 256 * 256 + p.second; }
  return std::max<size_t>(total, 1);
}

void Resources::upload(const std::vector<std::pair<const void*, size_t>>& pieces, void* device, std::vector<size_t>& offsets) const
{
  const size_t total = upload_bytes(pieces);
  if (staging_done_) { CERTEX_CUDA(cudaEventSynchronize(staging_done_)); }  // the last copy out of the buffer (long finished, as a rule)
  if (total > staging_bytes_) {
    if (staging_) { cudaFreeHost(staging_); }
    staging_ = nullptr, staging_bytes_ = 0;
    const size_t want = std::max<size_t>(total * 2, size_t(1) << 20);
    CERTEX_CUDA(cudaHostAlloc(&staging_, want, cudaHostAllocDefault));
    staging_bytes_ = want;
  }
  if (!staging_done_) { CERTEX_CUDA(cudaEventCreateWithFlags(&staging_done_, cudaEventDisableTiming)); }
  offsets.clear();
  size_t at = 0;
  for (const auto& p : pieces) {
    at = (at + 255) / 256 * 256;
    offsets.push_back(at);
    if (p.second) { std::memcpy(static_cast<unsigned char*>(staging_) + at, p.first, p.second); }
    at += p.second;
  }
  CERTEX_CUDA(cudaMemcpyAsync(device, staging_, total, cudaMemcpyHostToDevice, stream));
  CERTEX_CUDA(cudaEventRecord(staging_done_, stream));
}

void Resources::sync() const { CERTEX_CUDA(cudaStreamSynchronize(stream)); }

void* Resources::pinned_block(int slot) const
{
  if (!pinned_) { CERTEX_CUDA(cudaHostAlloc(&pinned_, 256 * kPinnedSlots, cudaHostAllocDefault)); }
  return static_cast<unsigned char*>(pinned_) + 256 * (slot % kPinnedSlots);
}

// ============================================================================================ Index
Index::Index(const Resources& res, const IndexParams& params, int dtype, int64_t dim)
  : params_(params), dtype_(dtype), dim_(dim), device_(res.device), host_vectors_(params.host_vectors)
{
  CERTEX_EXPECTS(dim >= 1, "certex: the dimension must be positive");
  // every index can end on the dense path (filters, small sets, overflow), which keeps four queries in shared memory
  CERTEX_EXPECTS(dim <= kDenseMaxDim, "certex: at most " + std::to_string(kDenseMaxDim) + " dimensions per vector");
  CERTEX_EXPECTS(dtype >= kF32 && dtype <= kU8, "certex: vectors must be float32, float16, int8, or uint8");
  CERTEX_EXPECTS(params.metric == kL2 || params.metric == kIP || params.metric == kCos,
                 "certex: the metric must be L2Expanded, InnerProduct, or CosineExpanded");
  CERTEX_EXPECTS(params.anchor_stride >= 1, "certex: anchor_stride must be at least 1");
  const bool is_int = dtype == kI8 || dtype == kU8;
  CERTEX_EXPECTS(!(params.metric == kCos && is_int), "certex: the cosine metric needs float32 or float16 vectors");
  if (is_int && dim <= kMaxCodeBytes) {
    screen_kind_ = 1;  // the stored row is its own code
    pitch_       = static_cast<size_t>(round_up(dim, 128));
    code_pitch_  = pitch_;
  } else {
    pitch_ = static_cast<size_t>(round_up(dim * dtype_size(dtype), 16));
    if (!is_int && dim * 2 <= kMaxCodeBytes) {
      screen_kind_ = 2;  // fp16 codes
      code_pitch_  = static_cast<size_t>(round_up(dim * 2, 128));
    }
  }
  kb_ = static_cast<int>(code_pitch_ / 128);
  if (screen_kind_ == 2) {
    CERTEX_CUDA(cudaMalloc(&maxima_, 4 * sizeof(unsigned int)));
    CERTEX_CUDA(cudaMemsetAsync(maxima_, 0, 4 * sizeof(unsigned int), res.stream));
    res.sync();
  }
}

namespace {
/// The vectors of an index: device memory, or page-locked host memory mapped into the device's address space (with
/// unified addressing the same pointer serves host and device).
void* alloc_vectors(size_t bytes, bool on_host)
{
  void* p = nullptr;
  if (on_host) {
    const cudaError_t e = cudaHostAlloc(&p, std::max<size_t>(bytes, 1), cudaHostAllocMapped | cudaHostAllocPortable);
    if (e == cudaErrorMemoryAllocation) {
      cudaGetLastError();
      throw OutOfMemory("certex: out of page-locked host memory (" + std::to_string(bytes) + " bytes of vectors)");
    }
    CERTEX_CUDA(e);
  } else {
    CERTEX_CUDA(cudaMalloc(&p, std::max<size_t>(bytes, 1)));
  }
  return p;
}
void free_vectors(void* p, bool on_host)
{
  if (on_host) {
    cudaFreeHost(p);
  } else {
    cudaFree(p);
  }
}
}  // namespace

Index::~Index()
{
  free_vectors(vectors_, host_vectors_);
  cudaFree(removed_);
  cudaFree(labels_);
  cudaFree(part_ids_);
  cudaFree(lcodes_), cudaFree(linit_), cudaFree(lcmax_), cudaFree(lperm_), cudaFree(linv_);
  cudaFree(codes_);
  cudaFree(perm_);
  cudaFree(inv_);
  cudaFree(init_);
  cudaFree(cmax_);
  cudaFree(maxima_);
  cudaFree(sqnorm_);
  for (auto& kv : plans_) { cudaFree(kv.second.segs), cudaFree(kv.second.begin); }
}

Index::DevicePlan Index::device_plan(int nqt, int nt, int panel_tiles, int grid, int chunk_tiles) const
{
  const std::array<int, 5> key{nqt, nt, panel_tiles, grid, chunk_tiles};
  std::lock_guard<std::mutex> lock(plans_mutex_);
  auto it = plans_.find(key);
  if (it != plans_.end()) { return it->second; }
  DevicePlan d;
  if (plans_.size() >= kMaxPlans) { return d; }  // shapes keep changing (an index that grows between searches): not kept
  const ChunkedPlan plan = plan_chunked(nqt, nt, panel_tiles, grid, chunk_tiles);
  CERTEX_CUDA(cudaMalloc(&d.segs, std::max<size_t>(plan.segs.size(), 1) * sizeof(ScreenSeg)));
  if (cudaMalloc(&d.begin, plan.begin.size() * sizeof(int)) != cudaSuccess) {
    cudaFree(d.segs);
    throw Error("certex: out of device memory for a work split");
  }
  // blocking copies: the plan is complete before any stream of any thread can be given it
  cudaError_t e = cudaMemcpy(d.segs, plan.segs.data(), plan.segs.size() * sizeof(ScreenSeg), cudaMemcpyHostToDevice);
  if (e == cudaSuccess) { e = cudaMemcpy(d.begin, plan.begin.data(), plan.begin.size() * sizeof(int), cudaMemcpyHostToDevice); }
  if (e != cudaSuccess) {
    cudaFree(d.segs), cudaFree(d.begin);
    CERTEX_CUDA(e);
  }
  plans_[key] = d;
  return d;
}

void Index::reserve(const Resources& res, int64_t n)
{
  if (n <= capacity_) { return; }
  const int64_t cap = std::max<int64_t>(n, 2 * capacity_);
  void* v           = nullptr;
  uint8_t* r        = nullptr;
  int32_t* l        = nullptr;
  void* co          = nullptr;
  int32_t *pe = nullptr, *iv = nullptr, *in = nullptr, *cm = nullptr;
  double* sq  = nullptr;
  const int64_t pad_old = round_up(size_, kTile), pad_new = round_up(cap, kTile);
  v = alloc_vectors(static_cast<size_t>(cap) * pitch_, host_vectors_);
  CERTEX_CUDA(cudaMalloc(&r, static_cast<size_t>(round_up(cap, 4))));
  CERTEX_CUDA(cudaMemsetAsync(r, 0, static_cast<size_t>(round_up(cap, 4)), res.stream));
  if (labels_) {
    CERTEX_CUDA(cudaMalloc(&l, static_cast<size_t>(cap) * 4));
    CERTEX_CUDA(cudaMemsetAsync(l, 0xff, static_cast<size_t>(cap) * 4, res.stream));
  }
  // the squared norms the cosine verification would otherwise sum again for every candidate
  const bool keep_sqnorm = params_.metric == kCos && !host_vectors_ && (dtype_ == kF32 || dtype_ == kF16);
  if (keep_sqnorm) { CERTEX_CUDA(cudaMalloc(&sq, static_cast<size_t>(cap) * 8)); }
  if (screen_kind_) {
    const int32_t never = screen_kind_ == 2 ? static_cast<int32_t>(0xff800000u) : kNeverInit;  // -inf or -2^30
    CERTEX_CUDA(cudaMalloc(&co, static_cast<size_t>(cap) * code_pitch_));
    CERTEX_CUDA(cudaMalloc(&pe, static_cast<size_t>(cap) * 4));
    CERTEX_CUDA(cudaMalloc(&iv, static_cast<size_t>(cap) * 4));
    CERTEX_CUDA(cudaMalloc(&in, static_cast<size_t>(pad_new) * 4));
    CERTEX_CUDA(cudaMalloc(&cm, static_cast<size_t>(pad_new / kChainRows) * 4));
    launch_fill_i32(in, pad_new, never, res.stream);
    launch_fill_i32(cm, pad_new / kChainRows, never, res.stream);
    CERTEX_CUDA(cudaGetLastError());
  }
  if (size_ > 0) {
    const auto d2d = cudaMemcpyDeviceToDevice;
    CERTEX_CUDA(cudaMemcpyAsync(v, vectors_, static_cast<size_t>(size_) * pitch_, cudaMemcpyDefault, res.stream));
    CERTEX_CUDA(cudaMemcpyAsync(r, removed_, static_cast<size_t>(round_up(size_, 4)), d2d, res.stream));
    if (labels_) { CERTEX_CUDA(cudaMemcpyAsync(l, labels_, static_cast<size_t>(size_) * 4, d2d, res.stream)); }
    if (sq && sqnorm_) { CERTEX_CUDA(cudaMemcpyAsync(sq, sqnorm_, static_cast<size_t>(size_) * 8, d2d, res.stream)); }
    if (screen_kind_) {
      CERTEX_CUDA(cudaMemcpyAsync(co, codes_, static_cast<size_t>(size_) * code_pitch_, d2d, res.stream));
      CERTEX_CUDA(cudaMemcpyAsync(pe, perm_, static_cast<size_t>(size_) * 4, d2d, res.stream));
      CERTEX_CUDA(cudaMemcpyAsync(iv, inv_, static_cast<size_t>(size_) * 4, d2d, res.stream));
      CERTEX_CUDA(cudaMemcpyAsync(in, init_, static_cast<size_t>(pad_old) * 4, d2d, res.stream));
      CERTEX_CUDA(cudaMemcpyAsync(cm, cmax_, static_cast<size_t>(pad_old / kChainRows) * 4, d2d, res.stream));
    }
  }
  res.sync();
  void* old[8] = {vectors_, removed_, labels_, codes_, perm_, inv_, init_, cmax_};
  double* old_sq = sqnorm_;
  {
    std::unique_lock<ReaderGate> lock(rw_);  // waits for running searches, which read the old arrays
    vectors_ = v;
    removed_ = r;
    if (l) { labels_ = l; }
    codes_ = co, perm_ = pe, inv_ = iv, init_ = in, cmax_ = cm;
    if (sq) { sqnorm_ = sq; }
    capacity_ = cap;
  }
  if (sq) { cudaFree(old_sq); }
  free_vectors(old[0], host_vectors_);
  for (int i = 1; i < 8; ++i) {
    if (i != 2 || l) { cudaFree(old[i]); }
  }
}

void Index::extend(const Resources& res, const void* rows, int64_t n, bool on_host)
{
  if (n <= 0) { return; }
  std::lock_guard<std::mutex> w(writer_);
  CERTEX_EXPECTS(size_ + n < (int64_t(1) << 31) - 256, "certex: at most 2^31 - 257 vectors per index");
  reserve(res, size_ + n);
  uint8_t* dst          = static_cast<uint8_t*>(vectors_) + static_cast<size_t>(size_) * pitch_;
  const size_t row_bytes = static_cast<size_t>(dim_) * dtype_size(dtype_);
  const auto kind        = host_vectors_ ? cudaMemcpyDefault : on_host ? cudaMemcpyHostToDevice : cudaMemcpyDeviceToDevice;
  if (row_bytes == pitch_) {
    CERTEX_CUDA(cudaMemcpyAsync(dst, rows, static_cast<size_t>(n) * pitch_, kind, res.stream));
  } else {
    CERTEX_CUDA(cudaMemsetAsync(dst, 0, static_cast<size_t>(n) * pitch_, res.stream));
    CERTEX_CUDA(cudaMemcpy2DAsync(dst, pitch_, rows, row_bytes, row_bytes, static_cast<size_t>(n), kind, res.stream));
  }
  if (labels_) { CERTEX_CUDA(cudaMemsetAsync(labels_ + size_, 0xff, static_cast<size_t>(n) * 4, res.stream)); }
  if (sqnorm_) {
    launch_row_sqnorms(dst, pitch_, dtype_, static_cast<int>(dim_), n, sqnorm_ + size_, res.stream);
    CERTEX_CUDA(cudaGetLastError());
  }
  std::unique_lock<ReaderGate> lock(rw_, std::defer_lock);
  if (screen_kind_) {
    // The batch goes into sorted rows [size, size + n), ordered by squared norm; rows beyond the published size are
    // invisible to running searches, which bound tiles and candidates by their own size. With the L2 metric small
    // batches are not left as sorted runs of their own (chains of 16 rows would mix norms and the screen's keep rule
    // would loosen): the runs at the end of the index that are no longer than twice what follows them are sorted again
    // together with the batch, until a run reaches kFrozenRun rows. Those rows are visible, so searches wait meanwhile.
    int64_t a = size_, m = n;
    if (params_.metric == kL2) {
      while (!runs_.empty() && runs_.back().second <= 2 * m && runs_.back().second < kFrozenRun) {
        a = runs_.back().first;
        m += runs_.back().second;
        runs_.pop_back();
      }
      m = size_ + n - a;
      if (m < kFrozenRun) { runs_.emplace_back(a, m); }
    }
    if (a < size_) { lock.lock(); }
    Scratch scratch(res.stream);
    const bool f16     = screen_kind_ == 2;
    int32_t* e         = scratch.get<int32_t>(static_cast<size_t>(m));
    uint32_t* keys_in  = scratch.get<uint32_t>(static_cast<size_t>(m));
    uint32_t* keys_out = scratch.get<uint32_t>(static_cast<size_t>(m));
    int32_t* ids_in    = scratch.get<int32_t>(static_cast<size_t>(m));
    int32_t* ids_out   = scratch.get<int32_t>(static_cast<size_t>(m));
    const size_t tb    = sort_batch_temp_bytes(m);
    void* temp         = scratch.get<uint8_t>(tb);
    const void* src    = vectors_;  // code rows by id: the stored rows themselves (8-bit), or fresh fp16 codes
    int64_t src_id0    = 0;
    const uint8_t* from = static_cast<const uint8_t*>(vectors_) + static_cast<size_t>(a) * pitch_;
    if (f16) {
      uint8_t* fresh = scratch.get<uint8_t>(static_cast<size_t>(m) * code_pitch_);
      launch_encode_f16_rows(from, pitch_, dtype_, static_cast<int>(dim_), params_.metric, m, fresh, code_pitch_,
                             reinterpret_cast<float*>(e), maxima_, res.stream);
      src     = fresh;
      src_id0 = a;
    } else {
      launch_row_init(from, pitch_, dtype_, static_cast<int>(dim_), kL2, nullptr, 0, m, m, e, res.stream);
    }
    if (a < size_ && n_removed_ > 0) { launch_mask_removed(e, removed_ + a, size_ - a, f16, res.stream); }
    CERTEX_CUDA(cudaGetLastError());
    launch_sort_batch(e, m, static_cast<int32_t>(a), a, src, src_id0, code_pitch_, params_.metric, f16, keys_in, keys_out,
                      ids_in, ids_out, temp, tb, codes_, perm_, inv_, init_, res.stream);
    CERTEX_CUDA(cudaGetLastError());
    const int64_t c0 = a / kChainRows, c1 = (size_ + n + kChainRows - 1) / kChainRows;
    launch_chain_max(init_, c0, c1 - c0, cmax_, f16, res.stream);
    CERTEX_CUDA(cudaGetLastError());
    if (f16) {
      unsigned int h[4] = {0, 0, 0, 0};
      CERTEX_CUDA(cudaMemcpyAsync(h, maxima_, sizeof(h), cudaMemcpyDeviceToHost, res.stream));
      res.sync();
      std::memcpy(&n1max_, &h[0], 4);
      std::memcpy(&n2max_, &h[1], 4);
      std::memcpy(&emax_, &h[2], 4);
      code_overflow_ = h[3] != 0;
    }
  }
  res.sync();
  if (!lock.owns_lock()) { lock.lock(); }
  size_ += n;
}

void Index::remove(const Resources& res, const int64_t* ids_device, int64_t n_ids)
{
  if (n_ids <= 0) { return; }
  std::lock_guard<std::mutex> w(writer_);
  Scratch scratch(res.stream);
  auto* counter = scratch.get<unsigned long long>(1);
  CERTEX_CUDA(cudaMemsetAsync(counter, 0, sizeof(unsigned long long), res.stream));
  launch_remove(ids_device, n_ids, size_, removed_, init_, inv_, cmax_, screen_kind_ == 2, counter, res.stream);
  if (linv_ && n_part_ > 0) {  // the same rows in the label-ordered copy (the flags are set: nothing is counted twice)
    launch_remove(ids_device, n_ids, n_part_, removed_, linit_, linv_, lcmax_, screen_kind_ == 2, counter, res.stream);
  }
  CERTEX_CUDA(cudaGetLastError());
  unsigned long long n_new = 0;
  CERTEX_CUDA(cudaMemcpyAsync(&n_new, counter, sizeof(n_new), cudaMemcpyDeviceToHost, res.stream));
  res.sync();
  std::unique_lock<ReaderGate> lock(rw_);
  n_removed_ += static_cast<int64_t>(n_new);
}

void Index::set_labels(const Resources& res, const int32_t* labels_device, int64_t n, int64_t first)
{
  std::lock_guard<std::mutex> w(writer_);
  CERTEX_EXPECTS(first >= 0 && n >= 0 && first + n <= size_, "certex: labels beyond the vectors of the index");
  if (!labels_) {
    int32_t* l = nullptr;
    CERTEX_CUDA(cudaMalloc(&l, static_cast<size_t>(std::max<int64_t>(capacity_, 1)) * 4));
    CERTEX_CUDA(cudaMemsetAsync(l, 0xff, static_cast<size_t>(std::max<int64_t>(capacity_, 1)) * 4, res.stream));
    res.sync();
    std::unique_lock<ReaderGate> lock(rw_);
    labels_ = l;
  }
  if (n > 0) {
    CERTEX_CUDA(cudaMemcpyAsync(labels_ + first, labels_device, static_cast<size_t>(n) * 4, cudaMemcpyDeviceToDevice, res.stream));
  }
  res.sync();
  std::unique_lock<ReaderGate> lock(rw_);
  has_labels_ = true;
  if (first < n_part_ && n > 0) { n_part_ = 0; }  // labels of partitioned rows changed: the partition is void
}

void Index::partition_by_labels(const Resources& res)
{
  std::lock_guard<std::mutex> w(writer_);
  CERTEX_EXPECTS(has_labels_, "certex: the index has no labels");
  const int64_t n = size_;
  if (n == 0) { return; }
  int32_t* ids = nullptr;
  CERTEX_CUDA(cudaMalloc(&ids, static_cast<size_t>(n) * 4));
  std::vector<int32_t> distinct, counts;
  try {
    Scratch scratch(res.stream);
    int32_t* sorted   = scratch.get<int32_t>(static_cast<size_t>(n));
    int32_t* iota     = scratch.get<int32_t>(static_cast<size_t>(n));
    int32_t* d_dist   = scratch.get<int32_t>(static_cast<size_t>(n));
    int32_t* d_counts = scratch.get<int32_t>(static_cast<size_t>(n));
    int32_t* d_n      = scratch.get<int32_t>(1);
    const size_t tb   = label_partition_temp_bytes(n);
    void* temp        = scratch.get<uint8_t>(tb);
    launch_label_partition(labels_, n, sorted, iota, ids, d_dist, d_counts, d_n, temp, tb, res.stream);
    CERTEX_CUDA(cudaGetLastError());
    int32_t n_distinct = 0;
    CERTEX_CUDA(cudaMemcpyAsync(&n_distinct, d_n, 4, cudaMemcpyDeviceToHost, res.stream));
    res.sync();
    distinct.resize(static_cast<size_t>(n_distinct));
    counts.resize(static_cast<size_t>(n_distinct));
    CERTEX_CUDA(cudaMemcpyAsync(distinct.data(), d_dist, distinct.size() * 4, cudaMemcpyDeviceToHost, res.stream));
    CERTEX_CUDA(cudaMemcpyAsync(counts.data(), d_counts, counts.size() * 4, cudaMemcpyDeviceToHost, res.stream));
    res.sync();
  } catch (...) {
    cudaFree(ids);
    throw;
  }
  std::vector<int64_t> offsets(distinct.size() + 1, 0);
  for (size_t i = 0; i < distinct.size(); ++i) { offsets[i + 1] = offsets[i] + counts[i]; }

  // With a tensor-core screen: a copy of the code rows in label order, every label's block padded to whole tiles of
  // 256 rows, with its own e, chain maxima and row <-> id maps, so that a label's queries are screened against the
  // label's rows only (the reference's partition rows, cpp/src/neighbors/certex/certex.cu:1590-1604).
  void* lcodes = nullptr;
  int32_t *linit = nullptr, *lcmax = nullptr, *lperm = nullptr, *linv = nullptr;
  int64_t n_lrows = 0;
  std::vector<int64_t> tile0(distinct.size(), 0);
  if (screen_kind_ != 0 && !code_overflow_) {
    std::vector<int64_t> lrow0(distinct.size(), 0);
    for (size_t i = 0; i < distinct.size(); ++i) {
      lrow0[i] = n_lrows;
      tile0[i] = n_lrows / kTile;
      n_lrows += round_up(counts[i], kTile);
    }
    try {
      const bool f16      = screen_kind_ == 2;
      const int32_t never = f16 ? static_cast<int32_t>(0xff800000u) : kNeverInit;
      CERTEX_CUDA(cudaMalloc(&lcodes, static_cast<size_t>(n_lrows) * code_pitch_));
      CERTEX_CUDA(cudaMalloc(&linit, static_cast<size_t>(n_lrows) * 4));
      CERTEX_CUDA(cudaMalloc(&lcmax, static_cast<size_t>(n_lrows / kChainRows) * 4));
      CERTEX_CUDA(cudaMalloc(&lperm, static_cast<size_t>(n_lrows) * 4));
      CERTEX_CUDA(cudaMalloc(&linv, static_cast<size_t>(n) * 4));
      Scratch scratch(res.stream);
      int32_t* lsrc   = scratch.get<int32_t>(static_cast<size_t>(n_lrows));
      int64_t* d_off  = scratch.get<int64_t>(offsets.size());
      int64_t* d_row0 = scratch.get<int64_t>(lrow0.size());
      CERTEX_CUDA(cudaMemcpyAsync(d_off, offsets.data(), offsets.size() * 8, cudaMemcpyHostToDevice, res.stream));
      CERTEX_CUDA(cudaMemcpyAsync(d_row0, lrow0.data(), lrow0.size() * 8, cudaMemcpyHostToDevice, res.stream));
      launch_fill_i32(linit, n_lrows, never, res.stream);
      launch_fill_i32(lperm, n_lrows, -1, res.stream);
      launch_fill_i32(lsrc, n_lrows, -1, res.stream);
      // inside a label the copy is ordered by norm, like the main copy of the code rows: the screen's keep rule relies
      // on e being almost constant over 16 adjacent rows
      auto* keys_in   = scratch.get<unsigned long long>(static_cast<size_t>(n));
      auto* keys_out  = scratch.get<unsigned long long>(static_cast<size_t>(n));
      int32_t* order  = scratch.get<int32_t>(static_cast<size_t>(n));
      const size_t tb = label_norm_order_temp_bytes(n);
      void* temp      = scratch.get<uint8_t>(tb);
      launch_label_norm_order(ids, n, labels_, inv_, init_, f16, keys_in, keys_out, order, temp, tb, res.stream);
      launch_label_rows(order, n, d_off, d_row0, static_cast<int>(distinct.size()), inv_, init_, lperm, linv, lsrc, linit,
                        res.stream);
      launch_gather_rows(codes_, code_pitch_, lsrc, n_lrows, n_lrows, lcodes, code_pitch_, code_pitch_, res.stream);
      launch_chain_max(linit, 0, n_lrows / kChainRows, lcmax, f16, res.stream);
      CERTEX_CUDA(cudaGetLastError());
      res.sync();
    } catch (...) {
      cudaFree(ids), cudaFree(lcodes), cudaFree(linit), cudaFree(lcmax), cudaFree(lperm), cudaFree(linv);
      throw;
    }
  }
  void* old[6] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
  {
    std::unique_lock<ReaderGate> lock(rw_);
    old[0] = part_ids_, old[1] = lcodes_, old[2] = linit_, old[3] = lcmax_, old[4] = lperm_, old[5] = linv_;
    part_ids_     = ids;
    n_part_       = n;
    part_labels_  = std::move(distinct);
    part_offsets_ = std::move(offsets);
    part_tile0_   = std::move(tile0);
    lcodes_ = lcodes, linit_ = linit, lcmax_ = lcmax, lperm_ = lperm, linv_ = linv;
    n_lrows_ = n_lrows;
  }
  for (void* p : old) { cudaFree(p); }
}

// -------------------------------------------------------------------------------------------- search
void Index::search_dense(const Resources& res, const void* q, size_t qpitch, const int32_t* qsel, int q0, int nqb, int k,
                         const Admit& adm, double* best_s, int32_t* best_row, int64_t n) const
{
  if (nqb <= 0) { return; }
  Scratch scratch(res.stream);
  const int64_t ld      = round_up(std::max<int64_t>(n, 1), 4);
  const int64_t budget  = int64_t(1) << 30;  // bytes of score matrix per step
  const int step        = static_cast<int>(std::max<int64_t>(1, std::min<int64_t>({nqb, budget / (ld * 8), kDenseMaxQueries})));
  double* scores        = scratch.get<double>(static_cast<size_t>(step) * ld);
  const int parts       = select_topk_parts(n, k);
  double* part_s        = scratch.get<double>(static_cast<size_t>(step) * parts * k);
  int32_t* part_row     = scratch.get<int32_t>(static_cast<size_t>(step) * parts * k);
  for (int b = 0; b < nqb; b += step) {
    const int nb = std::min(step, nqb - b);
    launch_dense_scores(vectors_, pitch_, dtype_, static_cast<int>(dim_), params_.metric, n, q, qpitch,
                        qsel ? qsel + b : nullptr, q0 + b, nb, adm, scores, ld, res.stream);
    CERTEX_CUDA(cudaGetLastError());
    launch_select_topk(scores, ld, n, k, qsel ? qsel + b : nullptr, q0 + b, nb, best_s, best_row, part_s, part_row, res.stream);
    CERTEX_CUDA(cudaGetLastError());
  }
}

// One pass of the screen over all rows with given thresholds, then the exact scores of the survivors and the k best.
// qcodes: code rows of the nq queries (zero padded to a multiple of 128 rows); queries: their vectors; lists are
// written at query numbers q0 .. q0 + nq - 1. With `thr2` the queries that end in ovf_list also get a tighter threshold
// (see Refine).
void Index::screen_pass(const Resources& res, const uint8_t* qcodes, const int32_t* thr, const void* queries,
                        size_t row_bytes, int q0, int nq, int k, double* best_s, int32_t* best_row, int32_t* ovf_list,
                        unsigned int* ovf_count, unsigned long long* stats, int* err, int64_t n, int32_t* thr2,
                        const float* shift, const Admit& adm, std::vector<cudaEvent_t>* events) const
{
  Scratch scratch(res.stream);
  const int grid          = res.sm_count;
  const ScreenShape shape = shape_for(kb_);
  const int nqt           = static_cast<int>((nq + kQTile - 1) / kQTile);
  const int nt_all        = static_cast<int>((n + kTile - 1) / kTile);
  const uint32_t cap      = test_mode_ == 2 ? static_cast<uint32_t>(test_cap_) : static_cast<uint32_t>(std::max(2048, 2 * k));
  // a record holds the survivors of one chain of 16 rows: as many records as candidate slots always suffice
  const unsigned long long rec_cap = std::max<unsigned long long>(1ull << 20, static_cast<unsigned long long>(nq) * cap);
  uint32_t* cnt        = scratch.get<uint32_t>(static_cast<size_t>(nq));
  int32_t* cand        = scratch.get<int32_t>(static_cast<size_t>(nq) * cap);
  uint64_t* rec        = scratch.get<uint64_t>(static_cast<size_t>(rec_cap));
  auto* rec_count      = scratch.get<unsigned long long>(1);
  const DevicePlan plan = device_plan(nqt, nt_all, shape.panel_tiles, grid, chunk_tiles_for(code_pitch_));
  auto* d_segs          = static_cast<ScreenSeg*>(plan.segs);
  int* d_seg_begin      = plan.begin;
  if (!d_segs) { upload_plan(scratch, plan_chunked(nqt, nt_all, shape.panel_tiles, grid, chunk_tiles_for(code_pitch_)), d_segs, d_seg_begin); }
  CERTEX_CUDA(cudaMemsetAsync(cnt, 0, sizeof(uint32_t) * nq, res.stream));
  CERTEX_CUDA(cudaMemsetAsync(rec_count, 0, sizeof(unsigned long long), res.stream));
  const size_t cp        = code_pitch_;
  const CUtensorMap tm_q = make_code_map(qcodes, cp, static_cast<uint64_t>(round_up(nq, kQTile)), cp, kQueryTile);
  const CUtensorMap tm_x = make_code_map(codes_, cp, static_cast<uint64_t>(n), cp, kBaseTile);
  ScreenArgs a{};
  a.nq          = nq;
  a.kb          = kb_;
  a.panel_tiles = shape.panel_tiles;
  a.n_stages    = shape.n_stages;
  a.f16         = screen_kind_ == 2 ? 1 : 0;
  a.wide        = kb_ > 2 ? 1 : 0;
  a.q_signed    = dtype_ == kI8 ? 1u : 0u;
  a.x_signed    = a.q_signed;
  a.err         = err;
  a.mode        = kModeScreen;
  a.init        = init_;
  a.cmax        = cmax_;
  a.thr         = thr;
  a.rec         = rec;
  a.rec_count   = rec_count;
  a.rec_cap     = rec_cap;
  a.segs        = d_segs;
  a.seg_begin   = d_seg_begin;
  auto mark = [&] {
    if (events) {
      cudaEvent_t e;
      CERTEX_CUDA(cudaEventCreate(&e));
      CERTEX_CUDA(cudaEventRecord(e, res.stream));
      events->push_back(e);
    }
  };
  mark();
  CERTEX_CUDA(screen_i8_launch(tm_q, tm_x, a, grid, res.stream));
  mark();
  launch_expand_records(rec, rec_count, rec_cap, n, perm_, cnt, cand, cap, res.sm_count, res.stream);
  CERTEX_CUDA(cudaGetLastError());
  Refine rf{};
  rf.thr2  = thr2;
  rf.thr   = thr;
  rf.shift = shift;
  rf.kind  = screen_kind_;
  // 8-bit vectors kept in host memory: the exact stage reads the candidates' code rows, which are the vectors
  const bool from_codes = host_vectors_ && screen_kind_ == 1;
  launch_verify_select(from_codes ? codes_ : vectors_, pitch_, dtype_, static_cast<int>(dim_), params_.metric, queries, row_bytes,
                       nq, q0, cand, cnt, cap, k, adm, best_s, best_row, ovf_list, ovf_count, stats, rec_count, rec_cap, rf,
                       res.stream, from_codes ? inv_ : nullptr, sqnorm_);
  CERTEX_CUDA(cudaGetLastError());
}

void Index::search_screened(const Resources& res, const uint8_t* qbuf, const float* shift, const void* queries,
                            size_t row_bytes, int q0, int nq, int k, double* best_s, int32_t* best_row, int32_t* ovf_list,
                            unsigned int* ovf_count, unsigned long long* stats, int* err, int anchor_stride, int64_t n,
                            int32_t* thr2, const Admit& adm, std::vector<cudaEvent_t>* events) const
{
  // qbuf: the code rows of all queries of the call, zero padded to [round_up(total, 128), code_pitch_]; this batch is
  // rows [q0, q0 + nq). shift (fp16 codes only): the rounding allowance of every query.
  Scratch scratch(res.stream);
  const int grid          = res.sm_count;
  const ScreenShape shape = shape_for(kb_);
  const int nqt           = static_cast<int>((nq + kQTile - 1) / kQTile);
  // anchors: sorted rows 0, stride, 2 stride, ...; only whole tiles of 256 anchors take part
  const int nt_anchor     = static_cast<int>(n / (static_cast<int64_t>(anchor_stride) * kTile));
  const int n_groups      = nt_anchor * (kBaseTile / kGroupRows);
  const int64_t ld_g      = round_up(n_groups, 8);

  // The threshold stage at the screen's price (chains of 16 adjacent anchors, e per chain: kModeGroupBound) unless
  // anchors are masked one by one: a bitset filter, or many removed rows (a chain with a masked anchor drops out whole).
  const bool chained   = adm.bits == nullptr && n_removed_ * 64 <= n && test_mode_ != 5;
  int32_t* anchor_init = scratch.get<int32_t>(chained ? static_cast<size_t>(nt_anchor) * (kTile / kChainRows)
                                                      : static_cast<size_t>(nt_anchor) * kTile);
  int32_t* gmax        = scratch.get<int32_t>(static_cast<size_t>(nq) * ld_g);
  int32_t* thr         = scratch.get<int32_t>(static_cast<size_t>(nq));
  // an anchor tile is 256 rows spread over the whole set: chunks by bytes of anchor rows, as for the screen
  const DevicePlan plan_a = device_plan(nqt, nt_anchor, shape.panel_tiles, grid, chunk_tiles_for(code_pitch_));
  auto* d_segs            = static_cast<ScreenSeg*>(plan_a.segs);
  int* d_seg_begin        = plan_a.begin;
  if (!d_segs) { upload_plan(scratch, plan_chunked(nqt, nt_anchor, shape.panel_tiles, grid, chunk_tiles_for(code_pitch_)), d_segs, d_seg_begin); }
  if (chained) {  // the smallest e of every chain of 16 adjacent anchors
    // anchor a = sorted row a * stride; chain i of tile t = anchors (i * nt_anchor + t) * 16 .. + 15
    launch_gather_chain_min(init_, anchor_stride, static_cast<int64_t>(nt_anchor) * kChainRows * anchor_stride,
                            static_cast<int64_t>(kChainRows) * anchor_stride, nt_anchor, anchor_init, screen_kind_ == 2, res.stream);
  } else {        // e of the anchors; with a bitset filter the anchors it drops do not count
    launch_gather_init(init_, anchor_stride, nt_anchor, anchor_init, res.stream, adm.bits, perm_,
                       screen_kind_ == 2 ? static_cast<int32_t>(0xff800000u) : kNeverInit);
  }
  CERTEX_CUDA(cudaGetLastError());

  const size_t cp        = code_pitch_;
  const uint8_t* qb      = qbuf + static_cast<size_t>(q0) * cp;
  const CUtensorMap tm_q = make_code_map(qb, cp, static_cast<uint64_t>(round_up(nq, kQTile)), cp, kQueryTile);
  const CUtensorMap tm_a =
    chained ? make_chain_map(codes_, cp, static_cast<uint64_t>(anchor_stride) * cp, static_cast<uint64_t>(nt_anchor))
            : make_tile_map(codes_, cp, static_cast<uint64_t>(nt_anchor) * anchor_stride * cp,
                            static_cast<uint64_t>(anchor_stride) * cp, static_cast<uint64_t>(nt_anchor));
  ScreenArgs a{};
  a.nq          = nq;
  a.kb          = kb_;
  a.panel_tiles = shape.panel_tiles;
  a.n_stages    = shape.n_stages;
  a.f16         = screen_kind_ == 2 ? 1 : 0;
  a.wide        = kb_ > 2 ? 1 : 0;
  a.q_signed    = dtype_ == kI8 ? 1u : 0u;
  a.x_signed    = a.q_signed;
  a.err         = err;
  // 1 anchors: a value that some anchor of every group of 64 reaches (the group's maximum, or the chained bound)
  a.mode    = chained ? kModeGroupBound : kModeGroupMax;
  a.init    = anchor_init;
  a.cmax    = anchor_init;
  a.gmax    = gmax;
  a.ld_gmax = ld_g;
  a.segs    = d_segs;
  a.seg_begin = d_seg_begin;
  auto mark = [&] {
    if (events) {
      cudaEvent_t e;
      CERTEX_CUDA(cudaEventCreate(&e));
      CERTEX_CUDA(cudaEventRecord(e, res.stream));
      events->push_back(e);
    }
  };
  mark();
  CERTEX_CUDA(screen_i8_launch(tm_q, tm_a, a, grid, res.stream));
  mark();
  // 2 threshold: the k-th largest group maximum
  // (with an exchange between row shards also the k largest group values of every query, in the same launch)
  const bool wide_exchange = topk_hook != nullptr && k <= kTopkExchangeMaxK;
  int32_t* topk            = wide_exchange ? scratch.get<int32_t>(static_cast<size_t>(nq) * k) : nullptr;
  launch_kth_largest(gmax, ld_g, n_groups, k, nq, thr, res.stream, nullptr, 0x7fffffff, topk);
  if (screen_kind_ == 2) {
    launch_finish_thr_f16(thr, shift + q0, nq, 0, res.stream);
    if (wide_exchange) { launch_finish_thr_f16(topk, shift + q0, nq * k, 0, res.stream, k); }
  }
  CERTEX_CUDA(cudaGetLastError());
  // thr now holds, per query, (a key of) a score k rows of this index certainly reach: other shards may tighten it
  if (wide_exchange) {
    topk_hook(threshold_hook_ctx, topk, thr, nq, k, res.stream);
  } else if (threshold_hook) {
    threshold_hook(threshold_hook_ctx, thr, nq, res.stream);
  }
  if (screen_kind_ == 2) { launch_finish_thr_f16(thr, shift + q0, nq, 1, res.stream); }
  CERTEX_CUDA(cudaGetLastError());
  // 3 screen over all rows, 4 exact scores of the candidates and the k best
  screen_pass(res, qb, thr, queries, row_bytes, q0, nq, k, best_s, best_row, ovf_list, ovf_count, stats, err, n, thr2, shift,
              adm, events);
}

namespace {

/// The queries' numbers ordered by label, queries of one label in ascending order (a stable sort by label). Labels of
/// a call span a small range as a rule: one counting pass then; otherwise four radix passes over the label's bytes.
std::vector<int32_t> order_by_label(const std::vector<int32_t>& lab)
{
  const size_t nq = lab.size();
  std::vector<int32_t> order(nq);
  if (nq == 0) { return order; }
  int32_t lo = lab[0], hi = lab[0];
  for (int32_t l : lab) { lo = std::min(lo, l), hi = std::max(hi, l); }
  const uint64_t range = static_cast<uint64_t>(static_cast<int64_t>(hi) - static_cast<int64_t>(lo)) + 1;
  if (range <= (uint64_t(1) << 20)) {
    std::vector<uint32_t> at(static_cast<size_t>(range) + 1, 0u);
    for (int32_t l : lab) { ++at[static_cast<size_t>(static_cast<int64_t>(l) - lo) + 1]; }
    for (size_t i = 1; i <= range; ++i) { at[i] += at[i - 1]; }
    for (size_t i = 0; i < nq; ++i) { order[at[static_cast<size_t>(static_cast<int64_t>(lab[i]) - lo)]++] = static_cast<int32_t>(i); }
    return order;
  }
  std::vector<uint64_t> a(nq), b(nq);  // (label with the sign bit flipped, query number)
  for (size_t i = 0; i < nq; ++i) { a[i] = (static_cast<uint64_t>(static_cast<uint32_t>(lab[i]) ^ 0x80000000u) << 32) | i; }
  for (int pass = 0; pass < 4; ++pass) {
    size_t at[257] = {0};
    const int shift = 32 + 8 * pass;
    for (uint64_t v : a) { ++at[((v >> shift) & 255u) + 1]; }
    for (int i = 0; i < 256; ++i) { at[i + 1] += at[i]; }
    for (uint64_t v : a) { b[at[(v >> shift) & 255u]++] = v; }
    a.swap(b);
  }
  for (size_t i = 0; i < nq; ++i) { order[i] = static_cast<int32_t>(a[i] & 0xffffffffu); }
  return order;
}

}  // namespace

/// The queries of one label in a search by labels.
struct LabelRun {
  int64_t part_off  = 0;  // the label's entries in the partition
  int64_t n_in_part = 0;
  int64_t tile0     = 0;  // its first tile in the label-ordered copy of the screen's rows
  std::vector<int32_t> queries;
};

namespace {

/// Work split of a routed pass: run r pairs the query tiles [q_tile0[r], + nqt[r]) with its label's tiles. Segments of
/// at most `panel` query tiles are dealt to the CTAs in order, about the same number of units each, at most
/// `max_segs` per CTA. Returns how many runs fit (all, unless the segment slots ran out).
size_t plan_routed(const std::vector<LabelRun>& runs, size_t r0, size_t r1, const std::vector<int>& q_tile0, int panel,
                   int grid, int max_segs, std::vector<ScreenSeg>& segs, std::vector<int>& col0, std::vector<int>& seg_begin)
{
  int64_t units = 0;
  for (size_t r = r0; r < r1; ++r) {
    const int64_t nqt = (static_cast<int64_t>(runs[r].queries.size()) + kQTile - 1) / kQTile;
    units += nqt * ((runs[r].n_in_part + kTile - 1) / kTile);
  }
  const int64_t target = std::max<int64_t>(1, (units + grid - 1) / grid);
  segs.clear(), col0.clear(), seg_begin.assign(1, 0);
  int64_t filled = 0;
  size_t done    = r1;
  for (size_t r = r0; r < r1 && done == r1; ++r) {
    const size_t mark = segs.size();
    const size_t ctas = seg_begin.size();
    const int64_t keep = filled;
    const int nqt = static_cast<int>((runs[r].queries.size() + kQTile - 1) / kQTile);
    const int nt  = static_cast<int>((runs[r].n_in_part + kTile - 1) / kTile);
    const int t0  = static_cast<int>(runs[r].tile0);
    for (int qp = 0; qp < nqt && done == r1; qp += panel) {
      const int pq = std::min(panel, nqt - qp);
      for (int t = 0; t < nt;) {
        const bool last_cta = static_cast<int>(seg_begin.size()) == grid;
        const int in_cta    = static_cast<int>(segs.size()) - seg_begin.back();
        if (!last_cta && (filled >= target || in_cta == max_segs)) {
          seg_begin.push_back(static_cast<int>(segs.size()));
          filled = 0;
          continue;
        }
        if (last_cta && in_cta == max_segs) {  // no slot left: this run and the later ones wait for another pass
          done = r;
          break;
        }
        const int64_t room = last_cta ? int64_t(1) << 40 : target - filled;
        const int tiles    = static_cast<int>(std::min<int64_t>(nt - t, std::max<int64_t>(1, room / pq)));
        segs.push_back(ScreenSeg{q_tile0[r - r0] + qp, pq, t0 + t, t0 + t + tiles});
        col0.push_back(t0);
        filled += static_cast<int64_t>(tiles) * pq;
        t += tiles;
      }
    }
    if (done != r1) {  // undo the partial run
      segs.resize(mark), col0.resize(mark), seg_begin.resize(ctas);
      filled = keep;
    }
  }
  while (static_cast<int>(seg_begin.size()) < grid + 1) { seg_begin.push_back(static_cast<int>(segs.size())); }
  return done - r0;
}

}  // namespace

// One class of routed runs (groups of 64 rows, or with `fine` of 16): passes of at most 32 768 query slots. Returns the
// pairs the screens kept; runs' queries whose candidate list overflowed are appended to `dense`.
unsigned long long Index::search_routed(const Resources& res, const void* q, size_t qpitch, int k,
                                        std::vector<LabelRun>& routed, const bool fine, double* best_s, int32_t* best_row,
                                        SearchStats* st, std::vector<LabelRun>& dense) const
{
  unsigned long long pairs = 0;
  const int per_tile = fine ? kBaseTile / kChainRows : kBaseTile / kGroupRows;  // columns of gmax per tile
  for (size_t r0 = 0; r0 < routed.size();) {
    // as many runs as fit 32 768 query slots (a label's queries fill whole tiles of 128) and the segment slots
    size_t r1 = r0;
    int64_t n_slots = 0;
    std::vector<int> q_tile0;
    while (r1 < routed.size()) {
      const int64_t add = round_up(static_cast<int64_t>(routed[r1].queries.size()), kQTile);
      if (r1 > r0 && n_slots + add > 32768) { break; }
      if (add > 32768) {  // more queries of one label than a pass takes: the rest forms another run
        LabelRun rest = routed[r1];
        rest.queries.assign(routed[r1].queries.begin() + 32768, routed[r1].queries.end());
        routed[r1].queries.resize(32768);
        routed.insert(routed.begin() + static_cast<std::ptrdiff_t>(r1) + 1, std::move(rest));
        continue;
      }
      q_tile0.push_back(static_cast<int>(n_slots / kQTile));
      n_slots += add;
      ++r1;
    }
    const int grid          = res.sm_count;
    const ScreenShape shape = shape_for(kb_);
    std::vector<ScreenSeg> segs;
    std::vector<int> col0, seg_begin;
    r1 = r0 + plan_routed(routed, r0, r1, q_tile0, shape.panel_tiles, grid, 64, segs, col0, seg_begin);
    CERTEX_EXPECTS(r1 > r0, "certex: internal error: a label's queries do not fit one routed pass");
    // The thresholds of a large label come from a strided sample of its tiles (its rows are sorted by norm, so the sample
    // spans all norms; the group maxima of any subset of rows are valid): at least 1024 tiles (smaller labels take part
    // whole: every tile left out costs survivors, and their exact scores cost more than the tile), enough tiles for
    // 2k groups, for a sixteenth of the label, and for candidate lists that stay within half their capacity (about
    // 1.2 k rows per sampled fraction).
    const uint32_t cap = static_cast<uint32_t>(std::max(2048, 2 * k));
    std::vector<LabelRun> heads(routed.begin() + static_cast<std::ptrdiff_t>(r0), routed.begin() + static_cast<std::ptrdiff_t>(r1));
    std::vector<int> steps(heads.size(), 1);  // the sample of a large label: every steps[r]-th tile
    for (size_t r = 0; r < heads.size(); ++r) {
      LabelRun& h          = heads[r];
      const int64_t nt     = (h.n_in_part + kTile - 1) / kTile;
      const int64_t enough = (2 * static_cast<int64_t>(k) + per_tile - 1) / per_tile;
      const int64_t by_cap = (24 * static_cast<int64_t>(k) * nt + 10 * cap - 1) / (10 * static_cast<int64_t>(cap));
      const int64_t take   = std::min(nt, std::max({int64_t(1024), enough, (nt + 15) / 16, by_cap}));
      if (take < nt) {
        steps[r]    = static_cast<int>(nt / take);  // tiles tile0, tile0 + step, ... stay inside the label
        h.n_in_part = take * kTile;
      }
    }
    std::vector<ScreenSeg> segs_g;
    std::vector<int> col0_g, seg_begin_g;
    const size_t fit = plan_routed(heads, 0, heads.size(), q_tile0, shape.panel_tiles, grid, 64, segs_g, col0_g, seg_begin_g);
    CERTEX_EXPECTS(fit == heads.size(), "certex: internal error: the threshold pass of a routed search does not fit");
    std::vector<int> step_g(segs_g.size(), 1);
    for (size_t i = 0, r = 0; i < segs_g.size(); ++i) {  // segments come in the order of the runs
      while (heads[r].tile0 != col0_g[i]) { ++r; }
      step_g[i] = steps[r];
    }
    n_slots = 0;
    std::vector<int32_t> slot_query, slot_ng;
    int64_t max_tiles = 0;
    for (size_t r = r0; r < r1; ++r) {
      const LabelRun& run = routed[r];
      const int64_t nt    = (heads[r - r0].n_in_part + kTile - 1) / kTile;  // tiles that take part in the thresholds
      const int64_t add   = round_up(static_cast<int64_t>(run.queries.size()), kQTile);
      for (int64_t i = 0; i < add; ++i) {
        const bool real = i < static_cast<int64_t>(run.queries.size());
        slot_query.push_back(real ? run.queries[static_cast<size_t>(i)] : -1);
        slot_ng.push_back(real ? static_cast<int32_t>(nt * per_tile) : -1);
      }
      n_slots += add;
      max_tiles = std::max(max_tiles, nt);
    }
    const int ns = static_cast<int>(n_slots);

    Scratch scratch(res.stream);
    const bool f16       = screen_kind_ == 2;
    const size_t cp      = code_pitch_;
    const int n_groups   = static_cast<int>(max_tiles) * per_tile;
    const int64_t ld_g   = round_up(n_groups, 8);
    const unsigned long long rec_cap = std::max<unsigned long long>(1ull << 20, static_cast<unsigned long long>(ns) * cap);
    // the host's tables of the pass, sent in one copy (segs_g ...: the threshold pass over the leading tiles of every label)
    const std::vector<std::pair<const void*, size_t>> tables = {
      {slot_query.data(), slot_query.size() * 4},      {slot_ng.data(), slot_ng.size() * 4},
      {segs.data(), segs.size() * sizeof(ScreenSeg)},  {col0.data(), col0.size() * sizeof(int)},
      {seg_begin.data(), seg_begin.size() * sizeof(int)}, {segs_g.data(), segs_g.size() * sizeof(ScreenSeg)},
      {col0_g.data(), col0_g.size() * sizeof(int)},    {seg_begin_g.data(), seg_begin_g.size() * sizeof(int)},
      {step_g.data(), step_g.size() * sizeof(int)}};
    uint8_t* d_tables = scratch.get<uint8_t>(Resources::upload_bytes(tables));
    std::vector<size_t> at;
    res.upload(tables, d_tables, at);
    int32_t* d_slot_q    = reinterpret_cast<int32_t*>(d_tables + at[0]);
    int32_t* d_slot_ng   = reinterpret_cast<int32_t*>(d_tables + at[1]);
    ScreenSeg* d_segs    = reinterpret_cast<ScreenSeg*>(d_tables + at[2]);
    int* d_col0          = reinterpret_cast<int*>(d_tables + at[3]);
    int* d_seg_begin     = reinterpret_cast<int*>(d_tables + at[4]);
    ScreenSeg* d_segs_g  = reinterpret_cast<ScreenSeg*>(d_tables + at[5]);
    int* d_col0_g        = reinterpret_cast<int*>(d_tables + at[6]);
    int* d_seg_begin_g   = reinterpret_cast<int*>(d_tables + at[7]);
    int* d_step_g        = reinterpret_cast<int*>(d_tables + at[8]);
    uint8_t* q_rows      = scratch.get<uint8_t>(static_cast<size_t>(ns) * (f16 ? qpitch : cp));  // the queries in slot order
    uint8_t* q_codes     = f16 ? scratch.get<uint8_t>(static_cast<size_t>(ns) * cp) : q_rows;
    float* shift         = f16 ? scratch.get<float>(static_cast<size_t>(ns)) : nullptr;
    int32_t* gmax        = scratch.get<int32_t>(static_cast<size_t>(ns) * ld_g);
    int32_t* thr         = scratch.get<int32_t>(static_cast<size_t>(ns));
    uint32_t* cnt        = scratch.get<uint32_t>(static_cast<size_t>(ns));
    int32_t* cand        = scratch.get<int32_t>(static_cast<size_t>(ns) * cap);
    uint64_t* rec        = scratch.get<uint64_t>(static_cast<size_t>(rec_cap));
    auto* rec_count      = scratch.get<unsigned long long>(1);
    double* slot_s       = scratch.get<double>(static_cast<size_t>(ns) * k);
    int32_t* slot_row    = scratch.get<int32_t>(static_cast<size_t>(ns) * k);
    int32_t* ovf_list    = scratch.get<int32_t>(static_cast<size_t>(ns));
    unsigned int* d_flag = scratch.get<unsigned int>(4);  // [0] overflowed slots, [1] error code, [2] fp16 overflow
    auto* d_stats        = scratch.get<unsigned long long>(2);
    CERTEX_CUDA(cudaMemsetAsync(cnt, 0, sizeof(uint32_t) * ns, res.stream));
    CERTEX_CUDA(cudaMemsetAsync(rec_count, 0, sizeof(unsigned long long), res.stream));
    CERTEX_CUDA(cudaMemsetAsync(d_flag, 0, 4 * sizeof(unsigned int), res.stream));
    CERTEX_CUDA(cudaMemsetAsync(d_stats, 0, 2 * sizeof(unsigned long long), res.stream));
    // queries in slot order (8-bit vectors: zero padded to code rows, which the verification reads as well)
    const size_t q_rows_pitch = f16 ? qpitch : cp;
    launch_gather_rows(q, qpitch, d_slot_q, ns, ns, q_rows, q_rows_pitch, qpitch, res.stream);
    if (f16) {
      launch_encode_f16_queries(q_rows, qpitch, dtype_, static_cast<int>(dim_), ns, q_codes, cp, n1max_, n2max_, emax_, shift,
                                d_flag + 2, res.stream);
    }
    CERTEX_CUDA(cudaGetLastError());
    const CUtensorMap tm_q = make_code_map(q_codes, cp, static_cast<uint64_t>(ns), cp, kQueryTile);
    const CUtensorMap tm_x = make_code_map(lcodes_, cp, static_cast<uint64_t>(n_lrows_), cp, kBaseTile);
    ScreenArgs a{};
    a.nq          = ns;
    a.kb          = kb_;
    a.panel_tiles = shape.panel_tiles;
    a.n_stages    = shape.n_stages;
    a.f16         = f16 ? 1 : 0;
    a.wide        = kb_ > 2 ? 1 : 0;
    a.q_signed    = dtype_ == kI8 ? 1u : 0u;
    a.x_signed    = a.q_signed;
    a.err         = reinterpret_cast<int*>(d_flag + 1);
    a.segs        = d_segs_g;
    a.seg_begin   = d_seg_begin_g;
    a.seg_col0    = d_col0_g;
    a.seg_step    = d_step_g;
    a.plain_tiles = 1;
    a.fine_groups = fine ? 1 : 0;
    a.init        = linit_;
    // 1 group maxima over the label's own rows, 2 the k-th largest of them is the threshold
    a.mode    = kModeGroupMax;
    a.gmax    = gmax;
    a.ld_gmax = ld_g;
    std::vector<cudaEvent_t> events;
    auto mark = [&] {
      if (stats_sink) {
        cudaEvent_t e;
        CERTEX_CUDA(cudaEventCreate(&e));
        CERTEX_CUDA(cudaEventRecord(e, res.stream));
        events.push_back(e);
      }
    };
    mark();
    CERTEX_CUDA(screen_i8_launch(tm_q, tm_x, a, grid, res.stream));
    mark();
    launch_kth_largest(gmax, ld_g, n_groups, k, ns, thr, res.stream, d_slot_ng,
                       f16 ? static_cast<int32_t>(0x7f800000) : static_cast<int32_t>(0x7fffffff));
    if (f16) {
      launch_finish_thr_f16(thr, shift, ns, 0, res.stream);
      launch_finish_thr_f16(thr, shift, ns, 1, res.stream);
    }
    CERTEX_CUDA(cudaGetLastError());
    // 3 screen over all tiles of every label, 4 exact scores of the candidates
    a.mode      = kModeScreen;
    a.segs      = d_segs;
    a.seg_begin = d_seg_begin;
    a.seg_col0  = d_col0;
    a.seg_step  = nullptr;
    a.cmax      = lcmax_;
    a.thr       = thr;
    a.rec       = rec;
    a.rec_count = rec_count;
    a.rec_cap   = rec_cap;
    mark();
    CERTEX_CUDA(screen_i8_launch(tm_q, tm_x, a, grid, res.stream));
    mark();
    launch_expand_records(rec, rec_count, rec_cap, n_lrows_, lperm_, cnt, cand, cap, res.sm_count, res.stream);
    Admit plain{};
    plain.removed = removed_;
    const bool from_codes = host_vectors_ && screen_kind_ == 1;
    launch_verify_select(from_codes ? codes_ : vectors_, pitch_, dtype_, static_cast<int>(dim_), params_.metric, q_rows,
                         q_rows_pitch, ns, 0, cand, cnt, cap, k, plain, slot_s, slot_row, ovf_list, d_flag, d_stats, rec_count,
                         rec_cap, Refine{}, res.stream, from_codes ? inv_ : nullptr, sqnorm_);
    launch_scatter_best(slot_s, slot_row, d_slot_q, ns, k, best_s, best_row, res.stream);
    CERTEX_CUDA(cudaGetLastError());
    st->launches += f16 ? 10 : 8;
    unsigned int h_flag[4]        = {0, 0, 0, 0};
    unsigned long long h_stats[2] = {0, 0};
    std::vector<int32_t> h_ovf;
    CERTEX_CUDA(cudaMemcpyAsync(h_flag, d_flag, sizeof(h_flag), cudaMemcpyDeviceToHost, res.stream));
    CERTEX_CUDA(cudaMemcpyAsync(h_stats, d_stats, sizeof(h_stats), cudaMemcpyDeviceToHost, res.stream));
    res.sync();
    if (h_flag[0] > 0) {  // the list of the slots that overflowed: fetched only when there are any
      h_ovf.resize(std::min<size_t>(h_flag[0], static_cast<size_t>(ns)));
      CERTEX_CUDA(cudaMemcpyAsync(h_ovf.data(), ovf_list, h_ovf.size() * 4, cudaMemcpyDeviceToHost, res.stream));
      res.sync();
    }
    for (size_t e = 0; e + 3 < events.size(); e += 4) {
      float ms = 0;
      cudaEventElapsedTime(&ms, events[e], events[e + 1]);
      st->anchor_ms += ms;
      cudaEventElapsedTime(&ms, events[e + 2], events[e + 3]);
      st->screen_ms += ms;
      ++st->screen_passes;
    }
    for (cudaEvent_t e : events) { cudaEventDestroy(e); }
    CERTEX_EXPECTS(h_flag[1] == 0, "certex: the screening pass gave up on a wait (code " + std::to_string(h_flag[1]) + ")");
    st->routed_queries += static_cast<unsigned long long>(ns);
    pairs += h_stats[0];  // pairs the routed screen kept and the verification scored
    // slots whose list overflowed (every real slot, when a query coordinate did not fit fp16) go to the dense groups
    std::vector<char> again(static_cast<size_t>(ns), h_flag[2] != 0 ? 1 : 0);
    for (unsigned int i = 0; i < h_flag[0] && i < static_cast<unsigned int>(ns); ++i) { again[static_cast<size_t>(h_ovf[i])] = 1; }
    if (h_flag[0] != 0 || h_flag[2] != 0) {
      int64_t slot = 0;
      for (size_t r = r0; r < r1; ++r) {
        LabelRun redo = routed[r];
        redo.queries.clear();
        for (size_t i = 0; i < routed[r].queries.size(); ++i) {
          if (again[static_cast<size_t>(slot) + i]) { redo.queries.push_back(routed[r].queries[i]); }
        }
        slot += round_up(static_cast<int64_t>(routed[r].queries.size()), kQTile);
        if (!redo.queries.empty()) { dense.push_back(std::move(redo)); }
      }
    }
    r0 = r1;
  }
  return pairs;
}

unsigned long long Index::search_by_labels(const Resources& res, const void* q, size_t qpitch, int nq, int k,
                                           const Admit& adm, double* best_s, int32_t* best_row, int64_t n,
                                           SearchStats* st) const
{
  // The one host decision of the path: which queries share a label. Their labels come to the host and the queries are
  // ordered by label. A label with enough rows for a threshold (2k groups of 64) is screened on the tensor cores
  // against its block of the label-ordered copy of the code rows (routed pass); the other labels, the queries whose
  // candidate list overflowed, and every label when rows were added after the partition, are scored densely: every
  // label becomes a group (queries x that label's partition entries + the rows added since), and the groups are
  // scored, selected from and translated to ids in waves of bounded score memory, three launches per wave.
  std::vector<int32_t> lab(static_cast<size_t>(nq));
  CERTEX_CUDA(cudaMemcpyAsync(lab.data(), adm.query_labels, lab.size() * 4, cudaMemcpyDeviceToHost, res.stream));
  res.sync();
  const std::vector<int32_t> order = order_by_label(lab);  // the device waits for the host here: no comparison sort

  const int64_t n_tail = n - n_part_;
  const bool can_route = lcodes_ != nullptr && screen_kind_ != 0 && !code_overflow_ && n_tail == 0 && test_mode_ != 3;
  std::vector<LabelRun> routed, routed_fine, dense;
  for (int i = 0; i < nq;) {
    const int32_t l = lab[order[static_cast<size_t>(i)]];
    int j           = i;
    while (j < nq && lab[order[static_cast<size_t>(j)]] == l) { ++j; }
    LabelRun run;
    const auto it = std::lower_bound(part_labels_.begin(), part_labels_.end(), l);
    if (l >= 0 && it != part_labels_.end() && *it == l) {
      const size_t at = static_cast<size_t>(it - part_labels_.begin());
      run.part_off    = part_offsets_[at];
      run.n_in_part   = part_offsets_[at + 1] - part_offsets_[at];
      run.tile0       = part_tile0_.empty() ? 0 : part_tile0_[at];
    }
    run.queries.assign(order.begin() + i, order.begin() + j);
    // a threshold worth the passes needs about 2k groups: the k-th largest of them then sits near the best 1 % of the
    // label. Groups are 64 rows, or single chains of 16 rows for labels too small for that.
    const int64_t need = 2 * static_cast<int64_t>(k);
    if (can_route && run.n_in_part / kGroupRows >= need) {
      routed.push_back(std::move(run));
    } else if (can_route && run.n_in_part / kChainRows >= need) {
      routed_fine.push_back(std::move(run));
    } else {
      dense.push_back(std::move(run));
    }
    i = j;
  }
  unsigned long long pairs = 0;

  // ------------------------------------------------------------------ routed passes
  pairs += search_routed(res, q, qpitch, k, routed, false, best_s, best_row, st, dense);
  pairs += search_routed(res, q, qpitch, k, routed_fine, true, best_s, best_row, st, dense);

  // ------------------------------------------------------------------ dense groups
  std::vector<int32_t> dorder;
  for (const LabelRun& run : dense) { dorder.insert(dorder.end(), run.queries.begin(), run.queries.end()); }
  const int nd = static_cast<int>(dorder.size());
  if (nd == 0) { return pairs; }
  st->dense_queries += static_cast<unsigned long long>(nd);
  const int64_t budget  = int64_t(1) << 28;  // doubles of score memory per wave
  std::vector<LabelGroup> groups;
  std::vector<int64_t> row_off;
  std::vector<int32_t> row_n;
  Scratch keep(res.stream);
  int32_t* d_order = keep.get<int32_t>(static_cast<size_t>(nd));
  CERTEX_CUDA(cudaMemcpyAsync(d_order, dorder.data(), dorder.size() * 4, cudaMemcpyHostToDevice, res.stream));

  int wave_q0 = 0;           // first query (in label order) of the wave being collected
  int64_t wave_scores = 0, wave_blocks = 0, wave_max_cols = 0;
  auto flush = [&](int q_end) {
    if (q_end == wave_q0) { return; }
    Scratch scratch(res.stream);
    const int nqw      = q_end - wave_q0;
    double* scores     = scratch.get<double>(static_cast<size_t>(wave_scores));
    LabelGroup* d_grp  = scratch.get<LabelGroup>(groups.size());
    int64_t* d_off     = scratch.get<int64_t>(static_cast<size_t>(nqw));
    int32_t* d_n       = scratch.get<int32_t>(static_cast<size_t>(nqw));
    const int parts    = select_topk_parts(wave_max_cols, k);
    double* part_s     = scratch.get<double>(static_cast<size_t>(nqw) * parts * k);
    int32_t* part_row  = scratch.get<int32_t>(static_cast<size_t>(nqw) * parts * k);
    CERTEX_CUDA(cudaMemcpyAsync(d_grp, groups.data(), groups.size() * sizeof(LabelGroup), cudaMemcpyHostToDevice, res.stream));
    CERTEX_CUDA(cudaMemcpyAsync(d_off, row_off.data(), row_off.size() * 8, cudaMemcpyHostToDevice, res.stream));
    CERTEX_CUDA(cudaMemcpyAsync(d_n, row_n.data(), row_n.size() * 4, cudaMemcpyHostToDevice, res.stream));
    launch_dense_scores_grouped(vectors_, pitch_, dtype_, static_cast<int>(dim_), params_.metric, q, qpitch, d_order, d_grp,
                                static_cast<int>(groups.size()), wave_blocks, part_ids_, n_part_, n_tail, adm, scores, res.stream);
    CERTEX_CUDA(cudaGetLastError());
    launch_select_topk_ragged(scores, d_off, d_n, wave_max_cols, k, d_order + wave_q0, nqw, best_s, best_row, part_s, part_row,
                              res.stream);
    CERTEX_CUDA(cudaGetLastError());
    launch_group_columns_to_ids(best_row, k, d_order, d_grp, static_cast<int>(groups.size()), part_ids_, n_part_, res.stream);
    CERTEX_CUDA(cudaGetLastError());
    st->launches += 3;
    groups.clear();
    row_off.clear();
    row_n.clear();
    wave_q0 = q_end, wave_scores = 0, wave_blocks = 0, wave_max_cols = 0;
  };

  int i = 0;
  for (const LabelRun& run : dense) {
    const int j          = i + static_cast<int>(run.queries.size());
    const int64_t n_cols = run.n_in_part + n_tail;
    const int64_t ld     = round_up(n_cols, 4);
    const int at_most    = static_cast<int>(std::max<int64_t>(1, std::min<int64_t>(nd, budget / std::max<int64_t>(ld, 1))));
    for (int a = i; a < j;) {  // the label's queries, in pieces that fit the score memory of a wave
      const int nqg = std::min(j - a, at_most);
      if (wave_scores > 0 && wave_scores + static_cast<int64_t>(nqg) * ld > budget) { flush(a); }
      LabelGroup g{};
      g.q_begin   = a;
      g.nq        = nqg;
      g.part_off  = run.part_off;
      g.n_part    = static_cast<int32_t>(run.n_in_part);
      g.ld        = static_cast<int32_t>(ld);
      g.score_off = wave_scores;
      g.blk_begin = wave_blocks;
      groups.push_back(g);
      for (int t = 0; t < nqg; ++t) {
        row_off.push_back(wave_scores + static_cast<int64_t>(t) * ld);
        row_n.push_back(static_cast<int32_t>(n_cols));
      }
      wave_scores += static_cast<int64_t>(nqg) * ld;
      wave_blocks += grouped_blocks(nqg, n_cols);
      wave_max_cols = std::max(wave_max_cols, n_cols);
      pairs += static_cast<unsigned long long>(nqg) * static_cast<unsigned long long>(n_cols);
      a += nqg;
    }
    i = j;
  }
  flush(nd);
  return pairs;
}

int Index::anchor_stride_for(int64_t n, int k) const
{
  // anchors: every stride-th row in whole tiles of 256, and at least 2k groups of 64 anchors, or the threshold would be
  // useless. The k-th largest group maximum is roughly the (stride * k)-th best row: for larger k the anchors are taken
  // denser, so that the candidate lists stay a small multiple of k (the anchor pass costs 1 / stride of a screen pass).
  const int64_t by_k = std::max<int64_t>(1, static_cast<int64_t>(params_.anchor_stride) * 32 / k);
  return static_cast<int>(std::min<int64_t>({params_.anchor_stride, by_k, n / (kTile * ((2 * k + 3) / 4))}));
}

bool Index::will_screen(int k) const
{
  std::shared_lock<ReaderGate> lock(rw_);
  return screen_kind_ != 0 && !code_overflow_ && test_mode_ != 1 && k >= 1 && anchor_stride_for(size_, k) >= 1;
}

/// Counters of a screened search as the device leaves them, copied to page-locked host memory behind the search.
struct HostCounters {
  unsigned int count[4];          // [0] queries whose list overflowed, [1] error code of a pass, [2] after the second pass
  unsigned long long stats[2];    // pairs the screen kept, pairs the verification scored
  unsigned int q_ovf;             // a query coordinate beyond the fp16 range
};

/// A search between search_begin and search_end: the reader lock, the temporaries and what the repair needs.
struct Index::Pending {
  const Resources* res;
  std::shared_lock<ReaderGate> lock;
  Scratch scratch;
  SearchStats local{};
  SearchParams sp;
  const void* queries = nullptr;
  int64_t nq = 0, n = 0, id_base = 0, batch = 0;
  int k = 0;
  size_t row_bytes = 0;
  int64_t* neighbors = nullptr;
  float* distances   = nullptr;
  double* scores_out = nullptr;
  Admit adm{};
  double* best_s    = nullptr;
  int32_t* best_row = nullptr;
  bool screened     = false;  // the tensor-core screen ran: the counters decide whether the outputs stand
  uint8_t* qbuf     = nullptr;
  float* shift      = nullptr;
  unsigned int* q_ovf = nullptr;
  int32_t* ovf_list = nullptr;
  int32_t* thr2     = nullptr;
  unsigned int* d_count = nullptr;
  unsigned long long* d_stats = nullptr;
  std::vector<cudaEvent_t> events;
  cudaEvent_t ready = nullptr;
  cudaEvent_t first = nullptr;  // with statistics on: before the first operation of a screened search (ready then keeps time)
  int slot = 0;  // of the resources' page-locked blocks
  Pending(const Resources& r, ReaderGate& m) : res(&r), lock(m), scratch(r.stream) {}
  ~Pending()
  {
    for (cudaEvent_t e : events) { cudaEventDestroy(e); }
    if (ready) { cudaEventDestroy(ready); }
    if (first) { cudaEventDestroy(first); }
    --res->searches_in_flight_;
  }
};

Index::Pending* Index::search_begin(const Resources& res, const SearchParams& sp, const void* queries, int64_t nq, int k,
                                    int64_t* neighbors, float* distances, double* scores_out, const Filter& filter,
                                    int64_t id_base, unsigned long long* status_out) const
{
  CERTEX_EXPECTS(res.searches_in_flight_ < Resources::kMaxInFlight,
                 "certex: too many searches in flight on these resources (search_end the oldest first)");
  auto pending = std::make_unique<Pending>(res, rw_);
  ++res.searches_in_flight_;
  Pending& P            = *pending;
  P.slot                = static_cast<int>(res.next_slot_++ % Resources::kPinnedSlots);
  const int64_t n       = size_;
  CERTEX_EXPECTS(k >= 1 && k <= 2048, "certex: k must be between 1 and 2048");
  CERTEX_EXPECTS(n >= k, "certex: k exceeds the number of vectors added to the index");
  CERTEX_EXPECTS(sp.batch_size >= 1, "certex: batch_size must be positive");
  CERTEX_EXPECTS(nq >= 0 && nq < (int64_t(1) << 31), "certex: too many queries in one call");
  CERTEX_EXPECTS(!filter.query_labels || has_labels_, "certex: the index has no labels");
  // the filter must cover the rows of this snapshot (the size is read under the reader lock the call holds)
  CERTEX_EXPECTS(filter.words == nullptr || filter.covered_ids >= n,
                 filter.bitmap_cols > 0 ? "certex: the bitmap must hold one row of size() bits per query"
                                        : "certex: the bitset must cover every id of the index");
  if (status_out) { CERTEX_CUDA(cudaMemsetAsync(status_out, 0, sizeof(unsigned long long), res.stream)); }
  P.sp = sp, P.queries = queries, P.nq = nq, P.n = n, P.k = k, P.id_base = id_base;
  P.neighbors = neighbors, P.distances = distances, P.scores_out = scores_out;
  if (nq == 0) { return pending.release(); }
  if (test_mode_ == 4 && nq > test_cap_) { throw OutOfMemory("certex: out of device memory (simulated for a test)"); }

  Scratch& scratch       = P.scratch;
  const int d            = static_cast<int>(dim_);
  const size_t row_bytes = static_cast<size_t>(d) * dtype_size(dtype_);
  P.row_bytes            = row_bytes;
  double* best_s         = scratch.get<double>(static_cast<size_t>(nq) * k);
  int32_t* best_row      = scratch.get<int32_t>(static_cast<size_t>(nq) * k);
  P.best_s = best_s, P.best_row = best_row;

  Admit adm{};
  adm.removed         = removed_;
  adm.bits            = filter.words;
  adm.bitmap_cols     = filter.bitmap_cols;
  adm.row_labels      = filter.query_labels ? labels_ : nullptr;
  adm.query_labels    = filter.query_labels;
  P.adm               = adm;
  // A bitset (one bit per id for all queries) keeps the screen: the anchors it drops are left out of the thresholds and
  // the exact stage applies it to the kept pairs, as the reference does (cpp/src/neighbors/certex/detail/kernels.hpp:
  // 39-62). A bitmap (a row of bits per query) and label searches without a partition score every vector.
  const bool filtered = (filter.words != nullptr && filter.bitmap_cols > 0) || filter.query_labels != nullptr;

  const int stride    = anchor_stride_for(n, k);
  const bool screened = screen_kind_ != 0 && !code_overflow_ && !filtered && stride >= 1 && test_mode_ != 1;

  SearchStats& local = P.local;
  local.queries      = static_cast<unsigned long long>(nq);
  if (filter.query_labels && !filter.words && n_part_ > 0 && test_mode_ != 1) {
    local.survivors = search_by_labels(res, queries, row_bytes, static_cast<int>(nq), k, adm, best_s, best_row, n, &local);
    local.verified  = local.survivors;
  } else if (screened) {
    P.screened           = true;
    const int64_t nq_pad = round_up(nq, kQTile);
    uint8_t* qbuf        = scratch.get<uint8_t>(static_cast<size_t>(nq_pad) * code_pitch_);
    float* shift         = nullptr;
    // the call's counters in one block with the layout of HostCounters: one memset, one copy to the host
    auto* counters         = scratch.get<HostCounters>(1);
    unsigned int* d_count  = counters->count;  // [0] overflowed queries, [1] error code, [2] after the 2nd pass
    auto* d_stats          = counters->stats;
    unsigned int* q_ovf    = &counters->q_ovf;  // a query coordinate that does not fit fp16
    if (stats_sink) {
      CERTEX_CUDA(cudaEventCreate(&P.first));
      CERTEX_CUDA(cudaEventRecord(P.first, res.stream));
    }
    CERTEX_CUDA(cudaMemsetAsync(counters, 0, sizeof(HostCounters), res.stream));
    if (screen_kind_ == 2) {
      shift = scratch.get<float>(static_cast<size_t>(nq));
      CERTEX_CUDA(cudaMemsetAsync(qbuf + static_cast<size_t>(nq) * code_pitch_, 0, static_cast<size_t>(nq_pad - nq) * code_pitch_, res.stream));
      launch_encode_f16_queries(queries, row_bytes, dtype_, d, nq, qbuf, code_pitch_, n1max_, n2max_, emax_, shift, q_ovf, res.stream);
      CERTEX_CUDA(cudaGetLastError());
    } else {
      if (row_bytes != code_pitch_ || nq_pad != nq) {
        CERTEX_CUDA(cudaMemsetAsync(qbuf, 0, static_cast<size_t>(nq_pad) * code_pitch_, res.stream));
      }
      CERTEX_CUDA(cudaMemcpy2DAsync(qbuf, code_pitch_, queries, row_bytes, row_bytes, static_cast<size_t>(nq), cudaMemcpyDeviceToDevice, res.stream));
    }
    int32_t* ovf_list      = scratch.get<int32_t>(static_cast<size_t>(nq));
    int32_t* thr2          = scratch.get<int32_t>(static_cast<size_t>(nq));  // tighter thresholds of the queries in ovf_list
    const int64_t batch = std::min<int64_t>(sp.batch_size, 32768);
    P.qbuf = qbuf, P.shift = shift, P.q_ovf = q_ovf, P.ovf_list = ovf_list, P.thr2 = thr2, P.d_count = d_count;
    P.d_stats = d_stats, P.batch = batch;
    for (int64_t q0 = 0; q0 < nq; q0 += batch) {
      const int nb = static_cast<int>(std::min<int64_t>(batch, nq - q0));
      search_screened(res, qbuf, shift, queries, row_bytes, static_cast<int>(q0), nb, k, best_s, best_row, ovf_list, d_count,
                      d_stats, reinterpret_cast<int*>(d_count + 1), stride, n, thr2, adm, stats_sink ? &P.events : nullptr);
      local.launches += screen_kind_ == 2 ? 7 : 6;  // gather_init, GROUPMAX, kth_largest (+ thresholds), SCREEN, expand, verify
    }
    // The outputs are written now, as if no list had overflowed; the counters follow them to the host and search_end
    // looks at them once the caller has enqueued what it wanted behind the search.
    auto* host = static_cast<HostCounters*>(res.pinned_block(P.slot));
    CERTEX_CUDA(cudaMemcpyAsync(host, counters, sizeof(HostCounters), cudaMemcpyDeviceToHost, res.stream));
    if (status_out) {
      launch_search_status(d_count, q_ovf, status_out, res.stream);
      local.launches += 1;
    }
  } else {
    search_dense(res, queries, row_bytes, nullptr, 0, static_cast<int>(nq), k, adm, best_s, best_row, n);
    local.dense_queries = static_cast<unsigned long long>(nq);
    local.launches += 2;
    local.survivors     = static_cast<unsigned long long>(nq) * static_cast<unsigned long long>(n);
    local.verified      = local.survivors;
  }
  launch_finish(best_s, best_row, id_base, queries, row_bytes, dtype_, d, params_.metric, static_cast<int>(nq), k, neighbors,
                distances, scores_out, res.stream);
  CERTEX_CUDA(cudaGetLastError());
  local.launches += 1;  // finish
  if (P.screened) {
    CERTEX_CUDA(cudaEventCreateWithFlags(&P.ready, P.first ? cudaEventDefault : cudaEventDisableTiming));
    CERTEX_CUDA(cudaEventRecord(P.ready, res.stream));
  }
  return pending.release();
}

void Index::search_retarget(Pending* pending, int64_t* neighbors, float* distances, double* scores_out)
{
  CERTEX_EXPECTS(pending != nullptr, "certex: no search to retarget");
  pending->neighbors = neighbors, pending->distances = distances, pending->scores_out = scores_out;
}

bool Index::search_end(Pending* raw, bool refinish) const
{
  std::unique_ptr<Pending> pending(raw);
  CERTEX_EXPECTS(raw != nullptr, "certex: no search to finish");
  Pending& P          = *pending;
  const Resources& res = *P.res;
  SearchStats& local  = P.local;
  bool changed        = false;
  if (P.screened && P.nq > 0) {
    CERTEX_CUDA(cudaEventSynchronize(P.ready));  // the one host round trip of a search call
    const HostCounters h = *static_cast<const HostCounters*>(res.pinned_block(P.slot));
    if (P.first) {
      float ms = 0;
      cudaEventElapsedTime(&ms, P.first, P.ready);
      local.span_ms += ms;
    }
    auto add_times = [&](size_t per_pass) {
      for (size_t e = 0; e + per_pass - 1 < P.events.size(); e += per_pass) {
        float ms = 0;
        if (per_pass == 4) {
          cudaEventElapsedTime(&ms, P.events[e], P.events[e + 1]);
          local.anchor_ms += ms;
        }
        cudaEventElapsedTime(&ms, P.events[e + per_pass - 2], P.events[e + per_pass - 1]);
        local.screen_ms += ms;
        ++local.screen_passes;
      }
      for (cudaEvent_t e : P.events) { cudaEventDestroy(e); }
      P.events.clear();
    };
    add_times(4);
    CERTEX_EXPECTS(h.count[1] == 0, "certex: the screening pass gave up on a wait (code " + std::to_string(h.count[1]) + ")");
    local.survivors = h.stats[0];
    local.verified  = h.stats[1];
    const int k     = P.k;
    const int64_t n = P.n, nq = P.nq;
    Scratch& scratch = P.scratch;
    if (h.q_ovf) {  // a query coordinate beyond the fp16 range: no threshold of this call is trusted
      search_dense(res, P.queries, P.row_bytes, nullptr, 0, static_cast<int>(nq), k, P.adm, P.best_s, P.best_row, n);
      local.dense_queries = static_cast<unsigned long long>(nq);
      local.launches += 2;
      changed = true;
    } else if (h.count[0] > 0) {
      // Candidate lists that overflowed. Each of those queries got a tighter threshold from the candidates it did list;
      // they are screened once more with it, as a batch of their own. What overflows again is searched without the screen.
      const int n_ovf        = static_cast<int>(h.count[0]);
      const int64_t pad      = round_up(n_ovf, kQTile);
      uint8_t* qcodes2       = scratch.get<uint8_t>(static_cast<size_t>(pad) * code_pitch_);
      uint8_t* queries2      = scratch.get<uint8_t>(static_cast<size_t>(n_ovf) * P.row_bytes);
      float* shift2          = scratch.get<float>(static_cast<size_t>(n_ovf));
      double* best2_s        = scratch.get<double>(static_cast<size_t>(n_ovf) * k);
      int32_t* best2_row     = scratch.get<int32_t>(static_cast<size_t>(n_ovf) * k);
      int32_t* ovf2          = scratch.get<int32_t>(static_cast<size_t>(n_ovf));
      launch_gather_rows(P.qbuf, code_pitch_, P.ovf_list, n_ovf, pad, qcodes2, code_pitch_, code_pitch_, res.stream);
      launch_gather_rows(P.queries, P.row_bytes, P.ovf_list, n_ovf, n_ovf, queries2, P.row_bytes, P.row_bytes, res.stream);
      if (P.shift) { launch_gather_rows(P.shift, 4, P.ovf_list, n_ovf, n_ovf, shift2, 4, 4, res.stream); }
      CERTEX_CUDA(cudaGetLastError());
      for (int b0 = 0; b0 < n_ovf; b0 += static_cast<int>(P.batch)) {
        const int nb = std::min<int>(static_cast<int>(P.batch), n_ovf - b0);
        screen_pass(res, qcodes2 + static_cast<size_t>(b0) * code_pitch_, P.thr2 + b0, queries2, P.row_bytes, b0, nb, k, best2_s,
                    best2_row, ovf2, P.d_count + 2, P.d_stats, reinterpret_cast<int*>(P.d_count + 1), n, nullptr,
                    P.shift ? shift2 : nullptr, P.adm, stats_sink ? &P.events : nullptr);
        local.launches += 3;
      }
      launch_scatter_best(best2_s, best2_row, P.ovf_list, n_ovf, k, P.best_s, P.best_row, res.stream);
      launch_compose(ovf2, P.d_count + 2, n_ovf, P.ovf_list, res.stream);
      CERTEX_CUDA(cudaGetLastError());
      local.launches += 5;
      unsigned int h_count[4]       = {0, 0, 0, 0};
      unsigned long long h_stats[2] = {0, 0};
      CERTEX_CUDA(cudaMemcpyAsync(h_count, P.d_count, sizeof(h_count), cudaMemcpyDeviceToHost, res.stream));
      CERTEX_CUDA(cudaMemcpyAsync(h_stats, P.d_stats, sizeof(h_stats), cudaMemcpyDeviceToHost, res.stream));
      res.sync();
      add_times(2);
      CERTEX_EXPECTS(h_count[1] == 0, "certex: the screening pass gave up on a wait (code " + std::to_string(h_count[1]) + ")");
      local.survivors    = h_stats[0];
      local.verified     = h_stats[1];
      local.rescreened   = static_cast<unsigned long long>(n_ovf);
      if (h_count[2] > 0) {
        search_dense(res, P.queries, P.row_bytes, ovf2, 0, static_cast<int>(h_count[2]), k, P.adm, P.best_s, P.best_row, n);
        local.dense_queries = h_count[2];
        local.launches += 2;
        local.verified += static_cast<unsigned long long>(h_count[2]) * static_cast<unsigned long long>(n);
      }
      changed = true;
    }
    if (changed) {
      launch_finish(P.best_s, P.best_row, P.id_base, P.queries, P.row_bytes, dtype_, static_cast<int>(dim_), params_.metric,
                    static_cast<int>(nq), k, P.neighbors, P.distances, P.scores_out, res.stream);
      CERTEX_CUDA(cudaGetLastError());
      local.launches += 1;
    }
  }
  if (refinish && !changed && P.nq > 0) {
    launch_finish(P.best_s, P.best_row, P.id_base, P.queries, P.row_bytes, dtype_, static_cast<int>(dim_), params_.metric,
                  static_cast<int>(P.nq), P.k, P.neighbors, P.distances, P.scores_out, res.stream);
    CERTEX_CUDA(cudaGetLastError());
    local.launches += 1;
  }
  if (stats_sink && P.nq > 0) {
    stats_sink->launches += local.launches;
    stats_sink->screen_ms += local.screen_ms;
    stats_sink->anchor_ms += local.anchor_ms;
    stats_sink->span_ms += local.span_ms;
    stats_sink->screen_passes += local.screen_passes;
    stats_sink->queries += local.queries;
    stats_sink->survivors += local.survivors;
    stats_sink->verified += local.verified;
    stats_sink->dense_queries += local.dense_queries;
    stats_sink->rescreened += local.rescreened;
    stats_sink->routed_queries += local.routed_queries;
  }
  return changed;
}

void Index::search(const Resources& res, const SearchParams& sp, const void* queries, int64_t nq, int k,
                   int64_t* neighbors, float* distances, double* scores_out, const Filter& filter, int64_t id_base) const
{
  try {
    search_end(search_begin(res, sp, queries, nq, k, neighbors, distances, scores_out, filter, id_base, nullptr));
    return;
  } catch (const OutOfMemory&) {
    // no room for the temporaries of this many queries: the two halves one after the other, recursively
    // (cpp/src/neighbors/certex/certex.cu:1477-1502); a bitmap filter is cut at a whole word of query rows
    if (nq < 2 || (filter.bitmap_cols > 0 && nq < 64)) { throw; }
  }
  int64_t half = nq / 2;
  if (filter.bitmap_cols > 0) { half = half / 32 * 32; }
  const size_t row_bytes = static_cast<size_t>(dim_) * dtype_size(dtype_);
  for (int part = 0; part < 2; ++part) {
    const int64_t q0 = part == 0 ? 0 : half, m = part == 0 ? half : nq - half;
    Filter f = filter;
    if (f.query_labels) { f.query_labels += q0; }
    if (f.bitmap_cols > 0) { f.words += static_cast<size_t>(q0) * static_cast<size_t>(f.bitmap_cols) / 32; }
    search(res, sp, static_cast<const uint8_t*>(queries) + static_cast<size_t>(q0) * row_bytes, m, k,
           neighbors + static_cast<size_t>(q0) * k, distances + static_cast<size_t>(q0) * k,
           scores_out ? scores_out + static_cast<size_t>(q0) * k : nullptr, f, id_base);
  }
}

// -------------------------------------------------------------------------------------------- save / load
namespace {
constexpr uint32_t kFileMagic   = 0x30324243u;  // "CB20"
constexpr uint32_t kFileVersion = 1;

template <typename T>
void put(std::ostream& os, const T& v)
{
  os.write(reinterpret_cast<const char*>(&v), sizeof(T));
}
template <typename T>
T take(std::istream& is)
{
  T v{};
  is.read(reinterpret_cast<char*>(&v), sizeof(T));
  CERTEX_EXPECTS(is.good(), "certex: the index file is truncated");
  return v;
}
}  // namespace

void Index::save(const Resources& res, std::ostream& os) const
{
  std::shared_lock<ReaderGate> lock(rw_);
  put(os, kFileMagic);
  put(os, kFileVersion);
  put<int32_t>(os, params_.metric);
  put<int64_t>(os, dim_);
  put<int32_t>(os, params_.anchor_stride);
  put<int64_t>(os, size_);
  put<int64_t>(os, n_removed_);
  put<int32_t>(os, has_labels_ ? 1 : 0);
  const size_t row_bytes = static_cast<size_t>(dim_) * dtype_size(dtype_);
  std::vector<char> host(static_cast<size_t>(size_) * std::max(row_bytes, sizeof(int32_t)));
  if (size_ > 0) {
    CERTEX_CUDA(cudaMemcpy2DAsync(host.data(), row_bytes, vectors_, pitch_, row_bytes, static_cast<size_t>(size_), cudaMemcpyDefault, res.stream));
    res.sync();
    os.write(host.data(), static_cast<std::streamsize>(static_cast<size_t>(size_) * row_bytes));
    CERTEX_CUDA(cudaMemcpyAsync(host.data(), removed_, static_cast<size_t>(size_), cudaMemcpyDeviceToHost, res.stream));
    res.sync();
    os.write(host.data(), static_cast<std::streamsize>(size_));
    if (has_labels_) {
      CERTEX_CUDA(cudaMemcpyAsync(host.data(), labels_, static_cast<size_t>(size_) * 4, cudaMemcpyDeviceToHost, res.stream));
      res.sync();
      os.write(host.data(), static_cast<std::streamsize>(size_ * 4));
    }
  }
  CERTEX_EXPECTS(os.good(), "certex: cannot write the index file");
}

// An .npy record as RAFT's serialize_scalar / serialize_mdspan write it (the reference's files are a sequence of
// them): "\x93NUMPY", version, header length, a Python dict with 'descr', 'fortran_order' and 'shape', then the data.
namespace {
struct NpyRecord {
  size_t item  = 0;  // bytes per element
  size_t count = 1;  // elements
  char kind    = 0;  // 'i', 'u', 'f', ...
  int ndim     = 0;
  bool fortran = false;
};

NpyRecord npy_header(std::istream& is)
{
  char magic[8];
  is.read(magic, 8);
  CERTEX_EXPECTS(is.good() && std::memcmp(magic, "\x93NUMPY", 6) == 0, "certex: the index file is damaged (no array record)");
  uint32_t len = 0;
  if (magic[6] == 1) {
    len = take<uint16_t>(is);
  } else {
    len = take<uint32_t>(is);
  }
  CERTEX_EXPECTS(len > 0 && len < (1u << 20), "certex: the index file is damaged (array header)");
  std::string text(len, '\0');
  is.read(text.data(), len);
  CERTEX_EXPECTS(is.good(), "certex: the index file is truncated");
  NpyRecord r;
  const size_t at = text.find("'descr'");
  CERTEX_EXPECTS(at != std::string::npos, "certex: the index file is damaged (array type)");
  const size_t q0 = text.find('\'', text.find(':', at));
  const size_t q1 = text.find('\'', q0 + 1);
  CERTEX_EXPECTS(q0 != std::string::npos && q1 != std::string::npos && q1 > q0 + 2, "certex: the index file is damaged (array type)");
  const std::string descr = text.substr(q0 + 1, q1 - q0 - 1);  // e.g. "<i4", "|u1", "<f8"
  CERTEX_EXPECTS(descr[0] != '>', "certex: big-endian index files are not supported");
  r.kind = descr[1];
  r.item = static_cast<size_t>(std::stoul(descr.substr(2)));
  const size_t sh = text.find("'shape'");
  CERTEX_EXPECTS(sh != std::string::npos, "certex: the index file is damaged (array shape)");
  const size_t p0 = text.find('(', sh), p1 = text.find(')', sh);
  CERTEX_EXPECTS(p0 != std::string::npos && p1 != std::string::npos, "certex: the index file is damaged (array shape)");
  size_t c = p0 + 1;
  while (c < p1) {
    while (c < p1 && (text[c] == ' ' || text[c] == ',')) { ++c; }
    if (c >= p1) { break; }
    size_t used = 0;
    r.count *= static_cast<size_t>(std::stoull(text.substr(c, p1 - c), &used));
    c += used;
    ++r.ndim;
  }
  r.fortran = text.find("'fortran_order': True") != std::string::npos;
  return r;
}

template <typename T>
T npy_scalar(std::istream& is)
{
  const NpyRecord r = npy_header(is);
  CERTEX_EXPECTS(r.count == 1 && r.item == sizeof(T), "certex: the index file is damaged (scalar of another type)");
  return take<T>(is);
}

void npy_skip(std::istream& is)
{
  const NpyRecord r = npy_header(is);
  is.ignore(static_cast<std::streamsize>(r.item * r.count));
  CERTEX_EXPECTS(is.good(), "certex: the index file is truncated");
}

void npy_read(std::istream& is, char* dst, size_t bytes)
{
  const NpyRecord r = npy_header(is);
  CERTEX_EXPECTS(r.item * r.count == bytes, "certex: the index file is damaged (array of another size)");
  CERTEX_EXPECTS(r.ndim < 2 || !r.fortran, "certex: column-major arrays in an index file are not supported");
  is.read(dst, static_cast<std::streamsize>(bytes));
  CERTEX_EXPECTS(is.good(), "certex: the index file is truncated");
}
}  // namespace

std::unique_ptr<Index> Index::load(const Resources& res, std::istream& is, int dtype)
{
  if (is.peek() == 0x93) { return load_reference_file(res, is, dtype); }
  CERTEX_EXPECTS(take<uint32_t>(is) == kFileMagic, "certex: not an index file of this library");
  CERTEX_EXPECTS(take<uint32_t>(is) == kFileVersion, "certex: unknown index file version");
  IndexParams p;
  p.metric            = take<int32_t>(is);
  const int64_t dim   = take<int64_t>(is);
  p.anchor_stride     = take<int32_t>(is);
  const int64_t n     = take<int64_t>(is);
  const int64_t n_rem = take<int64_t>(is);
  const bool labeled  = take<int32_t>(is) != 0;
  return from_blocks(res, p, dtype, dim, n, n_rem, labeled, [&](char* dst, size_t bytes) {
    is.read(dst, static_cast<std::streamsize>(bytes));
    CERTEX_EXPECTS(is.good(), "certex: the index file is truncated");
  });
}

// A file written by the reference's serialize (cpp/src/neighbors/certex/certex_serialize.cu:40-132, format "CERX"
// version 1, read back at 135-240). Of its records the engine needs the vectors, the removal flags and the labels;
// the projection, the certificate rows and the anchors are the reference's screening data and are skipped (this
// engine screens with its own codes, made from the vectors on load).
std::unique_ptr<Index> Index::load_reference_file(const Resources& res, std::istream& is, int dtype)
{
  CERTEX_EXPECTS(npy_scalar<int32_t>(is) == 0x43455258, "certex: not a CertEx index file");
  CERTEX_EXPECTS(npy_scalar<int32_t>(is) == 1, "certex: unsupported CertEx serialization version");
  IndexParams p;
  const int metric = npy_scalar<int32_t>(is);  // cuvs::distance::DistanceType
  CERTEX_EXPECTS(metric == 0 || metric == 2 || metric == 6, "certex: the file's metric is not L2Expanded, InnerProduct or CosineExpanded");
  p.metric            = metric == 0 ? kL2 : metric == 6 ? kIP : kCos;
  const int64_t dim   = npy_scalar<int64_t>(is);
  p.width             = npy_scalar<int32_t>(is);
  p.anchor_stride     = npy_scalar<int32_t>(is);
  p.host_vectors      = npy_scalar<int32_t>(is) != 0;
  const int64_t n     = npy_scalar<int64_t>(is);
  const int64_t n_rem = npy_scalar<int64_t>(is);
  const bool labeled  = npy_scalar<int32_t>(is) != 0;
  p.int8_rows         = npy_scalar<int32_t>(is) != 0;
  for (int i = 0; i < 6; ++i) { (void)npy_scalar<double>(is); }  // alpha and the five certificate maxima
  npy_skip(is);  // center
  npy_skip(is);  // basis
  if (p.int8_rows) {
    (void)npy_scalar<double>(is);  // largest lifted squared norm
    npy_skip(is);                  // int8 codes
    npy_skip(is);                  // their scalars
  } else {
    npy_skip(is);  // fp16 certificate rows
  }
  npy_skip(is);  // anchor rows
  npy_skip(is);  // anchor vectors
  auto idx = from_blocks(res, p, dtype, dim, n, n_rem, labeled, [&](char* dst, size_t bytes) { npy_read(is, dst, bytes); });
  // k-means lists come last; with lists the reference keeps its rows in list order, which is not read here
  CERTEX_EXPECTS(npy_scalar<int32_t>(is) == 0, "certex: index files with k-means lists are not supported");
  return idx;
}

// The index of n vectors from three blocks in this order: the vectors [n, dim] dense, the removal flags [n] bytes,
// and (labeled) the labels [n] int32.
std::unique_ptr<Index> Index::from_blocks(const Resources& res, const IndexParams& p, int dtype, int64_t dim, int64_t n,
                                          int64_t n_rem, bool labeled, const std::function<void(char*, size_t)>& next_block)
{
  CERTEX_EXPECTS(n >= 0 && n_rem >= 0 && n_rem <= n, "certex: the index file is damaged (sizes)");
  auto idx = std::make_unique<Index>(res, p, dtype, dim);
  if (n > 0) {
    const size_t row_bytes = static_cast<size_t>(dim) * dtype_size(dtype);
    std::vector<char> host(static_cast<size_t>(n) * std::max(row_bytes, sizeof(int32_t)));
    next_block(host.data(), static_cast<size_t>(n) * row_bytes);
    idx->extend(res, host.data(), n, true);
    next_block(host.data(), static_cast<size_t>(n));
    CERTEX_CUDA(cudaMemcpyAsync(idx->removed_, host.data(), static_cast<size_t>(n), cudaMemcpyHostToDevice, res.stream));
    res.sync();
    idx->n_removed_ = n_rem;
    if (idx->screen_kind_ && n_rem > 0) {  // removed rows must never pass the screen
      Scratch scratch(res.stream);
      int64_t* ids     = scratch.get<int64_t>(static_cast<size_t>(n));
      auto* counter    = scratch.get<unsigned long long>(1);
      std::vector<int64_t> gone;
      for (int64_t i = 0; i < n; ++i) {
        if (host[static_cast<size_t>(i)]) { gone.push_back(i); }
      }
      CERTEX_CUDA(cudaMemcpyAsync(ids, gone.data(), gone.size() * 8, cudaMemcpyHostToDevice, res.stream));
      CERTEX_CUDA(cudaMemsetAsync(idx->removed_, 0, static_cast<size_t>(n), res.stream));
      CERTEX_CUDA(cudaMemsetAsync(counter, 0, 8, res.stream));
      launch_remove(ids, static_cast<int64_t>(gone.size()), n, idx->removed_, idx->init_, idx->inv_, idx->cmax_,
                    idx->screen_kind_ == 2, counter, res.stream);
      CERTEX_CUDA(cudaGetLastError());
      res.sync();
    }
    if (labeled) {
      next_block(host.data(), static_cast<size_t>(n) * 4);
      Scratch scratch(res.stream);
      int32_t* tmp = scratch.get<int32_t>(static_cast<size_t>(n));
      CERTEX_CUDA(cudaMemcpyAsync(tmp, host.data(), static_cast<size_t>(n) * 4, cudaMemcpyHostToDevice, res.stream));
      idx->set_labels(res, tmp, n, 0);
      idx->partition_by_labels(res);  // not stored: remade from the labels
    }
    res.sync();
  }
  return idx;
}

void merge_shards(const Resources& res, const double* scores, const int64_t* ids, int parts, int nq, int k,
                  const void* queries, int dtype, int64_t dim, int metric, int64_t* neighbors, float* distances,
                  double* scores_out, int64_t part_stride)
{
  CERTEX_EXPECTS(parts >= 1 && k >= 1 && k <= 2048, "certex: a merge takes at least one part and k up to 2048");
  Scratch scratch(res.stream);
  double* out_s        = scores_out ? scores_out : scratch.get<double>(static_cast<size_t>(nq) * k);
  const size_t qpitch  = static_cast<size_t>(dim) * dtype_size(dtype);
  const int64_t cells  = static_cast<int64_t>(nq) * k;
  if (part_stride == 0) { part_stride = cells; }
  // One block sorts at most 8192 candidates per query. More parts than that are merged in rounds: groups of
  // floor(8192 / k) lists each give one exact list of k (any of the final k best is among the k best of its group),
  // until one round takes what is left. The order is (score, id) in every round, so the result does not depend on the
  // grouping.
  constexpr int kMaxCandidates = 8192;
  while (static_cast<int64_t>(parts) * k > kMaxCandidates) {
    const int group   = kMaxCandidates / k;  // at least 4
    const int n_next  = (parts + group - 1) / group;
    double* next_s    = scratch.get<double>(static_cast<size_t>(n_next) * cells);
    int64_t* next_id  = scratch.get<int64_t>(static_cast<size_t>(n_next) * cells);
    for (int g = 0; g < n_next; ++g) {
      const int first = g * group, count = std::min(group, parts - first);
      launch_merge(scores + static_cast<size_t>(first) * part_stride, ids + static_cast<size_t>(first) * part_stride, count, nq, k,
                   queries, qpitch, dtype, static_cast<int>(dim), metric, next_id + static_cast<size_t>(g) * cells, nullptr,
                   next_s + static_cast<size_t>(g) * cells, res.stream, part_stride, false);
    }
    CERTEX_CUDA(cudaGetLastError());
    scores = next_s, ids = next_id, parts = n_next, part_stride = cells;
  }
  launch_merge(scores, ids, parts, nq, k, queries, qpitch, dtype, static_cast<int>(dim), metric, neighbors, distances, out_s,
               res.stream, part_stride, true);
  CERTEX_CUDA(cudaGetLastError());
}

int plan_routed_flat(int n_runs, const int32_t* n_query_tiles, const int32_t* n_base_tiles, int panel_tiles, int grid,
                     int max_segs, int32_t* segs_out, int cap_segs, int32_t* n_segs, int32_t* seg_begin)
{
  std::vector<LabelRun> runs(static_cast<size_t>(n_runs));
  std::vector<int> q_tile0(static_cast<size_t>(n_runs));
  int64_t tile = 0, slot = 0;
  for (int r = 0; r < n_runs; ++r) {
    runs[r].queries.assign(static_cast<size_t>(n_query_tiles[r]) * kQTile, 0);
    runs[r].n_in_part = static_cast<int64_t>(n_base_tiles[r]) * kTile;
    runs[r].tile0     = tile;
    q_tile0[r]        = static_cast<int>(slot);
    tile += n_base_tiles[r];
    slot += n_query_tiles[r];
  }
  std::vector<ScreenSeg> segs;
  std::vector<int> col0, begin;
  const size_t done = plan_routed(runs, 0, runs.size(), q_tile0, panel_tiles, grid, max_segs, segs, col0, begin);
  CERTEX_EXPECTS(static_cast<int>(segs.size()) <= cap_segs, "certex: more segments than the output holds");
  for (size_t i = 0; i < segs.size(); ++i) {
    segs_out[5 * i + 0] = segs[i].q_tile0, segs_out[5 * i + 1] = segs[i].n_qtiles;
    segs_out[5 * i + 2] = segs[i].t0, segs_out[5 * i + 3] = segs[i].t1, segs_out[5 * i + 4] = col0[i];
  }
  *n_segs = static_cast<int32_t>(segs.size());
  for (int b = 0; b <= grid; ++b) { seg_begin[b] = begin[static_cast<size_t>(b)]; }
  return static_cast<int>(done);
}

void order_by_label_flat(const int32_t* labels, int64_t n, int32_t* order)
{
  const std::vector<int32_t> lab(labels, labels + n);
  const std::vector<int32_t> got = order_by_label(lab);
  std::memcpy(order, got.data(), got.size() * sizeof(int32_t));
}

int plan_chunked_flat(int nqt, int nt, int panel_tiles, int grid, int chunk_tiles, int32_t* segs_out, int cap_segs,
                      int32_t* seg_begin)
{
  CERTEX_EXPECTS(nqt >= 1 && nt >= 1 && panel_tiles >= 1 && grid >= 1, "certex: sizes must be positive");
  const ChunkedPlan plan = plan_chunked(nqt, nt, panel_tiles, grid, chunk_tiles);
  CERTEX_EXPECTS(static_cast<int>(plan.segs.size()) <= cap_segs, "certex: more segments than the output holds");
  std::memcpy(segs_out, plan.segs.data(), plan.segs.size() * sizeof(ScreenSeg));
  for (int b = 0; b <= grid; ++b) { seg_begin[b] = plan.begin[static_cast<size_t>(b)]; }
  return plan.begin.back();
}

void plan_segments_flat(int nqt, int nt, int panel_tiles, int grid, int32_t* out)
{
  CERTEX_EXPECTS(nqt >= 1 && nt >= 1 && panel_tiles >= 1 && grid >= 1, "certex: sizes must be positive");
  const auto segs = plan_segments(nqt, nt, panel_tiles, grid);
  std::memcpy(out, segs.data(), segs.size() * sizeof(ScreenSeg));
}

void screen_raw(const Resources& res, const void* q_codes, int64_t nq, const void* x_codes, int64_t n, int64_t code_len,
                int code_kind, const int32_t* init, int mode, const int32_t* thr, int32_t* gmax, int64_t ld,
                uint32_t* cnt, int32_t* cand, uint32_t cap, float* elapsed_ms)
{
  const bool is_signed = code_kind == 1, f16 = code_kind == 2;
  Scratch scratch(res.stream);
  const int kb            = static_cast<int>(code_len / 128);
  const ScreenShape shape = shape_for(kb);
  const int grid          = res.sm_count;
  const int nqt           = static_cast<int>((nq + kQTile - 1) / kQTile);
  const int nt            = static_cast<int>((n + kTile - 1) / kTile);
  const ChunkedPlan plan  = plan_chunked(nqt, nt, shape.panel_tiles, grid, chunk_tiles_for(static_cast<size_t>(code_len)));
  ScreenSeg* d_segs       = scratch.get<ScreenSeg>(plan.segs.size());
  int* d_seg_begin        = scratch.get<int>(plan.begin.size());
  int* err                = scratch.get<int>(1);
  CERTEX_CUDA(cudaMemcpyAsync(d_segs, plan.segs.data(), plan.segs.size() * sizeof(ScreenSeg), cudaMemcpyHostToDevice, res.stream));
  CERTEX_CUDA(cudaMemcpyAsync(d_seg_begin, plan.begin.data(), plan.begin.size() * sizeof(int), cudaMemcpyHostToDevice, res.stream));
  CERTEX_CUDA(cudaMemsetAsync(err, 0, sizeof(int), res.stream));
  const CUtensorMap tm_q = make_code_map(q_codes, code_len, static_cast<uint64_t>(round_up(nq, kQTile)), code_len, kQueryTile);
  CUtensorMap tm_x = make_code_map(x_codes, code_len, static_cast<uint64_t>(n), code_len, kBaseTile);
  if (mode == kModeGroupBound) {
    // chains of 16 consecutive rows, tiles of 256 consecutive rows (padded), through the 4-D map
    uint8_t* x_pad = scratch.get<uint8_t>(static_cast<size_t>(nt) * kTile * code_len);
    CERTEX_CUDA(cudaMemsetAsync(x_pad, 0, static_cast<size_t>(nt) * kTile * code_len, res.stream));
    CERTEX_CUDA(cudaMemcpyAsync(x_pad, x_codes, static_cast<size_t>(n) * code_len, cudaMemcpyDeviceToDevice, res.stream));
    CUtensorMap m;
    const cuuint64_t dims[4]    = {static_cast<cuuint64_t>(code_len), static_cast<cuuint64_t>(kChainRows),
                                   static_cast<cuuint64_t>(kBaseTile / kChainRows), static_cast<cuuint64_t>(nt)};
    const cuuint64_t strides[3] = {static_cast<cuuint64_t>(code_len), static_cast<cuuint64_t>(kChainRows) * code_len,
                                   static_cast<cuuint64_t>(kTile) * code_len};
    const cuuint32_t box[4]     = {128, static_cast<cuuint32_t>(kChainRows), static_cast<cuuint32_t>(kBaseTile / kChainRows), 1};
    const cuuint32_t estr[4]    = {1, 1, 1, 1};
    const CUresult r = encode_tiled()(&m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, x_pad, dims, strides, box, estr,
                                      CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                      CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    CERTEX_EXPECTS(r == CUDA_SUCCESS, "certex: cuTensorMapEncodeTiled failed (" + std::to_string(int(r)) + ")");
    tm_x = m;
  }
  if (mode == kModeGroupMax) {
    // group maxima over consecutive rows: the pass reads whole tiles through the 3-D map, so the rows are padded
    uint8_t* x_pad = scratch.get<uint8_t>(static_cast<size_t>(nt) * kTile * code_len);
    CERTEX_CUDA(cudaMemsetAsync(x_pad, 0, static_cast<size_t>(nt) * kTile * code_len, res.stream));
    CERTEX_CUDA(cudaMemcpyAsync(x_pad, x_codes, static_cast<size_t>(n) * code_len, cudaMemcpyDeviceToDevice, res.stream));
    tm_x = make_tile_map(x_pad, code_len, code_len, static_cast<uint64_t>(kTile) * code_len, static_cast<uint64_t>(nt));
  }
  // init arrives for n rounded up to 64 rows; the pass reads whole base tiles, and chain maxima
  const int64_t n_in  = round_up(n, kGroupRows);
  const int64_t n_pad = static_cast<int64_t>(nt) * kTile;
  int32_t* init_pad   = scratch.get<int32_t>(static_cast<size_t>(n_pad));
  int32_t* cmax       = scratch.get<int32_t>(static_cast<size_t>(n_pad / kChainRows));
  launch_fill_i32(init_pad, n_pad, f16 ? static_cast<int32_t>(0xff800000u) : kNeverInit, res.stream);
  CERTEX_CUDA(cudaMemcpyAsync(init_pad, init, static_cast<size_t>(n_in) * 4, cudaMemcpyDeviceToDevice, res.stream));
  if (mode == kModeGroupBound) {  // the chained threshold pass takes the chains' minima
    launch_gather_chain_min(init_pad, 1, kChainRows, kTile, nt, cmax, f16, res.stream);
  } else {
    launch_chain_max(init_pad, 0, n_pad / kChainRows, cmax, f16, res.stream);
  }
  CERTEX_CUDA(cudaGetLastError());
  const unsigned long long rec_cap = std::max<unsigned long long>(1ull << 20, static_cast<unsigned long long>(nq) * 1024ull);
  uint64_t* rec   = scratch.get<uint64_t>(static_cast<size_t>(rec_cap));
  auto* rec_count = scratch.get<unsigned long long>(1);
  CERTEX_CUDA(cudaMemsetAsync(rec_count, 0, sizeof(unsigned long long), res.stream));
  ScreenArgs a{};
  a.init        = init_pad;
  a.cmax        = cmax;
  a.thr         = thr;
  a.gmax        = gmax;
  a.ld_gmax     = ld;
  a.rec         = rec;
  a.rec_count   = rec_count;
  a.rec_cap     = rec_cap;
  a.nq          = static_cast<int>(nq);
  a.kb          = kb;
  a.panel_tiles = shape.panel_tiles;
  a.n_stages    = shape.n_stages;
  a.mode        = mode;
  a.wide        = kb > 2 ? 1 : 0;
  a.f16         = f16 ? 1 : 0;
  a.q_signed    = is_signed ? 1u : 0u;
  a.x_signed    = a.q_signed;
  a.segs        = d_segs;
  a.seg_begin   = d_seg_begin;
  a.err         = err;
  cudaEvent_t e0, e1;
  CERTEX_CUDA(cudaEventCreate(&e0));
  CERTEX_CUDA(cudaEventCreate(&e1));
  CERTEX_CUDA(cudaEventRecord(e0, res.stream));
  const cudaError_t le = screen_i8_launch(tm_q, tm_x, a, grid, res.stream);
  CERTEX_CUDA(cudaEventRecord(e1, res.stream));
  if (mode == kModeScreen && le == cudaSuccess) {
    launch_expand_records(rec, rec_count, rec_cap, n, nullptr, cnt, cand, cap, res.sm_count, res.stream);
  }
  int h_err                  = 0;
  unsigned long long h_count = 0;
  CERTEX_CUDA(cudaMemcpyAsync(&h_err, err, sizeof(int), cudaMemcpyDeviceToHost, res.stream));
  CERTEX_CUDA(cudaMemcpyAsync(&h_count, rec_count, sizeof(h_count), cudaMemcpyDeviceToHost, res.stream));
  const cudaError_t se = cudaStreamSynchronize(res.stream);
  float ms             = 0;
  if (se == cudaSuccess) { cudaEventElapsedTime(&ms, e0, e1); }
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  CERTEX_CUDA(le);
  CERTEX_CUDA(se);
  CERTEX_EXPECTS(h_err == 0, "certex: the screening pass gave up on a wait (code " + std::to_string(h_err) + ")");
  CERTEX_EXPECTS(h_count <= rec_cap, "certex: the survivor record buffer overflowed");
  if (elapsed_ms) { *elapsed_ms = ms; }
}

}  // namespace certex_b200
