/*
 * C ABI of libcertex_b200: a B200 (sm_100a) exact k-nearest-neighbour engine that drops in behind the C API of
 * hpdic/libcertex. Every `cuvsCertex*` entry point below has the name, argument list and error behaviour of the
 * reference's c/include/cuvs/neighbors/certex.h (file:line given per function), so a program written against that
 * header links against this library unchanged.
 *
 * The reference header pulls its basic types from cuVS (<cuvs/core/c_api.h>, <cuvs/distance/distance.h>,
 * <cuvs/neighbors/common.h>) and DLPack (<dlpack/dlpack.h>). cuVS is not a dependency of this library, so the few
 * cuVS C types and functions the certex API needs are declared here with the same names, values and meaning; the
 * DLPack structures are declared here too (public DLPack v1.0 ABI) unless <dlpack/dlpack.h> was included first.
 *
 * Conventions (as in the reference, c/src/core/interop.hpp:86-131, c/src/core/exceptions.hpp:17-33):
 *  - every function returns CUVS_SUCCESS or CUVS_ERROR; after an error cuvsGetLastErrorText() gives the message of
 *    the calling thread; no C++ exception crosses this boundary;
 *  - tensors are borrowed for the duration of the call (the deleter is never invoked), must be dense row-major
 *    (strides NULL or matching), lanes == 1, and byte_offset is honoured; outputs are allocated by the caller;
 *  - all device work runs on the stream of the cuvsResources_t handle; searches return after their last kernel is
 *    enqueued (cuvsStreamSync to wait).
 */
#ifndef CERTEX_B200_H_
#define CERTEX_B200_H_

#include <stdbool.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define CERTEX_B200_EXPORT __attribute__((visibility("default")))

/* ------------------------------------------------------------------------------------------------ DLPack v1.0 ABI */
#ifndef DLPACK_DLPACK_H_
#define DLPACK_DLPACK_H_
typedef enum {
  kDLCPU         = 1,
  kDLCUDA        = 2,
  kDLCUDAHost    = 3,
  kDLCUDAManaged = 13
} DLDeviceType;

typedef struct {
  DLDeviceType device_type;
  int32_t device_id;
} DLDevice;

typedef enum {
  kDLInt    = 0U,
  kDLUInt   = 1U,
  kDLFloat  = 2U,
  kDLBfloat = 4U
} DLDataTypeCode;

typedef struct {
  uint8_t code;
  uint8_t bits;
  uint16_t lanes;
} DLDataType;

typedef struct {
  void* data;
  DLDevice device;
  int32_t ndim;
  DLDataType dtype;
  int64_t* shape;
  int64_t* strides;
  uint64_t byte_offset;
} DLTensor;

typedef struct DLManagedTensor {
  DLTensor dl_tensor;
  void* manager_ctx;
  void (*deleter)(struct DLManagedTensor* self);
} DLManagedTensor;
#endif /* DLPACK_DLPACK_H_ */

/* ------------------------------------------------------------------------------------- cuVS C types used by certex */
/** <cuvs/core/c_api.h>: status of every call. */
typedef enum { CUVS_ERROR = 0, CUVS_SUCCESS = 1 } cuvsError_t;

/** <cuvs/core/c_api.h>: opaque handle holding the device and the stream of a caller. */
typedef uintptr_t cuvsResources_t;

/** <cuvs/distance/distance.h>: the three metrics certex accepts keep their cuVS values. */
typedef enum { L2Expanded = 0, CosineExpanded = 2, InnerProduct = 6 } cuvsDistanceType;

/** <cuvs/neighbors/common.h>: filter kinds; `addr` of a BITSET / BITMAP filter is a DLManagedTensor* of uint32
 *  device words (bit j of word i is entry 32 i + j; a set bit keeps the vector). */
enum cuvsFilterType { NO_FILTER = 0, BITSET = 1, BITMAP = 2 };
typedef struct {
  uintptr_t addr;
  enum cuvsFilterType type;
} cuvsFilter;

CERTEX_B200_EXPORT cuvsError_t cuvsResourcesCreate(cuvsResources_t* res);
CERTEX_B200_EXPORT cuvsError_t cuvsResourcesDestroy(cuvsResources_t res);
/** Stream type is cudaStream_t, passed as void* so that this header needs no CUDA include. */
CERTEX_B200_EXPORT cuvsError_t cuvsStreamSet(cuvsResources_t res, void* stream);
CERTEX_B200_EXPORT cuvsError_t cuvsStreamGet(cuvsResources_t res, void** stream);
CERTEX_B200_EXPORT cuvsError_t cuvsStreamSync(cuvsResources_t res);
CERTEX_B200_EXPORT const char* cuvsGetLastErrorText(void);
CERTEX_B200_EXPORT void cuvsSetLastErrorText(const char* text);

/* --------------------------------------------------------------------------------------------- parameters */
/** certex.h:30-49. Every setting returns the same exact neighbours. `width`, `variance`, `pca_sample`, `n_lists`,
 *  `local_projections` and `int8_rows` tune the reference's projected screening rows; this engine has no projection
 *  (8-bit vectors are screened by their exact integer Gram product) and accepts them without effect.
 *  `host_vectors` (certex.hpp:56-61) keeps the vectors in page-locked host memory instead of device memory, which about
 *  halves the device memory of an 8-bit index: the screen's code rows stay on the device and the exact stage reads the
 *  candidates it scores from the host in place (for 8-bit indexes from the code rows, which are the vectors, so a
 *  screened search does not touch host memory; searches that score every vector -- per-query bitmaps, unpartitioned
 *  labels, tiny sets -- read them all over the host link and are slow). Results are the same either way. */
struct cuvsCertexIndexParams {
  cuvsDistanceType metric;
  int32_t width;
  double variance;
  int32_t anchor_stride;
  int64_t pca_sample;
  bool host_vectors;
  int32_t n_lists;
  bool local_projections;
  bool int8_rows;
};
typedef struct cuvsCertexIndexParams* cuvsCertexIndexParams_t;

/** certex.h:54 */
CERTEX_B200_EXPORT cuvsError_t cuvsCertexIndexParamsCreate(cuvsCertexIndexParams_t* params);
/** certex.h:57 */
CERTEX_B200_EXPORT cuvsError_t cuvsCertexIndexParamsDestroy(cuvsCertexIndexParams_t params);

/** certex.h:69-76. `batch_size` queries share one pass over the stored rows. `anchors` and `probe_lists` belong to
 *  stages this engine does not have and are accepted without effect. */
struct cuvsCertexSearchParams {
  int32_t anchors;
  int32_t batch_size;
  int32_t probe_lists;
};
typedef struct cuvsCertexSearchParams* cuvsCertexSearchParams_t;

/** certex.h:81 */
CERTEX_B200_EXPORT cuvsError_t cuvsCertexSearchParamsCreate(cuvsCertexSearchParams_t* params);
/** certex.h:84 */
CERTEX_B200_EXPORT cuvsError_t cuvsCertexSearchParamsDestroy(cuvsCertexSearchParams_t params);

/* --------------------------------------------------------------------------------------------- index */
/** certex.h:96-101: an opaque index of float32, float16, int8 or uint8 vectors. */
typedef struct {
  uintptr_t addr;
  DLDataType dtype;
} cuvsCertexIndex;
typedef cuvsCertexIndex* cuvsCertexIndex_t;

/** certex.h:104 */
CERTEX_B200_EXPORT cuvsError_t cuvsCertexIndexCreate(cuvsCertexIndex_t* index);
/** certex.h:107 */
CERTEX_B200_EXPORT cuvsError_t cuvsCertexIndexDestroy(cuvsCertexIndex_t index);
/** certex.h:110: vectors added so far, removed ones included. */
CERTEX_B200_EXPORT cuvsError_t cuvsCertexIndexGetSize(cuvsCertexIndex_t index, int64_t* size);
/** certex.h:113 */
CERTEX_B200_EXPORT cuvsError_t cuvsCertexIndexGetDim(cuvsCertexIndex_t index, int64_t* dim);

/** certex.h:139-142: build from a dataset [n_rows, dim] in device (kDLCUDA, kDLCUDAManaged) or host (kDLCPU,
 *  kDLCUDAHost) memory; the handle must be empty. */
CERTEX_B200_EXPORT cuvsError_t cuvsCertexBuild(cuvsResources_t res, cuvsCertexIndexParams_t params,
                                               DLManagedTensor* dataset, cuvsCertexIndex_t index);
/** certex.h:146-148: append vectors [n, dim]; they receive the next consecutive ids. */
CERTEX_B200_EXPORT cuvsError_t cuvsCertexExtend(cuvsResources_t res, DLManagedTensor* new_vectors,
                                                cuvsCertexIndex_t index);
/** certex.h:151-153: remove by id (int64 device vector); ids are never reused. */
CERTEX_B200_EXPORT cuvsError_t cuvsCertexRemove(cuvsResources_t res, DLManagedTensor* ids, cuvsCertexIndex_t index);
/** certex.h:157-160: labels (int32 device vector) of the vectors first, first + 1, ... */
CERTEX_B200_EXPORT cuvsError_t cuvsCertexSetLabels(cuvsResources_t res, DLManagedTensor* labels, int64_t first,
                                                   cuvsCertexIndex_t index);
/** certex.h:164: groups the ids by label and, when the index has a tensor-core screen, copies the code rows in label
 *  order, so that searches by label screen and score only the rows of the query's label. Speed only: results are the
 *  same with or without it. Vectors added later are found too (scored densely) until the next call. */
CERTEX_B200_EXPORT cuvsError_t cuvsCertexPartitionByLabels(cuvsResources_t res, cuvsCertexIndex_t index);

/** certex.h:184-190: exact k nearest neighbours, k = neighbors.shape[1]. queries [nq, dim] (device, index dtype),
 *  neighbors int64 [nq, k], distances float32 [nq, k] (device): squared Euclidean distances ascending, inner products
 *  descending, cosine distances (1 - cos) ascending. Entries beyond the admitted vectors: id -1, distance +inf
 *  (-inf for inner products). Ties between equal exact scores resolve to the smaller id. */
CERTEX_B200_EXPORT cuvsError_t cuvsCertexSearch(cuvsResources_t res, cuvsCertexSearchParams_t params,
                                                cuvsCertexIndex_t index, DLManagedTensor* queries,
                                                DLManagedTensor* neighbors, DLManagedTensor* distances,
                                                cuvsFilter filter);
/** certex.h:196-202: neighbours among the vectors whose label equals the query's (int32 device vector [nq]). */
CERTEX_B200_EXPORT cuvsError_t cuvsCertexSearchWithLabels(cuvsResources_t res, cuvsCertexSearchParams_t params,
                                                          cuvsCertexIndex_t index, DLManagedTensor* queries,
                                                          DLManagedTensor* query_labels, DLManagedTensor* neighbors,
                                                          DLManagedTensor* distances);
/** certex.h:214-216: save the index with its vectors. The file starts with the reference's 4-byte NumPy dtype
 *  prefix; the rest is this library's own layout (the reference cannot read it). */
CERTEX_B200_EXPORT cuvsError_t cuvsCertexSerialize(cuvsResources_t res, const char* filename, cuvsCertexIndex_t index);
/** certex.h:220-222: load into an empty handle; the vector type comes from the file. Reads this library's files and
 *  files in the reference's layout (cpp/src/neighbors/certex/certex_serialize.cu:40-132, without k-means lists): their
 *  vectors, removal flags and labels; the screening data is made anew. */
CERTEX_B200_EXPORT cuvsError_t cuvsCertexDeserialize(cuvsResources_t res, const char* filename,
                                                     cuvsCertexIndex_t index);

/* --------------------------------------------------------------------------- additions without a certex.h counterpart */
/**
 * Search that also returns the exact fp64 scores the ranking used and shifts ids by `id_base`. The reference returns
 * float32 distances only (`finish`, cpp/src/neighbors/certex/certex.cu:224-250); its internal `best_score` array is
 * what `scores` exposes: squared distance (L2), |q|^2 - 2<q,x> (inner product), 2 - 2cos (cosine), +inf where the id
 * is -1. `scores` (float64 [nq, k], device) may be NULL. `query_labels` may be NULL. `id_base` is the global id of the
 * index's first vector when the index is one row shard of a larger set
 * (first_id of cpp/src/neighbors/certex/certex_shards.cu:70-75).
 */
CERTEX_B200_EXPORT cuvsError_t certexB200SearchEx(cuvsResources_t res, cuvsCertexSearchParams_t params,
                                                  cuvsCertexIndex_t index, DLManagedTensor* queries,
                                                  DLManagedTensor* query_labels, DLManagedTensor* neighbors,
                                                  DLManagedTensor* distances, DLManagedTensor* scores,
                                                  cuvsFilter filter, int64_t id_base);

/**
 * Device merge of per-shard answers, the step the reference performs on the host in `search_sharded`
 * (cpp/src/neighbors/certex/certex_shards.cu:144-166): part_scores float64 [parts, nq, k] and part_ids int64
 * [parts, nq, k] (id -1 = missing) are merged per query by (score, id); neighbors / distances / scores as in
 * certexB200SearchEx (scores may be NULL). `queries` [nq, dim] is needed for inner-product distances.
 */
CERTEX_B200_EXPORT cuvsError_t certexB200MergeShards(cuvsResources_t res, cuvsDistanceType metric,
                                                     DLManagedTensor* queries, DLManagedTensor* part_scores,
                                                     DLManagedTensor* part_ids, DLManagedTensor* neighbors,
                                                     DLManagedTensor* distances, DLManagedTensor* scores);

/** Read-only facts of an index, the accessors of cuvs::neighbors::certex::index<T>
 *  (cpp/include/cuvs/neighbors/certex.hpp:131-457) that the reference's Python binding reads. */
typedef struct {
  int64_t size;
  int64_t dim;
  int64_t capacity;
  int64_t n_removed;
  int32_t metric;        /* cuvsDistanceType */
  int32_t anchor_stride;
  int32_t has_labels;
  int32_t integer_screen; /* 1: searches without a filter use the tensor-core screen */
  int64_t row_pitch_bytes;
  int64_t n_partitioned;
} certexB200IndexInfo;
CERTEX_B200_EXPORT cuvsError_t certexB200IndexGetInfo(cuvsCertexIndex_t index, certexB200IndexInfo* info);

/** index<T>::reserve (cpp/src/neighbors/certex/certex.cu:1879-1936): preallocate rows for later additions. */
CERTEX_B200_EXPORT cuvsError_t certexB200IndexReserve(cuvsResources_t res, cuvsCertexIndex_t index, int64_t n_rows);

/** Counters of the calling thread's searches between Begin and End: the reference's search_stats
 *  (cpp/src/neighbors/certex/detail/kernels.hpp:256-263). out[0..3] = queries, survivors of the screen, exact scores
 *  computed, queries answered by the dense (unscreened) path; out[4] = kernels launched; out[5], out[6] = device
 *  time in microseconds of the screen passes and of the anchor (group-maximum) passes, measured with CUDA events on
 *  the launching stream; out[7] = number of screen passes; out[8] = queries whose candidate list overflowed and that
 *  were screened a second time with a tighter threshold; out[9] = query slots of searches by label that went through
 *  the routed screen (a label's queries fill whole tiles of 128 slots); out[10] = device time in microseconds from
 *  the first to the last operation the screened searches enqueued; out[11..15] = 0, reserved. */
CERTEX_B200_EXPORT cuvsError_t certexB200StatsBegin(void);
CERTEX_B200_EXPORT cuvsError_t certexB200StatsEnd(uint64_t out[16]);

/** Exchange of thresholds between the row shards of one set: the reference's threshold hooks
 *  (cpp/src/neighbors/certex/detail/kernels.hpp:271-277) and the first round of its sharded search
 *  (cpp/src/neighbors/certex/certex_shards.cu:136-141). While a hook is set for the calling thread, every unfiltered
 *  screened search calls it once per batch of queries, between the anchor pass and the screen: keys [n] (device) are
 *  monotone int32 images of scores that k rows of this shard certainly reach for the n queries of the batch (larger =
 *  tighter). The hook may raise a key to what another shard of the same set certainly reaches, e.g. take the maximum
 *  over the shards with an all-reduce; it must enqueue its work on `stream`. certexB200IndexWillScreen tells whether a
 *  search for k neighbours will call it (every shard must agree before a collective is used). NULL removes the hook. */
typedef void (*certexB200ThresholdHook)(void* ctx, int32_t* keys, int64_t n, void* stream /* cudaStream_t */);
CERTEX_B200_EXPORT cuvsError_t certexB200SetThresholdHook(certexB200ThresholdHook hook, void* ctx);
CERTEX_B200_EXPORT cuvsError_t certexB200IndexWillScreen(cuvsCertexIndex_t index, int32_t k, int32_t* out);

/** Test hook: mode 0 automatic, 1 always the dense path, 2 screen with candidate lists of `cap` entries per query
 *  (small values exercise the overflow fallback), 3 searches by label score their label's rows densely instead of
 *  screening them, 4 a search call of more than `cap` queries fails the way an allocation failure would (on the host,
 *  no memory is exhausted), which exercises the halving of the call, 5 the threshold stage of plain searches computes
 *  exact group maxima (the variant that searches with a bitset filter or many removed vectors use) instead of the
 *  chained bound. */
CERTEX_B200_EXPORT cuvsError_t certexB200IndexSetTestMode(cuvsCertexIndex_t index, int32_t mode, int32_t cap);

/**
 * The tensor-core pass alone on caller buffers (device pointers), the seam of the reference's
 * detail/kernels.hpp:290-304 (`screen_int8`) and :125-135 (`anchor_groups`), for kernel-level tests and timing.
 * q_codes [nq_pad, code_len] and x_codes [n, code_len] are uint8 (is_signed = 0) or int8 (1) rows, or rows of float16
 * coordinates (2: code_len bytes = 2 bytes per coordinate; init, thr and the values compared are then float32 bit
 * patterns, the products accumulate in float32, group maxima come back as monotone int32 keys of floats and rows that
 * must never pass have init = -inf), code_len a multiple of 128 up to 4096,
 * nq_pad = nq rounded up to 128 with zero rows; init [n rounded up to 64] in row order (the per-row term added to the
 * product: -floor(|x|^2 / 2) for L2, -2^30 for rows that must never pass).
 * mode 0 (screen): keep iff init[x] + <q, x> >= thr[q]; cnt [nq] must be zeroed by the caller; cand [nq, cap].
 * mode 1 (group maxima): gmax [nq, ld] receives the maximum over every 64 rows of x, 4 * ceil(n / 256) groups.
 * mode 2 (rate probe): the same loads and MMAs with no epilogue and no output.
 * mode 3 (chained group bound): gmax [nq, ld] receives, per 64 rows, the maximum over their four chains of 16 rows of
 *   (largest <q, x> of the chain + smallest init of the chain): a value some row of the group reaches, at most the
 *   group maximum of mode 1; what the threshold stage of a plain search runs.
 * Returns after the pass has finished; a pass that gave up on a wait is an error.
 */
CERTEX_B200_EXPORT cuvsError_t certexB200ScreenRaw(cuvsResources_t res, const void* q_codes, int64_t nq,
                                                   const void* x_codes, int64_t n, int64_t code_len, int32_t is_signed,
                                                   const int32_t* init, int32_t mode, const int32_t* thr,
                                                   int32_t* gmax, int64_t ld, uint32_t* cnt, int32_t* cand,
                                                   uint32_t cap, float* elapsed_ms);

/** Profiling aid of the tensor-core pass, available in a trace build of the library only (`make trace` in csrc builds
 *  lib/libcertex_b200_trace.so; the regular library answers CUVS_ERROR): `trace` is a device buffer of units * 12 int64
 *  that CTA 0 of every later pass fills with SM clock stamps of its first `units` accumulator units; NULL switches it
 *  off. Per unit: 0 the MMA-issuing thread starts waiting for the unit's TMEM slot, 1 has it, 2 has issued and
 *  committed the unit's MMAs, 3 the first warp of the epilogue group that reads the unit starts waiting for it, 4 sees
 *  it complete, 5 has its columns in registers, 6 has released the slot, 7 is done with the unit, 8 / 9 = 4 / 5 for
 *  the last warp of that group. Process-wide, not for concurrent use. No counterpart in the reference. */
CERTEX_B200_EXPORT cuvsError_t certexB200ScreenTrace(void* trace, int32_t units);

/** Test hook (host only, no GPU needed): the split of n_query_tiles x n_base_tiles accumulator units over `grid` CTAs
 *  that the tensor-core pass uses. out receives grid * 4 segments of 4 ints (first query tile, query tiles, first base
 *  tile, end base tile); unused segments have end <= first. */
CERTEX_B200_EXPORT cuvsError_t certexB200PlanSegments(int32_t n_query_tiles, int32_t n_base_tiles, int32_t panel_tiles,
                                                      int32_t grid, int32_t* out);

/** Test hook (host only): how a search by labels groups its queries: order [n] = 0 .. n - 1 sorted by labels[i], equal
 *  labels in ascending order. */
CERTEX_B200_EXPORT cuvsError_t certexB200OrderByLabel(const int32_t* labels, int64_t n, int32_t* order);

/** Test hook (host only): the split that searches use, with the base tiles taken in chunks of chunk_tiles (0: one
 *  chunk) so that a chunk's rows stay in L2 while every query panel passes over them. segs receives 4 ints per segment
 *  (as above), *n_segs their number (at most cap_segs), seg_begin [grid + 1] the range of every CTA. */
CERTEX_B200_EXPORT cuvsError_t certexB200PlanChunked(int32_t n_query_tiles, int32_t n_base_tiles, int32_t panel_tiles,
                                                     int32_t grid, int32_t chunk_tiles, int32_t* segs, int32_t cap_segs,
                                                     int32_t* n_segs, int32_t* seg_begin);

/** Test hook (host only): the work split of a routed pass (searches by label). Run r pairs n_query_tiles[r] query
 *  tiles with its own n_base_tiles[r] base tiles; runs follow one another in both directions. segs receives 5 ints
 *  per segment (first query tile, query tiles <= panel_tiles, first base tile, end base tile, first base tile of the
 *  run), *n_segs their number (at most cap_segs), seg_begin [grid + 1] the range of every CTA (at most max_segs
 *  segments each), *runs_done how many runs fit (the rest waits for another pass). */
CERTEX_B200_EXPORT cuvsError_t certexB200PlanRouted(int32_t n_runs, const int32_t* n_query_tiles,
                                                    const int32_t* n_base_tiles, int32_t panel_tiles, int32_t grid,
                                                    int32_t max_segs, int32_t* segs, int32_t cap_segs, int32_t* n_segs,
                                                    int32_t* seg_begin, int32_t* runs_done);

/**
 * Exact search that allocates no device memory. It has no counterpart in the reference, whose searches take their
 * temporaries from a memory pool. It exists for callers that cannot allocate on the GPU at search time: a process in
 * which another allocator has already claimed the device's memory (an inference server that reserves the whole GPU at
 * start-up), or a latency-bound loop that cannot accept the device-wide synchronisation an allocation or a free may
 * cause. The caller passes plain device pointers to its own buffers: vectors [n_rows, dim] and queries
 * [n_queries, dim] of `dtype` (dense, 16-byte aligned, dim * sizeof(element) a multiple of 16), neighbors int64
 * [n_queries, k], distances float32 [n_queries, k]; results and conventions are those of cuvsCertexSearch on an index
 * built from the same vectors (every stored vector is scored in fp64, no screening).
 *
 * The temporaries live in one array of CERTEX_B200_STATIC_SCRATCH_BYTES that is part of the library image: every GPU on
 * which the library is used holds it from load to process exit. A call whose temporaries
 * (n_queries * n_rows * 8 bytes for the scores plus the selection lists) exceed it fails with CUVS_ERROR and a message
 * that names both sizes; so does a call with more than 7264 dimensions or 262 140 queries (the limits of one launch of
 * the scoring kernel), before anything is launched. The device that is current must be the one `res` was created on.
 * The first call on a device looks up the array's address on that device, and the first use of each of its three
 * kernels lets the CUDA runtime load that kernel, which may itself allocate or synchronise: make one warm-up call per
 * device at start-up, outside any stream capture. All calls share the array and it keeps
 * the previous call's contents: every value a call reads it has written itself, so no clearing is needed, but two
 * calls that overlap on the GPU (different streams, or different host threads without ordering between their
 * streams) race on it. Work is enqueued on the stream of `res`; the call returns without synchronising.
 */
#define CERTEX_B200_STATIC_SCRATCH_BYTES (16u << 20)
CERTEX_B200_EXPORT cuvsError_t certexB200SearchStatic(cuvsResources_t res, cuvsDistanceType metric, DLDataType dtype,
                                                      const void* vectors, int64_t n_rows, const void* queries,
                                                      int64_t n_queries, int64_t dim, int32_t k, int64_t* neighbors,
                                                      float* distances);

/* ------------------------------------------------------------------------------- row shards on the GPUs of one process */
/** An index split into contiguous row shards, one index per device: cuvs::neighbors::certex::sharded_index<T>
 *  (cpp/include/cuvs/neighbors/certex_shards.hpp:39-60). */
typedef struct certexB200Sharded* certexB200ShardedIndex_t;

/** build_sharded (certex_shards.hpp:70-90, cpp/src/neighbors/certex/certex_shards.cu:56-83): `dataset` is a host matrix
 *  [n, dim] of float32, float16, int8 or uint8; shard s is built on devices[s] from the rows
 *  [n s / S, n (s + 1) / S), all shards at the same time on one host thread each. A device may appear more than once.
 *  Of `params` the metric and anchor_stride are used. */
CERTEX_B200_EXPORT cuvsError_t certexB200ShardedBuild(const int32_t* devices, int32_t n_shards,
                                                      cuvsCertexIndexParams_t params, DLManagedTensor* dataset,
                                                      certexB200ShardedIndex_t* index);
CERTEX_B200_EXPORT cuvsError_t certexB200ShardedDestroy(certexB200ShardedIndex_t index);
/** Number of vectors over all shards (sharded_index<T>::size, certex_shards.hpp:51-58). */
CERTEX_B200_EXPORT cuvsError_t certexB200ShardedGetSize(certexB200ShardedIndex_t index, int64_t* size);
/** search on a sharded index (certex_shards.hpp:104-120, certex_shards.cu:85-167): queries [nq, dim], neighbors int64
 *  [nq, k] and distances float32 [nq, k] are HOST matrices. Every shard finds its exact k best on its own device (one
 *  host thread per shard), the lists are merged by (score, global id). Every shard must hold at least k vectors.
 *  Synchronous: the outputs are complete on return. */
CERTEX_B200_EXPORT cuvsError_t certexB200ShardedSearch(cuvsCertexSearchParams_t params, certexB200ShardedIndex_t index,
                                                       DLManagedTensor* queries, DLManagedTensor* neighbors,
                                                       DLManagedTensor* distances);

/** Version string "major.minor.patch". */
/* ------------------------------------------------------------------------------------------------------------------
 * Row shards over several processes, one GPU and one shard each, exchanged over NCCL. The reference's sharded search
 * (cpp/include/cuvs/neighbors/certex_shards.hpp:39-60, cpp/src/neighbors/certex/certex_shards.cu:85-167) keeps its
 * shards in one process and merges on the host; these entry points are the same search for one process per GPU:
 * every rank computes the exact local top-k of all queries, one ncclAllGather moves k (fp64 score, int64 id) pairs per
 * query and rank, and every rank merges by (score, id). NCCL is loaded at run time (the copy already in the process,
 * else libnccl.so.2); the library loads without it.
 *
 * certexB200CommGetUniqueId: one rank fills id (128 bytes, an ncclUniqueId) and the application sends it to the others.
 * certexB200CommInitRank: every rank, with its device current (ncclCommInitRank). certexB200CommAdopt wraps an
 * ncclComm_t that the application made and keeps. certexB200CommDestroy frees the buffers (and a communicator made by
 * InitRank).
 * certexB200DistributedSearch: called by every rank with the same queries (device, [nq, dim]), k, parameters and
 * share_thresholds; `index` is the rank's shard and id_base the global id of its first row; neighbors / distances /
 * scores (scores may be NULL) are device [nq, k] and receive the same merged answer on every rank. Every shard must
 * hold at least k vectors. share_thresholds != 0 adds the reference's first round (certex_shards.cu:136-141), on the
 * stream, once per batch of queries: for k <= 64 one ncclAllGather of every rank's k best threshold candidates per
 * query, of which each rank takes the k-th best (what one index over all rows would screen with); for larger k one
 * ncclAllReduce(max) over the ranks' own thresholds. The call waits for its stream once, at its end.
 * If the local search of a rank fails, every rank returns CUVS_ERROR for the call.
 * certexB200DistributedSearchBegin / End are the same search in two calls, for callers that keep the device busy
 * across searches: Begin enqueues the local search, the exchange and the merge on the resources' stream and returns
 * without waiting; End waits for that search only (not for work enqueued behind it) and, if a candidate list had
 * overflowed on some rank, runs the repair and a second exchange. The outputs are final when End has returned
 * CUVS_SUCCESS. Up to two searches may be between their Begin and End per communicator; they End in the order they
 * Began, every rank makes the same sequence of calls, and queries and outputs stay valid and untouched from Begin to
 * End. A Begin that returned CUVS_ERROR left nothing to End (*pending is NULL).
 */
typedef struct certexB200Comm* certexB200Comm_t;
CERTEX_B200_EXPORT cuvsError_t certexB200CommGetUniqueId(void* id /* 128 bytes */);
CERTEX_B200_EXPORT cuvsError_t certexB200CommInitRank(const void* id, int32_t n_ranks, int32_t rank, certexB200Comm_t* comm);
CERTEX_B200_EXPORT cuvsError_t certexB200CommAdopt(void* nccl_comm /* ncclComm_t */, certexB200Comm_t* comm);
CERTEX_B200_EXPORT cuvsError_t certexB200CommDestroy(certexB200Comm_t comm);
typedef struct certexB200PendingSearch* certexB200PendingSearch_t;
CERTEX_B200_EXPORT cuvsError_t certexB200DistributedSearchBegin(cuvsResources_t res, certexB200Comm_t comm,
                                                                cuvsCertexSearchParams_t params, cuvsCertexIndex_t index,
                                                                DLManagedTensor* queries, DLManagedTensor* neighbors,
                                                                DLManagedTensor* distances, DLManagedTensor* scores,
                                                                int64_t id_base, int32_t share_thresholds,
                                                                certexB200PendingSearch_t* pending);
CERTEX_B200_EXPORT cuvsError_t certexB200DistributedSearchEnd(certexB200PendingSearch_t pending);
CERTEX_B200_EXPORT cuvsError_t certexB200DistributedSearch(cuvsResources_t res, certexB200Comm_t comm,
                                                           cuvsCertexSearchParams_t params, cuvsCertexIndex_t index,
                                                           DLManagedTensor* queries, DLManagedTensor* neighbors,
                                                           DLManagedTensor* distances, DLManagedTensor* scores,
                                                           int64_t id_base, int32_t share_thresholds);

CERTEX_B200_EXPORT const char* certexB200Version(void);

#ifdef __cplusplus
}
#endif

#endif /* CERTEX_B200_H_ */
