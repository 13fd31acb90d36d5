// Integer screening pass on the sm_100a tensor cores.
//
// For 8-bit vectors the Gram product <q, x> is exact in int32, so the lower bound that the screen tests is the exact
// squared distance itself (or the exact inner-product score): nothing is lost to rounding and the verification stage
// only re-derives the survivors' scores in fp64 and breaks ties. The pass replaces the reference's `screen_int8`
// (cpp/src/neighbors/certex/detail/kernels.hpp:290-304, kernel cpp/src/neighbors/certex/detail/screen_int8.cu:99-229,
// an mma.sync kernel) and, in its second mode, the anchor pass `anchor_groups`
// (cpp/src/neighbors/certex/detail/kernels.hpp:125-135).
//
// One accumulator unit is 128 queries (TMEM lanes) x 256 stored rows (TMEM columns), K = 128 bytes per K block; one
// tcgen05.mma instruction covers the whole 128 x 256 unit for 32 bytes of K (N = 256 is what keeps the tensor pipe fed:
// with N = 128 the operand reads from shared memory cap the rate at about 60 % of peak).
//   value[q][x] = <q, x> + e[x]
//   e[x] = -floor(|x|^2 / 2) for L2, 0 for inner product, -2^30 for removed rows and padding
// SCREEN keeps every (q, x) with value >= thr[q]. The stored rows are kept sorted by |x|^2 (per appended batch), so e
// is almost constant over 16 adjacent rows and the epilogue never touches e per element: a thread (one query row, 64
// columns of the unit) takes the maximum of the raw products over each chain of 16 columns (3-input integer max, half
// an instruction per element) and tests  max + cmax[chain] >= thr  with cmax = max of e over the chain. That test
// never rejects a pair that should be kept. Only in a chain that passes it (rare) the columns are looked at one by
// one, still with cmax in place of their own e: what is kept is a superset of the pairs at or above the threshold,
// larger by the few rows whose e is below their chain's maximum, and the exact scores of the verification sort those
// out. The kept columns of a chain form one record (query, chain, 16-bit mask) in the warp's staging buffer in shared
// memory, and a half-full buffer goes to global memory with one atomic add for the whole batch.
// GROUPMAX writes gmax[q][group] = max over 64 anchors of value (exact, e is staged in shared memory with the tile);
// the k-th largest group maximum of a query is its threshold: k distinct stored rows are at least that close. The
// anchors of one tile are spread over the whole sorted set (column c of tile t is anchor c * n_tiles + t), so that the
// anchors of one cluster of similar rows do not share a group.
//
// The same kernel screens float data (F16 = true): the operands are the vectors rounded to fp16, the MMA is
// kind::f16 with fp32 accumulators, the per-row term e[x] = -|x|^2 / 2 and the thresholds are floats. What the fp16
// rounding and the fp32 accumulation can add to or take from <q, x> is bounded per query (Cauchy-Schwarz on the
// rounding residuals, see encode_f16 in kernels.cu) and sits inside thr[q], so the test keeps every pair that the
// exact arithmetic would keep. It replaces the reference's fp16 pass `screen`
// (cpp/src/neighbors/certex/detail/kernels.hpp:101-114; on B200 the mma.sync kernel of detail/screen_sm80.cu).
//
// Rows longer than two K blocks (WIDE = true: fp16 codes of more than 128 dimensions, 8-bit vectors of more than 256)
// do not fit shared memory as a resident query panel. There a stage of the ring holds one K block of up to two query
// tiles and of one base tile (64 KB), the MMAs of both query tiles accumulate over the K blocks into the two TMEM slots,
// and the e values of a tile travel through a small ring of their own.
//
// CTA = 18 warps: warps 0..15 are the epilogue (four warps per TMEM lane quarter, each owning one 64-column piece of
// every unit), warp 16 lane 0 issues TMA loads (query panel once per segment, base tiles through a ring of stages),
// warp 17 lane 0 issues tcgen05.mma. TMEM holds two accumulator slots of 256 columns: the MMAs of one unit run while the
// epilogue reads the other; a slot goes back to the MMA warp as soon as its columns are in registers. No cluster
// launch: each CTA loads its own tiles from its GPU's memory.
#include "screen_i8.cuh"

#include "ptx.cuh"

#include <math_constants.h>

namespace certex_b200 {

namespace {

using namespace ptx;

constexpr int kQTileBytes = kQueryTile * 128;  // one K block of a query tile: 128 rows x 128 bytes
constexpr int kBTileBytes = kBaseTile * 128;   // one K block of a base tile: 256 rows x 128 bytes
constexpr int kSlots      = 2;                 // TMEM accumulator slots (2 x 256 columns = all 512)
constexpr int kEpiWarps   = 16;
constexpr int kThreads    = 32 * (2 + kEpiWarps);
// The two single-thread roles sit in the last two warps; warps 0..15 are the epilogue (TMEM lane quarter = warp % 4).
constexpr int kTmaWarp    = kEpiWarps;
constexpr int kMmaWarp    = kEpiWarps + 1;
constexpr int kRecBuf     = 64;                // staged survivor records per epilogue warp (flushed when half full)
constexpr int kWideStage  = 2 * kQTileBytes + kBTileBytes;  // WIDE: one K block of two query tiles and a base tile
constexpr int kWideStages = 3;
constexpr int kERing      = 4;                 // WIDE: tiles whose e values may be in flight
#ifndef CERTEX_SPLIT_EPILOGUE
#define CERTEX_SPLIT_EPILOGUE 1
#endif
constexpr bool kSplit     = CERTEX_SPLIT_EPILOGUE != 0;  // two groups of 8 epilogue warps, one per TMEM slot

#ifndef CERTEX_SCREEN_TRACE
#define CERTEX_SCREEN_TRACE 0
#endif
#if CERTEX_SCREEN_TRACE
#define TRACE_AT(cond, unit, slot) \
  do {                             \
    if ((cond) && (unit) < static_cast<uint32_t>(p.trace_units)) { p.trace[static_cast<size_t>(unit) * 12 + (slot)] = clock64(); } \
  } while (0)
#else
#define TRACE_AT(cond, unit, slot) \
  do {                             \
  } while (0)
#endif


struct SharedCtl {
  uint64_t full[kMaxStages];    // TMA landed a base tile (GROUPMAX: and its e values) in the stage
  uint64_t empty[kMaxStages];   // the stage may be overwritten (GROUPMAX: also every epilogue warp is done with e)
  uint64_t tmem_full[kSlots];   // the MMAs of a unit are complete
  uint64_t tmem_empty[kSlots];  // the unit's accumulator is in registers (all 16 epilogue warps)
  uint64_t panel_full;
  uint64_t panel_empty;
  uint64_t drain;
  uint64_t e_full[kERing];      // WIDE: the e values of a tile have landed
  uint64_t e_empty[kERing];     // WIDE: every epilogue warp is done with them

  uint32_t tmem_base;
  int abort_flag;
  int rec_n[kEpiWarps];         // fill counts of the warps' record staging buffers
};

__device__ __forceinline__ int max3(int a, int b, int c) { return __vimax3_s32(a, b, c); }
__device__ __forceinline__ int addmax(int a, int b, int c) { return __viaddmax_s32(a, b, c); }  // max(a + b, c)

// Maximum of 16 adjacent accumulator columns (two chains).
__device__ __forceinline__ int max16(const int32_t* v)
{
  int m = max3(v[0], v[1], v[2]);
  int n = max3(v[3], v[4], v[5]);
  m     = max3(m, v[6], v[7]);
  n     = max3(n, v[8], v[9]);
  m     = max3(m, v[10], v[11]);
  n     = max3(n, v[12], v[13]);
  return max3(m, n, max(v[14], v[15]));
}

// Maximum of v[i] + e[i] over 32 columns, e in shared memory (two chains).
__device__ __forceinline__ int max32_plus(const int32_t* v, const int32_t* e)
{
  const int4* e4 = reinterpret_cast<const int4*>(e);
  int m = kNeverInit * 2 + 1, n = m;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int4 t = e4[i];
    m = addmax(v[4 * i], t.x, m);
    n = addmax(v[4 * i + 1], t.y, n);
    m = addmax(v[4 * i + 2], t.z, m);
    n = addmax(v[4 * i + 3], t.w, n);
  }
  return max(m, n);
}

// float versions; accumulators arrive as the raw 32 bits of an fp32 value
__device__ __forceinline__ float fmax3(float a, float b, float c) { return fmaxf(fmaxf(a, b), c); }

__device__ __forceinline__ float max16f(const int32_t* v)
{
  float m = fmax3(__int_as_float(v[0]), __int_as_float(v[1]), __int_as_float(v[2]));
  float n = fmax3(__int_as_float(v[3]), __int_as_float(v[4]), __int_as_float(v[5]));
  m       = fmax3(m, __int_as_float(v[6]), __int_as_float(v[7]));
  n       = fmax3(n, __int_as_float(v[8]), __int_as_float(v[9]));
  m       = fmax3(m, __int_as_float(v[10]), __int_as_float(v[11]));
  n       = fmax3(n, __int_as_float(v[12]), __int_as_float(v[13]));
  return fmax3(m, n, fmaxf(__int_as_float(v[14]), __int_as_float(v[15])));
}

__device__ __forceinline__ float max32f_plus(const int32_t* v, const int32_t* e)
{
  const float4* e4 = reinterpret_cast<const float4*>(e);
  float m = -CUDART_INF_F, n = m;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const float4 t = e4[i];
    m = fmaxf(m, __int_as_float(v[4 * i]) + t.x);
    n = fmaxf(n, __int_as_float(v[4 * i + 1]) + t.y);
    m = fmaxf(m, __int_as_float(v[4 * i + 2]) + t.z);
    n = fmaxf(n, __int_as_float(v[4 * i + 3]) + t.w);
  }
  return fmaxf(m, n);
}

// Maximum of v[i] + e[i] over one chain of 16 columns.
__device__ __forceinline__ int max16_plus(const int32_t* v, const int32_t* e)
{
  const int4* e4 = reinterpret_cast<const int4*>(e);
  int m = kNeverInit * 2 + 1, n = m;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int4 t = e4[i];
    m = addmax(v[4 * i], t.x, m);
    n = addmax(v[4 * i + 1], t.y, n);
    m = addmax(v[4 * i + 2], t.z, m);
    n = addmax(v[4 * i + 3], t.w, n);
  }
  return max(m, n);
}

__device__ __forceinline__ float max16f_plus(const int32_t* v, const int32_t* e)
{
  const float4* e4 = reinterpret_cast<const float4*>(e);
  float m = -CUDART_INF_F, n = m;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float4 t = e4[i];
    m = fmaxf(m, __int_as_float(v[4 * i]) + t.x);
    n = fmaxf(n, __int_as_float(v[4 * i + 1]) + t.y);
    m = fmaxf(m, __int_as_float(v[4 * i + 2]) + t.z);
    n = fmaxf(n, __int_as_float(v[4 * i + 3]) + t.w);
  }
  return fmaxf(m, n);
}

/// Monotone map of a float to an int32 (and back), so that integer selection kernels can rank floats.
__device__ __forceinline__ int32_t float_key(float f)
{
  const int32_t i = __float_as_int(f);
  return i ^ ((i >> 31) & 0x7fffffff);
}

// KB: K blocks per code row of the resident-panel variants, fixed at compile time (1 or 2) so that the issuing thread's
// loop over a unit's MMAs unrolls; 0 for WIDE, where the number of K blocks is a run-time value.
template <int MODE, bool F16, bool WIDE, int KB>
__global__ void __launch_bounds__(kThreads, 1) screen_i8_kernel(const __grid_constant__ CUtensorMap tm_q,
                                                                const __grid_constant__ CUtensorMap tm_x,
                                                                const ScreenArgs p)
{
  extern __shared__ uint8_t smem_raw[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  // the CTA's segments: a slice of one list (seg_begin), or its kMaxSegs slots of which the leading ones are used
  const int seg_first   = p.seg_begin ? p.seg_begin[blockIdx.x] : static_cast<int>(blockIdx.x) * kMaxSegs;
  const ScreenSeg* gsegs = p.segs + seg_first;
  const int* seg_col0    = p.seg_col0 ? p.seg_col0 + seg_first : nullptr;
  const int* seg_step    = p.seg_step ? p.seg_step + seg_first : nullptr;  // GROUPMAX over a strided sample of tiles
  int nseg               = 0;
  if (p.seg_begin) {
    nseg = p.seg_begin[blockIdx.x + 1] - seg_first;
  } else {
    while (nseg < kMaxSegs && gsegs[nseg].t1 > gsegs[nseg].t0) { ++nseg; }
  }
  if (nseg <= 0) { return; }  // uniform over the CTA

  // ---- shared memory carve-up (1024-byte aligned tiles for the 128-byte swizzle)
  const uint32_t base      = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* gen_base        = smem_raw + (base - smem_u32(smem_raw));
  const int kb             = WIDE ? p.kb : KB;
  const int ns             = WIDE ? kWideStages : p.n_stages;
  const uint32_t panel_off = 0;
  const uint32_t stage_off = WIDE ? 0u : panel_off + static_cast<uint32_t>(p.panel_tiles) * kb * kQTileBytes;
  const uint32_t init_off  = stage_off + (WIDE ? static_cast<uint32_t>(kWideStages * kWideStage)
                                               : static_cast<uint32_t>(ns) * kb * kBTileBytes);
  const uint32_t rec_off   = init_off + static_cast<uint32_t>(WIDE ? kERing : ns) * kBaseTile * 4;
  const uint32_t ctl_off   = rec_off + kEpiWarps * kRecBuf * 8;
  SharedCtl* ctl           = reinterpret_cast<SharedCtl*>(gen_base + ctl_off);
  const int32_t* init_smem = reinterpret_cast<const int32_t*>(gen_base + init_off);
  volatile int* abort_flag = &ctl->abort_flag;
#if CERTEX_SCREEN_TRACE
  const bool tr_cta = p.trace != nullptr && blockIdx.x == 0 && !WIDE;
#endif
  constexpr bool kNeedE    = MODE == kModeGroupMax;   // only the exact group maxima need the e of every row
  constexpr bool kGroups   = MODE == kModeGroupMax || MODE == kModeGroupBound;  // the passes of the threshold stage
  constexpr bool kChainE   = MODE == kModeScreen || MODE == kModeGroupBound;    // e enters per chain of 16 columns (p.cmax)
  constexpr bool kStageE   = kNeedE && !WIDE;          // resident panel: e travels with the stage; WIDE: in its own ring

  // every role walks the CTA's segment list in global memory (a segment is hundreds of units long: the read is nothing)
  const ScreenSeg* segs = gsegs;
  if (threadIdx.x == 0) {
    for (int i = 0; i < ns; ++i) {
      mbar_init(smem_u32(&ctl->full[i]), 1);
      mbar_init(smem_u32(&ctl->empty[i]), kStageE ? 1 + kEpiWarps : 1);
    }
    for (int i = 0; i < kSlots; ++i) {
      mbar_init(smem_u32(&ctl->tmem_full[i]), 1);
      mbar_init(smem_u32(&ctl->tmem_empty[i]), kSplit ? kEpiWarps / 2 : kEpiWarps);
    }
    mbar_init(smem_u32(&ctl->panel_full), 1);
    mbar_init(smem_u32(&ctl->panel_empty), 1);
    mbar_init(smem_u32(&ctl->drain), 1);
    for (int i = 0; i < kERing; ++i) {
      mbar_init(smem_u32(&ctl->e_full[i]), 1);
      mbar_init(smem_u32(&ctl->e_empty[i]), kEpiWarps);
    }

    ctl->abort_flag = 0;
    for (int i = 0; i < kEpiWarps; ++i) { ctl->rec_n[i] = 0; }
    fence_barrier_init();
    prefetch_tensormap(&tm_q);
    prefetch_tensormap(&tm_x);
  }
  if (warp == kMmaWarp) {
    tmem_alloc(smem_u32(&ctl->tmem_base), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = ctl->tmem_base;

  if (warp == kTmaWarp) {
    // ================================================================ TMA producer
    if (WIDE && lane == 0) {
      int ks = 0, ts = 0;  // K-block stages and tiles issued so far
      bool aborted = false;
      for (int s = 0; s < nseg && !aborted; ++s) {
        const ScreenSeg sg = segs[s];
        const int c0       = (kGroups && seg_col0) ? seg_col0[s] : 0;
        const int stp      = (kGroups && seg_step) ? seg_step[s] : 1;
        for (int t = sg.t0; t < sg.t1 && !aborted; ++t, ++ts) {
          const int ta = c0 + (t - c0) * stp;  // the tile that is read
          if (kNeedE) {
            const int er = ts % kERing;
            if (ts >= kERing && !mbar_wait(smem_u32(&ctl->e_empty[er]), ((ts / kERing) - 1) & 1, abort_flag, p.err, 8)) {
              aborted = true;
              break;
            }
            mbar_arrive_expect_tx(smem_u32(&ctl->e_full[er]), kBaseTile * 4);
            bulk_load_1d(base + init_off + er * kBaseTile * 4, p.init + static_cast<size_t>(ta) * kBaseTile, kBaseTile * 4,
                         smem_u32(&ctl->e_full[er]));
          }
          for (int b = 0; b < kb; ++b, ++ks) {
            const int st = ks % ns;
            if (ks >= ns && !mbar_wait(smem_u32(&ctl->empty[st]), ((ks / ns) - 1) & 1, abort_flag, p.err, 2)) {
              aborted = true;
              break;
            }
            const uint32_t fbar = smem_u32(&ctl->full[st]);
            const uint32_t dst  = base + stage_off + st * kWideStage;
            mbar_arrive_expect_tx(fbar, static_cast<uint32_t>(sg.n_qtiles) * kQTileBytes + kBTileBytes);
            for (int j = 0; j < sg.n_qtiles; ++j) {
              tma_load_2d(dst + j * kQTileBytes, &tm_q, b * 128, (sg.q_tile0 + j) * kQueryTile, fbar);
            }
            if (MODE == kModeGroupBound) {
              tma_load_4d(dst + 2 * kQTileBytes, &tm_x, b * 128, 0, 0, ta, fbar);
            } else if (MODE == kModeGroupMax && !p.plain_tiles) {
              tma_load_3d(dst + 2 * kQTileBytes, &tm_x, b * 128, 0, ta, fbar);
            } else {
              tma_load_2d(dst + 2 * kQTileBytes, &tm_x, b * 128, ta * kBaseTile, fbar);
            }
          }
        }
      }
      if (*abort_flag) {
        // let the copies that are still in flight land before the CTA leaves (bounded)
        for (int back = 1; back <= ns && back <= ks; ++back) {
          const int u        = ks - back;
          const long long t0 = clock64();
          while (!mbar_try_wait(smem_u32(&ctl->full[u % ns]), (u / ns) & 1) && clock64() - t0 < (1ll << 24)) {}
        }
        for (int back = 1; kNeedE && back <= kERing && back <= ts; ++back) {
          const int u        = ts - back;
          const long long t0 = clock64();
          while (!mbar_try_wait(smem_u32(&ctl->e_full[u % kERing]), (u / kERing) & 1) && clock64() - t0 < (1ll << 24)) {}
        }
      }
    } else if (lane == 0) {
      int ts       = 0;
      bool aborted = false;
      for (int s = 0; s < nseg && !aborted; ++s) {
        const ScreenSeg sg = segs[s];
        if (s > 0 && !mbar_wait(smem_u32(&ctl->panel_empty), (s - 1) & 1, abort_flag, p.err, 1)) { break; }
        const uint32_t pbar = smem_u32(&ctl->panel_full);
        mbar_arrive_expect_tx(pbar, static_cast<uint32_t>(sg.n_qtiles) * kb * kQTileBytes);
        for (int j = 0; j < sg.n_qtiles; ++j) {
          for (int b = 0; b < kb; ++b) {
            tma_load_2d(base + panel_off + (j * kb + b) * kQTileBytes, &tm_q, b * 128, (sg.q_tile0 + j) * kQueryTile, pbar);
          }
        }
        const int c0  = (kGroups && seg_col0) ? seg_col0[s] : 0;
        const int stp = (kGroups && seg_step) ? seg_step[s] : 1;
        for (int t = sg.t0; t < sg.t1; ++t, ++ts) {
          const int ta = c0 + (t - c0) * stp;  // the tile that is read
          const int st = ts % ns;
          if (ts >= ns && !mbar_wait(smem_u32(&ctl->empty[st]), ((ts / ns) - 1) & 1, abort_flag, p.err, 2)) {
            aborted = true;
            break;
          }
          const uint32_t fbar = smem_u32(&ctl->full[st]);
          mbar_arrive_expect_tx(fbar, static_cast<uint32_t>(kb) * kBTileBytes + (kStageE ? kBaseTile * 4 : 0));
          for (int b = 0; b < kb; ++b) {
            if (MODE == kModeGroupBound) {
              // anchors in chains: columns 16 i .. 16 i + 15 of tile t are 16 adjacent anchors, the chains of a tile are
              // spread over the whole (norm-sorted) set; the map is 4-D (bytes, anchor of the chain, chain, tile)
              tma_load_4d(base + stage_off + (st * kb + b) * kBTileBytes, &tm_x, b * 128, 0, 0, ta, fbar);
            } else if (MODE == kModeGroupMax && !p.plain_tiles) {
              // anchors: column c of tile t is anchor c * n_tiles + t, so every group of 64 columns samples the whole
              // (norm-sorted) set; the map is 3-D (bytes, column, tile)
              tma_load_3d(base + stage_off + (st * kb + b) * kBTileBytes, &tm_x, b * 128, 0, ta, fbar);
            } else {
              tma_load_2d(base + stage_off + (st * kb + b) * kBTileBytes, &tm_x, b * 128, ta * kBaseTile, fbar);
            }
          }
          if (kStageE) {
            bulk_load_1d(base + init_off + st * kBaseTile * 4, p.init + static_cast<size_t>(ta) * kBaseTile, kBaseTile * 4, fbar);
          }
        }
      }
      if (*abort_flag) {
        // let the copies that are still in flight land before the CTA leaves (bounded)
        for (int back = 1; back <= ns && back <= ts; ++back) {
          const int u        = ts - back;
          const long long t0 = clock64();
          while (!mbar_try_wait(smem_u32(&ctl->full[u % ns]), (u / ns) & 1) && clock64() - t0 < (1ll << 24)) {}
        }
      }
    }
  } else if (warp == kMmaWarp) {
    // ================================================================ MMA issuer
    if (lane == 0) {
      const uint32_t idesc = F16 ? instr_desc(1u, 0u, 0u, kQueryTile, kBaseTile)
                                 : instr_desc(2u, p.q_signed, p.x_signed, kQueryTile, kBaseTile);
      // descriptors differ only in their 14-bit start-address field: (byte offset >> 4) is added to the low word
      const uint64_t a_desc0 = smem_desc_sw128(base + panel_off);
      const uint64_t b_desc0 = smem_desc_sw128(base + stage_off);
      uint32_t gu = 0;
      bool ok = true;
      if (WIDE) {
        int ks = 0;
        for (int s = 0; s < nseg && ok; ++s) {
          const ScreenSeg sg = segs[s];
          for (int t = sg.t0; t < sg.t1 && ok; ++t, gu += sg.n_qtiles) {
            for (int b = 0; b < kb && ok; ++b, ++ks) {
              const int st = ks % ns;
              ok           = mbar_wait(smem_u32(&ctl->full[st]), (ks / ns) & 1, abort_flag, p.err, 4);
              if (!ok) { break; }
              tc_fence_after();
              const uint64_t s_desc = b_desc0 + static_cast<uint64_t>(st) * (kWideStage >> 4);
              for (int j = 0; j < sg.n_qtiles; ++j) {
                const int u    = static_cast<int>(gu) + j;
                const int slot = u & (kSlots - 1);
                if (b == 0 && u >= kSlots) {  // the slot's previous unit must be in the epilogue's registers
                  ok = mbar_wait(smem_u32(&ctl->tmem_empty[slot]), ((u >> 1) - 1) & 1, abort_flag, p.err, 5);
                  if (!ok) { break; }
                  tc_fence_after();
                }
                const uint32_t d_tmem = tmem + static_cast<uint32_t>(slot * kBaseTile);
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                  const uint64_t ad = s_desc + static_cast<uint64_t>(j * (kQTileBytes >> 4) + k * 2);
                  const uint64_t bd = s_desc + static_cast<uint64_t>(2 * (kQTileBytes >> 4) + k * 2);
                  if (F16) {
                    mma_f16(d_tmem, ad, bd, idesc, (b | k) != 0 ? 1u : 0u);
                  } else {
                    mma_i8(d_tmem, ad, bd, idesc, (b | k) != 0 ? 1u : 0u);
                  }
                }
                if (b == kb - 1) { tc_commit(smem_u32(&ctl->tmem_full[slot])); }
              }
              if (ok) { tc_commit(smem_u32(&ctl->empty[st])); }
            }
          }
        }
      }
      if (!WIDE) {
        // The thread that issues the MMAs is alone in its warp: every instruction it executes costs its full latency,
        // and a unit of a 128-byte row is only four MMA instructions long. So the loop is kept to the waits, the
        // instructions themselves and one add per descriptor: descriptors differ only in the low word (start address
        // >> 4), the accumulate flag is an immediate, ring positions and parities are carried instead of divided out.
        constexpr int kKB          = KB > 0 ? KB : 1;
        const uint32_t desc_hi     = static_cast<uint32_t>(a_desc0 >> 32);
        const uint32_t a_lo0       = static_cast<uint32_t>(a_desc0), b_lo0 = static_cast<uint32_t>(b_desc0);
        const uint32_t full_bar0   = smem_u32(&ctl->full[0]), empty_bar0 = smem_u32(&ctl->empty[0]);
        const uint32_t tfull_bar0  = smem_u32(&ctl->tmem_full[0]), tempty_bar0 = smem_u32(&ctl->tmem_empty[0]);
        int st = 0;
        uint32_t st_par = 0;
        for (int s = 0; s < nseg && ok; ++s) {
          const ScreenSeg sg = segs[s];
          ok                 = mbar_wait(smem_u32(&ctl->panel_full), s & 1, abort_flag, p.err, 3);
          for (int t = sg.t0; t < sg.t1 && ok; ++t) {
            ok = mbar_wait(full_bar0 + st * 8, st_par, abort_flag, p.err, 4);
            if (!ok) { break; }
            const uint32_t b_lo = b_lo0 + static_cast<uint32_t>(st) * (kKB * kBTileBytes >> 4);
            uint32_t a_lo       = a_lo0;
            for (int j = 0; j < sg.n_qtiles; ++j, ++gu, a_lo += kKB * kQTileBytes >> 4) {
              const uint32_t slot = gu & 1u;
              // a fresh barrier passes a wait for parity 1: the first unit of a slot does not wait
              if (MODE != kModeRate) {
                TRACE_AT(tr_cta, gu, 0);
                ok = mbar_wait(tempty_bar0 + slot * 8, ((gu >> 1) & 1u) ^ 1u, abort_flag, p.err, 5);
                if (!ok) { break; }
                TRACE_AT(tr_cta, gu, 1);
              }
              tc_fence_after();
              const uint32_t d_tmem = tmem + slot * kBaseTile;
#pragma unroll
              for (int b = 0; b < kKB; ++b) {
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                  const uint64_t ad = pack64(a_lo + b * (kQTileBytes >> 4) + k * 2, desc_hi);
                  const uint64_t bd = pack64(b_lo + b * (kBTileBytes >> 4) + k * 2, desc_hi);
                  if (b == 0 && k == 0) {
                    if (F16) { mma_f16_c<false>(d_tmem, ad, bd, idesc); } else { mma_i8_c<false>(d_tmem, ad, bd, idesc); }
                  } else {
                    if (F16) { mma_f16_c<true>(d_tmem, ad, bd, idesc); } else { mma_i8_c<true>(d_tmem, ad, bd, idesc); }
                  }
                }
              }
              tc_commit(tfull_bar0 + slot * 8);
              TRACE_AT(tr_cta, gu, 2);
            }
            if (ok) { tc_commit(empty_bar0 + st * 8); }
            if (++st == ns) { st = 0, st_par ^= 1u; }
          }
          if (ok) { tc_commit(smem_u32(&ctl->panel_empty)); }
        }
      }
      // every MMA issued above has completed before TMEM is released
      tc_commit(smem_u32(&ctl->drain));
      {
        const long long t0 = clock64();
        while (!mbar_try_wait(smem_u32(&ctl->drain), 0) && clock64() - t0 < kWaitLimitCycles) {}
      }
    }
  } else if (MODE != kModeRate) {
    // ================================================================ epilogue (16 warps, one 64-column piece each)
    const int ew             = warp;
    const int piece          = ew >> 2;   // which 64 columns of a unit
    const int quarter        = warp & 3;  // the TMEM lane quarter this warp may access
    const int row            = quarter * 32 + lane;
    const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
    uint64_t* rec_buf        = reinterpret_cast<uint64_t*>(gen_base + rec_off) + ew * kRecBuf;
    volatile int* rec_n      = &ctl->rec_n[ew];  // staged records of this warp

    uint32_t gu = 0;  // units of this CTA so far: slot = gu & 1, the slot's use number = gu >> 1
    bool ok     = true;

    // Staged records -> global memory: one atomic add reserves the range, the lanes copy.
    auto flush = [&](int n_rec) {
      unsigned long long at = 0;
      if (lane == 0) { at = atomicAdd(p.rec_count, static_cast<unsigned long long>(n_rec)); }
      at = __shfl_sync(0xffffffffu, at, 0);
      for (int i = lane; i < n_rec; i += 32) {
        if (at + i < p.rec_cap) { p.rec[at + i] = rec_buf[i]; }
      }
      __syncwarp();
      if (lane == 0) { *rec_n = 0; }
      __syncwarp();
    };
    // A chain of 16 columns whose maximum reached the query's threshold with the chain's largest e: the columns that
    // reach it with that same e form one record. (Rows are kept sorted by norm, so e is almost constant over a chain
    // and hardly any row is kept that the exact e would drop; the exact scores sort that out.) The record is staged
    // through the warp's buffer in shared memory, whose fill count is a shared-memory atomic: the few threads that get
    // here need no warp-wide step.
    auto record = [&](const int32_t* v, int thr, int ce, int q, int64_t row0) {
      uint32_t mask = 0;
      if (F16) {
        const float tf = __int_as_float(thr), cf = __int_as_float(ce);
#pragma unroll
        for (int i = 0; i < 16; ++i) { mask |= (__int_as_float(v[i]) + cf >= tf ? 1u : 0u) << i; }
      } else {
        const int t = thr - ce;  // no overflow: |thr|, |ce| <= 2^30 wherever a chain passed the test
#pragma unroll
        for (int i = 0; i < 16; ++i) { mask |= (v[i] >= t ? 1u : 0u) << i; }
      }
      const uint64_t r = make_record(static_cast<uint32_t>(q), static_cast<uint32_t>(row0 / kChainRows), mask);
      const int pos    = atomicAdd(const_cast<int*>(rec_n), 1);
      if (pos < kRecBuf) {
        rec_buf[pos] = r;
      } else {  // the staging buffer is full: straight to global memory
        const unsigned long long at = atomicAdd(p.rec_count, 1ull);
        if (at < p.rec_cap) { p.rec[at] = r; }
      }
    };

    // An epilogue warp is one serial stream of instructions per unit, and the pass is as fast as that stream (the MMAs
    // of a unit of a 128-byte row take about 610 cycles; a hundred dependent instructions of a warp that shares its
    // scheduler with four others take more). So the loops are plain nested loops over the segment's tiles and query
    // tiles with pointers that are bumped, nothing is recomputed per unit that is known per tile or per segment, and
    // warp-wide steps (the check of the record buffer) happen once per tile. Everything between a unit's completion and
    // the release of its slot also sits on the other path that bounds the pass (two slots: the MMAs of the next unit but
    // one wait for the release): the threshold and the chain maxima of e are loaded before the wait and not touched
    // until the slot is released, and the release follows tcgen05.wait::ld directly (it is warp-wide: when lane 0 is
    // past it, every lane's columns are in registers).
    const uint32_t tfull_bar0 = smem_u32(&ctl->tmem_full[0]), tempty_bar0 = smem_u32(&ctl->tmem_empty[0]);
    const int never_thr       = F16 ? __float_as_int(CUDART_INF_F) : 0x7fffffff;  // float bits when F16
    constexpr int kERingOrNs  = WIDE ? kERing : 0;
    int est = 0;            // GROUPMAX: ring position of the tile's e values and its parity
    uint32_t est_par = 0;
    const int e_ring = kERingOrNs ? kERingOrNs : ns;
#if CERTEX_SCREEN_TRACE
    const bool tr_w = tr_cta && lane == 0 && ew == 0, tr_x = tr_cta && lane == 0 && ew == kEpiWarps - 1;
#endif
    // With kSplit the 16 warps form two groups of 8, one per TMEM slot: group g reads the units of slot g (every other
    // unit), each warp two 64-column pieces of it. A warp then has two unit times for the fixed latencies of a unit
    // (noticing its completion, tcgen05.ld, the release) and its comparisons run while the other group waits; the price
    // is a later release: the second piece can only be loaded into the registers the first has left.
    const uint32_t grp = kSplit ? static_cast<uint32_t>(ew) >> 3 : 0u;
    const int piece0   = kSplit ? ((ew >> 2) & 1) * 2 : piece;  // first (or only) 64-column piece of this warp
    const uint32_t taddr_w = tmem + lane_base + static_cast<uint32_t>(piece0 * kGroupRows);
    for (int s = 0; s < nseg && ok; ++s) {
      const ScreenSeg sg = segs[s];
      const int nqt      = sg.n_qtiles;
      const int q_first  = sg.q_tile0 * kQueryTile + row;
      const int col0     = (kGroups && seg_col0) ? seg_col0[s] : 0;
      const int4* cm     = reinterpret_cast<const int4*>(p.cmax) + static_cast<size_t>(sg.t0) * (kBaseTile / kChainRows / 4) + piece0;
      for (int t = sg.t0; t < sg.t1 && ok; ++t, cm += kBaseTile / kChainRows / 4) {
        // the four chain maxima of e of each of this warp's pieces of the tile
        int4 ce0 = make_int4(0, 0, 0, 0), ce1 = ce0;
        if (kChainE) {
          ce0 = __ldg(cm);
          if (kSplit) { ce1 = __ldg(cm + 1); }
        }
        if (kNeedE) {
          // the tile's e values landed with (or, WIDE, ahead of) its code rows. Every warp waits for them, also one
          // that has no unit of its own in this tile: its release at the end of the tile must not run ahead of the
          // refill of the ring slot, or it would be counted for the wrong round
          ok = mbar_wait(WIDE ? smem_u32(&ctl->e_full[est]) : smem_u32(&ctl->full[est]), est_par, abort_flag, p.err, 6);
          if (!ok) { break; }
        }
        const int32_t* e   = init_smem + est * kBaseTile + piece0 * kGroupRows;  // GROUPMAX: the tile's e values
        const int64_t row0 = static_cast<int64_t>(t) * kBaseTile + piece0 * kGroupRows;
        bool kept          = false;
        int q              = q_first;
        for (int j = 0; j < nqt; ++j, ++gu, q += kQueryTile) {
          const uint32_t slot = gu & 1u;
          if (kSplit && slot != grp) { continue; }
          int thr = never_thr;
          if (MODE == kModeScreen && q < p.nq) { thr = __ldg(p.thr + q); }
          TRACE_AT(tr_w, gu, 3);
          ok = mbar_wait(tfull_bar0 + slot * 8, (gu >> 1) & 1u, abort_flag, p.err, 7);
          if (!ok) { break; }
          TRACE_AT(tr_w, gu, 4);
          TRACE_AT(tr_x, gu, 8);
          tc_fence_after();
          const uint32_t taddr = taddr_w + slot * kBaseTile;
          int32_t a[32], b[32];
          tmem_ld32(taddr, a);
          tmem_ld32(taddr + 32, b);
          tmem_wait_ld(a);
          reg_fence32(b);
          auto release = [&] {
            TRACE_AT(tr_w, gu, 5);
            TRACE_AT(tr_x, gu, 9);
            // the unit is in registers (tcgen05.wait::ld is warp-wide): the slot goes back to the MMA warp
            tc_fence_before();
            if (lane == 0) { mbar_arrive(tempty_bar0 + slot * 8); }
            TRACE_AT(tr_w, gu, 6);
          };
          // 32 columns (two chains) of a SCREEN piece: v = a or b, c0 / c1 their chain maxima of e
          auto screen32 = [&](const int32_t* v, int c0, int c1, int64_t r0) {
            bool h0, h1;
            if (F16) {
              const float tf = __int_as_float(thr);
              h0 = max16f(v) + __int_as_float(c0) >= tf;
              h1 = max16f(v + 16) + __int_as_float(c1) >= tf;
            } else {
              h0 = max16(v) + c0 >= thr;
              h1 = max16(v + 16) + c1 >= thr;
            }
            if (h0 | h1) {  // rare: the lanes that kept something stage their records, nobody else waits
              if (h0) { record(v, thr, c0, q, r0); }
              if (h1) { record(v + 16, thr, c1, q, r0 + 16); }
              kept = true;
            }
          };
          // GROUPMAX, 32 columns: partial results of a piece (.x/.y from a, .z/.w from b; coarse groups use .x and .z)
          auto gmax32 = [&](const int32_t* v, const int32_t* ev, int& m0, int& m1) {
            if (p.fine_groups) {
              m0 = F16 ? float_key(max16f_plus(v, ev)) : max16_plus(v, ev);
              m1 = F16 ? float_key(max16f_plus(v + 16, ev + 16)) : max16_plus(v + 16, ev + 16);
            } else {
              m0 = F16 ? __float_as_int(max32f_plus(v, ev)) : max32_plus(v, ev);
            }
          };
          // GROUPBOUND, 32 columns: max over the two chains of (largest product + the chain's smallest e)
          auto bound32 = [&](const int32_t* v, int c0, int c1) {
            if (F16) {
              return __float_as_int(fmaxf(max16f(v) + __int_as_float(c0), max16f(v + 16) + __int_as_float(c1)));
            }
            return max(max16(v) + c0, max16(v + 16) + c1);
          };
          // One group value per 64-column piece. Rows of gmax are far apart, so every 4-byte store of a thread is a memory
          // transaction of its own; with the two-group epilogue a thread holds two adjacent pieces of its row and
          // writes both values with one 8-byte store.
          int held = 0;  // kSplit: the value of the warp's first piece, until the second is known
          auto put = [&](int pc, int m) {
            int32_t* dst = p.gmax + static_cast<size_t>(q) * p.ld_gmax + (t - col0) * (kBaseTile / kGroupRows) + pc;
            if (!kSplit) {
              if (q < p.nq) { *dst = m; }
            } else if (pc == piece0) {
              held = m;
            } else if (q < p.nq) {
              *reinterpret_cast<int2*>(dst - 1) = make_int2(held, m);
            }
          };
          auto bound_store = [&](int ma, int mb, int pc) {
            put(pc, F16 ? float_key(fmaxf(__int_as_float(ma), __int_as_float(mb))) : max(ma, mb));
          };
          auto gmax_store = [&](const int4& m4, int pc) {
            if (q >= p.nq) { return; }
            if (p.fine_groups) {
              // one maximum per chain of 16 rows: four times as many groups, for labels too small for 2k groups of 64
              *reinterpret_cast<int4*>(p.gmax + static_cast<size_t>(q) * p.ld_gmax + (t - col0) * (kBaseTile / kChainRows) + pc * 4) = m4;
            } else {
              put(pc, F16 ? float_key(fmaxf(__int_as_float(m4.x), __int_as_float(m4.z))) : max(m4.x, m4.z));
            }
          };
          if (!kSplit) {
            release();
            if (MODE == kModeScreen) {
              screen32(a, ce0.x, ce0.y, row0);
              screen32(b, ce0.z, ce0.w, row0 + 32);
            } else if (MODE == kModeGroupBound) {
              bound_store(bound32(a, ce0.x, ce0.y), bound32(b, ce0.z, ce0.w), piece0);
            } else {
              int4 m4 = make_int4(0, 0, 0, 0);
              gmax32(a, e, m4.x, m4.y);
              gmax32(b, e + 32, m4.z, m4.w);
              gmax_store(m4, piece0);
            }
          } else {
            // first piece; each half of the second piece is fetched as soon as its registers are free
            int4 m4 = make_int4(0, 0, 0, 0);
            int ma = 0, mb = 0;
            if (MODE == kModeScreen) {
              screen32(a, ce0.x, ce0.y, row0);
            } else if (MODE == kModeGroupBound) {
              ma = bound32(a, ce0.x, ce0.y);
            } else {
              gmax32(a, e, m4.x, m4.y);
            }
            tmem_ld32(taddr + 64, a);
            if (MODE == kModeScreen) {
              screen32(b, ce0.z, ce0.w, row0 + 32);
            } else if (MODE == kModeGroupBound) {
              mb = bound32(b, ce0.z, ce0.w);
            } else {
              gmax32(b, e + 32, m4.z, m4.w);
            }
            tmem_ld32(taddr + 96, b);
            if (MODE == kModeGroupBound) { bound_store(ma, mb, piece0); }
            if (MODE == kModeGroupMax) { gmax_store(m4, piece0); }
            tmem_wait_ld(a);
            reg_fence32(b);
            release();
            if (MODE == kModeScreen) {
              screen32(a, ce1.x, ce1.y, row0 + 64);
              screen32(b, ce1.z, ce1.w, row0 + 96);
            } else if (MODE == kModeGroupBound) {
              bound_store(bound32(a, ce1.x, ce1.y), bound32(b, ce1.z, ce1.w), piece0 + 1);
            } else {
              gmax32(a, e + 64, m4.x, m4.y);
              gmax32(b, e + 96, m4.z, m4.w);
              gmax_store(m4, piece0 + 1);
            }
          }
          TRACE_AT(tr_w, gu, 7);
        }
        if (!ok) { break; }
        // the tile is done: staged records go out once the buffer is half full (records beyond its end go straight to
        // global memory meanwhile), and the tile's e values are released (GROUPMAX)
        if (MODE == kModeScreen && __any_sync(0xffffffffu, kept)) {
          const int staged = min(*rec_n, kRecBuf);
          if (staged > kRecBuf / 2) { flush(staged); }
        }
        if (kNeedE) {
          __syncwarp();
          if (lane == 0) { mbar_arrive(WIDE ? smem_u32(&ctl->e_empty[est]) : smem_u32(&ctl->empty[est])); }
          if (++est == e_ring) { est = 0, est_par ^= 1u; }
        }
      }
    }
    if (MODE == kModeScreen) {
      __syncwarp();
      const int staged = min(*rec_n, kRecBuf);
      if (staged > 0) { flush(staged); }
    }
  }

  // ---- teardown: all roles meet here, also when a wait gave up
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == kMmaWarp) { tmem_dealloc(tmem, 512); }
}

}  // namespace

size_t screen_smem_bytes_wide()
{
  return 1024 + static_cast<size_t>(kWideStages) * kWideStage + static_cast<size_t>(kERing) * kBaseTile * 4 +
         kEpiWarps * kRecBuf * 8 + sizeof(SharedCtl) + 64;
}

size_t screen_smem_bytes(int kb, int panel_tiles, int n_stages)
{
  return 1024 + static_cast<size_t>(panel_tiles) * kb * kQTileBytes + static_cast<size_t>(n_stages) * kb * kBTileBytes +
         static_cast<size_t>(n_stages) * kBaseTile * 4 + kEpiWarps * kRecBuf * 8 + sizeof(SharedCtl) + 64;
}

namespace {
long long* g_trace = nullptr;
int g_trace_units  = 0;
}  // namespace

void screen_set_trace(long long* trace, int units) { g_trace = trace, g_trace_units = trace ? units : 0; }
bool screen_trace_compiled() { return CERTEX_SCREEN_TRACE != 0; }

cudaError_t screen_i8_launch(const CUtensorMap& tm_q, const CUtensorMap& tm_x, const ScreenArgs& args_in, int grid, cudaStream_t stream)
{
  ScreenArgs args  = args_in;
  args.trace       = g_trace;
  args.trace_units = g_trace_units;
  const size_t smem = args.wide ? screen_smem_bytes_wide() : screen_smem_bytes(args.kb, args.panel_tiles, args.n_stages);
  // opt-in to large dynamic shared memory (cheap; set on every launch so that every device of the process has it)
  if (!args.wide && args.kb != 1 && args.kb != 2) { return cudaErrorInvalidValue; }
  const bool kb2 = args.kb == 2;
  auto kernel    = kb2 ? screen_i8_kernel<kModeRate, false, false, 2> : screen_i8_kernel<kModeRate, false, false, 1>;
  if (args.mode == kModeRate) {
    if (args.wide) { return cudaErrorInvalidValue; }
  } else if (args.mode == kModeScreen) {
    kernel = args.wide ? (args.f16 ? screen_i8_kernel<kModeScreen, true, true, 0> : screen_i8_kernel<kModeScreen, false, true, 0>)
             : args.f16 ? (kb2 ? screen_i8_kernel<kModeScreen, true, false, 2> : screen_i8_kernel<kModeScreen, true, false, 1>)
                        : (kb2 ? screen_i8_kernel<kModeScreen, false, false, 2> : screen_i8_kernel<kModeScreen, false, false, 1>);
  } else if (args.mode == kModeGroupBound) {
    kernel = args.wide ? (args.f16 ? screen_i8_kernel<kModeGroupBound, true, true, 0> : screen_i8_kernel<kModeGroupBound, false, true, 0>)
             : args.f16 ? (kb2 ? screen_i8_kernel<kModeGroupBound, true, false, 2> : screen_i8_kernel<kModeGroupBound, true, false, 1>)
                        : (kb2 ? screen_i8_kernel<kModeGroupBound, false, false, 2> : screen_i8_kernel<kModeGroupBound, false, false, 1>);
  } else {
    kernel = args.wide ? (args.f16 ? screen_i8_kernel<kModeGroupMax, true, true, 0> : screen_i8_kernel<kModeGroupMax, false, true, 0>)
             : args.f16 ? (kb2 ? screen_i8_kernel<kModeGroupMax, true, false, 2> : screen_i8_kernel<kModeGroupMax, true, false, 1>)
                        : (kb2 ? screen_i8_kernel<kModeGroupMax, false, false, 2> : screen_i8_kernel<kModeGroupMax, false, false, 1>);
  }
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
  if (e != cudaSuccess) { return e; }
  kernel<<<grid, kThreads, smem, stream>>>(tm_q, tm_x, args);
  return cudaGetLastError();
}

}  // namespace certex_b200
