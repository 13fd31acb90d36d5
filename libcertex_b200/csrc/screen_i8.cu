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
constexpr int kSharedSegs = 64;                // segments of a CTA (a CTA is never given more)

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
  ScreenSeg segs[kSharedSegs];
};

// Position in the CTA's unit sequence: for every base tile of a segment, the query tiles of the segment's panel.
struct Cursor {
  int s, t, j, ts, nqt, t1, q_tile0, col0;
  bool valid;
};

template <bool COL0>
__device__ __forceinline__ void cursor_seg(Cursor& c, const ScreenSeg* segs, const int* seg_col0, int nseg)
{
  c.valid = c.s < nseg;
  if (c.valid) {
    const ScreenSeg sg = segs[c.s];
    c.t                = sg.t0;
    c.t1               = sg.t1;
    c.nqt              = sg.n_qtiles;
    c.q_tile0          = sg.q_tile0;
    if (COL0) { c.col0 = seg_col0 ? seg_col0[c.s] : 0; }
  }
}

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
__device__ __forceinline__ int max32_plus(const int32_t (&v)[32], const int32_t* e)
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

__device__ __forceinline__ float max32f_plus(const int32_t (&v)[32], const int32_t* e)
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
    nseg = min(p.seg_begin[blockIdx.x + 1] - seg_first, kSharedSegs);
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
  constexpr bool kNeedE    = MODE == kModeGroupMax;   // only the group maxima need the exact e of every row
  constexpr bool kStageE   = kNeedE && !WIDE;          // resident panel: e travels with the stage; WIDE: in its own ring

  const ScreenSeg* segs = ctl->segs;
  if (threadIdx.x < nseg) { ctl->segs[threadIdx.x] = gsegs[threadIdx.x]; }
  if (threadIdx.x == 0) {
    for (int i = 0; i < ns; ++i) {
      mbar_init(smem_u32(&ctl->full[i]), 1);
      mbar_init(smem_u32(&ctl->empty[i]), kStageE ? 1 + kEpiWarps : 1);
    }
    for (int i = 0; i < kSlots; ++i) {
      mbar_init(smem_u32(&ctl->tmem_full[i]), 1);
      mbar_init(smem_u32(&ctl->tmem_empty[i]), kEpiWarps);
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
        const int c0       = (kNeedE && seg_col0) ? seg_col0[s] : 0;
        const int stp      = (kNeedE && seg_step) ? seg_step[s] : 1;
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
            if (MODE == kModeGroupMax && !p.plain_tiles) {
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
        const int c0  = (kNeedE && seg_col0) ? seg_col0[s] : 0;
        const int stp = (kNeedE && seg_step) ? seg_step[s] : 1;
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
            if (MODE == kModeGroupMax && !p.plain_tiles) {
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
                ok = mbar_wait(tempty_bar0 + slot * 8, ((gu >> 1) & 1u) ^ 1u, abort_flag, p.err, 5);
                if (!ok) { break; }
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

    Cursor cur;
    cur.s = 0, cur.j = 0, cur.ts = 0, cur.col0 = 0;
    cursor_seg<MODE == kModeGroupMax>(cur, segs, seg_col0, nseg);
    int gu  = 0;
    bool ok = true;

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

    // Everything between a unit's completion and the release of its slot sits on the path that bounds the pass (two
    // slots: the MMAs of the next unit but one wait for it): the loads of the query's threshold and of the chain maxima
    // of e are issued before the wait and their values are not touched until the slot is released.
    const uint32_t taddr0     = tmem + lane_base + static_cast<uint32_t>(piece * kGroupRows);
    const uint32_t tfull_bar0 = smem_u32(&ctl->tmem_full[0]), tempty_bar0 = smem_u32(&ctl->tmem_empty[0]);
    while (ok && cur.valid) {
      const uint32_t slot = static_cast<uint32_t>(gu) & 1u;
      const int q         = (cur.q_tile0 + cur.j) * kQueryTile + row;
      int thr             = F16 ? __float_as_int(CUDART_INF_F) : 0x7fffffff;  // float bits when F16
      int4 ce             = make_int4(0, 0, 0, 0);
      if (MODE == kModeScreen) {
        if (q < p.nq) { thr = __ldg(p.thr + q); }
        // the four chain maxima of e for this warp's piece (one address per warp)
        ce = __ldg(reinterpret_cast<const int4*>(p.cmax + static_cast<size_t>(cur.t) * (kBaseTile / kChainRows)) + piece);
      }
      if (!mbar_wait(tfull_bar0 + slot * 8, (static_cast<uint32_t>(gu) >> 1) & 1u, abort_flag, p.err, 7)) { break; }
      tc_fence_after();
      const uint32_t taddr = taddr0 + slot * kBaseTile;
      int32_t a[32], b[32];
      tmem_ld32(taddr, a);
      tmem_ld32(taddr + 32, b);
      tmem_wait_ld(a);
      reg_fence32(b);
      // the piece is in registers: the slot goes back to the MMA warp
      tc_fence_before();
      __syncwarp();
      if (lane == 0) { mbar_arrive(tempty_bar0 + slot * 8); }

      if (MODE == kModeScreen) {
        bool h0, h1, h2, h3;
        if (F16) {
          const float tf = __int_as_float(thr);
          h0 = max16f(a) + __int_as_float(ce.x) >= tf;
          h1 = max16f(a + 16) + __int_as_float(ce.y) >= tf;
          h2 = max16f(b) + __int_as_float(ce.z) >= tf;
          h3 = max16f(b + 16) + __int_as_float(ce.w) >= tf;
        } else {
          // thr and ce are first used here, long after their loads were issued: a use before the wait would stall the
          // warp on the load latency in front of the slot's release
          h0 = max16(a) + ce.x >= thr;
          h1 = max16(a + 16) + ce.y >= thr;
          h2 = max16(b) + ce.z >= thr;
          h3 = max16(b + 16) + ce.w >= thr;
        }
        if (__any_sync(0xffffffffu, h0 | h1 | h2 | h3)) {
          const int64_t row0 = static_cast<int64_t>(cur.t) * kBaseTile + piece * kGroupRows;
          if (h0) { record(a, thr, ce.x, q, row0); }
          if (h1) { record(a + 16, thr, ce.y, q, row0 + 16); }
          if (h2) { record(b, thr, ce.z, q, row0 + 32); }
          if (h3) { record(b + 16, thr, ce.w, q, row0 + 48); }
          __syncwarp();
          const int staged = min(*rec_n, kRecBuf);
          if (staged > kRecBuf / 2) { flush(staged); }
        }
      } else {
        // exact group maximum: e of the tile was staged with it
        const int er = WIDE ? cur.ts % kERing : cur.ts % ns;
        if (!mbar_wait(WIDE ? smem_u32(&ctl->e_full[er]) : smem_u32(&ctl->full[er]), (cur.ts / (WIDE ? kERing : ns)) & 1,
                       abort_flag, p.err, 6)) {
          break;
        }
        const int32_t* e = init_smem + er * kBaseTile + piece * kGroupRows;
        if (p.fine_groups) {
          // one maximum per chain of 16 rows: four times as many groups, for labels too small for 2k groups of 64
          int4 m4;
          if (F16) {
            m4.x = float_key(max16f_plus(a, e));
            m4.y = float_key(max16f_plus(a + 16, e + 16));
            m4.z = float_key(max16f_plus(b, e + 32));
            m4.w = float_key(max16f_plus(b + 16, e + 48));
          } else {
            m4.x = max16_plus(a, e);
            m4.y = max16_plus(a + 16, e + 16);
            m4.z = max16_plus(b, e + 32);
            m4.w = max16_plus(b + 16, e + 48);
          }
          if (q < p.nq) {
            *reinterpret_cast<int4*>(p.gmax + static_cast<size_t>(q) * p.ld_gmax +
                                     (cur.t - cur.col0) * (kBaseTile / kChainRows) + piece * 4) = m4;
          }
        } else {
          const int m = F16 ? float_key(fmaxf(max32f_plus(a, e), max32f_plus(b, e + 32)))
                            : max(max32_plus(a, e), max32_plus(b, e + 32));
          if (q < p.nq) {
            p.gmax[static_cast<size_t>(q) * p.ld_gmax + (cur.t - cur.col0) * (kBaseTile / kGroupRows) + piece] = m;
          }
        }
      }
      // next unit; a finished tile's e values are released (GROUPMAX)
      ++gu;
      if (++cur.j == cur.nqt) {
        cur.j = 0;
        if (kNeedE) {
          __syncwarp();
          if (lane == 0) { mbar_arrive(WIDE ? smem_u32(&ctl->e_empty[cur.ts % kERing]) : smem_u32(&ctl->empty[cur.ts % ns])); }
        }
        ++cur.ts;
        if (++cur.t == cur.t1) {
          ++cur.s;
          cursor_seg<MODE == kModeGroupMax>(cur, segs, seg_col0, nseg);
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

cudaError_t screen_i8_launch(const CUtensorMap& tm_q, const CUtensorMap& tm_x, const ScreenArgs& args, int grid, cudaStream_t stream)
{
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
