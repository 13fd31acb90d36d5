// Interface of the integer tensor-core screening pass (see screen_i8.cu).
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace certex_b200 {

constexpr int kMaxSegs   = 4;  // segments (query panel, base-tile range) one CTA may be given
constexpr int kMaxStages = 8;  // upper bound of the base-tile ring

constexpr int kQueryTile = 128;  // queries per accumulator unit (TMEM lanes)
constexpr int kBaseTile  = 256;  // stored rows per accumulator unit (TMEM columns, N of one MMA instruction)
constexpr int kGroupRows = 64;   // rows per group maximum (one epilogue warp's piece of a unit)

// kModeRate issues the loads and MMAs of every unit back to back with no epilogue (tensor-pipe rate probe).
// kModeGroupBound is the threshold stage at the screen's price: a tile's 16 chains are 16 adjacent anchors each (the
// 4-D anchor map below), e is taken per chain (its minimum, in `cmax`), and gmax receives per group of 64 columns
//   max over its four chains of (max of <q, x> over the chain + min of e over the chain),
// a value some row of the group reaches (the row with the chain's largest product has at least the chain's smallest e),
// so the k-th largest of them is still reached by k distinct rows. kModeGroupMax is the exact maximum of <q, x> + e.
enum : int { kModeScreen = 0, kModeGroupMax = 1, kModeRate = 2, kModeGroupBound = 3 };

/// Init value of a column that must never pass a threshold (removed rows, padding beyond the last row).
constexpr int32_t kNeverInit = -(1 << 30);

constexpr int kChainRows = 16;  // rows per chain: the unit of the conservative threshold test and of a survivor record

/// One contiguous piece of work of a CTA: query tiles [q_tile0, q_tile0 + n_qtiles) against base tiles [t0, t1)
/// (query tiles of 128 queries, base tiles of 256 rows).
struct ScreenSeg {
  int q_tile0;
  int n_qtiles;
  int t0;
  int t1;
};

/// A survivor record: bits 63..48 query (inside the batch), bits 47..16 chunk = row / 16, bits 15..0 one bit per row
/// of the chunk that reached the query's threshold.
__host__ __device__ inline uint64_t make_record(uint32_t q, uint32_t chunk, uint32_t mask16)
{
  return (static_cast<uint64_t>(q) << 48) | (static_cast<uint64_t>(chunk) << 16) | mask16;
}

struct ScreenArgs {
  const int32_t* init;            // [n_tiles * 256] per-row term e[x] added to <q, x> (kNeverInit: removed / padding)
  const int32_t* cmax;            // SCREEN: [n_tiles * 16] maximum of e over every chain of 16 rows; GROUPBOUND: minimum
  const int32_t* thr;             // SCREEN: [nq] keep iff <q, x> + e[x] >= thr[q]
  int32_t* gmax;                  // GROUPMAX: [nq, ld_gmax] maximum of <q, x> + e[x] over every group of 64 rows
  int64_t ld_gmax;
  uint64_t* rec;                  // SCREEN: survivor records
  unsigned long long* rec_count;  // SCREEN: records appended (may exceed rec_cap: overflow, the excess is not written)
  unsigned long long rec_cap;
  int nq;
  int kb;                         // K blocks of 128 bytes per row
  int panel_tiles;                // query tiles resident in shared memory
  int n_stages;                   // base-tile ring depth
  int mode;
  int f16;                        // 1: fp16 codes, fp32 accumulators; init / cmax / thr hold float bits, gmax float keys
  uint32_t q_signed;              // 0 = uint8 codes, 1 = int8 codes
  uint32_t x_signed;
  const ScreenSeg* segs;          // [grid, kMaxSegs]; unused entries have t1 <= t0. With seg_begin: one list
  const int* seg_begin;           // optional [grid + 1]: CTA b works on segs[seg_begin[b] .. seg_begin[b + 1])
  const int* seg_col0;            // optional, per segment: the tile whose groups are columns 0..3 of gmax (else tile 0)
  const int* seg_step;            // optional, GROUPMAX: tile t of a segment stands for tile col0 + (t - col0) * step
  int wide;                       // 1: rows of more than two K blocks; a segment then has at most two query tiles
  int plain_tiles;                // GROUPMAX: tile t is rows [256 t, 256 t + 256) of a 2-D map (else the 3-D anchor map)
  int fine_groups;                // GROUPMAX: one maximum per 16 rows (16 columns of gmax per tile) instead of per 64 (4)
  int* err;                       // set to a non-zero code when a bounded wait gave up
  long long* trace;               // trace builds only (see screen_set_trace): [trace_units, 12] clock stamps of CTA 0
  int trace_units;
};

size_t screen_smem_bytes(int kb, int panel_tiles, int n_stages);
size_t screen_smem_bytes_wide();

/// Profiling aid, effective only in a library built with -DCERTEX_SCREEN_TRACE=1 (make trace): CTA 0 of every later
/// pass writes SM clock stamps of its first `units` accumulator units to the device buffer `trace` ([units, 12] int64;
/// nullptr: off). The stamps cost time themselves (every instruction on the MMA-issuing thread's and the epilogue's
/// path does): a trace shows where a unit's round trip goes, not how fast the untraced pass is. Process-wide.
void screen_set_trace(long long* trace, int units);
bool screen_trace_compiled();

cudaError_t screen_i8_launch(const CUtensorMap& tm_q, const CUtensorMap& tm_x, const ScreenArgs& args, int grid, cudaStream_t stream);

}  // namespace certex_b200
