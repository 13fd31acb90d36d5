// Interface of the integer tensor-core screening pass (see screen_i8.cu).
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace certex_b200 {

constexpr int kMaxSegs   = 4;  // segments (query panel, base-tile range) one CTA may be given
constexpr int kMaxStages = 8;  // upper bound of the base-tile ring

enum : int { kModeScreen = 0, kModeGroupMax = 1 };

/// Init value of a column that must never pass a threshold (removed rows, padding beyond the last row).
constexpr int32_t kNeverInit = -(1 << 30);

/// One contiguous piece of work of a CTA: query tiles [q_tile0, q_tile0 + n_qtiles) against base tiles [t0, t1).
struct ScreenSeg {
  int q_tile0;
  int n_qtiles;
  int t0;
  int t1;
};

struct ScreenArgs {
  const int32_t* init;    // [n_tiles * 128] initial accumulator of every column (16-byte aligned)
  const int32_t* thr;     // SCREEN: [nq] keep iff acc >= thr[q]
  int32_t* gmax;          // GROUPMAX: [nq, ld_gmax] maximum of every 128-column group
  int64_t ld_gmax;
  uint32_t* cnt;          // SCREEN: [nq] candidates found (may exceed cap: overflow)
  int32_t* cand;          // SCREEN: [nq, cap] candidate rows
  uint32_t cap;
  int nq;
  int n_rows;             // rows >= n_rows are padding
  int kb;                 // K blocks of 128 bytes per row
  int panel_tiles;        // query tiles resident in shared memory
  int n_stages;           // base-tile ring depth
  int mode;
  uint32_t q_signed;      // 0 = uint8 codes, 1 = int8 codes
  uint32_t x_signed;
  const ScreenSeg* segs;  // [grid, kMaxSegs]; unused entries have t1 <= t0
  int* err;               // set to a non-zero code when a bounded wait gave up
};

size_t screen_smem_bytes(int kb, int panel_tiles, int n_stages);

cudaError_t screen_i8_launch(const CUtensorMap& tm_q, const CUtensorMap& tm_x, const ScreenArgs& args, int grid, cudaStream_t stream);

}  // namespace certex_b200
