// Integer screening pass on the sm_100a tensor cores.
//
// For 8-bit vectors the Gram product <q, x> is exact in int32, so the lower bound that the screen tests is the exact
// squared distance itself (or the exact inner-product score): nothing is lost to rounding and the verification stage
// only re-derives the survivors' scores in fp64 and breaks ties. The pass replaces the reference's `screen_int8`
// (cpp/src/neighbors/certex/detail/kernels.hpp:290-304, kernel cpp/src/neighbors/certex/detail/screen_int8.cu:99-229,
// an mma.sync kernel) and, in its second mode, the anchor pass `anchor_groups`
// (cpp/src/neighbors/certex/detail/kernels.hpp:125-135).
//
// One accumulator unit is 128 queries (TMEM lanes) x 128 stored rows (TMEM columns), K = 128 bytes per K block.
//   acc[q][x] = init[x] + <q, x>        init[x] = -floor(|x|^2 / 2) for L2, 0 for inner product, -2^30 for removed rows
// The per-row term is not added in the epilogue: the epilogue threads write init[] into the accumulator columns with
// tcgen05.st before the MMA of that unit starts, and every MMA accumulates onto it. The epilogue is then one running
// maximum per thread (3-input integer max) and one compare per 64 columns:
//   SCREEN    keep (q, x) iff acc >= thr[q]; survivors are appended to the per-query candidate list
//   GROUPMAX  gmax[q][tile] = max over the 128 columns (the k-th largest group maximum of a query is its threshold:
//             k distinct stored rows are at least that close)
//
// CTA = 10 warps: warp 0 lane 0 issues TMA loads (queries panel once per segment, base tiles through a ring of
// stages), warp 1 lane 0 issues tcgen05.mma, warps 2..9 are two epilogue groups of four warps (one per TMEM lane
// quarter) that take alternate units. TMEM holds four accumulator slots of 128 columns, so the MMA runs up to three
// units ahead of the epilogue. No cluster launch, no multicast: each CTA loads its own tiles from its GPU's memory.
#include "screen_i8.cuh"

#include "ptx.cuh"

namespace certex_b200 {

namespace {

using namespace ptx;

constexpr int kTileRows  = 128;
constexpr int kTileBytes = 128 * 128;  // one K block of one tile: 128 rows x 128 bytes
constexpr int kSlots     = 4;          // TMEM accumulator slots (4 x 128 columns = all 512)
constexpr int kThreads   = 320;

// Walks the CTA's units in issue order: for every base tile of a segment, the query tiles of the segment's panel.
struct Walker {
  const ScreenSeg* segs;
  int nseg;
  int s;     // segment
  int tile;  // base tile (absolute)
  int j;     // query tile inside the panel
  int ts;    // base tiles started before this one (ring position)
  bool valid;

  __device__ void init(const ScreenSeg* sg, int n)
  {
    segs  = sg;
    nseg  = n;
    s     = 0;
    j     = 0;
    ts    = 0;
    valid = n > 0;
    tile  = valid ? sg[0].t0 : 0;
  }
  __device__ void step()
  {
    if (!valid) { return; }
    if (++j == segs[s].n_qtiles) {
      j = 0;
      ++ts;
      if (++tile == segs[s].t1) {
        if (++s == nseg) {
          valid = false;
        } else {
          tile = segs[s].t0;
        }
      }
    }
  }
  __device__ void advance(int n)
  {
    for (int i = 0; i < n; ++i) { step(); }
  }
};

struct SharedCtl {
  uint64_t full[kMaxStages];
  uint64_t empty[kMaxStages];
  uint64_t tmem_full[kSlots];
  uint64_t tmem_ready[kSlots];
  uint64_t panel_full;
  uint64_t panel_empty;
  uint64_t drain;
  uint32_t tmem_base;
  int abort_flag;
  ScreenSeg segs[kMaxSegs];
};

__device__ __forceinline__ int max3(int a, int b, int c) { return __vimax3_s32(a, b, c); }

template <int N>
__device__ __forceinline__ int max_of(const int32_t (&v)[N])
{
  int m = max3(v[0], v[1], v[2]);
#pragma unroll
  for (int i = 3; i + 1 < N; i += 2) { m = max3(m, v[i], v[i + 1]); }
  if constexpr ((N - 3) % 2 == 1) { m = max(m, v[N - 1]); }
  return m;
}

template <int N>
__device__ __forceinline__ void emit_survivors(
  const int32_t (&v)[N], int thr, int q, int row0, int n_rows, uint32_t* cnt, int32_t* cand, uint32_t cap)
{
#pragma unroll
  for (int i = 0; i < N; ++i) {
    if (v[i] >= thr && row0 + i < n_rows) {
      const uint32_t pos = atomicAdd(cnt + q, 1u);
      if (pos < cap) { cand[static_cast<size_t>(q) * cap + pos] = row0 + i; }
    }
  }
}

__global__ void __launch_bounds__(kThreads, 1) screen_i8_kernel(const __grid_constant__ CUtensorMap tm_q,
                                                                const __grid_constant__ CUtensorMap tm_x,
                                                                const ScreenArgs p)
{
  extern __shared__ uint8_t smem_raw[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  const ScreenSeg* gsegs = p.segs + static_cast<size_t>(blockIdx.x) * kMaxSegs;
  int nseg               = 0;
  while (nseg < kMaxSegs && gsegs[nseg].t1 > gsegs[nseg].t0) { ++nseg; }
  if (nseg == 0) { return; }  // uniform over the CTA

  // ---- shared memory carve-up (1024-byte aligned tiles for the 128-byte swizzle)
  const uint32_t base      = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* gen_base        = smem_raw + (base - smem_u32(smem_raw));
  const int kb             = p.kb;
  const uint32_t panel_off = 0;
  const uint32_t stage_off = panel_off + static_cast<uint32_t>(p.panel_tiles) * kb * kTileBytes;
  const uint32_t init_off  = stage_off + static_cast<uint32_t>(p.n_stages) * kb * kTileBytes;
  const uint32_t ctl_off   = init_off + static_cast<uint32_t>(p.n_stages) * kTileRows * 4;
  SharedCtl* ctl           = reinterpret_cast<SharedCtl*>(gen_base + ctl_off);
  const int32_t* init_smem = reinterpret_cast<const int32_t*>(gen_base + init_off);
  volatile int* abort_flag = &ctl->abort_flag;
  const int ns             = p.n_stages;

  const ScreenSeg* segs = ctl->segs;
  if (threadIdx.x < kMaxSegs) { ctl->segs[threadIdx.x] = gsegs[threadIdx.x]; }
  if (threadIdx.x == 0) {
    for (int i = 0; i < ns; ++i) {
      mbar_init(smem_u32(&ctl->full[i]), 1);
      mbar_init(smem_u32(&ctl->empty[i]), 1);
    }
    for (int i = 0; i < kSlots; ++i) {
      mbar_init(smem_u32(&ctl->tmem_full[i]), 1);
      mbar_init(smem_u32(&ctl->tmem_ready[i]), 4);  // one arrival per warp of an epilogue group
    }
    mbar_init(smem_u32(&ctl->panel_full), 1);
    mbar_init(smem_u32(&ctl->panel_empty), 1);
    mbar_init(smem_u32(&ctl->drain), 1);
    ctl->abort_flag = 0;
    fence_barrier_init();
    prefetch_tensormap(&tm_q);
    prefetch_tensormap(&tm_x);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&ctl->tmem_base), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = ctl->tmem_base;

  if (warp == 0) {
    // ================================================================ TMA producer
    if (lane == 0) {
      int ts       = 0;
      bool aborted = false;
      for (int s = 0; s < nseg && !aborted; ++s) {
        const ScreenSeg sg = segs[s];
        if (s > 0 && !mbar_wait(smem_u32(&ctl->panel_empty), (s - 1) & 1, abort_flag, p.err, 1)) { break; }
        const uint32_t pbar = smem_u32(&ctl->panel_full);
        mbar_arrive_expect_tx(pbar, static_cast<uint32_t>(sg.n_qtiles) * kb * kTileBytes);
        for (int j = 0; j < sg.n_qtiles; ++j) {
          for (int b = 0; b < kb; ++b) {
            tma_load_2d(base + panel_off + (j * kb + b) * kTileBytes, &tm_q, b * 128, (sg.q_tile0 + j) * kTileRows, pbar);
          }
        }
        for (int t = sg.t0; t < sg.t1; ++t, ++ts) {
          const int st = ts % ns;
          if (ts >= ns && !mbar_wait(smem_u32(&ctl->empty[st]), ((ts / ns) - 1) & 1, abort_flag, p.err, 2)) {
            aborted = true;
            break;
          }
          const uint32_t fbar = smem_u32(&ctl->full[st]);
          mbar_arrive_expect_tx(fbar, static_cast<uint32_t>(kb) * kTileBytes + kTileRows * 4);
          for (int b = 0; b < kb; ++b) {
            tma_load_2d(base + stage_off + (st * kb + b) * kTileBytes, &tm_x, b * 128, t * kTileRows, fbar);
          }
          bulk_load_1d(base + init_off + st * kTileRows * 4, p.init + static_cast<size_t>(t) * kTileRows, kTileRows * 4, fbar);
        }
      }
      if (*abort_flag) {
        // let the copies that are still in flight land before the CTA leaves (bounded)
        for (int back = 1; back <= ns && back <= ts; ++back) {
          const int u         = ts - back;
          const long long t0  = clock64();
          while (!mbar_try_wait(smem_u32(&ctl->full[u % ns]), (u / ns) & 1) && clock64() - t0 < (1ll << 24)) {}
        }
      }
    }
  } else if (warp == 1) {
    // ================================================================ MMA issuer
    if (lane == 0) {
      const uint32_t idesc = instr_desc(2u, p.q_signed, p.x_signed, 128u, 128u);
      Walker w;
      w.init(segs, nseg);
      int gu = 0, cur_seg = -1;
      while (w.valid) {
        if (w.s != cur_seg) {
          cur_seg = w.s;
          if (!mbar_wait(smem_u32(&ctl->panel_full), cur_seg & 1, abort_flag, p.err, 3)) { break; }
        }
        const int st = w.ts % ns, slot = gu & (kSlots - 1);
        if (w.j == 0 && !mbar_wait(smem_u32(&ctl->full[st]), (w.ts / ns) & 1, abort_flag, p.err, 4)) { break; }
        if (!mbar_wait(smem_u32(&ctl->tmem_ready[slot]), (gu / kSlots) & 1, abort_flag, p.err, 5)) { break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem + static_cast<uint32_t>(slot * kTileRows);
        for (int b = 0; b < kb; ++b) {
          const uint32_t a_addr = base + panel_off + (w.j * kb + b) * kTileBytes;
          const uint32_t b_addr = base + stage_off + (st * kb + b) * kTileBytes;
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            mma_i8(d_tmem, smem_desc_sw128(a_addr + k * 32), smem_desc_sw128(b_addr + k * 32), idesc, 1u);
          }
        }
        tc_commit(smem_u32(&ctl->tmem_full[slot]));
        const bool last_q    = w.j == segs[w.s].n_qtiles - 1;
        const bool last_tile = last_q && w.tile == segs[w.s].t1 - 1;
        if (last_q) { tc_commit(smem_u32(&ctl->empty[st])); }
        if (last_tile) { tc_commit(smem_u32(&ctl->panel_empty)); }
        w.step();
        ++gu;
      }
      // every MMA issued above has completed before TMEM is released
      tc_commit(smem_u32(&ctl->drain));
      {
        const long long t0 = clock64();
        while (!mbar_try_wait(smem_u32(&ctl->drain), 0) && clock64() - t0 < kWaitLimitCycles) {}
      }
    }
  } else {
    // ================================================================ epilogue (two groups of four warps)
    const int ew = warp - 2, group = ew >> 2;
    const int quarter        = warp & 3;  // the TMEM lane quarter this warp may access
    const int row            = quarter * 32 + lane;
    const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;

    // Writes init[] of the unit's base tile into the unit's accumulator slot and hands the slot to the MMA warp.
    auto init_slot = [&](const Walker& w, int gu) -> bool {
      const int st = w.ts % ns, slot = gu & (kSlots - 1);
      if (!mbar_wait(smem_u32(&ctl->full[st]), (w.ts / ns) & 1, abort_flag, p.err, 6)) { return false; }
      const int4* src      = reinterpret_cast<const int4*>(init_smem + st * kTileRows);
      const uint32_t taddr = tmem + lane_base + static_cast<uint32_t>(slot * kTileRows);
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        int32_t v[64];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const int4 t = src[h * 16 + i];
          v[4 * i] = t.x, v[4 * i + 1] = t.y, v[4 * i + 2] = t.z, v[4 * i + 3] = t.w;
        }
        tmem_st64(taddr + h * 64, v);
      }
      tmem_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) { mbar_arrive(smem_u32(&ctl->tmem_ready[slot])); }
      return true;
    };

    Walker cur, nxt;
    cur.init(segs, nseg);
    cur.advance(group);
    nxt     = cur;
    int gu  = group, gun = group;
    bool ok = true;
    for (int i = 0; i < 2 && nxt.valid && ok; ++i) {  // the group's first two units have no predecessor in their slots
      ok = init_slot(nxt, gun);
      nxt.advance(2);
      gun += 2;
    }
    while (ok && cur.valid) {
      const int slot = gu & (kSlots - 1);
      const int q    = (segs[cur.s].q_tile0 + cur.j) * kTileRows + row;
      int thr        = 0x7fffffff;
      if (p.mode == kModeScreen && q < p.nq) { thr = __ldg(p.thr + q); }
      if (!mbar_wait(smem_u32(&ctl->tmem_full[slot]), (gu / kSlots) & 1, abort_flag, p.err, 7)) { break; }
      tc_fence_after();
      const uint32_t taddr = tmem + lane_base + static_cast<uint32_t>(slot * kTileRows);
      int32_t a[64], b[64];
      tmem_ld64(taddr, a);
      tmem_wait_ld(a);
      tmem_ld64(taddr + 64, b);
      const int ma = max_of(a);
      if (p.mode == kModeScreen) {
        if (ma >= thr) { emit_survivors(a, thr, q, cur.tile * kTileRows, p.n_rows, p.cnt, p.cand, p.cap); }
        tmem_wait_ld(b);
        const int mb = max_of(b);
        if (mb >= thr) { emit_survivors(b, thr, q, cur.tile * kTileRows + 64, p.n_rows, p.cnt, p.cand, p.cap); }
      } else {
        tmem_wait_ld(b);
        const int mb = max_of(b);
        if (q < p.nq) { p.gmax[static_cast<size_t>(q) * p.ld_gmax + cur.tile] = max(ma, mb); }
      }
      // the slot has been read: prepare it for the unit that uses it next
      if (nxt.valid) {
        ok = init_slot(nxt, gun);
        nxt.advance(2);
        gun += 2;
      }
      cur.advance(2);
      gu += 2;
    }
  }

  // ---- teardown: all roles meet here, also when a wait gave up
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == 1) { tmem_dealloc(tmem, 512); }
}

}  // namespace

size_t screen_smem_bytes(int kb, int panel_tiles, int n_stages)
{
  return 1024 + static_cast<size_t>(panel_tiles + n_stages) * kb * kTileBytes + static_cast<size_t>(n_stages) * kTileRows * 4 +
         sizeof(SharedCtl) + 64;
}

cudaError_t screen_i8_launch(const CUtensorMap& tm_q, const CUtensorMap& tm_x, const ScreenArgs& args, int grid, cudaStream_t stream)
{
  const size_t smem = screen_smem_bytes(args.kb, args.panel_tiles, args.n_stages);
  // opt-in to large dynamic shared memory (cheap; set on every launch so that every device of the process has it)
  cudaError_t e = cudaFuncSetAttribute(screen_i8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
  if (e != cudaSuccess) { return e; }
  screen_i8_kernel<<<grid, kThreads, smem, stream>>>(tm_q, tm_x, args);
  return cudaGetLastError();
}

}  // namespace certex_b200
