// Thin inline-PTX wrappers for the sm_100a features the kernels use: mbarrier, TMA (cp.async.bulk[.tensor], every load
// for the issuing CTA alone), tensor memory (tcgen05.alloc/ld) and the fifth-generation tensor-core MMA
// (tcgen05.mma / tcgen05.commit). Every wait in here is bounded; see `mbar_wait`.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace certex_b200 {
namespace ptx {

__device__ __forceinline__ uint32_t smem_u32(const void* p)
{
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// ---------------------------------------------------------------- mbarrier
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count)
{
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}

__device__ __forceinline__ void fence_barrier_init()
{
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void fence_proxy_async()
{
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar)
{
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes)
{
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}

/// One try_wait. The thread is suspended by the hardware until the phase completes or `kSuspendNs` have passed, so a
/// waiting warp does not compete for issue slots with the warps that have work.
constexpr uint32_t kSuspendNs = 200000;
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity)
{
  uint32_t ok;
  asm volatile(
    "{\n\t"
    ".reg .pred p;\n\t"
    "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
    "selp.b32 %0, 1, 0, p;\n\t"
    "}\n"
    : "=r"(ok)
    : "r"(bar), "r"(parity), "r"(kSuspendNs)
    : "memory");
  return ok != 0;
}

/// Cycles a wait may last before the kernel gives up (about two seconds at 2 GHz).
constexpr long long kWaitLimitCycles = 1ll << 32;

/**
 * Bounded wait on an mbarrier phase. Returns false when the CTA is aborting: either this wait ran out of time (it then
 * raises `*abort_flag` and records `code` in `*err`), or another thread of the CTA raised the flag. Callers leave their
 * loops on false and fall through to the common teardown.
 */
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* err, int code)
{
  if (mbar_try_wait(bar, parity)) { return true; }
  const long long t0 = clock64();
  while (true) {
    if (mbar_try_wait(bar, parity)) { return true; }
    if (*abort_flag) { return false; }
    if (clock64() - t0 > kWaitLimitCycles) {
      *abort_flag = 1;
      atomicCAS(err, 0, code);
      return false;
    }
  }
}

// ---------------------------------------------------------------- TMA
__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap* m)
{
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(m)) : "memory");
}

/// 2-D tiled load global -> this CTA's shared memory; completion is signalled on `bar` as transaction bytes.
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* m, int32_t x, int32_t y, uint32_t bar)
{
  asm volatile(
    "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
    :
    : "r"(dst), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar), "r"(x), "r"(y)
    : "memory");
}

/// 3-D tiled load (same shared-memory layout as the 2-D load of the box's two inner dimensions).
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* m, int32_t x, int32_t y, int32_t z, uint32_t bar)
{
  asm volatile(
    "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
    :
    : "r"(dst), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar), "r"(x), "r"(y), "r"(z)
    : "memory");
}

/// 4-D tiled load (the box's inner dimensions laid out in shared memory like the 2-D load's rows).
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* m, int32_t x, int32_t y, int32_t z, int32_t w,
                                            uint32_t bar)
{
  asm volatile(
    "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
    :
    : "r"(dst), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar), "r"(x), "r"(y), "r"(z), "r"(w)
    : "memory");
}

/// 1-D bulk copy global -> shared; both addresses 16-byte aligned, `bytes` a multiple of 16.
__device__ __forceinline__ void bulk_load_1d(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar)
{
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               :
               : "r"(dst), "l"(reinterpret_cast<uint64_t>(src)), "r"(bytes), "r"(bar)
               : "memory");
}

// ---------------------------------------------------------------- tensor memory
__device__ __forceinline__ void tmem_alloc(uint32_t smem_dst, uint32_t ncols)
{
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(ncols)
               : "memory");
}

__device__ __forceinline__ void tmem_relinquish()
{
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols)
{
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

/// mbarrier arrive once every tcgen05 operation this thread issued so far has completed.
__device__ __forceinline__ void tc_commit(uint32_t bar)
{
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

/// D[tmem] (+)= A[smem] * B[smem]^T, 8-bit integer operands, int32 accumulate.
__device__ __forceinline__ void mma_i8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t acc)
{
  asm volatile(
    "{\n\t"
    ".reg .pred p;\n\t"
    "setp.ne.b32 p, %4, 0;\n\t"
    "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t"
    "}\n"
    :
    : "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(acc)
    : "memory");
}

/// Same for fp16 operands (K = 16 elements = 32 bytes per instruction) with fp32 accumulate.
__device__ __forceinline__ void mma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t acc)
{
  asm volatile(
    "{\n\t"
    ".reg .pred p;\n\t"
    "setp.ne.b32 p, %4, 0;\n\t"
    "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
    "}\n"
    :
    : "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(acc)
    : "memory");
}

/// The same instructions with the accumulate flag fixed at compile time (no predicate register to set up): the
/// issuing thread's instruction count per MMA is what bounds the rate of short-K units.
template <bool ACC>
__device__ __forceinline__ void mma_i8_c(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc)
{
  asm volatile(
    "{\n\t"
    ".reg .pred p;\n\t"
    "setp.ne.b32 p, %4, 0;\n\t"
    "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t"
    "}\n"
    :
    : "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "n"(ACC ? 1 : 0)
    : "memory");
}

template <bool ACC>
__device__ __forceinline__ void mma_f16_c(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc)
{
  asm volatile(
    "{\n\t"
    ".reg .pred p;\n\t"
    "setp.ne.b32 p, %4, 0;\n\t"
    "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
    "}\n"
    :
    : "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "n"(ACC ? 1 : 0)
    : "memory");
}

/// A 64-bit descriptor from its two words (a register pair: no instruction when the halves sit in place).
__device__ __forceinline__ uint64_t pack64(uint32_t lo, uint32_t hi)
{
  uint64_t d;
  asm("mov.b64 %0, {%1, %2};" : "=l"(d) : "r"(lo), "r"(hi));
  return d;
}

/// a - b, saturating at the int32 limits.
__device__ __forceinline__ int sub_sat(int a, int b)
{
  int r;
  asm("sub.sat.s32 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  return r;
}

/**
 * Shared-memory matrix descriptor of a K-major operand tile stored as rows of 128 bytes with the 128-byte swizzle
 * (what a TMA box of 128 bytes x rows with CU_TENSOR_MAP_SWIZZLE_128B writes): 8-row groups are 1024 bytes apart
 * (stride byte offset), the leading byte offset is unused for swizzled K-major layouts and set to 1, descriptor
 * version 1 (sm_100), layout type 2 (SWIZZLE_128B). `addr` must lie in a 1024-byte aligned tile; a K step inside the
 * 128-byte row advances `addr` by its byte offset.
 */
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t addr)
{
  uint64_t d = 0;
  d |= static_cast<uint64_t>((addr & 0x3FFFFu) >> 4);
  d |= static_cast<uint64_t>(1) << 16;
  d |= static_cast<uint64_t>(1024 >> 4) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(2) << 61;
  return d;
}

/// Instruction descriptor: dense, K-major A and B, accumulator format c (1 = f32, 2 = s32), operand formats
/// (i8 kinds: 0 = u8, 1 = s8; f16 kinds: 0 = f16, 1 = bf16), M x N tile.
__host__ __device__ constexpr uint32_t instr_desc(uint32_t c_fmt, uint32_t a_fmt, uint32_t b_fmt, uint32_t m, uint32_t n)
{
  return (c_fmt << 4) | (a_fmt << 7) | (b_fmt << 10) | ((n >> 3) << 17) | ((m >> 4) << 24);
}

// 32 lanes x 32-bit, 32 consecutive columns per thread.
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, int32_t (&v)[32])
{
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
               : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
               : "r"(taddr)
               : "memory");
}

/// tcgen05.wait::ld that also names the 32 destination registers of a load as read-write operands, so that the
/// compiler cannot move a use of them above the wait.
__device__ __forceinline__ void tmem_wait_ld(int32_t (&v)[32])
{
  asm volatile("tcgen05.wait::ld.sync.aligned;" : "+r"(v[0]), "+r"(v[1]), "+r"(v[2]), "+r"(v[3]), "+r"(v[4]), "+r"(v[5]), "+r"(v[6]), "+r"(v[7]), "+r"(v[8]), "+r"(v[9]), "+r"(v[10]), "+r"(v[11]), "+r"(v[12]), "+r"(v[13]), "+r"(v[14]), "+r"(v[15]), "+r"(v[16]), "+r"(v[17]), "+r"(v[18]), "+r"(v[19]), "+r"(v[20]), "+r"(v[21]), "+r"(v[22]), "+r"(v[23]), "+r"(v[24]), "+r"(v[25]), "+r"(v[26]), "+r"(v[27]), "+r"(v[28]), "+r"(v[29]), "+r"(v[30]), "+r"(v[31]) : : "memory");
}

/// Compiler-only fence on 32 registers (no instruction): placed after a wait, it keeps uses of `v` below the wait.
__device__ __forceinline__ void reg_fence32(int32_t (&v)[32])
{
  asm volatile("" : "+r"(v[0]), "+r"(v[1]), "+r"(v[2]), "+r"(v[3]), "+r"(v[4]), "+r"(v[5]), "+r"(v[6]), "+r"(v[7]), "+r"(v[8]), "+r"(v[9]), "+r"(v[10]), "+r"(v[11]), "+r"(v[12]), "+r"(v[13]), "+r"(v[14]), "+r"(v[15]), "+r"(v[16]), "+r"(v[17]), "+r"(v[18]), "+r"(v[19]), "+r"(v[20]), "+r"(v[21]), "+r"(v[22]), "+r"(v[23]), "+r"(v[24]), "+r"(v[25]), "+r"(v[26]), "+r"(v[27]), "+r"(v[28]), "+r"(v[29]), "+r"(v[30]), "+r"(v[31]) : : "memory");
}

}  // namespace ptx
}  // namespace certex_b200
