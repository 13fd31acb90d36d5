// certexB200SearchStatic: an exact search that performs no device-memory allocation. Everything the dense search
// path needs beyond the caller's inputs and outputs (the fp64 score matrix, the partial and final selection lists)
// lives in one file-scope device array of fixed size, so the call consists of kernel launches only.
//
// Who needs this: a process whose GPU memory has been claimed up front by another allocator (an inference server
// that reserves the whole device at start-up leaves nothing for a later cudaMalloc), and loops with a latency budget
// that cannot absorb the device-wide synchronisation cudaMalloc / cudaFree may imply. Such callers own their input and
// output buffers already; this entry point adds no allocation of its own.
#include "../../include/certex_b200.h"

#include "engine.hpp"
#include "kernels.cuh"

#include <cuda_runtime.h>

#include <mutex>
#include <string>

namespace {

using namespace certex_b200;

constexpr size_t kStaticScratchBytes = size_t(16) << 20;  // CERTEX_B200_STATIC_SCRATCH_BYTES in the public header

// The scratch itself. In host code this name is only a handle for cudaGetSymbolAddress, never a device address.
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

constexpr int kMaxDevices = 64;
std::mutex g_mutex;
void* g_scratch_address[kMaxDevices] = {};  // device address of g_static_scratch on each device, filled on first use

cuvsError_t fail(const std::string& text)
{
  cuvsSetLastErrorText(text.c_str());
  return CUVS_ERROR;
}

size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

}  // namespace

extern "C" cuvsError_t certexB200SearchStatic(cuvsResources_t res, cuvsDistanceType metric, DLDataType dtype,
                                              const void* vectors, int64_t n_rows, const void* queries, int64_t n_queries,
                                              int64_t dim, int32_t k, int64_t* neighbors, float* distances)
{
  if (res == 0 || !vectors || !queries || !neighbors || !distances) { return fail("certex: null argument"); }
  int dt;
  if (dtype.lanes != 1) { return fail("certex: the element type must have one lane"); }
  if (dtype.code == kDLFloat && dtype.bits == 32) {
    dt = kF32;
  } else if (dtype.code == kDLFloat && dtype.bits == 16) {
    dt = kF16;
  } else if (dtype.code == kDLInt && dtype.bits == 8) {
    dt = kI8;
  } else if (dtype.code == kDLUInt && dtype.bits == 8) {
    dt = kU8;
  } else {
    return fail("certex: vectors must be float32, float16, int8, or uint8");
  }
  const int m = metric == L2Expanded ? kL2 : metric == InnerProduct ? kIP : metric == CosineExpanded ? kCos : -1;
  if (m < 0) { return fail("certex: the metric must be L2Expanded, InnerProduct, or CosineExpanded"); }
  if (m == kCos && (dt == kI8 || dt == kU8)) { return fail("certex: the cosine metric needs float32 or float16 vectors"); }
  if (n_rows < 1 || n_queries < 1 || dim < 1 || k < 1 || k > 2048 || k > n_rows) {
    return fail("certex: need n_rows >= k >= 1, k <= 2048, and at least one query");
  }
  // what one launch of the scoring kernel takes; checked before anything is launched, so that a refused call leaves
  // the outputs untouched
  if (dim > kDenseMaxDim) {
    return fail("certex: certexB200SearchStatic takes at most " + std::to_string(kDenseMaxDim) + " dimensions");
  }
  if (n_queries > kDenseMaxQueries || n_rows >= (int64_t(1) << 31)) {
    return fail("certex: certexB200SearchStatic takes at most " + std::to_string(kDenseMaxQueries) +
                " queries and fewer than 2^31 rows per call");
  }
  const size_t row_bytes = static_cast<size_t>(dim) * dtype_size(dt);
  if (row_bytes % 16 != 0 || reinterpret_cast<uintptr_t>(vectors) % 16 != 0) {
    return fail("certex: certexB200SearchStatic needs 16-byte aligned vectors whose rows are a multiple of 16 bytes");
  }
  // layout of the scratch: score matrix | final lists | partial lists of the chunked selection
  const int64_t ld     = (n_rows + 3) / 4 * 4;
  const int parts      = select_topk_parts(n_rows, k);
  const size_t nqk     = static_cast<size_t>(n_queries) * k;
  const size_t o_best  = align_up(static_cast<size_t>(n_queries) * ld * 8, 256);
  const size_t o_row   = align_up(o_best + nqk * 8, 256);
  const size_t o_parts = align_up(o_row + nqk * 4, 256);
  const size_t o_prow  = align_up(o_parts + nqk * parts * 8, 256);
  const size_t total   = o_prow + nqk * parts * 4;
  if (total > kStaticScratchBytes) {
    return fail("certex: certexB200SearchStatic needs " + std::to_string(total) + " bytes of scratch for this call, the fixed "
                "scratch holds " + std::to_string(kStaticScratchBytes) + " (about n_queries * n_rows * 8 bytes must fit)");
  }

  int device = 0;
  cudaError_t e = cudaGetDevice(&device);
  if (e != cudaSuccess) { return fail(std::string("certex: cudaGetDevice: ") + cudaGetErrorString(e)); }
  if (device < 0 || device >= kMaxDevices) { return fail("certex: device ordinal out of range"); }
  // the scratch address is the current device's, the stream is the resources': they must be the same device
  const int res_device = reinterpret_cast<const Resources*>(res)->device;
  if (res_device != device) {
    return fail("certex: certexB200SearchStatic was called with device " + std::to_string(device) +
                " current, but the resources were created on device " + std::to_string(res_device));
  }
  unsigned char* scratch = nullptr;
  {
    // first call on this device: ask the runtime where this device keeps the array (the device must be current)
    std::lock_guard<std::mutex> lock(g_mutex);
    if (g_scratch_address[device] == nullptr) {
      void* p = nullptr;
      e       = cudaGetSymbolAddress(&p, g_static_scratch);
      if (e != cudaSuccess || p == nullptr) {
        return fail(std::string("certex: cudaGetSymbolAddress of the static scratch failed: ") + cudaGetErrorString(e));
      }
      g_scratch_address[device] = p;
    }
    scratch = static_cast<unsigned char*>(g_scratch_address[device]);
  }

  cudaStream_t stream = nullptr;
  {
    void* s = nullptr;
    if (cuvsStreamGet(res, &s) != CUVS_SUCCESS) { return CUVS_ERROR; }
    stream = static_cast<cudaStream_t>(s);
  }
  double* scores    = reinterpret_cast<double*>(scratch);
  double* best_s    = reinterpret_cast<double*>(scratch + o_best);
  int32_t* best_row = reinterpret_cast<int32_t*>(scratch + o_row);
  double* part_s    = reinterpret_cast<double*>(scratch + o_parts);
  int32_t* part_row = reinterpret_cast<int32_t*>(scratch + o_prow);
  // Every element that a later kernel reads is written by an earlier kernel of this call (scores for all n_rows
  // columns, both lists in full), so nothing has to be cleared although the array keeps the previous call's contents.
  const Admit everything{};
  cudaGetLastError();  // an error left by earlier work of the thread is not this call's
  auto launched = [&](const char* what) {
    const cudaError_t le = cudaGetLastError();
    if (le == cudaSuccess) { return true; }
    fail(std::string("certex: certexB200SearchStatic could not launch the ") + what + " kernel: " + cudaGetErrorString(le));
    return false;
  };
  launch_dense_scores(vectors, row_bytes, dt, static_cast<int>(dim), m, n_rows, queries, row_bytes, nullptr, 0,
                      static_cast<int>(n_queries), everything, scores, ld, stream);
  if (!launched("scoring")) { return CUVS_ERROR; }  // nothing after a failed launch: later kernels would read stale scratch
  launch_select_topk(scores, ld, n_rows, k, nullptr, 0, static_cast<int>(n_queries), best_s, best_row, part_s, part_row, stream);
  if (!launched("selection")) { return CUVS_ERROR; }
  launch_finish(best_s, best_row, 0, queries, row_bytes, dt, static_cast<int>(dim), m, static_cast<int>(n_queries), k, neighbors,
                distances, nullptr, stream);
  if (!launched("output")) { return CUVS_ERROR; }
  return CUVS_SUCCESS;
}
