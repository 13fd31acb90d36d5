// Plain CUDA kernels of the exact search path: per-row init values of the integer screen, the per-query threshold,
// exact fp64 verification with top-k selection, the dense (unscreened) path, output conversion and the merge of
// per-shard answers.
//
// The exact score of a pair follows `warp_score` / `exact_score` of the reference
// (cpp/src/neighbors/certex/detail/certex_kernels.cuh:247-273, cpp/tests/neighbors/ann_certex.cuh:78-99):
//   L2 sum (q-x)^2, inner product |q|^2 - 2<q,x>, cosine 2 - 2<q,x>/sqrt(max(|q|^2 |x|^2, 1e-300)).
// Each thread walks one stored row from coordinate 0 to d-1 and rounds every product and every sum on its own
// (__dmul_rn / __dadd_rn, never a fused multiply-add), which is the order and rounding of the sequential CPU loop: the
// fp64 scores are bit-identical to it for every element type. Rows are read with 16-byte loads.
//
// The order among equal scores is (score, id) everywhere (selection, sort, merge).
#include "kernels.cuh"

#include "screen_i8.cuh"  // kNeverInit

#include <cub/cub.cuh>
#include <cuda_fp16.h>
#include <math_constants.h>

#include <algorithm>
#include <type_traits>

namespace certex_b200 {

namespace {

// ------------------------------------------------------------------------------------------- element access
template <typename T>
struct Elems;
// The double of a FINITE float32 (bits f) without the conversion instruction, whose pipe does about two per clock and
// SM: the float's sign, exponent field and mantissa are placed in a double's fields as they are, which gives
// x * 2^-896 (a subnormal float lands on a subnormal double, zero on zero), and one multiplication by 2^896 - exact,
// a power of two - restores x. Infinities and NaNs would come out finite: callers use it only on stored rows that
// passed the fp16 range check of the screen.
__device__ __forceinline__ double widen_finite(uint32_t f)
{
  const uint32_t hi = ((f & 0x7fffffffu) >> 3) | (f & 0x80000000u);
  return __dmul_rn(__hiloint2double(static_cast<int>(hi), static_cast<int>(f << 29)), 0x1p896);
}

template <>
struct Elems<float> {
  static constexpr int kPerVec = 4;
  __device__ static void unpack(const uint4& w, double (&o)[4])
  {
    o[0] = double(__uint_as_float(w.x)), o[1] = double(__uint_as_float(w.y));
    o[2] = double(__uint_as_float(w.z)), o[3] = double(__uint_as_float(w.w));
  }
  __device__ static void unpack_finite(const uint4& w, double (&o)[4])
  {
    o[0] = widen_finite(w.x), o[1] = widen_finite(w.y), o[2] = widen_finite(w.z), o[3] = widen_finite(w.w);
  }
  __device__ static double one(const void* p, int64_t i) { return double(static_cast<const float*>(p)[i]); }
};
template <>
struct Elems<__half> {
  static constexpr int kPerVec = 8;
  __device__ static void unpack(const uint4& w, double (&o)[8])
  {
    const uint32_t u[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const __half2 h = *reinterpret_cast<const __half2*>(&u[i]);
      o[2 * i]        = double(__low2float(h));
      o[2 * i + 1]    = double(__high2float(h));
    }
  }
  __device__ static void unpack_finite(const uint4& w, double (&o)[8])
  {
    const uint32_t u[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const __half2 h = *reinterpret_cast<const __half2*>(&u[i]);
      o[2 * i]        = widen_finite(__float_as_uint(__low2float(h)));
      o[2 * i + 1]    = widen_finite(__float_as_uint(__high2float(h)));
    }
  }
  __device__ static double one(const void* p, int64_t i) { return double(__half2float(static_cast<const __half*>(p)[i])); }
};
template <>
struct Elems<int8_t> {
  static constexpr int kPerVec = 16;
  __device__ static void unpack(const uint4& w, double (&o)[16])
  {
    const uint32_t u[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
    for (int i = 0; i < 16; ++i) { o[i] = double(int(int8_t((u[i >> 2] >> (8 * (i & 3))) & 0xffu))); }
  }
  __device__ static double one(const void* p, int64_t i) { return double(static_cast<const int8_t*>(p)[i]); }
};
template <>
struct Elems<uint8_t> {
  static constexpr int kPerVec = 16;
  __device__ static void unpack(const uint4& w, double (&o)[16])
  {
    const uint32_t u[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
    for (int i = 0; i < 16; ++i) { o[i] = double(int((u[i >> 2] >> (8 * (i & 3))) & 0xffu)); }
  }
  __device__ static double one(const void* p, int64_t i) { return double(static_cast<const uint8_t*>(p)[i]); }
};

__device__ __forceinline__ bool admitted(const Admit& a, int64_t q, int64_t row)
{
  if (a.removed && a.removed[row]) { return false; }
  if (a.bits) {
    const int64_t bit = a.bitmap_cols > 0 ? q * a.bitmap_cols + row : row;
    if (((a.bits[bit >> 5] >> (bit & 31)) & 1u) == 0u) { return false; }
  }
  if (a.row_labels) {
    const int32_t l = a.row_labels[row];
    if (l < 0 || l != a.query_labels[q]) { return false; }
  }
  return true;
}

// Accumulators of NQ queries against one stored row, coordinates in order. STORED_XX (cosine): |x|^2 is not summed here,
// the caller sets xx from the value kept with the row (the same sum, made once when the row was added).
template <int METRIC, int NQ, bool STORED_XX = false>
struct Acc {
  double s[NQ];  // L2: sum of squared differences; otherwise: inner product
  double xx;
  __device__ void clear()
  {
#pragma unroll
    for (int b = 0; b < NQ; ++b) { s[b] = 0; }
    xx = 0;
  }
  // qd: queries as doubles in shared memory, query b at qd + b * ldq
  __device__ __forceinline__ void add(double x, const double* qd, int ldq, int t)
  {
#pragma unroll
    for (int b = 0; b < NQ; ++b) {
      const double a = qd[b * ldq + t];
      if constexpr (METRIC == kL2) {
        const double diff = __dsub_rn(a, x);
        s[b]              = __dadd_rn(s[b], __dmul_rn(diff, diff));
      } else {
        s[b] = __dadd_rn(s[b], __dmul_rn(a, x));
      }
    }
    if constexpr (METRIC == kCos && !STORED_XX) { xx = __dadd_rn(xx, __dmul_rn(x, x)); }
  }
  // the same for one query whose coordinate the caller has loaded (a)
  __device__ __forceinline__ void add1(double x, double a)
  {
    if constexpr (METRIC == kL2) {
      const double diff = __dsub_rn(a, x);
      s[0]              = __dadd_rn(s[0], __dmul_rn(diff, diff));
    } else {
      s[0] = __dadd_rn(s[0], __dmul_rn(a, x));
    }
    if constexpr (METRIC == kCos && !STORED_XX) { xx = __dadd_rn(xx, __dmul_rn(x, x)); }
  }
  __device__ __forceinline__ double result(int b, double qq) const
  {
    if constexpr (METRIC == kL2) {
      return s[b];
    } else if constexpr (METRIC == kIP) {
      return __dsub_rn(qq, __dmul_rn(2.0, s[b]));
    } else {
      const double den = fmax(__dmul_rn(qq, xx), 1e-300);
      return __dsub_rn(2.0, __ddiv_rn(__dmul_rn(2.0, s[b]), __dsqrt_rn(den)));
    }
  }
};

// Walks one stored row (16-byte loads) and feeds every coordinate to `acc`. FINITE: the row holds no infinity or NaN
// (float types; see widen_finite).
template <typename T, int METRIC, int NQ, bool FINITE = false>
__device__ __forceinline__ void scan_row(const uint8_t* row, int d, const double* qd, int ldq, Acc<METRIC, NQ>& acc)
{
  constexpr int V   = Elems<T>::kPerVec;
  const uint4* p    = reinterpret_cast<const uint4*>(row);
  const int n_full  = d / V;
  for (int c = 0; c < n_full; ++c) {
    const uint4 w = __ldg(p + c);
    double x[V];
    if constexpr (FINITE) {
      Elems<T>::unpack_finite(w, x);
    } else {
      Elems<T>::unpack(w, x);
    }
#pragma unroll
    for (int e = 0; e < V; ++e) { acc.add(x[e], qd, ldq, c * V + e); }
  }
  for (int t = n_full * V; t < d; ++t) { acc.add(Elems<T>::one(row, t), qd, ldq, t); }
}

// Queries as doubles into shared memory and |q|^2 summed in coordinate order by one thread per query.
template <typename T>
__device__ void load_queries(const void* queries, size_t qpitch, const int64_t* qidx, int nqb, int d, double* qd, int ldq, double* qq)
{
  for (int b = 0; b < nqb; ++b) {
    const uint8_t* src = static_cast<const uint8_t*>(queries) + static_cast<size_t>(qidx[b]) * qpitch;
    for (int t = threadIdx.x; t < d; t += blockDim.x) { qd[b * ldq + t] = Elems<T>::one(src, t); }
  }
  __syncthreads();
  if (threadIdx.x < nqb) {
    double a = 0;
    for (int t = 0; t < d; ++t) {
      const double v = qd[threadIdx.x * ldq + t];
      a              = __dadd_rn(a, __dmul_rn(v, v));
    }
    qq[threadIdx.x] = a;
  }
  __syncthreads();
}

// ------------------------------------------------------------------------------------------- sorting helpers
__device__ __forceinline__ bool pair_less(double sa, int64_t ia, double sb, int64_t ib)
{
  return sa < sb || (sa == sb && ia < ib);
}

// In-place bitonic sort of n2 (a power of two) (score, id) pairs in shared memory, ascending by (score, id).
template <typename IdT>
__device__ void bitonic_sort(double* s, IdT* id, int n2)
{
  for (int size = 2; size <= n2; size <<= 1) {
    for (int stride = size >> 1; stride > 0; stride >>= 1) {
      __syncthreads();
      for (int i = threadIdx.x; i < (n2 >> 1); i += blockDim.x) {
        const int lo   = 2 * i - (i & (stride - 1));
        const int hi   = lo + stride;
        const bool asc = (lo & size) == 0;
        const double a = s[lo], b = s[hi];
        const IdT ia = id[lo], ib = id[hi];
        const bool swap = asc ? pair_less(b, ib, a, ia) : pair_less(a, ia, b, ib);
        if (swap) {
          s[lo] = b, s[hi] = a;
          id[lo] = ib, id[hi] = ia;
        }
      }
    }
  }
  __syncthreads();
}

// In-place bitonic sort of n2 (a power of two) 64-bit keys in shared memory, ascending.
__device__ void bitonic_sort_keys(unsigned long long* key, int n2)
{
  for (int size = 2; size <= n2; size <<= 1) {
    for (int stride = size >> 1; stride > 0; stride >>= 1) {
      __syncthreads();
      for (int i = threadIdx.x; i < (n2 >> 1); i += blockDim.x) {
        const int lo                 = 2 * i - (i & (stride - 1));
        const int hi                 = lo + stride;
        const unsigned long long a   = key[lo], b = key[hi];
        const bool asc               = (lo & size) == 0;
        if (asc ? b < a : a < b) { key[lo] = b, key[hi] = a; }
      }
    }
  }
  __syncthreads();
}

__device__ __forceinline__ unsigned long long ordered_key(double v)
{
  const unsigned long long b = static_cast<unsigned long long>(__double_as_longlong(v));
  return (b >> 63) ? ~b : (b | 0x8000000000000000ull);
}

__host__ __device__ inline int next_pow2(int v)
{
  int p = 1;
  while (p < v) { p <<= 1; }
  return p;
}

// ------------------------------------------------------------------------------------------- build-side kernels
// Eight lanes per row, 16 bytes per lane and step.
template <typename T>
__global__ void row_init_kernel(const uint8_t* vectors, size_t pitch, int d, int metric, const uint8_t* removed,
                                int64_t row0, int64_t n, int64_t n_pad, int32_t* init)
{
  const int64_t gt  = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int64_t r   = row0 + (gt >> 3);
  const int sub     = threadIdx.x & 7;
  const bool in     = r < row0 + n;
  long long sum     = 0;
  if (in && metric == kL2) {
    const uint4* p  = reinterpret_cast<const uint4*>(vectors + static_cast<size_t>(r) * pitch);
    const int n_vec = (d + 15) / 16;  // rows are zero padded to the pitch
    for (int c = sub; c < n_vec; c += 8) {
      const uint4 w       = __ldg(p + c);
      const uint32_t u[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const uint32_t byte = (u[i >> 2] >> (8 * (i & 3))) & 0xffu;
        const int v         = sizeof(T) == 1 && T(-1) < T(0) ? int(int8_t(byte)) : int(byte);
        sum += v * v;
      }
    }
  }
  sum += __shfl_xor_sync(0xffffffffu, sum, 1);
  sum += __shfl_xor_sync(0xffffffffu, sum, 2);
  sum += __shfl_xor_sync(0xffffffffu, sum, 4);
  if (sub == 0 && r < n_pad) {
    int32_t v = kNeverInit;
    if (in && !(removed && removed[r])) { v = metric == kL2 ? -static_cast<int32_t>(sum >> 1) : 0; }
    init[r] = v;
  }
}

// e of the anchors in tile order: out[t * 256 + c] = init[(c * n_tiles + t) * stride].
// With a bitset (one bit per id, set = keep) the anchors the filter drops get `never`, like removed rows: the threshold
// then comes from anchors the search may return.
__global__ void gather_init_kernel(const int32_t* init, int64_t stride, int64_t n_tiles, int32_t* out, const uint32_t* bits,
                                   const int32_t* perm, int32_t never)
{
  const int64_t j = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (j < n_tiles * kBaseTile) {
    const int64_t t = j / kBaseTile, c = j % kBaseTile;
    const int64_t r = (c * n_tiles + t) * stride;
    int32_t e       = init[r];
    if (bits) {
      const int32_t id = perm[r];
      if (((bits[id >> 5] >> (id & 31)) & 1u) == 0u) { e = never; }
    }
    out[j] = e;
  }
}

// Smallest e of every chain of 16 columns in the tile order of the chained anchor pass:
// out[t * 16 + i] = min over w < 16 of init[t * stride_t + i * stride_i + w * stride_w]  (int32 values, or floats by their bits).
__global__ void gather_chain_min_kernel(const int32_t* init, int64_t stride_w, int64_t stride_i, int64_t stride_t,
                                        int64_t n_tiles, int32_t* out, int is_float)
{
  const int64_t j = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (j >= n_tiles * (kBaseTile / kChainRows)) { return; }
  const int64_t t = j / (kBaseTile / kChainRows), i = j % (kBaseTile / kChainRows);
  const int32_t* src = init + t * stride_t + i * stride_i;
  if (is_float) {
    float m = __int_as_float(src[0]);
    for (int w = 1; w < kChainRows; ++w) { m = fminf(m, __int_as_float(src[w * stride_w])); }
    out[j] = __float_as_int(m);
  } else {
    int32_t m = src[0];
    for (int w = 1; w < kChainRows; ++w) { m = min(m, src[w * stride_w]); }
    out[j] = m;
  }
}

__global__ void remove_kernel(const int64_t* ids, int64_t n_ids, int64_t size, uint8_t* removed, int32_t* init,
                              const int32_t* inv, unsigned long long* n_new, int32_t never)
{
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= n_ids) { return; }
  const int64_t id = ids[i];
  if (id < 0 || id >= size) { return; }
  // byte-wide exchange through the containing 32-bit word
  uint32_t* word       = reinterpret_cast<uint32_t*>(removed + (id & ~int64_t(3)));
  const uint32_t bit   = 1u << (8 * (id & 3));
  const uint32_t prev  = atomicOr(word, bit);
  if ((prev & bit) == 0u) { atomicAdd(n_new, 1ull); }
  if (init) { init[inv ? inv[id] : id] = never; }
}

// cmax[c] = max of e over rows [16c, 16c + 16) for chains c0 .. c0 + n - 1 (e padded with kNeverInit).
__global__ void chain_max_kernel(const int32_t* init, int64_t c0, int64_t n, int32_t* cmax)
{
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= n) { return; }
  const int4* e = reinterpret_cast<const int4*>(init + (c0 + i) * 16);
  int m         = kNeverInit;
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const int4 t = e[k];
    m            = max(max(max(m, t.x), max(t.y, t.z)), t.w);
  }
  cmax[c0 + i] = m;
}

// The chains that hold removed ids get their maximum recomputed (after remove_kernel has marked the rows).
__global__ void chain_max_of_ids_kernel(const int64_t* ids, int64_t n_ids, int64_t size, const int32_t* inv,
                                        const int32_t* init, int32_t* cmax, int is_float)
{
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= n_ids) { return; }
  const int64_t id = ids[i];
  if (id < 0 || id >= size) { return; }
  const int64_t c = (inv ? inv[id] : id) / 16;
  if (is_float) {
    float m = -CUDART_INF_F;
    for (int k = 0; k < 16; ++k) { m = fmaxf(m, __int_as_float(init[c * 16 + k])); }
    cmax[c] = __float_as_int(m);
  } else {
    int m = kNeverInit;
    for (int k = 0; k < 16; ++k) { m = max(m, init[c * 16 + k]); }
    cmax[c] = m;
  }
}

// keys[j] = -e[j] (half the squared norm, ascending sort key; for floats the bits of the non-negative float),
// vals[j] = id0 + j.
__global__ void sort_keys_kernel(const int32_t* e, int64_t n, int32_t id0, uint32_t* keys, int32_t* vals, int is_float)
{
  const int64_t j = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (j < n) {
    keys[j] = is_float ? __float_as_uint(-__int_as_float(e[j])) : static_cast<uint32_t>(-e[j]);
    vals[j] = id0 + static_cast<int32_t>(j);
  }
}

// Sorted batch -> index arrays: perm[row0 + j] = id, inv[id] = row0 + j, init[row0 + j] = -key, and the code row.
// `src` holds the code row of id at src + (id - src_id0) * pitch.
__global__ void place_sorted_kernel(const uint32_t* keys, const int32_t* ids, int64_t n, int64_t row0, const uint8_t* src,
                                    int64_t src_id0, size_t pitch, uint8_t* codes, int32_t* perm, int32_t* inv, int32_t* init,
                                    int metric, int is_float)
{
  const int64_t gt   = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int chunks   = static_cast<int>(pitch / 16);
  const int64_t j    = gt / chunks;
  const int c        = static_cast<int>(gt % chunks);
  if (j >= n) { return; }
  const int32_t id = ids[j];
  reinterpret_cast<uint4*>(codes + static_cast<size_t>(row0 + j) * pitch)[c] =
    __ldg(reinterpret_cast<const uint4*>(src + static_cast<size_t>(id - src_id0) * pitch) + c);
  if (c == 0) {
    perm[row0 + j] = id;
    inv[id]        = static_cast<int32_t>(row0 + j);
    init[row0 + j] = metric != kL2 ? 0 : is_float ? __float_as_int(-__uint_as_float(keys[j])) : -static_cast<int32_t>(keys[j]);
  }
}

__global__ void mask_removed_kernel(int32_t* e, const uint8_t* removed, int64_t n, int32_t never)
{
  const int64_t j = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (j < n && removed[j]) { e[j] = never; }
}

__global__ void fill_i32_kernel(int32_t* p, int64_t n, int32_t v)
{
  const int64_t j = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (j < n) { p[j] = v; }
}

// ------------------------------------------------------------------------------------------- fp16 codes of float data
// One warp per row: the row rounded to fp16 (for the cosine metric: the row scaled to unit length first), and what the
// certified threshold test needs to know about the rounding:
//   |h|           norm of the fp16 code                          (rounded up)
//   |y - h|       norm of the rounding residual                  (rounded up)
//   e = -|x|^2/2  per-row term of the L2 value <q, x> - |x|^2/2  (rounded up; 0 for inner product and cosine)
// All sums are fp64. maxima[0..2] collect the largest |h|, |y - h| and |e| as float bits (non-negative floats order
// like their bits); maxima[3] is raised when a coordinate does not fit fp16.
template <typename T>
__global__ void encode_f16_rows_kernel(const uint8_t* vectors, size_t pitch, int d, int metric, int64_t n, uint8_t* codes,
                                       size_t code_pitch, float* e, unsigned int* maxima)
{
  const int64_t row = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int lane    = threadIdx.x & 31;
  if (row >= n) { return; }
  const uint8_t* src = vectors + static_cast<size_t>(row) * pitch;
  double xx          = 0;
  for (int t = lane; t < d; t += 32) {
    const double v = Elems<T>::one(src, t);
    xx += v * v;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) { xx += __shfl_xor_sync(0xffffffffu, xx, o); }
  const double scale = metric == kCos ? (xx > 0 ? 1.0 / sqrt(xx) : 0.0) : 1.0;
  __half* dst        = reinterpret_cast<__half*>(codes + static_cast<size_t>(row) * code_pitch);
  const int d_pad    = static_cast<int>(code_pitch / 2);
  double hh = 0, rr = 0;
  bool bad = false;
  for (int t = lane; t < d_pad; t += 32) {
    __half h = __float2half_rn(0.f);
    if (t < d) {
      const double y  = Elems<T>::one(src, t) * scale;
      h               = __double2half(y);
      const double hf = static_cast<double>(__half2float(h));
      bad |= isinf(hf) || isnan(hf);
      hh += hf * hf;
      rr += (y - hf) * (y - hf);
    }
    dst[t] = h;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    hh += __shfl_xor_sync(0xffffffffu, hh, o);
    rr += __shfl_xor_sync(0xffffffffu, rr, o);
  }
  bad = __any_sync(0xffffffffu, bad);
  if (lane == 0) {
    // the unit-length scaling is itself rounded (fp64): a relative 2^-50 on every coordinate, far inside the slack
    const float n1 = __double2float_ru(sqrt(hh) * (1.0 + 1e-9));
    const float n2 = __double2float_ru(sqrt(rr) * (1.0 + 1e-9) + (metric == kCos ? 1e-12 : 0.0));
    const float ev = metric == kL2 ? __double2float_ru(-0.5 * xx) : 0.f;
    e[row]         = ev;
    atomicMax(maxima + 0, __float_as_uint(n1));
    atomicMax(maxima + 1, __float_as_uint(n2));
    atomicMax(maxima + 2, __float_as_uint(fabsf(ev)));
    if (bad) { atomicExch(maxima + 3, 1u); }
  }
}

// One warp per query: the fp16 code of the query and shift[q] = 2 (E + slack), the amount by which the k-th largest
// group maximum of the anchors is lowered to become the screen's threshold. With h = fp16(q), x~ = fp16 code of a row:
//   <q, x> = <h, x~> + <q - h, x~> + <q, x - x~>,   |<q - h, x~>| <= |q - h| |x~|,   |<q, x - x~>| <= |q| |x - x~|
//   |acc - <h, x~>| <= gamma |h| |x~|    (fp32 accumulation of exact fp16 products, gamma = (d + 16) 2^-20)
// so |acc - <q, x>| <= E(q) = (|q - h| + gamma |h|) N1 + |q| N2 with N1, N2 the largest |x~|, |x - x~| of the index.
// slack covers the fp32 additions of the epilogue, the rounding of e and of the exact fp64 scores: 2^-18 (|h| N1 + Emax).
// The anchors give a value every one of k rows certainly reaches (their group maximum minus E + slack); a row is
// kept unless its value certainly lies below that (its maximum plus E + slack): hence twice.
template <typename T>
__global__ void encode_f16_queries_kernel(const uint8_t* queries, size_t qpitch, int d, int64_t nq, uint8_t* codes,
                                          size_t code_pitch, float n1max, float n2max, float emax, float* shift,
                                          unsigned int* overflow)
{
  const int64_t row = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int lane    = threadIdx.x & 31;
  if (row >= nq) { return; }
  const uint8_t* src = queries + static_cast<size_t>(row) * qpitch;
  __half* dst        = reinterpret_cast<__half*>(codes + static_cast<size_t>(row) * code_pitch);
  const int d_pad    = static_cast<int>(code_pitch / 2);
  double qq = 0, hh = 0, rr = 0;
  bool bad = false;
  for (int t = lane; t < d_pad; t += 32) {
    __half h = __float2half_rn(0.f);
    if (t < d) {
      const double y  = Elems<T>::one(src, t);
      h               = __double2half(y);
      const double hf = static_cast<double>(__half2float(h));
      bad |= isinf(hf) || isnan(hf);
      qq += y * y;
      hh += hf * hf;
      rr += (y - hf) * (y - hf);
    }
    dst[t] = h;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    qq += __shfl_xor_sync(0xffffffffu, qq, o);
    hh += __shfl_xor_sync(0xffffffffu, hh, o);
    rr += __shfl_xor_sync(0xffffffffu, rr, o);
  }
  bad = __any_sync(0xffffffffu, bad);
  if (lane == 0) {
    const double gamma = (d + 16) * 9.5367431640625e-07;  // 2^-20
    const double nqh = sqrt(hh) * (1.0 + 1e-9), dq = sqrt(rr) * (1.0 + 1e-9), nqn = sqrt(qq) * (1.0 + 1e-9);
    const double E     = (dq + gamma * nqh) * n1max + nqn * n2max;
    const double slack = 3.814697265625e-06 * (nqh * n1max + emax);  // 2^-18
    shift[row]         = __double2float_ru(2.0 * (E + slack) * (1.0 + 1e-6));
    if (bad) { atomicExch(overflow, 1u); }
  }
}

// fp16 codes, in two steps around the optional exchange of thresholds between shards. Step 0: thr[q] = the key of the
// k-th largest group maximum (see float_key in the screen kernel) -> the key of value - shift[q] / 2, a score that k
// rows of this index certainly reach in exact arithmetic. Step 1: such a key -> float bits of the screen's
// threshold, bound - shift[q] / 2. Both subtractions round down.
__global__ void finish_thr_f16_kernel(int32_t* thr, const float* shift, int nq, int step, int per)
{
  const int q = blockIdx.x * blockDim.x + threadIdx.x;
  if (q >= nq) { return; }
  const int32_t key = thr[q];
  const float v     = __int_as_float(key ^ ((key >> 31) & 0x7fffffff));
  const float r     = __fadd_rd(v, -__fmul_ru(0.5f, shift[q / per]));
  const int32_t b   = __float_as_int(r);
  thr[q]            = step == 0 ? (b ^ ((b >> 31) & 0x7fffffff)) : b;
}

__global__ void chain_max_f32_kernel(const float* init, int64_t c0, int64_t n, float* cmax)
{
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= n) { return; }
  float m = -CUDART_INF_F;
  for (int k = 0; k < 16; ++k) { m = fmaxf(m, init[(c0 + i) * 16 + k]); }
  cmax[c0 + i] = m;
}

// Survivor records -> per-query candidate lists. One thread per record; the appends of a query go through cnt[q].
__global__ void expand_records_kernel(const uint64_t* rec, const unsigned long long* rec_count, unsigned long long rec_cap,
                                      int64_t n_rows, const int32_t* perm, uint32_t* cnt, int32_t* cand, uint32_t cap)
{
  const unsigned long long n = min(*rec_count, rec_cap);
  for (unsigned long long i = static_cast<unsigned long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += static_cast<unsigned long long>(gridDim.x) * blockDim.x) {
    const uint64_t r     = rec[i];
    const uint32_t q     = static_cast<uint32_t>(r >> 48);
    const int64_t row0   = static_cast<int64_t>((r >> 16) & 0xffffffffull) * 16;
    uint32_t mask        = static_cast<uint32_t>(r & 0xffffu);
    while (mask) {
      const int b = __ffs(mask) - 1;
      mask &= mask - 1;
      const int32_t id = row0 + b < n_rows ? (perm ? perm[row0 + b] : static_cast<int32_t>(row0 + b)) : -1;
      if (id >= 0) {  // rows beyond the last one and padding rows of a label's block have no id
        const uint32_t pos = atomicAdd(cnt + q, 1u);
        if (pos < cap) { cand[static_cast<size_t>(q) * cap + pos] = id; }
      }
    }
  }
}

// rows [q, 0 : n_parts * k] = the lists parts[p, q, 0:k] of every part side by side.
__global__ void union_rows_kernel(const int32_t* parts, int n_parts, int nq, int k, int32_t* rows, int64_t ld)
{
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int m     = n_parts * k;
  if (i >= static_cast<int64_t>(nq) * m) { return; }
  const int64_t q = i / m;
  const int c     = static_cast<int>(i % m), part = c / k, j = c % k;
  rows[q * ld + c] = parts[(static_cast<int64_t>(part) * nq + q) * k + j];
}

// Block per query: the k-th largest of ng int32 values by a most-significant-digit radix walk. The row is copied to
// shared memory first when it fits (vals != global row).
// With ng_rows the rows have their own lengths; a negative length marks a row without a query: thr = never.
// Every thread of the block: out [k] = the k largest of row[0:ng] (any order) given their k-th, t: the values above it,
// then copies of it. (Which k of several equal values are meant does not matter to a threshold.) *counter is shared.
__device__ void emit_topk(const int32_t* row, int ng, int32_t t, int k, int32_t* out, uint32_t* counter)
{
  __syncthreads();
  if (threadIdx.x == 0) { *counter = 0; }
  __syncthreads();
  for (int i = threadIdx.x; i < ng; i += blockDim.x) {
    const int32_t v = row[i];
    if (v > t) {
      const uint32_t pos = atomicAdd(counter, 1u);
      if (pos < static_cast<uint32_t>(k)) { out[pos] = v; }  // fewer than k values lie above the k-th largest
    }
  }
  __syncthreads();
  for (int i = static_cast<int>(min(*counter, static_cast<uint32_t>(k))) + threadIdx.x; i < k; i += blockDim.x) { out[i] = t; }
}

// With topk [nq, k] the k largest values of every row are written there as well (emit_topk).
__global__ void __launch_bounds__(512, 4) kth_largest_kernel(const int32_t* gmax, int64_t ld, int ng, int k, int32_t* thr,
                                                              int in_smem, const int32_t* ng_rows, int32_t never, int32_t* topk)
{
  extern __shared__ int32_t row_smem[];
  __shared__ uint32_t hist[256];
  __shared__ uint32_t s_prefix, s_remaining;
  const int32_t* row = gmax + static_cast<int64_t>(blockIdx.x) * ld;
  int32_t* topk_row  = topk ? topk + static_cast<int64_t>(blockIdx.x) * k : nullptr;
  if (ng_rows) {
    ng = ng_rows[blockIdx.x];
    if (ng < 0) {
      if (threadIdx.x == 0) { thr[blockIdx.x] = never; }
      if (topk_row) {
        for (int i = threadIdx.x; i < k; i += blockDim.x) { topk_row[i] = never; }
      }
      return;
    }
  }
  if (ng < k) {
    if (threadIdx.x == 0) { thr[blockIdx.x] = static_cast<int32_t>(0x80000000u); }
    if (topk_row) {
      for (int i = threadIdx.x; i < k; i += blockDim.x) { topk_row[i] = static_cast<int32_t>(0x80000000u); }
    }
    return;
  }
  // The row goes to shared memory (when it fits) and its smallest and largest key are found on the way: the radix walk
  // then runs on key - smallest and starts at the highest byte in which the keys differ. Group maxima of one query lie
  // close together; walking all 32 bits would put nearly every value into one bin of the first passes, and the
  // shared-memory atomics on that bin would serialise.
  __shared__ uint32_t s_lo, s_hi;
  if (threadIdx.x == 0) {
    s_lo = 0xffffffffu;
    s_hi = 0u;
  }
  __syncthreads();
  uint32_t lo = 0xffffffffu, hi = 0u;
  auto see = [&](int32_t v) {
    const uint32_t key = static_cast<uint32_t>(v) ^ 0x80000000u;
    lo                 = min(lo, key);
    hi                 = max(hi, key);
  };
  if (in_smem) {
    const int n4 = ng >> 2;  // rows start 16-byte aligned (ld is a multiple of 8)
    for (int i = threadIdx.x; i < n4; i += blockDim.x) {
      const int4 v                         = __ldg(reinterpret_cast<const int4*>(row) + i);
      reinterpret_cast<int4*>(row_smem)[i] = v;
      see(v.x), see(v.y), see(v.z), see(v.w);
    }
    for (int i = (n4 << 2) + threadIdx.x; i < ng; i += blockDim.x) {
      row_smem[i] = row[i];
      see(row_smem[i]);
    }
    row = row_smem;
  } else {
    for (int i = threadIdx.x; i < ng; i += blockDim.x) { see(row[i]); }
  }
  const uint32_t my_hi = hi;  // the largest key this thread saw (0: none)
  // Small k: the k-th largest of the maxima of G groups of threads is a value that k elements reach (the k groups at
  // or above it hold one each), so only the few elements at or above it can be the k-th largest of the row: they are
  // collected in one more pass over the row and ranked by counting. No histogram, no contended atomics. When the list
  // does not hold them (many equal values), the radix walk below takes over.
  constexpr int kCollect = 1024;
  __shared__ uint32_t s_group[512], s_list[kCollect];
  __shared__ uint32_t s_bound, s_count, s_answer;
  const int n_threads = blockDim.x;
  if (in_smem && (n_threads == 512 || n_threads == 256 || n_threads == 128) && 2 * k <= n_threads) {
    int groups = 16;
    while (groups < 2 * k) { groups <<= 1; }
    const int per_group = n_threads / groups;  // 32, 16, ..., 1 threads
    uint32_t g_hi       = my_hi;
    for (int o = 1; o < per_group; o <<= 1) { g_hi = max(g_hi, __shfl_xor_sync(0xffffffffu, g_hi, o)); }
    if ((threadIdx.x & (per_group - 1)) == 0) { s_group[threadIdx.x / per_group] = g_hi; }
    if (threadIdx.x == 0) { s_count = 0; }
    __syncthreads();
    if (threadIdx.x < groups) {
      const uint32_t u = s_group[threadIdx.x];
      int rank         = 0;
      for (int j = 0; j < groups; ++j) {
        const uint32_t v = s_group[j];
        rank += (v > u || (v == u && j < static_cast<int>(threadIdx.x))) ? 1 : 0;
      }
      if (rank == k - 1) { s_bound = u; }
    }
    __syncthreads();
    const uint32_t bound = s_bound;
    for (int i = threadIdx.x; i < ng; i += n_threads) {
      const uint32_t key = static_cast<uint32_t>(row[i]) ^ 0x80000000u;
      if (key >= bound) {
        const uint32_t pos = atomicAdd(&s_count, 1u);
        if (pos < kCollect) { s_list[pos] = key; }
      }
    }
    __syncthreads();
    const int n_list = static_cast<int>(s_count);
    if (n_list <= kCollect) {  // n_list >= k: the k group maxima at or above the bound are k elements of the row
      for (int i = threadIdx.x; i < n_list; i += n_threads) {
        const uint32_t u = s_list[i];
        int greater = 0, at_least = 0;
        for (int j = 0; j < n_list; ++j) {
          const uint32_t v = s_list[j];
          greater += v > u ? 1 : 0;
          at_least += v >= u ? 1 : 0;
        }
        if (greater < k && k <= at_least) { s_answer = u; }  // every thread that gets here holds the same value
      }
      __syncthreads();
      const int32_t t = static_cast<int32_t>(s_answer ^ 0x80000000u);
      if (threadIdx.x == 0) { thr[blockIdx.x] = t; }
      if (topk_row) { emit_topk(row, ng, t, k, topk_row, &s_count); }
      return;
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    lo = min(lo, __shfl_xor_sync(0xffffffffu, lo, o));
    hi = max(hi, __shfl_xor_sync(0xffffffffu, hi, o));
  }
  if ((threadIdx.x & 31) == 0) {
    atomicMin(&s_lo, lo);
    atomicMax(&s_hi, hi);
  }
  __syncthreads();
  const uint32_t base  = s_lo;
  const uint32_t range = s_hi - base;
  const int top        = range == 0u ? 0 : 32 - __clz(range);  // bits in which key - base can be set
  uint32_t prefix = 0, mask = 0, remaining = static_cast<uint32_t>(k);
  for (int shift = ((top + 7) / 8 - 1) * 8; shift >= 0; shift -= 8) {
    for (int i = threadIdx.x; i < 256; i += blockDim.x) { hist[i] = 0; }
    __syncthreads();
    for (int i = threadIdx.x; i < ng; i += blockDim.x) {
      const uint32_t key = (static_cast<uint32_t>(row[i]) ^ 0x80000000u) - base;
      if ((key & mask) == prefix) { atomicAdd(&hist[(key >> shift) & 255u], 1u); }
    }
    __syncthreads();
    if (threadIdx.x < 32) {
      // bucket b (from the top) where the running count reaches `remaining`: warp scan over 8 buckets per lane
      const int lane = threadIdx.x;
      uint32_t c[8], sum = 0;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        c[i] = hist[255 - (lane * 8 + i)];
        sum += c[i];
      }
      uint32_t incl = sum;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const uint32_t v = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) { incl += v; }
      }
      const uint32_t before = incl - sum;
      const bool mine       = before < remaining && incl >= remaining;
      if (mine) {
        uint32_t cum = before;
        int i        = 0;
        for (; i < 7; ++i) {
          if (cum + c[i] >= remaining) { break; }
          cum += c[i];
        }
        s_prefix    = prefix | (static_cast<uint32_t>(255 - (lane * 8 + i)) << shift);
        s_remaining = remaining - cum;
      }
    }
    __syncthreads();
    prefix    = s_prefix;
    remaining = s_remaining;
    mask |= 0xffu << shift;
  }
  const int32_t t = static_cast<int32_t>((prefix + base) ^ 0x80000000u);
  if (threadIdx.x == 0) { thr[blockIdx.x] = t; }
  if (topk_row) { emit_topk(row, ng, t, k, topk_row, &s_count); }
}

// Warp per query: the k-th largest of the n_parts * k values parts[p, q, 0:k], p < n_parts, by counting ranks
// (m = n_parts * k <= kUnionMax). Shared memory: m ints per warp.
constexpr int kUnionMax = 512;
__global__ void union_kth_kernel(const int32_t* parts, int n_parts, int nq, int k, int32_t* thr)
{
  extern __shared__ int32_t union_smem[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int q    = blockIdx.x * (blockDim.x >> 5) + warp;
  if (q >= nq) { return; }  // warps are independent: no block-wide barrier below
  const int m = n_parts * k;
  int32_t* v  = union_smem + warp * m;
  for (int i = lane; i < m; i += 32) { v[i] = parts[(static_cast<int64_t>(i / k) * nq + q) * k + (i % k)]; }
  __syncwarp();
  for (int i = lane; i < m; i += 32) {
    const int32_t x = v[i];
    int rank        = 0;
    for (int j = 0; j < m; ++j) {
      const int32_t y = v[j];
      rank += (y > x || (y == x && j < i)) ? 1 : 0;
    }
    if (rank == k - 1) { thr[q] = x; }  // ranks are a permutation of 0 .. m - 1: exactly one element
  }
}

// Exact scores of 8-bit rows against an 8-bit query in integer arithmetic: <q, x> and |x|^2 by 4-way byte dot products
// (int32 is enough: 255^2 * 4096 < 2^31), the score |q|^2 + |x|^2 - 2 <q, x> (L2) or |q|^2 - 2 <q, x> in int64. Every
// partial sum of the fp64 loop over the coordinates is an integer below 2^53, so that loop returns this very integer:
// the results are bit-identical, without one conversion to double per coordinate. |score| < 2^31.
// A row is spread over kRowLanes adjacent lanes of a warp: lane `sub` takes the 16-byte pieces sub, sub + 8, ..., so
// that the lanes of a row read one 128-byte line together and a warp's load covers four whole lines; the partial sums
// are added across the lanes by shuffles (integers: exact in any order). kRowUnroll rows per lane group are in flight
// at once. Every lane of the warp must call it; row < 0 = no row. The results are valid in all lanes of a row.
// qb: the query's bytes in shared memory, zero padded to whole 16-byte vectors like the stored rows.
constexpr int kRowLanes  = 8;
constexpr int kRowUnroll = 4;
template <typename T, int METRIC>
__device__ __forceinline__ void int_row_scores(const uint8_t* vectors, size_t pitch, const int32_t (&row)[kRowUnroll], int d,
                                               const uint4* qb, long long qq, int sub, long long (&score)[kRowUnroll])
{
  const int n_vec = (d + 15) / 16;
  int ip[kRowUnroll], xx[kRowUnroll];
  const uint4* p[kRowUnroll];
#pragma unroll
  for (int u = 0; u < kRowUnroll; ++u) {
    ip[u] = 0, xx[u] = 0;
    p[u] = reinterpret_cast<const uint4*>(vectors + static_cast<size_t>(max(row[u], 0)) * pitch);
  }
  for (int c = sub; c < n_vec; c += kRowLanes) {
    const uint4 a = qb[c];
    uint4 w[kRowUnroll];
#pragma unroll
    for (int u = 0; u < kRowUnroll; ++u) { w[u] = row[u] >= 0 ? __ldg(p[u] + c) : make_uint4(0, 0, 0, 0); }
#pragma unroll
    for (int u = 0; u < kRowUnroll; ++u) {
      if constexpr (std::is_same<T, int8_t>::value) {
        ip[u] = __dp4a(static_cast<int>(w[u].x), static_cast<int>(a.x), ip[u]);
        ip[u] = __dp4a(static_cast<int>(w[u].y), static_cast<int>(a.y), ip[u]);
        ip[u] = __dp4a(static_cast<int>(w[u].z), static_cast<int>(a.z), ip[u]);
        ip[u] = __dp4a(static_cast<int>(w[u].w), static_cast<int>(a.w), ip[u]);
        if constexpr (METRIC == kL2) {
          xx[u] = __dp4a(static_cast<int>(w[u].x), static_cast<int>(w[u].x), xx[u]);
          xx[u] = __dp4a(static_cast<int>(w[u].y), static_cast<int>(w[u].y), xx[u]);
          xx[u] = __dp4a(static_cast<int>(w[u].z), static_cast<int>(w[u].z), xx[u]);
          xx[u] = __dp4a(static_cast<int>(w[u].w), static_cast<int>(w[u].w), xx[u]);
        }
      } else {
        ip[u] = static_cast<int>(__dp4a(w[u].x, a.x, static_cast<unsigned>(ip[u])));
        ip[u] = static_cast<int>(__dp4a(w[u].y, a.y, static_cast<unsigned>(ip[u])));
        ip[u] = static_cast<int>(__dp4a(w[u].z, a.z, static_cast<unsigned>(ip[u])));
        ip[u] = static_cast<int>(__dp4a(w[u].w, a.w, static_cast<unsigned>(ip[u])));
        if constexpr (METRIC == kL2) {
          xx[u] = static_cast<int>(__dp4a(w[u].x, w[u].x, static_cast<unsigned>(xx[u])));
          xx[u] = static_cast<int>(__dp4a(w[u].y, w[u].y, static_cast<unsigned>(xx[u])));
          xx[u] = static_cast<int>(__dp4a(w[u].z, w[u].z, static_cast<unsigned>(xx[u])));
          xx[u] = static_cast<int>(__dp4a(w[u].w, w[u].w, static_cast<unsigned>(xx[u])));
        }
      }
    }
  }
#pragma unroll
  for (int u = 0; u < kRowUnroll; ++u) {
#pragma unroll
    for (int o = 1; o < kRowLanes; o <<= 1) {
      ip[u] += __shfl_xor_sync(0xffffffffu, ip[u], o);
      if constexpr (METRIC == kL2) { xx[u] += __shfl_xor_sync(0xffffffffu, xx[u], o); }
    }
    score[u] = qq + static_cast<long long>(xx[u]) - 2ll * static_cast<long long>(ip[u]);
  }
}

__device__ __forceinline__ unsigned long long warp_min_u64(unsigned long long v)
{
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const unsigned long long other = __shfl_xor_sync(0xffffffffu, v, o);
    v                              = other < v ? other : v;
  }
  return v;
}

// The k smallest of n2 distinct 64-bit keys in shared memory (~0 = none), ascending into out [k], for small k and a
// block of at most kSelectWarps warps: every warp draws the k smallest of its share of the keys by k rounds of a warp
// minimum, then the first warp draws the k smallest of those lists the same way. No key moves in shared memory.
constexpr int kSelectWarps = 4;
constexpr int kSelectMaxK  = 32;
__device__ void select_smallest_keys(const unsigned long long* key, int n2, int k, unsigned long long* lists,
                                     unsigned long long* out)
{
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
  unsigned long long lo = 0;  // keys below lo are taken already
  for (int r = 0; r < k; ++r) {
    unsigned long long best = ~0ull;
    for (int j = warp * 32 + lane; j < n2; j += n_warps * 32) {
      const unsigned long long v = key[j];
      if (v >= lo && v < best) { best = v; }
    }
    best = warp_min_u64(best);
    if (lane == 0) { lists[warp * kSelectMaxK + r] = best; }
    lo = best == ~0ull ? best : best + 1;
  }
  __syncthreads();
  if (warp == 0) {
    lo = 0;
    for (int r = 0; r < k; ++r) {
      unsigned long long best = ~0ull;
      for (int j = lane; j < n_warps * kSelectMaxK; j += 32) {
        const unsigned long long v = (j % kSelectMaxK) < k ? lists[j] : ~0ull;
        if (v >= lo && v < best) { best = v; }
      }
      best = warp_min_u64(best);
      if (lane == 0) { out[r] = best; }
      lo = best == ~0ull ? best : best + 1;
    }
  }
  __syncthreads();
}

// ------------------------------------------------------------------------------------------- stored |x|^2 (cosine)
// Warp per 32 consecutive rows: out[r] = the sum over the coordinates, in order, of x_t^2 in fp64 with every product and
// every sum rounded on its own: bit for bit the sum the cosine verification makes for a candidate row (Acc). The rows
// come through a shared-memory tile as in verify_select_kernel, so that the loads cover whole lines.
constexpr int kSqnormStride = 144;
template <typename T>
__global__ void __launch_bounds__(128) row_sqnorm_kernel(const uint8_t* vectors, size_t pitch, int d, int64_t n, double* out)
{
  __shared__ __align__(16) uint8_t tiles[4 * 32 * kSqnormStride];
  constexpr int V    = Elems<T>::kPerVec;
  const int lane     = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t row0 = (static_cast<int64_t>(blockIdx.x) * 4 + warp) * 32;
  if (row0 >= n) { return; }  // warps are independent: no block-wide barrier below
  uint8_t* tile      = tiles + warp * 32 * kSqnormStride;
  const int piece = lane & 7, row_in_load = lane >> 3;
  const int n_pieces = static_cast<int>((static_cast<size_t>(d) * sizeof(T) + 15) / 16);  // rows are zero padded to the pitch
  const int64_t mine = row0 + lane;
  double xx          = 0;
  for (int p0 = 0; p0 < n_pieces; p0 += 8) {
    uint4 w[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int64_t r = row0 + 4 * j + row_in_load;
      w[j] = (r < n && p0 + piece < n_pieces) ? __ldg(reinterpret_cast<const uint4*>(vectors + static_cast<size_t>(r) * pitch) + p0 + piece)
                                              : make_uint4(0, 0, 0, 0);
    }
    __syncwarp();  // every lane is done with the slab before
#pragma unroll
    for (int j = 0; j < 8; ++j) { *reinterpret_cast<uint4*>(tile + (4 * j + row_in_load) * kSqnormStride + piece * 16) = w[j]; }
    __syncwarp();
    if (mine < n) {
      const int np = min(8, n_pieces - p0);
      for (int p = 0; p < np; ++p) {
        const uint4 x4 = *reinterpret_cast<const uint4*>(tile + lane * kSqnormStride + p * 16);
        double x[V];
        Elems<T>::unpack(x4, x);
        const int t0 = (p0 + p) * V;
        for (int e = 0; e < V && t0 + e < d; ++e) { xx = __dadd_rn(xx, __dmul_rn(x[e], x[e])); }
      }
    }
  }
  if (mine < n) { out[mine] = xx; }
}

// ------------------------------------------------------------------------------------------- verify + select
// Staging tiles of the float rows: per warp 32 rows of a 128-byte slab, 144 bytes apart (a lane's 16-byte reads of its
// own row then fall on distinct banks within every quarter warp).
constexpr int kStageStride = 144;
__device__ __forceinline__ uint8_t* stage_of(void* after_the_arrays)
{
  return reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(after_the_arrays) + 15) & ~static_cast<uintptr_t>(15));
}
// Dynamic shared memory: qd [d] doubles | sc [n2] doubles | id [n2] int32, n2 = next_pow2(cap); for 8-bit rows
// the query's bytes (in the space of qd) | n2 64-bit keys.
// Blocks of 128 threads for 8-bit rows (64 registers: 8 blocks per SM), of 256 threads for float rows (80 registers,
// which the fetch of the next slab during the walk of this one needs: 3 blocks per SM, as many as the shared memory allows).
template <typename T>
constexpr bool kByteRows = std::is_same<T, int8_t>::value || std::is_same<T, uint8_t>::value;
template <typename T, int METRIC, bool STORED_XX = false>
__global__ void __launch_bounds__(kByteRows<T> ? 1024 : 256, kByteRows<T> ? 1 : 3) verify_select_kernel(const uint8_t* vectors, size_t pitch, int d, const void* queries, size_t qpitch,
                                     int q0, const int32_t* cand, const uint32_t* cnt, uint32_t cap, int n2max, int k,
                                     Admit adm, double* best_s, int32_t* best_row, int32_t* ovf_list,
                                     unsigned int* ovf_count, unsigned long long* stats,
                                     const unsigned long long* rec_count, unsigned long long rec_cap, Refine rf,
                                     const int32_t* where, const double* sqnorm)
{
  extern __shared__ double sh[];
  __shared__ double s_qq;
  const int q       = q0 + blockIdx.x;  // number of the query in the call; cand / cnt are those of its batch
  const uint32_t c0 = cnt[blockIdx.x];
  // a candidate list that overflowed, or a survivor record buffer that did (then no list of the batch is complete):
  // the query is reported in ovf_list. What its list holds are still rows at or above its threshold, and the k-th best
  // exact score among them bounds the k-th neighbour: a tighter threshold for a second pass (rf).
  const bool over   = c0 > cap || (rec_count && *rec_count > rec_cap);
  if (over && rf.thr2 == nullptr) {
    if (threadIdx.x == 0) { ovf_list[atomicAdd(ovf_count, 1u)] = q; }
    return;
  }
  const uint32_t c = min(c0, cap);
  double* qd   = sh;
  double* sc   = sh + d;
  int32_t* ids = reinterpret_cast<int32_t*>(sc + n2max);
  const int64_t qi = q;
  constexpr bool kBytes = std::is_same<T, int8_t>::value || std::is_same<T, uint8_t>::value;
  __shared__ long long s_qq_int;
  if constexpr (kBytes) {
    // the query's bytes, zero padded to whole 16-byte vectors, in the space of qd; |q|^2 as an integer
    uint8_t* qbytes    = reinterpret_cast<uint8_t*>(qd);
    const uint8_t* src = static_cast<const uint8_t*>(queries) + static_cast<size_t>(q) * qpitch;
    const int padded   = (d + 15) / 16 * 16;
    for (int t = threadIdx.x; t < padded; t += blockDim.x) { qbytes[t] = t < d ? src[t] : 0; }
    __syncthreads();
    if (threadIdx.x < 32) {  // |q|^2: 255^2 * 4096 < 2^31
      int a = 0;
      for (int t = threadIdx.x; t < padded / 4; t += 32) {
        const uint32_t w = reinterpret_cast<const uint32_t*>(qbytes)[t];
        a = std::is_same<T, int8_t>::value ? __dp4a(static_cast<int>(w), static_cast<int>(w), a)
                                           : static_cast<int>(__dp4a(w, w, static_cast<unsigned>(a)));
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) { a += __shfl_xor_sync(0xffffffffu, a, o); }
      if (threadIdx.x == 0) {
        s_qq_int = a;
        s_qq     = __ll2double_rn(static_cast<long long>(a));
      }
    }
    __syncthreads();
  } else {
    load_queries<T>(queries, qpitch, &qi, 1, d, qd, d, &s_qq);
  }
  const int n2 = max(next_pow2(static_cast<int>(c)), 2);
  const int32_t* mine = cand + static_cast<size_t>(blockIdx.x) * cap;
  // One thread reports an overflowed query with the tighter threshold that the k-th best exact score `kth` among the
  // listed candidates gives (+inf: fewer than k).
  auto report_overflow = [&](double kth) {
    const unsigned int pos = atomicAdd(ovf_count, 1u);
    ovf_list[pos]          = q;
    int32_t t              = rf.thr[blockIdx.x];
    if (kth < CUDART_INF) {
      // the screen's value of a row as good as the k-th: <q, x> - |x|^2 / 2 (L2), <q, x> (inner product),
      // <q, x / |x|> (cosine)
      const double value = METRIC == kCos ? sqrt(s_qq) * (1.0 - 0.5 * kth) : 0.5 * (s_qq - kth);
      if (rf.kind == 1) {  // integer values: e = -floor(|x|^2 / 2) only raises a row's value
        const double cv  = ceil(value);
        const int32_t tv = cv >= 2147483647.0 ? 0x7fffffff : cv <= -2147483648.0 ? static_cast<int32_t>(0x80000000u)
                                                                                    : static_cast<int32_t>(cv);
        t = max(t, tv);
      } else {             // fp16 codes: the value the pass computes may be lower by half the query's allowance
        float f = __double2float_rd(value - 0.5 * static_cast<double>(rf.shift[q]));
        f       = nextafterf(f, -CUDART_INF_F);
        t       = __float_as_int(fmaxf(f, __int_as_float(t)));
      }
    }
    rf.thr2[pos] = t;
  };
  if constexpr (kBytes) {
    // integer scores (below 2^31 in magnitude) and ids sort as one 64-bit key: (score + 2^31) << 32 | id
    unsigned long long* keys = reinterpret_cast<unsigned long long*>(sc);
    __shared__ unsigned long long s_lists[kSelectWarps * kSelectMaxK], s_best[kSelectMaxK];
    constexpr int kGroups = 32 / kRowLanes;  // rows a warp's load covers
    const int sub         = threadIdx.x & (kRowLanes - 1);
    const int group       = (threadIdx.x >> 5) * kGroups + ((threadIdx.x & 31) / kRowLanes);
    const int n_groups    = (blockDim.x >> 5) * kGroups;
    for (int i = static_cast<int>(c) + threadIdx.x; i < n2; i += blockDim.x) { keys[i] = ~0ull; }
    for (int i0 = 0; i0 < static_cast<int>(c); i0 += n_groups * kRowUnroll) {  // the same trips for every lane of a warp
      int32_t row[kRowUnroll];
      bool ok[kRowUnroll];
      long long v[kRowUnroll];
#pragma unroll
      for (int u = 0; u < kRowUnroll; ++u) {
        const int i = i0 + u * n_groups + group;
        row[u]      = i < static_cast<int>(c) ? mine[i] : -1;
      }
#pragma unroll
      for (int u = 0; u < kRowUnroll; ++u) { ok[u] = row[u] >= 0 && admitted(adm, q, row[u]); }
      if (where) {  // `vectors` is not in id order: row `where[id]` of it holds the vector with that id
        int32_t at[kRowUnroll];
#pragma unroll
        for (int u = 0; u < kRowUnroll; ++u) { at[u] = row[u] >= 0 ? __ldg(where + row[u]) : -1; }
        int_row_scores<T, METRIC>(vectors, pitch, at, d, reinterpret_cast<const uint4*>(qd), s_qq_int, sub, v);
      } else {
        int_row_scores<T, METRIC>(vectors, pitch, row, d, reinterpret_cast<const uint4*>(qd), s_qq_int, sub, v);
      }
#pragma unroll
      for (int u = 0; u < kRowUnroll; ++u) {
        const int i = i0 + u * n_groups + group;
        if (sub == 0 && row[u] >= 0) {
          keys[i] = ok[u] ? (static_cast<unsigned long long>(v[u] + 2147483648ll) << 32) | static_cast<uint32_t>(row[u]) : ~0ull;
        }
      }
    }
    const bool small = k <= kSelectMaxK && n2 <= 512 && blockDim.x <= kSelectWarps * 32;
    __syncthreads();
    if (small) {
      select_smallest_keys(keys, n2, k, s_lists, s_best);
    } else {
      bitonic_sort_keys(keys, n2);
    }
    // entry t of the ranking, t < k: straight from the keys
    auto entry = [&](int t) { return small ? s_best[t] : (t < n2 ? keys[t] : ~0ull); };
    if (over) {
      if (threadIdx.x == 0) {
        const unsigned long long kk = entry(k - 1);
        report_overflow(kk != ~0ull ? __ll2double_rn(static_cast<long long>(kk >> 32) - 2147483648ll) : CUDART_INF);
      }
      return;
    }
    for (int t = threadIdx.x; t < k; t += blockDim.x) {
      const unsigned long long key             = entry(t);
      const bool have                          = key != ~0ull;
      best_s[static_cast<size_t>(q) * k + t]   = have ? __ll2double_rn(static_cast<long long>(key >> 32) - 2147483648ll) : CUDART_INF;
      best_row[static_cast<size_t>(q) * k + t] = have ? static_cast<int32_t>(key & 0xffffffffull) : -1;
    }
    if (threadIdx.x == 0 && stats) {
      atomicAdd(stats + 0, static_cast<unsigned long long>(c));  // survivors of the screen
      atomicAdd(stats + 1, static_cast<unsigned long long>(c));  // exact scores computed
    }
    return;
  } else {
    // Float rows: a thread sums its candidate's coordinates in order (the order of the fp64 reference loop), but the
    // rows come through shared memory: a warp fetches a 128-byte slab of 32 candidate rows with eight loads that each
    // cover four whole lines (eight lanes per row), parks it in its tile, and every lane then walks its own row's slab.
    // Per 512 bytes that is 4 + 4 + 4 memory wavefronts instead of the 32 of a warp whose lanes each load 16 bytes of
    // a different row.
    constexpr int V       = Elems<T>::kPerVec;  // coordinates per 16-byte piece
    const int lane        = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
    const int n_pieces    = static_cast<int>((static_cast<size_t>(d) * sizeof(T) + 15) / 16);  // rows are zero padded to the pitch
    uint8_t* tile         = stage_of(ids + n2max) + static_cast<size_t>(warp) * 32 * kStageStride;
    const int piece       = lane & 7, row_in_load = lane >> 3;
    for (int g = warp; g * 32 < n2; g += n_warps) {
      const int i   = g * 32 + lane;
      int32_t row   = 0x7fffffff;
      bool ok       = false;
      if (i < static_cast<int>(c)) {
        row = mine[i];
        ok  = admitted(adm, q, row);
      }
      Acc<METRIC, 1, STORED_XX> acc;
      acc.clear();
      if constexpr (STORED_XX) {
        if (ok) { acc.xx = __ldg(sqnorm + row); }
      }
      if (g * 32 < static_cast<int>(c)) {  // the same for every lane of the warp
        int32_t from[8];  // the rows this lane fetches pieces of
#pragma unroll
        for (int j = 0; j < 8; ++j) { from[j] = __shfl_sync(0xffffffffu, ok ? row : -1, 4 * j + row_in_load); }
        // The loads of the next slab are issued as soon as this slab's registers have been parked in the tile, so that
        // they are in flight while the lanes walk the tile (a warp alone then overlaps its memory latency with its sums).
        uint4 w[8];
        auto fetch = [&](int p0) {
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            w[j] = (from[j] >= 0 && p0 + piece < n_pieces)
                     ? __ldg(reinterpret_cast<const uint4*>(vectors + static_cast<size_t>(from[j]) * pitch) + p0 + piece)
                     : make_uint4(0, 0, 0, 0);
          }
        };
        fetch(0);
        for (int p0 = 0; p0 < n_pieces; p0 += 8) {
          __syncwarp();  // every lane is done with the slab before
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            *reinterpret_cast<uint4*>(tile + (4 * j + row_in_load) * kStageStride + piece * 16) = w[j];
          }
          __syncwarp();
          if (p0 + 8 < n_pieces) { fetch(p0 + 8); }
          if (ok) {
            const int np = min(8, n_pieces - p0);
            for (int p = 0; p < np; ++p) {
              const uint4 x4 = *reinterpret_cast<const uint4*>(tile + lane * kStageStride + p * 16);
              double x[V];
              Elems<T>::unpack_finite(x4, x);  // screened rows are finite
              const int t0 = (p0 + p) * V;
              if (t0 + V <= d) {
                // the query's doubles two at a time (t0 is a multiple of V, qd is 16-byte aligned): half the
                // shared-memory instructions of the walk
#pragma unroll
                for (int e = 0; e < V; e += 2) {
                  const double2 a = *reinterpret_cast<const double2*>(qd + t0 + e);
                  acc.add1(x[e], a.x);
                  acc.add1(x[e + 1], a.y);
                }
              } else {
                for (int e = 0; e < V && t0 + e < d; ++e) { acc.add(x[e], qd, d, t0 + e); }
              }
            }
          }
        }
      }
      if (i < n2) {
        sc[i]  = ok ? acc.result(0, s_qq) : CUDART_INF;
        ids[i] = row;
      }
    }
    bitonic_sort(sc, ids, n2);
  }
  if (over) {
    __syncthreads();
    if (threadIdx.x == 0) { report_overflow(k <= n2 ? sc[k - 1] : CUDART_INF); }
    return;
  }
  for (int t = threadIdx.x; t < k; t += blockDim.x) {
    const bool have                         = t < n2 && sc[t] < CUDART_INF;
    best_s[static_cast<size_t>(q) * k + t]   = have ? sc[t] : CUDART_INF;
    best_row[static_cast<size_t>(q) * k + t] = have ? ids[t] : -1;
  }
  if (threadIdx.x == 0 && stats) {
    atomicAdd(stats + 0, static_cast<unsigned long long>(c));  // survivors of the screen
    atomicAdd(stats + 1, static_cast<unsigned long long>(c));  // exact scores computed
  }
}

// out row i = in row sel[i] (or row i when sel is null), row_bytes of it, the rest of the out_pitch bytes zero; a negative
// sel[i] and rows [n, n_pad) give zero rows. 16-byte units when everything is 16-byte aligned.
__global__ void gather_rows_kernel(const uint8_t* in, size_t in_pitch, const int32_t* sel, int64_t n, uint8_t* out,
                                   size_t out_pitch, size_t row_bytes, int vec16)
{
  const int64_t row = blockIdx.x;
  int64_t from      = row < n ? (sel ? sel[row] : row) : -1;
  const uint8_t* src = from >= 0 ? in + static_cast<size_t>(from) * in_pitch : nullptr;
  uint8_t* dst       = out + static_cast<size_t>(row) * out_pitch;
  if (vec16) {
    const uint4 zero = make_uint4(0, 0, 0, 0);
    for (size_t b = threadIdx.x; b < out_pitch / 16; b += blockDim.x) {
      reinterpret_cast<uint4*>(dst)[b] = (src && b < row_bytes / 16) ? reinterpret_cast<const uint4*>(src)[b] : zero;
    }
  } else {
    for (size_t b = threadIdx.x; b < out_pitch; b += blockDim.x) { dst[b] = (src && b < row_bytes) ? src[b] : 0; }
  }
}

// Label layout of the partition entries: entry p (id part_ids[p], label number i found by its offset) goes to row
// lrow0[i] + (p - off[i]) of the label-ordered copy. Writes lperm [lrow] = id, linv [id] = lrow, lsrc [lrow] = the
// sorted row the codes are copied from, linit [lrow] = e of that row.
__global__ void label_rows_kernel(const int32_t* part_ids, int64_t n, const int64_t* off, const int64_t* lrow0, int n_labels,
                                  const int32_t* inv, const int32_t* init, int32_t* lperm, int32_t* linv, int32_t* lsrc,
                                  int32_t* linit)
{
  const int64_t p = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (p >= n) { return; }
  int lo = 0, hi = n_labels - 1;  // last label whose first entry is <= p
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (off[mid] <= p) {
      lo = mid;
    } else {
      hi = mid - 1;
    }
  }
  const int32_t id   = part_ids[p];
  const int64_t lrow = lrow0[lo] + (p - off[lo]);
  const int32_t srow = inv[id];
  lperm[lrow] = id;
  linv[id]    = static_cast<int32_t>(lrow);
  lsrc[lrow]  = srow;
  linit[lrow] = init[srow];
}

// best lists of the compact queries 0 .. n - 1 -> rows sel[i] of the call's lists
__global__ void scatter_best_kernel(const double* s2, const int32_t* row2, const int32_t* sel, int k, double* best_s,
                                    int32_t* best_row)
{
  if (sel[blockIdx.x] < 0) { return; }
  const size_t src = static_cast<size_t>(blockIdx.x) * k, dst = static_cast<size_t>(sel[blockIdx.x]) * k;
  for (int t = threadIdx.x; t < k; t += blockDim.x) {
    best_s[dst + t]   = s2[src + t];
    best_row[dst + t] = row2[src + t];
  }
}

// list[i] = sel[list[i]]: compact query numbers back to the numbers of the call
__global__ void compose_kernel(int32_t* list, const unsigned int* n, const int32_t* sel)
{
  const unsigned int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < *n) { list[i] = sel[list[i]]; }
}

// ------------------------------------------------------------------------------------------- dense path
constexpr int kDenseQ = 4;  // queries per block that share one walk over a stored row

template <typename T, int METRIC>
__global__ void dense_scores_kernel(const uint8_t* vectors, size_t pitch, int d, int64_t n, const void* queries,
                                    size_t qpitch, const int32_t* qsel, int q0, int nqb, Admit adm, double* out, int64_t ld)
{
  extern __shared__ double sh[];
  __shared__ double s_qq[kDenseQ];
  __shared__ int64_t s_qidx[kDenseQ];
  const int b0 = blockIdx.y * kDenseQ;
  const int nb = min(kDenseQ, nqb - b0);
  if (threadIdx.x < kDenseQ) {
    const int b = min(static_cast<int>(threadIdx.x), nb - 1);
    s_qidx[threadIdx.x] = qsel ? qsel[b0 + b] : q0 + b0 + b;
  }
  __syncthreads();
  load_queries<T>(queries, qpitch, s_qidx, kDenseQ, d, sh, d, s_qq);
  const int64_t row = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (row >= n) { return; }
  Acc<METRIC, kDenseQ> acc;
  acc.clear();
  scan_row<T, METRIC, kDenseQ>(vectors + static_cast<size_t>(row) * pitch, d, sh, d, acc);
#pragma unroll
  for (int b = 0; b < kDenseQ; ++b) {
    if (b < nb) {
      const bool ok = admitted(adm, s_qidx[b], row);
      out[static_cast<int64_t>(b0 + b) * ld + row] = ok ? acc.result(b, s_qq[b]) : CUDART_INF;
    }
  }
}

// Dense scores of label groups in one launch. Group g pairs the queries order[q_begin .. q_begin + nq) (all of one
// label) with the columns of that label: the n_part ids part_ids[part_off ..] of the label partition, then the rows
// tail0 .. tail0 + n_tail - 1 added after the partition was made (`adm` keeps those of the query's label). Blocks
// blk_begin[g] .. blk_begin[g + 1] - 1 belong to group g: quads of queries (slow) by chunks of 256 columns (fast).
template <typename T, int METRIC>
__global__ void dense_scores_grouped_kernel(const uint8_t* vectors, size_t pitch, int d, const void* queries, size_t qpitch,
                                            const int32_t* order, const LabelGroup* groups, int n_groups,
                                            const int32_t* part_ids, int64_t tail0, int64_t n_tail, Admit adm, double* out)
{
  extern __shared__ double sh[];
  __shared__ double s_qq[kDenseQ];
  __shared__ int64_t s_qidx[kDenseQ];
  int lo = 0, hi = n_groups - 1;  // last group whose first block is <= blockIdx.x
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (groups[mid].blk_begin <= static_cast<int64_t>(blockIdx.x)) {
      lo = mid;
    } else {
      hi = mid - 1;
    }
  }
  const LabelGroup g    = groups[lo];
  const int64_t n_cols  = g.n_part + n_tail;
  const int64_t chunks  = (n_cols + blockDim.x - 1) / blockDim.x;
  const int64_t local   = static_cast<int64_t>(blockIdx.x) - g.blk_begin;
  const int b0          = static_cast<int>(local / chunks) * kDenseQ;
  const int64_t col     = (local % chunks) * blockDim.x + threadIdx.x;
  const int nb          = min(kDenseQ, g.nq - b0);
  if (threadIdx.x < kDenseQ) {
    const int b         = min(static_cast<int>(threadIdx.x), nb - 1);
    s_qidx[threadIdx.x] = order[g.q_begin + b0 + b];
  }
  __syncthreads();
  load_queries<T>(queries, qpitch, s_qidx, kDenseQ, d, sh, d, s_qq);
  if (col >= n_cols) { return; }
  const int64_t row = col < g.n_part ? part_ids[g.part_off + col] : tail0 + (col - g.n_part);
  Acc<METRIC, kDenseQ> acc;
  acc.clear();
  scan_row<T, METRIC, kDenseQ>(vectors + static_cast<size_t>(row) * pitch, d, sh, d, acc);
#pragma unroll
  for (int b = 0; b < kDenseQ; ++b) {
    if (b < nb) {
      const bool ok = admitted(adm, s_qidx[b], row);
      out[g.score_off + static_cast<int64_t>(b0 + b) * g.ld + col] = ok ? acc.result(b, s_qq[b]) : CUDART_INF;
    }
  }
}

// Columns of a label group's score row -> ids, for the k winners of every query of the group (see above).
__global__ void group_columns_to_ids_kernel(int32_t* best_row, int k, const int32_t* order, const LabelGroup* groups,
                                            const int32_t* part_ids, int64_t tail0)
{
  const LabelGroup g = groups[blockIdx.x];
  for (int i = threadIdx.x; i < g.nq * k; i += blockDim.x) {
    const size_t o    = static_cast<size_t>(order[g.q_begin + i / k]) * k + (i % k);
    const int32_t col = best_row[o];
    if (col >= 0) { best_row[o] = col < g.n_part ? part_ids[g.part_off + col] : static_cast<int32_t>(tail0 + (col - g.n_part)); }
  }
}

// Block per query: radix walk to the k-th smallest score, then the winners (ties: smallest rows) are gathered, sorted
// and written. Shared memory: sel_s [k2] doubles | sel_id [k2] int32.
// With `row_off` the score rows are ragged: row blockIdx.x starts at scores + row_off[blockIdx.x] and has row_n[] columns.
__global__ void select_topk_kernel(const double* scores, int64_t ld, int64_t n_all, int k, const int32_t* qsel, int q0,
                                   double* best_s, int32_t* best_row, int64_t chunk, double* part_s, int32_t* part_row,
                                   const int64_t* row_off, const int32_t* row_n)
{
  extern __shared__ double sh[];
  __shared__ uint32_t hist[256];
  __shared__ unsigned long long s_prefix;
  __shared__ uint32_t s_remaining, s_less, s_eq_base;
  const int k2        = max(next_pow2(k), 2);
  double* sel_s       = sh;
  int32_t* sel_id     = reinterpret_cast<int32_t*>(sh + k2);
  // blockIdx.y selects a chunk of columns [col0, col0 + n); with several chunks the winners go to part_* and are merged
  const int64_t col0  = static_cast<int64_t>(blockIdx.y) * chunk;
  if (row_off) { n_all = row_n[blockIdx.x]; }
  const int64_t n     = max(static_cast<int64_t>(0), min(chunk, n_all - col0));
  const double* row   = scores + (row_off ? row_off[blockIdx.x] : static_cast<int64_t>(blockIdx.x) * ld) + col0;
  const int64_t qout  = qsel ? qsel[blockIdx.x] : q0 + static_cast<int>(blockIdx.x);
  const uint32_t want = static_cast<uint32_t>(min(static_cast<int64_t>(k), n));

  for (int i = threadIdx.x; i < k2; i += blockDim.x) {
    sel_s[i]  = CUDART_INF;
    sel_id[i] = 0x7fffffff;
  }
  unsigned long long prefix = 0, mask = 0;
  uint32_t remaining = want;
  if (want > 0) {
    for (int shift = 56; shift >= 0; shift -= 8) {
      for (int i = threadIdx.x; i < 256; i += blockDim.x) { hist[i] = 0; }
      __syncthreads();
      for (int64_t i = threadIdx.x; i < n; i += blockDim.x) {
        const unsigned long long key = ordered_key(row[i]);
        if ((key & mask) == prefix) { atomicAdd(&hist[(key >> shift) & 255ull], 1u); }
      }
      __syncthreads();
      if (threadIdx.x == 0) {
        uint32_t cum = 0;
        int b        = 0;
        for (; b < 255; ++b) {
          if (cum + hist[b] >= remaining) { break; }
          cum += hist[b];
        }
        s_prefix    = prefix | (static_cast<unsigned long long>(b) << shift);
        s_remaining = remaining - cum;
      }
      __syncthreads();
      prefix    = s_prefix;
      remaining = s_remaining;
      mask |= 0xffull << shift;
      __syncthreads();
    }
    // `prefix` is the key of the k-th smallest score; `remaining` of the rows that tie with it are wanted (smallest
    // rows first), all rows below it are wanted.
    const uint32_t n_less = want - remaining;
    if (threadIdx.x == 0) {
      s_less    = 0;
      s_eq_base = 0;
    }
    __syncthreads();
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = blockDim.x >> 5;
    __shared__ uint32_t warp_cnt[32];
    for (int64_t c0 = 0; c0 < n; c0 += blockDim.x) {
      const int64_t j = c0 + threadIdx.x;
      double v        = 0;
      bool eq         = false;
      if (j < n) {
        v                            = row[j];
        const unsigned long long key = ordered_key(v);
        if (key < prefix) {
          const uint32_t pos = atomicAdd(&s_less, 1u);
          sel_s[pos]         = v;
          sel_id[pos]        = static_cast<int32_t>(col0 + j);
        }
        eq = key == prefix;
      }
      const int any = __syncthreads_count(eq);
      if (any) {
        const uint32_t ball = __ballot_sync(0xffffffffu, eq);
        if (lane == 0) { warp_cnt[wid] = __popc(ball); }
        __syncthreads();
        uint32_t before = s_eq_base;
        for (int w = 0; w < wid; ++w) { before += warp_cnt[w]; }
        const uint32_t rank = before + __popc(ball & ((1u << lane) - 1u));
        if (eq && rank < remaining) {
          sel_s[n_less + rank]  = v;
          sel_id[n_less + rank] = static_cast<int32_t>(col0 + j);
        }
        __syncthreads();
        if (threadIdx.x == 0) {
          uint32_t tot = 0;
          for (int w = 0; w < nw; ++w) { tot += warp_cnt[w]; }
          s_eq_base += tot;
        }
        __syncthreads();
      }
    }
  }
  __syncthreads();
  bitonic_sort(sel_s, sel_id, k2);
  for (int t = threadIdx.x; t < k; t += blockDim.x) {
    const bool have = sel_s[t] < CUDART_INF;
    if (part_s) {
      const size_t o = (static_cast<size_t>(blockIdx.x) * gridDim.y + blockIdx.y) * k + t;
      part_s[o]      = have ? sel_s[t] : CUDART_INF;
      part_row[o]    = have ? sel_id[t] : 0x7fffffff;
    } else {
      best_s[static_cast<size_t>(qout) * k + t]   = have ? sel_s[t] : CUDART_INF;
      best_row[static_cast<size_t>(qout) * k + t] = have ? sel_id[t] : -1;
    }
  }
}

// Block per query: the k best of `parts` partial lists of k (score, row) pairs each, by (score, row).
// Shared memory: s [n2] doubles | row [n2] int32.
__global__ void merge_partials_kernel(const double* part_s, const int32_t* part_row, int parts, int k, int n2,
                                      const int32_t* qsel, int q0, double* best_s, int32_t* best_row)
{
  extern __shared__ double sh[];
  double* s    = sh;
  int32_t* row = reinterpret_cast<int32_t*>(sh + n2);
  const int m  = parts * k;
  for (int i = threadIdx.x; i < n2; i += blockDim.x) {
    s[i]   = i < m ? part_s[static_cast<size_t>(blockIdx.x) * m + i] : CUDART_INF;
    row[i] = i < m ? part_row[static_cast<size_t>(blockIdx.x) * m + i] : 0x7fffffff;
  }
  bitonic_sort(s, row, n2);
  const int64_t qout = qsel ? qsel[blockIdx.x] : q0 + static_cast<int>(blockIdx.x);
  for (int t = threadIdx.x; t < k; t += blockDim.x) {
    const bool have                            = s[t] < CUDART_INF;
    best_s[static_cast<size_t>(qout) * k + t]   = have ? s[t] : CUDART_INF;
    best_row[static_cast<size_t>(qout) * k + t] = have ? row[t] : -1;
  }
}

// ------------------------------------------------------------------------------------------- output
// Block per query. Distances as `finish` of the reference returns them (cpp/src/neighbors/certex/certex.cu:224-250).
template <typename T>
__global__ void finish_kernel(const double* best_s, const int32_t* best_row, const int64_t* best_id, int64_t id_base,
                              const void* queries, size_t qpitch, int d, int metric, int k, int64_t* neighbors,
                              float* distances, double* scores_out)
{
  __shared__ double s_qq;
  const int q = blockIdx.x;
  if (metric == kIP) {
    if (threadIdx.x == 0) {
      const uint8_t* src = static_cast<const uint8_t*>(queries) + static_cast<size_t>(q) * qpitch;
      double a           = 0;
      for (int t = 0; t < d; ++t) {
        const double v = Elems<T>::one(src, t);
        a              = __dadd_rn(a, __dmul_rn(v, v));
      }
      s_qq = a;
    }
    __syncthreads();
  }
  for (int t = threadIdx.x; t < k; t += blockDim.x) {
    const size_t o   = static_cast<size_t>(q) * k + t;
    const double s   = best_s[o];
    int64_t id       = -1;
    if (best_row) {
      if (best_row[o] >= 0) { id = id_base + best_row[o]; }
    } else {
      id = best_id[o];
    }
    float dist;
    if (id < 0) {
      dist = metric == kIP ? -CUDART_INF_F : CUDART_INF_F;
    } else if (metric == kL2) {
      dist = static_cast<float>(s);
    } else if (metric == kIP) {
      dist = static_cast<float>((s_qq - s) / 2);
    } else {
      dist = static_cast<float>(s / 2);
    }
    neighbors[o] = id;
    distances[o] = dist;
    if (scores_out) { scores_out[o] = id < 0 ? CUDART_INF : s; }
  }
}

// Block per query; shared memory: s [n2] doubles | id [n2] int64.
__global__ void search_status_kernel(const unsigned int* count, const unsigned int* q_ovf, unsigned long long* status)
{
  *status = (count[0] != 0 ? 1ull : 0ull) | (count[1] != 0 ? 2ull : 0ull) | (*q_ovf != 0 ? 4ull : 0ull);
}

__global__ void merge_kernel(const double* in_s, const int64_t* in_id, int parts, int nq, int k, int n2, double* out_s,
                             int64_t* out_id, int64_t part_stride)
{
  extern __shared__ double sh[];
  double* s   = sh;
  int64_t* id = reinterpret_cast<int64_t*>(sh + n2);
  const int q = blockIdx.x;
  const int m = parts * k;
  for (int i = threadIdx.x; i < n2; i += blockDim.x) {
    double v   = CUDART_INF;
    int64_t ii = 0x7fffffffffffffffll;
    if (i < m) {
      const size_t o = static_cast<size_t>(i / k) * part_stride + static_cast<size_t>(q) * k + (i % k);
      if (in_id[o] >= 0) {
        v  = in_s[o];
        ii = in_id[o];
      }
    }
    s[i]  = v;
    id[i] = ii;
  }
  bitonic_sort(s, id, n2);
  for (int t = threadIdx.x; t < k; t += blockDim.x) {
    const bool have                      = id[t] != 0x7fffffffffffffffll;
    out_s[static_cast<size_t>(q) * k + t]  = have ? s[t] : CUDART_INF;
    out_id[static_cast<size_t>(q) * k + t] = have ? id[t] : -1;
  }
}

// The same merge with a warp per query, for parts * k <= kMergeSmallMax candidates: every candidate's place is the number
// of candidates that come before it by (score, id); the first k are written. Shared memory: m doubles + m int64 per warp.
constexpr int kMergeSmallMax = 256;
__global__ void merge_small_kernel(const double* in_s, const int64_t* in_id, int parts, int nq, int k, double* out_s,
                                   int64_t* out_id, int64_t part_stride)
{
  extern __shared__ double merge_smem[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
  const int q    = blockIdx.x * warps + warp;
  if (q >= nq) { return; }  // warps are independent: no block-wide barrier below
  const int m = parts * k;
  double* s   = merge_smem + static_cast<size_t>(warp) * m;
  int64_t* id = reinterpret_cast<int64_t*>(merge_smem + static_cast<size_t>(warps) * m) + static_cast<size_t>(warp) * m;
  for (int i = lane; i < m; i += 32) {
    const size_t o = static_cast<size_t>(i / k) * part_stride + static_cast<size_t>(q) * k + (i % k);
    const int64_t ii = in_id[o];
    s[i]  = ii >= 0 ? in_s[o] : CUDART_INF;
    id[i] = ii >= 0 ? ii : 0x7fffffffffffffffll;
  }
  __syncwarp();
  for (int i = lane; i < m; i += 32) {
    const double x   = s[i];
    const int64_t xi = id[i];
    int place        = 0;
    for (int j = 0; j < m; ++j) {
      const double y   = s[j];
      const int64_t yi = id[j];
      place += (y < x || (y == x && (yi < xi || (yi == xi && j < i)))) ? 1 : 0;
    }
    if (place < k) {
      const bool have                           = xi != 0x7fffffffffffffffll;
      out_s[static_cast<size_t>(q) * k + place]  = have ? x : CUDART_INF;
      out_id[static_cast<size_t>(q) * k + place] = have ? xi : -1;
    }
  }
}

template <typename F>
void by_dtype(int dtype, F&& f)
{
  switch (dtype) {
    case kF32: f(float{}); break;
    case kF16: f(__half{}); break;
    case kI8: f(int8_t{}); break;
    default: f(uint8_t{}); break;
  }
}

template <typename Kernel>
void allow_smem(Kernel kernel, size_t bytes)
{
  // the 48 KB that need no opt-in include the kernel's static shared memory: leave room for it
  if (bytes > 32 * 1024) { cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(bytes)); }
}

}  // namespace

// ------------------------------------------------------------------------------------------- launchers
void launch_row_init(const void* vectors, size_t pitch, int dtype, int d, int metric, const uint8_t* removed,
                     int64_t row0, int64_t n, int64_t n_pad, int32_t* init, cudaStream_t s)
{
  const int64_t rows = n_pad - row0;
  if (rows <= 0) { return; }
  const int64_t threads = rows * 8;
  const int block       = 256;
  const auto grid       = static_cast<unsigned>((threads + block - 1) / block);
  if (dtype == kI8) {
    row_init_kernel<int8_t><<<grid, block, 0, s>>>(static_cast<const uint8_t*>(vectors), pitch, d, metric, removed, row0, n, n_pad, init);
  } else {
    row_init_kernel<uint8_t><<<grid, block, 0, s>>>(static_cast<const uint8_t*>(vectors), pitch, d, metric, removed, row0, n, n_pad, init);
  }
}

void launch_gather_init(const int32_t* init, int64_t stride, int64_t n_tiles, int32_t* out, cudaStream_t s,
                        const uint32_t* bits, const int32_t* perm, int32_t never)
{
  if (n_tiles <= 0) { return; }
  gather_init_kernel<<<static_cast<unsigned>(n_tiles), kBaseTile, 0, s>>>(init, stride, n_tiles, out, bits, perm, never);
}

void launch_gather_chain_min(const int32_t* init, int64_t stride_w, int64_t stride_i, int64_t stride_t, int64_t n_tiles,
                             int32_t* out, bool is_float, cudaStream_t s)
{
  if (n_tiles <= 0) { return; }
  const int64_t n = n_tiles * (kBaseTile / kChainRows);
  gather_chain_min_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, s>>>(init, stride_w, stride_i, stride_t, n_tiles, out,
                                                                                 is_float ? 1 : 0);
}

void launch_expand_records(const uint64_t* rec, const unsigned long long* rec_count, unsigned long long rec_cap,
                           int64_t n_rows, const int32_t* perm, uint32_t* cnt, int32_t* cand, uint32_t cap, int sm_count,
                           cudaStream_t s)
{
  expand_records_kernel<<<sm_count * 8, 256, 0, s>>>(rec, rec_count, rec_cap, n_rows, perm, cnt, cand, cap);
}

void launch_chain_max(const int32_t* init, int64_t c0, int64_t n, int32_t* cmax, bool is_float, cudaStream_t s)
{
  if (n <= 0) { return; }
  const auto grid = static_cast<unsigned>((n + 255) / 256);
  if (is_float) {
    chain_max_f32_kernel<<<grid, 256, 0, s>>>(reinterpret_cast<const float*>(init), c0, n, reinterpret_cast<float*>(cmax));
  } else {
    chain_max_kernel<<<grid, 256, 0, s>>>(init, c0, n, cmax);
  }
}

void launch_encode_f16_rows(const void* vectors, size_t pitch, int dtype, int d, int metric, int64_t n, void* codes,
                            size_t code_pitch, float* e, unsigned int* maxima, cudaStream_t s)
{
  if (n <= 0) { return; }
  const auto grid = static_cast<unsigned>((n * 32 + 255) / 256);
  if (dtype == kF32) {
    encode_f16_rows_kernel<float><<<grid, 256, 0, s>>>(static_cast<const uint8_t*>(vectors), pitch, d, metric, n,
                                                       static_cast<uint8_t*>(codes), code_pitch, e, maxima);
  } else {
    encode_f16_rows_kernel<__half><<<grid, 256, 0, s>>>(static_cast<const uint8_t*>(vectors), pitch, d, metric, n,
                                                        static_cast<uint8_t*>(codes), code_pitch, e, maxima);
  }
}

void launch_encode_f16_queries(const void* queries, size_t qpitch, int dtype, int d, int64_t nq, void* codes,
                               size_t code_pitch, float n1max, float n2max, float emax, float* shift,
                               unsigned int* overflow, cudaStream_t s)
{
  if (nq <= 0) { return; }
  const auto grid = static_cast<unsigned>((nq * 32 + 255) / 256);
  if (dtype == kF32) {
    encode_f16_queries_kernel<float><<<grid, 256, 0, s>>>(static_cast<const uint8_t*>(queries), qpitch, d, nq,
                                                          static_cast<uint8_t*>(codes), code_pitch, n1max, n2max, emax, shift, overflow);
  } else {
    encode_f16_queries_kernel<__half><<<grid, 256, 0, s>>>(static_cast<const uint8_t*>(queries), qpitch, d, nq,
                                                           static_cast<uint8_t*>(codes), code_pitch, n1max, n2max, emax, shift, overflow);
  }
}

void launch_finish_thr_f16(int32_t* thr, const float* shift, int nq, int step, cudaStream_t s, int per)
{
  if (nq <= 0) { return; }
  finish_thr_f16_kernel<<<(nq + 255) / 256, 256, 0, s>>>(thr, shift, nq, step, per);
}

void launch_union_kth(const int32_t* parts, int n_parts, int nq, int k, int32_t* scratch, int32_t* thr, cudaStream_t s)
{
  if (nq <= 0) { return; }
  const int m       = n_parts * k;
  if (m <= kUnionMax) {  // a warp per query ranks the values by counting
    const int warps = 4;
    union_kth_kernel<<<(nq + warps - 1) / warps, warps * 32, static_cast<size_t>(warps) * m * 4, s>>>(parts, n_parts, nq, k, thr);
    return;
  }
  const int64_t ld  = (m + 7) / 8 * 8;
  const int64_t tot = static_cast<int64_t>(nq) * m;
  union_rows_kernel<<<static_cast<unsigned>((tot + 255) / 256), 256, 0, s>>>(parts, n_parts, nq, k, scratch, ld);
  launch_kth_largest(scratch, ld, m, k, nq, thr, s);
}

void launch_fill_i32(int32_t* p, int64_t n, int32_t v, cudaStream_t s)
{
  if (n <= 0) { return; }
  fill_i32_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, s>>>(p, n, v);
}

void launch_mask_removed(int32_t* e, const uint8_t* removed, int64_t n, bool is_float, cudaStream_t s)
{
  if (n <= 0) { return; }
  const int32_t never = is_float ? static_cast<int32_t>(0xff800000u) : kNeverInit;
  mask_removed_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, s>>>(e, removed, n, never);
}

size_t sort_batch_temp_bytes(int64_t n)
{
  size_t bytes = 0;
  cub::DeviceRadixSort::SortPairs(nullptr, bytes, static_cast<const uint32_t*>(nullptr), static_cast<uint32_t*>(nullptr),
                                  static_cast<const int32_t*>(nullptr), static_cast<int32_t*>(nullptr), n);
  return bytes;
}

void launch_sort_batch(const int32_t* e, int64_t n, int32_t id0, int64_t row0, const void* src, int64_t src_id0, size_t pitch,
                       int metric, bool is_float, uint32_t* keys_in, uint32_t* keys_out, int32_t* ids_in, int32_t* ids_out,
                       void* temp, size_t temp_bytes, void* codes, int32_t* perm, int32_t* inv, int32_t* init, cudaStream_t s)
{
  if (n <= 0) { return; }
  sort_keys_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, s>>>(e, n, id0, keys_in, ids_in, is_float ? 1 : 0);
  cub::DeviceRadixSort::SortPairs(temp, temp_bytes, keys_in, keys_out, ids_in, ids_out, n, 0, 32, s);
  const int64_t threads = n * static_cast<int64_t>(pitch / 16);
  place_sorted_kernel<<<static_cast<unsigned>((threads + 255) / 256), 256, 0, s>>>(
    keys_out, ids_out, n, row0, static_cast<const uint8_t*>(src), src_id0, pitch, static_cast<uint8_t*>(codes), perm, inv, init,
    metric, is_float ? 1 : 0);
}

void launch_kth_largest(const int32_t* gmax, int64_t ld, int ng, int k, int nq, int32_t* thr, cudaStream_t s,
                        const int32_t* ng_rows, int32_t never, int32_t* topk)
{
  if (nq <= 0) { return; }
  const size_t bytes = static_cast<size_t>(ng) * 4;
  const int in_smem  = bytes <= 160 * 1024;
  if (in_smem) { allow_smem(kth_largest_kernel, bytes); }
  // short rows: smaller blocks, more of them per SM (the kernel is a chain of block-wide barriers)
  const int threads = ng > 4096 ? 512 : 2 * k <= 128 ? 128 : 2 * k <= 256 ? 256 : 512;
  kth_largest_kernel<<<nq, threads, in_smem ? bytes : 0, s>>>(gmax, ld, ng, k, thr, in_smem, ng_rows, never, topk);
}

void launch_remove(const int64_t* ids, int64_t n_ids, int64_t size, uint8_t* removed, int32_t* init, const int32_t* inv,
                   int32_t* cmax, bool is_float, unsigned long long* n_new, cudaStream_t s)
{
  if (n_ids <= 0) { return; }
  const auto grid     = static_cast<unsigned>((n_ids + 255) / 256);
  const int32_t never = is_float ? static_cast<int32_t>(0xff800000u) : kNeverInit;  // -inf or -2^30
  remove_kernel<<<grid, 256, 0, s>>>(ids, n_ids, size, removed, init, inv, n_new, never);
  if (init && cmax) { chain_max_of_ids_kernel<<<grid, 256, 0, s>>>(ids, n_ids, size, inv, init, cmax, is_float ? 1 : 0); }
}

void launch_verify_select(const void* vectors, size_t pitch, int dtype, int d, int metric, const void* queries,
                          size_t qpitch, int nq, int q0, const int32_t* cand, const uint32_t* cnt, uint32_t cap, int k,
                          Admit adm, double* best_s, int32_t* best_row, int32_t* ovf_list, unsigned int* ovf_count,
                          unsigned long long* stats, const unsigned long long* rec_count, unsigned long long rec_cap,
                          Refine rf, cudaStream_t s, const int32_t* where, const double* sqnorm)
{
  if (nq <= 0) { return; }
  const int n2max   = next_pow2(static_cast<int>(cap));
  const bool bytes  = dtype == kI8 || dtype == kU8;  // 8-bit rows rank 64-bit keys: no separate id array
  // float rows: a warp scores 32 candidates at a time, so a query with a few hundred candidates keeps 8 warps busy;
  // larger blocks leave warps idle at the barrier before the sort (measured on 768-dimensional rows with 153 and 664
  // candidates per query and on 128-dimensional keys with 2 394: 256 threads beat 128, 512 and 1024 in all three)
  const int threads = (dtype == kF32 || dtype == kF16) ? 256 : 128;
  // float rows: + 16 bytes of alignment and one staging tile per warp
  const size_t smem = sizeof(double) * (static_cast<size_t>(d) + n2max) +
                      (bytes ? 0 : sizeof(int32_t) * n2max + 16 + static_cast<size_t>(threads / 32) * 32 * kStageStride);
  by_dtype(dtype, [&](auto tag) {
    using T   = decltype(tag);
    auto go   = [&](auto kernel) {
      allow_smem(kernel, smem);
      kernel<<<nq, threads, smem, s>>>(static_cast<const uint8_t*>(vectors), pitch, d, queries, qpitch, q0, cand, cnt, cap,
                                   n2max, k, adm, best_s, best_row, ovf_list, ovf_count, stats, rec_count, rec_cap, rf,
                                   where, sqnorm);
    };
    if (metric == kL2) {
      go(verify_select_kernel<T, kL2>);
    } else if (metric == kIP) {
      go(verify_select_kernel<T, kIP>);
    } else if (sqnorm != nullptr && !bytes) {
      go(verify_select_kernel<T, kCos, true>);
    } else {
      go(verify_select_kernel<T, kCos>);
    }
  });
}

void launch_row_sqnorms(const void* vectors, size_t pitch, int dtype, int d, int64_t n, double* out, cudaStream_t s)
{
  if (n <= 0) { return; }
  const auto grid = static_cast<unsigned>((n + 127) / 128);
  if (dtype == kF16) {
    row_sqnorm_kernel<__half><<<grid, 128, 0, s>>>(static_cast<const uint8_t*>(vectors), pitch, d, n, out);
  } else {
    row_sqnorm_kernel<float><<<grid, 128, 0, s>>>(static_cast<const uint8_t*>(vectors), pitch, d, n, out);
  }
}

void launch_gather_rows(const void* in, size_t in_pitch, const int32_t* sel, int64_t n, int64_t n_pad, void* out,
                        size_t out_pitch, size_t row_bytes, cudaStream_t s)
{
  if (n_pad <= 0) { return; }
  const auto a    = reinterpret_cast<uintptr_t>(in) | reinterpret_cast<uintptr_t>(out) | in_pitch | out_pitch | row_bytes;
  gather_rows_kernel<<<static_cast<unsigned>(n_pad), 128, 0, s>>>(static_cast<const uint8_t*>(in), in_pitch, sel, n,
                                                                   static_cast<uint8_t*>(out), out_pitch, row_bytes,
                                                                   (a & 15) == 0 ? 1 : 0);
}

void launch_label_rows(const int32_t* part_ids, int64_t n, const int64_t* off, const int64_t* lrow0, int n_labels,
                       const int32_t* inv, const int32_t* init, int32_t* lperm, int32_t* linv, int32_t* lsrc, int32_t* linit,
                       cudaStream_t s)
{
  if (n <= 0) { return; }
  label_rows_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, s>>>(part_ids, n, off, lrow0, n_labels, inv, init, lperm,
                                                                            linv, lsrc, linit);
}

void launch_scatter_best(const double* s2, const int32_t* row2, const int32_t* sel, int n, int k, double* best_s,
                         int32_t* best_row, cudaStream_t s)
{
  if (n <= 0) { return; }
  scatter_best_kernel<<<n, 128, 0, s>>>(s2, row2, sel, k, best_s, best_row);
}

void launch_compose(int32_t* list, const unsigned int* n, int n_max, const int32_t* sel, cudaStream_t s)
{
  if (n_max <= 0) { return; }
  compose_kernel<<<(n_max + 255) / 256, 256, 0, s>>>(list, n, sel);
}

void launch_dense_scores(const void* vectors, size_t pitch, int dtype, int d, int metric, int64_t n, const void* queries,
                         size_t qpitch, const int32_t* qsel, int q0, int nqb, Admit adm, double* out, int64_t ld,
                         cudaStream_t s)
{
  if (nqb <= 0 || n <= 0) { return; }
  const size_t smem = sizeof(double) * static_cast<size_t>(d) * kDenseQ;
  const dim3 grid(static_cast<unsigned>((n + 255) / 256), static_cast<unsigned>((nqb + kDenseQ - 1) / kDenseQ));
  by_dtype(dtype, [&](auto tag) {
    using T = decltype(tag);
    auto go = [&](auto kernel) {
      allow_smem(kernel, smem);
      kernel<<<grid, 256, smem, s>>>(static_cast<const uint8_t*>(vectors), pitch, d, n, queries, qpitch, qsel, q0, nqb, adm, out, ld);
    };
    if (metric == kL2) {
      go(dense_scores_kernel<T, kL2>);
    } else if (metric == kIP) {
      go(dense_scores_kernel<T, kIP>);
    } else {
      go(dense_scores_kernel<T, kCos>);
    }
  });
}

int select_topk_parts(int64_t n, int k)
{
  // long rows are cut into chunks that separate blocks select from; at most 8192 partial winners per query
  if (n <= (1 << 18)) { return 1; }
  const int64_t by_size = (n + (1 << 17) - 1) >> 17;
  return static_cast<int>(std::max<int64_t>(1, std::min<int64_t>({by_size, 64, 8192 / k})));
}

void launch_select_topk(const double* scores, int64_t ld, int64_t n, int k, const int32_t* qsel, int q0, int nqb,
                        double* best_s, int32_t* best_row, double* part_s, int32_t* part_row, cudaStream_t s)
{
  if (nqb <= 0) { return; }
  const int k2      = next_pow2(k) < 2 ? 2 : next_pow2(k);
  const size_t smem = (sizeof(double) + sizeof(int32_t)) * static_cast<size_t>(k2);
  const int parts   = select_topk_parts(n, k);
  if (parts == 1) {
    select_topk_kernel<<<nqb, 256, smem, s>>>(scores, ld, n, k, qsel, q0, best_s, best_row, n, nullptr, nullptr, nullptr, nullptr);
    return;
  }
  const int64_t chunk = (n + parts - 1) / parts;
  select_topk_kernel<<<dim3(nqb, parts), 256, smem, s>>>(scores, ld, n, k, qsel, q0, best_s, best_row, chunk, part_s, part_row, nullptr, nullptr);
  const int n2       = next_pow2(parts * k);
  const size_t smem2 = (sizeof(double) + sizeof(int32_t)) * static_cast<size_t>(n2);
  allow_smem(merge_partials_kernel, smem2);
  merge_partials_kernel<<<nqb, 256, smem2, s>>>(part_s, part_row, parts, k, n2, qsel, q0, best_s, best_row);
}

void launch_select_topk_ragged(const double* scores, const int64_t* row_off, const int32_t* row_n, int64_t n_max, int k,
                               const int32_t* qsel, int nqb, double* best_s, int32_t* best_row, double* part_s,
                               int32_t* part_row, cudaStream_t s)
{
  if (nqb <= 0) { return; }
  const int k2      = next_pow2(k) < 2 ? 2 : next_pow2(k);
  const size_t smem = (sizeof(double) + sizeof(int32_t)) * static_cast<size_t>(k2);
  const int parts   = select_topk_parts(n_max, k);
  if (parts == 1) {
    select_topk_kernel<<<nqb, 256, smem, s>>>(scores, 0, 0, k, qsel, 0, best_s, best_row, std::max<int64_t>(n_max, 1), nullptr,
                                              nullptr, row_off, row_n);
    return;
  }
  const int64_t chunk = (n_max + parts - 1) / parts;
  select_topk_kernel<<<dim3(nqb, parts), 256, smem, s>>>(scores, 0, 0, k, qsel, 0, best_s, best_row, chunk, part_s, part_row,
                                                         row_off, row_n);
  const int n2       = next_pow2(parts * k);
  const size_t smem2 = (sizeof(double) + sizeof(int32_t)) * static_cast<size_t>(n2);
  allow_smem(merge_partials_kernel, smem2);
  merge_partials_kernel<<<nqb, 256, smem2, s>>>(part_s, part_row, parts, k, n2, qsel, 0, best_s, best_row);
}

void launch_dense_scores_grouped(const void* vectors, size_t pitch, int dtype, int d, int metric, const void* queries,
                                 size_t qpitch, const int32_t* order, const LabelGroup* groups, int n_groups,
                                 int64_t n_blocks, const int32_t* part_ids, int64_t tail0, int64_t n_tail, Admit adm,
                                 double* out, cudaStream_t s)
{
  if (n_groups <= 0 || n_blocks <= 0) { return; }
  const size_t smem = sizeof(double) * static_cast<size_t>(d) * kDenseQ;
  by_dtype(dtype, [&](auto tag) {
    using T = decltype(tag);
    auto go = [&](auto kernel) {
      allow_smem(kernel, smem);
      kernel<<<static_cast<unsigned>(n_blocks), 256, smem, s>>>(static_cast<const uint8_t*>(vectors), pitch, d, queries, qpitch,
                                                                 order, groups, n_groups, part_ids, tail0, n_tail, adm, out);
    };
    if (metric == kL2) {
      go(dense_scores_grouped_kernel<T, kL2>);
    } else if (metric == kIP) {
      go(dense_scores_grouped_kernel<T, kIP>);
    } else {
      go(dense_scores_grouped_kernel<T, kCos>);
    }
  });
}

int64_t grouped_blocks(int nq, int64_t n_cols)
{
  return static_cast<int64_t>((nq + kDenseQ - 1) / kDenseQ) * ((n_cols + 255) / 256);
}

void launch_group_columns_to_ids(int32_t* best_row, int k, const int32_t* order, const LabelGroup* groups, int n_groups,
                                 const int32_t* part_ids, int64_t tail0, cudaStream_t s)
{
  if (n_groups <= 0) { return; }
  group_columns_to_ids_kernel<<<n_groups, 256, 0, s>>>(best_row, k, order, groups, part_ids, tail0);
}

// ids of all rows sorted by label (stable: ascending ids inside a label), the distinct labels and their counts
__global__ void iota_kernel(int32_t* p, int64_t n)
{
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i < n) { p[i] = static_cast<int32_t>(i); }
}

// Order of the label-ordered copy of the screen's rows: by label, and inside a label by norm (the per-row term e of the
// screen), so that e is almost constant over 16 adjacent rows there too. keys [n]: (label, -e) of the partition
// entries; the sorted ids go to `order`. labels_of_ids: the label of every id; e is init[inv[id]].
__global__ void label_norm_keys_kernel(const int32_t* part_ids, int64_t n, const int32_t* labels_of_ids, const int32_t* inv,
                                       const int32_t* init, int is_float, unsigned long long* keys)
{
  const int64_t p = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (p >= n) { return; }
  const int32_t id   = part_ids[p];
  const int32_t e    = init[inv[id]];
  const uint32_t low = is_float ? __float_as_uint(-__int_as_float(e)) : static_cast<uint32_t>(-e);  // e <= 0
  const uint32_t top = static_cast<uint32_t>(labels_of_ids[id]) ^ 0x80000000u;                       // signed order
  keys[p]            = (static_cast<unsigned long long>(top) << 32) | low;
}

size_t label_norm_order_temp_bytes(int64_t n)
{
  size_t bytes = 0;
  cub::DeviceRadixSort::SortPairs(nullptr, bytes, static_cast<const unsigned long long*>(nullptr),
                                  static_cast<unsigned long long*>(nullptr), static_cast<const int32_t*>(nullptr),
                                  static_cast<int32_t*>(nullptr), n);
  return bytes;
}

void launch_label_norm_order(const int32_t* part_ids, int64_t n, const int32_t* labels_of_ids, const int32_t* inv,
                             const int32_t* init, bool is_float, unsigned long long* keys_in, unsigned long long* keys_out,
                             int32_t* order, void* temp, size_t temp_bytes, cudaStream_t s)
{
  if (n <= 0) { return; }
  label_norm_keys_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, s>>>(part_ids, n, labels_of_ids, inv, init,
                                                                                is_float ? 1 : 0, keys_in);
  cub::DeviceRadixSort::SortPairs(temp, temp_bytes, keys_in, keys_out, part_ids, order, n, 0, 64, s);
}

size_t label_partition_temp_bytes(int64_t n)
{
  size_t a = 0, b = 0;
  cub::DeviceRadixSort::SortPairs(nullptr, a, static_cast<const int32_t*>(nullptr), static_cast<int32_t*>(nullptr),
                                  static_cast<const int32_t*>(nullptr), static_cast<int32_t*>(nullptr), n);
  cub::DeviceRunLengthEncode::Encode(nullptr, b, static_cast<const int32_t*>(nullptr), static_cast<int32_t*>(nullptr),
                                     static_cast<int32_t*>(nullptr), static_cast<int32_t*>(nullptr), n);
  return std::max(a, b);
}

void launch_label_partition(const int32_t* labels, int64_t n, int32_t* labels_sorted, int32_t* ids_in, int32_t* part_ids,
                            int32_t* distinct, int32_t* counts, int32_t* n_distinct, void* temp, size_t temp_bytes,
                            cudaStream_t s)
{
  if (n <= 0) { return; }
  iota_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, s>>>(ids_in, n);
  cub::DeviceRadixSort::SortPairs(temp, temp_bytes, labels, labels_sorted, ids_in, part_ids, n, 0, 32, s);
  cub::DeviceRunLengthEncode::Encode(temp, temp_bytes, labels_sorted, distinct, counts, n_distinct, n, s);
}

void launch_finish(const double* best_s, const int32_t* best_row, int64_t id_base, const void* queries, size_t qpitch,
                   int dtype, int d, int metric, int nq, int k, int64_t* neighbors, float* distances, double* scores_out,
                   cudaStream_t s)
{
  if (nq <= 0) { return; }
  by_dtype(dtype, [&](auto tag) {
    using T = decltype(tag);
    finish_kernel<T><<<nq, 64, 0, s>>>(best_s, best_row, nullptr, id_base, queries, qpitch, d, metric, k, neighbors, distances, scores_out);
  });
}

void launch_search_status(const unsigned int* count, const unsigned int* q_ovf, unsigned long long* status, cudaStream_t s)
{
  search_status_kernel<<<1, 1, 0, s>>>(count, q_ovf, status);
}

void launch_merge(const double* in_s, const int64_t* in_id, int parts, int nq, int k, const void* queries, size_t qpitch,
                  int dtype, int d, int metric, int64_t* neighbors, float* distances, double* scores_out, cudaStream_t s,
                  int64_t part_stride, bool finish)
{
  if (nq <= 0) { return; }
  if (part_stride == 0) { part_stride = static_cast<int64_t>(nq) * k; }
  // merged (score, id) go to scores_out / neighbors first; finish_kernel then converts in place
  if (parts * k <= kMergeSmallMax) {
    const int warps = 4;
    merge_small_kernel<<<(nq + warps - 1) / warps, warps * 32, static_cast<size_t>(warps) * parts * k * 16, s>>>(
      in_s, in_id, parts, nq, k, scores_out, neighbors, part_stride);
  } else {
    const int n2      = next_pow2(parts * k) < 2 ? 2 : next_pow2(parts * k);
    const size_t smem = (sizeof(double) + sizeof(int64_t)) * static_cast<size_t>(n2);
    allow_smem(merge_kernel, smem);
    merge_kernel<<<nq, 256, smem, s>>>(in_s, in_id, parts, nq, k, n2, scores_out, neighbors, part_stride);
  }
  if (!finish) { return; }
  by_dtype(dtype, [&](auto tag) {
    using T = decltype(tag);
    finish_kernel<T><<<nq, 64, 0, s>>>(scores_out, nullptr, neighbors, 0, queries, qpitch, d, metric, k, neighbors, distances, scores_out);
  });
}

}  // namespace certex_b200
