/*
 * CPU oracle for exact k-nearest-neighbour search. TEST INFRASTRUCTURE ONLY: the product library never links,
 * loads or calls anything in this directory; only the test-suite, the smoke check and the CPU-baseline leg of the
 * benchmark do, and only as the checker or the timed CPU baseline.
 *
 * It restates the reference's own fp64 exhaustive check:
 *   - the score of one (query, vector) pair follows `exact_score`
 *     (cpp/tests/neighbors/ann_certex.cuh:78-99): one sequential loop over t = 0..d-1 in double precision,
 *     L2 `sum (a-b)^2`, inner product `qq - 2 ip`, cosine `2 - 2 ip / sqrt(max(qq xx, 1e-300))`;
 *     the same formulas are the device-side `warp_score` (cpp/src/neighbors/certex/detail/certex_kernels.cuh:247-273)
 *     and the loops of examples/c/exact_search.c:101-119;
 *   - the exhaustive search follows `count_inexact` (cpp/tests/neighbors/ann_certex.cuh:106-141): every admitted
 *     vector is scored and the k smallest scores win; a `keep(i, j)` predicate removes vectors from the candidates
 *     (removed ids, bitset, bitmap, labels).
 * The one rule added here, which the reference leaves open (it accepts any tied vector), is the order among equal
 * scores: (score ascending, id ascending). Missing entries (fewer than k admitted vectors) are id -1, score +inf,
 * as `finish` writes them (cpp/src/neighbors/certex/certex.cu:246-249).
 *
 * Build with -ffp-contract=off: each product and each sum is rounded on its own, which is what the CUDA kernels
 * reproduce with __dmul_rn/__dadd_rn, so float inputs give bit-identical fp64 scores on both sides.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

enum { ORACLE_F32 = 0, ORACLE_F16 = 1, ORACLE_I8 = 2, ORACLE_U8 = 3 };
enum { ORACLE_L2 = 0, ORACLE_IP = 1, ORACLE_COS = 2 };

static float half_to_float(uint16_t h)
{
  const uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
  uint32_t exp        = (h >> 10) & 0x1fu;
  uint32_t man        = h & 0x3ffu;
  uint32_t bits;
  if (exp == 0) {
    if (man == 0) {
      bits = sign;
    } else { /* subnormal half: normalise */
      int e = -1;
      do {
        man <<= 1;
        ++e;
      } while ((man & 0x400u) == 0);
      bits = sign | ((uint32_t)(127 - 15 - e) << 23) | ((man & 0x3ffu) << 13);
    }
  } else if (exp == 31) {
    bits = sign | 0x7f800000u | (man << 13);
  } else {
    bits = sign | ((exp + 127 - 15) << 23) | (man << 13);
  }
  float f;
  memcpy(&f, &bits, 4);
  return f;
}

static inline double elem(const void* base, int dtype, int64_t i)
{
  switch (dtype) {
    case ORACLE_F32: return (double)((const float*)base)[i];
    case ORACLE_F16: return (double)half_to_float(((const uint16_t*)base)[i]);
    case ORACLE_I8: return (double)((const int8_t*)base)[i];
    default: return (double)((const uint8_t*)base)[i];
  }
}

/* exact_score, cpp/tests/neighbors/ann_certex.cuh:78-99 */
static double score_rows(const double* q, const void* x, int dtype, int64_t row, int64_t d, int metric)
{
  double s = 0, qq = 0, xx = 0, ip = 0;
  const int64_t o = row * d;
  if (metric == ORACLE_L2) {
    for (int64_t t = 0; t < d; ++t) {
      const double diff = q[t] - elem(x, dtype, o + t);
      s += diff * diff;
    }
    return s;
  }
  for (int64_t t = 0; t < d; ++t) {
    const double a = q[t], b = elem(x, dtype, o + t);
    ip += a * b;
    qq += a * a;
    xx += b * b;
  }
  if (metric == ORACLE_IP) { return qq - 2 * ip; }
  const double den = qq * xx;
  return 2 - 2 * ip / sqrt(den > 1e-300 ? den : 1e-300);
}

/** Score of query i and vector j (both given in the same element type). */
double oracle_score(const void* x, const void* q, int dtype, int64_t i, int64_t j, int64_t d, int metric)
{
  double* qd = (double*)malloc(sizeof(double) * (size_t)d);
  for (int64_t t = 0; t < d; ++t) { qd[t] = elem(q, dtype, i * d + t); }
  const double s = score_rows(qd, x, dtype, j, d, metric);
  free(qd);
  return s;
}

typedef struct {
  double s;
  int64_t id;
} pair_t;

static inline int worse(pair_t a, pair_t b) /* a ranks after b */
{
  return a.s > b.s || (a.s == b.s && a.id > b.id);
}

static void sift_down(pair_t* h, int n, int i)
{
  for (;;) {
    int l = 2 * i + 1, r = l + 1, m = i;
    if (l < n && worse(h[l], h[m])) { m = l; }
    if (r < n && worse(h[r], h[m])) { m = r; }
    if (m == i) { return; }
    pair_t t = h[i];
    h[i]     = h[m];
    h[m]     = t;
    i        = m;
  }
}

static int cmp_pair(const void* a, const void* b)
{
  const pair_t* x = (const pair_t*)a;
  const pair_t* y = (const pair_t*)b;
  if (x->s < y->s) { return -1; }
  if (x->s > y->s) { return 1; }
  return (x->id > y->id) - (x->id < y->id);
}

/**
 * Exhaustive search. x [n, d] and q [nq, d] of `dtype`; ids [nq, k] and scores [nq, k] receive the k best
 * (score, id) pairs of every query, best first, id = id_base + row.
 * Optional predicates (NULL = absent), all "non-zero keeps":
 *   keep_row [n] bytes (removed ids / bitset), keep_pair [nq, n] bytes (bitmap),
 *   row_labels [n] + query_labels [nq] (a row is admitted iff its label equals the query's; -1 matches nothing).
 * Returns the number of threads used.
 */
int oracle_knn(const void* x,
               int64_t n,
               const void* q,
               int64_t nq,
               int64_t d,
               int dtype,
               int metric,
               int k,
               int64_t id_base,
               const uint8_t* keep_row,
               const uint8_t* keep_pair,
               const int32_t* row_labels,
               const int32_t* query_labels,
               int64_t* ids,
               double* scores,
               int n_threads)
{
  int used = 1;
#ifdef _OPENMP
  if (n_threads > 0) { omp_set_num_threads(n_threads); }
  used = omp_get_max_threads();
#endif
#pragma omp parallel
  {
    double* qd   = (double*)malloc(sizeof(double) * (size_t)d);
    pair_t* heap = (pair_t*)malloc(sizeof(pair_t) * (size_t)k);
#pragma omp for schedule(dynamic, 1)
    for (int64_t i = 0; i < nq; ++i) {
      for (int64_t t = 0; t < d; ++t) { qd[t] = elem(q, dtype, i * d + t); }
      int m = 0;
      for (int64_t j = 0; j < n; ++j) {
        if (keep_row && !keep_row[j]) { continue; }
        if (keep_pair && !keep_pair[i * n + j]) { continue; }
        if (row_labels && (row_labels[j] < 0 || row_labels[j] != query_labels[i])) { continue; }
        pair_t p;
        p.s  = score_rows(qd, x, dtype, j, d, metric);
        p.id = id_base + j;
        if (m < k) {
          heap[m++] = p;
          if (m == k) {
            for (int a = k / 2 - 1; a >= 0; --a) { sift_down(heap, k, a); }
          }
        } else if (worse(heap[0], p)) {
          heap[0] = p;
          sift_down(heap, k, 0);
        }
      }
      qsort(heap, (size_t)m, sizeof(pair_t), cmp_pair);
      for (int t = 0; t < k; ++t) {
        ids[i * k + t]    = t < m ? heap[t].id : -1;
        scores[i * k + t] = t < m ? heap[t].s : INFINITY;
      }
    }
    free(qd);
    free(heap);
  }
  return used;
}

/**
 * Merge of per-shard answers by (score, id), the order of the sharded search's host merge
 * (cpp/src/neighbors/certex/certex_shards.cu:144-166) with exact scores in place of float distances.
 * in_ids / in_scores: [n_shards, nq, k]; id -1 entries are skipped.
 */
void oracle_merge(const int64_t* in_ids,
                  const double* in_scores,
                  int n_shards,
                  int64_t nq,
                  int k,
                  int64_t* ids,
                  double* scores)
{
  pair_t* all = (pair_t*)malloc(sizeof(pair_t) * (size_t)n_shards * (size_t)k);
  for (int64_t i = 0; i < nq; ++i) {
    int m = 0;
    for (int s = 0; s < n_shards; ++s) {
      for (int t = 0; t < k; ++t) {
        const int64_t o = ((int64_t)s * nq + i) * k + t;
        if (in_ids[o] >= 0) {
          all[m].s  = in_scores[o];
          all[m].id = in_ids[o];
          ++m;
        }
      }
    }
    qsort(all, (size_t)m, sizeof(pair_t), cmp_pair);
    for (int t = 0; t < k; ++t) {
      ids[i * k + t]    = t < m ? all[t].id : -1;
      scores[i * k + t] = t < m ? all[t].s : INFINITY;
    }
  }
  free(all);
}

/**
 * int32 reference of the integer screening product: acc[i, j] = <q_i, x_j> + init[j] for uint8 (is_signed = 0) or
 * int8 codes of row pitch `pitch` bytes; the keep / not-keep decision of the tensor-core pass is checked against it.
 */
void oracle_int_gram(const void* q,
                     int64_t nq,
                     const void* x,
                     int64_t n,
                     int64_t d,
                     int64_t pitch_q,
                     int64_t pitch_x,
                     int is_signed,
                     const int32_t* init,
                     int32_t* acc)
{
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < nq; ++i) {
    for (int64_t j = 0; j < n; ++j) {
      int32_t s = init ? init[j] : 0;
      if (is_signed) {
        const int8_t* a = (const int8_t*)q + i * pitch_q;
        const int8_t* b = (const int8_t*)x + j * pitch_x;
        for (int64_t t = 0; t < d; ++t) { s += (int32_t)a[t] * (int32_t)b[t]; }
      } else {
        const uint8_t* a = (const uint8_t*)q + i * pitch_q;
        const uint8_t* b = (const uint8_t*)x + j * pitch_x;
        for (int64_t t = 0; t < d; ++t) { s += (int32_t)a[t] * (int32_t)b[t]; }
      }
      acc[i * n + j] = s;
    }
  }
}
