/* A plain C caller of the library, in the shape of the reference's examples/c/exact_search.c and
 * c/tests/neighbors/run_certex_c.c: build an index from device memory, search, compare every returned id and distance
 * with an fp64 loop over all vectors (ties to the smaller id), search again by label and through a saved copy.
 * Returns 0 when everything agrees. Compiled with gcc against include/certex_b200.h; needs one sm_100 GPU to run. */
#include <cuda_runtime_api.h>
#include <math.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "certex_b200.h"

#define CHECK(call)                                               \
  do {                                                            \
    if ((call) != CUVS_SUCCESS) {                                 \
      fprintf(stderr, "%s: %s\n", #call, cuvsGetLastErrorText()); \
      return 1;                                                   \
    }                                                             \
  } while (0)
#define CUDA(call)                                                      \
  do {                                                                  \
    if ((call) != cudaSuccess) {                                        \
      fprintf(stderr, "%s failed\n", #call);                            \
      return 1;                                                         \
    }                                                                   \
  } while (0)

enum { N = 20000, NQ = 64, DIM = 48, K = 10, LABELS = 4 };

static void tensor(DLManagedTensor* t, void* data, int64_t* shape, int ndim, uint8_t code, uint8_t bits)
{
  memset(t, 0, sizeof(*t));
  t->dl_tensor.data               = data;
  t->dl_tensor.device.device_type = kDLCUDA;
  t->dl_tensor.ndim               = ndim;
  t->dl_tensor.dtype.code         = code;
  t->dl_tensor.dtype.bits         = bits;
  t->dl_tensor.dtype.lanes        = 1;
  t->dl_tensor.shape              = shape;
}

static uint32_t next_u32(uint64_t* s)
{
  *s = *s * 6364136223846793005ull + 1442695040888963407ull;
  return (uint32_t)(*s >> 33);
}

/* ids of the K smallest (squared distance, id) pairs of query q among the vectors whose label is `label` (< 0: all) */
static void brute(const uint8_t* x, const int32_t* lab, const uint8_t* q, int32_t label, int64_t* ids, double* dist)
{
  int n = 0;
  for (int i = 0; i < N; ++i) {
    if (label >= 0 && lab[i] != label) { continue; }
    double s = 0;
    for (int t = 0; t < DIM; ++t) {
      const double diff = (double)q[t] - (double)x[(size_t)i * DIM + t];
      s += diff * diff;
    }
    int at = n < K ? n : K;
    while (at > 0 && (dist[at - 1] > s)) { --at; } /* equal scores keep the smaller id in front */
    if (at < K) {
      for (int j = (n < K ? n : K - 1); j > at; --j) {
        dist[j] = dist[j - 1];
        ids[j]  = ids[j - 1];
      }
      dist[at] = s;
      ids[at]  = i;
      if (n < K) { ++n; }
    }
  }
}

static int compare(const char* what, const uint8_t* x, const int32_t* lab, const uint8_t* q, const int32_t* qlab,
                   const int64_t* got_ids, const float* got_dist)
{
  for (int i = 0; i < NQ; ++i) {
    int64_t ids[K];
    double dist[K];
    brute(x, lab, q + (size_t)i * DIM, qlab ? qlab[i] : -1, ids, dist);
    for (int j = 0; j < K; ++j) {
      if (got_ids[i * K + j] != ids[j] || (double)got_dist[i * K + j] != (double)(float)dist[j]) {
        fprintf(stderr, "%s: query %d entry %d: got (%lld, %g), want (%lld, %g)\n", what, i, j,
                (long long)got_ids[i * K + j], got_dist[i * K + j], (long long)ids[j], dist[j]);
        return 1;
      }
    }
  }
  return 0;
}

int main(int argc, char** argv)
{
  const char* save_to = argc > 1 ? argv[1] : NULL;
  uint8_t* x    = malloc((size_t)N * DIM);
  uint8_t* q    = malloc((size_t)NQ * DIM);
  int32_t* lab  = malloc(sizeof(int32_t) * N);
  int32_t* qlab = malloc(sizeof(int32_t) * NQ);
  uint64_t seed = 12345;
  for (size_t i = 0; i < (size_t)N * DIM; ++i) { x[i] = (uint8_t)(next_u32(&seed) % 48 + (i % DIM) * 3); }
  for (size_t i = 0; i < (size_t)NQ * DIM; ++i) { q[i] = (uint8_t)(next_u32(&seed) % 48 + (i % DIM) * 3); }
  for (int i = 0; i < N; ++i) { lab[i] = (int32_t)(next_u32(&seed) % LABELS); }
  for (int i = 0; i < NQ; ++i) { qlab[i] = (int32_t)(next_u32(&seed) % LABELS); }
  memcpy(x + (size_t)777 * DIM, x + (size_t)5 * DIM, DIM); /* a duplicate: ties go to the smaller id */
  memcpy(q, x + (size_t)5 * DIM, DIM);

  void *dx, *dq, *dlab, *dqlab, *dn, *dd;
  CUDA(cudaMalloc(&dx, (size_t)N * DIM));
  CUDA(cudaMalloc(&dq, (size_t)NQ * DIM));
  CUDA(cudaMalloc(&dlab, sizeof(int32_t) * N));
  CUDA(cudaMalloc(&dqlab, sizeof(int32_t) * NQ));
  CUDA(cudaMalloc(&dn, sizeof(int64_t) * NQ * K));
  CUDA(cudaMalloc(&dd, sizeof(float) * NQ * K));
  CUDA(cudaMemcpy(dx, x, (size_t)N * DIM, cudaMemcpyHostToDevice));
  CUDA(cudaMemcpy(dq, q, (size_t)NQ * DIM, cudaMemcpyHostToDevice));
  CUDA(cudaMemcpy(dlab, lab, sizeof(int32_t) * N, cudaMemcpyHostToDevice));
  CUDA(cudaMemcpy(dqlab, qlab, sizeof(int32_t) * NQ, cudaMemcpyHostToDevice));

  cuvsResources_t res;
  CHECK(cuvsResourcesCreate(&res));
  int64_t x_shape[2] = {N, DIM}, q_shape[2] = {NQ, DIM}, o_shape[2] = {NQ, K}, l_shape[1] = {N}, ql_shape[1] = {NQ};
  DLManagedTensor tx, tq, tn, td, tl, tql;
  tensor(&tx, dx, x_shape, 2, kDLUInt, 8);
  tensor(&tq, dq, q_shape, 2, kDLUInt, 8);
  tensor(&tn, dn, o_shape, 2, kDLInt, 64);
  tensor(&td, dd, o_shape, 2, kDLFloat, 32);
  tensor(&tl, dlab, l_shape, 1, kDLInt, 32);
  tensor(&tql, dqlab, ql_shape, 1, kDLInt, 32);

  cuvsCertexIndexParams_t ip;
  cuvsCertexSearchParams_t sp;
  cuvsCertexIndex_t index;
  CHECK(cuvsCertexIndexParamsCreate(&ip));
  CHECK(cuvsCertexSearchParamsCreate(&sp));
  CHECK(cuvsCertexIndexCreate(&index));
  CHECK(cuvsCertexBuild(res, ip, &tx, index));
  int64_t size = 0, dim = 0;
  CHECK(cuvsCertexIndexGetSize(index, &size));
  CHECK(cuvsCertexIndexGetDim(index, &dim));
  if (size != N || dim != DIM) { return 2; }

  int64_t* ids = malloc(sizeof(int64_t) * NQ * K);
  float* dist  = malloc(sizeof(float) * NQ * K);
  cuvsFilter none;
  none.type = NO_FILTER;
  none.addr = 0;
  CHECK(cuvsCertexSearch(res, sp, index, &tq, &tn, &td, none));
  CHECK(cuvsStreamSync(res));
  CUDA(cudaMemcpy(ids, dn, sizeof(int64_t) * NQ * K, cudaMemcpyDeviceToHost));
  CUDA(cudaMemcpy(dist, dd, sizeof(float) * NQ * K, cudaMemcpyDeviceToHost));
  if (compare("search", x, lab, q, NULL, ids, dist)) { return 3; }
  if (ids[0] != 5 || ids[1] != 777) { return 4; }

  CHECK(cuvsCertexSetLabels(res, &tl, 0, index));
  CHECK(cuvsCertexPartitionByLabels(res, index));
  CHECK(cuvsCertexSearchWithLabels(res, sp, index, &tq, &tql, &tn, &td));
  CHECK(cuvsStreamSync(res));
  CUDA(cudaMemcpy(ids, dn, sizeof(int64_t) * NQ * K, cudaMemcpyDeviceToHost));
  CUDA(cudaMemcpy(dist, dd, sizeof(float) * NQ * K, cudaMemcpyDeviceToHost));
  if (compare("search by labels", x, lab, q, qlab, ids, dist)) { return 5; }

  if (save_to != NULL) {
    CHECK(cuvsCertexSerialize(res, save_to, index));
    CHECK(cuvsCertexIndexDestroy(index));
    CHECK(cuvsCertexIndexCreate(&index));
    CHECK(cuvsCertexDeserialize(res, save_to, index));
    CHECK(cuvsCertexSearchWithLabels(res, sp, index, &tq, &tql, &tn, &td));
    CHECK(cuvsStreamSync(res));
    CUDA(cudaMemcpy(ids, dn, sizeof(int64_t) * NQ * K, cudaMemcpyDeviceToHost));
    CUDA(cudaMemcpy(dist, dd, sizeof(float) * NQ * K, cudaMemcpyDeviceToHost));
    if (compare("search by labels after reload", x, lab, q, qlab, ids, dist)) { return 6; }
  }

  /* two row shards on this device: host matrices in and out */
  {
    int64_t xs[2] = {N, DIM}, qs[2] = {NQ, DIM}, os[2] = {NQ, K};
    DLManagedTensor hx, hq, hn, hd;
    tensor(&hx, (void*)x, xs, 2, kDLUInt, 8);
    tensor(&hq, (void*)q, qs, 2, kDLUInt, 8);
    tensor(&hn, ids, os, 2, kDLInt, 64);
    tensor(&hd, dist, os, 2, kDLFloat, 32);
    hx.dl_tensor.device.device_type = hq.dl_tensor.device.device_type = kDLCPU;
    hn.dl_tensor.device.device_type = hd.dl_tensor.device.device_type = kDLCPU;
    const int32_t devices[2]        = {0, 0};
    certexB200ShardedIndex_t sharded = NULL;
    int64_t total                    = 0;
    CHECK(certexB200ShardedBuild(devices, 2, ip, &hx, &sharded));
    CHECK(certexB200ShardedGetSize(sharded, &total));
    if (total != N) { return 8; }
    memset(ids, 0, sizeof(int64_t) * NQ * K);
    CHECK(certexB200ShardedSearch(sp, sharded, &hq, &hn, &hd));
    if (compare("sharded search", x, lab, q, NULL, ids, dist)) { return 9; }
    CHECK(certexB200ShardedDestroy(sharded));
  }

  /* an error comes back as a code and a message */
  int64_t bad_shape[2] = {NQ, DIM + 1};
  DLManagedTensor tbad;
  tensor(&tbad, dq, bad_shape, 2, kDLUInt, 8);
  if (cuvsCertexSearch(res, sp, index, &tbad, &tn, &td, none) != CUVS_ERROR || strlen(cuvsGetLastErrorText()) == 0) { return 7; }

  CHECK(cuvsCertexSearchParamsDestroy(sp));
  CHECK(cuvsCertexIndexParamsDestroy(ip));
  CHECK(cuvsCertexIndexDestroy(index));
  CHECK(cuvsResourcesDestroy(res));
  printf("ok\n");
  return 0;
}
