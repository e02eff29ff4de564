/* A C host of the C ABI (no Python, no torch): a decode-like chain of two masked contractions as ONE list
 * launch, each mask selected inside the launch from the activation the call is about to multiply -
 * x -> [select 4 of 16 blocks, W0] -> mid -> [select 3 of 8 blocks, W1] -> out - checked against a plain C
 * restatement of the reference's rule (scripts/bench_roundrobin_e2e_decode.py:90-113: block score = mean over the
 * batch of the block's L2 norm; keep the k best, equal scores to the lower id; multiply the kept channels only).
 * All values are small multiples of 1/4, so every sum is exact in fp32 and the comparison is for equality.
 * Prints "C_HOST_LIST OK" and exits 0, or says what differed. */
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "bas.h"

#define BATCH 16
#define K0 1024
#define N0 512
#define N1 256
#define KEEP0 4
#define KEEP1 3

#define CK(call)                                                                       \
  do {                                                                                 \
    cudaError_t e_ = (call);                                                           \
    if (e_ != cudaSuccess) {                                                           \
      fprintf(stderr, "%s: %s\n", #call, cudaGetErrorString(e_));                      \
      return 2;                                                                        \
    }                                                                                  \
  } while (0)
#define BK(call)                                                                       \
  do {                                                                                 \
    int s_ = (call);                                                                   \
    if (s_ != BAS_OK) {                                                                \
      fprintf(stderr, "%s: %s (cuda %d)\n", #call, bas_status_string(s_), bas_last_cuda_error()); \
      return 3;                                                                        \
    }                                                                                  \
  } while (0)

/* the five values used, as fp16 bits */
static uint16_t half_of_quarter(int q) {   /* q / 4, q in -2..2 */
  switch (q) {
    case -2: return 0xB800;
    case -1: return 0xB400;
    case 1: return 0x3400;
    case 2: return 0x3800;
    default: return 0x0000;
  }
}

static float float_of_half(uint16_t h) {
  const int sign = h >> 15, exp = (h >> 10) & 31, man = h & 1023;
  float v;
  if (exp == 0) v = ldexpf((float)man, -24);
  else if (exp == 31) v = man ? NAN : INFINITY;
  else v = ldexpf((float)(man + 1024), exp - 25);
  return sign ? -v : v;
}

static uint32_t rng_state = 12345u;
static int next_quarter(void) {
  rng_state = rng_state * 1664525u + 1013904223u;
  return (int)((rng_state >> 16) % 5u) - 2;
}

/* ids of the `keep` best blocks of x [BATCH][k], ascending */
static void select_blocks(const float* x, int k, int keep, int* ids) {
  const int nb = k / 64;
  double* score = (double*)malloc(sizeof(double) * (size_t)nb);
  char* taken = (char*)calloc((size_t)nb, 1);
  for (int j = 0; j < nb; ++j) {
    double s = 0.0;
    for (int b = 0; b < BATCH; ++b) {
      double e = 0.0;
      for (int i = 0; i < 64; ++i) {
        const double v = (double)x[(size_t)b * k + 64 * j + i];
        e += v * v;
      }
      s += sqrt(e);
    }
    score[j] = s / (double)BATCH;
  }
  for (int r = 0; r < keep; ++r) {          /* the best remaining block, the lower id among equals */
    int best = -1;
    for (int j = 0; j < nb; ++j)
      if (!taken[j] && (best < 0 || score[j] > score[best])) best = j;
    taken[best] = 1;
  }
  for (int j = 0, r = 0; j < nb; ++j)
    if (taken[j]) ids[r++] = j;
  free(score);
  free(taken);
}

/* y [BATCH][n] = x[:, kept channels] . w[n][k]^T restricted to the kept blocks */
static void masked_product(const float* x, const float* w, int k, int n, const int* ids, int keep, float* y) {
  for (int b = 0; b < BATCH; ++b)
    for (int c = 0; c < n; ++c) {
      float acc = 0.f;
      for (int r = 0; r < keep; ++r)
        for (int i = 0; i < 64; ++i) acc += x[(size_t)b * k + 64 * ids[r] + i] * w[(size_t)c * k + 64 * ids[r] + i];
      y[(size_t)b * n + c] = acc;
    }
}

int main(void) {
  const size_t nx = (size_t)BATCH * K0, nw0 = (size_t)N0 * K0, nw1 = (size_t)N1 * N0;
  uint16_t* xh = (uint16_t*)malloc(2 * nx);
  uint16_t* w0h = (uint16_t*)malloc(2 * nw0);
  uint16_t* w1h = (uint16_t*)malloc(2 * nw1);
  float* xf = (float*)malloc(4 * nx);
  float* w0f = (float*)malloc(4 * nw0);
  float* w1f = (float*)malloc(4 * nw1);
  for (size_t i = 0; i < nx; ++i) {
    /* block j of x is scaled by a block-dependent sparsity so that the block norms differ (and some tie) */
    const int j = (int)((i % K0) / 64);
    int q = next_quarter();
    if ((i + (size_t)j) % (size_t)(2 + j % 5) != 0) q = 0;
    xh[i] = half_of_quarter(q);
    xf[i] = (float)q / 4.f;
  }
  for (size_t i = 0; i < nw0; ++i) {
    int q = next_quarter();
    if (i % 3 != 0) q = 0;
    w0h[i] = half_of_quarter(q);
    w0f[i] = (float)q / 4.f;
  }
  for (size_t i = 0; i < nw1; ++i) {
    int q = next_quarter();
    if (i % 4 != 0) q = 0;
    w1h[i] = half_of_quarter(q);
    w1f[i] = (float)q / 4.f;
  }

  void *x_dev, *w0_dev, *w1_dev, *p0_dev, *p1_dev, *mid_dev, *out_dev;
  int32_t *ids0_dev, *ids1_dev;
  CK(cudaMalloc(&x_dev, 2 * nx));
  CK(cudaMalloc(&w0_dev, 2 * nw0));
  CK(cudaMalloc(&w1_dev, 2 * nw1));
  CK(cudaMalloc(&p0_dev, bas_packed_weight_bytes(N0, K0)));
  CK(cudaMalloc(&p1_dev, bas_packed_weight_bytes(N1, N0)));
  CK(cudaMalloc(&mid_dev, 2 * (size_t)BATCH * N0));
  CK(cudaMalloc(&out_dev, 2 * (size_t)BATCH * N1));
  CK(cudaMalloc((void**)&ids0_dev, 4 * KEEP0));
  CK(cudaMalloc((void**)&ids1_dev, 4 * KEEP1));
  CK(cudaMemcpy(x_dev, xh, 2 * nx, cudaMemcpyHostToDevice));
  CK(cudaMemcpy(w0_dev, w0h, 2 * nw0, cudaMemcpyHostToDevice));
  CK(cudaMemcpy(w1_dev, w1h, 2 * nw1, cudaMemcpyHostToDevice));
  CK(cudaMemset(mid_dev, 0xff, 2 * (size_t)BATCH * N0));
  CK(cudaMemset(out_dev, 0xff, 2 * (size_t)BATCH * N1));
  BK(bas_pack_weight(w0_dev, N0, K0, K0, p0_dev, NULL));
  BK(bas_pack_weight(w1_dev, N1, N0, N0, p1_dev, NULL));
  CK(cudaDeviceSynchronize());

  bas_list_call calls[4];
  memset(calls, 0, sizeof(calls));
  /* 0: the mask of x */
  calls[0].op = BAS_LIST_SELECT;
  calls[0].x_dev = x_dev;
  calls[0].ldx = K0;
  calls[0].batch = BATCH;
  calls[0].k = K0;
  calls[0].k_host = KEEP0;
  calls[0].score_kind = BAS_SCORE_NORM;
  calls[0].depends_on = -1;
  /* 1: mid = x W0^T with that mask */
  calls[1].x_dev = x_dev;
  calls[1].ldx = K0;
  calls[1].packed_dev = p0_dev;
  calls[1].y_dev = mid_dev;
  calls[1].ldy = N0;
  calls[1].batch = BATCH;
  calls[1].k = K0;
  calls[1].n = N0;
  calls[1].depends_on = -1;
  calls[1].mask_entry = 1;
  calls[1].ids_out_dev = ids0_dev;
  /* 2: the mask of mid, once call 1 has written it */
  calls[2].op = BAS_LIST_SELECT;
  calls[2].x_dev = mid_dev;
  calls[2].ldx = N0;
  calls[2].batch = BATCH;
  calls[2].k = N0;
  calls[2].k_host = KEEP1;
  calls[2].score_kind = BAS_SCORE_NORM;
  calls[2].depends_on = 1;
  /* 3: out = mid W1^T with that mask */
  calls[3].x_dev = mid_dev;
  calls[3].ldx = N0;
  calls[3].packed_dev = p1_dev;
  calls[3].y_dev = out_dev;
  calls[3].ldy = N1;
  calls[3].batch = BATCH;
  calls[3].k = N0;
  calls[3].n = N1;
  calls[3].depends_on = 1;
  calls[3].mask_entry = 3;
  calls[3].ids_out_dev = ids1_dev;

  bas_list* list = NULL;
  BK(bas_list_create(&list, calls, 4, 0));
  unsigned int status = 0;
  for (int run = 0; run < 2; ++run) BK(bas_list_run(list, NULL));
  BK(bas_list_read_status(list, &status, NULL));
  if (status != 0) {
    fprintf(stderr, "device status %#x\n", status);
    return 4;
  }

  uint16_t* midh = (uint16_t*)malloc(2 * (size_t)BATCH * N0);
  uint16_t* outh = (uint16_t*)malloc(2 * (size_t)BATCH * N1);
  int32_t ids0[KEEP0], ids1[KEEP1];
  CK(cudaMemcpy(midh, mid_dev, 2 * (size_t)BATCH * N0, cudaMemcpyDeviceToHost));
  CK(cudaMemcpy(outh, out_dev, 2 * (size_t)BATCH * N1, cudaMemcpyDeviceToHost));
  CK(cudaMemcpy(ids0, ids0_dev, sizeof(ids0), cudaMemcpyDeviceToHost));
  CK(cudaMemcpy(ids1, ids1_dev, sizeof(ids1), cudaMemcpyDeviceToHost));

  int want0[KEEP0], want1[KEEP1];
  float* mid_ref = (float*)malloc(4 * (size_t)BATCH * N0);
  float* out_ref = (float*)malloc(4 * (size_t)BATCH * N1);
  select_blocks(xf, K0, KEEP0, want0);
  masked_product(xf, w0f, K0, N0, want0, KEEP0, mid_ref);
  for (int r = 0; r < KEEP0; ++r)
    if (ids0[r] != want0[r]) {
      fprintf(stderr, "first mask: id %d is %d, expected %d\n", r, ids0[r], want0[r]);
      return 5;
    }
  float* midf = (float*)malloc(4 * (size_t)BATCH * N0);
  for (size_t i = 0; i < (size_t)BATCH * N0; ++i) {
    midf[i] = float_of_half(midh[i]);
    if (midf[i] != mid_ref[i]) {
      fprintf(stderr, "mid[%zu] = %g, expected %g\n", i, midf[i], mid_ref[i]);
      return 6;
    }
  }
  select_blocks(midf, N0, KEEP1, want1);
  masked_product(midf, w1f, N0, N1, want1, KEEP1, out_ref);
  for (int r = 0; r < KEEP1; ++r)
    if (ids1[r] != want1[r]) {
      fprintf(stderr, "second mask: id %d is %d, expected %d\n", r, ids1[r], want1[r]);
      return 7;
    }
  for (size_t i = 0; i < (size_t)BATCH * N1; ++i)
    if (float_of_half(outh[i]) != out_ref[i]) {
      fprintf(stderr, "out[%zu] = %g, expected %g\n", i, float_of_half(outh[i]), out_ref[i]);
      return 8;
    }
  bas_list_destroy(list);
  printf("C_HOST_LIST OK (masks %d %d %d %d | %d %d %d)\n", ids0[0], ids0[1], ids0[2], ids0[3], ids1[0], ids1[1], ids1[2]);
  return 0;
}
