/* Driver of tests/test_host_sanitizers.py: calls every host-only entry point of the C ABI with
 * many seeded descriptors (valid ones, edge sizes, and garbage) under AddressSanitizer and
 * UndefinedBehaviorSanitizer.  No GPU is needed: plan creation is expected to answer
 * GZ_ERR_NO_DEVICE (or to work, on a GPU box) and nothing else may go wrong. */
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#include "gemmzoo/gemm.h"

static uint64_t state = 0x9E3779B97F4A7C15ull;
static uint64_t rnd(void) {
  state ^= state << 13;
  state ^= state >> 7;
  state ^= state << 17;
  return state;
}

int main(void) {
  static const int pairs[][2] = {{GZ_DT_F16, GZ_DT_F16}, {GZ_DT_F16, GZ_DT_F32}, {GZ_DT_BF16, GZ_DT_BF16},
                                 {GZ_DT_BF16, GZ_DT_F32}, {GZ_DT_F32, GZ_DT_F32}, {GZ_DT_S8, GZ_DT_S32},
                                 {GZ_DT_S8, GZ_DT_BF16}, {GZ_DT_E4M3, GZ_DT_BF16}, {GZ_DT_E5M2, GZ_DT_F32}};
  static const int64_t sizes[] = {1, 2, 7, 8, 15, 16, 17, 31, 33, 63, 64, 65, 127, 128, 129, 255, 256, 300, 511, 512,
                                  1000, 1024, 4096, 8192, 14336, 16384, 100000, 2147482623, 2147483647};
  const int nsizes = (int)(sizeof(sizes) / sizeof(sizes[0]));
  static const int sms[] = {0, 1, 2, 3, 74, 132, 148, 160};
  long ok = 0, rejected = 0;
  for (int it = 0; it < 30000; ++it) {
    gz_gemm_desc d;
    memset(&d, 0, sizeof d);
    d.struct_size = sizeof d;
    const int garbage = (it % 4) == 3;
    const int* p = pairs[rnd() % 9];
    d.in_type = garbage ? (int)(rnd() % 9) - 1 : p[0];
    d.out_type = garbage ? (int)(rnd() % 9) - 1 : p[1];
    d.layout_a = garbage ? (int)(rnd() % 4) - 1 : (int)(rnd() % 2);
    d.layout_b = garbage ? (int)(rnd() % 4) - 1 : (int)(rnd() % 2);
    d.config = garbage ? (int)(rnd() % 20) - 2 : ((rnd() % 3) ? GZ_CFG_AUTO : (int)(rnd() % 11));
    d.flags = garbage ? (uint32_t)rnd() : (uint32_t)(rnd() & 0x3F) & (uint32_t)(rnd() & 0x3F);
    d.m = garbage ? (int64_t)(rnd() % 5) - 2 : sizes[rnd() % nsizes];
    d.n = sizes[rnd() % nsizes];
    d.k = sizes[rnd() % nsizes];
    if (rnd() % 4 == 0) d.lda = d.k + (int64_t)(rnd() % 24);
    if (rnd() % 4 == 0) d.ldb = d.n + (int64_t)(rnd() % 24);
    if (rnd() % 4 == 0) d.ldd = d.n + (int64_t)(rnd() % 24) - 4;
    d.batch = (rnd() % 5 == 0) ? (int64_t)(rnd() % 70000) - 10 : 0;
    if (garbage && rnd() % 8 == 0) d.struct_size = (uint32_t)(rnd() % 200);
    gz_plan_info info;
    const int sm = sms[rnd() % 8];
    const gz_status st = gz_gemm_desc_validate(&d, sm, (rnd() % 8) ? &info : NULL);
    if (st == GZ_OK) {
      ++ok;
    } else {
      ++rejected;
    }
    if (gz_status_string(st) == NULL) return 2;
    int64_t b = 0, e = 0;
    const int parts = (int)(rnd() % 10) - 1, part = (int)(rnd() % 10) - 1;
    if (gz_partition_columns(d.n, parts, part, (int64_t)(rnd() % 40) - 2, &b, &e) == GZ_OK && (b < 0 || e < b || e > d.n)) {
      printf("partition out of range\n");
      return 3;
    }
  }
  for (unsigned tm = 1; tm < 24; ++tm)
    for (unsigned tn = 1; tn < 24; ++tn)
      for (unsigned g = 0; g < 6; ++g)
        for (unsigned t = 0; t < tm * tn; ++t) {
          unsigned a = ~0u, b = ~0u;
          gz_tile_coords(tm, tn, g, t, &a, &b);
          if (a >= tm || b >= tn) {
            printf("tile out of range\n");
            return 4;
          }
        }
  /* entry points that need a plan or a device: null and no-device answers only */
  gz_plan* pl = NULL;
  gz_gemm_desc d;
  memset(&d, 0, sizeof d);
  d.struct_size = sizeof d;
  d.in_type = GZ_DT_BF16;
  d.out_type = GZ_DT_BF16;
  d.m = d.n = d.k = 256;
  const gz_status created = gz_gemm_plan_create(&pl, &d);
  if (created == GZ_OK) gz_gemm_plan_destroy(pl);
  float one = 1.0f, zero = 0.0f;
  (void)gz_gemm_run(NULL, NULL, NULL, NULL, NULL, &one, &zero, NULL);
  (void)gz_gemm_run_host(NULL, NULL, NULL, NULL, NULL, &one, &zero, NULL);
  (void)gz_gemm_plan_destroy(NULL);
  (void)gz_last_device_status(NULL, NULL, NULL);
  (void)gz_gemm_skinny_static(NULL, NULL, NULL, NULL, NULL, NULL, NULL, NULL);
  (void)gz_fill(NULL, 0, 0, 0, 0, 0, 0.0f, NULL);
  printf("HOST FUZZ OK accepted=%ld rejected=%ld plan_create=%d version=%d\n", ok, rejected, (int)created, gz_version());
  return 0;
}
