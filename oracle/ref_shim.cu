// Thin C exports around host helpers of the reference's own test code, compiled FROM the reference
// sources where they lie (never copied): its FP8 / BF16 encoders (src/e5m2effma.cuh:83-124) and the
// element load / store helpers of its host emulation (tests/test_util.h:21-56).  Used only to pin
// the CPU oracle and to generate golden vectors; builds into oracle/_ref (see oracle/Makefile).
// Compiled for a pre-FP8 architecture because the reference refuses newer ones at compile time;
// only host code is ever run.
#include "tests/test_util.h"
#include "tests/e5m2effma_ref.h"  // exact one-MAC model (array form of tests/ref_capi.cpp)

extern "C" {
float ref_e4(unsigned b) { return e4((uint8_t)b); }
float ref_e5(unsigned b) { return e5((uint8_t)b); }
unsigned ref_to_bf(float v) { return to_bf(v); }
unsigned ref_f32_to_e4m3(float v) { return e5ma::f32_to_e4m3(v); }
unsigned ref_f32_to_e5m2(float v) { return e5ma::f32_to_e5m2(v); }
float ref_hload(int t, const void *p, size_t i, float sinv) { return hload((e5ma_dtype)t, p, i, sinv); }
void ref_hstore(int t, void *p, size_t i, float v, float qs) { hstore((e5ma_dtype)t, p, i, v, qs); }
void ref_hstore_n(int t, void *p, size_t n, const float *v, float qs) {
  for (size_t i = 0; i < n; ++i) hstore((e5ma_dtype)t, p, i, v[i], qs);
}
void ref_lane_n(size_t n, const uint32_t *a, const uint32_t *b, const uint32_t *acc, int fa, int fb, uint32_t *out) {
  for (size_t i = 0; i < n; ++i) out[i] = e5ma_ref::lane(a[i], b[i], acc[i], fa, fb);
}
void ref_hload_n(int t, const void *p, size_t n, float sinv, float *out) {
  for (size_t i = 0; i < n; ++i) out[i] = hload((e5ma_dtype)t, p, i, sinv);
}
}
