// CPU oracle for the E5M2EffMA hot path -- TEST INFRASTRUCTURE, NOT PRODUCT CODE.
//
// A from-scratch restatement, in plain C++, of the host emulations the reference library uses
// to check its own kernels.  Only the test-suite, the smoke check and the cpu_baseline /
// reference legs of the benchmark may load this library; the CUDA library never does.
//
// What each part follows (paths are relative to the reference project):
//   element decode / encode ....... tests/test_util.h:21-56, src/e5m2effma.cuh:83-124
//   cast .......................... src/e5m2effma.cu:53-63 (with tests/test_e5m2effma.cu:161,176)
//   GEMM, ascending-k FMA chain ... tests/test_util.h:111-123,139-143
//   GEMV lane order ............... tests/test_util.h:124-138
//   Adam / AdamW .................. tests/test_adamw.cu:30-44, src/adamw_e5m2effma.cu:151-156
//   one MAC, BF16 accumulator ..... tests/e5m2effma_ref.h:114-129 (its exact model; here
//                                   RN_BF16(fmaf(a, b, acc)), which equals it because the
//                                   FMA is exact before its single rounding ... see orc_lane)
//
// Parity is pinned: tests/test_oracle_pins.py checks these functions against the reference's own
// exact one-MAC model and host encoders (compiled from the reference sources into oracle/_ref by
// oracle/Makefile) and against golden vectors generated from them (tests/golden).
//
// Build with -ffp-contract=off: every FMA below is written explicitly, as in the reference build.
#include <cmath>
#include <cstdint>
#include <cstring>
#include <cstdlib>
#include <vector>
#include <algorithm>
#ifdef _OPENMP
#include <omp.h>
#endif

// dtype codes of the C interface (include/e5m2effma.h)
enum { DT_E4M3 = 0, DT_BF16 = 1, DT_FP16 = 2, DT_FP32 = 3, DT_E5M2 = 4 };

static inline uint32_t f2u(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }
static inline float u2f(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }

// ---- decoders -----------------------------------------------------------------------------------
// E4M3: 1-4-3, bias 7, no Inf, 0x7F / 0xFF NaN.  E5M2: 1-5-2, bias 15, IEEE-like Inf / NaN.
static inline float dec_e4m3(uint8_t b) {
  const int e = (b >> 3) & 15, f = b & 7;
  float v;
  if ((b & 0x7F) == 0x7F) v = NAN;
  else if (e) v = ldexpf(1.f + (float)f / 8.f, e - 7);
  else v = ldexpf((float)f / 8.f, -6);
  return (b & 0x80) ? -v : v;
}
static inline float dec_e5m2(uint8_t b) {
  const int e = (b >> 2) & 31, f = b & 3;
  float v;
  if (e == 31) v = f ? NAN : INFINITY;
  else if (e) v = ldexpf(1.f + (float)f / 4.f, e - 15);
  else v = ldexpf((float)f / 4.f, -14);
  return (b & 0x80) ? -v : v;
}
static inline float dec_bf16(uint16_t h) { return u2f((uint32_t)h << 16); }
static inline float dec_f16(uint16_t h) {
  const uint32_t s = (uint32_t)(h & 0x8000) << 16, e = (h >> 10) & 31, f = h & 0x3FF;
  if (e == 31) return f ? u2f(0x7FFFFFFFu) : u2f(s | 0x7F800000u);  // NaN canonical, as cvt.f32.f16
  if (e) return u2f(s | ((e + 112) << 23) | (f << 13));
  const float v = ldexpf((float)f, -24);
  return s ? -v : v;
}

// ---- encoders -----------------------------------------------------------------------------------
// FP32 -> BF16, nearest even, every NaN -> 0x7FC0.
static inline uint16_t enc_bf16(float v) {
  const uint32_t u = f2u(v);
  if ((u & 0x7FFFFFFFu) > 0x7F800000u) return 0x7FC0;
  return (uint16_t)((u + 0x7FFFu + ((u >> 16) & 1u)) >> 16);
}
// FP32 -> FP16, nearest even, every NaN -> 0x7FFF (what __float2half_rn produces).
static inline uint16_t enc_f16(float v) {
  const uint32_t u = f2u(v), s = (u >> 16) & 0x8000u, a = u & 0x7FFFFFFFu;
  if (a > 0x7F800000u) return 0x7FFF;
  if (a >= 0x477FF000u) return (uint16_t)(s | 0x7C00u);   // >= 65520 rounds to Inf (Inf included)
  if (a < 0x33000001u) return (uint16_t)s;                // <= 2^-25: rounds to zero (tie to even)
  if (a < 0x38800000u) {                                  // subnormal half: grid 2^-24
    const float m = u2f(a) * 16777216.0f + 8388608.0f;    // exact scaling, RNE to an integer
    return (uint16_t)(s | (f2u(m) - 0x4B000000u));
  }
  const uint32_t r = a + 0xFFFu + ((a >> 13) & 1u);
  return (uint16_t)(s | ((r >> 13) - (112u << 10)));
}
// FP32 -> FP8 code by its definition: the nearest finite value, ties to the even code, values at
// or beyond the largest finite magnitude (Inf too) saturate, NaN -> 0x7F without a sign.  Written
// as a search over the midpoints of neighbouring codes so that it shares nothing with the
// bit-twiddling encoders it is used to check.
static float g_mid4[126], g_mid5[123], g_lut4[256], g_lut5[256];   // midpoints; decoded value of every code
static bool g_tables = false;
static void build_tables() {
  if (g_tables) return;
  for (int c = 0; c < 256; ++c) { g_lut4[c] = dec_e4m3((uint8_t)c); g_lut5[c] = dec_e5m2((uint8_t)c); }
  for (int c = 0; c < 126; ++c) g_mid4[c] = 0.5f * (dec_e4m3((uint8_t)c) + dec_e4m3((uint8_t)(c + 1)));
  for (int c = 0; c < 123; ++c) g_mid5[c] = 0.5f * (dec_e5m2((uint8_t)c) + dec_e5m2((uint8_t)(c + 1)));
  g_tables = true;
}
template <bool E5>
static inline uint8_t enc_fp8(float x) {
  const uint32_t u = f2u(x), s = (u >> 24) & 0x80u;
  const int top = E5 ? 123 : 126;
  const float *mid = E5 ? g_mid5 : g_mid4;
  const float a = fabsf(x);
  if (a != a) return 0x7F;
  if (a >= (E5 ? 57344.f : 448.f)) return (uint8_t)(s | (uint32_t)top);
  int lo = 0, hi = top;
  while (lo < hi) {
    const int c = (lo + hi) >> 1;
    if (a < mid[c] || (a == mid[c] && !(c & 1))) hi = c; else lo = c + 1;
  }
  return (uint8_t)(s | (uint32_t)lo);
}

// max(mx, a) for a statistic that starts at 0: a NaN never replaces mx, Inf does (what fmaxf gives
// the kernels; spelled as a comparison so that no compiler rewrite can change the NaN behaviour)
static inline float amax_step(float mx, float a) { return a > mx ? a : mx; }

static inline size_t esize(int t) { return (t == DT_E4M3 || t == DT_E5M2) ? 1 : t == DT_FP32 ? 4 : 2; }
static inline bool is_fp8(int t) { return t == DT_E4M3 || t == DT_E5M2; }

// value i of a typed array; FP8 values are multiplied by sinv (one FP32 multiply)
static inline float hload(int t, const void *p, size_t i, float sinv) {
  switch (t) {
    case DT_E4M3: return dec_e4m3(((const uint8_t *)p)[i]) * sinv;
    case DT_E5M2: return dec_e5m2(((const uint8_t *)p)[i]) * sinv;
    case DT_BF16: return dec_bf16(((const uint16_t *)p)[i]);
    case DT_FP16: return dec_f16(((const uint16_t *)p)[i]);
    default: return ((const float *)p)[i];
  }
}
static inline void hstore(int t, void *p, size_t i, float v, float qs) {
  switch (t) {
    case DT_E4M3: ((uint8_t *)p)[i] = enc_fp8<false>(v * qs); break;
    case DT_E5M2: ((uint8_t *)p)[i] = enc_fp8<true>(v * qs); break;
    case DT_BF16: ((uint16_t *)p)[i] = enc_bf16(v); break;
    case DT_FP16: ((uint16_t *)p)[i] = enc_f16(v); break;
    default: ((float *)p)[i] = v;
  }
}

#define CLONES __attribute__((target_clones("arch=x86-64-v4", "arch=x86-64-v3", "default")))

extern "C" {

int orc_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}
void orc_set_threads(int n) {
#ifdef _OPENMP
  if (n > 0) omp_set_num_threads(n);
#else
  (void)n;
#endif
}

float orc_decode(int dtype, const void *p, size_t i, float sinv) { return hload(dtype, p, i, sinv); }
void orc_encode(int dtype, void *p, size_t i, float v, float qs) { build_tables(); hstore(dtype, p, i, v, qs); }

// array forms for numpy callers
void orc_decode_n(int dtype, const void *p, size_t n, float sinv, float *out) {
#pragma omp parallel for schedule(static)
  for (size_t i = 0; i < n; ++i) out[i] = hload(dtype, p, i, sinv);
}
void orc_encode_n(int dtype, void *p, size_t n, const float *v, float qs) {
  build_tables();
#pragma omp parallel for schedule(static)
  for (size_t i = 0; i < n; ++i) hstore(dtype, p, i, v[i], qs);
}

// One MAC with a BF16 accumulator: RN_BF16(acc + a*b).  fa / fb: 0 = E4M3, 1 = E5M2 (the numbering
// of the reference's exact model).  fmaf is exact up to its single rounding to FP32; the FP32 result
// then rounds to BF16.  The reference proves (and its exhaustive test confirms) that this double
// rounding equals the single rounding of the exact sum for every finite operand triple.
uint32_t orc_lane(uint32_t a, uint32_t b, uint32_t acc, int fa, int fb) {
  const float va = fa ? dec_e5m2((uint8_t)a) : dec_e4m3((uint8_t)a);
  const float vb = fb ? dec_e5m2((uint8_t)b) : dec_e4m3((uint8_t)b);
  return enc_bf16(fmaf(va, vb, dec_bf16((uint16_t)acc)));
}

void orc_lane_n(size_t n, const uint32_t *a, const uint32_t *b, const uint32_t *acc, int fa, int fb, uint32_t *out) {
  for (size_t i = 0; i < n; ++i) out[i] = orc_lane(a[i], b[i], acc[i], fa, fb);
}

// Cast: v = src * scale_inv (FP8 source only); amax = max |v| via fmaxf (NaN drops out, Inf stays),
// max-reduced into *amax; dst = convert(v) (FP8 destination: v * scale first).
void orc_cast(int sdt, const void *src, int ddt, void *dst, size_t count, const float *scale_inv,
              const float *scale, float *amax) {
  build_tables();
  const float sinv = is_fp8(sdt) && scale_inv ? *scale_inv : 1.f;
  const float qs = is_fp8(ddt) && scale ? *scale : 1.f;
  float mx = 0.f;
#pragma omp parallel for schedule(static) reduction(max : mx)
  for (size_t i = 0; i < count; ++i) {
    const float v = hload(sdt, src, i, sinv);
    mx = amax_step(mx, fabsf(v));
    hstore(ddt, dst, i, v, qs);
  }
  if (amax && mx > 0.f) *amax = fmaxf(*amax, mx);
}

// ---- GEMM -----------------------------------------------------------------------------------
struct GemmArgs {
  int transa, transb, m, n, k;
  float alpha, beta;
  const void *a; int a_dtype; const float *a_sinv; int a_outer; int lda;
  const void *b; int b_dtype; const float *b_sinv; int b_outer; int ldb;
  const void *c; int c_dtype; const float *c_sinv; int ldc;   // c == NULL: no C term (beta ignored)
  void *d; int d_dtype; const float *d_scale; int ldd;
  const void *bias; int bias_dtype;
  float *amax;
};

// op(A) decoded to FP32 as At[kk * m + i]; op(B) as Bt[j * k + kk]  (raw values, scale 1)
// raw operand element (scale 1); FP8 through the table of decoded codes (same values as dec_*)
static inline float operand_value(int t, const void *p, size_t i) {
  if (t == DT_E4M3) return g_lut4[((const uint8_t *)p)[i]];
  if (t == DT_E5M2) return g_lut5[((const uint8_t *)p)[i]];
  return hload(t, p, i, 1.f);
}
static void decode_operands(const GemmArgs &g, std::vector<float> &At, std::vector<float> &Bt, int j0, int j1) {
  build_tables();
  const bool a_kc = g.transa == 1, b_kc = g.transb == 0;
  At.resize((size_t)g.k * g.m);
  if (a_kc) {   // walk the storage rows (K contiguous), 16 x 16 blocks keep both sides in cache lines
#pragma omp parallel for schedule(static)
    for (int ib = 0; ib < g.m; ib += 16)
      for (int kb = 0; kb < g.k; kb += 16)
        for (int i = ib; i < std::min(g.m, ib + 16); ++i)
          for (int kk = kb; kk < std::min(g.k, kb + 16); ++kk)
            At[(size_t)kk * g.m + i] = operand_value(g.a_dtype, g.a, (size_t)i * g.lda + kk);
  } else {
#pragma omp parallel for schedule(static)
    for (int kk = 0; kk < g.k; ++kk)
      for (int i = 0; i < g.m; ++i) At[(size_t)kk * g.m + i] = operand_value(g.a_dtype, g.a, (size_t)kk * g.lda + i);
  }
  Bt.resize((size_t)g.k * (j1 - j0));
#pragma omp parallel for schedule(static)
  for (int j = j0; j < j1; ++j)
    for (int kk = 0; kk < g.k; ++kk)
      Bt[(size_t)(j - j0) * g.k + kk] = operand_value(g.b_dtype, g.b, b_kc ? (size_t)j * g.ldb + kk : (size_t)kk * g.ldb + j);
}

// Ascending-k FMA chains for a 64-row x 4-column block over k-steps [k0, k1), continuing from and
// writing back to the accumulators acc0..acc3 (64 floats each).  Splitting k into blocks and
// parking the partial sums in memory in between does not change any output's operation order.
// ap: packed op(A) rows of this block, ap[kk * 64 + r].
CLONES static void chain_block(const float *ap, int k0, int k1, const float *b0, const float *b1, const float *b2,
                               const float *b3, float *acc0, float *acc1, float *acc2, float *acc3) {
  float a0[64], a1[64], a2[64], a3[64];
  for (int i = 0; i < 64; ++i) { a0[i] = acc0[i]; a1[i] = acc1[i]; a2[i] = acc2[i]; a3[i] = acc3[i]; }
  for (int kk = k0; kk < k1; ++kk) {
    const float *ar = ap + (size_t)kk * 64;
    const float x0 = b0[kk], x1 = b1[kk], x2 = b2[kk], x3 = b3[kk];
    for (int i = 0; i < 64; ++i) {
      const float av = ar[i];
      a0[i] = fmaf(av, x0, a0[i]); a1[i] = fmaf(av, x1, a1[i]);
      a2[i] = fmaf(av, x2, a2[i]); a3[i] = fmaf(av, x3, a3[i]);
    }
  }
  for (int i = 0; i < 64; ++i) { acc0[i] = a0[i]; acc1[i] = a1[i]; acc2[i] = a2[i]; acc3[i] = a3[i]; }
}

// The GEMV kernel of the reference sums in another order: lane l takes k = 256c + 8l + j
// (c ascending, j = 0..7) as one FMA chain, then the 32 lane sums meet in an xor-butterfly
// with offsets 16, 8, 4, 2, 1 (plain FP32 adds); lane 0's value is the result.
static float gemv_order_acc(const float *At, int m, int k, const float *bcol, int i) {
  float lanes[32];
  for (int l = 0; l < 32; ++l) {
    float p = 0.f;
    for (int kb = 8 * l; kb < k; kb += 256)
      for (int jj = 0; jj < 8; ++jj) p = fmaf(At[(size_t)(kb + jj) * m + i], bcol[kb + jj], p);
    lanes[l] = p;
  }
  for (int o = 16; o; o >>= 1) {
    float nx[32];
    for (int l = 0; l < 32; ++l) nx[l] = lanes[l] + lanes[l ^ o];
    memcpy(lanes, nx, sizeof nx);
  }
  return lanes[0];
}

static inline float out_scale(const GemmArgs &g, int i, int j) {
  const float a = is_fp8(g.a_dtype) && g.a_sinv ? (g.a_outer ? g.a_sinv[i] : g.a_sinv[0]) : 1.f;
  const float b = is_fp8(g.b_dtype) && g.b_sinv ? (g.b_outer ? g.b_sinv[j] : g.b_sinv[0]) : 1.f;
  return (g.alpha * a) * b;
}

// Epilogue of one output, the documented order; returns |v|.
static inline float finish(const GemmArgs &g, int i, int j, float acc, float csinv, float qs) {
  float v = acc * out_scale(g, i, j);
  if (g.bias) v = v + hload(g.bias_dtype, g.bias, (size_t)i, 1.f);
  if (g.c && g.beta != 0.f) v = fmaf(g.beta, hload(g.c_dtype, g.c, (size_t)j * g.ldc + i, csinv), v);
  hstore(g.d_dtype, g.d, (size_t)j * g.ldd + i, v, qs);
  return fabsf(v);
}

// order: 0 = ascending-k chain (tiled kernel of the reference), 1 = reference GEMV lane order.
// Columns [j0, j1) only (the others are left untouched) so that a caller can time or check a slab.
void orc_gemm_cols(const GemmArgs *gp, int order, int j0, int j1) {
  build_tables();
  const GemmArgs &g = *gp;
  if (g.m <= 0 || j1 <= j0) return;
  std::vector<float> At, Bt;
  decode_operands(g, At, Bt, j0, j1);
  const float csinv = g.c && is_fp8(g.c_dtype) && g.c_sinv ? *g.c_sinv : 1.f;
  const float qs = is_fp8(g.d_dtype) && g.d_scale ? *g.d_scale : 1.f;
  float mx = 0.f;
  const int nj = j1 - j0, njp = (nj + 3) / 4 * 4, nib = (g.m + 63) / 64;
  const int KB = 256;   // k-block: 64 rows x 256 k of packed A (64 KiB) stay cache-resident over all columns
#pragma omp parallel reduction(max : mx)
  {
    std::vector<float> ap((size_t)64 * std::max(g.k, 1)), acc((size_t)njp * 64), zero((size_t)std::max(g.k, 1), 0.f);
#pragma omp for schedule(dynamic, 1)
    for (int ibk = 0; ibk < nib; ++ibk) {
      const int i0 = ibk * 64, ib = std::min(64, g.m - i0);
      if (order == 0) {
        for (int kk = 0; kk < g.k; ++kk) {
          const float *src = At.data() + (size_t)kk * g.m + i0;
          float *dst = ap.data() + (size_t)kk * 64;
          for (int r = 0; r < 64; ++r) dst[r] = r < ib ? src[r] : 0.f;
        }
        std::fill(acc.begin(), acc.end(), 0.f);
        for (int k0 = 0; k0 < g.k; k0 += KB) {
          const int k1 = std::min(g.k, k0 + KB);
          for (int jj = 0; jj < njp; jj += 4) {
            const float *bc[4];
            for (int t = 0; t < 4; ++t) bc[t] = jj + t < nj ? Bt.data() + (size_t)(jj + t) * g.k : zero.data();
            float *a = acc.data() + (size_t)jj * 64;
            chain_block(ap.data(), k0, k1, bc[0], bc[1], bc[2], bc[3], a, a + 64, a + 128, a + 192);
          }
        }
      } else {
        for (int jj = 0; jj < nj; ++jj)
          for (int i = 0; i < ib; ++i)
            acc[(size_t)jj * 64 + i] = gemv_order_acc(At.data(), g.m, g.k, Bt.data() + (size_t)jj * g.k, i0 + i);
      }
      for (int jj = 0; jj < nj; ++jj)
        for (int i = 0; i < ib; ++i) mx = amax_step(mx, finish(g, i0 + i, j0 + jj, acc[(size_t)jj * 64 + i], csinv, qs));
    }
  }
  if (g.amax && mx > 0.f) *g.amax = fmaxf(*g.amax, mx);
}
void orc_gemm(const GemmArgs *g, int order) { orc_gemm_cols(g, order, 0, g->n); }

// Wide reference for the tolerance of tensor-core kernels, columns [j0, j1):
//   ref[(j-j0) * m + i] = the epilogue value v evaluated in double from the exact products,
//   mag[(j-j0) * m + i] = |s| * sum_k |a*b|   (the factor of the accumulation-order bound),
//   fix[(j-j0) * m + i] = |bias| + |beta*C|   (terms added in FP32 after the sum).
void orc_gemm_wide(const GemmArgs *gp, int j0, int j1, double *ref, double *mag, double *fix) {
  const GemmArgs &g = *gp;
  if (g.m <= 0 || j1 <= j0) return;
  std::vector<float> At, Bt;
  decode_operands(g, At, Bt, j0, j1);
  const float csinv = g.c && is_fp8(g.c_dtype) && g.c_sinv ? *g.c_sinv : 1.f;
#pragma omp parallel for schedule(dynamic, 1)
  for (int j = j0; j < j1; ++j) {
    std::vector<double> s((size_t)g.m, 0.0), sa((size_t)g.m, 0.0);
    const float *bcol = Bt.data() + (size_t)(j - j0) * g.k;
    for (int kk = 0; kk < g.k; ++kk) {
      const double x = bcol[kk];
      const float *ar = At.data() + (size_t)kk * g.m;
      for (int i = 0; i < g.m; ++i) { const double p = (double)ar[i] * x; s[i] += p; sa[i] += fabs(p); }
    }
    for (int i = 0; i < g.m; ++i) {
      const double sc = out_scale(g, i, j);
      double v = s[i] * sc, f = 0.0;
      if (g.bias) { const double b = hload(g.bias_dtype, g.bias, (size_t)i, 1.f); v += b; f += fabs(b); }
      if (g.c && g.beta != 0.f) {
        const double c = (double)g.beta * hload(g.c_dtype, g.c, (size_t)j * g.ldc + i, csinv);
        v += c; f += fabs(c);
      }
      const size_t o = (size_t)(j - j0) * g.m + i;
      ref[o] = v; mag[o] = sa[i] * fabs(sc); fix[o] = f;
    }
  }
}

// ---- Adam / AdamW -----------------------------------------------------------------------------
struct AdamCfg { float lr, beta1, beta2, eps, weight_decay; int step, adamw, bias_correction; float grad_scale; };

void orc_adam(const AdamCfg *cfg, size_t count, void *p_, int pt, const void *g_, int gt, void *m_, void *v_,
              int mt, void *q_, int qt, const float *qscale, float *amax) {
  build_tables();
  const float omb1 = (float)(1.0 - (double)cfg->beta1), omb2 = (float)(1.0 - (double)cfg->beta2);
  const float rbc1 = cfg->bias_correction ? (float)(1.0 / (1.0 - pow((double)cfg->beta1, cfg->step))) : 1.f;
  const float rbc2 = cfg->bias_correction ? (float)(1.0 / (1.0 - pow((double)cfg->beta2, cfg->step))) : 1.f;
  const float lr_wd = (float)((double)cfg->lr * cfg->weight_decay);
  const float gs = cfg->grad_scale == 0.f ? 1.f : cfg->grad_scale;
  const float qs = q_ && qscale ? *qscale : 1.f;
  float mx = 0.f;
#pragma omp parallel for schedule(static) reduction(max : mx)
  for (size_t i = 0; i < count; ++i) {
    float g = hload(gt, g_, i, 1.f) * gs, p = hload(pt, p_, i, 1.f);
    if (!cfg->adamw) g = fmaf(cfg->weight_decay, p, g);
    const float m = fmaf(cfg->beta1, hload(mt, m_, i, 1.f), omb1 * g);
    const float v = fmaf(cfg->beta2, hload(mt, v_, i, 1.f), omb2 * (g * g));
    const float u = (m * rbc1) / (sqrtf(v * rbc2) + cfg->eps);
    if (cfg->adamw) p = fmaf(-lr_wd, p, p);
    p = fmaf(-cfg->lr, u, p);
    hstore(pt, p_, i, p, 1.f); hstore(mt, m_, i, m, 1.f); hstore(mt, v_, i, v, 1.f);
    if (q_) { hstore(qt, q_, i, p, qs); mx = amax_step(mx, fabsf(p)); }
  }
  if (q_ && amax && mx > 0.f) *amax = fmaxf(*amax, mx);
}

}  // extern "C"
