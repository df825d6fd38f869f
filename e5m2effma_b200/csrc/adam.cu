// e5ma_adam: fused Adam / AdamW step, optional FP8 weight copy and its amax, one pass over HBM.
//
// Interface, validation order and the per-element arithmetic follow reference
// src/adamw_e5m2effma.cu:125-168 and include/e5m2effma.h:83-94 (IEEE division and square root,
// explicit FMAs, scalar factors prepared in double on the host).  The kernel is new: every array is
// streamed once with 16-byte accesses and cache-streaming hints, 8 elements per thread and step,
// a grid sized to the SM count, and one amax atomic per block.
//
// Algorithmic traffic per element for BF16 param/grad/moments with an FP8 copy:
// read p, g, m, v (8 B) + write p, m, v (6 B) + write q (1 B) = 15 B.
#include <math.h>
#include "common.cuh"

namespace e5b {

struct AdamScalars {
  float lr, beta1, beta2, omb1, omb2, rbc1, rbc2, eps, lr_wd, wd, gscale;
  int adamw;
};

__device__ __forceinline__ void adam_update(const AdamScalars &a, float g, float &p, float &m, float &v) {
  g = __fmul_rn(g, a.gscale);
  if (!a.adamw) g = __fmaf_rn(a.wd, p, g);
  m = __fmaf_rn(a.beta1, m, __fmul_rn(a.omb1, g));
  v = __fmaf_rn(a.beta2, v, __fmul_rn(a.omb2, __fmul_rn(g, g)));
  const float den = __fadd_rn(__fsqrt_rn(__fmul_rn(v, a.rbc2)), a.eps);
  const float u = __fdiv_rn(__fmul_rn(m, a.rbc1), den);
  if (a.adamw) p = __fmaf_rn(-a.lr_wd, p, p);
  p = __fmaf_rn(-a.lr, u, p);
}

// 8 consecutive elements starting at element i (i % 8 == 0, base 16-byte aligned)
template <int T>
__device__ __forceinline__ void load8(const void *base, size_t i, float x[8]) {
  if (T == E5MA_FP32) {
    const float4 *p = reinterpret_cast<const float4 *>(base) + i / 4;
    const float4 a = __ldcs(p), b = __ldcs(p + 1);
    x[0] = a.x; x[1] = a.y; x[2] = a.z; x[3] = a.w; x[4] = b.x; x[5] = b.y; x[6] = b.z; x[7] = b.w;
  } else {
    const uint4 a = __ldcs(reinterpret_cast<const uint4 *>(base) + i / 8);
    const uint32_t w[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      if (T == E5MA_BF16) { x[2 * e] = __uint_as_float(w[e] << 16); x[2 * e + 1] = __uint_as_float(w[e] & 0xFFFF0000u); }
      else { const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&w[e])); x[2 * e] = f.x; x[2 * e + 1] = f.y; }
    }
  }
}
template <int T>
__device__ __forceinline__ void store8(void *base, size_t i, const float x[8]) {
  if (T == E5MA_FP32) {
    float4 *p = reinterpret_cast<float4 *>(base) + i / 4;
    __stcs(p, make_float4(x[0], x[1], x[2], x[3]));
    __stcs(p + 1, make_float4(x[4], x[5], x[6], x[7]));
  } else {
    __stcs(reinterpret_cast<uint4 *>(base) + i / 8,
           make_uint4(enc_bf16x2(x[0], x[1]), enc_bf16x2(x[2], x[3]), enc_bf16x2(x[4], x[5]), enc_bf16x2(x[6], x[7])));
  }
}

// PT param dtype (FP32 / BF16), GT grad dtype (FP32 / BF16 / FP16), MT moment dtype (FP32 / BF16),
// QT dtype of the FP8 copy or -1 for none.  VEC: all pointers 16-byte aligned (the copy 8-byte);
// then groups of 8 elements use vector accesses and only count % 8 trailing elements go one by one.
// Both paths evaluate adam_update, so an element's result does not depend on the path.
template <int PT, int GT, int MT, int QT, bool VEC>
__global__ void __launch_bounds__(256) adam_kernel(AdamScalars a, size_t count, void *__restrict__ p_,
                                                   const void *__restrict__ g_, void *__restrict__ m_,
                                                   void *__restrict__ v_, uint8_t *__restrict__ q_,
                                                   const float *qscale_p, float *amax) {
  const float qs = QT != -1 ? ld_or_one(qscale_p) : 1.f;
  float mx = 0.f;
  const size_t tid = (size_t)blockIdx.x * blockDim.x + threadIdx.x, nthr = (size_t)gridDim.x * blockDim.x;
  const size_t groups = VEC ? count / 8 : 0;
  for (size_t gi = tid; gi < groups; gi += nthr) {
    const size_t i = gi * 8;
    float g[8], p[8], m[8], v[8];
    load8<GT>(g_, i, g); load8<PT>(p_, i, p); load8<MT>(m_, i, m); load8<MT>(v_, i, v);
#pragma unroll
    for (int e = 0; e < 8; ++e) adam_update(a, g[e], p[e], m[e], v[e]);
    store8<PT>(p_, i, p); store8<MT>(m_, i, m); store8<MT>(v_, i, v);
    if (QT != -1) {
      constexpr int Q = QT != -1 ? QT : E5MA_E4M3;
      uint32_t w[2];
#pragma unroll
      for (int h = 0; h < 2; ++h)
        w[h] = enc_fp8x2<Q>(__fmul_rn(p[4 * h], qs), __fmul_rn(p[4 * h + 1], qs)) |
               (enc_fp8x2<Q>(__fmul_rn(p[4 * h + 2], qs), __fmul_rn(p[4 * h + 3], qs)) << 16);
      __stcs(reinterpret_cast<uint2 *>(q_ + i), make_uint2(w[0], w[1]));
#pragma unroll
      for (int e = 0; e < 8; ++e) mx = fmaxf(mx, fabsf(p[e]));
    }
  }
  for (size_t i = groups * 8 + tid; i < count; i += nthr) {
    float p = load_elem(PT, p_, i, 1.f), m = load_elem(MT, m_, i, 1.f), v = load_elem(MT, v_, i, 1.f);
    adam_update(a, load_elem(GT, g_, i, 1.f), p, m, v);
    store_elem(PT, p_, i, p, 1.f);
    store_elem(MT, m_, i, m, 1.f);
    store_elem(MT, v_, i, v, 1.f);
    if (QT != -1) {
      constexpr int Q = QT != -1 ? QT : E5MA_E4M3;
      q_[i] = (uint8_t)enc_fp8<Q>(__fmul_rn(p, qs));
      mx = fmaxf(mx, fabsf(p));
    }
  }
  if (QT != -1 && amax) block_amax(amax, mx);
}

struct AdamPtrs { void *p; const void *g; void *m, *v; uint8_t *q; const float *qs; float *amax; };

template <int PT, int GT, int MT, int QT>
static cudaError_t adam_launch(const AdamScalars &a, size_t count, const AdamPtrs &x, int sms, cudaStream_t s) {
  const auto a16 = [](const void *p) { return ((uintptr_t)p & 15u) == 0; };
  const bool vec = a16(x.p) && a16(x.g) && a16(x.m) && a16(x.v) && ((uintptr_t)x.q & 7u) == 0;
  const size_t work = vec ? count / 8 + (count % 8) : count;
  size_t blocks = (work + 255) / 256;
  const size_t cap = (size_t)sms * 16;
  if (blocks > cap) blocks = cap;
  if (blocks == 0) blocks = 1;
  if (vec) adam_kernel<PT, GT, MT, QT, true><<<(unsigned)blocks, 256, 0, s>>>(a, count, x.p, x.g, x.m, x.v, x.q, x.qs, x.amax);
  else adam_kernel<PT, GT, MT, QT, false><<<(unsigned)blocks, 256, 0, s>>>(a, count, x.p, x.g, x.m, x.v, x.q, x.qs, x.amax);
  return cudaGetLastError();
}
template <int PT, int GT, int MT>
static cudaError_t adam_q(int qt, const AdamScalars &a, size_t count, const AdamPtrs &x, int sms, cudaStream_t s) {
  if (!x.q) return adam_launch<PT, GT, MT, -1>(a, count, x, sms, s);
  if (qt == E5MA_E5M2) return adam_launch<PT, GT, MT, E5MA_E5M2>(a, count, x, sms, s);
  return adam_launch<PT, GT, MT, E5MA_E4M3>(a, count, x, sms, s);
}
template <int PT, int GT>
static cudaError_t adam_m(int mt, int qt, const AdamScalars &a, size_t count, const AdamPtrs &x, int sms, cudaStream_t s) {
  if (mt == E5MA_BF16) return adam_q<PT, GT, E5MA_BF16>(qt, a, count, x, sms, s);
  return adam_q<PT, GT, E5MA_FP32>(qt, a, count, x, sms, s);
}
template <int PT>
static cudaError_t adam_g(int gt, int mt, int qt, const AdamScalars &a, size_t count, const AdamPtrs &x, int sms, cudaStream_t s) {
  if (gt == E5MA_BF16) return adam_m<PT, E5MA_BF16>(mt, qt, a, count, x, sms, s);
  if (gt == E5MA_FP16) return adam_m<PT, E5MA_FP16>(mt, qt, a, count, x, sms, s);
  return adam_m<PT, E5MA_FP32>(mt, qt, a, count, x, sms, s);
}

}  // namespace e5b

extern "C" e5ma_status e5ma_adam(const e5ma_adam_config *cfg, size_t count, const e5ma_tensor *param,
                                 const e5ma_tensor *grad, const e5ma_tensor *exp_avg,
                                 const e5ma_tensor *exp_avg_sq, const e5ma_tensor *param_fp8,
                                 cudaStream_t stream) {
  using namespace e5b;
  clear_error();
  if (!cfg || !param || !grad || !exp_avg || !exp_avg_sq || !param->data || !grad->data || !exp_avg->data ||
      !exp_avg_sq->data)
    return fail(E5MA_INVALID_VALUE, "e5ma_adam: cfg, param, grad, exp_avg, exp_avg_sq or their data is NULL");
  if (cfg->step < 1) return fail(E5MA_INVALID_VALUE, "e5ma_adam: step = %d, must be >= 1", cfg->step);
  const auto state_type = [](int t) { return t == E5MA_FP32 || t == E5MA_BF16; };
  if (!state_type(param->dtype))
    return fail(E5MA_NOT_SUPPORTED, "e5ma_adam: param must be FP32 or BF16 (dtype %d)", (int)param->dtype);
  if (!state_type(exp_avg->dtype) || exp_avg_sq->dtype != exp_avg->dtype)
    return fail(E5MA_NOT_SUPPORTED, "e5ma_adam: exp_avg and exp_avg_sq must both be FP32 or both BF16 (dtypes %d, %d)",
                (int)exp_avg->dtype, (int)exp_avg_sq->dtype);
  if (grad->dtype != E5MA_FP32 && grad->dtype != E5MA_BF16 && grad->dtype != E5MA_FP16)
    return fail(E5MA_NOT_SUPPORTED, "e5ma_adam: grad must be FP32, BF16 or FP16 (dtype %d)", (int)grad->dtype);
  const bool copy = param_fp8 && param_fp8->data;
  if (copy && !is_fp8(param_fp8->dtype))
    return fail(E5MA_INVALID_VALUE, "e5ma_adam: param_fp8 must have dtype E5MA_E4M3 or E5MA_E5M2 (dtype %d)",
                (int)param_fp8->dtype);
  if (copy && param_fp8->scaling != E5MA_SCALING_TENSOR)
    return fail(E5MA_INVALID_VALUE, "e5ma_adam: param_fp8 takes per-tensor scaling only");
  if (count == 0) return E5MA_OK;
  DeviceProps dp;
  if (e5ma_status st = require_blackwell("e5ma_adam", &dp)) return st;

  AdamScalars a;
  a.lr = cfg->lr; a.beta1 = cfg->beta1; a.beta2 = cfg->beta2; a.eps = cfg->eps; a.wd = cfg->weight_decay;
  a.omb1 = (float)(1.0 - (double)cfg->beta1);
  a.omb2 = (float)(1.0 - (double)cfg->beta2);
  a.rbc1 = cfg->bias_correction ? (float)(1.0 / (1.0 - pow((double)cfg->beta1, cfg->step))) : 1.f;
  a.rbc2 = cfg->bias_correction ? (float)(1.0 / (1.0 - pow((double)cfg->beta2, cfg->step))) : 1.f;
  a.lr_wd = (float)((double)cfg->lr * cfg->weight_decay);
  a.gscale = cfg->grad_scale == 0.f ? 1.f : cfg->grad_scale;
  a.adamw = cfg->adamw;

  AdamPtrs x;
  x.p = param->data; x.g = grad->data; x.m = exp_avg->data; x.v = exp_avg_sq->data;
  x.q = copy ? (uint8_t *)param_fp8->data : nullptr;
  x.qs = copy ? param_fp8->scale : nullptr;
  x.amax = copy ? param_fp8->amax : nullptr;
  const int qt = copy ? (int)param_fp8->dtype : E5MA_E4M3;
  const cudaError_t err = param->dtype == E5MA_BF16
                              ? adam_g<E5MA_BF16>(grad->dtype, exp_avg->dtype, qt, a, count, x, dp.sms, stream)
                              : adam_g<E5MA_FP32>(grad->dtype, exp_avg->dtype, qt, a, count, x, dp.sms, stream);
  return cuda_fail(err, "e5ma_adam: kernel launch");
}
