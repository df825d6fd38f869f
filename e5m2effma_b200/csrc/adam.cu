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
#include "../../include/e5m2effma_b200.h"

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
// NaN-free groups (the caller has checked): the converter alone is the documented rounding, no patching needed.
template <int T>
__device__ __forceinline__ void store8_nonan(void *base, size_t i, const float x[8]) {
  if (T == E5MA_FP32) {
    float4 *p = reinterpret_cast<float4 *>(base) + i / 4;
    __stcs(p, make_float4(x[0], x[1], x[2], x[3]));
    __stcs(p + 1, make_float4(x[4], x[5], x[6], x[7]));
  } else {
    __stcs(reinterpret_cast<uint4 *>(base) + i / 8,
           make_uint4(cvt_bf16x2_raw(x[0], x[1]), cvt_bf16x2_raw(x[2], x[3]), cvt_bf16x2_raw(x[4], x[5]), cvt_bf16x2_raw(x[6], x[7])));
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
// Elements [0, count) of one tensor, spread over nthr threads of which this is number tid: groups of 8
// elements with vector accesses when VEC, the rest one by one.  Returns the thread's max |p| (FP8 copy only).
template <int PT, int GT, int MT, int QT, bool VEC>
__device__ __forceinline__ float adam_range(const AdamScalars &a, size_t count, void *__restrict__ p_,
                                            const void *__restrict__ g_, void *__restrict__ m_, void *__restrict__ v_,
                                            uint8_t *__restrict__ q_, float qs, size_t tid, size_t nthr) {
  float mx = 0.f;
  const bool qs_finite = fabsf(qs) <= 3.4028234664e38f;   // an infinite scale turns p = 0 into NaN: no shortcut then
  const size_t groups = VEC ? count / 8 : 0;
  for (size_t gi = tid; gi < groups; gi += nthr) {
    const size_t i = gi * 8;
    float g[8], p[8], m[8], v[8];
    load8<GT>(g_, i, g); load8<PT>(p_, i, p); load8<MT>(m_, i, m); load8<MT>(v_, i, v);
#pragma unroll
    for (int e = 0; e < 8; ++e) adam_update(a, g[e], p[e], m[e], v[e]);
    // The hardware converters differ from the documented encoders only for NaN inputs.  One sum over the group's 24
    // results tells whether any is NaN (a NaN propagates through the adds; Inf - Inf also lands here, harmlessly):
    // without one -- practically always -- the 24 per-value NaN patches are skipped; the values stored are the same.
    float chk = 0.f;
#pragma unroll
    for (int e = 0; e < 8; ++e) chk += (p[e] + m[e]) + v[e];
    const bool clean = qs_finite && !is_nan(chk) && !is_nan(__fmul_rn(chk, qs));   // p = Inf with scale 0 gives NaN too
    if (clean) { store8_nonan<PT>(p_, i, p); store8_nonan<MT>(m_, i, m); store8_nonan<MT>(v_, i, v); }
    else { store8<PT>(p_, i, p); store8<MT>(m_, i, m); store8<MT>(v_, i, v); }
    if (QT != -1) {
      constexpr int Q = QT != -1 ? QT : E5MA_E4M3;
      uint32_t w[2];
      if (clean) {
#pragma unroll
        for (int h = 0; h < 2; ++h)
          w[h] = cvt_fp8x2_raw<Q>(__fmul_rn(p[4 * h], qs), __fmul_rn(p[4 * h + 1], qs)) |
                 (cvt_fp8x2_raw<Q>(__fmul_rn(p[4 * h + 2], qs), __fmul_rn(p[4 * h + 3], qs)) << 16);
      } else {
#pragma unroll
        for (int h = 0; h < 2; ++h)
          w[h] = enc_fp8x2<Q>(__fmul_rn(p[4 * h], qs), __fmul_rn(p[4 * h + 1], qs)) |
                 (enc_fp8x2<Q>(__fmul_rn(p[4 * h + 2], qs), __fmul_rn(p[4 * h + 3], qs)) << 16);
      }
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
  return mx;
}

template <int PT, int GT, int MT, int QT, bool VEC>
__global__ void __launch_bounds__(256) adam_kernel(AdamScalars a, size_t count, void *__restrict__ p_,
                                                   const void *__restrict__ g_, void *__restrict__ m_,
                                                   void *__restrict__ v_, uint8_t *__restrict__ q_,
                                                   const float *qscale_p, float *amax) {
  const float qs = QT != -1 ? ld_or_one(qscale_p) : 1.f;
  const size_t tid = (size_t)blockIdx.x * blockDim.x + threadIdx.x, nthr = (size_t)gridDim.x * blockDim.x;
  const float mx = adam_range<PT, GT, MT, QT, VEC>(a, count, p_, g_, m_, v_, q_, qs, tid, nthr);
  if (QT != -1 && amax) block_amax(amax, mx);
}

// ---- several tensors per launch ------------------------------------------------------------------
// The table travels by value in the kernel parameters (no device-side table to allocate or copy).  Every
// block owns one chunk of MT_CHUNK elements of one tensor; first_block[t] is the number of the first block
// of tensor t, so a block finds its tensor by a short scan.
constexpr int MT_MAX = 24;
constexpr size_t MT_CHUNK = 256 * 8 * 8;
struct AdamTable {
  void *p[MT_MAX]; const void *g[MT_MAX]; void *m[MT_MAX]; void *v[MT_MAX]; uint8_t *q[MT_MAX];
  const float *qs[MT_MAX]; float *amax[MT_MAX];
  size_t count[MT_MAX];
  unsigned first_block[MT_MAX + 1];
  unsigned char vec[MT_MAX];
  int n;
};

template <int PT, int GT, int MT, int QT>
__global__ void __launch_bounds__(256) adam_multi_kernel(AdamScalars a, const __grid_constant__ AdamTable tb) {
  int t = 0;
  while (t + 1 < tb.n && blockIdx.x >= tb.first_block[t + 1]) ++t;
  const size_t begin = (size_t)(blockIdx.x - tb.first_block[t]) * MT_CHUNK;
  const size_t len = tb.count[t] - begin < MT_CHUNK ? tb.count[t] - begin : MT_CHUNK;
  constexpr int PB = elem_bytes(PT), GB = elem_bytes(GT), MB = elem_bytes(MT);
  void *p_ = (uint8_t *)tb.p[t] + begin * PB;
  const void *g_ = (const uint8_t *)tb.g[t] + begin * GB;
  void *m_ = (uint8_t *)tb.m[t] + begin * MB, *v_ = (uint8_t *)tb.v[t] + begin * MB;
  uint8_t *q_ = QT != -1 ? tb.q[t] + begin : nullptr;
  const float qs = QT != -1 ? ld_or_one(tb.qs[t]) : 1.f;
  float mx;   // chunk starts are multiples of 16384 elements, so a tensor's alignment carries over to its chunks
  if (tb.vec[t]) mx = adam_range<PT, GT, MT, QT, true>(a, len, p_, g_, m_, v_, q_, qs, threadIdx.x, 256);
  else mx = adam_range<PT, GT, MT, QT, false>(a, len, p_, g_, m_, v_, q_, qs, threadIdx.x, 256);
  if (QT != -1 && tb.amax[t]) block_amax(tb.amax[t], mx);
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

namespace e5b {
template <int PT, int GT, int MT>
static cudaError_t adam_multi_q(int qt, bool copy, const AdamScalars &a, const AdamTable &tb, unsigned blocks, cudaStream_t s) {
  if (!copy) adam_multi_kernel<PT, GT, MT, -1><<<blocks, 256, 0, s>>>(a, tb);
  else if (qt == E5MA_E5M2) adam_multi_kernel<PT, GT, MT, E5MA_E5M2><<<blocks, 256, 0, s>>>(a, tb);
  else adam_multi_kernel<PT, GT, MT, E5MA_E4M3><<<blocks, 256, 0, s>>>(a, tb);
  return cudaGetLastError();
}
template <int PT, int GT>
static cudaError_t adam_multi_m(int mt, int qt, bool copy, const AdamScalars &a, const AdamTable &tb, unsigned blocks, cudaStream_t s) {
  return mt == E5MA_BF16 ? adam_multi_q<PT, GT, E5MA_BF16>(qt, copy, a, tb, blocks, s)
                         : adam_multi_q<PT, GT, E5MA_FP32>(qt, copy, a, tb, blocks, s);
}
template <int PT>
static cudaError_t adam_multi_g(int gt, int mt, int qt, bool copy, const AdamScalars &a, const AdamTable &tb, unsigned blocks, cudaStream_t s) {
  if (gt == E5MA_BF16) return adam_multi_m<PT, E5MA_BF16>(mt, qt, copy, a, tb, blocks, s);
  if (gt == E5MA_FP16) return adam_multi_m<PT, E5MA_FP16>(mt, qt, copy, a, tb, blocks, s);
  return adam_multi_m<PT, E5MA_FP32>(mt, qt, copy, a, tb, blocks, s);
}
}  // namespace e5b

extern "C" e5ma_status e5b_adam_multi(const e5ma_adam_config *cfg, int num_tensors, const size_t *counts,
                                      const e5ma_tensor *params, const e5ma_tensor *grads, const e5ma_tensor *exp_avgs,
                                      const e5ma_tensor *exp_avg_sqs, const e5ma_tensor *params_fp8, cudaStream_t stream) {
  using namespace e5b;
  clear_error();
  if (!cfg || !counts || !params || !grads || !exp_avgs || !exp_avg_sqs)
    return fail(E5MA_INVALID_VALUE, "e5b_adam_multi: cfg, counts or a tensor list is NULL");
  if (num_tensors < 0) return fail(E5MA_INVALID_VALUE, "e5b_adam_multi: num_tensors = %d", num_tensors);
  if (cfg->step < 1) return fail(E5MA_INVALID_VALUE, "e5b_adam_multi: step = %d, must be >= 1", cfg->step);
  const auto state_type = [](int t) { return t == E5MA_FP32 || t == E5MA_BF16; };
  bool any = false, copy = false;
  int pt = 0, gt = 0, mt = 0, qt = E5MA_E4M3;
  for (int t = 0; t < num_tensors; ++t) {
    if (!params[t].data || !grads[t].data || !exp_avgs[t].data || !exp_avg_sqs[t].data)
      return fail(E5MA_INVALID_VALUE, "e5b_adam_multi: tensor %d has a NULL data pointer", t);
    if (!state_type(params[t].dtype))
      return fail(E5MA_NOT_SUPPORTED, "e5b_adam_multi: param %d must be FP32 or BF16 (dtype %d)", t, (int)params[t].dtype);
    if (!state_type(exp_avgs[t].dtype) || exp_avg_sqs[t].dtype != exp_avgs[t].dtype)
      return fail(E5MA_NOT_SUPPORTED, "e5b_adam_multi: moments of tensor %d must both be FP32 or both BF16", t);
    if (grads[t].dtype != E5MA_FP32 && grads[t].dtype != E5MA_BF16 && grads[t].dtype != E5MA_FP16)
      return fail(E5MA_NOT_SUPPORTED, "e5b_adam_multi: grad %d must be FP32, BF16 or FP16 (dtype %d)", t, (int)grads[t].dtype);
    const bool c = params_fp8 && params_fp8[t].data;
    if (c && !is_fp8(params_fp8[t].dtype))
      return fail(E5MA_INVALID_VALUE, "e5b_adam_multi: param_fp8 %d must be E4M3 or E5M2 (dtype %d)", t, (int)params_fp8[t].dtype);
    if (c && params_fp8[t].scaling != E5MA_SCALING_TENSOR)
      return fail(E5MA_INVALID_VALUE, "e5b_adam_multi: param_fp8 takes per-tensor scaling only");
    if (!any) { pt = params[t].dtype; gt = grads[t].dtype; mt = exp_avgs[t].dtype; copy = c; qt = c ? (int)params_fp8[t].dtype : qt; any = true; }
    else if (pt != (int)params[t].dtype || gt != (int)grads[t].dtype || mt != (int)exp_avgs[t].dtype || copy != c ||
             (c && qt != (int)params_fp8[t].dtype))
      return fail(E5MA_INVALID_VALUE, "e5b_adam_multi: tensor %d differs in dtype (or in having an FP8 copy) from tensor 0; "
                  "group tensors of one kind per call", t);
  }
  if (!any) return E5MA_OK;
  DeviceProps dp;
  if (e5ma_status st = require_blackwell("e5b_adam_multi", &dp)) return st;

  AdamScalars a;
  a.lr = cfg->lr; a.beta1 = cfg->beta1; a.beta2 = cfg->beta2; a.eps = cfg->eps; a.wd = cfg->weight_decay;
  a.omb1 = (float)(1.0 - (double)cfg->beta1);
  a.omb2 = (float)(1.0 - (double)cfg->beta2);
  a.rbc1 = cfg->bias_correction ? (float)(1.0 / (1.0 - pow((double)cfg->beta1, cfg->step))) : 1.f;
  a.rbc2 = cfg->bias_correction ? (float)(1.0 / (1.0 - pow((double)cfg->beta2, cfg->step))) : 1.f;
  a.lr_wd = (float)((double)cfg->lr * cfg->weight_decay);
  a.gscale = cfg->grad_scale == 0.f ? 1.f : cfg->grad_scale;
  a.adamw = cfg->adamw;

  const auto a16 = [](const void *p) { return ((uintptr_t)p & 15u) == 0; };
  int t = 0;
  while (t < num_tensors) {   // one launch per MT_MAX non-empty tensors
    AdamTable tb;
    tb.n = 0;
    unsigned blocks = 0;
    for (; t < num_tensors && tb.n < MT_MAX; ++t) {
      if (counts[t] == 0) continue;
      const size_t nb = (counts[t] + MT_CHUNK - 1) / MT_CHUNK;
      if (nb > 0x7FFFFFFFu - blocks) break;   // keeps the grid inside 2^31 - 1 blocks; the rest goes to the next launch
      const int e = tb.n++;
      tb.p[e] = params[t].data; tb.g[e] = grads[t].data; tb.m[e] = exp_avgs[t].data; tb.v[e] = exp_avg_sqs[t].data;
      tb.q[e] = copy ? (uint8_t *)params_fp8[t].data : nullptr;
      tb.qs[e] = copy ? params_fp8[t].scale : nullptr;
      tb.amax[e] = copy ? params_fp8[t].amax : nullptr;
      tb.count[e] = counts[t];
      tb.first_block[e] = blocks;
      tb.vec[e] = a16(tb.p[e]) && a16(tb.g[e]) && a16(tb.m[e]) && a16(tb.v[e]) && ((uintptr_t)tb.q[e] & 7u) == 0;
      blocks += (unsigned)nb;
    }
    if (tb.n == 0) {
      if (t < num_tensors && counts[t] != 0)
        return fail(E5MA_INVALID_VALUE, "e5b_adam_multi: tensor %d is too large for one launch; use e5ma_adam", t);
      continue;
    }
    tb.first_block[tb.n] = blocks;
    const cudaError_t err = pt == E5MA_BF16 ? adam_multi_g<E5MA_BF16>(gt, mt, qt, copy, a, tb, blocks, stream)
                                            : adam_multi_g<E5MA_FP32>(gt, mt, qt, copy, a, tb, blocks, stream);
    if (err != cudaSuccess) return cuda_fail(err, "e5b_adam_multi: kernel launch");
  }
  return E5MA_OK;
}
