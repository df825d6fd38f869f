// Host core of the library (error state, device gate, status strings) and e5ma_cast: a
// vectorised single-pass conversion kernel with the amax statistic fused in.
//
// e5ma_cast follows reference src/e5m2effma.cu:85-101 (validation order, what scale_inv / scale /
// amax apply to) and computes, per element, what its cast_kernel does (src/e5m2effma.cu:53-63):
// v = src * scale_inv, amax = max |v|, dst = convert(v * scale).  The kernel itself is new: it is
// specialised per (source, destination) dtype pair and moves 16 bytes per access.
#include <stdarg.h>
#include <stdio.h>
#include <atomic>
#include <mutex>
#include <stdlib.h>
#include <string.h>
#include "common.cuh"
#include "tuned_sm100.h"
#include <vector>

namespace e5b {

static thread_local char t_error[512];

void clear_error() { t_error[0] = 0; }

e5ma_status fail(e5ma_status s, const char *fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(t_error, sizeof t_error, fmt, ap);
  va_end(ap);
  return s;
}

e5ma_status cuda_fail(cudaError_t e, const char *what) {
  if (e == cudaSuccess) return E5MA_OK;
  return fail(E5MA_CUDA_ERROR, "%s: CUDA error %d (%s): %s", what, (int)e, cudaGetErrorName(e), cudaGetErrorString(e));
}

// ---- switches and the route record ----------------------------------------------------------------
static std::atomic<int> g_opt[OPT_COUNT];
static const char *const kOptNames[OPT_COUNT] = {"FORCE_SIMT", "TC_PAIR", "TC_SPLIT", "TC_GRID", "TC_WIDE", "GEMV_KERNEL",
                                                 "GEMV_STAGES", "GEMV_U", "GEMV_MT", "MIXED_PAIR", "GEMV_KMAP", "WIDEN_GROUPS",
                                                 "GEMV_FMA_MAXN", "GEMV_F16", "TC_KSPLIT"};
static void opt_init() {
  static std::once_flag once;
  std::call_once(once, [] {
    for (int i = 0; i < OPT_COUNT; ++i) {
      char name[48];
      snprintf(name, sizeof name, "E5MA_%s", kOptNames[i]);
      const char *e = getenv(name);
      g_opt[i].store(e && e[0] ? atoi(e) : -1, std::memory_order_relaxed);
    }
    // the older spelling of the GEMV switch: E5MA_GEMV_ASYNC=0 meant the register-load kernel
    if (g_opt[OPT_GEMV_KERNEL].load() < 0)
      if (const char *e = getenv("E5MA_GEMV_ASYNC")) g_opt[OPT_GEMV_KERNEL].store(atoi(e) ? 1 : 0);
  });
}
int opt(Opt which) {
  opt_init();
  return g_opt[which].load(std::memory_order_relaxed);
}

// ---- tuned tables ---------------------------------------------------------------------------------
struct TunedGemm { int eb, m, n, k, plan; };
static const TunedGemm kTunedGemm[] = {E5B_TUNED_GEMM {0, 0, 0, 0, 0}};
struct TunedFile { std::vector<TunedGemm> gemm; int gemv[4] = {TUNED_NONE, TUNED_NONE, TUNED_NONE, TUNED_NONE}; };

// Text table: one entry per line, `gemm <elem bytes> <m> <n> <k> <plan>` or `gemv kernel|stages|kmap|fma_maxn <value>`;
// anything else (comments, blank lines) is skipped.
static const TunedFile &tuned_file() {
  static TunedFile tf;
  static std::once_flag once;
  std::call_once(once, [] {
    const char *path = getenv("E5MA_TUNE_FILE");
    FILE *f = path && path[0] ? fopen(path, "r") : nullptr;
    if (!f) return;
    char line[256];
    while (fgets(line, sizeof line, f)) {
      TunedGemm g;
      char key[32];
      int v;
      if (sscanf(line, "gemm %d %d %d %d %d", &g.eb, &g.m, &g.n, &g.k, &g.plan) == 5) tf.gemm.push_back(g);
      else if (sscanf(line, "gemv %31s %d", key, &v) == 2) {
        if (!strcmp(key, "kernel")) tf.gemv[0] = v;
        else if (!strcmp(key, "stages")) tf.gemv[1] = v;
        else if (!strcmp(key, "kmap")) tf.gemv[2] = v;
        else if (!strcmp(key, "fma_maxn")) tf.gemv[3] = v;
      }
    }
    fclose(f);
  });
  return tf;
}
int tuned_gemm_plan(int elem_bytes, int m, int n, int k) {
  for (const TunedGemm &g : tuned_file().gemm)
    if (g.eb == elem_bytes && g.m == m && g.n == n && g.k == k) return g.plan;
  for (const TunedGemm &g : kTunedGemm)
    if (g.eb == elem_bytes && g.m == m && g.n == n && g.k == k && g.eb != 0) return g.plan;
  return TUNED_NONE;
}
int tuned_gemv(int key) {
  if (key < 0 || key > 3) return TUNED_NONE;
  if (tuned_file().gemv[key] != TUNED_NONE) return tuned_file().gemv[key];
  const int compiled[4] = {E5B_TUNED_GEMV_KERNEL, E5B_TUNED_GEMV_STAGES, E5B_TUNED_GEMV_KMAP, E5B_TUNED_GEMV_FMA_MAXN};
  return compiled[key];
}

static thread_local int t_route = ROUTE_NONE;
void note_route(int r) { t_route = r; }

// Per-device cache; entries are written once (two threads racing write the same values) and
// published through the atomic flag.
e5ma_status require_blackwell(const char *who, DeviceProps *out) {
  static DeviceProps cache[64];
  static std::atomic<int> ready[64];
  int dev = -1;
  const cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return cuda_fail(e, "cudaGetDevice");
  DeviceProps p;
  if (dev >= 0 && dev < 64 && ready[dev].load(std::memory_order_acquire)) {
    p = cache[dev];
  } else {
    int ma = 0, mi = 0, sms = 0;
    cudaError_t q = cudaDeviceGetAttribute(&ma, cudaDevAttrComputeCapabilityMajor, dev);
    if (q == cudaSuccess) q = cudaDeviceGetAttribute(&mi, cudaDevAttrComputeCapabilityMinor, dev);
    if (q == cudaSuccess) q = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (q != cudaSuccess) return cuda_fail(q, "cudaDeviceGetAttribute");
    p.cc = ma * 10 + mi;
    p.sms = sms;
    if (dev >= 0 && dev < 64) { cache[dev] = p; ready[dev].store(1, std::memory_order_release); }
  }
  if (p.cc != 100)
    return fail(E5MA_NOT_SUPPORTED, "%s: device %d is sm_%d; this build of the library contains sm_100a code only "
                "(NVIDIA B200)", who, dev, p.cc);
  if (out) *out = p;
  return E5MA_OK;
}

// ---- cast kernel -----------------------------------------------------------------------------
// 16 consecutive elements per step: 16-byte accesses for every dtype (FP32: four of them).
// WIDE: the array base is 32-byte aligned, so 2- and 4-byte dtypes use 32-byte accesses (half as many
// memory instructions; the narrow-to-wide casts are limited by the load/store queues, not by arithmetic).
template <int T, bool WIDE>
__device__ __forceinline__ void load16(const void *base, size_t i, float sinv, float v[16]) {
  if (WIDE && T == E5MA_FP32) {
    const uint8_t *p = reinterpret_cast<const uint8_t *>(base) + i * 4;
#pragma unroll
    for (int q = 0; q < 2; ++q) {
      uint32_t r[8];
      ld32B_stream(p + 32 * q, r);
#pragma unroll
      for (int e = 0; e < 8; ++e) v[8 * q + e] = __uint_as_float(r[e]);
    }
  } else if (WIDE && (T == E5MA_BF16 || T == E5MA_FP16)) {
    uint32_t w[8];
    ld32B_stream(reinterpret_cast<const uint8_t *>(base) + i * 2, w);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      if (T == E5MA_BF16) { v[2 * e] = __uint_as_float(w[e] << 16); v[2 * e + 1] = __uint_as_float(w[e] & 0xFFFF0000u); }
      else { const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&w[e])); v[2 * e] = f.x; v[2 * e + 1] = f.y; }
    }
  } else if (T == E5MA_FP32) {
    const float4 *p = reinterpret_cast<const float4 *>(base) + i / 4;
#pragma unroll
    for (int q = 0; q < 4; ++q) { const float4 a = __ldcs(p + q); v[4 * q] = a.x; v[4 * q + 1] = a.y; v[4 * q + 2] = a.z; v[4 * q + 3] = a.w; }
  } else if (T == E5MA_BF16 || T == E5MA_FP16) {
    const uint4 *p = reinterpret_cast<const uint4 *>(base) + i / 8;
#pragma unroll
    for (int q = 0; q < 2; ++q) {
      const uint4 a = __ldcs(p + q);
      const uint32_t w[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        if (T == E5MA_BF16) { v[8 * q + 2 * e] = __uint_as_float(w[e] << 16); v[8 * q + 2 * e + 1] = __uint_as_float(w[e] & 0xFFFF0000u); }
        else { const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&w[e])); v[8 * q + 2 * e] = f.x; v[8 * q + 2 * e + 1] = f.y; }
      }
    }
  } else {
    const uint4 a = __ldcs(reinterpret_cast<const uint4 *>(base) + i / 16);
    const uint32_t w[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      dec_fp8x4<T>(w[e], v + 4 * e);
#pragma unroll
      for (int q = 0; q < 4; ++q) v[4 * e + q] = __fmul_rn(v[4 * e + q], sinv);
    }
  }
}
// RAW: the 16 values (and, for an FP8 destination, their products with qs) are known to hold no NaN: bare converters.
template <int T, bool WIDE, bool RAW = false>
__device__ __forceinline__ void store16(void *base, size_t i, float qs, const float v[16]) {
  if (WIDE && T == E5MA_FP32) {
    uint8_t *p = reinterpret_cast<uint8_t *>(base) + i * 4;
#pragma unroll
    for (int q = 0; q < 2; ++q) {
      uint32_t r[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) r[e] = __float_as_uint(v[8 * q + e]);
      st32B_stream(p + 32 * q, r);
    }
  } else if (WIDE && (T == E5MA_BF16 || T == E5MA_FP16)) {
    uint32_t w[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) w[e] = T == E5MA_BF16 ? (RAW ? cvt_bf16x2_raw(v[2 * e], v[2 * e + 1]) : enc_bf16x2(v[2 * e], v[2 * e + 1])) : enc_f16x2(v[2 * e], v[2 * e + 1]);
    st32B_stream(reinterpret_cast<uint8_t *>(base) + i * 2, w);
  } else if (T == E5MA_FP32) {
    float4 *p = reinterpret_cast<float4 *>(base) + i / 4;
#pragma unroll
    for (int q = 0; q < 4; ++q) __stcs(p + q, make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]));
  } else if (T == E5MA_BF16 || T == E5MA_FP16) {
    uint4 *p = reinterpret_cast<uint4 *>(base) + i / 8;
#pragma unroll
    for (int q = 0; q < 2; ++q) {
      uint32_t w[4];
#pragma unroll
      for (int e = 0; e < 4; ++e)
        w[e] = T == E5MA_BF16 ? (RAW ? cvt_bf16x2_raw(v[8 * q + 2 * e], v[8 * q + 2 * e + 1]) : enc_bf16x2(v[8 * q + 2 * e], v[8 * q + 2 * e + 1])) : enc_f16x2(v[8 * q + 2 * e], v[8 * q + 2 * e + 1]);
      __stcs(p + q, make_uint4(w[0], w[1], w[2], w[3]));
    }
  } else {
    uint32_t w[4];
#pragma unroll
    for (int e = 0; e < 4; ++e)
      w[e] = RAW ? cvt_fp8x2_raw<T>(__fmul_rn(v[4 * e], qs), __fmul_rn(v[4 * e + 1], qs)) |
                       (cvt_fp8x2_raw<T>(__fmul_rn(v[4 * e + 2], qs), __fmul_rn(v[4 * e + 3], qs)) << 16)
                 : enc_fp8x2<T>(__fmul_rn(v[4 * e], qs), __fmul_rn(v[4 * e + 1], qs)) |
                       (enc_fp8x2<T>(__fmul_rn(v[4 * e + 2], qs), __fmul_rn(v[4 * e + 3], qs)) << 16);
    __stcs(reinterpret_cast<uint4 *>(base) + i / 16, make_uint4(w[0], w[1], w[2], w[3]));
  }
}

// MODE 0: element by element.  MODE 1: both pointers are 16-byte aligned: whole 16-element groups go
// through the vector path in a grid-stride loop, the remaining count % 16 elements one at a time.
// MODE 2: both pointers are 32-byte aligned: as MODE 1 with 32-byte accesses.
template <int TS, int TD, int MODE>
__global__ void __launch_bounds__(256) cast_kernel(const void *__restrict__ src, void *__restrict__ dst, size_t count,
                                                   const float *sinv_p, const float *scale_p, float *amax) {
  const float sinv = ld_or_one(sinv_p), qs = ld_or_one(scale_p);
  float mx = 0.f;
  const size_t tid = (size_t)blockIdx.x * blockDim.x + threadIdx.x, nthr = (size_t)gridDim.x * blockDim.x;
  constexpr bool VEC = MODE != 0, WIDE = MODE == 2;
  constexpr bool patched = TD == E5MA_BF16 || is_fp8(TD);     // destinations whose encoders patch NaN
  const bool qs_finite = fabsf(qs) <= 3.4028234664e38f;
  const size_t groups = VEC ? count / 16 : 0;
  // G groups per step so that every thread keeps 64 bytes of loads in flight whatever the source width
  constexpr int G = 4 / elem_bytes(TS);
  size_t gidx = tid;
  for (; gidx + (G - 1) * nthr < groups; gidx += G * nthr) {
    float v[G][16];
#pragma unroll
    for (int u = 0; u < G; ++u) load16<TS, WIDE>(src, (gidx + u * nthr) * 16, sinv, v[u]);
#pragma unroll
    for (int u = 0; u < G; ++u) {
      float chk = 0.f;
#pragma unroll
      for (int e = 0; e < 16; ++e) { mx = fmaxf(mx, fabsf(v[u][e])); chk += v[u][e]; }
      // one sum tells whether the group holds a NaN (or +Inf and -Inf, or, through an infinite or zero scale, would
      // produce one): if not, the converters need no NaN patches
      if (patched && !is_nan(chk) && !(is_fp8(TD) && (!qs_finite || is_nan(__fmul_rn(chk, qs)))))
        store16<TD, WIDE, true>(dst, (gidx + u * nthr) * 16, qs, v[u]);
      else
        store16<TD, WIDE>(dst, (gidx + u * nthr) * 16, qs, v[u]);
    }
  }
  for (; gidx < groups; gidx += nthr) {
    float v[16];
    load16<TS, WIDE>(src, gidx * 16, sinv, v);
#pragma unroll
    for (int e = 0; e < 16; ++e) mx = fmaxf(mx, fabsf(v[e]));
    store16<TD, WIDE>(dst, gidx * 16, qs, v);
  }
  for (size_t i = groups * 16 + tid; i < count; i += nthr) {
    const float v = load_elem(TS, src, i, sinv);
    mx = fmaxf(mx, fabsf(v));
    store_elem(TD, dst, i, v, qs);
  }
  if (amax) block_amax(amax, mx);
}

// Source and destination overlap (an in-place cast between dtypes of one size, or a same-dtype "copy + amax"
// onto itself): element by element through ordinary, coherent accesses -- the kernel above reads through the
// non-coherent path and promises the compiler that the two arrays do not alias.  Element i is read and then
// written by the same thread, so an exact in-place cast is well defined; partial overlaps are the caller's
// business, as in the reference (src/e5m2effma.cu:85-101 checks nothing).
__global__ void __launch_bounds__(256) cast_alias_kernel(int ts, int td, const void *src, void *dst, size_t count,
                                                         const float *sinv_p, const float *scale_p, float *amax) {
  const float sinv = ld_or_one(sinv_p), qs = ld_or_one(scale_p);
  float mx = 0.f;
  const size_t nthr = (size_t)gridDim.x * blockDim.x;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += nthr) {
    float v;
    switch (ts) {
      case E5MA_E5M2: v = __fmul_rn(dec_e5m2(((const volatile uint8_t *)src)[i]), sinv); break;
      case E5MA_E4M3: v = __fmul_rn(dec_e4m3(((const volatile uint8_t *)src)[i]), sinv); break;
      case E5MA_BF16: v = dec_bf16(((const volatile uint16_t *)src)[i]); break;
      case E5MA_FP16: v = f16bits_to_f32(((const volatile uint16_t *)src)[i]); break;
      default: v = ((const volatile float *)src)[i];
    }
    mx = fmaxf(mx, fabsf(v));
    store_elem(td, dst, i, v, qs);
  }
  if (amax) block_amax(amax, mx);
}

template <int TS, int TD>
static cudaError_t cast_launch(const void *src, void *dst, size_t count, const float *sinv, const float *scale,
                               float *amax, int sms, cudaStream_t s) {
  const bool vec = (((uintptr_t)src | (uintptr_t)dst) & 15u) == 0;
  const size_t work = vec ? count / 16 + (count % 16) : count;
  size_t blocks = (work + 255) / 256;
  const size_t cap = (size_t)sms * 16;   // two sweeps of full occupancy, then grid-stride
  if (blocks > cap) blocks = cap;
  if (blocks == 0) blocks = 1;
  const bool wide = (((uintptr_t)src | (uintptr_t)dst) & 31u) == 0;
  if (wide) cast_kernel<TS, TD, 2><<<(unsigned)blocks, 256, 0, s>>>(src, dst, count, sinv, scale, amax);
  else if (vec) cast_kernel<TS, TD, 1><<<(unsigned)blocks, 256, 0, s>>>(src, dst, count, sinv, scale, amax);
  else cast_kernel<TS, TD, 0><<<(unsigned)blocks, 256, 0, s>>>(src, dst, count, sinv, scale, amax);
  return cudaGetLastError();
}

template <int TS>
static cudaError_t cast_dst(int td, const void *src, void *dst, size_t count, const float *sinv, const float *scale,
                            float *amax, int sms, cudaStream_t s) {
  switch (td) {
    case E5MA_E4M3: return cast_launch<TS, E5MA_E4M3>(src, dst, count, sinv, scale, amax, sms, s);
    case E5MA_BF16: return cast_launch<TS, E5MA_BF16>(src, dst, count, sinv, scale, amax, sms, s);
    case E5MA_FP16: return cast_launch<TS, E5MA_FP16>(src, dst, count, sinv, scale, amax, sms, s);
    case E5MA_FP32: return cast_launch<TS, E5MA_FP32>(src, dst, count, sinv, scale, amax, sms, s);
    default: return cast_launch<TS, E5MA_E5M2>(src, dst, count, sinv, scale, amax, sms, s);
  }
}

}  // namespace e5b

extern "C" const char *e5ma_last_error(void) { return e5b::t_error; }

extern "C" int e5b_set_option(const char *name, int value) {
  using namespace e5b;
  if (!name) return -1;
  opt_init();
  if (!strncmp(name, "E5MA_", 5)) name += 5;
  for (int i = 0; i < OPT_COUNT; ++i)
    if (!strcmp(name, kOptNames[i])) {
      g_opt[i].store(value < 0 ? -1 : value, std::memory_order_relaxed);
      return 0;
    }
  return -1;
}

extern "C" int e5b_last_route(void) { return e5b::t_route; }

extern "C" int e5b_tuned_plan(int elem_bytes, int m, int n, int k) {
  const int p = e5b::tuned_gemm_plan(elem_bytes, m, n, k);
  return p == e5b::TUNED_NONE ? -2 : p;
}

extern "C" const char *e5ma_status_string(e5ma_status s) {
  switch (s) {
    case E5MA_OK: return "E5MA_OK";
    case E5MA_INVALID_VALUE: return "E5MA_INVALID_VALUE";
    case E5MA_NOT_SUPPORTED: return "E5MA_NOT_SUPPORTED";
    case E5MA_CUDA_ERROR: return "E5MA_CUDA_ERROR";
  }
  return "unknown e5ma_status";
}

extern "C" e5ma_status e5ma_cast(const e5ma_tensor *src, const e5ma_tensor *dst, size_t count, cudaStream_t stream) {
  using namespace e5b;
  clear_error();
  if (!src || !dst || !src->data || !dst->data) return fail(E5MA_INVALID_VALUE, "e5ma_cast: src / dst or their data is NULL");
  const auto known = [](int t) { return t >= E5MA_E4M3 && t <= E5MA_E5M2; };
  if (!known(src->dtype) || !known(dst->dtype))
    return fail(E5MA_INVALID_VALUE, "e5ma_cast: invalid dtype (src %d, dst %d)", (int)src->dtype, (int)dst->dtype);
  if (src->scaling != E5MA_SCALING_TENSOR || dst->scaling != E5MA_SCALING_TENSOR)
    return fail(E5MA_INVALID_VALUE, "e5ma_cast: per-tensor scaling only");
  if (count == 0) return E5MA_OK;
  DeviceProps dp;
  if (e5ma_status st = require_blackwell("e5ma_cast", &dp)) return st;
  const float *sinv = is_fp8(src->dtype) ? src->scale_inv : nullptr;
  const float *scale = is_fp8(dst->dtype) ? dst->scale : nullptr;
  cudaError_t err;
  const uintptr_t s0 = (uintptr_t)src->data, s1 = s0 + count * elem_bytes(src->dtype);
  const uintptr_t d0 = (uintptr_t)dst->data, d1 = d0 + count * elem_bytes(dst->dtype);
  if (s0 < d1 && d0 < s1) {   // overlapping buffers
    size_t blocks = (count + 255) / 256;
    if (blocks > (size_t)dp.sms * 16) blocks = (size_t)dp.sms * 16;
    cast_alias_kernel<<<(unsigned)blocks, 256, 0, stream>>>(src->dtype, dst->dtype, src->data, dst->data, count, sinv, scale,
                                                            dst->amax);
    return cuda_fail(cudaGetLastError(), "e5ma_cast: kernel launch");
  }
  switch (src->dtype) {
    case E5MA_E4M3: err = cast_dst<E5MA_E4M3>(dst->dtype, src->data, dst->data, count, sinv, scale, dst->amax, dp.sms, stream); break;
    case E5MA_BF16: err = cast_dst<E5MA_BF16>(dst->dtype, src->data, dst->data, count, sinv, scale, dst->amax, dp.sms, stream); break;
    case E5MA_FP16: err = cast_dst<E5MA_FP16>(dst->dtype, src->data, dst->data, count, sinv, scale, dst->amax, dp.sms, stream); break;
    case E5MA_FP32: err = cast_dst<E5MA_FP32>(dst->dtype, src->data, dst->data, count, sinv, scale, dst->amax, dp.sms, stream); break;
    default: err = cast_dst<E5MA_E5M2>(dst->dtype, src->data, dst->data, count, sinv, scale, dst->amax, dp.sms, stream); break;
  }
  return cuda_fail(err, "e5ma_cast: kernel launch");
}

// ---- device-side barrier between the GPUs of a node (declared in include/e5m2effma_b200.h) ----------------------
// Flag area of a rank: words 0 .. 7 = "rank j has arrived at barrier number e", word 8 = this rank's own count of
// barriers.  Thread j of the single block: fence, release-store the new count into peer j's word `rank`, then poll
// this rank's word j until it has reached the count (system-scope acquire loads).  The stores of kernels that ran
// earlier on the stream (the epilogue broadcast of e5b_gemm_bcast) happen before this kernel starts, the release is
// cumulative over them, so a peer that has seen the flag sees the data.  The poll is bounded.
namespace e5b {
constexpr int PB_MAX_RANKS = 8;
struct PeerFlags { uint32_t *f[PB_MAX_RANKS]; };
__device__ unsigned int g_peer_fault;

__global__ void peer_barrier_kernel(int rank, int nranks, PeerFlags p) {
  __shared__ uint32_t count_s;
  uint32_t *mine = p.f[rank];
  if (threadIdx.x == 0) {
    count_s = mine[PB_MAX_RANKS] + 1u;
    mine[PB_MAX_RANKS] = count_s;
  }
  __syncthreads();
  const uint32_t count = count_s;
  const int j = threadIdx.x;
  if (j >= nranks || j == rank) return;
  __threadfence_system();
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p.f[j] + rank), "r"(count) : "memory");
  const unsigned long long t0 = clock64();
  for (;;) {
    uint32_t seen;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(mine + j) : "memory");
    if ((int32_t)(seen - count) >= 0) return;
    if ((unsigned long long)(clock64() - t0) > 4000000000ull) {
      atomicCAS(&g_peer_fault, 0u, (uint32_t)(j + 1));
      return;
    }
  }
}

unsigned int peer_fault_read_and_clear() {
  unsigned int v = 0, zero = 0;
  if (cudaMemcpyFromSymbol(&v, g_peer_fault, sizeof v) != cudaSuccess) return 0xFFFFFFFFu;
  if (v) cudaMemcpyToSymbol(g_peer_fault, &zero, sizeof zero);
  return v;
}
}  // namespace e5b

extern "C" e5ma_status e5b_peer_barrier(int rank, int nranks, void *const *flags, cudaStream_t stream) {
  using namespace e5b;
  clear_error();
  if (nranks < 1 || nranks > PB_MAX_RANKS || rank < 0 || rank >= nranks)
    return fail(E5MA_INVALID_VALUE, "e5b_peer_barrier: rank %d of %d ranks (1 .. %d ranks)", rank, nranks, PB_MAX_RANKS);
  if (!flags) return fail(E5MA_INVALID_VALUE, "e5b_peer_barrier: flags is NULL");
  PeerFlags p = {};
  for (int r = 0; r < nranks; ++r) {
    if (!flags[r] || ((uintptr_t)flags[r] & 3u)) return fail(E5MA_INVALID_VALUE, "e5b_peer_barrier: flags[%d] is NULL or not 4-byte aligned", r);
    p.f[r] = (uint32_t *)flags[r];
  }
  DeviceProps dp;
  if (const e5ma_status st = require_blackwell("e5b_peer_barrier", &dp)) return st;
  peer_barrier_kernel<<<1, 32, 0, stream>>>(rank, nranks, p);
  return cuda_fail(cudaGetLastError(), "e5b_peer_barrier: kernel launch");
}
