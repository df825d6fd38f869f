// Shared device and host pieces of the sm_100a E5M2EffMA library: FP8 / BF16 / FP16 element
// codecs built on the Blackwell conversion instructions, typed element access, the output
// (epilogue) description shared by the GEMM and GEMV kernels, the amax reduction and the
// host-side error state.
//
// Numerics contract (reference src/e5m2effma.cuh:83-124, include/e5m2effma.h:27-31): FP32
// arithmetic without flush-to-zero, explicit single-rounding operations, FP8 encodes are
// round-to-nearest-even saturating with every NaN -> 0x7F, BF16 encodes map every NaN to 0x7FC0.
// The hardware converters differ from that only for NaN inputs, which are patched here.
#pragma once
#include <stdint.h>
#include <atomic>
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include "../../include/e5m2effma.h"

namespace e5b {

__host__ __device__ constexpr bool is_fp8(int t) { return t == E5MA_E5M2 || t == E5MA_E4M3; }
__host__ __device__ constexpr int elem_bytes(int t) { return is_fp8(t) ? 1 : (t == E5MA_FP32 ? 4 : 2); }

// ---- decode --------------------------------------------------------------------------------
// Two FP8 codes (low 16 bits of w) -> two FP16 values, exact for both formats (E4M3 spans
// 2^-9 .. 448, E5M2 is the upper byte of an FP16); Inf / NaN codes become FP16 Inf / NaN.
__device__ __forceinline__ uint32_t e4m3x2_to_f16x2(uint32_t w) {
  uint32_t r;
  asm("{ .reg .b16 t; cvt.u16.u32 t, %1; cvt.rn.f16x2.e4m3x2 %0, t; }" : "=r"(r) : "r"(w));
  return r;
}
__device__ __forceinline__ uint32_t e5m2x2_to_f16x2(uint32_t w) { return __byte_perm(w, 0, 0x1404); }

__device__ __forceinline__ float f16bits_to_f32(uint32_t h) {
  return __half2float(__ushort_as_half((unsigned short)h));
}
__device__ __forceinline__ float dec_e4m3(uint32_t b) { return f16bits_to_f32(e4m3x2_to_f16x2(b & 0xFFu) & 0xFFFFu); }
__device__ __forceinline__ float dec_e5m2(uint32_t b) { return f16bits_to_f32((b & 0xFFu) << 8); }
__device__ __forceinline__ float dec_bf16(uint32_t h) { return __uint_as_float(h << 16); }

// Four FP8 codes of format T packed in w -> four FP32 values
template <int T>
__device__ __forceinline__ void dec_fp8x4(uint32_t w, float v[4]) {
  const uint32_t lo = T == E5MA_E4M3 ? e4m3x2_to_f16x2(w) : e5m2x2_to_f16x2(w);
  const uint32_t hi = T == E5MA_E4M3 ? e4m3x2_to_f16x2(w >> 16) : e5m2x2_to_f16x2(w >> 16);
  const float2 a = __half22float2(*reinterpret_cast<const __half2 *>(&lo));
  const float2 b = __half22float2(*reinterpret_cast<const __half2 *>(&hi));
  v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
}

// ---- FP8 -> FP32 / BF16 widening of packed codes -----------------------------------------------
// Four FP8 codes (bytes 0..3 of w, ascending k) -> four FP32 values, exact, subnormal codes included.
// E5M2 is the upper byte of an FP16, so masking puts codes 1, 3 (and, shifted, 0, 2) in place as FP16
// pairs; E4M3 pairs go through the hardware FP8 -> FP16 converter.  Then FP16 -> FP32 conversions.
// Most of the work runs on the floating-point pipes; the integer pipe only sees two operations.
template <int T>
__device__ __forceinline__ void fp8x4_to_f32(uint32_t w, float f[4]) {
  uint32_t h02, h13;   // FP16 pairs (code 0 | code 2) and (code 1 | code 3), or (0 | 1) and (2 | 3) for E4M3
  if (T == E5MA_E5M2) {
    h13 = w & 0xFF00FF00u;
    h02 = __byte_perm(w, 0, 0x2404);   // (b2 << 24) | (b0 << 8)
    const float2 a = __half22float2(*reinterpret_cast<const __half2 *>(&h02));
    const float2 b = __half22float2(*reinterpret_cast<const __half2 *>(&h13));
    f[0] = a.x; f[2] = a.y; f[1] = b.x; f[3] = b.y;
  } else {
    h02 = e4m3x2_to_f16x2(w);          // codes 0, 1
    h13 = e4m3x2_to_f16x2(w >> 16);    // codes 2, 3
    const float2 a = __half22float2(*reinterpret_cast<const __half2 *>(&h02));
    const float2 b = __half22float2(*reinterpret_cast<const __half2 *>(&h13));
    f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y;
  }
}
// ... -> BF16 pairs (k0,k1) and (k2,k3): an FP8 value has at most 4 significant bits, so the upper
// half of its FP32 encoding is its exact BF16 encoding; one byte permute packs two of them.
template <int T>
__device__ __forceinline__ void fp8x4_to_bf16x2(uint32_t w, uint32_t &lo, uint32_t &hi) {
  float f[4];
  fp8x4_to_f32<T>(w, f);
  lo = __byte_perm(__float_as_uint(f[0]), __float_as_uint(f[1]), 0x7632);
  hi = __byte_perm(__float_as_uint(f[2]), __float_as_uint(f[3]), 0x7632);
}

// ---- encode --------------------------------------------------------------------------------
__device__ __forceinline__ bool is_nan(float x) { return (__float_as_uint(x) & 0x7FFFFFFFu) > 0x7F800000u; }

// (lo, hi) -> two FP8 codes in the low 16 bits (lo in bits 0..7).  cvt.rn.satfinite rounds to
// nearest even and clamps finite overflow and Inf to the largest finite code; NaN is forced to 0x7F.
template <int T>
__device__ __forceinline__ uint32_t enc_fp8x2(float lo, float hi) {
  uint32_t r;
  if (T == E5MA_E4M3)
    asm("{ .reg .b16 t; cvt.rn.satfinite.e4m3x2.f32 t, %1, %2; cvt.u32.u16 %0, t; }" : "=r"(r) : "f"(hi), "f"(lo));
  else
    asm("{ .reg .b16 t; cvt.rn.satfinite.e5m2x2.f32 t, %1, %2; cvt.u32.u16 %0, t; }" : "=r"(r) : "f"(hi), "f"(lo));
  if (is_nan(lo)) r = (r & 0xFF00u) | 0x7Fu;
  if (is_nan(hi)) r = (r & 0x00FFu) | 0x7F00u;
  return r;
}
template <int T> __device__ __forceinline__ uint32_t enc_fp8(float v) { return enc_fp8x2<T>(v, 0.f) & 0xFFu; }

// (lo, hi) -> packed BF16 pair, nearest even; NaN -> 0x7FC0 (the converter alone gives 0x7FFF).
__device__ __forceinline__ uint32_t enc_bf16x2(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  if (is_nan(lo)) r = (r & 0xFFFF0000u) | 0x7FC0u;
  if (is_nan(hi)) r = (r & 0x0000FFFFu) | 0x7FC00000u;
  return r;
}
__device__ __forceinline__ uint32_t enc_bf16(float v) { return enc_bf16x2(v, 0.f) & 0xFFFFu; }
// The bare converters, for values the caller knows to be free of NaN (the only inputs the patches above change).
// The vectorised kernels test a whole group with one sum -- a NaN survives every addition -- and then skip the
// per-value patches; what is stored is the same.
__device__ __forceinline__ uint32_t cvt_bf16x2_raw(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}
template <int T>
__device__ __forceinline__ uint32_t cvt_fp8x2_raw(float lo, float hi) {
  uint32_t r;
  if (T == E5MA_E4M3)
    asm("{ .reg .b16 t; cvt.rn.satfinite.e4m3x2.f32 t, %1, %2; cvt.u32.u16 %0, t; }" : "=r"(r) : "f"(hi), "f"(lo));
  else
    asm("{ .reg .b16 t; cvt.rn.satfinite.e5m2x2.f32 t, %1, %2; cvt.u32.u16 %0, t; }" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}
__device__ __forceinline__ uint32_t enc_f16(float v) { return __half_as_ushort(__float2half_rn(v)); }
__device__ __forceinline__ uint32_t enc_f16x2(float lo, float hi) { return enc_f16(lo) | (enc_f16(hi) << 16); }

// ---- 32-byte global accesses (sm_100: 256-bit vector loads / stores), streaming cache hints ------
__device__ __forceinline__ void ld32B_stream(const void *p, uint32_t r[8]) {
  asm volatile("ld.global.nc.L1::no_allocate.v8.u32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]) : "l"(p));
}
__device__ __forceinline__ void st32B_stream(void *p, const uint32_t r[8]) {
  asm volatile("st.global.cs.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};"
               ::"l"(p), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]) : "memory");
}

// ---- typed scalar access ---------------------------------------------------------------------
__device__ __forceinline__ float ld_or_one(const float *p) { return p ? *p : 1.0f; }

// element i of an array of dtype t; FP8 values are multiplied by sinv (one rounding)
__device__ __forceinline__ float load_elem(int t, const void *p, size_t i, float sinv) {
  switch (t) {
    case E5MA_E5M2: return __fmul_rn(dec_e5m2(((const uint8_t *)p)[i]), sinv);
    case E5MA_E4M3: return __fmul_rn(dec_e4m3(((const uint8_t *)p)[i]), sinv);
    case E5MA_BF16: return dec_bf16(((const uint16_t *)p)[i]);
    case E5MA_FP16: return f16bits_to_f32(((const uint16_t *)p)[i]);
    default: return ((const float *)p)[i];
  }
}
// FP8 destinations store encode(v * qs)
__device__ __forceinline__ void store_elem(int t, void *p, size_t i, float v, float qs) {
  switch (t) {
    case E5MA_E5M2: ((uint8_t *)p)[i] = (uint8_t)enc_fp8<E5MA_E5M2>(__fmul_rn(v, qs)); break;
    case E5MA_E4M3: ((uint8_t *)p)[i] = (uint8_t)enc_fp8<E5MA_E4M3>(__fmul_rn(v, qs)); break;
    case E5MA_BF16: ((uint16_t *)p)[i] = (uint16_t)enc_bf16(v); break;
    case E5MA_FP16: ((uint16_t *)p)[i] = (uint16_t)enc_f16(v); break;
    default: ((float *)p)[i] = v;
  }
}

// ---- amax ----------------------------------------------------------------------------------
// max |v| over a warp, then one integer atomicMax per warp: non-negative floats (Inf included)
// order like their bit patterns; NaN never gets here because fmaxf drops it.
__device__ __forceinline__ float warp_max(float m) {
#pragma unroll
  for (int o = 16; o; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xFFFFFFFFu, m, o));
  return m;
}
__device__ __forceinline__ void amax_publish(float *amax, float m) {
  if (m > 0.f) atomicMax(reinterpret_cast<int *>(amax), __float_as_int(m));
}
// Whole block (blockDim.x a multiple of 32, at most 1024): one atomic per block.
__device__ __forceinline__ void block_amax(float *amax, float m) {
  __shared__ float part[32];
  m = warp_max(m);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  if (lane == 0) part[warp] = m;
  __syncthreads();
  if (warp == 0) {
    m = lane < nw ? part[lane] : 0.f;
    m = warp_max(m);
    if (lane == 0) amax_publish(amax, m);
  }
}

// ---- output description of GEMM / GEMV (reference include/e5m2effma.h:27-31) -------------------
constexpr int MAX_PEERS = 7;   // other GPUs of an 8-GPU node
struct OutDesc {
  const float *sa, *sb;   // scale_inv of FP8 A / B (NULL: 1)
  int sa_vec, sb_vec;     // 1: one factor per row i / per column j
  float alpha, beta;
  const void *c; int ldc, c_dtype; const float *c_sinv;   // c == NULL: no C term
  void *d; int ldd, d_dtype; const float *d_scale;
  float *amax;
  const void *bias; int bias_dtype;
  // e5b_gemm_bcast: every output element is also stored at the same element offset of these buffers (other GPUs'
  // copies of D, mapped into this device's address space); plain stores, no reads
  int npeers; void *peer[MAX_PEERS];
};

struct OutScalars { float s, qs, csinv; };   // per-tensor factors read once per thread

__device__ __forceinline__ OutScalars out_begin(const OutDesc &o) {
  OutScalars r;
  r.s = (o.sa_vec || o.sb_vec) ? 0.f : __fmul_rn(__fmul_rn(o.alpha, ld_or_one(o.sa)), ld_or_one(o.sb));
  r.qs = ld_or_one(o.d_scale);
  r.csinv = ld_or_one(o.c_sinv);
  return r;
}
// (alpha * sa[i]) * sb[j]
__device__ __forceinline__ float out_scale(const OutDesc &o, const OutScalars &r, int i, int j) {
  if (!o.sa_vec && !o.sb_vec) return r.s;
  const float a = o.sa_vec ? o.sa[i] : ld_or_one(o.sa), b = o.sb_vec ? o.sb[j] : ld_or_one(o.sb);
  return __fmul_rn(__fmul_rn(o.alpha, a), b);
}
// v = acc*s + bias[i]; v = fma(beta, C[i,j], v): the value before conversion
__device__ __forceinline__ float out_value(const OutDesc &o, const OutScalars &r, int i, int j, float acc) {
  float v = __fmul_rn(acc, out_scale(o, r, i, j));
  if (o.bias) v = __fadd_rn(v, load_elem(o.bias_dtype, o.bias, (size_t)i, 1.f));
  if (o.c) v = __fmaf_rn(o.beta, load_elem(o.c_dtype, o.c, (size_t)j * o.ldc + i, r.csinv), v);
  return v;
}
// one output through the whole epilogue; returns |v| for the amax statistic
__device__ __forceinline__ float out_store(const OutDesc &o, const OutScalars &r, int i, int j, float acc) {
  const float v = out_value(o, r, i, j, acc);
  store_elem(o.d_dtype, o.d, (size_t)j * o.ldd + i, v, r.qs);
  for (int p = 0; p < o.npeers; ++p) store_elem(o.d_dtype, o.peer[p], (size_t)j * o.ldd + i, v, r.qs);
  return fabsf(v);
}

// ---- host side -------------------------------------------------------------------------------
void clear_error();
e5ma_status fail(e5ma_status s, const char *fmt, ...) __attribute__((format(printf, 2, 3)));
e5ma_status cuda_fail(cudaError_t e, const char *what);   // E5MA_OK when e == cudaSuccess

struct DeviceProps { int cc; int sms; };

// Experiment / test switches of the kernel selection.  Each one starts from its E5MA_* environment variable,
// which is read once (the first time any switch is asked for); e5b_set_option() changes it afterwards.
// A negative value means "not set": the library's own choice applies.
enum Opt {
  OPT_FORCE_SIMT,     // E5MA_FORCE_SIMT    1: every GEMM runs the ascending-k CUDA-core kernel
  OPT_TC_PAIR,        // E5MA_TC_PAIR       0: no CTA-pair kernel
  OPT_TC_SPLIT,       // E5MA_TC_SPLIT      0: the last round of tiles is not cut into slices
  OPT_TC_GRID,        // E5MA_TC_GRID       n: at most n CTAs in the one-CTA tensor-core kernel
  OPT_TC_WIDE,        // E5MA_TC_WIDE       0: no wide (256 x up to 512) pair tiles; n >= 256: that tile width
  OPT_GEMV_KERNEL,    // E5MA_GEMV_KERNEL   0: register loads, 1: cp.async ring per warp, 2: persistent bulk-copy ring, 3: cp.async row streams per block
  OPT_GEMV_STAGES,    // E5MA_GEMV_STAGES   depth of the cp.async ring (2, 3, 4)
  OPT_GEMV_U,         // E5MA_GEMV_U        k-steps in flight per warp of the register-load kernel
  OPT_GEMV_MT,        // E5MA_GEMV_MT       2: 32 rows per block in the register-load kernel
  OPT_MIXED_PAIR,     // E5MA_MIXED_PAIR    0: FP8 x BF16 problems never take the CTA-pair kernel
  OPT_GEMV_KMAP,      // E5MA_GEMV_KMAP     1: each warp of the cp.async GEMV walks a contiguous eighth of K
  OPT_WIDEN_GROUPS,   // E5MA_WIDEN_GROUPS  1, 2: groups of warps that widen alternate k-blocks of a mixed FP8 x BF16 GEMM
  OPT_GEMV_FMA_MAXN,  // E5MA_GEMV_FMA_MAXN 0..4: largest batch of FP8 / BF16 activations that takes the FP32-pipe GEMV kernel
  OPT_GEMV_F16,       // E5MA_GEMV_F16      0: the cp.async GEMV never uses FP16 arithmetic (BF16 everywhere, as gemv_async_kernel)
  OPT_TC_KSPLIT,      // E5MA_TC_KSPLIT     0: the one-CTA GEMM never splits K over CTA pairs; 1: whenever at most half of the SMs have a tile
  OPT_COUNT
};
int opt(Opt which);

// Measured plan for a GEMM problem: the table named by E5MA_TUNE_FILE (read once), then the compiled-in table of
// tuned_sm100.h.  TUNED_NONE when neither has the problem.  GEMV settings likewise (key: 0 kernel, 1 stages, 2 kmap).
constexpr int TUNED_NONE = -1000000;
int tuned_gemm_plan(int elem_bytes, int m, int n, int k);
int tuned_gemv(int key);

// Which kernel the last e5ma_gemm call of this host thread launched (e5b_last_route()).
enum Route { ROUTE_NONE = 0, ROUTE_GEMV = 1, ROUTE_GEMV_PERSISTENT = 2, ROUTE_TC_PAIR = 3, ROUTE_TC_PAIR_WIDE = 4,
             ROUTE_TC_256 = 5, ROUTE_TC_128 = 6, ROUTE_SIMT = 7, ROUTE_TC_MIXED_PAIR = 8, ROUTE_GEMV_FMA = 9, ROUTE_GEMV_ROWS = 10,
             ROUTE_TC_256_KSPLIT = 11, ROUTE_TC_128_KSPLIT = 12, ROUTE_TC_256_KTAIL = 13, ROUTE_TC_128_KTAIL = 14 };
void note_route(int r);
// E5MA_OK and the properties of the current device when it is compute capability 10.x
e5ma_status require_blackwell(const char *who, DeviceProps *out);

// Opt-in to more than 48 KiB of dynamic shared memory, once per kernel and device.  One object per kernel
// (a function-local static of the launcher); safe when several host threads launch at once.
struct SmemOptIn {
  std::atomic<unsigned char> done[64];
  template <typename K>
  cudaError_t ensure(K kernel, int bytes) {
    int dev = 0;
    cudaGetDevice(&dev);
    std::atomic<unsigned char> &d = done[dev & 63];
    if (d.load(std::memory_order_acquire)) return cudaSuccess;
    const cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    if (e == cudaSuccess) d.store(1, std::memory_order_release);
    return e;
  }
};

// kernel launchers implemented in the other translation units
cudaError_t launch_gemv_mma(int a_dtype, int x_dtype, const uint8_t *A, int lda, const uint8_t *X, int ldx,
                            int m, int n, int k, const OutDesc &o, int sms, cudaStream_t s);
cudaError_t launch_gemm_simt(int a_dtype, int b_dtype, bool a_kc, bool b_kc, const uint8_t *A, int lda,
                             const uint8_t *B, int ldb, int m, int n, int k, const OutDesc &o, cudaStream_t s);
unsigned int peer_fault_read_and_clear();   // fault word of e5b_peer_barrier's bounded wait (after a device sync)
unsigned int gemv_fault_read_and_clear();   // fault word of the persistent GEMV's bounded waits (after a device sync)
// returns cudaErrorNotSupported when the problem is outside what the tensor-core kernel takes
cudaError_t launch_gemm_tc(int a_dtype, int b_dtype, bool a_kc, bool b_kc, const uint8_t *A, int lda,
                           const uint8_t *B, int ldb, int m, int n, int k, const OutDesc &o, int sms,
                           cudaStream_t s);

}  // namespace e5b
