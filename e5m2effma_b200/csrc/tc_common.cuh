// Pieces shared by the tensor-core GEMM kernels of gemm_tc.cu (one CTA per tile, and gemm_tc2.cuh: CTA
// pairs; one translation unit, which owns the fault word): PTX wrappers for mbarriers, TMA and tcgen05, shared-memory and instruction descriptors,
// the register-level epilogue, and the host-side tensor-map encoder.
#pragma once
#include <cuda.h>
#include <stdlib.h>
#include "common.cuh"
#include "../../include/e5m2effma_b200.h"

namespace e5b {
namespace tc {

constexpr int BM = 128;             // tile columns j = MMA M = TMEM lanes
constexpr int STAGE_K_BYTES = 128;  // bytes of K per stage = one swizzle row
constexpr int MMA_K_BYTES = 32;     // bytes of K per tcgen05.mma
constexpr int EPI_WARPS = 8;
constexpr int THREADS = 64 + 32 * EPI_WARPS;             // producer, MMA, epilogue (and FP8 -> BF16 widening)
constexpr unsigned long long WAIT_LIMIT = 4000000000ull;  // clock cycles (about two seconds)

__device__ unsigned int g_fault;    // 0 = none; else (role << 24) | detail of the first bounded wait that ran out

// ---- PTX wrappers ------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("{ .reg .b64 st; mbarrier.arrive.shared::cta.b64 st, [%0]; }" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("{ .reg .b64 st; mbarrier.arrive.expect_tx.shared::cta.b64 st, [%0], %1; }" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile("{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
               : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok != 0;
}
// Bounded wait: false when the limit ran out or another role already aborted.  peer_abort: cluster address of the
// abort flag of the other CTA of a pair (0: none) -- raised together with the local one, so that the peer leaves at
// its next poll instead of waiting out its own limit.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag, unsigned int who,
                                          uint32_t peer_abort = 0) {
  if (mbar_try(bar, parity)) return true;
  const unsigned long long t0 = clock64();
  for (;;) {
    for (int i = 0; i < 64; ++i)
      if (mbar_try(bar, parity)) return true;
    if (*abort_flag) return false;
    if ((unsigned long long)(clock64() - t0) > WAIT_LIMIT) {
      *abort_flag = 1;
      if (peer_abort) asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(peer_abort), "r"(1u) : "memory");
      atomicCAS(&g_fault, 0u, who);
      return false;
    }
  }
}

// The same wait with cluster-scope acquire: for barriers on which another CTA of the cluster arrives (release at
// cluster scope) after writing into this CTA's shared memory.
__device__ __forceinline__ bool mbar_try_cluster(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile("{ .reg .pred p; mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
               : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool mbar_wait_cluster(uint32_t bar, uint32_t parity, volatile int *abort_flag, unsigned int who) {
  if (mbar_try_cluster(bar, parity)) return true;
  const unsigned long long t0 = clock64();
  for (;;) {
    for (int i = 0; i < 64; ++i)
      if (mbar_try_cluster(bar, parity)) return true;
    if (*abort_flag) return false;
    if ((unsigned long long)(clock64() - t0) > WAIT_LIMIT) {
      *abort_flag = 1;
      atomicCAS(&g_fault, 0u, who);
      return false;
    }
  }
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *map, int c0, int c1, uint32_t bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
               ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(bar) : "memory");
}

// fetch a tensor map (a kernel parameter) into the descriptor cache before the first copy needs it
__device__ __forceinline__ void prefetch_map(const CUtensorMap *map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}

__device__ __forceinline__ void tmem_alloc(uint32_t slot_smem, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot_smem), "r"(cols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// D[tmem] (+)= A[smem desc] * B[smem desc]; KIND 0: kind::f8f6f4, 1: kind::f16
template <int KIND>
__device__ __forceinline__ void mma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  if (KIND == 0)
    asm volatile("{ .reg .pred p; setp.ne.b32 p, %4, 0; tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p; }"
                 ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
  else
    asm volatile("{ .reg .pred p; setp.ne.b32 p, %4, 0; tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p; }"
                 ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
// the mbarrier gets one arrival once every MMA issued so far by this thread has completed
__device__ __forceinline__ void mma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// 32 lanes x 32 consecutive columns of 32-bit accumulators: thread = lane, v[c] = column c
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float v[32]) {
  uint32_t r[32];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr) : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}

// Tile order.  Tiles are numbered so that GROUP_I consecutive tile rows (along i) are swept across all
// tile columns before the next group starts: the CTAs that run at the same time then share a band of
// op(A) that stays in L2 while op(B) streams past it, instead of re-reading all of op(A) from HBM for
// every few tile columns (which a plain i-fastest order does once op(A) outgrows the 126 MB L2).
constexpr int GROUP_I = 8;
__device__ __forceinline__ void tile_coords(int t, int tiles_i, int tiles_j, int &ti, int &tj) {
  const int per_group = GROUP_I * tiles_j;
  const int g = t / per_group, r = t - g * per_group;
  const int gi0 = g * GROUP_I;
  const int gsize = tiles_i - gi0 < GROUP_I ? tiles_i - gi0 : GROUP_I;
  ti = gi0 + r % gsize;
  tj = r / gsize;
}

// Shared-memory matrix descriptor of a K-major tile stored as rows of 128 bytes with the 128-byte
// swizzle (what a TMA box of 128 bytes x R rows produces): 8-row groups are 1024 bytes apart (SBO),
// the leading offset is not used by swizzled K-major layouts (encoded as 1), descriptor version 1,
// layout type 2 = 128-byte swizzle.  Addresses and offsets are in units of 16 bytes.
__device__ __forceinline__ uint64_t kmajor_sw128_desc(uint32_t smem_addr) {
  return (uint64_t)((smem_addr >> 4) & 0x3FFFu) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) |
         ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}

// The same for an MN-major tile (the operand is contiguous along its row index, e.g. op(A) stored m x k):
// TMA boxes of 128 bytes of MN x R k-rows land as R rows of 128 bytes with the 128-byte swizzle; a tile wider
// than 128 bytes of MN is several such boxes, lbo_bytes apart (leading offset); groups of 8 k-rows are
// 1024 bytes apart (stride offset).
__device__ __forceinline__ uint64_t mnmajor_sw128_desc(uint32_t smem_addr, uint32_t lbo_bytes) {
  return (uint64_t)((smem_addr >> 4) & 0x3FFFu) | ((uint64_t)((lbo_bytes >> 4) & 0x3FFFu) << 16) |
         ((uint64_t)(1024 >> 4) << 32) | ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}

// Instruction descriptor: FP32 accumulator (bits 4-5 = 1), operand formats at bits 7-9 / 10-12,
// bits 15 / 16 = 1 when operand A / B is MN-major (0: K-major), N / 8 at bits 17-22, M / 16 at bits 24-28.
__host__ __device__ constexpr uint32_t instr_desc(int fmt_a, int fmt_b, int mdim, int ndim, int a_mn = 0, int b_mn = 0) {
  return (1u << 4) | ((uint32_t)fmt_a << 7) | ((uint32_t)fmt_b << 10) | ((uint32_t)a_mn << 15) | ((uint32_t)b_mn << 16) |
         ((uint32_t)(ndim >> 3) << 17) | ((uint32_t)(mdim >> 4) << 24);
}

// ---- epilogue --------------------------------------------------------------------------------
template <int DT>
__device__ __forceinline__ void store_out(void *d, size_t idx, float v, float qs) {
  if (DT == E5MA_FP32) ((float *)d)[idx] = v;
  else if (DT == E5MA_BF16) ((uint16_t *)d)[idx] = (uint16_t)enc_bf16(v);
  else if (DT == E5MA_FP16) ((uint16_t *)d)[idx] = (uint16_t)enc_f16(v);
  else if (DT == E5MA_E5M2) ((uint8_t *)d)[idx] = (uint8_t)enc_fp8<E5MA_E5M2>(__fmul_rn(v, qs));
  else ((uint8_t *)d)[idx] = (uint8_t)enc_fp8<E5MA_E4M3>(__fmul_rn(v, qs));
}

// 32 consecutive elements of dtype T (FP32 or BF16) starting at a 16-byte aligned address
template <int T>
__device__ __forceinline__ void load32(const void *p, float v[32]) {
  if (T == E5MA_FP32) {
    const float4 *q = reinterpret_cast<const float4 *>(p);
#pragma unroll
    for (int e = 0; e < 8; ++e) { const float4 a = q[e]; v[4 * e] = a.x; v[4 * e + 1] = a.y; v[4 * e + 2] = a.z; v[4 * e + 3] = a.w; }
  } else {
    const uint4 *q = reinterpret_cast<const uint4 *>(p);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const uint4 a = q[e];
      const uint32_t w[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
      for (int h = 0; h < 4; ++h) { v[8 * e + 2 * h] = __uint_as_float(w[h] << 16); v[8 * e + 2 * h + 1] = __uint_as_float(w[h] & 0xFFFF0000u); }
    }
  }
}
// 32 consecutive outputs of dtype DT to a 16-byte aligned address
template <int DT>
__device__ __forceinline__ void store32(void *p, const float v[32], float qs) {
  if (DT == E5MA_FP32) {
    float4 *q = reinterpret_cast<float4 *>(p);
#pragma unroll
    for (int e = 0; e < 8; ++e) q[e] = make_float4(v[4 * e], v[4 * e + 1], v[4 * e + 2], v[4 * e + 3]);
  } else if (DT == E5MA_BF16 || DT == E5MA_FP16) {
    uint4 *q = reinterpret_cast<uint4 *>(p);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      uint32_t w[4];
#pragma unroll
      for (int h = 0; h < 4; ++h)
        w[h] = DT == E5MA_BF16 ? enc_bf16x2(v[8 * e + 2 * h], v[8 * e + 2 * h + 1]) : enc_f16x2(v[8 * e + 2 * h], v[8 * e + 2 * h + 1]);
      q[e] = make_uint4(w[0], w[1], w[2], w[3]);
    }
  } else {
    uint4 *q = reinterpret_cast<uint4 *>(p);
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      uint32_t w[4];
#pragma unroll
      for (int h = 0; h < 4; ++h) {
        const float *x = v + 16 * e + 4 * h;
        w[h] = enc_fp8x2<DT>(__fmul_rn(x[0], qs), __fmul_rn(x[1], qs)) | (enc_fp8x2<DT>(__fmul_rn(x[2], qs), __fmul_rn(x[3], qs)) << 16);
      }
      q[e] = make_uint4(w[0], w[1], w[2], w[3]);
    }
  }
}

// What the epilogue of one launch needs beyond OutDesc: whether D (and C) admit 16-byte vector
// access (base and leading dimension multiples of 16 bytes) and whether bias / C have a dtype the
// vector path reads directly.
// wgroups: into how many groups the epilogue warps split to widen alternate k-blocks of a mixed problem (1, 2).
// ksplit: the one-CTA kernel runs as 2-CTA clusters, each CTA adding up one half of K of the same tile.
// split: the last partial wave of tiles is cut into half tiles.  transposed: the kernel was given the
// operands in swapped roles (TMEM lanes are rows i, TMEM columns are columns j) and its m / n are swapped.
struct EpiMode { int vec; int split; int transposed; int mn_n; int mn_m; int wgroups; int ksplit; };   // mn_n / mn_m: the N-side / M-side operand is stored MN-contiguous

// One thread's 32 accumulators: column j, rows ib .. ib+31.  Fast path when the 32 rows are all
// inside the matrix and vector access is allowed; otherwise element by element.
template <int DT>
__device__ __forceinline__ float drain32(const OutDesc &o, const OutScalars &r, const EpiMode &md, float acc[32],
                                         int ib, int j, int m, float as_const, float sbj) {
  float mx = 0.f;
  if (md.vec && ib + 32 <= m) {
    if (o.sa_vec) {
      float sa[32];
      load32<E5MA_FP32>(o.sa + ib, sa);
#pragma unroll
      for (int e = 0; e < 32; ++e) acc[e] = __fmul_rn(acc[e], __fmul_rn(__fmul_rn(o.alpha, sa[e]), sbj));
    } else {
      const float s = (o.sa_vec || o.sb_vec) ? __fmul_rn(as_const, sbj) : r.s;
#pragma unroll
      for (int e = 0; e < 32; ++e) acc[e] = __fmul_rn(acc[e], s);
    }
    if (o.bias) {
      float b[32];
      if (o.bias_dtype == E5MA_FP32) load32<E5MA_FP32>((const float *)o.bias + ib, b);
      else load32<E5MA_BF16>((const uint16_t *)o.bias + ib, b);
#pragma unroll
      for (int e = 0; e < 32; ++e) acc[e] = __fadd_rn(acc[e], b[e]);
    }
    if (o.c) {
      float c[32];
      const size_t off = (size_t)j * o.ldc + ib;
      if (o.c_dtype == E5MA_FP32) load32<E5MA_FP32>((const float *)o.c + off, c);
      else load32<E5MA_BF16>((const uint16_t *)o.c + off, c);
#pragma unroll
      for (int e = 0; e < 32; ++e) acc[e] = __fmaf_rn(o.beta, c[e], acc[e]);
    }
#pragma unroll
    for (int e = 0; e < 32; ++e) mx = fmaxf(mx, fabsf(acc[e]));
    store32<DT>((uint8_t *)o.d + ((size_t)j * o.ldd + ib) * elem_bytes(DT), acc, r.qs);
  } else {
#pragma unroll
    for (int e = 0; e < 32; ++e) {   // fully unrolled: acc[] stays in registers
      const int i = ib + e;
      if (i < m) {
        const float a = o.sa_vec ? o.sa[i] : 0.f;
        const float s = (o.sa_vec || o.sb_vec) ? __fmul_rn(o.sa_vec ? __fmul_rn(o.alpha, a) : as_const, sbj) : r.s;
        float v = __fmul_rn(acc[e], s);
        if (o.bias) v = __fadd_rn(v, load_elem(o.bias_dtype, o.bias, (size_t)i, 1.f));
        if (o.c) v = __fmaf_rn(o.beta, load_elem(o.c_dtype, o.c, (size_t)j * o.ldc + i, r.csinv), v);
        mx = fmaxf(mx, fabsf(v));
        store_out<DT>(o.d, (size_t)j * o.ldd + i, v, r.qs);
      }
    }
  }
  return mx;
}

// e5b_gemm_bcast, column-per-lane epilogues: after a warp has drained its part of a tile into the local D -- rows
// [r0, r1) of the 32 columns starting at c0 -- it copies that block to every peer's D.  A lane's own stores are
// 32 to 128 bytes per column, 32 columns apart in memory; sent over NVLink like that they would travel as
// small, scattered writes (measured: the GEMM ran at half speed).  Copied back out of L2 instead, consecutive
// lanes take consecutive 16-byte pieces of one column, so every remote store instruction writes runs of up to
// 512 contiguous bytes.  Only this warp's own stores are read, so a warp-level barrier orders them.
template <int DT>
__device__ __forceinline__ void bcast_block(const OutDesc &o, int c0, int n, int r0, int r1) {
  if (o.npeers == 0 || r1 <= r0) return;
  __syncwarp();
  constexpr int ES = elem_bytes(DT);
  const int lane = threadIdx.x & 31;
  const int cols = n - c0 < 32 ? n - c0 : 32;
  if (cols <= 0) return;
  const size_t col_bytes = (size_t)o.ldd * ES;
  const uint8_t *src = (const uint8_t *)o.d + ((size_t)c0 * o.ldd + r0) * ES;
  const int run = (r1 - r0) * ES;                       // bytes per column
  const bool aligned = ((((uintptr_t)src) | col_bytes) & 15u) == 0;
  const int chunks = aligned ? run >> 4 : 0;            // whole 16-byte pieces per column
  for (int idx = lane; idx < cols * chunks; idx += 32) {
    const int c = idx / chunks, q = idx - c * chunks;
    const size_t off = (size_t)c * col_bytes + ((size_t)q << 4);
    const uint4 v = __ldcg(reinterpret_cast<const uint4 *>(src + off));
    const size_t doff = (size_t)(src - (const uint8_t *)o.d) + off;
    for (int p = 0; p < o.npeers; ++p) *reinterpret_cast<uint4 *>((uint8_t *)o.peer[p] + doff) = v;
  }
  const int rest0 = chunks << 4;                        // bytes of each column not covered above
  for (int idx = lane; idx < cols * (run - rest0); idx += 32) {
    const int c = idx / (run - rest0), b = rest0 + idx - c * (run - rest0);
    const size_t off = (size_t)c * col_bytes + b;
    const uint8_t v = __ldcg(src + off);
    const size_t doff = (size_t)(src - (const uint8_t *)o.d) + off;
    for (int p = 0; p < o.npeers; ++p) ((uint8_t *)o.peer[p])[doff] = v;
  }
}

// The same for a kernel that ran with swapped operand roles: the thread's TMEM lane is row i, its 32
// accumulators are columns jb .. jb+31.  Stores of one column by the 32 lanes of a warp are contiguous
// (32 consecutive i), so plain element stores coalesce; per-row terms were read once by the caller.
template <int DT>
__device__ __forceinline__ float drain32_t(const OutDesc &o, const OutScalars &r, float acc[32], int i, int jb, int n,
                                           float as_i, float sb_const, float bias_i) {
  float mx = 0.f;
  // scale, then bias
  if (o.sb_vec) {
#pragma unroll
    for (int e = 0; e < 32; ++e) acc[e] = __fmul_rn(acc[e], __fmul_rn(as_i, jb + e < n ? o.sb[jb + e] : 0.f));
  } else {
    const float s = o.sa_vec ? __fmul_rn(as_i, sb_const) : r.s;
#pragma unroll
    for (int e = 0; e < 32; ++e) acc[e] = __fmul_rn(acc[e], s);
  }
  if (o.bias) {
#pragma unroll
    for (int e = 0; e < 32; ++e) acc[e] = __fadd_rn(acc[e], bias_i);
  }
  // beta * C: all 32 loads are issued before the first is used
  if (o.c) {
    float c[32];
    if (o.c_dtype == E5MA_FP32) {
      const float *cp = (const float *)o.c + (size_t)jb * o.ldc + i;
#pragma unroll
      for (int e = 0; e < 32; ++e) c[e] = jb + e < n ? cp[(size_t)e * o.ldc] : 0.f;
    } else if (o.c_dtype == E5MA_BF16) {
      const uint16_t *cp = (const uint16_t *)o.c + (size_t)jb * o.ldc + i;
#pragma unroll
      for (int e = 0; e < 32; ++e) c[e] = jb + e < n ? dec_bf16(cp[(size_t)e * o.ldc]) : 0.f;
    } else {
#pragma unroll
      for (int e = 0; e < 32; ++e) c[e] = jb + e < n ? load_elem(o.c_dtype, o.c, (size_t)(jb + e) * o.ldc + i, r.csinv) : 0.f;
    }
#pragma unroll
    for (int e = 0; e < 32; ++e) acc[e] = __fmaf_rn(o.beta, c[e], acc[e]);
  }
#pragma unroll
  for (int e = 0; e < 32; ++e) {
    if (jb + e < n) {
      mx = fmaxf(mx, fabsf(acc[e]));
      store_out<DT>(o.d, (size_t)(jb + e) * o.ldd + i, acc[e], r.qs);
      for (int p = 0; p < o.npeers; ++p) store_out<DT>(o.peer[p], (size_t)(jb + e) * o.ldd + i, acc[e], r.qs);
    }
  }
  return mx;
}

// Widening of the FP8 operand of a mixed pair, one k-block: 512 raw 16-byte chunks -> 1024 BF16 chunks in the
// 128-byte-swizzled layout.  ct: index of the thread among the 256 epilogue threads.  K-contiguous operand
// (MN = false): raw row r = 64 codes along k of row r, four chunks c.  Operand contiguous along its rows' index
// (MN = true): raw row r = k-row of 128 codes, eight chunks; chunks 0..3 belong to the first 64-row box of the
// MN-major BF16 layout, 4..7 to the second.  Either way raw chunk c becomes the BF16 chunks 2c, 2c+1 of a
// 128-byte row, swizzled with the row index.
// NT: number of threads that share the block (ct = 0 .. NT - 1).
template <int FT, bool MN, int NT = 32 * EPI_WARPS>
__device__ __forceinline__ void widen_block(const uint8_t *raw, uint8_t *dst, int ct) {
#pragma unroll
  for (int idx = ct; idx < 512; idx += NT) {
    const uint4 q = *reinterpret_cast<const uint4 *>(raw + idx * 16);
    uint32_t w[8];
    fp8x4_to_bf16x2<FT>(q.x, w[0], w[1]);
    fp8x4_to_bf16x2<FT>(q.y, w[2], w[3]);
    fp8x4_to_bf16x2<FT>(q.z, w[4], w[5]);
    fp8x4_to_bf16x2<FT>(q.w, w[6], w[7]);
    const int r = MN ? idx >> 3 : idx >> 2, c = idx & 3;
    uint8_t *row = dst + r * 128 + (MN ? ((idx >> 2) & 1) * (64 * 128) : 0);
    *reinterpret_cast<uint4 *>(row + (((2 * c) ^ (r & 7)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
    *reinterpret_cast<uint4 *>(row + (((2 * c + 1) ^ (r & 7)) << 4)) = make_uint4(w[4], w[5], w[6], w[7]);
  }
}

// One 16-byte piece of a K-contiguous FP8 operand (16 codes of row r, chunk c = 0..3 of the 64-code k-block) ->
// its two BF16 chunks 2c, 2c + 1 of the row's 128 bytes in the 128-byte-swizzled layout (what widen_block does
// with pieces it reads from shared memory).
template <int FT>
__device__ __forceinline__ void widen_piece(const uint4 &q, uint8_t *dst, int r, int c) {
  uint32_t w[8];
  fp8x4_to_bf16x2<FT>(q.x, w[0], w[1]);
  fp8x4_to_bf16x2<FT>(q.y, w[2], w[3]);
  fp8x4_to_bf16x2<FT>(q.z, w[4], w[5]);
  fp8x4_to_bf16x2<FT>(q.w, w[6], w[7]);
  uint8_t *row = dst + r * 128;
  *reinterpret_cast<uint4 *>(row + (((2 * c) ^ (r & 7)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
  *reinterpret_cast<uint4 *>(row + (((2 * c + 1) ^ (r & 7)) << 4)) = make_uint4(w[4], w[5], w[6], w[7]);
}
__device__ __forceinline__ uint4 ld_stream16_tc(const void *p) {
  uint4 r;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(p));
  return r;
}

// ---- host side ---------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = [] {
    void *p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      p = nullptr;
    return (EncodeTiledFn)p;
  }();
  return fn;
}

// K-major operand: rows x k elements, row pitch ld elements.  Operands the MMA reads directly get
// boxes of 128 bytes of K x box_rows rows with the 128-byte swizzle; an FP8 operand that is widened
// in shared memory first (raw) gets plain 64-byte rows.
// MN-contiguous operand (rows x k elements stored k x rows... i.e. element (r, kk) at r + kk * ld): boxes of
// 128 bytes of rows x one stage of k (128 FP8 / 64 BF16 k-rows), 128-byte swizzle.
inline bool make_map_mn(CUtensorMap *map, const void *base, int elem_bytes, int k, int rows, int ld, bool raw = false) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  const cuuint64_t dims[2] = {(cuuint64_t)rows, (cuuint64_t)k};
  const cuuint64_t strides[1] = {(cuuint64_t)ld * elem_bytes};
  // raw (an FP8 operand that will be widened to BF16): 64 k-rows of 128 codes, not swizzled
  const cuuint32_t box[2] = {(cuuint32_t)(128 / elem_bytes), (cuuint32_t)(raw ? STAGE_K_BYTES / 2 : STAGE_K_BYTES / elem_bytes)};
  const cuuint32_t estr[2] = {1, 1};
  const CUtensorMapDataType dt = elem_bytes == 1 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  return fn(map, dt, 2, const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
            raw ? CU_TENSOR_MAP_SWIZZLE_NONE : CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// raw: boxes of 64 FP8 codes per row, not swizzled (an operand that will be widened to BF16)
inline bool make_map(CUtensorMap *map, const void *base, int elem_bytes, int k, int rows, int ld, int box_rows, bool raw) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  const cuuint64_t dims[2] = {(cuuint64_t)k, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)ld * elem_bytes};
  const cuuint32_t box[2] = {(cuuint32_t)(raw ? STAGE_K_BYTES / 2 : STAGE_K_BYTES / elem_bytes), (cuuint32_t)box_rows};
  const cuuint32_t estr[2] = {1, 1};
  const CUtensorMapDataType dt = elem_bytes == 1 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  return fn(map, dt, 2, const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
            raw ? CU_TENSOR_MAP_SWIZZLE_NONE : CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace tc
}  // namespace e5b
