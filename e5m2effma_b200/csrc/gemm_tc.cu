// Tensor-core GEMM for sm_100a: tcgen05.mma with TMA-fed shared-memory stages and FP32
// accumulators in tensor memory.  Replaces the FP32-FMA tile kernel of the reference
// (src/gemm_e5m2effma.cuh:117-233); the epilogue keeps its documented order
// (include/e5m2effma.h:27-31).
//
// Shape of the kernel
//   * One persistent CTA per SM walks over output tiles of BI rows (index i, BI = 256 or 128) by
//     128 columns (index j).  The MMA computes the transposed tile: its M side -- the 128 lanes of
//     tensor memory -- is j (rows of op(B)^T), its N side -- TMEM columns -- is i.  A thread that
//     reads its TMEM lane therefore holds consecutive i of one column j, which are contiguous in
//     the column-major D: the epilogue converts in registers and stores 16 bytes at a time.
//   * Warp 0 (one elected lane) is the TMA producer: per k-block it brings a 128-row x 128-byte box
//     of op(B)^T and a BI-row x 128-byte box of op(A) into a ring of shared-memory stages, both in
//     the 128-byte-swizzled K-major layout the MMA reads.  Rows beyond m / n and bytes beyond k are
//     zero-filled by TMA, so tails need no special code (k is a multiple of 16 elements, a zero
//     byte is +0 in every operand format).
//   * Warp 1 (one elected lane) issues the MMAs: four K = 32-byte steps per stage, accumulating into
//     one of two TMEM buffers; tcgen05.commit hands the stage back to the producer and, after the
//     last k-block, the accumulator to the epilogue.
//   * Warps 2..9 are the epilogue: a warp owns the TMEM lane quadrant (warp index mod 4) and one
//     half of the tile's i range, reads 32 accumulators of its lane at a time with tcgen05.ld and
//     applies scale, bias, beta * C, amax and the conversion.  While they drain one buffer the MMA
//     warp already fills the other.
//   * FP8 x FP8 (any E5M2 / E4M3 pairing) runs kind::f8f6f4, BF16 x BF16 runs kind::f16; one stage
//     is 128 bytes of K either way (128 FP8 or 64 BF16 elements), so the two differ only in the
//     instruction descriptor and the element type of the tensor maps.
//   * FP8 x BF16 pairs (either order) also run kind::f16: products must stay exact, so the FP8
//     operand is widened to BF16, which is exact (at most 4 significant bits).  TMA brings its raw
//     bytes (64 per row and k-block) into the stage; four converter warps (10..13) rewrite them as
//     BF16 in the swizzled K-major layout, fence towards the async proxy and signal the MMA warp.
//   * No cluster features are used: every CTA loads its own operand boxes.
//
// Every wait on an mbarrier is bounded.  A wait that runs out records a fault word, raises a
// block-wide abort flag that every role polls, and the CTA leaves through the common exit, where
// tensor memory is released.  e5b_gemm_fault() reads the word back.
#include <cuda.h>
#include <stdlib.h>
#include "common.cuh"

namespace e5b {
namespace tc {

constexpr int BM = 128;             // tile columns j = MMA M = TMEM lanes
constexpr int STAGE_K_BYTES = 128;  // bytes of K per stage = one swizzle row
constexpr int MMA_K_BYTES = 32;     // bytes of K per tcgen05.mma
constexpr int EPI_WARPS = 8;
constexpr int CONV_WARPS = 4;
constexpr int THREADS = 64 + 32 * EPI_WARPS;             // producer, MMA, epilogue
constexpr int THREADS_CONV = THREADS + 32 * CONV_WARPS;  // ... plus the FP8 -> BF16 converter warps
constexpr unsigned long long WAIT_LIMIT = 4000000000ull;  // clock cycles (about two seconds)

__device__ unsigned int g_fault;    // 0 = none; else (role << 24) | detail of the first bounded wait that ran out

// CONV: 0 both operands arrive ready for the MMA; 1 the i-side operand (op(A)) is FP8 and is
// widened to BF16 in shared memory; 2 the j-side operand (op(B)) is.
template <int BI, int CONV> struct Cfg {
  static constexpr int J_BYTES = BM * STAGE_K_BYTES;    // box of op(B)^T: 128 rows j
  static constexpr int I_BYTES = BI * STAGE_K_BYTES;    // box of op(A): BI rows i
  static constexpr int RAW_ROWS = CONV == 1 ? BI : (CONV == 2 ? BM : 0);
  static constexpr int RAW_BYTES = RAW_ROWS * (STAGE_K_BYTES / 2);   // 64 FP8 bytes per row and k-block
  static constexpr int STAGE_BYTES = J_BYTES + I_BYTES + RAW_BYTES;
  static constexpr int STAGES = CONV ? (BI == 256 ? 3 : 4) : (BI == 256 ? 4 : 6);
  static constexpr int NTHREADS = CONV ? THREADS_CONV : THREADS;
  static constexpr int TMEM_COLS = 2 * BI;
  // stages + barriers + slack for the 1 KiB alignment of the first stage
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 384;
};

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
// Bounded wait: false when the limit ran out or another role already aborted.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag, unsigned int who) {
  if (mbar_try(bar, parity)) return true;
  const unsigned long long t0 = clock64();
  for (;;) {
    for (int i = 0; i < 64; ++i)
      if (mbar_try(bar, parity)) return true;
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

// Shared-memory matrix descriptor of a K-major tile stored as rows of 128 bytes with the 128-byte
// swizzle (what a TMA box of 128 bytes x R rows produces): 8-row groups are 1024 bytes apart (SBO),
// the leading offset is not used by swizzled K-major layouts (encoded as 1), descriptor version 1,
// layout type 2 = 128-byte swizzle.  Addresses and offsets are in units of 16 bytes.
__device__ __forceinline__ uint64_t kmajor_sw128_desc(uint32_t smem_addr) {
  return (uint64_t)((smem_addr >> 4) & 0x3FFFu) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) |
         ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}

// Instruction descriptor: FP32 accumulator (bits 4-5 = 1), operand formats at bits 7-9 / 10-12,
// both operands K-major (bits 15, 16 = 0), N / 8 at bits 17-22, M / 16 at bits 24-28.
__host__ __device__ constexpr uint32_t instr_desc(int fmt_a, int fmt_b, int mdim, int ndim) {
  return (1u << 4) | ((uint32_t)fmt_a << 7) | ((uint32_t)fmt_b << 10) | ((uint32_t)(ndim >> 3) << 17) |
         ((uint32_t)(mdim >> 4) << 24);
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
struct EpiMode { int vec; int split; };   // split: the last partial wave of tiles is cut into half tiles

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

// ---- the kernel ------------------------------------------------------------------------------
// map_i: tensor map of op(A) (rows i, box BI rows); map_j: tensor map of op(B)^T (rows j, box 128 rows).
// With CONV the map of the FP8 operand has 64-byte unswizzled boxes and lands in the raw area.
// FT: dtype of the FP8 operand that is widened (CONV != 0).
template <int BI, int KIND, int DT, int CONV, int FT>
__global__ void __launch_bounds__(Cfg<BI, CONV>::NTHREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_i, const __grid_constant__ CUtensorMap map_j,
               const __grid_constant__ CUtensorMap map_ih, int m, int n, int k_bytes, uint32_t idesc, uint32_t idesc_half,
               OutDesc o, EpiMode md) {
  using C = Cfg<BI, CONV>;
  extern __shared__ uint8_t smem_raw[];
  // stage ring at the first 1 KiB boundary (the swizzle pattern repeats every 1024 bytes)
  const uint32_t ring = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t *after_ring = smem_raw + (ring - smem_u32(smem_raw)) + C::STAGES * C::STAGE_BYTES;
  uint64_t *bars = reinterpret_cast<uint64_t *>(after_ring);   // full[S], empty[S], acc_full[2], acc_empty[2], ready[S]
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 3 * C::STAGES + 4);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
  const uint32_t bar0 = smem_u32(bars);
  const auto full_bar = [&](int s) { return bar0 + 8u * s; };
  const auto empty_bar = [&](int s) { return bar0 + 8u * (C::STAGES + s); };
  const auto acc_full = [&](int b) { return bar0 + 8u * (2 * C::STAGES + b); };
  const auto acc_empty = [&](int b) { return bar0 + 8u * (2 * C::STAGES + 2 + b); };
  const auto ready_bar = [&](int s) { return bar0 + 8u * (2 * C::STAGES + 4 + s); };   // converted operand in place

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_i = (m + BI - 1) / BI, tiles_j = (n + BM - 1) / BM, tiles = tiles_i * tiles_j;
  const int kblocks = (k_bytes + STAGE_K_BYTES - 1) / STAGE_K_BYTES;

  // Work items.  Normally one item = one tile, dealt round-robin to the CTAs.  When the last round would
  // keep at most half of the CTAs busy, its tiles are cut into two half tiles (BI / 2 rows: map_ih boxes,
  // idesc_half) so that the round takes half as long.  Every role derives the same list from this.
  const int grid_n = gridDim.x;
  const int full_items = (tiles / grid_n) * grid_n, rem = tiles - full_items;
  const bool split = CONV == 0 && md.split && rem > 0 && 2 * rem <= grid_n;
  const int items = split ? full_items + 2 * rem : tiles;
  const auto item_at = [&](int item, int &i0, int &j0, int &rows) {
    int tile = item, hf = 0;
    rows = BI;
    if (split && item >= full_items) { const int h = item - full_items; tile = full_items + (h >> 1); hf = h & 1; rows = BI / 2; }
    i0 = (tile % tiles_i) * BI + hf * (BI / 2);
    j0 = (tile / tiles_i) * BM;
  };

  if (threadIdx.x == 0) {
    for (int s = 0; s < C::STAGES; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); mbar_init(ready_bar(s), CONV_WARPS); }
    for (int b = 0; b < 2; ++b) { mbar_init(acc_full(b), 1); mbar_init(acc_empty(b), EPI_WARPS); }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {   // one warp allocates (and later frees) the accumulator columns
    tmem_alloc(smem_u32(tmem_slot), C::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < items && ok; t += gridDim.x) {
        int i0, j0, rows;
        item_at(t, i0, j0, rows);
        const bool half_tile = rows != BI;
        for (int kb = 0; kb < kblocks; ++kb, ++it) {
          const int s = it % C::STAGES;
          const uint32_t ph = (it / C::STAGES) & 1u;
          if (!mbar_wait(empty_bar(s), ph ^ 1u, abort_flag, (1u << 24) | (uint32_t)kb)) { ok = false; break; }
          mbar_expect_tx(full_bar(s), C::J_BYTES + (half_tile ? C::I_BYTES / 2 : C::I_BYTES) + C::RAW_BYTES -
                                          (CONV == 1 ? C::I_BYTES : (CONV == 2 ? C::J_BYTES : 0)));
          const uint32_t sj = ring + s * C::STAGE_BYTES, si = sj + C::J_BYTES, sraw = si + C::I_BYTES;
          // coordinates are in elements of the tensor map: the innermost one counts bytes for FP8 and
          // 2-byte elements for BF16; a k-block is 128 FP8 or 64 BF16 (and then also 64 raw FP8) elements
          const int kc = kb * (KIND == 0 ? STAGE_K_BYTES : STAGE_K_BYTES / 2);
          tma_load_2d(CONV == 2 ? sraw : sj, &map_j, kc, j0, full_bar(s));
          tma_load_2d(CONV == 1 ? sraw : si, half_tile ? &map_ih : &map_i, kc, i0, full_bar(s));
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      uint32_t it = 0, lt = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < items && ok; t += gridDim.x, ++lt) {
        int i0, j0, rows;
        item_at(t, i0, j0, rows);
        const uint32_t idesc_t = rows != BI ? idesc_half : idesc;
        const uint32_t buf = lt & 1u, use = lt >> 1;
        if (!mbar_wait(acc_empty(buf), (use & 1u) ^ 1u, abort_flag, (2u << 24) | 0xFFFFu)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + buf * BI;
        for (int kb = 0; kb < kblocks; ++kb, ++it) {
          const int s = it % C::STAGES;
          const uint32_t ph = (it / C::STAGES) & 1u;
          if (!mbar_wait(full_bar(s), ph, abort_flag, (2u << 24) | (uint32_t)kb)) { ok = false; break; }
          if (CONV && !mbar_wait(ready_bar(s), ph, abort_flag, (4u << 24) | (uint32_t)kb)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sj = ring + s * C::STAGE_BYTES, si = sj + C::J_BYTES;
          const uint64_t dj = kmajor_sw128_desc(sj), di = kmajor_sw128_desc(si);
#pragma unroll
          for (int ks = 0; ks < STAGE_K_BYTES / MMA_K_BYTES; ++ks) {
            // stepping 32 bytes along K inside the swizzled row = +2 in the 16-byte address field
            mma_ss<KIND>(d_tmem, dj + 2u * ks, di + 2u * ks, idesc_t, (kb | ks) != 0);
          }
          mma_commit(empty_bar(s));
        }
        if (ok) mma_commit(acc_full(buf));
      }
    }
  } else if (CONV != 0 && warp >= 2 + EPI_WARPS) {
    // ---------------- converter warps: raw FP8 rows -> BF16 rows in the swizzled K-major layout ----------------
    // A raw row is 64 bytes = four 16-byte chunks; chunk c of row r (k = 16c .. 16c+15) becomes the two
    // 16-byte chunks 2c, 2c+1 of the 128-byte BF16 row, which the 128-byte swizzle stores at chunk
    // positions (2c) ^ (r & 7) and (2c+1) ^ (r & 7).
    const int ct = threadIdx.x - 32 * (2 + EPI_WARPS);
    uint32_t it = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < items && ok; t += gridDim.x) {
      for (int kb = 0; kb < kblocks; ++kb, ++it) {
        const int s = it % C::STAGES;
        const uint32_t ph = (it / C::STAGES) & 1u;
        ok = mbar_wait(full_bar(s), ph, abort_flag, (5u << 24) | (uint32_t)kb);
        ok = __all_sync(0xFFFFFFFFu, ok);
        if (!ok) break;
        uint8_t *stage = smem_raw + (ring - smem_u32(smem_raw)) + s * C::STAGE_BYTES;
        const uint8_t *raw = stage + C::J_BYTES + C::I_BYTES;
        uint8_t *dst = stage + (CONV == 1 ? C::J_BYTES : 0);
#pragma unroll 2
        for (int idx = ct; idx < C::RAW_ROWS * 4; idx += 32 * CONV_WARPS) {
          const int r = idx >> 2, c = idx & 3;
          const uint4 q = *reinterpret_cast<const uint4 *>(raw + idx * 16);
          uint32_t w[8];
          fp8x4_to_bf16x2<FT>(q.x, w[0], w[1]);
          fp8x4_to_bf16x2<FT>(q.y, w[2], w[3]);
          fp8x4_to_bf16x2<FT>(q.z, w[4], w[5]);
          fp8x4_to_bf16x2<FT>(q.w, w[6], w[7]);
          uint8_t *row = dst + r * 128;
          *reinterpret_cast<uint4 *>(row + (((2 * c) ^ (r & 7)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
          *reinterpret_cast<uint4 *>(row + (((2 * c + 1) ^ (r & 7)) << 4)) = make_uint4(w[4], w[5], w[6], w[7]);
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic-proxy writes -> tensor-core reads
        __syncwarp();
        if (lane == 0) mbar_arrive(ready_bar(s));
      }
    }
  } else {
    // ------------- epilogue warps: TMEM lane quadrant = warp % 4, half of the i range = (warp - 2) / 4 -------------
    const int quad = warp & 3, half = (warp - 2) >> 2;
    const OutScalars r = out_begin(o);
    const float as_const = __fmul_rn(o.alpha, o.sa_vec ? 1.f : ld_or_one(o.sa));
    const float sb_const = o.sb_vec ? 1.f : ld_or_one(o.sb);
    float mx = 0.f;
    uint32_t lt = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < items && ok; t += gridDim.x, ++lt) {
      int i0, j0, rows;
      item_at(t, i0, j0, rows);
      const uint32_t buf = lt & 1u, use = lt >> 1;
      ok = mbar_wait(acc_full(buf), use & 1u, abort_flag, (3u << 24) | (uint32_t)warp);
      ok = __all_sync(0xFFFFFFFFu, ok);
      if (!ok) break;
      tc_fence_after();
      const int j = j0 + quad * 32 + lane;
      const bool col_ok = j < n;
      const float sbj = col_ok && o.sb_vec ? o.sb[j] : sb_const;
      const uint32_t t_lane = tmem_base + ((uint32_t)(quad * 32) << 16) + buf * BI;
      for (int c0 = half * (BI / 2); c0 < (half + 1) * (BI / 2); c0 += 32) {
        if (c0 >= rows || i0 + c0 >= m) break;   // warp-uniform
        float acc[32];
        tmem_ld32(t_lane + c0, acc);
        if (col_ok) mx = fmaxf(mx, drain32<DT>(o, r, md, acc, i0 + c0, j, m, as_const, sbj));
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(acc_empty(buf));
    }
    if (o.amax) {
      mx = warp_max(mx);
      if (lane == 0) amax_publish(o.amax, mx);
    }
  }

  // common exit: everybody meets, then the allocating warp releases tensor memory
  tc_fence_before();
  __syncthreads();
  if (*abort_flag && threadIdx.x == 0) {
    // give copies that may still be in flight time to land before the shared memory is reused
    const unsigned long long t0 = clock64();
    while ((unsigned long long)(clock64() - t0) < 2000000ull) { }
  }
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, C::TMEM_COLS);
  }
}

// ---- host side ---------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
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
static bool make_map(CUtensorMap *map, const void *base, int elem_bytes, int k, int rows, int ld, int box_rows, bool raw) {
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

template <int BI, int KIND, int DT, int CONV, int FT>
static cudaError_t launch_cfg(const CUtensorMap &mi, const CUtensorMap &mj, const CUtensorMap &mih, int m, int n,
                              int k_bytes, uint32_t idesc, uint32_t idesc_half, const OutDesc &o, const EpiMode &md, int sms,
                              cudaStream_t s) {
  using C = Cfg<BI, CONV>;
  static bool attr_done[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!attr_done[dev & 63]) {
    const cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<BI, KIND, DT, CONV, FT>,
                                               cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES);
    if (e != cudaSuccess) return e;
    attr_done[dev & 63] = true;
  }
  const int tiles = ((m + BI - 1) / BI) * ((n + BM - 1) / BM);
  int grid = tiles < sms ? tiles : sms;
  if (const char *g = getenv("E5MA_TC_GRID")) {   // experiments: fewer CTAs than SMs
    const int v = atoi(g);
    if (v > 0 && v < grid) grid = v;
  }
  gemm_tc_kernel<BI, KIND, DT, CONV, FT><<<grid, C::NTHREADS, C::SMEM_BYTES, s>>>(mi, mj, mih, m, n, k_bytes, idesc, idesc_half, o, md);
  return cudaGetLastError();
}

template <int BI, int KIND, int CONV, int FT>
static cudaError_t launch_dt(const CUtensorMap &mi, const CUtensorMap &mj, const CUtensorMap &mih, int m, int n,
                             int k_bytes, uint32_t idesc, uint32_t idesc_half, const OutDesc &o, const EpiMode &md, int sms,
                             cudaStream_t s) {
  switch (o.d_dtype) {
    case E5MA_BF16: return launch_cfg<BI, KIND, E5MA_BF16, CONV, FT>(mi, mj, mih, m, n, k_bytes, idesc, idesc_half, o, md, sms, s);
    case E5MA_FP32: return launch_cfg<BI, KIND, E5MA_FP32, CONV, FT>(mi, mj, mih, m, n, k_bytes, idesc, idesc_half, o, md, sms, s);
    case E5MA_FP16: return launch_cfg<BI, KIND, E5MA_FP16, CONV, FT>(mi, mj, mih, m, n, k_bytes, idesc, idesc_half, o, md, sms, s);
    case E5MA_E5M2: return launch_cfg<BI, KIND, E5MA_E5M2, CONV, FT>(mi, mj, mih, m, n, k_bytes, idesc, idesc_half, o, md, sms, s);
    default: return launch_cfg<BI, KIND, E5MA_E4M3, CONV, FT>(mi, mj, mih, m, n, k_bytes, idesc, idesc_half, o, md, sms, s);
  }
}

template <int BI>
static cudaError_t launch_kind(int kind, int conv, int ft, const CUtensorMap &mi, const CUtensorMap &mj,
                               const CUtensorMap &mih, int m, int n, int k_bytes, uint32_t idesc, uint32_t idesc_half,
                               const OutDesc &o, const EpiMode &md, int sms, cudaStream_t s) {
  if (kind == 0) return launch_dt<BI, 0, 0, E5MA_E5M2>(mi, mj, mih, m, n, k_bytes, idesc, idesc_half, o, md, sms, s);
  if (conv == 0) return launch_dt<BI, 1, 0, E5MA_E5M2>(mi, mj, mih, m, n, k_bytes, idesc, idesc_half, o, md, sms, s);
  if (conv == 1)
    return ft == E5MA_E5M2 ? launch_dt<BI, 1, 1, E5MA_E5M2>(mi, mj, mih, m, n, k_bytes, idesc, idesc_half, o, md, sms, s)
                           : launch_dt<BI, 1, 1, E5MA_E4M3>(mi, mj, mih, m, n, k_bytes, idesc, idesc_half, o, md, sms, s);
  return ft == E5MA_E5M2 ? launch_dt<BI, 1, 2, E5MA_E5M2>(mi, mj, mih, m, n, k_bytes, idesc, idesc_half, o, md, sms, s)
                         : launch_dt<BI, 1, 2, E5MA_E4M3>(mi, mj, mih, m, n, k_bytes, idesc, idesc_half, o, md, sms, s);
}

}  // namespace tc

// Blackwell tile selection (takes the place of the reference's tuned per-architecture tables,
// src/e5m2effma_tuned.h): tiles of 256 rows x 128 columns when they fill the machine or m is large,
// else 128 x 128.  Operand pairs: FP8 x FP8 -> kind::f8f6f4; BF16 x BF16 -> kind::f16; FP8 x BF16 in
// either order -> kind::f16 with the FP8 side widened in shared memory.
cudaError_t launch_gemm_tc(int a_dtype, int b_dtype, bool a_kc, bool b_kc, const uint8_t *A, int lda,
                           const uint8_t *B, int ldb, int m, int n, int k, const OutDesc &o, int sms,
                           cudaStream_t s) {
  using namespace tc;
  if (!a_kc || !b_kc || k <= 0) return cudaErrorNotSupported;
  if (a_dtype == E5MA_FP32 || b_dtype == E5MA_FP32) return cudaErrorNotSupported;
  const bool f8 = is_fp8(a_dtype) && is_fp8(b_dtype);
  const int conv = f8 ? 0 : (is_fp8(a_dtype) ? 1 : (is_fp8(b_dtype) ? 2 : 0));
  const int kind = f8 ? 0 : 1;
  const int ft = conv == 1 ? a_dtype : (conv == 2 ? b_dtype : E5MA_E5M2);
  const int tiles256 = ((m + 255) / 256) * ((n + BM - 1) / BM);
  const bool wide = m > 128 && (tiles256 >= sms || m % 256 == 0 || m > 1024);
  const int bi = wide ? 256 : 128;
  CUtensorMap mi, mj, mih;   // mih: op(A) with half-height boxes, for the half tiles of the last round
  if (!make_map(&mi, A, elem_bytes(a_dtype), k, m, lda, bi, conv == 1) ||
      !make_map(&mj, B, elem_bytes(b_dtype), k, n, ldb, BM, conv == 2) ||
      !make_map(&mih, A, elem_bytes(a_dtype), k, m, lda, bi / 2, conv == 1))
    return cudaErrorNotSupported;
  // the MMA's A operand (M side) is op(B)^T, its B operand (N side) is op(A)
  const int fi = f8 ? (a_dtype == E5MA_E5M2 ? 1 : 0) : 1, fj = f8 ? (b_dtype == E5MA_E5M2 ? 1 : 0) : 1;
  const uint32_t idesc = instr_desc(fj, fi, BM, bi), idesc_half = instr_desc(fj, fi, BM, bi / 2);
  const int k_bytes = k * (f8 ? 1 : 2);   // bytes of K per operand row as the MMA sees it
  // 16-byte vector access in the epilogue: D (and C, bias) bases and column pitches must allow it
  const auto vec_ok = [](const void *p, int ld, int dtype) {
    return ((uintptr_t)p & 15u) == 0 && ((size_t)ld * elem_bytes(dtype)) % 16 == 0;
  };
  EpiMode md;
  md.split = wide ? 1 : 0;
  if (const char *e = getenv("E5MA_TC_SPLIT")) md.split = atoi(e) && wide;   // experiments
  md.vec = vec_ok(o.d, o.ldd, o.d_dtype);
  if (o.c && !((o.c_dtype == E5MA_FP32 || o.c_dtype == E5MA_BF16) && vec_ok(o.c, o.ldc, o.c_dtype))) md.vec = 0;
  if (o.bias && !((o.bias_dtype == E5MA_FP32 || o.bias_dtype == E5MA_BF16) && ((uintptr_t)o.bias & 15u) == 0)) md.vec = 0;
  if (o.sa_vec && ((uintptr_t)o.sa & 15u)) md.vec = 0;
  return wide ? launch_kind<256>(kind, conv, ft, mi, mj, mih, m, n, k_bytes, idesc, idesc_half, o, md, sms, s)
              : launch_kind<128>(kind, conv, ft, mi, mj, mih, m, n, k_bytes, idesc, idesc_half, o, md, sms, s);
}

}  // namespace e5b

// Reads and clears the fault word of the tensor-core GEMM on the current device (synchronises).
// 0: no bounded wait ever ran out.  Declared in include/e5m2effma_b200.h.
extern "C" unsigned int e5b_gemm_fault(void) {
  unsigned int v = 0, zero = 0;
  if (cudaMemcpyFromSymbol(&v, e5b::tc::g_fault, sizeof v) != cudaSuccess) return 0xFFFFFFFFu;
  cudaMemcpyToSymbol(e5b::tc::g_fault, &zero, sizeof zero);
  return v;
}
