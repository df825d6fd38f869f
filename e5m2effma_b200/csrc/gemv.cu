// Streaming GEMV / skinny GEMM:  D(m x n) = epilogue(W(m x k) * X(k x n)),  n <= 8, W in FP8 with
// K contiguous, X in FP8 or BF16 with K contiguous.  Takes the problems the reference routes to its
// gemv_kernel (src/gemm_e5m2effma.cu:100-102, src/gemv_e5m2effma.cuh:27-79) and replaces it.
//
// The kernel is bound by reading W once from HBM (m * k bytes; X, the scales and D are noise), so
// everything is arranged around that stream:
//   * every lane fetches W with 16-byte non-allocating loads; a block of 8 warps covers 1 KiB of
//     contiguous bytes of each of its rows per step, and the 8 warps split K between them;
//   * the FP8 bytes are widened to BF16 in registers (exact: at most 4 significant bits) and fed to
//     mma.sync.m16n8k16 with X as the 8-column operand, so all n <= 8 columns cost the same
//     instruction stream and the FP32 pipe stays free; products are exact, sums are FP32.  Where X is
//     (or converts exactly to) FP16 the same is done in FP16, whose widening costs a quarter of the
//     instructions (gemv_async16_kernel); FP32 activations run on the FP32 pipe (gemv_fma_kernel);
//   * the reduction over K may visit k in any order as long as W and X agree, so a lane's 16
//     contiguous bytes feed four consecutive MMAs without any shuffling;
//   * the 8 per-warp partial tiles meet in shared memory in a fixed order (deterministic), then one
//     thread per output runs the common epilogue and the block issues one amax atomic.
#include <stdlib.h>
#include "common.cuh"

namespace e5b {

__device__ __forceinline__ uint4 ld_stream16(const void *p) {
  uint4 r;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(p));
  return r;
}

__device__ __forceinline__ void mma_bf16_16816(float c[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
               "{%0, %1, %2, %3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

constexpr int GV_WARPS = 8;

// MT: 16-row tiles per block.  AT: dtype of W.  XT: dtype of X (E5M2, E4M3 or BF16).
// U: k-steps whose loads are all issued before the first of them is consumed (bytes in flight).
template <int MT, int AT, int XT, int U>
__global__ void __launch_bounds__(GV_WARPS * 32) gemv_mma_kernel(const uint8_t *__restrict__ W, int lda,
                                                                 const uint8_t *__restrict__ X, int ldx, int m, int n,
                                                                 int k, OutDesc o) {
  __shared__ float red[GV_WARPS][MT * 16][9];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;
  const int row0 = blockIdx.x * (MT * 16);
  constexpr int XB = XT == E5MA_BF16 ? 2 : 1;
  constexpr int XW = XT == E5MA_BF16 ? 2 : 1;   // 16-byte loads of X per 16 elements

  float acc[MT][4];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int e = 0; e < 4; ++e) acc[mt][e] = 0.f;

  const uint8_t *xcol = X + (size_t)g * ldx * XB;
  const bool xlive = g < n;
  const uint8_t *wrow[MT][2];
  bool wlive[MT][2];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt) {
    const int ra = row0 + mt * 16 + g, rb = ra + 8;
    wlive[mt][0] = ra < m; wlive[mt][1] = rb < m;
    wrow[mt][0] = W + (size_t)(wlive[mt][0] ? ra : 0) * lda;
    wrow[mt][1] = W + (size_t)(wlive[mt][1] ? rb : 0) * lda;
  }

  // A warp's step covers bytes [kc, kc + 128) of every row; this lane owns 16 bytes in each half.
  // The trip count must be the same for all lanes of the warp (mma.sync is warp-collective), so the
  // loop runs on the warp-uniform kc and the per-lane offset only enters the load predicates.
  for (int kc0 = warp * 128; kc0 < k; kc0 += U * GV_WARPS * 128) {
    uint4 wq[U][2][MT][2];      // [step][half][tile][row g / g+8]
    uint4 xq[U][2][XW];
#pragma unroll
    for (int u = 0; u < U; ++u)
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int kk = kc0 + u * GV_WARPS * 128 + t * 16 + h * 64;
        const bool kin = kk < k;
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
          for (int r = 0; r < 2; ++r)
            wq[u][h][mt][r] = kin && wlive[mt][r] ? ld_stream16(wrow[mt][r] + kk) : make_uint4(0, 0, 0, 0);
#pragma unroll
        for (int q = 0; q < XW; ++q)
          xq[u][h][q] = kin && xlive ? __ldg(reinterpret_cast<const uint4 *>(xcol + (size_t)kk * XB) + q) : make_uint4(0, 0, 0, 0);
      }
#pragma unroll
    for (int u = 0; u < U; ++u)
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        uint32_t xw[8];
        if (XT == E5MA_BF16) {
          xw[0] = xq[u][h][0].x; xw[1] = xq[u][h][0].y; xw[2] = xq[u][h][0].z; xw[3] = xq[u][h][0].w;
          xw[4] = xq[u][h][XW - 1].x; xw[5] = xq[u][h][XW - 1].y; xw[6] = xq[u][h][XW - 1].z; xw[7] = xq[u][h][XW - 1].w;
        } else {
          const uint32_t q[4] = {xq[u][h][0].x, xq[u][h][0].y, xq[u][h][0].z, xq[u][h][0].w};
#pragma unroll
          for (int e = 0; e < 4; ++e) fp8x4_to_bf16x2<XT == E5MA_BF16 ? E5MA_E5M2 : XT>(q[e], xw[2 * e], xw[2 * e + 1]);
        }
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
          const uint32_t qa[4] = {wq[u][h][mt][0].x, wq[u][h][mt][0].y, wq[u][h][mt][0].z, wq[u][h][mt][0].w};
          const uint32_t qb[4] = {wq[u][h][mt][1].x, wq[u][h][mt][1].y, wq[u][h][mt][1].z, wq[u][h][mt][1].w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            uint32_t a0, a2, a1, a3;
            fp8x4_to_bf16x2<AT>(qa[e], a0, a2);   // row g:   k pairs (0,1) and (2,3) of this word
            fp8x4_to_bf16x2<AT>(qb[e], a1, a3);   // row g+8
            mma_bf16_16816(acc[mt], a0, a1, a2, a3, xw[2 * e], xw[2 * e + 1]);
          }
        }
      }
  }

  // accumulator layout: c0,c1 = (row g, cols 2t, 2t+1); c2,c3 = (row g+8, same cols)
#pragma unroll
  for (int mt = 0; mt < MT; ++mt) {
    red[warp][mt * 16 + g][2 * t] = acc[mt][0];
    red[warp][mt * 16 + g][2 * t + 1] = acc[mt][1];
    red[warp][mt * 16 + g + 8][2 * t] = acc[mt][2];
    red[warp][mt * 16 + g + 8][2 * t + 1] = acc[mt][3];
  }
  __syncthreads();

  const OutScalars r = out_begin(o);
  float mx = 0.f;
  for (int idx = threadIdx.x; idx < MT * 16 * 8; idx += GV_WARPS * 32) {
    const int il = idx % (MT * 16), j = idx / (MT * 16), i = row0 + il;
    if (i < m && j < n) {
      float s = red[0][il][j];
#pragma unroll
      for (int w = 1; w < GV_WARPS; ++w) s = __fadd_rn(s, red[w][il][j]);
      mx = fmaxf(mx, out_store(o, r, i, j, s));
    }
  }
  if (o.amax) block_amax(o.amax, mx);
}

// ---- the same computation with an asynchronous weight pipeline ---------------------------------
// Every lane copies its own fragments (rows g and g+8, two 16-byte pieces of a warp's 128-byte k-step)
// with cp.async straight into a private shared-memory slot, GA_STAGES k-steps ahead, and reads them
// back when their group has landed.  The bytes in flight no longer occupy registers (the kernel
// above needs 64-80 registers for its load buffers, which caps it at 3-4 blocks per SM and leaves
// every warp waiting on its own loads); no barrier is involved because a lane only ever reads
// what it copied itself.  Out-of-range rows and k positions are copied with a source size of 0,
// which zero-fills the slot.

// wide: ask L2 to fetch the whole 256-byte pair of lines on a miss (the warp's next k-step is the other half)
__device__ __forceinline__ void cp_async16(uint32_t smem_dst, const void *gsrc, bool live, bool wide) {
  const int bytes = live ? 16 : 0;
  if (wide) asm volatile("cp.async.cg.shared.global.L2::256B [%0], [%1], 16, %2;" ::"r"(smem_dst), "l"(gsrc), "r"(bytes) : "memory");
  else asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_dst), "l"(gsrc), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// kmap 0: the eight warps interleave 128-byte k-steps (step it of warp w is k-block w + 8 it); kmap 1: each warp
// owns one contiguous eighth of K and walks it 128 bytes at a time (its consecutive steps are neighbours in DRAM).
template <int AT, int XT, int GA_STAGES>
__global__ void __launch_bounds__(GV_WARPS * 32) gemv_async_kernel(const uint8_t *__restrict__ W, int lda,
                                                                   const uint8_t *__restrict__ X, int ldx, int m, int n,
                                                                   int k, int kmap, OutDesc o) {
  extern __shared__ __align__(16) uint8_t ring_raw[];        // [warp][stage][fragment 0..3][lane] x 16 bytes
  __shared__ float red[GV_WARPS][16][9];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;
  const int row0 = blockIdx.x * 16;
  constexpr int XB = XT == E5MA_BF16 ? 2 : 1;
  constexpr int XW = XT == E5MA_BF16 ? 2 : 1;
  uint8_t *my_ring = ring_raw + (size_t)warp * GA_STAGES * 2048 + lane * 16;
  const uint32_t my_ring_s = (uint32_t)__cvta_generic_to_shared(my_ring);

  const int ra = row0 + g, rb = ra + 8;
  const bool la = ra < m, lb = rb < m;
  const uint8_t *wa = W + (size_t)(la ? ra : 0) * lda, *wb = W + (size_t)(lb ? rb : 0) * lda;
  // this warp's k-steps of 128 bytes: step it starts at kstart(it)
  const int kblocks = (k + 127) / 128, per_warp = (kblocks + GV_WARPS - 1) / GV_WARPS;
  const int steps = kmap ? (kblocks - warp * per_warp < per_warp ? (kblocks > warp * per_warp ? kblocks - warp * per_warp : 0) : per_warp)
                         : (k > warp * 128 ? (k - warp * 128 + GV_WARPS * 128 - 1) / (GV_WARPS * 128) : 0);
  const auto kstart = [&](int it) { return (kmap ? warp * per_warp + it : warp + GV_WARPS * it) * 128; };
  const bool wide = kmap != 0;
  const auto issue = [&](int it) {
    if (it < steps) {
      const int kc = kstart(it) + t * 16;
      const uint32_t dst = my_ring_s + (uint32_t)(it % GA_STAGES) * 2048;
      cp_async16(dst, wa + kc, la && kc < k, wide);
      cp_async16(dst + 512, wb + kc, lb && kc < k, wide);
      cp_async16(dst + 1024, wa + kc + 64, la && kc + 64 < k, wide);
      cp_async16(dst + 1536, wb + kc + 64, lb && kc + 64 < k, wide);
    }
    cp_async_commit();     // one group per step, also when it is empty: the wait below counts groups
  };
#pragma unroll
  for (int it = 0; it < GA_STAGES - 1; ++it) issue(it);

  // two accumulator sets: consecutive MMAs do not wait on each other's result
  float acc[4] = {0.f, 0.f, 0.f, 0.f}, acc2[4] = {0.f, 0.f, 0.f, 0.f};
  const uint8_t *xcol = X + (size_t)g * ldx * XB;
  const bool xlive = g < n;
  const auto load_x = [&](int it, uint4 (&xq)[2][XW]) {
    const int kc = kstart(it);
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int kk = kc + h * 64 + t * 16;
#pragma unroll
      for (int q = 0; q < XW; ++q)
        xq[h][q] = xlive && kk < k ? __ldg(reinterpret_cast<const uint4 *>(xcol + (size_t)kk * XB) + q) : make_uint4(0, 0, 0, 0);
    }
  };
  uint4 xq[2][XW], xn[2][XW];
  load_x(0, xq);
  for (int it = 0; it < steps; ++it) {
    issue(it + GA_STAGES - 1);
    load_x(it + 1, xn);               // X of the next step is fetched while this one is consumed (zeros beyond k)
    cp_async_wait<GA_STAGES - 1>();   // all but the newest GA_STAGES - 1 groups are complete: step `it` has landed
    const uint8_t *slot = my_ring + (size_t)(it % GA_STAGES) * 2048;
    uint4 wq[2][2];
    wq[0][0] = *reinterpret_cast<const uint4 *>(slot);
    wq[0][1] = *reinterpret_cast<const uint4 *>(slot + 512);
    wq[1][0] = *reinterpret_cast<const uint4 *>(slot + 1024);
    wq[1][1] = *reinterpret_cast<const uint4 *>(slot + 1536);
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      uint32_t xw[8];
      if (XT == E5MA_BF16) {
        xw[0] = xq[h][0].x; xw[1] = xq[h][0].y; xw[2] = xq[h][0].z; xw[3] = xq[h][0].w;
        xw[4] = xq[h][XW - 1].x; xw[5] = xq[h][XW - 1].y; xw[6] = xq[h][XW - 1].z; xw[7] = xq[h][XW - 1].w;
      } else {
        const uint32_t q[4] = {xq[h][0].x, xq[h][0].y, xq[h][0].z, xq[h][0].w};
#pragma unroll
        for (int e = 0; e < 4; ++e) fp8x4_to_bf16x2<XT == E5MA_BF16 ? E5MA_E5M2 : XT>(q[e], xw[2 * e], xw[2 * e + 1]);
      }
      const uint32_t qa[4] = {wq[h][0].x, wq[h][0].y, wq[h][0].z, wq[h][0].w};
      const uint32_t qb[4] = {wq[h][1].x, wq[h][1].y, wq[h][1].z, wq[h][1].w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        uint32_t a0, a2, a1, a3;
        fp8x4_to_bf16x2<AT>(qa[e], a0, a2);   // row g:   k pairs (0,1) and (2,3) of this word
        fp8x4_to_bf16x2<AT>(qb[e], a1, a3);   // row g+8
        mma_bf16_16816((e & 1) ? acc2 : acc, a0, a1, a2, a3, xw[2 * e], xw[2 * e + 1]);
      }
    }
#pragma unroll
    for (int h = 0; h < 2; ++h)
#pragma unroll
      for (int q = 0; q < XW; ++q) xq[h][q] = xn[h][q];
  }
#pragma unroll
  for (int e = 0; e < 4; ++e) acc[e] = __fadd_rn(acc[e], acc2[e]);
  cp_async_wait<0>();

  red[warp][g][2 * t] = acc[0];
  red[warp][g][2 * t + 1] = acc[1];
  red[warp][g + 8][2 * t] = acc[2];
  red[warp][g + 8][2 * t + 1] = acc[3];
  __syncthreads();
  const OutScalars r = out_begin(o);
  float mx = 0.f;
  if (threadIdx.x < 128) {
    const int il = threadIdx.x & 15, j = threadIdx.x >> 4, i = row0 + il;
    if (i < m && j < n) {
      float s = red[0][il][j];
#pragma unroll
      for (int w = 1; w < GV_WARPS; ++w) s = __fadd_rn(s, red[w][il][j]);
      mx = out_store(o, r, i, j, s);
    }
  }
  if (o.amax) block_amax(o.amax, mx);
}

// ---- tensor-core kernel with row streams -------------------------------------------------------------
// The arithmetic of gemv_async_kernel behind the access pattern of the FP32-pipe kernel below: the block's eight
// warps copy a stage of 16 rows x 512 bytes together, warp w rows 2w and 2w + 1 with one cp.async instruction per
// row (512 contiguous bytes per instruction, every row a sequential stream), S stages ahead; a stage that has landed
// is consumed by all warps, warp w taking bytes [64 w, 64 w + 64) of each row as two of the 16-byte fragments above.
// One block barrier per stage makes the copies of all warps visible and frees the slot consumed before it.  Rows
// are 576 bytes apart in shared memory, so the 16-byte reads of a quarter warp (two rows x four k-chunks) hit
// distinct banks.
constexpr int GR_PITCH = 512 + 64, GR_STAGE = 16 * GR_PITCH;

template <int AT, int XT, int S>
__global__ void __launch_bounds__(GV_WARPS * 32) gemv_rows_kernel(const uint8_t *__restrict__ W, int lda,
                                                                  const uint8_t *__restrict__ X, int ldx, int m, int n,
                                                                  int k, OutDesc o) {
  extern __shared__ __align__(16) uint8_t ring_raw[];        // [stage][row 0..15][576 bytes]
  __shared__ float red[GV_WARPS][16][9];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;
  const int row0 = blockIdx.x * 16;
  constexpr int XB = XT == E5MA_BF16 ? 2 : 1;
  constexpr int XW = XT == E5MA_BF16 ? 2 : 1;
  const uint32_t ring_s = (uint32_t)__cvta_generic_to_shared(ring_raw);

  // copies: rows 2 warp and 2 warp + 1, bytes [16 lane, 16 lane + 16) of the stage
  const int ca = row0 + 2 * warp, cb = ca + 1;
  const bool la = ca < m, lb = cb < m;
  const uint8_t *wa = W + (size_t)(la ? ca : 0) * lda + lane * 16, *wb = W + (size_t)(lb ? cb : 0) * lda + lane * 16;
  const uint32_t dst0 = ring_s + (uint32_t)(2 * warp) * GR_PITCH + lane * 16;
  const int stages = (k + 511) / 512;
  const auto issue = [&](int it) {
    if (it < stages) {
      const int kc = it * 512;
      const bool in = kc + lane * 16 < k;
      const uint32_t dst = dst0 + (uint32_t)(it % S) * GR_STAGE;
      cp_async16(dst, wa + kc, la && in, false);
      cp_async16(dst + GR_PITCH, wb + kc, lb && in, false);
    }
    cp_async_commit();
  };
#pragma unroll
  for (int it = 0; it < S - 1; ++it) issue(it);

  float acc[4] = {0.f, 0.f, 0.f, 0.f}, acc2[4] = {0.f, 0.f, 0.f, 0.f};
  const uint8_t *xcol = X + (size_t)g * ldx * XB;
  const bool xlive = g < n;
  const int koff = warp * 64 + t * 16;           // this lane's 16 k positions inside a stage
  const auto load_x = [&](int it, uint4 (&xq)[XW]) {
    const int kk = it * 512 + koff;
#pragma unroll
    for (int q = 0; q < XW; ++q)
      xq[q] = xlive && kk < k ? __ldg(reinterpret_cast<const uint4 *>(xcol + (size_t)kk * XB) + q) : make_uint4(0, 0, 0, 0);
  };
  uint4 xq[XW], xn[XW];
  load_x(0, xq);
  const uint8_t *frag = ring_raw + (size_t)g * GR_PITCH + koff;
  for (int it = 0; it < stages; ++it) {
    cp_async_wait<S - 2>();           // this thread's copies of stage `it` have landed ...
    __syncthreads();                  // ... everybody's have, and everybody is done with stage it - 1
    issue(it + S - 1);                // refills the slot of stage it - 1
    load_x(it + 1, xn);
    const uint8_t *slot = frag + (size_t)(it % S) * GR_STAGE;
    const uint4 wq0 = *reinterpret_cast<const uint4 *>(slot);
    const uint4 wq1 = *reinterpret_cast<const uint4 *>(slot + 8 * GR_PITCH);
    uint32_t xw[8];
    if (XT == E5MA_BF16) {
      xw[0] = xq[0].x; xw[1] = xq[0].y; xw[2] = xq[0].z; xw[3] = xq[0].w;
      xw[4] = xq[XW - 1].x; xw[5] = xq[XW - 1].y; xw[6] = xq[XW - 1].z; xw[7] = xq[XW - 1].w;
    } else {
      const uint32_t q[4] = {xq[0].x, xq[0].y, xq[0].z, xq[0].w};
#pragma unroll
      for (int e = 0; e < 4; ++e) fp8x4_to_bf16x2<XT == E5MA_BF16 ? E5MA_E5M2 : XT>(q[e], xw[2 * e], xw[2 * e + 1]);
    }
    const uint32_t qa[4] = {wq0.x, wq0.y, wq0.z, wq0.w};
    const uint32_t qb[4] = {wq1.x, wq1.y, wq1.z, wq1.w};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      uint32_t a0, a2, a1, a3;
      fp8x4_to_bf16x2<AT>(qa[e], a0, a2);   // row g:   k pairs (0,1) and (2,3) of this word
      fp8x4_to_bf16x2<AT>(qb[e], a1, a3);   // row g+8
      mma_bf16_16816((e & 1) ? acc2 : acc, a0, a1, a2, a3, xw[2 * e], xw[2 * e + 1]);
    }
#pragma unroll
    for (int q = 0; q < XW; ++q) xq[q] = xn[q];
  }
#pragma unroll
  for (int e = 0; e < 4; ++e) acc[e] = __fadd_rn(acc[e], acc2[e]);
  cp_async_wait<0>();

  red[warp][g][2 * t] = acc[0];
  red[warp][g][2 * t + 1] = acc[1];
  red[warp][g + 8][2 * t] = acc[2];
  red[warp][g + 8][2 * t + 1] = acc[3];
  __syncthreads();
  const OutScalars r = out_begin(o);
  float mx = 0.f;
  if (threadIdx.x < 128) {
    const int il = threadIdx.x & 15, j = threadIdx.x >> 4, i = row0 + il;
    if (i < m && j < n) {
      float s = red[0][il][j];
#pragma unroll
      for (int w = 1; w < GV_WARPS; ++w) s = __fadd_rn(s, red[w][il][j]);
      mx = out_store(o, r, i, j, s);
    }
  }
  if (o.amax) block_amax(o.amax, mx);
}

// ---- the same stream on the FP32 pipe: long contiguous reads, one FMA per product ------------------------
// A warp owns R whole rows (over 1 / KS of K) and walks them 512 bytes at a time: 16 bytes per lane and row, so
// one load instruction of a warp covers 512 contiguous bytes of one row and a row is read front to back by the
// same warp -- the access pattern DRAM likes best (measured on 8192 x 8192 weights, batch 1: 14.7 us against
// 16.1 us for the tensor-core kernel above, whose warps gather 16 rows x 128 bytes per step).  The price is the
// arithmetic: every lane keeps R x NC running sums of its own k positions and spends one FP32 FMA per product, as
// the reference's gemv_kernel does (src/gemv_e5m2effma.cuh:27-79), so the kernel only pays for small n -- and for
// FP32 activations, which do not fit a tensor-core operand without splitting them and which the reference routes
// here like every other skinny problem with FP8 weights (src/gemm_e5m2effma.cu:100-102).
// W is decoded exactly; X of any operand dtype becomes FP32 exactly; a butterfly adds the lanes, the KS parts meet
// in shared memory in a fixed order and 128 threads run the common epilogue.  NC = n rounded up to 1, 2, 4, 8.

// four consecutive X values of column storage `col` (XT elements) starting at element k0 -> FP32
template <int XT>
__device__ __forceinline__ void load_x4(const uint8_t *col, int k0, float x[4]) {
  if (XT == E5MA_FP32) {
    const float4 v = __ldg(reinterpret_cast<const float4 *>(col) + (k0 >> 2));
    x[0] = v.x; x[1] = v.y; x[2] = v.z; x[3] = v.w;
  } else if (XT == E5MA_BF16) {
    const uint2 v = __ldg(reinterpret_cast<const uint2 *>(col) + (k0 >> 2));
    x[0] = __uint_as_float(v.x << 16); x[1] = __uint_as_float(v.x & 0xFFFF0000u);
    x[2] = __uint_as_float(v.y << 16); x[3] = __uint_as_float(v.y & 0xFFFF0000u);
  } else {
    fp8x4_to_f32<XT == E5MA_E4M3 ? E5MA_E4M3 : E5MA_E5M2>(__ldg(reinterpret_cast<const uint32_t *>(col) + (k0 >> 2)), x);
  }
}

template <int AT, int XT, int NC, int R>
__global__ void __launch_bounds__(GV_WARPS * 32) gemv_fma_kernel(const uint8_t *__restrict__ W, int lda,
                                                                 const uint8_t *__restrict__ X, int ldx, int m, int n, int k,
                                                                 OutDesc o) {
  constexpr int GROUPS = 16 / R, KS = GV_WARPS / GROUPS;
  __shared__ float red[KS][16][9];
  constexpr int XB = XT == E5MA_FP32 ? 4 : (XT == E5MA_BF16 ? 2 : 1);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int grp = warp % GROUPS, ks = warp / GROUPS;
  const int row0 = blockIdx.x * 16 + grp * R;
  const int chunks = (k + 511) / 512, per = (chunks + KS - 1) / KS;
  const int kbeg = ks * per * 512, kend = (ks + 1) * per * 512 < k ? (ks + 1) * per * 512 : k;

  const uint8_t *wrow[R];
  bool live[R];
#pragma unroll
  for (int r = 0; r < R; ++r) {
    live[r] = row0 + r < m;
    wrow[r] = W + (size_t)(live[r] ? row0 + r : 0) * lda;
  }
  float acc[R][NC];
#pragma unroll
  for (int r = 0; r < R; ++r)
#pragma unroll
    for (int j = 0; j < NC; ++j) acc[r][j] = 0.f;

  uint4 cur[R], nxt[R];
  const auto load_w = [&](uint4 (&q)[R], int k0) {
#pragma unroll
    for (int r = 0; r < R; ++r) q[r] = live[r] && k0 < kend ? ld_stream16(wrow[r] + k0) : make_uint4(0, 0, 0, 0);
  };
  load_w(cur, kbeg + lane * 16);
  for (int kb = kbeg; kb < kend; kb += 512) {
    const int k0 = kb + lane * 16;
    load_w(nxt, k0 + 512);
    const bool in = k0 < kend;
#pragma unroll
    for (int q = 0; q < 4; ++q) {          // one 32-bit word of every row: four codes against four values of every column
      float wf[R][4];
#pragma unroll
      for (int r = 0; r < R; ++r) {
        const uint32_t word = q == 0 ? cur[r].x : q == 1 ? cur[r].y : q == 2 ? cur[r].z : cur[r].w;
        fp8x4_to_f32<AT>(word, wf[r]);
      }
#pragma unroll
      for (int j = 0; j < NC; ++j) {
        float x[4] = {0.f, 0.f, 0.f, 0.f};
        if (in && j < n) load_x4<XT>(X + (size_t)j * ldx * XB, k0 + 4 * q, x);
#pragma unroll
        for (int r = 0; r < R; ++r)
#pragma unroll
          for (int e = 0; e < 4; ++e) acc[r][j] = __fmaf_rn(wf[r][e], x[e], acc[r][j]);
      }
    }
#pragma unroll
    for (int r = 0; r < R; ++r) cur[r] = nxt[r];
  }

#pragma unroll
  for (int r = 0; r < R; ++r)
#pragma unroll
    for (int j = 0; j < NC; ++j) {
      float v = acc[r][j];
#pragma unroll
      for (int d = 16; d; d >>= 1) v = __fadd_rn(v, __shfl_xor_sync(0xFFFFFFFFu, v, d));
      if (lane == r * NC + j) red[ks][grp * R + r][j] = v;
    }
  __syncthreads();
  const OutScalars sc = out_begin(o);
  float mx = 0.f;
  if (threadIdx.x < 128) {
    const int il = threadIdx.x & 15, j = threadIdx.x >> 4, i = blockIdx.x * 16 + il;
    if (i < m && j < n) {
      float s = red[0][il][j];
#pragma unroll
      for (int p = 1; p < KS; ++p) s = __fadd_rn(s, red[p][il][j]);
      mx = out_store(o, sc, i, j, s);
    }
  }
  if (o.amax) block_amax(o.amax, mx);
}

// Wider batches on the FP32 pipe (FP32 activations only: the others have the tensor-core kernel).  Reading X per lane
// straight from L1 / L2 as above costs NC loads per four codes and drowns the weight stream (8192 x 8192, n = 8:
// 183 us).  Here every warp of the block owns two rows over all of K, so that all warps need the same 512 k
// positions of X at the same time: the block stages them in shared memory once per step (double-buffered, laid out
// [group of four k][lane] so that the lanes' 16-byte reads are conflict-free) and a lane reads them from there.
template <int AT, int NC>
__global__ void __launch_bounds__(GV_WARPS * 32) gemv_fma_staged_kernel(const uint8_t *__restrict__ W, int lda,
                                                                        const float *__restrict__ X, int ldx, int m, int n,
                                                                        int k, OutDesc o) {
  constexpr int R = 2;
  __shared__ __align__(16) float xs[2][NC][512];
  __shared__ float red[16][9];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int row0 = blockIdx.x * 16 + warp * R;
  const uint8_t *wrow[R];
  bool live[R];
#pragma unroll
  for (int r = 0; r < R; ++r) {
    live[r] = row0 + r < m;
    wrow[r] = W + (size_t)(live[r] ? row0 + r : 0) * lda;
  }
  float acc[R][NC];
#pragma unroll
  for (int r = 0; r < R; ++r)
#pragma unroll
    for (int j = 0; j < NC; ++j) acc[r][j] = 0.f;

  // X[j][kb + 4c .. 4c + 4) -> xs[buf][j][((c & 3) * 32 + (c >> 2)) * 4 ..]: c >> 2 is the lane that owns these k
  const auto stage = [&](int buf, int kb) {
    for (int idx = threadIdx.x; idx < NC * 128; idx += GV_WARPS * 32) {
      const int j = idx >> 7, c = idx & 127, kk = kb + 4 * c;
      const float4 v = j < n && kk < k ? __ldg(reinterpret_cast<const float4 *>(X + (size_t)j * ldx + kk)) : make_float4(0.f, 0.f, 0.f, 0.f);
      *reinterpret_cast<float4 *>(&xs[buf][j][((c & 3) * 32 + (c >> 2)) * 4]) = v;
    }
  };
  uint4 cur[R], nxt[R];
  const auto load_w = [&](uint4 (&q)[R], int k0) {
#pragma unroll
    for (int r = 0; r < R; ++r) q[r] = live[r] && k0 < k ? ld_stream16(wrow[r] + k0) : make_uint4(0, 0, 0, 0);
  };
  load_w(cur, lane * 16);
  stage(0, 0);
  __syncthreads();
  int buf = 0;
  for (int kb = 0; kb < k; kb += 512, buf ^= 1) {
    load_w(nxt, kb + 512 + lane * 16);
    if (kb + 512 < k) stage(buf ^ 1, kb + 512);
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      float wf[R][4];
#pragma unroll
      for (int r = 0; r < R; ++r) {
        const uint32_t word = q == 0 ? cur[r].x : q == 1 ? cur[r].y : q == 2 ? cur[r].z : cur[r].w;
        fp8x4_to_f32<AT>(word, wf[r]);
      }
#pragma unroll
      for (int j = 0; j < NC; ++j) {
        const float4 x = *reinterpret_cast<const float4 *>(&xs[buf][j][(q * 32 + lane) * 4]);
#pragma unroll
        for (int r = 0; r < R; ++r) {
          acc[r][j] = __fmaf_rn(wf[r][0], x.x, acc[r][j]);
          acc[r][j] = __fmaf_rn(wf[r][1], x.y, acc[r][j]);
          acc[r][j] = __fmaf_rn(wf[r][2], x.z, acc[r][j]);
          acc[r][j] = __fmaf_rn(wf[r][3], x.w, acc[r][j]);
        }
      }
    }
#pragma unroll
    for (int r = 0; r < R; ++r) cur[r] = nxt[r];
    __syncthreads();     // the other buffer is complete; this one may be overwritten by the next step's staging
  }

#pragma unroll
  for (int r = 0; r < R; ++r)
#pragma unroll
    for (int j = 0; j < NC; ++j) {
      float v = acc[r][j];
#pragma unroll
      for (int d = 16; d; d >>= 1) v = __fadd_rn(v, __shfl_xor_sync(0xFFFFFFFFu, v, d));
      if (lane == r * NC + j) red[warp * R + r][j] = v;
    }
  __syncthreads();
  const OutScalars sc = out_begin(o);
  float mx = 0.f;
  if (threadIdx.x < 128) {
    const int il = threadIdx.x & 15, j = threadIdx.x >> 4, i = blockIdx.x * 16 + il;
    if (i < m && j < n) mx = out_store(o, sc, i, j, red[il][j]);
  }
  if (o.amax) block_amax(o.amax, mx);
}

template <int AT, int XT>
static cudaError_t gemv_fma_x(const uint8_t *A, int lda, const uint8_t *X, int ldx, int m, int n, int k, const OutDesc &o,
                              cudaStream_t s) {
  const unsigned grid = (unsigned)((m + 15) / 16);
  if (n == 1) gemv_fma_kernel<AT, XT, 1, 4><<<grid, GV_WARPS * 32, 0, s>>>(A, lda, X, ldx, m, n, k, o);
  else if (n == 2) gemv_fma_kernel<AT, XT, 2, 4><<<grid, GV_WARPS * 32, 0, s>>>(A, lda, X, ldx, m, n, k, o);
  else if (XT == E5MA_FP32 && n <= 4) gemv_fma_staged_kernel<AT, 4><<<grid, GV_WARPS * 32, 0, s>>>(A, lda, reinterpret_cast<const float *>(X), ldx, m, n, k, o);
  else if (XT == E5MA_FP32) gemv_fma_staged_kernel<AT, 8><<<grid, GV_WARPS * 32, 0, s>>>(A, lda, reinterpret_cast<const float *>(X), ldx, m, n, k, o);
  else if (n <= 4) gemv_fma_kernel<AT, XT, 4, 2><<<grid, GV_WARPS * 32, 0, s>>>(A, lda, X, ldx, m, n, k, o);
  else return cudaErrorNotSupported;
  return cudaGetLastError();
}
template <int AT>
static cudaError_t gemv_fma(int x_dtype, const uint8_t *A, int lda, const uint8_t *X, int ldx, int m, int n, int k,
                            const OutDesc &o, cudaStream_t s) {
  switch (x_dtype) {
    case E5MA_FP32: return gemv_fma_x<AT, E5MA_FP32>(A, lda, X, ldx, m, n, k, o, s);
    case E5MA_BF16: return gemv_fma_x<AT, E5MA_BF16>(A, lda, X, ldx, m, n, k, o, s);
    case E5MA_E5M2: return gemv_fma_x<AT, E5MA_E5M2>(A, lda, X, ldx, m, n, k, o, s);
    case E5MA_E4M3: return gemv_fma_x<AT, E5MA_E4M3>(A, lda, X, ldx, m, n, k, o, s);
    default: return cudaErrorNotSupported;
  }
}

// ---- persistent kernel with a bulk-copy weight ring ------------------------------------------------
// One CTA per SM walks over 16-row tiles of W.  A producer warp streams the tile's rows into a ring of
// shared-memory stages with bulk asynchronous copies (16 rows x 1 KiB per stage, one copy per row, completion
// counted on an mbarrier), several stages ahead and across tile boundaries, so the bytes in flight cost neither
// registers nor issue slots of the eight consumer warps.  The consumers split a stage's 1 KiB of K between them
// (128 bytes per warp, as in the kernels above) and feed mma.sync.m16n8k16 with X as the 8-column operand.
//
// What makes the instruction stream short: X is staged once per CTA in shared memory as FP16, W is widened
// to FP16 with one byte permute (E5M2 is the upper byte of an FP16) or one converter instruction (E4M3) per two
// codes, and the FP16 tensor-core path is used -- products stay exact (4 x 11 significant bits), sums are FP32.
// FP8 X always converts exactly.  A BF16 X does whenever every value is representable in FP16, which the CTA
// checks while staging; if one is not (|x| >= 65520, or bits below 2^-24), the CTA stages X as BF16 instead and
// widens W to BF16 as the kernels above do.  Both paths add the same exact products in the same order, so the
// choice does not show in the result.
//
// Rows are padded to 1088 bytes in the ring and X columns to a pitch of 16 mod 128 bytes: the 16-byte reads of
// a quarter warp (two rows / columns x four k-chunks) then hit distinct banks.
// Per tile the eight partial 16 x 8 tiles meet in shared memory in a fixed order (two buffers alternate, one
// named barrier per tile) and 128 threads run the common epilogue.  Every mbarrier wait is bounded.
constexpr int GB_ROW_PITCH = 1024 + 64;
constexpr int GB_STAGE_BYTES = 16 * GB_ROW_PITCH;
constexpr int GB_MAX_STAGES = 8;
constexpr int GB_THREADS = GV_WARPS * 32 + 32;
constexpr unsigned long long GB_WAIT_LIMIT = 4000000000ull;

__device__ unsigned int g_gemv_fault;

__device__ __forceinline__ uint32_t gb_smem(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ bool gb_try(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile("{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
               : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool gb_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag, unsigned int who) {
  if (gb_try(bar, parity)) return true;
  const unsigned long long t0 = clock64();
  for (;;) {
    for (int i = 0; i < 64; ++i)
      if (gb_try(bar, parity)) return true;
    if (*abort_flag) return false;
    if ((unsigned long long)(clock64() - t0) > GB_WAIT_LIMIT) {
      *abort_flag = 1;
      atomicCAS(&g_gemv_fault, 0u, who);
      return false;
    }
  }
}
__device__ __forceinline__ void gb_bulk_load(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ void mma_f16_16816(float c[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                              uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
               "{%0, %1, %2, %3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// four FP8 codes (ascending k) -> FP16 pairs (k0,k1), (k2,k3), exact
template <int T>
__device__ __forceinline__ void fp8x4_to_f16x2(uint32_t w, uint32_t &lo, uint32_t &hi) {
  if (T == E5MA_E5M2) { lo = __byte_perm(w, 0, 0x1404); hi = __byte_perm(w, 0, 0x3424); }
  else { lo = e4m3x2_to_f16x2(w); hi = e4m3x2_to_f16x2(w >> 16); }
}

template <int AT, int XT>
__global__ void __launch_bounds__(GB_THREADS, 1) gemv_bulk_kernel(const uint8_t *__restrict__ W, int lda,
                                                                  const uint8_t *__restrict__ X, int ldx, int m, int n,
                                                                  int k, int stages, int x_pitch, OutDesc o) {
  extern __shared__ __align__(128) uint8_t gb_raw[];
  // [x: n columns x x_pitch bytes][ring: stages x 16 rows x 1088 bytes][red: 2 x 8 x 16 x 9 floats][barriers][flags]
  uint8_t *xs = gb_raw;
  uint8_t *ringp = xs + (size_t)n * x_pitch;
  float (*red)[GV_WARPS][16][9] = reinterpret_cast<float (*)[GV_WARPS][16][9]>(ringp + (size_t)stages * GB_STAGE_BYTES);
  uint64_t *bars = reinterpret_cast<uint64_t *>(reinterpret_cast<uint8_t *>(red) + 2 * GV_WARPS * 16 * 9 * sizeof(float));
  volatile int *abort_flag = reinterpret_cast<volatile int *>(bars + 2 * GB_MAX_STAGES);
  volatile int *x_fits_f16 = abort_flag + 1;
  const uint32_t bar0 = gb_smem(bars), ring_s = gb_smem(ringp);
  const auto full_bar = [&](int s) { return bar0 + 8u * s; };
  const auto empty_bar = [&](int s) { return bar0 + 8u * (GB_MAX_STAGES + s); };

  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;
  const int tiles = (m + 15) / 16, chunks = (k + 1023) / 1024;
  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(full_bar(s)), "r"(1));
      asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(empty_bar(s)), "r"(GV_WARPS));
    }
    *abort_flag = 0;
    *x_fits_f16 = 1;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  __syncthreads();

  float mx = 0.f;
  if (warp == GV_WARPS) {
    // ---------------- producer: one bulk copy per row and stage, issued by lanes 0..15 ----------------
    int s = 0;
    uint32_t ph = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x) {
      const int row = tile * 16 + lane;
      const bool live = lane < 16 && row < m;
      const int live_rows = m - tile * 16 < 16 ? m - tile * 16 : 16;
      const uint8_t *src = W + (size_t)(live ? row : 0) * lda;
      for (int c = 0; c < chunks; ++c) {
        const uint32_t bytes = (uint32_t)(k - c * 1024 < 1024 ? k - c * 1024 : 1024);
        ok = gb_wait(empty_bar(s), ph ^ 1u, abort_flag, (1u << 24) | (uint32_t)c);
        ok = __all_sync(0xFFFFFFFFu, ok);
        if (!ok) break;
        if (lane == 0)
          asm volatile("{ .reg .b64 st; mbarrier.arrive.expect_tx.shared::cta.b64 st, [%0], %1; }"
                       ::"r"(full_bar(s)), "r"(bytes * (uint32_t)live_rows) : "memory");
        __syncwarp();
        if (live) gb_bulk_load(ring_s + (uint32_t)s * GB_STAGE_BYTES + (uint32_t)lane * GB_ROW_PITCH, src + (size_t)c * 1024, bytes, full_bar(s));
        if (++s == stages) { s = 0; ph ^= 1u; }
      }
    }
  } else {
    // ---------------- consumers ----------------
    // X -> shared memory, FP16 when every value converts exactly (FP8 always does), else BF16 as it is
    const int ct = threadIdx.x;                       // 0 .. 255
    constexpr int XE = XT == E5MA_BF16 ? 8 : 16;      // elements per 16-byte load
    const int per_col = k / XE;                       // k is a multiple of 16
    bool fits = true;
    for (int idx = ct; idx < n * per_col; idx += GV_WARPS * 32) {
      const int j = idx / per_col, q = idx - j * per_col;
      const uint4 v = __ldg(reinterpret_cast<const uint4 *>(X + ((size_t)j * ldx + (size_t)q * XE) * (XT == E5MA_BF16 ? 2 : 1)));
      const uint32_t w[4] = {v.x, v.y, v.z, v.w};
      if (XT == E5MA_BF16) {
        uint32_t h[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float lo = __uint_as_float(w[e] << 16), hi = __uint_as_float(w[e] & 0xFFFF0000u);
          const __half2 hh = __floats2half2_rn(lo, hi);
          const float2 back = __half22float2(hh);
          fits = fits && back.x == lo && back.y == hi;
          h[e] = *reinterpret_cast<const uint32_t *>(&hh);
        }
        *reinterpret_cast<uint4 *>(xs + (size_t)j * x_pitch + (size_t)q * 16) = make_uint4(h[0], h[1], h[2], h[3]);
      } else {
        uint32_t h[8];
#pragma unroll
        for (int e = 0; e < 4; ++e) fp8x4_to_f16x2<XT == E5MA_BF16 ? E5MA_E5M2 : XT>(w[e], h[2 * e], h[2 * e + 1]);
        uint4 *dst = reinterpret_cast<uint4 *>(xs + (size_t)j * x_pitch + (size_t)q * 32);
        dst[0] = make_uint4(h[0], h[1], h[2], h[3]);
        dst[1] = make_uint4(h[4], h[5], h[6], h[7]);
      }
    }
    if (!fits) *x_fits_f16 = 0;
    asm volatile("bar.sync 1, %0;" ::"n"(GV_WARPS * 32) : "memory");
    const bool f16 = *x_fits_f16 != 0;
    if (XT == E5MA_BF16 && !f16) {
      asm volatile("bar.sync 1, %0;" ::"n"(GV_WARPS * 32) : "memory");   // everybody has read the flag and is done with the FP16 copy
      for (int idx = ct; idx < n * per_col; idx += GV_WARPS * 32) {
        const int j = idx / per_col, q = idx - j * per_col;
        *reinterpret_cast<uint4 *>(xs + (size_t)j * x_pitch + (size_t)q * 16) =
            __ldg(reinterpret_cast<const uint4 *>(X + ((size_t)j * ldx + (size_t)q * 8) * 2));
      }
      asm volatile("bar.sync 1, %0;" ::"n"(GV_WARPS * 32) : "memory");
    }

    const OutScalars r = out_begin(o);
    const uint8_t *xcol = xs + (size_t)g * x_pitch;
    const bool xlive = g < n;
    int s = 0;
    uint32_t ph = 0, lt = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x, ++lt) {
      float acc[4] = {0.f, 0.f, 0.f, 0.f}, acc2[4] = {0.f, 0.f, 0.f, 0.f};
      for (int c = 0; c < chunks; ++c) {
        ok = gb_wait(full_bar(s), ph, abort_flag, (2u << 24) | (uint32_t)c);
        ok = __all_sync(0xFFFFFFFFu, ok);
        if (!ok) break;
        const uint8_t *stage = ringp + (size_t)s * GB_STAGE_BYTES;
        const int kw = c * 1024 + warp * 128;            // first k of this warp's slice
        if (kw < k) {
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const int kk = kw + h * 64 + t * 16;
            const bool live = kk < k;
            uint4 qa = make_uint4(0, 0, 0, 0), qb = qa, x0 = qa, x1 = qa;
            if (live) {
              qa = *reinterpret_cast<const uint4 *>(stage + g * GB_ROW_PITCH + (kk - c * 1024));
              qb = *reinterpret_cast<const uint4 *>(stage + (g + 8) * GB_ROW_PITCH + (kk - c * 1024));
              if (xlive) {
                x0 = *reinterpret_cast<const uint4 *>(xcol + (size_t)kk * 2);
                x1 = *reinterpret_cast<const uint4 *>(xcol + (size_t)kk * 2 + 16);
              }
            }
            const uint32_t wa[4] = {qa.x, qa.y, qa.z, qa.w}, wb[4] = {qb.x, qb.y, qb.z, qb.w};
            const uint32_t xw[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
            if (f16) {
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                uint32_t a0, a2, a1, a3;
                fp8x4_to_f16x2<AT>(wa[e], a0, a2);
                fp8x4_to_f16x2<AT>(wb[e], a1, a3);
                mma_f16_16816((e & 1) ? acc2 : acc, a0, a1, a2, a3, xw[2 * e], xw[2 * e + 1]);
              }
            } else {
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                uint32_t a0, a2, a1, a3;
                fp8x4_to_bf16x2<AT>(wa[e], a0, a2);
                fp8x4_to_bf16x2<AT>(wb[e], a1, a3);
                mma_bf16_16816((e & 1) ? acc2 : acc, a0, a1, a2, a3, xw[2 * e], xw[2 * e + 1]);
              }
            }
          }
        }
        __syncwarp();
        if (lane == 0) asm volatile("{ .reg .b64 st; mbarrier.arrive.shared::cta.b64 st, [%0]; }" ::"r"(empty_bar(s)) : "memory");
        if (++s == stages) { s = 0; ph ^= 1u; }
      }
      if (!ok) break;
      // the eight partial tiles meet in a fixed order; buffers alternate so that the next tile's partials do not
      // overwrite what the 128 reducing threads of this tile may still be reading
      const int buf = lt & 1;
      red[buf][warp][g][2 * t] = __fadd_rn(acc[0], acc2[0]);
      red[buf][warp][g][2 * t + 1] = __fadd_rn(acc[1], acc2[1]);
      red[buf][warp][g + 8][2 * t] = __fadd_rn(acc[2], acc2[2]);
      red[buf][warp][g + 8][2 * t + 1] = __fadd_rn(acc[3], acc2[3]);
      asm volatile("bar.sync 1, %0;" ::"n"(GV_WARPS * 32) : "memory");
      if (threadIdx.x < 128) {
        const int il = threadIdx.x & 15, j = threadIdx.x >> 4, i = tile * 16 + il;
        if (i < m && j < n) {
          float sum = red[buf][0][il][j];
#pragma unroll
          for (int w = 1; w < GV_WARPS; ++w) sum = __fadd_rn(sum, red[buf][w][il][j]);
          mx = fmaxf(mx, out_store(o, r, i, j, sum));
        }
      }
    }
  }
  if (o.amax) block_amax(o.amax, mx);
  else __syncthreads();
}

// ---- the cp.async ring with FP16 arithmetic ---------------------------------------------------------
// gemv_async_kernel is bound by its instruction stream, and half of that stream widens W to BF16 (two converter
// instructions and half a byte permute per pair of codes; with FP8 activations, whose widening comes on top, the
// same weights take 18.1 us instead of 15.9 us).  To FP16 the widening is one instruction per pair: E5M2 is the
// upper byte of an FP16, E4M3 has a hardware converter.  Products of an FP8 and an FP16 value are exact in the
// FP32 accumulator, the sums are the same FP32 sums, so the result does not change -- provided X is FP16.  FP8
// activations always convert exactly (on the fly, same single instruction per pair).  BF16 activations are
// converted once per block into shared memory behind the ring (n columns of k FP16 values; the launcher offers
// this kernel only when that fits) and every value is checked on the way: if one does not survive the round trip
// (|x| >= 65520, or bits below 2^-24), the block runs the BF16 arithmetic of gemv_async_kernel instead.  Both
// paths add the same exact products in the same order.
template <int GA_STAGES>
struct GaRing {
  uint8_t *my_ring;
  uint32_t my_ring_s;
  const uint8_t *wa, *wb;
  bool la, lb;
  int k, kmap, warp, per_warp, steps, t;
  __device__ __forceinline__ int kstart(int it) const { return (kmap ? warp * per_warp + it : warp + GV_WARPS * it) * 128; }
  __device__ __forceinline__ void issue(int it) const {
    if (it < steps) {
      const int kc = kstart(it) + t * 16;
      const uint32_t dst = my_ring_s + (uint32_t)(it % GA_STAGES) * 2048;
      const bool wide = kmap != 0;
      cp_async16(dst, wa + kc, la && kc < k, wide);
      cp_async16(dst + 512, wb + kc, lb && kc < k, wide);
      cp_async16(dst + 1024, wa + kc + 64, la && kc + 64 < k, wide);
      cp_async16(dst + 1536, wb + kc + 64, lb && kc + 64 < k, wide);
    }
    cp_async_commit();
  }
};

// MODE 0: BF16 arithmetic, X (XT) from global memory.  MODE 1: FP16 arithmetic, FP8 X from global memory.
// MODE 2: FP16 arithmetic, X as FP16 in shared memory (xcol then points there).
template <int AT, int XT, int GA_STAGES, int MODE>
__device__ __forceinline__ void ga_mainloop(const GaRing<GA_STAGES> &rg, const uint8_t *xcol, bool xlive, float (&acc)[4],
                                            float (&acc2)[4]) {
  constexpr int XB = MODE == 2 ? 2 : (XT == E5MA_BF16 ? 2 : 1);
  constexpr int XW = XB;                        // 16-byte loads of X per 16 elements
  const int k = rg.k, t = rg.t;
  const auto load_x = [&](int it, uint4 (&xq)[2][XW]) {
    const int kc = rg.kstart(it);
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int kk = kc + h * 64 + t * 16;
#pragma unroll
      for (int q = 0; q < XW; ++q) {
        const uint4 *src = reinterpret_cast<const uint4 *>(xcol + (size_t)kk * XB) + q;
        xq[h][q] = xlive && kk < k ? (MODE == 2 ? *src : __ldg(src)) : make_uint4(0, 0, 0, 0);
      }
    }
  };
  uint4 xq[2][XW], xn[2][XW];
  if (MODE != 2) load_x(0, xq);
  for (int it = 0; it < rg.steps; ++it) {
    rg.issue(it + GA_STAGES - 1);
    if (MODE != 2) load_x(it + 1, xn);   // X of the next step is fetched while this one is consumed (zeros beyond k)
    else load_x(it, xq);                 // shared memory: no need to look ahead
    cp_async_wait<GA_STAGES - 1>();
    const uint8_t *slot = rg.my_ring + (size_t)(it % GA_STAGES) * 2048;
    uint4 wq[2][2];
    wq[0][0] = *reinterpret_cast<const uint4 *>(slot);
    wq[0][1] = *reinterpret_cast<const uint4 *>(slot + 512);
    wq[1][0] = *reinterpret_cast<const uint4 *>(slot + 1024);
    wq[1][1] = *reinterpret_cast<const uint4 *>(slot + 1536);
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      uint32_t xw[8];
      if (XW == 2) {
        xw[0] = xq[h][0].x; xw[1] = xq[h][0].y; xw[2] = xq[h][0].z; xw[3] = xq[h][0].w;
        xw[4] = xq[h][XW - 1].x; xw[5] = xq[h][XW - 1].y; xw[6] = xq[h][XW - 1].z; xw[7] = xq[h][XW - 1].w;
      } else {
        const uint32_t q[4] = {xq[h][0].x, xq[h][0].y, xq[h][0].z, xq[h][0].w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          if (MODE == 0) fp8x4_to_bf16x2<XT == E5MA_BF16 ? E5MA_E5M2 : XT>(q[e], xw[2 * e], xw[2 * e + 1]);
          else fp8x4_to_f16x2<XT == E5MA_BF16 ? E5MA_E5M2 : XT>(q[e], xw[2 * e], xw[2 * e + 1]);
        }
      }
      const uint32_t qa[4] = {wq[h][0].x, wq[h][0].y, wq[h][0].z, wq[h][0].w};
      const uint32_t qb[4] = {wq[h][1].x, wq[h][1].y, wq[h][1].z, wq[h][1].w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        uint32_t a0, a2, a1, a3;
        if (MODE == 0) {
          fp8x4_to_bf16x2<AT>(qa[e], a0, a2);   // row g:   k pairs (0,1) and (2,3) of this word
          fp8x4_to_bf16x2<AT>(qb[e], a1, a3);   // row g+8
          mma_bf16_16816((e & 1) ? acc2 : acc, a0, a1, a2, a3, xw[2 * e], xw[2 * e + 1]);
        } else {
          fp8x4_to_f16x2<AT>(qa[e], a0, a2);
          fp8x4_to_f16x2<AT>(qb[e], a1, a3);
          mma_f16_16816((e & 1) ? acc2 : acc, a0, a1, a2, a3, xw[2 * e], xw[2 * e + 1]);
        }
      }
    }
    if (MODE != 2) {
#pragma unroll
      for (int h = 0; h < 2; ++h)
#pragma unroll
        for (int q = 0; q < XW; ++q) xq[h][q] = xn[h][q];
    }
  }
}

template <int AT, int XT, int GA_STAGES>
__global__ void __launch_bounds__(GV_WARPS * 32) gemv_async16_kernel(const uint8_t *__restrict__ W, int lda,
                                                                     const uint8_t *__restrict__ X, int ldx, int m, int n,
                                                                     int k, int kmap, int x_pitch, OutDesc o) {
  extern __shared__ __align__(16) uint8_t ring_raw[];        // the ring as in gemv_async_kernel, then (BF16 X) n x x_pitch bytes of FP16
  __shared__ float red[GV_WARPS][16][9];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;
  const int row0 = blockIdx.x * 16;
  GaRing<GA_STAGES> rg;
  rg.my_ring = ring_raw + (size_t)warp * GA_STAGES * 2048 + lane * 16;
  rg.my_ring_s = (uint32_t)__cvta_generic_to_shared(rg.my_ring);
  const int ra = row0 + g, rb = ra + 8;
  rg.la = ra < m;
  rg.lb = rb < m;
  rg.wa = W + (size_t)(rg.la ? ra : 0) * lda;
  rg.wb = W + (size_t)(rg.lb ? rb : 0) * lda;
  const int kblocks = (k + 127) / 128;
  rg.per_warp = (kblocks + GV_WARPS - 1) / GV_WARPS;
  rg.k = k; rg.kmap = kmap; rg.warp = warp; rg.t = t;
  rg.steps = kmap ? (kblocks - warp * rg.per_warp < rg.per_warp ? (kblocks > warp * rg.per_warp ? kblocks - warp * rg.per_warp : 0) : rg.per_warp)
                  : (k > warp * 128 ? (k - warp * 128 + GV_WARPS * 128 - 1) / (GV_WARPS * 128) : 0);
#pragma unroll
  for (int it = 0; it < GA_STAGES - 1; ++it) rg.issue(it);      // the weights are on their way while X is staged

  float acc[4] = {0.f, 0.f, 0.f, 0.f}, acc2[4] = {0.f, 0.f, 0.f, 0.f};
  const bool xlive = g < n;
  if (XT == E5MA_BF16) {
    uint8_t *xs = ring_raw + (size_t)GV_WARPS * GA_STAGES * 2048;
    const int per_col = k / 8;                        // k is a multiple of 16
    bool fits = true;
    for (int idx = threadIdx.x; idx < n * per_col; idx += GV_WARPS * 32) {
      const int j = idx / per_col, q = idx - j * per_col;
      const uint4 v = __ldg(reinterpret_cast<const uint4 *>(X + ((size_t)j * ldx + (size_t)q * 8) * 2));
      const uint32_t w[4] = {v.x, v.y, v.z, v.w};
      uint32_t h[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float lo = __uint_as_float(w[e] << 16), hi = __uint_as_float(w[e] & 0xFFFF0000u);
        const __half2 hh = __floats2half2_rn(lo, hi);
        const float2 back = __half22float2(hh);
        fits = fits && back.x == lo && back.y == hi;
        h[e] = *reinterpret_cast<const uint32_t *>(&hh);
      }
      *reinterpret_cast<uint4 *>(xs + (size_t)j * x_pitch + (size_t)q * 16) = make_uint4(h[0], h[1], h[2], h[3]);
    }
    if (__syncthreads_and(fits)) ga_mainloop<AT, XT, GA_STAGES, 2>(rg, xs + (size_t)g * x_pitch, xlive, acc, acc2);
    else ga_mainloop<AT, XT, GA_STAGES, 0>(rg, X + (size_t)g * ldx * 2, xlive, acc, acc2);
  } else {
    ga_mainloop<AT, XT, GA_STAGES, 1>(rg, X + (size_t)g * ldx, xlive, acc, acc2);
  }
#pragma unroll
  for (int e = 0; e < 4; ++e) acc[e] = __fadd_rn(acc[e], acc2[e]);
  cp_async_wait<0>();

  red[warp][g][2 * t] = acc[0];
  red[warp][g][2 * t + 1] = acc[1];
  red[warp][g + 8][2 * t] = acc[2];
  red[warp][g + 8][2 * t + 1] = acc[3];
  __syncthreads();
  const OutScalars r = out_begin(o);
  float mx = 0.f;
  if (threadIdx.x < 128) {
    const int il = threadIdx.x & 15, j = threadIdx.x >> 4, i = row0 + il;
    if (i < m && j < n) {
      float s = red[0][il][j];
#pragma unroll
      for (int w = 1; w < GV_WARPS; ++w) s = __fadd_rn(s, red[w][il][j]);
      mx = out_store(o, r, i, j, s);
    }
  }
  if (o.amax) block_amax(o.amax, mx);
}


// Shared memory of the persistent kernel for a given problem, and the stage count that fits (0: does not fit).
struct BulkPlan { int stages, x_pitch, smem; };
static BulkPlan gemv_bulk_plan(int n, int k) {
  BulkPlan p;
  p.x_pitch = (k * 2 + 127) / 128 * 128 + 16;
  const int fixed = n * p.x_pitch + 2 * GV_WARPS * 16 * 9 * 4 + 2 * GB_MAX_STAGES * 8 + 64;
  p.stages = (232448 - 1024 - fixed) / GB_STAGE_BYTES;
  if (p.stages > GB_MAX_STAGES) p.stages = GB_MAX_STAGES;
  if (p.stages < 3) p.stages = 0;
  p.smem = fixed + p.stages * GB_STAGE_BYTES;
  return p;
}

template <int AT>
static cudaError_t gemv_bulk_x(int x_dtype, const uint8_t *A, int lda, const uint8_t *X, int ldx, int m, int n, int k,
                               const OutDesc &o, int sms, const BulkPlan &p, cudaStream_t s) {
  const int tiles = (m + 15) / 16;
  const unsigned grid = (unsigned)(tiles < sms ? tiles : sms);
#define E5B_GEMV_BULK(XT)                                                                                     \
  {                                                                                                           \
    static SmemOptIn optin;                                                                                   \
    if (const cudaError_t e = optin.ensure(gemv_bulk_kernel<AT, XT>, 232448 - 1024)) return e;                \
    gemv_bulk_kernel<AT, XT><<<grid, GB_THREADS, p.smem, s>>>(A, lda, X, ldx, m, n, k, p.stages, p.x_pitch, o); \
  }
  switch (x_dtype) {
    case E5MA_BF16: E5B_GEMV_BULK(E5MA_BF16) break;
    case E5MA_E5M2: E5B_GEMV_BULK(E5MA_E5M2) break;
    case E5MA_E4M3: E5B_GEMV_BULK(E5MA_E4M3) break;
    default: return cudaErrorNotSupported;
  }
#undef E5B_GEMV_BULK
  return cudaGetLastError();
}

unsigned int gemv_fault_read_and_clear() {
  unsigned int v = 0, zero = 0;
  if (cudaMemcpyFromSymbol(&v, g_gemv_fault, sizeof v) != cudaSuccess) return 0xFFFFFFFFu;
  cudaMemcpyToSymbol(g_gemv_fault, &zero, sizeof zero);
  return v;
}

template <int AT, int S>
static cudaError_t gemv_rows_x(int x_dtype, const uint8_t *A, int lda, const uint8_t *X, int ldx, int m, int n, int k,
                               const OutDesc &o, cudaStream_t s) {
  constexpr int SMEM = S * GR_STAGE;
  const unsigned grid = (unsigned)((m + 15) / 16);
#define E5B_GEMV_ROWS(XT)                                                                                  \
  {                                                                                                        \
    static SmemOptIn optin;                                                                                \
    if (const cudaError_t e = optin.ensure(gemv_rows_kernel<AT, XT, S>, SMEM)) return e;                   \
    gemv_rows_kernel<AT, XT, S><<<grid, GV_WARPS * 32, SMEM, s>>>(A, lda, X, ldx, m, n, k, o);             \
  }
  switch (x_dtype) {
    case E5MA_BF16: E5B_GEMV_ROWS(E5MA_BF16) break;
    case E5MA_E5M2: E5B_GEMV_ROWS(E5MA_E5M2) break;
    case E5MA_E4M3: E5B_GEMV_ROWS(E5MA_E4M3) break;
    default: return cudaErrorNotSupported;
  }
#undef E5B_GEMV_ROWS
  return cudaGetLastError();
}

template <int AT, int GA_STAGES>
static cudaError_t gemv_async_x(int x_dtype, const uint8_t *A, int lda, const uint8_t *X, int ldx, int m, int n, int k,
                                const OutDesc &o, cudaStream_t s) {
  constexpr int GA_SMEM = GV_WARPS * GA_STAGES * 2048;
  const unsigned grid = (unsigned)((m + 15) / 16);
  const int kmap = (opt(OPT_GEMV_KMAP) >= 0 ? opt(OPT_GEMV_KMAP) : tuned_gemv(2)) > 0 ? 1 : 0;
  // FP16 arithmetic (switch GEMV_F16, on by default): FP8 activations always; BF16 activations when their FP16 copy
  // (n columns of k values, rows padded against bank conflicts) fits in 32 KiB beside the ring
  const int x_pitch = k * 2 + 16;
  const bool f16 = opt(OPT_GEMV_F16) != 0 && (x_dtype != E5MA_BF16 || (size_t)n * x_pitch <= 32768);
  if (f16) {
    const int smem = GA_SMEM + (x_dtype == E5MA_BF16 ? n * x_pitch : 0);
#define E5B_GEMV16_CASE(XT)                                                                                                 \
  {                                                                                                                         \
    static SmemOptIn optin;                                                                                                 \
    if (const cudaError_t e = optin.ensure(gemv_async16_kernel<AT, XT, GA_STAGES>, GA_SMEM + 32768)) return e;              \
    gemv_async16_kernel<AT, XT, GA_STAGES><<<grid, GV_WARPS * 32, smem, s>>>(A, lda, X, ldx, m, n, k, kmap, x_pitch, o);    \
  }
    switch (x_dtype) {
      case E5MA_BF16: E5B_GEMV16_CASE(E5MA_BF16) break;
      case E5MA_E5M2: E5B_GEMV16_CASE(E5MA_E5M2) break;
      case E5MA_E4M3: E5B_GEMV16_CASE(E5MA_E4M3) break;
      default: return cudaErrorNotSupported;
    }
#undef E5B_GEMV16_CASE
    return cudaGetLastError();
  }
#define E5B_GEMV_CASE(XT, slot_)                                                                                            \
  {                                                                                                                         \
    static SmemOptIn optin;                                                                                                 \
    if (const cudaError_t e = optin.ensure(gemv_async_kernel<AT, XT, GA_STAGES>, GA_SMEM)) return e;                        \
    gemv_async_kernel<AT, XT, GA_STAGES><<<grid, GV_WARPS * 32, GA_SMEM, s>>>(A, lda, X, ldx, m, n, k, kmap, o);                       \
  }
  switch (x_dtype) {
    case E5MA_BF16: E5B_GEMV_CASE(E5MA_BF16, 0) break;
    case E5MA_E5M2: E5B_GEMV_CASE(E5MA_E5M2, 1) break;
    case E5MA_E4M3: E5B_GEMV_CASE(E5MA_E4M3, 2) break;
    default: return cudaErrorNotSupported;
  }
#undef E5B_GEMV_CASE
  return cudaGetLastError();
}

template <int MT, int AT, int U>
static cudaError_t gemv_xu(int x_dtype, const uint8_t *A, int lda, const uint8_t *X, int ldx, int m, int n, int k,
                           const OutDesc &o, cudaStream_t s) {
  const unsigned grid = (unsigned)((m + MT * 16 - 1) / (MT * 16));
  switch (x_dtype) {
    case E5MA_BF16: gemv_mma_kernel<MT, AT, E5MA_BF16, U><<<grid, GV_WARPS * 32, 0, s>>>(A, lda, X, ldx, m, n, k, o); break;
    case E5MA_E5M2: gemv_mma_kernel<MT, AT, E5MA_E5M2, U><<<grid, GV_WARPS * 32, 0, s>>>(A, lda, X, ldx, m, n, k, o); break;
    case E5MA_E4M3: gemv_mma_kernel<MT, AT, E5MA_E4M3, U><<<grid, GV_WARPS * 32, 0, s>>>(A, lda, X, ldx, m, n, k, o); break;
    default: return cudaErrorNotSupported;
  }
  return cudaGetLastError();
}

// U = 2 k-steps in flight per warp when K is long enough to have them; E5MA_GEMV_U (experiments) overrides
template <int MT, int AT>
static cudaError_t gemv_x(int x_dtype, const uint8_t *A, int lda, const uint8_t *X, int ldx, int m, int n, int k,
                          const OutDesc &o, cudaStream_t s) {
  int u = 1;   // measured on B200: one k-step per warp in flight (more registers cost occupancy and lose)
  if (opt(OPT_GEMV_U) > 0) u = opt(OPT_GEMV_U);
  if (u >= 4 && MT == 1) return gemv_xu<MT, AT, MT == 1 ? 4 : 2>(x_dtype, A, lda, X, ldx, m, n, k, o, s);
  if (u >= 2) return gemv_xu<MT, AT, 2>(x_dtype, A, lda, X, ldx, m, n, k, o, s);
  return gemv_xu<MT, AT, 1>(x_dtype, A, lda, X, ldx, m, n, k, o, s);
}

// Rows per block: 16 keeps more blocks in flight (m / 16 of them); 32 halves how often X is
// re-read from L2, which matters once X is no longer tiny next to a block's share of W.
cudaError_t launch_gemv_mma(int a_dtype, int x_dtype, const uint8_t *A, int lda, const uint8_t *X, int ldx,
                            int m, int n, int k, const OutDesc &o, int sms, cudaStream_t s) {
  // Measured on B200 (8192 x 8192 weights, batch 1 / 8): the cp.async pipeline with X prefetched one step
  // ahead takes 15.2 / 15.8 us, the register-load kernel 15.8 / 16.6 us.  the GEMV_KERNEL switch = 0
  // (experiments) selects the latter.
  // Persistent bulk-copy kernel: only on request (switch GEMV_KERNEL = 2) and when X fits beside a ring of at
  // least three stages.  Measured on B200 (8192 x 8192 weights): 24 us against 15.6 us for the cp.async kernel --
  // bulk copies keep too few bytes in flight per SM, whatever their size.
  // FP32 activations always, other activations up to the tuned batch size (switch GEMV_FMA_MAXN): the FP32-pipe kernel
  // (a request for a particular tensor-core kernel, switch GEMV_KERNEL, keeps them off it unless GEMV_FMA_MAXN is set too)
  const int fma_maxn = opt(OPT_GEMV_FMA_MAXN) >= 0 ? opt(OPT_GEMV_FMA_MAXN) : (opt(OPT_GEMV_KERNEL) >= 0 ? 0 : tuned_gemv(3));
  if (x_dtype == E5MA_FP32 || n <= (fma_maxn < 4 ? fma_maxn : 4)) {
    note_route(ROUTE_GEMV_FMA);
    if (a_dtype == E5MA_E5M2) return gemv_fma<E5MA_E5M2>(x_dtype, A, lda, X, ldx, m, n, k, o, s);
    if (a_dtype == E5MA_E4M3) return gemv_fma<E5MA_E4M3>(x_dtype, A, lda, X, ldx, m, n, k, o, s);
    return cudaErrorNotSupported;
  }
  const int which = opt(OPT_GEMV_KERNEL) >= 0 ? opt(OPT_GEMV_KERNEL) : tuned_gemv(0);
  const BulkPlan bp = gemv_bulk_plan(n, k);
  if (bp.stages && which == 2) {
    note_route(ROUTE_GEMV_PERSISTENT);
    if (a_dtype == E5MA_E5M2) return gemv_bulk_x<E5MA_E5M2>(x_dtype, A, lda, X, ldx, m, n, k, o, sms, bp, s);
    if (a_dtype == E5MA_E4M3) return gemv_bulk_x<E5MA_E4M3>(x_dtype, A, lda, X, ldx, m, n, k, o, sms, bp, s);
    return cudaErrorNotSupported;
  }
  note_route(ROUTE_GEMV);
  if (which == 3) {     // row streams: ring depth 3 or 4
    note_route(ROUTE_GEMV_ROWS);
    const int depth = (opt(OPT_GEMV_STAGES) > 0 ? opt(OPT_GEMV_STAGES) : tuned_gemv(1)) == 3 ? 3 : 4;
    if (a_dtype == E5MA_E5M2)
      return depth == 3 ? gemv_rows_x<E5MA_E5M2, 3>(x_dtype, A, lda, X, ldx, m, n, k, o, s) : gemv_rows_x<E5MA_E5M2, 4>(x_dtype, A, lda, X, ldx, m, n, k, o, s);
    if (a_dtype == E5MA_E4M3)
      return depth == 3 ? gemv_rows_x<E5MA_E4M3, 3>(x_dtype, A, lda, X, ldx, m, n, k, o, s) : gemv_rows_x<E5MA_E4M3, 4>(x_dtype, A, lda, X, ldx, m, n, k, o, s);
    return cudaErrorNotSupported;
  }
  const bool use_async = which != 0;
  if (use_async) {
    int stages = tuned_gemv(1);   // 2 = 32 KiB per block: every row tile of an 8192-row matrix is resident in one wave
    if (opt(OPT_GEMV_STAGES) > 0) stages = opt(OPT_GEMV_STAGES);
    if (a_dtype == E5MA_E5M2)
      return stages == 2 ? gemv_async_x<E5MA_E5M2, 2>(x_dtype, A, lda, X, ldx, m, n, k, o, s)
           : stages == 4 ? gemv_async_x<E5MA_E5M2, 4>(x_dtype, A, lda, X, ldx, m, n, k, o, s)
                         : gemv_async_x<E5MA_E5M2, 3>(x_dtype, A, lda, X, ldx, m, n, k, o, s);
    if (a_dtype == E5MA_E4M3)
      return stages == 2 ? gemv_async_x<E5MA_E4M3, 2>(x_dtype, A, lda, X, ldx, m, n, k, o, s)
           : stages == 4 ? gemv_async_x<E5MA_E4M3, 4>(x_dtype, A, lda, X, ldx, m, n, k, o, s)
                         : gemv_async_x<E5MA_E4M3, 3>(x_dtype, A, lda, X, ldx, m, n, k, o, s);
    return cudaErrorNotSupported;
  }
  bool wide = false;   // measured on B200: 16 rows per block wins for every n <= 8 (more blocks, fewer registers)
  (void)sms;
  wide = opt(OPT_GEMV_MT) == 2;   // experiments
  if (a_dtype == E5MA_E5M2)
    return wide ? gemv_x<2, E5MA_E5M2>(x_dtype, A, lda, X, ldx, m, n, k, o, s)
                : gemv_x<1, E5MA_E5M2>(x_dtype, A, lda, X, ldx, m, n, k, o, s);
  if (a_dtype == E5MA_E4M3)
    return wide ? gemv_x<2, E5MA_E4M3>(x_dtype, A, lda, X, ldx, m, n, k, o, s)
                : gemv_x<1, E5MA_E4M3>(x_dtype, A, lda, X, ldx, m, n, k, o, s);
  return cudaErrorNotSupported;
}

}  // namespace e5b
