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
//     instruction stream and the FP32 pipe stays free; products are exact, sums are FP32;
//   * the reduction over K may visit k in any order as long as W and X agree, so a lane's 16
//     contiguous bytes feed four consecutive MMAs without any shuffling;
//   * the 8 per-warp partial tiles meet in shared memory in a fixed order (deterministic), then one
//     thread per output runs the common epilogue and the block issues one amax atomic.
#include "common.cuh"

namespace e5b {

__device__ __forceinline__ uint4 ld_stream16(const void *p) {
  uint4 r;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(p));
  return r;
}

__device__ __forceinline__ uint32_t mul_bf16x2(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}

// Four FP8 codes (bytes 0..3 of w, ascending k) -> BF16 pairs (k0,k1) and (k2,k3).
// The 7 magnitude bits of a code, placed so that its exponent field lands in the BF16 exponent
// field, are the BF16 encoding of value * 2^-112 (E5M2, bias 15 -> 127) or value * 2^-120 (E4M3,
// bias 7 -> 127), subnormal codes included; one BF16 multiply by the power of two restores the value.
template <int T>
__device__ __forceinline__ void fp8x4_to_bf16x2(uint32_t w, uint32_t &lo, uint32_t &hi) {
  const uint32_t p0 = __byte_perm(w, 0, 0x1404);   // (b1 << 24) | (b0 << 8)
  const uint32_t p1 = __byte_perm(w, 0, 0x3424);   // (b3 << 24) | (b2 << 8)
  if (T == E5MA_E5M2) {
    const uint32_t k = 0x77807780u;                // 2^112 in both halves
    lo = mul_bf16x2((p0 & 0x80008000u) | ((p0 >> 3) & 0x0FE00FE0u), k);
    hi = mul_bf16x2((p1 & 0x80008000u) | ((p1 >> 3) & 0x0FE00FE0u), k);
  } else {
    const uint32_t k = 0x7B807B80u;                // 2^120 in both halves
    lo = mul_bf16x2((p0 & 0x80008000u) | ((p0 >> 4) & 0x07F007F0u), k);
    hi = mul_bf16x2((p1 & 0x80008000u) | ((p1 >> 4) & 0x07F007F0u), k);
  }
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
template <int MT, int AT, int XT>
__global__ void __launch_bounds__(GV_WARPS * 32) gemv_mma_kernel(const uint8_t *__restrict__ W, int lda,
                                                                 const uint8_t *__restrict__ X, int ldx, int m, int n,
                                                                 int k, OutDesc o) {
  __shared__ float red[GV_WARPS][MT * 16][9];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;
  const int row0 = blockIdx.x * (MT * 16);
  constexpr int XB = XT == E5MA_BF16 ? 2 : 1;

  float acc[MT][4];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int e = 0; e < 4; ++e) acc[mt][e] = 0.f;

  const uint8_t *xcol = X + (size_t)g * ldx * XB;
  const bool xlive = g < n;

  // A warp's step covers bytes [kc, kc + 128) of every row; this lane owns 16 bytes in each half.
  // The trip count must be the same for all lanes of the warp (mma.sync is warp-collective), so the
  // loop runs on the warp-uniform kc and the per-lane offset only enters the load predicates.
#pragma unroll 2
  for (int kc = warp * 128; kc < k; kc += GV_WARPS * 128) {
    const int kb = kc + t * 16;
    uint4 wa[MT][2], wb[MT][2];
    uint32_t xw[2][8];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int kk = kb + h * 64;
      const bool kin = kk < k;
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        const int ra = row0 + mt * 16 + g, rb = ra + 8;
        wa[mt][h] = kin && ra < m ? ld_stream16(W + (size_t)ra * lda + kk) : make_uint4(0, 0, 0, 0);
        wb[mt][h] = kin && rb < m ? ld_stream16(W + (size_t)rb * lda + kk) : make_uint4(0, 0, 0, 0);
      }
      if (XT == E5MA_BF16) {
        uint4 x0 = make_uint4(0, 0, 0, 0), x1 = x0;
        if (kin && xlive) {
          const uint4 *xp = reinterpret_cast<const uint4 *>(xcol + (size_t)kk * 2);
          x0 = __ldg(xp); x1 = __ldg(xp + 1);
        }
        xw[h][0] = x0.x; xw[h][1] = x0.y; xw[h][2] = x0.z; xw[h][3] = x0.w;
        xw[h][4] = x1.x; xw[h][5] = x1.y; xw[h][6] = x1.z; xw[h][7] = x1.w;
      } else {
        uint4 x0 = make_uint4(0, 0, 0, 0);
        if (kin && xlive) x0 = __ldg(reinterpret_cast<const uint4 *>(xcol + kk));
        const uint32_t q[4] = {x0.x, x0.y, x0.z, x0.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) fp8x4_to_bf16x2<XT == E5MA_BF16 ? E5MA_E5M2 : XT>(q[e], xw[h][2 * e], xw[h][2 * e + 1]);
      }
    }
#pragma unroll
    for (int h = 0; h < 2; ++h)
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        const uint32_t qa[4] = {wa[mt][h].x, wa[mt][h].y, wa[mt][h].z, wa[mt][h].w};
        const uint32_t qb[4] = {wb[mt][h].x, wb[mt][h].y, wb[mt][h].z, wb[mt][h].w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          uint32_t a0, a2, a1, a3;
          fp8x4_to_bf16x2<AT>(qa[e], a0, a2);   // row g:   k pairs (0,1) and (2,3) of this word
          fp8x4_to_bf16x2<AT>(qb[e], a1, a3);   // row g+8
          mma_bf16_16816(acc[mt], a0, a1, a2, a3, xw[h][2 * e], xw[h][2 * e + 1]);
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

template <int MT, int AT>
static cudaError_t gemv_x(int x_dtype, const uint8_t *A, int lda, const uint8_t *X, int ldx, int m, int n, int k,
                          const OutDesc &o, cudaStream_t s) {
  const unsigned grid = (unsigned)((m + MT * 16 - 1) / (MT * 16));
  switch (x_dtype) {
    case E5MA_BF16: gemv_mma_kernel<MT, AT, E5MA_BF16><<<grid, GV_WARPS * 32, 0, s>>>(A, lda, X, ldx, m, n, k, o); break;
    case E5MA_E5M2: gemv_mma_kernel<MT, AT, E5MA_E5M2><<<grid, GV_WARPS * 32, 0, s>>>(A, lda, X, ldx, m, n, k, o); break;
    case E5MA_E4M3: gemv_mma_kernel<MT, AT, E5MA_E4M3><<<grid, GV_WARPS * 32, 0, s>>>(A, lda, X, ldx, m, n, k, o); break;
    default: return cudaErrorNotSupported;
  }
  return cudaGetLastError();
}

// Rows per block: 16 keeps more blocks in flight (m / 16 of them); 32 halves how often X is
// re-read from L2, which matters once X is no longer tiny next to a block's share of W.
cudaError_t launch_gemv_mma(int a_dtype, int x_dtype, const uint8_t *A, int lda, const uint8_t *X, int ldx,
                            int m, int n, int k, const OutDesc &o, int sms, cudaStream_t s) {
  const bool wide = n > 2 && m >= sms * 32;
  if (a_dtype == E5MA_E5M2)
    return wide ? gemv_x<2, E5MA_E5M2>(x_dtype, A, lda, X, ldx, m, n, k, o, s)
                : gemv_x<1, E5MA_E5M2>(x_dtype, A, lda, X, ldx, m, n, k, o, s);
  if (a_dtype == E5MA_E4M3)
    return wide ? gemv_x<2, E5MA_E4M3>(x_dtype, A, lda, X, ldx, m, n, k, o, s)
                : gemv_x<1, E5MA_E4M3>(x_dtype, A, lda, X, ldx, m, n, k, o, s);
  return cudaErrorNotSupported;
}

}  // namespace e5b
