// e5ma_gemm: argument validation, output description, and the choice between the three kernels:
//   * the streaming GEMV kernels         (n <= 8, both operands K-contiguous, FP8 A, any x dtype; gemv.cu)
//   * the tcgen05 tensor-core kernel      (FP8 / BF16 operand pairs; gemm_tc.cu)
//   * the CUDA-core kernel in this file   (FP32 operands and every shape the others decline)
//
// Validation order, status codes and the meaning of every argument follow reference
// src/gemm_e5m2effma.cu:44-104; the GEMV routing rule is its line 100-102.  The CUDA-core kernel
// accumulates with one FP32 FMA per product in ascending k, the order the reference documents
// (include/e5m2effma.h:27-28), so its results match the host emulation bit for bit.
#include <stdlib.h>
#include "common.cuh"

namespace e5b {

// ---- CUDA-core GEMM: 64 x 64 output tile, 16-deep k slices, 4 x 4 outputs per thread ------------
constexpr int ST = 64, SK = 16;

// element (r, kk) of an operand whose r index is the outer one: K-contiguous storage puts it at
// r * ld + kk, otherwise at kk * ld + r
__device__ __forceinline__ float operand_at(int t, const uint8_t *p, bool kc, int ld, int r, int kk) {
  const size_t idx = kc ? (size_t)r * ld + kk : (size_t)kk * ld + r;
  return load_elem(t, p, idx, 1.f);
}

__global__ void __launch_bounds__(256) gemm_simt_kernel(int ta, int tb, bool a_kc, bool b_kc,
                                                        const uint8_t *__restrict__ A, int lda,
                                                        const uint8_t *__restrict__ B, int ldb, int m, int n, int k,
                                                        OutDesc o) {
  __shared__ __align__(16) float As[SK][ST + 4], Bs[SK][ST + 4];
  const int t = threadIdx.x, tx = t & 15, ty = t >> 4;
  const int i0 = blockIdx.y * ST, j0 = blockIdx.x * ST;
  float acc[4][4];
#pragma unroll
  for (int a = 0; a < 4; ++a)
#pragma unroll
    for (int b = 0; b < 4; ++b) acc[a][b] = 0.f;

  for (int k0 = 0; k0 < k; k0 += SK) {
    // 1024 elements per operand tile, 4 per thread, walking along the contiguous storage direction
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int ra = a_kc ? t >> 2 : (t & 15) * 4 + e, ka = a_kc ? (t & 3) * 4 + e : t >> 4;
      As[ka][ra] = i0 + ra < m ? operand_at(ta, A, a_kc, lda, i0 + ra, k0 + ka) : 0.f;
      const int rb = b_kc ? t >> 2 : (t & 15) * 4 + e, kb = b_kc ? (t & 3) * 4 + e : t >> 4;
      Bs[kb][rb] = j0 + rb < n ? operand_at(tb, B, b_kc, ldb, j0 + rb, k0 + kb) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < SK; ++kk) {
      const float4 av = *reinterpret_cast<const float4 *>(&As[kk][tx * 4]);
      const float4 bv = *reinterpret_cast<const float4 *>(&Bs[kk][ty * 4]);
      const float a[4] = {av.x, av.y, av.z, av.w}, b[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
      for (int x = 0; x < 4; ++x)
#pragma unroll
        for (int y = 0; y < 4; ++y) acc[x][y] = __fmaf_rn(a[x], b[y], acc[x][y]);
    }
    __syncthreads();
  }

  const OutScalars r = out_begin(o);
  float mx = 0.f;
#pragma unroll
  for (int y = 0; y < 4; ++y)
#pragma unroll
    for (int x = 0; x < 4; ++x) {
      const int i = i0 + tx * 4 + x, j = j0 + ty * 4 + y;
      if (i < m && j < n) mx = fmaxf(mx, out_store(o, r, i, j, acc[x][y]));
    }
  if (o.amax) block_amax(o.amax, mx);
}

cudaError_t launch_gemm_simt(int a_dtype, int b_dtype, bool a_kc, bool b_kc, const uint8_t *A, int lda,
                             const uint8_t *B, int ldb, int m, int n, int k, const OutDesc &o, cudaStream_t s) {
  const dim3 grid((n + ST - 1) / ST, (m + ST - 1) / ST);
  if (grid.y > 65535u) return cudaErrorInvalidConfiguration;
  gemm_simt_kernel<<<grid, 256, 0, s>>>(a_dtype, b_dtype, a_kc, b_kc, A, lda, B, ldb, m, n, k, o);
  return cudaGetLastError();
}

}  // namespace e5b

namespace e5b {
static e5ma_status gemm_impl(e5ma_op transa, e5ma_op transb, int m, int n, int k, float alpha, const e5ma_tensor *A, int lda,
                             const e5ma_tensor *B, int ldb, float beta, const e5ma_tensor *C, int ldc, const e5ma_tensor *D,
                             int ldd, const e5ma_tensor *bias, int num_peers, void *const *peer_d, cudaStream_t stream) {
  clear_error();
  const auto known = [](const e5ma_tensor *t) { return t->dtype >= E5MA_E4M3 && t->dtype <= E5MA_E5M2; };
  const auto operand_type = [](int t) { return is_fp8(t) || t == E5MA_BF16 || t == E5MA_FP32; };
  const auto op_known = [](e5ma_op x) { return x == E5MA_OP_N || x == E5MA_OP_T; };
  if (!A || !B || !D || !A->data || !B->data || !D->data)
    return fail(E5MA_INVALID_VALUE, "e5ma_gemm: A, B, D or their data is NULL");
  if (!op_known(transa) || !op_known(transb))
    return fail(E5MA_INVALID_VALUE, "e5ma_gemm: transa / transb must be E5MA_OP_N or E5MA_OP_T");
  if (m < 0 || n < 0 || k < 0) return fail(E5MA_INVALID_VALUE, "e5ma_gemm: negative size (m=%d n=%d k=%d)", m, n, k);
  if (!known(D)) return fail(E5MA_INVALID_VALUE, "e5ma_gemm: invalid D dtype %d", (int)D->dtype);
  if (!operand_type(A->dtype) || !operand_type(B->dtype))
    return fail(E5MA_NOT_SUPPORTED, "e5ma_gemm: A and B must be E5M2, E4M3, BF16 or FP32 (got dtypes %d, %d)",
                (int)A->dtype, (int)B->dtype);
  if (m == 0 || n == 0) return E5MA_OK;
  if (k % 16) return fail(E5MA_INVALID_VALUE, "e5ma_gemm: k = %d is not a multiple of 16", k);
  if (lda % 16 || ldb % 16)
    return fail(E5MA_INVALID_VALUE, "e5ma_gemm: lda = %d / ldb = %d must be multiples of 16", lda, ldb);
  if ((((uintptr_t)A->data) | ((uintptr_t)B->data)) & 15u)
    return fail(E5MA_INVALID_VALUE, "e5ma_gemm: A and B must be 16-byte aligned");
  const bool a_kc = transa == E5MA_OP_T, b_kc = transb == E5MA_OP_N;
  if (lda < (a_kc ? k : m)) return fail(E5MA_INVALID_VALUE, "e5ma_gemm: lda = %d < %d", lda, a_kc ? k : m);
  if (ldb < (b_kc ? k : n)) return fail(E5MA_INVALID_VALUE, "e5ma_gemm: ldb = %d < %d", ldb, b_kc ? k : n);
  if (ldd < m) return fail(E5MA_INVALID_VALUE, "e5ma_gemm: ldd = %d < m = %d", ldd, m);
  const bool has_bias = bias && bias->data;
  const bool c_given = beta != 0.f && C && C->data;
  if (has_bias && !known(bias)) return fail(E5MA_INVALID_VALUE, "e5ma_gemm: invalid bias dtype %d", (int)bias->dtype);
  if (c_given && !known(C)) return fail(E5MA_INVALID_VALUE, "e5ma_gemm: invalid C dtype %d", (int)C->dtype);
  if (c_given && ldc < m) return fail(E5MA_INVALID_VALUE, "e5ma_gemm: ldc = %d < m = %d", ldc, m);
  for (const e5ma_tensor *t : {A, B})
    if (t->scaling != E5MA_SCALING_TENSOR && t->scaling != E5MA_SCALING_OUTER)
      return fail(E5MA_INVALID_VALUE, "e5ma_gemm: invalid scaling of A or B");
  for (const e5ma_tensor *t : {A, B})
    if (t->scaling == E5MA_SCALING_OUTER && (!is_fp8(t->dtype) || !t->scale_inv))
      return fail(E5MA_INVALID_VALUE, "e5ma_gemm: E5MA_SCALING_OUTER needs an FP8 operand with a scale_inv vector");
  for (const e5ma_tensor *t : {C, D, bias})
    if (t && t->scaling != E5MA_SCALING_TENSOR)
      return fail(E5MA_INVALID_VALUE, "e5ma_gemm: C, D and bias take per-tensor scaling only");
  DeviceProps dp;
  if (e5ma_status st = require_blackwell("e5ma_gemm", &dp)) return st;

  // beta != 0 without a C tensor accumulates into D (its dtype, leading dimension and scale_inv)
  const bool accumulate = beta != 0.f && !c_given;
  const e5ma_tensor *Cx = accumulate ? D : C;
  OutDesc o;
  o.sa = is_fp8(A->dtype) ? A->scale_inv : nullptr;
  o.sb = is_fp8(B->dtype) ? B->scale_inv : nullptr;
  o.sa_vec = A->scaling == E5MA_SCALING_OUTER;
  o.sb_vec = B->scaling == E5MA_SCALING_OUTER;
  o.alpha = alpha; o.beta = beta;
  o.c = beta != 0.f ? Cx->data : nullptr;
  o.ldc = beta != 0.f ? (accumulate ? ldd : ldc) : 0;
  o.c_dtype = beta != 0.f ? (int)Cx->dtype : E5MA_FP32;
  o.c_sinv = beta != 0.f && is_fp8(Cx->dtype) ? Cx->scale_inv : nullptr;
  o.d = D->data; o.ldd = ldd; o.d_dtype = D->dtype;
  o.d_scale = is_fp8(D->dtype) ? D->scale : nullptr;
  o.amax = D->amax;
  o.bias = has_bias ? bias->data : nullptr;
  o.bias_dtype = has_bias ? (int)bias->dtype : E5MA_FP32;
  o.npeers = num_peers;
  for (int p = 0; p < MAX_PEERS; ++p) o.peer[p] = p < num_peers ? peer_d[p] : nullptr;

  const uint8_t *a = (const uint8_t *)A->data, *b = (const uint8_t *)B->data;
  cudaError_t err = cudaErrorNotSupported;
  // switch FORCE_SIMT (experiments and tests): every problem takes the ascending-k CUDA-core kernel
  note_route(ROUTE_NONE);
  if (opt(OPT_FORCE_SIMT) == 1) { /* keep err: falls through to the CUDA-core kernel */ }
  else if (n <= 8 && a_kc && b_kc && is_fp8(A->dtype) && k > 0)
    err = launch_gemv_mma(A->dtype, B->dtype, a, lda, b, ldb, m, n, k, o, dp.sms, stream);
  else if (A->dtype != E5MA_FP32 && B->dtype != E5MA_FP32 && k > 0)
    err = launch_gemm_tc(A->dtype, B->dtype, a_kc, b_kc, a, lda, b, ldb, m, n, k, o, dp.sms, stream);
  if (err == cudaErrorNotSupported) {
    note_route(ROUTE_SIMT);
    err = launch_gemm_simt(A->dtype, B->dtype, a_kc, b_kc, a, lda, b, ldb, m, n, k, o, stream);
  }
  return cuda_fail(err, "e5ma_gemm: kernel launch");
}
}  // namespace e5b

extern "C" e5ma_status e5ma_gemm(e5ma_op transa, e5ma_op transb, int m, int n, int k, float alpha,
                                 const e5ma_tensor *A, int lda, const e5ma_tensor *B, int ldb, float beta,
                                 const e5ma_tensor *C, int ldc, const e5ma_tensor *D, int ldd,
                                 const e5ma_tensor *bias, cudaStream_t stream) {
  return e5b::gemm_impl(transa, transb, m, n, k, alpha, A, lda, B, ldb, beta, C, ldc, D, ldd, bias, 0, nullptr, stream);
}

// e5ma_gemm whose epilogue also stores every output into other GPUs' copies of D (declared in
// include/e5m2effma_b200.h).  Argument checks of its own first, then those of e5ma_gemm in their usual order.
extern "C" e5ma_status e5b_gemm_bcast(e5ma_op transa, e5ma_op transb, int m, int n, int k, float alpha,
                                      const e5ma_tensor *A, int lda, const e5ma_tensor *B, int ldb, float beta,
                                      const e5ma_tensor *C, int ldc, const e5ma_tensor *D, int ldd,
                                      const e5ma_tensor *bias, int num_peers, void *const *peer_d, cudaStream_t stream) {
  using namespace e5b;
  clear_error();
  if (num_peers < 0 || num_peers > MAX_PEERS)
    return fail(E5MA_INVALID_VALUE, "e5b_gemm_bcast: num_peers = %d, must be 0..%d", num_peers, MAX_PEERS);
  if (num_peers > 0 && !peer_d) return fail(E5MA_INVALID_VALUE, "e5b_gemm_bcast: peer_d is NULL");
  for (int p = 0; p < num_peers; ++p) {
    if (!peer_d[p]) return fail(E5MA_INVALID_VALUE, "e5b_gemm_bcast: peer_d[%d] is NULL", p);
    if (D && D->data && (((uintptr_t)peer_d[p] ^ (uintptr_t)D->data) & 15u))
      return fail(E5MA_INVALID_VALUE, "e5b_gemm_bcast: peer_d[%d] must have the alignment of D (mod 16 bytes)", p);
  }
  return gemm_impl(transa, transb, m, n, k, alpha, A, lda, B, ldb, beta, C, ldc, D, ldd, bias, num_peers, peer_d, stream);
}
