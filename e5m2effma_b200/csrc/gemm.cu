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

// ---- CUDA-core GEMM: 128 x 128 output tile, 16-deep k slices, 8 x 8 outputs per thread -----------
// The classic register-tiled FP32 GEMM (what the reference's gemm_kernel is, src/gemm_e5m2effma.cuh:117-233): 256
// threads, every thread owns two groups of four rows and two groups of four columns of the tile (so that its
// shared-memory reads are 16-byte vectors without bank conflicts) and performs 64 FMAs per four such reads.  The
// next k slice is fetched into registers (eight elements of each operand per thread, one vector load along the
// operand's contiguous direction, decoded to FP32) while the current one is being multiplied.  Every output is one
// FMA chain in ascending k starting from zero: bit-identical to the host emulation, whatever the tile shape.
constexpr int ST = 128, SK = 16, SP = ST + 4;

// eight consecutive elements of an operand of dtype t starting at element idx (a multiple of 8) -> FP32, exact
__device__ __forceinline__ void load8_f32(int t, const uint8_t *p, size_t idx, float v[8]) {
  if (t == E5MA_FP32) {
    const float4 a = __ldg(reinterpret_cast<const float4 *>(p + idx * 4)), b = __ldg(reinterpret_cast<const float4 *>(p + idx * 4) + 1);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
  } else if (t == E5MA_BF16) {
    const uint4 q = __ldg(reinterpret_cast<const uint4 *>(p + idx * 2));
    const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int e = 0; e < 4; ++e) { v[2 * e] = __uint_as_float(w[e] << 16); v[2 * e + 1] = __uint_as_float(w[e] & 0xFFFF0000u); }
  } else {
    const uint2 q = __ldg(reinterpret_cast<const uint2 *>(p + idx));
    if (t == E5MA_E5M2) { fp8x4_to_f32<E5MA_E5M2>(q.x, v); fp8x4_to_f32<E5MA_E5M2>(q.y, v + 4); }
    else { fp8x4_to_f32<E5MA_E4M3>(q.x, v); fp8x4_to_f32<E5MA_E4M3>(q.y, v + 4); }
  }
}

// This thread's eight elements of the k slice starting at k0 of an operand whose tile starts at row r0 (rows: m / n
// index, `rows` of them in all).  K-contiguous storage: row r0 + (t & 127), k0 + 8 (t >> 7) .. + 8.  Otherwise: k row
// k0 + (t >> 4), rows r0 + 8 (t & 15) .. + 8.  Rows beyond the operand read as zero.
__device__ __forceinline__ void fetch8(int dt, const uint8_t *p, bool kc, int ld, int r0, int rows, int k0, int t, float v[8]) {
  if (kc) {
    const int r = r0 + (t & 127);
    if (r < rows) load8_f32(dt, p, (size_t)r * ld + k0 + 8 * (t >> 7), v);
    else
#pragma unroll
      for (int e = 0; e < 8; ++e) v[e] = 0.f;
  } else {
    const int r = r0 + 8 * (t & 15);
    const size_t base = (size_t)(k0 + (t >> 4)) * ld + r;
    if (r + 8 <= rows) load8_f32(dt, p, base, v);
    else
#pragma unroll
      for (int e = 0; e < 8; ++e) v[e] = r + e < rows ? load_elem(dt, p, base + e, 1.f) : 0.f;
  }
}
__device__ __forceinline__ void stash8(float (*S)[SP], bool kc, int t, const float v[8]) {
  if (kc) {
#pragma unroll
    for (int e = 0; e < 8; ++e) S[8 * (t >> 7) + e][t & 127] = v[e];
  } else {
    float *dst = &S[t >> 4][8 * (t & 15)];
    *reinterpret_cast<float4 *>(dst) = make_float4(v[0], v[1], v[2], v[3]);
    *reinterpret_cast<float4 *>(dst + 4) = make_float4(v[4], v[5], v[6], v[7]);
  }
}

__global__ void __launch_bounds__(256, 2) gemm_simt_kernel(int ta, int tb, bool a_kc, bool b_kc,
                                                           const uint8_t *__restrict__ A, int lda,
                                                           const uint8_t *__restrict__ B, int ldb, int m, int n, int k,
                                                           OutDesc o) {
  __shared__ __align__(16) float As[SK][SP], Bs[SK][SP];
  const int t = threadIdx.x, tx = t & 15, ty = t >> 4;
  const int i0 = blockIdx.y * ST, j0 = blockIdx.x * ST;
  float acc[8][8];
#pragma unroll
  for (int x = 0; x < 8; ++x)
#pragma unroll
    for (int y = 0; y < 8; ++y) acc[x][y] = 0.f;

  float pa[8], pb[8];
  if (k > 0) { fetch8(ta, A, a_kc, lda, i0, m, 0, t, pa); fetch8(tb, B, b_kc, ldb, j0, n, 0, t, pb); }
  for (int k0 = 0; k0 < k; k0 += SK) {
    stash8(As, a_kc, t, pa);
    stash8(Bs, b_kc, t, pb);
    __syncthreads();
    if (k0 + SK < k) { fetch8(ta, A, a_kc, lda, i0, m, k0 + SK, t, pa); fetch8(tb, B, b_kc, ldb, j0, n, k0 + SK, t, pb); }
#pragma unroll
    for (int kk = 0; kk < SK; ++kk) {
      const float4 a0 = *reinterpret_cast<const float4 *>(&As[kk][tx * 4]), a1 = *reinterpret_cast<const float4 *>(&As[kk][64 + tx * 4]);
      const float4 b0 = *reinterpret_cast<const float4 *>(&Bs[kk][ty * 4]), b1 = *reinterpret_cast<const float4 *>(&Bs[kk][64 + ty * 4]);
      const float a[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w}, b[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
      for (int x = 0; x < 8; ++x)
#pragma unroll
        for (int y = 0; y < 8; ++y) acc[x][y] = __fmaf_rn(a[x], b[y], acc[x][y]);
    }
    __syncthreads();
  }

  const OutScalars r = out_begin(o);
  float mx = 0.f;
#pragma unroll
  for (int y = 0; y < 8; ++y)
#pragma unroll
    for (int x = 0; x < 8; ++x) {
      const int i = i0 + (x < 4 ? tx * 4 + x : 64 + tx * 4 + x - 4), j = j0 + (y < 4 ? ty * 4 + y : 64 + ty * 4 + y - 4);
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
