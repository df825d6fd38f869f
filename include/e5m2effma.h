/* e5m2effma.h -- C interface of the B200 (sm_100a) implementation of the E5M2EffMA hot path.
 *
 * Binary-compatible with the interface of srose69/e5m2effma (its include/e5m2effma.h): the same
 * five entry points, enumerator values and structure layouts (sizeof(e5ma_tensor) == 48,
 * sizeof(e5ma_adam_config) == 36), so a program built against that header links against this
 * library unchanged.  What differs is the device: this build runs on compute capability 10.0
 * only and reports E5MA_NOT_SUPPORTED elsewhere.
 *
 * Matrices are column-major.  The GEMM computes
 *
 *     D(m x n) = alpha * (sa * sb) * op(A)(m x k) * op(B)(k x n) + bias(m) + beta * C(m x n)
 *
 *   transa == E5MA_OP_T : A is stored k x m, K contiguous, lda >= k
 *   transa == E5MA_OP_N : A is stored m x k,               lda >= m
 *   transb == E5MA_OP_N : B is stored k x n, K contiguous, ldb >= k
 *   transb == E5MA_OP_T : B is stored n x k,               ldb >= n
 *
 * A and B may each be E5M2, E4M3, BF16 or FP32.  sa / sb are the scale_inv factors of FP8
 * operands (taken as 1 when the pointer is NULL or the operand is not FP8); with
 * E5MA_SCALING_OUTER the factor is a vector, one float per row of op(A) (m floats) or per
 * column of op(B) (n floats).  bias has m entries.
 *
 * Accumulate mode: C may alias D; beta != 0 together with C == NULL (or C->data == NULL)
 * means C = D, i.e. D is updated in place (an FP32 main_grad += dY^T X with beta = 1).  C may
 * have any of the five dtypes; an FP8 C is multiplied by C->scale_inv.
 *
 * Output element, evaluated in FP32 without flushing subnormals, in this order:
 *     v = acc * s           with s = (alpha * sa[i]) * sb[j]
 *     v = v + bias[i]
 *     v = fma(beta, C[i,j], v)
 *     amax = max(amax, |v|)                    (NaN does not enter the maximum, Inf does)
 *     D[i,j] = convert(v)                      BF16 / FP16 / FP32: round to nearest even
 *                                              FP8: round to nearest even of v * D->scale,
 *                                              saturating to the largest finite value;
 *                                              every NaN becomes the code 0x7F
 * acc is the FP32 sum over k of the exact products.  On this device the sum is formed by the
 * tensor cores for FP8 and BF16 operand pairs (a different association than an ascending-k
 * chain; |error| <= k * 2^-23 * sum |a*b|) and by an ascending-k FP32 FMA chain otherwise.
 *
 * Problems with n <= 8, transa == T, transb == N and an FP8 A take the streaming GEMV kernel.
 *
 * Requirements: A and B 16-byte aligned; k, lda and ldb multiples of 16; ldc, ldd >= m.
 * GEMM operands must be finite (no E5M2 code with exponent 31, no E4M3 0x7F / 0xFF); this is
 * not checked.  Casts, C and bias decode Inf / NaN codes as Inf / NaN.
 *
 * All pointers inside e5ma_tensor are device pointers.  Calls enqueue work on the given stream
 * of the current device and return without synchronising; the four calls shared with the
 * original interface never allocate memory.
 */
#ifndef E5M2EFFMA_H
#define E5M2EFFMA_H

#define E5M2EFFMA_VERSION "0.2.0"

#include <stddef.h>
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Replaces: reference include/e5m2effma.h:54-59 (same enumerator values). */
typedef enum { E5MA_E4M3 = 0, E5MA_BF16 = 1, E5MA_FP16 = 2, E5MA_FP32 = 3, E5MA_E5M2 = 4 } e5ma_dtype;
typedef enum { E5MA_OP_N = 0, E5MA_OP_T = 1 } e5ma_op;
typedef enum { E5MA_OK = 0, E5MA_INVALID_VALUE = 1, E5MA_NOT_SUPPORTED = 2, E5MA_CUDA_ERROR = 3 } e5ma_status;
typedef enum { E5MA_SCALING_TENSOR = 0, E5MA_SCALING_OUTER = 1 } e5ma_scaling;

/* Replaces: reference include/e5m2effma.h:61-70 (same field order and offsets 0/8/16/24/32/40). */
typedef struct {
  void *data;             /* device pointer to the elements */
  e5ma_dtype dtype;
  const float *scale_inv; /* FP8 input: dequantisation factor (device; 1 float, or a vector
                             with E5MA_SCALING_OUTER); NULL means 1 */
  const float *scale;     /* FP8 output: quantisation factor (device, 1 float); NULL means 1 */
  float *amax;            /* optional statistic (device, 1 float): max |v| before quantisation,
                             max-reduced into the value already there; NULL switches it off */
  e5ma_scaling scaling;   /* E5MA_SCALING_OUTER only for FP8 GEMM operands; 0 otherwise */
} e5ma_tensor;

/* Replaces: reference include/e5m2effma.h:73-76, implemented there by src/gemm_e5m2effma.cu:44-104. */
e5ma_status e5ma_gemm(e5ma_op transa, e5ma_op transb, int m, int n, int k, float alpha,
                      const e5ma_tensor *A, int lda, const e5ma_tensor *B, int ldb, float beta,
                      const e5ma_tensor *C, int ldc, const e5ma_tensor *D, int ldd,
                      const e5ma_tensor *bias, cudaStream_t stream);

/* Element-wise conversion of count contiguous values between any two of the five dtypes:
 * v = src (times src->scale_inv for an FP8 source); dst->amax gets max |v|; dst = convert(v)
 * (an FP8 destination stores the saturating encoding of v * dst->scale).  Per-tensor scaling only.
 * Replaces: reference include/e5m2effma.h:81, implemented there by src/e5m2effma.cu:85-101. */
e5ma_status e5ma_cast(const e5ma_tensor *src, const e5ma_tensor *dst, size_t count, cudaStream_t stream);

/* One in-place Adam / AdamW step over count elements.
 *   param FP32 or BF16; grad FP32, BF16 or FP16; exp_avg and exp_avg_sq both FP32 or both BF16.
 *   param_fp8 (optional): E4M3 or E5M2 copy of the updated FP32 parameter times
 *   param_fp8->scale; param_fp8->amax receives max |param| (only when the copy is requested).
 * Per element, in FP32:
 *   g = grad * grad_scale;            if (!adamw) g = fma(weight_decay, p, g)
 *   m = fma(beta1, m, (1-beta1) * g); v = fma(beta2, v, (1-beta2) * (g*g))
 *   u = (m * rbc1) / (sqrt(v * rbc2) + eps),  rbc = 1 / (1 - beta^step), or 1 without correction
 *   if (adamw) p = fma(-(lr*weight_decay), p, p);   p = fma(-lr, u, p)
 * 1-beta, rbc and lr*weight_decay are computed in double on the host and rounded once.
 * Replaces: reference include/e5m2effma.h:95-106, implemented there by src/adamw_e5m2effma.cu:125-168. */
typedef struct {
  float lr, beta1, beta2, eps, weight_decay;
  int step;            /* counts from 1 */
  int adamw;           /* 1 decoupled weight decay, 0 L2 term folded into the gradient */
  int bias_correction; /* 1 applies 1 / (1 - beta^step) */
  float grad_scale;    /* multiplies the gradient; 0 is read as 1 */
} e5ma_adam_config;

e5ma_status e5ma_adam(const e5ma_adam_config *cfg, size_t count, const e5ma_tensor *param,
                      const e5ma_tensor *grad, const e5ma_tensor *exp_avg,
                      const e5ma_tensor *exp_avg_sq, const e5ma_tensor *param_fp8,
                      cudaStream_t stream);

/* Replaces: reference include/e5m2effma.h:108, src/e5m2effma.cu:103-111. */
const char *e5ma_status_string(e5ma_status status);

/* Message of the last failed e5ma_* call of the calling thread, "" after a success; the buffer
 * is overwritten by the next call on that thread.
 * Replaces: reference include/e5m2effma.h:112, src/e5m2effma.cu:83. */
const char *e5ma_last_error(void);

#ifdef __cplusplus
}
#endif
#endif /* E5M2EFFMA_H */
