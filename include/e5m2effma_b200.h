/* e5m2effma_b200.h -- additions of the sm_100a build that the original interface
 * (e5m2effma.h) does not have.  Nothing here is needed to use the five original entry points. */
#ifndef E5M2EFFMA_B200_H
#define E5M2EFFMA_B200_H

#include "e5m2effma.h"

#ifdef __cplusplus
extern "C" {
#endif

/* Diagnostic of the tensor-core GEMM.  Its kernels wait on hardware barriers with a time limit;
 * a wait that runs out makes the kernel give up cleanly (tensor memory released, no hang) and
 * record which role waited for what.  This call synchronises the current device's default
 * context, returns that record (0 = no wait ever ran out) and clears it.
 * No counterpart in the reference, whose kernels have no waits. */
unsigned int e5b_gemm_fault(void);

/* One Adam / AdamW step (the arithmetic of e5ma_adam, same cfg) over a list of num_tensors tensors in as
 * few launches as possible: up to 24 tensors share a launch, each block of the grid works on one
 * 16384-element chunk of one tensor.  counts[t] is the element count of tensor t; params, grads, exp_avgs,
 * exp_avg_sqs are arrays of num_tensors descriptors (host memory, read during the call only); params_fp8
 * is NULL or an array whose entries request an FP8 copy (+ amax) per tensor.  All tensors of a call must
 * agree in the dtypes of param / grad / moments and in having (and the dtype of) the FP8 copy; mixed
 * lists are split by the caller.  Nothing is allocated: the pointer table travels in the kernel
 * parameters.  No counterpart in the reference, whose optimizer launches one kernel per parameter
 * (binds/python/e5m2effma/optim.py:38-52). */
e5ma_status e5b_adam_multi(const e5ma_adam_config *cfg, int num_tensors, const size_t *counts,
                           const e5ma_tensor *params, const e5ma_tensor *grads, const e5ma_tensor *exp_avgs,
                           const e5ma_tensor *exp_avg_sqs, const e5ma_tensor *params_fp8, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* E5M2EFFMA_B200_H */
