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

#ifdef __cplusplus
}
#endif
#endif /* E5M2EFFMA_B200_H */
