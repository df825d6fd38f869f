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
 * record which role waited for what; e5ma_gemm has returned E5MA_OK long before, and D is then
 * undefined.  This call waits for all work of the current device (cudaDeviceSynchronize), returns
 * that record (0 = no wait ever ran out) and clears it.  A caller that needs certainty polls it
 * after the GEMMs it cares about.  The persistent GEMV and e5b_peer_barrier report through the same
 * call: bit 31 / bit 30 set, with the waiting role or peer in the low bits.
 * No counterpart in the reference, whose kernels have no waits. */
unsigned int e5b_gemm_fault(void);

/* Kernel-selection switches for experiments, the tuner and the tests.  name is one of FORCE_SIMT,
 * TC_PAIR, TC_SPLIT, TC_GRID, TC_WIDE, GEMV_KERNEL, GEMV_STAGES, GEMV_U, GEMV_MT, MIXED_PAIR (an
 * "E5MA_" prefix is accepted); each starts from the environment variable E5MA_<name>, read once per
 * process.  value < 0 restores the library's own choice.  Returns 0, or -1 for an unknown name.
 * Process-wide; not meant to be flipped while other threads are inside e5ma_gemm.
 * Takes the place of rebuilding the reference with another tuned table (src/e5m2effma_tuned.h). */
int e5b_set_option(const char *name, int value);

/* The tuned table's plan for a GEMM with operands of elem_bytes (1: FP8 pair, 2: BF16 pair) and this shape:
 * -1 one-CTA kernel, 0 the 256 x 256 CTA-pair kernel, W >= 64 the wide-tile pair kernel with 256 x W tiles;
 * -2 when the table has no entry (the built-in cost model then plans the problem).  The table is the one
 * compiled in (csrc/tuned_sm100.h, written by `python -m e5m2effma_b200.tune --header`), overridden entry by
 * entry by the text file named in E5MA_TUNE_FILE (written by `python -m e5m2effma_b200.tune --write FILE`,
 * read once per process).  Counterpart of the reference's generated src/e5m2effma_tuned.h. */
int e5b_tuned_plan(int elem_bytes, int m, int n, int k);

/* Which kernel the last e5ma_gemm call of the calling host thread launched: 0 none (rejected, or
 * m == 0 / n == 0), 1 streaming GEMV, 2 persistent GEMV, 3 CTA-pair tensor-core GEMM (256 x 256
 * tiles), 4 the same with wide tiles (256 x up to 512), 5 / 6 one-CTA tensor-core GEMM with
 * 256 x 128 / 128 x 128 tiles, 7 ascending-k CUDA-core GEMM, 8 CTA-pair GEMM for FP8 x BF16 pairs,
 * 9 streaming GEMV on the FP32 FMA pipe (FP32 activations, and small batches of the other formats),
 * 10 streaming GEMV with row streams (the tensor-core arithmetic of 1 behind block-wide copies of whole row segments),
 * 11 / 12 the kernels of 5 / 6 with K split over pairs of CTAs (few tiles, long K), 13 / 14 the same kernels with only
 * the tiles of the last, partly filled round shared by CTA pairs.
 * The tests use it to assert that a case really ran on the kernel it was written for.
 * No counterpart in the reference (one GEMM kernel, one GEMV kernel). */
int e5b_last_route(void);

/* e5ma_gemm (same arguments, same checks in the same order, same kernels) whose epilogue stores every
 * output element not only to D but also, at the same element offset, to num_peers (0..7) further
 * buffers peer_d[0..num_peers-1]: the other GPUs' copies of this call's block of D, mapped into the
 * current device's address space (CUDA IPC handles or peer access; each must have D's alignment
 * modulo 16 bytes and D's leading dimension).  This is the all-gather of a column- or row-sharded
 * output fused into the GEMM / GEMV that produces it: the stores travel over NVLink while the tensor
 * cores work on the next tile, no collective is launched and nothing is read from a peer.  amax is
 * reduced into this GPU's D->amax only.  The peers may read their copy once they know this call has
 * completed (an event, or any later collective on the same streams, e.g. the amax max-all-reduce).
 * peer_d is host memory, read during the call only.
 * No counterpart in the reference, which is a single-device library. */
e5ma_status e5b_gemm_bcast(e5ma_op transa, e5ma_op transb, int m, int n, int k, float alpha,
                           const e5ma_tensor *A, int lda, const e5ma_tensor *B, int ldb, float beta,
                           const e5ma_tensor *C, int ldc, const e5ma_tensor *D, int ldd,
                           const e5ma_tensor *bias, int num_peers, void *const *peer_d, cudaStream_t stream);

/* Device-side barrier between the GPUs of a node, for callers of e5b_gemm_bcast that have no other collective to
 * close the step with (the amax max-all-reduce of an FP8 output does that job where there is one): enqueues one small
 * kernel on `stream` that, once everything enqueued before it on this stream has completed, tells every other rank so
 * (one release store per peer, system scope) and returns when every other rank has told this one.  After it, the blocks
 * that the peers' e5b_gemm_bcast calls stored into this GPU's buffer are complete and visible to later work on the stream.
 * flags[r] (r = 0 .. nranks-1, nranks <= 8) is the address, valid on the current device, of rank r's flag area: 16
 * 32-bit words, zeroed once before the first barrier, mapped on every rank like the output buffers (flags[rank] is this
 * rank's own).  Every rank must enqueue the same sequence of barriers; the call count is kept in the flag area, so a
 * barrier can be captured in a CUDA graph and replayed.  The wait is bounded (about two seconds of SM clock): if a
 * peer never arrives the kernel gives up, the fault shows in e5b_gemm_fault() (bit 30) and the data must not be
 * trusted.  flags is host memory, read during the call only.  No counterpart in the reference (single device). */
e5ma_status e5b_peer_barrier(int rank, int nranks, void *const *flags, cudaStream_t stream);

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
