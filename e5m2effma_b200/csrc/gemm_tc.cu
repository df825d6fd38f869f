// placeholder until the tcgen05 kernel lands: declines every problem
#include "common.cuh"
namespace e5b {
cudaError_t launch_gemm_tc(int, int, bool, bool, const uint8_t *, int, const uint8_t *, int, int, int, int,
                           const OutDesc &, int, cudaStream_t) { return cudaErrorNotSupported; }
}
