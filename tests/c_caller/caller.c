/* A plain C caller of the library, as the reference's own tests and benches are (tests/test_gemm.cu,
 * bench/bench_gemm.cu call these functions through include/e5m2effma.h).  Compiled as C (gnu99) by
 * tests/test_c_caller.py: proves that the headers are valid C, that every entry point has C linkage with the
 * declared prototype, and that validation answers before any device work.  Prints one line per check. */
#include <stdio.h>
#include <string.h>
#include "e5m2effma.h"
#include "e5m2effma_b200.h"

/* the ABI the reference's callers were compiled against (include/e5m2effma.h:54-70, 95-101) */
typedef char tensor_is_48_bytes[sizeof(e5ma_tensor) == 48 ? 1 : -1];
typedef char config_is_36_bytes[sizeof(e5ma_adam_config) == 36 ? 1 : -1];
typedef char enum_values[(E5MA_E4M3 == 0 && E5MA_BF16 == 1 && E5MA_FP16 == 2 && E5MA_FP32 == 3 && E5MA_E5M2 == 4) ? 1 : -1];

/* prototypes: an assignment with a mismatching signature does not compile */
static e5ma_status (*const p_gemm)(e5ma_op, e5ma_op, int, int, int, float, const e5ma_tensor *, int, const e5ma_tensor *, int,
                                   float, const e5ma_tensor *, int, const e5ma_tensor *, int, const e5ma_tensor *,
                                   cudaStream_t) = e5ma_gemm;
static e5ma_status (*const p_cast)(const e5ma_tensor *, const e5ma_tensor *, size_t, cudaStream_t) = e5ma_cast;
static e5ma_status (*const p_adam)(const e5ma_adam_config *, size_t, const e5ma_tensor *, const e5ma_tensor *,
                                   const e5ma_tensor *, const e5ma_tensor *, const e5ma_tensor *, cudaStream_t) = e5ma_adam;
static const char *(*const p_str)(e5ma_status) = e5ma_status_string;
static const char *(*const p_err)(void) = e5ma_last_error;
static unsigned int (*const p_fault)(void) = e5b_gemm_fault;

int main(void) {
  int bad = 0;
  e5ma_tensor a = {0}, d = {0};
  (void)p_adam; (void)p_fault;
  printf("version %s\n", E5M2EFFMA_VERSION);
  printf("status_string(OK) = %s\n", p_str(E5MA_OK));
  /* NULL data: INVALID_VALUE, decided on the host */
  {
    const e5ma_status st = p_gemm(E5MA_OP_T, E5MA_OP_N, 16, 16, 16, 1.0f, &a, 16, &a, 16, 0.0f, NULL, 0, &d, 16, NULL, 0);
    printf("gemm(NULL data) -> %d (%s): %s\n", (int)st, p_str(st), p_err());
    bad += st != E5MA_INVALID_VALUE || strlen(p_err()) == 0;
  }
  {
    const e5ma_status st = p_cast(NULL, NULL, 4, 0);
    printf("cast(NULL) -> %d (%s): %s\n", (int)st, p_str(st), p_err());
    bad += st != E5MA_INVALID_VALUE;
  }
  /* an empty problem succeeds without touching a device and clears the message */
  {
    int x = 0;
    e5ma_status st;
    a.data = &x; a.dtype = E5MA_E5M2; d.data = &x; d.dtype = E5MA_BF16;
    st = p_gemm(E5MA_OP_T, E5MA_OP_N, 0, 16, 16, 1.0f, &a, 16, &a, 16, 0.0f, NULL, 0, &d, 16, NULL, 0);
    printf("gemm(m = 0) -> %d, last_error = \"%s\"\n", (int)st, p_err());
    bad += st != E5MA_OK || strlen(p_err()) != 0;
  }
  printf(bad ? "FAILED\n" : "ok\n");
  return bad;
}
