/* C ABI of libmoba_b200.so: the sm_100a MoBA sparse-attention kernels.
 *
 * Every entry point takes raw device pointers, explicit sizes and a CUDA stream, allocates
 * nothing, never synchronises the host, and returns an int status (MOBA_OK or a MOBA_ERR_*).
 * The caller owns every buffer, so a sequence of calls can be captured in a CUDA graph.
 */
#ifndef MOBA_B200_H_
#define MOBA_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
  MOBA_OK = 0,
  MOBA_ERR_INVALID = 1,     /* an argument violates the documented contract            */
  MOBA_ERR_CUDA = 2,        /* a CUDA runtime call or launch failed                      */
  MOBA_ERR_WORKSPACE = 3,   /* the workspace passed is smaller than *_workspace_bytes()  */
  MOBA_ERR_UNSUPPORTED = 4  /* shape outside the compiled envelope                       */
};

/* Human-readable text for a status code (static storage). */
const char* moba_status_string(int status);

/* Device self-test of the tcgen05 tile primitives (see csrc/selftest.cu). No reference counterpart. */
int moba_selftest_umma(int mode, const void* a, const void* b, float* d, int n, int k, unsigned* status, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* MOBA_B200_H_ */
