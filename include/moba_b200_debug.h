/* Profiling and self-test hooks of libmoba_b200.so.  None has a counterpart in the reference.
 * They are kept out of moba_b200.h because, unlike the entry points there, moba_profile_events
 * keeps process-wide state and is not thread-safe.
 */
#ifndef MOBA_B200_DEBUG_H_
#define MOBA_B200_DEBUG_H_

#ifdef __cplusplus
extern "C" {
#endif

/* Record the given CUDA events right before and after one kernel on its launch stream, so that its
 * duration can be read with cudaEventElapsedTime inside a larger timed region.  which: 1 forward
 * remote pass, 2 forward self pass, 3 backward main kernel, 4 decode attention.  Null events switch
 * it off.  Process-wide, not thread-safe. */
int moba_profile_events(int which, void* start, void* stop);

/* Device self-test of the tcgen05 tile primitives (csrc/selftest.cu): D = A * B in one CTA, in the
 * operand-major combination `mode` selects; d receives the FP32 accumulator [128, n]. */
int moba_selftest_umma(int mode, const void* a, const void* b, float* d, int n, int k, unsigned* status, void* stream);

/* Self-test of the bounded barrier wait every kernel uses: one thread waits at most limit_clocks SM
 * clocks (1 .. 2e9) for an mbarrier phase that nothing completes.  The kernel must return by itself,
 * set the barrier time-out bit of *status (value 1) and write 2 to *returned (1 would mean the wait
 * succeeded).  Enqueues on `stream` and returns. */
int moba_selftest_wait(long long limit_clocks, unsigned* status, int* returned, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* MOBA_B200_DEBUG_H_ */
