// Programmatic dependent launch for the chain of small kernels of a decode step.  A kernel launched through
// launch_dependent() may be made resident while its predecessor in the stream still runs, once every CTA of the
// predecessor has executed dependents_may_start() (or exited); it must call wait_for_predecessor() before it reads
// anything the predecessor wrote or writes anything the predecessor may still read, and it must not read such data
// through `const __restrict__` pointers or __ldg: loads the compiler may treat as invariant can be moved above the
// wait (seen: a stale position, one chunk early, exactly at chunk boundaries).  Both calls do nothing in a kernel
// that was launched the ordinary way.  MOBA_NO_PDL=1 in the environment makes every launch ordinary (for
// comparison); MOBA_PDL_MASK=<bits> keeps the dependent form only for the kinds whose bit is set (1 projections,
// 2 a step's first launch, 4 routing, 8 attention, 16 arg-max), which is how the rule above was found.
#pragma once
#include <cuda_runtime.h>
#include <stdlib.h>

namespace moba {

__device__ __forceinline__ void dependents_may_start() { asm volatile("griddepcontrol.launch_dependents;"); }
__device__ __forceinline__ void wait_for_predecessor() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

inline unsigned dependent_launch_mask() {
  static const unsigned mask = [] {
    const char* e = getenv("MOBA_NO_PDL");
    if (e && e[0] == '1') return 0u;
    const char* m = getenv("MOBA_PDL_MASK");
    return m ? (unsigned)strtoul(m, nullptr, 0) : ~0u;
  }();
  return mask;
}

template <typename... KArgs, typename... Args>
inline cudaError_t launch_dependent(unsigned kind, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = (dependent_launch_mask() & kind) ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

}  // namespace moba
