// Status strings of the C ABI.
#include "moba_b200.h"

extern "C" const char* moba_status_string(int status) {
  switch (status) {
    case MOBA_OK: return "ok";
    case MOBA_ERR_INVALID: return "invalid argument";
    case MOBA_ERR_CUDA: return "CUDA runtime error";
    case MOBA_ERR_WORKSPACE: return "workspace too small";
    case MOBA_ERR_UNSUPPORTED: return "shape outside the compiled envelope";
    default: return "unknown status";
  }
}

// Size of a descriptor struct as this library was compiled: a binding compares it with its own mirror when it loads the
// library (which = 0: moba_prefill_desc, 1: moba_cache_desc; 0 for anything else).
extern "C" size_t moba_abi_sizeof(int which) {
  return which == 0 ? sizeof(moba_prefill_desc) : which == 1 ? sizeof(moba_cache_desc) : 0;
}

// Profiling aid: events a caller registers are recorded on the launch stream immediately before and
// after the named kernel, so its duration can be read with cudaEventElapsedTime without a profiler.
// Process-wide and not thread-safe; pass null events to switch it off.
#include "moba_b200_debug.h"
#include "prefill_common.cuh"
namespace moba {
static cudaEvent_t g_prof[kProfSlots][2];
void prof_begin(int which, cudaStream_t st) {
  if (g_prof[which][0]) cudaEventRecord(g_prof[which][0], st);
}
void prof_end(int which, cudaStream_t st) {
  if (g_prof[which][1]) cudaEventRecord(g_prof[which][1], st);
}
}  // namespace moba

extern "C" int moba_profile_events(int which, void* start, void* stop) {
  if (which < 1 || which >= moba::kProfSlots) return MOBA_ERR_INVALID;
  moba::g_prof[which][0] = (cudaEvent_t)start;
  moba::g_prof[which][1] = (cudaEvent_t)stop;
  return MOBA_OK;
}
