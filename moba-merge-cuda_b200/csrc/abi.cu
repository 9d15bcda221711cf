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
