// Error plumbing shared by all entry points of the C ABI.
#include <stdarg.h>
#include <string.h>

#include "common.cuh"

namespace b200moe {
namespace {
thread_local char g_last_error[512] = "";
}

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_last_error, sizeof(g_last_error), fmt, ap);
  va_end(ap);
  return code;
}
}  // namespace b200moe

extern "C" const char* b200moe_last_error(void) { return b200moe::g_last_error; }

extern "C" const char* b200moe_status_string(int status) {
  switch (status) {
    case B200MOE_OK: return "ok";
    case B200MOE_E_BADARG: return "bad argument";
    case B200MOE_E_UNSUPPORTED: return "unsupported";
    case B200MOE_E_CUDA: return "CUDA error";
    case B200MOE_E_WORKSPACE: return "workspace missing or too small";
    case B200MOE_E_DEVICE_TIMEOUT: return "device-side wait timed out";
    default: return "unknown status";
  }
}

extern "C" int b200moe_abi_version(void) { return 5; }
