// Error plumbing shared by all entry points of the C ABI.
#include <stdarg.h>
#include <string.h>

#include "common.cuh"
#include "sm100_ptx.cuh"

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

extern "C" int b200moe_abi_version(void) { return 7; }

// ---- the failure path of the bounded waits, on its own -------------------------
namespace b200moe {
namespace {
// One CTA sets up an mbarrier that expects an arrival nobody makes and waits on it with the
// same routine, abort flag and teardown order as the grouped GEMM kernels, but with a short
// budget: the wait gives up, the flag goes up, the other warps see it and leave, and the
// status word is written.  Nothing faults and nothing spins without a limit.
__global__ void __launch_bounds__(64) bounded_wait_selftest_kernel(int32_t* status, long long budget_cycles) {
  __shared__ uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    ptx::mbar_init(&bar, 1);
    abort_flag = 0;
    ptx::fence_barrier_init();
  }
  __syncthreads();
  volatile int* af = &abort_flag;
  bool ok = true;
  if (threadIdx.x == 0) {
    ok = ptx::mbar_wait(&bar, 0, af, false, budget_cycles);   // phase 0 never completes
  } else if (threadIdx.x == 32) {
    // a second role, as the MMA issuer beside the producer: it polls the same barrier and
    // must leave through the abort flag once the first wait has given up
    ok = ptx::mbar_wait(&bar, 0, af, false, 4 * budget_cycles);
  }
  __syncthreads();
  if (threadIdx.x == 0 && *af != 0 && status != nullptr) {
    *reinterpret_cast<volatile int32_t*>(status) = 1;
    __threadfence_system();
  }
  (void)ok;
}
}  // namespace
}  // namespace b200moe

extern "C" int b200moe_selftest_bounded_wait(int32_t* status, int64_t budget_cycles, b200moe_stream stream) {
  B200_CHECK_ARG(status != nullptr, "selftest_bounded_wait: null status word");
  B200_CHECK_ARG(budget_cycles > 0 && budget_cycles <= 200000000LL,
                 "selftest_bounded_wait: budget must be in (0, 2e8] cycles (about 0.1 s)");
  b200moe::bounded_wait_selftest_kernel<<<1, 64, 0, b200moe::as_stream(stream)>>>(status, (long long)budget_cycles);
  B200_LAUNCH_OK("bounded_wait_selftest_kernel");
  return B200MOE_OK;
}

extern "C" int b200moe_status_to_code(int32_t status_word) {
  if (status_word == 0) return B200MOE_OK;
  return b200moe::fail(B200MOE_E_DEVICE_TIMEOUT,
                       "a kernel gave up a bounded wait on an mbarrier and left early: the outputs of the "
                       "calls since the status word was last cleared are incomplete");
}
