// Error text and ABI version of the library.
#include <stdarg.h>
#include <string.h>

#include "common.cuh"

namespace lbfq {
static thread_local char g_err[512] = "";
void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}
}  // namespace lbfq

extern "C" const char* lbfq_last_error(void) { return lbfq::g_err; }
extern "C" int lbfq_abi_version(void) { return 1; }

// Kernels launched by this library since load (all entry points count through check_launch()).
namespace lbfq { unsigned long long g_launches = 0; }
extern "C" unsigned long long lbfq_launch_count(void) { return lbfq::g_launches; }
