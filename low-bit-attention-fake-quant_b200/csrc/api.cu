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
