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
extern "C" int lbfq_abi_version(void) { return 2; }

// Kernels launched by this library since load (all entry points count through check_launch()).
namespace lbfq { unsigned long long g_launches = 0; }
extern "C" unsigned long long lbfq_launch_count(void) { return lbfq::g_launches; }

// Rows of `width` bytes between pitched host and device buffers, enqueued on `stream` (one cudaMemcpy2DAsync).
// `to_device` != 0: host -> device, else device -> host.
extern "C" int lbfq_copy_rows_async(void* dst, size_t dst_pitch, const void* src, size_t src_pitch, size_t width,
                                    size_t rows, int to_device, void* stream) {
  LBFQ_REQUIRE(dst != nullptr && src != nullptr, LBFQ_ERR_ARG, "null pointer");
  LBFQ_REQUIRE(width <= dst_pitch && width <= src_pitch, LBFQ_ERR_ARG, "row width exceeds a pitch");
  if (width == 0 || rows == 0) return LBFQ_OK;
  LBFQ_CUDA_OK(cudaMemcpy2DAsync(dst, dst_pitch, src, src_pitch, width, rows,
                                 to_device ? cudaMemcpyHostToDevice : cudaMemcpyDeviceToHost, (cudaStream_t)stream));
  return LBFQ_OK;
}
