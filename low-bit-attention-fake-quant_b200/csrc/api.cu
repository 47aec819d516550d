// Error text and ABI version of the library.
#include <stdarg.h>
#include <stdlib.h>
#include <string.h>

#include <atomic>

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
extern "C" int lbfq_abi_version(void) { return 4; }

namespace lbfq {
int sm_count() {
  static std::atomic<int> cached[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  int n = cached[dev].load(std::memory_order_relaxed);
  if (n == 0) {
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev].store(n, std::memory_order_relaxed);
  }
  return n;
}

static std::atomic<int> g_flags{-1};
static int flags_from_env() {
  auto on = [](const char* name) { const char* v = getenv(name); return v != nullptr && v[0] == '1'; };
  return (on("LBFQ_ATTN_GENERIC") ? LBFQ_FLAG_ATTN_GENERIC : 0) | (on("LBFQ_KMEANS_FFMA") ? LBFQ_FLAG_KMEANS_FFMA : 0) |
         (on("LBFQ_QM_CORR_FFMA") ? LBFQ_FLAG_QM_CORR_FFMA : 0) | (on("LBFQ_UNFUSED_PREPROCESS") ? LBFQ_FLAG_UNFUSED_PREPROCESS : 0) |
         (on("LBFQ_KMEANS_SORTED") ? LBFQ_FLAG_KMEANS_SORTED : 0);
}
int debug_flags() {
  int f = g_flags.load(std::memory_order_relaxed);
  if (f < 0) {
    f = flags_from_env();
    g_flags.store(f, std::memory_order_relaxed);
  }
  return f;
}
}  // namespace lbfq

extern "C" int lbfq_get_flags(void) { return lbfq::debug_flags(); }
extern "C" void lbfq_set_flags(int flags) { lbfq::g_flags.store(flags & 0x7fffffff, std::memory_order_relaxed); }

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

// The GPU's approximate reciprocal, element-wise. A test utility: the reference's quantizers divide by multiplying
// with this value (common.cuh), which a CPU cannot compute itself; a CPU restatement fetches it here.
namespace lbfq {
__global__ void rcp_approx_kernel(const float* __restrict__ x, float* __restrict__ y, long long n) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    y[i] = rcp_approx(x[i]);
}
}  // namespace lbfq
extern "C" int lbfq_rcp_approx(const float* x, float* y, long long n, void* stream) {
  LBFQ_REQUIRE(n >= 0, LBFQ_ERR_ARG, "negative element count");
  if (n == 0) return LBFQ_OK;
  LBFQ_REQUIRE(x != nullptr && y != nullptr, LBFQ_ERR_ARG, "null pointer");
  long long g = (n + 255) / 256;
  if (g > (long long)lbfq::sm_count() * 16) g = (long long)lbfq::sm_count() * 16;
  lbfq::rcp_approx_kernel<<<(int)g, 256, 0, (cudaStream_t)stream>>>(x, y, n);
  return lbfq::check_launch("rcp_approx");
}
