// Smoothing, Hadamard rotation, permutation and the qm.K correction.
//
// Replaces src/low_bit_fake_quant/preprocess.py (K9 smooth_k :10-57, K10
// group_mean_q :60-91, K11 smooth_v_per_block :94-132), the torch FWHT of
// src/low_bit_fake_quant/hadamard.py:25-117, the argsort / scatter / gather
// glue of src/low_bit_fake_quant/kmeans.py:84-95,126-135 and the fp32 matmul
// of attention.py:366-395 / the in-kernel correction of
// attention_triton.py:156-160. All of it is HBM-bound: 16-byte accesses along
// D, one read of the source per pass, means kept in fp32 and the centred
// values rounded once into the input dtype exactly as the reference stores them.

#include <atomic>

#include "tile_ops.cuh"
#include "qm_corr_tc.h"

namespace lbfq {

constexpr int kSumRows = 256;     // rows per partial sum of smooth_k (the reference's BLK_S)

// ---- K9 smooth_k -------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(kThreads)
k_partial_sum_kernel(const T* __restrict__ k, int S, int H, int D, float* __restrict__ partial) {
  __shared__ float buf[kThreads / 8][128 + 1];
  __shared__ float sums[128];
  const int ntile = (S + kSumRows - 1) / kSumRows;
  const int tile = blockIdx.x % ntile;
  const int h = (blockIdx.x / ntile) % H;
  const int b = blockIdx.x / (ntile * H);
  const int s0 = tile * kSumRows;
  const int nrows = min(kSumRows, S - s0);
  const T* src = k + (((size_t)b * S + s0) * H + h) * D;
  column_sums<T>(src, (size_t)H * D, nrows, D, buf, sums);
  if (threadIdx.x < D) partial[(((size_t)b * H + h) * ntile + tile) * D + threadIdx.x] = sums[threadIdx.x];
}

__global__ void k_mean_kernel(const float* __restrict__ partial, int ntile, int D, int S, float* __restrict__ mean) {
  const int bh = blockIdx.x;
  const int d = threadIdx.x;
  if (d >= D) return;
  float acc = 0.f;
  for (int t = 0; t < ntile; ++t) acc += partial[((size_t)bh * ntile + t) * D + d];
  mean[(size_t)bh * D + d] = acc * rcp_approx((float)S);        // the reference's `acc / S` (preprocess.py:29)
}

template <typename T>
__global__ void __launch_bounds__(kThreads)
sub_channel_mean_kernel(const T* __restrict__ x, T* __restrict__ out, const float* __restrict__ mean,
                        int B, int S, int H, int D) {
  const size_t total = (size_t)B * S * H * D / kVec;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (size_t)gridDim.x * blockDim.x) {
    const size_t e0 = i * kVec;
    const int d0 = (int)(e0 % D);
    const size_t row = e0 / D;
    const int h = (int)(row % H);
    const int b = (int)(row / H / S);
    float v[kVec];
    load8<T>(x + e0, v);
    const float* m = mean + ((size_t)b * H + h) * D + d0;
#pragma unroll
    for (int j = 0; j < kVec; ++j) v[j] = v[j] - m[j];
    store8<T>(out + e0, v);
  }
}

// ---- K10 / K11: subtract the column mean of each `block`-row group -----------
template <typename T>
__global__ void __launch_bounds__(kThreads)
block_mean_sub_kernel(const T* __restrict__ x, T* __restrict__ out, float* __restrict__ mean,
                      int S, int H, int D, int block) {
  __shared__ float buf[kThreads / 8][128 + 1];
  __shared__ float sums[128];
  const int nblk = S / block;
  const int blk = blockIdx.x % nblk;
  const int h = (blockIdx.x / nblk) % H;
  const int b = blockIdx.x / (nblk * H);
  const size_t base = (((size_t)b * S + (size_t)blk * block) * H + h) * D;
  const size_t rstride = (size_t)H * D;
  column_sums<T>(x + base, rstride, block, D, buf, sums);
  if (threadIdx.x < D) {
    float m = sums[threadIdx.x] * rcp_approx((float)block);      // the reference's `sum / BLK` (preprocess.py:82,117)
    sums[threadIdx.x] = m;
    mean[(((size_t)b * nblk + blk) * H + h) * D + threadIdx.x] = m;
  }
  __syncthreads();
  const int tpr = D / kVec, rpi = kThreads / tpr;
  const int tr = threadIdx.x / tpr, d0 = (threadIdx.x % tpr) * kVec;
  for (int r = tr; r < block; r += rpi) {
    float v[kVec];
    load8<T>(x + base + r * rstride + d0, v);
#pragma unroll
    for (int j = 0; j < kVec; ++j) v[j] = v[j] - sums[d0 + j];
    store8<T>(out + base + r * rstride + d0, v);
  }
}

// ---- Hadamard: one warp per row of D in {64, 128}; stages in the reference's
// order (stride 1, 2, 4, ...) so every fp32 add / subtract is the same one. ----
template <typename T, int D>
__global__ void __launch_bounds__(kThreads)
hadamard_kernel(const T* __restrict__ x, T* __restrict__ out, const int8_t* __restrict__ signs,
                int64_t rows, int H, float scale) {
  constexpr int E = D / 32;                       // elements per lane: 2 or 4
  const int lane = threadIdx.x & 31;
  const int64_t warp = (int64_t)blockIdx.x * (kThreads / 32) + (threadIdx.x >> 5);
  const int64_t nwarps = (int64_t)gridDim.x * (kThreads / 32);
  for (int64_t row = warp; row < rows; row += nwarps) {
    const T* src = x + row * D + lane * E;
    float v[E];
#pragma unroll
    for (int j = 0; j < E; ++j) v[j] = Elem<T>::load(src + j);
    hadamard_row<T, E>(v, signs ? signs + (size_t)(row % H) * D + lane * E : nullptr, lane);
    T* dst = out + row * D + lane * E;
#pragma unroll
    for (int j = 0; j < E; ++j) Elem<T>::store(dst + j, v[j] * scale);
  }
}

// ---- permutation -------------------------------------------------------------
// Stable counting sort of labels, one CTA per (b,h) slab (kmeans.py:84-88: order = stable argsort(labels),
// inverse[order[j]] = j). Up to 64 labels: histogram, scan, then the tokens in chunks of 1024 in token order -- a lane
// finds the lanes of its warp with the same label, the warp leaders publish their counts, an exclusive scan over
// the 32 warps per label turns them into positions. More labels: one warp per label scans the slab.
constexpr int kOrderMaxK = 64;
__global__ void __launch_bounds__(1024)
label_order_kernel(const int32_t* __restrict__ labels, int S, int k, int64_t* __restrict__ order,
                   int64_t* __restrict__ inverse) {
  __shared__ int counts[kOrderMaxK];
  __shared__ int offsets[kOrderMaxK];
  __shared__ int wc[32][kOrderMaxK];              // per warp and label: count, then start position
  const int32_t* lab = labels + (size_t)blockIdx.x * S;
  int64_t* ord = order + (size_t)blockIdx.x * S;
  int64_t* inv = inverse + (size_t)blockIdx.x * S;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int i = threadIdx.x; i < k; i += blockDim.x) counts[i] = 0;
  __syncthreads();
  // a label outside [0, k) (never produced by this library) is skipped, not used as an index
  for (int i = threadIdx.x; i < S; i += blockDim.x)
    if ((unsigned)lab[i] < (unsigned)k) atomicAdd(&counts[lab[i]], 1);
  __syncthreads();
  if (threadIdx.x == 0) {
    int run = 0;
    for (int c = 0; c < k; ++c) { offsets[c] = run; run += counts[c]; }
  }
  for (int base = 0; base < S; base += 1024) {
    for (int i = threadIdx.x; i < 32 * kOrderMaxK; i += blockDim.x) (&wc[0][0])[i] = 0;
    __syncthreads();
    const int i = base + (int)threadIdx.x;
    int lbl = i < S ? lab[i] : -1;
    const bool valid = (unsigned)lbl < (unsigned)k;
    if (!valid) lbl = -1;
    const unsigned peers = __match_any_sync(0xffffffffu, lbl);
    const int rank = __popc(peers & ((1u << lane) - 1u));
    if (valid && rank == 0) wc[warp][lbl] = __popc(peers);
    __syncthreads();
    if ((int)threadIdx.x < k) {                               // exclusive scan over the warps, in token order
      int run = offsets[threadIdx.x];
      for (int w = 0; w < 32; ++w) { const int c = wc[w][threadIdx.x]; wc[w][threadIdx.x] = run; run += c; }
      offsets[threadIdx.x] = run;
    }
    __syncthreads();
    if (valid) {
      const int p = wc[warp][lbl] + rank;
      ord[p] = i;
      inv[i] = p;
    }
    __syncthreads();
  }
}

__global__ void __launch_bounds__(1024)
label_order_scan_kernel(const int32_t* __restrict__ labels, int S, int k, int64_t* __restrict__ order,
                        int64_t* __restrict__ inverse) {
  extern __shared__ int sm_counts[];              // k counts, then k offsets
  int* counts = sm_counts;
  int* offsets = sm_counts + k;
  const int32_t* lab = labels + (size_t)blockIdx.x * S;
  int64_t* ord = order + (size_t)blockIdx.x * S;
  int64_t* inv = inverse + (size_t)blockIdx.x * S;
  for (int i = threadIdx.x; i < k; i += blockDim.x) counts[i] = 0;
  __syncthreads();
  for (int i = threadIdx.x; i < S; i += blockDim.x)
    if ((unsigned)lab[i] < (unsigned)k) atomicAdd(&counts[lab[i]], 1);
  __syncthreads();
  if (threadIdx.x == 0) {
    int run = 0;
    for (int c = 0; c < k; ++c) { offsets[c] = run; run += counts[c]; }
  }
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  for (int c = warp; c < k; c += nwarps) {
    int pos = offsets[c];
    for (int base = 0; base < S; base += 32) {
      const int i = base + lane;
      const bool hit = (i < S) && (lab[i] == c);
      const unsigned m = __ballot_sync(0xffffffffu, hit);
      if (hit) {
        const int p = pos + __popc(m & ((1u << lane) - 1u));
        ord[p] = i;
        inv[i] = p;
      }
      pos += __popc(m);
    }
  }
}

template <int BYTES_PER_ELEM>
__global__ void __launch_bounds__(kThreads)
gather_rows_kernel(const uint8_t* __restrict__ x, uint8_t* __restrict__ out, const int64_t* __restrict__ index,
                   int B, int S, int H, int D) {
  const int row_bytes = D * BYTES_PER_ELEM;
  const int cpr = row_bytes / 16;                 // 16-byte chunks per row
  const size_t total = (size_t)B * S * H * cpr;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (size_t)gridDim.x * blockDim.x) {
    const int c = (int)(i % cpr);
    const size_t row = i / cpr;                   // (b*S + j)*H + h
    const int h = (int)(row % H);
    const size_t bj = row / H;
    const int j = (int)(bj % S);
    const int b = (int)(bj / S);
    const int64_t srow = index[((size_t)b * H + h) * S + j];
    const uint4 val = *reinterpret_cast<const uint4*>(x + ((((size_t)b * S + srow) * H + h) * (size_t)row_bytes) + c * 16);
    *reinterpret_cast<uint4*>(out + row * (size_t)row_bytes + c * 16) = val;
  }
}

// ---- qm . K_smooth: fp32 tiled product, 64 groups x 64 keys per CTA -----------
constexpr int kCT = 64;

__device__ __forceinline__ void atomic_max_float(float* addr, float v) {
  if (v >= 0.f) atomicMax(reinterpret_cast<int*>(addr), __float_as_int(v));
  else atomicMin(reinterpret_cast<unsigned int*>(addr), __float_as_uint(v));
}

__global__ void fill_kernel(float* p, size_t n, float v) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) p[i] = v;
}

template <typename T>
__global__ void __launch_bounds__(kThreads)
qm_corr_kernel(const float* __restrict__ qm, const T* __restrict__ ks, int B, int S, int H, int D, int G,
               float sm_scale, float* __restrict__ corr, int s_pad, float* __restrict__ rowmax) {
  __shared__ float a_s[kCT][32 + 1];              // qm tile  [g][d-chunk]
  __shared__ float b_s[kCT][32 + 1];              // key tile [n][d-chunk]
  const int ntn = s_pad / kCT;
  const int ntg = (G + kCT - 1) / kCT;
  const int tn = blockIdx.x % ntn;
  const int tg = (blockIdx.x / ntn) % ntg;
  const int bh = blockIdx.x / (ntn * ntg);
  const int b = bh / H, h = bh % H;
  const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;      // 16 x 16 threads, 4 x 4 outputs each
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
  for (int d0 = 0; d0 < D; d0 += 32) {
    for (int idx = threadIdx.x; idx < kCT * 32; idx += kThreads) {
      const int r = idx / 32, c = idx % 32;
      const int g = tg * kCT + r;
      a_s[r][c] = g < G ? qm[(((size_t)b * G + g) * H + h) * D + d0 + c] : 0.f;
      const int n = tn * kCT + r;
      b_s[r][c] = n < S ? Elem<T>::load(ks + (((size_t)b * S + n) * H + h) * D + d0 + c) : 0.f;
    }
    __syncthreads();
#pragma unroll 8
    for (int c = 0; c < 32; ++c) {
      float av[4], bv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) av[i] = a_s[ty * 4 + i][c];
#pragma unroll
      for (int j = 0; j < 4; ++j) bv[j] = b_s[tx * 4 + j][c];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int g = tg * kCT + ty * 4 + i;
    const bool g_ok = g < G;                      // no early exit: the shuffles below need the full warp
    float4 o;
    float* op = reinterpret_cast<float*>(&o);
    float rm = -INFINITY;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = tn * kCT + tx * 4 + j;
      const float v = acc[i][j] * sm_scale;
      op[j] = n < S ? v : 0.f;
      if (n < S) rm = fmaxf(rm, v);
    }
    if (g_ok) *reinterpret_cast<float4*>(corr + (((size_t)bh * G + g) * s_pad) + tn * kCT + tx * 4) = o;
    if (rowmax) {
      // reduce over the 16 tx lanes that share this g (contiguous half-warp)
#pragma unroll
      for (int o2 = 8; o2 > 0; o2 >>= 1) rm = fmaxf(rm, __shfl_xor_sync(0xffffffffu, rm, o2));
      if (g_ok && tx == 0 && rm > -INFINITY) atomic_max_float(rowmax + (size_t)bh * G + g, rm);
    }
  }
}

}  // namespace lbfq

using namespace lbfq;

static int grid_for(size_t work_items, int threads) {
  size_t g = (work_items + threads - 1) / threads;
  const size_t cap = (size_t)sm_count() * 16;
  return (int)(g < cap ? (g ? g : 1) : cap);
}

extern "C" int64_t lbfq_smooth_k_scratch_floats(int B, int S, int H, int D) {
  return (int64_t)B * H * ((S + kSumRows - 1) / kSumRows) * D;
}

extern "C" int lbfq_smooth_k(const void* k, int dtype, int B, int S, int H, int D, void* out, float* mean,
                             float* partial, void* stream) {
  LBFQ_REQUIRE(B > 0 && S > 0 && H > 0, LBFQ_ERR_ARG, "smooth_k: unsupported shape (%d,%d,%d,%d)", B, S, H, D);
  // the column-sum tiles are laid out for 8 or 16 threads per row: other head dimensions would run past them
  LBFQ_REQUIRE(D == 64 || D == 128, LBFQ_ERR_ARG, "smooth_k: D must be 64 or 128; got %d", D);
  cudaStream_t st = (cudaStream_t)stream;
  const int ntile = (S + kSumRows - 1) / kSumRows;
  LBFQ_DISPATCH_DTYPE(dtype, T,
      k_partial_sum_kernel<T><<<B * H * ntile, kThreads, 0, st>>>((const T*)k, S, H, D, partial));
  if (int rc = check_launch("k_partial_sum")) return rc;
  k_mean_kernel<<<B * H, 128, 0, st>>>(partial, ntile, D, S, mean);
  if (int rc = check_launch("k_mean")) return rc;
  if (out == nullptr) return LBFQ_OK;                // the mean alone (the caller centres while quantising)
  const size_t total = (size_t)B * S * H * D / kVec;
  LBFQ_DISPATCH_DTYPE(dtype, T,
      sub_channel_mean_kernel<T><<<grid_for(total, kThreads), kThreads, 0, st>>>((const T*)k, (T*)out, mean, B, S, H, D));
  return check_launch("sub_channel_mean");
}

// ---------------------------------------------------------------------------
// smooth_k for callers that cannot allocate device memory.
//
// Some hosts of this library hand it input and output buffers but have no way
// to give it scratch: a plugin running inside another framework's memory
// pool, a region where allocation is forbidden (for example while the caller
// is recording work for later replay), or an embedder whose allocator is not
// reachable from the call site. For them the per-tile partial column sums of
// smooth_k live in a fixed array inside the library image instead of in a
// caller buffer. Every GPU that loads the library carries this array
// (kStaticScratchFloats * 4 bytes = 4 MiB) until the process exits.
// ---------------------------------------------------------------------------
constexpr int64_t kStaticScratchFloats = 1 << 20;
static __device__ __align__(256) float g_smooth_k_scratch[kStaticScratchFloats];

constexpr int kMaxDevices = 64;
// device address of the array, per device ordinal (threads that make the first call on a device together all look
// up, and store, the same address)
static std::atomic<float*> g_scratch_ptr[kMaxDevices];

// Host code must not pass `g_smooth_k_scratch` itself to a kernel: in host code that
// name is only a handle. The device address is asked for once per device, with that
// device current, and cached.
static int static_scratch_for_current_device(float** out) {
  int dev = -1;
  LBFQ_CUDA_OK(cudaGetDevice(&dev));
  LBFQ_REQUIRE(dev >= 0 && dev < kMaxDevices, LBFQ_ERR_UNSUPPORTED, "device ordinal %d outside the supported 0..%d", dev, kMaxDevices - 1);
  float* cached = g_scratch_ptr[dev].load(std::memory_order_acquire);
  if (cached == nullptr) {
    void* ptr = nullptr;
    LBFQ_CUDA_OK(cudaGetSymbolAddress(&ptr, g_smooth_k_scratch));
    LBFQ_REQUIRE(ptr != nullptr, LBFQ_ERR_CUDA, "cudaGetSymbolAddress returned a null address");
    cached = static_cast<float*>(ptr);
    g_scratch_ptr[dev].store(cached, std::memory_order_release);
  }
  *out = cached;
  return LBFQ_OK;
}

extern "C" int64_t lbfq_smooth_k_static_max_floats(void) { return kStaticScratchFloats; }

extern "C" int lbfq_smooth_k_static(const void* k, int dtype, int B, int S, int H, int D, void* out, float* mean,
                                    void* stream) {
  const int64_t need = lbfq_smooth_k_scratch_floats(B, S, H, D);
  LBFQ_REQUIRE(B > 0 && S > 0 && H > 0, LBFQ_ERR_ARG, "smooth_k: unsupported shape (%d,%d,%d,%d)", B, S, H, D);
  LBFQ_REQUIRE(D == 64 || D == 128, LBFQ_ERR_ARG, "smooth_k: D must be 64 or 128; got %d", D);
  LBFQ_REQUIRE(need <= kStaticScratchFloats, LBFQ_ERR_ARG,
               "smooth_k_static: this shape needs %lld scratch floats (B*H*ceil(S/256)*D) but the built-in array holds "
               "%lld; use lbfq_smooth_k with caller scratch", (long long)need, (long long)kStaticScratchFloats);
  float* scratch = nullptr;
  if (int rc = static_scratch_for_current_device(&scratch)) return rc;
  // every partial sum the second kernel reads is written by the first one in this call,
  // so nothing left over from an earlier call needs clearing
  return lbfq_smooth_k(k, dtype, B, S, H, D, out, mean, scratch, stream);
}

extern "C" int lbfq_block_mean_sub(const void* x, int dtype, int B, int S, int H, int D, int block,
                                   void* out, float* mean, void* stream) {
  LBFQ_REQUIRE(D == 64 || D == 128, LBFQ_ERR_ARG, "D must be 64 or 128; got %d", D);
  LBFQ_REQUIRE(block > 0 && S % block == 0, LBFQ_ERR_ARG, "S=%d must be divisible by block_s=%d", S, block);
  cudaStream_t st = (cudaStream_t)stream;
  LBFQ_DISPATCH_DTYPE(dtype, T,
      block_mean_sub_kernel<T><<<B * (S / block) * H, kThreads, 0, st>>>((const T*)x, (T*)out, mean, S, H, D, block));
  return check_launch("block_mean_sub");
}

extern "C" int lbfq_hadamard(const void* x, int dtype, int64_t rows, int H, int D, const int8_t* signs,
                             float scale, void* out, void* stream) {
  LBFQ_REQUIRE(D == 64 || D == 128, LBFQ_ERR_UNSUPPORTED, "hadamard: last dim must be 64 or 128; got %d", D);
  LBFQ_REQUIRE(rows > 0 && H > 0, LBFQ_ERR_ARG, "hadamard: empty input");
  cudaStream_t st = (cudaStream_t)stream;
  const int grid = grid_for((size_t)rows * 32, kThreads);
  if (D == 128) {
    LBFQ_DISPATCH_DTYPE(dtype, T,
        hadamard_kernel<T, 128><<<grid, kThreads, 0, st>>>((const T*)x, (T*)out, signs, rows, H, scale));
  } else {
    LBFQ_DISPATCH_DTYPE(dtype, T,
        hadamard_kernel<T, 64><<<grid, kThreads, 0, st>>>((const T*)x, (T*)out, signs, rows, H, scale));
  }
  return check_launch("hadamard");
}

extern "C" int lbfq_label_order(const int32_t* labels, int BH, int S, int k, int64_t* order, int64_t* inverse,
                                void* stream) {
  LBFQ_REQUIRE(BH > 0 && S > 0 && k > 0 && k <= 4096, LBFQ_ERR_ARG, "label_order: bad sizes BH=%d S=%d k=%d", BH, S, k);
  if (k <= kOrderMaxK) label_order_kernel<<<BH, 1024, 0, (cudaStream_t)stream>>>(labels, S, k, order, inverse);
  else label_order_scan_kernel<<<BH, 1024, 2 * k * sizeof(int), (cudaStream_t)stream>>>(labels, S, k, order, inverse);
  return check_launch("label_order");
}

extern "C" int lbfq_gather_rows(const void* x, int dtype, int B, int S, int H, int D, const int64_t* index,
                                void* out, void* stream) {
  LBFQ_REQUIRE(B > 0 && S > 0 && H > 0 && D > 0 && D % 8 == 0, LBFQ_ERR_ARG, "gather_rows: bad shape");
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == LBFQ_F32) {
    const size_t total = (size_t)B * S * H * (D * 4 / 16);
    gather_rows_kernel<4><<<grid_for(total, kThreads), kThreads, 0, st>>>((const uint8_t*)x, (uint8_t*)out, index, B, S, H, D);
  } else if (dtype == LBFQ_F16 || dtype == LBFQ_BF16) {
    const size_t total = (size_t)B * S * H * (D * 2 / 16);
    gather_rows_kernel<2><<<grid_for(total, kThreads), kThreads, 0, st>>>((const uint8_t*)x, (uint8_t*)out, index, B, S, H, D);
  } else {
    set_error("unsupported dtype code %d", dtype);
    return LBFQ_ERR_DTYPE;
  }
  return check_launch("gather_rows");
}

extern "C" int lbfq_qm_corr(const float* qm, const void* k_smooth, int dtype, int B, int S, int H, int D, int G,
                            float sm_scale, float* corr, int s_pad, float* rowmax, int32_t* status, void* stream) {
  LBFQ_REQUIRE(D % 32 == 0 && D <= 128, LBFQ_ERR_ARG, "qm_corr: D must be 64 or 128; got %d", D);
  LBFQ_REQUIRE(s_pad >= S && s_pad % kCT == 0, LBFQ_ERR_ARG, "qm_corr: s_pad=%d must be >= S and a multiple of %d", s_pad, kCT);
  LBFQ_REQUIRE(G > 0, LBFQ_ERR_ARG, "qm_corr: G must be positive");
  cudaStream_t st = (cudaStream_t)stream;
  if (rowmax) {
    fill_kernel<<<grid_for((size_t)B * H * G, 256), 256, 0, st>>>(rowmax, (size_t)B * H * G, -INFINITY);
    if (int rc = check_launch("fill")) return rc;
  }
  // BF16 keys take the tensor-core kernel; LBFQ_FLAG_QM_CORR_FFMA keeps the FP32 FFMA kernel (the cross-check)
  if (qm_corr_tc_eligible(dtype, D, S, k_smooth) && !(debug_flags() & LBFQ_FLAG_QM_CORR_FFMA))
    return qm_corr_tc(qm, k_smooth, B, S, H, D, G, sm_scale, corr, s_pad, rowmax, status, st);
  const int grid = B * H * ((G + kCT - 1) / kCT) * (s_pad / kCT);
  LBFQ_DISPATCH_DTYPE(dtype, T,
      qm_corr_kernel<T><<<grid, kThreads, 0, st>>>(qm, (const T*)k_smooth, B, S, H, D, G, sm_scale, corr, s_pad, rowmax));
  return check_launch("qm_corr");
}
