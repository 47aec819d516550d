// FP8 / MXFP8 quantizers and de-quantizers.
//
// Replaces the Triton kernels of src/low_bit_fake_quant/quant_triton.py
// (K1 fp8_block :26-58, K3 fp8_channel :134-176, K5 mxfp8_qk :221-271,
// K7 mxfp8_v :322-369 and the four de-quantizers) with HBM-bound CUDA kernels:
// every thread moves 8 consecutive elements of D per access (16-byte loads for
// BF16/F16), a CTA owns one scale block, reads it once from HBM (the second,
// quantising read of the same <= 64 KB tile is served by L1/L2) and writes the
// e4m3 codes straight into the layout the consumer wants: NHD for the public
// API, BHSD / BHDS (transposed through shared memory) for the attention kernel.
// Arithmetic is the reference's as its Triton kernels execute it on the GPU: amax floored at 1e-4,
// scale = amax * fl32(1/448), code = e4m3_rn_sat(clamp(x * rcp.approx(scale), +-448)) -- see common.cuh. One
// reciprocal per scale block, one multiplication per element.

#include "tile_ops.cuh"

namespace lbfq {

// ---------------------------------------------------------------------------
// K1: fp8_block -- one scale per (b, S-block, h) tile of block_s x D.
// ---------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(kThreads)
fp8_block_quant_kernel(const T* __restrict__ x, CodeDst dst, float* __restrict__ scale, int block_s,
                       const float* __restrict__ mean) {
  __shared__ float red[kThreads / 32];
  __shared__ float s_scale;
  __shared__ __align__(16) uint8_t tbuf[128 * kTPitch];
  const int nblk = dst.S / block_s;
  const int blk = blockIdx.x % nblk;
  const int h = (blockIdx.x / nblk) % dst.H;
  const int b = blockIdx.x / (nblk * dst.H);
  const int D = dst.D, tpr = D / kVec, rpi = kThreads / tpr;
  const int tr = threadIdx.x / tpr, d0 = (threadIdx.x % tpr) * kVec;
  const int s0 = blk * block_s;
  const T* src = x + (((size_t)b * dst.S + s0) * dst.H + h) * D;
  const size_t rstride = (size_t)dst.H * D;

  // optional centring: the tensor that is quantised is round_T(x - mean[b, h, :]), what smooth_k would have stored
  auto centre = [&](float (&v)[kVec], int dd) {
    if (mean != nullptr) {
      const float* m = mean + ((size_t)b * dst.H + h) * D + dd;
#pragma unroll
      for (int i = 0; i < kVec; ++i) v[i] = round_through<T>(v[i] - m[i]);
    }
  };
  float amax = 0.f;
  for (int r = tr; r < block_s; r += rpi) {
    float v[kVec];
    load8<T>(src + r * rstride + d0, v);
    centre(v, d0);
#pragma unroll
    for (int i = 0; i < kVec; ++i) amax = fmaxf(amax, fabsf(v[i]));
  }
  amax = warp_max(amax);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
  __syncthreads();
  if (threadIdx.x == 0) {
    float m = red[0];
#pragma unroll
    for (int i = 1; i < kThreads / 32; ++i) m = fmaxf(m, red[i]);
    float sc = scale_from_amax(fmaxf(m, kAmaxFloor));
    s_scale = sc;
    scale[((size_t)b * nblk + blk) * dst.H + h] = sc;
  }
  __syncthreads();
  const float sc = s_scale;
  const float rsc = rcp_approx(sc);
  store_tile(dst, b, h, s0, block_s, tbuf, [&](int r, int dd, float (&q)[kVec]) {
    float v[kVec];
    load8<T>(src + r * rstride + dd, v);
    centre(v, dd);
#pragma unroll
    for (int i = 0; i < kVec; ++i) q[i] = fminf(fmaxf(v[i] * rsc, -kFp8Max), kFp8Max);
  });
}

// ---------------------------------------------------------------------------
// K7: mxfp8_v -- power-of-two scale per (b, S-block, h, d); blocks along S.
// ---------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(kThreads)
mxfp8_v_quant_kernel(const T* __restrict__ x, CodeDst dst, float* __restrict__ scale, int block_s) {
  __shared__ float col_amax[kThreads / 8][128 + 1];   // [row-lane][d]
  __shared__ float col_scale[128];                    // 2^-e: the exact reciprocal of the power-of-two scale
  __shared__ __align__(16) uint8_t tbuf[128 * kTPitch];
  const int nblk = dst.S / block_s;
  const int blk = blockIdx.x % nblk;
  const int h = (blockIdx.x / nblk) % dst.H;
  const int b = blockIdx.x / (nblk * dst.H);
  const int D = dst.D, tpr = D / kVec, rpi = kThreads / tpr;
  const int tr = threadIdx.x / tpr, d0 = (threadIdx.x % tpr) * kVec;
  const int s0 = blk * block_s;
  const T* src = x + (((size_t)b * dst.S + s0) * dst.H + h) * D;
  const size_t rstride = (size_t)dst.H * D;

  float am[kVec];
#pragma unroll
  for (int i = 0; i < kVec; ++i) am[i] = 0.f;
  for (int r = tr; r < block_s; r += rpi) {
    float v[kVec];
    load8<T>(src + r * rstride + d0, v);
#pragma unroll
    for (int i = 0; i < kVec; ++i) am[i] = fmaxf(am[i], fabsf(v[i]));
  }
#pragma unroll
  for (int i = 0; i < kVec; ++i) col_amax[tr][d0 + i] = am[i];
  __syncthreads();
  if (threadIdx.x < D) {
    float m = 0.f;
    for (int r = 0; r < rpi; ++r) m = fmaxf(m, col_amax[r][threadIdx.x]);
    const int e = pow2_scale_exp(fmaxf(m, kAmaxFloor));
    col_scale[threadIdx.x] = pow2f(-e);
    scale[(((size_t)b * nblk + blk) * dst.H + h) * D + threadIdx.x] = pow2f(e);
  }
  __syncthreads();
  store_tile(dst, b, h, s0, block_s, tbuf, [&](int r, int dd, float (&q)[kVec]) {
    float v[kVec];
    load8<T>(src + r * rstride + dd, v);
#pragma unroll
    for (int i = 0; i < kVec; ++i)
      q[i] = fminf(fmaxf(v[i] * col_scale[dd + i], -kFp8Max), kFp8Max);     // x / 2^e, exact
  });
}

// ---------------------------------------------------------------------------
// K5: mxfp8_qk -- power-of-two scale per (b, s, h, 32-element group of D).
// One CTA handles kRows tokens of one (b, h); group amax is a shuffle over the
// block_d / 8 lanes that hold the group.
// ---------------------------------------------------------------------------
constexpr int kMxRows = 64;

template <typename T>
__global__ void __launch_bounds__(kThreads)
mxfp8_qk_quant_kernel(const T* __restrict__ x, CodeDst dst, float* __restrict__ scale,
                      uint8_t* __restrict__ scale_e8, int block_d) {
  __shared__ float grp_scale[kMxRows][128 / 8 + 1];   // scale of the group owning d0, per row
  __shared__ __align__(16) uint8_t tbuf[128 * kTPitch];
  const int ntile = (dst.S + kMxRows - 1) / kMxRows;
  const int tile = blockIdx.x % ntile;
  const int h = (blockIdx.x / ntile) % dst.H;
  const int b = blockIdx.x / (ntile * dst.H);
  const int D = dst.D, tpr = D / kVec, rpi = kThreads / tpr;
  const int tr = threadIdx.x / tpr, d0 = (threadIdx.x % tpr) * kVec;
  const int s0 = tile * kMxRows;
  const int nrows = min(kMxRows, dst.S - s0);
  const T* src = x + (((size_t)b * dst.S + s0) * dst.H + h) * D;
  const size_t rstride = (size_t)dst.H * D;
  const int lanes = block_d / kVec;             // lanes sharing one scale (power of two, <= 16)
  const int ngrp = D / block_d;

  for (int r = tr; r < kMxRows; r += rpi) {     // uniform trip count: shuffles stay converged
    float am = 0.f;
    if (r < nrows) {
      float v[kVec];
      load8<T>(src + r * rstride + d0, v);
#pragma unroll
      for (int i = 0; i < kVec; ++i) am = fmaxf(am, fabsf(v[i]));
    }
    for (int o = lanes >> 1; o > 0; o >>= 1) am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, o));
    if (r < nrows) {
      int e = pow2_scale_exp(fmaxf(am, kAmaxFloor));
      float sc = pow2f(e);
      grp_scale[r][d0 / kVec] = pow2f(-e);          // the exact reciprocal
      if ((d0 % block_d) == 0) {
        int g = d0 / block_d;
        scale[((((size_t)b * dst.S + s0 + r) * dst.H + h)) * ngrp + g] = sc;
        if (scale_e8) {
          // 128-token x 4-group tiles of 512 bytes in the order the block-scaled MMA reads scale
          // factors from tensor memory: byte (t % 32) * 16 + (t / 32) * 4 + g for token t of the tile
          const int tok = s0 + r, tile128 = tok >> 7, tt = tok & 127;
          scale_e8[(((size_t)b * dst.H + h) * (dst.s_pad >> 7) + tile128) * 512 + (tt & 31) * 16 + (tt >> 5) * 4 + g] =
              (uint8_t)(e + 127);
        }
      }
    }
  }
  __syncthreads();
  store_tile(dst, b, h, s0, nrows, tbuf, [&](int r, int dd, float (&q)[kVec]) {
    float v[kVec];
    load8<T>(src + r * rstride + dd, v);
    const float rsc = grp_scale[r][dd / kVec];
#pragma unroll
    for (int i = 0; i < kVec; ++i) q[i] = fminf(fmaxf(v[i] * rsc, -kFp8Max), kFp8Max);      // x / 2^e, exact
  });
}

// ---------------------------------------------------------------------------
// K3: fp8_channel -- one scale per (b, h, d) over all of S: a column-amax pass
// (atomicMax on the bit pattern of the non-negative amax), a finishing kernel
// that floors and divides, then the quantising pass.
// ---------------------------------------------------------------------------
constexpr int kChanRows = 256;

template <typename T>
__global__ void __launch_bounds__(kThreads)
channel_amax_kernel(const T* __restrict__ x, int S, int H, int D, unsigned int* __restrict__ amax_bits) {
  __shared__ float col_amax[kThreads / 8][128 + 1];
  const int ntile = (S + kChanRows - 1) / kChanRows;
  const int tile = blockIdx.x % ntile;
  const int h = (blockIdx.x / ntile) % H;
  const int b = blockIdx.x / (ntile * H);
  const int tpr = D / kVec, rpi = kThreads / tpr;
  const int tr = threadIdx.x / tpr, d0 = (threadIdx.x % tpr) * kVec;
  const int s0 = tile * kChanRows;
  const int nrows = min(kChanRows, S - s0);
  const T* src = x + (((size_t)b * S + s0) * H + h) * D;
  const size_t rstride = (size_t)H * D;
  float am[kVec];
#pragma unroll
  for (int i = 0; i < kVec; ++i) am[i] = 0.f;
  for (int r = tr; r < nrows; r += rpi) {
    float v[kVec];
    load8<T>(src + r * rstride + d0, v);
#pragma unroll
    for (int i = 0; i < kVec; ++i) am[i] = fmaxf(am[i], fabsf(v[i]));
  }
#pragma unroll
  for (int i = 0; i < kVec; ++i) col_amax[tr][d0 + i] = am[i];
  __syncthreads();
  if (threadIdx.x < D) {
    float m = 0.f;
    for (int r = 0; r < rpi; ++r) m = fmaxf(m, col_amax[r][threadIdx.x]);
    atomicMax(amax_bits + ((size_t)b * H + h) * D + threadIdx.x, __float_as_uint(m));
  }
}

__global__ void channel_scale_kernel(float* scale, int n) {
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) scale[i] = scale_from_amax(fmaxf(scale[i], kAmaxFloor));      // in place: amax -> scale
}

template <typename T>
__global__ void __launch_bounds__(kThreads)
channel_quant_kernel(const T* __restrict__ x, CodeDst dst, const float* __restrict__ scale) {
  __shared__ float col_rcp[128];
  __shared__ __align__(16) uint8_t tbuf[128 * kTPitch];
  const int ntile = (dst.S + kTChunk - 1) / kTChunk;
  const int tile = blockIdx.x % ntile;
  const int h = (blockIdx.x / ntile) % dst.H;
  const int b = blockIdx.x / (ntile * dst.H);
  const int D = dst.D;
  const int s0 = tile * kTChunk;
  const int nrows = min(kTChunk, dst.S - s0);
  const T* src = x + (((size_t)b * dst.S + s0) * dst.H + h) * D;
  const size_t rstride = (size_t)dst.H * D;
  if (threadIdx.x < D) {
    col_rcp[threadIdx.x] = rcp_approx(scale[((size_t)b * dst.H + h) * D + threadIdx.x]);
  }
  __syncthreads();
  store_tile(dst, b, h, s0, nrows, tbuf, [&](int r, int dd, float (&q)[kVec]) {
    float v[kVec];
    load8<T>(src + r * rstride + dd, v);
#pragma unroll
    for (int i = 0; i < kVec; ++i)
      q[i] = fminf(fmaxf(v[i] * col_rcp[dd + i], -kFp8Max), kFp8Max);
  });
}

// ---------------------------------------------------------------------------
// De-quantizers (K2, K4, K6, K8): code.fp32 * scale, one rounding into out dtype.
// kind: 0 fp8_block (B,S/blk,H); 1 channel (B,H,D); 2 mx_qk (B,S,H,D/blk); 3 mx_v (B,S/blk,H,D)
// ---------------------------------------------------------------------------
template <typename T>
__global__ void dequant_kernel(const uint8_t* __restrict__ codes, const float* __restrict__ scale,
                               T* __restrict__ out, int B, int S, int H, int D, int kind, int blk) {
  const size_t total = (size_t)B * S * H * D / kVec;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (size_t)gridDim.x * blockDim.x) {
    const size_t e0 = i * kVec;
    const int d0 = (int)(e0 % D);
    const size_t row = e0 / D;              // (b*S + s)*H + h
    const int h = (int)(row % H);
    const size_t bs = row / H;
    const int s = (int)(bs % S);
    const int b = (int)(bs / S);
    uint2 raw = *reinterpret_cast<const uint2*>(codes + e0);
    const uint8_t* c = reinterpret_cast<const uint8_t*>(&raw);
#pragma unroll
    for (int j = 0; j < kVec; ++j) {
      float sc;
      if (kind == 0) sc = scale[((size_t)b * (S / blk) + s / blk) * H + h];
      else if (kind == 1) sc = scale[((size_t)b * H + h) * D + d0 + j];
      else if (kind == 2) sc = scale[row * (D / blk) + (d0 + j) / blk];
      else sc = scale[(((size_t)b * (S / blk) + s / blk) * H + h) * D + d0 + j];
      Elem<T>::store(out + e0 + j, e4m3_to_f32(c[j]) * sc);
    }
  }
}

// ---------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------
static int check_common(int B, int S, int H, int D, int layout, int s_pad) {
  LBFQ_REQUIRE(B > 0 && S > 0 && H > 0, LBFQ_ERR_ARG, "B, S, H must be positive; got %d %d %d", B, S, H);
  LBFQ_REQUIRE(D == 64 || D == 128, LBFQ_ERR_ARG, "tensor.shape[-1] must be 64 or 128; got %d", D);
  LBFQ_REQUIRE(layout >= 0 && layout <= 2, LBFQ_ERR_ARG, "bad layout code %d", layout);
  if (layout != LBFQ_LAYOUT_NHD)
    LBFQ_REQUIRE(s_pad >= S && s_pad % 16 == 0, LBFQ_ERR_ARG, "s_pad=%d must be >= S=%d and a multiple of 16", s_pad, S);
  return LBFQ_OK;
}

// zero the rows S..s_pad-1 of a BHSD / BHDS code tensor
static int zero_pad(uint8_t* codes, int layout, int B, int S, int H, int D, int s_pad, cudaStream_t st) {
  if (layout == LBFQ_LAYOUT_NHD || s_pad == S) return LBFQ_OK;
  if (layout == LBFQ_LAYOUT_BHSD) {
    LBFQ_CUDA_OK(cudaMemset2DAsync(codes + (size_t)S * D, (size_t)s_pad * D, 0, (size_t)(s_pad - S) * D,
                                   (size_t)B * H, st));
  } else {
    LBFQ_CUDA_OK(cudaMemset2DAsync(codes + S, (size_t)s_pad, 0, (size_t)(s_pad - S), (size_t)B * H * D, st));
  }
  return LBFQ_OK;
}

}  // namespace lbfq

using namespace lbfq;

namespace lbfq { int channel_scale_launch(float* scale, int n, cudaStream_t st); }

static int fp8_block_quant_impl(const void* x, int dtype, int B, int S, int H, int D, int block_s, const float* mean,
                                uint8_t* codes, int layout, int s_pad, float* scale, void* stream);

extern "C" int lbfq_fp8_block_quant(const void* x, int dtype, int B, int S, int H, int D, int block_s,
                                    uint8_t* codes, int layout, int s_pad, float* scale, void* stream) {
  return fp8_block_quant_impl(x, dtype, B, S, H, D, block_s, nullptr, codes, layout, s_pad, scale, stream);
}

extern "C" int lbfq_fp8_block_quant_centered(const void* x, int dtype, int B, int S, int H, int D, int block_s,
                                             const float* mean, uint8_t* codes, int layout, int s_pad, float* scale,
                                             void* stream) {
  LBFQ_REQUIRE(mean != nullptr, LBFQ_ERR_ARG, "fp8_block_quant_centered: mean (B, H, D) is required");
  return fp8_block_quant_impl(x, dtype, B, S, H, D, block_s, mean, codes, layout, s_pad, scale, stream);
}

static int fp8_block_quant_impl(const void* x, int dtype, int B, int S, int H, int D, int block_s, const float* mean,
                                uint8_t* codes, int layout, int s_pad, float* scale, void* stream) {
  if (int rc = check_common(B, S, H, D, layout, s_pad)) return rc;
  LBFQ_REQUIRE(block_s > 0 && S % block_s == 0, LBFQ_ERR_ARG, "S=%d must be divisible by block_s=%d", S, block_s);
  if (layout == LBFQ_LAYOUT_BHDS)
    LBFQ_REQUIRE(block_s % 16 == 0, LBFQ_ERR_UNSUPPORTED, "transposed code layout needs block_s %% 16 == 0; got %d", block_s);
  cudaStream_t st = (cudaStream_t)stream;
  CodeDst dst{codes, layout, S, H, D, s_pad};
  const int grid = B * (S / block_s) * H;
  LBFQ_DISPATCH_DTYPE(dtype, T,
      fp8_block_quant_kernel<T><<<grid, kThreads, 0, st>>>((const T*)x, dst, scale, block_s, mean));
  if (int rc = check_launch("fp8_block_quant")) return rc;
  return zero_pad(codes, layout, B, S, H, D, s_pad, st);
}

extern "C" int lbfq_mxfp8_v_quant(const void* x, int dtype, int B, int S, int H, int D, int block_s,
                                  uint8_t* codes, int layout, int s_pad, float* scale, void* stream) {
  if (int rc = check_common(B, S, H, D, layout, s_pad)) return rc;
  LBFQ_REQUIRE(block_s > 0 && S % block_s == 0, LBFQ_ERR_ARG, "S=%d must be divisible by block_s=%d", S, block_s);
  if (layout == LBFQ_LAYOUT_BHDS)
    LBFQ_REQUIRE(block_s % 16 == 0, LBFQ_ERR_UNSUPPORTED, "transposed code layout needs block_s %% 16 == 0; got %d", block_s);
  cudaStream_t st = (cudaStream_t)stream;
  CodeDst dst{codes, layout, S, H, D, s_pad};
  const int grid = B * (S / block_s) * H;
  LBFQ_DISPATCH_DTYPE(dtype, T,
      mxfp8_v_quant_kernel<T><<<grid, kThreads, 0, st>>>((const T*)x, dst, scale, block_s));
  if (int rc = check_launch("mxfp8_v_quant")) return rc;
  return zero_pad(codes, layout, B, S, H, D, s_pad, st);
}

extern "C" int lbfq_mxfp8_qk_quant(const void* x, int dtype, int B, int S, int H, int D, int block_d,
                                   uint8_t* codes, int layout, int s_pad, float* scale, uint8_t* scale_e8,
                                   void* stream) {
  if (int rc = check_common(B, S, H, D, layout, s_pad)) return rc;
  LBFQ_REQUIRE(block_d > 0 && D % block_d == 0, LBFQ_ERR_ARG, "D=%d must be divisible by block_d=%d", D, block_d);
  LBFQ_REQUIRE(block_d % 8 == 0 && (block_d & (block_d - 1)) == 0, LBFQ_ERR_UNSUPPORTED,
               "block_d must be a power of two >= 8; got %d", block_d);
  if (layout == LBFQ_LAYOUT_BHDS)
    LBFQ_REQUIRE(S % 16 == 0, LBFQ_ERR_UNSUPPORTED, "transposed code layout needs S %% 16 == 0; got %d", S);
  if (scale_e8) {
    LBFQ_REQUIRE(layout != LBFQ_LAYOUT_NHD && s_pad % 128 == 0, LBFQ_ERR_ARG, "scale_e8 needs a BH-major layout with s_pad %% 128 == 0");
    LBFQ_REQUIRE(D / block_d <= 4, LBFQ_ERR_UNSUPPORTED, "scale_e8 holds at most 4 groups per token; got %d", D / block_d);
  }
  cudaStream_t st = (cudaStream_t)stream;
  CodeDst dst{codes, layout, S, H, D, s_pad};
  const int grid = B * ((S + kMxRows - 1) / kMxRows) * H;
  if (scale_e8)                // biased exponent 127 (scale 1.0) wherever no token writes
    LBFQ_CUDA_OK(cudaMemsetAsync(scale_e8, 127, (size_t)B * H * s_pad * 4, st));
  LBFQ_DISPATCH_DTYPE(dtype, T,
      mxfp8_qk_quant_kernel<T><<<grid, kThreads, 0, st>>>((const T*)x, dst, scale, scale_e8, block_d));
  if (int rc = check_launch("mxfp8_qk_quant")) return rc;
  return zero_pad(codes, layout, B, S, H, D, s_pad, st);
}

extern "C" int lbfq_fp8_channel_quant(const void* x, int dtype, int B, int S, int H, int D,
                                      uint8_t* codes, int layout, int s_pad, float* scale, void* stream) {
  if (int rc = check_common(B, S, H, D, layout, s_pad)) return rc;
  if (layout == LBFQ_LAYOUT_BHDS)
    LBFQ_REQUIRE(S % 16 == 0, LBFQ_ERR_UNSUPPORTED, "transposed code layout needs S %% 16 == 0; got %d", S);
  cudaStream_t st = (cudaStream_t)stream;
  CodeDst dst{codes, layout, S, H, D, s_pad};
  // the scale buffer doubles as the amax accumulator (bit pattern of a float >= 0)
  LBFQ_CUDA_OK(cudaMemsetAsync(scale, 0, sizeof(float) * (size_t)B * H * D, st));
  const int grid_a = B * ((S + kChanRows - 1) / kChanRows) * H;
  LBFQ_DISPATCH_DTYPE(dtype, T,
      channel_amax_kernel<T><<<grid_a, kThreads, 0, st>>>((const T*)x, S, H, D, (unsigned int*)scale));
  if (int rc = check_launch("channel_amax")) return rc;
  if (int rc = channel_scale_launch(scale, B * H * D, st)) return rc;
  const int grid_q = B * ((S + kTChunk - 1) / kTChunk) * H;
  LBFQ_DISPATCH_DTYPE(dtype, T,
      channel_quant_kernel<T><<<grid_q, kThreads, 0, st>>>((const T*)x, dst, scale));
  if (int rc = check_launch("channel_quant")) return rc;
  return zero_pad(codes, layout, B, S, H, D, s_pad, st);
}

namespace lbfq {
int channel_scale_launch(float* scale, int n, cudaStream_t st) {
  channel_scale_kernel<<<(n + 255) / 256, 256, 0, st>>>(scale, n);
  return check_launch("channel_scale");
}
}  // namespace lbfq

static int dequant_launch(const uint8_t* codes, const float* scale, int B, int S, int H, int D, int kind,
                          int blk, void* out, int out_dtype, void* stream) {
  LBFQ_REQUIRE(D == 64 || D == 128, LBFQ_ERR_ARG, "fp8.shape[-1] must be 64 or 128; got %d", D);
  LBFQ_REQUIRE(blk > 0, LBFQ_ERR_ARG, "block size must be positive");
  cudaStream_t st = (cudaStream_t)stream;
  const size_t total = (size_t)B * S * H * D / kVec;
  const int grid = (int)((total + 255) / 256 < (size_t)sm_count() * 16 ? (total + 255) / 256 : (size_t)sm_count() * 16);
  LBFQ_DISPATCH_DTYPE(out_dtype, T,
      dequant_kernel<T><<<grid, 256, 0, st>>>(codes, scale, (T*)out, B, S, H, D, kind, blk));
  return check_launch("dequant");
}

extern "C" int lbfq_fp8_block_dequant(const uint8_t* codes, const float* scale, int B, int S, int H, int D,
                                      int block_s, void* out, int out_dtype, void* stream) {
  LBFQ_REQUIRE(block_s > 0 && S % block_s == 0, LBFQ_ERR_ARG, "S=%d must be divisible by block_s=%d", S, block_s);
  return dequant_launch(codes, scale, B, S, H, D, 0, block_s, out, out_dtype, stream);
}
extern "C" int lbfq_fp8_channel_dequant(const uint8_t* codes, const float* scale, int B, int S, int H, int D,
                                        void* out, int out_dtype, void* stream) {
  return dequant_launch(codes, scale, B, S, H, D, 1, 1, out, out_dtype, stream);
}
extern "C" int lbfq_mxfp8_qk_dequant(const uint8_t* codes, const float* scale, int B, int S, int H, int D,
                                     int block_d, void* out, int out_dtype, void* stream) {
  LBFQ_REQUIRE(block_d > 0 && D % block_d == 0, LBFQ_ERR_ARG, "D=%d must be divisible by block_d=%d", D, block_d);
  return dequant_launch(codes, scale, B, S, H, D, 2, block_d, out, out_dtype, stream);
}
extern "C" int lbfq_mxfp8_v_dequant(const uint8_t* codes, const float* scale, int B, int S, int H, int D,
                                    int block_s, void* out, int out_dtype, void* stream) {
  LBFQ_REQUIRE(block_s > 0 && S % block_s == 0, LBFQ_ERR_ARG, "S=%d must be divisible by block_s=%d", S, block_s);
  return dequant_launch(codes, scale, B, S, H, D, 3, block_s, out, out_dtype, stream);
}
