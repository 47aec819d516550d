// Fused preprocessing: permutation gather + smoothing + Hadamard rotation + quantisation in one pass.
//
// The reference prepares each of Q, K, V through a chain of full-tensor kernels and torch copies
// (src/low_bit_fake_quant/attention.py:166-239 and :505-591: k-means gather kmeans.py:89-90,126-135 -> smooth_k /
// group_mean_q / smooth_v_per_block preprocess.py:10-193 -> apply_qk_hadamard hadamard.py:77-117 -> a quantizer of
// quant_triton.py -> permute().contiguous()). Every step is row-local once the permutation and the per-channel
// statistics are known, so here one CTA takes a group of consecutive re-ordered rows of one (b, h) into shared memory
// (gathered through `order`), applies the same steps in the same order with the same intermediate roundings into the
// input dtype (preprocess.py:35,89,124; hadamard.py:46), and writes the e4m3 codes straight into the layout the
// attention kernel reads: 2 bytes read and 1 byte written per element, plus the small statistics. The column sums and
// the quantizer arithmetic are the very device functions of the separate kernels (tile_ops.cuh), so codes, scales and
// means are bit-identical to the unfused sequence (tests/test_gpu_prep_fused.py).
//
// Quantities that need all of S first stay separate passes: the K channel mean (lbfq_smooth_k with out = NULL) comes
// in as `chan_mean`; the per-channel amax of V is an extra pass of this kernel (stage LBFQ_PREP_STAGE_AMAX) that does
// everything but quantise.

#include <type_traits>

#include "tile_ops.cuh"

namespace lbfq {

int channel_scale_launch(float* scale, int n, cudaStream_t st);      // quant.cu: amax -> scale, in place

namespace {

struct PrepParams {
  const void* x;
  int B, S, H, D;
  const int64_t* order;        // (B*H, S) source row of each re-ordered row, or null
  const float* chan_mean;      // (B, H, D) subtracted from every row (K smoothing), or null
  int smooth_block;            // > 0: subtract the column mean of every `smooth_block` rows (Q groups, V blocks)
  float* block_mean;           // (B, S / smooth_block, H, D), written unless null
  const int8_t* signs;         // (H, D) +-1 for this call's heads, or null
  int hadamard;
  float had_scale;
  int kind;                    // LBFQ_PREP_*
  int stage;                   // channel kind: 0 = amax pass, 1 = quantising pass
  int scale_block;             // rows per scale (fp8_block, mxfp8_v) or channels per scale (mxfp8_qk)
  int group;                   // rows per CTA
  CodeDst dst;
  float* scale;
  uint8_t* scale_e8;
  void* smooth_out;            // NHD tensor of the input dtype receiving the prepared rows, or null
};

template <typename T>
__global__ void __launch_bounds__(kThreads)
prep_fused_kernel(const PrepParams p) {
  extern __shared__ __align__(16) uint8_t prep_smem[];
  T* tile = reinterpret_cast<T*>(prep_smem);                    // [group][D]
  __shared__ float buf[kThreads / 8][128 + 1];
  __shared__ float sums[128];
  __shared__ float red[kThreads / 32];
  __shared__ float s_scale;
  __shared__ __align__(16) uint8_t tbuf[128 * kTPitch];

  const int D = p.D, G = p.group;
  const int ngrp = p.S / G;
  const int grp = blockIdx.x % ngrp;
  const int h = (blockIdx.x / ngrp) % p.H;
  const int b = blockIdx.x / (ngrp * p.H);
  const int s0 = grp * G;
  const size_t bh = (size_t)b * p.H + h;
  const int tpr = D / kVec, rpi = kThreads / tpr;
  const int tr = threadIdx.x / tpr, d0 = (threadIdx.x % tpr) * kVec;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const T* x = reinterpret_cast<const T*>(p.x);

  // ---- gather the group's rows (kmeans.py:89-90 / apply_kv_permutation, kmeans.py:126-135) ---------------------
  {
    constexpr int kChunkElems = 16 / sizeof(T);                // elements per 16-byte copy
    const int cpr = D / kChunkElems;                           // copies per row
    // A row is 128 or 256 bytes somewhere in a (B, S, H, D) tensor: what hides the latency of such a gather is the
    // number of copies in flight. Eight row indices are fetched first, then eight asynchronous 16-byte copies go
    // straight from global to shared memory; nothing waits before the whole tile has been requested.
    constexpr int kBatch = 8;
    const int total = G * cpr;
    const uint32_t tile_s = (uint32_t)__cvta_generic_to_shared(tile);
    for (int base = threadIdx.x; base < total; base += kThreads * kBatch) {
      int64_t srow[kBatch];
#pragma unroll
      for (int u = 0; u < kBatch; ++u) {
        const int idx = base + u * kThreads;
        const int r = min(idx, total - 1) / cpr;
        srow[u] = p.order ? p.order[bh * p.S + s0 + r] : (int64_t)(s0 + r);
      }
#pragma unroll
      for (int u = 0; u < kBatch; ++u) {
        const int idx = base + u * kThreads;
        if (idx < total) {
          const int r = idx / cpr, c = idx % cpr;
          const T* src = x + (((size_t)b * p.S + srow[u]) * p.H + h) * D + c * kChunkElems;
          const uint32_t dst = tile_s + (uint32_t)(((size_t)r * D + c * kChunkElems) * sizeof(T));
          asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
        }
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
    asm volatile("cp.async.wait_group 0;" ::: "memory");
  }
  __syncthreads();

  // ---- K smoothing: x - mean over all of S, rounded into the input dtype (preprocess.py:29-35) -----------------
  if (p.chan_mean != nullptr) {
    const float* m = p.chan_mean + bh * D + d0;
    for (int r = tr; r < G; r += rpi) {
      float v[kVec];
      load8<T>(tile + (size_t)r * D + d0, v);
#pragma unroll
      for (int j = 0; j < kVec; ++j) v[j] = v[j] - m[j];
      store8<T>(tile + (size_t)r * D + d0, v);
    }
    __syncthreads();
  }

  // ---- Q group / V block smoothing: x - column mean of each `smooth_block` rows (preprocess.py:82-89,117-124) ---
  if (p.smooth_block > 0) {
    const int nsb = G / p.smooth_block;
    for (int sb = 0; sb < nsb; ++sb) {
      T* sub = tile + (size_t)sb * p.smooth_block * D;
      column_sums<T>(sub, (size_t)D, p.smooth_block, D, buf, sums);           // same order as block_mean_sub_kernel
      if (threadIdx.x < D) {
        const float m = sums[threadIdx.x] * rcp_approx((float)p.smooth_block);
        sums[threadIdx.x] = m;
        if (p.block_mean != nullptr)
          p.block_mean[(((size_t)b * (p.S / p.smooth_block) + (s0 / p.smooth_block + sb)) * p.H + h) * D + threadIdx.x] = m;
      }
      __syncthreads();
      for (int r = tr; r < p.smooth_block; r += rpi) {
        float v[kVec];
        load8<T>(sub + (size_t)r * D + d0, v);
#pragma unroll
        for (int j = 0; j < kVec; ++j) v[j] = v[j] - sums[d0 + j];
        store8<T>(sub + (size_t)r * D + d0, v);
      }
      __syncthreads();
    }
  }

  // ---- the prepared rows themselves, before the rotation, where something else needs them (the smoothed K of the score bias,
  // attention.py:573-591: the correction uses the un-rotated tensors) ----
  if (p.smooth_out != nullptr && p.stage == 1) {
    constexpr int kChunkElems = 16 / sizeof(T);
    const int cpr = D / kChunkElems;
    T* out = reinterpret_cast<T*>(p.smooth_out);
    for (int idx = threadIdx.x; idx < G * cpr; idx += kThreads) {
      const int r = idx / cpr, c = idx % cpr;
      *reinterpret_cast<uint4*>(out + (((size_t)b * p.S + s0 + r) * p.H + h) * D + c * kChunkElems) =
          *reinterpret_cast<const uint4*>(tile + (size_t)r * D + c * kChunkElems);
    }
  }

  // ---- Hadamard rotation of every row (hadamard.py:25-47,77-117), one warp per row ------------------------------
  if (p.hadamard) {
    auto rotate = [&](auto e_c) {
      constexpr int E = decltype(e_c)::value;
      const int8_t* sg = p.signs ? p.signs + (size_t)h * D + lane * E : nullptr;
      for (int r = warp; r < G; r += kThreads / 32) {
        T* row = tile + (size_t)r * D + lane * E;
        float v[E];
#pragma unroll
        for (int j = 0; j < E; ++j) v[j] = Elem<T>::load(row + j);
        hadamard_row<T, E>(v, sg, lane);
#pragma unroll
        for (int j = 0; j < E; ++j) Elem<T>::store(row + j, v[j] * p.had_scale);
      }
    };
    if (D == 128) rotate(std::integral_constant<int, 4>{});
    else rotate(std::integral_constant<int, 2>{});
    __syncthreads();
  }

  // ---- quantise (quant_triton.py) -------------------------------------------------------------------------------
  const CodeDst& dst = p.dst;
  if (p.kind == LBFQ_PREP_FP8_BLOCK) {
    const int nsc = G / p.scale_block;
    for (int sb = 0; sb < nsc; ++sb) {
      const T* sub = tile + (size_t)sb * p.scale_block * D;
      float amax = 0.f;
      for (int r = tr; r < p.scale_block; r += rpi) {
        float v[kVec];
        load8<T>(sub + (size_t)r * D + d0, v);
#pragma unroll
        for (int i = 0; i < kVec; ++i) amax = fmaxf(amax, fabsf(v[i]));
      }
      amax = warp_max(amax);
      if (lane == 0) red[warp] = amax;
      __syncthreads();
      if (threadIdx.x == 0) {
        float m = red[0];
#pragma unroll
        for (int i = 1; i < kThreads / 32; ++i) m = fmaxf(m, red[i]);
        const float sc = scale_from_amax(fmaxf(m, kAmaxFloor));
        s_scale = sc;
        p.scale[((size_t)b * (p.S / p.scale_block) + (s0 / p.scale_block + sb)) * p.H + h] = sc;
      }
      __syncthreads();
      const float rsc = rcp_approx(s_scale);
      store_tile(dst, b, h, s0 + sb * p.scale_block, p.scale_block, tbuf, [&](int r, int dd, float (&q)[kVec]) {
        float v[kVec];
        load8<T>(sub + (size_t)r * D + dd, v);
#pragma unroll
        for (int i = 0; i < kVec; ++i) q[i] = fminf(fmaxf(v[i] * rsc, -kFp8Max), kFp8Max);
      });
      __syncthreads();
    }
  } else if (p.kind == LBFQ_PREP_FP8_CHANNEL) {
    if (p.stage == 0) {
      // column amax of the group into the (B, H, D) accumulator (bit pattern of a float >= 0)
      float am[kVec];
#pragma unroll
      for (int i = 0; i < kVec; ++i) am[i] = 0.f;
      for (int r = tr; r < G; r += rpi) {
        float v[kVec];
        load8<T>(tile + (size_t)r * D + d0, v);
#pragma unroll
        for (int i = 0; i < kVec; ++i) am[i] = fmaxf(am[i], fabsf(v[i]));
      }
#pragma unroll
      for (int i = 0; i < kVec; ++i) buf[tr][d0 + i] = am[i];
      __syncthreads();
      if (threadIdx.x < D) {
        float m = 0.f;
        for (int r = 0; r < rpi; ++r) m = fmaxf(m, buf[r][threadIdx.x]);
        atomicMax(reinterpret_cast<unsigned int*>(p.scale) + bh * D + threadIdx.x, __float_as_uint(m));
      }
    } else {
      if (threadIdx.x < D) sums[threadIdx.x] = rcp_approx(p.scale[bh * D + threadIdx.x]);
      __syncthreads();
      store_tile(dst, b, h, s0, G, tbuf, [&](int r, int dd, float (&q)[kVec]) {
        float v[kVec];
        load8<T>(tile + (size_t)r * D + dd, v);
#pragma unroll
        for (int i = 0; i < kVec; ++i) q[i] = fminf(fmaxf(v[i] * sums[dd + i], -kFp8Max), kFp8Max);
      });
    }
  } else if (p.kind == LBFQ_PREP_MXFP8_V) {
    const int nsc = G / p.scale_block;
    for (int sb = 0; sb < nsc; ++sb) {
      const T* sub = tile + (size_t)sb * p.scale_block * D;
      float am[kVec];
#pragma unroll
      for (int i = 0; i < kVec; ++i) am[i] = 0.f;
      for (int r = tr; r < p.scale_block; r += rpi) {
        float v[kVec];
        load8<T>(sub + (size_t)r * D + d0, v);
#pragma unroll
        for (int i = 0; i < kVec; ++i) am[i] = fmaxf(am[i], fabsf(v[i]));
      }
#pragma unroll
      for (int i = 0; i < kVec; ++i) buf[tr][d0 + i] = am[i];
      __syncthreads();
      if (threadIdx.x < D) {
        float m = 0.f;
        for (int r = 0; r < rpi; ++r) m = fmaxf(m, buf[r][threadIdx.x]);
        const int e = pow2_scale_exp(fmaxf(m, kAmaxFloor));
        sums[threadIdx.x] = pow2f(-e);
        p.scale[(((size_t)b * (p.S / p.scale_block) + (s0 / p.scale_block + sb)) * p.H + h) * D + threadIdx.x] = pow2f(e);
      }
      __syncthreads();
      store_tile(dst, b, h, s0 + sb * p.scale_block, p.scale_block, tbuf, [&](int r, int dd, float (&q)[kVec]) {
        float v[kVec];
        load8<T>(sub + (size_t)r * D + dd, v);
#pragma unroll
        for (int i = 0; i < kVec; ++i) q[i] = fminf(fmaxf(v[i] * sums[dd + i], -kFp8Max), kFp8Max);
      });
      __syncthreads();
    }
  } else {   // LBFQ_PREP_MXFP8_QK: one power-of-two scale per row and `scale_block` channels
    constexpr int kPitch = 128 / kVec + 1;                    // floats per row of the reciprocal-scale table
    constexpr int kRowsPerPass = 128;                         // rows the table (the column-sum buffer) holds at a time
    static_assert(kRowsPerPass * kPitch <= (int)(sizeof(buf) / sizeof(float)), "reciprocal-scale table");
    float* grp_rcp = &buf[0][0];                              // [row][D / 8]: reciprocal scale of the group owning d0
    const int lanes = p.scale_block / kVec;                   // lanes sharing one scale (power of two, <= 16)
    const int ngr = D / p.scale_block;
    for (int r0 = 0; r0 < G; r0 += kRowsPerPass) {
      const int nrows = min(kRowsPerPass, G - r0);
      for (int rr = tr; rr < kRowsPerPass; rr += rpi) {       // uniform trip count: the shuffles stay converged
        const int r = r0 + rr;
        float am = 0.f;
        if (rr < nrows) {
          float v[kVec];
          load8<T>(tile + (size_t)r * D + d0, v);
#pragma unroll
          for (int i = 0; i < kVec; ++i) am = fmaxf(am, fabsf(v[i]));
        }
        for (int o = lanes >> 1; o > 0; o >>= 1) am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, o));
        if (rr < nrows) {
          const int e = pow2_scale_exp(fmaxf(am, kAmaxFloor));
          grp_rcp[rr * kPitch + d0 / kVec] = pow2f(-e);
          if ((d0 % p.scale_block) == 0) {
            const int g = d0 / p.scale_block;
            p.scale[(((size_t)b * p.S + s0 + r) * p.H + h) * ngr + g] = pow2f(e);
            if (p.scale_e8) {
              // the tile order of lbfq_mxfp8_qk_quant: byte (t % 32) * 16 + (t / 32) * 4 + g of a 128-token tile
              const int tok = s0 + r, tile128 = tok >> 7, tt = tok & 127;
              p.scale_e8[(bh * (dst.s_pad >> 7) + tile128) * 512 + (tt & 31) * 16 + (tt >> 5) * 4 + g] = (uint8_t)(e + 127);
            }
          }
        }
      }
      __syncthreads();
      store_tile(dst, b, h, s0 + r0, nrows, tbuf, [&](int r, int dd, float (&q)[kVec]) {
        float v[kVec];
        load8<T>(tile + (size_t)(r0 + r) * D + dd, v);
        const float rsc = grp_rcp[r * kPitch + dd / kVec];
#pragma unroll
        for (int i = 0; i < kVec; ++i) q[i] = fminf(fmaxf(v[i] * rsc, -kFp8Max), kFp8Max);
      });
      __syncthreads();
    }
  }
}

}  // namespace

}  // namespace lbfq

using namespace lbfq;

extern "C" int lbfq_prep_group_rows(int kind, int smooth_block, int scale_block, int S, int D, int dtype) {
  // rows per CTA: a multiple of the smoothing block and of the rows one scale covers, at least 64, and small enough
  // for the tile to fit in shared memory; 0 when no such group exists (the caller then runs the separate kernels)
  auto gcd = [](long long a, long long b) { while (b) { long long t = a % b; a = b; b = t; } return a; };
  long long g = 1;
  if (smooth_block > 0) g = smooth_block;
  if (kind == LBFQ_PREP_FP8_BLOCK || kind == LBFQ_PREP_MXFP8_V) {
    if (scale_block <= 0) return 0;
    g = g / gcd(g, scale_block) * scale_block;
  }
  while (g < 64 && S % (g * 2) == 0) g *= 2;
  if (kind == LBFQ_PREP_FP8_CHANNEL || kind == LBFQ_PREP_MXFP8_QK)
    while (g < 128 && S % (g * 2) == 0) g *= 2;
  const long long esz = dtype == LBFQ_F32 ? 4 : 2;
  if (g <= 0 || S % g != 0 || g % 16 != 0 || g * D * esz > 160 * 1024) return 0;
  return (int)g;
}

extern "C" int lbfq_prep_fused(const lbfq_prep_args* a, void* stream) {
  LBFQ_REQUIRE(a != nullptr && a->x != nullptr, LBFQ_ERR_ARG, "prep_fused: null input");
  LBFQ_REQUIRE(a->B > 0 && a->S > 0 && a->H > 0, LBFQ_ERR_ARG, "B, S, H must be positive; got %d %d %d", a->B, a->S, a->H);
  LBFQ_REQUIRE(a->D == 64 || a->D == 128, LBFQ_ERR_ARG, "tensor.shape[-1] must be 64 or 128; got %d", a->D);
  LBFQ_REQUIRE(a->kind >= LBFQ_PREP_FP8_BLOCK && a->kind <= LBFQ_PREP_MXFP8_QK, LBFQ_ERR_ARG, "bad kind %d", a->kind);
  LBFQ_REQUIRE(a->layout >= 0 && a->layout <= 2, LBFQ_ERR_ARG, "bad layout code %d", a->layout);
  if (a->layout != LBFQ_LAYOUT_NHD)
    LBFQ_REQUIRE(a->s_pad >= a->S && a->s_pad % 16 == 0, LBFQ_ERR_ARG, "s_pad=%d must be >= S=%d and a multiple of 16", a->s_pad, a->S);
  if (a->smooth_block > 0)
    LBFQ_REQUIRE(a->S % a->smooth_block == 0, LBFQ_ERR_ARG, "S=%d must be divisible by block_s=%d", a->S, a->smooth_block);
  if (a->kind == LBFQ_PREP_FP8_BLOCK || a->kind == LBFQ_PREP_MXFP8_V)
    LBFQ_REQUIRE(a->scale_block > 0 && a->S % a->scale_block == 0, LBFQ_ERR_ARG, "S=%d must be divisible by block_s=%d", a->S, a->scale_block);
  if (a->kind == LBFQ_PREP_MXFP8_QK) {
    LBFQ_REQUIRE(a->scale_block > 0 && a->D % a->scale_block == 0, LBFQ_ERR_ARG, "D=%d must be divisible by block_d=%d", a->D, a->scale_block);
    LBFQ_REQUIRE(a->scale_block % 8 == 0 && (a->scale_block & (a->scale_block - 1)) == 0, LBFQ_ERR_UNSUPPORTED,
                 "block_d must be a power of two >= 8; got %d", a->scale_block);
    if (a->scale_e8) {
      LBFQ_REQUIRE(a->layout != LBFQ_LAYOUT_NHD && a->s_pad % 128 == 0, LBFQ_ERR_ARG, "scale_e8 needs a BH-major layout with s_pad %% 128 == 0");
      LBFQ_REQUIRE(a->D / a->scale_block <= 4, LBFQ_ERR_UNSUPPORTED, "scale_e8 holds at most 4 groups per token; got %d", a->D / a->scale_block);
    }
  }
  const int group = lbfq_prep_group_rows(a->kind, a->smooth_block, a->scale_block, a->S, a->D, a->dtype);
  LBFQ_REQUIRE(group > 0, LBFQ_ERR_UNSUPPORTED, "prep_fused: no row group fits shared memory for these block sizes");
  LBFQ_REQUIRE(a->codes != nullptr && a->scale != nullptr, LBFQ_ERR_ARG, "prep_fused: codes and scale are required");
  cudaStream_t st = (cudaStream_t)stream;
  PrepParams p{};
  p.x = a->x; p.B = a->B; p.S = a->S; p.H = a->H; p.D = a->D;
  p.order = a->order; p.chan_mean = a->chan_mean; p.smooth_block = a->smooth_block; p.block_mean = a->block_mean;
  p.signs = a->signs; p.hadamard = a->hadamard; p.had_scale = a->had_scale;
  p.kind = a->kind; p.scale_block = a->scale_block; p.group = group;
  p.dst = CodeDst{a->codes, a->layout, a->S, a->H, a->D, a->s_pad};
  p.scale = a->scale; p.scale_e8 = a->scale_e8; p.smooth_out = a->smooth_out;
  const size_t esz = a->dtype == LBFQ_F32 ? 4 : 2;
  const int smem = (int)((size_t)group * a->D * esz);
  const int grid = a->B * a->H * (a->S / group);
  auto run = [&](int stage) -> int {
    p.stage = stage;
    LBFQ_DISPATCH_DTYPE(a->dtype, T, {
      auto kern = prep_fused_kernel<T>;
      // static (column-sum and staging buffers) + dynamic (the tile) exceed the 48 KB a kernel gets without opting in
      LBFQ_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
      kern<<<grid, kThreads, smem, st>>>(p);
    });
    return check_launch("prep_fused");
  };
  if (a->kind == LBFQ_PREP_MXFP8_QK && a->scale_e8)          // biased exponent 127 (scale 1.0) wherever no token writes
    LBFQ_CUDA_OK(cudaMemsetAsync(a->scale_e8, 127, (size_t)a->B * a->H * a->s_pad * 4, st));
  if (a->kind == LBFQ_PREP_FP8_CHANNEL) {
    // the scale buffer doubles as the amax accumulator; the block means are written by the first pass only
    LBFQ_CUDA_OK(cudaMemsetAsync(a->scale, 0, sizeof(float) * (size_t)a->B * a->H * a->D, st));
    if (int rc = run(0)) return rc;
    if (int rc = channel_scale_launch(a->scale, a->B * a->H * a->D, st)) return rc;
    p.block_mean = nullptr;
    if (int rc = run(1)) return rc;
  } else {
    if (int rc = run(1)) return rc;
  }
  // zero the rows S..s_pad-1 of a BHSD / BHDS code tensor
  if (a->layout != LBFQ_LAYOUT_NHD && a->s_pad != a->S) {
    if (a->layout == LBFQ_LAYOUT_BHSD) {
      LBFQ_CUDA_OK(cudaMemset2DAsync(a->codes + (size_t)a->S * a->D, (size_t)a->s_pad * a->D, 0, (size_t)(a->s_pad - a->S) * a->D,
                                     (size_t)a->B * a->H, st));
    } else {
      LBFQ_CUDA_OK(cudaMemset2DAsync(a->codes + a->S, (size_t)a->s_pad, 0, (size_t)(a->s_pad - a->S), (size_t)a->B * a->H * a->D, st));
    }
  }
  return LBFQ_OK;
}
