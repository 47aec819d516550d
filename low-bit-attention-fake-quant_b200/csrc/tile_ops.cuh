// Tile-level building blocks shared by the quantizers, the smoothing kernels and their fused forms: 8-element
// accesses along D, column sums in one fixed order (so that a fused kernel reproduces the separate kernels' means bit
// for bit), and the stores of e4m3 codes into the NHD / BHSD / transposed BHDS layouts.
#pragma once

#include "common.cuh"

namespace lbfq {

constexpr int kThreads = 256;
constexpr int kVec = 8;          // elements of D per thread access
constexpr int kTChunk = 128;     // tokens staged per transposed store: 128-byte rows of the transposed codes
constexpr int kTPitch = kTChunk + 4;   // bytes between the channels' rows in the staging buffer

template <typename T>
__device__ __forceinline__ void load8(const T* p, float (&v)[kVec]) {
#pragma unroll
  for (int i = 0; i < kVec; ++i) v[i] = Elem<T>::load(p + i);
}
template <>
__device__ __forceinline__ void load8<__nv_bfloat16>(const __nv_bfloat16* p, float (&v)[kVec]) {
  uint4 raw = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 f = __bfloat1622float2(h[i]);
    v[2 * i] = f.x;
    v[2 * i + 1] = f.y;
  }
}
template <>
__device__ __forceinline__ void load8<__half>(const __half* p, float (&v)[kVec]) {
  uint4 raw = *reinterpret_cast<const uint4*>(p);
  const __half2* h = reinterpret_cast<const __half2*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 f = __half22float2(h[i]);
    v[2 * i] = f.x;
    v[2 * i + 1] = f.y;
  }
}
template <>
__device__ __forceinline__ void load8<float>(const float* p, float (&v)[kVec]) {
  float4 a = *reinterpret_cast<const float4*>(p);
  float4 b = *reinterpret_cast<const float4*>(p + 4);
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
  v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}

__device__ __forceinline__ uint2 pack8(const float (&q)[kVec]) {
  uint32_t lo = (uint32_t)f32x2_to_e4m3x2(q[0], q[1]) | ((uint32_t)f32x2_to_e4m3x2(q[2], q[3]) << 16);
  uint32_t hi = (uint32_t)f32x2_to_e4m3x2(q[4], q[5]) | ((uint32_t)f32x2_to_e4m3x2(q[6], q[7]) << 16);
  return make_uint2(lo, hi);
}

struct CodeDst {
  uint8_t* base;
  int layout;
  int S, H, D, s_pad;
};

// Store the codes of rows [s0, s0 + nrows) of slab (b, h); `quant(r, d0, q)`
// 4 x 4 byte transpose: a0..a3 hold bytes [c0 c1 c2 c3] of tokens 0..3; out[c] = [t0 t1 t2 t3] of channel c
__device__ __forceinline__ void transpose4x4(uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t* out) {
  const uint32_t t0 = __byte_perm(a0, a1, 0x5140), t1 = __byte_perm(a2, a3, 0x5140);   // channels 0, 1 of two tokens
  const uint32_t t2 = __byte_perm(a0, a1, 0x7362), t3 = __byte_perm(a2, a3, 0x7362);   // channels 2, 3
  out[0] = __byte_perm(t0, t1, 0x5410);
  out[1] = __byte_perm(t0, t1, 0x7632);
  out[2] = __byte_perm(t2, t3, 0x5410);
  out[3] = __byte_perm(t2, t3, 0x7632);
}

// fills the 8 quantised-and-clamped fp32 values of row r, columns d0..d0+7.
// NHD / BHSD are written directly (8-byte stores); BHDS goes through a
// shared-memory transpose so that global stores stay 16 bytes wide.
template <typename QuantFn>
__device__ __forceinline__ void store_tile(const CodeDst& dst, int b, int h, int s0, int nrows,
                                           uint8_t* tbuf, QuantFn quant) {
  const int D = dst.D;
  const int tpr = D / kVec;                   // threads per row
  const int rows_per_iter = kThreads / tpr;
  const int tr = threadIdx.x / tpr;
  const int d0 = (threadIdx.x % tpr) * kVec;
  if (dst.layout != LBFQ_LAYOUT_BHDS) {
    for (int r = tr; r < nrows; r += rows_per_iter) {
      float q[kVec];
      quant(r, d0, q);
      size_t off = dst.layout == LBFQ_LAYOUT_NHD
                       ? (((size_t)b * dst.S + (s0 + r)) * dst.H + h) * D + d0
                       : (((size_t)b * dst.H + h) * dst.s_pad + (s0 + r)) * D + d0;
      *reinterpret_cast<uint2*>(dst.base + off) = pack8(q);
    }
    return;
  }
  // Transposed layout: the codes of up to kTChunk tokens go through shared memory as [channel][token]. A thread
  // quantises four consecutive tokens of its eight channels and transposes the 4 x 8 bytes in registers
  // (byte permutes), so that it stores one 32-bit word per channel instead of four single bytes.
  for (int c0 = 0; c0 < nrows; c0 += kTChunk) {
    const int cn = min(kTChunk, nrows - c0);           // a multiple of 16 (checked on the host)
    for (int qd = tr; qd * 4 < cn; qd += rows_per_iter) {
      uint2 pk[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float q[kVec];
        quant(c0 + qd * 4 + j, d0, q);
        pk[j] = pack8(q);
      }
      uint32_t w[8];
      transpose4x4(pk[0].x, pk[1].x, pk[2].x, pk[3].x, w);
      transpose4x4(pk[0].y, pk[1].y, pk[2].y, pk[3].y, w + 4);
#pragma unroll
      for (int i = 0; i < kVec; ++i) *reinterpret_cast<uint32_t*>(tbuf + (d0 + i) * kTPitch + qd * 4) = w[i];
    }
    __syncthreads();
    // 16-byte row segments, read back as four words (the pitch keeps rows a word, not 16 bytes, apart)
    const int segs = cn / 16;
    for (int idx = threadIdx.x; idx < D * segs; idx += kThreads) {
      int d = idx / segs, sg = idx % segs;
      const uint32_t* src = reinterpret_cast<const uint32_t*>(tbuf + d * kTPitch + sg * 16);
      uint4 val = make_uint4(src[0], src[1], src[2], src[3]);
      size_t off = (((size_t)b * dst.H + h) * D + d) * dst.s_pad + (s0 + c0 + sg * 16);
      *reinterpret_cast<uint4*>(dst.base + off) = val;
    }
    __syncthreads();
  }
}

template <typename T>
__device__ __forceinline__ void store8(T* p, const float (&v)[kVec]) {
#pragma unroll
  for (int i = 0; i < kVec; ++i) Elem<T>::store(p + i, v[i]);
}
template <>
__device__ __forceinline__ void store8<__nv_bfloat16>(__nv_bfloat16* p, const float (&v)[kVec]) {
  uint4 raw;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
  *reinterpret_cast<uint4*>(p) = raw;
}

// ---- column sums of a row range of one (b, h), reduced in a fixed order -----
template <typename T>
__device__ __forceinline__ void column_sums(const T* src, size_t rstride, int nrows, int D,
                                            float (*buf)[128 + 1], float* out /* smem[D] */) {
  const int tpr = D / kVec, rpi = kThreads / tpr;
  const int tr = threadIdx.x / tpr, d0 = (threadIdx.x % tpr) * kVec;
  float acc[kVec];
#pragma unroll
  for (int i = 0; i < kVec; ++i) acc[i] = 0.f;
  for (int r = tr; r < nrows; r += rpi) {
    float v[kVec];
    load8<T>(src + r * rstride + d0, v);
#pragma unroll
    for (int i = 0; i < kVec; ++i) acc[i] += v[i];
  }
#pragma unroll
  for (int i = 0; i < kVec; ++i) buf[tr][d0 + i] = acc[i];
  __syncthreads();
  if (threadIdx.x < D) {
    float s = 0.f;
    for (int r = 0; r < rpi; ++r) s += buf[r][threadIdx.x];
    out[threadIdx.x] = s;
  }
  __syncthreads();
}


// One row of the Hadamard rotation held by a warp (E = D / 32 elements per lane): optional signs (rounded through T as
// the reference's `x * signs.to(x.dtype)` is), butterflies in the reference's order (stride 1, 2, 4, ...), the caller
// scales and rounds (src/low_bit_fake_quant/hadamard.py:25-47).
template <typename T, int E>
__device__ __forceinline__ void hadamard_row(float (&v)[E], const int8_t* sg /* this lane's E signs, or null */, int lane) {
  if (sg) {
#pragma unroll
    for (int j = 0; j < E; ++j) v[j] = round_through<T>(v[j] * (float)sg[j]);
  }
#pragma unroll
  for (int st = 1; st < E; st <<= 1) {
#pragma unroll
    for (int j = 0; j < E; ++j) {
      if ((j & st) == 0) {
        float a = v[j], b = v[j + st];
        v[j] = a + b;
        v[j + st] = a - b;
      }
    }
  }
#pragma unroll
  for (int m = 1; m < 32; m <<= 1) {
    const bool upper = (lane & m) != 0;
#pragma unroll
    for (int j = 0; j < E; ++j) {
      float other = __shfl_xor_sync(0xffffffffu, v[j], m);
      v[j] = upper ? (other - v[j]) : (v[j] + other);
    }
  }
}

}  // namespace lbfq
