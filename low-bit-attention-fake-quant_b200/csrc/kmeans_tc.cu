// k-means assignment on the tensor cores (BF16 tokens).
//
// argmin_c |c|^2 - 2 x.c needs the (tokens x centroids) Gram block x.c^T: a GEMM with M = tokens, N = k <= 64,
// K = D. The tokens are BF16 already; the FP32 centroids are split into three BF16 pieces
// (c = hi + mid + lo to 24 bits), so that x.c = x.hi + x.mid + x.lo is accumulated from exact BF16 x BF16
// products in FP32 -- the same value as the FP32 FFMA kernel up to summation order. One CTA walks a few
// consecutive 128-token tiles of one (b, h): TMA brings the 3 x 64 centroid rows once and the token tiles (two
// 64-channel panels, 128B swizzle) through a double buffer, one thread issues 3 x D/16 tcgen05.mma.kind::f16 per tile
// into one of two 64-column TMEM buffers, then thread == token reads its row of dot products back and takes the
// argmin (lowest index on ties, as the FFMA kernel does). The kernel is bound by reading the tokens once per Lloyd
// iteration (HBM / L2), not by arithmetic.
#include "attn_prims.cuh"
#include "kmeans_tc.h"

namespace lbfq {

using namespace attn;

namespace {

constexpr int kTcTok = 128;      // tokens per CTA (MMA M)
constexpr int kTcCen = 64;       // centroid rows per piece (MMA N), zero-padded above k

__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* map, int c0, int c1, int c2, int c3, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];"
      ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(bar) : "memory");
}
// (BH, k, D) fp32 -> (BH, 3, 64, D) bf16 pieces, rows >= k zero
__global__ void split_centroids_kernel(const float* __restrict__ cent, int BH, int k, int D, __nv_bfloat16* __restrict__ out) {
  const size_t total = (size_t)BH * kTcCen * D;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const int d = (int)(i % D);
    const int c = (int)((i / D) % kTcCen);
    const size_t bh = i / D / kTcCen;
    float v = c < k ? cent[(bh * k + c) * D + d] : 0.f;
    const __nv_bfloat16 hi = __float2bfloat16_rn(v);
    v -= __bfloat162float(hi);
    const __nv_bfloat16 mid = __float2bfloat16_rn(v);
    v -= __bfloat162float(mid);
    const __nv_bfloat16 lo = __float2bfloat16_rn(v);
    __nv_bfloat16* o = out + (bh * 3 * kTcCen + c) * D + d;
    o[0] = hi;
    o[(size_t)kTcCen * D] = mid;
    o[(size_t)2 * kTcCen * D] = lo;
  }
}

// centroids from the per-chunk sums and counts the assignment-with-sums kernel leaves behind (chunks added in order),
// their squared norms, and their three BF16 pieces for the next assignment
__global__ void __launch_bounds__(128)
chunk_mean_kernel(const float* __restrict__ psum, const int32_t* __restrict__ hist, int D, int k, int nchunk,
                  float* __restrict__ cent, float* __restrict__ cnorm, __nv_bfloat16* __restrict__ split) {
  __shared__ float red[4];
  const int c = blockIdx.x % k;
  const size_t bh = blockIdx.x / k;
  int n = 0;
  for (int ch = 0; ch < nchunk; ++ch) n += hist[(bh * nchunk + ch) * kTcCen + c];
  if (n == 0) return;                               // empty cluster keeps centroid, norm and pieces
  float v = 0.f;
  if (threadIdx.x < D) {
    float s = 0.f;
    for (int ch = 0; ch < nchunk; ++ch) s += psum[((bh * nchunk + ch) * k + c) * D + threadIdx.x];
    v = __fdiv_rn(s, (float)n);
    cent[(bh * k + c) * D + threadIdx.x] = v;
    float r = v;
    const __nv_bfloat16 hi = __float2bfloat16_rn(r);
    r -= __bfloat162float(hi);
    const __nv_bfloat16 mid = __float2bfloat16_rn(r);
    r -= __bfloat162float(mid);
    const __nv_bfloat16 lo = __float2bfloat16_rn(r);
    __nv_bfloat16* o = split + (bh * 3 * kTcCen + c) * D + threadIdx.x;
    o[0] = hi;
    o[(size_t)kTcCen * D] = mid;
    o[(size_t)2 * kTcCen * D] = lo;
  }
  float s2 = v * v;
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) s2 += __shfl_xor_sync(0xffffffffu, s2, off);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s2;
  __syncthreads();
  if (threadIdx.x == 0) cnorm[bh * k + c] = red[0] + red[1] + red[2] + red[3];
}

// One CTA walks kTcTiles consecutive 128-token tiles of one (b, h): the centroid pieces are loaded once, the token
// tiles go through two shared-memory buffers and two 64-column TMEM buffers. A producer warp (one thread) issues the
// TMA loads two tiles ahead and the MMAs; four consumer warps take the argmin of a tile while the next one is being
// multiplied. No CTA-wide barrier inside the loop: a TMEM buffer is handed back through an mbarrier the 128
// consumer threads arrive on, a shared-memory buffer through the MMAs' own commit.
constexpr int kTcTiles = 8;
constexpr int kTcWarps = 4;                        // consumer warps (128 tokens); one more warp loads and issues
constexpr int kTcThreads = (kTcWarps + 1) * 32;

template <int D>
__global__ void __launch_bounds__(kTcThreads)
assign_tc_kernel(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_c, int S, int H, int k,
                 const float* __restrict__ cnorm, int32_t* __restrict__ labels, int32_t* __restrict__ hist,
                 int32_t* __restrict__ status) {
  constexpr int NP = D / 64;                         // 64-channel panels (one 128-byte swizzle row each)
  constexpr int kA = kTcTok * 128;                   // bytes per token panel
  constexpr int kB = 3 * kTcCen * 128;               // bytes per centroid panel (three pieces)
  // The swizzled tiles want a 1 KB-aligned base, which the declared alignment of the dynamic shared-memory array
  // provides; no slack is allocated for rounding up (two CTAs of 112 KB share an SM), so a base that is not
  // aligned is refused below instead of being rounded.
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = smem_raw;
  const uint32_t sbase = smem_u32(smem);
  const uint32_t offA = 0, offB = 2 * NP * kA, offBar = offB + NP * kB;
  auto bar_full = [&](int buf) { return sbase + offBar + 8u * buf; };          // token tile (and, first, centroids) landed
  auto bar_done = [&](int buf) { return sbase + offBar + 16u + 8u * buf; };    // MMAs of the tile in this buffer done
  auto bar_tfree = [&](int buf) { return sbase + offBar + 32u + 8u * buf; };   // the tile's TMEM buffer has been read out
  volatile int* misc = (volatile int*)(smem + offBar + 48);       // [0] tmem base, [1] abort
  volatile int* abort_flag = misc + 1;
  // labels of this CTA's tokens, counted for the sort that follows (kept in the dynamic area: a static array would
  // push the 1 KB-aligned dynamic base up and cost the second CTA per SM)
  int* cnt = reinterpret_cast<int*>(smem + offBar + 64);

  const int ntile = (S + kTcTok - 1) / kTcTok;
  const int per_bh = (ntile + kTcTiles - 1) / kTcTiles;
  // heads vary fastest over the grid: the CTAs in flight together read the same token rows of the (B, S, H, D) input,
  // head by head, so each DRAM page is used whole while it is open
  const int h = blockIdx.x % H;
  const int tile0 = ((blockIdx.x / H) % per_bh) * kTcTiles;
  const int b = blockIdx.x / (H * per_bh);
  const int bh = b * H + h;
  const int n = min(kTcTiles, ntile - tile0);        // tiles of this CTA (>= 1)
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if ((sbase & 1023u) != 0) {
    // never expected: reported through the status word (the labels keep the valid values they held)
    if (threadIdx.x == 0 && status != nullptr) atomicCAS(status, 0, 55);
    return;
  }

  if (threadIdx.x < kTcCen) cnt[threadIdx.x] = 0;
  if (threadIdx.x == 0) {
    mbar_init(bar_full(0), 1);
    mbar_init(bar_full(1), 1);
    mbar_init(bar_done(0), 1);
    mbar_init(bar_done(1), 1);
    mbar_init(bar_tfree(0), kTcWarps * 32);
    mbar_init(bar_tfree(1), kTcWarps * 32);
    misc[1] = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 128;" ::"r"(sbase + offBar + 48) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = (uint32_t)misc[0];

  auto load_tile = [&](int i) {                       // thread 0: token tile i of this CTA into buffer i & 1
    const int buf = i & 1;
#pragma unroll
    for (int pn = 0; pn < NP; ++pn)
      tma_load_4d(sbase + offA + (buf * NP + pn) * kA, &tm_x, pn * 64, h, (tile0 + i) * kTcTok, b, bar_full(buf));
  };
  auto issue_mma = [&](int i) -> bool {               // thread 0: Gram block of tile i into TMEM buffer i & 1
    const int buf = i & 1;
    if (!mbar_wait(bar_full(buf), (uint32_t)((i >> 1) & 1), abort_flag, status, 51)) return false;
    tc_fence_after();
    const uint32_t idesc = make_idesc_bf16(kTcCen);
    bool first = true;
#pragma unroll
    for (int pc = 0; pc < 3; ++pc)
#pragma unroll
      for (int pn = 0; pn < NP; ++pn) {
        const uint64_t da = make_desc(sbase + offA + (buf * NP + pn) * kA, 128);
        const uint64_t db = make_desc(sbase + offB + pn * kB + pc * (kTcCen * 128), 128);
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) {
          mma_bf16_ss(tmem + buf * kTcCen, da + (uint64_t)(ks * 2), db + (uint64_t)(ks * 2), idesc, first ? 0u : 1u);
          first = false;
        }
      }
    tc_commit(bar_done(buf));
    return true;
  };

  if (warp == kTcWarps) {
    // ---- producer: TMA loads and MMA issue, one thread ----
    if (lane == 0) {
      mbar_expect_tx(bar_full(0), NP * (kA + kB));
#pragma unroll
      for (int pn = 0; pn < NP; ++pn) tma_load_3d(sbase + offB + pn * kB, &tm_c, pn * 64, 0, bh, bar_full(0));
      load_tile(0);
      if (n > 1) {
        mbar_expect_tx(bar_full(1), NP * kA);
        load_tile(1);
      }
      for (int i = 0; i < n; ++i) {
        const int buf = i & 1;
        // the TMEM buffer is free once every consumer thread has read tile i - 2 out of it
        if (i >= 2 && !mbar_wait(bar_tfree(buf), (uint32_t)(((i - 2) >> 1) & 1), abort_flag, status, 53)) break;
        if (!issue_mma(i)) break;
        if (i + 2 < n) {
          // the tile's shared-memory buffer is free once its MMAs have completed: refill it two tiles ahead
          if (!mbar_wait(bar_done(buf), (uint32_t)((i >> 1) & 1), abort_flag, status, 54)) break;
          mbar_expect_tx(bar_full(buf), NP * kA);
          load_tile(i + 2);
        }
      }
    }
  } else {
    // ---- consumers: thread == token == TMEM lane ----
    // |c|^2 of the slab's centroids, once per CTA; +inf above k, so that the argmin needs no bound check
    float cn[kTcCen];
#pragma unroll
    for (int c = 0; c < kTcCen; ++c) cn[c] = c < k ? cnorm[(size_t)bh * k + c] : INFINITY;
    for (int i = 0; i < n; ++i) {
      const int buf = i & 1;
      const bool ok = mbar_wait(bar_done(buf), (uint32_t)((i >> 1) & 1), abort_flag, status, 52);
      if (!__all_sync(0xffffffffu, ok)) break;           // a given-up wait ends every role's loop
      tc_fence_after();
      const uint32_t trow = tmem + buf * kTcCen + ((uint32_t)(warp * 32) << 16);
      uint32_t r0[32], r1[32];
      LBFQ_TMEM_LD32(r0, trow);
      LBFQ_TMEM_LD32(r1, trow + 32);
      tc_wait_ld();
      tc_fence_before();
      mbar_arrive(bar_tfree(buf));                       // the dot products are in registers
      float best = INFINITY;
      int best_i = 0;
#pragma unroll
      for (int c = 0; c < 32; ++c) {
        const float dist = cn[c] - 2.0f * __uint_as_float(r0[c]);
        if (dist < best) { best = dist; best_i = c; }            // ascending c: lowest index wins ties
      }
#pragma unroll
      for (int c = 0; c < 32; ++c) {
        const float dist = cn[32 + c] - 2.0f * __uint_as_float(r1[c]);
        if (dist < best) { best = dist; best_i = 32 + c; }
      }
      const int tok = (tile0 + i) * kTcTok + warp * 32 + lane;
      if (tok < S) {
        labels[(size_t)bh * S + tok] = best_i;
        atomicAdd(&cnt[best_i], 1);
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  // per-label counts of this CTA's chunk of kTcTiles * 128 tokens: (bh, chunk, 64)
  if (hist != nullptr && threadIdx.x < kTcCen)
    hist[((size_t)bh * per_bh + tile0 / kTcTiles) * kTcCen + threadIdx.x] = cnt[threadIdx.x];
  if (warp == 0) {
    if (*abort_flag && lane == 0) {
      // give in-flight bulk copies a bounded time to land before the CTA retires
      const long long t0 = wall_ns();
      while (wall_ns() - t0 < 1000000ll) { }
    }
    __syncwarp();
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 128;" ::"r"(tmem) : "memory");
  }
}

// ---------------------------------------------------------------------------------------------------------------
// Assignment and, in the same pass over the tokens, the sums the centroid update needs (D = 128).
//
// sums^T (channels x clusters) += tokens^T (channels x tokens) . onehot (tokens x clusters) is one more GEMM over the
// token tile that is in shared memory anyway: A is the tile read MN-major (channels contiguous: the two 64-channel
// panels TMA delivered are its two 64-wide groups), B a 128 x 64 BF16 tile in which the thread of each token sets a
// single 1.0 at its label. The products are exact (token x 1.0), the sums FP32, accumulated over the CTA's tiles in
// 64 more TMEM columns and written out once per CTA as (chunk, cluster, channel) partial sums; a small kernel adds
// the chunks in a fixed order and divides by the counts. That replaces the sort by label and the gather of the sorted
// rows in every Lloyd iteration. One CTA per SM: four token buffers, two consumer groups of 128 threads (tile i
// belongs to group i & 1), one producer thread.
constexpr int kSumBufs = 4;
constexpr int kSumThreads = (2 * 4 + 1) * 32;

// shared-memory descriptor of an MN-major operand in 128-byte-swizzled rows: 64 elements (128 bytes) of the M / N
// extent are contiguous, eight consecutive K rows form a 1 KB swizzle atom (stride between atoms along K: 1 KB),
// `lead_bytes` separates the 64-wide groups of the M / N extent
__device__ __forceinline__ uint64_t make_desc_mn(uint32_t saddr, uint32_t lead_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr >> 4) & 0x3fffu);
  d |= (uint64_t)((lead_bytes >> 4) & 0x3fffu) << 16;
  d |= (uint64_t)((1024u >> 4) & 0x3fffu) << 32;
  d |= (uint64_t)1 << 46;
  d |= 2ull << 61;
  return d;
}

__global__ void __launch_bounds__(kSumThreads)
assign_sum_tc_kernel(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_c, int S, int H, int k,
                     int tiles_per_cta, const float* __restrict__ cnorm, int32_t* __restrict__ labels, int32_t* __restrict__ hist,
                     float* __restrict__ psum, int32_t* __restrict__ status) {
  constexpr int D = 128, NP = 2;
  constexpr int kA = kTcTok * 128;                   // bytes per token panel
  constexpr int kB = 3 * kTcCen * 128;               // bytes per centroid panel (three pieces)
  constexpr int kOH = kTcTok * 128;                  // bytes of a one-hot tile (128 tokens x 64 clusters, BF16)
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = smem_raw;
  const uint32_t sbase = smem_u32(smem);
  constexpr uint32_t offA = 0, offB = kSumBufs * NP * kA, offOH = offB + NP * kB, offBar = offOH + 2 * kOH;
  auto bar_full = [&](int buf) { return sbase + offBar + 8u * buf; };            // token tile (and, first, centroids) landed
  auto bar_gdone = [&](int g) { return sbase + offBar + 32u + 8u * g; };         // Gram block of the group's tile done
  auto bar_tfree = [&](int g) { return sbase + offBar + 48u + 8u * g; };         // ... and read out of tensor memory
  auto bar_oh = [&](int g) { return sbase + offBar + 64u + 8u * g; };            // the group's one-hot tile is written
  auto bar_sdone = [&](int g) { return sbase + offBar + 80u + 8u * g; };         // the sums of the group's tile are done
  volatile int* misc = (volatile int*)(smem + offBar + 96);                       // [0] tmem base, [1] abort
  volatile int* abort_flag = misc + 1;
  int* cnt = reinterpret_cast<int*>(smem + offBar + 112);

  const int ntile = (S + kTcTok - 1) / kTcTok;
  const int per_bh = (ntile + tiles_per_cta - 1) / tiles_per_cta;
  const int h = blockIdx.x % H;
  const int chunk = (blockIdx.x / H) % per_bh;
  const int tile0 = chunk * tiles_per_cta;
  const int b = blockIdx.x / (H * per_bh);
  const int bh = b * H + h;
  const int n = min(tiles_per_cta, ntile - tile0);   // tiles of this CTA (>= 1)
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if ((sbase & 1023u) != 0) {
    if (threadIdx.x == 0 && status != nullptr) atomicCAS(status, 0, 55);
    return;
  }
  if (threadIdx.x < kTcCen) cnt[threadIdx.x] = 0;
  if (threadIdx.x == 0) {
    for (int i = 0; i < kSumBufs; ++i) mbar_init(bar_full(i), 1);
    for (int g = 0; g < 2; ++g) {
      mbar_init(bar_gdone(g), 1);
      mbar_init(bar_tfree(g), 4);                    // one arrival per warp of the group
      mbar_init(bar_oh(g), 4);
      mbar_init(bar_sdone(g), 1);
    }
    misc[1] = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 256;" ::"r"(sbase + offBar + 96) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = (uint32_t)misc[0];
  const uint32_t tsum = tmem + 2 * kTcCen;           // 64 columns behind the two Gram buffers
  const int last_g = (n - 1) & 1;
  const uint32_t last_par = (uint32_t)(((n - 1) >> 1) & 1);

  if (warp == 8) {
    // ---- producer: TMA loads and MMA issue, one thread ----
    if (lane == 0) {
      auto load_tile = [&](int i) {
        const int buf = i % kSumBufs;
#pragma unroll
        for (int pn = 0; pn < NP; ++pn)
          tma_load_4d(sbase + offA + (buf * NP + pn) * kA, &tm_x, pn * 64, h, (tile0 + i) * kTcTok, b, bar_full(buf));
      };
      mbar_expect_tx(bar_full(0), NP * (kA + kB));
#pragma unroll
      for (int pn = 0; pn < NP; ++pn) tma_load_3d(sbase + offB + pn * kB, &tm_c, pn * 64, 0, bh, bar_full(0));
      load_tile(0);
      for (int i = 1; i < n && i < kSumBufs; ++i) {
        mbar_expect_tx(bar_full(i), NP * kA);
        load_tile(i);
      }
      const uint32_t id_gram = make_idesc_bf16(kTcCen);
      const uint32_t id_sum = make_idesc_bf16(kTcCen) | (1u << 15) | (1u << 16);     // both operands MN-major
      for (int i = 0; i <= n + 1; ++i) {
        if (i < n) {
          const int buf = i % kSumBufs, g = i & 1;
          if (!mbar_wait(bar_full(buf), (uint32_t)((i / kSumBufs) & 1), abort_flag, status, 51)) break;
          if (i >= 2 && !mbar_wait(bar_tfree(g), (uint32_t)(((i - 2) >> 1) & 1), abort_flag, status, 53)) break;
          tc_fence_after();
          bool first = true;
#pragma unroll
          for (int pc = 0; pc < 3; ++pc)
#pragma unroll
            for (int pn = 0; pn < NP; ++pn) {
              const uint64_t da = make_desc(sbase + offA + (buf * NP + pn) * kA, 128);
              const uint64_t db = make_desc(sbase + offB + pn * kB + pc * (kTcCen * 128), 128);
#pragma unroll
              for (int ks = 0; ks < 4; ++ks) {
                mma_bf16_ss(tmem + g * kTcCen, da + (uint64_t)(ks * 2), db + (uint64_t)(ks * 2), id_gram, first ? 0u : 1u);
                first = false;
              }
            }
          tc_commit(bar_gdone(g));
        }
        if (i >= 1 && i - 1 < n) {
          const int j = i - 1, g = j & 1;
          if (!mbar_wait(bar_oh(g), (uint32_t)((j >> 1) & 1), abort_flag, status, 56)) break;
          tc_fence_after();
          const uint64_t da = make_desc_mn(sbase + offA + (j % kSumBufs) * NP * kA, kA);
          const uint64_t db = make_desc_mn(sbase + offOH + g * kOH, 16);
#pragma unroll
          for (int ks = 0; ks < kTcTok / 16; ++ks)      // 16 tokens = two 1 KB atoms per step
            mma_bf16_ss(tsum, da + (uint64_t)(ks * 128), db + (uint64_t)(ks * 128), id_sum, (j > 0 || ks > 0) ? 1u : 0u);
          tc_commit(bar_sdone(g));
        }
        if (i >= 2) {
          const int j = i - 2;
          if (j + kSumBufs < n) {
            // the tile's buffer is free once its sums are done: refill it
            if (!mbar_wait(bar_sdone(j & 1), (uint32_t)((j >> 1) & 1), abort_flag, status, 54)) break;
            mbar_expect_tx(bar_full(j % kSumBufs), NP * kA);
            load_tile(j + kSumBufs);
          }
        }
      }
    }
  } else {
    // ---- consumers: thread == token == TMEM lane of its group's tile ----
    const int g = warp >> 2, wq = warp & 3;
    const int row = wq * 32 + lane;                  // token within the tile
    float cn[kTcCen];
#pragma unroll
    for (int c = 0; c < kTcCen; ++c) cn[c] = c < k ? cnorm[(size_t)bh * k + c] : INFINITY;
    uint8_t* oh_row = smem + offOH + g * kOH + row * 128;
    for (int i = g; i < n; i += 2) {
      bool ok = mbar_wait(bar_gdone(g), (uint32_t)((i >> 1) & 1), abort_flag, status, 52);
      if (!__all_sync(0xffffffffu, ok)) break;
      tc_fence_after();
      const uint32_t trow = tmem + g * kTcCen + ((uint32_t)(wq * 32) << 16);
      uint32_t r0[32], r1[32];
      LBFQ_TMEM_LD32(r0, trow);
      LBFQ_TMEM_LD32(r1, trow + 32);
      tc_wait_ld();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_tfree(g));
      // argmin over four independent chains of sixteen clusters (ascending within a chain, chains merged in
      // ascending order with a strict comparison: the lowest index wins ties, as in the one-chain form)
      float bq[4];
      int iq[4];
#pragma unroll
      for (int q4 = 0; q4 < 4; ++q4) {
        bq[q4] = INFINITY;
        iq[q4] = q4 * 16;
#pragma unroll
        for (int c = 0; c < 16; ++c) {
          const int cc = q4 * 16 + c;
          const float dot = __uint_as_float(cc < 32 ? r0[cc] : r1[cc - 32]);
          const float dist = cn[cc] - 2.0f * dot;
          if (dist < bq[q4]) { bq[q4] = dist; iq[q4] = cc; }
        }
      }
      float best = bq[0];
      int best_i = iq[0];
#pragma unroll
      for (int q4 = 1; q4 < 4; ++q4)
        if (bq[q4] < best) { best = bq[q4]; best_i = iq[q4]; }
      const int tok = (tile0 + i) * kTcTok + row;
      const bool live = tok < S;
      // the one-hot tile of the group is free once the sums of its previous tile are done
      if (i >= 2) {
        ok = mbar_wait(bar_sdone(g), (uint32_t)(((i - 2) >> 1) & 1), abort_flag, status, 57);
        if (!__all_sync(0xffffffffu, ok)) break;
      }
      const int hot = live ? (best_i >> 3) : -1;                     // 16-byte chunk that holds the 1.0
      const uint32_t one = 0x3f80u << ((best_i & 1) * 16);            // BF16 1.0 at element best_i & 7 of the chunk
      const int wi = (best_i & 7) >> 1;
      const uint4 hot_v = make_uint4(wi == 0 ? one : 0u, wi == 1 ? one : 0u, wi == 2 ? one : 0u, wi == 3 ? one : 0u);
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        const uint4 v = (c == hot) ? hot_v : make_uint4(0u, 0u, 0u, 0u);
        *reinterpret_cast<uint4*>(oh_row + ((c ^ (row & 7)) << 4)) = v;
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");    // generic-proxy stores, read by the MMA
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_oh(g));
      if (live) {                                                      // off the path the producer waits on
        labels[(size_t)bh * S + tok] = best_i;
        atomicAdd(&cnt[best_i], 1);
      }
    }
    if (g == 0) {
      // the CTA's sums: lane == channel, one column per cluster
      const bool ok = mbar_wait(bar_sdone(last_g), last_par, abort_flag, status, 58);
      if (__all_sync(0xffffffffu, ok && *abort_flag == 0)) {
        tc_fence_after();
        const uint32_t trow = tsum + ((uint32_t)(wq * 32) << 16);
        uint32_t r0[32], r1[32];
        LBFQ_TMEM_LD32(r0, trow);
        LBFQ_TMEM_LD32(r1, trow + 32);
        tc_wait_ld();
        float* dst = psum + (((size_t)bh * per_bh + chunk) * k) * D + row;
#pragma unroll
        for (int c = 0; c < 32; ++c)
          if (c < k) dst[(size_t)c * D] = __uint_as_float(r0[c]);
#pragma unroll
        for (int c = 0; c < 32; ++c)
          if (32 + c < k) dst[(size_t)(32 + c) * D] = __uint_as_float(r1[c]);
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (hist != nullptr && threadIdx.x < kTcCen)
    hist[((size_t)bh * per_bh + chunk) * kTcCen + threadIdx.x] = cnt[threadIdx.x];
  if (warp == 0) {
    if (*abort_flag && lane == 0) {
      const long long t0 = wall_ns();
      while (wall_ns() - t0 < 1000000ll) { }
    }
    __syncwarp();
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 256;" ::"r"(tmem) : "memory");
  }
}

PFN_cuTensorMapEncodeTiled_v12000 encoder() {
  static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
  if (!fn) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = (PFN_cuTensorMapEncodeTiled_v12000)ptr;
  }
  return fn;
}

template <int D>
int launch_assign(const CUtensorMap& mx, const CUtensorMap& mc, int BH, int S, int H, int k, const float* cnorm,
                  int32_t* labels, int32_t* hist, int32_t* status, cudaStream_t st) {
  constexpr int NP = D / 64;
  const int smem_bytes = NP * (2 * kTcTok * 128 + 3 * kTcCen * 128) + 64 + kTcCen * 4;
  auto kern = assign_tc_kernel<D>;
  LBFQ_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes));
  const int ntile = (S + kTcTok - 1) / kTcTok;
  const int per_bh = (ntile + kTcTiles - 1) / kTcTiles;
  kern<<<BH * per_bh, kTcThreads, smem_bytes, st>>>(mx, mc, S, H, k, cnorm, labels, hist, status);
  return check_launch("kmeans assign (tensor cores)");
}

}  // namespace

bool kmeans_tc_eligible(int dtype, int D, int k) { return dtype == LBFQ_BF16 && (D == 64 || D == 128) && k <= kTcCen; }

int kmeans_tc_chunk_tokens() { return kTcTiles * kTcTok; }

size_t kmeans_tc_split_bytes(int BH, int D) { return (size_t)BH * 3 * kTcCen * D * sizeof(__nv_bfloat16); }

bool kmeans_tc_sums_eligible(int dtype, int D, int k) { return kmeans_tc_eligible(dtype, D, k) && D == 128; }

// Tiles per CTA of the assignment-with-sums kernel. It holds one CTA per SM, so a launch is a number of waves of
// CTAs each of which pays a prologue and a drain (about five tile times: measured 17 us per CTA of eight tiles) that
// no neighbour hides: the count that minimises waves x (tiles + 5) for this problem and this GPU, between 4 tiles
// (the scratch is sized for that) and one CTA per slab.
constexpr int kSumMinTiles = 4;
int kmeans_tc_sum_tiles(int BH, int S) {
  const int ntile = (S + kTcTok - 1) / kTcTok;
  const int sms = sm_count();
  int best = kTcTiles;
  long long best_cost = -1;
  for (int t = kSumMinTiles; t <= ntile || t == kSumMinTiles; ++t) {
    const long long ctas = (long long)BH * ((ntile + t - 1) / t);
    const long long waves = (ctas + sms - 1) / sms;
    const long long cost = waves * (t + 5);
    if (best_cost < 0 || cost < best_cost) { best_cost = cost; best = t; }
    if (t >= ntile) break;
  }
  return best;
}
int kmeans_tc_sum_chunks(int BH, int S) {
  const int ntile = (S + kTcTok - 1) / kTcTok;
  const int t = kmeans_tc_sum_tiles(BH, S);
  return (ntile + t - 1) / t;
}
int kmeans_tc_sum_chunks_max(int S) {
  const int ntile = (S + kTcTok - 1) / kTcTok;
  return (ntile + kSumMinTiles - 1) / kSumMinTiles;
}

int kmeans_tc_update_from_sums(const float* psum, const int32_t* hist, int BH, int S, int D, int k, float* cent,
                               float* cnorm, void* split, cudaStream_t st) {
  chunk_mean_kernel<<<BH * k, 128, 0, st>>>(psum, hist, D, k, kmeans_tc_sum_chunks(BH, S), cent, cnorm, (__nv_bfloat16*)split);
  return check_launch("kmeans update (chunk sums)");
}

int kmeans_tc_assign(const void* x, int B, int S, int H, int D, int k, const float* cent, const float* cnorm,
                     void* split, int32_t* labels, int32_t* hist, float* psum, bool split_current, int32_t* status,
                     cudaStream_t st) {
  const int BH = B * H;
  if (!split_current) {
    const size_t total = (size_t)BH * kTcCen * D;
    int g = (int)((total + 255) / 256);
    if (g > sm_count() * 8) g = sm_count() * 8;
    split_centroids_kernel<<<g, 256, 0, st>>>(cent, BH, k, D, (__nv_bfloat16*)split);
    if (int rc = check_launch("kmeans centroid split")) return rc;
  }

  auto enc = encoder();
  LBFQ_REQUIRE(enc != nullptr, LBFQ_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
  CUtensorMap mx, mc;
  {
    // tokens: x is (B, S, H, D) bf16
    cuuint64_t dims[4] = {(cuuint64_t)D, (cuuint64_t)H, (cuuint64_t)S, (cuuint64_t)B};
    cuuint64_t strides[3] = {(cuuint64_t)D * 2, (cuuint64_t)H * D * 2, (cuuint64_t)S * H * D * 2};
    cuuint32_t box[4] = {64, 1, (cuuint32_t)kTcTok, 1};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    CUresult r = enc(&mx, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(x), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    LBFQ_REQUIRE(r == CUDA_SUCCESS, LBFQ_ERR_CUDA, "cuTensorMapEncodeTiled (tokens) failed with code %d", (int)r);
  }
  {
    // centroid pieces: (BH, 3 * 64, D) bf16
    cuuint64_t dims[3] = {(cuuint64_t)D, (cuuint64_t)(3 * kTcCen), (cuuint64_t)BH};
    cuuint64_t strides[2] = {(cuuint64_t)D * 2, (cuuint64_t)3 * kTcCen * D * 2};
    cuuint32_t box[3] = {64, (cuuint32_t)(3 * kTcCen), 1};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = enc(&mc, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, split, dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    LBFQ_REQUIRE(r == CUDA_SUCCESS, LBFQ_ERR_CUDA, "cuTensorMapEncodeTiled (centroids) failed with code %d", (int)r);
  }
  if (psum != nullptr) {
    LBFQ_REQUIRE(D == 128 && hist != nullptr, LBFQ_ERR_ARG, "the centroid sums ride on the D = 128 assignment and come with the counts");
    constexpr int kSumSmem = kSumBufs * 2 * kTcTok * 128 + 2 * 3 * kTcCen * 128 + 2 * kTcTok * 128 + 112 + kTcCen * 4;
    LBFQ_CUDA_OK(cudaFuncSetAttribute(assign_sum_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSumSmem));
    const int tiles = kmeans_tc_sum_tiles(BH, S);
    const int ntile = (S + kTcTok - 1) / kTcTok;
    const int per_bh = (ntile + tiles - 1) / tiles;
    assign_sum_tc_kernel<<<BH * per_bh, kSumThreads, kSumSmem, st>>>(mx, mc, S, H, k, tiles, cnorm, labels, hist, psum, status);
    return check_launch("kmeans assign + sums (tensor cores)");
  }
  if (D == 128) return launch_assign<128>(mx, mc, BH, S, H, k, cnorm, labels, hist, status, st);
  return launch_assign<64>(mx, mc, BH, S, H, k, cnorm, labels, hist, status, st);
}

}  // namespace lbfq
