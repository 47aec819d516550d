// Lloyd k-means over the tokens of each (b, h) slab.
//
// Stands in for flash_kmeans.batch_kmeans_Euclid as called from
// src/low_bit_fake_quant/kmeans.py:77-81 (x fp32 (B*H, S, D), k clusters,
// max_iters iterations, tol = 0 so the iteration count is fixed, labels of the
// last assignment returned). That package is a third-party dependency whose
// source is not part of the reference tree; what is reproduced here is the
// published algorithm, with a deterministic seeding documented below.
//
//   seeding   : centroid j of slab g = the token at index
//               lo_j + mix32(mix32(mix32(seed) ^ g) ^ j) % (hi_j - lo_j), g = b * total_heads + head,
//               [lo_j, hi_j) the j-th of k equal strata of the S axis
//   assignment: argmin_c |c|^2 - 2 x.c   (fp32, lowest index on ties)
//   update    : mean of the assigned tokens, summed in a fixed order so that a
//               run is bit-reproducible; an empty cluster keeps its centroid
//
// The update uses the same stable counting sort that later produces the token
// order: tokens of one cluster become one contiguous segment, reduced by one CTA.

#include "common.cuh"
#include "kmeans_tc.h"

namespace lbfq {

constexpr int kThreads = 256;
constexpr int kTok = 128;      // tokens per assignment CTA
constexpr int kCen = 64;       // centroids per pass
constexpr int kDc = 32;        // D chunk staged in shared memory

__host__ __device__ __forceinline__ uint32_t mix32(uint32_t x) {
  x ^= x >> 16; x *= 0x7FEB352Du; x ^= x >> 15; x *= 0x846CA68Bu; x ^= x >> 16;
  return x;
}

template <typename T>
__global__ void init_centroids_kernel(const T* __restrict__ x, int S, int H, int D, int k, uint32_t seed,
                                      int head_offset, int total_heads, float* __restrict__ cent,
                                      float* __restrict__ cnorm) {
  const int j = blockIdx.x % k;
  const int bh = blockIdx.x / k;
  const int b = bh / H, h = bh % H;
  const int lo = (int)(((int64_t)j * S) / k);
  const int hi = (int)(((int64_t)(j + 1) * S) / k);
  const int span = max(hi - lo, 1);
  const uint32_t slab = (uint32_t)(b * total_heads + head_offset + h);     // index in the unsharded problem
  const uint32_t hsh = mix32(mix32(mix32(seed) ^ slab) ^ (uint32_t)j);
  const int idx = lo + (int)(hsh % (uint32_t)span);
  __shared__ float red[4];
  float v = 0.f;
  if (threadIdx.x < D) {
    v = Elem<T>::load(x + (((size_t)b * S + idx) * H + h) * D + threadIdx.x);
    cent[((size_t)bh * k + j) * D + threadIdx.x] = v;
  }
  float s = warp_sum(v * v);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x == 0) cnorm[(size_t)bh * k + j] = red[0] + red[1] + red[2] + red[3];
}

template <typename T>
__global__ void __launch_bounds__(kThreads)
assign_kernel(const T* __restrict__ x, int S, int H, int D, int k, const float* __restrict__ cent,
              const float* __restrict__ cnorm, int32_t* __restrict__ labels) {
  __shared__ float a_s[kDc][kTok + 4];    // [d][token]
  __shared__ float b_s[kDc][kCen + 4];    // [d][centroid]
  const int ntile = (S + kTok - 1) / kTok;
  const int tile = blockIdx.x % ntile;
  const int bh = blockIdx.x / ntile;
  const int b = bh / H, h = bh % H;
  const int t0 = tile * kTok;
  const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;   // 8 tokens x 4 centroids per thread
  float best[8];
  int best_i[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) { best[i] = INFINITY; best_i[i] = 0; }

  for (int c0 = 0; c0 < k; c0 += kCen) {
    float acc[8][4];
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
    for (int d0 = 0; d0 < D; d0 += kDc) {
      for (int idx = threadIdx.x; idx < kTok * kDc; idx += kThreads) {
        const int t = idx / kDc, d = idx % kDc;
        const int tok = t0 + t;
        a_s[d][t] = tok < S ? Elem<T>::load(x + (((size_t)b * S + tok) * H + h) * D + d0 + d) : 0.f;
      }
      for (int idx = threadIdx.x; idx < kCen * kDc; idx += kThreads) {
        const int c = idx / kDc, d = idx % kDc;
        b_s[d][c] = (c0 + c) < k ? cent[((size_t)bh * k + c0 + c) * D + d0 + d] : 0.f;
      }
      __syncthreads();
#pragma unroll 8
      for (int d = 0; d < kDc; ++d) {
        float av[8], bv[4];
#pragma unroll
        for (int i = 0; i < 8; ++i) av[i] = a_s[d][ty * 8 + i];
#pragma unroll
        for (int j = 0; j < 4; ++j) bv[j] = b_s[d][tx * 4 + j];
#pragma unroll
        for (int i = 0; i < 8; ++i)
#pragma unroll
          for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
      }
      __syncthreads();
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int c = c0 + tx * 4 + j;
      if (c < k) {
        const float cn = cnorm[(size_t)bh * k + c];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float dist = cn - 2.0f * acc[i][j];
          if (dist < best[i]) { best[i] = dist; best_i[i] = c; }   // ascending c: lowest index wins ties
        }
      }
    }
  }
  // combine the 16 tx lanes of a token row (lanes differ in tx only within a half-warp)
#pragma unroll
  for (int i = 0; i < 8; ++i) {
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best[i], o);
      const int oi = __shfl_xor_sync(0xffffffffu, best_i[i], o);
      if (ob < best[i] || (ob == best[i] && oi < best_i[i])) { best[i] = ob; best_i[i] = oi; }
    }
    const int tok = t0 + ty * 8 + i;
    if (tx == 0 && tok < S) labels[(size_t)bh * S + tok] = best_i[i];
  }
}

// Stable counting sort of one slab's labels, one CTA per slab; also emits the k + 1 segment offsets.
// Histogram, exclusive scan, then the tokens in chunks of 1024 in token order: a lane finds the lanes of its warp
// with the same label (__match_any_sync), the warp leaders of each label publish their counts, an exclusive scan
// over the 32 warps per label turns them into positions, and every lane stores its token. O(S) work per slab;
// the order inside a cluster is the token order, so the sums taken over it are bit-reproducible.
constexpr int kSortMaxK = 64;
__global__ void __launch_bounds__(1024)
sort_segments_kernel(const int32_t* __restrict__ labels, int S, int k, int32_t* __restrict__ order32,
                     int32_t* __restrict__ seg) {
  __shared__ int counts[kSortMaxK];
  __shared__ int offsets[kSortMaxK];
  __shared__ int wc[32][kSortMaxK];               // per warp and label: count, then start position
  const int32_t* lab = labels + (size_t)blockIdx.x * S;
  int32_t* ord = order32 + (size_t)blockIdx.x * S;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int i = threadIdx.x; i < k; i += blockDim.x) counts[i] = 0;
  __syncthreads();
  for (int i = threadIdx.x; i < S; i += blockDim.x)
    if ((unsigned)lab[i] < (unsigned)k) atomicAdd(&counts[lab[i]], 1);     // a label outside [0, k) is never an index
  __syncthreads();
  if (threadIdx.x == 0) {
    int run = 0;
    for (int c = 0; c < k; ++c) { offsets[c] = run; seg[(size_t)blockIdx.x * (k + 1) + c] = run; run += counts[c]; }
    seg[(size_t)blockIdx.x * (k + 1) + k] = run;
  }
  for (int base = 0; base < S; base += 1024) {
    for (int i = threadIdx.x; i < 32 * kSortMaxK; i += blockDim.x) (&wc[0][0])[i] = 0;
    __syncthreads();                                          // also orders `offsets` (first pass: thread 0's scan)
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
    if (valid) ord[wc[warp][lbl] + rank] = i;
    __syncthreads();
  }
}

// The same sort cut into chunks, for label counts that the assignment kernel has already taken per chunk of
// `chunk` (= 1024) tokens: one CTA per (slab, chunk) finds where each label's tokens of its chunk start (all smaller
// labels of the slab, then the same label in the earlier chunks) and ranks its 1024 tokens as above. The order it
// writes is the same stable order; the slab's work is spread over S / 1024 CTAs instead of one.
__global__ void __launch_bounds__(1024)
sort_chunks_kernel(const int32_t* __restrict__ labels, const int32_t* __restrict__ hist, int S, int k, int nchunk,
                   int32_t* __restrict__ order32, int32_t* __restrict__ seg) {
  __shared__ int total[kSortMaxK];
  __shared__ int before[kSortMaxK];
  __shared__ int offsets[kSortMaxK];
  __shared__ int wc[32][kSortMaxK];               // per warp and label: count, then start position
  const int chunk = blockIdx.x % nchunk;
  const size_t bh = blockIdx.x / nchunk;
  const int32_t* lab = labels + bh * S;
  int32_t* ord = order32 + bh * S;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int i = threadIdx.x; i < 32 * kSortMaxK; i += blockDim.x) (&wc[0][0])[i] = 0;
  if ((int)threadIdx.x < k) {
    const int32_t* hp = hist + bh * nchunk * kSortMaxK + threadIdx.x;
    int t = 0, bsum = 0;
    for (int j = 0; j < nchunk; ++j) {
      const int c = hp[(size_t)j * kSortMaxK];
      if (j < chunk) bsum += c;
      t += c;
    }
    total[threadIdx.x] = t;
    before[threadIdx.x] = bsum;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int run = 0;
    for (int c = 0; c < k; ++c) {
      offsets[c] = run + before[c];
      if (chunk == 0) seg[bh * (k + 1) + c] = run;
      run += total[c];
    }
    if (chunk == 0) seg[bh * (k + 1) + k] = run;
  }
  const int i = chunk * 1024 + (int)threadIdx.x;
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
  }
  __syncthreads();
  // the counts came from the assignment launch: a position is only used while it lies inside the slab
  if (valid) {
    const int pos = wc[warp][lbl] + rank;
    if ((unsigned)pos < (unsigned)S) ord[pos] = i;
  }
}

// the same sort for more labels than the shared-memory tables above hold: one warp per label scans the slab
__global__ void __launch_bounds__(1024)
sort_segments_scan_kernel(const int32_t* __restrict__ labels, int S, int k, int32_t* __restrict__ order32,
                          int32_t* __restrict__ seg) {
  extern __shared__ int sm_counts[];
  int* counts = sm_counts;
  int* offsets = sm_counts + k;
  const int32_t* lab = labels + (size_t)blockIdx.x * S;
  int32_t* ord = order32 + (size_t)blockIdx.x * S;
  for (int i = threadIdx.x; i < k; i += blockDim.x) counts[i] = 0;
  __syncthreads();
  for (int i = threadIdx.x; i < S; i += blockDim.x)
    if ((unsigned)lab[i] < (unsigned)k) atomicAdd(&counts[lab[i]], 1);
  __syncthreads();
  if (threadIdx.x == 0) {
    int run = 0;
    for (int c = 0; c < k; ++c) { offsets[c] = run; seg[(size_t)blockIdx.x * (k + 1) + c] = run; run += counts[c]; }
    seg[(size_t)blockIdx.x * (k + 1) + k] = run;
  }
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  for (int c = warp; c < k; c += nwarps) {
    int pos = offsets[c];
    for (int base = 0; base < S; base += 32) {
      const int i = base + lane;
      const bool hit = (i < S) && (lab[i] == c);
      const unsigned m = __ballot_sync(0xffffffffu, hit);
      if (hit) ord[pos + __popc(m & ((1u << lane) - 1u))] = i;
      pos += __popc(m);
    }
  }
}

// Cluster means in two steps, so that one large cluster does not keep a single CTA busy while the rest of the GPU
// idles: up to kMeanParts CTAs per (slab, cluster) each add a contiguous part of the cluster's sorted rows (fixed order
// inside a part), then one CTA adds the parts in order, divides and takes the squared norm. Bit-reproducible.
constexpr int kMeanParts = 8;
// many small clusters need no splitting (and their partial sums would be large)
static inline int mean_parts(int k) { return k <= 256 ? kMeanParts : 1; }

template <typename T>
__global__ void __launch_bounds__(kThreads)
segment_part_sums_kernel(const T* __restrict__ x, int S, int H, int D, int k, const int32_t* __restrict__ order32,
                         const int32_t* __restrict__ seg, float* __restrict__ psum, int parts) {
  __shared__ float buf[kThreads / 8][128 + 1];
  const int part = blockIdx.x % parts;
  const int c = (blockIdx.x / parts) % k;
  const int bh = blockIdx.x / (parts * k);
  const int b = bh / H, h = bh % H;
  const int cbeg = seg[(size_t)bh * (k + 1) + c], cend = seg[(size_t)bh * (k + 1) + c + 1];
  const int len = cend - cbeg;
  const int beg = cbeg + (int)(((int64_t)len * part) / parts);
  const int end = cbeg + (int)(((int64_t)len * (part + 1)) / parts);
  const int tpr = D / 8, rpi = kThreads / tpr;
  const int tr = threadIdx.x / tpr, d0 = (threadIdx.x % tpr) * 8;
  float acc[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i] = 0.f;
  if constexpr (sizeof(T) == 2) {
    // eight 16-bit channels = one 16-byte load; four rows in flight per thread, added in the order of the plain loop
    constexpr int U = 4;
    const int32_t* ord = order32 + (size_t)bh * S;
    int r = beg + tr;
    for (; r + (U - 1) * rpi < end; r += U * rpi) {
      uint4 w[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int tok = ord[r + u * rpi];
        w[u] = *reinterpret_cast<const uint4*>(x + (((size_t)b * S + tok) * H + h) * D + d0);
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const T* e = reinterpret_cast<const T*>(&w[u]);
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] += Elem<T>::load(e + i);
      }
    }
    for (; r < end; r += rpi) {
      const uint4 w = *reinterpret_cast<const uint4*>(x + (((size_t)b * S + ord[r]) * H + h) * D + d0);
      const T* e = reinterpret_cast<const T*>(&w);
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] += Elem<T>::load(e + i);
    }
  } else {
    for (int r = beg + tr; r < end; r += rpi) {
      const int tok = order32[(size_t)bh * S + r];
      const T* p = x + (((size_t)b * S + tok) * H + h) * D + d0;
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] += Elem<T>::load(p + i);
    }
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) buf[tr][d0 + i] = acc[i];
  __syncthreads();
  if (threadIdx.x < D) {
    float s = 0.f;
    for (int r = 0; r < rpi; ++r) s += buf[r][threadIdx.x];
    psum[(((size_t)bh * k + c) * parts + part) * D + threadIdx.x] = s;     // zero for an empty part
  }
}

__global__ void __launch_bounds__(128)
segment_mean_from_parts_kernel(const float* __restrict__ psum, const int32_t* __restrict__ seg, int D, int k, int parts,
                               float* __restrict__ cent, float* __restrict__ cnorm) {
  __shared__ float red[4];
  const int c = blockIdx.x % k;
  const size_t bh = blockIdx.x / k;
  const int n = seg[bh * (k + 1) + c + 1] - seg[bh * (k + 1) + c];
  if (n == 0) return;                               // empty cluster keeps centroid and norm
  float v = 0.f;
  if (threadIdx.x < D) {
    float s = 0.f;
    for (int p = 0; p < parts; ++p) s += psum[((bh * k + c) * parts + p) * D + threadIdx.x];
    v = __fdiv_rn(s, (float)n);
    cent[(bh * k + c) * D + threadIdx.x] = v;
  }
  const float s2 = warp_sum(v * v);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s2;
  __syncthreads();
  if (threadIdx.x == 0) cnorm[bh * k + c] = red[0] + red[1] + red[2] + red[3];
}

struct KmScratch {
  float* cent; float* cnorm; int32_t* order32; int32_t* seg; void* split; int32_t* hist; float* psum;
};
static size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }
static size_t scratch_layout(int BH, int S, int D, int k, uint8_t* base, KmScratch* out) {
  size_t off = 0;
  auto take = [&](size_t bytes) { size_t o = off; off = align_up(off + bytes, 256); return base ? base + o : nullptr; };
  uint8_t* p0 = take((size_t)BH * k * D * 4);
  uint8_t* p1 = take((size_t)BH * k * 4);
  uint8_t* p2 = take((size_t)BH * S * 4);
  uint8_t* p3 = take((size_t)BH * (k + 1) * 4);
  uint8_t* p4 = take(kmeans_tc_split_bytes(BH, D));       // BF16 pieces of the centroids (tensor-core assignment)
  const size_t nchunk = ((size_t)S + kmeans_tc_chunk_tokens() - 1) / kmeans_tc_chunk_tokens();
  const size_t nsum = (size_t)kmeans_tc_sum_chunks_max(S);   // chunks of the assignment that also takes the sums
  const size_t nhist = nchunk > nsum ? nchunk : nsum;
  uint8_t* p5 = take((size_t)BH * nhist * kSortMaxK * 4);    // per-chunk label counts from the tensor-core assignment
  // partial sums of the cluster means: per part of a sorted segment, or per chunk of the tensor-core assignment
  const size_t parts = nsum > (size_t)mean_parts(k) ? nsum : (size_t)mean_parts(k);
  uint8_t* p6 = take((size_t)BH * k * parts * D * 4);
  if (out) { out->split = p4; out->hist = (int32_t*)p5; out->psum = (float*)p6; }
  if (out) { out->cent = (float*)p0; out->cnorm = (float*)p1; out->order32 = (int32_t*)p2; out->seg = (int32_t*)p3; }
  return off;
}

}  // namespace lbfq

using namespace lbfq;

extern "C" int64_t lbfq_kmeans_scratch_bytes(int B, int S, int H, int D, int k) {
  return (int64_t)scratch_layout(B * H, S, D, k, nullptr, nullptr);
}

extern "C" int lbfq_kmeans_labels(const void* x, int dtype, int B, int S, int H, int D, int k, int iters,
                                  int seed, int head_offset, int total_heads, int32_t* labels, void* scratch,
                                  int32_t* status, void* stream) {
  LBFQ_REQUIRE(B > 0 && S > 0 && H > 0, LBFQ_ERR_ARG, "kmeans: empty input");
  LBFQ_REQUIRE(D == 64 || D == 128, LBFQ_ERR_ARG, "kmeans: D must be 64 or 128; got %d", D);
  LBFQ_REQUIRE(k > 0 && k <= S, LBFQ_ERR_ARG, "n_clusters must be in [1, S]; got %d for S=%d", k, S);
  LBFQ_REQUIRE(k <= 4096, LBFQ_ERR_UNSUPPORTED, "kmeans: k=%d above the supported 4096", k);
  if (total_heads <= 0) { total_heads = H; head_offset = 0; }
  LBFQ_REQUIRE(head_offset >= 0 && head_offset + H <= total_heads, LBFQ_ERR_ARG,
               "kmeans: heads [%d, %d) do not fit in %d total heads", head_offset, head_offset + H, total_heads);
  cudaStream_t st = (cudaStream_t)stream;
  const int BH = B * H;
  KmScratch sc;
  scratch_layout(BH, S, D, k, (uint8_t*)scratch, &sc);
  if (iters < 1) iters = 1;
  // every label is a valid cluster index from here on, whatever happens to an assignment launch (a launch whose
  // bounded wait expires leaves some labels unwritten and says so in `status`; the sorts index by label)
  LBFQ_CUDA_OK(cudaMemsetAsync(labels, 0, sizeof(int32_t) * (size_t)BH * S, st));
  LBFQ_CUDA_OK(cudaMemsetAsync(sc.order32, 0, sizeof(int32_t) * (size_t)BH * S, st));     // likewise every sorted position
  LBFQ_DISPATCH_DTYPE(dtype, T,
      init_centroids_kernel<T><<<BH * k, 128, 0, st>>>((const T*)x, S, H, D, k, (uint32_t)seed, head_offset, total_heads, sc.cent, sc.cnorm));
  if (int rc = check_launch("kmeans init")) return rc;
  const int ntile = (S + kTok - 1) / kTok;
  // LBFQ_FLAG_KMEANS_FFMA keeps the FP32 FFMA assignment (used to cross-check the two)
  const bool tc = kmeans_tc_eligible(dtype, D, k) && !(debug_flags() & LBFQ_FLAG_KMEANS_FFMA);
  // LBFQ_FLAG_KMEANS_SORTED keeps the update by sort + segment means (the cross-check of the sums taken inside the
  // assignment kernel)
  const bool tcsum = tc && kmeans_tc_sums_eligible(dtype, D, k) && kmeans_tc_chunk_tokens() == 1024 &&
                     !(debug_flags() & LBFQ_FLAG_KMEANS_SORTED);
  for (int it = 0; it < iters; ++it) {
    if (tc) {
      // the counts (and sums) are only wanted when an update follows (not after the last assignment)
      const bool more = it + 1 < iters;
      // (after an update from the sums the BF16 pieces of the centroids are current already)
      if (int rc = kmeans_tc_assign(x, B, S, H, D, k, sc.cent, sc.cnorm, sc.split, labels, more ? sc.hist : nullptr,
                                    (more && tcsum) ? sc.psum : nullptr, tcsum && it > 0, status, st)) return rc;
      if (more && tcsum) {
        if (int rc = kmeans_tc_update_from_sums(sc.psum, sc.hist, BH, S, D, k, sc.cent, sc.cnorm, sc.split, st)) return rc;
        continue;
      }
    } else {
      LBFQ_DISPATCH_DTYPE(dtype, T,
          assign_kernel<T><<<BH * ntile, kThreads, 0, st>>>((const T*)x, S, H, D, k, sc.cent, sc.cnorm, labels));
    }
    if (int rc = check_launch("kmeans assign")) return rc;
    if (it + 1 == iters) break;                     // labels of the last assignment are the result
    if (tc && kmeans_tc_chunk_tokens() == 1024) {
      const int nchunk = (S + 1023) / 1024;
      sort_chunks_kernel<<<BH * nchunk, 1024, 0, st>>>(labels, sc.hist, S, k, nchunk, sc.order32, sc.seg);
    } else if (k <= kSortMaxK) sort_segments_kernel<<<BH, 1024, 0, st>>>(labels, S, k, sc.order32, sc.seg);
    else sort_segments_scan_kernel<<<BH, 1024, 2 * k * sizeof(int), st>>>(labels, S, k, sc.order32, sc.seg);
    if (int rc = check_launch("kmeans sort")) return rc;
    LBFQ_DISPATCH_DTYPE(dtype, T,
        segment_part_sums_kernel<T><<<BH * k * mean_parts(k), kThreads, 0, st>>>((const T*)x, S, H, D, k, sc.order32, sc.seg, sc.psum, mean_parts(k)));
    if (int rc = check_launch("kmeans part sums")) return rc;
    segment_mean_from_parts_kernel<<<BH * k, 128, 0, st>>>(sc.psum, sc.seg, D, k, mean_parts(k), sc.cent, sc.cnorm);
    if (int rc = check_launch("kmeans update")) return rc;
  }
  return LBFQ_OK;
}
