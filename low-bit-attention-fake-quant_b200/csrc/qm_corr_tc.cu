// The score bias of the Q-smoothing correction on the tensor cores (BF16 keys).
//
// corr[b,h,g,n] = (qm[b,g,h,:] . k_smooth[b,n,h,:]) * sm_scale (attention_triton.py:156-160 of the reference, whose
// row max is _estimate_rowmax_from_qm_k, attention.py:366-395) is a GEMM with M = keys, N = Q groups, K = D. The keys
// are BF16 already; the FP32 group means are split into three BF16 pieces (qm = hi + mid + lo to 24 bits), so every
// product is exact and the sum is FP32: the FFMA kernel's value up to summation order. The operator is bound by
// writing corr (4 bytes per key and group) and reading the keys once, not by arithmetic.
//
// One CTA owns up to 128 groups of one (b, h) and walks kTiles consecutive 128-key tiles: the pieces are written
// into shared memory once, in the 128-byte-swizzled K-major layout the MMA descriptors expect; key tiles arrive
// by TMA through two buffers; one thread issues 3 x D/16 tcgen05.mma.kind::f16 per tile into one of two 128-column
// TMEM buffers; thread == key reads its row back and stores it (32 lanes = 128 contiguous bytes of one group's row).
#include "attn_prims.cuh"
#include "qm_corr_tc.h"

namespace lbfq {

using namespace attn;

namespace {

constexpr int kKeys = 128;       // keys per tile (MMA M)
constexpr int kGroups = 128;     // groups per CTA (MMA N), zero rows above G
constexpr int kTiles = 16;       // key tiles per CTA
constexpr int kQcThreads = 256;  // two warps per TMEM lane quarter: each takes half of the groups

__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* map, int c0, int c1, int c2, int c3, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];"
      ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(bar) : "memory");
}

// order-preserving map float -> int32 (for redux.sync.max) and back
__device__ __forceinline__ int float_key(float v) {
  const int i = __float_as_int(v);
  return i >= 0 ? i : (i ^ 0x7fffffff);
}
__device__ __forceinline__ float key_float(int k) { return __int_as_float(k >= 0 ? k : (k ^ 0x7fffffff)); }

__device__ __forceinline__ void atomic_max_f32(float* addr, float v) {
  if (v >= 0.f) atomicMax(reinterpret_cast<int*>(addr), __float_as_int(v));
  else atomicMin(reinterpret_cast<unsigned int*>(addr), __float_as_uint(v));
}

template <int D>
__global__ void __launch_bounds__(kQcThreads, 1)
qm_corr_tc_kernel(const __grid_constant__ CUtensorMap tm_k, const float* __restrict__ qm, int S, int H, int G,
                  float sm_scale, float* __restrict__ corr, int s_pad, float* __restrict__ rowmax,
                  int32_t* __restrict__ status) {
  constexpr int NP = D / 64;                         // 64-channel panels (one 128-byte swizzle row each)
  constexpr int kA = kKeys * 128;                    // bytes per key panel
  constexpr int kB = kGroups * 128;                  // bytes per (piece, panel) of the group means
  // the swizzled tiles want a 1 KB-aligned base, which the declared alignment of the array provides
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  const uint32_t sbase = smem_u32(smem);
  const uint32_t offA = 0, offB = 2 * NP * kA, offBar = offB + 3 * NP * kB;
  auto bar_full = [&](int buf) { return sbase + offBar + 8u * buf; };          // key tile landed
  auto bar_done = [&](int buf) { return sbase + offBar + 16u + 8u * buf; };    // MMAs of the tile in this buffer done
  volatile int* misc = (volatile int*)(smem + offBar + 32);       // [0] tmem base, [1] abort
  volatile int* abort_flag = misc + 1;

  const int ntile = (s_pad + kKeys - 1) / kKeys;
  const int per_bh = (ntile + kTiles - 1) / kTiles;
  // heads vary fastest over the grid: CTAs in flight together read the same key rows of the (B, S, H, D) input
  const int h = blockIdx.x % H;
  const int tile0 = ((blockIdx.x / H) % per_bh) * kTiles;
  const int b = blockIdx.x / (H * per_bh);
  const int bh = b * H + h;
  const int n_tiles = min(kTiles, ntile - tile0);
  const int g0 = blockIdx.y * kGroups;               // first group of this CTA
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    mbar_init(bar_full(0), 1);
    mbar_init(bar_full(1), 1);
    mbar_init(bar_done(0), 1);
    mbar_init(bar_done(1), 1);
    misc[1] = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 256;" ::"r"(sbase + offBar + 32) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }

  // ---- group means -> three BF16 pieces, 128B-swizzled K-major rows (16-byte chunk c of row r sits at c ^ (r & 7)) ----
  for (int item = threadIdx.x; item < kGroups * (D / 8); item += kQcThreads) {
    const int r = item / (D / 8), c = item % (D / 8);
    const int g = g0 + r;
    float v[8];
    if (g < G) {
      const float4* src = reinterpret_cast<const float4*>(qm + (((size_t)b * G + g) * H + h) * D + c * 8);
      const float4 lo4 = src[0], hi4 = src[1];
      v[0] = lo4.x; v[1] = lo4.y; v[2] = lo4.z; v[3] = lo4.w; v[4] = hi4.x; v[5] = hi4.y; v[6] = hi4.z; v[7] = hi4.w;
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] = 0.f;
    }
    __align__(16) __nv_bfloat16 pc[3][8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      float x = v[i];
      pc[0][i] = __float2bfloat16_rn(x);
      x -= __bfloat162float(pc[0][i]);
      pc[1][i] = __float2bfloat16_rn(x);
      x -= __bfloat162float(pc[1][i]);
      pc[2][i] = __float2bfloat16_rn(x);
    }
    const int pn = c / 8, cc = c % 8;
#pragma unroll
    for (int p = 0; p < 3; ++p)
      *reinterpret_cast<uint4*>(smem + offB + (p * NP + pn) * kB + r * 128 + ((cc ^ (r & 7)) * 16)) =
          *reinterpret_cast<const uint4*>(pc[p]);
  }
  // generic-proxy writes above are read by the tensor core through the async proxy
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = (uint32_t)misc[0];

  auto load_tile = [&](int i) {                       // thread 0: key tile i of this CTA into buffer i & 1
    const int buf = i & 1;
    mbar_expect_tx(bar_full(buf), NP * kA);
#pragma unroll
    for (int pn = 0; pn < NP; ++pn)
      tma_load_4d(sbase + offA + (buf * NP + pn) * kA, &tm_k, pn * 64, h, (tile0 + i) * kKeys, b, bar_full(buf));
  };
  auto issue_mma = [&](int i) -> bool {               // thread 0: products of tile i into TMEM buffer i & 1
    const int buf = i & 1;
    if (!mbar_wait(bar_full(buf), (uint32_t)((i >> 1) & 1), abort_flag, status, 61)) return false;
    tc_fence_after();
    const uint32_t idesc = make_idesc_bf16(kGroups);
    bool first = true;
#pragma unroll
    for (int p = 0; p < 3; ++p)
#pragma unroll
      for (int pn = 0; pn < NP; ++pn) {
        const uint64_t da = make_desc(sbase + offA + (buf * NP + pn) * kA, 128);
        const uint64_t db = make_desc(sbase + offB + (p * NP + pn) * kB, 128);
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) {
          mma_bf16_ss(tmem + buf * kGroups, da + (uint64_t)(ks * 2), db + (uint64_t)(ks * 2), idesc, first ? 0u : 1u);
          first = false;
        }
      }
    tc_commit(bar_done(buf));
    return true;
  };

  if (threadIdx.x == 0) {
    load_tile(0);
    if (n_tiles > 1) load_tile(1);
    issue_mma(0);
  }
  const int key_row = (warp & 3) * 32 + lane;         // TMEM lane == key within the tile
  const int half = warp >> 2;                         // which 64 of the CTA's groups this warp stores
  const int gbase = g0 + half * 64;
  // running max of this thread's key row over the CTA's tiles, one register per group; the 128 rows meet at the end
  float run[64];
#pragma unroll
  for (int j = 0; j < 64; ++j) run[j] = -INFINITY;
  for (int i = 0; i < n_tiles; ++i) {
    const int buf = i & 1;
    // the next tile's MMAs first (its TMEM buffer was read out two tiles ago, before the last barrier)
    if (threadIdx.x == 0 && i + 1 < n_tiles) issue_mma(i + 1);
    __syncwarp();
    const bool ok = mbar_wait(bar_done(buf), (uint32_t)((i >> 1) & 1), abort_flag, status, 62);
    const bool all_ok = __all_sync(0xffffffffu, ok);
    if (threadIdx.x == 0 && ok && i + 2 < n_tiles) load_tile(i + 2);   // the tile's shared-memory buffer is free again
    __syncwarp();
    if (all_ok) {
      tc_fence_after();
      const uint32_t trow = tmem + buf * kGroups + half * 64 + ((uint32_t)((warp & 3) * 32) << 16);
      uint32_t r0[32], r1[32];
      LBFQ_TMEM_LD32(r0, trow);
      LBFQ_TMEM_LD32(r1, trow + 32);
      tc_wait_ld();
      const int n = (tile0 + i) * kKeys + key_row;
      const bool n_real = n < S, n_store = n < s_pad;
      float* out = corr + ((size_t)bh * G + gbase) * s_pad + n;
      const int ng = min(64, G - gbase);               // warp-uniform
#pragma unroll
      for (int j = 0; j < 64; ++j) {
        if (j < ng) {
          const float v = __uint_as_float(j < 32 ? r0[j & 31] : r1[j & 31]) * sm_scale;
          if (n_store) *out = n_real ? v : 0.f;
          if (n_real) run[j] = fmaxf(run[j], v);
          out += s_pad;
        }
      }
    }
    tc_fence_before();
    // every thread has read this tile's TMEM buffer before tile i + 2 is multiplied into it; a given-up wait ends
    // the loop for all threads together
    if (__syncthreads_or(all_ok ? 0 : 1)) break;
  }
  if (rowmax != nullptr && *abort_flag == 0) {
    // the warp's 32 rows meet through redux.sync.max on an order-preserving integer image of the floats
#pragma unroll
    for (int j = 0; j < 64; ++j) {
      if (gbase + j < G) {                             // warp-uniform
        const float m = key_float(__reduce_max_sync(0xffffffffu, float_key(run[j])));
        if (lane == 0 && m > -INFINITY) atomic_max_f32(rowmax + (size_t)bh * G + gbase + j, m);
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    if (*abort_flag && lane == 0) {
      // give in-flight bulk copies a bounded time to land before the CTA retires
      const long long t0 = wall_ns();
      while (wall_ns() - t0 < 1000000ll) { }
    }
    __syncwarp();
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 256;" ::"r"(tmem) : "memory");
  }
}

PFN_cuTensorMapEncodeTiled_v12000 qc_encoder() {
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
int launch_qm_corr(const CUtensorMap& mk, const float* qm, int B, int S, int H, int G, float sm_scale, float* corr,
                   int s_pad, float* rowmax, int32_t* status, cudaStream_t st) {
  constexpr int NP = D / 64;
  const int smem_bytes = NP * (2 * kKeys * 128 + 3 * kGroups * 128) + 64 + 1024;
  auto kern = qm_corr_tc_kernel<D>;
  LBFQ_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes));
  const int ntile = (s_pad + kKeys - 1) / kKeys;
  const int per_bh = (ntile + kTiles - 1) / kTiles;
  dim3 grid(B * H * per_bh, (G + kGroups - 1) / kGroups, 1);
  kern<<<grid, kQcThreads, smem_bytes, st>>>(mk, qm, S, H, G, sm_scale, corr, s_pad, rowmax, status);
  return check_launch("qm_corr (tensor cores)");
}

}  // namespace

bool qm_corr_tc_eligible(int dtype, int D, int S, const void* k_smooth) {
  // a key tile is a 128-row TMA box: shorter inputs stay on the FFMA kernel
  return dtype == LBFQ_BF16 && (D == 64 || D == 128) && S >= kKeys && (reinterpret_cast<uintptr_t>(k_smooth) & 15) == 0;
}

int qm_corr_tc(const float* qm, const void* k_smooth, int B, int S, int H, int D, int G, float sm_scale, float* corr,
               int s_pad, float* rowmax, int32_t* status, cudaStream_t st) {
  auto enc = qc_encoder();
  LBFQ_REQUIRE(enc != nullptr, LBFQ_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
  CUtensorMap mk;
  // keys: (B, S, H, D) bf16; rows past S read as zero
  cuuint64_t dims[4] = {(cuuint64_t)D, (cuuint64_t)H, (cuuint64_t)S, (cuuint64_t)B};
  cuuint64_t strides[3] = {(cuuint64_t)D * 2, (cuuint64_t)H * D * 2, (cuuint64_t)S * H * D * 2};
  cuuint32_t box[4] = {64, 1, (cuuint32_t)kKeys, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = enc(&mk, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(k_smooth), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  LBFQ_REQUIRE(r == CUDA_SUCCESS, LBFQ_ERR_CUDA, "cuTensorMapEncodeTiled (keys) failed with code %d", (int)r);
  if (D == 128) return launch_qm_corr<128>(mk, qm, B, S, H, G, sm_scale, corr, s_pad, rowmax, status, st);
  return launch_qm_corr<64>(mk, qm, B, S, H, G, sm_scale, corr, s_pad, rowmax, status, st);
}

}  // namespace lbfq
