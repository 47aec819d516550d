// Device primitives shared by the attention kernels: bounded mbarrier waits, TMA and bulk copies,
// tcgen05 (MMA, TMEM load / store / copy, fences, commit), shared-memory and instruction descriptors,
// and the pre-digested kernel parameter block.
#pragma once

#include <cuda.h>
#include <cudaTypedefs.h>

#include "common.cuh"

namespace lbfq {
namespace attn {

constexpr int kTileM = 128;              // rows per softmax warpgroup
constexpr int kCtaM = 2 * kTileM;        // rows per CTA
constexpr int kChunk = 128;              // keys per TMA stage
constexpr int kStages = 3;
constexpr int kSoftmaxWarps = 8;         // 2 tiles x 4 lane quarters: one thread per query row
constexpr int kThreads = 384;            // 8 softmax warps + 1 warpgroup of service warps
constexpr int kOnesRows = 16;
// Register budget. `setmaxnreg.inc` blocks until the CTA's register pool -- the registers the CTA
// got at launch, kThreads x kRegsLaunch -- can satisfy it, so the two requests below must fit in
// that pool or the softmax warps would wait for ever.
constexpr int kRegsLaunch = (65536 / kThreads) / 8 * 8;      // what __launch_bounds__(kThreads, 1) yields
constexpr int kRegsSoftmax = 232;
constexpr int kRegsService = 40;
static_assert(kSoftmaxWarps * 32 * kRegsSoftmax + (kThreads - kSoftmaxWarps * 32) * kRegsService <= kThreads * kRegsLaunch,
              "setmaxnreg requests exceed the CTA's register pool");
static_assert(kRegsSoftmax % 8 == 0 && kRegsService % 8 == 0 && kRegsService >= 24, "setmaxnreg granularity");
#ifndef LBFQ_PARK_NS
#define LBFQ_PARK_NS 20000u
#endif
// Bound of every wait, in nanoseconds of the device-wide %globaltimer: far above any legitimate wait, and long enough
// to ride out a pause of the whole context (another process's start-up on the same driver has been seen to stall a
// running launch). The per-SM cycle counter is not used: it is not guaranteed to be continuous across such pauses.
constexpr long long kWaitNs = 4000000000ll;   // 4 s
__device__ __forceinline__ long long wall_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return (long long)t;
}

// ---------------------------------------------------------------------------
// PTX wrappers
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok != 0;
}
// Non-blocking test of a phase
__device__ __forceinline__ bool mbar_test(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok != 0;
}
// One probe that may park the thread for up to `ns` nanoseconds while the phase is pending (the hardware
// wakes it as soon as the phase completes), so that a waiting warp does not compete for issue slots.
__device__ __forceinline__ bool mbar_try_parked(uint32_t bar, uint32_t parity, uint32_t ns) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(bar), "r"(parity), "r"(ns) : "memory");
  return ok != 0;
}
// Bounded wait. Returns false when the wait was given up (here or elsewhere in
// the CTA); the caller must then leave its loop.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int32_t* status,
                                          int code) {
  if (mbar_try(bar, parity)) return true;
  const long long t0 = wall_ns();
  while (true) {
    if (mbar_try_parked(bar, parity, LBFQ_PARK_NS)) return true;
    if (*abort_flag) return false;
    if (wall_ns() - t0 > kWaitNs) {
      *abort_flag = 1;
      if (status) atomicCAS(status, 0, code);
      return false;
    }
  }
}

// Bounded wait for code that must stay convergent (warp-collective tcgen05.ld / st follow it): it always
// returns. When the wait is given up -- here, or earlier anywhere in the CTA -- the abort flag is set and every
// later wait falls through at once, so that all roles run to the end of their loops in step and the launch
// ends with `*status` raised and a result that the host discards.
__device__ __forceinline__ void mbar_wait_cont(uint32_t bar, uint32_t parity, volatile int* abort_flag, int32_t* status,
                                               int code) {
  if (mbar_try(bar, parity)) return;
  const long long t0 = wall_ns();
  while (!*abort_flag && !mbar_try_parked(bar, parity, LBFQ_PARK_NS)) {
    if (wall_ns() - t0 > kWaitNs) {
      *abort_flag = 1;
      if (status) atomicCAS(status, 0, code);
      return;
    }
  }
}

__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, int c0, int c1, int c2, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
      ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(bar) : "memory");
}

__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
// 32 rows x 16 bytes of shared memory -> 4 TMEM columns of lanes 0..31, replicated into every lane quarter
__device__ __forceinline__ void tc_cp_32x128b(uint32_t taddr, uint64_t sdesc) {
  asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
}

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tc_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// D[tmem] (+)= A[smem desc] . B[smem desc]^T
__device__ __forceinline__ void mma_f8_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t acc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(acc) : "memory");
}
// block-scaled: D[tmem] (+)= (A * 2^sfa)[smem desc] . (B * 2^sfb)[smem desc]^T, one UE8M0 scale per row and 32 K
__device__ __forceinline__ void mma_mxf8_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                            uint32_t sfa_tmem, uint32_t sfb_tmem, uint32_t acc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(acc), "r"(sfa_tmem), "r"(sfb_tmem) : "memory");
}
// D[tmem] (+)= A[tmem] . B[smem desc]^T
__device__ __forceinline__ void mma_f8_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t acc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(acc) : "memory");
}

// kind::f16 with BF16 operands: D[tmem] (+)= A[smem desc] . B[smem desc]^T
__device__ __forceinline__ void mma_bf16_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t acc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(acc) : "memory");
}
// ... with A read from tensor memory
__device__ __forceinline__ void mma_bf16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t acc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(acc) : "memory");
}

#define LBFQ_TMEM_LD32(r, addr)                                                                            \
  asm volatile(                                                                                           \
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "                                                           \
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "                           \
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"           \
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),   \
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]),         \
        "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]),       \
        "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]),       \
        "=r"(r[29]), "=r"(r[30]), "=r"(r[31])                                                            \
      : "r"(addr) : "memory")

#define LBFQ_TMEM_LD16(r, addr)                                                                            \
  asm volatile(                                                                                           \
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "                                                           \
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"                    \
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),   \
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]),         \
        "=r"(r[15])                                                                                       \
      : "r"(addr) : "memory")

#define LBFQ_TMEM_ST32(addr, r)                                                                            \
  asm volatile(                                                                                           \
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "                                                     \
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "                          \
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"                  \
      ::"r"(addr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), \
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),     \
        "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),   \
        "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])    \
      : "memory")

#define LBFQ_TMEM_ST16(addr, r)                                                                            \
  asm volatile(                                                                                           \
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "                                                     \
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"                          \
      ::"r"(addr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), \
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])      \
      : "memory")

template <int N>
__device__ __forceinline__ void tmem_ld(uint32_t (&r)[N], uint32_t addr) {
  static_assert(N == 16 || N == 32, "chunk of 16 or 32 columns");
  if constexpr (N == 32) { LBFQ_TMEM_LD32(r, addr); } else { LBFQ_TMEM_LD16(r, addr); }
}

__device__ __forceinline__ uint32_t tmem_ld1(uint32_t addr) {
  uint32_t v;
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x1.b32 {%0}, [%1];" : "=r"(v) : "r"(addr) : "memory");
  return v;
}
__device__ __forceinline__ void tmem_st8(uint32_t addr, const uint32_t* r) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
               ::"r"(addr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
               : "memory");
}

__device__ __forceinline__ void tmem_st4(uint32_t addr, const uint32_t* r) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x4.b32 [%0], {%1, %2, %3, %4};"
               ::"r"(addr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]) : "memory");
}

// four FP32 -> four e4m3 codes in one 32-bit word (a = byte 0 ... d = byte 3), round-to-nearest-even,
// saturating at +-448: two cvt.rn.satfinite.e4m3x2.f32 whose halves the assembler can merge in place
__device__ __forceinline__ uint32_t f32x4_to_e4m3x4(float a, float b, float c, float d) {
  uint32_t r;
  asm("{\n\t.reg .b16 lo, hi;\n\t"
      "cvt.rn.satfinite.e4m3x2.f32 lo, %2, %1;\n\t"
      "cvt.rn.satfinite.e4m3x2.f32 hi, %4, %3;\n\t"
      "mov.b32 %0, {lo, hi};\n\t}"
      : "=r"(r) : "f"(a), "f"(b), "f"(c), "f"(d));
  return r;
}

// two FP32 -> e4m3 (round-to-nearest-even, saturating) -> times `scale` in FP32 -> two BF16 in one word (a low):
// what the reference hands to its P.V product for the scaled P modes (attention_triton.py:338-360)
__device__ __forceinline__ uint32_t e4m3_round_scale_bf16x2(float a, float b, float scale) {
  float fa, fb;
  asm("{\n\t.reg .b16 c, lo, hi;\n\t.reg .b32 h2;\n\t"
      "cvt.rn.satfinite.e4m3x2.f32 c, %3, %2;\n\t"
      "cvt.rn.f16x2.e4m3x2 h2, c;\n\t"
      "mov.b32 {lo, hi}, h2;\n\t"
      "cvt.f32.f16 %0, lo;\n\t"
      "cvt.f32.f16 %1, hi;\n\t}"
      : "=f"(fa), "=f"(fb) : "f"(a), "f"(b));
  // both products in one packed multiplication: each half rounds like mul.rn.f32
  const float2 pr = __fmul2_rn(make_float2(fa, fb), make_float2(scale, scale));
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %2, %1;" : "=r"(r) : "f"(pr.x), "f"(pr.y));
  return r;
}

// acc += the two BF16 halves of `w`, each widened exactly (mixed-precision add, sm_100): lo into a, hi into b
__device__ __forceinline__ void add_bf16x2_f32(float& a, float& b, uint32_t w) {
  asm("{\n\t.reg .b16 lo, hi;\n\tmov.b32 {lo, hi}, %2;\n\t"
      "add.rn.f32.bf16 %0, lo, %0;\n\tadd.rn.f32.bf16 %1, hi, %1;\n\t}"
      : "+f"(a), "+f"(b) : "r"(w));
}

// max of three (max.f32 with three inputs, sm_100): NaN operands are dropped like fmaxf does
__device__ __forceinline__ float fmax3(float a, float b, float c) {
  float r;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
  return r;
}

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// K-major shared-memory matrix descriptor (Blackwell format, version 1):
// rows of `row_bytes` (128 -> 128B swizzle, 64 -> 64B swizzle), 8-row atoms
// packed back to back (stride byte offset = 8 * row_bytes).
__device__ __forceinline__ uint64_t make_desc(uint32_t saddr, int row_bytes) {
  const uint64_t layout = row_bytes == 128 ? 2ull : (row_bytes == 64 ? 4ull : 6ull);
  uint64_t d = 0;
  d |= (uint64_t)((saddr >> 4) & 0x3fffu);
  d |= (uint64_t)1 << 16;                                  // leading byte offset: unused for swizzled K-major
  d |= (uint64_t)(((8u * row_bytes) >> 4) & 0x3fffu) << 32;
  d |= (uint64_t)1 << 46;                                  // descriptor version
  d |= layout << 61;
  return d;
}
// kind::f8f6f4, A = B = e4m3, FP32 accumulator, both operands K-major, M = 128.
__host__ __device__ constexpr uint32_t make_idesc(int n) {
  return (1u << 4) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
}

// kind::f16, A = B = BF16, FP32 accumulator, both operands K-major, M = 128
__host__ __device__ constexpr uint32_t make_idesc_bf16(int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
}
// kind::mxf8f6f4.block_scale, e4m3 x e4m3, UE8M0 scales, K-major operands, M = 128; `sf` = which byte of
// the 32-bit scale columns (= which 32-wide K block) this instruction uses, for A and for B.
__host__ __device__ constexpr uint32_t make_idesc_mx(int n, int sf) {
  return ((uint32_t)sf << 4) | ((uint32_t)(n >> 3) << 17) | (1u << 23) | ((uint32_t)(128 >> 4) << 24) | ((uint32_t)sf << 29);
}
// 32 x 16-byte rows, contiguous (no swizzle): the source of a scale-factor copy
__device__ __forceinline__ uint64_t make_desc_sf(uint32_t saddr) {
  return (uint64_t)((saddr >> 4) & 0x3fffu) | ((uint64_t)1 << 16) | ((uint64_t)(128 >> 4) << 32) | ((uint64_t)1 << 46);
}

// ---------------------------------------------------------------------------
// kernel parameters (a device-side copy of lbfq_attn_args, pre-digested)
// ---------------------------------------------------------------------------
struct Params {
  int B, H, M, N, D;
  int qk_block;
  int qk_bf16;                 // 1: Q / K are BF16 (already de-quantised), Q.K^T is a BF16 MMA, no Q / K scales
  const float* q_scale;
  const float* k_scale;
  const uint8_t* q_sf;         // block-scaled Q/K: UE8M0 scale tiles
  const uint8_t* k_sf;
  int m_pad, n_pad;
  int v_kind;
  const float* v_scale;
  int v_block;
  float sm_scale, p_off;
  int p_kind;
  int block_m;
  const float* v_alpha;        // pre-divided by the V scale it rides on (alpha')
  int v_smooth_block;
  const float* corr;
  int q_smooth_block, corr_stride, n_groups;
  int corr_staged;             // 1: every 128-row tile lies in one Q group, corr rows go through shared memory
  int side_bytes;              // bytes of side vectors the producer stages per 128-key stage (0: none)
  const float* rowmax_est;
  const float* rowmax_init;
  int rm_mode;                 // 0 online, 1 frozen estimate, 2 estimate with thresholds
  int blasst;                  // 1: BLASST row skipping (online row max)
  int block_n;                 // keys per softmax block
  float log_lambda, lambda;
  int fill_kind;
  float fill_alpha;
  int uta_bins;
  float* stats;
  int tile_vote;               // 1: the rows of a 128-row tile vote on every key block (zero fill, no rowmax_init)
  int tile_pred;               // 1: a block is skipped only by the whole tile (the simulator's predicate)
  unsigned long long* elided;  // optional counter of (tile, block) pairs without P.V
  unsigned long long* counters; // optional row-max update counters (6), general kernel only
  void* out;
  int out_dtype, out_layout, out_exact;
  const int64_t* out_row_index;
  int32_t* status;
  // element counts of the side tensors, used by the LBFQ_BOUNDS debug build to validate every index
  long long n_v_scale, n_v_alpha, n_corr, n_qk_scale_q, n_qk_scale_k, n_out;
};

#ifdef LBFQ_BOUNDS
#define LBFQ_CHECK_IDX(idx, count, limit, code)                                                   \
  do {                                                                                            \
    if ((long long)(idx) < 0 || (long long)(idx) + (long long)(count) > (long long)(limit)) {    \
      if (p.status) atomicCAS(p.status, 0, (code));                                               \
      return;                                                                                     \
    }                                                                                             \
  } while (0)
#else
#define LBFQ_CHECK_IDX(idx, count, limit, code) do { } while (0)
#endif

// attention_fast.cu: online-softmax variant whose output accumulator lives in tensor memory
int fast_variant(const Params& p, bool blasst, bool qk_mx);
bool fast_blasst_fill(int fill_kind, int uta_bins, int block_n);
int launch_fast(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const CUtensorMap& ma, const Params& p,
                int block_n, int variant, cudaStream_t st);

}  // namespace attn
}  // namespace lbfq
