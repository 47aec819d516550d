// Streaming fake-quant attention for sm_100a: the general kernel, and the host side of lbfq_attention_fwd.
//
// Replaces `_fake_quant_attn_fwd_kernel` and its launcher
// (src/low_bit_fake_quant/attention_triton.py:48-671). Configurations in which every key block's P.V enters the
// output with weight one are dispatched to the kernel of attention_fast.cu, whose output accumulator lives in
// tensor memory; this kernel serves the rest (a per-block FP32 scale on P.V: fp8_block V; BLASST skip / fill;
// block-scaled mxfp8 Q / K; small score-bias groups or V-smoothing blocks), implements every mode, and is the
// cross-check of the other one (LBFQ_ATTN_GENERIC=1). The reference feeds
// de-quantised BF16 operands to BF16 `tl.dot`; here the e4m3 codes themselves
// are the MMA operands and every scale is applied in FP32 around the MMA:
//
//   S  = (Qc . Kc^T) * ((sq * sk) * sm_scale) [+ corr]      tcgen05.mma kind::f8f6f4, SS form,
//                                                           operands TMA-staged (128B swizzle),
//                                                           accumulator in tensor memory (TMEM)
//   P  = exp2((S - m) * log2e [+ offset]) -> e4m3           one thread per row, registers only
//   PV = Pc . Vc                                            tcgen05.mma, A = P read from TMEM (TS form),
//                                                           B = V^T tile (keys contiguous) + 16 rows of 1.0
//   A' = A' * alpha + c * (PV [* sv_d] + rowsum(Pc) * alpha_v')   FP32 registers, once per key block
//
// The per-(row, key block) arithmetic (running max, rescale factor alpha, the
// three P quantisers, V block scale, V-alpha correction, estimated-row-max
// thresholds, BLASST skip / fill and its counters) follows the reference kernel
// line by line; key blocks are walked in order with the reference's BLOCK_N so
// that every rounding decision of P sees the same running max.
//
// CTA = 256 query rows of one (b, h): two softmax warpgroups (one 128-row tile
// each, thread == row == TMEM lane), one TMA producer warp, one MMA-issuing warp
// per tile. Per tile the work is software-pipelined so that no thread waits on a
// tensor-core result it has just asked for: while block j's softmax runs, the
// tensor core computes P.V of block j-1 (P is double-buffered in TMEM) and
// Q.K^T of block j+1; block j-1's P.V is folded into the registers after block
// j's P has been handed over. K / V^T arrive in 128-key stages shared by both tiles. The extra 16
// rows of ones appended to every V^T stage make column D of the PV accumulator
// equal to rowsum(Pc), which the V-smoothing correction needs, for free.
// Every mbarrier wait is bounded; on expiry the kernel raises `*status`, all
// roles leave their loops, TMEM is released and the launch returns.

#include "attn_prims.cuh"

namespace lbfq {
namespace attn {


template <int D, int BN, bool QKBF = false>
struct Smem {
  // BF16 Q / K (the reference's de-quantised operands) double the Q tile and the K stages: two key stages then
  static constexpr int kNst = QKBF ? 2 : kStages;
  static constexpr int kQ = kTileM * D * (QKBF ? 2 : 1);      // bytes per Q tile
  static constexpr int kK = kChunk * D * (QKBF ? 2 : 1);      // bytes per K stage
  static constexpr int kV = (D + kOnesRows) * kChunk;         // bytes per V^T stage (with the rows of ones)
  static constexpr int offQ = 0;
  static constexpr int offK = offQ + 2 * kQ;
  static constexpr int offV = offK + kNst * kK;
  static constexpr int offQS = offV + kNst * kV;            // Q scale-factor tiles (block-scaled Q/K only)
  static constexpr int offKS = offQS + 2 * 512;                // K scale-factor tile per stage
  // side vectors staged per 128-key stage for the softmax threads (read with broadcast shared loads
  // instead of per-thread global loads): the score bias `corr` of each tile's Q group (128 floats per
  // tile), and per key block the V-smoothing vector alpha' and the mxfp8 V scales (D floats each)
  static constexpr int kSub = kChunk / BN;
  static constexpr int offCorr = offKS + kNst * 512;
  static constexpr int offAlpha = offCorr + kNst * 2 * kChunk * 4;
  static constexpr int offVs = offAlpha + kNst * kSub * D * 4;
  static constexpr int offBar = offVs + kNst * kSub * D * 4;
  static constexpr int kNumBar = 2 + 4 * kNst + 12 + 2 * kNst;
  static constexpr int offMisc = offBar + kNumBar * 8;
  static constexpr int offL = offMisc + 64;                   // partial row sums [tile][half][row]
  static constexpr int total = offL + 2 * 2 * kTileM * 4;
};

// ---------------------------------------------------------------------------
// the kernel
// ---------------------------------------------------------------------------
template <int D, int BN, bool BLASST, bool QKMX, bool QKBF = false>
__global__ void __launch_bounds__(kThreads, 1)
attn_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
            const __grid_constant__ CUtensorMap tm_v, const Params p) {
  static_assert(!(QKMX && QKBF), "one Q / K operand format per instantiation");
  using SM = Smem<D, BN, QKBF>;
  constexpr int NST = SM::kNst;                    // key stages
  constexpr int NSUB = kChunk / BN;                // key blocks per stage
  constexpr int PV_N = D + kOnesRows;              // PV accumulator columns
  constexpr int TCOLS = 256;                       // TMEM columns per tile
  constexpr int COL_S = 0, COL_P = 64, COL_O = 96, COL_SFA = 240, COL_SFB = 244;   // P: two buffers of 16 columns
  static_assert(BN == 32 || BN == 64, "block_n of 32 or 64");
  static_assert(COL_O + PV_N <= TCOLS, "TMEM budget");

  extern __shared__ __align__(1024) uint8_t smem_raw[];
  // rounded up to 1 KB by pointer arithmetic, so that the compiler still knows it points into shared memory
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  const uint32_t sbase = smem_u32(smem);
  const uint32_t bar0 = sbase + SM::offBar;
  // barrier map
  auto BAR_QFULL = [&](int t) { return bar0 + 8u * t; };
  auto BAR_KFULL = [&](int s) { return bar0 + 8u * (2 + s); };
  auto BAR_VFULL = [&](int s) { return bar0 + 8u * (2 + NST + s); };
  auto BAR_KFREE = [&](int s) { return bar0 + 8u * (2 + 2 * NST + s); };
  auto BAR_VFREE = [&](int s) { return bar0 + 8u * (2 + 3 * NST + s); };
  auto BAR_SFULL = [&](int t) { return bar0 + 8u * (2 + 4 * NST + t); };
  auto BAR_SFREE = [&](int t) { return bar0 + 8u * (2 + 4 * NST + 2 + t); };
  // P ready, one barrier per block parity: a warp can finish block j + 1 (whose S only waits for every thread to have
  // copied S of block j out) before a slower warp has delivered P of block j; with a single barrier that second
  // arrival would be counted into block j's phase. Two blocks ahead is impossible (S of block j + 2 waits for every
  // thread's copy of block j + 1).
  auto BAR_PRDY = [&](int t, int par) { return bar0 + 8u * (2 + 4 * NST + 4 + 2 * t + par); };
  auto BAR_PVFULL = [&](int t) { return bar0 + 8u * (2 + 4 * NST + 8 + t); };
  auto BAR_OFREE = [&](int t) { return bar0 + 8u * (2 + 4 * NST + 10 + t); };
  auto BAR_SIDEFULL = [&](int s) { return bar0 + 8u * (2 + 4 * NST + 12 + s); };
  auto BAR_SIDEFREE = [&](int s) { return bar0 + 8u * (2 + 4 * NST + 12 + NST + s); };
  volatile int* misc = (volatile int*)(smem + SM::offMisc);   // [0] tmem base, [1] abort, [2..5] elide flags, [6] early exit
  volatile int* abort_flag = misc + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int bh = blockIdx.y;
  const int b = bh / p.H, h = bh % p.H;
  const int m0 = blockIdx.x * kCtaM;
  const int nblk = (p.N + BN - 1) / BN;
  const int nchunk = (p.N + kChunk - 1) / kChunk;
  constexpr int kTmaWarp = kSoftmaxWarps, kMmaWarp0 = kSoftmaxWarps + 1;

  // ---- setup ----------------------------------------------------------------
  // A CTA scheduled after some other CTA has given up a wait retires at once.
  if (threadIdx.x == 0) misc[6] = (p.status != nullptr && *reinterpret_cast<volatile int32_t*>(p.status) != 0) ? 1 : 0;
  __syncthreads();
  if (misc[6]) return;
  if (threadIdx.x == 0) {
    for (int t = 0; t < 2; ++t) {
      mbar_init(BAR_QFULL(t), 1);
      mbar_init(BAR_SFULL(t), 1);
      mbar_init(BAR_SFREE(t), kTileM);
      mbar_init(BAR_PRDY(t, 0), kTileM);
      mbar_init(BAR_PRDY(t, 1), kTileM);
      mbar_init(BAR_PVFULL(t), 1);
      mbar_init(BAR_OFREE(t), kTileM);
    }
    for (int s = 0; s < NST; ++s) {
      mbar_init(BAR_KFULL(s), 1);
      mbar_init(BAR_VFULL(s), 1);
      mbar_init(BAR_KFREE(s), 2);
      mbar_init(BAR_VFREE(s), 2);
      mbar_init(BAR_SIDEFULL(s), 1);
      mbar_init(BAR_SIDEFREE(s), 2 * kTileM);
    }
    misc[1] = 0; misc[2] = 0; misc[3] = 0; misc[4] = 0; misc[5] = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  // rows of 1.0 (e4m3 0x38) under every V^T stage
  for (int i = threadIdx.x; i < NST * kOnesRows * kChunk / 16; i += kThreads) {
    const int s = i / (kOnesRows * kChunk / 16), r = i % (kOnesRows * kChunk / 16);
    *reinterpret_cast<uint4*>(smem + SM::offV + s * SM::kV + D * kChunk + r * 16) =
        make_uint4(0x38383838u, 0x38383838u, 0x38383838u, 0x38383838u);
  }
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  if (warp == kTmaWarp) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 512;" ::"r"(sbase + SM::offMisc) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = (uint32_t)misc[0];

  if (warp < kSoftmaxWarps) {
    // =========================== softmax warpgroups ===========================
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kRegsSoftmax));
    const int t = warp >> 2;                                   // tile
    const int row_in_tile = (warp & 3) * 32 + lane;
    const int row = m0 + t * kTileM + row_in_tile;             // query row within (b, h)
    const bool row_ok = row < p.M;
    const int rowc = row_ok ? row : (p.M - 1);
    const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
    const uint32_t tS = tmem_base + lane_base + t * TCOLS + COL_S;
    const uint32_t tP = tmem_base + lane_base + t * TCOLS + COL_P;
    const uint32_t tO = tmem_base + lane_base + t * TCOLS + COL_O;

    float sq = 1.f;
    if (p.q_scale != nullptr) sq = p.q_scale[((size_t)b * (p.M / p.qk_block) + rowc / p.qk_block) * p.H + h];
    const bool side = p.side_bytes > 0;
    const bool corr_smem = p.corr != nullptr && p.corr_staged != 0;
    const float* corr_row = nullptr;
    if (p.corr != nullptr && !corr_smem) {
      const int g = ((rowc / p.block_m) * p.block_m) / p.q_smooth_block;
      corr_row = p.corr + ((size_t)bh * p.n_groups + g) * p.corr_stride;
    }
    float m_i = -INFINITY;
    float est = 0.f;
    if (p.rowmax_est) { est = p.rowmax_est[(size_t)bh * p.M + rowc]; m_i = est; }
    else if (p.rowmax_init) { m_i = p.rowmax_init[(size_t)bh * p.M + rowc]; }
    float l_i = 0.f, max_seen = -INFINITY;
    float n_skip = 0.f, n_total = 0.f;
    int n_upd = 0, n_resc = 0, n_down = 0;       // optional diagnostic: row-max updates of this row
    float a_prev = 1.f, c_prev = 1.f;
    bool elided_prev = false;
    int blk_prev = 0;
    float acc[D];
#pragma unroll
    for (int i = 0; i < D; ++i) acc[i] = 0.f;

    // fold PV of block `jb` (scale c, rescale a) into the accumulator. The mode
    // switches are warp-uniform and hoisted out of the unrolled loops so that no
    // lane issues predicated-off work.
    auto accumulate = [&](int jb, float a, float c) {
      tc_fence_after();
      const bool rescale = __any_sync(0xffffffffu, a != 1.f);
      const bool scaled = __any_sync(0xffffffffu, c != 1.f);
      if (!p.v_alpha && p.v_kind != LBFQ_V_MX) {
#pragma unroll
        for (int c0 = 0; c0 < D; c0 += 32) {
          uint32_t r[32];
          LBFQ_TMEM_LD32(r, tO + c0);
          tc_wait_ld();
          // two columns per instruction (fma / mul / add .f32x2 round each half like the scalar forms)
          const float2 a2 = make_float2(a, a), cc2 = make_float2(c, c);
          if (rescale) {
#pragma unroll
            for (int i = 0; i < 32; i += 2) {
              const float2 v = __ffma2_rn(cc2, make_float2(__uint_as_float(r[i]), __uint_as_float(r[i + 1])),
                                          __fmul2_rn(make_float2(acc[c0 + i], acc[c0 + i + 1]), a2));
              acc[c0 + i] = v.x; acc[c0 + i + 1] = v.y;
            }
          } else if (scaled) {
#pragma unroll
            for (int i = 0; i < 32; i += 2) {
              const float2 v = __ffma2_rn(cc2, make_float2(__uint_as_float(r[i]), __uint_as_float(r[i + 1])),
                                          make_float2(acc[c0 + i], acc[c0 + i + 1]));
              acc[c0 + i] = v.x; acc[c0 + i + 1] = v.y;
            }
          } else {
#pragma unroll
            for (int i = 0; i < 32; i += 2) {
              const float2 v = __fadd2_rn(make_float2(acc[c0 + i], acc[c0 + i + 1]),
                                          make_float2(__uint_as_float(r[i]), __uint_as_float(r[i + 1])));
              acc[c0 + i] = v.x; acc[c0 + i + 1] = v.y;
            }
          }
        }
        return;
      }
      // Generic fold: per-column V scales (mxfp8 V) and / or the V-smoothing term. Both side vectors are
      // addressed through always-valid pointers (the unused one aliases the used tensor's base) and
      // selected by warp-uniform flags, never by pointer nullness.
      const bool has_av = p.v_alpha != nullptr;
      const bool has_vs = p.v_kind == LBFQ_V_MX;
      float rs = 0.f;
      if (has_av) rs = __uint_as_float(tmem_ld1(tO + D));
      // both vectors were staged by the producer with the stage that holds key block jb
      const int slot = ((jb / NSUB) % NST) * NSUB + (jb % NSUB);
      const float* av = reinterpret_cast<const float*>(smem + SM::offAlpha) + slot * D;
      const float* vs = reinterpret_cast<const float*>(smem + SM::offVs) + slot * D;
#pragma unroll
      for (int c0 = 0; c0 < D; c0 += 16) {
        uint32_t r[16];
        LBFQ_TMEM_LD16(r, tO + c0);
        tc_wait_ld();
        if (has_vs) {
          const float4* v4 = reinterpret_cast<const float4*>(vs + c0);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float4 w = v4[i];
            const float2 lo = __fmul2_rn(make_float2(__uint_as_float(r[4 * i + 0]), __uint_as_float(r[4 * i + 1])), make_float2(w.x, w.y));
            const float2 hi = __fmul2_rn(make_float2(__uint_as_float(r[4 * i + 2]), __uint_as_float(r[4 * i + 3])), make_float2(w.z, w.w));
            r[4 * i + 0] = __float_as_uint(lo.x); r[4 * i + 1] = __float_as_uint(lo.y);
            r[4 * i + 2] = __float_as_uint(hi.x); r[4 * i + 3] = __float_as_uint(hi.y);
          }
        }
        if (has_av) {
          const float4* a4 = reinterpret_cast<const float4*>(av + c0);
          const float2 rs2 = make_float2(rs, rs);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float4 w = a4[i];
            const float2 lo = __ffma2_rn(rs2, make_float2(w.x, w.y), make_float2(__uint_as_float(r[4 * i + 0]), __uint_as_float(r[4 * i + 1])));
            const float2 hi = __ffma2_rn(rs2, make_float2(w.z, w.w), make_float2(__uint_as_float(r[4 * i + 2]), __uint_as_float(r[4 * i + 3])));
            r[4 * i + 0] = __float_as_uint(lo.x); r[4 * i + 1] = __float_as_uint(lo.y);
            r[4 * i + 2] = __float_as_uint(hi.x); r[4 * i + 3] = __float_as_uint(hi.y);
          }
        }
        const float2 a2 = make_float2(a, a), cc2 = make_float2(c, c);
        if (rescale) {
#pragma unroll
          for (int i = 0; i < 16; i += 2) {
            const float2 v = __ffma2_rn(cc2, make_float2(__uint_as_float(r[i]), __uint_as_float(r[i + 1])),
                                        __fmul2_rn(make_float2(acc[c0 + i], acc[c0 + i + 1]), a2));
            acc[c0 + i] = v.x; acc[c0 + i + 1] = v.y;
          }
        } else {
#pragma unroll
          for (int i = 0; i < 16; i += 2) {
            const float2 v = __ffma2_rn(cc2, make_float2(__uint_as_float(r[i]), __uint_as_float(r[i + 1])),
                                        make_float2(acc[c0 + i], acc[c0 + i + 1]));
            acc[c0 + i] = v.x; acc[c0 + i + 1] = v.y;
          }
        }
      }
    };

    bool alive = true;
    for (int it = 0; it < nblk && alive; ++it) {
      // ---- (b) S -> P -------------------------------------------------------------
      if (!mbar_wait(BAR_SFULL(t), it & 1, abort_flag, p.status, 12)) { alive = false; break; }
      tc_fence_after();
      float s[BN];
      {
        uint32_t r[32];
        LBFQ_TMEM_LD32(r, tS);
        if constexpr (BN == 64) {
          uint32_t r2[32];
          LBFQ_TMEM_LD32(r2, tS + 32);
          tc_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; ++i) { s[i] = __uint_as_float(r[i]); s[32 + i] = __uint_as_float(r2[i]); }
        } else {
          tc_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; ++i) s[i] = __uint_as_float(r[i]);
        }
      }
      tc_fence_before();
      mbar_arrive(BAR_SFREE(t));

      const int n0 = it * BN;
      const int nvalid = min(BN, p.N - n0);
      float f = p.sm_scale;
      if (p.k_scale) {
        const float sk = p.k_scale[((size_t)b * (p.N / p.qk_block) + n0 / p.qk_block) * p.H + h];
        f = (sq * sk) * p.sm_scale;
      }
      if (side && (it % NSUB) == 0) {        // first key block of a stage: its side vectors must have landed
        const int c = it / NSUB;
        if (!mbar_wait(BAR_SIDEFULL(c % NST), (c / NST) & 1, abort_flag, p.status, 15)) { alive = false; break; }
      }
      const float2 f2 = make_float2(f, f);
      if (corr_smem) {
        const float4* c4 = reinterpret_cast<const float4*>(
            smem + SM::offCorr + (((it / NSUB) % NST) * 2 + t) * (kChunk * 4) + (it % NSUB) * (BN * 4));
#pragma unroll
        for (int i = 0; i < BN / 4; ++i) {
          const float4 cv = c4[i];               // same address in every lane: one broadcast wavefront
          const float2 lo = __ffma2_rn(make_float2(s[4 * i + 0], s[4 * i + 1]), f2, make_float2(cv.x, cv.y));
          const float2 hi = __ffma2_rn(make_float2(s[4 * i + 2], s[4 * i + 3]), f2, make_float2(cv.z, cv.w));
          s[4 * i + 0] = lo.x; s[4 * i + 1] = lo.y; s[4 * i + 2] = hi.x; s[4 * i + 3] = hi.y;
        }
      } else if (corr_row) {
        const float4* c4 = reinterpret_cast<const float4*>(corr_row + n0);
#pragma unroll
        for (int i = 0; i < BN / 4; ++i) {
          const float4 cv = __ldg(c4 + i);
          const float2 lo = __ffma2_rn(make_float2(s[4 * i + 0], s[4 * i + 1]), f2, make_float2(cv.x, cv.y));
          const float2 hi = __ffma2_rn(make_float2(s[4 * i + 2], s[4 * i + 3]), f2, make_float2(cv.z, cv.w));
          s[4 * i + 0] = lo.x; s[4 * i + 1] = lo.y; s[4 * i + 2] = hi.x; s[4 * i + 3] = hi.y;
        }
      } else {
#pragma unroll
        for (int i = 0; i < BN; i += 2) {
          const float2 v = __fmul2_rn(make_float2(s[i], s[i + 1]), f2);
          s[i] = v.x; s[i + 1] = v.y;
        }
      }
      if (nvalid < BN) {                    // ragged tail: only the last block of a sequence
#pragma unroll
        for (int i = 0; i < BN; ++i) if (i >= nvalid) s[i] = -INFINITY;
      }
      float bm0 = s[0], bm1 = s[1], bm2 = s[2], bm3 = s[3];
#pragma unroll
      for (int i = 4; i < BN; i += 4) {
        bm0 = fmaxf(bm0, s[i]); bm1 = fmaxf(bm1, s[i + 1]); bm2 = fmaxf(bm2, s[i + 2]); bm3 = fmaxf(bm3, s[i + 3]);
      }
      const float bmax = fmaxf(fmaxf(bm0, bm1), fmaxf(bm2, bm3));

      // ---- running max / rescale factor (attention_triton.py:164-217) ----------
      float m_new, alpha;
      bool skip = false;
      if (BLASST) {
        m_new = fmaxf(m_i, bmax);
        skip = (bmax - m_new) < p.log_lambda;
        alpha = skip ? 1.f : ex2((m_i - m_new) * kLog2e);
        if (skip) m_new = m_i;
        n_skip += (skip && row_ok) ? 1.f : 0.f;
        n_total += row_ok ? 1.f : 0.f;
      } else if (p.rm_mode == 2) {
        const float seen = fmaxf(max_seen, bmax);
        const float up = 16.0f / kLog2e, down = 32.0f / kLog2e;
        const bool under = (bmax - m_i) > up;
        const bool over = (m_i - seen) > down;
        const float down_m = (l_i == 0.f) ? seen : fmaxf(seen + down, m_i - 80.0f);
        m_new = (under || over) ? (under ? bmax : down_m) : m_i;
        alpha = (under || over) ? ((l_i == 0.f) ? 0.f : ex2((m_i - m_new) * kLog2e)) : 1.f;
        max_seen = seen;
      } else if (p.rm_mode == 1) {
        m_new = est;
        alpha = 1.f;
      } else {
        m_new = fmaxf(m_i, bmax);
        alpha = ex2((m_i - m_new) * kLog2e);
      }

      if (p.counters != nullptr) {
        // an update moves the row's reference max; it costs a rescale when the row already holds mass
        bool adjust, downward = false;
        if (!BLASST && p.rm_mode == 2) {
          adjust = m_new != m_i;
          downward = adjust && !((bmax - m_i) > 16.0f / kLog2e);
        } else {
          adjust = m_new > m_i;
        }
        n_upd += adjust ? 1 : 0;
        n_resc += (adjust && l_i != 0.f) ? 1 : 0;
        n_down += downward ? 1 : 0;
      }

      // whole-tile elision: every row of this 128-row tile skips and nothing is filled in
      bool elide = false;
      if (BLASST) {
        if (p.fill_kind == LBFQ_FILL_ZERO) {
          uint32_t all;
          asm volatile(
              "{\n\t.reg .pred pi, po;\n\tsetp.ne.b32 pi, %1, 0;\n\t"
              "barrier.cta.red.and.pred po, %2, 128, pi;\n\tselp.u32 %0, 1, 0, po;\n\t}"
              : "=r"(all) : "r"((uint32_t)(skip || !row_ok)), "r"(1 + t) : "memory");
          elide = all != 0;
        }
      }

      float c_blk = 1.f;
      if (!elide) {
        // ---- P = exp2(z), l += sum(P) (attention_triton.py:219-326) -------------
        // z = (s - m) * log2e + off in every mode (off = 0 for the scaled P modes, where the
        // product alone is what the reference computes: fma(x, c, 0) == x * c).
        const float off = p.p_kind == LBFQ_P_ELEMENTWISE ? p.p_off : 0.f;
        float psum, pmax;
        if (BLASST && skip) {
          // a skipped row contributes only its softmax-free fill (zero for the "zero" fill)
          psum = 0.f; pmax = 0.f;
          if (p.fill_kind == LBFQ_FILL_ZERO) {
#pragma unroll
            for (int i = 0; i < BN; ++i) s[i] = 0.f;
          } else {
            const float safe_n = (float)max(nvalid, 1);
            float sum = 0.f;
#pragma unroll
            for (int i = 0; i < BN; ++i) sum += (i < nvalid) ? s[i] : 0.f;
            const float mean = sum / safe_n;
            const float max_bound = safe_n * ex2((bmax - m_new) * kLog2e + off);
            float fill_p = 0.f;
            if (p.fill_kind == LBFQ_FILL_MAX) {
              fill_p = max_bound * p.fill_alpha / safe_n;
            } else if (p.fill_kind == LBFQ_FILL_MEAN) {
              fill_p = fminf(p.fill_alpha * safe_n * ex2((mean - m_new) * kLog2e + off), max_bound) / safe_n;
            } else if (p.fill_kind == LBFQ_FILL_LOGN) {
              float v2 = 0.f;
#pragma unroll
              for (int i = 0; i < BN; ++i) { const float cd = (i < nvalid) ? s[i] - mean : 0.f; v2 += cd * cd; }
              const float var = v2 / safe_n;
              fill_p = fminf(safe_n * ex2((mean + 0.5f * var - m_new) * kLog2e + off), max_bound) / safe_n;
            } else if (p.fill_kind == LBFQ_FILL_SAMPLE8) {
              const int stride = BN >= 8 ? BN / 8 : 1;
              float ssum = 0.f, cnt = 0.f;
#pragma unroll
              for (int i = 0; i < BN; i += stride)
                if (i < nvalid) { ssum += ex2((s[i] - m_new) * kLog2e + off); cnt += 1.f; }
              fill_p = fminf(p.fill_alpha * safe_n * ssum / fmaxf(cnt, 1.f), max_bound) / safe_n;
            } else if (p.fill_kind == LBFQ_FILL_THR) {
              const float off_scale = p.p_kind == LBFQ_P_ELEMENTWISE ? exp2f(p.p_off) : 1.f;
              fill_p = (p.fill_alpha * safe_n * p.lambda * off_scale) / safe_n;
            }
            if (p.fill_kind != LBFQ_FILL_UTA) {
#pragma unroll
              for (int i = 0; i < BN; ++i) s[i] = (i < nvalid) ? fill_p : 0.f;
              psum = fill_p * 0.f;
#pragma unroll
              for (int i = 0; i < BN; ++i) psum += s[i];
              pmax = fill_p;
            } else {                                           // UTA: one value per bin of BN / bins keys
              const int bin_size = BN / p.uta_bins;
              float bsum = 0.f, bmx = -INFINITY, bcnt = 0.f;
              int first = 0;
#pragma unroll
              for (int i = 0; i < BN; ++i) {
                if (i < nvalid) { bsum += s[i]; bmx = fmaxf(bmx, s[i]); bcnt += 1.f; }
                if (((i + 1) % bin_size) == 0) {
                  const float safe_c = fmaxf(bcnt, 1.f);
                  const float bound = safe_c * ex2((bmx - m_new) * kLog2e + off);
                  const float mass = p.fill_alpha * safe_c * ex2((bsum / safe_c - m_new) * kLog2e + off);
                  const float val = fminf(mass, bound) / safe_c;
#pragma unroll
                  for (int q = 0; q < BN; ++q)
                    if (q >= first && q <= i) s[q] = (q < nvalid) ? val : 0.f;
                  first = i + 1; bsum = 0.f; bmx = -INFINITY; bcnt = 0.f;
                }
              }
#pragma unroll
              for (int i = 0; i < BN; ++i) { psum += s[i]; pmax = fmaxf(pmax, s[i]); }
            }
          }
        } else {
          // masked columns hold -inf, so their exp2 is exactly 0 without a select
          float2 psa = make_float2(0.f, 0.f), psb = make_float2(0.f, 0.f);
          const float2 nm2 = make_float2(-m_new, -m_new), l2 = make_float2(kLog2e, kLog2e), off2 = make_float2(off, off);
#pragma unroll
          for (int i = 0; i < BN; i += 4) {
            const float2 za = __ffma2_rn(__fadd2_rn(make_float2(s[i], s[i + 1]), nm2), l2, off2);
            const float2 zb = __ffma2_rn(__fadd2_rn(make_float2(s[i + 2], s[i + 3]), nm2), l2, off2);
            const float2 pa = make_float2(ex2(za.x), ex2(za.y));
            const float2 pb = make_float2(ex2(zb.x), ex2(zb.y));
            s[i] = pa.x; s[i + 1] = pa.y; s[i + 2] = pb.x; s[i + 3] = pb.y;
            psa = __fadd2_rn(psa, pa);
            psb = __fadd2_rn(psb, pb);
          }
          psum = (psa.x + psa.y) + (psb.x + psb.y);
          // exp2 is monotonic: the largest P of the block is the P of the largest score, and it is
          // produced by the same instruction sequence, so it is bit-identical to max_i(P_i)
          pmax = ex2(fmaf(bmax - m_new, kLog2e, off));
        }
        l_i = l_i * alpha + psum;

        // ---- P quantisation (attention_triton.py:328-360) -----------------------
        uint32_t pk[BN / 4];
        if (p.p_kind == LBFQ_P_ELEMENTWISE) {
#pragma unroll
          for (int i = 0; i < BN / 4; ++i)
            pk[i] = f32x4_to_e4m3x4(s[4 * i], s[4 * i + 1], s[4 * i + 2], s[4 * i + 3]);
        } else {
          float inv;
          if (p.p_kind == LBFQ_P_MX) {
            const int e = pow2_scale_exp(fmaxf(pmax, 1e-4f));
            c_blk = pow2f(e);
            inv = pow2f(-e);
          } else {
            c_blk = scale_from_amax(fmaxf(pmax, 1e-12f));      // the reference's `amax / 448` and `p / s` (common.cuh)
            inv = rcp_approx(c_blk);
          }
          // the conversion saturates at 448, which is the reference's clamp
          const float2 inv2 = make_float2(inv, inv);
#pragma unroll
          for (int i = 0; i < BN / 4; ++i) {
            const float2 lo = __fmul2_rn(make_float2(s[4 * i], s[4 * i + 1]), inv2);
            const float2 hi = __fmul2_rn(make_float2(s[4 * i + 2], s[4 * i + 3]), inv2);
            pk[i] = f32x4_to_e4m3x4(lo.x, lo.y, hi.x, hi.y);
          }
        }
        const uint32_t tPb = tP + (it & 1) * 16;
        tmem_st8(tPb, pk);
        if constexpr (BN == 64) tmem_st8(tPb + 8, pk + 8);
        tc_wait_st();
      }
      if (p.v_kind == LBFQ_V_BLOCK)
        c_blk *= p.v_scale[((size_t)b * (p.N / p.v_block) + n0 / p.v_block) * p.H + h];
      if (BLASST && row_in_tile == 0) misc[2 + 2 * t + (it & 1)] = elide ? 1 : 0;   // per P buffer
      tc_fence_before();
      mbar_arrive(BAR_PRDY(t, it & 1));
      // ---- fold the previous block's P.V (issued while this block's softmax ran), then hand the
      // scratch accumulator back so that this block's P.V may be issued
      if (it > 0) {
        if (!mbar_wait(BAR_PVFULL(t), (it - 1) & 1, abort_flag, p.status, 11)) { alive = false; break; }
        if (!elided_prev) accumulate(blk_prev, a_prev, c_prev);
        tc_fence_before();
        mbar_arrive(BAR_OFREE(t));
        // the side vectors of a stage are dead once its last key block has been folded
        if (side && (blk_prev % NSUB) == NSUB - 1) mbar_arrive(BAR_SIDEFREE((blk_prev / NSUB) % NST));
      }
      a_prev = alpha; c_prev = c_blk; elided_prev = elide; blk_prev = it;
      m_i = m_new;
    }
    if (alive) {
      if (mbar_wait(BAR_PVFULL(t), (nblk - 1) & 1, abort_flag, p.status, 13)) {
        if (!elided_prev) accumulate(blk_prev, a_prev, c_prev);
      } else {
        alive = false;
      }
    }

    // ---- epilogue (attention_triton.py:387-407) ---------------------------------
    if (alive && row_ok) {
      const float inv_l = rcp_approx(l_i);                       // the reference's `1.0 / l_i` (attention_triton.py:387)
      const bool has_vsc = p.v_kind == LBFQ_V_CHANNEL;             // selected by flag; the pointer is always valid
      const float* vsc = has_vsc ? p.v_scale + (size_t)bh * D : p.v_scale;
      int64_t drow = row;
      if (p.out_row_index != nullptr) drow = p.out_row_index[(size_t)bh * p.M + row];
      const size_t o_off = p.out_layout == LBFQ_LAYOUT_NHD
                               ? (((size_t)b * p.M + drow) * p.H + h) * D
                               : ((size_t)bh * p.M + drow) * D;
      if (has_vsc) {
#pragma unroll
        for (int i = 0; i < D; ++i) acc[i] = (acc[i] * vsc[i]) * inv_l;
      } else {
#pragma unroll
        for (int i = 0; i < D; ++i) acc[i] = acc[i] * inv_l;
      }
      if (p.out_dtype == LBFQ_F32) {
        float4* o = reinterpret_cast<float4*>((float*)p.out + o_off);
#pragma unroll
        for (int i = 0; i < D / 4; ++i) {
          float4 v = make_float4(acc[4 * i], acc[4 * i + 1], acc[4 * i + 2], acc[4 * i + 3]);
          if (!p.out_exact) {
            v.x = round_through<__nv_bfloat16>(v.x); v.y = round_through<__nv_bfloat16>(v.y);
            v.z = round_through<__nv_bfloat16>(v.z); v.w = round_through<__nv_bfloat16>(v.w);
          }
          o[i] = v;
        }
      } else {
        uint4* o = reinterpret_cast<uint4*>((uint16_t*)p.out + o_off);
#pragma unroll
        for (int i = 0; i < D / 8; ++i) {
          uint32_t w[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float x0 = acc[8 * i + 2 * j], x1 = acc[8 * i + 2 * j + 1];
            if (p.out_dtype == LBFQ_BF16) {
              __nv_bfloat162 hh = __floats2bfloat162_rn(x0, x1);
              w[j] = *reinterpret_cast<uint32_t*>(&hh);
            } else {                                           // the kernel result is BF16; then .to(float16)
              __half2 hh = __floats2half2_rn(round_through<__nv_bfloat16>(x0), round_through<__nv_bfloat16>(x1));
              w[j] = *reinterpret_cast<uint32_t*>(&hh);
            }
          }
          o[i] = make_uint4(w[0], w[1], w[2], w[3]);
        }
      }
    }
    if (p.counters != nullptr) {                  // every lane takes part in the warp sums
      const bool live = row_ok && alive;
      const unsigned long long upd = live ? n_upd : 0, resc = live ? n_resc : 0, down = live ? n_down : 0;
      auto warp_sum = [](unsigned long long v) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
        return v;
      };
      const unsigned long long s_upd = warp_sum(upd), s_resc = warp_sum(resc), s_down = warp_sum(down);
      const unsigned long long s_rows = warp_sum(upd > 0 ? 1ull : 0ull);
      unsigned int mx = (unsigned int)upd;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) mx = max(mx, __shfl_xor_sync(0xffffffffu, mx, o));
      if (lane == 0) {
        atomicAdd(p.counters + 0, s_upd);
        atomicAdd(p.counters + 1, s_resc);
        atomicAdd(p.counters + 2, s_upd - s_down);
        atomicAdd(p.counters + 3, s_down);
        atomicAdd(p.counters + 4, s_rows);
        atomicMax(p.counters + 5, (unsigned long long)mx);
      }
    }
    if (BLASST && alive && row_ok && p.stats) {
      const int mb = row / p.block_m;
      atomicAdd(p.stats + ((size_t)mb * (p.B * p.H) + bh) * 2 + 0, n_skip);
      atomicAdd(p.stats + ((size_t)mb * (p.B * p.H) + bh) * 2 + 1, n_total);
    }
  } else {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegsService));
  }
  if (warp == kTmaWarp) {
    // =========================== TMA producer =====================================
    if (lane == 0) {
      for (int t = 0; t < 2; ++t) {
        mbar_expect_tx(BAR_QFULL(t), SM::kQ + (QKMX ? 512 : 0));
        if constexpr (QKBF) {                               // BF16: D / 64 panels of 128 rows x 128 bytes
          for (int pn = 0; pn < D / 64; ++pn)
            tma_load_3d(sbase + SM::offQ + t * SM::kQ + pn * (kTileM * 128), &tm_q, pn * 64, m0 + t * kTileM, bh, BAR_QFULL(t));
        } else {
          tma_load_3d(sbase + SM::offQ + t * SM::kQ, &tm_q, 0, m0 + t * kTileM, bh, BAR_QFULL(t));
        }
        if (QKMX) {
          // a tile beyond the padded rows has no scale tile: re-read the last one (its codes are zero-filled)
          const int tile128 = min((m0 + t * kTileM) >> 7, (p.m_pad >> 7) - 1);
          bulk_load(sbase + SM::offQS + t * 512, p.q_sf + ((size_t)bh * (p.m_pad >> 7) + tile128) * 512, 512, BAR_QFULL(t));
        }
      }
      for (int c = 0; c < nchunk; ++c) {
        const int st = c % NST;
        if (c >= NST) {
          const uint32_t par = ((c / NST) - 1) & 1;
          if (!mbar_wait(BAR_KFREE(st), par, abort_flag, p.status, 21)) break;
          if (!mbar_wait(BAR_VFREE(st), par, abort_flag, p.status, 22)) break;
        }
        mbar_expect_tx(BAR_KFULL(st), SM::kK + (QKMX ? 512 : 0));
        if constexpr (QKBF) {
          for (int pn = 0; pn < D / 64; ++pn)
            tma_load_3d(sbase + SM::offK + st * SM::kK + pn * (kChunk * 128), &tm_k, pn * 64, c * kChunk, bh, BAR_KFULL(st));
        } else {
          tma_load_3d(sbase + SM::offK + st * SM::kK, &tm_k, 0, c * kChunk, bh, BAR_KFULL(st));
        }
        if (QKMX) bulk_load(sbase + SM::offKS + st * 512, p.k_sf + ((size_t)bh * (p.n_pad >> 7) + c) * 512, 512, BAR_KFULL(st));
        mbar_expect_tx(BAR_VFULL(st), D * kChunk);
        tma_load_3d(sbase + SM::offV + st * SM::kV, &tm_v, c * kChunk, 0, bh, BAR_VFULL(st));
        if (p.side_bytes > 0) {
          if (c >= NST && !mbar_wait(BAR_SIDEFREE(st), ((c / NST) - 1) & 1, abort_flag, p.status, 23)) break;
          mbar_expect_tx(BAR_SIDEFULL(st), p.side_bytes);
          if (p.corr != nullptr && p.corr_staged) {
            for (int t = 0; t < 2; ++t) {
              const int g = min((m0 + t * kTileM) / p.q_smooth_block, p.n_groups - 1);
              bulk_load(sbase + SM::offCorr + (st * 2 + t) * (kChunk * 4),
                        p.corr + ((size_t)bh * p.n_groups + g) * p.corr_stride + (size_t)c * kChunk, kChunk * 4, BAR_SIDEFULL(st));
            }
          }
          for (int sub = 0; sub < NSUB; ++sub) {
            const int key = min(c * kChunk + sub * BN, p.N - 1);     // a block past the end re-reads the last one
            if (p.v_alpha != nullptr)
              bulk_load(sbase + SM::offAlpha + (st * NSUB + sub) * (D * 4),
                        p.v_alpha + (((size_t)b * (p.N / p.v_smooth_block) + key / p.v_smooth_block) * p.H + h) * D, D * 4,
                        BAR_SIDEFULL(st));
            if (p.v_kind == LBFQ_V_MX)
              bulk_load(sbase + SM::offVs + (st * NSUB + sub) * (D * 4),
                        p.v_scale + (((size_t)b * (p.N / p.v_block) + key / p.v_block) * p.H + h) * D, D * 4,
                        BAR_SIDEFULL(st));
          }
        }
      }
    }
  } else if (warp == kMmaWarp0 || warp == kMmaWarp0 + 1) {
    // =========================== MMA issuer of tile t ==============================
    const int t = warp - kMmaWarp0;
    if (lane == 0) {
      const uint32_t tS = tmem_base + t * TCOLS + COL_S;
      const uint32_t tP = tmem_base + t * TCOLS + COL_P;
      const uint32_t tO = tmem_base + t * TCOLS + COL_O;
      const uint32_t id_qk = make_idesc(BN);
      const uint32_t id_pv = make_idesc(PV_N);
      const uint64_t dq = make_desc(sbase + SM::offQ + t * SM::kQ, D);
      const uint32_t tSFA = tmem_base + t * TCOLS + COL_SFA;
      const uint32_t tSFB = tmem_base + t * TCOLS + COL_SFB;
      bool ok = mbar_wait(BAR_QFULL(t), 0, abort_flag, p.status, 31);
      if (QKMX && ok) tc_cp_32x128b(tSFA, make_desc_sf(sbase + SM::offQS + t * 512));
      auto issue_qk = [&](int j) -> bool {
        const int c = j / NSUB, sub = j % NSUB, st = c % NST;
        if (sub == 0 && !mbar_wait(BAR_KFULL(st), (c / NST) & 1, abort_flag, p.status, 32)) return false;
        tc_fence_after();
        const uint64_t dk = make_desc(sbase + SM::offK + st * SM::kK + sub * BN * D, D);
        if constexpr (QKMX) {
          // scale factors of this stage's 128 keys: 4 columns, one per group of 32 keys; tcgen05 operations
          // issued by one thread execute in order, so the copy cannot overtake earlier MMAs that read them
          if (sub == 0) tc_cp_32x128b(tSFB, make_desc_sf(sbase + SM::offKS + st * 512));
#pragma unroll
          for (int kk = 0; kk < D / 32; ++kk)
            mma_mxf8_ss(tS, dq + (uint64_t)(kk * 2), dk + (uint64_t)(kk * 2), make_idesc_mx(BN, kk), tSFA,
                        tSFB + sub * (BN / 32), kk > 0 ? 1u : 0u);
        } else if constexpr (QKBF) {
          // BF16 operands: K steps of 16 channels, four per 64-channel panel
          const uint32_t id_qk_bf16 = make_idesc_bf16(BN);
#pragma unroll
          for (int kk = 0; kk < D / 16; ++kk) {
            const uint64_t da = make_desc(sbase + SM::offQ + t * SM::kQ + (kk >> 2) * (kTileM * 128), 128) + (uint64_t)((kk & 3) * 2);
            const uint64_t db = make_desc(sbase + SM::offK + st * SM::kK + (kk >> 2) * (kChunk * 128) + sub * BN * 128, 128) +
                                (uint64_t)((kk & 3) * 2);
            mma_bf16_ss(tS, da, db, id_qk_bf16, kk > 0 ? 1u : 0u);
          }
        } else {
#pragma unroll
          for (int kk = 0; kk < D / 32; ++kk)
            mma_f8_ss(tS, dq + (uint64_t)(kk * 2), dk + (uint64_t)(kk * 2), id_qk, kk > 0 ? 1u : 0u);
        }
        tc_commit(BAR_SFULL(t));
        if (sub == NSUB - 1 || j == nblk - 1) tc_commit(BAR_KFREE(st));
        return true;
      };
      auto issue_pv = [&](int j) -> bool {
        const int c = j / NSUB, sub = j % NSUB, st = c % NST;
        if (sub == 0 && !mbar_wait(BAR_VFULL(st), (c / NST) & 1, abort_flag, p.status, 33)) return false;
        tc_fence_after();
        const bool elide = BLASST && misc[2 + 2 * t + (j & 1)] != 0;
        if (!elide) {
          const uint64_t dv = make_desc(sbase + SM::offV + st * SM::kV, kChunk);
#pragma unroll
          for (int kk = 0; kk < BN / 32; ++kk)
            mma_f8_ts(tO, tP + (j & 1) * 16 + kk * 8, dv + (uint64_t)((sub * BN + kk * 32) >> 4), id_pv, kk > 0 ? 1u : 0u);
        }
        tc_commit(BAR_PVFULL(t));
        if (sub == NSUB - 1 || j == nblk - 1) tc_commit(BAR_VFREE(st));
        return true;
      };
      if (ok) ok = issue_qk(0);
      for (int it = 0; it < nblk && ok; ++it) {
        // Q.K^T of the next block as soon as the softmax threads have copied S out
        if (it + 1 < nblk) {
          ok = mbar_wait(BAR_SFREE(t), it & 1, abort_flag, p.status, 34) && issue_qk(it + 1);
          if (!ok) break;
        }
        // P.V of this block once its P is in TMEM and the previous P.V has been folded
        ok = mbar_wait(BAR_PRDY(t, it & 1), (it >> 1) & 1, abort_flag, p.status, 35);
        if (ok && it > 0) ok = mbar_wait(BAR_OFREE(t), (it - 1) & 1, abort_flag, p.status, 36);
        if (ok) ok = issue_pv(it);
      }
    }
  }

  // ---- teardown -------------------------------------------------------------------
  tc_fence_before();
  __syncthreads();
  if (warp == kTmaWarp) {
    if (*abort_flag && lane == 0) {
      // give in-flight bulk copies a bounded time to land before the CTA retires
      const long long t0 = wall_ns();
      while (wall_ns() - t0 < 1000000ll) { }
    }
    __syncwarp();
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 512;" ::"r"(tmem_base) : "memory");
  }
}

// ---------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------
static PFN_cuTensorMapEncodeTiled_v12000 get_encode() {
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

// 3-D u8 tensor map: dims (inner, rows, slabs), box (box_inner, box_rows, 1)
static int make_map(CUtensorMap* map, const void* base, uint64_t inner, uint64_t rows, uint64_t slabs,
                    uint32_t box_inner, uint32_t box_rows) {
  auto enc = get_encode();
  LBFQ_REQUIRE(enc != nullptr, LBFQ_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
  cuuint64_t dims[3] = {inner, rows, slabs};
  cuuint64_t strides[2] = {inner, inner * rows};
  cuuint32_t box[3] = {box_inner, box_rows, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUtensorMapSwizzle sw = box_inner == 128 ? CU_TENSOR_MAP_SWIZZLE_128B
                          : box_inner == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_32B;
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  LBFQ_REQUIRE(r == CUDA_SUCCESS, LBFQ_ERR_CUDA, "cuTensorMapEncodeTiled failed with code %d", (int)r);
  return LBFQ_OK;
}

// 3-D bf16 tensor map: dims (inner, rows, slabs) in elements, box (box_inner <= 64 elements, box_rows, 1), 128B swizzle
static int make_map_bf16(CUtensorMap* map, const void* base, uint64_t inner, uint64_t rows, uint64_t slabs,
                         uint32_t box_inner, uint32_t box_rows) {
  auto enc = get_encode();
  LBFQ_REQUIRE(enc != nullptr, LBFQ_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
  cuuint64_t dims[3] = {inner, rows, slabs};
  cuuint64_t strides[2] = {inner * 2, inner * rows * 2};
  cuuint32_t box[3] = {box_inner, box_rows, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  LBFQ_REQUIRE(r == CUDA_SUCCESS, LBFQ_ERR_CUDA, "cuTensorMapEncodeTiled (bf16) failed with code %d", (int)r);
  return LBFQ_OK;
}

template <int D, int BN, bool BLASST, bool QKMX, bool QKBF = false>
static int launch(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const Params& p, cudaStream_t st) {
  using SM = Smem<D, BN, QKBF>;
  const int smem_bytes = SM::total + 1024;
  static_assert(SM::total + 1024 <= 227 * 1024, "shared memory of one CTA");
  auto kern = attn_kernel<D, BN, BLASST, QKMX, QKBF>;
  LBFQ_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes));
  dim3 grid((p.M + kCtaM - 1) / kCtaM, p.B * p.H, 1);
  kern<<<grid, kThreads, smem_bytes, st>>>(mq, mk, mv, p);
  return check_launch("attn_kernel");
}

}  // namespace attn
}  // namespace lbfq

using namespace lbfq;

// v_alpha' = v_alpha / (the V scale that multiplies the same PV term), written at granularity `g` keys: the smoothing
// block itself, or -- with a per-block V scale whose blocks are not the smoothing blocks -- their common divisor, so
// that every entry has one smoothing value and one scale
__global__ void alpha_prep_kernel(const float* __restrict__ alpha, float* __restrict__ out, const float* __restrict__ vscale,
                                  int v_kind, int B, int N, int H, int D, int g, int v_smooth_block, int v_block) {
  const int NB = N / g;
  const size_t total = (size_t)B * NB * H * D;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const int d = (int)(i % D);
    const int h = (int)((i / D) % H);
    const int nb = (int)((i / D / H) % NB);
    const int b = (int)(i / D / H / NB);
    const int key = nb * g;
    float a = alpha[(((size_t)b * (N / v_smooth_block) + key / v_smooth_block) * H + h) * D + d];
    if (v_kind == LBFQ_V_CHANNEL) a = __fdiv_rn(a, vscale[((size_t)b * H + h) * D + d]);
    else if (v_kind == LBFQ_V_BLOCK) a = __fdiv_rn(a, vscale[((size_t)b * (N / v_block) + key / v_block) * H + h]);
    out[i] = a;
  }
}

// V^T codes (B*H, D, n_pad) e4m3 -> BF16 of the same layout for the BF16 P.V of the TMEM-resident kernel: the codes
// themselves (per-channel V: the channel scale is applied in the epilogue) or codes * 2^e (mxfp8 V: exact in BF16,
// the operand the reference builds at attention.py:571-586)
__global__ void v_codes_to_bf16_kernel(const uint8_t* __restrict__ codes, __nv_bfloat16* __restrict__ out, int v_kind,
                                       const float* __restrict__ vscale, int B, int H, int D, int N, int n_pad, int v_block) {
  const size_t total8 = (size_t)B * H * D * n_pad / 8;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total8; i += (size_t)gridDim.x * blockDim.x) {
    const size_t e0 = i * 8;
    const int key0 = (int)(e0 % n_pad);
    const int d = (int)((e0 / n_pad) % D);
    const int bh = (int)(e0 / n_pad / D);
    const uint2 raw = *reinterpret_cast<const uint2*>(codes + e0);
    const uint8_t* c8 = reinterpret_cast<const uint8_t*>(&raw);
    float sc = 1.f;
    if (v_kind == LBFQ_V_MX) {
      const int b = bh / H, h = bh % H;
      const int blk = min(key0, N - 1) / v_block;              // 8 consecutive keys never straddle a block
      sc = vscale[(((size_t)b * (N / v_block) + blk) * H + h) * D + d];
    }
    __align__(16) __nv_bfloat16 o[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = __float2bfloat16_rn(e4m3_to_f32(c8[j]) * sc);
    *reinterpret_cast<uint4*>(out + e0) = *reinterpret_cast<const uint4*>(o);
  }
}

// mxfp8 Q / K codes (B, H, s_pad, D) with their UE8M0 scale tiles (the layout lbfq_mxfp8_qk_quant writes) -> BF16
// code * 2^e, which is exact: a power-of-two scale moves only the exponent. The TMEM-resident kernel has no columns
// left for scale factors next to two S buffers and a 128-column accumulator per tile, so it multiplies these as BF16
// operands: the same products as the block-scaled FP8 MMA, accumulated in FP32.
__global__ void qk_mx_to_bf16_kernel(const uint8_t* __restrict__ codes, const uint8_t* __restrict__ sf,
                                     __nv_bfloat16* __restrict__ out, size_t total8, int D, int block_d) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total8; i += (size_t)gridDim.x * blockDim.x) {
    const size_t e0 = i * 8;
    const int d0 = (int)(e0 % D);
    const size_t row = e0 / D;                                   // over (b, h, s_pad): 128-row tiles never straddle a slab
    const int tt = (int)(row & 127);
    const uint32_t e8 = sf[(row >> 7) * 512 + (tt & 31) * 16 + (tt >> 5) * 4 + d0 / block_d];
    const float sc = __uint_as_float(e8 << 23);                  // 2^(e8 - 127)
    const uint2 raw = *reinterpret_cast<const uint2*>(codes + e0);
    const uint8_t* c8 = reinterpret_cast<const uint8_t*>(&raw);
    __align__(16) __nv_bfloat16 o[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = __float2bfloat16_rn(e4m3_to_f32(c8[j]) * sc);
    *reinterpret_cast<uint4*>(out + e0) = *reinterpret_cast<const uint4*>(o);
  }
}

// alpha' (B, NB, H, D) fp32 -> (B, NB, H, D, 16) BF16: the three BF16 pieces h, m, l of each value laid out as
// [h m l h m h 0 0] twice, the B operand rows of the K-extension step of P.V (see attention_fast.cu)
__global__ void alpha_ext_kernel(const float* __restrict__ alpha, __nv_bfloat16* __restrict__ out, size_t total) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    float v = alpha[i];
    const __nv_bfloat16 h = __float2bfloat16_rn(v);
    v -= __bfloat162float(h);
    const __nv_bfloat16 m = __float2bfloat16_rn(v);
    v -= __bfloat162float(m);
    const __nv_bfloat16 l = __float2bfloat16_rn(v);
    const __nv_bfloat16 z = __float2bfloat16_rn(0.f);
    __align__(16) __nv_bfloat16 o[16] = {h, m, l, h, m, h, z, z, h, m, l, h, m, h, z, z};
    uint4* dst = reinterpret_cast<uint4*>(out + i * 16);
    dst[0] = reinterpret_cast<const uint4*>(o)[0];
    dst[1] = reinterpret_cast<const uint4*>(o)[1];
  }
}

static size_t align256(size_t v) { return (v + 255) / 256 * 256; }
// keys per entry of the prepared V-smoothing vector (see alpha_prep_kernel)
static int alpha_granularity(const lbfq_attn_args* a) {
  int g = a->v_smooth_block > 0 ? a->v_smooth_block : 1;
  if (a->v_kind == LBFQ_V_BLOCK && a->v_block > 0) {
    int x = g, y = a->v_block;
    while (y) { const int t = x % y; x = y; y = t; }
    g = x;
  }
  return g;
}
static size_t alpha_ws_bytes(const lbfq_attn_args* a) {
  if (!a->v_alpha) return 0;
  return align256((size_t)a->B * (a->N / alpha_granularity(a)) * a->H * a->D * 4);
}
// mx / dynamic P, or any P with the V-smoothing term, on FP8-block Q/K may take the BF16-P kernel, which wants a BF16
// copy of V^T (and the alpha' pieces) in the workspace
// mxfp8 Q / K go to the TMEM-resident kernel as BF16 operands wherever it serves the rest of the configuration
// (everything fast_variant() asks of a BF16-operand launch, stated on the arguments)
static bool mx_as_bf16(const lbfq_attn_args* a) {
  if (a->qk_kind != LBFQ_QK_MX || a->use_blasst || a->rowmax_counters != nullptr) return false;
  if (lbfq::debug_flags() & LBFQ_FLAG_ATTN_GENERIC) return false;
  if (a->v_kind != LBFQ_V_CHANNEL && a->v_kind != LBFQ_V_MX) return false;
  if (a->qm_corr != nullptr && a->q_smooth_block % 128 != 0) return false;
  if (a->v_alpha != nullptr && !(a->v_smooth_block == 64 || a->v_smooth_block % 128 == 0)) return false;
  if (a->block_n != 32 && a->block_n != 64) return false;
  return a->sm_scale > 0.f && a->qk_block > 0 && a->D % a->qk_block == 0 && a->qk_block % 8 == 0 && a->D / a->qk_block <= 4;
}
static size_t qk_bf16_ws_bytes(const lbfq_attn_args* a) {
  return mx_as_bf16(a) ? align256((size_t)a->B * a->H * a->m_pad * a->D * 2) + align256((size_t)a->B * a->H * a->n_pad * a->D * 2) : 0;
}
static bool may_want_v_bf16(const lbfq_attn_args* a) {
  if (mx_as_bf16(a)) return true;
  if (a->use_blasst && (a->v_alpha || a->qm_corr || !lbfq::attn::fast_blasst_fill(a->fill_kind, a->uta_bins, a->block_n)))
    return false;
  return (a->p_kind != LBFQ_P_ELEMENTWISE || a->v_alpha) && a->v_kind != LBFQ_V_BLOCK && a->qk_kind == LBFQ_QK_FP8_BLOCK;
}
static size_t v_bf16_ws_bytes(const lbfq_attn_args* a) {
  return may_want_v_bf16(a) ? align256((size_t)a->B * a->H * a->D * a->n_pad * 2) : 0;
}
static size_t alpha_ext_ws_bytes(const lbfq_attn_args* a) {
  const bool bf = a->qk_kind == LBFQ_QK_BF16;
  return ((bf || may_want_v_bf16(a)) && a->v_alpha) ? 8 * alpha_ws_bytes(a) : 0;      // 16 BF16 per FP32 value
}

static thread_local int g_last_variant = 0;
extern "C" int lbfq_attention_last_variant(void) { return g_last_variant; }

extern "C" int64_t lbfq_attention_workspace_bytes(const lbfq_attn_args* a) {
  if (!a) return 0;
  return (int64_t)(alpha_ws_bytes(a) + v_bf16_ws_bytes(a) + alpha_ext_ws_bytes(a) + qk_bf16_ws_bytes(a));
}

// BF16 pieces of alpha' into `dst` and the tensor map over them: (16, D, B * NB * H) BF16, one (D x 16) tile per
// (b, smoothing block, h), 32-byte rows, 32B swizzle
static int make_alpha_ext(const lbfq_attn_args* a, const lbfq::attn::Params& p, void* dst, CUtensorMap* ma, cudaStream_t st) {
  using namespace lbfq::attn;
  __nv_bfloat16* ext = reinterpret_cast<__nv_bfloat16*>(dst);
  const size_t total = (size_t)a->B * (a->N / a->v_smooth_block) * a->H * a->D;
  int ge = (int)((total + 255) / 256); if (ge > sm_count() * 16) ge = sm_count() * 16;
  alpha_ext_kernel<<<ge, 256, 0, st>>>(p.v_alpha, ext, total);
  if (int rc = check_launch("alpha_ext")) return rc;
  auto enc = get_encode();
  LBFQ_REQUIRE(enc != nullptr, LBFQ_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
  cuuint64_t dims[3] = {16, (cuuint64_t)a->D, (cuuint64_t)a->B * (a->N / a->v_smooth_block) * a->H};
  cuuint64_t strides[2] = {32, (cuuint64_t)a->D * 32};
  cuuint32_t box[3] = {16, (cuuint32_t)a->D, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = enc(ma, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, ext, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_32B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  LBFQ_REQUIRE(r == CUDA_SUCCESS, LBFQ_ERR_CUDA, "cuTensorMapEncodeTiled (alpha pieces) failed with code %d", (int)r);
  return LBFQ_OK;
}

extern "C" int lbfq_attention_fwd(const lbfq_attn_args* a, void* workspace, void* stream) {
  using namespace lbfq::attn;
  LBFQ_REQUIRE(a != nullptr, LBFQ_ERR_ARG, "null argument block");
  LBFQ_REQUIRE(a->B > 0 && a->H > 0 && a->M > 0 && a->N > 0, LBFQ_ERR_ARG, "empty attention problem");
  LBFQ_REQUIRE(a->D == 64 || a->D == 128, LBFQ_ERR_ARG, "head dim must be 64 or 128; got %d", a->D);
  LBFQ_REQUIRE(a->block_n == 32 || a->block_n == 64, LBFQ_ERR_UNSUPPORTED,
               "block_n=%d: this build has key blocks of 32 or 64", a->block_n);
  LBFQ_REQUIRE(a->block_m > 0, LBFQ_ERR_ARG, "block_m must be positive");
  LBFQ_REQUIRE(a->m_pad >= a->M && a->m_pad % 128 == 0 && a->n_pad >= a->N && a->n_pad % 128 == 0, LBFQ_ERR_ARG,
               "m_pad / n_pad must cover M / N and be multiples of 128");
  LBFQ_REQUIRE(a->q_codes && a->k_codes && a->v_codes && a->out, LBFQ_ERR_ARG, "null operand pointer");
  LBFQ_REQUIRE(a->qk_kind >= LBFQ_QK_FP8_BLOCK && a->qk_kind <= LBFQ_QK_BF16_V_CODES, LBFQ_ERR_ARG,
               "unknown qk_kind %d", a->qk_kind);
  const bool mx = a->qk_kind == LBFQ_QK_MX;
  const bool bfv = a->qk_kind == LBFQ_QK_BF16_V_CODES;        // BF16 Q / K, e4m3 V codes: the general kernel
  const bool bf = a->qk_kind == LBFQ_QK_BF16 || bfv;
  if (bf) {
    // nothing to check: the operands carry their scales already
  } else if (mx) {
    LBFQ_REQUIRE(a->q_scale_e8 && a->k_scale_e8, LBFQ_ERR_ARG, "mxfp8 Q/K needs the UE8M0 scale tiles");
    LBFQ_REQUIRE(a->qk_block > 0 && a->D % a->qk_block == 0 && a->D / a->qk_block <= 4, LBFQ_ERR_ARG,
                 "mxfp8_block_size=%d must divide D into at most 4 groups", a->qk_block);
  } else {
    LBFQ_REQUIRE(a->q_scale && a->k_scale && a->qk_block > 0, LBFQ_ERR_ARG, "fp8_block Q/K needs scales and a block size");
    LBFQ_REQUIRE(a->M % a->qk_block == 0 && a->N % a->qk_block == 0, LBFQ_ERR_ARG,
                 "S must be divisible by fp8_block_size=%d", a->qk_block);
    LBFQ_REQUIRE(a->qk_block % a->block_n == 0, LBFQ_ERR_UNSUPPORTED,
                 "fp8_block_size (%d) must be a multiple of block_n (%d)", a->qk_block, a->block_n);
  }
  LBFQ_REQUIRE(a->p_kind >= 0 && a->p_kind <= 2, LBFQ_ERR_ARG, "unknown p_quant_mode");
  LBFQ_REQUIRE(a->v_kind >= 0 && a->v_kind <= 2 && a->v_scale, LBFQ_ERR_ARG, "bad V quant kind / scale");
  if (a->v_kind != LBFQ_V_CHANNEL) {
    LBFQ_REQUIRE(a->v_block > 0 && a->N % a->v_block == 0, LBFQ_ERR_ARG, "S (%d) must be divisible by v_block_size (%d)", a->N, a->v_block);
    LBFQ_REQUIRE(a->v_block >= a->block_n && a->v_block % a->block_n == 0, LBFQ_ERR_ARG,
                 "v_block_size (%d) must be >= block_n (%d) and an integer multiple of block_n", a->v_block, a->block_n);
  }
  if (a->v_alpha) {
    LBFQ_REQUIRE(a->v_smooth_block > 0, LBFQ_ERR_ARG, "v_smooth_block must be > 0 when v_alpha is given");
    LBFQ_REQUIRE(a->v_smooth_block >= a->block_n && a->v_smooth_block % a->block_n == 0, LBFQ_ERR_ARG,
                 "v_smooth_block (%d) must be >= block_n (%d) and an integer multiple of block_n", a->v_smooth_block, a->block_n);
    LBFQ_REQUIRE(a->N % a->v_smooth_block == 0, LBFQ_ERR_ARG, "S (%d) must be divisible by v_smooth_block (%d)", a->N, a->v_smooth_block);
    LBFQ_REQUIRE(workspace != nullptr, LBFQ_ERR_ARG, "v_alpha needs the workspace of lbfq_attention_workspace_bytes");
  }
  if (a->qm_corr) {
    LBFQ_REQUIRE(a->q_smooth_block > 0, LBFQ_ERR_ARG, "q_smooth_block must be > 0 with qm_bhgd");
    LBFQ_REQUIRE(a->q_smooth_block >= a->block_m && a->q_smooth_block % a->block_m == 0, LBFQ_ERR_ARG,
                 "q_smooth_block (%d) must be >= block_m (%d) and an integer multiple of block_m", a->q_smooth_block, a->block_m);
    LBFQ_REQUIRE(a->M % a->q_smooth_block == 0, LBFQ_ERR_ARG, "S (%d) must be divisible by q_smooth_block (%d)", a->M, a->q_smooth_block);
    LBFQ_REQUIRE(a->corr_stride >= a->n_pad && a->corr_stride % 4 == 0, LBFQ_ERR_ARG, "corr_stride must cover n_pad");
  }
  LBFQ_REQUIRE(!(a->rowmax_est && a->rowmax_init), LBFQ_ERR_ARG, "rowmax_init_bhs and rowmax_est_bhs are mutually exclusive");
  if (a->use_blasst) {
    LBFQ_REQUIRE(a->blasst_lambda > 0.f && a->blasst_lambda < 1.f, LBFQ_ERR_ARG, "blasst_lambda must be in (0, 1); got %g", (double)a->blasst_lambda);
    LBFQ_REQUIRE(a->fill_kind >= 0 && a->fill_kind <= 6, LBFQ_ERR_ARG, "unknown blasst fill kind %d", a->fill_kind);
    if (a->fill_kind == LBFQ_FILL_UTA) {
      LBFQ_REQUIRE(a->uta_bins > 0 && a->block_n % a->uta_bins == 0, LBFQ_ERR_ARG,
                   "blasst UTA bins (%d) must divide block_n (%d)", a->uta_bins, a->block_n);
      LBFQ_REQUIRE(a->uta_bins <= 16, LBFQ_ERR_UNSUPPORTED, "at most 16 UTA bins are supported; got %d", a->uta_bins);
    }
  }
  if (a->blasst_tile_predicate) {
    LBFQ_REQUIRE(a->use_blasst, LBFQ_ERR_ARG, "blasst_tile_predicate requires use_blasst");
    LBFQ_REQUIRE(a->fill_kind == LBFQ_FILL_ZERO, LBFQ_ERR_ARG, "blasst_tile_predicate drops whole tiles: zero fill only");
    LBFQ_REQUIRE(a->rowmax_init == nullptr, LBFQ_ERR_UNSUPPORTED, "blasst_tile_predicate is built for the online row max without rowmax_init");
    LBFQ_REQUIRE(a->qk_kind == LBFQ_QK_FP8_BLOCK, LBFQ_ERR_UNSUPPORTED, "blasst_tile_predicate is served on FP8-block Q / K codes");
  }
  cudaStream_t st = (cudaStream_t)stream;

  Params p{};
  p.B = a->B; p.H = a->H; p.M = a->M; p.N = a->N; p.D = a->D;
  p.qk_block = mx ? 1 : (bf ? a->block_n : a->qk_block);
  p.q_scale = (mx || bf) ? nullptr : a->q_scale; p.k_scale = (mx || bf) ? nullptr : a->k_scale;
  p.qk_bf16 = bf ? 1 : 0;
  p.q_sf = a->q_scale_e8; p.k_sf = a->k_scale_e8; p.m_pad = a->m_pad; p.n_pad = a->n_pad;
  p.v_kind = a->v_kind; p.v_scale = a->v_scale; p.v_block = a->v_block > 0 ? a->v_block : a->block_n;
  p.sm_scale = a->sm_scale; p.p_off = a->p_max_offset; p.p_kind = a->p_kind; p.block_m = a->block_m;
  p.v_alpha = nullptr; p.v_smooth_block = a->v_smooth_block > 0 ? a->v_smooth_block : a->block_n;
  p.corr = a->qm_corr; p.q_smooth_block = a->q_smooth_block > 0 ? a->q_smooth_block : a->block_m;
  p.corr_stride = a->corr_stride; p.n_groups = a->qm_corr ? a->M / a->q_smooth_block : 0;
  p.corr_staged = (a->qm_corr && a->q_smooth_block % 128 == 0) ? 1 : 0;
  p.side_bytes = (p.corr_staged ? 2 * kChunk * 4 : 0) +
                 ((a->v_alpha ? 1 : 0) + (a->v_kind == LBFQ_V_MX ? 1 : 0)) * (kChunk / a->block_n) * a->D * 4;
  p.rowmax_est = a->rowmax_est; p.rowmax_init = a->rowmax_init;
  p.rm_mode = (a->rowmax_est && !a->use_blasst) ? (a->p_kind == LBFQ_P_DYNAMIC ? 2 : 1) : 0;
  p.blasst = a->use_blasst ? 1 : 0; p.block_n = a->block_n;
  p.log_lambda = a->use_blasst ? logf(a->blasst_lambda) : 0.f;
  p.lambda = a->use_blasst ? a->blasst_lambda : 0.f;
  p.fill_kind = a->use_blasst ? a->fill_kind : 0; p.fill_alpha = a->fill_alpha; p.uta_bins = a->uta_bins > 0 ? a->uta_bins : 1;
  p.stats = a->use_blasst ? a->blasst_stats : nullptr;
  // zero fill, on request (the tile predicate, or the counter of elided pairs): the rows of a tile vote on every key
  // block, and a block they all skip is not computed at all. Not the default: the vote costs more than the elided
  // work returns unless a large share of the (tile, block) pairs is elided.
  // (with rowmax_init a tile could skip its first block, whose P.V initialises the accumulator: no vote then)
  p.tile_vote = (a->use_blasst && a->fill_kind == LBFQ_FILL_ZERO && a->rowmax_init == nullptr &&
                 (a->blasst_tile_predicate || a->blasst_elided != nullptr)) ? 1 : 0;
  p.tile_pred = (a->use_blasst && a->blasst_tile_predicate) ? 1 : 0;
  p.elided = a->use_blasst ? a->blasst_elided : nullptr;
  p.counters = reinterpret_cast<unsigned long long*>(a->rowmax_counters);
  p.out = a->out; p.out_dtype = a->out_dtype; p.out_layout = a->out_layout; p.out_exact = a->out_fp32_exact;
  p.out_row_index = a->out_row_index; p.status = a->status;
  p.n_v_scale = a->v_kind == LBFQ_V_CHANNEL ? (long long)a->B * a->H * a->D
                : a->v_kind == LBFQ_V_BLOCK ? (long long)a->B * (a->N / p.v_block) * a->H
                                            : (long long)a->B * (a->N / p.v_block) * a->H * a->D;
  p.n_v_alpha = a->v_alpha ? (long long)a->B * (a->N / a->v_smooth_block) * a->H * a->D : 0;
  p.n_corr = a->qm_corr ? (long long)a->B * a->H * p.n_groups * a->corr_stride : 0;
  p.n_out = (long long)a->B * a->H * a->M * a->D;
  LBFQ_REQUIRE(p.out_dtype >= 0 && p.out_dtype <= 2, LBFQ_ERR_DTYPE, "unsupported dtype code %d", p.out_dtype);

  if (a->v_alpha) {
    const int gran = alpha_granularity(a);
    const size_t total = (size_t)a->B * (a->N / gran) * a->H * a->D;
    int g = (int)((total + 255) / 256); if (g > sm_count() * 8) g = sm_count() * 8;
    alpha_prep_kernel<<<g, 256, 0, st>>>(a->v_alpha, (float*)workspace, a->v_scale, a->v_kind, a->B, a->N, a->H, a->D,
                                        gran, a->v_smooth_block, a->v_kind == LBFQ_V_BLOCK ? a->v_block : 1);
    if (int rc = check_launch("alpha_prep")) return rc;
    p.v_alpha = (const float*)workspace;
    p.v_smooth_block = gran;                      // the kernels index the prepared vector, not the caller's
    p.n_v_alpha = (long long)total;
  }

  CUtensorMap mq, mk, mv;
  const uint64_t BH = (uint64_t)a->B * a->H;
  if (bfv) {
    // BF16 Q / K with V as e4m3 codes: the general kernel (every V kind, every BLASST fill, the stats tensor)
    LBFQ_REQUIRE(a->rowmax_counters == nullptr, LBFQ_ERR_UNSUPPORTED, "rowmax_counters are served on FP8-code operands only");
    if (int rc = make_map_bf16(&mq, a->q_codes, a->D, a->m_pad, BH, 64, kTileM)) return rc;
    if (int rc = make_map_bf16(&mk, a->k_codes, a->D, a->n_pad, BH, 64, kChunk)) return rc;
    if (int rc = make_map(&mv, a->v_codes, a->n_pad, a->D, BH, kChunk, a->D)) return rc;
    g_last_variant = 0;
    const bool blq = a->use_blasst != 0;
#define LBFQ_LAUNCH_BF(DD, NN)                                                                      \
  return blq ? launch<DD, NN, true, false, true>(mq, mk, mv, p, st) : launch<DD, NN, false, false, true>(mq, mk, mv, p, st)
    if (a->D == 128 && a->block_n == 64) { LBFQ_LAUNCH_BF(128, 64); }
    if (a->D == 128 && a->block_n == 32) { LBFQ_LAUNCH_BF(128, 32); }
    if (a->D == 64 && a->block_n == 64) { LBFQ_LAUNCH_BF(64, 64); }
    LBFQ_LAUNCH_BF(64, 32);
#undef LBFQ_LAUNCH_BF
  }
  if (bf) {
    // BF16 operands: only the TMEM-resident kernel multiplies them
    LBFQ_REQUIRE(a->rowmax_counters == nullptr, LBFQ_ERR_UNSUPPORTED, "rowmax_counters are served on FP8-code operands only");
    const int fvb = fast_variant(p, a->use_blasst != 0, false);
    LBFQ_REQUIRE(fvb == 2, LBFQ_ERR_UNSUPPORTED,
                 "BF16 operands are served for V per channel / pre-dequantised, without BLASST, with q_smooth_block a "
                 "multiple of 128 and v_smooth_block 64 or a multiple of 128; the FP8-code entry covers the rest");
    if (int rc = make_map_bf16(&mq, a->q_codes, a->D, a->m_pad, BH, 64, kTileM)) return rc;
    if (int rc = make_map_bf16(&mk, a->k_codes, a->D, a->n_pad, BH, 64, kChunk)) return rc;
    if (int rc = make_map_bf16(&mv, a->v_codes, a->n_pad, a->D, BH, 64, a->D)) return rc;
    CUtensorMap ma = mv;
    if (a->v_alpha)
      if (int rc = make_alpha_ext(a, p, (uint8_t*)workspace + alpha_ws_bytes(a), &ma, st)) return rc;
    g_last_variant = 1;
    return launch_fast(mq, mk, mv, ma, p, a->block_n, 2, st);
  }
  if (mx && mx_as_bf16(a)) {
    // mxfp8 Q / K as exact BF16 operands on the TMEM-resident kernel (see qk_mx_to_bf16_kernel)
    Params pb = p;
    pb.qk_bf16 = 1; pb.qk_block = a->block_n; pb.q_scale = nullptr; pb.k_scale = nullptr;
    if (fast_variant(pb, false, false) == 2) {
      LBFQ_REQUIRE(workspace != nullptr, LBFQ_ERR_ARG, "this configuration needs the workspace of lbfq_attention_workspace_bytes");
      LBFQ_REQUIRE(a->q_scale_e8 != nullptr && a->k_scale_e8 != nullptr, LBFQ_ERR_ARG, "mxfp8 Q / K need their scale tiles");
      uint8_t* ws = (uint8_t*)workspace;
      __nv_bfloat16* vb = reinterpret_cast<__nv_bfloat16*>(ws + alpha_ws_bytes(a));
      uint8_t* ext = ws + alpha_ws_bytes(a) + v_bf16_ws_bytes(a);
      __nv_bfloat16* qb = reinterpret_cast<__nv_bfloat16*>(ext + alpha_ext_ws_bytes(a));
      __nv_bfloat16* kb = reinterpret_cast<__nv_bfloat16*>((uint8_t*)qb + align256((size_t)a->B * a->H * a->m_pad * a->D * 2));
      const int cap = sm_count() * 16;
      auto blocks = [&](size_t n8) { const size_t g = (n8 + 255) / 256; return (int)(g > (size_t)cap ? cap : g); };
      const size_t q8 = (size_t)a->B * a->H * a->m_pad * a->D / 8, k8 = (size_t)a->B * a->H * a->n_pad * a->D / 8;
      qk_mx_to_bf16_kernel<<<blocks(q8), 256, 0, st>>>((const uint8_t*)a->q_codes, a->q_scale_e8, qb, q8, a->D, a->qk_block);
      if (int rc = check_launch("qk_mx_to_bf16")) return rc;
      qk_mx_to_bf16_kernel<<<blocks(k8), 256, 0, st>>>((const uint8_t*)a->k_codes, a->k_scale_e8, kb, k8, a->D, a->qk_block);
      if (int rc = check_launch("qk_mx_to_bf16")) return rc;
      const size_t v8 = (size_t)a->B * a->H * a->D * a->n_pad / 8;
      v_codes_to_bf16_kernel<<<blocks(v8), 256, 0, st>>>((const uint8_t*)a->v_codes, vb, a->v_kind, a->v_scale, a->B, a->H, a->D, a->N,
                                                         a->n_pad, p.v_block);
      if (int rc = check_launch("v_codes_to_bf16")) return rc;
      CUtensorMap mvb, ma;
      if (int rc = make_map_bf16(&mq, qb, a->D, a->m_pad, BH, 64, kTileM)) return rc;
      if (int rc = make_map_bf16(&mk, kb, a->D, a->n_pad, BH, 64, kChunk)) return rc;
      if (int rc = make_map_bf16(&mvb, vb, a->n_pad, a->D, BH, 64, a->D)) return rc;
      ma = mvb;
      if (a->v_alpha)
        if (int rc = make_alpha_ext(a, pb, ext, &ma, st)) return rc;
      g_last_variant = 1;
      return launch_fast(mq, mk, mvb, ma, pb, a->block_n, 2, st);
    }
  }
  if (int rc = make_map(&mq, a->q_codes, a->D, a->m_pad, BH, a->D, kTileM)) return rc;
  if (int rc = make_map(&mk, a->k_codes, a->D, a->n_pad, BH, a->D, kChunk)) return rc;
  if (int rc = make_map(&mv, a->v_codes, a->n_pad, a->D, BH, kChunk, a->D)) return rc;

  const bool bl = a->use_blasst != 0;
  // LBFQ_FLAG_ATTN_GENERIC keeps every configuration on the general kernel (used to cross-check the two)
  g_last_variant = 0;
  const int fv = ((debug_flags() & LBFQ_FLAG_ATTN_GENERIC) || p.counters != nullptr) ? 0 : fast_variant(p, bl, mx);
  if (fv == 1) {
    g_last_variant = 1;
    return launch_fast(mq, mk, mv, mv, p, a->block_n, 1, st);
  }
  if (fv == 2 && may_want_v_bf16(a)) {
    LBFQ_REQUIRE(workspace != nullptr, LBFQ_ERR_ARG, "this configuration needs the workspace of lbfq_attention_workspace_bytes");
    __nv_bfloat16* vb = reinterpret_cast<__nv_bfloat16*>((uint8_t*)workspace + alpha_ws_bytes(a));
    const size_t total8 = (size_t)a->B * a->H * a->D * a->n_pad / 8;
    int g = (int)((total8 + 255) / 256); if (g > sm_count() * 16) g = sm_count() * 16;
    v_codes_to_bf16_kernel<<<g, 256, 0, st>>>((const uint8_t*)a->v_codes, vb, a->v_kind, a->v_scale, a->B, a->H, a->D, a->N,
                                              a->n_pad, p.v_block);
    if (int rc = check_launch("v_codes_to_bf16")) return rc;
    CUtensorMap mvb, ma;
    if (int rc = make_map_bf16(&mvb, vb, a->n_pad, a->D, BH, 64, a->D)) return rc;
    ma = mvb;
    if (a->v_alpha)
      if (int rc = make_alpha_ext(a, p, (uint8_t*)workspace + alpha_ws_bytes(a) + v_bf16_ws_bytes(a), &ma, st)) return rc;
    g_last_variant = 1;
    return launch_fast(mq, mk, mvb, ma, p, a->block_n, 2, st);
  }
  LBFQ_REQUIRE(!p.tile_pred, LBFQ_ERR_UNSUPPORTED,
               "blasst_tile_predicate is served by the kernel with the accumulator in tensor memory only (per-channel or "
               "mxfp8 V, no score bias, no V-smoothing term)");
#define LBFQ_LAUNCH(DD, NN, MX)                                                                    \
  return bl ? launch<DD, NN, true, MX>(mq, mk, mv, p, st) : launch<DD, NN, false, MX>(mq, mk, mv, p, st)
  if (mx) {
    LBFQ_REQUIRE(a->qk_block == 32, LBFQ_ERR_UNSUPPORTED,
                 "mxfp8_block_size=%d: the block-scaled MMA of the general kernel scales 32 elements of D at a time", a->qk_block);
    // scale-factor columns of a 32-key block would start at odd TMEM columns, which the MMA rejects
    LBFQ_REQUIRE(a->block_n == 64, LBFQ_ERR_UNSUPPORTED, "mxfp8 Q/K on the general kernel needs block_n = 64; got %d", a->block_n);
    if (a->D == 128) { LBFQ_LAUNCH(128, 64, true); }
    LBFQ_LAUNCH(64, 64, true);
  }
  if (a->D == 128 && a->block_n == 64) { LBFQ_LAUNCH(128, 64, false); }
  if (a->D == 128 && a->block_n == 32) { LBFQ_LAUNCH(128, 32, false); }
  if (a->D == 64 && a->block_n == 64) { LBFQ_LAUNCH(64, 64, false); }
  LBFQ_LAUNCH(64, 32, false);
#undef LBFQ_LAUNCH
}
