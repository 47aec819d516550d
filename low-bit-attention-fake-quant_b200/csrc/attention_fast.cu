// Streaming fake-quant attention for sm_100a, output accumulator resident in tensor memory.
//
// Same operator as attention.cu (`_fake_quant_attn_fwd_kernel`, src/low_bit_fake_quant/attention_triton.py:48-671),
// specialised for the configurations in which every key block's P.V enters the output with weight one:
// element-wise (static offset) P quantisation, V quantised per channel, no V-smoothing term, no score bias,
// FP8 block scales on Q / K, row max tracked online or frozen to an estimate (template flags add the BF16-P
// modes, the score bias, the V-smoothing term and BLASST row skipping with its constant and per-bin fills). There
//
//   O <- O * alpha + Pc . Vc                                      (attention_triton.py:362-385)
//
// and alpha = exp2(m_old - m_new) is exactly 1 for every row whose running max did not move, so the tensor
// core accumulates P.V straight into one TMEM accumulator and the softmax threads touch O only in the blocks
// where some row of their warp raised its max (TMEM -> registers -> * alpha -> TMEM), plus once at the end.
//
// Per 128-row tile the tensor memory holds two S buffers (64 columns each) and O (D columns). P of block j is
// written over the first columns of S buffer j & 1 once S has been copied to registers, and Q.K^T of block
// j + 2 is issued behind P.V of block j by the same thread: tcgen05 operations of one thread execute in
// order, so neither the S buffer nor P needs a "free" barrier. Per key block a softmax thread waits on one
// barrier (S ready) and arrives on one (P ready).
//
// The score arithmetic is contracted the way a compiler contracts the reference's expression
// exp2((dot * f - m) * log2e + off) with f = (sq * sk) * sm_scale: the block max is taken over the raw dot
// products (f > 0), the running max is kept in the log2 domain, and every element costs one FFMA, one exp2,
// one add (row sum) and half a conversion.
//
// CTA = 256 query rows of one (b, h): 16 softmax warps (two threads per row, TMEM lane == row), one TMA
// producer warp, one MMA-issuing warp per tile. Every mbarrier wait is bounded; on expiry the kernel raises `*status`, all
// roles leave their loops, TMEM is released and the launch returns.

#include <type_traits>

#include "attn_prims.cuh"

namespace lbfq {
namespace attn {

namespace {

// Two threads per query row: each reads one half of the S block's columns, takes their maximum, and the two halves'
// maxima meet through shared memory and a 64-thread named barrier; each thread then computes the exponentials,
// the P codes and the accumulator rescale of its half. 16 softmax warps give every scheduler four of them to hide
// each other's waits.
constexpr int kFastSoftmaxWarps = 16;
constexpr int kFastThreads = (kFastSoftmaxWarps + 4) * 32;
constexpr int kFastRegsLaunch = (65536 / kFastThreads) / 8 * 8;   // what __launch_bounds__(kFastThreads, 1) yields
// Registers per thread after the roles split (setmaxnreg): the softmax warps take what the service warps give up.
// The BLASST instantiations carry more live state per block (fills, votes) and spill at 104, so they take 112 / 32;
// the plain ones are faster at 104 / 40 (measured on the benchmark stacks).
template <bool BL>
struct FastRegs {
  static constexpr int kSoftmax = BL ? 112 : 104;
  static constexpr int kService = BL ? 32 : 40;
  // `setmaxnreg.inc` blocks until the CTA's register pool can satisfy it: the requests must fit in the pool
  static_assert(kFastSoftmaxWarps * 32 * kSoftmax + 4 * 32 * kService <= kFastThreads * kFastRegsLaunch,
                "setmaxnreg requests exceed the CTA's register pool");
  static_assert(kSoftmax % 8 == 0 && kService % 8 == 0, "setmaxnreg granularity");
};

// PK = 0: P as e4m3 codes, P.V an FP8 MMA over the V^T codes (4 key stages).
// PK = 1: P re-scaled and rounded to BF16 as the reference does for its mx / dynamic P modes, P.V a BF16 MMA
//         over a BF16 copy of V^T (3 key stages: a V stage is twice as large).
// QB = 1: Q and K are BF16 tensors (the reference's de-quantised operands) and Q.K^T a BF16 MMA; two key stages.
// BL = 1: BLASST; the row-pair exchange carries three values per block (maximum, sum of scores, largest fill).
// TV = 1: BLASST with zero fill where the 256 threads of a 128-row tile vote on every key block: a block that all
//         rows skip costs no exponentials, no P and no P.V. With `tile_pred` the vote is also the only way to skip
//         (the tile-level predicate of the reference's simulator, blasst_skip.py:573-585).
// Key stages of the BF16-P instantiations. A build with fewer stages (-DLBFQ_FAST_PK_STAGES=2) leaves the shared
// memory that instruction-level profiling needs; it is not a shipped configuration.
#ifndef LBFQ_FAST_PK_STAGES
#define LBFQ_FAST_PK_STAGES 3
#endif
template <int D, int PK, int QB, int BL = 0>
struct FastSmem {
  static constexpr int kStages = QB ? 2 : (PK ? LBFQ_FAST_PK_STAGES : 4);
  static constexpr int kQ = kTileM * D * (QB ? 2 : 1);         // bytes per Q tile
  static constexpr int kK = kChunk * D * (QB ? 2 : 1);         // bytes per K stage
  static constexpr int kV = D * kChunk * (PK ? 2 : 1);        // bytes per V^T stage
  static constexpr int offQ = 0;
  static constexpr int offK = offQ + 2 * kQ;
  static constexpr int offV = offK + kStages * kK;
  static constexpr int offBar = offV + kStages * kV;
  static constexpr int kNumBar = 2 + 4 * kStages + 4 + 4 + 2 + 2 + 2 * kStages + 4;
  static constexpr int offMisc = offBar + kNumBar * 8;
  static constexpr int offL = offMisc + 64;                    // row sums of the two column halves [tile][half][row]
  // score-bias rows (`corr`) of each tile's Q group, staged per 128-key stage by the producer
  // block maxima exchanged between the two threads of a row: [block parity][tile][half][row]
  static constexpr int offX = offL + 2 * 2 * kTileM * 4;
  static constexpr int kXch = 2 * 2 * 2 * kTileM;             // floats per exchanged quantity
  static constexpr int offCorr = offX + (BL ? 3 : 1) * kXch * 4;
  // V-smoothing tiles for the K-extension of P.V: per stage up to two (D x 16) BF16 tiles (32-byte rows)
  static constexpr int kAext = D * 32;
  static constexpr int offAext = (offCorr + kStages * 2 * kChunk * 4 + 1023) / 1024 * 1024;   // TMA destination, swizzled
  static constexpr int total = offAext + (PK ? kStages * 2 * kAext : 0);
};

template <int D, int BN, bool CORR, int PK, bool VALPHA, int QB, bool BL = false, bool TV = false>
__global__ void __launch_bounds__(kFastThreads, 1)
attn_fast_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                 const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_a, const Params p) {
  static_assert(!VALPHA || PK == 1, "the V-smoothing term rides on the BF16 P.V");
  static_assert(!QB || PK == 1, "BF16 Q / K come with the BF16 P.V");
  static_assert(!BL || (!CORR && !VALPHA && QB == 0), "BLASST is built without score bias, V-smoothing term, BF16 Q / K");
  static_assert(!TV || BL, "the tile vote belongs to BLASST");
  // scores kept in the reference's own units (natural-log domain) instead of the log2 domain
  constexpr bool NAT = CORR || BL;
  using SM = FastSmem<D, PK, QB, BL ? 1 : 0>;
  constexpr int kFastStages = SM::kStages;
  constexpr int NSUB = kChunk / BN;                // key blocks per stage
  constexpr int TCOLS = 256;                       // TMEM columns per tile
  constexpr int COL_S = 0, S_STRIDE = 64, COL_O = 128;
  static_assert(BN == 32 || BN == 64, "block_n of 32 or 64");
  static_assert(COL_O + D <= TCOLS, "TMEM budget");

  extern __shared__ __align__(1024) uint8_t smem_raw[];
  // rounded up to 1 KB by pointer arithmetic, so that the compiler still knows it points into shared memory
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  const uint32_t sbase = smem_u32(smem);
  const uint32_t bar0 = sbase + SM::offBar;
  auto BAR_QFULL = [&](int t) { return bar0 + 8u * t; };
  auto BAR_KFULL = [&](int s) { return bar0 + 8u * (2 + s); };
  auto BAR_VFULL = [&](int s) { return bar0 + 8u * (2 + kFastStages + s); };
  auto BAR_KFREE = [&](int s) { return bar0 + 8u * (2 + 2 * kFastStages + s); };
  auto BAR_VFREE = [&](int s) { return bar0 + 8u * (2 + 3 * kFastStages + s); };
  auto BAR_SFULL = [&](int t, int buf) { return bar0 + 8u * (2 + 4 * kFastStages + 2 * t + buf); };
  // P ready, one barrier per S buffer: a warp may finish block j + 1 (its S is ready early) before a slower warp has
  // finished block j, and with a single barrier its second arrival would be counted into block j's phase. It cannot
  // be two blocks ahead: S of block j + 2 is issued behind P.V of block j, which waits for every arrival of block j.
  auto BAR_PRDY = [&](int t, int buf) { return bar0 + 8u * (2 + 4 * kFastStages + 4 + 2 * t + buf); };
  auto BAR_PENULT = [&](int t) { return bar0 + 8u * (2 + 4 * kFastStages + 8 + t); };   // P.V of block nblk - 2 done
  auto BAR_ODONE = [&](int t) { return bar0 + 8u * (2 + 4 * kFastStages + 10 + t); };   // P.V of the last block done
  auto BAR_SIDEFULL = [&](int s) { return bar0 + 8u * (2 + 4 * kFastStages + 12 + s); };
  auto BAR_SIDEFREE = [&](int s) { return bar0 + 8u * (2 + 4 * kFastStages + 12 + kFastStages + s); };
  // TV: the eight softmax warps of a tile have published their votes on a key block (one barrier per S buffer)
  auto BAR_VOTE = [&](int t, int buf) { return bar0 + 8u * (2 + 4 * kFastStages + 12 + 2 * kFastStages + 2 * t + buf); };
  volatile int* misc = (volatile int*)(smem + SM::offMisc);   // [0] tmem base, [1] abort, [6] early exit
  // TV: one byte per softmax warp, [block parity][tile][warp of the tile], 1 = every row of the warp skips the block
  uint8_t* const votes = smem + SM::offMisc + 32;
  constexpr unsigned long long kAllVotes = 0x0101010101010101ull;
  volatile int* abort_flag = misc + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int bh = blockIdx.y;
  const int b = bh / p.H, h = bh % p.H;
  const int m0 = blockIdx.x * kCtaM;
  const int nblk = (p.N + BN - 1) / BN;
  const int nchunk = (p.N + kChunk - 1) / kChunk;
  constexpr int kTmaWarp = kFastSoftmaxWarps, kMmaWarp0 = kFastSoftmaxWarps + 1;
  constexpr int HB = BN / 2;                       // S columns whose P one thread produces
  constexpr int HD = D / 2;                        // accumulator columns one thread rescales and stores

  // ---- setup ----------------------------------------------------------------
  // A CTA scheduled after some other CTA has given up a wait retires at once.
  if (threadIdx.x == 0) misc[6] = (p.status != nullptr && *reinterpret_cast<volatile int32_t*>(p.status) != 0) ? 1 : 0;
  __syncthreads();
  if (misc[6]) return;
  if (threadIdx.x == 0) {
    for (int t = 0; t < 2; ++t) {
      mbar_init(BAR_QFULL(t), 1);
      mbar_init(BAR_SFULL(t, 0), 1);
      mbar_init(BAR_SFULL(t, 1), 1);
      // arrivals per block: every thread of the tile (e4m3 P) or one per softmax warp of the tile (BF16 P), see below
      mbar_init(BAR_PRDY(t, 0), PK == 0 ? 2 * kTileM : kFastSoftmaxWarps / 2);
      mbar_init(BAR_PRDY(t, 1), PK == 0 ? 2 * kTileM : kFastSoftmaxWarps / 2);
      mbar_init(BAR_PENULT(t), 1);
      mbar_init(BAR_ODONE(t), 1);
      mbar_init(BAR_VOTE(t, 0), kFastSoftmaxWarps / 2);
      mbar_init(BAR_VOTE(t, 1), kFastSoftmaxWarps / 2);
    }
    for (int s = 0; s < kFastStages; ++s) {
      mbar_init(BAR_KFULL(s), 1);
      mbar_init(BAR_VFULL(s), 1);
      mbar_init(BAR_KFREE(s), 2);
      mbar_init(BAR_VFREE(s), 2);
      mbar_init(BAR_SIDEFULL(s), 1);
      mbar_init(BAR_SIDEFREE(s), CORR ? kFastSoftmaxWarps : 1);      // the bias rows' readers; the alpha' tiles go with V
    }
    misc[1] = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == kTmaWarp) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 512;" ::"r"(sbase + SM::offMisc) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = (uint32_t)misc[0];

  if (warp < kFastSoftmaxWarps) {
    // =========================== softmax warps ===========================
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(FastRegs<BL>::kSoftmax));
    const int t = warp >> 3;                                   // tile
    const int half = (warp >> 2) & 1;                          // which half of the columns this thread produces
    const int row_in_tile = (warp & 3) * 32 + lane;            // a warp reaches the TMEM lanes of its id mod 4
    const int row = m0 + t * kTileM + row_in_tile;             // query row within (b, h)
    const bool row_ok = row < p.M;
    const int rowc = row_ok ? row : (p.M - 1);
    const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
    const uint32_t tS = tmem_base + lane_base + t * TCOLS + COL_S;
    const uint32_t tO = tmem_base + lane_base + t * TCOLS + COL_O + half * HD;

    // BF16 operands are already de-quantised: no Q / K scales
    const float sq = QB ? 1.0f : p.q_scale[((size_t)b * (p.M / p.qk_block) + rowc / p.qk_block) * p.H + h];
    const float* ksc = QB ? nullptr : p.k_scale + (size_t)b * (p.N / p.qk_block) * p.H + h;
    const bool frozen = p.rm_mode == 1;
    const bool thresholds = PK != 0 && p.rm_mode == 2;   // estimated row max corrected by the up-16 / down-32 rule (dynamic P only)
    float max_seen = -INFINITY;
    bool l_pos = false;                          // the row sum is positive (kept as a flag: each thread holds half of it)
    // running max: in the log2 domain (the reference's m_i times log2e) without a score bias; with one the
    // scores are formed as the reference forms them, dot * f + corr, and the max stays in their own units
    constexpr float kDom = NAT ? 1.0f : kLog2e;
    float m2 = -INFINITY;
    if (p.rowmax_est) m2 = p.rowmax_est[(size_t)bh * p.M + rowc] * kDom;
    else if (p.rowmax_init) m2 = p.rowmax_init[(size_t)bh * p.M + rowc] * kDom;
    const float* corr_sm = reinterpret_cast<const float*>(smem + SM::offCorr) + t * kChunk;
    int side_sub = 0, side_stage = 0;
    uint32_t side_par = 0;
    float l_i = 0.f;                                           // row sum over this thread's columns
    float sk = QB ? 1.0f : ksc[0];
    const int blocks_per_scale = p.qk_block / BN;               // fp8_block_size is a multiple of block_n
    int scale_sub = 0;
    const uint32_t bar_sfull = BAR_SFULL(t, 0), bar_prdy = BAR_PRDY(t, 0);
    const bool p_el = p.p_kind == LBFQ_P_ELEMENTWISE, p_mx = p.p_kind == LBFQ_P_MX;
    const float p_off = p_el ? p.p_off : 0.f, sm_scale = p.sm_scale;  // the offset belongs to element-wise P only
    const int n_keys = p.N, k_stride = p.H;

    // Waits here never bail out (mbar_wait_cont): the warp stays convergent around the collective TMEM
    // accesses whatever happens, and a launch whose wait expired ends with `*status` raised.
    // Key blocks alternate between the two S buffers; the loop body is instantiated once per buffer so that
    // every TMEM and barrier address in it is a loop-invariant register.
    const uint32_t tS_mine[2] = {tS + half * HB, tS + S_STRIDE + half * HB};
    // each thread takes the maximum of its own half of a block's columns; the halves meet through shared memory
    // and a 64-thread named barrier per (tile, lane quarter) pair of warps (ids 2..9)
    float* xch = reinterpret_cast<float*>(smem + SM::offX);
    float* const x_mine[2] = {xch + ((0 * 2 + t) * 2 + half) * kTileM + row_in_tile, xch + ((1 * 2 + t) * 2 + half) * kTileM + row_in_tile};
    const float* const x_oth[2] = {xch + ((0 * 2 + t) * 2 + (1 - half)) * kTileM + row_in_tile,
                                   xch + ((1 * 2 + t) * 2 + (1 - half)) * kTileM + row_in_tile};
    const uint32_t pair_bar = 2u + (uint32_t)(t * 4 + (warp & 3));
    constexpr int PW = PK ? HB / 2 : HB / 4;         // 32-bit words of P per thread: two BF16 or four e4m3 per word
    const uint32_t tP[2] = {tS + half * PW, tS + S_STRIDE + half * PW};
    // K-extension columns of P (V-smoothing term): 16 BF16 = 8 columns behind the 32 columns of P, 4 per thread
    const uint32_t tA[2] = {tS + 32 + half * 4, tS + S_STRIDE + 32 + half * 4};
    const uint32_t bar_s[2] = {bar_sfull, bar_sfull + 8u};
    const uint32_t bar_penult = BAR_PENULT(t);
    const int last = nblk - 1;
    const int tail_valid = n_keys - last * BN;      // keys in the last block (BN unless the sequence is ragged)
    const bool fill_sum = BL && p.fill_kind == LBFQ_FILL_MEAN;   // the fill needs the block's mean score
    int n_skip = 0;                          // BLASST: blocks this row skipped
    bool s_seen = false;                     // this block's S-ready barrier was already observed (warp-uniform)
    uint32_t par = 0;                        // parity of the S-ready phases of the current pair of blocks

    // LAST: the sequence's final key block (the only one that can be ragged, has no successor to prefetch for or to
    // wait on); every other block runs the instantiation without those tests
    auto body = [&](auto buf_c, auto last_c, const int it) {
      constexpr int BUF = decltype(buf_c)::value;
      constexpr bool LAST = decltype(last_c)::value;
      if (!s_seen) mbar_wait_cont(bar_s[BUF], par, abort_flag, p.status, 12);
      s_seen = false;
      tc_fence_after();
      uint32_t mine[HB];
      tmem_ld(mine, tS_mine[BUF]);
      tc_wait_ld();
      // (sq * sk) * sm_scale in the reference's order; without a score bias straight into the log2 domain
      const float f = (sq * sk) * sm_scale;
      const float c = NAT ? 1.0f : f * kLog2e;
      constexpr bool more = !LAST;
      if (++scale_sub == blocks_per_scale) {   // next block's scale, off the critical path
        scale_sub = 0;
        if constexpr (!QB) {
          ksc += k_stride;
          if (more) sk = *ksc;
        }
      }
      // key block within its 128-key stage: with two blocks per stage it is the S buffer's index, a constant here
      [[maybe_unused]] const int sub_in_stage = (NSUB == 2) ? BUF : side_sub;
      if constexpr (CORR) {
        // scores = dot * f + corr (attention_triton.py:154-160)
        if (sub_in_stage == 0) mbar_wait_cont(BAR_SIDEFULL(side_stage), side_par, abort_flag, p.status, 15);
        const float* crow = corr_sm + side_stage * (2 * kChunk) + sub_in_stage * BN;
        const float4* cm = reinterpret_cast<const float4*>(crow + half * HB);
        const float2 f2 = make_float2(f, f);
#pragma unroll
        for (int i = 0; i < HB / 4; ++i) {
          const float4 a = cm[i];                          // same address in every lane: broadcast loads
          const float2 m01 = __ffma2_rn(make_float2(__uint_as_float(mine[4 * i]), __uint_as_float(mine[4 * i + 1])), f2, make_float2(a.x, a.y));
          const float2 m23 = __ffma2_rn(make_float2(__uint_as_float(mine[4 * i + 2]), __uint_as_float(mine[4 * i + 3])), f2, make_float2(a.z, a.w));
          mine[4 * i] = __float_as_uint(m01.x); mine[4 * i + 1] = __float_as_uint(m01.y);
          mine[4 * i + 2] = __float_as_uint(m23.x); mine[4 * i + 3] = __float_as_uint(m23.y);
        }
      }
      if constexpr (BL) {
        // scores = dot * f: the skip test and the fills are stated on them (attention_triton.py:154, 165-175)
        const float2 f2 = make_float2(f, f);
#pragma unroll
        for (int i = 0; i < HB; i += 2) {
          const float2 v = __fmul2_rn(make_float2(__uint_as_float(mine[i]), __uint_as_float(mine[i + 1])), f2);
          mine[i] = __float_as_uint(v.x); mine[i + 1] = __float_as_uint(v.y);
        }
      }
      const bool ragged = LAST && tail_valid < BN;
      if (ragged) {                            // ragged tail: only the last block of a sequence
#pragma unroll
        for (int i = 0; i < HB; ++i)
          if (half * HB + i >= tail_valid) mine[i] = 0xff800000u;
      }
      // three-input max (sm_100): two chains, two columns per instruction
      float bm0 = __uint_as_float(mine[0]), bm1 = __uint_as_float(mine[1]);
      static_assert((HB - 2) % 4 == 2, "the tail below takes the last two columns");
#pragma unroll
      for (int i = 2; i + 3 < HB; i += 4) {
        bm0 = fmax3(bm0, __uint_as_float(mine[i]), __uint_as_float(mine[i + 1]));
        bm1 = fmax3(bm1, __uint_as_float(mine[i + 2]), __uint_as_float(mine[i + 3]));
      }
      bm0 = fmax3(bm0, __uint_as_float(mine[HB - 2]), __uint_as_float(mine[HB - 1]));
      // the other half's maximum (a block's two slots alternate, so a slot is rewritten only after the barrier
      // of the next block, when its reader is done with it)
      const float own_max = fmaxf(bm0, bm1);
      *x_mine[BUF] = own_max;
      [[maybe_unused]] float row_sum = 0.f;                     // BLASST mean fill: sum of the block's valid scores
      if constexpr (BL) {
        if (fill_sum) {
          float2 sa = make_float2(0.f, 0.f), sb = make_float2(0.f, 0.f);
#pragma unroll
          for (int i = 0; i < HB; i += 4) {
            float2 a = make_float2(__uint_as_float(mine[i]), __uint_as_float(mine[i + 1]));
            float2 b2 = make_float2(__uint_as_float(mine[i + 2]), __uint_as_float(mine[i + 3]));
            if (ragged) {
              if (half * HB + i >= tail_valid) a.x = 0.f;
              if (half * HB + i + 1 >= tail_valid) a.y = 0.f;
              if (half * HB + i + 2 >= tail_valid) b2.x = 0.f;
              if (half * HB + i + 3 >= tail_valid) b2.y = 0.f;
            }
            sa = __fadd2_rn(sa, a);
            sb = __fadd2_rn(sb, b2);
          }
          row_sum = (sa.x + sa.y) + (sb.x + sb.y);
          x_mine[BUF][SM::kXch] = row_sum;
        }
      }
      // BLASST per-bin fill: one value per bin of BN / bins keys (a bin never straddles the two halves of the block).
      // A row skips exactly when both halves of its columns lie under the threshold, and a skipping row keeps its
      // running max: a thread whose own half qualifies computes its bins' fills now, against the old max, so that the
      // largest of them travels with the half's maximum through the one barrier of the block (wasted where only one
      // half qualifies). Only the scaled P modes need that maximum; with e4m3 P the bins are computed once the row is
      // known to skip.
      constexpr int kMinBin = BN / 16;                             // at most 16 bins per block are served
      [[maybe_unused]] float binval[HB / kMinBin];
      [[maybe_unused]] float fill_max_own = 0.f;
      [[maybe_unused]] const bool uta = BL && p.fill_kind == LBFQ_FILL_UTA;
      auto compute_bins = [&]() {
            const int nvalid = more ? BN : tail_valid;
            auto bins = [&](auto bs_c) {
              constexpr int BS = decltype(bs_c)::value;
              if constexpr (BS <= HB && BS >= kMinBin) {
                constexpr float kInvBs = 1.0f / BS;                 // a power of two: multiplying by it divides exactly
#pragma unroll
                for (int b0 = 0; b0 < HB; b0 += BS) {
                  float bsum = 0.f, bmx = -INFINITY, bcnt = 0.f;
#pragma unroll
                  for (int i = b0; i < b0 + BS; ++i) {
                    const float x = __uint_as_float(mine[i]);
                    if (ragged) {
                      const bool ok = half * HB + i < nvalid;
                      bsum += ok ? x : 0.f;
                      bcnt += ok ? 1.f : 0.f;
                    } else {
                      bsum += x;
                    }
                    bmx = fmaxf(bmx, x);                            // masked scores are -inf already
                  }
                  float val;
                  if (ragged) {
                    const float safe_c = fmaxf(bcnt, 1.f);
                    const float bound = safe_c * ex2(fmaf(bmx - m2, kLog2e, p_off));
                    const float mass = p.fill_alpha * safe_c * ex2(fmaf(bsum / safe_c - m2, kLog2e, p_off));
                    val = fminf(mass, bound) / safe_c;
                  } else {
                    const float bound = (float)BS * ex2(fmaf(bmx - m2, kLog2e, p_off));
                    const float mass = p.fill_alpha * (float)BS * ex2(fmaf(bsum * kInvBs - m2, kLog2e, p_off));
                    val = fminf(mass, bound) * kInvBs;
                  }
                  binval[b0 / BS] = val;
                  fill_max_own = fmaxf(fill_max_own, val);
                }
              }
            };
            switch (BN / p.uta_bins) {
              case 2: bins(std::integral_constant<int, 2>{}); break;
              case 4: bins(std::integral_constant<int, 4>{}); break;
              case 8: bins(std::integral_constant<int, 8>{}); break;
              case 16: bins(std::integral_constant<int, 16>{}); break;
              default: bins(std::integral_constant<int, 32>{}); break;
            }
      };
      if constexpr (BL && PK != 0) {
        if (uta) {
          if ((own_max - m2) < p.log_lambda) compute_bins();
          x_mine[BUF][2 * SM::kXch] = fill_max_own;
        }
      }
      [[maybe_unused]] bool warp_skip = false;
      if constexpr (TV) {
        // (max(a, b) - m) < log(lambda) holds exactly when it holds for a and for b: each thread tests its own half
        // of the columns and a warp publishes one byte, 1 = all of its rows' halves lie under the threshold (rows past
        // the end of the sequence agree with anything). Every warp arrives on the vote barrier and goes on; only a
        // warp that voted 1 waits there, further down, for the other seven votes.
        const bool half_skip = !row_ok || (own_max - m2) < p.log_lambda;
        warp_skip = __all_sync(0xffffffffu, half_skip);
        if (lane == 0) {
          votes[(BUF * 2 + t) * 8 + (warp & 7)] = warp_skip ? 1 : 0;
          mbar_arrive(BAR_VOTE(t, BUF));
        }
      }
      __syncwarp();                            // a named barrier counts warps: arrive once, converged
      asm volatile("bar.sync %0, 64;" ::"r"(pair_bar) : "memory");
      if constexpr (TV) {
        if (warp_skip) {
          // a warp is never two blocks ahead of another one, so the barrier's phase is the block pair's parity
          mbar_wait_cont(BAR_VOTE(t, BUF), (uint32_t)(it >> 1) & 1u, abort_flag, p.status, 16);
          if (*reinterpret_cast<const volatile unsigned long long*>(votes + (BUF * 2 + t) * 8) == kAllVotes) {
            // nothing of this block enters the tile: running max, row sum and accumulator stay as they are. The
            // arrival still tells the MMA thread that S has been read (it reads the votes itself and issues no P.V).
            n_skip += 1;
            tc_fence_before();
            if constexpr (PK == 0) {
              mbar_arrive(bar_prdy + 8u * BUF);
            } else {
              __syncwarp();
              if (lane == 0) mbar_arrive(bar_prdy + 8u * BUF);
            }
            return;
          }
        }
      }
      bm0 = own_max;
      bm1 = *x_oth[BUF];
      if constexpr (BL) {
        if (fill_sum) row_sum += x_oth[BUF][SM::kXch];           // commutative: both threads of the row get the same bits
      }
      const float bmax_raw = fmaxf(bm0, bm1);
      const float bmax = bmax_raw * c;

      // ---- running max / rescale factor (attention_triton.py:164-217) ----------
      constexpr float kUp = CORR ? 16.0f / kLog2e : 16.0f, kDown = CORR ? 32.0f / kLog2e : 32.0f;
      constexpr float kFloor = CORR ? 80.0f : 80.0f * kLog2e;
      float m_new;
      bool fresh = false;                      // thresholds mode, nothing accumulated yet: alpha = 0
      bool moved = !frozen;
      if (thresholds) {
        const float seen = fmaxf(max_seen, bmax);
        const bool under = (bmax - m2) > kUp;
        const bool over = (m2 - seen) > kDown;
        const float down_m = l_pos ? fmaxf(seen + kDown, m2 - kFloor) : seen;
        moved = under || over;
        m_new = moved ? (under ? bmax : down_m) : m2;
        fresh = moved && !l_pos;
        max_seen = seen;
      } else {
        m_new = frozen ? m2 : fmaxf(m2, bmax);
      }
      [[maybe_unused]] bool skip = false;                       // BLASST: this row's block is below the threshold (attention_triton.py:165-175)
      if constexpr (BL) {
        skip = (bmax - m_new) < p.log_lambda;
        if constexpr (TV) {
          if (p.tile_pred) skip = false;         // the tile as a whole kept this block: every row of it computes it
        }
        if (skip) m_new = m2;
        moved = !skip;
        n_skip += skip ? 1 : 0;
      }
      const float alpha = !moved ? 1.f : (fresh ? 0.f : ex2(NAT ? (m2 - m_new) * kLog2e : m2 - m_new));
      // ---- P = exp2(dot * c - m + off), l += sum(P) (attention_triton.py:219-326) ----
      // masked columns hold -inf, so their exp2 is exactly 0 without a select
      // two columns per instruction: fma.rn.f32x2 / add.rn.f32x2 round each half exactly like the scalar forms.
      // Without a score bias: exp2(dot * c + (off - m)), max in the log2 domain. With scores in their own units:
      // exp2(score * log2e + (off - m * log2e)), the reference's (score - m) * log2e + off contracted into one FMA.
      const float bias = NAT ? fmaf(-m_new, kLog2e, p_off) : p_off - m_new;
      const float2 c2 = make_float2(NAT ? kLog2e : c, NAT ? kLog2e : c);
      const float2 bias2 = make_float2(bias, bias);
      auto arg = [&](uint32_t x0, uint32_t x1) -> float2 {
        return __ffma2_rn(make_float2(__uint_as_float(x0), __uint_as_float(x1)), c2, bias2);
      };
      float2 psa = make_float2(0.f, 0.f), psb = make_float2(0.f, 0.f);
      uint32_t pk[PW];
      // exp2 is monotonic: the largest P of the block is the P of the largest score, produced by the same
      // instruction sequence as the elements, so it is bit-identical to max_i(P_i) -- and both threads of the
      // row know it without talking to each other
      [[maybe_unused]] float pmax = 1.f;
      [[maybe_unused]] float s_p = 1.f, inv_p = 1.f;
      // Without BLASST the scaled P modes never form p itself: q = p / s_P = exp2(z - log2 s_P) comes straight out of the
      // exponential (one multiplication per element less), and the row sum is s_P * sum(q).
      constexpr bool FOLD = PK != 0 && !BL;
      [[maybe_unused]] float bias_q = bias;
      [[maybe_unused]] float fill_const = 0.f;          // BLASST: the value a skipped row fills every column with
      if constexpr (BL) {
        // A skipped row contributes a softmax-free fill instead of its exponentials (attention_triton.py:231-324):
        // the fill values replace the scores in `mine`, their maximum stands in for the largest P.
        float fill_max = 0.f;
        fill_const = 0.f;
        if (skip) {
          const int nvalid = more ? BN : tail_valid;
          const float safe_n = (float)nvalid;                       // a block holds at least one key
          if (uta) {
            if constexpr (PK == 0) {
              // e4m3 P needs no largest fill: nothing to exchange, nothing to guess. The fills replace the scores.
              auto bins = [&](auto bs_c) {
                constexpr int BS = decltype(bs_c)::value;
                if constexpr (BS <= HB) {
#pragma unroll
                  for (int b0 = 0; b0 < HB; b0 += BS) {
                    float bsum = 0.f, bmx = -INFINITY, bcnt = 0.f;
#pragma unroll
                    for (int i = b0; i < b0 + BS; ++i) {
                      const bool ok = half * HB + i < nvalid;
                      const float x = __uint_as_float(mine[i]);
                      bsum += ok ? x : 0.f;
                      bmx = fmaxf(bmx, x);                          // masked scores are -inf already
                      bcnt += ok ? 1.f : 0.f;
                    }
                    const float safe_c = fmaxf(bcnt, 1.f);
                    const float bound = safe_c * ex2(fmaf(bmx - m_new, kLog2e, p_off));
                    const float mass = p.fill_alpha * safe_c * ex2(fmaf(bsum / safe_c - m_new, kLog2e, p_off));
                    const float val = fminf(mass, bound) / safe_c;
#pragma unroll
                    for (int i = b0; i < b0 + BS; ++i) mine[i] = (half * HB + i < nvalid) ? __float_as_uint(val) : 0u;
                  }
                }
              };
              switch (BN / p.uta_bins) {
                case 2: bins(std::integral_constant<int, 2>{}); break;
                case 4: bins(std::integral_constant<int, 4>{}); break;
                case 8: bins(std::integral_constant<int, 8>{}); break;
                case 16: bins(std::integral_constant<int, 16>{}); break;
                default: bins(std::integral_constant<int, 32>{}); break;
              }
            }
            fill_max = fill_max_own;
            if constexpr (PK != 0) fill_max = fmaxf(fill_max, x_oth[BUF][2 * SM::kXch]);
          } else {
            float fill_p = 0.f;
            if (p.fill_kind != LBFQ_FILL_ZERO) {
              // a full block holds the power of two BN keys: its reciprocal multiplies exactly
              auto per_key = [&](float x) { return ragged ? x / safe_n : x * (1.0f / BN); };
              const float max_bound = safe_n * ex2(fmaf(bmax - m_new, kLog2e, p_off));
              if (p.fill_kind == LBFQ_FILL_MAX) {
                fill_p = per_key(max_bound * p.fill_alpha);
              } else if (p.fill_kind == LBFQ_FILL_MEAN) {
                fill_p = per_key(fminf(p.fill_alpha * safe_n * ex2(fmaf(per_key(row_sum) - m_new, kLog2e, p_off)), max_bound));
              } else {                                              // LBFQ_FILL_THR
                const float off_scale = p_el ? exp2f(p_off) : 1.f;
                fill_p = per_key(p.fill_alpha * safe_n * p.lambda * off_scale);
              }
            }
            fill_max = fill_p;
            fill_const = fill_p;
            if (ragged) {
#pragma unroll
              for (int i = 0; i < HB; ++i) mine[i] = (half * HB + i < nvalid) ? __float_as_uint(fill_p) : 0u;
            }
          }
        }
        if constexpr (PK != 0) pmax = skip ? fill_max : ex2(fmaf(bmax, kLog2e, bias));
      } else if constexpr (PK != 0) {
        if constexpr (CORR) pmax = ex2(fmaf(bmax, kLog2e, bias));
        else pmax = ex2(fmaf(bmax_raw, c, bias));
      }
      if constexpr (PK != 0) {
        // P scale of the block (attention_triton.py:338-360): a power of two (mx) or amax / 448 (dynamic)
        if (p_el) {
          // element-wise P keeps scale 1 (it takes this path when the V-smoothing term needs the BF16 P.V)
        } else if (p_mx) {
          const int e = pow2_scale_exp(fmaxf(pmax, 1e-4f));
          s_p = pow2f(e);
          inv_p = pow2f(-e);
          if constexpr (FOLD) bias_q = bias - (float)e;                    // p * 2^-e = exp2(z - e)
        } else {
          s_p = scale_from_amax(fmaxf(pmax, 1e-12f));          // the reference's `amax / 448` and `p / s` (common.cuh)
          if constexpr (FOLD) {
            // p / s_P = 448 * exp2(z - z_max): the running max drops out of the quotient. (Blocks whose largest P is
            // under the 1e-12 floor keep the floored scale: exp2(z - log2(1e-12 / 448)).)
            constexpr float kLog2Fp8Max = 8.807354922057604f;              // log2(448)
            constexpr float kLog2Floor = -48.67133070387592f;              // log2(1e-12 / 448)
            if (pmax >= 1e-12f) bias_q = CORR ? fmaf(-bmax, kLog2e, kLog2Fp8Max) : fmaf(-bmax_raw, c, kLog2Fp8Max);
            else bias_q = bias - kLog2Floor;
          } else {
            inv_p = rcp_approx(s_p);
          }
        }
      }
      const float2 bias_q2 = make_float2(bias_q, bias_q);
      auto arg_q = [&](uint32_t x0, uint32_t x1) -> float2 {
        return __ffma2_rn(make_float2(__uint_as_float(x0), __uint_as_float(x1)), c2, bias_q2);
      };
      const float2 inv2 = make_float2(inv_p, inv_p);
      // row sum over the unquantised P, then the P operand of the block's P.V
      auto emit = [&](const int i, const float2 pa, const float2 pb) {
        psa = __fadd2_rn(psa, pa);
        psb = __fadd2_rn(psb, pb);
        if constexpr (PK == 0) {
          // the conversion saturates at 448, which is the reference's clamp (attention_triton.py:328-336)
          pk[i / 4] = f32x4_to_e4m3x4(pa.x, pa.y, pb.x, pb.y);
        } else {
          // e4m3(p / s) * s, rounded to BF16: the operand the reference gives its P.V product
          float2 qa = pa, qb = pb;                                        // FOLD: pa, pb are the quotients already
          if constexpr (!FOLD) { qa = __fmul2_rn(pa, inv2); qb = __fmul2_rn(pb, inv2); }
          pk[i / 2] = e4m3_round_scale_bf16x2(qa.x, qa.y, s_p);
          pk[i / 2 + 1] = e4m3_round_scale_bf16x2(qb.x, qb.y, s_p);
        }
      };
      // (Selecting fill or exponential lane by lane in one pass, so that a warp with both kinds of rows quantises
      // once, measured 20-30 % slower in the blocks where nothing skips: the scores stay live across the
      // exponentials. The two paths below diverge instead; a warp whose rows all skip computes no exponentials.)
      if (BL && PK != 0 && skip && uta) {
        // a bin's value is quantised once and replicated over the bin's columns; BS times the value is exact
        auto put = [&](auto bs_c) {
          constexpr int BS = decltype(bs_c)::value;
          if constexpr (BS <= HB && BS >= kMinBin) {
            if (ragged) {
              const int nvalid = more ? BN : tail_valid;
#pragma unroll
              for (int i = 0; i < HB; ++i) mine[i] = (half * HB + i < nvalid) ? __float_as_uint(binval[i / BS]) : 0u;
#pragma unroll
              for (int i = 0; i < HB; i += 4)
                emit(i, make_float2(__uint_as_float(mine[i]), __uint_as_float(mine[i + 1])),
                     make_float2(__uint_as_float(mine[i + 2]), __uint_as_float(mine[i + 3])));
            } else {
              float sum = 0.f;
#pragma unroll
              for (int b = 0; b < HB / BS; ++b) {
                const float v = binval[b];
                sum += v * (float)BS;
                if constexpr (PK == 0) {
                  if constexpr (BS >= 4) {
                    const uint32_t w = f32x4_to_e4m3x4(v, v, v, v);
#pragma unroll
                    for (int j = 0; j < BS / 4; ++j) pk[b * (BS / 4) + j] = w;
                  } else if (b % 2 == 0) {
                    pk[b / 2] = f32x4_to_e4m3x4(v, v, binval[b + 1], binval[b + 1]);
                  }
                } else {
                  const float q = v * inv_p;
                  const uint32_t w = e4m3_round_scale_bf16x2(q, q, s_p);
#pragma unroll
                  for (int j = 0; j < BS / 2; ++j) pk[b * (BS / 2) + j] = w;
                }
              }
              psa = make_float2(sum, 0.f);
            }
          }
        };
        switch (BN / p.uta_bins) {
          case 2: put(std::integral_constant<int, 2>{}); break;
          case 4: put(std::integral_constant<int, 4>{}); break;
          case 8: put(std::integral_constant<int, 8>{}); break;
          case 16: put(std::integral_constant<int, 16>{}); break;
          default: put(std::integral_constant<int, 32>{}); break;
        }
      } else if (BL && skip) {
        if (!ragged && !uta) {
          // one value in every column of a full block: quantised once; HB times the value is exact
          const float2 pf = make_float2(fill_const, fill_const);
          emit(0, pf, pf);
#pragma unroll
          for (int w = 1; w < PW; ++w) pk[w] = pk[0];
          psa = make_float2(fill_const * (HB / 4), fill_const * (HB / 4));
          psb = psa;
        } else {
#pragma unroll
          for (int i = 0; i < HB; i += 4)
            emit(i, make_float2(__uint_as_float(mine[i]), __uint_as_float(mine[i + 1])),
                 make_float2(__uint_as_float(mine[i + 2]), __uint_as_float(mine[i + 3])));
        }
      } else {
#pragma unroll
        for (int i = 0; i < HB; i += 4) {
          const float2 za = FOLD ? arg_q(mine[i], mine[i + 1]) : arg(mine[i], mine[i + 1]);
          const float2 zb = FOLD ? arg_q(mine[i + 2], mine[i + 3]) : arg(mine[i + 2], mine[i + 3]);
          emit(i, make_float2(ex2(za.x), ex2(za.y)), make_float2(ex2(zb.x), ex2(zb.y)));
        }
      }
      if constexpr (FOLD) l_i = fmaf(l_i, alpha, s_p * ((psa.x + psa.y) + (psb.x + psb.y)));     // sum(p) = s_P * sum(q)
      else l_i = l_i * alpha + ((psa.x + psa.y) + (psb.x + psb.y));
      if constexpr (PK != 0) l_pos = pmax > 0.f || (l_pos && alpha != 0.f);
      if (it > 0 && __any_sync(0xffffffffu, alpha != 1.f)) {
        // Some row of this warp raised its max: the accumulator must be rescaled before this block's P.V,
        // and P.V of the previous block must have completed. S of the next block was issued behind that
        // P.V by the same thread, and a commit covers everything issued before it: once the next S is ready
        // (a wait that is due at the top of the next block anyway), the accumulator is quiescent. The last
        // block has no successor and waits for its predecessor's P.V directly. A warp whose rows keep their
        // max -- nearly every warp after the first few hundred keys -- waits for nothing here.
        if (more) {
          mbar_wait_cont(bar_s[BUF ^ 1], BUF == 0 ? par : (par ^ 1u), abort_flag, p.status, 12);
          s_seen = true;
        } else {
          mbar_wait_cont(bar_penult, 0, abort_flag, p.status, 11);
        }
        tc_fence_after();                     // rescale this warp's half of its 32 accumulator rows in place
#pragma unroll
        for (int c0 = 0; c0 < HD; c0 += 32) {
          uint32_t r[32];
          LBFQ_TMEM_LD32(r, tO + c0);
          tc_wait_ld();
          const float2 a2 = make_float2(alpha, alpha);
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            const float2 v = __fmul2_rn(make_float2(__uint_as_float(r[i]), __uint_as_float(r[i + 1])), a2);
            r[i] = __float_as_uint(v.x); r[i + 1] = __float_as_uint(v.y);
          }
          LBFQ_TMEM_ST32(tO + c0, r);
        }
      }
      if constexpr (VALPHA) {
        // c_acc += rowsum(P) * alpha_v (attention_triton.py:378-383) as one more K step of P.V: this thread's part of
        // the row sum of the BF16 P, split into three BF16 pieces, against the pieces of alpha' staged by the
        // producer: (h + m + l) * (h' + m' + l') without the three smallest cross terms
        // (the sum has to see the BF16 rounding of P: summing the FP32 products instead moved the result by up to
        // 4e-3 of its RMS with dynamic P, whose few distinct codes per row and block round alike)
        float r0 = 0.f, r1 = 0.f, r2 = 0.f, r3 = 0.f;
#pragma unroll
        for (int w = 0; w < PW; w += 2) {
          add_bf16x2_f32(r0, r1, pk[w]);
          add_bf16x2_f32(r2, r3, pk[w + 1]);
        }
        float rs = (r0 + r1) + (r2 + r3);
        const __nv_bfloat16 rh = __float2bfloat16_rn(rs);
        rs -= __bfloat162float(rh);
        const __nv_bfloat16 rm = __float2bfloat16_rn(rs);
        rs -= __bfloat162float(rm);
        const __nv_bfloat16 rl = __float2bfloat16_rn(rs);
        const uint32_t uh = __bfloat16_as_ushort(rh), um = __bfloat16_as_ushort(rm), ul = __bfloat16_as_ushort(rl);
        const uint32_t ext[4] = {uh | (uh << 16), uh | (um << 16), um | (ul << 16), 0u};      // h h h m m l 0 0
        tmem_st4(tA[BUF], ext);
      }
      if constexpr (PW == 16) { LBFQ_TMEM_ST16(tP[BUF], pk); }
      else if constexpr (PW == 8) tmem_st8(tP[BUF], pk);
      else tmem_st4(tP[BUF], pk);
      tc_wait_st();                            // warp-collective: every lane's P is in tensor memory
      tc_fence_before();
      // the e4m3-P instantiations are faster with every thread arriving, the BF16-P ones with one arrival per warp
      // (measured on the two benchmark stacks: 1.3 % and 1.0 %)
      if constexpr (PK == 0) {
        mbar_arrive(bar_prdy + 8u * BUF);
      } else {
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_prdy + 8u * BUF);
      }
      m2 = m_new;
      if constexpr (CORR) {
        // the stage's bias rows are dead once its last key block has read them (every lane has: __syncwarp above)
        if ((sub_in_stage == NSUB - 1 || !more) && lane == 0) mbar_arrive(BAR_SIDEFREE(side_stage));
        if (++side_sub == NSUB) {
          side_sub = 0;
          if (++side_stage == kFastStages) { side_stage = 0; side_par ^= 1u; }
        }
      }
    };
    {
      using B0 = std::integral_constant<int, 0>;
      using B1 = std::integral_constant<int, 1>;
      int it = 0;
#pragma unroll 1
      for (; it + 2 < nblk; it += 2) {
        body(B0{}, std::false_type{}, it);
        body(B1{}, std::false_type{}, it + 1);
        par ^= 1u;
      }
      if (it + 1 < nblk) {
        body(B0{}, std::false_type{}, it);
        body(B1{}, std::true_type{}, it + 1);
      } else {
        body(B0{}, std::true_type{}, it);
      }
    }

    // ---- epilogue (attention_triton.py:387-407) ---------------------------------
    mbar_wait_cont(BAR_ODONE(t), 0, abort_flag, p.status, 13);
    // the row sum is the sum of the two column halves
    float* lsum = reinterpret_cast<float*>(smem + SM::offL);
    lsum[(t * 2 + half) * kTileM + row_in_tile] = l_i;
    asm volatile("bar.sync 1, %0;" ::"n"(kFastSoftmaxWarps * 32) : "memory");
    const bool store_ok = row_ok && *abort_flag == 0;          // the loads below are collective, the stores are not
    {
      tc_fence_after();
      // the reference's `1.0 / l_i` (attention_triton.py:387)
      const float inv_l = rcp_approx(lsum[(t * 2) * kTileM + row_in_tile] + lsum[(t * 2 + 1) * kTileM + row_in_tile]);
      const bool has_vsc = p.v_kind == LBFQ_V_CHANNEL;
      const float* vsc = (has_vsc ? p.v_scale + (size_t)bh * D : p.v_scale) + half * HD;
      int64_t drow = rowc;
      if (p.out_row_index != nullptr) drow = p.out_row_index[(size_t)bh * p.M + rowc];
      const size_t o_off = (p.out_layout == LBFQ_LAYOUT_NHD
                               ? (((size_t)b * p.M + drow) * p.H + h) * D
                               : ((size_t)bh * p.M + drow) * D) + half * HD;
#pragma unroll
      for (int c0 = 0; c0 < HD; c0 += 32) {
        uint32_t r[32];
        float a[32];
        LBFQ_TMEM_LD32(r, tO + c0);             // warp-collective: rows past M take part and store nothing
        tc_wait_ld();
        if (has_vsc) {
#pragma unroll
          for (int i = 0; i < 32; ++i) a[i] = (__uint_as_float(r[i]) * vsc[c0 + i]) * inv_l;
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) a[i] = __uint_as_float(r[i]) * inv_l;
        }
        if (!store_ok) {
          // rows past M, and every row of a launch that gave up a wait, only take part in the collective load
        } else if (p.out_dtype == LBFQ_F32) {
          float4* o = reinterpret_cast<float4*>((float*)p.out + o_off + c0);
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            float4 v = make_float4(a[4 * i], a[4 * i + 1], a[4 * i + 2], a[4 * i + 3]);
            if (!p.out_exact) {
              v.x = round_through<__nv_bfloat16>(v.x); v.y = round_through<__nv_bfloat16>(v.y);
              v.z = round_through<__nv_bfloat16>(v.z); v.w = round_through<__nv_bfloat16>(v.w);
            }
            o[i] = v;
          }
        } else {
          uint4* o = reinterpret_cast<uint4*>((uint16_t*)p.out + o_off + c0);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            uint32_t w[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const float x0 = a[8 * i + 2 * j], x1 = a[8 * i + 2 * j + 1];
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
    }
    if constexpr (BL) {
      // skipped and total row-decisions per block_m rows (attention_triton.py:404-407)
      if (half == 0 && row_ok && p.stats != nullptr && *abort_flag == 0) {
        float* st2 = p.stats + ((size_t)(row / p.block_m) * (p.B * p.H) + bh) * 2;
        atomicAdd(st2 + 0, (float)n_skip);
        atomicAdd(st2 + 1, (float)nblk);
      }
    }
  } else {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(FastRegs<BL>::kService));
  }
  if (warp == kTmaWarp) {
    // =========================== TMA producer =====================================
    if (lane == 0) {
      for (int t = 0; t < 2; ++t) {
        mbar_expect_tx(BAR_QFULL(t), SM::kQ);
        if constexpr (QB == 0) {
          tma_load_3d(sbase + SM::offQ + t * SM::kQ, &tm_q, 0, m0 + t * kTileM, bh, BAR_QFULL(t));
        } else {                                          // BF16: D / 64 panels of 128 rows x 128 bytes
          for (int pn = 0; pn < D / 64; ++pn)
            tma_load_3d(sbase + SM::offQ + t * SM::kQ + pn * (kTileM * 128), &tm_q, pn * 64, m0 + t * kTileM, bh, BAR_QFULL(t));
        }
      }
      for (int c = 0; c < nchunk; ++c) {
        const int st = c % kFastStages;
        if (c >= kFastStages) {
          const uint32_t par = ((c / kFastStages) - 1) & 1;
          if (!mbar_wait(BAR_KFREE(st), par, abort_flag, p.status, 21)) break;
        }
        mbar_expect_tx(BAR_KFULL(st), SM::kK);
        if constexpr (QB == 0) {
          tma_load_3d(sbase + SM::offK + st * SM::kK, &tm_k, 0, c * kChunk, bh, BAR_KFULL(st));
        } else {
          for (int pn = 0; pn < D / 64; ++pn)
            tma_load_3d(sbase + SM::offK + st * SM::kK + pn * (kChunk * 128), &tm_k, pn * 64, c * kChunk, bh, BAR_KFULL(st));
        }
        if (c >= kFastStages) {
          const uint32_t par = ((c / kFastStages) - 1) & 1;
          if (!mbar_wait(BAR_VFREE(st), par, abort_flag, p.status, 22)) break;
        }
        mbar_expect_tx(BAR_VFULL(st), SM::kV);
        if constexpr (PK == 0) {
          tma_load_3d(sbase + SM::offV + st * SM::kV, &tm_v, c * kChunk, 0, bh, BAR_VFULL(st));
        } else {                                      // BF16 V^T: two 64-key panels of D rows x 128 bytes
          tma_load_3d(sbase + SM::offV + st * SM::kV, &tm_v, c * kChunk, 0, bh, BAR_VFULL(st));
          tma_load_3d(sbase + SM::offV + st * SM::kV + D * 128, &tm_v, c * kChunk + 64, 0, bh, BAR_VFULL(st));
        }
        if constexpr (CORR || VALPHA) {
          // (the alpha' tiles are read by the same MMAs as V^T: the wait for the V stage above covers them)
          if (CORR && c >= kFastStages && !mbar_wait(BAR_SIDEFREE(st), ((c / kFastStages) - 1) & 1, abort_flag, p.status, 23)) break;
          const int vsb_c = min(p.v_smooth_block, kChunk);          // keys per V-smoothing tile within a stage
          const int ntile = VALPHA ? kChunk / vsb_c : 0;
          mbar_expect_tx(BAR_SIDEFULL(st), (CORR ? 2 * kChunk * 4 : 0) + ntile * SM::kAext);
          if constexpr (CORR) {
            for (int t = 0; t < 2; ++t) {
              const int g = min((m0 + t * kTileM) / p.q_smooth_block, p.n_groups - 1);
              bulk_load(sbase + SM::offCorr + (st * 2 + t) * (kChunk * 4),
                        p.corr + ((size_t)bh * p.n_groups + g) * p.corr_stride + (size_t)c * kChunk, kChunk * 4, BAR_SIDEFULL(st));
            }
          }
          if constexpr (VALPHA) {
            for (int sl = 0; sl < ntile; ++sl) {
              const int key = min(c * kChunk + sl * vsb_c, p.N - 1);   // a tile past the end re-reads the last one
              const int slab = (b * (p.N / p.v_smooth_block) + key / p.v_smooth_block) * p.H + h;
              tma_load_3d(sbase + SM::offAext + (st * 2 + sl) * SM::kAext, &tm_a, 0, 0, slab, BAR_SIDEFULL(st));
            }
          }
        }
      }
    }
  } else if (warp == kMmaWarp0 || warp == kMmaWarp0 + 1) {
    // =========================== MMA issuer of tile t ==============================
    const int t = warp - kMmaWarp0;
    if (lane == 0) {
      const uint32_t tS = tmem_base + t * TCOLS + COL_S;
      const uint32_t tO = tmem_base + t * TCOLS + COL_O;
      const uint32_t id_qk = make_idesc(BN);
      const uint32_t id_pv = make_idesc(D);
      const uint32_t id_pv_bf16 = make_idesc_bf16(D);
      // Descriptors differ from one stage / key block to the next only in their 14-bit start-address field (16-byte
      // units; shared memory ends below 2^18 bytes, so adding to the whole word never carries out of the field).
      const uint64_t dq = QB == 0 ? make_desc(sbase + SM::offQ + t * SM::kQ, D) : make_desc(sbase + SM::offQ + t * SM::kQ, 128);
      const uint64_t dk0 = QB == 0 ? make_desc(sbase + SM::offK, D) : make_desc(sbase + SM::offK, 128);
      const uint64_t dv0 = PK == 0 ? make_desc(sbase + SM::offV, kChunk) : make_desc(sbase + SM::offV, 128);
      [[maybe_unused]] const uint64_t da0 = make_desc(sbase + SM::offAext, 32);
      // smoothing blocks of 64 keys or of whole stages (the launcher admits nothing else here): tile index by shift
      [[maybe_unused]] const int sl_shift = min(p.v_smooth_block, kChunk) == 64 ? 6 : 7;
      bool ok = mbar_wait(BAR_QFULL(t), 0, abort_flag, p.status, 31);
      // The two instruction streams of this thread, each with its position in the ring of key stages: Q.K^T runs two
      // key blocks ahead of P.V. `ready` waits for the stage a block starts (long landed when its turn comes) and
      // forms the block's descriptors; `issue` only issues. The loop below calls `ready` for both streams *before*
      // it waits for P, so that nothing but the MMAs themselves stands between "P is ready" and "S of block it + 2
      // is ready", the round trip the softmax warps wait for.
      struct Pos { int sub, st; uint32_t par; };
      Pos qk{0, 0, 0u}, pv{0, 0, 0u};
      auto advance = [&](Pos& x) {
        if (++x.sub == NSUB) {
          x.sub = 0;
          if (++x.st == kFastStages) { x.st = 0; x.par ^= 1u; }
        }
      };
      uint64_t dk = 0, dv = 0;
      [[maybe_unused]] uint64_t da = 0;
      // `block`: wait for the stage; otherwise only look, and tell whether the stage is there
      auto ready_qk = [&](bool block, bool& have) -> bool {
        dk = dk0 + (uint64_t)((qk.st * SM::kK + qk.sub * BN * (QB == 0 ? D : 128)) >> 4);
        have = true;
        if (qk.sub != 0) return true;
        if (!block) {
          have = mbar_test(BAR_KFULL(qk.st), qk.par);
          return true;
        }
        return mbar_wait(BAR_KFULL(qk.st), qk.par, abort_flag, p.status, 32);
      };
      auto issue_qk = [&](int j) {
        if constexpr (QB == 0) {
#pragma unroll
          for (int kk = 0; kk < D / 32; ++kk)
            mma_f8_ss(tS + (j & 1) * S_STRIDE, dq + (uint64_t)(kk * 2), dk + (uint64_t)(kk * 2), id_qk, kk > 0 ? 1u : 0u);
        } else {
          // BF16: K steps of 16 channels, four per 64-channel panel
          const uint32_t id_qk_bf16 = make_idesc_bf16(BN);
#pragma unroll
          for (int kk = 0; kk < D / 16; ++kk)
            mma_bf16_ss(tS + (j & 1) * S_STRIDE, dq + (uint64_t)((((kk >> 2) * (kTileM * 128)) >> 4) + (kk & 3) * 2),
                        dk + (uint64_t)((((kk >> 2) * (kChunk * 128)) >> 4) + (kk & 3) * 2), id_qk_bf16, kk > 0 ? 1u : 0u);
        }
        tc_commit(BAR_SFULL(t, j & 1));
      };
      auto retire_qk = [&](int j) {
        if (qk.sub == NSUB - 1 || j == nblk - 1) tc_commit(BAR_KFREE(qk.st));
        advance(qk);
      };
      unsigned long long n_elided = 0;
      auto ready_pv = [&]() -> bool {
        // (the stage's V is awaited even when no P.V reads it: a stage is handed back only once its load has landed)
        if (pv.sub == 0 && !mbar_wait(BAR_VFULL(pv.st), pv.par, abort_flag, p.status, 33)) return false;
        if constexpr (VALPHA) {
          if (pv.sub == 0 && !mbar_wait(BAR_SIDEFULL(pv.st), pv.par, abort_flag, p.status, 37)) return false;
        }
        const int key0 = pv.sub * BN;
        if constexpr (PK == 0) {
          dv = dv0 + (uint64_t)((pv.st * SM::kV) >> 4) + (uint64_t)(key0 >> 4);
        } else {
          // keys key0 ... of the stage: panel key0 / 64, (key0 % 64) keys = 2 bytes each into its rows
          dv = dv0 + (uint64_t)((pv.st * SM::kV + (key0 >> 6) * (D * 128)) >> 4) + (uint64_t)(((key0 & 63) * 2) >> 4);
        }
        if constexpr (VALPHA) da = da0 + (uint64_t)(((pv.st * 2 + (key0 >> sl_shift)) * SM::kAext) >> 4);
        return true;
      };
      auto issue_pv = [&](int j) {
        bool elide = false;
        if constexpr (TV) {
          // every row of the tile skipped this block: there is no P. (Never the first block: a row's running max
          // starts at -inf, which no block is below.)
          elide = *reinterpret_cast<const volatile unsigned long long*>(votes + ((j & 1) * 2 + t) * 8) == kAllVotes;
          n_elided += elide ? 1 : 0;
        }
        if (elide) {
          // the commits below still fire: they track the operations issued so far
        } else if constexpr (PK == 0) {
#pragma unroll
          for (int kk = 0; kk < BN / 32; ++kk)
            mma_f8_ts(tO, tS + (j & 1) * S_STRIDE + kk * 8, dv + (uint64_t)(kk * 2), id_pv, (j > 0 || kk > 0) ? 1u : 0u);
        } else {
#pragma unroll
          for (int kk = 0; kk < BN / 16; ++kk)
            mma_bf16_ts(tO, tS + (j & 1) * S_STRIDE + kk * 8, dv + (uint64_t)(kk * 2), id_pv_bf16,
                        (j > 0 || kk > 0) ? 1u : 0u);
          // one more K step: the row-sum pieces (TMEM columns 32..39 of the block's buffer) against alpha' pieces
          if constexpr (VALPHA) mma_bf16_ts(tO, tS + (j & 1) * S_STRIDE + 32, da, id_pv_bf16, 1u);
        }
      };
      // (a commit covers everything this thread has issued so far: the stage hand-backs below may follow the next
      // Q.K^T, they only fire a little later)
      auto free_v = [&](int j) {
        if (pv.sub == NSUB - 1 || j == nblk - 1) tc_commit(BAR_VFREE(pv.st));
      };
      auto retire_pv = [&](int j) {
        if (j == nblk - 2) tc_commit(BAR_PENULT(t));
        if (j == nblk - 1) tc_commit(BAR_ODONE(t));
        if constexpr (kFastStages > 2) free_v(j);
        advance(pv);
      };
      bool have_k = true;
      for (int j = 0; j < 2 && j < nblk && ok; ++j) {
        ok = ready_qk(true, have_k);
        if (ok) {
          tc_fence_after();
          issue_qk(j);
          retire_qk(j);
        }
      }
      for (int it = 0; it < nblk && ok; ++it) {
        // P.V of this block once its P is in TMEM (and the rows that raised their max are rescaled), then
        // Q.K^T of block it + 2 into the S buffer that P has just been read from
        const bool more_qk = it + 2 < nblk;
        // With two key stages (BF16 Q / K) the loads are only just ahead of their use, and a wait for them placed
        // before the wait for P cost more than it saved (21.98 against 23.2 ms on the mxfp8 workload): those
        // instantiations wait for P first, as the MMA thread did before.
        constexpr bool kStagesFirst = kFastStages > 2;
        if constexpr (kStagesFirst) {
          ok = ready_pv();
          // (a K stage that has not landed yet must not hold up P.V: it is only looked at here, awaited behind P.V)
          if (ok && more_qk) ok = ready_qk(false, have_k);
        }
        if (ok) ok = mbar_wait(BAR_PRDY(t, it & 1), (it >> 1) & 1, abort_flag, p.status, 35);
        if (!ok) break;
        if constexpr (!kStagesFirst) {
          ok = ready_pv();
          have_k = false;
          if (!ok) break;
        }
        tc_fence_after();
        issue_pv(it);
        // with two stages the next V^T load is already awaited: its stage goes back before the next Q.K^T, not behind it
        if constexpr (kFastStages == 2) free_v(it);
        if (more_qk && !have_k) {
          ok = ready_qk(true, have_k);
          if (!ok) break;
          tc_fence_after();
        }
        if (more_qk) issue_qk(it + 2);                 // the softmax warps wait for this one: nothing else comes first
        retire_pv(it);
        if (more_qk) retire_qk(it + 2);
      }
      if constexpr (TV) {
        if (p.elided != nullptr && n_elided != 0) atomicAdd(p.elided, n_elided);
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

template <int D, int BN, bool CORR, int PK, bool VALPHA, int QB, bool BL = false, bool TV = false>
int launch_fast_t(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const CUtensorMap& ma, const Params& p,
                  cudaStream_t st) {
  using SM = FastSmem<D, PK, QB, BL ? 1 : 0>;
  const int smem_bytes = SM::total + 1024;
  auto kern = attn_fast_kernel<D, BN, CORR, PK, VALPHA, QB, BL, TV>;
  LBFQ_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes));
  dim3 grid((p.M + kCtaM - 1) / kCtaM, p.B * p.H, 1);
  kern<<<grid, kFastThreads, smem_bytes, st>>>(mq, mk, mv, ma, p);
  return check_launch("attn_fast_kernel");
}

}  // namespace

// BLASST fills the TMEM-resident kernel produces: the constant ones that need at most the block's mean score, and
// the per-bin fill when a bin lies within one half of the block's columns
bool fast_blasst_fill(int fill_kind, int uta_bins, int block_n) {
  if (fill_kind == LBFQ_FILL_ZERO || fill_kind == LBFQ_FILL_MAX || fill_kind == LBFQ_FILL_MEAN || fill_kind == LBFQ_FILL_THR)
    return true;
  if (fill_kind != LBFQ_FILL_UTA || uta_bins < 2 || block_n % uta_bins != 0) return false;
  const int bs = block_n / uta_bins;
  return bs >= 2 && bs <= block_n / 2;
}

// 0: the general kernel; 1: TMEM-resident with e4m3 P (element-wise P, no V-smoothing term); 2: TMEM-resident with
// BF16 P (mx / dynamic P, or any P with the V-smoothing term; needs a BF16 copy of V^T, and the alpha' pieces)
int fast_variant(const Params& p, bool blasst, bool qk_mx) {
  const bool common = !qk_mx && (p.qk_bf16 != 0 || (p.q_scale != nullptr && p.k_scale != nullptr)) &&
                      (p.corr == nullptr || p.corr_staged != 0) && p.sm_scale > 0.f;
  if (!common) return 0;
  const bool v_ok = p.v_kind == LBFQ_V_CHANNEL || p.v_kind == LBFQ_V_MX;
  if (blasst) {
    // row skipping is built for the plain stacks: FP8 block scales, no score bias, no V-smoothing term
    if (p.qk_bf16 || p.corr != nullptr || p.v_alpha != nullptr || p.rm_mode != 0) return 0;
    if (!fast_blasst_fill(p.fill_kind, p.uta_bins, p.block_n)) return 0;
    if (p.p_kind == LBFQ_P_ELEMENTWISE) return p.v_kind == LBFQ_V_CHANNEL ? 1 : 0;
    return v_ok ? 2 : 0;
  }
  // a 128-key stage holds whole V-smoothing tiles: blocks of 64 keys, or of a multiple of 128
  const bool alpha_ok = p.v_alpha == nullptr || p.v_smooth_block == 64 || p.v_smooth_block % 128 == 0;
  if (p.qk_bf16) return (v_ok && alpha_ok && (p.p_kind == LBFQ_P_DYNAMIC || p.rm_mode != 2)) ? 2 : 0;
  if (p.v_alpha != nullptr) return (v_ok && alpha_ok && (p.p_kind != LBFQ_P_ELEMENTWISE || p.rm_mode != 2)) ? 2 : 0;
  if (p.p_kind == LBFQ_P_ELEMENTWISE) return (p.v_kind == LBFQ_V_CHANNEL && (p.rm_mode == 0 || p.rm_mode == 1)) ? 1 : 0;
  return v_ok ? 2 : 0;
}

int launch_fast(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const CUtensorMap& ma, const Params& p,
                int block_n, int variant, cudaStream_t st) {
  const bool va = p.v_alpha != nullptr;
  if (p.blasst) {
#define LBFQ_FAST_BL(DD, NN)                                                                                      \
  if (p.tile_vote) {                                                                                              \
    if (variant == 2) return launch_fast_t<DD, NN, false, 1, false, 0, true, true>(mq, mk, mv, ma, p, st);        \
    return launch_fast_t<DD, NN, false, 0, false, 0, true, true>(mq, mk, mv, ma, p, st);                          \
  }                                                                                                               \
  if (variant == 2) return launch_fast_t<DD, NN, false, 1, false, 0, true>(mq, mk, mv, ma, p, st);                \
  return launch_fast_t<DD, NN, false, 0, false, 0, true>(mq, mk, mv, ma, p, st)
    if (p.D == 128 && block_n == 64) { LBFQ_FAST_BL(128, 64); }
    if (p.D == 128) { LBFQ_FAST_BL(128, 32); }
    if (block_n == 64) { LBFQ_FAST_BL(64, 64); }
    LBFQ_FAST_BL(64, 32);
#undef LBFQ_FAST_BL
  }
#define LBFQ_FAST3(DD, NN, CC, VV)                                                                                \
  if (p.qk_bf16) return launch_fast_t<DD, NN, CC, 1, VV, 1>(mq, mk, mv, ma, p, st);                               \
  return launch_fast_t<DD, NN, CC, 1, VV, 0>(mq, mk, mv, ma, p, st)
#define LBFQ_FAST2(DD, NN, CC)                                                                                    \
  if (variant == 2) {                                                                                             \
    if (va) { LBFQ_FAST3(DD, NN, CC, true); }                                                                     \
    LBFQ_FAST3(DD, NN, CC, false);                                                                                \
  }                                                                                                               \
  return launch_fast_t<DD, NN, CC, 0, false, 0>(mq, mk, mv, ma, p, st)
#define LBFQ_FAST(DD, NN)                                                                                         \
  if (p.corr != nullptr) { LBFQ_FAST2(DD, NN, true); }                                                            \
  LBFQ_FAST2(DD, NN, false)
  if (p.D == 128 && block_n == 64) { LBFQ_FAST(128, 64); }
  if (p.D == 128) { LBFQ_FAST(128, 32); }
  if (block_n == 64) { LBFQ_FAST(64, 64); }
  LBFQ_FAST(64, 32);
#undef LBFQ_FAST
#undef LBFQ_FAST2
#undef LBFQ_FAST3
}

}  // namespace attn
}  // namespace lbfq
