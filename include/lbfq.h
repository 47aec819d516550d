/*
 * lbfq.h -- C ABI of the B200 (sm_100a) fake-quant attention library.
 *
 * Every entry point is `extern "C"`, takes plain device pointers, sizes and a
 * CUDA stream (as `void*`, i.e. a `cudaStream_t`), returns 0 on success or a
 * negative LBFQ_ERR_* code, never throws and never allocates device memory:
 * the caller owns inputs, outputs and any workspace. After a non-zero return
 * `lbfq_last_error()` holds a message for the calling thread.
 *
 * Each declaration names the function of the reference project
 * (DongyunZou/low-bit-attention-fake-quant, paths relative to its root) whose
 * device work it replaces.
 *
 * Tensor conventions
 *   NHD  : (B, S, H, D) contiguous -- the reference's public layout.
 *   BHSD : (B, H, S_pad, D) contiguous, S_pad >= S; rows S..S_pad-1 are
 *          written as zero codes by the quantizers.
 *   BHDS : (B, H, D, S_pad) contiguous (token index fastest) -- the layout the
 *          attention kernel wants for V.
 *   D is 64 or 128. Codes are e4m3 ("fn": no inf, max 448) bytes.
 */
#ifndef LBFQ_H_
#define LBFQ_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- status codes ------------------------------------------------------- */
#define LBFQ_OK 0
#define LBFQ_ERR_ARG (-1)         /* bad shape / divisibility / mode (ValueError in the host mirror) */
#define LBFQ_ERR_DTYPE (-2)       /* unsupported element type (TypeError) */
#define LBFQ_ERR_UNSUPPORTED (-3) /* valid in the reference, not built here yet */
#define LBFQ_ERR_CUDA (-4)        /* a CUDA runtime / driver call failed */
#define LBFQ_ERR_DEVICE (-5)      /* a kernel reported a bounded-wait timeout */

/* ---- element types of floating-point tensors ----------------------------- */
#define LBFQ_F32 0
#define LBFQ_F16 1
#define LBFQ_BF16 2

/* ---- layouts of code tensors written by the quantizers ------------------- */
#define LBFQ_LAYOUT_NHD 0
#define LBFQ_LAYOUT_BHSD 1
#define LBFQ_LAYOUT_BHDS 2

const char* lbfq_last_error(void);
/* ABI version of this header; bumped when a signature or a struct layout changes.
 * 2: lbfq_attn_args gained `rowmax_counters` (appended); lbfq_fp8_block_quant_centered added; lbfq_smooth_k takes
 *    out = NULL.
 * 3: lbfq_kmeans_labels and lbfq_qm_corr take a `status` word (bounded waits of their tensor-core kernels report
 *    there); lbfq_get_flags / lbfq_set_flags replace per-call reads of the LBFQ_* environment variables.
 * 4: lbfq_attn_args gained `blasst_tile_predicate` and `blasst_elided` behind `blasst_stats`. */
int lbfq_abi_version(void);

/* Debug overrides. They are read from the environment (LBFQ_ATTN_GENERIC=1, LBFQ_KMEANS_FFMA=1,
 * LBFQ_QM_CORR_FFMA=1, LBFQ_UNFUSED_PREPROCESS=1, LBFQ_KMEANS_SORTED=1) once, when the library is first used; afterwards they change only
 * through lbfq_set_flags(). Each keeps a slower cross-check path in use: the general attention kernel, the FP32 FFMA
 * k-means assignment, the FP32 FFMA qm.K product, the one-kernel-per-step preprocessing, the k-means centroid update by
 * sort + segment means. Process-wide, not per thread. */
#define LBFQ_FLAG_ATTN_GENERIC 1
#define LBFQ_FLAG_KMEANS_FFMA 2
#define LBFQ_FLAG_QM_CORR_FFMA 4
#define LBFQ_FLAG_UNFUSED_PREPROCESS 8
#define LBFQ_FLAG_KMEANS_SORTED 16
int lbfq_get_flags(void);
void lbfq_set_flags(int flags);
/* Number of kernels this library has launched in the calling process (a plain counter,
 * not thread-safe; used by the benchmark to report its launch count). */
unsigned long long lbfq_launch_count(void);

/* ======================= quantizers (quant_triton.py) ===================== */

/* fp8_block_quant, src/low_bit_fake_quant/quant_triton.py:26-77.
 * x: NHD of `dtype`. scale: fp32 (B, S/block_s, H). codes: `layout`, with
 * `s_pad` rows per (b,h) when layout != NHD. */
int lbfq_fp8_block_quant(const void* x, int dtype, int B, int S, int H, int D, int block_s,
                         uint8_t* codes, int layout, int s_pad, float* scale, void* stream);
/* The same quantizer applied to round_dtype(x - mean[b, h, :]), mean fp32 (B, H, D): smooth_k
 * (src/low_bit_fake_quant/preprocess.py:10-57) followed by fp8_block_quant without storing the smoothed tensor;
 * codes and scales are those of the two-step sequence, bit for bit. */
int lbfq_fp8_block_quant_centered(const void* x, int dtype, int B, int S, int H, int D, int block_s,
                                  const float* mean, uint8_t* codes, int layout, int s_pad, float* scale,
                                  void* stream);

/* fp8_block_dequant, quant_triton.py:80-131. codes NHD -> out NHD of out_dtype. */
int lbfq_fp8_block_dequant(const uint8_t* codes, const float* scale, int B, int S, int H, int D,
                           int block_s, void* out, int out_dtype, void* stream);

/* fp8_per_channel_quant, quant_triton.py:134-176. scale: fp32 (B, H, D). */
int lbfq_fp8_channel_quant(const void* x, int dtype, int B, int S, int H, int D,
                           uint8_t* codes, int layout, int s_pad, float* scale, void* stream);

/* fp8_per_channel_dequant, quant_triton.py:179-218. */
int lbfq_fp8_channel_dequant(const uint8_t* codes, const float* scale, int B, int S, int H, int D,
                             void* out, int out_dtype, void* stream);

/* mxfp8_qk_quant, quant_triton.py:221-271. scale: fp32 (B, S, H, D/block_d)
 * holding 2**e. If `scale_e8` is non-null (needs s_pad % 128 == 0, D/block_d <= 4)
 * it also receives the biased exponents e+127 as bytes for the block-scaled MMA:
 * (B, H, s_pad/128, 512), each 512-byte tile holding 128 tokens x 4 groups at
 * byte (t % 32) * 16 + (t / 32) * 4 + g; unused bytes are 127 (scale 1). */
int lbfq_mxfp8_qk_quant(const void* x, int dtype, int B, int S, int H, int D, int block_d,
                        uint8_t* codes, int layout, int s_pad, float* scale, uint8_t* scale_e8,
                        void* stream);

/* mxfp8_qk_dequant, quant_triton.py:274-319. */
int lbfq_mxfp8_qk_dequant(const uint8_t* codes, const float* scale, int B, int S, int H, int D,
                          int block_d, void* out, int out_dtype, void* stream);

/* mxfp8_v_quant, quant_triton.py:322-369 (blocks run along S). scale: fp32
 * (B, S/block_s, H, D). */
int lbfq_mxfp8_v_quant(const void* x, int dtype, int B, int S, int H, int D, int block_s,
                       uint8_t* codes, int layout, int s_pad, float* scale, void* stream);

/* mxfp8_v_dequant, quant_triton.py:372-416. */
int lbfq_mxfp8_v_dequant(const uint8_t* codes, const float* scale, int B, int S, int H, int D,
                         int block_s, void* out, int out_dtype, void* stream);

/* ============ fused preprocessing: gather + smooth + rotate + quantise ===== */

/* Quantizer of a fused call */
#define LBFQ_PREP_FP8_BLOCK 0     /* fp8_block_quant: one FP32 scale per (b, scale_block rows, h) */
#define LBFQ_PREP_FP8_CHANNEL 1   /* fp8_per_channel_quant: one FP32 scale per (b, h, d); runs two passes */
#define LBFQ_PREP_MXFP8_V 2       /* mxfp8_v_quant: power-of-two scale per (b, scale_block rows, h, d) */
#define LBFQ_PREP_MXFP8_QK 3      /* mxfp8_qk_quant: power-of-two scale per (b, s, h, scale_block channels) */

/* One of Q, K, V prepared for the attention kernel in a single pass over the tensor. Replaces, for that tensor, the
 * chain of src/low_bit_fake_quant/attention.py:166-239,505-591: the k-means gather (kmeans.py:89-90,126-135), K / Q / V
 * smoothing (preprocess.py:10-193), apply_qk_hadamard (hadamard.py:77-117), a quantizer of quant_triton.py and the
 * NHD -> BHSD copy, applied in that order with the reference's intermediate roundings into the input dtype. Codes,
 * scales and means equal those of the separate entry points above and below, bit for bit. */
typedef struct lbfq_prep_args {
  const void* x;              /* NHD (B, S, H, D) of dtype */
  int dtype;
  int B, S, H, D;
  const int64_t* order;       /* (B*H, S): source row of each output row (a k-means order), or NULL */
  const float* chan_mean;     /* (B, H, D): subtracted from every row (the K mean of lbfq_smooth_k), or NULL */
  int smooth_block;           /* > 0: subtract the column mean of every smooth_block output rows (Q groups, V blocks) */
  float* block_mean;          /* (B, S/smooth_block, H, D) fp32 receiving those means (qm / v_alpha), or NULL */
  int hadamard;               /* 1: rotate every row (after the smoothing) */
  const int8_t* signs;        /* (H, D) of +-1 on the device for this call's heads, or NULL */
  float had_scale;            /* 1 / sqrt(D) */
  int kind;                   /* LBFQ_PREP_* */
  int scale_block;            /* rows per scale (FP8_BLOCK, MXFP8_V) or channels per scale (MXFP8_QK) */
  uint8_t* codes;             /* `layout` with s_pad rows per (b, h) when layout != NHD */
  int layout;
  int s_pad;
  float* scale;               /* shape of the corresponding quantizer's scale tensor */
  uint8_t* scale_e8;          /* MXFP8_QK only: UE8M0 tiles as lbfq_mxfp8_qk_quant writes them, or NULL */
  void* smooth_out;           /* NHD of dtype receiving the re-ordered, smoothed rows as they are before the rotation, or NULL */
} lbfq_prep_args;

/* Rows one CTA of lbfq_prep_fused would take for these block sizes, or 0 when no group fits shared memory (the
 * caller then uses the separate entry points). */
int lbfq_prep_group_rows(int kind, int smooth_block, int scale_block, int S, int D, int dtype);
int lbfq_prep_fused(const lbfq_prep_args* args, void* stream);

/* ================= smoothing / rotation (preprocess.py, hadamard.py) ====== */

/* smooth_k, src/low_bit_fake_quant/preprocess.py:10-57. k, out: NHD of dtype;
 * mean: fp32 (B, H, D). `partial` is caller scratch of
 * lbfq_smooth_k_scratch_floats(B,S,H,D) floats. `out` may be NULL: the mean alone is computed
 * (for lbfq_fp8_block_quant_centered). */
int64_t lbfq_smooth_k_scratch_floats(int B, int S, int H, int D);
int lbfq_smooth_k(const void* k, int dtype, int B, int S, int H, int D, void* out, float* mean,
                  float* partial, void* stream);

/* smooth_k without caller scratch. No counterpart in the reference: it exists for
 * hosts that can pass inputs and outputs but cannot allocate device memory for the
 * library (a plugin inside another framework's memory pool, an allocation-free
 * region). Same result as
 * lbfq_smooth_k; the partial sums live in a 4 MiB array built into the library
 * (resident on every GPU that loads it, until the process exits). Limits and rules:
 *  - B*H*ceil(S/256)*D must be <= lbfq_smooth_k_static_max_floats() (1,048,576);
 *    larger shapes are refused with LBFQ_ERR_ARG;
 *  - the first call on each device looks up the array's device address (with that
 *    device current);
 *  - all calls on a device share the one array: calls that may overlap on the GPU
 *    (different streams) race; serialise them. Nothing needs clearing between calls;
 *  - the looked-up address is kept per device ordinal for the life of the process: after
 *    cudaDeviceReset() in the same process it is stale, so do not reset a device this
 *    entry has been used on. Concurrent first calls from several threads are harmless
 *    (they look up the same address);
 *  - it calls no cudaMalloc / cudaFree / allocating library routine. */
int64_t lbfq_smooth_k_static_max_floats(void);
int lbfq_smooth_k_static(const void* k, int dtype, int B, int S, int H, int D, void* out, float* mean,
                         void* stream);

/* group_mean_q (preprocess.py:60-91,169-193) and smooth_v_per_block
 * (preprocess.py:94-166): subtract the column mean of each `block`-row group.
 * mean: fp32 (B, S/block, H, D). */
int lbfq_block_mean_sub(const void* x, int dtype, int B, int S, int H, int D, int block,
                        void* out, float* mean, void* stream);

/* apply_qk_hadamard / hadamard_transform_last_dim,
 * src/low_bit_fake_quant/hadamard.py:25-117: out = FWHT_D(x * sign[h]) * scale,
 * rounded once into dtype. signs: int8 (H, D) of +-1 on the device, or NULL. */
int lbfq_hadamard(const void* x, int dtype, int64_t rows, int H, int D, const int8_t* signs,
                  float scale, void* out, void* stream);

/* ======================= k-means reorder (kmeans.py) ====================== */

/* Lloyd iterations replacing flash_kmeans.batch_kmeans_Euclid as called from
 * src/low_bit_fake_quant/kmeans.py:77-81. x: NHD of dtype. labels: int32
 * (B*H, S). The centroid seeding hashes the slab index of the unsharded problem,
 * b * total_heads + head_offset + h, so a heads shard reproduces the full run
 * (total_heads <= 0 means "not sharded"). scratch: lbfq_kmeans_scratch_bytes(...) bytes.
 * status: device int (may be NULL) that the tensor-core assignment sets non-zero when one of its bounded waits
 * expires; the labels of such a call are valid cluster indices but not a k-means result. */
int64_t lbfq_kmeans_scratch_bytes(int B, int S, int H, int D, int k);
int lbfq_kmeans_labels(const void* x, int dtype, int B, int S, int H, int D, int k, int iters,
                       int seed, int head_offset, int total_heads, int32_t* labels, void* scratch,
                       int32_t* status, void* stream);

/* kmeans.py:84-88: order = stable argsort(labels), inverse[order[j]] = j.
 * labels int32 (BH, S), values in [0, k); order / inverse int64 (BH, S). */
int lbfq_label_order(const int32_t* labels, int BH, int S, int k, int64_t* order,
                     int64_t* inverse, void* stream);

/* kmeans.py:89-90 and apply_kv_permutation (kmeans.py:126-135):
 * out[b, j, h, :] = x[b, index[b*H+h, j], h, :], NHD -> NHD of the same dtype. */
int lbfq_gather_rows(const void* x, int dtype, int B, int S, int H, int D, const int64_t* index,
                     void* out, void* stream);

/* ================== qm . K_smooth correction (attention.py) =============== */

/* The per-key bias of the Q-smoothing correction (attention_triton.py:156-160)
 * and its row max (_estimate_rowmax_from_qm_k, attention.py:366-395):
 *   corr[b,h,g,n]   = (sum_d qm[b,g,h,d] * k_smooth[b,n,h,d]) * sm_scale   (fp32)
 *   rowmax[b,h,g]   = max_n corr[b,h,g,n]
 * qm: fp32 (B, G, H, D); k_smooth: NHD of dtype; corr: fp32 (B, H, G, s_pad),
 * columns >= S zero-filled; rowmax: fp32 (B, H, G), may be NULL. status: device int (may be NULL), set non-zero
 * when a bounded wait of the tensor-core kernel expires. */
int lbfq_qm_corr(const float* qm, const void* k_smooth, int dtype, int B, int S, int H, int D, int G,
                 float sm_scale, float* corr, int s_pad, float* rowmax, int32_t* status, void* stream);

/* ========================= streaming attention ============================ */

/* P quantisation modes (attention_triton.py:78) */
#define LBFQ_P_ELEMENTWISE 0
#define LBFQ_P_MX 1
#define LBFQ_P_DYNAMIC 2
/* V quantisation kinds */
#define LBFQ_V_CHANNEL 0
#define LBFQ_V_BLOCK 1
#define LBFQ_V_MX 2
/* Q/K quantisation kinds */
#define LBFQ_QK_FP8_BLOCK 0
#define LBFQ_QK_MX 1
/* Q, K and V^T are BF16 tensors holding the de-quantised (Q, K) / code-valued or de-quantised (V) operands the
 * reference's own launcher receives (attention_triton.py:410-436): q_codes, k_codes, v_codes then point to BF16 data
 * of the same shapes, Q.K^T and P.V run as BF16 MMAs, and q_scale / k_scale are not read. */
#define LBFQ_QK_BF16 2
/* Q and K are BF16 tensors as above, V^T stays e4m3 codes with its v_kind / v_scale (the reference's launcher is given
 * V as "FP8 cast to BF16", attention_triton.py:440-446: the values are e4m3 codes, so nothing is lost). Served by the
 * general kernel: Q.K^T a BF16 MMA, P.V an FP8 MMA with every scale applied in FP32 around it -- the route for the
 * per-block V scale (v_block_scale_bsh) and for BLASST through the reference's direct-launch signature. */
#define LBFQ_QK_BF16_V_CODES 3
/* BLASST fill kinds (attention_triton.py:39-45) */
#define LBFQ_FILL_ZERO 0
#define LBFQ_FILL_MAX 1
#define LBFQ_FILL_MEAN 2
#define LBFQ_FILL_LOGN 3
#define LBFQ_FILL_SAMPLE8 4
#define LBFQ_FILL_THR 5
#define LBFQ_FILL_UTA 6

/* Operands of one launch of the streaming kernel that replaces
 * `_fake_quant_attn_fwd_kernel` / `fake_quant_attention_triton`
 * (src/low_bit_fake_quant/attention_triton.py:48-671). Field names follow the
 * reference kernel's arguments. All pointers are device pointers; optional
 * ones are NULL when the feature is off. */
typedef struct lbfq_attn_args {
  int B, H, M, N, D;          /* M query rows, N keys per (b,h) */
  int m_pad, n_pad;           /* allocated rows of q_codes / k_codes,v_codes per (b,h); multiples of 128 */
  /* fp8 operands */
  const uint8_t* q_codes;     /* BHSD (B,H,m_pad,D) */
  const uint8_t* k_codes;     /* BHSD (B,H,n_pad,D) */
  const uint8_t* v_codes;     /* BHDS (B,H,D,n_pad) */
  /* Q/K scales */
  int qk_kind;                /* LBFQ_QK_* */
  const float* q_scale;       /* fp8_block: (B, M/qk_block, H) */
  const float* k_scale;       /* fp8_block: (B, N/qk_block, H) */
  int qk_block;               /* fp8_block_size */
  const uint8_t* q_scale_e8;  /* mx: (B,H,m_pad/128,512) biased exponents, tile order of lbfq_mxfp8_qk_quant */
  const uint8_t* k_scale_e8;  /* mx: (B,H,n_pad/128,512) */
  /* V scales */
  int v_kind;                 /* LBFQ_V_* */
  const float* v_scale;       /* channel: (B,H,D); block: (B, N/v_block, H); mx: (B, N/v_block, H, D) */
  int v_block;                /* v_fp8_block_size or v_mxfp8_block_size */
  /* softmax */
  float sm_scale;
  float p_max_offset;
  int p_kind;                 /* LBFQ_P_* */
  int block_m, block_n;       /* p_requant_block_m / _n of the reference launch */
  /* V smoothing correction (attention_triton.py:378-383) */
  const float* v_alpha;       /* (B, N/v_smooth_block, H, D) or NULL */
  int v_smooth_block;
  /* Q smoothing correction: per-key bias precomputed by lbfq_qm_corr */
  const float* qm_corr;       /* (B,H,G,corr_stride) or NULL */
  int q_smooth_block;
  int corr_stride;
  /* row-max modes */
  const float* rowmax_est;    /* (B,H,M) or NULL (attention_triton.py:126-129) */
  const float* rowmax_init;   /* (B,H,M) or NULL (attention_triton.py:130-133) */
  /* BLASST */
  int use_blasst;
  float blasst_lambda;
  int fill_kind;
  float fill_alpha;
  int uta_bins;
  float* blasst_stats;        /* (ceil(M/block_m), B*H, 2) fp32, zero-initialised by the caller, or NULL */
  /* 0: every row decides for itself (the reference kernel, attention_triton.py:165-175). 1: a key block is dropped
   * only when EVERY row of the 128-row tile finds it under the threshold, and then no row of the tile sees it (the
   * tile-level predicate of the reference's simulator, blasst_skip.py:573-585); zero fill only, online row max
   * without rowmax_init (so the first key block of a tile is always kept and the simulator's empty-tile rescue,
   * blasst_skip.py:586-595, has nothing to do). */
  int blasst_tile_predicate;
  /* Optional device counter, zero-initialised by the caller, or NULL: (128-row tile, key block) pairs whose
   * exponentials, P and P.V were not computed because every row of the tile skipped the block with zero fill. */
  unsigned long long* blasst_elided;
  /* output */
  void* out;                  /* rows written through out_row_index when given */
  int out_dtype;              /* LBFQ_BF16 / LBFQ_F16 / LBFQ_F32 (kernel rounds to BF16 first unless F32 debug) */
  int out_layout;             /* LBFQ_LAYOUT_NHD (B,M,H,D) or LBFQ_LAYOUT_BHSD (B,H,M,D) */
  const int64_t* out_row_index; /* (B*H, M): destination row of kernel row r (inverse Q reorder fused), or NULL */
  int out_fp32_exact;         /* 1: store the FP32 accumulator result without the BF16 rounding */
  int32_t* status;            /* device int: set non-zero if a bounded wait expired */
  /* Optional diagnostic (bench/count_rowmax_updates_triton.py:27-171 counts the same events in a kernel of its
   * own): six device counters, zero-initialised by the caller, or NULL. [0] row-max updates, [1] accumulator
   * rescales (updates of a row that already holds mass), [2] upward updates, [3] downward updates (estimated row
   * max only), [4] rows with at least one update, [5] largest number of updates of one row. Requests the general
   * kernel. */
  long long* rowmax_counters;
} lbfq_attn_args;

/* Bytes of caller-provided scratch the launch below needs (0 when V smoothing is off). */
int64_t lbfq_attention_workspace_bytes(const lbfq_attn_args* args);

/* Replaces the launch in fake_quant_attention_triton (attention_triton.py:626-668).
 * `workspace` holds lbfq_attention_workspace_bytes(args) bytes (may be NULL when that is 0). */
int lbfq_attention_fwd(const lbfq_attn_args* args, void* workspace, void* stream);

/* Which kernel the calling thread's last lbfq_attention_fwd launched: 0 = the general kernel (P.V folded in
 * registers per key block: fp8_block V, the logn / sample8 fills, BLASST combined with a score bias or a
 * V-smoothing term, the row-max counters), 1 = the kernel whose output accumulator stays in tensor memory (every P
 * mode, per-channel and mxfp8 V, FP8-block, mxfp8 or BF16 Q / K, score bias, V-smoothing term, the constant and
 * per-bin BLASST fills). LBFQ_FLAG_ATTN_GENERIC keeps every configuration on the general kernel. No counterpart in
 * the reference. */
int lbfq_attention_last_variant(void);

/* ============================ test utility ================================= */

/* y[i] = rcp.approx.f32(x[i]) on the device. The reference's Triton kernels divide by multiplying with the GPU's
 * approximate reciprocal (quant_triton.py:49,155; attention_triton.py:357,387), and so do the kernels here; the value
 * comes from a hardware table, so a CPU restatement that wants to follow the quantizers bit for bit asks the GPU for
 * it through this entry. No counterpart in the reference. */
int lbfq_rcp_approx(const float* x, float* y, long long n, void* stream);

/* ======================= host-buffer plumbing ============================== */

/* `rows` rows of `width` bytes between a pitched host buffer and a pitched device buffer, enqueued on `stream`
 * (to_device != 0: host -> device). Used by the host-buffer entry of the Python mirror to move a heads slice
 * (B, S, h0:h1, D) of an (B, S, H, D) host tensor without a staging copy. No counterpart in the reference,
 * whose callers hold their tensors on the device. */
int lbfq_copy_rows_async(void* dst, size_t dst_pitch, const void* src, size_t src_pitch, size_t width, size_t rows,
                         int to_device, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* LBFQ_H_ */
