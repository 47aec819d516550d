// k-means assignment on the tensor cores (kmeans_tc.cu), called from kmeans.cu.
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

namespace lbfq {
bool kmeans_tc_eligible(int dtype, int D, int k);
size_t kmeans_tc_split_bytes(int BH, int D);
// tokens per assignment CTA: the granularity of the per-chunk label counts
int kmeans_tc_chunk_tokens();
// x: (B, S, H, D) bf16; cent (B*H, k, D) fp32; cnorm (B*H, k) fp32; split: kmeans_tc_split_bytes scratch;
// hist: (B*H, chunks, 64) int32 per-chunk label counts, or NULL (chunks = ceil(S / chunk_tokens), or
// kmeans_tc_sum_chunks when psum is given); status: device word raised when
// a bounded wait expires (the labels of that call are then incomplete), or NULL.
// psum: (B*H, ceil(S / chunk_tokens), k, D) fp32 per-chunk sums of the tokens of every cluster, or NULL (needs
// kmeans_tc_sums_eligible and hist)
bool kmeans_tc_sums_eligible(int dtype, int D, int k);
// chunks per (b, h) slab of the per-chunk counts and sums when psum is given (the kernel picks its tiles per CTA from
// the problem size and the GPU), and the largest value that can take for a sequence length (scratch sizing)
int kmeans_tc_sum_chunks(int BH, int S);
int kmeans_tc_sum_chunks_max(int S);
// split_current: the BF16 pieces in `split` already match `cent` (kmeans_tc_update_from_sums wrote both)
int kmeans_tc_assign(const void* x, int B, int S, int H, int D, int k, const float* cent, const float* cnorm,
                     void* split, int32_t* labels, int32_t* hist, float* psum, bool split_current, int32_t* status,
                     cudaStream_t st);
// centroids, their norms and their BF16 pieces from the per-chunk sums and counts of the last kmeans_tc_assign with
// psum: chunks added in a fixed order; an empty cluster keeps what it had
int kmeans_tc_update_from_sums(const float* psum, const int32_t* hist, int BH, int S, int D, int k, float* cent,
                               float* cnorm, void* split, cudaStream_t st);
}  // namespace lbfq
