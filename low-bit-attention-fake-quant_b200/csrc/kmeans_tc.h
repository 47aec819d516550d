// k-means assignment on the tensor cores (kmeans_tc.cu), called from kmeans.cu.
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

namespace lbfq {
bool kmeans_tc_eligible(int dtype, int D, int k);
size_t kmeans_tc_split_bytes(int BH, int D);
// x: (B, S, H, D) bf16; cent (B*H, k, D) fp32; cnorm (B*H, k) fp32; split: kmeans_tc_split_bytes scratch
int kmeans_tc_assign(const void* x, int B, int S, int H, int D, int k, const float* cent, const float* cnorm,
                     void* split, int32_t* labels, cudaStream_t st);
}  // namespace lbfq
