// Score bias of the Q-smoothing correction on the tensor cores (qm_corr_tc.cu), called from preprocess.cu.
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

namespace lbfq {
bool qm_corr_tc_eligible(int dtype, int D, int S, const void* k_smooth);
// qm: fp32 (B, G, H, D); k_smooth: (B, S, H, D) bf16; corr: fp32 (B*H, G, s_pad); rowmax: fp32 (B*H, G) holding -inf,
// or NULL; status: device word raised when a bounded wait expires, or NULL
int qm_corr_tc(const float* qm, const void* k_smooth, int B, int S, int H, int D, int G, float sm_scale, float* corr,
               int s_pad, float* rowmax, int32_t* status, cudaStream_t st);
}  // namespace lbfq
