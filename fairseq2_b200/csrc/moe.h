// Host launchers of the mixture-of-experts routing kernels (moe.cu).
#pragma once

#include <cuda_runtime.h>

namespace fs2 {

// Per token: top-k of `logits` [T, E] (bf16 or fp32), gate = sigmoid(logit) or softmax over the selected k;
// writes expert ids [T, k], gates [T, k] (fp32), adds 1 to counts[e] per selection and, if `prob_sum` is given,
// the full-softmax probability of every expert into prob_sum[e] (for load-balancing losses).
void moe_route(const void* logits, bool bf16, int T, int E, int k, bool softmax_gate, int* expert_ids, float* gates,
               int* counts, float* prob_sum, cudaStream_t st);

// offsets[e] = exclusive prefix sum of counts; cursor[e] = 0. One block.
void moe_offsets(const int* counts, int* offsets, int* cursor, int E, cudaStream_t st);

// Dispatch: row (t, j) goes to slot p = offsets[e] + (arrival order within e); out[p, :] = x[t, :] * gate,
// src_row[p] = t, inv[t*k + j] = p. bf16 rows of D elements (D % 8 == 0).
void moe_dispatch(const void* x, const int* expert_ids, const float* gates, const int* offsets, int* cursor,
                  void* out, int* src_row, int* inv, int T, int k, int D, bool scale_by_gate, cudaStream_t st);

// Combine: y[t, :] (+)= sum over the slots p with src_row[p] == t of routed[p, :] (* gate[p] if given); implemented
// as a gather per token through inv[t, j] = p. bf16 in/out, fp32 accumulation.
void moe_combine(const void* routed, const int* inv, const float* slot_gates, void* y, int T, int k, int D,
                 bool accumulate, cudaStream_t st);

}  // namespace fs2
