// Parameters and host entry points of the varlen GQA attention kernels.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstddef>

namespace fs2 {

struct AttnParams {
    // [tokens, heads, D] views; *_tstride is the token stride in elements, heads are D apart.
    const __nv_bfloat16* q;
    const __nv_bfloat16* k;
    const __nv_bfloat16* v;
    __nv_bfloat16* o;
    const __nv_bfloat16* dout;
    __nv_bfloat16* dq;
    __nv_bfloat16* dk;
    __nv_bfloat16* dv;
    float* lse;    // [H, total_q]
    float* delta;  // [H, total_q]
    size_t q_tstride, k_tstride, v_tstride, o_tstride, do_tstride, dq_tstride, dk_tstride, dv_tstride;
    const int* q_begins;
    const int* q_lens;
    const int* k_begins;
    const int* k_lens;
    int num_seqs, total_q, total_k, max_q, max_k;
    int H, Hkv, D;
    int causal;
    int window;    // > 0 (causal only): query i sees keys j with i + shift - window < j <= i + shift; 0 = no limit
    float scale;
    // Dropout on the attention probabilities (mma.sync kernels only): an element (head, query token, key token) is
    // kept iff hash(seed, head, q, k) >= drop_threshold, and kept elements are scaled by keep_scale = 1 / (1 - p).
    // drop_threshold = 0 switches dropout off.
    unsigned int drop_threshold;
    float keep_scale;
    unsigned long long seed;
};

// Return nullptr on success, else a static error string.
const char* attn_forward(const AttnParams& p, cudaStream_t st);
const char* attn_backward(const AttnParams& p, cudaStream_t st);

// tcgen05/TMEM path (head_dim 128); `status` is the host-mapped status word for bounded waits.
const char* attn_forward_tc(const AttnParams& p, int* status, cudaStream_t st);
const char* attn_backward_tc(const AttnParams& p, int* status, cudaStream_t st);

// delta[h, t] = sum_d dO[t, h, d] * O[t, h, d] (first step of both backward paths)
const char* attn_delta(const AttnParams& p, cudaStream_t st);

}  // namespace fs2
