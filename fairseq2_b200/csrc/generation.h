// Host launchers of the generation-step kernels in generation.cu.
#pragma once

#include <cuda_runtime.h>

#include <cstdint>

namespace fs2 {

// Bans, per row, every token that would complete an n-gram already present in `seqs`.
void ngram_repeat_block(const long long* seqs, float* probs, int batch, int seq_len, int vocab, int n,
                        float ban_value, cudaStream_t st);

// One sampled index per row from the top-k / nucleus-filtered distribution.
void sample_top_p_top_k(const float* probs, const float* uniform, long long* out, int batch, int vocab, float p,
                        int k, cudaStream_t st);

// Fused beam-search step: scores[b, j*V + v] = beam_score[b, j] + lprobs[b*beams + j, v]; top `k` per batch row.
void beam_topk(const float* lprobs, const float* beam_scores, float* out_scores, long long* out_idx, int batch,
               int beams, int vocab, int k, cudaStream_t st);

}  // namespace fs2
