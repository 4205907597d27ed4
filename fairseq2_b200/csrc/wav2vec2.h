// Host launchers of the fused wav2vec 2.0 objective kernels (wav2vec2.cu).
#pragma once

#include <cuda_runtime.h>

namespace fs2 {

// x, tgt: [P, M] (bf16 or fp32, M <= 1024); distractors: [P, K] rows of tgt. logits [P, K + 1] =
// cos(x[p], candidate) / temp with candidate 0 = tgt[p]; distractors equal to the target get -inf.
// lse[p] = logsumexp(logits[p]); *loss_sum += sum_p lse[p] - logits[p, 0].
void w2v_contrastive_fwd(const void* x, const void* tgt, bool bf16, const int* distractors, int P, int K, int M,
                         float temp, float* logits, float* lse, float* loss_sum, cudaStream_t st);

// Gradient of `*scale * loss_sum`: dx [P, M] is written, dtgt [P, M] (fp32, zeroed by the caller) is accumulated.
void w2v_contrastive_bwd(const void* x, const void* tgt, bool bf16, const int* distractors, const float* logits,
                         const float* lse, const float* scale, int P, int K, int M, float temp, float* dx, float* dtgt,
                         cudaStream_t st);

// logits [R, V] with R = frames * G rows ordered (frame, codebook), V <= 512; entries [G * V, E]; noise [R, V] fp32
// Gumbel noise or null. Outputs: hard_idx [R] (argmax), sel [R] (sampled code when training, else argmax),
// prob_sum / hard_count [G, V] (accumulated; zeroed by the caller), y_soft [R, V] or null, q [R, E] = entries[sel].
void w2v_quantize_fwd(const void* logits, const float* noise, const void* entries, bool bf16, int R, int G, int V, int E,
                      float tau, bool training, int* hard_idx, int* sel, float* prob_sum, float* hard_count,
                      float* y_soft, void* q, cudaStream_t st);

// Straight-through backward: dlogits [R, V] fp32 (written), dentries [G * V, E] fp32 (accumulated).
void w2v_quantize_bwd(const void* dq, const void* entries, bool bf16, const float* y_soft, const int* sel, int R, int G,
                      int V, int E, float tau, float* dlogits, float* dentries, cudaStream_t st);

// First layer of the wav2vec 2.0 feature extractor (one input channel, kernel width 10): x [B, L] bf16 waveform,
// w [C, 10], optional bias / LayerNorm weight and bias [C] -> y [B, t_pad, C] bf16 channels-last =
// GELU(LayerNorm(conv + bias)) (bare conv + bias without LayerNorm); rows t >= t_valid are zero. The backward
// recomputes the row from the waveform and accumulates into zero-initialised fp32 dw [C, 10], dbias, dlnw, dlnb [C].
bool w2v_first_conv_supported(int C, int kernel_width);
void w2v_first_conv_fwd(const void* x, const void* w, const void* bias, const void* lnw, const void* lnb, void* y, int B,
                        int L, int t_valid, int t_pad, int C, int stride, float eps, int num_sms, cudaStream_t st);
void w2v_first_conv_bwd(const void* x, const void* w, const void* bias, const void* lnw, const void* lnb, const void* dy,
                        float* dw, float* dbias, float* dlnw, float* dlnb, int B, int L, int t_valid, int t_pad, int C,
                        int stride, float eps, int num_sms, cudaStream_t st);

}  // namespace fs2
