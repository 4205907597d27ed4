// Fused kernels of the wav2vec 2.0 self-supervised objective.
//
// contrastive_*: cosine-similarity logits between every masked position and its 1 + K candidates (the true
// quantized target and K distractors given as row indices into the target matrix), temperature, -inf for
// distractors identical to the target, and cross entropy against candidate 0 -- without ever materialising the
// [positions, K, M] distractor tensor that the gather + cosine_similarity formulation needs.
//
// quantize_*: Gumbel-softmax vector quantizer. Per (frame, codebook): arg-max code, softmax probabilities for the
// perplexity statistics, straight-through hard sample of softmax((logits + noise) / tau), and the code-book LOOKUP
// of the selected entry instead of the dense [frames, G*V, 1] x [1, G*V, E] product.
//
// One warp per row; fp32 math; bf16 or fp32 activations.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cfloat>
#include <cstdint>

#include "common.cuh"
#include "wav2vec2.h"

namespace fs2 {

namespace {

constexpr int MAX_M_PER_LANE = 32;   // feature dim up to 1024

template <typename T>
__device__ __forceinline__ float to_f(T v);
template <>
__device__ __forceinline__ float to_f<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

// logits[p, c], lse[p]; loss_sum += lse - logits[p, 0]
template <typename T>
__global__ void __launch_bounds__(256) contrastive_fwd_kernel(const T* __restrict__ x, const T* __restrict__ tgt,
                                                              const int* __restrict__ distractors, int P, int K, int M,
                                                              float inv_temp, float* __restrict__ logits,
                                                              float* __restrict__ lse, float* __restrict__ loss_sum) {
    const int p = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (p >= P) return;
    float xv[MAX_M_PER_LANE], tv[MAX_M_PER_LANE];
    float xx = 0.f;
#pragma unroll
    for (int i = 0; i < MAX_M_PER_LANE; ++i) {
        const int m = lane + 32 * i;
        xv[i] = m < M ? to_f(x[static_cast<size_t>(p) * M + m]) : 0.f;
        tv[i] = m < M ? to_f(tgt[static_cast<size_t>(p) * M + m]) : 0.f;
        xx += xv[i] * xv[i];
    }
    const float xn = sqrtf(warp_sum(xx));
    float mx = -FLT_MAX, sum = 0.f, l0 = 0.f;
    for (int c = 0; c <= K; ++c) {
        const int row = c == 0 ? p : distractors[static_cast<size_t>(p) * K + c - 1];
        float dot = 0.f, cc = 0.f;
        int differs = 0;
#pragma unroll
        for (int i = 0; i < MAX_M_PER_LANE; ++i) {
            const int m = lane + 32 * i;
            if (m < M) {
                const float v = c == 0 ? tv[i] : to_f(tgt[static_cast<size_t>(row) * M + m]);
                dot += xv[i] * v;
                cc += v * v;
                differs |= (v != tv[i]);
            }
        }
        dot = warp_sum(dot);
        cc = warp_sum(cc);
        differs = __any_sync(0xffffffffu, differs);
        float lg = dot / fmaxf(xn * sqrtf(cc), 1e-8f) * inv_temp;
        if (c > 0 && !differs) lg = -INFINITY;                 // a distractor equal to the target carries no signal
        if (lane == 0) logits[static_cast<size_t>(p) * (K + 1) + c] = lg;
        if (c == 0) l0 = lg;
        if (lg > mx) {
            sum = sum * __expf(mx - lg) + 1.f;
            mx = lg;
        } else if (lg != -INFINITY) {
            sum += __expf(lg - mx);
        }
    }
    if (lane == 0) {
        const float l = mx + __logf(sum);
        lse[p] = l;
        atomicAdd(loss_sum, l - l0);
    }
}

// dx[p] and atomic dtgt[row] for loss = sum_p (lse_p - logit_p0) scaled by `scale`
template <typename T>
__global__ void __launch_bounds__(256) contrastive_bwd_kernel(const T* __restrict__ x, const T* __restrict__ tgt,
                                                              const int* __restrict__ distractors,
                                                              const float* __restrict__ logits,
                                                              const float* __restrict__ lse,
                                                              const float* __restrict__ scale_ptr, int P, int K, int M,
                                                              float inv_temp, float* __restrict__ dx,
                                                              float* __restrict__ dtgt) {
    const int p = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (p >= P) return;
    const float scale = *scale_ptr;
    float xv[MAX_M_PER_LANE], acc[MAX_M_PER_LANE];
    float xx = 0.f;
#pragma unroll
    for (int i = 0; i < MAX_M_PER_LANE; ++i) {
        const int m = lane + 32 * i;
        xv[i] = m < M ? to_f(x[static_cast<size_t>(p) * M + m]) : 0.f;
        acc[i] = 0.f;
        xx += xv[i] * xv[i];
    }
    xx = warp_sum(xx);
    const float xn = sqrtf(xx);
    const float l = lse[p];
    for (int c = 0; c <= K; ++c) {
        const float lg = logits[static_cast<size_t>(p) * (K + 1) + c];
        if (lg == -INFINITY) continue;
        const float g = (__expf(lg - l) - (c == 0 ? 1.f : 0.f)) * scale * inv_temp;   // d loss / d cos
        const int row = c == 0 ? p : distractors[static_cast<size_t>(p) * K + c - 1];
        float cv[MAX_M_PER_LANE];
        float dot = 0.f, cc = 0.f;
#pragma unroll
        for (int i = 0; i < MAX_M_PER_LANE; ++i) {
            const int m = lane + 32 * i;
            cv[i] = m < M ? to_f(tgt[static_cast<size_t>(row) * M + m]) : 0.f;
            dot += xv[i] * cv[i];
            cc += cv[i] * cv[i];
        }
        dot = warp_sum(dot);
        cc = warp_sum(cc);
        const float denom = fmaxf(xn * sqrtf(cc), 1e-8f);
        const float cosv = dot / denom;
#pragma unroll
        for (int i = 0; i < MAX_M_PER_LANE; ++i) {
            const int m = lane + 32 * i;
            if (m < M) {
                acc[i] += g * (cv[i] / denom - cosv * xv[i] / fmaxf(xx, 1e-16f));
                atomicAdd(&dtgt[static_cast<size_t>(row) * M + m],
                          g * (xv[i] / denom - cosv * cv[i] / fmaxf(cc, 1e-16f)));
            }
        }
    }
#pragma unroll
    for (int i = 0; i < MAX_M_PER_LANE; ++i) {
        const int m = lane + 32 * i;
        if (m < M) dx[static_cast<size_t>(p) * M + m] = acc[i];
    }
}

// ---------------------------------------------------------------------------------------------- quantizer
constexpr int MAX_V_PER_LANE = 16;   // up to 512 entries per codebook

// Row r = (frame, codebook). hard_idx[r] = argmax logits; prob_sum[g, v] += softmax(logits)[v];
// hard_count[g, v] += [v == hard_idx]; y = softmax((logits + noise) / tau) (noise may be null: y = softmax(logits /
// tau)); sel[r] = argmax y (training) or hard_idx (eval); q[r, :] = entries[g * V + sel[r], :]; y_soft is kept for
// the backward when `y_soft` is not null.
template <typename T>
__global__ void __launch_bounds__(256) quantize_fwd_kernel(const T* __restrict__ logits, const float* __restrict__ noise,
                                                           const T* __restrict__ entries, int R, int G, int V, int E,
                                                           float inv_tau, int training, int* __restrict__ hard_idx,
                                                           int* __restrict__ sel, float* __restrict__ prob_sum,
                                                           float* __restrict__ hard_count, float* __restrict__ y_soft,
                                                           T* __restrict__ q) {
    const int r = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (r >= R) return;
    const int g = r % G;
    float lv[MAX_V_PER_LANE];
    float mx = -FLT_MAX;
    int am = 0;
#pragma unroll
    for (int i = 0; i < MAX_V_PER_LANE; ++i) {
        const int v = lane + 32 * i;
        lv[i] = v < V ? to_f(logits[static_cast<size_t>(r) * V + v]) : -FLT_MAX;
        if (lv[i] > mx) {
            mx = lv[i];
            am = v;
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float om = __shfl_xor_sync(0xffffffffu, mx, o);
        const int oa = __shfl_xor_sync(0xffffffffu, am, o);
        if (om > mx || (om == mx && oa < am)) {
            mx = om;
            am = oa;
        }
    }
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < MAX_V_PER_LANE; ++i) s += (lane + 32 * i < V) ? __expf(lv[i] - mx) : 0.f;
    s = warp_sum(s);
#pragma unroll
    for (int i = 0; i < MAX_V_PER_LANE; ++i) {
        const int v = lane + 32 * i;
        if (v < V) atomicAdd(&prob_sum[g * V + v], __expf(lv[i] - mx) / s);
    }
    if (lane == 0) {
        hard_idx[r] = am;
        atomicAdd(&hard_count[g * V + am], 1.f);
    }
    int pick = am;
    if (training) {
        float zv[MAX_V_PER_LANE];
        float zmx = -FLT_MAX;
        int zam = 0;
#pragma unroll
        for (int i = 0; i < MAX_V_PER_LANE; ++i) {
            const int v = lane + 32 * i;
            zv[i] = v < V ? (lv[i] + (noise ? noise[static_cast<size_t>(r) * V + v] : 0.f)) * inv_tau : -FLT_MAX;
            if (zv[i] > zmx) {
                zmx = zv[i];
                zam = v;
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float om = __shfl_xor_sync(0xffffffffu, zmx, o);
            const int oa = __shfl_xor_sync(0xffffffffu, zam, o);
            if (om > zmx || (om == zmx && oa < zam)) {
                zmx = om;
                zam = oa;
            }
        }
        float zs = 0.f;
#pragma unroll
        for (int i = 0; i < MAX_V_PER_LANE; ++i) zs += (lane + 32 * i < V) ? __expf(zv[i] - zmx) : 0.f;
        zs = warp_sum(zs);
        if (y_soft) {
#pragma unroll
            for (int i = 0; i < MAX_V_PER_LANE; ++i) {
                const int v = lane + 32 * i;
                if (v < V) y_soft[static_cast<size_t>(r) * V + v] = __expf(zv[i] - zmx) / zs;
            }
        }
        pick = zam;
    }
    if (lane == 0) sel[r] = pick;
    const T* src = entries + (static_cast<size_t>(g) * V + pick) * E;
    T* dst = q + static_cast<size_t>(r) * E;
    for (int e = lane; e < E; e += 32) dst[e] = src[e];
}

// dq [R, E] -> dlogits [R, V] through the straight-through estimator: dy[v] = <dq[r], entries[g, v]>,
// dlogits = y * (dy - sum_v y dy) * inv_tau; dentries[g, sel[r]] += dq[r].
template <typename T>
__global__ void __launch_bounds__(256) quantize_bwd_kernel(const T* __restrict__ dq, const T* __restrict__ entries,
                                                           const float* __restrict__ y_soft, const int* __restrict__ sel,
                                                           int R, int G, int V, int E, float inv_tau,
                                                           float* __restrict__ dlogits, float* __restrict__ dentries) {
    const int r = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (r >= R) return;
    const int g = r % G;
    const T* dqr = dq + static_cast<size_t>(r) * E;
    float dy[MAX_V_PER_LANE], yv[MAX_V_PER_LANE];
    float inner = 0.f;
#pragma unroll
    for (int i = 0; i < MAX_V_PER_LANE; ++i) {
        const int v = lane + 32 * i;
        dy[i] = 0.f;
        yv[i] = 0.f;
        if (v < V) {
            const T* ent = entries + (static_cast<size_t>(g) * V + v) * E;
            float d = 0.f;
            for (int e = 0; e < E; ++e) d += to_f(dqr[e]) * to_f(ent[e]);
            dy[i] = d;
            yv[i] = y_soft[static_cast<size_t>(r) * V + v];
            inner += yv[i] * d;
        }
    }
    inner = warp_sum(inner);
#pragma unroll
    for (int i = 0; i < MAX_V_PER_LANE; ++i) {
        const int v = lane + 32 * i;
        if (v < V) dlogits[static_cast<size_t>(r) * V + v] = yv[i] * (dy[i] - inner) * inv_tau;
    }
    float* de = dentries + (static_cast<size_t>(g) * V + sel[r]) * E;
    for (int e = lane; e < E; e += 32) atomicAdd(&de[e], to_f(dqr[e]));
}

}  // namespace

void w2v_contrastive_fwd(const void* x, const void* tgt, bool bf16, const int* distractors, int P, int K, int M,
                         float temp, float* logits, float* lse, float* loss_sum, cudaStream_t st) {
    if (P == 0) return;
    const int blocks = (P * 32 + 255) / 256;
    if (bf16)
        contrastive_fwd_kernel<__nv_bfloat16><<<blocks, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(x),
                                                                      static_cast<const __nv_bfloat16*>(tgt),
                                                                      distractors, P, K, M, 1.f / temp, logits, lse,
                                                                      loss_sum);
    else
        contrastive_fwd_kernel<float><<<blocks, 256, 0, st>>>(static_cast<const float*>(x),
                                                              static_cast<const float*>(tgt), distractors, P, K, M,
                                                              1.f / temp, logits, lse, loss_sum);
}

void w2v_contrastive_bwd(const void* x, const void* tgt, bool bf16, const int* distractors, const float* logits,
                         const float* lse, const float* scale, int P, int K, int M, float temp, float* dx, float* dtgt,
                         cudaStream_t st) {
    if (P == 0) return;
    const int blocks = (P * 32 + 255) / 256;
    if (bf16)
        contrastive_bwd_kernel<__nv_bfloat16><<<blocks, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(x),
                                                                      static_cast<const __nv_bfloat16*>(tgt),
                                                                      distractors, logits, lse, scale, P, K, M,
                                                                      1.f / temp, dx, dtgt);
    else
        contrastive_bwd_kernel<float><<<blocks, 256, 0, st>>>(static_cast<const float*>(x),
                                                              static_cast<const float*>(tgt), distractors, logits, lse,
                                                              scale, P, K, M, 1.f / temp, dx, dtgt);
}

void w2v_quantize_fwd(const void* logits, const float* noise, const void* entries, bool bf16, int R, int G, int V, int E,
                      float tau, bool training, int* hard_idx, int* sel, float* prob_sum, float* hard_count,
                      float* y_soft, void* q, cudaStream_t st) {
    if (R == 0) return;
    const int blocks = (R * 32 + 255) / 256;
    if (bf16)
        quantize_fwd_kernel<__nv_bfloat16><<<blocks, 256, 0, st>>>(
            static_cast<const __nv_bfloat16*>(logits), noise, static_cast<const __nv_bfloat16*>(entries), R, G, V, E,
            1.f / tau, training ? 1 : 0, hard_idx, sel, prob_sum, hard_count, y_soft, static_cast<__nv_bfloat16*>(q));
    else
        quantize_fwd_kernel<float><<<blocks, 256, 0, st>>>(static_cast<const float*>(logits), noise,
                                                           static_cast<const float*>(entries), R, G, V, E, 1.f / tau,
                                                           training ? 1 : 0, hard_idx, sel, prob_sum, hard_count, y_soft,
                                                           static_cast<float*>(q));
}

void w2v_quantize_bwd(const void* dq, const void* entries, bool bf16, const float* y_soft, const int* sel, int R, int G,
                      int V, int E, float tau, float* dlogits, float* dentries, cudaStream_t st) {
    if (R == 0) return;
    const int blocks = (R * 32 + 255) / 256;
    if (bf16)
        quantize_bwd_kernel<__nv_bfloat16><<<blocks, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(dq),
                                                                   static_cast<const __nv_bfloat16*>(entries), y_soft,
                                                                   sel, R, G, V, E, 1.f / tau, dlogits, dentries);
    else
        quantize_bwd_kernel<float><<<blocks, 256, 0, st>>>(static_cast<const float*>(dq),
                                                           static_cast<const float*>(entries), y_soft, sel, R, G, V, E,
                                                           1.f / tau, dlogits, dentries);
}

}  // namespace fs2
