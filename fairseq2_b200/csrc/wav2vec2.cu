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


// ------------------------------------------------- first feature-extractor layer (1 input channel)
// y[b, t, :] = GELU(LayerNorm_c(conv1d(x[b, :], w, stride)[t, :] + bias)) written channels-last, or the bare
// convolution + bias when the layer has no LayerNorm. With one input channel the layer is bound by writing its
// output (C values per KW input samples), so everything between the waveform and the first channels-last
// activation happens in registers: one warp per output position, lane l owns channels [(v * 32 + l) * 8, +8) for
// v < NV; the weights sit transposed ([tap][channel], fp32) in shared memory. Rows t >= t_valid (padding that makes
// later strides divide) are written as zeros.
__device__ __forceinline__ float gelu_f(float u) { return 0.5f * u * (1.f + erff(u * 0.70710678118654752f)); }
__device__ __forceinline__ float gelu_grad_f(float u) {
    return 0.5f * (1.f + erff(u * 0.70710678118654752f)) + u * 0.3989422804014327f * __expf(-0.5f * u * u);
}

template <int NV, int KW>
__device__ __forceinline__ void first_conv_row(const float* __restrict__ sw, const float* xk, int C, int lane,
                                               float (*z)[8]) {
#pragma unroll
    for (int v = 0; v < NV; ++v) {
        const int c0 = (v * 32 + lane) * 8;
#pragma unroll
        for (int e = 0; e < 8; ++e) z[v][e] = 0.f;
        if (c0 < C) {
#pragma unroll
            for (int k = 0; k < KW; ++k) {
                const float4 a = *reinterpret_cast<const float4*>(sw + k * C + c0);
                const float4 b = *reinterpret_cast<const float4*>(sw + k * C + c0 + 4);
                z[v][0] += xk[k] * a.x; z[v][1] += xk[k] * a.y; z[v][2] += xk[k] * a.z; z[v][3] += xk[k] * a.w;
                z[v][4] += xk[k] * b.x; z[v][5] += xk[k] * b.y; z[v][6] += xk[k] * b.z; z[v][7] += xk[k] * b.w;
            }
        }
    }
}

template <int NV, int KW>
__global__ void __launch_bounds__(256) first_conv_fwd_kernel(const __nv_bfloat16* __restrict__ x,
                                                             const __nv_bfloat16* __restrict__ w,
                                                             const __nv_bfloat16* __restrict__ bias,
                                                             const __nv_bfloat16* __restrict__ lnw,
                                                             const __nv_bfloat16* __restrict__ lnb,
                                                             __nv_bfloat16* __restrict__ y, int B, int L, int t_valid,
                                                             int t_pad, int C, int stride, float eps) {
    extern __shared__ float sw[];                        // [KW][C]
    for (int i = threadIdx.x; i < C * KW; i += blockDim.x) sw[(i % KW) * C + i / KW] = __bfloat162float(w[i]);
    __syncthreads();
    const int lane = threadIdx.x & 31;
    const long long warp = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
    const long long nwarps = (gridDim.x * static_cast<long long>(blockDim.x)) >> 5;
    float bv[NV][8], gw[NV][8], gb[NV][8];
#pragma unroll
    for (int v = 0; v < NV; ++v) {
        const int c0 = (v * 32 + lane) * 8;
#pragma unroll
        for (int e = 0; e < 8; ++e) bv[v][e] = gb[v][e] = 0.f, gw[v][e] = 1.f;
        if (c0 < C) {
            if (bias) load8(bias, c0, bv[v]);
            if (lnw) load8(lnw, c0, gw[v]);
            if (lnb) load8(lnb, c0, gb[v]);
        }
    }
    const long long total = static_cast<long long>(B) * t_pad;
    for (long long pos = warp; pos < total; pos += nwarps) {
        const int b = static_cast<int>(pos / t_pad), t = static_cast<int>(pos % t_pad);
        __nv_bfloat16* out = y + pos * C;
        float z[NV][8];
        if (t >= t_valid) {
#pragma unroll
            for (int v = 0; v < NV; ++v) {
                const int c0 = (v * 32 + lane) * 8;
#pragma unroll
                for (int e = 0; e < 8; ++e) z[v][e] = 0.f;
                if (c0 < C) store8(out, c0, z[v]);
            }
            continue;
        }
        const float mine = lane < KW ? __bfloat162float(x[static_cast<long long>(b) * L + static_cast<long long>(t) * stride + lane]) : 0.f;
        float xk[KW];
#pragma unroll
        for (int k = 0; k < KW; ++k) xk[k] = __shfl_sync(0xffffffffu, mine, k);
        first_conv_row<NV, KW>(sw, xk, C, lane, z);
        float sum = 0.f;
#pragma unroll
        for (int v = 0; v < NV; ++v)
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                z[v][e] += bv[v][e];
                sum += z[v][e];                           // lanes without channels hold zeros
            }
        if (lnw != nullptr) {
            const float mean = warp_sum(sum) / C;
            float var = 0.f;
#pragma unroll
            for (int v = 0; v < NV; ++v)
                if ((v * 32 + lane) * 8 < C)
#pragma unroll
                    for (int e = 0; e < 8; ++e) var += (z[v][e] - mean) * (z[v][e] - mean);
            const float rstd = rsqrtf(warp_sum(var) / C + eps);
#pragma unroll
            for (int v = 0; v < NV; ++v)
#pragma unroll
                for (int e = 0; e < 8; ++e) z[v][e] = gelu_f((z[v][e] - mean) * rstd * gw[v][e] + gb[v][e]);
        }
#pragma unroll
        for (int v = 0; v < NV; ++v) {
            const int c0 = (v * 32 + lane) * 8;
            if (c0 < C) store8(out, c0, z[v]);
        }
    }
}

// Backward of the above for channel slot blockIdx.y (the 256 channels whose gradients this pass accumulates): the
// row is recomputed from the waveform, so the forward pass saves nothing but its inputs. Accumulators per lane:
// dW [8][KW], dbias, dlnw, dlnb [8]; they are summed over the block in shared memory and added to the fp32 outputs.
template <int NV, int KW>
__global__ void __launch_bounds__(256) first_conv_bwd_kernel(const __nv_bfloat16* __restrict__ x,
                                                             const __nv_bfloat16* __restrict__ w,
                                                             const __nv_bfloat16* __restrict__ bias,
                                                             const __nv_bfloat16* __restrict__ lnw,
                                                             const __nv_bfloat16* __restrict__ lnb,
                                                             const __nv_bfloat16* __restrict__ dy,
                                                             float* __restrict__ dw, float* __restrict__ dbias,
                                                             float* __restrict__ dlnw, float* __restrict__ dlnb, int B,
                                                             int L, int t_valid, int t_pad, int C, int stride,
                                                             float eps) {
    extern __shared__ float sw[];                        // [KW][C] weights, then [(KW + 3)][256] block sums
    float* sacc = sw + KW * C;
    for (int i = threadIdx.x; i < C * KW; i += blockDim.x) sw[(i % KW) * C + i / KW] = __bfloat162float(w[i]);
    for (int i = threadIdx.x; i < (KW + 3) * 256; i += blockDim.x) sacc[i] = 0.f;
    __syncthreads();
    const int lane = threadIdx.x & 31;
    const int slot = blockIdx.y;
    const long long warp = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
    const long long nwarps = (gridDim.x * static_cast<long long>(blockDim.x)) >> 5;
    float bv[NV][8], gw[NV][8], gb[NV][8];
#pragma unroll
    for (int v = 0; v < NV; ++v) {
        const int c0 = (v * 32 + lane) * 8;
#pragma unroll
        for (int e = 0; e < 8; ++e) bv[v][e] = gb[v][e] = 0.f, gw[v][e] = 1.f;
        if (c0 < C) {
            if (bias) load8(bias, c0, bv[v]);
            if (lnw) load8(lnw, c0, gw[v]);
            if (lnb) load8(lnb, c0, gb[v]);
        }
    }
    float a_dw[8][KW], a_db[8], a_gw[8], a_gb[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) {
        a_db[e] = a_gw[e] = a_gb[e] = 0.f;
#pragma unroll
        for (int k = 0; k < KW; ++k) a_dw[e][k] = 0.f;
    }
    const long long total = static_cast<long long>(B) * t_pad;
    for (long long pos = warp; pos < total; pos += nwarps) {
        const int b = static_cast<int>(pos / t_pad), t = static_cast<int>(pos % t_pad);
        if (t >= t_valid) continue;
        const float mine = lane < KW ? __bfloat162float(x[static_cast<long long>(b) * L + static_cast<long long>(t) * stride + lane]) : 0.f;
        float xk[KW];
#pragma unroll
        for (int k = 0; k < KW; ++k) xk[k] = __shfl_sync(0xffffffffu, mine, k);
        float z[NV][8], g[NV][8];
        first_conv_row<NV, KW>(sw, xk, C, lane, z);
#pragma unroll
        for (int v = 0; v < NV; ++v) {
            const int c0 = (v * 32 + lane) * 8;
#pragma unroll
            for (int e = 0; e < 8; ++e) g[v][e] = 0.f;
            if (c0 < C) load8(dy + pos * C, c0, g[v]);
        }
        float dzs[8], xhs[8], gs[8];                     // this slot's dz, xhat and dLN-output
        if (lnw != nullptr) {
            float sum = 0.f;
#pragma unroll
            for (int v = 0; v < NV; ++v)
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    z[v][e] += bv[v][e];
                    sum += z[v][e];
                }
            const float mean = warp_sum(sum) / C;
            float var = 0.f;
#pragma unroll
            for (int v = 0; v < NV; ++v)
                if ((v * 32 + lane) * 8 < C)
#pragma unroll
                    for (int e = 0; e < 8; ++e) var += (z[v][e] - mean) * (z[v][e] - mean);
            const float rstd = rsqrtf(warp_sum(var) / C + eps);
            float s1 = 0.f, s2 = 0.f;
#pragma unroll
            for (int v = 0; v < NV; ++v)
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    const float xh = (z[v][e] - mean) * rstd;
                    const float go = g[v][e] * gelu_grad_f(xh * gw[v][e] + gb[v][e]);   // grad of the LN output
                    z[v][e] = xh;
                    g[v][e] = go;
                    s1 += go * gw[v][e];
                    s2 += go * gw[v][e] * xh;
                }
            s1 = warp_sum(s1) / C;
            s2 = warp_sum(s2) / C;
#pragma unroll
            for (int v = 0; v < NV; ++v)
                if (v == slot)
#pragma unroll
                    for (int e = 0; e < 8; ++e) {
                        xhs[e] = z[v][e];
                        gs[e] = g[v][e];
                        dzs[e] = rstd * (g[v][e] * gw[v][e] - s1 - z[v][e] * s2);
                    }
        } else {
#pragma unroll
            for (int v = 0; v < NV; ++v)
                if (v == slot)
#pragma unroll
                    for (int e = 0; e < 8; ++e) {
                        xhs[e] = 0.f;
                        gs[e] = 0.f;
                        dzs[e] = g[v][e];
                    }
        }
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            a_db[e] += dzs[e];
            a_gw[e] += gs[e] * xhs[e];
            a_gb[e] += gs[e];
#pragma unroll
            for (int k = 0; k < KW; ++k) a_dw[e][k] += dzs[e] * xk[k];
        }
    }
    // block sums in shared memory (lane l, element e -> column l * 8 + e of the slot), then one atomic per value
#pragma unroll
    for (int e = 0; e < 8; ++e) {
        const int col = lane * 8 + e;
#pragma unroll
        for (int k = 0; k < KW; ++k) atomicAdd(sacc + k * 256 + col, a_dw[e][k]);
        atomicAdd(sacc + KW * 256 + col, a_db[e]);
        atomicAdd(sacc + (KW + 1) * 256 + col, a_gw[e]);
        atomicAdd(sacc + (KW + 2) * 256 + col, a_gb[e]);
    }
    __syncthreads();
    for (int i = threadIdx.x; i < 256; i += blockDim.x) {
        const int c = slot * 256 + i;
        if (c >= C) continue;
#pragma unroll
        for (int k = 0; k < KW; ++k) atomicAdd(dw + c * KW + k, sacc[k * 256 + i]);
        if (dbias) atomicAdd(dbias + c, sacc[KW * 256 + i]);
        if (dlnw) atomicAdd(dlnw + c, sacc[(KW + 1) * 256 + i]);
        if (dlnb) atomicAdd(dlnb + c, sacc[(KW + 2) * 256 + i]);
    }
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


namespace {

template <int NV>
void first_conv_fwd_nv(const void* x, const void* w, const void* bias, const void* lnw, const void* lnb, void* y, int B,
                       int L, int t_valid, int t_pad, int C, int stride, float eps, int num_sms, cudaStream_t st) {
    constexpr int KW = 10;
    const size_t smem = static_cast<size_t>(KW) * C * sizeof(float);
    auto kernel = first_conv_fwd_kernel<NV, KW>;
    cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    kernel<<<num_sms * 2, 256, smem, st>>>(static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(w),
                                           static_cast<const __nv_bfloat16*>(bias),
                                           static_cast<const __nv_bfloat16*>(lnw),
                                           static_cast<const __nv_bfloat16*>(lnb), static_cast<__nv_bfloat16*>(y), B, L,
                                           t_valid, t_pad, C, stride, eps);
}

template <int NV>
void first_conv_bwd_nv(const void* x, const void* w, const void* bias, const void* lnw, const void* lnb, const void* dy,
                       float* dw, float* dbias, float* dlnw, float* dlnb, int B, int L, int t_valid, int t_pad, int C,
                       int stride, float eps, int num_sms, cudaStream_t st) {
    constexpr int KW = 10;
    const size_t smem = (static_cast<size_t>(KW) * C + (KW + 3) * 256) * sizeof(float);
    auto kernel = first_conv_bwd_kernel<NV, KW>;
    cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    dim3 grid(num_sms, NV);
    kernel<<<grid, 256, smem, st>>>(static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(w),
                                    static_cast<const __nv_bfloat16*>(bias), static_cast<const __nv_bfloat16*>(lnw),
                                    static_cast<const __nv_bfloat16*>(lnb), static_cast<const __nv_bfloat16*>(dy), dw,
                                    dbias, dlnw, dlnb, B, L, t_valid, t_pad, C, stride, eps);
}

}  // namespace

bool w2v_first_conv_supported(int C, int kernel_width) { return kernel_width == 10 && C % 8 == 0 && C >= 8 && C <= 1024; }

void w2v_first_conv_fwd(const void* x, const void* w, const void* bias, const void* lnw, const void* lnb, void* y, int B,
                        int L, int t_valid, int t_pad, int C, int stride, float eps, int num_sms, cudaStream_t st) {
    const int nv = (C / 8 + 31) / 32;
    if (nv == 1) first_conv_fwd_nv<1>(x, w, bias, lnw, lnb, y, B, L, t_valid, t_pad, C, stride, eps, num_sms, st);
    else if (nv == 2) first_conv_fwd_nv<2>(x, w, bias, lnw, lnb, y, B, L, t_valid, t_pad, C, stride, eps, num_sms, st);
    else if (nv == 3) first_conv_fwd_nv<3>(x, w, bias, lnw, lnb, y, B, L, t_valid, t_pad, C, stride, eps, num_sms, st);
    else first_conv_fwd_nv<4>(x, w, bias, lnw, lnb, y, B, L, t_valid, t_pad, C, stride, eps, num_sms, st);
}

void w2v_first_conv_bwd(const void* x, const void* w, const void* bias, const void* lnw, const void* lnb, const void* dy,
                        float* dw, float* dbias, float* dlnw, float* dlnb, int B, int L, int t_valid, int t_pad, int C,
                        int stride, float eps, int num_sms, cudaStream_t st) {
    const int nv = (C / 8 + 31) / 32;
    if (nv == 1) first_conv_bwd_nv<1>(x, w, bias, lnw, lnb, dy, dw, dbias, dlnw, dlnb, B, L, t_valid, t_pad, C, stride, eps, num_sms, st);
    else if (nv == 2) first_conv_bwd_nv<2>(x, w, bias, lnw, lnb, dy, dw, dbias, dlnw, dlnb, B, L, t_valid, t_pad, C, stride, eps, num_sms, st);
    else if (nv == 3) first_conv_bwd_nv<3>(x, w, bias, lnw, lnb, dy, dw, dbias, dlnw, dlnb, B, L, t_valid, t_pad, C, stride, eps, num_sms, st);
    else first_conv_bwd_nv<4>(x, w, bias, lnw, lnb, dy, dw, dbias, dlnw, dlnb, B, L, t_valid, t_pad, C, stride, eps, num_sms, st);
}

}  // namespace fs2
