// Mixture-of-experts routing kernels: fused top-k gate, expert histogram, dispatch (gather + scale into
// expert-sorted order) and combine (gather back per token). One warp handles one token row.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cfloat>
#include <cstdint>

#include "common.cuh"
#include "moe.h"

namespace fs2 {

namespace {

constexpr int MAX_E_PER_LANE = 8;    // up to 256 experts
constexpr int MAX_K = 8;

template <typename T>
__global__ void __launch_bounds__(256) moe_route_kernel(const T* __restrict__ logits, int T_, int E, int k,
                                                        int softmax_gate, int* __restrict__ expert_ids,
                                                        float* __restrict__ gates, int* __restrict__ counts,
                                                        float* __restrict__ prob_sum) {
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (warp >= T_) return;
    const T* row = logits + static_cast<size_t>(warp) * E;
    float v[MAX_E_PER_LANE];
#pragma unroll
    for (int i = 0; i < MAX_E_PER_LANE; ++i) {
        const int e = lane + 32 * i;
        float x = -FLT_MAX;
        if (e < E) {
            if constexpr (sizeof(T) == 2) x = __bfloat162float(row[e]);
            else x = row[e];
        }
        v[i] = x;
    }
    if (prob_sum != nullptr) {
        float mx = -FLT_MAX;
#pragma unroll
        for (int i = 0; i < MAX_E_PER_LANE; ++i) mx = fmaxf(mx, v[i]);
        mx = warp_max(mx);
        float ex[MAX_E_PER_LANE], s = 0.f;
#pragma unroll
        for (int i = 0; i < MAX_E_PER_LANE; ++i) {
            ex[i] = (lane + 32 * i < E) ? __expf(v[i] - mx) : 0.f;
            s += ex[i];
        }
        s = warp_sum(s);
#pragma unroll
        for (int i = 0; i < MAX_E_PER_LANE; ++i)
            if (lane + 32 * i < E) atomicAdd(&prob_sum[lane + 32 * i], ex[i] / s);
    }
    float top_v[MAX_K];
    int top_e[MAX_K];
    for (int j = 0; j < k; ++j) {
        // arg-max over the warp; ties go to the smaller expert index (as torch.topk does for equal values in order)
        float bv = -FLT_MAX;
        int be = E;
#pragma unroll
        for (int i = 0; i < MAX_E_PER_LANE; ++i) {
            const int e = lane + 32 * i;
            if (e < E && (v[i] > bv || (v[i] == bv && e < be))) {
                bv = v[i];
                be = e;
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int oe = __shfl_xor_sync(0xffffffffu, be, o);
            if (ov > bv || (ov == bv && oe < be)) {
                bv = ov;
                be = oe;
            }
        }
        top_v[j] = bv;
        top_e[j] = be;
        if ((be & 31) == lane) v[be >> 5] = -FLT_MAX;     // remove the winner
    }
    if (lane == 0) {
        float denom = 1.f, mx = top_v[0];
        if (softmax_gate) {
            denom = 0.f;
            for (int j = 0; j < k; ++j) denom += __expf(top_v[j] - mx);
        }
        for (int j = 0; j < k; ++j) {
            expert_ids[static_cast<size_t>(warp) * k + j] = top_e[j];
            gates[static_cast<size_t>(warp) * k + j] =
                softmax_gate ? __expf(top_v[j] - mx) / denom : 1.f / (1.f + __expf(-top_v[j]));
            atomicAdd(&counts[top_e[j]], 1);
        }
    }
}

__global__ void moe_offsets_kernel(const int* __restrict__ counts, int* __restrict__ offsets, int* __restrict__ cursor,
                                   int E) {
    if (threadIdx.x == 0) {
        int acc = 0;
        for (int e = 0; e < E; ++e) {
            offsets[e] = acc;
            acc += counts[e];
            cursor[e] = 0;
        }
        offsets[E] = acc;
    }
}

__global__ void __launch_bounds__(256) moe_dispatch_kernel(const __nv_bfloat16* __restrict__ x,
                                                           const int* __restrict__ expert_ids,
                                                           const float* __restrict__ gates,
                                                           const int* __restrict__ offsets, int* __restrict__ cursor,
                                                           __nv_bfloat16* __restrict__ out, int* __restrict__ src_row,
                                                           int* __restrict__ inv, int rows, int k, int D,
                                                           int scale_by_gate) {
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;     // one warp per (token, choice)
    const int lane = threadIdx.x & 31;
    if (warp >= rows) return;
    const int t = warp / k;
    int slot = 0;
    if (lane == 0) {
        const int e = expert_ids[warp];
        slot = offsets[e] + atomicAdd(&cursor[e], 1);
        src_row[slot] = t;
        inv[warp] = slot;
    }
    slot = __shfl_sync(0xffffffffu, slot, 0);
    const float g = scale_by_gate ? gates[warp] : 1.f;
    const __nv_bfloat16* src = x + static_cast<size_t>(t) * D;
    __nv_bfloat16* dst = out + static_cast<size_t>(slot) * D;
    for (int c = lane * 8; c < D; c += 256) {
        float f[8];
        load8(src, c, f);
        if (scale_by_gate) {
#pragma unroll
            for (int i = 0; i < 8; ++i) f[i] *= g;
        }
        store8(dst, c, f);
    }
}

__global__ void __launch_bounds__(256) moe_combine_kernel(const __nv_bfloat16* __restrict__ routed,
                                                          const int* __restrict__ inv,
                                                          const float* __restrict__ slot_gates,
                                                          __nv_bfloat16* __restrict__ y, int T_, int k, int D,
                                                          int accumulate) {
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;     // one warp per token
    const int lane = threadIdx.x & 31;
    if (warp >= T_) return;
    __nv_bfloat16* dst = y + static_cast<size_t>(warp) * D;
    for (int c = lane * 8; c < D; c += 256) {
        float acc[8];
        if (accumulate) load8(dst, c, acc);
        else {
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[i] = 0.f;
        }
        for (int j = 0; j < k; ++j) {
            const int slot = inv[warp * k + j];
            const float g = slot_gates ? slot_gates[warp * k + j] : 1.f;
            float f[8];
            load8(routed + static_cast<size_t>(slot) * D, c, f);
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[i] += g * f[i];
        }
        store8(dst, c, acc);
    }
}

}  // namespace

void moe_route(const void* logits, bool bf16, int T, int E, int k, bool softmax_gate, int* expert_ids, float* gates,
               int* counts, float* prob_sum, cudaStream_t st) {
    if (T == 0) return;
    const int blocks = (T * 32 + 255) / 256;
    if (bf16)
        moe_route_kernel<__nv_bfloat16><<<blocks, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(logits), T, E, k,
                                                                softmax_gate ? 1 : 0, expert_ids, gates, counts,
                                                                prob_sum);
    else
        moe_route_kernel<float><<<blocks, 256, 0, st>>>(static_cast<const float*>(logits), T, E, k,
                                                        softmax_gate ? 1 : 0, expert_ids, gates, counts, prob_sum);
}

void moe_offsets(const int* counts, int* offsets, int* cursor, int E, cudaStream_t st) {
    moe_offsets_kernel<<<1, 32, 0, st>>>(counts, offsets, cursor, E);
}

void moe_dispatch(const void* x, const int* expert_ids, const float* gates, const int* offsets, int* cursor, void* out,
                  int* src_row, int* inv, int T, int k, int D, bool scale_by_gate, cudaStream_t st) {
    const int rows = T * k;
    if (rows == 0) return;
    const int blocks = (rows * 32 + 255) / 256;
    moe_dispatch_kernel<<<blocks, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(x), expert_ids, gates, offsets, cursor,
                                                static_cast<__nv_bfloat16*>(out), src_row, inv, rows, k, D,
                                                scale_by_gate ? 1 : 0);
}

void moe_combine(const void* routed, const int* inv, const float* slot_gates, void* y, int T, int k, int D,
                 bool accumulate, cudaStream_t st) {
    if (T == 0) return;
    const int blocks = (T * 32 + 255) / 256;
    moe_combine_kernel<<<blocks, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(routed), inv, slot_gates,
                                               static_cast<__nv_bfloat16*>(y), T, k, D, accumulate ? 1 : 0);
}

}  // namespace fs2
