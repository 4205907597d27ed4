// Bandwidth-bound kernels: RMSNorm / LayerNorm (fwd + bwd), SwiGLU, rotary
// encoding, masked cross-entropy (loss + in-place logit gradient), AdamW,
// L2 norm and scaling. All use 16-byte vector accesses and fp32 arithmetic.

#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdint>

#include "common.cuh"
#include "elementwise.h"

namespace fs2 {

namespace {

constexpr int MAX_VPT = 8;  // upper bound on vectors of 8 elements cached per thread

// Threads per row of the forward kernels. From 1024 elements on, every thread owns two 16-byte vectors of the row: with
// one vector per thread a full SM has only 32 KB of loads in flight, too few to cover the memory latency at full
// bandwidth (8192 x 4096 bf16: 0.042 -> 0.037 ms). The backward kernels, which hold two cached rows and the weight
// gradient partials in registers, are faster with one vector per thread (0.089 ms against 0.117 ms) and prefetch
// the next row instead (0.075 ms).
inline int norm_block_bwd(int D) {
    int nvec = D / 8;
    int threads = ((nvec + 31) / 32) * 32;
    if (threads > 1024) threads = 1024;
    if (threads < 32) threads = 32;
    return threads;
}

inline int norm_block(int D) {
    int nvec = D / 8;
    int threads = nvec >= 128 ? (((nvec + 1) / 2 + 31) / 32) * 32 : ((nvec + 31) / 32) * 32;
    if (threads > 1024) threads = 1024;
    if (threads < 32) threads = 32;
    return threads;
}

// ------------------------------------------------------------------- RMSNorm
// With `res` the kernel is residual add + norm in one pass: h = x + res (rounded to the activation dtype, as a
// separate add would) is written to `sum_out` and normalised, so the sum is never re-read from memory.
template <typename T, int VPT>
__global__ void rms_norm_fwd_kernel(const T* __restrict__ x, const T* __restrict__ w, T* __restrict__ y,
                                    float* __restrict__ rstd, int rows, int D, float eps,
                                    const T* __restrict__ res, T* __restrict__ sum_out) {
    __shared__ float scratch[32];
    const int nvec = D / 8;
    for (int row = blockIdx.x; row < rows; row += gridDim.x) {
        const T* xr = x + static_cast<size_t>(row) * D;
        T* yr = y + static_cast<size_t>(row) * D;
        float cache[VPT][8];
        float ss = 0.f;
#pragma unroll
        for (int j = 0; j < VPT; ++j) {
            const int v = threadIdx.x + j * blockDim.x;
            if (v < nvec) {
                load8(xr, static_cast<size_t>(v) * 8, cache[j]);
                if (res != nullptr) {
                    float rv[8];
                    load8(res + static_cast<size_t>(row) * D, static_cast<size_t>(v) * 8, rv);
#pragma unroll
                    for (int e = 0; e < 8; ++e) {
                        float h = cache[j][e] + rv[e];
                        if constexpr (sizeof(T) == 2) h = __bfloat162float(__float2bfloat16_rn(h));
                        cache[j][e] = h;
                    }
                    store8(sum_out + static_cast<size_t>(row) * D, static_cast<size_t>(v) * 8, cache[j]);
                }
#pragma unroll
                for (int e = 0; e < 8; ++e) ss += cache[j][e] * cache[j][e];
            }
        }
        ss = block_sum(ss, scratch);
        const float r = rsqrtf(ss / D + eps);
        if (threadIdx.x == 0) rstd[row] = r;
#pragma unroll
        for (int j = 0; j < VPT; ++j) {
            const int v = threadIdx.x + j * blockDim.x;
            if (v < nvec) {
                float wv[8], o[8];
                load8(w, static_cast<size_t>(v) * 8, wv);
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    // match the reference: normalise in fp32, round to the
                    // activation dtype, then scale by the weight
                    float n = cache[j][e] * r;
                    if constexpr (sizeof(T) == 2) n = __bfloat162float(__float2bfloat16_rn(n));
                    o[e] = n * wv[e];
                }
                store8(yr, static_cast<size_t>(v) * 8, o);
            }
        }
    }
}

// Eight consecutive elements as they sit in memory (16 bytes of bf16, 32 of fp32): what a prefetch keeps in registers
// until the row is processed.
template <typename T>
struct Raw8;

template <>
struct Raw8<__nv_bfloat16> {
    bf16x8 v;
    __device__ __forceinline__ void load(const __nv_bfloat16* p, size_t i) { v = *reinterpret_cast<const bf16x8*>(p + i); }
    __device__ __forceinline__ void unpack(float* f) const { unpack8(v, f); }
};

template <>
struct Raw8<float> {
    float4 a, b;
    __device__ __forceinline__ void load(const float* p, size_t i) {
        a = *reinterpret_cast<const float4*>(p + i);
        b = *reinterpret_cast<const float4*>(p + i + 4);
    }
    __device__ __forceinline__ void unpack(float* f) const {
        f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w;
        f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
    }
};

// dx = rstd * (g - xhat * mean(g * xhat)), g = dy * w, xhat = x * rstd
// dw partial per block: sum over its rows of dy * xhat
// `dres` (may be null): a gradient that reaches x by another path (the residual connection); it is added to dx in
// the same pass, which is the backward of the fused residual add + norm.
template <typename T, int VPT>
__global__ void __launch_bounds__(1024) rms_norm_bwd_kernel(const T* __restrict__ dy, const T* __restrict__ x, const T* __restrict__ w,
                                    const float* __restrict__ rstd, T* __restrict__ dx, float* __restrict__ dw_part,
                                    int rows, int D, const T* __restrict__ dres) {
    __shared__ float scratch[32];
    const int nvec = D / 8;
    float dwacc[VPT][8];
    float wv[VPT][8];
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
        const int v = threadIdx.x + j * blockDim.x;
#pragma unroll
        for (int e = 0; e < 8; ++e) dwacc[j][e] = 0.f;
        if (v < nvec) load8(w, static_cast<size_t>(v) * 8, wv[j]);
    }
    // The loads of the next row are issued before this row's reduction, so that twice as many bytes are in flight
    // (with the 48 registers of this kernel only two 512-thread blocks fit on an SM).
    Raw8<T> ndy[VPT], nx[VPT];
    float nr = 0.f;
    auto fetch = [&](int row) {
        const size_t off = static_cast<size_t>(row) * D;
        nr = rstd[row];
#pragma unroll
        for (int j = 0; j < VPT; ++j) {
            const int v = threadIdx.x + j * blockDim.x;
            if (v < nvec) {
                ndy[j].load(dy + off, static_cast<size_t>(v) * 8);
                nx[j].load(x + off, static_cast<size_t>(v) * 8);
            }
        }
    };
    if (static_cast<int>(blockIdx.x) < rows) fetch(blockIdx.x);
    for (int row = blockIdx.x; row < rows; row += gridDim.x) {
        const size_t off = static_cast<size_t>(row) * D;
        const float r = nr;
        float g[VPT][8], xh[VPT][8];
        float dot = 0.f;
#pragma unroll
        for (int j = 0; j < VPT; ++j) {
            const int v = threadIdx.x + j * blockDim.x;
            if (v < nvec) {
                float dyv[8], xv[8];
                ndy[j].unpack(dyv);
                nx[j].unpack(xv);
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    xh[j][e] = xv[e] * r;
                    g[j][e] = dyv[e] * wv[j][e];
                    dot += g[j][e] * xh[j][e];
                    dwacc[j][e] += dyv[e] * xh[j][e];
                }
            }
        }
        if (row + static_cast<int>(gridDim.x) < rows) fetch(row + gridDim.x);
        dot = block_sum(dot, scratch);
        const float m = dot / D;
#pragma unroll
        for (int j = 0; j < VPT; ++j) {
            const int v = threadIdx.x + j * blockDim.x;
            if (v < nvec) {
                float o[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) o[e] = r * (g[j][e] - xh[j][e] * m);
                if (dres != nullptr) {
                    float dr[8];
                    load8(dres + off, static_cast<size_t>(v) * 8, dr);
#pragma unroll
                    for (int e = 0; e < 8; ++e) o[e] += dr[e];
                }
                store8(dx + off, static_cast<size_t>(v) * 8, o);
            }
        }
    }
    float* part = dw_part + static_cast<size_t>(blockIdx.x) * D;
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
        const int v = threadIdx.x + j * blockDim.x;
        if (v < nvec) store8(part, static_cast<size_t>(v) * 8, dwacc[j]);
    }
}

// out[d] = sum_p part[p, d]
__global__ void reduce_partials_kernel(const float* __restrict__ part, float* __restrict__ out, int P, int D) {
    const int d = blockIdx.x * blockDim.x + threadIdx.x;
    if (d >= D) return;
    float s = 0.f;
    for (int p = 0; p < P; ++p) s += part[static_cast<size_t>(p) * D + d];
    out[d] = s;
}

// ----------------------------------------------------------------- LayerNorm
__device__ __forceinline__ float gelu_exact(float n) { return 0.5f * n * (1.f + erff(n * 0.70710678118654752f)); }

__device__ __forceinline__ float gelu_exact_grad(float n) {
    return 0.5f * (1.f + erff(n * 0.70710678118654752f)) + n * 0.39894228040143268f * __expf(-0.5f * n * n);
}

// GELU = true applies the exact (erf) GELU to the normalised row in the same pass: the convolutional feature
// encoders of speech models are conv -> LayerNorm over channels -> GELU on channels-last rows.
template <typename T, int VPT, bool GELU = false>
__global__ void layer_norm_fwd_kernel(const T* __restrict__ x, const T* __restrict__ w, const T* __restrict__ b,
                                      T* __restrict__ y, float* __restrict__ mean, float* __restrict__ rstd, int rows,
                                      int D, float eps) {
    __shared__ float scratch[32];
    const int nvec = D / 8;
    for (int row = blockIdx.x; row < rows; row += gridDim.x) {
        const size_t off = static_cast<size_t>(row) * D;
        float cache[VPT][8];
        float s = 0.f;
#pragma unroll
        for (int j = 0; j < VPT; ++j) {
            const int v = threadIdx.x + j * blockDim.x;
            if (v < nvec) {
                load8(x + off, static_cast<size_t>(v) * 8, cache[j]);
#pragma unroll
                for (int e = 0; e < 8; ++e) s += cache[j][e];
            }
        }
        const float mu = block_sum(s, scratch) / D;
        float ss = 0.f;
#pragma unroll
        for (int j = 0; j < VPT; ++j) {
            const int v = threadIdx.x + j * blockDim.x;
            if (v < nvec) {
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    const float d = cache[j][e] - mu;
                    ss += d * d;
                }
            }
        }
        const float r = rsqrtf(block_sum(ss, scratch) / D + eps);
        if (threadIdx.x == 0) {
            mean[row] = mu;
            rstd[row] = r;
        }
#pragma unroll
        for (int j = 0; j < VPT; ++j) {
            const int v = threadIdx.x + j * blockDim.x;
            if (v < nvec) {
                float wv[8], bv[8], o[8];
                load8(w, static_cast<size_t>(v) * 8, wv);
                load8(b, static_cast<size_t>(v) * 8, bv);
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    o[e] = (cache[j][e] - mu) * r * wv[e] + bv[e];
                    if constexpr (GELU) o[e] = gelu_exact(o[e]);
                }
                store8(y + off, static_cast<size_t>(v) * 8, o);
            }
        }
    }
}

// dx = rstd * (g - mean(g) - xhat * mean(g * xhat)); dw += dy * xhat; db += dy
template <typename T, int VPT, bool GELU = false>
__global__ void layer_norm_bwd_kernel(const T* __restrict__ dy, const T* __restrict__ x, const T* __restrict__ w,
                                      const T* __restrict__ b, const float* __restrict__ mean,
                                      const float* __restrict__ rstd,
                                      T* __restrict__ dx, float* __restrict__ dw_part, float* __restrict__ db_part,
                                      int rows, int D) {
    __shared__ float scratch[32];
    const int nvec = D / 8;
    float dwacc[VPT][8], dbacc[VPT][8], wv[VPT][8], bv[GELU ? VPT : 1][8];
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
        const int v = threadIdx.x + j * blockDim.x;
#pragma unroll
        for (int e = 0; e < 8; ++e) dwacc[j][e] = dbacc[j][e] = 0.f;
        if (v < nvec) {
            load8(w, static_cast<size_t>(v) * 8, wv[j]);
            if constexpr (GELU) load8(b, static_cast<size_t>(v) * 8, bv[j]);
        }
    }
    for (int row = blockIdx.x; row < rows; row += gridDim.x) {
        const size_t off = static_cast<size_t>(row) * D;
        const float mu = mean[row], r = rstd[row];
        float g[VPT][8], xh[VPT][8];
        float s1 = 0.f, s2 = 0.f;
#pragma unroll
        for (int j = 0; j < VPT; ++j) {
            const int v = threadIdx.x + j * blockDim.x;
            if (v < nvec) {
                float dyv[8], xv[8];
                load8(dy + off, static_cast<size_t>(v) * 8, dyv);
                load8(x + off, static_cast<size_t>(v) * 8, xv);
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    xh[j][e] = (xv[e] - mu) * r;
                    if constexpr (GELU) dyv[e] *= gelu_exact_grad(xh[j][e] * wv[j][e] + bv[j][e]);
                    g[j][e] = dyv[e] * wv[j][e];
                    s1 += g[j][e];
                    s2 += g[j][e] * xh[j][e];
                    dwacc[j][e] += dyv[e] * xh[j][e];
                    dbacc[j][e] += dyv[e];
                }
            }
        }
        s1 = block_sum(s1, scratch) / D;
        s2 = block_sum(s2, scratch) / D;
#pragma unroll
        for (int j = 0; j < VPT; ++j) {
            const int v = threadIdx.x + j * blockDim.x;
            if (v < nvec) {
                float o[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) o[e] = r * (g[j][e] - s1 - xh[j][e] * s2);
                store8(dx + off, static_cast<size_t>(v) * 8, o);
            }
        }
    }
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
        const int v = threadIdx.x + j * blockDim.x;
        if (v < nvec) {
            store8(dw_part + static_cast<size_t>(blockIdx.x) * D, static_cast<size_t>(v) * 8, dwacc[j]);
            store8(db_part + static_cast<size_t>(blockIdx.x) * D, static_cast<size_t>(v) * 8, dbacc[j]);
        }
    }
}

// -------------------------------------------------------------------- SwiGLU
// sigmoid(x) = 0.5 * tanh(0.5 x) + 0.5 with the hardware tanh: one special-function instruction per element instead of
// an exponential plus a division (these kernels are memory-bound only as long as the XU pipe keeps up; the relative
// error of tanh.approx, about 2^-11, is below bf16 resolution).
__device__ __forceinline__ float fast_sigmoid(float x) {
    float t;
    asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(0.5f * x));
    return fmaf(0.5f, t, 0.5f);
}

// gate_up: [rows, 2F] (gate | up); y: [rows, F]
__global__ void swiglu_fwd_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ y, size_t rows,
                                  int F) {
    const size_t nvec_row = F / 8;
    const size_t total = rows * nvec_row;
    for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        const size_t row = i / nvec_row, v = i - row * nvec_row;
        float g[8], u[8], o[8];
        load8(gu + row * 2 * F, v * 8, g);
        load8(gu + row * 2 * F + F, v * 8, u);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            o[e] = g[e] * fast_sigmoid(g[e]) * u[e];
        }
        store8(y + row * F, v * 8, o);
    }
}

// Two-input form for operands that come from separate GEMMs (the experts' gate and up projections), bounded by a
// device-resident row count: only the first `num_tiles[0] * 128` rows of the capacity-sized buffers hold data.
__global__ void swiglu2_fwd_kernel(const __nv_bfloat16* __restrict__ g_, const __nv_bfloat16* __restrict__ u_,
                                   __nv_bfloat16* __restrict__ y, size_t rows, int F, const int* __restrict__ num_tiles) {
    if (num_tiles != nullptr) rows = min(rows, static_cast<size_t>(*num_tiles) * 128);
    const size_t total = rows * (F / 8);
    for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        float g[8], u[8], o[8];
        load8(g_, i * 8, g);
        load8(u_, i * 8, u);
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] = g[e] * fast_sigmoid(g[e]) * u[e];
        store8(y, i * 8, o);
    }
}

__global__ void swiglu2_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ g_,
                                   const __nv_bfloat16* __restrict__ u_, __nv_bfloat16* __restrict__ dg_,
                                   __nv_bfloat16* __restrict__ du_, size_t rows, int F,
                                   const int* __restrict__ num_tiles) {
    if (num_tiles != nullptr) rows = min(rows, static_cast<size_t>(*num_tiles) * 128);
    const size_t total = rows * (F / 8);
    for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        float g[8], u[8], d[8], dg[8], du[8];
        load8(g_, i * 8, g);
        load8(u_, i * 8, u);
        load8(dy, i * 8, d);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            const float sg = fast_sigmoid(g[e]);
            const float silu = g[e] * sg;
            du[e] = d[e] * silu;
            dg[e] = d[e] * u[e] * (sg + silu * (1.f - sg));
        }
        store8(dg_, i * 8, dg);
        store8(du_, i * 8, du);
    }
}

// dst[r] = src[r] for the first min(rows, num_tiles[0] * 128) rows (16-byte vectors).
__global__ void copy_rows_bounded_kernel(uint4* __restrict__ dst, const uint4* __restrict__ src, size_t rows,
                                         size_t vec_per_row, const int* __restrict__ num_tiles) {
    if (num_tiles != nullptr) rows = min(rows, static_cast<size_t>(*num_tiles) * 128);
    const size_t total = rows * vec_per_row;
    for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<size_t>(gridDim.x) * blockDim.x)
        dst[i] = src[i];
}

__global__ void swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ gu,
                                  __nv_bfloat16* __restrict__ dgu, size_t rows, int F) {
    const size_t nvec_row = F / 8;
    const size_t total = rows * nvec_row;
    for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        const size_t row = i / nvec_row, v = i - row * nvec_row;
        float g[8], u[8], d[8], dg[8], du[8];
        load8(gu + row * 2 * F, v * 8, g);
        load8(gu + row * 2 * F + F, v * 8, u);
        load8(dy + row * F, v * 8, d);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            const float sig = fast_sigmoid(g[e]);
            const float silu = g[e] * sig;
            du[e] = d[e] * silu;
            dg[e] = d[e] * u[e] * (sig + silu * (1.f - sig));
        }
        store8(dgu + row * 2 * F, v * 8, dg);
        store8(dgu + row * 2 * F + F, v * 8, du);
    }
}

// ---------------------------------------------------------------------- RoPE
// x: [tokens, heads, D] with token stride `tstride` and head stride `hstride`
// (elements). freqs: [L, D/2, 2] (cos, sin) fp32. pos[t] < 0 -> untouched.
__global__ void rope_kernel(__nv_bfloat16* __restrict__ x, const float* __restrict__ freqs,
                            const int* __restrict__ pos, size_t tokens, int heads, int D, size_t tstride,
                            size_t hstride, int max_pos, float sign) {
    const int vec_per_head = D / 8;
    const size_t total = tokens * heads * vec_per_head;
    for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        const int v = static_cast<int>(i % vec_per_head);
        const size_t th = i / vec_per_head;
        const int h = static_cast<int>(th % heads);
        const size_t t = th / heads;
        const int p = pos[t];
        if (p < 0 || p >= max_pos) continue;
        __nv_bfloat16* ptr = x + t * tstride + static_cast<size_t>(h) * hstride;
        float f[8], cs[8], o[8];
        load8(ptr, static_cast<size_t>(v) * 8, f);
        load8(freqs + (static_cast<size_t>(p) * (D / 2)) * 2, static_cast<size_t>(v) * 8, cs);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float c = cs[2 * e], s = cs[2 * e + 1] * sign;
            const float a = f[2 * e], b = f[2 * e + 1];
            o[2 * e] = a * c - b * s;
            o[2 * e + 1] = a * s + b * c;
        }
        store8(ptr, static_cast<size_t>(v) * 8, o);
    }
}

// ------------------------------------------------------ vocabulary-parallel embedding
// This rank holds rows [lo, lo + rows) of the table. out[t] = table[ids[t] - lo] for ids in range, else 0 (the other
// ranks contribute those rows; the sum over ranks is the lookup). One warp per token.
__global__ void __launch_bounds__(256) embed_vocab_parallel_fwd_kernel(const long long* __restrict__ ids,
                                                                       const __nv_bfloat16* __restrict__ table,
                                                                       __nv_bfloat16* __restrict__ out, size_t tokens,
                                                                       int D, long long lo, long long rows, float scale) {
    const size_t t = (blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (t >= tokens) return;
    const long long r = ids[t] - lo;
    const bool mine = r >= 0 && r < rows;
    for (int c = lane * 8; c < D; c += 256) {
        float f[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        if (mine) {
            load8(table + static_cast<size_t>(r) * D, c, f);
            if (scale != 1.f) {
#pragma unroll
                for (int e = 0; e < 8; ++e) f[e] *= scale;
            }
        }
        store8(out + t * D, c, f);
    }
}

// dtable[ids[t] - lo] += scale * dout[t] for ids in range (fp32 accumulation buffer, atomics: tokens repeat).
__global__ void __launch_bounds__(256) embed_vocab_parallel_bwd_kernel(const long long* __restrict__ ids,
                                                                       const __nv_bfloat16* __restrict__ dout,
                                                                       float* __restrict__ dtable, size_t tokens, int D,
                                                                       long long lo, long long rows, float scale) {
    const size_t t = (blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (t >= tokens) return;
    const long long r = ids[t] - lo;
    if (r < 0 || r >= rows) return;
    for (int c = lane * 8; c < D; c += 256) {
        float f[8];
        load8(dout + t * D, c, f);
#pragma unroll
        for (int e = 0; e < 8; ++e) atomicAdd(dtable + static_cast<size_t>(r) * D + c + e, f[e] * scale);
    }
}

// ------------------------------------------------------------- cross-entropy
// One block per row. logits (bf16, [rows, V]) are overwritten with
// (softmax - onehot) * mask[row]; row_loss[row] = (lse - logit[target]) * mask.
__global__ void ce_fwd_bwd_kernel(__nv_bfloat16* __restrict__ logits, const long long* __restrict__ targets,
                                  const float* __restrict__ mask, float* __restrict__ row_loss, int V, int pad_idx) {
    __shared__ float scratch[32];
    const size_t row = blockIdx.x;
    __nv_bfloat16* lr = logits + row * static_cast<size_t>(V);
    const long long tgt = targets[row];
    float mk = mask ? mask[row] : 1.f;
    if (tgt == pad_idx || tgt < 0 || tgt >= V) mk = 0.f;
    const int nvec = V / 8;
    if (mk == 0.f) {
        const float zf[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        const bf16x8 z = pack8(zf);
        for (int v = threadIdx.x; v < nvec; v += blockDim.x) *reinterpret_cast<bf16x8*>(lr + static_cast<size_t>(v) * 8) = z;
        if (threadIdx.x == 0) row_loss[row] = 0.f;
        return;
    }
    float mx = -INFINITY, sum = 0.f;
    for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
        float f[8];
        load8(lr, static_cast<size_t>(v) * 8, f);
        float lm = f[0];
#pragma unroll
        for (int e = 1; e < 8; ++e) lm = fmaxf(lm, f[e]);
        const float nm = fmaxf(mx, lm);
        float acc = 0.f;
#pragma unroll
        for (int e = 0; e < 8; ++e) acc += __expf(f[e] - nm);
        sum = sum * __expf(mx - nm) + acc;
        mx = nm;
    }
    const float gmx = block_max(mx, scratch);
    sum = (mx == -INFINITY) ? 0.f : sum * __expf(mx - gmx);
    const float gsum = block_sum(sum, scratch);
    const float lse = gmx + logf(gsum);
    const float tl = __bfloat162float(lr[tgt]);
    __syncthreads();  // everyone has read the target logit before it is overwritten
    if (threadIdx.x == 0) row_loss[row] = (lse - tl) * mk;
    const int tv = static_cast<int>(tgt / 8), te = static_cast<int>(tgt % 8);
    for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
        float f[8], o[8];
        load8(lr, static_cast<size_t>(v) * 8, f);
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] = __expf(f[e] - lse) * mk;
        if (v == tv) o[te] -= mk;
        store8(lr, static_cast<size_t>(v) * 8, o);
    }
}

// --------------------------------------------------------------------- AdamW
template <typename G>
__global__ void adamw_kernel(float* __restrict__ p, const G* __restrict__ g, float* __restrict__ m,
                             float* __restrict__ v, __nv_bfloat16* __restrict__ low, size_t n, float lr, float beta1,
                             float beta2, float eps, float wd, float bc1, float bc2_sqrt,
                             const float* __restrict__ grad_scale, const int* __restrict__ guard) {
    // `guard` is a device-memory copy of the status word of the bounded waits (refreshed once per optimizer step):
    // a collective that gave up left this step's gradients (or parameters) incomplete, so the update is skipped
    // and the weights stay as they were; the host raises. Device memory, not the host-mapped word itself: tens of
    // thousands of blocks reading one word over PCIe serialise (0.4 ms per launch on an 8 B-parameter model).
    if (guard != nullptr) {
        __shared__ int bad;
        if (threadIdx.x == 0) bad = *reinterpret_cast<const volatile int*>(guard);
        __syncthreads();
        if (bad != 0) return;
    }
    const float gs = grad_scale ? *grad_scale : 1.f;
    const size_t nvec = n / 8;
    const float step_size = lr / bc1;
    for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < nvec;
         i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        float pv[8], gv[8], mv[8], vv[8];
        load8(p, i * 8, pv);
        load8(g, i * 8, gv);
        load8(m, i * 8, mv);
        load8(v, i * 8, vv);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            const float gr = gv[e] * gs;
            pv[e] *= (1.f - lr * wd);
            mv[e] = beta1 * mv[e] + (1.f - beta1) * gr;
            vv[e] = beta2 * vv[e] + (1.f - beta2) * gr * gr;
            const float denom = sqrtf(vv[e]) / bc2_sqrt + eps;
            pv[e] -= step_size * mv[e] / denom;
        }
        store8(p, i * 8, pv);
        store8(m, i * 8, mv);
        store8(v, i * 8, vv);
        if (low) store8(low, i * 8, pv);
    }
    // tail (n not a multiple of 8)
    if (blockIdx.x == 0) {
        for (size_t i = nvec * 8 + threadIdx.x; i < n; i += blockDim.x) {
            float gr;
            if constexpr (sizeof(G) == 2) gr = __bfloat162float(g[i]) * gs;
            else gr = g[i] * gs;
            float pv = p[i] * (1.f - lr * wd);
            const float mv = beta1 * m[i] + (1.f - beta1) * gr;
            const float vv = beta2 * v[i] + (1.f - beta2) * gr * gr;
            pv -= step_size * mv / (sqrtf(vv) / bc2_sqrt + eps);
            p[i] = pv;
            m[i] = mv;
            v[i] = vv;
            if (low) low[i] = __float2bfloat16_rn(pv);
        }
    }
}

// dst (device memory) = *src (the host-mapped status word): one PCIe read per optimizer step.
__global__ void copy_status_kernel(const int* __restrict__ src, int* __restrict__ dst) {
    *dst = *reinterpret_cast<const volatile int*>(src);
}

template <typename T>
__global__ void l2_norm_sq_kernel(const T* __restrict__ x, size_t n, float* __restrict__ out) {
    __shared__ float scratch[32];
    const size_t nvec = n / 8;
    float acc = 0.f;
    for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < nvec;
         i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        float f[8];
        load8(x, i * 8, f);
#pragma unroll
        for (int e = 0; e < 8; ++e) acc += f[e] * f[e];
    }
    if (blockIdx.x == 0) {
        for (size_t i = nvec * 8 + threadIdx.x; i < n; i += blockDim.x) {
            float f;
            if constexpr (sizeof(T) == 2) f = __bfloat162float(x[i]);
            else f = x[i];
            acc += f * f;
        }
    }
    acc = block_sum(acc, scratch);
    if (threadIdx.x == 0) atomicAdd(out, acc);
}

template <typename T>
__global__ void scale_kernel(T* __restrict__ x, size_t n, const float* __restrict__ scale) {
    const float s = *scale;
    const size_t nvec = n / 8;
    for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < nvec;
         i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        float f[8];
        load8(x, i * 8, f);
#pragma unroll
        for (int e = 0; e < 8; ++e) f[e] *= s;
        store8(x, i * 8, f);
    }
    if (blockIdx.x == 0) {
        for (size_t i = nvec * 8 + threadIdx.x; i < n; i += blockDim.x) {
            if constexpr (sizeof(T) == 2) x[i] = __float2bfloat16_rn(__bfloat162float(x[i]) * s);
            else x[i] = x[i] * s;
        }
    }
}

inline int norm_vpt(int D, int threads) {
    const int nvec = D / 8;
    const int need = (nvec + threads - 1) / threads;
    return need <= 1 ? 1 : need <= 2 ? 2 : need <= 4 ? 4 : 8;
}

#define FS2_VPT_DISPATCH(VPT_VALUE, ...)                   \
    switch (VPT_VALUE) {                                   \
        case 1: { constexpr int VPT = 1; __VA_ARGS__; break; } \
        case 2: { constexpr int VPT = 2; __VA_ARGS__; break; } \
        case 4: { constexpr int VPT = 4; __VA_ARGS__; break; } \
        default: { constexpr int VPT = 8; __VA_ARGS__; break; } \
    }

inline int stream_grid(size_t work_items, int threads, int num_sms) {
    size_t blocks = (work_items + threads - 1) / threads;
    const size_t cap = static_cast<size_t>(num_sms) * 8;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    return static_cast<int>(blocks);
}

}  // namespace

// ------------------------------------------------------------------ launchers
int norm_bwd_grid(int rows, int num_sms) {
    int g = num_sms * 2;
    return rows < g ? rows : g;
}

void rms_norm_fwd(const void* x, const void* w, void* y, float* rstd, int rows, int D, float eps, bool bf16,
                  int num_sms, cudaStream_t st, const void* res, void* sum_out) {
    const int threads = norm_block(D);
    const int grid = rows < num_sms * 16 ? rows : num_sms * 16;
    FS2_VPT_DISPATCH(norm_vpt(D, threads),
        if (bf16)
            rms_norm_fwd_kernel<__nv_bfloat16, VPT><<<grid, threads, 0, st>>>(
                static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(w),
                static_cast<__nv_bfloat16*>(y), rstd, rows, D, eps, static_cast<const __nv_bfloat16*>(res),
                static_cast<__nv_bfloat16*>(sum_out));
        else
            rms_norm_fwd_kernel<float, VPT><<<grid, threads, 0, st>>>(
                static_cast<const float*>(x), static_cast<const float*>(w), static_cast<float*>(y), rstd, rows, D,
                eps, static_cast<const float*>(res), static_cast<float*>(sum_out)))
}

void rms_norm_bwd(const void* dy, const void* x, const void* w, const float* rstd, void* dx, float* dw_part,
                  float* dw, int rows, int D, bool bf16, int num_sms, cudaStream_t st, const void* dres) {
    const int threads = norm_block_bwd(D);
    const int grid = norm_bwd_grid(rows, num_sms);
    FS2_VPT_DISPATCH(norm_vpt(D, threads),
        if (bf16)
            rms_norm_bwd_kernel<__nv_bfloat16, VPT><<<grid, threads, 0, st>>>(
                static_cast<const __nv_bfloat16*>(dy), static_cast<const __nv_bfloat16*>(x),
                static_cast<const __nv_bfloat16*>(w), rstd, static_cast<__nv_bfloat16*>(dx), dw_part, rows, D,
                static_cast<const __nv_bfloat16*>(dres));
        else
            rms_norm_bwd_kernel<float, VPT><<<grid, threads, 0, st>>>(
                static_cast<const float*>(dy), static_cast<const float*>(x), static_cast<const float*>(w), rstd,
                static_cast<float*>(dx), dw_part, rows, D, static_cast<const float*>(dres)))
    reduce_partials_kernel<<<(D + 255) / 256, 256, 0, st>>>(dw_part, dw, grid, D);
}

void layer_norm_fwd(const void* x, const void* w, const void* b, void* y, float* mean, float* rstd, int rows, int D,
                    float eps, bool bf16, int num_sms, cudaStream_t st, bool gelu) {
    const int threads = norm_block(D);
    const int grid = rows < num_sms * 16 ? rows : num_sms * 16;
    if (gelu) {        // bf16 only
        FS2_VPT_DISPATCH(norm_vpt(D, threads),
            (layer_norm_fwd_kernel<__nv_bfloat16, VPT, true><<<grid, threads, 0, st>>>(
                static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(w),
                static_cast<const __nv_bfloat16*>(b), static_cast<__nv_bfloat16*>(y), mean, rstd, rows, D, eps)))
        return;
    }
    FS2_VPT_DISPATCH(norm_vpt(D, threads),
        if (bf16)
            layer_norm_fwd_kernel<__nv_bfloat16, VPT><<<grid, threads, 0, st>>>(
                static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(w),
                static_cast<const __nv_bfloat16*>(b), static_cast<__nv_bfloat16*>(y), mean, rstd, rows, D, eps);
        else
            layer_norm_fwd_kernel<float, VPT><<<grid, threads, 0, st>>>(
                static_cast<const float*>(x), static_cast<const float*>(w), static_cast<const float*>(b),
                static_cast<float*>(y), mean, rstd, rows, D, eps))
}

void layer_norm_bwd(const void* dy, const void* x, const void* w, const float* mean, const float* rstd, void* dx,
                    float* dw_part, float* db_part, float* dw, float* db, int rows, int D, bool bf16, int num_sms,
                    cudaStream_t st, const void* b_for_gelu) {
    const int threads = norm_block_bwd(D);
    const int grid = norm_bwd_grid(rows, num_sms);
    if (b_for_gelu != nullptr) {        // bf16 only: dy is the gradient of gelu(layer_norm(x))
        FS2_VPT_DISPATCH(norm_vpt(D, threads),
            (layer_norm_bwd_kernel<__nv_bfloat16, VPT, true><<<grid, threads, 0, st>>>(
                static_cast<const __nv_bfloat16*>(dy), static_cast<const __nv_bfloat16*>(x),
                static_cast<const __nv_bfloat16*>(w), static_cast<const __nv_bfloat16*>(b_for_gelu), mean, rstd,
                static_cast<__nv_bfloat16*>(dx), dw_part, db_part, rows, D)))
    } else {
    FS2_VPT_DISPATCH(norm_vpt(D, threads),
        if (bf16)
            layer_norm_bwd_kernel<__nv_bfloat16, VPT><<<grid, threads, 0, st>>>(
                static_cast<const __nv_bfloat16*>(dy), static_cast<const __nv_bfloat16*>(x),
                static_cast<const __nv_bfloat16*>(w), nullptr, mean, rstd, static_cast<__nv_bfloat16*>(dx), dw_part,
                db_part, rows, D);
        else
            layer_norm_bwd_kernel<float, VPT><<<grid, threads, 0, st>>>(
                static_cast<const float*>(dy), static_cast<const float*>(x), static_cast<const float*>(w), nullptr,
                mean, rstd, static_cast<float*>(dx), dw_part, db_part, rows, D))
    }
    reduce_partials_kernel<<<(D + 255) / 256, 256, 0, st>>>(dw_part, dw, grid, D);
    reduce_partials_kernel<<<(D + 255) / 256, 256, 0, st>>>(db_part, db, grid, D);
}

void swiglu2_fwd(const void* g, const void* u, void* y, size_t rows, int F, const int* num_tiles, int num_sms,
                 cudaStream_t st) {
    const size_t work = rows * (F / 8);
    if (work == 0) return;
    swiglu2_fwd_kernel<<<stream_grid(work, 256, num_sms), 256, 0, st>>>(
        static_cast<const __nv_bfloat16*>(g), static_cast<const __nv_bfloat16*>(u), static_cast<__nv_bfloat16*>(y), rows,
        F, num_tiles);
}

void swiglu2_bwd(const void* dy, const void* g, const void* u, void* dg, void* du, size_t rows, int F,
                 const int* num_tiles, int num_sms, cudaStream_t st) {
    const size_t work = rows * (F / 8);
    if (work == 0) return;
    swiglu2_bwd_kernel<<<stream_grid(work, 256, num_sms), 256, 0, st>>>(
        static_cast<const __nv_bfloat16*>(dy), static_cast<const __nv_bfloat16*>(g),
        static_cast<const __nv_bfloat16*>(u), static_cast<__nv_bfloat16*>(dg), static_cast<__nv_bfloat16*>(du), rows, F,
        num_tiles);
}

void copy_rows_bounded(void* dst, const void* src, size_t rows, size_t row_bytes, const int* num_tiles, int num_sms,
                       cudaStream_t st) {
    const size_t work = rows * (row_bytes / 16);
    if (work == 0) return;
    copy_rows_bounded_kernel<<<stream_grid(work, 512, num_sms), 512, 0, st>>>(
        static_cast<uint4*>(dst), static_cast<const uint4*>(src), rows, row_bytes / 16, num_tiles);
}

void swiglu_fwd(const void* gu, void* y, size_t rows, int F, int num_sms, cudaStream_t st) {
    const size_t work = rows * (F / 8);
    swiglu_fwd_kernel<<<stream_grid(work, 256, num_sms), 256, 0, st>>>(static_cast<const __nv_bfloat16*>(gu),
                                                                        static_cast<__nv_bfloat16*>(y), rows, F);
}

void swiglu_bwd(const void* dy, const void* gu, void* dgu, size_t rows, int F, int num_sms, cudaStream_t st) {
    const size_t work = rows * (F / 8);
    swiglu_bwd_kernel<<<stream_grid(work, 256, num_sms), 256, 0, st>>>(
        static_cast<const __nv_bfloat16*>(dy), static_cast<const __nv_bfloat16*>(gu),
        static_cast<__nv_bfloat16*>(dgu), rows, F);
}

void rope_inplace(void* x, const float* freqs, const int* pos, size_t tokens, int heads, int D, size_t tstride,
                  size_t hstride, int max_pos, bool inverse, int num_sms, cudaStream_t st) {
    const size_t work = tokens * heads * (D / 8);
    if (work == 0) return;
    rope_kernel<<<stream_grid(work, 256, num_sms), 256, 0, st>>>(static_cast<__nv_bfloat16*>(x), freqs, pos, tokens,
                                                                  heads, D, tstride, hstride, max_pos,
                                                                  inverse ? -1.f : 1.f);
}

void embed_vocab_parallel_fwd(const long long* ids, const void* table, void* out, size_t tokens, int D, long long lo,
                              long long rows, float scale, cudaStream_t st) {
    if (tokens == 0) return;
    const unsigned blocks = static_cast<unsigned>((tokens * 32 + 255) / 256);
    embed_vocab_parallel_fwd_kernel<<<blocks, 256, 0, st>>>(ids, static_cast<const __nv_bfloat16*>(table),
                                                            static_cast<__nv_bfloat16*>(out), tokens, D, lo, rows, scale);
}

void embed_vocab_parallel_bwd(const long long* ids, const void* dout, float* dtable, size_t tokens, int D, long long lo,
                              long long rows, float scale, cudaStream_t st) {
    if (tokens == 0) return;
    const unsigned blocks = static_cast<unsigned>((tokens * 32 + 255) / 256);
    embed_vocab_parallel_bwd_kernel<<<blocks, 256, 0, st>>>(ids, static_cast<const __nv_bfloat16*>(dout), dtable, tokens,
                                                            D, lo, rows, scale);
}

void ce_fwd_bwd(void* logits, const long long* targets, const float* mask, float* row_loss, int rows, int V,
                int pad_idx, cudaStream_t st) {
    if (rows == 0) return;
    ce_fwd_bwd_kernel<<<rows, 1024, 0, st>>>(static_cast<__nv_bfloat16*>(logits), targets, mask, row_loss, V,
                                             pad_idx);
}

void adamw(float* p, const void* g, bool g_bf16, float* m, float* v, void* low, size_t n, float lr, float beta1,
           float beta2, float eps, float wd, int step, const float* grad_scale, const int* guard, int num_sms,
           cudaStream_t st) {
    if (n == 0) return;
    const float bc1 = 1.f - powf(beta1, static_cast<float>(step));
    const float bc2 = 1.f - powf(beta2, static_cast<float>(step));
    const int grid = stream_grid(n / 8 + 1, 256, num_sms);
    if (g_bf16)
        adamw_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(p, static_cast<const __nv_bfloat16*>(g), m, v,
                                                          static_cast<__nv_bfloat16*>(low), n, lr, beta1, beta2, eps,
                                                          wd, bc1, sqrtf(bc2), grad_scale, guard);
    else
        adamw_kernel<float><<<grid, 256, 0, st>>>(p, static_cast<const float*>(g), m, v,
                                                  static_cast<__nv_bfloat16*>(low), n, lr, beta1, beta2, eps, wd, bc1,
                                                  sqrtf(bc2), grad_scale, guard);
}

void copy_status(const int* host_mapped_status, int* device_guard, cudaStream_t st) {
    copy_status_kernel<<<1, 1, 0, st>>>(host_mapped_status, device_guard);
}

void l2_norm_sq(const void* x, bool bf16, size_t n, float* out, int num_sms, cudaStream_t st) {
    if (n == 0) return;
    const int grid = stream_grid(n / 8 + 1, 512, num_sms);
    if (bf16) l2_norm_sq_kernel<__nv_bfloat16><<<grid, 512, 0, st>>>(static_cast<const __nv_bfloat16*>(x), n, out);
    else l2_norm_sq_kernel<float><<<grid, 512, 0, st>>>(static_cast<const float*>(x), n, out);
}

void scale_inplace(void* x, bool bf16, size_t n, const float* scale, int num_sms, cudaStream_t st) {
    if (n == 0) return;
    const int grid = stream_grid(n / 8 + 1, 256, num_sms);
    if (bf16) scale_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(static_cast<__nv_bfloat16*>(x), n, scale);
    else scale_kernel<float><<<grid, 256, 0, st>>>(static_cast<float*>(x), n, scale);
}

}  // namespace fs2

// ---------------------------------------------------------------------------
// Allocation-free RMSNorm backward (declared and documented in no_alloc.h).
// Same kernels as `rms_norm_bwd` above; only the home of the per-block partial
// sums differs: a fixed __device__ array instead of a caller-provided buffer.
// ---------------------------------------------------------------------------
#include <mutex>

#include "no_alloc.h"

namespace fs2 {
namespace {

static __device__ __align__(256) float g_no_alloc_scratch[FS2_NO_ALLOC_MAX_BLOCKS * FS2_NO_ALLOC_MAX_DIM];

constexpr int kMaxDevices = 64;
float* g_no_alloc_ptr[kMaxDevices] = {};
std::mutex g_no_alloc_mutex;
thread_local const char* g_no_alloc_error = "";

// Device address of the scratch array on the current device. In host code the
// array's name is only a handle, never an address a kernel may dereference.
float* no_alloc_scratch_ptr() {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
        g_no_alloc_error = "cudaGetDevice failed or device ordinal out of range";
        return nullptr;
    }
    std::lock_guard<std::mutex> lock(g_no_alloc_mutex);
    if (g_no_alloc_ptr[dev] == nullptr) {
        void* p = nullptr;
        const cudaError_t e = cudaGetSymbolAddress(&p, g_no_alloc_scratch);
        if (e != cudaSuccess || p == nullptr) {
            g_no_alloc_error = "cudaGetSymbolAddress failed for the static scratch array";
            return nullptr;
        }
        g_no_alloc_ptr[dev] = static_cast<float*>(p);
    }
    return g_no_alloc_ptr[dev];
}

}  // namespace
}  // namespace fs2

extern "C" const char* fs2_no_alloc_last_error() { return fs2::g_no_alloc_error; }

extern "C" int fs2_rms_norm_bwd_no_alloc(const void* dy, const void* x, const void* w, const float* rstd, void* dx,
                                         float* dw, int rows, int D, int is_bf16, cudaStream_t stream) {
    using namespace fs2;
    if (rows < 1) {
        g_no_alloc_error = "rows must be >= 1";
        return 1;
    }
    if (D < 8 || D % 8 != 0 || D > FS2_NO_ALLOC_MAX_DIM) {
        g_no_alloc_error = "D must be a multiple of 8 and at most FS2_NO_ALLOC_MAX_DIM (8192)";
        return 2;
    }
    const uintptr_t bits = reinterpret_cast<uintptr_t>(dy) | reinterpret_cast<uintptr_t>(x) |
                           reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(dx) |
                           reinterpret_cast<uintptr_t>(dw);
    if (dy == nullptr || x == nullptr || w == nullptr || rstd == nullptr || dx == nullptr || dw == nullptr ||
        (bits & 15u) != 0) {
        g_no_alloc_error = "all pointers must be non-null and 16-byte aligned";
        return 3;
    }
    // the scratch array is resolved for the current device while the kernels go to `stream`: both must be the same GPU
    int current = -1, stream_dev = -1;
    if (cudaGetDevice(&current) == cudaSuccess && cudaStreamGetDevice(stream, &stream_dev) == cudaSuccess) {
        if (stream_dev != current) {
            g_no_alloc_error = "the device that owns `stream` must be the current device of the calling thread";
            return 6;
        }
    } else {
        (void)cudaGetLastError();           // the query is unavailable: the header states the requirement
    }
    float* scratch = no_alloc_scratch_ptr();
    if (scratch == nullptr) return 4;
    const int threads = norm_block_bwd(D);
    const int grid = rows < FS2_NO_ALLOC_MAX_BLOCKS ? rows : FS2_NO_ALLOC_MAX_BLOCKS;
    FS2_VPT_DISPATCH(norm_vpt(D, threads),
        if (is_bf16)
            rms_norm_bwd_kernel<__nv_bfloat16, VPT><<<grid, threads, 0, stream>>>(
                static_cast<const __nv_bfloat16*>(dy), static_cast<const __nv_bfloat16*>(x),
                static_cast<const __nv_bfloat16*>(w), rstd, static_cast<__nv_bfloat16*>(dx), scratch, rows, D,
                nullptr);
        else
            rms_norm_bwd_kernel<float, VPT><<<grid, threads, 0, stream>>>(
                static_cast<const float*>(dy), static_cast<const float*>(x), static_cast<const float*>(w), rstd,
                static_cast<float*>(dx), scratch, rows, D, nullptr))
    reduce_partials_kernel<<<(D + 255) / 256, 256, 0, stream>>>(scratch, dw, grid, D);
    if (cudaGetLastError() != cudaSuccess) {
        g_no_alloc_error = "kernel launch failed";
        return 5;
    }
    g_no_alloc_error = "";
    return 0;
}
