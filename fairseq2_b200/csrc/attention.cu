// Variable-length causal GQA flash attention, forward and backward.
//
// Sequences are given as (begin offset, length) pairs into the flattened token
// axis for queries and keys separately, so packed batches (block-causal per
// document), padded batches and prefill-with-cache all use the same kernels.
// Causal masking is bottom-right aligned: query i sees keys j <= i + (Lk - Lq).
// K/V heads are addressed as h / (H / Hkv): grouped-query attention is never
// materialised. q/k/v/o/dq/dk/dv may be strided views ([T, heads, D] with an
// arbitrary token stride), which lets the kernels read and write the merged
// qkv projection buffer in place.
//
// Tensor-core path: bf16 mma.sync m16n8k16 with fp32 accumulation, operands
// staged through XOR-swizzled shared memory by cp.async and read by ldmatrix.
//
// Backward is split into two deterministic kernels (no atomics): `dkv` owns a
// 64-row K/V block and loops over the query blocks (and the G query heads that
// share the KV head); `dq` owns a 128-row query block and loops over K/V
// blocks, recomputing the probabilities from the saved log-sum-exp.

#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdint>

#include "attention.h"
#include "common.cuh"

namespace fs2 {

namespace {

constexpr float LOG2E = 1.4426950408889634f;

// ------------------------------------------------------------------ helpers
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool valid) {
    const int bytes = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                 : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                 : "r"(addr));
}

// D(16x8, fp32) += A(16x16, bf16, row) * B(16x8, bf16, col)
__device__ __forceinline__ void mma16816(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
        "{%0, %1, %2, %3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
}

// Shared tile of ROWS x D bf16, 16-byte chunks XOR-swizzled by (row & 7).
template <int D>
__device__ __forceinline__ uint32_t tile_addr(uint32_t base, int row, int chunk) {
    constexpr int CHUNKS = D / 8;
    return base + static_cast<uint32_t>((row * CHUNKS + (chunk ^ (row & 7))) * 16);
}

// Loads rows [row0, row0 + ROWS) of a [*, heads, D] tensor (token stride
// `tstride` elements) into a swizzled tile; rows >= nrows are zero-filled.
template <int D, int ROWS, int THREADS>
__device__ __forceinline__ void load_tile(uint32_t smem, const __nv_bfloat16* gptr, size_t tstride, int row0,
                                          int nrows) {
    constexpr int CHUNKS = D / 8;
    constexpr int TOTAL = ROWS * CHUNKS;
    for (int i = threadIdx.x; i < TOTAL; i += THREADS) {
        const int r = i / CHUNKS, c = i % CHUNKS;
        const int gr = row0 + r;
        const bool valid = gr < nrows;
        const __nv_bfloat16* src = gptr + static_cast<size_t>(valid ? gr : 0) * tstride + c * 8;
        cp_async16(tile_addr<D>(smem, r, c), src, valid);
    }
}

// A fragment (16 rows x 16 k) of a row-major tile: rows [r0, r0+16), k chunk pair kc (16 elements).
template <int D>
__device__ __forceinline__ void load_a_frag(uint32_t tile, int r0, int ks, uint32_t* a) {
    const int lane = threadIdx.x & 31;
    const int row = r0 + (lane & 15);
    const int chunk = ks * 2 + (lane >> 4);
    ldsm_x4(tile_addr<D>(tile, row, chunk), a[0], a[1], a[2], a[3]);
}

// B fragments for two adjacent n8 blocks from a tile stored [n][k] (k contiguous):
// n rows [n0, n0 + 16), k-step ks. b[0],b[1] -> n block 0; b[2],b[3] -> n block 1.
template <int D>
__device__ __forceinline__ void load_b_frag_nk(uint32_t tile, int n0, int ks, uint32_t* b) {
    const int lane = threadIdx.x & 31;
    const int id = lane >> 3;
    const int row = n0 + (id >> 1) * 8 + (lane & 7);
    const int chunk = ks * 2 + (id & 1);
    ldsm_x4(tile_addr<D>(tile, row, chunk), b[0], b[1], b[2], b[3]);
}

// B fragments for two adjacent n8 blocks from a tile stored [k][n] (n contiguous):
// k rows [k0, k0 + 16), n chunk pair starting at chunk nc. b[0],b[1] -> n block nc; b[2],b[3] -> nc + 1.
template <int D>
__device__ __forceinline__ void load_b_frag_kn(uint32_t tile, int k0, int nc, uint32_t* b) {
    const int lane = threadIdx.x & 31;
    const int id = lane >> 3;
    const int row = k0 + (id & 1) * 8 + (lane & 7);
    const int chunk = nc + (id >> 1);
    ldsm_x4_t(tile_addr<D>(tile, row, chunk), b[0], b[1], b[2], b[3]);
}

struct SeqInfo {
    int qb, ql, kb, kl, shift;
};

// Stateless dropout mask: the forward kernel and both backward kernels evaluate the same hash of (seed, head, global
// query token, global key token), so no mask is stored. Two rounds of the murmur3 finaliser.
__device__ __forceinline__ uint32_t mix32(uint32_t a) {
    a ^= a >> 16;
    a *= 0x85EBCA6Bu;
    a ^= a >> 13;
    a *= 0xC2B2AE35u;
    a ^= a >> 16;
    return a;
}
__device__ __forceinline__ bool dropout_keep(const AttnParams& p, int h, int qtok, int ktok) {
    uint32_t a = mix32(static_cast<uint32_t>(qtok) ^ static_cast<uint32_t>(p.seed));
    a = mix32(a + static_cast<uint32_t>(ktok) * 0x9E3779B1u + static_cast<uint32_t>(h) * 0x7F4A7C15u +
              static_cast<uint32_t>(p.seed >> 32));
    return a >= p.drop_threshold;
}

__device__ __forceinline__ SeqInfo seq_info(const AttnParams& p, int s) {
    SeqInfo i;
    i.qb = p.q_begins[s];
    i.ql = p.q_lens[s];
    i.kb = p.k_begins[s];
    i.kl = p.k_lens[s];
    i.shift = i.kl - i.ql;
    return i;
}

// ------------------------------------------------------------------ forward
// grid (q blocks, seqs, H); 256 threads; BLOCK_M = 128, BLOCK_N = 64.
template <int D>
__global__ void __launch_bounds__(256, 1) attn_fwd_kernel(const AttnParams p) {
    constexpr int BM = 128, BN = 64, THREADS = 256;
    constexpr int KS = D / 16;      // k-steps over the head dim
    constexpr int NB_D = D / 8;     // n8 blocks over the head dim
    extern __shared__ __align__(128) uint8_t smem_raw[];
    const uint32_t sQ = smem_u32(smem_raw);
    const uint32_t sK0 = sQ + BM * D * 2;
    const uint32_t sV0 = sK0 + 2 * BN * D * 2;

    const SeqInfo si = seq_info(p, blockIdx.y);
    const int m0 = blockIdx.x * BM;
    if (m0 >= si.ql) return;
    const int h = blockIdx.z;
    const int hk = h / (p.H / p.Hkv);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    const __nv_bfloat16* qg = p.q + static_cast<size_t>(si.qb) * p.q_tstride + static_cast<size_t>(h) * D;
    const __nv_bfloat16* kg = p.k + static_cast<size_t>(si.kb) * p.k_tstride + static_cast<size_t>(hk) * D;
    const __nv_bfloat16* vg = p.v + static_cast<size_t>(si.kb) * p.v_tstride + static_cast<size_t>(hk) * D;

    int n_end = si.kl;  // exclusive bound on visible keys for this q block
    if (p.causal) n_end = min(si.kl, m0 + BM + si.shift);
    const int nblocks = n_end > 0 ? (n_end + BN - 1) / BN : 0;

    load_tile<D, BM, THREADS>(sQ, qg, p.q_tstride, m0, si.ql);
    if (nblocks > 0) {
        load_tile<D, BN, THREADS>(sK0, kg, p.k_tstride, 0, si.kl);
        load_tile<D, BN, THREADS>(sV0, vg, p.v_tstride, 0, si.kl);
    }
    cp_async_commit();

    float acc_o[NB_D][4];
#pragma unroll
    for (int i = 0; i < NB_D; ++i) acc_o[i][0] = acc_o[i][1] = acc_o[i][2] = acc_o[i][3] = 0.f;
    float row_max[2] = {-INFINITY, -INFINITY};
    float row_sum[2] = {0.f, 0.f};
    const float sl2 = p.scale * LOG2E;

    uint32_t qf[KS][4];
    const int r_lo = m0 + warp * 16 + (lane >> 2);  // query row (within the sequence) of c0/c1; c2/c3 is +8

    for (int j = 0; j < nblocks; ++j) {
        const int buf = j & 1;
        const uint32_t sK = sK0 + buf * BN * D * 2;
        const uint32_t sV = sV0 + buf * BN * D * 2;
        if (j + 1 < nblocks) {
            load_tile<D, BN, THREADS>(sK0 + (buf ^ 1) * BN * D * 2, kg, p.k_tstride, (j + 1) * BN, si.kl);
            load_tile<D, BN, THREADS>(sV0 + (buf ^ 1) * BN * D * 2, vg, p.v_tstride, (j + 1) * BN, si.kl);
            cp_async_commit();
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        if (j == 0) {
#pragma unroll
            for (int ks = 0; ks < KS; ++ks) load_a_frag<D>(sQ, warp * 16, ks, qf[ks]);
        }

        float acc_s[BN / 8][4];
#pragma unroll
        for (int i = 0; i < BN / 8; ++i) acc_s[i][0] = acc_s[i][1] = acc_s[i][2] = acc_s[i][3] = 0.f;
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
#pragma unroll
            for (int nb = 0; nb < BN / 16; ++nb) {
                uint32_t b[4];
                load_b_frag_nk<D>(sK, nb * 16, ks, b);
                mma16816(acc_s[2 * nb], qf[ks], b[0], b[1]);
                mma16816(acc_s[2 * nb + 1], qf[ks], b[2], b[3]);
            }
        }

        // masking (key bound and causal diagonal)
        const int n0 = j * BN;
        const bool need_mask = (n0 + BN > si.kl) || (p.causal && (n0 + BN - 1 > m0 + warp * 16 + si.shift));
        if (need_mask) {
#pragma unroll
            for (int nb = 0; nb < BN / 8; ++nb) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int col = n0 + nb * 8 + (lane & 3) * 2 + (e & 1);
                    const int row = r_lo + (e >> 1) * 8;
                    const bool dead = col >= si.kl || (p.causal && col > row + si.shift);
                    if (dead) acc_s[nb][e] = -INFINITY;
                }
            }
        }

        // online softmax
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            float mx = row_max[r];
#pragma unroll
            for (int nb = 0; nb < BN / 8; ++nb) mx = fmaxf(mx, fmaxf(acc_s[nb][2 * r], acc_s[nb][2 * r + 1]));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
            const float mref = (mx == -INFINITY) ? 0.f : mx;
            const float corr = exp2f((row_max[r] - mref) * sl2);  // row_max = -inf -> 0
            row_max[r] = mx;
            float s = 0.f;
#pragma unroll
            for (int nb = 0; nb < BN / 8; ++nb) {
                const float p0 = exp2f((acc_s[nb][2 * r] - mref) * sl2);
                const float p1 = exp2f((acc_s[nb][2 * r + 1] - mref) * sl2);
                acc_s[nb][2 * r] = p0;
                acc_s[nb][2 * r + 1] = p1;
                s += p0 + p1;
            }
            row_sum[r] = row_sum[r] * corr + s;
#pragma unroll
            for (int nb = 0; nb < NB_D; ++nb) {
                acc_o[nb][2 * r] *= corr;
                acc_o[nb][2 * r + 1] *= corr;
            }
        }

        if (p.drop_threshold) {
            // the normaliser above keeps every probability; only the product with V sees the dropped ones as zero
#pragma unroll
            for (int nb = 0; nb < BN / 8; ++nb) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int col = j * BN + nb * 8 + (lane & 3) * 2 + (e & 1);
                    const int row = r_lo + (e >> 1) * 8;
                    if (!dropout_keep(p, h, si.qb + row, si.kb + col)) acc_s[nb][e] = 0.f;
                }
            }
        }

        // O += P V
#pragma unroll
        for (int ks = 0; ks < BN / 16; ++ks) {
            uint32_t a[4];
            a[0] = pack_bf16(acc_s[2 * ks][0], acc_s[2 * ks][1]);
            a[1] = pack_bf16(acc_s[2 * ks][2], acc_s[2 * ks][3]);
            a[2] = pack_bf16(acc_s[2 * ks + 1][0], acc_s[2 * ks + 1][1]);
            a[3] = pack_bf16(acc_s[2 * ks + 1][2], acc_s[2 * ks + 1][3]);
#pragma unroll
            for (int nc = 0; nc < NB_D; nc += 2) {
                uint32_t b[4];
                load_b_frag_kn<D>(sV, ks * 16, nc, b);
                mma16816(acc_o[nc], a, b[0], b[1]);
                mma16816(acc_o[nc + 1], a, b[2], b[3]);
            }
        }
        __syncthreads();  // all warps are done with this K/V buffer before it is refilled
    }
    if (nblocks == 0) cp_async_wait<0>();

    // epilogue
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        float s = row_sum[r];
        s += __shfl_xor_sync(0xffffffffu, s, 1);
        s += __shfl_xor_sync(0xffffffffu, s, 2);
        row_sum[r] = s;
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int row = r_lo + r * 8;
        if (row >= si.ql) continue;
        const float inv = (row_sum[r] > 0.f ? 1.f / row_sum[r] : 0.f) * (p.drop_threshold ? p.keep_scale : 1.f);
        __nv_bfloat16* og = p.o + static_cast<size_t>(si.qb + row) * p.o_tstride + static_cast<size_t>(h) * D;
#pragma unroll
        for (int nb = 0; nb < NB_D; ++nb) {
            const uint32_t v = pack_bf16(acc_o[nb][2 * r] * inv, acc_o[nb][2 * r + 1] * inv);
            *reinterpret_cast<uint32_t*>(og + nb * 8 + (lane & 3) * 2) = v;
        }
        if ((lane & 3) == 0) {
            const float lse = row_sum[r] > 0.f ? row_max[r] * p.scale + logf(row_sum[r]) : -INFINITY;
            p.lse[static_cast<size_t>(h) * p.total_q + si.qb + row] = lse;
        }
    }
}

// delta[h, t] = sum_d dO[t, h, d] * O[t, h, d]; one warp per (t, h).
template <int D>
__global__ void attn_delta_kernel(const AttnParams p) {
    const size_t w = (blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    const size_t total = static_cast<size_t>(p.total_q) * p.H;
    if (w >= total) return;
    const size_t t = w / p.H;
    const int h = static_cast<int>(w % p.H);
    const __nv_bfloat16* o = p.o + t * p.o_tstride + static_cast<size_t>(h) * D;
    const __nv_bfloat16* d = p.dout + t * p.do_tstride + static_cast<size_t>(h) * D;
    float acc = 0.f;
    for (int i = lane * 2; i < D; i += 64) {
        const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(o + i));
        const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(d + i));
        acc += a.x * b.x + a.y * b.y;
    }
    acc = warp_sum(acc);
    if (lane == 0) p.delta[static_cast<size_t>(h) * p.total_q + t] = acc;
}

// ------------------------------------------------------------ backward: dK,dV
// grid (kv blocks, seqs, Hkv); 128 threads; CTA owns 64 K/V rows (16 per warp),
// loops over the G query heads of the group and over 64-row query blocks.
template <int D>
__global__ void __launch_bounds__(128, 1) attn_bwd_dkv_kernel(const AttnParams p) {
    constexpr int BN = 64, BM = 64, THREADS = 128;
    constexpr int KS = D / 16, NB_D = D / 8;
    extern __shared__ __align__(128) uint8_t smem_raw[];
    const uint32_t sK = smem_u32(smem_raw);
    const uint32_t sV = sK + BN * D * 2;
    const uint32_t sQ0 = sV + BN * D * 2;
    const uint32_t sDO0 = sQ0 + 2 * BM * D * 2;
    float* sLse = reinterpret_cast<float*>(smem_raw + (2 * BN + 4 * BM) * D * 2);  // [2][BM]
    float* sDelta = sLse + 2 * BM;                                                  // [2][BM]

    const SeqInfo si = seq_info(p, blockIdx.y);
    const int n0 = blockIdx.x * BN;
    if (n0 >= si.kl) return;
    const int hk = blockIdx.z;
    const int G = p.H / p.Hkv;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    const __nv_bfloat16* kg = p.k + static_cast<size_t>(si.kb) * p.k_tstride + static_cast<size_t>(hk) * D;
    const __nv_bfloat16* vg = p.v + static_cast<size_t>(si.kb) * p.v_tstride + static_cast<size_t>(hk) * D;

    // first query block that can see key n0 (causal): q >= n0 - shift
    int mb_start = 0;
    if (p.causal) mb_start = max(0, n0 - si.shift) / BM;
    const int mb_end = (si.ql + BM - 1) / BM;
    const int iters_per_head = max(0, mb_end - mb_start);
    const int total_iters = iters_per_head * G;

    auto issue_q = [&](int it, int buf) {
        const int g = it / iters_per_head;
        const int mb = mb_start + it % iters_per_head;
        const int h = hk * G + g;
        const __nv_bfloat16* qg = p.q + static_cast<size_t>(si.qb) * p.q_tstride + static_cast<size_t>(h) * D;
        const __nv_bfloat16* dog = p.dout + static_cast<size_t>(si.qb) * p.do_tstride + static_cast<size_t>(h) * D;
        load_tile<D, BM, THREADS>(sQ0 + buf * BM * D * 2, qg, p.q_tstride, mb * BM, si.ql);
        load_tile<D, BM, THREADS>(sDO0 + buf * BM * D * 2, dog, p.do_tstride, mb * BM, si.ql);
        if (threadIdx.x < BM) {
            const int row = mb * BM + threadIdx.x;
            const bool ok = row < si.ql;
            const size_t idx = static_cast<size_t>(h) * p.total_q + si.qb + (ok ? row : 0);
            sLse[buf * BM + threadIdx.x] = ok ? p.lse[idx] : INFINITY;  // +inf -> probability 0
            sDelta[buf * BM + threadIdx.x] = ok ? p.delta[idx] : 0.f;
        }
    };

    load_tile<D, BN, THREADS>(sK, kg, p.k_tstride, n0, si.kl);
    load_tile<D, BN, THREADS>(sV, vg, p.v_tstride, n0, si.kl);
    if (total_iters > 0) issue_q(0, 0);
    cp_async_commit();

    float acc_dk[NB_D][4], acc_dv[NB_D][4];
#pragma unroll
    for (int i = 0; i < NB_D; ++i) {
        acc_dk[i][0] = acc_dk[i][1] = acc_dk[i][2] = acc_dk[i][3] = 0.f;
        acc_dv[i][0] = acc_dv[i][1] = acc_dv[i][2] = acc_dv[i][3] = 0.f;
    }
    const float sl2 = p.scale * LOG2E;
    const int key_lo = n0 + warp * 16 + (lane >> 2);  // key row of c0/c1; c2/c3 is +8

    for (int it = 0; it < total_iters; ++it) {
        const int buf = it & 1;
        if (it + 1 < total_iters) {
            issue_q(it + 1, buf ^ 1);
            cp_async_commit();
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        const uint32_t sQ = sQ0 + buf * BM * D * 2;
        const uint32_t sDO = sDO0 + buf * BM * D * 2;
        const float* lse = sLse + buf * BM;
        const float* delta = sDelta + buf * BM;
        const int mb = mb_start + it % iters_per_head;
        const int q0 = mb * BM;
        const int h_cur = hk * G + it / iters_per_head;

        // S^T = K Q^T  (16 keys x 64 queries per warp)
        float acc_s[BM / 8][4];
        float acc_dp[BM / 8][4];
#pragma unroll
        for (int i = 0; i < BM / 8; ++i) {
            acc_s[i][0] = acc_s[i][1] = acc_s[i][2] = acc_s[i][3] = 0.f;
            acc_dp[i][0] = acc_dp[i][1] = acc_dp[i][2] = acc_dp[i][3] = 0.f;
        }
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
            uint32_t ak[4], av[4];
            load_a_frag<D>(sK, warp * 16, ks, ak);
            load_a_frag<D>(sV, warp * 16, ks, av);
#pragma unroll
            for (int nb = 0; nb < BM / 16; ++nb) {
                uint32_t bq[4], bd[4];
                load_b_frag_nk<D>(sQ, nb * 16, ks, bq);
                load_b_frag_nk<D>(sDO, nb * 16, ks, bd);
                mma16816(acc_s[2 * nb], ak, bq[0], bq[1]);
                mma16816(acc_s[2 * nb + 1], ak, bq[2], bq[3]);
                mma16816(acc_dp[2 * nb], av, bd[0], bd[1]);
                mma16816(acc_dp[2 * nb + 1], av, bd[2], bd[3]);
            }
        }
        // P^T and dS^T
#pragma unroll
        for (int nb = 0; nb < BM / 8; ++nb) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int qc = nb * 8 + (lane & 3) * 2 + (e & 1);   // query column inside the block
                const int key = key_lo + (e >> 1) * 8;
                const int qrow = q0 + qc;
                const bool dead = key >= si.kl || (p.causal && key > qrow + si.shift);
                const float pr = dead ? 0.f : exp2f(acc_s[nb][e] * sl2 - lse[qc] * LOG2E);
                float m = 1.f;
                if (p.drop_threshold) m = dropout_keep(p, h_cur, si.qb + qrow, si.kb + key) ? p.keep_scale : 0.f;
                acc_s[nb][e] = pr * m;                                   // dV sees the dropped probabilities
                acc_dp[nb][e] = pr * (acc_dp[nb][e] * m - delta[qc]) * p.scale;
            }
        }
        // dV += P^T dO ; dK += dS^T Q      (k = query index)
#pragma unroll
        for (int ks = 0; ks < BM / 16; ++ks) {
            uint32_t ap[4], ads[4];
            ap[0] = pack_bf16(acc_s[2 * ks][0], acc_s[2 * ks][1]);
            ap[1] = pack_bf16(acc_s[2 * ks][2], acc_s[2 * ks][3]);
            ap[2] = pack_bf16(acc_s[2 * ks + 1][0], acc_s[2 * ks + 1][1]);
            ap[3] = pack_bf16(acc_s[2 * ks + 1][2], acc_s[2 * ks + 1][3]);
            ads[0] = pack_bf16(acc_dp[2 * ks][0], acc_dp[2 * ks][1]);
            ads[1] = pack_bf16(acc_dp[2 * ks][2], acc_dp[2 * ks][3]);
            ads[2] = pack_bf16(acc_dp[2 * ks + 1][0], acc_dp[2 * ks + 1][1]);
            ads[3] = pack_bf16(acc_dp[2 * ks + 1][2], acc_dp[2 * ks + 1][3]);
#pragma unroll
            for (int nc = 0; nc < NB_D; nc += 2) {
                uint32_t b[4];
                load_b_frag_kn<D>(sDO, ks * 16, nc, b);
                mma16816(acc_dv[nc], ap, b[0], b[1]);
                mma16816(acc_dv[nc + 1], ap, b[2], b[3]);
                load_b_frag_kn<D>(sQ, ks * 16, nc, b);
                mma16816(acc_dk[nc], ads, b[0], b[1]);
                mma16816(acc_dk[nc + 1], ads, b[2], b[3]);
            }
        }
        __syncthreads();
    }
    if (total_iters == 0) {
        cp_async_wait<0>();
    }

#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int key = key_lo + r * 8;
        if (key >= si.kl) continue;
        __nv_bfloat16* dkg = p.dk + static_cast<size_t>(si.kb + key) * p.dk_tstride + static_cast<size_t>(hk) * D;
        __nv_bfloat16* dvg = p.dv + static_cast<size_t>(si.kb + key) * p.dv_tstride + static_cast<size_t>(hk) * D;
#pragma unroll
        for (int nb = 0; nb < NB_D; ++nb) {
            const int c = nb * 8 + (lane & 3) * 2;
            *reinterpret_cast<uint32_t*>(dkg + c) = pack_bf16(acc_dk[nb][2 * r], acc_dk[nb][2 * r + 1]);
            *reinterpret_cast<uint32_t*>(dvg + c) = pack_bf16(acc_dv[nb][2 * r], acc_dv[nb][2 * r + 1]);
        }
    }
}

// --------------------------------------------------------------- backward: dQ
// grid (q blocks, seqs, H); 256 threads; CTA owns 128 query rows (16 per warp).
template <int D>
__global__ void __launch_bounds__(256, 1) attn_bwd_dq_kernel(const AttnParams p) {
    constexpr int BM = 128, BN = 64, THREADS = 256;
    constexpr int KS = D / 16, NB_D = D / 8;
    extern __shared__ __align__(128) uint8_t smem_raw[];
    const uint32_t sQ = smem_u32(smem_raw);
    const uint32_t sDO = sQ + BM * D * 2;
    const uint32_t sK0 = sDO + BM * D * 2;
    const uint32_t sV0 = sK0 + 2 * BN * D * 2;

    const SeqInfo si = seq_info(p, blockIdx.y);
    const int m0 = blockIdx.x * BM;
    if (m0 >= si.ql) return;
    const int h = blockIdx.z;
    const int hk = h / (p.H / p.Hkv);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    const __nv_bfloat16* qg = p.q + static_cast<size_t>(si.qb) * p.q_tstride + static_cast<size_t>(h) * D;
    const __nv_bfloat16* dog = p.dout + static_cast<size_t>(si.qb) * p.do_tstride + static_cast<size_t>(h) * D;
    const __nv_bfloat16* kg = p.k + static_cast<size_t>(si.kb) * p.k_tstride + static_cast<size_t>(hk) * D;
    const __nv_bfloat16* vg = p.v + static_cast<size_t>(si.kb) * p.v_tstride + static_cast<size_t>(hk) * D;

    int n_end = si.kl;
    if (p.causal) n_end = min(si.kl, m0 + BM + si.shift);
    const int nblocks = n_end > 0 ? (n_end + BN - 1) / BN : 0;

    load_tile<D, BM, THREADS>(sQ, qg, p.q_tstride, m0, si.ql);
    load_tile<D, BM, THREADS>(sDO, dog, p.do_tstride, m0, si.ql);
    if (nblocks > 0) {
        load_tile<D, BN, THREADS>(sK0, kg, p.k_tstride, 0, si.kl);
        load_tile<D, BN, THREADS>(sV0, vg, p.v_tstride, 0, si.kl);
    }
    cp_async_commit();

    const int r_lo = m0 + warp * 16 + (lane >> 2);
    float lse_r[2], delta_r[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int row = r_lo + r * 8;
        const bool ok = row < si.ql;
        const size_t idx = static_cast<size_t>(h) * p.total_q + si.qb + (ok ? row : 0);
        lse_r[r] = ok ? p.lse[idx] : INFINITY;
        delta_r[r] = ok ? p.delta[idx] : 0.f;
    }

    float acc_dq[NB_D][4];
#pragma unroll
    for (int i = 0; i < NB_D; ++i) acc_dq[i][0] = acc_dq[i][1] = acc_dq[i][2] = acc_dq[i][3] = 0.f;
    const float sl2 = p.scale * LOG2E;

    for (int j = 0; j < nblocks; ++j) {
        const int buf = j & 1;
        const uint32_t sK = sK0 + buf * BN * D * 2;
        const uint32_t sV = sV0 + buf * BN * D * 2;
        if (j + 1 < nblocks) {
            load_tile<D, BN, THREADS>(sK0 + (buf ^ 1) * BN * D * 2, kg, p.k_tstride, (j + 1) * BN, si.kl);
            load_tile<D, BN, THREADS>(sV0 + (buf ^ 1) * BN * D * 2, vg, p.v_tstride, (j + 1) * BN, si.kl);
            cp_async_commit();
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();

        float acc_s[BN / 8][4], acc_dp[BN / 8][4];
#pragma unroll
        for (int i = 0; i < BN / 8; ++i) {
            acc_s[i][0] = acc_s[i][1] = acc_s[i][2] = acc_s[i][3] = 0.f;
            acc_dp[i][0] = acc_dp[i][1] = acc_dp[i][2] = acc_dp[i][3] = 0.f;
        }
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
            uint32_t aq[4], ad[4];
            load_a_frag<D>(sQ, warp * 16, ks, aq);
            load_a_frag<D>(sDO, warp * 16, ks, ad);
#pragma unroll
            for (int nb = 0; nb < BN / 16; ++nb) {
                uint32_t bk[4], bv[4];
                load_b_frag_nk<D>(sK, nb * 16, ks, bk);
                load_b_frag_nk<D>(sV, nb * 16, ks, bv);
                mma16816(acc_s[2 * nb], aq, bk[0], bk[1]);
                mma16816(acc_s[2 * nb + 1], aq, bk[2], bk[3]);
                mma16816(acc_dp[2 * nb], ad, bv[0], bv[1]);
                mma16816(acc_dp[2 * nb + 1], ad, bv[2], bv[3]);
            }
        }
        const int n0 = j * BN;
#pragma unroll
        for (int nb = 0; nb < BN / 8; ++nb) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int col = n0 + nb * 8 + (lane & 3) * 2 + (e & 1);
                const int r = e >> 1;
                const int row = r_lo + r * 8;
                const bool dead = col >= si.kl || (p.causal && col > row + si.shift);
                const float pr = dead ? 0.f : exp2f(acc_s[nb][e] * sl2 - lse_r[r] * LOG2E);
                float m = 1.f;
                if (p.drop_threshold) m = dropout_keep(p, h, si.qb + row, si.kb + col) ? p.keep_scale : 0.f;
                acc_dp[nb][e] = pr * (acc_dp[nb][e] * m - delta_r[r]) * p.scale;
            }
        }
        // dQ += dS K   (k = key index)
#pragma unroll
        for (int ks = 0; ks < BN / 16; ++ks) {
            uint32_t a[4];
            a[0] = pack_bf16(acc_dp[2 * ks][0], acc_dp[2 * ks][1]);
            a[1] = pack_bf16(acc_dp[2 * ks][2], acc_dp[2 * ks][3]);
            a[2] = pack_bf16(acc_dp[2 * ks + 1][0], acc_dp[2 * ks + 1][1]);
            a[3] = pack_bf16(acc_dp[2 * ks + 1][2], acc_dp[2 * ks + 1][3]);
#pragma unroll
            for (int nc = 0; nc < NB_D; nc += 2) {
                uint32_t b[4];
                load_b_frag_kn<D>(sK, ks * 16, nc, b);
                mma16816(acc_dq[nc], a, b[0], b[1]);
                mma16816(acc_dq[nc + 1], a, b[2], b[3]);
            }
        }
        __syncthreads();
    }
    if (nblocks == 0) cp_async_wait<0>();

#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int row = r_lo + r * 8;
        if (row >= si.ql) continue;
        __nv_bfloat16* dqg = p.dq + static_cast<size_t>(si.qb + row) * p.dq_tstride + static_cast<size_t>(h) * D;
#pragma unroll
        for (int nb = 0; nb < NB_D; ++nb) {
            *reinterpret_cast<uint32_t*>(dqg + nb * 8 + (lane & 3) * 2) =
                pack_bf16(acc_dq[nb][2 * r], acc_dq[nb][2 * r + 1]);
        }
    }
}

template <typename K>
cudaError_t set_smem(K kern, int bytes) {
    return cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
}

}  // namespace

const char* attn_forward(const AttnParams& p, cudaStream_t st) {
    if (p.num_seqs == 0 || p.total_q == 0) return nullptr;
    const dim3 grid((p.max_q + 127) / 128, p.num_seqs, p.H);
    cudaError_t e;
    if (p.D == 128) {
        constexpr int smem = (128 + 4 * 64) * 128 * 2;
        e = set_smem(attn_fwd_kernel<128>, smem);
        if (e != cudaSuccess) return cudaGetErrorString(e);
        attn_fwd_kernel<128><<<grid, 256, smem, st>>>(p);
    } else if (p.D == 64) {
        constexpr int smem = (128 + 4 * 64) * 64 * 2;
        e = set_smem(attn_fwd_kernel<64>, smem);
        if (e != cudaSuccess) return cudaGetErrorString(e);
        attn_fwd_kernel<64><<<grid, 256, smem, st>>>(p);
    } else {
        return "attention: head_dim must be 64 or 128";
    }
    e = cudaGetLastError();
    return e == cudaSuccess ? nullptr : cudaGetErrorString(e);
}

const char* attn_delta(const AttnParams& p, cudaStream_t st) {
    if (p.num_seqs == 0 || p.total_q == 0) return nullptr;
    const size_t warps = static_cast<size_t>(p.total_q) * p.H;
    const int dgrid = static_cast<int>((warps * 32 + 255) / 256);
    if (p.D == 128) attn_delta_kernel<128><<<dgrid, 256, 0, st>>>(p);
    else if (p.D == 64) attn_delta_kernel<64><<<dgrid, 256, 0, st>>>(p);
    else return "attention: head_dim must be 64 or 128";
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? nullptr : cudaGetErrorString(e);
}

const char* attn_backward(const AttnParams& p, cudaStream_t st) {
    if (p.num_seqs == 0 || p.total_q == 0) return nullptr;
    cudaError_t e;
    const size_t warps = static_cast<size_t>(p.total_q) * p.H;
    const int dgrid = static_cast<int>((warps * 32 + 255) / 256);
    const dim3 grid_kv((p.max_k + 63) / 64, p.num_seqs, p.Hkv);
    const dim3 grid_q((p.max_q + 127) / 128, p.num_seqs, p.H);
    if (p.D == 128) {
        constexpr int smem_kv = (2 * 64 + 4 * 64) * 128 * 2 + 4 * 64 * 4;
        constexpr int smem_q = (2 * 128 + 4 * 64) * 128 * 2;
        attn_delta_kernel<128><<<dgrid, 256, 0, st>>>(p);
        e = set_smem(attn_bwd_dkv_kernel<128>, smem_kv);
        if (e != cudaSuccess) return cudaGetErrorString(e);
        attn_bwd_dkv_kernel<128><<<grid_kv, 128, smem_kv, st>>>(p);
        e = set_smem(attn_bwd_dq_kernel<128>, smem_q);
        if (e != cudaSuccess) return cudaGetErrorString(e);
        attn_bwd_dq_kernel<128><<<grid_q, 256, smem_q, st>>>(p);
    } else if (p.D == 64) {
        constexpr int smem_kv = (2 * 64 + 4 * 64) * 64 * 2 + 4 * 64 * 4;
        constexpr int smem_q = (2 * 128 + 4 * 64) * 64 * 2;
        attn_delta_kernel<64><<<dgrid, 256, 0, st>>>(p);
        e = set_smem(attn_bwd_dkv_kernel<64>, smem_kv);
        if (e != cudaSuccess) return cudaGetErrorString(e);
        attn_bwd_dkv_kernel<64><<<grid_kv, 128, smem_kv, st>>>(p);
        e = set_smem(attn_bwd_dq_kernel<64>, smem_q);
        if (e != cudaSuccess) return cudaGetErrorString(e);
        attn_bwd_dq_kernel<64><<<grid_q, 256, smem_q, st>>>(p);
    } else {
        return "attention: head_dim must be 64 or 128";
    }
    e = cudaGetLastError();
    return e == cudaSuccess ? nullptr : cudaGetErrorString(e);
}

}  // namespace fs2
