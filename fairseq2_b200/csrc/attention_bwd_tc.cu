// Flash-attention backward on the 5th-generation tensor cores (sm_100a), head_dim 128.
//
// Two deterministic kernels (no atomics), both built like the forward kernel: TMA -> 128B-swizzled
// shared memory -> tcgen05.mma with accumulators in TMEM -> tcgen05.ld; 320 threads = TMA producer
// warp, MMA issuer warp and two compute warpgroups. Thread t of a warpgroup owns TMEM lane t; the
// two warpgroups split the 64 score columns of a tile between them (and the accumulator columns in
// the epilogue), so every scheduler has two compute warps whose exp2 / tcgen05.ld latencies overlap.
//
// dQ kernel: a CTA owns 128 query rows of one head. Q and dO are copied once into tensor memory and
//   are the A operands of every score MMA from there; per 64-row K/V tile the
//   issuer computes S = Q K^T and dP = dO V^T into a double-buffered TMEM pair, the compute warps
//   turn them into dS = P * (dP - delta) (P = exp2(S * scale - lse)), written back as bf16 over the
//   dP columns they came from, and dQ += dS K accumulates in TMEM with dS read as the A operand
//   straight from tensor memory (K read as an MN-major B operand).
//
// dK/dV kernel: a CTA owns 128 key/value rows of one KV head. K and V stay resident; it walks the
//   query heads of the group and their 64-row query tiles, computing S^T = K Q^T and dP^T = V dO^T,
//   then P^T and dS^T as bf16 written over the score columns, and dV += P^T dO, dK += dS^T Q
//   accumulate in TMEM over the whole walk (A operands from tensor memory, Q and dO read as
//   MN-major B operands).
//
// Operands in tensor memory matter because these kernels are bound by the rate at which the tensor
// core reads operands from shared memory: measured here, an MMA costs max(math, operand bytes / 64 B
// per cycle), so a 128 x 64 x 16 MMA with both operands in shared memory (6 KB) takes 96 cycles for
// 32 cycles of math, and 32 with A in tensor memory. The
// tensor pipe executes the MMAs of the issuing thread in order, so the scores of tile i+2 cannot
// overwrite a buffer before the accumulating MMAs of tile i, issued earlier, have read it.
//
// The softmax scale is applied once to the dQ / dK accumulators in the epilogue.
// Every barrier wait is bounded; a wait that gives up records a code in the host-visible status
// word, raises a CTA-wide abort flag and every role falls through to the teardown that frees TMEM.

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdint>

#include "attention.h"
#include "attention_tc.cuh"
#include "common.cuh"

namespace fs2 {

namespace {

using namespace tc;

constexpr int HD = 128;
constexpr int BOX128 = 128 * 64 * 2;     // [128 rows][64 cols] bf16 box
constexpr int BOX64 = 64 * 64 * 2;       // [64 rows][64 cols] bf16 box
constexpr int BIG_TILE = 2 * BOX128;     // [128][128]
constexpr int SMALL_TILE = 2 * BOX64;    // [64][128]
constexpr int BWD_WGS = 2;                       // compute warpgroups
constexpr int BWD_THREADS = 64 + 128 * BWD_WGS;
constexpr uint32_t BWD_TMEM_COLS = 512;

// Shared memory: two resident [128][128] tiles and a ring of stages (each two [64][128] tiles).
// A stage is released only after the accumulating MMA that reads it has completed, so the ring must be deep
// enough for the TMA loads to run ahead of that point.
constexpr int STAGE_BYTES = 2 * SMALL_TILE;
constexpr int OFF_RES0 = 0;
constexpr int OFF_RES1 = OFF_RES0 + BIG_TILE;
constexpr int OFF_STG = OFF_RES1 + BIG_TILE;
constexpr int DQ_NSTG = 5, KV_NSTG = 4;
constexpr int MAX_NSTG = 6;
constexpr int DQ_OFF_BAR = OFF_STG + DQ_NSTG * STAGE_BYTES;
constexpr int DQ_SMEM_BYTES = DQ_OFF_BAR + 256 + 1024;
// dK/dV kernel: per compute warp, -lse * log2(e) and delta of its 32 query columns, double-buffered
constexpr int KV_OFF_VEC = OFF_STG + KV_NSTG * STAGE_BYTES;
constexpr int KV_VEC_BYTES = 8 * 2 * 2 * 32 * 4;
constexpr int KV_OFF_BAR = KV_OFF_VEC + KV_VEC_BYTES;
constexpr int KV_SMEM_BYTES = KV_OFF_BAR + 256 + 1024;
static_assert(DQ_SMEM_BYTES <= 232448 && KV_SMEM_BYTES <= 232448, "shared memory budget of one CTA exceeded");

enum : int {
    B_RES_FULL = 0,
    B_STG_FULL = 1,                        // [MAX_NSTG]
    B_STG_EMPTY = B_STG_FULL + MAX_NSTG,   // [MAX_NSTG]
    B_ACC_FULL = B_STG_EMPTY + MAX_NSTG,   // [2] score pair in TMEM ready
    B_OP_FULL = B_ACC_FULL + 2,            // [2] bf16 operand(s) written over the score pair
    B_DONE = B_OP_FULL + 2,
    B_RESA_FULL = B_DONE + 1,              // resident A operands copied to tensor memory
    B_NUM = B_RESA_FULL + 1
};
static_assert(8 * B_NUM + 16 <= 256, "barrier area");

struct Ctx {
    uint32_t base;
    uint32_t bar_base;
    uint32_t tmem_base;
    volatile int* abort_flag;
    int* status;
    __device__ __forceinline__ uint32_t bar(int slot) const { return bar_base + 8u * static_cast<uint32_t>(slot); }
    __device__ __forceinline__ bool wait(int slot, uint32_t parity) const {
        return mbar_wait_bounded(bar(slot), parity, abort_flag, WAIT_NS);
    }
    __device__ __forceinline__ void fail(int code) const {
        if (!*abort_flag) report_status(status, kStatusTimeout | (code << 8));
        *abort_flag = 1;
    }
};

__device__ __forceinline__ void bwd_setup(Ctx& c, uint8_t* smem_raw, int* status, int off_bar) {
    const uint32_t raw = smem_u32(smem_raw);
    c.base = (raw + 1023u) & ~1023u;
    uint8_t* smem = smem_raw + (c.base - raw);
    uint8_t* bar_ptr = smem + off_bar;
    c.bar_base = smem_u32(bar_ptr);
    c.status = status;
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(bar_ptr + 8 * B_NUM);
    c.abort_flag = reinterpret_cast<volatile int*>(bar_ptr + 8 * B_NUM + 8);
    const int warp = threadIdx.x >> 5;
    if (threadIdx.x == 0) {
        mbar_init(c.bar(B_RES_FULL), 1);
        mbar_init(c.bar(B_DONE), 1);
        mbar_init(c.bar(B_RESA_FULL), 128 * BWD_WGS);
        for (int s = 0; s < MAX_NSTG; ++s) {
            mbar_init(c.bar(B_STG_FULL + s), 1);
            mbar_init(c.bar(B_STG_EMPTY + s), 1);
        }
        for (int s = 0; s < 2; ++s) {
            mbar_init(c.bar(B_ACC_FULL + s), 1);
            mbar_init(c.bar(B_OP_FULL + s), 128 * BWD_WGS);
        }
        *c.abort_flag = 0;
        fence_barrier_init();
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), BWD_TMEM_COLS);
        tmem_relinquish();
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    c.tmem_base = *tmem_slot;
}

__device__ __forceinline__ void bwd_teardown(const Ctx& c) {
    __syncthreads();
    if (*c.abort_flag) {
        const uint64_t t0 = global_timer_ns();
        while (global_timer_ns() - t0 < 200000ull) __nanosleep(1000);
        __syncthreads();
    }
    tcgen05_fence_after();
    if ((threadIdx.x >> 5) == 1) tmem_dealloc(c.tmem_base, BWD_TMEM_COLS);
}

// D[128 x 64] = A[128 x 128 (K-major, two 64-col boxes of 128 rows)] * B[64 x 128 (K-major, two boxes of 64 rows)]^T
__device__ __forceinline__ void mma_scores(uint32_t d_tmem, uint32_t a_s, uint32_t b_s, uint32_t idesc) {
#pragma unroll
    for (int k = 0; k < HD / 16; ++k) {
        const uint64_t da = make_smem_desc(a_s + (k >> 2) * BOX128 + (k & 3) * 32, 16, 1024);
        const uint64_t db = make_smem_desc(b_s + (k >> 2) * BOX64 + (k & 3) * 32, 16, 1024);
        umma_bf16(d_tmem, da, db, idesc, k > 0 ? 1u : 0u);
    }
}

// Same with A[128 x 128] as bf16 in tensor memory (64 columns from `a_tmem`).
__device__ __forceinline__ void mma_scores_ts(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_s, uint32_t idesc) {
#pragma unroll
    for (int k = 0; k < HD / 16; ++k) {
        const uint64_t db = make_smem_desc(b_s + (k >> 2) * BOX64 + (k & 3) * 32, 16, 1024);
        umma_bf16_ts(d_tmem, a_tmem + static_cast<uint32_t>(k * 8), db, idesc, k > 0 ? 1u : 0u);
    }
}

// Copies row `row` of a 128B-swizzled [128][128] bf16 tile (two [128][64] boxes) from shared memory into the 64
// columns from `taddr` of this thread's TMEM lane: element k of the row lands in column k / 2, half k % 2.
__device__ __forceinline__ void copy_row_to_tmem(uint32_t tile_s, int row, uint32_t taddr) {
#pragma unroll
    for (int bx = 0; bx < 2; ++bx) {
#pragma unroll
        for (int hf = 0; hf < 2; ++hf) {
            uint32_t r[16];
#pragma unroll
            for (int c4 = 0; c4 < 4; ++c4) {
                const uint32_t chunk = static_cast<uint32_t>(hf * 4 + c4);
                const uint32_t src = tile_s + static_cast<uint32_t>(bx) * BOX128 + static_cast<uint32_t>(row) * 128u +
                                     (((chunk ^ static_cast<uint32_t>(row & 7)) & 7u) << 4);
                asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                             : "=r"(r[4 * c4]), "=r"(r[4 * c4 + 1]), "=r"(r[4 * c4 + 2]), "=r"(r[4 * c4 + 3])
                             : "r"(src));
            }
            tmem_st_32x16(taddr + static_cast<uint32_t>(bx * 32 + hf * 16), r);
        }
    }
}

// D[128 x 128] (+)= A[128 x 64] * B[64 x 128 (row-major [64][128] tile read MN-major)]. A is bf16 in tensor memory:
// warpgroup g wrote K elements [32 g, 32 g + 32) as 16 packed columns starting at column 32 g of `a_tmem`.
__device__ __forceinline__ void mma_accum(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_s, uint32_t idesc, bool first) {
#pragma unroll
    for (int k = 0; k < 64 / 16; ++k) {
        const uint32_t ta = a_tmem + static_cast<uint32_t>((k >> 1) * 32 + (k & 1) * 8);
        const uint64_t db = make_smem_desc(b_s + k * 16 * 128, BOX64, 1024);
        umma_bf16_ts(d_tmem, ta, db, idesc, (first && k == 0) ? 0u : 1u);
    }
}

// Packs 32 floats to bf16 pairs and writes them as 16 columns of this thread's TMEM lane.
__device__ __forceinline__ void store_operand(uint32_t taddr, const float* e) {
    uint32_t r[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) r[j] = pack2_bf16(e[2 * j], e[2 * j + 1]);
    tmem_st_32x16(taddr, r);
}

// Epilogue: TMEM accumulator [128 lanes][128 cols] * mul -> bf16 row in global memory.
// Chunks [c0, c1) of 32 columns each.
__device__ __forceinline__ void store_acc_row(uint32_t t_lane_col, float mul, __nv_bfloat16* dst, bool valid,
                                              int c0 = 0, int c1 = 4) {
    for (int c = c0; c < c1; ++c) {
        uint32_t v[32];
        tmem_ld_32x32(t_lane_col + c * 32, v);
        tmem_ld_wait();
        if (valid) {
#pragma unroll
            for (int g = 0; g < 4; ++g) {
                uint4 w;
                w.x = pack2_bf16(__uint_as_float(v[8 * g]) * mul, __uint_as_float(v[8 * g + 1]) * mul);
                w.y = pack2_bf16(__uint_as_float(v[8 * g + 2]) * mul, __uint_as_float(v[8 * g + 3]) * mul);
                w.z = pack2_bf16(__uint_as_float(v[8 * g + 4]) * mul, __uint_as_float(v[8 * g + 5]) * mul);
                w.w = pack2_bf16(__uint_as_float(v[8 * g + 6]) * mul, __uint_as_float(v[8 * g + 7]) * mul);
                *reinterpret_cast<uint4*>(dst + c * 32 + g * 8) = w;
            }
        }
    }
}

// ============================================================================ dQ kernel
// grid (H, seqs, q tiles of 128): heads fastest, so the long query tiles of every head are scheduled first
__global__ void __launch_bounds__(BWD_THREADS, 1)
attn_bwd_dq_tc_kernel(const __grid_constant__ CUtensorMap tma_q, const __grid_constant__ CUtensorMap tma_do,
                      const __grid_constant__ CUtensorMap tma_k, const __grid_constant__ CUtensorMap tma_v,
                      const AttnParams p, int* status) {
    const int seq = blockIdx.y, h = blockIdx.x;
    const int q_len = p.q_lens[seq], k_len = p.k_lens[seq];
    const int qblk = static_cast<int>(gridDim.z) - 1 - static_cast<int>(blockIdx.z);
    const int q0 = qblk * 128;
    if (q0 >= q_len) return;
    const int q_begin = p.q_begins[seq], k_begin = p.k_begins[seq];
    const int shift = k_len - q_len;
    const int q_last = min(q0 + 128, q_len) - 1;
    const int kv_hi = p.causal ? min(k_len, q_last + shift + 1) : k_len;
    const bool windowed = p.causal && p.window > 0;
    const int it0 = windowed ? max(0, q0 + shift - p.window + 1) / 64 : 0;     // first key tile inside the window
    const int n_iter = kv_hi > 0 ? max(0, (kv_hi + 63) / 64 - it0) : 0;
    const int kvh = h / (p.H / p.Hkv);
    const int warp = __shfl_sync(0xffffffffu, threadIdx.x >> 5, 0), lane = threadIdx.x & 31;   // warp-uniform for the compiler

    if (n_iter == 0) {
        // no visible key: the gradient of these query rows is zero
        if (warp >= 2 && warp < 6) {
            const int row = (warp & 3) * 32 + lane;
            if (q0 + row < q_len) {
                __nv_bfloat16* dst = p.dq + static_cast<size_t>(q_begin + q0 + row) * p.dq_tstride + static_cast<size_t>(h) * HD;
                for (int c = 0; c < HD / 8; ++c) *reinterpret_cast<uint4*>(dst + 8 * c) = make_uint4(0, 0, 0, 0);
            }
        }
        return;
    }

    extern __shared__ uint8_t smem_raw[];
    Ctx c;
    bwd_setup(c, smem_raw, status, DQ_OFF_BAR);
    if (threadIdx.x == 0) {
        prefetch_tmap(&tma_q);
        prefetch_tmap(&tma_do);
        prefetch_tmap(&tma_k);
        prefetch_tmap(&tma_v);
    }
    const uint32_t q_s = c.base + OFF_RES0, do_s = c.base + OFF_RES1;

    if (warp == 0) {
        if (lane == 0) {
            const uint32_t rb = c.bar(B_RES_FULL);
            mbar_arrive_expect_tx(rb, 2 * BIG_TILE);
            tma_load_2d(q_s, &tma_q, rb, h * HD, q_begin + q0);
            tma_load_2d(q_s + BOX128, &tma_q, rb, h * HD + 64, q_begin + q0);
            tma_load_2d(do_s, &tma_do, rb, h * HD, q_begin + q0);
            tma_load_2d(do_s + BOX128, &tma_do, rb, h * HD + 64, q_begin + q0);
            for (int i = 0; i < n_iter; ++i) {
                const int st = i % DQ_NSTG;
                const uint32_t ph = static_cast<uint32_t>(i / DQ_NSTG) & 1u;
                if (!c.wait(B_STG_EMPTY + st, ph ^ 1u)) {
                    c.fail(0x41);
                    break;
                }
                const uint32_t fb = c.bar(B_STG_FULL + st);
                const uint32_t k_s = c.base + OFF_STG + st * STAGE_BYTES, v_s = k_s + SMALL_TILE;
                const int row = k_begin + (it0 + i) * 64;
                mbar_arrive_expect_tx(fb, 2 * SMALL_TILE);
                tma_load_2d(k_s, &tma_k, fb, kvh * HD, row);
                tma_load_2d(k_s + BOX64, &tma_k, fb, kvh * HD + 64, row);
                tma_load_2d(v_s, &tma_v, fb, kvh * HD, row);
                tma_load_2d(v_s + BOX64, &tma_v, fb, kvh * HD + 64, row);
            }
        }
    } else if (warp == 1) {
        // The whole warp runs the issue loop converged; only the tcgen05 instructions are predicated on one lane.
        const bool leader = elect_one();
        const uint32_t tmem = __shfl_sync(0xffffffffu, c.tmem_base, 0);
        const uint32_t id_s = make_idesc_bf16(128, 64, false);
        const uint32_t id_acc = make_idesc_bf16(128, 128, true);
        bool ok = c.wait(B_RESA_FULL, 0u);     // Q and dO are in tensor memory (columns 384.. and 448..)
        if (!ok && leader) c.fail(0x42);
        tcgen05_fence_after();
        const uint32_t q_t = tmem + 384u, do_t = tmem + 448u;
        auto accumulate = [&](int j) -> bool {     // dQ += dS_j K_j
            const int b = j & 1, st = j % DQ_NSTG;
            if (!c.wait(B_OP_FULL + b, static_cast<uint32_t>(j >> 1) & 1u)) return false;
            tcgen05_fence_after();
            const uint32_t k_s = c.base + OFF_STG + st * STAGE_BYTES;
            if (leader) {
                mma_accum(tmem + 256u, tmem + static_cast<uint32_t>(b * 128 + 64), k_s, id_acc, j == 0);
                umma_commit(c.bar(B_STG_EMPTY + st));
            }
            return true;
        };
        for (int i = 0; i < n_iter && ok; ++i) {
            const int b = i & 1, st = i % DQ_NSTG;
            // the score pair b is free: the MMAs that read tile i - 2 from it were issued before this point
            ok = c.wait(B_STG_FULL + st, static_cast<uint32_t>(i / DQ_NSTG) & 1u);
            if (!ok) {
                if (leader) c.fail(0x43);
                break;
            }
            tcgen05_fence_after();
            const uint32_t k_s = c.base + OFF_STG + st * STAGE_BYTES, v_s = k_s + SMALL_TILE;
            if (leader) {
                mma_scores_ts(tmem + static_cast<uint32_t>(b * 128), q_t, k_s, id_s);        // S
                mma_scores_ts(tmem + static_cast<uint32_t>(b * 128 + 64), do_t, v_s, id_s);  // dP
                umma_commit(c.bar(B_ACC_FULL + b));
            }
            if (i > 0 && !accumulate(i - 1)) {
                if (leader) c.fail(0x44);
                ok = false;
            }
        }
        if (ok && !accumulate(n_iter - 1)) {
            if (leader) c.fail(0x45);
            ok = false;
        }
        if (ok && leader) umma_commit(c.bar(B_DONE));
        __syncwarp();
    } else {
        const int quad = warp & 3;                 // the TMEM lane quarter this warp may read
        const int cc = (warp - 2) >> 2;            // warpgroup = which half of the score columns
        const int row = quad * 32 + lane;
        const int q_row = q0 + row;
        const bool row_ok = q_row < q_len;
        const uint32_t t_lane = c.tmem_base + (static_cast<uint32_t>(quad * 32) << 16);
        const float sl2 = p.scale * LOG2E;
        const size_t stat_idx = static_cast<size_t>(h) * p.total_q + q_begin + q_row;
        const float neg_lse2 = row_ok ? -p.lse[stat_idx] * LOG2E : -INFINITY;   // -inf -> probability 0
        const float delta = row_ok ? p.delta[stat_idx] : 0.f;
        const int lim = p.causal ? min(k_len - 1, q_row + shift) : k_len - 1;
        const int lo = windowed ? q_row + shift - p.window + 1 : -(1 << 30);
        // one warpgroup moves Q, the other dO, from the TMA-written tiles into tensor memory
        bool ok = warp_wait(c.bar(B_RES_FULL), 0u, c.abort_flag);
        if (ok) {
            copy_row_to_tmem(cc == 0 ? q_s : do_s, row, t_lane + (cc == 0 ? 384u : 448u));
            tmem_st_wait();
            tcgen05_fence_before();
            mbar_arrive(c.bar(B_RESA_FULL));
        }
        for (int i = 0; ok && i < n_iter; ++i) {
            const int b = i & 1;
            const uint32_t ph = static_cast<uint32_t>(i >> 1) & 1u;
            const int kv0 = (it0 + i) * 64;
            if (!warp_wait(c.bar(B_ACC_FULL + b), ph, c.abort_flag)) {
                ok = false;
                break;
            }
            tcgen05_fence_after();
            const int rel = lim - kv0, rel_lo = lo - kv0;
            const uint32_t t_s = t_lane + static_cast<uint32_t>(b * 128);
            // this warpgroup's 32 of the 64 key columns
            uint32_t s[32], dp[32];
            tmem_ld_32x32(t_s + cc * 32, s);
            tmem_ld_32x32(t_s + 64 + cc * 32, dp);
            tmem_ld_wait();
            float e[32];
            // Only the tiles that the diagonal (or the window edge) crosses need the per-element mask; rows past
            // the end of the sequence have lse = +inf and give 0 without it.
            const int c_lo = cc * 32;
            if (__all_sync(0xffffffffu, rel >= c_lo + 31 && rel_lo <= c_lo)) {
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                    const float pr = ex2_approx(fmaf(__uint_as_float(s[j]), sl2, neg_lse2));
                    e[j] = pr * (__uint_as_float(dp[j]) - delta);
                }
            } else {
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                    const float pr = ex2_approx(fmaf(__uint_as_float(s[j]), sl2, neg_lse2));
                    const float ds = pr * (__uint_as_float(dp[j]) - delta);
                    e[j] = (c_lo + j <= rel && c_lo + j >= rel_lo) ? ds : 0.f;
                }
            }
            store_operand(t_s + 64 + cc * 32, e);     // dS over the dP columns it came from
            tmem_st_wait();
            tcgen05_fence_before();
            mbar_arrive(c.bar(B_OP_FULL + b));
        }
        if (ok) ok = warp_wait(c.bar(B_DONE), 0u, c.abort_flag);
        if (!ok) {
            if (lane == 0) c.fail(0x46);
        } else {
            tcgen05_fence_after();
            __nv_bfloat16* dst = p.dq + static_cast<size_t>(q_begin + q_row) * p.dq_tstride + static_cast<size_t>(h) * HD;
            store_acc_row(t_lane + 256u, p.scale, dst, row_ok, 2 * cc, 2 * cc + 2);
        }
    }
    bwd_teardown(c);
}

// ========================================================================= dK/dV kernel
// grid (Hkv, seqs, kv tiles of 128): heads fastest, so the early key tiles (seen by the most queries under a causal
// mask) of every head are scheduled first
__global__ void __launch_bounds__(BWD_THREADS, 1)
attn_bwd_dkv_tc_kernel(const __grid_constant__ CUtensorMap tma_q, const __grid_constant__ CUtensorMap tma_do,
                       const __grid_constant__ CUtensorMap tma_k, const __grid_constant__ CUtensorMap tma_v,
                       const AttnParams p, int* status) {
    const int seq = blockIdx.y, kvh = blockIdx.x;
    const int q_len = p.q_lens[seq], k_len = p.k_lens[seq];
    const int kv0 = static_cast<int>(blockIdx.z) * 128;
    if (kv0 >= k_len) return;
    const int q_begin = p.q_begins[seq], k_begin = p.k_begins[seq];
    const int shift = k_len - q_len;
    const int G = p.H / p.Hkv;
    // first query row that can see this tile (causal: q + shift >= kv0), rounded down to a 64-row tile
    const int q_lo = p.causal ? max(0, kv0 - shift) : 0;
    const int jt_lo = q_lo / 64;
    // sliding window: query rows beyond q_hi no longer see the last key of this tile
    const bool windowed = p.causal && p.window > 0;
    const int kv_last = min(kv0 + 128, k_len) - 1;
    const int q_hi = windowed ? min(q_len, kv_last - shift + p.window) : q_len;     // exclusive
    const int jt_hi = (q_hi + 63) / 64;
    const int per_head = max(0, jt_hi - jt_lo);
    const int n_iter = per_head * G;
    const int warp = __shfl_sync(0xffffffffu, threadIdx.x >> 5, 0), lane = threadIdx.x & 31;   // warp-uniform for the compiler

    if (n_iter == 0) {
        // no query sees these keys: zero gradients
        if (warp >= 2 && warp < 6) {
            const int row = (warp & 3) * 32 + lane;
            if (kv0 + row < k_len) {
                const size_t t = static_cast<size_t>(k_begin + kv0 + row);
                __nv_bfloat16* dk = p.dk + t * p.dk_tstride + static_cast<size_t>(kvh) * HD;
                __nv_bfloat16* dv = p.dv + t * p.dv_tstride + static_cast<size_t>(kvh) * HD;
                for (int c = 0; c < HD / 8; ++c) {
                    *reinterpret_cast<uint4*>(dk + 8 * c) = make_uint4(0, 0, 0, 0);
                    *reinterpret_cast<uint4*>(dv + 8 * c) = make_uint4(0, 0, 0, 0);
                }
            }
        }
        return;
    }

    extern __shared__ uint8_t smem_raw[];
    Ctx c;
    bwd_setup(c, smem_raw, status, KV_OFF_BAR);
    if (threadIdx.x == 0) {
        prefetch_tmap(&tma_q);
        prefetch_tmap(&tma_do);
        prefetch_tmap(&tma_k);
        prefetch_tmap(&tma_v);
    }
    const uint32_t k_s = c.base + OFF_RES0, v_s = c.base + OFF_RES1;
    float* vec = reinterpret_cast<float*>(smem_raw + (c.base - smem_u32(smem_raw)) + KV_OFF_VEC);

    if (warp == 0) {
        if (lane == 0) {
            const uint32_t rb = c.bar(B_RES_FULL);
            mbar_arrive_expect_tx(rb, 2 * BIG_TILE);
            tma_load_2d(k_s, &tma_k, rb, kvh * HD, k_begin + kv0);
            tma_load_2d(k_s + BOX128, &tma_k, rb, kvh * HD + 64, k_begin + kv0);
            tma_load_2d(v_s, &tma_v, rb, kvh * HD, k_begin + kv0);
            tma_load_2d(v_s + BOX128, &tma_v, rb, kvh * HD + 64, k_begin + kv0);
            for (int i = 0; i < n_iter; ++i) {
                const int st = i % KV_NSTG;
                const uint32_t ph = static_cast<uint32_t>(i / KV_NSTG) & 1u;
                const int h = kvh * G + i / per_head;
                const int row = q_begin + (jt_lo + i % per_head) * 64;
                if (!c.wait(B_STG_EMPTY + st, ph ^ 1u)) {
                    c.fail(0x51);
                    break;
                }
                const uint32_t fb = c.bar(B_STG_FULL + st);
                const uint32_t q_s = c.base + OFF_STG + st * STAGE_BYTES, do_s = q_s + SMALL_TILE;
                mbar_arrive_expect_tx(fb, 2 * SMALL_TILE);
                tma_load_2d(q_s, &tma_q, fb, h * HD, row);
                tma_load_2d(q_s + BOX64, &tma_q, fb, h * HD + 64, row);
                tma_load_2d(do_s, &tma_do, fb, h * HD, row);
                tma_load_2d(do_s + BOX64, &tma_do, fb, h * HD + 64, row);
            }
        }
    } else if (warp == 1) {
        // The whole warp runs the issue loop converged; only the tcgen05 instructions are predicated on one lane.
        const bool leader = elect_one();
        const uint32_t tmem = __shfl_sync(0xffffffffu, c.tmem_base, 0);
        const uint32_t id_s = make_idesc_bf16(128, 64, false);
        const uint32_t id_acc = make_idesc_bf16(128, 128, true);
        bool ok = c.wait(B_RES_FULL, 0u);
        if (!ok && leader) c.fail(0x52);
        auto accumulate = [&](int j) -> bool {     // dV += P^T dO_j ; dK += dS^T Q_j
            const int b = j & 1, st = j % KV_NSTG;
            if (!c.wait(B_OP_FULL + b, static_cast<uint32_t>(j >> 1) & 1u)) return false;
            tcgen05_fence_after();
            const uint32_t q_s = c.base + OFF_STG + st * STAGE_BYTES, do_s = q_s + SMALL_TILE;
            const uint32_t pt_t = tmem + static_cast<uint32_t>(b * 128), dst_t = pt_t + 64u;
            if (leader) {
                mma_accum(tmem + 256u, pt_t, do_s, id_acc, j == 0);
                mma_accum(tmem + 384u, dst_t, q_s, id_acc, j == 0);
                umma_commit(c.bar(B_STG_EMPTY + st));
            }
            return true;
        };
        for (int i = 0; i < n_iter && ok; ++i) {
            const int b = i & 1, st = i % KV_NSTG;
            // the score pair b is free: the MMAs that read tile i - 2 from it were issued before this point
            ok = c.wait(B_STG_FULL + st, static_cast<uint32_t>(i / KV_NSTG) & 1u);
            if (!ok) {
                if (leader) c.fail(0x53);
                break;
            }
            tcgen05_fence_after();
            const uint32_t q_s = c.base + OFF_STG + st * STAGE_BYTES, do_s = q_s + SMALL_TILE;
            if (leader) {
                mma_scores(tmem + static_cast<uint32_t>(b * 128), k_s, q_s, id_s);         // S^T
                mma_scores(tmem + static_cast<uint32_t>(b * 128 + 64), v_s, do_s, id_s);   // dP^T
                umma_commit(c.bar(B_ACC_FULL + b));
            }
            if (i > 0 && !accumulate(i - 1)) {
                if (leader) c.fail(0x54);
                ok = false;
            }
        }
        if (ok && !accumulate(n_iter - 1)) {
            if (leader) c.fail(0x55);
            ok = false;
        }
        if (ok && leader) umma_commit(c.bar(B_DONE));
        __syncwarp();
    } else {
        const int quad = warp & 3;                 // the TMEM lane quarter this warp may read
        const int cc = (warp - 2) >> 2;            // warpgroup = which half of the 64 query columns
        const int row = quad * 32 + lane;          // key/value row inside the tile
        const int kv_row = kv0 + row;
        const bool row_ok = kv_row < k_len;
        const uint32_t t_lane = c.tmem_base + (static_cast<uint32_t>(quad * 32) << 16);
        const float sl2 = p.scale * LOG2E;
        bool ok = true;
        // Every warp stages -lse * log2(e) and delta of its 32 query columns of the NEXT tile in its own slice of
        // shared memory (a warp-level sync suffices) and reads them back four columns per load.
        float* my_vec = vec + (warp - 2) * (2 * 2 * 32);
        auto load_stats = [&](int i, float& nl, float& dl) {
            const int h = kvh * G + i / per_head;
            const int q = (jt_lo + i % per_head) * 64 + cc * 32 + lane;
            const size_t idx = static_cast<size_t>(h) * p.total_q + q_begin + q;
            nl = (q < q_len) ? -p.lse[idx] * LOG2E : -INFINITY;   // -inf -> probability 0
            dl = (q < q_len) ? p.delta[idx] : 0.f;
        };
        auto stage_stats = [&](int i, float nl, float dl) {
            float* dst = my_vec + (i & 1) * 64;
            dst[lane] = nl;
            dst[32 + lane] = dl;
        };
        float nl_next, dl_next;
        load_stats(0, nl_next, dl_next);
        stage_stats(0, nl_next, dl_next);
        for (int i = 0; i < n_iter; ++i) {
            const int b = i & 1;
            const uint32_t ph = static_cast<uint32_t>(i >> 1) & 1u;
            const int qt0 = (jt_lo + i % per_head) * 64;
            // the loads for the next tile are in flight during this tile's math and staged at its end
            if (i + 1 < n_iter) load_stats(i + 1, nl_next, dl_next);
            __syncwarp();
            if (!warp_wait(c.bar(B_ACC_FULL + b), ph, c.abort_flag)) {
                ok = false;
                break;
            }
            tcgen05_fence_after();
            // query column j (row qt0 + j) sees key kv_row iff kv_row <= qt0 + j + shift
            const int jmin = p.causal ? kv_row - shift - qt0 : 0;     // columns below jmin are masked
            const int jmax = windowed ? kv_row - shift + p.window - 1 - qt0 : (1 << 30);   // and above jmax
            const uint32_t t_s = t_lane + static_cast<uint32_t>(b * 128);
            const float4* nl4 = reinterpret_cast<const float4*>(my_vec + b * 64);
            const float4* dl4 = nl4 + 8;
            uint32_t s[32], dp[32];
            tmem_ld_32x32(t_s + cc * 32, s);
            tmem_ld_32x32(t_s + 64 + cc * 32, dp);
            tmem_ld_wait();
            float pe[32], de[32];
            const int c_lo = cc * 32;
            // only the tiles that the diagonal (or the window edge) crosses need the per-element mask
            const bool all_live = __all_sync(0xffffffffu, row_ok && jmin <= c_lo && jmax >= c_lo + 31);
#pragma unroll
            for (int g = 0; g < 8; ++g) {
                const float4 n4 = nl4[g], d4 = dl4[g];
                const float nl_j[4] = {n4.x, n4.y, n4.z, n4.w}, dl_j[4] = {d4.x, d4.y, d4.z, d4.w};
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const int j = 4 * g + u;
                    const float pr = ex2_approx(fmaf(__uint_as_float(s[j]), sl2, nl_j[u]));
                    pe[j] = pr;
                    de[j] = pr * (__uint_as_float(dp[j]) - dl_j[u]);
                }
            }
            if (!all_live) {
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                    const bool live = row_ok && c_lo + j >= jmin && c_lo + j <= jmax;
                    pe[j] = live ? pe[j] : 0.f;
                    de[j] = live ? de[j] : 0.f;
                }
            }
            store_operand(t_s + cc * 32, pe);          // P^T over the S^T columns it came from
            store_operand(t_s + 64 + cc * 32, de);     // dS^T over the dP^T columns
            tmem_st_wait();
            tcgen05_fence_before();
            mbar_arrive(c.bar(B_OP_FULL + b));
            if (i + 1 < n_iter) stage_stats(i + 1, nl_next, dl_next);
        }
        if (ok) ok = warp_wait(c.bar(B_DONE), 0u, c.abort_flag);
        if (!ok) {
            if (lane == 0) c.fail(0x56);
        } else {
            tcgen05_fence_after();
            const size_t t = static_cast<size_t>(k_begin + kv_row);
            if (cc == 0)
                store_acc_row(t_lane + 256u, 1.0f, p.dv + t * p.dv_tstride + static_cast<size_t>(kvh) * HD, row_ok);
            else
                store_acc_row(t_lane + 384u, p.scale, p.dk + t * p.dk_tstride + static_cast<size_t>(kvh) * HD, row_ok);
        }
    }
    bwd_teardown(c);
}

}  // namespace

// delta = rowsum(dO * O); defined with the mma.sync kernels
const char* attn_delta(const AttnParams& p, cudaStream_t st);

const char* attn_backward_tc(const AttnParams& p, int* status, cudaStream_t st) {
    if (p.num_seqs == 0 || p.total_q == 0) return nullptr;
    if (p.D != HD) return "attn_backward_tc: head_dim must be 128";
    const size_t strides[] = {p.q_tstride, p.k_tstride, p.v_tstride, p.do_tstride, p.dq_tstride, p.dk_tstride, p.dv_tstride};
    for (size_t s : strides)
        if (s % 8) return "attn_backward_tc: row pitches must be multiples of 16 bytes";
    const void* ptrs[] = {p.q, p.k, p.v, p.dout, p.dq, p.dk, p.dv};
    for (const void* ptr : ptrs)
        if (reinterpret_cast<uintptr_t>(ptr) % 16) return "attn_backward_tc: operands must be 16-byte aligned";
    const char* err = attn_delta(p, st);
    if (err != nullptr) return err;
    const uint64_t qcols = static_cast<uint64_t>(p.H) * HD, kcols = static_cast<uint64_t>(p.Hkv) * HD;
    CUtensorMap q128, do128, k64, v64, q64, do64, k128, v128;
    if (!make_view_tmap(&q128, p.q, p.total_q, qcols, p.q_tstride, 128) ||
        !make_view_tmap(&do128, p.dout, p.total_q, qcols, p.do_tstride, 128) ||
        !make_view_tmap(&k64, p.k, p.total_k, kcols, p.k_tstride, 64) ||
        !make_view_tmap(&v64, p.v, p.total_k, kcols, p.v_tstride, 64) ||
        !make_view_tmap(&q64, p.q, p.total_q, qcols, p.q_tstride, 64) ||
        !make_view_tmap(&do64, p.dout, p.total_q, qcols, p.do_tstride, 64) ||
        !make_view_tmap(&k128, p.k, p.total_k, kcols, p.k_tstride, 128) ||
        !make_view_tmap(&v128, p.v, p.total_k, kcols, p.v_tstride, 128))
        return tmap_error();
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attn_bwd_dq_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             DQ_SMEM_BYTES);
        if (e == cudaSuccess)
            e = cudaFuncSetAttribute(attn_bwd_dkv_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     KV_SMEM_BYTES);
        if (e != cudaSuccess) return cudaGetErrorString(e);
        configured = true;
    }
    const dim3 grid_kv(p.Hkv, p.num_seqs, (p.max_k + 127) / 128);
    const dim3 grid_q(p.H, p.num_seqs, (p.max_q + 127) / 128);
    attn_bwd_dkv_tc_kernel<<<grid_kv, BWD_THREADS, KV_SMEM_BYTES, st>>>(q64, do64, k128, v128, p, status);
    attn_bwd_dq_tc_kernel<<<grid_q, BWD_THREADS, DQ_SMEM_BYTES, st>>>(q128, do128, k64, v64, p, status);
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? nullptr : cudaGetErrorString(e);
}

}  // namespace fs2
