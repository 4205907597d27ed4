// Flash-attention forward on the 5th-generation tensor cores (sm_100a), head_dim 128.
//
//   TMA (cp.async.bulk.tensor, 128B swizzle) -> shared memory -> tcgen05.mma with the
//   score tile S = Q K^T and the partial output P V accumulated in TMEM -> tcgen05.ld.
//
// One CTA owns 128 query rows of one head of one (packed) sequence; 192 threads:
//   warp 0      : TMA producer (Q once, then a two-stage ring of K and V tiles)
//   warp 1      : TMEM allocator and MMA issuer
//   warps 2..5  : softmax; thread t owns query row t of the tile, i.e. TMEM lane t, so the
//                 row maximum and row sum need no cross-thread reduction
//
// Per key/value tile of 128 rows the issuer runs S(i) = Q K_i^T into one of two TMEM score
// buffers while the softmax warps are still busy with S(i-1); the softmax warps write
// P = exp2(S * scale - max) as bf16 into a swizzled shared-memory tile that becomes the A
// operand of PV(i) = P V_i (V is consumed as an MN-major B operand straight from its
// row-major tile). PV(i) lands in one of two TMEM output buffers; the softmax warps fold it
// into their fp32 register accumulators with the usual online-softmax rescale one iteration
// later, so tensor-core work and exponentials overlap.
//
// TMEM: 2 x 128 columns of scores + 2 x 128 columns of partial outputs = 512 columns.
// Shared memory: Q 32 KB, K 2 x 32 KB, V 2 x 32 KB, P 2 x 32 KB.
//
// Every barrier wait is bounded; a wait that gives up records a code in the host-visible
// status word, raises a CTA-wide abort flag and every role falls through to the teardown
// that frees TMEM.

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>

#include "attention.h"
#include "attention_tc.cuh"
#include "common.cuh"

namespace fs2 {

namespace {

using namespace tc;

constexpr int TQ = 128;                      // query rows per CTA
constexpr int TK = 128;                      // key/value rows per iteration
constexpr int HD = 128;                      // head dimension
constexpr int BOX_BYTES = 128 * 64 * 2;      // one [128 rows][64 cols] bf16 TMA box
constexpr int TILE_BYTES = 2 * BOX_BYTES;    // a [128][128] bf16 tile = two boxes
constexpr int STAGES = 2;
constexpr int OFF_Q = 0;
constexpr int OFF_K = OFF_Q + TILE_BYTES;
constexpr int OFF_V = OFF_K + STAGES * TILE_BYTES;
constexpr int OFF_P = OFF_V + STAGES * TILE_BYTES;
constexpr int OFF_BAR = OFF_P + 2 * TILE_BYTES;
constexpr int BAR_BYTES = 256;
constexpr int TC_SMEM_BYTES = OFF_BAR + BAR_BYTES + 1024;
constexpr int TC_THREADS = 192;
constexpr uint32_t TMEM_COLS = 512;
constexpr uint64_t WAIT_LIMIT_NS = 2000000000ull;
constexpr float LOG2E_F = 1.4426950408889634f;

static_assert(TC_SMEM_BYTES <= 232448, "shared memory budget of one CTA exceeded");

// barrier slots (8 bytes each)
enum : int {
    BAR_Q_FULL = 0,
    BAR_K_FULL = 1,    // [2]
    BAR_K_EMPTY = 3,   // [2]
    BAR_V_FULL = 5,    // [2]
    BAR_V_EMPTY = 7,   // [2]
    BAR_S_FULL = 9,    // [2]
    BAR_S_EMPTY = 11,  // [2]
    BAR_P_FULL = 13,   // [2]
    BAR_PV_FULL = 15,  // [2]
    BAR_PV_EMPTY = 17, // [2]
    NUM_BARS = 19
};


// WINDOWED compiles the sliding-window bounds in; the plain instantiation keeps the softmax loop free of them (the
// softmax warps are the bottleneck of this kernel: one extra instruction per score costs several percent).
template <bool WINDOWED>
__global__ void __launch_bounds__(TC_THREADS, 1)
attn_fwd_tc_kernel(const __grid_constant__ CUtensorMap tma_q, const __grid_constant__ CUtensorMap tma_k,
                   const __grid_constant__ CUtensorMap tma_v, const AttnParams p, int* status) {
    // ------------------------------------------------------------- tile geometry
    // Heads vary fastest and tiles slowest, so that the block scheduler hands out the long (late) query tiles of ALL
    // heads before any short one: with tiles fastest, the last head's long tiles start late and the SMs that
    // finished early idle behind them.
    const int seq = blockIdx.y;
    const int h = blockIdx.x;
    const int q_len = p.q_lens[seq], k_len = p.k_lens[seq];
    const int qblk = static_cast<int>(gridDim.z) - 1 - static_cast<int>(blockIdx.z);   // long tiles first
    const int q0 = qblk * TQ;
    if (q0 >= q_len) return;
    const int q_begin = p.q_begins[seq], k_begin = p.k_begins[seq];
    const int shift = k_len - q_len;                       // causal mask is bottom-right aligned
    const int q_last = min(q0 + TQ, q_len) - 1;
    const int kv_hi = p.causal ? min(k_len, q_last + shift + 1) : k_len;
    if (kv_hi <= 0) return;                                // nothing to attend to: output stays zero
    // sliding window: the first key any row of this tile can see, rounded down to a key tile
    constexpr bool windowed = WINDOWED;
    const int it0 = windowed ? max(0, q0 + shift - p.window + 1) / TK : 0;
    const int n_iter = (kv_hi + TK - 1) / TK - it0;
    if (n_iter <= 0) return;
    const int kvh = h / (p.H / p.Hkv);

    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t* smem = smem_raw + (base - raw);
    uint8_t* bar_ptr = smem + OFF_BAR;
    const uint32_t bar_base = smem_u32(bar_ptr);
    auto bar = [&](int slot) { return bar_base + 8u * static_cast<uint32_t>(slot); };
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(bar_ptr + 8 * NUM_BARS);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(bar_ptr + 8 * NUM_BARS + 8);

    const int warp = __shfl_sync(0xffffffffu, threadIdx.x >> 5, 0);   // warp-uniform for the compiler
    const int lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        mbar_init(bar(BAR_Q_FULL), 1);
        for (int s = 0; s < 2; ++s) {
            mbar_init(bar(BAR_K_FULL + s), 1);
            mbar_init(bar(BAR_K_EMPTY + s), 1);
            mbar_init(bar(BAR_V_FULL + s), 1);
            mbar_init(bar(BAR_V_EMPTY + s), 1);
            mbar_init(bar(BAR_S_FULL + s), 1);
            mbar_init(bar(BAR_S_EMPTY + s), 128);
            mbar_init(bar(BAR_P_FULL + s), 128);
            mbar_init(bar(BAR_PV_FULL + s), 1);
            mbar_init(bar(BAR_PV_EMPTY + s), 128);
        }
        *abort_flag = 0;
        fence_barrier_init();
        prefetch_tmap(&tma_q);
        prefetch_tmap(&tma_k);
        prefetch_tmap(&tma_v);
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), TMEM_COLS);
        tmem_relinquish();
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ---------------------------------------------------------------- producer
        if (lane == 0) {
            const uint32_t qb = bar(BAR_Q_FULL);
            mbar_arrive_expect_tx(qb, TILE_BYTES);
            tma_load_2d(base + OFF_Q, &tma_q, qb, h * HD, q_begin + q0);
            tma_load_2d(base + OFF_Q + BOX_BYTES, &tma_q, qb, h * HD + 64, q_begin + q0);
            for (int i = 0; i < n_iter; ++i) {
                const int st = i & 1;
                const uint32_t ph = static_cast<uint32_t>(i >> 1) & 1u;
                const int row = k_begin + (it0 + i) * TK;
                if (!mbar_wait_bounded(bar(BAR_K_EMPTY + st), ph ^ 1u, abort_flag, WAIT_LIMIT_NS)) {
                    if (!*abort_flag) report_status(status, kStatusTimeout | (0x11 << 8));
                    *abort_flag = 1;
                    break;
                }
                const uint32_t kb = bar(BAR_K_FULL + st);
                mbar_arrive_expect_tx(kb, TILE_BYTES);
                tma_load_2d(base + OFF_K + st * TILE_BYTES, &tma_k, kb, kvh * HD, row);
                tma_load_2d(base + OFF_K + st * TILE_BYTES + BOX_BYTES, &tma_k, kb, kvh * HD + 64, row);
                if (!mbar_wait_bounded(bar(BAR_V_EMPTY + st), ph ^ 1u, abort_flag, WAIT_LIMIT_NS)) {
                    if (!*abort_flag) report_status(status, kStatusTimeout | (0x12 << 8));
                    *abort_flag = 1;
                    break;
                }
                const uint32_t vb = bar(BAR_V_FULL + st);
                mbar_arrive_expect_tx(vb, TILE_BYTES);
                tma_load_2d(base + OFF_V + st * TILE_BYTES, &tma_v, vb, kvh * HD, row);
                tma_load_2d(base + OFF_V + st * TILE_BYTES + BOX_BYTES, &tma_v, vb, kvh * HD + 64, row);
            }
        }
    } else if (warp == 1) {
        // -------------------------------------------------------------- MMA issuer
        // The whole warp runs the issue loop converged and only the tcgen05 instructions are predicated on one lane,
        // so that descriptors and addresses stay in uniform registers.
        const bool leader = elect_one();
        const uint32_t tmem = __shfl_sync(0xffffffffu, tmem_base, 0);
        auto fail = [&](int code) {
            if (leader) {
                if (!*abort_flag) report_status(status, kStatusTimeout | (code << 8));
                *abort_flag = 1;
            }
        };
        const uint32_t idesc_s = make_idesc_bf16(128, 128, false);
        const uint32_t idesc_pv = make_idesc_bf16(128, 128, true);
        bool ok = mbar_wait_bounded(bar(BAR_Q_FULL), 0u, abort_flag, WAIT_LIMIT_NS);
        if (!ok) fail(0x21);
        // PV(j) = P_j V_j into output buffer j & 1
        auto issue_pv = [&](int j) -> bool {
            const int b = j & 1;
            const uint32_t ph = static_cast<uint32_t>(j >> 1) & 1u;
            if (!mbar_wait_bounded(bar(BAR_V_FULL + b), ph, abort_flag, WAIT_LIMIT_NS)) return false;
            if (!mbar_wait_bounded(bar(BAR_P_FULL + b), ph, abort_flag, WAIT_LIMIT_NS)) return false;
            if (!mbar_wait_bounded(bar(BAR_PV_EMPTY + b), ph ^ 1u, abort_flag, WAIT_LIMIT_NS)) return false;
            tcgen05_fence_after();
            const uint32_t d_tmem = tmem + 256u + static_cast<uint32_t>(b * 128);
            const uint32_t p_s = base + OFF_P + b * TILE_BYTES;
            const uint32_t v_s = base + OFF_V + b * TILE_BYTES;
            if (leader) {
#pragma unroll
                for (int k = 0; k < TK / 16; ++k) {
                    const uint64_t da = make_smem_desc(p_s + (k >> 2) * BOX_BYTES + (k & 3) * 32, 16, 1024);
                    const uint64_t db = make_smem_desc(v_s + k * 16 * 128, BOX_BYTES, 1024);
                    umma_bf16(d_tmem, da, db, idesc_pv, k > 0 ? 1u : 0u);
                }
                umma_commit(bar(BAR_PV_FULL + b));
                umma_commit(bar(BAR_V_EMPTY + b));
            }
            return true;
        };
        for (int i = 0; i < n_iter && ok; ++i) {
            const int b = i & 1;
            const uint32_t ph = static_cast<uint32_t>(i >> 1) & 1u;
            ok = mbar_wait_bounded(bar(BAR_K_FULL + b), ph, abort_flag, WAIT_LIMIT_NS) &&
                 mbar_wait_bounded(bar(BAR_S_EMPTY + b), ph ^ 1u, abort_flag, WAIT_LIMIT_NS);
            if (!ok) {
                fail(0x22);
                break;
            }
            tcgen05_fence_after();
            const uint32_t d_tmem = tmem + static_cast<uint32_t>(b * 128);
            const uint32_t q_s = base + OFF_Q;
            const uint32_t k_s = base + OFF_K + b * TILE_BYTES;
            if (leader) {
#pragma unroll
                for (int k = 0; k < HD / 16; ++k) {
                    const uint32_t off = (k >> 2) * BOX_BYTES + (k & 3) * 32;
                    umma_bf16(d_tmem, make_smem_desc(q_s + off, 16, 1024), make_smem_desc(k_s + off, 16, 1024),
                              idesc_s, k > 0 ? 1u : 0u);
                }
                umma_commit(bar(BAR_S_FULL + b));
                umma_commit(bar(BAR_K_EMPTY + b));
            }
            if (i > 0 && !issue_pv(i - 1)) {
                fail(0x23);
                ok = false;
            }
        }
        if (ok && !issue_pv(n_iter - 1)) fail(0x24);
        __syncwarp();
    } else {
        // ----------------------------------------------------------------- softmax
        const int quad = warp & 3;                     // TMEM lane quadrant of this warp
        const int row = quad * 32 + lane;              // query row inside the tile
        const int q_row = q0 + row;
        const uint32_t t_lane = tmem_base + (static_cast<uint32_t>(quad * 32) << 16);
        const float sl2 = p.scale * LOG2E_F;
        const int lim = p.causal ? min(k_len - 1, q_row + shift) : k_len - 1;   // last visible key of this row
        const int lo = windowed ? q_row + shift - p.window + 1 : -(1 << 30);    // first visible key of this row
        float m = -INFINITY, l = 0.f, alpha_prev = 1.f;
        float o[HD];
#pragma unroll
        for (int j = 0; j < HD; ++j) o[j] = 0.f;
        bool ok = true;

        auto fold_pv = [&](int j, float alpha) -> bool {
            const int b = j & 1;
            const uint32_t ph = static_cast<uint32_t>(j >> 1) & 1u;
            if (!warp_wait(bar(BAR_PV_FULL + b), ph, abort_flag)) return false;
            tcgen05_fence_after();
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                uint32_t v[32];
                tmem_ld_32x32(t_lane + 256u + static_cast<uint32_t>(b * 128 + c * 32), v);
                tmem_ld_wait();
#pragma unroll
                for (int j2 = 0; j2 < 32; ++j2) o[c * 32 + j2] = fmaf(o[c * 32 + j2], alpha, __uint_as_float(v[j2]));
            }
            tcgen05_fence_before();
            mbar_arrive(bar(BAR_PV_EMPTY + b));
            return true;
        };

        for (int i = 0; i < n_iter; ++i) {
            const int b = i & 1;
            const uint32_t ph = static_cast<uint32_t>(i >> 1) & 1u;
            const int kv0 = (it0 + i) * TK;
            if (!warp_wait(bar(BAR_S_FULL + b), ph, abort_flag)) {
                ok = false;
                break;
            }
            tcgen05_fence_after();
            const bool need_mask = (kv0 + TK > k_len) || (p.causal && kv0 + TK - 1 > q0 + shift) ||
                                   (windowed && q_last + shift - p.window + 1 > kv0);
            const int rel = lim - kv0;                 // columns > rel are masked
            const int rel_lo = lo - kv0;               // columns < rel_lo are masked (sliding window)
            const uint32_t t_s = t_lane + static_cast<uint32_t>(b * 128);
            // pass 1: row maximum
            float mx = -INFINITY;
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                uint32_t v[32];
                tmem_ld_32x32(t_s + c * 32, v);
                tmem_ld_wait();
                if (need_mask) {
#pragma unroll
                    for (int j = 0; j < 32; ++j)
                        if (c * 32 + j <= rel && (!WINDOWED || c * 32 + j >= rel_lo)) mx = fmaxf(mx, __uint_as_float(v[j]));
                } else {
#pragma unroll
                    for (int j = 0; j < 32; ++j) mx = fmaxf(mx, __uint_as_float(v[j]));
                }
            }
            const float m_new = fmaxf(m, mx);
            const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
            const float alpha = ex2_approx((m - m_use) * sl2);        // m = -inf -> 0
            const float neg_ms = -m_use * sl2;
            // pass 2: probabilities -> bf16 tile in shared memory (128B-swizzled, K-major)
            float rowsum = 0.f;
            const uint32_t p_row = base + OFF_P + b * TILE_BYTES + static_cast<uint32_t>(row) * 128u;
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                uint32_t v[32];
                tmem_ld_32x32(t_s + c * 32, v);
                tmem_ld_wait();
                float e[32];
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                    float pr = ex2_approx(fmaf(__uint_as_float(v[j]), sl2, neg_ms));
                    if (need_mask && (c * 32 + j > rel || (WINDOWED && c * 32 + j < rel_lo))) pr = 0.f;
                    e[j] = pr;
                    rowsum += pr;
                }
                const uint32_t sub = p_row + static_cast<uint32_t>(c >> 1) * BOX_BYTES;
#pragma unroll
                for (int g = 0; g < 4; ++g) {
                    const uint32_t chunk = static_cast<uint32_t>((c & 1) * 4 + g);
                    const uint32_t dst = sub + (((chunk ^ static_cast<uint32_t>(row & 7)) & 7u) << 4);
                    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst),
                                 "r"(pack2_bf16(e[8 * g], e[8 * g + 1])), "r"(pack2_bf16(e[8 * g + 2], e[8 * g + 3])),
                                 "r"(pack2_bf16(e[8 * g + 4], e[8 * g + 5])), "r"(pack2_bf16(e[8 * g + 6], e[8 * g + 7]))
                                 : "memory");
                }
            }
            tcgen05_fence_before();
            mbar_arrive(bar(BAR_S_EMPTY + b));         // score buffer may be overwritten by S(i + 2)
            fence_proxy_async_smem();                  // make the P tile visible to the tensor core
            mbar_arrive(bar(BAR_P_FULL + b));
            l = l * alpha + rowsum;
            m = m_new;
            if (i > 0 && !fold_pv(i - 1, alpha_prev)) {
                ok = false;
                break;
            }
            alpha_prev = alpha;
        }
        if (ok) ok = fold_pv(n_iter - 1, alpha_prev);
        if (!ok) {
            if (lane == 0 && !*abort_flag) report_status(status, kStatusTimeout | (0x31 << 8));
            *abort_flag = 1;
        } else if (q_row < q_len) {
            const float inv = l > 0.f ? 1.f / l : 0.f;
            __nv_bfloat16* og = p.o + static_cast<size_t>(q_begin + q_row) * p.o_tstride + static_cast<size_t>(h) * HD;
#pragma unroll
            for (int c = 0; c < HD / 8; ++c) {
                uint4 w;
                w.x = pack2_bf16(o[8 * c] * inv, o[8 * c + 1] * inv);
                w.y = pack2_bf16(o[8 * c + 2] * inv, o[8 * c + 3] * inv);
                w.z = pack2_bf16(o[8 * c + 4] * inv, o[8 * c + 5] * inv);
                w.w = pack2_bf16(o[8 * c + 6] * inv, o[8 * c + 7] * inv);
                *reinterpret_cast<uint4*>(og + 8 * c) = w;
            }
            p.lse[static_cast<size_t>(h) * p.total_q + q_begin + q_row] =
                l > 0.f ? m * p.scale + logf(l) : -INFINITY;
        }
    }

    // ----------------------------------------------------------------- teardown
    __syncthreads();
    if (*abort_flag) {
        // give copies that were already in flight time to land before the CTA retires
        const uint64_t t0 = global_timer_ns();
        while (global_timer_ns() - t0 < 200000ull) __nanosleep(1000);
        __syncthreads();
    }
    tcgen05_fence_after();
    if (warp == 1) tmem_dealloc(tmem_base, TMEM_COLS);
}

}  // namespace

const char* attn_forward_tc(const AttnParams& p, int* status, cudaStream_t st) {
    if (p.num_seqs == 0 || p.total_q == 0) return nullptr;
    if (p.D != HD) return "attn_forward_tc: head_dim must be 128";
    if (p.q_tstride % 8 || p.k_tstride % 8 || p.v_tstride % 8 || p.o_tstride % 8 ||
        reinterpret_cast<uintptr_t>(p.q) % 16 || reinterpret_cast<uintptr_t>(p.k) % 16 ||
        reinterpret_cast<uintptr_t>(p.v) % 16 || reinterpret_cast<uintptr_t>(p.o) % 16)
        return "attn_forward_tc: operands must be 16-byte aligned with 16-byte aligned row pitch";
    CUtensorMap tq, tk, tv;
    if (!make_view_tmap(&tq, p.q, p.total_q, static_cast<uint64_t>(p.H) * HD, p.q_tstride, 128) ||
        !make_view_tmap(&tk, p.k, p.total_k, static_cast<uint64_t>(p.Hkv) * HD, p.k_tstride, 128) ||
        !make_view_tmap(&tv, p.v, p.total_k, static_cast<uint64_t>(p.Hkv) * HD, p.v_tstride, 128))
        return tmap_error();
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attn_fwd_tc_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             TC_SMEM_BYTES);
        if (e == cudaSuccess)
            e = cudaFuncSetAttribute(attn_fwd_tc_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     TC_SMEM_BYTES);
        if (e != cudaSuccess) return cudaGetErrorString(e);
        configured = true;
    }
    const dim3 grid(p.H, p.num_seqs, (p.max_q + TQ - 1) / TQ);
    if (p.causal && p.window > 0)
        attn_fwd_tc_kernel<true><<<grid, TC_THREADS, TC_SMEM_BYTES, st>>>(tq, tk, tv, p, status);
    else
        attn_fwd_tc_kernel<false><<<grid, TC_THREADS, TC_SMEM_BYTES, st>>>(tq, tk, tv, p, status);
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? nullptr : cudaGetErrorString(e);
}

}  // namespace fs2
