// Persistent, warp-specialised bf16 GEMM for sm_100a:
//
//   TMA (cp.async.bulk.tensor) -> 128B-swizzled shared memory -> tcgen05.mma
//   (operands from smem descriptors, fp32 accumulators in TMEM) -> tcgen05.ld
//   -> swizzled staging tile -> TMA store (or TMA reduce-add for accumulation).
//
// One CTA per SM, 192 threads:
//   warp 0      : TMA producer (one elected lane)
//   warp 1      : TMEM allocator + MMA issuer (one elected lane)
//   warps 2..5  : epilogue; warp w owns TMEM lanes [32*(w%4), 32*(w%4)+32)
//
// CTA tile 128x256, K block 64 (one 128-byte swizzle row), 4 smem stages
// (48 KB each) and a double-buffered accumulator (2 x 256 TMEM columns), so the
// epilogue of tile i overlaps the main loop of tile i+1.
//
// Operand layouts. C[M,N] = A * B^T with
//   K-major A  : memory [M, K] row-major          (a_mn = false)
//   MN-major A : memory [K, M] row-major          (a_mn = true)
//   K-major B  : memory [N, K] row-major          (b_mn = false)
//   MN-major B : memory [K, N] row-major          (b_mn = true)
// which covers forward (x W^T), dgrad (dy W) and wgrad (dy^T x) of a linear
// layer without a transpose pass.
//
// Every barrier wait is bounded (2 s); a wait that gives up records a code in
// a host-visible status word, raises a CTA-wide abort flag, and all roles fall
// through to the common teardown that frees TMEM.
//
// Plain GEMMs with enough tiles run on the CTA-pair variant of this kernel (`gemm_pair_kernel`,
// `cta_group::2`, 256 x 256 tile per pair of SMs) further down; the fused all-gather / reduce-scatter
// epilogues and the grouped modes use the single-CTA kernel.

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdint>
#include <cstdio>
#include <cstdlib>

#include "common.cuh"
#include "gemm_tcgen05.h"

namespace fs2 {

namespace {

constexpr int BM = 128;
constexpr int BN = 256;
constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr int STAGES = 4;
constexpr int A_BYTES = BM * BK * 2;            // 16 KB
constexpr int B_BYTES = BN * BK * 2;            // 32 KB
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;  // 48 KB
constexpr int EPI_BYTES = 128 * 128;            // 128 rows x 128 B
constexpr int MN_BLOCK_BYTES = 64 * 128;        // one [64 k-rows][64 mn] TMA box
constexpr int BAR_BYTES = 256;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 2 * EPI_BYTES + BAR_BYTES + 1024;
constexpr int TMEM_COLS = 512;
constexpr int NUM_THREADS = 192;
constexpr int GROUP_M = 16;
constexpr uint64_t WAIT_LIMIT_NS = 2000000000ull;

static_assert(SMEM_BYTES <= 232448, "shared memory budget of one CTA exceeded");

__device__ __forceinline__ uint32_t make_idesc(bool a_mn, bool b_mn) {
    uint32_t d = 0;
    d |= 1u << 4;                         // D format: f32
    d |= 1u << 7;                         // A format: bf16
    d |= 1u << 10;                        // B format: bf16
    d |= (a_mn ? 1u : 0u) << 15;          // A major: 0 = K, 1 = MN
    d |= (b_mn ? 1u : 0u) << 16;          // B major
    d |= static_cast<uint32_t>(BN >> 3) << 17;
    d |= static_cast<uint32_t>(BM >> 4) << 24;
    return d;
}

// Named barrier over the 128 epilogue threads that also ORs a predicate.
__device__ __forceinline__ bool epi_bar_or(bool pred) {
    uint32_t r;
    asm volatile(
        "{\n\t"
        ".reg .pred p, q;\n\t"
        "setp.ne.u32 p, %1, 0;\n\t"
        "barrier.cta.red.or.pred q, 1, 128, p;\n\t"
        "selp.u32 %0, 1, 0, q;\n\t"
        "}"
        : "=r"(r)
        : "r"(static_cast<uint32_t>(pred))
        : "memory");
    return r != 0;
}

__device__ __forceinline__ void epi_bar_sync() { asm volatile("barrier.cta.sync 1, 128;" ::: "memory"); }

// Tile order of the fused all-gather: blocks of the gathered operand are visited in arrival order (own shard,
// then the peers in ring order) and every block is used for all tiles that need it before moving on.
template <int GATHER>
__device__ __forceinline__ void gather_tile_coords(int t, int num_m, int num_n, int rank, int world, int per_rank,
                                                   int& m_tile, int& n_tile, int& gblock) {
    if constexpr (GATHER == 1) {
        const int idx = t / num_n;
        m_tile = ((rank + idx / per_rank) % world) * per_rank + idx % per_rank;
        n_tile = t % num_n;
        gblock = m_tile;
    } else {
        const int idx = t / num_m;
        n_tile = ((rank + idx / per_rank) % world) * per_rank + idx % per_rank;
        m_tile = t % num_m;
        gblock = n_tile;
    }
}

__device__ __forceinline__ void tile_coords(int t, int num_m, int num_n, int& m_tile, int& n_tile) {
    const int per_group = GROUP_M * num_n;
    const int g = t / per_group;
    const int first_m = g * GROUP_M;
    const int gsize = min(GROUP_M, num_m - first_m);
    const int r = t - g * per_group;
    m_tile = first_m + r % gsize;
    n_tile = r / gsize;
}

// Destination of the fused reduce-scatter epilogue: row block r of C (rows [r * rows_per_rank, (r + 1) *
// rows_per_rank)) is summed into `out[r]`, an fp32 [rows_per_rank, N] buffer in rank r's memory that this GPU
// reaches through a peer mapping.
struct PeerOut {
    void* out[8];
    int rows_per_rank;
    int slice;          // bf16 scatter mode: index of this rank's slice inside every owner's [world, rows, N] buffer
};

// Arguments of the fused all-gather: the gathered operand (A when GATHER == 1, B when GATHER == 2) is assembled in
// `dst` from the `world` row shards `src[r]` (peer mappings) by the first `ncopy` CTAs of the grid while the other
// CTAs compute. `flags[b]` reaches `epoch` once block b (BM rows of A / BN rows of B) has landed.
struct GatherArgs {
    const void* src[8];
    void* dst;
    unsigned int* flags;
    unsigned int epoch;
    int ncopy;
    int rows_per_rank;
    int rank;
    int world;
    long long row_bytes;
    int inplace;        // the own shard already sits at its place in `dst`: only the peers' shards are copied
    // Grouped (mixture-of-experts) modes, MODE 3 and 4; all tables live in device memory, nothing is read on the host
    const int* tile_row0;      // MODE 3: first row of m-tile i in the expert-sorted, 128-row padded activation buffer
    const int* tile_expert;    // MODE 3: expert of m-tile i
    const int* num_m_tiles;    // MODE 3: number of valid m-tiles
    const int* group_offsets;  // MODE 4: padded row offset of every expert, [experts + 1], multiples of 128
    int group_rows_b;          // MODE 3: rows one expert occupies in B's tensor map
    int experts;               // MODE 4
};

// Tile of a grouped GEMM (MODE 3: per-expert row blocks times a per-expert weight; MODE 4: per-expert weight gradient).
struct GroupedTile {
    int m0, n0, b_row_add, c_row0, kb_begin, kb_end;
};

template <int MODE>
__device__ __forceinline__ GroupedTile grouped_tile(int t, int num_m, int num_n, int M, const GatherArgs& ga) {
    GroupedTile g;
    if constexpr (MODE == 3) {
        const int mi = t / num_n;
        g.m0 = ga.tile_row0[mi];
        g.n0 = (t % num_n) * BN;
        g.b_row_add = ga.tile_expert[mi] * ga.group_rows_b;
        g.c_row0 = g.m0;
        g.kb_begin = 0;
        g.kb_end = -1;                   // caller substitutes the full K range
    } else {
        const int per = num_m * num_n;
        const int e = t / per, r = t % per;
        g.m0 = (r / num_n) * BM;
        g.n0 = (r % num_n) * BN;
        g.b_row_add = 0;
        g.c_row0 = e * M + g.m0;
        g.kb_begin = ga.group_offsets[e] / BK;
        g.kb_end = ga.group_offsets[e + 1] / BK;
    }
    return g;
}

// PEER_RED: instead of storing C locally, every tile goes straight into the memory of the rank that owns its rows,
// so a row-parallel GEMM and the reduce-scatter that follows it are one kernel and the NVLink traffic of tile i
// overlaps the tensor-core work of tile i + 1. Two forms: with OUT_F32 the fp32 tile is summed in place in the
// owner's [rows, N] buffer (red.global.add); without it the tile is rounded to bf16 and written with plain 16-byte
// stores into this rank's slice of the owner's [world, rows, N] buffer, and the owner sums the slices afterwards
// (half the bytes on the wire, no atomics, a deterministic sum).
//
// GATHER: all-gather of one operand fused into the GEMM. Copier CTAs pull the peers' shards over NVLink exactly
// once into local memory, block by block in the order in which the compute CTAs consume them (own shard first),
// and publish a flag per block; a compute CTA's TMA producer waits for the flag of the block its tile needs, so
// the GEMM starts on local data immediately and the remaining transfers hide behind tensor-core work.
template <bool A_MN, bool B_MN, bool OUT_F32, bool PEER_RED = false, int GATHER = 0>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
            const __grid_constant__ CUtensorMap tma_c, int M, int N, int K, int accumulate_and_splits, int* status,
            const PeerOut po, const GatherArgs ga) {
    int accumulate = accumulate_and_splits;
    constexpr bool kGather = GATHER == 1 || GATHER == 2;  // GATHER 3 / 4 are the grouped (MoE) modes
    constexpr int GROUPED = GATHER == 3 ? 1 : (GATHER == 4 ? 2 : 0);
    constexpr int GBLK = GATHER == 2 ? BN : BM;          // rows of the gathered operand per flag
    if constexpr (kGather) {
        if (static_cast<int>(blockIdx.x) < ga.ncopy) {
            // Copier CTA: one thread moves its blocks with bulk copies, peer memory -> shared memory -> local
            // memory, COPY_BUFS chunks of COPY_CHUNK bytes in flight, so no registers stage the data and ~200 KB
            // per copier CTA are outstanding on NVLink.
            if (threadIdx.x != 0) return;
            extern __shared__ uint8_t copier_smem[];
            const uint32_t craw = smem_u32(copier_smem);
            const uint32_t cbase = (craw + 1023u) & ~1023u;
            constexpr uint32_t COPY_CHUNK = 32768;
            constexpr int COPY_BUFS = STAGES * STAGE_BYTES / COPY_CHUNK;
            const uint32_t cbar = cbase + STAGES * STAGE_BYTES + 2 * EPI_BYTES;
            for (int b = 0; b < COPY_BUFS; ++b) mbar_init(cbar + 8 * b, 1);
            fence_barrier_init();
            const int per_rank = ga.rows_per_rank / GBLK;
            const int total = per_rank * ga.world;
            const long long blk_bytes = static_cast<long long>(GBLK) * ga.row_bytes;
            const int nch = static_cast<int>((blk_bytes + COPY_CHUNK - 1) / COPY_CHUNK);
            const int first = ga.inplace ? per_rank : 0;      // arrival order starts with the own shard
            if (ga.inplace && blockIdx.x == 0) {
                for (int b = 0; b < per_rank; ++b)
                    asm volatile("st.release.gpu.global.u32 [%0], %1;"
                                 ::"l"(ga.flags + ga.rank * per_rank + b), "r"(ga.epoch) : "memory");
            }
            const int mine = total - first - static_cast<int>(blockIdx.x);
            const int my_blocks = mine > 0 ? (mine + ga.ncopy - 1) / ga.ncopy : 0;
            const long long total_chunks = static_cast<long long>(my_blocks) * nch;
            int abort_local = 0;
            bool failed = false;
            // chunk c -> (source, destination, bytes, block, last chunk of its block?)
            auto locate = [&](long long c, const char*& from, char*& to, uint32_t& bytes, int& gblock, bool& last) {
                const int i = first + static_cast<int>(blockIdx.x) + static_cast<int>(c / nch) * ga.ncopy;
                const int k = static_cast<int>(c % nch);
                const int src_rank = (ga.rank + i / per_rank) % ga.world;
                const int bi = i % per_rank;
                gblock = src_rank * per_rank + bi;
                const long long off = static_cast<long long>(k) * COPY_CHUNK;
                from = static_cast<const char*>(ga.src[src_rank]) + bi * blk_bytes + off;
                to = static_cast<char*>(ga.dst) + gblock * blk_bytes + off;
                bytes = static_cast<uint32_t>(min(static_cast<long long>(COPY_CHUNK), blk_bytes - off));
                last = k == nch - 1;
            };
            auto issue_load = [&](long long c) {
                const char* from; char* to; uint32_t bytes; int gblock; bool last;
                locate(c, from, to, bytes, gblock, last);
                const int slot = static_cast<int>(c % COPY_BUFS);
                mbar_arrive_expect_tx(cbar + 8 * slot, bytes);
                bulk_load(cbase + slot * COPY_CHUNK, from, bytes, cbar + 8 * slot);
            };
            long long issued = 0;
            for (; issued < total_chunks && issued < COPY_BUFS; ++issued) issue_load(issued);
            long long c = 0;
            for (; c < total_chunks; ++c) {
                const int slot = static_cast<int>(c % COPY_BUFS);
                if (!mbar_wait_bounded(cbar + 8 * slot, static_cast<uint32_t>((c / COPY_BUFS) & 1), &abort_local,
                                       WAIT_LIMIT_NS)) {
                    report_status(status, 0x71);
                    failed = true;
                    break;
                }
                const char* from; char* to; uint32_t bytes; int gblock; bool last;
                locate(c, from, to, bytes, gblock, last);
                bulk_store(to, cbase + slot * COPY_CHUNK, bytes);
                tma_commit_group();
                if (last) {
                    tma_wait_group<0>();                                   // the whole block has landed
                    asm volatile("fence.proxy.async.global;" ::: "memory");
                    __threadfence();
                    asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(ga.flags + gblock), "r"(ga.epoch) : "memory");
                }
                if (issued < total_chunks) {
                    tma_wait_group_read<0>();                              // the store has read this buffer
                    issue_load(issued);
                    ++issued;
                }
            }
            tma_wait_group<0>();
            if (failed) {
                // loads still in flight target this CTA's shared memory: give each a bounded chance to land
                for (long long d = c + 1; d < issued; ++d)
                    mbar_wait_bounded(cbar + 8 * static_cast<int>(d % COPY_BUFS),
                                      static_cast<uint32_t>((d / COPY_BUFS) & 1), &abort_local, WAIT_LIMIT_NS);
            }
            return;
        }
    }
    const int ncopy = kGather ? ga.ncopy : 0;
    const int first_tile = static_cast<int>(blockIdx.x) - ncopy;
    const int tile_stride = static_cast<int>(gridDim.x) - ncopy;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t* smem = smem_raw + (base - raw);

    const uint32_t epi_base = base + STAGES * STAGE_BYTES;
    uint8_t* bar_ptr = smem + STAGES * STAGE_BYTES + 2 * EPI_BYTES;
    const uint32_t bar_base = smem_u32(bar_ptr);
    // barrier slots (8 B each): full[4] empty[4] tmem_full[2] tmem_empty[2]
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
    auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + a); };
    auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + 2 + a); };
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(bar_ptr + 8 * (2 * STAGES + 4));
    volatile int* abort_flag = reinterpret_cast<volatile int*>(bar_ptr + 8 * (2 * STAGES + 4) + 8);

    const int warp = __shfl_sync(0xffffffffu, threadIdx.x >> 5, 0);   // warp-uniform for the compiler
    const int lane = threadIdx.x & 31;

    const int num_m = GROUPED == 1 ? *ga.num_m_tiles : (M + BM - 1) / BM;
    const int num_n = (N + BN - 1) / BN;
    // split-K: `accumulate` carries the number of K splits in its bits 8 and up (0/1 = none). Tile t then covers
    // output tile t % (num_m * num_n) over the K range of split t / (num_m * num_n) and is reduce-added into C.
    const int k_splits = (accumulate >> 8) > 1 ? (accumulate >> 8) : 1;
    accumulate &= 1;
    const int num_mn = num_m * num_n;
    const int num_tiles = GROUPED == 2 ? num_mn * ga.experts : num_mn * k_splits;
    const int num_kb_total = (K + BK - 1) / BK;
    const int kb_per_split = (num_kb_total + k_splits - 1) / k_splits;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(tfull_bar(a), 1);
            mbar_init(tempty_bar(a), 128);
        }
        *abort_flag = 0;
        fence_barrier_init();
        prefetch_tmap(&tma_a);
        prefetch_tmap(&tma_b);
        prefetch_tmap(&tma_c);
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
        // ------------------------------------------------------------ producer
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int t = first_tile; t < num_tiles && ok; t += tile_stride) {
                int mt = 0, nt = 0;
                GroupedTile gt{};
                if constexpr (GROUPED != 0) {
                    gt = grouped_tile<GATHER>(t, num_m, num_n, M, ga);
                } else if constexpr (kGather) {
                    int gblock;
                    gather_tile_coords<GATHER>(t, num_m, num_n, ga.rank, ga.world, ga.rows_per_rank / GBLK, mt, nt, gblock);
                    // wait until the copier CTAs have landed this block of the gathered operand
                    const uint64_t t0 = global_timer_ns();
                    uint32_t seen, spins = 0;
                    while (true) {
                        asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(seen) : "l"(ga.flags + gblock) : "memory");
                        if (static_cast<int32_t>(seen - ga.epoch) >= 0) break;
                        if ((++spins & 63u) == 0 && (*abort_flag || global_timer_ns() - t0 > WAIT_LIMIT_NS)) {
                            if (!*abort_flag) report_status(status, kStatusTimeout | (5 << 8));
                            *abort_flag = 1;
                            ok = false;
                            break;
                        }
                    }
                    if (!ok) break;
                    fence_proxy_async_smem();
                    asm volatile("fence.proxy.async.global;" ::: "memory");   // generic-proxy copies -> TMA reads
                } else {
                    tile_coords(t % num_mn, num_m, num_n, mt, nt);
                }
                const int m0 = GROUPED != 0 ? gt.m0 : mt * BM, n0 = GROUPED != 0 ? gt.n0 : nt * BN;
                const int b_add = GROUPED != 0 ? gt.b_row_add : 0;
                int kb_begin = (t / num_mn) * kb_per_split;
                int kb_end = min(num_kb_total, kb_begin + kb_per_split);
                if constexpr (GROUPED == 1) { kb_begin = 0; kb_end = num_kb_total; }
                if constexpr (GROUPED == 2) { kb_begin = gt.kb_begin; kb_end = gt.kb_end; }
                for (int kb = kb_begin; kb < kb_end; ++kb) {
                    if (!mbar_wait_bounded(empty_bar(stage), phase ^ 1u, abort_flag, WAIT_LIMIT_NS)) {
                        if (!*abort_flag) report_status(status, kStatusTimeout | (1 << 8));
                        *abort_flag = 1;
                        ok = false;
                        break;
                    }
                    const uint32_t a_s = base + stage * STAGE_BYTES;
                    const uint32_t b_s = a_s + A_BYTES;
                    const uint32_t fb = full_bar(stage);
                    mbar_arrive_expect_tx(fb, STAGE_BYTES);
                    const int k0 = kb * BK;
                    if constexpr (!A_MN) {
                        tma_load_2d(a_s, &tma_a, fb, k0, m0);
                    } else {
#pragma unroll
                        for (int h = 0; h < BM / 64; ++h) tma_load_2d(a_s + h * MN_BLOCK_BYTES, &tma_a, fb, m0 + h * 64, k0);
                    }
                    if constexpr (!B_MN) {
                        tma_load_2d(b_s, &tma_b, fb, k0, n0 + b_add);
                    } else {
#pragma unroll
                        for (int h = 0; h < BN / 64; ++h)
                            tma_load_2d(b_s + h * MN_BLOCK_BYTES, &tma_b, fb, n0 + h * 64, k0 + b_add);
                    }
                    if (++stage == STAGES) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ---------------------------------------------------------- MMA issuer
        // The whole warp runs the loop converged and only the tcgen05 instructions are predicated on one elected
        // lane: descriptors and addresses then stay in uniform registers. Inside a divergent `if (lane == 0)` every
        // operand is moved to a uniform register per instruction, which costs tens of cycles per MMA.
        const bool issue = elect_one();
        const uint32_t tmem = __shfl_sync(0xffffffffu, tmem_base, 0);
        auto fail = [&](int code) {
            if (issue) {
                if (!*abort_flag) report_status(status, kStatusTimeout | (code << 8));
                *abort_flag = 1;
            }
        };
        const uint32_t idesc = make_idesc(A_MN, B_MN);
        int stage = 0;
        uint32_t phase = 0;
        int acc = 0;
        uint32_t acc_phase = 0;
        bool ok = true;
        for (int t = first_tile; t < num_tiles && ok; t += tile_stride) {
            if (!mbar_wait_bounded(tempty_bar(acc), acc_phase ^ 1u, abort_flag, WAIT_LIMIT_NS)) {
                fail(2);
                break;
            }
            tcgen05_fence_after();
            const uint32_t d_tmem = tmem + static_cast<uint32_t>(acc * BN);
            int kb_begin = (t / num_mn) * kb_per_split;
            int kb_end = min(num_kb_total, kb_begin + kb_per_split);
            if constexpr (GROUPED == 1) { kb_begin = 0; kb_end = num_kb_total; }
            if constexpr (GROUPED == 2) {
                const GroupedTile gt = grouped_tile<GATHER>(t, num_m, num_n, M, ga);
                kb_begin = gt.kb_begin;
                kb_end = gt.kb_end;
            }
            for (int kb = kb_begin; kb < kb_end; ++kb) {
                if (!mbar_wait_bounded(full_bar(stage), phase, abort_flag, WAIT_LIMIT_NS)) {
                    fail(3);
                    ok = false;
                    break;
                }
                tcgen05_fence_after();
                const uint32_t a_s = base + stage * STAGE_BYTES;
                const uint32_t b_s = a_s + A_BYTES;
                if (issue) {
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k) {
                        uint64_t da, db;
                        if constexpr (!A_MN) da = make_smem_desc(a_s + k * UMMA_K * 2, 16, 1024);
                        else da = make_smem_desc(a_s + k * UMMA_K * 128, MN_BLOCK_BYTES, 1024);
                        if constexpr (!B_MN) db = make_smem_desc(b_s + k * UMMA_K * 2, 16, 1024);
                        else db = make_smem_desc(b_s + k * UMMA_K * 128, MN_BLOCK_BYTES, 1024);
                        umma_bf16(d_tmem, da, db, idesc, (kb > kb_begin || k > 0) ? 1u : 0u);
                    }
                    umma_commit(empty_bar(stage));
                }
                if (++stage == STAGES) {
                    stage = 0;
                    phase ^= 1u;
                }
            }
            if (!ok) break;
            if (issue) umma_commit(tfull_bar(acc));
            acc ^= 1;
            if (acc == 0) acc_phase ^= 1u;
        }
        __syncwarp();
    } else {
        // ------------------------------------------------------------ epilogue
        const int q = warp & 3;                       // TMEM lane quadrant of this warp
        const int row = q * 32 + lane;                // row inside the CTA tile
        const bool leader = (threadIdx.x == 64);      // first epilogue thread issues the stores
        constexpr int CHUNK_COLS = OUT_F32 ? 32 : 64;
        constexpr int NCHUNK = BN / CHUNK_COLS;
        int acc = 0;
        uint32_t acc_phase = 0;
        int buf = 0;
        for (int t = first_tile; t < num_tiles; t += tile_stride) {
            int mt = 0, nt = 0;
            GroupedTile gt{};
            if constexpr (GROUPED != 0) {
                gt = grouped_tile<GATHER>(t, num_m, num_n, M, ga);
            } else if constexpr (kGather) {
                int gblock;
                gather_tile_coords<GATHER>(t, num_m, num_n, ga.rank, ga.world, ga.rows_per_rank / GBLK, mt, nt, gblock);
            } else {
                tile_coords(t % num_mn, num_m, num_n, mt, nt);
            }
            const int m0 = GROUPED != 0 ? gt.c_row0 : mt * BM, n0 = GROUPED != 0 ? gt.n0 : nt * BN;
            const bool got = mbar_wait_bounded(tfull_bar(acc), acc_phase, abort_flag, WAIT_LIMIT_NS);
            if (epi_bar_or(!got)) {
                if (leader && !*abort_flag) report_status(status, kStatusTimeout | (4 << 8));
                *abort_flag = 1;
                break;
            }
            tcgen05_fence_after();
            const uint32_t t_row = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + static_cast<uint32_t>(acc * BN);
#pragma unroll 1
            for (int c = 0; c < NCHUNK; ++c) {
                const int col0 = c * CHUNK_COLS;
                if (n0 + col0 >= N) break;  // uniform over the CTA
                if constexpr (!PEER_RED) {
                    if (leader) tma_wait_group_read<1>();
                }
                epi_bar_sync();
                const uint32_t sbuf = epi_base + buf * EPI_BYTES;
                const uint32_t srow = sbuf + row * 128;
                if constexpr (OUT_F32) {
                    uint32_t v[32];
                    tmem_ld_32x32(t_row + col0, v);
                    tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        const uint32_t dst = srow + (((j ^ (row & 7)) & 7) << 4);
                        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(v[4 * j]),
                                     "r"(v[4 * j + 1]), "r"(v[4 * j + 2]), "r"(v[4 * j + 3])
                                     : "memory");
                    }
                } else {
                    uint32_t v[64];
                    tmem_ld_32x32(t_row + col0, v);
                    tmem_ld_32x32(t_row + col0 + 32, v + 32);
                    tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        uint32_t p[4];
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(v[8 * j + 2 * e]),
                                                                      __uint_as_float(v[8 * j + 2 * e + 1]));
                            p[e] = *reinterpret_cast<uint32_t*>(&h);
                        }
                        const uint32_t dst = srow + (((j ^ (row & 7)) & 7) << 4);
                        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(p[0]), "r"(p[1]),
                                     "r"(p[2]), "r"(p[3])
                                     : "memory");
                    }
                }
                if constexpr (PEER_RED) {
                    epi_bar_sync();
                    // 128 threads sweep the staged [128 rows][128 bytes] chunk: 8 threads cover one 128-byte row
                    // segment, so every instruction of a warp touches four full 128-byte lines of the owner
                    const int e = static_cast<int>(threadIdx.x) - 64;
                    const int j = e & 7;
                    constexpr int PER16 = OUT_F32 ? 4 : 8;              // elements per 16-byte piece
#pragma unroll
                    for (int it = 0; it < 8; ++it) {
                        const int r = it * 16 + (e >> 3);
                        const int grow = m0 + r, gcol = n0 + col0 + j * PER16;
                        if (grow < M && gcol < N) {
                            const uint32_t src = sbuf + r * 128 + (((j ^ (r & 7)) & 7) << 4);
                            const int owner = grow / po.rows_per_rank;
                            const size_t lrow = static_cast<size_t>(grow - owner * po.rows_per_rank);
                            if constexpr (OUT_F32) {
                                float4 v;
                                asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];"
                                             : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(src));
                                float* dst = static_cast<float*>(po.out[owner]) + lrow * N + gcol;
                                asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};"
                                             ::"l"(dst), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
                            } else {
                                uint4 v;
                                asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                                             : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(src));
                                __nv_bfloat16* dst = static_cast<__nv_bfloat16*>(po.out[owner]) +
                                    (static_cast<size_t>(po.slice) * po.rows_per_rank + lrow) * N + gcol;
                                asm volatile("st.global.v4.b32 [%0], {%1, %2, %3, %4};"
                                             ::"l"(dst), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
                            }
                        }
                    }
                } else {
                    fence_proxy_async_smem();
                    epi_bar_sync();
                    if (leader) {
                        if (accumulate) tma_reduce_add_2d(&tma_c, sbuf, n0 + col0, m0);
                        else tma_store_2d(&tma_c, sbuf, n0 + col0, m0);
                        tma_commit_group();
                    }
                }
                buf ^= 1;
            }
            tcgen05_fence_before();
            mbar_arrive(tempty_bar(acc));
            acc ^= 1;
            if (acc == 0) acc_phase ^= 1u;
        }
        if constexpr (!PEER_RED) {
            if (leader) tma_wait_group<0>();
        }
    }

    // -------------------------------------------------------------- teardown
    __syncthreads();
    if (*abort_flag) {
        // Give copies that were already in flight time to land before the CTA retires.
        const uint64_t t0 = global_timer_ns();
        while (global_timer_ns() - t0 < 200000ull) __nanosleep(1000);
        __syncthreads();
    }
    tcgen05_fence_after();
    if (warp == 1) tmem_dealloc(tmem_base, TMEM_COLS);
}

// ================================================================= CTA-pair kernel
// The plain GEMM on pairs of CTAs (`cta_group::2`): a cluster of two CTAs on neighbouring SMs computes a 256 x 256
// tile with ONE stream of tcgen05.mma issued by the first CTA of the pair. Each CTA stages its own 128 rows of A and
// only ITS HALF (128 rows) of the B tile, so per MMA it reads 8 KB of operands from shared memory instead of 12 KB and
// loads a third less from L2; the accumulator rows of each CTA stay in its own tensor memory and its own epilogue
// warps write them out. Under the power cap (where a long training step runs) this is what separates the
// single-CTA kernel from a library GEMM.
//
// Synchronisation across the pair: both producers issue their TMA loads against the FIRST CTA's "full" barrier
// (`cp.async.bulk.tensor ... cta_group::2`, one expect-tx of the pair's bytes by the first CTA); the issuer releases
// a stage and publishes an accumulator with commits that arrive on the barrier of the same name in both CTAs; the
// second CTA's epilogue threads arrive on the first CTA's "accumulator drained" barrier through its cluster address.
// Every wait is bounded as in the single-CTA kernel.
constexpr int STAGES2 = 6;
constexpr int B2_BYTES = 128 * BK * 2;               // this CTA's half of the 256-row B tile
constexpr int STAGE2_BYTES = A_BYTES + B2_BYTES;     // 32 KB
constexpr int SMEM2_BYTES = STAGES2 * STAGE2_BYTES + 2 * EPI_BYTES + BAR_BYTES + 1024;
static_assert(SMEM2_BYTES <= 232448, "shared memory budget of one CTA exceeded");

__device__ __forceinline__ uint32_t cluster_cta_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}

__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// The address, in the cluster's shared window, of `addr` in the shared memory of CTA `rank` of the cluster.
__device__ __forceinline__ uint32_t cluster_map(uint32_t addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}

__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}

// TMA load into this CTA's shared memory whose bytes are counted on a barrier of the pair's first CTA.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t smem_dst, const void* tmap, uint32_t bar_cluster_addr, int x,
                                                 int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_dst), "l"(tmap), "r"(bar_cluster_addr), "r"(x), "r"(y)
        : "memory");
}

__device__ __forceinline__ void umma_bf16_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                               uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t"
        "}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}

// Arrives, once the MMAs issued so far are done, on the barrier at offset `bar` in BOTH CTAs of the pair (two
// commits: this CTA's barrier and, through its cluster address, the partner's).
__device__ __forceinline__ void umma_commit_pair(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];"
                 ::"r"(cluster_map(bar, 1)) : "memory");
}

__device__ __forceinline__ uint32_t make_idesc_pair(bool a_mn, bool b_mn) {
    uint32_t d = 0;
    d |= 1u << 4;                         // D format: f32
    d |= 1u << 7;                         // A format: bf16
    d |= 1u << 10;                        // B format: bf16
    d |= (a_mn ? 1u : 0u) << 15;
    d |= (b_mn ? 1u : 0u) << 16;
    d |= static_cast<uint32_t>(256 >> 3) << 17;   // N
    d |= static_cast<uint32_t>(256 >> 4) << 24;   // M of the pair
    return d;
}

template <bool A_MN, bool B_MN, bool OUT_F32>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                 const __grid_constant__ CUtensorMap tma_c, int M, int N, int K, int accumulate, int tail_splits,
                 int* status) {
    const uint32_t cta = cluster_cta_rank();          // 0 = the CTA that issues the MMAs
    const int first_tile = static_cast<int>(blockIdx.x >> 1);
    const int tile_stride = static_cast<int>(gridDim.x >> 1);
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t* smem = smem_raw + (base - raw);

    const uint32_t epi_base = base + STAGES2 * STAGE2_BYTES;
    uint8_t* bar_ptr = smem + STAGES2 * STAGE2_BYTES + 2 * EPI_BYTES;
    const uint32_t bar_base = smem_u32(bar_ptr);
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES2 + s); };
    auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * STAGES2 + a); };
    auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * STAGES2 + 2 + a); };
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(bar_ptr + 8 * (2 * STAGES2 + 4));
    volatile int* abort_flag = reinterpret_cast<volatile int*>(bar_ptr + 8 * (2 * STAGES2 + 4) + 8);

    const int warp = __shfl_sync(0xffffffffu, threadIdx.x >> 5, 0);
    const int lane = threadIdx.x & 31;

    constexpr int PM = 2 * BM;                         // rows of the pair's tile
    const int num_m = (M + PM - 1) / PM;
    const int num_n = (N + BN - 1) / BN;
    const int k_splits = (accumulate >> 8) > 1 ? (accumulate >> 8) : 1;
    accumulate &= 1;
    const int num_mn = num_m * num_n;
    const int num_kb_total = (K + BK - 1) / BK;
    const int kb_per_split = (num_kb_total + k_splits - 1) / k_splits;
    // Work units. Normally unit u is output tile u % num_mn over the K range of split u / num_mn. With
    // `tail_splits` > 1 (no global split-K) the tiles of the last, partial wave are each cut into `tail_splits`
    // K slices that are reduce-added into C, so that the pairs which would idle in that wave share its work.
    const int full_tiles = tail_splits > 1 ? (num_mn / tile_stride) * tile_stride : num_mn;
    const int kb_per_tail = tail_splits > 1 ? (num_kb_total + tail_splits - 1) / tail_splits : num_kb_total;
    const int num_tiles = tail_splits > 1 ? full_tiles + (num_mn - full_tiles) * tail_splits : num_mn * k_splits;
    auto unit = [&](int u, int& tile, int& kb_begin, int& kb_end, int& acc_flag) {
        if (tail_splits > 1) {
            if (u < full_tiles) {
                tile = u;
                kb_begin = 0;
                kb_end = num_kb_total;
                acc_flag = accumulate;
            } else {
                const int v = u - full_tiles;
                tile = full_tiles + v / tail_splits;
                kb_begin = (v % tail_splits) * kb_per_tail;
                kb_end = min(num_kb_total, kb_begin + kb_per_tail);
                acc_flag = 1;
            }
        } else {
            tile = u % num_mn;
            kb_begin = (u / num_mn) * kb_per_split;
            kb_end = min(num_kb_total, kb_begin + kb_per_split);
            acc_flag = accumulate;
        }
    };

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES2; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(tfull_bar(a), 1);
            mbar_init(tempty_bar(a), 256);             // the epilogue threads of both CTAs
        }
        *abort_flag = 0;
        fence_barrier_init();
        prefetch_tmap(&tma_a);
        prefetch_tmap(&tma_b);
        prefetch_tmap(&tma_c);
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(const_cast<uint32_t*>(tmem_slot))), "r"(static_cast<uint32_t>(TMEM_COLS)) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tcgen05_fence_before();
    __syncthreads();
    cluster_sync_all();                                // the partner's barriers exist before anything signals them
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ------------------------------------------------------------ producer (both CTAs)
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int t = first_tile; t < num_tiles && ok; t += tile_stride) {
                int tile, kb_begin, kb_end, acc_flag, mt, nt;
                unit(t, tile, kb_begin, kb_end, acc_flag);
                tile_coords(tile, num_m, num_n, mt, nt);
                const int m0 = mt * PM + static_cast<int>(cta) * BM;       // this CTA's rows of A
                const int n0 = nt * BN + static_cast<int>(cta) * (BN / 2); // this CTA's half of B
                for (int kb = kb_begin; kb < kb_end; ++kb) {
                    if (!mbar_wait_bounded(empty_bar(stage), phase ^ 1u, abort_flag, WAIT_LIMIT_NS)) {
                        if (!*abort_flag) report_status(status, kStatusTimeout | (0x11 << 8));
                        *abort_flag = 1;
                        ok = false;
                        break;
                    }
                    const uint32_t a_s = base + stage * STAGE2_BYTES;
                    const uint32_t b_s = a_s + A_BYTES;
                    if (cta == 0) mbar_arrive_expect_tx(full_bar(stage), 2 * STAGE2_BYTES);
                    const uint32_t fb = cluster_map(full_bar(stage), 0);
                    const int k0 = kb * BK;
                    if constexpr (!A_MN) {
                        tma_load_2d_pair(a_s, &tma_a, fb, k0, m0);
                    } else {
#pragma unroll
                        for (int h = 0; h < BM / 64; ++h) tma_load_2d_pair(a_s + h * MN_BLOCK_BYTES, &tma_a, fb, m0 + h * 64, k0);
                    }
                    if constexpr (!B_MN) {
                        tma_load_2d_pair(b_s, &tma_b, fb, k0, n0);
                    } else {
#pragma unroll
                        for (int h = 0; h < BN / 2 / 64; ++h)
                            tma_load_2d_pair(b_s + h * MN_BLOCK_BYTES, &tma_b, fb, n0 + h * 64, k0);
                    }
                    if (++stage == STAGES2) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ---------------------------------------------------------- MMA issuer (first CTA of the pair only)
        if (cta == 0) {
            const bool issue = elect_one();
            const uint32_t tmem = __shfl_sync(0xffffffffu, tmem_base, 0);
            auto fail = [&](int code) {
                if (issue) {
                    if (!*abort_flag) report_status(status, kStatusTimeout | (code << 8));
                    *abort_flag = 1;
                }
            };
            const uint32_t idesc = make_idesc_pair(A_MN, B_MN);
            int stage = 0;
            uint32_t phase = 0;
            int acc = 0;
            uint32_t acc_phase = 0;
            bool ok = true;
            for (int t = first_tile; t < num_tiles && ok; t += tile_stride) {
                if (!mbar_wait_bounded(tempty_bar(acc), acc_phase ^ 1u, abort_flag, WAIT_LIMIT_NS)) {
                    fail(0x12);
                    break;
                }
                tcgen05_fence_after();
                const uint32_t d_tmem = tmem + static_cast<uint32_t>(acc * BN);
                int tile, kb_begin, kb_end, acc_flag;
                unit(t, tile, kb_begin, kb_end, acc_flag);
                for (int kb = kb_begin; kb < kb_end; ++kb) {
                    if (!mbar_wait_bounded(full_bar(stage), phase, abort_flag, WAIT_LIMIT_NS)) {
                        fail(0x13);
                        ok = false;
                        break;
                    }
                    tcgen05_fence_after();
                    const uint32_t a_s = base + stage * STAGE2_BYTES;
                    const uint32_t b_s = a_s + A_BYTES;
                    if (issue) {
#pragma unroll
                        for (int k = 0; k < BK / UMMA_K; ++k) {
                            uint64_t da, db;
                            if constexpr (!A_MN) da = make_smem_desc(a_s + k * UMMA_K * 2, 16, 1024);
                            else da = make_smem_desc(a_s + k * UMMA_K * 128, MN_BLOCK_BYTES, 1024);
                            if constexpr (!B_MN) db = make_smem_desc(b_s + k * UMMA_K * 2, 16, 1024);
                            else db = make_smem_desc(b_s + k * UMMA_K * 128, MN_BLOCK_BYTES, 1024);
                            umma_bf16_pair(d_tmem, da, db, idesc, (kb > kb_begin || k > 0) ? 1u : 0u);
                        }
                        umma_commit_pair(empty_bar(stage));
                    }
                    if (++stage == STAGES2) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
                if (!ok) break;
                if (issue) umma_commit_pair(tfull_bar(acc));
                acc ^= 1;
                if (acc == 0) acc_phase ^= 1u;
            }
            __syncwarp();
        }
    } else {
        // ------------------------------------------------------------ epilogue (both CTAs, own accumulator rows)
        const int q = warp & 3;
        const int row = q * 32 + lane;
        const bool leader = (threadIdx.x == 64);
        constexpr int CHUNK_COLS = OUT_F32 ? 32 : 64;
        constexpr int NCHUNK = BN / CHUNK_COLS;
        int acc = 0;
        uint32_t acc_phase = 0;
        int buf = 0;
        for (int t = first_tile; t < num_tiles; t += tile_stride) {
            int tile, kb_begin, kb_end, acc_flag, mt, nt;
            unit(t, tile, kb_begin, kb_end, acc_flag);
            tile_coords(tile, num_m, num_n, mt, nt);
            const int m0 = mt * PM + static_cast<int>(cta) * BM, n0 = nt * BN;
            const bool got = mbar_wait_bounded(tfull_bar(acc), acc_phase, abort_flag, WAIT_LIMIT_NS);
            if (epi_bar_or(!got)) {
                if (leader && !*abort_flag) report_status(status, kStatusTimeout | (0x14 << 8));
                *abort_flag = 1;
                break;
            }
            tcgen05_fence_after();
            const uint32_t t_row = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + static_cast<uint32_t>(acc * BN);
#pragma unroll 1
            for (int c = 0; c < NCHUNK; ++c) {
                const int col0 = c * CHUNK_COLS;
                if (n0 + col0 >= N) break;  // uniform over the CTA
                if (leader) tma_wait_group_read<1>();
                epi_bar_sync();
                const uint32_t sbuf = epi_base + buf * EPI_BYTES;
                const uint32_t srow = sbuf + row * 128;
                if constexpr (OUT_F32) {
                    uint32_t v[32];
                    tmem_ld_32x32(t_row + col0, v);
                    tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        const uint32_t dst = srow + (((j ^ (row & 7)) & 7) << 4);
                        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(v[4 * j]),
                                     "r"(v[4 * j + 1]), "r"(v[4 * j + 2]), "r"(v[4 * j + 3])
                                     : "memory");
                    }
                } else {
                    uint32_t v[64];
                    tmem_ld_32x32(t_row + col0, v);
                    tmem_ld_32x32(t_row + col0 + 32, v + 32);
                    tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        uint32_t pk[4];
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(v[8 * j + 2 * e]),
                                                                      __uint_as_float(v[8 * j + 2 * e + 1]));
                            pk[e] = *reinterpret_cast<uint32_t*>(&h);
                        }
                        const uint32_t dst = srow + (((j ^ (row & 7)) & 7) << 4);
                        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(pk[0]), "r"(pk[1]),
                                     "r"(pk[2]), "r"(pk[3])
                                     : "memory");
                    }
                }
                fence_proxy_async_smem();
                epi_bar_sync();
                if (leader && m0 < M) {
                    if (acc_flag) tma_reduce_add_2d(&tma_c, sbuf, n0 + col0, m0);
                    else tma_store_2d(&tma_c, sbuf, n0 + col0, m0);
                    tma_commit_group();
                }
                buf ^= 1;
            }
            tcgen05_fence_before();
            // "accumulator drained" lives in the first CTA of the pair
            if (cta == 0) mbar_arrive(tempty_bar(acc));
            else mbar_arrive_cluster(cluster_map(tempty_bar(acc), 0));
            acc ^= 1;
            if (acc == 0) acc_phase ^= 1u;
        }
        if (leader) tma_wait_group<0>();
    }

    // -------------------------------------------------------------- teardown
    __syncthreads();
    if (*abort_flag) {
        const uint64_t t0 = global_timer_ns();
        while (global_timer_ns() - t0 < 200000ull) __nanosleep(1000);
        __syncthreads();
    }
    cluster_sync_all();       // neither CTA leaves while its partner may still signal its barriers or read its tiles
    tcgen05_fence_after();
    if (warp == 1)
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                     "r"(static_cast<uint32_t>(TMEM_COLS)) : "memory");
}

// ---------------------------------------------------------------- host side
using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                              const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                              CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeFn get_encode_fn() {
    static EncodeFn fn = nullptr;
    if (fn == nullptr) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult qres;
        cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres);
        if (e != cudaSuccess || p == nullptr) return nullptr;
        fn = reinterpret_cast<EncodeFn>(p);
    }
    return fn;
}

// 2-D row-major tensor [rows, cols] of `elem_bytes` elements; box [box_rows, box_cols].
thread_local char g_tmap_err[256];

// `ld` is the distance between consecutive rows in elements (0 = `cols`, a dense matrix). It may be SMALLER than
// `cols`: rows then overlap in memory, which is how a strided convolution over a channels-last signal becomes a GEMM
// without materialising the patches.
bool make_tmap(CUtensorMap* m, const void* ptr, CUtensorMapDataType dt, int elem_bytes, uint64_t rows, uint64_t cols,
               uint32_t box_rows, uint32_t box_cols, uint64_t ld = 0) {
    EncodeFn fn = get_encode_fn();
    if (fn == nullptr) {
        snprintf(g_tmap_err, sizeof(g_tmap_err), "cuTensorMapEncodeTiled entry point not found");
        return false;
    }
    cuuint64_t dims[2] = {cols, rows};
    cuuint64_t strides[1] = {(ld ? ld : cols) * static_cast<uint64_t>(elem_bytes)};
    cuuint32_t box[2] = {box_cols, box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(m, dt, 2, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        snprintf(g_tmap_err, sizeof(g_tmap_err),
                 "cuTensorMapEncodeTiled failed with CUresult %d (ptr %p, rows %llu, cols %llu, elem %d B, box %ux%u)",
                 static_cast<int>(r), ptr, static_cast<unsigned long long>(rows),
                 static_cast<unsigned long long>(cols), elem_bytes, box_rows, box_cols);
        return false;
    }
    return true;
}

template <bool A_MN, bool B_MN, bool OUT_F32>
cudaError_t launch(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc, int M, int N, int K,
                   int accumulate, int* status, int num_sms, cudaStream_t stream, int k_splits = 1) {
    auto kern = gemm_kernel<A_MN, B_MN, OUT_F32>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
        if (e != cudaSuccess) return e;
        configured = true;
    }
    const int num_kb = (K + BK - 1) / BK;
    if (k_splits > num_kb) k_splits = num_kb;
    if (k_splits > 1) {                       // no empty splits: ceil(num_kb / ceil(num_kb / splits))
        const int per = (num_kb + k_splits - 1) / k_splits;
        k_splits = (num_kb + per - 1) / per;
    }
    if (k_splits < 1) k_splits = 1;
    const int num_tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN) * k_splits;
    const int grid = num_tiles < num_sms ? num_tiles : num_sms;
    kern<<<grid, NUM_THREADS, SMEM_BYTES, stream>>>(ta, tb, tc, M, N, K, (accumulate & 1) | (k_splits << 8), status,
                                                    PeerOut{}, GatherArgs{});
    return cudaGetLastError();
}

// Launch of the CTA-pair kernel: clusters of two CTAs, as many pairs as the device can keep resident at once (a pair
// needs two free SMs of one GPC, so this can be fewer than num_sms / 2).
template <bool A_MN, bool B_MN, bool OUT_F32>
cudaError_t launch_pair(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc, int M, int N, int K,
                        int accumulate, int* status, int num_sms, cudaStream_t stream, int k_splits,
                        void* dense_c, size_t c_elem_bytes) {
    auto kern = gemm_pair_kernel<A_MN, B_MN, OUT_F32>;
    static int max_pairs = 0;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cudaLaunchConfig_t cfg{};
    cfg.blockDim = dim3(NUM_THREADS);
    cfg.dynamicSmemBytes = SMEM2_BYTES;
    cfg.stream = stream;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (max_pairs == 0) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM2_BYTES);
        if (e != cudaSuccess) return e;
        cfg.gridDim = dim3(static_cast<unsigned>(num_sms & ~1));
        int n = 0;
        e = cudaOccupancyMaxActiveClusters(&n, kern, &cfg);
        if (e != cudaSuccess) return e;
        if (n < 1) return cudaErrorInvalidConfiguration;
        max_pairs = n;
    }
    const int num_kb = (K + BK - 1) / BK;
    if (k_splits > num_kb) k_splits = num_kb;
    if (k_splits > 1) {
        const int per = (num_kb + k_splits - 1) / k_splits;
        k_splits = (num_kb + per - 1) / per;
    }
    if (k_splits < 1) k_splits = 1;
    const int num_mn = ((M + 2 * BM - 1) / (2 * BM)) * ((N + BN - 1) / BN);
    const int num_tiles = num_mn * k_splits;
    const int pairs = std::min(std::min(num_tiles, max_pairs), num_sms / 2);
    cfg.gridDim = dim3(static_cast<unsigned>(2 * pairs));
    // Partial last wave: cut its tiles along K so that every pair has work (see the kernel). Worth it when the
    // time saved exceeds that of zeroing C, which the reduce-adds of the slices need unless C is accumulated into.
    int tail_splits = 1;
    const int rem = num_mn % pairs;
    if (k_splits == 1 && num_mn > pairs && rem > 0 && (accumulate || dense_c != nullptr)) {
        // two slices at most: a + b is the same in either order, so the result does not depend on which pair
        // finishes first (three or more reduce-adds would make the last bit vary from run to run)
        int sp = std::min(std::min(pairs / rem, 2), num_kb / 8);
        if (sp > 1) {
            const int per = (num_kb + sp - 1) / sp;
            sp = (num_kb + per - 1) / per;                      // no empty slice
        }
        if (sp > 1) {
            const double tile_us = 2.0 * 256 * 256 * K / (1.35e15 / 74) * 1e6;
            const double saved_us = tile_us * (1.0 - 1.0 / sp);
            const double zero_us = accumulate ? 0.0 : 2.0 + static_cast<double>(M) * N * c_elem_bytes / 5.0e6;
            if (saved_us > 1.5 * zero_us) {
                tail_splits = sp;
                if (!accumulate) {
                    cudaError_t e = cudaMemsetAsync(dense_c, 0, static_cast<size_t>(M) * N * c_elem_bytes, stream);
                    if (e != cudaSuccess) return e;
                }
            }
        }
    }
    return cudaLaunchKernelEx(&cfg, kern, ta, tb, tc, M, N, K, (accumulate & 1) | (k_splits << 8), tail_splits, status);
}

// The pair kernel is used for plain GEMMs that are large enough to fill the device with 256 x 256 tiles;
// FAIRSEQ2_B200_GEMM_PAIR=0 selects the single-CTA kernel for them as well.
bool pair_kernel_enabled() {
    const char* e = std::getenv("FAIRSEQ2_B200_GEMM_PAIR");      // read per call: tests switch it
    return e == nullptr || e[0] != '0';
}

}  // namespace

const char* gemm_bf16_tcgen05(const void* a, const void* b, void* c, int M, int N, int K, bool a_mn, bool b_mn,
                              bool out_f32, bool accumulate, int* status, int num_sms, cudaStream_t stream) {
    return gemm_bf16_tcgen05_view(a, 0, 0, b, 0, 0, c, 0, 0, M, N, K, a_mn, b_mn, out_f32, accumulate, status, num_sms,
                                  stream, 1);
}

const char* gemm_bf16_tcgen05_view(const void* a, long long lda, long long a_rows, const void* b, long long ldb,
                                   long long b_rows, void* c, long long ldc, long long c_rows, int M, int N, int K,
                                   bool a_mn, bool b_mn, bool out_f32, bool accumulate, int* status, int num_sms,
                                   cudaStream_t stream, int k_splits) {
    if (k_splits > 1 && !accumulate) return "gemm: split-K needs accumulate (a zeroed or meaningful output)";
    CUtensorMap ta, tb, tc;
    bool ok = true;
    g_tmap_err[0] = 0;
    // `*_rows` (0 = all) is the number of rows that exist in memory; tiles beyond it read zeros / are not written
    const uint64_t ar = a_rows ? a_rows : (a_mn ? K : M), br = b_rows ? b_rows : (b_mn ? K : N);
    const uint64_t cr = c_rows ? c_rows : M;
    if (!a_mn) ok = ok && make_tmap(&ta, a, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, ar, K, BM, BK, lda);
    else ok = ok && make_tmap(&ta, a, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, ar, M, BK, 64, lda);
    if (!b_mn) ok = ok && make_tmap(&tb, b, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, br, K, BN, BK, ldb);
    else ok = ok && make_tmap(&tb, b, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, br, N, BK, 64, ldb);
    if (out_f32) ok = ok && make_tmap(&tc, c, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, cr, N, 128, 32, ldc);
    else ok = ok && make_tmap(&tc, c, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, cr, N, 128, 64, ldc);
    if (!ok) return g_tmap_err;
    cudaError_t e;
    const int acc = accumulate ? 1 : 0;
    const long long tiles256 = static_cast<long long>((M + 255) / 256) * ((N + 255) / 256) * (k_splits > 1 ? k_splits : 1);
    if (pair_kernel_enabled() && tiles256 >= num_sms / 2) {
        // each CTA of a pair loads 128 rows of a K-major B
        if (!b_mn && !make_tmap(&tb, b, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, br, K, 128, BK, ldb)) return g_tmap_err;
        // the tail split zeroes C first unless it accumulates: only for a dense, fully present C
        void* dense_c = (ldc == 0 || ldc == N) && (c_rows == 0 || c_rows >= M) ? c : nullptr;
        const size_t c_elem = out_f32 ? 4 : 2;
#define FS2_LAUNCH2(AM, BMN, F32) \
    e = launch_pair<AM, BMN, F32>(ta, tb, tc, M, N, K, acc, status, num_sms, stream, k_splits, dense_c, c_elem)
        if (!a_mn && !b_mn) { if (out_f32) FS2_LAUNCH2(false, false, true); else FS2_LAUNCH2(false, false, false); }
        else if (!a_mn && b_mn) { if (out_f32) FS2_LAUNCH2(false, true, true); else FS2_LAUNCH2(false, true, false); }
        else if (a_mn && !b_mn) { if (out_f32) FS2_LAUNCH2(true, false, true); else FS2_LAUNCH2(true, false, false); }
        else { if (out_f32) FS2_LAUNCH2(true, true, true); else FS2_LAUNCH2(true, true, false); }
#undef FS2_LAUNCH2
        if (e != cudaSuccess) return cudaGetErrorString(e);
        return nullptr;
    }
#define FS2_LAUNCH(AM, BMN, F32) e = launch<AM, BMN, F32>(ta, tb, tc, M, N, K, acc, status, num_sms, stream, k_splits)
    if (!a_mn && !b_mn) { if (out_f32) FS2_LAUNCH(false, false, true); else FS2_LAUNCH(false, false, false); }
    else if (!a_mn && b_mn) { if (out_f32) FS2_LAUNCH(false, true, true); else FS2_LAUNCH(false, true, false); }
    else if (a_mn && !b_mn) { if (out_f32) FS2_LAUNCH(true, false, true); else FS2_LAUNCH(true, false, false); }
    else { if (out_f32) FS2_LAUNCH(true, true, true); else FS2_LAUNCH(true, true, false); }
#undef FS2_LAUNCH
    if (e != cudaSuccess) return cudaGetErrorString(e);
    return nullptr;
}

// C[M,N] (bf16) = A * B^T where one operand is the concatenation of `world` row shards that live on the peers.
// gather_b = false: A = concat_r a_shards[r] ([rows_per_rank, K] each), B = `other` [N, K] is local;
// gather_b = true : B = concat_r b_shards[r], A = `other` [M, K] is local.
// `gathered` is local scratch for the assembled operand, `flags` one zero-initialised word per block.
const char* gemm_allgather_bf16_tcgen05(const void* const* shards, int world, int rank, int rows_per_rank,
                                        const void* other, void* gathered, unsigned int* flags, unsigned int epoch,
                                        bool gather_b, void* c, int M, int N, int K, int ncopy, bool inplace,
                                        int* status, int num_sms, cudaStream_t stream, bool other_mn) {
    if (world < 1 || world > 8) return "gemm_allgather: between 1 and 8 ranks are supported";
    if (other_mn && gather_b) return "gemm_allgather: an MN-major local operand is only supported when A is gathered";
    const int blk = gather_b ? BN : BM;
    if (rows_per_rank % blk) return "gemm_allgather: the shard height must be a multiple of the tile height";
    if ((gather_b ? N : M) != rows_per_rank * world) return "gemm_allgather: shards do not add up to the operand";
    CUtensorMap ta, tb, tc;
    g_tmap_err[0] = 0;
    if (!make_tmap(&ta, gather_b ? other : gathered, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, M, K, BM, BK) ||
        !(other_mn ? make_tmap(&tb, other, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, K, N, BK, 64)
                   : make_tmap(&tb, gather_b ? gathered : other, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, N, K, BN, BK)) ||
        !make_tmap(&tc, c, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, M, N, 128, 64))
        return g_tmap_err;
    GatherArgs ga{};
    for (int r = 0; r < world; ++r) ga.src[r] = shards[r];
    ga.dst = gathered;
    ga.flags = flags;
    ga.epoch = epoch;
    ga.rows_per_rank = rows_per_rank;
    ga.rank = rank;
    ga.world = world;
    ga.row_bytes = static_cast<long long>(K) * 2;
    ga.inplace = inplace ? 1 : 0;
    const int num_tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
    if (ncopy < 1) ncopy = 1;
    if (ncopy > num_sms / 4) ncopy = num_sms / 4;
    ga.ncopy = ncopy;
    int grid = num_tiles + ncopy;
    if (grid > num_sms) grid = num_sms;            // every CTA must be resident: compute CTAs wait on copier CTAs
    cudaError_t e;
    if (!gather_b && other_mn) {
        auto kern = gemm_kernel<false, true, false, false, 1>;
        static bool configured = false;
        if (!configured) {
            e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
            if (e != cudaSuccess) return cudaGetErrorString(e);
            configured = true;
        }
        kern<<<grid, NUM_THREADS, SMEM_BYTES, stream>>>(ta, tb, tc, M, N, K, 0, status, PeerOut{}, ga);
    } else if (!gather_b) {
        auto kern = gemm_kernel<false, false, false, false, 1>;
        static bool configured = false;
        if (!configured) {
            e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
            if (e != cudaSuccess) return cudaGetErrorString(e);
            configured = true;
        }
        kern<<<grid, NUM_THREADS, SMEM_BYTES, stream>>>(ta, tb, tc, M, N, K, 0, status, PeerOut{}, ga);
    } else {
        auto kern = gemm_kernel<false, false, false, false, 2>;
        static bool configured = false;
        if (!configured) {
            e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
            if (e != cudaSuccess) return cudaGetErrorString(e);
            configured = true;
        }
        kern<<<grid, NUM_THREADS, SMEM_BYTES, stream>>>(ta, tb, tc, M, N, K, 0, status, PeerOut{}, ga);
    }
    e = cudaGetLastError();
    return e == cudaSuccess ? nullptr : cudaGetErrorString(e);
}

const char* gemm_reduce_scatter_bf16_tcgen05(const void* a, const void* b, float* const* peer_out, int world,
                                             int rows_per_rank, int M, int N, int K, int* status, int num_sms,
                                             cudaStream_t stream) {
    if (world < 1 || world > 8) return "gemm_reduce_scatter: between 1 and 8 ranks are supported";
    if (rows_per_rank <= 0 || rows_per_rank * world < M) return "gemm_reduce_scatter: rows_per_rank * world must cover M";
    if (N % 4) return "gemm_reduce_scatter: N must be a multiple of 4";
    CUtensorMap ta, tb;
    g_tmap_err[0] = 0;
    if (!make_tmap(&ta, a, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, M, K, BM, BK) ||
        !make_tmap(&tb, b, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, N, K, BN, BK))
        return g_tmap_err;
    PeerOut po{};
    for (int r = 0; r < world; ++r) po.out[r] = peer_out[r];
    po.rows_per_rank = rows_per_rank;
    auto kern = gemm_kernel<false, false, true, true>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
        if (e != cudaSuccess) return cudaGetErrorString(e);
        configured = true;
    }
    const int num_tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
    const int grid = num_tiles < num_sms ? num_tiles : num_sms;
    kern<<<grid, NUM_THREADS, SMEM_BYTES, stream>>>(ta, tb, ta, M, N, K, 0, status, po, GatherArgs{});
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? nullptr : cudaGetErrorString(e);
}

// Grouped GEMM for mixture-of-experts layers in ONE launch, with every size that depends on the routing read from
// device memory. `a` is the expert-sorted activation buffer [rows_cap, K] whose per-expert row ranges are padded to
// multiples of 128 (padding rows are zero); m-tile i covers rows [tile_row0[i], +128) and belongs to expert
// tile_expert[i]; `b` holds all experts' weights, [E, N, K] (K-major) or [E, K, N] (`b_mn`); c = [rows_cap, N] bf16.
const char* gemm_grouped_bf16_tcgen05(const void* a, const void* b, void* c, int rows_cap, int N, int K, bool b_mn,
                                      int experts, const int* tile_row0, const int* tile_expert,
                                      const int* num_m_tiles, int max_m_tiles, int* status, int num_sms,
                                      cudaStream_t stream) {
    if (rows_cap <= 0 || N <= 0 || K <= 0 || experts <= 0 || max_m_tiles <= 0) return "gemm_grouped: bad sizes";
    CUtensorMap ta, tb, tc;
    g_tmap_err[0] = 0;
    if (!make_tmap(&ta, a, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, rows_cap, K, BM, BK) ||
        !(b_mn ? make_tmap(&tb, b, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, static_cast<uint64_t>(experts) * K, N, BK, 64)
               : make_tmap(&tb, b, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, static_cast<uint64_t>(experts) * N, K, BN, BK)) ||
        !make_tmap(&tc, c, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, rows_cap, N, 128, 64))
        return g_tmap_err;
    GatherArgs ga{};
    ga.tile_row0 = tile_row0;
    ga.tile_expert = tile_expert;
    ga.num_m_tiles = num_m_tiles;
    ga.group_rows_b = b_mn ? K : N;
    ga.experts = experts;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_kernel<false, false, false, false, 3>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
        if (e == cudaSuccess)
            e = cudaFuncSetAttribute(gemm_kernel<false, true, false, false, 3>,
                                     cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
        if (e != cudaSuccess) return cudaGetErrorString(e);
        configured = true;
    }
    const long long max_tiles = static_cast<long long>(max_m_tiles) * ((N + BN - 1) / BN);
    const int grid = max_tiles < num_sms ? static_cast<int>(max_tiles) : num_sms;
    if (b_mn)
        gemm_kernel<false, true, false, false, 3><<<grid, NUM_THREADS, SMEM_BYTES, stream>>>(
            ta, tb, tc, rows_cap, N, K, 0, status, PeerOut{}, ga);
    else
        gemm_kernel<false, false, false, false, 3><<<grid, NUM_THREADS, SMEM_BYTES, stream>>>(
            ta, tb, tc, rows_cap, N, K, 0, status, PeerOut{}, ga);
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? nullptr : cudaGetErrorString(e);
}

// Weight gradients of all experts in one launch: dw[e] [M, N] = x[rows of e]^T @ dy[rows of e], the row range of
// expert e being [offsets[e], offsets[e + 1]) (device array, multiples of 128, never empty). x: [rows, M], dy: [rows, N].
const char* gemm_grouped_wgrad_bf16_tcgen05(const void* x, const void* dy, void* dw, bool out_f32, int rows, int M,
                                            int N, int experts, const int* offsets, int* status, int num_sms,
                                            cudaStream_t stream) {
    if (rows <= 0 || M <= 0 || N <= 0 || experts <= 0) return "gemm_grouped_wgrad: bad sizes";
    if (M % BM) return "gemm_grouped_wgrad: the per-expert output height must be a multiple of 128";
    CUtensorMap ta, tb, tc;
    g_tmap_err[0] = 0;
    const uint64_t crow = static_cast<uint64_t>(experts) * M;
    if (!make_tmap(&ta, x, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, rows, M, BK, 64) ||
        !make_tmap(&tb, dy, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, rows, N, BK, 64) ||
        !(out_f32 ? make_tmap(&tc, dw, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, crow, N, 128, 32)
                  : make_tmap(&tc, dw, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, crow, N, 128, 64)))
        return g_tmap_err;
    GatherArgs ga{};
    ga.group_offsets = offsets;
    ga.experts = experts;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_kernel<true, true, false, false, 4>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
        if (e == cudaSuccess)
            e = cudaFuncSetAttribute(gemm_kernel<true, true, true, false, 4>,
                                     cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
        if (e != cudaSuccess) return cudaGetErrorString(e);
        configured = true;
    }
    const long long tiles = static_cast<long long>(experts) * (M / BM) * ((N + BN - 1) / BN);
    const int grid = tiles < num_sms ? static_cast<int>(tiles) : num_sms;
    if (out_f32)
        gemm_kernel<true, true, true, false, 4><<<grid, NUM_THREADS, SMEM_BYTES, stream>>>(ta, tb, tc, M, N, rows, 0,
                                                                                           status, PeerOut{}, ga);
    else
        gemm_kernel<true, true, false, false, 4><<<grid, NUM_THREADS, SMEM_BYTES, stream>>>(ta, tb, tc, M, N, rows, 0,
                                                                                            status, PeerOut{}, ga);
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? nullptr : cudaGetErrorString(e);
}

const char* gemm_scatter_bf16_tcgen05(const void* a, const void* b, bool b_mn, void* const* peer_slices, int world,
                                      int rank, int rows_per_rank, int M, int N, int K, int* status, int num_sms,
                                      cudaStream_t stream) {
    if (world < 1 || world > 8 || rank < 0 || rank >= world) return "gemm_scatter: between 1 and 8 ranks are supported";
    if (rows_per_rank <= 0 || rows_per_rank * world < M) return "gemm_scatter: rows_per_rank * world must cover M";
    if (N % 8) return "gemm_scatter: N must be a multiple of 8";
    CUtensorMap ta, tb;
    g_tmap_err[0] = 0;
    if (!make_tmap(&ta, a, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, M, K, BM, BK) ||
        !(b_mn ? make_tmap(&tb, b, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, K, N, BK, 64)
               : make_tmap(&tb, b, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, N, K, BN, BK)))
        return g_tmap_err;
    PeerOut po{};
    for (int r = 0; r < world; ++r) po.out[r] = peer_slices[r];
    po.rows_per_rank = rows_per_rank;
    po.slice = rank;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_kernel<false, false, false, true>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
        if (e == cudaSuccess)
            e = cudaFuncSetAttribute(gemm_kernel<false, true, false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     SMEM_BYTES);
        if (e != cudaSuccess) return cudaGetErrorString(e);
        configured = true;
    }
    const int num_tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
    const int grid = num_tiles < num_sms ? num_tiles : num_sms;
    if (b_mn)
        gemm_kernel<false, true, false, true><<<grid, NUM_THREADS, SMEM_BYTES, stream>>>(ta, tb, ta, M, N, K, 0, status,
                                                                                          po, GatherArgs{});
    else
        gemm_kernel<false, false, false, true><<<grid, NUM_THREADS, SMEM_BYTES, stream>>>(ta, tb, ta, M, N, K, 0, status,
                                                                                           po, GatherArgs{});
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? nullptr : cudaGetErrorString(e);
}

}  // namespace fs2
