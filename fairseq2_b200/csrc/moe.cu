// Mixture-of-experts routing kernels: fused top-k gate, expert histogram, dispatch (gather + scale into
// expert-sorted order) and combine (gather back per token). One warp handles one token row.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cfloat>
#include <cstdint>

#include "comm_dev.cuh"
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

// Layout of the expert-sorted activation buffer for the grouped GEMM: every expert's row range is padded to a
// multiple of 128 rows (at least 128, so no expert is empty), offsets[e] is its first row, tile_row0/tile_expert list
// the 128-row tiles in order, num_tiles[0] their count. One block; E <= 256.
__global__ void moe_grouped_layout_kernel(const int* __restrict__ counts, int E, int* __restrict__ offsets,
                                          int* __restrict__ cursor, int* __restrict__ tile_row0,
                                          int* __restrict__ tile_expert, int* __restrict__ num_tiles) {
    if (threadIdx.x == 0) {
        int row = 0, tile = 0;
        for (int e = 0; e < E; ++e) {
            offsets[e] = row;
            cursor[e] = 0;
            int padded = (counts[e] + 127) / 128 * 128;
            if (padded == 0) padded = 128;
            for (int r = 0; r < padded; r += 128) {
                tile_row0[tile] = row + r;
                tile_expert[tile] = e;
                ++tile;
            }
            row += padded;
        }
        offsets[E] = row;
        num_tiles[0] = tile;
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

// ------------------------------------------------------------------ expert parallelism over peer memory
//
// W ranks, E experts, rank r owns experts [r * El, (r + 1) * El). The all-to-alls of the classic formulation are
// folded into the routing kernels: dispatch STORES each token row straight into the owning rank's inbox, combine
// LOADS each token's expert outputs straight from the owners' outboxes. Row positions are agreed on without a
// second exchange: every rank publishes its per-expert counts to everyone, after which each rank can compute the
// layout of every inbox (rows ordered by expert, then by source rank, then by arrival).

// One block. Publishes counts[E] into row `rank` of every peer's [W, E] table, waits (bounded) until all rows of
// the own table arrived, then derives
//   send_base[e]  : first inbox row (at the owner of e) of this rank's rows for expert e
//   group_sizes[i]: rows that local expert i receives from all ranks;  total[0] = their sum
//   cursor[e] = 0
__global__ void __launch_bounds__(256) moe_ep_layout_kernel(CommPeers peers, const int* __restrict__ counts,
                                                            long long table_byte_off, int E, int El,
                                                            int* __restrict__ send_base, int* __restrict__ cursor,
                                                            int* __restrict__ group_sizes, int* __restrict__ total,
                                                            int slot, uint32_t epoch, int* status) {
    const int W = peers.world;
    for (int e = threadIdx.x; e < E; e += blockDim.x) {
        const int c = counts[e];
        for (int r = 0; r < W; ++r) {
            int* tbl = reinterpret_cast<int*>(static_cast<char*>(peers.base[r]) + table_byte_off);
            tbl[peers.rank * E + e] = c;
        }
    }
    __threadfence_system();
    __syncthreads();
    if (!signal_and_wait(peers, slot, epoch, true, status, 40)) return;
    const volatile int* tbl = reinterpret_cast<const volatile int*>(static_cast<char*>(peers.base[peers.rank]) + table_byte_off);
    for (int e = threadIdx.x; e < E; e += blockDim.x) {
        const int owner_first = (e / El) * El;
        int base = 0;
        for (int e2 = owner_first; e2 < e; ++e2)
            for (int s = 0; s < W; ++s) base += tbl[s * E + e2];
        for (int s = 0; s < peers.rank; ++s) base += tbl[s * E + e];
        send_base[e] = base;
        cursor[e] = 0;
    }
    for (int i = threadIdx.x; i < El; i += blockDim.x) {
        int n = 0;
        for (int s = 0; s < W; ++s) n += tbl[s * E + peers.rank * El + i];
        group_sizes[i] = n;
    }
    if (threadIdx.x == 0) {
        int n = 0;
        for (int i = 0; i < El; ++i)
            for (int s = 0; s < W; ++s) n += tbl[s * E + peers.rank * El + i];
        total[0] = n;
    }
}

// Layout of the inboxes for the single-launch grouped GEMM: at every owner the rows of local expert i occupy a range
// that starts on a multiple of 128 rows and is padded to one (at least one tile, so that no expert is empty); inside
// a range rows are ordered by source rank, then by arrival. Every rank derives the layout of EVERY inbox from the
// exchanged count table, so senders know where their rows go without a second exchange.
//
// Overflow: an inbox holds `cap` rows (a multiple of 128, at least 128 per local expert). If the padded ranges of
// an owner do not fit, the ranges are cut (each later expert keeps one tile) and the rows that do not fit are
// DROPPED: their `dest` is -1, combine reads zero for them, and the push kernel counts them.
//
// One block. Outputs for all E experts: send_base[e] (first inbox row, at the owner of e, of this rank's rows),
// limit[e] (first row of e's range that holds no accepted row); for the El local experts: offsets[El + 1] (range
// starts), group_sizes[El] (accepted rows), the tile tables of the grouped GEMM, total[0] = rows in use incl. padding.
__global__ void __launch_bounds__(256) moe_ep_layout_padded_kernel(
    CommPeers peers, const int* __restrict__ counts, long long table_byte_off, int E, int El, int cap,
    int* __restrict__ send_base, int* __restrict__ limit, int* __restrict__ cursor, int* __restrict__ offsets,
    int* __restrict__ group_sizes, int* __restrict__ tile_row0, int* __restrict__ tile_expert,
    int* __restrict__ num_tiles, int* __restrict__ total, int slot, uint32_t epoch, int* status) {
    __shared__ int n_all[256];      // rows for expert e from all ranks
    __shared__ int n_before[256];   // rows for expert e from the ranks before this one
    const int W = peers.world;
    for (int e = threadIdx.x; e < E; e += blockDim.x) {
        const int c = counts[e];
        for (int r = 0; r < W; ++r) {
            int* tbl = reinterpret_cast<int*>(static_cast<char*>(peers.base[r]) + table_byte_off);
            tbl[peers.rank * E + e] = c;
        }
    }
    __threadfence_system();
    __syncthreads();
    if (!signal_and_wait(peers, slot, epoch, true, status, 41)) return;
    const volatile int* tbl =
        reinterpret_cast<const volatile int*>(static_cast<char*>(peers.base[peers.rank]) + table_byte_off);
    for (int e = threadIdx.x; e < E; e += blockDim.x) {
        int n = 0, b = 0;
        for (int s = 0; s < W; ++s) {
            const int c = tbl[s * E + e];
            if (s < peers.rank) b += c;
            n += c;
        }
        n_all[e] = n;
        n_before[e] = b;
        cursor[e] = 0;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int tile = 0;
        for (int o = 0; o < W; ++o) {
            int row = 0;
            for (int i = 0; i < El; ++i) {
                const int e = o * El + i;
                const int n = n_all[e];
                int want = (n + 127) / 128;                                   // tiles the expert would like
                if (want < 1) want = 1;
                int room = (cap - row) / 128 - (El - 1 - i);                 // tiles left after reserving one per later expert
                if (room < 1) room = 1;                                      // cap >= 128 * El is checked on the host
                const int tiles = want < room ? want : room;
                const int accepted = n < tiles * 128 ? n : tiles * 128;
                int first = row + n_before[e];
                send_base[e] = first;
                limit[e] = row + accepted;
                if (o == peers.rank) {
                    offsets[i] = row;
                    group_sizes[i] = accepted;
                    for (int t = 0; t < tiles; ++t) {
                        tile_row0[tile] = row + t * 128;
                        tile_expert[tile] = i;
                        ++tile;
                    }
                }
                row += tiles * 128;
            }
            if (o == peers.rank) {
                offsets[El] = row;
                total[0] = row;
                num_tiles[0] = tile;
            }
        }
    }
}

// Zeroes the padding rows [offsets[i] + group_sizes[i], offsets[i + 1]) of every local expert's range in the inbox:
// the grouped weight-gradient GEMM runs over whole ranges, so rows that no sender wrote must not hold old data.
__global__ void __launch_bounds__(256) moe_ep_zero_padding_kernel(__nv_bfloat16* __restrict__ inbox,
                                                                  const int* __restrict__ offsets,
                                                                  const int* __restrict__ group_sizes, int D) {
    const int i = blockIdx.x;
    const int beg = offsets[i] + group_sizes[i], end = offsets[i + 1];
    const long long nvec = static_cast<long long>(end - beg) * D / 8;
    __nv_bfloat16* base = inbox + static_cast<size_t>(beg) * D;
    const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
    for (long long v = blockIdx.y * static_cast<long long>(blockDim.x) + threadIdx.x; v < nvec;
         v += static_cast<long long>(gridDim.y) * blockDim.x)
        st16(base + v * 8, zero);
}

// One warp per (token, choice): stores x[t] (* gate) into row `dest[t, j] % cap` of the inbox of rank
// `dest[t, j] / cap`. With `assign` the destination is chosen here (send_base + arrival order) and recorded in
// `dest`; without it the rows go where an earlier call put them (used by the backward of combine).
__global__ void __launch_bounds__(256) moe_ep_push_kernel(CommPeers peers, const __nv_bfloat16* __restrict__ x,
                                                          const int* __restrict__ expert_ids,
                                                          const float* __restrict__ gates,
                                                          const int* __restrict__ send_base, int* __restrict__ cursor,
                                                          long long inbox_byte_off, int* __restrict__ dest, int rows,
                                                          int k, int D, int El, int cap, int assign,
                                                          const int* __restrict__ limit, int* __restrict__ dropped) {
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (warp >= rows) return;
    const int t = warp / k;
    int d = 0;
    if (lane == 0) {
        if (assign) {
            const int e = expert_ids[warp];
            const int row = send_base[e] + atomicAdd(&cursor[e], 1);
            // a row beyond the expert's range (or beyond the inbox) is dropped: nothing is stored, combine reads zero
            const bool fits = row < cap && row >= 0 && (limit == nullptr || row < limit[e]);
            d = fits ? (e / El) * cap + row : -1;
            if (!fits && dropped != nullptr) atomicAdd(dropped, 1);
            dest[warp] = d;
        } else {
            d = dest[warp];
        }
    }
    d = __shfl_sync(0xffffffffu, d, 0);
    if (d < 0) return;
    const float g = gates ? gates[warp] : 1.f;
    const __nv_bfloat16* src = x + static_cast<size_t>(t) * D;
    __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(static_cast<char*>(peers.base[d / cap]) + inbox_byte_off) +
                         static_cast<size_t>(d % cap) * D;
    for (int c = lane * 8; c < D; c += 256) {
        float f[8];
        load8(src, c, f);
        if (gates) {
#pragma unroll
            for (int i = 0; i < 8; ++i) f[i] *= g;
        }
        const bf16x8 p = pack8(f);
        st16(dst + c, *reinterpret_cast<const uint4*>(&p));
    }
}

// One warp per token: y[t] (+)= sum_j gate[t, j] * outbox(dest[t, j]) with 16-byte peer loads. If `x` is given,
// dgate[t, j] = <outbox row, x[t]> is produced as well (the gradient of a gate that scaled the pushed row).
__global__ void __launch_bounds__(256) moe_ep_pull_kernel(CommPeers peers, long long outbox_byte_off,
                                                          const int* __restrict__ dest,
                                                          const float* __restrict__ gates,
                                                          __nv_bfloat16* __restrict__ y,
                                                          const __nv_bfloat16* __restrict__ x,
                                                          float* __restrict__ dgate, int T_, int k, int D, int cap,
                                                          int accumulate) {
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (warp >= T_) return;
    __nv_bfloat16* dst = y + static_cast<size_t>(warp) * D;
    float dots[MAX_K];
#pragma unroll
    for (int j = 0; j < MAX_K; ++j) dots[j] = 0.f;
    for (int c = lane * 8; c < D; c += 256) {
        float acc[8];
        if (accumulate) load8(dst, c, acc);
        else {
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[i] = 0.f;
        }
        float xv[8];
        if (x) load8(x + static_cast<size_t>(warp) * D, c, xv);
#pragma unroll
        for (int j = 0; j < MAX_K; ++j) {
            if (j >= k) break;
            const int d = dest[warp * k + j];
            if (d < 0) continue;
            const __nv_bfloat16* src =
                reinterpret_cast<const __nv_bfloat16*>(static_cast<const char*>(peers.base[d / cap]) + outbox_byte_off) +
                static_cast<size_t>(d % cap) * D;
            const uint4 raw = ld_peer16(src + c);
            bf16x8 p;
            *reinterpret_cast<uint4*>(&p) = raw;
            float f[8];
            unpack8(p, f);
            const float g = gates ? gates[warp * k + j] : 1.f;
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[i] += g * f[i];
            if (x) {
#pragma unroll
                for (int i = 0; i < 8; ++i) dots[j] += f[i] * xv[i];
            }
        }
        store8(dst, c, acc);
    }
    if (x && dgate) {
#pragma unroll
        for (int j = 0; j < MAX_K; ++j) {
            if (j >= k) break;
            const float s = warp_sum(dots[j]);
            if (lane == 0) dgate[warp * k + j] = s;
        }
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

void moe_grouped_layout(const int* counts, int E, int* offsets, int* cursor, int* tile_row0, int* tile_expert,
                        int* num_tiles, cudaStream_t st) {
    moe_grouped_layout_kernel<<<1, 32, 0, st>>>(counts, E, offsets, cursor, tile_row0, tile_expert, num_tiles);
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

void moe_ep_layout(const CommPeers& peers, const int* counts, long long table_byte_off, int E, int* send_base,
                   int* cursor, int* group_sizes, int* total, int slot, uint32_t epoch, int* status, cudaStream_t st) {
    moe_ep_layout_kernel<<<1, 256, 0, st>>>(peers, counts, table_byte_off, E, E / peers.world, send_base, cursor,
                                            group_sizes, total, slot, epoch, status);
}

void moe_ep_push(const CommPeers& peers, const void* x, const int* expert_ids, const float* gates, const int* send_base,
                 int* cursor, long long inbox_byte_off, int* dest, int T, int k, int D, int E, int cap, bool assign,
                 const int* limit, int* dropped, cudaStream_t st) {
    const int rows = T * k;
    if (rows == 0) return;
    const int blocks = (rows * 32 + 255) / 256;
    moe_ep_push_kernel<<<blocks, 256, 0, st>>>(peers, static_cast<const __nv_bfloat16*>(x), expert_ids, gates, send_base,
                                               cursor, inbox_byte_off, dest, rows, k, D, E / peers.world, cap,
                                               assign ? 1 : 0, limit, dropped);
}

void moe_ep_layout_padded(const CommPeers& peers, const int* counts, long long table_byte_off, int E, int cap,
                          int* send_base, int* limit, int* cursor, int* offsets, int* group_sizes, int* tile_row0,
                          int* tile_expert, int* num_tiles, int* total, void* inbox, int D, int slot, uint32_t epoch,
                          int* status, cudaStream_t st) {
    const int El = E / peers.world;
    moe_ep_layout_padded_kernel<<<1, 256, 0, st>>>(peers, counts, table_byte_off, E, El, cap, send_base, limit, cursor,
                                                   offsets, group_sizes, tile_row0, tile_expert, num_tiles, total, slot,
                                                   epoch, status);
    moe_ep_zero_padding_kernel<<<dim3(El, 8), 256, 0, st>>>(static_cast<__nv_bfloat16*>(inbox), offsets, group_sizes, D);
}

void moe_ep_pull(const CommPeers& peers, long long outbox_byte_off, const int* dest, const float* gates, void* y,
                 const void* x, float* dgate, int T, int k, int D, int cap, bool accumulate, cudaStream_t st) {
    if (T == 0) return;
    const int blocks = (T * 32 + 255) / 256;
    moe_ep_pull_kernel<<<blocks, 256, 0, st>>>(peers, outbox_byte_off, dest, gates, static_cast<__nv_bfloat16*>(y),
                                               static_cast<const __nv_bfloat16*>(x), dgate, T, k, D, cap,
                                               accumulate ? 1 : 0);
}

}  // namespace fs2
