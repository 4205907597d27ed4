// Host launchers of the mixture-of-experts routing kernels (moe.cu).
#pragma once

#include <cuda_runtime.h>

#include <cstdint>

#include "comm.h"

namespace fs2 {

// Per token: top-k of `logits` [T, E] (bf16 or fp32), gate = sigmoid(logit) or softmax over the selected k;
// writes expert ids [T, k], gates [T, k] (fp32), adds 1 to counts[e] per selection and, if `prob_sum` is given,
// the full-softmax probability of every expert into prob_sum[e] (for load-balancing losses).
void moe_route(const void* logits, bool bf16, int T, int E, int k, bool softmax_gate, int* expert_ids, float* gates,
               int* counts, float* prob_sum, cudaStream_t st);

// offsets[e] = exclusive prefix sum of counts; cursor[e] = 0. One block.
void moe_offsets(const int* counts, int* offsets, int* cursor, int E, cudaStream_t st);

// Padded layout for the single-launch grouped GEMM: offsets[E + 1] (row ranges padded to multiples of 128, never
// empty), cursor[E] = 0, the list of 128-row tiles (tile_row0, tile_expert; at most rows / 128 + E entries) and their
// number. One block.
void moe_grouped_layout(const int* counts, int E, int* offsets, int* cursor, int* tile_row0, int* tile_expert,
                        int* num_tiles, cudaStream_t st);

// Dispatch: row (t, j) goes to slot p = offsets[e] + (arrival order within e); out[p, :] = x[t, :] * gate,
// src_row[p] = t, inv[t*k + j] = p. bf16 rows of D elements (D % 8 == 0).
void moe_dispatch(const void* x, const int* expert_ids, const float* gates, const int* offsets, int* cursor,
                  void* out, int* src_row, int* inv, int T, int k, int D, bool scale_by_gate, cudaStream_t st);

// Combine: y[t, :] (+)= sum over the slots p with src_row[p] == t of routed[p, :] (* gate[p] if given); implemented
// as a gather per token through inv[t, j] = p. bf16 in/out, fp32 accumulation.
void moe_combine(const void* routed, const int* inv, const float* slot_gates, void* y, int T, int k, int D,
                 bool accumulate, cudaStream_t st);

// Expert parallelism over peer memory (rank r owns experts [r * E / W, (r + 1) * E / W)).
//
// moe_ep_layout: one block; publishes counts[E] to every peer's [W, E] table at `table_byte_off`, waits (bounded,
// epoch flag `slot`) for all rows, then fills send_base[E], cursor[E] = 0, group_sizes[E / W], total[1].
void moe_ep_layout(const CommPeers& peers, const int* counts, long long table_byte_off, int E, int* send_base,
                   int* cursor, int* group_sizes, int* total, int slot, uint32_t epoch, int* status, cudaStream_t st);

// moe_ep_push: row (t, j) of x [T, D] (* gate if given) is stored into the inbox (at `inbox_byte_off`, `cap` rows of
// D bf16) of the rank owning its expert. `assign`: positions are taken from send_base/cursor and written to
// dest[t, j] = owner * cap + row (-1 if the inbox is full); otherwise dest is read.
// `limit` (may be null): limit[e] = first inbox row of expert e's range that takes no row (rows at or beyond it are
// dropped); `dropped` (may be null): device counter of dropped rows.
void moe_ep_push(const CommPeers& peers, const void* x, const int* expert_ids, const float* gates, const int* send_base,
                 int* cursor, long long inbox_byte_off, int* dest, int T, int k, int D, int E, int cap, bool assign,
                 const int* limit, int* dropped, cudaStream_t st);

// Count exchange + inbox layout in the 128-row padded form of the single-launch grouped GEMM (per local expert a
// range that starts and ends on a tile boundary), with the tile tables of this rank's inbox, and zeroing of the
// padding rows of `inbox`. `cap`: rows per inbox, a multiple of 128 and at least 128 per local expert.
void moe_ep_layout_padded(const CommPeers& peers, const int* counts, long long table_byte_off, int E, int cap,
                          int* send_base, int* limit, int* cursor, int* offsets, int* group_sizes, int* tile_row0,
                          int* tile_expert, int* num_tiles, int* total, void* inbox, int D, int slot, uint32_t epoch,
                          int* status, cudaStream_t st);

// moe_ep_pull: y[t] (+)= sum_j gate[t, j] * outbox row dest[t, j] (peer loads); optionally dgate[t, j] = <row, x[t]>.
void moe_ep_pull(const CommPeers& peers, long long outbox_byte_off, const int* dest, const float* gates, void* y,
                 const void* x, float* dgate, int T, int k, int D, int cap, bool accumulate, cudaStream_t st);

}  // namespace fs2
