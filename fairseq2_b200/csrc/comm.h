// Host launchers of the symmetric-memory collective kernels (comm.cu).
#pragma once

#include <cuda_runtime.h>

#include <cstdint>

namespace fs2 {

constexpr int kCommMaxRanks = 8;       // one NVSwitch box
constexpr int kCommMaxSegments = 32;
constexpr int kCommFlagBytes = 64 * 1024;  // flag area at the start of every arena

struct CommPeers {
    void* base[kCommMaxRanks];  // arena base of every rank, mapped into this process
    int world;
    int rank;
    unsigned long long wait_limit_ns;
};

struct CommSegments {
    int count;
    long long off[kCommMaxSegments];    // element offset of the segment in a rank's shard buffer
    long long numel[kCommMaxSegments];  // elements per rank
};

void comm_barrier(const CommPeers& peers, int slot, uint32_t epoch, int* status, cudaStream_t st);
void comm_signal(const CommPeers& peers, int slot, uint32_t epoch, cudaStream_t st);
// In-place sum (times `scale`) of the `numel` elements (bf16 or fp32, a multiple of 16 bytes) at `byte_off` of every
// arena, through the NVSwitch multicast mapping `multicast_base` of the arena (multimem.ld_reduce / multimem.st).
// `counter` is a zero-initialised word in local memory; `slot_in` / `slot_out` are two epoch-flag slots.
void comm_allreduce_multimem(const CommPeers& peers, void* multicast_base, long long byte_off, long long numel, bool f32,
                             float scale, int slot_in, int slot_out, uint32_t epoch, unsigned int* counter, int blocks,
                             int* status, cudaStream_t st);
// out[i] = sum over w < world of slices[w * n + i] (bf16 in, fp32 sum, bf16 or fp32 out); n a multiple of 8.
void comm_reduce_slices(const void* slices, int world, long long n, void* out, bool out_f32, cudaStream_t st);
// out[off_s + i] = scale * (own_full[W * off_s + rank * numel_s + i] + sum_k staged[k][off_s + i]); local memory only.
// `norm_out` (may be null): the sum of squares of everything stored is added to it.
void comm_reduce_staged(const void* own_full, const void* const* staged, int count, const CommSegments& segs, int rank,
                        int world, void* out, bool out_f32, float scale, bool accumulate, int blocks, float* norm_out,
                        cudaStream_t st);
// Waits (bounded) until every peer's flag in `slot` has reached `epoch`, without signalling.
void comm_wait(const CommPeers& peers, int slot, uint32_t epoch, int* status, cudaStream_t st);
void comm_allgather_segments(const CommPeers& peers, const CommSegments& segs, long long shard_byte_off, void* full,
                             long long shard_numel, int slot, uint32_t epoch, int blocks, int* status,
                             cudaStream_t st);
// Reduce-scatter by peer loads: out[off_s + i] = scale * sum_r peer_r.full[W * off_s + rank * numel_s + i]. With
// `norm_out` (may be null) the sum of squares of the stored shard is added to that device scalar in the same pass.
void comm_reducescatter_segments(const CommPeers& peers, const CommSegments& segs, long long full_byte_off, void* out,
                                 bool out_f32, long long shard_numel, float scale, bool accumulate, int slot,
                                 uint32_t epoch, int blocks, float* norm_out, int* status, cudaStream_t st);
void comm_allreduce_f32(const CommPeers& peers, long long byte_off, float* out, long long numel, int op, int slot,
                        uint32_t epoch, int blocks, int* status, cudaStream_t st);
void comm_pull(const CommPeers& peers, int src_rank, long long byte_off, void* dst, long long bytes, int slot,
               uint32_t epoch, int blocks, int* status, cudaStream_t st);
void comm_alltoall(const CommPeers& peers, long long byte_off, void* dst, const long long* send_offs, int elem_bytes,
                   int slot, uint32_t epoch, int blocks, int* status, cudaStream_t st);

// Vocabulary-parallel embedding with a token-sharded result: the owner of a row pushes it into the output buffer of
// the rank that owns the token (forward), and pulls that token's gradient from it (backward).
void embed_push(const CommPeers& peers, const long long* ids, const void* table, long long lo, long long rows,
                long long out_byte_off, long long tokens, int D, long long rows_per_rank, cudaStream_t st);
void embed_pull_bwd(const CommPeers& peers, const long long* ids, long long dout_byte_off, float* dtable, long long lo,
                    long long rows, long long tokens, int D, long long rows_per_rank, cudaStream_t st);

// Reduce-scatter of bf16 gradients fused with the AdamW step of the local fp32 shard (`p`, `m`, `v`: shard-sized
// fp32; `low`: optional bf16 copy of the updated parameters). `step` is the 1-based step count; `scale_ptr` (may be
// null) is a device scalar multiplied into `scale`.
void comm_reducescatter_adamw(const CommPeers& peers, const CommSegments& segs, long long full_byte_off, float* p,
                              float* m, float* v, void* low, float scale, float lr, float beta1, float beta2, float eps,
                              float wd, int step, const float* scale_ptr, int slot, uint32_t epoch, int blocks,
                              int* status, cudaStream_t st);

// In-place all-reduce (sum * scale) of `numel` bf16/fp32 elements at `byte_off` of every arena; `counter` points at
// TWO zeroed device words (end of phase 1, end of phase 2); at most `blocks` <= number of SMs CTAs. The kernel ends
// only after every peer has finished reading this rank's bucket, so the bucket may be rewritten right after it.
void comm_allreduce_inplace(const CommPeers& peers, long long byte_off, long long numel, bool f32, float scale,
                            int slot_in, int slot_mid, uint32_t epoch, unsigned int* counter, int blocks, int* status,
                            cudaStream_t st);

}  // namespace fs2
