// Host entry point of the tcgen05 bf16 GEMM (see gemm_tcgen05.cu).
#pragma once

#include <cuda_runtime.h>

namespace fs2 {

// C[M,N] (+)= A * B^T. `a` is [M,K] (or [K,M] when a_mn), `b` is [N,K] (or
// [K,N] when b_mn), `c` is bf16 or fp32 [M,N]; all row-major, 16-byte aligned
// bases and row pitches. `status` points to host-mapped memory that receives a
// non-zero code if a bounded wait inside the kernel gave up.
// Returns nullptr on success, else a static error string.
const char* gemm_bf16_tcgen05(const void* a, const void* b, void* c, int M, int N, int K, bool a_mn, bool b_mn,
                              bool out_f32, bool accumulate, int* status, int num_sms, cudaStream_t stream);

// The same GEMM over strided views: `lda`/`ldb`/`ldc` are row pitches in elements (0 = dense) and may be smaller
// than the row length, so that rows overlap in memory (a strided 1-D convolution over a channels-last signal is
// A[r, :] = x[r * stride * C : r * stride * C + k * C]). `a_rows`/`b_rows`/`c_rows` (0 = all) give the number of
// rows that exist in memory: tiles beyond them read zeros and are not written. With `accumulate` the output tile is
// added (TMA reduce-add), which also sums rows of C that overlap. `k_splits` > 1 (needs `accumulate`) cuts the
// reduction dimension into that many ranges handled by different CTAs: for long-K, small-output products such as the
// weight gradient of a convolution.
const char* gemm_bf16_tcgen05_view(const void* a, long long lda, long long a_rows, const void* b, long long ldb,
                                   long long b_rows, void* c, long long ldc, long long c_rows, int M, int N, int K,
                                   bool a_mn, bool b_mn, bool out_f32, bool accumulate, int* status, int num_sms,
                                   cudaStream_t stream, int k_splits = 1);

// GEMM fused with the all-gather of one operand (see gemm_tcgen05.cu): `shards[r]` is rank r's [rows_per_rank, K]
// bf16 shard (peer mapping), `gathered` local scratch for the whole operand, `flags` one word per tile-height block
// (zero before the first call; `epoch` must grow by one per call), `ncopy` the number of CTAs that move data.
const char* gemm_allgather_bf16_tcgen05(const void* const* shards, int world, int rank, int rows_per_rank,
                                        const void* other, void* gathered, unsigned int* flags, unsigned int epoch,
                                        bool gather_b, void* c, int M, int N, int K, int ncopy, bool inplace,
                                        int* status, int num_sms, cudaStream_t stream, bool other_mn = false);

// Row-parallel GEMM fused with its reduce-scatter: C = A[M,K] * B[N,K]^T is never stored locally; every fp32
// tile is added into `peer_out[r]` ([rows_per_rank, N] fp32 in rank r's memory, zeroed beforehand), where r owns
// the tile's rows. The caller brackets the launch with cross-rank barriers (buffers zeroed / all adds landed).
const char* gemm_reduce_scatter_bf16_tcgen05(const void* a, const void* b, float* const* peer_out, int world,
                                             int rows_per_rank, int M, int N, int K, int* status, int num_sms,
                                             cudaStream_t stream);

// Same GEMM, bf16 scatter form: the tile is rounded to bf16 and stored into slice `rank` of `peer_slices[r]`
// ([world, rows_per_rank, N] bf16 in rank r's memory). After a cross-rank barrier the owner sums its `world` slices.
// `b_mn`: B is given as [K, N] row-major (e.g. a weight used untransposed in a backward pass).
const char* gemm_scatter_bf16_tcgen05(const void* a, const void* b, bool b_mn, void* const* peer_slices, int world,
                                      int rank, int rows_per_rank, int M, int N, int K, int* status, int num_sms,
                                      cudaStream_t stream);

// Grouped (mixture-of-experts) GEMMs with device-resident routing tables; see gemm_tcgen05.cu.
const char* gemm_grouped_bf16_tcgen05(const void* a, const void* b, void* c, int rows_cap, int N, int K, bool b_mn,
                                      int experts, const int* tile_row0, const int* tile_expert,
                                      const int* num_m_tiles, int max_m_tiles, int* status, int num_sms,
                                      cudaStream_t stream);
const char* gemm_grouped_wgrad_bf16_tcgen05(const void* x, const void* dy, void* dw, bool out_f32, int rows, int M,
                                            int N, int experts, const int* offsets, int* status, int num_sms,
                                            cudaStream_t stream);

}  // namespace fs2
