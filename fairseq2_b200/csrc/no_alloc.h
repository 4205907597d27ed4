// RMSNorm backward for callers that must not allocate device memory.
//
// This entry point has no counterpart in the reference; it exists for hosts
// that embed the kernels where the CUDA allocator is off limits: code running
// inside a stream capture, inside another framework's memory-planning phase,
// in a real-time loop that forbids allocator locks, or in a plugin whose host
// application owns every byte of device memory. The regular
// `rms_norm_bwd` binding asks torch's allocator for the per-block partial-sum
// buffer on every call; this variant keeps that buffer in a fixed, file-scope
// `__device__` array instead, so a call performs no cudaMalloc/cudaFree and
// uses no allocating library routine.
//
// Limits (a call outside them is rejected with a non-zero return value and a
// message retrievable through `fs2_no_alloc_last_error()`):
//   * D (row width) must be a multiple of 8 and at most FS2_NO_ALLOC_MAX_DIM (8192);
//   * rows >= 1; all pointers 16-byte aligned; dtype bf16 or fp32;
//   * the scratch array holds FS2_NO_ALLOC_MAX_BLOCKS x FS2_NO_ALLOC_MAX_DIM
//     floats (4 MiB). Every GPU that loads this library keeps those 4 MiB
//     resident until the process exits.
//
// Behaviour to know about:
//   * Call with the device that owns `stream` current on the calling thread
//     (cudaSetDevice): the scratch array is looked up for the current device
//     and the kernels are launched into `stream`. A stream of another device is
//     rejected with return value 6.
//   * The first call on each device resolves the device address of the scratch
//     array (cudaGetSymbolAddress). Make that first call outside of any stream
//     capture; later calls only launch kernels.
//   * All calls on a device share the one scratch array. Calls that may overlap
//     on the GPU (different streams without an ordering between them) race on
//     it; serialise them on one stream or with events. Nothing in the array
//     has to be cleared between calls: each call overwrites every partial it
//     later reads.
#pragma once

#include <cuda_runtime.h>

#define FS2_NO_ALLOC_MAX_BLOCKS 128
#define FS2_NO_ALLOC_MAX_DIM 8192

extern "C" {

// dx[rows, D] and dw[D] (fp32) are outputs supplied by the caller; dy, x are
// [rows, D], w is [D] (same dtype as x), rstd is fp32 [rows] as produced by the
// forward pass. Returns 0 on success.
int fs2_rms_norm_bwd_no_alloc(const void* dy, const void* x, const void* w, const float* rstd, void* dx, float* dw,
                              int rows, int D, int is_bf16, cudaStream_t stream);

// Static, human-readable description of the last failure on this thread.
const char* fs2_no_alloc_last_error();
}
