// Collective kernels over symmetric (peer-mapped) memory for one NVSwitch box.
//
// Every rank maps the same arena of every peer into its address space; the
// kernels move data with plain 16-byte peer loads/stores over NVLink -- no TMA,
// no library call. They use no shared memory and few registers, so their CTAs
// co-reside with the persistent GEMM CTAs instead of displacing them.
//
// Synchronisation is by monotonically increasing flags ("epochs") that live in
// the first bytes of each rank's arena. A rank signals by storing the epoch
// into slot [slot * MAX_RANKS + its_rank] of every peer's flag area; a rank
// waits by polling its own flag area. Every wait is bounded: after the time
// limit the kernel stores a code into the host-mapped status word and returns
// without touching peer data, so the context stays usable.

#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cmath>
#include <cstdint>

#include "comm.h"
#include "comm_dev.cuh"
#include "common.cuh"

namespace fs2 {

namespace {

// ---------------------------------------------------------------------------
__global__ void barrier_kernel(CommPeers peers, int slot, uint32_t epoch, int* status) {
    signal_and_wait(peers, slot, epoch, true, status, 16);
}

__global__ void wait_kernel(CommPeers peers, int slot, uint32_t epoch, int* status) {
    signal_and_wait(peers, slot, epoch, false, status, 19);
}

__global__ void signal_kernel(CommPeers peers, int slot, uint32_t epoch) {
    if (threadIdx.x == 0 && blockIdx.x == 0) {
        __threadfence_system();
        for (int r = 0; r < peers.world; ++r) {
            uint32_t* f = reinterpret_cast<uint32_t*>(peers.base[r]) + slot * kCommMaxRanks + peers.rank;
            st_release_sys(f, epoch);
        }
    }
}

// Segment table: parameter `s` owns [off, off + numel) of every rank's shard
// buffer and the region [W * off, W * (off + numel)) of a full buffer, rank r's
// slice starting at W * off + r * numel.

// All-gather: full[W*off_s + r*numel_s + i] = peer_r.shard[off_s + i]. 2-byte elements.
// grid = (blocks, W); blockIdx.y selects the source rank (rotated so that ranks start on
// different peers). Each thread keeps AG_UNROLL independent 16-byte peer loads in flight:
// NVLink latency x bandwidth needs megabytes outstanding per GPU.
constexpr int AG_UNROLL = 8;

__global__ void __launch_bounds__(512) allgather_segments_kernel(
    CommPeers peers, CommSegments segs, long long shard_byte_off, __nv_bfloat16* __restrict__ full,
    long long shard_numel, int slot, uint32_t epoch, int* status) {
    if (epoch != 0 && !signal_and_wait(peers, slot, epoch, false, status, 17)) return;
    const int W = peers.world;
    const int r = (peers.rank + blockIdx.y) % W;
    const __nv_bfloat16* src =
        reinterpret_cast<const __nv_bfloat16*>(reinterpret_cast<const char*>(peers.base[r]) + shard_byte_off);
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    for (int s = 0; s < segs.count; ++s) {
        const long long off = segs.off[s];
        const long long nvec = segs.numel[s] / 8;
        const __nv_bfloat16* sp = src + off;
        __nv_bfloat16* dp = full + W * off + r * segs.numel[s];
        for (long long v0 = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; v0 < nvec;
             v0 += stride * AG_UNROLL) {
            uint4 buf[AG_UNROLL];
#pragma unroll
            for (int u = 0; u < AG_UNROLL; ++u) {
                const long long v = v0 + u * stride;
                if (v < nvec) buf[u] = ld_peer16(sp + v * 8);
            }
#pragma unroll
            for (int u = 0; u < AG_UNROLL; ++u) {
                const long long v = v0 + u * stride;
                if (v < nvec) st16(dp + v * 8, buf[u]);
            }
        }
    }
}

// Reduce-scatter: out[off_s + i] = scale * sum_r peer_r.full[W*off_s + rank*numel_s + i]; bf16 in,
// fp32 accumulate. All W peer loads of the unrolled vectors are issued before the first use.
// Vectors per thread and peer in flight: few ranks mean few peers per vector, so more vectors are unrolled to keep
// about the same number of bytes outstanding on NVLink.
template <int W>
struct RsUnroll {
    static constexpr int value = W <= 2 ? 8 : (W <= 4 ? 4 : 2);
};

// What happens to a reduced (and scaled) vector of 8 gradients at shard element index j.
template <typename OutT>
struct StoreSink {
    OutT* out;
    int accumulate;
    float sumsq;   // running sum of squares of what this thread stored (the thread's share of the gradient norm)
    __device__ __forceinline__ void operator()(size_t j, float* acc) {
        if (accumulate) {
            float prev[8];
            load8(out, j, prev);
#pragma unroll
            for (int e = 0; e < 8; ++e) acc[e] += prev[e];
        }
#pragma unroll
        for (int e = 0; e < 8; ++e) sumsq = fmaf(acc[e], acc[e], sumsq);
        store8(out, j, acc);
    }
};

// Adds the block's sum of the per-thread `sumsq` to `*norm_out` (one atomic per block).
__device__ __forceinline__ void publish_sumsq(float sumsq, float* norm_out) {
    __shared__ float scratch[32];
    const float total = block_sum(sumsq, scratch);
    if (threadIdx.x == 0) atomicAdd(norm_out, total);
}

// AdamW applied to the freshly reduced gradient while it is still in registers: the fp32 gradient shard is never
// written to (or re-read from) memory.
struct AdamWSink {
    float* p;
    float* m;
    float* v;
    __nv_bfloat16* low;   // bf16 copy of the updated parameters (may be null)
    float lr, beta1, beta2, eps, wd, step_size, bc2_sqrt;
    __device__ __forceinline__ void operator()(size_t j, float* g) {
        float pv[8], mv[8], vv[8];
        load8(p, j, pv);
        load8(m, j, mv);
        load8(v, j, vv);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            pv[e] *= (1.f - lr * wd);
            mv[e] = beta1 * mv[e] + (1.f - beta1) * g[e];
            vv[e] = beta2 * vv[e] + (1.f - beta2) * g[e] * g[e];
            pv[e] -= step_size * mv[e] / (sqrtf(vv[e]) / bc2_sqrt + eps);
        }
        store8(p, j, pv);
        store8(m, j, mv);
        store8(v, j, vv);
        if (low) store8(low, j, pv);
    }
};

template <typename Sink, int W>
__device__ __forceinline__ void reducescatter_body(const CommPeers& peers, const CommSegments& segs,
                                                   long long full_byte_off, Sink& sink, float scale) {
    const __nv_bfloat16* srcs[W];
#pragma unroll
    for (int k = 0; k < W; ++k) {
        const int r = (peers.rank + k) % W;
        srcs[k] = reinterpret_cast<const __nv_bfloat16*>(reinterpret_cast<const char*>(peers.base[r]) + full_byte_off);
    }
    constexpr int RS_UNROLL = RsUnroll<W>::value;
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    for (int s = 0; s < segs.count; ++s) {
        const long long off = segs.off[s];
        const long long nvec = segs.numel[s] / 8;
        const long long src_base = W * off + peers.rank * segs.numel[s];
        for (long long v0 = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; v0 < nvec;
             v0 += stride * RS_UNROLL) {
            uint4 raw[RS_UNROLL][W];
#pragma unroll
            for (int u = 0; u < RS_UNROLL; ++u) {
                const long long v = v0 + u * stride;
                if (v < nvec) {
#pragma unroll
                    for (int k = 0; k < W; ++k) raw[u][k] = ld_peer16(srcs[k] + src_base + v * 8);
                }
            }
#pragma unroll
            for (int u = 0; u < RS_UNROLL; ++u) {
                const long long v = v0 + u * stride;
                if (v >= nvec) continue;
                float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
                for (int k = 0; k < W; ++k) {
                    bf16x8 p;
                    *reinterpret_cast<uint4*>(&p) = raw[u][k];
                    float f[8];
                    unpack8(p, f);
#pragma unroll
                    for (int e = 0; e < 8; ++e) acc[e] += f[e];
                }
                const size_t j = static_cast<size_t>(off + v * 8);
#pragma unroll
                for (int e = 0; e < 8; ++e) acc[e] *= scale;
                sink(j, acc);
            }
        }
    }
}

template <typename Sink>
__device__ __forceinline__ void reducescatter_dispatch(const CommPeers& peers, const CommSegments& segs,
                                                       long long full_byte_off, Sink& sink, float scale) {
    switch (peers.world) {
        case 1: reducescatter_body<Sink, 1>(peers, segs, full_byte_off, sink, scale); break;
        case 2: reducescatter_body<Sink, 2>(peers, segs, full_byte_off, sink, scale); break;
        case 3: reducescatter_body<Sink, 3>(peers, segs, full_byte_off, sink, scale); break;
        case 4: reducescatter_body<Sink, 4>(peers, segs, full_byte_off, sink, scale); break;
        case 5: reducescatter_body<Sink, 5>(peers, segs, full_byte_off, sink, scale); break;
        case 6: reducescatter_body<Sink, 6>(peers, segs, full_byte_off, sink, scale); break;
        case 7: reducescatter_body<Sink, 7>(peers, segs, full_byte_off, sink, scale); break;
        default: reducescatter_body<Sink, 8>(peers, segs, full_byte_off, sink, scale); break;
    }
}

// With `norm_out` the kernel is the whole gradient path of an FSDP unit between backward and optimizer: peer loads of
// the W bf16 slices, fp32 sum, averaging factor, ONE store of the fp32 shard, and the unit's contribution to the
// squared global gradient norm (clipping then only needs the tiny all-reduce of that scalar; AdamW takes the clip
// factor as a device scalar). Without it, a plain reduce-scatter.
template <typename OutT>
__global__ void __launch_bounds__(512) reducescatter_segments_kernel(
    CommPeers peers, CommSegments segs, long long full_byte_off, OutT* __restrict__ out, long long shard_numel,
    float scale, int accumulate, int slot, uint32_t epoch, float* norm_out, int* status) {
    if (!signal_and_wait(peers, slot, epoch, true, status, 18)) return;
    StoreSink<OutT> sink{out, accumulate, 0.f};
    reducescatter_dispatch(peers, segs, full_byte_off, sink, scale);
    if (norm_out != nullptr) publish_sumsq(sink.sumsq, norm_out);
}

// Reduce-scatter fused with the optimizer step of the local shard (no gradient clipping between the two).
// `scale_ptr` (may be null): a device scalar multiplied into `scale` -- the loss normalisation of the step, known only
// on the device (the all-reduced number of targets) when the kernel is queued.
__global__ void __launch_bounds__(512) reducescatter_adamw_kernel(CommPeers peers, CommSegments segs,
                                                                  long long full_byte_off, AdamWSink sink, float scale,
                                                                  const float* __restrict__ scale_ptr, int slot,
                                                                  uint32_t epoch, int* status) {
    if (!signal_and_wait(peers, slot, epoch, true, status, 24)) return;
    AdamWSink local = sink;
    if (scale_ptr != nullptr) scale *= *scale_ptr;
    reducescatter_dispatch(peers, segs, full_byte_off, local, scale);
}

// Second half of the copy-engine reduce-scatter: the peers' slices of this rank's shard have been copied into local
// staging buffers (shard layout), the own slice still sits in the local full-gradient buffer. Sums own + staged in
// ring order (the order of the load/store kernel above, so both paths give the same bits) from local memory only.
struct StagedSlices {
    const __nv_bfloat16* p[kCommMaxRanks];
    int count;
};

template <typename OutT>
__global__ void __launch_bounds__(512) reduce_staged_kernel(const __nv_bfloat16* __restrict__ own_full,
                                                            StagedSlices staged, CommSegments segs, int rank, int world,
                                                            OutT* __restrict__ out, float scale, int accumulate,
                                                            float* norm_out) {
    StoreSink<OutT> sink{out, accumulate, 0.f};
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    for (int s = 0; s < segs.count; ++s) {
        const long long off = segs.off[s];
        const long long nvec = segs.numel[s] / 8;
        const __nv_bfloat16* own = own_full + world * off + rank * segs.numel[s];
        for (long long v = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; v < nvec; v += stride) {
            float acc[8];
            load8(own, static_cast<size_t>(v * 8), acc);
            for (int k = 0; k < staged.count; ++k) {
                float f[8];
                load8(staged.p[k] + off, static_cast<size_t>(v * 8), f);
#pragma unroll
                for (int e = 0; e < 8; ++e) acc[e] += f[e];
            }
#pragma unroll
            for (int e = 0; e < 8; ++e) acc[e] *= scale;
            sink(static_cast<size_t>(off + v * 8), acc);
        }
    }
    if (norm_out != nullptr) publish_sumsq(sink.sumsq, norm_out);
}

template <typename OutT>
__global__ void __launch_bounds__(256) reduce_slices_kernel(const __nv_bfloat16* __restrict__ slices, int world,
                                                            long long n, OutT* __restrict__ out) {
    const long long nvec = n / 8;
    for (long long v = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; v < nvec;
         v += static_cast<long long>(gridDim.x) * blockDim.x) {
        float acc[8];
        load8(slices, static_cast<size_t>(v * 8), acc);
        for (int w = 1; w < world; ++w) {
            float f[8];
            load8(slices + w * n, static_cast<size_t>(v * 8), f);
#pragma unroll
            for (int e = 0; e < 8; ++e) acc[e] += f[e];
        }
        store8(out, static_cast<size_t>(v * 8), acc);
    }
}

// One-shot all-reduce of `numel` fp32 values staged at `byte_off` of every arena.
// op: 0 sum, 1 mean, 2 product, 3 min, 4 max.
__global__ void allreduce_f32_kernel(CommPeers peers, long long byte_off, float* __restrict__ out, long long numel,
                                     int op, int slot, uint32_t epoch, int* status) {
    if (!signal_and_wait(peers, slot, epoch, true, status, 19)) return;
    const int W = peers.world;
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < numel;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        float acc = 0.f;
        for (int r = 0; r < W; ++r) {
            const float* src = reinterpret_cast<const float*>(reinterpret_cast<const char*>(peers.base[r]) + byte_off);
            float v;
            asm volatile("ld.relaxed.sys.global.L1::no_allocate.f32 %0, [%1];" : "=f"(v) : "l"(src + i) : "memory");
            if (r == 0) acc = v;
            else if (op <= 1) acc += v;
            else if (op == 2) acc *= v;
            else if (op == 3) acc = fminf(acc, v);
            else acc = fmaxf(acc, v);
        }
        if (op == 1) acc /= W;
        out[i] = acc;
    }
}

// In-place two-shot all-reduce (+ scale) of a bucket that lives at `byte_off` of every arena.
//   phase 1: this rank sums slice `rank` of every peer's bucket (fp32 accumulation), scales it and writes it
//            back into its own bucket;
//   phase 2: once every peer has published its reduced slice, the other slices are pulled over NVLink.
// Every element crosses NVLink twice per rank ((W-1)/W in, (W-1)/W out), the minimum for an all-reduce, and the
// averaging factor of data parallelism is applied on the way instead of by a separate pass over the gradients.
// `counter` (device memory, zero between launches) detects the last CTA of phase 1.
template <typename T, int W>
__device__ __forceinline__ void allreduce_phase1(const CommPeers& peers, long long byte_off, long long chunk,
                                                 long long numel, float scale) {
    constexpr int PER = 16 / sizeof(T);
    const long long beg = peers.rank * chunk;
    const long long end = beg + chunk < numel ? beg + chunk : numel;
    const long long nvec = end > beg ? (end - beg) / PER : 0;
    char* mine = reinterpret_cast<char*>(peers.base[peers.rank]) + byte_off + beg * sizeof(T);
    for (long long v = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; v < nvec;
         v += static_cast<long long>(gridDim.x) * blockDim.x) {
        uint4 in[W];
#pragma unroll
        for (int r = 0; r < W; ++r) {
            const int src = (peers.rank + r) % W;     // start on different peers
            in[r] = ld_peer16(reinterpret_cast<const char*>(peers.base[src]) + byte_off + beg * sizeof(T) + v * 16);
        }
        float acc[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] = 0.f;
#pragma unroll
        for (int r = 0; r < W; ++r) {
            if constexpr (sizeof(T) == 2) {
                float f[8];
                unpack8(*reinterpret_cast<const bf16x8*>(&in[r]), f);
#pragma unroll
                for (int i = 0; i < 8; ++i) acc[i] += f[i];
            } else {
                const float* f = reinterpret_cast<const float*>(&in[r]);
#pragma unroll
                for (int i = 0; i < 4; ++i) acc[i] += f[i];
            }
        }
        uint4 out;
        if constexpr (sizeof(T) == 2) {
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[i] *= scale;
            bf16x8 pk = pack8(acc);
            out = *reinterpret_cast<uint4*>(&pk);
        } else {
            float* f = reinterpret_cast<float*>(&out);
#pragma unroll
            for (int i = 0; i < 4; ++i) f[i] = acc[i] * scale;
        }
        st16(mine + v * 16, out);
    }
}

template <typename T>
__global__ void __launch_bounds__(512) allreduce_inplace_kernel(CommPeers peers, long long byte_off, long long numel,
                                                                float scale, int slot_in, int slot_mid,
                                                                uint32_t epoch, unsigned int* counter, int* status) {
    // slot_in carries two epochs per call: 2 * epoch - 1 = "my bucket holds this call's input",
    // 2 * epoch = "I have finished reading every peer's bucket" (the trailing handshake below)
    if (!signal_and_wait(peers, slot_in, 2 * epoch - 1, true, status, 22)) return;
    constexpr int PER = 16 / sizeof(T);
    const int W = peers.world;
    // slices are multiples of one 16-byte vector; `numel` itself is a multiple of PER (host-checked)
    long long chunk = (numel + W - 1) / W;
    chunk = (chunk + PER - 1) / PER * PER;
    switch (W) {
        case 1: allreduce_phase1<T, 1>(peers, byte_off, chunk, numel, scale); break;
        case 2: allreduce_phase1<T, 2>(peers, byte_off, chunk, numel, scale); break;
        case 3: allreduce_phase1<T, 3>(peers, byte_off, chunk, numel, scale); break;
        case 4: allreduce_phase1<T, 4>(peers, byte_off, chunk, numel, scale); break;
        case 5: allreduce_phase1<T, 5>(peers, byte_off, chunk, numel, scale); break;
        case 6: allreduce_phase1<T, 6>(peers, byte_off, chunk, numel, scale); break;
        case 7: allreduce_phase1<T, 7>(peers, byte_off, chunk, numel, scale); break;
        default: allreduce_phase1<T, 8>(peers, byte_off, chunk, numel, scale); break;
    }
    // the last CTA to finish phase 1 publishes "my slice is reduced" to every peer
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence_system();
        const unsigned int prev = atomicAdd(counter, 1u);
        if (prev == gridDim.x - 1) {
            *counter = 0;
            __threadfence_system();
            for (int r = 0; r < W; ++r) {
                uint32_t* f = reinterpret_cast<uint32_t*>(peers.base[r]) + slot_mid * kCommMaxRanks + peers.rank;
                st_release_sys(f, epoch);
            }
        }
    }
    if (!signal_and_wait(peers, slot_mid, epoch, false, status, 23)) return;
    // phase 2: pull the reduced slices of the peers
    char* mine = reinterpret_cast<char*>(peers.base[peers.rank]) + byte_off;
    for (int r = 1; r < W; ++r) {
        const int src = (peers.rank + r) % W;
        const long long beg = src * chunk;
        const long long end = beg + chunk < numel ? beg + chunk : numel;
        const long long nvec = end > beg ? (end - beg) / PER : 0;
        const char* from = reinterpret_cast<const char*>(peers.base[src]) + byte_off + beg * sizeof(T);
        char* to = mine + beg * sizeof(T);
        for (long long v = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; v < nvec;
             v += static_cast<long long>(gridDim.x) * blockDim.x)
            st16(to + v * 16, ld_peer16(from + v * 16));
    }
    // Trailing handshake: the bucket may be overwritten (by the next backward pass) as soon as this kernel has
    // finished, so the kernel ends only when every peer has pulled what it needs from this rank's bucket. The last
    // CTA to finish phase 2 announces "done reading" and waits (bounded) for the same announcement of every peer.
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned int prev = atomicAdd(counter + 1, 1u);
        if (prev == gridDim.x - 1) {
            counter[1] = 0;
            __threadfence_system();
            signal_all(peers, slot_in, 2 * epoch);
            wait_all_one_thread(peers, slot_in, 2 * epoch, status, 28);
        }
    }
}

// In-place all-reduce through the NVSwitch multicast mapping of the arena (NVLS): every rank owns 1/W of the buffer,
// reads it with multimem.ld_reduce -- the switch fetches the W copies and returns their sum, accumulated in fp32 --
// scales it and writes it back with multimem.st, which the switch delivers to all W copies. Each GPU therefore moves
// 1/W of the buffer in and 1/W out instead of (W-1)/W each way, and issues 1/W of the loads.
template <typename T>
__global__ void __launch_bounds__(512) allreduce_multimem_kernel(CommPeers peers, char* mc_base, long long byte_off,
                                                                 long long numel, float scale, int slot_in, int slot_out,
                                                                 uint32_t epoch, unsigned int* counter, int* status) {
    if (!signal_and_wait(peers, slot_in, epoch, true, status, 26)) return;
    constexpr int PER = 16 / sizeof(T);
    const int W = peers.world;
    const long long nvec = numel / PER;
    const long long per_rank = (nvec + W - 1) / W;
    const long long beg = peers.rank * per_rank;
    const long long end = beg + per_rank < nvec ? beg + per_rank : nvec;
    char* mc = mc_base + byte_off;
    for (long long v = beg + blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; v < end;
         v += static_cast<long long>(gridDim.x) * blockDim.x) {
        char* addr = mc + v * 16;
        if constexpr (sizeof(T) == 4) {
            float a, b, c, d;
            asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
                         : "=f"(a), "=f"(b), "=f"(c), "=f"(d) : "l"(addr) : "memory");
            a *= scale; b *= scale; c *= scale; d *= scale;
            asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};"
                         ::"l"(addr), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
        } else {
            uint4 r;
            asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
                         : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(addr) : "memory");
            bf16x8 p;
            *reinterpret_cast<uint4*>(&p) = r;
            float f[8];
            unpack8(p, f);
#pragma unroll
            for (int i = 0; i < 8; ++i) f[i] *= scale;
            p = pack8(f);
            r = *reinterpret_cast<uint4*>(&p);
            asm volatile("multimem.st.relaxed.sys.global.v4.bf16x2 [%0], {%1, %2, %3, %4};"
                         ::"l"(addr), "r"(r.x), "r"(r.y), "r"(r.z), "r"(r.w) : "memory");
        }
    }
    // the last CTA to finish tells every peer that this rank's slice has been written everywhere
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence_system();
        const unsigned int prev = atomicAdd(counter, 1u);
        if (prev == gridDim.x - 1) {
            *counter = 0;
            __threadfence_system();
            for (int r = 0; r < W; ++r) {
                uint32_t* f = reinterpret_cast<uint32_t*>(peers.base[r]) + slot_out * kCommMaxRanks + peers.rank;
                st_release_sys(f, epoch);
            }
        }
    }
    signal_and_wait(peers, slot_out, epoch, false, status, 27);
}

// Pull copy: dst[i] = peer_src.arena[byte_off + i] for `bytes` bytes (multiple of 16).
__global__ void pull_kernel(CommPeers peers, int src_rank, long long byte_off, char* __restrict__ dst,
                            long long bytes, int slot, uint32_t epoch, int* status) {
    if (!signal_and_wait(peers, slot, epoch, true, status, 20)) return;
    const char* src = reinterpret_cast<const char*>(peers.base[src_rank]) + byte_off;
    const long long nvec = bytes / 16;
    for (long long v = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; v < nvec;
         v += static_cast<long long>(gridDim.x) * blockDim.x)
        st16(dst + v * 16, ld_peer16(src + v * 16));
}

// All-to-all with equal or variable splits, pull based. Every rank staged its
// send buffer at `byte_off`; `send_offs` ([W, W+1] int64 element offsets, row r =
// rank r's prefix sums over destinations) is replicated on every rank.
__global__ void alltoall_kernel(CommPeers peers, long long byte_off, char* __restrict__ dst,
                                const long long* __restrict__ send_offs, int elem_bytes, int slot, uint32_t epoch,
                                int* status) {
    if (!signal_and_wait(peers, slot, epoch, true, status, 21)) return;
    const int W = peers.world;
    const int src_rank = blockIdx.y;
    long long dst_elem = 0;
    for (int r = 0; r < src_rank; ++r)
        dst_elem += send_offs[r * (W + 1) + peers.rank + 1] - send_offs[r * (W + 1) + peers.rank];
    const long long beg = send_offs[src_rank * (W + 1) + peers.rank];
    const long long end = send_offs[src_rank * (W + 1) + peers.rank + 1];
    const char* src = reinterpret_cast<const char*>(peers.base[src_rank]) + byte_off + beg * elem_bytes;
    char* out = dst + dst_elem * elem_bytes;
    const long long bytes = (end - beg) * elem_bytes;
    const bool vec_ok = ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(out)) & 15) == 0;
    if (vec_ok) {
        const long long nvec = bytes / 16;
        for (long long v = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; v < nvec;
             v += static_cast<long long>(gridDim.x) * blockDim.x)
            st16(out + v * 16, ld_peer16(src + v * 16));
        for (long long b = nvec * 16 + blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; b < bytes;
             b += static_cast<long long>(gridDim.x) * blockDim.x)
            out[b] = src[b];
    } else {
        for (long long b = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; b < bytes;
             b += static_cast<long long>(gridDim.x) * blockDim.x)
            out[b] = src[b];
    }
}


// ------------------------------------------------ vocabulary-parallel embedding, token-sharded result
// This rank holds rows [lo, lo + rows) of the table. Token t's embedding belongs to rank t / rows_per_rank of the
// tensor-parallel group (sequence-parallel residual stream), so the rank that owns the row writes it straight into
// that rank's output buffer over NVLink: every output row has exactly one writer and no reduction is needed. One
// warp per token. The caller separates the launch from the consumer with a barrier.
__global__ void __launch_bounds__(256) embed_push_kernel(CommPeers peers, const long long* __restrict__ ids,
                                                         const __nv_bfloat16* __restrict__ table, long long lo,
                                                         long long rows, long long out_byte_off, long long tokens,
                                                         int D, long long rows_per_rank) {
    const long long t = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (t >= tokens) return;
    const long long r = ids[t] - lo;
    if (r < 0 || r >= rows) return;
    const int owner = static_cast<int>(t / rows_per_rank);
    char* dst = static_cast<char*>(peers.base[owner]) + out_byte_off + (t - owner * rows_per_rank) * D * 2;
    const char* src = reinterpret_cast<const char*>(table + r * D);
    for (int c = lane * 16; c < D * 2; c += 512) st16(dst + c, *reinterpret_cast<const uint4*>(src + c));
}

// Backward of the above: every rank staged its token shard of d(out) at `dout_byte_off` of its arena; the rank
// that owns the row of token t reads that token's gradient from rank t / rows_per_rank and adds it to its fp32
// table gradient (atomics: tokens repeat).
__global__ void __launch_bounds__(256) embed_pull_bwd_kernel(CommPeers peers, const long long* __restrict__ ids,
                                                             long long dout_byte_off, float* __restrict__ dtable,
                                                             long long lo, long long rows, long long tokens, int D,
                                                             long long rows_per_rank) {
    const long long t = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (t >= tokens) return;
    const long long r = ids[t] - lo;
    if (r < 0 || r >= rows) return;
    const int owner = static_cast<int>(t / rows_per_rank);
    const char* src = static_cast<const char*>(peers.base[owner]) + dout_byte_off + (t - owner * rows_per_rank) * D * 2;
    float* dst = dtable + r * D;
    for (int c = lane * 8; c < D; c += 256) {
        const uint4 v = ld_peer16(src + c * 2);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float2 f = __bfloat1622float2(h[e]);
            atomicAdd(dst + c + 2 * e, f.x);
            atomicAdd(dst + c + 2 * e + 1, f.y);
        }
    }
}

}  // namespace

void comm_barrier(const CommPeers& peers, int slot, uint32_t epoch, int* status, cudaStream_t st) {
    barrier_kernel<<<1, 32, 0, st>>>(peers, slot, epoch, status);
}

void comm_wait(const CommPeers& peers, int slot, uint32_t epoch, int* status, cudaStream_t st) {
    wait_kernel<<<1, 32, 0, st>>>(peers, slot, epoch, status);
}

void comm_signal(const CommPeers& peers, int slot, uint32_t epoch, cudaStream_t st) {
    signal_kernel<<<1, 32, 0, st>>>(peers, slot, epoch);
}

void comm_allgather_segments(const CommPeers& peers, const CommSegments& segs, long long shard_byte_off, void* full,
                             long long shard_numel, int slot, uint32_t epoch, int blocks, int* status,
                             cudaStream_t st) {
    dim3 grid(blocks, peers.world);
    allgather_segments_kernel<<<grid, 512, 0, st>>>(peers, segs, shard_byte_off, static_cast<__nv_bfloat16*>(full),
                                                    shard_numel, slot, epoch, status);
}

void comm_reducescatter_segments(const CommPeers& peers, const CommSegments& segs, long long full_byte_off, void* out,
                                 bool out_f32, long long shard_numel, float scale, bool accumulate, int slot,
                                 uint32_t epoch, int blocks, float* norm_out, int* status, cudaStream_t st) {
    if (out_f32)
        reducescatter_segments_kernel<float><<<blocks, 512, 0, st>>>(peers, segs, full_byte_off,
                                                                     static_cast<float*>(out), shard_numel, scale,
                                                                     accumulate ? 1 : 0, slot, epoch, norm_out, status);
    else
        reducescatter_segments_kernel<__nv_bfloat16><<<blocks, 512, 0, st>>>(
            peers, segs, full_byte_off, static_cast<__nv_bfloat16*>(out), shard_numel, scale, accumulate ? 1 : 0,
            slot, epoch, norm_out, status);
}

void comm_allreduce_f32(const CommPeers& peers, long long byte_off, float* out, long long numel, int op, int slot,
                        uint32_t epoch, int blocks, int* status, cudaStream_t st) {
    allreduce_f32_kernel<<<blocks, 256, 0, st>>>(peers, byte_off, out, numel, op, slot, epoch, status);
}

void embed_push(const CommPeers& peers, const long long* ids, const void* table, long long lo, long long rows,
                long long out_byte_off, long long tokens, int D, long long rows_per_rank, cudaStream_t st) {
    if (tokens == 0) return;
    const unsigned blocks = static_cast<unsigned>((tokens * 32 + 255) / 256);
    embed_push_kernel<<<blocks, 256, 0, st>>>(peers, ids, static_cast<const __nv_bfloat16*>(table), lo, rows,
                                              out_byte_off, tokens, D, rows_per_rank);
}

void embed_pull_bwd(const CommPeers& peers, const long long* ids, long long dout_byte_off, float* dtable, long long lo,
                    long long rows, long long tokens, int D, long long rows_per_rank, cudaStream_t st) {
    if (tokens == 0) return;
    const unsigned blocks = static_cast<unsigned>((tokens * 32 + 255) / 256);
    embed_pull_bwd_kernel<<<blocks, 256, 0, st>>>(peers, ids, dout_byte_off, dtable, lo, rows, tokens, D,
                                                  rows_per_rank);
}

void comm_pull(const CommPeers& peers, int src_rank, long long byte_off, void* dst, long long bytes, int slot,
               uint32_t epoch, int blocks, int* status, cudaStream_t st) {
    pull_kernel<<<blocks, 512, 0, st>>>(peers, src_rank, byte_off, static_cast<char*>(dst), bytes, slot, epoch,
                                        status);
}

void comm_alltoall(const CommPeers& peers, long long byte_off, void* dst, const long long* send_offs, int elem_bytes,
                   int slot, uint32_t epoch, int blocks, int* status, cudaStream_t st) {
    dim3 grid(blocks, peers.world);
    alltoall_kernel<<<grid, 512, 0, st>>>(peers, byte_off, static_cast<char*>(dst), send_offs, elem_bytes, slot,
                                          epoch, status);
}

void comm_reducescatter_adamw(const CommPeers& peers, const CommSegments& segs, long long full_byte_off, float* p,
                              float* m, float* v, void* low, float scale, float lr, float beta1, float beta2, float eps,
                              float wd, int step, const float* scale_ptr, int slot, uint32_t epoch, int blocks,
                              int* status, cudaStream_t st) {
    AdamWSink sink{};
    sink.p = p;
    sink.m = m;
    sink.v = v;
    sink.low = static_cast<__nv_bfloat16*>(low);
    sink.lr = lr;
    sink.beta1 = beta1;
    sink.beta2 = beta2;
    sink.eps = eps;
    sink.wd = wd;
    sink.step_size = lr / (1.f - powf(beta1, static_cast<float>(step)));
    sink.bc2_sqrt = sqrtf(1.f - powf(beta2, static_cast<float>(step)));
    reducescatter_adamw_kernel<<<blocks, 512, 0, st>>>(peers, segs, full_byte_off, sink, scale, scale_ptr, slot, epoch,
                                                       status);
}

void comm_reduce_slices(const void* slices, int world, long long n, void* out, bool out_f32, cudaStream_t st) {
    const long long nvec = n / 8;
    const int blocks = static_cast<int>(nvec / 256 < 1 ? 1 : (nvec / 256 > 1184 ? 1184 : nvec / 256));
    if (out_f32)
        reduce_slices_kernel<float><<<blocks, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(slices), world, n,
                                                            static_cast<float*>(out));
    else
        reduce_slices_kernel<__nv_bfloat16><<<blocks, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(slices), world, n,
                                                                    static_cast<__nv_bfloat16*>(out));
}

void comm_reduce_staged(const void* own_full, const void* const* staged, int count, const CommSegments& segs, int rank,
                        int world, void* out, bool out_f32, float scale, bool accumulate, int blocks, float* norm_out,
                        cudaStream_t st) {
    StagedSlices sl;
    sl.count = count;
    for (int k = 0; k < count; ++k) sl.p[k] = static_cast<const __nv_bfloat16*>(staged[k]);
    if (out_f32)
        reduce_staged_kernel<float><<<blocks, 512, 0, st>>>(static_cast<const __nv_bfloat16*>(own_full), sl, segs, rank,
                                                            world, static_cast<float*>(out), scale, accumulate ? 1 : 0,
                                                            norm_out);
    else
        reduce_staged_kernel<__nv_bfloat16><<<blocks, 512, 0, st>>>(static_cast<const __nv_bfloat16*>(own_full), sl,
                                                                    segs, rank, world, static_cast<__nv_bfloat16*>(out),
                                                                    scale, accumulate ? 1 : 0, norm_out);
}

void comm_allreduce_multimem(const CommPeers& peers, void* multicast_base, long long byte_off, long long numel, bool f32,
                             float scale, int slot_in, int slot_out, uint32_t epoch, unsigned int* counter, int blocks,
                             int* status, cudaStream_t st) {
    char* mc = static_cast<char*>(multicast_base);
    if (f32)
        allreduce_multimem_kernel<float><<<blocks, 512, 0, st>>>(peers, mc, byte_off, numel, scale, slot_in, slot_out,
                                                                 epoch, counter, status);
    else
        allreduce_multimem_kernel<__nv_bfloat16><<<blocks, 512, 0, st>>>(peers, mc, byte_off, numel, scale, slot_in,
                                                                         slot_out, epoch, counter, status);
}

void comm_allreduce_inplace(const CommPeers& peers, long long byte_off, long long numel, bool f32, float scale,
                            int slot_in, int slot_mid, uint32_t epoch, unsigned int* counter, int blocks, int* status,
                            cudaStream_t st) {
    if (f32)
        allreduce_inplace_kernel<float><<<blocks, 512, 0, st>>>(peers, byte_off, numel, scale, slot_in, slot_mid, epoch,
                                                                counter, status);
    else
        allreduce_inplace_kernel<__nv_bfloat16><<<blocks, 512, 0, st>>>(peers, byte_off, numel, scale, slot_in,
                                                                        slot_mid, epoch, counter, status);
}

}  // namespace fs2
