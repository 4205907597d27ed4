// Device-side helpers shared by the kernels that talk to peers through the symmetric arena (comm.cu, moe.cu):
// release/acquire accesses to the epoch flags, 16-byte peer loads/stores, and the bounded signal-and-wait.
#pragma once

#include <cuda_runtime.h>

#include <cstdint>

#include "comm.h"
#include "common.cuh"

namespace fs2 {

namespace {

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// 16-byte load that bypasses L1 (peer data changes between epochs).
__device__ __forceinline__ uint4 ld_peer16(const void* p) {
    uint4 v;
    asm volatile("ld.relaxed.sys.global.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p)
                 : "memory");
    return v;
}

__device__ __forceinline__ void st16(void* p, uint4 v) {
    asm volatile("st.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
                 : "memory");
}

// One thread stores `epoch` into this rank's column of `slot` in every rank's flag page.
__device__ __forceinline__ void signal_all(const CommPeers& peers, int slot, uint32_t epoch) {
    for (int r = 0; r < peers.world; ++r) {
        uint32_t* f = reinterpret_cast<uint32_t*>(peers.base[r]) + slot * kCommMaxRanks + peers.rank;
        st_release_sys(f, epoch);
    }
}

// One thread waits (bounded) until every peer's flag in `slot` reached `epoch`; no block-wide synchronisation.
__device__ __forceinline__ bool wait_all_one_thread(const CommPeers& peers, int slot, uint32_t epoch, int* status,
                                                    int site) {
    const uint32_t* mine = reinterpret_cast<const uint32_t*>(peers.base[peers.rank]) + slot * kCommMaxRanks;
    const uint64_t t0 = global_timer_ns();
    for (int r = 0; r < peers.world; ++r) {
        uint32_t spins = 0;
        while (static_cast<int32_t>(ld_acquire_sys(mine + r) - epoch) < 0) {
            if ((++spins & 255u) == 0 && global_timer_ns() - t0 > peers.wait_limit_ns) {
                report_status(status, kStatusTimeout | (site << 8));
                return false;
            }
        }
    }
    return true;
}

// Thread 0 of the block signals (optionally) and waits until every peer's flag
// in `slot` reached `epoch`; returns false for the whole block on time-out.
__device__ __forceinline__ bool signal_and_wait(const CommPeers& peers, int slot, uint32_t epoch, bool do_signal,
                                                int* status, int site) {
    __shared__ int ok_flag;
    if (threadIdx.x == 0) {
        int ok = 1;
        if (do_signal && blockIdx.x == 0) {
            __threadfence_system();
            for (int r = 0; r < peers.world; ++r) {
                uint32_t* f = reinterpret_cast<uint32_t*>(peers.base[r]) + slot * kCommMaxRanks + peers.rank;
                st_release_sys(f, epoch);
            }
        }
        const uint32_t* mine = reinterpret_cast<const uint32_t*>(peers.base[peers.rank]) + slot * kCommMaxRanks;
        const uint64_t t0 = global_timer_ns();
        for (int r = 0; r < peers.world && ok; ++r) {
            uint32_t spins = 0;
            // epochs only grow; compare with wrap-around safe arithmetic
            while (static_cast<int32_t>(ld_acquire_sys(mine + r) - epoch) < 0) {
                if ((++spins & 255u) == 0 && global_timer_ns() - t0 > peers.wait_limit_ns) {
                    ok = 0;
                    report_status(status, kStatusTimeout | (site << 8));
                    break;
                }
            }
        }
        ok_flag = ok;
    }
    __syncthreads();
    return ok_flag != 0;
}

}  // namespace

}  // namespace fs2
