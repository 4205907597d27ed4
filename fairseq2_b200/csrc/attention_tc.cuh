// Helpers shared by the tcgen05 attention kernels (forward and backward).
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>

#include "common.cuh"

namespace fs2 {
namespace tc {

constexpr uint64_t WAIT_NS = 2000000000ull;
constexpr float LOG2E = 1.4426950408889634f;

// Instruction descriptor of a bf16 x bf16 -> f32 tcgen05.mma with a K-major A operand.
__device__ __forceinline__ uint32_t make_idesc_bf16(int m, int n, bool b_mn) {
    uint32_t d = 0;
    d |= 1u << 4;                                  // D: f32
    d |= 1u << 7;                                  // A: bf16
    d |= 1u << 10;                                 // B: bf16
    d |= (b_mn ? 1u : 0u) << 16;                   // B major: 0 = K, 1 = MN
    d |= static_cast<uint32_t>(n >> 3) << 17;
    d |= static_cast<uint32_t>(m >> 4) << 24;
    return d;
}

__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ uint32_t pack2_bf16(float a, float b) {
    __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
}

// Warp-uniform bounded wait: every lane takes the same branch because the TMEM loads that
// follow are warp-collective.
__device__ __forceinline__ bool warp_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
    const bool got = mbar_wait_bounded(bar, parity, abort_flag, WAIT_NS);
    return __all_sync(0xffffffffu, got);
}

// Stores 8 bf16 (one 16-byte chunk) of row `row` at chunk index `chunk` (0..7) of a 128B-swizzled,
// K-major [rows][64] tile that starts at shared address `tile` (1024-byte aligned).
__device__ __forceinline__ void st_swizzled_chunk(uint32_t tile, int row, uint32_t chunk, const float* e) {
    const uint32_t dst = tile + static_cast<uint32_t>(row) * 128u + (((chunk ^ static_cast<uint32_t>(row & 7)) & 7u) << 4);
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(pack2_bf16(e[0], e[1])),
                 "r"(pack2_bf16(e[2], e[3])), "r"(pack2_bf16(e[4], e[5])), "r"(pack2_bf16(e[6], e[7]))
                 : "memory");
}

// ------------------------------------------------------------------ host side
using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                              const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                              CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeFn encode_fn() {
    static EncodeFn fn = nullptr;
    if (fn == nullptr) {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) != cudaSuccess)
            return nullptr;
        fn = reinterpret_cast<EncodeFn>(ptr);
    }
    return fn;
}

inline char* tmap_error() {
    static thread_local char buf[256];
    return buf;
}

// [rows, cols] bf16 view whose rows are `row_stride` elements apart; box = [box_rows][64 cols], 128B swizzle.
inline bool make_view_tmap(CUtensorMap* m, const void* ptr, uint64_t rows, uint64_t cols, uint64_t row_stride,
                           uint32_t box_rows) {
    EncodeFn fn = encode_fn();
    if (fn == nullptr) {
        snprintf(tmap_error(), 256, "cuTensorMapEncodeTiled entry point not found");
        return false;
    }
    cuuint64_t dims[2] = {cols, rows};
    cuuint64_t strides[1] = {row_stride * 2};
    cuuint32_t box[2] = {64, box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        snprintf(tmap_error(), 256, "cuTensorMapEncodeTiled failed with CUresult %d (rows %llu, cols %llu, stride %llu)",
                 static_cast<int>(r), static_cast<unsigned long long>(rows), static_cast<unsigned long long>(cols),
                 static_cast<unsigned long long>(row_stride));
        return false;
    }
    return true;
}

}  // namespace tc
}  // namespace fs2
