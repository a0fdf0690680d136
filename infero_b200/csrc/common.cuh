// Shared device helpers: element types, 32-bit conversions, block reductions and the
// error record that every launcher of this library reports through.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>

typedef __nv_bfloat16 bf16;

// Element type tags passed across the C boundary.
enum : int { INFERO_F32 = 0, INFERO_BF16 = 1 };

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(bf16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 from_f32<bf16>(float v) { return __float2bfloat16_rn(v); }

// Read element i of a vector whose type is only known at run time (norm weights and
// biases keep the width they were stored in).
__device__ __forceinline__ float load_any(const void* p, int dtype, size_t i) {
    return dtype == INFERO_F32 ? ((const float*)p)[i] : __bfloat162float(((const bf16*)p)[i]);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over a block of up to 1024 threads; every thread gets the result.  The order of
// the additions depends only on blockDim, never on the data or the grid.
__device__ __forceinline__ float block_sum(float v, float* smem32) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarps = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) smem32[warp] = v;
    __syncthreads();
    float r = (lane < nwarps) ? smem32[lane] : 0.f;
    r = warp_sum(r);
    return r;
}

// ---- error reporting -------------------------------------------------------------------
// Launchers return 0 on success.  On failure they return non-zero and leave a message
// that infero_last_error() hands to the caller.
void infero_set_error(const char* fmt, ...);
int infero_check_launch(const char* what);

#define INFERO_REQUIRE(cond, ...)                 \
    do {                                          \
        if (!(cond)) {                            \
            infero_set_error(__VA_ARGS__);        \
            return 1;                             \
        }                                         \
    } while (0)
