// Shared helpers of the hand-written sm_100a kernels: element types, conversions, warp and
// block reductions, and the C-ABI conventions of every launcher.
//
// Every launcher is `extern "C" int cml_<name>(..., void* stream)`: pointers are device
// pointers, `stream` is a cudaStream_t, the return value is 0 or a cudaError_t / a negative
// library code (CML_ERR_*). Launchers allocate nothing; scratch memory is passed in.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>

#define CML_DTYPE_F32 0
#define CML_DTYPE_BF16 1

#define CML_ERR_BAD_DTYPE (-2)
#define CML_ERR_BAD_SIZE (-3)
#define CML_ERR_BAD_ALIGN (-4)

// Tokens of a cache page. The host-side page allocator uses the same number.
#define CML_PAGE 64

typedef __nv_bfloat16 bf16;

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(bf16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 from_f32<bf16>(float v) { return __float2bfloat16_rn(v); }

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

// Sum over the block in a fixed order (lane tree, then warps in index order), so the result
// of a row does not depend on anything but the row. `red` holds at least 33 floats.
__device__ __forceinline__ float block_sum(float v, float* red) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    if (lane == 0) red[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = 0.f;
        for (int i = 0; i < nwarps; ++i) t += red[i];
        if (lane == 0) red[32] = t;
    }
    __syncthreads();
    float out = red[32];
    __syncthreads();
    return out;
}

static inline int cml_launch_status() {
    cudaError_t e = cudaGetLastError();
    return (int)e;
}
