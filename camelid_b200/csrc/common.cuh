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

// Sum over the block in a fixed order (lane tree inside a warp, then the same tree over the
// warps' sums, which every warp computes for itself), so the result of a row does not depend
// on anything but the row, and one barrier is enough. `red` holds at least 32 floats; a second
// call may follow only after another barrier of the block (the settled-row loops have one).
__device__ __forceinline__ float block_sum(float v, float* red) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    if (lane == 0) red[warp] = v;
    __syncthreads();
    return warp_sum(lane < nwarps ? red[lane] : 0.f);
}

// Programmatic dependent launch: a kernel launched with `launch_pdl` may begin while the
// kernel before it in the stream is still running; `pdl_wait()` holds a thread until every
// earlier kernel has completed and its writes are visible, so it comes before the first
// access to anything an earlier kernel wrote (or still reads). `pdl_launch_dependents()`
// lets the next kernel start its own prologue early. Without the launch attribute both are
// no-ops. cml_set_dependent_launch(0) makes this module launch plainly.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

static int cml_dependent_launch_on = 1;
static inline bool cml_pdl_enabled() { return cml_dependent_launch_on == 1; }
#ifndef CML_NO_LAUNCH_SETTER      // one definition per module: a second source file of a module defines this first
extern "C" void cml_set_dependent_launch(int on) { cml_dependent_launch_on = on ? 1 : 0; }
#endif

template <typename... KArgs, typename... Args>
static inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                     Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = cml_pdl_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

// Raises a kernel's limit of dynamic shared memory, once per kernel and size: the call costs
// about as much as a launch's own bookkeeping and a step launches each kernel many times.
template <auto Kernel>
static inline cudaError_t cml_allow_smem(size_t smem) {
    static size_t allowed = 0;
    if (smem <= allowed) return cudaSuccess;
    const cudaError_t e = cudaFuncSetAttribute(Kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e == cudaSuccess) allowed = smem;
    return e;
}

static inline int cml_sm_count() {
    static int sms = 0;
    if (sms <= 0) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
            sms = 148;
    }
    return sms;
}

static inline int cml_launch_status() {
    cudaError_t e = cudaGetLastError();
    return (int)e;
}
