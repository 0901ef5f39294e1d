// Shared helpers of the sm_100a kernels: element types, error reporting,
// warp and block reductions.  Every exported function is `extern "C"`, takes a
// CUDA stream, launches asynchronously and returns 0 or an error code; the
// message of the last error is kept per thread (hymt2_last_error).
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define HYMT2_API extern "C" __attribute__((visibility("default")))

enum Hymt2DType : int { HYMT2_F32 = 0, HYMT2_BF16 = 1 };

enum Hymt2Error : int {
    HYMT2_OK = 0,
    HYMT2_ERR_ARGUMENT = -1,   // a size or type that the kernel does not take
    HYMT2_ERR_LAUNCH = -2,     // the CUDA runtime refused the launch
    HYMT2_ERR_DEVICE = -3,     // a device-side check or bounded wait gave up
};

void hymt2_set_error(const char* fmt, ...);
int hymt2_check_launch(const char* what);

#define HYMT2_REQUIRE(cond, ...)                 \
    do {                                         \
        if (!(cond)) {                           \
            hymt2_set_error(__VA_ARGS__);        \
            return HYMT2_ERR_ARGUMENT;           \
        }                                        \
    } while (0)

// ---------------------------------------------------------------------------
// element access as float
// ---------------------------------------------------------------------------
__device__ __forceinline__ float to_float(float v) { return v; }
__device__ __forceinline__ float to_float(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_float(float v);
template <> __device__ __forceinline__ float from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) {
    return __float2bfloat16_rn(v);
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

// Sum over a block of up to 1024 threads; every thread gets the result.
// `scratch` holds at least 33 floats of shared memory.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarps = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < nwarps ? scratch[lane] : 0.f;
        t = warp_sum(t);
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}
__device__ __forceinline__ float block_max(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarps = (blockDim.x + 31) >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < nwarps ? scratch[lane] : -INFINITY;
        t = warp_max(t);
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}

// ---------------------------------------------------------------------------
// Programmatic dependent launch: a kernel launched through launch_pdl may start while the
// kernel before it in the stream still runs.  It must call pdl_wait() before it touches
// anything that an earlier kernel wrote (or will overwrite something an earlier kernel reads);
// what it does before that (set-up, loads of weights) overlaps the earlier kernel's tail.
// pdl_launch_dependents() lets the next kernel's blocks be scheduled early.
// ---------------------------------------------------------------------------
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

bool hymt2_pdl_enabled();

template <typename... KArgs, typename... Args>
cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = hymt2_pdl_enabled() ? 1 : 0;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

// Dispatch on a runtime dtype code to a typed lambda-like macro body.
#define HYMT2_DISPATCH_DTYPE(code, T, ...)                                   \
    do {                                                                     \
        if ((code) == HYMT2_F32) { using T = float; __VA_ARGS__; }           \
        else if ((code) == HYMT2_BF16) { using T = __nv_bfloat16; __VA_ARGS__; } \
        else { hymt2_set_error("unknown dtype code %d", (int)(code)); return HYMT2_ERR_ARGUMENT; } \
    } while (0)
