// Shared helpers of the sm_100a kernels: the C ABI conventions, error reporting,
// element conversion and block reductions.
//
// Every exported function is `extern "C"`, takes raw device pointers plus a CUDA
// stream, launches on that stream and returns 0, or a non-zero code after storing a
// message that `ri_last_error()` returns.  Nothing here allocates device memory.
#pragma once

#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <stdio.h>
#include <stdarg.h>

#define RI_API extern "C" __attribute__((visibility("default")))

enum RiDtype { RI_F32 = 0, RI_BF16 = 1 };

namespace ri {

inline char* error_buffer() {
    static thread_local char buf[768];
    return buf;
}

inline int fail(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(error_buffer(), 768, fmt, ap);
    va_end(ap);
    return 1;
}

inline int check_launch(const char* what) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail("%s: launch failed: %s", what, cudaGetErrorString(e));
    return 0;
}

template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

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

// Block-wide sum / max; `scratch` holds at least 33 floats of shared memory.  All threads
// of the block must call; all get the result.  blockDim.x must be a multiple of 32.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
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
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
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

// The reference's SiLU, stable on both sides (math.rs:137-146).
__device__ __forceinline__ float silu_f32(float x) {
    if (x >= 0.f) {
        return x / (1.f + expf(-x));
    } else {
        float e = expf(x);
        return x * e / (1.f + e);
    }
}

}  // namespace ri

#define RI_DEFINE_LAST_ERROR() \
    RI_API const char* ri_last_error() { return ri::error_buffer(); }
