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
#include <stdlib.h>
#include <atomic>

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

// ---------------------------------------------------------------------------------------
// Programmatic dependent launch.  A kernel launched with `launch_dependent` may start while
// the kernel before it in the stream is still running: it runs its prologue (index math,
// barrier set-up, loads of data no earlier kernel writes, such as weights) and must call
// `wait_for_previous_kernels()` before it touches anything an earlier kernel reads or writes.
// `let_next_kernel_start()` tells the scheduler that the next kernel may be brought onto the
// SMs; its own wait still holds it until this kernel has finished and its writes are visible.
// Setting RI_B200_NO_PDL=1 launches everything strictly one after another.
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ void wait_for_previous_kernels() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void let_next_kernel_start() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

inline bool pdl_enabled() {
    static int on = -1;
    if (on < 0) {
        const char* e = getenv("RI_B200_NO_PDL");
        on = (e != nullptr && e[0] == '1') ? 0 : 1;
    }
    return on == 1;
}

template <typename... KArgs, typename... Args>
inline cudaError_t launch_dependent(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                    cudaStream_t stream, Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

inline int check_launch(cudaError_t e, const char* what) {
    if (e != cudaSuccess) return fail("%s: launch failed: %s", what, cudaGetErrorString(e));
    return check_launch(what);
}

// A kernel's limit of dynamic shared memory is an attribute of ONE device's copy of the kernel.  This
// remembers, per device, that it has been raised: a bit per device (0..63), set with an atomic OR, so
// every device a process uses is configured once, whichever host thread gets there first (two threads
// that race both set the same value).  Devices beyond 63 are configured at every call.
struct PerDeviceOnce {
    std::atomic<unsigned long long> done{0ull};
};

template <typename Kernel>
inline int raise_dynamic_smem(Kernel kernel, int bytes, PerDeviceOnce& once, const char* what) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return fail("%s: cudaGetDevice failed: %s", what, cudaGetErrorString(e));
    const bool tracked = dev >= 0 && dev < 64;
    if (tracked && ((once.done.load(std::memory_order_acquire) >> dev) & 1ull)) return 0;
    e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    if (e != cudaSuccess) return fail("%s: cannot raise dynamic shared memory: %s", what, cudaGetErrorString(e));
    if (tracked) once.done.fetch_or(1ull << dev, std::memory_order_release);
    return 0;
}

}  // namespace ri

// ---------------------------------------------------------------------------------------
// The checked build (-DRI_CHECK_BOUNDS; `RI_B200_CHECK_BOUNDS=1` makes the Python side compile and load
// it from a folder of its own).  Kernels that reach memory through a table (a token id into the
// embedding, a slot and a page number into the cache) compare the index with its limit first.  An index
// outside is recorded in the library (which check, the index, the limit: the first one; and how many
// there were) and the access is skipped or bent to a safe place: the kernel finishes, nothing faults,
// and the host reads the record with `ri_bounds_report`.  Limits that the kernels are not given as
// arguments (vocabulary, slots, pages) are set once per library with `ri_bounds_set_limits`; a limit of
// 0 is not checked.  In the ordinary build every check is the constant `true` and costs nothing.
// ---------------------------------------------------------------------------------------
enum { RI_LIMIT_VOCAB = 0, RI_LIMIT_SLOTS = 1, RI_LIMIT_PAGES = 2 };
enum { RI_CHECK_TOKEN_ID = 1, RI_CHECK_SLOT = 2, RI_CHECK_PAGE_INDEX = 3, RI_CHECK_PAGE = 4 };

#ifdef RI_CHECK_BOUNDS
namespace ri {
__device__ int g_limits[3];
__device__ int g_bounds[4];        // {check, index, limit} of the first index outside its range, and their number

// `record`: whether this thread writes the record (an index that every thread of a block checks alike is
// recorded by its first thread only, so that the count is of indices, not of threads).
__device__ __forceinline__ bool in_range(long long i, long long limit, int check, bool record) {
    if (limit <= 0 || (i >= 0 && i < limit)) return true;
    if (record && atomicAdd(&g_bounds[3], 1) == 0) {
        g_bounds[0] = check;
        g_bounds[1] = (int)i;
        g_bounds[2] = (int)limit;
    }
    return false;
}
}  // namespace ri
#define RI_IN_LIMIT(i, which, check) ri::in_range((long long)(i), (long long)ri::g_limits[which], check, true)
#define RI_BLOCK_IN_RANGE(i, limit, check) ri::in_range((long long)(i), (long long)(limit), check, threadIdx.x == 0)
#define RI_BLOCK_IN_LIMIT(i, which, check) \
    ri::in_range((long long)(i), (long long)ri::g_limits[which], check, threadIdx.x == 0)
#define RI_DEFINE_BOUNDS()                                                                                     \
    RI_API int ri_bounds_set_limits(int vocab, int slots, int pages) {                                         \
        const int v[3] = {vocab, slots, pages};                                                                \
        cudaError_t e = cudaMemcpyToSymbol(ri::g_limits, v, sizeof(v));                                        \
        return e == cudaSuccess ? 0 : ri::fail("bounds: cannot set the limits: %s", cudaGetErrorString(e));   \
    }                                                                                                          \
    /* out[0..4): check, index, limit, count; the record is cleared.  Synchronises the device. */              \
    RI_API int ri_bounds_report(int* out) {                                                                    \
        const int zero[4] = {0, 0, 0, 0};                                                                      \
        cudaError_t e = cudaMemcpyFromSymbol(out, ri::g_bounds, 4 * sizeof(int));                              \
        if (e == cudaSuccess) e = cudaMemcpyToSymbol(ri::g_bounds, zero, sizeof(zero));                        \
        return e == cudaSuccess ? 0 : ri::fail("bounds: cannot read the record: %s", cudaGetErrorString(e));  \
    }
#else
#define RI_IN_LIMIT(i, which, check) true
#define RI_BLOCK_IN_RANGE(i, limit, check) true
#define RI_BLOCK_IN_LIMIT(i, which, check) true
#define RI_DEFINE_BOUNDS()                                                                                     \
    RI_API int ri_bounds_set_limits(int, int, int) { return ri::fail("this library is not a checked build"); } \
    RI_API int ri_bounds_report(int*) { return ri::fail("this library is not a checked build"); }
#endif

#define RI_DEFINE_LAST_ERROR() \
    RI_DEFINE_BOUNDS()         \
    RI_API const char* ri_last_error() { return ri::error_buffer(); }
