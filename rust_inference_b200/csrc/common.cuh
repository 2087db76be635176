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
//
// The timeline build (-DRI_TIMELINE; `RI_B200_TIMELINE=1` makes the Python side compile and load it from
// a folder of its own) makes these two calls keep a record per kernel launch, written by thread 0 of
// block 0: the device-wide timer when the kernel came onto an SM, when its wait for the kernel before
// ended, and at up to RI_TIMELINE_PHASES places a kernel marks with RI_PHASE(k), all with plain stores;
// RI_PHASE_LATEST(k) keeps the latest time at which thread 0 of any block passed.
// `ri_timeline_read` hands the records to the host, which sees a captured step kernel by kernel with
// the overlap it really has.  In the ordinary build none of this exists.
// ---------------------------------------------------------------------------------------
#define RI_TIMELINE_PHASES 6
#ifdef RI_TIMELINE
#define RI_TIMELINE_CAP 4096
#define RI_TIMELINE_WORDS (5 + RI_TIMELINE_PHASES)        // entry time, entry line, wait time, wait line, grid id, phases
__device__ unsigned long long g_timeline[RI_TIMELINE_CAP * RI_TIMELINE_WORDS];
__device__ unsigned int g_timeline_n;
__device__ __forceinline__ unsigned long long global_timer() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
// A launch's record is found by the launch's own number (%gridid, which the hardware gives every
// launch), so that no mark has to wait for an atomic's answer and nothing is kept in shared memory
// (several kernels lay out their shared memory to the byte).  The host sees two launches that fell on
// one record by their count.
__device__ __forceinline__ unsigned long long* timeline_record(unsigned long long& grid) {
    asm volatile("mov.u64 %0, %%gridid;" : "=l"(grid));
    return g_timeline + (size_t)(grid % RI_TIMELINE_CAP) * RI_TIMELINE_WORDS;
}
__device__ __forceinline__ bool timeline_writer() {
    return (blockIdx.x | blockIdx.y | blockIdx.z) == 0 && (threadIdx.x | threadIdx.y | threadIdx.z) == 0;
}
__device__ __forceinline__ void timeline_entry(int line) {
    if (!timeline_writer()) return;
    unsigned long long grid;
    unsigned long long* rec = timeline_record(grid);
    rec[0] = global_timer();
    rec[1] = (unsigned long long)line;
    rec[4] = grid + 1;
    atomicAdd(&g_timeline_n, 1u);                          // the answer is not used: nothing waits for it
}
__device__ __forceinline__ void timeline_mark(int word, int line) {
    if (!timeline_writer()) return;
    unsigned long long grid;
    unsigned long long* rec = timeline_record(grid);
    rec[word] = global_timer();
    if (word == 2) rec[3] = (unsigned long long)line;
}
// the latest time at which thread 0 of ANY block passed this place (one fire-and-forget atomic per block)
__device__ __forceinline__ void timeline_mark_latest(int word) {
    if ((threadIdx.x | threadIdx.y | threadIdx.z) != 0) return;
    unsigned long long grid;
    unsigned long long* rec = timeline_record(grid);
    atomicMax(rec + word, global_timer());
}
#define RI_PHASE(k) ri::timeline_mark(5 + (k), __LINE__)
#define RI_PHASE_LATEST(k) ri::timeline_mark_latest(5 + (k))
__device__ __forceinline__ void wait_for_previous_kernels(int line = __builtin_LINE()) {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    timeline_mark(2, line);
}
__device__ __forceinline__ void let_next_kernel_start(int line = __builtin_LINE()) {
    timeline_entry(line);
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
#else
#define RI_PHASE(k) ((void)0)
#define RI_PHASE_LATEST(k) ((void)0)
__device__ __forceinline__ void wait_for_previous_kernels() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void let_next_kernel_start() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
#endif

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

#ifdef RI_TIMELINE
#define RI_DEFINE_TIMELINE()                                                                                   \
    /* Copies the table of RI_TIMELINE_CAP records (RI_TIMELINE_WORDS words each; a record whose first word  */ \
    /* is 0 is empty) to `out`, clears it and returns how many launches were recorded since the last call    */ \
    /* (-1: error).  Synchronises the device.                                                                */ \
    RI_API int ri_timeline_read(unsigned long long* out, int cap) {                                            \
        if (cap < RI_TIMELINE_CAP) return ri::fail("timeline: room for %d records needed", RI_TIMELINE_CAP), -1; \
        unsigned int n = 0;                                                                                    \
        const size_t bytes = sizeof(unsigned long long) * RI_TIMELINE_CAP * RI_TIMELINE_WORDS;                 \
        cudaError_t e = cudaDeviceSynchronize();                                                               \
        if (e == cudaSuccess) e = cudaMemcpyFromSymbol(&n, ri::g_timeline_n, sizeof(n));                       \
        if (e == cudaSuccess) e = cudaMemcpyFromSymbol(out, ri::g_timeline, bytes);                            \
        void* base = nullptr;                                                                                  \
        if (e == cudaSuccess) e = cudaGetSymbolAddress(&base, ri::g_timeline);                                 \
        if (e == cudaSuccess) e = cudaMemset(base, 0, bytes);                                                  \
        const unsigned int zero = 0;                                                                           \
        if (e == cudaSuccess) e = cudaMemcpyToSymbol(ri::g_timeline_n, &zero, sizeof(zero));                   \
        if (e != cudaSuccess) return ri::fail("timeline: cannot read the records: %s", cudaGetErrorString(e)), -1; \
        return (int)n;                                                                                         \
    }
#else
#define RI_DEFINE_TIMELINE() \
    RI_API int ri_timeline_read(unsigned long long*, int) { return ri::fail("this library is not a timeline build"), -1; }
#endif

#define RI_DEFINE_LAST_ERROR() \
    RI_DEFINE_BOUNDS()         \
    RI_DEFINE_TIMELINE()       \
    RI_API const char* ri_last_error() { return ri::error_buffer(); }
