// Row-wise kernels of the decoder step: embedding gather, RMSNorm, rotary position
// encoding fused with the cache write, and the standalone SiLU-gate.
//
// The residual stream is float32 in both precisions; `T` is the activation/storage
// type (float or bf16).  Statistics, rotation and SiLU are computed in float32.
#include "common.cuh"

using namespace ri;

// ----------------------------------------------------------------------------
// embedding: out[t, :] = table[ids[t], :]        (transformer.rs:74-75)
// ----------------------------------------------------------------------------
template <typename T>
__global__ void embed_gather_kernel(const T* __restrict__ table, const int* __restrict__ ids,
                                    float* __restrict__ out, int hidden) {
    const int t = blockIdx.x;
    let_next_kernel_start();
    wait_for_previous_kernels();          // the ids may come from the previous step's sampler
    const int id = ids[t];
    float* o = out + (size_t)t * hidden;
    if (!RI_BLOCK_IN_LIMIT(id, RI_LIMIT_VOCAB, RI_CHECK_TOKEN_ID)) {           // checked build: recorded, the row left zero
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) o[i] = 0.f;
        return;
    }
    const T* row = table + (size_t)id * hidden;
    if (sizeof(T) == 2 && (hidden & 7) == 0 && (reinterpret_cast<uintptr_t>(table) & 15) == 0 &&
        (reinterpret_cast<uintptr_t>(out) & 15) == 0) {
        // 16 bytes (8 elements) per load, up to four loads of a thread on their way together: the row comes
        // from memory in one trip, not in one trip per element
        constexpr int AHEAD = 4;
        const uint4* src = reinterpret_cast<const uint4*>(row);
        const int n8 = hidden >> 3;
        for (int base = threadIdx.x; base < n8; base += AHEAD * blockDim.x) {
            uint4 v[AHEAD];
#pragma unroll
            for (int j = 0; j < AHEAD; ++j) {
                const int i = base + j * blockDim.x;
                if (i < n8) v[j] = src[i];
            }
#pragma unroll
            for (int j = 0; j < AHEAD; ++j) {
                const int i = base + j * blockDim.x;
                if (i < n8) {
                    const T* e = reinterpret_cast<const T*>(&v[j]);
                    float4* dst = reinterpret_cast<float4*>(o + 8 * (size_t)i);
                    dst[0] = make_float4(to_f32<T>(e[0]), to_f32<T>(e[1]), to_f32<T>(e[2]), to_f32<T>(e[3]));
                    dst[1] = make_float4(to_f32<T>(e[4]), to_f32<T>(e[5]), to_f32<T>(e[6]), to_f32<T>(e[7]));
                }
            }
        }
        return;
    }
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) o[i] = to_f32<T>(row[i]);
}

RI_API int ri_embed_gather(const void* table, int dtype, const int* ids, float* out, int n_tokens,
                           int hidden, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    cudaError_t e = cudaSuccess;
    if (dtype == RI_F32)
        e = launch_dependent(embed_gather_kernel<float>, n_tokens, 256, 0, stream, (const float*)table, ids, out, hidden);
    else if (dtype == RI_BF16)
        e = launch_dependent(embed_gather_kernel<__nv_bfloat16>, n_tokens, 256, 0, stream, (const __nv_bfloat16*)table, ids, out, hidden);
    else
        return fail("embed_gather: unknown dtype %d", dtype);
    return check_launch(e, "embed_gather");
}

// ----------------------------------------------------------------------------
// RMSNorm (math.rs:237-256): ss = sum x^2; rms = sqrt(ss/n + eps); y = x * (1/rms) * w.
// `rows` (may be null) picks the input row of each output row, so the final norm
// runs on the wanted positions only.
// ----------------------------------------------------------------------------
template <typename T>
__global__ void rmsnorm_kernel(const float* __restrict__ x, const float* __restrict__ w,
                               const int* __restrict__ rows, T* __restrict__ out, int n, float eps) {
    __shared__ float scratch[33];
    const int r = blockIdx.x;
    let_next_kernel_start();
    wait_for_previous_kernels();          // x is the residual stream the previous kernel wrote
    const float* xr = x + (size_t)(rows ? rows[r] : r) * n;
    float ss = 0.f;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        float v = xr[i];
        ss += v * v;
    }
    ss = block_sum(ss, scratch);
    const float rms = sqrtf(ss / (float)n + eps);
    const float scale = 1.0f / rms;
    T* o = out + (size_t)r * n;
    for (int i = threadIdx.x; i < n; i += blockDim.x) o[i] = from_f32<T>(xr[i] * scale * w[i]);
}

template <typename T> __device__ __forceinline__ void store4(T* p, float a, float b, float c, float d);
template <> __device__ __forceinline__ void store4<float>(float* p, float a, float b, float c, float d) {
    *reinterpret_cast<float4*>(p) = make_float4(a, b, c, d);
}
template <> __device__ __forceinline__ void store4<__nv_bfloat16>(__nv_bfloat16* p, float a, float b, float c, float d) {
    __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
    uint2 v;
    v.x = *reinterpret_cast<uint32_t*>(&lo);
    v.y = *reinterpret_cast<uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(p) = v;
}

// The same in one pass for rows that are a multiple of 4 wide and at most 4 * PER * blockDim long:
// every thread keeps its float4s of the row in registers, so the row is read once, and the weights
// (which no kernel writes) are fetched before the wait for the previous kernel.
template <typename T, int PER>
__global__ void __launch_bounds__(1024)
rmsnorm_vec_kernel(const float* __restrict__ x, const float* __restrict__ w, const int* __restrict__ rows,
                   T* __restrict__ out, int n, float eps) {
    __shared__ float scratch[33];
    const int r = blockIdx.x, n4 = n >> 2;
    float4 wv[PER], xv[PER];
#pragma unroll
    for (int j = 0; j < PER; ++j) {
        const int i = threadIdx.x + j * blockDim.x;
        wv[j] = i < n4 ? reinterpret_cast<const float4*>(w)[i] : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    const int in_row = rows ? rows[r] : r;                // the wanted rows are fixed before the step's first kernel
    let_next_kernel_start();
    wait_for_previous_kernels();
    const float4* xr = reinterpret_cast<const float4*>(x + (size_t)in_row * n);
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < PER; ++j) {
        const int i = threadIdx.x + j * blockDim.x;
        xv[j] = i < n4 ? xr[i] : make_float4(0.f, 0.f, 0.f, 0.f);
        ss += xv[j].x * xv[j].x + xv[j].y * xv[j].y + xv[j].z * xv[j].z + xv[j].w * xv[j].w;
    }
    ss = block_sum(ss, scratch);
    const float rms = sqrtf(ss / (float)n + eps);
    const float scale = 1.0f / rms;
    T* o = out + (size_t)r * n;
#pragma unroll
    for (int j = 0; j < PER; ++j) {
        const int i = threadIdx.x + j * blockDim.x;
        if (i < n4)
            store4<T>(o + 4 * i, xv[j].x * scale * wv[j].x, xv[j].y * scale * wv[j].y, xv[j].z * scale * wv[j].z,
                      xv[j].w * scale * wv[j].w);
    }
    RI_PHASE_LATEST(5);
}

// Steps of many rows (prompts): one warp per row, the row in registers, no block-wide barrier; the
// weights are read again by every warp (they stay in L1/L2).  CH float4s per lane: rows of up to 512 * CH.
template <typename T, int CH>
__global__ void __launch_bounds__(256)
rmsnorm_warp_kernel(const float* __restrict__ x, const float* __restrict__ w, const int* __restrict__ rows,
                    T* __restrict__ out, int n_rows, int n, float eps) {
    const int lane = threadIdx.x & 31, n4 = n >> 2;
    const int r = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    let_next_kernel_start();
    wait_for_previous_kernels();
    if (r >= n_rows) return;
    const float4* xr = reinterpret_cast<const float4*>(x + (size_t)(rows ? rows[r] : r) * n);
    float4 xv[CH];
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < CH; ++j) {
        const int i = lane + j * 32;
        xv[j] = i < n4 ? xr[i] : make_float4(0.f, 0.f, 0.f, 0.f);
        ss += xv[j].x * xv[j].x + xv[j].y * xv[j].y + xv[j].z * xv[j].z + xv[j].w * xv[j].w;
    }
    ss = warp_sum(ss);
    const float scale = 1.0f / sqrtf(ss / (float)n + eps);
    T* o = out + (size_t)r * n;
#pragma unroll
    for (int j = 0; j < CH; ++j) {
        const int i = lane + j * 32;
        if (i < n4) {
            const float4 wv = reinterpret_cast<const float4*>(w)[i];
            store4<T>(o + 4 * i, xv[j].x * scale * wv.x, xv[j].y * scale * wv.y, xv[j].z * scale * wv.z,
                      xv[j].w * scale * wv.w);
        }
    }
}

template <typename T>
cudaError_t launch_rmsnorm(const float* x, const float* w, const int* rows, T* out, int n_rows, int n, float eps,
                           cudaStream_t stream) {
    const bool vec = n % 4 == 0 && (uintptr_t)x % 16 == 0 && (uintptr_t)w % 16 == 0 && (uintptr_t)out % 16 == 0;
    const int n4 = n / 4;
    if (vec && n_rows >= 256 && n4 <= 32 * 64) {
        // many rows: a warp per row (measured at 2,048 rows of 3584: 14-16 us with a block per row)
        const int ch = (n4 + 31) / 32;
        const int blocks = (n_rows + 7) / 8;
        if (ch <= 8) return launch_dependent(rmsnorm_warp_kernel<T, 8>, blocks, 256, 0, stream, x, w, rows, out, n_rows, n, eps);
        if (ch <= 16) return launch_dependent(rmsnorm_warp_kernel<T, 16>, blocks, 256, 0, stream, x, w, rows, out, n_rows, n, eps);
        if (ch <= 32) return launch_dependent(rmsnorm_warp_kernel<T, 32>, blocks, 256, 0, stream, x, w, rows, out, n_rows, n, eps);
        return launch_dependent(rmsnorm_warp_kernel<T, 64>, blocks, 256, 0, stream, x, w, rows, out, n_rows, n, eps);
    }
    if (vec && n4 <= 4 * 1024) {
        // as many threads as float4s, rounded up to whole warps, at most 1024
        int threads = ((n4 + 31) / 32) * 32;
        if (threads > 1024) threads = 1024;
        const int per = (n4 + threads - 1) / threads;
        if (per <= 1) return launch_dependent(rmsnorm_vec_kernel<T, 1>, n_rows, threads, 0, stream, x, w, rows, out, n, eps);
        if (per <= 2) return launch_dependent(rmsnorm_vec_kernel<T, 2>, n_rows, threads, 0, stream, x, w, rows, out, n, eps);
        return launch_dependent(rmsnorm_vec_kernel<T, 4>, n_rows, threads, 0, stream, x, w, rows, out, n, eps);
    }
    const int threads = n >= 1024 ? 256 : 128;
    return launch_dependent(rmsnorm_kernel<T>, n_rows, threads, 0, stream, x, w, rows, out, n, eps);
}

RI_API int ri_rmsnorm(const float* x, const float* w, const int* rows, void* out, int out_dtype,
                      int n_rows, int n, float eps, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    cudaError_t e = cudaSuccess;
    if (out_dtype == RI_F32)
        e = launch_rmsnorm<float>(x, w, rows, (float*)out, n_rows, n, eps, stream);
    else if (out_dtype == RI_BF16)
        e = launch_rmsnorm<__nv_bfloat16>(x, w, rows, (__nv_bfloat16*)out, n_rows, n, eps, stream);
    else
        return fail("rmsnorm: unknown dtype %d", out_dtype);
    return check_launch(e, "rmsnorm");
}

// ----------------------------------------------------------------------------
// Rotary position encoding + cache write.
//
// qkv is [n_tokens, ld] with q at column 0 (n_heads*hd), k at q_dim, v at q_dim + kv_dim.
// Every q head and every k head is rotated with the table row of the token's position
// (attention.rs:78-87, rope.rs:88-97); q is rotated in place, rotated k and plain v go
// to the token's cache position (attention.rs:89-90, kv_cache.rs:52-75).
//
// style 0: pairs (i, i + hd/2); style 1: pairs (2i, 2i+1), the reference's.
// Cache layer layout: [page][kv head][page_size][hd]; page of position p of sequence b is
// page_table[slot(b) * max_pages + p / page_size].
// ----------------------------------------------------------------------------
template <typename T>
__global__ void rope_cache_write_kernel(T* __restrict__ qkv, int ld, const float* __restrict__ cos_t,
                                        const float* __restrict__ sin_t, const int* __restrict__ token_pos,
                                        const int* __restrict__ token_seq, const int* __restrict__ seq_slot,
                                        const int* __restrict__ page_table, int max_pages,
                                        T* __restrict__ kcache, T* __restrict__ vcache,
                                        int n_heads, int n_kv_heads, int hd, int page_size, int style,
                                        int write_kv) {
    const int t = blockIdx.x;
    let_next_kernel_start();
    wait_for_previous_kernels();          // the projections come from the previous kernel
    const int pos = token_pos[t];
    const int half = hd >> 1;
    T* row = qkv + (size_t)t * ld;
    const float* c = cos_t + (size_t)pos * half;
    const float* s = sin_t + (size_t)pos * half;
    const int q_dim = n_heads * hd, kv_dim = n_kv_heads * hd;

    size_t cache_base = 0;
    if (write_kv) {
        const int slot = seq_slot[token_seq[t]];
        // checked build: a slot, a page index or a page outside its range is recorded and nothing is written
        if (!RI_BLOCK_IN_LIMIT(slot, RI_LIMIT_SLOTS, RI_CHECK_SLOT) || !RI_BLOCK_IN_RANGE(pos / page_size, max_pages, RI_CHECK_PAGE_INDEX)) {
            write_kv = 0;
        } else {
            const int page = page_table[(size_t)slot * max_pages + pos / page_size];
            if (!RI_BLOCK_IN_LIMIT(page, RI_LIMIT_PAGES, RI_CHECK_PAGE)) write_kv = 0;
            cache_base = ((size_t)page * n_kv_heads * page_size + (pos % page_size)) * hd;
        }
    }
    const size_t head_stride = (size_t)page_size * hd;

    // q heads: rotate in place
    for (int idx = threadIdx.x; idx < n_heads * half; idx += blockDim.x) {
        const int h = idx / half, i = idx % half;
        const int i0 = style == 0 ? i : 2 * i;
        const int i1 = style == 0 ? i + half : 2 * i + 1;
        T* v = row + h * hd;
        const float x0 = to_f32<T>(v[i0]), x1 = to_f32<T>(v[i1]);
        v[i0] = from_f32<T>(x0 * c[i] - x1 * s[i]);
        v[i1] = from_f32<T>(x0 * s[i] + x1 * c[i]);
    }
    if (!write_kv) return;
    // k heads: rotate into the cache
    for (int idx = threadIdx.x; idx < n_kv_heads * half; idx += blockDim.x) {
        const int h = idx / half, i = idx % half;
        const int i0 = style == 0 ? i : 2 * i;
        const int i1 = style == 0 ? i + half : 2 * i + 1;
        const T* v = row + q_dim + h * hd;
        const float x0 = to_f32<T>(v[i0]), x1 = to_f32<T>(v[i1]);
        T* dst = kcache + cache_base + h * head_stride;
        dst[i0] = from_f32<T>(x0 * c[i] - x1 * s[i]);
        dst[i1] = from_f32<T>(x0 * s[i] + x1 * c[i]);
    }
    // v heads: copy
    for (int idx = threadIdx.x; idx < kv_dim; idx += blockDim.x) {
        const int h = idx / hd, d = idx % hd;
        vcache[cache_base + h * head_stride + d] = row[q_dim + kv_dim + idx];
    }
}

// The same for bf16 rows whose head size is a multiple of 16, moved 16 bytes at a time: a thread takes
// 8 consecutive elements of a head (and, for the half-split pairing, their 8 partners half a head on),
// rotates them in float32 and writes them back the same way.
__device__ __forceinline__ void unpack8(const uint4& v, float* f) {
    const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 x = __bfloat1622float2(p[i]);
        f[2 * i] = x.x;
        f[2 * i + 1] = x.y;
    }
}
__device__ __forceinline__ uint4 pack8(const float* f) {
    uint4 v;
    __nv_bfloat162* p = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) p[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
    return v;
}

__global__ void rope_cache_write_vec_kernel(__nv_bfloat16* __restrict__ qkv, int ld, const float* __restrict__ cos_t,
                                            const float* __restrict__ sin_t, const int* __restrict__ token_pos,
                                            const int* __restrict__ token_seq, const int* __restrict__ seq_slot,
                                            const int* __restrict__ page_table, int max_pages,
                                            __nv_bfloat16* __restrict__ kcache, __nv_bfloat16* __restrict__ vcache,
                                            int n_heads, int n_kv_heads, int hd, int page_size, int style,
                                            int write_kv) {
    const int t = blockIdx.x;
    let_next_kernel_start();
    const int pos = token_pos[t];                     // positions, slots, pages and angles: fixed before the step
    const int half = hd >> 1;
    const float* c = cos_t + (size_t)pos * half;
    const float* s = sin_t + (size_t)pos * half;
    const int q_dim = n_heads * hd, kv_dim = n_kv_heads * hd;
    size_t cache_base = 0;
    if (write_kv) {
        const int slot = seq_slot[token_seq[t]];
        // checked build: a slot, a page index or a page outside its range is recorded and nothing is written
        if (!RI_BLOCK_IN_LIMIT(slot, RI_LIMIT_SLOTS, RI_CHECK_SLOT) || !RI_BLOCK_IN_RANGE(pos / page_size, max_pages, RI_CHECK_PAGE_INDEX)) {
            write_kv = 0;
        } else {
            const int page = page_table[(size_t)slot * max_pages + pos / page_size];
            if (!RI_BLOCK_IN_LIMIT(page, RI_LIMIT_PAGES, RI_CHECK_PAGE)) write_kv = 0;
            cache_base = ((size_t)page * n_kv_heads * page_size + (pos % page_size)) * hd;
        }
    }
    const size_t head_stride = (size_t)page_size * hd;
    wait_for_previous_kernels();          // the projections come from the previous kernel
    __nv_bfloat16* row = qkv + (size_t)t * ld;

    const int heads = n_heads + (write_kv ? n_kv_heads : 0);
    if (style == 0) {
        const int per_head = half / 8;                // chunk pairs of a head
        for (int idx = threadIdx.x; idx < heads * per_head; idx += blockDim.x) {
            const int h = idx / per_head, j = idx % per_head;
            const __nv_bfloat16* src = row + (size_t)h * hd + 8 * j;      // q heads, then k heads: one run of columns
            float lo[8], hi[8], cs[8], sn[8], ylo[8], yhi[8];
            unpack8(*reinterpret_cast<const uint4*>(src), lo);
            unpack8(*reinterpret_cast<const uint4*>(src + half), hi);
            *reinterpret_cast<float4*>(cs) = *reinterpret_cast<const float4*>(c + 8 * j);
            *reinterpret_cast<float4*>(cs + 4) = *reinterpret_cast<const float4*>(c + 8 * j + 4);
            *reinterpret_cast<float4*>(sn) = *reinterpret_cast<const float4*>(s + 8 * j);
            *reinterpret_cast<float4*>(sn + 4) = *reinterpret_cast<const float4*>(s + 8 * j + 4);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                ylo[i] = lo[i] * cs[i] - hi[i] * sn[i];
                yhi[i] = lo[i] * sn[i] + hi[i] * cs[i];
            }
            __nv_bfloat16* dst = h < n_heads ? row + (size_t)h * hd + 8 * j
                                             : kcache + cache_base + (size_t)(h - n_heads) * head_stride + 8 * j;
            *reinterpret_cast<uint4*>(dst) = pack8(ylo);
            *reinterpret_cast<uint4*>(dst + half) = pack8(yhi);
        }
    } else {
        const int per_head = hd / 8;                  // chunks of a head, 4 adjacent pairs each
        for (int idx = threadIdx.x; idx < heads * per_head; idx += blockDim.x) {
            const int h = idx / per_head, j = idx % per_head;
            const __nv_bfloat16* src = row + (size_t)h * hd + 8 * j;
            float x[8], y[8], cs[4], sn[4];
            unpack8(*reinterpret_cast<const uint4*>(src), x);
            *reinterpret_cast<float4*>(cs) = *reinterpret_cast<const float4*>(c + 4 * j);
            *reinterpret_cast<float4*>(sn) = *reinterpret_cast<const float4*>(s + 4 * j);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                y[2 * i] = x[2 * i] * cs[i] - x[2 * i + 1] * sn[i];
                y[2 * i + 1] = x[2 * i] * sn[i] + x[2 * i + 1] * cs[i];
            }
            __nv_bfloat16* dst = h < n_heads ? row + (size_t)h * hd + 8 * j
                                             : kcache + cache_base + (size_t)(h - n_heads) * head_stride + 8 * j;
            *reinterpret_cast<uint4*>(dst) = pack8(y);
        }
    }
    if (!write_kv) return;
    const int v_chunks = hd / 8;
    for (int idx = threadIdx.x; idx < n_kv_heads * v_chunks; idx += blockDim.x) {
        const int h = idx / v_chunks, j = idx % v_chunks;
        *reinterpret_cast<uint4*>(vcache + cache_base + (size_t)h * head_stride + 8 * j) =
            *reinterpret_cast<const uint4*>(row + q_dim + kv_dim + (size_t)h * hd + 8 * j);
    }
}

RI_API int ri_rope_cache_write(void* qkv, int dtype, int ld, const float* cos_t, const float* sin_t,
                               const int* token_pos, const int* token_seq, const int* seq_slot,
                               const int* page_table, int max_pages, void* kcache, void* vcache,
                               int n_tokens, int n_heads, int n_kv_heads, int hd, int page_size,
                               int style, int write_kv, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (hd % 2) return fail("rope_cache_write: head_dim %d is odd", hd);
    if (style != 0 && style != 1) return fail("rope_cache_write: unknown style %d", style);
    const int work = n_heads * hd / 2;
    const int threads = work >= 256 ? 256 : (work >= 128 ? 128 : 64);
    cudaError_t e = cudaSuccess;
    const bool aligned = hd % 16 == 0 && ld % 8 == 0 && (uintptr_t)qkv % 16 == 0 && (uintptr_t)kcache % 16 == 0 &&
                         (uintptr_t)vcache % 16 == 0 && (uintptr_t)cos_t % 16 == 0 && (uintptr_t)sin_t % 16 == 0;
    if (dtype == RI_BF16 && aligned) {
        const int items = (n_heads + n_kv_heads) * hd / 16;
        const int vthreads = items >= 256 ? 256 : (items >= 128 ? 128 : 64);
        e = launch_dependent(rope_cache_write_vec_kernel, n_tokens, vthreads, 0, stream,
            (__nv_bfloat16*)qkv, ld, cos_t, sin_t, token_pos, token_seq, seq_slot, page_table, max_pages,
            (__nv_bfloat16*)kcache, (__nv_bfloat16*)vcache, n_heads, n_kv_heads, hd, page_size, style, write_kv);
        return check_launch(e, "rope_cache_write");
    }
    if (dtype == RI_F32)
        e = launch_dependent(rope_cache_write_kernel<float>, n_tokens, threads, 0, stream,
            (float*)qkv, ld, cos_t, sin_t, token_pos, token_seq, seq_slot, page_table, max_pages,
            (float*)kcache, (float*)vcache, n_heads, n_kv_heads, hd, page_size, style, write_kv);
    else if (dtype == RI_BF16)
        e = launch_dependent(rope_cache_write_kernel<__nv_bfloat16>, n_tokens, threads, 0, stream,
            (__nv_bfloat16*)qkv, ld, cos_t, sin_t, token_pos, token_seq, seq_slot, page_table, max_pages,
            (__nv_bfloat16*)kcache, (__nv_bfloat16*)vcache, n_heads, n_kv_heads, hd, page_size, style, write_kv);
    else
        return fail("rope_cache_write: unknown dtype %d", dtype);
    return check_launch(e, "rope_cache_write");
}

// ----------------------------------------------------------------------------
// The same, fed from float32 accumulators.  When the q/k/v projection of a small step is split
// over K, its pieces are summed into a zeroed float32 buffer acc[n_tokens, ld]; this kernel adds
// the bias, rotates in float32 (q and k never pass through the storage type before rotation),
// writes q to q_out[n_tokens, q_dim] and k, v to the cache, and puts zeros back into `acc`, so
// that the buffer is clean for the next projection.
// ----------------------------------------------------------------------------
template <typename T>
__global__ void rope_cache_write_acc_kernel(float* __restrict__ acc, int ld, const float* __restrict__ bias,
                                            T* __restrict__ q_out, const float* __restrict__ cos_t,
                                            const float* __restrict__ sin_t, const int* __restrict__ token_pos,
                                            const int* __restrict__ token_seq, const int* __restrict__ seq_slot,
                                            const int* __restrict__ page_table, int max_pages,
                                            T* __restrict__ kcache, T* __restrict__ vcache, int n_heads,
                                            int n_kv_heads, int hd, int page_size, int style, int write_kv) {
    constexpr int PER = 4;                 // items a thread handles at once: their loads go out together
    const int t = blockIdx.x;
    const int half = hd >> 1;
    const int q_dim = n_heads * hd, kv_dim = n_kv_heads * hd;
    const int n_pairs = (n_heads + n_kv_heads) * half;
    float* row = acc + (size_t)t * ld;
    let_next_kernel_start();
    // Positions, slots, the page table, the angle tables and the bias are written by no kernel of the
    // step: they are read (for the first round of items) while the projection before this still runs.
    const int pos = token_pos[t];
    const float* c = cos_t + (size_t)pos * half;
    const float* s = sin_t + (size_t)pos * half;
    size_t cache_base = 0;
    if (write_kv) {
        const int slot = seq_slot[token_seq[t]];
        // checked build: a slot, a page index or a page outside its range is recorded and nothing is written
        if (!RI_BLOCK_IN_LIMIT(slot, RI_LIMIT_SLOTS, RI_CHECK_SLOT) || !RI_BLOCK_IN_RANGE(pos / page_size, max_pages, RI_CHECK_PAGE_INDEX)) {
            write_kv = 0;
        } else {
            const int page = page_table[(size_t)slot * max_pages + pos / page_size];
            if (!RI_BLOCK_IN_LIMIT(page, RI_LIMIT_PAGES, RI_CHECK_PAGE)) write_kv = 0;
            cache_base = ((size_t)page * n_kv_heads * page_size + (pos % page_size)) * hd;
        }
    }
    const size_t head_stride = (size_t)page_size * hd;

    float cs[PER], sn[PER], b0[PER], b1[PER];
    int c0[PER], c1[PER];
    auto constants = [&](int base) {
#pragma unroll
        for (int j = 0; j < PER; ++j) {
            const int idx = base + j * blockDim.x;
            if (idx < n_pairs) {
                const int h = idx / half, i = idx % half;
                c0[j] = h * hd + (style == 0 ? i : 2 * i);
                c1[j] = h * hd + (style == 0 ? i + half : 2 * i + 1);
                b0[j] = bias ? bias[c0[j]] : 0.f;
                b1[j] = bias ? bias[c1[j]] : 0.f;
                cs[j] = c[i];
                sn[j] = s[i];
            }
        }
    };
    constants(threadIdx.x);
    float v_first[PER], vb_first[PER];    // the first round of values and their bias
#pragma unroll
    for (int j = 0; j < PER; ++j) {
        const int idx = threadIdx.x + j * blockDim.x;
        vb_first[j] = (bias != nullptr && idx < kv_dim) ? bias[q_dim + kv_dim + idx] : 0.f;
    }
    wait_for_previous_kernels();          // the projections come from the previous kernel

    // the first round of values goes out with the first round of pairs: one trip to memory, not two
#pragma unroll
    for (int j = 0; j < PER; ++j) {
        const int idx = threadIdx.x + j * blockDim.x;
        if (idx < kv_dim) v_first[j] = row[q_dim + kv_dim + idx];
    }
    // rotary pairs of the q heads and then the k heads (same column order in the accumulator)
    for (int base = threadIdx.x; base < n_pairs; base += PER * blockDim.x) {
        if (base != (int)threadIdx.x) constants(base);
        float x0[PER], x1[PER];
#pragma unroll
        for (int j = 0; j < PER; ++j) {
            const int idx = base + j * blockDim.x;
            if (idx < n_pairs) {
                x0[j] = row[c0[j]] + b0[j];
                x1[j] = row[c1[j]] + b1[j];
            }
        }
#pragma unroll
        for (int j = 0; j < PER; ++j) {
            const int idx = base + j * blockDim.x;
            if (idx < n_pairs) {
                row[c0[j]] = 0.f;
                row[c1[j]] = 0.f;
                const float y0 = x0[j] * cs[j] - x1[j] * sn[j], y1 = x0[j] * sn[j] + x1[j] * cs[j];
                if (c0[j] < q_dim) {
                    q_out[(size_t)t * q_dim + c0[j]] = from_f32<T>(y0);
                    q_out[(size_t)t * q_dim + c1[j]] = from_f32<T>(y1);
                } else if (write_kv) {
                    const int h = (c0[j] - q_dim) / hd;
                    T* dst = kcache + cache_base + h * head_stride;
                    dst[c0[j] - q_dim - h * hd] = from_f32<T>(y0);
                    dst[c1[j] - q_dim - h * hd] = from_f32<T>(y1);
                }
            }
        }
    }
    // values: bias added, stored as they are
    for (int base = threadIdx.x; base < kv_dim; base += PER * blockDim.x) {
        float v[PER];
#pragma unroll
        for (int j = 0; j < PER; ++j) {
            const int idx = base + j * blockDim.x;
            if (idx < kv_dim) {
                if (base == (int)threadIdx.x) {
                    v[j] = v_first[j] + vb_first[j];
                } else {
                    v[j] = row[q_dim + kv_dim + idx];
                    if (bias) v[j] += bias[q_dim + kv_dim + idx];
                }
            }
        }
#pragma unroll
        for (int j = 0; j < PER; ++j) {
            const int idx = base + j * blockDim.x;
            if (idx < kv_dim) {
                row[q_dim + kv_dim + idx] = 0.f;
                if (write_kv) vcache[cache_base + (idx / hd) * head_stride + (idx % hd)] = from_f32<T>(v[j]);
            }
        }
    }
    RI_PHASE_LATEST(5);
}

RI_API int ri_rope_cache_write_acc(float* acc, int ld, const float* bias, void* q_out, int dtype, const float* cos_t,
                                   const float* sin_t, const int* token_pos, const int* token_seq,
                                   const int* seq_slot, const int* page_table, int max_pages, void* kcache,
                                   void* vcache, int n_tokens, int n_heads, int n_kv_heads, int hd, int page_size,
                                   int style, int write_kv, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (hd % 2) return fail("rope_cache_write: head_dim %d is odd", hd);
    if (style != 0 && style != 1) return fail("rope_cache_write: unknown style %d", style);
    if (ld != (n_heads + 2 * n_kv_heads) * hd) return fail("rope_cache_write: accumulator rows of %d, expected %d", ld, (n_heads + 2 * n_kv_heads) * hd);
    const int work = (n_heads + n_kv_heads) * hd / 2;
    const int threads = work >= 512 ? 512 : (work >= 256 ? 256 : 128);
    cudaError_t e = cudaSuccess;
    if (dtype == RI_F32)
        e = launch_dependent(rope_cache_write_acc_kernel<float>, n_tokens, threads, 0, stream,
            acc, ld, bias, (float*)q_out, cos_t, sin_t, token_pos, token_seq, seq_slot, page_table, max_pages,
            (float*)kcache, (float*)vcache, n_heads, n_kv_heads, hd, page_size, style, write_kv);
    else if (dtype == RI_BF16)
        e = launch_dependent(rope_cache_write_acc_kernel<__nv_bfloat16>, n_tokens, threads, 0, stream,
            acc, ld, bias, (__nv_bfloat16*)q_out, cos_t, sin_t, token_pos, token_seq, seq_slot, page_table, max_pages,
            (__nv_bfloat16*)kcache, (__nv_bfloat16*)vcache, n_heads, n_kv_heads, hd, page_size, style, write_kv);
    else
        return fail("rope_cache_write: unknown dtype %d", dtype);
    return check_launch(e, "rope_cache_write_acc");
}

// ----------------------------------------------------------------------------
// SiLU-gate: out[t, i] = silu(gu[t, i]) * gu[t, inter + i]      (mlp.rs:35-43)
// ----------------------------------------------------------------------------
template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ gu, T* __restrict__ out, int inter, size_t total) {
    size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const size_t t = idx / inter;
    const int i = (int)(idx % inter);
    const T* row = gu + t * 2 * (size_t)inter;
    out[idx] = from_f32<T>(silu_f32(to_f32<T>(row[i])) * to_f32<T>(row[inter + i]));
}

// ---------------------------------------------------------------------------------------
// Load-time helpers: a change of precision, and seeded normal numbers for the random-weights mode.
// ---------------------------------------------------------------------------------------
template <typename TI, typename TO>
__global__ void cast_kernel(const TI* __restrict__ in, TO* __restrict__ out, size_t n) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = from_f32<TO>(to_f32<TI>(in[i]));      // bf16 -> float32 is exact; float32 -> bf16 rounds to nearest even
}

RI_API int ri_cast(const void* in, int in_dtype, void* out, int out_dtype, long long n, cudaStream_t stream) {
    if (n <= 0) return 0;
    const unsigned blocks = (unsigned)((n + 255) / 256);
    if (in_dtype == RI_F32 && out_dtype == RI_BF16)
        cast_kernel<float, __nv_bfloat16><<<blocks, 256, 0, stream>>>((const float*)in, (__nv_bfloat16*)out, (size_t)n);
    else if (in_dtype == RI_BF16 && out_dtype == RI_F32)
        cast_kernel<__nv_bfloat16, float><<<blocks, 256, 0, stream>>>((const __nv_bfloat16*)in, (float*)out, (size_t)n);
    else
        return fail("cast: from dtype %d to dtype %d is not a change between float32 and bfloat16", in_dtype, out_dtype);
    return check_launch("cast");
}

__device__ __forceinline__ unsigned long long fill_mix64(unsigned long long z) {
    z += 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

// Element i of a tensor keyed `key` is mean + std * sqrt(-2 ln u1) * cos(2 pi u2), with u1 in (0, 1] and
// u2 in [0, 1) the upper and the next 24 bits of mix64(key ^ mix64(i)): the same number whatever the
// launch shape, the device or the order tensors are made in.
template <typename T>
__global__ void fill_normal_kernel(T* __restrict__ out, size_t n, unsigned long long key, float mean, float std) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const unsigned long long z = fill_mix64(key ^ fill_mix64((unsigned long long)i));
    const float u1 = (float)((z >> 40) + 1ull) * (1.0f / 16777216.0f);
    const float u2 = (float)((z >> 16) & 0xFFFFFFull) * (1.0f / 16777216.0f);
    out[i] = from_f32<T>(mean + std * sqrtf(-2.0f * logf(u1)) * cospif(2.0f * u2));
}

RI_API int ri_fill_normal(void* out, int dtype, long long n, unsigned long long key, float mean, float std,
                          cudaStream_t stream) {
    if (n <= 0) return 0;
    const unsigned blocks = (unsigned)((n + 255) / 256);
    if (dtype == RI_F32) fill_normal_kernel<float><<<blocks, 256, 0, stream>>>((float*)out, (size_t)n, key, mean, std);
    else if (dtype == RI_BF16) fill_normal_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>((__nv_bfloat16*)out, (size_t)n, key, mean, std);
    else return fail("fill_normal: unknown dtype %d", dtype);
    return check_launch("fill_normal");
}

// ---------------------------------------------------------------------------------------
// The end of a decode step of n sequences (one token each): every sequence is one position
// longer, so the step's int32 arrays move on by one and the next step of the same sequences
// needs nothing from the host.  token_pos, seq_start and seq_len each grow by 1; token_ids
// already hold what the sampler drew.  Optionally (null pointers switch a part off): the
// sampler's per-row draw counters grow by 1; the drawn tokens are copied into slot
// (*turn % host_slots) of a ring in pinned host memory and into slot (*turn % log_slots) of a
// ring on the device; then *turn grows by 1.  One thread block; it runs last in the step.
// ---------------------------------------------------------------------------------------
__global__ void advance_decode_kernel(int* __restrict__ token_pos, int* __restrict__ seq_start,
                                      int* __restrict__ seq_len, int n, const int* __restrict__ token_ids,
                                      int* __restrict__ draw_counter, int* __restrict__ turn,
                                      int* __restrict__ host_ring, int host_slots, int* __restrict__ log_ring,
                                      int log_slots) {
    let_next_kernel_start();
    wait_for_previous_kernels();          // every kernel of the step has read the arrays; the sampler has written the tokens
    const int t = turn ? *turn : 0;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        token_pos[i] += 1;
        seq_start[i] += 1;
        seq_len[i] += 1;
        if (draw_counter) draw_counter[i] += 1;
        if (host_ring || log_ring) {
            const int tok = token_ids[i];
            if (host_ring) host_ring[(size_t)(t % host_slots) * n + i] = tok;
            if (log_ring) log_ring[(size_t)(t % log_slots) * n + i] = tok;
        }
    }
    if (host_ring) __threadfence_system();
    __syncthreads();                      // everyone has read *turn
    if (threadIdx.x == 0 && turn) *turn = t + 1;
}

RI_API int ri_advance_decode(int* token_pos, int* seq_start, int* seq_len, int n, const int* token_ids,
                             int* draw_counter, int* turn, int* host_ring, int host_slots, int* log_ring,
                             int log_slots, cudaStream_t stream) {
    if (n <= 0) return 0;
    if ((host_ring && host_slots < 1) || (log_ring && log_slots < 1)) return fail("advance_decode: a ring needs at least one slot");
    if ((host_ring || log_ring) && (!turn || !token_ids)) return fail("advance_decode: rings need the turn counter and the tokens");
    cudaError_t e = launch_dependent(advance_decode_kernel, dim3(1), dim3(256), (size_t)0, stream, token_pos, seq_start,
                                     seq_len, n, token_ids, draw_counter, turn, host_ring, host_slots, log_ring, log_slots);
    return check_launch(e, "advance_decode");
}

RI_API int ri_silu_mul(const void* gu, void* out, int dtype, int n_tokens, int inter, cudaStream_t stream) {
    const size_t total = (size_t)n_tokens * inter;
    if (total == 0) return 0;
    const unsigned blocks = (unsigned)((total + 255) / 256);
    if (dtype == RI_F32)
        silu_mul_kernel<float><<<blocks, 256, 0, stream>>>((const float*)gu, (float*)out, inter, total);
    else if (dtype == RI_BF16)
        silu_mul_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>((const __nv_bfloat16*)gu, (__nv_bfloat16*)out, inter, total);
    else
        return fail("silu_mul: unknown dtype %d", dtype);
    return check_launch("silu_mul");
}

RI_DEFINE_LAST_ERROR()
