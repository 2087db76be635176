// Attention over the paged cache for any head size, any number of heads and groups and
// any mix of query lengths: the 32-bit path's kernel and the bf16 path's fallback.
//
// One block per (query token, query head).  The token at position p of its sequence
// sees the cached keys 0..p of its slot, nothing else: causal by construction, as in
// attention.rs:92-121.  scores = dot(q, k) * scale, the scale applied to the finished dot
// product (attention.rs:100-110); softmax with the maximum subtracted (math.rs:104-118),
// here computed online over chunks of keys; weighted sum of the values (attention.rs:
// 114-120).  Query head h reads kv head h / (n_heads / n_kv_heads) (attention.rs:95-98).
// All arithmetic is float32 with accurate expf.
//
// `window` > 0 limits the keys to the last `window` positions (p-window+1 .. p); the
// dense decoder passes 0.
#include "common.cuh"

using namespace ri;

namespace {

constexpr int THREADS = 128;
constexpr int MAX_ACC = 4;          // head_dim <= THREADS * MAX_ACC

template <typename T>
__global__ void __launch_bounds__(THREADS)
attn_generic_kernel(const T* __restrict__ q, int q_ld, const T* __restrict__ kcache,
                    const T* __restrict__ vcache, const int* __restrict__ page_table, int max_pages,
                    const int* __restrict__ token_pos, const int* __restrict__ token_seq,
                    const int* __restrict__ seq_slot, T* __restrict__ out, int out_ld, int n_heads,
                    int n_kv_heads, int hd, int page_size, float scale, int window) {
    extern __shared__ float smem[];
    float* qs = smem;                 // [hd]
    float* ps = smem + hd;            // [THREADS]
    int* key_off = reinterpret_cast<int*>(ps + THREADS);   // [THREADS] element offset of each key row / hd
    __shared__ float scratch[33];

    const int t = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
    const int kvh = h / (n_heads / n_kv_heads);
    const int pos = token_pos[t];
    const int slot = seq_slot[token_seq[t]];
    const int* pages = page_table + (size_t)slot * max_pages;

    for (int d = tid; d < hd; d += THREADS) qs[d] = to_f32<T>(q[(size_t)t * q_ld + h * hd + d]);

    const int first = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    const int n_keys = pos + 1;

    float m = -INFINITY, l = 0.f;
    float acc[MAX_ACC];
#pragma unroll
    for (int a = 0; a < MAX_ACC; ++a) acc[a] = 0.f;

    for (int c0 = first; c0 < n_keys; c0 += THREADS) {
        const int j = c0 + tid;
        float s = -INFINITY;
        __syncthreads();              // qs ready (first pass); ps / key_off free (later passes)
        if (j < n_keys) {
            int page = pages[j / page_size];
            if (!RI_IN_LIMIT(page, RI_LIMIT_PAGES, RI_CHECK_PAGE)) page = 0;      // checked build: recorded, read from a page that exists
            const size_t row = ((size_t)page * n_kv_heads + kvh) * page_size + (j % page_size);
            key_off[tid] = (int)row;  // rows fit in 31 bits: checked on the host
            const T* kr = kcache + row * hd;
            float dot = 0.f;
            for (int d = 0; d < hd; ++d) dot = fmaf(qs[d], to_f32<T>(kr[d]), dot);
            s = dot * scale;
        }
        const float cmax = block_max(s, scratch);
        const float m_new = fmaxf(m, cmax);
        const float p = (j < n_keys) ? expf(s - m_new) : 0.f;
        ps[tid] = p;
        const float csum = block_sum(p, scratch);      // also makes ps / key_off visible
        const float alpha = (m == -INFINITY) ? 0.f : expf(m - m_new);
        l = l * alpha + csum;
        m = m_new;
        const int cn = min(THREADS, n_keys - c0);
#pragma unroll
        for (int a = 0; a < MAX_ACC; ++a) {
            const int d = tid + a * THREADS;
            if (d < hd) {
                float o = acc[a] * alpha;
                for (int jj = 0; jj < cn; ++jj)
                    o = fmaf(ps[jj], to_f32<T>(vcache[(size_t)key_off[jj] * hd + d]), o);
                acc[a] = o;
            }
        }
    }
    const float inv = 1.0f / l;
#pragma unroll
    for (int a = 0; a < MAX_ACC; ++a) {
        const int d = tid + a * THREADS;
        if (d < hd) out[(size_t)t * out_ld + h * hd + d] = from_f32<T>(acc[a] * inv);
    }
}

}  // namespace

RI_API int ri_attention_generic(const void* q, int q_ld, const void* kcache, const void* vcache,
                                const int* page_table, int max_pages, const int* token_pos,
                                const int* token_seq, const int* seq_slot, void* out, int out_ld, int dtype,
                                int n_tokens, int n_heads, int n_kv_heads, int hd, int page_size,
                                long long cache_rows, float scale, int window, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (n_kv_heads <= 0 || n_heads % n_kv_heads)
        return fail("attention: %d heads are not a multiple of %d kv heads", n_heads, n_kv_heads);
    if (hd > THREADS * MAX_ACC) return fail("attention: head_dim %d exceeds %d", hd, THREADS * MAX_ACC);
    if (cache_rows > 0x7fffffffLL) return fail("attention: cache of %lld rows exceeds 2^31", cache_rows);
    if (n_heads > 65535) return fail("attention: %d heads exceed the grid limit", n_heads);
    const size_t smem = (size_t)(hd + 2 * THREADS) * sizeof(float);
    dim3 grid(n_tokens, n_heads);
    if (dtype == RI_F32)
        attn_generic_kernel<float><<<grid, THREADS, smem, stream>>>(
            (const float*)q, q_ld, (const float*)kcache, (const float*)vcache, page_table, max_pages, token_pos,
            token_seq, seq_slot, (float*)out, out_ld, n_heads, n_kv_heads, hd, page_size, scale, window);
    else if (dtype == RI_BF16)
        attn_generic_kernel<__nv_bfloat16><<<grid, THREADS, smem, stream>>>(
            (const __nv_bfloat16*)q, q_ld, (const __nv_bfloat16*)kcache, (const __nv_bfloat16*)vcache, page_table,
            max_pages, token_pos, token_seq, seq_slot, (__nv_bfloat16*)out, out_ld, n_heads, n_kv_heads, hd,
            page_size, scale, window);
    else
        return fail("attention: unknown dtype %d", dtype);
    return check_launch("attention_generic");
}

RI_DEFINE_LAST_ERROR()
