// bf16 attention over the paged cache on the tensor cores, head sizes 64 and 128.
//
// What it computes is attention.rs:95-121: for query head h (kv head h / n_rep),
// scores = dot(q, k) * scale over the keys 0..position of the token's slot, softmax with
// the maximum subtracted (math.rs:104-118), weighted sum of the values; all statistics
// and accumulators in float32, here with an online softmax over pages of 64 keys.
//
// The kernels share the building blocks (XOR-swizzled shared tiles, ldmatrix, mma.sync
// m16n8k16 with float32 accumulation):
//
//  attn_decode   one token per sequence.  A CTA serves one (sequence, kv head, split): the
//                n_rep (<= 16) query heads that share the kv head are the 16 rows of the
//                MMA, so each key and value is read once for all of them.  The keys of the
//                sequence are cut into `n_splits` runs of pages so that a small batch still
//                fills the GPU; inside a CTA the 4 warps take 16 keys of each page each.
//                Every split writes an un-normalised partial result and its (max, sum) to
//                scratch memory; attn_combine merges them by log-sum-exp.  Pages come in by
//                cp.async.
//  attn_decode_tma  the same computation with the pages brought in by TMA through a ring of
//                stages (one elected thread issues the copies, the compute warps never meet
//                at a block-wide barrier in the loop).  With 2 to 8 splits the CTAs of one
//                (sequence, kv head) can form a thread-block cluster: each keeps its partial
//                result in shared memory and sends it to the CTA that merges that slice of
//                the outputs; after a cluster barrier every CTA writes its slice of the final
//                rows: no scratch, no second kernel.  This is what decode steps take.
//  attn_prefill  any number of new tokens per sequence (whole prompts, or a continuation).
//                A CTA serves 64 consecutive query tokens of one head; the warps take 16
//                query rows each and walk the key pages up to the causal limit: the token
//                at position p sees keys 0..p (window > 0: p-window+1..p).
//
// Keys and values are only ever read from the cache: the step's new tokens were written
// there (after rotation) before attention runs, so prefill, continuation and decode use
// one convention.
#include "tcgen05_common.cuh"
#include "attention_decode_static.h"

#include <cooperative_groups.h>

using namespace ri;

namespace {

constexpr int PAGE = 64;            // keys per cache page (fixed by the tile shapes below)
constexpr int THREADS = 128;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// A [rows][HD] bf16 tile in shared memory; the 16-byte chunk c of row r lives at chunk
// (c & ~7) | ((c ^ r) & 7), so that the 8 rows an ldmatrix reads hit 8 different bank groups.
template <int HD>
__device__ __forceinline__ uint32_t tile_off(int r, int c) {
    return (uint32_t)(r * (HD * 2) + (((c & ~7) | ((c ^ r) & 7)) << 4));
}

// Copy `rows` rows of HD bf16 (consecutive in global memory) into a swizzled tile; all threads call.
template <int HD>
__device__ __forceinline__ void load_tile_async(uint32_t tile, const __nv_bfloat16* src, int rows) {
    constexpr int CPR = HD / 8;                       // 16-byte chunks per row
    for (int idx = threadIdx.x; idx < rows * CPR; idx += THREADS) {
        const int r = idx / CPR, c = idx % CPR;
        cp_async16(tile + tile_off<HD>(r, c), src + (size_t)r * HD + c * 8);
    }
}

// S[16 x 16 keys] (+)= Q[16 x HD] * K[keys kbase .. kbase+15]^T for one warp; q: A fragments of all k-steps.
template <int HD>
__device__ __forceinline__ void qk_16keys(const uint32_t (*q)[4], uint32_t ktile, int kbase, float (*s)[4]) {
    const int lane = threadIdx.x & 31;
    const int mi = lane >> 3, rr = lane & 7;
    // The k-steps go round four accumulators, so that an MMA waits for the one four steps before it and not
    // for its neighbour: a decode step's CTAs have a page or two each and nothing else to fill the pipe with.
    constexpr int CH = (HD / 16) < 4 ? (HD / 16) : 4;
    float part[CH][2][4];
#pragma unroll
    for (int c = 0; c < CH; ++c)
#pragma unroll
        for (int e = 0; e < 4; ++e) part[c][0][e] = part[c][1][e] = 0.f;
#pragma unroll
    for (int ks = 0; ks < HD / 16; ++ks) {
        // matrices: (keys 0-7, k 0-7), (keys 0-7, k 8-15), (keys 8-15, k 0-7), (keys 8-15, k 8-15)
        const int row = kbase + (mi >> 1) * 8 + rr;
        const int chunk = ks * 2 + (mi & 1);
        uint32_t b0, b1, b2, b3;
        ldmatrix_x4(ktile + tile_off<HD>(row, chunk), b0, b1, b2, b3);
        mma_bf16(part[ks % CH][0], q[ks], b0, b1);
        mma_bf16(part[ks % CH][1], q[ks], b2, b3);
    }
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        float a0 = 0.f, a1 = 0.f;
#pragma unroll
        for (int c = 0; c < CH; ++c) {
            a0 += part[c][0][e];
            a1 += part[c][1][e];
        }
        s[0][e] += a0;
        s[1][e] += a1;
    }
}

// O[16 x HD] += P[16 x 16 keys] * V[keys kbase .. kbase+15]; p: one A fragment.
template <int HD>
__device__ __forceinline__ void pv_16keys(const uint32_t* p, uint32_t vtile, int kbase, float (*o)[4]) {
    const int lane = threadIdx.x & 31;
    const int mi = lane >> 3, rr = lane & 7;
#pragma unroll
    for (int dp = 0; dp < HD / 16; ++dp) {
        // transposed loads: (keys 0-7, d 0-7), (keys 8-15, d 0-7), (keys 0-7, d 8-15), (keys 8-15, d 8-15)
        const int row = kbase + (mi & 1) * 8 + rr;
        const int chunk = dp * 2 + (mi >> 1);
        uint32_t b0, b1, b2, b3;
        ldmatrix_x4_trans(vtile + tile_off<HD>(row, chunk), b0, b1, b2, b3);
        mma_bf16(o[2 * dp], p, b0, b1);
        mma_bf16(o[2 * dp + 1], p, b2, b3);
    }
}

// Online-softmax update of one warp's 16 rows with a fresh S[16 x (NT*8)] tile (already scaled and
// masked with -inf).  Rows g and g+8 of the thread; statistics are shared by the 4 threads of a quad.
template <int NT, int ONT>
__device__ __forceinline__ void softmax_update(float (*s)[4], float* m, float* l, float (*o)[4]) {
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        float mx = -INFINITY;
#pragma unroll
        for (int t = 0; t < NT; ++t) mx = fmaxf(mx, fmaxf(s[t][2 * half], s[t][2 * half + 1]));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        const float m_new = fmaxf(m[half], mx);
        const float base = (m_new == -INFINITY) ? 0.f : m_new;      // nothing visible yet: exp(-inf - 0) = 0
        const float alpha = expf(m[half] - base);                    // m = -inf gives 0
        float sum = 0.f;
#pragma unroll
        for (int t = 0; t < NT; ++t) {
            const float p0 = expf(s[t][2 * half] - base), p1 = expf(s[t][2 * half + 1] - base);
            s[t][2 * half] = p0;
            s[t][2 * half + 1] = p1;
            sum += p0 + p1;
        }
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
        sum += __shfl_xor_sync(0xffffffffu, sum, 2);
        l[half] = l[half] * alpha + sum;
        m[half] = m_new;
#pragma unroll
        for (int t = 0; t < ONT; ++t) {
            o[t][2 * half] *= alpha;
            o[t][2 * half + 1] *= alpha;
        }
    }
}

constexpr int MAX_CLUSTER_SPLITS = 8;                          // the portable cluster size

// The merge of a CTA's four warps, each of which saw a quarter of the keys: `so` holds their unnormalised
// outputs [4][16][HD + 4], `sml` their running maximum and sum per row [4][16][2].  Returns outputs d .. d+3 of
// row r scaled to the row's maximum M over the warps, and M and the row's sum L.  Every thread works the
// statistics of its row out itself (four loads and exponentials that overlap) instead of waiting at a barrier
// for one thread per row.
template <int HD>
__device__ __forceinline__ float4 merge_warps(const float* so, const float* sml, int r, int d, float& M, float& L) {
    constexpr int SO_LD = HD + 4;
    float2 ml[4];
#pragma unroll
    for (int w = 0; w < 4; ++w) ml[w] = *reinterpret_cast<const float2*>(sml + ((w * 16 + r) << 1));
    M = fmaxf(fmaxf(ml[0].x, ml[1].x), fmaxf(ml[2].x, ml[3].x));
    L = 0.f;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int w = 0; w < 4; ++w) {
        const float f = (M == -INFINITY) ? 0.f : expf(ml[w].x - M);
        const float4 x = *reinterpret_cast<const float4*>(so + (w * 16 + r) * SO_LD + d);
        L += f * ml[w].y;
        acc.x += f * x.x;
        acc.y += f * x.y;
        acc.z += f * x.z;
        acc.w += f * x.w;
    }
    return acc;
}

// four consecutive outputs as bfloat16: one 8-byte store where the row allows it
__device__ __forceinline__ void store_bf16x4(__nv_bfloat16* p, float a, float b, float c, float d, bool wide) {
    const __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
    if (wide) {
        uint2 v;
        v.x = *reinterpret_cast<const uint32_t*>(&lo);
        v.y = *reinterpret_cast<const uint32_t*>(&hi);
        *reinterpret_cast<uint2*>(p) = v;
    } else {                                              // rows that are only 4-byte aligned
        *reinterpret_cast<__nv_bfloat162*>(p) = lo;
        *reinterpret_cast<__nv_bfloat162*>(p + 2) = hi;
    }
}

// floats of shared memory a CTA keeps for what its cluster sends it (see cluster_merge)
template <int HD>
constexpr int CLUSTER_RECV_FLOATS = 16 * HD + 4 * MAX_CLUSTER_SPLITS + MAX_CLUSTER_SPLITS * 16 * 2;

// The splits of a (sequence, kv head) as the CTAs of one thread-block cluster (its z extent): what every CTA
// does once its four warps' partial results lie in `so` / `sml`.  Every CTA merges its warps and sends the
// result to the CTA that merges that part of the output over the splits (runs of `chunk` outputs, a
// multiple of 4, so that everything moves as float4): plain stores into the peers' shared memory, nothing is
// read remotely.  `recv` is this CTA's area for what the peers send ([n_splits][chunk] outputs, then
// [n_splits][16][2] statistics: CLUSTER_RECV_FLOATS<HD> floats, at the same place in every CTA and outside
// anything a CTA still works on).  All NT threads of the CTA call; the CTA has arrived at the cluster's
// barrier once, near its start.  `ok` false: the CTA gave up on its pages; it sends and stores nothing but
// still meets its cluster at the barriers.
template <int HD, int NT>
__device__ __forceinline__ void cluster_merge(const float* so, const float* sml, float* recv, int n_rep, int n_splits,
                                              int split, int token, int kvh, __nv_bfloat16* __restrict__ out,
                                              int out_ld, bool ok) {
    namespace cg = cooperative_groups;
    cg::cluster_group cluster = cg::this_cluster();
    const int total = n_rep * HD;
    const int chunk = (((total + n_splits - 1) / n_splits) + 3) & ~3;
    float* recv_o = recv;                                                   // [n_splits][chunk]
    float* recv_ml = recv + 16 * HD + 4 * MAX_CLUSTER_SPLITS;               // [n_splits][16][2]
    // every CTA of the cluster has arrived at the barrier near its start by now: all of them exist, so
    // their shared memory may be written
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
    if (ok)
        for (int it = threadIdx.x; it < n_rep * (HD / 4); it += NT) {
            const int r = it / (HD / 4), d = (it % (HD / 4)) * 4;
            float M, L;
            const float4 acc = merge_warps<HD>(so, sml, r, d, M, L);
            const int idx = r * HD + d, owner = idx / chunk;
            *reinterpret_cast<float4*>(cluster.map_shared_rank(recv_o, owner) + split * chunk + (idx - owner * chunk)) = acc;
            // the row's statistics go with the first piece of the row that a CTA merges: to the CTAs that need them
            if (d == 0 || idx == owner * chunk)
                *reinterpret_cast<float2*>(cluster.map_shared_rank(recv_ml, owner) + (split * 16 + r) * 2) = make_float2(M, L);
        }
    RI_PHASE(3);
    cluster.sync();                                       // everything sent has arrived
    RI_PHASE(4);
    const int lo = split * chunk, hi = min(total, lo + chunk);
    const bool wide = ((reinterpret_cast<uintptr_t>(out) & 7) == 0) && ((out_ld & 3) == 0);
    if (ok)
        for (int idx = lo + 4 * (int)threadIdx.x; idx < hi; idx += 4 * NT) {
            const int r = idx / HD, d = idx % HD;
            float2 ml[MAX_CLUSTER_SPLITS];
            float M = -INFINITY;
#pragma unroll
            for (int sp = 0; sp < MAX_CLUSTER_SPLITS; ++sp)
                if (sp < n_splits) {
                    ml[sp] = *reinterpret_cast<const float2*>(recv_ml + (sp * 16 + r) * 2);
                    M = fmaxf(M, ml[sp].x);
                }
            float L = 0.f;
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int sp = 0; sp < MAX_CLUSTER_SPLITS; ++sp)
                if (sp < n_splits) {
                    const float f = (ml[sp].x == -INFINITY) ? 0.f : expf(ml[sp].x - M);
                    const float4 x = *reinterpret_cast<const float4*>(recv_o + sp * chunk + (idx - lo));
                    L += f * ml[sp].y;
                    acc.x += f * x.x;
                    acc.y += f * x.y;
                    acc.z += f * x.z;
                    acc.w += f * x.w;
                }
            const float inv = 1.0f / L;
            store_bf16x4(out + (size_t)token * out_ld + (size_t)(kvh * n_rep + r) * HD + d, acc.x * inv, acc.y * inv,
                         acc.z * inv, acc.w * inv, wide);
        }
    RI_PHASE_LATEST(5);
    // nobody reads or writes a peer's shared memory after that barrier: a CTA may leave when it is done
}

// What a CTA that merged its warps does with row r, outputs d .. d+3, when it is not part of a cluster: the
// final result if it saw the whole sequence, else its partial result for the kernel that merges the splits.
template <int HD>
__device__ __forceinline__ void write_merged(const float* so, const float* sml, int r, int d, int b, int h, int token,
                                             int n_heads, int n_splits, int split, float* __restrict__ part_o,
                                             float* __restrict__ part_ml, __nv_bfloat16* __restrict__ out, int out_ld) {
    float M, L;
    const float4 acc = merge_warps<HD>(so, sml, r, d, M, L);
    if (n_splits == 1) {
        const bool wide = ((reinterpret_cast<uintptr_t>(out) & 7) == 0) && ((out_ld & 3) == 0);
        store_bf16x4(out + (size_t)token * out_ld + (size_t)h * HD + d, acc.x / L, acc.y / L, acc.z / L, acc.w / L, wide);
    } else {
        const size_t row = ((size_t)b * n_heads + h) * n_splits + split;
        float* po = part_o + row * HD + d;
        if ((reinterpret_cast<uintptr_t>(part_o) & 15) == 0) {
            *reinterpret_cast<float4*>(po) = acc;
        } else {
            po[0] = acc.x;
            po[1] = acc.y;
            po[2] = acc.z;
            po[3] = acc.w;
        }
        if (d == 0) {
            part_ml[row * 2] = M;
            part_ml[row * 2 + 1] = L;
        }
    }
}

// ---------------------------------------------------------------------------------------------
// decode: one token per sequence, split over runs of pages
// ---------------------------------------------------------------------------------------------
constexpr int NBUF = 3;             // page buffers of the cp.async decode kernel: with three, a run of three pages is in
                                    // flight before the kernel has even waited for its predecessor

template <int HD>
__global__ void __launch_bounds__(THREADS)
attn_decode_kernel(const __nv_bfloat16* __restrict__ q, int q_ld, const __nv_bfloat16* __restrict__ kcache,
                   const __nv_bfloat16* __restrict__ vcache, const int* __restrict__ page_table, int max_pages,
                   const int* __restrict__ seq_slot, const int* __restrict__ seq_len,
                   const int* __restrict__ cu_seqlens, int n_heads, int n_kv_heads, float scale, int window,
                   int n_splits, float* __restrict__ part_o, float* __restrict__ part_ml,
                   __nv_bfloat16* __restrict__ out, int out_ld) {
    constexpr int TILE = PAGE * HD * 2;                 // bytes of one K or V page tile
    extern __shared__ __align__(128) uint8_t smem[];
    // [NBUF buffers][K tile, V tile], then the Q tile [16][HD]
    const uint32_t kv_base = smem_u32(smem);
    const uint32_t q_tile = kv_base + 2 * NBUF * TILE;

    const int b = blockIdx.x, kvh = blockIdx.y, split = blockIdx.z;
    let_next_kernel_start();
    // What the step fixed before its first kernel (lengths, slots, the page table) and the pages that
    // hold only older positions are written by no kernel of this step: they are read, and the first
    // page's copy is started, while the kernel before this one still runs.
    const int n_rep = n_heads / n_kv_heads;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, tq = lane & 3;
    const int n_keys = seq_len[b];                       // counts the new token, whose key is in the cache by then
    const int token = cu_seqlens[b];
    const int first_key = (window > 0 && n_keys - window > 0) ? n_keys - window : 0;
    const int* pages = page_table + (size_t)seq_slot[b] * max_pages;

    const int pg_lo = first_key / PAGE, pg_hi = (n_keys + PAGE - 1) / PAGE;    // pages [pg_lo, pg_hi)
    const int per = (pg_hi - pg_lo + n_splits - 1) / n_splits;
    const int pg_begin = pg_lo + split * per, pg_end = min(pg_hi, pg_begin + per);

    auto issue = [&](int pg, int buf) {
        int page = pages[pg];
        if (!RI_BLOCK_IN_LIMIT(page, RI_LIMIT_PAGES, RI_CHECK_PAGE)) page = 0;    // checked build: recorded, read from a page that exists
        const size_t base = ((size_t)page * n_kv_heads + kvh) * PAGE * HD;
        load_tile_async<HD>(kv_base + (2 * buf) * TILE, kcache + base, PAGE);
        load_tile_async<HD>(kv_base + (2 * buf + 1) * TILE, vcache + base, PAGE);
        cp_async_commit();
    };
    // up to NBUF pages are on their way before the wait; the page of the new token (the sequence's last) is
    // still being written by the kernel before and has to stay behind it
    const int n_pages = max(0, pg_end - pg_begin);
    int issued = 0;
    while (issued < n_pages && issued < NBUF && pg_begin + issued != pg_hi - 1) {
        issue(pg_begin + issued, issued);
        ++issued;
    }
    wait_for_previous_kernels();          // q and the newest key and value come from the kernel before
    // Q rows: head kvh*n_rep + r for r < n_rep, zero above
    for (int idx = threadIdx.x; idx < 16 * (HD / 8); idx += THREADS) {
        const int r = idx / (HD / 8), c = idx % (HD / 8);
        uint4 v = make_uint4(0, 0, 0, 0);
        if (r < n_rep) v = *reinterpret_cast<const uint4*>(q + (size_t)token * q_ld + (size_t)(kvh * n_rep + r) * HD + c * 8);
        *reinterpret_cast<uint4*>(smem + 2 * NBUF * TILE + tile_off<HD>(r, c)) = v;
    }
    __syncthreads();                                      // Q tile written

    uint32_t qf[HD / 16][4];
    {
        const int row = lane & 15, half = lane >> 4;
#pragma unroll
        for (int ks = 0; ks < HD / 16; ++ks)
            ldmatrix_x4(q_tile + tile_off<HD>(row, ks * 2 + half), qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3]);
    }

    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
    float o[HD / 8][4];
#pragma unroll
    for (int t = 0; t < HD / 8; ++t) o[t][0] = o[t][1] = o[t][2] = o[t][3] = 0.f;

    for (int pg = pg_begin; pg < pg_end; ++pg) {
        const int i = pg - pg_begin, buf = i % NBUF;
        // page j goes to buffer j % NBUF, which the barrier at the end of page j - NBUF has set free
        while (issued < n_pages && issued <= i + NBUF - 1) {
            issue(pg_begin + issued, issued % NBUF);
            ++issued;
        }
        // the copies complete in the order they were issued: all but the ones behind this page's
        const int behind = issued - i - 1;
        if (behind >= 2) cp_async_wait<2>(); else if (behind == 1) cp_async_wait<1>(); else cp_async_wait<0>();
        __syncthreads();                                  // this page's tiles have landed for everyone
        const uint32_t ktile = kv_base + (2 * buf) * TILE, vtile = ktile + TILE;
        const int kbase = warp * 16;                      // this warp's 16 keys of the page
        const int key0 = pg * PAGE + kbase;
        if (key0 < n_keys && key0 + 16 > first_key) {
            float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
            qk_16keys<HD>(qf, ktile, kbase, s);
#pragma unroll
            for (int t = 0; t < 2; ++t)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int key = key0 + t * 8 + 2 * tq + (e & 1);
                    s[t][e] = (key < n_keys && key >= first_key) ? s[t][e] * scale : -INFINITY;
                }
            softmax_update<2, HD / 8>(s, m, l, o);
            uint32_t pf[4] = {pack_bf16(s[0][0], s[0][1]), pack_bf16(s[0][2], s[0][3]),
                              pack_bf16(s[1][0], s[1][1]), pack_bf16(s[1][2], s[1][3])};
            pv_16keys<HD>(pf, vtile, kbase, o);
        }
        __syncthreads();                                  // everyone is done with this buffer
    }

    // ---- merge the 4 warps (each saw a quarter of the keys) through shared memory ----
    constexpr int SO_LD = HD + 4;                         // padded rows: the 8 rows a warp stores at once hit 8 bank groups
    float* so = reinterpret_cast<float*>(smem);           // [4][16][SO_LD]
    float* sml = so + 4 * 16 * SO_LD;                     // [4][16][2]
#pragma unroll
    for (int t = 0; t < HD / 8; ++t) {
        const int d = t * 8 + 2 * tq;
        *reinterpret_cast<float2*>(so + (warp * 16 + g) * SO_LD + d) = make_float2(o[t][0], o[t][1]);
        *reinterpret_cast<float2*>(so + (warp * 16 + g + 8) * SO_LD + d) = make_float2(o[t][2], o[t][3]);
    }
    if (tq == 0) {
        sml[((warp * 16 + g) << 1)] = m[0];
        sml[((warp * 16 + g) << 1) + 1] = l[0];
        sml[((warp * 16 + g + 8) << 1)] = m[1];
        sml[((warp * 16 + g + 8) << 1) + 1] = l[1];
    }
    __syncthreads();                                      // every warp's partial result is in shared memory
    for (int it = threadIdx.x; it < n_rep * (HD / 4); it += THREADS) {
        const int r = it / (HD / 4), d = (it % (HD / 4)) * 4;
        write_merged<HD>(so, sml, r, d, b, kvh * n_rep + r, token, n_heads, n_splits, split, part_o, part_ml, out, out_ld);
    }
}

// ---------------------------------------------------------------------------------------------
// decode, fed by TMA: the same computation, with the K and V pages brought in by tensor-map copies
// (128-byte swizzle, one elected thread) through a ring of RING stages guarded by mbarriers, so
// that several pages are in flight per CTA and the compute warps never meet at a block-wide
// barrier.  A page tile is [head_dim / 64][64 keys][128 bytes]; inside a 128-byte row the 16-byte
// chunk c sits at c ^ (row & 7), which is what the TMA swizzle writes and what ldmatrix wants.
// ---------------------------------------------------------------------------------------------
constexpr int RING = 3;
constexpr int DECODE_TMA_THREADS = 160;              // 4 compute warps + 1 producer warp

template <int HD>
__device__ __forceinline__ uint32_t atom_off(int r, int c) {      // c: 16-byte chunk index along head_dim
    return (uint32_t)((c >> 3) * (PAGE * 128) + r * 128 + (((c & 7) ^ (r & 7)) << 4));
}

template <int HD>
__device__ __forceinline__ void qk_16keys_atoms(const uint32_t (*q)[4], uint32_t ktile, int kbase, float (*s)[4]) {
    const int lane = threadIdx.x & 31;
    const int mi = lane >> 3, rr = lane & 7;
#pragma unroll
    for (int ks = 0; ks < HD / 16; ++ks) {
        const int row = kbase + (mi >> 1) * 8 + rr;
        const int chunk = ks * 2 + (mi & 1);
        uint32_t b0, b1, b2, b3;
        ldmatrix_x4(ktile + atom_off<HD>(row, chunk), b0, b1, b2, b3);
        mma_bf16(s[0], q[ks], b0, b1);
        mma_bf16(s[1], q[ks], b2, b3);
    }
}

template <int HD>
__device__ __forceinline__ void pv_16keys_atoms(const uint32_t* p, uint32_t vtile, int kbase, float (*o)[4]) {
    const int lane = threadIdx.x & 31;
    const int mi = lane >> 3, rr = lane & 7;
#pragma unroll
    for (int dp = 0; dp < HD / 16; ++dp) {
        const int row = kbase + (mi & 1) * 8 + rr;
        const int chunk = dp * 2 + (mi >> 1);
        uint32_t b0, b1, b2, b3;
        ldmatrix_x4_trans(vtile + atom_off<HD>(row, chunk), b0, b1, b2, b3);
        mma_bf16(o[2 * dp], p, b0, b1);
        mma_bf16(o[2 * dp + 1], p, b2, b3);
    }
}

template <int HD, bool CLUSTER>
__global__ void __launch_bounds__(DECODE_TMA_THREADS)
attn_decode_tma_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                       const __nv_bfloat16* __restrict__ q, int q_ld, const int* __restrict__ page_table,
                       int max_pages, const int* __restrict__ seq_slot, const int* __restrict__ seq_len,
                       const int* __restrict__ cu_seqlens, int n_heads, int n_kv_heads, float scale, int window,
                       int n_splits, float* __restrict__ part_o, float* __restrict__ part_ml,
                       __nv_bfloat16* __restrict__ out, int out_ld, int* status) {
    constexpr int TILE = PAGE * HD * 2;                 // bytes of one K or V page tile
    constexpr int ATOMS = HD / 64;
    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t full_bar[RING], empty_bar[RING];
    __shared__ volatile int abort_flag;
    uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);      // swizzled tiles: 1024-byte aligned
    const uint32_t kv_base = smem_u32(smem);            // [RING][K tile, V tile], then the Q tile [16][HD]
    const uint32_t q_tile = kv_base + 2 * RING * TILE;

    const int b = blockIdx.x, kvh = blockIdx.y, split = blockIdx.z;
    const int n_rep = n_heads / n_kv_heads;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, tq = lane & 3;
    if (threadIdx.x == 0) {
        for (int i = 0; i < RING; ++i) {
            tc::mbar_init(smem_u32(&full_bar[i]), 1);
            tc::mbar_init(smem_u32(&empty_bar[i]), 4);          // one arrival per compute warp
        }
        abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    let_next_kernel_start();
    if (CLUSTER) asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");   // "this CTA runs": waited for before the merge
    // Lengths, slots and the page table were fixed before the step's first kernel, and pages that hold
    // only older positions are written by no kernel of this step: the producer starts on them while
    // the kernel before this one still runs.  q and the sequence's last page wait for it.
    const int n_keys = seq_len[b];
    const int token = cu_seqlens[b];
    const int first_key = (window > 0 && n_keys - window > 0) ? n_keys - window : 0;
    const int pg_lo = first_key / PAGE, pg_hi = (n_keys + PAGE - 1) / PAGE;
    const int per = (pg_hi - pg_lo + n_splits - 1) / n_splits;
    const int pg_begin = pg_lo + split * per, pg_end = min(pg_hi, pg_begin + per);

    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
    float o[HD / 8][4];
#pragma unroll
    for (int t = 0; t < HD / 8; ++t) o[t][0] = o[t][1] = o[t][2] = o[t][3] = 0.f;

    if (warp == 4) {
        // ---------------- producer ----------------
        if (lane == 0) {
            const int* pages = page_table + (size_t)seq_slot[b] * max_pages;
            int issued = 0;
            int page_next = pg_begin < pg_end ? pages[pg_begin] : 0;   // a page's number is fetched one turn ahead
            for (int pg = pg_begin; pg < pg_end; ++pg) {
                const int j = pg - pg_begin, s = j % RING;
                const int page_now = page_next;
                if (pg + 1 < pg_end) page_next = pages[pg + 1];
                if (pg == pg_hi - 1) wait_for_previous_kernels();      // the page the new key and value went to
                if (!tc::mbar_wait(smem_u32(&empty_bar[s]), (uint32_t)((j / RING) & 1) ^ 1u) || abort_flag) {
                    tc::report(status, 21);
                    abort_flag = 1;
                    break;
                }
                const int row = (page_now * n_kv_heads + kvh) * PAGE;
                const uint32_t bar = smem_u32(&full_bar[s]);
                tc::mbar_expect_tx(bar, 2 * TILE);
#pragma unroll
                for (int a = 0; a < ATOMS; ++a) {
                    tc::tma_load_2d(kv_base + (2 * s) * TILE + a * PAGE * 128, &map_k, bar, a * 64, row);
                    tc::tma_load_2d(kv_base + (2 * s + 1) * TILE + a * PAGE * 128, &map_v, bar, a * 64, row);
                }
                issued = j + 1;
            }
            // do not leave while a copy into this CTA's shared memory may be in flight
            for (int j = max(0, issued - RING); j < issued; ++j)
                if (!tc::mbar_wait(smem_u32(&full_bar[j % RING]), (uint32_t)((j / RING) & 1))) { tc::report(status, 24); break; }
        }
    } else {
        // ---------------- compute: warp w takes keys 16w .. 16w+15 of every page ----------------
        wait_for_previous_kernels();          // q comes from the kernel before
        for (int idx = threadIdx.x; idx < 16 * (HD / 8); idx += 128) {
            const int r = idx / (HD / 8), c = idx % (HD / 8);
            uint4 v = make_uint4(0, 0, 0, 0);
            if (r < n_rep) v = *reinterpret_cast<const uint4*>(q + (size_t)token * q_ld + (size_t)(kvh * n_rep + r) * HD + c * 8);
            *reinterpret_cast<uint4*>(smem + 2 * RING * TILE + tile_off<HD>(r, c)) = v;
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");          // the four compute warps: Q tile written
        RI_PHASE(0);
        uint32_t qf[HD / 16][4];
        {
            const int row = lane & 15, half = lane >> 4;
#pragma unroll
            for (int ks = 0; ks < HD / 16; ++ks)
                ldmatrix_x4(q_tile + tile_off<HD>(row, ks * 2 + half), qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3]);
        }
        for (int pg = pg_begin; pg < pg_end; ++pg) {
            const int j = pg - pg_begin, s = j % RING;
            if (!tc::mbar_wait(smem_u32(&full_bar[s]), (uint32_t)((j / RING) & 1)) || abort_flag) {
                if (lane == 0) { tc::report(status, 22); abort_flag = 1; }
                break;
            }
            const uint32_t ktile = kv_base + (2 * s) * TILE, vtile = ktile + TILE;
            const int kbase = warp * 16;
            const int key0 = pg * PAGE + kbase;
            if (key0 < n_keys && key0 + 16 > first_key) {
                float sc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
                qk_16keys_atoms<HD>(qf, ktile, kbase, sc);
#pragma unroll
                for (int t = 0; t < 2; ++t)
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int key = key0 + t * 8 + 2 * tq + (e & 1);
                        sc[t][e] = (key < n_keys && key >= first_key) ? sc[t][e] * scale : -INFINITY;
                    }
                softmax_update<2, HD / 8>(sc, m, l, o);
                uint32_t pf[4] = {pack_bf16(sc[0][0], sc[0][1]), pack_bf16(sc[0][2], sc[0][3]),
                                  pack_bf16(sc[1][0], sc[1][1]), pack_bf16(sc[1][2], sc[1][3])};
                pv_16keys_atoms<HD>(pf, vtile, kbase, o);
            }
            __syncwarp();
            if (lane == 0) tc::mbar_arrive(smem_u32(&empty_bar[s]));       // this warp is done with the stage
        }
    }
    RI_PHASE(1);
    __syncthreads();                      // every page consumed, every copy landed: the ring is free
    RI_PHASE_LATEST(2);

    // ---- merge the 4 compute warps (each saw a quarter of the keys) through shared memory ----
    constexpr int SO_LD = HD + 4;                         // padded rows: the 8 rows a warp stores at once hit 8 bank groups
    float* so = reinterpret_cast<float*>(smem);           // [4][16][SO_LD]
    float* sml = so + 4 * 16 * SO_LD;                     // [4][16][2]
    if (warp < 4) {
#pragma unroll
        for (int t = 0; t < HD / 8; ++t) {
            const int d = t * 8 + 2 * tq;
            *reinterpret_cast<float2*>(so + (warp * 16 + g) * SO_LD + d) = make_float2(o[t][0], o[t][1]);
            *reinterpret_cast<float2*>(so + (warp * 16 + g + 8) * SO_LD + d) = make_float2(o[t][2], o[t][3]);
        }
        if (tq == 0) {
            sml[((warp * 16 + g) << 1)] = m[0];
            sml[((warp * 16 + g) << 1) + 1] = l[0];
            sml[((warp * 16 + g + 8) << 1)] = m[1];
            sml[((warp * 16 + g + 8) << 1) + 1] = l[1];
        }
    }
    __syncthreads();
    if constexpr (CLUSTER) {
        // the splits of this (sequence, kv head) are the CTAs of one cluster: merged here, no scratch, no second kernel
        float* recv = reinterpret_cast<float*>(smem + 2 * RING * TILE + 16 * HD * 2);
        cluster_merge<HD, DECODE_TMA_THREADS>(so, sml, recv, n_rep, n_splits, split, token, kvh, out, out_ld, !abort_flag);
        return;
    }
    if (abort_flag) return;
    for (int it = threadIdx.x; it < n_rep * (HD / 4); it += DECODE_TMA_THREADS) {
        const int r = it / (HD / 4), d = (it % (HD / 4)) * 4;
        write_merged<HD>(so, sml, r, d, b, kvh * n_rep + r, token, n_heads, n_splits, split, part_o, part_ml, out, out_ld);
    }
}

// out[b, h, :] = sum_s exp(M_s - M) O_s / sum_s exp(M_s - M) L_s over the splits
__global__ void attn_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                    const int* __restrict__ cu_seqlens, int n_heads, int hd, int n_splits,
                                    __nv_bfloat16* __restrict__ out, int out_ld) {
    const int b = blockIdx.x, h = blockIdx.y;
    let_next_kernel_start();
    wait_for_previous_kernels();
    const size_t row0 = ((size_t)b * n_heads + h) * n_splits;
    float M = -INFINITY;
    for (int s = 0; s < n_splits; ++s) M = fmaxf(M, part_ml[(row0 + s) * 2]);
    float L = 0.f;
    for (int s = 0; s < n_splits; ++s) {
        const float ms = part_ml[(row0 + s) * 2];
        if (ms != -INFINITY) L += expf(ms - M) * part_ml[(row0 + s) * 2 + 1];
    }
    const float inv = 1.0f / L;
    const int token = cu_seqlens[b];
    for (int d = threadIdx.x; d < hd; d += blockDim.x) {
        float acc = 0.f;
        for (int s = 0; s < n_splits; ++s) {
            const float ms = part_ml[(row0 + s) * 2];
            if (ms != -INFINITY) acc += expf(ms - M) * part_o[(row0 + s) * hd + d];
        }
        out[(size_t)token * out_ld + (size_t)h * hd + d] = __float2bfloat16_rn(acc * inv);
    }
}

// ---------------------------------------------------------------------------------------------
// prefill / continuation: 64 query tokens of one head per CTA
// ---------------------------------------------------------------------------------------------
template <int HD>
__global__ void __launch_bounds__(THREADS)
attn_prefill_kernel(const __nv_bfloat16* __restrict__ q, int q_ld, const __nv_bfloat16* __restrict__ kcache,
                    const __nv_bfloat16* __restrict__ vcache, const int* __restrict__ page_table, int max_pages,
                    const int* __restrict__ seq_slot, const int* __restrict__ seq_start,
                    const int* __restrict__ cu_seqlens, int n_heads, int n_kv_heads, float scale, int window,
                    __nv_bfloat16* __restrict__ out, int out_ld) {
    constexpr int TILE = PAGE * HD * 2;
    extern __shared__ __align__(128) uint8_t smem[];
    const uint32_t kv_base = smem_u32(smem);
    const uint32_t q_tile = kv_base + 4 * TILE;           // [64][HD]

    const int b = blockIdx.z, h = blockIdx.y;
    let_next_kernel_start();
    wait_for_previous_kernels();
    const int tok0 = cu_seqlens[b], n_new = cu_seqlens[b + 1] - tok0;
    const int q0 = blockIdx.x * 64;                       // first query (among the new tokens) of this CTA
    if (q0 >= n_new) return;
    const int kvh = h / (n_heads / n_kv_heads);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, tq = lane & 3;
    const int start = seq_start[b];                       // positions cached before this step
    const int* pages = page_table + (size_t)seq_slot[b] * max_pages;
    const int rows = min(64, n_new - q0);

    // positions of the CTA's first and last query
    const int pos_lo = start + q0, pos_hi = start + q0 + rows - 1;
    const int first_key = (window > 0 && pos_lo - window + 1 > 0) ? pos_lo - window + 1 : 0;
    const int pg_begin = first_key / PAGE, pg_end = pos_hi / PAGE + 1;

    for (int idx = threadIdx.x; idx < 64 * (HD / 8); idx += THREADS) {
        const int r = idx / (HD / 8), c = idx % (HD / 8);
        uint4 v = make_uint4(0, 0, 0, 0);
        if (r < rows) v = *reinterpret_cast<const uint4*>(q + (size_t)(tok0 + q0 + r) * q_ld + (size_t)h * HD + c * 8);
        *reinterpret_cast<uint4*>(smem + 4 * TILE + tile_off<HD>(r, c)) = v;
    }
    auto issue = [&](int pg, int buf) {
        int page = pages[pg];
        if (!RI_BLOCK_IN_LIMIT(page, RI_LIMIT_PAGES, RI_CHECK_PAGE)) page = 0;    // checked build: recorded, read from a page that exists
        const size_t base = ((size_t)page * n_kv_heads + kvh) * PAGE * HD;
        load_tile_async<HD>(kv_base + (2 * buf) * TILE, kcache + base, PAGE);
        load_tile_async<HD>(kv_base + (2 * buf + 1) * TILE, vcache + base, PAGE);
        cp_async_commit();
    };
    issue(pg_begin, 0);
    __syncthreads();

    uint32_t qf[HD / 16][4];
    {
        const int row = warp * 16 + (lane & 15), half = lane >> 4;
#pragma unroll
        for (int ks = 0; ks < HD / 16; ++ks)
            ldmatrix_x4(q_tile + tile_off<HD>(row, ks * 2 + half), qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3]);
    }
    // this thread's two query rows and their positions
    const int r0 = warp * 16 + g, r1 = r0 + 8;
    const int p0 = start + q0 + r0, p1 = start + q0 + r1;
    const int warp_pos_lo = start + q0 + warp * 16, warp_pos_hi = warp_pos_lo + 15;

    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
    float o[HD / 8][4];
#pragma unroll
    for (int t = 0; t < HD / 8; ++t) o[t][0] = o[t][1] = o[t][2] = o[t][3] = 0.f;

    for (int pg = pg_begin; pg < pg_end; ++pg) {
        const int buf = (pg - pg_begin) & 1;
        if (pg + 1 < pg_end) {
            issue(pg + 1, buf ^ 1);
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        const uint32_t ktile = kv_base + (2 * buf) * TILE, vtile = ktile + TILE;
        const int key_lo = pg * PAGE;
        // the warp skips pages none of its rows can see
        const bool any = key_lo <= warp_pos_hi && (window <= 0 || key_lo + PAGE - 1 > warp_pos_lo - window);
        if (any) {
            const bool full = key_lo + PAGE - 1 <= warp_pos_lo && (window <= 0 || key_lo > warp_pos_hi - window);
#pragma unroll
            for (int kb = 0; kb < PAGE / 16; ++kb) {
                float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
                qk_16keys<HD>(qf, ktile, kb * 16, s);
#pragma unroll
                for (int t = 0; t < 2; ++t)
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int key = key_lo + kb * 16 + t * 8 + 2 * tq + (e & 1);
                        const int pos = (e & 2) ? p1 : p0;
                        const bool vis = full || (key <= pos && (window <= 0 || key > pos - window));
                        s[t][e] = vis ? s[t][e] * scale : -INFINITY;
                    }
                softmax_update<2, HD / 8>(s, m, l, o);
                uint32_t pf[4] = {pack_bf16(s[0][0], s[0][1]), pack_bf16(s[0][2], s[0][3]),
                                  pack_bf16(s[1][0], s[1][1]), pack_bf16(s[1][2], s[1][3])};
                pv_16keys<HD>(pf, vtile, kb * 16, o);
            }
        }
        __syncthreads();
    }

    const float inv0 = 1.0f / l[0], inv1 = 1.0f / l[1];
#pragma unroll
    for (int t = 0; t < HD / 8; ++t) {
        const int d = t * 8 + 2 * tq;
        if (r0 < rows)
            *reinterpret_cast<uint32_t*>(out + (size_t)(tok0 + q0 + r0) * out_ld + (size_t)h * HD + d) =
                pack_bf16(o[t][0] * inv0, o[t][1] * inv0);
        if (r1 < rows)
            *reinterpret_cast<uint32_t*>(out + (size_t)(tok0 + q0 + r1) * out_ld + (size_t)h * HD + d) =
                pack_bf16(o[t][2] * inv1, o[t][3] * inv1);
    }
}

template <int HD>
int launch_decode(const void* q, int q_ld, const void* kc, const void* vc, const int* page_table, int max_pages,
                  const int* seq_slot, const int* seq_len, const int* cu_seqlens, int n_seqs, int n_heads,
                  int n_kv_heads, float scale, int window, int n_splits, float* part_o, float* part_ml, void* out,
                  int out_ld, cudaStream_t stream) {
    constexpr int SMEM = 2 * NBUF * PAGE * HD * 2 + 16 * HD * 2;      // the merge area lies over the page buffers
    static_assert((4 * 16 * (HD + 4) + 4 * 16 * 2 + 4 * 16 + 16 * 2) * 4 <= SMEM, "merge area must fit");
    static PerDeviceOnce configured;       // per device: the attribute belongs to a device's copy of the kernel
    if (int rc = raise_dynamic_smem(attn_decode_kernel<HD>, SMEM, configured, "attention")) return rc;
    dim3 grid(n_seqs, n_kv_heads, n_splits);
    cudaError_t e = launch_dependent(
        attn_decode_kernel<HD>, grid, dim3(THREADS), (size_t)SMEM, stream, (const __nv_bfloat16*)q, q_ld,
        (const __nv_bfloat16*)kc, (const __nv_bfloat16*)vc, page_table, max_pages, seq_slot, seq_len, cu_seqlens,
        n_heads, n_kv_heads, scale, window, n_splits, part_o, part_ml, (__nv_bfloat16*)out, out_ld);
    if (int rc = check_launch(e, "attn_decode")) return rc;
    if (n_splits > 1) {
        e = launch_dependent(attn_combine_kernel, dim3(n_seqs, n_heads), dim3(HD >= 128 ? 128 : 64), (size_t)0, stream,
                             (const float*)part_o, (const float*)part_ml, cu_seqlens, n_heads, (int)HD, n_splits,
                             (__nv_bfloat16*)out, out_ld);
        return check_launch(e, "attn_combine");
    }
    return 0;
}

template <int HD>
int launch_decode_tma(const CUtensorMap& mk, const CUtensorMap& mv, const void* q, int q_ld, const int* page_table,
                      int max_pages, const int* seq_slot, const int* seq_len, const int* cu_seqlens, int n_seqs,
                      int n_heads, int n_kv_heads, float scale, int window, int n_splits, float* part_o,
                      float* part_ml, void* out, int out_ld, int* status, cudaStream_t stream) {
    constexpr int SMEM = 2 * RING * PAGE * HD * 2 + 16 * HD * 2 + 1024;
    static_assert((4 * 16 * (HD + 4) + 4 * 16 * 2 + 4 * 16 + 16 * 2) * 4 <= 2 * RING * PAGE * HD * 2, "merge area must fit the ring");
    static PerDeviceOnce configured;       // per device: the attribute belongs to a device's copy of the kernel
    if (int rc = raise_dynamic_smem(attn_decode_tma_kernel<HD, false>, SMEM, configured, "attention")) return rc;
    dim3 grid(n_seqs, n_kv_heads, n_splits);
    cudaError_t e = launch_dependent(
        attn_decode_tma_kernel<HD, false>, grid, dim3(DECODE_TMA_THREADS), (size_t)SMEM, stream, mk, mv, (const __nv_bfloat16*)q,
        q_ld, page_table, max_pages, seq_slot, seq_len, cu_seqlens, n_heads, n_kv_heads, scale, window, n_splits, part_o,
        part_ml, (__nv_bfloat16*)out, out_ld, status);
    if (int rc = check_launch(e, "attn_decode_tma")) return rc;
    if (n_splits > 1) {
        e = launch_dependent(attn_combine_kernel, dim3(n_seqs, n_heads), dim3(HD >= 128 ? 128 : 64), (size_t)0, stream,
                             (const float*)part_o, (const float*)part_ml, cu_seqlens, n_heads, (int)HD, n_splits,
                             (__nv_bfloat16*)out, out_ld);
        return check_launch(e, "attn_combine");
    }
    return 0;
}

// The TMA-fed kernel with the splits of a (sequence, kv head) as one cluster.
template <int HD>
constexpr int tma_cluster_smem_bytes() {
    return 2 * RING * PAGE * HD * 2 + 16 * HD * 2 + CLUSTER_RECV_FLOATS<HD> * 4 + 1024;
}

template <int HD>
PerDeviceOnce& tma_cluster_configured() {
    static PerDeviceOnce once;
    return once;
}

template <int HD>
void tma_cluster_config(cudaLaunchConfig_t& cfg, cudaLaunchAttribute* attr, int n_seqs, int n_kv_heads, int n_splits,
                        cudaStream_t stream) {
    cfg = {};
    cfg.gridDim = dim3(n_seqs, n_kv_heads, n_splits);
    cfg.blockDim = dim3(DECODE_TMA_THREADS);
    cfg.dynamicSmemBytes = tma_cluster_smem_bytes<HD>();
    cfg.stream = stream;
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = (unsigned)n_splits;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 2 : 1;
}

template <int HD>
int launch_decode_tma_cluster(const CUtensorMap& mk, const CUtensorMap& mv, const void* q, int q_ld, const int* page_table,
                              int max_pages, const int* seq_slot, const int* seq_len, const int* cu_seqlens, int n_seqs,
                              int n_heads, int n_kv_heads, float scale, int window, int n_splits, void* out, int out_ld,
                              int* status, cudaStream_t stream) {
    auto kernel = attn_decode_tma_kernel<HD, true>;
    if (int rc = raise_dynamic_smem(kernel, tma_cluster_smem_bytes<HD>(), tma_cluster_configured<HD>(), "attention")) return rc;
    cudaLaunchConfig_t cfg;
    cudaLaunchAttribute attr[2];
    tma_cluster_config<HD>(cfg, attr, n_seqs, n_kv_heads, n_splits, stream);
    cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, mk, mv, (const __nv_bfloat16*)q, q_ld, page_table, max_pages, seq_slot,
                                       seq_len, cu_seqlens, n_heads, n_kv_heads, scale, window, n_splits, (float*)nullptr,
                                       (float*)nullptr, (__nv_bfloat16*)out, out_ld, status);
    return check_launch(e, "attn_decode_tma_cluster");
}

// How many clusters of n_splits CTAs of that kernel the device holds at once.
template <int HD>
int decode_tma_cluster_capacity(int n_splits, int* clusters) {
    auto kernel = attn_decode_tma_kernel<HD, true>;
    if (int rc = raise_dynamic_smem(kernel, tma_cluster_smem_bytes<HD>(), tma_cluster_configured<HD>(), "attention")) return rc;
    cudaLaunchConfig_t cfg;
    cudaLaunchAttribute attr[2];
    tma_cluster_config<HD>(cfg, attr, 1, 1, n_splits, nullptr);
    cfg.numAttrs = 1;
    cudaError_t e = cudaOccupancyMaxActiveClusters(clusters, kernel, &cfg);
    if (e != cudaSuccess) return fail("attention_decode: cannot ask how many clusters fit: %s", cudaGetErrorString(e));
    return 0;
}

template <int HD>
int launch_prefill(const void* q, int q_ld, const void* kc, const void* vc, const int* page_table, int max_pages,
                   const int* seq_slot, const int* seq_start, const int* cu_seqlens, int n_seqs, int max_new,
                   int n_heads, int n_kv_heads, float scale, int window, void* out, int out_ld, cudaStream_t stream) {
    constexpr int SMEM = 4 * PAGE * HD * 2 + 64 * HD * 2;
    static PerDeviceOnce configured;       // per device: the attribute belongs to a device's copy of the kernel
    if (int rc = raise_dynamic_smem(attn_prefill_kernel<HD>, SMEM, configured, "attention")) return rc;
    dim3 grid((max_new + 63) / 64, n_heads, n_seqs);
    cudaError_t e = launch_dependent(
        attn_prefill_kernel<HD>, grid, dim3(THREADS), (size_t)SMEM, stream, (const __nv_bfloat16*)q, q_ld,
        (const __nv_bfloat16*)kc, (const __nv_bfloat16*)vc, page_table, max_pages, seq_slot, seq_start, cu_seqlens,
        n_heads, n_kv_heads, scale, window, (__nv_bfloat16*)out, out_ld);
    return check_launch(e, "attn_prefill");
}

int check_common(int hd, int page_size, int n_heads, int n_kv_heads, int q_ld, int out_ld, const void* q,
                 const void* out) {
    if (hd != 64 && hd != 128) return fail("attention_mma: head_dim %d is not 64 or 128", hd);
    if (page_size != PAGE) return fail("attention_mma: cache pages of %d positions, the kernel is built for %d", page_size, PAGE);
    if (n_kv_heads <= 0 || n_heads % n_kv_heads) return fail("attention_mma: %d heads, %d kv heads", n_heads, n_kv_heads);
    if (q_ld % 8 || out_ld % 2 || (uintptr_t)q % 16 || (uintptr_t)out % 4)
        return fail("attention_mma: q rows must be 16-byte aligned (ld %d), out rows 4-byte aligned (ld %d)", q_ld, out_ld);
    return 0;
}

}  // namespace

// 1 if the tensor-core kernels take this shape (the caller falls back to the generic kernel otherwise)
RI_API int ri_attention_mma_supports(int hd, int page_size, int n_heads, int n_kv_heads, int decode) {
    if (hd != 64 && hd != 128) return 0;
    if (page_size != PAGE) return 0;
    if (n_kv_heads <= 0 || n_heads % n_kv_heads) return 0;
    if (decode && n_heads / n_kv_heads > 16) return 0;
    return 1;
}

// Scratch for the split partial results, in floats: part_o needs n_seqs*n_heads*n_splits*hd,
// part_ml n_seqs*n_heads*n_splits*2.  They may be null when n_splits == 1.
RI_API int ri_attention_decode(const void* q, int q_ld, const void* kcache, const void* vcache, const int* page_table,
                               int max_pages, const int* seq_slot, const int* seq_len, const int* cu_seqlens,
                               void* out, int out_ld, int n_seqs, int n_heads, int n_kv_heads, int hd, int page_size,
                               float scale, int window, int n_splits, float* part_o, float* part_ml,
                               cudaStream_t stream) {
    if (n_seqs <= 0) return 0;
    if (int rc = check_common(hd, page_size, n_heads, n_kv_heads, q_ld, out_ld, q, out)) return rc;
    if (n_heads / n_kv_heads > 16) return fail("attention_decode: %d query heads per kv head exceed 16", n_heads / n_kv_heads);
    if (n_splits < 1 || n_splits > 65535) return fail("attention_decode: %d splits", n_splits);
    if (n_splits > 1 && (part_o == nullptr || part_ml == nullptr)) return fail("attention_decode: splits need scratch");
    if (n_kv_heads > 65535) return fail("attention_decode: %d kv heads exceed the grid limit", n_kv_heads);
    if (hd == 64)
        return launch_decode<64>(q, q_ld, kcache, vcache, page_table, max_pages, seq_slot, seq_len, cu_seqlens, n_seqs,
                                 n_heads, n_kv_heads, scale, window, n_splits, part_o, part_ml, out, out_ld, stream);
    return launch_decode<128>(q, q_ld, kcache, vcache, page_table, max_pages, seq_slot, seq_len, cu_seqlens, n_seqs,
                              n_heads, n_kv_heads, scale, window, n_splits, part_o, part_ml, out, out_ld, stream);
}

// The same with the cache pages brought in by TMA.  map_k / map_v: tensor maps (128 bytes each) of the
// layer's K and V viewed as [pages * kv heads * 64, head_dim] with a {64, 64} box and 128-byte swizzle.
// `status` (may be null) is a host-visible int that receives a code if a bounded wait ran out.
RI_API int ri_attention_decode_tma(const void* map_k, const void* map_v, const void* q, int q_ld,
                                   const int* page_table, int max_pages, const int* seq_slot, const int* seq_len,
                                   const int* cu_seqlens, void* out, int out_ld, int n_seqs, int n_heads,
                                   int n_kv_heads, int hd, int page_size, float scale, int window, int n_splits,
                                   float* part_o, float* part_ml, int* status, cudaStream_t stream) {
    if (n_seqs <= 0) return 0;
    if (int rc = check_common(hd, page_size, n_heads, n_kv_heads, q_ld, out_ld, q, out)) return rc;
    if (n_heads / n_kv_heads > 16) return fail("attention_decode: %d query heads per kv head exceed 16", n_heads / n_kv_heads);
    if (n_splits < 1 || n_splits > 65535) return fail("attention_decode: %d splits", n_splits);
    if (n_splits > 1 && (part_o == nullptr || part_ml == nullptr)) return fail("attention_decode: splits need scratch");
    if (n_kv_heads > 65535) return fail("attention_decode: %d kv heads exceed the grid limit", n_kv_heads);
    const CUtensorMap& mk = *reinterpret_cast<const CUtensorMap*>(map_k);
    const CUtensorMap& mv = *reinterpret_cast<const CUtensorMap*>(map_v);
    if (hd == 64)
        return launch_decode_tma<64>(mk, mv, q, q_ld, page_table, max_pages, seq_slot, seq_len, cu_seqlens, n_seqs, n_heads,
                                     n_kv_heads, scale, window, n_splits, part_o, part_ml, out, out_ld, status, stream);
    return launch_decode_tma<128>(mk, mv, q, q_ld, page_table, max_pages, seq_slot, seq_len, cu_seqlens, n_seqs, n_heads,
                                  n_kv_heads, scale, window, n_splits, part_o, part_ml, out, out_ld, status, stream);
}

// The same with the 2..8 splits of a (sequence, kv head) as one thread-block cluster that merges its own partial
// results through distributed shared memory: no scratch and no second kernel.
RI_API int ri_attention_decode_tma_cluster(const void* map_k, const void* map_v, const void* q, int q_ld,
                                           const int* page_table, int max_pages, const int* seq_slot,
                                           const int* seq_len, const int* cu_seqlens, void* out, int out_ld, int n_seqs,
                                           int n_heads, int n_kv_heads, int hd, int page_size, float scale, int window,
                                           int n_splits, int* status, cudaStream_t stream) {
    if (n_seqs <= 0) return 0;
    if (int rc = check_common(hd, page_size, n_heads, n_kv_heads, q_ld, out_ld, q, out)) return rc;
    if (n_heads / n_kv_heads > 16) return fail("attention_decode: %d query heads per kv head exceed 16", n_heads / n_kv_heads);
    if (n_splits < 2 || n_splits > MAX_CLUSTER_SPLITS)
        return fail("attention_decode: a cluster takes 2 to %d splits, not %d", MAX_CLUSTER_SPLITS, n_splits);
    if (n_kv_heads > 65535) return fail("attention_decode: %d kv heads exceed the grid limit", n_kv_heads);
    const CUtensorMap& mk = *reinterpret_cast<const CUtensorMap*>(map_k);
    const CUtensorMap& mv = *reinterpret_cast<const CUtensorMap*>(map_v);
    if (hd == 64)
        return launch_decode_tma_cluster<64>(mk, mv, q, q_ld, page_table, max_pages, seq_slot, seq_len, cu_seqlens, n_seqs,
                                             n_heads, n_kv_heads, scale, window, n_splits, out, out_ld, status, stream);
    return launch_decode_tma_cluster<128>(mk, mv, q, q_ld, page_table, max_pages, seq_slot, seq_len, cu_seqlens, n_seqs,
                                          n_heads, n_kv_heads, scale, window, n_splits, out, out_ld, status, stream);
}

// clusters[0] = how many clusters of n_splits CTAs of that kernel the current device holds at the same time
RI_API int ri_attention_decode_tma_cluster_capacity(int hd, int n_splits, int* clusters) {
    if (hd != 64 && hd != 128) return fail("attention_mma: head_dim %d is not 64 or 128", hd);
    if (n_splits < 2 || n_splits > MAX_CLUSTER_SPLITS)
        return fail("attention_decode: a cluster takes 2 to %d splits, not %d", MAX_CLUSTER_SPLITS, n_splits);
    return hd == 64 ? decode_tma_cluster_capacity<64>(n_splits, clusters) : decode_tma_cluster_capacity<128>(n_splits, clusters);
}

RI_API int ri_attention_prefill(const void* q, int q_ld, const void* kcache, const void* vcache, const int* page_table,
                                int max_pages, const int* seq_slot, const int* seq_start, const int* cu_seqlens,
                                void* out, int out_ld, int n_seqs, int max_new, int n_heads, int n_kv_heads, int hd,
                                int page_size, float scale, int window, cudaStream_t stream) {
    if (n_seqs <= 0 || max_new <= 0) return 0;
    if (int rc = check_common(hd, page_size, n_heads, n_kv_heads, q_ld, out_ld, q, out)) return rc;
    if (n_heads > 65535 || n_seqs > 65535) return fail("attention_prefill: %d heads / %d sequences exceed the grid limit", n_heads, n_seqs);
    if (hd == 64)
        return launch_prefill<64>(q, q_ld, kcache, vcache, page_table, max_pages, seq_slot, seq_start, cu_seqlens, n_seqs,
                                  max_new, n_heads, n_kv_heads, scale, window, out, out_ld, stream);
    return launch_prefill<128>(q, q_ld, kcache, vcache, page_table, max_pages, seq_slot, seq_start, cu_seqlens, n_seqs,
                               max_new, n_heads, n_kv_heads, scale, window, out, out_ld, stream);
}

// ---------------------------------------------------------------------------------------------
// The allocation-free variant (see attention_decode_static.h).  The scratch for the split
// partial results is this file-scope device array.  In host code its name is only a stand-in
// for the symbol, not a device address, so the address is looked up once per device with
// cudaGetSymbolAddress and that pointer is what the kernel receives.
// ---------------------------------------------------------------------------------------------
static __device__ __align__(256) float g_decode_static_scratch[RI_DECODE_STATIC_SCRATCH_FLOATS];

namespace {
constexpr int MAX_DEVICES = 64;
// One address per device, looked up on that device's first call.  Atomic: two host threads that make a
// device's first call together both store the same address.
std::atomic<float*> g_decode_static_ptr[MAX_DEVICES];

// The device address of the scratch array on the current device; looked up on the first call.
int decode_static_scratch(float** ptr) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return fail("attention_decode_static: cudaGetDevice failed: %s", cudaGetErrorString(e));
    if (dev < 0 || dev >= MAX_DEVICES) return fail("attention_decode_static: device %d is out of range", dev);
    float* p = g_decode_static_ptr[dev].load(std::memory_order_acquire);
    if (p == nullptr) {
        e = cudaGetSymbolAddress((void**)&p, g_decode_static_scratch);
        if (e != cudaSuccess || p == nullptr)
            return fail("attention_decode_static: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
        g_decode_static_ptr[dev].store(p, std::memory_order_release);
    }
    *ptr = p;
    return 0;
}
}  // namespace

RI_API int ri_attention_decode_static(const void* q, int q_ld, const void* kcache, const void* vcache,
                                      const int* page_table, int max_pages, const int* seq_slot, const int* seq_len,
                                      const int* cu_seqlens, void* out, int out_ld, int n_seqs, int n_heads,
                                      int n_kv_heads, int hd, int page_size, float scale, int window, int n_splits,
                                      cudaStream_t stream) {
    if (n_seqs <= 0) return 0;
    if (n_heads <= 0 || hd <= 0 || n_splits < 1)
        return fail("attention_decode_static: %d heads, head_dim %d, %d splits", n_heads, hd, n_splits);
    const long long rows = (long long)n_seqs * n_heads * n_splits;
    const long long need = rows * (hd + 2);
    if (need > RI_DECODE_STATIC_SCRATCH_FLOATS)
        return fail("attention_decode_static: %d sequences x %d heads x %d splits x (head_dim %d + 2) = %lld floats "
                    "exceed the built-in scratch of %d floats; use fewer splits or ri_attention_decode with your own scratch",
                    n_seqs, n_heads, n_splits, hd, need, RI_DECODE_STATIC_SCRATCH_FLOATS);
    float* scratch = nullptr;
    if (int rc = decode_static_scratch(&scratch)) return rc;
    float* part_o = scratch;                    // rows * hd floats
    float* part_ml = scratch + rows * hd;       // rows * 2 floats
    return ri_attention_decode(q, q_ld, kcache, vcache, page_table, max_pages, seq_slot, seq_len, cu_seqlens, out,
                               out_ld, n_seqs, n_heads, n_kv_heads, hd, page_size, scale, window, n_splits, part_o,
                               part_ml, stream);
}

RI_DEFINE_LAST_ERROR()
