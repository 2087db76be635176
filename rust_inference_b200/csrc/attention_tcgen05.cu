// Causal bf16 attention for prompts and continuations on the 5th-generation tensor cores.
//
// What it computes is attention.rs:95-121 for every new token of every sequence: scores of the
// token's query against the keys 0..position of its slot, scaled by 1/sqrt(head_dim), softmax with
// the maximum subtracted (math.rs:104-118), weighted sum of the values.  Keys and values are read
// from the paged cache only (the step's own tokens were written there first).
//
// A CTA serves 128 consecutive query tokens of one head and walks the key pages (64 keys each) up
// to the causal limit:
//   S = Q K^T     tcgen05.mma, M = 128 queries, N = 64 keys, K = head_dim; Q and the K page come
//                 to shared memory by TMA (128-byte swizzle, both K-major); S lives in tensor memory.
//   softmax       128 threads, one per query row (= one TMEM lane): the thread reads its 64 scores
//                 with tcgen05.ld, so maxima and sums need no exchange between threads.  Scores
//                 are kept in the base-2 domain.  The running maximum used for scaling only moves
//                 when the true maximum exceeds it by more than 2^8, so P stays below 256 and the
//                 accumulator is rescaled rarely (exactness is kept: the final division by the
//                 row sum uses the same scaling).
//   O += P V      P goes back to tensor memory as bf16, over the scores it was made from, and is the
//                 A operand; the V page, [keys][head_dim] as the cache holds it, is the B operand
//                 in MN-major form; O accumulates in tensor memory in float32.
// Warp 0 issues the TMA loads, warp 1 the MMAs, warps 2-5 are the softmax rows.  There are two score
// buffers in tensor memory: S of page j+1 is computed while the softmax of page j runs, and the
// softmax computes its exponentials before it waits for P V of the page before (it needs that only
// to overwrite P and to rescale O).  Two CTAs fit on an SM (96 KiB of shared memory, 256 TMEM columns).
//
// All mbarrier waits are bounded; on a timeout the kernel records a code in the host-visible
// status word and winds down.
#include "tcgen05_common.cuh"

using namespace ri;
using namespace ri::tc;

namespace {

constexpr int BM = 128;            // queries per CTA
constexpr int BN = 64;             // keys per step = one cache page
constexpr int THREADS = 192;
constexpr int RESCALE_LOG2 = 8;    // the scaling maximum follows the true one in steps of at least 2^8

enum AttnStatus { ST_ATTN_PRODUCER = 11, ST_ATTN_MMA = 12, ST_ATTN_SOFTMAX = 13, ST_ATTN_DRAIN = 14, ST_ATTN_SMEM = 15 };

// MN-major B operand (the V page: rows are keys, 128-byte rows of 64 head_dim values, written by TMA
// with 128-byte swizzle): groups of 8 key rows are 1024 bytes apart (stride byte offset), the next 64
// head_dim columns are a tile of their own `atom_stride` bytes further (leading byte offset).
__device__ __forceinline__ uint64_t make_smem_desc_mn(uint32_t addr, uint32_t atom_stride) {
    uint64_t d = 0;
    d |= (uint64_t)((addr & 0x3FFFF) >> 4);
    d |= (uint64_t)((atom_stride >> 4) & 0x3FFF) << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}

// D[tmem] (+)= A[tmem] * B[smem]: the A operand (128 rows x 16 bf16, two to a 32-bit column, 8 columns) comes from
// tensor memory, where the softmax threads put the probabilities.
__device__ __forceinline__ void umma_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t b_desc, uint32_t idesc, bool accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(tmem_d), "r"(tmem_a), "l"(b_desc), "r"(idesc), "r"((uint32_t)accumulate)
        : "memory");
}

__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t* r) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
          "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
// 2^x on the special-function unit.  Its relative error (about 2^-22) is far below the bf16 rounding
// of P that follows; -inf gives 0.
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

template <int HD>
__global__ void __launch_bounds__(THREADS, 2)
attn_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                       const __grid_constant__ CUtensorMap map_v, const int* __restrict__ page_table, int max_pages,
                       const int* __restrict__ seq_slot, const int* __restrict__ seq_start,
                       const int* __restrict__ cu_seqlens, int n_heads, int n_kv_heads, float scale_log2, int window,
                       __nv_bfloat16* __restrict__ out, int out_ld, uint32_t smem_bytes, int* status) {
    constexpr int ATOMS = HD / 64;                       // 64-wide (128-byte) column tiles per row of head_dim
    constexpr int Q_BYTES = ATOMS * BM * 128;            // [atom][128 queries][64]
    constexpr int K_BYTES = ATOMS * BN * 128;            // one buffer: [atom][64 keys][64]
    constexpr int V_BYTES = ATOMS * BN * 128;
    constexpr int S_COL = 0, O_COL = 2 * BN;             // two score buffers, then the output accumulator
    constexpr int TMEM_COLS = 256;
    constexpr uint32_t IDESC_S = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
    constexpr uint32_t IDESC_PV = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((uint32_t)(HD >> 3) << 17) |
                                  ((uint32_t)(BM >> 4) << 24);

    // Everything lives in dynamic shared memory: the tiles (1024-byte aligned for the 128-byte swizzle) and,
    // behind them, the barriers.  With head_dim 128 the tiles take 96 KiB and two CTAs share an SM only if
    // nothing is spent on alignment: the kernel declares no static shared memory, so that the dynamic part
    // starts at the CTA's window, and checks that it fits.
    extern __shared__ uint8_t smem_raw[];
    struct Sync {
        uint64_t q_full, k_full[2], k_empty[2], v_full[2], v_empty[2], s_full[2], p_full, pv_done;
        uint32_t tmem_base_slot;
        volatile int abort_flag;
    };

    const int b = blockIdx.y, h = blockIdx.x;
    const int tok0 = cu_seqlens[b], n_new = cu_seqlens[b + 1] - tok0;
    // the last query tiles see the most keys: they go first, so the short ones fill the tail
    const int q0 = (int)(gridDim.z - 1 - blockIdx.z) * BM;
    if (q0 >= n_new) return;                                                // uniform over the CTA
    const int kvh = h / (n_heads / n_kv_heads);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int start = seq_start[b];
    const int rows = min(BM, n_new - q0);
    const int pos_lo = start + q0, pos_hi = start + q0 + rows - 1;
    const int first_key = (window > 0 && pos_lo - window + 1 > 0) ? pos_lo - window + 1 : 0;
    const int pg_begin = first_key / BN, n_pages = pos_hi / BN + 1 - pg_begin;

    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    const uint32_t q_smem = base, k_smem = q_smem + Q_BYTES, v_smem = k_smem + 2 * K_BYTES;
    constexpr uint32_t TILE_BYTES = Q_BYTES + 2 * K_BYTES + 2 * V_BYTES;
    if (base - raw + TILE_BYTES + (uint32_t)sizeof(Sync) > smem_bytes) {          // uniform over the CTA
        if (threadIdx.x == 0) report(status, ST_ATTN_SMEM);
        return;
    }
    Sync& sy = *reinterpret_cast<Sync*>(smem_raw + (base - raw) + TILE_BYTES);
    uint64_t &q_full = sy.q_full, &p_full = sy.p_full, &pv_done = sy.pv_done;
    uint64_t (&k_full)[2] = sy.k_full, (&k_empty)[2] = sy.k_empty, (&v_full)[2] = sy.v_full, (&v_empty)[2] = sy.v_empty;
    uint64_t (&s_full)[2] = sy.s_full;
    uint32_t& tmem_base_slot = sy.tmem_base_slot;
    volatile int& abort_flag = sy.abort_flag;

    if (threadIdx.x == 0) {
        mbar_init(smem_u32(&q_full), 1);
        for (int i = 0; i < 2; ++i) { mbar_init(smem_u32(&k_full[i]), 1); mbar_init(smem_u32(&k_empty[i]), 1); }
        for (int i = 0; i < 2; ++i) { mbar_init(smem_u32(&v_full[i]), 1); mbar_init(smem_u32(&v_empty[i]), 1); }
        mbar_init(smem_u32(&s_full[0]), 1);
        mbar_init(smem_u32(&s_full[1]), 1);
        mbar_init(smem_u32(&p_full), 4);          // one arrival per softmax warp
        mbar_init(smem_u32(&pv_done), 1);
        abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)),
                     "r"((uint32_t)TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_slot;
    let_next_kernel_start();

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            wait_for_previous_kernels();           // q and the newest keys and values come from the kernel before
            const int* pages = page_table + (size_t)seq_slot[b] * max_pages;
            mbar_expect_tx(smem_u32(&q_full), Q_BYTES);
            for (int a = 0; a < ATOMS; ++a)
                tma_load_2d(q_smem + a * BM * 128, &map_q, smem_u32(&q_full), h * HD + a * 64, tok0 + q0);
            int k_issued = 0, v_issued = 0;
            int page_next = pages[pg_begin];                        // a page's number is fetched one turn ahead
            for (int j = 0; j < n_pages; ++j) {
                const int row = (page_next * n_kv_heads + kvh) * BN;
                if (j + 1 < n_pages) page_next = pages[pg_begin + j + 1];
                const int kb = j & 1;
                if (!mbar_wait(smem_u32(&k_empty[kb]), (uint32_t)((j >> 1) & 1) ^ 1u) || abort_flag) {
                    report(status, ST_ATTN_PRODUCER); abort_flag = 1; break;
                }
                mbar_expect_tx(smem_u32(&k_full[kb]), K_BYTES);
                for (int a = 0; a < ATOMS; ++a)
                    tma_load_2d(k_smem + kb * K_BYTES + a * BN * 128, &map_k, smem_u32(&k_full[kb]), a * 64, row);
                k_issued = j + 1;
                if (!mbar_wait(smem_u32(&v_empty[kb]), (uint32_t)((j >> 1) & 1) ^ 1u) || abort_flag) {
                    report(status, ST_ATTN_PRODUCER); abort_flag = 1; break;
                }
                mbar_expect_tx(smem_u32(&v_full[kb]), V_BYTES);
                for (int a = 0; a < ATOMS; ++a)
                    tma_load_2d(v_smem + kb * V_BYTES + a * BN * 128, &map_v, smem_u32(&v_full[kb]), a * 64, row);
                v_issued = j + 1;
            }
            // do not leave while a copy into this CTA's shared memory may be in flight
            if (!mbar_wait(smem_u32(&q_full), 0)) report(status, ST_ATTN_DRAIN);
            for (int j = max(0, k_issued - 2); j < k_issued; ++j)
                if (!mbar_wait(smem_u32(&k_full[j & 1]), (uint32_t)((j >> 1) & 1))) { report(status, ST_ATTN_DRAIN); break; }
            for (int j = max(0, v_issued - 2); j < v_issued; ++j)
                if (!mbar_wait(smem_u32(&v_full[j & 1]), (uint32_t)((j >> 1) & 1))) { report(status, ST_ATTN_DRAIN); break; }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            bool ok = mbar_wait(smem_u32(&q_full), 0);
            if (!ok) { report(status, ST_ATTN_MMA); abort_flag = 1; }
            // One thread issues every MMA, and a lone thread gets a dependent instruction out only every few
            // cycles: the descriptors are built once, and a page's MMAs add constants to their address field
            // (shared memory ends below 256 KiB, so the 14-bit field never carries).
            const uint64_t q_desc = make_smem_desc(q_smem), k_desc = make_smem_desc(k_smem);
            const uint64_t v_desc = make_smem_desc_mn(v_smem, BN * 128);
            const uint32_t k_full0 = smem_u32(&k_full[0]), k_empty0 = smem_u32(&k_empty[0]), s_full0 = smem_u32(&s_full[0]);
            const uint32_t v_full0 = smem_u32(&v_full[0]), v_empty0 = smem_u32(&v_empty[0]);
            const uint32_t p_full_a = smem_u32(&p_full), pv_done_a = smem_u32(&pv_done);
            // scores of page j go to buffer j & 1, so S(j+1) is computed while the softmax of page j runs
            auto issue_s = [&](int j) -> bool {
                const uint32_t kb = (uint32_t)j & 1u;
                if (!mbar_wait(k_full0 + 8u * kb, (uint32_t)((j >> 1) & 1))) return false;
                tc_fence_after();
                const uint64_t kd = k_desc + (uint64_t)(kb * (uint32_t)(K_BYTES >> 4));
                const uint32_t s_acc = tmem_base + S_COL + kb * BN;
#pragma unroll
                for (int ks = 0; ks < HD / 16; ++ks)
                    umma(s_acc, q_desc + (uint64_t)(((ks / 4) * BM * 128 + (ks % 4) * 32) >> 4),
                         kd + (uint64_t)(((ks / 4) * BN * 128 + (ks % 4) * 32) >> 4), IDESC_S, ks > 0);
                umma_commit(k_empty0 + 8u * kb);
                umma_commit(s_full0 + 8u * kb);
                return true;
            };
            if (ok && !issue_s(0)) { report(status, ST_ATTN_MMA); abort_flag = 1; ok = false; }
            for (int j = 0; j < n_pages && ok; ++j) {
                // the buffer S(j+1) goes to was read by the softmax of page j-1, which arrived on p_full before PV(j-1)
                if (j + 1 < n_pages && !issue_s(j + 1)) { report(status, ST_ATTN_MMA); abort_flag = 1; break; }
                const uint32_t vb = (uint32_t)j & 1u;
                if (!mbar_wait(p_full_a, vb) || !mbar_wait(v_full0 + 8u * vb, (uint32_t)((j >> 1) & 1))) {
                    report(status, ST_ATTN_MMA); abort_flag = 1; break;
                }
                tc_fence_after();
                const uint64_t vd = v_desc + (uint64_t)(vb * (uint32_t)(V_BYTES >> 4));
#pragma unroll
                for (int ks = 0; ks < BN / 16; ++ks)
                    // P of page j lies, two bf16 to a column, over the first half of the score buffer it came from
                    umma_ts(tmem_base + O_COL, tmem_base + S_COL + vb * BN + ks * 8, vd + (uint64_t)(ks * 16 * 128 >> 4),
                            IDESC_PV, j > 0 || ks > 0);
                umma_commit(v_empty0 + 8u * vb);
                umma_commit(pv_done_a);
            }
        }
    } else {
        // ---------------- softmax: one thread per query row ----------------
        const int lane_base = (warp & 3) * 32;
        const int r = lane_base + lane;                       // row of the tile = TMEM lane
        const int pos = start + q0 + r;
        const uint32_t trow = tmem_base + ((uint32_t)lane_base << 16);
        float m_used = -INFINITY, l = 0.f;
        bool ok = true;
        for (int j = 0; j < n_pages; ++j) {
            if (!mbar_wait(smem_u32(&s_full[j & 1]), (uint32_t)((j >> 1) & 1)) || abort_flag) {
                if (lane == 0) { report(status, ST_ATTN_SOFTMAX); abort_flag = 1; }
                ok = false;
                break;
            }
            tc_fence_after();
            uint32_t sv[BN];
#pragma unroll
            for (int c = 0; c < BN; c += 16) tmem_ld16(trow + S_COL + (j & 1) * BN + c, sv + c);
            tmem_wait_ld();
            const int key0 = (pg_begin + j) * BN;
            // The maximum is taken over the raw scores (the scale is positive), and scale and maximum
            // are folded into one multiply-add per score: p = 2^(s * scale_log2 - m).
            float mx_raw = -INFINITY;
            // pages that every row of the warp sees whole need no mask
            const bool whole = key0 + BN - 1 <= pos_lo + lane_base && (window <= 0 || key0 > pos_lo + lane_base + 31 - window);
            if (whole) {
#pragma unroll
                for (int c = 0; c < BN; c += 2)
                    mx_raw = fmaxf(mx_raw, fmaxf(__uint_as_float(sv[c]), __uint_as_float(sv[c + 1])));
            } else {
#pragma unroll
                for (int c = 0; c < BN; ++c) {
                    const int key = key0 + c;
                    const bool vis = key <= pos && (window <= 0 || key > pos - window);
                    if (!vis) sv[c] = 0xff800000u;              // -inf
                    mx_raw = fmaxf(mx_raw, __uint_as_float(sv[c]));
                }
            }
            const float mx = mx_raw * scale_log2;                // -inf stays -inf
            // move the scaling maximum only when the true one ran ahead of it by more than 2^8
            const bool move = mx > m_used + (float)RESCALE_LOG2;
            const float m_new = move ? mx : m_used;
            const float alpha = (!move) ? 1.f : ((m_used == -INFINITY) ? 0.f : fast_exp2(m_used - m_new));
            const float neg_mref = (m_new == -INFINITY) ? 0.f : -m_new;   // nothing visible yet: every p is 0
            // the exponentials do not need the previous P V product; everything after this does
            // two scores at a time through the packed float32 pipe (one FMA and one ADD per pair)
            const float2 scale2 = make_float2(scale_log2, scale_log2), shift2 = make_float2(neg_mref, neg_mref);
            float2 sum2 = make_float2(0.f, 0.f);
            uint32_t pk[BN / 2];
#pragma unroll
            for (int c = 0; c < BN; c += 2) {
                const float2 e = __ffma2_rn(make_float2(__uint_as_float(sv[c]), __uint_as_float(sv[c + 1])), scale2, shift2);
                const float2 p = make_float2(fast_exp2(e.x), fast_exp2(e.y));
                sum2 = __fadd2_rn(sum2, p);
                pk[c >> 1] = pack2(p.x, p.y);
            }
            const float sum = sum2.x + sum2.y;
            if (j > 0) {
                // P's buffer and the accumulator are free once PV of the page before has finished
                if (!mbar_wait(smem_u32(&pv_done), (uint32_t)((j - 1) & 1)) || abort_flag) {
                    if (lane == 0) { report(status, ST_ATTN_SOFTMAX); abort_flag = 1; }
                    ok = false;
                    break;
                }
                tc_fence_after();
                if (__any_sync(0xffffffffu, move)) {            // rescale the accumulator (uniform over the warp)
#pragma unroll 1
                    for (int c = 0; c < HD; c += 16) {
                        uint32_t o[16];
                        tmem_ld16(trow + O_COL + c, o);
                        tmem_wait_ld();
#pragma unroll
                        for (int i = 0; i < 16; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
                        tmem_st16(trow + O_COL + c, o);
                    }
                    tmem_wait_st();
                }
            }
            l = l * alpha + sum;
            m_used = m_new;
            // P goes back to tensor memory, over the scores it was made from (this thread has read its row of
            // them): the product P V takes its A operand from there, so P never passes through shared memory
#pragma unroll
            for (int c = 0; c < BN / 2; c += 16) tmem_st16(trow + S_COL + (j & 1) * BN + c, pk + c);
            tmem_wait_st();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&p_full));
        }
        if (ok) {
            if (!mbar_wait(smem_u32(&pv_done), (uint32_t)((n_pages - 1) & 1))) {
                if (lane == 0) { report(status, ST_ATTN_SOFTMAX); abort_flag = 1; }
                ok = false;
            }
        }
        tc_fence_after();
        if (ok && !abort_flag) {
            wait_for_previous_kernels();          // `out` must not be written while an earlier kernel may read it
            const float inv = 1.0f / l;
            __nv_bfloat16* dst = out + (size_t)(tok0 + q0 + r) * out_ld + (size_t)h * HD;
#pragma unroll 1
            for (int c = 0; c < HD; c += 16) {
                uint32_t o[16];
                tmem_ld16(trow + O_COL + c, o);
                tmem_wait_ld();
                if (r < rows) {
                    uint4 lo, hi;
                    lo.x = pack2(__uint_as_float(o[0]) * inv, __uint_as_float(o[1]) * inv);
                    lo.y = pack2(__uint_as_float(o[2]) * inv, __uint_as_float(o[3]) * inv);
                    lo.z = pack2(__uint_as_float(o[4]) * inv, __uint_as_float(o[5]) * inv);
                    lo.w = pack2(__uint_as_float(o[6]) * inv, __uint_as_float(o[7]) * inv);
                    hi.x = pack2(__uint_as_float(o[8]) * inv, __uint_as_float(o[9]) * inv);
                    hi.y = pack2(__uint_as_float(o[10]) * inv, __uint_as_float(o[11]) * inv);
                    hi.z = pack2(__uint_as_float(o[12]) * inv, __uint_as_float(o[13]) * inv);
                    hi.w = pack2(__uint_as_float(o[14]) * inv, __uint_as_float(o[15]) * inv);
                    *reinterpret_cast<uint4*>(dst + c) = lo;
                    *reinterpret_cast<uint4*>(dst + c + 8) = hi;
                }
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)TMEM_COLS) : "memory");
    }
}

template <int HD>
int launch(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const int* page_table, int max_pages,
           const int* seq_slot, const int* seq_start, const int* cu_seqlens, int n_seqs, int max_new, int n_heads,
           int n_kv_heads, float scale, int window, void* out, int out_ld, int* status, cudaStream_t stream) {
    constexpr int ATOMS = HD / 64;
    // Q, two K and two V pages, P, the barriers; with head_dim 128 no room for alignment padding is left if
    // two CTAs are to share an SM (the kernel refuses, with a status code, a shared window that needs any)
    constexpr int TILES = ATOMS * BM * 128 + 4 * ATOMS * BN * 128;
    constexpr int SMEM = TILES + (HD >= 128 ? 256 : 1024 + 256);
    auto kernel = attn_prefill_tc_kernel<HD>;
    static PerDeviceOnce configured;       // per device: the attribute belongs to a device's copy of the kernel
    if (int rc = raise_dynamic_smem(kernel, SMEM, configured, "attention_tcgen05")) return rc;
    // blocks are handed out x fastest: every head and sequence of the longest query tiles first, the short
    // tiles last, so the causal triangle's tail is filled with small pieces
    dim3 grid(n_heads, n_seqs, (max_new + BM - 1) / BM);
    const float scale_log2 = scale * 1.4426950408889634f;
    cudaError_t e = launch_dependent(kernel, grid, dim3(THREADS), (size_t)SMEM, stream, mq, mk, mv, page_table, max_pages,
                                     seq_slot, seq_start, cu_seqlens, n_heads, n_kv_heads, scale_log2, window,
                                     (__nv_bfloat16*)out, out_ld, (uint32_t)SMEM, status);
    return check_launch(e, "attention_tcgen05");
}

}  // namespace

RI_API int ri_attention_tcgen05_supports(int hd, int page_size, int n_heads, int n_kv_heads, int q_ld, int out_ld) {
    if (hd != 64 && hd != 128) return 0;
    if (page_size != BN) return 0;
    if (n_kv_heads <= 0 || n_heads % n_kv_heads) return 0;
    if (q_ld % 8 || out_ld % 8) return 0;
    return 1;
}

// Tensor maps (128 bytes each, 64-byte aligned storage):
//   which 0: the query rows, a matrix [rows, cols] with row stride ld (the packed q/k/v buffer); box of 128 rows
//   which 1: one cache layer viewed as [pages * kv heads * 64, head_dim]; box of 64 rows (keys or values)
RI_API int ri_attention_tcgen05_encode(void* map_out, int which, const void* ptr, long long rows, long long cols,
                                       long long ld) {
    if ((uintptr_t)map_out % 64) return fail("attention_tcgen05: tensor map storage must be 64-byte aligned");
    return encode_map(reinterpret_cast<CUtensorMap*>(map_out), ptr, rows, cols, ld, which == 0 ? BM : BN,
                      which == 0 ? "attention_tcgen05 (queries)" : "attention_tcgen05 (cache)");
}

RI_API int ri_attention_tcgen05_prefill(const void* map_q, const void* map_k, const void* map_v, const int* page_table,
                                        int max_pages, const int* seq_slot, const int* seq_start,
                                        const int* cu_seqlens, void* out, int out_ld, int n_seqs, int max_new,
                                        int n_heads, int n_kv_heads, int hd, int page_size, float scale, int window,
                                        int* status, cudaStream_t stream) {
    if (n_seqs <= 0 || max_new <= 0) return 0;
    if (!ri_attention_tcgen05_supports(hd, page_size, n_heads, n_kv_heads, 8, out_ld))
        return fail("attention_tcgen05: head_dim %d, pages of %d, %d heads over %d kv heads, out rows of %d are not supported",
                    hd, page_size, n_heads, n_kv_heads, out_ld);
    if ((uintptr_t)out % 16) return fail("attention_tcgen05: out is not 16-byte aligned");
    if (n_heads > 65535 || n_seqs > 65535) return fail("attention_tcgen05: %d heads / %d sequences exceed the grid limit", n_heads, n_seqs);
    const CUtensorMap& mq = *reinterpret_cast<const CUtensorMap*>(map_q);
    const CUtensorMap& mk = *reinterpret_cast<const CUtensorMap*>(map_k);
    const CUtensorMap& mv = *reinterpret_cast<const CUtensorMap*>(map_v);
    if (hd == 64)
        return launch<64>(mq, mk, mv, page_table, max_pages, seq_slot, seq_start, cu_seqlens, n_seqs, max_new, n_heads,
                          n_kv_heads, scale, window, out, out_ld, status, stream);
    return launch<128>(mq, mk, mv, page_table, max_pages, seq_slot, seq_start, cu_seqlens, n_seqs, max_new, n_heads,
                       n_kv_heads, scale, window, out, out_ld, status, stream);
}

RI_DEFINE_LAST_ERROR()
