// out[tokens, features] = X[tokens, K] * W[features, K]^T for bf16 operands on the
// 5th-generation tensor cores: tcgen05.mma with the accumulator in tensor memory,
// operands brought to shared memory by TMA (128-byte swizzle), float32 accumulation.
//
// The product is computed transposed: the MMA's M dimension runs over 128 *features*
// (rows of W, the A operand), its N dimension over TN *tokens* (rows of X, the B
// operand), TN any multiple of 16 up to 256 (the kernel is compiled for 16, 32, 64, 128 and 256
// and runs a narrower tile inside the next larger one).  So a decode step with a handful of tokens
// still fills the 128-row MMA with weights, and a long step can take the tile width that leaves the
// least idle tail in the last wave of its persistent grid.  The SiLU-gate projection of steps of more than 128
// tokens takes the token-major kernel further down (128 tokens x 256 weight rows per tile).
// Both operands are K-major, which is how the reference lays its matrices out
// ([out, in] row-major, quant.rs:45-50) and how activations are packed.
//
// The grid is persistent: as many CTAs as fit the GPU at once, each walking its share of
// the output tiles (token tile fastest, so CTAs that run together share a weight tile in
// L2).  Warp 0 issues the TMA loads, warp 1 allocates tensor memory and issues the MMAs
// (one elected thread), warps 2-5 run the epilogue: each reads its 32 lanes of the
// accumulator with tcgen05.ld and writes the result.  There are two accumulator buffers
// in tensor memory, so the epilogue of one tile runs while the MMAs of the next fill the
// other.  K can be split over tiles; the split pieces are combined with float32 atomic
// adds, which only the residual epilogue allows.
//
// Epilogues (float32 arithmetic):
//   0  out<bf16> = acc + bias                         (q/k/v projection, attention.rs:66-76)
//   1  out<f32>  = acc + bias                         (logits, transformer.rs:97)
//   2  out<f32> += acc                                (o / down projection onto the residual
//                                                      stream, transformer.rs:38-39, :47)
//   3  out<bf16> = silu(acc) * acc2, acc2 = X W2^T    (SwiGLU, mlp.rs:35-43): two accumulators
//                                                      fed by the same X tile
//
// Every wait on an mbarrier is bounded.  A wait that runs out stores a code in the
// host-visible status word, the CTA stops issuing work, waits (bounded) for its own
// copies in flight, frees its tensor memory and returns.
//
// TMA needs 16-byte row strides: K must be a multiple of 8.  Everything else (tokens,
// features, K not a multiple of the tile) is handled by TMA's zero fill and by bounds
// checks in the epilogue.
#include "tcgen05_common.cuh"

using namespace ri;
using namespace ri::tc;

namespace {

constexpr int BLOCK_F = 128;                       // features per tile (MMA M)
constexpr int BLOCK_K = 64;                        // bf16 per k-block: one 128-byte swizzled row
constexpr int A_BYTES = BLOCK_F * BLOCK_K * 2;     // 16 KiB
constexpr int MAX_STAGES = 8;
constexpr int THREADS = 192;
constexpr int SMEM_BUDGET = 200 * 1024;

enum Status { ST_OK = 0, ST_PRODUCER_TIMEOUT = 1, ST_MMA_TIMEOUT = 2, ST_EPILOGUE_TIMEOUT = 3, ST_DRAIN_TIMEOUT = 4 };

// Instruction descriptor of kind::f16: D float32, A and B bf16, both K-major, M = 128, N = TN.
__host__ __device__ constexpr uint32_t make_idesc(int tn) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(tn >> 3) << 17) | ((uint32_t)(BLOCK_F >> 4) << 24);
}

// SiLU without a branch, for results that are rounded to bf16 right away: x / (1 + e^-x).  For very
// negative x the exponential overflows to +inf and the quotient is -0, the limit of the reference's
// x e^x / (1 + e^x) (math.rs:137-146); the fast exponential and division are exact to a few ulp of
// float32, far below bf16's 8 bits.
__device__ __forceinline__ float silu_to_bf16(float x) { return __fdividef(x, 1.f + __expf(-x)); }

template <int MODE>
__device__ __forceinline__ void store_result(void* out_, size_t o, float acc, float bias, float acc2) {
    if (MODE == 0) {
        reinterpret_cast<__nv_bfloat16*>(out_)[o] = __float2bfloat16_rn(acc + bias);
    } else if (MODE == 1) {
        reinterpret_cast<float*>(out_)[o] = acc + bias;
    } else if (MODE == 2) {
        // one add per element and split: a reduction without a return value, so the epilogue never
        // waits on a load
        atomicAdd(reinterpret_cast<float*>(out_) + o, acc);
    } else {
        reinterpret_cast<__nv_bfloat16*>(out_)[o] = __float2bfloat16_rn(silu_to_bf16(acc) * acc2);
    }
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

__host__ __device__ constexpr int tmem_cols(int need) { return need <= 32 ? 32 : need <= 64 ? 64 : need <= 128 ? 128 : need <= 256 ? 256 : 512; }

template <int TN, bool DUAL, int MODE>
__global__ void __launch_bounds__(THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_w2,
               const __grid_constant__ CUtensorMap map_x, const float* __restrict__ bias, void* __restrict__ out_,
               int n_tok, int n_feat, int K, int kb_per_split, int split_k, int stages, int tn, int* status) {
    // TN is the widest token tile this instance holds (shared memory and tensor memory are laid out
    // for it); tn <= TN, a multiple of 16, is the width it runs: the box of map_x has tn rows.
    constexpr int B_BYTES = TN * BLOCK_K * 2;
    constexpr int STAGE_BYTES = (DUAL ? 2 : 1) * A_BYTES + B_BYTES;
    const uint32_t stage_tx = (uint32_t)((DUAL ? 2 : 1) * A_BYTES + tn * BLOCK_K * 2);   // bytes TMA brings per stage
    constexpr int ACC_COLS = DUAL ? 2 * TN : TN;               // columns of one accumulator buffer
    constexpr int TMEM_COLS = tmem_cols(2 * ACC_COLS);         // two buffers: epilogue of a tile overlaps the next main loop
    const uint32_t IDESC = make_idesc(tn);

    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t full_bar[MAX_STAGES];
    __shared__ __align__(8) uint64_t empty_bar[MAX_STAGES];
    __shared__ __align__(8) uint64_t acc_full[2];
    __shared__ __align__(8) uint64_t acc_empty[2];
    __shared__ uint32_t tmem_base_slot;
    __shared__ volatile int abort_flag;

    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;     // swizzled tiles want 1024-byte alignment
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int total_kb = (K + BLOCK_K - 1) / BLOCK_K;
    // Tiles are numbered with the token tile fastest, so that CTAs running together share a weight
    // tile in L2; a CTA takes tiles blockIdx.x, blockIdx.x + gridDim.x, ...
    const int n_tok_tiles = (n_tok + tn - 1) / tn, n_feat_tiles = (n_feat + BLOCK_F - 1) / BLOCK_F;
    const int total_tiles = n_tok_tiles * n_feat_tiles * split_k;
    const int my_tiles = ((int)blockIdx.x < total_tiles) ? (total_tiles - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;

    if (threadIdx.x == 0) {
        for (int s = 0; s < stages; ++s) {
            mbar_init(smem_u32(&full_bar[s]), 1);
            mbar_init(smem_u32(&empty_bar[s]), 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(smem_u32(&acc_full[i]), 1);
            mbar_init(smem_u32(&acc_empty[i]), 4);             // one arrival per epilogue warp
        }
        abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)),
                     "r"((uint32_t)TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_slot;
    const uint32_t full0 = smem_u32(&full_bar[0]), empty0 = smem_u32(&empty_bar[0]);
    let_next_kernel_start();

    // coordinates of the CTA's i-th tile
    auto tile_coords = [&](int i, int& f0, int& t0, int& kb_begin, int& n_kb) {
        const int tile = (int)blockIdx.x + i * (int)gridDim.x;
        const int tt = tile % n_tok_tiles, rest = tile / n_tok_tiles;
        const int ft = rest % n_feat_tiles, sp = rest / n_feat_tiles;
        f0 = ft * BLOCK_F;
        t0 = tt * tn;
        kb_begin = sp * kb_per_split;
        n_kb = min(total_kb, kb_begin + kb_per_split) - kb_begin;          // >= 1 by construction of the split
    };

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            // One thread runs this loop once per k-block, and a lone thread issues a dependent
            // instruction only every few cycles: the ring position and its parity are carried along
            // instead of being divided out of a counter, so that an iteration stays well below the
            // time the tensor core needs for a k-block.
            int it = 0;                      // k-blocks issued so far, over all of this CTA's tiles
            int s = 0;                       // ring position of the next k-block
            uint32_t ph = 0;                 // its pass through the ring, modulo 2
            bool waited = false;             // the activations come from the kernel before: wait once
            bool alive = true;
            for (int i = 0; i < my_tiles && alive; ++i) {
                int f0, t0, kb_begin, n_kb;
                tile_coords(i, f0, t0, kb_begin, n_kb);
                if (abort_flag) break;
                int kb = 0;
                if (!waited) {
                    // The weights are written by no kernel, so their tiles for the first round of stages
                    // go out at once; the activations wait for the previous kernel.
                    const int ahead = min(stages, n_kb);
                    for (int j = 0; j < ahead; ++j) {
                        const uint32_t bar = smem_u32(&full_bar[j]);
                        const uint32_t stage = smem_base + (uint32_t)j * STAGE_BYTES;
                        const int kx = (kb_begin + j) * BLOCK_K;
                        mbar_expect_tx(bar, stage_tx);
                        tma_load_2d(stage, &map_w, bar, kx, f0);
                        if (DUAL) tma_load_2d(stage + A_BYTES, &map_w2, bar, kx, f0);
                    }
                    wait_for_previous_kernels();
                    waited = true;
                    for (int j = 0; j < ahead; ++j)
                        tma_load_2d(smem_base + (uint32_t)j * STAGE_BYTES + (DUAL ? 2 : 1) * A_BYTES, &map_x,
                                    smem_u32(&full_bar[j]), (kb_begin + j) * BLOCK_K, t0);
                    kb = ahead;
                    it = ahead;
                    if (ahead == stages) ph = 1; else s = ahead;
                }
                int kx = (kb_begin + kb) * BLOCK_K;
                for (; kb < n_kb; ++kb, ++it, kx += BLOCK_K) {
                    if (!mbar_wait(empty0 + 8u * s, ph ^ 1u)) {
                        if (!abort_flag) report(status, ST_PRODUCER_TIMEOUT);
                        abort_flag = 1;
                        alive = false;
                        break;
                    }
                    const uint32_t bar = full0 + 8u * s;
                    const uint32_t stage = smem_base + (uint32_t)s * STAGE_BYTES;
                    mbar_expect_tx(bar, stage_tx);
                    tma_load_2d(stage, &map_w, bar, kx, f0);
                    if (DUAL) tma_load_2d(stage + A_BYTES, &map_w2, bar, kx, f0);
                    tma_load_2d(stage + (DUAL ? 2 : 1) * A_BYTES, &map_x, bar, kx, t0);
                    if (++s == stages) { s = 0; ph ^= 1u; }
                }
            }
            // Do not leave while a copy into this CTA's shared memory may still be in flight:
            // the last `stages` loads issued must have landed (immediate on the normal path).
            for (int j = max(0, it - stages); j < it; ++j) {
                if (!mbar_wait(full0 + 8u * (uint32_t)(j % stages), (uint32_t)(j / stages) & 1u)) {
                    report(status, ST_DRAIN_TIMEOUT);
                    break;
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            int s = 0;
            uint32_t ph = 0;
            bool alive = true;
            // descriptors of stage 0; a stage further on adds its byte offset / 16 to the address field
            // (shared memory ends below 256 KiB, so the 14-bit field never carries)
            const uint64_t desc_a0 = make_smem_desc(smem_base);
            const uint64_t desc_b0 = make_smem_desc(smem_base + (DUAL ? 2 : 1) * A_BYTES);
            for (int i = 0; i < my_tiles && alive; ++i) {
                int f0, t0, kb_begin, n_kb;
                tile_coords(i, f0, t0, kb_begin, n_kb);
                const int buf = i & 1;
                // the epilogue must have emptied this accumulator buffer (two tiles ago)
                if (!mbar_wait(smem_u32(&acc_empty[buf]), (uint32_t)((i >> 1) & 1) ^ 1u)) {
                    report(status, ST_MMA_TIMEOUT);
                    abort_flag = 1;
                    break;
                }
                tc_fence_after();
                const uint32_t acc = tmem_base + (uint32_t)(buf * ACC_COLS);
                for (int kb = 0; kb < n_kb; ++kb) {
                    if (!mbar_wait(full0 + 8u * s, ph)) {
                        report(status, ST_MMA_TIMEOUT);
                        abort_flag = 1;
                        alive = false;
                        break;
                    }
                    tc_fence_after();
                    const uint64_t off = (uint64_t)((uint32_t)s * (uint32_t)(STAGE_BYTES >> 4));
                    const uint64_t a0 = desc_a0 + off, b0 = desc_b0 + off;
#pragma unroll
                    for (int k = 0; k < BLOCK_K / 16; ++k) {
                        // 16 bf16 = 32 bytes further along K inside the swizzled row: 2 in the address field
                        umma(acc, a0 + 2 * k, b0 + 2 * k, IDESC, kb > 0 || k > 0);
                        if (DUAL) umma(acc + TN, a0 + (A_BYTES >> 4) + 2 * k, b0 + 2 * k, IDESC, kb > 0 || k > 0);
                    }
                    umma_commit(empty0 + 8u * s);              // frees the stage once these MMAs have read it
                    if (++s == stages) { s = 0; ph ^= 1u; }
                }
                umma_commit(smem_u32(&acc_full[buf]));         // accumulator complete (or aborted: flag says which)
            }
        }
    } else {
        // ---------------- epilogue: warps 2..5 ----------------
        wait_for_previous_kernels();          // `out` may still be read or written by the kernel before
        const int lane_base = (warp & 3) * 32;                 // the TMEM lanes this warp may read
        for (int i = 0; i < my_tiles; ++i) {
            int f0, t0, kb_begin, n_kb;
            tile_coords(i, f0, t0, kb_begin, n_kb);
            const int buf = i & 1;
            const bool landed = mbar_wait(smem_u32(&acc_full[buf]), (uint32_t)((i >> 1) & 1));
            if (!landed && lane == 0) {
                report(status, ST_EPILOGUE_TIMEOUT);
                abort_flag = 1;
            }
            tc_fence_after();
            if (!landed || abort_flag) break;
            const int f = f0 + lane_base + lane;
            const bool f_ok = f < n_feat;
            const float b = (bias != nullptr && f_ok) ? bias[f] : 0.f;
            const uint32_t trow = tmem_base + ((uint32_t)lane_base << 16) + (uint32_t)(buf * ACC_COLS);
#pragma unroll 1
            for (int c0 = 0; c0 < tn; c0 += 16) {
                if (t0 + c0 >= n_tok) break;                   // uniform over the warp
                uint32_t v[16], u[16];
                tmem_ld16(trow + c0, v);
                if (DUAL) tmem_ld16(trow + TN + c0, u);
                tmem_wait_ld();
                if (f_ok) {
                    // a group of 16 tokens that lies inside the matrix runs without per-token branches,
                    // so the 16 independent chains interleave; the ragged last group takes the checked path
                    const bool whole = t0 + c0 + 16 <= n_tok;
                    const size_t o0 = (size_t)(t0 + c0) * n_feat + f;
                    if (whole) {
#pragma unroll
                        for (int j = 0; j < 16; ++j)
                            store_result<MODE>(out_, o0 + (size_t)j * n_feat, __uint_as_float(v[j]), b,
                                               DUAL ? __uint_as_float(u[j]) : 0.f);
                    } else {
                        for (int j = 0; j < 16; ++j)
                            if (t0 + c0 + j < n_tok)
                                store_result<MODE>(out_, o0 + (size_t)j * n_feat, __uint_as_float(v[j]), b,
                                                   DUAL ? __uint_as_float(u[j]) : 0.f);
                    }
                }
            }
            // this warp has read its part of the buffer: hand it back to the MMA issuer
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&acc_empty[buf]));
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)TMEM_COLS)
                     : "memory");
    }
}

// ---------------------------------------------------------------------------------------------
// The token-major orientation, for steps of more than 128 tokens (prompts).
//
// Here the MMA's M dimension runs over 128 tokens (rows of X, the A operand) and its N dimension
// over 256 rows of W (the B operand): 256 features, or, for the SiLU-gate epilogue, 128 gate rows
// stacked on the 128 up rows of the same features, so that one MMA per K-slice feeds both and a
// token's gate and up values sit in the same TMEM lane.  Against the feature-major kernel with two
// N = 128 MMAs per K-slice this reads 25% fewer operand bytes from shared memory per MAC (the main
// loop of that shape sat at the 128 B/clk shared-memory limit), and every epilogue thread owns a
// token and writes runs of 16 consecutive features with 16-byte stores.
// Same ring, same persistent grid, same two accumulator buffers.
// ---------------------------------------------------------------------------------------------
constexpr int TM_TOK = 128;                         // tokens per tile (MMA M)
constexpr int TM_ROWS = 256;                        // rows of W per tile (MMA N)
constexpr int TM_STAGE_BYTES = (TM_TOK + TM_ROWS) * BLOCK_K * 2;     // 48 KiB

template <bool DUAL, int MODE>
__global__ void __launch_bounds__(THREADS, 1)
gemm_tm_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_w2,
               const __grid_constant__ CUtensorMap map_x, const float* __restrict__ bias, void* __restrict__ out_,
               int n_tok, int n_feat, int K, int stages, int* status) {
    constexpr int FEATS = DUAL ? TM_ROWS / 2 : TM_ROWS;        // output features per tile
    constexpr int X_BYTES = TM_TOK * BLOCK_K * 2;
    constexpr int TMEM_COLS = 2 * TM_ROWS;                     // two accumulator buffers
    constexpr uint32_t IDESC = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(TM_ROWS >> 3) << 17) |
                               ((uint32_t)(TM_TOK >> 4) << 24);

    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t full_bar[MAX_STAGES];
    __shared__ __align__(8) uint64_t empty_bar[MAX_STAGES];
    __shared__ __align__(8) uint64_t acc_full[2];
    __shared__ __align__(8) uint64_t acc_empty[2];
    __shared__ uint32_t tmem_base_slot;
    __shared__ volatile int abort_flag;

    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n_kb = (K + BLOCK_K - 1) / BLOCK_K;
    const int n_tok_tiles = (n_tok + TM_TOK - 1) / TM_TOK, n_feat_tiles = (n_feat + FEATS - 1) / FEATS;
    const int total_tiles = n_tok_tiles * n_feat_tiles;
    const int my_tiles = ((int)blockIdx.x < total_tiles) ? (total_tiles - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;

    if (threadIdx.x == 0) {
        for (int s = 0; s < stages; ++s) {
            mbar_init(smem_u32(&full_bar[s]), 1);
            mbar_init(smem_u32(&empty_bar[s]), 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(smem_u32(&acc_full[i]), 1);
            mbar_init(smem_u32(&acc_empty[i]), 4);
        }
        abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)),
                     "r"((uint32_t)TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_slot;
    const uint32_t full0 = smem_u32(&full_bar[0]), empty0 = smem_u32(&empty_bar[0]);
    let_next_kernel_start();

    // token tiles vary fastest, so CTAs that run together share the weight rows in L2
    auto tile_coords = [&](int i, int& f0, int& t0) {
        const int tile = (int)blockIdx.x + i * (int)gridDim.x;
        t0 = (tile % n_tok_tiles) * TM_TOK;
        f0 = (tile / n_tok_tiles) * FEATS;
    };
    // the W rows of one stage: 256 features, or 128 gate rows then the 128 up rows of the same features
    auto load_w = [&](uint32_t stage, uint32_t bar, int kx, int f0) {
        tma_load_2d(stage + X_BYTES, &map_w, bar, kx, f0);
        if (DUAL) tma_load_2d(stage + X_BYTES + A_BYTES, &map_w2, bar, kx, f0);
        else tma_load_2d(stage + X_BYTES + A_BYTES, &map_w, bar, kx, f0 + BLOCK_F);
    };


    if (warp == 0) {
        if (lane == 0) {
            int it = 0, s = 0;               // k-blocks issued; ring position and pass parity, carried along
            uint32_t ph = 0;
            bool waited = false, alive = true;
            for (int i = 0; i < my_tiles && alive; ++i) {
                int f0, t0;
                tile_coords(i, f0, t0);
                if (abort_flag) break;
                int kb = 0;
                if (!waited) {
                    const int ahead = min(stages, n_kb);
                    for (int j = 0; j < ahead; ++j) {            // weights first: no kernel writes them
                        const uint32_t bar = smem_u32(&full_bar[j]);
                        mbar_expect_tx(bar, TM_STAGE_BYTES);
                        load_w(smem_base + (uint32_t)j * TM_STAGE_BYTES, bar, j * BLOCK_K, f0);
                    }
                    wait_for_previous_kernels();                 // the activations come from the kernel before
                    waited = true;
                    for (int j = 0; j < ahead; ++j)
                        tma_load_2d(smem_base + (uint32_t)j * TM_STAGE_BYTES, &map_x, smem_u32(&full_bar[j]), j * BLOCK_K, t0);
                    kb = ahead;
                    it = ahead;
                    if (ahead == stages) ph = 1; else s = ahead;
                }
                for (; kb < n_kb; ++kb, ++it) {
                    if (!mbar_wait(empty0 + 8u * s, ph ^ 1u)) {
                        if (!abort_flag) report(status, ST_PRODUCER_TIMEOUT);
                        abort_flag = 1;
                        alive = false;
                        break;
                    }
                    const uint32_t bar = full0 + 8u * s;
                    const uint32_t stage = smem_base + (uint32_t)s * TM_STAGE_BYTES;
                    mbar_expect_tx(bar, TM_STAGE_BYTES);
                    load_w(stage, bar, kb * BLOCK_K, f0);
                    tma_load_2d(stage, &map_x, bar, kb * BLOCK_K, t0);
                    if (++s == stages) { s = 0; ph ^= 1u; }
                }
            }
            for (int j = max(0, it - stages); j < it; ++j)
                if (!mbar_wait(smem_u32(&full_bar[j % stages]), (uint32_t)(j / stages) & 1u)) {
                    report(status, ST_DRAIN_TIMEOUT);
                    break;
                }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            int s = 0;
            uint32_t ph = 0;
            bool alive = true;
            const uint64_t desc_x0 = make_smem_desc(smem_base), desc_w0 = make_smem_desc(smem_base + X_BYTES);
            for (int i = 0; i < my_tiles && alive; ++i) {
                const int buf = i & 1;
                if (!mbar_wait(smem_u32(&acc_empty[buf]), ((uint32_t)(i >> 1) & 1u) ^ 1u)) {
                    report(status, ST_MMA_TIMEOUT);
                    abort_flag = 1;
                    break;
                }
                tc_fence_after();
                const uint32_t acc = tmem_base + (uint32_t)(buf * TM_ROWS);
                for (int kb = 0; kb < n_kb; ++kb) {
                    if (!mbar_wait(full0 + 8u * s, ph)) {
                        report(status, ST_MMA_TIMEOUT);
                        abort_flag = 1;
                        alive = false;
                        break;
                    }
                    tc_fence_after();
                    const uint64_t off = (uint64_t)((uint32_t)s * (uint32_t)(TM_STAGE_BYTES >> 4));
#pragma unroll
                    for (int k = 0; k < BLOCK_K / 16; ++k)
                        umma(acc, desc_x0 + off + 2 * k, desc_w0 + off + 2 * k, IDESC, kb > 0 || k > 0);
                    umma_commit(empty0 + 8u * s);
                    if (++s == stages) { s = 0; ph ^= 1u; }
                }
                umma_commit(smem_u32(&acc_full[buf]));
            }
        }
    } else {
        // ---------------- epilogue: a thread owns a token, writes runs of 16 features ----------------
        wait_for_previous_kernels();
        const int lane_base = (warp & 3) * 32;
        const bool aligned = n_feat % 8 == 0;                      // rows of `out` keep 16-byte alignment
        for (int i = 0; i < my_tiles; ++i) {
            int f0, t0;
            tile_coords(i, f0, t0);
            const int buf = i & 1;
            const bool landed = mbar_wait(smem_u32(&acc_full[buf]), (uint32_t)(i >> 1) & 1u);
            if (!landed && lane == 0) {
                report(status, ST_EPILOGUE_TIMEOUT);
                abort_flag = 1;
            }
            tc_fence_after();
            if (!landed || abort_flag) break;
            const int t = t0 + lane_base + lane;
            const bool t_ok = t < n_tok;
            const uint32_t trow = tmem_base + ((uint32_t)lane_base << 16) + (uint32_t)(buf * TM_ROWS);
#pragma unroll 1
            for (int c0 = 0; c0 < FEATS; c0 += 16) {
                if (f0 + c0 >= n_feat) break;                       // uniform over the warp
                uint32_t v[16], u[16];
                tmem_ld16(trow + c0, v);
                if (DUAL) tmem_ld16(trow + TM_ROWS / 2 + c0, u);
                tmem_wait_ld();
                if (!t_ok) continue;
                const size_t o0 = (size_t)t * n_feat + f0 + c0;
                const bool whole = aligned && f0 + c0 + 16 <= n_feat;
                float r[16];
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    const float a = __uint_as_float(v[j]);
                    if (MODE == 3) r[j] = silu_to_bf16(a) * __uint_as_float(u[j]);
                    else if (MODE == 2) r[j] = a;
                    else r[j] = a + ((bias != nullptr && f0 + c0 + j < n_feat) ? bias[f0 + c0 + j] : 0.f);
                }
                if (whole) {
                    if (MODE == 0 || MODE == 3) {
                        __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(out_) + o0;
                        uint4 lo, hi;
                        lo.x = pack_bf16x2(r[0], r[1]);  lo.y = pack_bf16x2(r[2], r[3]);
                        lo.z = pack_bf16x2(r[4], r[5]);  lo.w = pack_bf16x2(r[6], r[7]);
                        hi.x = pack_bf16x2(r[8], r[9]);  hi.y = pack_bf16x2(r[10], r[11]);
                        hi.z = pack_bf16x2(r[12], r[13]); hi.w = pack_bf16x2(r[14], r[15]);
                        *reinterpret_cast<uint4*>(dst) = lo;
                        *reinterpret_cast<uint4*>(dst + 8) = hi;
                    } else {
                        float4* dst = reinterpret_cast<float4*>(reinterpret_cast<float*>(out_) + o0);
#pragma unroll
                        for (int q4 = 0; q4 < 4; ++q4) {
                            float4 x = make_float4(r[4 * q4], r[4 * q4 + 1], r[4 * q4 + 2], r[4 * q4 + 3]);
                            if (MODE == 2) {                     // K is not split here: a plain read-add-write
                                const float4 old = dst[q4];
                                x.x += old.x; x.y += old.y; x.z += old.z; x.w += old.w;
                            }
                            dst[q4] = x;
                        }
                    }
                } else {
                    for (int j = 0; j < 16; ++j)
                        if (f0 + c0 + j < n_feat) {
                            if (MODE == 0 || MODE == 3) reinterpret_cast<__nv_bfloat16*>(out_)[o0 + j] = __float2bfloat16_rn(r[j]);
                            else if (MODE == 1) reinterpret_cast<float*>(out_)[o0 + j] = r[j];
                            else reinterpret_cast<float*>(out_)[o0 + j] += r[j];
                        }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&acc_empty[buf]));
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)TMEM_COLS)
                     : "memory");
    }
}

// ---------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------
// A bf16 matrix [rows, K] row-major as a 2-D tensor map with a {64, box_rows} box, 128-byte swizzle,
// zero fill outside the tensor.
int make_map(CUtensorMap* map, const void* ptr, long long rows, long long K, int box_rows, const char* what) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return fail("gemm_tcgen05: cuTensorMapEncodeTiled is not available from the driver");
    if ((uintptr_t)ptr % 16) return fail("gemm_tcgen05: %s is not 16-byte aligned", what);
    cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)K * 2};
    cuuint32_t box[2] = {(cuuint32_t)BLOCK_K, (cuuint32_t)box_rows};
    cuuint32_t elem[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, elem,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail("gemm_tcgen05: cuTensorMapEncodeTiled failed for %s (code %d)", what, (int)r);
    return 0;
}

int sm_count() {
    static int n = 0;
    if (n == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    }
    return n;
}

int g_smem_budget = 0;       // 0: the default for the tile; set through ri_gemm_tcgen05_set_smem_budget

template <int TN, bool DUAL, int MODE>
int launch(int tn, const CUtensorMap& mw, const CUtensorMap& mw2, const CUtensorMap& mx, const float* bias, void* out,
           int n_tok, int n_feat, int K, int split_k, int* status, cudaStream_t stream) {
    constexpr int STAGE_BYTES = (DUAL ? 2 : 1) * A_BYTES + TN * BLOCK_K * 2;
    const int total_kb = (K + BLOCK_K - 1) / BLOCK_K;
    // Small token tiles (decode) leave room for a second CTA on the SM, so that the next kernel's
    // CTAs can settle in and prefetch their weights while this one drains.
    int budget = g_smem_budget > 0 ? g_smem_budget : (3 * STAGE_BYTES <= 108 * 1024 && TN <= 64 ? 108 * 1024 : SMEM_BUDGET);
    if (budget > SMEM_BUDGET) budget = SMEM_BUDGET;
    int stages = budget / STAGE_BYTES;
    if (stages > MAX_STAGES) stages = MAX_STAGES;
    if (stages > total_kb) stages = total_kb;
    if (stages < 1) stages = 1;
    const size_t smem = (size_t)stages * STAGE_BYTES + 1024;
    if (split_k < 1) split_k = 1;
    if (split_k > total_kb) split_k = total_kb;
    int kb_per_split = (total_kb + split_k - 1) / split_k;
    split_k = (total_kb + kb_per_split - 1) / kb_per_split;          // no empty split
    auto kernel = gemm_tc_kernel<TN, DUAL, MODE>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BUDGET + 1024);
        if (e != cudaSuccess) return fail("gemm_tcgen05: cannot raise dynamic shared memory: %s", cudaGetErrorString(e));
        configured = true;
    }
    const long long total_tiles = (long long)((n_tok + tn - 1) / tn) * ((n_feat + BLOCK_F - 1) / BLOCK_F) * split_k;
    if (total_tiles > 0x7fffffffLL) return fail("gemm_tcgen05: %lld tiles exceed the index range", total_tiles);
    // a persistent grid: as many CTAs as fit the GPU at once (two per SM when the ring is small and
    // two accumulator buffers of each fit tensor memory), each walking its share of the tiles
    constexpr int ACC_COLS = DUAL ? 2 * TN : TN;
    const int per_sm = (smem <= 110 * 1024 && 4 * ACC_COLS <= 512) ? 2 : 1;
    long long ctas = (long long)sm_count() * per_sm;
    if (ctas > total_tiles) ctas = total_tiles;
    dim3 grid((unsigned)ctas);
    cudaError_t e = launch_dependent(kernel, grid, dim3(THREADS), smem, stream, mw, mw2, mx, bias, out, n_tok, n_feat, K,
                                     kb_per_split, split_k, stages, tn, status);
    return check_launch(e, "gemm_tcgen05");
}

template <bool DUAL, int MODE>
int launch_tm(const CUtensorMap& mw, const CUtensorMap& mw2, const CUtensorMap& mx, const float* bias, void* out,
              int n_tok, int n_feat, int K, int* status, cudaStream_t stream) {
    const int total_kb = (K + BLOCK_K - 1) / BLOCK_K;
    int stages = SMEM_BUDGET / TM_STAGE_BYTES;
    if (stages > total_kb) stages = total_kb;
    const size_t smem = (size_t)stages * TM_STAGE_BYTES + 1024;
    auto kernel = gemm_tm_kernel<DUAL, MODE>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BUDGET + 1024);
        if (e != cudaSuccess) return fail("gemm_tcgen05: cannot raise dynamic shared memory: %s", cudaGetErrorString(e));
        configured = true;
    }
    constexpr int FEATS = DUAL ? TM_ROWS / 2 : TM_ROWS;
    const long long total_tiles = (long long)((n_tok + TM_TOK - 1) / TM_TOK) * ((n_feat + FEATS - 1) / FEATS);
    if (total_tiles > 0x7fffffffLL) return fail("gemm_tcgen05: %lld tiles exceed the index range", total_tiles);
    long long ctas = sm_count();
    if (ctas > total_tiles) ctas = total_tiles;
    cudaError_t e = launch_dependent(kernel, dim3((unsigned)ctas), dim3(THREADS), smem, stream, mw, mw2, mx, bias, out,
                                     n_tok, n_feat, K, stages, status);
    return check_launch(e, "gemm_tcgen05 (token-major)");
}

template <bool DUAL, int MODE>
int pick_tile(int tn, const CUtensorMap& mw, const CUtensorMap& mw2, const CUtensorMap& mx, const float* bias,
              void* out, int n_tok, int n_feat, int K, int split_k, int* status, cudaStream_t stream) {
    // the narrowest compiled instance that holds a tile of tn tokens
    if (tn < 16 || tn > 256 || tn % 16) return fail("gemm_tcgen05: no tile of %d tokens", tn);
    if (tn <= 16) return launch<16, DUAL, MODE>(tn, mw, mw2, mx, bias, out, n_tok, n_feat, K, split_k, status, stream);
    if (tn <= 32) return launch<32, DUAL, MODE>(tn, mw, mw2, mx, bias, out, n_tok, n_feat, K, split_k, status, stream);
    if (tn <= 64) return launch<64, DUAL, MODE>(tn, mw, mw2, mx, bias, out, n_tok, n_feat, K, split_k, status, stream);
    if (tn <= 128) return launch<128, DUAL, MODE>(tn, mw, mw2, mx, bias, out, n_tok, n_feat, K, split_k, status, stream);
    if constexpr (!DUAL)
        return launch<256, DUAL, MODE>(tn, mw, mw2, mx, bias, out, n_tok, n_feat, K, split_k, status, stream);
    return fail("gemm_tcgen05: the SiLU-gate epilogue has no tile of %d tokens", tn);
}

}  // namespace

// Shared memory a CTA may use for its stage ring, in bytes (0 restores the defaults).  For tuning.
RI_API int ri_gemm_tcgen05_set_smem_budget(int bytes) {
    g_smem_budget = bytes;
    return 0;
}

int g_long_tile = 0;         // 0: pick by the grid; set through ri_gemm_tcgen05_set_long_tile

// Token tile of steps of more than 128 tokens in the feature-major kernel: a multiple of 16 in
// 128..256, or 0 to let the grid decide.  For tuning.
RI_API int ri_gemm_tcgen05_set_long_tile(int tn) {
    if (tn != 0 && (tn < 128 || tn > 256 || tn % 16)) return fail("gemm_tcgen05: no long tile of %d tokens", tn);
    g_long_tile = tn;
    return 0;
}

// How a product of n_tok tokens, n_feat features and inner size K is cut: the token tile (rows of the
// activation box, written to *tile) and, for the residual epilogue (mode 2, the only one that can
// add partial sums), over how many pieces K is split (*split; 1 for the other modes).
//
//  up to 128 tokens   one token tile, as narrow as the step allows.  Such steps stream weights:
//                     measured in a replayed graph at 8 tokens, the o, q/k/v and down projections of
//                     a 3584-wide model are fastest with about two CTAs per SM (7-10 pieces) and at
//                     least 4 k-blocks per piece (more for wider steps, whose pieces end in more atomics).
//  beyond, SiLU-gate  the token-major kernel, 128 tokens per tile.
//  beyond, others     the feature-major kernel.  Measured at 192..4,096 tokens: a k-block takes about
//                     as long whatever the tile's width (128..256), so what counts is how many rounds
//                     the persistent grid makes and how long a work item's K run is.  Every width of
//                     128..256 and every split is tried on depth x (k-blocks per item + a dozen for
//                     the item's epilogue and ramp); ties go to the narrower tile.  (Down projection
//                     of 512 tokens: 256 x 5 pieces, 63.5 us, against 128 x 2, 100 us.)
RI_API int ri_gemm_tcgen05_plan(int n_tok, int n_feat, int K, int mode, int* tile, int* split) {
    const long long feat_tiles = (n_feat + BLOCK_F - 1) / BLOCK_F;
    const long long ctas = sm_count();
    const int total_kb = (K + BLOCK_K - 1) / BLOCK_K;
    const bool can_split = mode == 2;
    int tn = 16, sp = 1;
    if (n_tok <= 128) {
        tn = n_tok <= 16 ? 16 : (n_tok + 15) / 16 * 16;
        if (can_split && feat_tiles < ctas) {
            // every piece ends in tn x 128 atomic adds, so wider steps want longer pieces: at least a tenth of
            // the tile's width in k-blocks (128 tokens, K = 3584: 4-5 pieces, 11 us, against 10 pieces, 13 us)
            const int min_kb = tn / 10 > 4 ? (tn + 9) / 10 : 4;
            long long want = (2 * ctas) / feat_tiles;
            if (want > total_kb / min_kb) want = total_kb / min_kb;
            sp = want < 1 ? 1 : (int)want;
        }
    } else if (mode == 3) {
        tn = 128;
    } else {
        constexpr long long ITEM_OVERHEAD = 12;               // in k-blocks
        long long best_cost = -1;
        const int max_split = can_split ? (total_kb / 4 < 10 ? (total_kb / 4 < 1 ? 1 : total_kb / 4) : 10) : 1;
        for (int t = 128; t <= 256; t += 16) {
            if (g_long_tile && t != g_long_tile) continue;
            const long long tiles = (long long)((n_tok + t - 1) / t) * feat_tiles;
            for (int s = 1; s <= max_split; ++s) {
                const long long items = tiles * s;
                const long long cost = ((items + ctas - 1) / ctas) * ((total_kb + s - 1) / s + ITEM_OVERHEAD);
                if (best_cost < 0 || cost < best_cost) {
                    best_cost = cost;
                    tn = t;
                    sp = s;
                }
            }
        }
    }
    if (tile) *tile = tn;
    if (split) *split = sp;
    return 0;
}

// Encode the tensor map of a bf16 matrix [rows, K] (row-major, 16-byte aligned, K a multiple of 8)
// into the 128 bytes at `map_out` (64-byte aligned).  box_rows is 128 for a weight matrix and the
// token tile (ri_gemm_tcgen05_plan, for the same sizes and mode as the product) for activations.  Maps only depend on pointer and shape, so the
// caller keeps them: weights encode once, activation buffers once per shape.
RI_API int ri_gemm_tcgen05_encode(void* map_out, const void* ptr, long long rows, long long K, int box_rows) {
    if ((uintptr_t)map_out % 64) return fail("gemm_tcgen05: tensor map storage must be 64-byte aligned");
    if (K <= 0 || K % 8) return fail("gemm_tcgen05: K = %lld must be a positive multiple of 8 (16-byte rows for TMA)", K);
    if (box_rows < 8 || box_rows > 256) return fail("gemm_tcgen05: box of %d rows", box_rows);
    return make_map(reinterpret_cast<CUtensorMap*>(map_out), ptr, rows, K, box_rows, "matrix");
}

// X [n_tok, K] with map_x (box rows = the token tile of ri_gemm_tcgen05_plan), W (and W2) [n_feat, K] with
// map_w / map_w2 (box rows 128).  split_k 0 takes the plan's split.  `status` (may be null) is a host-visible int that receives a non-zero code if a wait ran out.
RI_API int ri_gemm_tcgen05(const void* map_x, const void* map_w, const void* map_w2, const float* bias, void* out,
                           int mode, int n_tok, int n_feat, int K, int split_k, int* status, cudaStream_t stream) {
    if (n_tok <= 0 || n_feat <= 0) return 0;
    if (K <= 0 || K % 8) return fail("gemm_tcgen05: K = %d must be a positive multiple of 8 (16-byte rows for TMA)", K);
    if (mode < 0 || mode > 3) return fail("gemm_tcgen05: unknown epilogue mode %d", mode);
    if (mode == 3 && map_w2 == nullptr) return fail("gemm_tcgen05: the SiLU-gate epilogue needs a second matrix");
    if (mode == 2 && bias != nullptr) return fail("gemm_tcgen05: the residual epilogue takes no bias");
    if (mode != 2 && split_k > 1) return fail("gemm_tcgen05: only the residual epilogue can split K");
    const bool dual = mode == 3;
    int tn = 0, planned_split = 1;
    ri_gemm_tcgen05_plan(n_tok, n_feat, K, mode, &tn, &planned_split);
    if (split_k <= 0) split_k = planned_split;
    const CUtensorMap& mw = *reinterpret_cast<const CUtensorMap*>(map_w);
    const CUtensorMap& mw2 = dual ? *reinterpret_cast<const CUtensorMap*>(map_w2) : mw;
    const CUtensorMap& mx = *reinterpret_cast<const CUtensorMap*>(map_x);
    // Measured at 2,048 tokens of a 3584-wide model: the SiLU-gate projection runs at 1,334 TFLOP/s
    // token-major against 1,145 feature-major; q/k/v, o and down are 3-12% faster feature-major.
    if (dual && n_tok > TM_TOK) return launch_tm<true, 3>(mw, mw2, mx, bias, out, n_tok, n_feat, K, status, stream);
    switch (mode) {
        case 0: return pick_tile<false, 0>(tn, mw, mw2, mx, bias, out, n_tok, n_feat, K, split_k, status, stream);
        case 1: return pick_tile<false, 1>(tn, mw, mw2, mx, bias, out, n_tok, n_feat, K, split_k, status, stream);
        case 2: return pick_tile<false, 2>(tn, mw, mw2, mx, bias, out, n_tok, n_feat, K, split_k, status, stream);
        default: return pick_tile<true, 3>(tn, mw, mw2, mx, bias, out, n_tok, n_feat, K, split_k, status, stream);
    }
}

RI_DEFINE_LAST_ERROR()
