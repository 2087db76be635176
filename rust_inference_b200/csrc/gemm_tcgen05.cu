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
// tokens takes the token-major kernel further down (128 tokens x 256 weight rows per tile), and long steps
// whose tiles fill the grid run token-major on pairs of SMs (tcgen05 cta_group::2, at the end of the device code).
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
    RI_PHASE_LATEST(5);
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

// The token-major epilogue of one tile: the thread's token (TMEM lane) times the tile's features, 16 at a time
// from the accumulator at `trow` (SiLU-gate: gate values in the first 128 columns, up values in the second).
template <bool DUAL, int MODE>
__device__ __forceinline__ void tm_write_tile(uint32_t trow, int t, bool t_ok, int f0, int n_feat, bool aligned,
                                              const float* __restrict__ bias, void* __restrict__ out_,
                                              bool pieces = false) {     // MODE 2: other work items add to the same tile
    constexpr int FEATS = DUAL ? TM_ROWS / 2 : TM_ROWS;
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
                    if (MODE == 2 && pieces) {           // four adds in one reduction, no value returned
                        asm volatile("red.relaxed.gpu.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst + q4), "f"(x.x),
                                     "f"(x.y), "f"(x.z), "f"(x.w) : "memory");
                        continue;
                    }
                    if (MODE == 2) {                     // K is not split: a plain read-add-write
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
                    else if (pieces) atomicAdd(reinterpret_cast<float*>(out_) + o0 + j, r[j]);
                    else reinterpret_cast<float*>(out_)[o0 + j] += r[j];
                }
        }
    }
}

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
            tm_write_tile<DUAL, MODE>(trow, t, t_ok, f0, n_feat, aligned, bias, out_);
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
// The token-major product on pairs of SMs (tcgen05 cta_group::2), for long steps.
//
// Two CTAs of a cluster share one MMA of M = 256 tokens x N = 256 rows of W: each CTA holds 128 of
// the tokens (its half of A, and its half of the accumulator in its own tensor memory) and 128 of the
// W rows (its half of B; the tensor cores read the other half from the partner's shared memory).  A
// CTA so brings 32 KiB per k-block from L2 instead of 48 for the same 128 x 256 x 64 multiply-adds,
// which is what long steps are bound by (asking tiles into L2 ahead of time made them slower, not
// faster), and its ring holds six stages instead of four.  For the SiLU-gate projection the first CTA
// loads the gate rows and the second the up rows of the same 128 features.
//
// The first CTA of the pair issues the MMAs.  Both CTAs' TMA loads report to its `full` barrier; its
// commits arrive at the `empty` and `acc_full` barriers of both (multicast); the epilogue warps of both
// arrive at its `acc_empty` barrier.  Tensor memory is allocated and freed by both, as a pair.
// ---------------------------------------------------------------------------------------------
constexpr int PAIR_STAGE_BYTES = 2 * A_BYTES;       // 128 tokens + 128 W rows per CTA and k-block: 32 KiB
constexpr int PAIR_TOK = 2 * TM_TOK;                // tokens per pair tile

__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// The address, in the cluster's shared window, of the first CTA's copy of a shared variable of this CTA.
__device__ __forceinline__ uint32_t in_first_cta(uint32_t local_addr) {
    uint32_t a;
    asm volatile("mapa.shared::cluster.u32 %0, %1, 0;" : "=r"(a) : "r"(local_addr));
    return a;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// A tile into this CTA's shared memory whose arrival is counted by a barrier of the pair's first CTA.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, uint32_t cluster_bar, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(map), "r"(cluster_bar), "r"(x), "r"(y)
        : "memory");
}
__device__ __forceinline__ void umma_pair(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, bool accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"((uint32_t)accumulate)
        : "memory");
}
// Arrives at the barrier at this address in both CTAs of the pair once the MMAs issued so far are done.
__device__ __forceinline__ void umma_commit_pair(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(bar), "h"((uint16_t)3) : "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_bar) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_bar) : "memory");
}

template <bool DUAL, int MODE>
__global__ void __launch_bounds__(THREADS, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_w2,
                 const __grid_constant__ CUtensorMap map_x, const float* __restrict__ bias, void* __restrict__ out_,
                 int n_tok, int n_feat, int K, int kb_per_split, int split_k, int stages, int* status) {
    constexpr int FEATS = DUAL ? TM_ROWS / 2 : TM_ROWS;        // output features per tile
    constexpr int TMEM_COLS = 2 * TM_ROWS;                     // two accumulator buffers
    // D float32, A and B bf16, both K-major, N = 256, M = 256 over the pair
    constexpr uint32_t IDESC = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(TM_ROWS >> 3) << 17) |
                               ((uint32_t)(PAIR_TOK >> 4) << 24);

    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t full_bar[MAX_STAGES];     // used in the first CTA only
    __shared__ __align__(8) uint64_t empty_bar[MAX_STAGES];
    __shared__ __align__(8) uint64_t acc_full[2];
    __shared__ __align__(8) uint64_t acc_empty[2];             // used in the first CTA only
    __shared__ uint32_t tmem_base_slot;
    __shared__ volatile int abort_flag;

    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int rank = (int)cluster_rank();                      // 0: issues the MMAs
    const int pair = (int)blockIdx.x >> 1, n_pairs = (int)gridDim.x >> 1;
    const int n_kb = (K + BLOCK_K - 1) / BLOCK_K;
    const int n_tok_tiles = (n_tok + PAIR_TOK - 1) / PAIR_TOK, n_feat_tiles = (n_feat + FEATS - 1) / FEATS;
    const int total_tiles = n_tok_tiles * n_feat_tiles * split_k;            // work items: tiles x pieces of K
    const int my_tiles = (pair < total_tiles) ? (total_tiles - 1 - pair) / n_pairs + 1 : 0;

    if (threadIdx.x == 0) {
        for (int s = 0; s < stages; ++s) {
            mbar_init(smem_u32(&full_bar[s]), 1);
            mbar_init(smem_u32(&empty_bar[s]), 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(smem_u32(&acc_full[i]), 1);
            mbar_init(smem_u32(&acc_empty[i]), 8);             // one arrival per epilogue warp of the pair
        }
        abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)),
                     "r"((uint32_t)TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    cluster_sync_all();                                        // the partner's barriers stand before anything arrives there
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_slot;
    const uint32_t full0 = smem_u32(&full_bar[0]), empty0 = smem_u32(&empty_bar[0]);
    const uint32_t full0_first = in_first_cta(full0);
    let_next_kernel_start();

    // token tiles vary fastest, so pairs that run together share the weight rows in L2
    auto tile_coords = [&](int i, int& f0, int& t0, int& kb_begin, int& kb_end) {
        const int item = pair + i * n_pairs;
        const int rest = item / n_tok_tiles, sp = rest / n_feat_tiles;
        t0 = (item - rest * n_tok_tiles) * PAIR_TOK;
        f0 = (rest - sp * n_feat_tiles) * FEATS;
        kb_begin = sp * kb_per_split;
        kb_end = min(n_kb, kb_begin + kb_per_split);             // > kb_begin by construction of the split
    };

    if (warp == 0) {
        // ---------------- TMA producer (both CTAs) ----------------
        if (lane == 0) {
            int it = 0, s = 0;
            uint32_t ph = 0;
            bool alive = true;
            wait_for_previous_kernels();                         // the activations come from the kernel before
            // this CTA's half of the W rows: gate (first CTA) or up (second) rows of the tile's features, or the
            // first or second 128 of its 256 features
            const CUtensorMap* my_w = (DUAL && rank == 1) ? &map_w2 : &map_w;
            const int w_off = DUAL ? 0 : rank * BLOCK_F;
            for (int i = 0; i < my_tiles && alive; ++i) {
                int f0, t0, kb_begin, kb_end;
                tile_coords(i, f0, t0, kb_begin, kb_end);
                if (abort_flag) break;
                for (int kb = kb_begin; kb < kb_end; ++kb, ++it) {
                    if (!mbar_wait(empty0 + 8u * s, ph ^ 1u)) {
                        if (!abort_flag) report(status, ST_PRODUCER_TIMEOUT);
                        abort_flag = 1;
                        alive = false;
                        break;
                    }
                    const uint32_t stage = smem_base + (uint32_t)s * PAIR_STAGE_BYTES;
                    if (rank == 0) mbar_expect_tx(full0 + 8u * s, 2 * PAIR_STAGE_BYTES);       // both CTAs' bytes
                    tma_load_2d_pair(stage, &map_x, full0_first + 8u * s, kb * BLOCK_K, t0 + rank * TM_TOK);
                    tma_load_2d_pair(stage + A_BYTES, my_w, full0_first + 8u * s, kb * BLOCK_K, f0 + w_off);
                    if (++s == stages) { s = 0; ph ^= 1u; }
                }
            }
            // Do not leave while a copy into this CTA's shared memory may still be in flight: a stage whose
            // `empty` barrier has completed again was read by the MMAs, so its copy had landed.
            for (int j = 0; j < stages && it > 0; ++j) {
                if (!mbar_wait(empty0 + 8u * s, ph ^ 1u)) {
                    report(status, ST_DRAIN_TIMEOUT);
                    break;
                }
                if (++s == stages) { s = 0; ph ^= 1u; }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer (first CTA) ----------------
        if (lane == 0 && rank == 0) {
            int s = 0;
            uint32_t ph = 0;
            bool alive = true;
            const uint64_t desc_x0 = make_smem_desc(smem_base), desc_w0 = make_smem_desc(smem_base + A_BYTES);
            for (int i = 0; i < my_tiles && alive; ++i) {
                int f0, t0, kb_begin, kb_end;
                tile_coords(i, f0, t0, kb_begin, kb_end);
                const int buf = i & 1;
                if (!mbar_wait(smem_u32(&acc_empty[buf]), ((uint32_t)(i >> 1) & 1u) ^ 1u)) {
                    report(status, ST_MMA_TIMEOUT);
                    abort_flag = 1;
                    break;
                }
                tc_fence_after();
                const uint32_t acc = tmem_base + (uint32_t)(buf * TM_ROWS);
                for (int kb = kb_begin; kb < kb_end; ++kb) {
                    if (!mbar_wait(full0 + 8u * s, ph)) {
                        report(status, ST_MMA_TIMEOUT);
                        abort_flag = 1;
                        alive = false;
                        break;
                    }
                    tc_fence_after();
                    const uint64_t off = (uint64_t)((uint32_t)s * (uint32_t)(PAIR_STAGE_BYTES >> 4));
#pragma unroll
                    for (int k = 0; k < BLOCK_K / 16; ++k)
                        umma_pair(acc, desc_x0 + off + 2 * k, desc_w0 + off + 2 * k, IDESC, kb > kb_begin || k > 0);
                    umma_commit_pair(empty0 + 8u * s);           // frees the stage in both CTAs
                    if (++s == stages) { s = 0; ph ^= 1u; }
                }
                umma_commit_pair(smem_u32(&acc_full[buf]));
            }
        }
    } else {
        // ---------------- epilogue (both CTAs): a thread owns a token, writes runs of 16 features ----------------
        const int lane_base = (warp & 3) * 32;
        const bool aligned = n_feat % 8 == 0;
        const uint32_t acc_empty_first = in_first_cta(smem_u32(&acc_empty[0]));
        wait_for_previous_kernels();
        for (int i = 0; i < my_tiles; ++i) {
            int f0, t0, kb_begin, kb_end;
            tile_coords(i, f0, t0, kb_begin, kb_end);
            const int buf = i & 1;
            const bool landed = mbar_wait(smem_u32(&acc_full[buf]), (uint32_t)(i >> 1) & 1u);
            if (!landed && lane == 0) {
                report(status, ST_EPILOGUE_TIMEOUT);
                abort_flag = 1;
            }
            tc_fence_after();
            if (!landed || abort_flag) break;
            const int t = t0 + rank * TM_TOK + lane_base + lane;
            const bool t_ok = t < n_tok;
            const uint32_t trow = tmem_base + ((uint32_t)lane_base << 16) + (uint32_t)(buf * TM_ROWS);
            tm_write_tile<DUAL, MODE>(trow, t, t_ok, f0, n_feat, aligned, bias, out_, split_k > 1);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(acc_empty_first + 8u * (uint32_t)buf);
        }
    }

    // nothing of the pair's tensor or shared memory is freed while the partner may still use it
    tc_fence_before();
    cluster_sync_all();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)TMEM_COLS)
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

template <int TN, bool DUAL, int MODE>
int launch(int tn, const CUtensorMap& mw, const CUtensorMap& mw2, const CUtensorMap& mx, const float* bias, void* out,
           int n_tok, int n_feat, int K, int split_k, int* status, cudaStream_t stream) {
    constexpr int STAGE_BYTES = (DUAL ? 2 : 1) * A_BYTES + TN * BLOCK_K * 2;
    const int total_kb = (K + BLOCK_K - 1) / BLOCK_K;
    // Small token tiles (decode) leave room for a second CTA on the SM, so that the next kernel's
    // CTAs can settle in and prefetch their weights while this one drains.
    const int budget = (3 * STAGE_BYTES <= 108 * 1024 && TN <= 64) ? 108 * 1024 : SMEM_BUDGET;
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
    static PerDeviceOnce configured;       // per device: the attribute belongs to a device's copy of the kernel
    if (int rc = raise_dynamic_smem(kernel, SMEM_BUDGET + 1024, configured, "gemm_tcgen05")) return rc;
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
    static PerDeviceOnce configured;       // per device: the attribute belongs to a device's copy of the kernel
    if (int rc = raise_dynamic_smem(kernel, SMEM_BUDGET + 1024, configured, "gemm_tcgen05")) return rc;
    constexpr int FEATS = DUAL ? TM_ROWS / 2 : TM_ROWS;
    const long long total_tiles = (long long)((n_tok + TM_TOK - 1) / TM_TOK) * ((n_feat + FEATS - 1) / FEATS);
    if (total_tiles > 0x7fffffffLL) return fail("gemm_tcgen05: %lld tiles exceed the index range", total_tiles);
    long long ctas = sm_count();
    if (ctas > total_tiles) ctas = total_tiles;
    cudaError_t e = launch_dependent(kernel, dim3((unsigned)ctas), dim3(THREADS), smem, stream, mw, mw2, mx, bias, out,
                                     n_tok, n_feat, K, stages, status);
    return check_launch(e, "gemm_tcgen05 (token-major)");
}

int g_pair_min_tokens = 512;     // steps of at least this many tokens may run on pairs of SMs (0: never)
bool g_pair_always = false;      // ... whatever their tiles make of the grid (tests)

// Whether a product runs on pairs of SMs.  Measured on a 3584-wide model at 512, 2,048 and 8,192 tokens: where
// the pair tiles fill the grid's rounds as well as the single-CTA tiles do, pairs are 2-5% faster (SiLU-gate
// projection 367 -> 357 us at 2,048 tokens, q/k/v 218 -> 208 us at 8,192); where they leave a round half
// empty (o and down projections: 112 tiles of 256 x 256 on 74 pairs) they lose up to 15%.  The adding epilogue
// cannot split K here, so it stays with the single-CTA kernel.
// Pieces of K for the adding epilogue on pairs: the count that leaves the busiest pair the fewest k-blocks,
// with a dozen per work item for its epilogue and ramp.
int pair_split(int n_tok, int n_feat, int K) {
    const int total_kb = (K + BLOCK_K - 1) / BLOCK_K;
    const long long tiles = (long long)((n_tok + PAIR_TOK - 1) / PAIR_TOK) * ((n_feat + TM_ROWS - 1) / TM_ROWS);
    const long long pairs = sm_count() / 2;
    long long best = -1;
    int split = 1;
    for (int sp = 1; sp <= 10 && (sp == 1 || total_kb / sp >= 8); ++sp) {
        const long long cost = ((tiles * sp + pairs - 1) / pairs) * ((total_kb + sp - 1) / sp + 12);
        if (best < 0 || cost < best) { best = cost; split = sp; }
    }
    return split;
}

bool on_pairs(int n_tok, int n_feat, int mode) {
    if (g_pair_min_tokens <= 0 || n_tok < g_pair_min_tokens) return false;
    if (g_pair_always) return true;
    if (mode == 2) return false;
    const long long feats = mode == 3 ? TM_ROWS / 2 : TM_ROWS;
    const long long tiles = (long long)((n_tok + PAIR_TOK - 1) / PAIR_TOK) * ((n_feat + feats - 1) / feats);
    const long long pairs = sm_count() / 2;
    const long long rounds = (tiles + pairs - 1) / pairs;
    return tiles * 100 >= rounds * pairs * 93;               // the last round at least ~93% full on average
}

template <bool DUAL, int MODE>
int launch_pair(const CUtensorMap& mw, const CUtensorMap& mw2, const CUtensorMap& mx, const float* bias, void* out,
                int n_tok, int n_feat, int K, int split_k, int* status, cudaStream_t stream) {
    const int total_kb = (K + BLOCK_K - 1) / BLOCK_K;
    if (split_k < 1 || MODE != 2) split_k = 1;
    if (split_k > total_kb) split_k = total_kb;
    const int kb_per_split = (total_kb + split_k - 1) / split_k;
    split_k = (total_kb + kb_per_split - 1) / kb_per_split;          // no empty piece
    int stages = SMEM_BUDGET / PAIR_STAGE_BYTES;
    if (stages > MAX_STAGES) stages = MAX_STAGES;
    if (stages > total_kb) stages = total_kb;
    const size_t smem = (size_t)stages * PAIR_STAGE_BYTES + 1024;
    auto kernel = gemm_pair_kernel<DUAL, MODE>;
    static PerDeviceOnce configured;       // per device: the attribute belongs to a device's copy of the kernel
    if (int rc = raise_dynamic_smem(kernel, SMEM_BUDGET + 1024, configured, "gemm_tcgen05")) return rc;
    constexpr int FEATS = DUAL ? TM_ROWS / 2 : TM_ROWS;
    const long long total_tiles = (long long)((n_tok + PAIR_TOK - 1) / PAIR_TOK) * ((n_feat + FEATS - 1) / FEATS) * split_k;
    if (total_tiles > 0x7fffffffLL) return fail("gemm_tcgen05: %lld tiles exceed the index range", total_tiles);
    long long pairs = sm_count() / 2;
    if (pairs > total_tiles) pairs = total_tiles;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(2 * pairs));
    cfg.blockDim = dim3(THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 2 : 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, mw, mw2, mx, bias, out, n_tok, n_feat, K, kb_per_split, split_k, stages, status);
    return check_launch(e, "gemm_tcgen05 (pairs of SMs)");
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

// Steps of at least n_tok tokens may run on pairs of SMs (0: never); with always != 0 they do, whatever
// their tiles make of the grid.  For comparisons and tests; plans made before the call no longer hold.
RI_API int ri_gemm_tcgen05_set_pairs(int n_tok, int always) {
    g_pair_min_tokens = n_tok < 0 ? 0 : n_tok;
    g_pair_always = always != 0;
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
    if (on_pairs(n_tok, n_feat, mode)) {
        tn = TM_TOK;                                              // pairs of SMs: each CTA's box holds 128 tokens
        if (mode == 2) sp = pair_split(n_tok, n_feat, K);
    } else if (n_tok <= 128) {
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
    if (on_pairs(n_tok, n_feat, mode)) {
        switch (mode) {
            case 0: return launch_pair<false, 0>(mw, mw2, mx, bias, out, n_tok, n_feat, K, 1, status, stream);
            case 1: return launch_pair<false, 1>(mw, mw2, mx, bias, out, n_tok, n_feat, K, 1, status, stream);
            case 2: return launch_pair<false, 2>(mw, mw2, mx, bias, out, n_tok, n_feat, K, split_k, status, stream);
            default: return launch_pair<true, 3>(mw, mw2, mx, bias, out, n_tok, n_feat, K, 1, status, stream);
        }
    }
    if (dual && n_tok > TM_TOK) return launch_tm<true, 3>(mw, mw2, mx, bias, out, n_tok, n_feat, K, status, stream);
    switch (mode) {
        case 0: return pick_tile<false, 0>(tn, mw, mw2, mx, bias, out, n_tok, n_feat, K, split_k, status, stream);
        case 1: return pick_tile<false, 1>(tn, mw, mw2, mx, bias, out, n_tok, n_feat, K, split_k, status, stream);
        case 2: return pick_tile<false, 2>(tn, mw, mw2, mx, bias, out, n_tok, n_feat, K, split_k, status, stream);
        default: return pick_tile<true, 3>(tn, mw, mw2, mx, bias, out, n_tok, n_feat, K, split_k, status, stream);
    }
}

RI_DEFINE_LAST_ERROR()
