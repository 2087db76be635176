// On-device sampling from float32 logits, one thread block per row.
//
// The order of operations is the reference's (sampler.rs:72-106): repetition penalty,
// greedy if temperature <= 0, divide by temperature, softmax, top-k, top-p, draw.
//   penalty  for each id among the row's recent tokens (repeats apply again):
//            l > 0 ? l / p : l * p                                   (sampler.rs:109-127)
//   greedy   index of the maximum, the first one on ties             (math.rs:328-339)
//   softmax  m = max, e = exp(x - m), p = e * (1 / sum e)            (math.rs:104-118)
//   top-k    zero everything below the k-th largest probability (ties kept),
//            renormalise                                             (sampler.rs:130-160)
//   top-p    keep the smallest prefix of the descending order (ties by index) whose sum
//            reaches p, renormalise                                  (sampler.rs:163-196)
//   draw     first i whose running sum reaches u                     (sampler.rs:199-210)
//
// Where the reference sorts the vocabulary twice per token (sampler.rs:137-142, :164-169),
// this finds the thresholds by bisection over the bit patterns of the probabilities
// (non-negative floats order like their bits), 31 passes each, with fixed-order block
// reductions: the result does not depend on the batch a row is in or on thread timing.
// With top-k (up to 1,024) those passes run over a short list of candidates in shared memory
// instead of the vocabulary: three passes over the row in all (maximum, sum, candidates).
//
// The uniform number comes from a counter-based generator keyed by (seed, row stream,
// row counter) instead of the reference's sequential xorshift64 (sampler.rs:213-218), so
// a sequence draws the same numbers whatever else is in its batch.  u lies in (0, 1].
//
// The logits buffer is overwritten (it becomes the probabilities), as the reference
// overwrites its logits slice.
#include "common.cuh"

using namespace ri;

namespace {

constexpr int THREADS = 1024;

__device__ __forceinline__ unsigned long long mix64(unsigned long long z) {
    z += 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

// u in (0, 1] with 24 bits, from (seed, stream, counter).
__device__ __forceinline__ float uniform_open_closed(unsigned long long seed, unsigned stream, unsigned counter) {
    unsigned long long z = mix64(seed ^ mix64(((unsigned long long)stream << 32) | counter));
    return (float)((z >> 40) + 1ull) * (1.0f / 16777216.0f);
}

__device__ __forceinline__ int block_sum_int(int v, int* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        int t = lane < nwarps ? scratch[lane] : 0;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}

// The row's token, to the device array and, if given, to a second place as well: memory of the host
// that the device can write, so that the host can read the token without a copy of its own.
__device__ __forceinline__ void store_token(int* out, int* mirror, int r, int token) {
    out[r] = token;
    if (mirror != nullptr) {
        *reinterpret_cast<volatile int*>(mirror + r) = token;
        __threadfence_system();
    }
}

constexpr int WARPS = THREADS / 32;
constexpr int SEG_CAP = 128;                 // candidates a warp can hold from its stretch of the row
constexpr int CAP = WARPS * SEG_CAP;

// What is left of a row once its probabilities stand in p[0..n) (global memory, or a compact list in shared
// memory whose entries are in ascending id order, with their ids in `ids`): top-k, top-p and the draw, in the
// reference's order.  All threads of the block call.  Returns nothing; thread(s) store the token.
__device__ void finish_row(float* p, int n, const int* ids, int top_k, float top_p, float u, int* out, int* mirror,
                           int r, float* fscratch, int* iscratch, float* chunk_sum, int* chunk_cnt) {
    const int tid = threadIdx.x;
    // ---- top-k (sampler.rs:130-160); a candidate list is always renormalised: the rest of its row is zeroed ----
    if (top_k > 0 && (top_k < n || ids != nullptr)) {
        unsigned t = 0;
        for (int bit = 30; bit >= 0; --bit) {
            const unsigned cand = t | (1u << bit);
            int cnt = 0;
            for (int i = tid; i < n; i += THREADS) cnt += (__float_as_uint(p[i]) >= cand);
            if (block_sum_int(cnt, iscratch) >= top_k) t = cand;      // at least k values are >= cand
        }
        const float threshold = __uint_as_float(t);                   // the k-th largest probability
        float s = 0.f;
        for (int i = tid; i < n; i += THREADS) {
            float v = p[i];
            if (v < threshold) { v = 0.f; p[i] = 0.f; }
            s += v;
        }
        s = block_sum(s, fscratch);
        if (s > 0.f) {
            const float inv = 1.0f / s;
            for (int i = tid; i < n; i += THREADS) p[i] *= inv;
        }
        __syncthreads();
    }

    const int chunk = (n + THREADS - 1) / THREADS;           // contiguous entries owned by a thread in scans
    const int lo = min(n, tid * chunk), hi = min(n, lo + chunk);

    // ---- top-p (sampler.rs:163-196) ----
    if (top_p > 0.f && top_p < 1.f) {
        unsigned t = 0;
        for (int bit = 30; bit >= 0; --bit) {
            const unsigned cand = t | (1u << bit);
            float mass = 0.f;
            for (int i = tid; i < n; i += THREADS) {
                const float v = p[i];
                if (__float_as_uint(v) >= cand) mass += v;
            }
            if (block_sum(mass, fscratch) >= top_p) t = cand;          // values >= cand already reach p
        }
        // t is the value of the last element the descending walk takes.  Everything above it is kept;
        // of the elements equal to it, the first `keep` by index (the stable order) are kept.
        const float tval = __uint_as_float(t);
        float above = 0.f;
        int ties = 0;
        for (int i = tid; i < n; i += THREADS) {
            const float v = p[i];
            if (v > tval) above += v;
            ties += (v == tval);
        }
        above = block_sum(above, fscratch);
        const int n_ties = block_sum_int(ties, iscratch);
        int keep = n_ties;
        if (t != 0 && tval > 0.f) {
            keep = (int)ceilf((top_p - above) / tval);
            keep = max(1, min(n_ties, keep));
        }
        // rank of every tie by index: per-thread counts over contiguous chunks, then a scan
        int mine = 0;
        for (int i = lo; i < hi; ++i) mine += (p[i] == tval);
        chunk_cnt[tid] = mine;
        __syncthreads();
        if (tid == 0) {
            int run = 0;
            for (int i = 0; i < THREADS; ++i) { const int c = chunk_cnt[i]; chunk_cnt[i] = run; run += c; }
        }
        __syncthreads();
        int rank = chunk_cnt[tid];
        float s = 0.f;
        for (int i = lo; i < hi; ++i) {
            float v = p[i];
            if (v == tval) {
                if (rank >= keep) { v = 0.f; p[i] = 0.f; }
                ++rank;
            } else if (v < tval) {
                v = 0.f; p[i] = 0.f;
            }
            s += v;
        }
        s = block_sum(s, fscratch);
        if (s > 0.f) {
            const float inv = 1.0f / s;
            for (int i = lo; i < hi; ++i) p[i] *= inv;
        }
        __syncthreads();
    }

    // ---- draw (sampler.rs:199-210): first i whose running sum reaches u ----
    float mine = 0.f;
    int last_pos = -1;
    for (int i = lo; i < hi; ++i) {
        const float v = p[i];
        mine += v;
        if (v > 0.f) last_pos = i;
    }
    chunk_sum[tid] = mine;
    chunk_cnt[tid] = last_pos;
    __syncthreads();
    if (tid == 0) {
        // fixed-order scan of the 1024 chunk sums; remembers the last entry with any probability
        float run = 0.f;
        int owner = -1, last = -1;
        for (int i = 0; i < THREADS; ++i) {
            const float before = run;
            run += chunk_sum[i];
            if (chunk_cnt[i] >= 0) last = chunk_cnt[i];
            if (owner < 0 && run >= u) { owner = i; chunk_sum[i] = before; }
        }
        iscratch[0] = owner;
        iscratch[1] = last;
    }
    __syncthreads();
    const int owner = iscratch[0];
    if (owner < 0) {
        // rounding left the total just below u: the last id that has probability (the
        // reference falls back to the last id of the vocabulary, sampler.rs:208-209)
        if (tid == 0) {
            const int e = iscratch[1] >= 0 ? iscratch[1] : n - 1;
            store_token(out, mirror, r, ids ? ids[e] : e);
        }
        return;
    }
    if (tid == owner) {
        float run = chunk_sum[tid];
        int tok = last_pos;
        for (int i = lo; i < hi; ++i) {
            run += p[i];
            if (run >= u && p[i] > 0.f) { tok = i; break; }
        }
        store_token(out, mirror, r, ids ? ids[tok] : tok);
    }
}

__global__ void __launch_bounds__(THREADS)
sample_kernel(float* __restrict__ logits, int vocab, int* out, float temperature, int top_k,
              float top_p, float penalty, const int* __restrict__ recent, int recent_ld,
              const int* __restrict__ recent_count, unsigned long long seed, const int* __restrict__ row_stream,
              const int* __restrict__ row_counter, int counter_offset, int* __restrict__ mirror,
              const int* newest) {      // `newest` and `out` may be the same buffer: a row reads before it writes
    __shared__ float fscratch[33];
    __shared__ int iscratch[33];
    __shared__ float chunk_sum[THREADS];
    __shared__ int chunk_cnt[THREADS];
    __shared__ float cand_p[CAP];
    __shared__ int cand_i[CAP];
    __shared__ int seg_count[WARPS + 1];
    __shared__ float s_tau;

    const int r = blockIdx.x, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    let_next_kernel_start();
    wait_for_previous_kernels();          // the logits come from the kernel before
    float* p = logits + (size_t)r * vocab;

    // ---- repetition penalty (sampler.rs:109-127) ----
    if (penalty != 1.0f && (recent != nullptr || newest != nullptr)) {
        if (tid == 0) {
            const int n = recent != nullptr ? recent_count[r] : 0;
            for (int i = 0; i <= n; ++i) {
                // the row's recent ids, then the newest one, which may still be on the device only
                if (i == n && newest == nullptr) break;
                const int id = i < n ? recent[(size_t)r * recent_ld + i] : newest[r];
                if (id >= 0 && id < vocab) {
                    if (p[id] > 0.f) p[id] /= penalty; else p[id] *= penalty;
                }
            }
        }
        __syncthreads();
    }

    // ---- greedy (sampler.rs:81-83, math.rs:328-339): first maximum ----
    if (temperature <= 0.f) {
        float best = -INFINITY;
        int best_i = 0x7fffffff;
        for (int i = tid; i < vocab; i += THREADS) {
            const float v = p[i];
            if (v > best) { best = v; best_i = i; }        // strided, ascending: keeps the first in its stride
        }
        const float m = block_max(best, fscratch);
        int cand = (best == m) ? best_i : 0x7fffffff;
        // smallest index among the threads holding the maximum
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) cand = min(cand, __shfl_xor_sync(0xffffffffu, cand, o));
        __syncthreads();
        if ((tid & 31) == 0) iscratch[tid >> 5] = cand;
        __syncthreads();
        if (tid < 32) {
            int t = iscratch[tid];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) t = min(t, __shfl_xor_sync(0xffffffffu, t, o));
            if (tid == 0) store_token(out, mirror, r, (t == 0x7fffffff) ? 0 : t);
        }
        return;
    }

    // ---- temperature and softmax (sampler.rs:86-92, math.rs:104-118), without storing anything yet:
    // x = l / T, m = max x, z = sum exp(x - m); the probability of id i is exp(x_i - m) * (1 / z).
    // Dividing by T > 0 keeps the order, so the maximum is taken over the logits and divided once. ----
    float tmax = -INFINITY;
    if ((vocab & 3) == 0) {
        const float4* p4 = reinterpret_cast<const float4*>(p);
#pragma unroll 4
        for (int i = tid; i < (vocab >> 2); i += THREADS) {
            const float4 v = p4[i];
            tmax = fmaxf(fmaxf(tmax, fmaxf(v.x, v.y)), fmaxf(v.z, v.w));
        }
    } else {
#pragma unroll 4
        for (int i = tid; i < vocab; i += THREADS) tmax = fmaxf(tmax, p[i]);
    }
    tmax = tmax / temperature;                               // the largest x this thread saw
    const float m = block_max(tmax, fscratch);
    const float u = uniform_open_closed(seed, (unsigned)row_stream[r], (unsigned)(row_counter[r] + counter_offset));
    // the second pass is made warp by warp over contiguous stretches of the row, so that what it finds keeps
    // the order of the ids
    const int per = ((vocab + WARPS - 1) / WARPS + 31) / 32 * 32;
    const int w_lo = min(vocab, warp * per), w_hi = min(vocab, w_lo + per);
    const bool nucleus = top_p > 0.f && top_p < 1.f;

    // ---- the short way for top-k: only the few ids that can be among the k largest are kept, in a list in
    // shared memory, and everything after works on that list.  The k-th largest of the threads' own maxima is
    // a lower bound of the k-th largest of the row (they are k entries of the row), so every id that reaches
    // it is a candidate; all others lie below the k-th largest and would be zeroed.  The bound is taken a
    // shade lower than it is, since two x that differ in their last bits can give the same probability. ----
    if (top_k > 0 && top_k < vocab && top_k <= THREADS) {
        chunk_sum[tid] = tmax;
        __syncthreads();
        int above = 0;                                       // threads whose maximum comes before this one's
        for (int j = 0; j < THREADS; ++j) {
            const float o = chunk_sum[j];
            above += (o > tmax) || (o == tmax && j < tid);
        }
        if (above == top_k - 1) s_tau = tmax - (fabsf(tmax - m) + 1.f) * 2e-6f;
        if (tid < WARPS + 1) seg_count[tid] = 0;
        __syncthreads();
        const float tau = s_tau;
        int cnt = 0;
        float lsum = 0.f;
#pragma unroll 4
        for (int base = w_lo; base < w_hi; base += 32) {
            const int i = base + lane;
            const float x = i < w_hi ? p[i] / temperature : -INFINITY;
            lsum += expf(x - m);                             // exp(-inf) = 0 past the end
            const bool take = x >= tau;
            const unsigned mask = __ballot_sync(0xffffffffu, take);
            if (mask) {
                const int pos = cnt + __popc(mask & ((1u << lane) - 1u));
                if (take && pos < SEG_CAP) {
                    cand_p[warp * SEG_CAP + pos] = x;
                    cand_i[warp * SEG_CAP + pos] = i;
                }
                cnt += __popc(mask);
            }
        }
        if (lane == 0) {
            seg_count[warp] = cnt;
            if (cnt > SEG_CAP) seg_count[WARPS] = 1;         // a stretch with more candidates than it can hold
        }
        const float z = block_sum(lsum, fscratch);           // (also makes the counts visible)
        const float inv_z = 1.0f / z;
        if (seg_count[WARPS] == 0) {
            // close the gaps between the warps' lists (read through registers, then write in place) and turn
            // the candidates' x into probabilities
            float vals[CAP / THREADS];
            int idxs[CAP / THREADS], dst[CAP / THREADS];
#pragma unroll
            for (int j = 0; j < CAP / THREADS; ++j) {
                const int slot = tid + j * THREADS, w = slot / SEG_CAP, pos = slot % SEG_CAP;
                dst[j] = -1;
                if (pos < seg_count[w]) {
                    int off = 0;
                    for (int k = 0; k < w; ++k) off += seg_count[k];
                    dst[j] = off + pos;
                    vals[j] = expf(cand_p[slot] - m) * inv_z;
                    idxs[j] = cand_i[slot];
                }
            }
            __syncthreads();
#pragma unroll
            for (int j = 0; j < CAP / THREADS; ++j)
                if (dst[j] >= 0) { cand_p[dst[j]] = vals[j]; cand_i[dst[j]] = idxs[j]; }
            int n = 0;
            for (int k = 0; k < WARPS; ++k) n += seg_count[k];
            __syncthreads();
            finish_row(cand_p, n, cand_i, top_k, top_p, u, out, mirror, r, fscratch, iscratch, chunk_sum, chunk_cnt);
            return;
        }
        // too many ties for the list: the long way below handles any row
        for (int i = tid; i < vocab; i += THREADS) p[i] = expf(p[i] / temperature - m) * inv_z;
        __syncthreads();
        finish_row(p, vocab, nullptr, top_k, top_p, u, out, mirror, r, fscratch, iscratch, chunk_sum, chunk_cnt);
        return;
    }

    // ---- the sum, warp by warp ----
    float lsum = 0.f;
#pragma unroll 4
    for (int base = w_lo; base < w_hi; base += 32) {
        const int i = base + lane;
        if (i < w_hi) lsum += expf(p[i] / temperature - m);
    }
    const float wsum = warp_sum(lsum);                       // this warp's stretch
    const float z = block_sum(lsum, fscratch);
    const float inv_z = 1.0f / z;

    if (!nucleus && !(top_k > 0 && top_k < vocab)) {
        // ---- plain temperature sampling: the draw (sampler.rs:199-210) needs no stored probabilities.  The
        // stretch in which the running sum reaches u is found from the warps' sums; its warp walks it again. ----
        if (lane == 0) chunk_sum[warp] = wsum * inv_z;
        __syncthreads();
        if (tid == 0) {
            float run = 0.f;
            int owner = -1;
            for (int w = 0; w < WARPS; ++w) {
                const float before = run;
                run += chunk_sum[w];
                if (owner < 0 && run >= u) { owner = w; fscratch[0] = before; }
            }
            iscratch[0] = owner;
        }
        __syncthreads();
        const int owner = iscratch[0];
        if (owner < 0) {
            // rounding left the total just below u: the last id (sampler.rs:208-209)
            if (tid == 0) store_token(out, mirror, r, vocab - 1);
            return;
        }
        if (warp == owner) {
            float run = fscratch[0];
            int tok = -1;
            for (int base = w_lo; base < w_hi && tok < 0; base += 32) {
                const int i = base + lane;
                const float pr = i < w_hi ? expf(p[i] / temperature - m) * inv_z : 0.f;
                float incl = pr;                             // inclusive prefix sum over the 32 lanes
#pragma unroll
                for (int o = 1; o < 32; o <<= 1) {
                    const float t = __shfl_up_sync(0xffffffffu, incl, o);
                    if (lane >= o) incl += t;
                }
                const unsigned hit = __ballot_sync(0xffffffffu, run + incl >= u && pr > 0.f);
                if (hit) tok = base + __ffs(hit) - 1;
                run += __shfl_sync(0xffffffffu, incl, 31);
            }
            if (lane == 0) store_token(out, mirror, r, tok >= 0 ? tok : w_hi - 1);
        }
        return;
    }

    // ---- the long way: the probabilities take the place of the logits, and every step walks the whole row ----
    for (int i = tid; i < vocab; i += THREADS) p[i] = expf(p[i] / temperature - m) * inv_z;
    __syncthreads();
    finish_row(p, vocab, nullptr, top_k, top_p, u, out, mirror, r, fscratch, iscratch, chunk_sum, chunk_cnt);
}

}  // namespace

// logits: float32 [rows, vocab], overwritten.  out: int32 [rows].
// recent (may be null): int32 [rows, recent_ld] with recent_count[r] valid ids per row, oldest first.
// row_stream / row_counter: int32 [rows], which sequence a row is and how many tokens it has drawn;
// counter_offset is added to every row's counter (rows that advance together keep their array).
// mirror (may be null): int32 [rows] in host memory the device can write; receives the tokens too.
// newest (may be null): int32 [rows] on the device, one more recent id per row (the token of the step
// before, which the host may not have read yet); penalised after the ids of `recent`.
RI_API int ri_sample(float* logits, int rows, int vocab, int* out, float temperature, int top_k, float top_p,
                     float penalty, const int* recent, int recent_ld, const int* recent_count,
                     unsigned long long seed, const int* row_stream, const int* row_counter, int counter_offset,
                     int* mirror, const int* newest, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (vocab <= 0) return fail("sample: vocabulary of %d", vocab);
    if (penalty <= 0.f) return fail("sample: repetition penalty %f must be positive", penalty);
    if (temperature > 0.f && (row_stream == nullptr || row_counter == nullptr))
        return fail("sample: temperature sampling needs row streams and counters");
    if (mirror != nullptr) {
        // the kernel stores through this pointer: it must be host memory that the device reaches under the same address
        cudaPointerAttributes attr;
        if (cudaPointerGetAttributes(&attr, mirror) != cudaSuccess || attr.type != cudaMemoryTypeHost ||
            attr.devicePointer != (void*)mirror) {
            cudaGetLastError();
            return fail("sample: the mirror is not pinned host memory that the device can write");
        }
    }
    cudaError_t e = launch_dependent(sample_kernel, dim3(rows), dim3(THREADS), (size_t)0, stream, logits, vocab, out,
                                     temperature, top_k, top_p, penalty, recent, recent_ld, recent_count, seed,
                                     row_stream, row_counter, counter_offset, mirror, newest);
    return check_launch(e, "sample");
}

RI_DEFINE_LAST_ERROR()
