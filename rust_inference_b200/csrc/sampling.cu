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
//
// Two kernels compute the same thing.  `sample_kernel` gives a row to one thread block: any
// vocabulary, any options.  `sample_cluster_kernel` gives a row to a thread-block cluster of eight,
// each block taking a contiguous eighth of the row; the blocks exchange their maxima, sums and
// candidates through distributed shared memory.  A block alone spends tens of microseconds on the
// exponentials of a 150,000-entry row while 140 SMs idle at a batch of eight; the cluster is used for
// large vocabularies whenever the options allow it (greedy, plain temperature, top-k up to 256 with or
// without top-p).
#include "common.cuh"
#include <atomic>

#include <cooperative_groups.h>

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

// The same for a compact list of at most THREADS candidates (ascending id order, ids in `ids`): an entry per
// thread.  Instead of finding the thresholds by bisection, every thread counts its entry's place in the
// descending order (ties by position, as a stable sort leaves them), which takes n steps and no block-wide
// reduction; the k-th largest is the entry at place k - 1, and top-p keeps an entry while the entries before
// it in that order have not reached p.  The draw is one thread's walk over the list in id order.
__device__ void finish_short(const float* p, int n, const int* ids, int top_k, float top_p, float u, int* out, int* mirror,
                             int r, float* fscratch, float* chunk_sum, int* chunk_cnt) {
    const int tid = threadIdx.x;
    float v = tid < n ? p[tid] : 0.f;
    int place = 0;
    for (int j = 0; j < n; ++j) {
        const float o = p[j];
        place += (o > v) || (o == v && j < tid);
    }
    // ---- top-k (sampler.rs:130-160): ties with the k-th largest are kept; the list is always renormalised ----
    if (top_k > 0) {
        if (top_k < n) {
            if (tid < n && place == top_k - 1) fscratch[0] = v;
            __syncthreads();
            const float threshold = fscratch[0];
            __syncthreads();
            if (v < threshold) v = 0.f;
        }
        const float s = block_sum(v, fscratch);
        if (s > 0.f) v *= 1.0f / s;
    }
    // ---- top-p (sampler.rs:163-196) ----
    if (top_p > 0.f && top_p < 1.f) {
        if (tid < n) { chunk_sum[tid] = v; chunk_cnt[tid] = place; }
        __syncthreads();
        float before = 0.f;
        for (int j = 0; j < n; ++j)
            if (chunk_cnt[j] < place) before += chunk_sum[j];
        if (!(before < top_p)) v = 0.f;
        __syncthreads();
        const float s = block_sum(v, fscratch);
        if (s > 0.f) v *= 1.0f / s;
    }
    // ---- draw (sampler.rs:199-210): first entry at which the running sum reaches u ----
    __syncthreads();
    if (tid < n) chunk_sum[tid] = v;
    __syncthreads();
    if (tid == 0) {
        float run = 0.f;
        int tok = -1, last = -1;
        for (int j = 0; j < n && tok < 0; ++j) {
            const float q = chunk_sum[j];
            run += q;
            if (q > 0.f) {
                last = j;
                if (run >= u) tok = j;
            }
        }
        const int e = tok >= 0 ? tok : (last >= 0 ? last : n - 1);
        store_token(out, mirror, r, ids[e]);
    }
}

// Repetition penalty (sampler.rs:109-127) on the ids of [lo, hi): l > 0 ? l / penalty : l * penalty for each id
// among the row's recent tokens and then the newest one, which may still be on the device only; an id that
// occurs several times is penalised that often.  A thread per entry of the list: the first occurrence of an id
// applies the penalty as often as the id occurs.  `list` holds THREADS ints; longer lists are walked by one thread.
__device__ void apply_penalty(float* p, int lo, int hi, float penalty, const int* __restrict__ recent, int recent_ld,
                              const int* __restrict__ recent_count, const int* newest, int r, int* list) {
    const int tid = threadIdx.x;
    const int n_recent = recent != nullptr ? recent_count[r] : 0;
    const int n = n_recent + (newest != nullptr ? 1 : 0);
    if (n <= THREADS) {
        if (tid < n) list[tid] = tid < n_recent ? recent[(size_t)r * recent_ld + tid] : newest[r];
        __syncthreads();
        if (tid < n) {
            const int id = list[tid];
            if (id >= lo && id < hi) {
                bool first = true;
                int times = 0;
                for (int j = 0; j < n; ++j) {
                    const bool same = list[j] == id;
                    first = first && !(same && j < tid);
                    times += same;
                }
                if (first) {
                    float v = p[id];
                    for (int t = 0; t < times; ++t) v = v > 0.f ? v / penalty : v * penalty;
                    p[id] = v;
                }
            }
        }
    } else if (tid == 0) {
        for (int i = 0; i < n; ++i) {
            const int id = i < n_recent ? recent[(size_t)r * recent_ld + i] : newest[r];
            if (id >= lo && id < hi) {
                if (p[id] > 0.f) p[id] /= penalty; else p[id] *= penalty;
            }
        }
    }
    __syncthreads();
}

__global__ void __launch_bounds__(THREADS)
sample_kernel(float* __restrict__ logits, int vocab, int* out, float temperature, int top_k,
              float top_p, float penalty, const int* __restrict__ recent, int recent_ld,
              const int* __restrict__ recent_count, unsigned long long seed, const unsigned long long* __restrict__ seed_ptr,
              const int* __restrict__ row_stream,
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

    if (penalty != 1.0f && (recent != nullptr || newest != nullptr))
        apply_penalty(p, 0, vocab, penalty, recent, recent_ld, recent_count, newest, r, chunk_cnt);

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
    if (seed_ptr != nullptr) seed = *seed_ptr;                   // a seed kept on the device (a captured step's)
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
            if (n <= THREADS) finish_short(cand_p, n, cand_i, top_k, top_p, u, out, mirror, r, fscratch, chunk_sum, chunk_cnt);
            else finish_row(cand_p, n, cand_i, top_k, top_p, u, out, mirror, r, fscratch, iscratch, chunk_sum, chunk_cnt);
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


// ---------------------------------------------------------------------------------------------
// A row per cluster.
// ---------------------------------------------------------------------------------------------
constexpr int CLUSTER = 8;
constexpr int GROUPS = CLUSTER * WARPS;      // stretches of a row: one per warp of the cluster, in id order

__global__ void __launch_bounds__(THREADS)
sample_cluster_kernel(float* __restrict__ logits, int vocab, int per_cta, int* out, float temperature, int top_k,
                      float top_p, float penalty, const int* __restrict__ recent, int recent_ld,
                      const int* __restrict__ recent_count, unsigned long long seed, const unsigned long long* __restrict__ seed_ptr,
              const int* __restrict__ row_stream,
                      const int* __restrict__ row_counter, int counter_offset, int* __restrict__ mirror,
                      const int* newest) {      // `newest` and `out` may be the same buffer: a row reads before it writes
    namespace cg = cooperative_groups;
    __shared__ float fscratch[33];
    __shared__ int iscratch[33];
    __shared__ float chunk_sum[THREADS];
    __shared__ int chunk_cnt[THREADS];
    __shared__ float cand_p[CAP];
    __shared__ int cand_i[CAP];
    __shared__ int seg_count[WARPS + 1];
    __shared__ float warp_z[WARPS];
    // written by the other blocks of the cluster
    __shared__ float rx_wmax[GROUPS];
    __shared__ float rx_sum[CLUSTER];
    __shared__ int rx_cnt[CLUSTER];
    __shared__ float rx_best[CLUSTER];
    __shared__ int rx_best_i[CLUSTER];

    cg::cluster_group cluster = cg::this_cluster();
    const int rank = (int)cluster.block_rank();
    const int r = blockIdx.y, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");   // "this block runs": waited for before the first exchange
    if (tid == 0) seg_count[WARPS] = 0;                          // (the exchanges below make it visible in time)
    let_next_kernel_start();
    wait_for_previous_kernels();          // the logits come from the kernel before
    float* p = logits + (size_t)r * vocab;
    const int c_lo = min(vocab, rank * per_cta), c_hi = min(vocab, c_lo + per_cta);     // this block's part of the row

    // every block goes through the list and changes the ids of its part
    if (penalty != 1.0f && (recent != nullptr || newest != nullptr))
        apply_penalty(p, c_lo, c_hi, penalty, recent, recent_ld, recent_count, newest, r, chunk_cnt);

    // ---- greedy (sampler.rs:81-83, math.rs:328-339): first maximum ----
    if (temperature <= 0.f) {
        float best = -INFINITY;
        int best_i = 0x7fffffff;
        // eight loads in flight per thread: the walk is bound by the latency of its loads, not by their number
        for (int i0 = c_lo + tid; i0 < c_hi; i0 += THREADS * 8) {
            float v[8];
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                const int i = i0 + k * THREADS;
                v[k] = i < c_hi ? p[i] : -INFINITY;
            }
#pragma unroll
            for (int k = 0; k < 8; ++k)                            // ids ascend with k: a later one must be larger to win
                if (v[k] > best) { best = v[k]; best_i = i0 + k * THREADS; }
        }
        const float m = block_max(best, fscratch);
        int cand = (best == m) ? best_i : 0x7fffffff;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) cand = min(cand, __shfl_xor_sync(0xffffffffu, cand, o));
        __syncthreads();
        if (lane == 0) iscratch[warp] = cand;
        __syncthreads();
        asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
        if (tid < 32) {
            int t = iscratch[tid];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) t = min(t, __shfl_xor_sync(0xffffffffu, t, o));
            if (tid == 0) {
                cluster.map_shared_rank(rx_best, 0)[rank] = m;
                cluster.map_shared_rank(rx_best_i, 0)[rank] = t;
            }
        }
        cluster.sync();
        if (rank == 0 && tid == 0) {
            float bm = -INFINITY;
            int bi = 0x7fffffff;
            for (int c = 0; c < CLUSTER; ++c)                    // parts are in id order: a later one must be larger to win
                if (rx_best[c] > bm && rx_best_i[c] != 0x7fffffff) { bm = rx_best[c]; bi = rx_best_i[c]; }
            store_token(out, mirror, r, bi == 0x7fffffff ? 0 : bi);
        }
        return;
    }

    // ---- the maximum (the order of operations and the formulas are those of sample_kernel) ----
    const int per = per_cta / WARPS;                             // a warp's stretch; a multiple of 32
    const int w_lo = min(c_hi, c_lo + warp * per), w_hi = min(c_hi, w_lo + per);
    float tmax = -INFINITY;
    for (int i0 = w_lo + lane; i0 < w_hi; i0 += 32 * 8) {        // eight loads in flight per thread
        float v[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            const int i = i0 + k * 32;
            v[k] = i < w_hi ? p[i] : -INFINITY;
        }
#pragma unroll
        for (int k = 0; k < 8; ++k) tmax = fmaxf(tmax, v[k]);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, o));
    tmax = tmax / temperature;                                   // the largest x of this warp's stretch
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
    if (lane < CLUSTER) cluster.map_shared_rank(rx_wmax, lane)[rank * WARPS + warp] = tmax;
    if (seed_ptr != nullptr) seed = *seed_ptr;                   // a seed kept on the device (a captured step's)
    const float u = uniform_open_closed(seed, (unsigned)row_stream[r], (unsigned)(row_counter[r] + counter_offset));
    cluster.sync();
    float m = -INFINITY;
    for (int g = lane; g < GROUPS; g += 32) m = fmaxf(m, rx_wmax[g]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    const bool nucleus = top_p > 0.f && top_p < 1.f;
    const bool shortlist = top_k > 0 && top_k < vocab;           // the host sends top_k <= GROUPS only

    // ---- candidates for top-k: the k-th largest of the stretches' maxima is a lower bound of the k-th largest of
    // the row; every id that reaches it (a shade lower: see sample_kernel) goes on the list ----
    float tau = INFINITY;
    if (shortlist) {
        if (tid < GROUPS) {
            const float mine = rx_wmax[tid];
            int above = 0;
            for (int j = 0; j < GROUPS; ++j) {
                const float o = rx_wmax[j];
                above += (o > mine) || (o == mine && j < tid);
            }
            if (above == top_k - 1) fscratch[0] = mine - (fabsf(mine - m) + 1.f) * 2e-6f;
        }
        __syncthreads();
        tau = fscratch[0];
        __syncthreads();
    }

    // ---- the sum, and the candidates in id order ----
    int cnt = 0;
    float lsum = 0.f;
#pragma unroll 4
    for (int base = w_lo; base < w_hi; base += 32) {
        const int i = base + lane;
        const float x = i < w_hi ? p[i] / temperature : -INFINITY;
        lsum += expf(x - m);                                     // exp(-inf) = 0 past the end
        if (shortlist) {
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
    }
    const float wsum = warp_sum(lsum);
    if (lane == 0) {
        warp_z[warp] = wsum;
        seg_count[warp] = cnt;
        if (cnt > SEG_CAP) seg_count[WARPS] = 1;                 // a stretch with more candidates than it can hold
    }
    const float cta_z = block_sum(lsum, fscratch);               // (also makes the counts visible)
    int n_mine = 0;
    for (int k = 0; k < WARPS; ++k) n_mine += seg_count[k];
    if (seg_count[WARPS]) n_mine = CAP + 1;                      // marks the overflow for every block
    if (tid < CLUSTER) {
        cluster.map_shared_rank(rx_sum, tid)[rank] = cta_z;
        cluster.map_shared_rank(rx_cnt, tid)[rank] = n_mine;
    }
    cluster.sync();
    float z = 0.f;
    int n_all = 0, n_before = 0;
    for (int c = 0; c < CLUSTER; ++c) {                          // fixed order: the same sums in every block
        if (c == rank) n_before = n_all;
        z += rx_sum[c];
        n_all = min(CAP + 1, n_all + rx_cnt[c]);
    }
    const float inv_z = 1.0f / z;

    if (!nucleus && !shortlist) {
        // ---- plain temperature sampling: the block, then the warp, in whose part the running sum reaches u ----
        int owner_cta = -1;
        float run = 0.f, before_cta = 0.f;
        for (int c = 0; c < CLUSTER; ++c) {
            const float before = run;
            run += rx_sum[c] * inv_z;
            if (owner_cta < 0 && run >= u) { owner_cta = c; before_cta = before; }
        }
        if (owner_cta < 0) {
            // rounding left the total just below u: the last id (sampler.rs:208-209)
            if (rank == CLUSTER - 1 && tid == 0) store_token(out, mirror, r, vocab - 1);
            return;
        }
        if (rank != owner_cta) return;
        if (tid == 0) {
            float wrun = before_cta;
            int owner = -1;
            for (int w = 0; w < WARPS; ++w) {
                const float before = wrun;
                wrun += warp_z[w] * inv_z;
                if (owner < 0 && wrun >= u) { owner = w; fscratch[0] = before; }
            }
            iscratch[0] = owner;
        }
        __syncthreads();
        int owner = iscratch[0];
        float start = fscratch[0];
        if (owner < 0) {                                         // the block's sum reached u, its warps' sums fell short by rounding
            owner = WARPS - 1;
            while (owner > 0 && min(c_hi, c_lo + owner * per) >= c_hi) --owner;
            start = -1.f;                                        // walk the last stretch and take its last id with probability
        }
        if (warp == owner) {
            float wrun = start < 0.f ? 0.f : start;
            int tok = -1, last = -1;
            for (int base = w_lo; base < w_hi && tok < 0; base += 32) {
                const int i = base + lane;
                const float pr = i < w_hi ? expf(p[i] / temperature - m) * inv_z : 0.f;
                float incl = pr;                                 // inclusive prefix sum over the 32 lanes
#pragma unroll
                for (int o = 1; o < 32; o <<= 1) {
                    const float t = __shfl_up_sync(0xffffffffu, incl, o);
                    if (lane >= o) incl += t;
                }
                const unsigned has = __ballot_sync(0xffffffffu, pr > 0.f);
                if (has) last = base + 31 - __clz(has);
                const unsigned hit = __ballot_sync(0xffffffffu, start >= 0.f && wrun + incl >= u && pr > 0.f);
                if (hit) tok = base + __ffs(hit) - 1;
                wrun += __shfl_sync(0xffffffffu, incl, 31);
            }
            if (lane == 0) store_token(out, mirror, r, tok >= 0 ? tok : (last >= 0 ? last : w_hi - 1));
        }
        return;
    }

    if (shortlist && n_all <= CAP) {
        // ---- every block sends its candidates, as probabilities, to their place in the first block's list ----
        float* dst_p = cluster.map_shared_rank(cand_p, 0);
        int* dst_i = cluster.map_shared_rank(cand_i, 0);
        float vals[CAP / THREADS];
        int idxs[CAP / THREADS], dst[CAP / THREADS];
#pragma unroll
        for (int j = 0; j < CAP / THREADS; ++j) {
            const int slot = tid + j * THREADS, w = slot / SEG_CAP, pos = slot % SEG_CAP;
            dst[j] = -1;
            if (pos < seg_count[w]) {
                int off = n_before;
                for (int k = 0; k < w; ++k) off += seg_count[k];
                dst[j] = off + pos;
                vals[j] = expf(cand_p[slot] - m) * inv_z;
                idxs[j] = cand_i[slot];
            }
        }
        cluster.sync();                                          // the first block has read its own list: it may be overwritten
#pragma unroll
        for (int j = 0; j < CAP / THREADS; ++j)
            if (dst[j] >= 0) { dst_p[dst[j]] = vals[j]; dst_i[dst[j]] = idxs[j]; }
        cluster.sync();
        if (rank == 0) {
            if (n_all <= THREADS) finish_short(cand_p, n_all, cand_i, top_k, top_p, u, out, mirror, r, fscratch, chunk_sum, chunk_cnt);
            else finish_row(cand_p, n_all, cand_i, top_k, top_p, u, out, mirror, r, fscratch, iscratch, chunk_sum, chunk_cnt);
        }
        return;
    }

    // ---- the long way (more ties than the list holds): every block turns its part of the row into
    // probabilities, the first one walks the whole row ----
    for (int i = c_lo + tid; i < c_hi; i += THREADS) p[i] = expf(p[i] / temperature - m) * inv_z;
    __threadfence();
    cluster.sync();
    if (rank == 0)
        finish_row(p, vocab, nullptr, top_k, top_p, u, out, mirror, r, fscratch, iscratch, chunk_sum, chunk_cnt);
}

}  // namespace

int g_cluster_min_vocab = 32768;
int g_cluster_any_rows = 0;            // 1: clusters however many rows there are (for tests and comparisons)

// SMs of the current device (asked once per device)
static int sm_count() {
    static std::atomic<int> known[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    int n = known[dev].load(std::memory_order_relaxed);
    if (n == 0) {
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        known[dev].store(n, std::memory_order_relaxed);
    }
    return n;
}

// logits: float32 [rows, vocab], overwritten.  out: int32 [rows].
// recent (may be null): int32 [rows, recent_ld] with recent_count[r] valid ids per row, oldest first.
// row_stream / row_counter: int32 [rows], which sequence a row is and how many tokens it has drawn;
// counter_offset is added to every row's counter (rows that advance together keep their array).
// mirror (may be null): int32 [rows] in host memory the device can write; receives the tokens too.
// newest (may be null): int32 [rows] on the device, one more recent id per row (the token of the step
// before, which the host may not have read yet); penalised after the ids of `recent`.
// seed_dev (may be null): a 64-bit seed on the device that takes the place of `seed` (a captured step
// keeps its seed there, so that another seed needs no other capture).
RI_API int ri_sample(float* logits, int rows, int vocab, int* out, float temperature, int top_k, float top_p,
                     float penalty, const int* recent, int recent_ld, const int* recent_count,
                     unsigned long long seed, const int* row_stream, const int* row_counter, int counter_offset,
                     int* mirror, const int* newest, const unsigned long long* seed_dev, cudaStream_t stream) {
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
    // A cluster per row when the row is long enough to be worth it and the options allow it: greedy, plain
    // temperature, or a top-k that the stretches' maxima can bound (with or without top-p).
    const bool no_top_k = top_k <= 0 || top_k >= vocab;
    const bool plain = no_top_k && !(top_p > 0.f && top_p < 1.f);
    // And while the clusters are few enough: a cluster's blocks take an SM each, so rows beyond SMs / 8 run in
    // turns.  Measured at a vocabulary of 152,064 (cluster against a block per row, microseconds): greedy 8 rows
    // 4.1 / 7.7, 24 rows 7.2 / 7.2, 32 rows 10.3 / 7.2, 64 rows 17.1 / 7.6; temperature 0.8 with top-k 40 and
    // top-p 0.95: 8 rows 22 / 86, 32 rows 52 / 87, 64 rows 85 / 88.
    const int sms = sm_count();
    const int most_rows = temperature <= 0.f ? (sms + sms / 4) / CLUSTER : (4 * sms) / CLUSTER;
    const bool by_cluster = g_cluster_min_vocab > 0 && vocab >= g_cluster_min_vocab && rows <= 65535 &&
                            (g_cluster_any_rows || rows <= most_rows) &&
                            (temperature <= 0.f || plain || (!no_top_k && top_k <= GROUPS));
    if (by_cluster) {
        // a block's part: an equal share rounded up so that each of its warps has whole groups of 32 ids
        const int per_cta = ((vocab + CLUSTER - 1) / CLUSTER + THREADS - 1) / THREADS * THREADS;
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(CLUSTER, rows);
        cfg.blockDim = dim3(THREADS);
        cfg.dynamicSmemBytes = 0;
        cfg.stream = stream;
        cudaLaunchAttribute attr[2];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = CLUSTER;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[1].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = pdl_enabled() ? 2 : 1;
        cudaError_t e = cudaLaunchKernelEx(&cfg, sample_cluster_kernel, logits, vocab, per_cta, out, temperature, top_k, top_p,
                                           penalty, recent, recent_ld, recent_count, seed, seed_dev, row_stream, row_counter,
                                           counter_offset, mirror, newest);
        return check_launch(e, "sample (cluster)");
    }
    cudaError_t e = launch_dependent(sample_kernel, dim3(rows), dim3(THREADS), (size_t)0, stream, logits, vocab, out,
                                     temperature, top_k, top_p, penalty, recent, recent_ld, recent_count, seed, seed_dev,
                                     row_stream, row_counter, counter_offset, mirror, newest);
    return check_launch(e, "sample");
}

// Rows of at least this many entries are sampled by a cluster of blocks where the options allow it
// (0: never).  For comparisons and tests.
RI_API int ri_sample_set_cluster_min_vocab(int vocab) {
    g_cluster_min_vocab = vocab < 0 ? 0 : vocab;
    return 0;
}

// 1: rows of such a length are sampled by clusters however many rows a call brings (0: only while the
// clusters are few enough to run together).  For comparisons and tests.
RI_API int ri_sample_set_cluster_any_rows(int on) {
    g_cluster_any_rows = on ? 1 : 0;
    return 0;
}

RI_DEFINE_LAST_ERROR()
