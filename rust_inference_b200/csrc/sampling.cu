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

__global__ void __launch_bounds__(THREADS)
sample_kernel(float* __restrict__ logits, int vocab, int* __restrict__ out, float temperature, int top_k,
              float top_p, float penalty, const int* __restrict__ recent, int recent_ld,
              const int* __restrict__ recent_count, unsigned long long seed, const int* __restrict__ row_stream,
              const int* __restrict__ row_counter, int counter_offset, int* __restrict__ mirror) {
    __shared__ float fscratch[33];
    __shared__ int iscratch[33];
    __shared__ float chunk_sum[THREADS];
    __shared__ int chunk_cnt[THREADS];
    __shared__ int s_token;

    const int r = blockIdx.x, tid = threadIdx.x;
    let_next_kernel_start();
    wait_for_previous_kernels();          // the logits come from the kernel before
    float* p = logits + (size_t)r * vocab;

    // ---- repetition penalty (sampler.rs:109-127) ----
    if (penalty != 1.0f && recent != nullptr) {
        if (tid == 0) {
            const int n = recent_count[r];
            for (int i = 0; i < n; ++i) {
                const int id = recent[(size_t)r * recent_ld + i];
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

    // ---- temperature and softmax (sampler.rs:86-92, math.rs:104-118) ----
    float lmax = -INFINITY;
    for (int i = tid; i < vocab; i += THREADS) {
        const float x = p[i] / temperature;
        p[i] = x;
        lmax = fmaxf(lmax, x);
    }
    const float m = block_max(lmax, fscratch);
    float lsum = 0.f;
    for (int i = tid; i < vocab; i += THREADS) {
        const float e = expf(p[i] - m);
        p[i] = e;
        lsum += e;
    }
    const float z = block_sum(lsum, fscratch);
    const float inv_z = 1.0f / z;
    for (int i = tid; i < vocab; i += THREADS) p[i] *= inv_z;
    __syncthreads();

    // ---- top-k (sampler.rs:130-160) ----
    if (top_k > 0 && top_k < vocab) {
        unsigned t = 0;
        for (int bit = 30; bit >= 0; --bit) {
            const unsigned cand = t | (1u << bit);
            int cnt = 0;
            for (int i = tid; i < vocab; i += THREADS) cnt += (__float_as_uint(p[i]) >= cand);
            if (block_sum_int(cnt, iscratch) >= top_k) t = cand;      // at least k values are >= cand
        }
        const float threshold = __uint_as_float(t);                   // the k-th largest probability
        float s = 0.f;
        for (int i = tid; i < vocab; i += THREADS) {
            float v = p[i];
            if (v < threshold) { v = 0.f; p[i] = 0.f; }
            s += v;
        }
        s = block_sum(s, fscratch);
        if (s > 0.f) {
            const float inv = 1.0f / s;
            for (int i = tid; i < vocab; i += THREADS) p[i] *= inv;
        }
        __syncthreads();
    }

    const int chunk = (vocab + THREADS - 1) / THREADS;       // contiguous ids owned by a thread in scans
    const int lo = min(vocab, tid * chunk), hi = min(vocab, lo + chunk);

    // ---- top-p (sampler.rs:163-196) ----
    if (top_p > 0.f && top_p < 1.f) {
        unsigned t = 0;
        for (int bit = 30; bit >= 0; --bit) {
            const unsigned cand = t | (1u << bit);
            float mass = 0.f;
            for (int i = tid; i < vocab; i += THREADS) {
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
        for (int i = tid; i < vocab; i += THREADS) {
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
    const float u = uniform_open_closed(seed, (unsigned)row_stream[r], (unsigned)(row_counter[r] + counter_offset));
    float mine = 0.f;
    int last_pos = -1;
    for (int i = lo; i < hi; ++i) {
        const float v = p[i];
        mine += v;
        if (v > 0.f) last_pos = i;
    }
    chunk_sum[tid] = mine;
    chunk_cnt[tid] = last_pos;
    if (tid == 0) s_token = -1;
    __syncthreads();
    if (tid == 0) {
        // fixed-order scan of the 1024 chunk sums; remembers the last id with any probability
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
        if (tid == 0) store_token(out, mirror, r, iscratch[1] >= 0 ? iscratch[1] : vocab - 1);
        return;
    }
    if (tid == owner) {
        float run = chunk_sum[tid];
        int tok = last_pos;
        for (int i = lo; i < hi; ++i) {
            run += p[i];
            if (run >= u && p[i] > 0.f) { tok = i; break; }
        }
        store_token(out, mirror, r, tok);
    }
}

}  // namespace

// logits: float32 [rows, vocab], overwritten.  out: int32 [rows].
// recent (may be null): int32 [rows, recent_ld] with recent_count[r] valid ids per row, oldest first.
// row_stream / row_counter: int32 [rows], which sequence a row is and how many tokens it has drawn;
// counter_offset is added to every row's counter (rows that advance together keep their array).
// mirror (may be null): int32 [rows] in host memory the device can write; receives the tokens too.
RI_API int ri_sample(float* logits, int rows, int vocab, int* out, float temperature, int top_k, float top_p,
                     float penalty, const int* recent, int recent_ld, const int* recent_count,
                     unsigned long long seed, const int* row_stream, const int* row_counter, int counter_offset,
                     int* mirror, cudaStream_t stream) {
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
                                     row_stream, row_counter, counter_offset, mirror);
    return check_launch(e, "sample");
}

RI_DEFINE_LAST_ERROR()
