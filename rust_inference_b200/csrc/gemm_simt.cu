// out[M, N] = X[M, K] * W[N, K]^T on the FFMA pipe, float32 accumulation, any M, N, K.
//
// This is the true 32-bit contraction (no tensor-core mode of any kind touches the
// operands), and the fallback of the bf16 path for shapes the tensor-core kernel refuses.
// It restates the reference's mat-vec, y_r = sum_c W[r, c] x_c over a row-major [out, in]
// matrix (quant.rs:178-206, math.rs:212-229), for a batch of rows of X at once.
//
// Epilogues (all arithmetic in float32):
//   0  out<T>   = acc + bias                          (q/k/v projection, attention.rs:66-76)
//   1  out<f32> = acc + bias                          (logits, transformer.rs:97)
//   2  out<f32> += acc                                (o / down projection onto the residual
//                                                      stream, transformer.rs:38-39, :47)
//   3  out<T>   = silu(acc) * acc2, acc2 = X * W2^T   (SwiGLU, mlp.rs:35-43)
#include "common.cuh"

using namespace ri;

namespace {

constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4, THREADS = 256;

template <typename T> struct Vec4;
template <> struct Vec4<float> {
    using type = float4;
    __device__ static void unpack(const float4& v, float* o) { o[0] = v.x; o[1] = v.y; o[2] = v.z; o[3] = v.w; }
};
template <> struct Vec4<__nv_bfloat16> {
    using type = uint2;
    __device__ static void unpack(const uint2& v, float* o) {
        const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&v.x);
        const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&v.y);
        o[0] = __low2float(a); o[1] = __high2float(a); o[2] = __low2float(b); o[3] = __high2float(b);
    }
};

// Loads 4 consecutive k-elements of row `r` (if r < rows) starting at k0 into o[4], zero beyond K.
template <typename T, bool VEC>
__device__ __forceinline__ void load4(const T* __restrict__ base, int r, int rows, int k0, int K, float* o) {
    o[0] = o[1] = o[2] = o[3] = 0.f;
    if (r >= rows) return;
    const T* p = base + (size_t)r * K + k0;
    if (VEC && k0 + 3 < K) {
        typename Vec4<T>::type v = *reinterpret_cast<const typename Vec4<T>::type*>(p);
        Vec4<T>::unpack(v, o);
    } else {
#pragma unroll
        for (int i = 0; i < 4; ++i)
            if (k0 + i < K) o[i] = to_f32<T>(p[i]);
    }
}

template <typename T, int MODE, bool VEC>
__global__ void __launch_bounds__(THREADS)
gemm_simt_kernel(const T* __restrict__ X, const T* __restrict__ W, const T* __restrict__ W2,
                 const float* __restrict__ bias, void* __restrict__ out_, int M, int N, int K) {
    constexpr bool DUAL = MODE == 3;
    __shared__ float Xs[BK][BM + 4];
    __shared__ float Ws[BK][BN + 4];
    __shared__ float W2s[DUAL ? BK : 1][DUAL ? BN + 4 : 1];

    const int tid = threadIdx.x;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    const int lr = tid >> 2;            // 0..63: tile row this thread loads
    const int lk = (tid & 3) * 4;       // 0,4,8,12: first k of its 4 elements
    const int ty = tid >> 4, tx = tid & 15;

    float acc[TM][TN];
    float acc2[DUAL ? TM : 1][DUAL ? TN : 1];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            acc[i][j] = 0.f;
            if (DUAL) acc2[i][j] = 0.f;
        }

    for (int k0 = 0; k0 < K; k0 += BK) {
        float xv[4], wv[4], w2v[4];
        load4<T, VEC>(X, m0 + lr, M, k0 + lk, K, xv);
        load4<T, VEC>(W, n0 + lr, N, k0 + lk, K, wv);
        if (DUAL) load4<T, VEC>(W2, n0 + lr, N, k0 + lk, K, w2v);
        __syncthreads();      // previous tile fully consumed
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            Xs[lk + i][lr] = xv[i];
            Ws[lk + i][lr] = wv[i];
            if (DUAL) W2s[lk + i][lr] = w2v[i];
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < BK; ++k) {
            const float4 a = *reinterpret_cast<const float4*>(&Xs[k][ty * TM]);
            const float4 b = *reinterpret_cast<const float4*>(&Ws[k][tx * TN]);
            const float av[4] = {a.x, a.y, a.z, a.w}, bv[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
            if (DUAL) {
                const float4 b2 = *reinterpret_cast<const float4*>(&W2s[k][tx * TN]);
                const float b2v[4] = {b2.x, b2.y, b2.z, b2.w};
#pragma unroll
                for (int i = 0; i < TM; ++i)
#pragma unroll
                    for (int j = 0; j < TN; ++j) acc2[i][j] = fmaf(av[i], b2v[j], acc2[i][j]);
            }
        }
    }

#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int m = m0 + ty * TM + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            const int n = n0 + tx * TN + j;
            if (n >= N) continue;
            const size_t o = (size_t)m * N + n;
            float v = acc[i][j];
            if (MODE == 0) {
                if (bias) v += bias[n];
                reinterpret_cast<T*>(out_)[o] = from_f32<T>(v);
            } else if (MODE == 1) {
                if (bias) v += bias[n];
                reinterpret_cast<float*>(out_)[o] = v;
            } else if (MODE == 2) {
                reinterpret_cast<float*>(out_)[o] += v;
            } else {
                reinterpret_cast<T*>(out_)[o] = from_f32<T>(silu_f32(v) * acc2[i][j]);
            }
        }
    }
}

template <typename T, int MODE>
int launch(const void* X, const void* W, const void* W2, const float* bias, void* out, int M, int N, int K,
           cudaStream_t stream) {
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
    const size_t align = 4 * sizeof(T);
    const bool vec = (K % 4 == 0) && ((uintptr_t)X % align == 0) && ((uintptr_t)W % align == 0) &&
                     (W2 == nullptr || (uintptr_t)W2 % align == 0);
    if (vec)
        gemm_simt_kernel<T, MODE, true><<<grid, THREADS, 0, stream>>>((const T*)X, (const T*)W, (const T*)W2, bias, out, M, N, K);
    else
        gemm_simt_kernel<T, MODE, false><<<grid, THREADS, 0, stream>>>((const T*)X, (const T*)W, (const T*)W2, bias, out, M, N, K);
    return check_launch("gemm_simt");
}

template <typename T>
int dispatch_mode(int mode, const void* X, const void* W, const void* W2, const float* bias, void* out, int M,
                  int N, int K, cudaStream_t stream) {
    switch (mode) {
        case 0: return launch<T, 0>(X, W, W2, bias, out, M, N, K, stream);
        case 1: return launch<T, 1>(X, W, W2, bias, out, M, N, K, stream);
        case 2: return launch<T, 2>(X, W, W2, bias, out, M, N, K, stream);
        case 3: return launch<T, 3>(X, W, W2, bias, out, M, N, K, stream);
    }
    return fail("gemm_simt: unknown epilogue mode %d", mode);
}

}  // namespace

RI_API int ri_gemm_simt(const void* X, const void* W, const void* W2, const float* bias, void* out, int dtype,
                        int mode, int M, int N, int K, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0) return fail("gemm_simt: K must be positive, found %d", K);
    if (mode == 3 && W2 == nullptr) return fail("gemm_simt: the SiLU-gate epilogue needs a second matrix");
    if (mode == 2 && bias != nullptr) return fail("gemm_simt: the residual epilogue takes no bias");
    if (dtype == RI_F32) return dispatch_mode<float>(mode, X, W, W2, bias, out, M, N, K, stream);
    if (dtype == RI_BF16) return dispatch_mode<__nv_bfloat16>(mode, X, W, W2, bias, out, M, N, K, stream);
    return fail("gemm_simt: unknown dtype %d", dtype);
}

RI_DEFINE_LAST_ERROR()
