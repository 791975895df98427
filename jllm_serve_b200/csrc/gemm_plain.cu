// out[m, n] (+)= sum_k a[m, k] * w[n, k] (+ bias[n]) on the CUDA cores, true 32-bit accumulation.
//
// This is the matrix product of the float32 path (no tensor cores, no reduced-precision mode) and the
// fallback of the bfloat16 path for shapes the tensor-core kernels refuse. Each output element is one
// accumulator that takes its products in ascending k with fused multiply-adds, so an element's value
// does not depend on the tile it falls in, on M, or on the other rows of the batch.
#include "common.cuh"

namespace {

constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;

template <typename Tin, typename Tout>
__global__ void __launch_bounds__(256)
gemm_plain_kernel(const Tin* __restrict__ a, int lda, const Tin* __restrict__ w, int ldw, VecRef bias, int has_bias,
                  Tout* __restrict__ out, int ldo, int accumulate, int M, int N, int K) {
    __shared__ float as[BK][BM + 4];
    __shared__ float ws[BK][BN + 4];
    const int tid = threadIdx.x;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    const int tx = tid % 16, ty = tid / 16;  // thread computes rows ty*4.., cols tx*4..
    float acc[TM][TN] = {};
    // loader mapping: 64 rows x 16 k = 1024 values, 4 per thread: row = tid / 4, k = (tid % 4) * 4 .. +3
    const int lr = tid / 4, lk = (tid % 4) * 4;
    for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int k = k0 + lk + j;
            const int m = m0 + lr, n = n0 + lr;
            as[lk + j][lr] = (m < M && k < K) ? to_float(a[(size_t)m * lda + k]) : 0.f;
            ws[lk + j][lr] = (n < N && k < K) ? to_float(w[(size_t)n * ldw + k]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < BK; ++k) {
            float av[TM], wv[TN];
#pragma unroll
            for (int i = 0; i < TM; ++i) av[i] = as[k][ty * TM + i];
#pragma unroll
            for (int j = 0; j < TN; ++j) wv[j] = ws[k][tx * TN + j];
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(av[i], wv[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int m = m0 + ty * TM + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            const int n = n0 + tx * TN + j;
            if (n >= N) continue;
            float v = acc[i][j];
            if (has_bias) v += bias[n];
            Tout* dst = out + (size_t)m * ldo + n;
            if (accumulate) v += to_float(*dst);
            *dst = from_float<Tout>(v);
        }
    }
}

template <typename Tin, typename Tout>
int launch(const void* a, int lda, const void* w, int ldw, VecRef bias, int has_bias, void* out, int ldo,
           int accumulate, int M, int N, int K, cudaStream_t stream) {
    const dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
    gemm_plain_kernel<Tin, Tout><<<grid, 256, 0, stream>>>((const Tin*)a, lda, (const Tin*)w, ldw, bias, has_bias,
                                                           (Tout*)out, ldo, accumulate, M, N, K);
    return jllm_check_launch("gemm_plain");
}

}  // namespace

JLLM_EXPORT int jllm_gemm_plain(const void* a, int in_dtype, int lda, const void* w, int ldw, const void* bias,
                                int bias_dtype, void* out, int out_dtype, int ldo, int accumulate, int M, int N, int K,
                                cudaStream_t stream) {
    JLLM_REQUIRE(M >= 0 && N > 0 && K > 0, "gemm: M=%d N=%d K=%d", M, N, K);
    JLLM_REQUIRE(lda >= K && ldw >= K && ldo >= N, "gemm: strides lda=%d ldw=%d ldo=%d for K=%d N=%d", lda, ldw, ldo, K, N);
    JLLM_REQUIRE((M + BM - 1) / BM <= 65535, "gemm: M=%d is above %d rows", M, 65535 * BM);
    if (M == 0) return JLLM_OK;
    const VecRef b{bias, bias_dtype};
    const int hb = bias != nullptr;
    if (in_dtype == JLLM_F32 && out_dtype == JLLM_F32)
        return launch<float, float>(a, lda, w, ldw, b, hb, out, ldo, accumulate, M, N, K, stream);
    if (in_dtype == JLLM_BF16 && out_dtype == JLLM_F32)
        return launch<__nv_bfloat16, float>(a, lda, w, ldw, b, hb, out, ldo, accumulate, M, N, K, stream);
    if (in_dtype == JLLM_BF16 && out_dtype == JLLM_BF16)
        return launch<__nv_bfloat16, __nv_bfloat16>(a, lda, w, ldw, b, hb, out, ldo, accumulate, M, N, K, stream);
    return jllm_fail(JLLM_UNSUPPORTED, "gemm: float32 inputs with a bfloat16 result are not built");
}
