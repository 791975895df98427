// out[m, n] (+)= sum_k a[m, k] * w[n, k] (+ bias[n]) for a few rows (m <= 64): the decode-step product.
//
// With so few rows the product is a stream of the weight matrix: every weight is read once from HBM
// and used for all rows, so the kernel is built around the weight loads. The roles of the tensor-core
// operands are swapped: 16 (or 32) weight rows are the M side of mma.sync.m16n8k16 and 8 tokens are
// its N side, so no tensor-core rows are wasted on padding tokens. Each thread loads 16 contiguous
// bytes of a weight row straight from global memory into the registers of the A fragment; the k index
// inside one 32-wide chunk is permuted (thread t owns k = 8t .. 8t+7), and the activation fragment is
// loaded with the same permutation, which a sum over k does not notice. The 8 warps of a block take
// interleaved 64-wide k blocks, and their partial sums are added in shared memory in a fixed order:
// results are deterministic.
//
// The weights are read in the PACKED layout all bfloat16 products share (ops.pack_weight: tiles of 128 rows x 64 k,
// a row of a tile 128 bytes, its 16-byte chunk c at chunk position c ^ (row & 7), tile (t, kb) at
// (t * k_blocks + kb) * 16 KB; padded with zeros). A warp's load of 8 rows x 64 bytes then comes from one 1 KB
// stretch of memory instead of 8 rows that lie a whole row apart.
//
// Requirements (else the caller uses the CUDA-core kernel): bfloat16 inputs, K a multiple of 8,
// 16-byte aligned rows (lda a multiple of 8; aligned base pointers), 1 <= M <= 64.
#include "common.cuh"

namespace {

constexpr int WARPS = 8;
constexpr int KCHUNK = 32;

__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint4 load_16(const __nv_bfloat16* p) {
    return __ldg(reinterpret_cast<const uint4*>(p));
}

// streaming load of weights: read once, do not keep in L1
__device__ __forceinline__ uint4 load_16_stream(const __nv_bfloat16* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

template <int NT, int RT, int UNROLL, typename Tout>
__global__ void __launch_bounds__(WARPS * 32, 2)
gemm_small_m_kernel(const __nv_bfloat16* __restrict__ a, int lda, const __nv_bfloat16* __restrict__ w, int k_blocks,
                    VecRef bias, int has_bias, Tout* __restrict__ out, int ldo, int accumulate, int M, int N, int K,
                    int swiglu) {
    extern __shared__ float red[];  // [WARPS][RT * 16][NT * 8]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int n0 = blockIdx.x * (16 * RT);
    float acc[RT][NT][4];
#pragma unroll
    for (int r = 0; r < RT; ++r)
#pragma unroll
        for (int j = 0; j < NT; ++j)
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[r][j][i] = 0.f;

    // where this thread's weight rows start in the packed layout (rows beyond N are zeros there; beyond the padded
    // rows there is nothing: those are not read)
    const __nv_bfloat16* wrow[RT][2];
    bool wok[RT][2];
    const int padded_rows = (N + 127) & ~127;
#pragma unroll
    for (int r = 0; r < RT; ++r)
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int n = n0 + r * 16 + h * 8 + g;
            wok[r][h] = n < padded_rows;
            const int nn = wok[r][h] ? n : 0;
            wrow[r][h] = w + (size_t)(nn >> 7) * k_blocks * 8192 + (size_t)(nn & 127) * 64;
        }
    const __nv_bfloat16* arow[NT];
    bool aok[NT];
#pragma unroll
    for (int j = 0; j < NT; ++j) {
        const int m = j * 8 + g;
        aok[j] = m < M;
        arow[j] = a + (size_t)(aok[j] ? m : 0) * lda;
    }
    const uint4 zero = make_uint4(0, 0, 0, 0);
    const int chunks = (K + KCHUNK - 1) / KCHUNK;
    uint4 wv[UNROLL][RT][2];
    static_assert(UNROLL % 2 == 0, "a warp takes the two halves of a k block together");
    // the u-th 32-wide chunk of the batch that starts at k block c0: k blocks c0, c0 + WARPS, ..., two chunks each
    auto chunk_of = [&](int c0, int u) { return 2 * (c0 + (u >> 1) * WARPS) + (u & 1); };
    auto load_weights = [&](int c0) {
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            // 32-wide chunk cc of k: k block cc / 2, 16-byte chunks (cc % 2) * 4 + t of the row's 128 bytes, which lie
            // at chunk position (that) ^ (row & 7); row & 7 = g for all of this thread's rows. A warp takes BOTH
            // halves of a k block one after the other, so that it reads whole 128-byte lines: its 16 rows of a k block
            // are one contiguous 2 KB piece of the packed weight.
            const int cc = chunk_of(c0, u);
            const bool kin = cc < chunks;
            const size_t at = (size_t)(cc >> 1) * 8192 + (size_t)(((((cc & 1) << 2) + t) ^ g) << 3);
#pragma unroll
            for (int r = 0; r < RT; ++r)
#pragma unroll
                for (int h = 0; h < 2; ++h) wv[u][r][h] = (kin && wok[r][h]) ? load_16_stream(wrow[r][h] + at) : zero;
        }
    };
    // The weights do not depend on the kernel before this one: the first batch is requested while that kernel
    // is still running. The kernels between two products (norms, RoPE, the attention combine) are tiny: the weight
    // stream would otherwise pause for them.
    load_weights(warp);
    pdl_wait();
    pdl_trigger();
    const int k_blocks_here = (chunks + 1) >> 1;
    for (int c0 = warp; c0 < k_blocks_here; c0 += WARPS * (UNROLL / 2)) {
        // the activations of these chunks: issued before any of the weights is waited for, so that their
        // (L2) latency overlaps the weights' (HBM) latency instead of following it
        uint4 xv[UNROLL][NT];
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            const int cc = chunk_of(c0, u);
            const int k = cc * KCHUNK + 8 * t;
            const bool kin = cc < chunks && k < K;
#pragma unroll
            for (int j = 0; j < NT; ++j) xv[u][j] = (kin && aok[j]) ? load_16(arow[j] + k) : zero;
        }
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
#pragma unroll
            for (int j = 0; j < NT; ++j) {
#pragma unroll
                for (int r = 0; r < RT; ++r) {
                    mma_bf16_16816(acc[r][j], wv[u][r][0].x, wv[u][r][1].x, wv[u][r][0].y, wv[u][r][1].y, xv[u][j].x,
                                   xv[u][j].y);
                    mma_bf16_16816(acc[r][j], wv[u][r][0].z, wv[u][r][1].z, wv[u][r][0].w, wv[u][r][1].w, xv[u][j].z,
                                   xv[u][j].w);
                }
            }
        }
        if (c0 + WARPS * (UNROLL / 2) < k_blocks_here) load_weights(c0 + WARPS * (UNROLL / 2));
    }
    // partial sums of the 8 warps -> shared memory, laid out [warp][token][row] so the final pass writes
    // consecutive output features from consecutive threads
    constexpr int ROWS = RT * 16, TOK = NT * 8;
    float* mine = red + (size_t)warp * ROWS * TOK;
#pragma unroll
    for (int r = 0; r < RT; ++r)
#pragma unroll
        for (int j = 0; j < NT; ++j) {
            const int row = r * 16 + g, tok = j * 8 + 2 * t;
            mine[(tok + 0) * ROWS + row] = acc[r][j][0];
            mine[(tok + 1) * ROWS + row] = acc[r][j][1];
            mine[(tok + 0) * ROWS + row + 8] = acc[r][j][2];
            mine[(tok + 1) * ROWS + row + 8] = acc[r][j][3];
        }
    __syncthreads();
    for (int e = threadIdx.x; e < ROWS * TOK; e += WARPS * 32) {
        const int tok = e / ROWS, row = e % ROWS;
        const int n = n0 + row;
        if (tok >= M || n >= N) continue;
        float v = 0.f;
#pragma unroll
        for (int wi = 0; wi < WARPS; ++wi) v += red[(size_t)wi * ROWS * TOK + e];
        if (swiglu) {
            // rows come in blocks of 16: 8 gate rows, then the 8 up rows of the same hidden units
            if ((row & 15) >= 8) continue;
            float u = 0.f;
#pragma unroll
            for (int wi = 0; wi < WARPS; ++wi) u += red[(size_t)wi * ROWS * TOK + e + 8];
            out[(size_t)tok * ldo + (n >> 4) * 8 + (row & 7)] = from_float<Tout>(__fmul_rn(v / (1.f + expf(-v)), u));
            continue;
        }
        if (has_bias) v += bias[n];
        Tout* dst = out + (size_t)tok * ldo + n;
        if (accumulate) v += to_float(*dst);
        *dst = from_float<Tout>(v);
    }
}

template <int NT, int RT, int UNROLL>
int launch(const void* a, int lda, const void* w, int k_blocks, VecRef bias, int has_bias, void* out, int out_dtype, int ldo,
           int accumulate, int M, int N, int K, int swiglu, cudaStream_t stream) {
    const int grid = (N + 16 * RT - 1) / (16 * RT);
    const size_t smem = (size_t)WARPS * RT * 16 * NT * 8 * sizeof(float);
    if (out_dtype == JLLM_F32) {
        auto kern = gemm_small_m_kernel<NT, RT, UNROLL, float>;
        if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        jllm_launch(kern, dim3(grid), dim3(WARPS * 32), smem, stream, LAUNCH_DEPENDENT_WANTS_L1, (const __nv_bfloat16*)a, lda,
                    (const __nv_bfloat16*)w, k_blocks, bias, has_bias, (float*)out, ldo, accumulate, M, N, K, swiglu);
    } else {
        auto kern = gemm_small_m_kernel<NT, RT, UNROLL, __nv_bfloat16>;
        if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        jllm_launch(kern, dim3(grid), dim3(WARPS * 32), smem, stream, LAUNCH_DEPENDENT_WANTS_L1, (const __nv_bfloat16*)a, lda,
                    (const __nv_bfloat16*)w, k_blocks, bias, has_bias, (__nv_bfloat16*)out, ldo, accumulate, M, N, K, swiglu);
    }
    return jllm_check_launch("gemm_small_m");
}

}  // namespace

// Returns 1 if jllm_gemm_small_m takes this product.
JLLM_EXPORT int jllm_gemm_small_m_fits(const void* a, int lda, const void* w_packed, int M, int N, int K) {
    return M >= 1 && M <= 64 && N >= 1 && K >= 8 && K % 8 == 0 && lda % 8 == 0 && ((uintptr_t)a % 16) == 0 &&
           ((uintptr_t)w_packed % 16) == 0;
}

// w_packed: ops.pack_weight of the [N, K] weight, k_blocks = ceil(K / 64) its k blocks.
JLLM_EXPORT int jllm_gemm_small_m(const void* a, int lda, const void* w, int k_blocks, const void* bias, int bias_dtype,
                                  void* out, int out_dtype, int ldo, int accumulate, int M, int N, int K,
                                  int swiglu, cudaStream_t stream) {
    JLLM_REQUIRE(jllm_gemm_small_m_fits(a, lda, w, M, N, K),
                 "gemm_small_m: needs 1 <= M <= 64, K %% 8 == 0 and 16-byte aligned rows (M=%d N=%d K=%d lda=%d)",
                 M, N, K, lda);
    JLLM_REQUIRE(k_blocks == (K + 63) / 64, "gemm_small_m: the packed weight has %d k blocks, K=%d needs %d", k_blocks, K,
                 (K + 63) / 64);
    JLLM_REQUIRE(ldo >= (swiglu ? N / 2 : N), "gemm_small_m: ldo=%d < N=%d", ldo, N);
    JLLM_REQUIRE(!swiglu || (N % 16 == 0 && !bias && !accumulate),
                 "gemm_small_m: the SwiGLU epilogue needs N %% 16 == 0, no bias and no accumulation (N=%d)", N);
    const VecRef b{bias, bias_dtype};
    const int hb = bias != nullptr;
    // How many weight rows a block takes (16 or 32) and how many batches of loads a warp keeps in flight, measured
    // on the layer shapes of an 8B model. What counts is that every SM has two resident blocks with enough bytes on
    // their way: a matrix with few rows (at most one 32-row block per SM) is cut into 16-row blocks; up to 8 tokens
    // the blocks are 16 rows with the deeper unroll, except where 32-row blocks make between one and two rounds.
    const int sms = jllm_device_sm_count() > 0 ? jllm_device_sm_count() : 1;
    const int blocks32 = (N + 31) / 32;
    bool wide = blocks32 > sms;
    int deep = 0;
    if (M <= 8) wide = blocks32 > sms && blocks32 <= 2 * sms;
    // (with the packed weight a warp's batch of four k blocks is four contiguous 2 KB pieces: twice as deep an unroll,
    // which paid on row-major weights, is slower here: gate_up at 8 rows 37.7 us against 34.8)
#define JLLM_GO(NT, RT, UN) return launch<NT, RT, UN>(a, lda, w, k_blocks, b, hb, out, out_dtype, ldo, accumulate, M, N, K, swiglu, stream)
    if (M <= 8) { if (wide) { if (deep) JLLM_GO(1, 2, 8); JLLM_GO(1, 2, 4); } if (deep) JLLM_GO(1, 1, 8); JLLM_GO(1, 1, 4); }
    if (M <= 16) { if (wide) JLLM_GO(2, 2, 4); if (deep) JLLM_GO(2, 1, 8); JLLM_GO(2, 1, 4); }
    if (M <= 32) { if (wide) JLLM_GO(4, 2, 2); JLLM_GO(4, 1, 4); }
    if (wide) JLLM_GO(8, 2, 2);
    JLLM_GO(8, 1, 2);
#undef JLLM_GO
}
