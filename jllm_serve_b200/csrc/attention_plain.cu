// Causal grouped-query attention over the paged cache, one thread block per (row, query head).
//
// The kernel of the float32 path, and the one the bfloat16 path falls back to for head sizes its
// tensor-core kernels refuse. A row at position P of request `seg` sees the keys [first, P] of that
// request, first = max(0, P + 1 - window) under a window, else 0. Two passes over the keys: the
// maximum score first (exact in any order), then exp(score - max), their sum and the weighted sum of
// the values, both in ascending key order. A row's result therefore depends on its own query and
// keys only: not on how the prompt was cut, not on the other rows of the batch, not on the pages.
//
// Layouts: q [rows, q_stride] with head h at h * head_dim; cache K and V
// [pages, kv_heads, page_size, head_dim]; out [rows, out_stride]; block_tables [segments, table_stride]
// (page id of position p of a segment: table[p / page_size]).
#include "common.cuh"

namespace {

constexpr int THREADS = 128;
constexpr int MAX_DIMS_PER_THREAD = 4;  // head_dim <= 512

template <typename T>
__global__ void __launch_bounds__(THREADS)
attention_plain_kernel(const T* __restrict__ q, int q_stride, const T* __restrict__ k_cache,
                       const T* __restrict__ v_cache, T* __restrict__ out, int out_stride,
                       const int* __restrict__ row_seg, const int* __restrict__ row_pos,
                       const int* __restrict__ block_tables, int table_stride, int heads, int kv_heads, int head_dim,
                       int page_size, int num_pages, int window, float scale) {
    extern __shared__ float smem[];
    float* qs = smem;                  // head_dim
    float* es = qs + head_dim;         // THREADS
    float* scratch = es + THREADS;     // 33
    const int r = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
    const int kvh = h / (heads / kv_heads);
    const int P = row_pos[r];
    const int first = window > 0 ? max(0, P + 1 - window) : 0;
    const int* table = block_tables + (size_t)row_seg[r] * table_stride;
    const T* qrow = q + (size_t)r * q_stride + (size_t)h * head_dim;
    for (int i = tid; i < head_dim; i += THREADS) qs[i] = to_float(qrow[i]);
    __syncthreads();

    auto key_row = [&](const T* cache, int s) -> const T* {   // nullptr only in the checked build, for a bad table
        const long long page = jllm_page_of(table, s / page_size, table_stride, num_pages);
        if (kCheckBounds && page < 0) return nullptr;
        return cache + (((size_t)page * kv_heads + kvh) * page_size + (s % page_size)) * head_dim;
    };
    auto score_of = [&](int s) -> float {
        const T* kr = key_row(k_cache, s);
        if (kCheckBounds && kr == nullptr) return -INFINITY;
        float acc = 0.f;
        for (int i = 0; i < head_dim; ++i) acc = fmaf(qs[i], to_float(kr[i]), acc);
        return __fmul_rn(acc, scale);
    };

    float m = -INFINITY;
    for (int s = first + tid; s <= P; s += THREADS) m = fmaxf(m, score_of(s));
    m = block_max(m, scratch);

    float acc[MAX_DIMS_PER_THREAD] = {};
    float sum = 0.f;
    for (int s0 = first; s0 <= P; s0 += THREADS) {
        const int s = s0 + tid;
        __syncthreads();
        es[tid] = s <= P ? expf(score_of(s) - m) : 0.f;
        __syncthreads();
        const int n = min(THREADS, P + 1 - s0);
        for (int j = 0; j < n; ++j) {
            const float e = es[j];
            sum += e;
            const T* vr = key_row(v_cache, s0 + j);
            if (kCheckBounds && vr == nullptr) continue;
#pragma unroll
            for (int c = 0; c < MAX_DIMS_PER_THREAD; ++c) {
                const int d = tid + c * THREADS;
                if (d < head_dim) acc[c] = fmaf(e, to_float(vr[d]), acc[c]);
            }
        }
    }
    const float inv = 1.f / sum;
    T* orow = out + (size_t)r * out_stride + (size_t)h * head_dim;
#pragma unroll
    for (int c = 0; c < MAX_DIMS_PER_THREAD; ++c) {
        const int d = tid + c * THREADS;
        if (d < head_dim) orow[d] = from_float<T>(__fmul_rn(acc[c], inv));
    }
}

}  // namespace

JLLM_BOUNDS_READER(attention_plain)

JLLM_EXPORT int jllm_attention_plain(const void* q, int q_stride, const void* k_cache, const void* v_cache, void* out,
                                     int out_stride, const int* row_seg, const int* row_pos, const int* block_tables,
                                     int table_stride, int rows, int heads, int kv_heads, int head_dim, int page_size,
                                     int window, float scale, int dtype, cudaStream_t stream) {
    JLLM_REQUIRE(rows >= 0 && heads > 0 && kv_heads > 0 && heads % kv_heads == 0 && head_dim > 0 && page_size > 0,
                 "attention: rows=%d heads=%d kv_heads=%d head_dim=%d page_size=%d", rows, heads, kv_heads, head_dim,
                 page_size);
    JLLM_REQUIRE(head_dim <= THREADS * MAX_DIMS_PER_THREAD, "attention: head_dim=%d is above %d", head_dim,
                 THREADS * MAX_DIMS_PER_THREAD);
    JLLM_REQUIRE(heads <= 65535 && window >= 0, "attention: heads=%d window=%d", heads, window);
    if (rows == 0) return JLLM_OK;
    const dim3 grid(rows, heads);
    const int num_pages = jllm_pool_pages();
    const size_t smem = (head_dim + THREADS + 33) * sizeof(float);
    if (dtype == JLLM_F32)
        attention_plain_kernel<float><<<grid, THREADS, smem, stream>>>(
            (const float*)q, q_stride, (const float*)k_cache, (const float*)v_cache, (float*)out, out_stride, row_seg,
            row_pos, block_tables, table_stride, heads, kv_heads, head_dim, page_size, num_pages, window, scale);
    else
        attention_plain_kernel<__nv_bfloat16><<<grid, THREADS, smem, stream>>>(
            (const __nv_bfloat16*)q, q_stride, (const __nv_bfloat16*)k_cache, (const __nv_bfloat16*)v_cache,
            (__nv_bfloat16*)out, out_stride, row_seg, row_pos, block_tables, table_stride, heads, kv_heads, head_dim,
            page_size, num_pages, window, scale);
    return jllm_check_launch("attention_plain");
}
