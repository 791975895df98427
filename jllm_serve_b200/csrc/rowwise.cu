// Row-wise kernels: embedding gather, RMSNorm, SwiGLU, and the fused per-head q/k RMSNorm +
// rotary position encoding + write of keys and values into the paged cache.
//
// All arithmetic is 32-bit float whatever the storage type; each row's result depends on that row
// alone (fixed reduction order), so it is the same in any batch.
#include <cstdlib>

#include "head_rotate.cuh"

// ---------------------------------------------------------------------------------------------------
// x[r, :] = table[ids[r], :]  (float residual stream from a float or bfloat16 table)
// ---------------------------------------------------------------------------------------------------
template <typename T>
__global__ void embed_rows_kernel(const int* __restrict__ ids, const T* __restrict__ table, float* __restrict__ x,
                                  int dim, int vocab) {
    const int r = blockIdx.x;
    int id = ids[r];
    jllm_in_bounds(id, vocab, BOUNDS_TOKEN);           // checked build: recorded
    id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);  // ids are validated on the host; never read out of bounds
    const T* src = table + (size_t)id * dim;
    float* dst = x + (size_t)r * dim;
    for (int i = threadIdx.x; i < dim; i += blockDim.x) dst[i] = to_float(src[i]);
}

JLLM_BOUNDS_READER(rowwise)

JLLM_EXPORT int jllm_embed_rows(const int* ids, const void* table, int table_dtype, float* x, int rows, int dim,
                                int vocab, cudaStream_t stream) {
    JLLM_REQUIRE(rows >= 0 && dim > 0 && vocab > 0, "embed_rows: rows=%d dim=%d vocab=%d", rows, dim, vocab);
    if (rows == 0) return JLLM_OK;
    if (table_dtype == JLLM_F32)
        embed_rows_kernel<float><<<rows, 256, 0, stream>>>(ids, (const float*)table, x, dim, vocab);
    else
        embed_rows_kernel<__nv_bfloat16><<<rows, 256, 0, stream>>>(ids, (const __nv_bfloat16*)table, x, dim, vocab);
    return jllm_check_launch("embed_rows");
}

// ---------------------------------------------------------------------------------------------------
// ids[r] < 0 stands for "row -ids[r] - 1 of the tokens the step before sampled" (still on the device, the host has not
// read them yet): put them in place. One block; a step has at most some hundreds of rows.
// ---------------------------------------------------------------------------------------------------
__global__ void feed_tokens_kernel(int* __restrict__ ids, const int* __restrict__ sampled, int rows, int sampled_rows) {
    for (int r = threadIdx.x; r < rows; r += blockDim.x) {
        const int t = ids[r];
        if (t < 0) {
            const int j = -t - 1;
            ids[r] = j < sampled_rows ? sampled[j] : 0;
        }
    }
}

JLLM_EXPORT int jllm_feed_tokens(int* ids, const int* sampled, int rows, int sampled_rows, cudaStream_t stream) {
    JLLM_REQUIRE(rows >= 0 && sampled_rows >= 0, "feed_tokens: rows=%d sampled=%d", rows, sampled_rows);
    if (rows == 0) return JLLM_OK;
    feed_tokens_kernel<<<1, 256, 0, stream>>>(ids, sampled, rows, sampled_rows);
    return jllm_check_launch("feed_tokens");
}

// ---------------------------------------------------------------------------------------------------
// RMSNorm: out[r] = (x[src(r)] * (1 / sqrt(mean(x^2) + eps))) * gain, src(r) = row_index ? row_index[r] : r
// The scale is taken in double from a float mean, as the reference does.
// ---------------------------------------------------------------------------------------------------
// (rms_scale: head_rotate.cuh)

template <typename Tout>
__global__ void rmsnorm_kernel(const float* __restrict__ x, VecRef gain, Tout* __restrict__ out,
                               const int* __restrict__ row_index, int dim, float eps) {
    __shared__ float scratch[33];
    pdl_wait();
    pdl_trigger();
    const int r = blockIdx.x;
    const float* src = x + (size_t)(row_index ? row_index[r] : r) * dim;
    float ss = 0.f;
    for (int i = threadIdx.x; i < dim; i += blockDim.x) {
        const float v = src[i];
        ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, scratch);
    const float s = rms_scale(ss, dim, eps);
    Tout* dst = out + (size_t)r * dim;
    for (int i = threadIdx.x; i < dim; i += blockDim.x) dst[i] = from_float<Tout>(__fmul_rn(__fmul_rn(src[i], s), gain[i]));
}

// The same for widths that are a multiple of 4 and at most 8192: the row is read once, as float4, and kept in
// registers between the sum of squares and the scaling.
template <typename Tout>
__global__ void __launch_bounds__(256)
rmsnorm_vec_kernel(const float* __restrict__ x, VecRef gain, Tout* __restrict__ out, const int* __restrict__ row_index,
                   int dim, float eps) {
    __shared__ float scratch[33];
    pdl_wait();
    pdl_trigger();
    const int r = blockIdx.x, n4 = dim >> 2;
    const float4* src = reinterpret_cast<const float4*>(x + (size_t)(row_index ? row_index[r] : r) * dim);
    float4 v[8];
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const int i = threadIdx.x + 256 * j;
        v[j] = i < n4 ? src[i] : make_float4(0.f, 0.f, 0.f, 0.f);
        ss = fmaf(v[j].x, v[j].x, ss);
        ss = fmaf(v[j].y, v[j].y, ss);
        ss = fmaf(v[j].z, v[j].z, ss);
        ss = fmaf(v[j].w, v[j].w, ss);
    }
    ss = block_sum(ss, scratch);
    const float s = rms_scale(ss, dim, eps);
    Tout* dst = out + (size_t)r * dim;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const int i = threadIdx.x + 256 * j;
        if (i >= n4) break;
        const float a = __fmul_rn(__fmul_rn(v[j].x, s), gain[4 * i + 0]), b = __fmul_rn(__fmul_rn(v[j].y, s), gain[4 * i + 1]);
        const float c = __fmul_rn(__fmul_rn(v[j].z, s), gain[4 * i + 2]), d = __fmul_rn(__fmul_rn(v[j].w, s), gain[4 * i + 3]);
        if constexpr (sizeof(Tout) == 4) {
            reinterpret_cast<float4*>(dst)[i] = make_float4(a, b, c, d);
        } else {
            __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
            uint2 p;
            p.x = *reinterpret_cast<uint32_t*>(&lo);
            p.y = *reinterpret_cast<uint32_t*>(&hi);
            reinterpret_cast<uint2*>(dst)[i] = p;
        }
    }
}

JLLM_EXPORT int jllm_rmsnorm(const float* x, const void* gain, int gain_dtype, void* out, int out_dtype,
                             const int* row_index, int rows, int dim, float eps, cudaStream_t stream) {
    JLLM_REQUIRE(rows >= 0 && dim > 0, "rmsnorm: rows=%d dim=%d", rows, dim);
    if (rows == 0) return JLLM_OK;
    const VecRef g{gain, gain_dtype};
    if (dim % 4 == 0 && dim <= 8192 && ((uintptr_t)x % 16) == 0 && ((uintptr_t)out % 16) == 0) {
        if (out_dtype == JLLM_F32)
            jllm_launch(rmsnorm_vec_kernel<float>, dim3(rows), dim3(256), 0, stream, true, x, g, (float*)out, row_index, dim,
                        eps);
        else
            jllm_launch(rmsnorm_vec_kernel<__nv_bfloat16>, dim3(rows), dim3(256), 0, stream, true, x, g,
                        (__nv_bfloat16*)out, row_index, dim, eps);
        return jllm_check_launch("rmsnorm");
    }
    const int threads = dim >= 2048 ? 512 : 256;
    if (out_dtype == JLLM_F32)
        jllm_launch(rmsnorm_kernel<float>, dim3(rows), dim3(threads), 0, stream, true, x, g, (float*)out, row_index, dim, eps);
    else
        jllm_launch(rmsnorm_kernel<__nv_bfloat16>, dim3(rows), dim3(threads), 0, stream, true, x, g, (__nv_bfloat16*)out,
                    row_index, dim, eps);
    return jllm_check_launch("rmsnorm");
}

// ---------------------------------------------------------------------------------------------------
// SwiGLU: h[r, j] = silu(gate_up[r, j]) * gate_up[r, hidden + j],  silu(g) = g / (1 + exp(-g))
// ---------------------------------------------------------------------------------------------------
template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ gate_up, T* __restrict__ h, int hidden, size_t total) {
    pdl_wait();
    pdl_trigger();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t r = i / hidden, j = i - r * hidden;
        const float g = to_float(gate_up[r * 2 * hidden + j]);
        const float u = to_float(gate_up[r * 2 * hidden + hidden + j]);
        h[i] = from_float<T>(__fmul_rn(g / (1.f + expf(-g)), u));
    }
}

JLLM_EXPORT int jllm_swiglu(const void* gate_up, void* h, int dtype, int rows, int hidden, cudaStream_t stream) {
    JLLM_REQUIRE(rows >= 0 && hidden > 0, "swiglu: rows=%d hidden=%d", rows, hidden);
    if (rows == 0) return JLLM_OK;
    const size_t total = (size_t)rows * hidden;
    const size_t most = (size_t)(jllm_device_sm_count() > 0 ? jllm_device_sm_count() : 1) * 16;   // the kernel strides
    const int blocks = (int)((total + 255) / 256 > most ? most : (total + 255) / 256);
    if (dtype == JLLM_F32)
        jllm_launch(swiglu_kernel<float>, dim3(blocks), dim3(256), 0, stream, true, (const float*)gate_up, (float*)h, hidden,
                    total);
    else
        jllm_launch(swiglu_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, true, (const __nv_bfloat16*)gate_up,
                    (__nv_bfloat16*)h, hidden, total);
    return jllm_check_launch("swiglu");
}

// ---------------------------------------------------------------------------------------------------
// Per (row, head): optional RMSNorm over the head, rotate-half RoPE over the first rotary_dim values,
// then queries go back in place and keys / values go into the paged cache.
//
// qkv is [rows, row_stride] with queries, keys, values side by side ((heads + 2 kv_heads) * head_dim values;
// heads * head_dim when the run reads another run's cache and writes no keys or values). The cache of one layer run is
// K[pages, kv_heads, page_size, head_dim] and V alike; row r is written at slot[r] = page * page_size + offset.
// cos/sin are [positions, rotary_dim / 2] float tables (angles made in double on the host).
// ---------------------------------------------------------------------------------------------------
template <typename T>
__global__ void qk_norm_rope_store_kernel(T* __restrict__ qkv, VecRef q_gain, VecRef k_gain, int use_norm, float eps,
                                          const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                                          int rotary_dim, const int* __restrict__ positions,
                                          const int* __restrict__ slots, T* __restrict__ k_cache,
                                          T* __restrict__ v_cache, int heads, int kv_heads, int head_dim,
                                          int page_size, int num_slots, int row_stride) {
    extern __shared__ float vec[];  // head_dim floats + 33 scratch
    float* scratch = vec + head_dim;
    pdl_wait();
    pdl_trigger();
    const int r = blockIdx.x, h = blockIdx.y;
    T* src = qkv + (size_t)r * row_stride + (size_t)h * head_dim;
    const bool is_q = h < heads, is_k = !is_q && h < heads + kv_heads;
    for (int i = threadIdx.x; i < head_dim; i += blockDim.x) vec[i] = to_float(src[i]);
    __syncthreads();
    if (is_q || is_k) {
        if (use_norm) {
            float ss = 0.f;
            for (int i = threadIdx.x; i < head_dim; i += blockDim.x) ss = fmaf(vec[i], vec[i], ss);
            ss = block_sum(ss, scratch);
            const float s = rms_scale(ss, head_dim, eps);
            const VecRef g = is_q ? q_gain : k_gain;
            for (int i = threadIdx.x; i < head_dim; i += blockDim.x) vec[i] = __fmul_rn(__fmul_rn(vec[i], s), g[i]);
            __syncthreads();
        }
        if (rotary_dim > 0) {
            const int half = rotary_dim >> 1;
            const float* c = cos_t + (size_t)positions[r] * half;
            const float* s = sin_t + (size_t)positions[r] * half;
            for (int i = threadIdx.x; i < half; i += blockDim.x) {
                const float a = vec[i], b = vec[i + half];
                vec[i] = __fsub_rn(__fmul_rn(a, c[i]), __fmul_rn(b, s[i]));
                vec[i + half] = __fadd_rn(__fmul_rn(b, c[i]), __fmul_rn(a, s[i]));
            }
            __syncthreads();
        }
    }
    if (is_q) {
        for (int i = threadIdx.x; i < head_dim; i += blockDim.x) src[i] = from_float<T>(vec[i]);
    } else {
        const int kvh = is_k ? h - heads : h - heads - kv_heads;
        const int slot = slots[r];
        if (!jllm_in_bounds(slot, num_slots, BOUNDS_SLOT)) return;      // checked build: the write is dropped
        const size_t page = slot / page_size, off = slot % page_size;
        T* dst = (is_k ? k_cache : v_cache) + ((page * kv_heads + kvh) * page_size + off) * head_dim;
        for (int i = threadIdx.x; i < head_dim; i += blockDim.x) dst[i] = from_float<T>(vec[i]);
    }
}

// The same with one warp per (row, head), for head sizes 64, 128 and 256 rotated over their whole width: lane l
// owns V = head_dim / 64 neighbouring values of the first half and their partners in the second half, so the
// rotation needs no exchange and the sum of squares is a warp shuffle; 8 heads per block, no shared memory.
template <typename T, int V>
__global__ void __launch_bounds__(256)
qk_norm_rope_store_warp_kernel(T* __restrict__ qkv, VecRef q_gain, VecRef k_gain, int use_norm, float eps,
                               const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                               const int* __restrict__ positions, const int* __restrict__ slots, T* __restrict__ k_cache,
                               T* __restrict__ v_cache, int heads, int kv_heads, int page_size, int num_slots, int row_stride,
                               int heads_total, long long items) {
    constexpr int HD = 64 * V, HALF = 32 * V;
    pdl_wait();
    pdl_trigger();
    const long long item = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
    if (item >= items) return;
    const int r = (int)(item / heads_total), h = (int)(item % heads_total), lane = threadIdx.x & 31;
    T* src = qkv + (size_t)r * row_stride + (size_t)h * HD;
    const bool is_q = h < heads, is_k = !is_q && h < heads + kv_heads;
    float a[V], b[V];
#pragma unroll
    for (int i = 0; i < V; ++i) {
        a[i] = to_float(src[lane * V + i]);
        b[i] = to_float(src[HALF + lane * V + i]);
    }
    if (is_q || is_k)
        head_norm_rope<V>(a, b, lane, use_norm, eps, is_q ? q_gain : k_gain, cos_t + (size_t)positions[r] * HALF,
                          sin_t + (size_t)positions[r] * HALF);
    T* dst = src;
    if (!is_q) {
        const int kvh = is_k ? h - heads : h - heads - kv_heads;
        const int slot = slots[r];
        if (!jllm_in_bounds(slot, num_slots, BOUNDS_SLOT)) return;      // checked build: the write is dropped
        const size_t page = slot / page_size, off = slot % page_size;
        dst = (is_k ? k_cache : v_cache) + ((page * kv_heads + kvh) * page_size + off) * HD;
    }
#pragma unroll
    for (int i = 0; i < V; ++i) {
        dst[lane * V + i] = from_float<T>(a[i]);
        dst[HALF + lane * V + i] = from_float<T>(b[i]);
    }
}

// The same for bfloat16 with 16-byte accesses: 4 V lanes share one (row, head), each owning 8 neighbouring values of
// the first half and their partners in the second half; a warp takes 8 / V heads of a row side by side (they are
// neighbours in memory), so that it has 1 KB of loads in flight instead of 128 bytes. The arithmetic of one value
// is that of the kernels above.
template <int V>
__global__ void __launch_bounds__(256)
qk_norm_rope_store_vec_kernel(__nv_bfloat16* __restrict__ qkv, VecRef q_gain, VecRef k_gain, int use_norm, float eps,
                              const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                              const int* __restrict__ positions, const int* __restrict__ slots,
                              __nv_bfloat16* __restrict__ k_cache, __nv_bfloat16* __restrict__ v_cache, int heads,
                              int kv_heads, int page_size, int num_slots, int row_stride, int heads_total, long long items) {
    constexpr int HD = 64 * V, HALF = 32 * V, LANES = 4 * V, PER_WARP = 32 / LANES;
    pdl_wait();
    pdl_trigger();
    const int lane = threadIdx.x & 31, sub = lane % LANES;
    const long long item = ((long long)blockIdx.x * 8 + (threadIdx.x >> 5)) * PER_WARP + lane / LANES;
    const bool live = item < items;
    const int r = live ? (int)(item / heads_total) : 0, h = live ? (int)(item % heads_total) : 0;
    __nv_bfloat16* src = qkv + (size_t)r * row_stride + (size_t)h * HD;
    const bool is_q = h < heads, is_k = !is_q && h < heads + kv_heads;
    float a[8], b[8];
    {
        const uint4 ua = live ? *reinterpret_cast<const uint4*>(src + sub * 8) : make_uint4(0, 0, 0, 0);
        const uint4 ub = live ? *reinterpret_cast<const uint4*>(src + HALF + sub * 8) : make_uint4(0, 0, 0, 0);
        const __nv_bfloat162* pa = reinterpret_cast<const __nv_bfloat162*>(&ua);
        const __nv_bfloat162* pb = reinterpret_cast<const __nv_bfloat162*>(&ub);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 fa = __bfloat1622float2(pa[i]), fb = __bfloat1622float2(pb[i]);
            a[2 * i] = fa.x; a[2 * i + 1] = fa.y;
            b[2 * i] = fb.x; b[2 * i + 1] = fb.y;
        }
    }
    if (is_q || is_k) {
        if (use_norm) {
            float ss = 0.f;
#pragma unroll
            for (int i = 0; i < 8; ++i) ss = fmaf(a[i], a[i], ss);
#pragma unroll
            for (int i = 0; i < 8; ++i) ss = fmaf(b[i], b[i], ss);
#pragma unroll
            for (int o = LANES / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
            const float s = rms_scale(ss, HD, eps);
            const VecRef g = is_q ? q_gain : k_gain;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                a[i] = __fmul_rn(__fmul_rn(a[i], s), g[sub * 8 + i]);
                b[i] = __fmul_rn(__fmul_rn(b[i], s), g[HALF + sub * 8 + i]);
            }
        }
        const float4* c4 = reinterpret_cast<const float4*>(cos_t + (size_t)positions[r] * HALF + sub * 8);
        const float4* s4 = reinterpret_cast<const float4*>(sin_t + (size_t)positions[r] * HALF + sub * 8);
        const float4 c0 = c4[0], c1 = c4[1], s0 = s4[0], s1 = s4[1];
        const float c[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
        const float sn[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const float x0 = a[i], x1 = b[i];
            a[i] = __fsub_rn(__fmul_rn(x0, c[i]), __fmul_rn(x1, sn[i]));
            b[i] = __fadd_rn(__fmul_rn(x1, c[i]), __fmul_rn(x0, sn[i]));
        }
    }
    if (!live) return;
    __nv_bfloat16* dst = src;
    if (!is_q) {
        const int kvh = is_k ? h - heads : h - heads - kv_heads;
        const int slot = slots[r];
        if (!jllm_in_bounds(slot, num_slots, BOUNDS_SLOT)) return;      // checked build: the write is dropped
        const size_t page = slot / page_size, off = slot % page_size;
        dst = (is_k ? k_cache : v_cache) + ((page * kv_heads + kvh) * page_size + off) * HD;
    }
    uint4 oa, ob;
    __nv_bfloat162* qa = reinterpret_cast<__nv_bfloat162*>(&oa);
    __nv_bfloat162* qb = reinterpret_cast<__nv_bfloat162*>(&ob);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        qa[i] = __floats2bfloat162_rn(a[2 * i], a[2 * i + 1]);
        qb[i] = __floats2bfloat162_rn(b[2 * i], b[2 * i + 1]);
    }
    *reinterpret_cast<uint4*>(dst + sub * 8) = oa;
    *reinterpret_cast<uint4*>(dst + HALF + sub * 8) = ob;
}

JLLM_EXPORT int jllm_qk_norm_rope_store(void* qkv, int dtype, const void* q_gain, const void* k_gain, int gain_dtype,
                                        int use_norm, float eps, const float* cos_t, const float* sin_t,
                                        int rotary_dim, const int* positions, const int* slots, void* k_cache,
                                        void* v_cache, int write_kv, int rows, int row_stride, int heads, int kv_heads,
                                        int head_dim, int page_size, cudaStream_t stream) {
    JLLM_REQUIRE(rows >= 0 && heads > 0 && kv_heads > 0 && head_dim > 0 && page_size > 0,
                 "qk_norm_rope_store: rows=%d heads=%d kv_heads=%d head_dim=%d page_size=%d", rows, heads, kv_heads,
                 head_dim, page_size);
    JLLM_REQUIRE(rotary_dim >= 0 && rotary_dim % 2 == 0 && rotary_dim <= head_dim,
                 "qk_norm_rope_store: rotary_dim=%d must be even and at most head_dim=%d", rotary_dim, head_dim);
    JLLM_REQUIRE(row_stride >= (write_kv ? heads + 2 * kv_heads : heads) * head_dim,
                 "qk_norm_rope_store: row_stride=%d is too small", row_stride);
    JLLM_REQUIRE(head_dim <= 8192, "qk_norm_rope_store: head_dim=%d is above 8192", head_dim);
    if (rows == 0) return JLLM_OK;
    const int num_slots = (int)min((long long)jllm_pool_pages() * page_size, 2147483647ll);   // 0 = not known
    const dim3 grid(rows, write_kv ? heads + 2 * kv_heads : heads);
    const int threads = head_dim <= 64 ? 32 : (head_dim <= 128 ? 64 : 128);
    const size_t smem = (head_dim + 33) * sizeof(float);
    const VecRef qg{q_gain, gain_dtype}, kg{k_gain, gain_dtype};
    if ((head_dim == 64 || head_dim == 128 || head_dim == 256) && rotary_dim == head_dim) {
        const int heads_total = write_kv ? heads + 2 * kv_heads : heads;
        const long long items = (long long)rows * heads_total;
        const dim3 wgrid((unsigned)((items + 7) / 8));
#define JLLM_WARP_ROPE(T, V)                                                                                          \
    jllm_launch(qk_norm_rope_store_warp_kernel<T, V>, wgrid, dim3(256), 0, stream, true, (T*)qkv, qg, kg, use_norm, eps, \
                cos_t, sin_t, positions, slots, (T*)k_cache, (T*)v_cache, heads, kv_heads, page_size, num_slots, row_stride,      \
                heads_total, items)
        const int v = head_dim / 64;
        // the 16-byte kernel from 32 rows on (fewer rows are too few warps for it; JLLM_B200_ROPE_VEC_MIN_ROWS moves that)
        static const int vec_min_rows = [] {
            const char* e = getenv("JLLM_B200_ROPE_VEC_MIN_ROWS");
            return e ? atoi(e) : 32;
        }();
        if (dtype == JLLM_BF16 && rows >= vec_min_rows && row_stride % 8 == 0 && ((uintptr_t)qkv % 16) == 0 && ((uintptr_t)k_cache % 16) == 0 &&
            ((uintptr_t)v_cache % 16) == 0 && ((uintptr_t)cos_t % 16) == 0 && ((uintptr_t)sin_t % 16) == 0) {
            const long long per_block = 8 * (8 / v);
            const dim3 vgrid((unsigned)((items + per_block - 1) / per_block));
#define JLLM_VEC_ROPE(V)                                                                                              \
    jllm_launch(qk_norm_rope_store_vec_kernel<V>, vgrid, dim3(256), 0, stream, true, (__nv_bfloat16*)qkv, qg, kg,     \
                use_norm, eps, cos_t, sin_t, positions, slots, (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, heads, \
                kv_heads, page_size, num_slots, row_stride, heads_total, items)
            if (v == 1) JLLM_VEC_ROPE(1); else if (v == 2) JLLM_VEC_ROPE(2); else JLLM_VEC_ROPE(4);
#undef JLLM_VEC_ROPE
            return jllm_check_launch("qk_norm_rope_store");
        }
        if (dtype == JLLM_F32) {
            if (v == 1) JLLM_WARP_ROPE(float, 1); else if (v == 2) JLLM_WARP_ROPE(float, 2); else JLLM_WARP_ROPE(float, 4);
        } else {
            if (v == 1) JLLM_WARP_ROPE(__nv_bfloat16, 1); else if (v == 2) JLLM_WARP_ROPE(__nv_bfloat16, 2);
            else JLLM_WARP_ROPE(__nv_bfloat16, 4);
        }
#undef JLLM_WARP_ROPE
        return jllm_check_launch("qk_norm_rope_store");
    }
    if (dtype == JLLM_F32)
        jllm_launch(qk_norm_rope_store_kernel<float>, grid, dim3(threads), smem, stream, true,
            (float*)qkv, qg, kg, use_norm, eps, cos_t, sin_t, rotary_dim, positions, slots, (float*)k_cache,
            (float*)v_cache, heads, kv_heads, head_dim, page_size, num_slots, row_stride);
    else
        jllm_launch(qk_norm_rope_store_kernel<__nv_bfloat16>, grid, dim3(threads), smem, stream, true,
            (__nv_bfloat16*)qkv, qg, kg, use_norm, eps, cos_t, sin_t, rotary_dim, positions, slots,
            (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, heads, kv_heads, head_dim, page_size, num_slots, row_stride);
    return jllm_check_launch("qk_norm_rope_store");
}
