// Paged grouped-query attention for rows that each bring ONE query position (decode steps), bfloat16.
//
// The work is a stream of the request's keys and values, shared by the G = heads / kv_heads query heads
// of one kv head, so a block handles (row, kv head, split of the key range) and every key and value it
// loads serves all G heads. The G heads are the M side of mma.sync.m16n8k16 (up to 16; rows beyond G are
// zero), keys are the N side of Q K^T and the K side of P V. Keys and values go from global memory
// straight into tensor-core fragments with 16-byte loads:
//   * Q K^T: thread (g, t) loads 8 contiguous head_dim values of key g; the k index inside a 32-wide
//     chunk is permuted the same way for Q, which a dot product does not notice;
//   * P V: thread (g, t) loads 8 contiguous dims [8g, 8g+8) of the four keys 2t, 2t+1, 2t+8, 2t+9 and
//     pairs them with byte permutes; the output dims come out permuted (dim = 8 n + j in the j-th MMA)
//     and are put back in order when they are written.
// Each warp walks 16-key blocks of the block's key range with an online softmax (float32, base 2);
// the warps' states are merged in shared memory, and if the key range was split over several blocks
// the partial (max, sum, output) go to scratch memory and a second kernel combines them.
//
// Keys outside [first, P] are never loaded (their pages may be gone or hold other requests' data).
// Requirements: bfloat16, head_dim a multiple of 16 and at most 256, G <= 16.
#include "common.cuh"

namespace {

constexpr int WARPS = 4;
constexpr float LOG2E = 1.4426950408889634f;

__device__ __forceinline__ void mma_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                          uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

__device__ __forceinline__ uint4 ld16(const __nv_bfloat16* p) { return *reinterpret_cast<const uint4*>(p); }

__device__ __forceinline__ uint32_t reg_of(const uint4& v, int i) {
    return i == 0 ? v.x : (i == 1 ? v.y : (i == 2 ? v.z : v.w));
}

// HDC = ceil(head_dim / 64): the output is kept as HDC chunks of 64 dims (8 MMAs of 8 dims each)
template <int HDC>
__global__ void __launch_bounds__(WARPS * 32)
attention_decode_kernel(const __nv_bfloat16* __restrict__ q, int q_stride, const __nv_bfloat16* __restrict__ k_cache,
                        const __nv_bfloat16* __restrict__ v_cache, __nv_bfloat16* __restrict__ out, int out_stride,
                        const int* __restrict__ row_seg, const int* __restrict__ row_pos,
                        const int* __restrict__ block_tables, int table_stride, int heads, int kv_heads, int head_dim,
                        int page_size, int num_pages, int window, float scale_log2, int splits,
                        float* __restrict__ part_o, float* __restrict__ part_ml) {
    extern __shared__ float smem[];  // [WARPS][16][head_dim] outputs, then [WARPS][16][2] (max, sum)
    const int r = blockIdx.x, kvh = blockIdx.y, split = blockIdx.z;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int G = heads / kv_heads;
    pdl_wait();
    pdl_trigger();
    const int P = row_pos[r];
    const int first = window > 0 ? max(0, P + 1 - window) : 0;
    const int n_keys = P + 1 - first;
    // the block's share of the keys, in whole 16-key blocks
    const int blocks_total = (n_keys + 15) >> 4;
    const int blocks_per_split = (blocks_total + splits - 1) / splits;
    const int blk_lo = split * blocks_per_split, blk_hi = min(blocks_total, blk_lo + blocks_per_split);
    const int* table = block_tables + (size_t)row_seg[r] * table_stride;
    const uint4 zero4 = make_uint4(0, 0, 0, 0);

    // Q fragments: rows g and g + 8 of the (up to 16) heads of this kv head, k permuted per 32-wide chunk
    constexpr int KC = HDC * 2;  // 32-wide chunks of head_dim
    uint4 qf[KC][2];
#pragma unroll
    for (int c = 0; c < KC; ++c)
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int row = g + 8 * h, d = c * 32 + 8 * t;
            qf[c][h] = (row < G && d < head_dim)
                           ? ld16(q + (size_t)r * q_stride + (size_t)(kvh * G + row) * head_dim + d) : zero4;
        }

    float o[HDC][8][4];
#pragma unroll
    for (int c = 0; c < HDC; ++c)
#pragma unroll
        for (int j = 0; j < 8; ++j)
#pragma unroll
            for (int i = 0; i < 4; ++i) o[c][j][i] = 0.f;
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};

    const size_t page_stride = (size_t)kv_heads * page_size * head_dim;
    for (int blk = blk_lo + warp; blk < blk_hi; blk += WARPS) {
        const int base = first + blk * 16;
        // ---- scores of 16 keys: two 8-key tiles ----
        float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
        for (int tile = 0; tile < 2; ++tile) {
            const int key = base + tile * 8 + g;
            bool ok = key <= P;
            const __nv_bfloat16* krow = nullptr;
            if (ok) {
                const long long page = jllm_page_of(table, key / page_size, table_stride, num_pages);
                if (kCheckBounds && page < 0) ok = false;      // checked build: a bad table entry reads nothing
                else krow = k_cache + (size_t)page * page_stride + ((size_t)kvh * page_size + key % page_size) * head_dim;
            }
#pragma unroll
            for (int c = 0; c < KC; ++c) {
                const int d = c * 32 + 8 * t;
                const uint4 kv = (ok && d < head_dim) ? ld16(krow + d) : zero4;
                mma_16816(s[tile], qf[c][0].x, qf[c][1].x, qf[c][0].y, qf[c][1].y, kv.x, kv.y);
                mma_16816(s[tile], qf[c][0].z, qf[c][1].z, qf[c][0].w, qf[c][1].w, kv.z, kv.w);
            }
        }
        // ---- mask, online softmax (rows g and g + 8) ----
        float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int tile = 0; tile < 2; ++tile)
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int key = base + tile * 8 + 2 * t + (i & 1);
                s[tile][i] = key <= P ? s[tile][i] * scale_log2 : -INFINITY;
                mx[i >> 1] = fmaxf(mx[i >> 1], s[tile][i]);
            }
        float corr[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
            mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
            const float m_new = fmaxf(m[h], mx[h]);   // finite: the block holds at least one visible key
            corr[h] = exp2f(m[h] - m_new);
            m[h] = m_new;
            l[h] *= corr[h];
        }
        float p[2][4];
#pragma unroll
        for (int tile = 0; tile < 2; ++tile)
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                p[tile][i] = exp2f(s[tile][i] - m[i >> 1]);
                l[i >> 1] += p[tile][i];
            }
        const uint32_t pa0 = pack_bf16(p[0][0], p[0][1]), pa1 = pack_bf16(p[0][2], p[0][3]);
        const uint32_t pa2 = pack_bf16(p[1][0], p[1][1]), pa3 = pack_bf16(p[1][2], p[1][3]);
        // ---- values of the 4 keys this thread pairs up ----
        const __nv_bfloat16* vrow[4];
        bool vok[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int key = base + 2 * t + (i & 1) + 8 * (i >> 1);
            vok[i] = key <= P;
            vrow[i] = nullptr;
            if (vok[i]) {
                const long long page = jllm_page_of(table, key / page_size, table_stride, num_pages);
                if (kCheckBounds && page < 0) vok[i] = false;
                else vrow[i] = v_cache + (size_t)page * page_stride + ((size_t)kvh * page_size + key % page_size) * head_dim;
            }
        }
#pragma unroll
        for (int c = 0; c < HDC; ++c) {
            const int d = c * 64 + 8 * g;
            uint4 vv[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) vv[i] = (vok[i] && d < head_dim) ? ld16(vrow[i] + d) : zero4;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                o[c][j][0] *= corr[0];
                o[c][j][1] *= corr[0];
                o[c][j][2] *= corr[1];
                o[c][j][3] *= corr[1];
                const uint32_t sel = (j & 1) ? 0x7632u : 0x5410u;
                const uint32_t b0 = __byte_perm(reg_of(vv[0], j >> 1), reg_of(vv[1], j >> 1), sel);
                const uint32_t b1 = __byte_perm(reg_of(vv[2], j >> 1), reg_of(vv[3], j >> 1), sel);
                mma_16816(o[c][j], pa0, pa1, pa2, pa3, b0, b1);
            }
        }
    }
    // ---- merge the warps: (max, sum) first, then the outputs scaled to the common max ----
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        l[h] += __shfl_xor_sync(0xffffffffu, l[h], 1);
        l[h] += __shfl_xor_sync(0xffffffffu, l[h], 2);
    }
    float* so = smem;
    float* sml = smem + (size_t)WARPS * 16 * head_dim;
    if (t == 0) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            sml[(warp * 16 + g + 8 * h) * 2 + 0] = m[h];
            sml[(warp * 16 + g + 8 * h) * 2 + 1] = l[h];
        }
    }
    __syncthreads();
    float scale_w[2], m_all[2], l_all[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int row = g + 8 * h;
        float mm = -INFINITY;
        for (int w = 0; w < WARPS; ++w) mm = fmaxf(mm, sml[(w * 16 + row) * 2]);
        float ll = 0.f;
        for (int w = 0; w < WARPS; ++w) {
            const float mw = sml[(w * 16 + row) * 2];
            ll += mw == -INFINITY ? 0.f : sml[(w * 16 + row) * 2 + 1] * exp2f(mw - mm);
        }
        m_all[h] = mm;
        l_all[h] = ll;
        scale_w[h] = m[h] == -INFINITY ? 0.f : exp2f(m[h] - mm);
    }
#pragma unroll
    for (int c = 0; c < HDC; ++c)
#pragma unroll
        for (int j = 0; j < 8; ++j)
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int row = g + 8 * (i >> 1);
                const int d = c * 64 + 8 * (2 * t + (i & 1)) + j;
                if (d < head_dim) so[((size_t)warp * 16 + row) * head_dim + d] = o[c][j][i] * scale_w[i >> 1];
            }
    __syncthreads();
    for (int e = threadIdx.x; e < G * head_dim; e += WARPS * 32) {
        const int row = e / head_dim, d = e % head_dim;
        float acc = 0.f;
        for (int w = 0; w < WARPS; ++w) acc += so[((size_t)w * 16 + row) * head_dim + d];
        const int head = kvh * G + row;
        // every thread recomputes its row's totals from shared memory (cheap, and no extra barrier)
        float mm = -INFINITY, ll = 0.f;
        for (int w = 0; w < WARPS; ++w) mm = fmaxf(mm, sml[(w * 16 + row) * 2]);
        for (int w = 0; w < WARPS; ++w) {
            const float mw = sml[(w * 16 + row) * 2];
            ll += mw == -INFINITY ? 0.f : sml[(w * 16 + row) * 2 + 1] * exp2f(mw - mm);
        }
        if (splits == 1) {
            out[(size_t)r * out_stride + (size_t)head * head_dim + d] = __float2bfloat16_rn(acc / ll);
        } else {
            const size_t slot = ((size_t)r * heads + head) * splits + split;
            part_o[slot * head_dim + d] = acc;
            if (d == 0) {
                part_ml[slot * 2 + 0] = mm;
                part_ml[slot * 2 + 1] = ll;
            }
        }
    }
    (void)m_all;
    (void)l_all;
}

// out[r, head] = sum_s o_s 2^(m_s - M) / sum_s l_s 2^(m_s - M) over the splits, in the order of the splits
__global__ void attention_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                         __nv_bfloat16* __restrict__ out, int out_stride, int heads, int head_dim,
                                         int splits) {
    constexpr int MAX_SPLITS = 32;
    __shared__ float weight[MAX_SPLITS];
    __shared__ float inv_total;
    pdl_wait();
    pdl_trigger();
    const int r = blockIdx.x, head = blockIdx.y;
    const size_t slot0 = ((size_t)r * heads + head) * splits;
    if (threadIdx.x < 32) {
        // one lane per split: all (max, sum) pairs are fetched at once; the sums over splits go in split order
        const int s = threadIdx.x;
        const float ms = s < splits ? part_ml[(slot0 + s) * 2] : -INFINITY;
        const float ls = s < splits ? part_ml[(slot0 + s) * 2 + 1] : 0.f;
        float M = ms;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, o));
        const float w = ms == -INFINITY ? 0.f : exp2f(ms - M);
        weight[s] = w;
        float L = 0.f;
        for (int i = 0; i < splits; ++i) L += __shfl_sync(0xffffffffu, ls * w, i);
        if (s == 0) inv_total = 1.f / L;
    }
    __syncthreads();
    const float inv = inv_total;
    for (int d = threadIdx.x; d < head_dim; d += blockDim.x) {
        float acc = 0.f;
#pragma unroll 8
        for (int s = 0; s < splits; ++s) acc += part_o[(slot0 + s) * head_dim + d] * weight[s];
        out[(size_t)r * out_stride + (size_t)head * head_dim + d] = __float2bfloat16_rn(acc * inv);
    }
}

}  // namespace

JLLM_BOUNDS_READER(attention_decode)

namespace {
// a test's switch: the partials are added up by the combine kernels, as where the library's counters do not reach
int g_separate_combine = 0;
}
JLLM_EXPORT void jllm_attention_decode_separate_combine(int on) { g_separate_combine = on; }

#include "attention_decode_staged.cuh"

// Floats of scratch the split path needs: (head_dim + 2) per (row, head, split).
JLLM_EXPORT long long jllm_attention_decode_scratch_floats(int rows, int heads, int head_dim, int splits) {
    return splits <= 1 ? 0 : (long long)rows * heads * splits * (head_dim + 2);
}

namespace {

int decode_split(const void* q, int q_stride, const void* k_cache, const void* v_cache, void* out, int out_stride,
                 const int* row_seg, const int* row_pos, const int* block_tables, int table_stride, int rows, int heads,
                 int kv_heads, int head_dim, int page_size, int window, float scale, int splits, float* scratch,
                 const staged::Fresh& fresh, cudaStream_t stream) {
    JLLM_REQUIRE(rows >= 0 && heads > 0 && kv_heads > 0 && heads % kv_heads == 0 && page_size > 0,
                 "attention_decode: rows=%d heads=%d kv_heads=%d page_size=%d", rows, heads, kv_heads, page_size);
    JLLM_REQUIRE(head_dim % 16 == 0 && head_dim >= 16 && head_dim <= 256,
                 "attention_decode: head_dim=%d must be a multiple of 16 in [16, 256]", head_dim);
    JLLM_REQUIRE(heads / kv_heads <= 16, "attention_decode: %d query heads per kv head, at most 16", heads / kv_heads);
    JLLM_REQUIRE(q_stride % 8 == 0 && ((uintptr_t)q % 16) == 0 && ((uintptr_t)k_cache % 16) == 0 &&
                     ((uintptr_t)v_cache % 16) == 0,
                 "attention_decode: q, K and V must be 16-byte aligned (q_stride=%d)", q_stride);
    JLLM_REQUIRE(splits >= 1 && splits <= 32 && kv_heads <= 65535, "attention_decode: splits=%d must be in [1, 32]", splits);
    JLLM_REQUIRE(splits == 1 || scratch != nullptr, "attention_decode: %d splits need scratch memory", splits);
    if (rows == 0) return JLLM_OK;
    const dim3 grid(rows, kv_heads, splits);
    const size_t smem = ((size_t)WARPS * 16 * head_dim + WARPS * 16 * 2) * sizeof(float);
    float* part_o = scratch;
    float* part_ml = scratch ? scratch + (size_t)rows * heads * splits * head_dim : nullptr;
    const float scale_log2 = scale * LOG2E;
    const int hdc = (head_dim + 63) / 64;
    if (head_dim == 64 || head_dim == 128 || head_dim == 256) {
        // the common head sizes stream the cache through a shared-memory ring (attention_decode_staged.cuh)
        // The last block of a (row, kv head) pair adds the pair's partials up itself where the library's counters reach,
        // up to 8 splits: with more (few rows, long ranges) one block's adding of all of a pair's parts is slower than
        // the combine kernel's block per head (a step of one row at 4,096 keys: 3.46 ms against 3.43 ms).
        int* counters = splits > 1 && splits <= 8 && (long long)rows * kv_heads <= staged::PAIR_COUNTERS && !g_separate_combine
                            ? staged::pair_counters() : nullptr;
#define JLLM_STAGED(HD)                                                                                             \
    staged::launch<HD>(q, q_stride, k_cache, v_cache, out, out_stride, row_seg, row_pos, block_tables, table_stride, \
                       rows, heads, kv_heads, page_size, window, scale_log2, splits, part_o, part_ml, counters, fresh, stream)
        if (head_dim == 64) JLLM_STAGED(64); else if (head_dim == 128) JLLM_STAGED(128); else JLLM_STAGED(256);
#undef JLLM_STAGED
        int rc2 = jllm_check_launch("attention_decode_staged");
        if (rc2 != JLLM_OK || splits == 1 || counters != nullptr) return rc2;
        jllm_launch(attention_combine_kernel, dim3(rows, heads), dim3(128), 0, stream, true, (const float*)part_o,
                    (const float*)part_ml, (__nv_bfloat16*)out, out_stride, heads, head_dim, splits);
        return jllm_check_launch("attention_combine");
    }
    JLLM_REQUIRE(fresh.qkv == nullptr, "attention_decode: head_dim=%d has no kernel that norms and rotates its own row", head_dim);
#define JLLM_LAUNCH(HDC)                                                                                            \
    {                                                                                                               \
        auto kern = attention_decode_kernel<HDC>;                                                                   \
        if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);   \
        kern<<<grid, WARPS * 32, smem, stream>>>((const __nv_bfloat16*)q, q_stride, (const __nv_bfloat16*)k_cache,  \
                                                 (const __nv_bfloat16*)v_cache, (__nv_bfloat16*)out, out_stride,    \
                                                 row_seg, row_pos, block_tables, table_stride, heads, kv_heads,     \
                                                 head_dim, page_size, jllm_pool_pages(), window, scale_log2, splits, \
                                                 part_o, part_ml);                                                  \
    }
    if (hdc == 1) JLLM_LAUNCH(1) else if (hdc == 2) JLLM_LAUNCH(2) else if (hdc == 3) JLLM_LAUNCH(3) else JLLM_LAUNCH(4)
#undef JLLM_LAUNCH
    int rc = jllm_check_launch("attention_decode");
    if (rc != JLLM_OK || splits == 1) return rc;
    attention_combine_kernel<<<dim3(rows, heads), 128, 0, stream>>>(part_o, part_ml, (__nv_bfloat16*)out, out_stride,
                                                                   heads, head_dim, splits);
    return jllm_check_launch("attention_combine");
}

}  // namespace

JLLM_EXPORT int jllm_attention_decode(const void* q, int q_stride, const void* k_cache, const void* v_cache, void* out,
                                      int out_stride, const int* row_seg, const int* row_pos, const int* block_tables,
                                      int table_stride, int rows, int heads, int kv_heads, int head_dim, int page_size,
                                      int window, float scale, int splits, float* scratch, cudaStream_t stream) {
    return decode_split(q, q_stride, k_cache, v_cache, out, out_stride, row_seg, row_pos, block_tables, table_stride, rows,
                        heads, kv_heads, head_dim, page_size, window, scale, splits, scratch, staged::Fresh{}, stream);
}

// Floats of scratch of the evenly dealt variant: (head_dim + 2) per head of a kv head, for every pair and every block.
JLLM_EXPORT long long jllm_attention_decode_flat_scratch_floats(int rows, int heads, int kv_heads, int head_dim, int blocks) {
    return ((long long)rows * kv_heads + blocks) * (heads / kv_heads) * (head_dim + 2);
}

// Decode attention with the key tiles of all (row, kv head) pairs dealt out evenly over `blocks` blocks (head sizes
// 64, 128, 256; at most 1,024 rows; at most 62 blocks per kv head, so that a pair's tiles fall to at most 64 blocks).
namespace {

int decode_flat(const void* q, int q_stride, const void* k_cache, const void* v_cache, void* out, int out_stride,
                const int* row_seg, const int* row_pos, const int* block_tables, int table_stride, int rows, int heads,
                int kv_heads, int head_dim, int page_size, int window, float scale, int blocks, float* scratch,
                const staged::Fresh& fresh, cudaStream_t stream) {
    JLLM_REQUIRE(rows >= 0 && rows <= staged::FLAT_MAX_ROWS && heads > 0 && kv_heads > 0 && heads % kv_heads == 0 &&
                     page_size > 0 && heads / kv_heads <= 16,
                 "attention_decode_flat: rows=%d (at most %d) heads=%d kv_heads=%d page_size=%d", rows,
                 staged::FLAT_MAX_ROWS, heads, kv_heads, page_size);
    JLLM_REQUIRE(head_dim == 64 || head_dim == 128 || head_dim == 256, "attention_decode_flat: head_dim=%d is not 64, 128 or 256",
                 head_dim);
    JLLM_REQUIRE(q_stride % 8 == 0 && ((uintptr_t)q % 16) == 0 && ((uintptr_t)k_cache % 16) == 0 &&
                     ((uintptr_t)v_cache % 16) == 0,
                 "attention_decode_flat: q, K and V must be 16-byte aligned (q_stride=%d)", q_stride);
    // a pair holds at most 1 / kv_heads of all tiles, so its tiles fall to at most blocks / kv_heads + 2 blocks: 64 at most
    JLLM_REQUIRE(blocks >= 1 && blocks <= 62 * kv_heads && scratch != nullptr,
                 "attention_decode_flat: %d blocks with %d kv heads (at most 62 per kv head), scratch %p", blocks, kv_heads,
                 (void*)scratch);
    if (rows == 0) return JLLM_OK;
    const int G = heads / kv_heads;
    float* part_o = scratch;
    float* part_ml = scratch + ((size_t)rows * kv_heads + blocks) * G * head_dim;
    const float scale_log2 = scale * LOG2E;
    // (a run of the deal is never empty when there are at least as many key tiles as blocks: every pair has one or more)
    int* counters = (long long)rows * kv_heads <= staged::PAIR_COUNTERS && (long long)rows * kv_heads >= blocks &&
                            !g_separate_combine ? staged::pair_counters() : nullptr;
#define JLLM_FLAT(HD)                                                                                                  \
    staged::launch_flat<HD>(q, q_stride, k_cache, v_cache, out, out_stride, row_seg, row_pos, block_tables, table_stride, \
                            rows, heads, kv_heads, page_size, window, scale_log2, blocks, part_o, part_ml, counters, fresh, stream)
    if (head_dim == 64) JLLM_FLAT(64); else if (head_dim == 128) JLLM_FLAT(128); else JLLM_FLAT(256);
#undef JLLM_FLAT
    return jllm_check_launch("attention_decode_flat");
}

}  // namespace

JLLM_EXPORT int jllm_attention_decode_flat(const void* q, int q_stride, const void* k_cache, const void* v_cache, void* out,
                                           int out_stride, const int* row_seg, const int* row_pos, const int* block_tables,
                                           int table_stride, int rows, int heads, int kv_heads, int head_dim, int page_size,
                                           int window, float scale, int blocks, float* scratch, cudaStream_t stream) {
    return decode_flat(q, q_stride, k_cache, v_cache, out, out_stride, row_seg, row_pos, block_tables, table_stride, rows,
                       heads, kv_heads, head_dim, page_size, window, scale, blocks, scratch, staged::Fresh{}, stream);
}

// Decode attention that first finishes its own row: `qkv` ([rows, stride]: query, key and value heads side by side) is as
// the QKV product left it. Every block norms (use_norm) and rotates the queries of its kv head, and the block that holds
// a row's newest position makes that key and value, writes them to the cache (k_cache, v_cache: written here) and uses
// them. Head sizes 64, 128, 256, rotated over their whole width (cos_t, sin_t: [positions, head_dim / 2]). `flat` 0: `n`
// key splits per (row, kv head); 1: the key tiles of all pairs dealt out over `n` blocks. The same bits as
// jllm_qk_norm_rope_store followed by jllm_attention_decode(_flat).
JLLM_EXPORT int jllm_attention_decode_fresh(const void* qkv, int qkv_stride, const void* q_gain, const void* k_gain,
                                            int gain_dtype, int use_norm, float eps, const float* cos_t, const float* sin_t,
                                            void* k_cache, void* v_cache, void* out, int out_stride, const int* row_seg,
                                            const int* row_pos, const int* block_tables, int table_stride, int rows,
                                            int heads, int kv_heads, int head_dim, int page_size, int window, float scale,
                                            int flat, int n, float* scratch, cudaStream_t stream) {
    JLLM_REQUIRE(head_dim == 64 || head_dim == 128 || head_dim == 256, "attention_decode_fresh: head_dim=%d is not 64, 128 or 256",
                 head_dim);
    JLLM_REQUIRE(qkv != nullptr && cos_t != nullptr && sin_t != nullptr && (!use_norm || (q_gain != nullptr && k_gain != nullptr)),
                 "attention_decode_fresh: needs qkv, the angle tables and, with the norm, both gains");
    staged::Fresh fresh{};
    fresh.qkv = (const __nv_bfloat16*)qkv;
    fresh.stride = qkv_stride;
    fresh.use_norm = use_norm;
    fresh.eps = eps;
    fresh.q_gain = VecRef{q_gain, gain_dtype};
    fresh.k_gain = VecRef{k_gain, gain_dtype};
    fresh.cos_t = cos_t;
    fresh.sin_t = sin_t;
    fresh.k_out = (__nv_bfloat16*)k_cache;
    fresh.v_out = (__nv_bfloat16*)v_cache;
    if (flat)
        return decode_flat(qkv, qkv_stride, k_cache, v_cache, out, out_stride, row_seg, row_pos, block_tables, table_stride,
                           rows, heads, kv_heads, head_dim, page_size, window, scale, n, scratch, fresh, stream);
    return decode_split(qkv, qkv_stride, k_cache, v_cache, out, out_stride, row_seg, row_pos, block_tables, table_stride,
                        rows, heads, kv_heads, head_dim, page_size, window, scale, n, scratch, fresh, stream);
}

// ---------------------------------------------------------------------------------------------------
// The same attention with the split scratch inside the library: see attention_decode_static.h.
// ---------------------------------------------------------------------------------------------------
#include "attention_decode_static.h"

namespace {

// Partial (output, max, sum) of the key-range splits. The memory belongs to the library image: every GPU
// that loads the library holds these 8 MiB until the process exits. In host code this name is only a
// stand-in for the symbol (not a device address); the address comes from cudaGetSymbolAddress below.
static __device__ __align__(256) float g_decode_static_scratch[JLLM_ATTENTION_DECODE_STATIC_FLOATS];

constexpr int MAX_DEVICES = 64;
float* g_static_scratch_ptr[MAX_DEVICES] = {};

// Once per device, with that device current: look the array's device address up.
int static_scratch_for_current_device(float** out) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return jllm_fail(JLLM_CUDA_ERROR, "attention_decode_static: cudaGetDevice: %s", cudaGetErrorString(e));
    if (dev < 0 || dev >= MAX_DEVICES)
        return jllm_fail(JLLM_UNSUPPORTED, "attention_decode_static: device %d is beyond the %d devices it keeps track of",
                         dev, MAX_DEVICES);
    if (g_static_scratch_ptr[dev] == nullptr) {
        float* ptr = nullptr;
        e = cudaGetSymbolAddress((void**)&ptr, g_decode_static_scratch);
        if (e != cudaSuccess || ptr == nullptr)
            return jllm_fail(JLLM_CUDA_ERROR, "attention_decode_static: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
        g_static_scratch_ptr[dev] = ptr;
    }
    *out = g_static_scratch_ptr[dev];
    return JLLM_OK;
}

}  // namespace

JLLM_EXPORT long long jllm_attention_decode_static_capacity() { return JLLM_ATTENTION_DECODE_STATIC_FLOATS; }

JLLM_EXPORT int jllm_attention_decode_static(const void* q, int q_stride, const void* k_cache, const void* v_cache,
                                             void* out, int out_stride, const int* row_seg, const int* row_pos,
                                             const int* block_tables, int table_stride, int rows, int heads,
                                             int kv_heads, int head_dim, int page_size, int window, float scale,
                                             int splits, cudaStream_t stream) {
    JLLM_REQUIRE(rows >= 0 && heads > 0 && head_dim > 0 && splits >= 1, "attention_decode_static: rows=%d heads=%d "
                 "head_dim=%d splits=%d", rows, heads, head_dim, splits);
    const long long need = jllm_attention_decode_scratch_floats(rows, heads, head_dim, splits);
    if (need > (long long)JLLM_ATTENTION_DECODE_STATIC_FLOATS)
        return jllm_fail(JLLM_BAD_ARGUMENT,
                         "attention_decode_static: %d rows x %d heads x %d splits x (head_dim %d + 2) = %lld floats of "
                         "scratch, the built-in array holds %lld; use fewer splits or rows, or jllm_attention_decode "
                         "with scratch of your own", rows, heads, splits, head_dim, need,
                         (long long)JLLM_ATTENTION_DECODE_STATIC_FLOATS);
    float* scratch = nullptr;
    const int rc = static_scratch_for_current_device(&scratch);
    if (rc != JLLM_OK) return rc;
    // Nothing in the array has to start at zero: every (row, head, split) slot that the combine step reads
    // is written by the block of that split in the same call, also when the split holds no keys.
    return jllm_attention_decode(q, q_stride, k_cache, v_cache, out, out_stride, row_seg, row_pos, block_tables,
                                 table_stride, rows, heads, kv_heads, head_dim, page_size, window, scale, splits,
                                 scratch, stream);
}
