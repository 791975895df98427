// Paged causal flash attention for prompt portions (bfloat16): rows of a batch attend to their own
// request's cached keys and values, a tile of 128 query rows of one head per block.
//
// A block first finds its tile: tiles are numbered segment after segment (a segment = one request's rows
// in this step), ceil(rows / 128) tiles each. Its 8 warps take 16 query rows each. Keys and values come
// in tiles of 64 positions, gathered from the request's pages into shared memory with cp.async (16-byte
// chunks, XOR-swizzled against bank conflicts, double-buffered so the next tile loads while this one is
// used). Scores S = Q K^T and the output O += P V run on mma.sync.m16n8k16 with operands from ldmatrix;
// the softmax is the online one in float32 (base 2), with the running maximum and sum per row in
// registers. A row at position P sees keys [first, P], first = max(0, P + 1 - window) under a window.
// Key tiles that no row of the query tile can see are skipped; positions that no row may see inside a
// loaded tile are masked to -inf, and key rows past the last visible position are zero-filled instead of
// read (their pages may belong to nobody).
//
// Layouts as everywhere: q [rows, q_stride] (head h at h * head_dim), cache K and V
// [pages, kv_heads, page_size, head_dim], out [rows, out_stride]. Built for head_dim 64, 128 and 256;
// other sizes go to the plain kernel.
#include "common.cuh"

namespace {

constexpr int BQ = 128, BKV = 64, WARPS = 8, THREADS = WARPS * 32;
constexpr float LOG2E = 1.4426950408889634f;

__device__ __forceinline__ void mma_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void cp_async_16(uint32_t dst, const void* src, int src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory"); }

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// byte offset of 16-byte chunk c of row r in a [rows][HD] bfloat16 tile, chunks XOR-swizzled by the row
template <int HD>
__device__ __forceinline__ uint32_t tile_offset(int r, int c) {
    return (uint32_t)((r * (HD / 8) + (c ^ (r & 7))) * 16);
}

template <int HD>
__global__ void __launch_bounds__(THREADS)
attention_prefill_kernel(const __nv_bfloat16* __restrict__ q, int q_stride, const __nv_bfloat16* __restrict__ k_cache,
                         const __nv_bfloat16* __restrict__ v_cache, __nv_bfloat16* __restrict__ out, int out_stride,
                         const int* __restrict__ seg_start, const int* __restrict__ seg_len,
                         const int* __restrict__ seg_kv_len, const int* __restrict__ block_tables, int table_stride,
                         int num_segs, int heads, int kv_heads, int page_size, int num_pages, int window,
                         float scale_log2) {
    constexpr int CHUNKS = HD / 8;               // 16-byte chunks per row
    constexpr int TILE_BYTES = BKV * HD * 2;
    extern __shared__ __align__(128) uint8_t smem[];
    const uint32_t s_q = (uint32_t)__cvta_generic_to_shared(smem);
    const uint32_t s_k = s_q + BQ * HD * 2;      // two K tiles, then two V tiles
    const uint32_t s_v = s_k + 2 * TILE_BYTES;

    // ---- which tile of which segment ----
    int seg = 0, tile = blockIdx.x;
    for (; seg < num_segs; ++seg) {
        const int nt = (seg_len[seg] + BQ - 1) / BQ;
        if (tile < nt) break;
        tile -= nt;
    }
    if (seg >= num_segs) return;                 // the grid is an upper bound on the number of tiles
    const int head = blockIdx.y, kvh = head / (heads / kv_heads);
    const int n_rows = seg_len[seg], q0 = tile * BQ;
    const int rows_here = min(BQ, n_rows - q0);
    const int row0 = seg_start[seg] + q0;                       // first batch row of the tile
    const int pos0 = seg_kv_len[seg] - n_rows + q0;             // position of that row
    const int pos_last = pos0 + rows_here - 1;
    const int* table = block_tables + (size_t)seg * table_stride;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;

    // ---- Q tile -> shared memory (rows past the segment's end are zero) ----
    for (int i = threadIdx.x; i < BQ * CHUNKS; i += THREADS) {
        const int r = i / CHUNKS, c = i % CHUNKS;
        const __nv_bfloat16* src = q + (size_t)(row0 + min(r, rows_here - 1)) * q_stride + (size_t)head * HD + c * 8;
        cp_async_16(s_q + tile_offset<HD>(r, c), src, r < rows_here ? 16 : 0);
    }
    cp_async_commit();

    const int first_key = window > 0 ? max(0, pos0 + 1 - window) : 0;
    const int kt_lo = first_key / BKV, kt_hi = pos_last / BKV;  // inclusive range of key tiles
    const size_t page_stride = (size_t)kv_heads * page_size * HD;
    const int page_shift = (page_size & (page_size - 1)) == 0 ? __ffs(page_size) - 1 : -1;

    auto load_kv = [&](int kt, int buf) {
        const uint32_t dk = s_k + buf * TILE_BYTES, dv = s_v + buf * TILE_BYTES;
        for (int i = threadIdx.x; i < BKV * CHUNKS; i += THREADS) {
            const int r = i / CHUNKS, c = i % CHUNKS;
            const int key = kt * BKV + r;
            bool ok = key >= first_key && key <= pos_last;
            size_t off = 0;
            if (ok) {
                const int pg = page_shift >= 0 ? key >> page_shift : key / page_size;
                const int in_page = page_shift >= 0 ? key & (page_size - 1) : key % page_size;
                const long long page = jllm_page_of(table, pg, table_stride, num_pages);
                if (kCheckBounds && page < 0) ok = false;       // checked build: a bad table entry reads nothing
                else off = (size_t)page * page_stride + ((size_t)kvh * page_size + in_page) * HD + c * 8;
            }
            cp_async_16(dk + tile_offset<HD>(r, c), k_cache + off, ok ? 16 : 0);
            cp_async_16(dv + tile_offset<HD>(r, c), v_cache + off, ok ? 16 : 0);
        }
        cp_async_commit();
    };
    load_kv(kt_lo, 0);

    // ---- Q fragments of this warp's 16 rows ----
    cp_async_wait<1>();
    __syncthreads();
    uint32_t qf[HD / 16][4];
#pragma unroll
    for (int ks = 0; ks < HD / 16; ++ks)
        ldmatrix_x4(qf[ks], s_q + tile_offset<HD>(warp * 16 + (lane & 15), ks * 2 + (lane >> 4)));

    float o[HD / 8][4];
#pragma unroll
    for (int j = 0; j < HD / 8; ++j)
#pragma unroll
        for (int i = 0; i < 4; ++i) o[j][i] = 0.f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    // positions of this thread's two rows (rows past the end act like the last real row and are not stored)
    int pos_r[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) pos_r[h] = pos0 + min(warp * 16 + g + 8 * h, rows_here - 1);

    for (int kt = kt_lo; kt <= kt_hi; ++kt) {
        const int buf = (kt - kt_lo) & 1;
        if (kt < kt_hi) {
            load_kv(kt + 1, buf ^ 1);
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        // a warp whose rows all lie before this key tile has nothing to do in it (causal), but still takes part
        // in the loads and barriers
        if (kt * BKV <= pos0 + min(warp * 16 + 15, rows_here - 1)) {
            const uint32_t sk = s_k + buf * TILE_BYTES, sv = s_v + buf * TILE_BYTES;
            // ---- S = Q K^T: 16 rows x 64 keys per warp ----
            float s[BKV / 8][4];
    #pragma unroll
            for (int j = 0; j < BKV / 8; ++j)
    #pragma unroll
                for (int i = 0; i < 4; ++i) s[j][i] = 0.f;
    #pragma unroll
            for (int ks = 0; ks < HD / 16; ++ks) {
    #pragma unroll
                for (int jp = 0; jp < BKV / 16; ++jp) {
                    uint32_t kf[4];
                    ldmatrix_x4(kf, sk + tile_offset<HD>(jp * 16 + (lane & 7) + ((lane >> 4) << 3), ks * 2 + ((lane >> 3) & 1)));
                    mma_16816(s[2 * jp], qf[ks], kf[0], kf[1]);
                    mma_16816(s[2 * jp + 1], qf[ks], kf[2], kf[3]);
                }
            }
            // ---- mask and online softmax ----
            const int key0 = kt * BKV;
            float mx[2] = {-INFINITY, -INFINITY};
            // a tile that every row of this warp sees whole (all keys at or before the warp's first position and
            // inside every row's window) needs no mask: true for all but the tiles on the diagonal and the window's edge
            const int warp_first = pos0 + min(warp * 16, rows_here - 1), warp_last = pos0 + min(warp * 16 + 15, rows_here - 1);
            const bool whole = key0 + BKV - 1 <= warp_first && (window <= 0 || key0 >= warp_last + 1 - window);
            if (whole) {
    #pragma unroll
                for (int j = 0; j < BKV / 8; ++j)
    #pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        s[j][i] *= scale_log2;
                        mx[i >> 1] = fmaxf(mx[i >> 1], s[j][i]);
                    }
            } else {
    #pragma unroll
                for (int j = 0; j < BKV / 8; ++j)
    #pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const int key = key0 + j * 8 + 2 * t + (i & 1), P = pos_r[i >> 1];
                        const bool vis = key <= P && (window <= 0 || key >= P + 1 - window);
                        s[j][i] = vis ? s[j][i] * scale_log2 : -INFINITY;
                        mx[i >> 1] = fmaxf(mx[i >> 1], s[j][i]);
                    }
            }
            float corr[2], m_use[2];
    #pragma unroll
            for (int h = 0; h < 2; ++h) {
                mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
                mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
                const float m_new = fmaxf(m_run[h], mx[h]);
                m_use[h] = m_new == -INFINITY ? 0.f : m_new;        // a row that sees nothing yet: avoid inf - inf
                corr[h] = exp2f(m_run[h] - m_use[h]);
                m_run[h] = m_new;
                l_run[h] *= corr[h];
            }
    #pragma unroll
            for (int j = 0; j < HD / 8; ++j) {
                o[j][0] *= corr[0];
                o[j][1] *= corr[0];
                o[j][2] *= corr[1];
                o[j][3] *= corr[1];
            }
            uint32_t pf[BKV / 16][4];
    #pragma unroll
            for (int j = 0; j < BKV / 8; ++j) {
                const float p0 = exp2f(s[j][0] - m_use[0]), p1 = exp2f(s[j][1] - m_use[0]);
                const float p2 = exp2f(s[j][2] - m_use[1]), p3 = exp2f(s[j][3] - m_use[1]);
                l_run[0] += p0 + p1;
                l_run[1] += p2 + p3;
                pf[j >> 1][(j & 1) * 2 + 0] = pack_bf16(p0, p1);
                pf[j >> 1][(j & 1) * 2 + 1] = pack_bf16(p2, p3);
            }
            // ---- O += P V ----
    #pragma unroll
            for (int kk = 0; kk < BKV / 16; ++kk) {
    #pragma unroll
                for (int jp = 0; jp < HD / 16; ++jp) {
                    uint32_t vf[4];
                    ldmatrix_x4_trans(vf, sv + tile_offset<HD>(kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, jp * 2 + (lane >> 4)));
                    mma_16816(o[2 * jp], pf[kk], vf[0], vf[1]);
                    mma_16816(o[2 * jp + 1], pf[kk], vf[2], vf[3]);
                }
            }
        }
        __syncthreads();   // everyone is done with this buffer before the load after next overwrites it
    }
    // ---- normalise and store ----
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 1);
        l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 2);
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int r = warp * 16 + g + 8 * h;
        if (r >= rows_here) continue;
        const float inv = 1.f / l_run[h];
        __nv_bfloat16* dst = out + (size_t)(row0 + r) * out_stride + (size_t)head * HD;
#pragma unroll
        for (int j = 0; j < HD / 8; ++j) {
            const uint32_t v = pack_bf16(o[j][2 * h] * inv, o[j][2 * h + 1] * inv);
            *reinterpret_cast<uint32_t*>(dst + j * 8 + 2 * t) = v;
        }
    }
}

template <int HD>
int launch(const void* q, int q_stride, const void* k_cache, const void* v_cache, void* out, int out_stride,
           const int* seg_start, const int* seg_len, const int* seg_kv_len, const int* block_tables, int table_stride,
           int num_segs, int rows, int heads, int kv_heads, int page_size, int window, float scale,
           cudaStream_t stream) {
    const size_t smem = (size_t)BQ * HD * 2 + 4 * (size_t)BKV * HD * 2;
    auto kern = attention_prefill_kernel<HD>;
    if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    const dim3 grid((rows + BQ - 1) / BQ + num_segs, heads);
    kern<<<grid, THREADS, smem, stream>>>((const __nv_bfloat16*)q, q_stride, (const __nv_bfloat16*)k_cache,
                                          (const __nv_bfloat16*)v_cache, (__nv_bfloat16*)out, out_stride, seg_start,
                                          seg_len, seg_kv_len, block_tables, table_stride, num_segs, heads, kv_heads,
                                          page_size, jllm_pool_pages(), window, scale * LOG2E);
    return jllm_check_launch("attention_prefill");
}

}  // namespace

JLLM_BOUNDS_READER(attention_prefill)

JLLM_EXPORT int jllm_attention_prefill_fits(int head_dim) { return head_dim == 64 || head_dim == 128 || head_dim == 256; }

JLLM_EXPORT int jllm_attention_prefill(const void* q, int q_stride, const void* k_cache, const void* v_cache, void* out,
                                       int out_stride, const int* seg_start, const int* seg_len, const int* seg_kv_len,
                                       const int* block_tables, int table_stride, int num_segs, int rows, int heads,
                                       int kv_heads, int head_dim, int page_size, int window, float scale,
                                       cudaStream_t stream) {
    JLLM_REQUIRE(rows >= 0 && num_segs >= 0 && heads > 0 && kv_heads > 0 && heads % kv_heads == 0 && page_size > 0,
                 "attention_prefill: rows=%d segments=%d heads=%d kv_heads=%d page_size=%d", rows, num_segs, heads,
                 kv_heads, page_size);
    JLLM_REQUIRE(jllm_attention_prefill_fits(head_dim), "attention_prefill: head_dim=%d is not 64, 128 or 256", head_dim);
    JLLM_REQUIRE(q_stride % 8 == 0 && out_stride % 2 == 0 && ((uintptr_t)q % 16) == 0 && ((uintptr_t)k_cache % 16) == 0 &&
                     ((uintptr_t)v_cache % 16) == 0 && ((uintptr_t)out % 4) == 0,
                 "attention_prefill: q, K, V must be 16-byte aligned (q_stride=%d out_stride=%d)", q_stride, out_stride);
    JLLM_REQUIRE(heads <= 65535, "attention_prefill: heads=%d", heads);
    if (rows == 0 || num_segs == 0) return JLLM_OK;
#define JLLM_ARGS q, q_stride, k_cache, v_cache, out, out_stride, seg_start, seg_len, seg_kv_len, block_tables, \
                  table_stride, num_segs, rows, heads, kv_heads, page_size, window, scale, stream
    if (head_dim == 64) return launch<64>(JLLM_ARGS);
    if (head_dim == 128) return launch<128>(JLLM_ARGS);
    return launch<256>(JLLM_ARGS);
#undef JLLM_ARGS
}
