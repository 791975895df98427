// Paged causal flash attention for prompt portions on the 5th-generation tensor cores (head size 128).
//
// One block per (128 query rows of a segment, head). Both products of attention run as tcgen05.mma with
// their accumulators in tensor memory (TMEM):
//     S = Q K^T   A = Q tile [128 rows x 128] in shared memory (K-major), B = K tile [128 keys x 128] (K-major),
//                 D = S in TMEM, 128 lanes x 128 columns of float32, two such buffers;
//     O += P V    A = P tile [128 rows x 128 keys] (bfloat16, written to shared memory by the softmax warps),
//                 B = V tile [128 keys x 128] read as an MN-major operand (its rows are keys, the K side of this
//                 product), D = O in TMEM, 128 lanes x 128 columns.
// Warp roles: warp 0 loads (Q and whole K / V tiles by TMA, one box per page and 64-column half, straight out
// of the paged cache seen as a 2-D tensor [pages * kv_heads * page_size, 128]; the tiles at the edges of the
// visible key range by cp.async with zero fill, because rows past a request's last position may hold anything);
// warp 1 issues the MMAs; warps 2-5 are the softmax: thread = query row = TMEM lane. Per key tile a softmax
// thread reads its row of S twice (maximum, then exp2 and the bfloat16 P), rescales its row of O in TMEM when
// the running maximum moved, and hands P to the MMA warp. S for tile j + 1 is computed while the softmax of
// tile j runs (two S buffers). Softmax state is float32, base 2.
//
// All tiles in shared memory use the 128-byte swizzle on 64-column halves: [half][row][64 columns]. The same
// bytes serve K (K-major B of the first product) and V (MN-major B of the second).
// Every mbarrier wait is bounded; a wait that runs out raises the error word and all roles leave.
//
// Requirements: bfloat16, head_dim 128, page_size a power of two <= 128, 16-byte aligned q rows.
#include "tcgen05_common.cuh"

namespace {

using namespace tc;

constexpr int BQ = 128, BKV = 128, HD = 128, THREADS = 192;
constexpr int TILE_BYTES = 128 * HD * 2;           // 32 KB: Q, each K, each V and P
constexpr int HALF_BYTES = 128 * 64 * 2;           // one 64-column half of a tile
constexpr float LOG2E = 1.4426950408889634f;
constexpr size_t SMEM_BYTES = 6 * TILE_BYTES + 1024 + 256;
constexpr int TMEM_COLS = 512;                      // S0 at 0, S1 at 128, O at 256

__global__ void __launch_bounds__(THREADS, 1)
attention_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                            const __grid_constant__ CUtensorMap map_v, const __nv_bfloat16* __restrict__ k_cache,
                            const __nv_bfloat16* __restrict__ v_cache, __nv_bfloat16* __restrict__ out, int out_stride,
                            const int* __restrict__ seg_start, const int* __restrict__ seg_len,
                            const int* __restrict__ seg_kv_len, const int* __restrict__ block_tables, int table_stride,
                            int num_segs, int heads, int kv_heads, int page_size, int page_shift, int num_pages, int window,
                            float scale_log2, int* __restrict__ error_word) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* aligned = smem_raw + (base - smem_u32(smem_raw));
    const uint32_t s_q = base, s_p = base + TILE_BYTES;
    auto s_k = [&](int b) { return base + (2 + b) * TILE_BYTES; };
    auto s_v = [&](int b) { return base + (4 + b) * TILE_BYTES; };
    const uint32_t bars = base + 6 * TILE_BYTES;
    enum { Q_FULL = 0, K_FULL = 1, V_FULL = 3, K_EMPTY = 5, V_EMPTY = 7, S_FULL = 9, S_EMPTY = 11, P_READY = 13, PV_DONE = 14 };
    auto bar = [&](int i) { return bars + 8u * i; };
    uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(aligned + 6 * TILE_BYTES + 8 * 16);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_base_slot + 1);

    // ---- which tile of which segment ----
    // blocks start in the order of the grid: the tiles with the most keys before them (the last of a segment) first
    int seg = 0, tile = gridDim.y - 1 - blockIdx.y;
    for (; seg < num_segs; ++seg) {
        const int nt = (seg_len[seg] + BQ - 1) / BQ;
        if (tile < nt) break;
        tile -= nt;
    }
    if (seg >= num_segs) return;                       // whole block: before any barrier or allocation
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int head = blockIdx.x, kvh = head / (heads / kv_heads);
    const int n_rows = seg_len[seg], q0 = tile * BQ;
    const int rows_here = min(BQ, n_rows - q0);
    const int row0 = seg_start[seg] + q0;
    const int pos0 = seg_kv_len[seg] - n_rows + q0, pos_last = pos0 + rows_here - 1;
    const int first_key = window > 0 ? max(0, pos0 + 1 - window) : 0;
    const int kt_lo = first_key / BKV, kt_hi = pos_last / BKV, n_tiles = kt_hi - kt_lo + 1;
    const int* table = block_tables + (size_t)seg * table_stride;

    if (threadIdx.x == 0) {
        mbar_init(bar(Q_FULL), 1);
        for (int b = 0; b < 2; ++b) {
            mbar_init(bar(K_FULL + b), 1);
            mbar_init(bar(V_FULL + b), 1);
            mbar_init(bar(K_EMPTY + b), 1);
            mbar_init(bar(V_EMPTY + b), 1);
            mbar_init(bar(S_FULL + b), 1);
            mbar_init(bar(S_EMPTY + b), 128);
        }
        mbar_init(bar(P_READY), 128);
        mbar_init(bar(PV_DONE), 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 2) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_base_slot)),
                     "r"(TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_base_slot;
    pdl_wait();
    pdl_trigger();

    if (warp == 0) {
        // ---------------- loader ----------------
        bool ok = true;
        if (lane == 0) {
            mbar_expect_tx(bar(Q_FULL), TILE_BYTES);
            tma_load_2d(s_q, &map_q, head * HD, row0, bar(Q_FULL));
            tma_load_2d(s_q + HALF_BYTES, &map_q, head * HD + 64, row0, bar(Q_FULL));
        }
        for (int j = 0; j < n_tiles && ok; ++j) {
            const int b = j & 1, key0 = (kt_lo + j) * BKV;
            const bool whole = key0 >= first_key && key0 + BKV - 1 <= pos_last;   // every row is a live, written key
            for (int which = 0; which < 2 && ok; ++which) {                        // 0: keys, 1: values
                const int full = (which ? V_FULL : K_FULL) + b, empty = (which ? V_EMPTY : K_EMPTY) + b;
                const uint32_t dst = which ? s_v(b) : s_k(b);
                if (j >= 2) {
                    if (lane == 0) ok = mbar_wait(bar(empty), ((j >> 1) - 1) & 1u, abort_flag);
                    ok = __shfl_sync(0xffffffffu, ok, 0);
                    if (!ok) break;
                }
                if (whole) {
                    // one lane per page: the table look-ups and the copies' issue run side by side
                    if (lane == 0) mbar_expect_tx(bar(full), TILE_BYTES);
                    __syncwarp();
                    const CUtensorMap* map = which ? &map_v : &map_k;
                    const int first_page = key0 >> page_shift;
                    for (int p = lane; p < (BKV >> page_shift); p += 32) {
                        // checked build: a bad entry gives -1 and a box of negative rows, which TMA fills with zeros
                        const long long pg = jllm_page_of(table, first_page + p, table_stride, num_pages);
                        const int y = (int)((pg * kv_heads + kvh) * page_size);
                        const uint32_t d = dst + ((p << page_shift) << 7);
                        tma_load_2d(d, map, 0, y, bar(full));
                        tma_load_2d(d + HALF_BYTES, map, 64, y, bar(full));
                    }
                } else {
                    // edge tile: row by row, zero where no live key is (16 chunks of 16 bytes per row)
                    const __nv_bfloat16* cache = which ? v_cache : k_cache;
                    for (int i = lane; i < BKV * 16; i += 32) {
                        const int r = i >> 4, c = i & 15;
                        const int key = key0 + r;
                        bool live = key >= first_key && key <= pos_last;
                        size_t off = 0;
                        if (live) {
                            const long long pg = jllm_page_of(table, key >> page_shift, table_stride, num_pages);
                            if (kCheckBounds && pg < 0) live = false;
                            else off = (((size_t)pg * kv_heads + kvh) * page_size + (key & (page_size - 1))) * HD + c * 8;
                        }
                        const uint32_t d = dst + (c >> 3) * HALF_BYTES + r * 128 + (((c & 7) ^ (r & 7)) << 4);
                        cp_async_16(d, cache + off, live ? 16 : 0);
                    }
                    asm volatile("cp.async.wait_all;" ::: "memory");
                    fence_async_proxy();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(bar(full));
                }
            }
        }
        if (!ok && lane == 0) { *abort_flag = 1; atomicExch(error_word, 21); }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            bool ok = mbar_wait(bar(Q_FULL), 0, abort_flag);
            auto issue_s = [&](int j) {       // S[j & 1] = Q K_j^T
                const int b = j & 1;
                if (!mbar_wait(bar(K_FULL + b), (j >> 1) & 1u, abort_flag)) return false;
                if (j >= 2 && !mbar_wait(bar(S_EMPTY + b), ((j >> 1) - 1) & 1u, abort_flag)) return false;
                tcgen05_fence_after();
                const uint32_t d = tmem_base + b * 128;
#pragma unroll
                for (int k = 0; k < HD / 16; ++k) {
                    const uint32_t o = (k >> 2) * HALF_BYTES + (k & 3) * 32;
                    tcgen05_mma_bf16(d, smem_desc_sw128(s_q + o), smem_desc_sw128(s_k(b) + o), IDESC_128x128_KK, k > 0);
                }
                tcgen05_commit(bar(S_FULL + b));
                tcgen05_commit(bar(K_EMPTY + b));
                return true;
            };
            if (ok) ok = issue_s(0);
            for (int j = 0; j < n_tiles && ok; ++j) {
                const int b = j & 1;
                if (j + 1 < n_tiles) ok = issue_s(j + 1);
                if (!ok) break;
                if (!mbar_wait(bar(P_READY), j & 1u, abort_flag) || !mbar_wait(bar(V_FULL + b), (j >> 1) & 1u, abort_flag)) {
                    ok = false;
                    break;
                }
                tcgen05_fence_after();
                const uint32_t d = tmem_base + 256;
#pragma unroll
                for (int k = 0; k < BKV / 16; ++k) {
                    // A: 16 keys further along P's rows; B: 16 key rows further down V (two 8-row groups)
                    const uint32_t pa = s_p + (k >> 2) * HALF_BYTES + (k & 3) * 32;
                    tcgen05_mma_bf16(d, smem_desc_sw128(pa), smem_desc_mn_sw128(s_v(b) + k * 2048, HALF_BYTES), IDESC_128x128_KMN,
                                     (j > 0 || k > 0) ? 1u : 0u);
                }
                tcgen05_commit(bar(PV_DONE));
                tcgen05_commit(bar(V_EMPTY + b));
            }
            if (!ok) { *abort_flag = 1; atomicExch(error_word, 22); }
        }
    } else {
        // ---------------- softmax: thread = query row = TMEM lane ----------------
        const int quad = warp & 3, r = quad * 32 + lane;
        const uint32_t lane_addr = tmem_base + ((uint32_t)(quad * 32) << 16);
        const int P = pos0 + min(r, rows_here - 1);            // rows past the end copy the last row, and are not stored
        const int lo = window > 0 ? max(0, P + 1 - window) : 0;
        float m = -INFINITY, l = 0.f;
        bool ok = true;
        for (int j = 0; j < n_tiles && ok; ++j) {
            const int b = j & 1, key0 = (kt_lo + j) * BKV;
            if (!mbar_wait(bar(S_FULL + b), (j >> 1) & 1u, abort_flag)) { ok = false; break; }
            tcgen05_fence_after();
            const bool masked = key0 + BKV - 1 > pos0 || key0 < lo || (window > 0 && key0 < pos_last + 1 - window);
            // the row of S: four loads in flight, one wait
            uint32_t v[4][32];
#pragma unroll
            for (int c = 0; c < 4; ++c) tmem_ld_32x32b_x32(lane_addr + b * 128 + c * 32, v[c]);
            tmem_ld_wait();
            if (masked) {
#pragma unroll
                for (int c = 0; c < 4; ++c)
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        const int key = key0 + c * 32 + i;
                        if (!(key <= P && key >= lo)) v[c][i] = __float_as_uint(-INFINITY);
                    }
            }
            // (four chains, then their maximum: one chain of 128 dependent comparisons is pure latency)
            float mxs[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
            for (int c = 0; c < 4; ++c)
#pragma unroll
                for (int i = 0; i < 32; ++i) mxs[i & 3] = fmaxf(mxs[i & 3], __uint_as_float(v[c][i]));
            const float mx = fmaxf(fmaxf(mxs[0], mxs[1]), fmaxf(mxs[2], mxs[3]));
            // The reference point of the exponentials only moves when the maximum grew by more than 2^8: until
            // then p stays below 256, which bfloat16 and the float32 sum hold as well, and O needs no rescaling.
            const float m_cand = fmaxf(m, mx * scale_log2);
            const float m_new = (m_cand - m > 8.f) ? m_cand : m;
            const float m_use = m_new == -INFINITY ? 0.f : m_new;
            const float corr = fast_exp2(m - m_use);
            // p = 2^(s * scale - reference) as bfloat16, and the row's sum
            uint32_t pk[64];
            float sum = 0.f;
#pragma unroll
            for (int c = 0; c < 4; ++c)
#pragma unroll
                for (int i = 0; i < 32; i += 2) {
                    const float p0 = fast_exp2(fmaf(__uint_as_float(v[c][i]), scale_log2, -m_use));
                    const float p1 = fast_exp2(fmaf(__uint_as_float(v[c][i + 1]), scale_log2, -m_use));
                    sum += p0 + p1;
                    __nv_bfloat162 b2 = __floats2bfloat162_rn(p0, p1);
                    pk[(c * 32 + i) >> 1] = *reinterpret_cast<uint32_t*>(&b2);
                }
            tcgen05_fence_before();
            mbar_arrive(bar(S_EMPTY + b));                        // this row of S has been read
            m = m_new;
            l = l * corr + sum;
            // P's buffer and O are free once the product of the tile before has completed
            if (j > 0 && !mbar_wait(bar(PV_DONE), (j - 1) & 1u, abort_flag)) { ok = false; break; }
            tcgen05_fence_after();
            uint8_t* prow = aligned + TILE_BYTES + r * 128;
#pragma unroll
            for (int c = 0; c < 16; ++c) {                        // 16 chunks of 8 keys; halves of 64 keys
                uint4 val = make_uint4(pk[4 * c], pk[4 * c + 1], pk[4 * c + 2], pk[4 * c + 3]);
                *reinterpret_cast<uint4*>(prow + (c >> 3) * HALF_BYTES + (((c & 7) ^ (r & 7)) << 4)) = val;
            }
            if (j > 0 && __any_sync(0xffffffffu, corr != 1.f)) {  // the reference moved for a row of this warp
                uint32_t o[4][32];
#pragma unroll
                for (int c = 0; c < 4; ++c) tmem_ld_32x32b_x32(lane_addr + 256 + c * 32, o[c]);
                tmem_ld_wait();
#pragma unroll
                for (int c = 0; c < 4; ++c) {
#pragma unroll
                    for (int i = 0; i < 32; ++i) o[c][i] = __float_as_uint(__uint_as_float(o[c][i]) * corr);
                    tmem_st_32x32b_x32(lane_addr + 256 + c * 32, o[c]);
                }
                tmem_st_wait();
            }
            fence_async_proxy();                                  // P was written with ordinary stores
            tcgen05_fence_before();
            mbar_arrive(bar(P_READY));
        }
        // ---- O / l -> out ----
        if (ok && !mbar_wait(bar(PV_DONE), (n_tiles - 1) & 1u, abort_flag)) ok = false;
        if (ok) {
            tcgen05_fence_after();
            const float inv = 1.f / l;
            __nv_bfloat16* dst = out + (size_t)(row0 + r) * out_stride + (size_t)head * HD;
#pragma unroll 1
            for (int c0 = 0; c0 < HD; c0 += 32) {
                uint32_t v[32];
                tmem_ld_32x32b_x32(lane_addr + 256 + c0, v);
                tmem_ld_wait();
                if (r < rows_here) {
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        uint32_t w[4];
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            __nv_bfloat162 b2 = __floats2bfloat162_rn(__uint_as_float(v[8 * i + 2 * e]) * inv,
                                                                      __uint_as_float(v[8 * i + 2 * e + 1]) * inv);
                            w[e] = *reinterpret_cast<uint32_t*>(&b2);
                        }
                        *reinterpret_cast<uint4*>(dst + c0 + 8 * i) = make_uint4(w[0], w[1], w[2], w[3]);
                    }
                }
            }
        }
        if (!ok && lane == 0) { *abort_flag = 1; atomicExch(error_word, 23); }
    }
    tcgen05_fence_before();
    __syncthreads();
    if (warp == 2) {
        tcgen05_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

__device__ int g_attention_tc_error_word = 0;

int* attention_tc_error_word() {
    static int* words[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    if (!words[dev]) {
        void* p = nullptr;
        if (cudaGetSymbolAddress(&p, g_attention_tc_error_word) != cudaSuccess) return nullptr;
        words[dev] = static_cast<int*>(p);
    }
    return words[dev];
}

}  // namespace

// the error word of the tcgen05 attention kernels (this one and the two-tile kernel of attention_prefill_pair.cu)
int* jllm_attention_tc_error_word_ptr() { return attention_tc_error_word(); }

JLLM_BOUNDS_READER(attention_prefill_tc)

JLLM_EXPORT int jllm_attention_prefill_tc_fits(int head_dim, int page_size, int q_stride, int out_stride) {
    return head_dim == 128 && page_size >= 1 && page_size <= 128 && (page_size & (page_size - 1)) == 0 &&
           q_stride % 8 == 0 && out_stride % 8 == 0;
}

JLLM_EXPORT int jllm_attention_prefill_tc_error() {
    int* word = attention_tc_error_word();
    if (!word) return -1;
    int v = 0;
    if (cudaMemcpy(&v, word, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
    if (v) cudaMemset(word, 0, sizeof(int));
    return v;
}

JLLM_EXPORT int jllm_attention_prefill_tc(const void* q, int q_stride, const void* k_cache, const void* v_cache,
                                          long long cache_pages, void* out, int out_stride, const int* seg_start,
                                          const int* seg_len, const int* seg_kv_len, const int* block_tables,
                                          int table_stride, int num_segs, int rows, int heads, int kv_heads,
                                          int head_dim, int page_size, int window, float scale, cudaStream_t stream) {
    JLLM_REQUIRE(rows >= 0 && num_segs >= 0 && heads > 0 && kv_heads > 0 && heads % kv_heads == 0 && cache_pages > 0,
                 "attention_prefill_tc: rows=%d segments=%d heads=%d kv_heads=%d pages=%lld", rows, num_segs, heads,
                 kv_heads, cache_pages);
    JLLM_REQUIRE(jllm_attention_prefill_tc_fits(head_dim, page_size, q_stride, out_stride),
                 "attention_prefill_tc: needs head_dim 128, a power-of-two page size <= 128 and 16-byte aligned rows "
                 "(head_dim=%d page_size=%d q_stride=%d out_stride=%d)", head_dim, page_size, q_stride, out_stride);
    JLLM_REQUIRE(((uintptr_t)q % 16) == 0 && ((uintptr_t)k_cache % 16) == 0 && ((uintptr_t)v_cache % 16) == 0 &&
                     ((uintptr_t)out % 16) == 0 && rows / BQ + num_segs < 65535,
                 "attention_prefill_tc: q, K, V and out must be 16-byte aligned");
    if (rows == 0 || num_segs == 0) return JLLM_OK;
    CUtensorMap map_q, map_k, map_v;
    int rc = tensor_map_for(q, rows, (long long)heads * head_dim, q_stride, BQ, &map_q);
    if (rc != JLLM_OK) return rc;
    const long long cache_rows = cache_pages * kv_heads * page_size;
    rc = tensor_map_for(k_cache, cache_rows, head_dim, head_dim, page_size, &map_k);
    if (rc != JLLM_OK) return rc;
    rc = tensor_map_for(v_cache, cache_rows, head_dim, head_dim, page_size, &map_v);
    if (rc != JLLM_OK) return rc;
    int* error_word = attention_tc_error_word();
    if (!error_word) return jllm_fail(JLLM_CUDA_ERROR, "attention_prefill_tc: no error word");
    int page_shift = 0;
    while ((1 << page_shift) < page_size) ++page_shift;
    auto kern = attention_prefill_tc_kernel;
    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES);
    const dim3 grid(heads, (rows + BQ - 1) / BQ + num_segs);
    jllm_launch(kern, grid, dim3(THREADS), SMEM_BYTES, stream, true, map_q, map_k, map_v, (const __nv_bfloat16*)k_cache,
                (const __nv_bfloat16*)v_cache, (__nv_bfloat16*)out, out_stride, seg_start, seg_len, seg_kv_len,
                block_tables, table_stride, num_segs, heads, kv_heads, page_size, page_shift, (int)cache_pages, window,
                scale * LOG2E, error_word);
    return jllm_check_launch("attention_prefill_tc");
}
