// Paged causal flash attention for prompt portions on tcgen05, two query tiles per block (head size 128).
//
// One block per (256 query rows of a segment, head): query tiles A (the first 128 rows) and B (the next 128) share
// every key / value tile that the loader brings in. Tensor memory holds S_A, S_B, O_A, O_B (4 x 128 columns of
// float32). The probabilities never touch shared memory: a softmax thread writes its row of P as packed bfloat16 over
// the first 64 columns of its own S (tcgen05.st), and the second product reads its A operand from tensor memory:
//     S_x = Q_x K^T          A, B from shared memory (K-major)            D = S_x
//     O_x += P_x V           A = P_x from tensor memory, B = V (MN-major)  D = O_x
// Warp roles: warp 0 loads (TMA boxes per page and 64-column half for whole tiles, cp.async with zero fill for the
// tiles at the edges of the visible keys), warp 1 issues the MMAs, warps 2-5 are the softmax of tile A and warps 6-9
// that of tile B (thread = query row = TMEM lane). The MMA warp issues, per key tile j,
//     P_A ready?  O_A += P_A V_j,  S_A = Q_A K_(j+1)^T,   P_B ready?  O_B += P_B V_j,  S_B = Q_B K_(j+1)^T
// so while the softmax of one query tile runs, the tensor cores work for the other one. The MMAs of one thread
// complete in order: "S_x of tile j + 1 is complete" therefore also says that O_x += P_x V_j has completed, and the
// softmax may overwrite S_x with P_x and rescale O_x without another barrier. O is rescaled only when a row's maximum
// grew by more than 2^8 (the reference point of the exponentials stays until then).
// Every mbarrier wait is bounded; a wait that runs out raises the error word and all roles leave.
//
// Requirements: bfloat16, head_dim 128, page_size a power of two <= 128, 16-byte aligned q rows.
#include "tcgen05_common.cuh"

namespace {

using namespace tc;

constexpr int BQ = 128, BKV = 128, HD = 128, THREADS = 320;
constexpr int TILE_BYTES = 128 * HD * 2;           // 32 KB: each Q, K and V tile
constexpr int HALF_BYTES = 128 * 64 * 2;           // one 64-column half of a tile
constexpr float LOG2E = 1.4426950408889634f;
constexpr size_t SMEM_BYTES = 6 * TILE_BYTES + 1024 + 256;
constexpr int TMEM_COLS = 512;                      // S_A 0, S_B 128, O_A 256, O_B 384

// D[tmem] (+)= A[tmem] * B[smem]: the A operand (128 rows x 16 bfloat16, packed two to a column) from tensor memory
__device__ __forceinline__ void tcgen05_mma_bf16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc,
                                                    uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(tmem_d), "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}

__global__ void __launch_bounds__(THREADS, 1)
attention_prefill_pair_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                              const __grid_constant__ CUtensorMap map_v, const __nv_bfloat16* __restrict__ k_cache,
                              const __nv_bfloat16* __restrict__ v_cache, __nv_bfloat16* __restrict__ out, int out_stride,
                              const int* __restrict__ seg_start, const int* __restrict__ seg_len,
                              const int* __restrict__ seg_kv_len, const int* __restrict__ block_tables,
                              int table_stride, int num_segs, int heads, int kv_heads, int page_size, int page_shift,
                              int num_pages, int window, float scale_log2, int* __restrict__ error_word) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* aligned = smem_raw + (base - smem_u32(smem_raw));
    auto s_q = [&](int x) { return base + x * TILE_BYTES; };
    auto s_k = [&](int b) { return base + (2 + b) * TILE_BYTES; };
    auto s_v = [&](int b) { return base + (4 + b) * TILE_BYTES; };
    const uint32_t bars = base + 6 * TILE_BYTES;
    // Q_FULL; K_FULL[2], V_FULL[2], K_EMPTY[2], V_EMPTY[2]; then per query tile x: S_FULL, P_READY, PV_DONE
    enum { Q_FULL = 0, K_FULL = 1, V_FULL = 3, K_EMPTY = 5, V_EMPTY = 7, S_FULL = 9, P_READY = 11, PV_DONE = 13 };
    auto bar = [&](int i) { return bars + 8u * i; };
    uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(aligned + 6 * TILE_BYTES + 8 * 16);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_base_slot + 1);

    // ---- which pair of tiles of which segment: the pairs with the most keys before them start first ----
    int seg = 0, pair = gridDim.y - 1 - blockIdx.y;
    for (; seg < num_segs; ++seg) {
        const int np = (seg_len[seg] + 2 * BQ - 1) / (2 * BQ);
        if (pair < np) break;
        pair -= np;
    }
    if (seg >= num_segs) return;                       // whole block: before any barrier or allocation
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int head = blockIdx.x, kvh = head / (heads / kv_heads);
    const int n_rows = seg_len[seg], q0 = pair * 2 * BQ;
    const int rows_here = min(2 * BQ, n_rows - q0);                    // rows of both tiles
    const int row0 = seg_start[seg] + q0;
    const int pos0 = seg_kv_len[seg] - n_rows + q0, pos_last = pos0 + rows_here - 1;
    const int first_key = window > 0 ? max(0, pos0 + 1 - window) : 0;
    const int kt_lo = first_key / BKV;
    // key tiles that each query tile walks (tile B none if the pair has at most 128 rows)
    const int rows_x[2] = {min(BQ, rows_here), max(0, rows_here - BQ)};
    const int n_x[2] = {(pos0 + rows_x[0] - 1) / BKV - kt_lo + 1, rows_x[1] > 0 ? pos_last / BKV - kt_lo + 1 : 0};
    const int n_tiles = max(n_x[0], n_x[1]);
    const int* table = block_tables + (size_t)seg * table_stride;

    if (threadIdx.x == 0) {
        mbar_init(bar(Q_FULL), 1);
        for (int b = 0; b < 2; ++b) {
            mbar_init(bar(K_FULL + b), 1);
            mbar_init(bar(V_FULL + b), 1);
            mbar_init(bar(K_EMPTY + b), 1);
            mbar_init(bar(V_EMPTY + b), 1);
            mbar_init(bar(S_FULL + b), 1);
            mbar_init(bar(P_READY + b), 128);
            mbar_init(bar(PV_DONE + b), 1);
        }
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
            mbar_expect_tx(bar(Q_FULL), rows_x[1] > 0 ? 2 * TILE_BYTES : TILE_BYTES);
            for (int x = 0; x < (rows_x[1] > 0 ? 2 : 1); ++x) {
                tma_load_2d(s_q(x), &map_q, head * HD, row0 + x * BQ, bar(Q_FULL));
                tma_load_2d(s_q(x) + HALF_BYTES, &map_q, head * HD + 64, row0 + x * BQ, bar(Q_FULL));
            }
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
        if (!ok && lane == 0) { *abort_flag = 1; atomicExch(error_word, 31); }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            bool ok = mbar_wait(bar(Q_FULL), 0, abort_flag);
            auto issue_s = [&](int x, int j) {      // S_x = Q_x K_j^T (the K tile has been waited for)
                const uint32_t d = tmem_base + x * 128;
#pragma unroll
                for (int k = 0; k < HD / 16; ++k) {
                    const uint32_t o = (k >> 2) * HALF_BYTES + (k & 3) * 32;
                    tcgen05_mma_bf16(d, smem_desc_sw128(s_q(x) + o), smem_desc_sw128(s_k(j & 1) + o), IDESC_128x128_KK, k > 0);
                }
                tcgen05_commit(bar(S_FULL + x));
            };
            auto issue_pv = [&](int x, int j) {     // O_x += P_x V_j
                const uint32_t d = tmem_base + 256 + x * 128, a = tmem_base + x * 128;
#pragma unroll
                for (int k = 0; k < BKV / 16; ++k)
                    tcgen05_mma_bf16_ts(d, a + k * 8, smem_desc_mn_sw128(s_v(j & 1) + k * 2048, HALF_BYTES), IDESC_128x128_KMN,
                                        (j > 0 || k > 0) ? 1u : 0u);
                tcgen05_commit(bar(PV_DONE + x));
            };
            if (ok) ok = mbar_wait(bar(K_FULL + 0), 0, abort_flag);
            if (ok) {
                tcgen05_fence_after();
                for (int x = 0; x < 2; ++x)
                    if (n_x[x] > 0) issue_s(x, 0);
                tcgen05_commit(bar(K_EMPTY + 0));
            }
            for (int j = 0; j < n_tiles && ok; ++j) {
                const int b = j & 1;
                if (!mbar_wait(bar(V_FULL + b), (j >> 1) & 1u, abort_flag)) { ok = false; break; }
                const bool more = j + 1 < n_tiles;
                if (more && !mbar_wait(bar(K_FULL + (b ^ 1)), ((j + 1) >> 1) & 1u, abort_flag)) { ok = false; break; }
                for (int x = 0; x < 2 && ok; ++x) {
                    if (j < n_x[x]) {
                        if (!mbar_wait(bar(P_READY + x), j & 1u, abort_flag)) { ok = false; break; }
                        tcgen05_fence_after();
                        issue_pv(x, j);
                    }
                    if (j + 1 < n_x[x]) issue_s(x, j + 1);
                }
                if (!ok) break;
                tcgen05_commit(bar(V_EMPTY + b));
                if (more) tcgen05_commit(bar(K_EMPTY + (b ^ 1)));
            }
            if (!ok) { *abort_flag = 1; atomicExch(error_word, 32); }
        }
    } else {
        // ---------------- softmax of tile x: thread = query row = TMEM lane ----------------
        const int x = warp >= 6 ? 1 : 0, quad = warp & 3, r = quad * 32 + lane;
        const int n_mine = n_x[x];
        if (n_mine > 0) {
            const uint32_t lane_addr = tmem_base + ((uint32_t)(quad * 32) << 16);
            const uint32_t s_addr = lane_addr + x * 128, o_addr = lane_addr + 256 + x * 128;
            const int P = pos0 + x * BQ + min(r, rows_x[x] - 1);   // rows past the end copy the last row, and are not stored
            const int lo = window > 0 ? max(0, P + 1 - window) : 0;
            const int pos0_x = pos0 + x * BQ;
            float m = -INFINITY, l = 0.f;
            bool ok = true;
            for (int j = 0; j < n_mine && ok; ++j) {
                const int key0 = (kt_lo + j) * BKV;
                if (!mbar_wait(bar(S_FULL + x), j & 1u, abort_flag)) { ok = false; break; }
                tcgen05_fence_after();
                const bool masked = key0 + BKV - 1 > pos0_x || key0 < lo;
                uint32_t v[4][32];
#pragma unroll
                for (int c = 0; c < 4; ++c) tmem_ld_32x32b_x32(s_addr + c * 32, v[c]);
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
                // (four chains, then their maximum: one chain of 128 dependent comparisons is pure latency for a warp
                // that has its scheduler almost to itself)
                float mxs[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
                for (int c = 0; c < 4; ++c)
#pragma unroll
                    for (int i = 0; i < 32; ++i) mxs[i & 3] = fmaxf(mxs[i & 3], __uint_as_float(v[c][i]));
                const float mx = fmaxf(fmaxf(mxs[0], mxs[1]), fmaxf(mxs[2], mxs[3]));
                const float m_cand = fmaxf(m, mx * scale_log2);
                const float m_new = (m_cand - m > 8.f) ? m_cand : m;
                const float m_use = m_new == -INFINITY ? 0.f : m_new;
                const float corr = fast_exp2(m - m_use);
                float sums[2] = {0.f, 0.f};
                // P over the first 64 columns of S: two stores of 32 packed columns
#pragma unroll
                for (int half = 0; half < 2; ++half) {
                    uint32_t pk[32];
#pragma unroll
                    for (int c = 0; c < 2; ++c)
#pragma unroll
                        for (int i = 0; i < 32; i += 2) {
                            const float p0 = fast_exp2(fmaf(__uint_as_float(v[2 * half + c][i]), scale_log2, -m_use));
                            const float p1 = fast_exp2(fmaf(__uint_as_float(v[2 * half + c][i + 1]), scale_log2, -m_use));
                            sums[(i >> 1) & 1] += p0 + p1;
                            __nv_bfloat162 b2 = __floats2bfloat162_rn(p0, p1);
                            pk[(c * 32 + i) >> 1] = *reinterpret_cast<uint32_t*>(&b2);
                        }
                    tmem_st_32x32b_x32(s_addr + half * 32, pk);
                }
                m = m_new;
                l = l * corr + (sums[0] + sums[1]);
                if (j > 0 && __any_sync(0xffffffffu, corr != 1.f)) {  // the reference moved for a row of this warp
#pragma unroll 1
                    for (int c = 0; c < 4; ++c) {
                        uint32_t o[32];
                        tmem_ld_32x32b_x32(o_addr + c * 32, o);
                        tmem_ld_wait();
#pragma unroll
                        for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * corr);
                        tmem_st_32x32b_x32(o_addr + c * 32, o);
                    }
                }
                tmem_st_wait();
                tcgen05_fence_before();
                mbar_arrive(bar(P_READY + x));
            }
            // ---- O / l -> out ----
            if (ok && !mbar_wait(bar(PV_DONE + x), (n_mine - 1) & 1u, abort_flag)) ok = false;
            if (ok) {
                tcgen05_fence_after();
                const float inv = 1.f / l;
                __nv_bfloat16* dst = out + (size_t)(row0 + x * BQ + r) * out_stride + (size_t)head * HD;
#pragma unroll 1
                for (int c0 = 0; c0 < HD; c0 += 32) {
                    uint32_t v[32];
                    tmem_ld_32x32b_x32(o_addr + c0, v);
                    tmem_ld_wait();
                    if (r < rows_x[x]) {
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
            if (!ok && lane == 0) { *abort_flag = 1; atomicExch(error_word, 33); }
        }
    }
    tcgen05_fence_before();
    __syncthreads();
    if (warp == 2) {
        tcgen05_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

}  // namespace

int* jllm_attention_tc_error_word_ptr();   // attention_prefill_tc.cu: one error word for both tcgen05 attention kernels

JLLM_BOUNDS_READER(attention_prefill_pair)

JLLM_EXPORT int jllm_attention_prefill_pair(const void* q, int q_stride, const void* k_cache, const void* v_cache,
                                            long long cache_pages, void* out, int out_stride, const int* seg_start,
                                            const int* seg_len, const int* seg_kv_len, const int* block_tables,
                                            int table_stride, int num_segs, int rows, int heads, int kv_heads,
                                            int head_dim, int page_size, int window, float scale, cudaStream_t stream) {
    JLLM_REQUIRE(rows >= 0 && num_segs >= 0 && heads > 0 && kv_heads > 0 && heads % kv_heads == 0 && cache_pages > 0,
                 "attention_prefill_pair: rows=%d segments=%d heads=%d kv_heads=%d pages=%lld", rows, num_segs, heads,
                 kv_heads, cache_pages);
    JLLM_REQUIRE(head_dim == 128 && page_size >= 1 && page_size <= 128 && (page_size & (page_size - 1)) == 0 &&
                     q_stride % 8 == 0 && out_stride % 8 == 0,
                 "attention_prefill_pair: needs head_dim 128, a power-of-two page size <= 128 and 16-byte aligned rows "
                 "(head_dim=%d page_size=%d q_stride=%d out_stride=%d)", head_dim, page_size, q_stride, out_stride);
    JLLM_REQUIRE(((uintptr_t)q % 16) == 0 && ((uintptr_t)k_cache % 16) == 0 && ((uintptr_t)v_cache % 16) == 0 &&
                     ((uintptr_t)out % 16) == 0,
                 "attention_prefill_pair: q, K, V and out must be 16-byte aligned");
    JLLM_REQUIRE(rows / (2 * BQ) + num_segs < 65535, "attention_prefill_pair: %d rows in %d segments are too many blocks",
                 rows, num_segs);
    if (rows == 0 || num_segs == 0) return JLLM_OK;
    CUtensorMap map_q, map_k, map_v;
    int rc = tensor_map_for(q, rows, (long long)heads * head_dim, q_stride, BQ, &map_q);
    if (rc != JLLM_OK) return rc;
    const long long cache_rows = cache_pages * kv_heads * page_size;
    rc = tensor_map_for(k_cache, cache_rows, head_dim, head_dim, page_size, &map_k);
    if (rc != JLLM_OK) return rc;
    rc = tensor_map_for(v_cache, cache_rows, head_dim, head_dim, page_size, &map_v);
    if (rc != JLLM_OK) return rc;
    int* error_word = jllm_attention_tc_error_word_ptr();
    if (!error_word) return jllm_fail(JLLM_CUDA_ERROR, "attention_prefill_pair: no error word");
    int page_shift = 0;
    while ((1 << page_shift) < page_size) ++page_shift;
    auto kern = attention_prefill_pair_kernel;
    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES);
    const dim3 grid(heads, (rows + 2 * BQ - 1) / (2 * BQ) + num_segs);
    jllm_launch(kern, grid, dim3(THREADS), SMEM_BYTES, stream, true, map_q, map_k, map_v, (const __nv_bfloat16*)k_cache,
                (const __nv_bfloat16*)v_cache, (__nv_bfloat16*)out, out_stride, seg_start, seg_len, seg_kv_len,
                block_tables, table_stride, num_segs, heads, kv_heads, page_size, page_shift, (int)cache_pages, window,
                scale * LOG2E, error_word);
    return jllm_check_launch("attention_prefill_pair");
}
