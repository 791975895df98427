// out[m, n] (+)= sum_k a[m, k] * w[n, k] (+ bias[n]) for FEW rows m (a decode step, at most 256): a stream of the
// weights through the 5th-generation tensor cores with the operands swapped.
//
// With few rows the product is nothing but reading W once, so everything is shaped for that read:
//   * W is kept PACKED (ops.pack_weight, once at load): tiles of 128 weight rows x 64 k, each tile the 16 KB image
//     that the tensor cores read from shared memory (rows of 128 bytes, 128-byte swizzle), tile (t, kb) at
//     (t * k_blocks + kb) * 16 KB. One tile is ONE contiguous bulk copy (cp.async.bulk, no multicast) completing on
//     a stage's mbarrier: no thread's registers hold weights, and the memory system sees 16 KB bursts;
//   * the weight rows are the M side of tcgen05.mma (128 rows a tile), the token rows the N side (padded to a
//     multiple of 16), so no tensor-core work is spent on padding 8 tokens to 128; the accumulator [128 weight rows
//     x tokens] lives in tensor memory, two of them so that an epilogue overlaps the next tile's stream;
//   * the k blocks of ALL tiles, in tile order, are dealt out in equal runs over one block per SM, so every SM
//     streams the same number of bytes whatever the matrix's height; a tile whose k blocks fall to several blocks
//     is finished by those blocks together: each parks its part, and when all have, those that end their run in the
//     tile each add up a share of the token columns over the parts in k order (the result does not depend on who
//     came when);
//   * the activations' tile of a k block (tokens x 64) comes by TMA from the [rows, K] matrix (L2 resident);
//   * the producer requests its first weights BEFORE it waits for the kernel in front of it (programmatic dependent
//     launch): weights do not depend on it.
// Roles: warp 0 (one lane) producer, warp 1 (one lane) MMA issuer, warps 2-5 epilogue (bias / float32 residual add /
// SwiGLU over interleaved gate and up rows / store). Every wait is bounded and raises the error word of
// gemm_tcgen05 (codes 11-13).
#include "tcgen05_common.cuh"

namespace {

using namespace tc;

constexpr int WM = 128, BK = 64;
constexpr int W_TILE_BYTES = WM * BK * 2;       // 16 KB
constexpr int THREADS = 192;
constexpr int MAX_TOKENS = 256;                  // the N side of one tcgen05.mma; two accumulators of 256 columns are all of tensor memory
constexpr int MAX_TILES = 65536;                 // counter words at the head of the workspace

__device__ __forceinline__ void tmem_ld_32x32b_x16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}

template <typename Tout>
__global__ void __launch_bounds__(THREADS, 1)
gemm_stream_kernel(const __grid_constant__ CUtensorMap map_a, const __nv_bfloat16* __restrict__ w_packed, VecRef bias,
                   int has_bias, Tout* __restrict__ out, int ldo, int accumulate, int M, int N, int k_blocks, int swiglu,
                   int ntok, int stages, uint32_t tmem_cols, float* __restrict__ partials,
                   int* __restrict__ counters, int* __restrict__ error_word) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* aligned = smem_raw + (base - smem_u32(smem_raw));
    const uint32_t b_bytes = (uint32_t)ntok * 128u, stage_bytes = W_TILE_BYTES + b_bytes;
    const uint32_t bars = base + (uint32_t)stages * stage_bytes;
    auto full_bar = [&](int s) { return bars + 8u * s; };
    auto empty_bar = [&](int s) { return bars + 8u * (stages + s); };
    auto acc_full_bar = [&](int b) { return bars + 8u * (2 * stages + b); };
    auto acc_empty_bar = [&](int b) { return bars + 8u * (2 * stages + 2 + b); };
    uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(aligned + (size_t)stages * stage_bytes + 8 * (2 * stages + 4));
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_base_slot + 1);
    volatile int* last_flag = reinterpret_cast<volatile int*>(tmem_base_slot + 2);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tiles = (N + WM - 1) / WM;
    // the work: (tile, k block) pairs in tile order, one equal run per block
    const long long total = (long long)tiles * k_blocks;
    const long long run_lo = total * blockIdx.x / gridDim.x, run_hi = total * (blockIdx.x + 1) / gridDim.x;

    if (threadIdx.x == 0) {
        for (int s = 0; s < stages; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(acc_full_bar(b), 1);
            mbar_init(acc_empty_bar(b), 4);
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 2) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_base_slot)),
                     "r"(tmem_cols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_base_slot;
    const uint32_t acc_cols = tmem_cols >> 1;       // columns of one accumulator

    if (warp == 0) {
        // ---------------- producer: weights by bulk copy, activations by TMA ----------------
        if (lane == 0) {
            bool ok = true;
            const long long n = run_hi - run_lo;
            const int early = (int)min((long long)stages, n);
            // the first weights are requested before the kernel in front of this one has finished
            for (int i = 0; i < early; ++i) {
                const long long g = run_lo + i;
                mbar_expect_tx(full_bar(i), stage_bytes);
                bulk_copy(base + (uint32_t)i * stage_bytes, w_packed + (size_t)g * (WM * BK), W_TILE_BYTES, full_bar(i));
            }
            pdl_wait();
            pdl_trigger();
            for (int i = 0; i < early; ++i) {
                const int kb = (int)((run_lo + i) % k_blocks);
                tma_load_2d(base + (uint32_t)i * stage_bytes + W_TILE_BYTES, &map_a, kb * BK, 0, full_bar(i));
            }
            int s = early == stages ? 0 : early;
            uint32_t parity = early == stages ? 0u : 1u;      // the ring's second lap waits for the first lap's release
            for (long long i = early; i < n; ++i) {
                const long long g = run_lo + i;
                const int kb = (int)(g % k_blocks);
                if (!mbar_wait(empty_bar(s), parity, abort_flag)) { ok = false; break; }
                const uint32_t dst = base + (uint32_t)s * stage_bytes;
                mbar_expect_tx(full_bar(s), stage_bytes);
                bulk_copy(dst, w_packed + (size_t)g * (WM * BK), W_TILE_BYTES, full_bar(s));
                tma_load_2d(dst + W_TILE_BYTES, &map_a, kb * BK, 0, full_bar(s));
                if (++s == stages) { s = 0; parity ^= 1u; }
            }
            if (!ok) { *abort_flag = 1; atomicExch(error_word, 11); }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            // kind::f16: float32 accumulate, A and B bfloat16, both K-major, N = tokens, M = 128 weight rows
            const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(ntok >> 3) << 17) | ((uint32_t)(WM >> 4) << 24);
            bool ok = true;
            int s = 0;
            uint32_t parity = 0, segment = 0;
            long long g = run_lo;
            while (ok && g < run_hi) {
                const int kb0 = (int)(g % k_blocks);
                const long long seg_end = min(run_hi, g + (k_blocks - kb0));      // the tile's k blocks that are this block's
                const uint32_t buf = segment & 1u;
                if (!mbar_wait(acc_empty_bar(buf), ((segment >> 1) & 1u) ^ 1u, abort_flag)) { ok = false; break; }
                tcgen05_fence_after();
                const uint32_t tmem_d = tmem_base + buf * acc_cols;
                for (bool first = true; g < seg_end; ++g, first = false) {
                    if (!mbar_wait(full_bar(s), parity, abort_flag)) { ok = false; break; }
                    tcgen05_fence_after();
                    const uint32_t w_addr = base + (uint32_t)s * stage_bytes, b_addr = w_addr + W_TILE_BYTES;
#pragma unroll
                    for (int k = 0; k < BK / 16; ++k)
                        tcgen05_mma_bf16(tmem_d, smem_desc_sw128(w_addr + k * 32), smem_desc_sw128(b_addr + k * 32), idesc,
                                         (!first || k > 0) ? 1u : 0u);
                    tcgen05_commit(empty_bar(s));
                    if (++s == stages) { s = 0; parity ^= 1u; }
                }
                if (ok) tcgen05_commit(acc_full_bar(buf));
                ++segment;
            }
            if (!ok) { *abort_flag = 1; atomicExch(error_word, 12); }
        }
    } else {
        // ---------------- epilogue: warps 2..5, TMEM lanes 32 * (warp % 4) = weight rows of the tile ----------------
        pdl_wait();          // the residual stream it may add into was written by the kernels before
        pdl_trigger();
        const int quad = warp & 3;
        bool ok = true;
        uint32_t segment = 0;
        long long g = run_lo;
        const int G = gridDim.x;
        auto run_start = [&](long long c) { return total * c / G; };
        auto block_of = [&](long long index) { return (int)(((index + 1) * G + total - 1) / total - 1); };
        while (ok && g < run_hi) {
            const int tile = (int)(g / k_blocks), kb0 = (int)(g % k_blocks);
            const long long seg_end = min(run_hi, g + (k_blocks - kb0));
            const int kb1 = kb0 + (int)(seg_end - g);
            const uint32_t buf = segment & 1u;
            if (!mbar_wait(acc_full_bar(buf), (segment >> 1) & 1u, abort_flag)) { ok = false; break; }
            tcgen05_fence_after();
            const int row_in_tile = quad * 32 + lane;
            const int n = tile * WM + row_in_tile;                 // this thread's weight row = output column
            const uint32_t taddr = tmem_base + buf * acc_cols + ((uint32_t)(quad * 32) << 16);
            // value of (token m, weight row n): bias / residual / SwiGLU and the store
            auto finalize16 = [&](const float (&v)[16], int m0) {
                if (swiglu) {
                    // rows come in blocks of 16: 8 gate rows, then the 8 up rows of the same hidden units
                    const int unit = (n >> 4) * 8 + (n & 7);
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const float other = __shfl_xor_sync(0xffffffffu, v[j], 8);
                        if ((lane & 8) == 0 && n + 8 < N && m0 + j < M) {
                            const float gt = v[j];
                            out[(size_t)(m0 + j) * ldo + unit] = from_float<Tout>(__fdividef(gt, 1.f + __expf(-gt)) * other);
                        }
                    }
                } else if (n < N) {
                    const float b = has_bias ? bias[n] : 0.f;
                    Tout* dst = out + (size_t)m0 * ldo + n;
                    float old[16];
                    // all the old values are requested before the first store (a load behind a store through the
                    // same pointer would wait for it: 16 round trips instead of one)
#pragma unroll
                    for (int j = 0; j < 16; ++j) old[j] = (accumulate && m0 + j < M) ? to_float(dst[(size_t)j * ldo]) : 0.f;
#pragma unroll
                    for (int j = 0; j < 16; ++j)
                        if (m0 + j < M) dst[(size_t)j * ldo] = from_float<Tout>((v[j] + b) + old[j]);
                }
            };
            if (kb0 == 0 && kb1 == k_blocks) {                      // the whole tile is this block's
#pragma unroll 1
                for (int c0 = 0; c0 < ntok; c0 += 16) {
                    uint32_t raw[16];
                    tmem_ld_32x32b_x16(taddr + c0, raw);
                    tmem_ld_wait();
                    float v[16];
#pragma unroll
                    for (int j = 0; j < 16; ++j) v[j] = __uint_as_float(raw[j]);
                    finalize16(v, c0);
                }
                tcgen05_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(acc_empty_bar(buf));
            } else {
                // ---- this block holds some of the tile's k blocks: park the part ([block][first or later part of the
                // block][token][128 rows]); the blocks that hold parts of one tile are consecutive ----
                const long long tile_g0 = (long long)tile * k_blocks;
                const int c_first = block_of(tile_g0), parts = block_of(tile_g0 + k_blocks - 1) - c_first + 1;
                auto part_of = [&](int c) {
                    const int slot = run_start(c) >= tile_g0 ? 0 : 1;
                    return partials + (size_t)(2 * c + slot) * MAX_TOKENS * WM + row_in_tile;
                };
                float* mine = part_of(blockIdx.x);
#pragma unroll 1
                for (int c0 = 0; c0 < ntok; c0 += 16) {
                    uint32_t raw[16];
                    tmem_ld_32x32b_x16(taddr + c0, raw);
                    tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < 16; ++j) __stcg(mine + (size_t)(c0 + j) * WM, __uint_as_float(raw[j]));
                }
                tcgen05_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(acc_empty_bar(buf));
                asm volatile("bar.sync 1, 128;" ::: "memory");       // the four epilogue warps have written
                // The parts of a tile are added up by the blocks that hold one and END their run in it: number p of them takes
                // the 16-token chunks p, p + np, ... (a block may have none), so that each has one batch of loads to wait
                // for instead of one block having them all. They finish their runs at about the same time, so waiting for
                // one another costs little, and nothing is behind that wait in their runs. The block that only BEGINS its
                // run in this tile (the tile's last holder, if its run goes on into other tiles) parks its part long
                // before and waits for nobody: a wait there would hold up its later tiles, and through them the blocks
                // that wait for those. Every holder counts itself in; the wait is a bounded one on that counter (all
                // blocks of the grid are resident, one per SM).
                const int p_me = (int)blockIdx.x - c_first, chunks = ntok >> 4;
                const bool tail_goes_on = run_start(c_first + parts) > tile_g0 + k_blocks;
                const int np = parts - (tail_goes_on ? 1 : 0);              // holders that take part in the adding
                const bool takes_part = seg_end == run_hi;                   // (p_me < np says the same)
                const bool has_share = takes_part && p_me < chunks;
                if (warp == 2 && lane == 0) {
                    __threadfence();
                    atomicAdd(&counters[tile], 1);
                    int seen = has_share ? 0 : parts;
                    for (uint32_t spin = 0; seen < parts && spin < SPIN_LIMIT; ++spin) {
                        asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(seen) : "l"(counters + tile) : "memory");
                        if (seen < parts) {
                            if ((spin & 255u) == 255u && *abort_flag) break;
                            __nanosleep(32);
                        }
                    }
                    *last_flag = seen >= parts;
                }
                asm volatile("bar.sync 1, 128;" ::: "memory");
                if (!*last_flag) { ok = false; break; }
                if (has_share) {
#pragma unroll 1
                    for (int c0 = p_me * 16; c0 < ntok; c0 += np * 16) {
                        float acc[16];
#pragma unroll
                        for (int j = 0; j < 16; ++j) acc[j] = 0.f;
                        for (int p0 = 0; p0 < parts; p0 += 4) {     // four parts' loads in flight, added in k order
                            float x[4][16];
#pragma unroll
                            for (int q = 0; q < 4; ++q) {
                                const float* src = part_of(c_first + min(p0 + q, parts - 1)) + (size_t)c0 * WM;
#pragma unroll
                                for (int j = 0; j < 16; ++j) x[q][j] = __ldcg(src + (size_t)j * WM);
                            }
#pragma unroll
                            for (int q = 0; q < 4; ++q)
                                if (p0 + q < parts) {
#pragma unroll
                                    for (int j = 0; j < 16; ++j) acc[j] += x[q][j];
                                }
                        }
                        finalize16(acc, c0);
                    }
                }
                // of those that take part, the one that is done last puts the tile's two counters back to zero for the next
                // product (all have read the first counter by then, and the early holder never reads it)
                asm volatile("bar.sync 1, 128;" ::: "memory");
                if (takes_part && warp == 2 && lane == 0) {
                    if (atomicAdd(&counters[MAX_TILES + tile], 1) == np - 1) {
                        counters[tile] = 0;
                        counters[MAX_TILES + tile] = 0;
                        __threadfence();
                    }
                }
            }
            g = seg_end;
            ++segment;
        }
        if (!ok && lane == 0) { *abort_flag = 1; atomicExch(error_word, 13); }
    }
    tcgen05_fence_before();
    __syncthreads();
    if (warp == 2) {
        tcgen05_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(tmem_cols) : "memory");
    }
}

}  // namespace

// The error word is gemm_tcgen05's (one word for the tcgen05 products).
int* jllm_gemm_error_word();

JLLM_EXPORT long long jllm_gemm_stream_workspace_floats() { return 2LL * MAX_TILES + 2LL * 160 * MAX_TOKENS * WM; }

// a [M, K] bfloat16 (row stride lda), w_packed: ops.pack_weight of the [N, K] weight (k padded to k_blocks * 64, rows
// to a multiple of 128, zeros), out [M, N] (or [M, N / 2] with swiglu) float32 or bfloat16. `workspace`: zeroed floats
// (counters, then parked parts), at least jllm_gemm_stream_workspace_floats().
JLLM_EXPORT int jllm_gemm_stream(const void* a, int lda, const void* w_packed, int k_blocks, const void* bias,
                                 int bias_dtype, void* out, int out_dtype, int ldo, int accumulate, int M, int N, int K,
                                 int swiglu, float* workspace, long long workspace_floats, int max_blocks,
                                 cudaStream_t stream) {
    JLLM_REQUIRE(M >= 1 && M <= MAX_TOKENS && N >= 1 && K >= 8 && K % 8 == 0 && lda % 8 == 0 && ((uintptr_t)a % 16) == 0 &&
                     ((uintptr_t)w_packed % 16) == 0,
                 "gemm_stream: needs 1 <= rows <= %d, K %% 8 == 0 and 16-byte aligned rows and weights "
                 "(M=%d N=%d K=%d lda=%d)", MAX_TOKENS, M, N, K, lda);
    JLLM_REQUIRE(k_blocks == (K + BK - 1) / BK, "gemm_stream: the packed weight has %d k blocks, K=%d needs %d", k_blocks, K,
                 (K + BK - 1) / BK);
    JLLM_REQUIRE(ldo >= (swiglu ? N / 2 : N), "gemm_stream: ldo=%d < N=%d", ldo, N);
    JLLM_REQUIRE(!swiglu || (N % 16 == 0 && !bias && !accumulate),
                 "gemm_stream: the SwiGLU epilogue needs N %% 16 == 0, no bias and no accumulation (N=%d)", N);
    const int tiles = (N + WM - 1) / WM;
    JLLM_REQUIRE(tiles <= MAX_TILES && workspace != nullptr && workspace_floats >= jllm_gemm_stream_workspace_floats(),
                 "gemm_stream: %d tiles (at most %d) and a workspace of %lld floats (got %lld)", tiles, MAX_TILES,
                 jllm_gemm_stream_workspace_floats(), workspace_floats);
    const int sms = jllm_device_sm_count() > 0 ? jllm_device_sm_count() : 1;
    const int ntok = (M + 15) / 16 * 16;
    uint32_t acc_cols = 32;
    while ((int)acc_cols < ntok) acc_cols <<= 1;
    const uint32_t tmem_cols = 2 * acc_cols;
    const size_t stage_bytes = W_TILE_BYTES + (size_t)ntok * 128;
    const size_t budget = 200 * 1024;
    int stages = (int)(budget / stage_bytes);
    if (stages > 12) stages = 12;
    const size_t smem = (size_t)stages * stage_bytes + 1024 + 8 * (2 * stages + 4) + 64;
    CUtensorMap map_a;
    int rc = tc::tensor_map_for(a, M, K, lda, ntok, &map_a);
    if (rc != JLLM_OK) return rc;
    int* error_word = jllm_gemm_error_word();
    if (!error_word) return jllm_fail(JLLM_CUDA_ERROR, "gemm_stream: no error word");
    const long long total = (long long)tiles * k_blocks;
    int grid = total < sms ? (int)total : sms;
    if (grid > 160) grid = 160;
    if (max_blocks > 0 && grid > max_blocks) grid = max_blocks;
    int* counters = reinterpret_cast<int*>(workspace);
    float* partials = workspace + 2 * MAX_TILES;      // two counters per tile (counted in, done), then the parked parts
    const VecRef b{bias, bias_dtype};
#define JLLM_STREAM_GO(T)                                                                                           \
    do {                                                                                                            \
        auto kern = gemm_stream_kernel<T>;                                                                          \
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);                         \
        jllm_launch(kern, dim3(grid), dim3(THREADS), smem, stream, LAUNCH_DEPENDENT, map_a,                          \
                    (const __nv_bfloat16*)w_packed, b, (int)(bias != nullptr), (T*)out, ldo, accumulate, M, N, k_blocks, \
                    swiglu, ntok, stages, tmem_cols, partials, counters, error_word);                               \
    } while (0)
    if (out_dtype == JLLM_F32) JLLM_STREAM_GO(float); else JLLM_STREAM_GO(__nv_bfloat16);
#undef JLLM_STREAM_GO
    return jllm_check_launch("gemm_stream");
}
