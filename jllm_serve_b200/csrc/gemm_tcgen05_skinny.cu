// out[m, n] (+)= sum_k a[m, k] * w[n, k] (+ bias[n]) for few rows (m <= 128) on tcgen05: the operands swapped,
// the weight matrix streamed through a deep TMA ring, K split over blocks.
//
// With few rows the product is a stream of the weights and the only question is how many bytes every SM
// keeps in flight. Here a block keeps up to ten 18-34 KB stages on their way with a single producer lane:
// each stage is a 128 x 64 tile of W (the M side of the MMA: no tensor-core row is wasted on padding rows)
// and a (rows padded to 16) x 64 tile of the activations (the N side). The accumulator D[weight row, token]
// lives in tensor memory, two of them, so the epilogue of one unit overlaps the stream of the next.
//
// Work units are (128-row tile of W, slice of K); a persistent grid of one block per SM walks them. When K
// is split, every unit writes its partial tile to a workspace and bumps the tile's counter; the block that
// finds the counter at "all others done" adds the partials in slice order (so the result does not depend
// on which block came last) and runs the epilogue: bias, float32 residual add, or SwiGLU over interleaved
// gate / up rows (a lane holds a gate value, lane + 8 its up value). Nobody ever waits for another block.
// The counters return to zero by themselves. All mbarrier waits are bounded, as in gemm_tcgen05.cu.
//
// Requirements: bfloat16, 1 <= M <= 128, K a multiple of 8, 16-byte aligned rows; workspace of
// jllm_gemm_skinny_workspace_floats() floats whose first JLLM_SKINNY_MAX_TILES words start as zero.
#include "tcgen05_common.cuh"

namespace {

using namespace tc;

constexpr int BW = 128, BK = 64, THREADS = 192, MAX_STAGES = 10, MAX_TILES = 4096;
constexpr int W_BYTES = BW * BK * 2;
constexpr size_t SMEM_LIMIT = 200 * 1024;

__device__ __forceinline__ void tmem_ld_32x32b_x16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}

struct Plan {
    int tiles, splits, k_blocks, stages, tok_pad, stage_bytes, tmem_cols;
};

template <typename Tout>
__global__ void __launch_bounds__(THREADS, 1)
gemm_skinny_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_a, VecRef bias,
                   int has_bias, Tout* __restrict__ out, int ldo, int accumulate, int M, int N, int K, int swiglu,
                   Plan plan, float* __restrict__ partials, int* __restrict__ counters, int* __restrict__ error_word) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* aligned = smem_raw + (base - smem_u32(smem_raw));
    const int stages = plan.stages, stage_bytes = plan.stage_bytes;
    const uint32_t bars = base + stages * stage_bytes;
    auto full_bar = [&](int s) { return bars + 8u * s; };
    auto empty_bar = [&](int s) { return bars + 8u * (MAX_STAGES + s); };
    auto acc_full_bar = [&](int b) { return bars + 8u * (2 * MAX_STAGES + b); };
    auto acc_empty_bar = [&](int b) { return bars + 8u * (2 * MAX_STAGES + 2 + b); };
    uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(aligned + stages * stage_bytes + 8 * (2 * MAX_STAGES + 4));
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_base_slot + 1);
    volatile int* last_flag = reinterpret_cast<volatile int*>(tmem_base_slot + 2);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int units = plan.tiles * plan.splits;
    const int tok_pad = plan.tok_pad;
    // instruction descriptor: float32 accumulate, bfloat16 A and B, both K-major, N = padded tokens, M = 128
    const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(tok_pad >> 3) << 17) | ((uint32_t)(BW >> 4) << 24);

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
                     "r"(plan.tmem_cols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_base_slot;

    // the k blocks of split s of a tile: an even share, the first (k_blocks % splits) slices one block longer
    auto slice = [&](int s, int& lo, int& hi) {
        const int q = plan.k_blocks / plan.splits, r = plan.k_blocks % plan.splits;
        lo = s * q + min(s, r);
        hi = lo + q + (s < r ? 1 : 0);
    };

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        // The weights do not depend on the kernel before this one: the ring is first filled with weight tiles
        // alone, then the producer waits for the predecessor and adds the activation tiles of those stages
        // (a stage's barrier completes when both have landed). After that every stage gets both at once.
        if (lane == 0) {
            struct Cursor {
                int unit, kb, hi;
            };
            auto start_unit = [&](Cursor& c) {
                if (c.unit < units) {
                    int lo;
                    slice(c.unit % plan.splits, lo, c.hi);
                    c.kb = lo;
                }
            };
            auto advance = [&](Cursor& c) {
                if (++c.kb >= c.hi) {
                    c.unit += gridDim.x;
                    start_unit(c);
                }
            };
            Cursor head{(int)blockIdx.x, 0, 0};
            start_unit(head);
            Cursor first = head;
            int filled = 0;
            for (; filled < stages && head.unit < units; ++filled, advance(head)) {
                mbar_expect_tx(full_bar(filled), stage_bytes);
                tma_load_2d(base + filled * stage_bytes, &map_w, head.kb * BK, (head.unit / plan.splits) * BW, full_bar(filled));
            }
            pdl_wait();
            pdl_trigger();
            for (int j = 0; j < filled; ++j, advance(first))
                tma_load_2d(base + j * stage_bytes + W_BYTES, &map_a, first.kb * BK, 0, full_bar(j));
            bool ok = true;
            for (uint32_t it = filled; head.unit < units; ++it, advance(head)) {
                const int s = it % stages;
                if (!mbar_wait(empty_bar(s), ((it / stages) & 1u) ^ 1u, abort_flag)) { ok = false; break; }
                const uint32_t dst = base + s * stage_bytes;
                mbar_expect_tx(full_bar(s), stage_bytes);
                tma_load_2d(dst, &map_w, head.kb * BK, (head.unit / plan.splits) * BW, full_bar(s));
                tma_load_2d(dst + W_BYTES, &map_a, head.kb * BK, 0, full_bar(s));
            }
            if (!ok) { *abort_flag = 1; atomicExch(error_word, 11); }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            uint32_t it = 0, local = 0;
            bool ok = true;
            for (int unit = blockIdx.x; unit < units && ok; unit += gridDim.x, ++local) {
                const int split = unit % plan.splits;
                int lo, hi;
                slice(split, lo, hi);
                const uint32_t buf = local & 1u;
                if (!mbar_wait(acc_empty_bar(buf), ((local >> 1) & 1u) ^ 1u, abort_flag)) { ok = false; break; }
                tcgen05_fence_after();
                const uint32_t tmem_d = tmem_base + buf * tok_pad;
                for (int kb = lo; kb < hi; ++kb, ++it) {
                    const int s = it % stages;
                    if (!mbar_wait(full_bar(s), (it / stages) & 1u, abort_flag)) { ok = false; break; }
                    tcgen05_fence_after();
                    const uint32_t w_addr = base + s * stage_bytes, a_addr = w_addr + W_BYTES;
#pragma unroll
                    for (int k = 0; k < BK / 16; ++k)
                        tcgen05_mma_bf16(tmem_d, smem_desc_sw128(w_addr + k * 32), smem_desc_sw128(a_addr + k * 32), idesc,
                                         (kb > lo || k > 0) ? 1u : 0u);
                    tcgen05_commit(empty_bar(s));
                }
                if (ok) tcgen05_commit(acc_full_bar(buf));
            }
            if (!ok) { *abort_flag = 1; atomicExch(error_word, 12); }
        }
    } else {
        // ---------------- epilogue: warps 2..5; lane = weight row, columns = tokens ----------------
        pdl_wait();          // out (a residual) and the workspace may still be in use by the predecessor
        pdl_trigger();
        const int quad = warp & 3;
        uint32_t local = 0;
        bool ok = true;
        for (int unit = blockIdx.x; unit < units && ok; unit += gridDim.x, ++local) {
            const int tile = unit / plan.splits, split = unit % plan.splits;
            const uint32_t buf = local & 1u;
            if (!mbar_wait(acc_full_bar(buf), (local >> 1) & 1u, abort_flag)) { ok = false; break; }
            tcgen05_fence_after();
            const int row_in_tile = quad * 32 + lane;
            const int n = tile * BW + row_in_tile;
            const uint32_t taddr = tmem_base + buf * tok_pad + ((uint32_t)(quad * 32) << 16);
            // partial tiles: [unit][128 weight rows][tok_pad tokens], so a thread's 16 tokens are 64 contiguous bytes
            float4* mine = reinterpret_cast<float4*>(partials + ((size_t)unit * BW + row_in_tile) * tok_pad);
            bool finish = plan.splits == 1;
            if (plan.splits > 1) {
                for (int c0 = 0; c0 < tok_pad; c0 += 16) {
                    uint32_t v[16];
                    tmem_ld_32x32b_x16(taddr + c0, v);
                    tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < 4; ++j)
                        __stcg(mine + (c0 >> 2) + j, make_float4(__uint_as_float(v[4 * j]), __uint_as_float(v[4 * j + 1]),
                                                                 __uint_as_float(v[4 * j + 2]), __uint_as_float(v[4 * j + 3])));
                }
                tcgen05_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(acc_empty_bar(buf));      // the accumulator is free again
                asm volatile("bar.sync 1, 128;" ::: "memory");       // the four epilogue warps have written
                if (warp == 2 && lane == 0) {
                    __threadfence();                                  // ... and their writes go out before the count
                    const int seen = atomicAdd(&counters[tile], 1);
                    *last_flag = seen == plan.splits - 1;
                    if (seen == plan.splits - 1) {
                        counters[tile] = 0;                           // back to zero for the next product
                        __threadfence();
                    }
                }
                asm volatile("bar.sync 1, 128;" ::: "memory");
                finish = *last_flag != 0;
            }
            if (finish) {
                for (int c0 = 0; c0 < tok_pad; c0 += 16) {
                    float acc[16];
                    if (plan.splits == 1) {
                        uint32_t v[16];
                        tmem_ld_32x32b_x16(taddr + c0, v);
                        tmem_ld_wait();
#pragma unroll
                        for (int j = 0; j < 16; ++j) acc[j] = __uint_as_float(v[j]);
                    } else {
#pragma unroll
                        for (int j = 0; j < 16; ++j) acc[j] = 0.f;
                        // slice order (deterministic), eight slices' loads in flight at a time
                        for (int s0 = 0; s0 < plan.splits; s0 += 8) {
                            float4 part[8][4];
#pragma unroll
                            for (int u = 0; u < 8; ++u) {
                                const float4* p = reinterpret_cast<const float4*>(
                                    partials + ((size_t)(tile * plan.splits + min(s0 + u, plan.splits - 1)) * BW + row_in_tile) * tok_pad) + (c0 >> 2);
#pragma unroll
                                for (int j = 0; j < 4; ++j) part[u][j] = __ldcg(p + j);
                            }
#pragma unroll
                            for (int u = 0; u < 8; ++u) {
                                if (s0 + u < plan.splits) {
#pragma unroll
                                    for (int j = 0; j < 4; ++j) {
                                        acc[4 * j + 0] += part[u][j].x;
                                        acc[4 * j + 1] += part[u][j].y;
                                        acc[4 * j + 2] += part[u][j].z;
                                        acc[4 * j + 3] += part[u][j].w;
                                    }
                                }
                            }
                        }
                    }
                    if (swiglu) {
                        // rows in blocks of 16: 8 gate rows then their 8 up rows; lane + 8 holds the up value
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            const float up = __shfl_down_sync(0xffffffffu, acc[j], 8);
                            if ((lane & 15) < 8 && n + 8 < N && c0 + j < M) {
                                const float g = acc[j];
                                out[(size_t)(c0 + j) * ldo + (n >> 4) * 8 + (lane & 7)] =
                                    from_float<Tout>(__fdividef(g, 1.f + __expf(-g)) * up);
                            }
                        }
                    } else if (n < N) {
                        const float b = has_bias ? bias[n] : 0.f;
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            if (c0 + j < M) {
                                Tout* dst = out + (size_t)(c0 + j) * ldo + n;
                                float r = acc[j] + b;
                                if (accumulate) r += to_float(*dst);
                                *dst = from_float<Tout>(r);
                            }
                        }
                    }
                }
                if (plan.splits == 1) {
                    tcgen05_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(acc_empty_bar(buf));
                }
            }
        }
        if (!ok && lane == 0) { *abort_flag = 1; atomicExch(error_word, 13); }
    }
    pdl_trigger();
    tcgen05_fence_before();
    __syncthreads();
    if (warp == 2) {
        tcgen05_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(plan.tmem_cols) : "memory");
    }
}

Plan make_plan(int M, int N, int K, int sms) {
    Plan p;
    p.tiles = (N + BW - 1) / BW;
    p.k_blocks = (K + BK - 1) / BK;
    p.tok_pad = M <= 16 ? 16 : (M <= 32 ? 32 : (M <= 64 ? 64 : 128));
    p.stage_bytes = W_BYTES + p.tok_pad * BK * 2;
    p.stages = (int)((SMEM_LIMIT - 2048) / p.stage_bytes);
    if (p.stages > MAX_STAGES) p.stages = MAX_STAGES;
    // as many units as fit two rounds of the persistent grid without spilling into a third (a unit more than
    // that would leave most SMs idle for a whole unit), each slice at least 4 k blocks long
    int want = (2 * sms) / p.tiles;
    if (want >= 2 && (sms / p.tiles) * p.tiles * 1 >= sms * 3 / 4 && p.k_blocks / (sms / p.tiles) < 8) want = sms / p.tiles;
    int most = p.k_blocks / 4 > 0 ? p.k_blocks / 4 : 1;
    p.splits = want < 1 ? 1 : (want > most ? most : want);
    if (p.splits > 32) p.splits = 32;
    p.tmem_cols = 2 * p.tok_pad < 32 ? 32 : 2 * p.tok_pad;
    return p;
}

__device__ int g_skinny_error_word = 0;

int* skinny_error_word() {
    static int* words[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    if (!words[dev]) {
        void* p = nullptr;
        if (cudaGetSymbolAddress(&p, g_skinny_error_word) != cudaSuccess) return nullptr;
        words[dev] = static_cast<int*>(p);
    }
    return words[dev];
}

int sm_count() {
    static int sms = 0;
    if (!sms) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    }
    return sms;
}

}  // namespace

JLLM_EXPORT int jllm_gemm_skinny_fits(const void* a, int lda, const void* w, int ldw, int M, int N, int K) {
    return M >= 1 && M <= 128 && N >= 1 && (N + BW - 1) / BW <= MAX_TILES && K >= 8 && K % 8 == 0 && lda % 8 == 0 &&
           ldw % 8 == 0 && ((uintptr_t)a % 16) == 0 && ((uintptr_t)w % 16) == 0;
}

// Floats of workspace for this product: MAX_TILES counter words, then the split partials.
JLLM_EXPORT long long jllm_gemm_skinny_workspace_floats(int M, int N, int K) {
    const Plan p = make_plan(M, N, K, 148);
    return MAX_TILES + (p.splits > 1 ? (long long)p.tiles * p.splits * p.tok_pad * BW : 0);
}

JLLM_EXPORT int jllm_gemm_skinny_error() {
    int* word = skinny_error_word();
    if (!word) return -1;
    int v = 0;
    if (cudaMemcpy(&v, word, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
    if (v) cudaMemset(word, 0, sizeof(int));
    return v;
}

JLLM_EXPORT int jllm_gemm_skinny(const void* a, int lda, const void* w, int ldw, const void* bias, int bias_dtype,
                                 void* out, int out_dtype, int ldo, int accumulate, int M, int N, int K, int swiglu,
                                 float* workspace, long long workspace_floats, int force_splits, cudaStream_t stream) {
    JLLM_REQUIRE(jllm_gemm_skinny_fits(a, lda, w, ldw, M, N, K),
                 "gemm_skinny: needs 1 <= M <= 128, K %% 8 == 0 and 16-byte aligned rows (M=%d N=%d K=%d lda=%d ldw=%d)", M,
                 N, K, lda, ldw);
    JLLM_REQUIRE(ldo >= (swiglu ? N / 2 : N), "gemm_skinny: ldo=%d < N=%d", ldo, N);
    JLLM_REQUIRE(!swiglu || (N % 16 == 0 && !bias && !accumulate),
                 "gemm_skinny: the SwiGLU epilogue needs N %% 16 == 0, no bias and no accumulation (N=%d)", N);
    Plan plan = make_plan(M, N, K, sm_count());
    if (force_splits > 0) plan.splits = force_splits > plan.k_blocks ? plan.k_blocks : force_splits;
    const long long need = MAX_TILES + (plan.splits > 1 ? (long long)plan.tiles * plan.splits * plan.tok_pad * BW : 0);
    JLLM_REQUIRE(workspace != nullptr && workspace_floats >= need, "gemm_skinny: workspace of %lld floats, %lld needed",
                 workspace_floats, need);
    CUtensorMap map_w, map_a;
    int rc = tensor_map_for(w, N, K, ldw, BW, &map_w);
    if (rc != JLLM_OK) return rc;
    rc = tensor_map_for(a, M, K, lda, plan.tok_pad, &map_a);
    if (rc != JLLM_OK) return rc;
    int* error_word = skinny_error_word();
    if (!error_word) return jllm_fail(JLLM_CUDA_ERROR, "gemm_skinny: no error word");
    const int units = plan.tiles * plan.splits;
    const int grid = units < sm_count() ? units : sm_count();
    const size_t smem = (size_t)plan.stages * plan.stage_bytes + 1024 + 512;
    const VecRef b{bias, bias_dtype};
    int* counters = reinterpret_cast<int*>(workspace);
    float* partials = workspace + MAX_TILES;
    if (out_dtype == JLLM_F32) {
        auto kern = gemm_skinny_kernel<float>;
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        jllm_launch(kern, dim3(grid), dim3(THREADS), smem, stream, true, map_w, map_a, b, (int)(bias != nullptr),
                    (float*)out, ldo, accumulate, M, N, K, swiglu, plan, partials, counters, error_word);
    } else {
        auto kern = gemm_skinny_kernel<__nv_bfloat16>;
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        jllm_launch(kern, dim3(grid), dim3(THREADS), smem, stream, true, map_w, map_a, b, (int)(bias != nullptr),
                    (__nv_bfloat16*)out, ldo, accumulate, M, N, K, swiglu, plan, partials, counters, error_word);
    }
    return jllm_check_launch("gemm_skinny");
}
