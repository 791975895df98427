// out[m, n] (+)= sum_k a[m, k] * w[n, k] (+ bias[n]) on the 5th-generation tensor cores (tcgen05), bfloat16.
//
// The prefill product. A persistent kernel, one block per SM, walks 128 x BN output tiles (BN = 256 for big
// products, narrower when the rows are few):
//   * warp 0 (one lane) is the producer: for every 64-wide k block it waits for a free stage and brings a
//     128 x 64 tile of A (a tiled TMA copy into 128-byte-swizzled shared memory) and a BN x 64 tile of W, which
//     is kept PACKED in exactly that shared-memory image (ops.pack_weight), so its tile is one or two plain
//     contiguous bulk copies of up to 16 KB; all complete on the stage's "full" mbarrier (no multicast: every
//     block loads its own copy);
//   * warp 1 (one lane) issues the MMAs: 4 x tcgen05.mma (M 128, N 256, K 16) per k block, operands
//     described by shared-memory descriptors, the float32 accumulator in tensor memory (TMEM);
//     tcgen05.commit frees the stage, and after the last k block signals "accumulator full";
//   * warps 2-5 are the epilogue: each reads its 32 TMEM lanes (= 32 rows of the tile) with
//     tcgen05.ld, adds bias / the float32 residual, and stores float32 or bfloat16.
// TMEM holds two accumulators (2 x 256 columns), so the epilogue of one tile overlaps the main loop of
// the next. Tiles are visited with m fastest, so the blocks running together share W tiles in L2.
//
// Edges need no special code in the main loop: TMA fills out-of-range rows and k with zeros, and the
// epilogue stores only what lies inside [M, N]. Every mbarrier wait is bounded: if one runs out, the
// kernel raises an error word that the host reads, all roles leave their loops, and TMEM is freed.
//
// Requirements (else the caller uses another kernel): bfloat16, K a multiple of 8, row strides
// multiples of 8 elements, 16-byte aligned base pointers.
#include "gemm_epilogue.cuh"

namespace {

using namespace tc;

constexpr int BM = 128, BK = 64;
constexpr int A_BYTES = BM * BK * 2;
// The tile's width BN is a template parameter: 256 for the big products of a prefill; narrower tiles when the
// rows are few (more than the weight-stream kernel takes, at most a few hundred), so that every SM has a tile of
// the weight matrix to stream. Narrow tiles have small stages, so the ring is deeper.
__host__ __device__ constexpr int stages_for(int bn) { return bn >= 256 ? 4 : bn >= 192 ? 5 : bn >= 128 ? 6 : 8; }
constexpr int JLLM_TC_MAX_TILES = 65536;  // counter words at the head of the workspace of streamed products
constexpr int THREADS = 192;           // warp 0 TMA, warp 1 MMA, warps 2..5 epilogue
constexpr int TMEM_COLS = 512;
constexpr int STAGING_BYTES = 4 * STAGING_WARP_FLOATS * 4;   // a 32 x 32 block for each of the four epilogue warps
__host__ __device__ constexpr size_t smem_bytes_for(int bn) {
    return (size_t)stages_for(bn) * (A_BYTES + bn * BK * 2) + 1024 /* alignment slack */ + 256 /* barriers */ +
           STAGING_BYTES;
}

// Instruction descriptor of kind::f16: float32 accumulate (1 at [4,6)), A and B bfloat16 (1 at [7,10) and
// [10,13)), both K-major (0 at 15 and 16), N >> 3 at [17,23), M >> 4 at [24,29).
__host__ __device__ constexpr uint32_t idesc_for(int bn) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(bn >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
}

template <typename Tout, int BN>
__global__ void __launch_bounds__(THREADS, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_out, int bulk_out,
                    const __nv_bfloat16* __restrict__ w_packed, VecRef bias,
                    int has_bias, Tout* __restrict__ out, int ldo, int accumulate, int M, int N, int K, int swiglu,
                    int stream, float* __restrict__ partials, int* __restrict__ counters, int* __restrict__ error_word,
                    int starve) {
    // `starve` (a test of the bounded waits, never set otherwise): the first stage's barrier expects 16 bytes more than
    // the copies bring, so it never completes, and every wait gives up after 1,024 tries instead of 4 million.
    const uint32_t spin = starve ? 1024u : SPIN_LIMIT;
    constexpr int STAGES = stages_for(BN), B_BYTES = BN * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
    constexpr uint32_t IDESC = idesc_for(BN);
    static_assert(BN % 32 == 0 && BN >= 32 && BN <= 256, "tile width");
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;   // swizzled tiles want 1024-byte alignment
    uint8_t* aligned = smem_raw + (base - smem_u32(smem_raw));
    // the stages, the epilogue's staging (1024-byte aligned, as the stages are), the barriers
    const uint32_t bars = base + STAGES * STAGE_BYTES + STAGING_BYTES;
    // barriers: full[STAGES], empty[STAGES], acc_full[2], acc_empty[2]; then the TMEM base and the abort flag
    auto full_bar = [&](int s) { return bars + 8u * s; };
    auto empty_bar = [&](int s) { return bars + 8u * (STAGES + s); };
    auto acc_full_bar = [&](int b) { return bars + 8u * (2 * STAGES + b); };
    auto acc_empty_bar = [&](int b) { return bars + 8u * (2 * STAGES + 2 + b); };
    uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(aligned + STAGES * STAGE_BYTES + STAGING_BYTES + 8 * (2 * STAGES + 4));
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_base_slot + 1);
    volatile int* last_flag = reinterpret_cast<volatile int*>(tmem_base_slot + 2);
    uint8_t* staging = aligned + STAGES * STAGE_BYTES;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tiles_m = (M + BM - 1) / BM, tiles_n = (N + BN - 1) / BN, tiles = tiles_m * tiles_n;
    const int k_blocks = (K + BK - 1) / BK;
    const int padded_rows = (N + 127) & ~127;       // rows of the packed weight
    // The work of a block. Plain: whole tiles, tile = block, block + grid, ... Streamed (stream-K): only the full
    // rounds of tiles go that way; the tiles of the last, partly filled round are cut up instead: their (tile, k
    // block) pairs, in tile order, are dealt out as one equal run per block, and every block walks its run FIRST
    // and its whole tiles after it, so that no SM idles through a round and what the cutting costs (parked partial
    // tiles and their adding up, in the epilogue warps) lies under the main loops of the whole tiles that follow.
    // Of the blocks that hold k blocks of one tile, the one with the tile's FIRST k blocks finishes it: that part
    // is the last of its run, and the others' parts are the first of theirs, so they are parked by the time it
    // asks for them and nobody who is waited for waits himself. Blocks that run at the same time always work on
    // neighbouring tiles, which share their W and A tiles in L2. All three roles walk the same units with this.
    const int whole_tiles = stream ? tiles / (int)gridDim.x * (int)gridDim.x : tiles;
    const long long sk_kb = (long long)(tiles - whole_tiles) * k_blocks;     // streamed (tile, k block) pairs
    // (fewer pairs than blocks: the first `dealt` blocks take one each, so that no run between two others is empty)
    const long long dealt = min((long long)gridDim.x, max(sk_kb, 1LL));
    auto run_start = [&](long long c) { return sk_kb * min(c, dealt) / dealt; };
    const long long run_lo = run_start(blockIdx.x), run_hi = run_start(blockIdx.x + 1);
    struct Walk {
        long long at;
        int i;
    };
    auto first_unit = [&]() { return Walk{run_lo, 0}; };
    auto next_unit = [&](Walk& w, int& tile, int& lo, int& hi) {
        if (w.at < run_hi) {
            const int st = (int)(w.at / k_blocks);
            tile = whole_tiles + st;
            lo = (int)(w.at - (long long)st * k_blocks);
            hi = (int)min((long long)k_blocks, lo + (run_hi - w.at));
            w.at += hi - lo;
            return true;
        }
        const int t = blockIdx.x + w.i * gridDim.x;
        if (t >= whole_tiles) return false;
        tile = t;
        lo = 0;
        hi = k_blocks;
        ++w.i;
        return true;
    };

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(acc_full_bar(b), 1);
            mbar_init(acc_empty_bar(b), 4);   // one arrival per epilogue warp
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 2) {   // one warp allocates all 512 TMEM columns (one block per SM: nobody else wants any)
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_base_slot)),
                     "r"(TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_base_slot;
    pdl_wait();       // barriers and tensor memory were set up while the kernel before this one was finishing
    pdl_trigger();

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            // (stage and phase are counted, not divided out: with narrow tiles this one thread's instructions per
            // k block are what the product waits for)
            int s = 0;
            uint32_t parity = 1, dst = base;
            bool ok = true;
            Walk walk = first_unit();
            int tile, lo, hi;
            while (ok && next_unit(walk, tile, lo, hi)) {
                const int m0 = (tile % tiles_m) * BM, n0 = (tile / tiles_m) * BN;
                // The W tile: rows [n0, n0 + BN) of every k block, as one or two contiguous pieces of the packed layout
                // (a piece ends where a packed tile of 128 rows ends; a BN-row tile meets at most two of them). Rows
                // beyond the padded matrix do not exist: their part of a stage keeps what it held, and the columns they
                // would give are never stored. Everything that does not change with the k block is worked out here:
                // this one thread's instructions per k block are what a product of narrow tiles waits for.
                const int w_rows = min(BN, padded_rows - n0);
                const int in_tile = n0 & 127;
                const uint32_t bytes0 = (uint32_t)min(128 - in_tile, w_rows) * 128u;
                const uint32_t bytes1 = (uint32_t)w_rows * 128u - bytes0;
                const __nv_bfloat16* src = w_packed + ((size_t)(n0 >> 7) * k_blocks + lo) * 8192 + (size_t)in_tile * 64;
                const size_t next_tile = (size_t)k_blocks * 8192 - (size_t)in_tile * 64;      // to the tile below, row 0
                const uint32_t tx = A_BYTES + bytes0 + bytes1;
                uint32_t extra = starve ? 16u : 0u;         // the wait test: the first barrier expects too much
                for (int kb = lo; kb < hi; ++kb, src += 8192) {
                    if (!mbar_wait(empty_bar(s), parity, abort_flag, spin)) { ok = false; break; }
                    mbar_expect_tx(full_bar(s), tx + extra);
                    extra = 0;
                    tma_load_2d(dst, &map_a, kb * BK, m0, full_bar(s));
                    bulk_copy(dst + A_BYTES, src, bytes0, full_bar(s));
                    if (bytes1) bulk_copy(dst + A_BYTES + bytes0, src + next_tile, bytes1, full_bar(s));
                    dst += STAGE_BYTES;
                    if (++s == STAGES) { s = 0; parity ^= 1u; dst = base; }
                }
            }
            if (!ok) { *abort_flag = 1; atomicExch(error_word, 1); }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            uint32_t local_tile = 0, parity = 0, a_addr = base;
            int s = 0;
            bool ok = true;
            Walk walk = first_unit();
            int tile, lo, hi;
            for (; ok && next_unit(walk, tile, lo, hi); ++local_tile) {
                const uint32_t buf = local_tile & 1u;
                if (!mbar_wait(acc_empty_bar(buf), ((local_tile >> 1) & 1u) ^ 1u, abort_flag, spin)) { ok = false; break; }
                tcgen05_fence_after();
                const uint32_t tmem_d = tmem_base + buf * BN;
                for (int kb = lo; kb < hi; ++kb) {
                    if (!mbar_wait(full_bar(s), parity, abort_flag, spin)) { ok = false; break; }
                    tcgen05_fence_after();
                    const uint32_t b_addr = a_addr + A_BYTES;
#pragma unroll
                    for (int k = 0; k < BK / 16; ++k) {
                        // 16 bfloat16 = 32 bytes further along k inside the 128-byte swizzled rows
                        tcgen05_mma_bf16(tmem_d, smem_desc_sw128(a_addr + k * 32), smem_desc_sw128(b_addr + k * 32), IDESC,
                                         (kb > lo || k > 0) ? 1u : 0u);
                    }
                    tcgen05_commit(empty_bar(s));   // arrives when the MMAs above have read the stage
                    a_addr += STAGE_BYTES;
                    if (++s == STAGES) { s = 0; parity ^= 1u; a_addr = base; }
                }
                if (ok) tcgen05_commit(acc_full_bar(buf));
            }
            if (!ok) { *abort_flag = 1; atomicExch(error_word, 2); }
        }
    } else {
        // ---------------- epilogue: warps 2..5, TMEM lanes 32 * (warp % 4) ----------------
        const int quad = warp & 3;
        const TileEpilogue<Tout> ep{out, ldo, M, N, accumulate, has_bias, swiglu, bias, bulk_out ? &map_out : nullptr};
        uint32_t local_tile = 0;
        bool ok = true;
        Walk walk = first_unit();
        int tile, k_lo, k_hi;
        for (; ok && next_unit(walk, tile, k_lo, k_hi); ++local_tile) {
            const int m0 = (tile % tiles_m) * BM, n0 = (tile / tiles_m) * BN;
            const uint32_t buf = local_tile & 1u;
            if (!mbar_wait(acc_full_bar(buf), (local_tile >> 1) & 1u, abort_flag, spin)) { ok = false; break; }
            tcgen05_fence_after();
            const uint32_t taddr = tmem_base + buf * BN + ((uint32_t)(quad * 32) << 16);
            // bias / residual / SwiGLU and the store of 32 columns of this thread's row
            const int row0 = m0 + quad * 32;
            const bool whole = ep.rows_whole(row0);
            float* my_staging = reinterpret_cast<float*>(staging + quad * (bulk_out ? BULK_WARP_BYTES : STAGING_WARP_FLOATS * 4));
            auto finalize = [&](uint32_t (&v)[32], int c0) { ep.store(v, row0, lane, n0 + c0, whole, my_staging); };
            if (k_lo == 0 && k_hi == k_blocks) {      // the whole tile is this block's
#pragma unroll 1
                for (int c0 = 0; c0 < BN; c0 += 32) {
                    uint32_t v[32];
                    tmem_ld_32x32b_x32(taddr + c0, v);
                    tmem_ld_wait();
                    finalize(v, c0);
                }
                tcgen05_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(acc_empty_bar(buf));
                continue;
            }
            // ---- the tile's k blocks are spread over several (consecutive) blocks ----
            if (k_lo > 0) {
                // Not the tile's first k blocks: this is the first unit of the block's run. Park the part ([block][BN
                // columns][128 rows]: a warp's 32 rows of one column are 128 contiguous bytes) and count it in.
                float* mine = partials + (size_t)blockIdx.x * BM * BN + quad * 32 + lane;
#pragma unroll 1
                for (int c0 = 0; c0 < BN; c0 += 32) {
                    uint32_t v[32];
                    tmem_ld_32x32b_x32(taddr + c0, v);
                    tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < 32; ++j) __stcg(mine + (size_t)(c0 + j) * BM, __uint_as_float(v[j]));
                }
                tcgen05_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(acc_empty_bar(buf));
                asm volatile("bar.sync 1, 128;" ::: "memory");           // the four epilogue warps have written
                if (warp == 2 && lane == 0) {
                    __threadfence();
                    atomicAdd(&counters[tile], 1);
                }
                continue;
            }
            // The tile's first k blocks, the last unit of this block's run: wait (bounded) until the blocks after this
            // one have parked theirs, add them to the accumulator in k order (so the sum does not depend on who was
            // when) and finish the tile. All blocks of the grid are resident, one per SM.
            const long long tile_last_kb = (long long)(tile - whole_tiles + 1) * k_blocks - 1;
            const int others = (int)(((tile_last_kb + 1) * dealt + sk_kb - 1) / sk_kb - 1) - (int)blockIdx.x;
            if (warp == 2 && lane == 0) {
                int seen = 0;
                for (uint32_t tries = 0; seen < others && tries < spin; ++tries) {
                    asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(seen) : "l"(counters + tile) : "memory");
                    if (seen < others) {
                        if ((tries & 255u) == 255u && *abort_flag) break;
                        __nanosleep(32);
                    }
                }
                if (seen >= others) counters[tile] = 0;               // back to zero for the next product
                *last_flag = seen >= others;
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");
            if (!*last_flag) { ok = false; break; }
            const float* theirs = partials + (size_t)(blockIdx.x + 1) * BM * BN + quad * 32 + lane;
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += 32) {
                uint32_t v[32];
                tmem_ld_32x32b_x32(taddr + c0, v);
                float x[32];
#pragma unroll
                for (int j = 0; j < 32; ++j) x[j] = __ldcg(theirs + (size_t)(c0 + j) * BM);
                tmem_ld_wait();
                for (int p = 1;; ++p) {
#pragma unroll
                    for (int j = 0; j < 32; ++j) v[j] = __float_as_uint(__uint_as_float(v[j]) + x[j]);
                    if (p >= others) break;
#pragma unroll
                    for (int j = 0; j < 32; ++j) x[j] = __ldcg(theirs + (size_t)p * BM * BN + (size_t)(c0 + j) * BM);
                }
                finalize(v, c0);
            }
            tcgen05_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(acc_empty_bar(buf));
        }
        ep.bulk_done(lane);
        if (!ok && lane == 0) { *abort_flag = 1; atomicExch(error_word, 3); }
    }
    tcgen05_fence_before();
    __syncthreads();
    if (warp == 2) {
        tcgen05_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

// ---- host side: tensor maps (cached) and the launch ---------------------------------------------------------

// The error word lives in device memory that belongs to the library (no allocation): its address is looked
// up once per device.
__device__ int g_gemm_error_word = 0;

int* error_word_for_device() {
    static int* words[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    if (!words[dev]) {
        void* p = nullptr;
        if (cudaGetSymbolAddress(&p, g_gemm_error_word) != cudaSuccess) return nullptr;
        words[dev] = static_cast<int*>(p);
    }
    return words[dev];
}

}  // namespace

int* jllm_gemm_error_word() { return error_word_for_device(); }      // shared with the weight-stream product

JLLM_EXPORT int jllm_gemm_tcgen05_fits(const void* a, int lda, const void* w_packed, int M, int N, int K) {
    return M >= 1 && N >= 1 && K >= 8 && K % 8 == 0 && lda % 8 == 0 && ((uintptr_t)a % 16) == 0 &&
           ((uintptr_t)w_packed % 16) == 0;
}

// Reads and clears the error word that a kernel whose wait ran out has raised (0 = none). Synchronises the device.
JLLM_EXPORT int jllm_gemm_tcgen05_error() {
    int* word = error_word_for_device();
    if (!word) return -1;
    int v = 0;
    if (cudaMemcpy(&v, word, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
    if (v) cudaMemset(word, 0, sizeof(int));
    return v;
}

// A test of the bounded waits: the NEXT product launched through jllm_gemm_tcgen05 by this thread starves (its first
// barrier expects more bytes than arrive and its waits give up after 1,024 tries): it must return, raise the error
// word and leave the device usable. The test keeps that product to a single tile.
namespace {
thread_local int g_starve_next = 0;
}
JLLM_EXPORT void jllm_gemm_tcgen05_starve_next() { g_starve_next = 1; }

// A test's switch: float32 outputs are stored (and added into) by the epilogue warps' own loads and stores, as where
// the output's rows allow no tensor map, instead of by bulk copies. For the paired product too.
int g_plain_stores = 0;
JLLM_EXPORT void jllm_gemm_plain_stores(int on) { g_plain_stores = on; }

// w: ops.pack_weight of the [N, K] weight (k_blocks_packed = ceil(K / 64) its k blocks).
JLLM_EXPORT int jllm_gemm_tcgen05(const void* a, int lda, const void* w, int k_blocks_packed, const void* bias, int bias_dtype,
                                  void* out, int out_dtype, int ldo, int accumulate, int M, int N, int K, int max_blocks,
                                  int swiglu, float* workspace, long long workspace_floats, int stream_mode,
                                  int tile_width, cudaStream_t stream) {
    JLLM_REQUIRE(jllm_gemm_tcgen05_fits(a, lda, w, M, N, K),
                 "gemm_tcgen05: needs K %% 8 == 0 and 16-byte aligned rows (M=%d N=%d K=%d lda=%d)", M, N, K, lda);
    JLLM_REQUIRE(k_blocks_packed == (K + BK - 1) / BK, "gemm_tcgen05: the packed weight has %d k blocks, K=%d needs %d",
                 k_blocks_packed, K, (K + BK - 1) / BK);
    JLLM_REQUIRE(ldo >= (swiglu ? N / 2 : N), "gemm_tcgen05: ldo=%d < N=%d", ldo, N);
    JLLM_REQUIRE(!swiglu || (N % 16 == 0 && !bias && !accumulate),
                 "gemm_tcgen05: the SwiGLU epilogue needs N %% 16 == 0, no bias and no accumulation (N=%d)", N);
    const int sms = jllm_device_sm_count() > 0 ? jllm_device_sm_count() : 1;
    // The tile width: a block's time for a tile grows with the bytes it pulls in (its rows of A and BN rows of W
    // per k block), and the product takes as many rounds as the tiles need on the SMs there are.
    const int widths[5] = {256, 192, 128, 64, 32};
    const int tiles_m = (M + BM - 1) / BM, rows_per_tile = M < BM ? M : BM;
    int BN = 256;
    long long best = -1;
    for (int i = 0; i < 5; ++i) {
        const long long t = (long long)tiles_m * ((N + widths[i] - 1) / widths[i]);
        const long long cost = ((t + sms - 1) / sms) * (rows_per_tile + widths[i]);
        if (best < 0 || cost < best) { best = cost; BN = widths[i]; }
    }
    bool streamed = false;
    if (tile_width > 0) BN = tile_width;
    JLLM_REQUIRE(BN == 256 || BN == 192 || BN == 128 || BN == 64 || BN == 32, "gemm_tcgen05: tile width %d", BN);
    CUtensorMap map_a;
    int rc = tensor_map_for(a, M, K, lda, BM, &map_a);
    if (rc != JLLM_OK) return rc;
    // a float32 output leaves by tiled bulk copies (the residual add as a reduce in L2) where its rows allow a tensor map
    CUtensorMap map_out = {};
    const int bulk_out = out_dtype == JLLM_F32 && !swiglu && ldo % 4 == 0 && ((uintptr_t)out % 16) == 0 && !g_plain_stores;
    if (bulk_out) {
        rc = tensor_map_out_f32(out, M, N, ldo, &map_out);
        if (rc != JLLM_OK) return rc;
    }
    int* error_word = error_word_for_device();
    if (!error_word) return jllm_fail(JLLM_CUDA_ERROR, "gemm_tcgen05: no error word");
    const int tiles = tiles_m * ((N + BN - 1) / BN);
    const int k_blocks = (K + BK - 1) / BK;
    // stream_mode 1: the tiles of a last, partly filled round are streamed (stream-K), and fewer tiles than SMs are cut
    // up too. Not the default: on the layer shapes of an 8B model with 2,048 rows the SMs that the last round leaves
    // idle cost little (the busy ones run the faster for it: the products are bound by what the memory system and the
    // power limit give all SMs together), and the parked partial tiles cost about as much (QKV 81 us streamed, 82
    // plain; O 63 / 60; gate_up 318 / 289; down 184 / 191). The workspace of a streamed product holds one counter per
    // tile (zero before the first product, left zero by every product) and one parked partial tile per block.
    int grid = tiles < sms ? tiles : sms;
    if (stream_mode == 1) {
        const long long all_kb = (long long)tiles * k_blocks;
        grid = all_kb < sms ? (int)all_kb : sms;
    }
    if (max_blocks > 0 && grid > max_blocks) grid = max_blocks;
    const long long need = JLLM_TC_MAX_TILES + (long long)grid * BM * BN;
    if (stream_mode == 1) {
        const bool room = workspace != nullptr && workspace_floats >= need && tiles <= JLLM_TC_MAX_TILES;
        JLLM_REQUIRE(room, "gemm_tcgen05: a streamed product of %d tiles on %d blocks needs a workspace of %lld floats "
                           "(got %lld) and at most %d tiles", tiles, grid, need, workspace_floats, JLLM_TC_MAX_TILES);
        streamed = true;
    }
    int* counters = reinterpret_cast<int*>(workspace);
    float* partials = workspace ? workspace + JLLM_TC_MAX_TILES : nullptr;
    const int splits = streamed ? 1 : 0;      // the kernel's `stream` argument
    const int starve = g_starve_next;
    g_starve_next = 0;
    JLLM_REQUIRE(!starve || (tiles == 1 && k_blocks <= 2), "gemm_tcgen05: the starved product of the wait test is one "
                 "tile of at most two k blocks (got %d tiles, %d k blocks)", tiles, k_blocks);
    const VecRef b{bias, bias_dtype};
#define JLLM_TC_GO(T, W)                                                                                              \
    do {                                                                                                              \
        auto kern = gemm_tcgen05_kernel<T, W>;                                                                        \
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_bytes_for(W));             \
        jllm_launch(kern, dim3(grid), dim3(THREADS), smem_bytes_for(W), stream, true, map_a, map_out, bulk_out,        \
                    (const __nv_bfloat16*)w, b,                                                                      \
                    (int)(bias != nullptr), (T*)out, ldo, accumulate, M, N, K, swiglu, splits, partials, counters,    \
                    error_word, starve);                                                                              \
    } while (0)
#define JLLM_TC_WIDTHS(T)                                                                                             \
    switch (BN) {                                                                                                     \
        case 256: JLLM_TC_GO(T, 256); break;                                                                          \
        case 192: JLLM_TC_GO(T, 192); break;                                                                          \
        case 128: JLLM_TC_GO(T, 128); break;                                                                          \
        case 64: JLLM_TC_GO(T, 64); break;                                                                            \
        default: JLLM_TC_GO(T, 32); break;                                                                            \
    }
    if (out_dtype == JLLM_F32) {
        JLLM_TC_WIDTHS(float)
    } else {
        JLLM_TC_WIDTHS(__nv_bfloat16)
    }
#undef JLLM_TC_WIDTHS
#undef JLLM_TC_GO
    return jllm_check_launch("gemm_tcgen05");
}
