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
#include "tcgen05_common.cuh"

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
constexpr int STAGING_ROW = 36;        // floats of a staged row of 32 values: 16-byte aligned, and rows fall in other banks
constexpr int STAGING_BYTES = 4 * 32 * STAGING_ROW * 4;      // 32 rows for each of the four epilogue warps
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
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a, const __nv_bfloat16* __restrict__ w_packed, VecRef bias,
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
    const uint32_t bars = base + STAGES * STAGE_BYTES;
    // barriers: full[STAGES], empty[STAGES], acc_full[2], acc_empty[2]; then the TMEM base and the abort flag
    auto full_bar = [&](int s) { return bars + 8u * s; };
    auto empty_bar = [&](int s) { return bars + 8u * (STAGES + s); };
    auto acc_full_bar = [&](int b) { return bars + 8u * (2 * STAGES + b); };
    auto acc_empty_bar = [&](int b) { return bars + 8u * (2 * STAGES + 2 + b); };
    uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(aligned + STAGES * STAGE_BYTES + 8 * (2 * STAGES + 4));
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_base_slot + 1);
    volatile int* last_flag = reinterpret_cast<volatile int*>(tmem_base_slot + 2);
    float* staging = reinterpret_cast<float*>(aligned + STAGES * STAGE_BYTES + 256);     // behind the barriers

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tiles_m = (M + BM - 1) / BM, tiles_n = (N + BN - 1) / BN, tiles = tiles_m * tiles_n;
    const int k_blocks = (K + BK - 1) / BK;
    const int padded_rows = (N + 127) & ~127;       // rows of the packed weight
    // The work of a block: whole tiles, tile = block, block + grid, ... as long as full rounds of tiles last. The
    // tiles of a last, partly filled round are streamed instead (stream-K): their (tile, k block) pairs, in tile
    // order, are cut into one equal run per block, so that no SM idles through that round; a tile whose k blocks
    // lie in several blocks' runs is finished by whichever of them comes last (below). Blocks that run at the
    // same time always work on neighbouring tiles, which share their W and A tiles in L2. All three roles walk
    // the same units with this.
    const int whole_tiles = stream ? tiles / (int)gridDim.x * (int)gridDim.x : tiles;
    const long long sk_kb = (long long)(tiles - whole_tiles) * k_blocks;     // streamed (tile, k block) pairs
    const long long run_lo = sk_kb * blockIdx.x / gridDim.x, run_hi = sk_kb * (blockIdx.x + 1) / gridDim.x;
    struct Walk {
        long long at;
        int i;
    };
    auto first_unit = [&]() { return Walk{run_lo, 0}; };
    auto next_unit = [&](Walk& w, int& tile, int& lo, int& hi) {
        const int t = blockIdx.x + w.i * gridDim.x;
        if (t < whole_tiles) {
            tile = t;
            lo = 0;
            hi = k_blocks;
            ++w.i;
            return true;
        }
        if (w.at >= run_hi) return false;
        const int st = (int)(w.at / k_blocks);
        tile = whole_tiles + st;
        lo = (int)(w.at - (long long)st * k_blocks);
        hi = (int)min((long long)k_blocks, lo + (run_hi - w.at));
        w.at += hi - lo;
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
        uint32_t local_tile = 0;
        bool ok = true;
        Walk walk = first_unit();
        int tile, k_lo, k_hi;
        for (; ok && next_unit(walk, tile, k_lo, k_hi); ++local_tile) {
            const int m0 = (tile % tiles_m) * BM, n0 = (tile / tiles_m) * BN;
            const uint32_t buf = local_tile & 1u;
            if (!mbar_wait(acc_full_bar(buf), (local_tile >> 1) & 1u, abort_flag, spin)) { ok = false; break; }
            tcgen05_fence_after();
            const int row = m0 + quad * 32 + lane;
            const uint32_t taddr = tmem_base + buf * BN + ((uint32_t)(quad * 32) << 16);
            // bias / residual / SwiGLU and the store of 32 columns of this thread's row
            // all 32 rows of this warp lie inside the matrix, and float32 rows can be accessed 16 bytes at a time
            const bool rows_whole = !swiglu && m0 + quad * 32 + 32 <= M && sizeof(Tout) == 4 && (ldo & 3) == 0 &&
                                    (((uintptr_t)out) & 15u) == 0;
            // Through shared memory, so that a warp's accesses are whole lines: a thread holds 32 values of ONE row, and
            // written (or added) from there a warp's instruction would touch 32 rows with 16 bytes each. The warp parks
            // its 32 x 32 block and takes it back four rows at a time, eight threads to a row: four full 128-byte lines
            // per instruction, and all eight loads of a residual add are on their way before the first store.
            auto staged_rows = [&](uint32_t (&v)[32], int c0) {
                const int n_base = n0 + c0;
                float* mine = staging + quad * (32 * STAGING_ROW);
                float4* srow = reinterpret_cast<float4*>(mine + lane * STAGING_ROW);
#pragma unroll
                for (int j = 0; j < 8; ++j)
                    srow[j] = make_float4(__uint_as_float(v[4 * j]), __uint_as_float(v[4 * j + 1]),
                                          __uint_as_float(v[4 * j + 2]), __uint_as_float(v[4 * j + 3]));
                __syncwarp();
                const int sub = lane >> 3, c4 = (lane & 7) * 4;
                float4 bv = make_float4(0.f, 0.f, 0.f, 0.f);
                if (has_bias)
                    bv = make_float4(bias[n_base + c4], bias[n_base + c4 + 1], bias[n_base + c4 + 2], bias[n_base + c4 + 3]);
                float* d0 = reinterpret_cast<float*>(out) + (size_t)(m0 + quad * 32 + sub) * ldo + n_base + c4;
                float4 old[8];
                if (accumulate) {
#pragma unroll
                    for (int p = 0; p < 8; ++p) old[p] = *reinterpret_cast<const float4*>(d0 + (size_t)(4 * p) * ldo);
                }
#pragma unroll
                for (int p = 0; p < 8; ++p) {
                    float4 x = *reinterpret_cast<const float4*>(mine + (4 * p + sub) * STAGING_ROW + c4);
                    x.x += bv.x; x.y += bv.y; x.z += bv.z; x.w += bv.w;
                    if (accumulate) { x.x += old[p].x; x.y += old[p].y; x.z += old[p].z; x.w += old[p].w; }
                    *reinterpret_cast<float4*>(d0 + (size_t)(4 * p) * ldo) = x;
                }
                __syncwarp();
            };
            auto finalize = [&](uint32_t (&v)[32], int c0) {
                if (rows_whole && n0 + c0 + 32 <= N) {
                    staged_rows(v, c0);
                } else if (row < M && swiglu) {
                    // columns come in blocks of 16: 8 gate columns, then the 8 up columns of the same hidden units
                    const int n_base = n0 + c0;
                    Tout* dst = out + (size_t)row * ldo + (n_base >> 1);
                    // (the tensor-core path may use the fast exponential: its result is rounded to bfloat16 anyway)
                    float hv[16];
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const int cg = (j >> 3) * 16 + (j & 7);
                        const float gt = __uint_as_float(v[cg]), up = __uint_as_float(v[cg + 8]);
                        hv[j] = __fdividef(gt, 1.f + __expf(-gt)) * up;
                    }
                    if (sizeof(Tout) == 2 && n_base + 32 <= N && ((((uintptr_t)dst) & 15u) == 0)) {
                        uint32_t p[8];
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            __nv_bfloat162 b2 = __floats2bfloat162_rn(hv[2 * j], hv[2 * j + 1]);
                            p[j] = *reinterpret_cast<uint32_t*>(&b2);
                        }
                        reinterpret_cast<uint4*>(dst)[0] = make_uint4(p[0], p[1], p[2], p[3]);
                        reinterpret_cast<uint4*>(dst)[1] = make_uint4(p[4], p[5], p[6], p[7]);
                    } else {
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            const int cg = (j >> 3) * 16 + (j & 7);
                            if (n_base + cg + 8 < N) dst[j] = from_float<Tout>(hv[j]);
                        }
                    }
                } else if (row < M) {
                    const int n_base = n0 + c0;
                    Tout* dst = out + (size_t)row * ldo + n_base;
                    if (n_base + 32 <= N) {
                        if constexpr (sizeof(Tout) == 4) {
                            float4* d4 = reinterpret_cast<float4*>(dst);
                            const bool vec = (((uintptr_t)dst) & 15u) == 0;
#pragma unroll
                            for (int j = 0; j < 8; ++j) {
                                float4 r;
                                r.x = __uint_as_float(v[4 * j + 0]);
                                r.y = __uint_as_float(v[4 * j + 1]);
                                r.z = __uint_as_float(v[4 * j + 2]);
                                r.w = __uint_as_float(v[4 * j + 3]);
                                if (has_bias) {
                                    r.x += bias[n_base + 4 * j + 0];
                                    r.y += bias[n_base + 4 * j + 1];
                                    r.z += bias[n_base + 4 * j + 2];
                                    r.w += bias[n_base + 4 * j + 3];
                                }
                                if (vec) {
                                    if (accumulate) {
                                        const float4 o = d4[j];
                                        r.x += o.x; r.y += o.y; r.z += o.z; r.w += o.w;
                                    }
                                    d4[j] = r;
                                } else {
                                    float* d = reinterpret_cast<float*>(dst) + 4 * j;
                                    if (accumulate) { r.x += d[0]; r.y += d[1]; r.z += d[2]; r.w += d[3]; }
                                    d[0] = r.x; d[1] = r.y; d[2] = r.z; d[3] = r.w;
                                }
                            }
                        } else {
                            const bool vec = (((uintptr_t)dst) & 15u) == 0;
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                uint32_t p[4];
#pragma unroll
                                for (int e = 0; e < 4; ++e) {
                                    float lo = __uint_as_float(v[8 * j + 2 * e]), hi = __uint_as_float(v[8 * j + 2 * e + 1]);
                                    if (has_bias) { lo += bias[n_base + 8 * j + 2 * e]; hi += bias[n_base + 8 * j + 2 * e + 1]; }
                                    if (accumulate) { lo += to_float(dst[8 * j + 2 * e]); hi += to_float(dst[8 * j + 2 * e + 1]); }
                                    __nv_bfloat162 b2 = __floats2bfloat162_rn(lo, hi);
                                    p[e] = *reinterpret_cast<uint32_t*>(&b2);
                                }
                                if (vec) {
                                    reinterpret_cast<uint4*>(dst)[j] = make_uint4(p[0], p[1], p[2], p[3]);
                                } else {
#pragma unroll
                                    for (int e = 0; e < 4; ++e) {
                                        __nv_bfloat162 b2 = *reinterpret_cast<__nv_bfloat162*>(&p[e]);
                                        dst[8 * j + 2 * e] = b2.x;
                                        dst[8 * j + 2 * e + 1] = b2.y;
                                    }
                                }
                            }
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; ++j) {
                            if (n_base + j < N) {
                                float r = __uint_as_float(v[j]);
                                if (has_bias) r += bias[n_base + j];
                                if (accumulate) r += to_float(dst[j]);
                                dst[j] = from_float<Tout>(r);
                            }
                        }
                    }
                }
            };
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
            // ---- the tile's k blocks are spread over several blocks: park this part ([block][first or later unit
            // of the block][BN columns][128 rows]: a warp's 32 rows of one column are 128 contiguous bytes); the
            // blocks that hold parts of the tile are consecutive ----
            auto run_start = [&](long long c) { return sk_kb * c / gridDim.x; };
            auto block_of = [&](long long kb_index) {   // the block whose run holds this streamed (tile, k block) pair
                return (int)(((kb_index + 1) * gridDim.x + sk_kb - 1) / sk_kb - 1);
            };
            const long long tile_kb0 = (long long)(tile - whole_tiles) * k_blocks;
            const int c_first = block_of(tile_kb0), parts = block_of(tile_kb0 + k_blocks - 1) - c_first + 1;
            auto part_of = [&](int c) {                 // where block c parked its part of this tile
                const int slot = run_start(c) >= tile_kb0 ? 0 : 1;
                return partials + (size_t)(2 * c + slot) * BM * BN + quad * 32 + lane;
            };
            float* mine = part_of(blockIdx.x);
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
                const int seen = atomicAdd(&counters[tile], 1);
                *last_flag = seen == parts - 1;
                if (seen == parts - 1) {
                    counters[tile] = 0;                               // back to zero for the next product
                    __threadfence();
                }
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");
            if (*last_flag == 0) continue;
            // ---- the block that came last adds the parts in k order (deterministic) and finishes the tile ----
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += 32) {
                float acc[32];
#pragma unroll
                for (int j = 0; j < 32; ++j) acc[j] = 0.f;
                for (int s0 = 0; s0 < parts; s0 += 2) {     // two parts' loads in flight at a time, added in k order
                    const float* p0 = part_of(c_first + s0) + (size_t)c0 * BM;
                    const float* p1 = part_of(c_first + min(s0 + 1, parts - 1)) + (size_t)c0 * BM;
                    float x0[32], x1[32];
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        x0[j] = __ldcg(p0 + (size_t)j * BM);
                        x1[j] = __ldcg(p1 + (size_t)j * BM);
                    }
                    const bool two = s0 + 1 < parts;
#pragma unroll
                    for (int j = 0; j < 32; ++j) acc[j] = two ? (acc[j] + x0[j]) + x1[j] : acc[j] + x0[j];
                }
                uint32_t v[32];
#pragma unroll
                for (int j = 0; j < 32; ++j) v[j] = __float_as_uint(acc[j]);
                finalize(v, c0);
            }
        }
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
    // The tiles of a last, partly filled round can be streamed (stream-K, stream_mode 1). It is not done by default:
    // on the layer shapes of an 8B model with 2,048 rows the parked partial tiles and their adding up cost what the
    // idle SMs of the last round cost (QKV 92 us streamed, 81 us plain; gate_up 307 / 291; down 207 / 178).
    bool streamed = false;
    if (tile_width > 0) BN = tile_width;
    JLLM_REQUIRE(BN == 256 || BN == 192 || BN == 128 || BN == 64 || BN == 32, "gemm_tcgen05: tile width %d", BN);
    CUtensorMap map_a;
    int rc = tensor_map_for(a, M, K, lda, BM, &map_a);
    if (rc != JLLM_OK) return rc;
    int* error_word = error_word_for_device();
    if (!error_word) return jllm_fail(JLLM_CUDA_ERROR, "gemm_tcgen05: no error word");
    const int tiles = tiles_m * ((N + BN - 1) / BN);
    const int k_blocks = (K + BK - 1) / BK;
    // stream_mode: 1 = streamed, else plain. The workspace of a streamed product holds one counter per tile (zero
    // before the first product, left zero by every product) and two parked partial tiles per block.
    int grid = tiles < sms ? tiles : sms;
    if (stream_mode > 0) {
        streamed = true;
        const long long all_kb = (long long)tiles * k_blocks;
        grid = all_kb < sms ? (int)all_kb : sms;
    }
    if (max_blocks > 0 && grid > max_blocks) grid = max_blocks;
    const long long need = JLLM_TC_MAX_TILES + (long long)grid * 2 * BM * BN;
    const bool room = workspace != nullptr && workspace_floats >= need && tiles <= JLLM_TC_MAX_TILES;
    if (streamed)
        JLLM_REQUIRE(room, "gemm_tcgen05: a streamed product of %d tiles on %d blocks needs a workspace of %lld floats "
                           "(got %lld) and at most %d tiles", tiles, grid, need, workspace_floats, JLLM_TC_MAX_TILES);
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
        jllm_launch(kern, dim3(grid), dim3(THREADS), smem_bytes_for(W), stream, true, map_a, (const __nv_bfloat16*)w, b, \
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
