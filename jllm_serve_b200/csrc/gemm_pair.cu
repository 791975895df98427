// out[m, n] (+)= sum_k a[m, k] * w[n, k] (+ bias[n]) on the 5th-generation tensor cores, two SMs to a tile
// (tcgen05 cta_group::2), bfloat16. The product of a prefill with many rows.
//
// What bounds the one-SM product (gemm_tcgen05.cu) on big shapes is what an SM can take in: 48 KB per k block (128
// rows of A, 256 rows of W) for 128 x 256 x 64 multiply-adds. Here two blocks, a cluster of two on neighbouring SMs,
// share a 256 x 256 tile: each brings 128 rows of A and 128 of the tile's 256 rows of W (32 KB per k block for the
// same multiply-adds), one thread of the pair's first block issues MMAs of M 256 that read both blocks' shared memory,
// and each block ends up with its 128 rows of the tile in its own tensor memory.
//
//   * warp 0 (one lane) of BOTH blocks is a producer: it waits for its free stage and brings its A tile (tiled TMA
//     copy, 128-byte swizzle) and its W tile (the PACKED weight is that shared-memory image already: a tiled copy
//     without swizzle of its 16 KB). Every copy completes on the FIRST block's "full" barrier of the stage, which
//     expects the bytes of both blocks;
//   * warp 1 (one lane) of the first block issues 4 x tcgen05.mma.cta_group::2 (M 256, N 256, K 16) per k block;
//     tcgen05.commit, multicast to both blocks, frees the stage in both and, after a tile's last k block, tells both
//     blocks' epilogues that the accumulator is full;
//   * warps 2-5 of both blocks are the epilogue of their block's 128 rows (gemm_epilogue.cuh); when a block's four
//     warps have read an accumulator they tell the first block, whose MMA thread may then use it again.
// Tensor memory holds two accumulators, so a tile's epilogue overlaps the next tile's main loop. The pairs walk the
// tiles with m fastest. Edges: TMA fills rows beyond M and k beyond K with zeros; a block whose half of the W rows lies
// beyond the (padded) matrix brings none, and its columns are never stored.
//
// Every wait is bounded: if one runs out, the kernel raises the error word that the host reads, tells its partner,
// all roles leave their loops, both blocks meet at the cluster's barrier and tensor memory is freed.
#include <mutex>
#include <unordered_map>

#include "gemm_epilogue.cuh"

namespace {

using namespace tc;

constexpr int BM = 128, PAIR_M = 256, BN = 256, BK = 64;
constexpr int A_BYTES = BM * BK * 2, W_BYTES = 128 * BK * 2, STAGE_BYTES = A_BYTES + W_BYTES;
constexpr int STAGES = 6;
constexpr int THREADS = 192;           // warp 0 producer, warp 1 MMA (first block), warps 2..5 epilogue
constexpr int TMEM_COLS = 512;
constexpr int PAIR_MAX_TILES = 65536;   // two counter words per tile at the head of the workspace of streamed products
constexpr int STAGING_BYTES = 4 * STAGING_WARP_FLOATS * 4;
constexpr size_t SMEM_BYTES = (size_t)STAGES * STAGE_BYTES + 1024 /* alignment slack */ + 256 /* barriers */ + STAGING_BYTES;

// kind::f16: float32 accumulate, A and B bfloat16, both K-major, N >> 3 at [17,23), M >> 4 at [24,29): M is the pair's 256
constexpr uint32_t IDESC = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(PAIR_M >> 4) << 24);

__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// the address, in the cluster's shared window, of `addr` (an address in this block's shared memory) in block `rank`
__device__ __forceinline__ uint32_t in_block(uint32_t addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void store_cluster(uint32_t cluster_addr, int v) {
    asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(cluster_addr), "r"(v) : "memory");
}
// a tiled copy into THIS block's shared memory that completes on a barrier that may be the partner's
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t cluster_bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(cluster_bar)
        : "memory");
}
__device__ __forceinline__ void mma_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}
// arrives, when the MMAs issued so far are done, on the barrier at this offset in both blocks of the pair
__device__ __forceinline__ void commit_pair(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(bar), "h"((uint16_t)3)
                 : "memory");
}

template <typename Tout>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(THREADS, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                 const __grid_constant__ CUtensorMap map_out, int bulk_out, VecRef bias,
                 int has_bias, Tout* __restrict__ out, int ldo, int accumulate, int M, int N, int K, int swiglu,
                 int stream, float* __restrict__ partials, int* __restrict__ counters, int* __restrict__ error_word) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;   // swizzled tiles want 1024-byte alignment
    uint8_t* aligned = smem_raw + (base - smem_u32(smem_raw));
    // the stages, the epilogue's staging (1024-byte aligned, as the stages are), the barriers
    const uint32_t bars = base + STAGES * STAGE_BYTES + STAGING_BYTES;
    // barriers: full[STAGES] (the first block's are used), empty[STAGES] (each block its own), acc_full[2] (each its
    // own), acc_empty[2] (the first block's); then the TMEM base and the abort flag
    auto full_bar = [&](int s) { return bars + 8u * s; };
    auto empty_bar = [&](int s) { return bars + 8u * (STAGES + s); };
    auto acc_full_bar = [&](int b) { return bars + 8u * (2 * STAGES + b); };
    auto acc_empty_bar = [&](int b) { return bars + 8u * (2 * STAGES + 2 + b); };
    uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(aligned + STAGES * STAGE_BYTES + STAGING_BYTES + 8 * (2 * STAGES + 4));
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_base_slot + 1);
    volatile int* parts_flag = reinterpret_cast<volatile int*>(tmem_base_slot + 2);
    const uint32_t fix_bar = bars + 8u * (2 * STAGES + 4) + 16u;   // parked parts arriving by bulk copy (behind the three words)
    uint8_t* staging = aligned + STAGES * STAGE_BYTES;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_rank();             // 0: the pair's first block, which issues the MMAs
    const int pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;
    const int tiles_m = (M + PAIR_M - 1) / PAIR_M, tiles_n = (N + BN - 1) / BN, tiles = tiles_m * tiles_n;
    const int k_blocks = (K + BK - 1) / BK;
    const int packed_tiles = (N + 127) >> 7;          // 128-row tiles of the packed weight
    // The work of a pair. Plain: whole tiles, tile = pair, pair + pairs, ... Streamed (stream-K): only the full rounds
    // of tiles go that way; the tiles of the last, partly filled round are cut up instead: their (tile, k block)
    // pairs, in tile order, are dealt out as one equal run per pair of blocks, and every pair walks its run FIRST and
    // its whole tiles after it, so that no SM idles through a round and what the cutting costs (parked partial tiles
    // and their adding up, in the epilogue warps) lies under the main loops of the whole tiles that follow. Of the
    // pairs that hold k blocks of one tile, the one with the tile's FIRST k blocks finishes it: that part is the last
    // of its run, and the others' parts are the first of theirs, so they are parked by the time it asks for them and
    // nobody who is waited for waits himself. All roles walk the same units with this.
    const int whole_tiles = stream ? tiles / pairs * pairs : tiles;
    const long long sk_kb = (long long)(tiles - whole_tiles) * k_blocks;     // streamed (tile, k block) pairs
    // (fewer of them than pairs of blocks: the first `dealt` take one each, so that no run between two others is empty)
    const long long dealt = min((long long)pairs, max(sk_kb, 1LL));
    auto run_start = [&](long long c) { return sk_kb * min(c, dealt) / dealt; };
    const long long run_lo = run_start(pair), run_hi = run_start(pair + 1);
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
        const int t = pair + w.i * pairs;
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
            mbar_init(acc_empty_bar(b), 8);   // one arrival per epilogue warp of both blocks
        }
        mbar_init(fix_bar, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 2) {   // the same warp of both blocks allocates all 512 columns in both (one block per SM)
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_base_slot)),
                     "r"(TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tcgen05_fence_before();
    __syncthreads();
    cluster_sync_all();      // the partner's barriers are set up and its tensor memory is there before anything reaches them
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_base_slot;
    pdl_wait();
    pdl_trigger();

    auto give_up = [&](int code) {
        *abort_flag = 1;
        store_cluster(in_block(smem_u32(const_cast<int*>(abort_flag)), rank ^ 1u), 1);
        atomicExch(error_word, code);
    };

    if (warp == 0) {
        // ---------------- producer (both blocks) ----------------
        if (lane == 0) {
            int s = 0;
            uint32_t parity = 1, dst = base;
            bool ok = true;
            Walk walk = first_unit();
            int tile, lo, hi;
            while (ok && next_unit(walk, tile, lo, hi)) {
                const int m0 = (tile % tiles_m) * PAIR_M + (int)rank * BM, tn = (tile / tiles_m) * 2;
                const bool mine = tn + (int)rank < packed_tiles;           // this block's half of the W rows exists
                const uint32_t tx = 2 * A_BYTES + (tn + 1 < packed_tiles ? 2 : 1) * W_BYTES;     // both blocks' bytes
                int wy = ((tn + (int)rank) * k_blocks + lo) * 128;         // row of the packed weight's k block
                for (int kb = lo; kb < hi; ++kb, wy += 128) {
                    if (!mbar_wait(empty_bar(s), parity, abort_flag)) { ok = false; break; }
                    const uint32_t full0 = in_block(full_bar(s), 0);
                    if (rank == 0) mbar_expect_tx(full_bar(s), tx);
                    tma_load_2d_pair(dst, &map_a, kb * BK, m0, full0);
                    if (mine) tma_load_2d_pair(dst + A_BYTES, &map_w, 0, wy, full0);
                    dst += STAGE_BYTES;
                    if (++s == STAGES) { s = 0; parity ^= 1u; dst = base; }
                }
            }
            if (!ok) give_up(21);
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer (the first block) ----------------
        if (lane == 0 && rank == 0) {
            uint32_t local_tile = 0, parity = 0, a_addr = base;
            int s = 0;
            bool ok = true;
            Walk walk = first_unit();
            int tile, lo, hi;
            for (; ok && next_unit(walk, tile, lo, hi); ++local_tile) {
                const uint32_t buf = local_tile & 1u;
                if (!mbar_wait(acc_empty_bar(buf), ((local_tile >> 1) & 1u) ^ 1u, abort_flag)) { ok = false; break; }
                tcgen05_fence_after();
                const uint32_t tmem_d = tmem_base + buf * BN;
                for (int kb = lo; kb < hi; ++kb) {
                    if (!mbar_wait(full_bar(s), parity, abort_flag)) { ok = false; break; }
                    tcgen05_fence_after();
                    const uint32_t b_addr = a_addr + A_BYTES;
#pragma unroll
                    for (int k = 0; k < BK / 16; ++k)
                        mma_pair(tmem_d, smem_desc_sw128(a_addr + k * 32), smem_desc_sw128(b_addr + k * 32), IDESC,
                                 (kb > lo || k > 0) ? 1u : 0u);
                    commit_pair(empty_bar(s));          // both blocks' stage is free when these MMAs have read it
                    a_addr += STAGE_BYTES;
                    if (++s == STAGES) { s = 0; parity ^= 1u; a_addr = base; }
                }
                if (ok) commit_pair(acc_full_bar(buf));
            }
            if (!ok) give_up(22);
        }
    } else {
        // ---------------- epilogue: warps 2..5 of both blocks, TMEM lanes 32 * (warp % 4) ----------------
        const int quad = warp & 3;
        const TileEpilogue<Tout> ep{out, ldo, M, N, accumulate, has_bias, swiglu, bias, bulk_out ? &map_out : nullptr};
        float* my_staging = reinterpret_cast<float*>(staging + quad * (bulk_out ? BULK_WARP_BYTES : STAGING_WARP_FLOATS * 4));
        uint32_t local_tile = 0, fix_parity = 0;
        bool ok = true;
        Walk walk = first_unit();
        int tile, k_lo, k_hi;
        for (; ok && next_unit(walk, tile, k_lo, k_hi); ++local_tile) {
            const int row0 = (tile % tiles_m) * PAIR_M + (int)rank * BM + quad * 32, n0 = (tile / tiles_m) * BN;
            const uint32_t buf = local_tile & 1u;
            if (!mbar_wait(acc_full_bar(buf), (local_tile >> 1) & 1u, abort_flag)) { ok = false; break; }
            tcgen05_fence_after();
            const uint32_t taddr = tmem_base + buf * BN + ((uint32_t)(quad * 32) << 16);
            const bool whole = ep.rows_whole(row0);
            auto release = [&]() {         // this warp has read the accumulator
                tcgen05_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive_cluster(in_block(acc_empty_bar(buf), 0));
            };
            if (k_lo == 0 && k_hi == k_blocks) {      // the whole tile is this pair's
#pragma unroll 1
                for (int c0 = 0; c0 < BN; c0 += 32) {
                    uint32_t v[32];
                    tmem_ld_32x32b_x32(taddr + c0, v);
                    tmem_ld_wait();
                    if (n0 + c0 < N) ep.store(v, row0, lane, n0 + c0, whole, my_staging);
                }
                release();
                continue;
            }
            // ---- the tile's k blocks are spread over several (consecutive) pairs; a block works with the blocks of
            // its own rank in them, which hold the same 128 rows ----
            int* counter = counters + 2 * tile + (int)rank;
            if (k_lo > 0) {
                // Not the tile's first k blocks: this is the first unit of the pair's run. Park the part ([block][BN
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
                release();
                asm volatile("bar.sync 1, 128;" ::: "memory");           // the four epilogue warps have written
                if (warp == 2 && lane == 0) {
                    __threadfence();
                    atomicAdd(counter, 1);
                }
                continue;
            }
            // The tile's first k blocks, the last unit of this pair's run: wait (bounded) until the pairs after this
            // one have parked theirs, add them to the accumulator in k order (so the sum does not depend on who was
            // when) and finish the tile. All blocks of the grid are resident.
            const long long tile_last_kb = (long long)(tile - whole_tiles + 1) * k_blocks - 1;
            const int others = (int)(((tile_last_kb + 1) * dealt + sk_kb - 1) / sk_kb - 1) - pair;
            if (warp == 2 && lane == 0) {
                int seen = 0;
                for (uint32_t tries = 0; seen < others && tries < SPIN_LIMIT; ++tries) {
                    asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(seen) : "l"(counter) : "memory");
                    if (seen < others) {
                        if ((tries & 255u) == 255u && *abort_flag) break;
                        __nanosleep(32);
                    }
                }
                if (seen >= others) *counter = 0;                     // back to zero for the next product
                *parts_flag = seen >= others;
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");
            if (!*parts_flag) { ok = false; break; }
            // Nothing follows this unit in this pair's work (always so when the product has fewer tiles than pairs): every
            // product of the pair is done, so the ring of stages is idle, and the parked parts come into it by bulk copies,
            // a stage's worth (64 columns of one part) each, as many pieces at a time as the ring holds with all their
            // parts: 192 KB on their way instead of one load per thread and column, the adding in the same order.
            const bool ring_idle = walk.at >= run_hi && (long long)pair + (long long)walk.i * pairs >= whole_tiles;
            if (ring_idle && others <= STAGES) {
                constexpr int PIECE = 64;
                static_assert(PIECE * BM * 4 == STAGE_BYTES, "a piece of a parked part fills one stage");
                const int per_round = STAGES / others;
                for (int p0 = 0; ok && p0 < BN / PIECE; p0 += per_round) {
                    const int p1 = min(BN / PIECE, p0 + per_round);
                    if (warp == 2 && lane == 0) {
                        // the parts were written by other blocks' ordinary stores (seen through the counter) and the ring
                        // was read by this block's ordinary loads: both before the copies of the asynchronous proxy
                        asm volatile("fence.proxy.async;" ::: "memory");
                        mbar_expect_tx(fix_bar, (uint32_t)((p1 - p0) * others) * STAGE_BYTES);
                        for (int pc = p0; pc < p1; ++pc)
                            for (int q = 0; q < others; ++q)
                                bulk_copy(base + (uint32_t)((pc - p0) * others + q) * STAGE_BYTES,
                                          partials + (size_t)(blockIdx.x + 2 * (q + 1)) * BM * BN + (size_t)pc * PIECE * BM,
                                          STAGE_BYTES, fix_bar);
                    }
                    if (!mbar_wait(fix_bar, fix_parity, abort_flag)) { ok = false; break; }
                    fix_parity ^= 1u;
#pragma unroll 1
                    for (int pc = p0; pc < p1; ++pc)
#pragma unroll 1
                        for (int h = 0; h < PIECE; h += 32) {
                            const int c0 = pc * PIECE + h;
                            uint32_t v[32];
                            tmem_ld_32x32b_x32(taddr + c0, v);
                            tmem_ld_wait();
                            for (int q = 0; q < others; ++q) {
                                const float* src = reinterpret_cast<const float*>(aligned + (size_t)((pc - p0) * others + q) * STAGE_BYTES) +
                                                   (size_t)h * BM + quad * 32 + lane;
#pragma unroll
                                for (int j = 0; j < 32; ++j) v[j] = __float_as_uint(__uint_as_float(v[j]) + src[(size_t)j * BM]);
                            }
                            if (n0 + c0 < N) ep.store(v, row0, lane, n0 + c0, whole, my_staging);
                        }
                    asm volatile("bar.sync 1, 128;" ::: "memory");      // all have read the ring: the next round may overwrite it
                }
                if (!ok) break;
                release();
                asm volatile("bar.sync 1, 128;" ::: "memory");
                continue;
            }
            const float* theirs = partials + (size_t)(blockIdx.x + 2) * BM * BN + quad * 32 + lane;
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
                    for (int j = 0; j < 32; ++j) x[j] = __ldcg(theirs + (size_t)(2 * p) * BM * BN + (size_t)(c0 + j) * BM);
                }
                if (n0 + c0 < N) ep.store(v, row0, lane, n0 + c0, whole, my_staging);
            }
            release();
            // (the next unit's wait on another flag value cannot pass a warp that has not read this one yet)
            asm volatile("bar.sync 1, 128;" ::: "memory");
        }
        ep.bulk_done(lane);
        if (!ok && lane == 0) give_up(23);
    }
    tcgen05_fence_before();
    __syncthreads();
    cluster_sync_all();      // neither block leaves, or frees tensor memory, while the other may still reach into it
    if (warp == 2) {
        tcgen05_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

// The packed weight ([tiles of 128 rows][k blocks][128 rows][64 values], each 16 KB tile the swizzled shared-memory
// image) as a matrix of 128-byte rows, copied in boxes of one tile without any further swizzle.
struct PackedKey {
    const void* ptr;
    long long rows;
    bool operator==(const PackedKey& o) const { return ptr == o.ptr && rows == o.rows; }
};
struct PackedKeyHash {
    size_t operator()(const PackedKey& k) const { return std::hash<const void*>()(k.ptr) * 1000003u ^ std::hash<long long>()(k.rows); }
};
int packed_map_for(const void* ptr, long long rows, CUtensorMap* out) {
    static std::unordered_map<PackedKey, CUtensorMap, PackedKeyHash> cache;
    static std::mutex mu;
    const PackedKey key{ptr, rows};
    std::lock_guard<std::mutex> lock(mu);
    auto it = cache.find(key);
    if (it != cache.end()) {
        *out = it->second;
        return JLLM_OK;
    }
    EncodeTiledFn fn = encode_fn();
    if (!fn) return jllm_fail(JLLM_CUDA_ERROR, "gemm_pair: the driver does not offer cuTensorMapEncodeTiled");
    const cuuint64_t dims[2] = {64, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {128};
    const cuuint32_t box[2] = {64, 128};
    const cuuint32_t elem[2] = {1, 1};
    CUtensorMap map;
    const CUresult r = fn(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, elem,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
        return jllm_fail(JLLM_CUDA_ERROR, "gemm_pair: cuTensorMapEncodeTiled failed (%d) for a packed weight of %lld rows",
                         (int)r, rows);
    if (cache.size() > 4096) cache.clear();
    cache.emplace(key, map);
    *out = map;
    return JLLM_OK;
}

// how many pairs the device runs at a time (clusters of two with this much shared memory), looked up once per kernel
template <typename Tout>
int resident_pairs() {
    static int pairs = -1;
    if (pairs >= 0) return pairs;
    auto kern = gemm_pair_kernel<Tout>;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES) != cudaSuccess) return 0;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * (jllm_device_sm_count() > 0 ? jllm_device_sm_count() : 2));
    cfg.blockDim = dim3(THREADS);
    cfg.dynamicSmemBytes = SMEM_BYTES;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess) {
        cudaGetLastError();
        n = 0;
    }
    pairs = n;
    return pairs;
}

}  // namespace

int* jllm_gemm_error_word();
extern int g_plain_stores;

JLLM_EXPORT int jllm_gemm_pair_fits(const void* a, int lda, const void* w_packed, int M, int N, int K) {
    return M >= 1 && N >= 1 && K >= 8 && K % 8 == 0 && lda % 8 == 0 && ((uintptr_t)a % 16) == 0 &&
           ((uintptr_t)w_packed % 16) == 0;
}

// w: ops.pack_weight of the [N, K] weight (k_blocks_packed = ceil(K / 64) its k blocks).
JLLM_EXPORT int jllm_gemm_pair(const void* a, int lda, const void* w, int k_blocks_packed, const void* bias, int bias_dtype,
                               void* out, int out_dtype, int ldo, int accumulate, int M, int N, int K, int max_pairs,
                               int swiglu, float* workspace, long long workspace_floats, int stream_mode,
                               cudaStream_t stream) {
    JLLM_REQUIRE(jllm_gemm_pair_fits(a, lda, w, M, N, K),
                 "gemm_pair: needs K %% 8 == 0 and 16-byte aligned rows (M=%d N=%d K=%d lda=%d)", M, N, K, lda);
    JLLM_REQUIRE(k_blocks_packed == (K + BK - 1) / BK, "gemm_pair: the packed weight has %d k blocks, K=%d needs %d",
                 k_blocks_packed, K, (K + BK - 1) / BK);
    JLLM_REQUIRE(ldo >= (swiglu ? N / 2 : N), "gemm_pair: ldo=%d < N=%d", ldo, N);
    JLLM_REQUIRE(!swiglu || (N % 16 == 0 && !bias && !accumulate),
                 "gemm_pair: the SwiGLU epilogue needs N %% 16 == 0, no bias and no accumulation (N=%d)", N);
    const long long packed_rows = (long long)((N + 127) / 128) * k_blocks_packed * 128;
    JLLM_REQUIRE(packed_rows < (1LL << 31), "gemm_pair: a packed weight of %lld rows of 128 bytes is too long", packed_rows);
    CUtensorMap map_a, map_w;
    int rc = tensor_map_for(a, M, K, lda, BM, &map_a);
    if (rc != JLLM_OK) return rc;
    rc = packed_map_for(w, packed_rows, &map_w);
    if (rc != JLLM_OK) return rc;
    CUtensorMap map_out = {};
    const int bulk_out = out_dtype == JLLM_F32 && !swiglu && ldo % 4 == 0 && ((uintptr_t)out % 16) == 0 && !g_plain_stores;
    if (bulk_out) {
        rc = tensor_map_out_f32(out, M, N, ldo, &map_out);
        if (rc != JLLM_OK) return rc;
    }
    int* error_word = jllm_gemm_error_word();
    if (!error_word) return jllm_fail(JLLM_CUDA_ERROR, "gemm_pair: no error word");
    const int tiles = ((M + PAIR_M - 1) / PAIR_M) * ((N + BN - 1) / BN);
    int pairs = out_dtype == JLLM_F32 ? resident_pairs<float>() : resident_pairs<__nv_bfloat16>();
    JLLM_REQUIRE(pairs >= 1, "gemm_pair: the device runs no cluster of two blocks with %zu bytes of shared memory", SMEM_BYTES);
    // (a streamed product of fewer tiles than pairs still runs on all pairs: every tile is cut up then)
    const long long units = stream_mode == 1 ? (long long)tiles * k_blocks_packed : (long long)tiles;
    if (pairs > units) pairs = (int)units;
    if (max_pairs > 0 && pairs > max_pairs) pairs = max_pairs;
    // stream_mode 1: the tiles of a last, partly filled round are cut up over all pairs (stream-K). Not the default: what
    // an idle pair in the last round loses, the busy ones win back (they share one memory system and one power limit).
    // The O product of 2,048 rows (128 tiles on 74 pairs), a pair's main loops by the device's clock: plain 21.0 us for
    // its first tile, 18.6 us for its second, which only 54 pairs have; streamed 17.5 us for 0.73 of a tile, then
    // 20.2 us for a whole one; 50 us against 48 to 56 us in all. The workspace holds two counters per tile (zero
    // before the first product, left zero by every product) and one parked partial tile per block.
    const long long need = 2LL * PAIR_MAX_TILES + 2LL * pairs * BM * BN;
    int streamed = 0;
    if (stream_mode == 1) {
        const bool room = workspace != nullptr && workspace_floats >= need && tiles <= PAIR_MAX_TILES;
        JLLM_REQUIRE(room, "gemm_pair: a streamed product of %d tiles on %d pairs needs a workspace of %lld floats (got "
                           "%lld) and at most %d tiles", tiles, pairs, need, workspace_floats, PAIR_MAX_TILES);
        streamed = 1;
    }
    int* counters = reinterpret_cast<int*>(workspace);
    float* partials = workspace ? workspace + 2 * PAIR_MAX_TILES : nullptr;
    const VecRef b{bias, bias_dtype};
    if (out_dtype == JLLM_F32) {
        jllm_launch(gemm_pair_kernel<float>, dim3(2 * pairs), dim3(THREADS), SMEM_BYTES, stream, true, map_a, map_w, map_out,
                    bulk_out, b,
                    (int)(bias != nullptr), (float*)out, ldo, accumulate, M, N, K, swiglu, streamed, partials, counters,
                    error_word);
    } else {
        jllm_launch(gemm_pair_kernel<__nv_bfloat16>, dim3(2 * pairs), dim3(THREADS), SMEM_BYTES, stream, true, map_a, map_w,
                    map_out, 0, b, (int)(bias != nullptr), (__nv_bfloat16*)out, ldo, accumulate, M, N, K, swiglu, streamed, partials,
                    counters, error_word);
    }
    return jllm_check_launch("gemm_pair");
}

// The pairs of blocks the device runs at a time (0: none, the product is not offered).
JLLM_EXPORT int jllm_gemm_pair_resident() { return resident_pairs<float>(); }
