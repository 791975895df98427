// Decode attention for head sizes 64, 128 and 256: the same block layout and split scheme as the direct
// kernel of attention_decode.cu, but keys and values travel through shared memory in a ring of stages.
//
// A decode step is a stream of the cache: what matters is how many bytes each SM has in flight. Here the
// 128 threads of a block gather a tile of 64 keys and 64 values (from up to 64 / page_size pages) into
// XOR-swizzled shared memory with cp.async, three tiles deep, so about two tiles (64 KB at head size 128)
// are always on their way while the tensor cores work on a third. Warp w owns keys [16 w, 16 w + 16) of
// every tile: S = Q K^T and O += P V with mma.sync.m16n8k16 from ldmatrix fragments, the G query heads
// of the kv head being the 16 rows of the M side (rows beyond G are zero). Each warp keeps its own online
// softmax state; the four are merged at the end exactly as in the direct kernel, and the per-split
// partials go to the same scratch layout and combine kernel.
#pragma once
#include "head_rotate.cuh"

namespace staged {

constexpr int WARPS = 4, THREADS = 128, TILE = 64, STAGES = 3;

__device__ __forceinline__ void mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ldsm4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm4t(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void cp16(uint32_t dst, const void* src, int bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
}
// 2^x by the special-function unit alone (the bfloat16 path rounds the result to 8 bits of mantissa anyway)
__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ void commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N>
__device__ __forceinline__ void wait_group() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory"); }

template <int HD>
__device__ __forceinline__ uint32_t off(int r, int c) { return (uint32_t)((r * (HD / 8) + (c ^ (r & 7))) * 16); }

// What the kernel in front of a FRESH launch left undone: the step's own queries, key and value lie in `qkv` as the QKV
// product wrote them ([rows, stride]: query heads, key heads, value heads side by side), not yet normed, rotated or
// written to the cache. The attention then does that work for its own row: every block norms and rotates the G
// queries of its kv head on their way into shared memory, and the one block whose keys hold the row's newest position
// makes that key (norm, rotation) and value, writes them to the cache and puts them into its own tile. One launch
// and its dependent wait less per layer than with a kernel of their own. qkv == nullptr: a plain launch.
struct Fresh {
    const __nv_bfloat16* qkv;
    int stride, use_norm;
    float eps;
    VecRef q_gain, k_gain;
    const float* cos_t;        // [positions, HD / 2]
    const float* sin_t;
    __nv_bfloat16* k_out;      // the cache, to be written
    __nv_bfloat16* v_out;
};

// a head from global memory into the registers of a warp, as head_norm_rope wants it
template <int V>
__device__ __forceinline__ void head_load(const __nv_bfloat16* __restrict__ src, int lane, float (&a)[V], float (&b)[V]) {
#pragma unroll
    for (int i = 0; i < V; ++i) {
        a[i] = __bfloat162float(src[lane * V + i]);
        b[i] = __bfloat162float(src[32 * V + lane * V + i]);
    }
}
// ... and back as bfloat16 into row `row` of a swizzled tile in shared memory
template <int HD>
__device__ __forceinline__ void head_store(uint8_t* tile, int row, int lane, const float (&a)[HD / 64],
                                           const float (&b)[HD / 64]) {
    constexpr int V = HD / 64, HALF = HD / 2;
#pragma unroll
    for (int i = 0; i < V; ++i) {
        const int e0 = lane * V + i, e1 = HALF + e0;
        *reinterpret_cast<__nv_bfloat16*>(tile + off<HD>(row, e0 >> 3) + (e0 & 7) * 2) = __float2bfloat16_rn(a[i]);
        *reinterpret_cast<__nv_bfloat16*>(tile + off<HD>(row, e1 >> 3) + (e1 & 7) * 2) = __float2bfloat16_rn(b[i]);
    }
}

// The keys [first + tile_lo * 64, ...) of n_tiles tiles of one (row, kv head), for the G query heads of that kv head:
// the result goes to `out` if these are all the row's keys (`whole`), else as a partial (sums, maximum, weight) for
// head j of the group to part_o + j * o_stride and part_ml + j * ml_stride. All threads of the block call it.
template <int HD>
__device__ __forceinline__ void attend(uint8_t* smem_raw, const __nv_bfloat16* __restrict__ q, int q_stride,
                                       const __nv_bfloat16* __restrict__ k_cache, const __nv_bfloat16* __restrict__ v_cache,
                                       __nv_bfloat16* __restrict__ out, int out_stride, const int* __restrict__ table,
                                       int table_len, int num_pages, int heads, int kv_heads, int page_size,
                                       float scale_log2, int r, int kvh, int P,
                                       int first, int tile_lo, int n_tiles, bool whole, float* __restrict__ part_o,
                                       size_t o_stride, float* __restrict__ part_ml, size_t ml_stride,
                                       const Fresh& fresh, bool early = false) {
    // `early`: the block has not yet waited for the kernel in front of it (programmatic dependent launch). That kernel
    // wrote the queries and the key and value of position P; the block tables and the positions came from the host
    // before the step, and the keys and values of earlier positions were written by earlier steps. So the rows of
    // the first two tiles are looked up, and those tiles requested if they end before P, while that kernel still
    // runs; the wait comes before anything of position P or of the queries is touched.
    constexpr int CHUNKS = HD / 8, TILE_BYTES = TILE * HD * 2, STAGE_BYTES = 2 * TILE_BYTES;
    const uint32_t s_q = (uint32_t)__cvta_generic_to_shared(smem_raw);
    const uint32_t s_kv = s_q + 16 * HD * 2;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int G = heads / kv_heads;
    const size_t page_stride = (size_t)kv_heads * page_size * HD;
    const int page_shift = (page_size & (page_size - 1)) == 0 ? __ffs(page_size) - 1 : -1;

    // Q: the G heads of this kv head as rows 0 .. G-1 of a 16-row tile (the rest zero)
    const bool fused = fresh.qkv != nullptr;
    auto load_q = [&]() {
        for (int i = threadIdx.x; i < 16 * CHUNKS; i += THREADS) {
            const int row = i / CHUNKS, c = i % CHUNKS;
            const __nv_bfloat16* src = q + (size_t)r * q_stride + (size_t)(kvh * G + min(row, G - 1)) * HD + c * 8;
            cp16(s_q + off<HD>(row, c), src, row < G ? 16 : 0);
        }
    };
    // Where the rows of a tile lie in the cache (element offset of the key's first value, -1 past the end): looked
    // up by one thread per row a tile ahead of the copies, so that no copy waits for a page-table load.
    __shared__ long long s_row_base[2][TILE];
    __shared__ __align__(16) __nv_bfloat16 s_fresh[2 * HD];       // the row's newest key and value (a fresh launch)
    auto find_rows = [&](int i) {
        if (i < n_tiles && threadIdx.x < TILE) {
            const int key = first + (tile_lo + i) * TILE + threadIdx.x;
            long long o = -1;
            if (key <= P) {
                const int pg = page_shift >= 0 ? key >> page_shift : key / page_size;
                const int in_page = page_shift >= 0 ? key & (page_size - 1) : key % page_size;
                const long long page = jllm_page_of(table, pg, table_len, num_pages);   // -1: checked build, bad entry
                if (!kCheckBounds || page >= 0)
                    o = (long long)((size_t)page * page_stride + ((size_t)kvh * page_size + in_page) * HD);
            }
            s_row_base[i & 1][threadIdx.x] = o;
        }
    };
    auto load_tile = [&](int i) {   // tile i of this block's range into stage i % STAGES
        if (i < n_tiles) {
            const uint32_t dk = s_kv + (i % STAGES) * STAGE_BYTES, dv = dk + TILE_BYTES;
            // consecutive threads take consecutive 16-byte chunks of a row (coalesced reads, conflict-free writes)
#pragma unroll
            for (int j = threadIdx.x; j < TILE * CHUNKS; j += THREADS) {
                const int row = j / CHUNKS, c = j % CHUNKS;
                const long long base_o = s_row_base[i & 1][row];
                const bool ok = base_o >= 0;
                const size_t o = ok ? (size_t)base_o + c * 8 : 0;
                cp16(dk + off<HD>(row, c), k_cache + o, ok ? 16 : 0);
                cp16(dv + off<HD>(row, c), v_cache + o, ok ? 16 : 0);
            }
        }
        commit();   // an empty group keeps the group count in step with the tile count
    };
    static_assert(STAGES == 3, "the row look-ahead below is written for a ring of three stages");
    find_rows(0);
    find_rows(1);
    __syncthreads();
    // a tile may be requested before the wait if all its keys lie before position P
    const int last_of_0 = first + (tile_lo + 1) * TILE - 1, last_of_1 = last_of_0 + TILE;
    const bool pre0 = early && last_of_0 < P, pre1 = early && last_of_1 < P;
    if (pre0) load_tile(0);
    if (pre1) load_tile(1);
    if (early) {
        pdl_wait();
        pdl_trigger();
    }
    // A fresh launch: this row's queries, and in one block of the pair its newest key and value, are still to be made.
    // Their raw values are asked for first, then the first tiles, and the arithmetic is done while the tiles travel.
    constexpr int V = HD / 64;
    const int fresh_tile = (P - first) / TILE - tile_lo;      // of this block's tiles, the one with position P (if any)
    const bool makes_kv = fused && fresh_tile >= 0 && fresh_tile < n_tiles;
    float qa[V], qb[V], ka[V], kb[V];
    uint4 vv = make_uint4(0, 0, 0, 0);
    if (fused) {
        const __nv_bfloat16* mine = fresh.qkv + (size_t)r * fresh.stride;
        if (warp < G) head_load<V>(mine + (size_t)(kvh * G + warp) * HD, lane, qa, qb);
        if (makes_kv && warp == 0) head_load<V>(mine + (size_t)(heads + kvh) * HD, lane, ka, kb);
        if (makes_kv && warp == 1 && lane < CHUNKS)
            vv = *reinterpret_cast<const uint4*>(mine + (size_t)(heads + kv_heads + kvh) * HD + lane * 8);
    } else {
        load_q();
    }
    if (!pre0) load_tile(0); else if (!pre1) load_tile(1);     // (each load_tile commits a group; Q rides in this one)
    if (!pre0 && !pre1) load_tile(1);
    if (pre0 && pre1) commit();                                 // Q alone
    if (fused) {
        const float* cos_row = fresh.cos_t + (size_t)P * (HD / 2);
        const float* sin_row = fresh.sin_t + (size_t)P * (HD / 2);
        // the queries: a warp per head, norm and rotation in registers, bfloat16 into the tile (visible to all after the
        // barrier that the first key tile waits at); rows beyond the G heads are zero
        for (int row = warp; row < 16; row += WARPS) {
            if (row < G) {
                if (row != warp) head_load<V>(fresh.qkv + (size_t)r * fresh.stride + (size_t)(kvh * G + row) * HD, lane, qa, qb);
                head_norm_rope<V>(qa, qb, lane, fresh.use_norm, fresh.eps, fresh.q_gain, cos_row, sin_row);
                head_store<HD>(smem_raw, row, lane, qa, qb);
            } else {
                for (int c = lane; c < CHUNKS; c += 32)
                    *reinterpret_cast<uint4*>(smem_raw + off<HD>(row, c)) = make_uint4(0, 0, 0, 0);
            }
        }
        if (makes_kv) {
            // The row's newest key and value fall to this block: warp 0 makes the key (norm, rotation), warp 1 takes the
            // value; both write the cache and park their HD values in shared memory until the tile that holds position P
            // has arrived (the barriers of the loop lie between).
            const int pg = page_shift >= 0 ? P >> page_shift : P / page_size;
            const int in_page = page_shift >= 0 ? P & (page_size - 1) : P % page_size;
            const long long page = jllm_page_of(table, pg, table_len, num_pages);       // -1: checked build, bad entry
            const bool writes = !kCheckBounds || page >= 0;
            const size_t at = writes ? (size_t)page * page_stride + ((size_t)kvh * page_size + in_page) * HD : 0;
            if (warp == 0) {
                head_norm_rope<V>(ka, kb, lane, fresh.use_norm, fresh.eps, fresh.k_gain, cos_row, sin_row);
                __nv_bfloat16* dst = writes ? fresh.k_out + at : nullptr;
#pragma unroll
                for (int i = 0; i < V; ++i) {
                    const int e0 = lane * V + i, e1 = HD / 2 + e0;
                    const __nv_bfloat16 v0 = __float2bfloat16_rn(ka[i]), v1 = __float2bfloat16_rn(kb[i]);
                    s_fresh[e0] = v0;
                    s_fresh[e1] = v1;
                    if (dst != nullptr) {
                        dst[e0] = v0;
                        dst[e1] = v1;
                    }
                }
            } else if (warp == 1 && lane < CHUNKS) {
                reinterpret_cast<uint4*>(s_fresh + HD)[lane] = vv;
                if (writes) *reinterpret_cast<uint4*>(fresh.v_out + at + lane * 8) = vv;
            }
        }
    }
    __syncthreads();        // everyone has read the rows of tile 0: its slot takes those of tile 2
    find_rows(2);

    uint32_t qf[HD / 16][4];
    float o[HD / 8][4];
#pragma unroll
    for (int j = 0; j < HD / 8; ++j)
#pragma unroll
        for (int i = 0; i < 4; ++i) o[j][i] = 0.f;
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};

    for (int i = 0; i < n_tiles; ++i) {
        // tile i has landed (the groups of later tiles may still be in flight); before the first tile everything that
        // was asked for so far, because Q may have been asked for after tile 1
        if (i == 0) wait_group<0>(); else wait_group<STAGES - 2>();
        __syncthreads();            // ... for every thread's part of it; and everyone is done with tile i - 1
        load_tile(i + STAGES - 1);  // refills the stage that tile i - 1 used
        find_rows(i + STAGES);      // into the slot that tile i + 1's copies (issued an iteration ago) have left
        if (i == 0) {
#pragma unroll
            for (int ks = 0; ks < HD / 16; ++ks) ldsm4(qf[ks], s_q + off<HD>(lane & 15, ks * 2 + (lane >> 4)));
        }
        const uint32_t sk = s_kv + (i % STAGES) * STAGE_BYTES, sv = sk + TILE_BYTES;
        if (fused && i == fresh_tile) {
            // This tile holds the row's newest position (the copy brought whatever the cache held there): the key and value
            // made at the start go into their row of the tile. (One block of a (row, kv head) pair comes here, once.)
            uint8_t* tile_k = smem_raw + 16 * HD * 2 + (size_t)(i % STAGES) * STAGE_BYTES;
            const int row = P - first - (tile_lo + i) * TILE;
            if (threadIdx.x < 2 * CHUNKS) {
                const int which = threadIdx.x / CHUNKS, c = threadIdx.x % CHUNKS;     // 0: key, 1: value
                *reinterpret_cast<uint4*>(tile_k + which * TILE_BYTES + off<HD>(row, c)) =
                    reinterpret_cast<const uint4*>(s_fresh)[which * CHUNKS + c];
            }
            __syncthreads();
        }
        const int key0 = first + (tile_lo + i) * TILE + warp * 16;
        if (key0 > P) continue;     // this warp's 16 keys of the last tile are all past the end (warp-uniform)
        float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
        for (int ks = 0; ks < HD / 16; ++ks) {
            uint32_t kf[4];
            ldsm4(kf, sk + off<HD>(warp * 16 + (lane & 7) + ((lane >> 4) << 3), ks * 2 + ((lane >> 3) & 1)));
            mma(s[0], qf[ks], kf[0], kf[1]);
            mma(s[1], qf[ks], kf[2], kf[3]);
        }
        float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int tile = 0; tile < 2; ++tile)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int key = key0 + tile * 8 + 2 * t + (e & 1);
                s[tile][e] = key <= P ? s[tile][e] * scale_log2 : -INFINITY;
                mx[e >> 1] = fmaxf(mx[e >> 1], s[tile][e]);
            }
        float corr[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
            mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
            const float m_new = fmaxf(m[h], mx[h]);   // finite: key0 <= P, so the warp sees at least one key
            corr[h] = ex2(m[h] - m_new);
            m[h] = m_new;
            l[h] *= corr[h];
        }
        const bool rescale = !__all_sync(0xffffffffu, corr[0] == 1.f && corr[1] == 1.f);   // no row's maximum moved
        uint32_t pf[4];
#pragma unroll
        for (int tile = 0; tile < 2; ++tile) {
            const float p0 = ex2(s[tile][0] - m[0]), p1 = ex2(s[tile][1] - m[0]);
            const float p2 = ex2(s[tile][2] - m[1]), p3 = ex2(s[tile][3] - m[1]);
            l[0] += p0 + p1;
            l[1] += p2 + p3;
            __nv_bfloat162 a = __floats2bfloat162_rn(p0, p1), b = __floats2bfloat162_rn(p2, p3);
            pf[tile * 2 + 0] = *reinterpret_cast<uint32_t*>(&a);
            pf[tile * 2 + 1] = *reinterpret_cast<uint32_t*>(&b);
        }
#pragma unroll
        for (int jp = 0; jp < HD / 16; ++jp) {
            uint32_t vf[4];
            ldsm4t(vf, sv + off<HD>(warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, jp * 2 + (lane >> 4)));
            if (rescale) {
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    o[2 * jp + e][0] *= corr[0];
                    o[2 * jp + e][1] *= corr[0];
                    o[2 * jp + e][2] *= corr[1];
                    o[2 * jp + e][3] *= corr[1];
                }
            }
            mma(o[2 * jp], pf, vf[0], vf[1]);
            mma(o[2 * jp + 1], pf, vf[2], vf[3]);
        }
    }
    wait_group<0>();
    __syncthreads();                // the stages are free: they become the merge area
    // ---- merge the four warps (as the direct kernel does) ----
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        l[h] += __shfl_xor_sync(0xffffffffu, l[h], 1);
        l[h] += __shfl_xor_sync(0xffffffffu, l[h], 2);
    }
    float* so = reinterpret_cast<float*>(smem_raw + 16 * HD * 2);   // [WARPS][16][HD]
    float* sml = so + WARPS * 16 * HD;                               // [WARPS][16][2]
    if (t == 0) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            sml[(warp * 16 + g + 8 * h) * 2 + 0] = m[h];
            sml[(warp * 16 + g + 8 * h) * 2 + 1] = l[h];
        }
    }
    __syncthreads();
    float scale_w[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        float mm = -INFINITY;
        for (int w = 0; w < WARPS; ++w) mm = fmaxf(mm, sml[(w * 16 + g + 8 * h) * 2]);
        scale_w[h] = m[h] == -INFINITY ? 0.f : exp2f(m[h] - mm);
    }
#pragma unroll
    for (int j = 0; j < HD / 8; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e)
            so[((size_t)warp * 16 + g + 8 * (e >> 1)) * HD + j * 8 + 2 * t + (e & 1)] = o[j][e] * scale_w[e >> 1];
    __syncthreads();
    for (int e = threadIdx.x; e < G * HD; e += THREADS) {
        const int row = e / HD, d = e % HD;
        float acc = 0.f, mm = -INFINITY, ll = 0.f;
        for (int w = 0; w < WARPS; ++w) acc += so[((size_t)w * 16 + row) * HD + d];
        for (int w = 0; w < WARPS; ++w) mm = fmaxf(mm, sml[(w * 16 + row) * 2]);
        for (int w = 0; w < WARPS; ++w) {
            const float mw = sml[(w * 16 + row) * 2];
            ll += mw == -INFINITY ? 0.f : sml[(w * 16 + row) * 2 + 1] * exp2f(mw - mm);
        }
        if (whole) {
            out[(size_t)r * out_stride + (size_t)(kvh * G + row) * HD + d] = __float2bfloat16_rn(acc / ll);
        } else {
            part_o[(size_t)row * o_stride + d] = acc;
            if (d == 0) {
                part_ml[(size_t)row * ml_stride + 0] = mm;
                part_ml[(size_t)row * ml_stride + 1] = ll;
            }
        }
    }
}

// ---- the partials of a (row, kv head) pair added up inside the attention kernel ------------------------------------
// Every block that has written a partial of the pair counts itself in (after a fence: its partial is visible to the
// device first); the one that finds itself last adds the partials up, in the order of the parts whoever it is, and puts
// the counter back to zero for the next launch. Nobody waits for anybody. The counters belong to the library (zero
// when it is loaded): launches of these kernels on one device must not overlap.
constexpr int PAIR_COUNTERS = 1 << 16;
__device__ int g_pair_counters[PAIR_COUNTERS];

// true in all threads of the one block that is the `expected`-th to arrive; all threads of the block call it
__device__ __forceinline__ bool last_of_pair(int* counter, int expected) {
    __shared__ int s_last;
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        const int seen = atomicAdd(counter, 1);
        s_last = seen == expected - 1;
        if (s_last) *counter = 0;
    }
    __syncthreads();
    const bool last = s_last != 0;
    if (last) __threadfence();
    return last;
}

// out_pair[row * HD + d] for the G heads of the pair from `parts` partials: part p of head `row` has its sums at
// po + p * o_part + row * o_row and (maximum, weight) at pml + p * ml_part + row * ml_row. A warp per head; the
// arithmetic and its order are those of the combine kernels. parts <= 64.
template <int HD>
__device__ __forceinline__ void combine_pair(const float* __restrict__ po, size_t o_part, size_t o_row,
                                             const float* __restrict__ pml, size_t ml_part, size_t ml_row, int parts,
                                             int G, __nv_bfloat16* __restrict__ out_pair) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int row = warp; row < G; row += WARPS) {
        float ms[2], ls[2], w[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int p = lane + 32 * h;
            ms[h] = p < parts ? __ldcg(pml + p * ml_part + row * ml_row) : -INFINITY;
            ls[h] = p < parts ? __ldcg(pml + p * ml_part + row * ml_row + 1) : 0.f;
        }
        float M = fmaxf(ms[0], ms[1]);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, o));
        float L = 0.f;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            w[h] = ms[h] == -INFINITY ? 0.f : exp2f(ms[h] - M);
            for (int i = 0; i < 32 && i + 32 * h < parts; ++i) L += __shfl_sync(0xffffffffu, ls[h] * w[h], i);
        }
        const float inv = 1.f / L;
        float acc[HD / 32];
#pragma unroll
        for (int j = 0; j < HD / 32; ++j) acc[j] = 0.f;
        for (int p0 = 0; p0 < parts; p0 += 4) {        // four parts' loads on their way at a time; added in part order
            float x[4][HD / 32], wq[4];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const int p = p0 + q;
                wq[q] = __shfl_sync(0xffffffffu, p < 32 ? w[0] : w[1], p & 31);
                if (p >= parts) wq[q] = 0.f;
                const float* src = po + (size_t)min(p, parts - 1) * o_part + row * o_row + lane;
#pragma unroll
                for (int j = 0; j < HD / 32; ++j) x[q][j] = __ldcg(src + 32 * j);
            }
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                if (wq[q] == 0.f) continue;
#pragma unroll
                for (int j = 0; j < HD / 32; ++j) acc[j] += x[q][j] * wq[q];
            }
        }
#pragma unroll
        for (int j = 0; j < HD / 32; ++j) out_pair[(size_t)row * HD + lane + 32 * j] = __float2bfloat16_rn(acc[j] * inv);
    }
}

template <int HD>
__global__ void __launch_bounds__(THREADS)
attention_decode_staged_kernel(const __nv_bfloat16* __restrict__ q, int q_stride,
                               const __nv_bfloat16* __restrict__ k_cache, const __nv_bfloat16* __restrict__ v_cache,
                               __nv_bfloat16* __restrict__ out, int out_stride, const int* __restrict__ row_seg,
                               const int* __restrict__ row_pos, const int* __restrict__ block_tables, int table_stride,
                               int heads, int kv_heads, int page_size, int num_pages, int window, float scale_log2,
                               int splits, float* __restrict__ part_o, float* __restrict__ part_ml,
                               int* __restrict__ counters, const Fresh fresh) {
    extern __shared__ __align__(128) uint8_t smem_raw[];
    const int r = blockIdx.x, kvh = blockIdx.y, split = blockIdx.z;
    const int G = heads / kv_heads;
    // (the wait for the kernel in front, which wrote the newest key and value of every row and the queries, is inside
    // `attend`, behind the look-ups and the first requests that do not depend on it)
    const int P = row_pos[r];
    const int first = window > 0 ? max(0, P + 1 - window) : 0;
    const int tiles_total = (P + 1 - first + TILE - 1) / TILE;
    const int tiles_per_split = (tiles_total + splits - 1) / splits;
    const int tile_lo = split * tiles_per_split, tile_hi = min(tiles_total, tile_lo + tiles_per_split);
    const int* table = block_tables + (size_t)row_seg[r] * table_stride;
    // partials: (row, head, split) -> head_dim sums in part_o, (maximum, weight) in part_ml
    const size_t slot = ((size_t)r * heads + kvh * G) * splits + split;
    attend<HD>(smem_raw, q, q_stride, k_cache, v_cache, out, out_stride, table, table_stride, num_pages, heads, kv_heads,
               page_size, scale_log2, r, kvh, P, first, tile_lo, max(0, tile_hi - tile_lo), splits == 1, part_o + slot * HD,
               (size_t)splits * HD, part_ml + slot * 2, (size_t)splits * 2, fresh, true);
    // (without counters a combine kernel follows)
    if (splits > 1 && counters != nullptr && last_of_pair(counters + (size_t)r * kv_heads + kvh, splits)) {
        const size_t slot0 = ((size_t)r * heads + kvh * G) * splits;
        combine_pair<HD>(part_o + slot0 * HD, (size_t)HD, (size_t)splits * HD, part_ml + slot0 * 2, (size_t)2,
                         (size_t)splits * 2, splits, G, out + (size_t)r * out_stride + (size_t)kvh * G * HD);
    }
}

// ---- the same attention with the key tiles of all (row, kv head) pairs dealt out evenly ----------------------------------
// With one block per (row, kv head, split) the blocks of a step rarely fill the SMs evenly (8 rows x 8 kv heads x 4
// splits are 256 blocks for 296 places: most SMs carry two blocks, the rest one, and the step waits for the former).
// Here the key tiles of all pairs, in the order (row, kv head, tile), are cut into one equal run per block, as many
// blocks as there are places. A block's run may end inside a pair and go on in the next one: for every stretch it
// writes a partial (sums, maximum, weight) at slot pair + block, a number no other stretch has, and the combine kernel
// adds the partials of a pair in block order.
constexpr int FLAT_MAX_ROWS = 1024;

// s_cum[i] = key tiles of rows 0 .. i - 1 (of one kv head each); called by warp 0
__device__ __forceinline__ void flat_prefix(const int* __restrict__ row_pos, int rows, int window, int* s_cum) {
    const int lane = threadIdx.x & 31;
    int carry = 0;
    for (int base = 0; base < rows; base += 32) {
        const int r = base + lane;
        int incl = 0;
        if (r < rows) {
            const int P = row_pos[r], first = window > 0 ? max(0, P + 1 - window) : 0;
            incl = (P + 1 - first + TILE - 1) / TILE;
        }
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int v = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= o) incl += v;
        }
        if (r < rows) s_cum[r + 1] = carry + incl;
        carry += __shfl_sync(0xffffffffu, incl, 31);
    }
    if (lane == 0) s_cum[0] = 0;
}

template <int HD>
__global__ void __launch_bounds__(THREADS)
attention_decode_flat_kernel(const __nv_bfloat16* __restrict__ q, int q_stride, const __nv_bfloat16* __restrict__ k_cache,
                             const __nv_bfloat16* __restrict__ v_cache, __nv_bfloat16* __restrict__ out, int out_stride,
                             const int* __restrict__ row_seg, const int* __restrict__ row_pos,
                             const int* __restrict__ block_tables, int table_stride, int rows, int heads, int kv_heads,
                             int page_size, int num_pages, int window, float scale_log2, float* __restrict__ part_o,
                             float* __restrict__ part_ml, int* __restrict__ counters, const Fresh fresh) {
    extern __shared__ __align__(128) uint8_t smem_raw[];
    __shared__ int s_cum[FLAT_MAX_ROWS + 1];
    pdl_wait();
    pdl_trigger();
    if (threadIdx.x < 32) flat_prefix(row_pos, rows, window, s_cum);
    __syncthreads();
    const int G = heads / kv_heads;
    const long long all = (long long)kv_heads * s_cum[rows];
    long long at = all * blockIdx.x / gridDim.x;
    const long long end = all * (blockIdx.x + 1) / gridDim.x;
    int lo = 0, hi = rows - 1;                       // the row whose tiles hold position `at`
    while (lo < hi) {
        const int mid = (lo + hi) >> 1;
        if ((long long)kv_heads * s_cum[mid + 1] <= at) lo = mid + 1; else hi = mid;
    }
    int r = lo;
    while (at < end) {
        while ((long long)kv_heads * s_cum[r + 1] <= at) ++r;
        const int tiles_r = s_cum[r + 1] - s_cum[r];
        const long long in_row = at - (long long)kv_heads * s_cum[r];
        const int kvh = (int)(in_row / tiles_r), tile_lo = (int)(in_row % tiles_r);
        const int n = (int)min((long long)(tiles_r - tile_lo), end - at);
        const int P = row_pos[r], first = window > 0 ? max(0, P + 1 - window) : 0;
        const size_t slot = (size_t)r * kv_heads + kvh + blockIdx.x;
        // the blocks whose runs meet this pair follow one another (the host sees to it that no run is empty)
        const long long start = at - tile_lo;
        auto block_of = [&](long long tile) { return (int)(((tile + 1) * gridDim.x + all - 1) / all - 1); };
        const int b_first = block_of(start), parts = block_of(start + tiles_r - 1) - b_first + 1;
        const bool alone = counters != nullptr && parts == 1;       // this block has all of the pair: no partial
        attend<HD>(smem_raw, q, q_stride, k_cache, v_cache, out, out_stride, block_tables + (size_t)row_seg[r] * table_stride,
                   table_stride, num_pages, heads, kv_heads, page_size, scale_log2, r, kvh, P, first, tile_lo, n, alone,
                   part_o + slot * G * HD,
                   (size_t)HD, part_ml + slot * G * 2, (size_t)2, fresh);
        at += n;
        if (counters != nullptr && !alone && last_of_pair(counters + (size_t)r * kv_heads + kvh, parts)) {
            const size_t slot0 = (size_t)r * kv_heads + kvh + b_first;      // the slots of the pair's parts follow one another
            combine_pair<HD>(part_o + slot0 * G * HD, (size_t)G * HD, (size_t)HD, part_ml + slot0 * G * 2, (size_t)G * 2,
                             (size_t)2, parts, G, out + (size_t)r * out_stride + (size_t)kvh * G * HD);
        }
        __syncthreads();                              // shared memory is the next stretch's
    }
}

// out[r, head] from the partials of the blocks whose runs met the pair (r, kv head of the head), in block order
__global__ void attention_combine_flat_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                              __nv_bfloat16* __restrict__ out, int out_stride,
                                              const int* __restrict__ row_pos, int rows, int heads, int kv_heads,
                                              int head_dim, int window, int blocks) {
    constexpr int MAX_PARTS = 64;
    __shared__ int s_cum[FLAT_MAX_ROWS + 1];
    __shared__ float weight[MAX_PARTS];
    __shared__ float inv_total;
    pdl_wait();
    pdl_trigger();
    if (threadIdx.x < 32) flat_prefix(row_pos, rows, window, s_cum);
    __syncthreads();
    const int r = blockIdx.x, head = blockIdx.y, G = heads / kv_heads, kvh = head / G, row = head % G;
    const long long all = (long long)kv_heads * s_cum[rows];
    const int tiles_r = s_cum[r + 1] - s_cum[r];
    const long long start = (long long)kv_heads * s_cum[r] + (long long)kvh * tiles_r;
    auto block_of = [&](long long tile) { return (int)(((tile + 1) * blocks + all - 1) / all - 1); };
    const int b_first = block_of(start), parts = min(MAX_PARTS, block_of(start + tiles_r - 1) - b_first + 1);
    const size_t slot0 = (size_t)r * kv_heads + kvh + b_first;      // the slots of the pair's parts follow one another
    if (threadIdx.x < 32) {
        const int lane = threadIdx.x;
        float ms[2], ls[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int p = lane + 32 * h;
            // a block between the first and the last whose run is empty (more blocks than tiles) wrote nothing
            const long long lo = all * (b_first + p) / blocks, hi = all * (b_first + p + 1) / blocks;
            const bool wrote = p < parts && max(lo, start) < min(hi, start + tiles_r);
            ms[h] = wrote ? part_ml[((slot0 + p) * G + row) * 2] : -INFINITY;
            ls[h] = wrote ? part_ml[((slot0 + p) * G + row) * 2 + 1] : 0.f;
        }
        float M = fmaxf(ms[0], ms[1]);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, o));
        float L = 0.f;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const float w = ms[h] == -INFINITY ? 0.f : exp2f(ms[h] - M);
            weight[lane + 32 * h] = w;
            for (int i = 0; i < 32 && i + 32 * h < parts; ++i) L += __shfl_sync(0xffffffffu, ls[h] * w, i);
        }
        if (lane == 0) inv_total = 1.f / L;
    }
    __syncthreads();
    const float inv = inv_total;
    for (int d = threadIdx.x; d < head_dim; d += blockDim.x) {
        float acc = 0.f;
#pragma unroll 4
        for (int p = 0; p < parts; ++p)
            if (weight[p] != 0.f) acc += part_o[((slot0 + p) * G + row) * head_dim + d] * weight[p];
        out[(size_t)r * out_stride + (size_t)head * head_dim + d] = __float2bfloat16_rn(acc * inv);
    }
}

template <int HD>
void launch_flat(const void* q, int q_stride, const void* k_cache, const void* v_cache, void* out, int out_stride,
                 const int* row_seg, const int* row_pos, const int* block_tables, int table_stride, int rows, int heads,
                 int kv_heads, int page_size, int window, float scale_log2, int blocks, float* part_o, float* part_ml,
                 int* counters, const Fresh& fresh, cudaStream_t stream) {
    const size_t stage_bytes = (size_t)STAGES * 2 * TILE * HD * 2;
    const size_t merge_bytes = ((size_t)WARPS * 16 * HD + WARPS * 16 * 2) * sizeof(float);
    const size_t smem = 16 * HD * 2 + (stage_bytes > merge_bytes ? stage_bytes : merge_bytes);
    auto kern = attention_decode_flat_kernel<HD>;
    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    jllm_launch(kern, dim3(blocks), dim3(THREADS), smem, stream, true, (const __nv_bfloat16*)q, q_stride,
                (const __nv_bfloat16*)k_cache, (const __nv_bfloat16*)v_cache, (__nv_bfloat16*)out, out_stride, row_seg,
                row_pos, block_tables, table_stride, rows, heads, kv_heads, page_size, jllm_pool_pages(), window, scale_log2,
                part_o, part_ml, counters, fresh);
    if (counters == nullptr)
        jllm_launch(attention_combine_flat_kernel, dim3(rows, heads), dim3(128), 0, stream, true, (const float*)part_o,
                    (const float*)part_ml, (__nv_bfloat16*)out, out_stride, row_pos, rows, heads, kv_heads, HD, window,
                    blocks);
}

template <int HD>
void launch(const void* q, int q_stride, const void* k_cache, const void* v_cache, void* out, int out_stride,
            const int* row_seg, const int* row_pos, const int* block_tables, int table_stride, int rows, int heads,
            int kv_heads, int page_size, int window, float scale_log2, int splits, float* part_o, float* part_ml,
            int* counters, const Fresh& fresh, cudaStream_t stream) {
    const size_t stage_bytes = (size_t)STAGES * 2 * TILE * HD * 2;
    const size_t merge_bytes = ((size_t)WARPS * 16 * HD + WARPS * 16 * 2) * sizeof(float);
    const size_t smem = 16 * HD * 2 + (stage_bytes > merge_bytes ? stage_bytes : merge_bytes);
    auto kern = attention_decode_staged_kernel<HD>;
    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    jllm_launch(kern, dim3(rows, kv_heads, splits), dim3(THREADS), smem, stream, true,
        (const __nv_bfloat16*)q, q_stride, (const __nv_bfloat16*)k_cache, (const __nv_bfloat16*)v_cache,
        (__nv_bfloat16*)out, out_stride, row_seg, row_pos, block_tables, table_stride, heads, kv_heads, page_size,
        jllm_pool_pages(), window, scale_log2, splits, part_o, part_ml, counters, fresh);
}

// The library's pair counters on the current device (nullptr: the combine kernels run instead).
inline int* pair_counters() {
    static int* ptrs[64] = {};
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    if (ptrs[dev] == nullptr) {
        void* p = nullptr;
        if (cudaGetSymbolAddress(&p, g_pair_counters) != cudaSuccess) {
            cudaGetLastError();
            return nullptr;
        }
        ptrs[dev] = static_cast<int*>(p);
    }
    return ptrs[dev];
}

}  // namespace staged
