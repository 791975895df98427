// The epilogue of the tcgen05 products, shared by their kernels: 32 float32 accumulator values per thread (32
// consecutive columns of ONE row; the lanes of a warp hold 32 consecutive rows, as tcgen05.ld 32x32b gives them) get the
// bias / the residual / SwiGLU and are stored as float32 or bfloat16, only where they lie inside [M, N].
#pragma once
#include "tcgen05_common.cuh"

namespace tc {

constexpr int STAGING_ROW = 36;        // floats of a staged row of 32 values: 16-byte aligned, and rows fall in other banks
constexpr int STAGING_WARP_FLOATS = 32 * STAGING_ROW;      // shared memory a warp needs for `staged`
constexpr int BULK_WARP_BYTES = 32 * 32 * 4;                // ... and for `bulk`: a 32 x 32 block, 1024-byte aligned

template <typename Tout>
struct TileEpilogue {
    Tout* out;
    int ldo, M, N, accumulate, has_bias, swiglu;
    VecRef bias;
    // not null: a float32 output written (or added into) by tiled bulk copies of 32 x 32 blocks from shared memory,
    // which the copy engine clips to [M, N]; the residual add is then done where the data lies (in L2), the SM neither
    // loads the old values nor waits for them
    const CUtensorMap* out_map;

    // The warp's 32 x 32 block leaves through shared memory by one bulk copy: rows of 128 bytes whose 16-byte chunk c
    // lies at chunk position c ^ (row & 7) (the 128-byte swizzle of the output's tensor map: a quarter warp's 16-byte
    // stores fall into eight different chunks). `stage`: the warp's 4 KB of shared memory, 1024-byte aligned. The
    // copy before this one must have read the buffer; `bulk_done` waits for the last ones to be written.
    __device__ __forceinline__ void bulk(uint32_t (&v)[32], int row0, int lane, int n_base, uint32_t stage) const {
        if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
        __syncwarp();
#pragma unroll
        for (int c = 0; c < 8; ++c) {
            float4 x = make_float4(__uint_as_float(v[4 * c]), __uint_as_float(v[4 * c + 1]), __uint_as_float(v[4 * c + 2]),
                                   __uint_as_float(v[4 * c + 3]));
            if (has_bias) {      // (columns beyond N are clipped by the copy; the bias is not read there)
                const int n = n_base + 4 * c;
                if (n < N) x.x += bias[n];
                if (n + 1 < N) x.y += bias[n + 1];
                if (n + 2 < N) x.z += bias[n + 2];
                if (n + 3 < N) x.w += bias[n + 3];
            }
            asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(stage + lane * 128 + ((c ^ (lane & 7)) << 4)),
                         "f"(x.x), "f"(x.y), "f"(x.z), "f"(x.w)
                         : "memory");
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (lane == 0) {
            if (accumulate)
                asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.bulk_group [%0, {%2, %3}], [%1];"
                             ::"l"(out_map), "r"(stage), "r"(n_base), "r"(row0)
                             : "memory");
            else
                asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
                             ::"l"(out_map), "r"(stage), "r"(n_base), "r"(row0)
                             : "memory");
            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        }
    }
    // before the kernel ends: this warp's bulk copies have been written
    __device__ __forceinline__ void bulk_done(int lane) const {
        if (out_map != nullptr && lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
    }

    // All 32 rows of the warp lie inside the matrix and float32 rows can be accessed 16 bytes at a time: the block goes
    // through shared memory (`staged`).
    __device__ __forceinline__ bool rows_whole(int row0) const {
        return !swiglu && row0 + 32 <= M && sizeof(Tout) == 4 && (ldo & 3) == 0 && (((uintptr_t)out) & 15u) == 0;
    }

    // Through shared memory, so that a warp's accesses are whole lines: a thread holds 32 values of ONE row, and
    // written (or added) from there a warp's instruction would touch 32 rows with 16 bytes each. The warp parks
    // its 32 x 32 block and takes it back four rows at a time, eight threads to a row: four full 128-byte lines
    // per instruction, and all eight loads of a residual add are on their way before the first store.
    __device__ __forceinline__ void staged(uint32_t (&v)[32], int row0, int lane, int n_base, float* mine) const {
        float4* srow = reinterpret_cast<float4*>(mine + lane * STAGING_ROW);
#pragma unroll
        for (int j = 0; j < 8; ++j)
            srow[j] = make_float4(__uint_as_float(v[4 * j]), __uint_as_float(v[4 * j + 1]), __uint_as_float(v[4 * j + 2]),
                                  __uint_as_float(v[4 * j + 3]));
        __syncwarp();
        const int sub = lane >> 3, c4 = (lane & 7) * 4;
        float4 bv = make_float4(0.f, 0.f, 0.f, 0.f);
        if (has_bias)
            bv = make_float4(bias[n_base + c4], bias[n_base + c4 + 1], bias[n_base + c4 + 2], bias[n_base + c4 + 3]);
        float* d0 = reinterpret_cast<float*>(out) + (size_t)(row0 + sub) * ldo + n_base + c4;
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
    }

    // v: columns [n_base, n_base + 32) of row row0 + lane. `whole` = rows_whole(row0); `mine`: the warp's staging
    // (STAGING_WARP_FLOATS floats, or BULK_WARP_BYTES aligned to 1024 bytes with an output map).
    __device__ __forceinline__ void store(uint32_t (&v)[32], int row0, int lane, int n_base, bool whole, float* mine) const {
        const int row = row0 + lane;
        if (out_map != nullptr) {
            if (row0 < M && n_base < N) bulk(v, row0, lane, n_base, smem_u32(mine));
        } else if (whole && n_base + 32 <= N) {
            staged(v, row0, lane, n_base, mine);
        } else if (row < M && swiglu) {
            // columns come in blocks of 16: 8 gate columns, then the 8 up columns of the same hidden units
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
    }
};

}  // namespace tc
