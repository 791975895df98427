// One head of a query or key in the registers of a warp: RMSNorm over the head and rotate-half RoPE over its whole
// width, for head sizes 64 * V. Lane l owns V neighbouring values of the first half (a) and their partners in the
// second half (b), so the rotation needs no exchange and the sum of squares is a warp shuffle. Shared by the row-wise
// kernel (`qk_norm_rope_store`) and the decode attention that does this work for its own row, so that a key is the same
// bits whichever of them made it.
#pragma once
#include "common.cuh"

// The scale of an RMSNorm, taken in double from a float mean, as the reference does.
__device__ __forceinline__ float rms_scale(float sum_squares, int n, float eps) {
    const float mean = sum_squares / (float)n + eps;
    return (float)(1.0 / sqrt((double)mean));
}

// a[i] = x[lane * V + i], b[i] = x[32 * V + lane * V + i]; cos_row / sin_row: the 32 * V angles of the row's position
template <int V>
__device__ __forceinline__ void head_norm_rope(float (&a)[V], float (&b)[V], int lane, int use_norm, float eps, VecRef gain,
                                               const float* __restrict__ cos_row, const float* __restrict__ sin_row) {
    constexpr int HD = 64 * V, HALF = 32 * V;
    if (use_norm) {
        float ss = 0.f;
#pragma unroll
        for (int i = 0; i < V; ++i) ss = fmaf(a[i], a[i], ss);
#pragma unroll
        for (int i = 0; i < V; ++i) ss = fmaf(b[i], b[i], ss);
        ss = warp_sum(ss);
        const float s = rms_scale(ss, HD, eps);
#pragma unroll
        for (int i = 0; i < V; ++i) {
            a[i] = __fmul_rn(__fmul_rn(a[i], s), gain[lane * V + i]);
            b[i] = __fmul_rn(__fmul_rn(b[i], s), gain[HALF + lane * V + i]);
        }
    }
    const float* c = cos_row + lane * V;
    const float* sn = sin_row + lane * V;
#pragma unroll
    for (int i = 0; i < V; ++i) {
        const float x0 = a[i], x1 = b[i];
        a[i] = __fsub_rn(__fmul_rn(x0, c[i]), __fmul_rn(x1, sn[i]));
        b[i] = __fadd_rn(__fmul_rn(x1, c[i]), __fmul_rn(x0, sn[i]));
    }
}
