// Choosing the next token on the device: argmax (lowest index among equal maxima) and sampling
// with temperature, top-k, top-p and min-p, one thread block per row of logits.
//
// Sampling follows the reference's order (src/main/java/org/robomiri/jllm/sampling/Sampler.java:352-432):
// candidates = the top-k largest logits (all when top-k is off); weight = exp((logit - max) / T);
// top-p keeps the shortest prefix, in descending order, whose share of the candidates' mass reaches
// top_p; min-p zeroes weights below min_p (the largest weight is 1); then r = u * total and the first
// candidate whose running sum exceeds r is drawn. With top-k and top-p both off the walk is in index
// order, otherwise in descending order of logit (lower index first among equals).
//
// Nothing is sorted. Logit and index make one 64-bit key that orders the vocabulary strictly
// (higher logit first, then lower index); "the k-th key", "the key where the mass reaches p" and
// "the key where the running sum passes r" are each found by bisection over the key with a block-wide
// count or sum per probe. With 0 < top-k <= 1024 the candidates are first gathered into shared memory.
// The uniform number u in [0, 1) comes from the host, one per row and step.
#include "common.cuh"

namespace {

constexpr int THREADS = 1024;
constexpr int MAX_SHARED_CANDIDATES = 1024;

__device__ __forceinline__ unsigned long long order_key(float logit, int index) {
    unsigned int b = __float_as_uint(logit);
    b = (b & 0x80000000u) ? ~b : (b | 0x80000000u);
    return ((unsigned long long)b << 32) | (unsigned int)(~(unsigned int)index);
}

__device__ __forceinline__ double block_sum_double(double v, double* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        double t = lane < (THREADS >> 5) ? scratch[lane] : 0.0;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}

struct ArgBest {
    float v;
    int i;
};
__device__ __forceinline__ ArgBest better(ArgBest a, ArgBest b) {
    return (b.v > a.v || (b.v == a.v && b.i < a.i)) ? b : a;
}

__device__ int block_argmax(const float* __restrict__ row, int vocab, ArgBest* scratch) {
    ArgBest best{-INFINITY, 0x7fffffff};
    for (int i = threadIdx.x; i < vocab; i += THREADS) best = better(best, ArgBest{row[i], i});
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        ArgBest other{__shfl_xor_sync(0xffffffffu, best.v, o), __shfl_xor_sync(0xffffffffu, best.i, o)};
        best = better(best, other);
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    __syncthreads();
    if (lane == 0) scratch[warp] = best;
    __syncthreads();
    if (warp == 0) {
        ArgBest t = lane < (THREADS >> 5) ? scratch[lane] : ArgBest{-INFINITY, 0x7fffffff};
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            ArgBest other{__shfl_xor_sync(0xffffffffu, t.v, o), __shfl_xor_sync(0xffffffffu, t.i, o)};
            t = better(t, other);
        }
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    const int r = scratch[32].i;
    return r == 0x7fffffff ? 0 : r;  // a row of NaNs: index 0, as a plain scan from index 0 gives
}

__global__ void __launch_bounds__(THREADS) argmax_kernel(const float* __restrict__ logits, int ld, int vocab,
                                                          int* __restrict__ out) {
    __shared__ ArgBest scratch[33];
    pdl_wait();
    pdl_trigger();
    const int t = block_argmax(logits + (size_t)blockIdx.x * ld, vocab, scratch);
    if (threadIdx.x == 0) out[blockIdx.x] = t;
}

// The same with a row dealt out over `parts` blocks (few rows of a long vocabulary: one block per row leaves the GPU
// to a handful of SMs, each reading 600 KB alone). Block (row, part) scans its stretch with 16-byte loads and parks its
// best (value, index); the block of a row that finds itself last at the row's counter (after a fence; nobody waits)
// takes the best of the parts. "Better" is a total order (higher value, then lower index), so the result does not depend
// on who came when. Scratch and counters belong to the library (zero when it is loaded, left at zero): launches on one
// device must not overlap.
constexpr int ARGMAX_MAX_ROWS = 4096, ARGMAX_MAX_PARTS = 32;
__device__ ArgBest g_argmax_parts[ARGMAX_MAX_ROWS * ARGMAX_MAX_PARTS];
__device__ int g_argmax_counters[ARGMAX_MAX_ROWS];

__global__ void __launch_bounds__(256) argmax_parts_kernel(const float* __restrict__ logits, int ld, int vocab, int parts,
                                                           int* __restrict__ out) {
    __shared__ ArgBest scratch[9];
    __shared__ int s_last;
    pdl_wait();
    pdl_trigger();
    const int r = blockIdx.x, part = blockIdx.y, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const float* row = logits + (size_t)r * ld;
    // stretches of whole groups of four columns (the rows are 16-byte aligned: the host sees to it)
    const int groups = (vocab + 3) >> 2, g_lo = (int)((long long)groups * part / parts),
              g_hi = (int)((long long)groups * (part + 1) / parts);
    ArgBest best{-INFINITY, 0x7fffffff};
    for (int g = g_lo + threadIdx.x; g < g_hi; g += 256) {
        const int i = 4 * g;
        if (i + 3 < vocab) {
            const float4 v = *reinterpret_cast<const float4*>(row + i);
            best = better(best, ArgBest{v.x, i});
            best = better(best, ArgBest{v.y, i + 1});
            best = better(best, ArgBest{v.z, i + 2});
            best = better(best, ArgBest{v.w, i + 3});
        } else {
            for (int j = i; j < vocab; ++j) best = better(best, ArgBest{row[j], j});
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        ArgBest other{__shfl_xor_sync(0xffffffffu, best.v, o), __shfl_xor_sync(0xffffffffu, best.i, o)};
        best = better(best, other);
    }
    if (lane == 0) scratch[warp] = best;
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < 8; ++w) best = better(best, scratch[w]);
        g_argmax_parts[r * ARGMAX_MAX_PARTS + part] = best;
        __threadfence();
        const int seen = atomicAdd(&g_argmax_counters[r], 1);
        s_last = seen == parts - 1;
        if (s_last) g_argmax_counters[r] = 0;
    }
    __syncthreads();
    if (s_last && warp == 0) {
        __threadfence();
        ArgBest t{-INFINITY, 0x7fffffff};
        if (lane < parts) {
            t.v = __ldcg(&g_argmax_parts[r * ARGMAX_MAX_PARTS + lane].v);
            t.i = __ldcg(&g_argmax_parts[r * ARGMAX_MAX_PARTS + lane].i);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            ArgBest other{__shfl_xor_sync(0xffffffffu, t.v, o), __shfl_xor_sync(0xffffffffu, t.i, o)};
            t = better(t, other);
        }
        if (lane == 0) out[r] = t.i == 0x7fffffff ? 0 : t.i;      // a row of NaNs: index 0
    }
}

__global__ void __launch_bounds__(THREADS)
sample_kernel(const float* __restrict__ logits, int ld, int vocab, const float* __restrict__ temperature,
              const int* __restrict__ top_k, const float* __restrict__ top_p, const float* __restrict__ min_p,
              const double* __restrict__ uniform, int* __restrict__ out) {
    __shared__ ArgBest arg_scratch[33];
    __shared__ double dscratch[33];
    __shared__ float cand_logit[MAX_SHARED_CANDIDATES];
    __shared__ int cand_index[MAX_SHARED_CANDIDATES];
    __shared__ int cand_count;
    __shared__ double chunk_prefix[THREADS + 1];
    __shared__ int chosen;

    const int row_id = blockIdx.x, tid = threadIdx.x;
    const float* row = logits + (size_t)row_id * ld;
    const float T = temperature[row_id];
    const int k = top_k[row_id];
    const float p = top_p[row_id], mp = min_p[row_id];
    const int best = block_argmax(row, vocab, arg_scratch);
    if (T == 0.f || k == 1) {
        if (tid == 0) out[row_id] = best;
        return;
    }
    const float max_logit = row[best];
    const float inv_t = 1.f / T;
    const double u = uniform[row_id];
    auto weight = [&](float l) -> float {
        const float w = expf((l - max_logit) * inv_t);
        return w;
    };
    const bool limited_k = k > 0 && k < vocab;

    if (!limited_k && !(p < 1.f)) {
        // index order: each thread owns a contiguous run of the vocabulary
        const int per = (vocab + THREADS - 1) / THREADS;
        const int lo = min(vocab, tid * per), hi = min(vocab, lo + per);
        double mine = 0.0;
        for (int i = lo; i < hi; ++i) {
            const float w = weight(row[i]);
            mine += (mp > 0.f && w < mp) ? 0.f : w;
        }
        chunk_prefix[tid + 1] = mine;
        if (tid == 0) {
            chunk_prefix[0] = 0.0;
            chosen = -1;
        }
        __syncthreads();
        if (tid == 0)
            for (int i = 1; i <= THREADS; ++i) chunk_prefix[i] += chunk_prefix[i - 1];
        __syncthreads();
        const double r = u * chunk_prefix[THREADS];
        if (chunk_prefix[tid] <= r && r < chunk_prefix[tid + 1]) {
            double acc = chunk_prefix[tid];
            int pick = -1;
            for (int i = lo; i < hi && pick < 0; ++i) {
                const float w = weight(row[i]);
                acc += (mp > 0.f && w < mp) ? 0.f : w;
                if (r < acc) pick = i;
            }
            if (pick >= 0) chosen = pick;
        }
        __syncthreads();
        if (tid == 0) out[row_id] = chosen >= 0 ? chosen : best;
        return;
    }

    // ---- descending order through the 64-bit key ----
    const unsigned long long key_max = order_key(max_logit, best);
    unsigned long long key_k = 0;  // candidates: key >= key_k
    if (limited_k) {
        // the k-th largest key: the largest K with count{key >= K} >= k
        unsigned long long lo = 0, hi = key_max;
        while (lo < hi) {
            const unsigned long long mid = lo + ((hi - lo + 1) >> 1);
            double c = 0.0;
            for (int i = tid; i < vocab; i += THREADS) c += order_key(row[i], i) >= mid ? 1.0 : 0.0;
            c = block_sum_double(c, dscratch);
            if (c >= (double)k) lo = mid; else hi = mid - 1;
        }
        key_k = lo;
    }
    const bool in_shared = limited_k && k <= MAX_SHARED_CANDIDATES;
    if (in_shared) {
        if (tid == 0) cand_count = 0;
        __syncthreads();
        for (int i = tid; i < vocab; i += THREADS) {
            const float l = row[i];
            if (order_key(l, i) >= key_k) {
                const int at = atomicAdd(&cand_count, 1);
                if (at < MAX_SHARED_CANDIDATES) {
                    cand_logit[at] = l;
                    cand_index[at] = i;
                }
            }
        }
        __syncthreads();
    }
    const int n = in_shared ? min(cand_count, MAX_SHARED_CANDIDATES) : vocab;
    // mass of the candidates with key >= K (and, if `kept_only`, weight not zeroed by min-p), all above key_cut
    auto mass_from = [&](unsigned long long K, unsigned long long key_cut, bool apply_min_p) -> double {
        double s = 0.0;
        for (int j = tid; j < n; j += THREADS) {
            const float l = in_shared ? cand_logit[j] : row[j];
            const int i = in_shared ? cand_index[j] : j;
            const unsigned long long key = order_key(l, i);
            if (key >= K && key >= key_cut) {
                const float w = weight(l);
                s += (apply_min_p && mp > 0.f && w < mp) ? 0.f : w;
            }
        }
        return block_sum_double(s, dscratch);
    };
    unsigned long long key_cut = key_k;
    if (p < 1.f) {
        const double total = mass_from(0, key_k, false);
        const double want = (double)p * total;
        unsigned long long lo = key_k, hi = key_max;  // the largest K with mass{key >= K} >= want
        while (lo < hi) {
            const unsigned long long mid = lo + ((hi - lo + 1) >> 1);
            if (mass_from(mid, key_k, false) >= want) lo = mid; else hi = mid - 1;
        }
        key_cut = lo;
    }
    const double total_kept = mass_from(0, key_cut, true);
    const double r = u * total_kept;
    unsigned long long lo = key_cut, hi = key_max;  // the largest K with kept mass{key >= K} > r
    while (lo < hi) {
        const unsigned long long mid = lo + ((hi - lo + 1) >> 1);
        if (mass_from(mid, key_cut, true) > r) lo = mid; else hi = mid - 1;
    }
    if (tid == 0) {
        const int token = (int)(~(unsigned int)(lo & 0xffffffffull));
        out[row_id] = (token >= 0 && token < vocab) ? token : best;
    }
}

}  // namespace

JLLM_EXPORT int jllm_argmax(const float* logits, int ld, int rows, int vocab, int* out, cudaStream_t stream) {
    JLLM_REQUIRE(rows >= 0 && vocab > 0 && ld >= vocab, "argmax: rows=%d vocab=%d ld=%d", rows, vocab, ld);
    if (rows == 0) return JLLM_OK;
    // few rows: as many blocks per row as give every SM about two, each with 4,096 columns or more
    const int sms = jllm_device_sm_count() > 0 ? jllm_device_sm_count() : 1;
    int parts = (2 * sms + rows - 1) / rows;
    if (parts > ARGMAX_MAX_PARTS) parts = ARGMAX_MAX_PARTS;
    if (parts > vocab / 4096) parts = vocab / 4096;
    if (parts >= 2 && rows <= ARGMAX_MAX_ROWS && ld % 4 == 0 && ((uintptr_t)logits % 16) == 0) {
        jllm_launch(argmax_parts_kernel, dim3(rows, parts), dim3(256), 0, stream, true, logits, ld, vocab, parts, out);
        return jllm_check_launch("argmax");
    }
    jllm_launch(argmax_kernel, dim3(rows), dim3(THREADS), 0, stream, true, logits, ld, vocab, out);
    return jllm_check_launch("argmax");
}

JLLM_EXPORT int jllm_sample(const float* logits, int ld, int rows, int vocab, const float* temperature,
                            const int* top_k, const float* top_p, const float* min_p, const double* uniform, int* out,
                            cudaStream_t stream) {
    JLLM_REQUIRE(rows >= 0 && vocab > 0 && ld >= vocab, "sample: rows=%d vocab=%d ld=%d", rows, vocab, ld);
    if (rows == 0) return JLLM_OK;
    sample_kernel<<<rows, THREADS, 0, stream>>>(logits, ld, vocab, temperature, top_k, top_p, min_p, uniform, out);
    return jllm_check_launch("sample");
}
