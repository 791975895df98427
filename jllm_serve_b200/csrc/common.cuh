// Shared pieces of the sm_100a kernels: element types, error reporting, block reductions.
//
// Every exported launcher returns 0 on success and a non-zero code otherwise; the text of the
// last error of the calling thread is read with jllm_last_error(). Launchers never allocate:
// the caller passes inputs, outputs and (where a kernel needs it) scratch memory.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdarg>
#include <cstdio>

#define JLLM_EXPORT extern "C" __attribute__((visibility("default")))

enum JllmDtype : int { JLLM_F32 = 0, JLLM_BF16 = 1 };

enum JllmError : int {
    JLLM_OK = 0,
    JLLM_BAD_ARGUMENT = 1,   // a size or option the kernels refuse
    JLLM_CUDA_ERROR = 2,     // a CUDA call failed
    JLLM_UNSUPPORTED = 3,    // a combination that is not built
};

int jllm_fail(int code, const char* fmt, ...);
int jllm_check_launch(const char* what);
int jllm_device_sm_count();      // SMs of the current device (asked once), 0 if unknown
int jllm_pool_pages();           // pages of the cache pool in use, as the host declared them (0 = unknown)

#define JLLM_REQUIRE(cond, ...)                                   \
    do {                                                          \
        if (!(cond)) return jllm_fail(JLLM_BAD_ARGUMENT, __VA_ARGS__); \
    } while (0)

// ---- bounds checks of what the kernels read through tables (a build with -DJLLM_CHECK_BOUNDS) --------------------
// The kernels follow page tables, slot lists and token ids that the host packed. In the ordinary build they trust
// them. In the checked build (a second library, chosen with JLLM_B200_CHECK_BOUNDS=1) every table index, page id,
// cache slot and token id is compared with its limit first; an access that would leave its array is SKIPPED (a key
// then counts as absent, a write is dropped) and the first such case is recorded in a word of this translation unit:
// {what, index, limit, how many}. Nothing traps and nothing hangs: the host reads the words after the step
// (`jllm_bounds_error_<file>`) and raises. A limit of 0 or less means "not known to this caller": only negative
// indices are caught then.
enum : int { BOUNDS_TABLE_INDEX = 1, BOUNDS_PAGE = 2, BOUNDS_SLOT = 3, BOUNDS_TOKEN = 4, BOUNDS_ROW = 5 };
#ifdef JLLM_CHECK_BOUNDS
constexpr bool kCheckBounds = true;
static __device__ int jllm_bounds_word[4];
__device__ __noinline__ static void jllm_bounds_record(int what, long long index, long long limit) {
    if (atomicAdd(&jllm_bounds_word[3], 1) == 0) {
        jllm_bounds_word[0] = what;
        jllm_bounds_word[1] = (int)max(-2147483647ll, min(2147483647ll, index));
        jllm_bounds_word[2] = (int)max(-2147483647ll, min(2147483647ll, limit));
    }
}
#define JLLM_BOUNDS_READER(file)                                                                   \
    JLLM_EXPORT int jllm_bounds_error_##file(int* out4) {                                          \
        int zero[4] = {0, 0, 0, 0};                                                                \
        if (cudaMemcpyFromSymbol(out4, jllm_bounds_word, sizeof(zero)) != cudaSuccess) return JLLM_CUDA_ERROR; \
        if (out4[3] && cudaMemcpyToSymbol(jllm_bounds_word, zero, sizeof(zero)) != cudaSuccess) return JLLM_CUDA_ERROR; \
        return JLLM_OK;                                                                            \
    }
#else
constexpr bool kCheckBounds = false;
#define JLLM_BOUNDS_READER(file)                                  \
    JLLM_EXPORT int jllm_bounds_error_##file(int* out4) {         \
        out4[0] = out4[1] = out4[2] = out4[3] = 0;                \
        return JLLM_OK;                                           \
    }
#endif

// True if `index` may be used; always true in the ordinary build (the check compiles to nothing).
__device__ __forceinline__ bool jllm_in_bounds(long long index, long long limit, int what) {
#ifdef JLLM_CHECK_BOUNDS
    if (index < 0 || (limit > 0 && index >= limit)) {
        jllm_bounds_record(what, index, limit);
        return false;
    }
#endif
    return true;
}

// The page of block `b` of a request's table; in the checked build -1 if the block lies outside the table's row or the
// page outside the pool (the caller then skips the access).
__device__ __forceinline__ long long jllm_page_of(const int* __restrict__ table, int b, int table_len, int num_pages) {
#ifdef JLLM_CHECK_BOUNDS
    if (!jllm_in_bounds(b, table_len, BOUNDS_TABLE_INDEX)) return -1;
    const int page = table[b];
    return jllm_in_bounds(page, num_pages, BOUNDS_PAGE) ? page : -1;
#else
    return table[b];
#endif
}

// ---- programmatic dependent launch ---------------------------------------------------------------------
// A decode step is a chain of some hundreds of short kernels. Launched the ordinary way each one starts
// only when its predecessor has drained, and its own ramp-up (block scheduling, first loads) is dead time.
// With programmatic dependent launch the next kernel's blocks become resident while the predecessor still
// runs: they may do work that does not depend on it (a matrix product fetches its first weights), then
// wait with pdl_wait() until the predecessor has completed and its writes are visible. Every kernel calls
// pdl_wait() before it reads anything a predecessor wrote or writes anything a predecessor may read, and
// only then pdl_trigger(), so at most one successor is resident early. Without the launch attribute both
// calls return at once.
//
// One thing limits this. An SM cannot change how its memory is split between shared memory and L1 while blocks
// are resident on it. A kernel whose blocks arrive while a predecessor with a large shared-memory allocation (the
// staged decode attention, the tcgen05 kernels) still holds the SM runs with that predecessor's split, that is
// with little L1, and so does every kernel that overlaps it in turn, until one launch waits for the SMs to drain.
// The row kernel of the decode products re-reads its activations through L1 (every block reads all of them) and
// runs at half its speed that way. A launch that says it wants L1 (LAUNCH_DEPENDENT_WANTS_L1) is therefore made
// plainly when a large-shared-memory kernel has been launched since the last plain launch.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

bool jllm_pdl_enabled();
enum : int { LAUNCH_PLAIN = 0, LAUNCH_DEPENDENT = 1, LAUNCH_DEPENDENT_WANTS_L1 = 2 };
bool jllm_launch_overlaps(size_t dynamic_smem, int how);     // decides, and keeps the record the decision needs

template <typename... KArgs, typename... Args>
inline cudaError_t jllm_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                               int how, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = jllm_launch_overlaps(smem, how) ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// ---- element access: everything is computed in float -------------------------------------------------

__device__ __forceinline__ float to_float(float v) { return v; }
__device__ __forceinline__ float to_float(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_float(float v);
template <> __device__ __forceinline__ float from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// A vector (gain, bias) whose stored type is known only at run time.
struct VecRef {
    const void* p;
    int dtype;
    __device__ __forceinline__ float operator[](int i) const {
        return dtype == JLLM_F32 ? static_cast<const float*>(p)[i]
                                 : __bfloat162float(static_cast<const __nv_bfloat16*>(p)[i]);
    }
};

// ---- reductions with a fixed order: the result of a row never depends on what else is in the batch ----

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over a block of up to 1024 threads; every thread gets the result. `scratch` holds 33 floats.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < warps ? scratch[lane] : 0.f;
        t = warp_sum(t);
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}

__device__ __forceinline__ float block_max(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = (blockDim.x + 31) >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < warps ? scratch[lane] : -INFINITY;
        t = warp_max(t);
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}
