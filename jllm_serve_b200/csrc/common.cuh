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

#define JLLM_REQUIRE(cond, ...)                                   \
    do {                                                          \
        if (!(cond)) return jllm_fail(JLLM_BAD_ARGUMENT, __VA_ARGS__); \
    } while (0)

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
// The decode products re-read their activations through L1 (every block reads all of them): behind a tcgen05
// product a 16 x 4096 x 12288 product took 47 us as a dependent launch and 22 us launched plainly, and a decode
// step at batch 16 6.8 ms instead of 5.6. A launch that says it wants L1 (LAUNCH_DEPENDENT_WANTS_L1) is
// therefore made plainly when a large-shared-memory kernel has been launched since the last plain launch.
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
