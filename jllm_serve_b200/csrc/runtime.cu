// Error reporting of the kernel library, and what the host asks about the device.
#include "common.cuh"

#include <cstdlib>
#include <cstring>

namespace {
thread_local char g_error[1024] = "";
}

int jllm_fail(int code, const char* fmt, ...) {
    va_list args;
    va_start(args, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, args);
    va_end(args);
    return code;
}

int jllm_check_launch(const char* what) {
    const cudaError_t e = cudaGetLastError();
    if (e == cudaSuccess) return JLLM_OK;
    return jllm_fail(JLLM_CUDA_ERROR, "%s: %s (%s)", what, cudaGetErrorString(e), cudaGetErrorName(e));
}

namespace {
int g_pdl = -1;
}

bool jllm_pdl_enabled() {
    if (g_pdl < 0) {
        const char* e = getenv("JLLM_B200_PDL");
        g_pdl = (e && e[0] == '0') ? 0 : 1;
    }
    return g_pdl == 1;
}

namespace {
bool g_little_l1 = false;      // a kernel with a large shared-memory allocation was launched since the last plain launch
}

bool jllm_launch_overlaps(size_t dynamic_smem, int how) {
    bool overlaps = how != LAUNCH_PLAIN && jllm_pdl_enabled();
    if (how == LAUNCH_DEPENDENT_WANTS_L1 && g_little_l1) overlaps = false;
    if (!overlaps) g_little_l1 = false;                     // the SMs drain before this kernel starts
    if (dynamic_smem > 48 * 1024) g_little_l1 = true;       // what needs the opt-in allocation shrinks L1
    return overlaps;
}

// What jllm_launch would decide for a kernel with this much dynamic shared memory launched this way (0 plain,
// 1 dependent, 2 dependent and wants L1), with the same record kept: 1 = it overlaps its predecessor. For tests
// of the rule; launches nothing.
JLLM_EXPORT int jllm_launch_plan(long long dynamic_smem, int how) {
    return jllm_launch_overlaps((size_t)dynamic_smem, how) ? 1 : 0;
}

// 1 = kernels of a step are launched as programmatic dependents of their predecessors (default), 0 = plainly.
JLLM_EXPORT void jllm_set_pdl(int on) { g_pdl = on ? 1 : 0; }

JLLM_EXPORT const char* jllm_last_error() { return g_error; }

// The library is built for one architecture only. Returns 0 if the current device can run it.
JLLM_EXPORT int jllm_check_device() {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return jllm_fail(JLLM_CUDA_ERROR, "no CUDA device: %s", cudaGetErrorString(e));
    cudaDeviceProp prop;
    e = cudaGetDeviceProperties(&prop, dev);
    if (e != cudaSuccess) return jllm_fail(JLLM_CUDA_ERROR, "cudaGetDeviceProperties: %s", cudaGetErrorString(e));
    if (prop.major != 10)
        return jllm_fail(JLLM_UNSUPPORTED, "the kernels are built for sm_100a (B200); device %d is %s, sm_%d%d", dev,
                         prop.name, prop.major, prop.minor);
    return JLLM_OK;
}

// The SMs of the current device, asked once per device (0 if it cannot be asked). Grids and split counts are sized
// from this, never from a number written into the code.
int jllm_device_sm_count() {
    static int counts[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 0;
    if (counts[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess) counts[dev] = n;
    }
    return counts[dev];
}

// Pages of the cache pool that the launches which follow read and write (0 = not known). Only the build with bounds
// checks uses it: there every page id is compared with it and every cache slot with pages x page size.
namespace {
int g_pool_pages = 0;
}
int jllm_pool_pages() { return g_pool_pages; }
JLLM_EXPORT void jllm_set_pool_pages(int pages) { g_pool_pages = pages > 0 ? pages : 0; }

// 1 if this library was built with bounds checks (-DJLLM_CHECK_BOUNDS), else 0.
JLLM_EXPORT int jllm_checks_bounds() { return kCheckBounds ? 1 : 0; }

JLLM_EXPORT int jllm_sm_count() { return jllm_device_sm_count(); }

JLLM_EXPORT int jllm_abi_version() { return 1; }
