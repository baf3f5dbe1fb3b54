// Shared declarations of the flashgs_b200 CUDA library (sm_100a).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/flashgs_b200.h"

#define FGS_ABI_VERSION 3

namespace fgs {

constexpr unsigned FULL_MASK = 0xffffffffu;

// Device address of the per-device status word (an OR of FGS_ERR_* bits raised by
// kernels). Resolved once per device; returns nullptr if the lookup failed.
int* device_status_ptr();

// Launch-error check shared by the entry points: returns FGS_OK or FGS_ERR_CUDA.
inline int launch_status()
{
    return cudaGetLastError() == cudaSuccess ? FGS_OK : FGS_ERR_CUDA;
}

// Host-side camera block handed to the preprocess kernel by value.
// view/proj are column-major (m[4*c + r]); see fgs_view_proj_matrices().
struct PreCam {
    float view[16];
    float proj[16];
    float cam[3];
    float tan_fovx, tan_fovy, focal_x, focal_y;
    int W, H, block_x, block_y, grid_x, grid_y, row_begin, row_end;
    int cull_columns;   // 1: bound each row's column range in closed form before the exact tile test
};

__device__ __forceinline__ unsigned lane_id() { return threadIdx.x & 31u; }
__device__ __forceinline__ unsigned lanemask_lt()
{
    unsigned m;
    asm("mov.u32 %0, %%lanemask_lt;" : "=r"(m));
    return m;
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// ---- chained launches (programmatic dependent launch) ----
// The kernels of a frame follow one another on one stream, each needing the one before it complete. Launched with the
// programmatic-serialization attribute, a kernel's blocks may become resident while the kernel before it is still
// draining -- once every block of that kernel has started and executed chain_release() -- and stop at chain_wait()
// until it has completed and its writes are visible. What overlaps is launch latency and ramp-up, nothing else:
// chain_wait() is the first statement of every kernel launched this way, so no kernel touches memory before all
// earlier work on the stream is complete (a kernel's completion implies that of everything before it, because it
// waited itself). Under stream capture, and when switched off (test hook), the launch is a plain one and
// chain_wait() returns at once.
__device__ __forceinline__ void chain_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void chain_release() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

extern int g_chained_launches;   // fgs_host.cu; fgs_debug_chained_launches()

template <typename... KArgs, typename... Args>
inline cudaError_t chain_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args... args)
{
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 0;
    if (g_chained_launches) {
        cudaStreamCaptureStatus capturing = cudaStreamCaptureStatusNone;
        if (cudaStreamIsCapturing(st, &capturing) == cudaSuccess && capturing == cudaStreamCaptureStatusNone) cfg.numAttrs = 1;
    }
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// ---- checked build (-DFGS_DEBUG_BOUNDS) ----
// Every global store, every index computed from data (a Gaussian index read from a list, a destination derived
// from counters) and every computed shared-memory index is compared with the extent of what it addresses before the
// access; an index outside it is counted, the first one is recorded (source line, index, extent) and the access is
// SKIPPED -- nothing faults, nothing traps. The counters live once per source file; fgs_device_status() gathers
// them and raises FGS_ERR_BOUNDS. In the normal build the checks compile to nothing.
#ifdef FGS_DEBUG_BOUNDS
static __device__ unsigned long long g_bounds_report[4];   // violations, line of the first, its index, its extent
__device__ __forceinline__ bool index_ok(long long i, long long n, int line)
{
    if (i >= 0 && i < n) return true;
    if (atomicAdd(&g_bounds_report[0], 1ull) == 0ull) {
        g_bounds_report[1] = (unsigned long long)line;
        g_bounds_report[2] = (unsigned long long)i;
        g_bounds_report[3] = (unsigned long long)n;
    }
    return false;
}
#define FGS_INDEX_OK(i, n) fgs::index_ok((long long)(i), (long long)(n), __LINE__)
// Defines the function that copies (and optionally clears) this source file's counters.
#define FGS_BOUNDS_REPORT_FN(NAME)                                                                              \
    extern "C" int NAME(unsigned long long* out4, int reset)                                                    \
    {                                                                                                           \
        if (cudaMemcpyFromSymbol(out4, fgs::g_bounds_report, 4 * sizeof(unsigned long long)) != cudaSuccess) return FGS_ERR_CUDA; \
        if (reset) {                                                                                            \
            const unsigned long long zero[4] = { 0, 0, 0, 0 };                                                  \
            if (cudaMemcpyToSymbol(fgs::g_bounds_report, zero, sizeof zero) != cudaSuccess) return FGS_ERR_CUDA; \
        }                                                                                                       \
        return FGS_OK;                                                                                          \
    }
#else
#define FGS_INDEX_OK(i, n) true
#define FGS_BOUNDS_REPORT_FN(NAME)
#endif

} // namespace fgs
