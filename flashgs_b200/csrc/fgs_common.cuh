// Shared declarations of the flashgs_b200 CUDA library (sm_100a).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/flashgs_b200.h"

#define FGS_ABI_VERSION 2

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

} // namespace fgs
