// Host-side pieces of the flashgs_b200 library: status word, status strings and the
// camera matrices.

#include "fgs_common.cuh"

#include <cstring>
#include <mutex>

namespace fgs {

namespace {
// One status word per device that loads the library.
__device__ int g_device_status;

constexpr int kMaxDevices = 64;
int* g_status_ptr[kMaxDevices];
std::mutex g_status_mutex;
} // namespace

int* device_status_ptr()
{
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
    std::lock_guard<std::mutex> lock(g_status_mutex);
    if (!g_status_ptr[dev]) {
        void* p = nullptr;
        if (cudaGetSymbolAddress(&p, g_device_status) != cudaSuccess) return nullptr;
        g_status_ptr[dev] = static_cast<int*>(p);
    }
    return g_status_ptr[dev];
}

// View and view-projection matrices exactly as the reference builds them on the host
// (csrc/cuda_rasterizer/preprocess.cu:420-448): one rounding per operation, GLM 0.9.9.8
// operation order (mat3*vec3: csrc/glm/detail/type_mat3x3.inl:468-474; mat4*mat4:
// csrc/glm/detail/type_mat4x4.inl:630-648). This file is compiled with host FMA
// contraction off so that the products below are not fused.
void host_view_proj(int width, int height, const float* pos, const float* rot, float fx, float fy,
                    float zFar, float zNear, float* view, float* proj)
{
    // GLM column c of the rotation = row c of the row-major [3,3] input (csrc/pybind.cpp:141-143)
    const float* c0 = rot; const float* c1 = rot + 3; const float* c2 = rot + 6;
    const float nx = -pos[0], ny = -pos[1], nz = -pos[2];
    float tr[3];
    for (int r = 0; r < 3; r++) tr[r] = c0[r] * nx + c1[r] * ny + c2[r] * nz;
    const float v[16] = { c0[0], c0[1], c0[2], 0.0f, c1[0], c1[1], c1[2], 0.0f,
                          c2[0], c2[1], c2[2], 0.0f, tr[0], tr[1], tr[2], 1.0f };
    std::memcpy(view, v, sizeof v);

    const float top = height / (2.0f * fy) * zNear;
    const float bottom = -top;
    const float right = width / (2.0f * fx) * zNear;
    const float left = -right;
    float Pm[4][4];   // GLM indexing [column][row]
    std::memset(Pm, 0, sizeof Pm);
    const float z_sign = 1.0f;
    Pm[0][0] = 2.0f * zNear / (right - left);
    Pm[1][1] = 2.0f * zNear / (top - bottom);
    Pm[0][2] = (right + left) / (right - left);
    Pm[1][2] = (top + bottom) / (top - bottom);
    Pm[3][2] = z_sign;
    Pm[2][2] = z_sign * zFar / (zFar - zNear);
    Pm[2][3] = -(zFar * zNear) / (zFar - zNear);
    // proj = transpose(Pm) * view
    for (int c = 0; c < 4; c++)
        for (int r = 0; r < 4; r++)
            proj[4 * c + r] = ((Pm[r][0] * v[4 * c + 0] + Pm[r][1] * v[4 * c + 1]) + Pm[r][2] * v[4 * c + 2]) + Pm[r][3] * v[4 * c + 3];
}

} // namespace fgs

namespace fgs { int g_chained_launches = 1; }

// Test hook: zero makes every kernel launch a plain one (no programmatic dependent launch).
extern "C" void fgs_debug_chained_launches(int on) { fgs::g_chained_launches = on; }

extern "C" int fgs_abi_version(void) { return FGS_ABI_VERSION; }

extern "C" const char* fgs_status_string(int status)
{
    switch (status) {
    case FGS_OK: return "ok";
    case FGS_ERR_BAD_ARG: return "bad argument";
    case FGS_ERR_CUDA: return "CUDA runtime or launch error";
    case FGS_ERR_PAIR_OVERFLOW: return "pair buffer overflow";
    case FGS_ERR_LOOKBACK_TIMEOUT: return "device-side wait timed out";
    case FGS_ERR_TEMP_TOO_SMALL: return "sort scratch too small";
    case FGS_ERR_BOUNDS: return "index outside its extent (checked build)";
    default: return "several errors or unknown status";
    }
}

#ifdef FGS_DEBUG_BOUNDS
// per source file with kernels: its counters of the checked build
extern "C" int fgs_debug_bounds_preprocess(unsigned long long* out4, int reset);
extern "C" int fgs_debug_bounds_sort(unsigned long long* out4, int reset);
extern "C" int fgs_debug_bounds_render(unsigned long long* out4, int reset);

// Checked build: the counters of all source files as 3 x 4 values (preprocess, sort, render; each: violations, source
// line of the first, its index, its extent). Returns the total number of violations, or a negative value on error.
extern "C" long long fgs_debug_bounds_report(unsigned long long* out12, int reset)
{
    unsigned long long local[12];
    unsigned long long* o = out12 ? out12 : local;
    if (cudaDeviceSynchronize() != cudaSuccess) return -FGS_ERR_CUDA;
    if (fgs_debug_bounds_preprocess(o, reset) != FGS_OK || fgs_debug_bounds_sort(o + 4, reset) != FGS_OK ||
        fgs_debug_bounds_render(o + 8, reset) != FGS_OK)
        return -FGS_ERR_CUDA;
    return (long long)(o[0] + o[4] + o[8]);
}
#endif

extern "C" int fgs_device_status(int reset, void* stream)
{
    int* p = fgs::device_status_ptr();
    if (!p) return -FGS_ERR_CUDA;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    int host = 0;
    if (cudaMemcpyAsync(&host, p, sizeof(int), cudaMemcpyDeviceToHost, st) != cudaSuccess) return -FGS_ERR_CUDA;
    if (cudaStreamSynchronize(st) != cudaSuccess) return -FGS_ERR_CUDA;
    if (reset && host != 0) {
        if (cudaMemsetAsync(p, 0, sizeof(int), st) != cudaSuccess) return -FGS_ERR_CUDA;
    }
#ifdef FGS_DEBUG_BOUNDS
    const long long violations = fgs_debug_bounds_report(nullptr, reset);
    if (violations < 0) return -FGS_ERR_CUDA;
    if (violations > 0) host |= FGS_ERR_BOUNDS;
#endif
    return host;
}

extern "C" int fgs_view_proj_matrices(int width, int height, const float* cam_position, const float* cam_rotation,
                                      float focal_x, float focal_y, float zFar, float zNear,
                                      float* view16, float* proj16)
{
    if (!cam_position || !cam_rotation || !view16 || !proj16 || width <= 0 || height <= 0) return FGS_ERR_BAD_ARG;
    fgs::host_view_proj(width, height, cam_position, cam_rotation, focal_x, focal_y, zFar, zNear, view16, proj16);
    return FGS_OK;
}
