// Preprocess + key duplication for sm_100a.
//
// One kernel does what flashgs::preprocess does (csrc/cuda_rasterizer/preprocess.cu:243-418):
// near/opacity cull, projection, EWA 2D covariance, conic, exact AABB of the 1/256
// iso-ellipse, exact ellipse-vs-tile test, (tile|depth) key emission, degree-3 SH colour
// and the feature records the blend stage reads.
//
// Design (B200): a block of 256 threads owns 256 consecutive Gaussians -- of the scene, or, when the caller gives
// scratch for it, of the list of Gaussians that a first streaming kernel found able to reach the image or strip.
//   1. position / opacity / covariance of the block are fetched with 16-byte loads into
//      shared memory (the [P,3] and [P,6] rows are 12 and 24 bytes, so per-thread loads
//      could not be vectorised); each thread then projects its own Gaussian.
//   2. Work items are (Gaussian, tile row, 32-tile window of that row). The items of the
//      block's Gaussians are laid end to end with a block-wide exclusive scan and all 256
//      warps walk the item space together; a lane finds the Gaussian an item belongs to
//      by binary search in the scan. A splat covering thousands of tiles is thus spread over
//      the whole block instead of serialising a warp.
//      For its item a thread first bounds, in closed form and with generous margins, the
//      column range in which the iso-ellipse can reach the row's band of pixels, and then
//      runs the exact reference test only on the tiles of that range. For needle-like
//      splats this skips most of the bounding rectangle; the margins are far wider than the
//      float error of either computation, so the set of hits is the one the exact test
//      alone would give (the parity tests compare it pair by pair).
//   3. The exact tests are spread evenly too: a warp takes 32 items, lays their candidate
//      tiles end to end (warp scan) and tests 32 candidates at a time, one per lane, whatever
//      item they belong to (a lane finds its candidate's item from a bit mask of the items'
//      first candidates). Hits are compacted by ballot into a per-warp staging buffer in
//      shared memory; a full buffer is written out with ONE atomicAdd on the global pair
//      counter and coalesced stores, and what is left at the end goes out with one atomicAdd
//      for the whole block.
//   4. Gaussians with at least one hit fetch their 192-byte SH record with 16-byte loads
//      and write the three feature records.
//
// The float expressions keep the operation order of the reference so that the device
// compiler's FMA contraction sees the same expression trees: the tile lists depend on
// float comparisons and (int) truncations of these values. In the exact tile test, where a
// splat tangent to a tile edge flips on a single rounding, every operation is pinned with
// intrinsics to what the reference's build does (see segment_hits_ellipse).

#include "fgs_common.cuh"

#include <cstring>

namespace fgs {
namespace {

constexpr int PRE_THREADS = 256;
constexpr int PRE_WARPS = PRE_THREADS / 32;
#ifndef FGS_PRE_BLOCKS_PER_SM
#define FGS_PRE_BLOCKS_PER_SM 4
#endif
constexpr int PRE_BLOCKS_PER_SM = FGS_PRE_BLOCKS_PER_SM;   // resident blocks per SM the register budget is set for
constexpr int STG_CAP = 256;              // hits a warp can hold before it writes them out
constexpr int STG_FLUSH = STG_CAP - 32;   // write out once a further round of 32 tests might not fit

constexpr float kLog2e = 1.4426950216293334961f;
constexpr float kLn2 = 0.69314718055f;

__device__ __forceinline__ float approx_sqrt(float x) { float y; asm volatile("sqrt.approx.f32 %0, %1;" : "=f"(y) : "f"(x)); return y; }
__device__ __forceinline__ float approx_rsqrt(float x) { float y; asm volatile("rsqrt.approx.f32 %0, %1;" : "=f"(y) : "f"(x)); return y; }
__device__ __forceinline__ float approx_lg2(float x) { float y; asm volatile("lg2.approx.f32 %0, %1;" : "=f"(y) : "f"(x)); return y; }
__device__ __forceinline__ float max_f32(float a, float b) { float d; asm volatile("max.f32 %0, %1, %2;" : "=f"(d) : "f"(a), "f"(b)); return d; }

// preprocess.cu:64-67 -- the literals are doubles, so the arithmetic is done in fp64
__device__ __forceinline__ float ndc_to_pix(float v, int S) { return ((v + 1.0) * S - 1.0) * 0.5; }

struct f3 { float x, y, z; };

// preprocess.cu:69-77
__device__ __forceinline__ f3 xform4x3(const f3& p, const float* m)
{
    f3 t = {
        m[0] * p.x + m[4] * p.y + m[8] * p.z + m[12],
        m[1] * p.x + m[5] * p.y + m[9] * p.z + m[13],
        m[2] * p.x + m[6] * p.y + m[10] * p.z + m[14],
    };
    return t;
}

// Column-major 3x3 product in GLM's operation order (csrc/glm/detail/type_mat3x3.inl:486-519):
// r[c][q] = a[0][q]*b[c][0] + a[1][q]*b[c][1] + a[2][q]*b[c][2]
__device__ __forceinline__ void mul3(const float (&a)[3][3], const float (&b)[3][3], float (&r)[3][3])
{
#pragma unroll
    for (int c = 0; c < 3; c++)
#pragma unroll
        for (int q = 0; q < 3; q++)
            r[c][q] = a[0][q] * b[c][0] + a[1][q] * b[c][1] + a[2][q] * b[c][2];
}

// preprocess.cu:103-143
__device__ __forceinline__ f3 cov2d(const f3& p, const PreCam& cam, const float* cov3)
{
    f3 t = xform4x3(p, cam.view);
    const float limx = 1.3f * cam.tan_fovx;
    const float limy = 1.3f * cam.tan_fovy;
    const float txtz = t.x / t.z;
    const float tytz = t.y / t.z;
    t.x = fminf(limx, fmaxf(-limx, txtz)) * t.z;
    t.y = fminf(limy, fmaxf(-limy, tytz)) * t.z;

    const float J[3][3] = {
        { cam.focal_x / t.z, 0.0f, -(cam.focal_x * t.x) / (t.z * t.z) },
        { 0.0f, cam.focal_y / t.z, -(cam.focal_y * t.y) / (t.z * t.z) },
        { 0.0f, 0.0f, 0.0f } };
    const float* v = cam.view;
    const float Wm[3][3] = { { v[0], v[4], v[8] }, { v[1], v[5], v[9] }, { v[2], v[6], v[10] } };
    float T[3][3];
    mul3(Wm, J, T);
    const float Vt[3][3] = {   // transpose of the symmetric Vrk, spelled out as GLM's transpose does
        { cov3[0], cov3[1], cov3[2] }, { cov3[1], cov3[3], cov3[4] }, { cov3[2], cov3[4], cov3[5] } };
    const float Tt[3][3] = { { T[0][0], T[1][0], T[2][0] }, { T[0][1], T[1][1], T[2][1] }, { T[0][2], T[1][2], T[2][2] } };
    float A[3][3], C[3][3];
    mul3(Tt, Vt, A);
    mul3(A, T, C);
    C[0][0] += 0.3f;
    C[1][1] += 0.3f;
    return { C[0][0], C[0][1], C[1][1] };
}

// preprocess.cu:187-194. Which multiply-add pairs are fused decides the outcome for splats tangent to a tile edge,
// and the reference's build (its setup.py compiles with -O1) does not fuse the same way at its two call sites:
// against it, on 29.4 M pairs, the forms below reproduce every pair -- t1 as a separate multiply and add in the
// test of the vertical edge (VERTICAL) and fused in the test of the horizontal edge, everything else fused as
// written. Explicit intrinsics pin the choice so that it does not depend on this file's optimisation level.
template <bool VERTICAL>
__device__ __forceinline__ bool segment_hits_ellipse(float a, float b, float c, float d, float l, float r)
{
    const float delta = __fmaf_rn(b, b, -__fmul_rn(__fmul_rn(4.0f, a), c));
    const float a2 = __fmul_rn(2.0f, a);
    const float t1 = VERTICAL ? __fadd_rn(__fmul_rn(l - d, a2), b) : __fmaf_rn(l - d, a2, b);
    const float t2 = __fmaf_rn(r - d, a2, b);
    return delta >= 0.0f && (t1 <= 0.0f || __fmul_rn(t1, t1) <= delta) && (t2 >= 0.0f || __fmul_rn(t2, t2) <= delta);
}

// preprocess.cu:196-241: centre inside the tile's pixel box, or the iso-ellipse crosses the
// nearest vertical edge, or the nearest horizontal edge.
__device__ __forceinline__ bool tile_hit(int tx, int ty, int bx, int by, float cx_pix, float cy_pix,
                                         float conx, float cony, float conz, float power)
{
    const int minx = tx * bx, miny = ty * by;
    const int maxx = minx + bx - 1, maxy = miny + by - 1;
    if (cx_pix >= minx && cx_pix <= maxx && cy_pix >= miny && cy_pix <= maxy) return true;

    float a, b, c, dx, dy;
    const float w = __fmul_rn(2.0f, power);
    if (cx_pix * 2.0f < minx + maxx) dx = cx_pix - minx; else dx = cx_pix - maxx;
    a = conz;
    b = __fmul_rn(__fmul_rn(-2.0f, cony), dx);
    c = __fmaf_rn(__fmul_rn(conx, dx), dx, -w);
    if (segment_hits_ellipse<true>(a, b, c, cy_pix, miny, maxy)) return true;

    if (cy_pix * 2.0f < miny + maxy) dy = cy_pix - miny; else dy = cy_pix - maxy;
    a = conx;
    b = __fmul_rn(__fmul_rn(-2.0f, cony), dy);
    c = __fmaf_rn(__fmul_rn(conz, dy), dy, -w);
    return segment_hits_ellipse<false>(a, b, c, cx_pix, minx, maxx);
}

// preprocess.cu:145-185; sh holds the 16 coefficients as [coef][rgb]

__device__ __forceinline__ void sh_color(const float (&sh)[48], const f3& p, const float* campos, float& r, float& g, float& bl)
{
    const float SH_C0 = 0.28209479177387814f, SH_C1 = 0.4886025119029199f;
    const float C2[5] = { 1.0925484305920792f, -1.0925484305920792f, 0.31539156525252005f, -1.0925484305920792f, 0.5462742152960396f };
    const float C3[7] = { -0.5900435899266435f, 2.890611442640554f, -0.4570457994644658f, 0.3731763325901154f,
                          -0.4570457994644658f, 1.445305721320277f, -0.5900435899266435f };
    float dx = p.x - campos[0], dy = p.y - campos[1], dz = p.z - campos[2];
    const float l2 = dx * dx + dy * dy + dz * dz;
    const float rs = approx_rsqrt(l2);
    const float x = dx * rs, y = dy * rs, z = dz * rs;
    const float xx = x * x, yy = y * y, zz = z * z;
    const float xy = x * y, yz = y * z, xz = x * z;
    float res[3];
#pragma unroll
    for (int ch = 0; ch < 3; ch++) {
        float v = SH_C0 * sh[ch] + 0.5f;
        v = v - SH_C1 * y * sh[3 + ch] + SH_C1 * z * sh[6 + ch] - SH_C1 * x * sh[9 + ch];
        v = v +
            C2[0] * xy * sh[12 + ch] +
            C2[1] * yz * sh[15 + ch] +
            C2[2] * (2.0f * zz - xx - yy) * sh[18 + ch] +
            C2[3] * xz * sh[21 + ch] +
            C2[4] * (xx - yy) * sh[24 + ch];
        v = v +
            C3[0] * y * (3.0f * xx - yy) * sh[27 + ch] +
            C3[1] * xy * z * sh[30 + ch] +
            C3[2] * y * (4.0f * zz - xx - yy) * sh[33 + ch] +
            C3[3] * z * (2.0f * zz - 3.0f * xx - 3.0f * yy) * sh[36 + ch] +
            C3[4] * x * (4.0f * zz - xx - yy) * sh[39 + ch] +
            C3[5] * z * (xx - yy) * sh[42 + ch] +
            C3[6] * x * (xx - 3.0f * yy) * sh[45 + ch];
        res[ch] = max_f32(v, 0.0f);
    }
    r = res[0]; g = res[1]; bl = res[2];
}

// Cooperative copy of `nfloats` floats starting at a 16-byte aligned global address into
// shared memory: whole float4s first, then the ragged tail one float at a time.
// Same copy, asynchronous (cp.async, 16 bytes per request) for the whole float4s; the ragged tail is copied
// at once with plain loads. The caller commits and waits for the group.
__device__ __forceinline__ void stage_floats_async(float* dst, const float* src, int nfloats)
{
    const int nv = nfloats >> 2;
    for (int i = threadIdx.x; i < nv; i += PRE_THREADS)
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((unsigned)__cvta_generic_to_shared(dst + 4 * i)), "l"(src + 4 * i) : "memory");
    for (int i = (nv << 2) + threadIdx.x; i < nfloats; i += PRE_THREADS) dst[i] = __ldg(src + i);
}

template <bool VEC>
__device__ __forceinline__ void stage_floats(float* dst, const float* src, int nfloats)
{
    if (VEC) {
        const int nv = nfloats >> 2;
        for (int i = threadIdx.x; i < nv; i += PRE_THREADS)
            reinterpret_cast<float4*>(dst)[i] = __ldg(reinterpret_cast<const float4*>(src) + i);
        for (int i = (nv << 2) + threadIdx.x; i < nfloats; i += PRE_THREADS) dst[i] = __ldg(src + i);
    } else {
        for (int i = threadIdx.x; i < nfloats; i += PRE_THREADS) dst[i] = __ldg(src + i);
    }
}

// True when a splat certainly has no tile in the strip of tile rows [cam.row_begin, cam.row_end).
// The vertical screen variance is at most |row y of J|^2 * trace(Sigma) + 0.3 (J's row has norm
// focal_y/z * sqrt(1 + (y/z)^2) with y/z clamped, the view rotation preserves norms, the largest eigenvalue of a
// PSD matrix is at most its trace); the bound is padded by 2 % and a whole tile, so nothing the exact rectangle
// would keep is dropped. Written so that a NaN (degenerate input) is never dropped.
__device__ __forceinline__ bool misses_strip(const PreCam& cam, float view_z, float opacity, const float* c3, float projy)
{
    const float fz = cam.focal_y / view_z;
    const float ly = 1.3f * cam.tan_fovy;
    const float var = fz * fz * (1.0f + ly * ly) * (c3[0] + c3[3] + c3[5]) * 1.02f + 0.3f;
    const float pw_strip = fmaxf(kLn2 * 8.0f + kLn2 * approx_lg2(opacity), 0.0f);
    const float reach = 1.414214f * sqrtf(var * pw_strip) * 1.02f + 2.0f + (float)cam.block_y;
    const float py_strip = ndc_to_pix(projy, cam.H);
    return py_strip + reach < (float)(cam.row_begin * cam.block_y) || py_strip - reach > (float)(cam.row_end * cam.block_y);
}

// The same bound for the image's columns: true when the splat certainly lies left or right of the image.
__device__ __forceinline__ bool misses_columns(const PreCam& cam, float view_z, float opacity, const float* c3, float projx)
{
    const float fz = cam.focal_x / view_z;
    const float lx = 1.3f * cam.tan_fovx;
    const float var = fz * fz * (1.0f + lx * lx) * (c3[0] + c3[3] + c3[5]) * 1.02f + 0.3f;
    const float pw = fmaxf(kLn2 * 8.0f + kLn2 * approx_lg2(opacity), 0.0f);
    const float reach = 1.414214f * sqrtf(var * pw) * 1.02f + 2.0f + (float)cam.block_x;
    const float px = ndc_to_pix(projx, cam.W);
    return px + reach < 0.0f || px - reach > (float)(cam.grid_x * cam.block_x);
}

// Largest value of ln(256 * opacity) for an opacity in (0, 1]: the 1/256 iso-level of a fully opaque splat.
constexpr float kPowerMax = 5.5451774f;

// Scene preparation, once per scene: one 16-byte record per Gaussian with all the index-list kernel needs --
// position and q = trace(Sigma) * ln(256 * opacity), the product that the reach bound of misses_strip is made of
// (q < 0 marks an opacity below 1/255, which the opacity cull drops whatever the camera; an opacity above 1, which
// no sigmoid produces, gives q = +inf: never dropped). The index-list kernel then streams 16 bytes per Gaussian
// instead of 40.
__global__ void __launch_bounds__(PRE_THREADS)
scene_bounds_kernel(int P, const float* __restrict__ positions, const float* __restrict__ opacities,
                    const float* __restrict__ cov3ds, float4* __restrict__ bounds)
{
    const int i = blockIdx.x * PRE_THREADS + threadIdx.x;
    if (i >= P) return;
    const float opacity = __ldg(opacities + i);
    const float trace = __ldg(cov3ds + 6 * (size_t)i) + __ldg(cov3ds + 6 * (size_t)i + 3) + __ldg(cov3ds + 6 * (size_t)i + 5);
    const float pw = fmaxf(kLn2 * 8.0f + kLn2 * approx_lg2(opacity), 0.0f);
    float q = trace * pw;
    if (255.0f * opacity < 1.0f) q = -1.0f;
    else if (pw > kPowerMax) q = __int_as_float(0x7f800000);
    bounds[i] = make_float4(__ldg(positions + 3 * (size_t)i), __ldg(positions + 3 * (size_t)i + 1), __ldg(positions + 3 * (size_t)i + 2), q);
}

// Strip rendering, first step: the indices of the Gaussians that pass the near and opacity culls and can reach the
// strip, appended to list[1...] (list[0] counts them; any order). A rank that renders one strip of N then runs the
// expensive kernel below on about 1/N of the scene instead of on all of it.
// BOUNDS: the Gaussians come as the prepared 16-byte records (scene_bounds_kernel) instead of as position, opacity
// and covariance rows; the reach bound is the same expression with ln(256 * opacity) replaced by its maximum in the
// low-pass term, so it is never smaller and the list is a superset of the other variant's.
#ifndef FGS_CULL_PER_BLOCK
#define FGS_CULL_PER_BLOCK 4096
#endif
constexpr int CULL_PER_BLOCK = FGS_CULL_PER_BLOCK;           // Gaussians a block of the index-list kernel looks at
constexpr int CULL_PER_WARP = CULL_PER_BLOCK / PRE_WARPS;    // ... of which a warp can keep at most this many

template <bool BOUNDS>
__global__ void __launch_bounds__(PRE_THREADS)
strip_cull_kernel(int P, const float* __restrict__ positions, const float* __restrict__ opacities,
                  const float* __restrict__ cov3ds, const float4* __restrict__ bounds,
                  const __grid_constant__ PreCam cam, int* __restrict__ list)
{
    chain_release();
    chain_wait();   // nothing is read or written before the kernels ahead on the stream are complete
    // A block looks at CULL_PER_BLOCK consecutive Gaussians, 256 at a time; every warp collects the indices it keeps
    // in its own shared-memory region, and the block appends all of them to the list with ONE atomicAdd at the end
    // (every block adds to the same counter: one add per 256 Gaussians made the kernel wait on that word).
    __shared__ int s_keep[PRE_WARPS][CULL_PER_WARP];
    __shared__ int s_count[PRE_WARPS];
    __shared__ int s_base;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const unsigned lt = lanemask_lt();
    const int block_first = blockIdx.x * CULL_PER_BLOCK;
    int kept_here = 0;   // indices this warp holds (the same in every lane)

    auto reaches = [&](const f3& p, float q_or_opacity, const float* c3) -> bool {
        const f3 p_view = xform4x3(p, cam.view);
        if (p_view.z <= 0.2f) return false;
        const float* pm = cam.proj;
        const float hx = pm[0] * p.x + pm[4] * p.y + pm[8] * p.z + pm[12];
        const float hy = pm[1] * p.x + pm[5] * p.y + pm[9] * p.z + pm[13];
        const float hw = pm[3] * p.x + pm[7] * p.y + pm[11] * p.z + pm[15];
        if (BOUNDS) {
            // This variant runs over the whole scene on every GPU and is bound by instruction issue, so it uses the
            // cheap forms -- reciprocals instead of divisions, the approximate square root, float pixel coordinates:
            // their errors (parts in a million) vanish in the bound's pads (2 %, 2 pixels, a whole tile).
            if (q_or_opacity < 0.0f) return false;
            const float p_w = __frcp_rn(hw + 0.0000001f);
            const float inv_z = __frcp_rn(p_view.z);
            const float fzy = cam.focal_y * inv_z, ly = 1.3f * cam.tan_fovy;
            const float fzx = cam.focal_x * inv_z, lx = 1.3f * cam.tan_fovx;
            // (|J row|^2 trace 1.02 + 0.3) * power <= |J row|^2 1.02 q + 0.3 kPowerMax
            const float reach_y = 1.414214f * approx_sqrt(fzy * fzy * (1.0f + ly * ly) * 1.02f * q_or_opacity + 0.3f * kPowerMax) * 1.02f + 2.0f + (float)cam.block_y;
            const float reach_x = 1.414214f * approx_sqrt(fzx * fzx * (1.0f + lx * lx) * 1.02f * q_or_opacity + 0.3f * kPowerMax) * 1.02f + 2.0f + (float)cam.block_x;
            const float py = ((hy * p_w + 1.0f) * (float)cam.H - 1.0f) * 0.5f, px = ((hx * p_w + 1.0f) * (float)cam.W - 1.0f) * 0.5f;
            const bool off_rows = py + reach_y < (float)(cam.row_begin * cam.block_y) || py - reach_y > (float)(cam.row_end * cam.block_y);
            const bool off_cols = px + reach_x < 0.0f || px - reach_x > (float)(cam.grid_x * cam.block_x);
            return !off_rows && !off_cols;
        }
        const float p_w = 1.0f / (hw + 0.0000001f);
        if (255.0f * q_or_opacity < 1.0f) return false;
        return !misses_strip(cam, p_view.z, q_or_opacity, c3, hy * p_w) && !misses_columns(cam, p_view.z, q_or_opacity, c3, hx * p_w);
    };

    constexpr int BATCH = 4;   // records requested before the first is looked at
    for (int c0 = 0; c0 < CULL_PER_BLOCK; c0 += BATCH * PRE_THREADS) {
        float4 rec[BATCH];
        if (BOUNDS) {
#pragma unroll
            for (int u = 0; u < BATCH; u++) {
                const int i = block_first + c0 + u * PRE_THREADS + tid;
                rec[u] = i < P ? __ldg(bounds + i) : make_float4(0.f, 0.f, 0.f, -1.f);
            }
        }
#pragma unroll
        for (int u = 0; u < BATCH; u++) {
            const int i = block_first + c0 + u * PRE_THREADS + tid;
            bool keep = false;
            if (i < P) {
                if (BOUNDS) {
                    const f3 p = { rec[u].x, rec[u].y, rec[u].z };
                    keep = reaches(p, rec[u].w, nullptr);
                } else {
                    const f3 p = { __ldg(positions + 3 * (size_t)i), __ldg(positions + 3 * (size_t)i + 1), __ldg(positions + 3 * (size_t)i + 2) };
                    float c3[6];
#pragma unroll
                    for (int q = 0; q < 6; q++) c3[q] = __ldg(cov3ds + 6 * (size_t)i + q);
                    keep = reaches(p, __ldg(opacities + i), c3);
                }
            }
            const unsigned kept = __ballot_sync(FULL_MASK, keep);
            if (keep && FGS_INDEX_OK(kept_here + __popc(kept & lt), CULL_PER_WARP)) s_keep[warp][kept_here + __popc(kept & lt)] = i;
            kept_here += __popc(kept);
        }
    }
    if (lane == 0) s_count[warp] = kept_here;
    __syncthreads();
    if (tid == 0) {
        int total = 0;
        for (int w = 0; w < PRE_WARPS; w++) total += s_count[w];
        s_base = total > 0 ? atomicAdd(list, total) : 0;   // one atomic per block
    }
    __syncthreads();
    int at = s_base;
    for (int w = 0; w < warp; w++) at += s_count[w];
    for (int j = lane; j < kept_here; j += 32)
        if (FGS_INDEX_OK(at + j, P)) list[1 + at + j] = s_keep[warp][j];
}

// Optional per-phase cycle accounting (compile with -DFGS_PRE_TIMING): thread 0 of every block adds the SM
// cycles spent in each phase to g_pre_cycles; read with fgs_debug_pre_phase_cycles.
#ifdef FGS_PRE_TIMING
__device__ unsigned long long g_pre_cycles[8];
#define FGS_PT(i) do { if (threadIdx.x == 0) { const long long now_ = clock64(); atomicAdd(&g_pre_cycles[i], (unsigned long long)(now_ - t_prev_)); t_prev_ = now_; } } while (0)
#else
#define FGS_PT(i) do { } while (0)
#endif

template <bool VEC>
__global__ void __launch_bounds__(PRE_THREADS, PRE_BLOCKS_PER_SM)
preprocess_kernel(int P,
                  const float* __restrict__ positions, const float* __restrict__ opacities,
                  const float* __restrict__ cov3ds, const float* __restrict__ shs,
                  const __grid_constant__ PreCam cam,
                  float2* __restrict__ points_xy, float4* __restrict__ rgb_depth, float4* __restrict__ conic_opacity,
                  uint64_t* __restrict__ keys, uint32_t* __restrict__ values, long long capacity,
                  int* __restrict__ curr_offset, int* __restrict__ status, const int* __restrict__ list,
                  unsigned* __restrict__ tile_count)
{
    chain_release();
    chain_wait();   // nothing is read or written before the kernels ahead on the stream are complete
    __shared__ __align__(16) float s_pos[PRE_THREADS * 3];
    __shared__ __align__(16) float s_cov[PRE_THREADS * 6];
    __shared__ __align__(16) float s_opa[PRE_THREADS];
    __shared__ float2 s_xy[PRE_THREADS];
    __shared__ float4 s_con[PRE_THREADS];      // conic.x, conic.y, conic.z, power
    __shared__ int4 s_rect[PRE_THREADS];       // min_x, min_y, width, float_bits(depth)
    __shared__ float4 s_cull[PRE_THREADS];     // enlarged w, dx_max (< 0: no culling), dy_max, dy where x is largest
    __shared__ int s_prefix[PRE_THREADS + 1];  // exclusive scan of the item counts
    __shared__ uint8_t s_vis[PRE_THREADS];
    __shared__ int4 s_rec[PRE_WARPS][32];      // per lane of a warp: first candidate number, Gaussian, tile row, first column
    __shared__ uint8_t s_src[PRE_WARPS][32];   // the lanes that have candidates, in lane order
    __shared__ uint2 s_stage[PRE_WARPS][STG_CAP];   // hits waiting to be written: tile, Gaussian
    __shared__ int s_wsum[PRE_WARPS];
    __shared__ int s_wcnt[PRE_WARPS];
    __shared__ int s_tail_base;
    __shared__ int s_idx[PRE_THREADS];         // scene index of the block's Gaussians

#ifdef FGS_PRE_TIMING
    long long t_prev_ = clock64();
#endif
    const int tid = threadIdx.x;
    const int lane = tid & 31, warp = tid >> 5;
    // The block's Gaussians: 256 consecutive ones of the scene, or (strip rendering behind strip_cull_kernel)
    // 256 consecutive entries of the list of those that can reach the strip.
    const int base = blockIdx.x * PRE_THREADS;
    const int total_here = list != nullptr ? min(P, max(list[0], 0)) : P;
    if (base >= total_here) return;
    const int n_here = min(PRE_THREADS, total_here - base);
    if (list != nullptr) {
        int i = tid < n_here ? list[1 + base + tid] : 0;
        if (!FGS_INDEX_OK(i, P)) i = 0;   // checked build: a list entry outside the scene is reported and replaced
        s_idx[tid] = i;
        if (tid < n_here) {
#pragma unroll
            for (int q = 0; q < 3; q++) s_pos[3 * tid + q] = __ldg(positions + 3 * (size_t)i + q);
            if (VEC) {   // a covariance row is 24 bytes: 8-byte aligned whenever the array is
                const float2* c2 = reinterpret_cast<const float2*>(cov3ds + 6 * (size_t)i);
#pragma unroll
                for (int q = 0; q < 3; q++) {
                    const float2 v = __ldg(c2 + q);
                    s_cov[6 * tid + 2 * q] = v.x; s_cov[6 * tid + 2 * q + 1] = v.y;
                }
            } else {
#pragma unroll
                for (int q = 0; q < 6; q++) s_cov[6 * tid + q] = __ldg(cov3ds + 6 * (size_t)i + q);
            }
            s_opa[tid] = __ldg(opacities + i);
        }
    } else if (VEC) {
        s_idx[tid] = base + tid;
        stage_floats_async(s_pos, positions + (size_t)base * 3, n_here * 3);
        stage_floats_async(s_cov, cov3ds + (size_t)base * 6, n_here * 6);
        stage_floats_async(s_opa, opacities + base, n_here);
        asm volatile("cp.async.commit_group;" ::: "memory");
        asm volatile("cp.async.wait_group 0;" ::: "memory");
    } else {
        s_idx[tid] = base + tid;
        stage_floats<false>(s_pos, positions + (size_t)base * 3, n_here * 3);
        stage_floats<false>(s_cov, cov3ds + (size_t)base * 6, n_here * 6);
        stage_floats<false>(s_opa, opacities + base, n_here);
    }
    s_vis[tid] = 0;
    __syncthreads();
    FGS_PT(0);

    // ---- per-Gaussian projection (preprocess.cu:282-316) ----
    bool point_valid = false;
    f3 p_orig = { 0.f, 0.f, 0.f };
    float depth = 0.f, log2_opacity = 0.f, power = 0.f;
    float2 point_xy = { 0.f, 0.f };
    f3 conic = { 0.f, 0.f, 0.f };
    int minx = 0, miny = 0, maxx = 0, maxy = 0;
    if (tid < n_here) {
        do {
            p_orig = { s_pos[3 * tid], s_pos[3 * tid + 1], s_pos[3 * tid + 2] };
            const f3 p_view = xform4x3(p_orig, cam.view);
            depth = p_view.z;
            if (p_view.z <= 0.2f) break;
            const float opacity = s_opa[tid];
            if (255.0f * opacity < 1.0f) break;

            const float* pm = cam.proj;
            const float hx = pm[0] * p_orig.x + pm[4] * p_orig.y + pm[8] * p_orig.z + pm[12];
            const float hy = pm[1] * p_orig.x + pm[5] * p_orig.y + pm[9] * p_orig.z + pm[13];
            const float hw = pm[3] * p_orig.x + pm[7] * p_orig.y + pm[11] * p_orig.z + pm[15];
            const float p_w = 1.0f / (hw + 0.0000001f);
            const float projx = hx * p_w, projy = hy * p_w;

            // rendering a strip of tile rows: drop, before the covariance work, splats that cannot reach it
            if ((cam.row_begin > 0 || cam.row_end < cam.grid_y) && misses_strip(cam, p_view.z, opacity, s_cov + 6 * tid, projy)) break;

            const f3 cov = cov2d(p_orig, cam, s_cov + 6 * tid);
            const float det = (cov.x * cov.z - cov.y * cov.y);
            const float det_inv = 1.f / det;
            conic = { cov.z * det_inv, -cov.y * det_inv, cov.x * det_inv };

            log2_opacity = approx_lg2(opacity);
            power = kLn2 * 8.0f + kLn2 * log2_opacity;
            const int width = (int)(1.414214f * approx_sqrt(cov.x * power) + 1.0f);
            const int height = (int)(1.414214f * approx_sqrt(cov.z * power) + 1.0f);

            point_xy = { ndc_to_pix(projx, cam.W), ndc_to_pix(projy, cam.H) };
            // getRect, preprocess.cu:90-100, then the strip clamp on rows
            minx = min(cam.grid_x, max(0, (int)((point_xy.x - width) / (float)cam.block_x)));
            miny = min(cam.grid_y, max(0, (int)((point_xy.y - height) / (float)cam.block_y)));
            maxx = min(cam.grid_x, max(0, (int)((point_xy.x + width) / (float)cam.block_x) + 1));
            maxy = min(cam.grid_y, max(0, (int)((point_xy.y + height) / (float)cam.block_y) + 1));
            miny = max(miny, cam.row_begin);
            maxy = min(maxy, cam.row_end);
            point_valid = (maxx > minx) && (maxy > miny);
        } while (false);
    }

    FGS_PT(1);
    // Work items of this Gaussian: one per (tile row, window of 32 tile columns).
    const int rect_w = point_valid ? (maxx - minx) : 0;
    const int nseg = (rect_w + 31) >> 5;
    const int items = point_valid ? nseg * (maxy - miny) : 0;
    s_xy[tid] = point_xy;
    s_con[tid] = make_float4(conic.x, conic.y, conic.z, power);
    s_rect[tid] = make_int4(minx, miny, rect_w, __float_as_int(depth));
    {
        // Closed-form extent of the (slightly enlarged) iso-ellipse A dx^2 + 2B dx dy + C dy^2 <= w:
        // |dx| <= sqrt(C w / det), |dy| <= sqrt(A w / det); x is extreme at dy = -+ (B/C) dx_max.
        // The enlargement grows with the conditioning A*C/det of the quadratic, which is what
        // amplifies rounding in the exact test near tangency; ill-conditioned or degenerate
        // conics are not culled at all (dx_max < 0 marks that).
        const float A = conic.x, B = conic.y, C = conic.z;
        const float det = A * C - B * B;
        const float cond = (A * C) / det;
        float4 cull = make_float4(0.f, -1.f, 0.f, 0.f);
        if (cam.cull_columns && point_valid && det > 0.f && A > 0.f && C > 0.f && cond < 5000.f) {
            const float w = 2.0f * power * (1.0f + 1e-3f + 2e-4f * cond);
            const float dxmax = sqrtf(C * w / det);
            cull = make_float4(w, dxmax, sqrtf(A * w / det), -(B / C) * dxmax);
        }
        s_cull[tid] = cull;
    }

    // ---- block-wide exclusive scan of the item counts ----
    int incl = items;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int v = __shfl_up_sync(FULL_MASK, incl, o);
        if (lane >= o) incl += v;
    }
    if (lane == 31) s_wsum[warp] = incl;
    __syncthreads();
    int wbase = 0;
#pragma unroll
    for (int w = 0; w < PRE_WARPS; w++) wbase += (w < warp) ? s_wsum[w] : 0;
    s_prefix[tid] = wbase + incl - items;
    if (tid == PRE_THREADS - 1) s_prefix[PRE_THREADS] = wbase + incl;
    __syncthreads();
    FGS_PT(2);
    const int total = s_prefix[PRE_THREADS];

    // ---- walk the item space: each warp takes 32 consecutive items at a time ----
    const float margin = 0.5f;   // pixels, on both the band and the column range
    uint2* stage = s_stage[warp];
    int staged = 0;              // hits of this warp waiting in stage[] (the same in every lane)
    const unsigned lt = lanemask_lt(), le = lt | (1u << lane);
    auto write_staged = [&](long long first, int count) {
        for (int i = lane; i < count; i += 32) {
            if (!FGS_INDEX_OK(i, STG_CAP)) continue;
            const uint2 e = stage[i];
            const long long o = first + i;
            if (!FGS_INDEX_OK(e.y, PRE_THREADS) || !FGS_INDEX_OK(e.x, cam.grid_x * cam.grid_y)) continue;
            if (o >= 0 && o < capacity) {
                keys[o] = ((uint64_t)e.x << 32) | (uint32_t)s_rect[e.y].w;
                values[o] = (uint32_t)s_idx[e.y];
                if (tile_count != nullptr) atomicAdd(tile_count + e.x, 1u);   // pairs per tile, for the sort that follows
            } else {
                atomicOr(status, FGS_ERR_PAIR_OVERFLOW);
            }
        }
    };
    for (int c0 = warp * 32; c0 < total; c0 += PRE_THREADS) {
        // 1. this lane's item: its Gaussian, tile row and the candidate columns [x_begin, x_end)
        const int item = c0 + lane;
        int g = 0, ty = 0, x_begin = 0, x_end = 0;
        if (item < total) {
            int lo = 0, hi = PRE_THREADS;   // largest g with s_prefix[g] <= item
#pragma unroll
            for (int st = 0; st < 8; st++) {
                const int mid = (lo + hi) >> 1;
                if (s_prefix[mid] <= item) lo = mid; else hi = mid;
            }
            g = lo;
            if (!FGS_INDEX_OK(g, PRE_THREADS)) g = 0;
            const int4 rc = s_rect[g];
            const int t = item - s_prefix[g];
            const int ns = (rc.z + 31) >> 5;
            const int row = (ns == 1) ? t : t / ns;
            const int seg = t - row * ns;
            ty = rc.y + row;
            x_begin = rc.x + (seg << 5);
            x_end = min(rc.x + rc.z, x_begin + 32);
            const float4 cu = s_cull[g];
            if (cu.y >= 0.f) {
                const float2 c = s_xy[g];
                const float4 q = s_con[g];
                // band of pixel rows of this tile row, relative to the centre, clipped to the ellipse's extent
                const float d_lo = fmaxf((float)(ty * cam.block_y) - c.y - margin, -cu.z);
                const float d_hi = fminf((float)(ty * cam.block_y + cam.block_y - 1) - c.y + margin, cu.z);
                if (d_lo > d_hi) {
                    x_end = x_begin;
                } else {
                    const float det = q.x * q.z - q.y * q.y;
                    const float s_lo = approx_sqrt(fmaxf(0.f, q.x * cu.x - det * d_lo * d_lo));
                    const float s_hi = approx_sqrt(fmaxf(0.f, q.x * cu.x - det * d_hi * d_hi));
                    const float inv_a = __frcp_rn(q.x);
                    const float xh = (cu.w >= d_lo && cu.w <= d_hi) ? cu.y
                                     : fmaxf((-q.y * d_lo + s_lo) * inv_a, (-q.y * d_hi + s_hi) * inv_a);
                    const float xl = (-cu.w >= d_lo && -cu.w <= d_hi) ? -cu.y
                                     : fminf((-q.y * d_lo - s_lo) * inv_a, (-q.y * d_hi - s_hi) * inv_a);
                    // tiles whose pixel box [tx*bx, tx*bx + bx - 1] meets [c.x + xl - margin, c.x + xh + margin]
                    const float inv_bx = 1.0f / (float)cam.block_x;
                    const float fl = ceilf((c.x + xl - margin - (float)(cam.block_x - 1)) * inv_bx);
                    const float fr = floorf((c.x + xh + margin) * inv_bx);
                    x_begin = max(x_begin, (int)fmaxf(fl, -1.0e6f));
                    x_end = min(x_end, (int)fminf(fr, 1.0e6f) + 1);
                }
            }
        }
        FGS_PT(5);
        // 2. the candidate tiles of the warp's 32 items laid end to end
        const int cnt = max(x_end - x_begin, 0);
        int inc = cnt;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int v = __shfl_up_sync(FULL_MASK, inc, o);
            if (lane >= o) inc += v;
        }
        const int excl = inc - cnt;
        const int candidates = __shfl_sync(FULL_MASK, inc, 31);
        if (candidates == 0) continue;
        const unsigned has = __ballot_sync(FULL_MASK, cnt > 0);
        __syncwarp();   // the previous round's reads of s_rec / s_src are over
        if (cnt > 0 && FGS_INDEX_OK(__popc(has & lt), 32)) s_src[warp][__popc(has & lt)] = (uint8_t)lane;
        s_rec[warp][lane] = make_int4(excl, g, ty, x_begin);
        __syncwarp();
        // 3. 32 candidates at a time, one exact test per lane; hits go to the warp's staging buffer
        for (int b0 = 0; b0 < candidates; b0 += 32) {
            // bit i of starts: an item's candidates begin at candidate b0 + i
            const unsigned starts = __reduce_or_sync(FULL_MASK, (cnt > 0 && excl >= b0 && excl < b0 + 32) ? (1u << (excl - b0)) : 0u);
            const int before = __popc(__ballot_sync(FULL_MASK, cnt > 0 && excl < b0));
            const int j = b0 + lane;
            bool hit = false;
            int tile = 0, gs = 0;
            if (j < candidates) {
                // the item this candidate belongs to: the last one that begins at or before it
                int src_at = before + __popc(starts & le) - 1;
                if (!FGS_INDEX_OK(src_at, 32)) src_at = 0;
                int src_lane = s_src[warp][src_at];
                if (!FGS_INDEX_OK(src_lane, 32)) src_lane = 0;
                const int4 rc = s_rec[warp][src_lane];
                const int tx = rc.w + (j - rc.x);
                gs = rc.y;
                const float2 c = s_xy[gs];
                const float4 q = s_con[gs];
                hit = tile_hit(tx, rc.z, cam.block_x, cam.block_y, c.x, c.y, q.x, q.y, q.z, q.w);
                tile = rc.z * cam.grid_x + tx;
            }
            const unsigned hits = __ballot_sync(FULL_MASK, hit);
            if (hit && FGS_INDEX_OK(staged + __popc(hits & lt), STG_CAP) && FGS_INDEX_OK(gs, PRE_THREADS)) {
                stage[staged + __popc(hits & lt)] = make_uint2((unsigned)tile, (unsigned)gs);
                s_vis[gs] = 1;
            }
            staged += __popc(hits);
            if (staged >= STG_FLUSH) {   // one atomicAdd on the global pair counter per flush
                __syncwarp();
                int first = 0;
                if (lane == 0) first = atomicAdd(curr_offset, staged);
                first = __shfl_sync(FULL_MASK, first, 0);
                write_staged(first, staged);
                staged = 0;
                __syncwarp();
            }
        }
        FGS_PT(6);
    }
    if (lane == 0) s_wcnt[warp] = staged;
    __syncthreads();
    FGS_PT(3);
    // what the warps still hold is written after the feature phase, at offsets from ONE atomicAdd for the block
    if (tid == 0) {
        int rest = 0;
        for (int w = 0; w < PRE_WARPS; w++) rest += s_wcnt[w];
        s_tail_base = rest > 0 ? atomicAdd(curr_offset, rest) : 0;
    }

    // ---- features of visible Gaussians (preprocess.cu:411-417) ----
    if (tid < n_here && s_vis[tid] && FGS_INDEX_OK(s_idx[tid], P)) {
        const int idx = s_idx[tid];
        float sh[48];
        if (VEC) {
            const float4* s4 = reinterpret_cast<const float4*>(shs + (size_t)idx * 48);
#pragma unroll
            for (int i = 0; i < 12; i++) {
                const float4 v = __ldg(s4 + i);
                sh[4 * i] = v.x; sh[4 * i + 1] = v.y; sh[4 * i + 2] = v.z; sh[4 * i + 3] = v.w;
            }
        } else {
#pragma unroll
            for (int i = 0; i < 48; i++) sh[i] = __ldg(shs + (size_t)idx * 48 + i);
        }
        float r, g, b;
        sh_color(sh, p_orig, cam.cam, r, g, b);
        points_xy[idx] = point_xy;
        conic_opacity[idx] = make_float4((-0.5f * kLog2e) * conic.x, -kLog2e * conic.y, (-0.5f * kLog2e) * conic.z, log2_opacity);
        rgb_depth[idx] = make_float4(r, g, b, depth);
    }
    FGS_PT(4);
    __syncthreads();
    {
        long long first = s_tail_base;
        for (int w = 0; w < warp; w++) first += s_wcnt[w];
        write_staged(first, staged);
    }
}

} // namespace

int g_debug_no_column_cull = 0;

// Host matrices in the reference's operation order; see fgs_view_proj_matrices().
void host_view_proj(int width, int height, const float* pos, const float* rot, float fx, float fy,
                    float zFar, float zNear, float* view, float* proj);

} // namespace fgs

FGS_BOUNDS_REPORT_FN(fgs_debug_bounds_preprocess)

#ifdef FGS_PRE_TIMING
extern "C" int fgs_debug_pre_phase_cycles(unsigned long long* out8, int reset)
{
    if (cudaMemcpyFromSymbol(out8, fgs::g_pre_cycles, sizeof(unsigned long long) * 8) != cudaSuccess) return FGS_ERR_CUDA;
    if (reset) { unsigned long long z[8] = {0}; cudaMemcpyToSymbol(fgs::g_pre_cycles, z, sizeof z); }
    return FGS_OK;
}
#endif

// Test hook: non-zero makes the next preprocess calls run the exact tile test on every tile of a
// splat's bounding rectangle, as the reference does, instead of first narrowing each row's column
// range. Both settings must produce the same pair set; the tests compare them.
extern "C" void fgs_debug_preprocess_no_column_cull(int on) { fgs::g_debug_no_column_cull = on; }

namespace fgs {
// `events`, when given, holds three events: recorded before the index-list kernel, between the two kernels and after
// the main kernel (the measurement entry point below).
static int preprocess_impl(int P, const float* positions, const float* shs, const float* opacities, const float* cov3ds,
                           int width, int height, int block_x, int block_y,
                           const float* cam_position, const float* cam_rotation,
                           float focal_x, float focal_y, float zFar, float zNear,
                           int tile_row_begin, int tile_row_end,
                           float* points_xy, float* rgb_depth, float* conic_opacity,
                           uint64_t* keys_unsorted, uint32_t* values_unsorted, int64_t pair_capacity,
                           int* curr_offset, int* cull_scratch, int64_t cull_scratch_ints, void* stream, cudaEvent_t* events,
                           const float* scene_bounds = nullptr, uint32_t* tile_counts = nullptr)
{
    if (P < 0 || width <= 0 || height <= 0 || block_x <= 0 || block_y <= 0 || pair_capacity < 0) return FGS_ERR_BAD_ARG;
    if (cull_scratch != nullptr && cull_scratch_ints < (int64_t)P + 1) return FGS_ERR_TEMP_TOO_SMALL;
    if (!cam_position || !cam_rotation || !curr_offset) return FGS_ERR_BAD_ARG;
    if (P == 0) return FGS_OK;
    if (!positions || !shs || !opacities || !cov3ds || !points_xy || !rgb_depth || !conic_opacity ||
        !keys_unsorted || !values_unsorted)
        return FGS_ERR_BAD_ARG;
    int* status = device_status_ptr();
    if (!status) return FGS_ERR_CUDA;

    PreCam cam;
    host_view_proj(width, height, cam_position, cam_rotation, focal_x, focal_y, zFar, zNear, cam.view, cam.proj);
    std::memcpy(cam.cam, cam_position, 3 * sizeof(float));
    cam.tan_fovx = width / (2.0f * focal_x);    // preprocess.cu:465-466
    cam.tan_fovy = height / (2.0f * focal_y);
    cam.focal_x = focal_x; cam.focal_y = focal_y;
    cam.W = width; cam.H = height; cam.block_x = block_x; cam.block_y = block_y;
    cam.grid_x = (width + block_x - 1) / block_x;
    cam.grid_y = (height + block_y - 1) / block_y;
    cam.row_begin = tile_row_begin < 0 ? 0 : tile_row_begin;
    cam.row_end = (tile_row_end < 0 || tile_row_end > cam.grid_y) ? cam.grid_y : tile_row_end;
    cam.cull_columns = g_debug_no_column_cull ? 0 : 1;

    const bool vec = aligned16(positions) && aligned16(shs) && aligned16(opacities) && aligned16(cov3ds);
    const int groups = (P + PRE_THREADS - 1) / PRE_THREADS;
    const int blocks = groups;   // one block per 256 Gaussians (with a list: blocks past its end return at once)
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    // With scratch for the index list: first the cheap pass that lists the Gaussians reaching the rendered rows and
    // the image's columns (for a whole frame too: about a third of the scene lies outside the image).
    const int* list = nullptr;
    // pairs per tile for the sort: only images whose tile ids the tile-bucketed sort takes (see fgs_sort_pairs_counted)
    if (tile_counts != nullptr && (int64_t)cam.grid_x * cam.grid_y >= FGS_TILE_COUNT_WORDS) tile_counts = nullptr;
    if (tile_counts != nullptr && cudaMemsetAsync(tile_counts, 0, sizeof(uint32_t) * FGS_TILE_COUNT_WORDS, st) != cudaSuccess)
        return FGS_ERR_CUDA;
    if (events) cudaEventRecord(events[0], st);
    if (cull_scratch != nullptr) {
        if (cudaMemsetAsync(cull_scratch, 0, sizeof(int), st) != cudaSuccess) return FGS_ERR_CUDA;
        const int cull_blocks = (P + CULL_PER_BLOCK - 1) / CULL_PER_BLOCK;
        if (scene_bounds != nullptr && aligned16(scene_bounds))
            chain_launch(strip_cull_kernel<true>, dim3(cull_blocks), dim3(PRE_THREADS), 0, st, P, positions, opacities, cov3ds, reinterpret_cast<const float4*>(scene_bounds), cam, cull_scratch);
        else
            chain_launch(strip_cull_kernel<false>, dim3(cull_blocks), dim3(PRE_THREADS), 0, st, P, positions, opacities, cov3ds, nullptr, cam, cull_scratch);
        list = cull_scratch;
    }
    if (events) cudaEventRecord(events[1], st);
    if (vec)
        chain_launch(preprocess_kernel<true>, dim3(blocks), dim3(PRE_THREADS), 0, st, P, positions, opacities, cov3ds, shs, cam,
            reinterpret_cast<float2*>(points_xy), reinterpret_cast<float4*>(rgb_depth), reinterpret_cast<float4*>(conic_opacity),
            keys_unsorted, values_unsorted, (long long)pair_capacity, curr_offset, status, list, tile_counts);
    else
        chain_launch(preprocess_kernel<false>, dim3(blocks), dim3(PRE_THREADS), 0, st, P, positions, opacities, cov3ds, shs, cam,
            reinterpret_cast<float2*>(points_xy), reinterpret_cast<float4*>(rgb_depth), reinterpret_cast<float4*>(conic_opacity),
            keys_unsorted, values_unsorted, (long long)pair_capacity, curr_offset, status, list, tile_counts);
    if (events) cudaEventRecord(events[2], st);
    return launch_status();
}
} // namespace fgs

extern "C" int fgs_preprocess_strip_culled(int P, const float* positions, const float* shs, const float* opacities, const float* cov3ds,
                                           int width, int height, int block_x, int block_y,
                                           const float* cam_position, const float* cam_rotation,
                                           float focal_x, float focal_y, float zFar, float zNear,
                                           int tile_row_begin, int tile_row_end,
                                           float* points_xy, float* rgb_depth, float* conic_opacity,
                                           uint64_t* keys_unsorted, uint32_t* values_unsorted, int64_t pair_capacity,
                                           int* curr_offset, int* cull_scratch, int64_t cull_scratch_ints, void* stream)
{
    return fgs::preprocess_impl(P, positions, shs, opacities, cov3ds, width, height, block_x, block_y, cam_position, cam_rotation,
                                focal_x, focal_y, zFar, zNear, tile_row_begin, tile_row_end, points_xy, rgb_depth, conic_opacity,
                                keys_unsorted, values_unsorted, pair_capacity, curr_offset, cull_scratch, cull_scratch_ints, stream, nullptr);
}

extern "C" int fgs_scene_bounds(int P, const float* positions, const float* opacities, const float* cov3ds, float* bounds, void* stream)
{
    if (P < 0) return FGS_ERR_BAD_ARG;
    if (P == 0) return FGS_OK;
    if (!positions || !opacities || !cov3ds || !bounds || !fgs::aligned16(bounds)) return FGS_ERR_BAD_ARG;
    fgs::scene_bounds_kernel<<<(P + fgs::PRE_THREADS - 1) / fgs::PRE_THREADS, fgs::PRE_THREADS, 0, static_cast<cudaStream_t>(stream)>>>(
        P, positions, opacities, cov3ds, reinterpret_cast<float4*>(bounds));
    return fgs::launch_status();
}

extern "C" int fgs_preprocess_prepared(int P, const float* positions, const float* shs, const float* opacities, const float* cov3ds,
                                       int width, int height, int block_x, int block_y,
                                       const float* cam_position, const float* cam_rotation,
                                       float focal_x, float focal_y, float zFar, float zNear,
                                       int tile_row_begin, int tile_row_end,
                                       float* points_xy, float* rgb_depth, float* conic_opacity,
                                       uint64_t* keys_unsorted, uint32_t* values_unsorted, int64_t pair_capacity,
                                       int* curr_offset, int* cull_scratch, int64_t cull_scratch_ints,
                                       const float* scene_bounds, uint32_t* tile_counts, void* stream)
{
    if (scene_bounds != nullptr && (cull_scratch == nullptr || !fgs::aligned16(scene_bounds))) return FGS_ERR_BAD_ARG;
    return fgs::preprocess_impl(P, positions, shs, opacities, cov3ds, width, height, block_x, block_y, cam_position, cam_rotation,
                                focal_x, focal_y, zFar, zNear, tile_row_begin, tile_row_end, points_xy, rgb_depth, conic_opacity,
                                keys_unsorted, values_unsorted, pair_capacity, curr_offset, cull_scratch, cull_scratch_ints, stream, nullptr,
                                scene_bounds, tile_counts);
}

extern "C" int fgs_preprocess_profile(int P, const float* positions, const float* shs, const float* opacities, const float* cov3ds,
                                      int width, int height, int block_x, int block_y,
                                      const float* cam_position, const float* cam_rotation,
                                      float focal_x, float focal_y, float zFar, float zNear,
                                      int tile_row_begin, int tile_row_end,
                                      float* points_xy, float* rgb_depth, float* conic_opacity,
                                      uint64_t* keys_unsorted, uint32_t* values_unsorted, int64_t pair_capacity,
                                      int* curr_offset, int* cull_scratch, int64_t cull_scratch_ints,
                                      const float* scene_bounds, uint32_t* tile_counts, void* stream, float* kernel_ms2)
{
    if (!kernel_ms2) return FGS_ERR_BAD_ARG;
    cudaEvent_t ev[3];
    for (auto& e : ev)
        if (cudaEventCreate(&e) != cudaSuccess) return FGS_ERR_CUDA;
    int st = fgs::preprocess_impl(P, positions, shs, opacities, cov3ds, width, height, block_x, block_y, cam_position, cam_rotation,
                                  focal_x, focal_y, zFar, zNear, tile_row_begin, tile_row_end, points_xy, rgb_depth, conic_opacity,
                                  keys_unsorted, values_unsorted, pair_capacity, curr_offset, cull_scratch, cull_scratch_ints, stream, ev,
                                  scene_bounds, tile_counts);
    kernel_ms2[0] = kernel_ms2[1] = 0.0f;
    if (st == FGS_OK && P > 0) {
        if (cudaStreamSynchronize(static_cast<cudaStream_t>(stream)) != cudaSuccess) st = FGS_ERR_CUDA;
        if (st == FGS_OK && (cudaEventElapsedTime(&kernel_ms2[0], ev[0], ev[1]) != cudaSuccess ||
                             cudaEventElapsedTime(&kernel_ms2[1], ev[1], ev[2]) != cudaSuccess))
            st = FGS_ERR_CUDA;
    }
    for (auto& e : ev) cudaEventDestroy(e);
    return st;
}

extern "C" int fgs_preprocess_strip(int P, const float* positions, const float* shs, const float* opacities, const float* cov3ds,
                                    int width, int height, int block_x, int block_y,
                                    const float* cam_position, const float* cam_rotation,
                                    float focal_x, float focal_y, float zFar, float zNear,
                                    int tile_row_begin, int tile_row_end,
                                    float* points_xy, float* rgb_depth, float* conic_opacity,
                                    uint64_t* keys_unsorted, uint32_t* values_unsorted, int64_t pair_capacity,
                                    int* curr_offset, void* stream)
{
    return fgs_preprocess_strip_culled(P, positions, shs, opacities, cov3ds, width, height, block_x, block_y,
                                       cam_position, cam_rotation, focal_x, focal_y, zFar, zNear, tile_row_begin, tile_row_end,
                                       points_xy, rgb_depth, conic_opacity, keys_unsorted, values_unsorted, pair_capacity,
                                       curr_offset, nullptr, 0, stream);
}

extern "C" int fgs_preprocess(int P, const float* positions, const float* shs, const float* opacities, const float* cov3ds,
                              int width, int height, int block_x, int block_y,
                              const float* cam_position, const float* cam_rotation,
                              float focal_x, float focal_y, float zFar, float zNear,
                              float* points_xy, float* rgb_depth, float* conic_opacity,
                              uint64_t* keys_unsorted, uint32_t* values_unsorted, int64_t pair_capacity,
                              int* curr_offset, void* stream)
{
    return fgs_preprocess_strip(P, positions, shs, opacities, cov3ds, width, height, block_x, block_y,
                                cam_position, cam_rotation, focal_x, focal_y, zFar, zNear, 0, -1,
                                points_xy, rgb_depth, conic_opacity, keys_unsorted, values_unsorted, pair_capacity,
                                curr_offset, stream);
}
