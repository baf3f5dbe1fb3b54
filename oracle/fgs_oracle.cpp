// CPU oracle for the forward 3D Gaussian Splatting raster path.
//
// THIS IS TEST INFRASTRUCTURE, NOT PRODUCT CODE. It restates, stage by stage and
// in plain C++17 + OpenMP, what the reference's CUDA kernels compute, so that the
// CUDA library can be checked against it and so that a host-core baseline can be
// timed. Nothing in the product package may call into it.
//
// Parity status: the reference ships no tests, golden vectors or CPU path for
// this pipeline, so this restatement is pinned (a) by hand-derivable known-answer
// tests and (b) by fixtures recorded from the reference's own CUDA build run on a
// B200 (tests/golden/). Where the reference uses approximate PTX instructions
// (lg2.approx, sqrt.approx, rsqrt.approx, ex2.approx.ftz) the oracle uses the
// correctly rounded libm functions, so decisions that sit within an ulp or two of
// a threshold may differ from a GPU run; the tests count and bound those cases.
//
// Each function cites the reference lines it follows (paths are relative to the
// reference project root).
//
// Floating point: compiled with -ffp-contract=off. The device compiler contracts
// a*b+c into fma in the reference build; the places where that is expected are
// written with fma_() so that the contraction can be switched (FGSO_CONTRACT).

#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <numeric>
#include <parallel/algorithm>
#include <vector>
#ifdef _OPENMP
#include <omp.h>
#endif

namespace {

int g_contract = 1;  // 1: mirror device FMA contraction, 0: one rounding per operation

inline float fma_(float a, float b, float c) { return g_contract ? std::fmaf(a, b, c) : a * b + c; }
inline double fmad_(double a, double b, double c) { return g_contract ? std::fma(a, b, c) : a * b + c; }

inline uint32_t f2u(float f) { uint32_t u; std::memcpy(&u, &f, 4); return u; }

// ---- host matrices: csrc/cuda_rasterizer/preprocess.cu:420-448 -------------------------------
// GLM stores columns; m[4*c + r] is column c, row r, exactly the float order the
// kernels index (preprocess.cu:69-88). The reference runs this on the host with one
// rounding per operation, in the operation order of GLM 0.9.9.8
// (csrc/glm/detail/type_mat3x3.inl:468-474 for mat3*vec3,
//  csrc/glm/detail/type_mat4x4.inl:630-648 for mat4*mat4).
void view_matrix(const float pos[3], const float rot[9], float view[16])
{
    // pybind.cpp:141-143: GLM column c of cam_rotation = row c of the [3,3] tensor
    const float* c0 = rot + 0; const float* c1 = rot + 3; const float* c2 = rot + 6;
    const float nx = -pos[0], ny = -pos[1], nz = -pos[2];
    float t[3];
    for (int r = 0; r < 3; r++) t[r] = c0[r] * nx + c1[r] * ny + c2[r] * nz;
    const float v[16] = { c0[0], c0[1], c0[2], 0.0f, c1[0], c1[1], c1[2], 0.0f,
                          c2[0], c2[1], c2[2], 0.0f, t[0], t[1], t[2], 1.0f };
    std::memcpy(view, v, sizeof v);
}

void proj_matrix(int width, int height, const float view[16], float fx, float fy, float zFar, float zNear, float proj[16])
{
    const float top = height / (2.0f * fy) * zNear, bottom = -top;
    const float right = width / (2.0f * fx) * zNear, left = -right;
    float P[4][4];  // P[c][r], GLM indexing
    std::memset(P, 0, sizeof P);
    P[0][0] = 2.0f * zNear / (right - left);
    P[1][1] = 2.0f * zNear / (top - bottom);
    P[0][2] = (right + left) / (right - left);
    P[1][2] = (top + bottom) / (top - bottom);
    P[3][2] = 1.0f;
    P[2][2] = 1.0f * zFar / (zFar - zNear);
    P[2][3] = -(zFar * zNear) / (zFar - zNear);
    float A[4][4];  // A = transpose(P): A[c][r] = P[r][c]
    for (int c = 0; c < 4; c++) for (int r = 0; r < 4; r++) A[c][r] = P[r][c];
    for (int c = 0; c < 4; c++)
        for (int r = 0; r < 4; r++)
            proj[4 * c + r] = ((A[0][r] * view[4 * c + 0] + A[1][r] * view[4 * c + 1]) + A[2][r] * view[4 * c + 2]) + A[3][r] * view[4 * c + 3];
}

// preprocess.cu:69-88
inline float xform_row(const float* m, int r, float x, float y, float z)
{
    // ((m[r]*x + m[4+r]*y) + m[8+r]*z) + m[12+r]
    float a = fma_(m[r], x, m[4 + r] * y);
    a = fma_(m[8 + r], z, a);
    return a + m[12 + r];
}

struct Cam {
    float view[16], proj[16], pos[3];
    float tan_fovx, tan_fovy, fx, fy;
    int W, H, bx, by, gx, gy, ty0, ty1;
};

struct Splat {   // per-Gaussian intermediate state of preprocess.cu:270-316
    bool valid = false;
    float px, py, cx, cy, cz, power, depth, l2o;
    int minx, miny, maxx, maxy;
};

// preprocess.cu:103-143
inline void cov2d(const Cam& c, float x, float y, float z, const float* cov3, float out[3])
{
    float tx = xform_row(c.view, 0, x, y, z), ty = xform_row(c.view, 1, x, y, z), tz = xform_row(c.view, 2, x, y, z);
    const float limx = 1.3f * c.tan_fovx, limy = 1.3f * c.tan_fovy;
    const float txtz = tx / tz, tytz = ty / tz;
    tx = std::min(limx, std::max(-limx, txtz)) * tz;
    ty = std::min(limy, std::max(-limy, tytz)) * tz;
    // GLM mat3 from nine scalars fills columns: J[c][r]
    const float J[3][3] = { { c.fx / tz, 0.0f, -(c.fx * tx) / (tz * tz) },
                            { 0.0f, c.fy / tz, -(c.fy * ty) / (tz * tz) },
                            { 0.0f, 0.0f, 0.0f } };
    const float* v = c.view;
    const float Wm[3][3] = { { v[0], v[4], v[8] }, { v[1], v[5], v[9] }, { v[2], v[6], v[10] } };
    float T[3][3], Vt[3][3], Tt[3][3], A[3][3], C[3][3];
    auto mul3 = [](const float a[3][3], const float b[3][3], float r[3][3]) {
        // type_mat3x3.inl:486-519: r[c][q] = a[0][q]*b[c][0] + a[1][q]*b[c][1] + a[2][q]*b[c][2]
        for (int cc = 0; cc < 3; cc++)
            for (int q = 0; q < 3; q++) {
                float s = fma_(a[0][q], b[cc][0], a[1][q] * b[cc][1]);
                r[cc][q] = fma_(a[2][q], b[cc][2], s);
            }
    };
    mul3(Wm, J, T);
    const float Vrk[3][3] = { { cov3[0], cov3[1], cov3[2] }, { cov3[1], cov3[3], cov3[4] }, { cov3[2], cov3[4], cov3[5] } };
    for (int a = 0; a < 3; a++) for (int b = 0; b < 3; b++) { Vt[a][b] = Vrk[b][a]; Tt[a][b] = T[b][a]; }
    mul3(Tt, Vt, A);
    mul3(A, T, C);
    out[0] = C[0][0] + 0.3f; out[1] = C[0][1]; out[2] = C[1][1] + 0.3f;
}

// preprocess.cu:64-67 (double-precision literals promote the whole expression)
inline float ndc2pix(float v, int S) { return (float)(fmad_((double)v + 1.0, (double)S, -1.0) * 0.5); }

// preprocess.cu:282-316 with the strip clamp [ty0,ty1) on tile rows
inline Splat project(const Cam& c, const float* pos, float opacity, const float* cov3, int64_t cnt[2])
{
    Splat s;
    const float x = pos[0], y = pos[1], z = pos[2];
    s.depth = xform_row(c.view, 2, x, y, z);
    if (s.depth <= 0.2f) return s;
    cnt[0]++;
    if (255.0f * opacity < 1.0f) return s;
    cnt[1]++;
    const float hx = xform_row(c.proj, 0, x, y, z), hy = xform_row(c.proj, 1, x, y, z), hw = xform_row(c.proj, 3, x, y, z);
    const float pw = 1.0f / (hw + 0.0000001f);
    const float prx = hx * pw, pry = hy * pw;
    float cv[3];
    cov2d(c, x, y, z, cov3, cv);
    const float det = fma_(cv[0], cv[2], -(cv[1] * cv[1]));
    const float det_inv = 1.0f / det;
    s.cx = cv[2] * det_inv; s.cy = -cv[1] * det_inv; s.cz = cv[0] * det_inv;
    s.l2o = std::log2(opacity);
    const float ln2 = 0.69314718055f;
    s.power = fma_(ln2, s.l2o, ln2 * 8.0f);
    const int width = (int)fma_(1.414214f, std::sqrt(cv[0] * s.power), 1.0f);
    const int height = (int)fma_(1.414214f, std::sqrt(cv[2] * s.power), 1.0f);
    s.px = ndc2pix(prx, c.W); s.py = ndc2pix(pry, c.H);
    // getRect, preprocess.cu:90-100
    auto clampi = [](int v, int hi) { return std::min(hi, std::max(0, v)); };
    s.minx = clampi((int)((s.px - (float)width) / (float)c.bx), c.gx);
    s.miny = clampi((int)((s.py - (float)height) / (float)c.by), c.gy);
    s.maxx = clampi((int)((s.px + (float)width) / (float)c.bx) + 1, c.gx);
    s.maxy = clampi((int)((s.py + (float)height) / (float)c.by) + 1, c.gy);
    s.miny = std::max(s.miny, c.ty0); s.maxy = std::min(s.maxy, c.ty1);
    s.valid = s.maxx > s.minx && s.maxy > s.miny;
    return s;
}

// preprocess.cu:187-194. The reference's build fuses t1's multiply and add at the call for the horizontal edge but
// not at the call for the vertical edge (found by comparing 29.4 M pairs with it on a B200: only this combination
// reproduces every pair); `vertical` selects the form.
inline bool segment_hits(float a, float b, float c, float d, float l, float r, bool vertical)
{
    const float delta = fma_(b, b, -((4.0f * a) * c));
    const float t1 = vertical ? (l - d) * (2.0f * a) + b : fma_(l - d, 2.0f * a, b);
    const float t2 = fma_(r - d, 2.0f * a, b);
    return delta >= 0.0f && (t1 <= 0.0f || t1 * t1 <= delta) && (t2 >= 0.0f || t2 * t2 <= delta);
}

// preprocess.cu:196-241
inline bool tile_hit(const Splat& s, int tx, int ty, int bx, int by)
{
    const int minx = tx * bx, miny = ty * by, maxx = minx + bx - 1, maxy = miny + by - 1;
    if (s.px >= (float)minx && s.px <= (float)maxx && s.py >= (float)miny && s.py <= (float)maxy) return true;
    const float w = 2.0f * s.power;
    float dx = (s.px * 2.0f < (float)(minx + maxx)) ? s.px - (float)minx : s.px - (float)maxx;
    float a = s.cz, b = (-2.0f * s.cy) * dx, c = fma_(s.cx * dx, dx, -w);
    if (segment_hits(a, b, c, s.py, (float)miny, (float)maxy, true)) return true;
    float dy = (s.py * 2.0f < (float)(miny + maxy)) ? s.py - (float)miny : s.py - (float)maxy;
    a = s.cx; b = (-2.0f * s.cy) * dy; c = fma_(s.cz * dy, dy, -w);
    return segment_hits(a, b, c, s.px, (float)minx, (float)maxx, false);
}

// preprocess.cu:145-185
inline void sh_color(const float* sh, const float p[3], const float cam[3], float rgb[3])
{
    const float C0 = 0.28209479177387814f, C1 = 0.4886025119029199f;
    const float C2[5] = { 1.0925484305920792f, -1.0925484305920792f, 0.31539156525252005f, -1.0925484305920792f, 0.5462742152960396f };
    const float C3[7] = { -0.5900435899266435f, 2.890611442640554f, -0.4570457994644658f, 0.3731763325901154f,
                          -0.4570457994644658f, 1.445305721320277f, -0.5900435899266435f };
    float dx = p[0] - cam[0], dy = p[1] - cam[1], dz = p[2] - cam[2];
    const float l2 = fma_(dz, dz, fma_(dx, dx, dy * dy));
    const float rs = 1.0f / std::sqrt(l2);
    const float x = dx * rs, y = dy * rs, z = dz * rs;
    const float xx = x * x, yy = y * y, zz = z * z, xy = x * y, yz = y * z, xz = x * z;
    const float basis[16] = {
        C0, -(C1 * y), C1 * z, -(C1 * x),
        C2[0] * xy, C2[1] * yz, C2[2] * (fma_(2.0f, zz, -xx) - yy), C2[3] * xz, C2[4] * (xx - yy),
        (C3[0] * y) * fma_(3.0f, xx, -yy), (C3[1] * xy) * z, (C3[2] * y) * (fma_(4.0f, zz, -xx) - yy),
        (C3[3] * z) * fma_(-3.0f, yy, fma_(2.0f, zz, -(3.0f * xx))), (C3[4] * x) * (fma_(4.0f, zz, -xx) - yy),
        (C3[5] * z) * (xx - yy), (C3[6] * x) * fma_(-3.0f, yy, xx) };
    for (int ch = 0; ch < 3; ch++) {
        float r = fma_(C0, sh[ch], 0.5f);
        for (int k = 1; k < 16; k++) r = fma_(basis[k], sh[3 * k + ch], r);
        rgb[ch] = std::max(r, 0.0f);
    }
}

inline float ex2_ftz(float x)
{
    float r = std::exp2(x);
    return (std::fabs(r) < 1.17549435e-38f) ? 0.0f : r;   // ex2.approx.ftz flushes subnormal results
}

} // namespace

extern "C" {

// 0/1: switch mirroring of device FMA contraction; returns the previous value.
int fgso_set_contract(int on) { int p = g_contract; g_contract = on ? 1 : 0; return p; }

int fgso_max_threads()
{
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

// preprocess.cu:420-448, 463-466
void fgso_view_proj(int width, int height, const float* pos, const float* rot, float fx, float fy,
                    float zFar, float zNear, float* view, float* proj)
{
    view_matrix(pos, rot, view);
    proj_matrix(width, height, view, fx, fy, zFar, zNear, proj);
}

// Whole preprocess + duplication stage (preprocess.cu:243-418, 452-488).
// Pairs are emitted in a canonical order (Gaussian index, then tile row, then tile
// column); the reference's order is the arrival order of its atomics and is not
// defined. Features of Gaussians that emit no pair are left untouched, as in the
// reference. counters = {P1 (pass near cull), P2 (pass both culls), V (visible), R (pairs)}.
// Returns R, or -1 when R exceeds `capacity` (nothing beyond capacity is written).
int64_t fgso_preprocess(int P, const float* positions, const float* shs, const float* opacities, const float* cov3ds,
                        int width, int height, int block_x, int block_y,
                        const float* cam_pos, const float* cam_rot, float fx, float fy, float zFar, float zNear,
                        int tile_y0, int tile_y1,
                        float* points_xy, float* rgb_depth, float* conic_opacity,
                        uint64_t* keys, uint32_t* values, int64_t capacity, int64_t* counters)
{
    Cam c;
    fgso_view_proj(width, height, cam_pos, cam_rot, fx, fy, zFar, zNear, c.view, c.proj);
    std::memcpy(c.pos, cam_pos, 12);
    c.tan_fovx = width / (2.0f * fx); c.tan_fovy = height / (2.0f * fy);
    c.fx = fx; c.fy = fy; c.W = width; c.H = height; c.bx = block_x; c.by = block_y;
    c.gx = (width + block_x - 1) / block_x; c.gy = (height + block_y - 1) / block_y;
    c.ty0 = std::max(0, tile_y0); c.ty1 = (tile_y1 < 0) ? c.gy : std::min(c.gy, tile_y1);

    const int CH = 4096;
    const int nch = (P + CH - 1) / CH;
    std::vector<std::vector<uint64_t>> ck(nch);
    std::vector<std::vector<uint32_t>> cvv(nch);
    int64_t p1 = 0, p2 = 0, vis = 0;
    const float log2e = 1.4426950216293334961f;
#pragma omp parallel for schedule(dynamic, 1) reduction(+ : p1, p2, vis)
    for (int ch = 0; ch < nch; ch++) {
        auto& K = ck[ch]; auto& Vv = cvv[ch];
        for (int i = ch * CH; i < std::min(P, (ch + 1) * CH); i++) {
            int64_t cnt[2] = { 0, 0 };
            Splat s = project(c, positions + 3 * (size_t)i, opacities[i], cov3ds + 6 * (size_t)i, cnt);
            p1 += cnt[0]; p2 += cnt[1];
            if (!s.valid) continue;
            bool any = false;
            for (int ty = s.miny; ty < s.maxy; ty++)
                for (int tx = s.minx; tx < s.maxx; tx++)
                    if (tile_hit(s, tx, ty, block_x, block_y)) {
                        K.push_back(((uint64_t)(uint32_t)(ty * c.gx + tx) << 32) | f2u(s.depth));
                        Vv.push_back((uint32_t)i);
                        any = true;
                    }
            if (!any) continue;
            vis++;
            // preprocess.cu:411-417
            points_xy[2 * (size_t)i] = s.px; points_xy[2 * (size_t)i + 1] = s.py;
            float* co = conic_opacity + 4 * (size_t)i;
            co[0] = (-0.5f * log2e) * s.cx; co[1] = -log2e * s.cy; co[2] = (-0.5f * log2e) * s.cz; co[3] = s.l2o;
            float rgb[3];
            sh_color(shs + 48 * (size_t)i, positions + 3 * (size_t)i, c.pos, rgb);
            float* rd = rgb_depth + 4 * (size_t)i;
            rd[0] = rgb[0]; rd[1] = rgb[1]; rd[2] = rgb[2]; rd[3] = s.depth;
        }
    }
    int64_t R = 0;
    std::vector<int64_t> off(nch + 1, 0);
    for (int ch = 0; ch < nch; ch++) { off[ch] = R; R += (int64_t)ck[ch].size(); }
    if (counters) { counters[0] = p1; counters[1] = p2; counters[2] = vis; counters[3] = R; }
    if (R > capacity) return -1;
#pragma omp parallel for schedule(dynamic, 8)
    for (int ch = 0; ch < nch; ch++) {
        if (ck[ch].empty()) continue;
        std::memcpy(keys + off[ch], ck[ch].data(), ck[ch].size() * 8);
        std::memcpy(values + off[ch], cvv[ch].data(), cvv[ch].size() * 4);
    }
    return R;
}

// sort.cu:9-24: position of the highest set bit plus one (== bit_length)
uint32_t fgso_higher_msb(uint32_t n)
{
    uint32_t msb = sizeof(n) * 4, step = msb;
    while (step > 1) { step /= 2; if (n >> msb) msb += step; else msb -= step; }
    if (n >> msb) msb++;
    return msb;
}

// sort.cu:28-44: stable sort of (key, value) pairs on key bits [0, 32 + bit_length(#tiles)).
// The reference calls a library radix sort whose contract is exactly that; a stable
// comparison sort on the masked key gives the same output.
void fgso_sort(int64_t n, int width, int height, int block_x, int block_y,
               const uint64_t* keys_in, const uint32_t* vals_in, uint64_t* keys_out, uint32_t* vals_out)
{
    const uint32_t tiles = (uint32_t)(((width + block_x - 1) / block_x) * ((height + block_y - 1) / block_y));
    const int end_bit = 32 + (int)fgso_higher_msb(tiles);
    const uint64_t mask = end_bit >= 64 ? ~0ull : ((1ull << end_bit) - 1);
    std::vector<int64_t> idx((size_t)n);
    std::iota(idx.begin(), idx.end(), 0);
    // multi-threaded merge sort; stable like the reference's radix sort
    __gnu_parallel::stable_sort(idx.begin(), idx.end(), [&](int64_t a, int64_t b) { return (keys_in[a] & mask) < (keys_in[b] & mask); });
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; i++) { keys_out[i] = keys_in[idx[i]]; vals_out[i] = vals_in[idx[i]]; }
}

// render.cu:9-31 and the memset at render.cu:557
void fgso_ranges(int64_t n, const uint64_t* keys_sorted, int num_tiles, int32_t* ranges)
{
    std::memset(ranges, 0, sizeof(int32_t) * 2 * (size_t)num_tiles);
    for (int64_t i = 0; i < n; i++) {
        const uint32_t cur = (uint32_t)(keys_sorted[i] >> 32);
        if (i == 0) ranges[2 * cur] = 0;
        else {
            const uint32_t prev = (uint32_t)(keys_sorted[i - 1] >> 32);
            if (cur != prev) { ranges[2 * prev + 1] = (int32_t)i; ranges[2 * cur] = (int32_t)i; }
        }
        if (i == n - 1) ranges[2 * cur + 1] = (int32_t)n;
    }
}

// Blend stage: render.cu:40-73 (pixel math, quantisation), 199-547 (control flow).
// Stop rule (render.cu:315, 394-407, 486-487): splats are consumed two at a time;
// after each pair the tile stops when every pixel of the BLOCK_X x BLOCK_Y tile,
// including pixels that lie outside the image, has T < 1e-4. Pixels below the
// threshold keep accumulating until the whole tile stops.
// out_u8 [H,W,3] is what the reference writes. The float outputs have no reference
// counterpart and are defined here: out_rgb = C + T'*bg (T' = T flushed to 0 below
// 1e-4), out_alpha = 1 - T, out_depth = sum of depth_i * alpha_i * T_i.
// consumed[tile] receives the number of splats blended for that tile (may be null).
// Only tile rows [tile_y0, tile_y1) are rendered (tile_y1 < 0: all rows).
void fgso_render(int width, int height, int block_x, int block_y,
                 const float* points_xy, const float* rgb_depth, const float* conic_opacity,
                 const uint32_t* vals_sorted, const int32_t* ranges, const float* bg,
                 int tile_y0, int tile_y1,
                 uint8_t* out_u8, float* out_rgb, float* out_alpha, float* out_depth, int32_t* consumed)
{
    const int gx = (width + block_x - 1) / block_x, gy = (height + block_y - 1) / block_y;
    const int y0 = std::max(0, tile_y0), y1 = tile_y1 < 0 ? gy : std::min(gy, tile_y1);
    const int npx = block_x * block_y;
#pragma omp parallel for schedule(dynamic, 4) collapse(2)
    for (int ty = y0; ty < y1; ty++)
        for (int tx = 0; tx < gx; tx++) {
            const int tile = ty * gx + tx;
            const int32_t r0 = ranges[2 * tile], r1 = ranges[2 * tile + 1];
            std::vector<float> T(npx, 1.0f), Cr(npx, 0.0f), Cg(npx, 0.0f), Cb(npx, 0.0f), D(npx, 0.0f);
            int32_t k = r0;
            while (k < r1) {
                const int32_t kend = std::min(r1, k + 2);
                for (; k < kend; k++) {
                    const uint32_t g = vals_sorted[k];
                    const float sx = points_xy[2 * (size_t)g], sy = points_xy[2 * (size_t)g + 1];
                    const float* co = conic_opacity + 4 * (size_t)g;
                    const float* rd = rgb_depth + 4 * (size_t)g;
                    for (int py = 0; py < block_y; py++)
                        for (int px = 0; px < block_x; px++) {
                            const int p = py * block_x + px;
                            const float dx = sx - (float)(tx * block_x + px), dy = sy - (float)(ty * block_y + py);
                            float pw = fma_(co[0] * dx, dx, co[3]);
                            pw = fma_(co[2] * dy, dy, pw);
                            pw = fma_(co[1] * dx, dy, pw);
                            const float alpha = ex2_ftz(pw);
                            const float aT = alpha * T[p];
                            Cr[p] = fma_(rd[0], aT, Cr[p]); Cg[p] = fma_(rd[1], aT, Cg[p]); Cb[p] = fma_(rd[2], aT, Cb[p]);
                            D[p] = fma_(rd[3], aT, D[p]);
                            T[p] -= aT;
                        }
                }
                bool done = true;
                for (int p = 0; p < npx && done; p++) done = T[p] < 0.0001f;
                if (done) break;
            }
            if (consumed) consumed[tile] = k - r0;
            auto enc = [](float x) { return (uint8_t)std::min(std::max(0.0f, x * 255.0f), 255.0f); };
            for (int py = 0; py < block_y; py++)
                for (int px = 0; px < block_x; px++) {
                    const int X = tx * block_x + px, Y = ty * block_y + py;
                    if (X >= width || Y >= height) continue;
                    const int p = py * block_x + px;
                    const size_t pix = (size_t)Y * width + X;
                    const float Traw = T[p];
                    const float Tq = (r1 > r0 && Traw < 0.0001f) ? 0.0f : Traw;
                    const float c3[3] = { fma_(Tq, bg[0], Cr[p]), fma_(Tq, bg[1], Cg[p]), fma_(Tq, bg[2], Cb[p]) };
                    if (out_u8) for (int ch = 0; ch < 3; ch++) out_u8[3 * pix + ch] = enc(c3[ch]);
                    if (out_rgb) for (int ch = 0; ch < 3; ch++) out_rgb[3 * pix + ch] = c3[ch];
                    if (out_alpha) out_alpha[pix] = 1.0f - Traw;
                    if (out_depth) out_depth[pix] = D[p];
                }
        }
}

} // extern "C"
