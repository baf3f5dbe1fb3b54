// Scene loader: binary PLY of a trained 3D Gaussian Splatting model -> the four input arrays.
//
// Replaces loadPly_torch / computeCov3D (csrc/pybind.cpp:12-120). Host code only (this file holds no kernel;
// it is compiled with the rest of the library, with host FMA contraction off). The record layout is the one
// the reference reads: 62 little-endian floats per vertex -- position 3, normal 3, f_dc 3, f_rest 45
// (channel-major), opacity (logit) 1, log-scale 3, rotation quaternion 4 (w, x, y, z)
// (csrc/pybind.cpp:12-20). Outputs: position [N,3]; shs [N,48] re-laid out as [coef][rgb]
// (csrc/pybind.cpp:105-111); opacity = sigmoid; cov3d [N,6] from exp(scale) and the normalised quaternion
// (csrc/pybind.cpp:22-56,112-117). The arithmetic follows the reference's operation order with one
// rounding per operation, so the arrays are bit-identical to the reference's.
//
// The header is scanned like the reference does (whitespace-separated tokens: the count follows the token
// "vertex", the data follow the first newline after "end_header"); the file is read in large blocks instead
// of one read per vertex.

#include "fgs_common.cuh"

#include <cmath>
#include <cstdio>
#include <cstring>
#include <string>
#include <vector>

namespace {

constexpr int kFloatsPerVertex = 62;

// Returns the vertex count and leaves `f` positioned at the first data byte; < 0 on error.
long long read_header(FILE* f)
{
    long long count = 0;
    bool end_header = false;
    char tok[256];
    while (std::fscanf(f, "%255s", tok) == 1) {
        if (std::strcmp(tok, "vertex") == 0) {
            if (std::fscanf(f, "%lld", &count) != 1 || count <= 0) return -2;   // "Vertex number is not positive"
        } else if (std::strcmp(tok, "end_header") == 0) {
            end_header = true;
            std::fgetc(f);   // the newline that ends the header
            break;
        }
    }
    if (!end_header) return -3;   // "Cannot find end of header"
    return count;
}

// csrc/pybind.cpp:22-56 with GLM 0.9.9.8 operation order (mat3 from nine scalars fills columns;
// M = S * R scales row r by s[r]; Sigma = transpose(M) * M).
void cov3d_from(const float s[3], const float q[4], float* cov)
{
    const float r = q[0], x = q[1], y = q[2], z = q[3];
    const float R[3][3] = {
        { 1.f - 2.f * (y * y + z * z), 2.f * (x * y - r * z), 2.f * (x * z + r * y) },
        { 2.f * (x * y + r * z), 1.f - 2.f * (x * x + z * z), 2.f * (y * z - r * x) },
        { 2.f * (x * z - r * y), 2.f * (y * z + r * x), 1.f - 2.f * (x * x + y * y) } };
    float M[3][3];   // [column][row]
    for (int c = 0; c < 3; c++)
        for (int rr = 0; rr < 3; rr++) {
            // S[0][rr]*R[c][0] + S[1][rr]*R[c][1] + S[2][rr]*R[c][2] with S diagonal: the two zero products add +-0
            float acc = 0.f;
            for (int k = 0; k < 3; k++) {
                const float term = (k == rr ? s[rr] : 0.f) * R[c][k];
                acc = (k == 0) ? term : acc + term;
            }
            M[c][rr] = acc;
        }
    auto sig = [&](int c, int rr) { return M[rr][0] * M[c][0] + M[rr][1] * M[c][1] + M[rr][2] * M[c][2]; };
    cov[0] = sig(0, 0); cov[1] = sig(0, 1); cov[2] = sig(0, 2);
    cov[3] = sig(1, 1); cov[4] = sig(1, 2); cov[5] = sig(2, 2);
}

} // namespace

// Number of vertices declared by the PLY header, or a negative FGS_ERR_* value.
extern "C" long long fgs_ply_vertex_count(const char* path)
{
    if (!path) return -FGS_ERR_BAD_ARG;
    FILE* f = std::fopen(path, "rb");
    if (!f) return -FGS_ERR_BAD_ARG;
    const long long n = read_header(f);
    std::fclose(f);
    return n < 0 ? -FGS_ERR_BAD_ARG : n;
}

// Fills HOST arrays position [n,3], shs [n,48], opacity [n], cov3d [n,6]; n must be the header's count.
extern "C" int fgs_ply_load(const char* path, long long n, float* position, float* shs, float* opacity, float* cov3d)
{
    if (!path || n <= 0 || !position || !shs || !opacity || !cov3d) return FGS_ERR_BAD_ARG;
    FILE* f = std::fopen(path, "rb");
    if (!f) return FGS_ERR_BAD_ARG;
    const long long declared = read_header(f);
    if (declared != n) { std::fclose(f); return FGS_ERR_BAD_ARG; }
    const long long block = 1 << 16;
    std::vector<float> buf((size_t)block * kFloatsPerVertex);
    for (long long v0 = 0; v0 < n; v0 += block) {
        const long long cnt = (n - v0 < block) ? (n - v0) : block;
        if ((long long)std::fread(buf.data(), sizeof(float) * kFloatsPerVertex, (size_t)cnt, f) != cnt) {
            std::fclose(f);
            return FGS_ERR_BAD_ARG;   // truncated file (the reference would use whatever the stream left behind)
        }
        for (long long i = 0; i < cnt; i++) {
            const float* r = buf.data() + (size_t)i * kFloatsPerVertex;
            const long long v = v0 + i;
            std::memcpy(position + 3 * v, r, 12);
            const float* sh_in = r + 6;   // after position and normal
            float* sh = shs + 48 * v;
            sh[0] = sh_in[0]; sh[1] = sh_in[1]; sh[2] = sh_in[2];
            for (int j = 1; j < 16; j++) {
                sh[3 * j + 0] = sh_in[(j - 1) + 3];
                sh[3 * j + 1] = sh_in[(j - 1) + 16 + 2];
                sh[3 * j + 2] = sh_in[(j - 1) + 16 * 2 + 1];
            }
            opacity[v] = 1.0f / (1.0f + std::exp(-r[54]));
            const float s[3] = { std::exp(r[55]), std::exp(r[56]), std::exp(r[57]) };
            // glm::normalize: v * inversesqrt(dot(v, v)), dot summed as (x*x + y*y) + (z*z + w*w)
            const float q0 = r[58], q1 = r[59], q2 = r[60], q3 = r[61];
            const float inv = 1.0f / std::sqrt((q0 * q0 + q1 * q1) + (q2 * q2 + q3 * q3));
            const float q[4] = { q0 * inv, q1 * inv, q2 * inv, q3 * inv };
            cov3d_from(s, q, cov3d + 6 * v);
        }
    }
    std::fclose(f);
    return FGS_OK;
}
