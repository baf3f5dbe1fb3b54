// Tile ranges and per-tile front-to-back alpha blending for sm_100a.
//
// Replaces flashgs::render_16x16 / 32x16 / 32x32 (csrc/cuda_rasterizer/render.cu:549-608):
// the memset + identifyTileRanges pair (render.cu:9-31,557) and renderCUDA (render.cu:199-547).
//
// Tile ranges: one thread per tile finds the first and one-past-last position of its tile id
// in the sorted key list by binary search (about 2*log2(R) cached reads per tile instead of a
// pass over all R keys plus a memset); tiles without pairs get (0,0) as in the reference.
//
// Blend: one warp per tile, laid out 8x4 over the tile; a thread owns a TX x TY block of pixels
// (2x4 for 16x16 tiles). The sorted splat list of the tile is consumed in batches of 32: lane l
// reads the l-th index of the batch (one coalesced 128-byte read) and gathers that splat's
// three feature records straight into shared memory with cp.async (8 + 16 + 16 bytes), two
// batches in flight, so that the gather of batch b+1 and the index read of batch b+2 overlap
// the arithmetic of batch b. All lanes then read each splat from shared memory as a broadcast.
// The exponent of a splat at pixel (x, y) is split into per-column terms (computed TX times),
// a per-row term (TY times) and two FMAs per pixel; alpha = ex2.approx.ftz(exponent). The arithmetic
// runs on horizontal pixel pairs with the packed fp32x2 add/mul/fma instructions of sm_100.
//
// Stop rule, identical to the reference's (render.cu:315,394-407,486-487): splats are consumed
// two at a time and after each pair a warp vote ends the tile once every pixel of the tile
// (also those outside the image) has T < 1e-4; pixels already below the threshold keep
// accumulating until then. There is no alpha clamp and no minimum-alpha skip (render.cu:40-52).
//
// Output: the tile's 8-bit RGB rows are assembled in shared memory and leave as 16-byte stores
// when the image width is a multiple of the tile width; otherwise as guarded byte stores. Nothing
// outside the image is written.

#include "fgs_common.cuh"

namespace fgs {
namespace {

#ifndef FGS_BLEND_WARPS
#define FGS_BLEND_WARPS 2
#endif
constexpr int BLEND_WARPS = FGS_BLEND_WARPS;   // tiles per block (one warp each); 1 lets the hardware scheduler balance tiles individually
constexpr int BATCH = 32;           // splats per staged batch (one per lane)
constexpr int STAGES = 2;

constexpr int RANGE_TILES = 256, RANGE_THREADS = RANGE_TILES + 32;
__global__ void tile_ranges_kernel(const uint64_t* __restrict__ keys, int n, const int* __restrict__ n_dev, int num_tiles,
                                   int2* __restrict__ ranges)
{
    chain_release();
    chain_wait();   // nothing is read or written before the kernels ahead on the stream are complete
    const int tile = blockIdx.x * RANGE_TILES + threadIdx.x;
    if (n_dev != nullptr) {   // count produced on the device by the same frame (bounded by the buffers' capacity n)
        const int v = *n_dev;
        n = v < 0 ? 0 : (v < n ? v : n);
    }
    // first index whose tile id is >= t
    auto lower = [&](uint32_t t) {
        int lo = 0, hi = n;
        while (lo < hi) {
            const int mid = (int)(((unsigned)lo + (unsigned)hi) >> 1);
            if ((uint32_t)(__ldg(keys + mid) >> 32) < t) lo = mid + 1; else hi = mid;
        }
        return lo;
    };
    // One search per thread: a tile's list ends where the next tile's starts. Threads 0..RANGE_TILES-1 search the
    // starts of the block's tiles, thread RANGE_TILES the start of the tile behind them.
    __shared__ int s_first[RANGE_TILES + 1];
    if (threadIdx.x <= RANGE_TILES) s_first[threadIdx.x] = lower((uint32_t)tile);
    __syncthreads();
    if (threadIdx.x >= RANGE_TILES || tile >= num_tiles) return;
    const int first = s_first[threadIdx.x], last = s_first[threadIdx.x + 1];
    if (FGS_INDEX_OK(tile, num_tiles)) ranges[tile] = (last > first) ? make_int2(first, last) : make_int2(0, 0);
}

__device__ __forceinline__ float ex2_approx_ftz(float x)
{
    float y;
    asm volatile("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ void cp_async_8(void* smem, const void* gmem)
{
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"((unsigned)__cvta_generic_to_shared(smem)), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async_16(void* smem, const void* gmem)
{
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((unsigned)__cvta_generic_to_shared(smem)), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// Two fp32 lanes in one 64-bit register: Blackwell issues add/mul/fma on such pairs as one instruction
// (each lane rounds exactly like the scalar instruction), which halves the issue slots of the pixel math.
typedef unsigned long long f32x2;
__device__ __forceinline__ f32x2 pack2(float lo, float hi) { f32x2 r; asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi)); return r; }
__device__ __forceinline__ void unpack2(f32x2 v, float& lo, float& hi) { asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v)); }
__device__ __forceinline__ f32x2 fma2(f32x2 a, f32x2 b, f32x2 c) { f32x2 d; asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c)); return d; }
__device__ __forceinline__ f32x2 mul2(f32x2 a, f32x2 b) { f32x2 d; asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b)); return d; }
__device__ __forceinline__ f32x2 sub2(f32x2 a, f32x2 b) { f32x2 d; asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b)); return d; }

// render.cu:54-57
__device__ __forceinline__ uint8_t encode_u8(float x) { return (uint8_t)fminf(fmaxf(0.0f, x * 255.0f), 255.0f); }

struct BlendStage {
    float2 xy[BATCH];
    float4 con[BATCH];    // conic_opacity record
    float4 rgbd[BATCH];   // rgb_depth record
};

template <int BX, int BY, bool EXTRA>
// Resident blocks per SM the register budget is set for: 12 gives 80 registers without spills. 14 (72 registers, one
// spilled) measured the same on the 6 M-Gaussian frame, 16 (64 registers) 4 % slower, no limit (92 registers) 20 % slower.
#ifndef FGS_BLEND_MIN_BLOCKS
#define FGS_BLEND_MIN_BLOCKS 12
#endif
__global__ void __launch_bounds__(BLEND_WARPS * 32, FGS_BLEND_MIN_BLOCKS)
blend_kernel(const int2* __restrict__ ranges, const uint32_t* __restrict__ point_list,
             int width, int height, int grid_x, int row_begin, int num_strip_tiles,
             const float2* __restrict__ points_xy, const float4* __restrict__ rgb_depth,
             const float4* __restrict__ conic_opacity,
             float bg_r, float bg_g, float bg_b, int vector_store, int list_len, const int* __restrict__ list_len_dev,
             uint8_t* __restrict__ out_color, float* __restrict__ out_rgb, float* __restrict__ out_alpha,
             float* __restrict__ out_depth, int* __restrict__ consumed, const int* __restrict__ tile_order, int row_end)
{
    chain_release();
    chain_wait();   // nothing is read or written before the kernels ahead on the stream are complete
    constexpr int TX = BX / 8, TY = BY / 4;
    __shared__ __align__(16) BlendStage s_stage[BLEND_WARPS][STAGES];
    __shared__ __align__(16) uint8_t s_out[BLEND_WARPS][BY][BX * 3];

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int strip_tile = blockIdx.x * BLEND_WARPS + warp;
    if (strip_tile >= num_strip_tiles) return;          // whole warp leaves; no block-wide barrier is used
    // The warp's tile: the strip's tiles in row-major order, or in the order the caller asks for (heaviest first keeps
    // the launch's tail short). An entry that is not a tile of the strip is ignored.
    int tile_y = row_begin + strip_tile / grid_x;
    int tile_x = strip_tile - (strip_tile / grid_x) * grid_x;
    if (tile_order != nullptr) {
        const int t = tile_order[strip_tile];
        tile_y = t / grid_x;
        tile_x = t - tile_y * grid_x;
        if (t < 0 || tile_y < row_begin || tile_y >= row_end) return;
    }
    const int tile = tile_y * grid_x + tile_x;
    int2 range = ranges[tile];
#ifdef FGS_DEBUG_BOUNDS
    {   // checked build: a tile's range must lie inside the sorted list
        int len = list_len;
        if (list_len_dev != nullptr) { const int v = *list_len_dev; len = v < 0 ? 0 : (v < len ? v : len); }
        if (range.y != range.x && !(FGS_INDEX_OK(range.x, len) && FGS_INDEX_OK(range.y - 1, len) && range.y > range.x)) range = make_int2(0, 0);
    }
#endif
    const int n = range.y - range.x;
    BlendStage* stage = s_stage[warp];

    const int lx = lane & 7, ly = lane >> 3;
    const int px0 = tile_x * BX + lx * TX, py0 = tile_y * BY + ly * TY;
    // Pixels are handled as horizontal pairs (columns 2p and 2p+1 of the thread's block) in packed registers.
    constexpr int PX = TX / 2;
    f32x2 px2[PX], py2[TY];
#pragma unroll
    for (int p = 0; p < PX; p++) px2[p] = pack2((float)(px0 + 2 * p), (float)(px0 + 2 * p + 1));
#pragma unroll
    for (int i = 0; i < TY; i++) py2[i] = pack2((float)(py0 + i), (float)(py0 + i));

    f32x2 T2[TY][PX], Cr2[TY][PX], Cg2[TY][PX], Cb2[TY][PX], D2[TY][PX];
#pragma unroll
    for (int i = 0; i < TY; i++)
#pragma unroll
        for (int p = 0; p < PX; p++) { T2[i][p] = pack2(1.0f, 1.0f); Cr2[i][p] = Cg2[i][p] = Cb2[i][p] = D2[i][p] = pack2(0.0f, 0.0f); }

    int used = 0;
    if (n > 0) {
        const uint32_t* list = point_list + range.x;
        const int batches = (n + BATCH - 1) / BATCH;
        auto gather = [&](int b, uint32_t idx) {
            if (b * BATCH + lane < n) {
                BlendStage& s = stage[b % STAGES];
                cp_async_8(&s.xy[lane], points_xy + idx);
                cp_async_16(&s.con[lane], conic_opacity + idx);
                cp_async_16(&s.rgbd[lane], rgb_depth + idx);
            }
            cp_async_commit();
        };
        uint32_t idx_next = (lane < n) ? __ldg(list + lane) : 0u;
        gather(0, idx_next);
        idx_next = (BATCH + lane < n) ? __ldg(list + BATCH + lane) : 0u;

        bool stop = false;
        for (int b = 0; b < batches && !stop; b++) {
            if (b + 1 < batches) {
                gather(b + 1, idx_next);
                idx_next = ((b + 2) * BATCH + lane < n) ? __ldg(list + (b + 2) * BATCH + lane) : 0u;
                cp_async_wait<1>();
            } else {
                cp_async_wait<0>();
            }
            __syncwarp();
            const BlendStage& s = stage[b % STAGES];
            const int cnt = min(BATCH, n - b * BATCH);
            for (int k = 0; k < cnt; k += 2) {
#pragma unroll
                for (int h = 0; h < 2; h++) {
                    if (k + h < cnt) {
                        const float2 xy = s.xy[k + h];
                        const float4 co = s.con[k + h];
                        const float4 rd = s.rgbd[k + h];
                        const f32x2 sx2 = pack2(xy.x, xy.x), sy2 = pack2(xy.y, xy.y);
                        const f32x2 cx2 = pack2(co.x, co.x), cy2 = pack2(co.y, co.y), cz2 = pack2(co.z, co.z), cw2 = pack2(co.w, co.w);
                        const f32x2 r2 = pack2(rd.x, rd.x), g2 = pack2(rd.y, rd.y), b2 = pack2(rd.z, rd.z), z2 = pack2(rd.w, rd.w);
                        f32x2 A2[PX], B2[PX];   // per column: co.w + co.x*dx^2 and co.y*dx
#pragma unroll
                        for (int p = 0; p < PX; p++) {
                            const f32x2 dx2 = sub2(sx2, px2[p]);
                            A2[p] = fma2(mul2(cx2, dx2), dx2, cw2);
                            B2[p] = mul2(cy2, dx2);
                        }
#pragma unroll
                        for (int i = 0; i < TY; i++) {
                            const f32x2 dy2 = sub2(sy2, py2[i]);
                            // The exponent in the reference's operation order (render.cu:44): w + (x*dx)*dx, then + (z*dy)*dy,
                            // then + (y*dx)*dy, each step one fused multiply-add. With it the 8-bit image of the headline
                            // workload is byte for byte the reference's. Folding z*dy into the last step saves one multiply
                            // per row and splat (8 % of the kernel) but rounds differently: about 1 byte in 17 000 then
                            // differs by one level (FGS_BLEND_FOLDED_EXPONENT selects that form).
#ifndef FGS_BLEND_FOLDED_EXPONENT
                            const f32x2 rz2 = mul2(cz2, dy2);
#endif
#pragma unroll
                            for (int p = 0; p < PX; p++) {
                                float p0, p1;
#ifndef FGS_BLEND_FOLDED_EXPONENT
                                unpack2(fma2(B2[p], dy2, fma2(rz2, dy2, A2[p])), p0, p1);
#else
                                const f32x2 t2 = fma2(cz2, dy2, B2[p]);
                                unpack2(fma2(t2, dy2, A2[p]), p0, p1);
#endif
                                const f32x2 aT2 = mul2(pack2(ex2_approx_ftz(p0), ex2_approx_ftz(p1)), T2[i][p]);
                                Cr2[i][p] = fma2(r2, aT2, Cr2[i][p]);
                                Cg2[i][p] = fma2(g2, aT2, Cg2[i][p]);
                                Cb2[i][p] = fma2(b2, aT2, Cb2[i][p]);
                                if (EXTRA) D2[i][p] = fma2(z2, aT2, D2[i][p]);
                                T2[i][p] = sub2(T2[i][p], aT2);
                            }
                        }
                    }
                }
                bool done = true;
#pragma unroll
                for (int i = 0; i < TY; i++)
#pragma unroll
                    for (int p = 0; p < PX; p++) {
                        float t0, t1;
                        unpack2(T2[i][p], t0, t1);
                        done = done && (t0 < 0.0001f) && (t1 < 0.0001f);
                    }
                if (__all_sync(FULL_MASK, done)) { stop = true; used = b * BATCH + min(k + 2, cnt); break; }
            }
            __syncwarp();
        }
        if (!stop) used = n;
        cp_async_wait<0>();
    }
    if (consumed && lane == 0) consumed[tile] = used;

    // ---- write-out (render.cu:59-73; background-only tiles: render.cu:530-546, here bounds-checked) ----
    float T[TY][TX], Cr[TY][TX], Cg[TY][TX], Cb[TY][TX], D[TY][TX];
#pragma unroll
    for (int i = 0; i < TY; i++)
#pragma unroll
        for (int p = 0; p < PX; p++) {
            unpack2(T2[i][p], T[i][2 * p], T[i][2 * p + 1]);
            unpack2(Cr2[i][p], Cr[i][2 * p], Cr[i][2 * p + 1]);
            unpack2(Cg2[i][p], Cg[i][2 * p], Cg[i][2 * p + 1]);
            unpack2(Cb2[i][p], Cb[i][2 * p], Cb[i][2 * p + 1]);
            unpack2(D2[i][p], D[i][2 * p], D[i][2 * p + 1]);
        }
    uint8_t (*so)[BX * 3] = s_out[warp];
#pragma unroll
    for (int i = 0; i < TY; i++)
#pragma unroll
        for (int j = 0; j < TX; j++) {
            const float Traw = T[i][j];
            const float Tq = (n > 0 && Traw < 0.0001f) ? 0.0f : Traw;
            const float r = Cr[i][j] + Tq * bg_r, g = Cg[i][j] + Tq * bg_g, bl = Cb[i][j] + Tq * bg_b;
            const int cx = lx * TX + j, cy = ly * TY + i;
            so[cy][cx * 3 + 0] = encode_u8(r);
            so[cy][cx * 3 + 1] = encode_u8(g);
            so[cy][cx * 3 + 2] = encode_u8(bl);
            if (EXTRA) {
                const int X = px0 + j, Y = py0 + i;
                if (X < width && Y < height && FGS_INDEX_OK((size_t)Y * width + X, (size_t)height * width)) {
                    const size_t pix = (size_t)Y * width + X;
                    if (out_rgb) { out_rgb[3 * pix] = r; out_rgb[3 * pix + 1] = g; out_rgb[3 * pix + 2] = bl; }
                    if (out_alpha) out_alpha[pix] = 1.0f - Traw;
                    if (out_depth) out_depth[pix] = D[i][j];
                }
            }
        }
    if (out_color == nullptr) return;
    __syncwarp();
    const int X0 = tile_x * BX, Y0 = tile_y * BY;
    if (vector_store) {
        constexpr int CHUNKS_PER_ROW = BX * 3 / 16;
        for (int c = lane; c < BY * CHUNKS_PER_ROW; c += 32) {
            const int row = c / CHUNKS_PER_ROW, part = c - row * CHUNKS_PER_ROW;
            if (Y0 + row < height && FGS_INDEX_OK(((size_t)(Y0 + row) * width + X0) * 3 + part * 16 + 15, (size_t)height * width * 3)) {
                const uint4 v = *reinterpret_cast<const uint4*>(&so[row][part * 16]);
                *reinterpret_cast<uint4*>(out_color + ((size_t)(Y0 + row) * width + X0) * 3 + part * 16) = v;
            }
        }
    } else {
        for (int c = lane; c < BY * BX * 3; c += 32) {
            const int row = c / (BX * 3), col = c - row * (BX * 3);
            const int X = X0 + col / 3;
            if (Y0 + row < height && X < width && FGS_INDEX_OK(((size_t)(Y0 + row) * width + X) * 3 + (col - (col / 3) * 3), (size_t)height * width * 3))
                out_color[((size_t)(Y0 + row) * width + X) * 3 + (col - (col / 3) * 3)] = so[row][col];
        }
    }
}

template <int BX, int BY>
int launch_render(int num_rendered, int width, int height,
                  const float* points_xy, const float* rgb_depth, const float* conic_opacity,
                  const uint64_t* keys_sorted, const uint32_t* values_sorted, int* ranges, const float* bg,
                  int row_begin, int row_end,
                  uint8_t* out_color, float* out_rgb, float* out_alpha, float* out_depth, int* consumed, cudaStream_t st,
                  const int* n_dev = nullptr, const int* tile_order = nullptr)
{
    const int grid_x = (width + BX - 1) / BX, grid_y = (height + BY - 1) / BY;
    const int num_tiles = grid_x * grid_y;
    if (row_begin < 0) row_begin = 0;
    if (row_end < 0 || row_end > grid_y) row_end = grid_y;
    chain_launch(tile_ranges_kernel, dim3((num_tiles + RANGE_TILES - 1) / RANGE_TILES), dim3(RANGE_THREADS), 0, st, keys_sorted, num_rendered, n_dev, num_tiles,
                                                               reinterpret_cast<int2*>(ranges));
    if (row_end <= row_begin) return launch_status();
    const int strip_tiles = (row_end - row_begin) * grid_x;
    const int blocks = (strip_tiles + BLEND_WARPS - 1) / BLEND_WARPS;
    const int vec = (out_color != nullptr) && (width % BX == 0) && aligned16(out_color);
    const bool extra = out_rgb || out_alpha || out_depth;
    if (extra)
        chain_launch(blend_kernel<BX, BY, true>, dim3(blocks), dim3(BLEND_WARPS * 32), 0, st, 
            reinterpret_cast<const int2*>(ranges), values_sorted, width, height, grid_x, row_begin, strip_tiles,
            reinterpret_cast<const float2*>(points_xy), reinterpret_cast<const float4*>(rgb_depth),
            reinterpret_cast<const float4*>(conic_opacity), bg[0], bg[1], bg[2], vec, num_rendered, n_dev,
            out_color, out_rgb, out_alpha, out_depth, consumed, tile_order, row_end);
    else
        chain_launch(blend_kernel<BX, BY, false>, dim3(blocks), dim3(BLEND_WARPS * 32), 0, st, 
            reinterpret_cast<const int2*>(ranges), values_sorted, width, height, grid_x, row_begin, strip_tiles,
            reinterpret_cast<const float2*>(points_xy), reinterpret_cast<const float4*>(rgb_depth),
            reinterpret_cast<const float4*>(conic_opacity), bg[0], bg[1], bg[2], vec, num_rendered, n_dev,
            out_color, nullptr, nullptr, nullptr, consumed, tile_order, row_end);
    return launch_status();
}

} // namespace

int sort_pairs_device_count(int capacity, const int* n_dev, int width, int height, int block_x, int block_y,
                            void* temp, size_t temp_bytes, const uint64_t* keys_unsorted, const uint32_t* values_unsorted,
                            uint64_t* keys_sorted, uint32_t* values_sorted, void* stream, bool counts_in_scratch);
void sort_scratch_regions(int64_t capacity, size_t* tile_count_off, size_t* list_off, size_t* list_bytes);
} // namespace fgs

extern "C" int fgs_preprocess_prepared(int P, const float* positions, const float* shs, const float* opacities, const float* cov3ds,
                                       int width, int height, int block_x, int block_y,
                                       const float* cam_position, const float* cam_rotation,
                                       float focal_x, float focal_y, float zFar, float zNear,
                                       int tile_row_begin, int tile_row_end,
                                       float* points_xy, float* rgb_depth, float* conic_opacity,
                                       uint64_t* keys_unsorted, uint32_t* values_unsorted, int64_t pair_capacity,
                                       int* curr_offset, int* cull_scratch, int64_t cull_scratch_ints,
                                       const float* scene_bounds, uint32_t* tile_counts, void* stream);

FGS_BOUNDS_REPORT_FN(fgs_debug_bounds_render)

#ifdef FGS_DEBUG_BOUNDS
namespace fgs {
__global__ void bounds_selftest_kernel(int index, int extent, int* touched)
{
    if (FGS_INDEX_OK(index, extent)) *touched = 1;   // the "access" the check guards
}
} // namespace fgs
// Checked build: runs the check itself on (index, extent) with one thread, touching a caller-owned int only when the
// index is inside the extent; lets a test see that a violation is counted, recorded and skipped.
extern "C" int fgs_debug_bounds_selftest(int index, int extent, int* touched, void* stream)
{
    if (!touched) return FGS_ERR_BAD_ARG;
    fgs::bounds_selftest_kernel<<<1, 1, 0, static_cast<cudaStream_t>(stream)>>>(index, extent, touched);
    return fgs::launch_status();
}
#endif

// One whole frame without any host round trip: preprocess -> sort -> tile ranges -> blend, the pair count staying on
// the device. See include/flashgs_b200.h.
extern "C" int fgs_render_frame(int P, const float* positions, const float* shs, const float* opacities, const float* cov3ds,
                                int width, int height, int block_x, int block_y,
                                const float* cam_position, const float* cam_rotation,
                                float focal_x, float focal_y, float zFar, float zNear, const float* bg_color,
                                float* points_xy, float* rgb_depth, float* conic_opacity,
                                uint64_t* keys_unsorted, uint32_t* values_unsorted,
                                uint64_t* keys_sorted, uint32_t* values_sorted, int64_t pair_capacity,
                                void* sort_temp, size_t sort_temp_bytes, int* ranges, int* curr_offset,
                                int tile_row_begin, int tile_row_end, uint8_t* out_color,
                                int* consumed, const int* tile_order, const float* scene_bounds, void* stream)
{
    using namespace fgs;
    if (scene_bounds != nullptr && !aligned16(scene_bounds)) return FGS_ERR_BAD_ARG;
    if (pair_capacity <= 0 || pair_capacity >= (1 << 30) || !curr_offset || !out_color || !bg_color || !ranges) return FGS_ERR_BAD_ARG;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (cudaMemsetAsync(curr_offset, 0, sizeof(int), st) != cudaSuccess) return FGS_ERR_CUDA;
    // The sort's scratch is idle while preprocess runs. Preprocess leaves two things in it: the list of the Gaussians
    // that can reach the image (or the strip), in the alternate value buffer at the scratch's end, and the pairs per
    // tile, in the sort's own table -- the sort then starts from that table instead of counting the pairs again.
    int* cull_list = nullptr;
    uint32_t* tile_counts = nullptr;
    if (sort_temp != nullptr && aligned16(sort_temp) && sort_temp_bytes >= fgs_sort_temp_bytes(pair_capacity)) {
        size_t count_off = 0, list_off = 0, list_bytes = 0;
        sort_scratch_regions(pair_capacity, &count_off, &list_off, &list_bytes);
        if (list_bytes >= ((size_t)P + 1) * sizeof(int)) cull_list = reinterpret_cast<int*>(static_cast<char*>(sort_temp) + list_off);
        const int64_t tiles = (block_x > 0 && block_y > 0 && width > 0 && height > 0)
                                  ? (int64_t)((width + block_x - 1) / block_x) * ((height + block_y - 1) / block_y) : FGS_TILE_COUNT_WORDS;
        if (tiles < FGS_TILE_COUNT_WORDS)
            tile_counts = reinterpret_cast<uint32_t*>(static_cast<char*>(sort_temp) + count_off);
    }
    int rc = fgs_preprocess_prepared(P, positions, shs, opacities, cov3ds, width, height, block_x, block_y, cam_position,
                                     cam_rotation, focal_x, focal_y, zFar, zNear, tile_row_begin, tile_row_end, points_xy,
                                     rgb_depth, conic_opacity, keys_unsorted, values_unsorted, pair_capacity, curr_offset,
                                     cull_list, cull_list ? (int64_t)P + 1 : 0, cull_list ? scene_bounds : nullptr, tile_counts, stream);
    if (rc != FGS_OK) return rc;
    rc = sort_pairs_device_count((int)pair_capacity, curr_offset, width, height, block_x, block_y, sort_temp, sort_temp_bytes,
                                 keys_unsorted, values_unsorted, keys_sorted, values_sorted, stream, tile_counts != nullptr);
    if (rc != FGS_OK) return rc;
#define FGS_FRAME_CASE(BX, BY)                                                                                          \
    if (block_x == BX && block_y == BY)                                                                                 \
        return launch_render<BX, BY>((int)pair_capacity, width, height, points_xy, rgb_depth, conic_opacity, keys_sorted, \
                                     values_sorted, ranges, bg_color, tile_row_begin, tile_row_end, out_color, nullptr,  \
                                     nullptr, nullptr, consumed, st, curr_offset, tile_order);
    FGS_FRAME_CASE(16, 16)
    FGS_FRAME_CASE(32, 16)
    FGS_FRAME_CASE(32, 32)
#undef FGS_FRAME_CASE
    return FGS_ERR_BAD_ARG;
}

extern "C" int fgs_tile_ranges(int num_rendered, int num_tiles, const uint64_t* keys_sorted, int* ranges, void* stream)
{
    if (num_rendered < 0 || num_tiles <= 0 || !ranges || (num_rendered > 0 && !keys_sorted)) return FGS_ERR_BAD_ARG;
    fgs::chain_launch(fgs::tile_ranges_kernel, dim3((num_tiles + fgs::RANGE_TILES - 1) / fgs::RANGE_TILES), dim3(fgs::RANGE_THREADS), 0, static_cast<cudaStream_t>(stream), 
        keys_sorted, num_rendered, nullptr, num_tiles, reinterpret_cast<int2*>(ranges));
    return fgs::launch_status();
}

extern "C" int fgs_render_ex(int block_x, int block_y, int num_rendered, int width, int height,
                             const float* points_xy, const float* rgb_depth, const float* conic_opacity,
                             const uint64_t* keys_sorted, const uint32_t* values_sorted,
                             int* ranges, const float* bg_color,
                             int tile_row_begin, int tile_row_end,
                             uint8_t* out_color, float* out_rgb, float* out_alpha, float* out_depth, int* consumed,
                             const int* tile_order, void* stream)
{
    using namespace fgs;
    if (num_rendered < 0 || width <= 0 || height <= 0 || !ranges || !bg_color) return FGS_ERR_BAD_ARG;
    if (!out_color && !out_rgb && !out_alpha && !out_depth && !consumed) return FGS_ERR_BAD_ARG;
    if (num_rendered > 0 && (!points_xy || !rgb_depth || !conic_opacity || !keys_sorted || !values_sorted)) return FGS_ERR_BAD_ARG;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
#define FGS_RENDER_CASE(BX, BY)                                                                                        \
    if (block_x == BX && block_y == BY)                                                                                \
        return launch_render<BX, BY>(num_rendered, width, height, points_xy, rgb_depth, conic_opacity, keys_sorted,     \
                                     values_sorted, ranges, bg_color, tile_row_begin, tile_row_end, out_color, out_rgb, \
                                     out_alpha, out_depth, consumed, st, nullptr, tile_order);
    FGS_RENDER_CASE(16, 16)
    FGS_RENDER_CASE(32, 16)
    FGS_RENDER_CASE(32, 32)
#undef FGS_RENDER_CASE
    return FGS_ERR_BAD_ARG;
}

#define FGS_RENDER_ENTRY(NAME, BX, BY)                                                                               \
    extern "C" int NAME(int num_rendered, int width, int height, const float* points_xy, const float* rgb_depth,     \
                        const float* conic_opacity, const uint64_t* keys_sorted, const uint32_t* values_sorted,      \
                        int* ranges, const float* bg_color, uint8_t* out_color, void* stream)                        \
    {                                                                                                                \
        if (!out_color) return FGS_ERR_BAD_ARG;                                                                      \
        return fgs_render_ex(BX, BY, num_rendered, width, height, points_xy, rgb_depth, conic_opacity, keys_sorted,  \
                             values_sorted, ranges, bg_color, 0, -1, out_color, nullptr, nullptr, nullptr, nullptr,  \
                             nullptr, stream);                                                                       \
    }
FGS_RENDER_ENTRY(fgs_render_16x16, 16, 16)
FGS_RENDER_ENTRY(fgs_render_32x16, 32, 16)
FGS_RENDER_ENTRY(fgs_render_32x32, 32, 32)
#undef FGS_RENDER_ENTRY
