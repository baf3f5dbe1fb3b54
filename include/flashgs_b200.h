/*
 * flashgs_b200 -- C ABI of the B200 (sm_100a) forward 3D Gaussian Splatting raster path.
 *
 * The entry points below are what a binding of the reference's operator API
 * (namespace flashgs, csrc/ops.h:32-65, bound to Python in csrc/pybind.cpp:233-271)
 * needs: plain pointers and sizes, no C++ or torch types. Unless stated otherwise
 * every pointer is a DEVICE pointer on the current CUDA device, every buffer is
 * owned by the caller, nothing is allocated and no state is kept between calls,
 * all work is enqueued on `stream` (a cudaStream_t passed as void*, NULL = the
 * legacy default stream, which is what the reference's bindings always use) and
 * the call returns without waiting for the GPU.
 *
 * Every function returns FGS_OK (0) or one of the FGS_ERR_* codes. Failures
 * detected on the device (pair buffer overflow, a look-back wait that ran out of
 * its poll budget) are recorded in a per-device status word that
 * fgs_device_status() reads.
 */
#ifndef FLASHGS_B200_H
#define FLASHGS_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FGS_OK 0
#define FGS_ERR_BAD_ARG 1          /* null pointer, non-positive size, unsupported tile shape */
#define FGS_ERR_CUDA 2             /* a CUDA runtime call or kernel launch failed */
#define FGS_ERR_PAIR_OVERFLOW 4    /* more (tile, Gaussian) pairs than the pair buffers hold */
#define FGS_ERR_LOOKBACK_TIMEOUT 8 /* a bounded device-side wait gave up */
#define FGS_ERR_TEMP_TOO_SMALL 16  /* sort scratch smaller than fgs_sort_temp_bytes() */
#define FGS_ERR_BOUNDS 32          /* checked build only (-DFGS_DEBUG_BOUNDS): a kernel met an index outside its extent
                                      and skipped the access; see fgs_debug_bounds_report in flashgs_b200_test.h */

/* Length, in 32-bit words, of a per-tile pair-count table (fgs_preprocess_prepared -> fgs_sort_pairs_counted). */
#define FGS_TILE_COUNT_WORDS 65536

/* Version of this ABI; bumped when a signature changes. */
int fgs_abi_version(void);

/* Human-readable name of a status code (static storage). */
const char* fgs_status_string(int status);

/*
 * Reads (and, if `reset` is non-zero, clears) the device status word of the
 * current device: an OR of the FGS_ERR_* codes raised by kernels since the last
 * reset. Synchronises `stream`. Returns a negative value if the read itself failed.
 */
int fgs_device_status(int reset, void* stream);

/*
 * Host-only helper: the 4x4 view and view-projection matrices (column-major,
 * 16 floats each) the preprocess stage uses. Replaces getViewMatrix /
 * getProjectionMatrix (csrc/cuda_rasterizer/preprocess.cu:420-448).
 * `cam_position` (3 floats) and `cam_rotation` (9 floats, camera-to-world,
 * row-major) are HOST pointers.
 */
int fgs_view_proj_matrices(int width, int height, const float* cam_position, const float* cam_rotation,
                           float focal_x, float focal_y, float zFar, float zNear,
                           float* view16, float* proj16);

/*
 * Cull, project, shade and duplicate. Replaces flashgs::preprocess
 * (csrc/ops.h:32-39, csrc/cuda_rasterizer/preprocess.cu:243-418,452-488).
 *
 *   positions [P,3], shs [P,48] ([coef][rgb]), opacities [P], cov3ds [P,6]   inputs, fp32
 *   cam_position [3], cam_rotation [9]                                       HOST pointers
 *   points_xy [P,2], rgb_depth [P,4], conic_opacity [P,4]                    outputs, written only for
 *                                                                            Gaussians that emit a pair
 *   keys_unsorted [pair_capacity] = (tile_id << 32) | float_bits(depth)
 *   values_unsorted [pair_capacity] = Gaussian index
 *   curr_offset [1]   in/out pair counter; the caller zeroes it before the call
 *                     (example.py:69); it keeps counting past pair_capacity while
 *                     stores beyond the capacity are dropped and
 *                     FGS_ERR_PAIR_OVERFLOW is raised in the device status word.
 *
 * The order of pairs is unspecified (as in the reference, where it is the arrival
 * order of atomics).
 */
int fgs_preprocess(int P, const float* positions, const float* shs, const float* opacities, const float* cov3ds,
                   int width, int height, int block_x, int block_y,
                   const float* cam_position, const float* cam_rotation,
                   float focal_x, float focal_y, float zFar, float zNear,
                   float* points_xy, float* rgb_depth, float* conic_opacity,
                   uint64_t* keys_unsorted, uint32_t* values_unsorted, int64_t pair_capacity,
                   int* curr_offset, void* stream);

/*
 * Same as fgs_preprocess, restricted to tile rows [tile_row_begin, tile_row_end):
 * pairs are emitted only for tiles of those rows, with GLOBAL tile ids, so that the
 * union of the strips' pair sets equals the whole-frame pair set. Used to split one
 * frame into horizontal strips across GPUs. No counterpart in the reference, which
 * is single-GPU (csrc/cuda_rasterizer/preprocess.cu:314 is the rule that drops
 * Gaussians whose clamped tile rectangle is empty; the strip clamp reuses it).
 */
int fgs_preprocess_strip(int P, const float* positions, const float* shs, const float* opacities, const float* cov3ds,
                         int width, int height, int block_x, int block_y,
                         const float* cam_position, const float* cam_rotation,
                         float focal_x, float focal_y, float zFar, float zNear,
                         int tile_row_begin, int tile_row_end,
                         float* points_xy, float* rgb_depth, float* conic_opacity,
                         uint64_t* keys_unsorted, uint32_t* values_unsorted, int64_t pair_capacity,
                         int* curr_offset, void* stream);

/*
 * fgs_preprocess_strip with scratch for an index list (`cull_scratch`, at least P + 1 ints, contents undefined on
 * entry and exit): a first, cheap kernel lists the Gaussians that pass the near and opacity culls and whose
 * vertical reach (bounded from the trace of the 3-D covariance) meets the strip; the preprocess kernel then runs on
 * that list only. A rank that renders one strip of N thus does the expensive work for about 1/N of the scene. Same
 * pair set and feature records as fgs_preprocess_strip (the pair ORDER differs; neither is defined). The list is
 * built for a whole frame as well (rows 0 and -1): it then drops the Gaussians left, right, above and below the
 * image. With a null scratch the call is fgs_preprocess_strip. No counterpart in the reference.
 */
int fgs_preprocess_strip_culled(int P, const float* positions, const float* shs, const float* opacities, const float* cov3ds,
                                int width, int height, int block_x, int block_y,
                                const float* cam_position, const float* cam_rotation,
                                float focal_x, float focal_y, float zFar, float zNear,
                                int tile_row_begin, int tile_row_end,
                                float* points_xy, float* rgb_depth, float* conic_opacity,
                                uint64_t* keys_unsorted, uint32_t* values_unsorted, int64_t pair_capacity,
                                int* curr_offset, int* cull_scratch, int64_t cull_scratch_ints, void* stream);

/*
 * Scene preparation for fgs_preprocess_prepared, once per scene (not per frame): fills `bounds` [P,4] (16-byte
 * aligned) with one record per Gaussian -- position and trace(covariance) * ln(256 * opacity), negative for an
 * opacity below 1/255 -- which is all the index-list kernel needs to decide whether a Gaussian can reach a strip.
 * No counterpart in the reference.
 */
int fgs_scene_bounds(int P, const float* positions, const float* opacities, const float* cov3ds, float* bounds, void* stream);

/*
 * fgs_preprocess_strip_culled whose index-list kernel streams the prepared records of fgs_scene_bounds (16 bytes per
 * Gaussian) instead of position, opacity and covariance (40 bytes): that kernel runs over the WHOLE scene on every
 * GPU that renders a strip, so it is the part of a frame that does not shrink with the number of GPUs. The list
 * is a superset of fgs_preprocess_strip_culled's; pairs and feature records are the same. `scene_bounds` may be
 * NULL (then this is fgs_preprocess_strip_culled); with it, `cull_scratch` is required. The records must describe
 * the arrays passed here.
 * `tile_counts` (NULL, or FGS_TILE_COUNT_WORDS words): preprocess knows each pair's tile at the moment it emits the
 * pair, so it can count the pairs per tile as it goes (the table is zeroed first; entry t = pairs of tile t that
 * were stored, i.e. that fitted the pair buffers); fgs_sort_pairs_counted then skips the pass over all keys that
 * would recount them. Ignored for images with more than FGS_TILE_COUNT_WORDS tiles. No counterpart in the reference.
 */
int fgs_preprocess_prepared(int P, const float* positions, const float* shs, const float* opacities, const float* cov3ds,
                            int width, int height, int block_x, int block_y,
                            const float* cam_position, const float* cam_rotation,
                            float focal_x, float focal_y, float zFar, float zNear,
                            int tile_row_begin, int tile_row_end,
                            float* points_xy, float* rgb_depth, float* conic_opacity,
                            uint64_t* keys_unsorted, uint32_t* values_unsorted, int64_t pair_capacity,
                            int* curr_offset, int* cull_scratch, int64_t cull_scratch_ints,
                            const float* scene_bounds, uint32_t* tile_counts, void* stream);

/*
 * fgs_preprocess_prepared with CUDA events around its two kernels: waits for the stream and fills
 * kernel_ms2[0] (the index-list kernel; 0 without scratch) and kernel_ms2[1] (the main kernel). A measurement
 * aid for benchmarks: it creates and destroys events and blocks the host. No counterpart in the reference.
 */
int fgs_preprocess_profile(int P, const float* positions, const float* shs, const float* opacities, const float* cov3ds,
                           int width, int height, int block_x, int block_y,
                           const float* cam_position, const float* cam_rotation,
                           float focal_x, float focal_y, float zFar, float zNear,
                           int tile_row_begin, int tile_row_end,
                           float* points_xy, float* rgb_depth, float* conic_opacity,
                           uint64_t* keys_unsorted, uint32_t* values_unsorted, int64_t pair_capacity,
                           int* curr_offset, int* cull_scratch, int64_t cull_scratch_ints,
                           const float* scene_bounds, uint32_t* tile_counts, void* stream, float* kernel_ms2);

/*
 * Scratch bytes fgs_sort_pairs needs for up to `num_rendered` pairs. Replaces
 * flashgs::get_sort_buffer_size (csrc/ops.h:47, csrc/cuda_rasterizer/sort.cu:46-54). Host-only.
 */
size_t fgs_sort_temp_bytes(int64_t num_rendered);

/*
 * Sort of (key, value) pairs on key bits [0, 32 + bit_length(#tiles)); bits at or above that width travel with
 * their keys and are never compared. Replaces flashgs::sort_gaussian (csrc/ops.h:41-45,
 * csrc/cuda_rasterizer/sort.cu:28-44). Inputs are left intact; outputs go to keys_sorted / values_sorted; `temp`
 * must be 16-byte aligned and at least fgs_sort_temp_bytes(num_rendered) bytes.
 *
 * Pairs whose sorted bits are EQUAL (two Gaussians of one tile at exactly the same depth): the reference's
 * library sort is stable, so it leaves them in input order -- and the input order of the raster path is the
 * arrival order of preprocess's atomics, which changes from run to run. fgs_sort_pairs returns them in ascending
 * order of their values (Gaussian indices) instead, for images of at most 65536 tile values: that is the stable
 * result for one of the possible arrival orders, it makes the sorted list a function of the SET of pairs (the same
 * frame twice gives the same bytes), and it lets the sort group the pairs by tile without any block waiting for
 * another. (Keys that carry bits above the sorted width, and images with more tiles, keep input order.)
 * fgs_sort_pairs_stable has the same signature and the library sort's exact contract -- equal keys in input
 * order, always -- at the price of look-back digit passes; use it where the pair list does not come from
 * fgs_preprocess and its order matters.
 */
int fgs_sort_pairs(int num_rendered, int width, int height, int block_x, int block_y,
                   void* temp, size_t temp_bytes,
                   const uint64_t* keys_unsorted, const uint32_t* values_unsorted,
                   uint64_t* keys_sorted, uint32_t* values_sorted, void* stream);
int fgs_sort_pairs_stable(int num_rendered, int width, int height, int block_x, int block_y,
                          void* temp, size_t temp_bytes,
                          const uint64_t* keys_unsorted, const uint32_t* values_unsorted,
                          uint64_t* keys_sorted, uint32_t* values_sorted, void* stream);

/*
 * fgs_sort_pairs given the pairs per tile (`tile_counts`, FGS_TILE_COUNT_WORDS words, as fgs_preprocess_prepared
 * leaves them for the same image, tile shape and pair list): the sort starts from that table instead of reading
 * all keys once to build it. The table is checked against num_rendered on the device: if its total differs the
 * sort moves nothing, raises FGS_ERR_BAD_ARG in the device status word and leaves the outputs undefined (it never
 * writes outside them). With a NULL table, or an image with more than FGS_TILE_COUNT_WORDS tiles, it is
 * fgs_sort_pairs. No counterpart in the reference.
 */
int fgs_sort_pairs_counted(int num_rendered, int width, int height, int block_x, int block_y,
                           void* temp, size_t temp_bytes,
                           const uint64_t* keys_unsorted, const uint32_t* values_unsorted,
                           uint64_t* keys_sorted, uint32_t* values_sorted, const uint32_t* tile_counts, void* stream);

/*
 * fgs_sort_pairs for callers that have no scratch buffer to give and must not allocate one: code that runs
 * where device allocation is off limits (inside another framework's memory plan, in a callback, in a process
 * whose allocator is owned by someone else). It has no counterpart in the reference, whose sort always takes
 * caller scratch. The scratch lives in a fixed array inside the library (about 5.8 MB that every GPU loading
 * the library holds until the process ends), so the call is limited to fgs_sort_static_max_pairs() = 262144
 * pairs and returns FGS_ERR_TEMP_TOO_SMALL beyond that (FGS_ERR_BAD_ARG for a negative count). Nothing is allocated or freed, by this library or by any
 * library it calls. The first call on each device looks up the array's device address (with that device
 * current); make that first call outside any stream capture. All calls on a device share the one array and
 * it keeps what the previous call left (the entry point clears the parts that must start at zero), so two
 * calls that overlap on the GPU -- different streams, or different host threads -- race: keep them ordered.
 * (The address look-up itself is behind a lock; it is the array's CONTENTS that concurrent calls would share.)
 * Inputs, outputs and result are those of fgs_sort_pairs.
 */
int fgs_sort_static_max_pairs(void);
int fgs_sort_pairs_static(int num_rendered, int width, int height, int block_x, int block_y,
                          const uint64_t* keys_unsorted, const uint32_t* values_unsorted,
                          uint64_t* keys_sorted, uint32_t* values_sorted, void* stream);

/*
 * fgs_sort_pairs_counted with CUDA events recorded around each of its kernel launches; waits for the stream and
 * fills launch_ms[i] and launch_kind[i] for every launch i (kinds: 0 histogram, 1 tile-grouping or digit pass,
 * 2 tile segments, 3 in-block tile sort); *num_launches receives the count (0 when num_rendered is 0). Both arrays
 * must hold `capacity` >= 24 entries. A measurement aid for benchmarks: it creates and destroys events
 * and blocks the host, so it is not for the frame loop. No counterpart in the reference.
 */
int fgs_sort_pairs_profile(int num_rendered, int width, int height, int block_x, int block_y,
                           void* temp, size_t temp_bytes,
                           const uint64_t* keys_unsorted, const uint32_t* values_unsorted,
                           uint64_t* keys_sorted, uint32_t* values_sorted, const uint32_t* tile_counts, void* stream,
                           float* launch_ms, int* launch_kind, int capacity, int* num_launches);

/*
 * Tile ranges + front-to-back alpha blending into an 8-bit RGB image.
 * Replace flashgs::render_16x16 / render_32x16 / render_32x32
 * (csrc/ops.h:49-65, csrc/cuda_rasterizer/render.cu:549-608).
 *
 *   ranges [tiles,2] int32   scratch/out: [first, one-past-last) index of each tile in the
 *                            sorted list, (0,0) for tiles without pairs
 *   bg_color [3]             HOST pointer
 *   out_color [H,W,3] uint8  every pixel of the image is written; nothing outside it is
 */
int fgs_render_16x16(int num_rendered, int width, int height,
                     const float* points_xy, const float* rgb_depth, const float* conic_opacity,
                     const uint64_t* keys_sorted, const uint32_t* values_sorted,
                     int* ranges, const float* bg_color, uint8_t* out_color, void* stream);
int fgs_render_32x16(int num_rendered, int width, int height,
                     const float* points_xy, const float* rgb_depth, const float* conic_opacity,
                     const uint64_t* keys_sorted, const uint32_t* values_sorted,
                     int* ranges, const float* bg_color, uint8_t* out_color, void* stream);
int fgs_render_32x32(int num_rendered, int width, int height,
                     const float* points_xy, const float* rgb_depth, const float* conic_opacity,
                     const uint64_t* keys_sorted, const uint32_t* values_sorted,
                     int* ranges, const float* bg_color, uint8_t* out_color, void* stream);

/*
 * General form of the render entry points: any of the three tile shapes, an
 * optional restriction to tile rows [tile_row_begin, tile_row_end) (only those
 * rows of the image are written; pass 0 and -1 for the whole frame), and optional
 * float outputs that the reference does not have (any of them may be NULL):
 *   out_rgb [H,W,3]  = C + T*bg before quantisation
 *   out_alpha [H,W]  = 1 - T
 *   out_depth [H,W]  = sum of depth_i * alpha_i * T_i
 *   consumed [tiles] = number of splats blended per tile (the reference's stop rule,
 *                      csrc/cuda_rasterizer/render.cu:315,394-407)
 * out_color may be NULL when only float outputs are wanted.
 *   tile_order [tiles of the rendered rows]  (may be NULL) the order in which the tiles are taken up, as whole-frame
 *                      tile ids; every tile of the rendered rows must appear once (an entry outside them is ignored,
 *                      a tile that is missing is not rendered). The image does not depend on the order; the time
 *                      does: the launch ends with its slowest tiles, so handing over the tiles in descending order of
 *                      the `consumed` counts of the previous frame of the same view shortens its tail.
 */
int fgs_render_ex(int block_x, int block_y, int num_rendered, int width, int height,
                  const float* points_xy, const float* rgb_depth, const float* conic_opacity,
                  const uint64_t* keys_sorted, const uint32_t* values_sorted,
                  int* ranges, const float* bg_color,
                  int tile_row_begin, int tile_row_end,
                  uint8_t* out_color, float* out_rgb, float* out_alpha, float* out_depth, int* consumed,
                  const int* tile_order, void* stream);

/*
 * One whole frame in a single call that never waits for the GPU: zero the pair counter, preprocess (optionally a
 * strip of tile rows), sort, tile ranges, blend. The pair count stays on the device (curr_offset), so there is no
 * host read-back between the stages as the reference's operator signatures force (example.py:79 reads the
 * counter because csrc/ops.h:41,49 take it as a host int); the caller may read curr_offset afterwards, at its
 * own pace, to learn the count. All buffers as in the per-stage entry points; pair_capacity is the length of the
 * four pair buffers and sort_temp must hold fgs_sort_temp_bytes(pair_capacity) (when it also holds P + 1 ints,
 * its head carries preprocess's index list of the Gaussians that can reach the image, see
 * fgs_preprocess_strip_culled: the sort does not need its scratch until preprocess is done). If the frame produces more
 * pairs than pair_capacity the surplus is dropped, the image is built from the pairs that fit and
 * FGS_ERR_PAIR_OVERFLOW is raised in the device status word. `consumed` and `tile_order` (both may be NULL) are
 * fgs_render_ex's, `scene_bounds` (may be NULL) is fgs_preprocess_prepared's. No counterpart in the reference.
 */
int fgs_render_frame(int P, const float* positions, const float* shs, const float* opacities, const float* cov3ds,
                     int width, int height, int block_x, int block_y,
                     const float* cam_position, const float* cam_rotation,
                     float focal_x, float focal_y, float zFar, float zNear, const float* bg_color,
                     float* points_xy, float* rgb_depth, float* conic_opacity,
                     uint64_t* keys_unsorted, uint32_t* values_unsorted,
                     uint64_t* keys_sorted, uint32_t* values_sorted, int64_t pair_capacity,
                     void* sort_temp, size_t sort_temp_bytes, int* ranges, int* curr_offset,
                     int tile_row_begin, int tile_row_end, uint8_t* out_color,
                     int* consumed, const int* tile_order, const float* scene_bounds, void* stream);

/*
 * Tile ranges only (the first half of the render entry points). Replaces
 * identifyTileRanges plus the memset before it (csrc/cuda_rasterizer/render.cu:9-31,557).
 */
int fgs_tile_ranges(int num_rendered, int num_tiles, const uint64_t* keys_sorted, int* ranges, void* stream);

/*
 * Scene loading (host only, no GPU work). Replace loadPly_torch / computeCov3D (csrc/pybind.cpp:12-120):
 * a binary PLY with 62 floats per vertex (position, normal, f_dc, f_rest channel-major, opacity logit,
 * log-scale, quaternion w,x,y,z) becomes position [n,3], shs [n,48] as [coef][rgb], opacity = sigmoid,
 * cov3d [n,6] (xx, xy, xz, yy, yz, zz). fgs_ply_vertex_count returns the header's vertex count or a negative
 * FGS_ERR_* value; fgs_ply_load fills HOST arrays sized for that count.
 */
long long fgs_ply_vertex_count(const char* path);
int fgs_ply_load(const char* path, long long n, float* position, float* shs, float* opacity, float* cov3d);

#ifdef __cplusplus
}
#endif
#endif /* FLASHGS_B200_H */
