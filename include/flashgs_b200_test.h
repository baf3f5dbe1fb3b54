/*
 * flashgs_b200 -- switches that exist for the test-suite only.
 *
 * These three functions flip process-global switches inside libflashgs_b200.so. They are not part of the
 * operator ABI (include/flashgs_b200.h), are not synchronised with anything -- a call changes the behaviour of
 * every later preprocess or sort call of the process, from whatever thread -- and have no counterpart in the
 * reference. The tests use them, from one thread, to compare two code paths that must agree and to make a bounded
 * device-side wait run out without faulting or hanging the GPU; they always restore the default afterwards.
 * Production code must not call them.
 */
#ifndef FLASHGS_B200_TEST_H
#define FLASHGS_B200_TEST_H

#ifdef __cplusplus
extern "C" {
#endif

/*
 * Non-zero: the next preprocess calls run the exact tile test on every tile of a splat's bounding rectangle, as
 * the reference does (csrc/cuda_rasterizer/preprocess.cu:318-410), instead of first narrowing each row's column
 * range in closed form. Both settings must give the same pair set. 0 restores the default.
 */
void fgs_debug_preprocess_no_column_cull(int on);

/*
 * Non-zero: the next sorts skip the tile-bucketed paths and run plain look-back digit passes over all live key
 * bits, the direct equivalent of the library call at csrc/cuda_rasterizer/sort.cu:35-39. 0 restores the default.
 */
void fgs_debug_sort_plain(int on);

/*
 * 0: every kernel is launched plainly; non-zero (the default): the kernels of a frame are launched with the
 * programmatic-serialization attribute, so that a kernel's blocks are resident and waiting when the kernel before it
 * ends. Results are the same either way; the tests compare the two.
 */
void fgs_debug_chained_launches(int on);

/*
 * part >= 0: in the next look-back digit passes (fgs_sort_pairs_stable, or any sort of an image with more than
 * 65536 tiles) the partition with this index does not publish its look-back words, so later partitions run out of
 * their poll budget: the sort returns, FGS_ERR_LOOKBACK_TIMEOUT is raised in the device status word and the output
 * is meaningless. -1 restores the default.
 */
void fgs_debug_sort_skip_publish(int part);

/*
 * The two functions below exist only in the CHECKED flavour of the library (libflashgs_b200_checked.so, built with
 * -DFGS_DEBUG_BOUNDS by `python -m flashgs_b200.build --checked`). In that flavour every kernel compares each global
 * store, each index it computed from data and each computed shared-memory index with the extent of what it
 * addresses, and SKIPS an access that falls outside (nothing faults or traps); fgs_device_status() then carries
 * FGS_ERR_BOUNDS. It stands in for a memory checker on machines where none can be run, at a cost in speed.
 *
 * fgs_debug_bounds_report: waits for the device, then fills out12 (may be NULL) with 3 x 4 values -- for the
 * preprocess, sort and render kernels: number of violations, source line of the first one, its index, its extent
 * -- clears the counters if `reset` is non-zero, and returns the total number of violations (negative on error).
 * fgs_debug_bounds_selftest: applies the check to (index, extent) in a one-thread kernel that writes 1 to the
 * caller-owned device int `touched` only if the index passes: shows that a violation is counted and skipped.
 */
long long fgs_debug_bounds_report(unsigned long long* out12, int reset);
int fgs_debug_bounds_selftest(int index, int extent, int* touched, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* FLASHGS_B200_TEST_H */
