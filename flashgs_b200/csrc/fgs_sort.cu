// Sort of (64-bit key, 32-bit value) pairs on the live key bits, sm_100a.
//
// Replaces the library radix sort the reference calls (csrc/cuda_rasterizer/sort.cu:28-44): a sort on key bits
// [0, end_bit), end_bit = 32 + bit_length(#tiles) (csrc/cuda_rasterizer/sort.cu:9-24,39), inputs preserved, outputs in
// separate buffers. Two variants share the in-block tile sorts:
//
//   * fgs_sort_pairs (the default): the pairs are first GROUPED BY TILE, in any order inside a tile, by two passes in
//     which no block waits for another (per-tile counts -> cursors; a block reserves room for each of its runs with
//     one atomicAdd): tile_hist_kernel (unless the caller hands the counts over), tile_scan_kernel,
//     multisplit_kernel; then every tile is ordered in shared memory by (depth bits, value): local_sort_kernel,
//     long_list_kernel for lists longer than 4096. Pairs with identical keys come out in ascending order of their
//     values, so the result depends on the set of pairs only, not on their input order.
//   * fgs_sort_pairs_stable: the library sort's contract (identical keys in input order): one histogram kernel over
//     the tile digits, one "onesweep" kernel per tile digit -- a block (256 sorting threads and 64 look-back
//     threads) takes the next partition of 4096 pairs from a ticket counter, ranks its keys by digit (lanes with
//     equal digits meet through bit masks in shared memory; per-warp counters keep the order), publishes its
//     per-digit counts and obtains the counts of all earlier partitions by decoupled look-back, then moves keys and
//     values through shared memory so that every digit's run leaves as contiguous global stores -- segments_kernel,
//     and the tile sorts by (depth bits, position). Images with more than 65 535 tiles go through such passes for
//     all their digits (no tile sorts).
//   Each pass reads 12 bytes and writes 12 bytes per pair once; passes ping-pong between the output buffers and an
//   alternate pair buffer inside the caller's scratch.
//
// Every wait on another block (the stable variant has them, the default none) is bounded: the look-back gives up
// after a fixed poll budget, raises FGS_ERR_LOOKBACK_TIMEOUT in the device status word, still publishes its own
// (then meaningless) prefix so that later partitions do not wait on it, and the block ends without scattering.
// Tickets are handed out in launch order, so a block only ever waits on partitions whose blocks are already running.

#include "fgs_common.cuh"

#include <mutex>

namespace fgs {
namespace {

#ifndef FGS_SORT_THREADS
#define FGS_SORT_THREADS 256
#endif
#ifndef FGS_SORT_ITEMS
#define FGS_SORT_ITEMS 16
#endif
#ifndef FGS_LOOKBACK_SLEEP_NS
#define FGS_LOOKBACK_SLEEP_NS 200
#endif
#ifndef FGS_LOOKBACK_WINDOW
#define FGS_LOOKBACK_WINDOW 6
#endif
constexpr int SORT_THREADS = FGS_SORT_THREADS;
constexpr int SORT_WARPS = SORT_THREADS / 32;
constexpr int SORT_ITEMS = FGS_SORT_ITEMS;               // pairs per thread
constexpr int SORT_PART = SORT_THREADS * SORT_ITEMS;    // pairs per partition
constexpr int RADIX_BITS = 8;
constexpr int RADIX = 1 << RADIX_BITS;
constexpr int MAX_PASSES = 8;
constexpr int MAX_TILE_BITS = 16;                        // tile-bucketed path: at most 2^16 tile values
constexpr int MAX_TILE_VALUES = 1 << MAX_TILE_BITS;
constexpr int LOCAL_CAP = 4096;
constexpr int LOCAL_CLASSES = 4;                        // list-length classes of the tile sort: <=1024, <=2048, <=LOCAL_CAP, longer
constexpr int HIST_THREADS = 256;
static_assert(RADIX <= SORT_THREADS, "thread d < RADIX owns digit value d in the scans and the look-back");

constexpr uint32_t FLAG_AGGREGATE = 1u << 30;           // this partition's count only
constexpr uint32_t FLAG_INCLUSIVE = 2u << 30;           // count of this and all earlier partitions
constexpr uint32_t FLAG_MASK = 3u << 30;
constexpr uint32_t VALUE_MASK = ~FLAG_MASK;
constexpr int LOOKBACK_MAX_POLLS = 1 << 20;             // x (sleep + one L2 read): gives up after about a second
constexpr int LOOKBACK_WINDOW = FGS_LOOKBACK_WINDOW;                      // earlier partitions inspected per round trip
#ifndef FGS_SORT_BLOCKS_PER_SM
#define FGS_SORT_BLOCKS_PER_SM 2
#endif
constexpr int PASS_BLOCKS_PER_SM = FGS_SORT_BLOCKS_PER_SM;   // resident digit-pass blocks per SM (shared memory: two stages each)
constexpr int STAGE_BYTES = SORT_PART * 12;             // keys + values of one partition
constexpr int LOOKBACK_SLEEP_NS = FGS_LOOKBACK_SLEEP_NS;
constexpr int SORT_SMEM_BYTES = 2 * STAGE_BYTES;        // IN stage + OUT stage
constexpr int MBAR_MAX_POLLS = 1 << 20;                 // tries of at most ~1 us each: a bulk copy gets about a second

__device__ __forceinline__ void st_relaxed(uint32_t* p, uint32_t v)
{
    asm volatile("st.relaxed.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

struct SortLayout {
    size_t tickets_off, flag_off, hist_off, tilecnt_off, status_off, seg_off, class_off, cursor_off, bucket_off, alt_keys_off, alt_vals_off, total;
    int parts;
};

inline size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

// Words of the small tables of the tile-grouping passes (behind bucket_off): the cursors of the coarse buckets,
// where each coarse bucket starts (one more entry: the pair count), and the running number of second-pass units.
constexpr int MAX_BUCKETS = 256;
constexpr size_t BUCKET_TABLE_WORDS = MAX_BUCKETS + 2 * (MAX_BUCKETS + 1) + 2;

constexpr size_t LAYOUT_HIST_OFF = 256;
constexpr size_t LAYOUT_TILECNT_OFF = LAYOUT_HIST_OFF + (size_t)MAX_PASSES * RADIX * 4;
constexpr size_t LAYOUT_STATUS_OFF = LAYOUT_TILECNT_OFF + (size_t)MAX_TILE_VALUES * 4;

// Everything in front of status_off starts at zero in every sort (one memset, or the clearing kernel when the
// pair count lives on the device): tickets, class counts and tickets, digit counts, per-tile pair counts.
constexpr size_t layout_total(size_t n)
{
    const size_t parts = (n + SORT_PART - 1) / SORT_PART;
    const size_t seg_off = (LAYOUT_STATUS_OFF + (size_t)MAX_PASSES * parts * RADIX * 4 + 255) / 256 * 256;
    const size_t class_off = (seg_off + (size_t)MAX_TILE_VALUES * 8 + 255) / 256 * 256;
    const size_t cursor_off = (class_off + (size_t)LOCAL_CLASSES * MAX_TILE_VALUES * 4 + 255) / 256 * 256;
    const size_t bucket_off = (cursor_off + (size_t)MAX_TILE_VALUES * 4 + 255) / 256 * 256;
    const size_t alt_keys_off = (bucket_off + BUCKET_TABLE_WORDS * 4 + 255) / 256 * 256;
    const size_t alt_vals_off = (alt_keys_off + n * 8 + 255) / 256 * 256;
    return (alt_vals_off + n * 4 + 255) / 256 * 256;
}

inline SortLayout make_layout(int64_t n)
{
    SortLayout L;
    if (n < 1) n = 1;
    L.parts = (int)((n + SORT_PART - 1) / SORT_PART);
    L.tickets_off = 0;                                           // MAX_PASSES tickets
    L.flag_off = 128;                                            // one spare word, then the class counts and tickets
    L.hist_off = LAYOUT_HIST_OFF;                                // MAX_PASSES x RADIX counts
    L.tilecnt_off = LAYOUT_TILECNT_OFF;                          // pairs per tile value
    L.status_off = LAYOUT_STATUS_OFF;                            // passes x parts x RADIX look-back words
    L.seg_off = align_up(L.status_off + (size_t)MAX_PASSES * L.parts * RADIX * 4, 256);   // [first, last) per tile value
    L.class_off = align_up(L.seg_off + (size_t)MAX_TILE_VALUES * 8, 256);                 // tile ids per length class
    L.cursor_off = align_up(L.class_off + (size_t)LOCAL_CLASSES * MAX_TILE_VALUES * 4, 256);   // next free place per tile
    L.bucket_off = align_up(L.cursor_off + (size_t)MAX_TILE_VALUES * 4, 256);             // tables of the coarse buckets
    L.alt_keys_off = align_up(L.bucket_off + BUCKET_TABLE_WORDS * 4, 256);
    L.alt_vals_off = align_up(L.alt_keys_off + (size_t)n * 8, 256);
    L.total = align_up(L.alt_vals_off + (size_t)n * 4, 256);
    return L;
}

// The pair count of a sort is either a host value or, for the frame entry point that never waits for the GPU,
// a device counter written by an earlier kernel on the same stream; `n` is then the capacity that bounds it.
__device__ __forceinline__ int device_count(int n, const int* n_dev)
{
    if (n_dev == nullptr) return n;
    const int v = *n_dev;
    return v < 0 ? 0 : (v < n ? v : n);
}

// Clears the ticket counters, flags, digit counts and the look-back words of the partitions a sort of the
// device-side count uses (the host-count path uses a memset of exactly that region instead).
__global__ void clear_bookkeeping_kernel(uint32_t* __restrict__ base_words, size_t head_words, uint32_t* __restrict__ status_words,
                                         int slots, int parts_stride, int n, const int* __restrict__ n_dev,
                                         size_t keep_begin, size_t keep_end)
{
    chain_release();
    chain_wait();   // nothing is read or written before the kernels ahead on the stream are complete
    n = device_count(n, n_dev);
    const int parts = (n + SORT_PART - 1) / SORT_PART;
    const size_t per_slot = (size_t)parts * RADIX;
    const size_t total = head_words + (size_t)slots * per_slot;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        if (i < head_words) { if (i < keep_begin || i >= keep_end) base_words[i] = 0; }   // [keep_begin, keep_end): counts an earlier kernel left
        else {
            const size_t j = i - head_words;
            const size_t slot = j / per_slot;
            status_words[slot * (size_t)parts_stride * RADIX + (j - slot * per_slot)] = 0;
        }
    }
}

__device__ __forceinline__ bool aligned16_dev(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// ---- digit histograms of passes [first_pass, last_pass) in one read of the keys ----
__global__ void __launch_bounds__(HIST_THREADS)
histogram_kernel(const uint64_t* __restrict__ keys, int n, const int* __restrict__ n_dev, int first_pass, int last_pass,
                 int end_bit, uint32_t* __restrict__ hist)
{
    n = device_count(n, n_dev);
    __shared__ uint32_t s_hist[MAX_PASSES * RADIX];
    const int np = last_pass - first_pass;
    for (int i = threadIdx.x; i < np * RADIX; i += HIST_THREADS) s_hist[i] = 0;
    __syncthreads();
    const uint64_t live = end_bit >= 64 ? ~0ull : ((1ull << end_bit) - 1ull);
    auto count = [&](uint64_t key) {
        const uint64_t k = (key & live) >> (first_pass * RADIX_BITS);
        for (int p = 0; p < np; p++)
            atomicAdd(&s_hist[p * RADIX + (uint32_t)((k >> (p * RADIX_BITS)) & (RADIX - 1))], 1u);
    };
    // two keys per 16-byte load, two loads in flight per thread; the ragged end (and an unaligned array) key by key
    const int64_t stride = (int64_t)gridDim.x * HIST_THREADS, me = (int64_t)blockIdx.x * HIST_THREADS + threadIdx.x;
    const int64_t pairs = aligned16_dev(keys) ? n / 2 : 0;
    const ulonglong2* keys2 = reinterpret_cast<const ulonglong2*>(keys);
    for (int64_t i = me; i < pairs; i += 2 * stride) {
        const ulonglong2 a = __ldg(keys2 + i);
        const bool second = i + stride < pairs;
        const ulonglong2 c = second ? __ldg(keys2 + i + stride) : make_ulonglong2(0, 0);
        count(a.x); count(a.y);
        if (second) { count(c.x); count(c.y); }
    }
    for (int64_t i = 2 * pairs + me; i < n; i += stride) count(__ldg(keys + i));
    __syncthreads();
    for (int i = threadIdx.x; i < np * RADIX; i += HIST_THREADS) {
        const uint32_t c = s_hist[i];
        if (c) atomicAdd(hist + first_pass * RADIX + i, c);
    }
}

// ---- asynchronous bulk copies (TMA, 1-D, into this block only) and their mbarrier ----
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_load(void* dst_smem, const void* src_gmem, uint32_t bytes, uint64_t* bar)
{
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_u32(dst_smem)), "l"(src_gmem), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
// Bounded wait for a phase of the barrier; false if the poll budget ran out.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity)
{
    const uint32_t addr = smem_u32(bar);
    for (int i = 0; i < MBAR_MAX_POLLS; i++) {
        uint32_t ok;
        // the last operand caps how long one try may suspend the thread (nanoseconds)
        asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, 1000;\n selp.u32 %0, 1, 0, p;\n}"
                     : "=r"(ok) : "r"(addr), "r"(parity) : "memory");
        if (ok) return true;
    }
    return false;
}

// Optional per-phase cycle accounting of the pass kernel (compile with -DFGS_SORT_TIMING): thread 0 of
// every block adds the SM cycles it spent in each phase to g_phase_cycles; read with fgs_debug_sort_phase_cycles.
#ifdef FGS_SORT_TIMING
__device__ unsigned long long g_phase_cycles[8];
#define FGS_T(i) do { if (tid == 0) { const long long now_ = clock64(); atomicAdd(&g_phase_cycles[i], (unsigned long long)(now_ - t_prev_)); t_prev_ = now_; } } while (0)
#else
#define FGS_T(i) do { } while (0)
#endif


// ---- named barriers between the warp roles of the pass kernel ----
__device__ __forceinline__ void bar_sync(int id, int count) { asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(count) : "memory"); }
__device__ __forceinline__ void bar_arrive(int id, int count) { asm volatile("bar.arrive %0, %1;" ::"r"(id), "r"(count) : "memory"); }

__device__ __forceinline__ uint4 ld_relaxed_v4(const uint32_t* p)
{
    uint4 v;
    asm volatile("ld.relaxed.gpu.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_relaxed_v4(uint32_t* p, uint4 v)
{
    asm volatile("st.relaxed.gpu.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

// ---- one onesweep pass ----
// Persistent blocks (two per SM) of SORT_THREADS "sorting" threads plus LB_THREADS "look-back" threads.
//
// Sorting warps, per partition of SORT_PART pairs: wait for the bulk copy (TMA) that brought the partition
// into the IN stage and pull it into registers; count the digits (shared-memory adds), publish the counts and
// hand them to the look-back warps; rank by digit (the IN stage serves as scratch for the bit masks); start
// the copy of the next partition into the IN stage; write out the PREVIOUS partition, whose global digit
// offsets the look-back warps have produced meanwhile; reorder the current partition into the OUT stage.
// Look-back warps, per partition: walk back over earlier partitions' status words until an inclusive prefix
// is found, publish this partition's inclusive prefix, hand the offsets back.
// The look-back of partition i therefore runs while the sorting warps write out partition i-1 and rank
// partition i+1: persistent blocks advance in lock-step, which makes the walk long (it crosses the partitions
// of all blocks that started together), and this keeps that wait off the sorting warps' path.
constexpr int LB_THREADS = 64;                              // each owns 4 digit values (16-byte status accesses)
constexpr int PASS_THREADS = SORT_THREADS + LB_THREADS;
constexpr int BAR_SORTERS = 1;                              // barrier ids; 0 is __syncthreads
constexpr int BAR_COUNTS = 2;                               // +parity: counts of a partition are in shared memory
constexpr int BAR_OFFSETS = 4;                              // +parity: global offsets of a partition are in shared memory
constexpr uint32_t NO_TICKET = 0xFFFFFFFFu;
static_assert(LB_THREADS * 4 == RADIX, "a look-back thread owns four digit values");
static_assert(SORT_THREADS == RADIX, "sorting thread d owns digit value d");

// Digit of a key: SHIFT is a multiple of 8 known at compile time, so the digit is a byte of the low or of
// the high word and costs one shift-and-mask.
template <int SHIFT>
__device__ __forceinline__ uint32_t digit_of(uint64_t key, uint32_t digit_mask)
{
    const uint32_t word = SHIFT < 32 ? (uint32_t)key : (uint32_t)(key >> 32);
    return (word >> (SHIFT & 31)) & digit_mask;
}

template <int SHIFT>
__global__ void __launch_bounds__(PASS_THREADS, PASS_BLOCKS_PER_SM)
onesweep_kernel(const uint64_t* __restrict__ keys_in, const uint32_t* __restrict__ vals_in,
                uint64_t* __restrict__ keys_out, uint32_t* __restrict__ vals_out,
                int n, int num_parts, uint32_t digit_mask, int use_bulk,
                uint32_t* __restrict__ ticket, const uint32_t* __restrict__ hist,
                uint32_t* __restrict__ status_words, int* __restrict__ dev_status, int skip_publish_part,
                const int* __restrict__ n_dev)
{
    if (n_dev != nullptr) {
        n = device_count(n, n_dev);
        num_parts = (n + SORT_PART - 1) / SORT_PART;
    }
    extern __shared__ __align__(128) unsigned char s_dyn[];   // IN stage | OUT stage, each keys 8*PART | values 4*PART
    __shared__ __align__(8) uint64_t s_bar;                   // completion of the bulk copy into IN
    __shared__ uint32_t s_whist[SORT_WARPS][RADIX];           // per-warp digit counts, then exclusive warp offsets
    __shared__ __align__(16) uint32_t s_count[2][RADIX];      // block digit counts of a partition (by parity)
    __shared__ __align__(16) uint32_t s_gstart[2][RADIX];     // global index where the partition's run of a digit starts
    __shared__ uint32_t s_local_start[2][RADIX];              // where that run starts inside the reordered partition
    __shared__ uint32_t s_delta[RADIX];                       // s_gstart - s_local_start of the partition being written out
    __shared__ __align__(16) uint32_t s_digit_base[RADIX];    // exclusive scan of the global histogram
    __shared__ uint32_t s_scan[RADIX / 32];
    __shared__ uint32_t s_tickets[4];                         // partition of iteration i lives in s_tickets[i & 3]
    __shared__ int s_copy_issued[2];                          // by iteration parity: IN is being filled by a bulk copy
    __shared__ volatile int s_abort;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    uint64_t* in_keys = reinterpret_cast<uint64_t*>(s_dyn);
    uint32_t* in_vals = reinterpret_cast<uint32_t*>(s_dyn + SORT_PART * 8);
    uint64_t* out_keys = reinterpret_cast<uint64_t*>(s_dyn + STAGE_BYTES);
    uint32_t* out_vals = reinterpret_cast<uint32_t*>(s_dyn + STAGE_BYTES + SORT_PART * 8);
    auto full_part = [&](uint32_t part) { return part < (uint32_t)num_parts && (int64_t)(part + 1) * SORT_PART <= (int64_t)n; };

    if (tid == 0) {
        mbar_init(&s_bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        s_abort = 0;
        s_tickets[0] = atomicAdd(ticket, 1u);
        s_tickets[1] = atomicAdd(ticket, 1u);
    }
    // exclusive scan of the global histogram: where each digit's output region starts
    if (tid < RADIX) {
        const uint32_t g = hist[tid];
        uint32_t inc = g;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const uint32_t a = __shfl_up_sync(FULL_MASK, inc, o);
            if (lane >= o) inc += a;
        }
        if (lane == 31) s_scan[warp] = inc;
        __syncwarp();
        s_digit_base[tid] = inc - g;    // completed below
    }
    __syncthreads();
    if (tid < RADIX) {
        uint32_t off = 0;
#pragma unroll
        for (int w = 0; w < RADIX / 32; w++) off += (w < warp) ? s_scan[w] : 0;
        s_digit_base[tid] += off;
    }
    __syncthreads();

    if (tid >= SORT_THREADS) {
        // ======================= look-back warps =======================
        const int t4 = (tid - SORT_THREADS) * 4;   // first of this thread's four digit values
        for (int it = 0;; it++) {
            const uint32_t part = s_tickets[it & 3];
            if (part >= (uint32_t)num_parts) break;
            const int b = it & 1;
            bar_sync(BAR_COUNTS + b, PASS_THREADS);                  // counts of this partition are ready
            const uint4 cnt = *reinterpret_cast<const uint4*>(&s_count[b][t4]);
            uint32_t* my_status = status_words + (size_t)part * RADIX + t4;
            const bool publish = (int)part != skip_publish_part;

            uint32_t earlier[4] = { 0, 0, 0, 0 };
            bool done[4] = { part == 0, part == 0, part == 0, part == 0 };
            bool failed = false;
            int64_t p0 = (int64_t)part - 1;     // nearest partition not yet accounted for
            int polls = 0;
            while (!(done[0] && done[1] && done[2] && done[3]) && !s_abort) {
                uint4 sw[LOOKBACK_WINDOW];
#pragma unroll
                for (int k = 0; k < LOOKBACK_WINDOW; k++)
                    sw[k] = (p0 - k >= 0) ? ld_relaxed_v4(status_words + (size_t)(p0 - k) * RADIX + t4)
                                          : make_uint4(FLAG_INCLUSIVE, FLAG_INCLUSIVE, FLAG_INCLUSIVE, FLAG_INCLUSIVE);
                int used = 0;   // window entries consumed, nearest partition first, while all four words are published
#pragma unroll
                for (int k = 0; k < LOOKBACK_WINDOW; k++) {
                    const uint32_t w4[4] = { sw[k].x, sw[k].y, sw[k].z, sw[k].w };
                    bool ready = used == k;
#pragma unroll
                    for (int q = 0; q < 4; q++) ready = ready && (done[q] || (w4[q] & FLAG_MASK) != 0);
                    if (ready) {
#pragma unroll
                        for (int q = 0; q < 4; q++)
                            if (!done[q]) { earlier[q] += w4[q] & VALUE_MASK; done[q] = (w4[q] & FLAG_MASK) == FLAG_INCLUSIVE; }
                        used = k + 1;
                    }
                }
                p0 -= used;
#ifdef FGS_SORT_TIMING
                if (t4 == 0) { atomicAdd(&g_phase_cycles[6], 1ull); if (used == 0) atomicAdd(&g_phase_cycles[7], 1ull); }
#endif
                if (used == 0) {    // the nearest partition has not published yet: back off before asking again
                    if (++polls > LOOKBACK_MAX_POLLS) { failed = true; break; }
                    __nanosleep(LOOKBACK_SLEEP_NS);
                }
            }
            if (failed) { atomicOr(dev_status, FGS_ERR_LOOKBACK_TIMEOUT); s_abort = 1; }
            if (publish && part > 0)
                st_relaxed_v4(my_status, make_uint4(FLAG_INCLUSIVE | ((earlier[0] + cnt.x) & VALUE_MASK), FLAG_INCLUSIVE | ((earlier[1] + cnt.y) & VALUE_MASK),
                                                    FLAG_INCLUSIVE | ((earlier[2] + cnt.z) & VALUE_MASK), FLAG_INCLUSIVE | ((earlier[3] + cnt.w) & VALUE_MASK)));
            const uint4 base = *reinterpret_cast<const uint4*>(&s_digit_base[t4]);
            *reinterpret_cast<uint4*>(&s_gstart[b][t4]) = make_uint4(base.x + earlier[0], base.y + earlier[1], base.z + earlier[2], base.w + earlier[3]);
            bar_arrive(BAR_OFFSETS + b, PASS_THREADS);               // offsets of this partition are ready
        }
        return;
    }

    // ======================= sorting warps =======================
    const unsigned lt = lanemask_lt();
    uint32_t in_parity = 0;
    bool copy_pending = false;      // thread 0: a bulk copy into IN has been started and not yet waited for
    // Thread 0 only: start the bulk copy of the partition of iteration `iter` into IN, if it is a whole,
    // 16-byte aligned partition; otherwise (ragged tail, unaligned input, after a failed wait) the sorting
    // threads fetch it with plain loads when its turn comes.
    auto prefetch = [&](int iter, uint32_t part) {
        const bool issue = use_bulk && full_part(part) && !s_abort;
        if (issue) {
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            mbar_expect_tx(&s_bar, SORT_PART * 12);
            bulk_load(in_keys, keys_in + (size_t)part * SORT_PART, SORT_PART * 8, &s_bar);
            bulk_load(in_vals, vals_in + (size_t)part * SORT_PART, SORT_PART * 4, &s_bar);
            copy_pending = true;
        }
        s_copy_issued[iter & 1] = issue ? 1 : 0;
    };
    // write the reordered partition held in OUT to its digits' global runs
    auto write_out = [&](int valid, const uint32_t* gstart, const uint32_t* lstart) {
        s_delta[tid] = gstart[tid] - lstart[tid];   // destination index minus index inside OUT, per digit (mod 2^32)
        bar_sync(BAR_SORTERS, SORT_THREADS);
#pragma unroll
        for (int i = 0; i < SORT_ITEMS; i++) {
            const int j = i * SORT_THREADS + tid;
            if (j < valid) {
                const uint64_t k = out_keys[j];
                const uint32_t dst = s_delta[digit_of<SHIFT>(k, digit_mask)] + (uint32_t)j;
                if (FGS_INDEX_OK(dst, n)) {
                    keys_out[dst] = k;
                    vals_out[dst] = out_vals[j];
                }
            }
        }
    };
    if (tid == 0) prefetch(0, s_tickets[0]);
    bar_sync(BAR_SORTERS, SORT_THREADS);
#ifdef FGS_SORT_TIMING
    long long t_prev_ = clock64();
#endif

    int it = 0, prev_valid = 0;
    for (;; it++) {
        const uint32_t part = s_tickets[it & 3];
        if (part >= (uint32_t)num_parts) break;
        const int b = it & 1;
        const int64_t part_base = (int64_t)part * SORT_PART;
        const int valid = (int)min((int64_t)SORT_PART, (int64_t)n - part_base);
        const bool bulk = s_copy_issued[b] != 0;
        // Thread 0 requests the ticket after next now and stores it at the end of the iteration, so the
        // round trip of the atomic never stalls the block.
        uint32_t ticket_after_next = 0;
        if (tid == 0) ticket_after_next = atomicAdd(ticket, 1u);
        for (int i = tid; i < SORT_WARPS * RADIX; i += SORT_THREADS) (&s_whist[0][0])[i] = 0;
        s_count[b][tid] = 0;

        uint64_t key[SORT_ITEMS];
        uint32_t val[SORT_ITEMS];
        const int wbase = warp * (32 * SORT_ITEMS);   // warp-striped: item i of lane l sits at wbase + i*32 + l
        if (bulk) {
            if (!mbar_wait(&s_bar, in_parity)) { atomicOr(dev_status, FGS_ERR_LOOKBACK_TIMEOUT); s_abort = 1; }
            else copy_pending = false;
            in_parity ^= 1u;
#pragma unroll
            for (int i = 0; i < SORT_ITEMS; i++) { key[i] = in_keys[wbase + i * 32 + lane]; val[i] = in_vals[wbase + i * 32 + lane]; }
        } else {
#pragma unroll
            for (int i = 0; i < SORT_ITEMS; i++) {
                const int local = wbase + i * 32 + lane;
                key[i] = local < valid ? __ldg(keys_in + part_base + local) : ~0ull;
                val[i] = local < valid ? __ldg(vals_in + part_base + local) : 0u;
            }
        }
        bar_sync(BAR_SORTERS, SORT_THREADS);   // s_whist zeroed; every thread holds its items, IN is free again
        // The block's digit counts first, by shared-memory adds, so that they can be published and the look-back of
        // this partition can start before the ranking instead of after it: the look-back's latency is what the
        // pass waits for.
#pragma unroll
        for (int i = 0; i < SORT_ITEMS; i++) atomicAdd(&s_count[b][digit_of<SHIFT>(key[i], digit_mask)], 1u);
        bar_sync(BAR_SORTERS, SORT_THREADS);
        // published by the sorting thread itself, at once: later partitions wait for exactly this word, and the
        // look-back warps may still be busy with the previous partition
        if ((int)part != skip_publish_part)
            st_relaxed(status_words + (size_t)part * RADIX + tid, (part == 0 ? FLAG_INCLUSIVE : FLAG_AGGREGATE) | s_count[b][tid]);
        bar_arrive(BAR_COUNTS + b, PASS_THREADS);   // the look-back warps take it from here
        FGS_T(0);

        // Rank within the warp, item by item, so equal digits keep their input order. The lanes holding the same
        // digit find one another through shared memory: every lane ORs its bit into the warp's word of its digit
        // and reads the word back (two instructions instead of eight votes and their logic). The words live in
        // the IN stage, which is free until the next partition's copy is started after this phase; two sets are
        // used in turn, and the lowest lane of a group clears its word after use, so that a set is clean again
        // when its turn comes. That lane also adds the group's size to the warp's counter of the digit and hands
        // the old value to the group.
        uint32_t* my_masks = reinterpret_cast<uint32_t*>(s_dyn) + warp * (2 * RADIX);
#pragma unroll
        for (int i = 0; i < 2 * RADIX / 32; i++) my_masks[i * 32 + lane] = 0;
        __syncwarp();
        uint32_t rank[SORT_ITEMS];
#pragma unroll
        for (int i = 0; i < SORT_ITEMS; i++) {
            const uint32_t d = digit_of<SHIFT>(key[i], digit_mask);
            volatile uint32_t* word = my_masks + (i & 1) * RADIX + d;
            atomicOr(const_cast<uint32_t*>(word), 1u << lane);
            __syncwarp();
            const unsigned peers = *word;
            __syncwarp();
            uint32_t pre = 0;
            if ((peers & lt) == 0) {
                *word = 0;
                pre = atomicAdd(&s_whist[warp][d], (uint32_t)__popc(peers));
            }
            pre = __shfl_sync(FULL_MASK, pre, __ffs(peers) - 1);
            rank[i] = pre + __popc(peers & lt);
        }
        bar_sync(BAR_SORTERS, SORT_THREADS);
        if (tid == 0) prefetch(it + 1, s_tickets[(it + 1) & 3]);   // IN is no longer used by the ranking
        FGS_T(1);

        // thread d owns digit value d: block count, exclusive warp offsets, start of the run inside the partition
        uint32_t count = 0;
#pragma unroll
        for (int w = 0; w < SORT_WARPS; w++) {
            const uint32_t c = s_whist[w][tid];
            s_whist[w][tid] = count;
            count += c;
        }
        uint32_t inc_l = count;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const uint32_t a = __shfl_up_sync(FULL_MASK, inc_l, o);
            if (lane >= o) inc_l += a;
        }
        if (lane == 31) s_scan[warp] = inc_l;
        bar_sync(BAR_SORTERS, SORT_THREADS);
        {
            uint32_t off_l = 0;
#pragma unroll
            for (int w = 0; w < RADIX / 32; w++) off_l += (w < warp) ? s_scan[w] : 0;
            s_local_start[b][tid] = off_l + inc_l - count;
        }
        FGS_T(2);

        // the previous partition: its offsets have been looked up while this one was loaded and ranked
        if (it > 0) {
            bar_sync(BAR_OFFSETS + (b ^ 1), PASS_THREADS);
            FGS_T(4);
            write_out(s_abort ? 0 : prev_valid, s_gstart[b ^ 1], s_local_start[b ^ 1]);
            FGS_T(5);
        }
        bar_sync(BAR_SORTERS, SORT_THREADS);   // OUT is free, s_local_start[b] is complete

        // reorder this partition into OUT
#pragma unroll
        for (int i = 0; i < SORT_ITEMS; i++) {
            const uint32_t d = digit_of<SHIFT>(key[i], digit_mask);
            const uint32_t pos = s_local_start[b][d] + s_whist[warp][d] + rank[i];
            if (FGS_INDEX_OK(pos, SORT_PART)) {
                out_keys[pos] = key[i];
                out_vals[pos] = val[i];
            }
        }
        prev_valid = valid;
        // after a failed wait no further partitions are started: both loops end within two iterations
        if (tid == 0) s_tickets[(it + 2) & 3] = s_abort ? NO_TICKET : ticket_after_next;
        bar_sync(BAR_SORTERS, SORT_THREADS);   // OUT complete, ticket visible
        FGS_T(3);
    }
    if (it > 0) {   // the last partition
        const int b = (it - 1) & 1;
        bar_sync(BAR_OFFSETS + b, PASS_THREADS);
        write_out(s_abort ? 0 : prev_valid, s_gstart[b], s_local_start[b]);
    }
    // Leaving after a failed wait: a copy into IN may still be in flight; wait for it (bounded) so that
    // nothing writes into shared memory after the block is gone.
    if (tid == 0 && copy_pending) mbar_wait(&s_bar, in_parity);
}

// ---- tile-bucketed path: after the digit passes over the tile bits, every tile's pairs are contiguous ----
// One thread per tile value: [first, one-past-last) of that tile in the tile-grouped list, by binary search;
// non-empty tiles are appended to the work list of their length class.
constexpr int SEG_TILES = 256, SEG_THREADS = SEG_TILES + 32;
__global__ void segments_kernel(const uint64_t* __restrict__ keys, int n, const int* __restrict__ n_dev, int tile_values,
                                uint32_t tile_mask, int2* __restrict__ seg,
                                int* __restrict__ class_count, uint32_t* __restrict__ class_tiles)
{
    n = device_count(n, n_dev);
    // One search per thread: a tile ends where the next one starts. Threads 0..SEG_TILES-1 of a block search the
    // starts of the block's tiles, thread SEG_TILES the start of the tile behind them.
    const int t = blockIdx.x * SEG_TILES + threadIdx.x;
    auto lower = [&](uint32_t v) {
        int lo = 0, hi = n;
        while (lo < hi) {
            const int mid = (int)(((unsigned)lo + (unsigned)hi) >> 1);
            if (((uint32_t)(__ldg(keys + mid) >> 32) & tile_mask) < v) lo = mid + 1; else hi = mid;
        }
        return lo;
    };
    __shared__ int s_first[SEG_TILES + 1];
    __shared__ int s_class_count[LOCAL_CLASSES], s_class_base[LOCAL_CLASSES];
    if (threadIdx.x < LOCAL_CLASSES) s_class_count[threadIdx.x] = 0;
    if (threadIdx.x <= SEG_TILES) s_first[threadIdx.x] = t < tile_values ? lower((uint32_t)t) : n;
    __syncthreads();
    int c = -1, slot = 0;
    if (threadIdx.x < SEG_TILES && t < tile_values) {
        const int first = s_first[threadIdx.x], last = s_first[threadIdx.x + 1];
        if (FGS_INDEX_OK(t, MAX_TILE_VALUES)) seg[t] = make_int2(first, last);
        const int len = last - first;
        if (len > 0) {   // queue the tile for the sort of its length class
            c = len <= 1024 ? 0 : (len <= 2048 ? 1 : (len <= LOCAL_CAP ? 2 : 3));
            slot = atomicAdd(&s_class_count[c], 1);
        }
    }
    // the block reserves its places in the classes' work lists with one atomic per class (tens of thousands of
    // threads adding to the same four counters take longer than the searches)
    __syncthreads();
    if (threadIdx.x < LOCAL_CLASSES && s_class_count[threadIdx.x] > 0)
        s_class_base[threadIdx.x] = atomicAdd(class_count + threadIdx.x, s_class_count[threadIdx.x]);
    __syncthreads();
    if (c >= 0 && FGS_INDEX_OK(s_class_base[c] + slot, MAX_TILE_VALUES)) class_tiles[(size_t)c * MAX_TILE_VALUES + s_class_base[c] + slot] = (uint32_t)t;
}

// ---- tile grouping without any wait between blocks ----
// The in-block tile sorts need every tile's pairs contiguous, in ANY order (they order a tile's pairs themselves).
// That weaker requirement is met without look-back: count the pairs of every tile value (tile_hist_kernel), turn
// the counts into each tile's [first, last) and a cursor per tile (tile_scan_kernel), then move the pairs in two
// passes (multisplit_kernel). The first pass splits by the upper half of the tile bits into coarse buckets, the
// second splits every coarse bucket by the lower half into its tiles. A block takes one partition, counts its
// digits in shared memory, reserves room for each digit's run with ONE atomicAdd on that destination's cursor,
// reorders the partition in shared memory and writes the runs as contiguous stores. Blocks never wait for one
// another, so there is no look-back chain, no ordering between blocks and nothing that can time out; the price is
// that the order inside a tile is the order in which blocks happened to reserve their runs, which is why the
// tile sorts of this path order by (depth bits, value) and not by (depth bits, position).
#ifndef FGS_MS_BLOCKS_PER_SM
#define FGS_MS_BLOCKS_PER_SM 3
#endif
#ifndef FGS_MS_ITEMS
#define FGS_MS_ITEMS 16
#endif
#ifndef FGS_MS_LATE_VALUES
#define FGS_MS_LATE_VALUES 1   // 1: read a partition's values after the ranking instead of with its keys
#endif

#ifndef FGS_MS_THREADS
#define FGS_MS_THREADS 256
#endif
constexpr int MS_THREADS = FGS_MS_THREADS;            // thread d < MS_DIGITS owns digit value d (at most 8 bits per pass)
constexpr int MS_DIGITS = MAX_BUCKETS;
constexpr int MS_ITEMS = FGS_MS_ITEMS;
constexpr int MS_PART = MS_THREADS * MS_ITEMS;        // pairs per partition
constexpr int MS_SMEM_BYTES = MS_PART * 12;           // the partition reordered by digit: keys, then values
constexpr int MS_BLOCKS_PER_SM = FGS_MS_BLOCKS_PER_SM;
constexpr int TILE_HIST_THREADS = 1024;
constexpr int TILE_HIST_SMEM_VALUES = 49152;          // tile values whose counters fit one block's shared memory
constexpr int TILE_SCAN_THREADS = 1024;
static_assert(MS_THREADS >= MS_DIGITS && MS_THREADS % 32 == 0, "a pass has at most as many digit values as the block has threads");

// Pairs per tile value, added to tile_count[] (zero on entry). With `in_smem` a block counts into shared memory
// (tile_values * 4 bytes of dynamic shared memory) and adds its non-zero counters to the global ones at the end;
// otherwise every key adds to the global counter directly (more tile values than fit, or very few keys).
__global__ void __launch_bounds__(TILE_HIST_THREADS, 1)
tile_hist_kernel(const uint64_t* __restrict__ keys, int n, const int* __restrict__ n_dev, uint32_t tile_mask, int tile_values,
                 int in_smem, uint32_t* __restrict__ tile_count)
{
    chain_release();
    chain_wait();   // nothing is read or written before the kernels ahead on the stream are complete
    extern __shared__ __align__(16) uint32_t s_tiles[];
    n = device_count(n, n_dev);
    if (in_smem) {
        for (int i = threadIdx.x; i < tile_values; i += TILE_HIST_THREADS) s_tiles[i] = 0;
        __syncthreads();
    }
    auto count = [&](uint64_t key) {
        const uint32_t t = (uint32_t)(key >> 32) & tile_mask;
        if (!FGS_INDEX_OK(t, tile_values)) return;
        if (in_smem) atomicAdd(&s_tiles[t], 1u); else atomicAdd(tile_count + t, 1u);
    };
    const int64_t stride = (int64_t)gridDim.x * TILE_HIST_THREADS, me = (int64_t)blockIdx.x * TILE_HIST_THREADS + threadIdx.x;
    const int64_t pairs = aligned16_dev(keys) ? n / 2 : 0;
    const ulonglong2* keys2 = reinterpret_cast<const ulonglong2*>(keys);
    for (int64_t i = me; i < pairs; i += 2 * stride) {
        const ulonglong2 a = __ldg(keys2 + i);
        const bool second = i + stride < pairs;
        const ulonglong2 c = second ? __ldg(keys2 + i + stride) : make_ulonglong2(0, 0);
        count(a.x); count(a.y);
        if (second) { count(c.x); count(c.y); }
    }
    for (int64_t i = 2 * pairs + me; i < n; i += stride) count(__ldg(keys + i));
    if (in_smem) {
        __syncthreads();
        for (int i = threadIdx.x; i < tile_values; i += TILE_HIST_THREADS) {
            const uint32_t c = s_tiles[i];
            if (c) atomicAdd(tile_count + i, c);
        }
    }
}

// From the pairs per tile value: every tile's [first, last) in the tile-grouped list and its cursor (= first), the
// work lists of the tile sorts' length classes, and the tables of the coarse buckets (a bucket is the run of
// 2^lo_bits consecutive tile values that share their upper bits): where each bucket starts, its cursor, and the
// running count of the second pass's units (partitions cut inside a bucket).
// A block owns SCAN_CHUNK consecutive tile values. It finds the pairs in front of its chunk by summing the counts
// of all earlier tiles itself (at most 64 K coalesced loads spread over its threads: cheaper than any hand-over
// between blocks, and nobody waits for anybody), scans its own counts, and writes its tiles' outputs. The block
// that finishes last (a ticket drawn after a fence; no block waits for it) builds the unit table from the
// buckets' starts and checks the total against the pair count.
constexpr int SCAN_CHUNK = TILE_SCAN_THREADS;   // one tile value per thread

__global__ void __launch_bounds__(TILE_SCAN_THREADS, 1)
tile_scan_kernel(const uint32_t* __restrict__ tile_count, int tile_values, int lo_bits,
                 int2* __restrict__ seg, uint32_t* __restrict__ cursor, uint32_t* bucket_tables,
                 int* class_count, uint32_t* __restrict__ class_tiles,
                 int n_pairs, const int* __restrict__ n_dev, int* __restrict__ dev_status, uint32_t* done_ticket)
{
    chain_release();
    chain_wait();   // nothing is read or written before the kernels ahead on the stream are complete
    constexpr int WARPS = TILE_SCAN_THREADS / 32;
    __shared__ uint32_t s_wsum[2][WARPS];
    __shared__ uint32_t s_units[MAX_BUCKETS];
    __shared__ uint32_t s_usum[MAX_BUCKETS / 32];
    __shared__ int s_last;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const unsigned lt = lanemask_lt();
    const uint32_t lo_mask = (1u << lo_bits) - 1u;
    const int buckets = max(1, tile_values >> lo_bits);
    uint32_t* hi_cursor = bucket_tables;                      // [0, B) cursors of the coarse buckets
    uint32_t* bucket_first = bucket_tables + MAX_BUCKETS;     // [B + 1] where each bucket starts, then the total
    uint32_t* unit_prefix = bucket_first + MAX_BUCKETS + 1;   // [B + 1] exclusive unit counts, then their total

    const int chunk0 = blockIdx.x * SCAN_CHUNK;
    const int t = chunk0 + tid;
    // pairs of all earlier tiles: eight independent loads in flight per thread
    uint32_t before = 0;
    for (int b = 0; b < chunk0; b += 8 * TILE_SCAN_THREADS) {
        uint32_t v[8];
#pragma unroll
        for (int u = 0; u < 8; u++) {
            const int i = b + u * TILE_SCAN_THREADS + tid;
            v[u] = i < chunk0 ? tile_count[i] : 0u;
        }
#pragma unroll
        for (int u = 0; u < 8; u++) before += v[u];
    }
    const uint32_t c = t < tile_values ? tile_count[t] : 0u;
    uint32_t inc = c, red = before;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const uint32_t a = __shfl_up_sync(FULL_MASK, inc, o);
        if (lane >= o) inc += a;
        red += __shfl_xor_sync(FULL_MASK, red, o);
    }
    if (lane == 31) s_wsum[0][warp] = inc;
    if (lane == 0) s_wsum[1][warp] = red;
    __syncthreads();
    uint32_t first = inc - c, base = 0, chunk_total = 0;
    for (int w = 0; w < WARPS; w++) {
        const uint32_t s = s_wsum[0][w];
        if (w < warp) first += s;
        chunk_total += s;
        base += s_wsum[1][w];
    }
    first += base;
    if (t < tile_values && FGS_INDEX_OK(t, MAX_TILE_VALUES)) {
        seg[t] = make_int2((int)first, (int)(first + c));
        cursor[t] = first;
        if (((uint32_t)t & lo_mask) == 0 && FGS_INDEX_OK(t >> lo_bits, MAX_BUCKETS)) {
            bucket_first[t >> lo_bits] = first;
            hi_cursor[t >> lo_bits] = first;
        }
    }
    const int k = c == 0 ? -1 : (c <= 1024u ? 0 : (c <= 2048u ? 1 : (c <= (uint32_t)LOCAL_CAP ? 2 : 3)));
#pragma unroll
    for (int q = 0; q < LOCAL_CLASSES; q++) {   // the warp reserves its places in class q's work list with one add
        const unsigned in_class = __ballot_sync(FULL_MASK, k == q);
        if (in_class) {
            uint32_t at = 0;
            if (lane == 0) at = (uint32_t)atomicAdd(class_count + q, __popc(in_class));
            at = __shfl_sync(FULL_MASK, at, 0);
            if (k == q && FGS_INDEX_OK(at + __popc(in_class & lt), MAX_TILE_VALUES))
                class_tiles[(size_t)q * MAX_TILE_VALUES + at + __popc(in_class & lt)] = (uint32_t)t;
        }
    }
    // the block that finishes last completes the tables
    __threadfence();
    __syncthreads();
    if (tid == 0) s_last = atomicAdd(done_ticket, 1u) == gridDim.x - 1 ? 1 : 0;
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    const uint32_t total = (uint32_t)((volatile int2*)seg)[tile_values - 1].y;
    // The counts must add up to the number of pairs (they do when this sort counted them itself; a table handed in by
    // the caller is checked here): otherwise nothing is moved -- no work for the passes, no lists for the tile sorts.
    const bool consistent = total == (uint32_t)device_count(n_pairs, n_dev);
    if (!consistent && tid == 0) atomicOr(dev_status, FGS_ERR_BAD_ARG);
    if (!consistent && tid < LOCAL_CLASSES) class_count[tid] = 0;
    if (tid < MAX_BUCKETS) {
        uint32_t units = 0;
        if (tid < buckets) {
            const uint32_t bf = ((volatile uint32_t*)bucket_first)[tid];
            const uint32_t next = tid + 1 < buckets ? ((volatile uint32_t*)bucket_first)[tid + 1] : total;
            units = consistent ? (next - bf + MS_PART - 1) / MS_PART : 0u;
            if (!consistent) hi_cursor[tid] = 0x80000000u;   // every destination of the first pass falls outside the list
        }
        uint32_t uinc = units;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const uint32_t a = __shfl_up_sync(FULL_MASK, uinc, o);
            if (lane >= o) uinc += a;
        }
        if (lane == 31) s_usum[warp] = uinc;
        s_units[tid] = uinc - units;   // exclusive inside the warp
    }
    if (tid == 0) bucket_first[buckets] = total;
    __syncthreads();
    if (tid < MAX_BUCKETS) {
        uint32_t off = 0;
        for (int w = 0; w < warp; w++) off += s_usum[w];
        if (tid < buckets) unit_prefix[tid] = off + s_units[tid];
        if (tid == MAX_BUCKETS - 1) {
            uint32_t all = 0;
            for (int w = 0; w < MAX_BUCKETS / 32; w++) all += s_usum[w];
            unit_prefix[buckets] = all;
        }
    }
}

// One pass of the tile grouping. SECOND == false: unit = partition `blockIdx.x` of the whole list, digit = upper
// tile bits, destination cursors = the coarse buckets'. SECOND == true: unit = one partition cut inside one coarse
// bucket (found from the running unit counts), digit = lower tile bits, destination cursors = the tiles' of that
// bucket. Every destination index comes from cursors that were derived from counts of these very keys, so it lies
// inside the list; `n` (or the device count) bounds the reads.
template <bool SECOND>
__global__ void __launch_bounds__(MS_THREADS, MS_BLOCKS_PER_SM)
multisplit_kernel(const uint64_t* __restrict__ keys_in, const uint32_t* __restrict__ vals_in,
                  uint64_t* __restrict__ keys_out, uint32_t* __restrict__ vals_out,
                  int n, const int* __restrict__ n_dev, uint32_t tile_mask, int lo_bits, int buckets,
                  const uint32_t* bucket_tables, uint32_t* cursors)
{
    chain_release();
    chain_wait();   // nothing is read or written before the kernels ahead on the stream are complete
    extern __shared__ __align__(16) unsigned char s_ms[];      // reordered partition: keys [MS_PART], values [MS_PART]
    __shared__ uint32_t s_cnt[MS_DIGITS];                       // pairs per digit value in this partition
    __shared__ uint32_t s_lstart[MS_DIGITS];                    // where a digit's run starts in the reordered partition
    __shared__ uint32_t s_delta[MS_DIGITS];                     // destination index minus index in the reordered partition
    __shared__ uint32_t s_wsum[MS_DIGITS / 32];
    __shared__ uint32_t s_units[SECOND ? MAX_BUCKETS + 1 : 1];
    uint64_t* st_keys = reinterpret_cast<uint64_t*>(s_ms);
    uint32_t* st_vals = reinterpret_cast<uint32_t*>(s_ms + MS_PART * 8);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    n = device_count(n, n_dev);

    int64_t base;
    int count;
    uint32_t cursor_base = 0;
    if (!SECOND) {
        base = (int64_t)blockIdx.x * MS_PART;
        if (base >= n) return;
        count = (int)min((int64_t)MS_PART, (int64_t)n - base);
    } else {
        const uint32_t* bucket_first = bucket_tables + MAX_BUCKETS;
        const uint32_t* unit_prefix = bucket_first + MAX_BUCKETS + 1;
        for (int i = tid; i <= buckets; i += MS_THREADS) s_units[i] = unit_prefix[i];
        __syncthreads();
        const uint32_t u = blockIdx.x;
        if (u >= s_units[buckets]) return;
        int lo = 0, hi = buckets;   // largest h with s_units[h] <= u
        while (hi - lo > 1) {
            const int mid = (lo + hi) >> 1;
            if (s_units[mid] <= u) lo = mid; else hi = mid;
        }
        const uint32_t first = bucket_first[lo], last = bucket_first[lo + 1];
        base = (int64_t)first + (int64_t)(u - s_units[lo]) * MS_PART;
        count = (int)min((int64_t)MS_PART, (int64_t)last - base);
        if (count <= 0 || base + count > (int64_t)n) return;   // inconsistent tables: touch nothing
        cursor_base = (uint32_t)lo << lo_bits;
    }
    const uint32_t lo_mask = (1u << lo_bits) - 1u;
    auto digit_of_key = [&](uint64_t key) {
        const uint32_t t = (uint32_t)(key >> 32) & tile_mask;
        return SECOND ? (t & lo_mask) : (t >> lo_bits);
    };

    if (tid < MS_DIGITS) s_cnt[tid] = 0;
    uint64_t key[MS_ITEMS];
#pragma unroll
    for (int i = 0; i < MS_ITEMS; i++) {
        const int j = i * MS_THREADS + tid;
        key[i] = j < count ? __ldg(keys_in + base + j) : 0ull;
    }
#if !FGS_MS_LATE_VALUES
    uint32_t val[MS_ITEMS];
#pragma unroll
    for (int i = 0; i < MS_ITEMS; i++) {
        const int j = i * MS_THREADS + tid;
        val[i] = j < count ? __ldg(vals_in + base + j) : 0u;
    }
#endif
    __syncthreads();
    // Place inside the digit's run: the arrival number of a shared-memory add (any order will do). Letting the lanes
    // that hold the same digit meet first and add as one group (bit masks in shared memory, as the stable digit pass
    // ranks) was measured slower here: 0.27 ms per pass against 0.17.
    uint32_t slot[MS_ITEMS];
#pragma unroll
    for (int i = 0; i < MS_ITEMS; i++) {
        const int j = i * MS_THREADS + tid;
        slot[i] = j < count ? atomicAdd(&s_cnt[digit_of_key(key[i])], 1u) : 0u;
    }
    __syncthreads();
    // thread d: exclusive scan of the counts (start of digit d's run in the reordered partition), and the
    // reservation of the run's place at its destination
    const bool owner = tid < MS_DIGITS;   // whole warps
    const uint32_t c = owner ? s_cnt[tid] : 0u;
    uint32_t inc = c;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const uint32_t a = __shfl_up_sync(FULL_MASK, inc, o);
        if (lane >= o) inc += a;
    }
    if (owner && lane == 31) s_wsum[warp] = inc;
    __syncthreads();
    uint32_t off = 0;
#pragma unroll
    for (int w = 0; w < MS_DIGITS / 32; w++) off += (w < warp) ? s_wsum[w] : 0;
    const uint32_t lstart = off + inc - c;
    if (owner) s_lstart[tid] = lstart;
    uint32_t gstart = 0;
    if (owner && c && FGS_INDEX_OK(cursor_base + tid, SECOND ? MAX_TILE_VALUES : MAX_BUCKETS))
        gstart = atomicAdd(cursors + cursor_base + tid, c);   // its round trip overlaps the reordering below
#if FGS_MS_LATE_VALUES
    // the values are not needed before this point: fetched now, they do not hold registers during the ranking
    uint32_t val[MS_ITEMS];
#pragma unroll
    for (int i = 0; i < MS_ITEMS; i++) {
        const int j = i * MS_THREADS + tid;
        val[i] = j < count ? __ldg(vals_in + base + j) : 0u;
    }
#endif
    __syncthreads();
#pragma unroll
    for (int i = 0; i < MS_ITEMS; i++) {
        const int j = i * MS_THREADS + tid;
        if (j < count) {
            const uint32_t pos = s_lstart[digit_of_key(key[i])] + slot[i];
            if (FGS_INDEX_OK(pos, MS_PART)) {
                st_keys[pos] = key[i];
                st_vals[pos] = val[i];
            }
        }
    }
    if (owner) s_delta[tid] = gstart - lstart;
    __syncthreads();
    for (int j = tid; j < count; j += MS_THREADS) {
        const uint64_t k = st_keys[j];
        const uint32_t dst = s_delta[digit_of_key(k)] + (uint32_t)j;
        if (FGS_INDEX_OK(dst, n) && dst < (uint32_t)n) {   // always true for consistent tables
            keys_out[dst] = k;
            vals_out[dst] = st_vals[j];
        }
    }
}

// A list longer than the in-block sort's capacity: the block sorts it where it lies, in global memory, by a
// least-significant-digit radix sort over the 32 depth bits (four stable 8-bit passes; a pass in which every
// element has the same digit is skipped). The list ping-pongs between its place in the tile-grouped buffers (a)
// and its place in the output (b) and is copied to the output at the end if it stopped in (a). Stable, so the
// result is again what a stable sort of the whole pair list gives for this tile.
constexpr int LONG_THREADS = 512, LONG_ITEMS = 8;
constexpr int LONG_MAX_PASSES = 8;   // four depth digits, preceded by four value digits when ties go by value
// bookkeeping (the digit histograms, run, lstart, per-warp counts, scan, flag) in front of the reordered chunk
constexpr int LONG_BOOK_BYTES = ((LONG_MAX_PASSES + 2) * RADIX * 4 + (LONG_THREADS / 32) * RADIX * 4 + (RADIX / 32) * 4 + 16 + 15) / 16 * 16;
constexpr int LONG_SMEM_BYTES = LONG_BOOK_BYTES + LONG_THREADS * LONG_ITEMS * 12;

// BY_VALUE: pairs with equal depth bits end up in ascending order of their values (four more digit passes, over
// the value, run first); otherwise they keep the order they have in the tile-grouped list.
template <int THREADS, int ITEMS, bool BY_VALUE>
__device__ void long_list_sort(uint64_t* ka, uint32_t* va, uint64_t* kb, uint32_t* vb, int n, unsigned char* smem)
{
    constexpr int WARPS = THREADS / 32, CHUNK = THREADS * ITEMS, PASSES = BY_VALUE ? 8 : 4, FIRST_DEPTH_PASS = PASSES - 4;
    static_assert(THREADS >= RADIX, "thread d owns digit value d");
    static_assert(THREADS == LONG_THREADS && ITEMS == LONG_ITEMS && PASSES <= LONG_MAX_PASSES, "the shared-memory layout is sized for these");
    uint32_t* hist = reinterpret_cast<uint32_t*>(smem);                     // [PASSES][RADIX] digit counts of the whole list
    uint32_t* run = hist + LONG_MAX_PASSES * RADIX;                         // [RADIX] where each digit's run continues
    uint32_t* whist = run + RADIX;                                          // [WARPS][RADIX] per-warp counts of a chunk, then exclusive warp offsets
    uint32_t* scan = whist + WARPS * RADIX;                                 // [RADIX / 32]
    uint32_t* lstart = scan + RADIX / 32;                                   // [RADIX] where a digit's run starts inside the reordered chunk
    int* same = reinterpret_cast<int*>(lstart + RADIX);
    uint64_t* stage_k = reinterpret_cast<uint64_t*>(smem + LONG_BOOK_BYTES);       // [CHUNK] the chunk, reordered by digit
    uint32_t* stage_v = reinterpret_cast<uint32_t*>(smem + LONG_BOOK_BYTES + CHUNK * 8);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const unsigned lt = lanemask_lt();
    // digit of pass `pass`: a byte of the value (the first passes, when ties go by value) or of the depth bits
    auto digit_of_pair = [&](uint64_t key, uint32_t val, int pass) {
        const uint32_t word = pass < FIRST_DEPTH_PASS ? val : (uint32_t)key;
        return (word >> ((pass & 3) * RADIX_BITS)) & (RADIX - 1);
    };
    // all digit histograms from one read of the list
    for (int i = tid; i < PASSES * RADIX; i += THREADS) hist[i] = 0;
    __syncthreads();
    for (int i0 = 0; i0 < n; i0 += THREADS * 4) {
        uint32_t dw[4], vw[4];
#pragma unroll
        for (int u = 0; u < 4; u++) {
            const int i = i0 + u * THREADS + tid;
            dw[u] = i < n ? (uint32_t)ka[i] : 0u;
            vw[u] = (BY_VALUE && i < n) ? va[i] : 0u;
        }
#pragma unroll
        for (int u = 0; u < 4; u++) {
            const bool ok = i0 + u * THREADS + tid < n;
            const unsigned live = __ballot_sync(FULL_MASK, ok);
#pragma unroll
            for (int p = 0; p < PASSES; p++) {
                const uint32_t d = digit_of_pair(dw[u], vw[u], p);
                // depths of one tile often share their upper digits: one add for the warp instead of 32 colliding ones
                const uint32_t d0 = __shfl_sync(FULL_MASK, d, __ffs(live | 0x80000000u) - 1);
                const bool uniform = __all_sync(FULL_MASK, !ok || d == d0);
                if (uniform) { if (ok && (live & lt) == 0) atomicAdd(&hist[p * RADIX + d], (uint32_t)__popc(live)); }
                else if (ok) atomicAdd(&hist[p * RADIX + d], 1u);
            }
        }
    }
    uint64_t* src_k = ka; uint32_t* src_v = va; uint64_t* dst_k = kb; uint32_t* dst_v = vb;
    for (int pass = 0; pass < PASSES; pass++) {
        __syncthreads();   // the histograms are complete; the previous pass's stores are visible to the block
        if (tid == 0) *same = 0;
        __syncthreads();
        uint32_t count = 0, inc = 0;
        if (tid < RADIX) {
            count = hist[pass * RADIX + tid];
            if (count == (uint32_t)n) *same = 1;
            inc = count;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const uint32_t v = __shfl_up_sync(FULL_MASK, inc, o);
                if (lane >= o) inc += v;
            }
            if (lane == 31) scan[warp] = inc;
        }
        __syncthreads();
        if (tid < RADIX) {
            uint32_t off = 0;
            for (int w = 0; w < warp; w++) off += scan[w];
            run[tid] = off + inc - count;
        }
        __syncthreads();
        if (*same) continue;   // every element has the same digit: nothing would move
        for (int c0 = 0; c0 < n; c0 += CHUNK) {
            for (int i = tid; i < WARPS * RADIX; i += THREADS) whist[i] = 0;
            __syncthreads();
            uint64_t key[ITEMS];
            uint32_t val[ITEMS], rank[ITEMS];
            const int wb = c0 + warp * (32 * ITEMS);   // warp-striped: item q of lane l is element wb + q*32 + l
#pragma unroll
            for (int q = 0; q < ITEMS; q++) {
                const int i = wb + q * 32 + lane;
                const bool ok = i < n;
                key[q] = ok ? src_k[i] : 0ull;
                val[q] = ok ? src_v[i] : 0u;
            }
            // ranking as in the digit pass: equal digits meet through bit masks in shared memory (two sets of words per
            // warp in the reorder buffer, which is free at this point), the group's lowest lane adds the group to the
            // warp's counter and hands the old value on
            static_assert(WARPS * 2 * RADIX * 4 <= CHUNK * 8, "mask words fit the reorder buffer");
            uint32_t* my_masks = reinterpret_cast<uint32_t*>(stage_k) + warp * (2 * RADIX);
#pragma unroll
            for (int i = 0; i < 2 * RADIX / 32; i++) my_masks[i * 32 + lane] = 0;
            __syncwarp();
#pragma unroll
            for (int q = 0; q < ITEMS; q++) {
                const bool ok = wb + q * 32 + lane < n;
                const uint32_t d = digit_of_pair(key[q], val[q], pass);
                volatile uint32_t* word = my_masks + (q & 1) * RADIX + d;
                if (ok) atomicOr(const_cast<uint32_t*>(word), 1u << lane);
                __syncwarp();
                const unsigned peers = ok ? *word : (1u << lane);
                __syncwarp();
                uint32_t pre = 0;
                if (ok && (peers & lt) == 0) {
                    *word = 0;
                    pre = atomicAdd(&whist[warp * RADIX + d], (uint32_t)__popc(peers));
                }
                pre = __shfl_sync(FULL_MASK, pre, __ffs(peers) - 1);
                rank[q] = pre + __popc(peers & lt);
            }
            __syncthreads();
            // thread d: the chunk's count of digit d, the warps' exclusive offsets inside it, and (scan over the
            // digits) where its run starts in the reordered chunk
            uint32_t chunk_count = 0, cinc = 0;
            if (tid < RADIX) {
                for (int w = 0; w < WARPS; w++) {
                    const uint32_t c = whist[w * RADIX + tid];
                    whist[w * RADIX + tid] = chunk_count;
                    chunk_count += c;
                }
                cinc = chunk_count;
#pragma unroll
                for (int o = 1; o < 32; o <<= 1) {
                    const uint32_t v = __shfl_up_sync(FULL_MASK, cinc, o);
                    if (lane >= o) cinc += v;
                }
                if (lane == 31) scan[warp] = cinc;
            }
            __syncthreads();
            if (tid < RADIX) {
                uint32_t off = 0;
                for (int w = 0; w < warp; w++) off += scan[w];
                lstart[tid] = off + cinc - chunk_count;
            }
            __syncthreads();
            // reorder the chunk in shared memory, then write each digit's run to its place: neighbouring threads
            // store to neighbouring addresses (scattering element by element costs a memory transaction each)
#pragma unroll
            for (int q = 0; q < ITEMS; q++) {
                if (wb + q * 32 + lane < n) {
                    const uint32_t d = digit_of_pair(key[q], val[q], pass);
                    const uint32_t pos = lstart[d] + whist[warp * RADIX + d] + rank[q];
                    if (FGS_INDEX_OK(pos, CHUNK)) {
                        stage_k[pos] = key[q];
                        stage_v[pos] = val[q];
                    }
                }
            }
            __syncthreads();
            const int valid = min(CHUNK, n - c0);
            for (int j = tid; j < valid; j += THREADS) {
                const uint64_t k = stage_k[j];
                const uint32_t v = stage_v[j];
                const uint32_t d = digit_of_pair(k, v, pass);
                const uint32_t pos = run[d] + ((uint32_t)j - lstart[d]);
                if (FGS_INDEX_OK(pos, n)) {
                    dst_k[pos] = k;
                    dst_v[pos] = v;
                }
            }
            __syncthreads();
            if (tid < RADIX) run[tid] += chunk_count;
        }
        uint64_t* tk = src_k; src_k = dst_k; dst_k = tk;
        uint32_t* tv = src_v; src_v = dst_v; dst_v = tv;
    }
    __syncthreads();
    if (src_k != kb)
        for (int i = tid; i < n; i += THREADS) { kb[i] = src_k[i]; vb[i] = src_v[i]; }
}

template <bool BY_VALUE>
__global__ void __launch_bounds__(LONG_THREADS, 2)
long_list_kernel(uint64_t* keys_grouped, uint32_t* vals_grouped, uint64_t* keys_out, uint32_t* vals_out,
                 const int2* __restrict__ seg, const int* __restrict__ work_count, const uint32_t* __restrict__ work_tiles,
                 int* __restrict__ work_ticket)
{
    chain_release();
    chain_wait();   // nothing is read or written before the kernels ahead on the stream are complete
    extern __shared__ __align__(16) unsigned char s_long[];   // LONG_SMEM_BYTES
    __shared__ int s_w;
    const int work = *work_count;
    for (;;) {   // persistent blocks draw lists from the class's work list
        __syncthreads();
        if (threadIdx.x == 0) s_w = atomicAdd(work_ticket, 1);
        __syncthreads();
        const int w = s_w;
        if (w >= work) break;
        const int2 r = seg[work_tiles[w]];
        long_list_sort<LONG_THREADS, LONG_ITEMS, BY_VALUE>(keys_grouped + r.x, vals_grouped + r.x, keys_out + r.x, vals_out + r.x, r.y - r.x, s_long);
    }
}

// One block per tile: order the tile's pairs in shared memory, then write keys and values in that order (the keys
// are rebuilt from the tile word and the sorted depths). Two orders, chosen at compile time:
//   BY_VALUE == false: by (depth bits, position inside the tile's list). The position makes equal depths keep
//     their input order, i.e. the result is what a stable sort of the whole list gives when the tile-grouped list
//     is in input order (the stable path); the values are gathered by position at the end.
//   BY_VALUE == true: by (depth bits, value). The result no longer depends on the order inside the tile-grouped
//     list at all (the wait-free tile grouping leaves it arbitrary): the sorted list is a function of the SET of
//     pairs. The values are read up front with the keys (coalesced) and travel inside the sort entries, so nothing
//     is gathered at the end. A list whose keys carry bits above the sorted width (never the case for keys built
//     by the preprocess stage) falls back to positions as the entries' low words, with ties in list order.
//
// The order is found by a bucket sort: depths of one tile are spread fairly evenly between the tile's nearest
// and farthest splat, so CAP equal-width depth buckets receive about one element each. The depths stay in
// registers; one shared-memory add per element counts its bucket and returns its arrival number; after a scan
// of the counts the elements are stored bucket by bucket, and one thread per ELEMENT counts the smaller entries of
// its bucket, which is its final place. A tile whose depths pile up in one bucket (more than LOCAL_BUCKET_LIMIT
// elements) is sorted by a bitonic network over the whole tile instead, so the cost stays bounded for any input.
//
// Three instantiations cover list lengths (0,1024], (1024,2048] and (2048,LOCAL_CAP] with shared-memory
// footprints that grow with the class, so that the many short lists run with many blocks per SM; each is a
// small grid of persistent blocks that walks the work list built for its class (an empty
// class costs one launch of blocks that return at once). Longer lists go to long_list_kernel.
#ifndef FGS_LOCAL_BUCKET_LIMIT
#define FGS_LOCAL_BUCKET_LIMIT 192
#endif
#ifndef FGS_LOCAL_BUCKETS_PER_CAP_LOG2
#define FGS_LOCAL_BUCKETS_PER_CAP_LOG2 0   // buckets = CAP * 2^this
#endif
constexpr int LOCAL_BUCKET_LIMIT = FGS_LOCAL_BUCKET_LIMIT;
__host__ __device__ constexpr int local_buckets(int cap) { return FGS_LOCAL_BUCKETS_PER_CAP_LOG2 >= 0 ? cap << (FGS_LOCAL_BUCKETS_PER_CAP_LOG2 >= 0 ? FGS_LOCAL_BUCKETS_PER_CAP_LOG2 : 0) : cap >> (FGS_LOCAL_BUCKETS_PER_CAP_LOG2 < 0 ? -(FGS_LOCAL_BUCKETS_PER_CAP_LOG2) : 0); }
// The bucket tables (counts, starts) are read by threads that own CONSECUTIVE buckets during the scan: thread t reads
// words t*PER ... t*PER + PER - 1, i.e. a warp reads with a stride of PER words and, unpadded, hits each bank PER
// times (the scan then makes up almost half of the kernel's shared-memory traffic). One spare word per 32 spreads
// such a warp over all banks.
#ifndef FGS_LOCAL_PAD
#define FGS_LOCAL_PAD 1
#endif
__host__ __device__ constexpr int bucket_slot(int i) { return FGS_LOCAL_PAD ? i + (i >> 5) : i; }
template <int CAP> constexpr int local_smem_bytes() { return CAP * 8 + CAP * 8 + (bucket_slot(local_buckets(CAP)) + 1) * 4 + (bucket_slot(local_buckets(CAP)) + 1) * 4; }

#ifdef FGS_SORT_TIMING
__device__ unsigned long long g_local_cycles[8];
#define FGS_LT(i) do { if (tid == 0) { const long long now_ = clock64(); atomicAdd(&g_local_cycles[i], (unsigned long long)(now_ - lt_prev_)); lt_prev_ = now_; } } while (0)
#else
#define FGS_LT(i) do { } while (0)
#endif

// BLOCKS: resident blocks per SM that the shared-memory footprint allows; it caps the registers accordingly.
template <int CAP, int THREADS, int BLOCKS, bool BY_VALUE>
__global__ void __launch_bounds__(THREADS, BLOCKS)
local_sort_kernel(const uint64_t* __restrict__ keys_grouped, const uint32_t* __restrict__ vals_grouped,
                  uint64_t* __restrict__ keys_out, uint32_t* __restrict__ vals_out,
                  const int2* __restrict__ seg,
                  const int* __restrict__ work_count, const uint32_t* __restrict__ work_tiles, int* __restrict__ work_ticket)
{
    chain_release();
    chain_wait();   // nothing is read or written before the kernels ahead on the stream are complete
    constexpr int NB = local_buckets(CAP);   // depth buckets
    constexpr int ITEMS = CAP / THREADS;     // elements per thread: positions tid + q * THREADS of the list
    extern __shared__ __align__(16) unsigned char s_local[];
    uint64_t* a = reinterpret_cast<uint64_t*>(s_local);                         // [CAP] depth << 32 | low word, sorted
    uint64_t* bk = reinterpret_cast<uint64_t*>(s_local + CAP * 8);              // [CAP] the same entries, bucket by bucket
    uint32_t* start = reinterpret_cast<uint32_t*>(s_local + CAP * 16);          // [NB + 1], at bucket_slot()
    uint32_t* cursor = start + bucket_slot(NB) + 1;                             // [NB], at bucket_slot()
    __shared__ uint32_t s_min, s_max, s_tile_word, s_wsum[THREADS / 32];
    __shared__ int s_piled;
    __shared__ int2 s_seg;   // the list the block sorts next; y < x: none

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
#ifdef FGS_SORT_TIMING
    long long lt_prev_ = clock64();
#endif
    const int work = *work_count;
    // Persistent blocks draw lists of the class's work list from a ticket counter. The keys (and values) of the NEXT
    // list are requested while the current one is ranked and written out, so their latency is not waited for.
    uint64_t kk[ITEMS];
    uint32_t vv[BY_VALUE ? ITEMS : 1];
    auto fetch = [&](const int2 rr) {
#pragma unroll
        for (int q = 0; q < ITEMS; q++) {
            const int i = tid + q * THREADS;
            kk[q] = i < rr.y - rr.x ? __ldg(keys_grouped + rr.x + i) : 0ull;
            if (BY_VALUE) vv[q] = i < rr.y - rr.x ? __ldg(vals_grouped + rr.x + i) : 0u;
        }
    };
    if (tid == 0) {
        const int w = atomicAdd(work_ticket, 1);
        s_seg = w < work ? seg[work_tiles[w]] : make_int2(0, -1);
    }
    __syncthreads();
    int2 r = s_seg;
    fetch(r);
    while (r.y >= r.x) {
    const int n = r.y - r.x;
    __syncthreads();   // the previous list's shared memory, and s_seg, are no longer read
    int next_ticket = 0;
    if (tid == 0) { s_min = 0xFFFFFFFFu; s_max = 0u; s_piled = 0; s_tile_word = (uint32_t)(kk[0] >> 32); next_ticket = atomicAdd(work_ticket, 1); }
    for (int i = tid; i <= bucket_slot(NB); i += THREADS) cursor[i] = 0;
    FGS_LT(0);
    // The depths stay in registers until they are placed. The high words of a list's keys all hold the tile,
    // unless the caller left bits above the sorted width in them; "mixed" records that, and the write-out then
    // fetches each key's own high word.
    uint32_t d[ITEMS], lo = 0xFFFFFFFFu, hi = 0u, high_and = 0xFFFFFFFFu, high_or = 0u;
#pragma unroll
    for (int q = 0; q < ITEMS; q++) {
        d[q] = (uint32_t)kk[q];
        if (tid + q * THREADS < n) {
            lo = min(lo, d[q]); hi = max(hi, d[q]);
            high_and &= (uint32_t)(kk[q] >> 32); high_or |= (uint32_t)(kk[q] >> 32);
        }
    }
    __syncthreads();   // cursor[] is zero, s_min / s_max / s_tile_word are set up
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        lo = min(lo, __shfl_xor_sync(FULL_MASK, lo, o));
        hi = max(hi, __shfl_xor_sync(FULL_MASK, hi, o));
    }
    if (lane == 0) { atomicMin(&s_min, lo); atomicMax(&s_max, hi); }
    const uint32_t tile_word = s_tile_word;
    const int mixed = __syncthreads_or(n > tid && (high_and != tile_word || high_or != tile_word));
    FGS_LT(1);
    // low word of the sort entries: the value (ties by value, nothing to gather later) or the position in the list
    const bool by_value = BY_VALUE && !mixed;
    uint32_t low[ITEMS];
#pragma unroll
    for (int q = 0; q < ITEMS; q++) low[q] = by_value ? vv[BY_VALUE ? q : 0] : (uint32_t)(tid + q * THREADS);
    uint32_t next_tile = 0;
    if (tid == 0 && next_ticket < work) next_tile = __ldg(work_tiles + next_ticket);
    const uint32_t dmin = s_min, span = s_max - s_min;
    bool gathered = false, fetched = false;
    if (span == 0 && !by_value) {
        // all depths equal and ties in list order: the input order is the sorted order
#pragma unroll
        for (int q = 0; q < ITEMS; q++) {
            const int i = tid + q * THREADS;
            if (i < n) a[i] = ((uint64_t)d[q] << 32) | low[q];
        }
        gathered = true;
    } else if (span != 0) {
        // bucket of a depth: the high word of (depth - nearest depth) * mult, with mult about NB * 2^32 / (span + 1)
        // (rounded in float, hence the clamp): integer arithmetic, monotone in the depth
        const float ratio = 4294967296.0f * (float)NB / ((float)span + 1.0f);
        const uint32_t mult = ratio >= 4294967040.0f ? 0xFFFFFFFFu : (uint32_t)ratio;
        auto bucket_of = [&](uint32_t dd) { return min((int)__umulhi(dd - dmin, mult), NB - 1); };
        // one atomic per element: it counts the bucket and hands the element its arrival number inside it
        uint32_t where[ITEMS];   // bucket | arrival number << 16 (both below 65536)
#pragma unroll
        for (int q = 0; q < ITEMS; q++) {
            const int i = tid + q * THREADS;
            if (i < n) {
                const int b = bucket_of(d[q]);
                if (FGS_INDEX_OK(b, NB)) where[q] = (uint32_t)b | (atomicAdd(&cursor[bucket_slot(b)], 1u) << 16);
            }
        }
        int2 next_seg = make_int2(0, -1);
        if (tid == 0 && next_ticket < work) next_seg = seg[next_tile];
        __syncthreads();
        FGS_LT(2);
        // exclusive scan of the bucket counts: consecutive buckets per thread, then warps, then the block
        constexpr int PER = NB / THREADS;
        uint32_t sum = 0, biggest = 0;
#pragma unroll
        for (int q = 0; q < PER; q++) { const uint32_t c = cursor[bucket_slot(tid * PER + q)]; sum += c; biggest = max(biggest, c); }
        if (biggest > LOCAL_BUCKET_LIMIT) s_piled = 1;
        uint32_t inc = sum;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const uint32_t v = __shfl_up_sync(FULL_MASK, inc, o);
            if (lane >= o) inc += v;
        }
        if (lane == 31) s_wsum[warp] = inc;
        __syncthreads();
        uint32_t off = inc - sum;
        for (int ww = 0; ww < warp; ww++) off += s_wsum[ww];
#pragma unroll
        for (int q = 0; q < PER; q++) { start[bucket_slot(tid * PER + q)] = off; off += cursor[bucket_slot(tid * PER + q)]; }
        if (tid == THREADS - 1) start[bucket_slot(NB)] = off;
        if (tid == 0) s_seg = next_seg;
        __syncthreads();
        FGS_LT(3);
        if (s_piled == 0) {
#pragma unroll
            for (int q = 0; q < ITEMS; q++) {
                const int i = tid + q * THREADS;
                if (i < n) {
                    const uint32_t at = start[bucket_slot((int)(where[q] & 0xFFFFu))] + (where[q] >> 16);
                    if (FGS_INDEX_OK(at, n)) bk[at] = ((uint64_t)d[q] << 32) | low[q];
                }
            }
            fetch(s_seg);   // the registers are free again: request the next list's keys
            fetched = true;
            __syncthreads();
            FGS_LT(4);
            // every bucket in order: one thread per ELEMENT counts the smaller entries of its bucket, so a bucket of
            // L elements costs L steps on L threads, not L^2 on one; the element then goes to its final place in
            // a[]. Entries that are equal as a whole (the same key AND value twice in the input) go in bucket order.
            // (Letting every thread rank its own elements against separate 32-bit depth and low-word arrays -- half the
            // bytes per comparison, no re-read of the element -- was measured slower: 0.45 ms against 0.34 for the
            // tile sorts of the 6 M-Gaussian frame; neighbouring threads here walk neighbouring buckets.)
            for (int x = tid; x < n; x += THREADS) {
                const uint64_t kc = bk[x];
                const int bkt = bucket_of((uint32_t)(kc >> 32));
                const int s0 = (int)start[bucket_slot(bkt)], s1 = (int)start[bucket_slot(bkt + 1)];
                int rank = 0;
                for (int y = s0; y < s1; y++) {
                    const uint64_t other = bk[y];
                    rank += (other < kc) || (other == kc && y < x);
                }
                if (FGS_INDEX_OK(s0 + rank, n)) a[s0 + rank] = kc;
            }
            FGS_LT(5);
            gathered = true;
        } else {
#pragma unroll
            for (int q = 0; q < ITEMS; q++) {
                const int i = tid + q * THREADS;
                if (i < n) a[i] = ((uint64_t)d[q] << 32) | low[q];
            }
        }
    } else {
        // all depths equal, ties by value: the network below orders the values
#pragma unroll
        for (int q = 0; q < ITEMS; q++) {
            const int i = tid + q * THREADS;
            if (i < n) a[i] = ((uint64_t)d[q] << 32) | low[q];
        }
    }
    if (span == 0 && tid == 0) s_seg = next_ticket < work ? seg[next_tile] : make_int2(0, -1);
    __syncthreads();
    if (!gathered) {
        // bitonic network over the whole list (positions beyond n hold the largest key)
        int m = 2;
        while (m < n) m <<= 1;
        for (int i = n + tid; i < m; i += THREADS) a[i] = ~0ull;
        __syncthreads();
        for (int k = 2; k <= m; k <<= 1) {
            for (int j = k >> 1; j > 0; j >>= 1) {
                for (int t = tid; t < (m >> 1); t += THREADS) {
                    const int i = ((t & ~(j - 1)) << 1) | (t & (j - 1));
                    const int p = i | j;
                    const bool up = (i & k) == 0;
                    const uint64_t x = a[i], y = a[p];
                    if ((x > y) == up) { a[i] = y; a[p] = x; }
                }
                __syncthreads();
            }
        }
    }
    const int2 r_next = s_seg;
    if (!fetched) fetch(r_next);
    // a[i] = depth << 32 | low word of the i-th smallest entry
    for (int i = tid; i < n; i += THREADS) {
        const uint64_t k = a[i];
        const uint32_t low_word = (uint32_t)k;
        if (by_value) {
            keys_out[r.x + i] = ((uint64_t)tile_word << 32) | (k >> 32);
            vals_out[r.x + i] = low_word;
        } else if (FGS_INDEX_OK(low_word, n)) {
            const uint32_t high = mixed ? (uint32_t)(__ldg(keys_grouped + r.x + low_word) >> 32) : tile_word;
            keys_out[r.x + i] = ((uint64_t)high << 32) | (k >> 32);
            vals_out[r.x + i] = __ldg(vals_grouped + r.x + low_word);
        }
    }
    FGS_LT(6);
    r = r_next;
    }
}

// sort.cu:9-24 computes the position of the highest set bit plus one
inline int bit_length(uint32_t v) { int b = 0; while (v) { b++; v >>= 1; } return b; }

int g_debug_skip_publish_part = -1;

} // namespace
} // namespace fgs

FGS_BOUNDS_REPORT_FN(fgs_debug_bounds_sort)

#ifdef FGS_SORT_TIMING
extern "C" int fgs_debug_local_phase_cycles(unsigned long long* out8, int reset)
{
    if (cudaMemcpyFromSymbol(out8, fgs::g_local_cycles, sizeof(unsigned long long) * 8) != cudaSuccess) return FGS_ERR_CUDA;
    if (reset) { unsigned long long z[8] = {0}; cudaMemcpyToSymbol(fgs::g_local_cycles, z, sizeof z); }
    return FGS_OK;
}
extern "C" int fgs_debug_sort_phase_cycles(unsigned long long* out8, int reset)
{
    if (cudaMemcpyFromSymbol(out8, fgs::g_phase_cycles, sizeof(unsigned long long) * 8) != cudaSuccess) return FGS_ERR_CUDA;
    if (reset) { unsigned long long z[8] = {0}; cudaMemcpyToSymbol(fgs::g_phase_cycles, z, sizeof z); }
    return FGS_OK;
}
#endif

// Test hook: the partition with this index does not publish its look-back words in the next
// sorts (-1 = off). Later partitions then run out of their poll budget, which exercises the
// bounded wait without faulting or hanging the device.
extern "C" void fgs_debug_sort_skip_publish(int part) { fgs::g_debug_skip_publish_part = part; }

extern "C" size_t fgs_sort_temp_bytes(int64_t num_rendered)
{
    return fgs::make_layout(num_rendered).total;
}

namespace fgs {
int g_debug_plain_sort = 0;

// Launch kinds reported by the profiling entry point.
enum { LAUNCH_HISTOGRAM = 0, LAUNCH_DIGIT_PASS = 1, LAUNCH_SEGMENTS = 2, LAUNCH_LOCAL_SORT = 3 };
constexpr int MAX_LAUNCHES = 2 * MAX_PASSES + 8;

// Order of pairs whose sorted key bits are equal.
enum { ORDER_BY_VALUE = 0,   // ascending value: the wait-free tile grouping (images of at most 2^16 tile values)
       ORDER_STABLE = 1 };   // input order, as the reference's library sort leaves them: look-back digit passes

// Per-device facts and one-time kernel attribute settings, filled under a lock on the first sort of a device.
struct SortDevice { bool ready; int sm_count; };
static SortDevice g_sort_device[64];
static std::mutex g_sort_device_mutex;

static int sort_device(int* dev_out, int* sm_count_out)
{
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return FGS_ERR_CUDA;
    std::lock_guard<std::mutex> guard(g_sort_device_mutex);
    SortDevice& d = g_sort_device[dev];
    if (!d.ready) {
        if (cudaDeviceGetAttribute(&d.sm_count, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || d.sm_count <= 0)
            return FGS_ERR_CUDA;
        cudaError_t e = cudaSuccess;
#define FGS_OPT_IN(SHIFT) if (e == cudaSuccess) e = cudaFuncSetAttribute(onesweep_kernel<SHIFT>, cudaFuncAttributeMaxDynamicSharedMemorySize, SORT_SMEM_BYTES);
        FGS_OPT_IN(0) FGS_OPT_IN(8) FGS_OPT_IN(16) FGS_OPT_IN(24) FGS_OPT_IN(32) FGS_OPT_IN(40) FGS_OPT_IN(48) FGS_OPT_IN(56)
#undef FGS_OPT_IN
        auto opt_in = [&](const void* fn, int bytes) {
            if (e == cudaSuccess) e = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
        };
        opt_in((const void*)local_sort_kernel<LOCAL_CAP, 256, 2, false>, local_smem_bytes<LOCAL_CAP>());
        opt_in((const void*)local_sort_kernel<LOCAL_CAP, 256, 2, true>, local_smem_bytes<LOCAL_CAP>());
        opt_in((const void*)local_sort_kernel<2048, 256, 4, false>, local_smem_bytes<2048>());
        opt_in((const void*)local_sort_kernel<2048, 256, 4, true>, local_smem_bytes<2048>());
        opt_in((const void*)long_list_kernel<false>, LONG_SMEM_BYTES);
        opt_in((const void*)long_list_kernel<true>, LONG_SMEM_BYTES);
        opt_in((const void*)multisplit_kernel<false>, MS_SMEM_BYTES);
        opt_in((const void*)multisplit_kernel<true>, MS_SMEM_BYTES);
        opt_in((const void*)tile_hist_kernel, TILE_HIST_SMEM_VALUES * 4);
        if (e != cudaSuccess) return FGS_ERR_CUDA;
        d.ready = true;
    }
    *dev_out = dev;
    *sm_count_out = d.sm_count;
    return FGS_OK;
}

// `events`, when given, receives one recorded event before the first kernel and one after every kernel;
// `kinds` the kind of each kernel; `num_launches` how many there were.
static int sort_pairs_impl(int num_rendered, int width, int height, int block_x, int block_y,
                           void* temp, size_t temp_bytes,
                           const uint64_t* keys_unsorted, const uint32_t* values_unsorted,
                           uint64_t* keys_sorted, uint32_t* values_sorted, void* stream,
                           cudaEvent_t* events, int* kinds, int* num_launches, const int* n_dev = nullptr,
                           int order = ORDER_BY_VALUE, const uint32_t* given_counts = nullptr, bool counts_in_scratch = false)
{
    // given_counts: pairs per tile left by preprocess in a caller-owned table; counts_in_scratch: left in this
    // scratch's own table (the frame entry point). Either way the pass that would count them is skipped.
    // With n_dev the count lives on the device (clamped to num_rendered, which is then the buffers' capacity).
    if (num_launches) *num_launches = 0;
    if (num_rendered < 0 || num_rendered >= (1 << 30) || width <= 0 || height <= 0 || block_x <= 0 || block_y <= 0)
        return FGS_ERR_BAD_ARG;
    if (num_rendered == 0) return FGS_OK;
    if (!temp || !keys_unsorted || !values_unsorted || !keys_sorted || !values_sorted || !aligned16(temp))
        return FGS_ERR_BAD_ARG;
    const int n = num_rendered;
    const SortLayout L = make_layout(n);
    if (temp_bytes < L.total) return FGS_ERR_TEMP_TOO_SMALL;
    int* dev_status = device_status_ptr();
    if (!dev_status) return FGS_ERR_CUDA;
    cudaStream_t st = static_cast<cudaStream_t>(stream);

    const uint32_t tiles = (uint32_t)(((width + block_x - 1) / block_x) * ((height + block_y - 1) / block_y));
    const int end_bit = 32 + bit_length(tiles);
    const int passes = (end_bit + RADIX_BITS - 1) / RADIX_BITS;
    if (passes > MAX_PASSES) return FGS_ERR_BAD_ARG;
    const int tile_bits = end_bit - 32;
    const int depth_passes = 32 / RADIX_BITS;
    // Tile-bucketed path: the pairs are grouped by tile first, then every tile is sorted by depth inside a block.
    const int tile_passes = passes - depth_passes;
    // With lists this long on average, the tile passes plus the long lists' own depth passes are no fewer than
    // the plain sort's (the count is only known here when it is not on the device).
    const bool very_long_lists = n_dev == nullptr && (int64_t)n > (int64_t)tiles * 16384;
    const bool bucketed = !g_debug_plain_sort && !very_long_lists && tile_bits <= MAX_TILE_BITS && tile_passes >= 1;
    const bool by_value = bucketed && order == ORDER_BY_VALUE;

    char* base = static_cast<char*>(temp);
    uint32_t* tickets = reinterpret_cast<uint32_t*>(base + L.tickets_off);
    uint32_t* hist = reinterpret_cast<uint32_t*>(base + L.hist_off);
    uint32_t* tile_count = reinterpret_cast<uint32_t*>(base + L.tilecnt_off);
    uint32_t* status_words = reinterpret_cast<uint32_t*>(base + L.status_off);
    int2* seg = reinterpret_cast<int2*>(base + L.seg_off);
    uint32_t* tile_cursor = reinterpret_cast<uint32_t*>(base + L.cursor_off);
    uint32_t* bucket_tables = reinterpret_cast<uint32_t*>(base + L.bucket_off);
    uint64_t* alt_keys = reinterpret_cast<uint64_t*>(base + L.alt_keys_off);
    uint32_t* alt_vals = reinterpret_cast<uint32_t*>(base + L.alt_vals_off);

    int dev = 0, sms = 0;
    if (sort_device(&dev, &sms) != FGS_OK) return FGS_ERR_CUDA;

    // ticket counters and look-back regions in use: one per look-back digit pass (none on the wait-free path)
    const int slots = by_value ? 0 : (bucketed ? tile_passes : passes);
    const bool have_counts = by_value && (given_counts != nullptr || counts_in_scratch);
    if (n_dev == nullptr) {
        // with counts from outside, the scratch's own table is not used: only what lies in front of it is cleared
        const size_t clear_bytes = have_counts ? L.tilecnt_off : L.status_off + (size_t)slots * L.parts * RADIX * 4;
        if (cudaMemsetAsync(base, 0, clear_bytes, st) != cudaSuccess) return FGS_ERR_CUDA;
    } else {
        const bool keep = have_counts && counts_in_scratch;
        chain_launch(clear_bookkeeping_kernel, dim3(sms * 8), dim3(256), 0, st, reinterpret_cast<uint32_t*>(base), L.status_off / 4, status_words,
                                                          slots, L.parts, n, n_dev,
                                                          keep ? L.tilecnt_off / 4 : 0, keep ? L.status_off / 4 : 0);
    }

    int launches = 0;
    auto mark = [&](int kind) {
        if (events) cudaEventRecord(events[launches + 1], st);
        if (kinds) kinds[launches] = kind;
        launches++;
    };
    if (events) cudaEventRecord(events[0], st);

    const int resident = PASS_BLOCKS_PER_SM * sms;   // persistent blocks
    const int grid_blocks = L.parts < resident ? L.parts : resident;
    // one look-back digit pass: digit `p` of the key, bookkeeping slot `slot`
    auto digit_pass = [&](int p, int slot, const uint64_t* src_k, const uint32_t* src_v, uint64_t* dst_k, uint32_t* dst_v) -> int {
        const int shift = p * RADIX_BITS;
        const int bits = (end_bit - shift) < RADIX_BITS ? (end_bit - shift) : RADIX_BITS;
        const int use_bulk = aligned16(src_k) && aligned16(src_v);
#define FGS_PASS(SHIFT)                                                                                            \
    case SHIFT:                                                                                                    \
        onesweep_kernel<SHIFT><<<grid_blocks, PASS_THREADS, SORT_SMEM_BYTES, st>>>(                                \
            src_k, src_v, dst_k, dst_v, n, L.parts, (1u << bits) - 1u, use_bulk, tickets + slot, hist + p * RADIX, \
            status_words + (size_t)slot * L.parts * RADIX, dev_status, g_debug_skip_publish_part, n_dev); \
        break;
        switch (shift) {
            FGS_PASS(0) FGS_PASS(8) FGS_PASS(16) FGS_PASS(24) FGS_PASS(32) FGS_PASS(40) FGS_PASS(48) FGS_PASS(56)
        default: return FGS_ERR_BAD_ARG;
        }
#undef FGS_PASS
        return FGS_OK;
    };

    const int tile_values = 1 << (tile_bits < MAX_TILE_BITS ? tile_bits : MAX_TILE_BITS);
    int* class_count = reinterpret_cast<int*>(base + L.flag_off) + 1;   // behind the spare word, cleared above: the classes' list lengths, then their tickets
    uint32_t* class_tiles = reinterpret_cast<uint32_t*>(base + L.class_off);
    auto grid_for = [&](int per_sm) { return tile_values < per_sm * sms ? tile_values : per_sm * sms; };

    if (by_value) {
        // ---- wait-free tile grouping, then tile sorts by (depth bits, value) ----
        const uint32_t* counts = tile_count;
        if (have_counts) {
            if (given_counts != nullptr) counts = given_counts;
        } else {
            const int in_smem = tile_values <= TILE_HIST_SMEM_VALUES && n >= 4 * tile_values;
            int hist_blocks = (int)(((int64_t)n + 65535) / 65536);
            hist_blocks = hist_blocks < 1 ? 1 : (hist_blocks > sms ? sms : hist_blocks);
            chain_launch(tile_hist_kernel, dim3(hist_blocks), dim3(TILE_HIST_THREADS), in_smem ? (size_t)tile_values * 4 : 0, st, 
                keys_unsorted, n, n_dev, (uint32_t)tile_values - 1u, tile_values, in_smem, tile_count);
            mark(LAUNCH_HISTOGRAM);
        }
        // lower and upper halves of the tile bits: at most 8 bits each
        const int lo_bits = tile_bits <= RADIX_BITS ? tile_bits : tile_bits / 2;
        const int buckets = tile_values >> lo_bits;
        chain_launch(tile_scan_kernel, dim3((tile_values + SCAN_CHUNK - 1) / SCAN_CHUNK), dim3(TILE_SCAN_THREADS), 0, st, 
            counts, tile_values, lo_bits, seg, tile_cursor, bucket_tables, class_count, class_tiles, n, n_dev, dev_status,
            tickets /* the first ticket word: cleared above, not used by any pass of this path */);
        mark(LAUNCH_SEGMENTS);
        const int ms_parts = (int)(((int64_t)n + MS_PART - 1) / MS_PART);
        const uint64_t* src_k = keys_unsorted;
        const uint32_t* src_v = values_unsorted;
        if (buckets > 1) {
            chain_launch(multisplit_kernel<false>, dim3(ms_parts), dim3(MS_THREADS), MS_SMEM_BYTES, st, 
                src_k, src_v, keys_sorted, values_sorted, n, n_dev, (uint32_t)tile_values - 1u, lo_bits, buckets,
                bucket_tables, bucket_tables /* the coarse buckets' cursors lead the tables */);
            mark(LAUNCH_DIGIT_PASS);
            src_k = keys_sorted;
            src_v = values_sorted;
        }
        // every coarse bucket is cut into partitions of its own: at most one ragged partition more per bucket
        chain_launch(multisplit_kernel<true>, dim3(ms_parts + buckets), dim3(MS_THREADS), MS_SMEM_BYTES, st, 
            src_k, src_v, alt_keys, alt_vals, n, n_dev, (uint32_t)tile_values - 1u, lo_bits, buckets, bucket_tables, tile_cursor);
        mark(LAUNCH_DIGIT_PASS);
        chain_launch(local_sort_kernel<1024, 128, 8, true>, dim3(grid_for(12)), dim3(128), local_smem_bytes<1024>(), st, 
            alt_keys, alt_vals, keys_sorted, values_sorted, seg, class_count + 0, class_tiles, class_count + LOCAL_CLASSES + 0);
        mark(LAUNCH_LOCAL_SORT);
        chain_launch(local_sort_kernel<2048, 256, 4, true>, dim3(grid_for(6)), dim3(256), local_smem_bytes<2048>(), st, 
            alt_keys, alt_vals, keys_sorted, values_sorted, seg, class_count + 1, class_tiles + MAX_TILE_VALUES, class_count + LOCAL_CLASSES + 1);
        mark(LAUNCH_LOCAL_SORT);
        chain_launch(local_sort_kernel<LOCAL_CAP, 256, 2, true>, dim3(grid_for(3)), dim3(256), local_smem_bytes<LOCAL_CAP>(), st, 
            alt_keys, alt_vals, keys_sorted, values_sorted, seg, class_count + 2, class_tiles + 2 * MAX_TILE_VALUES, class_count + LOCAL_CLASSES + 2);
        mark(LAUNCH_LOCAL_SORT);
        chain_launch(long_list_kernel<true>, dim3(grid_for(2)), dim3(LONG_THREADS), LONG_SMEM_BYTES, st, 
            alt_keys, alt_vals, keys_sorted, values_sorted, seg, class_count + 3, class_tiles + 3 * MAX_TILE_VALUES, class_count + LOCAL_CLASSES + 3);
        mark(LAUNCH_LOCAL_SORT);
        if (num_launches) *num_launches = launches;
        return launch_status();
    }

    int hist_blocks = L.parts < sms * 8 ? L.parts : sms * 8;
    // the bucketed path needs the tile digits' counts only
    histogram_kernel<<<hist_blocks, HIST_THREADS, 0, st>>>(keys_unsorted, n, n_dev, bucketed ? depth_passes : 0, passes, end_bit, hist);
    mark(LAUNCH_HISTOGRAM);

    if (bucketed) {
        // tile digits, least significant first; the last one leaves the tile-grouped list in the alternate buffers
        const uint64_t* src_k = keys_unsorted;
        const uint32_t* src_v = values_unsorted;
        for (int i = 0; i < tile_passes; i++) {
            const bool to_alt = ((tile_passes - 1 - i) & 1) == 0;
            uint64_t* dst_k = to_alt ? alt_keys : keys_sorted;
            uint32_t* dst_v = to_alt ? alt_vals : values_sorted;
            if (digit_pass(depth_passes + i, i, src_k, src_v, dst_k, dst_v) != FGS_OK) return FGS_ERR_BAD_ARG;
            mark(LAUNCH_DIGIT_PASS);
            src_k = dst_k;
            src_v = dst_v;
        }
        segments_kernel<<<(tile_values + SEG_TILES - 1) / SEG_TILES, SEG_THREADS, 0, st>>>(alt_keys, n, n_dev, tile_values, (uint32_t)tile_values - 1u, seg,
                                                                  class_count, class_tiles);
        mark(LAUNCH_SEGMENTS);
        chain_launch(local_sort_kernel<1024, 128, 9, false>, dim3(grid_for(12)), dim3(128), local_smem_bytes<1024>(), st, 
            alt_keys, alt_vals, keys_sorted, values_sorted, seg, class_count + 0, class_tiles, class_count + LOCAL_CLASSES + 0);
        mark(LAUNCH_LOCAL_SORT);
        chain_launch(local_sort_kernel<2048, 256, 4, false>, dim3(grid_for(6)), dim3(256), local_smem_bytes<2048>(), st, 
            alt_keys, alt_vals, keys_sorted, values_sorted, seg, class_count + 1, class_tiles + MAX_TILE_VALUES, class_count + LOCAL_CLASSES + 1);
        mark(LAUNCH_LOCAL_SORT);
        chain_launch(local_sort_kernel<LOCAL_CAP, 256, 2, false>, dim3(grid_for(3)), dim3(256), local_smem_bytes<LOCAL_CAP>(), st, 
            alt_keys, alt_vals, keys_sorted, values_sorted, seg, class_count + 2, class_tiles + 2 * MAX_TILE_VALUES, class_count + LOCAL_CLASSES + 2);
        mark(LAUNCH_LOCAL_SORT);
        chain_launch(long_list_kernel<false>, dim3(grid_for(2)), dim3(LONG_THREADS), LONG_SMEM_BYTES, st, 
            alt_keys, alt_vals, keys_sorted, values_sorted, seg, class_count + 3, class_tiles + 3 * MAX_TILE_VALUES, class_count + LOCAL_CLASSES + 3);
        mark(LAUNCH_LOCAL_SORT);
    }
    // the plain sort: all digits, least significant first (images with more tiles than the bucketed path takes)
    if (!bucketed) {
        const uint64_t* src_k = keys_unsorted;
        const uint32_t* src_v = values_unsorted;
        for (int p = 0; p < passes; p++) {
            const bool to_out = ((passes - 1 - p) & 1) == 0;
            uint64_t* dst_k = to_out ? keys_sorted : alt_keys;
            uint32_t* dst_v = to_out ? values_sorted : alt_vals;
            if (digit_pass(p, p, src_k, src_v, dst_k, dst_v) != FGS_OK) return FGS_ERR_BAD_ARG;
            mark(LAUNCH_DIGIT_PASS);
            src_k = dst_k;
            src_v = dst_v;
        }
    }
    if (num_launches) *num_launches = launches;
    return launch_status();
}
} // namespace fgs

namespace fgs {
// Sort whose pair count is the device counter *n_dev (at most `capacity`); used by the frame entry point.
int sort_pairs_device_count(int capacity, const int* n_dev, int width, int height, int block_x, int block_y,
                            void* temp, size_t temp_bytes, const uint64_t* keys_unsorted, const uint32_t* values_unsorted,
                            uint64_t* keys_sorted, uint32_t* values_sorted, void* stream, bool counts_in_scratch)
{
    if (!n_dev || capacity <= 0) return FGS_ERR_BAD_ARG;
    return sort_pairs_impl(capacity, width, height, block_x, block_y, temp, temp_bytes, keys_unsorted, values_unsorted,
                           keys_sorted, values_sorted, stream, nullptr, nullptr, nullptr, n_dev, ORDER_BY_VALUE, nullptr,
                           counts_in_scratch);
}

// Where the frame entry point may let preprocess leave its per-tile counts (inside the sort's scratch) and its index
// list (the alternate value buffer at the scratch's end, which the sort does not touch before its second pass).
void sort_scratch_regions(int64_t capacity, size_t* tile_count_off, size_t* list_off, size_t* list_bytes)
{
    const SortLayout L = make_layout(capacity);
    *tile_count_off = L.tilecnt_off;
    *list_off = L.alt_vals_off;
    *list_bytes = L.total - L.alt_vals_off;
}
} // namespace fgs

// Test hook: non-zero makes the next sorts skip the tile-bucketed paths and run the plain digit passes only.
extern "C" void fgs_debug_sort_plain(int on) { fgs::g_debug_plain_sort = on; }

extern "C" int fgs_sort_pairs(int num_rendered, int width, int height, int block_x, int block_y,
                              void* temp, size_t temp_bytes,
                              const uint64_t* keys_unsorted, const uint32_t* values_unsorted,
                              uint64_t* keys_sorted, uint32_t* values_sorted, void* stream)
{
    return fgs::sort_pairs_impl(num_rendered, width, height, block_x, block_y, temp, temp_bytes, keys_unsorted,
                                values_unsorted, keys_sorted, values_sorted, stream, nullptr, nullptr, nullptr);
}

extern "C" int fgs_sort_pairs_counted(int num_rendered, int width, int height, int block_x, int block_y,
                                      void* temp, size_t temp_bytes,
                                      const uint64_t* keys_unsorted, const uint32_t* values_unsorted,
                                      uint64_t* keys_sorted, uint32_t* values_sorted, const uint32_t* tile_counts, void* stream)
{
    return fgs::sort_pairs_impl(num_rendered, width, height, block_x, block_y, temp, temp_bytes, keys_unsorted,
                                values_unsorted, keys_sorted, values_sorted, stream, nullptr, nullptr, nullptr, nullptr,
                                fgs::ORDER_BY_VALUE, tile_counts);
}

extern "C" int fgs_sort_pairs_stable(int num_rendered, int width, int height, int block_x, int block_y,
                                     void* temp, size_t temp_bytes,
                                     const uint64_t* keys_unsorted, const uint32_t* values_unsorted,
                                     uint64_t* keys_sorted, uint32_t* values_sorted, void* stream)
{
    return fgs::sort_pairs_impl(num_rendered, width, height, block_x, block_y, temp, temp_bytes, keys_unsorted,
                                values_unsorted, keys_sorted, values_sorted, stream, nullptr, nullptr, nullptr, nullptr,
                                fgs::ORDER_STABLE);
}

extern "C" int fgs_sort_pairs_profile(int num_rendered, int width, int height, int block_x, int block_y,
                                      void* temp, size_t temp_bytes,
                                      const uint64_t* keys_unsorted, const uint32_t* values_unsorted,
                                      uint64_t* keys_sorted, uint32_t* values_sorted, const uint32_t* tile_counts, void* stream,
                                      float* launch_ms, int* launch_kind, int capacity, int* num_launches)
{
    using namespace fgs;
    if (!launch_ms || !launch_kind || !num_launches || capacity < MAX_LAUNCHES) return FGS_ERR_BAD_ARG;
    cudaEvent_t ev[MAX_LAUNCHES + 1];
    for (auto& e : ev)
        if (cudaEventCreate(&e) != cudaSuccess) return FGS_ERR_CUDA;
    int launches = 0;
    int st = sort_pairs_impl(num_rendered, width, height, block_x, block_y, temp, temp_bytes, keys_unsorted,
                             values_unsorted, keys_sorted, values_sorted, stream, ev, launch_kind, &launches, nullptr,
                             ORDER_BY_VALUE, tile_counts);
    *num_launches = 0;
    if (st == FGS_OK && launches > 0) {
        if (cudaStreamSynchronize(static_cast<cudaStream_t>(stream)) != cudaSuccess) st = FGS_ERR_CUDA;
        for (int i = 0; st == FGS_OK && i < launches; i++)
            if (cudaEventElapsedTime(&launch_ms[i], ev[i], ev[i + 1]) != cudaSuccess) st = FGS_ERR_CUDA;
        if (st == FGS_OK) *num_launches = launches;
    }
    for (auto& e : ev) cudaEventDestroy(e);
    return st;
}

// ---- sorting without any caller-provided or allocated scratch ----
// Scratch for fgs_sort_pairs_static: a fixed array inside the library's device image. Every GPU that loads the
// library carries these bytes until the process exits, which is why the limit is modest.
#define FGS_STATIC_SORT_MAX_PAIRS (1 << 18)
namespace fgs {
namespace {
constexpr size_t static_sort_bytes() { return layout_total(FGS_STATIC_SORT_MAX_PAIRS); }
static __device__ __align__(256) unsigned char g_static_sort_scratch[static_sort_bytes()];
void* g_static_sort_ptr[64];   // device address of the array, per device, resolved on first use (under the lock below)
std::mutex g_static_sort_mutex;
} // namespace
} // namespace fgs

extern "C" int fgs_sort_static_max_pairs(void) { return FGS_STATIC_SORT_MAX_PAIRS; }

extern "C" int fgs_sort_pairs_static(int num_rendered, int width, int height, int block_x, int block_y,
                                     const uint64_t* keys_unsorted, const uint32_t* values_unsorted,
                                     uint64_t* keys_sorted, uint32_t* values_sorted, void* stream)
{
    using namespace fgs;
    if (num_rendered < 0) return FGS_ERR_BAD_ARG;
    if (num_rendered > FGS_STATIC_SORT_MAX_PAIRS) return FGS_ERR_TEMP_TOO_SMALL;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return FGS_ERR_CUDA;
    void* scratch = nullptr;
    {
        std::lock_guard<std::mutex> guard(g_static_sort_mutex);
        if (!g_static_sort_ptr[dev]) {
            // In host code the array's name is only a handle; the address kernels can use comes from the runtime,
            // asked for with this device current.
            void* p = nullptr;
            if (cudaGetSymbolAddress(&p, g_static_sort_scratch) != cudaSuccess || !p) return FGS_ERR_CUDA;
            g_static_sort_ptr[dev] = p;
        }
        scratch = g_static_sort_ptr[dev];
    }
    if (make_layout(FGS_STATIC_SORT_MAX_PAIRS).total > static_sort_bytes()) return FGS_ERR_TEMP_TOO_SMALL;
    return sort_pairs_impl(num_rendered, width, height, block_x, block_y, scratch, static_sort_bytes(),
                           keys_unsorted, values_unsorted, keys_sorted, values_sorted, stream, nullptr, nullptr, nullptr);
}
