// Onesweep least-significant-digit radix sort of (64-bit key, 32-bit value) pairs, sm_100a.
//
// Replaces the library radix sort the reference calls (csrc/cuda_rasterizer/sort.cu:28-44):
// a STABLE sort on key bits [0, end_bit), end_bit = 32 + bit_length(#tiles)
// (csrc/cuda_rasterizer/sort.cu:9-24,39), inputs preserved, outputs in separate buffers.
//
// Structure:
//   * one histogram kernel reads the keys once and counts every 8-bit digit of the live
//     bits (ceil(end_bit / 8) digits; bits at or above end_bit are never looked at);
//   * one "onesweep" kernel per digit: a block (512 threads) takes the next partition of 4096 pairs from a
//     ticket counter, ranks its keys by digit (warp match + per-warp counters, which keeps the
//     sort stable), publishes its per-digit counts and obtains the counts of all earlier
//     partitions by decoupled look-back, then moves keys and values through shared memory so
//     that every digit's run leaves as contiguous global stores.
//   Each pass reads 12 bytes and writes 12 bytes per pair once; passes ping-pong between the
//   output buffers and an alternate pair buffer inside the caller's scratch.
//
// Every wait on another block is bounded: the look-back gives up after a fixed poll budget,
// raises FGS_ERR_LOOKBACK_TIMEOUT in the device status word, still publishes its own
// (then meaningless) prefix so that later partitions do not wait on it, and the block ends
// without scattering. Tickets are handed out in launch order, so a block only ever waits on
// partitions whose blocks are already running.

#include "fgs_common.cuh"

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
#ifndef FGS_SORT_STAGES
#define FGS_SORT_STAGES 2      // 2: bulk-copy prefetch of the next partition; 1: plain loads, smaller footprint
#endif
#ifndef FGS_SORT_BLOCKS_PER_SM
#define FGS_SORT_BLOCKS_PER_SM 2
#endif
#ifndef FGS_LOOKBACK_WINDOW
#define FGS_LOOKBACK_WINDOW 8
#endif
constexpr int SORT_THREADS = FGS_SORT_THREADS;
constexpr int SORT_WARPS = SORT_THREADS / 32;
constexpr int SORT_ITEMS = FGS_SORT_ITEMS;               // pairs per thread
constexpr int SORT_PART = SORT_THREADS * SORT_ITEMS;    // pairs per partition
constexpr int RADIX_BITS = 8;
constexpr int RADIX = 1 << RADIX_BITS;
constexpr int MAX_PASSES = 8;
constexpr int HIST_THREADS = 256;
static_assert(RADIX <= SORT_THREADS, "thread d < RADIX owns digit value d in the scans and the look-back");

constexpr uint32_t FLAG_AGGREGATE = 1u << 30;           // this partition's count only
constexpr uint32_t FLAG_INCLUSIVE = 2u << 30;           // count of this and all earlier partitions
constexpr uint32_t FLAG_MASK = 3u << 30;
constexpr uint32_t VALUE_MASK = ~FLAG_MASK;
constexpr int LOOKBACK_MAX_POLLS = 1 << 20;             // x (sleep + one L2 read): gives up after about a second
constexpr int LOOKBACK_WINDOW = FGS_LOOKBACK_WINDOW;                      // earlier partitions inspected per round trip
constexpr int STAGE_BYTES = SORT_PART * 12;             // keys + values of one partition
constexpr int LOOKBACK_SLEEP_NS = FGS_LOOKBACK_SLEEP_NS;
constexpr int SORT_STAGES = FGS_SORT_STAGES;
constexpr int SORT_BLOCKS_PER_SM = FGS_SORT_BLOCKS_PER_SM;
constexpr int SORT_SMEM_BYTES = SORT_STAGES * STAGE_BYTES;
constexpr int MBAR_MAX_POLLS = 1 << 20;                 // tries of at most ~1 us each: a bulk copy gets about a second

__device__ __forceinline__ uint32_t ld_relaxed(const uint32_t* p)
{
    uint32_t v;
    asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_relaxed(uint32_t* p, uint32_t v)
{
    asm volatile("st.relaxed.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

struct SortLayout {
    size_t tickets_off, hist_off, status_off, alt_keys_off, alt_vals_off, total;
    int parts;
};

inline size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

inline SortLayout make_layout(int64_t n)
{
    SortLayout L;
    if (n < 1) n = 1;
    L.parts = (int)((n + SORT_PART - 1) / SORT_PART);
    L.tickets_off = 0;                                           // MAX_PASSES tickets (+ padding)
    L.hist_off = 256;                                            // MAX_PASSES x RADIX counts
    L.status_off = L.hist_off + (size_t)MAX_PASSES * RADIX * 4;  // passes x parts x RADIX words
    L.alt_keys_off = align_up(L.status_off + (size_t)MAX_PASSES * L.parts * RADIX * 4, 256);
    L.alt_vals_off = align_up(L.alt_keys_off + (size_t)n * 8, 256);
    L.total = align_up(L.alt_vals_off + (size_t)n * 4, 256);
    return L;
}

// ---- digit histograms of all passes in one read of the keys ----
__global__ void __launch_bounds__(HIST_THREADS)
histogram_kernel(const uint64_t* __restrict__ keys, int n, int passes, int end_bit, uint32_t* __restrict__ hist)
{
    __shared__ uint32_t s_hist[MAX_PASSES * RADIX];
    for (int i = threadIdx.x; i < passes * RADIX; i += HIST_THREADS) s_hist[i] = 0;
    __syncthreads();
    const uint64_t live = end_bit >= 64 ? ~0ull : ((1ull << end_bit) - 1ull);
    for (int64_t i = (int64_t)blockIdx.x * HIST_THREADS + threadIdx.x; i < n; i += (int64_t)gridDim.x * HIST_THREADS) {
        const uint64_t k = __ldg(keys + i) & live;
        for (int p = 0; p < passes; p++)
            atomicAdd(&s_hist[p * RADIX + (uint32_t)((k >> (p * RADIX_BITS)) & (RADIX - 1))], 1u);
    }
    __syncthreads();
    for (int i = threadIdx.x; i < passes * RADIX; i += HIST_THREADS) {
        const uint32_t c = s_hist[i];
        if (c) atomicAdd(hist + i, c);
    }
}

// ---- one onesweep pass ----
// Lanes of the warp that hold the same 8-bit digit: one vote per bit (the match.any instruction gives the
// same mask but measured several hundred cycles per call here; eight votes are an order of magnitude cheaper).
__device__ __forceinline__ unsigned match_digit(uint32_t d)
{
    unsigned peers = FULL_MASK;
#pragma unroll
    for (int b = 0; b < RADIX_BITS; b++) {
        const bool bit = (d >> b) & 1u;
        const unsigned vote = __ballot_sync(FULL_MASK, bit);
        peers &= bit ? vote : ~vote;
    }
    return peers;
}

// ---- asynchronous bulk copies (TMA, 1-D, no multicast) and their mbarrier ----
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

// ---- one onesweep pass ----
// Persistent blocks (two per SM). A block owns two shared-memory stages of one partition each
// (4096 keys + 4096 values): while it ranks and scatters the partition in one stage, the bulk
// copy of its next partition is already filling the other, so the HBM reads of a block never
// stop. The stage that was just consumed into registers doubles as the buffer in which the
// partition is reordered before it is written out.
__global__ void __launch_bounds__(SORT_THREADS, SORT_BLOCKS_PER_SM)
onesweep_kernel(const uint64_t* __restrict__ keys_in, const uint32_t* __restrict__ vals_in,
                uint64_t* __restrict__ keys_out, uint32_t* __restrict__ vals_out,
                int n, int num_parts, int shift, uint32_t digit_mask, int use_bulk,
                uint32_t* __restrict__ ticket, const uint32_t* __restrict__ hist,
                uint32_t* __restrict__ status_words, int* __restrict__ dev_status, int skip_publish_part)
{
    extern __shared__ __align__(128) unsigned char s_dyn[];   // 2 stages x (keys 8*PART | values 4*PART)
    __shared__ __align__(8) uint64_t s_bar[2];
    __shared__ uint16_t s_whist[SORT_WARPS][RADIX];    // per-warp digit counts, then exclusive warp offsets
    __shared__ uint32_t s_local_start[RADIX];           // start of each digit's run inside the partition
    __shared__ int64_t s_global_delta[RADIX];           // global index of a digit's run minus its local start
    __shared__ uint32_t s_digit_base[RADIX];            // exclusive scan of the global histogram
    __shared__ uint32_t s_scan[RADIX / 32];
    __shared__ uint32_t s_tickets[4];                   // partition of iteration i lives in s_tickets[i & 3]
    __shared__ int s_abort;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const unsigned lt = lanemask_lt();
    auto stage_keys = [&](int st) { return reinterpret_cast<uint64_t*>(s_dyn + (size_t)st * STAGE_BYTES); };
    auto stage_vals = [&](int st) { return reinterpret_cast<uint32_t*>(s_dyn + (size_t)st * STAGE_BYTES + SORT_PART * 8); };
    // Thread 0: start the bulk copy of a full partition into a stage (the ragged last partition and
    // unaligned inputs are copied with plain loads by the whole block when the stage is consumed).
    uint32_t pending = 0;   // thread 0: bit st = a bulk copy into stage st has been started and not yet waited for
    auto prefetch = [&](int st, uint32_t part) {
        if (use_bulk && part < (uint32_t)num_parts && (int64_t)(part + 1) * SORT_PART <= (int64_t)n) {
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            mbar_expect_tx(&s_bar[st], SORT_PART * 12);
            bulk_load(stage_keys(st), keys_in + (size_t)part * SORT_PART, SORT_PART * 8, &s_bar[st]);
            bulk_load(stage_vals(st), vals_in + (size_t)part * SORT_PART, SORT_PART * 4, &s_bar[st]);
            pending |= 1u << st;
        }
    };

    if (tid == 0) {
        mbar_init(&s_bar[0], 1);
        mbar_init(&s_bar[1], 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        s_abort = 0;
        const uint32_t first = atomicAdd(ticket, 1u);
        s_tickets[0] = first;
        if (SORT_STAGES == 2) prefetch(0, first);
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

    uint32_t phase_bits = 0;   // bit st = parity to wait for on stage st
#ifdef FGS_SORT_TIMING
    long long t_prev_ = clock64();
#endif
    for (int it = 0;; it++) {
        const int st = (SORT_STAGES == 2) ? (it & 1) : 0;
        const uint32_t part = s_tickets[it & 3];
        if (part >= (uint32_t)num_parts) break;
        const int64_t part_base = (int64_t)part * SORT_PART;
        const int valid = (int)min((int64_t)SORT_PART, (int64_t)n - part_base);
        const bool bulk = SORT_STAGES == 2 && use_bulk && valid == SORT_PART;
        // Thread 0: start the copy of the next partition (its ticket was taken one iteration ago) into
        // the other stage, and request the ticket after that; the ticket is only stored at the end of
        // the iteration, so its round trip to the L2 never stalls the block.
        uint32_t ticket_after_next = 0;
        if (tid == 0) {
            if (SORT_STAGES == 2) prefetch(st ^ 1, s_tickets[(it + 1) & 3]);
            ticket_after_next = atomicAdd(ticket, 1u);
        }
        for (int i = tid; i < SORT_WARPS * RADIX / 2; i += SORT_THREADS) reinterpret_cast<uint32_t*>(&s_whist[0][0])[i] = 0;

        uint64_t* sk = stage_keys(st);
        uint32_t* sv = stage_vals(st);
        uint64_t key[SORT_ITEMS];
        uint32_t val[SORT_ITEMS];
        const int wbase = warp * (32 * SORT_ITEMS);   // warp-striped: item i of lane l sits at wbase + i*32 + l
        if (bulk) {
            if (!mbar_wait(&s_bar[st], (phase_bits >> st) & 1u)) { atomicOr(dev_status, FGS_ERR_LOOKBACK_TIMEOUT); s_abort = 1; }
            else pending &= ~(1u << st);
            phase_bits ^= 1u << st;
#pragma unroll
            for (int i = 0; i < SORT_ITEMS; i++) { key[i] = sk[wbase + i * 32 + lane]; val[i] = sv[wbase + i * 32 + lane]; }
        } else {
#pragma unroll
            for (int i = 0; i < SORT_ITEMS; i++) {
                const int local = wbase + i * 32 + lane;
                key[i] = local < valid ? __ldg(keys_in + part_base + local) : ~0ull;
                val[i] = local < valid ? __ldg(vals_in + part_base + local) : 0u;
            }
        }
        __syncthreads();   // s_whist zeroed, every thread holds its items
        FGS_T(0);
        if (s_abort) break;

        // rank within the warp, item by item, so equal digits keep their input order
        uint32_t rank[SORT_ITEMS];
#pragma unroll
        for (int i = 0; i < SORT_ITEMS; i++) {
            const uint32_t d = (uint32_t)(key[i] >> shift) & digit_mask;
            const unsigned peers = match_digit(d);
            const int leader = __ffs(peers) - 1;
            uint32_t pre = 0;
            if (lane == leader) {
                pre = s_whist[warp][d];
                s_whist[warp][d] = (uint16_t)(pre + __popc(peers));
            }
            pre = __shfl_sync(FULL_MASK, pre, leader);
            rank[i] = pre + __popc(peers & lt);
            __syncwarp();
        }
        __syncthreads();
        FGS_T(1);

        // threads 0..RADIX-1: thread d owns digit value d
        uint32_t count = 0, inc_l = 0;
        uint32_t* my_status = status_words + (size_t)part * RADIX + tid;
        const bool publish = (int)part != skip_publish_part;
        // Look-back window: the status words of the LOOKBACK_WINDOW nearest earlier partitions are
        // requested together, right after this partition's own count is published, and only looked at
        // after the block has reordered its items in shared memory, so their latency is hidden and a
        // look-back that has to cross several partitions costs one round trip, not one per partition.
        uint32_t sw[LOOKBACK_WINDOW];
        int64_t p0 = (int64_t)part - 1;
        if (tid < RADIX) {
#pragma unroll
            for (int w = 0; w < SORT_WARPS; w++) {
                const uint32_t c = s_whist[w][tid];
                s_whist[w][tid] = (uint16_t)count;   // exclusive offset of warp w inside the digit's run
                count += c;
            }
            if (publish) st_relaxed(my_status, (part == 0 ? FLAG_INCLUSIVE : FLAG_AGGREGATE) | count);
#pragma unroll
            for (int k = 0; k < LOOKBACK_WINDOW; k++)
                sw[k] = (p0 - k >= 0) ? ld_relaxed(status_words + (size_t)(p0 - k) * RADIX + tid) : FLAG_INCLUSIVE;
            inc_l = count;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const uint32_t a = __shfl_up_sync(FULL_MASK, inc_l, o);
                if (lane >= o) inc_l += a;
            }
            if (lane == 31) s_scan[warp] = inc_l;
        }
        __syncthreads();
        uint32_t local_start = 0;
        if (tid < RADIX) {
            uint32_t off_l = 0;
#pragma unroll
            for (int w = 0; w < RADIX / 32; w++) off_l += (w < warp) ? s_scan[w] : 0;
            local_start = off_l + inc_l - count;
            s_local_start[tid] = local_start;
        }
        __syncthreads();
        FGS_T(2);

        // place keys and values at their partition-local sorted position (the stage is free: its
        // contents live in registers)
#pragma unroll
        for (int i = 0; i < SORT_ITEMS; i++) {
            const uint32_t d = (uint32_t)(key[i] >> shift) & digit_mask;
            const uint32_t pos = s_local_start[d] + s_whist[warp][d] + rank[i];
            sk[pos] = key[i];
            sv[pos] = val[i];
        }
        FGS_T(3);

        // decoupled look-back over earlier partitions for digit `tid`
        if (tid < RADIX) {
            uint32_t earlier = 0;
            bool done = (part == 0), failed = false;
            int polls = 0;
            while (!done) {
                int used = 0;   // window entries consumed, nearest partition first, while they are published
#pragma unroll
                for (int k = 0; k < LOOKBACK_WINDOW; k++) {
                    if (!done && used == k) {
                        const uint32_t f = sw[k] & FLAG_MASK;
                        if (f != 0) {
                            earlier += sw[k] & VALUE_MASK;
                            used = k + 1;
                            done = (f == FLAG_INCLUSIVE);   // partition 0 always publishes FLAG_INCLUSIVE
                        }
                    }
                }
                if (done) break;
                if (used == 0) {
                    // the nearest unread partition has not published yet: wait for that one word only (polling
                    // whole windows from every block saturates the L2) and back off between polls
                    if (++polls > LOOKBACK_MAX_POLLS) { failed = true; break; }
                    __nanosleep(LOOKBACK_SLEEP_NS);
                    sw[0] = ld_relaxed(status_words + (size_t)p0 * RADIX + tid);
                    continue;
                }
                p0 -= used;
#pragma unroll
                for (int k = 0; k < LOOKBACK_WINDOW; k++)
                    sw[k] = (p0 - k >= 0) ? ld_relaxed(status_words + (size_t)(p0 - k) * RADIX + tid) : FLAG_INCLUSIVE;
            }
            if (failed) { atomicOr(dev_status, FGS_ERR_LOOKBACK_TIMEOUT); s_abort = 1; }
            if (publish && part > 0) st_relaxed(my_status, FLAG_INCLUSIVE | ((earlier + count) & VALUE_MASK));
            s_global_delta[tid] = (int64_t)s_digit_base[tid] + (int64_t)earlier - (int64_t)local_start;
        }
        __syncthreads();
        FGS_T(4);
        if (s_abort) break;

        // runs of equal digits are contiguous in shared memory and in the destination
#pragma unroll
        for (int i = 0; i < SORT_ITEMS; i++) {
            const int j = i * SORT_THREADS + tid;
            if (j < valid) {
                const uint64_t k = sk[j];
                const uint32_t d = (uint32_t)(k >> shift) & digit_mask;
                const int64_t dst = s_global_delta[d] + j;
                keys_out[dst] = k;
                vals_out[dst] = sv[j];
            }
        }
        FGS_T(5);
        if (tid == 0) s_tickets[(it + 2) & 3] = ticket_after_next;
        __syncthreads();   // the stage may now be refilled by the copy started in the next iteration
        FGS_T(6);
    }

    // Leaving early (a wait gave up): a copy into the other stage may still be in flight; wait for it
    // (bounded) so that nothing writes into shared memory after the block is gone.
    if (tid == 0) {
        for (int st = 0; st < 2; st++)
            if (pending & (1u << st)) mbar_wait(&s_bar[st], (phase_bits >> st) & 1u);
    }
}

__global__ void copy_pairs_kernel(const uint64_t* __restrict__ ki, const uint32_t* __restrict__ vi,
                                  uint64_t* __restrict__ ko, uint32_t* __restrict__ vo, int n)
{
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        ko[i] = ki[i];
        vo[i] = vi[i];
    }
}

// sort.cu:9-24 computes the position of the highest set bit plus one
inline int bit_length(uint32_t v) { int b = 0; while (v) { b++; v >>= 1; } return b; }

int g_debug_skip_publish_part = -1;

} // namespace
} // namespace fgs

#ifdef FGS_SORT_TIMING
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
// `events`, when given, receives passes + 2 recorded events: before the histogram kernel, after it,
// and after every onesweep pass; `passes_out` receives the pass count.
static int sort_pairs_impl(int num_rendered, int width, int height, int block_x, int block_y,
                           void* temp, size_t temp_bytes,
                           const uint64_t* keys_unsorted, const uint32_t* values_unsorted,
                           uint64_t* keys_sorted, uint32_t* values_sorted, void* stream,
                           cudaEvent_t* events, int* passes_out)
{
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

    char* base = static_cast<char*>(temp);
    uint32_t* tickets = reinterpret_cast<uint32_t*>(base + L.tickets_off);
    uint32_t* hist = reinterpret_cast<uint32_t*>(base + L.hist_off);
    uint32_t* status_words = reinterpret_cast<uint32_t*>(base + L.status_off);
    uint64_t* alt_keys = reinterpret_cast<uint64_t*>(base + L.alt_keys_off);
    uint32_t* alt_vals = reinterpret_cast<uint32_t*>(base + L.alt_vals_off);

    static bool smem_opt_in[64];
    static int sm_count[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return FGS_ERR_CUDA;
    if (!smem_opt_in[dev]) {
        if (cudaDeviceGetAttribute(&sm_count[dev], cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sm_count[dev] <= 0)
            return FGS_ERR_CUDA;
        if (cudaFuncSetAttribute(onesweep_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SORT_SMEM_BYTES) != cudaSuccess)
            return FGS_ERR_CUDA;
        smem_opt_in[dev] = true;
    }

    const size_t clear_bytes = L.status_off + (size_t)passes * L.parts * RADIX * 4;
    if (cudaMemsetAsync(base, 0, clear_bytes, st) != cudaSuccess) return FGS_ERR_CUDA;

    if (passes_out) *passes_out = passes;
    if (events) cudaEventRecord(events[0], st);
    int hist_blocks = L.parts < 148 * 8 ? L.parts : 148 * 8;
    histogram_kernel<<<hist_blocks, HIST_THREADS, 0, st>>>(keys_unsorted, n, passes, end_bit, hist);
    if (events) cudaEventRecord(events[1], st);

    const uint64_t* src_k = keys_unsorted;
    const uint32_t* src_v = values_unsorted;
    const int resident = SORT_BLOCKS_PER_SM * sm_count[dev];   // persistent blocks
    const int grid_blocks = L.parts < resident ? L.parts : resident;
    for (int p = 0; p < passes; p++) {
        const bool to_out = ((passes - 1 - p) & 1) == 0;
        uint64_t* dst_k = to_out ? keys_sorted : alt_keys;
        uint32_t* dst_v = to_out ? values_sorted : alt_vals;
        const int shift = p * RADIX_BITS;
        const int bits = (end_bit - shift) < RADIX_BITS ? (end_bit - shift) : RADIX_BITS;
        const int use_bulk = aligned16(src_k) && aligned16(src_v);
        onesweep_kernel<<<grid_blocks, SORT_THREADS, SORT_SMEM_BYTES, st>>>(src_k, src_v, dst_k, dst_v, n, L.parts, shift,
                                                         (1u << bits) - 1u, use_bulk, tickets + p, hist + p * RADIX,
                                                         status_words + (size_t)p * L.parts * RADIX,
                                                         dev_status, g_debug_skip_publish_part);
        src_k = dst_k;
        src_v = dst_v;
        if (events) cudaEventRecord(events[2 + p], st);
    }
    return launch_status();
}
} // namespace fgs

extern "C" int fgs_sort_pairs(int num_rendered, int width, int height, int block_x, int block_y,
                              void* temp, size_t temp_bytes,
                              const uint64_t* keys_unsorted, const uint32_t* values_unsorted,
                              uint64_t* keys_sorted, uint32_t* values_sorted, void* stream)
{
    return fgs::sort_pairs_impl(num_rendered, width, height, block_x, block_y, temp, temp_bytes, keys_unsorted,
                                values_unsorted, keys_sorted, values_sorted, stream, nullptr, nullptr);
}

extern "C" int fgs_sort_pairs_profile(int num_rendered, int width, int height, int block_x, int block_y,
                                      void* temp, size_t temp_bytes,
                                      const uint64_t* keys_unsorted, const uint32_t* values_unsorted,
                                      uint64_t* keys_sorted, uint32_t* values_sorted, void* stream,
                                      float* launch_ms, int launch_ms_len, int* num_launches)
{
    using namespace fgs;
    if (!launch_ms || !num_launches || launch_ms_len < MAX_PASSES + 1) return FGS_ERR_BAD_ARG;
    cudaEvent_t ev[MAX_PASSES + 2];
    for (auto& e : ev)
        if (cudaEventCreate(&e) != cudaSuccess) return FGS_ERR_CUDA;
    int passes = 0;
    int st = sort_pairs_impl(num_rendered, width, height, block_x, block_y, temp, temp_bytes, keys_unsorted,
                             values_unsorted, keys_sorted, values_sorted, stream, ev, &passes);
    *num_launches = 0;
    if (st == FGS_OK && num_rendered > 0) {
        if (cudaStreamSynchronize(static_cast<cudaStream_t>(stream)) != cudaSuccess) st = FGS_ERR_CUDA;
        for (int i = 0; st == FGS_OK && i < passes + 1; i++)
            if (cudaEventElapsedTime(&launch_ms[i], ev[i], ev[i + 1]) != cudaSuccess) st = FGS_ERR_CUDA;
        if (st == FGS_OK) *num_launches = passes + 1;
    }
    for (auto& e : ev) cudaEventDestroy(e);
    return st;
}
