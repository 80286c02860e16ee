// Binning: prefix sum of per-block instance counts, (tile, Gaussian) instance
// emission, a stable least-significant-digit radix sort of the instance keys
// and per-tile range extraction.  All kernels are hand written (no CUB).
//
// Replaces, with identical results (same key width, same stable order, same
// uint2 ranges), the reference sequence
//   cub::DeviceScan::InclusiveSum + blocking D2H copy + create_instances_cu +
//   cub::DeviceRadixSort::SortPairs + extract_instance_ranges_cu
// (rasterization/src/hybrid_blend/inference.cu:109-165, rasterization/src/shared_kernels.cu:7-95).
//
// Differences in how the work is organised:
//  * the per-Gaussian prefix sum is never materialised: the preprocess kernel leaves one
//    count per block of 256 Gaussians, one small kernel scans those, and the emission
//    kernel rebuilds the in-block offsets in shared memory;
//  * the instance count stays on the device: emission, sort and range kernels run
//    persistent grids (a multiple of the SM count) and read the count from the frame
//    status, so the frame has no host synchronisation in the middle;
//  * a Gaussian's instances are emitted by the whole block (coalesced runs), not by one thread;
//  * digits are up to 9 bits wide, so tile keys of up to 18 bits need two passes; every
//    pass stages the locally sorted tile in shared memory so that global writes are runs.
#include "kernels.h"

#include <algorithm>

namespace htgs {

FrameGeometry make_geometry(int mode, int width, int height) {
    FrameGeometry g;
    g.width = width; g.height = height;
    g.tile_w = mode_tile_w(mode); g.tile_h = mode_tile_h(mode);
    g.grid_w = (width + g.tile_w - 1) / g.tile_w;
    g.grid_h = (height + g.tile_h - 1) / g.tile_h;
    g.n_tiles = g.grid_w * g.grid_h;
    return g;
}

static int bit_length(uint32_t v) { int b = 0; while (v) { ++b; v >>= 1; } return b; }   // rasterization/include/rasterization_utils.h:3-13

SortPlan make_sort_plan(int mode, int n_tiles) {
    SortPlan p{};
    const int tile_bits = bit_length(uint32_t(n_tiles > 0 ? n_tiles - 1 : 0));
    if (mode == HTGS_MODE_ALPHA_BLEND_GLOBAL_ORDERING) { p.key_bytes = 8; p.end_bit = tile_bits + 32; }   // alpha_blend_global_ordering/inference.cu:45
    else { p.end_bit = tile_bits; p.key_bytes = tile_bits <= 16 ? 2 : 4; }                                 // hybrid_blend/inference.cu:121-129
    p.n_passes = (p.end_bit + kMaxRadixBits - 1) / kMaxRadixBits;
    int at = 0;
    for (int i = 0; i < p.n_passes; ++i) {
        const int base = p.end_bit / p.n_passes, rem = p.end_bit % p.n_passes;
        p.bits[i] = base + (i < rem ? 1 : 0);
        p.shift[i] = at;
        at += p.bits[i];
    }
    p.final_buffer = p.n_passes & 1;
    return p;
}

namespace {

constexpr int kSortThreads = 256;
constexpr int kSortItems = kSortTile / kSortThreads;   // 16
constexpr int kSortWarps = kSortThreads / 32;          // 8

__device__ __forceinline__ uint32_t warp_inclusive_scan(uint32_t v) {
    #pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const uint32_t t = __shfl_up_sync(0xffffffffu, v, o);
        if ((threadIdx.x & 31) >= o) v += t;
    }
    return v;
}

// Exclusive scan of block sums -> block offsets; publishes the instance count.  One CTA: every thread takes a run of
// consecutive values (so that the whole array is covered in ONE round: load, thread-local sums, one block scan, store)
// instead of looping over the array 1024 values at a time with four barriers per round.
constexpr int kScanThreads = 1024;
constexpr int kScanRun = 16;            // values per thread and round: 16384 block sums (4.2 M Gaussians) per round
__global__ void __launch_bounds__(kScanThreads) scan_block_sums_kernel(const uint32_t* __restrict__ block_sums, uint32_t* __restrict__ block_offsets,
                                                                     uint32_t n_blocks, uint32_t capacity, FrameStatus* status) {
    __shared__ unsigned long long warp_tot[kScanThreads / 32];
    __shared__ unsigned long long carry_s;
    if (threadIdx.x == 0) carry_s = 0ull;
    __syncthreads();
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (uint32_t base = 0; base < n_blocks; base += kScanThreads * kScanRun) {
        const uint32_t first = base + threadIdx.x * kScanRun;
        uint32_t v[kScanRun];
        unsigned long long mine = 0;
        #pragma unroll
        for (int i = 0; i < kScanRun; ++i) { v[i] = first + i < n_blocks ? block_sums[first + i] : 0u; mine += v[i]; }
        unsigned long long inc = mine;
        #pragma unroll
        for (int o = 1; o < 32; o <<= 1) { const unsigned long long t = __shfl_up_sync(0xffffffffu, inc, o); if (lane >= uint32_t(o)) inc += t; }
        if (lane == 31) warp_tot[warp] = inc;
        __syncthreads();
        if (warp == 0) {
            const unsigned long long t = warp_tot[lane];
            unsigned long long s = t;
            #pragma unroll
            for (int o = 1; o < 32; o <<= 1) { const unsigned long long u = __shfl_up_sync(0xffffffffu, s, o); if (lane >= uint32_t(o)) s += u; }
            warp_tot[lane] = s - t;
        }
        __syncthreads();
        unsigned long long running = carry_s + warp_tot[warp] + (inc - mine);
        #pragma unroll
        for (int i = 0; i < kScanRun; ++i) {
            if (first + i < n_blocks) block_offsets[first + i] = running > 0xffffffffull ? 0xffffffffu : uint32_t(running);
            running += v[i];
        }
        __syncthreads();
        if (threadIdx.x == kScanThreads - 1) carry_s = running;
        __syncthreads();
    }
    if (threadIdx.x == 0) {
        const unsigned long long total = carry_s;
        status->n_instances = total > 0xffffffffull ? 0xffffffffu : uint32_t(total);
        status->overflow = total > (unsigned long long)capacity ? 1u : 0u;
    }
}

template <typename KeyT> struct KeyOps;
template <> struct KeyOps<uint16_t> { static __device__ __forceinline__ uint16_t make(uint32_t tile, uint32_t) { return uint16_t(tile); } static __device__ __forceinline__ uint32_t tile(uint16_t k) { return k; } };
template <> struct KeyOps<uint32_t> { static __device__ __forceinline__ uint32_t make(uint32_t tile, uint32_t) { return tile; } static __device__ __forceinline__ uint32_t tile(uint32_t k) { return k; } };
template <> struct KeyOps<uint64_t> { static __device__ __forceinline__ uint64_t make(uint32_t tile, uint32_t depth_bits) { return (uint64_t(tile) << 32) | depth_bits; } static __device__ __forceinline__ uint32_t tile(uint64_t k) { return uint32_t(k >> 32); } };

// One block per 256 Gaussians (the blocks of the preprocess kernel).  The block's instances are
// written cooperatively: slot j of the block belongs to the Gaussian whose in-block exclusive
// offset is the last one <= j; inside a Gaussian the order is row-major over its tile box
// (rasterization/src/shared_kernels.cu:21-28), so the emitted stream is identical to the reference's.
template <typename KeyT>
__global__ void __launch_bounds__(kPreprocessBlock) emit_instances_kernel(
    const uint32_t* __restrict__ n_touched, const ushort4* __restrict__ bounds, const EvalRecord* __restrict__ eval,
    const uint32_t* __restrict__ block_sums, const uint32_t* __restrict__ block_offsets, KeyT* __restrict__ keys, uint32_t* __restrict__ prims,
    uint32_t n_primitives, uint32_t grid_w, uint32_t capacity, const FrameStatus* __restrict__ status)
{
    const uint32_t total = block_sums[blockIdx.x];
    if (total == 0 || status->overflow) return;   // a frame that does not fit its instance buffers is skipped by every later stage
    __shared__ uint32_t excl[kPreprocessBlock + 1];
    __shared__ ushort4 box[kPreprocessBlock];
    __shared__ uint32_t depth_bits[kPreprocessBlock];
    __shared__ uint32_t warp_tot[kPreprocessBlock / 32];
    const uint32_t first = blockIdx.x * kPreprocessBlock;
    const uint32_t idx = first + threadIdx.x;
    const uint32_t cnt = idx < n_primitives ? n_touched[idx] : 0u;
    if (cnt) {
        box[threadIdx.x] = bounds[idx];
        if constexpr (sizeof(KeyT) == 8) depth_bits[threadIdx.x] = __float_as_uint(eval[idx].mt3.w);
    }
    const uint32_t inc = warp_inclusive_scan(cnt);
    if ((threadIdx.x & 31) == 31) warp_tot[threadIdx.x >> 5] = inc;
    __syncthreads();
    uint32_t warp_base = 0;
    #pragma unroll
    for (int w = 0; w < kPreprocessBlock / 32; ++w) if (w < int(threadIdx.x >> 5)) warp_base += warp_tot[w];
    excl[threadIdx.x] = warp_base + inc - cnt;
    if (threadIdx.x == 0) excl[kPreprocessBlock] = total;
    __syncthreads();
    const uint32_t base = block_offsets[blockIdx.x];
    for (uint32_t j = threadIdx.x; j < total; j += kPreprocessBlock) {
        // upper_bound(excl, j) - 1 over the 256 entries
        uint32_t lo = 0, hi = kPreprocessBlock;
        #pragma unroll
        for (int it = 0; it < 8; ++it) {
            const uint32_t mid = (lo + hi) >> 1;
            if (excl[mid] <= j) lo = mid; else hi = mid;
        }
        const uint32_t local = j - excl[lo];
        const ushort4 b = box[lo];
        const uint32_t w = uint32_t(b.y) - uint32_t(b.x);
        const uint32_t ly = local / w;
        const uint32_t lx = local - ly * w;
        const uint32_t tile = (uint32_t(b.z) + ly) * grid_w + uint32_t(b.x) + lx;
        const uint64_t dst = uint64_t(base) + j;
        if (dst < capacity) {
            uint32_t db = 0;
            if constexpr (sizeof(KeyT) == 8) db = depth_bits[lo];
            keys[dst] = KeyOps<KeyT>::make(tile, db);
            prims[dst] = first + lo;
        }
    }
}

__device__ __forceinline__ uint32_t frame_instances(const FrameStatus* status, uint32_t capacity) {
    const uint32_t n = status->n_instances;
    return status->overflow ? 0u : (n < capacity ? n : capacity);
}

template <typename KeyT>
__device__ __forceinline__ uint32_t digit_of(KeyT k, int shift, uint32_t mask) { return uint32_t(k >> shift) & mask; }

// ---- stable LSD radix sort, one kernel per pass ("onesweep") ------------------------------------------------------------
// One kernel counts the digits of EVERY pass in a single read of the keys; then each pass is ONE scatter kernel whose sort
// blocks learn where their digits start from their predecessors through a table of published counts (decoupled look-back)
// instead of a histogram kernel and a scan kernel in front of every scatter.
//
// Scratch (zeroed once per frame): per pass a ticket counter, the digit histogram, and one 64-bit word per (sort block, digit):
// bits 62-63 = state (0 nothing yet, 1 the block's own count, 2 the count summed over the block and all its predecessors),
// bits 0-61 = the count.  A word is written with one 8-byte store, so state and count can never be seen apart.
// Blocks take their number from the pass's ticket counter when they start, so a block only ever waits for blocks that are
// already running; every wait is bounded and reports through the frame status instead of spinning forever.
constexpr unsigned long long kLookbackAggregate = 1ull << 62, kLookbackPrefix = 2ull << 62, kLookbackValue = (1ull << 62) - 1ull;
constexpr uint32_t kLookbackPolls = 1u << 20;      // about half a second of polling before a block gives up
constexpr int kLookbackBatch = 8;                 // predecessors read per step of the walk

struct SortScratch {
    uint32_t* tickets;                   // [8]
    uint32_t* digit_hist;                // [8][kMaxRadixBins]
    unsigned long long* lookback[8];     // per pass [sort_blocks_cap][1 << bits]
    size_t bytes;
};
__host__ SortScratch carve_sort_scratch(void* base, const SortPlan& plan, uint32_t sort_blocks_cap) {
    SortScratch sc{};
    unsigned char* p = static_cast<unsigned char*>(base);
    size_t off = 0;
    sc.tickets = reinterpret_cast<uint32_t*>(p + off); off += 64;
    sc.digit_hist = reinterpret_cast<uint32_t*>(p + off); off += size_t(8) * kMaxRadixBins * sizeof(uint32_t);
    for (int i = 0; i < plan.n_passes; ++i) {
        sc.lookback[i] = reinterpret_cast<unsigned long long*>(p + off);
        off += size_t(sort_blocks_cap) * (size_t(1) << plan.bits[i]) * sizeof(unsigned long long);
    }
    sc.bytes = off;
    return sc;
}

struct PassTable { int n_passes; int shift[8]; int bits[8]; };

// Digit histograms of all passes in one read of the keys.  A thread takes 16 bytes of consecutive keys per load and
// counts runs of equal digits before touching shared memory: a Gaussian's instances are neighbouring tiles, so the high
// digits of consecutive keys agree (one atomic per run) while the low digits differ (no two lanes on one counter).
template <typename KeyT>
__global__ void __launch_bounds__(256) radix_histogram_all_kernel(const KeyT* __restrict__ keys, uint32_t* __restrict__ digit_hist,
                                                                   const FrameStatus* status, uint32_t capacity, const __grid_constant__ PassTable passes) {
    constexpr uint32_t kRun = 16 / sizeof(KeyT);
    __shared__ uint32_t hist[8 * kMaxRadixBins];
    const uint32_t n = frame_instances(status, capacity);
    for (uint32_t i = threadIdx.x; i < uint32_t(passes.n_passes) * kMaxRadixBins; i += 256) hist[i] = 0;
    __syncthreads();
    const uint32_t n_runs = (n + kRun - 1) / kRun;
    for (uint32_t r = blockIdx.x * 256 + threadIdx.x; r < n_runs; r += gridDim.x * 256) {
        const uint32_t first = r * kRun;
        KeyT k[kRun];
        uint32_t count = kRun;
        if (first + kRun <= n) {
            const uint4 raw = __ldg(reinterpret_cast<const uint4*>(keys + first));      // the key buffers are 256-byte aligned
            __builtin_memcpy(k, &raw, 16);
        } else {
            count = n - first;
            #pragma unroll
            for (uint32_t i = 0; i < kRun; ++i) k[i] = i < count ? keys[first + i] : KeyT(0);
        }
        for (int p = 0; p < passes.n_passes; ++p) {
            const int shift = passes.shift[p];
            const uint32_t mask = (1u << passes.bits[p]) - 1u;
            uint32_t run_digit = uint32_t(k[0] >> shift) & mask, run_length = 1;
            #pragma unroll
            for (uint32_t i = 1; i < kRun; ++i) {
                if (i < count) {
                    const uint32_t d = uint32_t(k[i] >> shift) & mask;
                    if (d == run_digit) ++run_length;
                    else { atomicAdd(&hist[p * kMaxRadixBins + run_digit], run_length); run_digit = d; run_length = 1; }
                }
            }
            atomicAdd(&hist[p * kMaxRadixBins + run_digit], run_length);
        }
    }
    __syncthreads();
    for (uint32_t i = threadIdx.x; i < uint32_t(passes.n_passes) * kMaxRadixBins; i += 256) {
        const uint32_t v = hist[i];
        if (v) atomicAdd(&digit_hist[i], v);
    }
}

// Exclusive scan of up to 512 values held in shared memory by 256 threads (two per thread).
__device__ __forceinline__ void block_exclusive_scan_512(uint32_t* vals, uint32_t n_bins, uint32_t* warp_tot) {
    const uint32_t i0 = 2 * threadIdx.x, i1 = i0 + 1;
    const uint32_t a = i0 < n_bins ? vals[i0] : 0u, b = i1 < n_bins ? vals[i1] : 0u;
    const uint32_t s = a + b;
    const uint32_t inc = warp_inclusive_scan(s);
    if ((threadIdx.x & 31) == 31) warp_tot[threadIdx.x >> 5] = inc;
    __syncthreads();
    uint32_t warp_base = 0;
    #pragma unroll
    for (int w = 0; w < kSortWarps; ++w) if (w < int(threadIdx.x >> 5)) warp_base += warp_tot[w];
    const uint32_t excl = warp_base + inc - s;
    if (i0 < n_bins) vals[i0] = excl;
    if (i1 < n_bins) vals[i1] = excl + a;
    __syncthreads();
}

// One pass: stable scatter.  Warp w of a sort block owns the 512 consecutive keys [w*512, (w+1)*512) of the block's tile
// and visits them in 16 rounds of 32, so (warp, round, lane) order is input order.  Ranks inside a round come from per-bit
// warp ballots; per-warp digit counters in shared memory chain the rounds; a scan over warps and digits turns them into
// positions in the locally sorted tile, which is staged in shared memory and written out as runs.  Where a digit's run
// starts in the output comes from the pass's digit histogram plus what the preceding sort blocks published.
template <typename KeyT>
__global__ void __launch_bounds__(kSortThreads, 3) radix_scatter_kernel(
    const KeyT* __restrict__ keys_in, const uint32_t* __restrict__ prims_in, KeyT* __restrict__ keys_out, uint32_t* __restrict__ prims_out,
    const uint32_t* __restrict__ digit_hist, unsigned long long* lookback, uint32_t* ticket,
    FrameStatus* status, uint32_t capacity, int shift, int bits)
{
    extern __shared__ __align__(16) unsigned char smem_raw[];
    uint32_t* warp_count = reinterpret_cast<uint32_t*>(smem_raw);                 // [kSortWarps][n_bins]
    const uint32_t n_bins_layout = 1u << bits;
    uint32_t* block_excl = warp_count + kSortWarps * n_bins_layout;               // [n_bins]
    uint32_t* global_base = block_excl + n_bins_layout;                           // [n_bins]
    uint32_t* digit_base = global_base + n_bins_layout;                           // [n_bins]
    uint32_t* prims_s = digit_base + n_bins_layout;                               // [kSortTile]
    KeyT* keys_s = reinterpret_cast<KeyT*>(prims_s + kSortTile);                  // [kSortTile]
    __shared__ uint32_t warp_tot[kSortWarps];
    __shared__ uint32_t s_blk, s_failed;

    const uint32_t n = frame_instances(status, capacity);
    const uint32_t n_blocks = (n + kSortTile - 1) / kSortTile;
    const uint32_t n_bins = 1u << bits, mask = n_bins - 1;
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    // exclusive prefix of the digit totals (same for every sort block)
    for (uint32_t d = threadIdx.x; d < n_bins; d += kSortThreads) digit_base[d] = digit_hist[d];
    if (threadIdx.x == 0) s_failed = 0;
    __syncthreads();
    block_exclusive_scan_512(digit_base, n_bins, warp_tot);

    for (;;) {
        if (threadIdx.x == 0) s_blk = atomicAdd(ticket, 1u);
        for (uint32_t i = threadIdx.x; i < kSortWarps * n_bins; i += kSortThreads) warp_count[i] = 0;
        __syncthreads();
        const uint32_t blk = s_blk;
        if (blk >= n_blocks) break;
        const uint32_t base = blk * kSortTile + warp * (kSortItems * 32);
        KeyT key[kSortItems];
        uint32_t prim[kSortItems];
        uint32_t rank[kSortItems];
        #pragma unroll
        for (int r = 0; r < kSortItems; ++r) {
            const uint32_t idx = base + r * 32 + lane;
            if (idx < n) { key[r] = keys_in[idx]; prim[r] = prims_in[idx]; }
            else { key[r] = KeyT(0); prim[r] = 0; }
        }
        uint32_t* my_count = warp_count + warp * n_bins;
        #pragma unroll
        for (int r = 0; r < kSortItems; ++r) {
            const uint32_t idx = base + r * 32 + lane;
            const bool valid = idx < n;
            const uint32_t valid_mask = __ballot_sync(0xffffffffu, valid);
            rank[r] = 0;
            // lanes holding the same digit: one ballot per digit bit (fixed cost; the hardware match instruction was measured
            // slower here: 122 / 97 us per pass instead of 85 / 72 us at 7.8 M keys)
            const uint32_t d = valid ? digit_of(key[r], shift, mask) : 0u;
            uint32_t peers = valid_mask;
            for (int b = 0; b < bits; ++b) {
                const bool bit = (d >> b) & 1u;
                const uint32_t bal = __ballot_sync(0xffffffffu, bit);
                peers &= bit ? bal : ~bal;
            }
            if (valid) {
                const int leader = __ffs(peers) - 1;
                uint32_t old = 0;
                if (int(lane) == leader) { old = my_count[d]; my_count[d] = old + __popc(peers); }
                old = __shfl_sync(peers, old, leader);
                rank[r] = old + __popc(peers & lanemask_lt());
            }
            __syncwarp();
        }
        __syncthreads();
        // per digit: exclusive prefix over warps, the block's count; publish it and look back for where the digit's run starts
        for (uint32_t d = threadIdx.x; d < n_bins; d += kSortThreads) {
            uint32_t running = 0;
            #pragma unroll
            for (int w = 0; w < kSortWarps; ++w) { const uint32_t t = warp_count[w * n_bins + d]; warp_count[w * n_bins + d] = running; running += t; }
            block_excl[d] = running;
            volatile unsigned long long* mine = lookback + size_t(blk) * n_bins + d;
            unsigned long long before = 0;          // instances with this digit in the preceding sort blocks
            if (blk == 0) {
                *mine = kLookbackPrefix | running;
            } else {
                *mine = kLookbackAggregate | running;
                // Walk back over the predecessors, kLookbackBatch words per step: the loads of a step are independent, so a
                // long walk (the blocks of the first wave all start together and find no summed count nearby) costs one
                // memory round trip per batch instead of one per predecessor.
                uint32_t polls = 0;
                bool done = false;
                for (uint32_t p = blk; p > 0 && !done;) {
                    const uint32_t step = min(uint32_t(kLookbackBatch), p);
                    unsigned long long v[kLookbackBatch];
                    #pragma unroll
                    for (uint32_t i = 0; i < kLookbackBatch; ++i) {
                        volatile const unsigned long long* theirs = lookback + size_t(p - 1u - (i < step ? i : 0u)) * n_bins + d;
                        v[i] = *theirs;
                    }
                    #pragma unroll
                    for (uint32_t i = 0; i < kLookbackBatch; ++i) {
                        if (done || i >= step) continue;
                        unsigned long long x = v[i];
                        if ((x >> 62) == 0ull) {
                            volatile const unsigned long long* theirs = lookback + size_t(p - 1u - i) * n_bins + d;
                            while ((x >> 62) == 0ull && ++polls < kLookbackPolls) x = *theirs;
                            if ((x >> 62) == 0ull) { s_failed = 1; done = true; continue; }     // gave up: report, never spin forever
                        }
                        before += x & kLookbackValue;
                        if (x & kLookbackPrefix) done = true;
                    }
                    p -= step;
                }
                *mine = kLookbackPrefix | ((before + running) & kLookbackValue);
            }
            global_base[d] = digit_base[d] + uint32_t(before);
        }
        __syncthreads();
        block_exclusive_scan_512(block_excl, n_bins, warp_tot);
        const bool failed = s_failed != 0;
        // local stable placement
        #pragma unroll
        for (int r = 0; r < kSortItems; ++r) {
            const uint32_t idx = base + r * 32 + lane;
            if (idx < n) {
                const uint32_t d = digit_of(key[r], shift, mask);
                const uint32_t lp = block_excl[d] + my_count[d] + rank[r];
                keys_s[lp] = key[r];
                prims_s[lp] = prim[r];
            }
        }
        __syncthreads();
        const uint32_t in_block = min(uint32_t(kSortTile), n - blk * kSortTile);
        if (!failed) {
            #pragma unroll
            for (int i = 0; i < kSortItems; ++i) {
                const uint32_t j = i * kSortThreads + threadIdx.x;
                if (j < in_block) {
                    const KeyT k = keys_s[j];
                    const uint32_t d = digit_of(k, shift, mask);
                    const uint32_t dst = global_base[d] + (j - block_excl[d]);
                    keys_out[dst] = k;
                    prims_out[dst] = prims_s[j];
                }
            }
        }
        __syncthreads();
    }
    if (threadIdx.x == 0 && s_failed) atomicOr(&status->error, 2u);
}

template <typename KeyT> constexpr size_t scatter_smem_bytes(int bits = kMaxRadixBits) {
    return (size_t(kSortWarps + 3) * (size_t(1) << bits) + kSortTile) * sizeof(uint32_t) + size_t(kSortTile) * sizeof(KeyT);
}

// Tile ranges from the sorted keys (rasterization/src/shared_kernels.cu:56-95); ranges were zeroed before.
// A thread takes kRangeRun consecutive keys with one 16-byte load (plus the key in front of them), so the sorted keys
// are read once, in full sectors, and a thread has all its loads in flight before its first comparison.
template <typename KeyT>
__global__ void __launch_bounds__(256) tile_ranges_kernel(const KeyT* __restrict__ keys, uint2* __restrict__ ranges, const FrameStatus* status, uint32_t capacity) {
    constexpr uint32_t kRangeRun = 16 / sizeof(KeyT);            // 8 / 4 / 2 keys per 16-byte load
    const uint32_t n = frame_instances(status, capacity);
    const uint32_t n_runs = (n + kRangeRun - 1) / kRangeRun;
    for (uint32_t r = blockIdx.x * blockDim.x + threadIdx.x; r < n_runs; r += gridDim.x * blockDim.x) {
        const uint32_t first = r * kRangeRun;
        KeyT k[kRangeRun];
        if (first + kRangeRun <= n) {
            const uint4 raw = __ldg(reinterpret_cast<const uint4*>(keys + first));      // the key buffers are 256-byte aligned
            __builtin_memcpy(k, &raw, 16);
        } else {
            #pragma unroll
            for (uint32_t i = 0; i < kRangeRun; ++i) k[i] = first + i < n ? keys[first + i] : KeyT(0);
        }
        uint32_t prev = first ? KeyOps<KeyT>::tile(keys[first - 1]) : 0xffffffffu;
        #pragma unroll
        for (uint32_t i = 0; i < kRangeRun; ++i) {
            const uint32_t at = first + i;
            if (at < n) {
                const uint32_t tile = KeyOps<KeyT>::tile(k[i]);
                if (at == 0) ranges[tile].x = 0;
                else if (prev != tile) { ranges[prev].y = at; ranges[tile].x = at; }
                if (at == n - 1) ranges[tile].y = n;
                prev = tile;
            }
        }
    }
}

template <typename KeyT>
cudaError_t emit_sort_ranges_t(const HtgsScene& scene, const FrameGeometry& geo, const SortPlan& plan, const PrimBuffers& prim, const InstBuffers& inst,
                               uint2* tile_ranges, FrameStatus* status, int sm_count, cudaStream_t stream, cudaEvent_t* ev, uint32_t* launches) {
    const uint32_t n = uint32_t(scene.n_primitives);
    const uint32_t prim_blocks = (n + kPreprocessBlock - 1) / kPreprocessBlock;
    cudaError_t err = cudaMemsetAsync(tile_ranges, 0, sizeof(uint2) * size_t(geo.n_tiles), stream);
    if (err != cudaSuccess) return err;
    if (prim_blocks == 0 || inst.capacity == 0) {
        if (ev) { cudaEventRecord(ev[0], stream); cudaEventRecord(ev[1], stream); cudaEventRecord(ev[2], stream); }
        return cudaSuccess;
    }
    emit_instances_kernel<KeyT><<<prim_blocks, kPreprocessBlock, 0, stream>>>(
        prim.n_touched, prim.bounds, prim.eval, prim.block_sums, prim.block_offsets, static_cast<KeyT*>(inst.keys[0]), inst.prims[0], n,
        uint32_t(geo.grid_w), inst.capacity, status);
    if (ev) cudaEventRecord(ev[0], stream);
    if (launches) *launches += 1;
    const uint32_t persistent = uint32_t(sm_count) * 4;
    static PerDeviceOnce configured;
    err = configured.run([] { return cudaFuncSetAttribute(radix_scatter_kernel<KeyT>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(scatter_smem_bytes<KeyT>())); });
    if (err != cudaSuccess) return err;
    int cur = 0;
    if (plan.n_passes > 0) {
        const SortScratch sc = carve_sort_scratch(inst.sort_scratch, plan, inst.sort_blocks_cap);
        if ((err = cudaMemsetAsync(inst.sort_scratch, 0, sc.bytes, stream)) != cudaSuccess) return err;
        PassTable passes{};
        passes.n_passes = plan.n_passes;
        for (int p = 0; p < plan.n_passes; ++p) { passes.shift[p] = plan.shift[p]; passes.bits[p] = plan.bits[p]; }
        const uint32_t hist_grid = std::min<uint32_t>(inst.sort_blocks_cap ? inst.sort_blocks_cap : 1u, uint32_t(sm_count) * 8u);
        radix_histogram_all_kernel<KeyT><<<hist_grid, 256, 0, stream>>>(static_cast<const KeyT*>(inst.keys[0]), sc.digit_hist, status, inst.capacity, passes);
        if (launches) *launches += 1;
        for (int p = 0; p < plan.n_passes; ++p) {
            KeyT* kin = static_cast<KeyT*>(inst.keys[cur]);
            KeyT* kout = static_cast<KeyT*>(inst.keys[cur ^ 1]);
            const size_t smem = scatter_smem_bytes<KeyT>(plan.bits[p]);
            const uint32_t resident = uint32_t(std::min<size_t>(3, (227 * 1024) / (smem + 1024)));   // scatter blocks one SM holds (3 by registers)
            const uint32_t scatter_grid = std::min<uint32_t>(inst.sort_blocks_cap ? inst.sort_blocks_cap : 1u, uint32_t(sm_count) * resident);
            radix_scatter_kernel<KeyT><<<scatter_grid, kSortThreads, smem, stream>>>(
                kin, inst.prims[cur], kout, inst.prims[cur ^ 1], sc.digit_hist + size_t(p) * kMaxRadixBins, sc.lookback[p], sc.tickets + p, status,
                inst.capacity, plan.shift[p], plan.bits[p]);
            cur ^= 1;
            if (launches) *launches += 1;
        }
    }
    if (ev) cudaEventRecord(ev[1], stream);
    tile_ranges_kernel<KeyT><<<persistent, 256, 0, stream>>>(static_cast<const KeyT*>(inst.keys[cur]), tile_ranges, status, inst.capacity);
    if (ev) cudaEventRecord(ev[2], stream);
    if (launches) *launches += 1;
    return cudaGetLastError();
}

}  // namespace

size_t sort_scratch_bytes(const SortPlan& plan, uint32_t sort_blocks_cap) { return carve_sort_scratch(nullptr, plan, sort_blocks_cap).bytes; }

cudaError_t launch_scan_only(const HtgsScene& scene, const PrimBuffers& prim, uint32_t capacity, FrameStatus* status, cudaStream_t stream) {
    const uint32_t n = uint32_t(scene.n_primitives);
    const uint32_t prim_blocks = (n + kPreprocessBlock - 1) / kPreprocessBlock;
    scan_block_sums_kernel<<<1, kScanThreads, 0, stream>>>(prim.block_sums, prim.block_offsets, prim_blocks, capacity, status);
    return cudaGetLastError();
}

cudaError_t launch_emit_sort_ranges(int mode, const HtgsScene& scene, const FrameGeometry& geo, const SortPlan& plan, const PrimBuffers& prim,
                                    const InstBuffers& inst, uint2* tile_ranges, FrameStatus* status, int sm_count, cudaStream_t stream,
                                    cudaEvent_t* stage_events, uint32_t* launches) {
    (void)mode;
    switch (plan.key_bytes) {
        case 2: return emit_sort_ranges_t<uint16_t>(scene, geo, plan, prim, inst, tile_ranges, status, sm_count, stream, stage_events, launches);
        case 4: return emit_sort_ranges_t<uint32_t>(scene, geo, plan, prim, inst, tile_ranges, status, sm_count, stream, stage_events, launches);
        case 8: return emit_sort_ranges_t<uint64_t>(scene, geo, plan, prim, inst, tile_ranges, status, sm_count, stream, stage_events, launches);
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace htgs
