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

// Exclusive scan of block sums -> block offsets; publishes the instance count.
__global__ void __launch_bounds__(1024) scan_block_sums_kernel(const uint32_t* __restrict__ block_sums, uint32_t* __restrict__ block_offsets,
                                                               uint32_t n_blocks, uint32_t capacity, FrameStatus* status) {
    __shared__ uint32_t warp_tot[32];
    __shared__ unsigned long long carry_s;
    if (threadIdx.x == 0) carry_s = 0ull;
    __syncthreads();
    for (uint32_t base = 0; base < n_blocks; base += 1024) {
        const uint32_t i = base + threadIdx.x;
        const uint32_t v = i < n_blocks ? block_sums[i] : 0u;
        const uint32_t inc = warp_inclusive_scan(v);
        if ((threadIdx.x & 31) == 31) warp_tot[threadIdx.x >> 5] = inc;
        __syncthreads();
        if (threadIdx.x < 32) {
            const uint32_t t = warp_tot[threadIdx.x];
            const uint32_t s = warp_inclusive_scan(t);
            warp_tot[threadIdx.x] = s - t;
        }
        __syncthreads();
        const unsigned long long carry = carry_s;
        const unsigned long long excl = carry + warp_tot[threadIdx.x >> 5] + (inc - v);
        if (i < n_blocks) block_offsets[i] = excl > 0xffffffffull ? 0xffffffffu : uint32_t(excl);
        __syncthreads();
        if (threadIdx.x == 1023) carry_s = excl + v;
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

// Pass step 1: per-sort-block digit histograms -> table[digit][block].
template <typename KeyT>
__global__ void __launch_bounds__(kSortThreads) radix_histogram_kernel(const KeyT* __restrict__ keys, uint32_t* __restrict__ table, uint32_t table_stride,
                                                                       const FrameStatus* status, uint32_t capacity, int shift, int bits) {
    __shared__ uint32_t hist[kMaxRadixBins];
    const uint32_t n = frame_instances(status, capacity);
    const uint32_t n_blocks = (n + kSortTile - 1) / kSortTile;
    const uint32_t n_bins = 1u << bits, mask = n_bins - 1;
    for (uint32_t blk = blockIdx.x; blk < n_blocks; blk += gridDim.x) {
        for (uint32_t d = threadIdx.x; d < n_bins; d += kSortThreads) hist[d] = 0;
        __syncthreads();
        const uint32_t base = blk * kSortTile;
        #pragma unroll
        for (int i = 0; i < kSortItems; ++i) {
            const uint32_t idx = base + i * kSortThreads + threadIdx.x;
            if (idx < n) atomicAdd(&hist[digit_of(keys[idx], shift, mask)], 1u);
        }
        __syncthreads();
        for (uint32_t d = threadIdx.x; d < n_bins; d += kSortThreads) table[size_t(d) * table_stride + blk] = hist[d];
        __syncthreads();
    }
}

// Pass step 2: one block per digit scans its row of the table in place (exclusive) and stores the digit total.
__global__ void __launch_bounds__(kSortThreads) radix_scan_rows_kernel(uint32_t* __restrict__ table, uint32_t table_stride, uint32_t* __restrict__ digit_totals,
                                                                       const FrameStatus* status, uint32_t capacity) {
    __shared__ uint32_t warp_tot[kSortWarps];
    __shared__ uint32_t carry_s;
    const uint32_t n = frame_instances(status, capacity);
    const uint32_t n_blocks = (n + kSortTile - 1) / kSortTile;
    uint32_t* row = table + size_t(blockIdx.x) * table_stride;
    if (threadIdx.x == 0) carry_s = 0;
    __syncthreads();
    for (uint32_t base = 0; base < n_blocks; base += kSortThreads) {
        const uint32_t i = base + threadIdx.x;
        const uint32_t v = i < n_blocks ? row[i] : 0u;
        const uint32_t inc = warp_inclusive_scan(v);
        if ((threadIdx.x & 31) == 31) warp_tot[threadIdx.x >> 5] = inc;
        __syncthreads();
        uint32_t warp_base = 0;
        #pragma unroll
        for (int w = 0; w < kSortWarps; ++w) if (w < int(threadIdx.x >> 5)) warp_base += warp_tot[w];
        const uint32_t carry = carry_s;
        const uint32_t excl = carry + warp_base + inc - v;
        if (i < n_blocks) row[i] = excl;
        __syncthreads();
        if (threadIdx.x == kSortThreads - 1) carry_s = excl + v;
        __syncthreads();
    }
    if (threadIdx.x == 0) digit_totals[blockIdx.x] = carry_s;
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

// Pass step 3: stable scatter.  Warp w of a sort block owns the 512 consecutive keys
// [w*512, (w+1)*512) of the block's tile and visits them in 16 rounds of 32, so (warp, round, lane)
// order is input order.  Ranks inside a round come from per-bit warp ballots; per-warp digit counters
// in shared memory chain the rounds; a scan over warps and digits turns them into positions in the
// locally sorted tile, which is staged in shared memory and written out as runs.
template <typename KeyT>
__global__ void __launch_bounds__(kSortThreads, 3) radix_scatter_kernel(
    const KeyT* __restrict__ keys_in, const uint32_t* __restrict__ prims_in, KeyT* __restrict__ keys_out, uint32_t* __restrict__ prims_out,
    const uint32_t* __restrict__ table, uint32_t table_stride, const uint32_t* __restrict__ digit_totals,
    const FrameStatus* status, uint32_t capacity, int shift, int bits)
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

    const uint32_t n = frame_instances(status, capacity);
    const uint32_t n_blocks = (n + kSortTile - 1) / kSortTile;
    const uint32_t n_bins = 1u << bits, mask = n_bins - 1;
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    // exclusive prefix of the digit totals (same for every sort block)
    for (uint32_t d = threadIdx.x; d < n_bins; d += kSortThreads) digit_base[d] = digit_totals[d];
    __syncthreads();
    block_exclusive_scan_512(digit_base, n_bins, warp_tot);

    for (uint32_t blk = blockIdx.x; blk < n_blocks; blk += gridDim.x) {
        for (uint32_t i = threadIdx.x; i < kSortWarps * n_bins; i += kSortThreads) warp_count[i] = 0;
        __syncthreads();
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
            // lanes holding the same digit: one ballot per digit bit (fixed cost; a hardware match over 32 mostly
            // distinct tile digits is slower)
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
        // per digit: exclusive prefix over warps, block count
        for (uint32_t d = threadIdx.x; d < n_bins; d += kSortThreads) {
            uint32_t running = 0;
            #pragma unroll
            for (int w = 0; w < kSortWarps; ++w) { const uint32_t t = warp_count[w * n_bins + d]; warp_count[w * n_bins + d] = running; running += t; }
            block_excl[d] = running;
        }
        __syncthreads();
        block_exclusive_scan_512(block_excl, n_bins, warp_tot);
        for (uint32_t d = threadIdx.x; d < n_bins; d += kSortThreads)
            global_base[d] = digit_base[d] + table[size_t(d) * table_stride + blk] - block_excl[d];
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
        #pragma unroll
        for (int i = 0; i < kSortItems; ++i) {
            const uint32_t j = i * kSortThreads + threadIdx.x;
            if (j < in_block) {
                const KeyT k = keys_s[j];
                const uint32_t dst = global_base[digit_of(k, shift, mask)] + j;
                keys_out[dst] = k;
                prims_out[dst] = prims_s[j];
            }
        }
        __syncthreads();
    }
}

template <typename KeyT> constexpr size_t scatter_smem_bytes(int bits = kMaxRadixBits) {
    return (size_t(kSortWarps + 3) * (size_t(1) << bits) + kSortTile) * sizeof(uint32_t) + size_t(kSortTile) * sizeof(KeyT);
}

// Tile ranges from the sorted keys (rasterization/src/shared_kernels.cu:56-95); ranges were zeroed before.
template <typename KeyT>
__global__ void __launch_bounds__(256) tile_ranges_kernel(const KeyT* __restrict__ keys, uint2* __restrict__ ranges, const FrameStatus* status, uint32_t capacity) {
    const uint32_t n = frame_instances(status, capacity);
    for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
        const uint32_t tile = KeyOps<KeyT>::tile(keys[i]);
        if (i == 0) ranges[tile].x = 0;
        else {
            const uint32_t prev = KeyOps<KeyT>::tile(keys[i - 1]);
            if (prev != tile) { ranges[prev].y = i; ranges[tile].x = i; }
        }
        if (i == n - 1) ranges[tile].y = n;
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
    for (int p = 0; p < plan.n_passes; ++p) {
        KeyT* kin = static_cast<KeyT*>(inst.keys[cur]);
        KeyT* kout = static_cast<KeyT*>(inst.keys[cur ^ 1]);
        const size_t smem = scatter_smem_bytes<KeyT>(plan.bits[p]);
        const uint32_t resident = uint32_t(std::min<size_t>(3, (227 * 1024) / (smem + 1024)));   // scatter blocks one SM holds (3 by registers)
        const uint32_t scatter_grid = std::min<uint32_t>(inst.sort_blocks_cap ? inst.sort_blocks_cap : 1u, uint32_t(sm_count) * resident);
        const uint32_t hist_grid = std::min<uint32_t>(inst.sort_blocks_cap ? inst.sort_blocks_cap : 1u, uint32_t(sm_count) * 16u);
        radix_histogram_kernel<KeyT><<<hist_grid, kSortThreads, 0, stream>>>(kin, inst.radix_table, inst.sort_blocks_cap, status, inst.capacity, plan.shift[p], plan.bits[p]);
        radix_scan_rows_kernel<<<1u << plan.bits[p], kSortThreads, 0, stream>>>(inst.radix_table, inst.sort_blocks_cap, inst.digit_totals, status, inst.capacity);
        radix_scatter_kernel<KeyT><<<scatter_grid, kSortThreads, smem, stream>>>(
            kin, inst.prims[cur], kout, inst.prims[cur ^ 1], inst.radix_table, inst.sort_blocks_cap, inst.digit_totals, status, inst.capacity,
            plan.shift[p], plan.bits[p]);
        cur ^= 1;
        if (launches) *launches += 3;
    }
    if (ev) cudaEventRecord(ev[1], stream);
    tile_ranges_kernel<KeyT><<<persistent, 256, 0, stream>>>(static_cast<const KeyT*>(inst.keys[cur]), tile_ranges, status, inst.capacity);
    if (ev) cudaEventRecord(ev[2], stream);
    if (launches) *launches += 1;
    return cudaGetLastError();
}

}  // namespace

cudaError_t launch_scan_only(const HtgsScene& scene, const PrimBuffers& prim, uint32_t capacity, FrameStatus* status, cudaStream_t stream) {
    const uint32_t n = uint32_t(scene.n_primitives);
    const uint32_t prim_blocks = (n + kPreprocessBlock - 1) / kPreprocessBlock;
    scan_block_sums_kernel<<<1, 1024, 0, stream>>>(prim.block_sums, prim.block_offsets, prim_blocks, capacity, status);
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
