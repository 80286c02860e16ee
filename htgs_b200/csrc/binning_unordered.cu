// Unordered binning for the relaxed-precision path: per-tile lists of Gaussian indices built as a counting sort
// with atomics, without sort keys.
//
// HYBRID_BLEND on the relaxed-precision path does not depend on the order of a tile's list (the core is the set of
// the K nearest fragments, the tail a sum), so the stable radix sort of (tile, Gaussian) pairs that the exact kernels
// need (rasterization/src/hybrid_blend/fast_inference.cu: create_instances_cu + cub::DeviceRadixSort::SortPairs +
// extract_instance_ranges_cu) is replaced by
//   1. count:  every (Gaussian, tile) instance adds 1 to its tile's counter,
//   2. scan:   exclusive prefix over the tiles -> begin of every tile's list,
//   3. place:  every instance takes the next free position of its tile with an atomic and stores the Gaussian index.
// A (Gaussian, tile) instance of the Gaussian's tile box is dropped when the conservative outline of the Gaussian (the
// ellipse the blend kernels test per pixel) does not reach the tile's 8 x 8 pixel square at all: the box of a slanted or
// round outline has empty corners, and such an instance could only be staged and rejected pixel by pixel.
// Passes 1 and 3 walk the list of VISIBLE Gaussians (about one in six), 256 per block iteration, and generate the
// block's instances cooperatively (slot -> owner by binary search over the in-block prefix, as the ordered emission
// kernel does).  The order inside a tile's list is the order in which the atomics arrive: two runs of the same frame
// can differ in the last bits of the tail sums.  `htgs_set_fast_deterministic` selects the ordered binning instead.
#include "kernels.h"

namespace htgs {

namespace {

constexpr int kBinBlock = 256;

__device__ __forceinline__ uint32_t warp_inclusive_scan_u32(uint32_t v) {
    #pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const uint32_t t = __shfl_up_sync(0xffffffffu, v, o);
        if ((threadIdx.x & 31) >= o) v += t;
    }
    return v;
}

// Smallest value of the outline form q = a x^2 + b2 x y + c y^2 (x, y relative to the outline's centre) over the square
// [x0, x0 + 7] x [y0, y0 + 7]: zero if the centre lies inside, else attained on one of the four edges, where q is a
// parabola in the free coordinate.  "Accept everything" records (a = b2 = c = 0) give 0, "reject everything" records
// (centre at infinity) give NaN, which compares false.
// `slopes` = (-b2 / (2 c), -b2 / (2 a)): where the parabola along a vertical / horizontal edge has its vertex, per unit of
// the fixed coordinate (computed once per Gaussian).
__device__ __forceinline__ bool outline_reaches_tile(const float4& c0, float cc, float2 slopes, float tile_x0, float tile_y0) {
    const float a = c0.z, b2 = c0.w;
    const float x0 = tile_x0 - c0.x, x1 = x0 + 7.0f, y0 = tile_y0 - c0.y, y1 = y0 + 7.0f;
    if (x0 <= 0.0f && x1 >= 0.0f && y0 <= 0.0f && y1 >= 0.0f) return true;
    auto q = [&](float x, float y) { return x * (a * x + b2 * y) + cc * y * y; };
    auto along_y = [&](float x) { return q(x, fminf(fmaxf(slopes.x * x, y0), y1)); };   // edge x = const
    auto along_x = [&](float y) { return q(fminf(fmaxf(slopes.y * y, x0), x1), y); };   // edge y = const
    const float q_min = fminf(fminf(along_y(x0), along_y(x1)), fminf(along_x(y0), along_x(y1)));
    return q_min <= 1.001f;
}

// PLACE = false: pass 1 (ranges[tile].y counts the tile's instances).  PLACE = true: pass 3 (ranges[tile].y is the
// tile's cursor, it starts at the tile's begin and ends at its end).
template <bool PLACE>
__global__ void __launch_bounds__(kBinBlock) bin_visible_kernel(
    const uint32_t* __restrict__ visible_list, const uint32_t* __restrict__ n_touched, const ushort4* __restrict__ bounds,
    const CullRecord* __restrict__ cull, uint2* __restrict__ ranges, uint32_t* __restrict__ prims_sorted, const FrameStatus* __restrict__ status, uint32_t grid_w, uint32_t capacity)
{
    __shared__ uint32_t excl[kBinBlock + 1];
    __shared__ ushort4 box[kBinBlock];
    __shared__ uint32_t owner[kBinBlock];
    __shared__ float4 outline4[kBinBlock];
    __shared__ float outline_c[kBinBlock];
    __shared__ float2 outline_slopes[kBinBlock];
    __shared__ uint32_t warp_tot[kBinBlock / 32];
    if (status->overflow) return;   // the frame is re-run with larger buffers
    const uint32_t n_visible = status->n_visible;
    for (uint32_t first = blockIdx.x * kBinBlock; first < n_visible; first += gridDim.x * kBinBlock) {
        const uint32_t i = first + threadIdx.x;
        uint32_t cnt = 0;
        if (i < n_visible) {
            const uint32_t g = visible_list[i];
            cnt = n_touched[g];
            box[threadIdx.x] = bounds[g];
            owner[threadIdx.x] = g;
            outline4[threadIdx.x] = ldg4(reinterpret_cast<const float*>(cull + g));
            const float c_yy = __ldg(reinterpret_cast<const float*>(cull + g) + 4);
            outline_c[threadIdx.x] = c_yy;
            // a = b2 = c = 0 ("accept everything") gives 0 / 0 = NaN, which the clamps below turn into an edge end point
            outline_slopes[threadIdx.x] = make_float2(-0.5f * outline4[threadIdx.x].w / c_yy, -0.5f * outline4[threadIdx.x].w / outline4[threadIdx.x].z);
        }
        const uint32_t inc = warp_inclusive_scan_u32(cnt);
        if ((threadIdx.x & 31) == 31) warp_tot[threadIdx.x >> 5] = inc;
        __syncthreads();
        uint32_t warp_base = 0, total = 0;
        #pragma unroll
        for (int w = 0; w < kBinBlock / 32; ++w) {
            if (w < int(threadIdx.x >> 5)) warp_base += warp_tot[w];
            total += warp_tot[w];
        }
        excl[threadIdx.x] = warp_base + inc - cnt;
        if (threadIdx.x == 0) excl[kBinBlock] = total;
        __syncthreads();
        for (uint32_t j = threadIdx.x; j < total; j += kBinBlock) {
            // upper_bound(excl, j) - 1 over the 256 entries
            uint32_t lo = 0, hi = kBinBlock;
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
            const uint32_t tile_xi = uint32_t(b.x) + lx, tile_yi = uint32_t(b.z) + ly;
            if (!outline_reaches_tile(outline4[lo], outline_c[lo], outline_slopes[lo], float(tile_xi * 8), float(tile_yi * 8))) continue;
            const uint32_t tile = tile_yi * grid_w + tile_xi;
            if constexpr (PLACE) {
                const uint32_t pos = atomicAdd(&ranges[tile].y, 1u);
                if (pos < capacity) prims_sorted[pos] = owner[lo];
            } else {
                atomicAdd(&ranges[tile].y, 1u);
            }
        }
        __syncthreads();   // shared arrays are reused by the next iteration
    }
}

// Exclusive prefix over the tile counters: ranges[tile] = (begin, begin).  One block; every thread owns a run of
// consecutive tiles (sums it, takes its offset from a block scan of the 1024 run totals, writes the run).
__global__ void __launch_bounds__(1024) scan_tiles_kernel(uint2* __restrict__ ranges, uint32_t n_tiles) {
    __shared__ uint32_t warp_tot[32];
    const uint32_t per_thread = (n_tiles + 1023u) / 1024u;
    const uint32_t begin_tile = min(threadIdx.x * per_thread, n_tiles);
    const uint32_t end_tile = min(begin_tile + per_thread, n_tiles);
    uint32_t sum = 0;
    for (uint32_t t = begin_tile; t < end_tile; ++t) sum += ranges[t].y;
    const uint32_t inc = warp_inclusive_scan_u32(sum);
    if ((threadIdx.x & 31) == 31) warp_tot[threadIdx.x >> 5] = inc;
    __syncthreads();
    if (threadIdx.x < 32) {
        const uint32_t t = warp_tot[threadIdx.x];
        const uint32_t s = warp_inclusive_scan_u32(t);
        warp_tot[threadIdx.x] = s - t;
    }
    __syncthreads();
    uint32_t running = warp_tot[threadIdx.x >> 5] + (inc - sum);
    for (uint32_t t = begin_tile; t < end_tile; ++t) {
        const uint32_t c = ranges[t].y;
        ranges[t] = make_uint2(running, running);
        running += c;
    }
}

}  // namespace

cudaError_t launch_bin_unordered(const HtgsScene& scene, const FrameGeometry& geo, const PrimBuffers& prim, uint32_t* prims_sorted, uint32_t capacity,
                                 uint2* tile_ranges, FrameStatus* status, int sm_count, cudaStream_t stream, cudaEvent_t* ev, uint32_t* launches) {
    cudaError_t err = cudaMemsetAsync(tile_ranges, 0, sizeof(uint2) * size_t(geo.n_tiles), stream);
    if (err != cudaSuccess) return err;
    if (scene.n_primitives <= 0 || capacity == 0 || geo.n_tiles == 0) {
        if (ev) { cudaEventRecord(ev[0], stream); cudaEventRecord(ev[1], stream); cudaEventRecord(ev[2], stream); }
        return cudaSuccess;
    }
    const uint32_t max_blocks = (uint32_t(scene.n_primitives) + kBinBlock - 1) / kBinBlock;
    const uint32_t grid = min(max_blocks, uint32_t(sm_count) * 8u);
    bin_visible_kernel<false><<<grid, kBinBlock, 0, stream>>>(prim.visible_list, prim.n_touched, prim.bounds, prim.cull, tile_ranges, prims_sorted, status,
                                                              uint32_t(geo.grid_w), capacity);
    if (ev) cudaEventRecord(ev[0], stream);
    scan_tiles_kernel<<<1, 1024, 0, stream>>>(tile_ranges, uint32_t(geo.n_tiles));
    if (ev) cudaEventRecord(ev[1], stream);
    bin_visible_kernel<true><<<grid, kBinBlock, 0, stream>>>(prim.visible_list, prim.n_touched, prim.bounds, prim.cull, tile_ranges, prims_sorted, status,
                                                             uint32_t(geo.grid_w), capacity);
    if (ev) cudaEventRecord(ev[2], stream);
    if (launches) *launches += 3;
    return cudaGetLastError();
}

}  // namespace htgs
