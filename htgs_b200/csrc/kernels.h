// Host-side launch interface between the C-ABI layer (api.cu) and the kernel
// translation units.  Plain pointers only.
#pragma once

#include "common.cuh"

namespace htgs {

struct PrimBuffers {
    uint32_t* n_touched;      // [N]
    ushort4* bounds;          // [N] x_min,x_max,y_min,y_max in tiles
    EvalRecord* eval;         // [N]
    CullRecord* cull;         // [N]
    uint8_t* clamp;           // [N] bit c set: colour channel c was clamped at 0 (training only, else null)
    uint32_t* block_sums;     // [ceil(N/256)] instances emitted by each block of 256 Gaussians
    uint32_t* block_offsets;  // [ceil(N/256)] exclusive prefix of block_sums
};

struct InstBuffers {
    void* keys[2];            // ping-pong key buffers, `key_bytes` wide
    uint32_t* prims[2];       // ping-pong Gaussian indices
    uint32_t* radix_table;    // [n_bins_max * sort_blocks_cap]
    uint32_t* digit_totals;   // [n_bins_max]
    uint32_t capacity;        // instances the buffers can hold
    uint32_t sort_blocks_cap; // ceil(capacity / kSortTile)
};

constexpr int kPreprocessBlock = 256;
constexpr int kSortTile = 4096;        // keys per sort block (256 threads x 16)
constexpr int kMaxRadixBits = 9;
constexpr int kMaxRadixBins = 1 << kMaxRadixBits;

struct SortPlan {
    int key_bytes;     // 2, 4, 8
    int end_bit;       // bits to sort
    int n_passes;
    int bits[8];       // digit width per pass
    int shift[8];      // digit position per pass
    int final_buffer;  // which ping-pong buffer holds the sorted result
};
SortPlan make_sort_plan(int mode, int n_tiles);

struct FrameGeometry {
    int width, height, grid_w, grid_h, n_tiles, tile_w, tile_h;
};
FrameGeometry make_geometry(int mode, int width, int height);

// preprocess.cu
cudaError_t launch_preprocess(int mode, bool train, const HtgsScene& scene, const HtgsView& view, const FrameGeometry& geo,
                              const PrimBuffers& prim, FrameStatus* status, cudaStream_t stream);

// binning.cu: scan of block sums, instance emission, stable radix sort, tile ranges.
// Everything after the scan reads the instance count from `status` on the device.
cudaError_t launch_scan_only(const HtgsScene& scene, const PrimBuffers& prim, uint32_t capacity, FrameStatus* status, cudaStream_t stream);
// `stage_events` (optional): events recorded after emission, after the sort and after the range kernel.
cudaError_t launch_emit_sort_ranges(int mode, const HtgsScene& scene, const FrameGeometry& geo, const SortPlan& plan, const PrimBuffers& prim,
                                    const InstBuffers& inst, uint2* tile_ranges, FrameStatus* status, int sm_count, cudaStream_t stream,
                                    cudaEvent_t* stage_events = nullptr, uint32_t* launches = nullptr);

// blend.cu
struct BlendOutputs {
    float* image;
    float* depth;
    float* alpha;     // may be null
    bool to_chw;
    bool use_median_depth;
    bool collect_stats;
};
cudaError_t launch_blend_inference(int mode, int K, const FrameGeometry& geo, const PrimBuffers& prim, const uint32_t* prims_sorted,
                                   const uint2* tile_ranges, const BlendOutputs& out, FrameStatus* status, int sm_count, cudaStream_t stream);
cudaError_t configure_blend_kernels();

}  // namespace htgs
