// Host-side launch interface between the C-ABI layer (api.cu) and the kernel
// translation units.  Plain pointers only.
#pragma once

#include "common.cuh"

#include <atomic>
#include <mutex>

namespace htgs {

// One-time, per-device set-up of a kernel instantiation (its dynamic shared-memory limit), safe when several host
// threads, each with its own context, launch the same kernel at once.  A set-up that fails is retried by the next call.
struct PerDeviceOnce {
    std::mutex mutex;
    std::atomic<bool> done[64] = {};
    template <typename F> cudaError_t run(F&& setup) {
        int device = 0;
        cudaGetDevice(&device);
        if (device < 0 || device >= 64) return setup();
        if (done[device].load(std::memory_order_acquire)) return cudaSuccess;
        std::lock_guard<std::mutex> lock(mutex);
        if (done[device].load(std::memory_order_relaxed)) return cudaSuccess;
        const cudaError_t err = setup();
        if (err == cudaSuccess) done[device].store(true, std::memory_order_release);
        return err;
    }
};

struct PrimBuffers {
    uint32_t* n_touched;      // [N]
    ushort4* bounds;          // [N] x_min,x_max,y_min,y_max in tiles
    EvalRecord* eval;         // [N]
    CullRecord* cull;         // [N]
    uint8_t* clamp;           // [N] bit c set: colour channel c was clamped at 0 (training only, else null)
    uint32_t* block_sums;     // [ceil(N/256)] instances emitted by each block of 256 Gaussians
    uint32_t* block_offsets;  // [ceil(N/256)] exclusive prefix of block_sums
    uint32_t* visible_list;   // [N] indices of the Gaussians that survived culling (first n_visible entries, unordered)
};

struct InstBuffers {
    void* keys[2];            // ping-pong key buffers, `key_bytes` wide
    uint32_t* prims[2];       // ping-pong Gaussian indices
    void* sort_scratch;       // ticket counters, digit histograms and look-back words of the radix passes (sort_scratch_bytes)
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
size_t sort_scratch_bytes(const SortPlan& plan, uint32_t sort_blocks_cap);   // binning.cu

struct FrameGeometry {
    int width, height, grid_w, grid_h, n_tiles, tile_w, tile_h;
};
FrameGeometry make_geometry(int mode, int width, int height);

// preprocess.cu
// `fast_records`: write FastRecord instead of EvalRecord (inference of the modes launch_blend_fast supports).
cudaError_t launch_preprocess(int mode, bool train, const HtgsScene& scene, const HtgsView& view, const FrameGeometry& geo,
                              const PrimBuffers& prim, FrameStatus* status, cudaStream_t stream, bool fast_records = false);

// binning.cu: scan of block sums, instance emission, stable radix sort, tile ranges.
// Everything after the scan reads the instance count from `status` on the device.
cudaError_t launch_scan_only(const HtgsScene& scene, const PrimBuffers& prim, uint32_t capacity, FrameStatus* status, cudaStream_t stream);
// `stage_events` (optional): events recorded after emission, after the sort and after the range kernel.
cudaError_t launch_emit_sort_ranges(int mode, const HtgsScene& scene, const FrameGeometry& geo, const SortPlan& plan, const PrimBuffers& prim,
                                    const InstBuffers& inst, uint2* tile_ranges, FrameStatus* status, int sm_count, cudaStream_t stream,
                                    cudaEvent_t* stage_events = nullptr, uint32_t* launches = nullptr);

// binning_unordered.cu: per-tile lists without sort keys (counting sort with atomics; the order inside a list is not
// defined).  Writes `tile_ranges` and `prims_sorted`; expects `status->n_instances / overflow` from launch_scan_only.
// `stage_events` (optional): events recorded after the count pass, the tile scan and the placement pass.
cudaError_t launch_bin_unordered(const HtgsScene& scene, const FrameGeometry& geo, const PrimBuffers& prim, uint32_t* prims_sorted, uint32_t capacity,
                                 uint2* tile_ranges, FrameStatus* status, int sm_count, cudaStream_t stream, cudaEvent_t* stage_events = nullptr,
                                 uint32_t* launches = nullptr);

// blend.cu
struct BlendOutputs {
    float* image;
    float* depth;
    float* alpha;     // may be null
    bool to_chw;
    bool use_median_depth;
    bool collect_stats;
};
// per-pixel buffers the training forward leaves for the backward pass; pixel slots are tile-major
// (slot = tile * pixels_per_tile + pixel_in_tile) and every array is plane-major over `padded_pixels` slots
struct TrainPixelBuffers {
    uint32_t* idx_core;      // [K][padded_pixels] per core entry the position of its Gaussian in the tile's sorted list, 0xffffffff = none (HYBRID, FIRST_K)
    float4* info_core;       // [K][padded_pixels] (dC/dalpha factors, blending weight)                 (HYBRID, FIRST_K)
    float* info_tail;        // [6][padded_pixels] HYBRID tail terms / [5][padded_pixels] OIT terms
    uint32_t padded_pixels;  // n_tiles * pixels_per_tile
};

int effective_k(int mode, int K);
cudaError_t launch_blend(int mode, int K, bool train, const FrameGeometry& geo, const PrimBuffers& prim, const uint32_t* prims_sorted,
                         const uint2* tile_ranges, const BlendOutputs& out, const TrainPixelBuffers& tout, FrameStatus* status, cudaStream_t stream);

// blend_fast.cu: relaxed-precision inference (RGB only) for HYBRID_BLEND, ALPHA_BLEND_FIRST_K and OIT_BLEND.  `supports` tells
// whether (mode, K) has a fast kernel; these kernels do not depend on the order of a tile's list.
bool blend_fast_supports(int mode, int K);
cudaError_t launch_blend_fast(int mode, int K, const FrameGeometry& geo, const PrimBuffers& prim, const uint32_t* prims_sorted, const uint2* tile_ranges,
                              float* image, bool to_chw, FrameStatus* status, cudaStream_t stream);

// weights.cu
// `credit_tail` (HYBRID_BLEND only): also run the second walk that credits `alpha * tail weight` to every fragment.
cudaError_t launch_max_weights(int mode, int K, const FrameGeometry& geo, const PrimBuffers& prim, const uint32_t* prims_sorted, const uint2* tile_ranges,
                               float* max_weights, float weight_threshold, bool credit_tail, cudaStream_t stream);

// train.cu: backward pass
struct GradAccumBuffers {
    float4* accum;           // [N][5] float4: dL/dVPMT1, dL/dVPMT2, dL/dVPMT4, (dL/drgb, dL/dopacity), (sum |dL/dposition|, 0, 0, 0)
};
constexpr int kBackwardAccumulate = 1, kBackwardChainRule = 2;
struct BackwardOutputs {
    float* grad_positions; float* grad_scales; float* grad_rotations; float* grad_opacities; float* grad_sh_0; float* grad_sh_rest;
    float* densification_info;   // [rows][N] or null
    int densification_rows;      // 0, 2 or 3
    bool use_distance_scaling;
    float4* compact_rows = nullptr;       // when set: header + compact rows (common.cuh) are written INSTEAD of the six tensors
    uint32_t compact_capacity = 0;        // rows the buffer holds behind its header
};
cudaError_t launch_visibility(const uint32_t* n_touched, uint8_t* visible, uint32_t n, cudaStream_t stream);
cudaError_t launch_backward(int mode, int K, const HtgsScene& scene, const HtgsView& view, const FrameGeometry& geo, const PrimBuffers& prim,
                            const uint32_t* prims_sorted, const uint2* tile_ranges, const TrainPixelBuffers& tin, const float* grad_image,
                            const float* image, const GradAccumBuffers& acc, const BackwardOutputs& out, cudaEvent_t outputs_cleared, int sm_count,
                            uint32_t first, uint32_t count, int stages, cudaStream_t stream);
// `stages`: kBackwardAccumulate = the per-tile (per-pixel for GLOBAL_ORDERING) pass that accumulates one record per Gaussian,
// kBackwardChainRule = the per-Gaussian kernel that turns the records into the six gradients; both for a whole backward pass.
// `outputs_cleared`: event after which rows [first, first + count) of the six tensors are zero, or null to clear them here.
// [first, first + count): the Gaussians whose gradients the call computes (everything else is left untouched); a proper part
// of the scene is refused (cudaErrorNotSupported) for GLOBAL_ORDERING.
cudaError_t clear_backward_outputs(const HtgsScene& scene, const BackwardOutputs& out, uint32_t first, uint32_t count, cudaStream_t stream);


// api.cu: internals shared with the other translation units (C++ linkage: not part of the C-ABI).
int backward_with_accum(HtgsContext* ctx, const HtgsScene* scene, const HtgsView* view, const HtgsTrainBlobs* blobs, uint32_t n_instances,
                        const float* grad_image, const float* image, const HtgsGradients* grads, void* accum, uint32_t first, uint32_t count, int stages,
                        void* stream, void* compact_rows = nullptr, uint32_t compact_capacity = 0);
// compact_rows: when not null the chain rule writes header + compact rows (common.cuh) there and leaves the six tensors alone
int context_device(const HtgsContext* ctx);
void set_last_error(const char* message);   // message htgs_last_error() returns on the calling thread

}  // namespace htgs
