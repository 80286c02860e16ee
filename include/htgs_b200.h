/*
 * htgs_b200 - C ABI of the sm_100a (B200) rasterizer core.
 *
 * Drop-in boundary for the rasterizer of nerficg-project/HTGS.  The entry points
 * below are what the reference's pybind module `HTGSCudaBackend._C` binds
 * (torch_bindings/bindings.cpp:8-16), restated with plain pointers and sizes:
 * no torch types cross this boundary.  All pointers are DEVICE pointers unless
 * a comment says "host".  File:line citations are relative to
 * HTGSCudaBackend/HTGSCudaBackend/ of the reference.
 *
 * Threading: a context is bound to one CUDA device and must not be used from
 * two host threads at once.  Calls are stream-ordered on the stream passed in
 * and re-entrant across contexts (camera matrices are read from device memory
 * by the kernels; nothing is uploaded to __constant__ memory).  An entry point
 * that takes a context makes the context's device current while it runs and
 * puts the caller's current device back before it returns.
 */
#ifndef HTGS_B200_H
#define HTGS_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* RasterizerMode (torch_bindings/rasterization.py:9-13) */
enum HtgsMode {
    HTGS_MODE_HYBRID_BLEND = 0,
    HTGS_MODE_ALPHA_BLEND_FIRST_K = 1,
    HTGS_MODE_ALPHA_BLEND_GLOBAL_ORDERING = 2,
    HTGS_MODE_OIT_BLEND = 3
};

enum HtgsStatus {
    HTGS_OK = 0,
    HTGS_ERR_INVALID_ARGUMENT = 1,
    HTGS_ERR_UNSUPPORTED_MODE = 2,   /* the reference throws "unsupported rasterizer mode" (rasterization/src/rasterization_api.cu:171-172) */
    HTGS_ERR_WORKSPACE_TOO_SMALL = 3,
    HTGS_ERR_CUDA = 4,
    HTGS_ERR_DEVICE_FLAG = 5         /* a kernel reported an internal error (e.g. a bounded wait gave up) */
};

/* The six per-Gaussian input tensors of `rasterize` / `diff_rasterize`
 * (torch_bindings/rasterization.py:140-150), contiguous float32. */
typedef struct HtgsScene {
    const float* positions;   /* [N,3] */
    const float* scales;      /* [N,3] activated */
    const float* rotations;   /* [N,4] (r,x,y,z), unit length */
    const float* opacities;   /* [N,1] activated */
    const float* sh_0;        /* [N,1,3] */
    const float* sh_rest;     /* [N,B,3]; may be NULL when B == 0 */
    int32_t n_primitives;     /* N */
    int32_t total_sh_bases;   /* B = sh_rest.size(1) */
} HtgsScene;

/* RasterizerSettings (torch_bindings/rasterization.py:16-42).  The matrices stay device
 * tensors, as in the reference, so that building a view never forces a host sync. */
typedef struct HtgsView {
    const float* M;             /* [4,4] world -> view, row-major */
    const float* VPM;           /* [4,4] world -> screen, row-major */
    const float* cam_position;  /* [3] */
    int32_t mode;               /* HtgsMode */
    int32_t K;                  /* HYBRID_BLEND / ALPHA_BLEND_FIRST_K only; rounded down to a power of two <= 32 */
    int32_t active_sh_bases;    /* 1, 4, 9 or 16 */
    int32_t width;
    int32_t height;
    float near_plane;
    float far_plane;
    float scale_modifier;       /* ignored (treated as 1) by the training forward, as in the reference */
} HtgsView;

/* Host-side summary of the last frame. */
typedef struct HtgsFrameInfo {
    uint32_t n_instances;        /* (tile, Gaussian) instances */
    uint32_t n_visible;          /* Gaussians that passed culling */
    uint32_t key_bytes;          /* 2, 4 or 8: width of the sort key used */
    uint32_t end_bit;            /* number of key bits that were sorted */
    uint32_t reruns;             /* times the frame was re-run after growing the internal workspace */
    uint32_t device_error;       /* device-side error flags (0 = none) */
    uint32_t kernel_launches;    /* kernels of this library launched for the frame (re-runs included) */
    uint32_t reserved;
    uint64_t workspace_bytes;    /* bytes a caller-provided workspace must have for this frame */
    uint64_t candidate_pairs;    /* statistics mode only: (pixel, Gaussian) pairs that passed the outline test */
    uint64_t accepted_fragments; /* statistics mode only: fragments accepted by the exact test */
    uint64_t warp_trips;           /* statistics mode, HYBRID_BLEND: warp-level evaluations of one candidate per lane */
    uint64_t warp_trips_inserting; /* ... in which at least one lane inserted into its K-buffer (the insertion chain ran) */
    uint64_t lane_insertions;      /* ... and the number of lanes that inserted */
} HtgsFrameInfo;

/* Device pointers into the workspace of the last htgs_render call of a context; valid
 * until the next call on that context.  For parity tests and profiling. */
typedef struct HtgsIntermediates {
    const uint32_t* n_touched;     /* [N] tiles touched per Gaussian (0 = culled) */
    const uint16_t* bounds;        /* [N,4] x_min,x_max,y_min,y_max in tiles (undefined where n_touched == 0) */
    const void* eval_records;      /* [N] 80-byte records: vpmt1, vpmt2, vpmt4, mt3, rgba (float4 each) */
    const void* cull_records;      /* [N] 32-byte records */
    const void* keys_unsorted;     /* [n_instances] keys in emission order (key_bytes wide) */
    const uint32_t* prims_unsorted;/* [n_instances] */
    const void* keys_sorted;       /* [n_instances] */
    const uint32_t* prims_sorted;  /* [n_instances] Gaussian index per sorted instance */
    const uint32_t* tile_ranges;   /* [n_tiles,2] begin,end into the sorted arrays; (0,0) for empty tiles */
    uint32_t n_tiles;
    uint32_t grid_width;
    uint32_t grid_height;
    uint32_t key_bytes;
} HtgsIntermediates;

typedef struct HtgsContext HtgsContext;

/* Library management.  htgs_last_error() returns the message of the last failing call of
 * the calling host thread. */
HtgsContext* htgs_create(int device);
void htgs_destroy(HtgsContext* ctx);
const char* htgs_last_error(void);
int htgs_version(void);

/* Bytes of workspace htgs_render needs for `instance_capacity` instances. */
size_t htgs_render_workspace_bytes(const HtgsScene* scene, const HtgsView* view, uint64_t instance_capacity);

/*
 * Forward render.  Replaces `_C.render` = htgs::rasterization::inference_wrapper
 * (rasterization/include/rasterization_api.h:57-77, rasterization/src/rasterization_api.cu:365-516).
 *   image: [3,H,W] if to_chw else [H,W,3], clamped to [0,1];  depth: [H,W];
 *   alpha: [H,W] or NULL.  Alpha is not an output of the reference; it is the total opacity the
 *          reference uses internally to normalise the mean depth.
 * workspace == NULL selects the context's own grow-only workspace (the frame is re-run once
 * after growing when the instance count exceeds its capacity).  With a caller workspace that is too
 * small the call returns HTGS_ERR_WORKSPACE_TOO_SMALL and info->workspace_bytes says what is needed.
 * The call synchronises `stream` once, at its end, to read the frame status.
 */
int htgs_render(HtgsContext* ctx, const HtgsScene* scene, const HtgsView* view, float* image, float* depth, float* alpha,
                int to_chw, int use_median_depth, void* workspace, size_t workspace_bytes, void* stream, HtgsFrameInfo* info);

/*
 * Forward render without a host wait.  No counterpart in the reference, which blocks in the middle of every frame to
 * read the instance count (rasterization/src/hybrid_blend/inference.cu:118-119); htgs_render still waits once, at its end.
 *
 * htgs_render_async queues the whole frame on `stream` (same arguments and results as htgs_render, always with the
 * context's own workspace) and returns at once; the 64-byte frame status lands in pinned host memory behind the frame.
 * htgs_frame_result waits for that status, checks it and fills `info`; the next call of any frame-level entry point on
 * the same context performs the same check first and reports a failure of the earlier frame as its own.  One host thread
 * keeps two frames in flight by alternating between two contexts, each with its own stream.
 *
 * What the deferred check can find: a device-side error flag, or instance buffers that were too small for the frame
 * (the context sizes them from the frames it has seen).  In the second case the check grows the workspace and renders
 * the frame again on the same stream before it returns (info->reruns > 0); work the caller queued on the stream between
 * htgs_render_async and the check has then read an image without its instances.  A caller that cannot tolerate that
 * renders each new kind of view once with htgs_render first, or checks info->reruns and repeats the dependent work.
 * The scene, view and output pointers must stay valid until the check.
 */
int htgs_render_async(HtgsContext* ctx, const HtgsScene* scene, const HtgsView* view, float* image, float* depth, float* alpha,
                      int to_chw, int use_median_depth, void* stream);
int htgs_frame_result(HtgsContext* ctx, HtgsFrameInfo* info);

/* As htgs_render with HOST buffers: inputs are copied to the device and the image/depth back inside the
 * call (used for end-to-end measurement and by callers without device memory of their own). */
int htgs_render_host(HtgsContext* ctx, const HtgsScene* host_scene, const HtgsView* host_view, float* host_image, float* host_depth,
                     int to_chw, int use_median_depth, HtgsFrameInfo* info);

int htgs_get_intermediates(HtgsContext* ctx, HtgsIntermediates* out);

/*
 * Training forward and backward.  Replace `_C.forward` / `_C.backward` = forward_wrapper / backward_wrapper
 * (rasterization/include/rasterization_api.h:8-55, rasterization/src/rasterization_api.cu:37-363).
 *
 * As in the reference, the forward leaves four opaque byte blobs for the backward (per Gaussian, per tile,
 * per instance, per pixel); the caller owns them (the Python layer allocates them with torch, exactly like
 * the reference's resizable byte tensors).  Three sizes are known up front, the per-instance one only after
 * the instance count is: htgs_forward_begin runs preprocess + prefix sum and returns the count (one host
 * synchronisation, as in the reference), htgs_forward_finish runs the rest.
 *   image: [3,H,W], NOT clamped; scale_modifier is ignored (1), as in the reference's training forward.
 */
typedef struct HtgsTrainBlobs {
    void* per_primitive; size_t per_primitive_bytes;
    void* per_tile;      size_t per_tile_bytes;
    void* per_instance;  size_t per_instance_bytes;
    void* per_pixel;     size_t per_pixel_bytes;
} HtgsTrainBlobs;

int htgs_forward_blob_sizes(const HtgsScene* scene, const HtgsView* view, size_t* per_primitive_bytes, size_t* per_tile_bytes, size_t* per_pixel_bytes);
size_t htgs_forward_instance_bytes(const HtgsView* view, uint64_t n_instances);
/* n_instances rounded up to 2^k or 1.5 * 2^k (at most 50 % more).  The per-instance blob may be larger than
 * htgs_forward_instance_bytes(view, n_instances); a caller whose allocator caches freed blocks by size should allocate
 * htgs_forward_instance_bytes(view, c) bytes with c = htgs_forward_instance_capacity(n_instances), or the largest c it has used
 * so far: the instance count differs from view to view, and a request that outgrows the cached block costs a cudaMalloc inside
 * the training step - and more of them when the allocator then carves the request out of another tensor's cached block. */
uint64_t htgs_forward_instance_capacity(uint64_t n_instances);
int htgs_forward_begin(HtgsContext* ctx, const HtgsScene* scene, const HtgsView* view, void* per_primitive, size_t per_primitive_bytes,
                       void* stream, uint32_t* n_instances);
int htgs_forward_finish(HtgsContext* ctx, const HtgsScene* scene, const HtgsView* view, const HtgsTrainBlobs* blobs, uint32_t n_instances,
                        float* image, void* stream, HtgsFrameInfo* info);

/* Outputs of the backward pass.  Every element of the six gradient tensors is written (zeros for culled
 * Gaussians), so they need not be cleared.  `scratch` (htgs_backward_scratch_bytes) holds the per-Gaussian
 * accumulation records and is cleared by the call.  `densification_info` ([rows,N], rows 2 or 3) is
 * updated in place as in the reference (rasterization/src/rasterization_api.cu:219-223), or NULL. */
typedef struct HtgsGradients {
    float* grad_positions;   /* [N,3] */
    float* grad_scales;      /* [N,3] */
    float* grad_rotations;   /* [N,4] */
    float* grad_opacities;   /* [N,1] */
    float* grad_sh_0;        /* [N,1,3] */
    float* grad_sh_rest;     /* [N,B,3] */
    void* scratch;
    size_t scratch_bytes;
    float* densification_info;
    int32_t densification_rows;
    int32_t use_distance_scaling;
} HtgsGradients;

size_t htgs_backward_scratch_bytes(const HtgsScene* scene);
/* grad_image: [3,H,W]; image: the forward's output, read only by ALPHA_BLEND_GLOBAL_ORDERING (may be NULL otherwise).
 * Stream-ordered, no host synchronisation. */
int htgs_backward(HtgsContext* ctx, const HtgsScene* scene, const HtgsView* view, const HtgsTrainBlobs* blobs, uint32_t n_instances,
                  const float* grad_image, const float* image, const HtgsGradients* grads, void* stream);

/* The backward pass over the Gaussians [first_gaussian, first_gaussian + n_gaussians) only: rows of the six gradient tensors
 * (and of densification_info) inside the range are computed exactly as htgs_backward computes them, everything outside is
 * left untouched.  No counterpart in the reference.  A multi-GPU trainer calls it for one range after the other and starts
 * summing a finished range over the ranks while the next one is computed (a tile's list is ascending in Gaussian index, so a
 * range costs its share of the pass).  ALPHA_BLEND_GLOBAL_ORDERING, whose pass needs every fragment in front of a fragment,
 * accepts the whole scene only (HTGS_ERR_UNSUPPORTED_MODE otherwise).  `grads->scratch` as for htgs_backward; the call
 * clears the scratch rows of its range.  Stream-ordered, no host synchronisation. */
int htgs_backward_range(HtgsContext* ctx, const HtgsScene* scene, const HtgsView* view, const HtgsTrainBlobs* blobs, uint32_t n_instances,
                        const float* grad_image, const float* image, const HtgsGradients* grads, uint32_t first_gaussian, uint32_t n_gaussians,
                        void* stream);

/* The two stages of htgs_backward as separate calls, for trainers that start summing gradients over the ranks before the
 * whole pass has finished without splitting the per-tile pass.  No counterparts in the reference.
 *   htgs_backward_accumulate:    clears the six tensors and the scratch and runs the per-tile pass (per-pixel for
 *                                ALPHA_BLEND_GLOBAL_ORDERING) that accumulates one record per Gaussian in `grads->scratch`;
 *   htgs_backward_finish_range:  turns the records of the Gaussians [first_gaussian, first_gaussian + n_gaussians) into rows of the
 *                                six gradient tensors (and updates densification_info for them).  Works for all four modes.
 * htgs_backward equals accumulate followed by finish_range over the whole scene.  Stream-ordered, no host synchronisation. */
int htgs_backward_accumulate(HtgsContext* ctx, const HtgsScene* scene, const HtgsView* view, const HtgsTrainBlobs* blobs, uint32_t n_instances,
                             const float* grad_image, const float* image, const HtgsGradients* grads, void* stream);
int htgs_backward_finish_range(HtgsContext* ctx, const HtgsScene* scene, const HtgsView* view, const HtgsTrainBlobs* blobs, const HtgsGradients* grads,
                               uint32_t first_gaussian, uint32_t n_gaussians, void* stream);

/* Which Gaussians the training forward kept: visible[i] = 1 when Gaussian i passed culling and touches a tile (these are
 * the only rows of the six gradient tensors the backward pass can make non-zero), else 0.  Reads the per-Gaussian blob
 * htgs_forward_begin filled.  No counterpart in the reference; multi-GPU training uses it to exchange only the rows some
 * rank can have touched.  Stream-ordered, no host synchronisation. */
int htgs_forward_visibility(const HtgsScene* scene, const HtgsTrainBlobs* blobs, uint8_t* visible, void* stream);

/* Packing of per-Gaussian rows for the multi-GPU gradient exchange.  No counterpart in the reference.
 * `tensors` are row-major float tensors with one row per Gaussian (e.g. the six gradients, widths 3, 3, 4, 1, 3, 3 B);
 * htgs_gather_rows copies rows index[0..count) of all of them into packed[count][sum of widths] (tensor after tensor inside
 * a packed row), htgs_scatter_rows copies packed rows back.  `index` (device memory) must hold row numbers inside the
 * tensors (they live on the device and are not checked) and distinct ones for the scatter.  Stream-ordered, no host
 * synchronisation. */
#define HTGS_MAX_ROW_TENSORS 8
typedef struct HtgsRowTensors {
    float* data[HTGS_MAX_ROW_TENSORS];
    int32_t width[HTGS_MAX_ROW_TENSORS];
    int32_t n_tensors;
} HtgsRowTensors;
int htgs_gather_rows(const HtgsRowTensors* tensors, const int64_t* index, int64_t count, float* packed, void* stream);
int htgs_scatter_rows(const HtgsRowTensors* tensors, const int64_t* index, int64_t count, const float* packed, void* stream);

/*
 * Compact gradient rows: what the ranks of a multi-GPU trainer send one another.  No counterpart in the reference.
 *
 * A view keeps about a sixth of a scene's Gaussians, and of the 59 floats of a kept Gaussian's gradient row (SH degree 3) the
 * 48 of grad_sh_0 / grad_sh_rest are the 3-vector dL/drgb times functions of the view direction
 * (rasterization/include/kernel_utils.cuh:190-281 of the reference).  htgs_backward_compact is htgs_backward, except that it
 * does not compute the six tensors of `grads` (all NULL, or all given: then the call clears them, overlapped with its kernels,
 * ready for htgs_expand_add_rows) and writes to `rows` one 64-byte header (row count, camera
 * position, active SH bases) followed by one 64-byte row per kept Gaussian, in no particular order: index, dL/dposition,
 * dL/dscale, dL/dopacity, dL/drotation, dL/drgb after the clamp mask.  `rows` holds htgs_compact_rows_bytes(capacity_rows)
 * bytes, 16-byte aligned; capacity_rows must be at least the number of Gaussians the forward kept (HtgsFrameInfo.n_visible;
 * the scene's size always suffices): rows beyond the capacity are dropped and the header's count tells.
 * `grads->scratch` and `grads->densification_info` are used as by htgs_backward.
 *
 * htgs_expand_add_rows reads such a buffer - this rank's or, after an all-gather or through peer access, another rank's - and
 * ADDS the dense rows it stands for to the six tensors of `grads` (clear them first; `scene` supplies positions, the
 * scene's size and SH layout).  The SH rows are rebuilt with the arithmetic of the backward pass, so expanding a rank's own
 * buffer into cleared tensors reproduces htgs_backward's output bit for bit, and ranks that expand the same buffers in the
 * same order end up with identical sums.  Both calls are stream-ordered and do not synchronise with the host.
 */
size_t htgs_compact_rows_bytes(uint32_t capacity_rows);
/* Copies a compact-row buffer - header and the rows it counts, at most capacity_rows - from `src`, which may be another GPU's
 * buffer (htgs_peer_buffer_open), to `dst` (htgs_compact_rows_bytes(capacity_rows) bytes).  Stream-ordered. */
int htgs_copy_rows(void* dst, const void* src, uint32_t capacity_rows, void* stream);
int htgs_backward_compact(HtgsContext* ctx, const HtgsScene* scene, const HtgsView* view, const HtgsTrainBlobs* blobs, uint32_t n_instances,
                          const float* grad_image, const float* image, const HtgsGradients* grads, void* rows, uint32_t capacity_rows, void* stream);
int htgs_expand_add_rows(const HtgsScene* scene, const void* rows, uint32_t capacity_rows, const HtgsGradients* grads, void* stream);
/* The same sums with every dense row written once: SETS all rows of the six tensors of `grads` to the sum over `buffers`
 * (n_buffers of them, 1..16, each with room for capacity_rows rows), added up per Gaussian in the order given, starting from
 * zero - the additions htgs_expand_add_rows performs buffer after buffer on cleared tensors, so the results are bit-identical to
 * that - and zero for Gaussians no buffer holds; the tensors need not be cleared.  With many buffers this is several times
 * faster (one write per dense row instead of a read and a write per buffer that holds it).  The buffers must be memory of this
 * GPU (rows are fetched one by one: copy a peer's buffer with htgs_copy_rows first).  `scratch`:
 * htgs_expand_sum_scratch_bytes(scene, n_buffers) bytes (4 bytes per Gaussian and buffer).  Stream-ordered. */
size_t htgs_expand_sum_scratch_bytes(const HtgsScene* scene, int n_buffers);
int htgs_expand_sum_rows(const HtgsScene* scene, const void* const* buffers, int n_buffers, uint32_t capacity_rows, void* scratch, size_t scratch_bytes,
                         const HtgsGradients* grads, void* stream);

/*
 * Device buffers that the other ranks' GPUs read directly (peer access over NVLink): the transport of the compact rows that needs
 * no collective to move them and no agreement on sizes.  No counterpart in the reference.
 *   htgs_peer_buffer_create:  cudaMalloc of `bytes` on `device`, cleared, plus the 64-byte handle other PROCESSES open it with;
 *   htgs_peer_buffer_open:    maps another process's buffer into this process for `device` (enables peer access on first use);
 *   htgs_peer_buffer_close / _destroy: undo the two (close every mapping before the owner destroys the buffer).
 * A rank writes its compact rows into its own buffer (htgs_backward_compact), all ranks pass a barrier on their streams (any
 * collective will do), and every rank reads every other rank's buffer through its mapping, with plain loads: either
 * htgs_expand_add_rows directly on the mapping (fine for two ranks), or htgs_copy_rows into local memory first, each rank
 * starting with a different peer, and htgs_expand_add_rows on the copies.  The second form keeps every GPU's memory read by one
 * peer at a time; with the first, all ranks expand rank 0's buffer at the same moment (the sums must be formed in one order on
 * all ranks) and queue on rank 0's links.  With two buffers per rank used in turn, the barrier of the next step also orders a
 * buffer's readers before its next writer.  create / open / close / destroy synchronise with the host (allocation).
 */
#define HTGS_PEER_HANDLE_BYTES 64
int htgs_peer_buffer_create(int device, size_t bytes, void** ptr, void* handle);
int htgs_peer_buffer_open(int device, const void* handle, void** ptr);
int htgs_peer_buffer_close(int device, void* ptr);
int htgs_peer_buffer_destroy(int device, void* ptr);

/*
 * Backward pass that allocates nothing.  No counterpart in the reference.
 *
 * Same inputs, outputs and results as htgs_backward, but `grads->scratch` is ignored: the per-Gaussian
 * accumulation records live in a fixed array inside the library (10 MiB of device memory per GPU that loads
 * the library, held until the process exits).  It exists for hosts that cannot hand over a scratch buffer
 * because they may not allocate device memory at the point of the call: a plug-in inside an application that
 * owns all allocations, or a process that has given every free byte to another allocator.  The call performs
 * no cudaMalloc / cudaFree and calls no allocating library routine (the side stream and the events a context uses are
 * created by htgs_create).
 *   - Scenes with more than htgs_backward_static_max_gaussians() (131072) Gaussians are rejected with
 *     HTGS_ERR_INVALID_ARGUMENT; use htgs_backward for those.
 *   - The first call on a device looks up the device address of the array (cudaGetSymbolAddress); make that
 *     first call before any stream capture.
 *   - All calls on a device share the one array.  Each call clears it before use, but two calls whose kernels
 *     overlap on the GPU (different streams, different host threads) race on it: run them one after the other.
 */
int htgs_backward_static_max_gaussians(void);
int htgs_backward_static(HtgsContext* ctx, const HtgsScene* scene, const HtgsView* view, const HtgsTrainBlobs* blobs, uint32_t n_instances,
                         const float* grad_image, const float* image, const HtgsGradients* grads, void* stream);

/*
 * Relaxed-precision forward, RGB only.  Replaces `_C_benchmarking.benchmark` = fast_inference_wrapper
 * (rasterization/include/fast_inference_api.h:7-25, rasterization/src/fast_inference_api.cu:21-162), the reference's
 * fast-math build.  `image` is [3,H,W] (to_chw) or [H,W,3], clamped to [0,1].  HYBRID_BLEND and ALPHA_BLEND_FIRST_K with K
 * rounded to 4, 8, 16 or 32, and OIT_BLEND, run dedicated kernels whose result agrees with the reference's fast path to about
 * 1e-3 per channel (not bit for bit); GLOBAL_ORDERING and smaller K run the exact kernels of htgs_render.  Workspace handling
 * as htgs_render.
 *
 * The dedicated kernels do not depend on the order of a tile's list, so by default the lists are built with atomics
 * instead of the stable sort: two renders of the same frame can then differ in the last bits (the order of a float
 * sum), never by more than the tolerance above.  htgs_set_fast_deterministic(ctx, 1) selects the ordered binning
 * (bit-reproducible, about 0.25 ms slower per frame at 3 M Gaussians).  No counterpart in the reference.
 */
int htgs_set_fast_deterministic(HtgsContext* ctx, int enable);
int htgs_render_fast(HtgsContext* ctx, const HtgsScene* scene, const HtgsView* view, float* image, int to_chw, void* workspace,
                     size_t workspace_bytes, void* stream, HtgsFrameInfo* info);
/* htgs_render_fast without the host wait; the rules of htgs_render_async apply, htgs_frame_result completes it. */
int htgs_render_fast_async(HtgsContext* ctx, const HtgsScene* scene, const HtgsView* view, float* image, int to_chw, void* stream);

/*
 * Per-Gaussian maximum blending weight over the pixels of one view.  Replaces `_C.update_max_weights` =
 * update_max_weights_wrapper (rasterization/include/rasterization_api.h:79-97).  `max_weights` [N] is raised in place
 * (maximum with what it holds); scene->sh_0 / sh_rest are not read and may be NULL.  Workspace handling as htgs_render.
 */
int htgs_update_max_weights(HtgsContext* ctx, const HtgsScene* scene, const HtgsView* view, float* max_weights, float weight_threshold,
                            void* workspace, size_t workspace_bytes, void* stream, HtgsFrameInfo* info);
/* HYBRID_BLEND only.  The reference's kernel source has a second walk over each tile's list that credits
 * `alpha * tail weight` of the pixel to every fragment (rasterization/include/hybrid_blend/kernels/update_max_weights.cuh:170-210).
 * enable = 1 performs that walk; enable = 0 credits the K-buffer (core) weights only.  See the library's design notes for
 * which of the two the reference extension's build for this GPU was measured to produce. */
int htgs_set_max_weights_tail_credit(HtgsContext* ctx, int enable);

/*
 * 3D smoothing-filter update for one view.  Replaces `_C.update_3d_filter_cuda` = update_3d_filter_wrapper
 * (filter3d/include/filter3d_api.h:7-20, filter3d/src/filter3d_api.cu:6-47).  positions [N,3], w2c [4,4] row-major,
 * filter_3d [N] (updated in place: min with distance2filter * view depth), visibility_mask [N] bytes (set to 1 for points
 * in view that were updated).  Stream-ordered, no host synchronisation.
 */
int htgs_update_3d_filter(const float* positions, const float* w2c, float* filter_3d, uint8_t* visibility_mask, int32_t n_points,
                          int32_t width, int32_t height, float focal_x, float focal_y, float center_x, float center_y, float near_plane,
                          float clipping_tolerance, float distance2filter, void* stream);

/*
 * The same update for several views in one pass over the points (no counterpart in the reference, whose caller loops over
 * the views, Model.py:126-145): equal, bit for bit, to calling htgs_update_3d_filter once per view in order, but the
 * positions are read once per 48 views instead of once per view.  `views` is a HOST array (camera parameters travel as
 * kernel arguments); every other pointer is a device pointer.  Stream-ordered, no host synchronisation, no allocation.
 */
typedef struct HtgsFilterView {
    float w2c[16];                 /* world -> view, row-major */
    int32_t width, height;
    float focal_x, focal_y, center_x, center_y, near_plane;
} HtgsFilterView;
int htgs_update_3d_filter_views(const float* positions, const HtgsFilterView* views, int32_t n_views, float* filter_3d, uint8_t* visibility_mask,
                                int32_t n_points, float clipping_tolerance, float distance2filter, void* stream);

/*
 * Fused parameter activations of the Gaussian model, forward and backward (one pass over N).  Replaces the element-wise
 * PyTorch operations the reference's model applies before every rasterizer call (Model.py:45-49 exp / normalize / expit,
 * Model.py:82-100 the 3D-filter adjustment):
 *   scales = exp(raw_scales), rotations = raw_rotations / max(|raw_rotations|, 1e-12), opacities = expit(raw_opacities);
 *   with filter_3d [N] != NULL: scales = sqrt(scales^2 + f^2), opacities *= prod_i exp(raw_scales_i) / scales_i.
 * raw_scales / scales [N,3], raw_rotations / rotations [N,4], raw_opacities / opacities [N]; outputs may not alias inputs.
 * The backward takes the gradients with respect to the three outputs and returns those with respect to the raw inputs.
 * Stream-ordered, no host synchronisation.
 */
int htgs_activate(const float* raw_scales, const float* raw_rotations, const float* raw_opacities, const float* filter_3d, float* scales,
                  float* rotations, float* opacities, int32_t n_primitives, void* stream);
int htgs_activate_backward(const float* raw_scales, const float* raw_rotations, const float* raw_opacities, const float* filter_3d,
                           const float* grad_scales, const float* grad_rotations, const float* grad_opacities, float* grad_raw_scales,
                           float* grad_raw_rotations, float* grad_raw_opacities, int32_t n_primitives, void* stream);

/* Measurement aids (off by default; they do not change results).
 * Profiling: CUDA events are recorded on the frame's stream between the stages; after the call
 * htgs_get_stage_ms fills out_ms[0..HTGS_N_STAGES) with the device time of each stage in ms.
 * Statistics: the blend kernel also counts candidate pairs and accepted fragments (HtgsFrameInfo). */
enum HtgsStage {
    HTGS_STAGE_PREPROCESS = 0, HTGS_STAGE_SCAN = 1, HTGS_STAGE_EMIT = 2, HTGS_STAGE_SORT = 3,
    HTGS_STAGE_RANGES = 4, HTGS_STAGE_BLEND = 5, HTGS_STAGE_TOTAL = 6, HTGS_N_STAGES = 7
};
/* Frames of several contexts in flight on one GPU: by default the short kernels at the front of a frame (preprocess, scans,
 * sort) run on a context-owned stream of the highest priority, ordered after everything queued on the caller's stream
 * before the call and before the blend kernel, which stays on the caller's stream; the block scheduler then places them
 * ahead of the queued CTAs of another frame's blend kernel.  Results do not change.  0 keeps every kernel on the caller's stream. */
int htgs_set_front_priority(HtgsContext* ctx, int enable);
int htgs_set_profiling(HtgsContext* ctx, int enable);
int htgs_get_stage_ms(HtgsContext* ctx, float* out_ms);
int htgs_set_collect_stats(HtgsContext* ctx, int enable);

/* Plain device<->host copies for callers that have no CUDA runtime binding of their own (tests). */
int htgs_memcpy_d2h(void* host_dst, const void* device_src, size_t bytes);
int htgs_memcpy_h2d(void* device_dst, const void* host_src, size_t bytes);

#ifdef __cplusplus
}
#endif

#endif /* HTGS_B200_H */
