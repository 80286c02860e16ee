// C-ABI layer: contexts, workspace carving and the stream-ordered frame drivers.
// Host code only; the kernels live in preprocess.cu, binning.cu and blend.cu.
//
// A forward frame is: status reset -> preprocess -> scan of block sums -> instance
// emission -> stable radix sort -> tile ranges -> blend -> asynchronous copy of the
// 64-byte frame status to pinned host memory.  There is one host synchronisation, at
// the end (the reference blocks in the middle of every frame to read the instance
// count: rasterization/src/hybrid_blend/inference.cu:118-119).  The instance buffers are
// sized speculatively; if a frame needs more, the kernels skip the instance stages, the
// status says so, and the driver grows the workspace and runs the frame again.
#include <algorithm>
#include <cstdio>
#include <cstring>
#include <string>
#include <vector>

#include "kernels.h"

using namespace htgs;

namespace {

thread_local std::string g_last_error;

int fail(int code, const std::string& msg) { g_last_error = msg; return code; }
int fail_cuda(cudaError_t err, const char* what) {
    g_last_error = std::string(what) + ": " + cudaGetErrorString(err);
    return HTGS_ERR_CUDA;
}

// Makes the context's device current for the duration of a call and puts the caller's device back afterwards.
struct DeviceGuard {
    int previous = -1;
    cudaError_t status = cudaSuccess;
    explicit DeviceGuard(int device) {
        status = cudaGetDevice(&previous);
        if (status == cudaSuccess && previous != device) status = cudaSetDevice(device);
        else previous = -1;   // nothing to restore
    }
    ~DeviceGuard() { if (previous >= 0) cudaSetDevice(previous); }
    DeviceGuard(const DeviceGuard&) = delete;
    DeviceGuard& operator=(const DeviceGuard&) = delete;
};

constexpr size_t kAlign = 256;
inline size_t align_up(size_t v) { return (v + kAlign - 1) & ~(kAlign - 1); }

struct Carver {
    unsigned char* base;
    size_t offset = 0;
    explicit Carver(void* b) : base(static_cast<unsigned char*>(b)) {}
    template <typename T> T* take(size_t count) {
        offset = align_up(offset);
        T* p = base ? reinterpret_cast<T*>(base + offset) : nullptr;
        offset += count * sizeof(T);
        return p;
    }
    template <typename T> T* take_bytes(size_t bytes) {
        offset = align_up(offset);
        T* p = base ? reinterpret_cast<T*>(base + offset) : nullptr;
        offset += bytes;
        return p;
    }
};

struct FrameLayout {
    FrameStatus* status;
    PrimBuffers prim;
    InstBuffers inst;
    uint2* tile_ranges;
    size_t bytes;
};

FrameLayout carve_frame(void* blob, int n_primitives, int n_tiles, const SortPlan& plan, uint64_t instance_capacity, bool training) {
    FrameLayout L{};
    Carver c(blob);
    const size_t n = size_t(n_primitives);
    const size_t prim_blocks = (n + kPreprocessBlock - 1) / kPreprocessBlock;
    L.status = c.take<FrameStatus>(1);
    L.prim.n_touched = c.take<uint32_t>(n);
    L.prim.bounds = c.take<ushort4>(n);
    L.prim.eval = c.take<EvalRecord>(n);
    L.prim.cull = c.take<CullRecord>(n);
    L.prim.clamp = training ? c.take<uint8_t>(n) : nullptr;
    L.prim.block_sums = c.take<uint32_t>(prim_blocks + 1);
    L.prim.block_offsets = c.take<uint32_t>(prim_blocks + 1);
    L.prim.visible_list = c.take<uint32_t>(n);
    L.tile_ranges = c.take<uint2>(size_t(n_tiles));
    const uint64_t cap = instance_capacity > 0xfffffff0ull ? 0xfffffff0ull : instance_capacity;
    L.inst.capacity = uint32_t(cap);
    L.inst.sort_blocks_cap = uint32_t((cap + kSortTile - 1) / kSortTile);
    L.inst.keys[0] = c.take_bytes<void>(size_t(cap) * plan.key_bytes);
    L.inst.keys[1] = c.take_bytes<void>(size_t(cap) * plan.key_bytes);
    L.inst.prims[0] = c.take<uint32_t>(size_t(cap));
    L.inst.prims[1] = c.take<uint32_t>(size_t(cap));
    L.inst.sort_scratch = c.take_bytes<void>(sort_scratch_bytes(plan, L.inst.sort_blocks_cap));
    L.bytes = align_up(c.offset);
    return L;
}

int validate(const HtgsScene* scene, const HtgsView* view, bool needs_colour = true) {
    if (!scene || !view) return fail(HTGS_ERR_INVALID_ARGUMENT, "scene and view must not be null");
    if (view->mode < 0 || view->mode > 3) return fail(HTGS_ERR_UNSUPPORTED_MODE, "unsupported rasterizer mode");
    if (scene->n_primitives < 0) return fail(HTGS_ERR_INVALID_ARGUMENT, "n_primitives must be >= 0");
    if (view->width <= 0 || view->height <= 0) return fail(HTGS_ERR_INVALID_ARGUMENT, "width and height must be positive");
    if (view->width > 65535 * 8 || view->height > 65535 * 8) return fail(HTGS_ERR_INVALID_ARGUMENT, "image too large for 16-bit tile coordinates");
    if (scene->n_primitives > 0 && (!scene->positions || !scene->scales || !scene->rotations || !scene->opacities || (needs_colour && !scene->sh_0)))
        return fail(HTGS_ERR_INVALID_ARGUMENT, "per-Gaussian input pointers must not be null");
    if (scene->total_sh_bases < 0) return fail(HTGS_ERR_INVALID_ARGUMENT, "total_sh_bases must be >= 0");
    const int a = view->active_sh_bases;
    if (a != 1 && a != 4 && a != 9 && a != 16) return fail(HTGS_ERR_INVALID_ARGUMENT, "active_sh_bases must be 1, 4, 9 or 16");
    if (needs_colour && a - 1 > scene->total_sh_bases) return fail(HTGS_ERR_INVALID_ARGUMENT, "active_sh_bases needs more coefficients than sh_rest holds");
    if (needs_colour && a > 1 && !scene->sh_rest) return fail(HTGS_ERR_INVALID_ARGUMENT, "sh_rest must not be null when active_sh_bases > 1");
    if (!view->M || !view->VPM || !view->cam_position) return fail(HTGS_ERR_INVALID_ARGUMENT, "camera pointers must not be null");
    if ((view->mode == HTGS_MODE_HYBRID_BLEND || view->mode == HTGS_MODE_ALPHA_BLEND_FIRST_K) && view->K < 1)
        return fail(HTGS_ERR_INVALID_ARGUMENT, "K must be >= 1");
    return HTGS_OK;
}

}  // namespace

// What htgs_render_async queued and htgs_frame_result (or the next call on the context) still has to check.
struct PendingFrame {
    bool active = false;
    HtgsScene scene{};
    HtgsView view{};
    BlendOutputs out{};
    void* workspace = nullptr;          // caller's workspace, or null for the context's own
    size_t workspace_bytes = 0;
    cudaStream_t stream = nullptr;
    float* max_weights = nullptr;
    float weight_threshold = 0.0f;
    bool fast = false;
    FrameGeometry geo{};
    SortPlan plan{};
    FrameLayout layout{};
    uint64_t capacity = 0;
    uint32_t reruns = 0, launches = 0;
    bool profiled = false;              // stage events were recorded for this frame
};

struct HtgsContext {
    int device = 0;
    int sm_count = 0;
    FrameStatus* host_status = nullptr;     // pinned
    void* workspace = nullptr;              // internal grow-only workspace
    size_t workspace_bytes = 0;
    uint64_t instance_capacity = 0;         // capacity the internal workspace was last carved for
    // staging buffers of htgs_render_host
    void* host_path_buf = nullptr;
    size_t host_path_bytes = 0;
    cudaStream_t host_path_stream = nullptr;
    // what the last frame used (htgs_get_intermediates)
    FrameLayout last_layout{};
    SortPlan last_plan{};
    FrameGeometry last_geo{};
    uint32_t last_n_instances = 0;
    bool has_last = false;
    HtgsFrameInfo last_info{};
    // the frame whose status has not been read yet (htgs_render_async)
    PendingFrame pending{};
    cudaEvent_t frame_done = nullptr;       // recorded after the status copy of a frame
    // measurement aids
    bool profiling = false;
    bool collect_stats = false;
    bool fast_deterministic = false;        // htgs_render_fast: ordered (radix sort) instead of unordered (atomic) binning
    bool max_weights_tail_credit = false;   // htgs_set_max_weights_tail_credit
    cudaEvent_t events[8] = {};
    bool events_created = false;
    // With several frames in flight on one GPU (one context and stream each), the short kernels at the front of a
    // frame (preprocess, scans, sort) go to a stream of the highest priority, so that the block scheduler places them ahead of
    // the queued CTAs of ANOTHER frame's blend kernel instead of behind all of them; the blend stays on the caller's stream.
    // The stream and its two events are created with the context, so that no later call has to create driver objects.
    bool front_priority = true;             // htgs_set_front_priority
    cudaStream_t front_stream = nullptr;
    cudaEvent_t front_begin = nullptr, front_end = nullptr;
    float stage_ms[HTGS_N_STAGES] = {};
};

namespace htgs {
int context_device(const HtgsContext* ctx) { return ctx ? ctx->device : -1; }
void set_last_error(const char* message) { g_last_error = message ? message : ""; }
}  // namespace htgs

static int finish_frame(HtgsContext* ctx, HtgsFrameInfo* info);

// A call on a context whose previous frame was queued with htgs_render_async checks that frame first.
static int settle_pending(HtgsContext* ctx) {
    if (!ctx->pending.active) return HTGS_OK;
    const int rc = finish_frame(ctx, nullptr);
    if (rc != HTGS_OK) g_last_error = "deferred check of the previous frame: " + g_last_error;
    return rc;
}

extern "C" {

int htgs_version(void) { return 110; }

const char* htgs_last_error(void) { return g_last_error.c_str(); }

HtgsContext* htgs_create(int device) {
    int count = 0;
    cudaError_t err = cudaGetDeviceCount(&count);
    if (err != cudaSuccess || count == 0) { fail_cuda(err != cudaSuccess ? err : cudaErrorNoDevice, "htgs_create: no CUDA device"); return nullptr; }
    if (device < 0 || device >= count) { fail(HTGS_ERR_INVALID_ARGUMENT, "htgs_create: bad device index"); return nullptr; }
    DeviceGuard guard(device);
    if (guard.status != cudaSuccess) { fail_cuda(guard.status, "cudaSetDevice"); return nullptr; }
    cudaDeviceProp prop;
    if ((err = cudaGetDeviceProperties(&prop, device)) != cudaSuccess) { fail_cuda(err, "cudaGetDeviceProperties"); return nullptr; }
    if (prop.major != 10) { fail(HTGS_ERR_INVALID_ARGUMENT, "htgs_create: this library is built for sm_100a (B200) only"); return nullptr; }
    HtgsContext* ctx = new HtgsContext();
    ctx->device = device;
    ctx->sm_count = prop.multiProcessorCount;
    int least = 0, greatest = 0;
    if ((err = cudaHostAlloc(reinterpret_cast<void**>(&ctx->host_status), sizeof(FrameStatus), cudaHostAllocDefault)) != cudaSuccess ||
        (err = cudaDeviceGetStreamPriorityRange(&least, &greatest)) != cudaSuccess ||
        (err = cudaStreamCreateWithPriority(&ctx->front_stream, cudaStreamNonBlocking, greatest)) != cudaSuccess ||
        (err = cudaEventCreateWithFlags(&ctx->front_begin, cudaEventDisableTiming)) != cudaSuccess ||
        (err = cudaEventCreateWithFlags(&ctx->front_end, cudaEventDisableTiming)) != cudaSuccess ||
        (err = cudaEventCreateWithFlags(&ctx->frame_done, cudaEventDisableTiming)) != cudaSuccess) {
        fail_cuda(err, "htgs_create: pinned status word, side stream and events");
        htgs_destroy(ctx);
        return nullptr;
    }
    std::memset(ctx->host_status, 0, sizeof(FrameStatus));
    return ctx;
}

void htgs_destroy(HtgsContext* ctx) {
    if (!ctx) return;
    DeviceGuard guard(ctx->device);
    if (ctx->pending.active) cudaEventSynchronize(ctx->frame_done);
    if (ctx->workspace) cudaFree(ctx->workspace);
    if (ctx->host_path_buf) cudaFree(ctx->host_path_buf);
    if (ctx->host_path_stream) cudaStreamDestroy(ctx->host_path_stream);
    if (ctx->host_status) cudaFreeHost(ctx->host_status);
    if (ctx->events_created) for (auto& e : ctx->events) cudaEventDestroy(e);
    if (ctx->front_stream) cudaStreamDestroy(ctx->front_stream);
    if (ctx->front_begin) cudaEventDestroy(ctx->front_begin);
    if (ctx->front_end) cudaEventDestroy(ctx->front_end);
    if (ctx->frame_done) cudaEventDestroy(ctx->frame_done);
    delete ctx;
}

size_t htgs_render_workspace_bytes(const HtgsScene* scene, const HtgsView* view, uint64_t instance_capacity) {
    if (validate(scene, view) != HTGS_OK) return 0;
    const FrameGeometry geo = make_geometry(view->mode, view->width, view->height);
    const SortPlan plan = make_sort_plan(view->mode, geo.n_tiles);
    return carve_frame(nullptr, scene->n_primitives, geo.n_tiles, plan, instance_capacity, false).bytes;
}

}  // extern "C"

// Queues one frame (all kernels, the copy of the 64-byte status to pinned memory and the `frame_done` event) on the
// frame's stream; does not wait for anything.
static int enqueue_frame(HtgsContext* ctx, PendingFrame& f) {
    cudaError_t err;
    const HtgsScene& scene = f.scene;
    const HtgsView& view = f.view;
    const FrameGeometry& geo = f.geo;
    const SortPlan& plan = f.plan;
    const FrameLayout& L = f.layout;
    BlendOutputs out = f.out;
    uint32_t* launches = &f.launches;
    cudaStream_t stream = f.stream;
    const bool prof = ctx->profiling;
    f.profiled = prof;
    if (prof && !ctx->events_created) {
        for (auto& e : ctx->events) if ((err = cudaEventCreate(&e)) != cudaSuccess) return fail_cuda(err, "cudaEventCreate");
        ctx->events_created = true;
    }
    cudaEvent_t* ev = ctx->events;   // 0 start, 1 preprocess, 2 scan, 3 emit, 4 sort, 5 ranges, 6 blend
    out.collect_stats = ctx->collect_stats;
    cudaStream_t const caller_stream = stream;
    const bool front_priority = ctx->front_priority;
    if (front_priority) {
        // everything the caller queued before this call (camera upload, the previous frame) comes first
        if ((err = cudaEventRecord(ctx->front_begin, caller_stream)) != cudaSuccess) return fail_cuda(err, "front event record");
        if ((err = cudaStreamWaitEvent(ctx->front_stream, ctx->front_begin, 0)) != cudaSuccess) return fail_cuda(err, "front stream wait");
        stream = ctx->front_stream;
    }
    if ((err = cudaMemsetAsync(L.status, 0, sizeof(FrameStatus), stream)) != cudaSuccess) return fail_cuda(err, "status reset");
    if (prof) cudaEventRecord(ev[0], stream);
    if ((err = launch_preprocess(view.mode, false, scene, view, geo, L.prim, L.status, stream, f.fast)) != cudaSuccess) return fail_cuda(err, "preprocess");
    if (prof) cudaEventRecord(ev[1], stream);
    if ((err = launch_scan_only(scene, L.prim, L.inst.capacity, L.status, stream)) != cudaSuccess) return fail_cuda(err, "scan");
    if (prof) cudaEventRecord(ev[2], stream);
    *launches += (scene.n_primitives > 0 ? 2 : 0) + 1;
    const uint32_t* prims_sorted = L.inst.prims[plan.final_buffer];
    if (f.fast && !ctx->fast_deterministic) {
        if ((err = launch_bin_unordered(scene, geo, L.prim, L.inst.prims[plan.final_buffer], L.inst.capacity, L.tile_ranges, L.status, ctx->sm_count,
                                        stream, prof ? ev + 3 : nullptr, launches)) != cudaSuccess) return fail_cuda(err, "unordered binning");
    } else if ((err = launch_emit_sort_ranges(view.mode, scene, geo, plan, L.prim, L.inst, L.tile_ranges, L.status, ctx->sm_count, stream,
                                              prof ? ev + 3 : nullptr, launches)) != cudaSuccess) return fail_cuda(err, "binning");
    if (front_priority) {
        if ((err = cudaEventRecord(ctx->front_end, stream)) != cudaSuccess) return fail_cuda(err, "front event record");
        if ((err = cudaStreamWaitEvent(caller_stream, ctx->front_end, 0)) != cudaSuccess) return fail_cuda(err, "caller stream wait");
        stream = caller_stream;
    }
    if (f.max_weights) {
        if ((err = launch_max_weights(view.mode, view.K, geo, L.prim, prims_sorted, L.tile_ranges, f.max_weights, f.weight_threshold, ctx->max_weights_tail_credit,
                                      stream)) != cudaSuccess) return fail_cuda(err, "max weights");
    } else if (f.fast) {
        if ((err = launch_blend_fast(view.mode, view.K, geo, L.prim, prims_sorted, L.tile_ranges, out.image, out.to_chw, L.status, stream)) != cudaSuccess) return fail_cuda(err, "fast blend");
    } else if ((err = launch_blend(view.mode, view.K, false, geo, L.prim, prims_sorted, L.tile_ranges, out, TrainPixelBuffers{}, L.status, stream)) != cudaSuccess) return fail_cuda(err, "blend");
    *launches += 1;
    if (prof) cudaEventRecord(ev[6], stream);
    if ((err = cudaMemcpyAsync(ctx->host_status, L.status, sizeof(FrameStatus), cudaMemcpyDeviceToHost, stream)) != cudaSuccess) return fail_cuda(err, "status copy");
    if ((err = cudaEventRecord(ctx->frame_done, stream)) != cudaSuccess) return fail_cuda(err, "frame event record");
    return HTGS_OK;
}

// Carves the frame's buffers for `f.capacity` instances (growing the context's workspace if it is the one in use) and queues the frame.
static int carve_and_enqueue(HtgsContext* ctx, PendingFrame& f) {
    const bool internal = f.workspace == nullptr;
    if (internal) {
        const size_t need = carve_frame(nullptr, f.scene.n_primitives, f.geo.n_tiles, f.plan, f.capacity, false).bytes;
        if (need > ctx->workspace_bytes) {
            cudaError_t err;
            // the old workspace may still be in use by frames queued earlier (on this stream or the side stream)
            if ((err = cudaStreamSynchronize(f.stream)) != cudaSuccess) return fail_cuda(err, "synchronise before growing the workspace");
            if ((err = cudaStreamSynchronize(ctx->front_stream)) != cudaSuccess) return fail_cuda(err, "synchronise before growing the workspace");
            if (ctx->workspace) cudaFree(ctx->workspace);
            ctx->workspace = nullptr; ctx->workspace_bytes = 0;
            const size_t grow = need + need / 8;
            if ((err = cudaMalloc(&ctx->workspace, grow)) != cudaSuccess) return fail_cuda(err, "workspace allocation");
            ctx->workspace_bytes = grow;
        }
        ctx->instance_capacity = f.capacity;
        f.layout = carve_frame(ctx->workspace, f.scene.n_primitives, f.geo.n_tiles, f.plan, f.capacity, false);
    } else {
        f.layout = carve_frame(f.workspace, f.scene.n_primitives, f.geo.n_tiles, f.plan, f.capacity, false);
    }
    return enqueue_frame(ctx, f);
}

// First half of a render call: validation, sizing and queueing.  On success the frame is `ctx->pending`.
static int begin_frame(HtgsContext* ctx, const HtgsScene* scene, const HtgsView* view, float* image, float* depth, float* alpha,
                       int to_chw, int use_median_depth, void* workspace, size_t workspace_bytes, void* stream_ptr, HtgsFrameInfo* info,
                       float* max_weights, float weight_threshold, bool fast) {
    int rc = validate(scene, view, max_weights == nullptr);
    if (rc != HTGS_OK) return rc;
    if ((rc = settle_pending(ctx)) != HTGS_OK) return rc;
    PendingFrame& f = ctx->pending;
    f = PendingFrame{};
    f.scene = *scene; f.view = *view;
    f.stream = static_cast<cudaStream_t>(stream_ptr);
    f.geo = make_geometry(view->mode, view->width, view->height);
    f.fast = fast && !max_weights && blend_fast_supports(view->mode, view->K);   // other modes / K: the exact kernels serve the fast entry point
    f.plan = make_sort_plan(view->mode, f.geo.n_tiles);
    f.out = BlendOutputs{image, depth, alpha, to_chw != 0, use_median_depth != 0, false};
    f.workspace = workspace; f.workspace_bytes = workspace_bytes;
    f.max_weights = max_weights; f.weight_threshold = weight_threshold;
    if (workspace == nullptr) {
        f.capacity = ctx->instance_capacity ? ctx->instance_capacity : std::max<uint64_t>(uint64_t(scene->n_primitives) * 4, 1u << 20);
    } else {
        // largest capacity that fits the caller's workspace (the layout is monotone in capacity)
        const size_t fixed = carve_frame(nullptr, scene->n_primitives, f.geo.n_tiles, f.plan, 0, false).bytes;
        if (workspace_bytes < fixed + 4096) {
            if (info) { std::memset(info, 0, sizeof(*info)); info->workspace_bytes = fixed + 4096; }
            return fail(HTGS_ERR_WORKSPACE_TOO_SMALL, "workspace too small for the per-Gaussian buffers");
        }
        const size_t per_inst = size_t(f.plan.key_bytes) * 2 + 8 + (sort_scratch_bytes(f.plan, 1024) / 1024 + kSortTile - 1) / kSortTile + 1;
        uint64_t capacity = (workspace_bytes - fixed - 8 * kAlign) / per_inst;
        while (capacity > 0 && carve_frame(nullptr, scene->n_primitives, f.geo.n_tiles, f.plan, capacity, false).bytes > workspace_bytes) capacity -= std::min<uint64_t>(capacity, 4096);
        f.capacity = capacity;
    }
    if ((rc = carve_and_enqueue(ctx, f)) != HTGS_OK) return rc;
    f.active = true;
    return HTGS_OK;
}

// Second half: waits for the pending frame, reads its status, re-runs it after growing the workspace when its instance
// buffers were too small, and fills `info`.
static int finish_frame(HtgsContext* ctx, HtgsFrameInfo* info) {
    PendingFrame& f = ctx->pending;
    if (!f.active) {
        if (info) *info = ctx->last_info;
        return HTGS_OK;
    }
    const bool internal = f.workspace == nullptr;
    for (;;) {
        cudaError_t err;
        if ((err = cudaEventSynchronize(ctx->frame_done)) != cudaSuccess) { f.active = false; return fail_cuda(err, "frame synchronisation"); }
        if (f.profiled) {
            for (int i = 0; i < 6; ++i) cudaEventElapsedTime(&ctx->stage_ms[i], ctx->events[i], ctx->events[i + 1]);
            cudaEventElapsedTime(&ctx->stage_ms[HTGS_STAGE_TOTAL], ctx->events[0], ctx->events[6]);
        }
        const FrameStatus st = *ctx->host_status;
        ctx->last_layout = f.layout; ctx->last_plan = f.plan; ctx->last_geo = f.geo; ctx->last_n_instances = st.overflow ? 0 : st.n_instances; ctx->has_last = true;
        const uint64_t needed_capacity = uint64_t(st.n_instances) + uint64_t(st.n_instances) / 4 + 4096;
        HtgsFrameInfo& li = ctx->last_info;
        li.n_instances = st.n_instances; li.n_visible = st.n_visible; li.key_bytes = uint32_t(f.plan.key_bytes);
        li.end_bit = uint32_t(f.plan.end_bit); li.reruns = f.reruns; li.device_error = st.error;
        li.kernel_launches = f.launches; li.reserved = 0;
        li.candidate_pairs = st.candidate_pairs; li.accepted_fragments = st.accepted_fragments;
        li.warp_trips = st.warp_trips; li.warp_trips_inserting = st.warp_trips_inserting; li.lane_insertions = st.lane_insertions;
        li.workspace_bytes = carve_frame(nullptr, f.scene.n_primitives, f.geo.n_tiles, f.plan, st.overflow ? needed_capacity : f.capacity, false).bytes;
        if (info) *info = li;
        if (st.error) { f.active = false; return fail(HTGS_ERR_DEVICE_FLAG, "a kernel reported an internal error (bounded wait gave up)"); }
        if (!st.overflow) { f.active = false; return HTGS_OK; }
        f.active = false;
        if (st.n_instances == 0xffffffffu) return fail(HTGS_ERR_INVALID_ARGUMENT, "instance count does not fit 32 bits");
        if (!internal) return fail(HTGS_ERR_WORKSPACE_TOO_SMALL, "workspace too small for the instance buffers of this frame");
        if (f.reruns >= 2) return fail(HTGS_ERR_CUDA, "frame still overflows after growing the workspace");
        f.capacity = needed_capacity;
        ++f.reruns;
        const int rc = carve_and_enqueue(ctx, f);
        if (rc != HTGS_OK) return rc;
        f.active = true;
    }
}

static int render_core(HtgsContext* ctx, const HtgsScene* scene, const HtgsView* view, float* image, float* depth, float* alpha,
                       int to_chw, int use_median_depth, void* workspace, size_t workspace_bytes, void* stream_ptr, HtgsFrameInfo* info,
                       float* max_weights, float weight_threshold, bool fast, bool wait) {
    if (!ctx) return fail(HTGS_ERR_INVALID_ARGUMENT, "context must not be null");
    DeviceGuard guard(ctx->device);
    if (guard.status != cudaSuccess) return fail_cuda(guard.status, "cudaSetDevice");
    const int rc = begin_frame(ctx, scene, view, image, depth, alpha, to_chw, use_median_depth, workspace, workspace_bytes, stream_ptr, info, max_weights, weight_threshold, fast);
    if (rc != HTGS_OK || !wait) return rc;
    return finish_frame(ctx, info);
}

extern "C" {

int htgs_render(HtgsContext* ctx, const HtgsScene* scene, const HtgsView* view, float* image, float* depth, float* alpha,
                int to_chw, int use_median_depth, void* workspace, size_t workspace_bytes, void* stream_ptr, HtgsFrameInfo* info) {
    if (!image || !depth) return fail(HTGS_ERR_INVALID_ARGUMENT, "image and depth must not be null");
    return render_core(ctx, scene, view, image, depth, alpha, to_chw, use_median_depth, workspace, workspace_bytes, stream_ptr, info, nullptr, 0.0f, false, true);
}

int htgs_render_async(HtgsContext* ctx, const HtgsScene* scene, const HtgsView* view, float* image, float* depth, float* alpha,
                      int to_chw, int use_median_depth, void* stream_ptr) {
    if (!image || !depth) return fail(HTGS_ERR_INVALID_ARGUMENT, "image and depth must not be null");
    return render_core(ctx, scene, view, image, depth, alpha, to_chw, use_median_depth, nullptr, 0, stream_ptr, nullptr, nullptr, 0.0f, false, false);
}

int htgs_render_fast_async(HtgsContext* ctx, const HtgsScene* scene, const HtgsView* view, float* image, int to_chw, void* stream_ptr) {
    if (!image) return fail(HTGS_ERR_INVALID_ARGUMENT, "image must not be null");
    return render_core(ctx, scene, view, image, nullptr, nullptr, to_chw, 0, nullptr, 0, stream_ptr, nullptr, nullptr, 0.0f, true, false);
}

int htgs_frame_result(HtgsContext* ctx, HtgsFrameInfo* info) {
    if (!ctx) return fail(HTGS_ERR_INVALID_ARGUMENT, "context must not be null");
    DeviceGuard guard(ctx->device);
    if (guard.status != cudaSuccess) return fail_cuda(guard.status, "cudaSetDevice");
    return finish_frame(ctx, info);
}

int htgs_update_max_weights(HtgsContext* ctx, const HtgsScene* scene, const HtgsView* view, float* max_weights, float weight_threshold,
                            void* workspace, size_t workspace_bytes, void* stream_ptr, HtgsFrameInfo* info) {
    if (!max_weights) return fail(HTGS_ERR_INVALID_ARGUMENT, "max_weights must not be null");
    return render_core(ctx, scene, view, nullptr, nullptr, nullptr, 1, 0, workspace, workspace_bytes, stream_ptr, info, max_weights, weight_threshold, false, true);
}

int htgs_render_fast(HtgsContext* ctx, const HtgsScene* scene, const HtgsView* view, float* image, int to_chw, void* workspace,
                     size_t workspace_bytes, void* stream_ptr, HtgsFrameInfo* info) {
    if (!image) return fail(HTGS_ERR_INVALID_ARGUMENT, "image must not be null");
    return render_core(ctx, scene, view, image, nullptr, nullptr, to_chw, 0, workspace, workspace_bytes, stream_ptr, info, nullptr, 0.0f, true, true);
}

int htgs_get_intermediates(HtgsContext* ctx, HtgsIntermediates* out) {
    if (!ctx || !out) return fail(HTGS_ERR_INVALID_ARGUMENT, "null argument");
    if (ctx->pending.active) {
        DeviceGuard guard(ctx->device);
        const int rc = settle_pending(ctx);
        if (rc != HTGS_OK) return rc;
    }
    if (!ctx->has_last) return fail(HTGS_ERR_INVALID_ARGUMENT, "no frame has been rendered on this context");
    const FrameLayout& L = ctx->last_layout;
    const SortPlan& p = ctx->last_plan;
    out->n_touched = L.prim.n_touched;
    out->bounds = reinterpret_cast<const uint16_t*>(L.prim.bounds);
    out->eval_records = L.prim.eval;
    out->cull_records = L.prim.cull;
    const int unsorted = (p.n_passes == 0) ? 0 : (p.final_buffer ^ (p.n_passes & 1));   // emission always writes buffer 0
    out->keys_unsorted = (p.n_passes == 1 || p.n_passes == 0) ? L.inst.keys[unsorted] : nullptr;   // overwritten by later passes otherwise
    out->prims_unsorted = (p.n_passes == 1 || p.n_passes == 0) ? L.inst.prims[unsorted] : nullptr;
    out->keys_sorted = L.inst.keys[p.final_buffer];
    out->prims_sorted = L.inst.prims[p.final_buffer];
    out->tile_ranges = reinterpret_cast<const uint32_t*>(L.tile_ranges);
    out->n_tiles = uint32_t(ctx->last_geo.n_tiles);
    out->grid_width = uint32_t(ctx->last_geo.grid_w);
    out->grid_height = uint32_t(ctx->last_geo.grid_h);
    out->key_bytes = uint32_t(p.key_bytes);
    return HTGS_OK;
}

int htgs_set_profiling(HtgsContext* ctx, int enable) {
    if (!ctx) return fail(HTGS_ERR_INVALID_ARGUMENT, "context must not be null");
    ctx->profiling = enable != 0;
    return HTGS_OK;
}

int htgs_get_stage_ms(HtgsContext* ctx, float* out_ms) {
    if (!ctx || !out_ms) return fail(HTGS_ERR_INVALID_ARGUMENT, "null argument");
    for (int i = 0; i < HTGS_N_STAGES; ++i) out_ms[i] = ctx->stage_ms[i];
    return HTGS_OK;
}

int htgs_set_front_priority(HtgsContext* ctx, int enable) {
    if (!ctx) return fail(HTGS_ERR_INVALID_ARGUMENT, "context must not be null");
    ctx->front_priority = enable != 0;
    return HTGS_OK;
}

int htgs_set_fast_deterministic(HtgsContext* ctx, int enable) {
    if (!ctx) return fail(HTGS_ERR_INVALID_ARGUMENT, "context must not be null");
    ctx->fast_deterministic = enable != 0;
    return HTGS_OK;
}

int htgs_set_max_weights_tail_credit(HtgsContext* ctx, int enable) {
    if (!ctx) return fail(HTGS_ERR_INVALID_ARGUMENT, "context must not be null");
    ctx->max_weights_tail_credit = enable != 0;
    return HTGS_OK;
}

int htgs_set_collect_stats(HtgsContext* ctx, int enable) {
    if (!ctx) return fail(HTGS_ERR_INVALID_ARGUMENT, "context must not be null");
    ctx->collect_stats = enable != 0;
    return HTGS_OK;
}

int htgs_render_host(HtgsContext* ctx, const HtgsScene* hs, const HtgsView* hv, float* host_image, float* host_depth,
                     int to_chw, int use_median_depth, HtgsFrameInfo* info) {
    if (!ctx) return fail(HTGS_ERR_INVALID_ARGUMENT, "context must not be null");
    int rc = validate(hs, hv);
    if (rc != HTGS_OK) return rc;
    if (!host_image || !host_depth) return fail(HTGS_ERR_INVALID_ARGUMENT, "image and depth must not be null");
    cudaError_t err;
    DeviceGuard guard(ctx->device);
    if (guard.status != cudaSuccess) return fail_cuda(guard.status, "cudaSetDevice");
    if (!ctx->host_path_stream && (err = cudaStreamCreateWithFlags(&ctx->host_path_stream, cudaStreamNonBlocking)) != cudaSuccess) return fail_cuda(err, "cudaStreamCreate");
    cudaStream_t stream = ctx->host_path_stream;
    const size_t n = size_t(hs->n_primitives), B = size_t(hs->total_sh_bases), P = size_t(hv->width) * hv->height;
    Carver c(nullptr);
    c.take<float>(n * 3); c.take<float>(n * 3); c.take<float>(n * 4); c.take<float>(n); c.take<float>(n * 3); c.take<float>(n * B * 3);
    c.take<float>(16); c.take<float>(16); c.take<float>(4); c.take<float>(P * 3); c.take<float>(P);
    const size_t need = align_up(c.offset);
    if (need > ctx->host_path_bytes) {
        if (ctx->host_path_buf) cudaFree(ctx->host_path_buf);
        ctx->host_path_buf = nullptr; ctx->host_path_bytes = 0;
        if ((err = cudaMalloc(&ctx->host_path_buf, need)) != cudaSuccess) return fail_cuda(err, "device staging allocation");
        ctx->host_path_bytes = need;
    }
    Carver d(ctx->host_path_buf);
    float* positions = d.take<float>(n * 3); float* scales = d.take<float>(n * 3); float* rotations = d.take<float>(n * 4);
    float* opacities = d.take<float>(n); float* sh_0 = d.take<float>(n * 3); float* sh_rest = d.take<float>(n * B * 3);
    float* M = d.take<float>(16); float* VPM = d.take<float>(16); float* cam = d.take<float>(4);
    float* image = d.take<float>(P * 3); float* depth = d.take<float>(P);
    auto up = [&](float* dst, const float* src, size_t count) -> cudaError_t {
        return count ? cudaMemcpyAsync(dst, src, count * sizeof(float), cudaMemcpyHostToDevice, stream) : cudaSuccess;
    };
    if ((err = up(positions, hs->positions, n * 3)) != cudaSuccess || (err = up(scales, hs->scales, n * 3)) != cudaSuccess ||
        (err = up(rotations, hs->rotations, n * 4)) != cudaSuccess || (err = up(opacities, hs->opacities, n)) != cudaSuccess ||
        (err = up(sh_0, hs->sh_0, n * 3)) != cudaSuccess || (err = up(sh_rest, hs->sh_rest, n * B * 3)) != cudaSuccess ||
        (err = up(M, hv->M, 16)) != cudaSuccess || (err = up(VPM, hv->VPM, 16)) != cudaSuccess || (err = up(cam, hv->cam_position, 3)) != cudaSuccess)
        return fail_cuda(err, "host to device copy");
    HtgsScene ds = *hs;
    ds.positions = positions; ds.scales = scales; ds.rotations = rotations; ds.opacities = opacities; ds.sh_0 = sh_0; ds.sh_rest = sh_rest;
    HtgsView dv = *hv;
    dv.M = M; dv.VPM = VPM; dv.cam_position = cam;
    rc = htgs_render(ctx, &ds, &dv, image, depth, nullptr, to_chw, use_median_depth, nullptr, 0, stream, info);
    if (rc != HTGS_OK) return rc;
    if ((err = cudaMemcpyAsync(host_image, image, P * 3 * sizeof(float), cudaMemcpyDeviceToHost, stream)) != cudaSuccess) return fail_cuda(err, "image copy");
    if ((err = cudaMemcpyAsync(host_depth, depth, P * sizeof(float), cudaMemcpyDeviceToHost, stream)) != cudaSuccess) return fail_cuda(err, "depth copy");
    if ((err = cudaStreamSynchronize(stream)) != cudaSuccess) return fail_cuda(err, "synchronise");
    return HTGS_OK;
}

int htgs_memcpy_d2h(void* host_dst, const void* device_src, size_t bytes) {
    if (bytes == 0) return HTGS_OK;
    const cudaError_t err = cudaMemcpy(host_dst, device_src, bytes, cudaMemcpyDeviceToHost);
    return err == cudaSuccess ? HTGS_OK : fail_cuda(err, "cudaMemcpy D2H");
}

int htgs_memcpy_h2d(void* device_dst, const void* host_src, size_t bytes) {
    if (bytes == 0) return HTGS_OK;
    const cudaError_t err = cudaMemcpy(device_dst, host_src, bytes, cudaMemcpyHostToDevice);
    return err == cudaSuccess ? HTGS_OK : fail_cuda(err, "cudaMemcpy H2D");
}

}  // extern "C"

// ---------------------------------------------------------------------------------------------------
// training forward / backward
// ---------------------------------------------------------------------------------------------------
namespace {

struct PrimLayout { FrameStatus* status; PrimBuffers prim; size_t bytes; };
PrimLayout carve_primitive_blob(void* blob, int n_primitives) {
    PrimLayout L{};
    Carver c(blob);
    const size_t n = size_t(n_primitives);
    const size_t prim_blocks = (n + kPreprocessBlock - 1) / kPreprocessBlock;
    L.status = c.take<FrameStatus>(1);
    L.prim.n_touched = c.take<uint32_t>(n);
    L.prim.bounds = c.take<ushort4>(n);
    L.prim.eval = c.take<EvalRecord>(n);
    L.prim.cull = c.take<CullRecord>(n);
    L.prim.clamp = c.take<uint8_t>(n);
    L.prim.block_sums = c.take<uint32_t>(prim_blocks + 1);
    L.prim.block_offsets = c.take<uint32_t>(prim_blocks + 1);
    L.prim.visible_list = c.take<uint32_t>(n);
    L.bytes = align_up(c.offset);
    return L;
}

struct InstLayout { InstBuffers inst; size_t bytes; };
InstLayout carve_instance_blob(void* blob, const SortPlan& plan, uint64_t capacity) {
    InstLayout L{};
    Carver c(blob);
    const uint64_t cap = capacity > 0xfffffff0ull ? 0xfffffff0ull : capacity;
    L.inst.capacity = uint32_t(cap);
    L.inst.sort_blocks_cap = uint32_t((cap + kSortTile - 1) / kSortTile);
    L.inst.keys[0] = c.take_bytes<void>(size_t(cap) * plan.key_bytes);
    L.inst.keys[1] = c.take_bytes<void>(size_t(cap) * plan.key_bytes);
    L.inst.prims[0] = c.take<uint32_t>(size_t(cap));
    L.inst.prims[1] = c.take<uint32_t>(size_t(cap));
    L.inst.sort_scratch = c.take_bytes<void>(sort_scratch_bytes(plan, L.inst.sort_blocks_cap));
    L.bytes = align_up(c.offset);
    return L;
}

struct PixelLayout { TrainPixelBuffers px; size_t bytes; };
PixelLayout carve_pixel_blob(void* blob, int mode, int K, const FrameGeometry& geo) {
    PixelLayout L{};
    Carver c(blob);
    const size_t PP = size_t(geo.n_tiles) * geo.tile_w * geo.tile_h;
    const size_t k = size_t(effective_k(mode, K));
    L.px.padded_pixels = uint32_t(PP);
    if (mode == HTGS_MODE_HYBRID_BLEND || mode == HTGS_MODE_ALPHA_BLEND_FIRST_K) {
        L.px.idx_core = c.take<uint32_t>(k * PP);
        L.px.info_core = c.take<float4>(k * PP);
    }
    if (mode == HTGS_MODE_HYBRID_BLEND) L.px.info_tail = c.take<float>(6 * PP);
    if (mode == HTGS_MODE_OIT_BLEND) L.px.info_tail = c.take<float>(5 * PP);
    L.bytes = align_up(c.offset + 1);
    return L;
}

}  // namespace

extern "C" {

int htgs_forward_blob_sizes(const HtgsScene* scene, const HtgsView* view, size_t* per_primitive_bytes, size_t* per_tile_bytes, size_t* per_pixel_bytes) {
    const int rc = validate(scene, view);
    if (rc != HTGS_OK) return rc;
    const FrameGeometry geo = make_geometry(view->mode, view->width, view->height);
    if (per_primitive_bytes) *per_primitive_bytes = carve_primitive_blob(nullptr, scene->n_primitives).bytes;
    if (per_tile_bytes) *per_tile_bytes = align_up(sizeof(uint2) * size_t(geo.n_tiles) + 1);
    if (per_pixel_bytes) *per_pixel_bytes = carve_pixel_blob(nullptr, view->mode, view->K, geo).bytes;
    return HTGS_OK;
}

uint64_t htgs_forward_instance_capacity(uint64_t n_instances) {
    if (n_instances <= 4096) return 4096;
    int top = 63;
    while (!(n_instances >> top)) --top;                      // index of the highest set bit
    const uint64_t step = uint64_t(1) << (top - 1);           // two sizes per power of two: 2^k and 1.5 * 2^k
    const uint64_t rounded = (n_instances + step - 1) / step * step;
    return rounded < n_instances ? n_instances : rounded;     // (overflow: cannot happen below 2^60)
}

size_t htgs_forward_instance_bytes(const HtgsView* view, uint64_t n_instances) {
    if (!view || view->mode < 0 || view->mode > 3 || view->width <= 0 || view->height <= 0) return 0;
    const FrameGeometry geo = make_geometry(view->mode, view->width, view->height);
    return carve_instance_blob(nullptr, make_sort_plan(view->mode, geo.n_tiles), n_instances).bytes;
}

int htgs_forward_begin(HtgsContext* ctx, const HtgsScene* scene, const HtgsView* view, void* per_primitive, size_t per_primitive_bytes,
                       void* stream_ptr, uint32_t* n_instances) {
    if (!ctx || !n_instances) return fail(HTGS_ERR_INVALID_ARGUMENT, "null argument");
    int rc = validate(scene, view);
    if (rc != HTGS_OK) return rc;
    DeviceGuard guard(ctx->device);
    if (guard.status != cudaSuccess) return fail_cuda(guard.status, "cudaSetDevice");
    if ((rc = settle_pending(ctx)) != HTGS_OK) return rc;
    const PrimLayout L = carve_primitive_blob(per_primitive, scene->n_primitives);
    if (!per_primitive || per_primitive_bytes < L.bytes) return fail(HTGS_ERR_WORKSPACE_TOO_SMALL, "per-primitive blob too small");
    cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);
    const FrameGeometry geo = make_geometry(view->mode, view->width, view->height);
    cudaError_t err;
    if ((err = cudaMemsetAsync(L.status, 0, sizeof(FrameStatus), stream)) != cudaSuccess) return fail_cuda(err, "status reset");
    if ((err = launch_preprocess(view->mode, true, *scene, *view, geo, L.prim, L.status, stream)) != cudaSuccess) return fail_cuda(err, "preprocess");
    if ((err = launch_scan_only(*scene, L.prim, 0xfffffff0u, L.status, stream)) != cudaSuccess) return fail_cuda(err, "scan");
    if ((err = cudaMemcpyAsync(ctx->host_status, L.status, sizeof(FrameStatus), cudaMemcpyDeviceToHost, stream)) != cudaSuccess) return fail_cuda(err, "status copy");
    if ((err = cudaStreamSynchronize(stream)) != cudaSuccess) return fail_cuda(err, "synchronise");
    if (ctx->host_status->overflow) return fail(HTGS_ERR_INVALID_ARGUMENT, "instance count does not fit 32 bits");
    *n_instances = ctx->host_status->n_instances;
    return HTGS_OK;
}

int htgs_forward_finish(HtgsContext* ctx, const HtgsScene* scene, const HtgsView* view, const HtgsTrainBlobs* blobs, uint32_t n_instances,
                        float* image, void* stream_ptr, HtgsFrameInfo* info) {
    if (!ctx || !blobs || !image) return fail(HTGS_ERR_INVALID_ARGUMENT, "null argument");
    int rc = validate(scene, view);
    if (rc != HTGS_OK) return rc;
    DeviceGuard guard(ctx->device);
    if (guard.status != cudaSuccess) return fail_cuda(guard.status, "cudaSetDevice");
    if ((rc = settle_pending(ctx)) != HTGS_OK) return rc;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);
    const FrameGeometry geo = make_geometry(view->mode, view->width, view->height);
    const SortPlan plan = make_sort_plan(view->mode, geo.n_tiles);
    const PrimLayout P = carve_primitive_blob(blobs->per_primitive, scene->n_primitives);
    const InstLayout I = carve_instance_blob(blobs->per_instance, plan, n_instances);
    const PixelLayout X = carve_pixel_blob(blobs->per_pixel, view->mode, view->K, geo);
    if (!blobs->per_primitive || blobs->per_primitive_bytes < P.bytes || !blobs->per_instance || blobs->per_instance_bytes < I.bytes ||
        !blobs->per_pixel || blobs->per_pixel_bytes < X.bytes || !blobs->per_tile || blobs->per_tile_bytes < sizeof(uint2) * size_t(geo.n_tiles))
        return fail(HTGS_ERR_WORKSPACE_TOO_SMALL, "a forward blob is missing or too small");
    uint2* tile_ranges = static_cast<uint2*>(blobs->per_tile);
    uint32_t launches = 0;
    cudaError_t err;
    if ((err = launch_emit_sort_ranges(view->mode, *scene, geo, plan, P.prim, I.inst, tile_ranges, P.status, ctx->sm_count, stream, nullptr, &launches)) != cudaSuccess)
        return fail_cuda(err, "binning");
    const BlendOutputs out{image, nullptr, nullptr, true, false, false};
    if ((err = launch_blend(view->mode, view->K, true, geo, P.prim, I.inst.prims[plan.final_buffer], tile_ranges, out, X.px, P.status, stream)) != cudaSuccess)
        return fail_cuda(err, "blend");
    if ((err = cudaMemcpyAsync(ctx->host_status, P.status, sizeof(FrameStatus), cudaMemcpyDeviceToHost, stream)) != cudaSuccess) return fail_cuda(err, "status copy");
    if ((err = cudaStreamSynchronize(stream)) != cudaSuccess) return fail_cuda(err, "synchronise");
    const FrameStatus st = *ctx->host_status;
    if (info) {
        std::memset(info, 0, sizeof(*info));
        info->n_instances = st.n_instances; info->n_visible = st.n_visible; info->key_bytes = uint32_t(plan.key_bytes); info->end_bit = uint32_t(plan.end_bit);
        info->device_error = st.error; info->kernel_launches = launches + 4;
    }
    if (st.error) return fail(HTGS_ERR_DEVICE_FLAG, "a kernel reported an internal error (bounded wait gave up)");
    return HTGS_OK;
}

size_t htgs_backward_scratch_bytes(const HtgsScene* scene) {
    return scene ? align_up(size_t(scene->n_primitives > 0 ? scene->n_primitives : 0) * 5 * sizeof(float4) + 1) : 0;
}

int htgs_forward_visibility(const HtgsScene* scene, const HtgsTrainBlobs* blobs, uint8_t* visible, void* stream_ptr) {
    if (!scene || !blobs || (!visible && scene->n_primitives > 0)) return fail(HTGS_ERR_INVALID_ARGUMENT, "null argument");
    if (scene->n_primitives < 0) return fail(HTGS_ERR_INVALID_ARGUMENT, "negative primitive count");
    const PrimLayout P = carve_primitive_blob(blobs->per_primitive, scene->n_primitives);
    if (!blobs->per_primitive || blobs->per_primitive_bytes < P.bytes) return fail(HTGS_ERR_WORKSPACE_TOO_SMALL, "the per-Gaussian forward blob is missing or too small");
    const cudaError_t err = launch_visibility(P.prim.n_touched, visible, uint32_t(scene->n_primitives), static_cast<cudaStream_t>(stream_ptr));
    if (err != cudaSuccess) return fail_cuda(err, "forward visibility");
    return HTGS_OK;
}

int htgs_backward(HtgsContext* ctx, const HtgsScene* scene, const HtgsView* view, const HtgsTrainBlobs* blobs, uint32_t n_instances,
                  const float* grad_image, const float* image, const HtgsGradients* grads, void* stream_ptr) {
    if (!grads) return fail(HTGS_ERR_INVALID_ARGUMENT, "null argument");
    if (!grads->scratch || grads->scratch_bytes < htgs_backward_scratch_bytes(scene)) return fail(HTGS_ERR_WORKSPACE_TOO_SMALL, "backward scratch too small");
    return htgs::backward_with_accum(ctx, scene, view, blobs, n_instances, grad_image, image, grads, grads->scratch, 0,
                                     uint32_t(scene && scene->n_primitives > 0 ? scene->n_primitives : 0), kBackwardAccumulate | kBackwardChainRule, stream_ptr);
}

int htgs_backward_compact(HtgsContext* ctx, const HtgsScene* scene, const HtgsView* view, const HtgsTrainBlobs* blobs, uint32_t n_instances,
                          const float* grad_image, const float* image, const HtgsGradients* grads, void* rows, uint32_t capacity_rows, void* stream_ptr) {
    if (!grads || !rows) return fail(HTGS_ERR_INVALID_ARGUMENT, "null argument");
    if (!grads->scratch || grads->scratch_bytes < htgs_backward_scratch_bytes(scene)) return fail(HTGS_ERR_WORKSPACE_TOO_SMALL, "backward scratch too small");
    return htgs::backward_with_accum(ctx, scene, view, blobs, n_instances, grad_image, image, grads, grads->scratch, 0,
                                     uint32_t(scene && scene->n_primitives > 0 ? scene->n_primitives : 0), kBackwardAccumulate | kBackwardChainRule, stream_ptr,
                                     rows, capacity_rows);
}

int htgs_backward_accumulate(HtgsContext* ctx, const HtgsScene* scene, const HtgsView* view, const HtgsTrainBlobs* blobs, uint32_t n_instances,
                             const float* grad_image, const float* image, const HtgsGradients* grads, void* stream_ptr) {
    if (!grads) return fail(HTGS_ERR_INVALID_ARGUMENT, "null argument");
    if (!grads->scratch || grads->scratch_bytes < htgs_backward_scratch_bytes(scene)) return fail(HTGS_ERR_WORKSPACE_TOO_SMALL, "backward scratch too small");
    return htgs::backward_with_accum(ctx, scene, view, blobs, n_instances, grad_image, image, grads, grads->scratch, 0,
                                     uint32_t(scene && scene->n_primitives > 0 ? scene->n_primitives : 0), kBackwardAccumulate, stream_ptr);
}

int htgs_backward_finish_range(HtgsContext* ctx, const HtgsScene* scene, const HtgsView* view, const HtgsTrainBlobs* blobs, const HtgsGradients* grads,
                               uint32_t first_gaussian, uint32_t n_gaussians, void* stream_ptr) {
    if (!grads || !scene) return fail(HTGS_ERR_INVALID_ARGUMENT, "null argument");
    if (!grads->scratch || grads->scratch_bytes < htgs_backward_scratch_bytes(scene)) return fail(HTGS_ERR_WORKSPACE_TOO_SMALL, "backward scratch too small");
    if (scene->n_primitives < 0 || uint64_t(first_gaussian) + uint64_t(n_gaussians) > uint64_t(scene->n_primitives))
        return fail(HTGS_ERR_INVALID_ARGUMENT, "the range of Gaussians reaches beyond the scene");
    static const float unused = 0.0f;      // the chain rule reads neither the image gradient nor the image
    return htgs::backward_with_accum(ctx, scene, view, blobs, 0, &unused, &unused, grads, grads->scratch, first_gaussian, n_gaussians, kBackwardChainRule, stream_ptr);
}

int htgs_backward_range(HtgsContext* ctx, const HtgsScene* scene, const HtgsView* view, const HtgsTrainBlobs* blobs, uint32_t n_instances,
                        const float* grad_image, const float* image, const HtgsGradients* grads, uint32_t first_gaussian, uint32_t n_gaussians,
                        void* stream_ptr) {
    if (!grads || !scene) return fail(HTGS_ERR_INVALID_ARGUMENT, "null argument");
    if (!grads->scratch || grads->scratch_bytes < htgs_backward_scratch_bytes(scene)) return fail(HTGS_ERR_WORKSPACE_TOO_SMALL, "backward scratch too small");
    if (scene->n_primitives < 0 || uint64_t(first_gaussian) + uint64_t(n_gaussians) > uint64_t(scene->n_primitives))
        return fail(HTGS_ERR_INVALID_ARGUMENT, "the range of Gaussians reaches beyond the scene");
    if (view && view->mode == HTGS_MODE_ALPHA_BLEND_GLOBAL_ORDERING && !(first_gaussian == 0 && n_gaussians == uint32_t(scene->n_primitives)))
        return fail(HTGS_ERR_UNSUPPORTED_MODE, "ALPHA_BLEND_GLOBAL_ORDERING cannot run its backward pass over a part of the Gaussians");
    return htgs::backward_with_accum(ctx, scene, view, blobs, n_instances, grad_image, image, grads, grads->scratch, first_gaussian, n_gaussians,
                                     kBackwardAccumulate | kBackwardChainRule, stream_ptr);
}

}  // extern "C"

int htgs::backward_with_accum(HtgsContext* ctx, const HtgsScene* scene, const HtgsView* view, const HtgsTrainBlobs* blobs, uint32_t n_instances,
                             const float* grad_image, const float* image, const HtgsGradients* grads, void* accum_ptr, uint32_t first, uint32_t count,
                             int stages, void* stream_ptr, void* compact_rows, uint32_t compact_capacity) {
    if (!ctx || !blobs || !grads || !grad_image || !accum_ptr) return fail(HTGS_ERR_INVALID_ARGUMENT, "null argument");
    int rc = validate(scene, view);
    if (rc != HTGS_OK) return rc;
    DeviceGuard guard(ctx->device);
    if (guard.status != cudaSuccess) return fail_cuda(guard.status, "cudaSetDevice");
    if (view->mode == HTGS_MODE_ALPHA_BLEND_GLOBAL_ORDERING && !image) return fail(HTGS_ERR_INVALID_ARGUMENT, "ALPHA_BLEND_GLOBAL_ORDERING needs the forward image");
    if (compact_rows && (reinterpret_cast<uintptr_t>(compact_rows) & 15u) != 0) return fail(HTGS_ERR_INVALID_ARGUMENT, "the compact row buffer must be 16-byte aligned");
    const bool dense_given = grads->grad_positions || grads->grad_scales || grads->grad_rotations || grads->grad_opacities || grads->grad_sh_0 || grads->grad_sh_rest;
    if ((!compact_rows || dense_given) && scene->n_primitives > 0 && (!grads->grad_positions || !grads->grad_scales || !grads->grad_rotations || !grads->grad_opacities || !grads->grad_sh_0 ||
                                    (scene->total_sh_bases > 0 && !grads->grad_sh_rest)))
        return fail(HTGS_ERR_INVALID_ARGUMENT, "gradient output pointers must not be null");
    if (grads->densification_info && grads->densification_rows != 2 && grads->densification_rows != 3)
        return fail(HTGS_ERR_INVALID_ARGUMENT, "densification_info must have 2 or 3 rows");
    cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);
    const FrameGeometry geo = make_geometry(view->mode, view->width, view->height);
    const SortPlan plan = make_sort_plan(view->mode, geo.n_tiles);
    const PrimLayout P = carve_primitive_blob(blobs->per_primitive, scene->n_primitives);
    const InstLayout I = carve_instance_blob(blobs->per_instance, plan, n_instances);
    const PixelLayout X = carve_pixel_blob(blobs->per_pixel, view->mode, view->K, geo);
    const bool accumulate = (stages & kBackwardAccumulate) != 0;      // the chain rule alone reads the per-Gaussian blob only
    if (!blobs->per_primitive || blobs->per_primitive_bytes < P.bytes ||
        (accumulate && (!blobs->per_instance || blobs->per_instance_bytes < I.bytes || !blobs->per_pixel || blobs->per_pixel_bytes < X.bytes || !blobs->per_tile)))
        return fail(HTGS_ERR_WORKSPACE_TOO_SMALL, "a forward blob is missing or too small");
    const GradAccumBuffers acc{static_cast<float4*>(accum_ptr)};
    BackwardOutputs out{grads->grad_positions, grads->grad_scales, grads->grad_rotations, grads->grad_opacities, grads->grad_sh_0, grads->grad_sh_rest,
                        grads->densification_info, grads->densification_info ? grads->densification_rows : 0, grads->use_distance_scaling != 0};
    out.compact_rows = static_cast<float4*>(compact_rows);
    out.compact_capacity = compact_capacity;
    // The six gradient tensors are only written after the per-tile kernel (2 ms of arithmetic), so they are cleared (0.7 GB at
    // configuration 2) on the context's side stream meanwhile, ordered after whatever the caller queued before this call.
    cudaEvent_t outputs_cleared = nullptr;
    if (ctx->front_priority && count > 0 && accumulate && (!compact_rows || dense_given)) {
        cudaError_t e;
        if ((e = cudaEventRecord(ctx->front_begin, stream)) != cudaSuccess) return fail_cuda(e, "front event record");
        if ((e = cudaStreamWaitEvent(ctx->front_stream, ctx->front_begin, 0)) != cudaSuccess) return fail_cuda(e, "front stream wait");
        if ((e = clear_backward_outputs(*scene, out, first, count, ctx->front_stream)) != cudaSuccess) return fail_cuda(e, "clearing the gradient tensors");
        if ((e = cudaEventRecord(ctx->front_end, ctx->front_stream)) != cudaSuccess) return fail_cuda(e, "front event record");
        outputs_cleared = ctx->front_end;
    }
    const cudaError_t err = launch_backward(view->mode, view->K, *scene, *view, geo, P.prim, I.inst.prims[plan.final_buffer], static_cast<const uint2*>(blobs->per_tile),
                                            X.px, grad_image, image, acc, out, outputs_cleared, ctx->sm_count, first, count, stages, stream);
    if (err != cudaSuccess) return fail_cuda(err, "backward");
    return HTGS_OK;
}
