// The torch / pybind layer: extension modules `_C` and `_C_benchmarking` with the reference's function names, argument
// order and return values (torch_bindings/bindings.cpp:8-16, torch_bindings/bindings_benchmarking.cpp:6-8 of the
// reference; signatures rasterization/include/rasterization_api.h:8-97, rasterization/include/fast_inference_api.h:7-25,
// filter3d/include/filter3d_api.h:7-20), so that the reference's own Python surface (torch_bindings/rasterization.py,
// filter3d.py) runs on them unchanged.  PyTorch appears only here: outputs and the opaque blobs are torch tensors, the
// stream is torch's current stream, inputs are validated with TORCH_CHECK before anything is launched (the reference checks
// nothing: rasterization/src/rasterization_api.cu:80-88).  All work is done by the C-ABI library (include/htgs_b200.h).
//
// One source, two modules: compiled with -DHTGS_BINDINGS_BENCHMARKING it defines `_C_benchmarking` (`benchmark` only).
// Beyond the reference's five functions `_C` carries what this library's own surface needs (no counterpart in the
// reference): the last frame's statistics, the non-blocking render mode, the HYBRID max-weight switch, the visibility of
// a training forward, and the context handles, so that the ctypes binding and this one share one set of contexts.
#include <torch/extension.h>

#include <ATen/cuda/CUDAEvent.h>
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>

#include <atomic>
#include <map>
#include <memory>
#include <mutex>
#include <tuple>
#include <vector>

#include "../../include/htgs_b200.h"

namespace {

using torch::Tensor;

std::atomic<bool> g_deferred_checks{false};
std::atomic<bool> g_max_weights_tail_credit{false};
std::atomic<bool> g_track_visibility{false};
std::atomic<bool> g_accumulate_visibility{false};   // OR the masks of successive training forwards until reset (several forwards per step)

// One library context per (device, host thread, stream key): a context owns its workspace and pinned status word, so two
// frames in flight at once must not share one.  Blocking calls use stream key 0, the non-blocking mode the stream's handle.
struct ThreadState {
    std::map<std::pair<int, uintptr_t>, HtgsContext*> contexts;
    std::map<HtgsContext*, std::vector<Tensor>> queued;     // tensors of frames queued without a wait, kept alive until their check
    HtgsFrameInfo last_info{};
};
thread_local ThreadState tls;

HtgsContext* context_for(int device, uintptr_t stream_key) {
    auto key = std::make_pair(device, stream_key);
    auto it = tls.contexts.find(key);
    if (it != tls.contexts.end()) return it->second;
    HtgsContext* ctx = htgs_create(device);
    TORCH_CHECK(ctx != nullptr, "htgs_create(", device, ") failed: ", htgs_last_error());
    tls.contexts[key] = ctx;
    return ctx;
}

void check(int rc) {
    if (rc == HTGS_OK) return;
    if (rc == HTGS_ERR_UNSUPPORTED_MODE) throw std::runtime_error("unsupported rasterizer mode");   // the reference's message
    TORCH_CHECK(false, "htgs_b200 error ", rc, ": ", htgs_last_error());
}

struct VisibilityRecord { Tensor visible; std::shared_ptr<at::cuda::CUDAEvent> ready; };
std::mutex g_visibility_mutex;
std::map<int, VisibilityRecord> g_visibility;   // per device: what the last tracked training forward kept

void check_float_cuda(const Tensor& t, const char* name, const c10::Device& device) {
    TORCH_CHECK_TYPE(t.defined(), name, " must be a tensor");
    TORCH_CHECK_TYPE(t.scalar_type() == torch::kFloat32, name, " must be float32, got ", t.scalar_type());
    TORCH_CHECK_VALUE(t.device() == device, name, " is on ", t.device(), ", expected ", device);
}

struct SceneArgs {
    Tensor positions, scales, rotations, opacities, sh_0, sh_rest, M, VPM, cam_position;   // contiguous copies where needed
    HtgsScene scene{};
    HtgsView view{};
    c10::Device device{c10::kCUDA, 0};
    int64_t n = 0;
};

SceneArgs make_scene(const Tensor& positions, const Tensor& scales, const Tensor& rotations, const Tensor& opacities, const Tensor& sh_0,
                     const Tensor& sh_rest, const Tensor& M, const Tensor& VPM, const Tensor& cam_position, int mode, int K, int active_sh_bases,
                     int width, int height, float near_plane, float far_plane, float scale_modifier, bool with_colour = true) {
    SceneArgs a;
    TORCH_CHECK_VALUE(positions.defined() && positions.is_cuda(), "htgs_b200 rasterizer: tensors must live on a CUDA device");
    a.device = positions.device();
    a.n = positions.dim() >= 1 ? positions.size(0) : -1;
    check_float_cuda(positions, "positions", a.device); check_float_cuda(scales, "scales", a.device);
    check_float_cuda(rotations, "rotations", a.device); check_float_cuda(opacities, "opacities", a.device);
    check_float_cuda(M, "M", a.device); check_float_cuda(VPM, "VPM", a.device); check_float_cuda(cam_position, "cam_position", a.device);
    TORCH_CHECK_VALUE(positions.dim() == 2 && positions.size(1) == 3, "positions must have shape (N, 3)");
    TORCH_CHECK_VALUE(scales.dim() == 2 && scales.size(0) == a.n && scales.size(1) == 3, "scales must have shape (N, 3)");
    TORCH_CHECK_VALUE(rotations.dim() == 2 && rotations.size(0) == a.n && rotations.size(1) == 4, "rotations must have shape (N, 4)");
    TORCH_CHECK_VALUE(opacities.numel() == a.n, "opacities must hold N values");
    TORCH_CHECK_VALUE(M.dim() == 2 && M.size(0) == 4 && M.size(1) == 4, "M must have shape (4, 4)");
    TORCH_CHECK_VALUE(VPM.dim() == 2 && VPM.size(0) == 4 && VPM.size(1) == 4, "VPM must have shape (4, 4)");
    TORCH_CHECK_VALUE(cam_position.numel() == 3, "cam_position must have shape (3,)");
    a.positions = positions.contiguous(); a.scales = scales.contiguous(); a.rotations = rotations.contiguous(); a.opacities = opacities.contiguous();
    a.M = M.contiguous(); a.VPM = VPM.contiguous(); a.cam_position = cam_position.contiguous();
    int total_sh = 0;
    if (with_colour) {
        check_float_cuda(sh_0, "sh_0", a.device); check_float_cuda(sh_rest, "sh_rest", a.device);
        TORCH_CHECK_VALUE(sh_0.numel() == 3 * a.n, "sh_0 must have shape (N, 1, 3)");
        TORCH_CHECK_VALUE(sh_rest.dim() == 3 && sh_rest.size(0) == a.n && sh_rest.size(2) == 3, "sh_rest must have shape (N, B, 3)");
        a.sh_0 = sh_0.contiguous(); a.sh_rest = sh_rest.contiguous();
        total_sh = int(sh_rest.size(1));
    }
    a.scene.positions = a.positions.data_ptr<float>(); a.scene.scales = a.scales.data_ptr<float>();
    a.scene.rotations = a.rotations.data_ptr<float>(); a.scene.opacities = a.opacities.data_ptr<float>();
    a.scene.sh_0 = with_colour ? a.sh_0.data_ptr<float>() : nullptr;
    a.scene.sh_rest = (with_colour && a.sh_rest.numel() > 0) ? a.sh_rest.data_ptr<float>() : nullptr;
    a.scene.n_primitives = int32_t(a.n); a.scene.total_sh_bases = total_sh;
    a.view.M = a.M.data_ptr<float>(); a.view.VPM = a.VPM.data_ptr<float>(); a.view.cam_position = a.cam_position.data_ptr<float>();
    a.view.mode = mode; a.view.K = K; a.view.active_sh_bases = active_sh_bases; a.view.width = width; a.view.height = height;
    a.view.near_plane = near_plane; a.view.far_plane = far_plane; a.view.scale_modifier = scale_modifier;
    return a;
}

Tensor bytes_on(const c10::Device& device, size_t count) {
    return torch::empty({int64_t(count)}, torch::TensorOptions().dtype(torch::kByte).device(device));
}

// ---- `_C_benchmarking.benchmark` = fast_inference_wrapper (rasterization/include/fast_inference_api.h:7-25) ----------------
Tensor benchmark(const Tensor& positions, const Tensor& scales, const Tensor& rotations, const Tensor& opacities, const Tensor& sh_0,
                 const Tensor& sh_rest, const Tensor& M, const Tensor& VPM, const Tensor& cam_position, const int rasterizer_mode, const int K,
                 const int active_sh_bases, const int width, const int height, const float near_plane, const float far_plane,
                 const float scale_modifier, const bool to_chw) {
    SceneArgs a = make_scene(positions, scales, rotations, opacities, sh_0, sh_rest, M, VPM, cam_position, rasterizer_mode, K, active_sh_bases, width,
                             height, near_plane, far_plane, scale_modifier);
    const c10::cuda::CUDAGuard guard(a.device);
    const auto f32 = torch::TensorOptions().dtype(torch::kFloat32).device(a.device);
    Tensor image = to_chw ? torch::empty({3, height, width}, f32) : torch::empty({height, width, 3}, f32);
    cudaStream_t stream = c10::cuda::getCurrentCUDAStream(a.device.index()).stream();
    if (g_deferred_checks.load()) {
        HtgsContext* ctx = context_for(a.device.index(), reinterpret_cast<uintptr_t>(stream));
        const int rc = htgs_render_fast_async(ctx, &a.scene, &a.view, image.data_ptr<float>(), to_chw ? 1 : 0, stream);
        tls.queued[ctx] = {a.positions, a.scales, a.rotations, a.opacities, a.sh_0, a.sh_rest, a.M, a.VPM, a.cam_position, image};
        check(rc);
        return image;
    }
    HtgsFrameInfo info{};
    const int rc = htgs_render_fast(context_for(a.device.index(), 0), &a.scene, &a.view, image.data_ptr<float>(), to_chw ? 1 : 0, nullptr, 0, stream, &info);
    check(rc);
    tls.last_info = info;
    return image;
}

#ifndef HTGS_BINDINGS_BENCHMARKING

// ---- `_C.render` = inference_wrapper (rasterization/include/rasterization_api.h:57-77) -----------------------------------
std::tuple<Tensor, Tensor> render(const Tensor& positions, const Tensor& scales, const Tensor& rotations, const Tensor& opacities, const Tensor& sh_0,
                                  const Tensor& sh_rest, const Tensor& M, const Tensor& VPM, const Tensor& cam_position, const int rasterizer_mode,
                                  const int K, const int active_sh_bases, const int width, const int height, const float near_plane,
                                  const float far_plane, const float scale_modifier, const bool to_chw, const bool use_median_depth) {
    SceneArgs a = make_scene(positions, scales, rotations, opacities, sh_0, sh_rest, M, VPM, cam_position, rasterizer_mode, K, active_sh_bases, width,
                             height, near_plane, far_plane, scale_modifier);
    const c10::cuda::CUDAGuard guard(a.device);
    const auto f32 = torch::TensorOptions().dtype(torch::kFloat32).device(a.device);
    Tensor image = to_chw ? torch::empty({3, height, width}, f32) : torch::empty({height, width, 3}, f32);
    Tensor depth = torch::empty({height, width}, f32);
    cudaStream_t stream = c10::cuda::getCurrentCUDAStream(a.device.index()).stream();
    if (g_deferred_checks.load()) {
        HtgsContext* ctx = context_for(a.device.index(), reinterpret_cast<uintptr_t>(stream));
        const int rc = htgs_render_async(ctx, &a.scene, &a.view, image.data_ptr<float>(), depth.data_ptr<float>(), nullptr, to_chw ? 1 : 0,
                                         use_median_depth ? 1 : 0, stream);
        tls.queued[ctx] = {a.positions, a.scales, a.rotations, a.opacities, a.sh_0, a.sh_rest, a.M, a.VPM, a.cam_position, image, depth};
        check(rc);
        return {image, depth};
    }
    HtgsFrameInfo info{};
    const int rc = htgs_render(context_for(a.device.index(), 0), &a.scene, &a.view, image.data_ptr<float>(), depth.data_ptr<float>(), nullptr,
                               to_chw ? 1 : 0, use_median_depth ? 1 : 0, nullptr, 0, stream, &info);
    check(rc);
    tls.last_info = info;
    return {image, depth};
}

// ---- `_C.forward` = forward_wrapper (rasterization/include/rasterization_api.h:8-26) --------------------------------------
// The four byte tensors are opaque to the caller and only meaningful to `backward` of this module, as in the reference.
std::tuple<Tensor, Tensor, Tensor, Tensor, Tensor, int, int> forward(
    const Tensor& positions, const Tensor& scales, const Tensor& rotations, const Tensor& opacities, const Tensor& sh_0, const Tensor& sh_rest,
    const Tensor& M, const Tensor& VPM, const Tensor& cam_position, const int rasterizer_mode, const int K, const int active_sh_bases, const int width,
    const int height, const float near_plane, const float far_plane, const float scale_modifier) {
    (void)scale_modifier;   // the reference's training forward ignores it (treated as 1)
    SceneArgs a = make_scene(positions, scales, rotations, opacities, sh_0, sh_rest, M, VPM, cam_position, rasterizer_mode, K, active_sh_bases, width,
                             height, near_plane, far_plane, 1.0f);
    const c10::cuda::CUDAGuard guard(a.device);
    HtgsContext* ctx = context_for(a.device.index(), 0);
    size_t pp_bytes = 0, pt_bytes = 0, px_bytes = 0;
    check(htgs_forward_blob_sizes(&a.scene, &a.view, &pp_bytes, &pt_bytes, &px_bytes));
    Tensor per_primitive = bytes_on(a.device, pp_bytes), per_tile = bytes_on(a.device, pt_bytes), per_pixel = bytes_on(a.device, px_bytes);
    Tensor image = torch::empty({3, height, width}, torch::TensorOptions().dtype(torch::kFloat32).device(a.device));
    const c10::cuda::CUDAStream torch_stream = c10::cuda::getCurrentCUDAStream(a.device.index());
    cudaStream_t stream = torch_stream.stream();
    uint32_t n_instances = 0;
    check(htgs_forward_begin(ctx, &a.scene, &a.view, per_primitive.data_ptr(), pp_bytes, stream, &n_instances));
    if (g_track_visibility.load()) {   // before the rest of the forward is queued: the list is final and the stream is idle here
        Tensor visible = torch::empty({a.n}, torch::TensorOptions().dtype(torch::kBool).device(a.device));
        HtgsTrainBlobs head{};
        head.per_primitive = per_primitive.data_ptr(); head.per_primitive_bytes = pp_bytes;
        check(htgs_forward_visibility(&a.scene, &head, reinterpret_cast<uint8_t*>(visible.data_ptr()), stream));
        auto ready = std::make_shared<at::cuda::CUDAEvent>();
        std::lock_guard<std::mutex> lock(g_visibility_mutex);
        auto earlier = g_visibility.find(a.device.index());
        if (g_accumulate_visibility.load() && earlier != g_visibility.end() && earlier->second.visible.sizes() == visible.sizes())
            visible.logical_or_(earlier->second.visible);      // a row any forward of the step kept can be non-zero
        ready->record(torch_stream);
        g_visibility[a.device.index()] = VisibilityRecord{visible, ready};
    }
    // The instance count changes from view to view; exact sizes would miss torch's block cache on every heavier view, and the
    // allocator would carve the request out of some other tensor's cached block.  So: two sizes per power of two, and never
    // smaller than the largest size this device has needed so far (unless that is over four times too much: another scene) -
    // the same request step after step.
    static std::atomic<uint64_t> largest_capacity[64];
    uint64_t capacity = htgs_forward_instance_capacity(n_instances);
    if (a.device.index() >= 0 && a.device.index() < 64) {
        std::atomic<uint64_t>& seen = largest_capacity[a.device.index()];
        uint64_t before = seen.load();
        while (before < capacity && !seen.compare_exchange_weak(before, capacity)) {}
        if (before > capacity && before <= 4 * capacity) capacity = before;
    }
    const size_t pi_bytes = htgs_forward_instance_bytes(&a.view, capacity);
    Tensor per_instance = bytes_on(a.device, pi_bytes);
    HtgsTrainBlobs blobs{per_primitive.data_ptr(), pp_bytes, per_tile.data_ptr(), pt_bytes, per_instance.data_ptr(), pi_bytes, per_pixel.data_ptr(), px_bytes};
    HtgsFrameInfo info{};
    check(htgs_forward_finish(ctx, &a.scene, &a.view, &blobs, n_instances, image.data_ptr<float>(), stream, &info));
    tls.last_info = info;
    return {image, per_primitive, per_tile, per_instance, per_pixel, int(n_instances), 0};
}

// ---- `_C.backward` = backward_wrapper (rasterization/include/rasterization_api.h:28-55) ------------------------------------
// `image` / `opacities` may be empty tensors, as the reference's autograd function passes them (torch_bindings/rasterization.py:72-76).
std::tuple<Tensor, Tensor, Tensor, Tensor, Tensor, Tensor> backward(
    Tensor& densification_info, const Tensor& grad_image, const Tensor& image, const Tensor& positions, const Tensor& scales, const Tensor& rotations,
    const Tensor& opacities, const Tensor& sh_rest, const Tensor& per_primitive_buffers, const Tensor& per_tile_buffers,
    const Tensor& per_instance_buffers, const Tensor& per_pixel_buffers, const Tensor& M, const Tensor& VPM, const Tensor& cam_position,
    const int rasterizer_mode, const int K, const int active_sh_bases, const int width, const int height, const float near_plane, const float far_plane,
    const float scale_modifier, const int n_instances, const int instance_primitive_indices_selector, const bool use_distance_scaling) {
    (void)opacities; (void)scale_modifier; (void)instance_primitive_indices_selector;
    TORCH_CHECK_VALUE(positions.defined() && positions.is_cuda(), "htgs_b200 rasterizer: tensors must live on a CUDA device");
    const c10::Device device = positions.device();
    check_float_cuda(grad_image, "grad_image", device); check_float_cuda(positions, "positions", device); check_float_cuda(scales, "scales", device);
    check_float_cuda(rotations, "rotations", device); check_float_cuda(sh_rest, "sh_rest", device);
    check_float_cuda(M, "M", device); check_float_cuda(VPM, "VPM", device); check_float_cuda(cam_position, "cam_position", device);
    TORCH_CHECK(grad_image.dim() == 3 && grad_image.size(0) == 3 && grad_image.size(1) == height && grad_image.size(2) == width,
                "grad_image must have shape (3, ", height, ", ", width, ")");
    TORCH_CHECK_VALUE(sh_rest.dim() == 3, "sh_rest must have shape (N, B, 3)");
    const int64_t n = positions.size(0), total_sh = sh_rest.size(1);
    const c10::cuda::CUDAGuard guard(device);
    const Tensor g = grad_image.contiguous(), pos = positions.contiguous(), scl = scales.contiguous(), rot = rotations.contiguous(), shr = sh_rest.contiguous();
    const Tensor Mc = M.contiguous(), VPMc = VPM.contiguous(), camc = cam_position.contiguous();
    const Tensor img = image.numel() ? image.contiguous() : image;
    const auto f32 = torch::TensorOptions().dtype(torch::kFloat32).device(device);
    Tensor grad_positions = torch::empty({n, 3}, f32), grad_scales = torch::empty({n, 3}, f32), grad_rotations = torch::empty({n, 4}, f32);
    Tensor grad_opacities = torch::empty({n, 1}, f32), grad_sh_0 = torch::empty({n, 1, 3}, f32), grad_sh_rest = torch::empty({n, total_sh, 3}, f32);
    // opacities / sh_0 are not read by the backward kernels (the forward's records hold what is needed)
    HtgsScene scene{pos.data_ptr<float>(), scl.data_ptr<float>(), rot.data_ptr<float>(), pos.data_ptr<float>(), pos.data_ptr<float>(),
                    shr.numel() ? shr.data_ptr<float>() : nullptr, int32_t(n), int32_t(total_sh)};
    HtgsView view{Mc.data_ptr<float>(), VPMc.data_ptr<float>(), camc.data_ptr<float>(), rasterizer_mode, K, active_sh_bases, width, height, near_plane,
                  far_plane, 1.0f};
    Tensor scratch = bytes_on(device, htgs_backward_scratch_bytes(&scene));
    int rows = 0;
    if (densification_info.numel() > 0) {
        rows = int(densification_info.size(0));
        TORCH_CHECK(rows == 2 || rows == 3, "densification_info must be empty or have 2 or 3 rows");
        TORCH_CHECK(densification_info.scalar_type() == torch::kFloat32 && densification_info.device() == device && densification_info.is_contiguous() &&
                        densification_info.numel() == int64_t(rows) * n,
                    "densification_info must be a contiguous float32 tensor of shape [rows, N, 1] on the same device");
    }
    HtgsGradients grads{};
    grads.grad_positions = grad_positions.data_ptr<float>(); grads.grad_scales = grad_scales.data_ptr<float>();
    grads.grad_rotations = grad_rotations.data_ptr<float>(); grads.grad_opacities = grad_opacities.data_ptr<float>();
    grads.grad_sh_0 = grad_sh_0.data_ptr<float>(); grads.grad_sh_rest = grad_sh_rest.numel() ? grad_sh_rest.data_ptr<float>() : nullptr;
    grads.scratch = scratch.data_ptr(); grads.scratch_bytes = size_t(scratch.numel());
    grads.densification_info = rows ? densification_info.data_ptr<float>() : nullptr;
    grads.densification_rows = rows; grads.use_distance_scaling = use_distance_scaling ? 1 : 0;
    HtgsTrainBlobs blobs{per_primitive_buffers.data_ptr(), size_t(per_primitive_buffers.numel()), per_tile_buffers.data_ptr(), size_t(per_tile_buffers.numel()),
                         per_instance_buffers.data_ptr(), size_t(per_instance_buffers.numel()), per_pixel_buffers.data_ptr(), size_t(per_pixel_buffers.numel())};
    cudaStream_t stream = c10::cuda::getCurrentCUDAStream(device.index()).stream();
    check(htgs_backward(context_for(device.index(), 0), &scene, &view, &blobs, uint32_t(n_instances), g.data_ptr<float>(),
                        img.numel() ? img.data_ptr<float>() : nullptr, &grads, stream));
    return {grad_positions, grad_scales, grad_rotations, grad_opacities, grad_sh_0, grad_sh_rest};
}

// ---- `_C.update_max_weights` = update_max_weights_wrapper (rasterization/include/rasterization_api.h:79-97) -----------------
void update_max_weights(Tensor& max_weights, const Tensor& positions, const Tensor& scales, const Tensor& rotations, const Tensor& opacities,
                        const Tensor& M, const Tensor& VPM, const Tensor& cam_position, const int rasterizer_mode, const int K, const int active_sh_bases,
                        const int width, const int height, const float near_plane, const float far_plane, const float scale_modifier,
                        const float weight_threshold) {
    SceneArgs a = make_scene(positions, scales, rotations, opacities, Tensor(), Tensor(), M, VPM, cam_position, rasterizer_mode, K, active_sh_bases, width,
                             height, near_plane, far_plane, scale_modifier, false);
    check_float_cuda(max_weights, "max_weights", a.device);
    TORCH_CHECK(max_weights.numel() == a.n && max_weights.is_contiguous(), "max_weights is updated in place and must be a contiguous tensor of N values");
    const c10::cuda::CUDAGuard guard(a.device);
    HtgsContext* ctx = context_for(a.device.index(), 0);
    check(htgs_set_max_weights_tail_credit(ctx, g_max_weights_tail_credit.load() ? 1 : 0));
    HtgsFrameInfo info{};
    check(htgs_update_max_weights(ctx, &a.scene, &a.view, max_weights.data_ptr<float>(), weight_threshold, nullptr, 0,
                                  c10::cuda::getCurrentCUDAStream(a.device.index()).stream(), &info));
    tls.last_info = info;
}

// ---- `_C.update_3d_filter_cuda` = update_3d_filter_wrapper (filter3d/include/filter3d_api.h:7-20) -----------------------------
void update_3d_filter_cuda(const Tensor& positions, const Tensor& w2c, Tensor& filter_3d, Tensor& visibility_mask, const int width, const int height,
                           const float focal_x, const float focal_y, const float center_x, const float center_y, const float near_plane,
                           const float clipping_tolerance, const float distance2filter) {
    TORCH_CHECK_VALUE(positions.defined() && positions.is_cuda(), "htgs_b200: tensors must live on a CUDA device");
    const c10::Device device = positions.device();
    check_float_cuda(positions, "positions", device); check_float_cuda(w2c, "w2c", device); check_float_cuda(filter_3d, "filter_3d", device);
    TORCH_CHECK(visibility_mask.scalar_type() == torch::kBool && visibility_mask.device() == device, "visibility_mask must be a bool tensor on the same device");
    const int64_t n = positions.size(0);
    TORCH_CHECK(positions.dim() == 2 && positions.size(1) == 3 && w2c.numel() == 16 && filter_3d.numel() == n && visibility_mask.numel() == n,
                "expected positions [N,3], w2c [4,4], filter_3d [N,1], visibility_mask [N]");
    TORCH_CHECK(filter_3d.is_contiguous() && visibility_mask.is_contiguous(), "filter_3d and visibility_mask are updated in place and must be contiguous");
    const Tensor pos = positions.contiguous(), mat = w2c.contiguous();
    const c10::cuda::CUDAGuard guard(device);
    check(htgs_update_3d_filter(pos.data_ptr<float>(), mat.data_ptr<float>(), filter_3d.data_ptr<float>(), reinterpret_cast<uint8_t*>(visibility_mask.data_ptr()),
                                int32_t(n), width, height, focal_x, focal_y, center_x, center_y, near_plane, clipping_tolerance, distance2filter,
                                c10::cuda::getCurrentCUDAStream(device.index()).stream()));
}

// ---- what this library's own surface adds ---------------------------------------------------------------------------------------
std::vector<HtgsFrameInfo> frame_results(int device) {
    std::vector<HtgsFrameInfo> infos;
    for (auto& entry : tls.contexts) {
        if (device >= 0 && entry.first.first != device) continue;
        auto q = tls.queued.find(entry.second);
        if (q == tls.queued.end()) continue;
        HtgsFrameInfo info{};
        const int rc = htgs_frame_result(entry.second, &info);
        tls.queued.erase(q);
        check(rc);
        infos.push_back(info);
        tls.last_info = info;
    }
    return infos;
}

struct ReadyEvent {     // what `torch.cuda.Stream.wait_event` needs: an object with wait(stream)
    std::shared_ptr<at::cuda::CUDAEvent> event;
    void wait(const py::object& stream) const {
        const uintptr_t handle = stream.attr("cuda_stream").cast<uintptr_t>();
        const int device = stream.attr("device").attr("index").cast<int>();
        event->block(c10::cuda::getStreamFromExternal(reinterpret_cast<cudaStream_t>(handle), c10::DeviceIndex(device)));
    }
    void synchronize() const { event->synchronize(); }
};

#endif  // !HTGS_BINDINGS_BENCHMARKING

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
#ifdef HTGS_BINDINGS_BENCHMARKING
    m.def("benchmark", &benchmark);
#else
    m.def("update_3d_filter_cuda", &update_3d_filter_cuda);
    m.def("forward", &forward);
    m.def("backward", &backward);
    m.def("render", &render);
    m.def("update_max_weights", &update_max_weights);
    // no counterparts in the reference below this line
    m.def("benchmark", &benchmark);
    py::class_<HtgsFrameInfo>(m, "FrameInfo")
        .def_readonly("n_instances", &HtgsFrameInfo::n_instances).def_readonly("n_visible", &HtgsFrameInfo::n_visible)
        .def_readonly("key_bytes", &HtgsFrameInfo::key_bytes).def_readonly("end_bit", &HtgsFrameInfo::end_bit)
        .def_readonly("reruns", &HtgsFrameInfo::reruns).def_readonly("device_error", &HtgsFrameInfo::device_error)
        .def_readonly("kernel_launches", &HtgsFrameInfo::kernel_launches).def_readonly("workspace_bytes", &HtgsFrameInfo::workspace_bytes)
        .def_readonly("candidate_pairs", &HtgsFrameInfo::candidate_pairs).def_readonly("accepted_fragments", &HtgsFrameInfo::accepted_fragments)
        .def_readonly("warp_trips", &HtgsFrameInfo::warp_trips).def_readonly("warp_trips_inserting", &HtgsFrameInfo::warp_trips_inserting)
        .def_readonly("lane_insertions", &HtgsFrameInfo::lane_insertions);
    py::class_<ReadyEvent>(m, "ReadyEvent").def("wait", &ReadyEvent::wait).def("synchronize", &ReadyEvent::synchronize);
    m.def("frame_info", [] { return tls.last_info; }, "statistics of the calling thread's most recent frame");
    m.def("set_deferred_checks", [](bool enable) { if (!enable) frame_results(-1); g_deferred_checks.store(enable); });
    m.def("deferred_checks", [] { return g_deferred_checks.load(); });
    m.def("frame_results", &frame_results, py::arg("device") = -1);
    m.def("set_max_weights_tail_credit", [](bool enable) { g_max_weights_tail_credit.store(enable); });
    m.def("set_track_visibility", [](bool enable) {
        g_track_visibility.store(enable);
        if (!enable) { std::lock_guard<std::mutex> lock(g_visibility_mutex); g_visibility.clear(); }
    });
    m.def("set_accumulate_visibility", [](bool enable) { g_accumulate_visibility.store(enable); });
    m.def("reset_visibility", [](int device) {
        std::lock_guard<std::mutex> lock(g_visibility_mutex);
        if (device < 0) g_visibility.clear(); else g_visibility.erase(device);
    }, py::arg("device") = -1);
    m.def("last_visibility", [](int device) -> py::object {
        std::lock_guard<std::mutex> lock(g_visibility_mutex);
        auto it = g_visibility.find(device);
        if (it == g_visibility.end()) return py::none();
        return py::make_tuple(it->second.visible, ReadyEvent{it->second.ready});
    });
    m.def("context_handle", [](int device, uintptr_t stream_key) { return reinterpret_cast<uintptr_t>(context_for(device, stream_key)); },
          py::arg("device"), py::arg("stream_key") = 0, "the calling thread's library context for (device, stream key), as an integer handle");
    m.def("context_handles", [](int device) {
        std::vector<uintptr_t> out;
        for (auto& entry : tls.contexts) if (device < 0 || entry.first.first == device) out.push_back(reinterpret_cast<uintptr_t>(entry.second));
        return out;
    }, py::arg("device") = -1);
#endif
}
