// 3D smoothing-filter update (Mip-Splatting style): for every point inside the (tolerance-widened) frustum of a view,
// filter_3d = min(filter_3d, distance2filter * z) and the point is marked visible.
// Replaces update_3d_filter_cu / update_3d_filter_wrapper of the reference
// (filter3d/src/filter3d_kernels.cu:6-35, filter3d/src/filter3d_api.cu:6-47).  HBM-bound streaming kernel:
// 12 bytes read per point, 5 bytes read-modify-written for the points in view.
#include <algorithm>
#include <string>

#include "kernels.h"


namespace {

__global__ void __launch_bounds__(256) update_3d_filter_kernel(const float* __restrict__ positions, const float* __restrict__ w2c, float* __restrict__ filter_3d,
                                                                 uint8_t* __restrict__ visibility_mask, uint32_t n_points, float left, float right, float top,
                                                                 float bottom, float near_plane, float distance2filter) {
    using namespace htgs;
    const float4 r1 = ldg4(w2c), r2 = ldg4(w2c + 4), r3 = ldg4(w2c + 8);
    for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < n_points; i += gridDim.x * blockDim.x) {
        const float3 p = make_float3(__ldg(positions + 3 * size_t(i)), __ldg(positions + 3 * size_t(i) + 1), __ldg(positions + 3 * size_t(i) + 2));
        const float z = dot(f3(r3), p) + r3.w;
        if (z < near_plane) continue;
        const float x_clip = dot(f3(r1), p) + r1.w;
        if (x_clip < left * z || x_clip > right * z) continue;
        const float y_clip = dot(f3(r2), p) + r2.w;
        if (y_clip < top * z || y_clip > bottom * z) continue;
        const float filter_3d_new = distance2filter * z;
        if (filter_3d[i] < filter_3d_new) continue;
        filter_3d[i] = filter_3d_new;
        visibility_mask[i] = 1;
    }
}

// Several views in one pass over the points: the point and its running filter value stay in registers while the views'
// parameters (passed by value, they live in the kernel's constant bank) are applied one after the other.  Per view the
// arithmetic is that of update_3d_filter_kernel, and min / "was updated" accumulate exactly as a sequence of single-view
// calls would, so the result equals that sequence bit for bit while the positions are read once per launch instead of once
// per view.
constexpr int kViewsPerLaunch = 48;
struct __align__(16) FilterView { float r1[4], r2[4], r3[4], left, right, top, bottom, near_plane, pad[3]; };   // 80 bytes
struct FilterViewBatch { FilterView view[kViewsPerLaunch]; };                                     // 3840 bytes of kernel parameters

__global__ void __launch_bounds__(256) update_3d_filter_views_kernel(const float* __restrict__ positions, float* __restrict__ filter_3d,
                                                                       uint8_t* __restrict__ visibility_mask, uint32_t n_points,
                                                                       const __grid_constant__ FilterViewBatch batch, int n_views, float distance2filter) {
    // the parameters of up to 48 views exceed the per-SM constant cache: every block copies them to shared memory once
    __shared__ FilterView s_view[kViewsPerLaunch];
    {
        const float* src = reinterpret_cast<const float*>(&batch);
        float* dst = reinterpret_cast<float*>(s_view);
        for (int k = threadIdx.x; k < n_views * int(sizeof(FilterView) / 4); k += blockDim.x) dst[k] = src[k];
    }
    __syncthreads();
    for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < n_points; i += gridDim.x * blockDim.x) {
        const float3 p = make_float3(__ldg(positions + 3 * size_t(i)), __ldg(positions + 3 * size_t(i) + 1), __ldg(positions + 3 * size_t(i) + 2));
        float current = filter_3d[i];
        bool updated = false;
        for (int v = 0; v < n_views; ++v) {
            const float4 r3 = *reinterpret_cast<const float4*>(s_view[v].r3);
            const float z = (r3.x * p.x + r3.y * p.y + r3.z * p.z) + r3.w;
            if (z < s_view[v].near_plane) continue;
            const float4 r1 = *reinterpret_cast<const float4*>(s_view[v].r1);
            const float x_clip = (r1.x * p.x + r1.y * p.y + r1.z * p.z) + r1.w;
            if (x_clip < s_view[v].left * z || x_clip > s_view[v].right * z) continue;
            const float4 r2 = *reinterpret_cast<const float4*>(s_view[v].r2);
            const float y_clip = (r2.x * p.x + r2.y * p.y + r2.z * p.z) + r2.w;
            if (y_clip < s_view[v].top * z || y_clip > s_view[v].bottom * z) continue;
            const float filter_3d_new = distance2filter * z;
            if (current < filter_3d_new) continue;
            current = filter_3d_new;
            updated = true;
        }
        if (updated) { filter_3d[i] = current; visibility_mask[i] = 1; }
    }
}

void frustum_bounds(int32_t width, int32_t height, float focal_x, float focal_y, float center_x, float center_y, float clipping_tolerance,
                    float& left, float& right, float& top, float& bottom) {
    // frustum bounds in normalised camera coordinates (filter3d_api.cu:23-33)
    const float bounds_factor = clipping_tolerance + 0.5f;
    const float width_f = static_cast<float>(width), height_f = static_cast<float>(height);
    const float max_x_shifted = bounds_factor * width_f, max_y_shifted = bounds_factor * height_f;
    const float principal_offset_x = center_x - 0.5f * width_f, principal_offset_y = center_y - 0.5f * height_f;
    left = (-max_x_shifted - principal_offset_x) / focal_x; right = (max_x_shifted - principal_offset_x) / focal_x;
    top = (-max_y_shifted - principal_offset_y) / focal_y; bottom = (max_y_shifted - principal_offset_y) / focal_y;
}

}  // namespace

extern "C" int htgs_update_3d_filter_views(const float* positions, const HtgsFilterView* views, int32_t n_views, float* filter_3d,
                                           uint8_t* visibility_mask, int32_t n_points, float clipping_tolerance, float distance2filter, void* stream) {
    if (n_points < 0 || n_views < 0 || (n_points > 0 && n_views > 0 && (!positions || !views || !filter_3d || !visibility_mask))) {
        htgs::set_last_error("htgs_update_3d_filter_views: null pointer or negative size");
        return HTGS_ERR_INVALID_ARGUMENT;
    }
    if (n_points == 0 || n_views == 0) return HTGS_OK;
    int device = 0, sm_count = 148;
    cudaGetDevice(&device);
    cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, device);
    const uint32_t blocks = uint32_t(std::min<int64_t>((int64_t(n_points) + 255) / 256, int64_t(sm_count) * 8));
    for (int32_t first = 0; first < n_views; first += kViewsPerLaunch) {
        FilterViewBatch batch;
        const int count = std::min<int32_t>(kViewsPerLaunch, n_views - first);
        for (int v = 0; v < count; ++v) {
            const HtgsFilterView& in = views[first + v];
            FilterView& out = batch.view[v];
            for (int c = 0; c < 4; ++c) { out.r1[c] = in.w2c[c]; out.r2[c] = in.w2c[4 + c]; out.r3[c] = in.w2c[8 + c]; }
            frustum_bounds(in.width, in.height, in.focal_x, in.focal_y, in.center_x, in.center_y, clipping_tolerance, out.left, out.right, out.top, out.bottom);
            out.near_plane = in.near_plane;
            out.pad[0] = out.pad[1] = out.pad[2] = 0.0f;
        }
        update_3d_filter_views_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(positions, filter_3d, visibility_mask, uint32_t(n_points), batch, count,
                                                                                            distance2filter);
        const cudaError_t err = cudaGetLastError();
        if (err != cudaSuccess) {
            htgs::set_last_error((std::string("htgs_update_3d_filter_views: ") + cudaGetErrorString(err)).c_str());
            return HTGS_ERR_CUDA;
        }
    }
    return HTGS_OK;
}

extern "C" int htgs_update_3d_filter(const float* positions, const float* w2c, float* filter_3d, uint8_t* visibility_mask, int32_t n_points,
                                     int32_t width, int32_t height, float focal_x, float focal_y, float center_x, float center_y, float near_plane,
                                     float clipping_tolerance, float distance2filter, void* stream) {
    if (n_points < 0 || (n_points > 0 && (!positions || !w2c || !filter_3d || !visibility_mask))) {
        htgs::set_last_error("htgs_update_3d_filter: null pointer or negative size");
        return HTGS_ERR_INVALID_ARGUMENT;
    }
    if (n_points == 0) return HTGS_OK;
    float left, right, top, bottom;
    frustum_bounds(width, height, focal_x, focal_y, center_x, center_y, clipping_tolerance, left, right, top, bottom);
    int device = 0, sm_count = 148;
    cudaGetDevice(&device);
    cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, device);
    const uint32_t blocks = uint32_t(std::min<int64_t>((int64_t(n_points) + 255) / 256, int64_t(sm_count) * 8));
    update_3d_filter_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(positions, w2c, filter_3d, visibility_mask, uint32_t(n_points), left, right, top,
                                                                                  bottom, near_plane, distance2filter);
    const cudaError_t err = cudaGetLastError();
    if (err != cudaSuccess) {
        htgs::set_last_error((std::string("htgs_update_3d_filter: ") + cudaGetErrorString(err)).c_str());
        return HTGS_ERR_CUDA;
    }
    return HTGS_OK;
}
