// 3D smoothing-filter update (Mip-Splatting style): for every point inside the (tolerance-widened) frustum of a view,
// filter_3d = min(filter_3d, distance2filter * z) and the point is marked visible.
// Replaces update_3d_filter_cu / update_3d_filter_wrapper of the reference
// (filter3d/src/filter3d_kernels.cu:6-35, filter3d/src/filter3d_api.cu:6-47).  HBM-bound streaming kernel:
// 12 bytes read per point, 5 bytes read-modify-written for the points in view.
#include <algorithm>
#include <string>

#include "kernels.h"

extern "C" void htgs_set_last_error(const char* message);

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

}  // namespace

extern "C" int htgs_update_3d_filter(const float* positions, const float* w2c, float* filter_3d, uint8_t* visibility_mask, int32_t n_points,
                                     int32_t width, int32_t height, float focal_x, float focal_y, float center_x, float center_y, float near_plane,
                                     float clipping_tolerance, float distance2filter, void* stream) {
    if (n_points < 0 || (n_points > 0 && (!positions || !w2c || !filter_3d || !visibility_mask))) {
        htgs_set_last_error("htgs_update_3d_filter: null pointer or negative size");
        return HTGS_ERR_INVALID_ARGUMENT;
    }
    if (n_points == 0) return HTGS_OK;
    // frustum bounds in normalised camera coordinates (filter3d_api.cu:23-33)
    const float bounds_factor = clipping_tolerance + 0.5f;
    const float width_f = static_cast<float>(width), height_f = static_cast<float>(height);
    const float max_x_shifted = bounds_factor * width_f, max_y_shifted = bounds_factor * height_f;
    const float principal_offset_x = center_x - 0.5f * width_f, principal_offset_y = center_y - 0.5f * height_f;
    const float left = (-max_x_shifted - principal_offset_x) / focal_x, right = (max_x_shifted - principal_offset_x) / focal_x;
    const float top = (-max_y_shifted - principal_offset_y) / focal_y, bottom = (max_y_shifted - principal_offset_y) / focal_y;
    int device = 0, sm_count = 148;
    cudaGetDevice(&device);
    cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, device);
    const uint32_t blocks = uint32_t(std::min<int64_t>((int64_t(n_points) + 255) / 256, int64_t(sm_count) * 8));
    update_3d_filter_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(positions, w2c, filter_3d, visibility_mask, uint32_t(n_points), left, right, top,
                                                                                  bottom, near_plane, distance2filter);
    const cudaError_t err = cudaGetLastError();
    if (err != cudaSuccess) {
        htgs_set_last_error((std::string("htgs_update_3d_filter: ") + cudaGetErrorString(err)).c_str());
        return HTGS_ERR_CUDA;
    }
    return HTGS_OK;
}
