// Fused parameter activations of the Gaussian model, forward and backward: one pass over N instead of the
// four to six element-wise PyTorch passes of the reference's model (Model.py:45-49: exp / normalize / expit;
// Model.py:82-100: the 3D-filter adjustment of scales and opacities).
//
//   scales    = exp(raw_scales)                      with a 3D filter f:  sqrt(exp(raw_scales)^2 + f^2)
//   rotations = raw_rotations / max(|raw_rotations|, 1e-12)               (torch.nn.functional.normalize)
//   opacities = expit(raw_opacities)                 with a 3D filter:    expit(.) * prod_i s_i / sqrt(s_i^2 + f^2)
//
// HBM-bound: 32 (+4) bytes read and 32 written per Gaussian forward; 64 (+4) read and 32 written backward.
#include "kernels.h"

namespace htgs {

namespace {

constexpr int kActBlock = 256;

__global__ void __launch_bounds__(kActBlock) activate_kernel(
    const float* __restrict__ raw_scales, const float* __restrict__ raw_rotations, const float* __restrict__ raw_opacities,
    const float* __restrict__ filter_3d, float* __restrict__ scales, float* __restrict__ rotations, float* __restrict__ opacities, uint32_t n)
{
    const uint32_t i = blockIdx.x * kActBlock + threadIdx.x;
    if (i >= n) return;
    float s[3] = {expf(raw_scales[3 * size_t(i)]), expf(raw_scales[3 * size_t(i) + 1]), expf(raw_scales[3 * size_t(i) + 2])};
    float opacity = 1.0f / (1.0f + expf(-raw_opacities[i]));
    if (filter_3d) {
        const float f2 = filter_3d[i] * filter_3d[i];
        float det1 = 1.0f, det2 = 1.0f;
        #pragma unroll
        for (int c = 0; c < 3; ++c) {
            const float s2 = s[c] * s[c];
            det1 *= s2;
            det2 *= s2 + f2;
            s[c] = sqrtf(s2 + f2);
        }
        opacity *= sqrtf(det1 / det2);
    }
    scales[3 * size_t(i)] = s[0]; scales[3 * size_t(i) + 1] = s[1]; scales[3 * size_t(i) + 2] = s[2];
    opacities[i] = opacity;
    const float4 q = ldg4(raw_rotations + 4 * size_t(i));
    const float inv = 1.0f / fmaxf(sqrtf(q.x * q.x + q.y * q.y + q.z * q.z + q.w * q.w), 1e-12f);
    reinterpret_cast<float4*>(rotations)[i] = make_float4(q.x * inv, q.y * inv, q.z * inv, q.w * inv);
}

__global__ void __launch_bounds__(kActBlock) activate_backward_kernel(
    const float* __restrict__ raw_scales, const float* __restrict__ raw_rotations, const float* __restrict__ raw_opacities,
    const float* __restrict__ filter_3d, const float* __restrict__ grad_scales, const float* __restrict__ grad_rotations,
    const float* __restrict__ grad_opacities, float* __restrict__ grad_raw_scales, float* __restrict__ grad_raw_rotations,
    float* __restrict__ grad_raw_opacities, uint32_t n)
{
    const uint32_t i = blockIdx.x * kActBlock + threadIdx.x;
    if (i >= n) return;
    const float s[3] = {expf(raw_scales[3 * size_t(i)]), expf(raw_scales[3 * size_t(i) + 1]), expf(raw_scales[3 * size_t(i) + 2])};
    const float o = 1.0f / (1.0f + expf(-raw_opacities[i]));
    const float go = grad_opacities[i];
    float gs[3] = {grad_scales[3 * size_t(i)], grad_scales[3 * size_t(i) + 1], grad_scales[3 * size_t(i) + 2]};
    float d_raw_o = go * o * (1.0f - o);
    if (filter_3d) {
        const float f2 = filter_3d[i] * filter_3d[i];
        float coef = 1.0f, sf2[3];
        #pragma unroll
        for (int c = 0; c < 3; ++c) { sf2[c] = s[c] * s[c] + f2; coef *= s[c] * s[c] / sf2[c]; }
        coef = sqrtf(coef);
        d_raw_o *= coef;
        #pragma unroll
        for (int c = 0; c < 3; ++c) {
            // d sqrt(s^2 + f^2) / ds = s / sqrt(s^2 + f^2);   d coef / ds = coef * f^2 / (s * (s^2 + f^2))
            gs[c] = gs[c] * s[c] * rsqrtf(sf2[c]) + go * o * coef * f2 / (s[c] * sf2[c]);
        }
    }
    #pragma unroll
    for (int c = 0; c < 3; ++c) grad_raw_scales[3 * size_t(i) + c] = gs[c] * s[c];
    grad_raw_opacities[i] = d_raw_o;
    const float4 q = ldg4(raw_rotations + 4 * size_t(i));
    const float4 g = ldg4(grad_rotations + 4 * size_t(i));
    const float norm = sqrtf(q.x * q.x + q.y * q.y + q.z * q.z + q.w * q.w);
    float4 out;
    if (norm > 1e-12f) {
        const float inv = 1.0f / norm;
        const float4 u = make_float4(q.x * inv, q.y * inv, q.z * inv, q.w * inv);
        const float ug = u.x * g.x + u.y * g.y + u.z * g.z + u.w * g.w;
        out = make_float4((g.x - u.x * ug) * inv, (g.y - u.y * ug) * inv, (g.z - u.z * ug) * inv, (g.w - u.w * ug) * inv);
    } else {
        out = make_float4(g.x * 1e12f, g.y * 1e12f, g.z * 1e12f, g.w * 1e12f);   // the clamped branch of normalize: x / 1e-12
    }
    reinterpret_cast<float4*>(grad_raw_rotations)[i] = out;
}

}  // namespace

}  // namespace htgs

extern "C" {


static int activation_fail(int code, const char* message) { htgs::set_last_error(message); return code; }

int htgs_activate(const float* raw_scales, const float* raw_rotations, const float* raw_opacities, const float* filter_3d, float* scales,
                  float* rotations, float* opacities, int32_t n_primitives, void* stream) {
    if (n_primitives < 0 || (n_primitives > 0 && (!raw_scales || !raw_rotations || !raw_opacities || !scales || !rotations || !opacities)))
        return activation_fail(HTGS_ERR_INVALID_ARGUMENT, "htgs_activate: null pointer or negative count");
    if (n_primitives == 0) return HTGS_OK;
    const uint32_t n = uint32_t(n_primitives);
    htgs::activate_kernel<<<(n + htgs::kActBlock - 1) / htgs::kActBlock, htgs::kActBlock, 0, static_cast<cudaStream_t>(stream)>>>(
        raw_scales, raw_rotations, raw_opacities, filter_3d, scales, rotations, opacities, n);
    const cudaError_t err = cudaGetLastError();
    return err == cudaSuccess ? HTGS_OK : activation_fail(HTGS_ERR_CUDA, cudaGetErrorString(err));
}

int htgs_activate_backward(const float* raw_scales, const float* raw_rotations, const float* raw_opacities, const float* filter_3d,
                           const float* grad_scales, const float* grad_rotations, const float* grad_opacities, float* grad_raw_scales,
                           float* grad_raw_rotations, float* grad_raw_opacities, int32_t n_primitives, void* stream) {
    if (n_primitives < 0 || (n_primitives > 0 && (!raw_scales || !raw_rotations || !raw_opacities || !grad_scales || !grad_rotations || !grad_opacities ||
                                                  !grad_raw_scales || !grad_raw_rotations || !grad_raw_opacities)))
        return activation_fail(HTGS_ERR_INVALID_ARGUMENT, "htgs_activate_backward: null pointer or negative count");
    if (n_primitives == 0) return HTGS_OK;
    const uint32_t n = uint32_t(n_primitives);
    htgs::activate_backward_kernel<<<(n + htgs::kActBlock - 1) / htgs::kActBlock, htgs::kActBlock, 0, static_cast<cudaStream_t>(stream)>>>(
        raw_scales, raw_rotations, raw_opacities, filter_3d, grad_scales, grad_rotations, grad_opacities, grad_raw_scales, grad_raw_rotations,
        grad_raw_opacities, n);
    const cudaError_t err = cudaGetLastError();
    return err == cudaSuccess ? HTGS_OK : activation_fail(HTGS_ERR_CUDA, cudaGetErrorString(err));
}

}  // extern "C"
