// Per-Gaussian preprocess: exact perspective-correct screen bounds, ray-evaluation
// setup, SH -> RGB, view depth, plus two things the reference does not have:
// the per-block instance count (which replaces a separate prefix-sum pass over
// all Gaussians) and a conservative screen-space ellipse used by the blend
// kernels to skip (pixel, Gaussian) pairs the exact test would reject.
//
// Two kernels: a cull pass over all Gaussians and a finish pass over the list of visible ones (typically one in
// six), so that the expensive half (SH evaluation, float64 outline) runs in full warps.
//
// Replaces the sixteen preprocess_cu variants of the reference
// (rasterization/include/*/kernels/{forward,inference}.cuh:10-76) and the device helpers
// transform_and_cull / convert_sh_to_rgb (rasterization/include/kernel_utils.cuh:63-188).
// The float expression shapes of the bounds computation are kept as in the reference so
// that tile boxes are bit-identical; everything around them is new.
#include "kernels.h"

namespace htgs {

namespace {

struct Mat3 { float r11, r12, r13, r21, r22, r23, r31, r32, r33; };

// rasterization/include/kernel_utils.cuh:30-42.  The multiply-add contraction of every entry is
// written out with intrinsics: it is the rounding the reference build (nvcc 12.9, sm_100a, default
// -fmad) was measured to produce for each entry, and the compiler cannot re-associate intrinsics.
__device__ __forceinline__ Mat3 quat_to_mat(const float4& q) {
    const float r = q.x, x = q.y, y = q.z, z = q.w;
    const float yy_zz = __fadd_rn(__fmul_rn(y, y), __fmul_rn(z, z));
    const float xx_zz = __fmaf_rn(x, x, __fmul_rn(z, z));
    const float xx_yy = __fmaf_rn(x, x, __fmul_rn(y, y));
    const float rz = __fmul_rn(r, z), rx = __fmul_rn(r, x), xz = __fmul_rn(x, z);
    return {__fmaf_rn(-2.0f, yy_zz, 1.0f), __fmul_rn(2.0f, __fmaf_rn(x, y, -rz)), __fmul_rn(2.0f, __fmaf_rn(r, y, xz)),
            __fmul_rn(2.0f, __fmaf_rn(x, y, rz)), __fmaf_rn(-2.0f, xx_zz, 1.0f), __fmul_rn(2.0f, __fmaf_rn(y, z, -rx)),
            __fmul_rn(2.0f, __fmaf_rn(-r, y, xz)), __fmul_rn(2.0f, __fmaf_rn(y, z, rx)), __fmaf_rn(-2.0f, xx_yy, 1.0f)};
}

// Rows of (VP*M*T) and (M*T): kernel_utils.cuh:102,111,119,123 and hybrid_blend/kernels/inference.cuh:61.
// As for the rotation matrix, the contraction of each dot product is pinned to what the reference build
// was measured to round like: x*x' fused into y*y', then z*z' fused on top - except the first component
// of the rows built from VPM row 4 and M row 3, where y*y' is fused into x*x'.
__device__ __forceinline__ float dot3_pinned(const float3& a, const float3& b) {
    return __fmaf_rn(a.z, b.z, __fmaf_rn(a.x, b.x, __fmul_rn(a.y, b.y)));
}
__device__ __forceinline__ float dot3_pinned_alt(const float3& a, const float3& b) {
    return __fmaf_rn(a.z, b.z, __fmaf_rn(a.y, b.y, __fmul_rn(a.x, b.x)));
}
template <bool ALT_FIRST>
__device__ __forceinline__ float4 row_times_T(const float4& row, const float3& u, const float3& v, const float3& w, const float3& p) {
    const float3 r = f3(row);
    return make_float4(ALT_FIRST ? dot3_pinned_alt(r, u) : dot3_pinned(r, u), dot3_pinned(r, v), dot3_pinned(r, w), __fadd_rn(dot3_pinned(r, p), row.w));
}

// rasterization/include/kernel_utils.cuh:140-188
template <bool TRAIN>
__device__ __forceinline__ float3 sh_to_rgb(const float* __restrict__ sh_0, const float* __restrict__ sh_rest, const float3& position,
                                            const float3& cam_position, uint32_t idx, int active_sh_bases, int total_sh_bases,
                                            uint8_t* clamp_bits) {
    const float3 dc = make_float3(__ldg(sh_0 + 3 * size_t(idx)), __ldg(sh_0 + 3 * size_t(idx) + 1), __ldg(sh_0 + 3 * size_t(idx) + 2));
    float3 result = 0.5f + 0.28209479177387814f * dc;
    if (active_sh_bases > 1) {
        const float* c = sh_rest + size_t(idx) * size_t(total_sh_bases) * 3;
        auto coef = [&](int i) { return make_float3(__ldg(c + 3 * i), __ldg(c + 3 * i + 1), __ldg(c + 3 * i + 2)); };
        const float3 dir = normalize(position - cam_position);
        const float x = dir.x, y = dir.y, z = dir.z;
        result = result + (-0.48860251190291987f * y) * coef(0)
                        + (0.48860251190291987f * z) * coef(1)
                        + (-0.48860251190291987f * x) * coef(2);
        if (active_sh_bases > 4) {
            const float xx = x * x, yy = y * y, zz = z * z;
            const float xy = x * y, xz = x * z, yz = y * z;
            result = result + (1.0925484305920792f * xy) * coef(3)
                            + (-1.0925484305920792f * yz) * coef(4)
                            + (0.94617469575755997f * zz - 0.31539156525251999f) * coef(5)
                            + (-1.0925484305920792f * xz) * coef(6)
                            + (0.54627421529603959f * xx - 0.54627421529603959f * yy) * coef(7);
            if (active_sh_bases > 9) {
                result = result + (0.59004358992664352f * y * (-3.0f * xx + yy)) * coef(8)
                                + (2.8906114426405538f * xy * z) * coef(9)
                                + (0.45704579946446572f * y * (1.0f - 5.0f * zz)) * coef(10)
                                + (0.3731763325901154f * z * (5.0f * zz - 3.0f)) * coef(11)
                                + (0.45704579946446572f * x * (1.0f - 5.0f * zz)) * coef(12)
                                + (1.4453057213202769f * z * (xx - yy)) * coef(13)
                                + (0.59004358992664352f * x * (-xx + 3.0f * yy)) * coef(14);
            }
        }
    }
    if constexpr (TRAIN) {
        *clamp_bits = uint8_t((result.x < 0 ? 1 : 0) | (result.y < 0 ? 2 : 0) | (result.z < 0 ? 4 : 0));
    }
    return make_float3(fmaxf(0.0f, result.x), fmaxf(0.0f, result.y), fmaxf(0.0f, result.z));
}

// Conservative outline of { pixel : the exact per-fragment test can accept }.
//
// A fragment is accepted only if rho^2 <= max_cutoff_sq and opacity * exp(-rho^2 / 2) >= min_alpha, i.e.
// rho^2 <= L with L = min(max_cutoff_sq, 2 ln(opacity / min_alpha)).  rho^2(pixel) is the squared distance
// (in the Gaussian's unit frame) of the pixel ray to the centre, so the accepted set is the projected outline
// of the ellipsoid |q|^2 <= L: an ellipse whose dual conic is C_ab = L * sum_i T_a[i] T_b[i] - T_a[3] T_b[3]
// (rows a,b of VP*M*T).  Centre and shape are evaluated in float64 from the float32 rows the blend kernels use;
// the shape matrix is inflated by (0.3 px)^2 and the quadratic form relaxed by 2% to cover the float32
// rounding of the exact per-fragment evaluation.  An outline that is not a proper ellipse disables culling
// for the Gaussian ("accept everything"), and L <= 0 rejects everything.
template <int MODE>
__device__ __forceinline__ CullRecord make_cull_record(const float4& t1, const float4& t2, const float4& t4, float opacity) {
    using MT = ModeTraits<MODE>;
    CullRecord rec = {0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f};   // a = b2 = c = 0: every pixel passes
    const double level = fmin(double(MT::max_cutoff_sq), 2.0 * log(double(opacity) * double(MT::min_alpha_rcp))) * 1.001 + 1e-4;
    if (!(level > 0.0)) { rec.cx = __int_as_float(0x7f800000); return rec; }   // +inf: every comparison fails, nothing passes
    auto conic = [&](const float4& a, const float4& b) {
        return level * (double(a.x) * double(b.x) + double(a.y) * double(b.y) + double(a.z) * double(b.z)) - double(a.w) * double(b.w);
    };
    const double c44 = conic(t4, t4);
    if (c44 == 0.0) return rec;
    const double inv = 1.0 / c44;
    const double cx = conic(t1, t4) * inv, cy = conic(t2, t4) * inv;
    double sxx = cx * cx - conic(t1, t1) * inv;
    double syy = cy * cy - conic(t2, t2) * inv;
    const double sxy = cx * cy - conic(t1, t2) * inv;
    if (!(sxx > 0.0) || !(syy > 0.0)) return rec;
    const double det0 = sxx * syy - sxy * sxy;
    if (!(det0 > 0.0)) return rec;
    const double inflate = 0.09 + 1e-6 * (cx * cx + cy * cy);
    sxx += inflate; syy += inflate;
    const double det = sxx * syy - sxy * sxy;
    const double relax = 1.0 / 1.02;
    const double a = syy / det * relax, b2 = -2.0 * sxy / det * relax, c = sxx / det * relax;
    if (!isfinite(a) || !isfinite(b2) || !isfinite(c) || !isfinite(cx) || !isfinite(cy)) return rec;
    if (fabs(cx) > 1e6 || fabs(cy) > 1e6) return rec;   // float32 pixel offsets would lose the sub-pixel part
    rec.cx = float(cx); rec.cy = float(cy);
    rec.a = float(a); rec.b2 = float(b2); rec.c = float(c);
    return rec;
}

// Coefficients of the relaxed-precision record (see FastRecord): float64 from the float32 rows the exact path uses.
// `centre` receives the projected centre (pixels), which the quadratics are expanded around.
__device__ __forceinline__ void make_fast_record(const float4& t1, const float4& t2, const float4& t4, const float4& mt3, const float3& rgb,
                                                 float opacity, float4* dst, double (&centre)[2]) {
    struct D3 { double x, y, z; };
    auto cross3 = [](const D3& a, const D3& b) { return D3{a.y * b.z - a.z * b.y, a.z * b.x - a.x * b.z, a.x * b.y - a.y * b.x}; };
    auto dot3 = [](const D3& a, const D3& b) { return a.x * b.x + a.y * b.y + a.z * b.z; };
    const double w4 = double(t4.w);
    const double cx = double(t1.w) / w4, cy = double(t2.w) / w4;
    const D3 n4{double(t4.x), double(t4.y), double(t4.z)};
    const D3 a{double(t1.x) - n4.x * cx, double(t1.y) - n4.y * cx, double(t1.z) - n4.z * cx};
    const D3 b{double(t2.x) - n4.x * cy, double(t2.y) - n4.y * cy, double(t2.z) - n4.z * cy};
    const D3 d0 = cross3(a, b), dX = cross3(b, n4), dY = cross3(n4, a);
    const double inv = 1.0 / dot3(d0, d0);
    const double e_scale = -0.5 * 1.4426950408889634 * w4 * w4 * inv;
    const D3 m3{double(mt3.x), double(mt3.y), double(mt3.z)};
    const double z_scale = w4 * inv;
    const D3 dXa = cross3(dX, a), dYb = cross3(dY, b);
    float v[20] = {
        float(e_scale * dot3(b, b)), float(-2.0 * e_scale * dot3(a, b)), float(e_scale * dot3(a, a)), float(2.0 * inv * dot3(d0, dX)),
        float(2.0 * inv * dot3(d0, dY)), float(inv * dot3(dX, dX)), float(2.0 * inv * dot3(dX, dY)), float(inv * dot3(dY, dY)),
        float(-z_scale * dot3(m3, cross3(d0, b))), float(z_scale * dot3(m3, cross3(d0, a))), float(-z_scale * dot3(m3, cross3(dX, b))),
        float(z_scale * dot3(m3, D3{dXa.x - dYb.x, dXa.y - dYb.y, dXa.z - dYb.z})),
        float(z_scale * dot3(m3, cross3(dY, a))), mt3.w, log2f(opacity), rgb.x,
        rgb.y, rgb.z, 0.0f, 0.0f};
    bool finite = isfinite(cx) && isfinite(cy);
    #pragma unroll
    for (int i = 0; i < 20; ++i) finite = finite && isfinite(v[i]);
    if (!finite) {   // degenerate Gaussian: contributes nothing
        #pragma unroll
        for (int i = 0; i < 20; ++i) v[i] = 0.0f;
        v[14] = -__int_as_float(0x7f800000);
        centre[0] = centre[1] = 0.0;
    } else {
        centre[0] = cx; centre[1] = cy;
    }
    #pragma unroll
    for (int i = 0; i < 5; ++i) dst[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
}

// Pass 1, one thread per Gaussian: culling, tile box, and the rows VPMT1, VPMT2, VPMT4, MT3 (written where the
// evaluation record lives).  The visible Gaussians of a block are appended to `visible_list` (the order of the list
// depends on the order in which blocks finish; nothing downstream depends on it).
template <int MODE, bool TRAIN>
__global__ void __launch_bounds__(kPreprocessBlock) preprocess_cull_kernel(
    const float* __restrict__ positions, const float* __restrict__ scales, const float* __restrict__ rotations,
    const float* __restrict__ opacities, const float* __restrict__ M, const float* __restrict__ VPM,
    PrimBuffers out, FrameStatus* status, uint32_t n_primitives, uint32_t grid_w, uint32_t grid_h,
    float near_plane, float far_plane, float scale_modifier_arg)
{
    using MT = ModeTraits<MODE>;
    __shared__ uint32_t warp_sum[kPreprocessBlock / 32];
    __shared__ uint32_t warp_vis[kPreprocessBlock / 32];
    __shared__ uint32_t list_base;

    const uint32_t idx = blockIdx.x * kPreprocessBlock + threadIdx.x;
    const uint32_t warp = threadIdx.x >> 5;
    uint32_t n_touched = 0;

    if (idx < n_primitives) {
        const float4 M3 = ldg4(M + 8);
        const float3 position = make_float3(__ldg(positions + 3 * size_t(idx)), __ldg(positions + 3 * size_t(idx) + 1), __ldg(positions + 3 * size_t(idx) + 2));
        const float opacity = __ldg(opacities + idx);
        // near/far culling of the centre (kernel_utils.cuh:88-90)
        const float z = __fadd_rn(dot3_pinned(f3(M3), position), M3.w);
        if (!(z < near_plane || z > far_plane)) {
            const float scale_modifier = TRAIN ? 1.0f : scale_modifier_arg;
            const float3 scale = make_float3(__ldg(scales + 3 * size_t(idx)), __ldg(scales + 3 * size_t(idx) + 1), __ldg(scales + 3 * size_t(idx) + 2));
            const float4 q = ldg4(rotations + 4 * size_t(idx));
            const Mat3 R = quat_to_mat(q);
            const float3 u = make_float3(R.r11 * scale.x, R.r21 * scale.x, R.r31 * scale.x) * scale_modifier;
            const float3 v = make_float3(R.r12 * scale.y, R.r22 * scale.y, R.r32 * scale.y) * scale_modifier;
            const float3 w = make_float3(R.r13 * scale.z, R.r23 * scale.z, R.r33 * scale.z) * scale_modifier;
            const float4 VPM4 = ldg4(VPM + 12);
            const float4 T4 = row_times_T<true>(VPM4, u, v, w, position);
            // tight cutoff for the opacity threshold of the mode (kernel_utils.cuh:104-108)
            const float rho_cutoff = 2.0f * logf(opacity * MT::min_alpha_rcp);
            const float4 d = make_float4(rho_cutoff, rho_cutoff, rho_cutoff, -1.0f);
            const float s = dot(d, T4 * T4);
            if (s != 0.0f) {
                const float4 f = (1.0f / s) * d;
                // exact near/far culling by the screen-space z extent (kernel_utils.cuh:110-116)
                const float4 VPM3 = ldg4(VPM + 8);
                const float4 T3 = row_times_T<false>(VPM3, u, v, w, position);
                const float center_z = dot(f, T3 * T4);
                const float extent_z = sqrtf(fmaxf(center_z * center_z - dot(f, T3 * T3), 0.0f));
                const float z_min = center_z - extent_z;
                const float z_max = center_z + extent_z;
                if (!(z_min < -1.0f || z_max > 1.0f)) {
                    const float4 VPM1 = ldg4(VPM);
                    const float4 T1 = row_times_T<false>(VPM1, u, v, w, position);
                    const float center_x = dot(f, T1 * T4);
                    const float extent_x = sqrtf(fmaxf(center_x * center_x - dot(f, T1 * T1), 0.0f));
                    const float4 VPM2 = ldg4(VPM + 4);
                    const float4 T2 = row_times_T<false>(VPM2, u, v, w, position);
                    const float center_y = dot(f, T2 * T4);
                    const float extent_y = sqrtf(fmaxf(center_y * center_y - dot(f, T2 * T2), 0.0f));
                    // tile box (+0.5: pixel centres sit at integer coordinates; kernel_utils.cuh:126-137)
                    const float tw = float(MT::tile_w), th = float(MT::tile_h);
                    const uint32_t x_min = min(grid_w, static_cast<uint32_t>(max(0, __float2int_rd((center_x - extent_x + 0.5f) / tw))));
                    const uint32_t x_max = min(grid_w, static_cast<uint32_t>(max(0, __float2int_ru((center_x + extent_x + 0.5f) / tw))));
                    const uint32_t y_min = min(grid_h, static_cast<uint32_t>(max(0, __float2int_rd((center_y - extent_y + 0.5f) / th))));
                    const uint32_t y_max = min(grid_h, static_cast<uint32_t>(max(0, __float2int_ru((center_y + extent_y + 0.5f) / th))));
                    n_touched = (x_max - x_min) * (y_max - y_min);
                    if (n_touched != 0) {
                        out.bounds[idx] = make_ushort4((unsigned short)x_min, (unsigned short)x_max, (unsigned short)y_min, (unsigned short)y_max);
                        float4* dst = reinterpret_cast<float4*>(out.eval + idx);
                        dst[0] = T1; dst[1] = T2; dst[2] = T4;
                        if constexpr (MODE == HTGS_MODE_ALPHA_BLEND_GLOBAL_ORDERING) dst[3] = make_float4(0.0f, 0.0f, 0.0f, z);
                        else dst[3] = make_float4(dot3_pinned_alt(f3(M3), u), dot3_pinned(f3(M3), v), dot3_pinned(f3(M3), w), z);
                    }
                }
            }
        }
        out.n_touched[idx] = n_touched;
    }

    // per-block totals (instances, visible Gaussians) and the block's slice of the list of visible Gaussians
    const bool visible = n_touched != 0;
    const uint32_t ballot = __ballot_sync(0xffffffffu, visible);
    uint32_t sum = n_touched;
    #pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    if ((threadIdx.x & 31) == 0) { warp_sum[warp] = sum; warp_vis[warp] = __popc(ballot); }
    __syncthreads();
    if (threadIdx.x == 0) {
        uint32_t total = 0, total_vis = 0;
        #pragma unroll
        for (int i = 0; i < kPreprocessBlock / 32; ++i) { total += warp_sum[i]; total_vis += warp_vis[i]; }
        out.block_sums[blockIdx.x] = total;
        list_base = total_vis ? atomicAdd(&status->n_visible, total_vis) : 0u;
    }
    __syncthreads();
    if (visible) {
        uint32_t slot = list_base + __popc(ballot & lanemask_lt());
        #pragma unroll
        for (int i = 0; i < kPreprocessBlock / 32; ++i)
            if (i < int(warp)) slot += warp_vis[i];
        out.visible_list[slot] = idx;
    }
}

// Pass 2, one thread per VISIBLE Gaussian (grid-stride over the list): colour from the SH coefficients, the
// remaining parts of the evaluation record, the conservative outline.  Runs with full warps whatever the
// fraction of Gaussians that survived culling.
constexpr int kFinishBlock = 128;
template <int MODE, bool TRAIN, bool FAST>
__global__ void __launch_bounds__(kFinishBlock) preprocess_finish_kernel(
    const float* __restrict__ positions, const float* __restrict__ opacities, const float* __restrict__ sh_0, const float* __restrict__ sh_rest,
    const float* __restrict__ cam_position_ptr, PrimBuffers out, const FrameStatus* __restrict__ status, int active_sh_bases, int total_sh_bases)
{
    const uint32_t n_visible = status->n_visible;
    const float3 cam_position = make_float3(__ldg(cam_position_ptr), __ldg(cam_position_ptr + 1), __ldg(cam_position_ptr + 2));
    for (uint32_t i = blockIdx.x * kFinishBlock + threadIdx.x; i < n_visible; i += gridDim.x * kFinishBlock) {
        const uint32_t gi = out.visible_list[i];
        float4* dst = reinterpret_cast<float4*>(out.eval + gi);
        const float4 t1 = dst[0], t2 = dst[1], t4 = dst[2], m3 = dst[3];
        const float3 position = make_float3(__ldg(positions + 3 * size_t(gi)), __ldg(positions + 3 * size_t(gi) + 1), __ldg(positions + 3 * size_t(gi) + 2));
        const float opacity = __ldg(opacities + gi);
        uint8_t clamp_bits = 0;
        const float3 rgb = sh_0 ? sh_to_rgb<TRAIN>(sh_0, sh_rest, position, cam_position, gi, active_sh_bases, total_sh_bases, &clamp_bits)
                                : make_float3(0.0f, 0.0f, 0.0f);   // colour-less callers (update_max_weights)
        [[maybe_unused]] double centre[2] = {0.0, 0.0};
        if constexpr (FAST) make_fast_record(t1, t2, t4, m3, rgb, opacity, dst, centre);
        else dst[4] = make_float4(rgb.x, rgb.y, rgb.z, opacity);
        if constexpr (TRAIN) out.clamp[gi] = clamp_bits;
        CullRecord cr = make_cull_record<MODE>(t1, t2, t4, opacity);
        if constexpr (FAST) {
            // The fragment evaluation measures from the projected centre, the outline test from the centre of
            // the outline: the record carries the (small) difference, so that outline centre + difference
            // gives the projected centre to better than float32 resolution at the pixel's magnitude.
            cr.cx_lo = float(centre[0] - double(cr.cx));
            cr.cy_lo = float(centre[1] - double(cr.cy));
        }
        float4* cdst = reinterpret_cast<float4*>(out.cull + gi);
        cdst[0] = make_float4(cr.cx, cr.cy, cr.a, cr.b2);
        cdst[1] = make_float4(cr.c, cr.cx_lo, cr.cy_lo, 0.0f);
    }
}

int sm_count_of_current_device() {
    static std::atomic<int> cached[64] = {};
    int device = 0;
    cudaGetDevice(&device);
    if (device < 0 || device >= 64) return 148;
    int n = cached[device].load(std::memory_order_relaxed);
    if (!n) {
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || n <= 0) n = 148;
        cached[device].store(n, std::memory_order_relaxed);
    }
    return n;
}

template <int MODE, bool TRAIN, bool FAST>
cudaError_t launch_t(const HtgsScene& scene, const HtgsView& view, const FrameGeometry& geo, const PrimBuffers& prim, FrameStatus* status, cudaStream_t stream) {
    const uint32_t n = uint32_t(scene.n_primitives);
    const uint32_t blocks = (n + kPreprocessBlock - 1) / kPreprocessBlock;
    if (blocks == 0) return cudaSuccess;
    preprocess_cull_kernel<MODE, TRAIN><<<blocks, kPreprocessBlock, 0, stream>>>(
        scene.positions, scene.scales, scene.rotations, scene.opacities, view.M, view.VPM, prim, status, n, uint32_t(geo.grid_w),
        uint32_t(geo.grid_h), view.near_plane, view.far_plane, view.scale_modifier);
    cudaError_t err = cudaGetLastError();
    if (err != cudaSuccess) return err;
    const uint32_t finish_blocks = min((n + kFinishBlock - 1) / kFinishBlock, uint32_t(sm_count_of_current_device()) * 8u);
    preprocess_finish_kernel<MODE, TRAIN, FAST><<<finish_blocks, kFinishBlock, 0, stream>>>(
        scene.positions, scene.opacities, scene.sh_0, scene.sh_rest, view.cam_position, prim, status, view.active_sh_bases, scene.total_sh_bases);
    return cudaGetLastError();
}

}  // namespace

cudaError_t launch_preprocess(int mode, bool train, const HtgsScene& scene, const HtgsView& view, const FrameGeometry& geo,
                              const PrimBuffers& prim, FrameStatus* status, cudaStream_t stream, bool fast_records) {
    if (fast_records) {
        if (train) return cudaErrorInvalidValue;
        switch (mode) {
            case HTGS_MODE_HYBRID_BLEND: return launch_t<HTGS_MODE_HYBRID_BLEND, false, true>(scene, view, geo, prim, status, stream);
            case HTGS_MODE_ALPHA_BLEND_FIRST_K: return launch_t<HTGS_MODE_ALPHA_BLEND_FIRST_K, false, true>(scene, view, geo, prim, status, stream);
            case HTGS_MODE_OIT_BLEND: return launch_t<HTGS_MODE_OIT_BLEND, false, true>(scene, view, geo, prim, status, stream);
            default: return cudaErrorInvalidValue;
        }
    }
    switch (mode) {
#define HTGS_CASE(M) case M: return train ? launch_t<M, true, false>(scene, view, geo, prim, status, stream) : launch_t<M, false, false>(scene, view, geo, prim, status, stream);
        HTGS_CASE(HTGS_MODE_HYBRID_BLEND)
        HTGS_CASE(HTGS_MODE_ALPHA_BLEND_FIRST_K)
        HTGS_CASE(HTGS_MODE_ALPHA_BLEND_GLOBAL_ORDERING)
        HTGS_CASE(HTGS_MODE_OIT_BLEND)
#undef HTGS_CASE
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace htgs
