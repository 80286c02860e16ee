// Shared declarations of the sm_100a rasterizer core: per-mode constants, the
// device-side data layout, small vector algebra and PTX wrappers.
#pragma once

#include <cuda_runtime.h>
#include <cstdint>
#include <cfloat>

#include "../../include/htgs_b200.h"

namespace htgs {

// ---------------------------------------------------------------------------
// per-mode numerical constants; they are part of the numerical contract with
// the reference (rasterization/include/*/config.h:15-29)
// ---------------------------------------------------------------------------
constexpr float kTransmittanceThreshold = 1e-4f;
constexpr float kMaxFragmentAlpha = 1.0f;
constexpr float kOneMinusAlphaEps = 1e-8f;

template <int MODE> struct ModeTraits;
template <> struct ModeTraits<HTGS_MODE_HYBRID_BLEND> {
    static constexpr int tile_w = 8, tile_h = 8;
    static constexpr float min_alpha_rcp = 255.0f;
    static constexpr float min_alpha = 1.0f / 255.0f;
    static constexpr float max_cutoff_sq = 11.0825270903f;
    static constexpr float min_alpha_core = 1.0f / 20.0f;
};
template <> struct ModeTraits<HTGS_MODE_ALPHA_BLEND_FIRST_K> {
    static constexpr int tile_w = 8, tile_h = 8;
    static constexpr float min_alpha_rcp = 20.0f;
    static constexpr float min_alpha = 1.0f / 20.0f;
    static constexpr float max_cutoff_sq = 5.99146454711f;
    static constexpr float min_alpha_core = 0.0f;
};
template <> struct ModeTraits<HTGS_MODE_ALPHA_BLEND_GLOBAL_ORDERING> {
    static constexpr int tile_w = 16, tile_h = 16;
    static constexpr float min_alpha_rcp = 255.0f;
    static constexpr float min_alpha = 1.0f / 255.0f;
    static constexpr float max_cutoff_sq = 11.0825270903f;
    static constexpr float min_alpha_core = 0.0f;
};
template <> struct ModeTraits<HTGS_MODE_OIT_BLEND> {
    static constexpr int tile_w = 8, tile_h = 8;
    static constexpr float min_alpha_rcp = 255.0f;
    static constexpr float min_alpha = 1.0f / 255.0f;
    static constexpr float max_cutoff_sq = 11.0825270903f;
    static constexpr float min_alpha_core = 0.0f;
};

inline int mode_tile_w(int mode) { return mode == HTGS_MODE_ALPHA_BLEND_GLOBAL_ORDERING ? 16 : 8; }
inline int mode_tile_h(int mode) { return mode == HTGS_MODE_ALPHA_BLEND_GLOBAL_ORDERING ? 16 : 8; }

// ---------------------------------------------------------------------------
// data layout in HBM
// ---------------------------------------------------------------------------
// What the blend kernels need to evaluate one Gaussian at a pixel: 80 bytes,
// 16-byte aligned, so one record moves to shared memory with a single bulk
// asynchronous copy.  Rows of the 3x4 matrices (VP*M*T) and (M*T) of the
// reference (kernel_utils.cuh:98-123, hybrid_blend/kernels/inference.cuh:57-74).
struct __align__(16) EvalRecord {
    float4 vpmt1;
    float4 vpmt2;
    float4 vpmt4;
    float4 mt3;    // .w = view-space depth of the centre
    float4 rgba;   // view-dependent colour (clamped at 0), opacity
};
static_assert(sizeof(EvalRecord) == 80, "EvalRecord must be 80 bytes");

// Conservative screen-space outline of the fragment-acceptance region
// { pixel : alpha(pixel) >= min_alpha }, an ellipse
//   a*dx^2 + b2*dx*dy + c*dy^2 <= 1,  (dx,dy) = pixel - (cx,cy),
// computed in float64, inflated by a safety margin (see preprocess.cu).  It
// has no counterpart in the reference; it only removes (pixel, Gaussian)
// pairs that the exact per-fragment test would reject anyway.
struct __align__(16) CullRecord {
    float cx, cy;
    float a, b2;
    float c;
    float cx_lo, cy_lo;   // projected centre of the Gaussian minus (cx, cy); written and read by the relaxed-precision path only
    float pad;
};
static_assert(sizeof(CullRecord) == 32, "CullRecord must be 32 bytes");

// Relaxed-precision evaluation record (fast_rasterize path, HYBRID_BLEND), same size and place as EvalRecord.
// With (dx, dy) = pixel - (cx, cy), where (cx, cy) is the projected centre of the Gaussian, the two planes through
// the pixel ray (hybrid_blend/kernels/fast_inference.cuh:150-156) give m = w4 * (dy * a - dx * b) and
// d = d0 + dx * dX + dy * dY, so rho^2 = (m.m)/(d.d) and depth = MT3.(d x m)/(d.d) + MT3.w are ratios of
// quadratics in (dx, dy) whose coefficients are fixed per Gaussian (float64 in the preprocess, divided by d0.d0):
//   e     = q1xx dx^2 + q1xy dx dy + q1yy dy^2           = -0.5 * log2(e) * (m.m) / (d0.d0)
//   den   = 1 + q2x dx + q2y dy + q2xx dx^2 + q2xy dx dy + q2yy dy^2  = (d.d) / (d0.d0)
//   num_z = q3x dx + q3y dy + q3xx dx^2 + q3xy dx dy + q3yy dy^2       = MT3.(d x m) / (d0.d0)
//   alpha = min(exp2(e / den + log2_opacity), 1),   depth = num_z / den + depth_centre
// The centre travels with the outline record (CullRecord: outline centre cx, cy plus the difference cx_lo, cy_lo to the
// projected centre): a single float32 centre costs 6e-5 px at x ~ 1000, the dominant error of alpha for Gaussians of
// sub-pixel extent.  The staging thread turns it into a tile-relative offset, dx = x_in_tile + dx0.
struct __align__(16) FastRecord {
    float q1xx, q1xy, q1yy, q2x;
    float q2y, q2xx, q2xy, q2yy;
    float q3x, q3y, q3xx, q3xy;
    float q3yy, depth_centre, log2_opacity, r;
    float g, b, pad0, pad1;
};
static_assert(sizeof(FastRecord) == sizeof(EvalRecord), "FastRecord shares the storage of EvalRecord");

// Device-resident frame status, copied to the host at the end of a call.
struct FrameStatus {
    unsigned int n_instances;     // total (tile, Gaussian) instances of the frame
    unsigned int overflow;        // 1 if n_instances exceeded the instance capacity of the workspace
    unsigned int n_visible;       // Gaussians that survived culling
    unsigned int error;           // bounded waits that gave up, bad arguments seen on the device, ...
    unsigned long long candidate_pairs;     // statistics mode of the blend kernels
    unsigned long long accepted_fragments;  // statistics mode of the blend kernels
    unsigned long long warp_trips;          // statistics mode, HYBRID_BLEND: warp-level evaluations of one candidate per lane
    unsigned long long warp_trips_inserting;// ... of which at least one lane inserted into its K-buffer (the insertion chain ran)
    unsigned long long lane_insertions;     // ... and the lanes that inserted
    unsigned int reserved[2];
};

// ---------------------------------------------------------------------------
// vector algebra.  The expression shapes (association order of sums of
// products) follow the helper the reference uses (utils/helper_math.h: dot
// 1267-1274, cross 1451-1454, normalize 1328-1332), so that the compiler's
// multiply-add contraction yields the same rounding as the reference build.
// ---------------------------------------------------------------------------
__device__ __forceinline__ float3 f3(const float4& a) { return make_float3(a.x, a.y, a.z); }
__device__ __forceinline__ float dot(const float3& a, const float3& b) { return a.x * b.x + a.y * b.y + a.z * b.z; }
__device__ __forceinline__ float dot(const float4& a, const float4& b) { return a.x * b.x + a.y * b.y + a.z * b.z + a.w * b.w; }
__device__ __forceinline__ float3 cross(const float3& a, const float3& b) {
    return make_float3(a.y * b.z - a.z * b.y, a.z * b.x - a.x * b.z, a.x * b.y - a.y * b.x);
}
__device__ __forceinline__ float3 operator*(const float3& a, float s) { return make_float3(a.x * s, a.y * s, a.z * s); }
__device__ __forceinline__ float3 operator*(float s, const float3& a) { return make_float3(s * a.x, s * a.y, s * a.z); }
__device__ __forceinline__ float3 operator*(const float3& a, const float3& b) { return make_float3(a.x * b.x, a.y * b.y, a.z * b.z); }
__device__ __forceinline__ float3 operator+(const float3& a, const float3& b) { return make_float3(a.x + b.x, a.y + b.y, a.z + b.z); }
__device__ __forceinline__ float3 operator-(const float3& a, const float3& b) { return make_float3(a.x - b.x, a.y - b.y, a.z - b.z); }
__device__ __forceinline__ float3 operator+(float s, const float3& a) { return make_float3(s + a.x, s + a.y, s + a.z); }
__device__ __forceinline__ float3 operator-(const float3& a) { return make_float3(-a.x, -a.y, -a.z); }
__device__ __forceinline__ void operator+=(float3& a, const float3& b) { a.x += b.x; a.y += b.y; a.z += b.z; }
__device__ __forceinline__ float4 operator*(const float4& a, const float4& b) { return make_float4(a.x * b.x, a.y * b.y, a.z * b.z, a.w * b.w); }
__device__ __forceinline__ float4 operator*(const float4& a, float s) { return make_float4(a.x * s, a.y * s, a.z * s, a.w * s); }
__device__ __forceinline__ float4 operator*(float s, const float4& a) { return make_float4(s * a.x, s * a.y, s * a.z, s * a.w); }
__device__ __forceinline__ float4 operator-(const float4& a, const float4& b) { return make_float4(a.x - b.x, a.y - b.y, a.z - b.z, a.w - b.w); }
__device__ __forceinline__ float4 operator+(const float4& a, const float4& b) { return make_float4(a.x + b.x, a.y + b.y, a.z + b.z, a.w + b.w); }
__device__ __forceinline__ void operator+=(float4& a, const float4& b) { a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w; }
__device__ __forceinline__ float3 normalize(const float3& v) { const float inv_len = rsqrtf(dot(v, v)); return v * inv_len; }
__device__ __forceinline__ float length(const float3& v) { return sqrtf(dot(v, v)); }

__device__ __forceinline__ float4 ldg4(const float* p) { return __ldg(reinterpret_cast<const float4*>(p)); }

// ---------------------------------------------------------------------------
// PTX wrappers: mbarrier + bulk asynchronous copy (TMA, non-tensor, single-CTA destination)
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("{\n\t.reg .b64 st;\n\tmbarrier.arrive.shared::cta.b64 st, [%0];\n\t}" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("{\n\t.reg .b64 st;\n\tmbarrier.arrive.expect_tx.shared::cta.b64 st, [%0], %1;\n\t}" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded wait: gives up after `limit` polls and reports failure instead of spinning forever.
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity, uint32_t limit = (1u << 22)) {
    for (uint32_t i = 0; i < limit; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}
// global -> shared bulk copy; src/dst 16-byte aligned, bytes a multiple of 16; completion is
// signalled on the mbarrier as transferred bytes.
__device__ __forceinline__ void bulk_copy_g2s(void* dst_smem, const void* src_gmem, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_u32(dst_smem)), "l"(src_gmem), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ unsigned int lanemask_lt() { unsigned int m; asm("mov.u32 %0, %%lanemask_lt;" : "=r"(m)); return m; }

// ---------------------------------------------------------------------------
// Compact gradient rows (multi-GPU gradient exchange).  A buffer is one 64-byte header followed by 64-byte rows,
// one per Gaussian the view kept, in no particular order:
//     float4 0: Gaussian index (bits), dL/dposition          float4 2: dL/drotation (r, x, y, z)
//     float4 1: dL/dscale, dL/dopacity                       float4 3: dL/drgb after the clamp mask, 0
// The rows of grad_sh_0 and grad_sh_rest are products of dL/drgb with functions of the view direction
// (kernel_utils.cuh:190-281 of the reference), so a reader that has the camera position rebuilds them.
// ---------------------------------------------------------------------------
struct CompactGradientHeader {
    unsigned int count;            // rows appended (may exceed the capacity: rows beyond it were dropped)
    float cam_x, cam_y, cam_z;     // camera position of the view the rows were computed for
    unsigned int active_sh_bases;  // 1, 4, 9 or 16
    unsigned int reserved[11];
};
static_assert(sizeof(CompactGradientHeader) == 64, "the header takes one row");
constexpr int kCompactRowFloat4s = 4;
constexpr float kShBand0 = 0.28209479177387814f;

// dL/dsh_rest of one Gaussian: rows[i] = (basis function i + 1 of `dir`) * grad_rgb for the active bases; returns how many
// rows were written (0, 3, 8 or 15).  One definition for the kernel that writes dense gradients and for the kernels that
// rebuild them from compact rows, so that both produce the same bits.
__device__ __forceinline__ int sh_rest_gradient_rows(const float3& dir, const float3& grad_rgb, int active_sh_bases, float3 (&rows)[15]) {
    if (active_sh_bases <= 1) return 0;
    const float dx = dir.x, dy = dir.y, dz = dir.z;
    rows[0] = (-0.48860251190291987f * dy) * grad_rgb;
    rows[1] = (0.48860251190291987f * dz) * grad_rgb;
    rows[2] = (-0.48860251190291987f * dx) * grad_rgb;
    if (active_sh_bases <= 4) return 3;
    const float sxx = dx * dx, syy = dy * dy, szz = dz * dz, sxy = dx * dy, sxz = dx * dz, syz = dy * dz;
    rows[3] = (1.0925484305920792f * sxy) * grad_rgb;
    rows[4] = (-1.0925484305920792f * syz) * grad_rgb;
    rows[5] = (0.94617469575755997f * szz - 0.31539156525251999f) * grad_rgb;
    rows[6] = (-1.0925484305920792f * sxz) * grad_rgb;
    rows[7] = (0.54627421529603959f * sxx - 0.54627421529603959f * syy) * grad_rgb;
    if (active_sh_bases <= 9) return 8;
    rows[8] = (0.59004358992664352f * dy * (-3.0f * sxx + syy)) * grad_rgb;
    rows[9] = (2.8906114426405538f * sxy * dz) * grad_rgb;
    rows[10] = (0.45704579946446572f * dy * (1.0f - 5.0f * szz)) * grad_rgb;
    rows[11] = (0.3731763325901154f * dz * (5.0f * szz - 3.0f)) * grad_rgb;
    rows[12] = (0.45704579946446572f * dx * (1.0f - 5.0f * szz)) * grad_rgb;
    rows[13] = (1.4453057213202769f * dz * (sxx - syy)) * grad_rgb;
    rows[14] = (0.59004358992664352f * dx * (-sxx + 3.0f * syy)) * grad_rgb;
    return 15;
}

}  // namespace htgs
