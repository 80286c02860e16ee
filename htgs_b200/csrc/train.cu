// Backward pass of the rasterizer.
//
// Replaces the backward blend_cu / preprocess_cu pairs of the reference
//   HYBRID_BLEND                rasterization/include/hybrid_blend/kernels/backward.cuh:10-331
//   ALPHA_BLEND_FIRST_K         rasterization/include/alpha_blend_first_k/kernels/backward.cuh:10-206
//   ALPHA_BLEND_GLOBAL_ORDERING rasterization/include/alpha_blend_global_ordering/kernels/backward.cuh:10-251
//   OIT_BLEND                   rasterization/include/oit_blend/kernels/backward.cuh:10-290
// and the helpers convert_quaternion_to_rotation_matrix_backward / convert_sh_to_rgb_backward
// (rasterization/include/kernel_utils.cuh:44-61, 190-281).
//
// The chain rule is the reference's: gradients flow through alpha = opacity * G and the colour only
// (not through depth, thresholds, the min(.,1) clamp or the bounds).  The organisation is new:
//  * every mode accumulates the same per-Gaussian record of five float4 (dL/dVPMT1, dL/dVPMT2, dL/dVPMT4,
//    (dL/drgb, dL/dopacity), (sum |dL/dposition|, -, -, -)) with 16-byte vector reductions
//    (red.global.add.v4.f32): 4-5 per (Gaussian, tile) instead of 15-17 scalar atomics, and one
//    per-Gaussian kernel turns the record into the six output gradients (the reference repeats the
//    scale / rotation chain rule per fragment in two of its modes);
//  * HYBRID / FIRST_K / OIT: one thread per Gaussian of a tile batch first builds the 64-bit mask of
//    tile pixels its conservative outline can touch (3 flops per pixel); the (Gaussian, pixel) pairs of the
//    batch are then split evenly over the threads.  The forward pass saves core entries as positions in the
//    tile's list, so which pairs are core entries is a table filled once per batch, not a search per pair;
//  * GLOBAL_ORDERING needs the running transmittance per pixel, so it stays pixel-parallel, in independent
//    8x8-pixel CTAs; a warp only walks the staged Gaussians whose outline reaches its pixels, and the 32
//    pixel contributions to one Gaussian are summed with a transposing shuffle reduction into a
//    shared-memory record per staged Gaussian, flushed with vector reductions once per batch.
#include "kernels.h"

namespace htgs {

namespace {

__device__ __forceinline__ void red_add_v4(float4* addr, const float4& v) {
    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
}

// The backward pass is not bit-identical to the reference's in any case (its sums are atomic), so where a value only
// scales a gradient term it uses the hardware approximations (1 ulp reciprocal, 2 ulp exp2) instead of the IEEE sequences:
// about 25 of the ~160 instructions per pair.
__device__ __forceinline__ float rcp_approx(float x) { float y; asm("rcp.approx.f32 %0, %1;" : "=f"(y) : "f"(x)); return y; }
__device__ __forceinline__ float exp_approx(float x) { float y; asm("ex2.approx.f32 %0, %1;" : "=f"(y) : "f"(x * 1.4426950408889634f)); return y; }

// Whether the forward pass rejected the fragment for `alpha < min_alpha`.  The forward decides with IEEE arithmetic
// (1.0f / denominator, expf); the approximate alpha computed here differs from that value by less than 1e-6 of itself
// (1 ulp reciprocal, 2 ulp exp2, and the rounding of an exponent of magnitude <= 8), so it settles the question unless
// it lies within 4e-6 of the threshold, and only then is the forward's own arithmetic repeated: the decision is the
// forward's in every case, the approximations only ever scale gradient terms.
template <typename MT>
__device__ __forceinline__ bool rejected_by_forward(float alpha_approx, float opacity, float numerator_rho2, float denominator) {
    if (fabsf(alpha_approx - MT::min_alpha) < 4e-6f * MT::min_alpha) {
        const float G = expf(-0.5f * numerator_rho2 * (1.0f / denominator));
        return fminf(opacity * G, kMaxFragmentAlpha) < MT::min_alpha;
    }
    return alpha_approx < MT::min_alpha;
}

struct PairGrad {      // what one (pixel, Gaussian) pair adds to the Gaussian's record
    float4 dT1, dT2, dT4;
};

// Gradient of rho^2 = |m|^2 / |d|^2 w.r.t. the two planes through the pixel ray, then w.r.t. the rows
// VPMT1, VPMT2, VPMT4 (hybrid_blend/kernels/backward.cuh:258-285).
__device__ __forceinline__ PairGrad pair_gradient(const float4& plane_x_diag, const float4& plane_y_diag, const float3& m, const float3& d,
                                                  float numerator_rho2, float denominator_rcp, float dL_drho2, float pixel_x, float pixel_y) {
    const float dL_dnum = dL_drho2 * denominator_rcp;
    const float dL_ddenom = dL_drho2 * -numerator_rho2 * denominator_rcp * denominator_rcp;
    const float3 dL_dm = dL_dnum * 2.0f * m;
    const float3 dL_dd = dL_ddenom * 2.0f * d;
    const float3 nx = f3(plane_x_diag), ny = f3(plane_y_diag);
    const float4 dpx = make_float4(
        -plane_y_diag.w * dL_dm.x - plane_y_diag.z * dL_dd.y + plane_y_diag.y * dL_dd.z,
        -plane_y_diag.w * dL_dm.y + plane_y_diag.z * dL_dd.x - plane_y_diag.x * dL_dd.z,
        -plane_y_diag.w * dL_dm.z - plane_y_diag.y * dL_dd.x + plane_y_diag.x * dL_dd.y,
        dot(ny, dL_dm));
    const float4 dpy = make_float4(
        plane_x_diag.w * dL_dm.x + plane_x_diag.z * dL_dd.y - plane_x_diag.y * dL_dd.z,
        plane_x_diag.w * dL_dm.y - plane_x_diag.z * dL_dd.x + plane_x_diag.x * dL_dd.z,
        plane_x_diag.w * dL_dm.z + plane_x_diag.y * dL_dd.x - plane_x_diag.x * dL_dd.y,
        -dot(nx, dL_dm));
    PairGrad g;
    g.dT1 = dpx;
    g.dT2 = dpy;
    g.dT4 = (-pixel_x) * dpx - pixel_y * dpy;
    return g;
}

struct CameraCols { float3 c1, c2, c3; };   // columns 1..3 of rows (1,2,4) of VPM
__device__ __forceinline__ CameraCols load_camera_cols(const float* __restrict__ VPM) {
    const float4 r1 = ldg4(VPM), r2 = ldg4(VPM + 4), r4 = ldg4(VPM + 12);
    return {make_float3(r1.x, r2.x, r4.x), make_float3(r1.y, r2.y, r4.y), make_float3(r1.z, r2.z, r4.z)};
}

constexpr int kBwdThreads = 128;       // threads per tile: one staged instance each, and an even share of the batch's pairs
constexpr int kBwdThreadsLog2 = 7;
constexpr int kBwdMinBlocks = 5;       // resident CTAs per SM the register budget is held to (shared memory allows as many)
template <int MODE, int K> struct BwdSmem {
    static constexpr bool has_core = (MODE == HTGS_MODE_HYBRID_BLEND || MODE == HTGS_MODE_ALPHA_BLEND_FIRST_K);
    static constexpr bool has_tail = (MODE == HTGS_MODE_HYBRID_BLEND || MODE == HTGS_MODE_OIT_BLEND);
    static constexpr int idx_stride = ((K + 3) / 4) * 4 + 4;         // words per pixel row: 16-byte rows, odd multiple of 4 words -> conflict-free uint4 reads
    static constexpr size_t idx_off = 0;
    static constexpr size_t idx_bytes = has_core ? size_t(idx_stride) * 64 * 4 : 0;
    static constexpr size_t cg_off = idx_off + idx_bytes;
    static constexpr size_t cg_bytes = has_core ? size_t(K) * 64 * 16 : 0;
    static constexpr size_t tc_off = cg_off + cg_bytes;
    static constexpr size_t tc_bytes = has_tail ? 64 * 16 : 0;
    static constexpr size_t ta_off = tc_off + tc_bytes;
    static constexpr size_t ta_bytes = has_tail ? 64 * 4 : 0;
    static constexpr size_t stage_off = (ta_off + ta_bytes + 15) & ~size_t(15);
    static constexpr size_t stage_bytes = kBwdThreads * (4 * 16 + 8 + 4) + (kBwdThreads + 1) * 4 + 12;
    static constexpr size_t core_off = (stage_off + stage_bytes + 15) & ~size_t(15);     // [NT][64] core entry of each (staged instance, pixel) pair
    static constexpr size_t core_bytes = has_core ? size_t(kBwdThreads) * 64 : 0;
    static constexpr size_t total = core_off + core_bytes;
};

// HYBRID_BLEND / ALPHA_BLEND_FIRST_K / OIT_BLEND: one CTA per 8x8 tile, one thread per Gaussian of a batch of kBwdThreads.
template <int MODE, int K, bool ABS_GRAD>
__global__ void __launch_bounds__(kBwdThreads, kBwdMinBlocks) backward_tile_kernel(
    const uint2* __restrict__ tile_ranges, const uint32_t* __restrict__ prims_sorted, const EvalRecord* __restrict__ eval,
    const CullRecord* __restrict__ cull, TrainPixelBuffers tin, const float* __restrict__ grad_image, const float* __restrict__ VPM,
    float4* __restrict__ accum, uint32_t width, uint32_t height, uint32_t grid_w, uint32_t g_first, uint32_t g_end)
{
    using MT = ModeTraits<MODE>;
    using SM = BwdSmem<MODE, K>;
    constexpr bool kHybrid = MODE == HTGS_MODE_HYBRID_BLEND;
    constexpr bool kFirstK = MODE == HTGS_MODE_ALPHA_BLEND_FIRST_K;
    extern __shared__ __align__(16) unsigned char smem[];
    [[maybe_unused]] uint32_t* s_idx = reinterpret_cast<uint32_t*>(smem + SM::idx_off);   // [64 pixels][idx_stride] positions in the tile's list
    [[maybe_unused]] signed char* s_core = reinterpret_cast<signed char*>(smem + SM::core_off);
    [[maybe_unused]] float4* s_cg = reinterpret_cast<float4*>(smem + SM::cg_off);          // [K][64] (W * grad_pixel, A . grad_pixel)
    [[maybe_unused]] float4* s_tc = reinterpret_cast<float4*>(smem + SM::tc_off);          // [64] (full_weight * grad_pixel, common term)
    [[maybe_unused]] float* s_ta = reinterpret_cast<float*>(smem + SM::ta_off);            // [64] term divided by (1 - alpha)

    const uint32_t tid = threadIdx.x;
    const uint32_t tile_x = blockIdx.x, tile_y = blockIdx.y;
    const uint2 tile_range = tile_ranges[tile_y * grid_w + tile_x];
    uint2 range = tile_range;
    // A pass over the Gaussians [g_first, g_end) only: a tile's list is ascending in Gaussian index for these modes (instances
    // are emitted in index order and the tile sort is stable), so the pass walks one contiguous piece of it.
    if (g_first != 0u || g_end != 0xffffffffu) {
        auto lower_bound = [&](uint32_t lo, uint32_t hi, uint32_t g) {
            while (lo < hi) { const uint32_t mid = (lo + hi) >> 1; if (__ldg(prims_sorted + mid) < g) lo = mid + 1; else hi = mid; }
            return lo;
        };
        range.x = lower_bound(tile_range.x, tile_range.y, g_first);
        range.y = lower_bound(range.x, tile_range.y, g_end);
    }
    if (range.x >= range.y) return;
    const uint32_t n_pixels = width * height;
    const uint32_t PP = tin.padded_pixels;
    constexpr uint32_t NT = kBwdThreads;
    const uint32_t pix = tid & 63, part = tid >> 6;          // the per-pixel terms are set up by NT / 64 threads per pixel
    const uint32_t slot = (tile_y * grid_w + tile_x) * 64 + pix;

    // Software pipeline of the staging loads: the record and outline of the instance a thread stages in batch b + 1 are
    // requested while batch b is processed (its index was requested one batch earlier still), so that their latency
    // overlaps the pair loop instead of sitting between two barriers.  The first indices are requested before the
    // per-pixel terms are read, so that the two chains of dependent loads at the start of a tile overlap as well.
    uint32_t g_cur = 0, g_nxt = 0;
    float4 pT1 = make_float4(0, 0, 0, 0), pT2 = pT1, pT4 = pT1, pRGBA = pT1, pc0 = pT1;
    float pcc = 0.0f;
    auto request = [&](uint32_t g) {
        const float* rec = reinterpret_cast<const float*>(eval + g);
        pT1 = ldg4(rec); pT2 = ldg4(rec + 4); pT4 = ldg4(rec + 8); pRGBA = ldg4(rec + 16);
        pc0 = ldg4(reinterpret_cast<const float*>(cull + g));
        pcc = __ldg(reinterpret_cast<const float*>(cull + g) + 4);
    };
    if (range.x + tid < range.y) g_cur = __ldg(prims_sorted + range.x + tid);
    if (range.x + NT + tid < range.y) g_nxt = __ldg(prims_sorted + range.x + NT + tid);
    // ---- per-pixel terms of this tile (hybrid_blend/kernels/backward.cuh:137-176, oit_blend/kernels/backward.cuh:131-156)
    {
        const uint32_t px_i = tile_x * 8 + (pix & 7), py_i = tile_y * 8 + (pix >> 3);
        const bool inside = px_i < width && py_i < height;
        float3 grad_pixel = make_float3(0.0f, 0.0f, 0.0f);
        if (inside) {
            const uint32_t pixel_idx = width * py_i + px_i;
            grad_pixel = make_float3(__ldg(grad_image + pixel_idx), __ldg(grad_image + n_pixels + pixel_idx), __ldg(grad_image + 2 * n_pixels + pixel_idx));
        }
        if constexpr (SM::has_core) {
            #pragma unroll
            for (int k0 = 0; k0 < K; k0 += int(NT / 64)) {
                const int k = k0 + int(part);
                if (k >= K) break;
                uint32_t idx = 0xffffffffu;
                float4 cg = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                if (inside) {
                    idx = tin.idx_core[k * PP + slot];
                    if (idx != 0xffffffffu) {
                        const float4 info = tin.info_core[k * PP + slot];
                        const float3 drgb = info.w * grad_pixel;
                        cg = make_float4(drgb.x, drgb.y, drgb.z, dot(f3(info), grad_pixel));
                    }
                }
                s_idx[pix * SM::idx_stride + k] = idx;
                s_cg[k * 64 + pix] = cg;
            }
        }
        if constexpr (SM::has_tail) {
            float4 tc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            float ta = 0.0f;
            if (inside) {
                const float3 rgb_tail = make_float3(tin.info_tail[slot], tin.info_tail[PP + slot], tin.info_tail[2 * PP + slot]);
                const float alpha_sum_rcp = tin.info_tail[3 * PP + slot];
                const float transmittance_tail = tin.info_tail[4 * PP + slot];
                const float transmittance_core = kHybrid ? tin.info_tail[5 * PP + slot] : 1.0f;
                const float weight_tail = transmittance_core * alpha_sum_rcp;
                const float full_weight_tail = weight_tail * (1.0f - transmittance_tail);
                const float rgb_dot_grad = dot(rgb_tail, grad_pixel);
                const float3 part = full_weight_tail * grad_pixel;
                tc = make_float4(part.x, part.y, part.z, -full_weight_tail * alpha_sum_rcp * rgb_dot_grad);
                ta = weight_tail * transmittance_tail * rgb_dot_grad;
            }
            if (part == 0) {
                s_tc[pix] = tc;
                s_ta[pix] = ta;
            }
        }
    }
    // pixels of the tile that exist in the image, as a 64-bit mask (bit = row * 8 + column)
    uint64_t inside_mask = 0;
    {
        const uint32_t cols = min(8u, width - tile_x * 8), rows = min(8u, height - tile_y * 8);
        const uint64_t row_bits = (1ull << cols) - 1ull;
        for (uint32_t r = 0; r < rows; ++r) inside_mask |= row_bits << (8 * r);
    }
    [[maybe_unused]] CameraCols cam;
    if constexpr (ABS_GRAD) cam = load_camera_cols(VPM);
    if (range.x + tid < range.y) request(g_cur);
    __syncthreads();

    // ---- batches of NT instances; the (Gaussian, pixel) candidate pairs of a batch are split EVENLY over the
    //      NT threads (pairs of one Gaussian are contiguous, so a thread walks a few Gaussians back to back)
    float4* s_T1 = reinterpret_cast<float4*>(smem + SM::stage_off);
    float4* s_T2 = s_T1 + NT;
    float4* s_T4 = s_T2 + NT;
    float4* s_rgba = s_T4 + NT;
    unsigned long long* s_mask = reinterpret_cast<unsigned long long*>(s_rgba + NT);
    uint32_t* s_g = reinterpret_cast<uint32_t*>(s_mask + NT);
    uint32_t* s_off = s_g + NT;          // [NT + 1] exclusive prefix of the per-Gaussian pair counts
    __shared__ uint32_t s_warp_total[NT / 32];
    const float x0 = float(tile_x * 8), y0 = float(tile_y * 8);
    const uint32_t lane = tid & 31, warp = tid >> 5;
    // The training forward saved, per pixel and core entry, the POSITION of the entry's Gaussian in the tile's list, so the
    // entries that belong to a batch are those within NT of its start, and position - start is the staged slot.
    // FIRST_K gives gradient to stored fragments only: there the entries also set the pixel masks of the staged instances.
    // `limit`: staged instances of the batch (entries further down the list belong to a later batch, or - in a pass over a
    // range of Gaussians - to Gaussians beyond the range, whose slots in this batch hold nothing).
    [[maybe_unused]] auto scatter_core_entries = [&](uint32_t batch_pos, uint32_t limit) {
        const uint4* row = reinterpret_cast<const uint4*>(s_idx + pix * SM::idx_stride);
        auto put = [&](uint32_t j, int k) {
            s_core[j * 64 + pix] = (signed char)k;
            if constexpr (kFirstK) atomicOr(reinterpret_cast<uint32_t*>(s_mask + j) + (pix >> 5), 1u << (pix & 31));
        };
        #pragma unroll
        for (int k4 = 0; k4 < (K + 3) / 4; k4 += int(NT / 64)) {
            const int q = k4 + int(part);
            if (q >= (K + 3) / 4) break;
            const uint4 v = row[q];
            const uint32_t j0 = v.x - batch_pos, j1 = v.y - batch_pos, j2 = v.z - batch_pos, j3 = v.w - batch_pos;
            if (j0 < limit) put(j0, 4 * q);
            if (4 * q + 1 < K && j1 < limit) put(j1, 4 * q + 1);
            if (4 * q + 2 < K && j2 < limit) put(j2, 4 * q + 2);
            if (4 * q + 3 < K && j3 < limit) put(j3, 4 * q + 3);
        }
    };
    for (uint32_t batch_begin = range.x; batch_begin < range.y; batch_begin += NT) {
        __syncthreads();                  // previous batch fully consumed
        const uint32_t inst = batch_begin + tid;
        uint64_t my_mask = 0;
        const bool valid = inst < range.y;
        const float4 c0 = pc0;
        const float cc = pcc;
        if (valid) {
            s_T1[tid] = pT1; s_T2[tid] = pT2; s_T4[tid] = pT4; s_rgba[tid] = pRGBA;
            s_g[tid] = g_cur;
        }
        if constexpr (SM::has_core) {      // no pair of my instance is a core entry until the scatter below says so
            uint4* row = reinterpret_cast<uint4*>(s_core + tid * 64);
            const uint4 none = make_uint4(0xffffffffu, 0xffffffffu, 0xffffffffu, 0xffffffffu);
            row[0] = none; row[1] = none; row[2] = none; row[3] = none;
        }
        // next batch: its index is here, request its data; request the index of the batch after it
        g_cur = g_nxt;
        if (inst + NT < range.y) request(g_cur);
        if (inst + 2 * NT < range.y) g_nxt = __ldg(prims_sorted + inst + 2 * NT);
        if constexpr (kFirstK) {
            s_mask[tid] = 0;
            __syncthreads();
            scatter_core_entries(batch_begin - __ldg(&tile_ranges[blockIdx.y * grid_w + blockIdx.x].x), min(NT, range.y - batch_begin));   // the forward's stored core positions count from the start of the tile's list
            __syncthreads();
            my_mask = s_mask[tid];
        } else if (valid) {
            const float dx0 = x0 - c0.x, dy0 = y0 - c0.y;
            #pragma unroll
            for (int r = 0; r < 8; ++r) {
                const float dy = dy0 + float(r);
                const float b2dy = c0.w * dy, cdy2 = cc * dy * dy;
                #pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const float dx = dx0 + float(i);
                    const float q = dx * (c0.z * dx + b2dy) + cdy2;
                    if (q <= 1.0f) my_mask |= 1ull << (r * 8 + i);
                }
            }
            my_mask &= inside_mask;
        }
        if constexpr (!kFirstK) s_mask[tid] = my_mask;
        const uint32_t cnt = __popcll(my_mask);
        uint32_t inc = cnt;
        #pragma unroll
        for (int o = 1; o < 32; o <<= 1) { const uint32_t t = __shfl_up_sync(0xffffffffu, inc, o); if (lane >= uint32_t(o)) inc += t; }
        if (lane == 31) s_warp_total[warp] = inc;
        __syncthreads();
        uint32_t excl = inc - cnt, total_pairs = 0;
        #pragma unroll
        for (uint32_t w = 0; w < NT / 32; ++w) {
            const uint32_t t = s_warp_total[w];
            if (w < warp) excl += t;
            total_pairs += t;
        }
        s_off[tid] = excl;
        if (tid == 0) s_off[NT] = total_pairs;
        if constexpr (SM::has_core && !kFirstK) scatter_core_entries(batch_begin - __ldg(&tile_ranges[blockIdx.y * grid_w + blockIdx.x].x), min(NT, range.y - batch_begin));   // the forward's stored core positions count from the start of the tile's list
        __syncthreads();
        if (total_pairs == 0) continue;
        // my share of the pairs
        const uint32_t lo = uint32_t((uint64_t(tid) * total_pairs) >> kBwdThreadsLog2), hi = uint32_t((uint64_t(tid + 1) * total_pairs) >> kBwdThreadsLog2);
        uint32_t remaining = hi - lo;
        if (remaining == 0) continue;
        uint32_t j = 0;
        {
            uint32_t a = 0, b = NT;      // last j with s_off[j] <= lo
            #pragma unroll
            for (int it = 0; it < kBwdThreadsLog2; ++it) { const uint32_t mid = (a + b) >> 1; if (s_off[mid] <= lo) a = mid; else b = mid; }
            j = a;
        }
        uint64_t mask = s_mask[j];
        for (uint32_t skip = lo - s_off[j]; skip > 0; --skip) mask &= mask - 1;     // drop the pairs that belong to the previous thread
        float4 T1 = s_T1[j], T2 = s_T2[j], T4 = s_T4[j], rgba = s_rgba[j];
        uint32_t g = s_g[j];
        float4 aT1 = make_float4(0, 0, 0, 0), aT2 = aT1, aT4 = aT1, aC = aT1;   // aC = (dL/drgb, dL/dopacity)
        [[maybe_unused]] float abs_grad = 0.0f;
        bool touched = false;
        auto flush = [&]() {
            if (touched) {
                float4* rec = accum + size_t(g) * 5;
                red_add_v4(rec, aT1); red_add_v4(rec + 1, aT2); red_add_v4(rec + 2, aT4); red_add_v4(rec + 3, aC);
                if constexpr (ABS_GRAD) red_add_v4(rec + 4, make_float4(abs_grad, 0.0f, 0.0f, 0.0f));
            }
            aT1 = make_float4(0, 0, 0, 0); aT2 = aT1; aT4 = aT1; aC = aT1; abs_grad = 0.0f; touched = false;
        };
        for (; remaining > 0; --remaining) {
            while (mask == 0) {           // next Gaussian of my share (its mask is non-empty somewhere before `hi`)
                flush();
                ++j;
                mask = s_mask[j];
                T1 = s_T1[j]; T2 = s_T2[j]; T4 = s_T4[j]; rgba = s_rgba[j]; g = s_g[j];
            }
            const uint32_t p = uint32_t(__ffsll((long long)mask) - 1);
            mask &= mask - 1;
            const float pixel_x = x0 + float(p & 7), pixel_y = y0 + float(p >> 3);
            const float4 plane_x_diag = T1 - T4 * pixel_x;
            const float4 plane_y_diag = T2 - T4 * pixel_y;
            const float3 nx = f3(plane_x_diag), ny = f3(plane_y_diag);
            const float3 m = plane_x_diag.w * ny - nx * plane_y_diag.w;
            const float3 d = cross(nx, ny);
            const float numerator_rho2 = dot(m, m);
            const float denominator = dot(d, d);
            int core_idx = -1;
            if constexpr (SM::has_core) core_idx = s_core[j * 64 + p];
            if constexpr (kFirstK) {
                if (core_idx < 0) continue;                    // only stored fragments carry gradient (first_k backward.cuh:84-87)
            } else {
                if (numerator_rho2 > MT::max_cutoff_sq * denominator) continue;
            }
            const float denominator_rcp = rcp_approx(denominator);
            const float G = exp_approx(-0.5f * numerator_rho2 * denominator_rcp);
            const float alpha = fminf(rgba.w * G, kMaxFragmentAlpha);
            if constexpr (!kFirstK) { if (rejected_by_forward<MT>(alpha, rgba.w, numerator_rho2, denominator)) continue; }
            float3 dL_drgb;
            float dL_dalpha;
            if (core_idx >= 0) {
                const float4 cg = s_cg[core_idx * 64 + p];
                dL_drgb = f3(cg);
                dL_dalpha = cg.w;
            } else {
                if constexpr (SM::has_tail) {
                    const float4 tc = s_tc[p];
                    dL_drgb = f3(tc) * alpha;
                    dL_dalpha = tc.w + dot(f3(rgba), f3(tc)) + s_ta[p] * rcp_approx(fmaxf(1.0f - alpha, kOneMinusAlphaEps));
                } else {
                    continue;
                }
            }
            aC.x += dL_drgb.x; aC.y += dL_drgb.y; aC.z += dL_drgb.z;
            touched = true;
            if (dL_dalpha == 0.0f) continue;
            aC.w += dL_dalpha * G;
            const float dL_dG = dL_dalpha * rgba.w;
            const float dL_drho2 = dL_dG * -0.5f * G;
            const PairGrad pg = pair_gradient(plane_x_diag, plane_y_diag, m, d, numerator_rho2, denominator_rcp, dL_drho2, pixel_x, pixel_y);
            aT1 += pg.dT1; aT2 += pg.dT2; aT4 += pg.dT4;
            if constexpr (ABS_GRAD) {
                const float3 c4 = make_float3(pg.dT1.w, pg.dT2.w, pg.dT4.w);
                abs_grad += fabsf(dot(cam.c1, c4)) + fabsf(dot(cam.c2, c4)) + fabsf(dot(cam.c3, c4));
            }
        }
        flush();
    }
}

// Sum of 16 per-lane values over the warp in 16 shuffles instead of 80: at every step a lane keeps one half of its
// values, hands the other half to its partner and adds what the partner hands over.  After the steps with lane bits
// 4, 3, 2, 1 a lane holds ONE value summed over the 16 lanes that share its bit 0; the last shuffle completes it.
// On return the lane holds the warp total of v[transpose_reduce_index(lane)].
__device__ __forceinline__ uint32_t transpose_reduce_index(uint32_t lane) { return (lane >> 1) & 15u; }   // bit 4 -> 8, bit 3 -> 4, bit 2 -> 2, bit 1 -> 1
__device__ __forceinline__ float transpose_reduce16(const float (&v)[16], uint32_t lane) {
    float a8[8], a4[4], a2[2];
    const bool up16 = lane & 16u, up8 = lane & 8u, up4 = lane & 4u, up2 = lane & 2u;
    #pragma unroll
    for (int i = 0; i < 8; ++i) a8[i] = (up16 ? v[i + 8] : v[i]) + __shfl_xor_sync(0xffffffffu, up16 ? v[i] : v[i + 8], 16);
    #pragma unroll
    for (int i = 0; i < 4; ++i) a4[i] = (up8 ? a8[i + 4] : a8[i]) + __shfl_xor_sync(0xffffffffu, up8 ? a8[i] : a8[i + 4], 8);
    #pragma unroll
    for (int i = 0; i < 2; ++i) a2[i] = (up4 ? a4[i + 2] : a4[i]) + __shfl_xor_sync(0xffffffffu, up4 ? a4[i] : a4[i + 2], 4);
    float a1 = (up2 ? a2[1] : a2[0]) + __shfl_xor_sync(0xffffffffu, up2 ? a2[0] : a2[1], 2);
    a1 += __shfl_xor_sync(0xffffffffu, a1, 1);
    return a1;
}

// ALPHA_BLEND_GLOBAL_ORDERING: pixel-parallel, front to back in key order, using the final pixel colour so that
// "colour behind" = rgb_pixel - rgb_pixel_new (alpha_blend_global_ordering/kernels/backward.cuh:104-161).
// One CTA of two warps per 8x8 pixels; the four CTAs of a 16x16 binning tile walk the same list independently (a pixel
// shares no state with its neighbours) and each stops when ITS pixels are opaque.  Per batch of 64 staged Gaussians a
// warp first finds, with lane = Gaussian, which of them can touch its 8x4 pixels at all (the conservative outline the
// forward pass uses) and only walks those; the 16 values a pixel adds to a Gaussian's record are summed over the warp
// by transpose_reduce16 and added to a shared-memory record per staged Gaussian, flushed once per batch.
constexpr int kGoBatch = 64;
constexpr int kGoAccStride = 17;     // 16 values + sum |dL/dposition|; odd stride: rows and columns are both conflict-free
__global__ void __launch_bounds__(64) backward_global_kernel(
    const uint2* __restrict__ tile_ranges, const uint32_t* __restrict__ prims_sorted, const EvalRecord* __restrict__ eval,
    const CullRecord* __restrict__ cull, const float* __restrict__ grad_image, const float* __restrict__ image, const float* __restrict__ VPM,
    float4* __restrict__ accum, uint32_t width, uint32_t height, uint32_t grid_w, bool abs_grad_on)
{
    using MT = ModeTraits<HTGS_MODE_ALPHA_BLEND_GLOBAL_ORDERING>;
    __shared__ float4 s_T1[kGoBatch], s_T2[kGoBatch], s_T4[kGoBatch], s_rgba[kGoBatch], s_c0[kGoBatch];
    __shared__ float s_cc[kGoBatch];
    __shared__ uint32_t s_g[kGoBatch];
    __shared__ float s_acc[kGoBatch * kGoAccStride];
    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t tile_x = blockIdx.x, tile_y = blockIdx.y;                 // in units of 8 pixels
    const uint32_t px_i = tile_x * 8 + (tid & 7), py_i = tile_y * 8 + (tid >> 3);
    const bool inside = px_i < width && py_i < height;
    const float pixel_x = __uint2float_rn(px_i), pixel_y = __uint2float_rn(py_i);
    const float rect_x0 = float(tile_x * 8), rect_y0 = float(tile_y * 8 + warp * 4);
    const uint32_t n_pixels = width * height;
    float3 grad_pixel = make_float3(0, 0, 0), rgb_pixel = make_float3(0, 0, 0);
    if (inside) {
        const uint32_t pixel_idx = width * py_i + px_i;
        grad_pixel = make_float3(__ldg(grad_image + pixel_idx), __ldg(grad_image + n_pixels + pixel_idx), __ldg(grad_image + 2 * n_pixels + pixel_idx));
        rgb_pixel = make_float3(__ldg(image + pixel_idx), __ldg(image + n_pixels + pixel_idx), __ldg(image + 2 * n_pixels + pixel_idx));
    }
    const CameraCols cam = load_camera_cols(VPM);
    float3 rgb_pixel_new = make_float3(0, 0, 0);
    float transmittance = 1.0f;
    bool done = !inside;
    constexpr uint32_t kSplit = MT::tile_w / 8;                               // 8-pixel CTAs per binning tile edge
    const uint2 range = tile_ranges[(tile_y / kSplit) * grid_w + tile_x / kSplit];
    const uint32_t out_index = transpose_reduce_index(lane);
    for (uint32_t batch_begin = range.x; batch_begin < range.y; batch_begin += kGoBatch) {
        if (__syncthreads_count(done) == 64) break;
        const uint32_t batch = min(uint32_t(kGoBatch), range.y - batch_begin);
        if (tid < batch) {
            const uint32_t g = __ldg(prims_sorted + batch_begin + tid);
            const float* rec = reinterpret_cast<const float*>(eval + g);
            s_g[tid] = g;
            s_T1[tid] = ldg4(rec); s_T2[tid] = ldg4(rec + 4); s_T4[tid] = ldg4(rec + 8); s_rgba[tid] = ldg4(rec + 16);
            s_c0[tid] = ldg4(reinterpret_cast<const float*>(cull + g));
            s_cc[tid] = __ldg(reinterpret_cast<const float*>(cull + g) + 4);
        } else {
            s_c0[tid] = make_float4(__int_as_float(0x7f800000), 0.0f, 0.0f, 0.0f);   // an outline nothing is inside of
            s_cc[tid] = 0.0f;
        }
        for (uint32_t i = tid; i < kGoBatch * kGoAccStride; i += 64) s_acc[i] = 0.0f;
        __syncthreads();
        // which staged Gaussians can touch this warp's 8x4 pixels (lane = Gaussian)
        uint64_t todo = 0;
        #pragma unroll
        for (int half = 0; half < 2; ++half) {
            const float4 c0 = s_c0[half * 32 + lane];
            const float cc = s_cc[half * 32 + lane];
            const float dx0 = rect_x0 - c0.x, dy0 = rect_y0 - c0.y;
            bool touches = false;
            #pragma unroll
            for (int r = 0; r < 4; ++r) {
                const float dy = dy0 + float(r);
                const float b2dy = c0.w * dy, cdy2 = cc * dy * dy;
                #pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const float dx = dx0 + float(i);
                    const float q = dx * (c0.z * dx + b2dy) + cdy2;
                    touches |= q <= 1.0f;
                }
            }
            todo |= uint64_t(__ballot_sync(0xffffffffu, touches)) << (32 * half);
        }
        while (todo != 0) {
            if (__all_sync(0xffffffffu, done)) break;
            const uint32_t j = uint32_t(__ffsll((long long)todo) - 1);
            todo &= todo - 1;
            float v[16];
            #pragma unroll
            for (int c = 0; c < 16; ++c) v[c] = 0.0f;
            float v_abs = 0.0f;
            bool contributes = false;
            if (!done) {
                const float4 T1 = s_T1[j], T2 = s_T2[j], T4 = s_T4[j];
                const float4 plane_x_diag = T1 - T4 * pixel_x;
                const float4 plane_y_diag = T2 - T4 * pixel_y;
                const float3 nx = f3(plane_x_diag), ny = f3(plane_y_diag);
                const float3 m = plane_x_diag.w * ny - nx * plane_y_diag.w;
                const float3 d = cross(nx, ny);
                const float numerator_rho2 = dot(m, m);
                const float denominator = dot(d, d);
                if (!(numerator_rho2 > MT::max_cutoff_sq * denominator)) {
                    const float denominator_rcp = rcp_approx(denominator);
                    const float G = exp_approx(-0.5f * numerator_rho2 * denominator_rcp);
                    const float4 rgba = s_rgba[j];
                    const float opacity = rgba.w;
                    const float alpha = fminf(opacity * G, kMaxFragmentAlpha);
                    if (!rejected_by_forward<MT>(alpha, opacity, numerator_rho2, denominator)) {
                        const float blending_weight = transmittance * alpha;
                        const float3 dL_drgb = blending_weight * grad_pixel;
                        v[12] = dL_drgb.x; v[13] = dL_drgb.y; v[14] = dL_drgb.z;
                        contributes = true;
                        const float3 rgb = f3(rgba);
                        rgb_pixel_new += blending_weight * rgb;
                        const float one_minus_alpha = 1.0f - alpha;
                        const float one_minus_alpha_rcp = rcp_approx(fmaxf(one_minus_alpha, kOneMinusAlphaEps));
                        const float dL_dalpha = dot(transmittance * rgb - (rgb_pixel - rgb_pixel_new) * one_minus_alpha_rcp, grad_pixel);
                        if (dL_dalpha != 0.0f) {
                            v[15] = dL_dalpha * G;
                            const float dL_dG = dL_dalpha * opacity;
                            const float dL_drho2 = dL_dG * -0.5f * G;
                            const PairGrad pg = pair_gradient(plane_x_diag, plane_y_diag, m, d, numerator_rho2, denominator_rcp, dL_drho2, pixel_x, pixel_y);
                            v[0] = pg.dT1.x; v[1] = pg.dT1.y; v[2] = pg.dT1.z; v[3] = pg.dT1.w;
                            v[4] = pg.dT2.x; v[5] = pg.dT2.y; v[6] = pg.dT2.z; v[7] = pg.dT2.w;
                            v[8] = pg.dT4.x; v[9] = pg.dT4.y; v[10] = pg.dT4.z; v[11] = pg.dT4.w;
                            if (abs_grad_on) {
                                const float3 c4 = make_float3(pg.dT1.w, pg.dT2.w, pg.dT4.w);
                                v_abs = fabsf(dot(cam.c1, c4)) + fabsf(dot(cam.c2, c4)) + fabsf(dot(cam.c3, c4));
                            }
                        }
                        transmittance *= one_minus_alpha;
                        if (transmittance < kTransmittanceThreshold) done = true;
                    }
                }
            }
            if (__any_sync(0xffffffffu, contributes)) {
                const float total = transpose_reduce16(v, lane);
                if ((lane & 1u) == 0 && total != 0.0f) atomicAdd(&s_acc[j * kGoAccStride + out_index], total);
                if (abs_grad_on) {
                    #pragma unroll
                    for (int o = 16; o > 0; o >>= 1) v_abs += __shfl_xor_sync(0xffffffffu, v_abs, o);
                    if (lane == 0 && v_abs != 0.0f) atomicAdd(&s_acc[j * kGoAccStride + 16], v_abs);
                }
            }
        }
        __syncthreads();
        if (tid < batch) {
            const float* a = s_acc + tid * kGoAccStride;
            bool any = false;
            #pragma unroll
            for (int c = 0; c < 17; ++c) any |= a[c] != 0.0f;
            if (any) {
                float4* rec = accum + size_t(s_g[tid]) * 5;
                red_add_v4(rec, make_float4(a[0], a[1], a[2], a[3]));
                red_add_v4(rec + 1, make_float4(a[4], a[5], a[6], a[7]));
                red_add_v4(rec + 2, make_float4(a[8], a[9], a[10], a[11]));
                red_add_v4(rec + 3, make_float4(a[12], a[13], a[14], a[15]));
                if (abs_grad_on) red_add_v4(rec + 4, make_float4(a[16], 0.0f, 0.0f, 0.0f));
            }
        }
    }
}

// kernel_utils.cuh:44-61
__device__ __forceinline__ float4 quat_backward(const float4& q, const float (&dR)[9]) {
    const float r = q.x, x = q.y, y = q.z, z = q.w;
    const float r21_sub_r12 = dR[3] - dR[1], r21_add_r12 = dR[3] + dR[1];
    const float r13_sub_r31 = dR[2] - dR[6], r13_add_r31 = dR[2] + dR[6];
    const float r32_sub_r23 = dR[7] - dR[5], r32_add_r23 = dR[7] + dR[5];
    return make_float4(
        2.0f * (x * r32_sub_r23 + y * r13_sub_r31 + z * r21_sub_r12),
        2.0f * (r * r32_sub_r23 - 2.0f * x * (dR[4] + dR[8]) + y * r21_add_r12 + z * r13_add_r31),
        2.0f * (r * r13_sub_r31 + x * r21_add_r12 - 2.0f * y * (dR[0] + dR[8]) + z * r32_add_r23),
        2.0f * (r * r21_sub_r12 + x * r13_add_r31 + y * r32_add_r23 - 2.0f * z * (dR[0] + dR[4])));
}

// Per-Gaussian chain rule: accumulated record -> the six output gradients
// (hybrid_blend/kernels/backward.cuh:10-102; SH part kernel_utils.cuh:190-281).  Every output element is
// defined after the call (the launcher clears the tensors first), so the caller need not clear them.
//
// COMPACT: instead of the six dense rows (59 floats at SH degree 3) the kernel appends one 64-byte record per Gaussian the view
// kept to `out.compact_rows` (common.cuh: CompactGradientRow): the gradients of position, scale, rotation and opacity and the
// clamp-masked colour gradient.  The rows of grad_sh_0 / grad_sh_rest are (basis function of the view direction) x (colour
// gradient), so whoever knows the camera position can rebuild them (expand_compact_row below and exchange.cu); this is what
// the ranks of a multi-GPU trainer send one another instead of the dense rows.
template <bool COMPACT>
__global__ void __launch_bounds__(256) preprocess_backward_kernel(
    const float* __restrict__ positions, const float* __restrict__ scales, const float* __restrict__ rotations, const float* __restrict__ sh_rest,
    const float* __restrict__ M, const float* __restrict__ VPM, const float* __restrict__ cam_position_ptr,
    const uint32_t* __restrict__ n_touched, const uint8_t* __restrict__ clamp, const float4* __restrict__ accum, BackwardOutputs out,
    uint32_t n_primitives, int active_sh_bases, int total_sh_bases, uint32_t g_first, uint32_t g_end)
{
    const uint32_t idx = g_first + blockIdx.x * 256 + threadIdx.x;
    if constexpr (COMPACT) {
        if (blockIdx.x == 0 && threadIdx.x == 0) {      // header: the camera the receivers need (its first word, the row count, was cleared by the launcher)
            CompactGradientHeader* header = reinterpret_cast<CompactGradientHeader*>(out.compact_rows);
            header->cam_x = __ldg(cam_position_ptr); header->cam_y = __ldg(cam_position_ptr + 1); header->cam_z = __ldg(cam_position_ptr + 2);
            header->active_sh_bases = uint32_t(active_sh_bases);
        }
    }
    const bool kept = idx < g_end && n_touched[idx] != 0;      // outputs were cleared by the launcher
    if constexpr (!COMPACT) { if (!kept) return; }
    float3 grad_scale = make_float3(0, 0, 0), grad_rgb = make_float3(0, 0, 0), dL_dposition = make_float3(0, 0, 0);
    float4 grad_rotation = make_float4(0, 0, 0, 0);
    float grad_opacity = 0.0f;
    if (kept) {
    const float4 dT1 = accum[size_t(idx) * 5], dT2 = accum[size_t(idx) * 5 + 1], dT4 = accum[size_t(idx) * 5 + 2], dC = accum[size_t(idx) * 5 + 3];
    const float3 c1 = make_float3(dT1.x, dT2.x, dT4.x), c2 = make_float3(dT1.y, dT2.y, dT4.y), c3 = make_float3(dT1.z, dT2.z, dT4.z);
    const float3 c4 = make_float3(dT1.w, dT2.w, dT4.w);
    const float4 r1 = ldg4(VPM), r2 = ldg4(VPM + 4), r4 = ldg4(VPM + 12);
    const float3 VPM1 = f3(r1), VPM2 = f3(r2), VPM4 = f3(r4);
    const float3 VPM_c1 = make_float3(r1.x, r2.x, r4.x), VPM_c2 = make_float3(r1.y, r2.y, r4.y), VPM_c3 = make_float3(r1.z, r2.z, r4.z);

    const float3 scale = make_float3(scales[3 * size_t(idx)], scales[3 * size_t(idx) + 1], scales[3 * size_t(idx) + 2]);
    const float4 q = ldg4(rotations + 4 * size_t(idx));
    const float r = q.x, x = q.y, y = q.z, z = q.w;
    const float xx = x * x, yy = y * y, zz = z * z, xy = x * y, xz = x * z, yz = y * z, rx = r * x, ry = r * y, rz = r * z;
    const float3 R_c1 = make_float3(1.0f - 2.0f * (yy + zz), 2.0f * (xy + rz), 2.0f * (xz - ry));
    const float3 R_c2 = make_float3(2.0f * (xy - rz), 1.0f - 2.0f * (xx + zz), 2.0f * (yz + rx));
    const float3 R_c3 = make_float3(2.0f * (xz + ry), 2.0f * (yz - rx), 1.0f - 2.0f * (xx + yy));
    grad_scale = make_float3(
        dot(make_float3(dot(VPM1, R_c1), dot(VPM2, R_c1), dot(VPM4, R_c1)), c1),
        dot(make_float3(dot(VPM1, R_c2), dot(VPM2, R_c2), dot(VPM4, R_c2)), c2),
        dot(make_float3(dot(VPM1, R_c3), dot(VPM2, R_c3), dot(VPM4, R_c3)), c3));
    const float dR[9] = {
        dot(VPM_c1, c1) * scale.x, dot(VPM_c1, c2) * scale.y, dot(VPM_c1, c3) * scale.z,
        dot(VPM_c2, c1) * scale.x, dot(VPM_c2, c2) * scale.y, dot(VPM_c2, c3) * scale.z,
        dot(VPM_c3, c1) * scale.x, dot(VPM_c3, c2) * scale.y, dot(VPM_c3, c3) * scale.z};
    grad_rotation = quat_backward(q, dR);
    grad_opacity = dC.w;

    // colour: undo the clamp at 0, then SH backward
    const uint8_t cl = clamp[idx];
    grad_rgb = make_float3((cl & 1) ? 0.0f : dC.x, (cl & 2) ? 0.0f : dC.y, (cl & 4) ? 0.0f : dC.z);
    const float3 position = make_float3(positions[3 * size_t(idx)], positions[3 * size_t(idx) + 1], positions[3 * size_t(idx) + 2]);
    float3 drgb_dposition = make_float3(0, 0, 0);
    if (active_sh_bases > 1) {
        const float3* co = reinterpret_cast<const float3*>(sh_rest) + size_t(idx) * total_sh_bases;
        const float3 cam_position = make_float3(__ldg(cam_position_ptr), __ldg(cam_position_ptr + 1), __ldg(cam_position_ptr + 2));
        const float3 raw = position - cam_position;
        const float3 dir = normalize(raw);
        const float dx = dir.x, dy = dir.y, dz = dir.z;
        float3 gdx = -0.48860251190291987f * co[2];
        float3 gdy = -0.48860251190291987f * co[0];
        float3 gdz = 0.48860251190291987f * co[1];
        if (active_sh_bases > 4) {
            const float sxx = dx * dx, syy = dy * dy, szz = dz * dz, sxy = dx * dy, sxz = dx * dz, syz = dy * dz;
            gdx = gdx + (1.0925484305920792f * dy) * co[3] + (-1.0925484305920792f * dz) * co[6] + (1.0925484305920792f * dx) * co[7];
            gdy = gdy + (1.0925484305920792f * dx) * co[3] + (-1.0925484305920792f * dz) * co[4] + (-1.0925484305920792f * dy) * co[7];
            gdz = gdz + (-1.0925484305920792f * dy) * co[4] + (1.8923493915151202f * dz) * co[5] + (-1.0925484305920792f * dx) * co[6];
            if (active_sh_bases > 9) {
                gdx = gdx + (-3.5402615395598609f * sxy) * co[8] + (2.8906114426405538f * syz) * co[9]
                          + (0.45704579946446572f - 2.2852289973223288f * szz) * co[12] + (2.8906114426405538f * sxz) * co[13]
                          + (-1.7701307697799304f * sxx + 1.7701307697799304f * syy) * co[14];
                gdy = gdy + (-1.7701307697799304f * sxx + 1.7701307697799304f * syy) * co[8] + (2.8906114426405538f * sxz) * co[9]
                          + (0.45704579946446572f - 2.2852289973223288f * szz) * co[10] + (-2.8906114426405538f * syz) * co[13]
                          + (3.5402615395598609f * sxy) * co[14];
                gdz = gdz + (2.8906114426405538f * sxy) * co[9] + (-4.5704579946446566f * syz) * co[10]
                          + (5.597644988851731f * szz - 1.1195289977703462f) * co[11] + (-4.5704579946446566f * sxz) * co[12]
                          + (1.4453057213202769f * sxx - 1.4453057213202769f * syy) * co[13];
            }
        }
        const float3 gdir = make_float3(dot(gdx, grad_rgb), dot(gdy, grad_rgb), dot(gdz, grad_rgb));
        const float xr = raw.x, yr = raw.y, zr = raw.z;
        const float xxr = xr * xr, yyr = yr * yr, zzr = zr * zr, xyr = xr * yr, xzr = xr * zr, yzr = yr * zr;
        const float norm_sq = xxr + yyr + zzr;
        drgb_dposition = make_float3(
            (yyr + zzr) * gdir.x - xyr * gdir.y - xzr * gdir.z,
            -xyr * gdir.x + (xxr + zzr) * gdir.y - yzr * gdir.z,
            -xzr * gdir.x - yzr * gdir.y + (xxr + yyr) * gdir.z) * rsqrtf(norm_sq * norm_sq * norm_sq);
        if constexpr (!COMPACT) {
            float3 rows[15];
            const int written = sh_rest_gradient_rows(dir, grad_rgb, active_sh_bases, rows);
            float3* grad_sh_rest = reinterpret_cast<float3*>(out.grad_sh_rest) + size_t(idx) * total_sh_bases;
            #pragma unroll
            for (int i = 0; i < 15; ++i)
                if (i < written) grad_sh_rest[i] = rows[i];
        }
    }
    dL_dposition = make_float3(dot(VPM_c1, c4), dot(VPM_c2, c4), dot(VPM_c3, c4)) + drgb_dposition;
    if constexpr (!COMPACT) {
        reinterpret_cast<float3*>(out.grad_scales)[idx] = grad_scale;
        reinterpret_cast<float4*>(out.grad_rotations)[idx] = grad_rotation;
        out.grad_opacities[idx] = grad_opacity;
        reinterpret_cast<float3*>(out.grad_sh_0)[idx] = kShBand0 * grad_rgb;
        reinterpret_cast<float3*>(out.grad_positions)[idx] = dL_dposition;
    }
    if (out.densification_info != nullptr) {     // hybrid_blend/kernels/backward.cuh:85-98
        float z_scale = 1.0f;
        if (out.use_distance_scaling) {
            const float4 M3 = ldg4(M + 8);
            z_scale = (dot(f3(M3), position) + M3.w) * 0.5f;
        }
        float* info = out.densification_info;
        info[idx] += 1.0f;
        info[size_t(n_primitives) + idx] += length(dL_dposition * z_scale);
        if (out.densification_rows == 3) info[2 * size_t(n_primitives) + idx] += z_scale * accum[size_t(idx) * 5 + 4].x;
    }
    }   // kept
    if constexpr (COMPACT) {
        // one slot per kept Gaussian: a warp takes its slots with one atomic (the order of the rows carries no meaning)
        const uint32_t kept_mask = __ballot_sync(0xffffffffu, kept);
        if (kept_mask == 0) return;
        const uint32_t lane = threadIdx.x & 31u;
        uint32_t base = 0;
        if (lane == uint32_t(__ffs(kept_mask) - 1)) base = atomicAdd(reinterpret_cast<uint32_t*>(out.compact_rows), uint32_t(__popc(kept_mask)));
        base = __shfl_sync(0xffffffffu, base, __ffs(kept_mask) - 1);
        const uint32_t slot = base + uint32_t(__popc(kept_mask & ((1u << lane) - 1u)));
        if (kept && slot < out.compact_capacity) {      // rows beyond the capacity are dropped; the count tells the reader
            float4* row = out.compact_rows + 4 * (size_t(slot) + 1);
            row[0] = make_float4(__uint_as_float(idx), dL_dposition.x, dL_dposition.y, dL_dposition.z);
            row[1] = make_float4(grad_scale.x, grad_scale.y, grad_scale.z, grad_opacity);
            row[2] = grad_rotation;
            row[3] = make_float4(grad_rgb.x, grad_rgb.y, grad_rgb.z, 0.0f);
        }
    }
}

template <int MODE, int K>
cudaError_t launch_tile_backward(bool abs_grad, const FrameGeometry& geo, const PrimBuffers& prim, const uint32_t* prims_sorted, const uint2* tile_ranges,
                                 const TrainPixelBuffers& tin, const float* grad_image, const float* VPM, float4* accum, uint32_t g_first, uint32_t g_end,
                                 cudaStream_t stream) {
    using SM = BwdSmem<MODE, K>;
    const dim3 grid(geo.grid_w, geo.grid_h, 1);
    auto launch = [&](auto kernel) -> cudaError_t {
        // both instantiations have the same function-pointer type, so this lambda (and a static in it) is shared by them
        static PerDeviceOnce configured[2];
        if (SM::total > 48 * 1024) {
            const cudaError_t err = configured[abs_grad ? 1 : 0].run([&] { return cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(SM::total)); });
            if (err != cudaSuccess) return err;
        }
        kernel<<<grid, kBwdThreads, SM::total, stream>>>(tile_ranges, prims_sorted, prim.eval, prim.cull, tin, grad_image, VPM, accum,
                                                uint32_t(geo.width), uint32_t(geo.height), uint32_t(geo.grid_w), g_first, g_end);
        return cudaGetLastError();
    };
    return abs_grad ? launch(backward_tile_kernel<MODE, K, true>) : launch(backward_tile_kernel<MODE, K, false>);
}

template <int MODE>
cudaError_t launch_tile_backward_k(int K, bool abs_grad, const FrameGeometry& geo, const PrimBuffers& prim, const uint32_t* prims_sorted,
                                   const uint2* tile_ranges, const TrainPixelBuffers& tin, const float* grad_image, const float* VPM, float4* accum,
                                   uint32_t g_first, uint32_t g_end, cudaStream_t stream) {
    switch (K) {
        case 32: return launch_tile_backward<MODE, 32>(abs_grad, geo, prim, prims_sorted, tile_ranges, tin, grad_image, VPM, accum, g_first, g_end, stream);
        case 16: return launch_tile_backward<MODE, 16>(abs_grad, geo, prim, prims_sorted, tile_ranges, tin, grad_image, VPM, accum, g_first, g_end, stream);
        case 8: return launch_tile_backward<MODE, 8>(abs_grad, geo, prim, prims_sorted, tile_ranges, tin, grad_image, VPM, accum, g_first, g_end, stream);
        case 4: return launch_tile_backward<MODE, 4>(abs_grad, geo, prim, prims_sorted, tile_ranges, tin, grad_image, VPM, accum, g_first, g_end, stream);
        case 2: return launch_tile_backward<MODE, 2>(abs_grad, geo, prim, prims_sorted, tile_ranges, tin, grad_image, VPM, accum, g_first, g_end, stream);
        default: return launch_tile_backward<MODE, 1>(abs_grad, geo, prim, prims_sorted, tile_ranges, tin, grad_image, VPM, accum, g_first, g_end, stream);
    }
}

}  // namespace

namespace {
__global__ void __launch_bounds__(256) visibility_kernel(const uint32_t* __restrict__ n_touched, uint8_t* __restrict__ visible, uint32_t n) {
    const uint32_t i = blockIdx.x * 256 + threadIdx.x;
    if (i < n) visible[i] = n_touched[i] != 0;
}
}  // namespace

cudaError_t launch_visibility(const uint32_t* n_touched, uint8_t* visible, uint32_t n, cudaStream_t stream) {
    if (n == 0) return cudaSuccess;
    visibility_kernel<<<(n + 255) / 256, 256, 0, stream>>>(n_touched, visible, n);
    return cudaGetLastError();
}

cudaError_t clear_backward_outputs(const HtgsScene& scene, const BackwardOutputs& out, uint32_t first, uint32_t count, cudaStream_t stream) {
    const size_t n = size_t(count), at = size_t(first), B = size_t(scene.total_sh_bases);
    if (n == 0) return cudaSuccess;
    cudaError_t err;
    if ((err = cudaMemsetAsync(out.grad_positions + at * 3, 0, n * 3 * 4, stream)) != cudaSuccess) return err;
    if ((err = cudaMemsetAsync(out.grad_scales + at * 3, 0, n * 3 * 4, stream)) != cudaSuccess) return err;
    if ((err = cudaMemsetAsync(out.grad_rotations + at * 4, 0, n * 4 * 4, stream)) != cudaSuccess) return err;
    if ((err = cudaMemsetAsync(out.grad_opacities + at, 0, n * 4, stream)) != cudaSuccess) return err;
    if ((err = cudaMemsetAsync(out.grad_sh_0 + at * 3, 0, n * 3 * 4, stream)) != cudaSuccess) return err;
    if (B && (err = cudaMemsetAsync(out.grad_sh_rest + at * B * 3, 0, n * B * 3 * 4, stream)) != cudaSuccess) return err;
    return cudaSuccess;
}

namespace {
cudaError_t launch_chain_rule(const HtgsScene& scene, const HtgsView& view, const PrimBuffers& prim, const GradAccumBuffers& acc, const BackwardOutputs& out,
                              uint32_t n, uint32_t first, uint32_t count, cudaStream_t stream) {
    if (out.compact_rows != nullptr) {
        const cudaError_t err = cudaMemsetAsync(out.compact_rows, 0, sizeof(CompactGradientHeader), stream);
        if (err != cudaSuccess) return err;
        preprocess_backward_kernel<true><<<(count + 255) / 256, 256, 0, stream>>>(scene.positions, scene.scales, scene.rotations, scene.sh_rest, view.M, view.VPM,
                                                                                  view.cam_position, prim.n_touched, prim.clamp, acc.accum, out, n,
                                                                                  view.active_sh_bases, scene.total_sh_bases, first, first + count);
    } else {
        preprocess_backward_kernel<false><<<(count + 255) / 256, 256, 0, stream>>>(scene.positions, scene.scales, scene.rotations, scene.sh_rest, view.M, view.VPM,
                                                                                   view.cam_position, prim.n_touched, prim.clamp, acc.accum, out, n,
                                                                                   view.active_sh_bases, scene.total_sh_bases, first, first + count);
    }
    return cudaGetLastError();
}
}  // namespace

cudaError_t launch_backward(int mode, int K, const HtgsScene& scene, const HtgsView& view, const FrameGeometry& geo, const PrimBuffers& prim,
                            const uint32_t* prims_sorted, const uint2* tile_ranges, const TrainPixelBuffers& tin, const float* grad_image,
                            const float* image, const GradAccumBuffers& acc, const BackwardOutputs& out, cudaEvent_t outputs_cleared, int sm_count,
                            uint32_t first, uint32_t count, int stages, cudaStream_t stream) {
    (void)sm_count;
    const uint32_t n = uint32_t(scene.n_primitives);
    if (n == 0 || count == 0) return out.compact_rows ? cudaMemsetAsync(out.compact_rows, 0, sizeof(CompactGradientHeader), stream) : cudaSuccess;
    const bool whole = first == 0 && count == n;
    if (!(stages & kBackwardAccumulate)) {      // the per-Gaussian chain rule alone, over records an earlier call accumulated
        cudaError_t e = cudaSuccess;
        if (outputs_cleared != nullptr && (e = cudaStreamWaitEvent(stream, outputs_cleared, 0)) != cudaSuccess) return e;
        return launch_chain_rule(scene, view, prim, acc, out, n, first, count, stream);
    }
    // the pixel-parallel GLOBAL_ORDERING pass needs every fragment in front of a fragment: it cannot run over a part of the Gaussians
    if (!whole && mode == HTGS_MODE_ALPHA_BLEND_GLOBAL_ORDERING) return cudaErrorNotSupported;
    const uint32_t g_first = whole ? 0u : first, g_end = whole ? 0xffffffffu : first + count;
    cudaError_t err = cudaMemsetAsync(acc.accum + size_t(first) * 5, 0, size_t(count) * 5 * sizeof(float4), stream);
    if (err != cudaSuccess) return err;
    if (outputs_cleared == nullptr && (out.compact_rows == nullptr || out.grad_positions != nullptr) &&
        (err = clear_backward_outputs(scene, out, first, count, stream)) != cudaSuccess) return err;
    const bool abs_grad = out.densification_info != nullptr && out.densification_rows == 3;
    const int k = effective_k(mode, K);
    switch (mode) {
        case HTGS_MODE_HYBRID_BLEND:
            err = launch_tile_backward_k<HTGS_MODE_HYBRID_BLEND>(k, abs_grad, geo, prim, prims_sorted, tile_ranges, tin, grad_image, view.VPM, acc.accum, g_first, g_end, stream); break;
        case HTGS_MODE_ALPHA_BLEND_FIRST_K:
            err = launch_tile_backward_k<HTGS_MODE_ALPHA_BLEND_FIRST_K>(k, abs_grad, geo, prim, prims_sorted, tile_ranges, tin, grad_image, view.VPM, acc.accum, g_first, g_end, stream); break;
        case HTGS_MODE_OIT_BLEND:
            err = launch_tile_backward<HTGS_MODE_OIT_BLEND, 1>(abs_grad, geo, prim, prims_sorted, tile_ranges, tin, grad_image, view.VPM, acc.accum, g_first, g_end, stream); break;
        case HTGS_MODE_ALPHA_BLEND_GLOBAL_ORDERING: {
            const dim3 grid((geo.width + 7) / 8, (geo.height + 7) / 8, 1);
            backward_global_kernel<<<grid, 64, 0, stream>>>(tile_ranges, prims_sorted, prim.eval, prim.cull, grad_image, image, view.VPM, acc.accum,
                                                             uint32_t(geo.width), uint32_t(geo.height), uint32_t(geo.grid_w), abs_grad);
            err = cudaGetLastError();
            break;
        }
        default: return cudaErrorInvalidValue;
    }
    if (err != cudaSuccess) return err;
    if (outputs_cleared != nullptr && (err = cudaStreamWaitEvent(stream, outputs_cleared, 0)) != cudaSuccess) return err;
    if (!(stages & kBackwardChainRule)) return cudaSuccess;
    return launch_chain_rule(scene, view, prim, acc, out, n, first, count, stream);
}

}  // namespace htgs
