// update_max_weights: per-Gaussian maximum blending weight over the pixels of one view (importance for pruning).
// Replaces update_max_weights_cu of the four modes
//   rasterization/include/hybrid_blend/kernels/update_max_weights.cuh:59-212
//   rasterization/include/alpha_blend_first_k/kernels/update_max_weights.cuh:60-
//   rasterization/include/alpha_blend_global_ordering/kernels/update_max_weights.cuh:59-
//   rasterization/include/oit_blend/kernels/update_max_weights.cuh:57-
// The result is a maximum (atomicMax on the bit pattern of non-negative floats), so it does not depend on the
// order of evaluation and is bit-identical to the reference's.  The kernel has the shape of the blend kernel: a batch
// of instances is staged in shared memory, lane = Gaussian evaluates the conservative outline at the warp's 32 pixels
// and warp ballots transpose the result, then every lane walks the bit mask of its own candidates.  HYBRID and OIT
// need a second walk over the tile's list (every fragment is credited `alpha * tail weight` of its pixel), which has
// no alpha test of its own: its candidates are those of the outline only when `weight_threshold >= min_alpha`
// (then alpha * weight >= threshold implies alpha >= min_alpha), otherwise every staged instance.
#include "kernels.h"

namespace htgs {

namespace {

template <int MODE> struct WShape {
    static constexpr int tw = ModeTraits<MODE>::tile_w, th = ModeTraits<MODE>::tile_h, threads = tw * th;
    static constexpr int rows_per_warp = 32 / tw;
    static constexpr int chunk = 64;                   // candidate masks cover 64 staged instances
    static constexpr int chunks = threads / chunk;
};

__device__ __forceinline__ void raise_weight(unsigned int* max_weights, uint32_t primitive_idx, float weight) {
    const unsigned int bits = __float_as_uint(weight);
    if (max_weights[primitive_idx] < bits) atomicMax(&max_weights[primitive_idx], bits);
}

template <int MODE, int K>
__global__ void __launch_bounds__(WShape<MODE>::threads) max_weights_kernel(
    const uint2* __restrict__ tile_ranges, const uint32_t* __restrict__ prims_sorted, const EvalRecord* __restrict__ eval,
    const CullRecord* __restrict__ cull, unsigned int* __restrict__ max_weights, uint32_t width, uint32_t height, uint32_t grid_w, float weight_threshold, bool credit_tail)
{
    using MT = ModeTraits<MODE>;
    using WS = WShape<MODE>;
    constexpr bool kHybrid = MODE == HTGS_MODE_HYBRID_BLEND, kFirstK = MODE == HTGS_MODE_ALPHA_BLEND_FIRST_K;
    constexpr bool kGlobal = MODE == HTGS_MODE_ALPHA_BLEND_GLOBAL_ORDERING, kOit = MODE == HTGS_MODE_OIT_BLEND;
    constexpr bool kBuffer = kHybrid || kFirstK;
    __shared__ float4 s_T1[WS::threads], s_T2[WS::threads], s_T4[WS::threads], s_M3[WS::threads], s_c0[WS::threads];
    __shared__ float s_cc[WS::threads], s_op[WS::threads];
    __shared__ uint32_t s_g[WS::threads];
    const uint32_t tid = threadIdx.x;
    const uint32_t warp = tid >> 5, lane = tid & 31;
    const uint32_t px_i = blockIdx.x * WS::tw + (tid % WS::tw), py_i = blockIdx.y * WS::th + (tid / WS::tw);
    const bool inside = px_i < width && py_i < height;
    const float pixel_x = __uint2float_rn(px_i), pixel_y = __uint2float_rn(py_i);
    const float rect_x0 = float(blockIdx.x * WS::tw);
    const float rect_y0 = float(blockIdx.y * WS::th + warp * WS::rows_per_warp);
    const uint2 range = tile_ranges[blockIdx.y * grid_w + blockIdx.x];

    [[maybe_unused]] float kd[kBuffer ? K : 1], ka[kBuffer ? K : 1];
    [[maybe_unused]] uint32_t ki[kBuffer ? K : 1];
    if constexpr (kBuffer) {
        #pragma unroll
        for (int k = 0; k < K; ++k) { kd[k] = FLT_MAX; ka[k] = 0.0f; ki[k] = 0xffffffffu; }
    }
    float alpha_sum = 0.0f, transmittance = 1.0f;   // HB: tail; OIT / GO: pixel
    bool done = !inside;
    float second_pass_weight = 0.0f;
    const bool outline_in_second_pass = weight_threshold >= MT::min_alpha;

    const int n_passes = (kOit || (kHybrid && credit_tail)) ? 2 : 1;
    for (int pass = 0; pass < n_passes; ++pass) {
        const bool lane_active = !done && (pass == 0 || second_pass_weight >= weight_threshold);
        if (pass == 1 && __syncthreads_count(lane_active) == 0) break;   // no pixel of the tile has a tail to credit
        for (uint32_t batch_begin = range.x; batch_begin < range.y; batch_begin += WS::threads) {
            if constexpr (kGlobal) { if (__syncthreads_count(done) == WS::threads) break; } else __syncthreads();
            const uint32_t batch = min(uint32_t(WS::threads), range.y - batch_begin);
            if (tid < batch) {
                const uint32_t g = __ldg(prims_sorted + batch_begin + tid);
                const float* rec = reinterpret_cast<const float*>(eval + g);
                s_g[tid] = g;
                s_T1[tid] = ldg4(rec); s_T2[tid] = ldg4(rec + 4); s_T4[tid] = ldg4(rec + 8); s_M3[tid] = ldg4(rec + 12);
                s_op[tid] = __ldg(rec + 19);
                s_c0[tid] = ldg4(reinterpret_cast<const float*>(cull + g));
                s_cc[tid] = __ldg(reinterpret_cast<const float*>(cull + g) + 4);
            } else {
                s_c0[tid] = make_float4(__int_as_float(0x7f800000), 0.0f, 0.0f, 0.0f);   // outline that rejects every pixel
                s_cc[tid] = 0.0f;
            }
            __syncthreads();
            #pragma unroll 1
            for (int chunk = 0; chunk < WS::chunks; ++chunk) {
                const uint32_t chunk_base = chunk * WS::chunk;
                if (chunk_base >= batch) break;
                // ---- candidate masks ---------------------------------------------------------------------
                uint64_t cand = 0;
                if (pass == 0 || outline_in_second_pass) {
                    #pragma unroll
                    for (int half = 0; half < 2; ++half) {
                        const uint32_t j = chunk_base + half * 32 + lane;
                        const float4 c0 = s_c0[j];
                        const float cc = s_cc[j];
                        const float dx0 = rect_x0 - c0.x, dy0 = rect_y0 - c0.y;
                        uint32_t mine = 0;
                        #pragma unroll
                        for (int r = 0; r < WS::rows_per_warp; ++r) {
                            const float dy = dy0 + float(r);
                            const float b2dy = c0.w * dy, cdy2 = cc * dy * dy;
                            #pragma unroll
                            for (int i = 0; i < WS::tw; ++i) {
                                const float dx = dx0 + float(i);
                                const float q = dx * (c0.z * dx + b2dy) + cdy2;
                                const uint32_t touched = __ballot_sync(0xffffffffu, q <= 1.0f);
                                if (int(lane) == r * WS::tw + i) mine = touched;
                            }
                        }
                        cand |= uint64_t(mine) << (32 * half);
                    }
                } else {
                    const uint32_t in_chunk = min(uint32_t(WS::chunk), batch - chunk_base);
                    cand = in_chunk >= 64 ? ~0ull : ((1ull << in_chunk) - 1ull);
                }
                if (done || (pass == 1 && !(second_pass_weight >= weight_threshold))) cand = 0;
                // ---- every lane walks its own candidates, in list order, two per trip: the two evaluations (divide, expf,
                // depth) are independent instruction streams, the state updates follow in order ----------------------
                const uint32_t n_iter = __reduce_max_sync(0xffffffffu, uint32_t(__popcll(cand)));
                auto pop_candidate = [&](bool& valid) -> uint32_t {
                    valid = cand != 0;
                    const uint32_t j = chunk_base + (valid ? uint32_t(__ffsll((long long)cand) - 1) : 0u);
                    cand &= cand - 1;
                    return j;
                };
                auto evaluate = [&](bool valid, uint32_t j, float& alpha, float& depth) -> bool {
                    const float4 plane_x_diag = s_T1[j] - s_T4[j] * pixel_x;
                    const float4 plane_y_diag = s_T2[j] - s_T4[j] * pixel_y;
                    const float3 nx = f3(plane_x_diag), ny = f3(plane_y_diag);
                    const float3 m = plane_x_diag.w * ny - nx * plane_y_diag.w;
                    const float3 d = cross(nx, ny);
                    const float numerator_rho2 = dot(m, m);
                    const float denominator = dot(d, d);
                    const bool inside_cutoff = !(numerator_rho2 > MT::max_cutoff_sq * denominator);
                    const float denominator_rcp = 1.0f / denominator;
                    const float G = expf(-0.5f * numerator_rho2 * denominator_rcp);
                    alpha = fminf(s_op[j] * G, kMaxFragmentAlpha);
                    if constexpr (kBuffer) {
                        const float3 e = cross(d, m) * denominator_rcp;
                        const float4 MT3 = s_M3[j];
                        depth = dot(f3(MT3), e) + MT3.w;
                    } else {
                        depth = 0.0f;
                    }
                    return valid && inside_cutoff;
                };
                auto commit = [&](uint32_t j, float alpha, float depth) {
                    if (done) return;
                    if (pass == 1) {   // no alpha test in the second walk
                        const float blending_weight = alpha * second_pass_weight;
                        if (!(blending_weight < weight_threshold)) raise_weight(max_weights, s_g[j], blending_weight);
                        return;
                    }
                    if constexpr (kFirstK) {
                        if (depth >= kd[K - 1] || alpha < MT::min_alpha) return;
                        uint32_t primitive_idx = s_g[j];
                        #pragma unroll
                        for (int k = 0; k < K; ++k)
                            if (depth < kd[k]) {
                                const float td = kd[k]; kd[k] = depth; depth = td;
                                const float ta = ka[k]; ka[k] = alpha; alpha = ta;
                                const uint32_t ti = ki[k]; ki[k] = primitive_idx; primitive_idx = ti;
                            }
                    } else {
                        if (alpha < MT::min_alpha) return;
                        if constexpr (kHybrid) {
                            if (depth < kd[K - 1] && alpha >= MT::min_alpha_core) {
                                uint32_t primitive_idx = s_g[j];
                                #pragma unroll
                                for (int k = 0; k < K; ++k)
                                    if (depth < kd[k]) {
                                        const float td = kd[k]; kd[k] = depth; depth = td;
                                        const float ta = ka[k]; ka[k] = alpha; alpha = ta;
                                        const uint32_t ti = ki[k]; ki[k] = primitive_idx; primitive_idx = ti;
                                    }
                            }
                            alpha_sum += alpha;
                            transmittance *= 1.0f - alpha;
                        } else if constexpr (kGlobal) {
                            const float blending_weight = transmittance * alpha;
                            transmittance *= 1.0f - alpha;
                            if (transmittance < kTransmittanceThreshold) done = true;
                            if (!(blending_weight < weight_threshold)) raise_weight(max_weights, s_g[j], blending_weight);
                        } else {
                            alpha_sum += alpha;
                            transmittance *= 1.0f - alpha;
                        }
                    }
                };
                for (uint32_t it = 0; it < n_iter; it += 2) {
                    bool v0, v1;
                    const uint32_t j0 = pop_candidate(v0);
                    const uint32_t j1 = pop_candidate(v1);
                    float alpha0, alpha1, depth0, depth1;
                    const bool ok0 = evaluate(v0, j0, alpha0, depth0);
                    const bool ok1 = evaluate(v1, j1, alpha1, depth1);
                    if (ok0) commit(j0, alpha0, depth0);
                    if (ok1) commit(j1, alpha1, depth1);
                }
            }
        }
        if (pass == 0 && inside) {
            if constexpr (kBuffer) {
                float t = 1.0f;
                #pragma unroll
                for (int k = 0; k < K; ++k) {
                    const float alpha = ka[k];
                    const float blending_weight = t * alpha;
                    t *= 1.0f - alpha;
                    if (t < kTransmittanceThreshold) t = 0.0f;
                    if (blending_weight < weight_threshold || ki[k] == 0xffffffffu) continue;
                    raise_weight(max_weights, ki[k], blending_weight);
                }
                if constexpr (kHybrid) { if (alpha_sum >= weight_threshold) second_pass_weight = t * (1.0f - transmittance) * (1.0f / alpha_sum); }
            }
            if constexpr (kOit) { if (alpha_sum >= weight_threshold) second_pass_weight = (1.0f - transmittance) * (1.0f / alpha_sum); }
        }
    }
}

template <int MODE, int K>
cudaError_t launch_w(const FrameGeometry& geo, const PrimBuffers& prim, const uint32_t* prims_sorted, const uint2* tile_ranges, float* max_weights,
                     float weight_threshold, bool credit_tail, cudaStream_t stream) {
    const dim3 grid(geo.grid_w, geo.grid_h, 1);
    max_weights_kernel<MODE, K><<<grid, WShape<MODE>::threads, 0, stream>>>(tile_ranges, prims_sorted, prim.eval, prim.cull, reinterpret_cast<unsigned int*>(max_weights),
                                                                            uint32_t(geo.width), uint32_t(geo.height), uint32_t(geo.grid_w), weight_threshold, credit_tail);
    return cudaGetLastError();
}

template <int MODE>
cudaError_t launch_w_k(int K, const FrameGeometry& geo, const PrimBuffers& prim, const uint32_t* prims_sorted, const uint2* tile_ranges, float* max_weights,
                       float weight_threshold, bool credit_tail, cudaStream_t stream) {
    switch (K) {
        case 32: return launch_w<MODE, 32>(geo, prim, prims_sorted, tile_ranges, max_weights, weight_threshold, credit_tail, stream);
        case 16: return launch_w<MODE, 16>(geo, prim, prims_sorted, tile_ranges, max_weights, weight_threshold, credit_tail, stream);
        case 8: return launch_w<MODE, 8>(geo, prim, prims_sorted, tile_ranges, max_weights, weight_threshold, credit_tail, stream);
        case 4: return launch_w<MODE, 4>(geo, prim, prims_sorted, tile_ranges, max_weights, weight_threshold, credit_tail, stream);
        case 2: return launch_w<MODE, 2>(geo, prim, prims_sorted, tile_ranges, max_weights, weight_threshold, credit_tail, stream);
        default: return launch_w<MODE, 1>(geo, prim, prims_sorted, tile_ranges, max_weights, weight_threshold, credit_tail, stream);
    }
}

}  // namespace

cudaError_t launch_max_weights(int mode, int K, const FrameGeometry& geo, const PrimBuffers& prim, const uint32_t* prims_sorted, const uint2* tile_ranges,
                               float* max_weights, float weight_threshold, bool credit_tail, cudaStream_t stream) {
    const int k = effective_k(mode, K);
    switch (mode) {
        case HTGS_MODE_HYBRID_BLEND:
            // Without the tail credit HYBRID needs its K-buffer weights only, which is what the reference extension computes: its
            // link resolves HYBRID's kernel dispatcher to FIRST_K's copy (hybrid_blend/update_max_weights.cu:15-28 against
            // alpha_blend_first_k/update_max_weights.cu:15-28), so FIRST_K's kernel walks HYBRID's tile lists.  The same is done
            // here: fragments below alpha 1/20 are dropped at once instead of being summed into a tail nobody reads.
            if (!credit_tail) return launch_w_k<HTGS_MODE_ALPHA_BLEND_FIRST_K>(k, geo, prim, prims_sorted, tile_ranges, max_weights, weight_threshold, false, stream);
            return launch_w_k<HTGS_MODE_HYBRID_BLEND>(k, geo, prim, prims_sorted, tile_ranges, max_weights, weight_threshold, true, stream);
        case HTGS_MODE_ALPHA_BLEND_FIRST_K: return launch_w_k<HTGS_MODE_ALPHA_BLEND_FIRST_K>(k, geo, prim, prims_sorted, tile_ranges, max_weights, weight_threshold, credit_tail, stream);
        case HTGS_MODE_ALPHA_BLEND_GLOBAL_ORDERING: return launch_w<HTGS_MODE_ALPHA_BLEND_GLOBAL_ORDERING, 1>(geo, prim, prims_sorted, tile_ranges, max_weights, weight_threshold, credit_tail, stream);
        case HTGS_MODE_OIT_BLEND: return launch_w<HTGS_MODE_OIT_BLEND, 1>(geo, prim, prims_sorted, tile_ranges, max_weights, weight_threshold, credit_tail, stream);
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace htgs
