// Per-tile blend kernels (inference) for the four blend modes.
//
// Replaces blend_cu of the reference
//   HYBRID_BLEND               rasterization/include/hybrid_blend/kernels/inference.cuh:78-216
//   ALPHA_BLEND_FIRST_K        rasterization/include/alpha_blend_first_k/kernels/inference.cuh:79-208
//   ALPHA_BLEND_GLOBAL_ORDERING rasterization/include/alpha_blend_global_ordering/kernels/inference.cuh:78-176
//   OIT_BLEND                  rasterization/include/oit_blend/kernels/inference.cuh:78-177
// The per-fragment arithmetic (planes through the pixel ray, rho^2, G, alpha, depth of the point
// of maximum contribution) and every threshold decision are kept operation for operation, and each
// pixel still sees its tile's instances in list order, so results match the reference bit for bit.
// How the work is organised is different:
//
//  1. Staging.  One thread per instance of a batch starts ONE 80-byte bulk asynchronous copy (TMA,
//     cp.async.bulk) of the Gaussian's evaluation record into shared memory, completion tracked by an
//     mbarrier, and publishes the Gaussian's conservative screen-space outline (5 floats).  Index and
//     outline of the NEXT batch are prefetched into registers while the current batch is processed.
//  2. Candidate masks (overlap the copies in flight).  Inside a warp, lane l takes Gaussian l of the
//     batch and evaluates the 3-flop outline test at each of the warp's 32 pixels; one warp ballot per
//     pixel transposes the result, so that afterwards lane p holds the bit mask of the Gaussians that
//     can touch pixel p.  No divergence, no shared-memory queue.
//  3. Exact pass.  After the mbarrier completes, every lane walks the set bits of its own mask, so
//     (almost) every iteration of every lane is an accepted fragment: the expensive part (IEEE divide,
//     expf, depth, K-buffer insertion) runs converged instead of once per Gaussian per warp.  Every mode
//     evaluates two candidates per trip for instruction-level parallelism and commits them in list order.
//  4. K-buffer.  Registers hold only (depth, slot) pairs; the payloads live in a shared-memory pool of
//     K+1 slots per pixel, so an insertion moves 2 registers per level instead of 5-6.  The buffer
//     references K slots, one is free: a new fragment is written to the free slot, the insertion
//     chain carries (depth, slot) pairs exactly like the reference's swap chain carries whole
//     fragments, and the slot that falls out of the chain becomes the free one.
#include "kernels.h"

namespace htgs {

namespace {

// Pixels one CTA blends.  The binning tile of GLOBAL_ORDERING is 16x16 (its lists have to be the reference's), but its
// blend walks a list with per-pixel early termination and no state shared between pixels, so each binning tile is blended
// by split_x * split_y independent CTAs that read the same list: more and shorter-lived CTAs, a tighter outline test per
// CTA, and a CTA stops as soon as ITS pixels are opaque.
#ifndef HTGS_GO_BLEND_W
#define HTGS_GO_BLEND_W 8
#define HTGS_GO_BLEND_H 8
#endif
template <int MODE> struct TileShape {
    static constexpr bool split = MODE == HTGS_MODE_ALPHA_BLEND_GLOBAL_ORDERING;
    static constexpr int tw = split ? HTGS_GO_BLEND_W : ModeTraits<MODE>::tile_w, th = split ? HTGS_GO_BLEND_H : ModeTraits<MODE>::tile_h;
    static constexpr int split_x = ModeTraits<MODE>::tile_w / tw, split_y = ModeTraits<MODE>::tile_h / th;
    static constexpr int threads = tw * th;
    static constexpr int warps = threads / 32;
    static constexpr int rows_per_warp = 32 / tw;
    static constexpr int batch = threads;            // instances staged per iteration (one per thread)
    static constexpr int chunk = 64;                 // candidate masks are built and consumed 64 instances at a time
    static constexpr int chunks = batch / chunk;
};

template <int MODE, int K, bool TRAIN> struct SmemLayout {
    using TS = TileShape<MODE>;
    static constexpr bool has_kbuffer = (MODE == HTGS_MODE_HYBRID_BLEND || MODE == HTGS_MODE_ALPHA_BLEND_FIRST_K);
    static constexpr bool has_prim = (MODE == HTGS_MODE_ALPHA_BLEND_FIRST_K) || (MODE == HTGS_MODE_HYBRID_BLEND && TRAIN);
    static constexpr bool has_pool_idx = (MODE == HTGS_MODE_HYBRID_BLEND && TRAIN);
    static constexpr int pool_elem = (MODE == HTGS_MODE_HYBRID_BLEND) ? 16 : (MODE == HTGS_MODE_ALPHA_BLEND_FIRST_K ? 8 : 0);
    static constexpr size_t eval_off = 0;
    static constexpr size_t eval_bytes = size_t(TS::batch) * sizeof(EvalRecord);
    static constexpr size_t cull4_off = eval_off + eval_bytes;
    static constexpr size_t cull4_bytes = size_t(TS::batch) * 16;
    static constexpr size_t cullc_off = cull4_off + cull4_bytes;
    static constexpr size_t cullc_bytes = size_t(TS::batch) * 4;
    static constexpr size_t prim_off = cullc_off + cullc_bytes;
    static constexpr size_t prim_bytes = has_prim ? size_t(TS::batch) * 4 : 0;
    static constexpr size_t bar_off = (prim_off + prim_bytes + 15) & ~size_t(15);
    static constexpr size_t pool_off = bar_off + 16;
    static constexpr size_t pool_bytes = has_kbuffer ? size_t(K + 1) * TS::threads * pool_elem : 0;
    static constexpr size_t pool_idx_off = pool_off + pool_bytes;
    static constexpr size_t pool_idx_bytes = has_pool_idx ? size_t(K + 1) * TS::threads * 4 : 0;
    static constexpr size_t total = pool_idx_off + pool_idx_bytes;
};

// The shared per-fragment front end (hybrid_blend/kernels/inference.cuh:137-148).
struct FragmentFront {
    float3 m, d;
    float numerator_rho2, denominator;
};
__device__ __forceinline__ FragmentFront fragment_front(const float4& VPMT1, const float4& VPMT2, const float4& VPMT4, float pixel_x, float pixel_y) {
    FragmentFront f;
    const float4 plane_x_diag = VPMT1 - VPMT4 * pixel_x;
    const float4 plane_y_diag = VPMT2 - VPMT4 * pixel_y;
    const float3 plane_x_diag_normal = f3(plane_x_diag);
    const float3 plane_y_diag_normal = f3(plane_y_diag);
    f.m = plane_x_diag.w * plane_y_diag_normal - plane_x_diag_normal * plane_y_diag.w;
    f.d = cross(plane_x_diag_normal, plane_y_diag_normal);
    f.numerator_rho2 = dot(f.m, f.m);
    f.denominator = dot(f.d, f.d);
    return f;
}

// The reference's insertion chain (hybrid_blend/kernels/inference.cuh:159-167) on (depth, slot) pairs:
//     for k: if (carried.depth < kd[k]) swap(carried, entry[k]);
// Because kd is sorted, the DEPTH carried into level k is always max(depth, kd[k-1]) - with or without ties -
// so every level's comparison and new depth are computed from the old buffer in parallel; only the carried
// slot is still passed from level to level (one select per level on the critical path instead of a compare
// and a select).  Results, including the reference's behaviour for equal depths, are bit-identical to the chain.
// On return `depth` is the depth of the entry that fell out of the buffer and the result its slot.
// Slot numbers travel as floats (0..K are exact): the two selects per level that pass the slots along the chain become
// one add and two multiply-adds on the FMA pipes, which are mostly idle in this kernel, instead of two instructions on
// the ALU pipe that bounds it.  The comparison is materialised as 1.0f / 0.0f by a single `set` instruction.
using slot_t = float;
__device__ __forceinline__ uint32_t slot_index(slot_t s) { return uint32_t(__float2int_rz(s)); }
__device__ __forceinline__ float less_than_as_float(float a, float b) {
    float r;
    asm("set.lt.f32.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));
    return r;
}

template <int K>
__device__ __forceinline__ slot_t kbuffer_insert(float (&kd)[K], slot_t (&ks)[K], float& depth, slot_t slot) {
    float p[K];
    float nd[K];
    #pragma unroll
    for (int k = 0; k < K; ++k) {
        const float carried = k == 0 ? depth : fmaxf(depth, kd[k - 1]);
        p[k] = less_than_as_float(carried, kd[k]);
        nd[k] = fminf(carried, kd[k]);   // = carried where carried < kd[k], else kd[k]
    }
    const float out_depth = fmaxf(depth, kd[K - 1]);
    #pragma unroll
    for (int k = 0; k < K; ++k) {
        const slot_t mine = ks[k];
        const float t = slot - mine;
        ks[k] = fmaf(t, p[k], mine);      // p ? slot : mine
        slot = fmaf(-t, p[k], slot);      // p ? mine : slot
        kd[k] = nd[k];
    }
    depth = out_depth;
    return slot;
}

template <int MODE, int K, bool TRAIN, bool STATS>
__global__ void __launch_bounds__(TileShape<MODE>::threads) blend_kernel(
    const uint2* __restrict__ tile_ranges, const uint32_t* __restrict__ prims_sorted, const EvalRecord* __restrict__ eval,
    const CullRecord* __restrict__ cull, float* __restrict__ image, float* __restrict__ depth_out, float* __restrict__ alpha_out,
    TrainPixelBuffers tout, uint32_t width, uint32_t height, uint32_t grid_w, bool to_chw, bool use_median_depth, FrameStatus* status)
{
    using MT = ModeTraits<MODE>;
    using TS = TileShape<MODE>;
    using SL = SmemLayout<MODE, K, TRAIN>;
    constexpr bool kHybrid = MODE == HTGS_MODE_HYBRID_BLEND;
    constexpr bool kFirstK = MODE == HTGS_MODE_ALPHA_BLEND_FIRST_K;
    constexpr bool kGlobal = MODE == HTGS_MODE_ALPHA_BLEND_GLOBAL_ORDERING;
    extern __shared__ __align__(128) unsigned char smem[];
    EvalRecord* s_eval = reinterpret_cast<EvalRecord*>(smem + SL::eval_off);
    float4* s_cull4 = reinterpret_cast<float4*>(smem + SL::cull4_off);
    float* s_cullc = reinterpret_cast<float*>(smem + SL::cullc_off);
    [[maybe_unused]] uint32_t* s_prim = reinterpret_cast<uint32_t*>(smem + SL::prim_off);
    uint64_t* s_bar = reinterpret_cast<uint64_t*>(smem + SL::bar_off);

    const uint32_t tid = threadIdx.x;
    const uint32_t warp = tid >> 5, lane = tid & 31;
    const uint32_t tile_x = blockIdx.x, tile_y = blockIdx.y;
    const uint32_t px_i = tile_x * TS::tw + (tid % TS::tw);
    const uint32_t py_i = tile_y * TS::th + (tid / TS::tw);
    const bool inside = px_i < width && py_i < height;
    const float pixel_x = __uint2float_rn(px_i);
    const float pixel_y = __uint2float_rn(py_i);

    if (tid == 0) { mbar_init(s_bar, TS::threads); mbar_fence_init(); }

    // ---- per-pixel state -------------------------------------------------------------------
    [[maybe_unused]] float kd[SL::has_kbuffer ? K : 1];
    [[maybe_unused]] slot_t ks[SL::has_kbuffer ? K : 1];
    [[maybe_unused]] float4* pool4 = reinterpret_cast<float4*>(smem + SL::pool_off);
    [[maybe_unused]] float2* pool2 = reinterpret_cast<float2*>(smem + SL::pool_off);
    [[maybe_unused]] uint32_t* pool_idx = reinterpret_cast<uint32_t*>(smem + SL::pool_idx_off);
    [[maybe_unused]] uint32_t free_slot = K;   // index of the pool slot no buffer entry refers to
    if constexpr (SL::has_kbuffer) {
        #pragma unroll
        for (int k = 0; k < K; ++k) {
            kd[k] = FLT_MAX; ks[k] = slot_t(k);
            if constexpr (kHybrid) pool4[k * TS::threads + tid] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            else pool2[k * TS::threads + tid] = make_float2(0.0f, __uint_as_float(0xffffffffu));
            if constexpr (SL::has_pool_idx) pool_idx[k * TS::threads + tid] = 0xffffffffu;
        }
    }
    // HYBRID tail / OIT accumulators / GLOBAL_ORDERING running blend
    float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);   // HB: premultiplied tail rgba; OIT: alpha-weighted rgb,depth; GO: rgb, depth
    float acc_depth = 0.0f;                              // HB: depth * alpha of the tail; OIT: alpha sum
    float transmittance = 1.0f;                          // HB: tail; OIT / GO: pixel
    bool done = !inside;

    const uint2 range = tile_ranges[(tile_y / TS::split_y) * grid_w + tile_x / TS::split_x];   // grid_w counts binning tiles
    uint32_t phase = 0;
    bool wait_failed = false;
    [[maybe_unused]] uint32_t stat_candidates = 0, stat_accepted = 0, stat_trips = 0, stat_trips_inserting = 0, stat_insertions = 0;
    // pixel rectangle of this warp (tw x rows_per_warp pixels; lane = row * tw + column)
    const float rect_x0 = float(tile_x * TS::tw);
    const float rect_y0 = float(tile_y * TS::th + warp * TS::rows_per_warp);

    // prefetch registers: Gaussian index and outline of the instance this thread stages next
    uint32_t g_next = 0;
    float4 c0_next = make_float4(__int_as_float(0x7f800000), 0.0f, 0.0f, 0.0f);   // "reject everything"
    float cc_next = 0.0f;
    if (range.x + tid < range.y) {
        g_next = __ldg(prims_sorted + range.x + tid);
        c0_next = ldg4(reinterpret_cast<const float*>(cull + g_next));
        cc_next = __ldg(reinterpret_cast<const float*>(cull + g_next) + 4);
    }
    __syncthreads();

    for (uint32_t batch_begin = range.x; batch_begin < range.y; batch_begin += TS::batch) {
        if constexpr (kGlobal) {
            if (__syncthreads_count(done) == TS::threads) break;
        } else {
            __syncthreads();
        }
        // ---- 1. staging: one instance per thread, from the prefetch registers ------------------------
        const bool valid_inst = batch_begin + tid < range.y;
        s_cull4[tid] = c0_next;
        s_cullc[tid] = cc_next;
        if (valid_inst) {
            mbar_arrive_expect_tx(s_bar, uint32_t(sizeof(EvalRecord)));
            bulk_copy_g2s(s_eval + tid, eval + g_next, uint32_t(sizeof(EvalRecord)), s_bar);
            if constexpr (SL::has_prim) s_prim[tid] = g_next;
        } else {
            mbar_arrive(s_bar);
        }
        const uint32_t inst_next = batch_begin + TS::batch + tid;
        const bool valid_next = inst_next < range.y;
        if (valid_next) g_next = __ldg(prims_sorted + inst_next);
        __syncthreads();
        bool copies_landed = false;
        #pragma unroll 1
        for (int chunk = 0; chunk < TS::chunks; ++chunk) {
            // ---- 2. candidate masks: lane = Gaussian, one ballot per pixel of the warp --------------
            uint64_t cand = 0;
            {
                #pragma unroll
                for (int half = 0; half < 2; ++half) {
                    const uint32_t j = chunk * TS::chunk + half * 32 + lane;
                    const float4 c0 = s_cull4[j];
                    const float cc = s_cullc[j];
                    const float dx0 = rect_x0 - c0.x, dy0 = rect_y0 - c0.y;
                    uint32_t mine = 0;
                    #pragma unroll
                    for (int r = 0; r < TS::rows_per_warp; ++r) {
                        const float dy = dy0 + float(r);
                        const float b2dy = c0.w * dy, cdy2 = cc * dy * dy;
                        #pragma unroll
                        for (int i = 0; i < TS::tw; ++i) {
                            const float dx = dx0 + float(i);
                            const float q = dx * (c0.z * dx + b2dy) + cdy2;
                            const uint32_t touched = __ballot_sync(0xffffffffu, q <= 1.0f);
                            if (int(lane) == r * TS::tw + i) mine = touched;
                        }
                    }
                    cand |= uint64_t(mine) << (32 * half);
                }
                if (done) cand = 0;
            }
            if (chunk == 0) {   // the index prefetched before the barrier has arrived by now
                if (valid_next) {
                    c0_next = ldg4(reinterpret_cast<const float*>(cull + g_next));
                    cc_next = __ldg(reinterpret_cast<const float*>(cull + g_next) + 4);
                } else {
                    c0_next = make_float4(__int_as_float(0x7f800000), 0.0f, 0.0f, 0.0f);
                    cc_next = 0.0f;
                }
            }
            // ---- 3. exact pass ------------------------------------------------------------------------
            if (!copies_landed) {
                if (!mbar_wait_bounded(s_bar, phase)) wait_failed = true;
                phase ^= 1;
                copies_landed = true;
            }
            const uint32_t n_cand = __popcll(cand);
            if constexpr (STATS) stat_candidates += n_cand;
            const uint32_t n_iter = __reduce_max_sync(0xffffffffu, n_cand);
            const uint32_t chunk_base = chunk * TS::chunk;
            auto pop_candidate = [&](bool& valid) -> uint32_t {
                valid = cand != 0;
                const uint32_t j = valid ? uint32_t(__ffsll((long long)cand) - 1) : 0u;
                cand &= cand - 1;
                return chunk_base + j;
            };
            if constexpr (kHybrid) {
                // Two candidates per trip: their evaluations are independent instruction streams (the compiler
                // interleaves them), which hides the latency of the divide / expf / dot chains; the buffer
                // and tail updates then happen strictly in list order.
                // Inference keeps premultiplied colours in the buffer (inference.cuh:158), the training forward
                // keeps (rgb, alpha) and the Gaussian index (forward.cuh:159-171).
                auto evaluate = [&](bool valid, uint32_t j, float& depth, float4& frag) -> bool {
                    const float4* rec = reinterpret_cast<const float4*>(s_eval + j);
                    const FragmentFront fr = fragment_front(rec[0], rec[1], rec[2], pixel_x, pixel_y);
                    const float numerator_rho2 = fr.numerator_rho2;
                    const float denominator = fr.denominator;
                    const bool inside_cutoff = !(numerator_rho2 > MT::max_cutoff_sq * denominator);
                    const float denominator_rcp = 1.0f / denominator;
                    const float4 rgba_in = rec[4];
                    const float G = expf(-0.5f * numerator_rho2 * denominator_rcp);
                    const float alpha = fminf(rgba_in.w * G, kMaxFragmentAlpha);
                    const float3 eval_point_diag = cross(fr.d, fr.m) * denominator_rcp;
                    const float4 MT3 = rec[3];
                    depth = dot(f3(MT3), eval_point_diag) + MT3.w;
                    if constexpr (TRAIN) frag = make_float4(rgba_in.x, rgba_in.y, rgba_in.z, alpha);
                    else frag = make_float4(rgba_in.x * alpha, rgba_in.y * alpha, rgba_in.z * alpha, alpha);
                    return valid && inside_cutoff && !(alpha < MT::min_alpha);
                };
                auto commit = [&](float depth, float4 frag, uint32_t j) {
                    if constexpr (STATS) ++stat_accepted;
                    if (depth < kd[K - 1] && frag.w >= MT::min_alpha_core) {
                        pool4[free_slot * TS::threads + tid] = frag;
                        if constexpr (TRAIN) pool_idx[free_slot * TS::threads + tid] = batch_begin - range.x + j;   // position in the tile's list: what the backward pass looks up
                        free_slot = slot_index(kbuffer_insert<K>(kd, ks, depth, slot_t(free_slot)));   // the entry that fell out: a real fragment or an empty one
                        frag = pool4[free_slot * TS::threads + tid];
                    }
                    if constexpr (TRAIN) {
                        acc += make_float4(frag.x * frag.w, frag.y * frag.w, frag.z * frag.w, frag.w);
                    } else {
                        acc += frag;
                        if (!use_median_depth) acc_depth += depth * frag.w;
                    }
                    transmittance *= 1.0f - frag.w;
                };
                for (uint32_t it = 0; it < n_iter; it += 2) {
                    bool v0, v1;
                    const uint32_t j0 = pop_candidate(v0);
                    const uint32_t j1 = pop_candidate(v1);
                    float depth0, depth1;
                    float4 frag0, frag1;
                    const bool ok0 = evaluate(v0, j0, depth0, frag0);
                    const bool ok1 = evaluate(v1, j1, depth1, frag1);
                    if constexpr (STATS) {   // how often the insertion chain runs for the warp (the branch in commit is the warp vote)
                        const bool in0 = ok0 && depth0 < kd[K - 1] && frag0.w >= MT::min_alpha_core;
                        stat_trips += 1; stat_trips_inserting += __any_sync(0xffffffffu, in0) ? 1 : 0; stat_insertions += in0 ? 1 : 0;
                    }
                    if (ok0) commit(depth0, frag0, j0);
                    if constexpr (STATS) {
                        const bool in1 = ok1 && depth1 < kd[K - 1] && frag1.w >= MT::min_alpha_core;
                        stat_trips += 1; stat_trips_inserting += __any_sync(0xffffffffu, in1) ? 1 : 0; stat_insertions += in1 ? 1 : 0;
                    }
                    if (ok1) commit(depth1, frag1, j1);
                }
            } else {
                // The other three modes use the same two-candidates-per-trip shape: both evaluations (divide, expf, depth) are
                // independent instruction streams; the state updates happen in list order.  A fragment counts iff it passes
                // the cutoff, the alpha threshold and (FIRST_K) the depth test against the buffer - conditions that do not
                // depend on the order in which they are checked (alpha_blend_first_k/kernels/inference.cuh:147-160,
                // alpha_blend_global_ordering/kernels/inference.cuh:139-160, oit_blend/kernels/inference.cuh:139-160).
                constexpr bool kNeedsPointDepth = kFirstK || (!kGlobal && !TRAIN);
                auto evaluate = [&](bool valid, uint32_t j, float& alpha, float& depth, float4& rgba_in) -> bool {
                    const float4* rec = reinterpret_cast<const float4*>(s_eval + j);
                    const FragmentFront fr = fragment_front(rec[0], rec[1], rec[2], pixel_x, pixel_y);
                    const float numerator_rho2 = fr.numerator_rho2;
                    const float denominator = fr.denominator;
                    const bool inside_cutoff = !(numerator_rho2 > MT::max_cutoff_sq * denominator);
                    const float denominator_rcp = 1.0f / denominator;
                    rgba_in = rec[4];
                    const float G = expf(-0.5f * numerator_rho2 * denominator_rcp);
                    alpha = fminf(rgba_in.w * G, kMaxFragmentAlpha);
                    const float4 MT3 = rec[3];
                    if constexpr (kNeedsPointDepth) {
                        const float3 eval_point_diag = cross(fr.d, fr.m) * denominator_rcp;
                        depth = dot(f3(MT3), eval_point_diag) + MT3.w;
                    } else {
                        depth = MT3.w;
                    }
                    return valid && inside_cutoff && !(alpha < MT::min_alpha);
                };
                auto commit = [&](uint32_t j, float alpha, float depth, const float4& rgba_in) {
                    if constexpr (kFirstK) {
                        if (depth >= kd[K - 1]) return;
                        if constexpr (STATS) ++stat_accepted;
                        pool2[free_slot * TS::threads + tid] = make_float2(alpha, __uint_as_float(TRAIN ? batch_begin - range.x + j : s_prim[j]));
                        free_slot = slot_index(kbuffer_insert<K>(kd, ks, depth, slot_t(free_slot)));
                    } else if constexpr (kGlobal) {
                        if (done) return;
                        if constexpr (STATS) ++stat_accepted;
                        const float blending_weight = transmittance * alpha;
                        acc.x += blending_weight * rgba_in.x; acc.y += blending_weight * rgba_in.y; acc.z += blending_weight * rgba_in.z;
                        if constexpr (!TRAIN) {
                            if (use_median_depth) acc.w = (transmittance > 0.5f) ? depth : acc.w;
                            else acc.w += blending_weight * depth;
                        }
                        transmittance *= 1.0f - alpha;
                        if (transmittance < kTransmittanceThreshold) done = true;
                    } else {   // OIT_BLEND
                        if constexpr (STATS) ++stat_accepted;
                        if constexpr (TRAIN) {
                            acc.x += alpha * rgba_in.x; acc.y += alpha * rgba_in.y; acc.z += alpha * rgba_in.z;
                        } else {
                            acc += alpha * make_float4(rgba_in.x, rgba_in.y, rgba_in.z, depth);
                        }
                        acc_depth += alpha;
                        transmittance *= 1.0f - alpha;
                    }
                };
                for (uint32_t it = 0; it < n_iter; it += 2) {
                    bool v0, v1;
                    const uint32_t j0 = pop_candidate(v0);
                    const uint32_t j1 = pop_candidate(v1);
                    float alpha0, alpha1, depth0, depth1;
                    float4 rgba0, rgba1;
                    const bool ok0 = evaluate(v0, j0, alpha0, depth0, rgba0);
                    const bool ok1 = evaluate(v1, j1, alpha1, depth1, rgba1);
                    if (ok0) commit(j0, alpha0, depth0, rgba0);
                    if (ok1) commit(j1, alpha1, depth1, rgba1);
                }
            }
        }   // chunk loop
    }

    if (wait_failed) atomicOr(&status->error, 1u);
    if constexpr (STATS) {
        const uint32_t c = __reduce_add_sync(0xffffffffu, stat_candidates), a = __reduce_add_sync(0xffffffffu, stat_accepted);
        if (lane == 0) { atomicAdd(&status->candidate_pairs, (unsigned long long)c); atomicAdd(&status->accepted_fragments, (unsigned long long)a); }
        const uint32_t ins = __reduce_add_sync(0xffffffffu, stat_insertions);
        if (lane == 0 && stat_trips) {
            atomicAdd(&status->warp_trips, (unsigned long long)stat_trips); atomicAdd(&status->warp_trips_inserting, (unsigned long long)stat_trips_inserting);
            atomicAdd(&status->lane_insertions, (unsigned long long)ins);
        }
    }
    if (!inside) return;

    const uint32_t pixel_idx = width * py_i + px_i;
    const uint32_t n_pixels = width * height;

    if constexpr (TRAIN) {
        // ---- training forward: unclamped CHW image + what the backward pass needs per pixel ------------
        const uint32_t slot_base = (tile_y * grid_w + tile_x) * TS::threads + tid;   // tile-major pixel slot
        const uint32_t PP = tout.padded_pixels;
        float3 rgb_pixel = make_float3(0.0f, 0.0f, 0.0f);
        if constexpr (kHybrid) {
            // hybrid_blend/kernels/forward.cuh:176-233
            float transmittance_core = 1.0f;
            #pragma unroll
            for (int k = 0; k < K; ++k) {
                if (transmittance_core >= kTransmittanceThreshold) {
                    const float4 rgba = pool4[slot_index(ks[k]) * TS::threads + tid];
                    const float blending_weight = transmittance_core * rgba.w;
                    rgb_pixel += blending_weight * f3(rgba);
                    transmittance_core *= 1.0f - rgba.w;
                    if (transmittance_core < kTransmittanceThreshold) transmittance_core = 0.0f;
                }
            }
            float3 weighted_rgb_tail = make_float3(0.0f, 0.0f, 0.0f);
            float tail_info[6] = {0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f};   // the reference leaves these unwritten without tail mass; zeros make the backward terms vanish
            if (acc.w >= MT::min_alpha) {
                const float alpha_sum_tail_rcp = 1.0f / acc.w;
                const float3 rgb_tail = f3(acc);
                weighted_rgb_tail = transmittance_core * (1.0f - transmittance) * alpha_sum_tail_rcp * rgb_tail;
                tail_info[0] = rgb_tail.x; tail_info[1] = rgb_tail.y; tail_info[2] = rgb_tail.z;
                tail_info[3] = alpha_sum_tail_rcp; tail_info[4] = transmittance; tail_info[5] = transmittance_core;
            }
            #pragma unroll
            for (int c = 0; c < 6; ++c) tout.info_tail[c * PP + slot_base] = tail_info[c];
            float3 rgb_pixel_new = make_float3(0.0f, 0.0f, 0.0f);
            transmittance_core = 1.0f;
            #pragma unroll
            for (int k = 0; k < K; ++k) {
                const uint32_t primitive_idx = pool_idx[slot_index(ks[k]) * TS::threads + tid];
                const bool skip = primitive_idx == 0xffffffffu || transmittance_core < kTransmittanceThreshold;
                tout.idx_core[k * PP + slot_base] = skip ? 0xffffffffu : primitive_idx;
                if (!skip) {
                    const float4 rgba = pool4[slot_index(ks[k]) * TS::threads + tid];
                    const float blending_weight = transmittance_core * rgba.w;
                    rgb_pixel_new += blending_weight * f3(rgba);
                    const float one_minus_alpha = 1.0f - rgba.w;
                    const float one_minus_alpha_rcp = 1.0f / fmaxf(one_minus_alpha, kOneMinusAlphaEps);
                    tout.info_core[k * PP + slot_base] = make_float4(
                        rgba.x * transmittance_core - (rgb_pixel.x - rgb_pixel_new.x + weighted_rgb_tail.x) * one_minus_alpha_rcp,
                        rgba.y * transmittance_core - (rgb_pixel.y - rgb_pixel_new.y + weighted_rgb_tail.y) * one_minus_alpha_rcp,
                        rgba.z * transmittance_core - (rgb_pixel.z - rgb_pixel_new.z + weighted_rgb_tail.z) * one_minus_alpha_rcp,
                        blending_weight);
                    transmittance_core *= one_minus_alpha;
                }
            }
            rgb_pixel += weighted_rgb_tail;
        } else if constexpr (kFirstK) {
            // alpha_blend_first_k/kernels/forward.cuh:167-213
            float t = 1.0f;
            bool stop = false;
            float3 rgbs_core[K];
            #pragma unroll
            for (int k = 0; k < K; ++k) {
                rgbs_core[k] = make_float3(0.0f, 0.0f, 0.0f);
                if (!stop && t >= kTransmittanceThreshold) {
                    const float2 cell = pool2[slot_index(ks[k]) * TS::threads + tid];
                    const uint32_t position = __float_as_uint(cell.y);       // in the tile's list (training stores positions)
                    if (position == 0xffffffffu) stop = true;
                    else {
                        const float alpha = cell.x;
                        const uint32_t primitive_idx = __ldg(prims_sorted + range.x + position);
                        const float3 rgb = f3(ldg4(reinterpret_cast<const float*>(eval + primitive_idx) + 16));
                        rgbs_core[k] = rgb;
                        const float blending_weight = t * alpha;
                        rgb_pixel += blending_weight * rgb;
                        t *= 1.0f - alpha;
                    }
                }
            }
            float3 rgb_pixel_new = make_float3(0.0f, 0.0f, 0.0f);
            t = 1.0f;
            #pragma unroll
            for (int k = 0; k < K; ++k) {
                const float2 cell = pool2[slot_index(ks[k]) * TS::threads + tid];
                const uint32_t primitive_idx = __float_as_uint(cell.y);
                const bool skip = primitive_idx == 0xffffffffu || t < kTransmittanceThreshold;
                tout.idx_core[k * PP + slot_base] = skip ? 0xffffffffu : primitive_idx;
                if (!skip) {
                    const float alpha = cell.x;
                    const float3 rgb = rgbs_core[k];
                    const float blending_weight = t * alpha;
                    rgb_pixel_new += blending_weight * rgb;
                    const float one_minus_alpha = 1.0f - alpha;
                    const float one_minus_alpha_rcp = 1.0f / fmaxf(one_minus_alpha, kOneMinusAlphaEps);
                    tout.info_core[k * PP + slot_base] = make_float4(
                        rgb.x * t - (rgb_pixel.x - rgb_pixel_new.x) * one_minus_alpha_rcp,
                        rgb.y * t - (rgb_pixel.y - rgb_pixel_new.y) * one_minus_alpha_rcp,
                        rgb.z * t - (rgb_pixel.z - rgb_pixel_new.z) * one_minus_alpha_rcp,
                        blending_weight);
                    t *= one_minus_alpha;
                }
            }
        } else if constexpr (kGlobal) {
            rgb_pixel = f3(acc);
        } else {
            // oit_blend/kernels/forward.cuh:143-163
            float info[5] = {0.0f, 0.0f, 0.0f, 0.0f, 0.0f};
            if (acc_depth >= MT::min_alpha) {
                const float alpha_sum_rcp = 1.0f / acc_depth;
                rgb_pixel = (1.0f - transmittance) * alpha_sum_rcp * f3(acc);
                info[0] = acc.x; info[1] = acc.y; info[2] = acc.z; info[3] = alpha_sum_rcp; info[4] = transmittance;
            }
            #pragma unroll
            for (int c = 0; c < 5; ++c) tout.info_tail[c * PP + slot_base] = info[c];
        }
        image[pixel_idx] = rgb_pixel.x;
        image[n_pixels + pixel_idx] = rgb_pixel.y;
        image[2 * n_pixels + pixel_idx] = rgb_pixel.z;
        return;
    } else {
    // ---- inference compositing ----------------------------------------------------------------------
    float3 rgb_pixel = make_float3(0.0f, 0.0f, 0.0f);
    float depth_pixel = 0.0f;
    float alpha_pixel = 0.0f;
    if constexpr (kHybrid) {
        // hybrid_blend/kernels/inference.cuh:174-199
        float transmittance_core = 1.0f;
        #pragma unroll
        for (int k = 0; k < K; ++k) {
            if (transmittance_core >= kTransmittanceThreshold) {
                const float4 rgba_premultiplied = pool4[slot_index(ks[k]) * TS::threads + tid];
                rgb_pixel += transmittance_core * f3(rgba_premultiplied);
                const float depth = kd[k];
                if (use_median_depth) depth_pixel = (transmittance_core > 0.5f && depth < FLT_MAX) ? depth : depth_pixel;
                else depth_pixel += transmittance_core * rgba_premultiplied.w * depth;
                transmittance_core *= 1.0f - rgba_premultiplied.w;
            }
        }
        float total_alpha = 1.0f - transmittance_core;
        if (transmittance_core >= kTransmittanceThreshold && acc.w >= MT::min_alpha) {
            const float weight_tail = transmittance_core * (1.0f - transmittance);
            rgb_pixel += weight_tail * (1.0f / acc.w) * f3(acc);
            if (!use_median_depth) depth_pixel += weight_tail * (1.0f / acc.w) * acc_depth;
            total_alpha += weight_tail;
        }
        if (!use_median_depth) depth_pixel = (total_alpha > 0.0f) ? depth_pixel / total_alpha : 0.0f;
        alpha_pixel = total_alpha;
    } else if constexpr (kFirstK) {
        // alpha_blend_first_k/kernels/inference.cuh:172-191
        float t = 1.0f;
        bool stop = false;
        #pragma unroll
        for (int k = 0; k < K; ++k) {
            if (!stop && t >= kTransmittanceThreshold) {
                const float2 cell = pool2[slot_index(ks[k]) * TS::threads + tid];
                const uint32_t primitive_idx = __float_as_uint(cell.y);
                if (primitive_idx == 0xffffffffu) { stop = true; }
                else {
                    const float alpha = cell.x;
                    const float blending_weight = t * alpha;
                    const float4 rgba = ldg4(reinterpret_cast<const float*>(eval + primitive_idx) + 16);
                    rgb_pixel += blending_weight * f3(rgba);
                    const float depth = kd[k];
                    if (use_median_depth) depth_pixel = (t > 0.5f) ? depth : depth_pixel;
                    else depth_pixel += blending_weight * depth;
                    t *= 1.0f - alpha;
                }
            }
        }
        if (!use_median_depth) depth_pixel = (t < 1.0f) ? depth_pixel / (1.0f - t) : 0.0f;
        alpha_pixel = 1.0f - t;
    } else if constexpr (kGlobal) {
        rgb_pixel = f3(acc);
        depth_pixel = acc.w;
        if (!use_median_depth) depth_pixel = (transmittance < 1.0f) ? depth_pixel / (1.0f - transmittance) : 0.0f;
        alpha_pixel = 1.0f - transmittance;
    } else {
        // oit_blend/kernels/inference.cuh:150-160
        float4 rgbd_pixel = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        if (acc_depth >= MT::min_alpha) {
            const float alpha = 1.0f - transmittance;
            rgbd_pixel = alpha * (1.0f / acc_depth) * acc;
            rgbd_pixel.w = rgbd_pixel.w / alpha;
            alpha_pixel = alpha;
        }
        rgb_pixel = f3(rgbd_pixel);
        depth_pixel = rgbd_pixel.w;
    }
    if (to_chw) {
        image[pixel_idx] = __saturatef(rgb_pixel.x);
        image[n_pixels + pixel_idx] = __saturatef(rgb_pixel.y);
        image[2 * n_pixels + pixel_idx] = __saturatef(rgb_pixel.z);
    } else {
        const uint32_t base_idx = 3 * pixel_idx;
        image[base_idx] = __saturatef(rgb_pixel.x);
        image[base_idx + 1] = __saturatef(rgb_pixel.y);
        image[base_idx + 2] = __saturatef(rgb_pixel.z);
    }
    if (depth_out) depth_out[pixel_idx] = depth_pixel;
    if (alpha_out) alpha_out[pixel_idx] = alpha_pixel;
    }
}

template <int MODE, int K, bool TRAIN, bool STATS>
cudaError_t launch_blend_t(const FrameGeometry& geo, const PrimBuffers& prim, const uint32_t* prims_sorted, const uint2* tile_ranges,
                           const BlendOutputs& out, const TrainPixelBuffers& tout, FrameStatus* status, cudaStream_t stream) {
    using SL = SmemLayout<MODE, K, TRAIN>;
    auto kernel = blend_kernel<MODE, K, TRAIN, STATS>;
    static PerDeviceOnce configured;
    const cudaError_t err = configured.run([&] { return cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(SL::total)); });
    if (err != cudaSuccess) return err;
    using TS = TileShape<MODE>;
    const dim3 grid((geo.width + TS::tw - 1) / TS::tw, (geo.height + TS::th - 1) / TS::th, 1);
    kernel<<<grid, TS::threads, SL::total, stream>>>(tile_ranges, prims_sorted, prim.eval, prim.cull, out.image, out.depth, out.alpha, tout,
                                                                  uint32_t(geo.width), uint32_t(geo.height), uint32_t(geo.grid_w), out.to_chw,
                                                                  out.use_median_depth, status);
    return cudaGetLastError();
}

template <int MODE, int K>
cudaError_t launch_mode_k(bool train, const FrameGeometry& geo, const PrimBuffers& prim, const uint32_t* prims_sorted, const uint2* tile_ranges,
                          const BlendOutputs& out, const TrainPixelBuffers& tout, FrameStatus* status, cudaStream_t stream) {
    if (train) return launch_blend_t<MODE, K, true, false>(geo, prim, prims_sorted, tile_ranges, out, tout, status, stream);
    return out.collect_stats ? launch_blend_t<MODE, K, false, true>(geo, prim, prims_sorted, tile_ranges, out, tout, status, stream)
                             : launch_blend_t<MODE, K, false, false>(geo, prim, prims_sorted, tile_ranges, out, tout, status, stream);
}

// K is rounded down to a power of two <= 32 (hybrid_blend/inference.cu:15-28)
template <int MODE>
cudaError_t launch_mode(bool train, int K, const FrameGeometry& geo, const PrimBuffers& prim, const uint32_t* prims_sorted, const uint2* tile_ranges,
                        const BlendOutputs& out, const TrainPixelBuffers& tout, FrameStatus* status, cudaStream_t stream) {
    if (K >= 32) return launch_mode_k<MODE, 32>(train, geo, prim, prims_sorted, tile_ranges, out, tout, status, stream);
    if (K >= 16) return launch_mode_k<MODE, 16>(train, geo, prim, prims_sorted, tile_ranges, out, tout, status, stream);
    if (K >= 8) return launch_mode_k<MODE, 8>(train, geo, prim, prims_sorted, tile_ranges, out, tout, status, stream);
    if (K >= 4) return launch_mode_k<MODE, 4>(train, geo, prim, prims_sorted, tile_ranges, out, tout, status, stream);
    if (K >= 2) return launch_mode_k<MODE, 2>(train, geo, prim, prims_sorted, tile_ranges, out, tout, status, stream);
    return launch_mode_k<MODE, 1>(train, geo, prim, prims_sorted, tile_ranges, out, tout, status, stream);
}

}  // namespace

int effective_k(int mode, int K) {
    if (mode != HTGS_MODE_HYBRID_BLEND && mode != HTGS_MODE_ALPHA_BLEND_FIRST_K) return 1;
    return K >= 32 ? 32 : K >= 16 ? 16 : K >= 8 ? 8 : K >= 4 ? 4 : K >= 2 ? 2 : 1;
}

cudaError_t launch_blend(int mode, int K, bool train, const FrameGeometry& geo, const PrimBuffers& prim, const uint32_t* prims_sorted,
                         const uint2* tile_ranges, const BlendOutputs& out, const TrainPixelBuffers& tout, FrameStatus* status, cudaStream_t stream) {
    switch (mode) {
        case HTGS_MODE_HYBRID_BLEND: return launch_mode<HTGS_MODE_HYBRID_BLEND>(train, K, geo, prim, prims_sorted, tile_ranges, out, tout, status, stream);
        case HTGS_MODE_ALPHA_BLEND_FIRST_K: return launch_mode<HTGS_MODE_ALPHA_BLEND_FIRST_K>(train, K, geo, prim, prims_sorted, tile_ranges, out, tout, status, stream);
        case HTGS_MODE_ALPHA_BLEND_GLOBAL_ORDERING: return launch_mode_k<HTGS_MODE_ALPHA_BLEND_GLOBAL_ORDERING, 1>(train, geo, prim, prims_sorted, tile_ranges, out, tout, status, stream);
        case HTGS_MODE_OIT_BLEND: return launch_mode_k<HTGS_MODE_OIT_BLEND, 1>(train, geo, prim, prims_sorted, tile_ranges, out, tout, status, stream);
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace htgs
