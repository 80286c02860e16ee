// Relaxed-precision inference for HYBRID_BLEND, ALPHA_BLEND_FIRST_K and OIT_BLEND: the kernels behind fast_rasterize.
//
// Replaces blend_cu of rasterization/include/{hybrid_blend,alpha_blend_first_k,oit_blend}/kernels/fast_inference.cuh
// (the reference's fast-math build; HYBRID keeps a half-precision K-buffer; RGB only, no depth output).  Results agree with that kernel to
// about 1e-3 per channel, not bit for bit: this path trades the operation-for-operation evaluation of the
// exact kernel (blend.cu) for fewer instructions per fragment.
//
//  * Staging and candidate masks are those of the exact kernel: one 80-byte bulk asynchronous copy per instance,
//    outline test with lane = Gaussian, 32 warp ballots per 32 Gaussians, every lane then walks its own mask.
//  * Per fragment, rho^2 and depth are ratios of quadratics in (pixel - projected centre) whose coefficients the
//    preprocess stored per Gaussian (FastRecord): 6 shared-memory loads, 20 multiply-adds, one approximate
//    reciprocal and one approximate exp2 instead of two plane constructions, two cross products, an IEEE divide
//    and expf.  The rho^2 cutoff test is implied by the alpha test (opacity <= 1) and dropped.
//  * K-buffer.  The K nearest core fragments of a pixel are kept UNSORTED in shared memory: one key per entry (the
//    fragment depth with its low log2(K) mantissa bits replaced by the entry's position, so the largest key names
//    the entry to evict) and a half-precision premultiplied RGBA payload (as the reference's fast path stores it).
//    An insertion overwrites the entry of the largest key, re-reads the one row of four keys that changed and
//    updates the per-row maxima it keeps in registers: about 20 ALU-pipe instructions and 9 shared-memory wavefronts
//    instead of 5 instructions per level of a sorted chain.
//    Entries are sorted once per pixel when the tile is composited.  Fragments of exactly equal depth are ordered by
//    position instead of by arrival.  FIRST_K uses the same buffer with (alpha, Gaussian index) payloads and no tail;
//    OIT has no buffer at all and skips the depth polynomial.
#include "kernels.h"

#include <cuda_fp16.h>


namespace htgs {

namespace {

constexpr int kFastThreads = 64;     // 8 x 8 pixel tile, one thread per pixel
constexpr int kFastBatch = 64;       // instances staged per iteration, one per thread

template <int MODE, int K> struct FastSmem {
    static constexpr bool has_kbuffer = MODE != HTGS_MODE_OIT_BLEND;
    static constexpr bool has_prim = MODE == HTGS_MODE_ALPHA_BLEND_FIRST_K;
    static constexpr size_t rec_off = 0;
    static constexpr size_t rec_bytes = size_t(kFastBatch) * sizeof(FastRecord);
    static constexpr size_t cull4_off = rec_off + rec_bytes;
    static constexpr size_t cullc_off = cull4_off + size_t(kFastBatch) * 16;
    static constexpr size_t ctr_off = cullc_off + size_t(kFastBatch) * 4;      // float2: projected centre relative to the tile origin
    static constexpr size_t prim_off = ctr_off + size_t(kFastBatch) * 8;        // Gaussian index of every staged instance (FIRST_K)
    static constexpr size_t bar_off = prim_off + (has_prim ? size_t(kFastBatch) * 4 : 0);
    static constexpr size_t keys_off = bar_off + 16;
    static constexpr size_t keys_bytes = has_kbuffer ? size_t(K) * kFastThreads * 4 : 0;     // uint4 [K/4][threads]
    static constexpr size_t pay_off = keys_off + keys_bytes;
    static constexpr size_t pay_bytes = has_kbuffer ? size_t(K) * kFastThreads * 8 : 0;      // 8-byte payload [K][threads]
    static constexpr size_t total = pay_off + pay_bytes;
    static_assert(bar_off % 16 == 0 && keys_off % 16 == 0, "shared-memory sections must stay 16-byte aligned");
};

__device__ __forceinline__ float rcp_approx(float x) { float y; asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x)); return y; }
__device__ __forceinline__ float exp2_approx(float x) { float y; asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x)); return y; }

// maximum of N keys as a tree of three-input max
template <int N>
__device__ __forceinline__ uint32_t reduce_max(const uint32_t (&v)[N]) {
    if constexpr (N == 1) return v[0];
    else if constexpr (N == 2) return max(v[0], v[1]);
    else {
        constexpr int M = N / 3 + N % 3;
        uint32_t r[M];
        #pragma unroll
        for (int i = 0; i < N / 3; ++i) r[i] = __vimax3_u32(v[3 * i], v[3 * i + 1], v[3 * i + 2]);
        #pragma unroll
        for (int i = 0; i < N % 3; ++i) r[N / 3 + i] = v[3 * (N / 3) + i];
        return reduce_max<M>(r);
    }
}

// Core keys: 32-bit unsigned, ordered like the depth, carrying the entry's position in the low log2(K) bits.
// The depth keeps its full 23-bit mantissa; the exponent is re-based to a window of 2^(9 - log2 K) binades starting
// at 2^kMinExp (K = 16: [2^-12, 2^20), K = 32: [2^-4, 2^12)); depths outside the window (or negative) saturate, which
// only loses the order among fragments that all lie outside it.
template <int K> struct KeyCodec {
    static constexpr int pos_bits = K == 4 ? 2 : K == 8 ? 3 : K == 16 ? 4 : 5;
    static constexpr int exp_bits = 9 - pos_bits;
    static constexpr int min_exp = K == 32 ? -4 : -12;
    static constexpr int32_t base = int32_t(127 + min_exp) << 23;
    static constexpr int32_t limit = int32_t((1u << (23 + exp_bits)) - 1u);
    static __device__ __forceinline__ uint32_t encode(float depth, uint32_t pos) {
        const int32_t rel = min(max(__float_as_int(depth) - base, 0), limit);
        return uint32_t(rel) * uint32_t(K) + pos;
    }
    static __device__ __forceinline__ float decode(uint32_t key) { return __int_as_float(int32_t(key >> pos_bits) + base); }
    static constexpr uint32_t empty = 0xffffffffu & ~uint32_t(K - 1);
};

__device__ __forceinline__ uint2 pack_half4(float x, float y, float z, float w) {
    const __half2 a = __floats2half2_rn(x, y), b = __floats2half2_rn(z, w);
    return make_uint2(*reinterpret_cast<const uint32_t*>(&a), *reinterpret_cast<const uint32_t*>(&b));
}
__device__ __forceinline__ float4 unpack_half4(uint2 p) {
    const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&p.x));
    const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&p.y));
    return make_float4(a.x, a.y, b.x, b.y);
}

// Replace the entry with the largest key by (depth, payload); returns the payload that fell out (zeros for an
// entry that was still empty).  Entry c keeps its key in component (c & 3) of uint4 row (c >> 2).  Registers hold
// the maximum of every row (`row_max`), so that only the row that changed is read back: one vector load instead
// of K/4 (shared-memory bandwidth is what bounds this kernel).
template <int K>
__device__ __forceinline__ uint2 core_replace(uint32_t* keys, uint2* pay, uint32_t tid, float depth, uint2 payload, uint32_t (&row_max)[K / 4],
                                              uint32_t& kmax) {
    const uint32_t c = kmax & uint32_t(K - 1);
    uint2* slot = pay + c * kFastThreads + tid;
    const uint2 evicted = *slot;
    *slot = payload;
    const uint32_t q = c >> 2;
    uint4* row_ptr = reinterpret_cast<uint4*>(keys) + q * kFastThreads + tid;
    reinterpret_cast<uint32_t*>(row_ptr)[c & 3u] = KeyCodec<K>::encode(depth, c);
    const uint4 row = *row_ptr;
    const uint32_t m = max(__vimax3_u32(row.x, row.y, row.z), row.w);
    #pragma unroll
    for (int i = 0; i < K / 4; ++i) row_max[i] = (q == uint32_t(i)) ? m : row_max[i];
    kmax = reduce_max<K / 4>(row_max);
    return evicted;
}

template <int MODE, int K>
__global__ void __launch_bounds__(kFastThreads) blend_fast_kernel(
    const uint2* __restrict__ tile_ranges, const uint32_t* __restrict__ prims_sorted, const FastRecord* __restrict__ records,
    const CullRecord* __restrict__ cull, float* __restrict__ image, uint32_t width, uint32_t height, uint32_t grid_w, bool to_chw,
    FrameStatus* status)
{
    using SL = FastSmem<MODE, K>;
    using MT = ModeTraits<MODE>;
    constexpr bool kHybrid = MODE == HTGS_MODE_HYBRID_BLEND;
    constexpr bool kFirstK = MODE == HTGS_MODE_ALPHA_BLEND_FIRST_K;
    constexpr bool kOit = MODE == HTGS_MODE_OIT_BLEND;
    static_assert(kHybrid || kFirstK || kOit, "no relaxed-precision kernel for this mode");
    extern __shared__ __align__(128) unsigned char smem[];
    FastRecord* s_rec = reinterpret_cast<FastRecord*>(smem + SL::rec_off);
    float4* s_cull4 = reinterpret_cast<float4*>(smem + SL::cull4_off);
    float* s_cullc = reinterpret_cast<float*>(smem + SL::cullc_off);
    uint64_t* s_bar = reinterpret_cast<uint64_t*>(smem + SL::bar_off);
    float2* s_ctr = reinterpret_cast<float2*>(smem + SL::ctr_off);
    [[maybe_unused]] uint32_t* s_prim = reinterpret_cast<uint32_t*>(smem + SL::prim_off);
    [[maybe_unused]] uint32_t* keys = reinterpret_cast<uint32_t*>(smem + SL::keys_off);
    [[maybe_unused]] uint2* pay = reinterpret_cast<uint2*>(smem + SL::pay_off);

    const uint32_t tid = threadIdx.x;
    const uint32_t warp = tid >> 5, lane = tid & 31;
    const uint32_t tile_x = blockIdx.x, tile_y = blockIdx.y;
    const uint32_t px_i = tile_x * 8 + (tid & 7);
    const uint32_t py_i = tile_y * 8 + (tid >> 3);
    const bool inside = px_i < width && py_i < height;
    const float local_x = float(tid & 7), local_y = float(tid >> 3);   // pixel position inside the tile

    if (tid == 0) { mbar_init(s_bar, kFastThreads); mbar_fence_init(); }

    // empty core: the largest keys, carrying their position; zero payloads (FIRST_K: alpha 0, no Gaussian)
    if constexpr (SL::has_kbuffer) {
        #pragma unroll
        for (int c = 0; c < K; ++c) {
            keys[((c >> 2) * kFastThreads + tid) * 4 + (c & 3)] = KeyCodec<K>::empty | uint32_t(c);
            pay[c * kFastThreads + tid] = make_uint2(0u, kFirstK ? 0xffffffffu : 0u);
        }
    }
    [[maybe_unused]] uint32_t row_max[K / 4];
    #pragma unroll
    for (int q = 0; q < K / 4; ++q) row_max[q] = KeyCodec<K>::empty | uint32_t(4 * q + 3);
    [[maybe_unused]] uint32_t kmax = 0xffffffffu;            // position K-1
    [[maybe_unused]] float depth_max = __int_as_float(0x7f800000);   // depth a fragment has to beat to enter the core
    float4 tail = make_float4(0.0f, 0.0f, 0.0f, 0.0f);       // HYBRID tail / OIT sums: premultiplied rgb, alpha sum
    float transmittance_tail = 1.0f;

    const uint2 range = tile_ranges[tile_y * grid_w + tile_x];
    uint32_t phase = 0;
    bool wait_failed = false;
    const float rect_x0 = float(tile_x * 8);
    const float tile_y0 = float(tile_y * 8);
    const float rect_y0 = float(tile_y * 8 + warp * 4);

    uint32_t g_next = 0;
    float4 c0_next = make_float4(__int_as_float(0x7f800000), 0.0f, 0.0f, 0.0f);   // "reject everything"
    float4 c1_next = make_float4(0.0f, 0.0f, 0.0f, 0.0f);                         // c, cx_lo, cy_lo
    if (range.x + tid < range.y) {
        g_next = __ldg(prims_sorted + range.x + tid);
        c0_next = ldg4(reinterpret_cast<const float*>(cull + g_next));
        c1_next = ldg4(reinterpret_cast<const float*>(cull + g_next) + 4);
    }
    __syncthreads();

    for (uint32_t batch_begin = range.x; batch_begin < range.y; batch_begin += kFastBatch) {
        __syncthreads();
        // ---- staging: one instance per thread, from the prefetch registers ----------------------------
        const bool valid_inst = batch_begin + tid < range.y;
        s_cull4[tid] = c0_next;
        s_cullc[tid] = c1_next.x;
        s_ctr[tid] = make_float2((rect_x0 - c0_next.x) - c1_next.y, (tile_y0 - c0_next.y) - c1_next.z);
        if (valid_inst) {
            mbar_arrive_expect_tx(s_bar, uint32_t(sizeof(FastRecord)));
            bulk_copy_g2s(s_rec + tid, records + g_next, uint32_t(sizeof(FastRecord)), s_bar);
            if constexpr (SL::has_prim) s_prim[tid] = g_next;
        } else {
            mbar_arrive(s_bar);
        }
        const uint32_t inst_next = batch_begin + kFastBatch + tid;
        const bool valid_next = inst_next < range.y;
        if (valid_next) g_next = __ldg(prims_sorted + inst_next);
        __syncthreads();
        // ---- candidate masks: lane = Gaussian, one ballot per pixel of the warp ------------------------
        uint64_t cand = 0;
        #pragma unroll
        for (int half = 0; half < 2; ++half) {
            const uint32_t j = half * 32 + lane;
            const float4 c0 = s_cull4[j];
            const float cc = s_cullc[j];
            const float dx0 = rect_x0 - c0.x, dy0 = rect_y0 - c0.y;
            uint32_t mine = 0;
            #pragma unroll
            for (int r = 0; r < 4; ++r) {
                const float dy = dy0 + float(r);
                const float b2dy = c0.w * dy, cdy2 = cc * dy * dy;
                #pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const float dx = dx0 + float(i);
                    const float q = dx * (c0.z * dx + b2dy) + cdy2;
                    const uint32_t touched = __ballot_sync(0xffffffffu, q <= 1.0f);
                    if (int(lane) == r * 8 + i) mine = touched;
                }
            }
            cand |= uint64_t(mine) << (32 * half);
        }
        if (!inside) cand = 0;
        if (valid_next) {   // the index prefetched before the barrier has arrived by now
            c0_next = ldg4(reinterpret_cast<const float*>(cull + g_next));
            c1_next = ldg4(reinterpret_cast<const float*>(cull + g_next) + 4);
        } else {
            c0_next = make_float4(__int_as_float(0x7f800000), 0.0f, 0.0f, 0.0f);
            c1_next = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        }
        // ---- fragments -----------------------------------------------------------------------------------
        if (!mbar_wait_bounded(s_bar, phase)) wait_failed = true;
        phase ^= 1;
        const uint32_t n_iter = __reduce_max_sync(0xffffffffu, uint32_t(__popcll(cand)));
        auto pop_candidate = [&](bool& valid) -> uint32_t {
            valid = cand != 0;
            const uint32_t j = valid ? uint32_t(__ffsll((long long)cand) - 1) : 0u;
            cand &= cand - 1;
            return j;
        };
        auto evaluate = [&](uint32_t j, float& depth, float4& frag) {
            const float4* rec = reinterpret_cast<const float4*>(s_rec + j);
            const float2 ctr = s_ctr[j];
            const float4 r0 = rec[0], r1 = rec[1], r3 = rec[3], r4 = rec[4];
            const float dx = local_x + ctr.x, dy = local_y + ctr.y;
            const float xx = dx * dx, xy = dx * dy, yy = dy * dy;
            const float e = fmaf(r0.x, xx, fmaf(r0.y, xy, r0.z * yy));
            const float den = fmaf(r0.w, dx, fmaf(r1.y, xx, 1.0f)) + fmaf(r1.x, dy, fmaf(r1.z, xy, r1.w * yy));
            const float den_rcp = rcp_approx(den);
            const float alpha = fminf(exp2_approx(fmaf(e, den_rcp, r3.z)), kMaxFragmentAlpha);
            if constexpr (kOit) {
                depth = 0.0f;   // the RGB-only OIT result does not depend on depth
            } else {
                const float4 r2 = rec[2];
                const float num_z = fmaf(r2.x, dx, fmaf(r2.z, xx, r2.w * xy)) + fmaf(r2.y, dy, r3.x * yy);
                depth = fmaf(num_z, den_rcp, r3.y);
            }
            if constexpr (kFirstK) frag = make_float4(0.0f, 0.0f, 0.0f, alpha);   // the colour is fetched when the tile is composited
            else frag = make_float4(r3.w * alpha, r4.x * alpha, r4.y * alpha, alpha);
        };
        auto commit = [&](uint32_t j, float depth, float4 frag) {
            if constexpr (kHybrid) {
                if (depth < depth_max && frag.w >= MT::min_alpha_core) {
                    frag = unpack_half4(core_replace<K>(keys, pay, tid, depth, pack_half4(frag.x, frag.y, frag.z, frag.w), row_max, kmax));
                    depth_max = KeyCodec<K>::decode(kmax);
                }
                tail += frag;
                transmittance_tail *= 1.0f - frag.w;
            } else if constexpr (kFirstK) {
                if (depth < depth_max) {   // whatever falls out of the buffer is dropped (alpha_blend_first_k/kernels/fast_inference.cuh:147-160)
                    core_replace<K>(keys, pay, tid, depth, make_uint2(__float_as_uint(frag.w), s_prim[j]), row_max, kmax);
                    depth_max = KeyCodec<K>::decode(kmax);
                }
            } else {   // oit_blend/kernels/fast_inference.cuh:138-141
                tail += frag;
                transmittance_tail *= 1.0f - frag.w;
            }
        };
        for (uint32_t it = 0; it < n_iter; it += 2) {
            bool v0, v1;
            const uint32_t j0 = pop_candidate(v0);
            const uint32_t j1 = pop_candidate(v1);
            float depth0, depth1;
            float4 frag0, frag1;
            evaluate(j0, depth0, frag0);
            evaluate(j1, depth1, frag1);
            if (v0 && !(frag0.w < MT::min_alpha)) commit(j0, depth0, frag0);
            if (v1 && !(frag1.w < MT::min_alpha)) commit(j1, depth1, frag1);
        }
    }

    if (wait_failed) atomicOr(&status->error, 1u);
    if (!inside) return;

    float3 rgb_pixel = make_float3(0.0f, 0.0f, 0.0f);
    if constexpr (SL::has_kbuffer) {
        // ---- composite: sort the core entries by key, blend front to back (hybrid_blend/kernels/fast_inference.cuh:193-216,
        // alpha_blend_first_k/kernels/fast_inference.cuh:166-180)
        uint32_t v[K];
        {
            const uint4* rows = reinterpret_cast<const uint4*>(keys) + tid;
            #pragma unroll
            for (int q = 0; q < K / 4; ++q) {
                const uint4 row = rows[q * kFastThreads];
                v[4 * q] = row.x; v[4 * q + 1] = row.y; v[4 * q + 2] = row.z; v[4 * q + 3] = row.w;
            }
        }
        #pragma unroll
        for (int k = 2; k <= K; k <<= 1) {
            #pragma unroll
            for (int j = k >> 1; j > 0; j >>= 1) {
                #pragma unroll
                for (int i = 0; i < K; ++i) {
                    const int l = i ^ j;
                    if (l > i) {
                        const uint32_t lo = min(v[i], v[l]), hi = max(v[i], v[l]);
                        if ((i & k) == 0) { v[i] = lo; v[l] = hi; } else { v[i] = hi; v[l] = lo; }
                    }
                }
            }
        }
        float transmittance_core = 1.0f;
        #pragma unroll
        for (int k = 0; k < K; ++k) {
            if (transmittance_core >= kTransmittanceThreshold) {
                const uint32_t c = v[k] & uint32_t(K - 1);
                const uint2 cell = pay[c * kFastThreads + tid];
                if constexpr (kHybrid) {
                    const float4 rgba = unpack_half4(cell);
                    rgb_pixel += transmittance_core * f3(rgba);
                    transmittance_core *= 1.0f - rgba.w;
                } else {
                    if (cell.y == 0xffffffffu) { transmittance_core = 0.0f; continue; }   // empty entries sort last: nothing follows
                    const float alpha = __uint_as_float(cell.x);
                    const float* rec = reinterpret_cast<const float*>(records + cell.y);
                    const float3 rgb = make_float3(__ldg(rec + 15), __ldg(rec + 16), __ldg(rec + 17));   // FastRecord::r, g, b
                    rgb_pixel += (transmittance_core * alpha) * rgb;
                    transmittance_core *= 1.0f - alpha;
                }
            }
        }
        if constexpr (kHybrid) {
            if (transmittance_core >= kTransmittanceThreshold && tail.w >= MT::min_alpha) {
                const float weight_tail = transmittance_core * (1.0f - transmittance_tail);
                rgb_pixel += weight_tail * (1.0f / tail.w) * f3(tail);
            }
        }
    } else {
        // oit_blend/kernels/fast_inference.cuh:147-152
        if (tail.w >= MT::min_alpha) rgb_pixel = ((1.0f - transmittance_tail) * (1.0f / tail.w)) * f3(tail);
    }
    const uint32_t pixel_idx = width * py_i + px_i;
    if (to_chw) {
        const uint32_t n_pixels = width * height;
        image[pixel_idx] = __saturatef(rgb_pixel.x);
        image[n_pixels + pixel_idx] = __saturatef(rgb_pixel.y);
        image[2 * n_pixels + pixel_idx] = __saturatef(rgb_pixel.z);
    } else {
        image[3 * pixel_idx] = __saturatef(rgb_pixel.x);
        image[3 * pixel_idx + 1] = __saturatef(rgb_pixel.y);
        image[3 * pixel_idx + 2] = __saturatef(rgb_pixel.z);
    }
}

template <int MODE, int K>
cudaError_t launch_fast_k(const FrameGeometry& geo, const PrimBuffers& prim, const uint32_t* prims_sorted, const uint2* tile_ranges, float* image,
                          bool to_chw, FrameStatus* status, cudaStream_t stream) {
    using SL = FastSmem<MODE, K>;
    static PerDeviceOnce configured;
    const cudaError_t cfg = configured.run([] {
        const cudaError_t err = cudaFuncSetAttribute(blend_fast_kernel<MODE, K>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(SL::total));
        if (err != cudaSuccess) return err;
        return cudaFuncSetAttribute(blend_fast_kernel<MODE, K>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    });
    if (cfg != cudaSuccess) return cfg;
    if (geo.n_tiles == 0) return cudaSuccess;
    blend_fast_kernel<MODE, K><<<dim3(geo.grid_w, geo.grid_h), kFastThreads, SL::total, stream>>>(
        tile_ranges, prims_sorted, reinterpret_cast<const FastRecord*>(prim.eval), prim.cull, image, uint32_t(geo.width), uint32_t(geo.height),
        uint32_t(geo.grid_w), to_chw, status);
    return cudaGetLastError();
}

template <int MODE>
cudaError_t launch_fast_mode(int K, const FrameGeometry& geo, const PrimBuffers& prim, const uint32_t* prims_sorted, const uint2* tile_ranges,
                             float* image, bool to_chw, FrameStatus* status, cudaStream_t stream) {
    switch (effective_k(MODE, K)) {
        case 4: return launch_fast_k<MODE, 4>(geo, prim, prims_sorted, tile_ranges, image, to_chw, status, stream);
        case 8: return launch_fast_k<MODE, 8>(geo, prim, prims_sorted, tile_ranges, image, to_chw, status, stream);
        case 16: return launch_fast_k<MODE, 16>(geo, prim, prims_sorted, tile_ranges, image, to_chw, status, stream);
        case 32: return launch_fast_k<MODE, 32>(geo, prim, prims_sorted, tile_ranges, image, to_chw, status, stream);
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace

bool blend_fast_supports(int mode, int K) {
    if (mode == HTGS_MODE_OIT_BLEND) return true;
    if (mode != HTGS_MODE_HYBRID_BLEND && mode != HTGS_MODE_ALPHA_BLEND_FIRST_K) return false;
    const int k = effective_k(mode, K);
    return k == 4 || k == 8 || k == 16 || k == 32;
}

cudaError_t launch_blend_fast(int mode, int K, const FrameGeometry& geo, const PrimBuffers& prim, const uint32_t* prims_sorted, const uint2* tile_ranges,
                              float* image, bool to_chw, FrameStatus* status, cudaStream_t stream) {
    switch (mode) {
        case HTGS_MODE_HYBRID_BLEND: return launch_fast_mode<HTGS_MODE_HYBRID_BLEND>(K, geo, prim, prims_sorted, tile_ranges, image, to_chw, status, stream);
        case HTGS_MODE_ALPHA_BLEND_FIRST_K: return launch_fast_mode<HTGS_MODE_ALPHA_BLEND_FIRST_K>(K, geo, prim, prims_sorted, tile_ranges, image, to_chw, status, stream);
        case HTGS_MODE_OIT_BLEND: return launch_fast_k<HTGS_MODE_OIT_BLEND, 4>(geo, prim, prims_sorted, tile_ranges, image, to_chw, status, stream);
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace htgs
