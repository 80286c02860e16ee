// CPU oracle for the HTGS rasterizer hot path.  TEST INFRASTRUCTURE ONLY.
//
// This file is a CPU restatement of the reference CUDA rasterizer
// (HTGSCudaBackend).  It is used as the checker by tests/, by the smoke entry
// and as the "cpu_baseline"/"reference" arm of bench.py.  The product (the
// CUDA library under htgs_b200/csrc) never links or calls it.
//
// The reference has no CPU path (Renderer.py:76-77), so every function below
// follows a CUDA kernel of the reference and cites it by file:line relative
// to HTGSCudaBackend/HTGSCudaBackend/ ("R/" = rasterization/).
//
// Parity pinning: the reference ships no tests or golden vectors.  The oracle
// is pinned against outputs of the reference extension itself, generated on a
// B200 by tests/golden/make_golden.py and committed under tests/golden/.
//
// Everything is templated on the scalar type: float64 is the reported CPU
// baseline and the tolerance oracle, float32 (same operation order, fused
// multiply-adds where a CUDA compiler would most plausibly contract them) is
// the debugging aid for the integer stages.  libm's logf/expf are not the
// CUDA ones, so the float32 variant is close to, but not bit-identical with,
// a GPU run.
//
// Build: see oracle/Makefile  (g++ -O3 -march=x86-64-v3 -shared -fPIC -pthread).

#include <algorithm>
#include <atomic>
#include <cfloat>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <thread>
#include <vector>

namespace {

// ----------------------------------------------------------------------------
// small vector algebra (the handful of operations the reference takes from
// utils/helper_math.h: dot 1267-1274, cross 1451-1454, normalize 1328-1332)
// ----------------------------------------------------------------------------
template <typename R> struct Vec3 { R x, y, z; };
template <typename R> struct Vec4 { R x, y, z, w; };

template <typename R> inline R mul_add(R a, R b, R c);
template <> inline float mul_add<float>(float a, float b, float c) { return std::fmaf(a, b, c); }
template <> inline double mul_add<double>(double a, double b, double c) { return a * b + c; }

template <typename R> inline R dot3(const Vec3<R>& a, const Vec3<R>& b) {
    return mul_add(a.z, b.z, mul_add(a.x, b.x, a.y * b.y));
}
template <typename R> inline R dot4(const Vec4<R>& a, const Vec4<R>& b) {
    return mul_add(a.w, b.w, mul_add(a.z, b.z, mul_add(a.x, b.x, a.y * b.y)));
}
template <typename R> inline Vec3<R> cross3(const Vec3<R>& a, const Vec3<R>& b) {
    return {mul_add(a.y, b.z, -(a.z * b.y)), mul_add(a.z, b.x, -(a.x * b.z)), mul_add(a.x, b.y, -(a.y * b.x))};
}
template <typename R> inline Vec3<R> xyz(const Vec4<R>& a) { return {a.x, a.y, a.z}; }
template <typename R> inline Vec4<R> mul4(const Vec4<R>& a, const Vec4<R>& b) { return {a.x * b.x, a.y * b.y, a.z * b.z, a.w * b.w}; }
template <typename R> inline Vec3<R> scale3(const Vec3<R>& a, R s) { return {a.x * s, a.y * s, a.z * s}; }

// per-mode numerical constants: R/include/*/config.h:15-22
struct ModeConstants {
    int tile_w, tile_h;
    float min_alpha_rcp;      // bound cutoff uses 2*ln(opacity * this)
    float min_alpha;          // fragment rejection threshold
    float max_cutoff_sq;      // rho^2 rejection
    float min_alpha_core;     // HYBRID_BLEND only
};
constexpr float kTransmittanceThreshold = 1e-4f;
constexpr float kOneMinusAlphaEps = 1e-8f;

inline ModeConstants mode_constants(int mode) {
    switch (mode) {
        case 1: return {8, 8, 20.0f, 1.0f / 20.0f, 5.99146454711f, 0.0f};          // ALPHA_BLEND_FIRST_K
        case 2: return {16, 16, 255.0f, 1.0f / 255.0f, 11.0825270903f, 0.0f};      // ALPHA_BLEND_GLOBAL_ORDERING
        case 3: return {8, 8, 255.0f, 1.0f / 255.0f, 11.0825270903f, 0.0f};        // OIT_BLEND
        default: return {8, 8, 255.0f, 1.0f / 255.0f, 11.0825270903f, 1.0f / 20.0f}; // HYBRID_BLEND
    }
}

template <typename R> struct Camera {
    Vec4<R> M3;        // third row of the world->view matrix
    Vec4<R> VPM[4];    // rows of VP * M
    Vec3<R> cam;
};
template <typename R> Camera<R> load_camera(const float* M, const float* VPM, const float* cam) {
    Camera<R> c;
    c.M3 = {R(M[8]), R(M[9]), R(M[10]), R(M[11])};
    for (int r = 0; r < 4; ++r) c.VPM[r] = {R(VPM[4 * r]), R(VPM[4 * r + 1]), R(VPM[4 * r + 2]), R(VPM[4 * r + 3])};
    c.cam = {R(cam[0]), R(cam[1]), R(cam[2])};
    return c;
}

template <typename F> void parallel_for(int64_t n, int n_threads, F&& body) {
    if (n_threads <= 1 || n < 2) { for (int64_t i = 0; i < n; ++i) body(i); return; }
    std::atomic<int64_t> next{0};
    const int64_t chunk = std::max<int64_t>(1, n / (int64_t(n_threads) * 16));
    std::vector<std::thread> pool;
    for (int t = 0; t < n_threads; ++t)
        pool.emplace_back([&]() {
            for (;;) {
                const int64_t lo = next.fetch_add(chunk);
                if (lo >= n) break;
                const int64_t hi = std::min(n, lo + chunk);
                for (int64_t i = lo; i < hi; ++i) body(i);
            }
        });
    for (auto& th : pool) th.join();
}

// ----------------------------------------------------------------------------
// per-Gaussian preprocess
// ----------------------------------------------------------------------------
// transform_and_cull: R/include/kernel_utils.cuh:63-138 (quaternion 30-42)
// SH evaluation:      R/include/kernel_utils.cuh:140-188
// kernel body:        R/include/hybrid_blend/kernels/inference.cuh:10-76
//                     (GLOBAL_ORDERING stores the view depth z instead of MT3:
//                      R/include/alpha_blend_global_ordering/kernels/inference.cuh:61)
template <typename R> struct PreprocessOut {
    uint32_t* n_touched;   // [N]
    uint32_t* bounds;      // [N,4] x_min,x_max,y_min,y_max in tiles
    R* vpmt1;              // [N,4]
    R* vpmt2;              // [N,4]
    R* vpmt4;              // [N,4]
    R* mt3;                // [N,4]  (w = view depth z)
    R* rgba;               // [N,4]
    uint8_t* clamp;        // [3,N] or null: 1 where the channel was clamped at 0
};

template <typename R>
void preprocess_one(int64_t i, const float* positions, const float* scales, const float* rotations, const float* opacities,
                    const float* sh_0, const float* sh_rest, const Camera<R>& cam, const ModeConstants& mc,
                    int64_t n, int grid_w, int grid_h, int active_sh, int total_sh, R near_plane, R far_plane,
                    R scale_modifier, const PreprocessOut<R>& o) {
    o.n_touched[i] = 0;
    const Vec3<R> p = {R(positions[3 * i]), R(positions[3 * i + 1]), R(positions[3 * i + 2])};
    const R opacity = R(opacities[i]);
    const R z = dot3(xyz(cam.M3), p) + cam.M3.w;
    if (z < near_plane || z > far_plane) return;

    const Vec3<R> s = {R(scales[3 * i]), R(scales[3 * i + 1]), R(scales[3 * i + 2])};
    const R qr = R(rotations[4 * i]), qx = R(rotations[4 * i + 1]), qy = R(rotations[4 * i + 2]), qz = R(rotations[4 * i + 3]);
    const R xx = qx * qx, yy = qy * qy, zz = qz * qz, xy = qx * qy, xz = qx * qz, yz = qy * qz, rx = qr * qx, ry = qr * qy, rz = qr * qz;
    const R r11 = R(1) - R(2) * (yy + zz), r12 = R(2) * (xy - rz), r13 = R(2) * (xz + ry);
    const R r21 = R(2) * (xy + rz), r22 = R(1) - R(2) * (xx + zz), r23 = R(2) * (yz - rx);
    const R r31 = R(2) * (xz - ry), r32 = R(2) * (yz + rx), r33 = R(1) - R(2) * (xx + yy);
    const Vec3<R> u = scale3<R>({r11 * s.x, r21 * s.x, r31 * s.x}, scale_modifier);
    const Vec3<R> v = scale3<R>({r12 * s.y, r22 * s.y, r32 * s.y}, scale_modifier);
    const Vec3<R> w = scale3<R>({r13 * s.z, r23 * s.z, r33 * s.z}, scale_modifier);
    auto row_times_T = [&](const Vec4<R>& row) -> Vec4<R> {
        const Vec3<R> r3 = xyz(row);
        return {dot3(r3, u), dot3(r3, v), dot3(r3, w), dot3(r3, p) + row.w};
    };
    const Vec4<R> t4 = row_times_T(cam.VPM[3]);
    const R rho = R(2) * std::log(opacity * R(mc.min_alpha_rcp));
    const Vec4<R> dq = {rho, rho, rho, R(-1)};
    const R sden = dot4(dq, mul4(t4, t4));
    if (sden == R(0)) return;
    const R inv = R(1) / sden;
    const Vec4<R> f = {inv * dq.x, inv * dq.y, inv * dq.z, inv * dq.w};
    const Vec4<R> t3 = row_times_T(cam.VPM[2]);
    const R cz = dot4(f, mul4(t3, t4));
    const R ez = std::sqrt(std::max(cz * cz - dot4(f, mul4(t3, t3)), R(0)));
    if (cz - ez < R(-1) || cz + ez > R(1)) return;
    const Vec4<R> t1 = row_times_T(cam.VPM[0]);
    const R cx = dot4(f, mul4(t1, t4));
    const R ex = std::sqrt(std::max(cx * cx - dot4(f, mul4(t1, t1)), R(0)));
    const Vec4<R> t2 = row_times_T(cam.VPM[1]);
    const R cy = dot4(f, mul4(t2, t4));
    const R ey = std::sqrt(std::max(cy * cy - dot4(f, mul4(t2, t2)), R(0)));

    auto lo_tile = [](R v_, int tile, int grid) -> uint32_t {
        const R q = v_ / R(tile);
        const double fl = std::floor(double(q));
        const int64_t k = fl < -2147483648.0 ? INT32_MIN : (fl > 2147483647.0 ? INT32_MAX : int64_t(fl));
        return uint32_t(std::min<int64_t>(grid, std::max<int64_t>(0, k)));
    };
    auto hi_tile = [](R v_, int tile, int grid) -> uint32_t {
        const R q = v_ / R(tile);
        const double ce = std::ceil(double(q));
        const int64_t k = ce < -2147483648.0 ? INT32_MIN : (ce > 2147483647.0 ? INT32_MAX : int64_t(ce));
        return uint32_t(std::min<int64_t>(grid, std::max<int64_t>(0, k)));
    };
    const uint32_t x0 = lo_tile(cx - ex + R(0.5), mc.tile_w, grid_w), x1 = hi_tile(cx + ex + R(0.5), mc.tile_w, grid_w);
    const uint32_t y0 = lo_tile(cy - ey + R(0.5), mc.tile_h, grid_h), y1 = hi_tile(cy + ey + R(0.5), mc.tile_h, grid_h);
    // NaN extents: CUDA's float->int conversion of NaN gives 0 for both ends, i.e. an empty box
    const uint32_t count = (std::isnan(double(cx - ex)) || std::isnan(double(cy - ey))) ? 0u : (x1 - x0) * (y1 - y0);
    if (count == 0) return;

    o.n_touched[i] = count;
    o.bounds[4 * i] = x0; o.bounds[4 * i + 1] = x1; o.bounds[4 * i + 2] = y0; o.bounds[4 * i + 3] = y1;
    R* a = o.vpmt1 + 4 * i; a[0] = t1.x; a[1] = t1.y; a[2] = t1.z; a[3] = t1.w;
    a = o.vpmt2 + 4 * i; a[0] = t2.x; a[1] = t2.y; a[2] = t2.z; a[3] = t2.w;
    a = o.vpmt4 + 4 * i; a[0] = t4.x; a[1] = t4.y; a[2] = t4.z; a[3] = t4.w;
    const Vec3<R> m3 = xyz(cam.M3);
    a = o.mt3 + 4 * i; a[0] = dot3(m3, u); a[1] = dot3(m3, v); a[2] = dot3(m3, w); a[3] = z;

    // view-dependent colour
    R c[3];
    for (int ch = 0; ch < 3; ++ch) c[ch] = R(0.5) + R(0.28209479177387814f) * R(sh_0[3 * i + ch]);
    if (active_sh > 1) {
        const float* k = sh_rest + i * int64_t(total_sh) * 3;
        Vec3<R> dvec = {p.x - cam.cam.x, p.y - cam.cam.y, p.z - cam.cam.z};
        const R inv_len = R(1) / std::sqrt(dot3(dvec, dvec));
        const R x = dvec.x * inv_len, y = dvec.y * inv_len, zc = dvec.z * inv_len;
        R basis[15];
        int nb = 3;
        basis[0] = R(-0.48860251190291987f) * y;
        basis[1] = R(0.48860251190291987f) * zc;
        basis[2] = R(-0.48860251190291987f) * x;
        if (active_sh > 4) {
            const R x2 = x * x, y2 = y * y, z2 = zc * zc, xy_ = x * y, xz_ = x * zc, yz_ = y * zc;
            basis[3] = R(1.0925484305920792f) * xy_;
            basis[4] = R(-1.0925484305920792f) * yz_;
            basis[5] = R(0.94617469575755997f) * z2 - R(0.31539156525251999f);
            basis[6] = R(-1.0925484305920792f) * xz_;
            basis[7] = R(0.54627421529603959f) * x2 - R(0.54627421529603959f) * y2;
            nb = 8;
            if (active_sh > 9) {
                basis[8] = R(0.59004358992664352f) * y * (R(-3) * x2 + y2);
                basis[9] = R(2.8906114426405538f) * xy_ * zc;
                basis[10] = R(0.45704579946446572f) * y * (R(1) - R(5) * z2);
                basis[11] = R(0.3731763325901154f) * zc * (R(5) * z2 - R(3));
                basis[12] = R(0.45704579946446572f) * x * (R(1) - R(5) * z2);
                basis[13] = R(1.4453057213202769f) * zc * (x2 - y2);
                basis[14] = R(0.59004358992664352f) * x * (-x2 + R(3) * y2);
                nb = 15;
            }
        }
        // the reference adds the terms left to right: ((rgb + b0*k0) + b1*k1) + ...
        for (int ch = 0; ch < 3; ++ch) {
            R acc = c[ch];
            for (int b = 0; b < nb; ++b) acc = mul_add(basis[b], R(k[3 * b + ch]), acc);
            c[ch] = acc;
        }
    }
    if (o.clamp) for (int ch = 0; ch < 3; ++ch) o.clamp[ch * n + i] = c[ch] < R(0) ? 1 : 0;
    a = o.rgba + 4 * i;
    a[0] = std::max(R(0), c[0]); a[1] = std::max(R(0), c[1]); a[2] = std::max(R(0), c[2]); a[3] = opacity;
}

// ----------------------------------------------------------------------------
// per-fragment evaluation shared by all blend modes
// R/include/hybrid_blend/kernels/inference.cuh:137-155
// ----------------------------------------------------------------------------
template <typename R> struct Fragment {
    R rho2_num, denom, denom_rcp, G, alpha, depth;
    Vec3<R> m, d;
    Vec4<R> plane_x, plane_y;
};

template <typename R>
inline void fragment_planes(const R* t1, const R* t2, const R* t4, R px, R py, Fragment<R>& fr) {
    fr.plane_x = {t1[0] - t4[0] * px, t1[1] - t4[1] * px, t1[2] - t4[2] * px, t1[3] - t4[3] * px};
    fr.plane_y = {t2[0] - t4[0] * py, t2[1] - t4[1] * py, t2[2] - t4[2] * py, t2[3] - t4[3] * py};
    const Vec3<R> nx = xyz(fr.plane_x), ny = xyz(fr.plane_y);
    fr.m = {fr.plane_x.w * ny.x - nx.x * fr.plane_y.w, fr.plane_x.w * ny.y - nx.y * fr.plane_y.w, fr.plane_x.w * ny.z - nx.z * fr.plane_y.w};
    fr.d = cross3(nx, ny);
    fr.rho2_num = dot3(fr.m, fr.m);
    fr.denom = dot3(fr.d, fr.d);
}
template <typename R> inline R fragment_depth(const R* mt3, const Fragment<R>& fr) {
    const Vec3<R> e = scale3(cross3(fr.d, fr.m), fr.denom_rcp);
    return dot3<R>({mt3[0], mt3[1], mt3[2]}, e) + mt3[3];
}

template <typename R> struct BlendIn {
    const uint32_t* ranges;    // [n_tiles,2]
    const uint32_t* prim_idx;  // sorted instance -> primitive
    const R *vpmt1, *vpmt2, *vpmt4, *mt3, *rgba;
    int width, height, grid_w, grid_h;
    int K;
    bool use_median_depth;
};

// HYBRID_BLEND inference: R/include/hybrid_blend/kernels/inference.cuh:78-216
template <typename R>
void blend_hybrid_pixel(const BlendIn<R>& in, const ModeConstants& mc, int tile, int px_i, int py_i, R* rgb_out, R* depth_out, R* alpha_out) {
    const int K = in.K;
    std::vector<Vec4<R>> core(K, Vec4<R>{0, 0, 0, 0});
    std::vector<R> core_depth(K, R(FLT_MAX));
    R t_tail = 1; Vec4<R> tail = {0, 0, 0, 0}; R tail_depth = 0;
    const R px = R(px_i), py = R(py_i);
    for (uint32_t it = in.ranges[2 * tile]; it < in.ranges[2 * tile + 1]; ++it) {
        const int64_t g = in.prim_idx[it];
        Fragment<R> fr;
        fragment_planes(in.vpmt1 + 4 * g, in.vpmt2 + 4 * g, in.vpmt4 + 4 * g, px, py, fr);
        if (fr.rho2_num > R(mc.max_cutoff_sq) * fr.denom) continue;
        fr.denom_rcp = R(1) / fr.denom;
        fr.G = std::exp(R(-0.5) * fr.rho2_num * fr.denom_rcp);
        fr.alpha = std::min(in.rgba[4 * g + 3] * fr.G, R(1));
        if (fr.alpha < R(mc.min_alpha)) continue;
        R depth = fragment_depth(in.mt3 + 4 * g, fr);
        Vec4<R> frag = {in.rgba[4 * g] * fr.alpha, in.rgba[4 * g + 1] * fr.alpha, in.rgba[4 * g + 2] * fr.alpha, fr.alpha};
        if (depth < core_depth[K - 1] && fr.alpha >= R(mc.min_alpha_core)) {
            for (int k = 0; k < K; ++k)
                if (depth < core_depth[k]) { std::swap(depth, core_depth[k]); std::swap(frag, core[k]); }
        }
        tail.x += frag.x; tail.y += frag.y; tail.z += frag.z; tail.w += frag.w;
        if (!in.use_median_depth) tail_depth += depth * frag.w;
        t_tail *= R(1) - frag.w;
    }
    R rgb[3] = {0, 0, 0}; R dpx = 0; R t_core = 1;
    for (int k = 0; k < K && t_core >= R(kTransmittanceThreshold); ++k) {
        rgb[0] += t_core * core[k].x; rgb[1] += t_core * core[k].y; rgb[2] += t_core * core[k].z;
        if (in.use_median_depth) dpx = (t_core > R(0.5) && core_depth[k] < R(FLT_MAX)) ? core_depth[k] : dpx;
        else dpx += t_core * core[k].w * core_depth[k];
        t_core *= R(1) - core[k].w;
    }
    R total_alpha = R(1) - t_core;
    if (t_core >= R(kTransmittanceThreshold) && tail.w >= R(mc.min_alpha)) {
        const R wt = t_core * (R(1) - t_tail);
        const R rcp = R(1) / tail.w;
        rgb[0] += wt * rcp * tail.x; rgb[1] += wt * rcp * tail.y; rgb[2] += wt * rcp * tail.z;
        if (!in.use_median_depth) dpx += wt * rcp * tail_depth;
        total_alpha += wt;
    }
    if (!in.use_median_depth) dpx = total_alpha > R(0) ? dpx / total_alpha : R(0);
    for (int c = 0; c < 3; ++c) rgb_out[c] = std::min(std::max(rgb[c], R(0)), R(1));
    *depth_out = dpx;
    *alpha_out = total_alpha;   // not an output of the reference; same quantity it uses to normalise mean depth (188-199)
}

// ALPHA_BLEND_FIRST_K inference: R/include/alpha_blend_first_k/kernels/inference.cuh:79-208
template <typename R>
void blend_first_k_pixel(const BlendIn<R>& in, const ModeConstants& mc, int tile, int px_i, int py_i, R* rgb_out, R* depth_out, R* alpha_out) {
    const int K = in.K;
    std::vector<R> core_alpha(K, R(0)), core_depth(K, R(FLT_MAX));
    std::vector<uint32_t> core_idx(K, UINT32_MAX);
    const R px = R(px_i), py = R(py_i);
    for (uint32_t it = in.ranges[2 * tile]; it < in.ranges[2 * tile + 1]; ++it) {
        const int64_t g = in.prim_idx[it];
        Fragment<R> fr;
        fragment_planes(in.vpmt1 + 4 * g, in.vpmt2 + 4 * g, in.vpmt4 + 4 * g, px, py, fr);
        if (fr.rho2_num > R(mc.max_cutoff_sq) * fr.denom) continue;
        fr.denom_rcp = R(1) / fr.denom;
        R depth = fragment_depth(in.mt3 + 4 * g, fr);
        if (depth >= core_depth[K - 1]) continue;
        fr.G = std::exp(R(-0.5) * fr.rho2_num * fr.denom_rcp);
        R alpha = std::min(in.rgba[4 * g + 3] * fr.G, R(1));
        if (alpha < R(mc.min_alpha)) continue;
        uint32_t idx = uint32_t(g);
        for (int k = 0; k < K; ++k)
            if (depth < core_depth[k]) { std::swap(depth, core_depth[k]); std::swap(alpha, core_alpha[k]); std::swap(idx, core_idx[k]); }
    }
    R rgb[3] = {0, 0, 0}; R dpx = 0; R t = 1;
    for (int k = 0; k < K && t >= R(kTransmittanceThreshold); ++k) {
        if (core_idx[k] == UINT32_MAX) break;
        const R wgt = t * core_alpha[k];
        const R* c = in.rgba + 4 * int64_t(core_idx[k]);
        rgb[0] += wgt * c[0]; rgb[1] += wgt * c[1]; rgb[2] += wgt * c[2];
        if (in.use_median_depth) dpx = t > R(0.5) ? core_depth[k] : dpx; else dpx += wgt * core_depth[k];
        t *= R(1) - core_alpha[k];
    }
    if (!in.use_median_depth) dpx = t < R(1) ? dpx / (R(1) - t) : R(0);
    for (int c = 0; c < 3; ++c) rgb_out[c] = std::min(std::max(rgb[c], R(0)), R(1));
    *depth_out = dpx; *alpha_out = R(1) - t;
}

// ALPHA_BLEND_GLOBAL_ORDERING inference: R/include/alpha_blend_global_ordering/kernels/inference.cuh:78-176
// (mt3[3] holds the per-Gaussian view depth z)
template <typename R>
void blend_global_pixel(const BlendIn<R>& in, const ModeConstants& mc, int tile, int px_i, int py_i, R* rgb_out, R* depth_out, R* alpha_out) {
    R rgb[3] = {0, 0, 0}; R dpx = 0; R t = 1;
    const R px = R(px_i), py = R(py_i);
    for (uint32_t it = in.ranges[2 * tile]; it < in.ranges[2 * tile + 1]; ++it) {
        const int64_t g = in.prim_idx[it];
        Fragment<R> fr;
        fragment_planes(in.vpmt1 + 4 * g, in.vpmt2 + 4 * g, in.vpmt4 + 4 * g, px, py, fr);
        if (fr.rho2_num > R(mc.max_cutoff_sq) * fr.denom) continue;
        fr.denom_rcp = R(1) / fr.denom;
        fr.G = std::exp(R(-0.5) * fr.rho2_num * fr.denom_rcp);
        const R alpha = std::min(in.rgba[4 * g + 3] * fr.G, R(1));
        if (alpha < R(mc.min_alpha)) continue;
        const R wgt = t * alpha;
        rgb[0] += wgt * in.rgba[4 * g]; rgb[1] += wgt * in.rgba[4 * g + 1]; rgb[2] += wgt * in.rgba[4 * g + 2];
        const R depth = in.mt3[4 * g + 3];
        if (in.use_median_depth) dpx = t > R(0.5) ? depth : dpx; else dpx += wgt * depth;
        t *= R(1) - alpha;
        if (t < R(kTransmittanceThreshold)) break;
    }
    if (!in.use_median_depth) dpx = t < R(1) ? dpx / (R(1) - t) : R(0);
    for (int c = 0; c < 3; ++c) rgb_out[c] = std::min(std::max(rgb[c], R(0)), R(1));
    *depth_out = dpx; *alpha_out = R(1) - t;
}

// OIT_BLEND inference: R/include/oit_blend/kernels/inference.cuh:78-177
template <typename R>
void blend_oit_pixel(const BlendIn<R>& in, const ModeConstants& mc, int tile, int px_i, int py_i, R* rgb_out, R* depth_out, R* alpha_out) {
    R acc[4] = {0, 0, 0, 0}; R alpha_sum = 0; R t = 1;
    const R px = R(px_i), py = R(py_i);
    for (uint32_t it = in.ranges[2 * tile]; it < in.ranges[2 * tile + 1]; ++it) {
        const int64_t g = in.prim_idx[it];
        Fragment<R> fr;
        fragment_planes(in.vpmt1 + 4 * g, in.vpmt2 + 4 * g, in.vpmt4 + 4 * g, px, py, fr);
        if (fr.rho2_num > R(mc.max_cutoff_sq) * fr.denom) continue;
        fr.denom_rcp = R(1) / fr.denom;
        fr.G = std::exp(R(-0.5) * fr.rho2_num * fr.denom_rcp);
        const R alpha = std::min(in.rgba[4 * g + 3] * fr.G, R(1));
        if (alpha < R(mc.min_alpha)) continue;
        const R depth = fragment_depth(in.mt3 + 4 * g, fr);
        acc[0] += alpha * in.rgba[4 * g]; acc[1] += alpha * in.rgba[4 * g + 1]; acc[2] += alpha * in.rgba[4 * g + 2]; acc[3] += alpha * depth;
        alpha_sum += alpha;
        t *= R(1) - alpha;
    }
    R out[4] = {0, 0, 0, 0}; R a = 0;
    if (alpha_sum >= R(mc.min_alpha)) {
        a = R(1) - t;
        const R s = a * (R(1) / alpha_sum);
        for (int c = 0; c < 4; ++c) out[c] = s * acc[c];
        out[3] = out[3] / a;
    }
    for (int c = 0; c < 3; ++c) rgb_out[c] = std::min(std::max(out[c], R(0)), R(1));
    *depth_out = out[3]; *alpha_out = a;
}

template <typename R>
void blend_image(int mode, const BlendIn<R>& in, R* image, R* depth, R* alpha, bool to_chw, int n_threads) {
    const ModeConstants mc = mode_constants(mode);
    const int n_tiles = in.grid_w * in.grid_h;
    const int64_t n_pixels = int64_t(in.width) * in.height;
    parallel_for(n_tiles, n_threads, [&](int64_t tile) {
        const int tx = int(tile % in.grid_w), ty = int(tile / in.grid_w);
        for (int ly = 0; ly < mc.tile_h; ++ly)
            for (int lx = 0; lx < mc.tile_w; ++lx) {
                const int px = tx * mc.tile_w + lx, py = ty * mc.tile_h + ly;
                if (px >= in.width || py >= in.height) continue;
                R rgb[3], d, a;
                switch (mode) {
                    case 1: blend_first_k_pixel(in, mc, int(tile), px, py, rgb, &d, &a); break;
                    case 2: blend_global_pixel(in, mc, int(tile), px, py, rgb, &d, &a); break;
                    case 3: blend_oit_pixel(in, mc, int(tile), px, py, rgb, &d, &a); break;
                    default: blend_hybrid_pixel(in, mc, int(tile), px, py, rgb, &d, &a); break;
                }
                const int64_t pix = int64_t(py) * in.width + px;
                if (to_chw) { image[pix] = rgb[0]; image[n_pixels + pix] = rgb[1]; image[2 * n_pixels + pix] = rgb[2]; }
                else { image[3 * pix] = rgb[0]; image[3 * pix + 1] = rgb[1]; image[3 * pix + 2] = rgb[2]; }
                depth[pix] = d;
                if (alpha) alpha[pix] = a;
            }
    });
}


// ----------------------------------------------------------------------------
// binning: instance emission, stable sort, per-tile ranges
// ----------------------------------------------------------------------------
// emission order and keys: R/src/shared_kernels.cu:7-54
// key width / sorted bit range: R/src/hybrid_blend/inference.cu:61-64,121-129,145-152
//                               R/src/alpha_blend_global_ordering/inference.cu (end_bit + 32)
// ranges: R/src/shared_kernels.cu:56-95 (tiles without instances keep the memset value 0,0)
struct Binning {
    std::vector<uint64_t> keys;        // emission order
    std::vector<uint32_t> prims;       // emission order
    std::vector<uint64_t> sorted_keys;
    std::vector<uint32_t> sorted_prims;
    std::vector<uint32_t> ranges;      // [n_tiles,2]
};

int bit_length(uint32_t v) { int b = 0; while (v) { ++b; v >>= 1; } return b; }   // R/include/rasterization_utils.h:3-13

void bin_instances(const uint32_t* n_touched, const uint32_t* bounds, const float* depth_or_null, int64_t n,
                   int grid_w, int n_tiles, Binning& out) {
    int64_t total = 0;
    for (int64_t i = 0; i < n; ++i) total += n_touched[i];
    out.keys.resize(total); out.prims.resize(total);
    int64_t at = 0;
    for (int64_t i = 0; i < n; ++i) {
        if (n_touched[i] == 0) continue;
        uint64_t depth_bits = 0;
        if (depth_or_null) { uint32_t b; std::memcpy(&b, depth_or_null + i, 4); depth_bits = b; }
        for (uint32_t y = bounds[4 * i + 2]; y < bounds[4 * i + 3]; ++y)
            for (uint32_t x = bounds[4 * i]; x < bounds[4 * i + 1]; ++x) {
                const uint64_t tile = uint64_t(y) * grid_w + x;
                out.keys[at] = depth_or_null ? ((tile << 32) | depth_bits) : tile;
                out.prims[at] = uint32_t(i);
                ++at;
            }
    }
    out.sorted_keys.resize(total); out.sorted_prims.resize(total);
    if (!depth_or_null) {
        // stable counting sort by tile index
        std::vector<int64_t> start(size_t(n_tiles) + 1, 0);
        for (int64_t j = 0; j < total; ++j) ++start[out.keys[j] + 1];
        for (int t = 0; t < n_tiles; ++t) start[t + 1] += start[t];
        for (int64_t j = 0; j < total; ++j) { const int64_t d = start[out.keys[j]]++; out.sorted_keys[d] = out.keys[j]; out.sorted_prims[d] = out.prims[j]; }
    } else {
        std::vector<int64_t> order(total);
        for (int64_t j = 0; j < total; ++j) order[j] = j;
        const int end_bit = bit_length(uint32_t(n_tiles - 1)) + 32;
        const uint64_t mask = end_bit >= 64 ? ~uint64_t(0) : ((uint64_t(1) << end_bit) - 1);
        std::stable_sort(order.begin(), order.end(), [&](int64_t a, int64_t b) { return (out.keys[a] & mask) < (out.keys[b] & mask); });
        for (int64_t j = 0; j < total; ++j) { out.sorted_keys[j] = out.keys[order[j]]; out.sorted_prims[j] = out.prims[order[j]]; }
    }
    out.ranges.assign(size_t(n_tiles) * 2, 0);
    for (int64_t j = 0; j < total; ++j) {
        const uint64_t tile = depth_or_null ? (out.sorted_keys[j] >> 32) : out.sorted_keys[j];
        if (j == 0) out.ranges[2 * tile] = 0;
        else {
            const uint64_t prev = depth_or_null ? (out.sorted_keys[j - 1] >> 32) : out.sorted_keys[j - 1];
            if (prev != tile) { out.ranges[2 * prev + 1] = uint32_t(j); out.ranges[2 * tile] = uint32_t(j); }
        }
        if (j == total - 1) out.ranges[2 * tile + 1] = uint32_t(total);
    }
}

template <typename R>
void run_preprocess(const float* positions, const float* scales, const float* rotations, const float* opacities,
                    const float* sh_0, const float* sh_rest, const float* M, const float* VPM, const float* cam_position,
                    int64_t n, int mode, int active_sh, int total_sh, int width, int height, float near_plane, float far_plane,
                    float scale_modifier, const PreprocessOut<R>& out, int n_threads) {
    const ModeConstants mc = mode_constants(mode);
    const Camera<R> cam = load_camera<R>(M, VPM, cam_position);
    const int grid_w = (width + mc.tile_w - 1) / mc.tile_w, grid_h = (height + mc.tile_h - 1) / mc.tile_h;
    parallel_for(n, n_threads, [&](int64_t i) {
        preprocess_one<R>(i, positions, scales, rotations, opacities, sh_0, sh_rest, cam, mc, n, grid_w, grid_h, active_sh,
                          total_sh, R(near_plane), R(far_plane), R(scale_modifier), out);
    });
}

template <typename R>
int64_t run_render(const float* positions, const float* scales, const float* rotations, const float* opacities,
                   const float* sh_0, const float* sh_rest, const float* M, const float* VPM, const float* cam_position,
                   int64_t n, int mode, int K, int active_sh, int total_sh, int width, int height, float near_plane,
                   float far_plane, float scale_modifier, int to_chw, int use_median_depth, R* image, R* depth, R* alpha,
                   int n_threads) {
    const ModeConstants mc = mode_constants(mode);
    const int grid_w = (width + mc.tile_w - 1) / mc.tile_w, grid_h = (height + mc.tile_h - 1) / mc.tile_h;
    std::vector<uint32_t> n_touched(n), bounds(size_t(n) * 4);
    std::vector<R> t1(size_t(n) * 4), t2(size_t(n) * 4), t4(size_t(n) * 4), mt3(size_t(n) * 4), rgba(size_t(n) * 4);
    PreprocessOut<R> po{n_touched.data(), bounds.data(), t1.data(), t2.data(), t4.data(), mt3.data(), rgba.data(), nullptr};
    run_preprocess<R>(positions, scales, rotations, opacities, sh_0, sh_rest, M, VPM, cam_position, n, mode, active_sh, total_sh,
                      width, height, near_plane, far_plane, scale_modifier, po, n_threads);
    std::vector<float> zf;
    if (mode == 2) { zf.resize(n); for (int64_t i = 0; i < n; ++i) zf[i] = n_touched[i] ? float(mt3[4 * i + 3]) : 0.0f; }
    Binning bin;
    bin_instances(n_touched.data(), bounds.data(), mode == 2 ? zf.data() : nullptr, n, grid_w, grid_w * grid_h, bin);
    BlendIn<R> in{bin.ranges.data(), bin.sorted_prims.data(), t1.data(), t2.data(), t4.data(), mt3.data(), rgba.data(),
                  width, height, grid_w, grid_h, K, use_median_depth != 0};
    blend_image<R>(mode, in, image, depth, alpha, to_chw != 0, n_threads);
    return int64_t(bin.sorted_prims.size());
}

// ----------------------------------------------------------------------------
// update_max_weights: per-Gaussian maximum blending weight over the pixels of a view
// R/include/hybrid_blend/kernels/update_max_weights.cuh:59-212 (core weights, then a second pass over the
// tile's list that credits alpha * tail_weight to every fragment inside the cutoff),
// first_k :60-, global_ordering :59-, oit :57- analogues.  Sequential over tiles (small cases only).
// `hybrid_tail_credit` = false restates what the reference EXTENSION computes for HYBRID_BLEND: its link keeps
// alpha_blend_first_k's copy of the dispatcher template both modes define (R/src/hybrid_blend/update_max_weights.cu:15-28,
// R/src/alpha_blend_first_k/update_max_weights.cu:15-28), so HYBRID's lists are walked by FIRST_K's kernel, which keeps
// the K nearest fragments with alpha >= 1/20 and has no second pass: HYBRID's core weights and nothing else.
// ----------------------------------------------------------------------------
template <typename R>
void max_weights_image(int mode, const BlendIn<R>& in, R weight_threshold, R* max_weights, bool hybrid_tail_credit) {
    const ModeConstants mc = mode_constants(mode);
    const int K = in.K;
    auto raise = [&](int64_t g, R w) { if (max_weights[g] < w) max_weights[g] = w; };
    for (int tile = 0; tile < in.grid_w * in.grid_h; ++tile) {
        const int tx = tile % in.grid_w, ty = tile / in.grid_w;
        for (int ly = 0; ly < mc.tile_h; ++ly)
            for (int lx = 0; lx < mc.tile_w; ++lx) {
                const int pxi = tx * mc.tile_w + lx, pyi = ty * mc.tile_h + ly;
                if (pxi >= in.width || pyi >= in.height) continue;
                const R px = R(pxi), py = R(pyi);
                std::vector<R> ka(K, R(0)), kd(K, R(FLT_MAX));
                std::vector<uint32_t> ki(K, UINT32_MAX);
                R alpha_sum = 0, t = 1;
                bool done = false;
                for (uint32_t it = in.ranges[2 * tile]; it < in.ranges[2 * tile + 1] && !done; ++it) {
                    const int64_t g = in.prim_idx[it];
                    Fragment<R> fr;
                    fragment_planes(in.vpmt1 + 4 * g, in.vpmt2 + 4 * g, in.vpmt4 + 4 * g, px, py, fr);
                    if (fr.rho2_num > R(mc.max_cutoff_sq) * fr.denom) continue;
                    fr.denom_rcp = R(1) / fr.denom;
                    R depth = 0;
                    if (mode == 1) { depth = fragment_depth(in.mt3 + 4 * g, fr); if (depth >= kd[K - 1]) continue; }
                    R alpha = std::min(in.rgba[4 * g + 3] * std::exp(R(-0.5) * fr.rho2_num * fr.denom_rcp), R(1));
                    if (alpha < R(mc.min_alpha)) continue;
                    if (mode == 2) {
                        const R w = t * alpha;
                        t *= R(1) - alpha;
                        if (t < R(kTransmittanceThreshold)) done = true;
                        if (!(w < weight_threshold)) raise(g, w);
                        continue;
                    }
                    if (mode == 0) depth = fragment_depth(in.mt3 + 4 * g, fr);
                    if (mode == 1 || (mode == 0 && depth < kd[K - 1] && alpha >= R(mc.min_alpha_core))) {
                        uint32_t idx = uint32_t(g);
                        for (int k = 0; k < K; ++k)
                            if (depth < kd[k]) { std::swap(depth, kd[k]); std::swap(alpha, ka[k]); std::swap(idx, ki[k]); }
                    }
                    if (mode != 1) { alpha_sum += alpha; t *= R(1) - alpha; }
                }
                if (mode == 2) continue;
                R second = 0;
                if (mode == 0 || mode == 1) {
                    R tc = 1;
                    for (int k = 0; k < K; ++k) {
                        const R w = tc * ka[k];
                        tc *= R(1) - ka[k];
                        if (tc < R(kTransmittanceThreshold)) tc = 0;
                        if (w < weight_threshold || ki[k] == UINT32_MAX) continue;
                        raise(ki[k], w);
                    }
                    if (mode == 0 && hybrid_tail_credit && alpha_sum >= weight_threshold) second = tc * (R(1) - t) * (R(1) / alpha_sum);
                } else if (alpha_sum >= weight_threshold) {
                    second = (R(1) - t) * (R(1) / alpha_sum);
                }
                if (mode == 1 || !(second >= weight_threshold)) continue;
                for (uint32_t it = in.ranges[2 * tile]; it < in.ranges[2 * tile + 1]; ++it) {
                    const int64_t g = in.prim_idx[it];
                    Fragment<R> fr;
                    fragment_planes(in.vpmt1 + 4 * g, in.vpmt2 + 4 * g, in.vpmt4 + 4 * g, px, py, fr);
                    if (fr.rho2_num > R(mc.max_cutoff_sq) * fr.denom) continue;
                    const R alpha = std::min(in.rgba[4 * g + 3] * std::exp(R(-0.5) * fr.rho2_num * (R(1) / fr.denom)), R(1));
                    const R w = alpha * second;
                    if (w < weight_threshold) continue;
                    raise(g, w);
                }
            }
    }
}

}  // namespace

// ----------------------------------------------------------------------------
// C entry points (loaded with ctypes by oracle/oracle.py)
// ----------------------------------------------------------------------------
#define SCENE_ARGS const float *positions, const float *scales, const float *rotations, const float *opacities, \
                   const float *sh_0, const float *sh_rest, const float *M, const float *VPM, const float *cam_position
#define SCENE_PASS positions, scales, rotations, opacities, sh_0, sh_rest, M, VPM, cam_position

extern "C" {

int htgs_oracle_hardware_threads() { return int(std::thread::hardware_concurrency()); }

void htgs_oracle_tile_size(int mode, int* tile_w, int* tile_h) { const ModeConstants mc = mode_constants(mode); *tile_w = mc.tile_w; *tile_h = mc.tile_h; }

void htgs_oracle_preprocess_f32(SCENE_ARGS, int64_t n, int mode, int active_sh, int total_sh, int width, int height, float near_plane,
                                float far_plane, float scale_modifier, uint32_t* n_touched, uint32_t* bounds, float* vpmt1, float* vpmt2,
                                float* vpmt4, float* mt3, float* rgba, uint8_t* clamp, int n_threads) {
    PreprocessOut<float> po{n_touched, bounds, vpmt1, vpmt2, vpmt4, mt3, rgba, clamp};
    run_preprocess<float>(SCENE_PASS, n, mode, active_sh, total_sh, width, height, near_plane, far_plane, scale_modifier, po, n_threads);
}
void htgs_oracle_preprocess_f64(SCENE_ARGS, int64_t n, int mode, int active_sh, int total_sh, int width, int height, float near_plane,
                                float far_plane, float scale_modifier, uint32_t* n_touched, uint32_t* bounds, double* vpmt1, double* vpmt2,
                                double* vpmt4, double* mt3, double* rgba, uint8_t* clamp, int n_threads) {
    PreprocessOut<double> po{n_touched, bounds, vpmt1, vpmt2, vpmt4, mt3, rgba, clamp};
    run_preprocess<double>(SCENE_PASS, n, mode, active_sh, total_sh, width, height, near_plane, far_plane, scale_modifier, po, n_threads);
}

// Emission + stable sort + ranges from given per-Gaussian tile boxes.  `depth` is null except for
// ALPHA_BLEND_GLOBAL_ORDERING.  Call once with null outputs to learn the instance count.
int64_t htgs_oracle_bin(const uint32_t* n_touched, const uint32_t* bounds, const float* depth, int64_t n, int grid_w, int n_tiles,
                        uint64_t* keys, uint32_t* prims, uint64_t* sorted_keys, uint32_t* sorted_prims, uint32_t* ranges) {
    if (!sorted_prims) { int64_t total = 0; for (int64_t i = 0; i < n; ++i) total += n_touched[i]; return total; }
    Binning bin;
    bin_instances(n_touched, bounds, depth, n, grid_w, n_tiles, bin);
    const size_t t = bin.keys.size();
    if (keys) std::memcpy(keys, bin.keys.data(), t * 8);
    if (prims) std::memcpy(prims, bin.prims.data(), t * 4);
    if (sorted_keys) std::memcpy(sorted_keys, bin.sorted_keys.data(), t * 8);
    std::memcpy(sorted_prims, bin.sorted_prims.data(), t * 4);
    if (ranges) std::memcpy(ranges, bin.ranges.data(), size_t(n_tiles) * 8);
    return int64_t(t);
}

void htgs_oracle_blend_f32(int mode, const uint32_t* ranges, const uint32_t* prim_idx, const float* vpmt1, const float* vpmt2, const float* vpmt4,
                           const float* mt3, const float* rgba, int width, int height, int K, int use_median_depth, int to_chw, float* image,
                           float* depth, float* alpha, int n_threads) {
    const ModeConstants mc = mode_constants(mode);
    BlendIn<float> in{ranges, prim_idx, vpmt1, vpmt2, vpmt4, mt3, rgba, width, height, (width + mc.tile_w - 1) / mc.tile_w,
                      (height + mc.tile_h - 1) / mc.tile_h, K, use_median_depth != 0};
    blend_image<float>(mode, in, image, depth, alpha, to_chw != 0, n_threads);
}
void htgs_oracle_blend_f64(int mode, const uint32_t* ranges, const uint32_t* prim_idx, const double* vpmt1, const double* vpmt2, const double* vpmt4,
                           const double* mt3, const double* rgba, int width, int height, int K, int use_median_depth, int to_chw, double* image,
                           double* depth, double* alpha, int n_threads) {
    const ModeConstants mc = mode_constants(mode);
    BlendIn<double> in{ranges, prim_idx, vpmt1, vpmt2, vpmt4, mt3, rgba, width, height, (width + mc.tile_w - 1) / mc.tile_w,
                       (height + mc.tile_h - 1) / mc.tile_h, K, use_median_depth != 0};
    blend_image<double>(mode, in, image, depth, alpha, to_chw != 0, n_threads);
}

void htgs_oracle_max_weights_f32(int mode, const uint32_t* ranges, const uint32_t* prim_idx, const float* vpmt1, const float* vpmt2, const float* vpmt4,
                                 const float* mt3, const float* rgba, int width, int height, int K, float weight_threshold, float* max_weights, int hybrid_tail_credit) {
    const ModeConstants mc = mode_constants(mode);
    BlendIn<float> in{ranges, prim_idx, vpmt1, vpmt2, vpmt4, mt3, rgba, width, height, (width + mc.tile_w - 1) / mc.tile_w,
                      (height + mc.tile_h - 1) / mc.tile_h, K, false};
    max_weights_image<float>(mode, in, weight_threshold, max_weights, hybrid_tail_credit != 0);
}
void htgs_oracle_max_weights_f64(int mode, const uint32_t* ranges, const uint32_t* prim_idx, const double* vpmt1, const double* vpmt2, const double* vpmt4,
                                 const double* mt3, const double* rgba, int width, int height, int K, double weight_threshold, double* max_weights, int hybrid_tail_credit) {
    const ModeConstants mc = mode_constants(mode);
    BlendIn<double> in{ranges, prim_idx, vpmt1, vpmt2, vpmt4, mt3, rgba, width, height, (width + mc.tile_w - 1) / mc.tile_w,
                       (height + mc.tile_h - 1) / mc.tile_h, K, false};
    max_weights_image<double>(mode, in, weight_threshold, max_weights, hybrid_tail_credit != 0);
}

// whole forward (preprocess -> bin -> blend); returns the instance count
int64_t htgs_oracle_render_f32(SCENE_ARGS, int64_t n, int mode, int K, int active_sh, int total_sh, int width, int height, float near_plane,
                               float far_plane, float scale_modifier, int to_chw, int use_median_depth, float* image, float* depth, float* alpha,
                               int n_threads) {
    return run_render<float>(SCENE_PASS, n, mode, K, active_sh, total_sh, width, height, near_plane, far_plane, scale_modifier, to_chw,
                             use_median_depth, image, depth, alpha, n_threads);
}
int64_t htgs_oracle_render_f64(SCENE_ARGS, int64_t n, int mode, int K, int active_sh, int total_sh, int width, int height, float near_plane,
                               float far_plane, float scale_modifier, int to_chw, int use_median_depth, double* image, double* depth, double* alpha,
                               int n_threads) {
    return run_render<double>(SCENE_PASS, n, mode, K, active_sh, total_sh, width, height, near_plane, far_plane, scale_modifier, to_chw,
                              use_median_depth, image, depth, alpha, n_threads);
}

}  // extern "C"
