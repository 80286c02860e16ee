// Packing of per-Gaussian rows for the multi-GPU gradient exchange.  No counterpart in the reference (it is single-GPU).
//
// A training view keeps about a sixth of a scene's Gaussians and its backward pass leaves every other row of the six
// gradient tensors zero, so the ranks only have to sum the rows of Gaussians SOME rank kept.  htgs_gather_rows copies
// those rows of up to 8 row-major float tensors (widths 3, 3, 4, 1, 3, 3 B for the rasterizer's inputs) into one dense
// [count, sum of widths] buffer, which one all-reduce sums; htgs_scatter_rows writes the sums back.  Both are pure
// streaming kernels (one warp per row, lanes on consecutive floats of the packed row): the packed side is fully
// coalesced, the tensor side moves whole rows of 4 to 540 bytes.
#include "kernels.h"

#include <cstring>


namespace htgs {

namespace {

constexpr int kRowBlock = 256;

struct RowTable {
    float* ptr[HTGS_MAX_ROW_TENSORS];
    int32_t width[HTGS_MAX_ROW_TENSORS];
    int32_t begin[HTGS_MAX_ROW_TENSORS + 1];   // first packed column of tensor k; begin[n_tensors] = packed row width
    int32_t n_tensors;
};

// One warp per kRowsPerTrip rows and trip: the lanes walk the packed rows' columns (no division, the row indices are read
// once per warp), so a warp's accesses are one contiguous run in the packed buffer and one contiguous run per tensor, and
// every lane has kRowsPerTrip independent loads in flight before its first store.
constexpr int kRowsPerTrip = 8;
template <bool GATHER>
__global__ void __launch_bounds__(kRowBlock) move_rows_kernel(const __grid_constant__ RowTable table, const int64_t* __restrict__ index,
                                                              uint32_t count, float* __restrict__ packed) {
    const uint32_t row_width = uint32_t(table.begin[table.n_tensors]);
    const uint32_t lane = threadIdx.x & 31u;
    const uint32_t warps = gridDim.x * (kRowBlock / 32);
    for (uint32_t r0 = (blockIdx.x * (kRowBlock / 32) + (threadIdx.x >> 5)) * kRowsPerTrip; r0 < count; r0 += warps * kRowsPerTrip) {
        size_t row[kRowsPerTrip];
        #pragma unroll
        for (int i = 0; i < kRowsPerTrip; ++i) row[i] = r0 + i < count ? size_t(__ldg(index + r0 + i)) : size_t(0);
        for (uint32_t c = lane; c < row_width; c += 32) {
            int k = 0;
            #pragma unroll
            for (int t = 1; t < HTGS_MAX_ROW_TENSORS; ++t) k += (t < table.n_tensors && c >= uint32_t(table.begin[t])) ? 1 : 0;
            float* column = table.ptr[k] + (c - uint32_t(table.begin[k]));
            const size_t width = size_t(table.width[k]);
            float v[kRowsPerTrip];
            #pragma unroll
            for (int i = 0; i < kRowsPerTrip; ++i)
                if (r0 + i < count) v[i] = GATHER ? column[row[i] * width] : packed[size_t(r0 + i) * row_width + c];
            #pragma unroll
            for (int i = 0; i < kRowsPerTrip; ++i)
                if (r0 + i < count) {
                    if (GATHER) packed[size_t(r0 + i) * row_width + c] = v[i];
                    else column[row[i] * width] = v[i];
                }
        }
    }
}

int exchange_fail(int code, const char* message) { htgs::set_last_error(message); return code; }

// Compact rows -> dense gradients: rebuilds the rows of grad_sh_0 / grad_sh_rest from the colour gradient and the view
// direction (position of the Gaussian minus the camera position in the buffer's header, exactly as the backward pass of the
// rank that made the row computes them) and ADDS all six rows to the dense tensors.  `rows` may be memory of another GPU
// (peer access enabled): the kernel only reads it, with plain 16-byte loads, each byte once.
//
// A warp takes 32 rows at a time.  (1) It reads their 2 KB as four fully coalesced 512-byte loads and turns them by 90 degrees
// through shared memory, so that lane t holds row t.  (2) Lane t computes the 59 values of its row into a shared-memory tile.
// (3) The warp adds the tile to the tensors with the lanes on consecutive floats of a dense row (the 45 floats of a grad_sh_rest
// row are two instructions touching six sectors, instead of 45 instructions touching 32 sectors each with one lane per row).
struct DenseGradients {
    float* positions; float* scales; float* rotations; float* opacities; float* sh_0; float* sh_rest;
};
constexpr int kExpandWarps = 4;
constexpr int kExpandValues = 59;     // 3 + 3 + 4 + 1 + 3 + 45
constexpr int kExpandStride = 61;     // odd: lane t writing column c and lane c reading row t are both conflict-free
constexpr int kExpandGroup = 8;       // dense rows whose loads are in flight together (a row's load must not wait for the previous row's store)
static_assert(kExpandValues <= kExpandStride && 32 % kExpandGroup == 0, "tile layout");
__global__ void __launch_bounds__(kExpandWarps * 32) expand_add_rows_kernel(const float4* __restrict__ rows, uint32_t capacity, const float* __restrict__ positions,
                                                                            DenseGradients out, uint32_t n_primitives, int total_sh_bases) {
    __shared__ __align__(16) float s_tile[kExpandWarps][32 * kExpandStride];      // first the 32 compact rows (2 KB), then the 32 x 59 values
    const CompactGradientHeader* header = reinterpret_cast<const CompactGradientHeader*>(rows);
    const uint32_t count = min(header->count, capacity);
    const float3 cam = make_float3(header->cam_x, header->cam_y, header->cam_z);
    const int active = min(int(header->active_sh_bases), total_sh_bases + 1);
    const int sh_floats = 3 * (active > 9 ? 15 : active > 4 ? 8 : active > 1 ? 3 : 0);      // floats of a grad_sh_rest row that get a value
    const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;
    float* tile = s_tile[warp];
    float4* my_rows = reinterpret_cast<float4*>(tile);
    const uint32_t n_warps = gridDim.x * kExpandWarps;
    const size_t sh_row = size_t(total_sh_bases) * 3;
    for (uint32_t base = (blockIdx.x * kExpandWarps + warp) * 32u; base < count; base += n_warps * 32u) {
        const uint32_t here = min(32u, count - base);          // rows of this trip
        const float4* src = rows + kCompactRowFloat4s * (size_t(base) + 1);
        #pragma unroll
        for (int k = 0; k < kCompactRowFloat4s; ++k)
            if (k * 32u + lane < here * kCompactRowFloat4s) my_rows[k * 32 + lane] = src[k * 32 + lane];
        __syncwarp();
        float4 a = make_float4(0, 0, 0, 0), b = a, c = a, d = a;
        if (lane < here) {
            a = my_rows[lane * kCompactRowFloat4s]; b = my_rows[lane * kCompactRowFloat4s + 1];
            c = my_rows[lane * kCompactRowFloat4s + 2]; d = my_rows[lane * kCompactRowFloat4s + 3];
        }
        __syncwarp();      // every lane holds its row: the tile may overwrite the staged rows
        uint32_t idx = 0xffffffffu;
        if (lane < here) {
            idx = __float_as_uint(a.x);
            if (idx >= n_primitives) idx = 0xffffffffu;      // not a row of this scene: skipped rather than written out of bounds
            float* t = tile + lane * kExpandStride;
            t[0] = a.y; t[1] = a.z; t[2] = a.w;
            t[3] = b.x; t[4] = b.y; t[5] = b.z;
            t[6] = c.x; t[7] = c.y; t[8] = c.z; t[9] = c.w;
            t[10] = b.w;
            const float3 grad_rgb = make_float3(d.x, d.y, d.z);
            const float3 band0 = kShBand0 * grad_rgb;
            t[11] = band0.x; t[12] = band0.y; t[13] = band0.z;
            if (sh_floats > 0 && idx != 0xffffffffu) {
                const size_t g = idx;
                const float3 position = make_float3(__ldg(positions + 3 * g), __ldg(positions + 3 * g + 1), __ldg(positions + 3 * g + 2));
                const float3 dir = normalize(position - cam);
                float3 sh[15];
                const int written = sh_rest_gradient_rows(dir, grad_rgb, active, sh);
                #pragma unroll
                for (int i = 0; i < 15; ++i)
                    if (i < written) { t[14 + 3 * i] = sh[i].x; t[15 + 3 * i] = sh[i].y; t[16 + 3 * i] = sh[i].z; }
            }
        }
        __syncwarp();
        // grad_sh_rest: lanes on consecutive floats of a dense row (45 floats = two steps), kExpandGroup rows' loads in flight together
        const bool lo = int(lane) < sh_floats, hi = int(lane) + 32 < sh_floats;
        for (uint32_t r0 = 0; r0 < here; r0 += kExpandGroup) {
            float* dst[kExpandGroup];
            float v0[kExpandGroup], v1[kExpandGroup];
            #pragma unroll
            for (int j = 0; j < kExpandGroup; ++j) {
                const uint32_t g = __shfl_sync(0xffffffffu, idx, int(r0) + j);      // lanes beyond `here` hold the invalid mark
                dst[j] = g == 0xffffffffu ? nullptr : out.sh_rest + size_t(g) * sh_row;
                v0[j] = (dst[j] && lo) ? dst[j][lane] : 0.0f;
                v1[j] = (dst[j] && hi) ? dst[j][lane + 32] : 0.0f;
            }
            #pragma unroll
            for (int j = 0; j < kExpandGroup; ++j) {
                const float* v = tile + (r0 + j) * kExpandStride + 14;
                if (dst[j] && lo) dst[j][lane] = v0[j] + v[lane];
                if (dst[j] && hi) dst[j][lane + 32] = v1[j] + v[lane + 32];
            }
        }
        // the five narrow tensors: element e of the trip's 32 x width block belongs to row e / width; all loads first
        float* p3[3][3]; float old3[3][3]; uint32_t r3[3], c3[3];
        #pragma unroll
        for (int k = 0; k < 3; ++k) {
            const uint32_t e = k * 32u + lane, r = e / 3u, cc = e - 3u * r;
            const uint32_t g = __shfl_sync(0xffffffffu, idx, int(r));
            r3[k] = r; c3[k] = cc;
            p3[k][0] = g == 0xffffffffu ? nullptr : out.positions + size_t(g) * 3 + cc;
            p3[k][1] = g == 0xffffffffu ? nullptr : out.scales + size_t(g) * 3 + cc;
            p3[k][2] = g == 0xffffffffu ? nullptr : out.sh_0 + size_t(g) * 3 + cc;
            #pragma unroll
            for (int t = 0; t < 3; ++t) old3[k][t] = p3[k][t] ? *p3[k][t] : 0.0f;
        }
        float* p4[4]; float old4[4]; uint32_t r4[4], c4[4];
        #pragma unroll
        for (int k = 0; k < 4; ++k) {
            const uint32_t e = k * 32u + lane, r = e >> 2, cc = e & 3u;
            const uint32_t g = __shfl_sync(0xffffffffu, idx, int(r));
            r4[k] = r; c4[k] = cc;
            p4[k] = g == 0xffffffffu ? nullptr : out.rotations + size_t(g) * 4 + cc;
            old4[k] = p4[k] ? *p4[k] : 0.0f;
        }
        const float old_opacity = idx != 0xffffffffu ? out.opacities[idx] : 0.0f;
        #pragma unroll
        for (int k = 0; k < 3; ++k) {
            const float* t = tile + r3[k] * kExpandStride + c3[k];
            if (p3[k][0]) { *p3[k][0] = old3[k][0] + t[0]; *p3[k][1] = old3[k][1] + t[3]; *p3[k][2] = old3[k][2] + t[11]; }
        }
        #pragma unroll
        for (int k = 0; k < 4; ++k)
            if (p4[k]) *p4[k] = old4[k] + tile[r4[k] * kExpandStride + 6 + c4[k]];
        if (idx != 0xffffffffu) out.opacities[idx] = old_opacity + tile[lane * kExpandStride + 10];
        __syncwarp();
    }
}

// Sum of several compact-row buffers as dense gradients, every dense row written ONCE (htgs_expand_sum_rows).
// Expanding buffer after buffer with expand_add_rows_kernel reads and writes a dense row once per buffer that holds it; with
// many buffers (8 ranks) that is most of the exchange's time.  Here a table is built first - table[s][g] = row of Gaussian g in
// buffer s, or -1 - and then one kernel walks the Gaussians: a warp takes 32 consecutive ones, every lane adds up its
// Gaussian's rows from all buffers in registers, in buffer order starting from zero (the very additions the buffer-by-buffer
// expansion performs, so the bits are the same), and the warp stores the 32 dense rows of each tensor as one contiguous block.
// Rows of Gaussians no buffer holds are written as zeros: the tensors need not be cleared.
constexpr int kMaxSources = 16;
constexpr int kGatherGroup = 2;
static_assert(kMaxSources % kGatherGroup == 0, "groups of buffers");
struct CompactSources {
    const float4* rows[kMaxSources];
    int n;
};
__global__ void __launch_bounds__(256) build_slot_table_kernel(const __grid_constant__ CompactSources src, uint32_t capacity, int32_t* __restrict__ table,
                                                               uint32_t n_primitives) {
    const int s = int(blockIdx.y);
    const float4* rows = src.rows[s];
    const uint32_t count = min(reinterpret_cast<const CompactGradientHeader*>(rows)->count, capacity);
    int32_t* mine = table + size_t(s) * n_primitives;
    for (uint32_t r = blockIdx.x * 256 + threadIdx.x; r < count; r += gridDim.x * 256) {
        const uint32_t idx = __float_as_uint(reinterpret_cast<const float*>(rows + kCompactRowFloat4s * (size_t(r) + 1))[0]);
        if (idx < n_primitives) mine[idx] = int32_t(r);
    }
}

__global__ void __launch_bounds__(kExpandWarps * 32) gather_sum_rows_kernel(const __grid_constant__ CompactSources src, uint32_t capacity,
                                                                            const int32_t* __restrict__ table, const float* __restrict__ positions,
                                                                            DenseGradients out, uint32_t n_primitives, int total_sh_bases) {
    __shared__ __align__(16) float s_tile[kExpandWarps][32 * kExpandValues];      // 32 x 45 for grad_sh_rest, then the narrow tensors' 32 x (3 + 3 + 3 + 4 + 1)
    const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;
    float* tile = s_tile[warp];
    const uint32_t n_chunks = (n_primitives + 31u) / 32u;
    const uint32_t n_warps = gridDim.x * kExpandWarps;
    const uint32_t sh_width = uint32_t(total_sh_bases) * 3u;
    for (uint32_t chunk = blockIdx.x * kExpandWarps + warp; chunk < n_chunks; chunk += n_warps) {
        const uint32_t g = chunk * 32u + lane;
        const bool inside = g < n_primitives;
        const uint32_t here = min(32u, n_primitives - chunk * 32u);
        float acc[kExpandValues];
        #pragma unroll
        for (int i = 0; i < kExpandValues; ++i) acc[i] = 0.0f;
        float3 position = make_float3(0, 0, 0);
        bool have_position = false;
        // buffers in groups of kGatherGroup: the group's table entries, then its rows, are all in flight before the first is used
        #pragma unroll 1
        for (int s0 = 0; s0 < src.n; s0 += kGatherGroup) {
            int32_t slot[kGatherGroup];
            #pragma unroll
            for (int j = 0; j < kGatherGroup; ++j) slot[j] = (s0 + j < src.n && inside) ? table[size_t(s0 + j) * n_primitives + g] : -1;
            float4 ra[kGatherGroup], rb[kGatherGroup], rc[kGatherGroup], rd[kGatherGroup];
            #pragma unroll
            for (int j = 0; j < kGatherGroup; ++j) {
                ra[j] = make_float4(__uint_as_float(0xffffffffu), 0, 0, 0);
                if (slot[j] >= 0) {
                    const float4* rows = src.rows[s0 + j];
                    if (uint32_t(slot[j]) < min(reinterpret_cast<const CompactGradientHeader*>(rows)->count, capacity)) {
                        const float4* row = rows + kCompactRowFloat4s * (size_t(slot[j]) + 1);
                        ra[j] = row[0]; rb[j] = row[1]; rc[j] = row[2]; rd[j] = row[3];
                    }
                }
            }
            #pragma unroll
            for (int j = 0; j < kGatherGroup; ++j) {
                if (slot[j] < 0 || __float_as_uint(ra[j].x) != g) continue;      // no row, a stale table entry or a foreign row: adds nothing
                const float4 a = ra[j], b = rb[j], c = rc[j], d = rd[j];
                const CompactGradientHeader* header = reinterpret_cast<const CompactGradientHeader*>(src.rows[s0 + j]);
                // __fadd_rn: the products below must be rounded before they are added (no multiply-add contraction), as they
                // are when the buffer-by-buffer expansion passes them through shared memory
                acc[0] = __fadd_rn(acc[0], a.y); acc[1] = __fadd_rn(acc[1], a.z); acc[2] = __fadd_rn(acc[2], a.w);
                acc[3] = __fadd_rn(acc[3], b.x); acc[4] = __fadd_rn(acc[4], b.y); acc[5] = __fadd_rn(acc[5], b.z);
                acc[6] = __fadd_rn(acc[6], c.x); acc[7] = __fadd_rn(acc[7], c.y); acc[8] = __fadd_rn(acc[8], c.z); acc[9] = __fadd_rn(acc[9], c.w);
                acc[10] = __fadd_rn(acc[10], b.w);
                const float3 grad_rgb = make_float3(d.x, d.y, d.z);
                const float3 band0 = kShBand0 * grad_rgb;
                acc[11] = __fadd_rn(acc[11], band0.x); acc[12] = __fadd_rn(acc[12], band0.y); acc[13] = __fadd_rn(acc[13], band0.z);
                const int active = min(int(header->active_sh_bases), total_sh_bases + 1);
                if (active > 1) {
                    if (!have_position) {
                        position = make_float3(__ldg(positions + 3 * size_t(g)), __ldg(positions + 3 * size_t(g) + 1), __ldg(positions + 3 * size_t(g) + 2));
                        have_position = true;
                    }
                    const float3 dir = normalize(position - make_float3(header->cam_x, header->cam_y, header->cam_z));
                    float3 sh[15];
                    const int written = sh_rest_gradient_rows(dir, grad_rgb, active, sh);
                    #pragma unroll
                    for (int i = 0; i < 15; ++i)
                        if (i < written) {
                            acc[14 + 3 * i] = __fadd_rn(acc[14 + 3 * i], sh[i].x); acc[15 + 3 * i] = __fadd_rn(acc[15 + 3 * i], sh[i].y);
                            acc[16 + 3 * i] = __fadd_rn(acc[16 + 3 * i], sh[i].z);
                        }
                }
            }
        }
        // The chunk's 32 rows of a tensor are one contiguous, 16-byte aligned block of the tensor (32 rows x width x 4 bytes): the
        // lanes lay their values out in shared memory exactly like that block and the warp stores it with 16-byte stores.
        float* t_sh = tile;                                  // [32][sh_width]
        float* t_pos = tile + 32 * 45;                       // [32][3]
        float* t_scale = t_pos + 96;                         // [32][3]
        float* t_sh0 = t_scale + 96;                         // [32][3]
        float* t_rot = t_sh0 + 96;                           // [32][4]
        float* t_opacity = t_rot + 128;                      // [32]
        t_pos[lane * 3] = acc[0]; t_pos[lane * 3 + 1] = acc[1]; t_pos[lane * 3 + 2] = acc[2];
        t_scale[lane * 3] = acc[3]; t_scale[lane * 3 + 1] = acc[4]; t_scale[lane * 3 + 2] = acc[5];
        reinterpret_cast<float4*>(t_rot)[lane] = make_float4(acc[6], acc[7], acc[8], acc[9]);
        t_opacity[lane] = acc[10];
        t_sh0[lane * 3] = acc[11]; t_sh0[lane * 3 + 1] = acc[12]; t_sh0[lane * 3 + 2] = acc[13];
        #pragma unroll
        for (int i = 0; i < 45; ++i)
            if (uint32_t(i) < sh_width) t_sh[lane * sh_width + i] = acc[14 + i];
        __syncwarp();
        const size_t first = size_t(chunk) * 32u;
        if (here == 32u) {
            float4* dst = reinterpret_cast<float4*>(out.sh_rest + first * sh_width);
            for (uint32_t e = lane; e < 8u * sh_width; e += 32) dst[e] = reinterpret_cast<const float4*>(t_sh)[e];
            if (lane < 24u) {
                reinterpret_cast<float4*>(out.positions + first * 3)[lane] = reinterpret_cast<const float4*>(t_pos)[lane];
                reinterpret_cast<float4*>(out.scales + first * 3)[lane] = reinterpret_cast<const float4*>(t_scale)[lane];
                reinterpret_cast<float4*>(out.sh_0 + first * 3)[lane] = reinterpret_cast<const float4*>(t_sh0)[lane];
            }
            reinterpret_cast<float4*>(out.rotations + first * 4)[lane] = reinterpret_cast<const float4*>(t_rot)[lane];
            if (lane < 8u) reinterpret_cast<float4*>(out.opacities + first)[lane] = reinterpret_cast<const float4*>(t_opacity)[lane];
        } else {      // the scene's last, partial chunk
            for (uint32_t e = lane; e < here * sh_width; e += 32) out.sh_rest[first * sh_width + e] = t_sh[e];
            for (uint32_t e = lane; e < here * 3u; e += 32) {
                out.positions[first * 3 + e] = t_pos[e]; out.scales[first * 3 + e] = t_scale[e]; out.sh_0[first * 3 + e] = t_sh0[e];
            }
            for (uint32_t e = lane; e < here * 4u; e += 32) out.rotations[first * 4 + e] = t_rot[e];
            if (lane < here) out.opacities[first + lane] = t_opacity[lane];
        }
        __syncwarp();
    }
}

// Copies a compact-row buffer (header + the rows its header counts, at most `capacity`) with 16-byte loads and stores, every
// thread with several loads in flight.  `src` is typically another GPU's buffer: a rank pulls the other ranks' buffers into
// local memory one after the other, each rank starting with a different peer, so that at any time every GPU's memory is read by
// one other GPU instead of by all of them.
constexpr int kCopyInFlight = 8;
__global__ void __launch_bounds__(256) copy_rows_kernel(const float4* __restrict__ src, float4* __restrict__ dst, uint32_t capacity) {
    const CompactGradientHeader* header = reinterpret_cast<const CompactGradientHeader*>(src);
    const size_t n4 = (size_t(min(header->count, capacity)) + 1) * kCompactRowFloat4s;      // header included
    const size_t stride = size_t(gridDim.x) * 256;
    for (size_t i = size_t(blockIdx.x) * 256 + threadIdx.x; i < n4; i += stride * kCopyInFlight) {
        float4 v[kCopyInFlight];
        #pragma unroll
        for (int k = 0; k < kCopyInFlight; ++k)
            if (i + k * stride < n4) v[k] = src[i + k * stride];
        #pragma unroll
        for (int k = 0; k < kCopyInFlight; ++k)
            if (i + k * stride < n4) dst[i + k * stride] = v[k];
    }
}

int move_rows(bool gather, const HtgsRowTensors* tensors, const int64_t* index, int64_t count, float* packed, void* stream) {
    if (!tensors || count < 0 || tensors->n_tensors < 1 || tensors->n_tensors > HTGS_MAX_ROW_TENSORS)
        return exchange_fail(HTGS_ERR_INVALID_ARGUMENT, "row exchange: null argument, negative count or too many tensors");
    if (count == 0) return HTGS_OK;
    if (!index || !packed) return exchange_fail(HTGS_ERR_INVALID_ARGUMENT, "row exchange: null index or packed buffer");
    RowTable table{};
    table.n_tensors = tensors->n_tensors;
    int32_t begin = 0;
    for (int k = 0; k < tensors->n_tensors; ++k) {
        if (!tensors->data[k] || tensors->width[k] < 1) return exchange_fail(HTGS_ERR_INVALID_ARGUMENT, "row exchange: a tensor is null or has no columns");
        table.ptr[k] = tensors->data[k];
        table.width[k] = tensors->width[k];
        table.begin[k] = begin;
        begin += tensors->width[k];
    }
    table.begin[tensors->n_tensors] = begin;
    if (count > int64_t(0xffffffffu)) return exchange_fail(HTGS_ERR_INVALID_ARGUMENT, "row exchange: more than 2^32 - 1 rows");
    const uint64_t rows_per_block = uint64_t(kRowBlock / 32) * kRowsPerTrip;
    const uint64_t blocks = (uint64_t(count) + rows_per_block - 1) / rows_per_block;
    const uint32_t grid = uint32_t(blocks < (1u << 16) ? blocks : (1u << 16));
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (gather) move_rows_kernel<true><<<grid, kRowBlock, 0, s>>>(table, index, uint32_t(count), packed);
    else move_rows_kernel<false><<<grid, kRowBlock, 0, s>>>(table, index, uint32_t(count), packed);
    const cudaError_t err = cudaGetLastError();
    return err == cudaSuccess ? HTGS_OK : exchange_fail(HTGS_ERR_CUDA, cudaGetErrorString(err));
}

}  // namespace

}  // namespace htgs

extern "C" {

int htgs_gather_rows(const HtgsRowTensors* tensors, const int64_t* index, int64_t count, float* packed, void* stream) {
    return htgs::move_rows(true, tensors, index, count, packed, stream);
}

size_t htgs_compact_rows_bytes(uint32_t capacity_rows) { return (size_t(capacity_rows) + 1) * sizeof(htgs::CompactGradientHeader); }

int htgs_expand_add_rows(const HtgsScene* scene, const void* rows, uint32_t capacity_rows, const HtgsGradients* grads, void* stream) {
    using namespace htgs;
    if (!scene || !rows || !grads) return exchange_fail(HTGS_ERR_INVALID_ARGUMENT, "expand rows: null argument");
    if (scene->n_primitives < 0 || scene->total_sh_bases < 0 || scene->total_sh_bases > 15)
        return exchange_fail(HTGS_ERR_INVALID_ARGUMENT, "expand rows: bad scene sizes");
    if (scene->n_primitives == 0 || capacity_rows == 0) return HTGS_OK;
    if (!scene->positions || !grads->grad_positions || !grads->grad_scales || !grads->grad_rotations || !grads->grad_opacities || !grads->grad_sh_0 ||
        (scene->total_sh_bases > 0 && !grads->grad_sh_rest))
        return exchange_fail(HTGS_ERR_INVALID_ARGUMENT, "expand rows: positions and the six gradient tensors must not be null");
    if ((reinterpret_cast<uintptr_t>(rows) & 15u) != 0) return exchange_fail(HTGS_ERR_INVALID_ARGUMENT, "expand rows: the row buffer must be 16-byte aligned");
    const DenseGradients out{grads->grad_positions, grads->grad_scales, grads->grad_rotations, grads->grad_opacities, grads->grad_sh_0, grads->grad_sh_rest};
    const uint32_t rows_per_block = kExpandWarps * 32u;
    const uint32_t blocks = (capacity_rows + rows_per_block - 1u) / rows_per_block;
    expand_add_rows_kernel<<<blocks < 148u * 32u ? blocks : 148u * 32u, kExpandWarps * 32, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const float4*>(rows), capacity_rows, scene->positions, out, uint32_t(scene->n_primitives), int(scene->total_sh_bases));
    const cudaError_t err = cudaGetLastError();
    return err == cudaSuccess ? HTGS_OK : exchange_fail(HTGS_ERR_CUDA, cudaGetErrorString(err));
}

size_t htgs_expand_sum_scratch_bytes(const HtgsScene* scene, int n_buffers) {
    if (!scene || scene->n_primitives <= 0 || n_buffers <= 0) return 0;
    return size_t(n_buffers) * size_t(scene->n_primitives) * sizeof(int32_t);
}

int htgs_expand_sum_rows(const HtgsScene* scene, const void* const* buffers, int n_buffers, uint32_t capacity_rows, void* scratch, size_t scratch_bytes,
                         const HtgsGradients* grads, void* stream_ptr) {
    using namespace htgs;
    if (!scene || !buffers || !grads) return exchange_fail(HTGS_ERR_INVALID_ARGUMENT, "expand sum: null argument");
    if (n_buffers < 1 || n_buffers > kMaxSources) return exchange_fail(HTGS_ERR_INVALID_ARGUMENT, "expand sum: between 1 and 16 buffers");
    if (scene->n_primitives < 0 || scene->total_sh_bases < 0 || scene->total_sh_bases > 15)
        return exchange_fail(HTGS_ERR_INVALID_ARGUMENT, "expand sum: bad scene sizes");
    if (scene->n_primitives == 0) return HTGS_OK;
    if (!scene->positions || !grads->grad_positions || !grads->grad_scales || !grads->grad_rotations || !grads->grad_opacities || !grads->grad_sh_0 ||
        (scene->total_sh_bases > 0 && !grads->grad_sh_rest))
        return exchange_fail(HTGS_ERR_INVALID_ARGUMENT, "expand sum: positions and the six gradient tensors must not be null");
    if (!scratch || scratch_bytes < htgs_expand_sum_scratch_bytes(scene, n_buffers)) return exchange_fail(HTGS_ERR_WORKSPACE_TOO_SMALL, "expand sum: scratch too small");
    if (((reinterpret_cast<uintptr_t>(grads->grad_positions) | reinterpret_cast<uintptr_t>(grads->grad_scales) | reinterpret_cast<uintptr_t>(grads->grad_rotations) |
          reinterpret_cast<uintptr_t>(grads->grad_opacities) | reinterpret_cast<uintptr_t>(grads->grad_sh_0) | reinterpret_cast<uintptr_t>(grads->grad_sh_rest)) & 15u) != 0)
        return exchange_fail(HTGS_ERR_INVALID_ARGUMENT, "expand sum: the six gradient tensors must be 16-byte aligned (they are written with 16-byte stores)");
    CompactSources src{};
    src.n = n_buffers;
    for (int s = 0; s < n_buffers; ++s) {
        if (!buffers[s] || (reinterpret_cast<uintptr_t>(buffers[s]) & 15u) != 0)
            return exchange_fail(HTGS_ERR_INVALID_ARGUMENT, "expand sum: a buffer is null or not 16-byte aligned");
        src.rows[s] = static_cast<const float4*>(buffers[s]);
    }
    cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);
    const uint32_t n = uint32_t(scene->n_primitives);
    cudaError_t err = cudaMemsetAsync(scratch, 0xff, size_t(n_buffers) * n * sizeof(int32_t), stream);
    if (err != cudaSuccess) return exchange_fail(HTGS_ERR_CUDA, cudaGetErrorString(err));
    if (capacity_rows > 0) {
        const uint32_t blocks = (capacity_rows + 255u) / 256u;
        build_slot_table_kernel<<<dim3(blocks < 148u * 4u ? blocks : 148u * 4u, unsigned(n_buffers), 1), 256, 0, stream>>>(src, capacity_rows, static_cast<int32_t*>(scratch), n);
        if ((err = cudaGetLastError()) != cudaSuccess) return exchange_fail(HTGS_ERR_CUDA, cudaGetErrorString(err));
    }
    const DenseGradients out{grads->grad_positions, grads->grad_scales, grads->grad_rotations, grads->grad_opacities, grads->grad_sh_0, grads->grad_sh_rest};
    const uint32_t chunk_blocks = ((n + 31u) / 32u + kExpandWarps - 1u) / kExpandWarps;
    gather_sum_rows_kernel<<<chunk_blocks < 148u * 32u ? chunk_blocks : 148u * 32u, kExpandWarps * 32, 0, stream>>>(
        src, capacity_rows, static_cast<const int32_t*>(scratch), scene->positions, out, n, int(scene->total_sh_bases));
    err = cudaGetLastError();
    return err == cudaSuccess ? HTGS_OK : exchange_fail(HTGS_ERR_CUDA, cudaGetErrorString(err));
}

int htgs_copy_rows(void* dst, const void* src, uint32_t capacity_rows, void* stream) {
    using namespace htgs;
    if (!dst || !src) return exchange_fail(HTGS_ERR_INVALID_ARGUMENT, "copy rows: null argument");
    if (((reinterpret_cast<uintptr_t>(dst) | reinterpret_cast<uintptr_t>(src)) & 15u) != 0)
        return exchange_fail(HTGS_ERR_INVALID_ARGUMENT, "copy rows: the buffers must be 16-byte aligned");
    copy_rows_kernel<<<148 * 4, 256, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<const float4*>(src), static_cast<float4*>(dst), capacity_rows);
    const cudaError_t err = cudaGetLastError();
    return err == cudaSuccess ? HTGS_OK : exchange_fail(HTGS_ERR_CUDA, cudaGetErrorString(err));
}

// Buffers another process's GPU can read: plain cudaMalloc memory (no pool, no virtual-memory mapping), exported and opened
// with the CUDA IPC calls.  Opening enables peer access between the two devices if it is not enabled yet.
int htgs_peer_buffer_create(int device, size_t bytes, void** ptr, void* handle) {
    using namespace htgs;
    if (!ptr || !handle || bytes == 0) return exchange_fail(HTGS_ERR_INVALID_ARGUMENT, "peer buffer: null argument or empty buffer");
    int previous = -1;
    cudaError_t err = cudaGetDevice(&previous);
    if (err == cudaSuccess) err = cudaSetDevice(device);
    void* p = nullptr;
    if (err == cudaSuccess) err = cudaMalloc(&p, bytes);
    if (err == cudaSuccess) err = cudaMemset(p, 0, bytes);
    cudaIpcMemHandle_t h;
    if (err == cudaSuccess) err = cudaIpcGetMemHandle(&h, p);
    if (previous >= 0) cudaSetDevice(previous);
    if (err != cudaSuccess) {
        if (p) cudaFree(p);
        return exchange_fail(HTGS_ERR_CUDA, cudaGetErrorString(err));
    }
    static_assert(sizeof(cudaIpcMemHandle_t) == HTGS_PEER_HANDLE_BYTES, "handle size");
    memcpy(handle, &h, sizeof(h));
    *ptr = p;
    return HTGS_OK;
}

int htgs_peer_buffer_open(int device, const void* handle, void** ptr) {
    using namespace htgs;
    if (!ptr || !handle) return exchange_fail(HTGS_ERR_INVALID_ARGUMENT, "peer buffer: null argument");
    int previous = -1;
    cudaError_t err = cudaGetDevice(&previous);
    if (err == cudaSuccess) err = cudaSetDevice(device);
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, sizeof(h));
    void* p = nullptr;
    if (err == cudaSuccess) err = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
    if (previous >= 0) cudaSetDevice(previous);
    if (err != cudaSuccess) { cudaGetLastError(); return exchange_fail(HTGS_ERR_CUDA, cudaGetErrorString(err)); }
    *ptr = p;
    return HTGS_OK;
}

int htgs_peer_buffer_close(int device, void* ptr) {
    using namespace htgs;
    if (!ptr) return HTGS_OK;
    int previous = -1;
    cudaError_t err = cudaGetDevice(&previous);
    if (err == cudaSuccess) err = cudaSetDevice(device);
    if (err == cudaSuccess) err = cudaIpcCloseMemHandle(ptr);
    if (previous >= 0) cudaSetDevice(previous);
    return err == cudaSuccess ? HTGS_OK : exchange_fail(HTGS_ERR_CUDA, cudaGetErrorString(err));
}

int htgs_peer_buffer_destroy(int device, void* ptr) {
    using namespace htgs;
    if (!ptr) return HTGS_OK;
    int previous = -1;
    cudaError_t err = cudaGetDevice(&previous);
    if (err == cudaSuccess) err = cudaSetDevice(device);
    if (err == cudaSuccess) err = cudaFree(ptr);
    if (previous >= 0) cudaSetDevice(previous);
    return err == cudaSuccess ? HTGS_OK : exchange_fail(HTGS_ERR_CUDA, cudaGetErrorString(err));
}

int htgs_scatter_rows(const HtgsRowTensors* tensors, const int64_t* index, int64_t count, const float* packed, void* stream) {
    return htgs::move_rows(false, tensors, index, count, const_cast<float*>(packed), stream);
}

}  // extern "C"
