// Packing of per-Gaussian rows for the multi-GPU gradient exchange.  No counterpart in the reference (it is single-GPU).
//
// A training view keeps about a sixth of a scene's Gaussians and its backward pass leaves every other row of the six
// gradient tensors zero, so the ranks only have to sum the rows of Gaussians SOME rank kept.  htgs_gather_rows copies
// those rows of up to 8 row-major float tensors (widths 3, 3, 4, 1, 3, 3 B for the rasterizer's inputs) into one dense
// [count, sum of widths] buffer, which one all-reduce sums; htgs_scatter_rows writes the sums back.  Both are pure
// streaming kernels (one warp per row, lanes on consecutive floats of the packed row): the packed side is fully
// coalesced, the tensor side moves whole rows of 4 to 540 bytes.
#include "kernels.h"


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

int htgs_scatter_rows(const HtgsRowTensors* tensors, const int64_t* index, int64_t count, const float* packed, void* stream) {
    return htgs::move_rows(false, tensors, index, count, const_cast<float*>(packed), stream);
}

}  // extern "C"
