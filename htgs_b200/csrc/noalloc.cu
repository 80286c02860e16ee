// htgs_backward_static: the backward pass for callers that are not allowed to allocate device memory.
//
// The regular htgs_backward wants a caller-provided scratch buffer for its per-Gaussian accumulation
// records (80 bytes per Gaussian).  A host that embeds the rasterizer in a fixed memory budget - a render
// plug-in whose host application owns every allocation, or a training loop that has handed all free memory
// to another allocator - may have no way to produce that buffer.  This variant keeps the records in a
// file-scope device array instead, so the call itself performs no cudaMalloc / cudaFree and uses no
// allocating library routine.  The price is a fixed upper bound on the number of Gaussians and 10 MiB of
// device memory that every GPU loading this library holds until the process exits.
#include <string>

#include "kernels.h"

namespace {

constexpr int kStaticMaxGaussians = 131072;                       // 131072 * 5 * 16 B = 10 MiB
static __device__ __align__(256) float4 g_static_accum[size_t(kStaticMaxGaussians) * 5];

constexpr int kMaxDevices = 64;
float4* g_static_accum_ptr[kMaxDevices] = {};                     // device address of the array, per device

}  // namespace

extern "C" int htgs_backward_static_max_gaussians(void) { return kStaticMaxGaussians; }

extern "C" int htgs_backward_static(HtgsContext* ctx, const HtgsScene* scene, const HtgsView* view, const HtgsTrainBlobs* blobs, uint32_t n_instances,
                                    const float* grad_image, const float* image, const HtgsGradients* grads, void* stream) {
    if (!ctx || !scene) { htgs::set_last_error("htgs_backward_static: null argument"); return HTGS_ERR_INVALID_ARGUMENT; }
    if (scene->n_primitives > kStaticMaxGaussians) {
        htgs::set_last_error("htgs_backward_static: scene has more than 131072 Gaussians, the capacity of the built-in scratch; use htgs_backward with a caller-provided scratch buffer");
        return HTGS_ERR_INVALID_ARGUMENT;
    }
    const int device = htgs::context_device(ctx);
    if (device < 0 || device >= kMaxDevices) { htgs::set_last_error("htgs_backward_static: device index out of range"); return HTGS_ERR_INVALID_ARGUMENT; }
    if (!g_static_accum_ptr[device]) {
        // First call on this device: translate the host-side symbol into the device address, with that device current.
        // (The symbol name itself is NOT a device pointer in host code; passing it to a kernel would be wrong.)
        int current = -1;
        cudaError_t err = cudaGetDevice(&current);
        if (err == cudaSuccess && current != device) err = cudaSetDevice(device);
        void* ptr = nullptr;
        if (err == cudaSuccess) err = cudaGetSymbolAddress(&ptr, g_static_accum);
        if (err != cudaSuccess || !ptr) {
            htgs::set_last_error((std::string("htgs_backward_static: cudaGetSymbolAddress failed: ") + cudaGetErrorString(err)).c_str());
            return HTGS_ERR_CUDA;
        }
        g_static_accum_ptr[device] = static_cast<float4*>(ptr);
    }
    return htgs::backward_with_accum(ctx, scene, view, blobs, n_instances, grad_image, image, grads, g_static_accum_ptr[device], 0, uint32_t(scene->n_primitives > 0 ? scene->n_primitives : 0),
                                     htgs::kBackwardAccumulate | htgs::kBackwardChainRule, stream);
}
