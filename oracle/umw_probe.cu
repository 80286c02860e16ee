// Probe for ONE question about the reference: what does its HYBRID_BLEND `update_max_weights` give a Gaussian that only
// ever lands in the order-independent tail?  Test infrastructure, like everything under oracle/: never linked, loaded or
// executed by the product.
//
// The kernel source (rasterization/include/hybrid_blend/kernels/update_max_weights.cuh:170-210 of the reference) walks each
// tile's list a second time and credits `alpha * tail_weight` to every fragment, so a lone Gaussian of opacity 0.03 (below
// the 1/20 a fragment needs to enter the K-buffer) should end with a weight near 0.027.  The reference EXTENSION leaves it
// at 0.  The cause is a duplicate definition: rasterization/src/hybrid_blend/update_max_weights.cu:15-28 and
// rasterization/src/alpha_blend_first_k/update_max_weights.cu:15-28 both define the global function template
// `update_max_weights_k_templated` and instantiate it with the same argument types, so the two instantiations share one
// (weak) symbol and the linker keeps the first it meets.  The extension links alpha_blend_first_k before hybrid_blend:
// HYBRID_BLEND's host code then launches FIRST_K's kernel, which has no tail, on HYBRID's tile lists - the K nearest
// fragments with alpha >= 1/20, i.e. exactly HYBRID's K-buffer weights and nothing else.
//
// This driver calls the reference's own host function htgs::rasterization::hybrid_blend::update_max_weights
// (rasterization/src/hybrid_blend/update_max_weights.cu:30-165), compiled from the sources where they lie, on two
// Gaussians: the faint one and, a few tiles away, an opaque one that enters the K-buffer.  The Makefile links it three
// ways - with HYBRID's translation unit alone, and with FIRST_K's before or after it - and
// tests/test_gpu_max_weights.py compares the answers.
//
// Output: one line "tail_only <w0> core <w1>".
#include <cstdio>
#include <cstdlib>
#include <functional>
#include <vector>

#include <cuda_runtime.h>

#include "hybrid_blend/update_max_weights.h"

#define CHECK(call) do { cudaError_t e_ = (call); if (e_ != cudaSuccess) { std::fprintf(stderr, "%s: %s\n", #call, cudaGetErrorString(e_)); return 2; } } while (0)

int main(int argc, char** argv) {
    const float weight_threshold = argc > 1 ? float(std::atof(argv[1])) : 0.01f;
    const int K = argc > 2 ? std::atoi(argv[2]) : 16;
    const int n = 2, width = 64, height = 64;
    const float near_plane = 0.2f, far_plane = 100.0f, focal = 64.0f, centre = 32.0f;
    const float positions[n * 3] = {-0.25f, 0.0f, 3.0f, 0.25f, 0.0f, 3.0f};
    const float scales[n * 3] = {0.05f, 0.05f, 0.05f, 0.05f, 0.05f, 0.05f};
    const float rotations[n * 4] = {1.0f, 0.0f, 0.0f, 0.0f, 1.0f, 0.0f, 0.0f, 0.0f};
    const float opacities[n] = {0.03f, 0.9f};
    // camera contract of the reference's renderer (Renderer.py:34-44): M = identity, VPM = VP @ M
    const float M[16] = {1, 0, 0, 0, 0, 1, 0, 0, 0, 0, 1, 0, 0, 0, 0, 1};
    const float zs = (far_plane + near_plane) / (far_plane - near_plane), zo = -2.0f * far_plane * near_plane / (far_plane - near_plane);
    const float VPM[16] = {focal, 0, centre - 0.5f, 0, 0, focal, centre - 0.5f, 0, 0, 0, zs, zo, 0, 0, 1, 0};

    float *d_pos, *d_scale, *d_rot, *d_op, *d_M, *d_VPM, *d_w;
    CHECK(cudaMalloc(&d_pos, sizeof(positions))); CHECK(cudaMalloc(&d_scale, sizeof(scales))); CHECK(cudaMalloc(&d_rot, sizeof(rotations)));
    CHECK(cudaMalloc(&d_op, sizeof(opacities))); CHECK(cudaMalloc(&d_M, sizeof(M))); CHECK(cudaMalloc(&d_VPM, sizeof(VPM))); CHECK(cudaMalloc(&d_w, n * sizeof(float)));
    CHECK(cudaMemcpy(d_pos, positions, sizeof(positions), cudaMemcpyHostToDevice)); CHECK(cudaMemcpy(d_scale, scales, sizeof(scales), cudaMemcpyHostToDevice));
    CHECK(cudaMemcpy(d_rot, rotations, sizeof(rotations), cudaMemcpyHostToDevice)); CHECK(cudaMemcpy(d_op, opacities, sizeof(opacities), cudaMemcpyHostToDevice));
    CHECK(cudaMemcpy(d_M, M, sizeof(M), cudaMemcpyHostToDevice)); CHECK(cudaMemcpy(d_VPM, VPM, sizeof(VPM), cudaMemcpyHostToDevice));
    CHECK(cudaMemset(d_w, 0, n * sizeof(float)));

    std::vector<char*> blobs;
    auto alloc = [&blobs](size_t bytes) -> char* {
        char* p = nullptr;
        if (cudaMalloc(&p, bytes + 256) != cudaSuccess) return nullptr;
        blobs.push_back(p);
        return p;
    };
    htgs::rasterization::hybrid_blend::update_max_weights(alloc, alloc, alloc, reinterpret_cast<const float3*>(d_pos), reinterpret_cast<const float3*>(d_scale),
                                                          reinterpret_cast<const float4*>(d_rot), d_op, reinterpret_cast<const float4*>(d_M),
                                                          reinterpret_cast<const float4*>(d_VPM), d_w, K, n, width, height, near_plane, far_plane, weight_threshold);
    CHECK(cudaDeviceSynchronize());
    float w[n] = {};
    CHECK(cudaMemcpy(w, d_w, sizeof(w), cudaMemcpyDeviceToHost));
    std::printf("tail_only %.9g core %.9g\n", w[0], w[1]);
    for (char* p : blobs) cudaFree(p);
    return 0;
}
