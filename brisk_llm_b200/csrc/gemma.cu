// The few extra kernels of the Gemma 3 layer variants (brisk-llm src/model.h:24): the embedding scale, the RMS norm a
// projection's output gets before it joins the residual stream, and the soft cap of the logits. The tanh-GELU gate is
// gelu_mul() in formats.cuh, applied by launch_gate_mul; the sliding window is a parameter of the attention kernels.
#include "common.cuh"
#include "formats.cuh"
#include "kernels.h"
#include "rowops.cuh"

namespace bk {
namespace {

__global__ void __launch_bounds__(256) scale_rows_kernel(float* x, size_t count, float scale) {
    const size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i < count) x[i] = __fmul_rn(x[i], scale);
}

// One CTA per token row: p = proj * scale * weight (rms_norm's order, src/model.cpp:87-97), then hidden += p.
__global__ void __launch_bounds__(256) post_norm_add_kernel(const float* __restrict__ proj, const float* __restrict__ weight,
                                                            float* __restrict__ hidden, uint32_t cols, float eps) {
    __shared__ double red[32];
    const float* p = proj + size_t(blockIdx.x) * cols;
    float* h = hidden + size_t(blockIdx.x) * cols;
    const float scale = cta_rms_scale(p, cols, eps, red);
    for (uint32_t i = threadIdx.x; i < cols; i += blockDim.x) {
        h[i] = __fadd_rn(h[i], __fmul_rn(__fmul_rn(p[i], scale), weight[i]));
    }
}

__global__ void __launch_bounds__(256) softcap_kernel(float* logits, size_t count, float cap) {
    const size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i < count) logits[i] = __fmul_rn(cap, tanh_via_double(__fdiv_rn(logits[i], cap)));
}

}  // namespace

void launch_scale_rows(float* x, size_t count, float scale, cudaStream_t s) {
    scale_rows_kernel<<<unsigned((count + 255) / 256), 256, 0, s>>>(x, count, scale);
    BK_CUDA(cudaGetLastError());
}

void launch_post_norm_add(const float* proj, const float* weight, float* hidden, uint32_t n, uint32_t cols, float eps, cudaStream_t s) {
    post_norm_add_kernel<<<n, 256, 0, s>>>(proj, weight, hidden, cols, eps);
    BK_CUDA(cudaGetLastError());
}

void launch_softcap(float* logits, size_t count, float cap, cudaStream_t s) {
    softcap_kernel<<<unsigned((count + 255) / 256), 256, 0, s>>>(logits, count, cap);
    BK_CUDA(cudaGetLastError());
}

}  // namespace bk
