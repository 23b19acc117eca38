// RMS norm + activation quantisation, one pass per token row.
//
// The integer matrix kernels multiply weights by activations quantised exactly as the reference
// CPU engine quantises them, so that the block dot products are the same integers:
//   quantize_q8_0 (src/quant.cpp:115-142): d = amax/127 (f32), q = rint(x * (1/d)), stored scale = half(d)
//   quantize_q8_k (src/quant.cpp:146-194): inverse = -127/x_extreme (first of equal magnitudes),
//                                          d = 1/inverse, q = min(127, rint(inverse*x)), sums of 16
//   rms_norm      (src/model.cpp:87-97):   squares in f32, sum in f64, y = x * (1/sqrt(mean+eps)) * w
// All divisions and roots are IEEE-rounded; products are separate roundings (no contraction).
#include "kernels.h"
#include "rowops.cuh"

namespace bk {
namespace {

__global__ void __launch_bounds__(256) norm_quant_kernel(const float* __restrict__ x, uint32_t ldx, const float* __restrict__ weight,
                                                         float eps, uint32_t cols, DevActMut act, int want0, int wantk) {
    extern __shared__ float row[];  // the (normed) row
    __shared__ double red[32];
    const uint32_t t = blockIdx.x, tid = threadIdx.x;
    const float* xr = x + size_t(t) * ldx;
    if (weight != nullptr) {
        const float scale = cta_rms_scale(xr, cols, eps, red);
        for (uint32_t i = tid; i < cols; i += 256) row[i] = __fmul_rn(__fmul_rn(xr[i], scale), weight[i]);
    } else {
        for (uint32_t i = tid; i < cols; i += 256) row[i] = xr[i];
    }
    __syncthreads();
    if (act.f32 != nullptr) {
        float* o = act.f32 + size_t(t) * cols;
        for (uint32_t i = tid; i < cols; i += 256) o[i] = row[i];
    }
    if (want0) cta_quantize_q8_0(row, cols, act.q0 + size_t(t) * cols, act.d0 + size_t(t) * (cols / 32), act.s0 + size_t(t) * (cols / 32));
    if (wantk) cta_quantize_q8_k(row, cols, act.qk + size_t(t) * cols, act.dk + size_t(t) * (cols / 256), act.bs + size_t(t) * (cols / 16));
}

}  // namespace

void launch_norm_quant(const float* x, uint32_t ldx, const float* weight, float eps, uint32_t n, uint32_t cols,
                       const DevActMut& act, bool want0, bool wantk, cudaStream_t s) {
    const size_t smem = size_t(cols) * sizeof(float);
    static DeviceOnce once;
    if (smem > 48 * 1024 && once.first()) BK_CUDA(cudaFuncSetAttribute(norm_quant_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    norm_quant_kernel<<<n, 256, smem, s>>>(x, ldx, weight, eps, cols, act, want0 ? 1 : 0, wantk ? 1 : 0);
    BK_CUDA(cudaGetLastError());
}

}  // namespace bk
