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

namespace bk {
namespace {

__global__ void __launch_bounds__(256) norm_quant_kernel(const float* __restrict__ x, uint32_t ldx, const float* __restrict__ weight,
                                                         float eps, uint32_t cols, DevActMut act, int want0, int wantk) {
    extern __shared__ float row[];  // the (normed) row
    __shared__ double red[8];
    const uint32_t t = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const float* xr = x + size_t(t) * ldx;

    if (weight != nullptr) {
        double part = 0.0;
        for (uint32_t i = tid; i < cols; i += 256) {
            const float v = xr[i];
            part += double(__fmul_rn(v, v));
        }
        part = warp_sum(part);
        if (lane == 0) red[warp] = part;
        __syncthreads();
        double total = 0.0;
#pragma unroll
        for (int w = 0; w < 8; ++w) total += red[w];
        const float mean = float(total / double(cols));
        const float scale = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(mean, eps)));
        for (uint32_t i = tid; i < cols; i += 256) row[i] = __fmul_rn(__fmul_rn(xr[i], scale), weight[i]);
    } else {
        for (uint32_t i = tid; i < cols; i += 256) row[i] = xr[i];
    }
    __syncthreads();

    if (act.f32 != nullptr) {
        float* o = act.f32 + size_t(t) * cols;
        for (uint32_t i = tid; i < cols; i += 256) o[i] = row[i];
    }
    if (want0) {
        const uint32_t nb = cols / 32;
        for (uint32_t b = warp; b < nb; b += 8) {
            const float v = row[b * 32 + lane];
            const float amax = warp_max(fabsf(v));
            const float d = __fdiv_rn(amax, 127.0f);
            const float inv = d != 0.0f ? __fdiv_rn(1.0f, d) : 0.0f;
            const int q = __float2int_rn(__fmul_rn(v, inv));
            act.q0[size_t(t) * cols + b * 32 + lane] = int8_t(q);
            const int s = warp_sum(q);
            if (lane == 0) {
                act.d0[size_t(t) * nb + b] = __half2float(__float2half_rn(d));
                act.s0[size_t(t) * nb + b] = s;
            }
        }
    }
    if (wantk) {
        const uint32_t nb = cols / 256;
        for (uint32_t b = warp; b < nb; b += 8) {
            const float* v = row + b * 256 + lane * 8;
            float vals[8];
            float amax = 0.0f, ext = 0.0f;
            uint32_t idx = 0;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                vals[i] = v[i];
                const float ax = fabsf(vals[i]);
                if (ax > amax) {
                    amax = ax;
                    ext = vals[i];
                    idx = lane * 8 + i;
                }
            }
            // Largest magnitude, the earliest element on ties - what a sequential strict '>' scan finds.
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float oa = __shfl_xor_sync(0xffffffffu, amax, o);
                const float oe = __shfl_xor_sync(0xffffffffu, ext, o);
                const uint32_t oi = __shfl_xor_sync(0xffffffffu, idx, o);
                if (oa > amax || (oa == amax && oi < idx)) {
                    amax = oa;
                    ext = oe;
                    idx = oi;
                }
            }
            int8_t* qo = act.qk + size_t(t) * cols + b * 256 + lane * 8;
            if (amax == 0.0f) {
                *reinterpret_cast<uint2*>(qo) = make_uint2(0u, 0u);
                if ((lane & 1) == 0) act.bs[size_t(t) * (cols / 16) + b * 16 + (lane >> 1)] = 0;
                if (lane == 0) act.dk[size_t(t) * nb + b] = 0.0f;
                continue;
            }
            const float inv = __fdiv_rn(-127.0f, ext);
            uint32_t w[2] = {0u, 0u};
            int sum = 0;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const int q = int(fminf(127.0f, rintf(__fmul_rn(inv, vals[i]))));
                sum += q;
                w[i >> 2] |= uint32_t(uint8_t(int8_t(q))) << (8 * (i & 3));
            }
            *reinterpret_cast<uint2*>(qo) = make_uint2(w[0], w[1]);
            sum += __shfl_xor_sync(0xffffffffu, sum, 1);
            if ((lane & 1) == 0) act.bs[size_t(t) * (cols / 16) + b * 16 + (lane >> 1)] = int16_t(sum);
            if (lane == 0) act.dk[size_t(t) * nb + b] = __fdiv_rn(1.0f, inv);
        }
    }
}

}  // namespace

void launch_norm_quant(const float* x, uint32_t ldx, const float* weight, float eps, uint32_t n, uint32_t cols,
                       const DevActMut& act, bool want0, bool wantk, cudaStream_t s) {
    const size_t smem = size_t(cols) * sizeof(float);
    static bool raised = false;
    if (smem > 48 * 1024 && !raised) {
        BK_CUDA(cudaFuncSetAttribute(norm_quant_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        raised = true;
    }
    norm_quant_kernel<<<n, 256, smem, s>>>(x, ldx, weight, eps, cols, act, want0 ? 1 : 0, wantk ? 1 : 0);
    BK_CUDA(cudaGetLastError());
}

}  // namespace bk
