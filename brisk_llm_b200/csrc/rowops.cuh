// CTA-cooperative operations on one activation row held in shared memory: RMS-norm scale, Q8_0 and Q8_K
// quantisation. Bit-exact restatements of the reference's scalar code:
//   rms_norm      (src/model.cpp:87-97):   squares in f32, sum in f64, scale = 1/sqrt(mean + eps) in f32
//   quantize_q8_0 (src/quant.cpp:115-142): d = amax/127 (f32), q = rint(x * (1/d)), stored scale = half(d)
//   quantize_q8_k (src/quant.cpp:146-194): inverse = -127/x_extreme (first of equal magnitudes), d = 1/inverse,
//                                          q = min(127, rint(inverse*x)), sums of 16
// Divisions and roots are IEEE-rounded; products are separate roundings. All threads of the CTA must call these
// (they contain barriers); blockDim.x must be a multiple of 32 and at most 1024.
#pragma once

#include "common.cuh"

namespace bk {

// 1/sqrt(mean(x^2) + eps) of x[0..cols). `red` is shared scratch of >= 32 doubles.
__device__ __forceinline__ float cta_rms_scale(const float* x, uint32_t cols, float eps, double* red) {
    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, warps = blockDim.x >> 5;
    double part = 0.0;
    for (uint32_t i = tid; i < cols; i += blockDim.x) {
        const float v = x[i];
        part += double(__fmul_rn(v, v));
    }
    part = warp_sum(part);
    __syncthreads();  // red may still be read by a previous call
    if (lane == 0) red[warp] = part;
    __syncthreads();
    double total = 0.0;
    for (uint32_t w = 0; w < warps; ++w) total += red[w];
    const float mean = float(total / double(cols));
    return __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(mean, eps)));
}

// row[0..cols) -> q (int8), d (f16-rounded scale widened to f32), s (sum of the block's q). ONE LANE PER BLOCK: each
// lane reads its 32 values (as eight float4, in an order rotated by the lane so that the quarter-warps hit distinct
// shared-memory banks), takes the maximum, divides once, converts and packs. No shuffles - on this GPU a warp shuffle
// issues at a quarter of the ALU rate, and the reduction-per-block form spent most of its time in them - and no
// redundant divisions. `row` must be 16-byte aligned.
__device__ __forceinline__ void cta_quantize_q8_0(const float* row, uint32_t cols, int8_t* q, float* d, int32_t* s) {
    const uint32_t nb = cols / 32;
    const float4* row4 = reinterpret_cast<const float4*>(row);
    uint32_t* q4 = reinterpret_cast<uint32_t*>(q);
    for (uint32_t b = threadIdx.x; b < nb; b += blockDim.x) {
        const uint32_t rot = threadIdx.x & 7;
        float4 v[8];
        float amax = 0.0f;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            v[i] = row4[b * 8 + ((i + rot) & 7)];
            amax = fmaxf(amax, fmaxf(fmaxf(fabsf(v[i].x), fabsf(v[i].y)), fmaxf(fabsf(v[i].z), fabsf(v[i].w))));
        }
        const float dd = __fdiv_rn(amax, 127.0f);
        const float inv = dd != 0.0f ? __fdiv_rn(1.0f, dd) : 0.0f;
        int sum = 0;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int q0 = __float2int_rn(__fmul_rn(v[i].x, inv)), q1 = __float2int_rn(__fmul_rn(v[i].y, inv));
            const int q2 = __float2int_rn(__fmul_rn(v[i].z, inv)), q3 = __float2int_rn(__fmul_rn(v[i].w, inv));
            sum += q0 + q1 + q2 + q3;
            q4[b * 8 + ((i + rot) & 7)] = uint32_t(q0 & 0xFF) | (uint32_t(q1 & 0xFF) << 8) | (uint32_t(q2 & 0xFF) << 16) | (uint32_t(q3 & 0xFF) << 24);
        }
        d[b] = __half2float(__float2half_rn(dd));
        s[b] = sum;
    }
}

// row[0..cols) -> qk (int8), dk (f32 scale per 256), bs (int16 sums of 16). One warp per 256-value super-block.
__device__ __forceinline__ void cta_quantize_q8_k(const float* row, uint32_t cols, int8_t* qk, float* dk, int16_t* bs) {
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    const uint32_t nb = cols / 256;
    for (uint32_t b = warp; b < nb; b += warps) {
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
        int8_t* qo = qk + b * 256 + lane * 8;
        if (amax == 0.0f) {
            *reinterpret_cast<uint2*>(qo) = make_uint2(0u, 0u);
            if ((lane & 1) == 0) bs[b * 16 + (lane >> 1)] = 0;
            if (lane == 0) dk[b] = 0.0f;
            continue;
        }
        const float inv = __fdiv_rn(-127.0f, ext);
        uint32_t w[2] = {0u, 0u};
        int sum = 0;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int qi = int(fminf(127.0f, rintf(__fmul_rn(inv, vals[i]))));
            sum += qi;
            w[i >> 2] |= uint32_t(uint8_t(int8_t(qi))) << (8 * (i & 3));
        }
        *reinterpret_cast<uint2*>(qo) = make_uint2(w[0], w[1]);
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
        if ((lane & 1) == 0) bs[b * 16 + (lane >> 1)] = int16_t(sum);
        if (lane == 0) dk[b] = __fdiv_rn(1.0f, inv);
    }
}

}  // namespace bk
