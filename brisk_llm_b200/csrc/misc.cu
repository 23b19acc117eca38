// Per-token vector kernels of the token loop: embedding lookup, per-head norm + RoPE + K/V cache write,
// split-position attention with a combine pass, and the greedy arg-max that keeps decoding on the device.
#include "kernels.h"

namespace bk {
namespace {

// ---- embedding: one token row of the embedding matrix, decoded exactly like the reference's dequantize_*
// (src/quant.cpp:196-307, :565-578; embedding_row, src/model.cpp:27-70), read from the repacked planes. ----
__global__ void embed_kernel(const DevMatrix m, const int32_t* __restrict__ tokens, float* __restrict__ hidden) {
    const uint32_t t = blockIdx.x;
    const uint32_t row = uint32_t(tokens[t]);
    float* out = hidden + size_t(t) * m.cols;
    for (uint32_t u = threadIdx.x; u < m.units; u += blockDim.x) {
        const size_t i = size_t(row) * m.units + u;
        const uint8_t* qa = m.qa + i * 16;
        switch (m.type) {
            case T_F32:
                for (int k = 0; k < 4; ++k) out[u * 4 + k] = reinterpret_cast<const float*>(qa)[k];
                break;
            case T_F16:
                for (int k = 0; k < 8; ++k) out[u * 8 + k] = __half2float(reinterpret_cast<const __half*>(qa)[k]);
                break;
            case T_Q4_0: {
                const float d = __half2float(m.d[i]);
                for (int k = 0; k < 16; ++k) {
                    out[u * 32 + k] = __fmul_rn(float(int(qa[k] & 0xF) - 8), d);
                    out[u * 32 + 16 + k] = __fmul_rn(float(int(qa[k] >> 4) - 8), d);
                }
                break;
            }
            case T_Q8_0: {
                const float d = __half2float(m.d[size_t(row) * m.blocks + (u >> 1)]);
                for (int k = 0; k < 16; ++k) out[u * 16 + k] = __fmul_rn(float(reinterpret_cast<const int8_t*>(qa)[k]), d);
                break;
            }
            case T_Q4_K: {
                const uint32_t sb = u >> 3, j = u & 7, g = j >> 1, hf = j & 1;
                const size_t blk = size_t(row) * m.blocks + sb;
                const uint8_t* s = m.sc + blk * 16;
                const float d = __half2float(m.d[2 * blk]), dmin = __half2float(m.d[2 * blk + 1]);
                const float d1 = __fmul_rn(d, float(s[2 * g])), m1 = __fmul_rn(dmin, float(s[8 + 2 * g]));
                const float d2 = __fmul_rn(d, float(s[2 * g + 1])), m2 = __fmul_rn(dmin, float(s[9 + 2 * g]));
                float* y = out + sb * 256 + g * 64 + hf * 16;
                for (int k = 0; k < 16; ++k) {
                    y[k] = __fsub_rn(__fmul_rn(d1, float(qa[k] & 0xF)), m1);
                    y[32 + k] = __fsub_rn(__fmul_rn(d2, float(qa[k] >> 4)), m2);
                }
                break;
            }
            case T_Q6_K: {
                const uint32_t sb = u >> 2, c = u & 3;
                const size_t blk = size_t(row) * m.blocks + sb;
                const uint8_t* qb = m.qb + i * 16;
                const uint8_t* qc = m.qc + i * 16;
                const int8_t* s = reinterpret_cast<const int8_t*>(m.sc) + blk * 16 + (c >> 1) * 8 + (c & 1);
                const float d = __half2float(m.d[blk]);
                float* y = out + sb * 256 + (c >> 1) * 128 + (c & 1) * 16;
                for (int k = 0; k < 16; ++k) {
                    const int q0 = int((qa[k] & 0xF) | (((qc[k] >> 0) & 3) << 4)) - 32;
                    const int q1 = int((qb[k] & 0xF) | (((qc[k] >> 2) & 3) << 4)) - 32;
                    const int q2 = int((qa[k] >> 4) | (((qc[k] >> 4) & 3) << 4)) - 32;
                    const int q3 = int((qb[k] >> 4) | (((qc[k] >> 6) & 3) << 4)) - 32;
                    y[k] = __fmul_rn(__fmul_rn(d, float(s[0])), float(q0));
                    y[32 + k] = __fmul_rn(__fmul_rn(d, float(s[2])), float(q1));
                    y[64 + k] = __fmul_rn(__fmul_rn(d, float(s[4])), float(q2));
                    y[96 + k] = __fmul_rn(__fmul_rn(d, float(s[6])), float(q3));
                }
                break;
            }
            case T_TQ2_0: {
                const uint32_t sb = u >> 2, c = u & 3;
                const float d = __half2float(m.d[size_t(row) * m.blocks + sb]);
                float* y = out + sb * 256 + (c >> 1) * 128 + (c & 1) * 16;
                for (int l = 0; l < 4; ++l)
                    for (int k = 0; k < 16; ++k) y[32 * l + k] = __fmul_rn(float(int((qa[k] >> (2 * l)) & 3) - 1), d);
                break;
            }
            default: break;
        }
    }
}

// ---- per-head RMS norm (optional) + RoPE on q and k, K/V -> f16 cache (src/model.cpp:1022-1046) ----
__global__ void __launch_bounds__(128) qk_norm_rope_store_kernel(const RopeArgs a) {
    __shared__ float head[512];
    __shared__ double red[4];
    const uint32_t t = blockIdx.x, h = blockIdx.y, tid = threadIdx.x, dim = a.dim, half = dim / 2;
    const bool is_q = h < a.heads;
    const uint32_t kvh = is_q ? 0 : h - a.heads;
    float* src = is_q ? a.q + size_t(t) * a.heads * dim + size_t(h) * dim : a.k + size_t(t) * a.kv_heads * dim + size_t(kvh) * dim;
    const float* norm = is_q ? a.q_norm : a.k_norm;
    const uint32_t pos = *a.position + t;

    for (uint32_t i = tid; i < dim; i += 128) head[i] = src[i];
    __syncthreads();
    if (norm != nullptr) {
        double part = 0.0;
        for (uint32_t i = tid; i < dim; i += 128) part += double(__fmul_rn(head[i], head[i]));
        part = warp_sum(part);
        if ((tid & 31) == 0) red[tid >> 5] = part;
        __syncthreads();
        const double total = red[0] + red[1] + red[2] + red[3];
        const float mean = float(total / double(dim));
        const float scale = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(mean, a.eps)));
        for (uint32_t i = tid; i < dim; i += 128) head[i] = __fmul_rn(__fmul_rn(head[i], scale), norm[i]);
        __syncthreads();
    }
    const float* rope = a.rope + size_t(pos) * dim;
    float out0 = 0.0f, out1 = 0.0f;
    uint32_t i0 = 0, i1 = 0;
    const bool active = tid < half;
    if (active) {
        const float c = rope[2 * tid], s = rope[2 * tid + 1];
        i0 = a.neox ? tid : 2 * tid;
        i1 = a.neox ? tid + half : 2 * tid + 1;
        const float x0 = head[i0], x1 = head[i1];
        out0 = __fsub_rn(__fmul_rn(x0, c), __fmul_rn(x1, s));
        out1 = __fadd_rn(__fmul_rn(x0, s), __fmul_rn(x1, c));
    }
    if (is_q) {
        if (active) {
            src[i0] = out0;
            src[i1] = out1;
        }
        return;
    }
    const size_t base = (size_t(kvh) * a.max_context + pos) * dim;
    if (active) {
        a.k_cache[base + i0] = __float2half_rn(out0);
        a.k_cache[base + i1] = __float2half_rn(out1);
    }
    const float* v = a.v + size_t(t) * a.kv_heads * dim + size_t(kvh) * dim;
    for (uint32_t i = tid; i < dim; i += 128) a.v_cache[base + i] = __float2half_rn(v[i]);
}

// ---- attention --------------------------------------------------------------------------------------------
// Causal attention of token t (absolute position P + t) over cached positions 0..P+t, all query heads of one
// K/V head per CTA (GQA: each cached row is read once for the group), positions split across CTAs. A warp walks
// positions with stride 4; lanes hold dim/32 values of the row, the score is a warp-shuffle dot product, and each
// (warp, head) keeps an online-softmax state (max, sum, accumulator). The reference computes softmax over the whole
// row (max, f32 exp, f64 sum, src/kernels_f32.cpp:256-284); the split form differs from it by float rounding only.
constexpr uint32_t kMaxGroup = 16;  // query heads per K/V head, at most (kMaxHeadsPerKv, src/model.h:34)

template <int VPL>  // values per lane: dim / 32
__global__ void __launch_bounds__(128) attn_partial_kernel(const AttnArgs a, uint32_t split_len, uint32_t splits) {
    const uint32_t s = blockIdx.x, kvh = blockIdx.y, t = blockIdx.z;
    const uint32_t visible = *a.position + t + 1;
    const uint32_t begin = s * split_len;
    if (begin >= visible) return;
    const uint32_t end = min(visible, begin + split_len);
    const uint32_t group = a.heads / a.kv_heads, dim = a.dim;
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;

    extern __shared__ float smem[];  // [4 warps][group][dim + 2] partial states

    const __half* kbase = a.k_cache + size_t(kvh) * a.max_context * dim;
    const __half* vbase = a.v_cache + size_t(kvh) * a.max_context * dim;

    // Heads are processed in chunks of 4 to bound registers; K/V rows of a split stay in L1/L2 across chunks.
    for (uint32_t g0 = 0; g0 < group; g0 += 4) {
        const uint32_t gn = min(4u, group - g0);
        float qv[4][VPL], acc[4][VPL], m[4], l[4];
#pragma unroll
        for (int g = 0; g < 4; ++g) {
            m[g] = -INFINITY;
            l[g] = 0.0f;
#pragma unroll
            for (int i = 0; i < VPL; ++i) {
                acc[g][i] = 0.0f;
                qv[g][i] = g < int(gn) ? a.q[size_t(t) * a.heads * dim + size_t(kvh * group + g0 + g) * dim + lane * VPL + i] : 0.0f;
            }
        }
        for (uint32_t p = begin + warp; p < end; p += 4) {
            float kf[VPL], vf[VPL];
            const __half* kr = kbase + size_t(p) * dim + lane * VPL;
            const __half* vr = vbase + size_t(p) * dim + lane * VPL;
            if constexpr (VPL == 4) {
                const uint2 kk = *reinterpret_cast<const uint2*>(kr);
                const uint2 vv = *reinterpret_cast<const uint2*>(vr);
                const float2 k0 = __half22float2(*reinterpret_cast<const __half2*>(&kk.x)), k1 = __half22float2(*reinterpret_cast<const __half2*>(&kk.y));
                const float2 v0 = __half22float2(*reinterpret_cast<const __half2*>(&vv.x)), v1 = __half22float2(*reinterpret_cast<const __half2*>(&vv.y));
                kf[0] = k0.x; kf[1] = k0.y; kf[2] = k1.x; kf[3] = k1.y;
                vf[0] = v0.x; vf[1] = v0.y; vf[2] = v1.x; vf[3] = v1.y;
            } else {
#pragma unroll
                for (int i = 0; i < VPL; ++i) {
                    kf[i] = __half2float(kr[i]);
                    vf[i] = __half2float(vr[i]);
                }
            }
#pragma unroll
            for (int g = 0; g < 4; ++g) {
                if (g < int(gn)) {
                    float dot = 0.0f;
#pragma unroll
                    for (int i = 0; i < VPL; ++i) dot = fmaf(qv[g][i], kf[i], dot);
                    dot = __fmul_rn(warp_sum(dot), a.scale);
                    const float mn = fmaxf(m[g], dot);
                    const float corr = expf(m[g] - mn);  // exp(-inf) = 0 on the first position
                    const float e = expf(dot - mn);
                    l[g] = fmaf(l[g], corr, e);
#pragma unroll
                    for (int i = 0; i < VPL; ++i) acc[g][i] = fmaf(acc[g][i], corr, __fmul_rn(e, vf[i]));
                    m[g] = mn;
                }
            }
        }
        // Merge the four warps' states, then one partial (max, sum, acc) per (token, head, split).
        for (uint32_t g = 0; g < gn; ++g) {
            float* st = smem + (size_t(warp) * 4 + g) * (dim + 2);
#pragma unroll
            for (int i = 0; i < VPL; ++i) st[lane * VPL + i] = acc[g][i];
            if (lane == 0) {
                st[dim] = m[g];
                st[dim + 1] = l[g];
            }
        }
        __syncthreads();
        for (uint32_t g = 0; g < gn; ++g) {
            const float* s0 = smem + (0 * 4 + g) * (dim + 2);
            const float* s1 = smem + (1 * 4 + g) * (dim + 2);
            const float* s2 = smem + (2 * 4 + g) * (dim + 2);
            const float* s3 = smem + (3 * 4 + g) * (dim + 2);
            const float M = fmaxf(fmaxf(s0[dim], s1[dim]), fmaxf(s2[dim], s3[dim]));
            const float c0 = expf(s0[dim] - M), c1 = expf(s1[dim] - M), c2 = expf(s2[dim] - M), c3 = expf(s3[dim] - M);
            float* o = a.partial + ((size_t(t) * a.heads + kvh * group + g0 + g) * splits + s) * (dim + 2);
            for (uint32_t i = threadIdx.x; i < dim; i += 128) o[i] = s0[i] * c0 + s1[i] * c1 + s2[i] * c2 + s3[i] * c3;
            if (threadIdx.x == 0) {
                o[dim] = M;
                o[dim + 1] = s0[dim + 1] * c0 + s1[dim + 1] * c1 + s2[dim + 1] * c2 + s3[dim + 1] * c3;
            }
        }
        __syncthreads();
    }
}

__global__ void __launch_bounds__(128) attn_combine_kernel(const AttnArgs a, uint32_t split_len, uint32_t splits) {
    const uint32_t h = blockIdx.x, t = blockIdx.y, dim = a.dim;
    const uint32_t visible = *a.position + t + 1;
    const uint32_t used = (visible + split_len - 1) / split_len;
    const float* p = a.partial + (size_t(t) * a.heads + h) * splits * (dim + 2);
    float M = -INFINITY;
    for (uint32_t s = 0; s < used; ++s) M = fmaxf(M, p[s * (dim + 2) + dim]);
    float denom = 0.0f;
    for (uint32_t s = 0; s < used; ++s) denom = fmaf(p[s * (dim + 2) + dim + 1], expf(p[s * (dim + 2) + dim] - M), denom);
    const float inv = __fdiv_rn(1.0f, denom);
    for (uint32_t i = threadIdx.x; i < dim; i += 128) {
        float v = 0.0f;
        for (uint32_t s = 0; s < used; ++s) v = fmaf(p[s * (dim + 2) + i], expf(p[s * (dim + 2) + dim] - M), v);
        a.out[size_t(t) * a.heads * dim + size_t(h) * dim + i] = __fmul_rn(v, inv);
    }
}

// ---- greedy arg-max -------------------------------------------------------------------------------------
constexpr uint32_t kArgmaxBlocks = 148;

__device__ __forceinline__ void better(float& v, int32_t& i, float ov, int32_t oi) {
    if (ov > v || (ov == v && oi < i)) {  // first maximum wins (std::max_element, src/sampler.cpp:11-13)
        v = ov;
        i = oi;
    }
}

__global__ void __launch_bounds__(256) argmax_stage1(const float* __restrict__ logits, uint32_t vocab, float* pv, int32_t* pi) {
    const uint32_t row = blockIdx.y;
    const float* x = logits + size_t(row) * vocab;
    float v = -INFINITY;
    int32_t idx = 0x7fffffff;
    for (uint32_t i = blockIdx.x * 256 + threadIdx.x; i < vocab; i += kArgmaxBlocks * 256) better(v, idx, x[i], int32_t(i));
    __shared__ float sv[8];
    __shared__ int32_t si[8];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) better(v, idx, __shfl_xor_sync(0xffffffffu, v, o), __shfl_xor_sync(0xffffffffu, idx, o));
    if ((threadIdx.x & 31) == 0) {
        sv[threadIdx.x >> 5] = v;
        si[threadIdx.x >> 5] = idx;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < 8; ++w) better(v, idx, sv[w], si[w]);
        pv[row * kArgmaxBlocks + blockIdx.x] = v;
        pi[row * kArgmaxBlocks + blockIdx.x] = idx;
    }
}

__global__ void __launch_bounds__(256) argmax_stage2(const float* pv, const int32_t* pi, int32_t* out) {
    const uint32_t row = blockIdx.x;
    float v = -INFINITY;
    int32_t idx = 0x7fffffff;
    if (threadIdx.x < kArgmaxBlocks) {
        v = pv[row * kArgmaxBlocks + threadIdx.x];
        idx = pi[row * kArgmaxBlocks + threadIdx.x];
    }
    __shared__ float sv[8];
    __shared__ int32_t si[8];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) better(v, idx, __shfl_xor_sync(0xffffffffu, v, o), __shfl_xor_sync(0xffffffffu, idx, o));
    if ((threadIdx.x & 31) == 0) {
        sv[threadIdx.x >> 5] = v;
        si[threadIdx.x >> 5] = idx;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < 8; ++w) better(v, idx, sv[w], si[w]);
        out[row] = idx;
    }
}

__global__ void advance_kernel(int32_t* token_slot, const int32_t* chosen, uint32_t* position, int32_t* history, uint32_t* history_len) {
    const int32_t tok = *chosen;
    *token_slot = tok;
    *position += 1;
    if (history != nullptr) {
        history[*history_len] = tok;
        *history_len += 1;
    }
}

}  // namespace

void launch_embed(const DevMatrix& embd, const int32_t* tokens_dev, uint32_t n, float* hidden, cudaStream_t s) {
    embed_kernel<<<n, 128, 0, s>>>(embd, tokens_dev, hidden);
    BK_CUDA(cudaGetLastError());
}

void launch_qk_norm_rope_store(const RopeArgs& a, cudaStream_t s) {
    if (a.dim > 512 || a.dim % 2 != 0) throw CudaError("cuda: head size must be even and at most 512");
    qk_norm_rope_store_kernel<<<dim3(a.n, a.heads + a.kv_heads), 128, 0, s>>>(a);
    BK_CUDA(cudaGetLastError());
}

uint32_t attn_split_len() { return 64; }

static uint32_t split_len_for(uint32_t n, uint32_t max_context) {
    if (n > uint32_t(kMaxSmallBatch)) return 256;  // prompt batches: many tokens already fill the GPU
    return max_context > 4096 ? 128 : 32;          // decode: short splits, one wave of CTAs
}

size_t attn_partial_floats(uint32_t n, uint32_t heads, uint32_t dim, uint32_t max_context) {
    const uint32_t sl = split_len_for(n, max_context);
    const uint32_t splits = (max_context + sl - 1) / sl;
    return size_t(n) * heads * splits * (dim + 2);
}

void launch_attention(const AttnArgs& a, cudaStream_t s) {
    const uint32_t group = a.heads / a.kv_heads;
    if (a.dim % 32 != 0 || a.dim > 128 || group > kMaxGroup) throw CudaError("cuda: head size must be 32, 64, 96 or 128 and at most 16 query heads per K/V head");
    const uint32_t sl = split_len_for(a.n, a.max_context);
    const uint32_t splits = (a.max_context + sl - 1) / sl;
    const uint32_t used = (a.max_visible + sl - 1) / sl;
    const dim3 grid(used, a.kv_heads, a.n);
    const size_t smem = size_t(4) * 4 * (a.dim + 2) * sizeof(float);
    switch (a.dim / 32) {
        case 1: attn_partial_kernel<1><<<grid, 128, smem, s>>>(a, sl, splits); break;
        case 2: attn_partial_kernel<2><<<grid, 128, smem, s>>>(a, sl, splits); break;
        case 3: attn_partial_kernel<3><<<grid, 128, smem, s>>>(a, sl, splits); break;
        default: attn_partial_kernel<4><<<grid, 128, smem, s>>>(a, sl, splits); break;
    }
    BK_CUDA(cudaGetLastError());
    attn_combine_kernel<<<dim3(a.heads, a.n), 128, 0, s>>>(a, sl, splits);
    BK_CUDA(cudaGetLastError());
}

size_t argmax_scratch_elems(uint32_t) { return size_t(kArgmaxBlocks) * 64; }

void launch_argmax(const float* logits, uint32_t vocab, uint32_t n, int32_t* out_token, float* scratch_val, int32_t* scratch_idx,
                   cudaStream_t s) {
    argmax_stage1<<<dim3(kArgmaxBlocks, n), 256, 0, s>>>(logits, vocab, scratch_val, scratch_idx);
    BK_CUDA(cudaGetLastError());
    argmax_stage2<<<n, 256, 0, s>>>(scratch_val, scratch_idx, out_token);
    BK_CUDA(cudaGetLastError());
}

void launch_advance(int32_t* token_slot, const int32_t* chosen, uint32_t* position, int32_t* history, uint32_t* history_len,
                    cudaStream_t s) {
    advance_kernel<<<1, 1, 0, s>>>(token_slot, chosen, position, history, history_len);
    BK_CUDA(cudaGetLastError());
}

}  // namespace bk
