// Per-token vector kernels of the token loop: embedding lookup, per-head norm + RoPE + K/V cache write,
// split-position attention with a combine pass, and the greedy arg-max that keeps decoding on the device.
#include <cstdio>
#include <mutex>
#include <string>
#include <utility>

#include "exact_math.h"
#include <cstdlib>

#include "kernels.h"

namespace bk {
namespace {

// No-op unless the kernel was launched as a programmatic dependent of its predecessor (the decode step does that).
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

template <class... Params, class... Args>
void launch_pdl(void (*kernel)(Params...), dim3 grid, dim3 block, size_t smem, cudaStream_t s, Args&&... args) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr{};
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    BK_CUDA(cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...));
}

// ---- embedding: one token row of the embedding matrix, decoded exactly like the reference's dequantize_*
// (src/quant.cpp:196-307, :565-578; embedding_row, src/model.cpp:27-70), read from the repacked planes. ----
__global__ void embed_kernel(const DevMatrix m, const int32_t* tokens, float* __restrict__ hidden) {
    pdl_wait();
    const uint32_t t = blockIdx.x;
    uint32_t row = uint32_t(tokens[t]);
    if (row >= m.rows) row = 0;  // the host checks ids it is given; an id chosen on the device is checked where it is chosen, this is the last guard
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
            case T_Q4_1: {  // dequantize_q4_1, src/quant.cpp:207-217
                const float d = __half2float(m.d[2 * i]), mm = __half2float(m.d[2 * i + 1]);
                for (int k = 0; k < 16; ++k) {
                    out[u * 32 + k] = __fadd_rn(__fmul_rn(float(qa[k] & 0xF), d), mm);
                    out[u * 32 + 16 + k] = __fadd_rn(__fmul_rn(float(qa[k] >> 4), d), mm);
                }
                break;
            }
            case T_Q5_0: {  // dequantize_q5_0, src/quant.cpp:219-232
                const float d = __half2float(m.d[i]);
                const uint32_t qh = reinterpret_cast<const uint32_t*>(m.qb)[i];
                for (int k = 0; k < 16; ++k) {
                    const int lo = int(qa[k] & 0xF) | int(((qh >> k) & 1) << 4);
                    const int hi = int(qa[k] >> 4) | int(((qh >> (k + 16)) & 1) << 4);
                    out[u * 32 + k] = __fmul_rn(float(lo - 16), d);
                    out[u * 32 + 16 + k] = __fmul_rn(float(hi - 16), d);
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
            case T_Q5_K: {  // dequantize_q5_k, src/quant.cpp:263-283
                const uint32_t sb = u >> 3, j = u & 7, g = j >> 1, hf = j & 1;
                const size_t blk = size_t(row) * m.blocks + sb;
                const uint8_t* s = m.sc + blk * 16;
                const uint32_t qh = reinterpret_cast<const uint32_t*>(m.qb)[i];
                const float d = __half2float(m.d[2 * blk]), dmin = __half2float(m.d[2 * blk + 1]);
                const float d1 = __fmul_rn(d, float(s[2 * g])), m1 = __fmul_rn(dmin, float(s[8 + 2 * g]));
                const float d2 = __fmul_rn(d, float(s[2 * g + 1])), m2 = __fmul_rn(dmin, float(s[9 + 2 * g]));
                float* y = out + sb * 256 + g * 64 + hf * 16;
                for (int k = 0; k < 16; ++k) {
                    y[k] = __fsub_rn(__fmul_rn(d1, float(int(qa[k] & 0xF) | int(((qh >> k) & 1) << 4))), m1);
                    y[32 + k] = __fsub_rn(__fmul_rn(d2, float(int(qa[k] >> 4) | int(((qh >> (16 + k)) & 1) << 4))), m2);
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
    // `half` pairs rotate: all dim / 2 of them, or (partial rotary, src/model.cpp:104-115, :1024) only the pairs within the
    // first rope_dim values - NeoX pairs (i, i + rope_dim / 2) - while the rest of the head passes through.
    const uint32_t t = blockIdx.x, h = blockIdx.y, tid = threadIdx.x, dim = a.dim, half = (a.rope_dim != 0 ? a.rope_dim : dim) / 2;
    const bool is_q = h < a.heads;
    const uint32_t kvh = is_q ? 0 : h - a.heads;
    float* src = is_q ? a.q + size_t(t) * a.heads * dim + size_t(h) * dim : a.k + size_t(t) * a.kv_heads * dim + size_t(kvh) * dim;
    const float* norm = is_q ? a.q_norm : a.k_norm;
    const uint32_t pos = *a.position + t;

    const float* bias = is_q ? a.q_bias : a.k_bias;  // add_bias before norm and RoPE (src/model.cpp:1026-1030)
    if (bias != nullptr) {
        bias += size_t(is_q ? h : kvh) * dim;
        for (uint32_t i = tid; i < dim; i += 128) head[i] = __fadd_rn(src[i], bias[i]);
    } else {
        for (uint32_t i = tid; i < dim; i += 128) head[i] = src[i];
    }
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
        for (uint32_t i = 2 * half + tid; i < dim; i += 128) src[i] = head[i];  // unrotated tail (biased / normed values)
        return;
    }
    const size_t base = (size_t(kvh) * a.max_context + pos) * dim;
    if (active) {
        a.k_cache[base + i0] = __float2half_rn(out0);
        a.k_cache[base + i1] = __float2half_rn(out1);
    }
    for (uint32_t i = 2 * half + tid; i < dim; i += 128) a.k_cache[base + i] = __float2half_rn(head[i]);
    const float* v = a.v + size_t(t) * a.kv_heads * dim + size_t(kvh) * dim;
    if (a.v_bias != nullptr) {
        const float* vb = a.v_bias + size_t(kvh) * dim;
        for (uint32_t i = tid; i < dim; i += 128) a.v_cache[base + i] = __float2half_rn(__fadd_rn(v[i], vb[i]));
    } else {
        for (uint32_t i = tid; i < dim; i += 128) a.v_cache[base + i] = __float2half_rn(v[i]);
    }
}

// ---- attention --------------------------------------------------------------------------------------------
// Causal attention of token t (absolute position P + t) over cached positions 0..P+t, in the reference's own
// order of float operations (src/model.cpp:1050-1093 over src/kernels_f32.cpp:231-284), so that the result is
// bit-identical to the CPU engine's and the 8-bit re-quantisation that follows sees the same values:
//   scores   s[p] = dot_f32(q, k_p) * scale, dot_f32 = 16 interleaved partial sums, then their sum in order
//   softmax  e[p] = expf(s[p] - max) (glibc's expf, see exact_math.h), sum in f64, p[p] = e[p] * float(1/sum)
//   output   out[i] = ((p[0]*v_0[i] + p[1]*v_1[i]) + p[2]*v_2[i]) + ...   one position after the other
// Three kernels: scores (a thread per position, all query heads of one K/V head), softmax (a CTA per row),
// weighted sum (a thread per output value, walking the positions in order).
constexpr uint32_t kMaxGroup = 16;  // query heads per K/V head, at most (kMaxHeadsPerKv, src/model.h:34)

// Tokens of a batch that share one pass over the cached K (or V) rows: 16 for long contexts (every tile re-reads all
// visible rows, so fewer, larger tiles win: measured 1436 -> 956 ms of attention in an 8192-token prefill of the 7B-class
// model), 8 for short ones (more CTAs to fill the GPU: 512-token prefill of the 0.6B-class model 50.8 k vs 49.4 k tok/s).
constexpr uint32_t kLongContext = 1024;

// grid (position chunks of 128, K/V heads, token tiles). A thread owns one cached position: it reads that K row once
// and scores it against every (token, query head) of the tile, each score in dot_f32's order.
template <int GROUP, int DIM, uint32_t kTokTile>
__global__ void __launch_bounds__(128) attn_scores_kernel(const AttnArgs a) {
    extern __shared__ float qs[];  // [kTokTile][GROUP][DIM]
    const uint32_t kvh = blockIdx.y, t0 = blockIdx.z * kTokTile;
    const uint32_t tn = min(kTokTile, a.n - t0);
    const uint32_t base_visible = *a.position + t0 + 1;        // positions the tile's first token sees
    const uint32_t last_visible = base_visible + tn - 1;       // ... and its last
    const uint32_t p = blockIdx.x * 128 + threadIdx.x;
    if (blockIdx.x * 128 >= last_visible) return;
    for (uint32_t i = threadIdx.x; i < tn * GROUP * DIM; i += 128) {
        const uint32_t j = i / (GROUP * DIM), rest = i % (GROUP * DIM);
        qs[i] = a.q[size_t(t0 + j) * a.heads * DIM + size_t(kvh) * GROUP * DIM + rest];
    }
    __syncthreads();
    if (p >= last_visible) return;
    const uint4* kr = reinterpret_cast<const uint4*>(a.k_cache + (size_t(kvh) * a.max_context + p) * DIM);
    // The K row stays in registers: widened to f32 up to 128 values; a 256-wide row is kept as packed halves (128 registers)
    // and widened sixteen values at a time where it is used.
    constexpr bool kPacked = DIM > 128;
    float kf[kPacked ? 1 : DIM];
    uint4 kraw[kPacked ? DIM / 8 : 1];
#pragma unroll
    for (int i = 0; i < DIM / 8; ++i) {
        const uint4 raw = kr[i];
        if constexpr (kPacked) {
            kraw[i] = raw;
        } else {
            const __half2* h = reinterpret_cast<const __half2*>(&raw);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float2 f = __half22float2(h[j]);
                kf[8 * i + 2 * j] = f.x;
                kf[8 * i + 2 * j + 1] = f.y;
            }
        }
    }
    for (uint32_t j = 0; j < tn; ++j) {
        if (p >= base_visible + j) continue;  // token j does not see this position
#pragma unroll
        for (int g = 0; g < GROUP; ++g) {
            const float4* q4 = reinterpret_cast<const float4*>(qs + (j * GROUP + g) * DIM);
            float lanes[16];
#pragma unroll
            for (int l = 0; l < 16; ++l) lanes[l] = 0.0f;
#pragma unroll
            for (int i = 0; i < DIM; i += 16) {
                float kk[16];
                if constexpr (kPacked) {
#pragma unroll
                    for (int u = 0; u < 2; ++u) {
                        const uint4 raw = kraw[i / 8 + u];
                        const __half2* h = reinterpret_cast<const __half2*>(&raw);
#pragma unroll
                        for (int x = 0; x < 4; ++x) {
                            const float2 f = __half22float2(h[x]);
                            kk[8 * u + 2 * x] = f.x;
                            kk[8 * u + 2 * x + 1] = f.y;
                        }
                    }
                } else {
#pragma unroll
                    for (int x = 0; x < 16; ++x) kk[x] = kf[i + x];
                }
#pragma unroll
                for (int l = 0; l < 4; ++l) {
                    const float4 q = q4[i / 4 + l];
                    lanes[4 * l + 0] = __fadd_rn(lanes[4 * l + 0], __fmul_rn(q.x, kk[4 * l + 0]));
                    lanes[4 * l + 1] = __fadd_rn(lanes[4 * l + 1], __fmul_rn(q.y, kk[4 * l + 1]));
                    lanes[4 * l + 2] = __fadd_rn(lanes[4 * l + 2], __fmul_rn(q.z, kk[4 * l + 2]));
                    lanes[4 * l + 3] = __fadd_rn(lanes[4 * l + 3], __fmul_rn(q.w, kk[4 * l + 3]));
                }
            }
            float sum = 0.0f;
#pragma unroll
            for (int l = 0; l < 16; ++l) sum = __fadd_rn(sum, lanes[l]);
            a.scores[(size_t(t0 + j) * a.heads + kvh * GROUP + g) * a.max_context + p] = __fmul_rn(sum, a.scale);
        }
    }
}

__global__ void __launch_bounds__(256) attn_softmax_kernel(const AttnArgs a) {
    const uint32_t h = blockIdx.x, t = blockIdx.y, tid = threadIdx.x;
    const uint32_t visible = *a.position + t + 1;
    // a sliding-window layer normalises over the last `window` positions only (src/model.cpp:1084-1088)
    const uint32_t start = a.window != 0 && visible > a.window ? visible - a.window : 0;
    float* s = a.scores + (size_t(t) * a.heads + h) * a.max_context;
    __shared__ float redf[8];
    __shared__ double redd[8];
    float mx = -INFINITY;
    for (uint32_t p = start + tid; p < visible; p += 256) mx = fmaxf(mx, s[p]);
    mx = warp_max(mx);
    if ((tid & 31) == 0) redf[tid >> 5] = mx;
    __syncthreads();
    mx = redf[0];
#pragma unroll
    for (int w = 1; w < 8; ++w) mx = fmaxf(mx, redf[w]);
    double part = 0.0;
    for (uint32_t p = start + tid; p < visible; p += 256) {
        const float e = exact_expf(__fsub_rn(s[p], mx));
        s[p] = e;
        part += double(e);
    }
    part = warp_sum(part);
    if ((tid & 31) == 0) redd[tid >> 5] = part;
    __syncthreads();
    double total = 0.0;
#pragma unroll
    for (int w = 0; w < 8; ++w) total += redd[w];
    const float inv = float(1.0 / total);
    for (uint32_t p = start + tid; p < visible; p += 256) s[p] = __fmul_rn(s[p], inv);
}

// grid (heads x parts, token tiles), one thread per value of the head; a 256-wide head is summed as two independent
// 128-wide parts (every output value is its own sum over the positions). V rows and the tile's probabilities are staged through
// shared memory in chunks of 64 positions, so every cached row is read once per kTokTile tokens; each thread keeps one
// accumulator per token and adds p * v position after position, as weighted_sum_f32 does.
constexpr uint32_t kWChunk = 64;

template <uint32_t kTokTile>
__global__ void __launch_bounds__(128) attn_weighted_kernel(const AttnArgs a) {
    extern __shared__ __align__(16) unsigned char wraw[];  // V chunk [kWChunk][dim] f16 | probabilities [kTokTile][kWChunk] f32
    const uint32_t parts = (a.dim + 127) / 128, dim = a.dim / parts;  // dim: the 64 or 128 values this CTA sums
    const uint32_t h = blockIdx.x / parts, doff = blockIdx.x % parts * dim, t0 = blockIdx.y * kTokTile, tid = threadIdx.x;
    const uint32_t row_shift = dim == 128 ? 4 : 3;  // 16-byte pieces per staged row: dim / 8
    const uint32_t tn = min(kTokTile, a.n - t0);
    const uint32_t kvh = h / (a.heads / a.kv_heads);
    const uint32_t base_visible = *a.position + t0 + 1, last_visible = base_visible + tn - 1;
    __half* vs = reinterpret_cast<__half*>(wraw);
    float* ws = reinterpret_cast<float*>(wraw + size_t(kWChunk) * dim * sizeof(__half));
    const __half* vbase = a.v_cache + size_t(kvh) * a.max_context * a.dim + doff;
    float acc[kTokTile];
#pragma unroll
    for (int j = 0; j < int(kTokTile); ++j) acc[j] = 0.0f;
    // Sliding-window layer: token j sums positions [start_j, visible_j) with start_j = max(0, visible_j - window), in order
    // (src/model.cpp:1085-1091). Chunks below the first token's start are skipped; chunks at or above the last token's start
    // are seen in full by every token of the tile.
    const uint32_t win = a.window;
    const uint32_t start_first = win != 0 && base_visible > win ? base_visible - win : 0;
    const uint32_t start_last = win != 0 && last_visible > win ? last_visible - win : 0;
    for (uint32_t c0 = start_first / kWChunk * kWChunk; c0 < last_visible; c0 += kWChunk) {
        const uint32_t cn = min(kWChunk, last_visible - c0);
        __syncthreads();  // the previous chunk is fully consumed
        for (uint32_t i = tid; i < cn * dim / 8; i += 128) {
            const uint32_t row = i >> row_shift, piece = i & ((1u << row_shift) - 1);
            reinterpret_cast<uint4*>(vs)[i] = *reinterpret_cast<const uint4*>(vbase + size_t(c0 + row) * a.dim + piece * 8);
        }
        for (uint32_t i = tid; i < tn * kWChunk; i += 128) {
            const uint32_t j = i / kWChunk, pp = c0 + i % kWChunk;
            const uint32_t vis = base_visible + j, st = win != 0 && vis > win ? vis - win : 0;
            ws[i] = pp < vis && pp >= st ? a.scores[(size_t(t0 + j) * a.heads + h) * a.max_context + pp] : 0.0f;
        }
        __syncthreads();
        if (tid < dim) {
            if (c0 + cn <= base_visible && c0 >= start_last && tn == kTokTile && cn % 4 == 0) {
                // Every token of the tile sees the whole chunk (all chunks but the last one or two): no causal tests, and the
                // probabilities of four positions come in one 16-byte read per token. Per token the products are still added
                // in position order.
                for (uint32_t pp = 0; pp < cn; pp += 4) {
                    const float v0 = __half2float(vs[(pp + 0) * dim + tid]), v1 = __half2float(vs[(pp + 1) * dim + tid]);
                    const float v2 = __half2float(vs[(pp + 2) * dim + tid]), v3 = __half2float(vs[(pp + 3) * dim + tid]);
#pragma unroll
                    for (int j = 0; j < int(kTokTile); ++j) {
                        const float4 w = *reinterpret_cast<const float4*>(ws + j * kWChunk + pp);
                        acc[j] = __fadd_rn(acc[j], __fmul_rn(w.x, v0));
                        acc[j] = __fadd_rn(acc[j], __fmul_rn(w.y, v1));
                        acc[j] = __fadd_rn(acc[j], __fmul_rn(w.z, v2));
                        acc[j] = __fadd_rn(acc[j], __fmul_rn(w.w, v3));
                    }
                }
            } else {
                for (uint32_t pp = 0; pp < cn; ++pp) {
                    const float v = __half2float(vs[pp * dim + tid]);
#pragma unroll
                    for (int j = 0; j < int(kTokTile); ++j) {
                        // a position past token j's causal limit must not touch its sum at all (adding 0*v could turn -0 into +0)
                        const uint32_t vis = base_visible + j, st = win != 0 && vis > win ? vis - win : 0;
                        if (c0 + pp < vis && c0 + pp >= st && j < int(tn)) acc[j] = __fadd_rn(acc[j], __fmul_rn(ws[j * kWChunk + pp], v));
                    }
                }
            }
        }
    }
    if (tid < dim) {
#pragma unroll
        for (int j = 0; j < int(kTokTile); ++j) {
            if (j < int(tn)) a.out[size_t(t0 + j) * a.heads * a.dim + size_t(h) * a.dim + doff + tid] = acc[j];
        }
    }
}

}  // namespace

// ---- greedy arg-max -------------------------------------------------------------------------------------
constexpr uint32_t kArgmaxBlocks = 148;

__device__ __forceinline__ void better(float& v, int32_t& i, float ov, int32_t oi) {
    if (ov > v || (ov == v && oi < i)) {  // first maximum wins (std::max_element, src/sampler.cpp:11-13)
        v = ov;
        i = oi;
    }
}

__global__ void __launch_bounds__(256) argmax_stage1(const float* logits, uint32_t vocab, float* pv, int32_t* pi) {
    asm volatile("griddepcontrol.wait;" ::: "memory");  // no-op unless launched as a programmatic dependent
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

// `logits`/`vocab` restate what std::max_element (src/sampler.cpp:11-13) does with NaN: a comparison with NaN is false, so
// a NaN is never chosen over the running maximum - and never displaced when it IS the running maximum, which only
// element 0 can be. A row that starts with NaN, and a row of nothing but NaN, therefore answer 0; the result is always
// an id inside the vocabulary, whatever the logits hold.
__global__ void __launch_bounds__(256) argmax_stage2(const float* pv, const int32_t* pi, const float* logits, uint32_t vocab, int32_t* out,
                                                     int32_t* token_slot, uint32_t* position, int32_t* history, uint32_t* history_len) {
    asm volatile("griddepcontrol.wait;" ::: "memory");
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
        const float first = logits[size_t(row) * vocab];
        if (first != first || uint32_t(idx) >= vocab) idx = 0;
        out[row] = idx;
        if (token_slot != nullptr) {  // feed the decode loop: next input token, next position, history
            *token_slot = idx;
            *position += 1;
            if (history != nullptr) {
                history[*history_len] = idx;
                *history_len += 1;
            }
        }
    }
}



namespace {
__global__ void tp_unpack_kernel(const float* __restrict__ gathered, float* dst, uint32_t n, uint32_t rows_l, uint32_t tp, int add) {
    const size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x;
    const size_t total = size_t(n) * rows_l * tp;
    if (i >= total) return;
    const uint32_t full = rows_l * tp;
    const uint32_t t = uint32_t(i / full), c = uint32_t(i % full);
    const uint32_t rank = c / rows_l, r = c % rows_l;
    const float v = gathered[(size_t(rank) * n + t) * rows_l + r];
    dst[i] = add ? __fadd_rn(dst[i], v) : v;
}
}  // namespace

void launch_tp_unpack(const float* gathered, float* dst, uint32_t n, uint32_t rows_l, uint32_t tp, bool add, cudaStream_t s) {
    const size_t total = size_t(n) * rows_l * tp;
    tp_unpack_kernel<<<unsigned((total + 255) / 256), 256, 0, s>>>(gathered, dst, n, rows_l, tp, add ? 1 : 0);
    BK_CUDA(cudaGetLastError());
}

void launch_embed(const DevMatrix& embd, const int32_t* tokens_dev, uint32_t n, float* hidden, cudaStream_t s) {
    launch_pdl(embed_kernel, dim3(n), dim3(128), 0, s, embd, tokens_dev, hidden);
}

void launch_qk_norm_rope_store(const RopeArgs& a, cudaStream_t s) {
    if (a.dim > 512 || a.dim % 2 != 0) throw CudaError("cuda: head size must be even and at most 512");
    qk_norm_rope_store_kernel<<<dim3(a.n, a.heads + a.kv_heads), 128, 0, s>>>(a);
    BK_CUDA(cudaGetLastError());
}

int chain_mode() {  // read at every call: the tests switch it between sessions of one process
    const char* env = std::getenv("BRISK_CUDA_CHAIN");
    return env == nullptr ? -1 : std::atoi(env) != 0 ? 1 : 0;
}

size_t attn_scratch_floats(uint32_t n, uint32_t heads, uint32_t max_context) { return size_t(n) * heads * max_context; }

void launch_attention(const AttnArgs& a, cudaStream_t s) {
    const uint32_t group = a.heads / a.kv_heads;
    if ((a.dim != 64 && a.dim != 128 && a.dim != 256) || group > kMaxGroup) throw CudaError("cuda: attention takes head sizes 64, 128 and 256 and at most 16 query heads per K/V head");
    const uint32_t tile = a.max_visible > kLongContext ? 16u : 8u;
    const uint32_t tiles = (a.n + tile - 1) / tile;
    const dim3 grid((a.max_visible + 127) / 128, a.kv_heads, tiles);
    const size_t smem = size_t(tile) * group * a.dim * sizeof(float);
#define BK_SCORES_T(G, D, T)                                                                                                                  \
    do {                                                                                                                                      \
        if (smem > 48 * 1024) BK_CUDA(cudaFuncSetAttribute(attn_scores_kernel<G, D, T>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem))); \
        attn_scores_kernel<G, D, T><<<grid, 128, smem, s>>>(a);                                                                               \
    } while (0)
#define BK_SCORES(G)                                                            \
    if (a.dim == 128) {                                                         \
        if (tile == 16) BK_SCORES_T(G, 128, 16);                                \
        else BK_SCORES_T(G, 128, 8);                                            \
    } else if (a.dim == 64) {                                                   \
        if (tile == 16) BK_SCORES_T(G, 64, 16);                                 \
        else BK_SCORES_T(G, 64, 8);                                             \
    } else {                                                                    \
        if (tile == 16) BK_SCORES_T(G, 256, 16);                                \
        else BK_SCORES_T(G, 256, 8);                                            \
    }
    switch (group) {
        case 1: BK_SCORES(1); break;
        case 2: BK_SCORES(2); break;
        case 3: BK_SCORES(3); break;
        case 4: BK_SCORES(4); break;
        case 5: BK_SCORES(5); break;
        case 6: BK_SCORES(6); break;
        case 7: BK_SCORES(7); break;
        case 8: BK_SCORES(8); break;
        default: throw CudaError("cuda: query heads per K/V head must be 1 to 8");
    }
#undef BK_SCORES
#undef BK_SCORES_T
    BK_CUDA(cudaGetLastError());
    {
        static const int sms = [] {
            int dev = 0, count = 148;
            if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&count, cudaDevAttrMultiProcessorCount, dev);
            return count;
        }();
        const int mode = chain_mode();
        if (mode != 0 && (a.n <= kChainMaxTokens || mode == 1) && attn_chain_fits(a.n, a.heads, a.kv_heads, a.dim, a.max_visible, uint32_t(sms))) {
            launch_attn_chain(a, uint32_t(sms), s);
            return;
        }
    }
    attn_softmax_kernel<<<dim3(a.heads, a.n), 256, 0, s>>>(a);
    BK_CUDA(cudaGetLastError());
    const uint32_t parts = (a.dim + 127) / 128;
    if (a.n == 1) {  // a single token (models that take these kernels for their decode steps too): no tile to share V rows with
        const size_t smem_1 = size_t(kWChunk) * (a.dim / parts) * sizeof(__half) + size_t(kWChunk) * sizeof(float);
        attn_weighted_kernel<1><<<dim3(a.heads * parts, 1), 128, smem_1, s>>>(a);
        BK_CUDA(cudaGetLastError());
        return;
    }
    const size_t smem_w = size_t(kWChunk) * (a.dim / parts) * sizeof(__half) + size_t(tile) * kWChunk * sizeof(float);
    if (tile == 16) attn_weighted_kernel<16><<<dim3(a.heads * parts, tiles), 128, smem_w, s>>>(a);
    else attn_weighted_kernel<8><<<dim3(a.heads * parts, tiles), 128, smem_w, s>>>(a);
    BK_CUDA(cudaGetLastError());
}

size_t argmax_scratch_elems(uint32_t) { return size_t(kArgmaxBlocks) * 64; }

void launch_argmax(const float* logits, uint32_t vocab, uint32_t n, int32_t* out_token, float* scratch_val, int32_t* scratch_idx,
                   cudaStream_t s) {
    argmax_stage1<<<dim3(kArgmaxBlocks, n), 256, 0, s>>>(logits, vocab, scratch_val, scratch_idx);
    BK_CUDA(cudaGetLastError());
    argmax_stage2<<<n, 256, 0, s>>>(scratch_val, scratch_idx, logits, vocab, out_token, nullptr, nullptr, nullptr, nullptr);
    BK_CUDA(cudaGetLastError());
}

void launch_argmax_advance(const float* logits, uint32_t vocab, int32_t* out_token, float* scratch_val, int32_t* scratch_idx,
                           int32_t* token_slot, uint32_t* position, int32_t* history, uint32_t* history_len, cudaStream_t s) {
    launch_pdl(argmax_stage1, dim3(kArgmaxBlocks, 1), dim3(256), 0, s, logits, vocab, scratch_val, scratch_idx);
    launch_pdl(argmax_stage2, dim3(1), dim3(256), 0, s, (const float*)scratch_val, (const int32_t*)scratch_idx, logits, vocab, out_token, token_slot,
               position, history, history_len);
}

}  // namespace bk

// ---- arg-max for callers that must not allocate ---------------------------------------------------------
// The two-stage arg-max keeps one (value, index) pair per CTA and row between its stages. The session allocates that
// scratch with cudaMalloc; this variant keeps it in the library image instead: every GPU that loads the library carries
// these 76 KB until the process exits, and in exchange the call touches no allocator at all.
namespace {
constexpr uint32_t kStaticArgmaxRows = 64;  // rows one call may reduce (the most logits rows a scoring call returns)
static __device__ __align__(256) unsigned char g_static_argmax_scratch[kStaticArgmaxRows * bk::kArgmaxBlocks * 8];
constexpr int kMaxDevices = 64;
void* g_static_argmax_address[kMaxDevices] = {};  // device address of the array, per device, filled on first use
std::once_flag g_static_argmax_once[kMaxDevices];  // host threads may make their first call on a device at the same time
cudaError_t g_static_argmax_status[kMaxDevices] = {};
}  // namespace

extern "C" int brisk_cuda_argmax_static(const float* logits, uint32_t vocab, uint32_t rows, int32_t* out_tokens, void* stream, char* err,
                                        size_t errlen) {
    auto fail = [&](const std::string& what) {
        if (err != nullptr && errlen > 0) std::snprintf(err, errlen, "%s", what.c_str());
        return -1;
    };
    if (rows == 0) return 0;
    if (logits == nullptr || out_tokens == nullptr || vocab == 0) return fail("cuda: arg-max needs logits, an output and a non-empty vocabulary");
    if (rows > kStaticArgmaxRows) {
        return fail("cuda: the allocation-free arg-max reduces at most " + std::to_string(kStaticArgmaxRows) + " rows per call, got " +
                    std::to_string(rows));
    }
    int device = -1;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) return fail(std::string("cuda: cudaGetDevice failed: ") + cudaGetErrorString(e));
    if (device < 0 || device >= kMaxDevices) return fail("cuda: device ordinal out of range");
    // In host code the array's name is only a handle; the kernels need the address it has on the current device.
    std::call_once(g_static_argmax_once[device], [device] {
        void* address = nullptr;
        g_static_argmax_status[device] = cudaGetSymbolAddress(&address, g_static_argmax_scratch);
        g_static_argmax_address[device] = address;
    });
    if (g_static_argmax_status[device] != cudaSuccess || g_static_argmax_address[device] == nullptr) {
        return fail(std::string("cuda: cudaGetSymbolAddress failed: ") + cudaGetErrorString(g_static_argmax_status[device]));
    }
    unsigned char* base = static_cast<unsigned char*>(g_static_argmax_address[device]);
    float* partial_value = reinterpret_cast<float*>(base);
    int32_t* partial_index = reinterpret_cast<int32_t*>(base + size_t(kStaticArgmaxRows) * bk::kArgmaxBlocks * 4);
    // Stage 1 writes every pair stage 2 reads for these rows, so nothing of the previous call has to be cleared.
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    bk::argmax_stage1<<<dim3(bk::kArgmaxBlocks, rows), 256, 0, s>>>(logits, vocab, partial_value, partial_index);
    bk::argmax_stage2<<<rows, 256, 0, s>>>(partial_value, partial_index, logits, vocab, out_tokens, nullptr, nullptr, nullptr, nullptr);
    e = cudaGetLastError();
    if (e != cudaSuccess) return fail(std::string("cuda: arg-max launch failed: ") + cudaGetErrorString(e));
    return 0;
}

namespace bk {


}  // namespace bk
