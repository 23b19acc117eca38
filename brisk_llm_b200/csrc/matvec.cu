// Streaming multiply: a few token rows (1..8) against whole weight matrices, HBM-bound.
//
// One warp owns RW consecutive weight rows and walks their 16-byte units with lane stride, so each
// load instruction of a warp covers 512 contiguous bytes of a row and every lane keeps RW independent
// 16-byte loads in flight. The arithmetic is the reference's (src/quant.cpp:445-596): integer dot per
// block against Q8_0/Q8_K activations, one f32 scaling per block, f32 sum over blocks IN BLOCK ORDER.
// Integer partial sums of lanes that share a block are combined with shuffles before the conversion to
// float, so each block's term is the float the CPU computes; the 32 terms a warp produces per step are
// then transposed through shared memory so that one lane per (row, token) adds them one after the other,
// continuing its running sum - the same sequence of roundings as the CPU's loop. Results are therefore
// bit-identical to the reference's generic kernels, which matters because the next step re-quantises
// them to 8 bits: a 1-ulp difference occasionally flips a rounding there and the flip then spreads.
// (F16/F32 matrices - the output head of the ternary model - use lane-partial sums and a tree: their
// results feed only the arg-max or the sampler, never another quantisation.)
#include <type_traits>

#include "exact_math.h"
#include "kernels.h"

namespace bk {
namespace {

constexpr int kWarps = 8;  // warps per CTA

struct Params {
    DevMatrix m[3];
    float* out[3];
    uint32_t ldo[3];
    uint32_t first_group[4];  // prefix sums of row groups per target
    int count;
    int epi;
    DevAct act;
    uint32_t tok0, ntok;  // tokens [tok0, tok0 + ntok) of act
};

__device__ __forceinline__ int dp4a(uint32_t a, uint32_t b, int c) { return __dp4a(int(a), int(b), c); }

// ---- per-format unit arithmetic -------------------------------------------------------------------------
// Each format provides: W (a unit's weights in registers), X (the matching activations of one token),
// loadw / loadx, and term(): the f32 contribution of the unit, already including every scale. term() may
// shuffle, so all 32 lanes call it together; `valid` masks lanes past the row end.

struct FQ4_0 {
    static constexpr int kLanesPerTerm = 1;
    static constexpr bool kExact = true;
    struct W { uint4 q; float d; };
    struct X { uint4 lo, hi; float d; int s; };
    static __device__ __forceinline__ W loadw(const DevMatrix& m, uint32_t row, uint32_t u) {
        const size_t i = size_t(row) * m.units + u;
        return {ld_stream(m.qa + i * 16), __half2float(m.d[i])};
    }
    static __device__ __forceinline__ X loadx(const DevAct& a, uint32_t t, uint32_t u) {
        const uint4* p = reinterpret_cast<const uint4*>(a.q0 + size_t(t) * a.cols + u * 32);
        const size_t b = size_t(t) * (a.cols / 32) + u;
        return {p[0], p[1], a.d0[b], a.s0[b]};
    }
    static __device__ __forceinline__ float term(const W& w, const X& x, bool valid, uint32_t) {
        int acc = 0;
        acc = dp4a(w.q.x & 0x0F0F0F0Fu, x.lo.x, acc);
        acc = dp4a(w.q.y & 0x0F0F0F0Fu, x.lo.y, acc);
        acc = dp4a(w.q.z & 0x0F0F0F0Fu, x.lo.z, acc);
        acc = dp4a(w.q.w & 0x0F0F0F0Fu, x.lo.w, acc);
        acc = dp4a((w.q.x >> 4) & 0x0F0F0F0Fu, x.hi.x, acc);
        acc = dp4a((w.q.y >> 4) & 0x0F0F0F0Fu, x.hi.y, acc);
        acc = dp4a((w.q.z >> 4) & 0x0F0F0F0Fu, x.hi.z, acc);
        acc = dp4a((w.q.w >> 4) & 0x0F0F0F0Fu, x.hi.w, acc);
        acc -= 8 * x.s;  // sum((q-8)*x) = sum(q*x) - 8*sum(x)
        return valid ? __fmul_rn(__fmul_rn(float(acc), w.d), x.d) : 0.0f;
    }
};

struct FQ8_0 {
    static constexpr int kLanesPerTerm = 2;
    static constexpr bool kExact = true;
    struct W { uint4 q; float d; };
    struct X { uint4 q; float d; };
    static __device__ __forceinline__ W loadw(const DevMatrix& m, uint32_t row, uint32_t u) {
        const size_t i = size_t(row) * m.units + u;
        return {ld_stream(m.qa + i * 16), __half2float(m.d[size_t(row) * m.blocks + (u >> 1)])};
    }
    static __device__ __forceinline__ X loadx(const DevAct& a, uint32_t t, uint32_t u) {
        return {*reinterpret_cast<const uint4*>(a.q0 + size_t(t) * a.cols + u * 16), a.d0[size_t(t) * (a.cols / 32) + (u >> 1)]};
    }
    static __device__ __forceinline__ float term(const W& w, const X& x, bool valid, uint32_t u) {
        int acc = 0;
        acc = dp4a(w.q.x, x.q.x, acc);
        acc = dp4a(w.q.y, x.q.y, acc);
        acc = dp4a(w.q.z, x.q.z, acc);
        acc = dp4a(w.q.w, x.q.w, acc);
        acc = valid ? acc : 0;
        acc += __shfl_xor_sync(0xffffffffu, acc, 1);  // the block's other half
        return (valid && (u & 1) == 0) ? __fmul_rn(__fmul_rn(float(acc), w.d), x.d) : 0.0f;
    }
};

struct FQ4_K {
    static constexpr int kLanesPerTerm = 8;
    static constexpr bool kExact = true;
    struct W { uint4 q; uint32_t sc0, sc1, mn0, mn1; float d, dmin; };
    struct X { uint4 lo, hi; float d; int bs0, bs1; };
    static __device__ __forceinline__ W loadw(const DevMatrix& m, uint32_t row, uint32_t u) {
        const size_t i = size_t(row) * m.units + u;
        const size_t blk = size_t(row) * m.blocks + (u >> 3);
        const uint32_t g = (u & 7) >> 1;
        const uint8_t* s = m.sc + blk * 16;
        const __half2 dd = reinterpret_cast<const __half2*>(m.d)[blk];
        return {ld_stream(m.qa + i * 16), s[2 * g], s[2 * g + 1], s[8 + 2 * g], s[9 + 2 * g], __low2float(dd), __high2float(dd)};
    }
    static __device__ __forceinline__ X loadx(const DevAct& a, uint32_t t, uint32_t u) {
        const uint32_t sb = u >> 3, j = u & 7, g = j >> 1, hf = j & 1;
        const int8_t* base = a.qk + size_t(t) * a.cols + sb * 256 + g * 64 + hf * 16;
        const int16_t* bs = a.bs + size_t(t) * (a.cols / 16) + sb * 16 + 4 * g + hf;
        return {*reinterpret_cast<const uint4*>(base), *reinterpret_cast<const uint4*>(base + 32), a.dk[size_t(t) * (a.cols / 256) + sb], bs[0], bs[2]};
    }
    static __device__ __forceinline__ float term(const W& w, const X& x, bool valid, uint32_t u) {
        int lo = 0, hi = 0;
        lo = dp4a(w.q.x & 0x0F0F0F0Fu, x.lo.x, lo);
        lo = dp4a(w.q.y & 0x0F0F0F0Fu, x.lo.y, lo);
        lo = dp4a(w.q.z & 0x0F0F0F0Fu, x.lo.z, lo);
        lo = dp4a(w.q.w & 0x0F0F0F0Fu, x.lo.w, lo);
        hi = dp4a((w.q.x >> 4) & 0x0F0F0F0Fu, x.hi.x, hi);
        hi = dp4a((w.q.y >> 4) & 0x0F0F0F0Fu, x.hi.y, hi);
        hi = dp4a((w.q.z >> 4) & 0x0F0F0F0Fu, x.hi.z, hi);
        hi = dp4a((w.q.w >> 4) & 0x0F0F0F0Fu, x.hi.w, hi);
        int weighted = valid ? int(w.sc0) * lo + int(w.sc1) * hi : 0;
        int offsets = valid ? int(w.mn0) * x.bs0 + int(w.mn1) * x.bs1 : 0;
#pragma unroll
        for (int o = 1; o < 8; o <<= 1) {  // the super-block's 8 units sit in 8 neighbouring lanes
            weighted += __shfl_xor_sync(0xffffffffu, weighted, o);
            offsets += __shfl_xor_sync(0xffffffffu, offsets, o);
        }
        if (!valid || (u & 7) != 0) return 0.0f;
        return __fmul_rn(x.d, __fsub_rn(__fmul_rn(w.d, float(weighted)), __fmul_rn(w.dmin, float(offsets))));
    }
};

struct FQ6_K {
    static constexpr int kLanesPerTerm = 4;
    static constexpr bool kExact = true;
    struct W { uint4 a, b, c; int sc[4]; float d; };
    struct X { uint4 q[4]; float d; int bs[4]; };
    static __device__ __forceinline__ W loadw(const DevMatrix& m, uint32_t row, uint32_t u) {
        const size_t i = size_t(row) * m.units + u;
        const size_t blk = size_t(row) * m.blocks + (u >> 2);
        const uint32_t c = u & 3;
        const int8_t* s = reinterpret_cast<const int8_t*>(m.sc) + blk * 16 + (c >> 1) * 8 + (c & 1);
        W w;
        w.a = ld_stream(m.qa + i * 16);
        w.b = ld_stream(m.qb + i * 16);
        w.c = ld_stream(m.qc + i * 16);
#pragma unroll
        for (int k = 0; k < 4; ++k) w.sc[k] = s[2 * k];
        w.d = __half2float(m.d[blk]);
        return w;
    }
    static __device__ __forceinline__ X loadx(const DevAct& a, uint32_t t, uint32_t u) {
        const uint32_t sb = u >> 2, c = u & 3;
        const int8_t* base = a.qk + size_t(t) * a.cols + sb * 256 + (c >> 1) * 128 + (c & 1) * 16;
        const int16_t* bs = a.bs + size_t(t) * (a.cols / 16) + sb * 16 + (c >> 1) * 8 + (c & 1);
        X x;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            x.q[k] = *reinterpret_cast<const uint4*>(base + 32 * k);
            x.bs[k] = bs[2 * k];
        }
        x.d = a.dk[size_t(t) * (a.cols / 256) + sb];
        return x;
    }
    static __device__ __forceinline__ int group(uint4 v, uint4 x) {
        int acc = 0;
        acc = dp4a(v.x, x.x, acc);
        acc = dp4a(v.y, x.y, acc);
        acc = dp4a(v.z, x.z, acc);
        acc = dp4a(v.w, x.w, acc);
        return acc;
    }
    static __device__ __forceinline__ uint32_t join(uint32_t low, uint32_t high2) { return low | high2; }
    static __device__ __forceinline__ float term(const W& w, const X& x, bool valid, uint32_t u) {
        const uint32_t L = 0x0F0F0F0Fu, H = 0x30303030u;
        uint4 v0 = make_uint4((w.a.x & L) | ((w.c.x << 4) & H), (w.a.y & L) | ((w.c.y << 4) & H), (w.a.z & L) | ((w.c.z << 4) & H), (w.a.w & L) | ((w.c.w << 4) & H));
        uint4 v1 = make_uint4((w.b.x & L) | ((w.c.x << 2) & H), (w.b.y & L) | ((w.c.y << 2) & H), (w.b.z & L) | ((w.c.z << 2) & H), (w.b.w & L) | ((w.c.w << 2) & H));
        uint4 v2 = make_uint4(((w.a.x >> 4) & L) | (w.c.x & H), ((w.a.y >> 4) & L) | (w.c.y & H), ((w.a.z >> 4) & L) | (w.c.z & H), ((w.a.w >> 4) & L) | (w.c.w & H));
        uint4 v3 = make_uint4(((w.b.x >> 4) & L) | ((w.c.x >> 2) & H), ((w.b.y >> 4) & L) | ((w.c.y >> 2) & H), ((w.b.z >> 4) & L) | ((w.c.z >> 2) & H), ((w.b.w >> 4) & L) | ((w.c.w >> 2) & H));
        int weighted = 0;
        weighted += w.sc[0] * (group(v0, x.q[0]) - 32 * x.bs[0]);  // (q - 32) * x summed = q*x - 32*sum(x)
        weighted += w.sc[1] * (group(v1, x.q[1]) - 32 * x.bs[1]);
        weighted += w.sc[2] * (group(v2, x.q[2]) - 32 * x.bs[2]);
        weighted += w.sc[3] * (group(v3, x.q[3]) - 32 * x.bs[3]);
        weighted = valid ? weighted : 0;
        weighted += __shfl_xor_sync(0xffffffffu, weighted, 1);
        weighted += __shfl_xor_sync(0xffffffffu, weighted, 2);
        if (!valid || (u & 3) != 0) return 0.0f;
        return __fmul_rn(__fmul_rn(x.d, w.d), float(weighted));
    }
};

struct FTQ2_0 {
    static constexpr int kLanesPerTerm = 4;
    static constexpr bool kExact = true;
    struct W { uint4 q; float d; };
    struct X { uint4 q[4]; float d; int bsum; };
    static __device__ __forceinline__ W loadw(const DevMatrix& m, uint32_t row, uint32_t u) {
        const size_t i = size_t(row) * m.units + u;
        return {ld_stream(m.qa + i * 16), __half2float(m.d[size_t(row) * m.blocks + (u >> 2)])};
    }
    static __device__ __forceinline__ X loadx(const DevAct& a, uint32_t t, uint32_t u) {
        const uint32_t sb = u >> 2, c = u & 3;
        const int8_t* base = a.qk + size_t(t) * a.cols + sb * 256 + (c >> 1) * 128 + (c & 1) * 16;
        const int16_t* bs = a.bs + size_t(t) * (a.cols / 16) + sb * 16 + (c >> 1) * 8 + (c & 1);
        X x;
        x.bsum = 0;
#pragma unroll
        for (int l = 0; l < 4; ++l) {
            x.q[l] = *reinterpret_cast<const uint4*>(base + 32 * l);
            x.bsum += bs[2 * l];
        }
        x.d = a.dk[size_t(t) * (a.cols / 256) + sb];
        return x;
    }
    static __device__ __forceinline__ float term(const W& w, const X& x, bool valid, uint32_t u) {
        const uint32_t M = 0x03030303u;
        int acc = 0;
#pragma unroll
        for (int l = 0; l < 4; ++l) {
            acc = dp4a((w.q.x >> (2 * l)) & M, x.q[l].x, acc);
            acc = dp4a((w.q.y >> (2 * l)) & M, x.q[l].y, acc);
            acc = dp4a((w.q.z >> (2 * l)) & M, x.q[l].z, acc);
            acc = dp4a((w.q.w >> (2 * l)) & M, x.q[l].w, acc);
        }
        acc = valid ? acc - x.bsum : 0;  // sum((q-1)*x) = sum(q*x) - sum(x)
        acc += __shfl_xor_sync(0xffffffffu, acc, 1);
        acc += __shfl_xor_sync(0xffffffffu, acc, 2);
        if (!valid || (u & 3) != 0) return 0.0f;
        return __fmul_rn(__fmul_rn(x.d, w.d), float(acc));
    }
};

// Unquantised weights against raw f32 activations (the reference's dot_f32 path for widened F16 tensors).
struct FF16 {
    static constexpr int kLanesPerTerm = 1;
    static constexpr bool kExact = false;
    struct W { uint4 q; };
    struct X { float4 a, b; };
    static __device__ __forceinline__ W loadw(const DevMatrix& m, uint32_t row, uint32_t u) {
        return {ld_stream(m.qa + (size_t(row) * m.units + u) * 16)};
    }
    static __device__ __forceinline__ X loadx(const DevAct& a, uint32_t t, uint32_t u) {
        const float4* p = reinterpret_cast<const float4*>(a.f32 + size_t(t) * a.cols + u * 8);
        return {p[0], p[1]};
    }
    static __device__ __forceinline__ float term(const W& w, const X& x, bool valid, uint32_t) {
        const __half2* h = reinterpret_cast<const __half2*>(&w.q);
        const float2 f0 = __half22float2(h[0]), f1 = __half22float2(h[1]), f2 = __half22float2(h[2]), f3 = __half22float2(h[3]);
        float s = __fmul_rn(f0.x, x.a.x);
        s = fmaf(f0.y, x.a.y, s);
        s = fmaf(f1.x, x.a.z, s);
        s = fmaf(f1.y, x.a.w, s);
        s = fmaf(f2.x, x.b.x, s);
        s = fmaf(f2.y, x.b.y, s);
        s = fmaf(f3.x, x.b.z, s);
        s = fmaf(f3.y, x.b.w, s);
        return valid ? s : 0.0f;
    }
};

struct FF32 {
    static constexpr int kLanesPerTerm = 1;
    static constexpr bool kExact = false;
    struct W { float4 q; };
    struct X { float4 a; };
    static __device__ __forceinline__ W loadw(const DevMatrix& m, uint32_t row, uint32_t u) {
        const uint4 v = ld_stream(m.qa + (size_t(row) * m.units + u) * 16);
        return {make_float4(__uint_as_float(v.x), __uint_as_float(v.y), __uint_as_float(v.z), __uint_as_float(v.w))};
    }
    static __device__ __forceinline__ X loadx(const DevAct& a, uint32_t t, uint32_t u) {
        return {*reinterpret_cast<const float4*>(a.f32 + size_t(t) * a.cols + u * 4)};
    }
    static __device__ __forceinline__ float term(const W& w, const X& x, bool valid, uint32_t) {
        float s = __fmul_rn(w.q.x, x.a.x);
        s = fmaf(w.q.y, x.a.y, s);
        s = fmaf(w.q.z, x.a.z, s);
        s = fmaf(w.q.w, x.a.w, s);
        return valid ? s : 0.0f;
    }
};

__device__ __forceinline__ float silu_mul(float g, float u) {
    // gate / (1 + exp(-gate)) * up, as silu_mul_f32 (src/kernels_f32.cpp:287-289)
    return __fmul_rn(__fdiv_rn(g, __fadd_rn(1.0f, exact_expf(-g))), u);
}
__device__ __forceinline__ float relu2_mul(float g, float u) {
    const float r = fmaxf(g, 0.0f);  // src/model.cpp:1135-1138
    return __fmul_rn(__fmul_rn(r, r), u);
}

// RW rows of one matrix (or, for the pair epilogues, RW rows of gate and the same RW rows of up) times NTOK tokens.
// A "chain" is one output's running sum; chain c = (matrix a, row r, token t) lives in lane c.
template <class F, int NTOK, int RW, bool PAIR>
__global__ void __launch_bounds__(kWarps * 32) matvec_kernel(const Params p) {
    constexpr int MATS = PAIR ? 2 : 1;
    constexpr int CHAINS = MATS * RW * NTOK;
    static_assert(CHAINS <= 32, "one lane per chain");
    __shared__ float tile[F::kExact ? kWarps : 1][F::kExact ? CHAINS : 1][33];

    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t group = blockIdx.x * kWarps + warp;
    if (group >= p.first_group[PAIR ? 1 : p.count]) return;
    int target = 0;
    if (!PAIR) {
        while (target + 1 < p.count && group >= p.first_group[target + 1]) ++target;
    }
    const DevMatrix& m = p.m[target];
    const uint32_t row0 = (group - p.first_group[target]) * RW;

    float acc[MATS][RW][NTOK];  // lane-partial sums (inexact formats only)
#pragma unroll
    for (int a = 0; a < MATS; ++a)
#pragma unroll
        for (int r = 0; r < RW; ++r)
#pragma unroll
            for (int t = 0; t < NTOK; ++t) acc[a][r][t] = 0.0f;
    float run = 0.0f;  // this lane's chain (exact formats)

    const uint32_t units = m.units;
    for (uint32_t u0 = 0; u0 < units; u0 += 32) {
        const uint32_t u = u0 + lane;
        const bool valid = u < units;
        const uint32_t uu = valid ? u : 0;
        typename F::W w[MATS][RW];
#pragma unroll
        for (int a = 0; a < MATS; ++a)
#pragma unroll
            for (int r = 0; r < RW; ++r) w[a][r] = F::loadw(p.m[PAIR ? a : target], min(row0 + r, m.rows - 1), uu);
#pragma unroll
        for (int t = 0; t < NTOK; ++t) {
            if (t < int(p.ntok)) {
                const typename F::X x = F::loadx(p.act, p.tok0 + t, uu);
#pragma unroll
                for (int a = 0; a < MATS; ++a)
#pragma unroll
                    for (int r = 0; r < RW; ++r) {
                        const float term = F::term(w[a][r], x, valid, uu);
                        if constexpr (F::kExact) tile[warp][(a * RW + r) * NTOK + t][lane] = term;
                        else acc[a][r][t] = __fadd_rn(acc[a][r][t], term);
                    }
            }
        }
        if constexpr (F::kExact) {
            __syncwarp();
            if (lane < CHAINS) {
                const int cnt = int(min(32u, units - u0));
                const float* mine = tile[warp][lane];
#pragma unroll 8
                for (int j = 0; j < cnt; j += F::kLanesPerTerm) run = __fadd_rn(run, mine[j]);
            }
            __syncwarp();
        }
    }

    if constexpr (F::kExact) {
        // lane c holds chain c; for a pair the up value of the same (row, token) sits RW*NTOK lanes further.
        const float other = PAIR ? __shfl_down_sync(0xffffffffu, run, (RW * NTOK) & 31) : 0.0f;
        if (lane < RW * NTOK) {
            const uint32_t r = lane / NTOK, t = lane % NTOK;
            if (t < p.ntok && row0 + r < m.rows) {
                float* o = p.out[PAIR ? 0 : target] + size_t(p.tok0 + t) * p.ldo[PAIR ? 0 : target] + row0 + r;
                if (PAIR) *o = p.epi == EPI_SILU_MUL ? silu_mul(run, other) : relu2_mul(run, other);
                else if (p.epi == EPI_ADD) *o = __fadd_rn(*o, run);
                else *o = run;
            }
        }
    } else {
#pragma unroll
        for (int r = 0; r < RW; ++r) {
#pragma unroll
            for (int t = 0; t < NTOK; ++t) {
                const float v0 = warp_sum(acc[0][r][t]);
                const float v1 = PAIR ? warp_sum(acc[MATS - 1][r][t]) : 0.0f;
                if (lane == 0 && t < int(p.ntok) && row0 + r < m.rows) {
                    float* o = p.out[PAIR ? 0 : target] + size_t(p.tok0 + t) * p.ldo[PAIR ? 0 : target] + row0 + r;
                    if (PAIR) *o = p.epi == EPI_SILU_MUL ? silu_mul(v0, v1) : relu2_mul(v0, v1);
                    else if (p.epi == EPI_ADD) *o = __fadd_rn(*o, v0);
                    else *o = v0;
                }
            }
        }
    }
}

template <class F, int NTOK, int RW, bool PAIR>
void launch_one(const Params& p, uint32_t groups, cudaStream_t s) {
    const unsigned grid = (groups + kWarps - 1) / kWarps;
    matvec_kernel<F, NTOK, RW, PAIR><<<grid, kWarps * 32, 0, s>>>(p);
}

// Rows per warp: as many as keep one lane per chain (<= 32 chains) and divide every target's row count.
//   1 token : 8 | 4 | 1        2-4 tokens: 4 | 1        5-8 tokens: 4 (pair: 2) | 1
template <class F, bool PAIR>
void dispatch_tile(Params& p, cudaStream_t s) {
    auto divides = [&](uint32_t rw) {
        for (int i = 0; i < p.count; ++i)
            if (p.m[i].rows % rw != 0) return false;
        return true;
    };
    auto groups_for = [&](uint32_t rw) {
        uint32_t groups = 0;
        const int targets = PAIR ? 1 : p.count;
        for (int i = 0; i < targets; ++i) {
            p.first_group[i] = groups;
            groups += (p.m[i].rows + rw - 1) / rw;
        }
        p.first_group[targets] = groups;
        return groups;
    };
    constexpr bool heavy = std::is_same_v<F, FQ6_K>;  // many registers per row: cap the rows per warp
    if (p.ntok == 1) {
        if (!heavy && divides(8)) launch_one<F, 1, 8, PAIR>(p, groups_for(8), s);
        else if (divides(4)) launch_one<F, 1, 4, PAIR>(p, groups_for(4), s);
        else launch_one<F, 1, 1, PAIR>(p, groups_for(1), s);
    } else if (p.ntok <= 4) {
        if (divides(4)) launch_one<F, 4, 4, PAIR>(p, groups_for(4), s);
        else launch_one<F, 4, 1, PAIR>(p, groups_for(1), s);
    } else {
        constexpr int RW8 = PAIR ? 2 : 4;
        if (divides(RW8)) launch_one<F, 8, RW8, PAIR>(p, groups_for(RW8), s);
        else launch_one<F, 8, 1, PAIR>(p, groups_for(1), s);
    }
}

template <class F>
void dispatch(Params& p, bool pair, uint32_t n, cudaStream_t s) {
    for (uint32_t t0 = 0; t0 < n; t0 += kMaxSmallBatch) {
        p.tok0 = t0;
        p.ntok = n - t0 < uint32_t(kMaxSmallBatch) ? n - t0 : kMaxSmallBatch;
        if (pair) dispatch_tile<F, true>(p, s);
        else dispatch_tile<F, false>(p, s);
        BK_CUDA(cudaGetLastError());
    }
}

}  // namespace

void launch_matvec(const MatTarget* targets, int count, const DevAct& act, uint32_t n, Epilogue epi, cudaStream_t s) {
    const bool pair = epi == EPI_SILU_MUL || epi == EPI_RELU2_MUL;
    if (count < 1 || count > 3 || (pair && count != 2)) throw CudaError("cuda: launch_matvec takes 1 to 3 targets (2 for a pair)");
    Params p{};
    p.count = count;
    p.epi = epi;
    p.act = act;
    for (int i = 0; i < count; ++i) {
        if (targets[i].m.type != targets[0].m.type || targets[i].m.cols != targets[0].m.cols) {
            throw CudaError("cuda: fused multiply needs matrices of one type and input size");
        }
        p.m[i] = targets[i].m;
        p.out[i] = targets[i].out;
        p.ldo[i] = targets[i].ldo;
    }
    if (pair && targets[0].m.rows != targets[1].m.rows) throw CudaError("cuda: gate and up must have the same rows");
    switch (targets[0].m.type) {
        case T_Q4_0: dispatch<FQ4_0>(p, pair, n, s); break;
        case T_Q8_0: dispatch<FQ8_0>(p, pair, n, s); break;
        case T_Q4_K: dispatch<FQ4_K>(p, pair, n, s); break;
        case T_Q6_K: dispatch<FQ6_K>(p, pair, n, s); break;
        case T_TQ2_0: dispatch<FTQ2_0>(p, pair, n, s); break;
        case T_F16: dispatch<FF16>(p, pair, n, s); break;
        case T_F32: dispatch<FF32>(p, pair, n, s); break;
        default: throw CudaError("cuda: unsupported weight type");
    }
}

}  // namespace bk
