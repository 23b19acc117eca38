// Per-format unit arithmetic of the streaming multiply, shared by the batched-by-8 kernel (matvec.cu) and the fused
// single-token kernels (decode.cu). See DevMatrix / DevAct in common.cuh for the layouts these read.
#pragma once

#include "common.cuh"
#include "exact_math.h"

namespace bk {

__device__ __forceinline__ int dp4a(uint32_t a, uint32_t b, int c) { return __dp4a(int(a), int(b), c); }

// ---- per-format unit arithmetic -------------------------------------------------------------------------
// Each format provides: W (a unit's weights in registers), X (the matching activations of one token),
// loadw / loadx, and term(): the f32 contribution of the unit, already including every scale. term() may
// shuffle, so all 32 lanes call it together; `valid` masks lanes past the row end. loadw() only loads - scales stay
// f16 in W and are widened in term() - so that a kernel can issue a unit's loads long before it uses them without an
// arithmetic instruction on a loaded value stalling the warp in between.

struct FQ4_0 {
    static constexpr int kRegs = 5;  // 32-bit registers one unit of weights occupies (W is padded to 16-byte alignment)
    static constexpr int kLanesPerTerm = 1;
    static constexpr bool kExact = true;
    struct W { uint4 q; __half d; };
    struct X { uint4 lo, hi; float d; int s; };
    static __device__ __forceinline__ W loadw(const DevMatrix& m, uint32_t row, uint32_t u) {
        const size_t i = size_t(row) * m.units + u;
        return {ld_stream(m.qa + i * 16), m.d[i]};
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
        return valid ? __fmul_rn(__fmul_rn(float(acc), __half2float(w.d)), x.d) : 0.0f;
    }
};

// Spreads the low four bits of n into bit 4 of four bytes: the fifth bits of four 5-bit quants, ready to OR onto nibbles.
__device__ __forceinline__ uint32_t fifth_bits(uint32_t n) { return (((n & 0xFu) * 0x00204081u) & 0x01010101u) << 4; }

// weight = q * d + m (src/quant.cpp:484-498): the offset meets the activation block's sum, scaled by the activation scale first.
struct FQ4_1 {
    static constexpr int kRegs = 5;  // 32-bit registers one unit of weights occupies (W is padded to 16-byte alignment)
    static constexpr int kLanesPerTerm = 1;
    static constexpr bool kExact = true;
    struct W { uint4 q; __half2 dm; };
    using X = FQ4_0::X;
    static __device__ __forceinline__ W loadw(const DevMatrix& m, uint32_t row, uint32_t u) {
        const size_t i = size_t(row) * m.units + u;
        return {ld_stream(m.qa + i * 16), reinterpret_cast<const __half2*>(m.d)[i]};
    }
    static __device__ __forceinline__ X loadx(const DevAct& a, uint32_t t, uint32_t u) { return FQ4_0::loadx(a, t, u); }
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
        const float scaled = __fmul_rn(__fmul_rn(float(acc), __low2float(w.dm)), x.d);
        const float offset = __fmul_rn(__high2float(w.dm), __fmul_rn(x.d, float(x.s)));
        return valid ? __fadd_rn(scaled, offset) : 0.0f;
    }
};

// weight = (q - 16) * d with 5-bit q (src/quant.cpp:458-472): bit i of qh is the fifth bit of value i.
struct FQ5_0 {
    static constexpr int kRegs = 6;  // 32-bit registers one unit of weights occupies (W is padded to 16-byte alignment)
    static constexpr int kLanesPerTerm = 1;
    static constexpr bool kExact = true;
    struct W { uint4 q; uint32_t qh; __half d; };
    using X = FQ4_0::X;
    static __device__ __forceinline__ W loadw(const DevMatrix& m, uint32_t row, uint32_t u) {
        const size_t i = size_t(row) * m.units + u;
        return {ld_stream(m.qa + i * 16), reinterpret_cast<const uint32_t*>(m.qb)[i], m.d[i]};
    }
    static __device__ __forceinline__ X loadx(const DevAct& a, uint32_t t, uint32_t u) { return FQ4_0::loadx(a, t, u); }
    static __device__ __forceinline__ float term(const W& w, const X& x, bool valid, uint32_t) {
        int acc = 0;
        acc = dp4a((w.q.x & 0x0F0F0F0Fu) | fifth_bits(w.qh), x.lo.x, acc);
        acc = dp4a((w.q.y & 0x0F0F0F0Fu) | fifth_bits(w.qh >> 4), x.lo.y, acc);
        acc = dp4a((w.q.z & 0x0F0F0F0Fu) | fifth_bits(w.qh >> 8), x.lo.z, acc);
        acc = dp4a((w.q.w & 0x0F0F0F0Fu) | fifth_bits(w.qh >> 12), x.lo.w, acc);
        acc = dp4a(((w.q.x >> 4) & 0x0F0F0F0Fu) | fifth_bits(w.qh >> 16), x.hi.x, acc);
        acc = dp4a(((w.q.y >> 4) & 0x0F0F0F0Fu) | fifth_bits(w.qh >> 20), x.hi.y, acc);
        acc = dp4a(((w.q.z >> 4) & 0x0F0F0F0Fu) | fifth_bits(w.qh >> 24), x.hi.z, acc);
        acc = dp4a(((w.q.w >> 4) & 0x0F0F0F0Fu) | fifth_bits(w.qh >> 28), x.hi.w, acc);
        acc -= 16 * x.s;  // sum((q-16)*x) = sum(q*x) - 16*sum(x)
        return valid ? __fmul_rn(__fmul_rn(float(acc), __half2float(w.d)), x.d) : 0.0f;
    }
};

struct FQ8_0 {
    static constexpr int kRegs = 5;  // 32-bit registers one unit of weights occupies (W is padded to 16-byte alignment)
    static constexpr int kLanesPerTerm = 2;
    static constexpr bool kExact = true;
    struct W { uint4 q; __half d; };
    struct X { uint4 q; float d; };
    static __device__ __forceinline__ W loadw(const DevMatrix& m, uint32_t row, uint32_t u) {
        const size_t i = size_t(row) * m.units + u;
        return {ld_stream(m.qa + i * 16), m.d[size_t(row) * m.blocks + (u >> 1)]};
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
        return (valid && (u & 1) == 0) ? __fmul_rn(__fmul_rn(float(acc), __half2float(w.d)), x.d) : 0.0f;
    }
};

struct FQ4_K {
    static constexpr int kRegs = 9;  // 32-bit registers one unit of weights occupies (W is padded to 16-byte alignment)
    static constexpr int kLanesPerTerm = 8;
    static constexpr bool kExact = true;
    struct W { uint4 q; uint32_t sc0, sc1, mn0, mn1; __half2 dd; };
    struct X { uint4 lo, hi; float d; int bs0, bs1; };
    static __device__ __forceinline__ W loadw(const DevMatrix& m, uint32_t row, uint32_t u) {
        const size_t i = size_t(row) * m.units + u;
        const size_t blk = size_t(row) * m.blocks + (u >> 3);
        const uint32_t g = (u & 7) >> 1;
        const uint8_t* s = m.sc + blk * 16;
        const __half2 dd = reinterpret_cast<const __half2*>(m.d)[blk];
        return {ld_stream(m.qa + i * 16), s[2 * g], s[2 * g + 1], s[8 + 2 * g], s[9 + 2 * g], dd};
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
        return __fmul_rn(x.d, __fsub_rn(__fmul_rn(__low2float(w.dd), float(weighted)), __fmul_rn(__high2float(w.dd), float(offsets))));
    }
};

// Q4_K's arithmetic with a fifth bit per weight (src/quant.cpp:523-547).
struct FQ5_K {
    static constexpr int kRegs = 10;  // 32-bit registers one unit of weights occupies (W is padded to 16-byte alignment)
    static constexpr int kLanesPerTerm = 8;
    static constexpr bool kExact = true;
    struct W { uint4 q; uint32_t qh, sc0, sc1, mn0, mn1; __half2 dd; };
    using X = FQ4_K::X;
    static __device__ __forceinline__ W loadw(const DevMatrix& m, uint32_t row, uint32_t u) {
        const size_t i = size_t(row) * m.units + u;
        const size_t blk = size_t(row) * m.blocks + (u >> 3);
        const uint32_t g = (u & 7) >> 1;
        const uint8_t* s = m.sc + blk * 16;
        const __half2 dd = reinterpret_cast<const __half2*>(m.d)[blk];
        return {ld_stream(m.qa + i * 16), reinterpret_cast<const uint32_t*>(m.qb)[i], s[2 * g], s[2 * g + 1], s[8 + 2 * g], s[9 + 2 * g], dd};
    }
    static __device__ __forceinline__ X loadx(const DevAct& a, uint32_t t, uint32_t u) { return FQ4_K::loadx(a, t, u); }
    static __device__ __forceinline__ float term(const W& w, const X& x, bool valid, uint32_t u) {
        int lo = 0, hi = 0;
        lo = dp4a((w.q.x & 0x0F0F0F0Fu) | fifth_bits(w.qh), x.lo.x, lo);
        lo = dp4a((w.q.y & 0x0F0F0F0Fu) | fifth_bits(w.qh >> 4), x.lo.y, lo);
        lo = dp4a((w.q.z & 0x0F0F0F0Fu) | fifth_bits(w.qh >> 8), x.lo.z, lo);
        lo = dp4a((w.q.w & 0x0F0F0F0Fu) | fifth_bits(w.qh >> 12), x.lo.w, lo);
        hi = dp4a(((w.q.x >> 4) & 0x0F0F0F0Fu) | fifth_bits(w.qh >> 16), x.hi.x, hi);
        hi = dp4a(((w.q.y >> 4) & 0x0F0F0F0Fu) | fifth_bits(w.qh >> 20), x.hi.y, hi);
        hi = dp4a(((w.q.z >> 4) & 0x0F0F0F0Fu) | fifth_bits(w.qh >> 24), x.hi.z, hi);
        hi = dp4a(((w.q.w >> 4) & 0x0F0F0F0Fu) | fifth_bits(w.qh >> 28), x.hi.w, hi);
        int weighted = valid ? int(w.sc0) * lo + int(w.sc1) * hi : 0;
        int offsets = valid ? int(w.mn0) * x.bs0 + int(w.mn1) * x.bs1 : 0;
#pragma unroll
        for (int o = 1; o < 8; o <<= 1) {
            weighted += __shfl_xor_sync(0xffffffffu, weighted, o);
            offsets += __shfl_xor_sync(0xffffffffu, offsets, o);
        }
        if (!valid || (u & 7) != 0) return 0.0f;
        return __fmul_rn(x.d, __fsub_rn(__fmul_rn(__low2float(w.dd), float(weighted)), __fmul_rn(__high2float(w.dd), float(offsets))));
    }
};

struct FQ6_K {
    static constexpr int kRegs = 17;  // 32-bit registers one unit of weights occupies (W is padded to 16-byte alignment)
    static constexpr int kLanesPerTerm = 4;
    static constexpr bool kExact = true;
    struct W { uint4 a, b, c; int sc[4]; __half d; };
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
        w.d = m.d[blk];
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
        return __fmul_rn(__fmul_rn(x.d, __half2float(w.d)), float(weighted));
    }
};

struct FTQ2_0 {
    static constexpr int kRegs = 5;  // 32-bit registers one unit of weights occupies (W is padded to 16-byte alignment)
    static constexpr int kLanesPerTerm = 4;
    static constexpr bool kExact = true;
    struct W { uint4 q; __half d; };
    struct X { uint4 q[4]; float d; int bsum; };
    static __device__ __forceinline__ W loadw(const DevMatrix& m, uint32_t row, uint32_t u) {
        const size_t i = size_t(row) * m.units + u;
        return {ld_stream(m.qa + i * 16), m.d[size_t(row) * m.blocks + (u >> 2)]};
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
        return __fmul_rn(__fmul_rn(x.d, __half2float(w.d)), float(acc));
    }
};

// Unquantised weights against raw f32 activations (the reference's dot_f32 path for widened F16 tensors).
struct FF16 {
    static constexpr int kRegs = 4;  // 32-bit registers one unit of weights occupies (W is padded to 16-byte alignment)
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
    static constexpr int kRegs = 4;  // 32-bit registers one unit of weights occupies (W is padded to 16-byte alignment)
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
// tanhf as the host's C library computes it. The CPU engine calls that library's tanhf (std::tanh on a float), whose
// result is not always the correctly rounded one (glibc 2.39: 2.8 % of all inputs differ by one or two units in the last
// place), and an activation that differs in its last bit can become a different 8-bit integer in the next multiply. So
// the device computes base(|z|) = float(tanh(double(|z|))) and adds a correction from a table with one 4-bit entry per
// float in [2^-25, 22): entry = (library's bits - base's bits) + 8, filled at session creation from the device's own base
// values and the host library's results (build_tanh_table, gemma.cu). Below 2^-25 both round to z, from 22 on both to 1.
// Without a table (nullptr) the result is base itself: correct to rounding, not bit for bit with the CPU engine.
constexpr uint32_t kTanhTableLo = 0x33000000u;  // bits of 2^-25f
constexpr uint32_t kTanhTableHi = 0x41b00000u;  // bits of 22.0f
__device__ __forceinline__ float tanh_base(float az) { return float(tanh(double(az))); }
__device__ __forceinline__ float tanh_like_host(float z, const uint8_t* __restrict__ table) {
    const float az = fabsf(z);
    uint32_t bits = __float_as_uint(tanh_base(az));
    const uint32_t in = __float_as_uint(az);
    if (table != nullptr && in >= kTanhTableLo && in < kTanhTableHi) {
        const uint32_t i = in - kTanhTableLo;
        const int nibble = (__ldg(table + (i >> 1)) >> ((i & 1) * 4)) & 0xF;
        bits = uint32_t(int(bits) + nibble - 8);
    }
    return copysignf(__uint_as_float(bits), z);
}
__device__ __forceinline__ float gelu_mul(float x, float u, const uint8_t* __restrict__ tanh_table) {
    // 0.5 x (1 + tanh(sqrt(2/pi) (x + 0.044715 x^3))) * up in the scalar code's order of operations (gelu_mul_f32,
    // src/kernels_f32.cpp:291-296)
    const float cube = __fmul_rn(__fmul_rn(__fmul_rn(0.044715f, x), x), x);
    const float t = tanh_like_host(__fmul_rn(0.7978845608f, __fadd_rn(x, cube)), tanh_table);
    return __fmul_rn(__fmul_rn(__fmul_rn(0.5f, x), __fadd_rn(1.0f, t)), u);
}

}  // namespace bk
