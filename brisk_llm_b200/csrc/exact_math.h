// Single-precision exp with the results of the C library the reference CPU engine calls (glibc's
// expf on x86-64), usable on the host and on the device.
//
// Why: the token loop re-quantises activations to 8 bits and stores K/V as f16 after every step.
// A 1-ulp difference in an exp (SiLU, softmax) occasionally flips one of those roundings, and the
// flip then spreads through the following layers until logits differ in the third digit. CUDA's
// expf is accurate to 2 ulp but not identical to glibc's, so the kernels use this restatement.
//
// Algorithm (the published table-driven exp used by glibc and ARM's optimized routines for
// float): in double precision, z = x * 32/ln2; k = round(z) by the 1.5*2^52 shift trick;
// r = z - k in [-1/2, 1/2]; 2^(k/32) = 2^(k >> 5) * T[k & 31] assembled in the exponent bits;
// 2^(r/32) by a cubic minimax polynomial; the product is rounded once to float. The table holds
// the correctly rounded doubles 2^(i/32) with i << 47 subtracted so that adding k << 47 yields the
// scaled value directly. tests/test_exact_math.py checks it bit for bit against the host libm.
#pragma once

#include <cstdint>
#include <cstring>

#if defined(__CUDACC__)
#define BK_HD __host__ __device__ __forceinline__
#else
#define BK_HD inline
#endif

namespace bk {

#define BK_EXP2_TABLE                                                                                    \
    0x3ff0000000000000ull, 0x3fefd9b0d3158574ull, 0x3fefb5586cf9890full, 0x3fef9301d0125b51ull,     \
    0x3fef72b83c7d517bull, 0x3fef54873168b9aaull, 0x3fef387a6e756238ull, 0x3fef1e9df51fdee1ull,     \
    0x3fef06fe0a31b715ull, 0x3feef1a7373aa9cbull, 0x3feedea64c123422ull, 0x3feece086061892dull,     \
    0x3feebfdad5362a27ull, 0x3feeb42b569d4f82ull, 0x3feeab07dd485429ull, 0x3feea47eb03a5585ull,     \
    0x3feea09e667f3bcdull, 0x3fee9f75e8ec5f74ull, 0x3feea11473eb0187ull, 0x3feea589994cce13ull,     \
    0x3feeace5422aa0dbull, 0x3feeb737b0cdc5e5ull, 0x3feec49182a3f090ull, 0x3feed503b23e255dull,     \
    0x3feee89f995ad3adull, 0x3feeff76f2fb5e47ull, 0x3fef199bdd85529cull, 0x3fef3720dcef9069ull,     \
    0x3fef5818dcfba487ull, 0x3fef7c97337b9b5full, 0x3fefa4afa2a490daull, 0x3fefd0765b6e4540ull      

static const uint64_t kExp2TableHost[32] = {BK_EXP2_TABLE};
#if defined(__CUDACC__)
// In global memory, read through the read-only cache: lanes of a warp look up different entries, which constant
// memory would serve one address at a time.
static __device__ const uint64_t kExp2TableDev[32] = {BK_EXP2_TABLE};
#endif

BK_HD float exact_expf(float x) {
    if (x != x) return x + x;
    if (x > 0x1.62e42ep6f) return __builtin_huge_valf();  // overflow
    if (x < -0x1.9fe368p6f) return 0.0f;                  // below the smallest subnormal
    const double n = 32.0;
    const double inv_ln2_n = 0x1.71547652b82fep+0 * n;
    const double shift = 0x1.8p52;
    const double c0 = 0x1.c6af84b912394p-5 / n / n / n, c1 = 0x1.ebfce50fac4f3p-3 / n / n, c2 = 0x1.62e42ff0c52d6p-1 / n;
#if defined(__CUDA_ARCH__)
    const double z = __dmul_rn(inv_ln2_n, double(x));
    double kd = __dadd_rn(z, shift);
    const uint64_t ki = uint64_t(__double_as_longlong(kd));
    kd = __dsub_rn(kd, shift);
    const double r = __dsub_rn(z, kd);
    const double s = __longlong_as_double((long long)(__ldg(&kExp2TableDev[ki & 31]) + (ki << 47)));
    const double p = __dadd_rn(__dmul_rn(c0, r), c1);
    const double r2 = __dmul_rn(r, r);
    double y = __dadd_rn(__dmul_rn(c2, r), 1.0);
    y = __dadd_rn(__dmul_rn(p, r2), y);
    return __double2float_rn(__dmul_rn(y, s));
#else
    const double z = inv_ln2_n * double(x);
    double kd = z + shift;
    uint64_t ki;
    std::memcpy(&ki, &kd, 8);
    kd -= shift;
    const double r = z - kd;
    const uint64_t sb = kExp2TableHost[ki & 31] + (ki << 47);
    double s;
    std::memcpy(&s, &sb, 8);
    const double p = c0 * r + c1;
    const double r2 = r * r;
    double y = c2 * r + 1.0;
    y = p * r2 + y;
    return float(y * s);
#endif
}

#if defined(__CUDACC__)
// exact_expf with the 2^(i/32) table at `table` (32 entries, e.g. a copy in shared memory: a kernel that keeps almost no L1
// would otherwise fetch the entry from L2 on every call).
__device__ __forceinline__ float exact_expf_tab(float x, const uint64_t* table) {
    if (x != x) return x + x;
    if (x > 0x1.62e42ep6f) return __builtin_huge_valf();
    if (x < -0x1.9fe368p6f) return 0.0f;
    const double n = 32.0;
    const double inv_ln2_n = 0x1.71547652b82fep+0 * n;
    const double shift = 0x1.8p52;
    const double c0 = 0x1.c6af84b912394p-5 / n / n / n, c1 = 0x1.ebfce50fac4f3p-3 / n / n, c2 = 0x1.62e42ff0c52d6p-1 / n;
    const double z = __dmul_rn(inv_ln2_n, double(x));
    double kd = __dadd_rn(z, shift);
    const uint64_t ki = uint64_t(__double_as_longlong(kd));
    kd = __dsub_rn(kd, shift);
    const double r = __dsub_rn(z, kd);
    const double s = __longlong_as_double((long long)(table[ki & 31] + (ki << 47)));
    const double p = __dadd_rn(__dmul_rn(c0, r), c1);
    const double r2 = __dmul_rn(r, r);
    double y = __dadd_rn(__dmul_rn(c2, r), 1.0);
    y = __dadd_rn(__dmul_rn(p, r2), y);
    return __double2float_rn(__dmul_rn(y, s));
}
__device__ __forceinline__ const uint64_t* exp2_table_device() { return kExp2TableDev; }
// The same value again without a branch in it (the three special cases are selected at the end), so that a caller's
// unrolled loop overlaps several of them: the double-precision operations of one exp form a single dependent chain.
__device__ __forceinline__ float exact_expf_flat(float x, const uint64_t* table) {
    const double n = 32.0;
    const double inv_ln2_n = 0x1.71547652b82fep+0 * n;
    const double shift = 0x1.8p52;
    const double c0 = 0x1.c6af84b912394p-5 / n / n / n, c1 = 0x1.ebfce50fac4f3p-3 / n / n, c2 = 0x1.62e42ff0c52d6p-1 / n;
    const bool special = !(x <= 0x1.62e42ep6f && x >= -0x1.9fe368p6f);  // NaN, overflow or underflow
    const float xs = special ? 0.0f : x;                               // keeps the table index and the shifts in range
    const double z = __dmul_rn(inv_ln2_n, double(xs));
    double kd = __dadd_rn(z, shift);
    const uint64_t ki = uint64_t(__double_as_longlong(kd));
    kd = __dsub_rn(kd, shift);
    const double r = __dsub_rn(z, kd);
    const double s = __longlong_as_double((long long)(table[ki & 31] + (ki << 47)));
    const double p = __dadd_rn(__dmul_rn(c0, r), c1);
    const double r2 = __dmul_rn(r, r);
    double y = __dadd_rn(__dmul_rn(c2, r), 1.0);
    y = __dadd_rn(__dmul_rn(p, r2), y);
    const float main_path = __double2float_rn(__dmul_rn(y, s));
    return x != x ? x + x : x > 0x1.62e42ep6f ? __builtin_huge_valf() : x < -0x1.9fe368p6f ? 0.0f : main_path;
}
#endif

}  // namespace bk
