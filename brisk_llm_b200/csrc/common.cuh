// Shared declarations of the B200 token-loop library: device-side weight and activation
// layouts, error plumbing, small device helpers. Compiled for sm_100a only, with FMA
// contraction off (-fmad=false): float expressions round where the reference CPU engine's do,
// and fused multiply-adds appear only where written as fmaf().
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <atomic>
#include <cstddef>
#include <cstdint>
#include <stdexcept>
#include <string>

namespace bk {

// ggml tensor-type ids (same numbering as include/brisk_cuda.h).
enum : int { T_F32 = 0, T_F16 = 1, T_Q4_0 = 2, T_Q4_1 = 3, T_Q5_0 = 6, T_Q8_0 = 8, T_Q4_K = 12, T_Q5_K = 13, T_Q6_K = 14, T_BF16 = 30, T_TQ2_0 = 35 };

constexpr int kMaxSmallBatch = 8;  // tokens one pass of the streaming (matvec-family) kernels covers

struct CudaError : std::runtime_error {
    using std::runtime_error::runtime_error;
};

inline void check(cudaError_t e, const char* what, const char* file, int line) {
    if (e != cudaSuccess) {
        throw CudaError(std::string("cuda: ") + what + " failed: " + cudaGetErrorString(e) + " (" + file + ":" +
                        std::to_string(line) + ")");
    }
}
#define BK_CUDA(expr) ::bk::check((expr), #expr, __FILE__, __LINE__)

// A kernel's function attributes (its opt-in to more than 48 KB of dynamic shared memory) belong to one device's
// context, and one process may hold sessions on several GPUs: first() is true once per device, for the current device.
struct DeviceOnce {
    std::atomic<bool> done[64] = {};
    bool first() {
        int device = 0;
        if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return true;
        return !done[device].exchange(true);
    }
};

// A weight matrix in HBM after the load-time repack. File blocks (18/34/66/144/210 bytes) cannot be
// read with aligned vector loads, so every format is split into planes whose elements are 16-byte
// "units" of packed quants plus separately stored scales; unit u of row r sits at index r*units+u,
// so a warp reading consecutive units of a row issues fully coalesced 16-byte loads.
//
//   Q4_0   unit = one 32-value block: qa[16 B] (file nibble order); d: f16 per block
//   Q4_1   as Q4_0;                                                 d: half2 (d, m) per block
//   Q5_0   as Q4_0; qb: the block's 32 fifth bits (one u32);        d: f16 per block
//   Q8_0   unit = half a block (16 int8);                           d: f16 per block (unit/2)
//   Q4_K   unit = 16 bytes of qs: 16 low-nibble values of sub-block 2g and 16 high-nibble values of
//          sub-block 2g+1 (g = (unit%8)/2, half (unit%2) of each); sc: 16 B per super-block =
//          8 unpacked 6-bit scales then 8 mins; d: half2 (d, dmin) per super-block
//   Q5_K   as Q4_K; qb: one u32 per unit - bits 0..15 the fifth bits of the unit's 16 low-nibble values,
//          bits 16..31 those of its 16 high-nibble values
//   Q6_K   unit = 64 values: qa/qb = the two 16-byte runs of low nibbles, qc = 16 bytes of high bit
//          pairs; 4 units per super-block; sc: 16 int8 per super-block; d: f16 per super-block
//   TQ2_0  unit = 16 bytes = 4 runs of 16 ternary values; 4 units per super-block; d: f16 per super-block
//   F16 / F32: qa = the row-major values, no other plane (BF16 files are widened to F32 at upload)
struct DevMatrix {
    int type = T_F32;
    uint32_t rows = 0, cols = 0;
    uint32_t units = 0;   // 16-byte units per row (quantised types)
    uint32_t blocks = 0;  // scale blocks per row (32-value blocks or 256-value super-blocks)
    const uint8_t* qa = nullptr;
    const uint8_t* qb = nullptr;
    const uint8_t* qc = nullptr;
    const uint8_t* sc = nullptr;
    const __half* d = nullptr;
    size_t bytes = 0;  // all planes together
};

// Quantised activations of n token rows over `cols` inputs, as the reference's Session::multiply makes
// them once per multiply (src/model.cpp:579-601), in planes instead of BlockQ8_0/BlockQ8_K structs:
//   Q8_0 family: q[n][cols] int8, d0[n][cols/32] (the f16-rounded scale, widened), s0[n][cols/32] = sum of the
//                block's q (folds Q4_0's -8 offset into one multiply per block)
//   Q8_K family: qk[n][cols] int8, dk[n][cols/256] f32, bs[n][cols/16] int16 sums of 16
// f32[n][cols] is the unquantised row (F16/F32 weights multiply it directly, src/model.cpp:641-646).
struct DevAct {
    const float* f32 = nullptr;
    const int8_t* q0 = nullptr;
    const float* d0 = nullptr;
    const int32_t* s0 = nullptr;
    const int8_t* qk = nullptr;
    const float* dk = nullptr;
    const int16_t* bs = nullptr;
    uint32_t cols = 0;
};

inline bool takes_q8_k(int type) { return type == T_Q4_K || type == T_Q5_K || type == T_Q6_K || type == T_TQ2_0; }
inline uint32_t block_elems(int type) {
    return type == T_Q4_0 || type == T_Q4_1 || type == T_Q5_0 || type == T_Q8_0 ? 32u : (type == T_F32 || type == T_F16 || type == T_BF16 ? 1u : 256u);
}
inline uint32_t block_bytes(int type) {
    switch (type) {
        case T_F32: return 4;
        case T_F16: return 2;
        case T_BF16: return 2;
        case T_Q4_0: return 18;
        case T_Q4_1: return 20;
        case T_Q5_0: return 22;
        case T_Q5_K: return 176;
        case T_Q8_0: return 34;
        case T_Q4_K: return 144;
        case T_Q6_K: return 210;
        case T_TQ2_0: return 66;
        default: return 0;
    }
}

#ifdef __CUDACC__
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ double warp_sum(double v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ int warp_sum(int v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
// 16-byte read-only load that bypasses L1 allocation: weights are streamed once per token.
__device__ __forceinline__ uint4 ld_stream(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
#endif

}  // namespace bk
