// Batched multiply for prompt processing: int8 tensor-core MMA on Q8_0-quantised activations, with the reference's
// per-block arithmetic kept intact.
//
// For Q4_0 / Q8_0 weights the reference computes, per (row, token), sum over 32-value blocks IN ORDER of
// float(int_dot) * d_w * d_x (src/quant.cpp:445-482). Here one m16n8k32 s8 MMA yields the 16x8 integer block dots of
// a tile; each thread then scales its four results (two separate f32 multiplies) and adds them to f32 accumulators it
// alone owns, walking the blocks in order - the same sequence of roundings as the CPU, so results are bit-identical
// and the next 8-bit re-quantisation sees the same values. K is never split across threads. Q4_0's nibbles are
// widened in registers (the low nibbles of a 4-byte word are exactly the MMA fragment for k = 4t..4t+3, the high
// nibbles the fragment for k = 16+4t..) and its -8 offset is taken off the fragment once, four bytes at a time, so the
// integer block dot comes out of the MMA complete. The MMA's C operand is the constant 0x4B400000 - the bit pattern of
// the float 1.5 * 2^23 - so that each result, read as a float, is exactly 1.5 * 2^23 + dot (|dot| <= 32 * 127 * 127 <
// 2^22): one exact f32 subtraction stands in for the integer-to-float conversion and nothing is zeroed between MMAs.
//
// Tiling: CTA = 128 rows x 64 tokens, 8 warps of 32 x 32 - or, for matrices with so few rows that such tiles would leave
// half of the SMs idle, 64 rows x 64 tokens with warps of 16 x 32; weights, activations and their scales are staged through
// shared memory with cp.async, two stages of 8 blocks (256 columns). Padding of 16 bytes per row keeps the fragment
// reads bank-conflict free. The per-block rescale (5 ALU instructions per output and block) bounds the kernel, not the
// tensor pipe: that is the price of integer-exact semantics.
#include <cstdlib>
#include <cstring>

#include "kernels.h"

namespace bk {
namespace {

constexpr int GN = 64, KB = 8, GWARPS = 8;  // GM, the rows of a CTA tile, is 64 * MI (MI = 16-row MMA tiles per warp)

template <int WBYTES, int GM>  // bytes of quants per block and row: 16 (Q4_0) or 32 (Q8_0); rows of the CTA tile
struct Stage {
    static constexpr int kARow = KB * WBYTES + 16;
    static constexpr int kBRow = KB * 32 + 16;
    static constexpr int kA = GM * kARow;         // weight quants
    static constexpr int kAd = GM * KB * 2;       // weight scales (f16)
    static constexpr int kB = GN * kBRow;         // activation quants
    static constexpr int kBd = GN * KB * 4;       // activation scales (f32)
    static constexpr int kBytes = kA + kAd + kB + kBd;
};

__device__ __forceinline__ void cp_async8(void* smem, const void* gmem) {
    const uint32_t a = uint32_t(__cvta_generic_to_shared(smem));
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(a), "l"(gmem) : "memory");
}

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
    const uint32_t a = uint32_t(__cvta_generic_to_shared(smem));
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(a), "l"(gmem) : "memory");
}

constexpr int kMagicBits = 0x4B400000;     // 1.5 * 2^23 as a float
constexpr float kMagic = 12582912.0f;

// d = a x b + kMagicBits in every element
__device__ __forceinline__ void mma_s8(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
        : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(kMagicBits));
}

// Two f32 operations per instruction (packed f32x2, IEEE round-to-nearest in each half: the same results as two scalar
// instructions). Not used for the final addition: a mul.rn.f32x2 whose only use is an add.rn.f32x2 is contracted into a
// fused multiply-add by the assembler (measured), and the reference does not fuse.
using f32x2 = unsigned long long;
__device__ __forceinline__ f32x2 pack2(float a, float b) { f32x2 r; asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(a), "f"(b)); return r; }
__device__ __forceinline__ f32x2 pack2(int a, int b) { f32x2 r; asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "r"(a), "r"(b)); return r; }
__device__ __forceinline__ void unpack2(f32x2 v, float& a, float& b) { asm("mov.b64 {%0, %1}, %2;" : "=f"(a), "=f"(b) : "l"(v)); }
__device__ __forceinline__ f32x2 sub2(f32x2 a, f32x2 b) { f32x2 r; asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b)); return r; }
__device__ __forceinline__ f32x2 mul2(f32x2 a, f32x2 b) { f32x2 r; asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b)); return r; }

// Two outputs of one row (token columns 2t and 2t + 1): each block's term added to its running sum in the reference's order,
// (float(dot) * d_w) * d_x, then the add.
__device__ __forceinline__ void add_terms(float& acc0, float& acc1, int biased0, int biased1, f32x2 dw2, f32x2 dx2) {
    float t0, t1;
    unpack2(mul2(mul2(sub2(pack2(biased0, biased1), pack2(kMagic, kMagic)), dw2), dx2), t0, t1);
    acc0 = __fadd_rn(acc0, t0);
    acc1 = __fadd_rn(acc1, t1);
}

struct GemmParams {
    DevMatrix m;
    DevAct act;
    float* out;
    uint32_t ldo, n;
    int epi;  // EPI_STORE or EPI_ADD
};

template <int WBYTES, int MI>
__global__ void __launch_bounds__(GWARPS * 32, 2) gemm_q8_kernel(const GemmParams p) {
    constexpr int GM = 64 * MI;
    using S = Stage<WBYTES, GM>;
    extern __shared__ __align__(16) unsigned char smem[];
    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t g = lane >> 2, t = lane & 3;
    const uint32_t row_base = blockIdx.x * GM, tok_base = blockIdx.y * GN;
    const uint32_t wr = (warp & 3) * (16 * MI), wt = (warp >> 2) * 32;  // this warp's (16 MI) x 32 corner inside the CTA tile
    const uint32_t nb = p.m.blocks;                              // 32-value blocks per row
    // Rows are walked in chunks of KB blocks. A row whose block count is a multiple of 4 but not of 8 (1152 or 896 values)
    // ends in a chunk of 4 blocks: its other 4 are neither loaded nor multiplied, so every output is still the sum over
    // its own blocks in order.
    const uint32_t chunks = (nb + KB - 1) / KB;
    const bool aligned8 = nb % KB == 0;  // else the f16 scale rows start on 8-byte, not 16-byte, boundaries

    auto stage_ptr = [&](int s) { return smem + size_t(s) * S::kBytes; };
    auto load_stage = [&](int s, uint32_t chunk) {
        unsigned char* base = stage_ptr(s);
        const uint32_t b0 = chunk * KB;
        const uint32_t valid = min(uint32_t(KB), nb - b0);  // blocks of this chunk that exist: KB, or 4 in a short last chunk
        // weights: GM rows x KB*WBYTES bytes, 16-byte pieces
        constexpr int kPiecesA = KB * WBYTES / 16;
        for (uint32_t i = tid; i < GM * kPiecesA; i += GWARPS * 32) {
            const uint32_t r = i / kPiecesA, piece = i % kPiecesA;
            if (piece * 16 >= valid * WBYTES) continue;
            const uint32_t row = min(row_base + r, p.m.rows - 1);
            cp_async16(base + r * S::kARow + piece * 16, p.m.qa + (size_t(row) * nb + b0) * WBYTES + piece * 16);
        }
        for (uint32_t r = tid; r < GM; r += GWARPS * 32) {
            const uint32_t row = min(row_base + r, p.m.rows - 1);
            const __half* src = p.m.d + size_t(row) * nb + b0;
            unsigned char* dst = base + S::kA + r * KB * 2;
            if (aligned8) {
                cp_async16(dst, src);
            } else {
                cp_async8(dst, src);
                if (valid > 4) cp_async8(dst + 8, src + 4);
            }
        }
        unsigned char* bq = base + S::kA + S::kAd;
        for (uint32_t i = tid; i < GN * (KB * 2); i += GWARPS * 32) {
            const uint32_t r = i / (KB * 2), piece = i % (KB * 2);
            if (piece >= valid * 2) continue;
            const uint32_t tok = min(tok_base + r, p.n - 1);
            cp_async16(bq + r * S::kBRow + piece * 16, p.act.q0 + size_t(tok) * p.act.cols + b0 * 32 + piece * 16);
        }
        unsigned char* bd = bq + S::kB;
        for (uint32_t i = tid; i < GN * 2; i += GWARPS * 32) {
            const uint32_t r = i >> 1, piece = i & 1;
            if (piece * 4 >= valid) continue;
            const uint32_t tok = min(tok_base + r, p.n - 1);
            cp_async16(bd + r * KB * 4 + piece * 16, p.act.d0 + size_t(tok) * nb + b0 + piece * 4);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };

    float acc[MI][4][4];
#pragma unroll
    for (int mi = 0; mi < MI; ++mi)
#pragma unroll
        for (int ni = 0; ni < 4; ++ni)
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[mi][ni][j] = 0.0f;

    load_stage(0, 0);
    for (uint32_t chunk = 0; chunk < chunks; ++chunk) {
        if (chunk + 1 < chunks) {
            load_stage((chunk + 1) & 1, chunk + 1);
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncthreads();
        const unsigned char* base = stage_ptr(chunk & 1);
        const unsigned char* aq = base;
        const __half* ad = reinterpret_cast<const __half*>(base + S::kA);
        const unsigned char* bq = base + S::kA + S::kAd;
        const float* bd = reinterpret_cast<const float*>(bq + S::kB);
        const int valid = int(min(uint32_t(KB), nb - chunk * KB));
#pragma unroll
        for (int b = 0; b < KB; ++b) {
            if (b >= 4 && valid <= 4) continue;  // the short last chunk of a row of 8k + 4 blocks
            uint32_t a[MI][4];
            f32x2 dw2[MI][2];  // each row's weight scale, twice (for the row's two token columns)
#pragma unroll
            for (int mi = 0; mi < MI; ++mi) {
                const uint32_t r0 = wr + mi * 16 + g, r1 = r0 + 8;
                if (WBYTES == 16) {
                    const uint32_t w0 = *reinterpret_cast<const uint32_t*>(aq + r0 * S::kARow + b * 16 + 4 * t);
                    const uint32_t w1 = *reinterpret_cast<const uint32_t*>(aq + r1 * S::kARow + b * 16 + 4 * t);
                    a[mi][0] = __vsub4(w0 & 0x0F0F0F0Fu, 0x08080808u);
                    a[mi][1] = __vsub4(w1 & 0x0F0F0F0Fu, 0x08080808u);
                    a[mi][2] = __vsub4((w0 >> 4) & 0x0F0F0F0Fu, 0x08080808u);
                    a[mi][3] = __vsub4((w1 >> 4) & 0x0F0F0F0Fu, 0x08080808u);
                } else {
                    a[mi][0] = *reinterpret_cast<const uint32_t*>(aq + r0 * S::kARow + b * 32 + 4 * t);
                    a[mi][1] = *reinterpret_cast<const uint32_t*>(aq + r1 * S::kARow + b * 32 + 4 * t);
                    a[mi][2] = *reinterpret_cast<const uint32_t*>(aq + r0 * S::kARow + b * 32 + 16 + 4 * t);
                    a[mi][3] = *reinterpret_cast<const uint32_t*>(aq + r1 * S::kARow + b * 32 + 16 + 4 * t);
                }
                const float d0 = __half2float(ad[r0 * KB + b]), d1 = __half2float(ad[r1 * KB + b]);
                dw2[mi][0] = pack2(d0, d0);
                dw2[mi][1] = pack2(d1, d1);
            }
#pragma unroll
            for (int ni = 0; ni < 4; ++ni) {
                const uint32_t tb = wt + ni * 8;
                const uint32_t b0 = *reinterpret_cast<const uint32_t*>(bq + (tb + g) * S::kBRow + b * 32 + 4 * t);
                const uint32_t b1 = *reinterpret_cast<const uint32_t*>(bq + (tb + g) * S::kBRow + b * 32 + 16 + 4 * t);
                const uint32_t c0 = tb + 2 * t, c1 = c0 + 1;  // the two token columns this thread's results belong to
                const f32x2 dx2 = pack2(bd[c0 * KB + b], bd[c1 * KB + b]);
#pragma unroll
                for (int mi = 0; mi < MI; ++mi) {
                    int c[4];
                    mma_s8(c, a[mi][0], a[mi][1], a[mi][2], a[mi][3], b0, b1);
                    // (row g, col 2t) (row g, col 2t+1) (row g+8, col 2t) (row g+8, col 2t+1)
                    add_terms(acc[mi][ni][0], acc[mi][ni][1], c[0], c[1], dw2[mi][0], dx2);
                    add_terms(acc[mi][ni][2], acc[mi][ni][3], c[2], c[3], dw2[mi][1], dx2);
                }
            }
        }
        __syncthreads();  // the stage is free for the load issued two iterations from now
    }

#pragma unroll
    for (int mi = 0; mi < MI; ++mi) {
#pragma unroll
        for (int ni = 0; ni < 4; ++ni) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const uint32_t row = row_base + wr + mi * 16 + g + (j >= 2 ? 8 : 0);
                const uint32_t tok = tok_base + wt + ni * 8 + 2 * t + (j & 1);
                if (row < p.m.rows && tok < p.n) {
                    float* o = p.out + size_t(tok) * p.ldo + row;
                    *o = p.epi == EPI_ADD ? __fadd_rn(*o, acc[mi][ni][j]) : acc[mi][ni][j];
                }
            }
        }
    }
}

}  // namespace

bool gemm_tc_supports(int type, uint32_t cols);  // gemm_tc.cu: the same arithmetic on tcgen05 / tensor memory
void launch_gemm_tc(const MatTarget& tg, const DevAct& act, uint32_t n, Epilogue epi, cudaStream_t s);
// BRISK_CUDA_GEMM=tc / mma picks the prompt GEMM of Q4_0 / Q8_0 matrices (read at every call); unset: kGemmTcDefault
constexpr bool kGemmTcDefault = false;
static bool gemm_tc_on() {
    const char* env = std::getenv("BRISK_CUDA_GEMM");
    return env == nullptr ? kGemmTcDefault : std::strcmp(env, "tc") == 0;
}
bool gemm_k_supports(int type);  // gemm_k.cu: the 256-value super-block formats
void launch_gemm_k(const MatTarget& tg, const DevAct& act, uint32_t n, Epilogue epi, cudaStream_t s);

// Q4_0 / Q8_0 rows of a multiple of 4 blocks (128 values): whole chunks of 8 blocks plus, at most, one chunk of 4.
bool gemm_supports(int type, uint32_t cols) { return ((type == T_Q4_0 || type == T_Q8_0) && cols % 128 == 0) || gemm_k_supports(type); }

// out = weights x activations for one target (EPI_STORE / EPI_ADD).
template <int WBYTES, int MI>
static void launch_gemm_tile(const GemmParams& p, cudaStream_t s) {
    constexpr int GM = 64 * MI;
    constexpr size_t smem = 2 * Stage<WBYTES, GM>::kBytes;
    static DeviceOnce once;
    if (once.first()) {
        BK_CUDA(cudaFuncSetAttribute(gemm_q8_kernel<WBYTES, MI>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)));
        BK_CUDA(cudaFuncSetAttribute(gemm_q8_kernel<WBYTES, MI>, cudaFuncAttributePreferredSharedMemoryCarveout, 100));
    }
    const dim3 grid((p.m.rows + GM - 1) / GM, (p.n + GN - 1) / GN);
    gemm_q8_kernel<WBYTES, MI><<<grid, GWARPS * 32, smem, s>>>(p);
    BK_CUDA(cudaGetLastError());
}

static void launch_gemm_one(const MatTarget& tg, const DevAct& act, uint32_t n, Epilogue epi, cudaStream_t s) {
    if (n >= 32 && gemm_tc_on() && gemm_tc_supports(tg.m.type, tg.m.cols)) {
        launch_gemm_tc(tg, act, n, epi, s);
        return;
    }
    const GemmParams p{tg.m, act, tg.out, tg.ldo, n, int(epi)};
    static const int sms = [] {
        int dev = 0, count = 148;
        if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&count, cudaDevAttrMultiProcessorCount, dev);
        return count;
    }();
    // 128-row tiles unless they would leave SMs without a CTA: then 64-row tiles, twice as many CTAs
    const uint32_t big_tiles = ((tg.m.rows + 127) / 128) * ((n + GN - 1) / GN);
    const bool small = big_tiles < uint32_t(sms);
    if (tg.m.type == T_Q4_0) {
        if (small) launch_gemm_tile<16, 1>(p, s);
        else launch_gemm_tile<16, 2>(p, s);
    } else {
        if (small) launch_gemm_tile<32, 1>(p, s);
        else launch_gemm_tile<32, 2>(p, s);
    }
}

bool launch_gemm(const MatTarget* targets, int count, const DevAct& act, uint32_t n, Epilogue epi, cudaStream_t s) {
    if (epi == EPI_SILU_MUL || epi == EPI_RELU2_MUL) return false;  // the caller runs gate and up separately, then launch_gate_mul
    for (int i = 0; i < count; ++i) {
        if (!gemm_supports(targets[i].m.type, targets[i].m.cols)) return false;
    }
    for (int i = 0; i < count; ++i) {
        if (gemm_k_supports(targets[i].m.type)) launch_gemm_k(targets[i], act, n, epi, s);
        else launch_gemm_one(targets[i], act, n, epi, s);
    }
    return true;
}

}  // namespace bk
