// Prompt multiply on int8 tensor cores for the 256-value super-block formats (Q4_K, Q6_K, TQ2_0) against Q8_K
// activations, with the reference's integer arithmetic and float order (src/quant.cpp:500-596):
//
//   TQ2_0  acc   = sum over the super-block of q*x            (8 MMAs of k = 32 chained in int32)
//          term  = (x.d * w.d) * float(acc - sum(x))
//   Q4_K   per 32-value sub-block sb: dot_sb = q*x (one MMA)   weighted += scale[sb] * dot_sb
//                                                              offsets  += min[sb] * (bsum[2sb] + bsum[2sb+1])
//          term  = x.d * (w.d * float(weighted) - w.dmin * float(offsets))
//   Q6_K   per 16-value group g: dot_g = q6*x (one k = 16 MMA) weighted += scale[g] * (dot_g - 32 * bsum[g])
//          term  = (x.d * w.d) * float(weighted)
//   out[token][row] = sum of the terms over super-blocks, in order, by the one thread that owns the output.
//
// Everything before the float expression is exact integer work, so results are bit-identical to the CPU kernels.
// Tiling as in gemm.cu: CTA = 128 rows x 64 tokens, 8 warps of 32 x 32, two cp.async stages of one super-block each.
#include "kernels.h"

namespace bk {
namespace {

constexpr int KM = 128, KN = 64, KWARPS = 8;

__device__ __forceinline__ void cp16(void* smem, const void* gmem) {
    const uint32_t a = uint32_t(__cvta_generic_to_shared(smem));
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(a), "l"(gmem) : "memory");
}
__device__ __forceinline__ void mma_k32(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma_k16(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t b0) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%0,%1,%2,%3};"
                 : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
                 : "r"(a0), "r"(a1), "r"(b0));
}

struct KParams {
    DevMatrix m;
    DevAct act;
    float* out;
    uint32_t ldo, n;
    int epi;
};

// Shared-memory stage of one super-block. Row strides carry 16 bytes of padding so that the 8 rows a warp's fragment
// loads touch fall into different banks.
template <int TYPE>
struct KStage {
    static constexpr int kQ = TYPE == T_TQ2_0 ? 64 : TYPE == T_Q4_K ? 128 : 192;  // quant bytes per row and super-block
    static constexpr int kARow = kQ + 16;
    static constexpr int kA = KM * kARow;
    static constexpr int kSc = TYPE == T_TQ2_0 ? 0 : KM * 16;  // sub-block scales (and mins)
    static constexpr int kD = KM * 4;                          // d (and dmin) as f16
    static constexpr int kBRow = 256 + 16;
    static constexpr int kB = KN * kBRow;
    static constexpr int kBd = KN * 4;
    static constexpr int kBs = KN * 32;  // 16 int16 sums of 16
    static constexpr int kBytes = kA + kSc + kD + kB + kBd + kBs;
};

template <int TYPE>
__global__ void __launch_bounds__(KWARPS * 32, 1) gemm_k_kernel(const KParams p) {
    using S = KStage<TYPE>;
    extern __shared__ __align__(16) unsigned char smem[];
    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t g = lane >> 2, t = lane & 3;
    const uint32_t row_base = blockIdx.x * KM, tok_base = blockIdx.y * KN;
    const uint32_t wr = (warp & 3) * 32, wt = (warp >> 2) * 32;
    const uint32_t nsb = p.m.blocks;  // super-blocks per row

    auto load_stage = [&](int s, uint32_t sb) {
        unsigned char* base = smem + size_t(s) * S::kBytes;
        constexpr int kPieces = S::kQ / 16;
        for (uint32_t i = tid; i < KM * kPieces; i += KWARPS * 32) {
            const uint32_t r = i / kPieces, piece = i % kPieces;
            const uint32_t row = min(row_base + r, p.m.rows - 1);
            const unsigned char* src;
            if (TYPE == T_Q6_K) {
                // three planes of 64 bytes per super-block: qa | qb | qc
                const uint8_t* plane = piece < 4 ? p.m.qa : piece < 8 ? p.m.qb : p.m.qc;
                src = plane + (size_t(row) * nsb + sb) * 64 + (piece & 3) * 16;
            } else {
                src = p.m.qa + (size_t(row) * nsb + sb) * S::kQ + piece * 16;
            }
            cp16(base + r * S::kARow + piece * 16, src);
        }
        if (TYPE != T_TQ2_0) {
            for (uint32_t r = tid; r < KM; r += KWARPS * 32) {
                const uint32_t row = min(row_base + r, p.m.rows - 1);
                cp16(base + S::kA + r * 16, p.m.sc + (size_t(row) * nsb + sb) * 16);
            }
        }
        // d planes are 2 (TQ2_0, Q6_K) or 4 (Q4_K) bytes per super-block: too small for cp.async, plain loads
        uint16_t* dd = reinterpret_cast<uint16_t*>(base + S::kA + S::kSc);
        for (uint32_t r = tid; r < KM; r += KWARPS * 32) {
            const uint32_t row = min(row_base + r, p.m.rows - 1);
            const uint16_t* src = reinterpret_cast<const uint16_t*>(p.m.d);
            if (TYPE == T_Q4_K) {
                dd[2 * r] = src[2 * (size_t(row) * nsb + sb)];
                dd[2 * r + 1] = src[2 * (size_t(row) * nsb + sb) + 1];
            } else {
                dd[2 * r] = src[size_t(row) * nsb + sb];
            }
        }
        unsigned char* bq = base + S::kA + S::kSc + S::kD;
        for (uint32_t i = tid; i < KN * 16; i += KWARPS * 32) {
            const uint32_t r = i >> 4, piece = i & 15;
            const uint32_t tok = min(tok_base + r, p.n - 1);
            cp16(bq + r * S::kBRow + piece * 16, p.act.qk + size_t(tok) * p.act.cols + sb * 256 + piece * 16);
        }
        float* bd = reinterpret_cast<float*>(bq + S::kB);
        unsigned char* bs = bq + S::kB + S::kBd;
        for (uint32_t r = tid; r < KN; r += KWARPS * 32) {
            const uint32_t tok = min(tok_base + r, p.n - 1);
            bd[r] = p.act.dk[size_t(tok) * nsb + sb];
            cp16(bs + r * 32, p.act.bs + (size_t(tok) * nsb + sb) * 16);
            cp16(bs + r * 32 + 16, p.act.bs + (size_t(tok) * nsb + sb) * 16 + 8);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };

    float acc[2][4][4];
#pragma unroll
    for (int mi = 0; mi < 2; ++mi)
#pragma unroll
        for (int ni = 0; ni < 4; ++ni)
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[mi][ni][j] = 0.0f;

    load_stage(0, 0);
    for (uint32_t sb = 0; sb < nsb; ++sb) {
        if (sb + 1 < nsb) {
            load_stage((sb + 1) & 1, sb + 1);
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncthreads();
        const unsigned char* base = smem + size_t(sb & 1) * S::kBytes;
        const unsigned char* aq = base;
        const unsigned char* asc = base + S::kA;
        const __half* ad = reinterpret_cast<const __half*>(base + S::kA + S::kSc);
        const unsigned char* bq = base + S::kA + S::kSc + S::kD;
        const float* bd = reinterpret_cast<const float*>(bq + S::kB);
        const int16_t* bs = reinterpret_cast<const int16_t*>(bq + S::kB + S::kBd);

        // integer accumulators of this super-block: [row tile][token tile][4 results]
        int weighted[2][4][4], offsets[2][4][4];
#pragma unroll
        for (int mi = 0; mi < 2; ++mi)
#pragma unroll
            for (int ni = 0; ni < 4; ++ni)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    weighted[mi][ni][j] = 0;
                    offsets[mi][ni][j] = 0;
                }

        if constexpr (TYPE == T_TQ2_0) {
#pragma unroll
            for (int jj = 0; jj < 2; ++jj) {  // halves of 128 values: units 2jj (k 0..15 of each run) and 2jj+1 (k 16..31)
                uint32_t w0[2][2], w1[2][2];
#pragma unroll
                for (int mi = 0; mi < 2; ++mi) {
                    const uint32_t r0 = wr + mi * 16 + g, r1 = r0 + 8;
                    w0[mi][0] = *reinterpret_cast<const uint32_t*>(aq + r0 * S::kARow + (2 * jj) * 16 + 4 * t);
                    w0[mi][1] = *reinterpret_cast<const uint32_t*>(aq + r0 * S::kARow + (2 * jj + 1) * 16 + 4 * t);
                    w1[mi][0] = *reinterpret_cast<const uint32_t*>(aq + r1 * S::kARow + (2 * jj) * 16 + 4 * t);
                    w1[mi][1] = *reinterpret_cast<const uint32_t*>(aq + r1 * S::kARow + (2 * jj + 1) * 16 + 4 * t);
                }
#pragma unroll
                for (int l = 0; l < 4; ++l) {  // run l: values jj*128 + 32l .. +31
                    const int kofs = jj * 128 + l * 32;
#pragma unroll
                    for (int ni = 0; ni < 4; ++ni) {
                        const unsigned char* brow = bq + (wt + ni * 8 + g) * S::kBRow + kofs;
                        const uint32_t b0 = *reinterpret_cast<const uint32_t*>(brow + 4 * t);
                        const uint32_t b1 = *reinterpret_cast<const uint32_t*>(brow + 16 + 4 * t);
#pragma unroll
                        for (int mi = 0; mi < 2; ++mi) {
                            mma_k32(weighted[mi][ni], (w0[mi][0] >> (2 * l)) & 0x03030303u, (w1[mi][0] >> (2 * l)) & 0x03030303u,
                                    (w0[mi][1] >> (2 * l)) & 0x03030303u, (w1[mi][1] >> (2 * l)) & 0x03030303u, b0, b1);
                        }
                    }
                }
            }
        } else if constexpr (TYPE == T_Q4_K) {
#pragma unroll
            for (int ch = 0; ch < 4; ++ch) {  // 64-value chunk: sub-blocks 2ch (low nibbles) and 2ch+1 (high nibbles)
                uint32_t w0[2][2], w1[2][2];
                int sc[2][2][2], mn[2][2][2];  // [row tile][row g / g+8][sub-block low / high]
#pragma unroll
                for (int mi = 0; mi < 2; ++mi) {
                    const uint32_t r0 = wr + mi * 16 + g, r1 = r0 + 8;
                    w0[mi][0] = *reinterpret_cast<const uint32_t*>(aq + r0 * S::kARow + (2 * ch) * 16 + 4 * t);
                    w0[mi][1] = *reinterpret_cast<const uint32_t*>(aq + r0 * S::kARow + (2 * ch + 1) * 16 + 4 * t);
                    w1[mi][0] = *reinterpret_cast<const uint32_t*>(aq + r1 * S::kARow + (2 * ch) * 16 + 4 * t);
                    w1[mi][1] = *reinterpret_cast<const uint32_t*>(aq + r1 * S::kARow + (2 * ch + 1) * 16 + 4 * t);
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        sc[mi][0][h] = asc[r0 * 16 + 2 * ch + h];
                        sc[mi][1][h] = asc[r1 * 16 + 2 * ch + h];
                        mn[mi][0][h] = asc[r0 * 16 + 8 + 2 * ch + h];
                        mn[mi][1][h] = asc[r1 * 16 + 8 + 2 * ch + h];
                    }
                }
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const int sbk = 2 * ch + h;
#pragma unroll
                    for (int ni = 0; ni < 4; ++ni) {
                        const uint32_t tb = wt + ni * 8;
                        const unsigned char* brow = bq + (tb + g) * S::kBRow + sbk * 32;
                        const uint32_t b0 = *reinterpret_cast<const uint32_t*>(brow + 4 * t);
                        const uint32_t b1 = *reinterpret_cast<const uint32_t*>(brow + 16 + 4 * t);
                        const uint32_t c0 = tb + 2 * t, c1 = c0 + 1;
                        const int bs0 = int(bs[c0 * 16 + 2 * sbk]) + int(bs[c0 * 16 + 2 * sbk + 1]);
                        const int bs1 = int(bs[c1 * 16 + 2 * sbk]) + int(bs[c1 * 16 + 2 * sbk + 1]);
#pragma unroll
                        for (int mi = 0; mi < 2; ++mi) {
                            int c[4] = {0, 0, 0, 0};
                            const uint32_t sh = h ? 4 : 0;
                            mma_k32(c, (w0[mi][0] >> sh) & 0x0F0F0F0Fu, (w1[mi][0] >> sh) & 0x0F0F0F0Fu, (w0[mi][1] >> sh) & 0x0F0F0F0Fu,
                                    (w1[mi][1] >> sh) & 0x0F0F0F0Fu, b0, b1);
                            weighted[mi][ni][0] += sc[mi][0][h] * c[0];
                            weighted[mi][ni][1] += sc[mi][0][h] * c[1];
                            weighted[mi][ni][2] += sc[mi][1][h] * c[2];
                            weighted[mi][ni][3] += sc[mi][1][h] * c[3];
                            offsets[mi][ni][0] += mn[mi][0][h] * bs0;
                            offsets[mi][ni][1] += mn[mi][0][h] * bs1;
                            offsets[mi][ni][2] += mn[mi][1][h] * bs0;
                            offsets[mi][ni][3] += mn[mi][1][h] * bs1;
                        }
                    }
                }
            }
        } else {  // Q6_K
#pragma unroll
            for (int u = 0; u < 4; ++u) {  // unit u: 64 values = four runs of 16: k-th run at (u>>1)*128 + 32k + (u&1)*16
                uint32_t a[2][2], b[2][2], cc[2][2];
#pragma unroll
                for (int mi = 0; mi < 2; ++mi) {
#pragma unroll
                    for (int hh = 0; hh < 2; ++hh) {
                        const uint32_t r = wr + mi * 16 + g + hh * 8;
                        a[mi][hh] = *reinterpret_cast<const uint32_t*>(aq + r * S::kARow + u * 16 + 4 * t);
                        b[mi][hh] = *reinterpret_cast<const uint32_t*>(aq + r * S::kARow + 64 + u * 16 + 4 * t);
                        cc[mi][hh] = *reinterpret_cast<const uint32_t*>(aq + r * S::kARow + 128 + u * 16 + 4 * t);
                    }
                }
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const int grp = (u >> 1) * 8 + 2 * k + (u & 1);  // 16-value group inside the super-block
                    const int kofs = (u >> 1) * 128 + 32 * k + (u & 1) * 16;
                    uint32_t v[2][2];
                    int sc[2][2];
#pragma unroll
                    for (int mi = 0; mi < 2; ++mi) {
#pragma unroll
                        for (int hh = 0; hh < 2; ++hh) {
                            const uint32_t L = 0x0F0F0F0Fu, H = 0x30303030u;
                            const uint32_t lo = k == 0 ? (a[mi][hh] & L) : k == 1 ? (b[mi][hh] & L) : k == 2 ? ((a[mi][hh] >> 4) & L) : ((b[mi][hh] >> 4) & L);
                            const uint32_t hi = k == 0 ? ((cc[mi][hh] << 4) & H) : k == 1 ? ((cc[mi][hh] << 2) & H) : k == 2 ? (cc[mi][hh] & H) : ((cc[mi][hh] >> 2) & H);
                            v[mi][hh] = lo | hi;
                            sc[mi][hh] = reinterpret_cast<const int8_t*>(asc)[(wr + mi * 16 + g + hh * 8) * 16 + grp];
                        }
                    }
#pragma unroll
                    for (int ni = 0; ni < 4; ++ni) {
                        const uint32_t tb = wt + ni * 8;
                        const uint32_t b0 = *reinterpret_cast<const uint32_t*>(bq + (tb + g) * S::kBRow + kofs + 4 * t);
                        const uint32_t c0 = tb + 2 * t, c1 = c0 + 1;
                        const int o0 = 32 * int(bs[c0 * 16 + grp]), o1 = 32 * int(bs[c1 * 16 + grp]);
#pragma unroll
                        for (int mi = 0; mi < 2; ++mi) {
                            int c[4] = {0, 0, 0, 0};
                            mma_k16(c, v[mi][0], v[mi][1], b0);
                            weighted[mi][ni][0] += sc[mi][0] * (c[0] - o0);
                            weighted[mi][ni][1] += sc[mi][0] * (c[1] - o1);
                            weighted[mi][ni][2] += sc[mi][1] * (c[2] - o0);
                            weighted[mi][ni][3] += sc[mi][1] * (c[3] - o1);
                        }
                    }
                }
            }
        }

        // the super-block's float term, added to the running sums in super-block order
#pragma unroll
        for (int mi = 0; mi < 2; ++mi) {
            const uint32_t r0 = wr + mi * 16 + g, r1 = r0 + 8;
            const float dw0 = __half2float(ad[2 * r0]), dw1 = __half2float(ad[2 * r1]);
            const float dm0 = TYPE == T_Q4_K ? __half2float(ad[2 * r0 + 1]) : 0.0f, dm1 = TYPE == T_Q4_K ? __half2float(ad[2 * r1 + 1]) : 0.0f;
#pragma unroll
            for (int ni = 0; ni < 4; ++ni) {
                const uint32_t c0 = wt + ni * 8 + 2 * t, c1 = c0 + 1;
                const float dx0 = bd[c0], dx1 = bd[c1];
                float term[4];
                if constexpr (TYPE == T_Q4_K) {
                    term[0] = __fmul_rn(dx0, __fsub_rn(__fmul_rn(dw0, float(weighted[mi][ni][0])), __fmul_rn(dm0, float(offsets[mi][ni][0]))));
                    term[1] = __fmul_rn(dx1, __fsub_rn(__fmul_rn(dw0, float(weighted[mi][ni][1])), __fmul_rn(dm0, float(offsets[mi][ni][1]))));
                    term[2] = __fmul_rn(dx0, __fsub_rn(__fmul_rn(dw1, float(weighted[mi][ni][2])), __fmul_rn(dm1, float(offsets[mi][ni][2]))));
                    term[3] = __fmul_rn(dx1, __fsub_rn(__fmul_rn(dw1, float(weighted[mi][ni][3])), __fmul_rn(dm1, float(offsets[mi][ni][3]))));
                } else {
                    int xs0 = 0, xs1 = 0;
                    if constexpr (TYPE == T_TQ2_0) {  // sum((q-1)*x) = sum(q*x) - sum(x)
#pragma unroll
                        for (int k = 0; k < 16; ++k) {
                            xs0 += bs[c0 * 16 + k];
                            xs1 += bs[c1 * 16 + k];
                        }
                    }
                    term[0] = __fmul_rn(__fmul_rn(dx0, dw0), float(weighted[mi][ni][0] - xs0));
                    term[1] = __fmul_rn(__fmul_rn(dx1, dw0), float(weighted[mi][ni][1] - xs1));
                    term[2] = __fmul_rn(__fmul_rn(dx0, dw1), float(weighted[mi][ni][2] - xs0));
                    term[3] = __fmul_rn(__fmul_rn(dx1, dw1), float(weighted[mi][ni][3] - xs1));
                }
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[mi][ni][j] = __fadd_rn(acc[mi][ni][j], term[j]);
            }
        }
        __syncthreads();
    }

#pragma unroll
    for (int mi = 0; mi < 2; ++mi)
#pragma unroll
        for (int ni = 0; ni < 4; ++ni)
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

template <int TYPE>
void launch_one(const KParams& p, cudaStream_t s) {
    constexpr size_t smem = 2 * KStage<TYPE>::kBytes;
    static DeviceOnce once;
    if (once.first()) BK_CUDA(cudaFuncSetAttribute(gemm_k_kernel<TYPE>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)));
    const dim3 grid((p.m.rows + KM - 1) / KM, (p.n + KN - 1) / KN);
    gemm_k_kernel<TYPE><<<grid, KWARPS * 32, smem, s>>>(p);
    BK_CUDA(cudaGetLastError());
}

}  // namespace

bool gemm_k_supports(int type) { return type == T_Q4_K || type == T_Q6_K || type == T_TQ2_0; }

void launch_gemm_k(const MatTarget& tg, const DevAct& act, uint32_t n, Epilogue epi, cudaStream_t s) {
    const KParams p{tg.m, act, tg.out, tg.ldo, n, int(epi)};
    switch (tg.m.type) {
        case T_Q4_K: launch_one<T_Q4_K>(p, s); break;
        case T_Q6_K: launch_one<T_Q6_K>(p, s); break;
        case T_TQ2_0: launch_one<T_TQ2_0>(p, s); break;
        default: throw CudaError("cuda: no super-block tensor kernel for this type");
    }
}

}  // namespace bk
