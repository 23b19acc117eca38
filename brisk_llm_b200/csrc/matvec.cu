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

#include "formats.cuh"
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

__global__ void gate_mul_kernel(float* gate, const float* up, size_t count, int mode, const uint8_t* tanh_table) {
    const size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i < count) gate[i] = mode == 2 ? gelu_mul(gate[i], up[i], tanh_table) : mode == 1 ? relu2_mul(gate[i], up[i]) : silu_mul(gate[i], up[i]);
}

}  // namespace

void launch_gate_mul(float* gate, const float* up, size_t count, int mode, cudaStream_t s, const uint8_t* tanh_table) {
    gate_mul_kernel<<<unsigned((count + 255) / 256), 256, 0, s>>>(gate, up, count, mode, tanh_table);
    BK_CUDA(cudaGetLastError());
}

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
        case T_Q4_1: dispatch<FQ4_1>(p, pair, n, s); break;
        case T_Q5_0: dispatch<FQ5_0>(p, pair, n, s); break;
        case T_Q8_0: dispatch<FQ8_0>(p, pair, n, s); break;
        case T_Q5_K: dispatch<FQ5_K>(p, pair, n, s); break;
        case T_Q4_K: dispatch<FQ4_K>(p, pair, n, s); break;
        case T_Q6_K: dispatch<FQ6_K>(p, pair, n, s); break;
        case T_TQ2_0: dispatch<FTQ2_0>(p, pair, n, s); break;
        case T_F16: dispatch<FF16>(p, pair, n, s); break;
        case T_F32: dispatch<FF32>(p, pair, n, s); break;
        default: throw CudaError("cuda: unsupported weight type");
    }
}

}  // namespace bk
