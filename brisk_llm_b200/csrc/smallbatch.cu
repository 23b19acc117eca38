// Multiply for 2..16 token rows (a speculative verify step of 1 + 8 tokens, a short eval_all): the weights stream from HBM
// once, whatever the token count, and the arithmetic is the reference's (src/quant.cpp:445-482: per (row, token) the sum over
// 32-value blocks IN ORDER of float(int_dot) * d_w * d_x), so the results are the CPU's bit for bit.
//
// The streaming kernel for single tokens (matvec.cu) does the integer dots with dp4a, one token at a time per weight
// register; at 4 tokens it takes 1.5-2.2x the time of one, at 9 tokens (two passes) 4-5x. Here the dots come from
// m16n8k32 int8 MMAs - 8 or 16 token columns cost what one does - and the work is laid out so that a matrix with few rows
// still fills the GPU:
//
//   CTA            32 weight rows (two MMA row tiles; for a gate/up pair 16 rows of each, so the activation is applied in
//                  the epilogue) x all tokens. 4096 rows give 128 CTAs (16 rows per CTA, 256 CTAs, measured slower: the
//                  activation traffic doubles).
//   stages         the CTA's next 8 blocks of every row - quants, f16 scales - and the tokens' quantised activations and
//                  scales go into a ring of 5 (Q8_0: 4) stages with cp.async, 16 bytes a piece and about two pieces per
//                  thread and chunk, four chunks ahead of the arithmetic. The rows go to padded pitches: fragment reads
//                  are conflict-free.
//   8 MMA warps    split a stage's 8 blocks, one each (16-block stages with two blocks per warp were measured: the same
//                  time for a whole verify step): fragments straight from the stage (Q4_0 nibbles are widened and
//                  re-centred in registers), one MMA per (row tile, 8 tokens), and each integer dot becomes its block's
//                  term (float(dot) * d_w) * d_x. The MMA's C operand is the bit pattern of 1.5 * 2^23, so the integer comes
//                  out as a float with one exact subtraction.
//   the chains     a sum over blocks in order cannot be split over warps - but its terms can be computed anywhere. The
//                  terms of a stage go to shared memory, and after one CTA barrier thread o adds the 8 terms of outputs
//                  (o, o + 256) to their running sums, in block order: 512 chains per CTA advance together.
//
#include "formats.cuh"
#include "kernels.h"

namespace bk {
namespace {

constexpr int kChunk = 8, kConsumers = 256;  // a CTA takes RT (1 or 2) tiles of 16 weight rows

template <int WBYTES, int NT, int RT>
struct Stage {
    static constexpr int kRows = 16 * RT;
    static constexpr int kStages = WBYTES == 16 ? 5 : 4;  // two CTAs per SM with two row tiles; more with one
    static constexpr int kWPitch = kChunk * WBYTES + 16;
    static constexpr int kW = kRows * kWPitch;
    static constexpr int kD = kRows * kChunk * 2;   // f16 scales [row][8]
    static constexpr int kXPitch = kChunk * 32 + 16;
    static constexpr int kX = 8 * NT * kXPitch;
    static constexpr int kDx = 8 * NT * kChunk * 4; // f32 scales [token][8]
    static constexpr int kBytes = kW + kD + kX + kDx;
    static constexpr int kTerms = kChunk * RT * 128 * NT * 4;  // one buffer of terms: [block][row tile][128 NT outputs]
    static constexpr int kTotal = kStages * kBytes + 2 * kTerms;
};

#ifdef BK_SB_TRACE  // development aid: cycle counts of CTA 0 - never compiled into the library
__device__ unsigned long long g_sb_trace[16];
#define SB_CLOCK() clock64()
#define SB_ADD(slot, since) do { if (blockIdx.x == 0 && threadIdx.x == 0) g_sb_trace[slot] += clock64() - (since); } while (0)
#else
#define SB_CLOCK() 0ll
#define SB_ADD(slot, since) do { } while (0)
#endif

struct SbParams {
    DevMatrix m[3];
    float* out[3];
    uint32_t ldo[3];
    uint32_t first_cta[4];
    int count, epi;
    DevAct act;
    uint32_t n;
};

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gmem) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(uint32_t(__cvta_generic_to_shared(smem_dst))), "l"(gmem) : "memory");
}

constexpr int kMagicBits = 0x4B400000;  // 1.5 * 2^23 as a float
constexpr float kMagic = 12582912.0f;
__device__ __forceinline__ void mma_s8(int (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
        : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "r"(kMagicBits));
}
// Two terms per instruction: packed f32x2 subtract and multiplies round each half exactly as the scalar instructions do
// (there is no add here for the assembler to fuse them with: the terms go to shared memory).
using f32x2 = unsigned long long;
__device__ __forceinline__ f32x2 pack2(float a, float b) { f32x2 r; asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(a), "f"(b)); return r; }
__device__ __forceinline__ f32x2 pack2(int a, int b) { f32x2 r; asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "r"(a), "r"(b)); return r; }
__device__ __forceinline__ f32x2 sub2(f32x2 a, f32x2 b) { f32x2 r; asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b)); return r; }
__device__ __forceinline__ f32x2 mul2(f32x2 a, f32x2 b) { f32x2 r; asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b)); return r; }
// ((float(dot0), float(dot1)) * d_w) * (d_x0, d_x1)
__device__ __forceinline__ f32x2 terms_of(int biased0, int biased1, f32x2 dw2, f32x2 dx2) {
    return mul2(mul2(sub2(pack2(biased0, biased1), pack2(kMagic, kMagic)), dw2), dx2);
}
// four nibbles 0..15, one per byte -> four signed bytes (nibble - 8): no borrow can cross a byte once bit 7 is set
__device__ __forceinline__ uint32_t recentre(uint32_t nibbles) { return ((nibbles | 0x80808080u) - 0x08080808u) ^ 0x80808080u; }

// Row tile j of this CTA: which matrix, which first row.
struct TileRef {
    int target;
    uint32_t row0;
};

template <int WBYTES, int NT, bool PAIR, int RT>
__global__ void __launch_bounds__(kConsumers) smallbatch_kernel(const SbParams p) {
    static_assert(RT == 2 || !PAIR, "a gate/up pair is one row tile of each");
    using S = Stage<WBYTES, NT, RT>;
    constexpr int kRows = S::kRows;
    extern __shared__ __align__(128) unsigned char smem[];
    constexpr int kStages = S::kStages;
    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

    TileRef tile[2];
    if (PAIR) {
        tile[0] = {0, blockIdx.x * 16};
        tile[1] = {1, blockIdx.x * 16};
    } else {
        int target = 0;
        while (target + 1 < p.count && blockIdx.x >= p.first_cta[target + 1]) ++target;
        const uint32_t row0 = (blockIdx.x - p.first_cta[target]) * kRows;
        tile[0] = {target, row0};
        tile[1] = {target, row0 + 16};  // unused with one row tile
    }
    const uint32_t nb = p.m[0].blocks, chunks = nb / kChunk;

    // One chunk (8 blocks of every row, the tokens' quantised activations and both sets of scales) into a stage, 16 bytes
    // per cp.async, about two per thread. (One cp.async.bulk per row and plane - 82 small bulk copies per chunk - was
    // tried first: the copy engine takes them one after the other, ~60 cycles each, and the chunk took 5000 cycles.)
    constexpr uint32_t kWPieces = kChunk * WBYTES / 16;  // 16-byte pieces of a row's quants
    const uint32_t pieces = kRows * kWPieces + kRows + p.n * (kChunk * 2) + p.n * 2;
    // Which pieces a thread copies does not change from chunk to chunk: their sources, destinations and per-chunk strides
    // are worked out once (the matrix descriptors sit in the kernel's parameters, and indexing those per piece and chunk
    // cost ~500 cycles of every chunk), so that a chunk's loads are an add and a cp.async each.
    constexpr int kMaxPieces = (kRows * kWPieces + kRows + kSmallBatchMax * (kChunk * 2) + kSmallBatchMax * 2 + kConsumers - 1) / kConsumers;
    const unsigned char* src[kMaxPieces];
    uint32_t dst[kMaxPieces], step[kMaxPieces];
#pragma unroll
    for (int k = 0; k < kMaxPieces; ++k) {
        const uint32_t i = tid + k * kConsumers;
        src[k] = nullptr;
        dst[k] = step[k] = 0;
        if (i >= pieces) continue;
        if (i < kRows * kWPieces + kRows) {
            const bool scales = i >= kRows * kWPieces;
            const uint32_t r = scales ? i - kRows * kWPieces : i / kWPieces, piece = scales ? 0 : i % kWPieces;
            const int target = r < 16 ? tile[0].target : tile[1].target;  // selects, not an indexed array: that would live in local memory
            const DevMatrix& m = p.m[target];
            const uint32_t row = min((r < 16 ? tile[0].row0 : tile[1].row0) + (r % 16), m.rows - 1);
            if (scales) {
                src[k] = reinterpret_cast<const unsigned char*>(m.d + size_t(row) * nb);
                dst[k] = S::kW + r * (kChunk * 2);
                step[k] = kChunk * 2;
            } else {
                src[k] = m.qa + size_t(row) * nb * WBYTES + piece * 16;
                dst[k] = r * S::kWPitch + piece * 16;
                step[k] = kChunk * WBYTES;
            }
        } else {
            const uint32_t j = i - (kRows * kWPieces + kRows);
            if (j < p.n * (kChunk * 2)) {
                const uint32_t t = j / (kChunk * 2), piece = j % (kChunk * 2);
                src[k] = reinterpret_cast<const unsigned char*>(p.act.q0 + size_t(t) * p.act.cols) + piece * 16;
                dst[k] = S::kW + S::kD + t * S::kXPitch + piece * 16;
                step[k] = kChunk * 32;
            } else {
                const uint32_t q = j - p.n * (kChunk * 2), t = q / 2, piece = q % 2;
                src[k] = reinterpret_cast<const unsigned char*>(p.act.d0 + size_t(t) * nb + piece * 4);
                dst[k] = S::kW + S::kD + S::kX + t * (kChunk * 4) + piece * 16;
                step[k] = kChunk * 4;
            }
        }
    }
    auto load_stage = [&](uint32_t c) {
        if (c < chunks) {
            unsigned char* st = smem + size_t(c % kStages) * S::kBytes;
#pragma unroll
            for (int k = 0; k < kMaxPieces; ++k) {
                if (src[k] != nullptr) cp_async16(st + dst[k], src[k] + size_t(c) * step[k]);
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");  // one group per chunk, empty or not
    };
    const long long t_begin = SB_CLOCK();
    for (uint32_t c = 0; c + 1 < uint32_t(kStages); ++c) load_stage(c);
    asm volatile("cp.async.wait_group %0;" ::"n"(kStages - 2) : "memory");
    __syncthreads();  // chunk 0 is complete
    SB_ADD(0, t_begin);

    // ---- consumers ----
    const uint32_t g = lane >> 2, t = lane & 3;
    float* terms = reinterpret_cast<float*>(smem + size_t(kStages) * S::kBytes);
    constexpr uint32_t kOut = 128 * NT;  // outputs per row tile
    float acc[2] = {0.0f, 0.0f};  // [1] unused with one row tile
    for (uint32_t c = 0; c < chunks; ++c) {
        const long long t_l = SB_CLOCK();
        load_stage(c + kStages - 1);  // into the stage of chunk c - 1: everybody left it before the barrier that ended the last iteration
        SB_ADD(1, t_l);
        const long long t_m = SB_CLOCK();
        const unsigned char* st = smem + size_t(c % kStages) * S::kBytes;
        const unsigned char* xs = st + S::kW + S::kD;
        const float* dxs = reinterpret_cast<const float*>(xs + S::kX);
        float* tb = terms + size_t(c & 1) * (S::kTerms / 4) + size_t(warp) * RT * kOut;  // this warp's block of the chunk
        uint32_t a[2][4];
        float dw[2][2];
#pragma unroll
        for (int j = 0; j < RT; ++j) {
            const uint32_t r0 = j * 16 + g, r1 = r0 + 8;
            if (WBYTES == 16) {
                const uint32_t w0 = *reinterpret_cast<const uint32_t*>(st + r0 * S::kWPitch + warp * 16 + 4 * t);
                const uint32_t w1 = *reinterpret_cast<const uint32_t*>(st + r1 * S::kWPitch + warp * 16 + 4 * t);
                a[j][0] = recentre(w0 & 0x0F0F0F0Fu);
                a[j][1] = recentre(w1 & 0x0F0F0F0Fu);
                a[j][2] = recentre((w0 >> 4) & 0x0F0F0F0Fu);
                a[j][3] = recentre((w1 >> 4) & 0x0F0F0F0Fu);
            } else {
                a[j][0] = *reinterpret_cast<const uint32_t*>(st + r0 * S::kWPitch + warp * 32 + 4 * t);
                a[j][1] = *reinterpret_cast<const uint32_t*>(st + r1 * S::kWPitch + warp * 32 + 4 * t);
                a[j][2] = *reinterpret_cast<const uint32_t*>(st + r0 * S::kWPitch + warp * 32 + 16 + 4 * t);
                a[j][3] = *reinterpret_cast<const uint32_t*>(st + r1 * S::kWPitch + warp * 32 + 16 + 4 * t);
            }
            const __half* ds = reinterpret_cast<const __half*>(st + S::kW);
            dw[j][0] = __half2float(ds[r0 * kChunk + warp]);
            dw[j][1] = __half2float(ds[r1 * kChunk + warp]);
        }
#pragma unroll
        for (int ni = 0; ni < NT; ++ni) {
            const uint32_t b0 = *reinterpret_cast<const uint32_t*>(xs + (ni * 8 + g) * S::kXPitch + warp * 32 + 4 * t);
            const uint32_t b1 = *reinterpret_cast<const uint32_t*>(xs + (ni * 8 + g) * S::kXPitch + warp * 32 + 16 + 4 * t);
            const f32x2 dx2 = pack2(dxs[(ni * 8 + 2 * t) * kChunk + warp], dxs[(ni * 8 + 2 * t + 1) * kChunk + warp]);
#pragma unroll
            for (int j = 0; j < RT; ++j) {
                int d[4];
                mma_s8(d, a[j], b0, b1);
                // outputs of a row tile are numbered  o = ((ni * 2 + half) * 4 + t) * 16 + g * 2 + (column & 1)
                float2* dst = reinterpret_cast<float2*>(tb + j * kOut + ((ni * 2) * 4 + t) * 16 + g * 2);
                *reinterpret_cast<f32x2*>(dst) = terms_of(d[0], d[1], pack2(dw[j][0], dw[j][0]), dx2);       // rows g
                *reinterpret_cast<f32x2*>(dst + 32) = terms_of(d[2], d[3], pack2(dw[j][1], dw[j][1]), dx2);  // rows g + 8: half 1, 64 floats on
            }
        }
        SB_ADD(2, t_m);
        const long long t_w = SB_CLOCK();
        asm volatile("cp.async.wait_group %0;" ::"n"(kStages - 2) : "memory");  // this thread's pieces of chunk c + 1 have landed
        SB_ADD(3, t_w);
        const long long t_s = SB_CLOCK();
        __syncthreads();  // the terms of chunk c and all of chunk c + 1 are visible; the stage of chunk c is free
        SB_ADD(4, t_s);
        const long long t_c = SB_CLOCK();
        if (tid < kOut) {
            const float* tc = terms + size_t(c & 1) * (S::kTerms / 4) + tid;
#pragma unroll
            for (int b = 0; b < kChunk; ++b) {
                acc[0] = __fadd_rn(acc[0], tc[(b * RT + 0) * kOut]);
                if (RT == 2) acc[1] = __fadd_rn(acc[1], tc[(b * RT + 1) * kOut]);
            }
        }
        SB_ADD(5, t_c);
    }

    if (tid < kOut) {
        const uint32_t col = tid & 1, og = (tid >> 1) & 7, ot = (tid >> 4) & 3, half = (tid >> 6) & 1, ni = tid >> 7;
        const uint32_t r = og + 8 * half, tok = ni * 8 + 2 * ot + col;
        if (tok < p.n) {
            if (PAIR) {
                const uint32_t row = tile[0].row0 + r;
                if (row < p.m[0].rows) {
                    float* o = p.out[0] + size_t(tok) * p.ldo[0] + row;
                    *o = p.epi == EPI_SILU_MUL ? silu_mul(acc[0], acc[1]) : relu2_mul(acc[0], acc[1]);
                }
            } else {
#pragma unroll
                for (int j = 0; j < RT; ++j) {
                    const uint32_t row = tile[j].row0 + r;
                    if (row < p.m[tile[j].target].rows) {
                        float* o = p.out[tile[j].target] + size_t(tok) * p.ldo[tile[j].target] + row;
                        *o = p.epi == EPI_ADD ? __fadd_rn(*o, acc[j]) : acc[j];
                    }
                }
            }
        }
    }
}

template <int WBYTES, int NT, bool PAIR, int RT>
void launch_variant(const SbParams& p, uint32_t ctas, cudaStream_t s) {
    using S = Stage<WBYTES, NT, RT>;
    static DeviceOnce once;
    if (once.first()) BK_CUDA(cudaFuncSetAttribute(smallbatch_kernel<WBYTES, NT, PAIR, RT>, cudaFuncAttributeMaxDynamicSharedMemorySize, S::kTotal));
    smallbatch_kernel<WBYTES, NT, PAIR, RT><<<ctas, kConsumers, S::kTotal, s>>>(p);
    BK_CUDA(cudaGetLastError());
}

template <int WBYTES>
void launch_type(const SbParams& p, uint32_t ctas, bool pair, int row_tiles, cudaStream_t s) {
    if (p.n <= 8) {
        if (pair) launch_variant<WBYTES, 1, true, 2>(p, ctas, s);
        else if (row_tiles == 2) launch_variant<WBYTES, 1, false, 2>(p, ctas, s);
        else launch_variant<WBYTES, 1, false, 1>(p, ctas, s);
    } else {
        if (pair) launch_variant<WBYTES, 2, true, 2>(p, ctas, s);
        else if (row_tiles == 2) launch_variant<WBYTES, 2, false, 2>(p, ctas, s);
        else launch_variant<WBYTES, 2, false, 1>(p, ctas, s);
    }
}

}  // namespace

bool smallbatch_supports(int type, uint32_t cols, uint32_t n) {
    return (type == T_Q4_0 || type == T_Q8_0) && cols % 256 == 0 && n >= 2 && n <= kSmallBatchMax;
}

// Same contract as launch_matvec, for 2..16 tokens of Q4_0 / Q8_0 matrices whose rows hold a multiple of 8 blocks;
// returns false (nothing launched) for anything else.
bool launch_smallbatch(const MatTarget* targets, int count, const DevAct& act, uint32_t n, Epilogue epi, cudaStream_t s) {
    const bool pair = epi == EPI_SILU_MUL || epi == EPI_RELU2_MUL;
    if (count < 1 || count > 3 || (pair && count != 2)) return false;
    for (int i = 0; i < count; ++i) {
        if (targets[i].m.type != targets[0].m.type || targets[i].m.cols != targets[0].m.cols) return false;
    }
    if (!smallbatch_supports(targets[0].m.type, targets[0].m.cols, n)) return false;
    if (pair && targets[0].m.rows != targets[1].m.rows) return false;
    SbParams p{};
    p.count = count;
    p.epi = epi;
    p.act = act;
    p.n = n;
    static const uint32_t sms = [] {
        int dev = 0, count = 148;
        if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&count, cudaDevAttrMultiProcessorCount, dev);
        return uint32_t(count);
    }();
    // Two row tiles (32 rows) per CTA share the activation loads. One tile per CTA (16 rows, twice the CTAs) for matrices of
    // few rows was measured and is slower - 4096 x 14336 at 9 tokens 49.2 us against 44.0, 4096 x 4096 19.7 against 18.4 - so
    // it stays a compile-time option of the kernel that nothing selects.
    (void)sms;
    const int row_tiles = 2;
    const uint32_t rows_per_cta = 16u * uint32_t(row_tiles);
    uint32_t ctas = 0;
    for (int i = 0; i < count; ++i) {
        p.m[i] = targets[i].m;
        p.out[i] = targets[i].out;
        p.ldo[i] = targets[i].ldo;
        if (!pair) {
            p.first_cta[i] = ctas;
            ctas += (targets[i].m.rows + rows_per_cta - 1) / rows_per_cta;
        }
    }
    if (pair) ctas = (targets[0].m.rows + 15) / 16;
    else p.first_cta[count] = ctas;
    if (targets[0].m.type == T_Q4_0) launch_type<16>(p, ctas, pair, row_tiles, s);
    else launch_type<32>(p, ctas, pair, row_tiles, s);
    return true;
}

}  // namespace bk
