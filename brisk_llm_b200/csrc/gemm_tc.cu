// Prompt multiply of Q4_0 / Q8_0 matrices on the fifth-generation tensor cores: tcgen05.mma.kind::i8 with the integer
// block dots in tensor memory, and the reference's per-block arithmetic (src/quant.cpp:445-482: the sum over 32-value
// blocks IN ORDER of float(int_dot) * d_w * d_x) done on the CUDA cores out of tensor memory - same integers, same f32
// roundings, so the results are the CPU's bit for bit, like gemm.cu's.
//
// One 32-value block is exactly the K of one kind::i8 MMA, and its integer dot has to meet its own pair of scales before
// the next block's is added, so every block gets its own MMA (no accumulation in tensor memory) and its own 64-column
// slice of tensor memory. CTA tile: 128 weight rows x 64 tokens; one CTA per SM; warps by role:
//
//   4 loader warps    thread = weight row: the row's next 4 blocks from global memory (registers, a chunk ahead), Q4_0
//                     nibbles widened and re-centred to s8, stored as the MMA's K-major operand tiles (8 x 16-byte core
//                     matrices, no swizzle); the tokens' s8 activations likewise; both sets of scales beside them. A ring
//                     of 5 stages of 4 blocks.
//   1 MMA warp        one thread issues 4 MMAs (128 x 64 x 32) per stage into one of two sets of 4 x 64 columns of tensor
//                     memory and commits them to an mbarrier
//   8 epilogue warps  thread = (row, 32 of the 64 tokens): tcgen05.ld of a block's 32 integers, then per output
//                     acc += (float(dot) * d_w) * d_x - a subtraction (the slice is preset to 1.5 * 2^23, so the integer
//                     arrives as a float) and two multiplies as packed f32x2 instructions on two outputs each, and an add -
//                     block after block; the running sums live in registers for the whole K loop
//
// Loaders, MMA and epilogue meet only at mbarriers (stage full / stage free / set full / set free); every wait is bounded
// and ends in an error word. The epilogue is the bound: 5 f32-pipe instructions per (row, token, block) is ~215 TMAC/s at
// full issue, against ~140 for the same arithmetic behind mma.sync fragments (gemm.cu), which also spends issue slots on
// fragment loads and on the MMAs themselves.
#include "kernels.h"

namespace bk {
namespace {

constexpr int kTM = 128, kTN = 64, kCB = 4;           // rows, tokens, blocks per stage
constexpr int kStages = 5;
constexpr int kLoaders = 128, kEpilogue = 256;
constexpr int kEC = kTN * 128 / kEpilogue;             // token columns per epilogue thread: 32 (16 with 512 epilogue threads: measured slower, 367 vs 287 us)
constexpr int kThreads = kLoaders + kEpilogue + 32;   // loaders (warps 0-3) | epilogue (warps 4-11) | MMA warp (12)
constexpr int kMmaWarp = (kLoaders + kEpilogue) / 32;
constexpr uint32_t kATile = kTM * 32, kBTile = kTN * 32;                                     // one block's operand tiles, bytes
constexpr uint32_t kStageBytes = kCB * (kATile + kBTile) + kTM * kCB * 2 + kTN * kCB * 4;   // + f16 weight scales + f32 token scales
constexpr long long kWaitCycles = 2000000000ll;  // about a second: a wait that lasts this long has failed
constexpr uint32_t kTmemCols = 512;

__device__ unsigned int g_gemm_tc_error;

#ifdef BK_TC_TRACE  // development aid: cycles CTA (0,0) spends waiting, by role - never compiled into the library
__device__ unsigned long long g_tc_trace[16];
#define TC_CLOCK() clock64()
#define TC_ADD(slot, since) do { if (blockIdx.x == 0 && blockIdx.y == 0 && (threadIdx.x & 31) == 0) atomicAdd(&g_tc_trace[slot], (unsigned long long)(clock64() - (since))); } while (0)
#else
#define TC_CLOCK() 0ll
#define TC_ADD(slot, since) do { } while (0)
#endif

struct TcParams {
    DevMatrix m;
    DevAct act;
    float* out;
    uint32_t ldo, n;
    int epi;
};

__device__ __forceinline__ uint32_t saddr(const void* p) { return uint32_t(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ void mbar_init(uint64_t* b, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(saddr(b)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* b) { asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(saddr(b)) : "memory"); }
__device__ __forceinline__ bool mbar_try_wait(uint64_t* b, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}" : "=r"(ok) : "r"(saddr(b)), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded: should a wait run out, the error word is set, `dead` makes this thread's later waits return at once, and the
// kernel ends (with garbage) and still frees its tensor memory.
__device__ __forceinline__ void mbar_wait(uint64_t* b, uint32_t parity, bool& dead) {
    if (dead || mbar_try_wait(b, parity)) return;
    const long long start = clock64();
    while (!mbar_try_wait(b, parity)) {
        if (clock64() - start > kWaitCycles) {  // bounded in time, not in tries: one try may itself sleep for a while
            atomicOr(&g_gemm_tc_error, 1u);
            dead = true;
            return;
        }
    }
}

// K-major operand tile without swizzle: core matrices of 8 rows x 16 bytes; `lbo` bytes between the two 16-byte halves of
// K, `sbo` bytes between groups of 8 rows. Bit 46: the descriptor version of this architecture.
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lbo, uint32_t sbo) {
    return uint64_t((addr >> 4) & 0x3FFF) | (uint64_t((lbo >> 4) & 0x3FFF) << 16) | (uint64_t((sbo >> 4) & 0x3FFF) << 32) | (1ull << 46);
}
// s32 accumulator, s8 x s8, both operands K-major, N = 64, M = 128
constexpr uint32_t kInstrDesc = (2u << 4) | (1u << 7) | (1u << 10) | (uint32_t(kTN >> 3) << 17) | (uint32_t(kTM >> 4) << 24);

// D += A x B: the slice was preset to kMagicBits by the epilogue, so the result read as a float is 1.5 * 2^23 + dot
__device__ __forceinline__ void mma_i8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc) {
    asm volatile(
        "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(kInstrDesc), "r"(1u), "r"(0u)
        : "memory");
}
constexpr uint32_t kMagicBits = 0x4B400000u;  // 1.5 * 2^23 as a float; |dot| <= 32 * 127 * 127 < 2^22
constexpr float kMagic = 12582912.0f;
// kEC columns of this warp's 32 lanes := kMagicBits
__device__ __forceinline__ void tmem_preset(uint32_t taddr) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%1,%1,%1,%1,%1,%1,%1,%1,%1,%1,%1,%1,%1,%1,%1,%1,%1,%1,%1,%1,%1,%1,%1,%1,%1,%1,%1,%1,%1,%1,%1};"
        ::"r"(taddr), "r"(kMagicBits)
        : "memory");
}
__device__ __forceinline__ void mma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(saddr(bar)) : "memory");
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_ld_nowait(uint32_t taddr, uint32_t (&v)[kEC]) {
    static_assert(kEC == 32, "the load below (and the preset above) is the x32 form");
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]),
          "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]),
          "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr)
        : "memory");
}
// Two f32 operations per instruction (packed f32x2, IEEE round-to-nearest in each half: the same results as two scalar
// instructions - measured on 4 M random operands). The epilogue is bound by its f32 instruction count. NOT used for the
// final addition: a mul.rn.f32x2 whose only use is an add.rn.f32x2 gets contracted into a fused multiply-add by the
// assembler (measured: 36 % of the results change, with or without -fmad=false), and the reference does not fuse.
using f32x2 = unsigned long long;
__device__ __forceinline__ f32x2 pack2(float a, float b) { f32x2 r; asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(a), "f"(b)); return r; }
__device__ __forceinline__ f32x2 pack2(uint32_t a, uint32_t b) { f32x2 r; asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "r"(a), "r"(b)); return r; }
__device__ __forceinline__ void unpack2(f32x2 v, float& a, float& b) { asm("mov.b64 {%0, %1}, %2;" : "=f"(a), "=f"(b) : "l"(v)); }
__device__ __forceinline__ f32x2 sub2(f32x2 a, f32x2 b) { f32x2 r; asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b)); return r; }
__device__ __forceinline__ f32x2 mul2(f32x2 a, f32x2 b) { f32x2 r; asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b)); return r; }

// four nibbles 0..15, one per byte -> four signed bytes (nibble - 8): no borrow can cross a byte once bit 7 is set
__device__ __forceinline__ uint32_t recentre(uint32_t nibbles) { return ((nibbles | 0x80808080u) - 0x08080808u) ^ 0x80808080u; }

template <int WBYTES>
__global__ void __launch_bounds__(kThreads, 1) gemm_tc_kernel(const TcParams p) {
    extern __shared__ __align__(128) unsigned char smem[];
    __shared__ __align__(8) uint64_t full[kStages], stage_free[kStages], set_full[2], set_free[2];
    __shared__ uint32_t tmem_slot;
    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t row_base = blockIdx.x * kTM, tok_base = blockIdx.y * kTN;
    const uint32_t nb = p.m.blocks, chunks = nb / kCB;

    if (tid == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(&full[s], kLoaders / 32);
            mbar_init(&stage_free[s], kEpilogue / 32);
        }
        for (int s = 0; s < 2; ++s) {
            mbar_init(&set_full[s], 1);
            mbar_init(&set_free[s], kEpilogue / 32);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == kMmaWarp) {  // the MMA warp owns the tensor memory: all 512 columns (one CTA per SM)
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(saddr(&tmem_slot)), "r"(kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(&tmem_slot);
    bool dead = false;

    // (Tried: 16 epilogue warps of 16 columns for more warps per scheduler. 21 warps leave 80 registers a thread, the loaders
    // spill, and setmaxnreg cannot help - it only moves registers inside what the CTA was launched with, so raising the
    // loaders without lowering anybody below the launch count waits forever. Measured 367 us against 287 for this form.)
    if (warp < kLoaders / 32) {
        // ---- loaders: thread = weight row (and, for the activations, half of a token's chunk) ----
        const uint32_t row = min(row_base + tid, p.m.rows - 1);
        const uint32_t tok = min(tok_base + tid / 2, p.n - 1), thalf = tid & 1;
        const uint8_t* wsrc = p.m.qa + size_t(row) * nb * WBYTES;
        const __half* dsrc = p.m.d + size_t(row) * nb;
        const int8_t* xsrc = p.act.q0 + size_t(tok) * p.act.cols + thalf * 64;
        const float* dxsrc = p.act.d0 + size_t(tok) * nb;
        constexpr int kWVec = kCB * WBYTES / 16;  // 16-byte pieces of a row's chunk: 4 (Q4_0) or 8 (Q8_0)
        struct Regs {
            uint4 wv[kWVec], xv[4];
            uint2 dv;
            uint4 dxv;
        };
        auto fetch = [&](Regs& g, uint32_t c) {
            if (c >= chunks) return;
#pragma unroll
            for (int i = 0; i < kWVec; ++i) g.wv[i] = __ldg(reinterpret_cast<const uint4*>(wsrc + size_t(c) * kCB * WBYTES) + i);
            g.dv = __ldg(reinterpret_cast<const uint2*>(dsrc + size_t(c) * kCB));
#pragma unroll
            for (int i = 0; i < 4; ++i) g.xv[i] = __ldg(reinterpret_cast<const uint4*>(xsrc + size_t(c) * kCB * 32) + i);
            if (thalf == 0) g.dxv = __ldg(reinterpret_cast<const uint4*>(dxsrc + size_t(c) * kCB));
        };
        auto fill = [&](const Regs& g, uint32_t c) {
            const uint32_t s = c % kStages, round = c / kStages;
            const long long t_w = TC_CLOCK();
            if (round > 0) mbar_wait(&stage_free[s], (round - 1) & 1, dead);
            if (warp == 0) TC_ADD(0, t_w);
            const long long t_f = TC_CLOCK();
            unsigned char* st = smem + size_t(s) * kStageBytes;
            // A tiles: [block][K half][row group][8 rows][16 bytes]
#pragma unroll
            for (int b = 0; b < kCB; ++b) {
                uint4 lo, hi;
                if (WBYTES == 16) {
                    const uint4 w = g.wv[b];
                    lo = make_uint4(recentre(w.x & 0x0F0F0F0Fu), recentre(w.y & 0x0F0F0F0Fu), recentre(w.z & 0x0F0F0F0Fu), recentre(w.w & 0x0F0F0F0Fu));
                    hi = make_uint4(recentre((w.x >> 4) & 0x0F0F0F0Fu), recentre((w.y >> 4) & 0x0F0F0F0Fu), recentre((w.z >> 4) & 0x0F0F0F0Fu),
                                    recentre((w.w >> 4) & 0x0F0F0F0Fu));
                } else {
                    lo = g.wv[(2 * b) % kWVec];
                    hi = g.wv[(2 * b + 1) % kWVec];
                }
                unsigned char* at = st + b * kATile + (tid / 8) * 128 + (tid % 8) * 16;
                *reinterpret_cast<uint4*>(at) = lo;
                *reinterpret_cast<uint4*>(at + kATile / 2) = hi;
            }
            // B tiles: this thread's two blocks of its token
            {
                const uint32_t t = tid / 2;
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    unsigned char* bt = st + kCB * kATile + (thalf * 2 + j) * kBTile + (t / 8) * 128 + (t % 8) * 16;
                    *reinterpret_cast<uint4*>(bt) = g.xv[2 * j];
                    *reinterpret_cast<uint4*>(bt + kBTile / 2) = g.xv[2 * j + 1];
                }
            }
            // scales: weights [row][4] f16, tokens [block][token] f32
            *reinterpret_cast<uint2*>(st + kCB * (kATile + kBTile) + tid * 8) = g.dv;
            if (thalf == 0) {
                float* dxs = reinterpret_cast<float*>(st + kCB * (kATile + kBTile) + kTM * kCB * 2);
                const uint32_t t = tid / 2;
                dxs[0 * kTN + t] = __uint_as_float(g.dxv.x);
                dxs[1 * kTN + t] = __uint_as_float(g.dxv.y);
                dxs[2 * kTN + t] = __uint_as_float(g.dxv.z);
                dxs[3 * kTN + t] = __uint_as_float(g.dxv.w);
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // the tensor core reads these stores through the async proxy
            __syncwarp();
            if (lane == 0) mbar_arrive(&full[s]);
            if (warp == 0) TC_ADD(1, t_f);
        };
        // two register sets, two chunks ahead of the stores: a chunk's loads have two stage times to arrive
        Regs g0, g1;
        fetch(g0, 0);
        fetch(g1, 1);
        for (uint32_t c = 0; c < chunks; c += 2) {
            fill(g0, c);
            fetch(g0, c + 2);
            if (c + 1 < chunks) {
                fill(g1, c + 1);
                fetch(g1, c + 3);
            }
        }
    } else if (warp == kMmaWarp) {
        // ---- MMA issue: one thread ----
        if (lane == 0) {
            for (uint32_t c = 0; c < chunks; ++c) {
                const uint32_t s = c % kStages, set = c & 1;
                const long long t_a = TC_CLOCK();
                mbar_wait(&full[s], (c / kStages) & 1, dead);
                TC_ADD(2, t_a);
                const long long t_b = TC_CLOCK();
                mbar_wait(&set_free[set], (c >> 1) & 1, dead);  // use u of a set waits for its u-th release; the 0th is the epilogue's preset
                TC_ADD(3, t_b);
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t a0 = saddr(smem + size_t(s) * kStageBytes), b0 = a0 + kCB * kATile;
#pragma unroll
                for (int b = 0; b < kCB; ++b) {
                    mma_i8(tmem_base + set * (kCB * kTN) + b * kTN, smem_desc(a0 + b * kATile, kATile / 2, 128), smem_desc(b0 + b * kBTile, kBTile / 2, 128));
                }
                mma_commit(&set_full[set]);
            }
        }
    } else {
        // ---- epilogue: thread = (row, 32 tokens) ----
        const uint32_t ew = warp - kLoaders / 32;                 // 0..7
        const uint32_t quarter = warp & 3, part = ew >> 2;        // tensor-memory lanes 32 quarter .., token columns kEC part ..
        const uint32_t r = quarter * 32 + lane;                   // row of the tile
        float acc[kEC];
#pragma unroll
        for (int j = 0; j < kEC; ++j) acc[j] = 0.0f;
        const f32x2 magic2 = pack2(kMagic, kMagic);
        const uint32_t tmem_mine = tmem_base + ((quarter * 32) << 16) + part * kEC;  // this warp's lanes, its columns of every slice
        for (uint32_t i = 0; i < 2 * kCB; ++i) tmem_preset(tmem_mine + i * kTN);
        asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncwarp();
        if (lane == 0) {  // both sets start out free (and preset)
            mbar_arrive(&set_free[0]);
            mbar_arrive(&set_free[1]);
        }
        for (uint32_t c = 0; c < chunks; ++c) {
            const uint32_t s = c % kStages, set = c & 1;
            const long long t_e = TC_CLOCK();
            mbar_wait(&set_full[set], (c >> 1) & 1, dead);
            if (ew == 0) TC_ADD(4, t_e);
            const long long t_g = TC_CLOCK();
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const unsigned char* st = smem + size_t(s) * kStageBytes;
            const __half* dws = reinterpret_cast<const __half*>(st + kCB * (kATile + kBTile)) + r * kCB;
            const float* dxs = reinterpret_cast<const float*>(st + kCB * (kATile + kBTile) + kTM * kCB * 2) + part * kEC;
            // Two register sets: the next block's integers are on their way out of tensor memory while this block's 32 outputs
            // are computed (tcgen05.wait::ld waits for every load issued so far, so the next load is issued right after it).
            uint32_t v0[kEC], v1[kEC];
            const uint32_t slice0 = tmem_mine + set * (kCB * kTN);
            auto consume = [&](const uint32_t (&v)[kEC], int b) {
                const float dw = __half2float(dws[b]);
                const f32x2 dw2 = pack2(dw, dw);
#pragma unroll
                for (int j4 = 0; j4 < kEC / 4; ++j4) {
                    const float4 dx = *reinterpret_cast<const float4*>(dxs + b * kTN + 4 * j4);
                    // float(dot) exactly with one subtraction: the slice held kMagicBits before the MMA added the dot to it;
                    // then (float(dot) * d_w) * d_x and the add, each rounded as the scalar instruction rounds
                    float t0, t1, t2, t3;
                    unpack2(mul2(mul2(sub2(pack2(v[4 * j4 + 0], v[4 * j4 + 1]), magic2), dw2), pack2(dx.x, dx.y)), t0, t1);
                    unpack2(mul2(mul2(sub2(pack2(v[4 * j4 + 2], v[4 * j4 + 3]), magic2), dw2), pack2(dx.z, dx.w)), t2, t3);
                    acc[4 * j4 + 0] = __fadd_rn(acc[4 * j4 + 0], t0);
                    acc[4 * j4 + 1] = __fadd_rn(acc[4 * j4 + 1], t1);
                    acc[4 * j4 + 2] = __fadd_rn(acc[4 * j4 + 2], t2);
                    acc[4 * j4 + 3] = __fadd_rn(acc[4 * j4 + 3], t3);
                }
            };
            static_assert(kCB == 4, "the block loop below is written out for four blocks");
            tmem_ld_nowait(slice0, v0);
            tmem_wait_ld();
            tmem_preset(slice0);  // for the MMA that uses this slice next
            tmem_ld_nowait(slice0 + kTN, v1);
            consume(v0, 0);
            tmem_wait_ld();
            tmem_preset(slice0 + kTN);
            tmem_ld_nowait(slice0 + 2 * kTN, v0);
            consume(v1, 1);
            tmem_wait_ld();
            tmem_preset(slice0 + 2 * kTN);
            tmem_ld_nowait(slice0 + 3 * kTN, v1);
            consume(v0, 2);
            tmem_wait_ld();
            tmem_preset(slice0 + 3 * kTN);
            consume(v1, 3);
            asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");  // the presets have landed
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(&set_free[set]);
                mbar_arrive(&stage_free[s]);
            }
            if (ew == 0) TC_ADD(5, t_g);
        }
        const uint32_t row = row_base + r;
        if (row < p.m.rows) {
#pragma unroll
            for (int j = 0; j < kEC; ++j) {
                const float value = acc[j];
                const uint32_t tok = tok_base + part * kEC + j;
                if (tok < p.n) {
                    float* o = p.out + size_t(tok) * p.ldo + row;
                    *o = p.epi == EPI_ADD ? __fadd_rn(*o, value) : value;
                }
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == kMmaWarp) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
    }
}

template <int WBYTES>
void launch_tile(const TcParams& p, cudaStream_t s) {
    constexpr size_t smem = size_t(kStages) * kStageBytes;
    static DeviceOnce once;
    if (once.first()) BK_CUDA(cudaFuncSetAttribute(gemm_tc_kernel<WBYTES>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)));
    const dim3 grid((p.m.rows + kTM - 1) / kTM, (p.n + kTN - 1) / kTN);
    gemm_tc_kernel<WBYTES><<<grid, kThreads, smem, s>>>(p);
    BK_CUDA(cudaGetLastError());
}

}  // namespace

unsigned int* gemm_tc_error_word() {
    unsigned int* p = nullptr;
    BK_CUDA(cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_gemm_tc_error));
    return p;
}

bool gemm_tc_supports(int type, uint32_t cols) { return (type == T_Q4_0 || type == T_Q8_0) && cols % 128 == 0; }

// out = weights x activations (EPI_STORE / EPI_ADD) for one Q4_0 / Q8_0 target on the tcgen05 path.
void launch_gemm_tc(const MatTarget& tg, const DevAct& act, uint32_t n, Epilogue epi, cudaStream_t s) {
    const TcParams p{tg.m, act, tg.out, tg.ldo, n, int(epi)};
    if (tg.m.type == T_Q4_0) launch_tile<16>(p, s);
    else launch_tile<32>(p, s);
}

}  // namespace bk
