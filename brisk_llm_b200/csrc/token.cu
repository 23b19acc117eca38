// One decoded token as ONE kernel launch: embedding row -> every layer -> output head -> arg-max -> next token and
// position, for models whose layer matrices and head are Q4_0 and small enough that an SM's share of a layer's weights
// fits its shared memory (the 0.6B class). One 512-thread CTA per SM, launched cooperatively so all CTAs are resident.
//
// A token of such a model is not bound by HBM (a layer is 9 MB: 1.4 us at full bandwidth) but by the chain of dependent
// operations, each needing the whole result vector of the one before. Measured on B200, three things decide the length
// of that chain, and the kernel is arranged around them:
//
//   * DOUBLE PRECISION IS SCARCE: an SM retires about two f64 lane-operations per clock (one warp instruction per 16
//     cycles), and the reference's arithmetic needs f64 in three places - the sums of squares of the RMS norms, the
//     softmax's exp (glibc's algorithm is double inside, exact_math.h) and its denominator. So every f64 value is
//     computed ONCE, by whoever owns the data, and travels with it: the owner of 32 residual values publishes their sum
//     of squares; a score task computes the exps of its own 32 positions and publishes them with their partial sum.
//   * WHO OWNS WHAT is aligned to the 32-value quantisation blocks: an output-projection / down-projection CTA owns whole
//     blocks of the hidden rows (and keeps the residual stream of those rows in registers), a gate/up CTA owns whole
//     blocks of the feed-forward rows, an attention CTA owns (head, 32 dimensions), a q/k/v CTA owns one whole head. The
//     owner therefore finishes the vector: per-head RMS norm + RoPE + K/V cache store for q/k/v, 8-bit quantisation
//     (quantize_q8_0, src/quant.cpp:115-142) for the attended and the gated vector - consumers of those two read a
//     quarter of the bytes and copy them straight into the activation planes.
//   * WEIGHTS NEVER WAIT FOR ACTIVATIONS: a CTA's rows of an operation (nibble plane and scale plane, cp.async.bulk,
//     completion on an mbarrier) are requested a whole layer ahead, the moment the same operation of the previous layer
//     has left the buffer; cached K rows and V slices are requested when the previous layer's attention has left theirs.
//
// Operations hand over through TAGGED WORDS in L2 (decode_body.cuh): one 64-bit {payload, tag} store per element,
// consumers re-read until the tag of this token, layer and operation is there; no grid barrier, no fence. Vectors
// alternate between two copies by layer parity. The code is kept small on purpose: the layer loop must stay inside the
// instruction cache (a first version of 124 KB lost ~2.5 us per layer to refetching it).
//
// All float arithmetic is the reference's, in the reference's order (the f64 sums are tree-ordered, as in the other
// single-token paths); results are bit-identical to the CPU engine and to the other paths. Every wait (tagged words,
// mbarriers) is bounded and ends in the error word.
#include <algorithm>
#include <cstdio>
#include <cstring>
#include <memory>

#include "decode_body.cuh"

namespace bk {
namespace {

constexpr uint32_t kTokThreads = 512;
constexpr uint32_t kTokWarps = 16;
constexpr uint32_t kVChunkPos = 512;           // positions per chunk of the V ring
constexpr uint32_t kSub = 256;                 // positions per product tile of the weighted sum
constexpr uint32_t kSliceW = 32;               // head dimensions per attention CTA: one quantisation block
constexpr uint32_t kTagsPerLayer = 8;          // q/k/v, scores, exps, attended, o, gated, down
constexpr uint32_t kMbarLimit = 1u << 22;      // try_wait rounds before a bulk copy is declared lost
constexpr uint32_t kNone = 0xffffffffu;

#ifdef BK_TOK_TRACE
#define TOK_STAMP(tr, k) do { if ((tr) != nullptr) (tr)[k] = (unsigned long long)clock64(); } while (0)
#define TOK_TRACE_PTR(P, l, slot) (((P).trace != nullptr && threadIdx.x == 0 && (l) == 5 && (blockIdx.x == 0 || blockIdx.x == 40 || blockIdx.x == 100)) \
    ? (P).trace + 4 * (2 + (P).n_layers * 6) + (blockIdx.x == 0 ? 0 : blockIdx.x == 40 ? 1 : 2) * 96 + (slot) * 12 : nullptr)
#else
#define TOK_STAMP(tr, k) do { } while (0)
#define TOK_TRACE_PTR(P, l, slot) nullptr
#endif

struct alignas(16) TokLayer {
    const uint8_t* nib[7];  // q k v o gate up down: 16-byte units of nibbles, row-major
    const __half* scl[7];   // their f16 block scales
    const float* attn_norm;
    const float* ffn_norm;
    const float* q_norm;
    const float* k_norm;
    const float* q_bias;
    const float* k_bias;
    const float* v_bias;
    __half* k_cache;
    __half* v_cache;
    uint64_t pad;
};
static_assert(sizeof(TokLayer) % 16 == 0, "copied in 16-byte pieces");

struct TokSmem {  // byte offsets into dynamic shared memory; `region` holds what a CTA's roles need, laid out per CTA
    uint32_t tabs, xlo, xhi, xd, xs, tile, hv, sslot, region, total;
    uint32_t sslot_bytes, n_sslots, head_rows, ring_slot_bytes, ring_chunks;
    uint32_t size_a, size_b, size_d, size_c;  // weight buffers of the roles
};

struct TokParams {
    const TokLayer* layers;
    uint32_t n_layers;
    uint32_t hidden, q_rows, kv_rows, ffn, heads, kv_heads, vocab, max_context;
    float eps, scale;
    int act;  // EPI_SILU_MUL or EPI_RELU2_MUL
    // role ranges over the CTAs
    uint32_t n_units;              // head units (q heads, then k heads, then v heads): CTA u < n_units owns unit u
    uint32_t bd_first, bd_ctas;    // CTAs owning hidden blocks (output and down projections)
    uint32_t c_first, c_ctas;      // CTAs owning feed-forward blocks (gate/up)
    uint32_t w_first;              // CTA w_first + t owns attention task t = head * slices + slice
    // tagged exchange vectors, two copies each (layer parity)
    uint2* ha[2];    // residual stream after the embedding / a down projection: hidden values ...
    uint2* hsa[2];   // ... and per 32-value block the f64 sum of their squares (two words)
    uint2* hb[2];    // after an output projection
    uint2* hsb[2];
    uint2* xq[2];    // q after per-head norm and RoPE
    uint2* xk[2];    // k after norm and RoPE, rounded to f16
    uint2* xv[2];    // v (+bias), unrounded
    uint2* sc[2];    // per (head, 32 positions): the maximum of those scores
    uint2* ex[2];    // exp(score - max) [heads][max_context]
    uint2* exs[2];   // per (head, 32 positions): f64 sum of those exps (two words)
    uint2* aq[2];    // attended vector, quantised: per block 8 words of 4 int8, scale, sum
    uint2* gq[2];    // gated vector, quantised likewise
    uint2* part;     // per CTA: {best value}, {best index}
    // model ends
    const uint8_t* embd_nib;
    const __half* embd_scl;
    const uint8_t* head_nib;
    const __half* head_scl;
    const float* output_norm;
    const float* rope;
    const float* hidden_in;  // the token's embedding row as plain floats when the embedding is not Q4_0, else nullptr
    float* hidden_out;       // final residual stream as plain floats (debug reads)
    float* logits;
    // step state
    int32_t* token;          // the token to evaluate; advancing, the next one is written here
    uint32_t* position;
    int32_t* chosen;         // arg-max of the logits
    int32_t* history;
    uint32_t* history_len;
    uint32_t* epoch;         // launches so far; tags of a launch start above epoch * tags_per_launch
    uint32_t tags_per_launch;
    unsigned int* error;
    int advance;
    unsigned long long* trace;  // optional: CTA 0 stamps the end of every phase (ns)
    TokSmem sm;
};

// What this CTA does, worked out once at the start of the kernel.
struct Roles {
    uint32_t unit;                // head unit of the q/k/v multiply, or kNone
    uint32_t bd_blk0, bd_blks;    // hidden blocks of the output / down projections (bd_blks = 0: none)
    uint32_t c_blk0, c_blks;      // feed-forward blocks of gate/up
    uint32_t wtask;               // attention task, or kNone
    uint32_t off_a, off_b, off_d, off_c, off_w;  // byte offsets of the roles' buffers inside the region
    // per multiply (q/k/v, output projection, gate/up, down): rows in the buffer, 16-byte units per row, first matrix, its first
    // row, buffer offset, and for q/k/v the head's index among its kind
    uint32_t op_rows[4], op_units[4], op_mat[4], op_first[4], op_off[4], op_head;
};

// The kernel's shared memory, declared at file scope: a device function that is handed a pointer to shared memory as an
// argument sees a generic pointer and compiles generic loads and stores (measured: the serial add chains ran at 21 cycles
// per add instead of 7); a function that names the array itself gets shared-memory instructions.
extern __shared__ __align__(128) unsigned char tok_smem[];
__shared__ double g_red[kTokWarps];
__shared__ uint64_t g_exp_table[32];
__shared__ Roles g_roles;
__shared__ __align__(8) uint64_t g_bars[4];
__shared__ __align__(8) uint64_t g_hbar[kTokWarps][2];

// ---- small device helpers ---------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t saddr(const void* p) { return uint32_t(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ void cta_sync() { asm volatile("bar.sync 1, 512;" ::: "memory"); }
__device__ __forceinline__ void bar_sync(int id, int count) { asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(count) : "memory"); }
__device__ __forceinline__ void bar_arrive(int id, int count) { asm volatile("bar.arrive %0, %1;" ::"r"(id), "r"(count) : "memory"); }

__device__ __forceinline__ void mbar_init(uint64_t* b, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(saddr(b)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* b, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(saddr(b)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* b, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}" : "=r"(ok) : "r"(saddr(b)), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded: a bulk copy from valid memory always completes; if it does not within the limit the error word is set and the
// caller goes on (with garbage), so the kernel still ends.
__device__ __noinline__ void mbar_wait(uint64_t* b, uint32_t parity, unsigned int* error) {
    for (uint32_t spin = 0; !mbar_try_wait(b, parity); ++spin) {
        if (spin == kMbarLimit || poll_abandoned(spin, error)) {
            poll_failed(error);
            return;
        }
    }
}
// Global -> this CTA's shared memory, completion counted in bytes on `bar`. Both addresses 16-byte aligned, bytes % 16 == 0.
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(saddr(dst)), "l"(src), "r"(bytes),
                 "r"(saddr(bar))
                 : "memory");
}
__device__ __forceinline__ void fence_async_proxy() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

__device__ __forceinline__ unsigned long long tok_now() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

__host__ __device__ inline uint32_t part_lo(uint32_t rows, uint32_t idx, uint32_t parts) { return uint32_t(uint64_t(rows) * idx / parts); }

// first maximum wins; a NaN is never chosen (comparisons with it are false)
__device__ __forceinline__ void tok_better(float& v, int32_t& i, float ov, int32_t oi) {
    if (ov > v || (ov == v && oi < i)) {
        v = ov;
        i = oi;
    }
}

// Two tagged words with one 16-byte load, re-read until both carry `tag` (bounded). Out of line: the single polls of the
// kernel share these few instructions.
__device__ __noinline__ uint2 poll_words2(const uint2* p, uint32_t tag, unsigned int* error) {
    uint4 v = ld_pairs2(p);
    for (uint32_t spin = 0; v.y != tag || v.w != tag; ++spin) {
        if (spin == kPollLimit || poll_abandoned(spin, error)) {
            poll_failed(error);
            break;
        }
        v = ld_pairs2(p);
    }
    return make_uint2(v.x, v.z);
}
// N pairs of tagged words, `stride` words apart, ALL loads in flight together and re-read together until every tag is
// there: a vector costs one L2 round trip per re-read, not one per load. Pairs at or past `count` are skipped (zeros).
template <int N>
__device__ __forceinline__ void poll_batch(const uint2* p, uint32_t stride, uint32_t first, uint32_t count, uint32_t tag, unsigned int* error, uint2 (&out)[N]) {
    uint4 v[N];
    for (uint32_t spin = 0;; ++spin) {
        bool complete = true;
#pragma unroll
        for (int k = 0; k < N; ++k) {
            const uint32_t e = first + k * stride;
            v[k] = e < count ? ld_pairs2(p + e) : make_uint4(0u, tag, 0u, tag);
        }
#pragma unroll
        for (int k = 0; k < N; ++k) complete = complete && v[k].y == tag && v[k].w == tag;
        if (complete) break;
        if (spin == kPollLimit || poll_abandoned(spin, error)) {
            poll_failed(error);
            break;
        }
    }
#pragma unroll
    for (int k = 0; k < N; ++k) out[k] = make_uint2(v[k].x, v[k].z);
}
// One tagged value, re-read until its tag is there (bounded). Out of line, like poll_words2.
__device__ __noinline__ float poll_word(const uint2* p, uint32_t tag, unsigned int* error) {
    uint2 v = ld_pair(p);
    for (uint32_t spin = 0; v.y != tag; ++spin) {
        if (spin == kPollLimit || poll_abandoned(spin, error)) {
            poll_failed(error);
            break;
        }
        v = ld_pair(p);
    }
    return __uint_as_float(v.x);
}
// The f64 butterfly sum, once in the code: a double-precision warp instruction occupies the SM's f64 unit for 16 cycles.
__device__ __noinline__ double warp_sum_f64(double v) {
#pragma unroll 1
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ void st_word(uint2* p, uint32_t payload, uint32_t tag) { st_pair(p, __uint_as_float(payload), tag); }
// A double as two tagged words, low half first.
__device__ __forceinline__ void st_double(uint2* p, double v, uint32_t tag) {
    const unsigned long long b = (unsigned long long)__double_as_longlong(v);
    st_word(p, uint32_t(b), tag);
    st_word(p + 1, uint32_t(b >> 32), tag);
}
__device__ __forceinline__ double words_double(uint2 w) { return __longlong_as_double((long long)((unsigned long long)w.x | ((unsigned long long)w.y << 32))); }

// ---- activation prologues -------------------------------------------------------------------------------------------
struct Planes {
    unsigned char* xlo;  // per block the 8-bit values 0..15 (they meet the low nibbles of the weights)
    unsigned char* xhi;  // per block the values 16..31
    float* xd;           // per block the f16-rounded scale
    int* xs;             // per block the sum of its 32 integers
};
__device__ __forceinline__ Planes planes_of(const TokParams& P, unsigned char* smem) {
    return Planes{smem + P.sm.xlo, smem + P.sm.xhi, reinterpret_cast<float*>(smem + P.sm.xd), reinterpret_cast<int*>(smem + P.sm.xs)};
}

// f32 input (the residual stream) with its owners' sums of squares: RMS norm (rms_norm, src/model.cpp:87-97), then
// quantize_q8_0 (src/quant.cpp:115-142). x: n tagged values (n % 256 == 0, n <= 4096); sums: per 32-value block the f64
// sum of squares as two words. Thread t < n/8 owns values 8t..8t+7 from the poll to the packed bytes: a block is four
// neighbouring lanes, its maximum and its sum two shuffles each. Warp 0 alone adds the block sums (f64 is scarce) and
// hands the scale over through shared memory. Contains two CTA barriers: all 512 threads call it.
__device__ __noinline__ void prologue_f32(const TokParams& P, unsigned char* smem, double* red, const uint2* x, const uint2* sums, uint32_t tag,
                                          uint32_t n, const float* norm) {
    smem = tok_smem;
    red = g_red;
    const uint32_t tid = threadIdx.x, lane = tid & 31;
    const bool mine = tid < n / 8;  // whole warps: n / 8 is a multiple of 32
    float v[8];
    float4 w0 = make_float4(0.f, 0.f, 0.f, 0.f), w1 = w0;
    if (mine) {
        w0 = __ldg(reinterpret_cast<const float4*>(norm) + 2 * tid);  // independent of the previous operation
        w1 = __ldg(reinterpret_cast<const float4*>(norm) + 2 * tid + 1);
    }
    // ONE warp waits for the input: it polls the owners' block sums, which they publish after their values. Everybody
    // else is parked at the barrier - sixteen warps re-reading L2 in a loop slow down whatever else runs on the SM and
    // the very stores they are waiting for.
    float* fs = reinterpret_cast<float*>(red);
    if (tid >= kTokThreads - 32) {
        double total = 0.0;
        for (uint32_t b = lane; b < n / 32; b += 32) total += words_double(poll_words2(sums + 2 * b, tag, P.error));
        total = warp_sum_f64(total);
        const bool pow2 = (n & (n - 1)) == 0;
        const double recip = __longlong_as_double((long long)(1023 - (31 - __clz(int(n)))) << 52);
        const float mean = float(pow2 ? total * recip : total / double(n));
        if (lane == 0) fs[0] = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(mean, P.eps)));
    }
    cta_sync();
    if (mine) {  // the values are (all but surely) there by now; their tags are still what decides
        uint2 w[4];
        poll_batch<4>(x + 8 * tid, 2, 0, 8, tag, P.error, w);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            v[2 * k] = __uint_as_float(w[k].x);
            v[2 * k + 1] = __uint_as_float(w[k].y);
        }
    }
    if (mine) {
        const float scale = fs[0];
        v[0] = __fmul_rn(__fmul_rn(v[0], scale), w0.x); v[1] = __fmul_rn(__fmul_rn(v[1], scale), w0.y);
        v[2] = __fmul_rn(__fmul_rn(v[2], scale), w0.z); v[3] = __fmul_rn(__fmul_rn(v[3], scale), w0.w);
        v[4] = __fmul_rn(__fmul_rn(v[4], scale), w1.x); v[5] = __fmul_rn(__fmul_rn(v[5], scale), w1.y);
        v[6] = __fmul_rn(__fmul_rn(v[6], scale), w1.z); v[7] = __fmul_rn(__fmul_rn(v[7], scale), w1.w);
        float amax = 0.0f;
#pragma unroll
        for (int k = 0; k < 8; ++k) amax = fmaxf(amax, fabsf(v[k]));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
        const float dd = __fdiv_rn(amax, 127.0f);
        const float inv = dd != 0.0f ? __fdiv_rn(1.0f, dd) : 0.0f;
        int q[8], sum = 0;
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            q[k] = __float2int_rn(__fmul_rn(v[k], inv));
            sum += q[k];
        }
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
        sum += __shfl_xor_sync(0xffffffffu, sum, 2);
        const uint32_t p0 = uint32_t(q[0] & 0xFF) | (uint32_t(q[1] & 0xFF) << 8) | (uint32_t(q[2] & 0xFF) << 16) | (uint32_t(q[3] & 0xFF) << 24);
        const uint32_t p1 = uint32_t(q[4] & 0xFF) | (uint32_t(q[5] & 0xFF) << 8) | (uint32_t(q[6] & 0xFF) << 16) | (uint32_t(q[7] & 0xFF) << 24);
        const Planes pl = planes_of(P, smem);
        const uint32_t b = tid >> 2, k4 = tid & 3;
        *reinterpret_cast<uint2*>((k4 < 2 ? pl.xlo : pl.xhi) + b * 16 + (k4 & 1) * 8) = make_uint2(p0, p1);
        if (k4 == 0) {
            pl.xd[b] = __half2float(__float2half_rn(dd));
            pl.xs[b] = sum;
        }
    }
    cta_sync();
}

// Input that its owners already quantised (the attended and the gated vector): per block ten words - eight of four 8-bit
// values, the scale, the sum - copied into the planes as they arrive. One CTA barrier: all 512 threads call it.
__device__ __noinline__ void prologue_q8(const TokParams& P, unsigned char* smem, const uint2* x, uint32_t tag, uint32_t nblocks) {
    smem = tok_smem;
    const Planes pl = planes_of(P, smem);
    // TWO warps fetch the whole vector, every word of it in every re-read (a few kilobytes): the wait ends with the data
    // already in registers, and the other fourteen warps are parked at the barrier instead of re-reading L2 in a loop.
    if (threadIdx.x >= kTokThreads - 64) {  // two warps, eight pairs per lane and re-read each: up to 102 blocks in one go
        const uint32_t lane = threadIdx.x & 31, pairs = nblocks * 5;
        for (uint32_t base = ((threadIdx.x >> 5) & 1) * 8 * 32; base < pairs; base += 2 * 8 * 32) {
            uint2 w[8];
            poll_batch<8>(x, 64, 2 * (base + lane), 2 * pairs, tag, P.error, w);
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                const uint32_t e = 2 * (base + lane + 32 * k);  // word index, even
                if (e < 2 * pairs) {
                    const uint32_t blk = e / 10, wi = e - 10 * blk;
                    if (wi < 8) {
                        *reinterpret_cast<uint2*>((wi < 4 ? pl.xlo : pl.xhi) + blk * 16 + (wi & 3) * 4) = w[k];
                    } else {
                        pl.xd[blk] = __uint_as_float(w[k].x);
                        pl.xs[blk] = int(w[k].y);
                    }
                }
            }
        }
    }
    cta_sync();
}

// One warp quantises the 32 values its lanes hold (lane = index in the block) and publishes the block's ten words.
__device__ __noinline__ void publish_block_q8(uint2* dst, float r, uint32_t tag) {
    const uint32_t lane = threadIdx.x & 31;
    const float amax = warp_max(fabsf(r));
    const float dd = __fdiv_rn(amax, 127.0f);
    const float inv = dd != 0.0f ? __fdiv_rn(1.0f, dd) : 0.0f;
    const int q = __float2int_rn(__fmul_rn(r, inv));
    const int sum = warp_sum(q);
    uint32_t word = uint32_t(q & 0xFF) << (8 * (lane & 3));
    word |= __shfl_xor_sync(0xffffffffu, word, 1);
    word |= __shfl_xor_sync(0xffffffffu, word, 2);
    if ((lane & 3) == 0) st_word(dst + (lane >> 2), word, tag);
    if (lane == 1) st_word(dst + 8, __float_as_uint(__half2float(__float2half_rn(dd))), tag);
    if (lane == 2) st_word(dst + 9, uint32_t(sum), tag);
}

// A row's block terms added in block order: one dependent chain of adds, 16 per pass with their four loads on top.
// blocks is a multiple of 8.
__device__ __forceinline__ float chain_row(const float* t, uint32_t blocks) {
    float run = 0.0f;
    uint32_t b = 0;
#pragma unroll 1
    for (; b + 16 <= blocks; b += 16) {
        const float4* c4 = reinterpret_cast<const float4*>(t + b);
        const float4 p0 = c4[0], p1 = c4[1], p2 = c4[2], p3 = c4[3];
        run = __fadd_rn(run, p0.x); run = __fadd_rn(run, p0.y); run = __fadd_rn(run, p0.z); run = __fadd_rn(run, p0.w);
        run = __fadd_rn(run, p1.x); run = __fadd_rn(run, p1.y); run = __fadd_rn(run, p1.z); run = __fadd_rn(run, p1.w);
        run = __fadd_rn(run, p2.x); run = __fadd_rn(run, p2.y); run = __fadd_rn(run, p2.z); run = __fadd_rn(run, p2.w);
        run = __fadd_rn(run, p3.x); run = __fadd_rn(run, p3.y); run = __fadd_rn(run, p3.z); run = __fadd_rn(run, p3.w);
    }
    if (b < blocks) {
        const float4* c4 = reinterpret_cast<const float4*>(t + b);
        const float4 p0 = c4[0], p1 = c4[1];
        run = __fadd_rn(run, p0.x); run = __fadd_rn(run, p0.y); run = __fadd_rn(run, p0.z); run = __fadd_rn(run, p0.w);
        run = __fadd_rn(run, p1.x); run = __fadd_rn(run, p1.y); run = __fadd_rn(run, p1.z); run = __fadd_rn(run, p1.w);
    }
    return run;
}

// The block term of Q4_0 against Q8_0 (dot_q4_0_q8_0, src/quant.cpp:445-456): integer dot of the block, minus 8 times the
// sum of the activations' integers, times the two scales - weight scale first.
__device__ __forceinline__ float q4_0_term(const uint4 q, const __half d, const uint4 lo, const uint4 hi, const float xd, const int xs) {
    int acc = 0;
    acc = dp4a(q.x & 0x0F0F0F0Fu, lo.x, acc);
    acc = dp4a(q.y & 0x0F0F0F0Fu, lo.y, acc);
    acc = dp4a(q.z & 0x0F0F0F0Fu, lo.z, acc);
    acc = dp4a(q.w & 0x0F0F0F0Fu, lo.w, acc);
    acc = dp4a((q.x >> 4) & 0x0F0F0F0Fu, hi.x, acc);
    acc = dp4a((q.y >> 4) & 0x0F0F0F0Fu, hi.y, acc);
    acc = dp4a((q.z >> 4) & 0x0F0F0F0Fu, hi.z, acc);
    acc = dp4a((q.w >> 4) & 0x0F0F0F0Fu, hi.w, acc);
    acc -= 8 * xs;
    return __fmul_rn(__fmul_rn(float(acc), __half2float(d)), xd);
}

// rows x units block terms out of shared memory into the tile: every warp takes (row, 32-block chunk) tasks, lane =
// block. Chunk-major, so a warp's consecutive tasks share the activation block it holds in registers.
__device__ __noinline__ void tile_terms(const TokParams& P, unsigned char* smem, const unsigned char* w, uint32_t rows, uint32_t units) {
    smem = tok_smem;
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5, tstride = units + 4;
    const __half* ws = reinterpret_cast<const __half*>(w + size_t(rows) * units * 16);
    float* tile = reinterpret_cast<float*>(smem + P.sm.tile);
    const uint4* xlo = reinterpret_cast<const uint4*>(smem + P.sm.xlo);
    const uint4* xhi = reinterpret_cast<const uint4*>(smem + P.sm.xhi);
    const float* xd = reinterpret_cast<const float*>(smem + P.sm.xd);
    const int* xs = reinterpret_cast<const int*>(smem + P.sm.xs);
    for (uint32_t c = 0; c * 32 < units; ++c) {
        const uint32_t u = c * 32 + lane;
        if (u < units) {
            const uint4 lo = xlo[u], hi = xhi[u];
            const float xdv = xd[u];
            const int xsv = xs[u];
            // two rows per pass: their loads are issued together, ahead of the arithmetic
#pragma unroll 1
            for (uint32_t j0 = warp; j0 < rows; j0 += 2 * kTokWarps) {
                const uint32_t j1 = j0 + kTokWarps, j1c = min(j1, rows - 1);
                const uint4 q0 = *reinterpret_cast<const uint4*>(w + (size_t(j0) * units + u) * 16);
                const uint4 q1 = *reinterpret_cast<const uint4*>(w + (size_t(j1c) * units + u) * 16);
                const __half d0 = ws[j0 * units + u], d1 = ws[j1c * units + u];
                tile[j0 * tstride + u] = q4_0_term(q0, d0, lo, hi, xdv, xsv);
                if (j1 < rows) tile[j1 * tstride + u] = q4_0_term(q1, d1, lo, hi, xdv, xsv);
            }
        }
    }
}

// ---- the four multiplies of a layer --------------------------------------------------------------------------------
// kind 0: q/k/v of this CTA's head unit   1: output projection (+residual)   2: gate/up (+activation)   3: down (+residual)
struct OpRows {
    uint32_t rows, units, mat, first, off;  // rows in the buffer, 16-byte units per row, first matrix, its first row, buffer offset
};
__device__ __forceinline__ OpRows op_rows(const Roles& R, uint32_t kind) { return OpRows{R.op_rows[kind], R.op_units[kind], R.op_mat[kind], R.op_first[kind], R.op_off[kind]}; }
__device__ __forceinline__ void fill_ops(const TokParams& P, Roles& R) {  // once, by one thread
    const uint32_t dim = P.q_rows / P.heads;
    for (uint32_t kind = 0; kind < 4; ++kind) {
        uint32_t rows = 0, units = 0, mat = 0, first = 0, off = 0;
        if (kind == 0) {
            if (R.unit != kNone) {
                mat = R.unit < P.heads ? 0 : R.unit < P.heads + P.kv_heads ? 1 : 2;
                R.op_head = R.unit - (mat == 0 ? 0 : mat == 1 ? P.heads : P.heads + P.kv_heads);
                first = R.op_head * dim; rows = dim; units = P.hidden / 32; off = R.off_a;
            }
        } else if (kind == 2) {
            mat = 4; first = R.c_blk0 * 32; rows = 64 * R.c_blks; units = P.hidden / 32; off = R.off_c;
        } else {
            mat = kind == 1 ? 3 : 6; first = R.bd_blk0 * 32; rows = 32 * R.bd_blks;
            units = (kind == 1 ? P.q_rows : P.ffn) / 32; off = kind == 1 ? R.off_b : R.off_d;
        }
        R.op_rows[kind] = rows; R.op_units[kind] = units; R.op_mat[kind] = mat; R.op_first[kind] = first; R.op_off[kind] = off;
    }
}

// Requests this CTA's rows of one multiply of `layer` into the multiply's buffer (one thread). Nibbles of all rows first,
// then their scales; gate/up: the gate rows, then the same rows of up.
__device__ __noinline__ void tok_request(const TokParams& P, unsigned char* smem, const Roles&, uint64_t* bars, uint32_t kind, uint32_t layer) {
    smem = tok_smem;
    bars = g_bars;
    const Roles& R = g_roles;
    const OpRows o = op_rows(R, kind);
    if (o.rows == 0) return;
    const TokLayer& L = reinterpret_cast<const TokLayer*>(smem + P.sm.tabs)[layer];
    unsigned char* dst = smem + P.sm.region + o.off;
    fence_async_proxy();  // the buffer's last readers were generic loads
    mbar_expect_tx(&bars[kind], o.rows * o.units * 18);
    const uint32_t segs = kind == 2 ? 2 : 1, seg_rows = o.rows / segs;
    for (uint32_t s = 0; s < segs; ++s) {
        const uint32_t m = o.mat + s;
        bulk_g2s(dst + size_t(s) * seg_rows * o.units * 16, L.nib[m] + size_t(o.first) * o.units * 16, seg_rows * o.units * 16, &bars[kind]);
        bulk_g2s(dst + size_t(o.rows) * o.units * 16 + size_t(s) * seg_rows * o.units * 2, L.scl[m] + size_t(o.first) * o.units, seg_rows * o.units * 2,
                 &bars[kind]);
    }
}

// Per-head RMS norm (optional) + RoPE of one head by ONE WARP (src/model.cpp:1031-1042, :104-115), from `hv` in shared
// memory. q: the rotated head goes out as tagged words. k: it is rounded to f16, stored to the cache and published as
// the rounded value (the score of the token's own position uses the cache's value).
// `rope` (the position's cos/sin row) and `norm` (the head's norm weights, or nullptr) are copies in shared memory.
__device__ __forceinline__ void head_norm_rope(const TokParams& P, const float* hv, const float* norm, const float* rope, int neox, uint32_t dim, uint2* out,
                                               uint32_t tag, __half* cache_row) {
    const uint32_t lane = threadIdx.x & 31;
    float scale = 1.0f;
    if (norm != nullptr) {
        double part = 0.0;
#pragma unroll 1
        for (uint32_t i = lane; i < dim; i += 32) part += double(__fmul_rn(hv[i], hv[i]));
        part = warp_sum_f64(part);
        const float mean = float(part * (1.0 / double(dim)));  // the head size is a power of two: the same value as the division
        scale = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(mean, P.eps)));
    }
#pragma unroll 1
    for (uint32_t p = lane; p < dim / 2; p += 32) {
        const uint32_t ia = neox ? p : 2 * p, ib = neox ? p + dim / 2 : 2 * p + 1;
        float x0 = hv[ia], x1 = hv[ib];
        if (norm != nullptr) {
            x0 = __fmul_rn(__fmul_rn(x0, scale), norm[ia]);
            x1 = __fmul_rn(__fmul_rn(x1, scale), norm[ib]);
        }
        const float c = rope[2 * p], sn = rope[2 * p + 1];
        float y0 = __fsub_rn(__fmul_rn(x0, c), __fmul_rn(x1, sn));
        float y1 = __fadd_rn(__fmul_rn(x0, sn), __fmul_rn(x1, c));
        if (cache_row != nullptr) {
            const __half h0 = __float2half_rn(y0), h1 = __float2half_rn(y1);
            cache_row[ia] = h0;
            cache_row[ib] = h1;
            y0 = __half2float(h0);
            y1 = __half2float(h1);
        }
        st_pair(out + ia, y0, tag);
        st_pair(out + ib, y1, tag);
    }
}

// Tags of layer l start at T = base + 2 + l * kTagsPerLayer: +0 q/k/v, +1 scores, +2 exps, +3 attended, +4 output
// projection, +5 gated, +6 down projection. base + 1 is the embedding.
__device__ __noinline__ float tok_op(const TokParams& P, unsigned char* smem, double* red, const Roles&, uint64_t* bars, const uint64_t* exp_table,
                                     const uint32_t kind, const uint32_t l, const uint32_t base, const uint32_t pos, const int neox, float hres) {
    smem = tok_smem;
    red = g_red;
    bars = g_bars;
    exp_table = g_exp_table;
    const Roles& R = g_roles;
    const OpRows o = op_rows(R, kind);
    if (o.rows == 0) return hres;  // not this CTA's role: it must not read the input either
    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t par = l & 1, T = base + 2 + l * kTagsPerLayer, tstride = o.units + 4;
    const TokLayer& Ly = reinterpret_cast<const TokLayer*>(smem + P.sm.tabs)[l];
    unsigned long long* tr = TOK_TRACE_PTR(P, l, kind);
    (void)tr;
    TOK_STAMP(tr, 0);
    mbar_wait(&bars[kind], par, P.error);  // requested a layer ago: long since there
    TOK_STAMP(tr, 1);
    float* hv = reinterpret_cast<float*>(smem + P.sm.hv);  // [dim] the head's raw values | [dim] its norm weights | [dim] the position's RoPE row
    const float* head_norm = kind != 0 ? nullptr : o.mat == 0 ? Ly.q_norm : o.mat == 1 ? Ly.k_norm : nullptr;
    if (kind == 0 && warp == 8 && head_norm != nullptr) {  // a warp with nothing else to do before the first barrier
        for (uint32_t i = lane; i < o.rows; i += 32) hv[o.rows + i] = __ldg(head_norm + i);
    }
    if (kind == 0) prologue_f32(P, smem, red, P.ha[par ^ 1], P.hsa[par ^ 1], l == 0 ? base + 1 : T - kTagsPerLayer + 6, P.hidden, Ly.attn_norm);
    else if (kind == 2) prologue_f32(P, smem, red, P.hb[par], P.hsb[par], T + 4, P.hidden, Ly.ffn_norm);
    else if (kind == 1) prologue_q8(P, smem, P.aq[par], T + 3, P.q_rows / 32);
    else prologue_q8(P, smem, P.gq[par], T + 5, P.ffn / 32);
    TOK_STAMP(tr, 2);
    tile_terms(P, smem, smem + P.sm.region + o.off, o.rows, o.units);
    TOK_STAMP(tr, 3);
    cta_sync();
    TOK_STAMP(tr, 4);
    const float* tile = reinterpret_cast<const float*>(smem + P.sm.tile);
    if (kind == 0) {
        const uint32_t dim = o.rows, m = o.mat, head = R.op_head;  // head: index among the q heads, or among the K/V heads
        const float* bias = m == 0 ? Ly.q_bias : m == 1 ? Ly.k_bias : Ly.v_bias;
        float r = 0.0f;
        if (tid < dim) {
            r = chain_row(tile + tid * tstride, o.units);
            if (bias != nullptr) r = __fadd_rn(r, bias[o.first + tid]);  // add_bias, src/model.cpp:1026-1030
        }
        const size_t cache_row = (size_t(head) * P.max_context + pos) * dim;
        if (m == 2) {
            if (tid < dim) {
                st_pair(P.xv[par] + o.first + tid, r, T);
                Ly.v_cache[cache_row + tid] = __float2half_rn(r);
            }
        } else {
            if (tid < dim) hv[tid] = r;
            TOK_STAMP(tr, 5);
            cta_sync();
            TOK_STAMP(tr, 6);
            if (warp == 0) {
                head_norm_rope(P, hv, head_norm != nullptr ? hv + dim : nullptr, hv + 2 * dim, neox, dim, (m == 0 ? P.xq[par] : P.xk[par]) + o.first, T,
                               m == 0 ? nullptr : Ly.k_cache + cache_row);
            }
        }
    } else if (kind == 2) {
        const uint32_t half = o.rows / 2;
        if (tid < half) {
            const float g = chain_row(tile + tid * tstride, o.units), u = chain_row(tile + (half + tid) * tstride, o.units);
            // silu_mul_f32 (src/kernels_f32.cpp:287-289): gate / (1 + exp(-gate)) * up; or the squared ReLU (src/model.cpp:1135-1138)
            const float r = P.act == EPI_SILU_MUL ? __fmul_rn(__fdiv_rn(g, __fadd_rn(1.0f, exact_expf_tab(-g, exp_table))), u) : relu2_mul(g, u);
            publish_block_q8(P.gq[par] + size_t(R.c_blk0 + warp) * 10, r, T + 5);
        }
    } else if (tid < o.rows) {
        const uint32_t row = o.first + tid, tag_out = kind == 1 ? T + 4 : T + 6;
        hres = __fadd_rn(hres, chain_row(tile + tid * tstride, o.units));
        st_pair((kind == 1 ? P.hb[par] : P.ha[par]) + row, hres, tag_out);
        if (kind == 3 && l + 1 == P.n_layers) P.hidden_out[row] = hres;
        const double sq = warp_sum_f64(double(__fmul_rn(hres, hres)));  // whole warps: the rows are whole blocks
        if (lane == 0) st_double((kind == 1 ? P.hsb[par] : P.hsa[par]) + 2 * (R.bd_blk0 + warp), sq, tag_out);
    }
    TOK_STAMP(tr, 7);
    return hres;
}

// ---- attention -----------------------------------------------------------------------------------------------------
// Scores and exps: WARP tasks of (query head, 32 positions) dealt round-robin over the CTAs; warps 0..n_sslots-1 of a CTA
// take its tasks, each with a slice of shared memory: the query head [dim] f32 | 32 K rows of dim halves padded by 16
// bytes (so the 16-byte reads of a quarter warp fall into distinct banks). The cached rows are requested ahead; the
// token's own row arrives as tagged words (already rounded to f16) and is put in its place among them. A task computes
// its 32 scores (dot_f32's 16 interleaved partial sums, src/kernels_f32.cpp:231-254), publishes their maximum, takes the
// head's maximum from all tasks' maxima, and publishes exp(score - max) of ITS positions with their f64 sum (softmax,
// src/kernels_f32.cpp:275-284).
__device__ __forceinline__ void scores_request(const TokParams& P, unsigned char* slot, const TokLayer& L, uint32_t task, uint32_t pos, uint32_t dim) {
    const uint32_t lane = threadIdx.x & 31;
    const uint32_t chunks = (pos + 1 + 31) / 32;
    const uint32_t kvh = (task / chunks) / (P.heads / P.kv_heads), p = (task % chunks) * 32 + lane;
    if (p < pos) {
        const __half* kr = L.k_cache + (size_t(kvh) * P.max_context + p) * dim;
        const uint32_t dst = saddr(slot + dim * 4 + lane * (dim * 2 + 16));
#pragma unroll 1
        for (uint32_t i = 0; i < dim / 8; ++i) cp_async16(dst + i * 16, kr + i * 8);
    }
}

// `count` tagged values (an even number) from src into dst (shared memory), by one warp: four loads per lane in flight.
__device__ __forceinline__ void warp_fetch_words(const uint2* src, float* dst, uint32_t count, uint32_t tag, unsigned int* error) {
    const uint32_t lane = threadIdx.x & 31;
    uint2 w[4];
    poll_batch<4>(src, 64, 2 * lane, count, tag, error, w);  // heads of up to 256 values
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const uint32_t e = 2 * lane + 64 * k;
        if (e < count) {
            dst[e] = __uint_as_float(w[k].x);
            dst[e + 1] = __uint_as_float(w[k].y);
        }
    }
}

template <int VPL>
__device__ __noinline__ void tok_scores(const TokParams& P, unsigned char* smem, const uint64_t* exp_table, uint32_t l, uint32_t base, uint32_t pos,
                                        uint32_t cta, uint32_t nctas) {
    smem = tok_smem;
    exp_table = g_exp_table;
    constexpr uint32_t dim = VPL * 32;
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (warp >= P.sm.n_sslots) return;
    const TokLayer* tabs = reinterpret_cast<const TokLayer*>(smem + P.sm.tabs);
    const uint32_t par = l & 1, T = base + 2 + l * kTagsPerLayer;
    const uint32_t group = P.heads / P.kv_heads, visible = pos + 1, chunks = (visible + 31) / 32, tasks = P.heads * chunks;
    unsigned char* slot = smem + P.sm.sslot + size_t(warp) * P.sm.sslot_bytes;
    float* qs = reinterpret_cast<float*>(slot);
    unsigned char* krows = slot + dim * 4;
    const uint4* krow = reinterpret_cast<const uint4*>(krows + lane * (dim * 2 + 16));
#pragma unroll 1
    for (uint32_t i = warp;; i += P.sm.n_sslots) {
        const uint32_t task = cta + i * nctas;
        if (task >= tasks) break;
        if (i >= P.sm.n_sslots) {  // beyond the task whose rows were requested ahead
            __syncwarp();
            scores_request(P, slot, tabs[l], task, pos, dim);
            cp_async_commit();
        }
        const uint32_t h = task / chunks, chunk = task % chunks, kvh = h / group, p = chunk * 32 + lane;
        unsigned long long* tr = (i == warp && warp == 0) ? TOK_TRACE_PTR(P, l, 5) : nullptr;
        (void)tr;
        TOK_STAMP(tr, 0);
        // one lane waits for the head (its last value), then the whole warp fetches it: whole warps re-reading L2 in a loop
        // compete with whatever else runs on this SM meanwhile (a multiply, the chain of a weighted sum)
        if (lane == 0) (void)poll_word(P.xq[par] + size_t(h) * dim + dim - 1, T, P.error);
        __syncwarp();
        warp_fetch_words(P.xq[par] + size_t(h) * dim, qs, dim, T, P.error);
        if (pos / 32 == chunk) {  // the token's own K row into the place of its position
            uint2 w[4];
            poll_batch<4>(P.xk[par] + size_t(kvh) * dim, 64, 2 * lane, dim, T, P.error, w);
            __half2* own = reinterpret_cast<__half2*>(krows + (pos & 31) * (dim * 2 + 16));
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const uint32_t e = 2 * lane + 64 * k;
                if (e < dim) own[e / 2] = __floats2half2_rn(__uint_as_float(w[k].x), __uint_as_float(w[k].y));  // exact: the values are f16 already
            }
        }
        TOK_STAMP(tr, 1);
        cp_async_wait_all();
        __syncwarp();
        TOK_STAMP(tr, 2);
        float lanes[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) lanes[j] = 0.0f;
#pragma unroll 2
        for (uint32_t e = 0; e < dim; e += 16) {
            const uint4 r0 = krow[e / 8], r1 = krow[e / 8 + 1];
            const __half2* h0 = reinterpret_cast<const __half2*>(&r0);
            const __half2* h1 = reinterpret_cast<const __half2*>(&r1);
            float kf[16];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float2 f0 = __half22float2(h0[j]), f1 = __half22float2(h1[j]);
                kf[2 * j] = f0.x; kf[2 * j + 1] = f0.y; kf[8 + 2 * j] = f1.x; kf[8 + 2 * j + 1] = f1.y;
            }
            const float4* q4 = reinterpret_cast<const float4*>(qs + e);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float4 qq = q4[j];
                lanes[4 * j + 0] = __fadd_rn(lanes[4 * j + 0], __fmul_rn(qq.x, kf[4 * j + 0]));
                lanes[4 * j + 1] = __fadd_rn(lanes[4 * j + 1], __fmul_rn(qq.y, kf[4 * j + 1]));
                lanes[4 * j + 2] = __fadd_rn(lanes[4 * j + 2], __fmul_rn(qq.z, kf[4 * j + 2]));
                lanes[4 * j + 3] = __fadd_rn(lanes[4 * j + 3], __fmul_rn(qq.w, kf[4 * j + 3]));
            }
        }
        float sum = 0.0f;
#pragma unroll
        for (int j = 0; j < 16; ++j) sum = __fadd_rn(sum, lanes[j]);
        const float sc = __fmul_rn(sum, P.scale);  // lanes past the last position hold whatever their stale rows gave: never published
        TOK_STAMP(tr, 3);
        // the maximum of these 32 scores is all a head's other tasks need of them
        const uint2* maxima = P.sc[par] + size_t(h) * (P.max_context / 32);
        const float cmx = warp_max(p < visible ? sc : -INFINITY);
        if (lane == 0) st_pair(P.sc[par] + size_t(h) * (P.max_context / 32) + chunk, cmx, T + 1);
        float mx = -INFINITY;
#pragma unroll 1
        for (uint32_t c = lane; c < chunks; c += 32) mx = fmaxf(mx, poll_word(maxima + c, T + 1, P.error));
        mx = warp_max(mx);
        double part = 0.0;
        if (p < visible) {
            const float e = exact_expf_tab(__fsub_rn(sc, mx), exp_table);
            st_pair(P.ex[par] + size_t(h) * P.max_context + p, e, T + 2);
            part = double(e);
        }
        part = warp_sum_f64(part);
        if (lane == 0) st_double(P.exs[par] + 2 * (size_t(h) * (P.max_context / 32) + chunk), part, T + 2);
        TOK_STAMP(tr, 4);
    }
    // the cached K rows of this warp's first task of the next layer (same positions, the next layer's cache)
    if (l + 1 < P.n_layers && cta + warp * nctas < tasks) {
        __syncwarp();
        scores_request(P, slot, tabs[l + 1], cta + warp * nctas, pos, dim);
    }
    cp_async_commit();
}

// Rows [first, last) of this CTA's V slice into the ring (16-byte pieces, every given thread a share).
__device__ __noinline__ void values_request(const TokParams& P, unsigned char* ring, const TokLayer& L, uint32_t kvh, uint32_t slice, uint32_t dim,
                                               uint32_t first, uint32_t last, uint32_t t0, uint32_t nthreads) {
    const __half* vbase = L.v_cache + size_t(kvh) * P.max_context * dim + slice * kSliceW;
    const uint32_t base = saddr(ring);  // only its shared-window address is used
    for (uint32_t c = t0; c < (last - first) * 4; c += nthreads) {
        const uint32_t row = first + (c >> 2), piece = c & 3;
        const uint32_t at = ((row / kVChunkPos) % P.sm.ring_chunks) * kVChunkPos + row % kVChunkPos;
        cp_async16(base + (at * kSliceW + piece * 8) * 2, vbase + size_t(row) * dim + piece * 8);
    }
}

// Weighted sum: this CTA's (query head, 32 head dimensions). The sum over positions is one serial chain of f32 adds per
// dimension (src/kernels_f32.cpp:265-273), so a head is split by dimensions, never by positions. Warp 0 carries the
// chains (lane = dimension); the other 15 warps compute the products p[pos] * v[pos][c] of 128 positions at a time into
// one of two tiles, a tile ahead of the chain. V comes through a ring of 512-position chunks requested when the previous
// layer had left it (refilled behind the products for longer contexts); the token's own V row comes from the tagged v
// vector. The 32 results are one quantisation block: the chain warp quantises and publishes it.
__device__ __noinline__ void tok_attend(const TokParams& P, unsigned char* smem, double* red, const Roles&, uint32_t l, uint32_t base, uint32_t pos) {
    smem = tok_smem;
    red = g_red;
    const Roles& R = g_roles;
    if (R.wtask == kNone) return;
    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t dim = P.q_rows / P.heads, slices = dim / kSliceW, group = P.heads / P.kv_heads;
    const uint32_t h = R.wtask / slices, slice = R.wtask % slices, kvh = h / group, visible = pos + 1;
    const uint32_t par = l & 1, T = base + 2 + l * kTagsPerLayer;
    const TokLayer* tabs = reinterpret_cast<const TokLayer*>(smem + P.sm.tabs);
    unsigned char* wbase = smem + P.sm.region + R.off_w;
    float* ps = reinterpret_cast<float*>(wbase);
    unsigned char* ring = wbase + P.max_context * 4;
    const __half* vring = reinterpret_cast<const __half*>(ring);
    __half* vown = reinterpret_cast<__half*>(ring + size_t(P.sm.ring_chunks) * kVChunkPos * kSliceW * 2);
    float* prod = reinterpret_cast<float*>(reinterpret_cast<unsigned char*>(vown) + 128);
    unsigned long long* tr = TOK_TRACE_PTR(P, l, 4);
    (void)tr;
    // Everybody meets here first: the warps that have nothing left to do for the previous layer's task wait, parked, for
    // its chain warp and for this CTA's score tasks - sixteen warps polling L2 in a loop would slow exactly those down.
    cta_sync();
    TOK_STAMP(tr, 0);
    if (warp == 1 || warp == 3) {
        // TWO warps fetch the head's softmax: the tasks' partial sums for the denominator, then every exp - all words of a
        // batch in every re-read, so the wait ends with the data in registers. p = e * float(1 / sum), scaled as it is stored.
        const uint32_t chunks = (visible + 31) / 32;
        double total = 0.0;
        for (uint32_t c = lane; c < chunks; c += 32) total += words_double(poll_words2(P.exs[par] + 2 * (size_t(h) * (P.max_context / 32) + c), T + 2, P.error));
        total = warp_sum_f64(total);
        const float inv = float(1.0 / total);
        const uint2* src = P.ex[par] + size_t(h) * P.max_context;
        const uint32_t even = visible & ~1u;  // pairs; an odd last word alone
        for (uint32_t base = (warp >> 1) * 8 * 64; base < even; base += 2 * 8 * 64) {  // eight pairs per lane and re-read: 512 positions per warp and pass
            uint2 w[8];
            poll_batch<8>(src, 64, base + 2 * lane, even, T + 2, P.error, w);
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                const uint32_t e = base + 2 * lane + 64 * k;
                if (e < even) {
                    ps[e] = __fmul_rn(__uint_as_float(w[k].x), inv);
                    ps[e + 1] = __fmul_rn(__uint_as_float(w[k].y), inv);
                }
            }
        }
        if (warp == 1 && lane == 0 && (visible & 1u)) ps[visible - 1] = __fmul_rn(poll_word(src + visible - 1, T + 2, P.error), inv);
    } else if (warp == 2) {  // the token's own V row, rounded as the cache rounds it
        vown[lane] = __float2half_rn(poll_word(P.xv[par] + size_t(kvh) * dim + slice * kSliceW + lane, T, P.error));
    }
    TOK_STAMP(tr, 2);
    cp_async_wait_all();  // this thread's share of the first V chunks
    TOK_STAMP(tr, 3);
    cta_sync();
    TOK_STAMP(tr, 4);
#ifdef BK_TOK_TRACE
    if (tr != nullptr) tr[9] = tok_now();
#endif
    const uint32_t nsub = (visible + kSub - 1) / kSub;
    const uint32_t ring_pos = P.sm.ring_chunks * kVChunkPos;
    const bool refills = pos > ring_pos;  // positions beyond what the ring held at the start
    // Products and chain ALTERNATE: all sixteen warps fill the tile with the products of 256 positions, then warp 0 alone adds
    // them while the others are parked at the barrier. Overlapping the two (products of the next tile during the chain)
    // measured slower: the chain then ran at 15-21 cycles per add instead of 7.
    const uint32_t c8 = lane & 7, r4 = lane >> 3;  // a lane's four columns 4 * c8 .. 4 * c8 + 3, its position within a group of four
    float acc = 0.0f;
#ifdef BK_TOK_TRACE
    if (tr != nullptr) tr[8] = 0;
#endif
    for (uint32_t s = 0; s < nsub; ++s) {
        const uint32_t first = s * kSub, rows = min(kSub, visible - first);
        if (refills && first != 0 && first % kVChunkPos == 0) {
            const uint32_t c = first / kVChunkPos;  // entering chunk c: chunk c - 1 is consumed (the barrier after its last chain)
            const uint32_t from = (c - 1 + P.sm.ring_chunks) * kVChunkPos;
            if (from < pos) values_request(P, ring, tabs[l], kvh, slice, dim, from, min(pos, from + kVChunkPos), tid, kTokThreads);
            cp_async_commit();
            asm volatile("cp.async.wait_group 1;" ::: "memory");  // everything but the chunk just requested: chunk c has landed
            cta_sync();
        }
        // The tile is [position][32 columns]. A lane computes four columns of one position - one 8-byte load of V, one of the
        // probability, one 16-byte store - so a product costs 2.5 instructions (written column-major, one product per
        // instruction, the products took three times as long as the chain they feed). The chain reads one float per add.
        const uint32_t at0 = ((first / kVChunkPos) % P.sm.ring_chunks) * kVChunkPos + first % kVChunkPos;  // a tile lies inside one chunk
#pragma unroll 2
        for (uint32_t r = warp * 4 + r4; r < rows; r += 4 * kTokWarps) {
            const uint32_t p = first + r;
            const uint2 raw = p == pos ? *reinterpret_cast<const uint2*>(vown + 4 * c8) : *reinterpret_cast<const uint2*>(vring + (at0 + r) * kSliceW + 4 * c8);
            const float2 v01 = __half22float2(*reinterpret_cast<const __half2*>(&raw.x)), v23 = __half22float2(*reinterpret_cast<const __half2*>(&raw.y));
            const float pr = ps[p];
            *reinterpret_cast<float4*>(prod + r * kSliceW + 4 * c8) = make_float4(__fmul_rn(pr, v01.x), __fmul_rn(pr, v01.y), __fmul_rn(pr, v23.x), __fmul_rn(pr, v23.y));
        }
        cta_sync();
#ifdef BK_TOK_TRACE
        const long long c0 = clock64();
#endif
        if (warp == 0) {
            const float* col = prod + lane;
            uint32_t j = 0;
            // 16 adds per pass with their loads on top
#pragma unroll 1
            for (; j + 16 <= rows; j += 16) {
                float t[16];
#pragma unroll
                for (int k = 0; k < 16; ++k) t[k] = col[(j + k) * kSliceW];
#pragma unroll
                for (int k = 0; k < 16; ++k) acc = __fadd_rn(acc, t[k]);
            }
            for (; j < rows; ++j) acc = __fadd_rn(acc, col[j * kSliceW]);
        }
#ifdef BK_TOK_TRACE
        if (tr != nullptr) tr[8] += (unsigned long long)(clock64() - c0);  // cycles in the chains alone
#endif
        if (s + 1 < nsub) cta_sync();  // the tile is free for the next 256 positions
    }
    TOK_STAMP(tr, 5);
    // the ring is free: the next layer's V slice (the same positions of its cache) - by the warps that have nothing else to do
    if (warp != 0 && l + 1 < P.n_layers) values_request(P, ring, tabs[l + 1], kvh, slice, dim, 0, min(pos, ring_pos), tid - 32, kTokThreads - 32);
    if (warp == 0) publish_block_q8(P.aq[par] + size_t(R.wtask) * 10, acc, T + 3);
    TOK_STAMP(tr, 6);
    cp_async_commit();
}

// ---- output head -------------------------------------------------------------------------------------------------
// Every CTA multiplies a contiguous range of the vocabulary's rows. A warp owns whole chunks of head_rows rows and
// streams them through two private slots: lane 0 requests chunk i + 2 into the slot chunk i just left, so no other warp
// is involved and nothing but the warp's own mbarrier is waited on.
struct HeadWalk {
    uint32_t lo, rows, chunks, units;
};
__device__ __forceinline__ HeadWalk head_walk(const TokParams& P, uint32_t cta, uint32_t nctas) {
    HeadWalk w;
    w.lo = part_lo(P.vocab, cta, nctas);
    w.rows = part_lo(P.vocab, cta + 1, nctas) - w.lo;
    w.chunks = (w.rows + P.sm.head_rows - 1) / P.sm.head_rows;
    w.units = P.hidden / 32;
    return w;
}
__device__ __forceinline__ void head_request(const TokParams& P, unsigned char* smem, const HeadWalk& w, uint32_t warp, uint32_t i, uint64_t* bar) {
    const uint32_t chunk = warp + i * kTokWarps;  // the warp's i-th chunk
    if (chunk >= w.chunks) return;
    const uint32_t hr = P.sm.head_rows, first = chunk * hr, nrows = min(hr, w.rows - first);
    unsigned char* slot = smem + P.sm.region + size_t(warp * 2 + (i & 1)) * P.sm.ring_slot_bytes;
    mbar_expect_tx(bar, nrows * w.units * 18);
    bulk_g2s(slot, P.head_nib + size_t(w.lo + first) * w.units * 16, nrows * w.units * 16, bar);
    bulk_g2s(slot + size_t(hr) * w.units * 16, P.head_scl + size_t(w.lo + first) * w.units, nrows * w.units * 2, bar);
}

__device__ __noinline__ void tok_head(const TokParams& P, unsigned char* smem, double* red, uint64_t (*hbar)[2], float* sv, int* si, uint32_t base,
                                      uint32_t pos, uint32_t cta, uint32_t nctas) {
    smem = tok_smem;
    red = g_red;
    hbar = g_hbar;
    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, L = P.n_layers;
    const HeadWalk w = head_walk(P, cta, nctas);
    const uint32_t units = w.units, tstride = units + 4, hr = P.sm.head_rows;
    const uint32_t tag_part = base + 2 + L * kTagsPerLayer;
    // every buffer of the layers is free now: the head's first chunks stream while the last residual values arrive
    cta_sync();
    if (lane == 0) {
        fence_async_proxy();
        head_request(P, smem, w, warp, 0, &hbar[warp][0]);
        head_request(P, smem, w, warp, 1, &hbar[warp][1]);
    }
    prologue_f32(P, smem, red, P.ha[(L - 1) & 1], P.hsa[(L - 1) & 1], base + 2 + (L - 1) * kTagsPerLayer + 6, P.hidden, P.output_norm);
    const uint4* xlo = reinterpret_cast<const uint4*>(smem + P.sm.xlo);
    const uint4* xhi = reinterpret_cast<const uint4*>(smem + P.sm.xhi);
    const float* xd = reinterpret_cast<const float*>(smem + P.sm.xd);
    const int* xs = reinterpret_cast<const int*>(smem + P.sm.xs);
    float* tile = reinterpret_cast<float*>(smem + P.sm.tile) + size_t(warp) * hr * tstride;
    float best = -INFINITY, first_logit = 0.0f;
    int32_t best_i = 0x7fffffff;
    for (uint32_t i = 0;; ++i) {
        const uint32_t chunk = warp + i * kTokWarps;
        if (chunk >= w.chunks) break;
        const uint32_t first = chunk * hr, nrows = min(hr, w.rows - first);
        const unsigned char* slot = smem + P.sm.region + size_t(warp * 2 + (i & 1)) * P.sm.ring_slot_bytes;
        const __half* ws = reinterpret_cast<const __half*>(slot + size_t(hr) * units * 16);
        mbar_wait(&hbar[warp][i & 1], (i >> 1) & 1, P.error);
        for (uint32_t u = lane; u < units; u += 32) {
            const uint4 lo = xlo[u], hi = xhi[u];
            const float xdv = xd[u];
            const int xsv = xs[u];
            for (uint32_t j = 0; j < nrows; ++j) {
                const uint4 q = *reinterpret_cast<const uint4*>(slot + (size_t(j) * units + u) * 16);
                tile[j * tstride + u] = q4_0_term(q, ws[j * units + u], lo, hi, xdv, xsv);
            }
        }
        __syncwarp();
        if (lane < nrows) {
            const float logit = chain_row(tile + lane * tstride, units);
            const uint32_t row = w.lo + first + lane;
            P.logits[row] = logit;
            if (row == 0) first_logit = logit;
            tok_better(best, best_i, logit, int32_t(row));
        }
        __syncwarp();  // the slot and the tile are free
        if (lane == 0) {
            fence_async_proxy();
            head_request(P, smem, w, warp, i + 2, &hbar[warp][i & 1]);
        }
    }
    // the CTA's candidate, then CTA 0 gathers all of them
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) tok_better(best, best_i, __shfl_xor_sync(0xffffffffu, best, o), __shfl_xor_sync(0xffffffffu, best_i, o));
    if (lane == 0) {
        sv[warp] = best;
        si[warp] = best_i;
    }
    cta_sync();
    if (warp == 0) {
        if (lane == 0) {
            for (uint32_t k = 1; k < kTokWarps; ++k) tok_better(best, best_i, sv[k], si[k]);
            st_pair(P.part + 2 * cta, best, tag_part);
            st_pair(P.part + 2 * cta + 1, __int_as_float(best_i), tag_part);
        }
        if (cta == 0) {
            float v = -INFINITY;
            int32_t idx = 0x7fffffff;
            for (uint32_t c0 = 0; c0 < nctas; c0 += 8 * 32) {  // up to eight candidates per lane in flight
                uint2 w2[8];
                poll_batch<8>(P.part, 64, c0 * 2 + 2 * lane, 2 * nctas, tag_part, P.error, w2);
#pragma unroll
                for (int k = 0; k < 8; ++k) {
                    if (c0 + lane + 32 * k < nctas) tok_better(v, idx, __uint_as_float(w2[k].x), int32_t(w2[k].y));
                }
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) tok_better(v, idx, __shfl_xor_sync(0xffffffffu, v, o), __shfl_xor_sync(0xffffffffu, idx, o));
            if (lane == 0) {
                // std::max_element (src/sampler.cpp:11-13): a NaN is never preferred, and a NaN at index 0 is never displaced
                if (first_logit != first_logit || uint32_t(idx) >= P.vocab) idx = 0;
                *P.chosen = idx;
                if (P.advance) {
                    *P.token = idx;
                    *P.position = pos + 1;
                    if (P.history != nullptr) {
                        const uint32_t n = *P.history_len;
                        P.history[n] = idx;
                        *P.history_len = n + 1;
                    }
                }
                *P.epoch = *P.epoch + 1;  // every CTA read it when the kernel started
            }
        }
    }
}

// ---- the kernel ----------------------------------------------------------------------------------------------------
template <int VPL, bool NEOX>
__global__ void __launch_bounds__(kTokThreads, 1) token_kernel(const __grid_constant__ TokParams P) {
    unsigned char* smem = tok_smem;
    double* red = g_red;
    __shared__ float sv[kTokWarps];
    __shared__ int si[kTokWarps];
    uint64_t* bars = g_bars;
    uint64_t (*hbar)[2] = g_hbar;
    uint64_t* exp_table = g_exp_table;
    Roles& R = g_roles;
    constexpr uint32_t dim = VPL * 32;
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, cta = blockIdx.x, nctas = gridDim.x;
    const uint32_t L = P.n_layers;
    constexpr uint32_t kIssuer = kTokThreads - 32;  // lane 0 of the last warp: never on the chain of a row sum

    if (tid == 0) {
        for (int k = 0; k < 4; ++k) mbar_init(&bars[k], 1);
        for (uint32_t k = 0; k < kTokWarps; ++k) {
            mbar_init(&hbar[k][0], 1);
            mbar_init(&hbar[k][1], 1);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        fence_async_proxy();
        Roles r;
        r.unit = cta < P.n_units ? cta : kNone;
        const uint32_t hb = P.hidden / 32, fb = P.ffn / 32, slices = dim / kSliceW;
        r.bd_blk0 = r.bd_blks = r.c_blk0 = r.c_blks = 0;
        if (cta >= P.bd_first && cta < P.bd_first + P.bd_ctas) {
            r.bd_blk0 = part_lo(hb, cta - P.bd_first, P.bd_ctas);
            r.bd_blks = part_lo(hb, cta - P.bd_first + 1, P.bd_ctas) - r.bd_blk0;
        }
        if (cta >= P.c_first && cta < P.c_first + P.c_ctas) {
            r.c_blk0 = part_lo(fb, cta - P.c_first, P.c_ctas);
            r.c_blks = part_lo(fb, cta - P.c_first + 1, P.c_ctas) - r.c_blk0;
        }
        r.wtask = (cta >= P.w_first && cta - P.w_first < P.heads * slices) ? cta - P.w_first : kNone;
        uint32_t off = 0;
        r.off_a = off; if (r.unit != kNone) off += P.sm.size_a;
        r.off_b = off; if (r.bd_blks != 0) off += P.sm.size_b;
        r.off_d = off; if (r.bd_blks != 0) off += P.sm.size_d;
        r.off_c = off; if (r.c_blks != 0) off += P.sm.size_c;
        r.off_w = off;
        r.op_head = 0;
        fill_ops(P, r);
        R = r;
    }
    if (tid < 32) exp_table[tid] = exp2_table_device()[tid];
    if (tid >= 64 && tid < 64 + dim) reinterpret_cast<float*>(smem + P.sm.hv)[2 * dim + tid - 64] = __ldg(P.rope + size_t(*P.position) * dim + tid - 64);
    {   // every layer's table into shared memory: the pointers are read on the way to each request
        const uint4* src = reinterpret_cast<const uint4*>(P.layers);
        uint4* dst = reinterpret_cast<uint4*>(smem + P.sm.tabs);
        for (uint32_t i = tid; i < L * (sizeof(TokLayer) / 16); i += kTokThreads) dst[i] = __ldg(src + i);
    }
    const uint32_t pos = *P.position;
    const uint32_t base = *P.epoch * P.tags_per_launch;
    uint32_t token = uint32_t(*P.token);
    if (token >= P.vocab) token = 0;  // ids from the host are checked there, ids chosen on the device where they are chosen: the last guard
    __syncthreads();
    const TokLayer* tabs = reinterpret_cast<const TokLayer*>(smem + P.sm.tabs);
    if (tid == kIssuer) {
        for (uint32_t k = 0; k < 4; ++k) tok_request(P, smem, R, bars, k, 0);
    }
    // what does not depend on this token: the cached K rows of this CTA's first score tasks, the V slice of its weighted sum
    if (warp < P.sm.n_sslots && cta + warp * nctas < P.heads * ((pos + 32) / 32)) {
        scores_request(P, smem + P.sm.sslot + size_t(warp) * P.sm.sslot_bytes, tabs[0], cta + warp * nctas, pos, dim);
    }
    if (R.wtask != kNone) {
        const uint32_t slices = dim / kSliceW, h = R.wtask / slices;
        values_request(P, smem + P.sm.region + R.off_w + P.max_context * 4, tabs[0], h / (P.heads / P.kv_heads), R.wtask % slices, dim, 0,
                       min(pos, P.sm.ring_chunks * kVChunkPos), tid, kTokThreads);
    }
    cp_async_commit();
    // development aid: thread 0 of CTAs 0, 40, 100 and the last one stamp the end of every phase (ns), a section each
    const uint32_t traced = cta == 0 ? 0 : cta == 40 ? 1 : cta == 100 ? 2 : cta == nctas - 1 ? 3 : kNone;
    unsigned long long* trace = (P.trace != nullptr && traced != kNone && tid == 0) ? P.trace + traced * (2 + L * 6) : nullptr;
    if (trace) trace[0] = tok_now();

    // the token's embedding row: the owners of the hidden blocks dequantise their values (embedding_row, src/model.cpp:27-70)
    float hres = 0.0f;
    if (tid < 32 * R.bd_blks) {
        const uint32_t r = R.bd_blk0 * 32 + tid;
        if (P.hidden_in != nullptr) {
            hres = P.hidden_in[r];
        } else {
            const uint32_t units = P.hidden / 32, u = r >> 5, wi = r & 31;
            const size_t unit = size_t(token) * units + u;
            const uint32_t byte = P.embd_nib[unit * 16 + (wi & 15)];
            const int q = int(wi < 16 ? (byte & 0xFu) : (byte >> 4));
            hres = __fmul_rn(float(q - 8), __half2float(P.embd_scl[unit]));
        }
        st_pair(P.ha[1] + r, hres, base + 1);
        const double sq = warp_sum_f64(double(__fmul_rn(hres, hres)));
        if (lane == 0) st_double(P.hsa[1] + 2 * (R.bd_blk0 + warp), sq, base + 1);
    }

    for (uint32_t l = 0; l < L; ++l) {
        const bool more = l + 1 < L;
        hres = tok_op(P, smem, red, R, bars, exp_table, 0, l, base, pos, NEOX, hres);
        if (tid == kIssuer && more) tok_request(P, smem, R, bars, 0, l + 1);
        if (trace) trace[1 + l * 6 + 0] = tok_now();
        tok_scores<VPL>(P, smem, exp_table, l, base, pos, cta, nctas);
        if (trace) trace[1 + l * 6 + 1] = tok_now();
        tok_attend(P, smem, red, R, l, base, pos);
        if (trace) trace[1 + l * 6 + 2] = tok_now();
        hres = tok_op(P, smem, red, R, bars, exp_table, 1, l, base, pos, NEOX, hres);
        if (tid == kIssuer && more) tok_request(P, smem, R, bars, 1, l + 1);
        if (trace) trace[1 + l * 6 + 3] = tok_now();
        hres = tok_op(P, smem, red, R, bars, exp_table, 2, l, base, pos, NEOX, hres);
        if (tid == kIssuer && more) tok_request(P, smem, R, bars, 2, l + 1);
        if (trace) trace[1 + l * 6 + 4] = tok_now();
        hres = tok_op(P, smem, red, R, bars, exp_table, 3, l, base, pos, NEOX, hres);
        if (tid == kIssuer && more) tok_request(P, smem, R, bars, 3, l + 1);
        if (trace) trace[1 + l * 6 + 5] = tok_now();
    }
    tok_head(P, smem, red, hbar, sv, si, base, pos, cta, nctas);
    if (trace) trace[1 + L * 6] = tok_now();
}

}  // namespace

// ---- host side -------------------------------------------------------------------------------------------------------
struct TokenPlan::Impl {
    TokParams params{};
    void (*kernel)(TokParams) = nullptr;
    TokLayer* layers_dev = nullptr;
    uint2* pairs_dev = nullptr;
    size_t pairs = 0;
    uint32_t* words_dev = nullptr;  // [0] epoch, [1] error
    uint32_t grid = 0;
    uint64_t launches_since_wipe = 0;
};

TokenPlan::TokenPlan() = default;
TokenPlan::~TokenPlan() {
    if (impl_ != nullptr) {
        if (impl_->layers_dev) cudaFree(impl_->layers_dev);
        if (impl_->pairs_dev) cudaFree(impl_->pairs_dev);
        if (impl_->words_dev) cudaFree(impl_->words_dev);
        delete impl_;
    }
}

namespace {
uint32_t align_up(uint32_t v, uint32_t a) { return (v + a - 1) / a * a; }
uint32_t ceil_div(uint32_t a, uint32_t b) { return (a + b - 1) / b; }
}  // namespace

bool TokenPlan::build(const std::vector<StepLayerArgs>& layers, const StepShared& sh, const TokenEnds& ends, uint32_t sms, cudaStream_t s, std::string& why_not) {
    if (layers.empty() || layers.size() > 96) {
        why_not = "layer count outside 1..96";
        return false;
    }
    for (const StepLayerArgs& L : layers) {
        for (const DevMatrix* m : {&L.q, &L.k, &L.v, &L.o, &L.gate, &L.up, &L.down}) {
            if (m->type != T_Q4_0) {
                why_not = "a layer matrix is not Q4_0";
                return false;
            }
        }
        if (L.attn_sub_norm != nullptr || L.ffn_sub_norm != nullptr) {
            why_not = "sub-norms ahead of the output or down projection";
            return false;
        }
    }
    if (ends.head.type != T_Q4_0) {
        why_not = "the output head is not Q4_0";
        return false;
    }
    const uint32_t dim = sh.dim, q_dim = sh.heads * dim, kv_dim = sh.kv_heads * dim, group = sh.heads / sh.kv_heads;
    if (sh.hidden_size % 256 != 0 || sh.hidden_size > 4096 || q_dim % 256 != 0 || sh.ffn_size % 256 != 0) {
        why_not = "a row length is not a multiple of 256, or the hidden size exceeds 4096";
        return false;
    }
    if ((dim != 64 && dim != 128) || group > 8) {
        why_not = "head size is not 64 or 128, or more than 8 query heads per K/V head";
        return false;
    }
    if (sh.max_context % 32 != 0) {
        why_not = "the context length is not a multiple of 32";
        return false;
    }
    const uint32_t n_units = sh.heads + 2 * sh.kv_heads, wtasks = sh.heads * (dim / kSliceW);
    if (n_units > sms || wtasks > sms || ends.vocab < sms) {
        why_not = "more heads (or fewer vocabulary rows) than SMs";
        return false;
    }
    int dev = 0, limit = 0, coop = 0;
    BK_CUDA(cudaGetDevice(&dev));
    BK_CUDA(cudaDeviceGetAttribute(&limit, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev));
    BK_CUDA(cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, dev));
    if (coop == 0) {
        why_not = "the device has no cooperative launch";
        return false;
    }

    // Who does what. q/k/v: one head unit per CTA from CTA 0. Output and down projection: the hidden blocks over the CTAs
    // after those (or over all of them). Gate/up: the feed-forward blocks from CTA 0. Attention: the last CTAs.
    const uint32_t L = uint32_t(layers.size());
    const uint32_t hu = sh.hidden_size / 32, qu = q_dim / 32, fu = sh.ffn_size / 32;
    TokParams base{};
    base.n_units = n_units;
    base.bd_ctas = std::min(hu, sms - std::min(n_units, sms - 1));
    base.bd_first = n_units + base.bd_ctas <= sms ? n_units : sms - base.bd_ctas;
    base.c_ctas = std::min(fu, sms);
    base.c_first = 0;
    base.w_first = sms - wtasks;
    const uint32_t bd_blks = ceil_div(hu, base.bd_ctas), c_blks = ceil_div(fu, base.c_ctas);
    const uint32_t size_a = align_up(dim * hu * 18, 128), size_b = align_up(32 * bd_blks * qu * 18, 128), size_d = align_up(32 * bd_blks * fu * 18, 128),
                   size_c = align_up(64 * c_blks * hu * 18, 128);
    TokSmem best{};
    bool fits = false;
    const uint32_t tries[][2] = {{4, 3}, {4, 2}, {3, 2}, {2, 3}, {2, 2}, {1, 2}};  // score slots, V ring chunks
    for (const auto& t : tries) {
        for (uint32_t hr : {8u, 4u, 2u, 1u}) {
            if (fits) break;
            TokSmem m{};
            m.n_sslots = t[0];
            m.ring_chunks = t[1];
            m.head_rows = hr;
            m.size_a = size_a; m.size_b = size_b; m.size_d = size_d; m.size_c = size_c;
            const uint32_t size_w = align_up(sh.max_context * 4 + m.ring_chunks * kVChunkPos * kSliceW * 2 + 128 + kSliceW * kSub * 4, 128);
            const uint32_t widest = std::max(std::max(sh.hidden_size, q_dim), sh.ffn_size);
            uint32_t off = 0;
            m.tabs = off; off = align_up(off + L * uint32_t(sizeof(TokLayer)), 128);
            m.xlo = off; off += widest / 32 * 16;
            m.xhi = off; off += widest / 32 * 16;
            m.xd = off; off += widest / 32 * 4;
            m.xs = off; off = align_up(off + widest / 32 * 4, 128);
            const uint32_t op_tile = std::max(std::max(dim * (hu + 4), 32 * bd_blks * (qu + 4)), std::max(64 * c_blks * (hu + 4), 32 * bd_blks * (fu + 4)));
            m.tile = off; off = align_up(off + std::max(op_tile, kTokWarps * hr * (hu + 4)) * 4, 128);
            m.hv = off; off += 3 * dim * 4;
            uint32_t region = 0;  // the largest sum of role buffers over the CTAs
            for (uint32_t cta = 0; cta < sms; ++cta) {
                uint32_t need = 0;
                if (cta < n_units) need += size_a;
                if (cta >= base.bd_first && cta < base.bd_first + base.bd_ctas) need += size_b + size_d;
                if (cta >= base.c_first && cta < base.c_first + base.c_ctas) need += size_c;
                if (cta >= base.w_first) need += size_w;
                region = std::max(region, need);
            }
            m.region = off; off += region;
            m.sslot_bytes = align_up(dim * 4 + 32 * (dim * 2 + 16), 128);
            m.sslot = off; off += m.n_sslots * m.sslot_bytes;
            m.ring_slot_bytes = hr * hu * 18;
            if (2 * kTokWarps * m.ring_slot_bytes > off - m.region) continue;  // the head's ring lies over the region and the score slots
            m.total = off;
            if (m.total + 4096 <= uint32_t(limit)) {
                best = m;
                fits = true;
            }
        }
        if (fits) break;
    }
    if (!fits) {
        why_not = "one SM's share of a layer's weights and the attention buffers exceed its shared memory";
        return false;
    }

    void (*kernel)(TokParams) = dim == 128 ? (sh.neox ? token_kernel<4, true> : token_kernel<4, false>) : (sh.neox ? token_kernel<2, true> : token_kernel<2, false>);
    BK_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(best.total)));
    int per_sm = 0;
    BK_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, int(kTokThreads), best.total));
    if (per_sm < 1) {
        why_not = "the kernel does not fit an SM";
        return false;
    }

    auto impl = std::make_unique<Impl>();
    impl->kernel = kernel;
    impl->grid = sms;
    const size_t rows_ctx = size_t(sh.heads) * sh.max_context;
    const size_t maxima = (rows_ctx / 32 + 1) & ~size_t(1);  // an even count keeps the next vector 16-byte aligned
    const size_t per_copy = 2 * (size_t(sh.hidden_size) + 2 * hu) + q_dim + 2 * kv_dim + maxima + rows_ctx + 2 * rows_ctx / 32 + size_t(qu) * 10 + size_t(fu) * 10;
    impl->pairs = 2 * per_copy + 2 * size_t(sms);
    BK_CUDA(cudaMalloc(&impl->pairs_dev, impl->pairs * sizeof(uint2)));
    BK_CUDA(cudaMemsetAsync(impl->pairs_dev, 0, impl->pairs * sizeof(uint2), s));  // tag 0 is never expected
    BK_CUDA(cudaMalloc(&impl->words_dev, 64));
    BK_CUDA(cudaMemsetAsync(impl->words_dev, 0, 64, s));
    const uint32_t one = 1;
    BK_CUDA(cudaMemcpyAsync(impl->words_dev, &one, sizeof(one), cudaMemcpyHostToDevice, s));  // epoch starts at 1

    TokParams& P = impl->params;
    P = base;
    uint2* at = impl->pairs_dev;
    auto take = [&](size_t n) {  // every vector starts 16-byte aligned: all counts are even
        uint2* p = at;
        at += n;
        return p;
    };
    for (int c = 0; c < 2; ++c) {
        P.ha[c] = take(sh.hidden_size);
        P.hsa[c] = take(2 * hu);
        P.hb[c] = take(sh.hidden_size);
        P.hsb[c] = take(2 * hu);
        P.xq[c] = take(q_dim);
        P.xk[c] = take(kv_dim);
        P.xv[c] = take(kv_dim);
        P.sc[c] = take(maxima);
        P.ex[c] = take(rows_ctx);
        P.exs[c] = take(2 * rows_ctx / 32);
        P.aq[c] = take(size_t(qu) * 10);
        P.gq[c] = take(size_t(fu) * 10);
    }
    P.part = take(2 * size_t(sms));

    std::vector<TokLayer> tabs(L);
    for (uint32_t l = 0; l < L; ++l) {
        const StepLayerArgs& A = layers[l];
        TokLayer& t = tabs[l];
        std::memset(static_cast<void*>(&t), 0, sizeof(t));
        const DevMatrix* ms[7] = {&A.q, &A.k, &A.v, &A.o, &A.gate, &A.up, &A.down};
        for (int k = 0; k < 7; ++k) {
            t.nib[k] = ms[k]->qa;
            t.scl[k] = ms[k]->d;
        }
        t.attn_norm = A.attn_norm; t.ffn_norm = A.ffn_norm; t.q_norm = A.q_norm; t.k_norm = A.k_norm;
        t.q_bias = A.q_bias; t.k_bias = A.k_bias; t.v_bias = A.v_bias;
        t.k_cache = A.k_cache; t.v_cache = A.v_cache;
    }
    BK_CUDA(cudaMalloc(&impl->layers_dev, L * sizeof(TokLayer)));
    BK_CUDA(cudaMemcpyAsync(impl->layers_dev, tabs.data(), L * sizeof(TokLayer), cudaMemcpyHostToDevice, s));
    BK_CUDA(cudaStreamSynchronize(s));  // tabs goes out of scope

    P.layers = impl->layers_dev;
    P.n_layers = L;
    P.hidden = sh.hidden_size; P.q_rows = q_dim; P.kv_rows = kv_dim; P.ffn = sh.ffn_size; P.heads = sh.heads; P.kv_heads = sh.kv_heads;
    P.vocab = ends.vocab; P.max_context = sh.max_context; P.eps = sh.eps; P.scale = sh.scale; P.act = sh.act_epi;
    embd_q4_0_ = ends.embd.type == T_Q4_0;
    P.embd_nib = ends.embd.qa; P.embd_scl = ends.embd.d;
    P.head_nib = ends.head.qa; P.head_scl = ends.head.d;
    P.output_norm = ends.output_norm; P.rope = sh.rope;
    P.hidden_in = embd_q4_0_ ? nullptr : sh.hidden;
    P.hidden_out = sh.hidden; P.logits = ends.logits;
    P.token = ends.token; P.position = const_cast<uint32_t*>(sh.position); P.chosen = ends.chosen;
    P.history = ends.history; P.history_len = ends.history_len;
    P.epoch = impl->words_dev; P.error = impl->words_dev + 1;
    P.tags_per_launch = L * kTagsPerLayer + 8;
    P.sm = best;
    impl_ = impl.release();
    char text[200];
    std::snprintf(text, sizeof text, "one launch per token: %u CTAs (%u head units, %u hidden-block, %u feed-forward-block, %u attention), %u KB shared, %u score slots, "
                  "V ring of %u chunks, head chunks of %u rows", sms, n_units, base.bd_ctas, base.c_ctas, wtasks, best.total / 1024, best.n_sslots, best.ring_chunks,
                  best.head_rows);
    description_ = text;
    return true;
}

void TokenPlan::launch(cudaStream_t s, bool advance) {
    // Tags must never repeat while old words are still in the buffers: long before the 32-bit range runs out, wipe them.
    if ((impl_->launches_since_wipe + 2) * impl_->params.tags_per_launch >= (uint64_t(1) << 32)) {
        BK_CUDA(cudaMemsetAsync(impl_->pairs_dev, 0, impl_->pairs * sizeof(uint2), s));
        const uint32_t one = 1;
        BK_CUDA(cudaMemcpyAsync(impl_->words_dev, &one, sizeof(one), cudaMemcpyHostToDevice, s));
        impl_->launches_since_wipe = 0;
    }
    ++impl_->launches_since_wipe;
    TokParams P = impl_->params;
    P.advance = advance ? 1 : 0;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(impl_->grid);
    cfg.blockDim = dim3(kTokThreads);
    cfg.dynamicSmemBytes = P.sm.total;
    cfg.stream = s;
    cudaLaunchAttribute attr{};
    attr.id = cudaLaunchAttributeCooperative;
    attr.val.cooperative = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    BK_CUDA(cudaLaunchKernelEx(&cfg, impl_->kernel, P));
}

void TokenPlan::set_trace(unsigned long long* words) { impl_->params.trace = words; }
const unsigned int* TokenPlan::error_word() const { return impl_->words_dev + 1; }
void TokenPlan::rearm(cudaStream_t s) {
    BK_CUDA(cudaMemsetAsync(impl_->words_dev + 1, 0, sizeof(uint32_t), s));
    BK_CUDA(cudaStreamSynchronize(s));
}

}  // namespace bk
