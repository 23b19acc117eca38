// One decoded token as ONE kernel launch: embedding row -> every layer -> output head -> arg-max -> next token and
// position, for models whose layer matrices are Q4_0 and small enough that one SM's share of a layer's weights fits its
// shared memory (the 0.6B class). One 512-thread CTA per SM, launched cooperatively so that all CTAs are resident.
//
// What bounds a token of such a model is not HBM (a layer is 9 MB: 1.4 us at full bandwidth) but the chain of ~170
// dependent operations, each needing the whole result vector of the one before. The kernel is arranged around that:
//
//   * WEIGHTS NEVER WAIT FOR ACTIVATIONS. Every CTA owns a fixed, contiguous range of each matrix's rows. Its share of
//     an operation's weights (nibble plane and scale plane, two cp.async.bulk copies per matrix segment, completion on
//     an mbarrier) is requested one whole layer ahead - the moment the same operation of the previous layer has
//     finished with the buffer - so when an operation's input arrives its weights are already in shared memory.
//     K rows and V slices of the cached positions are requested at the start of the layer in the same spirit.
//   * OPERATIONS HAND OVER THROUGH TAGGED PAIRS in L2 (see decode_body.cuh): each element is one 64-bit {value, tag}
//     store; consumers re-read until the tag of this token, layer and operation is there. No grid barrier, no fence.
//     Exchange vectors alternate between two copies by layer parity, so a vector is rewritten two layers later.
//   * THE RESIDUAL STREAM LIVES IN REGISTERS of the threads that own its rows (the o and down projections split the
//     hidden rows the same way), and is only broadcast, never read back.
//   * ONE PROLOGUE PER OPERATION: the threads that fetched the input vector keep it in registers, reduce the sum of
//     squares, scale, and quantise to 8 bits with two shuffles per 32-value block (8 values per thread); then every warp
//     multiplies (row, 32-block chunk) tasks out of shared memory, and one thread per row adds the row's block terms in
//     block order - the reference's order (src/quant.cpp:445-456, src/kernels.cpp:13-30).
//   * THE HEAD STREAMS through per-warp double-buffered bulk copies (8 rows each) over the shared memory the layers no
//     longer need, requested while the last down projection still runs; every CTA reduces its rows' maximum, CTA 0
//     gathers the 148 candidates, applies std::max_element's rule (src/sampler.cpp:11-13) and feeds the next step.
//
// All float arithmetic is the reference's, in the reference's order; results are bit-identical to the CPU engine and to
// the other single-token paths. Every wait (tagged pairs, mbarriers) is bounded and ends in the error word.
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
constexpr uint32_t kVRingChunks = 3;           // chunks the ring holds
constexpr uint32_t kSub = 128;                 // positions per product tile of the weighted sum
constexpr uint32_t kSubStride = kSub + 4;      // floats per column of a product tile
constexpr uint32_t kTagsPerLayer = 8;
constexpr uint32_t kMbarLimit = 1u << 22;      // try_wait rounds before a bulk copy is declared lost

struct alignas(16) TokLayer {
    const uint8_t* nib[7];  // q k v o gate up down: 16-byte units of nibbles, row-major
    const __half* scl[7];   // their f16 block scales
    const float* attn_norm;
    const float* ffn_norm;
    const float* q_norm;
    const float* k_norm;
    const float* attn_sub_norm;
    const float* ffn_sub_norm;
    const float* q_bias;
    const float* k_bias;
    const float* v_bias;
    __half* k_cache;
    __half* v_cache;
    uint64_t pad;
};
static_assert(sizeof(TokLayer) % 16 == 0, "copied in 16-byte pieces");

struct TokSmem {  // byte offsets into dynamic shared memory
    uint32_t tabs, xlo, xhi, xd, xs, tile, w_down, w_qkv, w_o, w_gu, sslot, ps, vring, vown, prod, ring, total;
    uint32_t sslot_bytes, n_sslots, head_rows, ring_slot_bytes;
};

struct TokParams {
    const TokLayer* layers;
    uint32_t n_layers;
    uint32_t hidden, q_rows, kv_rows, ffn, heads, kv_heads, vocab, max_context;
    float eps, scale;
    int act;  // EPI_SILU_MUL or EPI_RELU2_MUL
    // tagged exchange vectors, two copies each (layer parity)
    uint2* hid_a[2];   // residual stream after the embedding / a down projection
    uint2* hid_b[2];   // after an output projection
    uint2* xq[2];
    uint2* xk[2];
    uint2* xv[2];
    uint2* sc[2];      // scores [heads][max_context]
    uint2* att[2];
    uint2* gated[2];
    uint2* part;       // per CTA: {best value, tag}, {best index, tag}
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
    const int32_t* token;    // the token to evaluate
    uint32_t* position;
    int32_t* chosen;         // arg-max of the logits
    int32_t* token_slot;     // advance: next input token (may alias `token`)
    int32_t* history;
    uint32_t* history_len;
    uint32_t* epoch;         // launches so far; tags of a launch start above epoch * tags_per_launch
    uint32_t tags_per_launch;
    unsigned int* error;
    int advance;
    uint32_t slice_w;        // columns of V per weighted-sum CTA (16 or 32)
    unsigned long long* trace;  // optional: CTA 0 stamps the end of every phase (ns)
    TokSmem sm;
};

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
__device__ __forceinline__ void mbar_wait(uint64_t* b, uint32_t parity, unsigned int* error) {
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
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ unsigned long long tok_now() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

__host__ __device__ inline uint32_t part_lo(uint32_t rows, uint32_t cta, uint32_t nctas) { return uint32_t(uint64_t(rows) * cta / nctas); }

// `count` tagged values (a multiple of 64) from src into shared memory at dst, by one warp; bounded re-reads.
__device__ __forceinline__ void warp_fetch_pairs(const uint2* src, float* dst, uint32_t count, uint32_t tag, unsigned int* error) {
    const uint32_t lane = threadIdx.x & 31;
    const uint4* src2 = reinterpret_cast<const uint4*>(src);
    for (uint32_t base = 0; base < count / 2; base += 64) {
        uint4 v[2];
        for (uint32_t spin = 0;; ++spin) {
            v[0] = ld_pairs2(src2 + base + lane);
            v[1] = ld_pairs2(src2 + base + 32 + lane);
            if (v[0].y == tag && v[0].w == tag && v[1].y == tag && v[1].w == tag) break;
            if (spin == kPollLimit || poll_abandoned(spin, error)) {
                poll_failed(error);
                break;
            }
        }
#pragma unroll
        for (int k = 0; k < 2; ++k) {
            const uint32_t i = base + 32 * k + lane;
            dst[2 * i] = __uint_as_float(v[k].x);
            dst[2 * i + 1] = __uint_as_float(v[k].z);
        }
    }
}

// first maximum wins; a NaN is never chosen (comparisons with it are false)
__device__ __forceinline__ void tok_better(float& v, int32_t& i, float ov, int32_t oi) {
    if (ov > v || (ov == v && oi < i)) {
        v = ov;
        i = oi;
    }
}

// ---- one multiply --------------------------------------------------------------------------------------------------
struct Shape {  // this CTA's share of one operation: up to three runs of rows, each inside one matrix
    uint32_t rows, nseg;
    uint32_t seg_rows[3], seg_first[3], seg_mat[3];
};

// The tagged vector x (n values; n % 256 == 0, n <= 4096) -> optional RMS norm -> Q8_0 planes in shared memory
// (quantize_q8_0, src/quant.cpp:115-142; rms_norm, src/model.cpp:87-97). Thread t < n/8 owns values 8t..8t+7 from the poll
// to the packed bytes: a 32-value block is four neighbouring lanes, its maximum and its sum two shuffles each.
// Contains CTA barriers: all 512 threads call it.
#define TOK_STAMP(tr, k) do { if ((tr) != nullptr) (tr)[k] = tok_now(); } while (0)
__device__ __forceinline__ void tok_prologue(const TokParams& P, unsigned char* smem, double* red, const uint2* x, uint32_t tag, uint32_t n,
                                             const float* norm, unsigned long long* tr = nullptr) {
    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const bool mine = tid < n / 8;  // whole warps: n / 8 is a multiple of 32
    float v[8];
    float4 w0 = make_float4(0.f, 0.f, 0.f, 0.f), w1 = w0;
    if (mine) {
        if (norm != nullptr) {  // independent of the previous operation: in flight while the poll waits
            w0 = __ldg(reinterpret_cast<const float4*>(norm) + 2 * tid);
            w1 = __ldg(reinterpret_cast<const float4*>(norm) + 2 * tid + 1);
        }
        const uint4* src = reinterpret_cast<const uint4*>(x) + 4 * tid;
        uint4 a[4];
        for (uint32_t spin = 0;; ++spin) {
#pragma unroll
            for (int k = 0; k < 4; ++k) a[k] = ld_pairs2(src + k);
            bool complete = true;
#pragma unroll
            for (int k = 0; k < 4; ++k) complete = complete && a[k].y == tag && a[k].w == tag;
            if (complete) break;
            if (spin == kPollLimit || poll_abandoned(spin, P.error)) {
                poll_failed(P.error);
                break;
            }
        }
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            v[2 * k] = __uint_as_float(a[k].x);
            v[2 * k + 1] = __uint_as_float(a[k].z);
        }
    } else {
#pragma unroll
        for (int k = 0; k < 8; ++k) v[k] = 0.0f;
    }
    TOK_STAMP(tr, 2);
    if (norm != nullptr) {
        double part = 0.0;
#pragma unroll
        for (int k = 0; k < 8; ++k) part += double(__fmul_rn(v[k], v[k]));
        part = warp_sum(part);
        if (lane == 0) red[warp] = part;
        cta_sync();
        TOK_STAMP(tr, 3);
        double total = 0.0;
#pragma unroll
        for (uint32_t w = 0; w < kTokWarps; ++w) total += red[w];
        const bool pow2 = (n & (n - 1)) == 0;
        const double recip = __longlong_as_double((long long)(1023 - (31 - __clz(int(n)))) << 52);
        const float mean = float(pow2 ? total * recip : total / double(n));
        const float scale = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(mean, P.eps)));
        v[0] = __fmul_rn(__fmul_rn(v[0], scale), w0.x); v[1] = __fmul_rn(__fmul_rn(v[1], scale), w0.y);
        v[2] = __fmul_rn(__fmul_rn(v[2], scale), w0.z); v[3] = __fmul_rn(__fmul_rn(v[3], scale), w0.w);
        v[4] = __fmul_rn(__fmul_rn(v[4], scale), w1.x); v[5] = __fmul_rn(__fmul_rn(v[5], scale), w1.y);
        v[6] = __fmul_rn(__fmul_rn(v[6], scale), w1.z); v[7] = __fmul_rn(__fmul_rn(v[7], scale), w1.w);
    }
    if (mine) {
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
        // values 0..15 of a block meet the low nibbles of its weights, 16..31 the high nibbles: two planes of 16 bytes per block
        const uint32_t b = tid >> 2, k4 = tid & 3;
        unsigned char* plane = smem + (k4 < 2 ? P.sm.xlo : P.sm.xhi) + b * 16 + (k4 & 1) * 8;
        *reinterpret_cast<uint2*>(plane) = make_uint2(p0, p1);
        if (k4 == 0) {
            reinterpret_cast<float*>(smem + P.sm.xd)[b] = __half2float(__float2half_rn(dd));
            reinterpret_cast<int*>(smem + P.sm.xs)[b] = sum;
        }
    }
    TOK_STAMP(tr, 4);
    cta_sync();
    TOK_STAMP(tr, 5);
}

__device__ __forceinline__ float chain_row(const float* t, uint32_t blocks) {
    float run = 0.0f;
#pragma unroll 4
    for (uint32_t b = 0; b < blocks; b += 4) {
        const float4 q = *reinterpret_cast<const float4*>(t + b);
        run = __fadd_rn(run, q.x); run = __fadd_rn(run, q.y); run = __fadd_rn(run, q.z); run = __fadd_rn(run, q.w);
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

struct MulArgs {
    const uint2* x;
    uint32_t tag_x, tag_out, cols;
    const float* norm;
    const unsigned char* w;  // shared memory: this CTA's rows
    uint64_t* bar;
    uint32_t parity;
    int kind;                // 0: store per matrix (q/k/v), 1: add to the residual, 2: gate/up pair
    unsigned long long* tr;  // development aid: 10 stamps of this thread, or nullptr
    uint2* out[3];           // per segment
    float* plain;            // kind 1: also the plain copy of the result, or nullptr
    int act;
};

// One operation of this CTA: returns the residual value of row `tid` of the CTA's hidden rows (kind 1 updates it).
__device__ __noinline__ float tok_multiply(const TokParams& P, unsigned char* smem, double* red, const Shape& sh, const MulArgs& a, float hres) {
    if (sh.rows == 0) return hres;  // no rows here: this CTA must not read the input either
    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t units = a.cols / 32, tstride = units + 4;
    TOK_STAMP(a.tr, 0);
    mbar_wait(a.bar, a.parity, P.error);  // requested a layer ago: long since there
    TOK_STAMP(a.tr, 1);
    tok_prologue(P, smem, red, a.x, a.tag_x, a.cols, a.norm, a.tr);
    const unsigned char* wn = a.w;
    const __half* ws = reinterpret_cast<const __half*>(a.w + size_t(sh.rows) * units * 16);
    float* tile = reinterpret_cast<float*>(smem + P.sm.tile);
    const uint4* xlo = reinterpret_cast<const uint4*>(smem + P.sm.xlo);
    const uint4* xhi = reinterpret_cast<const uint4*>(smem + P.sm.xhi);
    const float* xd = reinterpret_cast<const float*>(smem + P.sm.xd);
    const int* xs = reinterpret_cast<const int*>(smem + P.sm.xs);
    const uint32_t chunks = (units + 31) / 32, tasks = sh.rows * chunks;
    uint32_t cur = 0xffffffffu;
    uint4 lo = make_uint4(0, 0, 0, 0), hi = lo;
    float xdv = 0.0f;
    int xsv = 0;
    for (uint32_t t = warp; t < tasks; t += kTokWarps) {  // chunk-major: a warp's consecutive tasks share the activation block
        const uint32_t c = t / sh.rows, j = t - c * sh.rows, u = c * 32 + lane;
        const bool valid = u < units;
        const uint32_t uu = valid ? u : 0;
        if (c != cur) {
            lo = xlo[uu]; hi = xhi[uu]; xdv = xd[uu]; xsv = xs[uu];
            cur = c;
        }
        const uint4 q = *reinterpret_cast<const uint4*>(wn + (size_t(j) * units + uu) * 16);
        const __half d = ws[j * units + uu];
        const float term = q4_0_term(q, d, lo, hi, xdv, xsv);
        if (valid) tile[j * tstride + u] = term;
    }
    TOK_STAMP(a.tr, 6);
    cta_sync();
    TOK_STAMP(a.tr, 7);
    if (a.kind == 2) {
        const uint32_t pairs = sh.rows / 2;
        if (tid < pairs) {
            const float* tg = tile + tid * tstride;
            const float* tu = tile + (pairs + tid) * tstride;
            float g = 0.0f, u = 0.0f;
#pragma unroll 2
            for (uint32_t b = 0; b < units; b += 4) {
                const float4 qg = *reinterpret_cast<const float4*>(tg + b), qu = *reinterpret_cast<const float4*>(tu + b);
                g = __fadd_rn(g, qg.x); u = __fadd_rn(u, qu.x);
                g = __fadd_rn(g, qg.y); u = __fadd_rn(u, qu.y);
                g = __fadd_rn(g, qg.z); u = __fadd_rn(u, qu.z);
                g = __fadd_rn(g, qg.w); u = __fadd_rn(u, qu.w);
            }
            const float r = a.act == EPI_SILU_MUL ? silu_mul(g, u) : relu2_mul(g, u);
            st_pair(a.out[0] + sh.seg_first[0] + tid, r, a.tag_out);
        }
    } else if (tid < sh.rows) {
        const float sum = chain_row(tile + tid * tstride, units);
        uint32_t j = tid, s = 0;
        while (j >= sh.seg_rows[s]) {
            j -= sh.seg_rows[s];
            ++s;
        }
        const uint32_t row = sh.seg_first[s] + j;
        if (a.kind == 1) {
            hres = __fadd_rn(hres, sum);
            st_pair(a.out[s] + row, hres, a.tag_out);
            if (a.plain != nullptr) a.plain[row] = hres;
        } else {
            st_pair(a.out[s] + row, sum, a.tag_out);
        }
    }
    TOK_STAMP(a.tr, 8);
    return hres;
}

// Requests this CTA's rows of one operation of `layer` into the operation's buffer (one thread).
__device__ __forceinline__ void tok_request(const Shape& sh, const TokLayer& L, unsigned char* dst, uint32_t cols, uint64_t* bar) {
    const uint32_t units = cols / 32;
    mbar_expect_tx(bar, sh.rows * units * 18);
    uint32_t joff = 0;
    for (uint32_t s = 0; s < sh.nseg; ++s) {
        const uint32_t m = sh.seg_mat[s], first = sh.seg_first[s], rows = sh.seg_rows[s];
        bulk_g2s(dst + size_t(joff) * units * 16, L.nib[m] + size_t(first) * units * 16, rows * units * 16, bar);
        bulk_g2s(dst + size_t(sh.rows) * units * 16 + size_t(joff) * units * 2, L.scl[m] + size_t(first) * units, rows * units * 2, bar);
        joff += rows;
    }
}

// ---- attention -----------------------------------------------------------------------------------------------------
// Scores: WARP tasks of (K/V head, 32 positions) dealt round-robin over the CTAs; the warps 0..n_sslots-1 of a CTA take
// its tasks, each with its own slice of shared memory: the group's query heads [group][dim] f32, the new K row [dim]
// f32, and 32 cached K rows of dim halves padded by 16 bytes (so that the 16-byte reads of a quarter warp fall into
// distinct banks). The K rows of a warp's first task are requested at the start of the layer. The task that covers the
// token's own position also norms, rotates and stores the new K row and stores the new V row.
__device__ __forceinline__ uint32_t score_tasks(const TokParams& P, uint32_t pos) { return P.kv_heads * ((pos + 1 + 31) / 32); }

template <int VPL>
__device__ __forceinline__ void scores_request(const TokParams& P, unsigned char* slot, const TokLayer& L, uint32_t task, uint32_t pos) {
    constexpr uint32_t dim = VPL * 32;
    const uint32_t lane = threadIdx.x & 31, group = P.heads / P.kv_heads;
    const uint32_t chunks = (pos + 1 + 31) / 32;
    const uint32_t kvh = task / chunks, p = (task % chunks) * 32 + lane;
    if (p < pos) {
        const __half* kr = L.k_cache + (size_t(kvh) * P.max_context + p) * dim;
        const uint32_t dst = saddr(slot + size_t(group + 1) * dim * 4 + size_t(lane) * (dim * 2 + 16));
#pragma unroll
        for (uint32_t i = 0; i < dim / 8; ++i) cp_async16(dst + i * 16, kr + i * 8);
    }
}

template <int VPL, bool NEOX>
__device__ __forceinline__ void tok_scores(const TokParams& P, unsigned char* smem, const TokLayer& L, uint32_t par, uint32_t tag_in, uint32_t tag_out,
                                           uint32_t pos, uint32_t cta, uint32_t nctas) {
    constexpr uint32_t dim = VPL * 32;
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (warp >= P.sm.n_sslots) return;
    const uint32_t group = P.heads / P.kv_heads, visible = pos + 1, chunks = (visible + 31) / 32, tasks = P.kv_heads * chunks;
    unsigned char* slot = smem + P.sm.sslot + size_t(warp) * P.sm.sslot_bytes;
    float* qs = reinterpret_cast<float*>(slot);
    float* knew = qs + group * dim;
    const uint4* krow = reinterpret_cast<const uint4*>(slot + size_t(group + 1) * dim * 4 + size_t(lane) * (dim * 2 + 16));
    const float* rope = P.rope + size_t(pos) * dim;
    for (uint32_t i = warp;; i += P.sm.n_sslots) {
        const uint32_t task = cta + i * nctas;
        if (task >= tasks) break;
        if (i >= P.sm.n_sslots) {  // beyond the task whose rows were requested at the start of the layer
            __syncwarp();
            scores_request<VPL>(P, slot, L, task, pos);
            cp_async_commit();
        }
        const uint32_t kvh = task / chunks, begin = (task % chunks) * 32, p = begin + lane;
        const bool owner = pos >= begin && pos < begin + 32, cached = p < pos;
        // the raw query heads of the group (adjacent in the q vector) and, for the owner, the raw new K row
        {
            const uint4* src = reinterpret_cast<const uint4*>(P.xq[par] + size_t(kvh) * group * dim);
            const uint32_t n2 = group * dim / 2;  // 16-byte pieces of two pairs
            for (uint32_t base = 0; base < n2; base += 64) {
                uint4 v[2];
                for (uint32_t spin = 0;; ++spin) {
                    bool complete = true;
#pragma unroll
                    for (int k = 0; k < 2; ++k) {
                        const uint32_t e = base + 32 * k + lane;
                        v[k] = e < n2 ? ld_pairs2(src + e) : make_uint4(0u, tag_in, 0u, tag_in);
                        complete = complete && v[k].y == tag_in && v[k].w == tag_in;
                    }
                    if (complete) break;
                    if (spin == kPollLimit || poll_abandoned(spin, P.error)) {
                        poll_failed(P.error);
                        break;
                    }
                }
#pragma unroll
                for (int k = 0; k < 2; ++k) {
                    const uint32_t e = base + 32 * k + lane;
                    if (e < n2) {
                        qs[2 * e] = __uint_as_float(v[k].x);
                        qs[2 * e + 1] = __uint_as_float(v[k].z);
                    }
                }
            }
            if (owner) {
                for (uint32_t e = lane; e < dim; e += 32) knew[e] = poll_pair(P.xk[par] + size_t(kvh) * dim + e, tag_in, P.error);
            }
        }
        __syncwarp();
        if (owner) {
            float kv[VPL];
#pragma unroll
            for (int k = 0; k < VPL; ++k) {
                const uint32_t e = NEOX ? lane + 32 * k : VPL * lane + k;
                kv[k] = knew[e];
                if (L.k_bias != nullptr) kv[k] = __fadd_rn(kv[k], L.k_bias[size_t(kvh) * dim + e]);  // add_bias, src/model.cpp:1026-1030
            }
            warp_head_norm_rope<VPL, NEOX>(kv, L.k_norm, rope, P.eps, knew);
            __syncwarp();
            const size_t row = (size_t(kvh) * P.max_context + pos) * dim;
            for (uint32_t e = lane; e < dim; e += 32) {
                const __half kh = __float2half_rn(knew[e]);
                knew[e] = __half2float(kh);  // the score of the own position uses the cache's f16 value
                L.k_cache[row + e] = kh;
                float v = poll_pair(P.xv[par] + size_t(kvh) * dim + e, tag_in, P.error);
                if (L.v_bias != nullptr) v = __fadd_rn(v, L.v_bias[size_t(kvh) * dim + e]);
                L.v_cache[row + e] = __float2half_rn(v);
            }
        }
        for (uint32_t g = 0; g < group; ++g) {
            float v[VPL];
#pragma unroll
            for (int k = 0; k < VPL; ++k) {
                const uint32_t e = NEOX ? lane + 32 * k : VPL * lane + k;
                v[k] = qs[g * dim + e];
                if (L.q_bias != nullptr) v[k] = __fadd_rn(v[k], L.q_bias[size_t(kvh * group + g) * dim + e]);
            }
            warp_head_norm_rope<VPL, NEOX>(v, L.q_norm, rope, P.eps, qs + g * dim);
        }
        // this lane's K row: the first task's rows were committed before the V slice's (one group may still be in flight)
        if (i < P.sm.n_sslots) cp_async_wait<1>();
        else cp_async_wait<0>();
        __syncwarp();
        if (p < visible) {
            for (uint32_t g = 0; g < group; ++g) {
                const float* q = qs + g * dim;
                float lanes[16];
#pragma unroll
                for (int j = 0; j < 16; ++j) lanes[j] = 0.0f;
#pragma unroll
                for (uint32_t e = 0; e < dim; e += 16) {
                    float kf[16];
                    if (!cached) {
#pragma unroll
                        for (int j = 0; j < 16; ++j) kf[j] = knew[e + j];
                    } else {
                        const uint4 r0 = krow[e / 8], r1 = krow[e / 8 + 1];
                        const __half2* h0 = reinterpret_cast<const __half2*>(&r0);
                        const __half2* h1 = reinterpret_cast<const __half2*>(&r1);
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const float2 f0 = __half22float2(h0[j]), f1 = __half22float2(h1[j]);
                            kf[2 * j] = f0.x; kf[2 * j + 1] = f0.y; kf[8 + 2 * j] = f1.x; kf[8 + 2 * j + 1] = f1.y;
                        }
                    }
                    const float4* q4 = reinterpret_cast<const float4*>(q + e);
#pragma unroll
                    for (int j = 0; j < 4; ++j) {  // dot_f32's 16 interleaved partial sums (src/kernels_f32.cpp:231-254)
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
                st_pair(P.sc[par] + size_t(kvh * group + g) * P.max_context + p, __fmul_rn(sum, P.scale), tag_out);
            }
        }
    }
}

// Softmax + weighted sum: CTA `cta` < heads * slices takes (query head, slice of slice_w head dimensions). The sum over
// positions is one serial chain of f32 adds per dimension (src/kernels_f32.cpp:265-273), so a head is split by
// dimensions, never by positions. Warp 0 carries the chains (lane = dimension); the other 15 warps compute the products
// p[pos] * v[pos][c] of 128 positions at a time into one of two tiles, a tile ahead of the chain. V comes through a
// ring of three 512-position chunks requested at the start of the layer (refilled behind the products for longer
// contexts); the token's own V row comes from the tagged v vector.
__device__ __forceinline__ void values_request(const TokParams& P, unsigned char* smem, const TokLayer& L, uint32_t cta, uint32_t first, uint32_t last,
                                               uint32_t tid0, uint32_t nthreads) {
    const uint32_t dim = P.q_rows / P.heads, width = P.slice_w, slices = dim / width, group = P.heads / P.kv_heads;
    const uint32_t h = cta / slices, slice = cta % slices, kvh = h / group;
    const uint32_t ppr = width / 8;  // 16-byte pieces per position
    const __half* vbase = L.v_cache + size_t(kvh) * P.max_context * dim + slice * width;
    const uint32_t ring = saddr(smem + P.sm.vring);
    constexpr uint32_t kRingPos = kVChunkPos * kVRingChunks;
    for (uint32_t c = tid0; c < (last - first) * ppr; c += nthreads) {
        const uint32_t row = first + c / ppr, piece = c % ppr;
        cp_async16(ring + ((row % kRingPos) * width + piece * 8) * 2, vbase + size_t(row) * dim + piece * 8);
    }
}

__device__ __noinline__ void tok_attend(const TokParams& P, unsigned char* smem, double* red, float* redf, const TokLayer& L, uint32_t par,
                                        uint32_t tag_qkv, uint32_t tag_scores, uint32_t tag_out, uint32_t pos, uint32_t cta, unsigned long long* tr) {
    const uint32_t dim = P.q_rows / P.heads, width = P.slice_w, slices = dim / width, group = P.heads / P.kv_heads;
    if (cta >= P.heads * slices) return;
    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t h = cta / slices, slice = cta % slices, kvh = h / group, visible = pos + 1;
    constexpr uint32_t kRingPos = kVChunkPos * kVRingChunks;
    float* ps = reinterpret_cast<float*>(smem + P.sm.ps);
    const __half* vring = reinterpret_cast<const __half*>(smem + P.sm.vring);
    __half* vown = reinterpret_cast<__half*>(smem + P.sm.vown);
    float* prod = reinterpret_cast<float*>(smem + P.sm.prod);
    const uint2* scores = P.sc[par] + size_t(h) * P.max_context;

    // softmax (src/kernels_f32.cpp:275-284): max, e = expf(s - max), f64 sum, p = e * float(1 / sum)
    TOK_STAMP(tr, 0);
    float mx = -INFINITY;
    for (uint32_t p = tid; p < visible; p += kTokThreads) {
        const float v = poll_pair(scores + p, tag_scores, P.error);
        ps[p] = v;
        mx = fmaxf(mx, v);
    }
    TOK_STAMP(tr, 1);
    mx = warp_max(mx);
    if (lane == 0) redf[warp] = mx;
    cta_sync();
    TOK_STAMP(tr, 2);
    mx = redf[0];
#pragma unroll
    for (uint32_t w = 1; w < kTokWarps; ++w) mx = fmaxf(mx, redf[w]);
    double part = 0.0;
    for (uint32_t p = tid; p < visible; p += kTokThreads) {
        const float e = exact_expf(__fsub_rn(ps[p], mx));
        ps[p] = e;
        part += double(e);
    }
    part = warp_sum(part);
    if (lane == 0) red[warp] = part;
    if (tid < width) {  // the token's own V row, rounded as the cache rounds it
        float v = poll_pair(P.xv[par] + size_t(kvh) * dim + slice * width + tid, tag_qkv, P.error);
        if (L.v_bias != nullptr) v = __fadd_rn(v, L.v_bias[size_t(kvh) * dim + slice * width + tid]);
        vown[tid] = __float2half_rn(v);
    }
    TOK_STAMP(tr, 3);
    cta_sync();
    TOK_STAMP(tr, 4);
    double total = 0.0;
#pragma unroll
    for (uint32_t w = 0; w < kTokWarps; ++w) total += red[w];
    const float inv = float(1.0 / total);
    for (uint32_t p = tid; p < visible; p += kTokThreads) ps[p] = __fmul_rn(ps[p], inv);
    cp_async_wait<0>();  // this thread's share of the first V chunks
    TOK_STAMP(tr, 5);
    cta_sync();
    TOK_STAMP(tr, 6);

    const uint32_t nsub = (visible + kSub - 1) / kSub;
    const bool refills = pos > kRingPos;  // positions beyond what the ring held at the start
    if (warp == 0) {
        float acc = 0.0f;
        for (uint32_t s = 0; s < nsub; ++s) {
            const uint32_t b = s & 1, rows = min(kSub, visible - s * kSub);
            bar_sync(2 + b, kTokThreads);  // tile b holds the products of sub-chunk s
            if (lane < width) {
                const float* mine = prod + (size_t(b) * width + lane) * kSubStride;
                uint32_t j = 0;
#pragma unroll 4
                for (; j + 4 <= rows; j += 4) {
                    const float4 q = *reinterpret_cast<const float4*>(mine + j);
                    acc = __fadd_rn(acc, q.x); acc = __fadd_rn(acc, q.y); acc = __fadd_rn(acc, q.z); acc = __fadd_rn(acc, q.w);
                }
                for (; j < rows; ++j) acc = __fadd_rn(acc, mine[j]);
            }
            if (s + 2 < nsub) bar_arrive(4 + b, kTokThreads);  // tile b may be rewritten
        }
        if (lane < width) st_pair(P.att[par] + size_t(h) * dim + slice * width + lane, acc, tag_out);
        TOK_STAMP(tr, 7);
    } else {
        const uint32_t ptid = tid - 32, nprod = kTokThreads - 32;
        for (uint32_t s = 0; s < nsub; ++s) {
            const uint32_t b = s & 1, base = s * kSub, rows = min(kSub, visible - base);
            if (refills && base != 0 && base % kVChunkPos == 0) {
                const uint32_t c = base / kVChunkPos;  // entering chunk c: chunk c - 1 is consumed once every producer is here
                bar_sync(6, nprod);
                const uint32_t first = (c + 2) * kVChunkPos, last = min(pos, first + kVChunkPos);
                if (first < pos) values_request(P, smem, L, cta, first, last, ptid, nprod);
                cp_async_commit();
                cp_async_wait<1>();  // everything but the chunk just requested: chunk c has landed
                bar_sync(6, nprod);
            }
            if (s >= 2) bar_sync(4 + b, kTokThreads);  // the chain is done with tile b
            float* tile = prod + size_t(b) * width * kSubStride;
            for (uint32_t e = ptid; e < rows * width; e += nprod) {
                const uint32_t r = e / width, col = e % width, p = base + r;
                const __half vv = p == pos ? vown[col] : vring[(p % kRingPos) * width + col];
                tile[col * kSubStride + r] = __fmul_rn(ps[p], __half2float(vv));
            }
            bar_arrive(2 + b, kTokThreads);
        }
    }
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
    unsigned char* slot = smem + P.sm.ring + size_t(warp * 2 + (i & 1)) * P.sm.ring_slot_bytes;
    mbar_expect_tx(bar, nrows * w.units * 18);
    bulk_g2s(slot, P.head_nib + size_t(w.lo + first) * w.units * 16, nrows * w.units * 16, bar);
    bulk_g2s(slot + size_t(hr) * w.units * 16, P.head_scl + size_t(w.lo + first) * w.units, nrows * w.units * 2, bar);
}

__device__ __noinline__ void tok_head(const TokParams& P, unsigned char* smem, double* red, uint64_t (*hbar)[2], float* sv, int* si, const uint2* x,
                                      uint32_t tag_x, uint32_t tag_part, uint32_t pos, uint32_t cta, uint32_t nctas) {
    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const HeadWalk w = head_walk(P, cta, nctas);
    const uint32_t units = w.units, tstride = units + 4, hr = P.sm.head_rows;
    tok_prologue(P, smem, red, x, tag_x, P.hidden, P.output_norm);
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
        const unsigned char* slot = smem + P.sm.ring + size_t(warp * 2 + (i & 1)) * P.sm.ring_slot_bytes;
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
            for (uint32_t c = lane; c < nctas; c += 32) {
                const float cv = poll_pair(P.part + 2 * c, tag_part, P.error);
                const int32_t ci = __float_as_int(poll_pair(P.part + 2 * c + 1, tag_part, P.error));
                tok_better(v, idx, cv, ci);
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) tok_better(v, idx, __shfl_xor_sync(0xffffffffu, v, o), __shfl_xor_sync(0xffffffffu, idx, o));
            if (lane == 0) {
                // std::max_element (src/sampler.cpp:11-13): a NaN is never preferred, and a NaN at index 0 is never displaced
                if (first_logit != first_logit || uint32_t(idx) >= P.vocab) idx = 0;
                *P.chosen = idx;
                if (P.advance) {
                    *P.token_slot = idx;
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
    extern __shared__ __align__(128) unsigned char smem[];
    __shared__ double red[kTokWarps];
    __shared__ float redf[kTokWarps];
    __shared__ float sv[kTokWarps];
    __shared__ int si[kTokWarps];
    __shared__ __align__(8) uint64_t bars[4];
    __shared__ __align__(8) uint64_t hbar[kTokWarps][2];
    __shared__ Shape shapes[4];
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
        // this CTA's rows of the four multiplies: q|k|v as one row space, o, gate/up pairs, down
        const uint32_t bounds[4] = {0, P.q_rows, P.q_rows + P.kv_rows, P.q_rows + 2 * P.kv_rows};
        Shape s{};
        {
            const uint32_t lo = part_lo(bounds[3], cta, nctas), hi = part_lo(bounds[3], cta + 1, nctas);
            for (uint32_t m = 0; m < 3; ++m) {
                const uint32_t a = max(lo, bounds[m]), e = min(hi, bounds[m + 1]);
                if (a < e) {
                    s.seg_rows[s.nseg] = e - a;
                    s.seg_first[s.nseg] = a - bounds[m];
                    s.seg_mat[s.nseg] = m;
                    ++s.nseg;
                    s.rows += e - a;
                }
            }
            shapes[0] = s;
        }
        {
            const uint32_t lo = part_lo(P.hidden, cta, nctas), hi = part_lo(P.hidden, cta + 1, nctas);
            s = Shape{};
            s.rows = hi - lo;
            s.nseg = s.rows != 0 ? 1 : 0;
            s.seg_rows[0] = hi - lo;
            s.seg_first[0] = lo;
            s.seg_mat[0] = 3;
            shapes[1] = s;
            s.seg_mat[0] = 6;
            shapes[3] = s;
        }
        {
            const uint32_t lo = part_lo(P.ffn, cta, nctas), hi = part_lo(P.ffn, cta + 1, nctas);
            s = Shape{};
            s.rows = 2 * (hi - lo);
            s.nseg = s.rows != 0 ? 2 : 0;
            s.seg_rows[0] = s.seg_rows[1] = hi - lo;
            s.seg_first[0] = s.seg_first[1] = lo;
            s.seg_mat[0] = 4;
            s.seg_mat[1] = 5;
            shapes[2] = s;
        }
    }
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
    unsigned char* wbuf[4] = {smem + P.sm.w_qkv, smem + P.sm.w_o, smem + P.sm.w_gu, smem + P.sm.w_down};
    const uint32_t wcols[4] = {P.hidden, P.q_rows, P.hidden, P.ffn};
    if (tid == kIssuer) {
        for (int k = 0; k < 4; ++k) tok_request(shapes[k], tabs[0], wbuf[k], wcols[k], &bars[k]);
    }
    unsigned long long* trace = (P.trace != nullptr && cta == 0 && tid == 0) ? P.trace : nullptr;
    if (trace) trace[0] = tok_now();

    // the token's embedding row: each owner of hidden rows dequantises its own values (embedding_row, src/model.cpp:27-70)
    float hres = 0.0f;
    if (tid < shapes[1].rows) {
        const uint32_t r = shapes[1].seg_first[0] + tid;
        if (P.hidden_in != nullptr) {
            hres = P.hidden_in[r];
        } else {
            const uint32_t units = P.hidden / 32, u = r >> 5, wi = r & 31;
            const size_t unit = size_t(token) * units + u;
            const uint32_t byte = P.embd_nib[unit * 16 + (wi & 15)];
            const int q = int(wi < 16 ? (byte & 0xFu) : (byte >> 4));
            hres = __fmul_rn(float(q - 8), __half2float(P.embd_scl[unit]));
        }
        st_pair(P.hid_a[1] + r, hres, base + 1);
    }

    const uint32_t slices = dim / P.slice_w, wtasks = P.heads * slices, stasks = score_tasks(P, pos);
    constexpr uint32_t kRingPos = kVChunkPos * kVRingChunks;
    for (uint32_t l = 0; l < L; ++l) {
        const TokLayer& Ly = tabs[l];
        const uint32_t par = l & 1, T = base + 2 + l * kTagsPerLayer;
        const bool more = l + 1 < L;
        // what does not depend on this token: the cached K rows of this CTA's score tasks, the V slice of its weighted sum
        if (warp < P.sm.n_sslots && cta + warp * nctas < stasks) {
            scores_request<VPL>(P, smem + P.sm.sslot + size_t(warp) * P.sm.sslot_bytes, Ly, cta + warp * nctas, pos);
        }
        cp_async_commit();
        if (cta < wtasks) values_request(P, smem, Ly, cta, 0, min(pos, kRingPos), tid, kTokThreads);
        cp_async_commit();

        MulArgs a{};
        a.act = P.act;
        unsigned long long* btr = (trace != nullptr && l == 5) ? trace + 2 + L * 6 : nullptr;  // 4 x 10 stamps inside layer 5's multiplies
        a.tr = btr;
        // q/k/v
        a.x = P.hid_a[(l + 1) & 1]; a.tag_x = l == 0 ? base + 1 : T - kTagsPerLayer + 5; a.tag_out = T; a.cols = P.hidden; a.norm = Ly.attn_norm;
        a.w = wbuf[0]; a.bar = &bars[0]; a.parity = par; a.kind = 0; a.plain = nullptr;
        for (uint32_t s = 0; s < shapes[0].nseg; ++s) a.out[s] = shapes[0].seg_mat[s] == 0 ? P.xq[par] : shapes[0].seg_mat[s] == 1 ? P.xk[par] : P.xv[par];
        hres = tok_multiply(P, smem, red, shapes[0], a, hres);
        if (tid == kIssuer && more) {
            fence_async_proxy();
            tok_request(shapes[0], tabs[l + 1], wbuf[0], wcols[0], &bars[0]);
        }
        if (trace) trace[1 + l * 6 + 0] = tok_now();

        tok_scores<VPL, NEOX>(P, smem, Ly, par, T, T + 1, pos, cta, nctas);
        if (trace) trace[1 + l * 6 + 1] = tok_now();
        tok_attend(P, smem, red, redf, Ly, par, T, T + 1, T + 2, pos, cta, btr ? btr + 40 : nullptr);
        if (trace) trace[1 + l * 6 + 2] = tok_now();

        // output projection + residual
        a.x = P.att[par]; a.tag_x = T + 2; a.tag_out = T + 3; a.cols = P.q_rows; a.norm = Ly.attn_sub_norm;
        a.w = wbuf[1]; a.bar = &bars[1]; a.kind = 1; a.out[0] = P.hid_b[par]; a.tr = btr ? btr + 10 : nullptr;
        hres = tok_multiply(P, smem, red, shapes[1], a, hres);
        if (tid == kIssuer && more) {
            fence_async_proxy();
            tok_request(shapes[1], tabs[l + 1], wbuf[1], wcols[1], &bars[1]);
        }
        if (trace) trace[1 + l * 6 + 3] = tok_now();

        // gate/up + activation
        a.x = P.hid_b[par]; a.tag_x = T + 3; a.tag_out = T + 4; a.cols = P.hidden; a.norm = Ly.ffn_norm;
        a.w = wbuf[2]; a.bar = &bars[2]; a.kind = 2; a.out[0] = P.gated[par]; a.tr = btr ? btr + 20 : nullptr;
        hres = tok_multiply(P, smem, red, shapes[2], a, hres);
        if (more) {
            if (tid == kIssuer) {
                fence_async_proxy();
                tok_request(shapes[2], tabs[l + 1], wbuf[2], wcols[2], &bars[2]);
            }
        } else {
            // last layer: everything but the down projection's buffer is free - the head's first chunks start streaming
            // (the barrier: a CTA without gate/up rows came here without one, and its chain warp may still be in the weighted sum)
            cta_sync();
            if (lane == 0) {
                const HeadWalk w = head_walk(P, cta, nctas);
                fence_async_proxy();
                head_request(P, smem, w, warp, 0, &hbar[warp][0]);
                head_request(P, smem, w, warp, 1, &hbar[warp][1]);
            }
        }
        if (trace) trace[1 + l * 6 + 4] = tok_now();

        // down projection + residual
        a.x = P.gated[par]; a.tag_x = T + 4; a.tag_out = T + 5; a.cols = P.ffn; a.norm = Ly.ffn_sub_norm;
        a.w = wbuf[3]; a.bar = &bars[3]; a.kind = 1; a.out[0] = P.hid_a[par]; a.plain = more ? nullptr : P.hidden_out; a.tr = btr ? btr + 30 : nullptr;
        hres = tok_multiply(P, smem, red, shapes[3], a, hres);
        if (tid == kIssuer && more) {
            fence_async_proxy();
            tok_request(shapes[3], tabs[l + 1], wbuf[3], wcols[3], &bars[3]);
        }
        if (trace) trace[1 + l * 6 + 5] = tok_now();
    }
    tok_head(P, smem, red, hbar, sv, si, P.hid_a[(L - 1) & 1], base + 2 + (L - 1) * kTagsPerLayer + 5, base + 2 + L * kTagsPerLayer, pos, cta, nctas);
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
    }
    if (ends.head.type != T_Q4_0) {
        why_not = "the output head is not Q4_0";
        return false;
    }
    const uint32_t q_dim = sh.heads * sh.dim, kv_dim = sh.kv_heads * sh.dim, group = sh.heads / sh.kv_heads;
    for (uint32_t n : {sh.hidden_size, q_dim, sh.ffn_size}) {
        if (n % 256 != 0 || n > 4096) {
            why_not = "a row length is not a multiple of 256 up to 4096";
            return false;
        }
    }
    if ((sh.dim != 64 && sh.dim != 128) || group > 8) {
        why_not = "head size is not 64 or 128, or more than 8 query heads per K/V head";
        return false;
    }
    uint32_t slice_w = 16;
    if (sh.heads * (sh.dim / slice_w) > sms) slice_w = 32;
    if (sh.heads * (sh.dim / slice_w) > sms) {
        why_not = "more (head, 32-column slice) tasks than SMs";
        return false;
    }
    if (ends.vocab < sms || sh.hidden_size < 32) {
        why_not = "fewer vocabulary rows than SMs";
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

    // shared-memory layout: what the head's ring may overwrite comes last
    const uint32_t L = uint32_t(layers.size());
    const uint32_t widest = std::max(std::max(sh.hidden_size, q_dim), sh.ffn_size);
    const uint32_t r_qkv = ceil_div(q_dim + 2 * kv_dim, sms), r_h = ceil_div(sh.hidden_size, sms), r_gu = 2 * ceil_div(sh.ffn_size, sms);
    const uint32_t hu = sh.hidden_size / 32, qu = q_dim / 32, fu = sh.ffn_size / 32;
    TokSmem best{};
    bool fits = false;
    for (uint32_t hr : {8u, 4u, 2u, 1u}) {
        for (uint32_t nss : {4u, 2u, 1u}) {
            if (fits) break;
            TokSmem m{};
            uint32_t off = 0;
            m.tabs = off; off = align_up(off + L * uint32_t(sizeof(TokLayer)), 128);
            m.xlo = off; off += widest / 32 * 16;
            m.xhi = off; off += widest / 32 * 16;
            m.xd = off; off += widest / 32 * 4;
            m.xs = off; off = align_up(off + widest / 32 * 4, 128);
            const uint32_t op_tile = std::max(std::max(r_qkv * (hu + 4), r_h * (qu + 4)), std::max(r_gu * (hu + 4), r_h * (fu + 4)));
            m.tile = off; off = align_up(off + std::max(op_tile, kTokWarps * hr * (hu + 4)) * 4, 128);
            m.w_down = off; off = align_up(off + r_h * fu * 18, 128);
            const uint32_t alias = off;
            m.w_qkv = off; off = align_up(off + r_qkv * hu * 18, 128);
            m.w_o = off; off = align_up(off + r_h * qu * 18, 128);
            m.w_gu = off; off = align_up(off + r_gu * hu * 18, 128);
            m.n_sslots = nss;
            m.sslot_bytes = align_up((group + 1) * sh.dim * 4 + 32 * (sh.dim * 2 + 16), 128);
            m.sslot = off; off += nss * m.sslot_bytes;
            m.ps = off; off = align_up(off + sh.max_context * 4, 128);
            m.vring = off; off = align_up(off + kVChunkPos * kVRingChunks * slice_w * 2, 128);
            m.vown = off; off += 128;
            m.prod = off; off = align_up(off + 2 * slice_w * kSubStride * 4, 128);
            m.head_rows = hr;
            m.ring_slot_bytes = hr * hu * 18;
            m.ring = alias;
            m.total = std::max(off, alias + 2 * kTokWarps * m.ring_slot_bytes);
            if (m.total + 2048 <= uint32_t(limit)) {
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

    void (*kernel)(TokParams) = sh.dim == 128 ? (sh.neox ? token_kernel<4, true> : token_kernel<4, false>) : (sh.neox ? token_kernel<2, true> : token_kernel<2, false>);
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
    // tagged vectors, two copies each: hid_a hid_b q k v scores attended gated, then the per-CTA arg-max candidates
    const size_t per_copy = 2 * size_t(sh.hidden_size) + 2 * q_dim + 2 * kv_dim + size_t(sh.heads) * sh.max_context + sh.ffn_size;
    impl->pairs = 2 * per_copy + 2 * size_t(sms);
    BK_CUDA(cudaMalloc(&impl->pairs_dev, impl->pairs * sizeof(uint2)));
    BK_CUDA(cudaMemsetAsync(impl->pairs_dev, 0, impl->pairs * sizeof(uint2), s));  // tag 0 is never expected
    BK_CUDA(cudaMalloc(&impl->words_dev, 64));
    BK_CUDA(cudaMemsetAsync(impl->words_dev, 0, 64, s));
    const uint32_t one = 1;
    BK_CUDA(cudaMemcpyAsync(impl->words_dev, &one, sizeof(one), cudaMemcpyHostToDevice, s));  // epoch starts at 1

    TokParams& P = impl->params;
    uint2* at = impl->pairs_dev;
    auto take = [&](size_t n) {
        uint2* p = at;
        at += n;
        return p;
    };
    for (int c = 0; c < 2; ++c) {
        P.hid_a[c] = take(sh.hidden_size);
        P.hid_b[c] = take(sh.hidden_size);
        P.xq[c] = take(q_dim);
        P.xk[c] = take(kv_dim);
        P.xv[c] = take(kv_dim);
        P.sc[c] = take(size_t(sh.heads) * sh.max_context);
        P.att[c] = take(q_dim);
        P.gated[c] = take(sh.ffn_size);
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
        t.attn_sub_norm = A.attn_sub_norm; t.ffn_sub_norm = A.ffn_sub_norm;
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
    P.token = ends.token; P.position = const_cast<uint32_t*>(sh.position); P.chosen = ends.chosen; P.token_slot = ends.token;
    P.history = ends.history; P.history_len = ends.history_len;
    P.epoch = impl->words_dev; P.error = impl->words_dev + 1;
    P.tags_per_launch = L * kTagsPerLayer + 8;
    P.slice_w = slice_w;
    P.sm = best;
    impl_ = impl.release();
    char text[160];
    std::snprintf(text, sizeof text, "one launch per token: %u CTAs, %u KB shared, %u score slots, head chunks of %u rows, %u-column value slices", sms,
                  best.total / 1024, best.n_sslots, best.head_rows, slice_w);
    description_ = text;
    return true;
}

void TokenPlan::launch(cudaStream_t s, bool advance) {
    // Tags must never repeat while old pairs are still in the buffers: long before the 32-bit range runs out, wipe them.
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
