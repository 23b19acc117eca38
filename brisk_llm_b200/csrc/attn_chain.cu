// Softmax + weighted sum of attention for 1..24 tokens at once, arranged around the one thing the reference's order of
// operations does not let anybody parallelise: out[i] = ((p[0]*v_0[i] + p[1]*v_1[i]) + p[2]*v_2[i]) + ... is a chain of
// dependent f32 additions per (token, head, i), one per visible position (src/kernels_f32.cpp:265-273), and the result
// has to be that chain's, bit for bit, because the 8-bit re-quantisation that follows turns a 1-ulp difference into a
// different integer every so often.
//
// A chain cannot go faster than one addition per ~4.9 cycles. What can be chosen is how many chains a lane runs at once
// and how many warps share a scheduler:
//
//   CTA    one token, HQ (1 or 2) query heads of one K/V head; each head's `dim` values are split over WPH warps, lane l of a
//          warp owning C = dim / (32 WPH) adjacent values (C = 1, 2 or 4)
//   V      the K/V head's rows come through a ring of 4 stages x 32 KB in shared memory; a stage is one run of bytes of the
//          cache and ONE bulk copy (cp.async.bulk, mbarrier completion) issued three stages ahead by one thread, and it
//          is read by every warp of the CTA: once per CTA, whatever HQ is
//   chain  per position a lane loads its C values (one shared load), widens them, multiplies by the position's probability
//          (read four positions at a time) and adds to its C running sums. Issue slots per position and warp: 4.25 / 6.25 /
//          11.25 for C = 1 / 2 / 4 - so with C = 1 a warp alone on its scheduler runs at the latency of the additions, and
//          with C = 4 a head costs the fewest slots. The launcher picks C so that an SM ends up with about four warps.
//
// Products that go through shared memory (an earlier form of this kernel: product warps and chain warps) cost 8 bytes of
// shared-memory traffic per product, 16 cycles per position with two heads on an SM; this form costs 2 bytes per value.
//
// Before the chains all threads compute the softmax of the CTA's HQ score rows into shared memory exactly as the other
// attention kernels do (max, e = expf(s - max) with glibc's expf, f64 sum, p = e * float(1 / sum); src/kernels_f32.cpp:
// 275-284) - with the same split of the f64 sum over 256 (virtual) threads, so the totals are the same doubles. The exps
// take their 2^(i/32) table from shared memory and run four at a time: with the table in global memory and one exp after
// the other they cost 850 cycles each and, at 8192 positions, as much as the chains.
#include "exact_math.h"
#include "kernels.h"

namespace bk {
namespace {

constexpr uint32_t kStages = 4;
constexpr uint32_t kStageBytes = 32 * 1024;
constexpr uint32_t kSumThreads = 256;  // the f64 sum is split the way a 256-thread CTA splits it
constexpr uint32_t kWaitLimit = 1u << 22;
__device__ unsigned int g_chain_error;  // set when a wait for a bulk copy ran out (never seen; every wait is bounded all the same)

#ifdef BK_CHAIN_TRACE  // development aid: cycle counts of CTA (0, 0) - never compiled into the library
__device__ unsigned long long g_chain_trace[32];
#define CHAIN_CLOCK() clock64()
#define CHAIN_ADD(slot, since) do { if (blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 0) g_chain_trace[slot] += clock64() - (since); } while (0)
#else
#define CHAIN_CLOCK() 0ll
#define CHAIN_ADD(slot, since) do { } while (0)
#endif

struct ChainParams {
    const float* scores;   // [n][heads][max_context] scaled scores
    const __half* v_cache; // [kv][max_context][dim]
    float* out;            // [n][heads * dim]
    const uint32_t* position;
    uint32_t n, heads, kv_heads, dim, max_context, window;
    uint32_t ps_stride;    // floats per probability row in shared memory
    uint32_t stage_rows;   // positions per stage of the V ring: kStageBytes / (dim * 2)
};

// The C values of one position a lane owns, as loaded from the ring.
template <int C>
struct Raw;
template <>
struct Raw<4> { using T = uint2; };
template <>
struct Raw<2> { using T = uint32_t; };
template <>
struct Raw<1> { using T = unsigned short; };

template <int C>
__device__ __forceinline__ void mul_add(float (&acc)[C], const typename Raw<C>::T& raw, float p) {
    if constexpr (C == 4) {
        const __half2* h = reinterpret_cast<const __half2*>(&raw);
        const float2 a = __half22float2(h[0]), b = __half22float2(h[1]);
        acc[0] = __fadd_rn(acc[0], __fmul_rn(p, a.x)); acc[1] = __fadd_rn(acc[1], __fmul_rn(p, a.y));
        acc[2] = __fadd_rn(acc[2], __fmul_rn(p, b.x)); acc[3] = __fadd_rn(acc[3], __fmul_rn(p, b.y));
    } else if constexpr (C == 2) {
        const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&raw));
        acc[0] = __fadd_rn(acc[0], __fmul_rn(p, a.x)); acc[1] = __fadd_rn(acc[1], __fmul_rn(p, a.y));
    } else {
        acc[0] = __fadd_rn(acc[0], __fmul_rn(p, __half2float(__ushort_as_half(raw))));
    }
}

template <int C, int HQ>
__global__ void __launch_bounds__(256) attn_chain_kernel(const ChainParams a) {
    using R = typename Raw<C>::T;
    extern __shared__ __align__(16) unsigned char smem[];
    __shared__ float redf[HQ][8];
    __shared__ double redd[HQ][8];
    __shared__ uint64_t tab[32];
    __shared__ __align__(8) uint64_t full[kStages];
    float* ps = reinterpret_cast<float*>(smem);                                             // [HQ][ps_stride]
    unsigned char* ring = smem + size_t(HQ) * a.ps_stride * sizeof(float);                  // [kStages][stage_rows][dim] f16
    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nt = blockDim.x;
    const uint32_t wph = nt / 32 / HQ;  // warps per head
    const uint32_t tok = blockIdx.y, h0 = blockIdx.x * HQ;
    const uint32_t kvh = h0 / (a.heads / a.kv_heads);
    const uint32_t visible = *a.position + tok + 1;
    // a sliding-window layer attends to the last `window` positions only (src/model.cpp:1084-1091)
    const uint32_t start = a.window != 0 && visible > a.window ? visible - a.window : 0;
    const uint32_t cnt = visible - start;
    const uint32_t row_bytes = a.dim * 2, rows = a.stage_rows;
    const unsigned char* vbase = reinterpret_cast<const unsigned char*>(a.v_cache + (size_t(kvh) * a.max_context + start) * a.dim);
    const uint32_t stages = (cnt + rows - 1) / rows;

    // Stage `st` of V into the ring: rows are contiguous in the cache, so a stage is one run of bytes and ONE bulk copy
    // (cp.async.bulk, completion counted on the stage's mbarrier) issued by one thread. Filled 16 bytes at a time with
    // cp.async the same stage took every thread 16 instructions and ~700 cycles of issue at three stages in flight.
    if (tid == 0) {
        for (uint32_t i = 0; i < kStages; ++i) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(uint32_t(__cvta_generic_to_shared(&full[i]))) : "memory");
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    auto request = [&](uint32_t st) {  // thread 0 only
        if (st < stages) {
            const uint32_t bytes = min(rows, cnt - st * rows) * row_bytes;
            const unsigned char* src = vbase + size_t(st) * rows * row_bytes;
            const uint32_t dst = uint32_t(__cvta_generic_to_shared(ring + size_t(st % kStages) * kStageBytes));
            const uint32_t bar = uint32_t(__cvta_generic_to_shared(&full[st % kStages]));
            asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
            asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
        }
    };
    if (tid == 0) {
        for (uint32_t st = 0; st + 1 < kStages; ++st) request(st);  // in flight while the softmax runs
    }

    // ---- softmax of the HQ rows ------------------------------------------------------------------------------------
    const long long t_begin = CHAIN_CLOCK();
    if (tid < 32) tab[tid] = exp2_table_device()[tid];
#pragma unroll
    for (int q = 0; q < HQ; ++q) {
        const float* s = a.scores + (size_t(tok) * a.heads + h0 + q) * a.max_context + start;
        float m = -INFINITY;
        uint32_t p = tid;
        for (; p + 7 * nt < cnt; p += 8 * nt) {  // eight loads in flight per thread: one after the other they cost an L2 round trip each
            float v[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) v[u] = __ldcg(s + p + u * nt);
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                ps[q * a.ps_stride + p + u * nt] = v[u];
                m = fmaxf(m, v[u]);
            }
        }
        for (; p < cnt; p += nt) {
            const float v = __ldcg(s + p);
            ps[q * a.ps_stride + p] = v;
            m = fmaxf(m, v);
        }
        m = warp_max(m);
        if (lane == 0) redf[q][warp] = m;
    }
    __syncthreads();
#pragma unroll
    for (int q = 0; q < HQ; ++q) {
        float* row = ps + q * a.ps_stride;
        float m = redf[q][0];
        for (uint32_t w = 1; w < nt / 32; ++w) m = fmaxf(m, redf[q][w]);
        // virtual thread vt of 256 sums positions vt, vt + 256, ... in that order, as a 256-thread CTA does
        for (uint32_t vt = tid; vt < kSumThreads; vt += nt) {
            double part = 0.0;
            uint32_t p = vt;
            for (; p + 3 * kSumThreads < cnt; p += 4 * kSumThreads) {
                const float e0 = exact_expf_flat(__fsub_rn(row[p], m), tab), e1 = exact_expf_flat(__fsub_rn(row[p + kSumThreads], m), tab);
                const float e2 = exact_expf_flat(__fsub_rn(row[p + 2 * kSumThreads], m), tab), e3 = exact_expf_flat(__fsub_rn(row[p + 3 * kSumThreads], m), tab);
                row[p] = e0; row[p + kSumThreads] = e1; row[p + 2 * kSumThreads] = e2; row[p + 3 * kSumThreads] = e3;
                part += double(e0); part += double(e1); part += double(e2); part += double(e3);
            }
            for (; p < cnt; p += kSumThreads) {
                const float e = exact_expf_flat(__fsub_rn(row[p], m), tab);
                row[p] = e;
                part += double(e);
            }
            part = warp_sum(part);
            if (lane == 0) redd[q][vt >> 5] = part;
        }
    }
    __syncthreads();
#pragma unroll
    for (int q = 0; q < HQ; ++q) {
        double total = 0.0;
#pragma unroll
        for (int w = 0; w < 8; ++w) total += redd[q][w];
        const float inv = float(1.0 / total);
        for (uint32_t p = tid; p < cnt; p += nt) ps[q * a.ps_stride + p] = __fmul_rn(ps[q * a.ps_stride + p], inv);
    }
    CHAIN_ADD(0, t_begin);
    const long long t_phase = CHAIN_CLOCK();

    // ---- the chains ------------------------------------------------------------------------------------------------
    const uint32_t hq = warp / wph, col = (warp % wph) * 32 * C + C * lane;
    const float* prow = ps + hq * a.ps_stride;
    float acc[C];
#pragma unroll
    for (int k = 0; k < C; ++k) acc[k] = 0.0f;
    bool dead = false;
    __syncthreads();  // the probabilities are complete (and the mbarriers initialised, long ago)
    for (uint32_t st = 0; st < stages; ++st) {
        const long long t_r = CHAIN_CLOCK();
        if (tid == 0) request(st + kStages - 1);  // into the stage everybody left at the end of the previous iteration
        CHAIN_ADD(4, t_r);
        const long long t_w = CHAIN_CLOCK();
        {   // bounded: a copy from the cache always lands; should the wait run out all the same, the error word says so
            const uint32_t bar = uint32_t(__cvta_generic_to_shared(&full[st % kStages])), parity = (st / kStages) & 1;
            uint32_t ok = 0;
            for (uint32_t spin = 0; ok == 0 && !dead; ++spin) {
                asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}" : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
                if (ok == 0 && spin == kWaitLimit) {
                    atomicOr(&g_chain_error, 1u);
                    dead = true;
                }
            }
        }
        CHAIN_ADD(2, t_w);
        const long long t_c = CHAIN_CLOCK();
        const uint32_t n_rows = min(rows, cnt - st * rows);
        const unsigned char* vs = ring + size_t(st % kStages) * kStageBytes + col * 2;
        const float* pp = prow + st * rows;
        // Batches of 8 positions in two register sets named apart, nothing but loads and arithmetic in the loop: the loads of
        // one batch are in flight while the other batch's additions - the dependent chain - run.
        R v0[8], v1[8];
        float4 p0[2], p1[2];
        auto load = [&](uint32_t r, R (&v)[8], float4 (&p)[2]) {
#pragma unroll
            for (int u = 0; u < 8; ++u) v[u] = *reinterpret_cast<const R*>(vs + (r + u) * row_bytes);
            p[0] = *reinterpret_cast<const float4*>(pp + r);
            p[1] = *reinterpret_cast<const float4*>(pp + r + 4);
        };
        auto run = [&](const R (&v)[8], const float4 (&p)[2]) {
            mul_add<C>(acc, v[0], p[0].x); mul_add<C>(acc, v[1], p[0].y); mul_add<C>(acc, v[2], p[0].z); mul_add<C>(acc, v[3], p[0].w);
            mul_add<C>(acc, v[4], p[1].x); mul_add<C>(acc, v[5], p[1].y); mul_add<C>(acc, v[6], p[1].z); mul_add<C>(acc, v[7], p[1].w);
        };
        const uint32_t pairs = n_rows / 16;
        if (pairs > 0) load(0, v0, p0);
#pragma unroll 1
        for (uint32_t i = 0; i + 1 < pairs; ++i) {
            load(16 * i + 8, v1, p1);
            run(v0, p0);
            load(16 * i + 16, v0, p0);
            run(v1, p1);
        }
        uint32_t r = 0;
        if (pairs > 0) {
            load(16 * pairs - 8, v1, p1);
            run(v0, p0);
            run(v1, p1);
            r = 16 * pairs;
        }
        for (; r < n_rows; ++r) mul_add<C>(acc, *reinterpret_cast<const R*>(vs + r * row_bytes), pp[r]);  // the last stage's last positions
        CHAIN_ADD(3, t_c);
        const long long t_s2 = CHAIN_CLOCK();
        __syncthreads();  // the stage may be overwritten
        CHAIN_ADD(6, t_s2);
    }
    CHAIN_ADD(1, t_phase);
    float* o = a.out + size_t(tok) * a.heads * a.dim + size_t(h0 + hq) * a.dim + col;
#pragma unroll
    for (int k = 0; k < C; ++k) o[k] = acc[k];
}

// ---- one token ------------------------------------------------------------------------------------------------------
// With a single token there are only `heads` chains of work per value and nothing to share V rows with, and the f16 -> f32
// widening that a chain lane does in the kernel above costs it ~3 cycles per position. So the single-token form separates
// the roles: a CTA takes 32 values of one head; warp 0 runs the 32 chains (one per lane: a shared load and a dependent add
// per position, two register sets), warps 1-7 produce the products p[pos] * v[pos][i] into a pair of 32 KB tiles of 256
// positions - each product lane asks for its own 8 bytes of V three tiles ahead with cp.async into a slot only it reads
// (a prefetch queue that costs no registers and no barrier), then loads them back, widens, multiplies and stores four
// products with one 16-byte store. Chain and producers meet at named barriers (bar.sync / bar.arrive: nothing spins).
// Shared-memory traffic is 8 bytes per product, which is why this form is for one token (32 products per position and CTA)
// and the form above for several.
constexpr uint32_t kOneThreads = 256, kOneW = 32, kOnePC = 256, kOneProducers = 7, kOneItems = 10, kOneDepth = 4;
constexpr uint32_t kOneTileFloats = kOnePC * kOneW;                                 // 32 KB
constexpr uint32_t kOneRingBytes = kOneDepth * kOneItems * kOneProducers * 32 * 8;  // 70 KB

__device__ __forceinline__ void bar_sync_one(int id) { asm volatile("bar.sync %0, %1;" ::"r"(id), "n"(kOneThreads) : "memory"); }
__device__ __forceinline__ void bar_arrive_one(int id) { asm volatile("bar.arrive %0, %1;" ::"r"(id), "n"(kOneThreads) : "memory"); }

__global__ void __launch_bounds__(kOneThreads) attn_chain_one_kernel(const ChainParams a) {
    extern __shared__ __align__(16) unsigned char smem[];
    __shared__ float redf[8];
    __shared__ double redd[8];
    __shared__ uint64_t tab[32];
    float* ps = reinterpret_cast<float*>(smem);                    // [ps_stride]
    float* tiles = ps + a.ps_stride;                               // [2][kOnePC][kOneW]
    unsigned char* ring = reinterpret_cast<unsigned char*>(tiles + 2 * kOneTileFloats);
    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t slices = a.dim / kOneW, slice = blockIdx.x % slices, h = blockIdx.x / slices;
    const uint32_t kvh = h / (a.heads / a.kv_heads);
    const uint32_t visible = *a.position + 1;
    const uint32_t start = a.window != 0 && visible > a.window ? visible - a.window : 0;
    const uint32_t cnt = visible - start;
    const __half* vbase = a.v_cache + (size_t(kvh) * a.max_context + start) * a.dim + slice * kOneW;

    // ---- softmax (the same operations and the same split of the f64 sum as everywhere else) ----
    if (tid < 32) tab[tid] = exp2_table_device()[tid];
    const float* s = a.scores + size_t(h) * a.max_context + start;
    float m = -INFINITY;
    {
        uint32_t p = tid;
        for (; p + 7 * kOneThreads < cnt; p += 8 * kOneThreads) {
            float v[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) v[u] = __ldcg(s + p + u * kOneThreads);
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                ps[p + u * kOneThreads] = v[u];
                m = fmaxf(m, v[u]);
            }
        }
        for (; p < cnt; p += kOneThreads) {
            const float v = __ldcg(s + p);
            ps[p] = v;
            m = fmaxf(m, v);
        }
    }
    m = warp_max(m);
    if (lane == 0) redf[warp] = m;
    __syncthreads();
    m = redf[0];
#pragma unroll
    for (int w = 1; w < 8; ++w) m = fmaxf(m, redf[w]);
    double part = 0.0;
    {
        uint32_t p = tid;
        for (; p + 3 * kOneThreads < cnt; p += 4 * kOneThreads) {
            const float e0 = exact_expf_flat(__fsub_rn(ps[p], m), tab), e1 = exact_expf_flat(__fsub_rn(ps[p + kOneThreads], m), tab);
            const float e2 = exact_expf_flat(__fsub_rn(ps[p + 2 * kOneThreads], m), tab), e3 = exact_expf_flat(__fsub_rn(ps[p + 3 * kOneThreads], m), tab);
            ps[p] = e0; ps[p + kOneThreads] = e1; ps[p + 2 * kOneThreads] = e2; ps[p + 3 * kOneThreads] = e3;
            part += double(e0); part += double(e1); part += double(e2); part += double(e3);
        }
        for (; p < cnt; p += kOneThreads) {
            const float e = exact_expf_flat(__fsub_rn(ps[p], m), tab);
            ps[p] = e;
            part += double(e);
        }
    }
    part = warp_sum(part);
    if (lane == 0) redd[warp] = part;
    __syncthreads();
    double total = 0.0;
#pragma unroll
    for (int w = 0; w < 8; ++w) total += redd[w];
    const float inv = float(1.0 / total);
    for (uint32_t p = tid; p < cnt; p += kOneThreads) ps[p] = __fmul_rn(ps[p], inv);
    __syncthreads();

    // ---- products and chains ----
    const uint32_t chunks = (cnt + kOnePC - 1) / kOnePC;
    if (warp >= 1) {
        const uint32_t pw = warp - 1, sub = lane >> 3, lg = lane & 7;  // 8 lanes per position (4 values each), 4 positions per item
        const uint32_t my_slot = (pw * 32 + lane) * 8;
        constexpr uint32_t kItemStride = kOneProducers * 32 * 8;
        auto request = [&](uint32_t chunk) {
            if (chunk < chunks) {
                const uint32_t rows = min(kOnePC, cnt - chunk * kOnePC);
                unsigned char* base = ring + size_t(chunk % kOneDepth) * kOneItems * kItemStride + my_slot;
#pragma unroll
                for (uint32_t i = 0; i < kOneItems; ++i) {
                    const uint32_t r = (i * kOneProducers + pw) * 4 + sub;
                    if (r < rows) {
                        const uint32_t dst = uint32_t(__cvta_generic_to_shared(base + i * kItemStride));
                        asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(dst), "l"(vbase + size_t(chunk * kOnePC + r) * a.dim + 4 * lg) : "memory");
                    }
                }
            }
            asm volatile("cp.async.commit_group;" ::: "memory");  // one group per chunk, empty or not
        };
#pragma unroll 1
        for (uint32_t d = 0; d + 1 < kOneDepth; ++d) request(d);
#pragma unroll 1
        for (uint32_t c = 0; c < chunks; ++c) {
            const uint32_t b = c & 1, rows = min(kOnePC, cnt - c * kOnePC);
            request(c + kOneDepth - 1);
            asm volatile("cp.async.wait_group %0;" ::"n"(kOneDepth - 1) : "memory");  // chunk c's values are in this lane's slots
            if (c >= 2) bar_sync_one(3 + b);  // the chain warp is done with this buffer's previous tile
            float* tile = tiles + size_t(b) * kOneTileFloats;
            const unsigned char* base = ring + size_t(c % kOneDepth) * kOneItems * kItemStride + my_slot;
            // all of the chunk's loads first, then the arithmetic
            uint2 raw[kOneItems];
            float pr[kOneItems];
#pragma unroll
            for (uint32_t i = 0; i < kOneItems; ++i) {
                const uint32_t r = min((i * kOneProducers + pw) * 4 + sub, rows - 1);
                raw[i] = *reinterpret_cast<const uint2*>(base + i * kItemStride);
                pr[i] = ps[c * kOnePC + r];
            }
#pragma unroll
            for (uint32_t i = 0; i < kOneItems; ++i) {
                const uint32_t r = (i * kOneProducers + pw) * 4 + sub;
                if (r < rows) {
                    const __half2* hv = reinterpret_cast<const __half2*>(&raw[i]);
                    const float2 v01 = __half22float2(hv[0]), v23 = __half22float2(hv[1]);
                    float4 prod;
                    prod.x = __fmul_rn(pr[i], v01.x); prod.y = __fmul_rn(pr[i], v01.y); prod.z = __fmul_rn(pr[i], v23.x); prod.w = __fmul_rn(pr[i], v23.y);
                    *reinterpret_cast<float4*>(tile + r * kOneW + 4 * lg) = prod;
                }
            }
            bar_arrive_one(1 + b);
        }
        asm volatile("cp.async.wait_group 0;" ::: "memory");
    } else {
        float acc = 0.0f;
        const float* tile0 = tiles + lane;
        auto load_batch = [&](const float* src, float (&dst)[8]) {
#pragma unroll
            for (int u = 0; u < 8; ++u) dst[u] = src[u * kOneW];
        };
        auto add_batch = [&](const float (&src)[8]) {
#pragma unroll
            for (int u = 0; u < 8; ++u) acc = __fadd_rn(acc, src[u]);
        };
        float s0[8], s1[8];
        uint32_t waited = 0;  // tiles 0 .. waited - 1 have been waited for
        if (cnt >= 16) {
            bar_sync_one(1);
            waited = 1;
            load_batch(tile0, s0);
        }
        uint32_t pos = 0;
#pragma unroll 1
        for (uint32_t c = 0; c < chunks; ++c) {
            const uint32_t rows = min(kOnePC, cnt - c * kOnePC), pairs = rows / 16;
            if (pairs == 0) break;  // a last tile of fewer than 16 positions: below
            const float* mine = tile0 + (c & 1) * kOneTileFloats;  // s0 holds its first 8 positions
#pragma unroll 1
            for (uint32_t i = 0; i + 1 < pairs; ++i) {
                load_batch(mine + (16 * i + 8) * kOneW, s1);
                add_batch(s0);
                load_batch(mine + (16 * i + 16) * kOneW, s0);
                add_batch(s1);
            }
            load_batch(mine + (16 * pairs - 8) * kOneW, s1);
            add_batch(s0);
            if (c + 1 < chunks && min(kOnePC, cnt - (c + 1) * kOnePC) >= 16) {  // the next tile's first batch, before this tile's last additions
                bar_sync_one(1 + ((c + 1) & 1));
                waited = c + 2;
                load_batch(tile0 + ((c + 1) & 1) * kOneTileFloats, s0);
            }
            add_batch(s1);
            pos = c * kOnePC + 16 * pairs;
            if (rows == kOnePC && c + 2 < chunks) bar_arrive_one(3 + (c & 1));  // a product warp waits for exactly these
        }
        if (pos < cnt) {  // what is left of the last tile: fewer than 16 positions
            const uint32_t c = pos / kOnePC;
            if (waited <= c) bar_sync_one(1 + (c & 1));
            const float* mine = tile0 + (c & 1) * kOneTileFloats;
            for (; pos < cnt; ++pos) acc = __fadd_rn(acc, mine[(pos % kOnePC) * kOneW]);
        }
        a.out[size_t(h) * a.dim + slice * kOneW + lane] = acc;
    }
}

size_t one_smem(uint32_t max_visible) { return size_t((max_visible + 3) & ~3u) * sizeof(float) + 2 * size_t(kOneTileFloats) * sizeof(float) + kOneRingBytes; }

struct Choice {
    int c = 0, hq = 0;
};

size_t smem_for(int hq, uint32_t max_visible) { return size_t(hq) * ((max_visible + 3) & ~3u) * sizeof(float) + size_t(kStages) * kStageBytes; }

// Warps per SM when every CTA gets an SM of its own: about four (one per scheduler) is the aim. Few (token, head) pairs:
// narrow lanes (C = 1), a head spread over dim/32 warps, each chain at the latency of its additions. Many: wide lanes, two
// heads per CTA sharing the V stream.
Choice choose(uint32_t n, uint32_t heads, uint32_t kv_heads, uint32_t dim, uint32_t max_visible, uint32_t sms) {
    const uint32_t group = heads / kv_heads;
    const uint64_t pairs = uint64_t(n) * heads;
    const int options[4][2] = {{1, 1}, {2, 2}, {2, 1}, {4, 2}};  // (C, HQ): rising work per warp; two heads per CTA (one V stream) before one
    Choice pick;
    for (const auto& o : options) {
        const uint32_t warps = o[1] * (dim / (32u * o[0]));
        if (dim % (32u * o[0]) != 0 || warps > 8 || (o[1] == 2 && group % 2 != 0)) continue;
        if (smem_for(o[1], max_visible) > 200 * 1024) continue;
        pick = Choice{o[0], o[1]};
        const uint64_t ctas = pairs / o[1];
        if (ctas * warps <= uint64_t(sms) * 4 + sms / 2) break;  // about four warps per SM or fewer: wide enough
    }
    return pick;
}

template <int C, int HQ>
void launch_variant(const ChainParams& p, cudaStream_t s) {
    const size_t smem = size_t(HQ) * p.ps_stride * sizeof(float) + size_t(kStages) * kStageBytes;
    static DeviceOnce once;
    if (once.first()) BK_CUDA(cudaFuncSetAttribute(attn_chain_kernel<C, HQ>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    const uint32_t threads = HQ * (p.dim / (32 * C)) * 32;
    attn_chain_kernel<C, HQ><<<dim3(p.heads / HQ, p.n), threads, smem, s>>>(p);
    BK_CUDA(cudaGetLastError());
}

}  // namespace

unsigned int* attn_chain_error_word() {
    unsigned int* p = nullptr;
    BK_CUDA(cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_chain_error));
    return p;
}

bool attn_chain_one_fits(uint32_t dim, uint32_t max_visible) { return dim % kOneW == 0 && one_smem(max_visible) <= 200 * 1024; }

// One token: a.scores holds its scaled scores [heads][max_context]; a.out receives the attended row.
void launch_attn_chain_one(const AttnArgs& a, cudaStream_t s) {
    ChainParams p{};
    p.scores = a.scores; p.v_cache = a.v_cache; p.out = a.out; p.position = a.position;
    p.n = 1; p.heads = a.heads; p.kv_heads = a.kv_heads; p.dim = a.dim; p.max_context = a.max_context; p.window = a.window;
    p.ps_stride = (a.max_visible + 3) & ~3u;
    static DeviceOnce once;
    if (once.first()) BK_CUDA(cudaFuncSetAttribute(attn_chain_one_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    attn_chain_one_kernel<<<a.heads * (a.dim / kOneW), kOneThreads, one_smem(a.max_visible), s>>>(p);
    BK_CUDA(cudaGetLastError());
}

bool attn_chain_fits(uint32_t n, uint32_t heads, uint32_t kv_heads, uint32_t dim, uint32_t max_visible, uint32_t sms) {
    return dim % 32 == 0 && dim <= 256 && heads % kv_heads == 0 && choose(n, heads, kv_heads, dim, max_visible, sms).c != 0;
}

// a.scores holds the scaled scores of the n tokens (rows of max_context floats); a.out receives the attended rows.
void launch_attn_chain(const AttnArgs& a, uint32_t sms, cudaStream_t s) {
    const Choice ch = choose(a.n, a.heads, a.kv_heads, a.dim, a.max_visible, sms);
    if (ch.c == 0) throw CudaError("cuda: context too long for the chained attention kernel");
    ChainParams p{};
    p.scores = a.scores; p.v_cache = a.v_cache; p.out = a.out; p.position = a.position;
    p.n = a.n; p.heads = a.heads; p.kv_heads = a.kv_heads; p.dim = a.dim; p.max_context = a.max_context; p.window = a.window;
    p.ps_stride = (a.max_visible + 3) & ~3u;
    p.stage_rows = kStageBytes / (a.dim * 2);
    if (ch.c == 1) launch_variant<1, 1>(p, s);
    else if (ch.c == 2 && ch.hq == 1) launch_variant<2, 1>(p, s);
    else if (ch.c == 2) launch_variant<2, 2>(p, s);
    else launch_variant<4, 2>(p, s);
}

}  // namespace bk
