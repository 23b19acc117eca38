// Device-side bodies of the single-token step, shared by the one-kernel-per-operation path (decode.cu) and the
// persistent whole-step kernel (step.cu). A body is handed a "gate": gate.wait() returns once the results of the
// previous operation are visible (griddepcontrol.wait in the first path, a grid-wide barrier in the second); loads
// that do not depend on the previous operation - the first weight units, cached K rows, V tiles - are issued before
// it. Values produced by an earlier operation of the same step are read with L2 loads (__ldcg), never through L1:
// inside the persistent kernel another SM wrote them during the same launch.
//
// All arithmetic is the reference's, in the reference's order (see formats.cuh, rowops.cuh, exact_math.h), so either
// path stays bit-identical to the CPU engine.
#pragma once

#include <type_traits>

#include "formats.cuh"
#include "kernels.h"
#include "rowops.cuh"

namespace bk {

constexpr int kDecWarps = 16;  // warps per CTA of every single-token kernel; the per-CTA prologue (norm + quantise) is shared by all of them

// ---- multiply ---------------------------------------------------------------------------------------------------
struct DecMatParams {
    DevMatrix m[3];
    float* out[3];
    uint32_t first_group[4];
    int count;
    int epi;
    const float* x;       // [cols] f32 input of the step (residual stream, attended row, gated activation)
    const float* weight;  // RMS-norm weight or nullptr (no norm)
    float eps;
    uint32_t cols;
    unsigned long long* trace;  // optional: 8 time stamps (ns) written by thread 0 of CTA 0, for BRISK_CUDA_TRACE
    int pdl;
};

// Row groups of `rw` rows: fills first_group for the targets (one entry for a gate/up pair) and returns the total.
inline uint32_t dec_assign_groups(DecMatParams& p, int rw, bool pair) {
    uint32_t groups = 0;
    const int targets = pair ? 1 : p.count;
    for (int i = 0; i < targets; ++i) {
        p.first_group[i] = groups;
        groups += (p.m[i].rows + rw - 1) / rw;
    }
    p.first_group[targets] = groups;
    return groups;
}

// Bytes of shared memory the multiply body takes for the activation row: f32 values, then the quantised planes.
inline size_t dec_act_smem(uint32_t cols) { return size_t(cols) * 4 + cols + (cols / 32) * 8 + 64; }
// Floats of the per-warp transpose tile for CHAINS row chains.
constexpr size_t dec_tile_floats(int chains) { return size_t(kDecWarps) * chains * 36; }

#ifdef __CUDACC__

__device__ __forceinline__ void dec_stamp(unsigned long long* trace, uint32_t cta, int slot) {
    if (trace != nullptr && cta == 0 && threadIdx.x == 0) {
        unsigned long long t;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
        trace[slot] = t;
    }
}

// ---- how a body exchanges vectors with the operations before and after it --------------------------------------
// PlainIo: ordinary f32 vectors; the caller's gate (a kernel boundary, a grid barrier) orders producer and consumer.
// TaggedIo: every element is an 8-byte pair {value bits, tag} written with ONE 8-byte store and read with 8- or
// 16-byte loads that bypass L1. A consumer knows the tag its producer writes (unique per token, layer and operation)
// and simply re-reads until every pair it needs carries that tag - value and tag arrive together, so no fence, no
// counter and no barrier is needed between operations: a CTA starts an operation the moment ITS inputs are complete.
// Safety of reuse: a buffer is overwritten only by an operation that has validated results which (transitively) could
// only be produced after every reader of the buffer's previous contents had finished reading; CTAs with no rows in
// an operation therefore must not read its input (they skip the prologue). Every poll loop is bounded: when it runs
// out the CTA sets *error and goes on with whatever it has read, so the kernel always ends.
struct PlainIo {
    static constexpr bool kTagged = false;
};
struct TaggedIo {
    static constexpr bool kTagged = true;
    uint32_t tag_x;     // tag of the input vector
    uint32_t tag_old;   // EPI_ADD: tag of the residual values being added to
    uint32_t tag_out;   // tag this operation writes
    unsigned int* error;
    float* plain_out;   // optional: also store the results as ordinary floats (the step's final residual stream)
};
constexpr uint32_t kPollLimitDefault = 1u << 20;  // re-reads of one batch before giving up (a fraction of a second)
#ifdef __CUDACC__
// The limit in force, per translation unit. Only the persistent step kernel's copy is ever changed: a test makes one of its
// waits run out (a tag nobody writes) to exercise the recovery path, with a limit of a few re-reads so that the kernel
// still ends at once.
static __constant__ uint32_t c_poll_limit = kPollLimitDefault;
#define kPollLimit c_poll_limit
#else
constexpr uint32_t kPollLimit = kPollLimitDefault;
#endif

// A pair travels as ONE 64-bit scalar (value in the low word, tag in the high word): a naturally aligned 64-bit access is
// single-copy atomic in the PTX memory model, so a reader sees the value and the tag of the same store. (A .v2.u32 access
// is modelled as two separate 32-bit accesses.) Two pairs at once: .v2.b64, each half atomic on its own.
__device__ __forceinline__ uint4 ld_pairs2(const void* p) {  // two {value, tag} pairs, from L2
    unsigned long long a, b;
    asm volatile("ld.relaxed.gpu.global.v2.b64 {%0,%1}, [%2];" : "=l"(a), "=l"(b) : "l"(p) : "memory");
    return make_uint4(uint32_t(a), uint32_t(a >> 32), uint32_t(b), uint32_t(b >> 32));
}
__device__ __forceinline__ uint2 ld_pair(const void* p) {
    unsigned long long a;
    asm volatile("ld.relaxed.gpu.global.b64 %0, [%1];" : "=l"(a) : "l"(p) : "memory");
    return make_uint2(uint32_t(a), uint32_t(a >> 32));
}
__device__ __forceinline__ void st_pair(void* p, float value, uint32_t tag) {
    const unsigned long long a = (static_cast<unsigned long long>(tag) << 32) | __float_as_uint(value);
    asm volatile("st.relaxed.gpu.global.b64 [%0], %1;" ::"l"(p), "l"(a) : "memory");
}
__device__ __forceinline__ void poll_failed(unsigned int* error) { atomicExch(error, 1u); }
// Once any wait of the launch has run out, every later wait gives up after a few re-reads instead of running its own full
// limit: a stalled producer then costs one limit, not one per dependent operation.
__device__ __forceinline__ bool poll_abandoned(uint32_t spin, const unsigned int* error) {
    return (spin & 1023u) == 1023u && *reinterpret_cast<const volatile unsigned int*>(error) != 0u;
}
// One tagged value; bounded.
__device__ __forceinline__ float poll_pair(const void* p, uint32_t tag, unsigned int* error) {
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

// One fused multiply by CTA `cta` of `nctas` (kDecWarps warps each): the CTA rebuilds the activation row in shared
// memory (x, optionally RMS-normed, then quantised the way F takes it) and its warps walk row groups of RW rows.
//   act_smem: dec_act_smem(cols) bytes, 16-byte aligned;  tile: dec_tile_floats(CHAINS) floats (exact formats);
//   red: 32 doubles.
// Ends with every thread past its last shared-memory access except the epilogue stores; callers that reuse the shared
// memory must put a barrier after it.
// RELAX (never the default, never in a parity test): a row's block terms are added as a butterfly over the lanes instead of
// in block order - the order a GPU kernel would naturally use. It exists to put a number on what that costs in agreement
// with the reference (BRISK_CUDA_RELAXED, see launch_dec_multiply).
template <class F, int RW, bool PAIR, int kDepth, class Gate, class Io = PlainIo, bool RELAX = false>
__device__ __forceinline__ void dec_multiply_body(const DecMatParams& p, const uint32_t cta, const uint32_t nctas, unsigned char* act_smem, float* tile,
                                                  double* red, Gate&& gate, const Io& io = Io{}) {
    static_assert(!Io::kTagged || F::kExact, "tagged exchange is implemented for the exact (quantised) formats");
    static_assert(!(RELAX && Io::kTagged), "the relaxed sum exists for the one-kernel-per-operation path only");
    constexpr bool kOrdered = F::kExact && !RELAX;  // block-order row sums through the shared-memory transpose
    constexpr int MATS = PAIR ? 2 : 1;
    constexpr int CHAINS = MATS * RW;
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t total_groups = p.first_group[PAIR ? 1 : p.count];
    // Row groups are dealt round-robin over the CTAs first, then over a CTA's warps: a matrix with fewer groups than
    // the grid has warps still streams through every SM's memory pipe.
    const uint32_t stride = nctas * kDecWarps;
    const uint32_t first = warp * nctas + cta;

    auto locate = [&](uint32_t group, int& target, uint32_t& row0) {
        target = 0;
        if (!PAIR) {
            while (target + 1 < p.count && group >= p.first_group[target + 1]) ++target;
        }
        row0 = (group - p.first_group[target]) * RW;
    };
    const uint32_t units = p.m[0].units;  // all targets share cols and type
    const uint32_t steps = (units + 31) / 32;
    auto load_weights = [&](uint32_t group, uint32_t step, typename F::W (&w)[MATS][RW]) {
        int target;
        uint32_t row0;
        locate(group, target, row0);
        const uint32_t u = step * 32 + lane;
        const uint32_t uu = u < units ? u : 0;
#pragma unroll
        for (int a = 0; a < MATS; ++a)
#pragma unroll
            for (int r = 0; r < RW; ++r) w[a][r] = F::loadw(p.m[PAIR ? a : target], min(row0 + r, p.m[target].rows - 1), uu);
    };

    if (cta >= total_groups) return;  // no rows for this CTA: it must not touch the input either (see TaggedIo)
    dec_stamp(p.trace, cta, 0);
    // Weights (and the norm weights) do not depend on the previous operation: get them in flight before waiting for
    // it. A ring of kDepth iterations of weights per lane, refilled in iteration order: kDepth = 1 for the layer
    // matrices of small models (a warp has one to three iterations), deeper for long walks (the output head, 7B-class
    // layers) so that enough bytes are in flight per SM to cover HBM latency.
    typename F::W wq[kDepth][MATS][RW];
    const bool any = first < total_groups;
    const uint32_t my_groups = any ? (total_groups - first + stride - 1) / stride : 0;
    const uint32_t my_iters = my_groups * steps;
    uint32_t agroup = first, astep = 0, issued = 0;  // the next iteration to load
    auto issue = [&](typename F::W (&slot)[MATS][RW]) {
        if (issued < my_iters) {
            load_weights(agroup, astep, slot);
            ++issued;
            if (++astep == steps) {
                astep = 0;
                agroup += stride;
            }
        }
    };
#pragma unroll
    for (int d = 0; d < kDepth; ++d) issue(wq[d]);
    const uint32_t cols = p.cols;
    constexpr uint32_t kT = kDecWarps * 32;
    const uint32_t n4 = cols / 4;
    const float4* w4 = reinterpret_cast<const float4*>(p.weight);
    float4 wpre[2];  // the norm weights of this thread's first two float4s (rows up to 4096 values): no dependence on the previous operation either
#pragma unroll
    for (int k = 0; k < 2; ++k) {
        const uint32_t i = threadIdx.x + k * kT;
        wpre[k] = (p.weight != nullptr && i < n4) ? w4[i] : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    }
    gate.wait();
    dec_stamp(p.trace, cta, 1);
    if (p.trace != nullptr && cta == 0 && threadIdx.x == 0) {  // tracing only: latency of one dependent load
        const float probe = *reinterpret_cast<const volatile float*>(p.x);
        if (probe == 123456.0f) p.trace[7] = 0;
        unsigned long long t;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
        p.trace[6] = t;
    }

    // Prologue: the activation row in shared memory - f32 (normed), then the planes this format multiplies by.
    // x as float4s (row lengths are multiples of 32), up to 8 per thread in flight so that their latencies overlap.
    float* xf = reinterpret_cast<float*>(act_smem);
    const float4* x4 = reinterpret_cast<const float4*>(p.x);
    float4* xf4 = reinterpret_cast<float4*>(xf);
    double part = 0.0;
    constexpr int kBatch = Io::kTagged ? 4 : 8;  // float4s per thread in flight (the tagged form holds twice the registers per float4)
    // K = how many float4s per thread this batch really has (1, 2, 4 or 8): a 1024-value row is one float4 for half of
    // the threads, and a fixed 8-way unrolled, predicated form would have every warp issue eight times the code.
    auto load_batch = [&](uint32_t base, auto kc) {
        constexpr int K = decltype(kc)::value;
        float4 xv[K];
        if constexpr (Io::kTagged) {
            // float4 i = pairs 4i..4i+3 = two 16-byte loads; the whole batch is re-read until every tag is there
            const uint4* xp = reinterpret_cast<const uint4*>(p.x);
            uint4 a[K], b[K];
            for (uint32_t spin = 0;; ++spin) {
                bool complete = true;
#pragma unroll
                for (int k = 0; k < K; ++k) {
                    const uint32_t i = base + threadIdx.x + k * kT;
                    if (i < n4) {
                        a[k] = ld_pairs2(xp + 2 * i);
                        b[k] = ld_pairs2(xp + 2 * i + 1);
                    } else {
                        a[k] = b[k] = make_uint4(0u, io.tag_x, 0u, io.tag_x);
                    }
                }
#pragma unroll
                for (int k = 0; k < K; ++k) complete = complete && a[k].y == io.tag_x && a[k].w == io.tag_x && b[k].y == io.tag_x && b[k].w == io.tag_x;
                if (complete) break;
                if (spin == kPollLimit || poll_abandoned(spin, io.error)) {
                    poll_failed(io.error);
                    break;
                }
            }
#pragma unroll
            for (int k = 0; k < K; ++k) xv[k] = make_float4(__uint_as_float(a[k].x), __uint_as_float(a[k].z), __uint_as_float(b[k].x), __uint_as_float(b[k].z));
        } else {
#pragma unroll
            for (int k = 0; k < K; ++k) {
                const uint32_t i = base + threadIdx.x + k * kT;
                xv[k] = i < n4 ? __ldcg(x4 + i) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            }
        }
#pragma unroll
        for (int k = 0; k < K; ++k) {
            const uint32_t i = base + threadIdx.x + k * kT;
            if (i < n4) xf4[i] = xv[k];
            part += double(__fmul_rn(xv[k].x, xv[k].x));  // padding adds exact zeros
            part += double(__fmul_rn(xv[k].y, xv[k].y));
            part += double(__fmul_rn(xv[k].z, xv[k].z));
            part += double(__fmul_rn(xv[k].w, xv[k].w));
        }
    };
    for (uint32_t base = 0; base < n4; base += kBatch * kT) {
        const uint32_t left = n4 - base;
        if (left <= kT) load_batch(base, std::integral_constant<int, 1>{});
        else if (left <= 2 * kT) load_batch(base, std::integral_constant<int, 2>{});
        else if (left <= 4 * kT || kBatch == 4) load_batch(base, std::integral_constant<int, 4>{});
        else load_batch(base, std::integral_constant<int, kBatch>{});
    }
    if (p.weight != nullptr) {
        part = warp_sum(part);
        if (lane == 0) red[warp] = part;
        __syncthreads();
        double total = 0.0;
#pragma unroll
        for (int w = 0; w < kDecWarps; ++w) total += red[w];
        // total / cols; a power-of-two length divides exactly by multiplying with its reciprocal (no f64 division)
        const bool pow2 = (cols & (cols - 1)) == 0;
        const double recip = __longlong_as_double((long long)(1023 - (31 - __clz(int(cols)))) << 52);
        const float mean = float(pow2 ? total * recip : total / double(cols));
        const float scale = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(mean, p.eps)));
        dec_stamp(p.trace, cta, 2);
        auto scale_batch = [&](uint32_t base, auto kc) {
            constexpr int K = decltype(kc)::value;
            float4 wv[K];
#pragma unroll
            for (int k = 0; k < K; ++k) {
                const uint32_t i = base + threadIdx.x + k * kT;
                if (k < 2 && base == 0) wv[k] = wpre[k];
                else wv[k] = i < n4 ? w4[i] : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            }
#pragma unroll
            for (int k = 0; k < K; ++k) {
                const uint32_t i = base + threadIdx.x + k * kT;
                if (i < n4) {  // the same thread wrote xf4[i] above
                    const float4 xx = xf4[i];
                    xf4[i] = make_float4(__fmul_rn(__fmul_rn(xx.x, scale), wv[k].x), __fmul_rn(__fmul_rn(xx.y, scale), wv[k].y),
                                         __fmul_rn(__fmul_rn(xx.z, scale), wv[k].z), __fmul_rn(__fmul_rn(xx.w, scale), wv[k].w));
                }
            }
        };
        for (uint32_t base = 0; base < n4; base += 8 * kT) {
            const uint32_t left = n4 - base;
            if (left <= kT) scale_batch(base, std::integral_constant<int, 1>{});
            else if (left <= 2 * kT) scale_batch(base, std::integral_constant<int, 2>{});
            else scale_batch(base, std::integral_constant<int, 8>{});
        }
    }
    __syncthreads();
    dec_stamp(p.trace, cta, 3);
    DevAct act{};
    act.cols = cols;
    act.f32 = xf;
    unsigned char* planes = act_smem + size_t(cols) * 4;
    if constexpr (std::is_same_v<F, FQ4_0> || std::is_same_v<F, FQ4_1> || std::is_same_v<F, FQ5_0> || std::is_same_v<F, FQ8_0>) {
        int8_t* q = reinterpret_cast<int8_t*>(planes);
        float* d = reinterpret_cast<float*>(planes + cols);
        int32_t* s = reinterpret_cast<int32_t*>(planes + cols + (cols / 32) * 4);
        cta_quantize_q8_0(xf, cols, q, d, s);
        act.q0 = q; act.d0 = d; act.s0 = s;
    } else if constexpr (F::kExact) {
        int8_t* q = reinterpret_cast<int8_t*>(planes);
        float* d = reinterpret_cast<float*>(planes + cols);
        int16_t* bs = reinterpret_cast<int16_t*>(planes + cols + ((cols / 256 + 3) / 4) * 16);
        cta_quantize_q8_k(xf, cols, q, d, bs);
        act.qk = q; act.dk = d; act.bs = bs;
    }
    __syncthreads();
    gate.prologue_done();
    dec_stamp(p.trace, cta, 4);
    if (!any) return;

    float run = 0.0f;
    float acc[MATS][RW];
#pragma unroll
    for (int a = 0; a < MATS; ++a)
#pragma unroll
        for (int r = 0; r < RW; ++r) acc[a][r] = 0.0f;

    float old = 0.0f;  // the residual value a chain lane adds to (EPI_ADD), fetched while the row is being multiplied
    uint32_t group = first, step = 0;
    for (uint32_t it0 = 0; it0 < my_iters; it0 += kDepth) {
#pragma unroll
        for (int d = 0; d < kDepth; ++d) {
            const uint32_t it = it0 + d;
            if (it >= my_iters) break;
            if (kOrdered && !PAIR && step == 0 && p.epi == EPI_ADD && lane < RW) {
                int target;
                uint32_t row0;
                locate(group, target, row0);
                if (row0 + lane < p.m[target].rows) {
                    if constexpr (Io::kTagged) old = poll_pair(reinterpret_cast<const uint2*>(p.out[target]) + row0 + lane, io.tag_old, io.error);
                    else old = __ldcg(p.out[target] + row0 + lane);
                }
            }
            typename F::W w[MATS][RW];
#pragma unroll
            for (int a = 0; a < MATS; ++a)
#pragma unroll
                for (int r = 0; r < RW; ++r) w[a][r] = wq[d][a][r];
            issue(wq[d]);  // refill this slot with the iteration kDepth later

            const uint32_t u = step * 32 + lane;
            const bool valid = u < units;
            const uint32_t uu = valid ? u : 0;
            const typename F::X x = F::loadx(act, 0, uu);
#pragma unroll
            for (int a = 0; a < MATS; ++a)
#pragma unroll
                for (int r = 0; r < RW; ++r) {
                    const float term = F::term(w[a][r], x, valid, uu);
                    if constexpr (kOrdered) tile[(warp * CHAINS + a * RW + r) * 36 + lane] = term;
                    else acc[a][r] = __fadd_rn(acc[a][r], term);
                }
            if constexpr (kOrdered) {
                __syncwarp();
                if (lane < CHAINS) {
                    const int cnt = int(min(32u, units - step * 32));
                    const float4* mine = reinterpret_cast<const float4*>(tile + (warp * CHAINS + lane) * 36);
                    float v[32];  // all of the step's terms first, then the serial adds
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        const float4 q = mine[j];
                        v[4 * j] = q.x; v[4 * j + 1] = q.y; v[4 * j + 2] = q.z; v[4 * j + 3] = q.w;
                    }
                    if (cnt == 32) {
#pragma unroll
                        for (int j = 0; j < 32; j += F::kLanesPerTerm) run = __fadd_rn(run, v[j]);
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; j += F::kLanesPerTerm) run = j < cnt ? __fadd_rn(run, v[j]) : run;
                    }
                }
                __syncwarp();
            }
            if (step + 1 == steps) {  // the group's rows are complete
                int target;
                uint32_t row0;
                locate(group, target, row0);
                const DevMatrix& m = p.m[target];
                float* outp = p.out[PAIR ? 0 : target];
                if constexpr (kOrdered) {
                    const float other = PAIR ? __shfl_down_sync(0xffffffffu, run, RW) : 0.0f;
                    if (lane < RW && row0 + lane < m.rows) {
                        float result;
                        if (PAIR) result = p.epi == EPI_SILU_MUL ? silu_mul(run, other) : relu2_mul(run, other);
                        else if (p.epi == EPI_ADD) result = __fadd_rn(old, run);
                        else result = run;
                        if constexpr (Io::kTagged) {
                            st_pair(reinterpret_cast<uint2*>(outp) + row0 + lane, result, io.tag_out);
                            if (io.plain_out != nullptr) io.plain_out[row0 + lane] = result;
                        } else {
                            outp[row0 + lane] = result;
                        }
                    }
                    run = 0.0f;
                } else {
#pragma unroll
                    for (int r = 0; r < RW; ++r) {
                        const float v0 = warp_sum(acc[0][r]);
                        const float v1 = PAIR ? warp_sum(acc[MATS - 1][r]) : 0.0f;
                        if (lane == 0 && row0 + r < m.rows) {
                            float* o = outp + row0 + r;
                            if (PAIR) *o = p.epi == EPI_SILU_MUL ? silu_mul(v0, v1) : relu2_mul(v0, v1);
                            else if (p.epi == EPI_ADD) *o = __fadd_rn(__ldcg(o), v0);
                            else *o = v0;
                        }
                        acc[0][r] = 0.0f;
                        acc[MATS - 1][r] = 0.0f;
                    }
                }
            }
            if (++step == steps) {
                step = 0;
                group += stride;
            }
        }
    }
    dec_stamp(p.trace, cta, 5);
}

// ---- attention ---------------------------------------------------------------------------------------------------
struct DecAttnParams {
    const float* q;       // [heads*dim] raw projections of this token
    const float* k;       // [kv*dim]
    const float* v;       // [kv*dim]
    const float* q_norm;  // [dim] or nullptr
    const float* k_norm;
    const float* q_bias;  // [heads*dim] / [kv*dim] / [kv*dim] projection biases added before norm and RoPE, or nullptr
    const float* k_bias;
    const float* v_bias;
    const float* rope;    // [max_context][dim]
    __half* k_cache;      // [kv][max_context][dim]
    __half* v_cache;
    float* scores;        // [heads][max_context]
    float* out;           // [heads*dim]
    const uint32_t* position;
    uint32_t heads, kv_heads, dim, max_context;
    float eps, scale;
    int neox;
    int pdl;
    uint32_t slice_width;  // columns of V one CTA of the weighted sum takes (see dec_attn_slice_width)
    unsigned long long* trace;  // optional development aid: time stamps (ns) of CTA 0 - 8 words for the scores, 8 for the weighted sum
};

// Per-head RMS norm (optional) + RoPE of one head by ONE WARP, as src/model.cpp:1031-1042. Lane l holds VPL = dim/32
// values chosen so that both members of every rotation pair sit in the same lane: elements l + 32k for the NeoX
// pairing (i, i + dim/2), elements VPL*l + k for the adjacent pairing (2i, 2i+1). No block-level barrier is needed.
// `src` is read with L2 loads (it was produced by the previous operation of the step).
template <int VPL, bool NEOX>
__device__ __forceinline__ void warp_head_load(const float* src, const float* bias, float (&v)[VPL]) {
    const uint32_t lane = threadIdx.x & 31;
#pragma unroll
    for (int k = 0; k < VPL; ++k) {
        const uint32_t i = NEOX ? lane + 32 * k : VPL * lane + k;
        v[k] = __ldcg(src + i);
        if (bias != nullptr) v[k] = __fadd_rn(v[k], bias[i]);  // add_bias, src/model.cpp:1026-1030
    }
}

template <int VPL, bool NEOX>
__device__ __forceinline__ void warp_head_norm_rope(float (&v)[VPL], const float* norm, const float* rope, float eps, float* dst) {
    constexpr uint32_t dim = VPL * 32;
    const uint32_t lane = threadIdx.x & 31;
    if (norm != nullptr) {
        double part = 0.0;
#pragma unroll
        for (int k = 0; k < VPL; ++k) part += double(__fmul_rn(v[k], v[k]));
        part = warp_sum(part);
        const float mean = float(part / double(dim));
        const float scale = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(mean, eps)));
#pragma unroll
        for (int k = 0; k < VPL; ++k) v[k] = __fmul_rn(__fmul_rn(v[k], scale), norm[NEOX ? lane + 32 * k : VPL * lane + k]);
    }
#pragma unroll
    for (int k = 0; k < VPL / 2; ++k) {
        // pair (a, b): NeoX -> registers k and k + VPL/2 (elements i, i + dim/2); adjacent -> registers 2k, 2k+1 (elements 2i, 2i+1)
        const int ra = NEOX ? k : 2 * k, rb = NEOX ? k + VPL / 2 : 2 * k + 1;
        const uint32_t ia = NEOX ? lane + 32 * ra : VPL * lane + ra, ib = NEOX ? lane + 32 * rb : VPL * lane + rb;
        const uint32_t pair = NEOX ? ia : ia / 2;  // index of the (cos, sin) entry
        const float c = rope[2 * pair], sn = rope[2 * pair + 1];
        const float x0 = v[ra], x1 = v[rb];
        dst[ia] = __fsub_rn(__fmul_rn(x0, c), __fmul_rn(x1, sn));
        dst[ib] = __fadd_rn(__fmul_rn(x0, sn), __fmul_rn(x1, c));
    }
}

template <int VPL, bool NEOX>
__device__ __forceinline__ void warp_norm_rope_head_impl(const float* src, const float* bias, const float* norm, const float* rope, float eps, float* dst) {
    float v[VPL];
    warp_head_load<VPL, NEOX>(src, bias, v);
    warp_head_norm_rope<VPL, NEOX>(v, norm, rope, eps, dst);
}

template <int VPL>
__device__ __forceinline__ void warp_norm_rope_head(const float* src, const float* bias, const float* norm, const float* rope, float eps, int neox, float* dst) {
    if (neox) warp_norm_rope_head_impl<VPL, true>(src, bias, norm, rope, eps, dst);
    else warp_norm_rope_head_impl<VPL, false>(src, bias, norm, rope, eps, dst);
}

// The new position's K and V rows of K/V head `kvh`: k (already normed and rotated, in `knew`) is rounded to f16,
// stored, and read back into `knew` so that the position's own score uses the cache's value; v is rounded and stored.
// One warp; call after the warp's warp_norm_rope_head into knew and a __syncwarp().
__device__ __forceinline__ void warp_store_new_kv(const DecAttnParams& a, uint32_t kvh, uint32_t pos, float* knew) {
    const size_t base = (size_t(kvh) * a.max_context + pos) * a.dim;
    for (uint32_t i = threadIdx.x & 31; i < a.dim; i += 32) {
        const __half kh = __float2half_rn(knew[i]);
        a.k_cache[base + i] = kh;
        knew[i] = __half2float(kh);
        float v = __ldcg(a.v + size_t(kvh) * a.dim + i);
        if (a.v_bias != nullptr) v = __fadd_rn(v, a.v_bias[size_t(kvh) * a.dim + i]);
        a.v_cache[base + i] = __float2half_rn(v);
    }
}

// ---- softmax + weighted sum: one CTA of NT threads per (query head, slice of the head's dimensions) --------------
// The weighted sum is a serial chain per output dimension (position after position, as the CPU engine adds), so a head
// cannot be split by positions - but it can be split by dimensions: each CTA recomputes the head's softmax (cheap) and
// streams only its `slice_width` (16 or 32) columns of V, so that V comes in through many SMs' memory pipes at once.
// Inside the CTA the work is arranged around the one thing that cannot be parallelised, the chain of f32 adds:
//   all threads   softmax of the head's scores into shared memory
//   all threads   per chunk of 512 positions: products p[pos] * v[pos][c] (independent) into shared memory, transposed
//   one warp      lane c adds column c's products in position order: one 16-byte shared load and four dependent adds
//                 per four positions - about the latency of the adds themselves
// while the chain of one chunk runs, the other threads already request the next chunk's V.
constexpr uint32_t kVChunk = 512;                 // positions per chunk
constexpr uint32_t kProdStride = kVChunk + 4;     // floats per column of the product buffer (+4: columns fall into different banks)

// The narrowest slice (16, then 32 columns) that still gives every (head, slice) task its own CTA.
inline uint32_t dec_attn_slice_width(uint32_t heads, uint32_t dim, uint32_t ctas) { return heads * (dim / 16) > ctas ? 32u : 16u; }
// probabilities [max_context] f32 | V chunk [kVChunk][width] f16 | products [width][kProdStride] f32
inline size_t dec_attn_out_smem(uint32_t max_context, uint32_t slice_width) {
    return ((size_t(max_context) * 4 + 15) & ~size_t(15)) + size_t(kVChunk) * slice_width * sizeof(__half) + size_t(slice_width) * kProdStride * sizeof(float);
}

// With TaggedAttnIo the scores, the token's own V row (taken from the tagged v vector and rounded to f16 here, since
// the cache row written earlier in the same launch is not ordered against anything this CTA can observe) and the
// output are tagged pairs.
struct TaggedAttnIo {
    static constexpr bool kTagged = true;
    uint32_t tag_scores, tag_v, tag_out;
    unsigned int* error;
};

// raw: dec_attn_out_smem() bytes; redf / redd: NT/32 floats / doubles. V rows of earlier positions are requested
// before gate.wait(); the row of the position written by this step only after it (or, tagged, taken from the v vector).
template <int NT, class Gate, class Io = PlainIo>
__device__ __forceinline__ void dec_attn_out_body(const DecAttnParams& a, const uint32_t h, const uint32_t slice, unsigned char* raw, float* redf,
                                                  double* redd, Gate&& gate, const Io& io = Io{}, const uint64_t* exp_table = nullptr) {
    constexpr int kWarps = NT / 32;
    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, dim = a.dim, width = a.slice_width;
    const uint32_t visible = *a.position + 1, pos = visible - 1;
    const uint32_t kvh = h / (a.heads / a.kv_heads);
    float* ps = reinterpret_cast<float*>(raw);
    __half* vt = reinterpret_cast<__half*>(raw + ((size_t(a.max_context) * 4 + 15) & ~size_t(15)));
    float* prod = reinterpret_cast<float*>(vt + size_t(kVChunk) * width);
    const float* s = a.scores + size_t(h) * a.max_context;
    const __half* vbase = a.v_cache + size_t(kvh) * a.max_context * dim + slice * width;

    const uint32_t row_shift = width == 16 ? 1 : 2;  // 16-byte pieces of one position's slice: 2 or 4
    // Requests rows [first, last) of V (absolute positions) into the chunk buffer; every thread takes a share.
    auto request_rows = [&](uint32_t chunk, uint32_t first, uint32_t last) {
        if (last <= first) return;
        const uint32_t base = chunk * kVChunk;
        const uint32_t pieces = (last - first) << row_shift;
        for (uint32_t c = tid; c < pieces; c += NT) {
            const uint32_t row = first + (c >> row_shift), col = (c & ((1u << row_shift) - 1)) * 8;
            const uint32_t sm_addr = uint32_t(__cvta_generic_to_shared(vt + (row - base) * width + col));
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(sm_addr), "l"(vbase + size_t(row) * dim + col) : "memory");
        }
    };
    unsigned long long* trace = (a.trace != nullptr && h == 0 && slice == 0) ? a.trace + 8 : nullptr;
    dec_stamp(trace, 0, 0);
    const uint32_t chunks = (visible + kVChunk - 1) / kVChunk;
    request_rows(0, 0, min(kVChunk, pos));  // every earlier position of the first chunk
    gate.wait();
    dec_stamp(trace, 0, 1);
    if (!Io::kTagged && pos < kVChunk) request_rows(0, pos, pos + 1);
    asm volatile("cp.async.commit_group;" ::: "memory");

    // softmax (src/kernels_f32.cpp:275-284): max, e = expf(s - max), f64 sum, p = e * float(1/sum). The row lives in
    // shared memory; the loops have run-time trip counts (one or two rounds at short contexts) - an unrolled,
    // predicated form issues its exp code eight times whether or not a thread has a score.
    float mx = -INFINITY;
    {
        uint32_t p = tid;
        if constexpr (!Io::kTagged) {
            for (; p + 3 * NT < visible; p += 4 * NT) {  // four loads in flight: one after the other each costs an L2 round trip
                float v[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) v[u] = __ldcg(s + p + u * NT);
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    ps[p + u * NT] = v[u];
                    mx = fmaxf(mx, v[u]);
                }
            }
        }
        for (; p < visible; p += NT) {
            float v;
            if constexpr (Io::kTagged) v = poll_pair(reinterpret_cast<const uint2*>(a.scores) + size_t(h) * a.max_context + p, io.tag_scores, io.error);
            else v = __ldcg(s + p);
            ps[p] = v;
            mx = fmaxf(mx, v);
        }
    }
    mx = warp_max(mx);
    if (lane == 0) redf[warp] = mx;
    __syncthreads();
    mx = redf[0];
#pragma unroll
    for (int w = 1; w < kWarps; ++w) mx = fmaxf(mx, redf[w]);
    dec_stamp(trace, 0, 2);
    // the exps without a branch in them and, where the caller has one, with the 2^(i/32) table in shared memory; two at a time,
    // added in the same order as one at a time
    const uint64_t* table = exp_table != nullptr ? exp_table : exp2_table_device();
    double part = 0.0;
    {
        uint32_t p = tid;
        for (; p + NT < visible; p += 2 * NT) {
            const float e0 = exact_expf_flat(__fsub_rn(ps[p], mx), table), e1 = exact_expf_flat(__fsub_rn(ps[p + NT], mx), table);
            ps[p] = e0;
            ps[p + NT] = e1;
            part += double(e0);
            part += double(e1);
        }
        if (p < visible) {
            const float e = exact_expf_flat(__fsub_rn(ps[p], mx), table);
            ps[p] = e;
            part += double(e);
        }
    }
    dec_stamp(trace, 0, 3);
    part = warp_sum(part);
    if (lane == 0) redd[warp] = part;
    __syncthreads();
    double total = 0.0;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) total += redd[w];
    const float inv = float(1.0 / total);
    dec_stamp(trace, 0, 4);
    for (uint32_t p = tid; p < visible; p += NT) ps[p] = __fmul_rn(ps[p], inv);

    // weighted sum (src/kernels_f32.cpp:265-273): out[i] += p[pos] * v[pos][i], position after position.
    float acc = 0.0f;
    for (uint32_t c = 0; c < chunks; ++c) {
        const uint32_t base = c * kVChunk, rows = min(kVChunk, visible - base);
        if constexpr (Io::kTagged) {
            if (c + 1 == chunks && tid < width) {  // the token's own row, from the tagged v vector
                float v = poll_pair(reinterpret_cast<const uint2*>(a.v) + size_t(kvh) * dim + slice * width + tid, io.tag_v, io.error);
                if (a.v_bias != nullptr) v = __fadd_rn(v, a.v_bias[size_t(kvh) * dim + slice * width + tid]);
                vt[(pos - base) * width + tid] = __float2half_rn(v);
            }
        }
        asm volatile("cp.async.wait_group 0;" ::: "memory");  // this thread's share of the chunk's V
        __syncthreads();  // V chunk c (and, the first time, the probabilities) complete; the previous chunk's chain is done
        if (c == 0) dec_stamp(trace, 0, 6);
        // products, transposed: consecutive threads take consecutive columns of one position
        for (uint32_t e = tid; e < rows * width; e += NT) {
            const uint32_t r = e >> (row_shift + 3), col = e & (width - 1);  // width is 16 or 32
            prod[col * kProdStride + r] = __fmul_rn(ps[base + r], __half2float(vt[e]));
        }
        __syncthreads();  // products complete; the V buffer is free again
        if (c == 0) dec_stamp(trace, 0, 7);
        if (c + 1 < chunks) {
            request_rows(c + 1, base + kVChunk, min(base + 2 * kVChunk, Io::kTagged ? pos : visible));
            asm volatile("cp.async.commit_group;" ::: "memory");
        }
        if (warp == 0 && lane < width) {
            const float* mine = prod + lane * kProdStride;
            uint32_t j = 0;
            if (rows >= 16) {  // the next 16 products are loaded while the current 16 adds - the dependent chain - run
                float4 n0 = *reinterpret_cast<const float4*>(mine), n1 = *reinterpret_cast<const float4*>(mine + 4);
                float4 n2 = *reinterpret_cast<const float4*>(mine + 8), n3 = *reinterpret_cast<const float4*>(mine + 12);
                for (; j + 16 <= rows; j += 16) {
                    const float4 p0 = n0, p1 = n1, p2 = n2, p3 = n3;
                    if (j + 32 <= rows) {
                        n0 = *reinterpret_cast<const float4*>(mine + j + 16); n1 = *reinterpret_cast<const float4*>(mine + j + 20);
                        n2 = *reinterpret_cast<const float4*>(mine + j + 24); n3 = *reinterpret_cast<const float4*>(mine + j + 28);
                    }
                    acc = __fadd_rn(acc, p0.x); acc = __fadd_rn(acc, p0.y); acc = __fadd_rn(acc, p0.z); acc = __fadd_rn(acc, p0.w);
                    acc = __fadd_rn(acc, p1.x); acc = __fadd_rn(acc, p1.y); acc = __fadd_rn(acc, p1.z); acc = __fadd_rn(acc, p1.w);
                    acc = __fadd_rn(acc, p2.x); acc = __fadd_rn(acc, p2.y); acc = __fadd_rn(acc, p2.z); acc = __fadd_rn(acc, p2.w);
                    acc = __fadd_rn(acc, p3.x); acc = __fadd_rn(acc, p3.y); acc = __fadd_rn(acc, p3.z); acc = __fadd_rn(acc, p3.w);
                }
            }
            for (; j < rows; ++j) acc = __fadd_rn(acc, mine[j]);
        }
    }
    dec_stamp(trace, 0, 5);
    if (warp == 0 && lane < width) {
        if constexpr (Io::kTagged) st_pair(reinterpret_cast<uint2*>(a.out) + size_t(h) * dim + slice * width + lane, acc, io.tag_out);
        else a.out[size_t(h) * dim + slice * width + lane] = acc;
    }
}

#endif  // __CUDACC__

}  // namespace bk
