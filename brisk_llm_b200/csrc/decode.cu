// Fused kernels of the single-token step (batch-1 decode), six per layer:
//
//   multiply   norm+quantise prologue -> q/k/v | o (+residual) | gate,up (+activation) | down (+residual) | head
//   scores     per-head norm + RoPE of q and of the new k, f16 K/V store, q.k for every visible position
//   attend     softmax + position-ordered weighted sum of V
//
// Every kernel can be launched with programmatic dependent launch (it then starts while its predecessor drains, issues
// the loads that do not depend on it - its first weight units - and only then waits, griddepcontrol.wait, for the
// predecessor's results); see pdl_mode() for why that is off by default. The activation vector a multiply needs (RMS
// norm, 8-bit quantisation) is recomputed by every CTA in shared memory instead of by a separate one-CTA kernel. All arithmetic is the reference's, in the
// reference's order (see formats.cuh, rowops.cuh, exact_math.h), so the step stays bit-identical to the CPU engine.
#include <cstdlib>
#include <type_traits>

#include "formats.cuh"
#include "kernels.h"
#include "rowops.cuh"

namespace bk {
namespace {

__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// How the step's kernels overlap: 0 = plain stream order (default); 1 = programmatic dependent launch, dependents
// released as soon as a kernel starts (several later kernels may sit resident, waiting); 2 = dependents released
// after a kernel's prologue (only the next kernel runs ahead). Measured on B200 with the 0.6B-shaped model, 8
// layers: 411 / 482 / 452 us per token for modes 0 / 1 / 2 - the resident waiting CTAs cost more than the weight
// prefetch gains, so the default is 0. BRISK_CUDA_PDL selects another mode for experiments.
int pdl_mode() {
    static const int mode = [] {
        const char* env = std::getenv("BRISK_CUDA_PDL");
        return env != nullptr ? std::atoi(env) : 0;
    }();
    return mode;
}

template <class... Params, class... Args>
void launch_pdl(void (*kernel)(Params...), dim3 grid, dim3 block, size_t smem, cudaStream_t s, Args&&... args) {
    if (pdl_mode() == 0) {
        kernel<<<grid, block, smem, s>>>(std::forward<Args>(args)...);
        BK_CUDA(cudaGetLastError());
        return;
    }
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr{};
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    BK_CUDA(cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...));
}

// ---- multiply ---------------------------------------------------------------------------------------------------
constexpr int kDecWarps = 16;  // the per-CTA prologue (norm + quantise) is shared by more warps, and there are fewer CTAs to repeat it

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

__device__ __forceinline__ void stamp(unsigned long long* trace, int slot) {
    if (trace != nullptr && blockIdx.x == 0 && threadIdx.x == 0) {
        unsigned long long t;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
        trace[slot] = t;

    }
}

template <class F, int RW, bool PAIR, int kDepth>
__global__ void __launch_bounds__(kDecWarps * 32) dec_matvec_kernel(const DecMatParams p) {
    constexpr int MATS = PAIR ? 2 : 1;
    constexpr int CHAINS = MATS * RW;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __shared__ __align__(16) float tile[F::kExact ? kDecWarps : 1][F::kExact ? CHAINS : 1][36];
    __shared__ double red[32];

    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t total_groups = p.first_group[PAIR ? 1 : p.count];
    const uint32_t stride = gridDim.x * kDecWarps;
    const uint32_t first = blockIdx.x * kDecWarps + warp;

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

    stamp(p.trace, 0);
    // Weights (and the norm weights) do not depend on the previous kernel: get them in flight before waiting for it.
    // A ring of kDepth iterations of weights per lane, refilled in iteration order: kDepth = 1 for the layer matrices
    // (a warp has one to three iterations), deeper for long walks (the output head, 7B-class layers) so that enough
    // bytes are in flight per SM to cover HBM latency.
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
    if (p.pdl == 1) pdl_launch_dependents();
    pdl_wait();
    stamp(p.trace, 1);
    if (p.trace != nullptr && blockIdx.x == 0 && threadIdx.x == 0) {  // tracing only: latency of one dependent load
        const float probe = *reinterpret_cast<const volatile float*>(p.x);
        if (probe == 123456.0f) p.trace[7] = 0;
        unsigned long long t;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
        p.trace[6] = t;
    }

    // Prologue: the activation row in shared memory - f32 (normed), then the planes this format multiplies by.
    // Loads are batched in registers (8 per thread in flight) so that their latencies overlap.
    float* xf = reinterpret_cast<float*>(smem_raw);
    constexpr uint32_t kT = kDecWarps * 32;
    // x as float4s (row lengths are multiples of 32), up to 8 per thread at a time so the loads overlap
    const float4* x4 = reinterpret_cast<const float4*>(p.x);
    float4* xf4 = reinterpret_cast<float4*>(xf);
    const uint32_t n4 = cols / 4;
    double part = 0.0;
    for (uint32_t base = 0; base < n4; base += 8 * kT) {
        float4 xv[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            const uint32_t i = base + threadIdx.x + k * kT;
            xv[k] = i < n4 ? x4[i] : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        }
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            const uint32_t i = base + threadIdx.x + k * kT;
            if (i < n4) xf4[i] = xv[k];
            part += double(__fmul_rn(xv[k].x, xv[k].x));  // padding adds exact zeros
            part += double(__fmul_rn(xv[k].y, xv[k].y));
            part += double(__fmul_rn(xv[k].z, xv[k].z));
            part += double(__fmul_rn(xv[k].w, xv[k].w));
        }
    }
    if (p.weight != nullptr) {
        part = warp_sum(part);
        if (lane == 0) red[warp] = part;
        __syncthreads();
        double total = 0.0;
#pragma unroll
        for (int w = 0; w < kDecWarps; ++w) total += red[w];
        const float mean = float(total / double(cols));
        const float scale = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(mean, p.eps)));
        stamp(p.trace, 2);
        const float4* w4 = reinterpret_cast<const float4*>(p.weight);
        for (uint32_t base = 0; base < n4; base += 8 * kT) {
            float4 wv[8];
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                const uint32_t i = base + threadIdx.x + k * kT;
                wv[k] = i < n4 ? w4[i] : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            }
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                const uint32_t i = base + threadIdx.x + k * kT;
                if (i < n4) {  // the same thread wrote xf4[i] above
                    const float4 xx = xf4[i];
                    xf4[i] = make_float4(__fmul_rn(__fmul_rn(xx.x, scale), wv[k].x), __fmul_rn(__fmul_rn(xx.y, scale), wv[k].y),
                                         __fmul_rn(__fmul_rn(xx.z, scale), wv[k].z), __fmul_rn(__fmul_rn(xx.w, scale), wv[k].w));
                }
            }
        }
    }
    __syncthreads();
    stamp(p.trace, 3);
    DevAct act{};
    act.cols = cols;
    act.f32 = xf;
    unsigned char* planes = smem_raw + size_t(cols) * 4;
    if constexpr (std::is_same_v<F, FQ4_0> || std::is_same_v<F, FQ8_0>) {
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
    if (p.pdl == 2) pdl_launch_dependents();
    stamp(p.trace, 4);
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
            if (F::kExact && !PAIR && step == 0 && p.epi == EPI_ADD && lane < RW) {
                int target;
                uint32_t row0;
                locate(group, target, row0);
                if (row0 + lane < p.m[target].rows) old = p.out[target][row0 + lane];
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
                    if constexpr (F::kExact) tile[warp][a * RW + r][lane] = term;
                    else acc[a][r] = __fadd_rn(acc[a][r], term);
                }
            if constexpr (F::kExact) {
                __syncwarp();
                if (lane < CHAINS) {
                    const int cnt = int(min(32u, units - step * 32));
                    const float4* mine = reinterpret_cast<const float4*>(tile[warp][lane]);
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
                if constexpr (F::kExact) {
                    const float other = PAIR ? __shfl_down_sync(0xffffffffu, run, RW) : 0.0f;
                    if (lane < RW && row0 + lane < m.rows) {
                        float* o = outp + row0 + lane;
                        if (PAIR) *o = p.epi == EPI_SILU_MUL ? silu_mul(run, other) : relu2_mul(run, other);
                        else if (p.epi == EPI_ADD) *o = __fadd_rn(old, run);
                        else *o = run;
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
                            else if (p.epi == EPI_ADD) *o = __fadd_rn(*o, v0);
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
    stamp(p.trace, 5);
}

template <class F, int RW, bool PAIR>
void launch_dec_one(DecMatParams& p, uint32_t sms, cudaStream_t s) {
    uint32_t groups = 0;
    const int targets = PAIR ? 1 : p.count;
    for (int i = 0; i < targets; ++i) {
        p.first_group[i] = groups;
        groups += (p.m[i].rows + RW - 1) / RW;
    }
    p.first_group[targets] = groups;
    const uint32_t want = (groups + kDecWarps - 1) / kDecWarps;
    const uint32_t grid = want < sms ? want : sms;  // one CTA per SM at most; warps walk the remaining row groups
    const size_t smem = size_t(p.cols) * 4 + p.cols + (p.cols / 32) * 8 + 64;
    // Ring depth: as deep as keeps the weights in flight per lane (matrices x rows x depth units of 16 bytes) at 8 or
    // fewer, so that they stay in registers; one iteration ahead is enough when a warp has only a few iterations.
    const uint32_t iters = ((groups + grid * kDecWarps - 1) / (grid * kDecWarps)) * ((p.m[0].units + 31) / 32);
    constexpr int kRegsPerIter = (PAIR ? 2 : 1) * RW * int(sizeof(typename F::W) / 4);  // registers one iteration's weights take
    constexpr int kDeep = kRegsPerIter * 4 <= 48 ? 4 : kRegsPerIter * 2 <= 48 ? 2 : 1;
    auto go = [&](auto kernel) {
        if (smem > 40 * 1024) BK_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024));
        launch_pdl(kernel, dim3(grid), dim3(kDecWarps * 32), smem, s, p);
    };
    if (iters > 2 && kDeep > 1) go(dec_matvec_kernel<F, RW, PAIR, kDeep>);
    else go(dec_matvec_kernel<F, RW, PAIR, 1>);
}

template <class F>
void dispatch_dec(DecMatParams& p, bool pair, uint32_t sms, cudaStream_t s) {
    uint32_t rows = 0;
    bool div4 = true, div2 = true;
    for (int i = 0; i < (pair ? 1 : p.count); ++i) rows += p.m[i].rows;
    for (int i = 0; i < p.count; ++i) {
        div4 = div4 && p.m[i].rows % 4 == 0;
        div2 = div2 && p.m[i].rows % 2 == 0;
    }
    // Rows per warp: more rows per warp share the activation loads and the serial adds (fewer instructions per weight
    // byte), as long as about half of all warps still get a row group.
    const uint32_t enough = sms * kDecWarps / 2;
    constexpr bool heavy = sizeof(typename F::W) > 32;  // K-quants: many registers per row, cap the rows per warp
    int rw = 1;
    if (div4 && !heavy && rows / 4 >= enough) rw = 4;
    else if (div2 && (!heavy || !pair) && rows / 2 >= enough) rw = 2;
    if (pair) {
        if (rw == 4) launch_dec_one<F, 4, true>(p, sms, s);
        else if (rw == 2) launch_dec_one<F, 2, true>(p, sms, s);
        else launch_dec_one<F, 1, true>(p, sms, s);
    } else {
        if (rw == 4) launch_dec_one<F, 4, false>(p, sms, s);
        else if (rw == 2) launch_dec_one<F, 2, false>(p, sms, s);
        else launch_dec_one<F, 1, false>(p, sms, s);
    }
}

// ---- attention scores with the per-head norm, RoPE and cache store in the prologue --------------------------------
struct DecAttnParams {
    const float* q;       // [heads*dim] raw projections of this token
    const float* k;       // [kv*dim]
    const float* v;       // [kv*dim]
    const float* q_norm;  // [dim] or nullptr
    const float* k_norm;
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
};

// Per-head RMS norm (optional) + RoPE of one head by ONE WARP, as src/model.cpp:1031-1042. Lane l holds VPL = dim/32
// values chosen so that both members of every rotation pair sit in the same lane: elements l + 32k for the NeoX
// pairing (i, i + dim/2), elements VPL*l + k for the adjacent pairing (2i, 2i+1). No block-level barrier is needed.
template <int VPL, bool NEOX>
__device__ __forceinline__ void warp_norm_rope_head_impl(const float* src, const float* norm, const float* rope, float eps, float* dst) {
    constexpr uint32_t dim = VPL * 32;
    const uint32_t lane = threadIdx.x & 31;
    float v[VPL];
#pragma unroll
    for (int k = 0; k < VPL; ++k) v[k] = src[NEOX ? lane + 32 * k : VPL * lane + k];
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
        constexpr int dummy = 0;
        (void)dummy;
        const int ra = NEOX ? k : 2 * k, rb = NEOX ? k + VPL / 2 : 2 * k + 1;
        const uint32_t ia = NEOX ? lane + 32 * ra : VPL * lane + ra, ib = NEOX ? lane + 32 * rb : VPL * lane + rb;
        const uint32_t pair = NEOX ? ia : ia / 2;  // index of the (cos, sin) entry
        const float c = rope[2 * pair], sn = rope[2 * pair + 1];
        const float x0 = v[ra], x1 = v[rb];
        dst[ia] = __fsub_rn(__fmul_rn(x0, c), __fmul_rn(x1, sn));
        dst[ib] = __fadd_rn(__fmul_rn(x0, sn), __fmul_rn(x1, c));
    }
}

template <int VPL>
__device__ __forceinline__ void warp_norm_rope_head(const float* src, const float* norm, const float* rope, float eps, int neox, float* dst) {
    if (neox) warp_norm_rope_head_impl<VPL, true>(src, norm, rope, eps, dst);
    else warp_norm_rope_head_impl<VPL, false>(src, norm, rope, eps, dst);
}

template <int GROUP, int DIM>
__global__ void __launch_bounds__(128) dec_attn_scores_kernel(const DecAttnParams a) {
    extern __shared__ float sm[];  // q heads [GROUP][DIM] | new k [DIM]
    if (a.pdl != 0) pdl_launch_dependents();
    pdl_wait();
    constexpr uint32_t dim = DIM;
    const uint32_t kvh = blockIdx.y;
    const uint32_t pos = *a.position, visible = pos + 1;
    const uint32_t begin = blockIdx.x * 128;
    if (begin >= visible) return;
    const uint32_t p = begin + threadIdx.x;
    // The cached K row of this thread's position: all of it in flight before anything else (the new position's own
    // row is produced below instead).
    uint4 kraw[DIM / 8];
    const bool cached = p < visible && p != pos;
    if (cached) {
        const uint4* kr = reinterpret_cast<const uint4*>(a.k_cache + (size_t(kvh) * a.max_context + p) * dim);
#pragma unroll
        for (int i = 0; i < DIM / 8; ++i) kraw[i] = kr[i];
    }
    float* qs = sm;
    float* knew = sm + GROUP * dim;
    const float* rope = a.rope + size_t(pos) * dim;
    const uint32_t warp = threadIdx.x >> 5;
    const bool owns_new = pos >= begin && pos < begin + 128;  // this CTA's chunk holds the token's own position
    for (uint32_t task = warp; task < GROUP + 1u; task += 4) {
        if (task < GROUP) {
            warp_norm_rope_head<DIM / 32>(a.q + size_t(kvh * GROUP + task) * dim, a.q_norm, rope, a.eps, a.neox, qs + task * dim);
        } else if (owns_new) {
            warp_norm_rope_head<DIM / 32>(a.k + size_t(kvh) * dim, a.k_norm, rope, a.eps, a.neox, knew);
            __syncwarp();
            const size_t base = (size_t(kvh) * a.max_context + pos) * dim;
            for (uint32_t i = threadIdx.x & 31; i < dim; i += 32) {
                const __half kh = __float2half_rn(knew[i]);
                a.k_cache[base + i] = kh;
                knew[i] = __half2float(kh);  // the score of the own position reads the cache's f16 value
                a.v_cache[base + i] = __float2half_rn(a.v[size_t(kvh) * dim + i]);
            }
        }
    }
    __syncthreads();
    if (p >= visible) return;
    float lanes[GROUP][16];
#pragma unroll
    for (int g = 0; g < GROUP; ++g)
#pragma unroll
        for (int j = 0; j < 16; ++j) lanes[g][j] = 0.0f;
#pragma unroll
    for (int i = 0; i < DIM; i += 16) {
        float kf[16];
        if (!cached) {
#pragma unroll
            for (int j = 0; j < 16; ++j) kf[j] = knew[i + j];
        } else {
            const __half2* h0 = reinterpret_cast<const __half2*>(&kraw[i / 8]);
            const __half2* h1 = reinterpret_cast<const __half2*>(&kraw[i / 8 + 1]);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float2 f0 = __half22float2(h0[j]), f1 = __half22float2(h1[j]);
                kf[2 * j] = f0.x; kf[2 * j + 1] = f0.y; kf[8 + 2 * j] = f1.x; kf[8 + 2 * j + 1] = f1.y;
            }
        }
#pragma unroll
        for (int g = 0; g < GROUP; ++g) {
            const float4* q4 = reinterpret_cast<const float4*>(qs + g * dim + i);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float4 q = q4[j];
                lanes[g][4 * j + 0] = __fadd_rn(lanes[g][4 * j + 0], __fmul_rn(q.x, kf[4 * j + 0]));
                lanes[g][4 * j + 1] = __fadd_rn(lanes[g][4 * j + 1], __fmul_rn(q.y, kf[4 * j + 1]));
                lanes[g][4 * j + 2] = __fadd_rn(lanes[g][4 * j + 2], __fmul_rn(q.z, kf[4 * j + 2]));
                lanes[g][4 * j + 3] = __fadd_rn(lanes[g][4 * j + 3], __fmul_rn(q.w, kf[4 * j + 3]));
            }
        }
    }
#pragma unroll
    for (int g = 0; g < GROUP; ++g) {
        float sum = 0.0f;
#pragma unroll
        for (int j = 0; j < 16; ++j) sum = __fadd_rn(sum, lanes[g][j]);
        a.scores[size_t(kvh * GROUP + g) * a.max_context + p] = __fmul_rn(sum, a.scale);
    }
}

// ---- softmax + weighted sum: one CTA per query head -----------------------------------------------------------------
constexpr uint32_t kVTile = 64;   // positions of V per stage
constexpr uint32_t kVStages = 4;  // stages in flight: the serial chain consumes a tile faster than L2 delivers one

__global__ void __launch_bounds__(256) dec_attn_out_kernel(const DecAttnParams a) {
    extern __shared__ __align__(16) unsigned char raw[];  // probabilities [max_context] | V ring kVStages x [kVTile][dim] f16
    __shared__ float redf[8];
    __shared__ double redd[8];
    if (a.pdl != 0) pdl_launch_dependents();
    pdl_wait();
    const uint32_t h = blockIdx.x, tid = threadIdx.x, dim = a.dim;
    const uint32_t visible = *a.position + 1;
    const uint32_t kvh = h / (a.heads / a.kv_heads);
    float* ps = reinterpret_cast<float*>(raw);
    __half* vt = reinterpret_cast<__half*>(raw + ((size_t(a.max_context) * 4 + 15) & ~size_t(15)));
    const float* s = a.scores + size_t(h) * a.max_context;
    const __half* vbase = a.v_cache + size_t(kvh) * a.max_context * dim;

    // V tiles stream through a ring of shared-memory stages with cp.async; start them before the softmax.
    const uint32_t tiles = (visible + kVTile - 1) / kVTile;
    const uint32_t chunks_per_tile = kVTile * dim / 8;  // 16-byte chunks
    auto stage = [&](uint32_t tile_index) {
        if (tile_index < tiles) {
            __half* dst = vt + size_t(tile_index % kVStages) * kVTile * dim;
            const __half* src = vbase + size_t(tile_index) * kVTile * dim;
            const uint32_t rows = min(kVTile, visible - tile_index * kVTile);
            for (uint32_t c = tid; c < chunks_per_tile; c += 256) {
                if (c * 8 < rows * dim) {
                    const uint32_t sm_addr = uint32_t(__cvta_generic_to_shared(dst + c * 8));
                    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(sm_addr), "l"(src + c * 8) : "memory");
                }
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");  // one group per tile index, empty past the end
    };
    for (uint32_t t = 0; t + 1 < kVStages; ++t) stage(t);

    // softmax (src/kernels_f32.cpp:275-284): max, e = expf(s - max), f64 sum, p = e * float(1/sum). Up to 8 scores per
    // thread stay in registers (contexts up to 2048); longer rows go through shared memory.
    const bool in_regs = visible <= 8 * 256;
    float sv[8];
    float mx = -INFINITY;
    if (in_regs) {
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            const uint32_t p = tid + k * 256;
            sv[k] = p < visible ? s[p] : -INFINITY;
            mx = fmaxf(mx, sv[k]);
        }
    } else {
        for (uint32_t p = tid; p < visible; p += 256) {
            const float v = s[p];
            ps[p] = v;
            mx = fmaxf(mx, v);
        }
    }
    mx = warp_max(mx);
    if ((tid & 31) == 0) redf[tid >> 5] = mx;
    __syncthreads();
    mx = redf[0];
#pragma unroll
    for (int w = 1; w < 8; ++w) mx = fmaxf(mx, redf[w]);
    double part = 0.0;
    if (in_regs) {
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            if (tid + k * 256 < visible) {
                sv[k] = exact_expf(__fsub_rn(sv[k], mx));
                part += double(sv[k]);
            }
        }
    } else {
        for (uint32_t p = tid; p < visible; p += 256) {
            const float e = exact_expf(__fsub_rn(ps[p], mx));
            ps[p] = e;
            part += double(e);
        }
    }
    part = warp_sum(part);
    if ((tid & 31) == 0) redd[tid >> 5] = part;
    __syncthreads();
    double total = 0.0;
#pragma unroll
    for (int w = 0; w < 8; ++w) total += redd[w];
    const float inv = float(1.0 / total);
    if (in_regs) {
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            const uint32_t p = tid + k * 256;
            if (p < visible) ps[p] = __fmul_rn(sv[k], inv);
        }
    } else {
        for (uint32_t p = tid; p < visible; p += 256) ps[p] = __fmul_rn(ps[p], inv);
    }

    // weighted sum (src/kernels_f32.cpp:265-273): out[i] += p[pos] * v[pos][i], position after position.
    float acc = 0.0f;
    for (uint32_t t = 0; t < tiles; ++t) {
        stage(t + kVStages - 1);  // refills the stage consumed in the previous iteration
        asm volatile("cp.async.wait_group %0;" ::"n"(kVStages - 1) : "memory");
        __syncthreads();  // tile t has landed for every thread (and ps is complete on the first pass)
        if (tid < dim) {
            const __half* tv = vt + size_t(t % kVStages) * kVTile * dim + tid;
            const uint32_t rows = min(kVTile, visible - t * kVTile);
            const float* pw = ps + t * kVTile;
            if (rows == kVTile) {
#pragma unroll
                for (uint32_t j = 0; j < kVTile; ++j) acc = __fadd_rn(acc, __fmul_rn(pw[j], __half2float(tv[j * dim])));
            } else {
                for (uint32_t j = 0; j < rows; ++j) acc = __fadd_rn(acc, __fmul_rn(pw[j], __half2float(tv[j * dim])));
            }
        }
        __syncthreads();  // everyone is done with tile t before its stage is refilled
    }
    if (tid < dim) a.out[size_t(h) * dim + tid] = acc;
}

}  // namespace

// The launchers below are declared in kernels.h.

void launch_dec_multiply(const MatTarget* targets, int count, const float* x, const float* norm_weight, float eps, uint32_t cols, Epilogue epi,
                         uint32_t sms, cudaStream_t s, unsigned long long* trace) {
    const bool pair = epi == EPI_SILU_MUL || epi == EPI_RELU2_MUL;
    if (count < 1 || count > 3 || (pair && count != 2)) throw CudaError("cuda: a fused multiply takes 1 to 3 targets (2 for a pair)");
    DecMatParams p{};
    p.count = count;
    p.epi = epi;
    p.x = x;
    p.weight = norm_weight;
    p.eps = eps;
    p.cols = cols;
    p.trace = trace;
    p.pdl = pdl_mode();
    for (int i = 0; i < count; ++i) {
        if (targets[i].m.type != targets[0].m.type || targets[i].m.cols != cols) throw CudaError("cuda: fused multiply needs matrices of one type and input size");
        p.m[i] = targets[i].m;
        p.out[i] = targets[i].out;
    }
    if (pair && targets[0].m.rows != targets[1].m.rows) throw CudaError("cuda: gate and up must have the same rows");
    switch (targets[0].m.type) {
        case T_Q4_0: dispatch_dec<FQ4_0>(p, pair, sms, s); break;
        case T_Q8_0: dispatch_dec<FQ8_0>(p, pair, sms, s); break;
        case T_Q4_K: dispatch_dec<FQ4_K>(p, pair, sms, s); break;
        case T_Q6_K: dispatch_dec<FQ6_K>(p, pair, sms, s); break;
        case T_TQ2_0: dispatch_dec<FTQ2_0>(p, pair, sms, s); break;
        case T_F16: dispatch_dec<FF16>(p, pair, sms, s); break;
        case T_F32: dispatch_dec<FF32>(p, pair, sms, s); break;
        default: throw CudaError("cuda: unsupported weight type");
    }
}

void launch_dec_attention(const RopeArgs& r, const AttnArgs& at, cudaStream_t s) {
    DecAttnParams a{};
    a.q = r.q; a.k = r.k; a.v = r.v; a.q_norm = r.q_norm; a.k_norm = r.k_norm; a.rope = r.rope;
    a.k_cache = r.k_cache; a.v_cache = r.v_cache; a.scores = at.scores; a.out = at.out; a.position = r.position;
    a.heads = r.heads; a.kv_heads = r.kv_heads; a.dim = r.dim; a.max_context = r.max_context;
    a.eps = r.eps; a.scale = at.scale; a.neox = r.neox;
    a.pdl = pdl_mode();
    const uint32_t group = a.heads / a.kv_heads;
    if (a.dim % 16 != 0 || a.dim > 256) throw CudaError("cuda: head size must be a multiple of 16 up to 256");
    const dim3 grid((a.max_context + 127) / 128, a.kv_heads);
    const size_t smem = size_t(group + 1) * a.dim * sizeof(float);
#define BK_SCORES(G)                                                                                       \
    if (a.dim == 128) launch_pdl(dec_attn_scores_kernel<G, 128>, grid, dim3(128), smem, s, a);             \
    else if (a.dim == 64) launch_pdl(dec_attn_scores_kernel<G, 64>, grid, dim3(128), smem, s, a);          \
    else throw CudaError("cuda: the single-token attention kernel takes head sizes 64 and 128")
    switch (group) {
        case 1: BK_SCORES(1); break;
        case 2: BK_SCORES(2); break;
        case 4: BK_SCORES(4); break;
        case 8: BK_SCORES(8); break;
        default: throw CudaError("cuda: query heads per K/V head must be 1, 2, 4 or 8");
    }
#undef BK_SCORES
    const size_t smem2 = ((size_t(a.max_context) * 4 + 15) & ~size_t(15)) + size_t(kVStages) * kVTile * a.dim * sizeof(__half);
    static bool raised = false;
    if (smem2 > 40 * 1024 && !raised) {
        BK_CUDA(cudaFuncSetAttribute(dec_attn_out_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        raised = true;
    }
    if (smem2 > 200 * 1024) throw CudaError("cuda: context too long for the single-token attention kernel");
    launch_pdl(dec_attn_out_kernel, dim3(a.heads), dim3(256), smem2, s, a);
}

}  // namespace bk
