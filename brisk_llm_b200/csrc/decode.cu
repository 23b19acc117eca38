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
#include <cstring>
#include <type_traits>

#include "decode_body.cuh"

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
struct PdlGate {  // the gate of the one-kernel-per-operation path: programmatic dependent launch, or nothing
    int pdl;
    __device__ __forceinline__ void wait() {
        if (pdl == 1) pdl_launch_dependents();
        pdl_wait();
    }
    __device__ __forceinline__ void prologue_done() {
        if (pdl == 2) pdl_launch_dependents();
    }
};

template <class F, int RW, bool PAIR, int kDepth, bool RELAX = false>
__global__ void __launch_bounds__(kDecWarps * 32) dec_matvec_kernel(const DecMatParams p) {
    constexpr int CHAINS = (PAIR ? 2 : 1) * RW;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __shared__ __align__(16) float tile[F::kExact && !RELAX ? dec_tile_floats(CHAINS) : 1];
    __shared__ double red[32];
    dec_multiply_body<F, RW, PAIR, kDepth, PdlGate, PlainIo, RELAX>(p, blockIdx.x, gridDim.x, smem_raw, tile, red, PdlGate{p.pdl});
}

// BRISK_CUDA_RELAXED: a comma-separated list of the orders to relax in the one-kernel-per-operation single-token path -
// "rowsum" (butterfly row sums in the multiplies), "attention" (split-position softmax and weighted sum combined afterwards,
// with the fast exp). Off by default and never used by a parity test: the exact order is what makes the results the
// reference's; these switches exist so that the cost of giving it up can be measured (tests/test_gpu_relaxed.py).
bool relaxed(const char* what) {
    const char* env = std::getenv("BRISK_CUDA_RELAXED");
    return env != nullptr && (std::strstr(env, what) != nullptr || std::strstr(env, "all") != nullptr);
}

template <class F, int RW, bool PAIR>
void launch_dec_one(DecMatParams& p, uint32_t sms, cudaStream_t s) {
    const uint32_t groups = dec_assign_groups(p, RW, PAIR);
    const uint32_t grid = groups < sms ? groups : sms;  // one CTA per SM; row groups go round-robin over CTAs, then warps
    const size_t smem = dec_act_smem(p.cols);
    // Ring depth: as deep as keeps the weights in flight per lane (matrices x rows x depth units of 16 bytes) at 8 or
    // fewer, so that they stay in registers; one iteration ahead is enough when a warp has only a few iterations.
    const uint32_t iters = ((groups + grid * kDecWarps - 1) / (grid * kDecWarps)) * ((p.m[0].units + 31) / 32);
    constexpr int kRegsPerIter = (PAIR ? 2 : 1) * RW * F::kRegs;  // registers one iteration's weights take
    constexpr int kDeep = kRegsPerIter * 4 <= 48 ? 4 : kRegsPerIter * 2 <= 48 ? 2 : 1;
    auto go = [&](auto kernel) {
        if (smem > 40 * 1024) BK_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024));
        launch_pdl(kernel, dim3(grid), dim3(kDecWarps * 32), smem, s, p);
    };
    if constexpr (F::kExact && RW <= 2) {  // the relaxed variants, for the measurement only (fewer shapes: compile time)
        if (relaxed("rowsum")) {
            go(dec_matvec_kernel<F, RW, PAIR, 1, true>);
            return;
        }
    }
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
    if (relaxed("rowsum")) div4 = false;
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
            warp_norm_rope_head<DIM / 32>(a.q + size_t(kvh * GROUP + task) * dim, a.q_bias ? a.q_bias + size_t(kvh * GROUP + task) * dim : nullptr, a.q_norm, rope, a.eps,
                                          a.neox, qs + task * dim);
        } else if (owns_new) {
            warp_norm_rope_head<DIM / 32>(a.k + size_t(kvh) * dim, a.k_bias ? a.k_bias + size_t(kvh) * dim : nullptr, a.k_norm, rope, a.eps, a.neox, knew);
            __syncwarp();
            warp_store_new_kv(a, kvh, pos, knew);
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
struct PdlGateEarly {  // releases the dependents as soon as the kernel runs
    int pdl;
    __device__ __forceinline__ void wait() {
        if (pdl != 0) pdl_launch_dependents();
        pdl_wait();
    }
};

__global__ void __launch_bounds__(256) dec_attn_out_kernel(const DecAttnParams a) {
    extern __shared__ __align__(16) unsigned char raw[];
    __shared__ float redf[8];
    __shared__ double redd[8];
    __shared__ uint64_t table[32];
    if (threadIdx.x < 32) table[threadIdx.x] = exp2_table_device()[threadIdx.x];  // ordered before its use by the body's first barrier
    dec_attn_out_body<256>(a, blockIdx.x, blockIdx.y, raw, redf, redd, PdlGateEarly{a.pdl}, PlainIo{}, table);
}

// ---- relaxed order, for the measurement only (BRISK_CUDA_RELAXED=attention) -------------------------------------------
// The usual GPU formulation of single-token attention: the positions are split into eight ranges, each range reduces its own
// maximum, its sum of (fast) exps and its weighted sum of V, and a second kernel combines the eight with the usual rescaling.
// Every sum is in another order than the reference's (position after position over the whole context, glibc's expf).
constexpr uint32_t kFlashSplits = 8;
constexpr uint32_t kFlashHeads = 64;
// the ranges' partial results [head][range][dim + 2]; in the library image because the step is captured into a graph, where
// nothing may be allocated (270 KB; only ever touched when the measurement switch is on)
__device__ float g_flash_partial[kFlashHeads * kFlashSplits * 130];
__global__ void __launch_bounds__(128) dec_attn_flash_kernel(const DecAttnParams a, float* partial) {
    const uint32_t h = blockIdx.x, split = blockIdx.y, dim = a.dim, tid = threadIdx.x;
    const uint32_t visible = *a.position + 1, kvh = h / (a.heads / a.kv_heads);
    const uint32_t per = (visible + kFlashSplits - 1) / kFlashSplits, begin = split * per, end = min(visible, begin + per);
    const float* s = a.scores + size_t(h) * a.max_context;
    __shared__ float red[4];
    float m = -INFINITY;
    for (uint32_t p = begin + tid; p < end; p += 128) m = fmaxf(m, s[p]);
    m = warp_max(m);
    if ((tid & 31) == 0) red[tid >> 5] = m;
    __syncthreads();
    m = fmaxf(fmaxf(red[0], red[1]), fmaxf(red[2], red[3]));
    float l = 0.0f, acc = 0.0f;
    for (uint32_t p = begin; p < end; ++p) {
        const float e = __expf(s[p] - m);
        l += e;
        if (tid < dim) acc = fmaf(e, __half2float(a.v_cache[(size_t(kvh) * a.max_context + p) * dim + tid]), acc);
    }
    float* out = partial + (size_t(h) * kFlashSplits + split) * (dim + 2);
    if (tid < dim) out[tid] = acc;
    if (tid == 0) {
        out[dim] = m;
        out[dim + 1] = l;
    }
}
__global__ void __launch_bounds__(128) dec_attn_combine_kernel(const DecAttnParams a, const float* partial) {
    const uint32_t h = blockIdx.x, dim = a.dim, tid = threadIdx.x;
    const float* in = partial + size_t(h) * kFlashSplits * (dim + 2);
    float m = -INFINITY;
    for (uint32_t i = 0; i < kFlashSplits; ++i) m = fmaxf(m, in[i * (dim + 2) + dim]);
    float l = 0.0f, acc = 0.0f;
    for (uint32_t i = 0; i < kFlashSplits; ++i) {
        const float li = in[i * (dim + 2) + dim + 1];
        if (li == 0.0f) continue;  // an empty range
        const float w = __expf(in[i * (dim + 2) + dim] - m);
        l = fmaf(li, w, l);
        if (tid < dim) acc = fmaf(in[i * (dim + 2) + tid], w, acc);
    }
    if (tid < dim) a.out[size_t(h) * dim + tid] = acc / l;
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
        case T_Q4_1: dispatch_dec<FQ4_1>(p, pair, sms, s); break;
        case T_Q5_0: dispatch_dec<FQ5_0>(p, pair, sms, s); break;
        case T_Q8_0: dispatch_dec<FQ8_0>(p, pair, sms, s); break;
        case T_Q5_K: dispatch_dec<FQ5_K>(p, pair, sms, s); break;
        case T_Q4_K: dispatch_dec<FQ4_K>(p, pair, sms, s); break;
        case T_Q6_K: dispatch_dec<FQ6_K>(p, pair, sms, s); break;
        case T_TQ2_0: dispatch_dec<FTQ2_0>(p, pair, sms, s); break;
        case T_F16: dispatch_dec<FF16>(p, pair, sms, s); break;
        case T_F32: dispatch_dec<FF32>(p, pair, sms, s); break;
        default: throw CudaError("cuda: unsupported weight type");
    }
}

bool dec_attention_fits(uint32_t max_context, uint32_t heads, uint32_t dim, uint32_t sms) {
    return dec_attn_out_smem(max_context, dec_attn_slice_width(heads, dim, sms)) <= 200 * 1024;
}

void launch_dec_attention(const RopeArgs& r, const AttnArgs& at, uint32_t sms, cudaStream_t s) {
    DecAttnParams a{};
    a.q = r.q; a.k = r.k; a.v = r.v; a.q_norm = r.q_norm; a.k_norm = r.k_norm; a.rope = r.rope;
    a.q_bias = r.q_bias; a.k_bias = r.k_bias; a.v_bias = r.v_bias;
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
        case 3: BK_SCORES(3); break;
        case 4: BK_SCORES(4); break;
        case 5: BK_SCORES(5); break;
        case 6: BK_SCORES(6); break;
        case 7: BK_SCORES(7); break;
        case 8: BK_SCORES(8); break;
        default: throw CudaError("cuda: query heads per K/V head must be 1 to 8");
    }
#undef BK_SCORES
    if (relaxed("attention")) {  // measurement only: split-position softmax and weighted sum
        float* partial = nullptr;
        BK_CUDA(cudaGetSymbolAddress(reinterpret_cast<void**>(&partial), g_flash_partial));
        if (a.heads > kFlashHeads || a.dim > 128) throw CudaError("cuda: the relaxed attention measurement takes up to 64 heads of up to 128 values");
        dec_attn_flash_kernel<<<dim3(a.heads, kFlashSplits), 128, 0, s>>>(a, partial);
        dec_attn_combine_kernel<<<a.heads, 128, 0, s>>>(a, partial);
        BK_CUDA(cudaGetLastError());
        return;
    }
    {
        // Long contexts (and BRISK_CUDA_CHAIN=1): the single-token kernel of attn_chain.cu instead of the fused one below -
        // same results; at 8192 positions ~43 us per layer against ~75.
        const int mode = chain_mode();
        if ((mode == 1 || (mode != 0 && a.max_context >= kChainOneMinContext)) && attn_chain_one_fits(a.dim, a.max_context)) {
            AttnArgs one = at;
            one.n = 1;
            one.max_visible = a.max_context;
            one.window = 0;
            launch_attn_chain_one(one, s);
            return;
        }
    }
    a.slice_width = dec_attn_slice_width(a.heads, a.dim, sms);
    const size_t smem2 = dec_attn_out_smem(a.max_context, a.slice_width);
    static DeviceOnce once;
    if (smem2 > 40 * 1024 && once.first()) BK_CUDA(cudaFuncSetAttribute(dec_attn_out_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    if (smem2 > 200 * 1024) throw CudaError("cuda: context too long for the single-token attention kernel");
    launch_pdl(dec_attn_out_kernel, dim3(a.heads, a.dim / a.slice_width), dim3(256), smem2, s, a);
}

}  // namespace bk
