// The whole single-token step of every layer as ONE persistent kernel: one CTA per SM, the layer operations as phases
// separated by grid-wide barriers instead of kernel boundaries.
//
//   per layer:  q/k/v multiply | scores (+ per-head norm, RoPE, K/V store) | softmax + weighted sum | output
//               projection (+residual) | gate/up (+activation) | down (+residual)
//
// Why: at batch 1 a layer operation of a 0.6B-class model moves a few megabytes and lasts 3-5 us as its own kernel, of
// which the weight stream is a fraction - the rest is launch and drain, the scheduling gap between graph nodes, and the
// first-load latency of every CTA. Inside one kernel a CTA issues the weight loads of its next rows BEFORE it waits at
// the barrier, so the HBM latency of a phase hides behind the tail of the previous one, and a barrier (one release
// reduction, one acquire poll) costs about a microsecond.
//
// The phases call the same device bodies as the one-kernel-per-operation path (decode_body.cuh): the arithmetic and its
// order are unchanged, results stay bit-identical to the CPU engine.
//
// Barrier: a monotonic arrival counter; barrier k opens when it reaches k x CTAs. Every CTA arrives once per phase and
// waits once per barrier, also when it has no work in a phase (otherwise its early arrivals would open a later barrier
// too soon). The last CTA to leave the kernel zeroes the counter for the next launch. Every wait is bounded: after
// kSpinLimit polls (about a second) the CTA sets the error word, stops waiting at this and every later barrier, and
// the kernel runs to its end with meaningless results; the host checks the word after the launch and raises. The launch
// is cooperative, so the CTAs are co-resident or the launch itself fails.
#include <algorithm>
#include <cstdio>
#include <cstring>
#include <initializer_list>
#include <utility>

#include "decode_body.cuh"

namespace bk {

struct StepLayerDesc {
    DecMatParams qkv, o, gate_up, down;
    DecAttnParams attn;
};

namespace {

constexpr uint32_t kStepThreads = kDecWarps * 32;
constexpr uint32_t kSpinLimit = 1u << 21;

struct StepParams {
    const StepLayerDesc* layers;
    uint32_t n_layers;
    unsigned int* sync;   // [0] arrivals, [1] exits, [2] error
    uint32_t tile_offset; // bytes from the start of dynamic shared memory to the transpose tile (after the widest activation row)
};

__device__ __forceinline__ unsigned int ld_acquire(const unsigned int* p) {
    unsigned int v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void red_release_add(unsigned int* p, unsigned int v) {
    asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

struct GridGate {
    unsigned int* sync;
    unsigned int target;  // arrivals that open the next barrier
    unsigned int nctas;
    bool waited;          // this phase's barrier has been passed (or the phase needs none)

    __device__ __forceinline__ void wait() {
        if (waited) return;
        waited = true;
        if (threadIdx.x == 0) {
            const volatile unsigned int* error = sync + 2;
            if (*error == 0) {
                unsigned int spins = 0;
                while (int(ld_acquire(sync) - target) < 0) {
                    if (++spins > kSpinLimit || ((spins & 255u) == 0 && *error != 0)) {
                        atomicExch(sync + 2, 1u);
                        break;
                    }
                    if (spins > 16) __nanosleep(64);
                }
            }
            __threadfence();
        }
        __syncthreads();
    }
    __device__ __forceinline__ void prologue_done() {}
    // End of a phase: make sure this phase's barrier was passed, publish the phase's results, arm the next barrier.
    __device__ __forceinline__ void arrive() {
        wait();
        __syncthreads();  // every thread's stores of this phase are issued
        if (threadIdx.x == 0) {
            __threadfence();
            red_release_add(sync, 1u);
        }
        target += nctas;
        waited = false;
    }
};

// Scores of the new token against every visible position: tasks of (K/V head, 512 positions), one position per thread,
// the query heads of the group one after another against the thread's K row. The row waits in shared memory (each
// thread copies its own 2*dim bytes with cp.async, requested before the barrier; rows are padded by 16 bytes so that the
// 16-byte reads of a quarter warp fall into distinct banks) - held in registers it would not fit the 128 registers a
// 512-thread CTA has per thread. The task that covers the token's own position norms, rotates and stores the new K and
// V rows. sm: (group + 1) * dim floats, then 512 padded K rows.
__host__ __device__ inline size_t step_scores_smem(uint32_t group, uint32_t dim) {
    return size_t(group + 1) * dim * sizeof(float) + size_t(kStepThreads) * (dim * 2 + 16);
}

__device__ __forceinline__ void step_scores(const DecAttnParams& a, const uint32_t cta, const uint32_t nctas, unsigned char* sm, GridGate& gate) {
    const uint32_t dim = a.dim, group = a.heads / a.kv_heads;
    const uint32_t pos = *a.position, visible = pos + 1;
    const uint32_t chunks = (visible + kStepThreads - 1) / kStepThreads;
    const uint32_t tasks = a.kv_heads * chunks;
    const uint32_t warp = threadIdx.x >> 5;
    float* qs = reinterpret_cast<float*>(sm);
    float* knew = qs + group * dim;
    const uint4* krow = reinterpret_cast<const uint4*>(sm + size_t(group + 1) * dim * sizeof(float) + size_t(threadIdx.x) * (dim * 2 + 16));
    const float* rope = a.rope + size_t(pos) * dim;
    for (uint32_t task = cta; task < tasks; task += nctas) {
        const uint32_t kvh = task / chunks, begin = (task % chunks) * kStepThreads;
        const uint32_t p = begin + threadIdx.x;
        const bool cached = p < visible && p != pos;
        if (cached) {
            const __half* kr = a.k_cache + (size_t(kvh) * a.max_context + p) * dim;
            const uint32_t dst = uint32_t(__cvta_generic_to_shared(krow));
            for (uint32_t i = 0; i < dim / 8; ++i) {
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst + i * 16), "l"(kr + i * 8) : "memory");
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
        gate.wait();
        const bool owns_new = pos >= begin && pos < begin + kStepThreads;
        for (uint32_t t = warp; t < group + 1u; t += kDecWarps) {
            if (t < group) {
                const float* src = a.q + size_t(kvh * group + t) * dim;
                if (dim == 128) warp_norm_rope_head<4>(src, a.q_norm, rope, a.eps, a.neox, qs + t * dim);
                else warp_norm_rope_head<2>(src, a.q_norm, rope, a.eps, a.neox, qs + t * dim);
            } else if (owns_new) {
                const float* src = a.k + size_t(kvh) * dim;
                if (dim == 128) warp_norm_rope_head<4>(src, a.k_norm, rope, a.eps, a.neox, knew);
                else warp_norm_rope_head<2>(src, a.k_norm, rope, a.eps, a.neox, knew);
                __syncwarp();
                warp_store_new_kv(a, kvh, pos, knew);
            }
        }
        asm volatile("cp.async.wait_group 0;" ::: "memory");  // this thread's own row
        __syncthreads();
        if (p < visible) {
            for (uint32_t g = 0; g < group; ++g) {
                float lanes[16];
#pragma unroll
                for (int j = 0; j < 16; ++j) lanes[j] = 0.0f;
                for (uint32_t i = 0; i < dim; i += 16) {
                    float kf[16];
                    if (!cached) {
#pragma unroll
                        for (int j = 0; j < 16; ++j) kf[j] = knew[i + j];
                    } else {
                        const uint4 r0 = krow[i / 8], r1 = krow[i / 8 + 1];
                        const __half2* h0 = reinterpret_cast<const __half2*>(&r0);
                        const __half2* h1 = reinterpret_cast<const __half2*>(&r1);
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const float2 f0 = __half22float2(h0[j]), f1 = __half22float2(h1[j]);
                            kf[2 * j] = f0.x; kf[2 * j + 1] = f0.y; kf[8 + 2 * j] = f1.x; kf[8 + 2 * j + 1] = f1.y;
                        }
                    }
                    const float4* q4 = reinterpret_cast<const float4*>(qs + g * dim + i);
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const float4 q = q4[j];
                        lanes[4 * j + 0] = __fadd_rn(lanes[4 * j + 0], __fmul_rn(q.x, kf[4 * j + 0]));
                        lanes[4 * j + 1] = __fadd_rn(lanes[4 * j + 1], __fmul_rn(q.y, kf[4 * j + 1]));
                        lanes[4 * j + 2] = __fadd_rn(lanes[4 * j + 2], __fmul_rn(q.z, kf[4 * j + 2]));
                        lanes[4 * j + 3] = __fadd_rn(lanes[4 * j + 3], __fmul_rn(q.w, kf[4 * j + 3]));
                    }
                }
                float sum = 0.0f;
#pragma unroll
                for (int j = 0; j < 16; ++j) sum = __fadd_rn(sum, lanes[j]);
                a.scores[size_t(kvh * group + g) * a.max_context + p] = __fmul_rn(sum, a.scale);
            }
        }
        __syncthreads();  // qs / knew and the K rows are rewritten by the CTA's next task
    }
}

constexpr int ring_depth(int regs_per_iter, bool deep) { return !deep ? 1 : regs_per_iter * 4 <= 48 ? 4 : regs_per_iter * 2 <= 48 ? 2 : 1; }

template <class F, int RWA, int RWO, int RWG, int RWD, bool DEEP>
__global__ void __launch_bounds__(kStepThreads, 1) step_kernel(const StepParams P) {
    extern __shared__ __align__(16) unsigned char smem[];
    __shared__ double red[32];
    __shared__ float redf[kDecWarps];
    constexpr int kWordsPerUnit = int(sizeof(typename F::W) / 4);
    float* tile = reinterpret_cast<float*>(smem + P.tile_offset);
    const uint32_t cta = blockIdx.x, nctas = gridDim.x;
    GridGate gate{P.sync, 0u, nctas, true};  // the first phase reads what earlier kernels wrote: no barrier

    for (uint32_t l = 0; l < P.n_layers; ++l) {
        const StepLayerDesc& L = P.layers[l];
        dec_multiply_body<F, RWA, false, ring_depth(RWA * kWordsPerUnit, DEEP)>(L.qkv, cta, nctas, smem, tile, red, gate);
        gate.arrive();

        step_scores(L.attn, cta, nctas, smem, gate);
        gate.arrive();

        for (uint32_t h = cta; h < L.attn.heads; h += nctas) {
            dec_attn_out_body<kStepThreads>(L.attn, h, smem, redf, red, gate);
            __syncthreads();  // the shared-memory row of probabilities is rewritten for the CTA's next head
        }
        gate.arrive();

        dec_multiply_body<F, RWO, false, ring_depth(RWO * kWordsPerUnit, DEEP)>(L.o, cta, nctas, smem, tile, red, gate);
        gate.arrive();

        dec_multiply_body<F, RWG, true, ring_depth(2 * RWG * kWordsPerUnit, DEEP)>(L.gate_up, cta, nctas, smem, tile, red, gate);
        gate.arrive();

        dec_multiply_body<F, RWD, false, ring_depth(RWD * kWordsPerUnit, DEEP)>(L.down, cta, nctas, smem, tile, red, gate);
        if (l + 1 < P.n_layers) gate.arrive();
    }

    // Leave: the last CTA out re-arms the counters for the next launch (every CTA is past all of its waits by then).
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        const unsigned int before = atomicAdd(P.sync + 1, 1u);
        if (before + 1 == nctas) {
            P.sync[0] = 0;
            P.sync[1] = 0;
            __threadfence();
        }
    }
}

using StepKernel = void (*)(StepParams);

struct Variant {
    int rw[4];  // rows per warp of the q/k/v, output, gate/up and down multiplies
    StepKernel kernel;
};

template <class F>
const Variant* variants(int& count) {
    constexpr bool heavy = sizeof(typename F::W) > 32;  // K-quants hold many registers per row
    if constexpr (heavy) {
        static const Variant v[] = {{{2, 2, 1, 2}, step_kernel<F, 2, 2, 1, 2, true>},
                                    {{2, 1, 1, 1}, step_kernel<F, 2, 1, 1, 1, false>},
                                    {{1, 1, 1, 1}, step_kernel<F, 1, 1, 1, 1, false>}};
        count = 3;
        return v;
    } else {
        static const Variant v[] = {{{4, 2, 4, 2}, step_kernel<F, 4, 2, 4, 2, true>},
                                    {{2, 1, 2, 1}, step_kernel<F, 2, 1, 2, 1, false>},
                                    {{1, 1, 1, 1}, step_kernel<F, 1, 1, 1, 1, false>}};
        count = 3;
        return v;
    }
}

const Variant* variants_of(int type, int& count) {
    switch (type) {
        case T_Q4_0: return variants<FQ4_0>(count);
        case T_Q8_0: return variants<FQ8_0>(count);
        case T_Q4_K: return variants<FQ4_K>(count);
        case T_Q6_K: return variants<FQ6_K>(count);
        case T_TQ2_0: return variants<FTQ2_0>(count);
        default: count = 0; return nullptr;
    }
}

// Rows per warp one multiply would like: more rows share the activation loads and the serial adds, as long as about
// half of all warps still get a row group (the rule of the one-kernel-per-operation path).
int wanted_rows_per_warp(const DecMatParams& p, bool pair, uint32_t sms) {
    uint32_t rows = 0;
    bool div4 = true, div2 = true;
    for (int i = 0; i < (pair ? 1 : p.count); ++i) rows += p.m[i].rows;
    for (int i = 0; i < p.count; ++i) {
        div4 = div4 && p.m[i].rows % 4 == 0;
        div2 = div2 && p.m[i].rows % 2 == 0;
    }
    const uint32_t enough = sms * kDecWarps / 2;
    if (div4 && rows / 4 >= enough) return 4;
    if (div2 && rows / 2 >= enough) return 2;
    return 1;
}

}  // namespace

struct StepPlan::Impl {
    StepKernel kernel = nullptr;
    StepLayerDesc* layers_dev = nullptr;
    unsigned int* sync_dev = nullptr;
    uint32_t n_layers = 0, grid = 0, tile_offset = 0;
    size_t smem = 0;
};

StepPlan::StepPlan() = default;
StepPlan::~StepPlan() {
    if (impl_ != nullptr) {
        if (impl_->layers_dev) cudaFree(impl_->layers_dev);
        if (impl_->sync_dev) cudaFree(impl_->sync_dev);
        delete impl_;
    }
}

bool StepPlan::build(const std::vector<StepLayerArgs>& layers, const StepShared& sh, uint32_t sms, cudaStream_t s, std::string& why_not) {
    if (layers.empty()) {
        why_not = "no layers";
        return false;
    }
    const int type = layers[0].q.type;
    for (const StepLayerArgs& L : layers) {
        for (const DevMatrix* m : {&L.q, &L.k, &L.v, &L.o, &L.gate, &L.up, &L.down}) {
            if (m->type != type) {
                why_not = "the layer matrices are not all of one type";
                return false;
            }
        }
    }
    int count = 0;
    const Variant* list = variants_of(type, count);
    if (list == nullptr) {
        why_not = "no persistent kernel for this weight type";
        return false;
    }
    if (sh.dim != 64 && sh.dim != 128) {
        why_not = "head size is not 64 or 128";
        return false;
    }
    const uint32_t group = sh.heads / sh.kv_heads;
    if (group > 8) {
        why_not = "more than 8 query heads per K/V head";
        return false;
    }

    std::vector<StepLayerDesc> descs(layers.size());
    for (size_t l = 0; l < layers.size(); ++l) {
        const StepLayerArgs& L = layers[l];
        StepLayerDesc& d = descs[l];
        std::memset(static_cast<void*>(&d), 0, sizeof(d));
        auto fill = [&](DecMatParams& p, std::initializer_list<std::pair<const DevMatrix*, float*>> targets, const float* x, const float* w, uint32_t cols, int epi) {
            p.count = 0;
            for (const auto& t : targets) {
                p.m[p.count] = *t.first;
                p.out[p.count] = t.second;
                ++p.count;
            }
            p.epi = epi; p.x = x; p.weight = w; p.eps = sh.eps; p.cols = cols; p.trace = nullptr; p.pdl = 0;
        };
        fill(d.qkv, {{&L.q, sh.q}, {&L.k, sh.k}, {&L.v, sh.v}}, sh.hidden, L.attn_norm, sh.hidden_size, EPI_STORE);
        fill(d.o, {{&L.o, sh.hidden}}, sh.attended, L.attn_sub_norm, sh.heads * sh.dim, EPI_ADD);
        fill(d.gate_up, {{&L.gate, sh.gated}, {&L.up, nullptr}}, sh.hidden, L.ffn_norm, sh.hidden_size, sh.act_epi);
        fill(d.down, {{&L.down, sh.hidden}}, sh.gated, L.ffn_sub_norm, sh.ffn_size, EPI_ADD);
        DecAttnParams& a = d.attn;
        a.q = sh.q; a.k = sh.k; a.v = sh.v; a.q_norm = L.q_norm; a.k_norm = L.k_norm; a.rope = sh.rope;
        a.k_cache = L.k_cache; a.v_cache = L.v_cache; a.scores = sh.scores; a.out = sh.attended; a.position = sh.position;
        a.heads = sh.heads; a.kv_heads = sh.kv_heads; a.dim = sh.dim; a.max_context = sh.max_context;
        a.eps = sh.eps; a.scale = sh.scale; a.neox = sh.neox; a.pdl = 0;
    }
    // One variant for all layers: the rows per warp every layer can take.
    int want[4] = {4, 4, 4, 4};
    for (StepLayerDesc& d : descs) {
        want[0] = std::min(want[0], wanted_rows_per_warp(d.qkv, false, sms));
        want[1] = std::min(want[1], wanted_rows_per_warp(d.o, false, sms));
        want[2] = std::min(want[2], wanted_rows_per_warp(d.gate_up, true, sms));
        want[3] = std::min(want[3], wanted_rows_per_warp(d.down, false, sms));
    }
    const Variant* pick = nullptr;
    for (int i = 0; i < count && pick == nullptr; ++i) {
        bool fits = true;
        for (int k = 0; k < 4; ++k) fits = fits && list[i].rw[k] <= want[k];
        if (fits) pick = &list[i];
    }
    if (pick == nullptr) {
        why_not = "no kernel variant fits the row counts";
        return false;
    }
    for (StepLayerDesc& d : descs) {
        dec_assign_groups(d.qkv, pick->rw[0], false);
        dec_assign_groups(d.o, pick->rw[1], false);
        dec_assign_groups(d.gate_up, pick->rw[2], true);
        dec_assign_groups(d.down, pick->rw[3], false);
    }

    const uint32_t widest = std::max(std::max(sh.hidden_size, sh.heads * sh.dim), sh.ffn_size);
    const size_t act = (dec_act_smem(widest) + 15) & ~size_t(15);
    const size_t multiply = act + dec_tile_floats(8) * sizeof(float);
    const size_t attention = std::max(dec_attn_out_smem(sh.max_context, sh.dim), step_scores_smem(group, sh.dim));
    const size_t smem = std::max(multiply, attention);
    int dev = 0, limit = 0, coop = 0;
    BK_CUDA(cudaGetDevice(&dev));
    BK_CUDA(cudaDeviceGetAttribute(&limit, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev));
    BK_CUDA(cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, dev));
    if (coop == 0) {
        why_not = "the device has no cooperative launch";
        return false;
    }
    if (smem + 1024 > size_t(limit)) {
        why_not = "the context is too long for the persistent kernel's shared memory";
        return false;
    }
    BK_CUDA(cudaFuncSetAttribute(pick->kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)));
    int per_sm = 0;
    BK_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, pick->kernel, int(kStepThreads), smem));
    if (per_sm < 1) {
        why_not = "the persistent kernel does not fit an SM";
        return false;
    }

    impl_ = new Impl();
    impl_->kernel = pick->kernel;
    impl_->n_layers = uint32_t(descs.size());
    impl_->grid = sms;
    impl_->tile_offset = uint32_t(act);
    impl_->smem = smem;
    BK_CUDA(cudaMalloc(&impl_->layers_dev, descs.size() * sizeof(StepLayerDesc)));
    BK_CUDA(cudaMalloc(&impl_->sync_dev, 64));
    BK_CUDA(cudaMemcpyAsync(impl_->layers_dev, descs.data(), descs.size() * sizeof(StepLayerDesc), cudaMemcpyHostToDevice, s));
    BK_CUDA(cudaMemsetAsync(impl_->sync_dev, 0, 64, s));
    BK_CUDA(cudaStreamSynchronize(s));  // descs goes out of scope
    char text[96];
    std::snprintf(text, sizeof text, "rows per warp %d/%d/%d/%d, %u CTAs, %zu KB shared", pick->rw[0], pick->rw[1], pick->rw[2], pick->rw[3], sms, smem / 1024);
    description_ = text;
    return true;
}

void StepPlan::launch(cudaStream_t s) const {
    StepParams P{};
    P.layers = impl_->layers_dev;
    P.n_layers = impl_->n_layers;
    P.sync = impl_->sync_dev;
    P.tile_offset = impl_->tile_offset;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(impl_->grid);
    cfg.blockDim = dim3(kStepThreads);
    cfg.dynamicSmemBytes = impl_->smem;
    cfg.stream = s;
    cudaLaunchAttribute attr{};
    attr.id = cudaLaunchAttributeCooperative;
    attr.val.cooperative = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    BK_CUDA(cudaLaunchKernelEx(&cfg, impl_->kernel, P));
}

const unsigned int* StepPlan::error_word() const { return impl_->sync_dev + 2; }

void StepPlan::rearm(cudaStream_t s) {
    BK_CUDA(cudaMemsetAsync(impl_->sync_dev, 0, 64, s));
    BK_CUDA(cudaStreamSynchronize(s));
}

}  // namespace bk
