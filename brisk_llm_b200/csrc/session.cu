// The CUDA session behind include/brisk_cuda.h: weights repacked once into HBM, an f16 K/V cache,
// scratch for one batch, the forward pass of Session::eval_batch (src/model.cpp:867-1212) as a
// sequence of kernel launches on one stream, and a captured CUDA graph for the single-token step.
#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <memory>
#include <string>
#include <thread>
#include <vector>

#include <dlfcn.h>

#include "../../include/brisk_cuda.h"
#include "kernels.h"

namespace bk {

// NCCL is bound at run time (dlopen), so the library has no link-time dependency on it and, inside a process that
// already loaded a NCCL (PyTorch's), uses that same copy. Only the five calls below are needed.
struct NcclId {
    char internal[128];
};
struct Nccl {
    void* lib = nullptr;
    int (*GetUniqueId)(NcclId*) = nullptr;
    int (*CommInitRank)(void**, int, NcclId, int) = nullptr;
    int (*AllGather)(const void*, void*, size_t, int, void*, cudaStream_t) = nullptr;
    int (*CommDestroy)(void*) = nullptr;
    const char* (*GetErrorString)(int) = nullptr;

    static Nccl& get() {
        static Nccl n = [] {
            Nccl x;
            const char* env = std::getenv("BRISK_NCCL_LIB");
            const char* names[] = {env, "libnccl.so.2", "libnccl.so"};
            for (const char* name : names) {
                if (name == nullptr) continue;
                x.lib = dlopen(name, RTLD_NOW | RTLD_GLOBAL);
                if (x.lib != nullptr) break;
            }
            if (x.lib == nullptr) return x;
            x.GetUniqueId = reinterpret_cast<int (*)(NcclId*)>(dlsym(x.lib, "ncclGetUniqueId"));
            x.CommInitRank = reinterpret_cast<int (*)(void**, int, NcclId, int)>(dlsym(x.lib, "ncclCommInitRank"));
            x.AllGather = reinterpret_cast<int (*)(const void*, void*, size_t, int, void*, cudaStream_t)>(dlsym(x.lib, "ncclAllGather"));
            x.CommDestroy = reinterpret_cast<int (*)(void*)>(dlsym(x.lib, "ncclCommDestroy"));
            x.GetErrorString = reinterpret_cast<const char* (*)(int)>(dlsym(x.lib, "ncclGetErrorString"));
            return x;
        }();
        return n;
    }
    bool ok() const { return lib && GetUniqueId && CommInitRank && AllGather && CommDestroy && GetErrorString; }
    void check(int rc, const char* what) const {
        if (rc != 0) throw CudaError(std::string("cuda: ") + what + " failed: " + (GetErrorString ? GetErrorString(rc) : "nccl error"));
    }
};
constexpr int kNcclFloat = 7;  // ncclFloat32

struct DevBuffer;

namespace {

constexpr uint32_t kMaxBatch = 512;   // tokens per prefill pass (the reference: 256 on the CPU, 512 on Metal)
constexpr uint32_t kMaxScored = 64;   // Engine::kMaxScoredTokens, src/engine.h:32

}  // namespace

struct DevBuffer {
    void* p = nullptr;
    size_t bytes = 0;
    DevBuffer() = default;
    DevBuffer(const DevBuffer&) = delete;
    DevBuffer& operator=(const DevBuffer&) = delete;
    ~DevBuffer() { if (p) cudaFree(p); }
    void alloc(size_t n) {
        bytes = n;
        BK_CUDA(cudaMalloc(&p, n ? n : 16));
    }
    template <class T> T* as() const { return static_cast<T*>(p); }
};

namespace {

struct Layer {
    DevMatrix q, k, v, o, gate, up, down;
    const float *attn_norm = nullptr, *q_norm = nullptr, *k_norm = nullptr, *attn_sub_norm = nullptr, *ffn_norm = nullptr, *ffn_sub_norm = nullptr;
    const float *q_bias = nullptr, *k_bias = nullptr, *v_bias = nullptr;  // this rank's rows
    const float *attn_post_norm = nullptr, *ffn_post_norm = nullptr;      // Gemma: norm of a projection before the residual add
    bool slides = false;                                                  // Gemma: sliding-window layer with the local RoPE table
    bool no_rope = false;                                                 // SmolLM3: the layer attends without rotation
    __half *k_cache = nullptr, *v_cache = nullptr;
};

std::string gb(uint64_t bytes) {
    char buf[32];
    std::snprintf(buf, sizeof buf, "%.2f GB", double(bytes) / 1e9);
    return buf;
}

// Mirrors the allocations of Session::load for a description and options (tensor-parallel share included).
brisk_cuda_memory estimate(const brisk_cuda_model& m, const brisk_cuda_options& opt) {
    brisk_cuda_memory e{};
    const uint64_t tp = opt.tp_size > 1 ? uint64_t(opt.tp_size) : 1;
    const uint64_t hidden = m.hidden, ffn = m.ffn, vocab = m.vocab_size, dim = m.head_dim;
    const uint64_t q_dim = uint64_t(m.head_count) * dim, kv_dim = uint64_t(m.kv_head_count) * dim;
    const uint64_t ctx = opt.max_context == 0 ? m.context_length : std::min<uint64_t>(opt.max_context, m.context_length);
    auto planes = [](int type, uint64_t rows, uint64_t cols) { return uint64_t(plane_sizes(type == T_BF16 ? int(T_F32) : type, uint32_t(rows), uint32_t(cols)).total()); };
    e.weights += planes(m.token_embd.type, vocab, hidden);
    if (m.output.data != nullptr || tp > 1) e.weights += planes(m.output.data != nullptr ? m.output.type : m.token_embd.type, vocab / tp, hidden);
    e.weights += hidden * 4;
    for (uint32_t l = 0; l < m.layer_count; ++l) {
        const brisk_cuda_layer& L = m.layers[l];
        e.weights += planes(L.q.type, q_dim / tp, hidden) + planes(L.k.type, kv_dim / tp, hidden) + planes(L.v.type, kv_dim / tp, hidden);
        e.weights += planes(L.o.type, hidden / tp, q_dim) + planes(L.gate.type, ffn / tp, hidden) + planes(L.up.type, ffn / tp, hidden);
        e.weights += planes(L.down.type, hidden / tp, ffn);
        e.weights += (2 * hidden + (L.q_norm ? dim : 0) + (L.k_norm ? dim : 0) + (L.attn_sub_norm ? q_dim : 0) + (L.ffn_sub_norm ? ffn : 0) +
                      (L.q_bias ? (q_dim + 2 * kv_dim) / tp : 0) + (L.attn_post_norm ? hidden : 0) + (L.ffn_post_norm ? hidden : 0)) * 4;
    }
    e.cache = uint64_t(m.layer_count) * 2 * (kv_dim / tp) * ctx * 2;
    const uint64_t widest = std::max(std::max(hidden, q_dim), ffn), batch = kMaxBatch;
    e.scratch += batch * (hidden + q_dim / tp + 2 * kv_dim / tp + q_dim / tp + 2 * ffn) * 4;  // residual, q, k, v, attended, gated, up
    e.scratch += batch * widest * (4 + 1 + 1) + batch * (widest / 32) * 8 + batch * (widest / 16) * 2 + batch * (widest / 256 + 1) * 4;  // activation planes
    e.scratch += batch * (uint64_t(m.head_count) / tp) * ctx * 4;  // attention scores of one batch
    e.scratch += uint64_t(kMaxScored) * vocab * 4;                 // logits
    e.scratch += ctx * dim * 4 + (ctx + 1) * 4;                    // RoPE table, token history
    if (m.sliding_window != 0) e.scratch += ctx * dim * 4;          // the sliding layers' RoPE table
    if (m.gelu != 0 || m.final_softcap != 0.0f) e.scratch += tanh_table_bytes();  // corrections of the device's tanh
    for (uint32_t l = 0; l < m.layer_count; ++l) {
        if (m.layers[l].no_rope) {
            e.scratch += ctx * dim * 4;  // the identity table of layers without rotation
            break;
        }
    }
    if (m.layer_count != 0 && (m.layers[0].attn_post_norm || m.layers[0].ffn_post_norm)) e.scratch += batch * hidden * 4;  // projection before its norm
    if (tp > 1) e.scratch += batch * std::max<uint64_t>(widest, vocab * kMaxScored / batch + 1) * 4 * 2 + batch * std::max(q_dim, ffn) * 4;
    return e;
}

bool type_supported(int t) {
    return t == T_F32 || t == T_F16 || t == T_BF16 || t == T_Q4_0 || t == T_Q4_1 || t == T_Q5_0 || t == T_Q8_0 || t == T_Q4_K || t == T_Q5_K || t == T_Q6_K ||
           t == T_TQ2_0;
}

}  // namespace

struct Session {
    // configuration
    uint32_t vocab = 0, hidden = 0, n_layers = 0, heads = 0, kv_heads = 0, head_dim = 0, ffn = 0;
    uint32_t q_dim = 0, kv_dim = 0;
    // Tensor parallelism: every matrix is split by OUTPUT rows (whole heads for q/k/v), so each output value is still
    // one rank's sum over all of its input blocks in order - bit-identical to the unsharded result - and the ranks
    // exchange activations with all-gathers. *_l are this rank's shares.
    int tp_size = 1, tp_rank = 0;
    void* comm = nullptr;
    uint32_t heads_l = 0, kv_heads_l = 0, q_dim_l = 0, kv_dim_l = 0, ffn_l = 0, hidden_l = 0, vocab_l = 0;
    uint64_t max_context = 0;
    float eps = 0, rope_base = 0;
    // Gemma 3 (src/model.cpp:169-176, :286): scaled embeddings, tanh-GELU gate, sliding window, soft cap of the logits.
    // Such a model runs every step, single tokens too, through the batched kernels plus the few kernels of gemma.cu.
    float embedding_scale = 1.0f, final_softcap = 0.0f;
    uint32_t sliding_window = 0;
    bool gelu = false, variant_layers = false;
    uint32_t rope_dim = 0;  // values of a head that rotate (Phi's partial rotary, src/model.cpp:178, :1024); head_dim: all
    bool unrotated_layers = false;  // SmolLM3: some layers attend without RoPE (src/model.h:97-110)
    int arch = 0, neox = 1, device = 0;
    uint32_t sms = 148;
    uint32_t flags = 0;

    // weights
    std::vector<std::unique_ptr<DevBuffer>> weight_buffers;
    std::vector<Layer> layers;
    DevMatrix embd, head;
    const float* output_norm = nullptr;
    uint64_t weight_bytes = 0, kv_bytes = 0;

    // state and scratch
    DevBuffer kv, rope, rope_local, rope_none, proj_b, tanh_table, tokens_dev, scalars, hidden_b, q_b, k_b, v_b, attended_b, ffn_b, up_b, logits_b, tp_local, tp_gathered, full_b, actf, actq0, actd0, acts0, actqk,
        actdk, actbs, partial, am_val, am_idx, history, logit_history, trace, topk_keys, topk_out;
    DevActMut act;
    float* logits_host = nullptr;     // pinned [64][vocab]
    int32_t* tokens_host = nullptr;   // pinned [kMaxBatch + 4]
    int32_t* topk_host = nullptr;     // pinned [2 * kMaxTopK]: ids, then the values' bits
    uint64_t position = 0;
    cudaStream_t stream = nullptr;
    cudaEvent_t ev0 = nullptr, ev1 = nullptr;
    cudaGraphExec_t step_graph = nullptr;
    uint64_t step_graph_nodes = 0;
    // The persistent all-layer kernel of the single-token step (step.cu), when the model is within what it covers.
    StepPlan step_plan;
    bool step_enabled = false;
    // One launch per token (token.cu): embedding, layers, head and arg-max in one kernel, where the model allows it.
    TokenPlan token_plan;
    bool token_enabled = false;
    bool advance_on_device = false;  // the device greedy loop: the token kernel also feeds the next step
    std::string step_note;                 // how it was configured, or why it is not used
    // Peer-store exchange of single tokens (tp_peer.cu): this rank's buffer of tagged pairs, the peers' buffers as mapped here.
    DevBuffer peer_buf, peer_table, peer_state;  // peer_state: [0] the next tag, [1] the error word
    std::vector<void*> peer_mapped;              // what cudaIpcOpenMemHandle returned (closed with the session)
    bool peer_on = false;
    unsigned int* gemm_tc_error_dev = nullptr;
    unsigned int* chain_error_dev = nullptr;  // the few-token attention kernel's error word (a device symbol)
    unsigned int* step_error_host = nullptr;  // pinned copy of the kernel's barrier-timeout word
    uint64_t persistent_steps = 0;
    uint64_t launches = 0;  // kernels launched by the current call
    // Per-phase device time, the counterpart of the reference's Session::Profile / BRISK_GPU_PROFILE
    // (src/model.h:242-245, src/metal/metal_session.mm:711-719). Enabled by brisk_cuda_profile_enable(): every phase is
    // then bracketed by CUDA events and the single-token step runs without its graph.
    enum Phase : int { PH_EMBED, PH_QKV, PH_ATTENTION, PH_ATTN_OUT, PH_GATE_UP, PH_DOWN, PH_HEAD, PH_EXCHANGE, PH_SAMPLE, PH_COUNT };
    bool profiling = false;
    bool capturing = false;  // a stream capture is recording the step: events recorded now would never run
    double phase_ms[PH_COUNT] = {};
    uint64_t phase_calls[PH_COUNT] = {};
    std::vector<cudaEvent_t> event_pool;
    struct Span { int phase; cudaEvent_t a, b; };
    std::vector<Span> spans;
    size_t events_used = 0;
    cudaEvent_t take_event() {
        if (events_used == event_pool.size()) {
            cudaEvent_t e;
            BK_CUDA(cudaEventCreate(&e));
            event_pool.push_back(e);
        }
        return event_pool[events_used++];
    }
    struct Scope {
        Session* s;
        Span span;
        Scope(Session* session, int phase) : s(session->profiling && !session->capturing ? session : nullptr) {
            if (s) {
                span = {phase, s->take_event(), s->take_event()};
                cudaEventRecord(span.a, s->stream);
            }
        }
        ~Scope() {
            if (s) {
                cudaEventRecord(span.b, s->stream);
                s->spans.push_back(span);
            }
        }
    };
    void collect_profile() {  // after the stream is idle
        for (const Span& sp : spans) {
            float ms = 0;
            if (cudaEventElapsedTime(&ms, sp.a, sp.b) == cudaSuccess) {
                phase_ms[sp.phase] += ms;
                phase_calls[sp.phase] += 1;
            } else {
                cudaGetLastError();  // not measured; leave no stale error for the next launch check
            }
        }
        spans.clear();
        events_used = 0;
    }
    brisk_cuda_stats stats{};
    std::string error;

    // device scalars: [0] position (u32), [1] chosen token, [2] history length
    uint32_t* d_position() const { return scalars.as<uint32_t>(); }
    int32_t* d_chosen() const { return scalars.as<int32_t>() + 1; }
    uint32_t* d_history_len() const { return scalars.as<uint32_t>() + 2; }

    ~Session() {
        if (stream) cudaStreamSynchronize(stream);
        // A graph that captured collectives keeps the communicator busy: release it before the communicator.
        if (step_graph) cudaGraphExecDestroy(step_graph);
        step_graph = nullptr;
        if (comm != nullptr && Nccl::get().ok()) Nccl::get().CommDestroy(comm);
        for (void* m : peer_mapped) cudaIpcCloseMemHandle(m);
        for (cudaEvent_t e : event_pool) cudaEventDestroy(e);
        if (ev0) cudaEventDestroy(ev0);
        if (ev1) cudaEventDestroy(ev1);
        if (stream) cudaStreamDestroy(stream);
        if (logits_host) cudaFreeHost(logits_host);
        if (tokens_host) cudaFreeHost(tokens_host);
        if (topk_host) cudaFreeHost(topk_host);
        if (step_error_host) cudaFreeHost(step_error_host);
    }

    // ---- load ------------------------------------------------------------------------------------------
    // Uploads rows [row0, row0 + rows) of a full_rows x cols tensor (row0 = 0, rows = full_rows: all of it).
    DevMatrix upload_matrix(const brisk_cuda_matrix& m, const char* what, uint64_t full_rows, uint64_t cols, DevBuffer& staging, uint64_t row0 = 0,
                            uint64_t rows = 0) {
        if (rows == 0) rows = full_rows;
        if (m.data == nullptr) throw CudaError(std::string("cuda: missing tensor ") + what);
        if (!type_supported(m.type)) throw CudaError(std::string("cuda: tensor ") + what + " has an unsupported type " + std::to_string(m.type));
        if (m.rows != full_rows || m.cols != cols) throw CudaError(std::string("cuda: tensor ") + what + " has an unexpected shape");
        const uint32_t be = block_elems(m.type);
        if (cols % be != 0 || cols % 32 != 0) throw CudaError(std::string("cuda: tensor ") + what + " row length is not a multiple of its block size");
        const uint64_t row_bytes = (cols / be) * block_bytes(m.type);
        if (m.bytes != full_rows * row_bytes) throw CudaError(std::string("cuda: tensor ") + what + " has unexpected quantised data");
        const uint64_t expect = rows * row_bytes;
        const int dev_type = m.type == T_BF16 ? int(T_F32) : m.type;  // BF16 is widened on upload, like the reference's load (src/model.cpp:439-449)
        auto buf = std::make_unique<DevBuffer>();
        buf->alloc(plane_sizes(dev_type, uint32_t(rows), uint32_t(cols)).total());
        DevMatrix d;
        bind_planes(d, dev_type, uint32_t(rows), uint32_t(cols), buf->as<uint8_t>());
        if (staging.bytes < expect) {
            BK_CUDA(cudaStreamSynchronize(stream));
            if (staging.p) cudaFree(staging.p);
            staging.p = nullptr;
            staging.alloc(expect);
        }
        BK_CUDA(cudaStreamSynchronize(stream));  // the previous repack still reads the staging buffer
        BK_CUDA(cudaMemcpyAsync(staging.p, static_cast<const uint8_t*>(m.data) + row0 * row_bytes, expect, cudaMemcpyHostToDevice, stream));
        if (m.type == T_BF16) launch_widen_bf16(d, staging.as<uint8_t>(), stream);
        else launch_repack(d, staging.as<uint8_t>(), stream);
        weight_bytes += expect;
        stats.h2d_bytes += expect;
        weight_buffers.push_back(std::move(buf));
        return d;
    }

    const float* upload_vector(const float* v, uint64_t n, const char* what, bool required) {
        if (v == nullptr) {
            if (required) throw CudaError(std::string("cuda: missing tensor ") + what);
            return nullptr;
        }
        auto buf = std::make_unique<DevBuffer>();
        buf->alloc(n * sizeof(float));
        BK_CUDA(cudaMemcpyAsync(buf->p, v, n * sizeof(float), cudaMemcpyHostToDevice, stream));
        weight_bytes += n * sizeof(float);
        const float* out = buf->as<float>();
        weight_buffers.push_back(std::move(buf));
        return out;
    }

    void load(const brisk_cuda_model& m, const brisk_cuda_options& opt) {
        if (m.abi_version != BRISK_CUDA_ABI_VERSION) throw CudaError("cuda: model description has a different ABI version");
        tp_size = opt.tp_size > 1 ? opt.tp_size : 1;
        tp_rank = tp_size > 1 ? opt.tp_rank : 0;
        if (tp_rank < 0 || tp_rank >= tp_size) throw CudaError("cuda: tensor-parallel rank out of range");
        vocab = m.vocab_size; hidden = m.hidden; n_layers = m.layer_count; heads = m.head_count; kv_heads = m.kv_head_count;
        head_dim = m.head_dim; ffn = m.ffn; eps = m.rms_epsilon; rope_base = m.rope_base; arch = m.arch; neox = m.rope_neox;
        flags = opt.flags;
        if (arch != BRISK_ARCH_QWEN3 && arch != BRISK_ARCH_LLAMA && arch != BRISK_ARCH_BITNET && arch != BRISK_ARCH_GEMMA3) {
            throw CudaError("cuda: unknown architecture id in the model description");
        }
        embedding_scale = m.embedding_scale != 0.0f ? m.embedding_scale : 1.0f;
        final_softcap = m.final_softcap;
        sliding_window = m.sliding_window;
        gelu = m.gelu != 0;
        if (gelu && arch == BRISK_ARCH_BITNET) throw CudaError("cuda: the squared-ReLU gate and the GELU gate exclude each other");
        if (!vocab || !hidden || !n_layers || !heads || !kv_heads || !ffn || !m.context_length) throw CudaError("cuda: a model dimension is zero");
        if (heads % kv_heads != 0) throw CudaError("cuda: head_count is not a multiple of head_count_kv");
        if (heads / kv_heads > 8) throw CudaError("cuda: more than 8 query heads per key/value head is not supported");
        if (head_dim != 64 && head_dim != 128 && head_dim != 256) throw CudaError("cuda: head size must be 64, 128 or 256");
        rope_dim = m.rope_dim != 0 ? m.rope_dim : head_dim;
        if (rope_dim > head_dim || rope_dim % 2 != 0) throw CudaError("cuda: the rotated width must be even and at most the head size");
        if (rope_dim != head_dim && !m.rope_neox) throw CudaError("cuda: partial rotary is built for the NeoX pairing");
        if (m.rope_factor_count != 0 && m.rope_factor_count != rope_dim / 2) throw CudaError("cuda: rope factor count must be half the rotated width");
        q_dim = heads * head_dim;
        kv_dim = kv_heads * head_dim;
        max_context = opt.max_context == 0 ? m.context_length : std::min<uint64_t>(opt.max_context, m.context_length);
        const uint32_t tp = uint32_t(tp_size);
        if (kv_heads % tp != 0 || ffn % (tp * 32) != 0 || hidden % (tp * 32) != 0 || vocab % tp != 0) {
            throw CudaError("cuda: the tensor-parallel degree must divide the K/V heads, the vocabulary and (in blocks of 32) the hidden and feed-forward sizes");
        }
        heads_l = heads / tp; kv_heads_l = kv_heads / tp; q_dim_l = heads_l * head_dim; kv_dim_l = kv_heads_l * head_dim;
        ffn_l = ffn / tp; hidden_l = hidden / tp; vocab_l = vocab / tp;
        if (tp_size > 1) {
            const Nccl& nccl = Nccl::get();
            if (!nccl.ok()) throw CudaError("cuda: tensor parallelism needs NCCL (libnccl.so.2 was not found; set BRISK_NCCL_LIB)");
            if (opt.tp_unique_id == nullptr) throw CudaError("cuda: tensor parallelism needs the id from brisk_cuda_tp_unique_id");
            NcclId id;
            std::memcpy(&id, opt.tp_unique_id, sizeof(id));
            nccl.check(nccl.CommInitRank(&comm, tp_size, id, tp_rank), "ncclCommInitRank");
        }

        {
            int count = 0;
            BK_CUDA(cudaDeviceGetAttribute(&count, cudaDevAttrMultiProcessorCount, opt.device));
            sms = uint32_t(count);
        }
        if (std::getenv("BRISK_NO_MEMORY_CHECK") == nullptr) {  // refuse up front what cannot fit (src/memory.cpp:114-135)
            const brisk_cuda_memory need_bytes = estimate(m, opt);
            size_t free_bytes = 0, total_bytes = 0;
            BK_CUDA(cudaMemGetInfo(&free_bytes, &total_bytes));
            if (const char* fake = std::getenv("BRISK_CUDA_ASSUME_FREE_BYTES")) free_bytes = std::strtoull(fake, nullptr, 10);  // tests
            const uint64_t total = need_bytes.weights + need_bytes.cache + need_bytes.scratch, margin = uint64_t(256) << 20;
            if (total + margin > free_bytes) {
                const uint64_t shortfall = total + margin - free_bytes;
                std::string hint = "a smaller file or quantisation";
                if (shortfall <= need_bytes.cache * 7 / 8 + need_bytes.scratch / 2 && max_context > 512) {
                    hint = "a shorter context (this estimate is for " + std::to_string(max_context) + " tokens and the cache is " + gb(need_bytes.cache) +
                           "), or " + hint;
                }
                throw CudaError("cuda: the model needs about " + gb(total) + " of device memory (" + gb(need_bytes.weights) + " weights, " +
                                gb(need_bytes.cache) + " cache, " + gb(need_bytes.scratch) + " scratch) but " + gb(free_bytes) +
                                " is free. Try " + hint + ", or set BRISK_NO_MEMORY_CHECK=1 to proceed regardless.");
            }
        }
        BK_CUDA(cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking));
        BK_CUDA(cudaEventCreate(&ev0));
        BK_CUDA(cudaEventCreate(&ev1));

        DevBuffer staging;
        embd = upload_matrix(m.token_embd, "token_embd.weight", vocab, hidden, staging);
        const uint64_t r = uint64_t(tp_rank);
        if (tp_size == 1) head = m.output.data != nullptr ? upload_matrix(m.output, "output.weight", vocab, hidden, staging) : embd;
        else head = upload_matrix(m.output.data != nullptr ? m.output : m.token_embd, "output.weight", vocab, hidden, staging, r * vocab_l, vocab_l);
        output_norm = upload_vector(m.output_norm, hidden, "output_norm.weight", true);
        layers.resize(n_layers);
        for (uint32_t l = 0; l < n_layers; ++l) {
            const brisk_cuda_layer& s = m.layers[l];
            Layer& d = layers[l];
            d.attn_norm = upload_vector(s.attn_norm, hidden, "attn_norm.weight", true);
            d.q = upload_matrix(s.q, "attn_q.weight", q_dim, hidden, staging, r * q_dim_l, q_dim_l);
            d.k = upload_matrix(s.k, "attn_k.weight", kv_dim, hidden, staging, r * kv_dim_l, kv_dim_l);
            d.v = upload_matrix(s.v, "attn_v.weight", kv_dim, hidden, staging, r * kv_dim_l, kv_dim_l);
            d.q_norm = upload_vector(s.q_norm, head_dim, "attn_q_norm.weight", false);
            d.k_norm = upload_vector(s.k_norm, head_dim, "attn_k_norm.weight", false);
            if ((s.q_bias != nullptr) != (s.k_bias != nullptr) || (s.q_bias != nullptr) != (s.v_bias != nullptr)) {
                throw CudaError("cuda: attn_q.bias, attn_k.bias and attn_v.bias come all three or not at all");
            }
            d.q_bias = upload_vector(s.q_bias ? s.q_bias + r * q_dim_l : nullptr, q_dim_l, "attn_q.bias", false);
            d.k_bias = upload_vector(s.k_bias ? s.k_bias + r * kv_dim_l : nullptr, kv_dim_l, "attn_k.bias", false);
            d.v_bias = upload_vector(s.v_bias ? s.v_bias + r * kv_dim_l : nullptr, kv_dim_l, "attn_v.bias", false);
            d.attn_sub_norm = upload_vector(s.attn_sub_norm, q_dim, "attn_sub_norm.weight", false);
            d.o = upload_matrix(s.o, "attn_output.weight", hidden, q_dim, staging, r * hidden_l, hidden_l);
            d.ffn_norm = upload_vector(s.ffn_norm, hidden, "ffn_norm.weight", true);
            d.gate = upload_matrix(s.gate, "ffn_gate.weight", ffn, hidden, staging, r * ffn_l, ffn_l);
            d.up = upload_matrix(s.up, "ffn_up.weight", ffn, hidden, staging, r * ffn_l, ffn_l);
            if (d.gate.type != d.up.type) throw CudaError("cuda: ffn_gate and ffn_up must share one type");
            d.ffn_sub_norm = upload_vector(s.ffn_sub_norm, ffn, "ffn_sub_norm.weight", false);
            d.down = upload_matrix(s.down, "ffn_down.weight", hidden, ffn, staging, r * hidden_l, hidden_l);
            d.attn_post_norm = upload_vector(s.attn_post_norm, hidden, "post_attention_norm.weight", false);
            d.ffn_post_norm = upload_vector(s.ffn_post_norm, hidden, "post_ffw_norm.weight", false);
            d.slides = s.slides != 0 && sliding_window != 0;
            d.no_rope = s.no_rope != 0;
            if (d.no_rope) unrotated_layers = true;
            if (d.attn_post_norm || d.ffn_post_norm || d.slides) variant_layers = true;
        }
        if (gelu || embedding_scale != 1.0f || final_softcap != 0.0f) variant_layers = true;
        if (head_dim > 128) variant_layers = true;  // the fused single-token kernels take heads of 64 and 128
        if (rope_dim != head_dim) variant_layers = true;  // ... and rotate whole heads
        BK_CUDA(cudaStreamSynchronize(stream));
        if (m.output.data == nullptr) {
            // A tied head is streamed once per token as the head; the embedding lookup reads one row of it.
        }

        // K/V cache: per layer [kv head][max_context][head_dim] f16, K then V (src/model.cpp:982-991).
        const size_t per = size_t(kv_heads_l) * max_context * head_dim;
        kv_bytes = size_t(n_layers) * 2 * per * sizeof(__half);
        kv.alloc(kv_bytes);
        BK_CUDA(cudaMemsetAsync(kv.p, 0, kv_bytes, stream));
        for (uint32_t l = 0; l < n_layers; ++l) {
            layers[l].k_cache = kv.as<__half>() + size_t(l) * 2 * per;
            layers[l].v_cache = layers[l].k_cache + per;
        }

        // RoPE table for every position, built like the reference builds it per batch (src/model.cpp:880-892):
        // theta starts at the position and is multiplied by base^(-2/dim) per pair, in f32, with the host's libm.
        // `width` values of a head rotate; the angles are built for that width (src/model.cpp:880-893). Rows keep the stride
        // head_dim. cos and sin carry rope_attn_factor (:887-888).
        const float attn_factor = m.rope_attn_factor != 0.0f ? m.rope_attn_factor : 1.0f;
        auto build_rope = [&](DevBuffer& dst, float base, float scale, bool factors, uint32_t width) {
            std::vector<float> table(size_t(max_context) * head_dim);
            const float theta_scale = std::pow(base, -2.0f / static_cast<float>(width));
            for (uint64_t p = 0; p < max_context; ++p) {
                float theta = static_cast<float>(p) * scale;
                float* r = table.data() + p * head_dim;
                for (uint32_t i = 0; i < width / 2; ++i) {
                    const float angle = factors && m.rope_factor_count != 0 ? theta / m.rope_factors[i] : theta;
                    r[2 * i] = std::cos(angle) * attn_factor;
                    r[2 * i + 1] = std::sin(angle) * attn_factor;
                    theta *= theta_scale;
                }
            }
            dst.alloc(table.size() * sizeof(float));
            BK_CUDA(cudaMemcpy(dst.p, table.data(), table.size() * sizeof(float), cudaMemcpyHostToDevice));
        };
        build_rope(rope, rope_base, m.rope_scale != 0.0f ? m.rope_scale : 1.0f, true, rope_dim);
        // The sliding layers rotate with their own base, an unscaled position and no per-frequency divisors (src/model.cpp:894).
        if (sliding_window != 0) build_rope(rope_local, m.rope_base_local, 1.0f, false, head_dim);
        // A layer without rotation (the reference rotates zero pairs there, src/model.cpp:1024) runs the same kernels over
        // a table of cos = 1, sin = 0: x0 * 1 - x1 * 0 and x0 * 0 + x1 * 1 return x0 and x1 themselves.
        if (unrotated_layers) {
            std::vector<float> table(size_t(max_context) * head_dim);
            for (size_t i = 0; i < table.size(); i += 2) {
                table[i] = 1.0f;
                table[i + 1] = 0.0f;
            }
            rope_none.alloc(table.size() * sizeof(float));
            BK_CUDA(cudaMemcpy(rope_none.p, table.data(), table.size() * sizeof(float), cudaMemcpyHostToDevice));
        }

        const uint32_t widest = std::max(std::max(hidden, q_dim), ffn);
        tokens_dev.alloc((kMaxBatch + 4) * sizeof(int32_t));
        scalars.alloc(64);
        BK_CUDA(cudaMemsetAsync(scalars.p, 0, 64, stream));
        hidden_b.alloc(size_t(kMaxBatch) * hidden * 4);
        q_b.alloc(size_t(kMaxBatch) * q_dim * 4);
        k_b.alloc(size_t(kMaxBatch) * kv_dim * 4);
        v_b.alloc(size_t(kMaxBatch) * kv_dim * 4);
        attended_b.alloc(size_t(kMaxBatch) * q_dim * 4);
        ffn_b.alloc(size_t(kMaxBatch) * ffn * 4);
        up_b.alloc(size_t(kMaxBatch) * ffn * 4);
        logits_b.alloc(size_t(kMaxScored) * vocab * 4);
        if (variant_layers) proj_b.alloc(size_t(kMaxBatch) * hidden * 4);
        if (gelu || final_softcap != 0.0f) {
            // The CPU engine's GELU and soft cap call the C library's tanhf; the table makes the device return the same bits
            // (tanh_like_host, formats.cuh). BRISK_CUDA_TANH_TABLE=0 skips it: results then agree to rounding only.
            const char* env = std::getenv("BRISK_CUDA_TANH_TABLE");
            if (env == nullptr || std::strcmp(env, "0") != 0) {
                tanh_table.alloc(tanh_table_bytes());
                build_tanh_table(tanh_table.as<uint8_t>(), std::thread::hardware_concurrency(), stream);
            }
        }
        actf.alloc(size_t(kMaxBatch) * widest * 4);
        actq0.alloc(size_t(kMaxBatch) * widest);
        actd0.alloc(size_t(kMaxBatch) * (widest / 32) * 4);
        acts0.alloc(size_t(kMaxBatch) * (widest / 32) * 4);
        actqk.alloc(size_t(kMaxBatch) * widest);
        actdk.alloc(size_t(kMaxBatch) * (widest / 256 + 1) * 4);
        actbs.alloc(size_t(kMaxBatch) * (widest / 16) * 2);
        act.f32 = actf.as<float>(); act.q0 = actq0.as<int8_t>(); act.d0 = actd0.as<float>(); act.s0 = acts0.as<int32_t>();
        act.qk = actqk.as<int8_t>(); act.dk = actdk.as<float>(); act.bs = actbs.as<int16_t>();
        partial.alloc(attn_scratch_floats(kMaxBatch, heads_l, uint32_t(max_context)) * 4);
        if (tp_size > 1) {
            const size_t widest_rows = std::max<size_t>(std::max<size_t>(q_dim, ffn), std::max<size_t>(hidden, size_t(vocab) * kMaxScored / kMaxBatch + 1));
            tp_local.alloc(size_t(kMaxBatch) * widest_rows / tp * 4 + 256);
            tp_gathered.alloc(size_t(kMaxBatch) * widest_rows * 4 + 256);
            full_b.alloc(size_t(kMaxBatch) * std::max(q_dim, ffn) * 4);
        }
        am_val.alloc(argmax_scratch_elems(vocab) * 4);
        am_idx.alloc(argmax_scratch_elems(vocab) * 4);
        history.alloc((max_context + 1) * sizeof(int32_t));
        topk_keys.alloc(topk_scratch_keys(vocab, kMaxTopK) * sizeof(unsigned long long));
        topk_out.alloc(2 * kMaxTopK * sizeof(int32_t));
        if (std::getenv("BRISK_CUDA_TRACE") != nullptr) {  // per-kernel phase time stamps of the decode multiplies
            trace.alloc(512 * 8 * sizeof(unsigned long long));
            BK_CUDA(cudaMemsetAsync(trace.p, 0, trace.bytes, stream));
        }
        BK_CUDA(cudaMallocHost(&logits_host, size_t(kMaxScored) * vocab * sizeof(float)));
        BK_CUDA(cudaMallocHost(&tokens_host, (kMaxBatch + 4) * sizeof(int32_t)));
        BK_CUDA(cudaMallocHost(&topk_host, 2 * kMaxTopK * sizeof(int32_t)));
        BK_CUDA(cudaMallocHost(&step_error_host, 4 * sizeof(unsigned int)));  // [0] the persistent kernel's word, [1] the peer exchange's, [2] the few-token attention's
        step_error_host[0] = step_error_host[1] = step_error_host[2] = step_error_host[3] = 0;  // [3]: the tcgen05 prompt multiply's
        chain_error_dev = attn_chain_error_word();
        gemm_tc_error_dev = gemm_tc_error_word();
        BK_CUDA(cudaStreamSynchronize(stream));
        plan_step();
        stats.weight_bytes = weight_bytes;
        stats.kv_bytes = kv_bytes;
    }

    void plan_step() {
        const char* env = std::getenv("BRISK_CUDA_STEP");
        if (tp_size > 1) step_note = "off: tensor parallel steps exchange activations between the operations";
        else if (unrotated_layers) step_note = "off: layers without RoPE take the per-operation kernels (the persistent kernel rotates every layer with one table)";
        else if (variant_layers) step_note = "off: Gemma layer variants (post-norms, GELU, sliding window), 256-wide heads and partial rotary run through the batched kernels";
        else if (flags & (BRISK_CUDA_FLAG_NO_MEGAKERNEL | BRISK_CUDA_FLAG_NO_PERSISTENT)) step_note = "off: disabled by the session's flags";
        else if (env != nullptr && std::strcmp(env, "0") == 0) step_note = "off: BRISK_CUDA_STEP=0";
        else if (trace.p != nullptr) step_note = "off: tracing the per-operation kernels";
        if (!step_note.empty()) return;
        std::vector<StepLayerArgs> args(n_layers);
        for (uint32_t l = 0; l < n_layers; ++l) {
            const Layer& L = layers[l];
            StepLayerArgs& a = args[l];
            a.q = L.q; a.k = L.k; a.v = L.v; a.o = L.o; a.gate = L.gate; a.up = L.up; a.down = L.down;
            a.attn_norm = L.attn_norm; a.q_norm = L.q_norm; a.k_norm = L.k_norm; a.attn_sub_norm = L.attn_sub_norm;
            a.ffn_norm = L.ffn_norm; a.ffn_sub_norm = L.ffn_sub_norm; a.k_cache = L.k_cache; a.v_cache = L.v_cache;
            a.q_bias = L.q_bias; a.k_bias = L.k_bias; a.v_bias = L.v_bias;
        }
        StepShared sh;
        sh.hidden = hidden_b.as<float>(); sh.q = q_b.as<float>(); sh.k = k_b.as<float>(); sh.v = v_b.as<float>();
        sh.attended = attended_b.as<float>(); sh.gated = ffn_b.as<float>(); sh.scores = partial.as<float>();
        sh.rope = rope.as<float>(); sh.position = d_position();
        sh.hidden_size = hidden; sh.ffn_size = ffn; sh.heads = heads; sh.kv_heads = kv_heads; sh.dim = head_dim;
        sh.max_context = uint32_t(max_context);
        sh.eps = eps; sh.scale = 1.0f / std::sqrt(static_cast<float>(head_dim)); sh.neox = neox;
        sh.act_epi = arch == BRISK_ARCH_BITNET ? EPI_RELU2_MUL : EPI_SILU_MUL;
        const bool tracing = std::getenv("BRISK_CUDA_STEP_TRACE") != nullptr;
        if (tracing) {  // per-phase stamps of every layer, then the stamps inside one layer's multiplies
            trace.alloc((size_t(n_layers) * 6 * 4 + 704) * sizeof(unsigned long long));  // also four sections of 2 + 6 per layer (the one-launch kernel)
            BK_CUDA(cudaMemset(trace.p, 0, trace.bytes));
            sh.body_trace = trace.as<unsigned long long>() + size_t(n_layers) * 6 * 4;
        }
        std::string why;
        // The one-launch token kernel (token.cu) is opt-in, BRISK_CUDA_TOKEN=1: bit-identical to the other paths, but on the
        // 0.6B-shaped model it measures ~840 us per token against ~745 us for the persistent kernel plus head and arg-max.
        const char* tok_env = std::getenv("BRISK_CUDA_TOKEN");
        if (tok_env != nullptr && std::strcmp(tok_env, "1") == 0) {
            TokenEnds ends;
            ends.embd = embd; ends.head = head; ends.output_norm = output_norm; ends.logits = logits_b.as<float>(); ends.vocab = vocab;
            ends.token = tokens_dev.as<int32_t>(); ends.chosen = d_chosen(); ends.history = history.as<int32_t>(); ends.history_len = d_history_len();
            token_enabled = token_plan.build(args, sh, ends, sms, stream, why);
            if (token_enabled) {
                step_note = "on: " + token_plan.description();
                if (tracing) token_plan.set_trace(trace.as<unsigned long long>());
                return;
            }
        }
        const std::string token_why = why;
        step_enabled = step_plan.build(args, sh, sms, stream, why);
        step_note = step_enabled ? "on: " + step_plan.description() : "off: " + why;
        if (!token_why.empty()) step_note += " (one launch per token: " + token_why + ")";
        if (step_enabled && tracing) step_plan.set_trace(trace.as<unsigned long long>());
    }

    // ---- forward ---------------------------------------------------------------------------------------
    struct Needs { bool q0 = false, qk = false, f32 = false; };
    static void need(Needs& n, int type) {
        if (type == T_F16 || type == T_F32) n.f32 = true;
        else if (takes_q8_k(type)) n.qk = true;
        else n.q0 = true;
    }

    // RMS norm (weight may be null: no norm) then the quantisations the consuming matrices take.
    DevAct prepare(const float* x, uint32_t ldx, const float* weight, uint32_t n, uint32_t cols, const Needs& nd) {
        DevActMut a = act;
        a.cols = cols;
        if (!nd.f32) a.f32 = nullptr;
        launch_norm_quant(x, ldx, weight, eps, n, cols, a, nd.q0, nd.qk, stream);
        ++launches;
        a.f32 = act.f32;
        return a.view();
    }

    // One multiply of the batched path: targets of one weight type share a launch of the streaming kernel; prompt
    // batches go to the tensor-core kernel where the type has one.
    void multiply(std::vector<MatTarget> targets, const DevAct& a, uint32_t n, Epilogue epi) {
        const bool pair = epi == EPI_SILU_MUL || epi == EPI_RELU2_MUL;
        if (pair) {
            if (small_batch_on() && launch_smallbatch(targets.data(), int(targets.size()), a, n, epi, stream)) {  // 2..16 tokens
                ++launches;
                return;
            }
            if (n >= 16 && gemm_supports(targets[0].m.type, targets[0].m.cols)) {
                // prompt batches: gate and up as two tensor-core multiplies, then the activation elementwise
                MatTarget gate{targets[0].m, targets[0].out, targets[0].ldo}, up{targets[1].m, up_b.as<float>(), targets[0].ldo};
                launch_gemm(&gate, 1, a, n, EPI_STORE, stream);
                launch_gemm(&up, 1, a, n, EPI_STORE, stream);
                launch_gate_mul(targets[0].out, up_b.as<float>(), size_t(n) * targets[0].ldo, epi == EPI_RELU2_MUL, stream);
                launches += 3;
                return;
            }
            launch_matvec(targets.data(), int(targets.size()), a, n, epi, stream);
            launches += (n + kMaxSmallBatch - 1) / kMaxSmallBatch;
            return;
        }
        while (!targets.empty()) {
            std::vector<MatTarget> same, rest;
            for (const MatTarget& t : targets) (t.m.type == targets[0].m.type ? same : rest).push_back(t);
            if (small_batch_on() && launch_smallbatch(same.data(), int(same.size()), a, n, epi, stream)) {  // 2..16 tokens
                ++launches;
            } else if (!(n >= 16 && launch_gemm(same.data(), int(same.size()), a, n, epi, stream))) {
                launch_matvec(same.data(), int(same.size()), a, n, epi, stream);
                launches += (n + kMaxSmallBatch - 1) / kMaxSmallBatch;
            } else {
                launches += same.size();
            }
            targets.swap(rest);
        }
    }

    // Tensor parallel: this rank's [n][rows_l] slice -> every rank's [n][rows_l * tp] (store or add), by an all-gather
    // into [rank][n][rows_l] and a re-layout kernel. No-op for a single GPU (kernels then write dst directly).
    void exchange(const float* local, float* dst, uint32_t n, uint32_t rows_l, bool add) {
        Scope sc(this, PH_EXCHANGE);
        const Nccl& nccl = Nccl::get();
        if (n == 1 && peer_fits(rows_l)) {  // one token, peers mapped: stores into every rank's buffer, no collective
            peer_exchange(local, dst, rows_l, add);
            return;
        }
        if (n == 1 && !add) {  // one token: the gathered order [rank][rows_l] IS the row order - no re-layout kernel
            nccl.check(nccl.AllGather(local, dst, rows_l, kNcclFloat, comm, stream), "ncclAllGather");
            ++launches;
            return;
        }
        nccl.check(nccl.AllGather(local, tp_gathered.p, size_t(n) * rows_l, kNcclFloat, comm, stream), "ncclAllGather");
        launch_tp_unpack(tp_gathered.as<float>(), dst, n, rows_l, uint32_t(tp_size), add, stream);
        launches += 2;
    }

    // One token, a projection that joins the residual stream: every rank has added its rows into its own slice of the (everywhere
    // identical) stream; the slices are gathered in place.
    void gather_in_place(float* full, uint32_t rows_l) {
        Scope sc(this, PH_EXCHANGE);
        if (peer_fits(rows_l)) {
            peer_exchange(full + size_t(tp_rank) * rows_l, full, rows_l, false);
            return;
        }
        const Nccl& nccl = Nccl::get();
        nccl.check(nccl.AllGather(full + size_t(tp_rank) * rows_l, full, rows_l, kNcclFloat, comm, stream), "ncclAllGather");
        ++launches;
    }

    bool peer_fits(uint32_t rows_l) const { return peer_on && size_t(rows_l) * size_t(tp_size) <= kPeerSlotPairs; }
    void peer_exchange(const float* local, float* dst, uint32_t rows_l, bool add) {
        launch_tp_peer_exchange(peer_table.as<uint2*>(), peer_state.as<uint32_t>(), peer_state.as<unsigned int>() + 1, uint32_t(tp_size), uint32_t(tp_rank),
                                kPeerSlotPairs, local, dst, rows_l, add, stream);
        ++launches;
    }
    // The 64 bytes a peer needs to map this rank's exchange buffer (allocated on the first call).
    void peer_handle(void* out64) {
        if (tp_size <= 1) throw CudaError("cuda: peer exchange buffers belong to tensor-parallel sessions");
        if (tp_size > 8) throw CudaError("cuda: the peer exchange takes up to 8 ranks");
        if (peer_buf.p == nullptr) {
            peer_buf.alloc(size_t(2) * kPeerSlotPairs * sizeof(uint2));
            BK_CUDA(cudaMemset(peer_buf.p, 0, peer_buf.bytes));  // tag 0 is never used
            peer_state.alloc(2 * sizeof(uint32_t));
            const uint32_t init[2] = {1, 0};
            BK_CUDA(cudaMemcpy(peer_state.p, init, sizeof init, cudaMemcpyHostToDevice));
        }
        cudaIpcMemHandle_t h;
        BK_CUDA(cudaIpcGetMemHandle(&h, peer_buf.p));
        static_assert(sizeof(h) == 64, "the ABI hands 64 bytes around");
        std::memcpy(out64, &h, sizeof h);
    }
    // handles: tp_size x 64 bytes in rank order (this rank's own entry is ignored). Every rank must have called
    // peer_handle() before any rank attaches, and all ranks attach before the next single-token step.
    void peer_attach(const void* handles) {
        if (peer_buf.p == nullptr) throw CudaError("cuda: brisk_cuda_tp_peer_handle first");
        std::vector<uint2*> table(size_t(tp_size), nullptr);
        for (int r = 0; r < tp_size; ++r) {
            if (r == tp_rank) {
                table[size_t(r)] = peer_buf.as<uint2>();
                continue;
            }
            cudaIpcMemHandle_t h;
            std::memcpy(&h, static_cast<const unsigned char*>(handles) + size_t(r) * sizeof h, sizeof h);
            void* mapped = nullptr;
            BK_CUDA(cudaIpcOpenMemHandle(&mapped, h, cudaIpcMemLazyEnablePeerAccess));
            peer_mapped.push_back(mapped);
            table[size_t(r)] = static_cast<uint2*>(mapped);
        }
        peer_table.alloc(table.size() * sizeof(uint2*));
        BK_CUDA(cudaMemcpy(peer_table.p, table.data(), table.size() * sizeof(uint2*), cudaMemcpyHostToDevice));
        if (step_graph) {  // a captured step holds all-gathers: capture again with the peer exchange
            cudaGraphExecDestroy(step_graph);
            step_graph = nullptr;
        }
        peer_on = true;
    }

    // The layers of one batch. n tokens are in tokens_dev, their first position in d_position(); max_visible bounds
    // position + n. single = true takes the fused single-token kernels (n == 1).
    void run_layers(uint32_t n, bool all_logits, uint32_t max_visible, bool single) {
        float* hid = hidden_b.as<float>();
        if (variant_layers) single = false;
        {
            Scope sc(this, PH_EMBED);
            launch_embed(embd, tokens_dev.as<int32_t>(), n, hid, stream);
            if (embedding_scale != 1.0f) {  // src/model.cpp:899-901
                launch_scale_rows(hid, size_t(n) * hidden, embedding_scale, stream);
                ++launches;
            }
        }
        ++launches;
        const float attn_scale = 1.0f / std::sqrt(static_cast<float>(head_dim));
        const bool tp = tp_size > 1;
        unsigned long long* tr = trace.p ? trace.as<unsigned long long>() : nullptr;
        uint32_t slot = 0;

        // out = W x (optionally RMS-normed, then quantised) for one group of targets sharing the input.
        auto apply = [&](std::vector<MatTarget> targets, const float* x, uint32_t ldx, const float* w, uint32_t cols, Epilogue epi, uint32_t count = 0) {
            if (count == 0) count = n;
            if (single) {
                unsigned long long* t = tr ? tr + 8 * (slot++ % 512) : nullptr;
                if (epi == EPI_SILU_MUL || epi == EPI_RELU2_MUL) {
                    launch_dec_multiply(targets.data(), int(targets.size()), x, w, eps, cols, epi, sms, stream, t);
                    ++launches;
                    return;
                }
                while (!targets.empty()) {  // one launch per weight type among the targets
                    std::vector<MatTarget> same, rest;
                    for (const MatTarget& tg : targets) (tg.m.type == targets[0].m.type ? same : rest).push_back(tg);
                    launch_dec_multiply(same.data(), int(same.size()), x, w, eps, cols, epi, sms, stream, t);
                    ++launches;
                    targets.swap(rest);
                }
                return;
            }
            Needs nd;
            for (const MatTarget& tg : targets) need(nd, tg.m.type);
            const DevAct a = prepare(x, ldx, w, count, cols, nd);
            multiply(std::move(targets), a, count, epi);
        };

        for (uint32_t l = 0; l < n_layers; ++l) {
            const Layer& L = layers[l];
            {
                Scope sc(this, PH_QKV);
                apply({{L.q, q_b.as<float>(), q_dim_l}, {L.k, k_b.as<float>(), kv_dim_l}, {L.v, v_b.as<float>(), kv_dim_l}}, hid, hidden, L.attn_norm,
                      hidden, EPI_STORE);
            }

            RopeArgs r{};
            r.q = q_b.as<float>(); r.k = k_b.as<float>(); r.v = v_b.as<float>();
            r.q_norm = L.q_norm; r.k_norm = L.k_norm; r.rope = L.no_rope ? rope_none.as<float>() : L.slides ? rope_local.as<float>() : rope.as<float>();
            r.q_bias = L.q_bias; r.k_bias = L.k_bias; r.v_bias = L.v_bias;
            r.k_cache = L.k_cache; r.v_cache = L.v_cache; r.position = d_position();
            r.n = n; r.heads = heads_l; r.kv_heads = kv_heads_l; r.dim = head_dim; r.max_context = uint32_t(max_context);
            r.eps = eps; r.neox = neox;
            r.rope_dim = (L.slides || L.no_rope) ? 0 : rope_dim;  // those tables span the whole head
            AttnArgs at{};
            at.q = q_b.as<float>(); at.k_cache = L.k_cache; at.v_cache = L.v_cache; at.out = attended_b.as<float>();
            at.scores = partial.as<float>(); at.position = d_position();
            at.n = n; at.heads = heads_l; at.kv_heads = kv_heads_l; at.dim = head_dim; at.max_context = uint32_t(max_context);
            at.max_visible = max_visible; at.scale = attn_scale; at.window = L.slides ? sliding_window : 0;
            {
                Scope sc(this, PH_ATTENTION);
                if (single) {
                    launch_dec_attention(r, at, sms, stream);
                    launches += 2;
                } else {
                    launch_qk_norm_rope_store(r, stream);
                    launch_attention(at, stream);
                    launches += 4;
                }
            }

            // attention output projection + residual
            // A projection's output joins the residual stream directly, or (Gemma) after an RMS norm of its own
            // (src/model.cpp:1116-1119, :1155-1158): then it is stored whole first.
            auto post_norm_add = [&](const float* weight) {
                launch_post_norm_add(proj_b.as<float>(), weight, hid, n, hidden, eps, stream);
                ++launches;
            };
            const float* attended = attended_b.as<float>();
            if (tp) {
                exchange(attended_b.as<float>(), full_b.as<float>(), n, q_dim_l, false);
                attended = full_b.as<float>();
                if (n == 1 && L.attn_post_norm == nullptr) {
                    {
                        Scope sc(this, PH_ATTN_OUT);
                        apply({{L.o, hid + size_t(tp_rank) * hidden_l, hidden_l}}, attended, q_dim, L.attn_sub_norm, q_dim, EPI_ADD);
                    }
                    gather_in_place(hid, hidden_l);
                } else {
                    {
                        Scope sc(this, PH_ATTN_OUT);
                        apply({{L.o, tp_local.as<float>(), hidden_l}}, attended, q_dim, L.attn_sub_norm, q_dim, EPI_STORE);
                    }
                    exchange(tp_local.as<float>(), L.attn_post_norm ? proj_b.as<float>() : hid, n, hidden_l, L.attn_post_norm == nullptr);
                    if (L.attn_post_norm) post_norm_add(L.attn_post_norm);
                }
            } else {
                Scope sc(this, PH_ATTN_OUT);
                if (L.attn_post_norm) {
                    apply({{L.o, proj_b.as<float>(), hidden}}, attended, q_dim, L.attn_sub_norm, q_dim, EPI_STORE);
                    post_norm_add(L.attn_post_norm);
                } else {
                    apply({{L.o, hid, hidden}}, attended, q_dim, L.attn_sub_norm, q_dim, EPI_ADD);
                }
            }

            // feed-forward + residual
            const Epilogue act_epi = arch == BRISK_ARCH_BITNET ? EPI_RELU2_MUL : EPI_SILU_MUL;
            const float* gated = ffn_b.as<float>();
            // gate and up into `dst` (row length ld): fused with the activation, or (GELU) two plain multiplies and an
            // elementwise kernel (gelu_mul_f32, src/kernels_f32.cpp:291-296).
            auto gate_up = [&](float* dst, uint32_t ld) {
                Scope sc(this, PH_GATE_UP);
                if (gelu) {
                    apply({{L.gate, dst, ld}, {L.up, up_b.as<float>(), ld}}, hid, hidden, L.ffn_norm, hidden, EPI_STORE);
                    launch_gate_mul(dst, up_b.as<float>(), size_t(n) * ld, 2, stream, tanh_table.as<uint8_t>());
                    ++launches;
                } else {
                    apply({{L.gate, dst, ld}, {L.up, nullptr, ld}}, hid, hidden, L.ffn_norm, hidden, act_epi);
                }
            };
            if (tp) {
                gate_up(tp_local.as<float>(), ffn_l);
                exchange(tp_local.as<float>(), ffn_b.as<float>(), n, ffn_l, false);
                if (n == 1 && L.ffn_post_norm == nullptr) {
                    {
                        Scope sc(this, PH_DOWN);
                        apply({{L.down, hid + size_t(tp_rank) * hidden_l, hidden_l}}, gated, ffn, L.ffn_sub_norm, ffn, EPI_ADD);
                    }
                    gather_in_place(hid, hidden_l);
                } else {
                    {
                        Scope sc(this, PH_DOWN);
                        apply({{L.down, tp_local.as<float>(), hidden_l}}, gated, ffn, L.ffn_sub_norm, ffn, EPI_STORE);
                    }
                    exchange(tp_local.as<float>(), L.ffn_post_norm ? proj_b.as<float>() : hid, n, hidden_l, L.ffn_post_norm == nullptr);
                    if (L.ffn_post_norm) post_norm_add(L.ffn_post_norm);
                }
            } else {
                gate_up(ffn_b.as<float>(), ffn);
                Scope sc(this, PH_DOWN);
                if (L.ffn_post_norm) {
                    apply({{L.down, proj_b.as<float>(), hidden}}, gated, ffn, L.ffn_sub_norm, ffn, EPI_STORE);
                    post_norm_add(L.ffn_post_norm);
                } else {
                    apply({{L.down, hid, hidden}}, gated, ffn, L.ffn_sub_norm, ffn, EPI_ADD);
                }
            }
        }
        const uint32_t rows = all_logits ? n : 1;
        const float* last = all_logits ? hid : hid + size_t(n - 1) * hidden;
        if (tp) {
            {
                Scope sc(this, PH_HEAD);
                apply({{head, tp_local.as<float>(), vocab_l}}, last, hidden, output_norm, hidden, EPI_STORE, rows);
            }
            exchange(tp_local.as<float>(), logits_b.as<float>(), rows, vocab_l, false);
        } else {
            Scope sc(this, PH_HEAD);
            apply({{head, logits_b.as<float>(), vocab}}, last, hidden, output_norm, hidden, EPI_STORE, rows);
        }
        if (final_softcap != 0.0f) {  // src/model.cpp:1206-1209
            launch_softcap(logits_b.as<float>(), size_t(rows) * vocab, final_softcap, tanh_table.as<uint8_t>(), stream);
            ++launches;
        }
    }

    void forward(uint32_t n, bool all_logits, uint32_t max_visible) { run_layers(n, all_logits, max_visible, false); }
    bool step_active() const { return (step_enabled || token_enabled) && !profiling; }
    bool token_active() const { return token_enabled && !profiling; }
    void forward_decode() {
        if (!step_active()) {
            run_layers(1, false, uint32_t(max_context), true);
            return;
        }
        if (token_enabled) {
            if (!token_plan.embeds_itself()) {
                launch_embed(embd, tokens_dev.as<int32_t>(), 1, hidden_b.as<float>(), stream);
                ++launches;
            }
            token_plan.launch(stream, advance_on_device);
            ++launches;
            ++persistent_steps;
            return;
        }
        // embedding | all layers in one persistent kernel | output head
        launch_embed(embd, tokens_dev.as<int32_t>(), 1, hidden_b.as<float>(), stream);
        step_plan.launch(stream);
        MatTarget target{head, logits_b.as<float>(), vocab};
        launch_dec_multiply(&target, 1, hidden_b.as<float>(), output_norm, eps, hidden, EPI_STORE, sms, stream, nullptr);
        launches += 3;
        ++persistent_steps;
    }
    // After the call's final synchronisation: did a barrier wait of the persistent kernel run out?
    // BRISK_CUDA_SMALLBATCH=0 keeps the streaming kernel for 2..16 tokens (a comparison aid); read at every call
    static bool small_batch_on() {
        const char* env = std::getenv("BRISK_CUDA_SMALLBATCH");
        return env == nullptr || std::atoi(env) != 0;
    }
    void queue_step_check() {
        // the few-token attention kernel waits for bulk copies (every wait bounded): its error word, read with the call's results
        BK_CUDA(cudaMemcpyAsync(step_error_host + 2, chain_error_dev, sizeof(unsigned int), cudaMemcpyDeviceToHost, stream));
        BK_CUDA(cudaMemcpyAsync(step_error_host + 3, gemm_tc_error_dev, sizeof(unsigned int), cudaMemcpyDeviceToHost, stream));
        if (peer_on) BK_CUDA(cudaMemcpyAsync(step_error_host + 1, peer_state.as<unsigned int>() + 1, sizeof(unsigned int), cudaMemcpyDeviceToHost, stream));
        if (token_enabled) BK_CUDA(cudaMemcpyAsync(step_error_host, token_plan.error_word(), sizeof(unsigned int), cudaMemcpyDeviceToHost, stream));
        else if (step_enabled) BK_CUDA(cudaMemcpyAsync(step_error_host, step_plan.error_word(), sizeof(unsigned int), cudaMemcpyDeviceToHost, stream));
    }
    void finish_step_check() {
        if (step_error_host[3] != 0) {
            step_error_host[3] = 0;
            BK_CUDA(cudaMemsetAsync(gemm_tc_error_dev, 0, sizeof(unsigned int), stream));
            throw CudaError("cuda: a wait inside the tcgen05 prompt multiply ran out; the results of this call are invalid");
        }
        if (step_error_host[1] != 0) {
            step_error_host[1] = 0;
            BK_CUDA(cudaMemsetAsync(peer_state.as<unsigned int>() + 1, 0, sizeof(unsigned int), stream));
            throw CudaError("cuda: a tensor-parallel peer did not deliver its share of an exchange in time; the results of this call are invalid");
        }
        if (step_error_host[2] != 0) {
            step_error_host[2] = 0;
            BK_CUDA(cudaMemsetAsync(chain_error_dev, 0, sizeof(unsigned int), stream));
            throw CudaError("cuda: a bulk copy of the few-token attention kernel did not complete in time; the results of this call are invalid");
        }
        if ((step_enabled || token_enabled) && *step_error_host != 0) {
            *step_error_host = 0;
            if (token_enabled) token_plan.rearm(stream);
            else step_plan.rearm(stream);
            step_enabled = token_enabled = false;  // later steps take the per-operation kernels
            step_note = "off: a grid barrier timed out";
            throw CudaError("cuda: a grid barrier of the single-token kernel timed out; the results of this call are invalid");
        }
    }

    // Three launches per token gain little from a graph; BRISK_CUDA_STEP_GRAPH=1 captures them all the same - unless the
    // kernel exchanges tagged pairs: its tags are a launch parameter that must change with every token, and a replayed
    // graph would launch with the tags of the token it was captured for.
    bool step_in_graph() const {
        static const bool on = [] {
            const char* env = std::getenv("BRISK_CUDA_STEP_GRAPH");
            return env != nullptr && std::atoi(env) != 0;
        }();
        return on && !token_enabled && step_plan.graph_safe();
    }

    void build_step_graph() {
        if (step_graph != nullptr || (flags & BRISK_CUDA_FLAG_NO_GRAPH) || (step_active() && !step_in_graph())) return;
        const uint64_t before = launches;
        cudaGraph_t graph = nullptr;
        BK_CUDA(cudaStreamBeginCapture(stream, cudaStreamCaptureModeThreadLocal));
        capturing = true;
        try {
            forward_decode();
        } catch (...) {
            capturing = false;
            cudaStreamEndCapture(stream, &graph);
            if (graph) cudaGraphDestroy(graph);
            throw;
        }
        capturing = false;
        BK_CUDA(cudaStreamEndCapture(stream, &graph));
        step_graph_nodes = launches - before;
        launches = before;
        const cudaError_t e = cudaGraphInstantiate(&step_graph, graph, 0);
        cudaGraphDestroy(graph);
        BK_CUDA(e);
    }

    void step_on_device() {  // one token whose id is tokens_dev[0] at *d_position()
        // The fused weighted sum keeps a head's probabilities of the whole context in shared memory; past that the batched
        // kernels, which have no such limit, take single tokens too.
        const bool too_long = !step_active() && !variant_layers &&
                              !dec_attention_fits(uint32_t(max_context), heads_l, head_dim, sms);
        if ((flags & BRISK_CUDA_FLAG_NO_MEGAKERNEL) || too_long) {
            forward(1, false, uint32_t(max_context));  // the batched kernels, one token
        } else if ((flags & BRISK_CUDA_FLAG_NO_GRAPH) || profiling || (step_active() && !step_in_graph())) {
            forward_decode();
        } else {
            build_step_graph();
            BK_CUDA(cudaGraphLaunch(step_graph, stream));
            launches += step_graph_nodes;
        }
    }

    void begin_call() {
        launches = 0;
        persistent_steps = 0;
        stats.h2d_bytes = stats.d2h_bytes = 0;
    }
    void end_call(float ms) {
        if (profiling) collect_profile();
        stats.device_ms = ms;
        stats.kernel_launches = launches;
        stats.persistent_steps = persistent_steps;
    }

    void check_tokens(const int32_t* tokens, uint64_t n, bool all) {
        if (all ? (n == 0 || n > kMaxScored) : n == 0) throw CudaError(all ? "cuda: eval_all takes 1 to 64 tokens" : "cuda: no tokens to evaluate");
        for (uint64_t i = 0; i < n; ++i) {
            if (tokens[i] < 0 || uint32_t(tokens[i]) >= vocab) throw CudaError("cuda: token id out of range");
        }
        if (n > max_context - position) throw CudaError("cuda: context length exceeded");
    }

    // topk > 0: instead of the last row of logits, its `topk` best (id, value) pairs go to the host (topk_host).
    const float* eval(const int32_t* tokens, uint64_t n, bool all, uint32_t topk = 0) {
        check_tokens(tokens, n, all);
        if (topk > kMaxTopK || topk > vocab) throw CudaError("cuda: top-k takes k from 1 to " + std::to_string(std::min<uint32_t>(kMaxTopK, vocab)));
        begin_call();
        BK_CUDA(cudaEventRecord(ev0, stream));
        for (uint64_t begin = 0; begin < n; begin += kMaxBatch) {
            const uint32_t cnt = uint32_t(std::min<uint64_t>(kMaxBatch, n - begin));
            BK_CUDA(cudaStreamSynchronize(stream));  // tokens_host is reused
            std::memcpy(tokens_host, tokens + begin, cnt * sizeof(int32_t));
            const uint32_t pos32 = uint32_t(position);
            std::memcpy(tokens_host + kMaxBatch, &pos32, sizeof(pos32));
            BK_CUDA(cudaMemcpyAsync(tokens_dev.p, tokens_host, cnt * sizeof(int32_t), cudaMemcpyHostToDevice, stream));
            BK_CUDA(cudaMemcpyAsync(d_position(), tokens_host + kMaxBatch, sizeof(uint32_t), cudaMemcpyHostToDevice, stream));
            stats.h2d_bytes += cnt * sizeof(int32_t) + sizeof(uint32_t);
            const bool last = begin + cnt == n;
            if (cnt == 1 && (!all || n == 1)) step_on_device();  // one token: its one row of logits is all there is, with or without `all`
            else forward(cnt, all, uint32_t(position + cnt));
            (void)last;
            position += cnt;
        }
        if (topk != 0) {
            launch_topk(logits_b.as<float>(), vocab, topk, topk_keys.as<unsigned long long>(), topk_out.as<int32_t>(),
                        reinterpret_cast<float*>(topk_out.as<int32_t>() + kMaxTopK), stream, &launches);
            BK_CUDA(cudaMemcpyAsync(topk_host, topk_out.p, 2 * kMaxTopK * sizeof(int32_t), cudaMemcpyDeviceToHost, stream));
            stats.d2h_bytes += 2 * size_t(topk) * sizeof(int32_t);
        } else {
            const size_t out_bytes = size_t(all ? n : 1) * vocab * sizeof(float);
            BK_CUDA(cudaMemcpyAsync(logits_host, logits_b.p, out_bytes, cudaMemcpyDeviceToHost, stream));
            stats.d2h_bytes += out_bytes;
        }
        BK_CUDA(cudaEventRecord(ev1, stream));
        queue_step_check();
        BK_CUDA(cudaStreamSynchronize(stream));
        float ms = 0;
        BK_CUDA(cudaEventElapsedTime(&ms, ev0, ev1));
        end_call(ms);
        try {
            finish_step_check();
        } catch (...) {
            position -= n;  // nothing of this call can be trusted: the cache rows it wrote are overwritten by the next call
            throw;
        }
        return logits_host;
    }

    void generate_greedy(int32_t first, uint64_t steps, int32_t* out_tokens, float* out_logits) {
        if (steps == 0) return;
        check_tokens(&first, 1, false);
        if (steps > max_context - position) throw CudaError("cuda: context length exceeded");
        begin_call();
        if (out_logits != nullptr && logit_history.bytes < steps * vocab * sizeof(float)) {
            if (logit_history.p) cudaFree(logit_history.p);
            logit_history.p = nullptr;
            logit_history.alloc(steps * vocab * sizeof(float));
        }
        const uint32_t pos32 = uint32_t(position);
        tokens_host[0] = first;
        std::memcpy(tokens_host + kMaxBatch, &pos32, sizeof(pos32));
        tokens_host[kMaxBatch + 1] = 0;
        tokens_host[kMaxBatch + 2] = 0;
        BK_CUDA(cudaMemcpyAsync(tokens_dev.p, tokens_host, sizeof(int32_t), cudaMemcpyHostToDevice, stream));
        BK_CUDA(cudaMemcpyAsync(scalars.p, tokens_host + kMaxBatch, 3 * sizeof(uint32_t), cudaMemcpyHostToDevice, stream));
        stats.h2d_bytes += 4 * sizeof(int32_t);
        build_step_graph();
        BK_CUDA(cudaEventRecord(ev0, stream));
        const bool fused_pick = token_active() && !(flags & BRISK_CUDA_FLAG_NO_MEGAKERNEL);
        for (uint64_t i = 0; i < steps; ++i) {
            advance_on_device = fused_pick;
            step_on_device();
            advance_on_device = false;
            if (out_logits != nullptr) {
                BK_CUDA(cudaMemcpyAsync(logit_history.as<float>() + i * vocab, logits_b.p, size_t(vocab) * sizeof(float), cudaMemcpyDeviceToDevice, stream));
            }
            if (!fused_pick) {
                Scope sc(this, PH_SAMPLE);
                launch_argmax_advance(logits_b.as<float>(), vocab, d_chosen(), am_val.as<float>(), am_idx.as<int32_t>(), tokens_dev.as<int32_t>(),
                                      d_position(), history.as<int32_t>(), d_history_len(), stream);
            }
            launches += 2;
        }
        BK_CUDA(cudaEventRecord(ev1, stream));
        BK_CUDA(cudaMemcpyAsync(out_tokens, history.p, steps * sizeof(int32_t), cudaMemcpyDeviceToHost, stream));
        stats.d2h_bytes += steps * sizeof(int32_t);
        if (out_logits != nullptr) {
            BK_CUDA(cudaMemcpyAsync(out_logits, logit_history.p, steps * vocab * sizeof(float), cudaMemcpyDeviceToHost, stream));
            stats.d2h_bytes += steps * vocab * sizeof(float);
        }
        queue_step_check();
        BK_CUDA(cudaStreamSynchronize(stream));
        float ms = 0;
        BK_CUDA(cudaEventElapsedTime(&ms, ev0, ev1));
        end_call(ms);
        finish_step_check();  // throws: the position stays where it was
        position += steps;
    }
};

}  // namespace bk

// ---- C ABI ------------------------------------------------------------------------------------------
struct brisk_cuda_session {
    bk::Session s;
};

namespace {

void put_error(char* err, size_t errlen, const std::string& what) {
    if (err != nullptr && errlen > 0) std::snprintf(err, errlen, "%s", what.c_str());
}

template <class Fn>
int guarded(brisk_cuda_session* session, Fn&& fn) {
    try {
        fn();
        return 0;
    } catch (const std::exception& e) {
        session->s.error = e.what();
        return -1;
    }
}

}  // namespace

extern "C" {

int brisk_cuda_device_count(void) {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    return n;
}

brisk_cuda_session* brisk_cuda_create(const brisk_cuda_model* model, const brisk_cuda_options* options, char* err, size_t errlen) {
    if (model == nullptr) {
        put_error(err, errlen, "cuda: no model description");
        return nullptr;
    }
    brisk_cuda_options opt{};
    if (options != nullptr) opt = *options;
    if (opt.tp_size < 1) opt.tp_size = 1;
    try {
        if (brisk_cuda_device_count() <= opt.device) throw bk::CudaError("cuda: no usable CUDA device (this backend has no CPU path)");
        BK_CUDA(cudaSetDevice(opt.device));
        auto session = std::make_unique<brisk_cuda_session>();
        session->s.device = opt.device;
        session->s.load(*model, opt);
        return session.release();
    } catch (const std::exception& e) {
        put_error(err, errlen, e.what());
        return nullptr;
    }
}

void brisk_cuda_destroy(brisk_cuda_session* session) {
    if (session == nullptr) return;
    cudaSetDevice(session->s.device);
    delete session;
}

int brisk_cuda_eval(brisk_cuda_session* session, const int32_t* tokens, uint64_t n, int all_logits, const float** logits) {
    return guarded(session, [&] {
        BK_CUDA(cudaSetDevice(session->s.device));
        const float* out = session->s.eval(tokens, n, all_logits != 0);
        if (logits != nullptr) *logits = out;
    });
}

int brisk_cuda_eval_topk(brisk_cuda_session* session, const int32_t* tokens, uint64_t n, uint32_t k, int32_t* out_ids, float* out_values) {
    return guarded(session, [&] {
        if (k == 0 || out_ids == nullptr || out_values == nullptr) throw bk::CudaError("cuda: top-k needs k >= 1 and both output arrays");
        BK_CUDA(cudaSetDevice(session->s.device));
        session->s.eval(tokens, n, false, k);
        std::memcpy(out_ids, session->s.topk_host, k * sizeof(int32_t));
        std::memcpy(out_values, session->s.topk_host + bk::kMaxTopK, k * sizeof(float));
    });
}

int brisk_cuda_rollback(brisk_cuda_session* session, uint64_t position) {
    return guarded(session, [&] {
        if (position > session->s.position) throw bk::CudaError("cuda: cannot roll forward");
        session->s.position = position;  // the cache keeps its storage; later entries are simply overwritten
    });
}

uint64_t brisk_cuda_position(const brisk_cuda_session* session) { return session->s.position; }
uint32_t brisk_cuda_vocab_size(const brisk_cuda_session* session) { return session->s.vocab; }
uint64_t brisk_cuda_max_context(const brisk_cuda_session* session) { return session->s.max_context; }
const char* brisk_cuda_last_error(const brisk_cuda_session* session) { return session->s.error.c_str(); }

int brisk_cuda_generate_greedy(brisk_cuda_session* session, int32_t first_token, uint64_t steps, int32_t* out_tokens, float* out_logits) {
    return guarded(session, [&] {
        BK_CUDA(cudaSetDevice(session->s.device));
        session->s.generate_greedy(first_token, steps, out_tokens, out_logits);
    });
}

int brisk_cuda_get_stats(const brisk_cuda_session* session, brisk_cuda_stats* out) {
    if (session == nullptr || out == nullptr) return -1;
    *out = session->s.stats;
    return 0;
}

int brisk_cuda_estimate_memory(const brisk_cuda_model* model, const brisk_cuda_options* options, brisk_cuda_memory* out) {
    if (model == nullptr || out == nullptr || model->layers == nullptr) return -1;
    brisk_cuda_options opt{};
    if (options != nullptr) opt = *options;
    *out = bk::estimate(*model, opt);
    return 0;
}

int brisk_cuda_profile(brisk_cuda_session* session, int enable, char* json, size_t len) {
    return guarded(session, [&] {
        bk::Session& s = session->s;
        static const char* names[bk::Session::PH_COUNT] = {"embed", "qkv", "attention", "attn_out", "gate_up", "down", "head", "exchange", "sample"};
        if (json != nullptr && len > 0) {
            std::string out = "{";
            for (int i = 0; i < bk::Session::PH_COUNT; ++i) {
                char buf[128];
                std::snprintf(buf, sizeof buf, "%s\"%s\": {\"ms\": %.6f, \"calls\": %llu}", i ? ", " : "", names[i], s.phase_ms[i],
                              static_cast<unsigned long long>(s.phase_calls[i]));
                out += buf;
            }
            out += "}";
            std::snprintf(json, len, "%s", out.c_str());
        }
        for (int i = 0; i < bk::Session::PH_COUNT; ++i) {
            s.phase_ms[i] = 0;
            s.phase_calls[i] = 0;
        }
        s.profiling = enable != 0;
    });
}

int brisk_cuda_step_path(brisk_cuda_session* session, char* text, size_t len) {
    if (session == nullptr || text == nullptr || len == 0) return -1;
    std::snprintf(text, len, "persistent step kernel %s", session->s.step_note.c_str());
    return 0;
}

int brisk_cuda_debug_buffer(brisk_cuda_session* session, const char* name, float* out, uint64_t count) {
    return guarded(session, [&] {
        bk::Session& s = session->s;
        const std::string n(name ? name : "");
        const bk::DevBuffer* b = n == "hidden" ? &s.hidden_b : n == "query" ? &s.q_b : n == "attended" ? &s.attended_b : n == "ffn" ? &s.ffn_b
                                 : n == "logits" ? &s.logits_b : nullptr;
        if (b == nullptr) throw bk::CudaError("cuda: unknown debug buffer '" + n + "'");
        if (count * sizeof(float) > b->bytes) throw bk::CudaError("cuda: debug read past the end of '" + n + "'");
        BK_CUDA(cudaSetDevice(s.device));
        BK_CUDA(cudaStreamSynchronize(s.stream));
        BK_CUDA(cudaMemcpy(out, b->p, count * sizeof(float), cudaMemcpyDeviceToHost));
    });
}

// Not part of the header: prints the phase stamps gathered with BRISK_CUDA_TRACE=1 (development aid).
int brisk_cuda_dump_trace(brisk_cuda_session* session, unsigned long long* out, uint64_t count) {
    bk::Session& s = session->s;
    if (s.trace.p == nullptr || count * 8 > s.trace.bytes) return -1;
    cudaStreamSynchronize(s.stream);
    return cudaMemcpy(out, s.trace.p, count * 8, cudaMemcpyDeviceToHost) == cudaSuccess ? 0 : -1;
}

int brisk_cuda_tp_unique_id(void* out128, char* err, size_t errlen) {
    try {
        const bk::Nccl& nccl = bk::Nccl::get();
        if (!nccl.ok()) throw bk::CudaError("cuda: tensor parallelism needs NCCL (libnccl.so.2 was not found; set BRISK_NCCL_LIB)");
        bk::NcclId id;
        nccl.check(nccl.GetUniqueId(&id), "ncclGetUniqueId");
        std::memcpy(out128, &id, sizeof(id));
        return 0;
    } catch (const std::exception& e) {
        put_error(err, errlen, e.what());
        return -1;
    }
}

int brisk_cuda_tp_peer_handle(brisk_cuda_session* session, void* out64) {
    return guarded(session, [&] {
        BK_CUDA(cudaSetDevice(session->s.device));
        session->s.peer_handle(out64);
    });
}

int brisk_cuda_tp_peer_attach(brisk_cuda_session* session, const void* handles) {
    return guarded(session, [&] {
        BK_CUDA(cudaSetDevice(session->s.device));
        session->s.peer_attach(handles);
    });
}

}  // extern "C"
