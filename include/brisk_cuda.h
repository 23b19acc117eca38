/* brisk_cuda.h - C ABI of the B200 (sm_100a) token-loop backend for brisk-llm.
 *
 * The reference has no C layer: its backends are C++ classes behind `brisk::Engine`
 * (src/engine.h:13-37), built at three call sites next to the Metal one
 * (src/main.cpp:203-212, :335-344; src/server.cpp:241-249). This header is the
 * boundary a `CudaSession : Engine` binds to: plain pointers and sizes, status
 * ints instead of exceptions, no C++ or torch types. Each entry point names the
 * reference interface it stands in for.
 *
 * Threading: one caller thread per session, like an Engine (the reference's server
 * serialises requests, src/server.cpp:160-205). Nothing here falls back to the CPU:
 * every call fails with a message when no CUDA device is usable.
 */
#ifndef BRISK_CUDA_H
#define BRISK_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define BRISK_CUDA_ABI_VERSION 4u

/* Tensor storage types, numbered as in ggml / the reference's TensorType (src/gguf.h:22-27).
 * Quantised data is passed exactly as it lies in a GGUF file: row after row of blocks
 * (block layouts: src/quant.h:26-130). */
enum brisk_cuda_type {
    BRISK_TYPE_F32 = 0,
    BRISK_TYPE_F16 = 1,
    BRISK_TYPE_Q4_0 = 2,
    BRISK_TYPE_Q4_1 = 3,
    BRISK_TYPE_Q5_0 = 6,
    BRISK_TYPE_Q8_0 = 8,
    BRISK_TYPE_Q4_K = 12,
    BRISK_TYPE_Q5_K = 13,
    BRISK_TYPE_Q6_K = 14,
    BRISK_TYPE_BF16 = 30, /* matrices only; widened to f32 on upload, as the reference widens it on load (src/model.cpp:439-449) */
    BRISK_TYPE_TQ2_0 = 35
};

/* Layer families (subset of brisk::Architecture, src/model.h:20-31). The id selects the gate activation and little
 * else; what a family needs beyond it travels in the fields below (absent norms are NULL, biases, no_rope, rope_dim ...).
 * Qwen2 and Phi3 files are described as BRISK_ARCH_QWEN3, SmolLM3 as BRISK_ARCH_LLAMA. */
enum brisk_cuda_arch {
    BRISK_ARCH_QWEN3 = 0,  /* per-head RMS norm on Q and K, SiLU-gated FFN, NeoX RoPE            */
    BRISK_ARCH_LLAMA = 1,  /* adjacent-pair RoPE, optional per-frequency divisors (rope_freqs)  */
    BRISK_ARCH_BITNET = 2, /* sub-norms before o_proj and down_proj, squared-ReLU gate, NeoX    */
    BRISK_ARCH_GEMMA3 = 3  /* Q/K norms, norms after attention and the feed-forward, tanh-GELU gate,
                              scaled embeddings, sliding-window layers with their own RoPE base,
                              optional soft cap on the logits (src/model.h:24, :63-71)           */
};

/* A rows x cols weight matrix, `rows` outputs over `cols` inputs (brisk::Matrix, src/model.h:123-134).
 * `data` is a HOST pointer that only has to stay valid during brisk_cuda_create(): the library
 * repacks into its own device layout and keeps no host pointer. */
typedef struct brisk_cuda_matrix {
    int32_t type; /* enum brisk_cuda_type */
    int32_t reserved;
    uint64_t rows;
    uint64_t cols;
    const void* data;
    uint64_t bytes;
} brisk_cuda_matrix;

/* One decoder layer (brisk::Model::Layer, src/model.h:143-176). Float vectors are f32 host
 * pointers; an absent one is NULL. */
typedef struct brisk_cuda_layer {
    const float* attn_norm;     /* [hidden]                                   */
    brisk_cuda_matrix q, k, v;  /* [heads*head_dim | kv*head_dim] x hidden    */
    const float* q_norm;        /* [head_dim] or NULL (qwen3)                 */
    const float* k_norm;        /* [head_dim] or NULL                         */
    const float* attn_sub_norm; /* [heads*head_dim] or NULL (bitnet)          */
    brisk_cuda_matrix o;        /* hidden x heads*head_dim                    */
    const float* ffn_norm;      /* [hidden]                                   */
    brisk_cuda_matrix gate, up; /* ffn x hidden                               */
    const float* ffn_sub_norm;  /* [ffn] or NULL (bitnet)                     */
    brisk_cuda_matrix down;     /* hidden x ffn                               */
    /* Projection biases (Qwen2-style files, src/model.cpp:411-416): all three or none. Added to the q/k/v
     * projections before the per-head norm and RoPE (src/model.cpp:1026-1030). */
    const float* q_bias;        /* [heads*head_dim] or NULL                   */
    const float* k_bias;        /* [kv*head_dim] or NULL                      */
    const float* v_bias;        /* [kv*head_dim] or NULL                      */
    /* Gemma: RMS norm of a projection's output before it is added to the residual stream
     * (src/model.h:161-162, src/model.cpp:1116-1119, :1150-1153). NULL: plain residual add. */
    const float* attn_post_norm; /* [hidden] or NULL                          */
    const float* ffn_post_norm;  /* [hidden] or NULL                          */
    /* 1: the layer attends only to the last `sliding_window` positions and rotates with the table of
     * rope_base_local (ModelConfig::layer_slides, src/model.h:87-90; src/model.cpp:1084-1085). */
    int32_t slides;
    /* 1: the layer attends without positional rotation (SmolLM3's every fourth layer, ModelConfig::layer_has_rope,
     * src/model.h:97-110; src/model.cpp:1024). */
    int32_t no_rope;
} brisk_cuda_layer;

/* POD mirror of the brisk::ModelConfig fields the supported families use (src/model.h:36-62)
 * plus the bound tensors (brisk::Model, src/model.cpp:326-421). */
typedef struct brisk_cuda_model {
    uint32_t abi_version; /* BRISK_CUDA_ABI_VERSION */
    int32_t arch;         /* enum brisk_cuda_arch   */
    uint32_t vocab_size;
    uint32_t hidden;
    uint32_t layer_count;
    uint32_t head_count;
    uint32_t kv_head_count;
    uint32_t head_dim;
    uint32_t ffn;
    uint32_t context_length;
    float rope_base;
    float rms_epsilon;
    int32_t rope_neox;           /* 1: pair (i, i+head_dim/2); 0: pair (2i, 2i+1)          */
    uint32_t rope_factor_count;  /* 0 or (rope_dim ? rope_dim : head_dim) / 2              */
    const float* rope_factors;   /* per-frequency divisors of the angle (src/model.cpp:886) */
    brisk_cuda_matrix token_embd; /* vocab x hidden                                        */
    brisk_cuda_matrix output;     /* vocab x hidden; data == NULL: tied to token_embd       */
    const float* output_norm;     /* [hidden]                                              */
    const brisk_cuda_layer* layers; /* [layer_count]                                        */
    /* Gemma 3 (src/model.cpp:169-176, :286). Zero in every field: none of it applies. */
    float rope_scale;        /* the position is multiplied by this before the angles are built (1 / rope.scaling.factor,
                                src/model.cpp:173, :882); 0 means 1                                                 */
    float rope_base_local;   /* RoPE base of the sliding layers (scale 1, no per-frequency divisors; src/model.cpp:894) */
    uint32_t sliding_window; /* positions a sliding layer sees; 0: no layer slides                                   */
    float embedding_scale;   /* embedding rows are multiplied by this (sqrt(hidden), src/model.cpp:899-901); 0 means 1 */
    float final_softcap;     /* logits = c * tanh(logits / c) when non-zero (src/model.cpp:1206-1209)                */
    int32_t gelu;            /* 1: gate with tanh-GELU instead of SiLU (src/model.cpp:1139-1140)                     */
    /* Phi-3 / Phi-4-mini (src/model.cpp:177-188, src/model.h:54-62). */
    uint32_t rope_dim;       /* leading values of a head that rotate (partial rotary); 0: all head_dim of them. The angles
                                are built for this width (src/model.cpp:893) and rope_factor_count is then rope_dim / 2     */
    float rope_attn_factor;  /* cos and sin are multiplied by this (src/model.cpp:887-888); 0 means 1. rope_factors are the
                                short or the long LongRoPE divisors, whichever the session's context selects
                                (src/model.cpp:691-694)                                                                 */
} brisk_cuda_model;

typedef struct brisk_cuda_options {
    uint64_t max_context; /* 0: the model's context_length (src/model.cpp:659)              */
    int32_t device;       /* CUDA ordinal                                                   */
    int32_t tp_rank;      /* tensor-parallel rank of this process, 0 when tp_size <= 1      */
    int32_t tp_size;      /* 1: no tensor parallelism                                       */
    uint32_t flags;       /* BRISK_CUDA_FLAG_*                                              */
    const void* tp_unique_id; /* 128 bytes from brisk_cuda_tp_unique_id(), same on all ranks */
} brisk_cuda_options;

#define BRISK_CUDA_FLAG_NO_GRAPH 1u      /* launch decode kernels one by one instead of replaying a CUDA graph */
#define BRISK_CUDA_FLAG_NO_MEGAKERNEL 2u /* single-token steps through the batched kernels instead of the fused ones */
#define BRISK_CUDA_FLAG_NO_PERSISTENT 4u /* single-token steps as one fused kernel per operation (replayed as a CUDA graph)
                                            instead of one persistent kernel for all layers */

typedef struct brisk_cuda_session brisk_cuda_session;

/* Counters of the most recent eval / generate call, for benchmarks. */
typedef struct brisk_cuda_stats {
    double device_ms;        /* CUDA-event time of the call's device work on the session's stream */
    uint64_t kernel_launches; /* kernels of this library launched (graph nodes count one each)     */
    uint64_t weight_bytes;    /* bytes of weight planes resident in HBM (all matrices + norms)     */
    uint64_t kv_bytes;        /* bytes of the f16 K/V cache                                        */
    uint64_t h2d_bytes;       /* host->device bytes copied by the call                             */
    uint64_t d2h_bytes;       /* device->host bytes copied by the call                             */
    uint64_t persistent_steps; /* single-token steps of the call that ran as the persistent all-layer kernel */
} brisk_cuda_stats;

/* Device memory a session will hold, before anything is allocated - the device-side analogue of estimate_memory /
 * MemoryEstimate (src/memory.h:13-24, src/memory.cpp:46-96). */
typedef struct brisk_cuda_memory {
    uint64_t weights; /* repacked weight planes and norm vectors of this rank            */
    uint64_t cache;   /* f16 K/V cache for the session's context                         */
    uint64_t scratch; /* one batch of activations, attention scores, logits, RoPE table  */
} brisk_cuda_memory;

/* Fills `out` for the session brisk_cuda_create(model, options) would build. Needs no GPU. brisk_cuda_create runs the
 * same estimate against the device's free memory and refuses, with the breakdown and a hint (a shorter context when the
 * cache is what does not fit), instead of running out of memory half-way - check_memory's behaviour
 * (src/memory.cpp:114-135); BRISK_NO_MEMORY_CHECK=1 skips the check, as in the reference. */
int brisk_cuda_estimate_memory(const brisk_cuda_model* model, const brisk_cuda_options* options, brisk_cuda_memory* out);

/* Number of usable CUDA devices; 0 when there is none or the driver is missing.
 * (The Metal backend's equivalent is the `gpu` flag check, src/main.cpp:204-212.) */
int brisk_cuda_device_count(void);

/* Builds a session: uploads and repacks every tensor once, allocates the f16 K/V cache for
 * min(max_context, context_length) positions and the scratch. Stands in for
 * `MetalSession(model, file, max_context)` (src/metal/metal_session.h:23) and
 * `Session(model, threads, max_context)` (src/model.cpp:655-702). Returns NULL and writes a
 * message into err on failure. */
brisk_cuda_session* brisk_cuda_create(const brisk_cuda_model* model, const brisk_cuda_options* options, char* err,
                                      size_t errlen);

/* Engine::~Engine (src/engine.h:15). */
void brisk_cuda_destroy(brisk_cuda_session* session);

/* Engine::eval (all_logits == 0) and Engine::eval_all (all_logits != 0) (src/engine.h:17-26,
 * src/model.cpp:704-727). Appends n tokens at the current position. *logits then points at
 * vocab floats (last token) or n*vocab floats (row i predicts the token after tokens[i]) in
 * pinned host memory owned by the session, valid until its next call. Errors, raised before any
 * work like the reference: n == 0 ("no tokens to evaluate"), all_logits with n > 64
 * ("eval_all takes 1 to 64 tokens"), an id outside [0, vocab) ("token id out of range"),
 * n > max_context - position ("context length exceeded"). Returns 0 on success. */
int brisk_cuda_eval(brisk_cuda_session* session, const int32_t* tokens, uint64_t n, int all_logits, const float** logits);

/* Engine::rollback (src/engine.h:29, src/model.cpp:735-751): O(1), only moves the cursor;
 * position > current position fails with "cannot roll forward". */
int brisk_cuda_rollback(brisk_cuda_session* session, uint64_t position);

/* Engine::position (src/engine.h:31). */
uint64_t brisk_cuda_position(const brisk_cuda_session* session);

uint32_t brisk_cuda_vocab_size(const brisk_cuda_session* session);
uint64_t brisk_cuda_max_context(const brisk_cuda_session* session);

/* Message of the session's most recent failure ("cuda: ..."), which the C++ shim rethrows as
 * std::runtime_error like the reference backends do (src/model.cpp:18, src/metal/metal_session.mm:27). */
const char* brisk_cuda_last_error(const brisk_cuda_session* session);

/* The greedy loop of cmd_generate (src/main.cpp:288-299) without its per-token host round trip:
 * evaluates `first_token`, picks the arg-max on the device (lowest id on ties, as
 * Sampler::sample does for temperature <= 0, src/sampler.cpp:11-13), feeds it back, `steps` times.
 * out_tokens[i] is the token chosen after step i; out_logits, if not NULL, receives the
 * [steps][vocab] logits the choices were made from. The session advances by `steps` positions. */
int brisk_cuda_generate_greedy(brisk_cuda_session* session, int32_t first_token, uint64_t steps, int32_t* out_tokens,
                               float* out_logits);

/* Engine::eval for a sampling host: appends the tokens like brisk_cuda_eval, but instead of the vocabulary-sized row of
 * logits returns its k best (id, logit) pairs, selected on the device - out_ids[k] / out_values[k], descending by value,
 * the lower id first among equal values, a NaN never ahead of a number. That is all Sampler::sample reads after its
 * std::partial_sort (src/sampler.cpp:15-46: the top_k candidates by value, then softmax, top-p cut and draw on those
 * alone), so a host sampler fed the k pairs draws what it would draw from the full row, and the per-token copy shrinks
 * from vocab * 4 bytes to k * 8. k: 1..64 (and at most the vocabulary size); k = 1 is the greedy pick. */
int brisk_cuda_eval_topk(brisk_cuda_session* session, const int32_t* tokens, uint64_t n, uint32_t k, int32_t* out_ids, float* out_values);

int brisk_cuda_get_stats(const brisk_cuda_session* session, brisk_cuda_stats* out);

/* Test hook, the counterpart of metal_matmul (src/metal/metal_session.h:39-47): out[t*rows + r] =
 * row r of w (file layout, `type`) times activation row t of x ([n][cols] f32), computed the way
 * Session::multiply does (src/model.cpp:551-653): activations quantised per row to Q8_0 (Q4_0,
 * Q8_0) or Q8_K (Q4_K, Q6_K, TQ2_0), integer block dots, f32 scaling; F16/F32 weights use raw f32
 * activations. All pointers are host pointers. */
int brisk_cuda_matmul(int32_t type, const void* w, uint64_t rows, uint64_t cols, const float* x, uint64_t n, float* out,
                      char* err, size_t errlen);

/* Bench hook, the counterpart of metal_matmul_seconds (src/metal/metal_session.h:49-59): uploads
 * `copies` repacked copies of w (so the working set can exceed L2), runs `iterations` multiplies
 * rotating over them and returns the mean device seconds per multiply in *seconds. */
int brisk_cuda_matmul_seconds(int32_t type, const void* w, uint64_t rows, uint64_t cols, uint64_t n, uint32_t copies,
                              uint32_t iterations, double* seconds, char* err, size_t errlen);

/* No counterpart in the reference. Greedy pick (first maximum, lowest id on ties - the rule of brisk_cuda_generate_greedy)
 * of each of `rows` rows of logits[rows][vocab], for hosts that must not allocate device memory at that point: an
 * embedder that has handed all of HBM to its own arena (a server that sizes its K/V pool to what cudaMemGetInfo
 * reports), or one that calls from a latency-critical thread where the implicit device-wide synchronisation of an
 * allocation is not acceptable. `logits` and `out_tokens` are DEVICE pointers owned by the caller; `stream` is a
 * cudaStream_t (NULL: the default stream). The scratch between the two reduction stages lives in a fixed 76 KB array
 * inside the library image, so: at most 64 rows per call (more is refused with a message); the array is shared by
 * every call on that device and keeps the last call's contents (the first stage overwrites all it uses, nothing needs
 * clearing); two calls whose kernels overlap on the GPU race on it - keep them on one stream or order them. The first
 * call on each device looks up the array's device address (with that device current); make that first call before any
 * stream capture begins. Calls no cudaMalloc/cudaFree and no allocating library routine. */
int brisk_cuda_argmax_static(const float* logits, uint32_t vocab, uint32_t rows, int32_t* out_tokens, void* stream, char* err,
                             size_t errlen);

/* How single-token steps run in this session, as text: "persistent step kernel on: <configuration>" or
 * "persistent step kernel off: <reason>" (tensor parallel, flags, a model outside what the kernel covers, a barrier
 * that timed out earlier). No reference counterpart; benchmarks record it next to their numbers. */
int brisk_cuda_step_path(brisk_cuda_session* session, char* text, size_t len);

/* Per-phase device time, the counterpart of Session::profile() / BRISK_PROFILE (src/model.h:242-245,
 * src/main.cpp:302-306) and BRISK_GPU_PROFILE (src/metal/metal_session.mm:711-719). Writes the time accumulated since
 * the previous call as JSON ({"qkv": {"ms": .., "calls": ..}, ...}) into `json` (may be NULL), clears the counters, and
 * switches profiling on or off. While it is on, every phase is bracketed by CUDA events and the single-token step
 * runs kernel by kernel instead of as a graph, so totals are slower than an unprofiled run: use it for shares. */
int brisk_cuda_profile(brisk_cuda_session* session, int enable, char* json, size_t len);

/* Debug hook, the counterpart of the BRISK_GPU_DEBUG / BRISK_CPU_DEBUG dumps (src/metal/metal_session.mm:1073-1100,
 * src/model.cpp:1183-1192): copies the first `count` floats of one scratch buffer as the last batch left it.
 * name: "hidden" (residual stream [n][hidden]), "query" (after norm and RoPE), "attended", "ffn" (gated activation),
 * "logits". Intended for layer-by-layer comparison with a one-layer model. */
int brisk_cuda_debug_buffer(brisk_cuda_session* session, const char* name, float* out, uint64_t count);

/* Tensor parallelism (no counterpart in the reference, which is single-process): rank 0 calls this
 * and hands the 128 bytes to every rank's brisk_cuda_options.tp_unique_id. */
int brisk_cuda_tp_unique_id(void* out128, char* err, size_t errlen);

/* Optional, after every rank's session exists: single-token steps then exchange activations by stores into the peers'
 * buffers (one small kernel per exchange) instead of NCCL all-gathers; prompts keep the all-gathers. Same results.
 * Every rank calls brisk_cuda_tp_peer_handle (64 bytes out: a CUDA IPC handle of its exchange buffer), the host program
 * gathers the handles in rank order (tp_size x 64 bytes), and every rank calls brisk_cuda_tp_peer_attach with them. All
 * ranks must have attached before any rank runs its next single-token step. One rank per GPU, all on one node. No
 * counterpart in the reference. */
int brisk_cuda_tp_peer_handle(brisk_cuda_session* session, void* out64);
int brisk_cuda_tp_peer_attach(brisk_cuda_session* session, const void* handles);

#ifdef __cplusplus
}
#endif

#endif /* BRISK_CUDA_H */
