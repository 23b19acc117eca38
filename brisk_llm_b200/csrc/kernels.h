// Host-callable launchers of the token-loop kernels. Everything runs on the stream given;
// nothing here allocates or synchronises.
#pragma once

#include <string>
#include <vector>

#include "common.cuh"

namespace bk {

// ---- load-time repack (repack.cu) -------------------------------------------------------------
// Bytes of each plane of a rows x cols matrix of `type` in the device layout (see DevMatrix).
struct PlaneSizes {
    size_t qa = 0, qb = 0, qc = 0, sc = 0, d = 0;
    size_t total() const { return qa + qb + qc + sc + d; }
};
PlaneSizes plane_sizes(int type, uint32_t rows, uint32_t cols);
// Carves the planes of `m` out of `base` (256-byte aligned sub-allocations) and fills m's fields.
void bind_planes(DevMatrix& m, int type, uint32_t rows, uint32_t cols, uint8_t* base);
// raw_dev: the matrix in file layout, already in device memory. Writes the planes of `m`.
void launch_repack(const DevMatrix& m, const uint8_t* raw_dev, cudaStream_t s);
// raw_dev: rows x cols bfloat16 values; m: an F32 matrix of the same shape. The reference widens BF16 (and F16)
// tensors to f32 when it loads them (src/model.cpp:439-449).
void launch_widen_bf16(const DevMatrix& m, const uint8_t* raw_dev, cudaStream_t s);

// ---- activations (activations.cu) -------------------------------------------------------------
struct DevActMut {
    float* f32 = nullptr;
    int8_t* q0 = nullptr;
    float* d0 = nullptr;
    int32_t* s0 = nullptr;
    int8_t* qk = nullptr;
    float* dk = nullptr;
    int16_t* bs = nullptr;
    uint32_t cols = 0;
    DevAct view() const { return DevAct{f32, q0, d0, s0, qk, dk, bs, cols}; }
};
// For each of n rows of x[n][ldx]: optional RMS norm (weight != nullptr: y = x * rsqrt(mean(x^2)+eps) * weight;
// the per-row scale uses `norm_cols` = cols values), then the f32 row (if act.f32), its Q8_0 planes (want0) and
// its Q8_K planes (wantk). x may alias act.f32.
void launch_norm_quant(const float* x, uint32_t ldx, const float* weight, float eps, uint32_t n, uint32_t cols,
                       const DevActMut& act, bool want0, bool wantk, cudaStream_t s);

// ---- streaming multiply: 1..8 token rows against whole weight rows (matvec.cu) ----------------
enum Epilogue : int {
    EPI_STORE = 0,     // out[t*ldo + r]  = dot
    EPI_ADD = 1,       // out[t*ldo + r] += dot            (residual stream)
    EPI_SILU_MUL = 2,  // pair (gate, up): out = silu(gate) * up
    EPI_RELU2_MUL = 3  // pair (gate, up): out = max(gate,0)^2 * up
};
struct MatTarget {
    DevMatrix m;
    float* out = nullptr;
    uint32_t ldo = 0;
};
// All targets share `act` (same cols) and the same type. For the pair epilogues pass exactly {gate, up}; the result
// goes to targets[0].out. n may exceed 8: the launcher walks token tiles.
void launch_matvec(const MatTarget* targets, int count, const DevAct& act, uint32_t n, Epilogue epi, cudaStream_t s);

// ---- 2..16 tokens on the int8 tensor path, weights streamed once (smallbatch.cu) ---------------------
// Same contract as launch_matvec; returns false (nothing launched) unless the targets are Q4_0 / Q8_0 with rows of a
// multiple of 8 blocks and 2 <= n <= kSmallBatchMax.
constexpr uint32_t kSmallBatchMax = 16;
bool launch_smallbatch(const MatTarget* targets, int count, const DevAct& act, uint32_t n, Epilogue epi, cudaStream_t s);

// ---- tensor-parallel exchange of one token by peer stores (tp_peer.cu) ---------------------------------
// bufs_dev: device array of the tp ranks' exchange buffers (2 slots of slot_pairs tagged pairs each) as mapped here;
// this rank's [rows_l] slice goes to every rank, dst receives (or is added) the whole [rows_l * tp] vector.
constexpr uint32_t kPeerSlotPairs = 65536;
void launch_tp_peer_exchange(uint2* const* bufs_dev, uint32_t* epoch, unsigned int* error, uint32_t tp, uint32_t rank, uint32_t slot_pairs,
                             const float* local, float* dst, uint32_t rows_l, bool add, cudaStream_t s);

// ---- batched multiply on the int8 tensor path (gemm.cu) ----------------------------------------
// Same contract as launch_matvec for n >= 16 tokens; returns false when this type/shape has no tensor kernel
// (the caller then uses launch_matvec).
bool launch_gemm(const MatTarget* targets, int count, const DevAct& act, uint32_t n, Epilogue epi, cudaStream_t s);
// The Q4_0 / Q8_0 prompt multiply on tcgen05 / tensor memory (gemm_tc.cu; BRISK_CUDA_GEMM=tc): its waits are bounded, and this
// word is non-zero on the device after a launch whose wait ran out.
unsigned int* gemm_tc_error_word();
bool gemm_supports(int type, uint32_t cols);
// The activation after separate gate and up multiplies. mode 0: gate[i] = silu(gate[i]) * up[i]; 1: max(gate[i],0)^2 * up[i];
// 2: tanh-GELU(gate[i]) * up[i] (gelu_mul_f32, src/kernels_f32.cpp:291-296), its tanh corrected by tanh_table (see
// build_tanh_table) when one is given.
void launch_gate_mul(float* gate, const float* up, size_t count, int mode, cudaStream_t s, const uint8_t* tanh_table = nullptr);

// ---- Gemma layer variants (gemma.cu) ------------------------------------------------------------
// x[i] *= scale: the embedding scale (src/model.cpp:899-901).
void launch_scale_rows(float* x, size_t count, float scale, cudaStream_t s);
// hidden[t][:] += rms_norm(proj[t][:]) * weight, the norm as in src/model.cpp:87-97 (post-norms, :1116-1119, :1155-1158).
void launch_post_norm_add(const float* proj, const float* weight, float* hidden, uint32_t n, uint32_t cols, float eps, cudaStream_t s);
// logits[i] = cap * tanh(logits[i] / cap) (src/model.cpp:1206-1209).
void launch_softcap(float* logits, size_t count, float cap, const uint8_t* tanh_table, cudaStream_t s);
// The table that makes the device's tanh return the bits of the host C library's tanhf (tanh_like_host, formats.cuh):
// one 4-bit correction per float in [2^-25, 22), tanh_table_bytes() in all. The device evaluates its own base function for
// every such float, the host evaluates its library's tanhf for the same inputs on `threads` threads, and the differences
// are uploaded to `table` (device memory of tanh_table_bytes()). Called once per session of a model that uses a tanh.
size_t tanh_table_bytes();
void build_tanh_table(uint8_t* table, unsigned threads, cudaStream_t s);

// ---- per-token vector work (misc.cu) -----------------------------------------------------------
// hidden[t][:] = dequantised row tokens[t] of the embedding matrix (Session::eval_batch's embedding_row).
void launch_embed(const DevMatrix& embd, const int32_t* tokens_dev, uint32_t n, float* hidden, cudaStream_t s);

struct RopeArgs {
    float* q;            // [n][heads*dim] in place
    float* k;            // [n][kv*dim]   (normed + rotated, then stored to the cache)
    const float* v;      // [n][kv*dim]
    const float* q_norm; // [dim] or nullptr
    const float* k_norm;
    uint32_t rope_dim = 0;          // leading values of a head that rotate (Phi's partial rotary); 0: all of them
    const float* q_bias = nullptr;  // [heads*dim] / [kv*dim] projection biases, or nullptr (all three or none)
    const float* k_bias = nullptr;
    const float* v_bias = nullptr;
    const float* rope;   // [max_context][dim]: cos, sin per pair, indexed by absolute position
    __half* k_cache;     // [kv][max_context][dim]
    __half* v_cache;
    const uint32_t* position; // device scalar: position of token 0 of this batch
    uint32_t n, heads, kv_heads, dim, max_context;
    float eps;
    int neox;
};
void launch_qk_norm_rope_store(const RopeArgs& a, cudaStream_t s);

struct AttnArgs {
    const float* q;        // [n][heads*dim]
    const __half* k_cache; // [kv][max_context][dim]
    const __half* v_cache;
    float* out;            // [n][heads*dim]
    float* scores;         // scratch: [n][heads][max_context]
    const uint32_t* position;
    uint32_t n, heads, kv_heads, dim, max_context;
    uint32_t max_visible;  // host-side upper bound of position + n (sizes the grid)
    float scale;
    uint32_t window = 0;   // sliding-window layer: a token attends to its last `window` positions only (0: to all)
};
size_t attn_scratch_floats(uint32_t n, uint32_t heads, uint32_t max_context);
void launch_attention(const AttnArgs& a, cudaStream_t s);
// Softmax + weighted sum for a few tokens (attn_chain.cu): a.scores holds their scaled scores. One CTA per (token, one or
// two query heads, slice of the head), chain warps and product warps; same results as the kernels above.
bool attn_chain_fits(uint32_t n, uint32_t heads, uint32_t kv_heads, uint32_t dim, uint32_t max_visible, uint32_t sms);
void launch_attn_chain(const AttnArgs& a, uint32_t sms, cudaStream_t s);
// The single-token form (product warps and a chain warp; same file): a.n is taken as 1.
bool attn_chain_one_fits(uint32_t dim, uint32_t max_visible);
void launch_attn_chain_one(const AttnArgs& a, cudaStream_t s);
constexpr uint32_t kChainOneMinContext = 2048;  // single tokens of sessions with at least this context take it
constexpr uint32_t kChainMaxTokens = 24;      // more tokens than this share V rows through the tiled kernel instead
// BRISK_CUDA_CHAIN: 0 never, 1 wherever it fits, unset: 2..kChainMaxTokens tokens, and single tokens (their own form of the
// kernel, below) in sessions whose context is at least kChainOneMinContext.
int chain_mode();
unsigned int* attn_chain_error_word();        // non-zero on the device after a launch whose wait for a bulk copy ran out

// ---- fused single-token step (decode.cu) -------------------------------------------------------------------------
// One multiply of the decode step: every CTA rebuilds the activation row in shared memory (x, optionally RMS-normed with
// norm_weight, then quantised the way the targets' type takes it) and multiplies its rows. Launched with programmatic
// dependent launch: weights are prefetched while the previous kernel drains. `sms` sizes the persistent grid.
void launch_dec_multiply(const MatTarget* targets, int count, const float* x, const float* norm_weight, float eps, uint32_t cols, Epilogue epi,
                         uint32_t sms, cudaStream_t s, unsigned long long* trace = nullptr);
// Attention of the single new token: scores kernel (per-head norm + RoPE of q and the new k, f16 K/V store in its
// prologue) and softmax + weighted-sum kernel. Takes the same argument structs as the batched kernels (n is 1).
void launch_dec_attention(const RopeArgs& r, const AttnArgs& at, uint32_t sms, cudaStream_t s);
// Whether a context of max_context positions fits the shared memory of that attention's weighted-sum kernel.
bool dec_attention_fits(uint32_t max_context, uint32_t heads, uint32_t dim, uint32_t sms);

// ---- the single-token step of all layers as one persistent kernel (step.cu) -------------------------------------
struct StepLayerArgs {
    DevMatrix q, k, v, o, gate, up, down;
    const float* attn_norm = nullptr;
    const float* q_norm = nullptr;
    const float* k_norm = nullptr;
    const float* attn_sub_norm = nullptr;
    const float* ffn_norm = nullptr;
    const float* ffn_sub_norm = nullptr;
    const float* q_bias = nullptr;
    const float* k_bias = nullptr;
    const float* v_bias = nullptr;
    __half* k_cache = nullptr;
    __half* v_cache = nullptr;
};
struct StepShared {  // the step's activation vectors and the model constants every layer shares
    float* hidden = nullptr;    // [hidden_size] residual stream, in and out
    float* q = nullptr;         // [heads*dim]
    float* k = nullptr;         // [kv_heads*dim]
    float* v = nullptr;
    float* attended = nullptr;  // [heads*dim]
    float* gated = nullptr;     // [ffn_size]
    float* scores = nullptr;    // [heads][max_context]
    const float* rope = nullptr;
    const uint32_t* position = nullptr;
    uint32_t hidden_size = 0, ffn_size = 0, heads = 0, kv_heads = 0, dim = 0, max_context = 0;
    float eps = 0.0f, scale = 0.0f;
    int neox = 0;
    int act_epi = EPI_SILU_MUL;
    unsigned long long* body_trace = nullptr;  // development aid: 4 x 8 words for the stamps inside one layer's multiplies
};
// Built once per session (the weights and buffers are fixed); launch() runs layers 0..n-1 of one token whose embedding
// is in `hidden` and whose position is in *position. build() returns false, with the reason, when the model is outside
// what the persistent kernel covers (mixed weight types in the layers, F16/F32 layer matrices, head sizes other than 64
// and 128, a context too long for its shared memory) - the caller then keeps the one-kernel-per-operation path.
// Every barrier wait inside the kernel is bounded; a wait that ran out sets the word at error_word() (device memory),
// which the caller copies back with the step's results and checks, then rearm()s.
class StepPlan {
public:
    StepPlan();
    ~StepPlan();
    StepPlan(const StepPlan&) = delete;
    StepPlan& operator=(const StepPlan&) = delete;
    bool build(const std::vector<StepLayerArgs>& layers, const StepShared& shared, uint32_t sms, cudaStream_t s, std::string& why_not);
    bool ready() const { return impl_ != nullptr; }
    // False when the launch parameters must differ from token to token (the tagged exchange): such a launch cannot be
    // replayed from a captured graph.
    bool graph_safe() const;
    void launch(cudaStream_t s);
    const unsigned int* error_word() const;
    // Development aid: 4 words per phase (6 per layer) written by CTA 0 - entry, barrier passed, finished (ns), polls.
    void set_trace(unsigned long long* words);
    void rearm(cudaStream_t s);
    const std::string& description() const { return description_; }

private:
    struct Impl;
    Impl* impl_ = nullptr;
    std::string description_;
};

// ---- one decoded token as one launch (token.cu) -------------------------------------------------------------------
// Embedding row, every layer, output head and arg-max of one token in a single cooperative kernel, for models whose layer
// matrices and head are Q4_0 and whose per-SM share of one layer fits shared memory. With advance the kernel also feeds
// the next step (*token = choice, *position += 1, history) exactly as launch_argmax_advance does.
struct TokenEnds {
    DevMatrix embd, head;
    const float* output_norm = nullptr;
    float* logits = nullptr;        // [vocab]
    uint32_t vocab = 0;
    int32_t* token = nullptr;       // device: the token to evaluate (and, advancing, the next one)
    int32_t* chosen = nullptr;      // device: arg-max of the logits
    int32_t* history = nullptr;
    uint32_t* history_len = nullptr;
};
class TokenPlan {
public:
    TokenPlan();
    ~TokenPlan();
    TokenPlan(const TokenPlan&) = delete;
    TokenPlan& operator=(const TokenPlan&) = delete;
    // false, with the reason, when the model is outside what the kernel covers
    bool build(const std::vector<StepLayerArgs>& layers, const StepShared& shared, const TokenEnds& ends, uint32_t sms, cudaStream_t s, std::string& why_not);
    bool ready() const { return impl_ != nullptr; }
    // The token's embedding row is read from the Q4_0 embedding inside the kernel; for any other embedding type the caller
    // writes it to shared.hidden first (embeds_itself() is false).
    bool embeds_itself() const { return embd_q4_0_; }
    void launch(cudaStream_t s, bool advance);
    const unsigned int* error_word() const;
    void set_trace(unsigned long long* words);  // development aid: CTA 0 stamps the end of every phase
    void rearm(cudaStream_t s);
    const std::string& description() const { return description_; }

private:
    struct Impl;
    Impl* impl_ = nullptr;
    bool embd_q4_0_ = false;
    std::string description_;
};

// ---- the k best logits of a row (topk.cu) --------------------------------------------------------------------------
constexpr uint32_t kMaxTopK = 64;
// out_ids[k], out_values[k]: descending by value, the lower id first among equal values; a NaN never ahead of a number.
// scratch: topk_scratch_keys(vocab, k) 64-bit words.
size_t topk_scratch_keys(uint32_t vocab, uint32_t k);
void launch_topk(const float* logits, uint32_t vocab, uint32_t k, unsigned long long* scratch, int32_t* out_ids, float* out_values, cudaStream_t s,
                 uint64_t* launches = nullptr);

// Tensor parallel re-layout: gathered[rank][t][rows_l] -> dst[t][rank*rows_l + r] (add: dst += ...), tp ranks.
void launch_tp_unpack(const float* gathered, float* dst, uint32_t n, uint32_t rows_l, uint32_t tp, bool add, cudaStream_t s);

// First maximum of each of n rows of logits[n][vocab] (lowest index on ties) -> out_token[n].
// If next_token/position are given (single row), also feeds the decode loop: *next_token = argmax, *position += 1,
// and appends the token to history[*history_len++].
void launch_argmax(const float* logits, uint32_t vocab, uint32_t n, int32_t* out_token, float* scratch_val,
                   int32_t* scratch_idx, cudaStream_t s);
size_t argmax_scratch_elems(uint32_t vocab);
// Arg-max of one row that also feeds the decode loop: *token_slot = choice, *position += 1, history[(*history_len)++] = choice.
void launch_argmax_advance(const float* logits, uint32_t vocab, int32_t* out_token, float* scratch_val, int32_t* scratch_idx,
                           int32_t* token_slot, uint32_t* position, int32_t* history, uint32_t* history_len, cudaStream_t s);

}  // namespace bk
