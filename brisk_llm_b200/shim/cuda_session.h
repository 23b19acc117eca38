// CudaSession: brisk-llm's Engine interface (src/engine.h:13-37) over the C ABI of the CUDA token loop
// (include/brisk_cuda.h). This is the file a brisk-llm maintainer adds next to src/metal/metal_session.h; it needs
// the reference's headers (engine.h, model.h, gguf.h) on the include path and links libbrisk_cuda.so.
//
// Like MetalSession it takes a Model built with repack=false (tensors in file layout, src/main.cpp:201) and the
// parsed file, because F16 tensors were widened to f32 by Model::load (src/model.cpp:439-449) and the GPU wants the
// file's own F16 bytes. Errors are rethrown as std::runtime_error("cuda: ...") like the reference's backends.
#pragma once

#include <algorithm>
#include <stdexcept>
#include <string>
#include <string_view>
#include <vector>

#include "engine.h"
#include "gguf.h"
#include "model.h"

extern "C" {
#include "brisk_cuda.h"
}

namespace brisk {

class CudaSession : public Engine {
public:
    CudaSession(const Model& model, const GgufFile& file, std::size_t max_context = 0, int device = 0, unsigned flags = 0) {
        const ModelConfig& c = model.config();
        int arch;
        switch (c.architecture) {
            case Architecture::Qwen3: arch = BRISK_ARCH_QWEN3; break;
            case Architecture::Qwen2: arch = BRISK_ARCH_QWEN3; break;  // the same layer without Q/K norms (NULL) and with q/k/v biases
            case Architecture::Phi3: arch = BRISK_ARCH_QWEN3; break;   // ... with partial rotary; the loader has split its fused tensors
            case Architecture::Llama: arch = BRISK_ARCH_LLAMA; break;
            case Architecture::BitNet: arch = BRISK_ARCH_BITNET; break;
            case Architecture::Gemma3: arch = BRISK_ARCH_GEMMA3; break;
            case Architecture::SmolLM3: arch = BRISK_ARCH_LLAMA; break;  // llama-shaped; its layers without RoPE are flagged below
            default: throw std::runtime_error("cuda: this architecture is not supported by the CUDA backend (qwen3, qwen2, llama, bitnet, gemma3, smollm3, phi3 are)");
        }
        std::vector<brisk_cuda_layer> layers(c.layer_count);
        for (std::size_t i = 0; i < layers.size(); ++i) {
            const Model::Layer& s = model.layers()[i];
            const std::string p = "blk." + std::to_string(i) + ".";
            brisk_cuda_layer& d = layers[i];
            d.attn_norm = s.attention_norm.data();
            d.q = describe(s.query, file, p + "attn_q.weight");
            d.k = describe(s.key, file, p + "attn_k.weight");
            d.v = describe(s.value, file, p + "attn_v.weight");
            d.q_norm = s.query_norm.empty() ? nullptr : s.query_norm.data();
            d.k_norm = s.key_norm.empty() ? nullptr : s.key_norm.data();
            d.q_bias = s.query_bias.empty() ? nullptr : s.query_bias.data();
            d.k_bias = s.key_bias.empty() ? nullptr : s.key_bias.data();
            d.v_bias = s.value_bias.empty() ? nullptr : s.value_bias.data();
            d.attn_sub_norm = s.attention_sub_norm.empty() ? nullptr : s.attention_sub_norm.data();
            d.o = describe(s.attention_output, file, p + "attn_output.weight");
            d.ffn_norm = s.feed_forward_norm.data();
            d.gate = describe(s.gate, file, p + "ffn_gate.weight");
            d.up = describe(s.up, file, p + "ffn_up.weight");
            d.ffn_sub_norm = s.feed_forward_sub_norm.empty() ? nullptr : s.feed_forward_sub_norm.data();
            d.down = describe(s.down, file, p + "ffn_down.weight");
            d.attn_post_norm = s.attention_post_norm.empty() ? nullptr : s.attention_post_norm.data();
            d.ffn_post_norm = s.feed_forward_post_norm.empty() ? nullptr : s.feed_forward_post_norm.data();
            d.slides = c.layer_slides(static_cast<std::uint32_t>(i)) ? 1 : 0;
            d.no_rope = c.layer_has_rope(i) ? 0 : 1;
        }
        brisk_cuda_model d{};
        d.abi_version = BRISK_CUDA_ABI_VERSION;
        d.arch = arch;
        d.vocab_size = c.vocab_size;
        d.hidden = c.embedding_dim;
        d.layer_count = c.layer_count;
        d.head_count = c.head_count;
        d.kv_head_count = c.kv_head_count;
        d.head_dim = c.head_dim;
        d.ffn = c.feed_forward_dim;
        d.context_length = c.context_length;
        d.rope_base = c.rope_base;
        d.rms_epsilon = c.rms_epsilon;
        d.rope_neox = c.rope_neox ? 1 : 0;
        // LongRoPE: a session whose context exceeds the original one takes the long divisors (src/model.cpp:691-694).
        const std::size_t context = max_context == 0 ? c.context_length : std::min<std::size_t>(max_context, c.context_length);
        const std::vector<float>& factors =
            !c.rope_factors_long.empty() && c.rope_original_context != 0 && context > c.rope_original_context ? c.rope_factors_long : c.rope_factors;
        d.rope_factor_count = static_cast<std::uint32_t>(factors.size());
        d.rope_factors = factors.empty() ? nullptr : factors.data();
        d.rope_dim = c.rope_dim;
        d.rope_attn_factor = c.rope_attn_factor;
        d.token_embd = describe(model.token_embedding(), file, "token_embd.weight");
        if (file.tensor("output.weight") != nullptr) d.output = describe(model.output_projection(), file, "output.weight");
        d.output_norm = model.output_norm().data();
        d.layers = layers.data();
        d.rope_scale = c.rope_scale;
        d.rope_base_local = c.rope_base_local;
        d.sliding_window = c.sliding_window;
        d.embedding_scale = c.embedding_scale;
        d.final_softcap = c.final_softcap;
        d.gelu = c.gelu ? 1 : 0;
        brisk_cuda_options opt{};
        opt.max_context = max_context;
        opt.device = device;
        opt.tp_size = 1;
        opt.flags = flags;
        char err[512] = {0};
        session_ = brisk_cuda_create(&d, &opt, err, sizeof err);
        if (session_ == nullptr) throw std::runtime_error(err);
        vocab_ = c.vocab_size;
    }
    ~CudaSession() override { brisk_cuda_destroy(session_); }
    CudaSession(const CudaSession&) = delete;
    CudaSession& operator=(const CudaSession&) = delete;

    using Engine::eval;
    std::span<const float> eval(std::span<const Token> tokens) override { return run(tokens, 0); }
    std::span<const float> eval_all(std::span<const Token> tokens) override { return run(tokens, 1); }
    void rollback(std::size_t position) override {
        if (brisk_cuda_rollback(session_, position) != 0) throw std::runtime_error(brisk_cuda_last_error(session_));
    }
    std::size_t position() const override { return brisk_cuda_position(session_); }

    // For a sampling caller: appends the tokens like eval(), but brings back only the k best (id, logit) pairs of the row,
    // selected on the device - descending by value - instead of the vocabulary-sized span. They are everything
    // Sampler::sample reads after its partial sort (src/sampler.cpp:15-46), so a Sampler overload taking candidates draws
    // from them what sample(span) draws from the full row (k >= the sampler's top_k).
    struct TopK {
        std::vector<Token> ids;
        std::vector<float> values;
    };
    TopK eval_topk(std::span<const Token> tokens, std::uint32_t k) {
        TopK out{std::vector<Token>(k), std::vector<float>(k)};
        if (brisk_cuda_eval_topk(session_, tokens.data(), tokens.size(), k, out.ids.data(), out.values.data()) != 0) {
            throw std::runtime_error(brisk_cuda_last_error(session_));
        }
        return out;
    }

    // Greedy decoding without the per-token host round trip of cmd_generate's loop (src/main.cpp:288-299).
    std::vector<Token> generate_greedy(Token first, std::size_t steps) {
        std::vector<Token> out(steps);
        if (brisk_cuda_generate_greedy(session_, first, steps, out.data(), nullptr) != 0) throw std::runtime_error(brisk_cuda_last_error(session_));
        return out;
    }

private:
    static brisk_cuda_matrix describe(const Matrix& m, const GgufFile& file, std::string_view name) {
        brisk_cuda_matrix out{};
        out.rows = m.rows;
        out.cols = m.cols;
        if (m.format == WeightFormat::F32) {
            const TensorInfo* info = file.tensor(name);
            if (info != nullptr && info->type == TensorType::F16) {  // the file's own halves, not the widened copy
                out.type = BRISK_TYPE_F16;
                out.data = info->data.data();
                out.bytes = info->data.size();
            } else {
                out.type = BRISK_TYPE_F32;
                out.data = m.f32.data();
                out.bytes = m.f32.size_bytes();
            }
            return out;
        }
        switch (m.format) {
            case WeightFormat::Q4_0: out.type = BRISK_TYPE_Q4_0; break;
            case WeightFormat::Q4_1: out.type = BRISK_TYPE_Q4_1; break;
            case WeightFormat::Q5_0: out.type = BRISK_TYPE_Q5_0; break;
            case WeightFormat::Q8_0: out.type = BRISK_TYPE_Q8_0; break;
            case WeightFormat::Q4_K: out.type = BRISK_TYPE_Q4_K; break;
            case WeightFormat::Q5_K: out.type = BRISK_TYPE_Q5_K; break;
            case WeightFormat::Q6_K: out.type = BRISK_TYPE_Q6_K; break;
            case WeightFormat::TQ2_0: out.type = BRISK_TYPE_TQ2_0; break;
            default: throw std::runtime_error("cuda: tensor '" + std::string(name) + "' has a format the CUDA backend does not read (build the Model with repack = false)");
        }
        out.data = m.bytes.data();
        out.bytes = m.bytes.size();
        return out;
    }
    std::span<const float> run(std::span<const Token> tokens, int all) {
        const float* logits = nullptr;
        if (brisk_cuda_eval(session_, tokens.data(), tokens.size(), all, &logits) != 0) throw std::runtime_error(brisk_cuda_last_error(session_));
        return {logits, (all != 0 ? tokens.size() : 1) * vocab_};
    }

    brisk_cuda_session* session_ = nullptr;
    std::size_t vocab_ = 0;
};

}  // namespace brisk
