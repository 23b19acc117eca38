// TEST INFRASTRUCTURE, NOT PRODUCT CODE.
//
// extern "C" doorway into the UNMODIFIED reference CPU engine (brisk-llm), so the
// Python tests can (1) pin the plain-C restatement in brisk_oracle.c against the
// real thing and (2) time the reference's own CPU path as the reported baseline.
// It is compiled together with the reference's own source files, taken from where
// they lie in a reference checkout (see the Makefile beside this file); none of
// those sources is copied here. The resulting library lands in oracle/_ref/.
//
// Every wrapper names the reference entry point it forwards to.
#include <algorithm>
#include <chrono>
#include <cstdint>
#include <cstring>
#include <memory>
#include <stdexcept>
#include <string>
#include <vector>

#include "engine.h"
#include "gguf.h"
#include "kernels.h"
#include "kernels_f32.h"
#include "mapped_file.h"
#include "model.h"
#include "quant.h"
#include "sampler.h"
#include "speculative.h"

namespace {

thread_local std::string g_error;

// ggml tensor-type ids are the wire format of this shim (same ids as include/brisk_cuda.h).
bool to_format(int ggml_type, brisk::WeightFormat& out) {
    switch (ggml_type) {
        case 2: out = brisk::WeightFormat::Q4_0; return true;
        case 3: out = brisk::WeightFormat::Q4_1; return true;
        case 6: out = brisk::WeightFormat::Q5_0; return true;
        case 8: out = brisk::WeightFormat::Q8_0; return true;
        case 13: out = brisk::WeightFormat::Q5_K; return true;
        case 12: out = brisk::WeightFormat::Q4_K; return true;
        case 14: out = brisk::WeightFormat::Q6_K; return true;
        case 35: out = brisk::WeightFormat::TQ2_0; return true;
        default: return false;
    }
}

struct RefSession {
    std::unique_ptr<brisk::MappedFile> mapped;
    std::unique_ptr<brisk::GgufFile> file;
    std::unique_ptr<brisk::Model> model;
    std::unique_ptr<brisk::Session> session;
};

}  // namespace

extern "C" {

const char* ref_last_error() { return g_error.c_str(); }

// kernels::kernel_set_name (src/kernels.cpp:265): "generic" on x86-64.
const char* ref_kernel_set_name() {
    static std::string name(brisk::kernels::kernel_set_name());
    return name.c_str();
}

// half_to_float / float_to_half (src/quant.cpp:61, :87)
float ref_half_to_float(std::uint16_t h) { return brisk::half_to_float(h); }
std::uint16_t ref_float_to_half(float f) { return brisk::float_to_half(f); }

// quantize_q8_0 (src/quant.cpp:115): out = count/32 blocks of 34 bytes.
void ref_quantize_q8_0(const float* x, void* out, std::uint64_t count) {
    brisk::quantize_q8_0(x, static_cast<brisk::BlockQ8_0*>(out), count);
}

// quantize_q8_k (src/quant.cpp:146), 8-bit: out = count/256 blocks of 292 bytes.
void ref_quantize_q8_k(const float* x, void* out, std::uint64_t count) {
    brisk::quantize_q8_k(x, static_cast<brisk::BlockQ8_K*>(out), count, 8);
}

// dequantize_* (src/quant.cpp:196-307, :565)
int ref_dequantize(int ggml_type, const void* blocks, float* out, std::uint64_t count) {
    brisk::WeightFormat f;
    if (!to_format(ggml_type, f)) return -1;
    switch (f) {
        case brisk::WeightFormat::Q4_0: brisk::dequantize_q4_0(static_cast<const brisk::BlockQ4_0*>(blocks), out, count); break;
        case brisk::WeightFormat::Q4_1: brisk::dequantize_q4_1(static_cast<const brisk::BlockQ4_1*>(blocks), out, count); break;
        case brisk::WeightFormat::Q5_0: brisk::dequantize_q5_0(static_cast<const brisk::BlockQ5_0*>(blocks), out, count); break;
        case brisk::WeightFormat::Q5_K: brisk::dequantize_q5_k(static_cast<const brisk::BlockQ5_K*>(blocks), out, count); break;
        case brisk::WeightFormat::Q8_0: brisk::dequantize_q8_0(static_cast<const brisk::BlockQ8_0*>(blocks), out, count); break;
        case brisk::WeightFormat::Q4_K: brisk::dequantize_q4_k(static_cast<const brisk::BlockQ4_K*>(blocks), out, count); break;
        case brisk::WeightFormat::Q6_K: brisk::dequantize_q6_k(static_cast<const brisk::BlockQ6_K*>(blocks), out, count); break;
        case brisk::WeightFormat::TQ2_0: brisk::dequantize_tq2_0(static_cast<const brisk::BlockTQ2_0*>(blocks), out, count); break;
        default: return -1;
    }
    return 0;
}

// What Session::multiply does for one quantised matrix (src/model.cpp:579-652):
// quantise each activation row (Q8_K for K-quants/ternary, Q8_0 otherwise), then
// generic_kernels(format).matvec (n == 1) or .matmul (src/kernels.cpp:13-30,129-163).
// out is [n][rows].
int ref_matmul(int ggml_type, const void* w, std::uint64_t rows, std::uint64_t cols, const float* x, std::uint64_t n,
               float* out) {
    brisk::WeightFormat f;
    if (!to_format(ggml_type, f)) return -1;
    try {
        const std::size_t blocks = cols / brisk::block_elements(f);
        const brisk::kernels::KernelSet k = brisk::kernels::generic_kernels(f);
        if (brisk::takes_q8_k(f)) {
            std::vector<brisk::BlockQ8_K> q(n * blocks);
            for (std::size_t t = 0; t < n; ++t) brisk::quantize_q8_k(x + t * cols, q.data() + t * blocks, cols, 8);
            if (n == 1) k.matvec(w, rows, cols, q.data(), out);
            else k.matmul(w, rows, cols, q.data(), n, out, rows);
        } else {
            std::vector<brisk::BlockQ8_0> q(n * blocks);
            for (std::size_t t = 0; t < n; ++t) brisk::quantize_q8_0(x + t * cols, q.data() + t * blocks, cols);
            if (n == 1) k.matvec(w, rows, cols, q.data(), out);
            else k.matmul(w, rows, cols, q.data(), n, out, rows);
        }
    } catch (const std::exception& e) {
        g_error = e.what();
        return -1;
    }
    return 0;
}

// F32 matrices (widened F16 heads) go through kernels::dot_f32 on raw activations (src/model.cpp:641-646).
void ref_matmul_f32(const float* w, std::uint64_t rows, std::uint64_t cols, const float* x, std::uint64_t n, float* out) {
    for (std::size_t r = 0; r < rows; ++r)
        for (std::size_t t = 0; t < n; ++t) out[t * rows + r] = brisk::kernels::dot_f32(w + r * cols, x + t * cols, cols);
}

// MappedFile + GgufFile::parse + Model(file, repack=false) + Session (src/main.cpp:178-212 with the flag a GPU
// backend gets: plain formats, 8-bit activations).
void* ref_session_create(const char* gguf_path, std::uint64_t threads, std::uint64_t max_context) {
    try {
        auto s = std::make_unique<RefSession>();
        s->mapped = std::make_unique<brisk::MappedFile>(gguf_path);
        s->file = std::make_unique<brisk::GgufFile>(brisk::GgufFile::parse(s->mapped->bytes()));
        s->model = std::make_unique<brisk::Model>(*s->file, /*repack=*/false);
        s->session = std::make_unique<brisk::Session>(*s->model, threads, max_context);
        return s.release();
    } catch (const std::exception& e) {
        g_error = e.what();
        return nullptr;
    }
}

void ref_session_destroy(void* h) { delete static_cast<RefSession*>(h); }

std::uint32_t ref_session_vocab(void* h) { return static_cast<RefSession*>(h)->model->config().vocab_size; }

// Engine::eval / Engine::eval_all (src/model.cpp:704-727). Copies the logits out: V floats, or n*V with all != 0.
int ref_session_eval(void* h, const std::int32_t* tokens, std::uint64_t n, int all, float* logits_out) {
    try {
        auto* s = static_cast<RefSession*>(h);
        const std::span<const brisk::Token> span(tokens, n);
        const std::span<const float> logits = all ? s->session->eval_all(span) : s->session->eval(span);
        if (logits_out != nullptr) std::memcpy(logits_out, logits.data(), logits.size() * sizeof(float));
        return 0;
    } catch (const std::exception& e) {
        g_error = e.what();
        return -1;
    }
}

// Engine::rollback / position (src/model.cpp:735-751)
int ref_session_rollback(void* h, std::uint64_t position) {
    try {
        static_cast<RefSession*>(h)->session->rollback(position);
        return 0;
    } catch (const std::exception& e) {
        g_error = e.what();
        return -1;
    }
}
std::uint64_t ref_session_position(void* h) { return static_cast<RefSession*>(h)->session->position(); }

// Engine::log_likelihood (src/engine.cpp:10-33)
int ref_session_log_likelihood(void* h, const std::int32_t* tokens, std::uint64_t n, double* out) {
    try {
        *out = static_cast<RefSession*>(h)->session->log_likelihood(std::span<const brisk::Token>(tokens, n));
        return 0;
    } catch (const std::exception& e) {
        g_error = e.what();
        return -1;
    }
}

// The greedy loop of cmd_generate (src/main.cpp:220-222,288-299): eval(prompt), then `steps` times
// next = Sampler(temperature 0).sample(logits); logits = eval(next). Writes the chosen ids, and, if asked,
// the logits each choice was made from ([steps][V]). Returns seconds spent in prefill and decode.
int ref_session_generate_greedy(void* h, const std::int32_t* prompt, std::uint64_t n_prompt, std::uint64_t steps,
                                std::int32_t* out_tokens, float* out_logits, double* prefill_s, double* decode_s) {
    try {
        auto* s = static_cast<RefSession*>(h);
        const std::size_t vocab = s->model->config().vocab_size;
        brisk::SamplerConfig config;
        config.temperature = 0.0f;
        brisk::Sampler sampler(config);
        const auto t0 = std::chrono::steady_clock::now();
        std::span<const float> logits = s->session->eval(std::span<const brisk::Token>(prompt, n_prompt));
        const auto t1 = std::chrono::steady_clock::now();
        for (std::size_t i = 0; i < steps; ++i) {
            if (out_logits != nullptr) std::memcpy(out_logits + i * vocab, logits.data(), vocab * sizeof(float));
            const brisk::Token next = sampler.sample(logits);
            out_tokens[i] = next;
            if (i + 1 < steps) logits = s->session->eval(next);
        }
        const auto t2 = std::chrono::steady_clock::now();
        if (prefill_s != nullptr) *prefill_s = std::chrono::duration<double>(t1 - t0).count();
        if (decode_s != nullptr) *decode_s = std::chrono::duration<double>(t2 - t1).count();
        return 0;
    } catch (const std::exception& e) {
        g_error = e.what();
        return -1;
    }
}

// Sampler::sample (src/sampler.cpp:9-46) `draws` times on one row of logits, with one Sampler (its generator advances
// from draw to draw). Tests feed it the full row and a row that holds only the device's top-k pairs (-inf elsewhere).
int ref_sampler_draws(const float* logits, std::uint64_t n, float temperature, std::uint32_t top_k, float top_p, std::uint64_t seed,
                      std::uint64_t draws, std::int32_t* out) {
    try {
        brisk::SamplerConfig config;
        config.temperature = temperature;
        config.top_k = top_k;
        config.top_p = top_p;
        config.seed = seed;
        brisk::Sampler sampler(config);
        for (std::uint64_t i = 0; i < draws; ++i) out[i] = sampler.sample(std::span<const float>(logits, n));
        return 0;
    } catch (const std::exception& e) {
        g_error = e.what();
        return -1;
    }
}

// LookupDrafter::observe + draft (src/speculative.cpp:45-65). Returns the number of guesses written.
std::uint64_t ref_lookup_draft(const std::int32_t* history, std::uint64_t n, std::uint64_t count, std::int32_t* out) {
    brisk::LookupDrafter drafter;
    drafter.observe(std::span<const brisk::Token>(history, n));
    const std::vector<brisk::Token> guesses = drafter.draft(count);
    std::copy(guesses.begin(), guesses.end(), out);
    return guesses.size();
}

// Speculator over the reference Session with a LookupDrafter (src/speculative.cpp:67-118): prompt minus its last
// token is evaluated, then rounds run until `want` tokens are settled. Returns how many were written (>= want is
// truncated to want) or -1.
std::int64_t ref_session_speculate(void* h, const std::int32_t* prompt, std::uint64_t n_prompt, std::uint64_t draft_tokens,
                                   std::uint64_t want, std::int32_t* out, std::uint64_t* rounds, std::uint64_t* accepted) {
    try {
        auto* s = static_cast<RefSession*>(h);
        brisk::LookupDrafter drafter;
        drafter.observe(std::span<const brisk::Token>(prompt, n_prompt));
        if (n_prompt > 1) s->session->eval(std::span<const brisk::Token>(prompt, n_prompt - 1));
        brisk::Speculator spec(*s->session, drafter, prompt[n_prompt - 1], draft_tokens);
        std::uint64_t written = 0;
        while (written < want) {
            for (const brisk::Token t : spec.step()) {
                if (written < want) out[written++] = t;
            }
        }
        if (rounds != nullptr) *rounds = spec.stats().rounds + spec.stats().plain;
        if (accepted != nullptr) *accepted = spec.stats().accepted;
        return static_cast<std::int64_t>(written);
    } catch (const std::exception& e) {
        g_error = e.what();
        return -1;
    }
}

}  // extern "C"
