// TEST INFRASTRUCTURE. Drives the UNMODIFIED reference's own callers of the token loop - Engine::log_likelihood
// (src/engine.cpp:10-33), the greedy loop of cmd_generate (src/main.cpp:288-299) with the reference Sampler, and
// Speculator with a LookupDrafter (src/speculative.cpp:72-118) - once over the reference CPU Session and once over
// CudaSession (brisk_llm_b200/shim/cuda_session.h), on the same GGUF file and token ids, and reports whether the two
// engines produced identical results. Built only where a reference checkout is present (make -C oracle driver).
//
//   ref_driver <model.gguf> <threads> <n_prompt> <n_decode> <seed>
#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <memory>
#include <random>
#include <vector>

#include "cuda_session.h"
#include "mapped_file.h"
#include "sampler.h"
#include "speculative.h"

using namespace brisk;

struct Result {
    std::vector<float> prefill_logits;
    std::vector<Token> greedy;
    double log_likelihood = 0;
    std::vector<Token> speculated;
    std::size_t spec_rounds = 0, spec_accepted = 0;
};

static Result run(Engine& engine, const std::vector<Token>& prompt, std::size_t decode, std::size_t vocab) {
    Result r;
    std::span<const float> logits = engine.eval(prompt);
    r.prefill_logits.assign(logits.begin(), logits.begin() + static_cast<std::ptrdiff_t>(vocab));
    SamplerConfig config;
    config.temperature = 0.0f;
    Sampler sampler(config);
    for (std::size_t i = 0; i < decode; ++i) {
        const Token next = sampler.sample(logits);
        r.greedy.push_back(next);
        logits = engine.eval(next);
    }
    engine.rollback(0);
    r.log_likelihood = engine.log_likelihood(prompt);
    engine.rollback(0);
    // a prompt that repeats itself, so the lookup drafter has something to propose
    std::vector<Token> rep;
    for (int k = 0; k < 4; ++k) rep.insert(rep.end(), prompt.begin(), prompt.begin() + std::min<std::size_t>(8, prompt.size()));
    LookupDrafter drafter;
    drafter.observe(rep);
    engine.eval(std::span<const Token>(rep.data(), rep.size() - 1));
    Speculator spec(engine, drafter, rep.back(), 8);
    while (r.speculated.size() < 24) {
        for (const Token t : spec.step()) r.speculated.push_back(t);
    }
    r.speculated.resize(24);
    r.spec_rounds = spec.stats().rounds + spec.stats().plain;
    r.spec_accepted = spec.stats().accepted;
    engine.rollback(0);
    return r;
}

int main(int argc, char** argv) {
    if (argc < 6) {
        std::fprintf(stderr, "usage: ref_driver model.gguf threads n_prompt n_decode seed\n");
        return 2;
    }
    try {
        const MappedFile mapped(argv[1]);
        const GgufFile file = GgufFile::parse(mapped.bytes());
        const Model model(file, /*repack=*/false);
        const std::size_t threads = std::strtoul(argv[2], nullptr, 10), n_prompt = std::strtoul(argv[3], nullptr, 10),
                          n_decode = std::strtoul(argv[4], nullptr, 10);
        std::mt19937 rng(static_cast<unsigned>(std::strtoul(argv[5], nullptr, 10)));
        const std::size_t vocab = model.config().vocab_size;
        std::vector<Token> prompt(n_prompt);
        for (Token& t : prompt) t = static_cast<Token>(rng() % vocab);

        Session cpu(model, threads, 0);
        const Result a = run(cpu, prompt, n_decode, vocab);
        CudaSession gpu(model, file, 0);
        const Result b = run(gpu, prompt, n_decode, vocab);

        double max_abs = 0;
        for (std::size_t i = 0; i < vocab; ++i) max_abs = std::max(max_abs, static_cast<double>(std::abs(a.prefill_logits[i] - b.prefill_logits[i])));
        const bool same_greedy = a.greedy == b.greedy, same_spec = a.speculated == b.speculated;
        std::printf("{\"prefill_logits_max_abs_diff\": %.9g, \"prefill_logits_bit_equal\": %s, \"greedy_equal\": %s, "
                    "\"log_likelihood_cpu\": %.12f, \"log_likelihood_cuda\": %.12f, \"speculated_equal\": %s, "
                    "\"spec_rounds\": [%zu, %zu], \"spec_accepted\": [%zu, %zu]}\n",
                    max_abs, std::memcmp(a.prefill_logits.data(), b.prefill_logits.data(), vocab * sizeof(float)) == 0 ? "true" : "false",
                    same_greedy ? "true" : "false", a.log_likelihood, b.log_likelihood, same_spec ? "true" : "false", a.spec_rounds, b.spec_rounds,
                    a.spec_accepted, b.spec_accepted);
        // error behaviour at the boundary: the same conditions must throw from both engines
        int mismatches = 0;
        auto throws = [](Engine& e, auto&& fn) {
            try {
                fn(e);
            } catch (const std::runtime_error&) {
                return true;
            }
            return false;
        };
        const std::vector<Token> none, bad{static_cast<Token>(vocab)}, many(65, 0);
        for (Engine* e : {static_cast<Engine*>(&cpu), static_cast<Engine*>(&gpu)}) {
            mismatches += !throws(*e, [&](Engine& x) { x.eval(none); });
            mismatches += !throws(*e, [&](Engine& x) { x.eval(bad); });
            mismatches += !throws(*e, [&](Engine& x) { x.eval_all(many); });
            mismatches += !throws(*e, [&](Engine& x) { x.rollback(1); });
        }
        std::printf("{\"boundary_errors_missing\": %d}\n", mismatches);
        return (same_greedy && same_spec && mismatches == 0) ? 0 : 1;
    } catch (const std::exception& e) {
        std::fprintf(stderr, "ref_driver: %s\n", e.what());
        return 3;
    }
}
