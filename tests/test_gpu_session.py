"""GPU parity of the whole token loop, through the C ABI (CudaSession), against the CPU oracle and the golden
vectors taken from the reference engine.

Tolerances written here are the stated ones for logits: max-abs-diff 2e-2 and relative L2 1e-3; greedy ids must be
identical except where the reference's top-2 logit gap is below that tolerance. On top of that, families whose output
head is quantised must match BIT FOR BIT: the kernels repeat the CPU engine's float operations in the CPU's order,
because a single differing ulp ahead of an 8-bit re-quantisation or an f16 cache store can flip a rounding and the
flip then spreads through the layers (measured: ~1e-2 relative after two layers). The ternary family's F16 head sums
in a different order, so its logits are held to 1e-5 instead (its residual stream is still bit-identical).
"""
import importlib.util
import os

import numpy as np
import pytest

import helpers as H
from brisk_llm_b200 import engine, formats, synth

pytestmark = pytest.mark.gpu

spec_ = importlib.util.spec_from_file_location("make_golden", os.path.join(H.GOLDEN, "make_golden.py"))
mg = importlib.util.module_from_spec(spec_)
spec_.loader.exec_module(mg)

MAX_ABS, REL_L2 = 2e-2, 1e-3


def close(got, want, exact=True):
    got, want = np.asarray(got), np.asarray(want)
    assert got.shape == want.shape
    assert np.abs(got - want).max() <= MAX_ABS, np.abs(got - want).max()
    assert H.rel_l2(got, want) <= REL_L2, H.rel_l2(got, want)
    if exact is None:  # only the stated tolerance
        return
    if exact:
        assert np.array_equal(got, want), (np.abs(got - want).max(), int((got != want).sum()))
    else:
        assert np.abs(got - want).max() <= 1e-5


def exactness(family):
    """True: bit for bit - Gemma 3 included: its GELU and soft cap go through the C library's tanhf on the CPU, which the
    device reproduces with its correction table. False: unquantised heads (F16, BF16) sum in another order, 1e-5."""
    return family not in ("bitnet", "mixed")


def greedy_agrees(got_ids, want_ids, want_logits):
    """Identical ids, except that a step whose reference top-2 gap is within tolerance may differ; the comparison
    stops there because the sequences legitimately diverge afterwards."""
    for i, (g, w) in enumerate(zip(got_ids, want_ids)):
        if g != w:
            top2 = np.sort(want_logits[i])[-2:]
            assert top2[1] - top2[0] < MAX_ABS, (i, g, w, top2)
            return i
    return len(want_ids)


@pytest.mark.parametrize("family", list(mg.FAMILIES) + list(mg.MORE_FAMILIES))
def test_golden_from_the_reference(family):
    g = np.load(os.path.join(H.GOLDEN, f"model_{family}.npz"))
    m = mg.golden_model(family)
    assert mg.model_digest(m).encode() == g["digest"].tobytes()
    toks = g["tokens"]
    ex = exactness(family)
    with engine.CudaSession(m) as s:
        close(s.eval(toks[:33]), g["prefill33"], ex)
        for i in range(4):
            close(s.eval(toks[33 + i:34 + i]), g["decode4"][i], ex)
        close(s.eval_all(toks[37:46]), g["eval_all9"], ex)
        s.rollback(35)
        assert s.position() == 35
        close(s.eval(toks[46:47]), g["after_rollback35"], ex)
        s.rollback(0)
        ll = s.log_likelihood(toks)
        assert abs(ll - g["log_likelihood48"][0]) < 5e-3 * 47, (ll, g["log_likelihood48"][0])
        # perplexity agreement to 3 decimals
        assert round(np.exp(-ll / 47), 3) == round(np.exp(-g["log_likelihood48"][0] / 47), 3)
        s.rollback(0)
        s.eval(toks[:19])
        ids, logits = s.generate_greedy(int(toks[19]), 16, want_logits=True)
        n = greedy_agrees(ids, g["greedy16_ids"], g["greedy16_logits"])
        close(logits[:max(n, 1)], g["greedy16_logits"][:max(n, 1)], ex)
        if ex:
            assert n == 16 and np.array_equal(ids, g["greedy16_ids"])


@pytest.mark.parametrize("context,prompt", [(1024, 600), (2048, 1300)])
def test_heads_of_256_values(context, prompt):
    """Gemma 3's head geometry (256-wide heads, one K/V head for four query heads) on an otherwise Qwen3-shaped layer, so that
    everything stays bit for bit: 8-token tiles below 1024 positions, 16-token tiles past them, then single tokens."""
    spec = synth.tiny(synth.QWEN3_0_6B, layers=2, vocab=512, context=context, heads=4, kv_heads=1, head_dim=256)
    m = synth.perturb_norms(synth.generate(spec, seed=51))
    toks = synth.random_tokens(spec, prompt + 8, seed=52)
    o = H.OracleSession(m)
    with engine.CudaSession(m) as s:
        assert "256-wide heads" in s.step_path()
        close(s.eval(toks[:prompt]), o.eval(toks[:prompt]))
        for i in range(prompt, prompt + 3):
            close(s.eval(toks[i:i + 1]), o.eval(toks[i:i + 1]))
        close(s.eval_all(toks[prompt + 3:prompt + 8]), o.eval_all(toks[prompt + 3:prompt + 8]))
        s.rollback(prompt)
        o.rollback(prompt)
        want_ids, want_logits = o.generate_greedy(toks[prompt:prompt + 1], 6)
        ids, logits = s.generate_greedy(int(toks[prompt]), 6, want_logits=True)
        assert np.array_equal(ids, want_ids) and np.array_equal(logits, want_logits)
    o.close()


def test_sliding_window_layers_are_bit_exact_without_a_tanh():
    """The sliding window, the local RoPE table and the embedding scale involve no tanh, so their kernels must reproduce
    the CPU engine bit for bit: the attended values of a one-layer Gemma-3-shaped model (its only layer slides), read
    before anything has passed through the GELU."""
    spec = synth.tiny(synth.QWEN3_0_6B, arch="gemma3", layers=1, vocab=512, context=2048, sliding_window=300)
    m = synth.perturb_norms(synth.generate(spec, seed=41))
    toks = synth.random_tokens(spec, 1310, seed=42)
    o = H.OracleSession(m)
    with engine.CudaSession(m) as s:
        # three device batches; the last (276 tokens) takes the 16-token tiles, every token's window starts mid-chunk
        s.eval(toks[:1300])
        o.eval(toks[:1300])
        q = spec.q_dim
        got = s.debug_buffer("attended", 276 * q).reshape(276, q)[256:]
        assert np.array_equal(got, o.debug_buffer("attended", 20 * q).reshape(20, q))
        for i in range(1300, 1303):  # single tokens through the same kernels
            s.eval(toks[i:i + 1])
            o.eval(toks[i:i + 1])
            assert np.array_equal(s.debug_buffer("attended", q), o.debug_buffer("attended", q))
    o.close()


@pytest.mark.parametrize("family,spec", [
    ("qwen3", synth.tiny(synth.QWEN3_0_6B, layers=4, vocab=2048, context=1024)),
    ("llama", synth.tiny(synth.LLAMA_3_2_1B, layers=3, vocab=1024, context=1024)),
    ("bitnet", synth.tiny(synth.BITNET_2B, layers=3, vocab=1024, context=1024)),
    ("mistral", synth.tiny(synth.MISTRAL_7B, layers=2, vocab=1024, context=1024)),
    # Qwen2-style q/k/v projection biases
    ("biased", synth.tiny(synth.MISTRAL_7B, layers=2, vocab=1024, context=1024, hidden=1024, heads=8, kv_heads=2, ffn=2048, qkv_bias=True)),
    # the formats beyond the benchmark configurations (Q5_K, Q4_1, Q5_0, a BF16 head), mixed as stock downloads mix them
    ("mixed", synth.tiny(synth.QWEN3_0_6B, layers=2, vocab=1024, context=1024, tied=False, fmt=formats.Q5_K,
                         fmt_overrides={"v": formats.Q4_1, "down": formats.Q5_0, "embd": formats.Q4_1, "output": formats.BF16})),
    # Phi-4-mini's layer at its own widths: 24 query heads on 8 K/V heads, the first 96 of 128 values rotate, scaled cos/sin,
    # the long LongRoPE divisors
    ("phi3", synth.tiny(synth.MISTRAL_7B, arch="phi3", layers=2, vocab=1024, context=1024, hidden=3072, heads=24, kv_heads=8, head_dim=128,
                        ffn=8192, rope_dim=96, rope_attn_factor=1.19, rope_original_context=512)),
    # the qwen2 architecture id: NeoX rotation, biases, no Q/K norms
    ("qwen2", synth.tiny(synth.MISTRAL_7B, arch="qwen2", layers=2, vocab=1024, context=1024, hidden=1536, heads=12, kv_heads=2, head_dim=128, ffn=2048, qkv_bias=True)),
    # 5 and 6 query heads per K/V head (Qwen2.5-14B, Qwen2.5-1.5B)
    ("group5", synth.tiny(synth.QWEN3_0_6B, layers=2, vocab=1024, context=1024, hidden=640, heads=5, kv_heads=1, ffn=1280)),
    ("group6", synth.tiny(synth.MISTRAL_7B, layers=2, vocab=1024, context=1024, hidden=768, heads=12, kv_heads=2, head_dim=64, ffn=1536, qkv_bias=True)),
    ("group3", synth.tiny(synth.QWEN3_0_6B, layers=2, vocab=1024, context=1024, hidden=768, heads=6, kv_heads=2, ffn=1536)),
    ("group7", synth.tiny(synth.MISTRAL_7B, layers=2, vocab=1024, context=1024, hidden=896, heads=14, kv_heads=2, head_dim=64, ffn=1792, qkv_bias=True)),
    # SmolLM3: llama-shaped, every fourth layer attends without RoPE
    ("smollm3", synth.tiny(synth.LLAMA_3_2_1B, arch="smollm3", layers=4, vocab=1024, context=1024)),
    # Gemma 3 layer variants: six layers sliding over 128 positions around one global layer with a scaled position,
    # post-norms, tanh-GELU, scaled embeddings, soft-capped logits
    ("gemma3", synth.tiny(synth.QWEN3_0_6B, arch="gemma3", layers=7, vocab=1024, context=1024, sliding_window=128,
                          rope_scaling_factor=8.0, final_softcap=30.0)),
])
def test_full_width_layers_against_the_oracle(family, spec):
    """The real layer widths of each configuration (few layers, small vocabulary), a 600-token prompt processed in
    two device batches, then teacher-forced decode steps and the on-device greedy loop."""
    m = synth.perturb_norms(synth.generate(spec, seed=5))
    toks = synth.random_tokens(spec, 640, seed=6)
    o = H.OracleSession(m)
    ex = exactness(family)
    with engine.CudaSession(m) as s:
        close(s.eval(toks[:600]), o.eval(toks[:600]), ex)
        # the residual stream of every prompt token of the last batch, bit for bit (all families without a tanh)
        got_hidden, want_hidden = s.debug_buffer("hidden", 88 * spec.hidden), o.debug_buffer("hidden", 88 * spec.hidden)
        if ex is None:
            assert H.rel_l2(got_hidden, want_hidden) <= REL_L2
        else:
            assert np.array_equal(got_hidden, want_hidden)
        for i in range(600, 606):
            close(s.eval(toks[i:i + 1]), o.eval(toks[i:i + 1]), ex)
        close(s.eval_all(toks[606:615]), o.eval_all(toks[606:615]), ex)
        s.rollback(603)
        o.rollback(603)
        want_ids, want_logits = o.generate_greedy(toks[615:616], 12)
        got_logits0 = s.eval(toks[615:616])
        close(got_logits0, want_logits[0], ex)
        s.rollback(603)
        ids, logits = s.generate_greedy(int(toks[615]), 12, want_logits=True)
        n = greedy_agrees(ids, want_ids, want_logits)
        close(logits[:max(n, 1)], want_logits[:max(n, 1)], ex)
        assert s.position() == 603 + 12
    o.close()


def test_generate_greedy_equals_the_eval_loop():
    spec = synth.tiny(synth.QWEN3_0_6B, layers=2, vocab=1024)
    m = synth.generate(spec, seed=2)
    toks = synth.random_tokens(spec, 20, seed=3)
    with engine.CudaSession(m) as s:
        logits = s.eval(toks)
        loop = []
        for _ in range(10):
            nxt = int(np.argmax(logits))
            loop.append(nxt)
            logits = s.eval([nxt])
        s.rollback(19)
        ids = s.generate_greedy(int(toks[19]), 10)
        assert list(ids) == loop
        st = s.stats()
        assert st["kernel_launches"] > 0 and st["device_ms"] > 0
    # same result when the step is launched kernel by kernel instead of as a CUDA graph
    from brisk_llm_b200 import abi
    with engine.CudaSession(m, flags=abi.FLAG_NO_GRAPH) as s:
        s.eval(toks[:19])
        assert list(s.generate_greedy(int(toks[19]), 10)) == loop


def test_argmax_takes_the_lowest_id_on_ties():
    # an all-zero head makes every logit exactly 0: greedy must pick id 0 (first maximum, as std::max_element)
    spec = synth.tiny(synth.QWEN3_0_6B, layers=1, vocab=512)
    m = synth.generate(spec, seed=2)
    t = dict(m.tensors)
    fmt, shape, data = t["token_embd.weight"]
    t["output.weight"] = (fmt, shape, np.zeros_like(data))
    m2 = synth.HostModel(spec, t)
    with engine.CudaSession(m2) as s:
        assert list(s.generate_greedy(7, 3)) == [0, 0, 0]


def test_error_behaviour_matches_the_reference():
    spec = synth.tiny(synth.QWEN3_0_6B, layers=1, vocab=512)
    m = synth.generate(spec, seed=2)
    with engine.CudaSession(m, max_context=16) as s:
        assert s.max_context == 16
        with pytest.raises(RuntimeError, match="cuda: no tokens to evaluate"):
            s.eval(np.zeros(0, np.int32))
        with pytest.raises(RuntimeError, match="cuda: token id out of range"):
            s.eval([512])
        with pytest.raises(RuntimeError, match="cuda: token id out of range"):
            s.eval([-1])
        with pytest.raises(RuntimeError, match="cuda: eval_all takes 1 to 64 tokens"):
            s.eval_all(np.zeros(65, np.int32))
        with pytest.raises(RuntimeError, match="cuda: context length exceeded"):
            s.eval(np.zeros(17, np.int32))
        assert s.position() == 0  # nothing was evaluated
        s.eval([1, 2, 3])
        with pytest.raises(RuntimeError, match="cuda: cannot roll forward"):
            s.rollback(4)
        s.eval(np.zeros(13, np.int32))
        with pytest.raises(RuntimeError, match="cuda: context length exceeded"):
            s.eval([1])
    with engine.CudaSession(m, max_context=10_000) as s:
        assert s.max_context == spec.context  # capped at the model's trained context


def test_speculative_verify_on_the_gpu_matches_the_oracle():
    """The reference's Speculator drives an Engine through eval_all + rollback (src/speculative.cpp:72-118); the same
    loop over CudaSession must settle the same tokens as over the oracle."""
    spec = synth.tiny(synth.MISTRAL_7B, layers=2, vocab=1024, hidden=512, heads=4, kv_heads=2, ffn=1024)
    m = synth.generate(spec, seed=8)
    prompt = np.tile(synth.random_tokens(spec, 8, seed=1), 4).astype(np.int32)
    o = H.OracleSession(m)
    want, _, _ = o.speculate(prompt, 8, 24)
    o.close()
    from brisk_llm_b200 import speculative
    with engine.CudaSession(m) as s:
        got, stats = speculative.speculate(s, prompt, 8, 24)
    first_diff = next((i for i, (a, b) in enumerate(zip(got, want)) if a != b), len(want))
    assert first_diff >= 20, (list(got), list(want))


def test_memory_preflight_refuses_what_cannot_fit(monkeypatch):
    """brisk_cuda_create checks its estimate against the device's free memory, like check_memory does for host RAM
    (src/memory.cpp:114-135); the free figure is overridden here so that nothing actually runs out of memory."""
    spec = synth.tiny(synth.QWEN3_0_6B, layers=2, vocab=1024, context=8192)
    m = synth.generate(spec, seed=2)
    need = engine.estimate_memory(m)
    margin = 256 << 20  # kept free on top of the estimate
    monkeypatch.setenv("BRISK_CUDA_ASSUME_FREE_BYTES", str(need["total"] + margin - need["cache"] // 2))
    with pytest.raises(RuntimeError, match="of device memory .* weights, .* cache, .* scratch.* is free. Try a shorter context"):
        engine.CudaSession(m)
    with engine.CudaSession(m, max_context=512) as s:  # the hint works
        assert s.max_context == 512
    monkeypatch.setenv("BRISK_NO_MEMORY_CHECK", "1")
    with engine.CudaSession(m) as s:
        assert s.max_context == 8192


@pytest.mark.parametrize("family,spec", [
    ("qwen3", synth.tiny(synth.QWEN3_0_6B, layers=3, vocab=1024, context=2048)),
    ("llama", synth.tiny(synth.LLAMA_3_2_1B, layers=2, vocab=1024, context=2048)),
    ("bitnet", synth.tiny(synth.BITNET_2B, layers=2, vocab=1024, context=2048)),
    ("mistral", synth.tiny(synth.MISTRAL_7B, layers=2, vocab=1024, context=2048)),
    ("biased", synth.tiny(synth.MISTRAL_7B, layers=2, vocab=1024, context=2048, hidden=1024, heads=8, kv_heads=2, ffn=2048, qkv_bias=True)),
    # query heads per K/V head that are not powers of two: 3 (Llama-3.2-3B, Phi-4-mini) and 7 (Qwen2.5-7B, with its biases)
    ("group3", synth.tiny(synth.QWEN3_0_6B, layers=2, vocab=1024, context=2048, hidden=768, heads=6, kv_heads=2, ffn=1536)),
    ("group7", synth.tiny(synth.MISTRAL_7B, layers=2, vocab=1024, context=2048, hidden=896, heads=14, kv_heads=2, head_dim=64, ffn=1792, qkv_bias=True)),
])
def test_the_three_single_token_paths_agree_bit_for_bit(family, spec, monkeypatch):
    """A single-token step can run as one launch for the whole token (embedding to arg-max; Q4_0 models of the 0.6B class),
    as one persistent kernel for all layers, as one fused kernel per operation, or through the batched kernels. All of
    them repeat the same float operations in the same order: their logits must be identical bits, at several context
    lengths (one that crosses the 512-position chunks of the attention phases included)."""
    from brisk_llm_b200 import abi
    # the persistent kernel is off by default for models with wide rows (slower there); force it, to test its variants
    monkeypatch.setenv("BRISK_CUDA_STEP", "force")
    m = synth.perturb_norms(synth.generate(spec, seed=11))
    toks = synth.random_tokens(spec, 1200, seed=12)
    results = {}
    for name, flags in (("token", 0), ("persistent", 0), ("per_operation", abi.FLAG_NO_PERSISTENT), ("batched", abi.FLAG_NO_MEGAKERNEL)):
        monkeypatch.setenv("BRISK_CUDA_TOKEN", "1" if name == "token" else "0")
        with engine.CudaSession(m, flags=flags) as s:
            uniform = len({f for n, (f, sh, d) in m.tensors.items() if n.startswith("blk.") and n.endswith(".weight") and not n.endswith("norm.weight")}) == 1
            if name == "token":
                if "one launch per token:" not in s.step_path().split("(")[0]:
                    assert family in ("llama", "bitnet", "mistral", "group7"), s.step_path()  # not Q4_0, or rows the kernel does not take
                    continue
                assert family in ("qwen3", "biased", "group3")
            persistent = name in ("token", "persistent") and uniform  # mixed weight types in the layers keep the per-operation kernels
            assert ("kernel on" in s.step_path()) == persistent, s.step_path()
            out = []
            at = 0
            # decode at positions 1.., 63.., 511.. (crossing 512), 641.. and 1123.. (past the 1024 positions up to which
            # the persistent kernel runs attention as one operation)
            for prompt in (1, 62, 448, 130, 480):
                if prompt > 1:
                    s.eval(toks[at:at + prompt - 1])
                    at += prompt - 1
                for _ in range(3):
                    out.append(s.eval(toks[at:at + 1]))
                    st = s.stats()
                    assert st["persistent_steps"] == (1 if persistent else 0)
                    at += 1
            ids, logits = s.generate_greedy(int(toks[at]), 5, want_logits=True)
            assert s.stats()["persistent_steps"] == (5 if persistent else 0)
            out.append(logits)
            out.append(np.asarray(ids, np.float32))
            results[name] = out
    base = "token" if "token" in results else "persistent"
    for other in ("persistent", "per_operation", "batched"):
        if other == base:
            continue
        # the ternary family's F16 head sums lane partials; the batched head kernel may group them differently
        exact = family != "bitnet" or other == "per_operation"
        for a, b in zip(results[base], results[other]):
            if exact:
                assert np.array_equal(a, b), (other, float(np.abs(a - b).max()))
            else:
                assert np.abs(a - b).max() <= 1e-5, (other, float(np.abs(a - b).max()))


def test_one_launch_per_token_at_long_contexts(monkeypatch):
    """The one-launch token kernel past the 1536 positions its value ring holds at once (chunks are refilled behind the
    products) and across further 512-position boundaries, against the per-operation kernels: identical bits, logits and ids."""
    from brisk_llm_b200 import abi
    spec = synth.tiny(synth.QWEN3_0_6B, layers=2, vocab=1024, context=4096)
    m = synth.perturb_norms(synth.generate(spec, seed=21))
    toks = synth.random_tokens(spec, 3700, seed=22)
    results = {}
    for name, flags in (("token", 0), ("per_operation", abi.FLAG_NO_PERSISTENT)):
        monkeypatch.setenv("BRISK_CUDA_TOKEN", "1" if name == "token" else "0")
        with engine.CudaSession(m, flags=flags) as s:
            assert ("one launch per token" in s.step_path()) == (name == "token"), s.step_path()
            out, at = [], 0
            for prompt in (1534, 510, 512, 1100):  # decode at 1534.., 2047.., 2562.., 3665..
                s.eval(toks[at:at + prompt])
                at += prompt
                for _ in range(3):
                    out.append(s.eval(toks[at:at + 1]))
                    at += 1
            ids, logits = s.generate_greedy(int(toks[at]), 4, want_logits=True)
            out += [logits, np.asarray(ids, np.float32)]
            results[name] = out
    for a, b in zip(results["token"], results["per_operation"]):
        assert np.array_equal(a, b), float(np.abs(a - b).max())


def test_default_choice_of_the_single_token_path(monkeypatch):
    """Where the persistent all-layer kernel is measured to be slower (rows wider than 4096 values) or does not apply
    (layer matrices of several types) sessions use one kernel per operation; step_path() says which and why. The
    one-launch token kernel (Q4_0 models of the 0.6B class) is opt-in: measured slower than the persistent kernel."""
    monkeypatch.delenv("BRISK_CUDA_TOKEN", raising=False)
    for spec, expect in ((synth.tiny(synth.QWEN3_0_6B, layers=1, vocab=512), "kernel on: tagged exchange"),
                         (synth.tiny(synth.MISTRAL_7B, layers=1, vocab=512), "off: activation rows wider than 4096"),
                         (synth.tiny(synth.LLAMA_3_2_1B, layers=1, vocab=512), "off: ")):
        with engine.CudaSession(synth.generate(spec, seed=1)) as s:
            assert expect in s.step_path(), s.step_path()
    monkeypatch.setenv("BRISK_CUDA_TOKEN", "1")
    with engine.CudaSession(synth.generate(synth.tiny(synth.QWEN3_0_6B, layers=1, vocab=512), seed=1)) as s:
        assert "kernel on: one launch per token" in s.step_path(), s.step_path()


@pytest.mark.parametrize("family,spec", [
    ("qwen3", synth.tiny(synth.QWEN3_0_6B, layers=2, vocab=512, context=2048)),
    ("mistral", synth.tiny(synth.MISTRAL_7B, layers=1, vocab=512, context=2048)),
])
def test_long_prompt_against_the_oracle(family, spec):
    """A 1300-token prompt: three device batches, the last of which sees more than 1024 positions and takes the
    16-token tiles of the batched attention; then decode steps at that context."""
    m = synth.perturb_norms(synth.generate(spec, seed=21))
    toks = synth.random_tokens(spec, 1310, seed=22)
    o = H.OracleSession(m)
    with engine.CudaSession(m) as s:
        close(s.eval(toks[:1300]), o.eval(toks[:1300]))
        # the residual stream of the prompt's last 20 tokens, bit for bit: the device's last batch holds 1300 - 2 * 512 = 276
        # tokens, the oracle's (CPU chunks of 256) the last 1300 - 5 * 256 = 20
        got = s.debug_buffer("hidden", 276 * spec.hidden).reshape(276, spec.hidden)[256:]
        assert np.array_equal(got, o.debug_buffer("hidden", 20 * spec.hidden).reshape(20, spec.hidden))
        for i in range(1300, 1304):
            close(s.eval(toks[i:i + 1]), o.eval(toks[i:i + 1]))
        close(s.eval_all(toks[1304:1310]), o.eval_all(toks[1304:1310]))
    o.close()


def test_a_wait_that_runs_out_is_reported_and_the_session_carries_on(monkeypatch):
    """Every wait inside the persistent kernel is bounded. A test-only switch makes one operation wait for a tag nobody
    writes, with a limit of a few re-reads: the kernel must still end at once (every access stays in bounds - nothing faults or
    hangs), the call must raise, the position must stay where it was, and the session must go on decoding - through the
    per-operation kernels - with results identical to the oracle's."""
    spec = synth.tiny(synth.QWEN3_0_6B, layers=3, vocab=1024, context=256)
    m = synth.perturb_norms(synth.generate(spec, seed=31))
    toks = synth.random_tokens(spec, 24, seed=32)
    o = H.OracleSession(m)
    monkeypatch.setenv("BRISK_CUDA_TEST_POLL_TIMEOUT", "1")
    monkeypatch.setenv("BRISK_CUDA_TOKEN", "0")
    with engine.CudaSession(m) as s:
        assert "kernel on: tagged exchange" in s.step_path()
        close(s.eval(toks[:16]), o.eval(toks[:16]))  # prompts take the batched kernels: unaffected
        with pytest.raises(RuntimeError, match="timed out"):
            s.eval(toks[16:17])  # one single-token step (not the device greedy loop, which would feed on the garbage)
        assert s.position() == 16
        assert "off: " in s.step_path()
        for i in range(16, 20):  # the same token again, and more: now one kernel per operation
            close(s.eval(toks[i:i + 1]), o.eval(toks[i:i + 1]))
            assert s.stats()["persistent_steps"] == 0
        ids, logits = s.generate_greedy(int(toks[20]), 3, want_logits=True)
        want_ids, want_logits = o.generate_greedy(toks[20:21], 3)
        assert np.array_equal(ids, want_ids) and np.array_equal(logits, want_logits)
    o.close()
    monkeypatch.delenv("BRISK_CUDA_TEST_POLL_TIMEOUT")
    with engine.CudaSession(m) as s:  # the next session has the full limit again
        assert "kernel on: tagged exchange" in s.step_path()
        s.eval(toks[:16])
        s.eval(toks[16:17])
        assert s.stats()["persistent_steps"] == 1
