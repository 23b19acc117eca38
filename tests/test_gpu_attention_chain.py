"""The chained softmax + weighted-sum kernel (csrc/attn_chain.cu) against the kernels it stands in for.

It takes the attention of few tokens (a speculative verify step of 1 + 8 tokens, a short eval_all) and of single tokens at long
contexts. The float operations and their order are the reference's (src/kernels_f32.cpp:265-284), as in the other attention
kernels, so logits must be identical bits whichever kernel ran; the oracle is the arbiter for one of the families.
BRISK_CUDA_CHAIN=0 keeps the older kernels, =1 takes the chained kernel wherever it fits.
"""
import numpy as np
import pytest

import helpers as H
from brisk_llm_b200 import abi, engine, synth

pytestmark = pytest.mark.gpu

FAMILIES = [
    ("qwen3", synth.tiny(synth.QWEN3_0_6B, layers=2, vocab=512, context=2048)),      # 128-wide heads, 2 per K/V head
    ("llama", synth.tiny(synth.LLAMA_3_2_1B, layers=2, vocab=512, context=2048)),    # 64-wide heads, 4 per K/V head
    ("mistral", synth.tiny(synth.MISTRAL_7B, layers=1, vocab=512, context=2048)),    # 128-wide, 4 per K/V head
    ("bitnet", synth.tiny(synth.BITNET_2B, layers=1, vocab=512, context=2048)),      # 20 heads, 4 per K/V head
    ("gemma3", synth.tiny(synth.GEMMA3_1B, layers=7, vocab=512, context=2048, sliding_window=300)),    # 256-wide heads, sliding-window layers
]


def run(model, toks, flags, monkeypatch, chain):
    monkeypatch.setenv("BRISK_CUDA_CHAIN", chain)
    out = []
    with engine.CudaSession(model, flags=flags) as s:
        at = 0
        # contexts: a handful of positions, one product buffer and a bit, several buffers, past a sliding window of 512
        for prompt, batch in ((3, 2), (70, 9), (190, 5), (300, 16), (520, 24), (130, 9), (1, 1), (1, 1)):
            if prompt > 1:
                s.eval(toks[at:at + prompt])
                at += prompt
            if batch == 1:
                out.append(s.eval(toks[at:at + 1]))
            else:
                out.append(s.eval_all(toks[at:at + batch]))
            at += batch
        ids, logits = s.generate_greedy(int(toks[at]), 4, want_logits=True)
        out.append(logits)
        out.append(np.asarray(ids, np.float32))
    return out


@pytest.mark.parametrize("family,spec", FAMILIES, ids=[f for f, _ in FAMILIES])
def test_few_tokens_and_single_tokens_match_the_older_kernels_bit_for_bit(family, spec, monkeypatch):
    m = synth.perturb_norms(synth.generate(spec, seed=41))
    toks = synth.random_tokens(spec, 1400, seed=42)
    # single tokens through one kernel per operation (the persistent kernel has its own attention phase)
    old = run(m, toks, abi.FLAG_NO_PERSISTENT, monkeypatch, "0")
    new = run(m, toks, abi.FLAG_NO_PERSISTENT, monkeypatch, "1")
    for i, (a, b) in enumerate(zip(old, new)):
        assert np.array_equal(a, b), (family, i, float(np.abs(a - b).max()))
    # and with single tokens through the batched kernels too (the path of models with layer variants)
    newer = run(m, toks, abi.FLAG_NO_MEGAKERNEL, monkeypatch, "1")
    exact = family != "bitnet"  # its F16 head sums lane partials; the batched head kernel may group them differently
    for i, (a, b) in enumerate(zip(old, newer)):
        if exact:
            assert np.array_equal(a, b), (family, i, float(np.abs(a - b).max()))
        else:
            assert np.abs(a - b).max() <= 1e-5, (family, i)


def test_verify_steps_against_the_oracle(monkeypatch):
    """eval_all of 1 + 8 tokens and the rollback, as a speculative verify step does, at growing contexts: the oracle's logits."""
    monkeypatch.setenv("BRISK_CUDA_CHAIN", "1")
    spec = synth.tiny(synth.MISTRAL_7B, layers=2, vocab=512, context=1024)
    m = synth.perturb_norms(synth.generate(spec, seed=43))
    toks = synth.random_tokens(spec, 700, seed=44)
    o = H.OracleSession(m)
    with engine.CudaSession(m) as s:
        at = 0
        for prompt in (5, 120, 400):
            got, want = s.eval(toks[at:at + prompt]), o.eval(toks[at:at + prompt])
            at += prompt
            assert np.array_equal(got, want)
            got, want = s.eval_all(toks[at:at + 9]), o.eval_all(toks[at:at + 9])
            assert np.array_equal(got, want), float(np.abs(got - want).max())
            s.rollback(at + 3)
            o.rollback(at + 3)
            at += 3
    o.close()
