"""The k best logits of a row, selected on the device (brisk_cuda_eval_topk), through the C ABI.

A sampling host needs nothing else of the row: the reference sampler orders the candidates by value, keeps top_k of them
and runs its softmax, top-p cut and draw on those (brisk-llm src/sampler.cpp:15-46). So the pairs must be exactly the k
largest of the row the plain eval returns - values bit for bit, descending, the lower id first among equal values - and
the reference's own Sampler, given a row that holds only those pairs, must draw the tokens it draws from the full row."""
import ctypes as C

import numpy as np
import pytest

import helpers as H
from brisk_llm_b200 import engine, synth

pytestmark = pytest.mark.gpu


def expected_topk(row, k):
    order = np.lexsort((np.arange(len(row)), -row.astype(np.float64)))  # by value descending, then id ascending
    return order[:k].astype(np.int32), row[order[:k]]


@pytest.mark.parametrize("vocab,k", [(1000, 1), (4096, 20), (5000, 64), (151936, 20), (151936, 64)])
def test_topk_is_the_top_of_the_row_eval_returns(vocab, k):
    spec = synth.tiny(synth.QWEN3_0_6B, layers=1, vocab=vocab, context=128)
    m = synth.generate(spec, seed=3)
    toks = synth.random_tokens(spec, 12, seed=4)
    with engine.CudaSession(m) as s:
        row = s.eval(toks[:9])
        s.rollback(0)
        ids, values = s.eval_topk(toks[:9], k)
        want_ids, want_values = expected_topk(row, k)
        assert np.array_equal(ids, want_ids) and np.array_equal(values, want_values)
        assert s.stats()["d2h_bytes"] == 8 * k  # k pairs come back, not the row
        # single-token steps take the other kernels: same contract
        row = s.eval(toks[9:10])
        s.rollback(9)
        ids, values = s.eval_topk(toks[9:10], k)
        want_ids, want_values = expected_topk(row, k)
        assert np.array_equal(ids, want_ids) and np.array_equal(values, want_values)
        assert s.position() == 10
        with pytest.raises(RuntimeError, match="top-k takes k"):
            s.eval_topk(toks[10:11], 65)
        assert s.position() == 10


def test_ties_and_nan_order():
    """Equal values keep the lower id in front; a NaN is never ahead of a number (launch_topk through the same entry point:
    a head made of a few distinct rows gives many equal logits)."""
    spec = synth.tiny(synth.QWEN3_0_6B, layers=1, vocab=2048, context=64)
    m = synth.generate(spec, seed=5)
    fmt, shape, data = m.tensors["token_embd.weight"]
    rows = data.reshape(shape[0], -1)
    rows[8:] = rows[np.arange(8, shape[0]) % 8]  # every logit value appears 256 times
    with engine.CudaSession(synth.HostModel(spec, m.tensors, m.rope_factors)) as s:
        toks = synth.random_tokens(spec, 5, seed=6)
        row = s.eval(toks)
        assert len(np.unique(row)) <= 8
        s.rollback(0)
        ids, values = s.eval_topk(toks, 40)
        want_ids, want_values = expected_topk(row, 40)
        assert np.array_equal(ids, want_ids) and np.array_equal(values, want_values)


@pytest.mark.skipif(not H.have_ref() or not hasattr(H.ref(), "ref_sampler_draws"), reason="needs the reference build (oracle/_ref) with its Sampler")
def test_the_reference_sampler_draws_the_same_tokens_from_the_pairs():
    spec = synth.tiny(synth.QWEN3_0_6B, layers=2, vocab=32000, context=128)
    m = synth.generate(spec, seed=7)
    toks = synth.random_tokens(spec, 20, seed=8)
    r = H.ref()
    with engine.CudaSession(m) as s:
        for step, (temperature, top_k, top_p) in enumerate([(0.8, 20, 0.95), (1.3, 40, 0.5), (0.7, 64, 1.0)]):
            row = s.eval(toks[:10 + step])
            s.rollback(0)
            ids, values = s.eval_topk(toks[:10 + step], top_k)
            s.rollback(0)
            assert len(np.unique(values)) == top_k  # distinct values: the partial sort's order among equals is unspecified
            sparse = np.full(spec.vocab, -np.inf, np.float32)
            sparse[ids] = values
            a, b = np.empty(200, np.int32), np.empty(200, np.int32)
            assert r.ref_sampler_draws(H.fptr(np.ascontiguousarray(row)), spec.vocab, temperature, top_k, top_p, 1234 + step, 200, H.iptr(a)) == 0
            assert r.ref_sampler_draws(H.fptr(sparse), spec.vocab, temperature, top_k, top_p, 1234 + step, 200, H.iptr(b)) == 0
            assert np.array_equal(a, b)
            assert len(set(a.tolist())) > 3  # it really samples
