"""The C oracle against golden vectors generated from the unmodified reference (tests/golden/make_golden.py).

Bit-exact: the oracle restates the reference's scalar arithmetic, operation for operation.
"""
import ctypes as C
import importlib.util
import os

import numpy as np
import pytest

import helpers as H
from brisk_llm_b200 import formats as F

spec = importlib.util.spec_from_file_location("make_golden", os.path.join(H.GOLDEN, "make_golden.py"))
mg = importlib.util.module_from_spec(spec)
spec.loader.exec_module(mg)

PRIM = dict(np.load(os.path.join(H.GOLDEN, "primitives.npz")))
PRIM.update(np.load(os.path.join(H.GOLDEN, "primitives_more.npz")))


def test_half_conversions():
    o = H.oracle()
    got = np.array([o.oracle_half_to_float(int(h)) for h in range(65536)], np.float32).view(np.uint32)
    assert np.array_equal(got, PRIM["half_to_float_bits"])
    got = np.array([o.oracle_float_to_half(float(v)) for v in PRIM["float_to_half_in"]], np.uint16)
    assert np.array_equal(got, PRIM["float_to_half_out"])
    # the reference's rounding cases (tests/kernels_test.cpp:33-37)
    assert o.oracle_float_to_half(1.0 + 1.0 / 2048) == 0x3C00
    assert o.oracle_float_to_half(1.0 + 3.0 / 2048) == 0x3C02
    assert o.oracle_float_to_half(65520.0) == 0x7C00
    assert o.oracle_float_to_half(1e-8) == 0
    # every non-NaN half survives a round trip (tests/kernels_test.cpp:26-32)
    for h in range(0, 65536, 7):
        f = o.oracle_half_to_float(h)
        if f == f:
            assert o.oracle_float_to_half(f) == h


def test_quantize_known_answer():
    # tests/kernels_test.cpp:40-47: x[i] = (i-16)/2 -> d = half(8/127), q[0] = -127, q[16] = 0, q[31] = 119
    o = H.oracle()
    x = ((np.arange(32) - 16) * 0.5).astype(np.float32)
    out = np.zeros(34, np.uint8)
    o.oracle_quantize_q8_0(H.fptr(x), out.ctypes.data, 32)
    assert np.array_equal(out, PRIM["q8_0_known_answer"])
    q = out[2:].view(np.int8)
    assert out[:2].view(np.uint16)[0] == o.oracle_float_to_half(8.0 / 127)
    assert q[0] == -127 and q[16] == 0 and q[31] == 119


def test_activation_quantisers_bytes():
    o = H.oracle()
    x = mg.primitive_inputs()
    q0 = np.zeros(len(x) // 32 * 34, np.uint8)
    qk = np.zeros(len(x) // 256 * 292, np.uint8)
    o.oracle_quantize_q8_0(H.fptr(x), q0.ctypes.data, len(x))
    o.oracle_quantize_q8_k(H.fptr(x), qk.ctypes.data, len(x))
    assert np.array_equal(q0, PRIM["q8_0_bytes"])
    assert np.array_equal(qk, PRIM["q8_k_bytes"])


@pytest.mark.parametrize("fmt", mg.FORMATS + mg.MORE_FORMATS, ids=lambda f: F.NAMES[f])
def test_dequantize_and_multiply(fmt):
    o = H.oracle()
    n = F.NAMES[fmt]
    wb, _ = H.random_matrix(fmt, 37, 1024, seed=100 + fmt)
    assert np.array_equal(wb, PRIM[f"w_{n}"]), "the seeded test matrix is not reproducible on this numpy"
    deq = np.empty(37 * 1024, np.float32)
    assert o.oracle_dequantize(fmt, wb.ctypes.data, H.fptr(deq), deq.size) == 0
    assert np.array_equal(deq, PRIM[f"deq_{n}"])
    assert np.array_equal(F.dequantize(fmt, wb, deq.size), PRIM[f"deq_{n}"])
    xs = mg.primitive_inputs().reshape(7, 1024)
    assert np.array_equal(H.oracle_matmul(fmt, wb, 37, 1024, xs[:1]), PRIM[f"matvec_{n}"])
    assert np.array_equal(H.oracle_matmul(fmt, wb, 37, 1024, xs), PRIM[f"matmul_{n}"])
    # the reference's own kernel test (tests/kernels_test.cpp:96-184): against a double-precision dot of the
    # dequantised row with the raw activations, tolerance 0.02 + 4*|row|_2*max|x|/254
    ref = xs.astype(np.float64) @ PRIM[f"deq_{n}"].reshape(37, 1024).astype(np.float64).T
    tol = 0.02 + 4 * np.linalg.norm(PRIM[f"deq_{n}"].reshape(37, 1024), axis=1)[None, :] * np.abs(xs).max(axis=1)[:, None] / 254
    assert np.all(np.abs(PRIM[f"matmul_{n}"] - ref) <= tol)


@pytest.mark.parametrize("family", list(mg.FAMILIES) + list(mg.MORE_FAMILIES))
def test_model_golden(family):
    g = np.load(os.path.join(H.GOLDEN, f"model_{family}.npz"))
    m = mg.golden_model(family)
    assert mg.model_digest(m).encode() == g["digest"].tobytes(), "the seeded model is not reproducible on this numpy"
    toks = g["tokens"]
    s = H.OracleSession(m)
    assert np.array_equal(s.eval(toks[:33]), g["prefill33"])
    for i in range(4):
        assert np.array_equal(s.eval(toks[33 + i:34 + i]), g["decode4"][i])
    assert np.array_equal(s.eval_all(toks[37:46]), g["eval_all9"])
    s.rollback(35)
    assert s.position() == 35
    assert np.array_equal(s.eval(toks[46:47]), g["after_rollback35"])
    s.rollback(0)
    assert s.log_likelihood(toks) == g["log_likelihood48"][0]
    s.rollback(0)
    ids, logits = s.generate_greedy(toks[:20], 16)
    assert np.array_equal(ids, g["greedy16_ids"])
    assert np.array_equal(logits, g["greedy16_logits"])
    s.rollback(0)
    out, rounds, acc = s.speculate(g["speculate_prompt"], 8, 24)
    assert np.array_equal(out, g["speculate24"])
    assert [rounds, acc] == list(g["speculate_rounds_accepted"])
    s.close()


def test_lookup_drafter_known_answers():
    # tests/speculative_test.cpp:19-42
    o = H.oracle()

    def draft(history, count):
        h = np.array(history, np.int32)
        out = np.zeros(max(count, 1), np.int32)
        n = o.oracle_lookup_draft(H.iptr(h) if len(h) else None, len(h), count, H.iptr(out))
        return list(out[:n])

    assert draft([], 5) == []
    assert draft([1, 2, 3, 4, 5, 1, 2, 3], 5) == [4, 5, 1, 2, 3]
    assert draft([1, 2, 3, 4, 5, 1, 2, 3], 1) == [4]
    assert draft([7, 8, 9, 7, 8, 10, 7, 8], 3) == [10, 7, 8]
    assert draft([5, 6, 1, 5], 4) == [6, 1, 5]
    assert draft([1, 2, 3], 4) == []


def test_oracle_error_behaviour():
    m = mg.golden_model("qwen3")
    s = H.OracleSession(m, max_context=16)
    with pytest.raises(RuntimeError, match="no tokens"):
        s.eval(np.zeros(0, np.int32))
    with pytest.raises(RuntimeError, match="out of range"):
        s.eval([m.spec.vocab])
    with pytest.raises(RuntimeError, match="eval_all takes 1 to 64"):
        s.eval_all(np.zeros(65, np.int32))
    with pytest.raises(RuntimeError, match="context length exceeded"):
        s.eval(np.zeros(17, np.int32))
    s.eval([1, 2, 3])
    with pytest.raises(RuntimeError, match="cannot roll forward"):
        s.rollback(4)
    s.close()
