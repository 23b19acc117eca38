"""The C oracle against the unmodified reference engine itself, where oracle/_ref/libbrisk_ref.so exists
(built by `make -C oracle ref` from a reference checkout). Skipped elsewhere; the golden fixtures cover that case."""
import ctypes as C
import os
import tempfile

import numpy as np
import pytest

import helpers as H
from brisk_llm_b200 import formats as F, gguf_io, synth

pytestmark = pytest.mark.skipif(not H.have_ref(), reason="no reference build (oracle/_ref) on this machine")


def test_reference_runs_generic_kernels():
    assert H.ref().ref_kernel_set_name() in (b"generic", b"neon", b"dotprod", b"i8mm")


@pytest.mark.parametrize("fmt", (F.Q4_0, F.Q4_1, F.Q5_0, F.Q8_0, F.Q4_K, F.Q5_K, F.Q6_K, F.TQ2_0), ids=lambda f: F.NAMES[f])
@pytest.mark.parametrize("rows,cols,n", [(36, 1024, 1), (37, 1024, 7), (48, 2048, 3), (5, 256, 2)])
def test_multiply_bit_exact(fmt, rows, cols, n):
    r = H.ref()
    wb, _ = H.random_matrix(fmt, rows, cols, seed=rows * 7 + fmt)
    x = np.random.default_rng(rows + n).standard_normal((n, cols)).astype(np.float32)
    want = np.empty((n, rows), np.float32)
    assert r.ref_matmul(fmt, wb.ctypes.data, rows, cols, H.fptr(x), n, H.fptr(want)) == 0
    assert np.array_equal(H.oracle_matmul(fmt, wb, rows, cols, x), want)


def test_f16_head_bit_exact():
    r = H.ref()
    rng = np.random.default_rng(3)
    w16 = (rng.standard_normal((33, 512)) * 0.02).astype(np.float16)
    x = rng.standard_normal((3, 512)).astype(np.float32)
    want = np.empty((3, 33), np.float32)
    w32 = w16.astype(np.float32)
    r.ref_matmul_f32(H.fptr(w32), 33, 512, H.fptr(x), 3, H.fptr(want))
    assert np.array_equal(H.oracle_matmul(F.F16, w16.view(np.uint8).reshape(-1), 33, 512, x), want)
    assert np.array_equal(H.oracle_matmul(F.F32, w32.view(np.uint8).reshape(-1), 33, 512, x), want)


@pytest.mark.parametrize("family,spec", [
    ("qwen3", synth.tiny(synth.QWEN3_0_6B, hidden=256, heads=4, kv_heads=2, ffn=512, context=512)),
    ("llama", synth.tiny(synth.LLAMA_3_2_1B, hidden=512, heads=8, kv_heads=2, ffn=1024, context=512)),
    ("bitnet", synth.tiny(synth.BITNET_2B, hidden=512, heads=4, kv_heads=1, ffn=768, context=512)),
    ("mistral", synth.tiny(synth.MISTRAL_7B, hidden=256, heads=4, kv_heads=2, ffn=512, layers=3, context=512)),
    # Qwen2-style projection biases on a llama-shaped model (src/model.cpp:411-416, :1026-1030)
    ("biased", synth.tiny(synth.MISTRAL_7B, hidden=256, heads=4, kv_heads=2, ffn=512, context=512, qkv_bias=True, fmt=F.Q8_0)),
    # the formats the reference reads beyond the benchmark configurations, mixed the way stock downloads mix them
    ("mixed", synth.tiny(synth.QWEN3_0_6B, hidden=256, heads=4, kv_heads=2, ffn=512, context=512, tied=False, fmt=F.Q5_K,
                         fmt_overrides={"v": F.Q4_1, "down": F.Q5_0, "embd": F.Q4_1, "output": F.BF16})),
    # Gemma 3: scaled embeddings, post-norms, tanh-GELU, layers 0-4 and 6 slide over 64 positions with their own RoPE base,
    # layer 5 is global with a scaled position, soft-capped logits (src/model.cpp:169-176, :1084-1085, :1116-1119, :1206-1209)
    ("gemma3", synth.tiny(synth.QWEN3_0_6B, arch="gemma3", layers=7, hidden=256, heads=4, kv_heads=2, ffn=512, context=512,
                          sliding_window=64, rope_scaling_factor=8.0, final_softcap=30.0)),
    # Qwen2.5-1.5B's geometry: 6 query heads per K/V head, q/k/v biases, NeoX rotation, no Q/K norms
    ("qwen2", synth.tiny(synth.MISTRAL_7B, arch="qwen2", hidden=384, heads=6, kv_heads=1, head_dim=64, ffn=768, context=512, qkv_bias=True)),
    # Phi-4-mini's layer: fused QKV and gate/up tensors in the file, 3 query heads per K/V head, the first 96 of 128 values
    # rotate, cos/sin scaled, LongRoPE divisors - the long ones (context past the original one) and the short ones
    ("phi3-long", synth.tiny(synth.MISTRAL_7B, arch="phi3", hidden=384, heads=3, kv_heads=1, head_dim=128, ffn=768, context=512,
                             rope_dim=96, rope_attn_factor=1.19, rope_original_context=256)),
    ("phi3-short", synth.tiny(synth.MISTRAL_7B, arch="phi3", hidden=384, heads=3, kv_heads=1, head_dim=128, ffn=768, context=512,
                              rope_dim=96, rope_attn_factor=1.19, rope_original_context=1024)),
    # SmolLM3: llama-shaped, the fourth layer attends without RoPE (src/model.cpp:168, :1024)
    ("smollm3", synth.tiny(synth.LLAMA_3_2_1B, arch="smollm3", layers=5, hidden=512, heads=8, kv_heads=2, ffn=1024, context=512)),
    # Gemma 3's head geometry: 256-wide heads, one K/V head for four query heads
    ("wide-heads", synth.tiny(synth.QWEN3_0_6B, hidden=256, heads=4, kv_heads=1, head_dim=256, ffn=512, context=512)),
])
def test_session_bit_exact(family, spec):
    r = H.ref()
    m = synth.perturb_norms(synth.generate(spec, seed=31))
    with tempfile.TemporaryDirectory() as d:
        path = os.path.join(d, "m.gguf")
        gguf_io.write_gguf(m, path)
        rs = r.ref_session_create(path.encode(), 3, 0)
        assert rs, r.ref_last_error()
        s = H.OracleSession(m)
        toks = synth.random_tokens(spec, 300, seed=2)
        V = spec.vocab
        want = np.empty(V, np.float32)
        # a prompt longer than one CPU batch (256) exercises the reference's chunking
        assert r.ref_session_eval(rs, H.iptr(toks[:270]), 270, 0, H.fptr(want)) == 0
        assert np.array_equal(s.eval(toks[:270]), want)
        wall = np.empty((5, V), np.float32)
        assert r.ref_session_eval(rs, H.iptr(toks[270:275]), 5, 1, H.fptr(wall)) == 0
        assert np.array_equal(s.eval_all(toks[270:275]), wall)
        r.ref_session_rollback(rs, 100)
        s.rollback(100)
        assert r.ref_session_eval(rs, H.iptr(toks[275:276]), 1, 0, H.fptr(want)) == 0
        assert np.array_equal(s.eval(toks[275:276]), want)
        assert s.position() == r.ref_session_position(rs) == 101
        r.ref_session_destroy(rs)
        s.close()


def test_gguf_writer_is_readable_by_the_reference_and_by_us():
    spec = synth.tiny(synth.LLAMA_3_2_1B, hidden=256, heads=8, kv_heads=2, ffn=512)
    m = synth.generate(spec, seed=1)
    with tempfile.TemporaryDirectory() as d:
        path = os.path.join(d, "m.gguf")
        gguf_io.write_gguf(m, path)
        rs = H.ref().ref_session_create(path.encode(), 1, 0)
        assert rs, H.ref().ref_last_error()
        assert H.ref().ref_session_vocab(rs) == spec.vocab
        H.ref().ref_session_destroy(rs)
        back = gguf_io.read_gguf(path)
        assert back.spec.arch == "llama" and back.spec.vocab == spec.vocab and back.spec.head_dim == spec.head_dim
        for name, (fmt, shape, data) in m.tensors.items():
            f2, s2, d2 = back.tensors[name]
            assert f2 == fmt and tuple(s2) == tuple(shape)
            assert np.array_equal(np.asarray(d2).view(np.uint8).ravel(), np.asarray(data).view(np.uint8).ravel())
        assert np.array_equal(back.rope_factors, m.rope_factors)
