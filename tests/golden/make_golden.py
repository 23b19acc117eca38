"""Generates tests/golden/*.npz from the UNMODIFIED reference CPU engine (oracle/_ref/libbrisk_ref.so).

Run where a reference checkout is present:  make -C oracle ref && python tests/golden/make_golden.py
(`--family NAME` writes model_NAME.npz of one of MORE_FAMILIES and leaves every other file untouched; so do
`--more-families-only` and `--more-formats-only` for their groups.)
The fixtures pin the C oracle (and through it the CUDA library) on machines that have no reference:
  primitives.npz  f16 conversions, quantize_q8_0 / quantize_q8_k bytes, dequantised rows and matvec/matmul
                  outputs of every format on seeded inputs (the shapes of the reference's kernels_test:
                  1024 columns, 7 tokens, 37 rows)
  model_<family>.npz  logits of prefill / decode / eval_all / rollback, log-likelihood, greedy ids and a
                  speculative run of a tiny seeded model of each family, plus the sha256 of its tensors
"""
import ctypes as C
import hashlib
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
import helpers as H  # noqa: E402
from brisk_llm_b200 import formats as F, gguf_io, synth  # noqa: E402

FAMILIES = {
    "qwen3": synth.tiny(synth.QWEN3_0_6B, hidden=256, heads=4, kv_heads=2, ffn=512, vocab=256),
    "llama": synth.tiny(synth.LLAMA_3_2_1B, hidden=256, heads=8, kv_heads=2, ffn=512, vocab=256),
    "bitnet": synth.tiny(synth.BITNET_2B, hidden=512, heads=4, kv_heads=1, ffn=768, vocab=256),
    "mistral": synth.tiny(synth.MISTRAL_7B, hidden=256, heads=4, kv_heads=2, ffn=512, vocab=256),
}
# Beyond the benchmark configurations (written by `--more-families-only`, which leaves the files above untouched):
# Qwen2-style projection biases, and the remaining weight formats mixed the way stock downloads mix them.
MORE_FAMILIES = {
    "biased": synth.tiny(synth.MISTRAL_7B, hidden=256, heads=4, kv_heads=2, ffn=512, vocab=256, qkv_bias=True, fmt=F.Q8_0),
    "mixed": synth.tiny(synth.QWEN3_0_6B, hidden=256, heads=4, kv_heads=2, ffn=512, vocab=256, tied=False, fmt=F.Q5_K,
                        fmt_overrides={"v": F.Q4_1, "down": F.Q5_0, "embd": F.Q4_1, "output": F.BF16}),
    # Phi-4-mini's layer: partial rotary (96 of 128), scaled cos/sin, short LongRoPE divisors, fused tensors in the file
    "phi3": synth.tiny(synth.MISTRAL_7B, arch="phi3", hidden=384, heads=3, kv_heads=1, head_dim=128, ffn=768, vocab=256,
                       rope_dim=96, rope_attn_factor=1.19, rope_original_context=1024),
    # Qwen2.5's layer: the qwen2 architecture id, biases, 6 query heads per K/V head
    "qwen2": synth.tiny(synth.MISTRAL_7B, arch="qwen2", hidden=384, heads=6, kv_heads=1, head_dim=64, ffn=768, vocab=256, qkv_bias=True),
    # SmolLM3: llama-shaped, the fourth layer attends without RoPE
    "smollm3": synth.tiny(synth.LLAMA_3_2_1B, arch="smollm3", layers=4, hidden=256, heads=8, kv_heads=2, ffn=512, vocab=256),
    # Gemma 3 layers: six sliding layers (window 16) around one global layer, soft-capped logits
    "gemma3": synth.tiny(synth.QWEN3_0_6B, arch="gemma3", layers=7, hidden=256, heads=4, kv_heads=2, ffn=512, vocab=256,
                         sliding_window=16, rope_scaling_factor=8.0, final_softcap=30.0),
}
FORMATS = (F.Q4_0, F.Q8_0, F.Q4_K, F.Q6_K, F.TQ2_0)
MORE_FORMATS = (F.Q4_1, F.Q5_0, F.Q5_K)  # formats the reference reads but the benchmark configurations do not use; in primitives_more.npz


def golden_model(family):
    spec = FAMILIES[family] if family in FAMILIES else MORE_FAMILIES[family]
    return synth.perturb_norms(synth.generate(spec, seed=11), seed=12)


def model_digest(model):
    h = hashlib.sha256()
    for name in sorted(model.tensors):
        h.update(name.encode())
        h.update(np.ascontiguousarray(model.tensors[name][2]).tobytes())
    return h.hexdigest()


def primitive_inputs():
    rng = np.random.default_rng(7)
    x = (rng.standard_normal(1024 * 7) * np.repeat(np.exp(rng.uniform(-3, 3, 7 * 32)), 32)).astype(np.float32)
    x[64:96] = 0.0       # an all-zero block
    x[256:512] = 0.0     # an all-zero super-block
    x[512] = 3.5
    x[513] = -3.5        # equal magnitudes: the first one sets the Q8_K scale's sign
    return x


def format_vectors(r, formats, out):
    """Per format: a seeded matrix, the reference's dequantisation of it, and its products with 1 and 7 activation rows."""
    xs = primitive_inputs().reshape(7, 1024)
    for fmt in formats:
        wb, _ = H.random_matrix(fmt, 37, 1024, seed=100 + fmt)
        deq = np.empty(37 * 1024, np.float32)
        assert r.ref_dequantize(fmt, wb.ctypes.data, H.fptr(deq), deq.size) == 0
        mv = np.empty((1, 37), np.float32)
        mm = np.empty((7, 37), np.float32)
        assert r.ref_matmul(fmt, wb.ctypes.data, 37, 1024, H.fptr(xs[:1].copy()), 1, H.fptr(mv)) == 0
        assert r.ref_matmul(fmt, wb.ctypes.data, 37, 1024, H.fptr(xs), 7, H.fptr(mm)) == 0
        n = F.NAMES[fmt]
        out[f"w_{n}"], out[f"deq_{n}"], out[f"matvec_{n}"], out[f"matmul_{n}"] = wb, deq, mv, mm


def more_formats():
    out = {}
    format_vectors(H.ref(), MORE_FORMATS, out)
    np.savez_compressed(os.path.join(HERE, "primitives_more.npz"), **out)


def main():
    r = H.ref()
    out = {}
    halves = np.arange(65536, dtype=np.uint16)
    out["half_to_float_bits"] = np.array([r.ref_half_to_float(int(h)) for h in halves], np.float32).view(np.uint32)
    rng = np.random.default_rng(5)
    f = (rng.standard_normal(20000) * np.exp(rng.uniform(-25, 13, 20000))).astype(np.float32)
    f[:6] = [1.0 + 1.0 / 2048, 1.0 + 3.0 / 2048, 65520.0, 1e-8, 0.0, -0.0]
    out["float_to_half_in"] = f
    out["float_to_half_out"] = np.array([r.ref_float_to_half(float(v)) for v in f], np.uint16)
    x = primitive_inputs()
    q0 = np.zeros(len(x) // 32 * 34, np.uint8)
    qk = np.zeros(len(x) // 256 * 292, np.uint8)
    r.ref_quantize_q8_0(H.fptr(x), q0.ctypes.data, len(x))
    r.ref_quantize_q8_k(H.fptr(x), qk.ctypes.data, len(x))
    out["q8_0_bytes"], out["q8_k_bytes"] = q0, qk
    # the reference's own known answer (tests/kernels_test.cpp:40-47)
    ka = ((np.arange(32) - 16) * 0.5).astype(np.float32)
    kq = np.zeros(34, np.uint8)
    r.ref_quantize_q8_0(H.fptr(ka), kq.ctypes.data, 32)
    out["q8_0_known_answer"] = kq
    format_vectors(r, FORMATS, out)
    np.savez_compressed(os.path.join(HERE, "primitives.npz"), **out)
    more_formats()

    family_vectors(r, FAMILIES)
    # LookupDrafter known answers (tests/speculative_test.cpp:19-42)
    print("golden written to", HERE)


def family_vectors(r, families):
    for family, spec in families.items():
        m = golden_model(family)
        path = f"/tmp/golden_{family}.gguf"
        gguf_io.write_gguf(m, path)
        s = r.ref_session_create(path.encode(), 4, 0)
        assert s, r.ref_last_error()
        V = spec.vocab
        toks = synth.random_tokens(spec, 48, seed=21)
        g = {"digest": np.frombuffer(model_digest(m).encode(), np.uint8), "tokens": toks}
        buf = np.empty(V, np.float32)
        assert r.ref_session_eval(s, H.iptr(toks[:33]), 33, 0, H.fptr(buf)) == 0
        g["prefill33"] = buf.copy()
        steps = []
        for i in range(33, 37):
            assert r.ref_session_eval(s, H.iptr(toks[i:i + 1]), 1, 0, H.fptr(buf)) == 0
            steps.append(buf.copy())
        g["decode4"] = np.stack(steps)
        allb = np.empty((9, V), np.float32)
        assert r.ref_session_eval(s, H.iptr(toks[37:46]), 9, 1, H.fptr(allb)) == 0
        g["eval_all9"] = allb
        assert r.ref_session_rollback(s, 35) == 0
        assert r.ref_session_eval(s, H.iptr(toks[46:47]), 1, 0, H.fptr(buf)) == 0
        g["after_rollback35"] = buf.copy()
        assert r.ref_session_rollback(s, 0) == 0
        ll = C.c_double()
        assert r.ref_session_log_likelihood(s, H.iptr(toks), 48, C.byref(ll)) == 0
        g["log_likelihood48"] = np.array([ll.value])
        assert r.ref_session_rollback(s, 0) == 0
        ids = np.empty(16, np.int32)
        lg = np.empty((16, V), np.float32)
        assert r.ref_session_generate_greedy(s, H.iptr(toks[:20]), 20, 16, H.iptr(ids), H.fptr(lg), None, None) == 0
        g["greedy16_ids"], g["greedy16_logits"] = ids, lg
        assert r.ref_session_rollback(s, 0) == 0
        rep = np.tile(toks[:8], 4).astype(np.int32)
        sp = np.empty(24, np.int32)
        rounds, acc = C.c_uint64(), C.c_uint64()
        assert r.ref_session_speculate(s, H.iptr(rep), len(rep), 8, 24, H.iptr(sp), C.byref(rounds), C.byref(acc)) == 24
        g["speculate_prompt"], g["speculate24"] = rep, sp
        g["speculate_rounds_accepted"] = np.array([rounds.value, acc.value])
        r.ref_session_destroy(s)
        os.remove(path)
        np.savez_compressed(os.path.join(HERE, f"model_{family}.npz"), **g)
        print(family, "ok", V)


if __name__ == "__main__":
    if "--more-formats-only" in sys.argv:
        more_formats()
    elif "--more-families-only" in sys.argv:
        family_vectors(H.ref(), MORE_FAMILIES)
    elif "--family" in sys.argv:  # one of MORE_FAMILIES, leaving every other file untouched
        name = sys.argv[sys.argv.index("--family") + 1]
        family_vectors(H.ref(), {name: MORE_FAMILIES[name]})
    else:
        main()
