"""Host-side pieces that need no GPU: the format encoders, the C ABI library's exported symbols, the build."""
import ctypes as C
import os
import re

import numpy as np
import pytest

import helpers as H
from brisk_llm_b200 import abi, formats as F, synth


@pytest.mark.parametrize("fmt", (F.Q4_0, F.Q4_1, F.Q5_0, F.Q8_0, F.Q4_K, F.Q5_K, F.Q6_K, F.TQ2_0, F.F16, F.BF16), ids=lambda f: F.NAMES[f])
def test_encoders_are_valid_and_close(fmt):
    wb, w = H.random_matrix(fmt, 16, 512, seed=fmt)
    assert wb.nbytes == 16 * F.row_bytes(fmt, 512)
    deq = np.empty(16 * 512, np.float32)
    assert H.oracle().oracle_dequantize(fmt, wb.ctypes.data, H.fptr(deq), deq.size) == 0
    assert np.array_equal(deq, F.dequantize(fmt, wb, deq.size))
    step = {F.Q4_0: 0.02 * 4 / 8, F.Q8_0: 0.02 * 4 / 127, F.Q4_K: 0.02 * 8 / 15, F.Q6_K: 0.02 * 4 / 32, F.TQ2_0: 1e-6, F.F16: 1e-4,
            F.Q4_1: 0.02 * 8 / 15, F.Q5_0: 0.02 * 4 / 16, F.Q5_K: 0.02 * 8 / 31, F.BF16: 1e-3}[fmt]
    assert np.abs(deq - w.ravel()).max() <= step


def test_llama3_rope_factors():
    f = synth.llama3_rope_factors(64, 5e5, 32.0, 1.0, 4.0, 8192)
    assert f.shape == (32,) and f[0] == 1.0 and f[-1] == 32.0
    assert np.all(np.diff(f) >= 0)


def test_weight_bytes_of_the_headline_shape():
    # 28 layers of Q4_0 + tied Q4_0 head + f32 norms (the per-token roofline numerator)
    s = synth.QWEN3_0_6B
    per_layer = (s.q_dim + 2 * s.kv_dim) * s.hidden + s.hidden * s.q_dim + 3 * s.ffn * s.hidden
    total = (s.layers * per_layer + s.vocab * s.hidden) * 18 // 32 + (s.layers * (2 * s.hidden + 2 * s.head_dim) + s.hidden) * 4
    assert total == 335_503_360


def test_library_exports_every_declared_symbol():
    header = open(os.path.join(H.ROOT, "include", "brisk_cuda.h")).read()
    declared = set(re.findall(r"\b(brisk_cuda_[a-z_0-9]+)\s*\(", header))
    assert declared == set(abi.SIGNATURES), declared ^ set(abi.SIGNATURES)
    if not os.path.exists(abi.LIB_PATH):
        from brisk_llm_b200 import build
        build.build()
    lib = C.CDLL(abi.LIB_PATH)
    for name in declared:
        assert hasattr(lib, name), name


def test_missing_library_fails_loudly(tmp_path):
    with pytest.raises(RuntimeError, match="no CPU path"):
        abi.load_library(str(tmp_path / "nope.so"))


def test_struct_sizes_match_the_header():
    # the C compiler's view of the same structs
    import subprocess, tempfile, textwrap
    src = textwrap.dedent('''
        #include <stdio.h>
        #include "brisk_cuda.h"
        int main(void) { printf("%zu %zu %zu %zu %zu\\n", sizeof(brisk_cuda_matrix), sizeof(brisk_cuda_layer), sizeof(brisk_cuda_model),
                                sizeof(brisk_cuda_options), sizeof(brisk_cuda_stats)); return 0; }''')
    with tempfile.TemporaryDirectory() as d:
        c = os.path.join(d, "s.c")
        open(c, "w").write(src)
        subprocess.run(["gcc", "-I", os.path.join(H.ROOT, "include"), c, "-o", os.path.join(d, "s")], check=True)
        got = [int(v) for v in subprocess.run([os.path.join(d, "s")], capture_output=True, text=True, check=True).stdout.split()]
    assert got == [C.sizeof(abi.Matrix), C.sizeof(abi.Layer), C.sizeof(abi.Model), C.sizeof(abi.Options), C.sizeof(abi.Stats)]


def test_lookup_drafter_and_speculator_host_logic():
    from brisk_llm_b200 import speculative
    d = speculative.LookupDrafter()
    assert d.draft(5) == []
    d.observe([1, 2, 3, 4, 5, 1, 2, 3])
    assert d.draft(5) == [4, 5, 1, 2, 3] and d.draft(1) == [4]
    r = speculative.LookupDrafter()
    r.observe([7, 8, 9, 7, 8, 10, 7, 8])
    assert r.draft(3) == [10, 7, 8]
    s1 = speculative.LookupDrafter()
    s1.observe([5, 6, 1, 5])
    assert s1.draft(4) == [6, 1, 5]
    f = speculative.LookupDrafter()
    f.observe([1, 2, 3])
    assert f.draft(4) == []
    # the Speculator over the oracle session settles exactly what the C restatement of the reference loop settles
    import importlib.util
    spec_ = importlib.util.spec_from_file_location("make_golden", os.path.join(H.GOLDEN, "make_golden.py"))
    mg = importlib.util.module_from_spec(spec_)
    spec_.loader.exec_module(mg)
    g = np.load(os.path.join(H.GOLDEN, "model_qwen3.npz"))
    s = H.OracleSession(mg.golden_model("qwen3"))
    got, stats = speculative.speculate(s, g["speculate_prompt"], 8, 24)
    assert np.array_equal(got, g["speculate24"])
    assert [stats["rounds"] + stats["plain"], stats["accepted"]] == list(g["speculate_rounds_accepted"])


def test_device_memory_estimate_needs_no_gpu():
    from brisk_llm_b200 import engine
    spec = synth.tiny(synth.QWEN3_0_6B, layers=2, vocab=1024, context=512)
    m = synth.generate(spec, seed=0)
    e = engine.estimate_memory(m)
    assert e["cache"] == 2 * 2 * spec.kv_dim * 512 * 2  # layers x (K, V) x kv_dim x context x f16
    file_bytes = sum(d.nbytes for n, (f, s, d) in m.tensors.items())
    assert file_bytes <= e["weights"] <= 1.1 * file_bytes + 64 * 256  # planes hold the file's bytes plus alignment padding
    half = engine.estimate_memory(m, max_context=256)
    assert half["cache"] * 2 == e["cache"] and half["scratch"] < e["scratch"]
    tp2 = engine.estimate_memory(m, tp_size=2)
    assert tp2["cache"] * 2 == e["cache"] and tp2["weights"] < e["weights"]


@pytest.mark.parametrize("spec", [
    synth.tiny(synth.MISTRAL_7B, arch="phi3", hidden=384, heads=3, kv_heads=1, head_dim=128, ffn=768, vocab=256, rope_dim=96,
               rope_attn_factor=1.19, rope_original_context=128),
    synth.tiny(synth.QWEN3_0_6B, arch="gemma3", layers=7, hidden=256, heads=4, kv_heads=2, ffn=512, vocab=256, sliding_window=16,
               rope_scaling_factor=8.0, final_softcap=30.0),
    synth.tiny(synth.LLAMA_3_2_1B, arch="smollm3", layers=4, hidden=256, heads=8, kv_heads=2, ffn=512, vocab=256),
    synth.tiny(synth.MISTRAL_7B, arch="qwen2", hidden=384, heads=6, kv_heads=1, head_dim=64, ffn=768, vocab=256, qkv_bias=True),
], ids=lambda s: s.arch)
def test_gguf_round_trip_of_the_layer_variants(spec, tmp_path):
    """What write_gguf puts into a file (Phi's fused QKV and gate/up tensors, Gemma's and Phi's metadata) comes back from
    read_gguf as the same tensors and the same model description."""
    from brisk_llm_b200 import gguf_io
    m = synth.perturb_norms(synth.generate(spec, seed=4))
    path = str(tmp_path / "m.gguf")
    gguf_io.write_gguf(m, path)
    back = gguf_io.read_gguf(path)
    assert set(back.tensors) >= {n for n in m.tensors}
    for name, (fmt, shape, data) in m.tensors.items():
        bf, bs, bd = back.tensors[name]
        assert (bf, tuple(bs)) == (fmt, tuple(shape)), name
        assert np.array_equal(np.asarray(bd).view(np.uint8).reshape(-1), np.ascontiguousarray(data).view(np.uint8).reshape(-1)), name
    a, b = m.c_model, back.c_model
    for field in ("arch", "vocab_size", "hidden", "layer_count", "head_count", "kv_head_count", "head_dim", "ffn", "context_length", "rope_neox",
                  "rope_factor_count", "sliding_window", "gelu", "rope_dim"):
        assert getattr(a, field) == getattr(b, field), field
    for field in ("rope_base", "rms_epsilon", "rope_scale", "rope_base_local", "embedding_scale", "final_softcap", "rope_attn_factor"):
        assert getattr(a, field) == pytest.approx(getattr(b, field)), field
    for i in range(spec.layers):
        assert (a.layers[i].slides, a.layers[i].no_rope) == (b.layers[i].slides, b.layers[i].no_rope)
        assert bool(a.layers[i].attn_post_norm) == bool(b.layers[i].attn_post_norm) and bool(a.layers[i].q_bias) == bool(b.layers[i].q_bias)


def test_memory_estimate_counts_the_gemma_tables():
    """A model whose GELU or soft cap needs the tanh correction table (one 4-bit entry per float of [2^-25, 22)) and a
    second RoPE table for its sliding layers is estimated with them."""
    from brisk_llm_b200 import engine
    plain = synth.tiny(synth.QWEN3_0_6B, layers=2, vocab=1024, context=512)
    gemma = synth.tiny(synth.QWEN3_0_6B, arch="gemma3", layers=2, vocab=1024, context=512, sliding_window=64)
    a, b = engine.estimate_memory(synth.generate(plain, seed=0)), engine.estimate_memory(synth.generate(gemma, seed=0))
    table = (0x41B00000 - 0x33000000) // 2
    rope_local = 512 * plain.head_dim * 4
    staged_projection = 512 * plain.hidden * 4
    assert b["scratch"] - a["scratch"] == table + rope_local + staged_projection
    assert b["weights"] - a["weights"] == 2 * 2 * plain.hidden * 4  # two post-norm vectors per layer


def test_ctypes_mirror_has_the_layout_of_the_c_header(tmp_path):
    """The Python structs are written by hand; a C compiler says what include/brisk_cuda.h really lays out."""
    import subprocess
    names = {"brisk_cuda_matrix": abi.Matrix, "brisk_cuda_layer": abi.Layer, "brisk_cuda_model": abi.Model,
             "brisk_cuda_options": abi.Options, "brisk_cuda_stats": abi.Stats, "brisk_cuda_memory": abi.Memory}
    src = tmp_path / "sizes.c"
    lines = ['#include <stdio.h>', '#include <stddef.h>', '#include "brisk_cuda.h"', 'int main(void) {']
    for n in names:
        lines.append(f'    printf("{n} %zu\\n", sizeof({n}));')
    lines += ['    printf("layer.q_bias %zu\\n", offsetof(brisk_cuda_layer, q_bias));',
              '    printf("model.layers %zu\\n", offsetof(brisk_cuda_model, layers));',
              '    printf("layer.slides %zu\\n", offsetof(brisk_cuda_layer, slides));',
              '    printf("model.gelu %zu\\n", offsetof(brisk_cuda_model, gelu));',
              '    printf("abi %u\\n", (unsigned)BRISK_CUDA_ABI_VERSION);', '    return 0;', '}']
    src.write_text("\n".join(lines))
    exe = tmp_path / "sizes"
    subprocess.run(["gcc", "-I", os.path.join(H.ROOT, "include"), str(src), "-o", str(exe)], check=True)
    out = dict(l.rsplit(" ", 1) for l in subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout.strip().split("\n"))
    for n, cls in names.items():
        assert int(out[n]) == C.sizeof(cls), n
    assert int(out["layer.q_bias"]) == abi.Layer.q_bias.offset
    assert int(out["model.layers"]) == abi.Model.layers.offset
    assert int(out["layer.slides"]) == abi.Layer.slides.offset
    assert int(out["model.gelu"]) == abi.Model.gelu.offset
    assert int(out["abi"]) == abi.ABI_VERSION


def test_bench_helpers_follow_the_workload():
    """The figures bench.py derives without a GPU: counted DRAM traffic of a token, the CPU arm's sample, the clock
    sampler's window."""
    import importlib.util
    import time
    spec_ = importlib.util.spec_from_file_location("bench_module", os.path.join(H.ROOT, "bench.py"))
    bench = importlib.util.module_from_spec(spec_)
    spec_.loader.exec_module(bench)
    spec = synth.PRESETS["qwen3-0.6b-q4_0"]
    # weights once + K and V rows of all layers at the mean context of the decode steps (f16) + one row of logits (f32)
    traffic = bench.analytic_traffic(spec, 1000, 512, 128)
    assert traffic == 1000 + spec.layers * 2 * spec.kv_heads * spec.head_dim * 2 * (512 + 64) + spec.vocab * 4
    # the 0.6B-class model runs its whole workload on the CPU, the 7B-class one a sample
    assert bench.cpu_sample_sizes(spec, 512, 128) == (512, 129)
    big = bench.cpu_sample_sizes(synth.PRESETS["mistral-7b-q4_0"], 8192, 512)
    assert 8 <= big[0] < 64 and 4 <= big[1] < 16
    # clock samples: only lines from the timed region count; a region shorter than the sampling period falls back to all lines
    s = bench.ClockSampler(0)
    s.proc = type("P", (), {"terminate": lambda self: None})()
    now = time.perf_counter()
    s.lines = [(now - 1.0, "1200, 1965, 300.0, Not Active, Not Active, Not Active, Active"),
               (now + 0.5, "1965, 1965, 900.0, Not Active, Not Active, Not Active, Not Active")]
    s.t0 = now
    inside = s.stop()
    assert inside["sm_mhz"] == 1965.0 and inside["reasons"] == [] and inside["samples"] == 1 and inside["window"] == "timed region"
    s.t0 = now + 2.0
    fallback = s.stop()
    assert fallback["samples"] == 2 and fallback["reasons"] == ["sw_power_cap"] and "warm-up" in fallback["window"]
