"""The reference's OWN callers of the token loop, over its CPU Session and over CudaSession (the C++ shim a maintainer
adds, brisk_llm_b200/shim/cuda_session.h): Sampler greedy loop, Engine::log_likelihood, Speculator + LookupDrafter, and
the error conditions at the boundary. oracle/_ref/ref_driver is built from a reference checkout (make -C oracle driver)
and travels with the repository's built files; the test is skipped where it is absent."""
import json
import os
import subprocess

import pytest

import helpers as H
from brisk_llm_b200 import gguf_io, synth

pytestmark = pytest.mark.gpu
DRIVER = os.path.join(H.ORACLE_DIR, "_ref", "ref_driver")


@pytest.mark.parametrize("family,spec", [
    ("qwen3", synth.tiny(synth.QWEN3_0_6B, layers=3, vocab=1024, hidden=512, heads=8, kv_heads=4, ffn=1024)),
    ("llama", synth.tiny(synth.LLAMA_3_2_1B, layers=2, vocab=1024, hidden=512, heads=8, kv_heads=2, ffn=1024)),
    ("bitnet", synth.tiny(synth.BITNET_2B, layers=2, vocab=1024, hidden=512, heads=4, kv_heads=1, ffn=768)),
    ("phi3", synth.tiny(synth.MISTRAL_7B, arch="phi3", layers=2, vocab=1024, hidden=384, heads=3, kv_heads=1, head_dim=128, ffn=768,
                        rope_dim=96, rope_attn_factor=1.19, rope_original_context=128)),
    ("qwen2", synth.tiny(synth.MISTRAL_7B, arch="qwen2", layers=2, vocab=1024, hidden=384, heads=6, kv_heads=1, head_dim=64, ffn=768, qkv_bias=True)),
    ("gemma3", synth.tiny(synth.QWEN3_0_6B, arch="gemma3", layers=7, vocab=1024, hidden=512, heads=8, kv_heads=4, ffn=1024,
                          sliding_window=16, rope_scaling_factor=8.0, final_softcap=30.0)),
])
def test_reference_callers_over_cuda_session(family, spec, tmp_path):
    if not os.path.exists(DRIVER):
        pytest.skip("oracle/_ref/ref_driver is not built on this machine")
    model = synth.perturb_norms(synth.generate(spec, seed=17))
    path = str(tmp_path / "m.gguf")
    gguf_io.write_gguf(model, path)
    r = subprocess.run([DRIVER, path, "4", "40", "12", "3"], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, (r.stdout, r.stderr)
    first, second = (json.loads(line) for line in r.stdout.strip().splitlines())
    assert first["greedy_equal"] and first["speculated_equal"]
    assert first["prefill_logits_max_abs_diff"] <= 2e-2
    if family != "bitnet":  # an F16 head sums in another order
        assert first["prefill_logits_bit_equal"]
        assert first["log_likelihood_cpu"] == first["log_likelihood_cuda"]
    else:
        assert abs(first["log_likelihood_cpu"] - first["log_likelihood_cuda"]) < 1e-3
    assert first["spec_rounds"][0] == first["spec_rounds"][1] and first["spec_accepted"][0] == first["spec_accepted"][1]
    assert second["boundary_errors_missing"] == 0
