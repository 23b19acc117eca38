"""Tensor-parallel token loop on 2, 4 and 8 GPUs (each case skipped where the machine has fewer): every rank holds its
share of every matrix's rows and of the K/V heads - one K/V head per GPU at 8 ranks; the logits every rank returns must
equal the CPU oracle's bit for bit, like the single-GPU path. Single-token steps exchange activations by stores into the
peers' buffers (csrc/tp_peer.cu) or, for comparison, by NCCL all-gathers."""
import os
import subprocess
import sys
import textwrap

import numpy as np
import pytest

import helpers as H

pytestmark = pytest.mark.gpu

WORKER = textwrap.dedent(r'''
    import os, sys, faulthandler
    log = open(os.path.join(sys.argv[2], "rank%s.log" % os.environ.get("RANK", "0")), "w")
    faulthandler.dump_traceback_later(90, exit=True, file=log)   # a stuck rank reports where, then exits
    def mark(what):
        log.write(what + "\n"); log.flush()
    sys.path.insert(0, sys.argv[1]); sys.path.insert(0, os.path.join(sys.argv[1], "tests"))
    import numpy as np
    import torch, torch.distributed as dist
    from brisk_llm_b200 import parallel, synth
    import helpers as H
    rank, local, world = parallel.env_rank()
    torch.cuda.set_device(local)
    dist.init_process_group("gloo")
    if sys.argv[3] == "gemma3":  # post-norms read the gathered projection, the GELU runs on this rank's slice, soft-capped logits
        spec = synth.tiny(synth.QWEN3_0_6B, arch="gemma3", layers=7, vocab=1024, hidden=1024, heads=8, kv_heads=4, ffn=2048, context=512,
                          sliding_window=16, rope_scaling_factor=8.0, final_softcap=30.0)
    else:  # 16 query heads on 8 K/V heads: at 8 ranks every GPU holds one K/V head and its two query heads
        spec = synth.tiny(synth.MISTRAL_7B, layers=2, vocab=1024, hidden=1024, heads=16, kv_heads=8, ffn=2048, context=512)
    model = synth.perturb_norms(synth.generate(spec, seed=4))
    toks = synth.random_tokens(spec, 80, seed=5)
    mark("model ready")
    s = parallel.tensor_parallel_session(model)
    mark("session ready")
    got = [s.eval(toks[:40]).copy()]
    mark("prefill done")
    for i in range(40, 44):
        got.append(s.eval(toks[i:i + 1]).copy())
    mark("single steps done")
    got.append(s.eval_all(toks[44:53]).copy())
    s.rollback(42)
    ids, logits = s.generate_greedy(int(toks[53]), 6, want_logits=True)
    mark("greedy done")
    s.close()
    if rank == 0:
        o = H.OracleSession(model)
        want = [o.eval(toks[:40])]
        for i in range(40, 44):
            want.append(o.eval(toks[i:i + 1]))
        want.append(o.eval_all(toks[44:53]))
        o.rollback(42)
        want_ids, want_logits = o.generate_greedy(toks[53:54], 6)
        for a, b in zip(got, want):
            assert np.array_equal(a, b), float(np.abs(a - b).max())
        assert np.array_equal(ids, want_ids) and np.array_equal(logits, want_logits)
    np.save(os.path.join(sys.argv[2], f"logits{rank}.npy"), got[-1])
    dist.barrier()
    dist.destroy_process_group()
''')


# exchange of single tokens: "peer" = stores into the peers' buffers (the default), "nccl" = all-gathers as for prompts
@pytest.mark.parametrize("family,world,exchange", [("llama", 2, "peer"), ("llama", 2, "nccl"), ("llama", 4, "peer"), ("llama", 8, "peer"),
                                                   ("gemma3", 2, "peer"), ("gemma3", 4, "peer")])
def test_tensor_parallel_matches_the_oracle(family, world, exchange, tmp_path):
    from brisk_llm_b200 import engine
    if engine.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    script = tmp_path / "tp_worker.py"
    script.write_text(WORKER)
    port = 29700 + os.getpid() % 200 + (0 if family == "llama" else 211) + 17 * world + (0 if exchange == "peer" else 7)
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", NCCL_IB_DISABLE="1", NCCL_SOCKET_IFNAME="lo", NCCL_DEBUG="WARN",
               BRISK_CUDA_TP_PEER="1" if exchange == "peer" else "0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
           "--master-port", str(port), str(script), H.ROOT, str(tmp_path), family]
    try:
        r = subprocess.run(cmd, capture_output=True, text=True, timeout=200, env=env)
    except subprocess.TimeoutExpired as e:
        logs = {f: open(tmp_path / f).read() for f in os.listdir(tmp_path) if f.endswith(".log")}
        pytest.fail(f"tensor-parallel workers did not finish: {logs} {str(e.stderr)[-2000:]}")
    logs = {f: open(tmp_path / f).read() for f in os.listdir(tmp_path) if f.endswith(".log")}
    log_dir = os.environ.get("BRISK_TEST_LOG_DIR")
    if r.returncode != 0 and log_dir:
        os.makedirs(log_dir, exist_ok=True)
        with open(os.path.join(log_dir, "tp_test_failure.log"), "w") as f:
            f.write(r.stdout + "\n---- stderr ----\n" + r.stderr + "\n---- rank logs ----\n" + repr(logs))
    assert r.returncode == 0, (logs, r.stdout[-1500:], r.stderr[-3000:])
    a = np.load(tmp_path / "logits0.npy")
    for rank in range(1, world):  # every rank holds the full, identical logits
        assert np.array_equal(a, np.load(tmp_path / f"logits{rank}.npy")), rank
