"""Multi-rank host logic on the CPU: two gloo ranks exchange the tensor-parallel group id the way GPU runs do, and the
row sharding + all-gather re-layout reproduce the unsharded multiply bit for bit (checked with the CPU oracle)."""
import os
import subprocess
import sys
import textwrap

import numpy as np
import pytest

import helpers as H
from brisk_llm_b200 import formats as F, parallel, synth

WORKER = textwrap.dedent('''
    import os, sys
    sys.path.insert(0, sys.argv[1])
    import torch.distributed as dist
    from brisk_llm_b200 import parallel
    dist.init_process_group("gloo")
    rank, local, world = parallel.env_rank()
    payload = bytes(range(128)) if rank == 0 else None
    got = parallel.broadcast_bytes(payload, 128, 0)
    assert got == bytes(range(128)), (rank, got[:8])
    import torch
    t = torch.tensor([float(rank + 1)], dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)   # the bench's max-over-ranks timing reduction
    assert t.item() == world
    dist.barrier()
    open(os.path.join(sys.argv[2], f"rank{rank}.ok"), "w").write("ok")
    dist.destroy_process_group()
''')


def test_two_gloo_ranks_share_the_group_id(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    port = 29500 + os.getpid() % 500
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", str(port), str(script), H.ROOT, str(tmp_path)]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr[-2000:]
    assert (tmp_path / "rank0.ok").exists() and (tmp_path / "rank1.ok").exists()


@pytest.mark.parametrize("fmt", (F.Q4_0, F.Q4_K, F.TQ2_0), ids=lambda f: F.NAMES[f])
@pytest.mark.parametrize("tp", (2, 4))
def test_row_sharding_is_bit_identical(fmt, tp):
    rows, cols, n = 64, 1024, 3
    wb, _ = H.random_matrix(fmt, rows, cols, seed=9)
    x = np.random.default_rng(1).standard_normal((n, cols)).astype(np.float32)
    want = H.oracle_matmul(fmt, wb, rows, cols, x)
    rb = F.row_bytes(fmt, cols)
    parts = []
    for rank in range(tp):
        b, e = parallel.shard_rows(rows, tp, rank)
        parts.append(H.oracle_matmul(fmt, wb[b * rb:e * rb], e - b, cols, x))  # this rank's [n][rows_l]
    gathered = np.stack(parts)  # what an all-gather leaves: [rank][n][rows_l]
    assert np.array_equal(parallel.unpack_gathered(gathered, n, rows // tp, tp), want)


def test_shape_checks():
    parallel.check_tp_shape(synth.MISTRAL_7B, 8)
    with pytest.raises(ValueError):
        parallel.check_tp_shape(synth.BITNET_2B, 2)   # 5 K/V heads
    with pytest.raises(ValueError):
        parallel.shard_rows(10, 4, 0)
