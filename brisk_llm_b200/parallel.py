"""Host-side plumbing for runs on several GPUs of one node: one process per GPU (torchrun / torch.distributed).

Two modes, as the workloads need them:
  replicas         every rank runs its own independent session (batch-1 decode of one sequence has nothing to shard
                   for the small configurations); nothing is exchanged on the data path
  tensor parallel  the 7B-class configuration: every weight matrix is split by output rows across the ranks
                   (whole heads for q/k/v) and the ranks all-gather activations inside the library (NCCL). Splitting
                   by rows - never by input columns - keeps each output the sum of ALL its input blocks in order on
                   one rank, so the sharded model stays bit-identical to the unsharded one.
The reference is single-process; these helpers have no counterpart there.
"""
from __future__ import annotations

import os

import numpy as np


def env_rank():
    return int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))


def shard_rows(rows: int, tp: int, rank: int) -> tuple[int, int]:
    """Row range [begin, end) of a matrix of `rows` outputs owned by `rank`."""
    if rows % tp != 0:
        raise ValueError(f"{rows} rows do not divide over {tp} ranks")
    per = rows // tp
    return rank * per, (rank + 1) * per


def check_tp_shape(spec, tp: int) -> None:
    """The conditions brisk_cuda_create enforces for a tensor-parallel degree."""
    if spec.kv_heads % tp or spec.vocab % tp or spec.hidden % (32 * tp) or spec.ffn % (32 * tp):
        raise ValueError("the tensor-parallel degree must divide the K/V heads, the vocabulary and (in blocks of 32) the hidden and feed-forward sizes")


def unpack_gathered(gathered: np.ndarray, n: int, rows_l: int, tp: int) -> np.ndarray:
    """What the library does after an all-gather: [rank][token][rows_l] -> [token][rank*rows_l + r]."""
    return np.ascontiguousarray(gathered.reshape(tp, n, rows_l).transpose(1, 0, 2)).reshape(n, tp * rows_l)


def broadcast_bytes(data: bytes | None, size: int, src: int = 0) -> bytes:
    """Broadcast `size` bytes from rank `src` over the default torch.distributed group (any backend)."""
    import torch
    import torch.distributed as dist
    device = "cuda" if dist.get_backend() == "nccl" else "cpu"
    t = torch.zeros(size, dtype=torch.uint8, device=device)
    if dist.get_rank() == src:
        t.copy_(torch.frombuffer(bytearray(data), dtype=torch.uint8))
    dist.broadcast(t, src)
    return bytes(t.cpu().numpy().tobytes())


def tensor_parallel_session(host_model, max_context: int = 0, flags: int = 0):
    """Creates this rank's share of a tensor-parallel session over the default process group (one GPU per rank)."""
    import torch.distributed as dist
    from . import engine
    rank, local, world = env_rank()
    check_tp_shape(host_model.spec, world)
    uid = engine.tp_unique_id() if rank == 0 else None
    uid = broadcast_bytes(uid, 128, 0) if world > 1 else uid
    sess = engine.CudaSession(host_model, max_context=max_context, device=local, flags=flags, tp_rank=rank, tp_size=world, tp_unique_id=uid)
    if world > 1 and os.environ.get("BRISK_CUDA_TP_PEER", "1") != "0":
        # single-token steps exchange by stores into the peers' buffers: every rank publishes a handle of its buffer, all map all
        handles = [None] * world
        dist.all_gather_object(handles, sess.tp_peer_handle())
        sess.tp_peer_attach(b"".join(handles))
        dist.barrier()  # nobody steps before everybody has attached
    return sess
