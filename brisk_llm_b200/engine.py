"""Host-side mirror of brisk-llm's `Engine` interface over the CUDA library's C ABI.

`CudaSession` has the reference interface's members with the same meaning and error behaviour
(brisk-llm src/engine.h:13-37; Session, src/model.cpp:704-751): `eval`, `eval_all` (at most 64
tokens), `rollback`, `position`, `log_likelihood`. Failures raise RuntimeError("cuda: ..."), as the
reference's backends throw std::runtime_error. Every call goes through libbrisk_cuda.so; there is
no other implementation behind this class.
"""
from __future__ import annotations

import ctypes as C
import math

import numpy as np

from . import abi

MAX_SCORED_TOKENS = 64  # Engine::kMaxScoredTokens


class CudaSession:
    def __init__(self, host_model, max_context: int = 0, device: int = 0, flags: int = 0, tp_rank: int = 0, tp_size: int = 1,
                 tp_unique_id: bytes | None = None):
        self._lib = abi.load_library()
        self._h = None
        opts = abi.Options()
        opts.max_context, opts.device, opts.flags = max_context, device, flags
        opts.tp_rank, opts.tp_size = tp_rank, tp_size
        self._uid = C.create_string_buffer(tp_unique_id, 128) if tp_unique_id else None
        opts.tp_unique_id = C.cast(self._uid, C.c_void_p) if self._uid else None
        err = C.create_string_buffer(512)
        self._h = self._lib.brisk_cuda_create(C.byref(host_model.c_model), C.byref(opts), err, len(err))
        if not self._h:
            raise RuntimeError(err.value.decode() or "cuda: session creation failed")
        self.vocab_size = self._lib.brisk_cuda_vocab_size(self._h)
        self.max_context = self._lib.brisk_cuda_max_context(self._h)

    def close(self):
        if self._h:
            self._lib.brisk_cuda_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    def _fail(self):
        raise RuntimeError(self._lib.brisk_cuda_last_error(self._h).decode())

    def _eval(self, tokens, all_logits: bool, copy: bool = True) -> np.ndarray:
        tokens = np.ascontiguousarray(np.atleast_1d(tokens), np.int32)
        out = C.POINTER(C.c_float)()
        if self._lib.brisk_cuda_eval(self._h, tokens.ctypes.data_as(C.POINTER(C.c_int32)), len(tokens), int(all_logits), C.byref(out)) != 0:
            self._fail()
        rows = len(tokens) if all_logits else 1
        view = np.ctypeslib.as_array(out, shape=(rows, self.vocab_size))  # pinned memory of the session
        if copy:
            view = view.copy()
        return view if all_logits else view[0]

    def eval(self, tokens, copy: bool = True) -> np.ndarray:
        """Appends the tokens; logits (vocab floats) for the token after the last one. With copy=False the result is a
        view of the session's pinned buffer, valid only until the session's next call (the reference's contract)."""
        return self._eval(tokens, False, copy)

    def eval_all(self, tokens, copy: bool = True) -> np.ndarray:
        """Like eval(), one row of logits per token; at most 64 tokens."""
        return self._eval(tokens, True, copy)

    def eval_topk(self, tokens, k: int):
        """Appends the tokens like eval(); instead of the logits row, its k best (ids, values) - descending, the lower id
        first among equal values - selected on the device. What a sampler needs after its partial sort (brisk-llm
        src/sampler.cpp:15-46), at k * 8 bytes per token instead of the vocabulary-sized row."""
        tokens = np.ascontiguousarray(np.atleast_1d(tokens), np.int32)
        ids = np.empty(k, np.int32)
        values = np.empty(k, np.float32)
        rc = self._lib.brisk_cuda_eval_topk(self._h, tokens.ctypes.data_as(C.POINTER(C.c_int32)), len(tokens), k,
                                            ids.ctypes.data_as(C.POINTER(C.c_int32)), values.ctypes.data_as(C.POINTER(C.c_float)))
        if rc != 0:
            self._fail()
        return ids, values

    def profile(self, enable: bool = True) -> dict:
        """Per-phase device milliseconds accumulated since the previous call (then cleared); switches profiling on/off."""
        import json
        buf = C.create_string_buffer(2048)
        if self._lib.brisk_cuda_profile(self._h, int(enable), buf, len(buf)) != 0:
            self._fail()
        return json.loads(buf.value.decode())

    def debug_buffer(self, name: str, count: int) -> np.ndarray:
        out = np.empty(count, np.float32)
        if self._lib.brisk_cuda_debug_buffer(self._h, name.encode(), out.ctypes.data_as(C.POINTER(C.c_float)), count) != 0:
            self._fail()
        return out

    def rollback(self, position: int) -> None:
        if self._lib.brisk_cuda_rollback(self._h, position) != 0:
            self._fail()

    def position(self) -> int:
        return self._lib.brisk_cuda_position(self._h)

    def tp_peer_handle(self) -> bytes:
        """64 bytes with which the other ranks of a tensor-parallel group map this rank's exchange buffer."""
        buf = C.create_string_buffer(64)
        if self._lib.brisk_cuda_tp_peer_handle(self._h, buf) != 0:
            self._fail()
        return buf.raw

    def tp_peer_attach(self, handles: bytes) -> None:
        """handles: every rank's tp_peer_handle() in rank order. Single-token steps then exchange by peer stores."""
        if self._lib.brisk_cuda_tp_peer_attach(self._h, handles) != 0:
            self._fail()

    def log_likelihood(self, tokens, chunk: int = MAX_SCORED_TOKENS) -> float:
        """Sum over i >= 1 of log p(tokens[i] | tokens[..i]) (Engine::log_likelihood, src/engine.cpp:10-33)."""
        tokens = np.ascontiguousarray(tokens, np.int32)
        if len(tokens) < 2:
            raise RuntimeError("need at least two tokens to score")
        chunk = max(1, min(int(chunk), MAX_SCORED_TOKENS))
        total = 0.0
        for begin in range(0, len(tokens), chunk):
            part = tokens[begin:begin + chunk]
            logits = self.eval_all(part)
            for t in range(len(part)):
                if begin + t + 1 >= len(tokens):
                    break
                row = logits[t]
                mx = row.max()
                total += float(row[tokens[begin + t + 1]] - mx) - math.log(np.exp((row - mx).astype(np.float64)).sum())
        return total

    def generate_greedy(self, first_token: int, steps: int, want_logits: bool = False):
        """`steps` greedy tokens without a host round trip per token (arg-max on the device, lowest id on ties)."""
        toks = np.empty(steps, np.int32)
        logits = np.empty((steps, self.vocab_size), np.float32) if want_logits else None
        rc = self._lib.brisk_cuda_generate_greedy(self._h, int(first_token), steps, toks.ctypes.data_as(C.POINTER(C.c_int32)),
                                                  logits.ctypes.data_as(C.POINTER(C.c_float)) if want_logits else None)
        if rc != 0:
            self._fail()
        return (toks, logits) if want_logits else toks

    def step_path(self) -> str:
        """How single-token steps run: 'persistent step kernel on: ...' or '... off: <reason>'."""
        buf = C.create_string_buffer(256)
        if self._lib.brisk_cuda_step_path(self._h, buf, len(buf)) != 0:
            self._fail()
        return buf.value.decode()

    def stats(self) -> dict:
        st = abi.Stats()
        self._lib.brisk_cuda_get_stats(self._h, C.byref(st))
        return {k: getattr(st, k) for k, _ in abi.Stats._fields_}


def tp_unique_id() -> bytes:
    """128 bytes identifying one tensor-parallel group; rank 0 makes it and hands it to every rank's CudaSession."""
    lib = abi.load_library()
    buf = C.create_string_buffer(128)
    err = C.create_string_buffer(512)
    if lib.brisk_cuda_tp_unique_id(buf, err, len(err)) != 0:
        raise RuntimeError(err.value.decode())
    return buf.raw


def estimate_memory(host_model, max_context: int = 0, tp_size: int = 1) -> dict:
    """Device bytes a session would hold (weights / cache / scratch), without touching a GPU."""
    lib = abi.load_library()
    opts = abi.Options()
    opts.max_context, opts.tp_size = max_context, tp_size
    mem = abi.Memory()
    if lib.brisk_cuda_estimate_memory(C.byref(host_model.c_model), C.byref(opts), C.byref(mem)) != 0:
        raise RuntimeError("cuda: memory estimate failed")
    return {"weights": mem.weights, "cache": mem.cache, "scratch": mem.scratch, "total": mem.weights + mem.cache + mem.scratch}


def device_count() -> int:
    return abi.load_library().brisk_cuda_device_count()


def matmul(fmt: int, w_bytes: np.ndarray, rows: int, cols: int, x: np.ndarray) -> np.ndarray:
    """out[t][r] = weight row r times activation row t, through the library's test hook (brisk_cuda_matmul)."""
    lib = abi.load_library()
    x = np.ascontiguousarray(x, np.float32).reshape(-1, cols)
    w = np.ascontiguousarray(w_bytes)
    out = np.empty((x.shape[0], rows), np.float32)
    err = C.create_string_buffer(512)
    rc = lib.brisk_cuda_matmul(fmt, w.ctypes.data, rows, cols, x.ctypes.data_as(C.POINTER(C.c_float)), x.shape[0],
                               out.ctypes.data_as(C.POINTER(C.c_float)), err, len(err))
    if rc != 0:
        raise RuntimeError(err.value.decode())
    return out


def matmul_seconds(fmt: int, w_bytes: np.ndarray, rows: int, cols: int, n: int, copies: int, iterations: int) -> float:
    lib = abi.load_library()
    w = np.ascontiguousarray(w_bytes)
    sec = C.c_double()
    err = C.create_string_buffer(512)
    if lib.brisk_cuda_matmul_seconds(fmt, w.ctypes.data, rows, cols, n, copies, iterations, C.byref(sec), err, len(err)) != 0:
        raise RuntimeError(err.value.decode())
    return sec.value
