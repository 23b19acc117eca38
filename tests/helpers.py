"""Test-side loaders of the two CPU checkers (oracle/liboracle.so, oracle/_ref/libbrisk_ref.so) and small utilities.

Only tests, smoke() and bench.py's cpu_baseline leg use these; the product never does.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from brisk_llm_b200 import abi, formats as F  # noqa: E402

ORACLE_DIR = os.path.join(ROOT, "oracle")
ORACLE_LIB = os.path.join(ORACLE_DIR, "liboracle.so")
REF_LIB = os.path.join(ORACLE_DIR, "_ref", "libbrisk_ref.so")
GOLDEN = os.path.join(ROOT, "tests", "golden")

_FP = C.POINTER(C.c_float)
_IP = C.POINTER(C.c_int32)


def fptr(a: np.ndarray):
    assert a.dtype == np.float32 and a.flags.c_contiguous
    return a.ctypes.data_as(_FP)


def iptr(a: np.ndarray):
    assert a.dtype == np.int32 and a.flags.c_contiguous
    return a.ctypes.data_as(_IP)


def build_oracle():
    if not os.path.exists(ORACLE_LIB) or os.path.getmtime(ORACLE_LIB) < os.path.getmtime(os.path.join(ORACLE_DIR, "brisk_oracle.c")):
        subprocess.run(["make", "-C", ORACLE_DIR, "liboracle.so"], check=True, capture_output=True)


_oracle = None


def oracle() -> C.CDLL:
    global _oracle
    if _oracle is None:
        build_oracle()
        lib = C.CDLL(ORACLE_LIB)
        lib.oracle_half_to_float.restype, lib.oracle_half_to_float.argtypes = C.c_float, [C.c_uint16]
        lib.oracle_float_to_half.restype, lib.oracle_float_to_half.argtypes = C.c_uint16, [C.c_float]
        lib.oracle_quantize_q8_0.argtypes = [_FP, C.c_void_p, C.c_uint64]
        lib.oracle_quantize_q8_k.argtypes = [_FP, C.c_void_p, C.c_uint64]
        lib.oracle_dequantize.argtypes = [C.c_int32, C.c_void_p, _FP, C.c_uint64]
        lib.oracle_matmul.argtypes = [C.c_int32, C.c_void_p, C.c_uint64, C.c_uint64, _FP, C.c_uint64, _FP]
        lib.oracle_session_create.restype = C.c_void_p
        lib.oracle_session_create.argtypes = [C.POINTER(abi.Model), C.c_uint64]
        lib.oracle_session_destroy.argtypes = [C.c_void_p]
        lib.oracle_last_error.restype = C.c_char_p
        lib.oracle_session_eval.argtypes = [C.c_void_p, _IP, C.c_uint64, C.c_int, _FP]
        lib.oracle_session_rollback.argtypes = [C.c_void_p, C.c_uint64]
        lib.oracle_session_position.restype, lib.oracle_session_position.argtypes = C.c_uint64, [C.c_void_p]
        lib.oracle_session_log_likelihood.argtypes = [C.c_void_p, _IP, C.c_uint64, C.POINTER(C.c_double)]
        lib.oracle_session_generate_greedy.argtypes = [C.c_void_p, _IP, C.c_uint64, C.c_uint64, _IP, _FP]
        lib.oracle_session_layer_trace.argtypes = [C.c_void_p, _FP]
        lib.oracle_session_debug_buffer.argtypes = [C.c_void_p, C.c_char_p, _FP, C.c_uint64]
        lib.oracle_lookup_draft.restype = C.c_uint64
        lib.oracle_lookup_draft.argtypes = [_IP, C.c_uint64, C.c_uint64, _IP]
        lib.oracle_session_speculate.restype = C.c_int64
        lib.oracle_session_speculate.argtypes = [C.c_void_p, _IP, C.c_uint64, C.c_uint64, C.c_uint64, _IP,
                                                 C.POINTER(C.c_uint64), C.POINTER(C.c_uint64)]
        _oracle = lib
    return _oracle


def have_ref() -> bool:
    return os.path.exists(REF_LIB)


_ref = None


def ref() -> C.CDLL:
    global _ref
    if _ref is None:
        lib = C.CDLL(REF_LIB)
        lib.ref_last_error.restype = C.c_char_p
        lib.ref_kernel_set_name.restype = C.c_char_p
        lib.ref_half_to_float.restype, lib.ref_half_to_float.argtypes = C.c_float, [C.c_uint16]
        lib.ref_float_to_half.restype, lib.ref_float_to_half.argtypes = C.c_uint16, [C.c_float]
        lib.ref_quantize_q8_0.argtypes = [_FP, C.c_void_p, C.c_uint64]
        lib.ref_quantize_q8_k.argtypes = [_FP, C.c_void_p, C.c_uint64]
        lib.ref_dequantize.argtypes = [C.c_int, C.c_void_p, _FP, C.c_uint64]
        lib.ref_matmul.argtypes = [C.c_int, C.c_void_p, C.c_uint64, C.c_uint64, _FP, C.c_uint64, _FP]
        lib.ref_matmul_f32.argtypes = [_FP, C.c_uint64, C.c_uint64, _FP, C.c_uint64, _FP]
        lib.ref_session_create.restype = C.c_void_p
        lib.ref_session_create.argtypes = [C.c_char_p, C.c_uint64, C.c_uint64]
        lib.ref_session_destroy.argtypes = [C.c_void_p]
        lib.ref_session_vocab.restype, lib.ref_session_vocab.argtypes = C.c_uint32, [C.c_void_p]
        lib.ref_session_eval.argtypes = [C.c_void_p, _IP, C.c_uint64, C.c_int, _FP]
        lib.ref_session_rollback.argtypes = [C.c_void_p, C.c_uint64]
        lib.ref_session_position.restype, lib.ref_session_position.argtypes = C.c_uint64, [C.c_void_p]
        lib.ref_session_log_likelihood.argtypes = [C.c_void_p, _IP, C.c_uint64, C.POINTER(C.c_double)]
        lib.ref_session_generate_greedy.argtypes = [C.c_void_p, _IP, C.c_uint64, C.c_uint64, _IP, _FP,
                                                    C.POINTER(C.c_double), C.POINTER(C.c_double)]
        lib.ref_lookup_draft.restype = C.c_uint64
        lib.ref_lookup_draft.argtypes = [_IP, C.c_uint64, C.c_uint64, _IP]
        lib.ref_session_speculate.restype = C.c_int64
        lib.ref_session_speculate.argtypes = [C.c_void_p, _IP, C.c_uint64, C.c_uint64, C.c_uint64, _IP,
                                              C.POINTER(C.c_uint64), C.POINTER(C.c_uint64)]
        if hasattr(lib, "ref_sampler_draws"):
            lib.ref_sampler_draws.argtypes = [_FP, C.c_uint64, C.c_float, C.c_uint32, C.c_float, C.c_uint64, C.c_uint64, _IP]
        _ref = lib
    return _ref


class OracleSession:
    """The oracle behind the Engine-shaped calls (eval / eval_all / rollback / position / log_likelihood)."""

    def __init__(self, host_model, max_context=0):
        self.lib = oracle()
        self.model = host_model
        self.vocab = host_model.spec.vocab
        self.h = self.lib.oracle_session_create(C.byref(host_model.c_model), max_context)

    def close(self):
        if self.h:
            self.lib.oracle_session_destroy(self.h)
            self.h = None

    def __del__(self):
        self.close()

    def _eval(self, tokens, all_logits):
        tokens = np.ascontiguousarray(tokens, np.int32)
        out = np.empty((len(tokens) if all_logits else 1, self.vocab), np.float32)
        if self.lib.oracle_session_eval(self.h, iptr(tokens), len(tokens), int(all_logits), fptr(out)) != 0:
            raise RuntimeError(self.lib.oracle_last_error().decode())
        return out if all_logits else out[0]

    def eval(self, tokens):
        return self._eval(np.atleast_1d(tokens), False)

    def eval_all(self, tokens):
        return self._eval(tokens, True)

    def rollback(self, position):
        if self.lib.oracle_session_rollback(self.h, position) != 0:
            raise RuntimeError(self.lib.oracle_last_error().decode())

    def position(self):
        return self.lib.oracle_session_position(self.h)

    def log_likelihood(self, tokens):
        tokens = np.ascontiguousarray(tokens, np.int32)
        out = C.c_double()
        if self.lib.oracle_session_log_likelihood(self.h, iptr(tokens), len(tokens), C.byref(out)) != 0:
            raise RuntimeError(self.lib.oracle_last_error().decode())
        return out.value

    def generate_greedy(self, prompt, steps, want_logits=True):
        prompt = np.ascontiguousarray(prompt, np.int32)
        toks = np.empty(steps, np.int32)
        logits = np.empty((steps, self.vocab), np.float32) if want_logits else None
        rc = self.lib.oracle_session_generate_greedy(self.h, iptr(prompt), len(prompt), steps, iptr(toks),
                                                     fptr(logits) if want_logits else None)
        if rc != 0:
            raise RuntimeError(self.lib.oracle_last_error().decode())
        return toks, logits

    def layer_trace(self):
        out = np.empty((self.model.spec.layers, self.model.spec.hidden), np.float32)
        self.lib.oracle_session_layer_trace(self.h, fptr(out))
        return out

    def debug_buffer(self, name, count):
        out = np.empty(count, np.float32)
        assert self.lib.oracle_session_debug_buffer(self.h, name.encode(), fptr(out), count) == 0
        return out

    def speculate(self, prompt, draft_tokens, want):
        prompt = np.ascontiguousarray(prompt, np.int32)
        out = np.empty(want, np.int32)
        rounds, acc = C.c_uint64(), C.c_uint64()
        n = self.lib.oracle_session_speculate(self.h, iptr(prompt), len(prompt), draft_tokens, want, iptr(out),
                                              C.byref(rounds), C.byref(acc))
        if n < 0:
            raise RuntimeError(self.lib.oracle_last_error().decode())
        return out, rounds.value, acc.value


def oracle_matmul(fmt, w_bytes, rows, cols, x):
    x = np.ascontiguousarray(x, np.float32).reshape(-1, cols)
    out = np.empty((x.shape[0], rows), np.float32)
    w = np.ascontiguousarray(w_bytes)
    assert oracle().oracle_matmul(fmt, w.ctypes.data, rows, cols, fptr(x), x.shape[0], fptr(out)) == 0
    return out


def random_matrix(fmt, rows, cols, seed=0, std=0.02):
    """f32 ~N(0, std) (ternary: uniform thirds times one scale) quantised to `fmt`: (bytes, f32 source)."""
    rng = np.random.default_rng(seed)
    if fmt == F.TQ2_0:
        w = rng.integers(-1, 2, size=(rows, cols)).astype(np.float32) * np.float32(np.float16(std))
    else:
        w = rng.standard_normal((rows, cols), dtype=np.float32) * np.float32(std)
    return F.quantize(fmt, w), w


def rel_l2(a, b):
    a = np.asarray(a, np.float64).ravel()
    b = np.asarray(b, np.float64).ravel()
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30))


class RefSession:
    """The unmodified reference engine (oracle/_ref/libbrisk_ref.so) behind the same calls as OracleSession. The model
    goes through a GGUF file the reference's own loader parses."""

    def __init__(self, host_model, max_context=0, threads=0):
        import tempfile
        from brisk_llm_b200 import gguf_io
        self.lib = ref()
        self.vocab = host_model.spec.vocab
        fd, self.path = tempfile.mkstemp(suffix=".gguf", prefix="brisk_ref_")
        os.close(fd)
        gguf_io.write_gguf(host_model, self.path)
        self.h = self.lib.ref_session_create(self.path.encode(), threads or (os.cpu_count() or 1), max_context or host_model.spec.context)
        if not self.h:
            os.remove(self.path)
            raise RuntimeError(self.lib.ref_last_error().decode())

    def close(self):
        if self.h:
            self.lib.ref_session_destroy(self.h)
            self.h = None
            os.remove(self.path)

    def __del__(self):
        self.close()

    def _eval(self, tokens, all_logits):
        tokens = np.ascontiguousarray(tokens, np.int32)
        out = np.empty((len(tokens) if all_logits else 1, self.vocab), np.float32)
        if self.lib.ref_session_eval(self.h, iptr(tokens), len(tokens), int(all_logits), fptr(out)) != 0:
            raise RuntimeError(self.lib.ref_last_error().decode())
        return out if all_logits else out[0]

    def eval(self, tokens):
        return self._eval(np.atleast_1d(tokens), False)

    def eval_all(self, tokens):
        return self._eval(tokens, True)

    def rollback(self, position):
        if self.lib.ref_session_rollback(self.h, position) != 0:
            raise RuntimeError(self.lib.ref_last_error().decode())

    def log_likelihood(self, tokens):
        tokens = np.ascontiguousarray(tokens, np.int32)
        out = C.c_double()
        if self.lib.ref_session_log_likelihood(self.h, iptr(tokens), len(tokens), C.byref(out)) != 0:
            raise RuntimeError(self.lib.ref_last_error().decode())
        return out.value

    def generate_greedy(self, prompt, steps, want_logits=True):
        """eval(prompt), then `steps` greedy picks; logits[i] is the row pick i was made from."""
        prompt = np.ascontiguousarray(prompt, np.int32)
        toks = np.empty(steps, np.int32)
        logits = np.empty((steps, self.vocab), np.float32) if want_logits else None
        rc = self.lib.ref_session_generate_greedy(self.h, iptr(prompt), len(prompt), steps, iptr(toks),
                                                  fptr(logits) if want_logits else None, None, None)
        if rc != 0:
            raise RuntimeError(self.lib.ref_last_error().decode())
        return toks, logits


def cpu_checker(host_model, max_context=0):
    """The reference engine itself where it was built (oracle/_ref), else the C restatement on all cores: (session, kind)."""
    if have_ref():
        return RefSession(host_model, max_context), "reference"
    os.environ.setdefault("BRISK_ORACLE_THREADS", str(os.cpu_count() or 1))
    return OracleSession(host_model, max_context), "port"
