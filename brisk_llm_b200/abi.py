"""ctypes mirror of include/brisk_cuda.h and the loader of the in-tree CUDA library.

The product path is libbrisk_cuda.so only. Loading fails loudly when the library has not been
built (`python -m brisk_llm_b200.build`), and nothing here falls back to a CPU implementation.
"""
from __future__ import annotations

import ctypes as C
import os

ABI_VERSION = 4
PKG_DIR = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(PKG_DIR, "libbrisk_cuda.so")

ARCH_QWEN3, ARCH_LLAMA, ARCH_BITNET, ARCH_GEMMA3 = 0, 1, 2, 3
ARCH_BY_NAME = {"qwen3": ARCH_QWEN3, "llama": ARCH_LLAMA, "bitnet": ARCH_BITNET, "bitnet-b1.58": ARCH_BITNET, "gemma3": ARCH_GEMMA3,
                "smollm3": ARCH_LLAMA,
                "qwen2": ARCH_QWEN3,
                "phi3": ARCH_QWEN3}  # Phi-3/4-mini: NeoX rotation of the first rope_dim values, no Q/K norms  # Qwen2/2.5: the Qwen3 layer without Q/K norms, with q/k/v biases  # llama-shaped; its layers without RoPE are flagged per layer
FLAG_NO_GRAPH, FLAG_NO_MEGAKERNEL, FLAG_NO_PERSISTENT = 1, 2, 4


class Matrix(C.Structure):
    _fields_ = [("type", C.c_int32), ("reserved", C.c_int32), ("rows", C.c_uint64), ("cols", C.c_uint64),
                ("data", C.c_void_p), ("bytes", C.c_uint64)]


_FP = C.POINTER(C.c_float)


class Layer(C.Structure):
    _fields_ = [("attn_norm", _FP), ("q", Matrix), ("k", Matrix), ("v", Matrix), ("q_norm", _FP), ("k_norm", _FP),
                ("attn_sub_norm", _FP), ("o", Matrix), ("ffn_norm", _FP), ("gate", Matrix), ("up", Matrix),
                ("ffn_sub_norm", _FP), ("down", Matrix), ("q_bias", _FP), ("k_bias", _FP), ("v_bias", _FP),
                ("attn_post_norm", _FP), ("ffn_post_norm", _FP), ("slides", C.c_int32), ("no_rope", C.c_int32)]


class Model(C.Structure):
    _fields_ = [("abi_version", C.c_uint32), ("arch", C.c_int32), ("vocab_size", C.c_uint32), ("hidden", C.c_uint32),
                ("layer_count", C.c_uint32), ("head_count", C.c_uint32), ("kv_head_count", C.c_uint32),
                ("head_dim", C.c_uint32), ("ffn", C.c_uint32), ("context_length", C.c_uint32),
                ("rope_base", C.c_float), ("rms_epsilon", C.c_float), ("rope_neox", C.c_int32),
                ("rope_factor_count", C.c_uint32), ("rope_factors", _FP), ("token_embd", Matrix), ("output", Matrix),
                ("output_norm", _FP), ("layers", C.POINTER(Layer)),
                ("rope_scale", C.c_float), ("rope_base_local", C.c_float), ("sliding_window", C.c_uint32),
                ("embedding_scale", C.c_float), ("final_softcap", C.c_float), ("gelu", C.c_int32),
                ("rope_dim", C.c_uint32), ("rope_attn_factor", C.c_float)]


class Options(C.Structure):
    _fields_ = [("max_context", C.c_uint64), ("device", C.c_int32), ("tp_rank", C.c_int32), ("tp_size", C.c_int32),
                ("flags", C.c_uint32), ("tp_unique_id", C.c_void_p)]


class Stats(C.Structure):
    _fields_ = [("device_ms", C.c_double), ("kernel_launches", C.c_uint64), ("weight_bytes", C.c_uint64),
                ("kv_bytes", C.c_uint64), ("h2d_bytes", C.c_uint64), ("d2h_bytes", C.c_uint64),
                ("persistent_steps", C.c_uint64)]


class Memory(C.Structure):
    _fields_ = [("weights", C.c_uint64), ("cache", C.c_uint64), ("scratch", C.c_uint64)]


# Every symbol include/brisk_cuda.h declares, with its ctypes signature.
SIGNATURES = {
    "brisk_cuda_device_count": (C.c_int, []),
    "brisk_cuda_step_path": (C.c_int, [C.c_void_p, C.c_char_p, C.c_size_t]),
    "brisk_cuda_estimate_memory": (C.c_int, [C.POINTER(Model), C.POINTER(Options), C.POINTER(Memory)]),
    "brisk_cuda_create": (C.c_void_p, [C.POINTER(Model), C.POINTER(Options), C.c_char_p, C.c_size_t]),
    "brisk_cuda_destroy": (None, [C.c_void_p]),
    "brisk_cuda_eval": (C.c_int, [C.c_void_p, C.POINTER(C.c_int32), C.c_uint64, C.c_int, C.POINTER(_FP)]),
    "brisk_cuda_eval_topk": (C.c_int, [C.c_void_p, C.POINTER(C.c_int32), C.c_uint64, C.c_uint32, C.POINTER(C.c_int32), _FP]),
    "brisk_cuda_rollback": (C.c_int, [C.c_void_p, C.c_uint64]),
    "brisk_cuda_position": (C.c_uint64, [C.c_void_p]),
    "brisk_cuda_vocab_size": (C.c_uint32, [C.c_void_p]),
    "brisk_cuda_max_context": (C.c_uint64, [C.c_void_p]),
    "brisk_cuda_last_error": (C.c_char_p, [C.c_void_p]),
    "brisk_cuda_generate_greedy": (C.c_int, [C.c_void_p, C.c_int32, C.c_uint64, C.POINTER(C.c_int32), _FP]),
    "brisk_cuda_get_stats": (C.c_int, [C.c_void_p, C.POINTER(Stats)]),
    "brisk_cuda_matmul": (C.c_int, [C.c_int32, C.c_void_p, C.c_uint64, C.c_uint64, _FP, C.c_uint64, _FP, C.c_char_p, C.c_size_t]),
    "brisk_cuda_matmul_seconds": (C.c_int, [C.c_int32, C.c_void_p, C.c_uint64, C.c_uint64, C.c_uint64, C.c_uint32,
                                            C.c_uint32, C.POINTER(C.c_double), C.c_char_p, C.c_size_t]),
    "brisk_cuda_argmax_static": (C.c_int, [C.c_void_p, C.c_uint32, C.c_uint32, C.c_void_p, C.c_void_p, C.c_char_p, C.c_size_t]),
    "brisk_cuda_profile": (C.c_int, [C.c_void_p, C.c_int, C.c_char_p, C.c_size_t]),
    "brisk_cuda_debug_buffer": (C.c_int, [C.c_void_p, C.c_char_p, _FP, C.c_uint64]),
    "brisk_cuda_tp_unique_id": (C.c_int, [C.c_void_p, C.c_char_p, C.c_size_t]),
    "brisk_cuda_tp_peer_handle": (C.c_int, [C.c_void_p, C.c_void_p]),
    "brisk_cuda_tp_peer_attach": (C.c_int, [C.c_void_p, C.c_void_p]),
}

_lib = None


def load_library(path: str | None = None) -> C.CDLL:
    """dlopen the CUDA library and attach signatures. Raises if it is missing: there is no other path."""
    global _lib
    if _lib is not None and path is None:
        return _lib
    p = path or LIB_PATH
    if not os.path.exists(p):
        raise RuntimeError(f"cuda: {p} is not built - run `python -m brisk_llm_b200.build` (nvcc, sm_100a); "
                           "this backend has no CPU path")
    lib = C.CDLL(p)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    if path is None:
        _lib = lib
    return lib
