"""Seeded synthetic models with the shapes of the benchmark configurations.

Real checkpoints cannot be fetched, so the workloads run on random weights with the named
architecture's shapes and value distributions: f32 ~N(0, 0.02) quantised to the configured format,
norm weights 1.0, ternary weights uniform over {-1, 0, 1} times one per-tensor scale. A HostModel
holds the tensors as file-layout bytes (what a GGUF holds) and hands them to the C ABI
(include/brisk_cuda.h) and, in tests, to the CPU oracle through the same structs.
"""
from __future__ import annotations

import ctypes as C
import math
from dataclasses import dataclass, field, replace

import numpy as np

from . import abi, formats as F


@dataclass(frozen=True)
class ModelSpec:
    name: str
    arch: str  # "qwen3" | "qwen2" | "llama" | "bitnet" | "gemma3" | "smollm3" | "phi3"
    layers: int
    hidden: int
    heads: int
    kv_heads: int
    head_dim: int
    ffn: int
    vocab: int
    context: int
    rope_base: float
    eps: float = 1e-6
    tied: bool = True
    fmt: int = F.Q4_0  # default matrix format
    fmt_overrides: dict = field(default_factory=dict)  # role -> format, roles: q k v o gate up down embd output
    llama3_rope: tuple | None = None  # (factor, low_freq_factor, high_freq_factor, original_context)
    std: float = 0.02
    qkv_bias: bool = False  # Qwen2-style projection biases (src/model.cpp:411-416)
    # Gemma 3 (src/model.cpp:169-176): window of the sliding layers (every layer whose index is not 5 mod 6), their RoPE
    # base, the file's rope.scaling.factor for the global layers, the soft cap of the logits
    sliding_window: int = 0
    rope_base_local: float = 10000.0
    rope_scaling_factor: float = 1.0
    final_softcap: float = 0.0
    # Phi-3 / Phi-4-mini (src/model.cpp:177-188): values of a head that rotate (0: all), the factor on cos and sin, and the
    # context up to which the short LongRoPE divisors apply (0: no divisors)
    rope_dim: int = 0
    rope_attn_factor: float = 1.0
    rope_original_context: int = 0

    def layer_has_rope(self, layer: int) -> bool:
        """SmolLM3: every fourth layer attends without positional rotation (src/model.cpp:168, src/model.h:97-110)."""
        return self.arch != "smollm3" or (layer + 1) % 4 != 0

    def layer_slides(self, layer: int) -> bool:
        return self.arch == "gemma3" and self.sliding_window != 0 and layer % 6 != 5

    def fmt_of(self, role: str) -> int:
        return self.fmt_overrides.get(role, self.fmt)

    @property
    def q_dim(self):
        return self.heads * self.head_dim

    @property
    def kv_dim(self):
        return self.kv_heads * self.head_dim


# The benchmark configurations (shapes of Qwen3-0.6B, Llama-3.2-1B, BitNet-b1.58-2B4T, Mistral-7B-v0.3).
QWEN3_0_6B = ModelSpec("qwen3-0.6b-q4_0", "qwen3", 28, 1024, 16, 8, 128, 3072, 151936, 2048, 1e6, 1e-6, True, F.Q4_0)
LLAMA_3_2_1B = ModelSpec("llama-3.2-1b-q4_k_m", "llama", 16, 2048, 32, 8, 64, 8192, 128256, 4096, 5e5, 1e-5, True, F.Q4_K,
                         {"v": F.Q6_K, "down": F.Q6_K, "embd": F.Q6_K}, (32.0, 1.0, 4.0, 8192))
BITNET_2B = ModelSpec("bitnet-2b4t-tq2_0", "bitnet", 30, 2560, 20, 5, 128, 6912, 128256, 4096, 5e5, 1e-5, True, F.TQ2_0,
                      {"embd": F.F16})
MISTRAL_7B = ModelSpec("mistral-7b-q4_0", "llama", 32, 4096, 32, 8, 128, 14336, 32768, 8704, 1e6, 1e-5, False, F.Q4_0)
# Beyond the benchmark configurations: the shape of Gemma-3-1B (256-wide heads, five sliding layers per global one).
GEMMA3_1B = ModelSpec("gemma3-1b-q4_0", "gemma3", 26, 1152, 4, 1, 256, 6912, 262144, 4096, 1e6, 1e-6, True, F.Q4_0,
                      sliding_window=512, rope_base_local=10000.0, rope_scaling_factor=1.0, final_softcap=0.0)
PRESETS = {s.name: s for s in (QWEN3_0_6B, LLAMA_3_2_1B, BITNET_2B, MISTRAL_7B, GEMMA3_1B)}


def tiny(spec: ModelSpec, layers=2, vocab=512, context=256, **kw) -> ModelSpec:
    """A few-layer, small-vocabulary model of the same family and head geometry, for parity tests."""
    return replace(spec, name=spec.name + "-tiny", layers=layers, vocab=vocab, context=context, **kw)


def llama3_rope_factors(head_dim: int, base: float, factor: float, low: float, high: float, orig_ctx: int) -> np.ndarray:
    """Per-frequency divisors of the RoPE angle for Llama-3 long-context scaling. The reference does not
    compute these: it reads them from the file's rope_freqs.weight (brisk-llm src/model.cpp:314-318)."""
    out = np.empty(head_dim // 2, np.float32)
    low_wavelen, high_wavelen = orig_ctx / low, orig_ctx / high
    for i in range(head_dim // 2):
        freq = base ** (-2.0 * i / head_dim)
        wavelen = 2 * math.pi / freq
        if wavelen < high_wavelen:
            out[i] = 1.0
        elif wavelen > low_wavelen:
            out[i] = factor
        else:
            smooth = (orig_ctx / wavelen - low) / (high - low)
            out[i] = 1.0 / ((1 - smooth) / factor + smooth)
    return out


class HostModel:
    """Tensors of one model in host memory (file layout) + the ctypes description of them."""

    def __init__(self, spec: ModelSpec, tensors: dict[str, tuple[int, tuple[int, int], np.ndarray]], rope_factors=None):
        self.spec = spec
        self.tensors = tensors  # name -> (format, (rows, cols), uint8 bytes or f32 vector)
        self.rope_factors = rope_factors
        self._keep = []
        self.c_model = self._describe()

    def matrix(self, name: str):
        return self.tensors[name]

    def _mat(self, name: str) -> abi.Matrix:
        fmt, (rows, cols), data = self.tensors[name]
        m = abi.Matrix()
        m.type, m.rows, m.cols = fmt, rows, cols
        m.data = data.ctypes.data
        m.bytes = data.nbytes
        return m

    def _vec(self, name: str):
        if name not in self.tensors:
            return None
        v = self.tensors[name][2]
        assert v.dtype == np.float32
        return v.ctypes.data_as(C.POINTER(C.c_float))

    def _describe(self) -> abi.Model:
        s = self.spec
        layers = (abi.Layer * s.layers)()
        for i in range(s.layers):
            p = f"blk.{i}."
            L = layers[i]
            L.attn_norm = self._vec(p + "attn_norm.weight")
            L.q, L.k, L.v = self._mat(p + "attn_q.weight"), self._mat(p + "attn_k.weight"), self._mat(p + "attn_v.weight")
            L.q_norm = self._vec(p + "attn_q_norm.weight")
            L.k_norm = self._vec(p + "attn_k_norm.weight")
            L.attn_sub_norm = self._vec(p + "attn_sub_norm.weight")
            L.o = self._mat(p + "attn_output.weight")
            L.ffn_norm = self._vec(p + "ffn_norm.weight")
            L.gate, L.up = self._mat(p + "ffn_gate.weight"), self._mat(p + "ffn_up.weight")
            L.ffn_sub_norm = self._vec(p + "ffn_sub_norm.weight")
            L.down = self._mat(p + "ffn_down.weight")
            L.q_bias, L.k_bias, L.v_bias = self._vec(p + "attn_q.bias"), self._vec(p + "attn_k.bias"), self._vec(p + "attn_v.bias")
            L.attn_post_norm, L.ffn_post_norm = self._vec(p + "post_attention_norm.weight"), self._vec(p + "post_ffw_norm.weight")
            L.slides = 1 if s.layer_slides(i) else 0
            L.no_rope = 0 if s.layer_has_rope(i) else 1
        m = abi.Model()
        m.abi_version = abi.ABI_VERSION
        m.arch = abi.ARCH_BY_NAME[s.arch]
        m.vocab_size, m.hidden, m.layer_count = s.vocab, s.hidden, s.layers
        m.head_count, m.kv_head_count, m.head_dim, m.ffn = s.heads, s.kv_heads, s.head_dim, s.ffn
        m.context_length = s.context
        m.rope_base, m.rms_epsilon = s.rope_base, s.eps
        m.rope_neox = 0 if s.arch in ("llama", "smollm3") else 1  # brisk-llm src/model.cpp:167
        if s.arch == "phi3":
            m.rope_dim, m.rope_attn_factor = s.rope_dim, s.rope_attn_factor
            if "rope_factors_short.weight" in self.tensors:  # a session picks by its context (src/model.cpp:691-694)
                which = "rope_factors_long.weight" if s.context > s.rope_original_context else "rope_factors_short.weight"
                self.rope_factors = self.tensors[which][2]
        if self.rope_factors is not None:
            m.rope_factor_count = len(self.rope_factors)
            m.rope_factors = self.rope_factors.ctypes.data_as(C.POINTER(C.c_float))
        if s.arch == "gemma3":
            m.rope_scale = float(np.float32(1.0) / np.float32(s.rope_scaling_factor))
            m.rope_base_local, m.sliding_window = s.rope_base_local, s.sliding_window
            m.embedding_scale = float(np.sqrt(np.float32(s.hidden)))
            m.final_softcap, m.gelu = s.final_softcap, 1
        m.token_embd = self._mat("token_embd.weight")
        if "output.weight" in self.tensors:
            m.output = self._mat("output.weight")
        m.output_norm = self._vec("output_norm.weight")
        m.layers = layers
        self._keep.append(layers)
        return m

    def weight_bytes(self) -> int:
        """Bytes one decoded token must read: every matrix once (the tied head counts once, as the head;
        the embedding lookup reads one row) plus the f32 norm vectors."""
        total = 0
        for name, (fmt, shape, data) in self.tensors.items():
            if name == "token_embd.weight" and "output.weight" in self.tensors:
                continue
            total += data.nbytes
        return total


def generate(spec: ModelSpec, seed: int = 0, share_layers: bool = False) -> HostModel:
    """Draw the weights. With share_layers every layer reuses layer 0's tensors (same shapes and
    distributions, a fraction of the generation time) - for throughput runs of the largest shape only."""
    rng = np.random.default_rng(seed)
    t: dict = {}

    def ones(name, n):
        t[name] = (F.F32, (1, n), np.ones(n, np.float32))

    def matrix(name, role, rows, cols):
        fmt = spec.fmt_of(role)
        if fmt == F.TQ2_0:
            w = rng.integers(-1, 2, size=(rows, cols), dtype=np.int8).astype(np.float32)
            scale = np.float32(np.float16(spec.std * math.sqrt(1.5)))
            # a +-1 in every block keeps the encoder's per-block scale at exactly `scale`
            w[:, ::256] = np.where(w[:, ::256] == 0, 1, w[:, ::256])
            w *= scale
        else:
            w = rng.standard_normal((rows, cols), dtype=np.float32) * np.float32(spec.std)
        t[name] = (fmt, (rows, cols), F.quantize(fmt, w))

    matrix("token_embd.weight", "embd", spec.vocab, spec.hidden)
    if not spec.tied:
        matrix("output.weight", "output", spec.vocab, spec.hidden)
    ones("output_norm.weight", spec.hidden)
    if spec.arch == "phi3" and spec.rope_original_context:
        half = (spec.rope_dim or spec.head_dim) // 2
        t["rope_factors_short.weight"] = (F.F32, (1, half), (1.0 + 0.05 * rng.random(half)).astype(np.float32))
        t["rope_factors_long.weight"] = (F.F32, (1, half), (1.0 + 3.0 * rng.random(half)).astype(np.float32))
    for i in range(spec.layers):
        p = f"blk.{i}."
        if share_layers and i > 0:
            for k in [k for k in t if k.startswith("blk.0.")]:
                t[p + k[len("blk.0."):]] = t[k]
            continue
        ones(p + "attn_norm.weight", spec.hidden)
        matrix(p + "attn_q.weight", "q", spec.q_dim, spec.hidden)
        matrix(p + "attn_k.weight", "k", spec.kv_dim, spec.hidden)
        matrix(p + "attn_v.weight", "v", spec.kv_dim, spec.hidden)
        if spec.qkv_bias:
            for nm, size in (("attn_q.bias", spec.q_dim), ("attn_k.bias", spec.kv_dim), ("attn_v.bias", spec.kv_dim)):
                t[p + nm] = (F.F32, (1, size), (rng.standard_normal(size) * 0.05).astype(np.float32))
        if spec.arch in ("qwen3", "gemma3"):
            ones(p + "attn_q_norm.weight", spec.head_dim)
            ones(p + "attn_k_norm.weight", spec.head_dim)
        if spec.arch == "bitnet":
            ones(p + "attn_sub_norm.weight", spec.q_dim)
            ones(p + "ffn_sub_norm.weight", spec.ffn)
        matrix(p + "attn_output.weight", "o", spec.hidden, spec.q_dim)
        if spec.arch == "gemma3":
            ones(p + "post_attention_norm.weight", spec.hidden)
            ones(p + "post_ffw_norm.weight", spec.hidden)
        ones(p + "ffn_norm.weight", spec.hidden)
        matrix(p + "ffn_gate.weight", "gate", spec.ffn, spec.hidden)
        matrix(p + "ffn_up.weight", "up", spec.ffn, spec.hidden)
        matrix(p + "ffn_down.weight", "down", spec.hidden, spec.ffn)
    factors = None
    if spec.llama3_rope is not None:
        f, lo, hi, oc = spec.llama3_rope
        factors = llama3_rope_factors(spec.head_dim, spec.rope_base, f, lo, hi, oc)
    return HostModel(spec, t, factors)


def perturb_norms(model: HostModel, seed: int = 1) -> HostModel:
    """Replace the all-ones norm vectors by 1 + N(0, 0.1), so that tests also catch a norm weight that is
    skipped or applied to the wrong vector."""
    rng = np.random.default_rng(seed)
    t = dict(model.tensors)
    for name, (fmt, shape, data) in model.tensors.items():
        if data.dtype == np.float32 and fmt == F.F32 and shape[0] == 1 and name.endswith("norm.weight"):
            t[name] = (fmt, shape, (1.0 + 0.1 * rng.standard_normal(shape[1])).astype(np.float32))
    return HostModel(model.spec, t, model.rope_factors)


def random_tokens(spec: ModelSpec, n: int, seed: int = 0) -> np.ndarray:
    return np.random.default_rng(seed).integers(0, spec.vocab, size=n, dtype=np.int32)
