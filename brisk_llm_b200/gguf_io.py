"""Minimal GGUF v3 writer and reader for the tensors and metadata the token loop needs.

The writer produces files the reference's loader accepts (metadata keys of brisk-llm
src/model.cpp:217-244,283-292; tensor names of :326-421; matrices stored as {cols, rows},
:462-466), so the same synthetic model can be fed to the reference CPU engine and, through
HostModel, to the CUDA library. The reader maps a file back into a HostModel.
"""
from __future__ import annotations

import struct

import numpy as np

from . import formats as F
from .synth import HostModel, ModelSpec

ALIGN = 32
_U32, _F32, _STR, _U64 = 4, 6, 8, 10
ARCH_NAME = {"qwen3": "qwen3", "llama": "llama", "bitnet": "bitnet-b1.58", "gemma3": "gemma3", "smollm3": "smollm3", "qwen2": "qwen2", "phi3": "phi3"}


def _s(b: bytes) -> bytes:
    return struct.pack("<Q", len(b)) + b


def write_gguf(model: HostModel, path: str) -> None:
    s = model.spec
    arch = ARCH_NAME[s.arch]
    kv = [("general.architecture", _STR, arch), ("general.name", _STR, s.name),
          (f"{arch}.block_count", _U32, s.layers), (f"{arch}.embedding_length", _U32, s.hidden),
          (f"{arch}.attention.head_count", _U32, s.heads), (f"{arch}.attention.head_count_kv", _U32, s.kv_heads),
          (f"{arch}.attention.key_length", _U32, s.head_dim), (f"{arch}.attention.value_length", _U32, s.head_dim),
          (f"{arch}.feed_forward_length", _U32, s.ffn), (f"{arch}.context_length", _U32, s.context),
          (f"{arch}.rope.freq_base", _F32, s.rope_base), (f"{arch}.attention.layer_norm_rms_epsilon", _F32, s.eps)]
    if s.arch == "gemma3":  # src/model.cpp:170-175
        kv += [(f"{arch}.attention.sliding_window", _U32, s.sliding_window), (f"{arch}.rope.freq_base_swa", _F32, s.rope_base_local),
               (f"{arch}.rope.scaling.factor", _F32, s.rope_scaling_factor), (f"{arch}.final_logit_softcapping", _F32, s.final_softcap)]
    tensors = dict(model.tensors)
    if s.arch == "phi3":  # src/model.cpp:177-188; Q, K, V rows in one tensor, gate and up rows in another (:370-382)
        kv += [(f"{arch}.rope.dimension_count", _U32, s.rope_dim or s.head_dim), (f"{arch}.rope.scaling.attn_factor", _F32, s.rope_attn_factor),
               (f"{arch}.rope.scaling.original_context_length", _U32, s.rope_original_context)]
        fused = {}
        for name, entry in tensors.items():
            if name.endswith(("attn_k.weight", "attn_v.weight", "ffn_gate.weight")):
                continue
            if name.endswith("attn_q.weight") or name.endswith("ffn_up.weight"):
                p = name[:name.rindex(".weight")].rsplit(".", 1)[0] + "."
                parts = ["attn_q.weight", "attn_k.weight", "attn_v.weight"] if name.endswith("attn_q.weight") else ["ffn_gate.weight", "ffn_up.weight"]
                group = [tensors[p + q] for q in parts]
                assert len({g[0] for g in group}) == 1, "fused tensors need one type"
                fused[p + ("attn_qkv.weight" if len(parts) == 3 else "ffn_up.weight")] = (
                    group[0][0], (sum(g[1][0] for g in group), group[0][1][1]), np.concatenate([np.ascontiguousarray(g[2]).reshape(-1) for g in group]))
            else:
                fused[name] = entry
        tensors = fused
    if model.rope_factors is not None and s.arch != "phi3":
        tensors["rope_freqs.weight"] = (F.F32, (1, len(model.rope_factors)), model.rope_factors)
    head = bytearray(b"GGUF" + struct.pack("<IQQ", 3, len(tensors), len(kv)))
    for key, typ, val in kv:
        head += _s(key.encode()) + struct.pack("<I", typ)
        head += {_U32: lambda v: struct.pack("<I", v), _F32: lambda v: struct.pack("<f", v),
                 _STR: lambda v: _s(v.encode())}[typ](val)
    offset = 0
    placed = []
    for name, (fmt, (rows, cols), data) in tensors.items():
        dims = (cols,) if rows == 1 and fmt == F.F32 and data.dtype == np.float32 and name != "token_embd.weight" else (cols, rows)
        head += _s(name.encode()) + struct.pack("<I", len(dims)) + b"".join(struct.pack("<Q", d) for d in dims)
        head += struct.pack("<IQ", fmt, offset)
        placed.append((offset, data))
        offset += (data.nbytes + ALIGN - 1) // ALIGN * ALIGN
    pad = (-len(head)) % ALIGN
    with open(path, "wb") as f:
        f.write(head + b"\0" * pad)
        base = f.tell()
        for off, data in placed:
            f.seek(base + off)
            f.write(np.ascontiguousarray(data).tobytes())
        f.truncate(base + offset)


class _Reader:
    def __init__(self, buf):
        self.b, self.p = buf, 0

    def take(self, fmt):
        v = struct.unpack_from("<" + fmt, self.b, self.p)
        self.p += struct.calcsize("<" + fmt)
        return v[0] if len(v) == 1 else v

    def string(self):
        n = self.take("Q")
        v = bytes(self.b[self.p:self.p + n]).decode("utf-8", "replace")
        self.p += n
        return v

    _SCALAR = {0: "B", 1: "b", 2: "H", 3: "h", 4: "I", 5: "i", 6: "f", 7: "?", 10: "Q", 11: "q", 12: "d"}

    def value(self, typ):
        if typ == 8:
            return self.string()
        if typ == 9:
            et, n = self.take("I"), self.take("Q")
            return [self.value(et) for _ in range(n)]
        return self.take(self._SCALAR[typ])


def read_gguf(path: str) -> HostModel:
    """Load a GGUF of a supported family into a HostModel (tensors stay views of one memory map)."""
    buf = np.memmap(path, dtype=np.uint8, mode="r")
    r = _Reader(buf)
    if bytes(buf[:4]) != b"GGUF":
        raise ValueError("gguf: bad magic")
    r.p = 4
    version, n_tensors, n_kv = r.take("I"), r.take("Q"), r.take("Q")
    if version not in (2, 3):
        raise ValueError(f"gguf: unsupported version {version}")
    meta = {}
    for _ in range(n_kv):
        key = r.string()
        meta[key] = r.value(r.take("I"))
    infos = []
    for _ in range(n_tensors):
        name = r.string()
        nd = r.take("I")
        dims = [r.take("Q") for _ in range(nd)]
        typ, off = r.take("I"), r.take("Q")
        infos.append((name, dims, typ, off))
    align = meta.get("general.alignment", ALIGN)
    base = (r.p + align - 1) // align * align
    arch = meta["general.architecture"]
    fam = {"qwen3": "qwen3", "llama": "llama", "bitnet": "bitnet", "bitnet-b1.58": "bitnet", "gemma3": "gemma3", "smollm3": "smollm3", "qwen2": "qwen2", "phi3": "phi3"}.get(arch)
    if fam is None:
        raise ValueError(f"gguf: architecture '{arch}' is not one this backend runs (qwen3, qwen2, llama, bitnet, gemma3, smollm3, phi3)")
    g = lambda k, d=None: meta.get(f"{arch}.{k}", d)
    tensors, rope = {}, None
    for name, dims, typ, off in infos:
        if typ not in F.BLOCK_BYTES:
            raise ValueError(f"gguf: tensor '{name}' has unsupported type {typ}")
        cols, rows = dims[0], (dims[1] if len(dims) > 1 else 1)
        nbytes = rows * F.row_bytes(typ, cols)
        raw = buf[base + off: base + off + nbytes]
        if len(dims) == 1 or name.endswith("_norm.weight") or name == "rope_freqs.weight":
            vec = F.dequantize(typ, raw, rows * cols) if typ != F.F32 else np.frombuffer(raw.tobytes(), np.float32).copy()
            if name == "rope_freqs.weight":
                rope = vec
                continue
            tensors[name] = (F.F32, (1, rows * cols), vec)
        else:
            tensors[name] = (typ, (rows, cols), raw)
    hidden, heads = g("embedding_length"), g("attention.head_count")
    if fam == "phi3":  # split the fused tensors by rows, as the reference's loader does (src/model.cpp:370-382)
        kv_heads = g("attention.head_count_kv")
        head_dim = g("attention.key_length", hidden // heads)
        for name in [n for n in tensors if n.endswith("attn_qkv.weight") or n.endswith("ffn_up.weight")]:
            typ, (rows, cols), raw = tensors.pop(name)
            rb = F.row_bytes(typ, cols)
            p = name.rsplit(".", 2)[0] + "."
            if name.endswith("attn_qkv.weight"):
                parts = [("attn_q.weight", heads * head_dim), ("attn_k.weight", kv_heads * head_dim), ("attn_v.weight", kv_heads * head_dim)]
            else:
                parts = [("ffn_gate.weight", rows // 2), ("ffn_up.weight", rows // 2)]
            at = 0
            for part, n_rows in parts:
                tensors[p + part] = (typ, (n_rows, cols), raw[at * rb:(at + n_rows) * rb])
                at += n_rows
    emb = tensors["token_embd.weight"]
    spec = ModelSpec(meta.get("general.name", "gguf"), fam, g("block_count"), hidden, heads, g("attention.head_count_kv"),
                     g("attention.key_length", hidden // heads), g("feed_forward_length"), emb[1][0], g("context_length"),
                     g("rope.freq_base"), g("attention.layer_norm_rms_epsilon"), "output.weight" not in tensors,
                     tensors["blk.0.attn_q.weight"][0])
    if fam == "phi3":
        from dataclasses import replace
        spec = replace(spec, rope_dim=g("rope.dimension_count", 0), rope_attn_factor=g("rope.scaling.attn_factor", 1.0),
                       rope_original_context=g("rope.scaling.original_context_length", 0))
    if fam == "gemma3":
        from dataclasses import replace
        spec = replace(spec, sliding_window=g("attention.sliding_window", 0), rope_base_local=g("rope.freq_base_swa", 10000.0),
                       rope_scaling_factor=g("rope.scaling.factor", 1.0), final_softcap=g("final_logit_softcapping", 0.0))
    return HostModel(spec, tensors, rope)
