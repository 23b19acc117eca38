"""Quantised weight formats of the token loop: ids, block sizes, and numpy encoders/decoders.

The byte layouts are the GGUF/ggml ones the reference reads in place (brisk-llm src/quant.h:26-130).
The reference ships no weight quantiser (its files come from an external tool), so the encoders
here are this package's own: any encoding that the reference's decoders (src/quant.cpp:196-307,
:565-578) read back is a valid file. Used to build synthetic models and test matrices.
"""
from __future__ import annotations

import numpy as np

F32, F16, Q4_0, Q4_1, Q5_0, Q8_0, Q4_K, Q5_K, Q6_K, BF16, TQ2_0 = 0, 1, 2, 3, 6, 8, 12, 13, 14, 30, 35

NAMES = {F32: "F32", F16: "F16", Q4_0: "Q4_0", Q4_1: "Q4_1", Q5_0: "Q5_0", Q8_0: "Q8_0", Q4_K: "Q4_K", Q5_K: "Q5_K", Q6_K: "Q6_K",
         BF16: "BF16", TQ2_0: "TQ2_0"}
BY_NAME = {v: k for k, v in NAMES.items()}
BLOCK_ELEMS = {F32: 1, F16: 1, BF16: 1, Q4_0: 32, Q4_1: 32, Q5_0: 32, Q8_0: 32, Q4_K: 256, Q5_K: 256, Q6_K: 256, TQ2_0: 256}
BLOCK_BYTES = {F32: 4, F16: 2, BF16: 2, Q4_0: 18, Q4_1: 20, Q5_0: 22, Q8_0: 34, Q4_K: 144, Q5_K: 176, Q6_K: 210, TQ2_0: 66}
TAKES_Q8_K = {Q4_K, Q5_K, Q6_K, TQ2_0}  # activations quantised per 256 (src/quant.h:21-22)


def row_bytes(fmt: int, cols: int) -> int:
    assert cols % BLOCK_ELEMS[fmt] == 0, (NAMES[fmt], cols)
    return cols // BLOCK_ELEMS[fmt] * BLOCK_BYTES[fmt]


def _rint(x):
    return np.rint(x)


def quantize_q4_0(x: np.ndarray) -> np.ndarray:
    """[..., 32k] f32 -> uint8 bytes. weight = (q - 8) * d; low nibble = element i, high = i + 16."""
    b = x.reshape(-1, 32).astype(np.float32)
    idx = np.argmax(np.abs(b), axis=1)
    mx = b[np.arange(b.shape[0]), idx]
    d = (mx / -8.0).astype(np.float32)
    inv = np.where(d != 0, 1.0 / np.where(d == 0, 1, d), 0).astype(np.float32)
    q = np.clip(np.floor(b * inv[:, None] + 8.5), 0, 15).astype(np.uint8)
    out = np.empty((b.shape[0], 18), np.uint8)
    out[:, 0:2] = d.astype(np.float16).view(np.uint8).reshape(-1, 2)
    out[:, 2:] = q[:, :16] | (q[:, 16:] << 4)
    return out.reshape(-1)


def quantize_q4_1(x: np.ndarray) -> np.ndarray:
    """weight = q * d + m with m the block minimum (src/quant.h:58-63); nibble order as Q4_0."""
    b = x.reshape(-1, 32).astype(np.float32)
    lo, hi = b.min(axis=1), b.max(axis=1)
    d = ((hi - lo) / 15.0).astype(np.float16).astype(np.float32)
    m = lo.astype(np.float16).astype(np.float32)
    inv = np.where(d != 0, 1.0 / np.where(d == 0, 1, d), 0).astype(np.float32)
    q = np.clip(_rint((b - m[:, None]) * inv[:, None]), 0, 15).astype(np.uint8)
    out = np.empty((b.shape[0], 20), np.uint8)
    out[:, 0:2] = d.astype(np.float16).view(np.uint8).reshape(-1, 2)
    out[:, 2:4] = m.astype(np.float16).view(np.uint8).reshape(-1, 2)
    out[:, 4:] = q[:, :16] | (q[:, 16:] << 4)
    return out.reshape(-1)


def quantize_q5_0(x: np.ndarray) -> np.ndarray:
    """weight = (q - 16) * d, q in 0..31: low four bits as Q4_0, the fifth bit of element i at bit i of the 32-bit qh
    (src/quant.h:66-72)."""
    b = x.reshape(-1, 32).astype(np.float32)
    idx = np.argmax(np.abs(b), axis=1)
    mx = b[np.arange(b.shape[0]), idx]
    d = (mx / -16.0).astype(np.float32)
    inv = np.where(d != 0, 1.0 / np.where(d == 0, 1, d), 0).astype(np.float32)
    q = np.clip(np.floor(b * inv[:, None] + 16.5), 0, 31).astype(np.uint32)
    qh = ((q >> 4) << np.arange(32, dtype=np.uint32)[None, :]).sum(axis=1).astype(np.uint32)
    out = np.empty((b.shape[0], 22), np.uint8)
    out[:, 0:2] = d.astype(np.float16).view(np.uint8).reshape(-1, 2)
    out[:, 2:6] = qh.view(np.uint8).reshape(-1, 4)
    out[:, 6:] = ((q[:, :16] & 0xF) | ((q[:, 16:] & 0xF) << 4)).astype(np.uint8)
    return out.reshape(-1)


def quantize_q8_0(x: np.ndarray) -> np.ndarray:
    b = x.reshape(-1, 32).astype(np.float32)
    d = (np.abs(b).max(axis=1) / 127.0).astype(np.float32)
    inv = np.where(d != 0, 1.0 / np.where(d == 0, 1, d), 0).astype(np.float32)
    q = _rint(b * inv[:, None]).astype(np.int8)
    out = np.empty((b.shape[0], 34), np.uint8)
    out[:, 0:2] = d.astype(np.float16).view(np.uint8).reshape(-1, 2)
    out[:, 2:] = q.view(np.uint8)
    return out.reshape(-1)


def quantize_tq2_0(x: np.ndarray) -> np.ndarray:
    """Ternary: weight = (q - 1) * d with d = max|x| of the block; bit pair l of byte 32j+m holds element 128j+32l+m."""
    b = x.reshape(-1, 256).astype(np.float32)
    d = np.abs(b).max(axis=1).astype(np.float32)
    inv = np.where(d != 0, 1.0 / np.where(d == 0, 1, d), 0).astype(np.float32)
    q = (np.clip(_rint(b * inv[:, None]), -1, 1) + 1).astype(np.uint8).reshape(-1, 2, 4, 32)  # [blk][j][l][m]
    qs = q[:, :, 0] | (q[:, :, 1] << 2) | (q[:, :, 2] << 4) | (q[:, :, 3] << 6)  # [blk][j][m]
    out = np.empty((b.shape[0], 66), np.uint8)
    out[:, :64] = qs.reshape(-1, 64)
    out[:, 64:] = d.astype(np.float16).view(np.uint8).reshape(-1, 2)
    return out.reshape(-1)


def quantize_q4_k(x: np.ndarray) -> np.ndarray:
    """weight = d*scale*q - dmin*min per 32-value sub-block, 6-bit scale/min, 4-bit q (src/quant.h:91-99)."""
    b = x.reshape(-1, 8, 32).astype(np.float32)
    lo = np.minimum(b.min(axis=2), 0.0)
    hi = b.max(axis=2)
    scale = (hi - lo) / 15.0
    mins = -lo
    d = (scale.max(axis=1) / 63.0).astype(np.float16).astype(np.float32)
    dmin = (mins.max(axis=1) / 63.0).astype(np.float16).astype(np.float32)
    safe = lambda v: np.where(v == 0, 1.0, v)
    sc = np.clip(_rint(scale / safe(d)[:, None]), 0, 63).astype(np.uint8)
    mn = np.clip(_rint(mins / safe(dmin)[:, None]), 0, 63).astype(np.uint8)
    eff = d[:, None] * sc
    q = np.clip(_rint((b + (dmin[:, None] * mn)[:, :, None]) / safe(eff)[:, :, None]), 0, 15).astype(np.uint8)
    out = np.empty((b.shape[0], 144), np.uint8)
    out[:, 0:2] = d.astype(np.float16).view(np.uint8).reshape(-1, 2)
    out[:, 2:4] = dmin.astype(np.float16).view(np.uint8).reshape(-1, 2)
    s = np.empty((b.shape[0], 12), np.uint8)
    s[:, 0:4] = (sc[:, 0:4] & 63) | ((sc[:, 4:8] >> 4) << 6)
    s[:, 4:8] = (mn[:, 0:4] & 63) | ((mn[:, 4:8] >> 4) << 6)
    s[:, 8:12] = (sc[:, 4:8] & 0xF) | ((mn[:, 4:8] & 0xF) << 4)
    out[:, 4:16] = s
    qc = q.reshape(-1, 4, 2, 32)  # chunk, (low sub-block, high sub-block), i
    out[:, 16:] = (qc[:, :, 0] | (qc[:, :, 1] << 4)).reshape(-1, 128)
    return out.reshape(-1)


def quantize_q5_k(x: np.ndarray) -> np.ndarray:
    """Q4_K with a fifth bit per weight (q in 0..31): bit sb of qh[i] is the high bit of weight i of sub-block sb
    (src/quant.h:101-110)."""
    b = x.reshape(-1, 8, 32).astype(np.float32)
    lo = np.minimum(b.min(axis=2), 0.0)
    hi = b.max(axis=2)
    scale = (hi - lo) / 31.0
    mins = -lo
    d = (scale.max(axis=1) / 63.0).astype(np.float16).astype(np.float32)
    dmin = (mins.max(axis=1) / 63.0).astype(np.float16).astype(np.float32)
    safe = lambda v: np.where(v == 0, 1.0, v)
    sc = np.clip(_rint(scale / safe(d)[:, None]), 0, 63).astype(np.uint8)
    mn = np.clip(_rint(mins / safe(dmin)[:, None]), 0, 63).astype(np.uint8)
    eff = d[:, None] * sc
    q = np.clip(_rint((b + (dmin[:, None] * mn)[:, :, None]) / safe(eff)[:, :, None]), 0, 31).astype(np.uint8)
    out = np.empty((b.shape[0], 176), np.uint8)
    out[:, 0:2] = d.astype(np.float16).view(np.uint8).reshape(-1, 2)
    out[:, 2:4] = dmin.astype(np.float16).view(np.uint8).reshape(-1, 2)
    s = np.empty((b.shape[0], 12), np.uint8)
    s[:, 0:4] = (sc[:, 0:4] & 63) | ((sc[:, 4:8] >> 4) << 6)
    s[:, 4:8] = (mn[:, 0:4] & 63) | ((mn[:, 4:8] >> 4) << 6)
    s[:, 8:12] = (sc[:, 4:8] & 0xF) | ((mn[:, 4:8] & 0xF) << 4)
    out[:, 4:16] = s
    out[:, 16:48] = ((q >> 4) << np.arange(8, dtype=np.uint8)[None, :, None]).sum(axis=1).astype(np.uint8)
    qc = (q & 0xF).reshape(-1, 4, 2, 32)
    out[:, 48:] = (qc[:, :, 0] | (qc[:, :, 1] << 4)).reshape(-1, 128)
    return out.reshape(-1)


def quantize_q6_k(x: np.ndarray) -> np.ndarray:
    """weight = d*scale*(q - 32) per 16-value sub-block, int8 scale, 6-bit q (src/quant.h:113-121)."""
    b = x.reshape(-1, 16, 16).astype(np.float32)
    idx = np.argmax(np.abs(b), axis=2)
    ext = np.take_along_axis(b, idx[:, :, None], axis=2)[:, :, 0]
    scale = ext / -32.0
    d = (np.abs(scale).max(axis=1) / 127.0).astype(np.float16).astype(np.float32)
    safe = lambda v: np.where(v == 0, 1.0, v)
    sc = np.clip(_rint(scale / safe(d)[:, None]), -128, 127).astype(np.int8)
    eff = d[:, None] * sc.astype(np.float32)
    q = (np.clip(_rint(b / safe(eff)[:, :, None]), -32, 31) + 32).astype(np.uint8).reshape(-1, 2, 4, 32)  # [blk][half][k][l]
    ql = np.empty((q.shape[0], 2, 64), np.uint8)
    ql[:, :, :32] = (q[:, :, 0] & 0xF) | ((q[:, :, 2] & 0xF) << 4)
    ql[:, :, 32:] = (q[:, :, 1] & 0xF) | ((q[:, :, 3] & 0xF) << 4)
    qh = (q[:, :, 0] >> 4) | ((q[:, :, 1] >> 4) << 2) | ((q[:, :, 2] >> 4) << 4) | ((q[:, :, 3] >> 4) << 6)
    out = np.empty((q.shape[0], 210), np.uint8)
    out[:, :128] = ql.reshape(-1, 128)
    out[:, 128:192] = qh.reshape(-1, 64)
    out[:, 192:208] = sc.view(np.uint8)
    out[:, 208:] = d.astype(np.float16).view(np.uint8).reshape(-1, 2)
    return out.reshape(-1)


_QUANTIZERS = {Q4_0: quantize_q4_0, Q4_1: quantize_q4_1, Q5_0: quantize_q5_0, Q8_0: quantize_q8_0, Q4_K: quantize_q4_k, Q5_K: quantize_q5_k,
               Q6_K: quantize_q6_k, TQ2_0: quantize_tq2_0}


def to_bf16(x: np.ndarray) -> np.ndarray:
    """f32 -> bfloat16 bit patterns (uint16), round to nearest even."""
    u = np.ascontiguousarray(x, np.float32).view(np.uint32)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)


def quantize(fmt: int, x: np.ndarray) -> np.ndarray:
    """f32 matrix [rows][cols] -> the file bytes of that matrix in `fmt` (uint8, row after row)."""
    if fmt == F32:
        return np.ascontiguousarray(x, np.float32).view(np.uint8).reshape(-1)
    if fmt == F16:
        return np.ascontiguousarray(x.astype(np.float16)).view(np.uint8).reshape(-1)
    if fmt == BF16:
        return to_bf16(x).view(np.uint8).reshape(-1)
    return _QUANTIZERS[fmt](np.ascontiguousarray(x, np.float32))


def dequantize(fmt: int, data: np.ndarray, count: int) -> np.ndarray:
    """Numpy decoder of each layout (weight order), for tests of the encoders and of the device repack."""
    raw = np.frombuffer(np.ascontiguousarray(data).tobytes(), np.uint8)
    if fmt == F32:
        return raw.view(np.float32)[:count].copy()
    if fmt == F16:
        return raw.view(np.float16)[:count].astype(np.float32)
    if fmt == BF16:
        return (raw.view(np.uint16)[:count].astype(np.uint32) << 16).view(np.float32)
    nb = count // BLOCK_ELEMS[fmt]
    blk = raw[: nb * BLOCK_BYTES[fmt]].reshape(nb, BLOCK_BYTES[fmt])
    h = lambda cols: np.ascontiguousarray(cols).view(np.float16).astype(np.float32).reshape(-1)
    if fmt == Q4_0:
        d = h(blk[:, 0:2])
        qs = blk[:, 2:]
        q = np.concatenate([qs & 0xF, qs >> 4], axis=1).astype(np.float32) - 8
        return (q * d[:, None]).reshape(-1)
    if fmt == Q4_1:
        d, m = h(blk[:, 0:2]), h(blk[:, 2:4])
        qs = blk[:, 4:]
        q = np.concatenate([qs & 0xF, qs >> 4], axis=1).astype(np.float32)
        return ((q * d[:, None]).astype(np.float32) + m[:, None]).astype(np.float32).reshape(-1)
    if fmt == Q5_0:
        d = h(blk[:, 0:2])
        qh = np.ascontiguousarray(blk[:, 2:6]).view(np.uint32).reshape(-1)
        qs = blk[:, 6:]
        bits = ((qh[:, None] >> np.arange(32, dtype=np.uint32)[None, :]) & 1).astype(np.int32)
        q = np.concatenate([qs & 0xF, qs >> 4], axis=1).astype(np.int32) | (bits << 4)
        return ((q - 16).astype(np.float32) * d[:, None]).reshape(-1)
    if fmt == Q8_0:
        d = h(blk[:, 0:2])
        return (blk[:, 2:].view(np.int8).astype(np.float32) * d[:, None]).reshape(-1)
    if fmt == TQ2_0:
        d = h(blk[:, 64:66])
        qs = blk[:, :64].reshape(nb, 2, 1, 32)
        q = (qs >> (2 * np.arange(4, dtype=np.uint8)).reshape(1, 1, 4, 1)) & 3
        return ((q.astype(np.float32) - 1) * d[:, None, None, None]).reshape(-1)
    if fmt == Q4_K:
        d, dmin = h(blk[:, 0:2]), h(blk[:, 2:4])
        s = blk[:, 4:16]
        sc = np.empty((nb, 8), np.uint8)
        mn = np.empty((nb, 8), np.uint8)
        sc[:, :4] = s[:, 0:4] & 63
        mn[:, :4] = s[:, 4:8] & 63
        sc[:, 4:] = (s[:, 8:12] & 0xF) | ((s[:, 0:4] >> 6) << 4)
        mn[:, 4:] = (s[:, 8:12] >> 4) | ((s[:, 4:8] >> 6) << 4)
        qs = blk[:, 16:].reshape(nb, 4, 32)
        q = np.stack([qs & 0xF, qs >> 4], axis=2).reshape(nb, 8, 32).astype(np.float32)
        d1 = (d[:, None] * sc.astype(np.float32)).astype(np.float32)
        m1 = (dmin[:, None] * mn.astype(np.float32)).astype(np.float32)
        return (d1[:, :, None] * q - m1[:, :, None]).astype(np.float32).reshape(-1)
    if fmt == Q5_K:
        d, dmin = h(blk[:, 0:2]), h(blk[:, 2:4])
        s = blk[:, 4:16]
        sc = np.empty((nb, 8), np.uint8)
        mn = np.empty((nb, 8), np.uint8)
        sc[:, :4] = s[:, 0:4] & 63
        mn[:, :4] = s[:, 4:8] & 63
        sc[:, 4:] = (s[:, 8:12] & 0xF) | ((s[:, 0:4] >> 6) << 4)
        mn[:, 4:] = (s[:, 8:12] >> 4) | ((s[:, 4:8] >> 6) << 4)
        qh = blk[:, 16:48]
        qs = blk[:, 48:].reshape(nb, 4, 32)
        q = np.stack([qs & 0xF, qs >> 4], axis=2).reshape(nb, 8, 32)
        high = (qh[:, None, :] >> np.arange(8, dtype=np.uint8)[None, :, None]) & 1
        q = (q | (high << 4)).astype(np.float32)
        d1 = (d[:, None] * sc.astype(np.float32)).astype(np.float32)
        m1 = (dmin[:, None] * mn.astype(np.float32)).astype(np.float32)
        return (d1[:, :, None] * q - m1[:, :, None]).astype(np.float32).reshape(-1)
    if fmt == Q6_K:
        ql = blk[:, :128].reshape(nb, 2, 64)
        qh = blk[:, 128:192].reshape(nb, 2, 32)
        sc = blk[:, 192:208].view(np.int8).astype(np.float32)
        d = h(blk[:, 208:210])
        q = np.empty((nb, 2, 4, 32), np.int32)
        q[:, :, 0] = (ql[:, :, :32] & 0xF) | ((qh & 3) << 4)
        q[:, :, 1] = (ql[:, :, 32:] & 0xF) | (((qh >> 2) & 3) << 4)
        q[:, :, 2] = (ql[:, :, :32] >> 4) | (((qh >> 4) & 3) << 4)
        q[:, :, 3] = (ql[:, :, 32:] >> 4) | (((qh >> 6) & 3) << 4)
        q = (q - 32).reshape(nb, 16, 16).astype(np.float32)
        return ((d[:, None] * sc)[:, :, None].astype(np.float32) * q).astype(np.float32).reshape(-1)
    raise ValueError(fmt)
