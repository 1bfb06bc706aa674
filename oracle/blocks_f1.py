"""CPU oracle (TEST INFRASTRUCTURE, not product code): codecs and product models of the 1- to 3-bit GGUF types the
real model file mixes with the four main ones: Q2_K, IQ2_XXS, IQ2_XS, IQ2_S, IQ3_XXS, IQ1_M.

Block structs: plugin/vllm_gguf_plugin/csrc/lcpp/ggml/src/ggml-common.h:300-309 (block_q2_K), 380-411 (block_iq2_xxs,
block_iq2_xs, block_iq2_s, block_iq3_xxs), 430-444 (block_iq1_m, iq1m_scale_t). The product models follow the
reference's MMVQ arithmetic, integer truncations included (ggml-cuda/vecdotq.cuh: 367-393 + 868-889 Q2_K, 1048-1078
IQ2_XXS, 1083-1119 IQ2_XS, 1124-1167 IQ2_S, 1172-1206 IQ3_XXS, 1286-1329 IQ1_M).

`dequantize` reproduces the float32 results of gguf-py / llama.cpp's C dequantiser bit for bit; pinned by
tests/test_oracle_blocks_f1.py against the reference's real-row fixtures (tests/fixtures/dequant/*.npz, read from the
reference tree when it is present; the outcome of that run is committed as tests/golden/fixture_check_f1.json) and
against committed gguf-py outputs on seeded blocks (tests/golden/dequant_blocks_f1.npz).

Only tests/, __graft_entry__.smoke() and bench.py's cpu_baseline / reference arm may import this package.
"""

from __future__ import annotations

import os
from dataclasses import dataclass

import numpy as np

Q2_K, IQ2_XXS, IQ2_XS, IQ3_XXS, IQ2_S, IQ1_M = 10, 16, 17, 18, 22, 29
TYPE_NAMES = {Q2_K: "Q2_K", IQ2_XXS: "IQ2_XXS", IQ2_XS: "IQ2_XS", IQ3_XXS: "IQ3_XXS", IQ2_S: "IQ2_S", IQ1_M: "IQ1_M"}
TYPE_IDS = {v: k for k, v in TYPE_NAMES.items()}
BLOCK_BYTES = {Q2_K: 84, IQ2_XXS: 66, IQ2_XS: 74, IQ3_XXS: 98, IQ2_S: 82, IQ1_M: 56}
QK_K = 256

_T = None


def tables():
    global _T
    if _T is None:
        z = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "tables_f1.npz"))
        _T = {k: z[k] for k in z.files}
    return _T


@dataclass
class DecodedF1:
    """Integer view of a weight matrix of one of these types.

    w8    int8  [N, K]      the integer fed to the int8 dot product: signed codebook value (IQ2_*, IQ3_XXS), the 2-bit
                            quant (Q2_K), 8 * (codebook value + delta) = 8 g +- 1 (IQ1_M)
    sub   int32 [N, K/g]    stored sub-scale field of each group of g values (g = 32: IQ2_XXS, IQ3_XXS; 16: the others)
    mins  int32 [N, K/16]   Q2_K only: 4-bit min of each 16-value group
    d     f32   [N, K/256]  superblock scale;  dmin: Q2_K only
    """

    type: int
    w8: np.ndarray
    sub: np.ndarray
    d: np.ndarray
    g: int
    mins: np.ndarray | None = None
    dmin: np.ndarray | None = None


def _blocks(raw, t):
    raw = np.ascontiguousarray(raw, dtype=np.uint8)
    if raw.ndim == 1:
        raw = raw[None]
    n, rb = raw.shape
    bs = BLOCK_BYTES[t]
    assert rb % bs == 0, (rb, bs)
    return raw.reshape(n, rb // bs, bs)


def _f16(b):
    return np.ascontiguousarray(b).view(np.float16).astype(np.float32)[..., 0]


def _u16(b):
    return np.ascontiguousarray(b).view(np.uint16)


def _u32(b):
    return np.ascontiguousarray(b).view(np.uint32)


def _sign_bits(bytes8):
    """uint8 [...] -> int32 [..., 8] of 0 / 1, bit i = sign of value i."""
    return ((bytes8[..., None] >> np.arange(8, dtype=np.uint8)) & 1).astype(np.int32)


def decode(raw: np.ndarray, t: int) -> DecodedF1:
    b = _blocks(raw, t)
    n, nb, _ = b.shape
    k = nb * QK_K
    T = tables()
    if t == IQ2_XXS:
        d = _f16(b[..., 0:2])
        q = _u32(b[..., 2:66]).reshape(n, nb, 8, 2)              # per 32 values: 4 index bytes, then signs + scale
        idx = np.ascontiguousarray(q[..., 0]).view(np.uint8).reshape(n, nb, 8, 4)
        aux = q[..., 1]
        sidx = (aux[..., None] >> (7 * np.arange(4, dtype=np.uint32))) & 0x7F
        sg = _sign_bits(T["ksigns"][sidx])                       # [n, nb, 8, 4, 8]
        mag = T["iq2xxs"][idx].astype(np.int32)
        w8 = (mag * (1 - 2 * sg)).reshape(n, k).astype(np.int8)
        return DecodedF1(t, w8, (aux >> 28).astype(np.int32).reshape(n, nb * 8), d, 32)
    if t == IQ2_XS:
        d = _f16(b[..., 0:2])
        q = _u16(b[..., 2:66]).reshape(n, nb, 32)                # per 8 values: 9-bit index, 7-bit sign index
        sc = b[..., 66:74].astype(np.int32)
        sg = _sign_bits(T["ksigns"][q >> 9])
        mag = T["iq2xs"][q & 511].astype(np.int32)
        w8 = (mag * (1 - 2 * sg)).reshape(n, k).astype(np.int8)
        sub = np.stack([sc & 0x0F, sc >> 4], -1).reshape(n, nb * 16)
        return DecodedF1(t, w8, sub.astype(np.int32), d, 16)
    if t == IQ2_S:
        d = _f16(b[..., 0:2])
        lo = b[..., 2:34].astype(np.int32)                       # low 8 index bits per 8 values
        sg = _sign_bits(b[..., 34:66])
        qh = b[..., 66:74].astype(np.int32)
        sc = b[..., 74:82].astype(np.int32)
        hi = (qh[..., None] >> (2 * np.arange(4))) & 3           # [n, nb, 8, 4]
        idx = lo | (hi.reshape(n, nb, 32) << 8)
        mag = T["iq2s"][idx].astype(np.int32)
        w8 = (mag * (1 - 2 * sg)).reshape(n, k).astype(np.int8)
        sub = np.stack([sc & 0x0F, sc >> 4], -1).reshape(n, nb * 16)
        return DecodedF1(t, w8, sub.astype(np.int32), d, 16)
    if t == IQ3_XXS:
        d = _f16(b[..., 0:2])
        idx = b[..., 2:66].reshape(n, nb, 8, 8)                  # per 32 values: 8 index bytes of 4 values each
        aux = _u32(b[..., 66:98]).reshape(n, nb, 8)
        sidx = (aux[..., None] >> (7 * np.arange(4, dtype=np.uint32))) & 0x7F
        sg = _sign_bits(T["ksigns"][sidx])                       # [n, nb, 8, 4, 8]
        mag = T["iq3xxs"][idx].astype(np.int32).reshape(n, nb, 8, 4, 8)
        w8 = (mag * (1 - 2 * sg)).reshape(n, k).astype(np.int8)
        return DecodedF1(t, w8, (aux >> 28).astype(np.int32).reshape(n, nb * 8), d, 32)
    if t == Q2_K:
        sc = b[..., 0:16].astype(np.int32)
        qs = b[..., 16:80].reshape(n, nb, 2, 1, 32)
        d = _f16(b[..., 80:82])
        dmin = _f16(b[..., 82:84])
        q = (qs >> (2 * np.arange(4, dtype=np.uint8)).reshape(1, 1, 1, 4, 1)) & 3   # [n, nb, 2, 4, 32]
        return DecodedF1(t, q.reshape(n, k).astype(np.int8), (sc & 0x0F).reshape(n, nb * 16), d, 16,
                         (sc >> 4).reshape(n, nb * 16), dmin)
    if t == IQ1_M:
        lo = b[..., 0:32].astype(np.int32)
        qh = b[..., 32:48].astype(np.int32)
        s16 = _u16(b[..., 48:56]).astype(np.int32)               # [n, nb, 4]
        dbits = ((s16[..., 0] >> 12) | ((s16[..., 1] >> 8) & 0x00F0) | ((s16[..., 2] >> 4) & 0x0F00) | (s16[..., 3] & 0xF000))
        d = dbits.astype(np.uint16).view(np.float16).astype(np.float32)
        nib = np.stack([qh & 0x0F, qh >> 4], -1).reshape(n, nb, 32)   # per 8 values: 3 index bits + delta sign
        idx = lo | ((nib & 7) << 8)
        g = T["iq1"][idx].astype(np.int32)                       # [n, nb, 32, 8] in {-1, 0, 1}
        w8 = 8 * g + np.where(nib & 8, -1, 1)[..., None]
        sub = ((s16[..., None] >> (3 * np.arange(4))) & 7).reshape(n, nb * 16)
        return DecodedF1(t, w8.reshape(n, k).astype(np.int8), sub.astype(np.int32), d, 16)
    raise ValueError(f"unsupported ggml type {t}")


def dequantize(raw: np.ndarray, t: int) -> np.ndarray:
    """float32 [N, K], in the float32 operation order of the C dequantiser."""
    dec = decode(raw, t)
    n, k = dec.w8.shape
    nb = k // QK_K
    g = dec.g
    d = dec.d.reshape(n, nb, 1).astype(np.float32)
    sub = dec.sub.reshape(n, nb, QK_K // g).astype(np.float32)
    w = dec.w8.reshape(n, nb, QK_K // g, g).astype(np.float32)
    half, quarter = np.float32(0.5), np.float32(0.25)
    if t == IQ3_XXS:
        db = (d * (half + sub)).astype(np.float32) * half
    elif t in (IQ2_XXS, IQ2_XS, IQ2_S):
        db = (d * (half + sub)).astype(np.float32) * quarter
    elif t == IQ1_M:
        db = (d * (2 * sub + 1)).astype(np.float32)
        return (db[..., None] * (w * np.float32(0.125))).astype(np.float32).reshape(n, k)   # g + delta = w8 / 8, exact
    else:  # Q2_K
        dl = (d * sub).astype(np.float32)
        ml = (dec.dmin.reshape(n, nb, 1).astype(np.float32) * dec.mins.reshape(n, nb, 16).astype(np.float32)).astype(np.float32)
        return ((dl[..., None] * w).astype(np.float32) - ml[..., None]).astype(np.float32).reshape(n, k)
    return (db.astype(np.float32)[..., None] * w).astype(np.float32).reshape(n, k)


def group_sums(dec: DecodedF1, q: np.ndarray) -> np.ndarray:
    """int32 [M, N, K/g]: S[c, r, s] = sum_i w8[r, g s + i] * q[c, g s + i]."""
    n, k = dec.w8.shape
    m = q.shape[0]
    g = dec.g
    w = dec.w8.reshape(n, k // g, g).astype(np.int32)
    a = q.reshape(m, k // g, g).astype(np.int32)
    return np.einsum("nsg,msg->mns", w, a, optimize=True).astype(np.int32)


def _tdiv(a, b):
    """C integer division (truncation toward zero)."""
    a = np.asarray(a, dtype=np.int64)
    return np.sign(a) * (np.abs(a) // b)


def product_q81(dec: DecodedF1, q: np.ndarray, d8: np.ndarray) -> np.ndarray:
    """float64 [M, N]: the reference's MMVQ arithmetic per 32-value block with exact integers, the float part in
    float64. q int8 [M, K]; d8 [M, K/32] activation scales (already rounded as stored)."""
    t = dec.type
    n, k = dec.w8.shape
    s = group_sums(dec, q).astype(np.int64)                      # [M, N, K/g]
    d = np.repeat(dec.d.astype(np.float64), 8, axis=1)           # [N, K/32]
    d8 = d8.astype(np.float64)
    if t == IQ3_XXS:
        ls = dec.sub.astype(np.int64)[None]
        v = _tdiv(ls * s + _tdiv(s, 2), 2)
    elif t == IQ2_XXS:
        ls = dec.sub.astype(np.int64)[None]
        v = _tdiv(s * (2 * ls + 1), 8)
    elif t in (IQ2_XS, IQ2_S):
        ls = dec.sub.astype(np.int64)[None]
        s0, s1, l0, l1 = s[..., 0::2], s[..., 1::2], ls[..., 0::2], ls[..., 1::2]
        v = _tdiv(s0 * l0 + s1 * l1 + _tdiv(s0 + s1, 2), 4)
    elif t == IQ1_M:
        sc = (2 * dec.sub.astype(np.int64) + 1)[None]
        v = (s[..., 0::2] * sc[..., 0::2] + s[..., 1::2] * sc[..., 1::2]).astype(np.float64) / 8.0
    elif t == Q2_K:
        m = q.shape[0]
        sq = q.reshape(m, k // 16, 16).astype(np.int64).sum(-1)                       # [M, K/16]
        d16 = np.repeat(dec.d.astype(np.float64), 16, axis=1)
        dm16 = np.repeat(dec.dmin.astype(np.float64), 16, axis=1)
        d8g = np.repeat(d8, 2, axis=1)                                                # [M, K/16]
        y = np.einsum("mns,ns,ms->mn", s.astype(np.float64), d16 * dec.sub, d8g, optimize=True)
        return y - (sq * d8g) @ (dm16 * dec.mins).T
    else:
        raise ValueError(t)
    return np.einsum("mns,ns,ms->mn", v.astype(np.float64), d, d8, optimize=True)


def product_full(raw: np.ndarray, t: int, x: np.ndarray) -> np.ndarray:
    return np.asarray(x).astype(np.float64) @ dequantize(raw, t).astype(np.float64).T
