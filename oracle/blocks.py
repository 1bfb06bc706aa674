"""CPU oracle (TEST INFRASTRUCTURE, not product code): GGUF weight-block codecs.

Restates, in numpy, how the reference's kernels read the four in-scope weight
formats. Block structs: csrc/lcpp/ggml/src/ggml-common.h:327-338 (block_q4_K),
362-368 (block_q6_K), 415-422 (block_iq3_s), 454-460 (block_iq4_xs), all under
plugin/vllm_gguf_plugin/. Integer decode follows the per-type vec_dot functions
in csrc/lcpp/ggml/src/ggml-cuda/vecdotq.cuh: 1211-1248 (IQ3_S), 1357-1380
(IQ4_XS), 918-966 + 508-531 (Q4_K), 1019-1043 + 627-648 (Q6_K).

The float dequantisation (`dequantize`) reproduces gguf-py's
`gguf.quants.dequantize` bit for bit; the reference pins gguf-py against
llama.cpp's C dequantiser on 84 real rows
(tests/cpu/test_dequant_fixtures.py:54-64). Pinned here by
tests/test_oracle_blocks.py against those fixtures (read from the reference
tree when it is present) and against committed gguf-py outputs on seeded blocks.

Only tests/, __graft_entry__.smoke() and bench.py's cpu_baseline / reference
arm may import this package.
"""

from __future__ import annotations

import json
import os
from dataclasses import dataclass

import numpy as np

Q4_K, Q6_K, IQ3_S, IQ4_XS = 12, 14, 21, 23
TYPE_NAMES = {Q4_K: "Q4_K", Q6_K: "Q6_K", IQ3_S: "IQ3_S", IQ4_XS: "IQ4_XS"}
TYPE_IDS = {v: k for k, v in TYPE_NAMES.items()}
BLOCK_BYTES = {Q4_K: 144, Q6_K: 210, IQ3_S: 110, IQ4_XS: 136}
QK_K = 256

_TABLES = None


def tables():
    """(iq3s_grid uint8 [512,4], iq4nl_values int8 [16]) from oracle/tables.json."""
    global _TABLES
    if _TABLES is None:
        with open(os.path.join(os.path.dirname(os.path.abspath(__file__)), "tables.json")) as f:
            t = json.load(f)
        _TABLES = (np.asarray(t["iq3s_grid"], dtype=np.uint8), np.asarray(t["iq4nl_values"], dtype=np.int8))
    return _TABLES


@dataclass
class Decoded:
    """Integer view of a weight matrix.

    w8    int8  [N, K]      integer weight value fed to the int8 dot product
    isc   int32 [N, K/g]    integer sub-scale of each group of g values
    imin  int32 [N, K/32]   Q4_K only: 6-bit min of each 32-value sub-block
    d     f32   [N, K/256]  superblock scale (from fp16)
    dmin  f32   [N, K/256]  Q4_K only
    g     values per integer sub-scale (32; 16 for Q6_K)
    """

    type: int
    w8: np.ndarray
    isc: np.ndarray
    d: np.ndarray
    g: int = 32
    imin: np.ndarray | None = None
    dmin: np.ndarray | None = None


def _blocks(raw: np.ndarray, t: int) -> np.ndarray:
    raw = np.ascontiguousarray(raw, dtype=np.uint8)
    if raw.ndim == 1:
        raw = raw[None]
    n, rb = raw.shape
    bs = BLOCK_BYTES[t]
    assert rb % bs == 0, (rb, bs)
    return raw.reshape(n, rb // bs, bs)


def _f16(b: np.ndarray) -> np.ndarray:
    return np.ascontiguousarray(b).view(np.float16).astype(np.float32)[..., 0]


def q4k_scale_min(scales: np.ndarray):
    """12 packed bytes -> (sc[8], m[8]) six-bit values (get_scale_min_k4, vecdotq.cuh:932-946)."""
    s = scales.astype(np.int32)
    sc = np.empty(s.shape[:-1] + (8,), dtype=np.int32)
    m = np.empty_like(sc)
    for j in range(4):
        sc[..., j] = s[..., j] & 63
        m[..., j] = s[..., j + 4] & 63
    for j in range(4, 8):
        sc[..., j] = (s[..., j + 4] & 0x0F) | ((s[..., j - 4] >> 6) << 4)
        m[..., j] = (s[..., j + 4] >> 4) | ((s[..., j] >> 6) << 4)
    return sc, m


def decode(raw: np.ndarray, t: int) -> Decoded:
    b = _blocks(raw, t)
    n, nb, _ = b.shape
    k = nb * QK_K
    if t == IQ3_S:
        grid, _ = tables()
        d = _f16(b[..., 0:2])
        qs = b[..., 2:66].astype(np.int32)                     # [n, nb, 64] low 8 index bits per 4-value group
        qh = b[..., 66:74].astype(np.int32)                    # [n, nb, 8]  bit e of byte s = 9th bit of group 8s+e
        signs = b[..., 74:106]                                 # [n, nb, 32] bit i of byte j = sign of value 8j+i
        scales = b[..., 106:110].astype(np.int32)              # 4-bit sub-scale per 32 values
        hi = (qh[..., :, None] >> np.arange(8)) & 1            # [n, nb, 8, 8]
        idx = qs | (hi.reshape(n, nb, 64) << 8)
        mag = grid[idx].astype(np.int32)                       # [n, nb, 64, 4]
        sg = (signs[..., :, None] >> np.arange(8, dtype=np.uint8)) & 1
        sg = sg.reshape(n, nb, 64, 4).astype(np.int32)
        w8 = (mag * (1 - 2 * sg)).reshape(n, k).astype(np.int8)
        ls = np.stack([scales & 0x0F, scales >> 4], -1).reshape(n, nb * 8)
        return Decoded(t, w8, (1 + 2 * ls).astype(np.int32), d)
    if t == IQ4_XS:
        _, kv = tables()
        d = _f16(b[..., 0:2])
        sh = np.ascontiguousarray(b[..., 2:4]).view(np.uint16)[..., 0].astype(np.int32)   # [n, nb]
        sl = b[..., 4:8].astype(np.int32)
        qs = b[..., 8:136].reshape(n, nb, 8, 16)
        lo = np.stack([sl & 0x0F, sl >> 4], -1).reshape(n, nb, 8)
        hi = (sh[..., None] >> (2 * np.arange(8))) & 3
        ls = lo | (hi << 4)
        q = np.concatenate([qs & 0x0F, qs >> 4], -1)           # [n, nb, 8, 32]: value i<16 low nibble, i>=16 high
        w8 = kv[q].reshape(n, k)
        return Decoded(t, w8, (ls - 32).reshape(n, nb * 8).astype(np.int32), d)
    if t == Q4_K:
        d = _f16(b[..., 0:2])
        dmin = _f16(b[..., 2:4])
        sc, m = q4k_scale_min(b[..., 4:16])
        qs = b[..., 16:144].reshape(n, nb, 4, 32)
        q = np.stack([qs & 0x0F, qs >> 4], 3)                  # [n, nb, 4, 2, 32]
        w8 = q.reshape(n, k).astype(np.int8)
        return Decoded(t, w8, sc.reshape(n, nb * 8), d, 32, m.reshape(n, nb * 8), dmin)
    if t == Q6_K:
        ql = b[..., 0:128].reshape(n, nb, 2, 64)
        qh = b[..., 128:192].reshape(n, nb, 2, 32)
        sc = np.ascontiguousarray(b[..., 192:208]).view(np.int8).astype(np.int32)
        d = _f16(b[..., 208:210])
        l4 = np.stack([ql[..., :32] & 0x0F, ql[..., 32:] & 0x0F, ql[..., :32] >> 4, ql[..., 32:] >> 4], 3)
        h2 = np.stack([(qh >> s) & 3 for s in (0, 2, 4, 6)], 3)  # [n, nb, 2, 4, 32]
        q = (l4 | (h2 << 4)).astype(np.int32) - 32
        return Decoded(t, q.reshape(n, k).astype(np.int8), sc.reshape(n, nb * 16), d, 16)
    raise ValueError(f"unsupported ggml type {t}")


def dequantize(raw: np.ndarray, t: int) -> np.ndarray:
    """float32 [N, K], the same float32 operation order as gguf-py's dequantize_blocks."""
    dec = decode(raw, t)
    n, k = dec.w8.shape
    nb = k // QK_K
    g = dec.g
    d = dec.d.reshape(n, nb, 1).astype(np.float32)
    ds = (d * dec.isc.reshape(n, nb, QK_K // g).astype(np.float32)).astype(np.float32)   # [n, nb, 256/g]
    w = dec.w8.reshape(n, nb, QK_K // g, g).astype(np.float32)
    out = (ds[..., None] * w).astype(np.float32)
    if t == Q4_K:
        dm = (dec.dmin.reshape(n, nb, 1) * dec.imin.reshape(n, nb, 8).astype(np.float32)).astype(np.float32)
        out = (out - dm[..., None]).astype(np.float32)
    return out.reshape(n, k)


def group_scales(dec: Decoded) -> np.ndarray:
    """float64 [N, K/g]: d * integer sub-scale, exact (used by the reference product models)."""
    n, k = dec.w8.shape
    per = QK_K // dec.g
    return np.repeat(dec.d.astype(np.float64), per, axis=1) * dec.isc.astype(np.float64)
