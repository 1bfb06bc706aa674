"""Seeded synthetic GGUF weight blocks and activations.

Stands in for the model file the reference measures on (its kit/synth.py:70-87 makes random-byte
blocks with finite scales for the same purpose). Blocks here are written field by field so the
value distributions are the stated ones:

  IQ3_S   d = f16(|N(0,1)| * 2e-3); 4 scale bytes uniform 0..255; the 64 nine-bit grid indices
          uniform on 0..511 (qs = low 8 bits, qh = 9th bits); 32 sign bytes uniform
  IQ4_XS  d = f16(|N(0,1)| * 1e-2); 8 six-bit scales uniform 0..63 (scales_l / scales_h);
          128 bytes of 4-bit indices uniform
  Q4_K    d, dmin = f16(|N(0,1)| * 1e-2); 8 six-bit sc and 8 six-bit m uniform 0..63 packed into
          12 bytes; 128 bytes of nibbles uniform
  Q6_K    ql[128], qh[64] uniform; 16 int8 sub-scales uniform; d = f16(|N(0,1)| * 1e-2)
  Q2_K, IQ2_XXS, IQ2_XS, IQ2_S, IQ3_XXS, IQ1_M (the other types of the model file): every index, sign and
          sub-scale byte uniform; d (and Q2_K's dmin) = f16(|N(0,1)| * 5e-3); IQ1_M's d is spread over the top
          nibbles of its four scale words as the format has it

Everything is numpy on the host; callers move the bytes to the GPU.
"""

from __future__ import annotations

import numpy as np

Q4_K, Q6_K, IQ3_S, IQ4_XS = 12, 14, 21, 23
Q2_K, IQ2_XXS, IQ2_XS, IQ3_XXS, IQ2_S, IQ1_M = 10, 16, 17, 18, 22, 29
BLOCK_BYTES = {Q4_K: 144, Q6_K: 210, IQ3_S: 110, IQ4_XS: 136, Q2_K: 84, IQ2_XXS: 66, IQ2_XS: 74, IQ3_XXS: 98, IQ2_S: 82,
               IQ1_M: 56}
TYPE_IDS = {"Q4_K": Q4_K, "Q6_K": Q6_K, "IQ3_S": IQ3_S, "IQ4_XS": IQ4_XS}
LOW_BIT_TYPE_IDS = {"Q2_K": Q2_K, "IQ2_XXS": IQ2_XXS, "IQ2_XS": IQ2_XS, "IQ3_XXS": IQ3_XXS, "IQ2_S": IQ2_S, "IQ1_M": IQ1_M}


def _f16_scale(rng, shape, mult):
    return (np.abs(rng.standard_normal(shape)) * mult).astype(np.float16)


def make_weight(ggml_type: int, rows: int, k: int, seed: int) -> np.ndarray:
    """uint8 [rows, k/256 * block_bytes] of valid blocks."""
    assert k % 256 == 0
    rng = np.random.default_rng(seed)
    nb = k // 256
    bs = BLOCK_BYTES[ggml_type]
    out = np.empty((rows, nb, bs), dtype=np.uint8)
    if ggml_type == IQ3_S:
        out[..., 0:2] = _f16_scale(rng, (rows, nb, 1), 2e-3).view(np.uint8)
        idx = rng.integers(0, 512, size=(rows, nb, 64), dtype=np.uint16)
        out[..., 2:66] = (idx & 0xFF).astype(np.uint8)
        hi = (idx >> 8).astype(np.uint8).reshape(rows, nb, 8, 8)
        out[..., 66:74] = (hi << np.arange(8, dtype=np.uint8)).sum(-1).astype(np.uint8)
        out[..., 74:106] = rng.integers(0, 256, size=(rows, nb, 32), dtype=np.uint8)
        out[..., 106:110] = rng.integers(0, 256, size=(rows, nb, 4), dtype=np.uint8)
    elif ggml_type == IQ4_XS:
        out[..., 0:2] = _f16_scale(rng, (rows, nb, 1), 1e-2).view(np.uint8)
        ls = rng.integers(0, 64, size=(rows, nb, 8), dtype=np.uint16)
        sh = ((ls >> 4) << (2 * np.arange(8, dtype=np.uint16))).sum(-1).astype(np.uint16)
        out[..., 2:4] = sh.reshape(rows, nb, 1).view(np.uint8)
        lo = (ls & 0x0F).astype(np.uint8)
        out[..., 4:8] = lo[..., 0::2] | (lo[..., 1::2] << 4)
        out[..., 8:136] = rng.integers(0, 256, size=(rows, nb, 128), dtype=np.uint8)
    elif ggml_type == Q4_K:
        out[..., 0:2] = _f16_scale(rng, (rows, nb, 1), 1e-2).view(np.uint8)
        out[..., 2:4] = _f16_scale(rng, (rows, nb, 1), 1e-2).view(np.uint8)
        sc = rng.integers(0, 64, size=(rows, nb, 8), dtype=np.uint8)
        mn = rng.integers(0, 64, size=(rows, nb, 8), dtype=np.uint8)
        s = np.empty((rows, nb, 12), dtype=np.uint8)
        s[..., 0:4] = (sc[..., 0:4] & 63) | ((sc[..., 4:8] >> 4) << 6)
        s[..., 4:8] = (mn[..., 0:4] & 63) | ((mn[..., 4:8] >> 4) << 6)
        s[..., 8:12] = (sc[..., 4:8] & 0x0F) | ((mn[..., 4:8] & 0x0F) << 4)
        out[..., 4:16] = s
        out[..., 16:144] = rng.integers(0, 256, size=(rows, nb, 128), dtype=np.uint8)
    elif ggml_type == Q6_K:
        out[..., 0:192] = rng.integers(0, 256, size=(rows, nb, 192), dtype=np.uint8)
        out[..., 192:208] = rng.integers(-128, 128, size=(rows, nb, 16), dtype=np.int8).view(np.uint8)
        out[..., 208:210] = _f16_scale(rng, (rows, nb, 1), 1e-2).view(np.uint8)
    elif ggml_type in (IQ2_XXS, IQ2_XS, IQ2_S, IQ3_XXS):
        out[...] = rng.integers(0, 256, size=(rows, nb, bs), dtype=np.uint8)
        out[..., 0:2] = _f16_scale(rng, (rows, nb, 1), 5e-3).view(np.uint8)
    elif ggml_type == Q2_K:
        out[...] = rng.integers(0, 256, size=(rows, nb, bs), dtype=np.uint8)
        out[..., 80:82] = _f16_scale(rng, (rows, nb, 1), 5e-3).view(np.uint8)
        out[..., 82:84] = _f16_scale(rng, (rows, nb, 1), 5e-3).view(np.uint8)
    elif ggml_type == IQ1_M:
        out[...] = rng.integers(0, 256, size=(rows, nb, bs), dtype=np.uint8)
        d = _f16_scale(rng, (rows, nb, 1), 5e-3).view(np.uint16).astype(np.uint32)[..., 0]
        sc = out[..., 48:56].copy().view(np.uint16).astype(np.uint32) & 0x0FFF
        for j in range(4):   # nibble j of d sits in the top nibble of scale word j
            sc[..., j] |= ((d >> (4 * j)) & 0xF) << 12
        out[..., 48:56] = sc.astype(np.uint16).view(np.uint8)
    else:
        raise ValueError(f"unsupported ggml type {ggml_type}")
    return out.reshape(rows, nb * bs)


def make_activation(m: int, k: int, seed: int, outliers: float = 0.0) -> np.ndarray:
    """float32 [m, k] ~ N(0,1); `outliers` = fraction of entries multiplied by 20."""
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((m, k)).astype(np.float32)
    if outliers > 0:
        x = np.where(rng.random((m, k)) < outliers, x * 20.0, x).astype(np.float32)
    return x


def nudge_ties_torch(x):
    """Move a 16-bit torch tensor off q8_1 rounding ties (x * 127/amax within 1e-4 of j + 0.5 for
    its 32- or 64-value group) by stepping the bit pattern one ulp toward zero, as the reference's
    parity-test input generator does (tests/gpu/test_kernel_parity.py:86-99). On such ties the
    GPU's approximate division may round either way, so no host model can be exact there."""
    import torch

    if x.dtype == torch.float32:
        return x
    n, k = x.shape
    for _ in range(8):
        tie = torch.zeros(n, k, dtype=torch.bool)
        for qk in (32, 64):
            b = x.float().abs().view(n, k // qk, qk)
            t = b * (127 / b.amax(-1, keepdim=True))
            tie |= ((t - t.floor() - 0.5).abs() < 1e-4).view(n, k)
        if not tie.any():
            return x
        x = torch.where(tie, (x.view(torch.int16) - 1).view(x.dtype), x)
    raise AssertionError("could not remove q8_1 rounding ties from x")
