"""CPU model (numpy) of the arithmetic of the prefill kernels that put the scales into fp16 tensor-core operands
(gsq_gemm3.cu: gemm3_acc_kernel, with the activation units of quantize_q8_1_tiles_kernel). Test infrastructure: only
tests/ import this.

These kernels are not a restatement of a reference kernel: the reference forms exact int32 sums per 32-value slice and
scales them in fp32 (plugin/vllm_gguf_plugin/csrc/lcpp_owned_iq3_mma.cu:768-970, csrc/lcpp/ggml/src/ggml-cuda/
mmq.cuh:961-1385), which oracle/product.py models. This module models what the fp16-operand forms compute instead,
rounding for rounding, so that a test can hold the CUDA kernel to its own arithmetic at fp32 accuracy (a few 1e-7 of
a row's norm) rather than only to the 1e-3 that separates it from the reference's.

  activations   q, d as the reference's MMQ quantiser (oracle/q8_1.quantize_mmq); per token 2^e bringing its largest
                magnitude to [2^13, 2^14); p = d * q * 2^e (exact in fp32); hi = fp16(p), lo = fp16(p - hi)
  weights       IQ3_S:  (1 + 2 ls) * g                 exact in fp16
                IQ4_XS: fp16((ls - 32) * table value)  rounds above 2048
                Q4_K:   fp16(q * fp16(d / sigma * sc)), sigma = d unless |dmin| > 64 |d| or d = 0
  per superblock  C = sum_k A[k] * hi[k] (+ A[k] * lo[k], split form), Q4_K adds
                  sum_s fp16(-16 dmin / sigma * m_s) * fp16(half(sum x)_s * 2^e / 16)
                  + fp16(128 d / sigma * sc_s) * fp16(sum_k (p - hi)[k] / 16)
  result        y = 2^-e * sum_sb scale_sb * C_sb, scale = d (sigma for Q4_K)
"""

from __future__ import annotations

import numpy as np

from . import blocks, q8_1

IQ3_S, IQ4_XS, Q4_K = 21, 23, 12
f16, f32, f64 = np.float16, np.float32, np.float64


def scaled_products(x: np.ndarray, half_d: bool):
    """x [M, K] -> (hi f16 [M, K], lo f16 [M, K], inv_up f32 [M], sums f16 [M, K/32] or None, lost f16 [M, K/32])."""
    x = np.asarray(x, dtype=f32)
    m, k = x.shape
    q, d, s = q8_1.quantize_mmq(x, q8_1.LAYOUT_DS4 if half_d else q8_1.LAYOUT_D4)
    amax = np.abs(x).max(axis=1)
    _, e = np.frexp(amax)
    up_exp = np.clip(14 - e, -100, 100)
    up_exp = np.where((amax > 0) & (amax <= f32(3.0e38)), up_exp, 0)
    up = np.ldexp(f32(1.0), up_exp).astype(f32)
    sums = None
    if half_d:
        d = d.astype(f16).astype(f32)
        sums = ((s.astype(f16).astype(f32) * up[:, None]).astype(f32) * f32(0.0625)).astype(f16)
    ds = (d * up[:, None]).astype(f32)
    p = (np.repeat(ds, 32, axis=1) * q.astype(f32)).astype(f32)
    hi = p.astype(f16)
    rest = (p - hi.astype(f32)).astype(f32)
    lo = rest.astype(f16)
    lost = (rest.reshape(m, k // 32, 32).astype(f64).sum(-1).astype(f32) * f32(0.0625)).astype(f16)
    return hi, lo, (f32(1.0) / up).astype(f32), sums, lost


def q4k_sigma(d: np.ndarray, dmin: np.ndarray) -> np.ndarray:
    d, dmin = d.astype(f32), dmin.astype(f32)
    sigma = np.where(np.abs(dmin) > f32(64.0) * np.abs(d), (np.abs(dmin) * f32(1.0 / 64.0)).astype(f32), d)
    return np.where(sigma == 0, f32(1.0), sigma).astype(f32)


def weight_operand(raw: np.ndarray, t: int):
    """-> (A f16-valued float64 [N, K], scale f32 [N, K/256], terms: None or (hm, hs) f16 [N, K/32] each)."""
    dec = blocks.decode(raw, t)
    n, k = dec.w8.shape
    if t == IQ3_S:
        a = dec.w8.astype(f64) * np.repeat(dec.isc, 32, axis=1).astype(f64)
        assert np.abs(a).max() <= 465
        return a, dec.d.astype(f32), None
    if t == IQ4_XS:
        a = (dec.w8.astype(f32) * np.repeat(dec.isc, 32, axis=1).astype(f32)).astype(f16)
        return a.astype(f64), dec.d.astype(f32), None
    assert t == Q4_K
    sigma = q4k_sigma(dec.d, dec.dmin)
    with np.errstate(divide="ignore", invalid="ignore"):
        ratio = (dec.d.astype(f32) / sigma).astype(f32)
        fm = ((f32(-16.0) * dec.dmin.astype(f32)).astype(f32) / sigma).astype(f32)
    fs = (f32(128.0) * ratio).astype(f32)
    sc, mn = dec.isc.astype(f32), dec.imin.astype(f32)
    f = (np.repeat(ratio, 8, axis=1) * sc).astype(f32).astype(f16)                       # [N, K/32]
    a = (dec.w8.astype(f32) * np.repeat(f.astype(f32), 32, axis=1)).astype(f32).astype(f16)
    hm = (np.repeat(fm, 8, axis=1) * mn).astype(f32).astype(f16)
    hs = (np.repeat(fs, 8, axis=1) * sc).astype(f32).astype(f16)
    return a.astype(f64), sigma, (hm, hs)


def product(raw: np.ndarray, t: int, x: np.ndarray, split: bool = False) -> np.ndarray:
    """float64 [M, N]: the rounded form (split: the form with the fp16 pair, IQ3_S / IQ4_XS)."""
    a, scale, terms = weight_operand(raw, t)
    hi, lo, inv_up, sums, lost = scaled_products(x, t == Q4_K)
    n, k = a.shape
    m = hi.shape[0]
    b = hi.astype(f64) + (lo.astype(f64) if split else 0.0)
    nsb = k // 256
    c = np.einsum("nsk,msk->mns", a.reshape(n, nsb, 256), b.reshape(m, nsb, 256), optimize=True)   # [M, N, K/256]
    if terms is not None:
        hm, hs = terms
        c = c + np.einsum("nsj,msj->mns", hm.astype(f64).reshape(n, nsb, 8), sums.astype(f64).reshape(m, nsb, 8), optimize=True)
        c = c + np.einsum("nsj,msj->mns", hs.astype(f64).reshape(n, nsb, 8), lost.astype(f64).reshape(m, nsb, 8), optimize=True)
    y = np.einsum("mns,ns->mn", c, scale.astype(f64), optimize=True)
    return y * inv_up.astype(f64)[:, None]
