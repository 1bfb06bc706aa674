"""CPU oracle (TEST INFRASTRUCTURE, not product code): the quantised product Y = Xq . W^T.

Three levels, from exact to loose:
  * block_sums       -- the int32 dot product of every 32-value slice (16 for Q6_K), the
                        `sumi` of csrc/lcpp/ggml/src/ggml-cuda/vecdotq.cuh:1233-1243 (IQ3_S),
                        1365-1374 (IQ4_XS), 517-524 (Q4_K `dot1`/`dot2`), 640-645 (Q6_K), and the
                        `C` tile of the reference's mma kernels. Pure integer arithmetic, so any
                        exact kernel must reproduce it bit for bit.
  * product_q81      -- float64 evaluation of the formula the reference's MMVQ kernels compute in
                        fp32: sum over slices of d_w * d_q8 * sub_scale * sumi (vecdotq.cuh:
                        1245-1247, 1376-1379, 526-530, 647) with the q8_1 scale rounded to half.
                        This is the "q81" model of tests/gpu/_refs.py:78-91 with exact slice sums.
  * product_xsum     -- Q4_K through the MMQ-family kernels: the min term uses half(sum x) of each
                        32-value activation block instead of d_q8 * sum(q) (the DS4 layout,
                        lcpp_owned_mma_k.cu:151-188; "xsum" model of _refs.py:84-86).
  * product_full     -- float64 X @ dequant(W)^T ("full" in _refs.py).
`rel_err` is the reference's acceptance metric (_refs.py:94-99): max over activation rows of
||y - ref|| / ||ref||.
"""

from __future__ import annotations

import numpy as np

from . import blocks


def block_sums(dec: blocks.Decoded, q: np.ndarray) -> np.ndarray:
    """int32 [M, N, K/g]: S[c, r, s] = sum_i w8[r, g*s+i] * q[c, g*s+i]."""
    n, k = dec.w8.shape
    m = q.shape[0]
    g = dec.g
    w = dec.w8.reshape(n, k // g, g).astype(np.int32)
    a = q.reshape(m, k // g, g).astype(np.int32)
    return np.einsum("nsg,msg->mns", w, a, optimize=True).astype(np.int32)


def q8_sums(q: np.ndarray, g: int = 32) -> np.ndarray:
    """int32 [M, K/g]: sum of the activation quants of each group (Q4_K's `dot2`)."""
    m, k = q.shape
    return q.reshape(m, k // g, g).astype(np.int32).sum(-1)


def product_q81(dec: blocks.Decoded, q: np.ndarray, d8: np.ndarray) -> np.ndarray:
    """float64 [M, N]. q int8 [M,K]; d8 [M, K/32] activation scales (already rounded as stored)."""
    n, k = dec.w8.shape
    g = dec.g
    gs = blocks.group_scales(dec)                                    # [N, K/g]
    d8g = np.repeat(d8.astype(np.float64), 32 // g, axis=1)          # [M, K/g]
    s = block_sums(dec, q).astype(np.float64)                        # [M, N, K/g]
    y = np.einsum("mns,ns,ms->mn", s, gs, d8g, optimize=True)
    if dec.imin is not None:
        mins = np.repeat(dec.dmin.astype(np.float64), 8, axis=1) * dec.imin.astype(np.float64)   # [N, K/32]
        qs = q8_sums(q).astype(np.float64) * d8.astype(np.float64)                                # [M, K/32]
        y = y - qs @ mins.T
    return y


def product_xsum(dec: blocks.Decoded, q: np.ndarray, d8: np.ndarray, xsum: np.ndarray) -> np.ndarray:
    """Q4_K with the min term taken from the stored activation-block sums xsum [M, K/32]."""
    assert dec.imin is not None
    gs = blocks.group_scales(dec)
    s = block_sums(dec, q).astype(np.float64)
    y = np.einsum("mns,ns,ms->mn", s, gs, d8.astype(np.float64), optimize=True)
    mins = np.repeat(dec.dmin.astype(np.float64), 8, axis=1) * dec.imin.astype(np.float64)
    return y - xsum.astype(np.float64) @ mins.T


def product_full(raw: np.ndarray, t: int, x: np.ndarray) -> np.ndarray:
    return np.asarray(x).astype(np.float64) @ blocks.dequantize(raw, t).astype(np.float64).T


def rel_err(y: np.ndarray, ref: np.ndarray) -> float:
    y = np.asarray(y, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    if y.size == 0:
        return 0.0
    num = np.linalg.norm(y - ref, axis=-1)
    den = np.maximum(np.linalg.norm(ref, axis=-1), 1e-30)
    return float((num / den).max())


def cpu_reference_linear(raw: np.ndarray, t: int, x: np.ndarray, threads: int | None = None):
    """The reference's CPU path for one linear: dequantise W (tools/ggml_ref.py:48-56 does this through
    libggml-base; gguf-py, which the reference pins bit-identical to it, is what `blocks.dequantize`
    restates) then an fp32 matmul on the host cores. -> (y float32 [M,N], seconds_dequant, seconds_matmul)."""
    import time

    import torch

    if threads:
        torch.set_num_threads(threads)
    t0 = time.perf_counter()
    w = blocks.dequantize(raw, t)
    t1 = time.perf_counter()
    y = torch.from_numpy(np.asarray(x, dtype=np.float32)) @ torch.from_numpy(w).T
    t2 = time.perf_counter()
    return y.numpy(), t1 - t0, t2 - t1
