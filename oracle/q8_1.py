"""CPU oracle (TEST INFRASTRUCTURE, not product code): q8_1 activation quantisation.

Restates the reference's owned quantisers in numpy float32:
  * MMVQ layout  -- quantize_q8_1_x, plugin/vllm_gguf_plugin/csrc/lcpp_shim.cu:274-294
    (block_q8_1 = half2(d, sum) then 32 x int8, 36 bytes, ggml-common.h:259-269);
    the warp sums follow the xor-shuffle tree 16,8,4,2,1 of
    csrc/lcpp/ggml/src/ggml-cuda/common.cuh:468-475.
  * MMQ layouts  -- quantize_mmq_q8_1_x, lcpp_shim.cu:298-355 (block_q8_1_mmq =
    16 scale bytes + 128 x int8 = 144 bytes, blocks stored [K/128][row],
    mmq.cuh:27-46): D4 keeps 4 fp32 d, DS4 keeps 4 half2(d, sum).
The reference's CPU model of the same arithmetic is tests/gpu/_refs.py:40-54.

PARITY NOTE: the reference is compiled with --use_fast_math
(plugin/setup.py:42), so x/d and 127/amax are approximate divisions on the GPU.
This float32 model is exact only on inputs without rounding ties
(`nudge_ties` below, the generator of tests/gpu/test_kernel_parity.py:76-99).
The reference holds no stored q8_1 golden bytes; "parity unpinned" on CPU except
through this restatement, and pinned GPU-vs-model on tie-free inputs.
"""

from __future__ import annotations

import numpy as np

QK8_1 = 32
BLOCK_Q8_1 = 36
QK8_1_MMQ = 128
BLOCK_Q8_1_MMQ = 144
LAYOUT_D4, LAYOUT_DS4 = 0, 1


def _roundf(t: np.ndarray) -> np.ndarray:
    """C roundf: half away from zero."""
    return np.sign(t) * np.floor(np.abs(t) + np.float32(0.5))


def _tree_sum(v: np.ndarray) -> np.ndarray:
    """Sum over the last axis (power of two) in butterfly order: offsets n/2, n/4, ..., 1."""
    v = v.astype(np.float32)
    while v.shape[-1] > 1:
        h = v.shape[-1] // 2
        v = (v[..., :h] + v[..., h:]).astype(np.float32)
    return v[..., 0]


def quantize_q8_1(x: np.ndarray):
    """x [M, K] (any float dtype; converted to float32 exactly) ->
    (q int8 [M, K], d_half float16 [M, K/32], sum_half float16 [M, K/32])."""
    xf = np.asarray(x).astype(np.float32)
    m, k = xf.shape
    assert k % QK8_1 == 0
    b = xf.reshape(m, k // QK8_1, QK8_1)
    amax = np.abs(b).max(-1)
    d = (amax / np.float32(127.0)).astype(np.float32)
    safe = np.where(d == 0, np.float32(1), d)
    with np.errstate(over="ignore", invalid="ignore"):
        t = (b / safe[..., None]).astype(np.float32)
    q = np.where((amax == 0)[..., None], np.float32(0), _roundf(t))
    s = _tree_sum(b)
    with np.errstate(over="ignore"):
        return q.astype(np.int8).reshape(m, k), d.astype(np.float16), s.astype(np.float16)


def q8_1_bytes(x: np.ndarray) -> np.ndarray:
    """The MMVQ-layout bytes lcpp_quantize_q8_1(X, type, mmq=False, vendored=False) returns:
    uint8 [M * K/32 * 36], row-major blocks, each half d, half sum, then 32 x int8."""
    q, d, s = quantize_q8_1(x)
    m, k = q.shape
    nb = k // QK8_1
    out = np.empty((m, nb, BLOCK_Q8_1), dtype=np.uint8)
    out[..., 0:2] = d.reshape(m, nb, 1).view(np.uint8)
    out[..., 2:4] = s.reshape(m, nb, 1).view(np.uint8)
    out[..., 4:36] = q.reshape(m, nb, 32).view(np.uint8)
    return out.reshape(-1)


def parse_q8_1_bytes(buf: np.ndarray, m: int, k: int):
    """Inverse view of q8_1_bytes: (q int8 [M,K], d f16 [M,K/32], sum f16 [M,K/32])."""
    nb = k // QK8_1
    b = np.ascontiguousarray(buf[: m * nb * BLOCK_Q8_1]).reshape(m, nb, BLOCK_Q8_1)
    d = np.ascontiguousarray(b[..., 0:2]).view(np.float16)[..., 0]
    s = np.ascontiguousarray(b[..., 2:4]).view(np.float16)[..., 0]
    q = np.ascontiguousarray(b[..., 4:36]).view(np.int8).reshape(m, k)
    return q, d, s


def quantize_mmq(x: np.ndarray, layout: int):
    """MMQ-style quantisation: d_inv = 127/amax, q = roundf(x * d_inv), d = 1/d_inv (fp32).
    No zero guard: an all-zero block gives d_inv = inf, x * d_inv = NaN, stored q = 0 on the GPU
    (float NaN -> int8 conversion saturates to 0) and d = 0.
    -> (q int8 [M,K], d float32 [M,K/32], sum float32 [M,K/32] (DS4 order: 4-value partials, then 4,2,1))."""
    xf = np.asarray(x).astype(np.float32)
    m, k = xf.shape
    assert k % QK8_1_MMQ == 0
    b = xf.reshape(m, k // 32, 32)
    amax = np.abs(b).max(-1)
    with np.errstate(divide="ignore", over="ignore", invalid="ignore"):
        d_inv = (np.float32(127.0) / amax).astype(np.float32)
        t = (b * d_inv[..., None]).astype(np.float32)
        q = _roundf(t)
        q = np.where(np.isnan(q), np.float32(0), q)
        d = (np.float32(1.0) / d_inv).astype(np.float32)
    p = b.reshape(m, k // 32, 8, 4)
    part = ((p[..., 0] + p[..., 1]).astype(np.float32) + p[..., 2]).astype(np.float32)
    part = (part + p[..., 3]).astype(np.float32)
    s = _tree_sum(part)
    return q.astype(np.int8).reshape(m, k), d, s


def q8_1_mmq_bytes(x: np.ndarray, layout: int) -> np.ndarray:
    """uint8 [K/128 * M * 144]: block (kb, row) at (kb * M + row) * 144 = 16 scale bytes + 128 int8."""
    q, d, s = quantize_mmq(x, layout)
    m, k = q.shape
    nkb = k // QK8_1_MMQ
    out = np.empty((nkb, m, BLOCK_Q8_1_MMQ), dtype=np.uint8)
    qq = q.reshape(m, nkb, 128).transpose(1, 0, 2)
    out[..., 16:] = np.ascontiguousarray(qq).view(np.uint8)
    d4 = d.reshape(m, nkb, 4).transpose(1, 0, 2)
    if layout == LAYOUT_D4:
        out[..., :16] = np.ascontiguousarray(d4).view(np.uint8).reshape(nkb, m, 16)
    else:
        s4 = s.reshape(m, nkb, 4).transpose(1, 0, 2)
        with np.errstate(over="ignore"):
            ds = np.stack([d4.astype(np.float16), s4.astype(np.float16)], -1)   # [nkb, m, 4, 2]
        out[..., :16] = np.ascontiguousarray(ds).view(np.uint8).reshape(nkb, m, 16)
    return out.reshape(-1)


def nudge_ties(x: np.ndarray, max_passes: int = 8) -> np.ndarray:
    """Move 16-bit inputs off q8_1 rounding ties: wherever |frac(|x| * 127/amax) - 0.5| < 1e-4 for
    the 32- or 64-value group, step the value's bit pattern one ulp toward zero; repeat until
    none is left (the generator of tests/gpu/test_kernel_parity.py:86-99). float32 input is
    returned unchanged, as there. x: float16 array, or bfloat16 given as uint16 bit patterns is not
    supported here (use torch for bf16 and pass through `nudge_ties_torch`)."""
    if x.dtype == np.float32:
        return x
    assert x.dtype == np.float16
    x = x.copy()
    n, k = x.shape
    for _ in range(max_passes):
        tie = np.zeros((n, k), dtype=bool)
        for qk in (32, 64):
            b = np.abs(x.astype(np.float32)).reshape(n, k // qk, qk)
            with np.errstate(divide="ignore", invalid="ignore"):
                t = b * (np.float32(127) / b.max(-1, keepdims=True))
            tie |= (np.abs(t - np.floor(t) - 0.5) < 1e-4).reshape(n, k)
        if not tie.any():
            return x
        bits = x.view(np.int16)
        x = np.where(tie, (bits - 1).astype(np.int16), bits).view(np.float16)
    raise AssertionError("could not remove q8_1 rounding ties")
