"""Routing: `_lcpp_op` against the reference's own function (golden table made by importing it,
tests/golden/make_golden.py) and against the cases its test pins (tests/cpu/test_lcpp_routing.py:14-116)."""

import json
import os

import pytest
import torch

from gsq_b200.quantization import linear

IQ3, MMA, OWN = "lcpp_mul_mat_vec_iq3", "lcpp_mul_mat_vec_iq3_mma", "lcpp_mul_mat_vec_own"
MMVQ, MMQ, MMA_K = "lcpp_mul_mat_vec_q", "lcpp_mul_mat_q", "lcpp_mul_mat_mma_k"
PACKED_VEC, PACKED_TILED = "lcpp_mul_mat_vec_iq3_mma_packed", "lcpp_mul_mat_iq3_packed"
Q4_K, Q6_K, IQ3_S, IQ4_XS, IQ1_M, IQ2_S, IQ2_XS = 12, 14, 21, 23, 29, 22, 17
BIG, K = 17408, 5120


def test_matches_reference_function_on_golden_grid(golden_dir):
    g = json.load(open(os.path.join(golden_dir, "routing.json")))
    assert len(g["cases"]) == 3800
    bad = [(n, t, rows, k, p, want, linear._lcpp_op(n, t, rows, k, p))
           for n, t, rows, k, p, want in g["cases"] if linear._lcpp_op(n, t, rows, k, p) != want]
    assert not bad, bad[:5]
    c = g["constants"]
    assert list(linear._OWN_QUANTIZE_OPS) == c["_OWN_QUANTIZE_OPS"]
    assert list(linear._X_DTYPE_OPS) == c["_X_DTYPE_OPS"]
    assert linear.PACKED_VEC_MAX_ROWS == c["PACKED_VEC_MAX_ROWS"]


@pytest.mark.parametrize("t,n,rows,want", [
    (IQ3_S, 1, 1024, IQ3), (IQ3_S, 5, BIG, IQ3), (IQ3_S, 6, BIG, MMA), (IQ3_S, 8, 1024, MMA), (IQ3_S, 9, BIG, MMQ),
    (Q4_K, 1, BIG, MMVQ), (Q4_K, 2, BIG, MMVQ), (Q4_K, 3, BIG, OWN), (Q4_K, 8, BIG, OWN), (Q4_K, 9, BIG, MMA_K),
    (Q4_K, 32, BIG, MMA_K), (Q4_K, 33, BIG, MMQ), (Q4_K, 3, 2049, OWN), (Q4_K, 4, 2048, MMVQ), (Q4_K, 8, 2048, MMQ),
    (IQ4_XS, 7, BIG, MMVQ), (IQ4_XS, 8, BIG, MMQ), (IQ4_XS, 16, 2049, MMA_K), (IQ4_XS, 17, 2049, MMQ),
    (IQ4_XS, 17, 12288, MMA_K), (IQ4_XS, 17, 12032, MMQ), (IQ4_XS, 33, BIG, MMQ),
    (Q6_K, 1, BIG, MMVQ), (Q6_K, 7, BIG, MMVQ), (Q6_K, 8, BIG, MMQ), (Q6_K, 32, BIG, MMQ),
    (IQ1_M, 9, BIG, MMVQ), (IQ1_M, 33, BIG, None),
])
def test_boundaries(t, n, rows, want):
    assert linear._lcpp_op(n, t, rows, K) == want
    assert linear._lcpp_op(n, t, rows, K, False) == want


@pytest.mark.parametrize("n,want", [(1, PACKED_VEC), (8, PACKED_VEC), (9, PACKED_TILED), (2048, PACKED_TILED)])
def test_packed(n, want):
    assert linear._lcpp_op(n, IQ3_S, BIG, K, True) == want
    assert linear._lcpp_op(3, Q4_K, BIG, K, True) == OWN      # a packed layer's other runs route as unpacked


class _Quantizer:
    """Stands in for torch.ops._C_gguf: records which type the shared quantise runs with."""

    def __init__(self):
        self.calls = []

    def lcpp_quantize_q8_1(self, x, qt, mmq, vendored):
        self.calls.append((qt, mmq, vendored))
        return "filled"


@pytest.mark.parametrize("n,types,rows,want,packed", [
    (4, [Q4_K, IQ2_XS], [2048, BIG], Q4_K, False),
    (8, [Q4_K], [BIG], Q4_K, False),
    (8, [Q4_K], [2048], None, False),
    (8, [IQ4_XS, Q4_K], [BIG, BIG], Q4_K, False),
    (8, [Q4_K, IQ3_S], [2048, BIG], IQ3_S, False),
    (9, [IQ3_S, Q4_K], [BIG, BIG], None, False),
    (16, [Q4_K, IQ1_M], [BIG, BIG], IQ1_M, False),
    (33, [IQ1_M, Q4_K], [BIG, BIG], None, False),
    (0, [IQ3_S], [BIG], None, False),
    (4, [IQ3_S, Q4_K], [BIG, BIG], IQ3_S, True),
    (9, [IQ3_S, IQ1_M], [BIG, BIG], IQ1_M, True),
])
def test_quantize_x_q8_1_fills(monkeypatch, n, types, rows, want, packed):
    """The shared quantise runs (once, block_q8_1 layout) iff some run's op reads q8_1; otherwise an
    unfilled buffer of the q8_1 size comes back."""
    q = _Quantizer()
    monkeypatch.setattr(torch.ops, "_C_gguf", q, raising=False)
    x = torch.zeros(n, 512, dtype=torch.bfloat16)
    out = linear._quantize_x_q8_1(x, [int(t) for t in types], rows, packed)
    if want is None:
        assert q.calls == [] and out.dtype == torch.uint8 and out.numel() == n * 512 // 32 * 36
    else:
        assert q.calls == [(int(want), False, False)] and out == "filled"


def test_zero_rows_return_before_routing():
    y = linear._fused_mul_mat_gguf(torch.zeros(0, 512, dtype=torch.bfloat16),
                                   torch.zeros(BIG, 512 // 256 * 110, dtype=torch.uint8), IQ3_S)
    assert y.shape == (0, BIG) and y.dtype == torch.bfloat16


def test_c_route():
    """gsq_route names the kernel family the library runs underneath the op names (what gsq_mul_mat_vec_q8 and
    gsq_linear choose)."""
    from gsq_b200 import _cabi

    r = _cabi.lib.gsq_route
    Q6_K, IQ4_XS = 14, 23
    assert r(1, IQ3_S, BIG, K, 1) == _cabi.KERNEL_MMV          # repacked IQ3_S: the tensor-core kernel from 1 row
    assert r(1, IQ3_S, BIG, K, 0) == _cabi.KERNEL_GEMV         # GGUF order: dp4a
    assert r(1, Q4_K, BIG, K, 0) == _cabi.KERNEL_GEMV and r(2, Q4_K, BIG, K, 0) == _cabi.KERNEL_MMV
    assert r(3, IQ4_XS, BIG, K, 0) == _cabi.KERNEL_GEMV and r(4, IQ4_XS, BIG, K, 0) == _cabi.KERNEL_MMV
    assert r(48, Q4_K, BIG, K, 0) == _cabi.KERNEL_MMV and r(49, Q4_K, BIG, K, 0) == _cabi.KERNEL_GEMM
    assert r(512, Q4_K, BIG, K, 0) == _cabi.KERNEL_GEMM_PREFILL and r(256, Q4_K, 5120, K, 0) == _cabi.KERNEL_GEMM_PREFILL
    assert r(255, Q4_K, 5120, K, 0) == _cabi.KERNEL_GEMM and r(128, Q4_K, BIG, K, 0) == _cabi.KERNEL_GEMM_PREFILL
    assert r(256, IQ4_XS, 5120, K, 0) == _cabi.KERNEL_GEMM_PREFILL and r(255, IQ4_XS, 5120, K, 0) == _cabi.KERNEL_GEMM
    assert r(128, IQ3_S, 17408, K, 1) == _cabi.KERNEL_GEMM_PREFILL and r(128, IQ3_S, 5120, K, 1) == _cabi.KERNEL_GEMM
    assert r(8192, Q6_K, 151936, K, 1) == _cabi.KERNEL_MMV     # repacked Q6_K: 48 rows per launch
    assert r(33, Q6_K, BIG, K, 0) == _cabi.KERNEL_GEMV         # GGUF order: dp4a, 8 rows per launch
    assert r(4, IQ2_S, BIG, K, 0) == _cabi.KERNEL_GEMV and r(300, IQ2_S, BIG, K, 0) == _cabi.KERNEL_GEMV   # low-bit types: dp4a
    assert r(4, 8, BIG, K, 0) == _cabi.KERNEL_NONE             # Q8_0: not a type of this route


def test_route_switch_keys_the_compile_cache():
    """The switch that changes apply()'s traced graph is registered where vLLM hashes its compile factors
    (plugin.py:156-161 of the reference does the same)."""
    reg = {}
    assert linear.register_compile_factor(reg) and callable(reg["VLLM_GGUF_LCPP"])
    import os

    assert reg["VLLM_GGUF_LCPP"]() == os.environ.get("VLLM_GGUF_LCPP")
    keep = reg["VLLM_GGUF_LCPP"]
    linear.register_compile_factor(reg)                # a second registration keeps the first entry
    assert reg["VLLM_GGUF_LCPP"] is keep


def test_prefill_precision_setting():
    """gsq_prefill_precision: a process-wide mode, returns the previous one, ignores values it does not know; the
    scratch gsq_linear asks for covers every form's activation units."""
    from gsq_b200 import _cabi, lcpp_ops

    lib = _cabi.lib
    assert lcpp_ops.set_prefill_precision(lcpp_ops.PREFILL_SPLIT) == lcpp_ops.PREFILL_ROUNDED      # rounded is the default
    try:
        assert lib.gsq_prefill_precision(99) == lcpp_ops.PREFILL_SPLIT and lib.gsq_prefill_precision(-1) == lcpp_ops.PREFILL_SPLIT
        assert lcpp_ops.set_prefill_precision(lcpp_ops.PREFILL_INTEGER) == lcpp_ops.PREFILL_SPLIT
    finally:
        assert lcpp_ops.set_prefill_precision(lcpp_ops.PREFILL_ROUNDED) == lcpp_ops.PREFILL_INTEGER
    m, k = 300, 5120
    blocks = (m + 255) // 256 * (k // 256)
    sb = lib.gsq_linear_scratch_bytes
    per_token = (m + 255) // 256 * 256 * 4

    def need(planes, sums):
        return blocks * (8 * planes * 16384 + (8192 if sums else 0)) + per_token

    # one fp16 plane of scaled products per slice in the default form (+ Q4_K's unit of sums), two in the split form
    for t, packed in ((IQ3_S, 1), (IQ4_XS, 0), (Q4_K, 0)):
        assert need(1, t == Q4_K) <= sb(BIG, m, k, t, packed) < need(2, False), t
    lcpp_ops.set_prefill_precision(lcpp_ops.PREFILL_SPLIT)
    try:
        assert sb(BIG, m, k, IQ3_S, 1) >= need(2, False)
    finally:
        lcpp_ops.set_prefill_precision(lcpp_ops.PREFILL_ROUNDED)
    assert sb(BIG, m, k, Q6_K, 1) < need(1, False)            # a type without a prefill GEMM: q8_1 blocks only
