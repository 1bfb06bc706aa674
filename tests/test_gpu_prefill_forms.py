"""The three forms of the prefill product of repacked IQ3_S (gsq_prefill_precision) against the reference kernels'
arithmetic (exact integer slice sums scaled in fp32: lcpp_owned_iq3_mma.cu:768-970), restated in float64 by the oracle:

  integer  the same arithmetic: <= 2e-6 of the row norm (fp32 accumulation order)
  split    d_x * q as an fp16 pair, sums over a superblock in tensor memory: <= 5e-6
  rounded  d_x * q as one fp16 number (the default): <= 1e-3, the bound stated for this path; about 3e-4 measured

on inputs that stress the per-token power-of-two scaling of the fp16 operands: blocks and whole tokens of zeros,
an outlier channel, activations from 1e-30 to 3e4, token counts that do not fill a block of 256, row counts that do
not fill a tile of 128."""

import ctypes
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import gsq_b200  # noqa: F401
from gsq_b200 import _cabi, lcpp_ops, synth
from gsq_b200.quantization import iq3_pack
from oracle import blocks, product, q8_1

pytestmark = pytest.mark.gpu
IQ3_S = 21
DEV = "cuda:0"
FORMS = {"rounded": (6, 1e-3), "split": (5, 5e-6), "integer": (7, 2e-6)}


def _case(rows, k, m, scale, seed, dtype=torch.float32):
    raw = synth.make_weight(IQ3_S, rows, k, seed)
    w = torch.from_numpy(raw).to(DEV)
    iq3_pack.pack_(w, IQ3_S)
    xa = synth.make_activation(m, k, seed + 1).astype(np.float64) * scale
    xa[min(3, m - 1), :64] = 0.0                      # two blocks of zeros
    if m > 100:
        xa[100, :] = 0.0                              # a token of zeros
    xa[min(5, m - 1), 7] = 40.0 * scale               # an outlier channel
    # values a 16-bit type holds, off the quantiser's rounding ties (bf16 for the fp32 cases: the range)
    x = synth.nudge_ties_torch(torch.from_numpy(xa.astype(np.float32)).to(torch.bfloat16 if dtype == torch.float32 else dtype)).to(dtype)
    q, d, _ = q8_1.quantize_mmq(x.float().numpy(), q8_1.LAYOUT_D4)
    return raw, w, x, product.product_q81(blocks.decode(raw, IQ3_S), q, d)


def _run(form, w, x, rows):
    old = _cabi.lib.gsq_debug_gemm_variant(form)
    old_mode = _cabi.lib.gsq_debug_mmv_mode(1)          # the prefill kernel at every token count, also below 49
    try:
        y = torch.ops._C_gguf.lcpp_mul_mat_iq3_packed(w, x.to(DEV), IQ3_S, rows)
        torch.cuda.synchronize()
    finally:
        _cabi.lib.gsq_debug_gemm_variant(old)
        _cabi.lib.gsq_debug_mmv_mode(old_mode)
    return y


@pytest.mark.parametrize("rows,k,m,scale", [(144, 1024, 70, 1.0), (128, 512, 300, 1e-3), (272, 5120, 700, 300.0),
                                            (256, 2048, 257, 3e4), (128, 1024, 512, 1e-30), (16, 512, 1, 1.0)])
def test_forms_against_the_reference_arithmetic(rows, k, m, scale):
    raw, w, x, ref = _case(rows, k, m, scale, 900 + rows + m)
    errs = {}
    for name, (form, tol) in FORMS.items():
        y = _run(form, w, x, rows)
        assert y.shape == (m, rows) and y.dtype == torch.float32
        got = y.cpu().numpy()
        assert np.isfinite(got).all(), name
        errs[name] = product.rel_err(got, ref)
        assert errs[name] <= tol, (name, errs)
        if m > 100:
            assert not got[100].any(), name           # a token of zeros gives zeros in every form
    print(f"{rows}x{k} m={m} scale {scale}:", {n: f"{e:.2e}" for n, e in errs.items()})


@pytest.mark.parametrize("dtype,tol", [(torch.float16, 1e-3), (torch.bfloat16, 5e-3)])
def test_forms_16bit(dtype, tol):
    raw, w, x, ref = _case(256, 1024, 300, 1.0, 77, dtype)
    for name, (form, _) in FORMS.items():
        y = _run(form, w, x, 256)
        assert y.dtype == dtype
        assert product.rel_err(y.float().cpu().numpy(), ref) <= tol, name


def test_default_route_and_the_setting():
    """The library's own choice from 256 tokens on is the rounded form; gsq_prefill_precision switches it, and a form is
    reproducible bit for bit from call to call."""
    raw, w, x, ref = _case(272, 2048, 300, 1.0, 55)
    lib = _cabi.lib
    forced = {name: _run(form, w, x, 272) for name, (form, _) in FORMS.items()}
    assert lib.gsq_debug_gemm_variant(0) == 0
    modes = {"rounded": lcpp_ops.PREFILL_ROUNDED, "split": lcpp_ops.PREFILL_SPLIT, "integer": lcpp_ops.PREFILL_INTEGER}
    assert lcpp_ops.set_prefill_precision(lcpp_ops.PREFILL_ROUNDED) == lcpp_ops.PREFILL_ROUNDED      # the default
    try:
        for name, mode in modes.items():
            lcpp_ops.set_prefill_precision(mode)
            y = torch.ops._C_gguf.lcpp_mul_mat_iq3_packed(w, x.to(DEV), IQ3_S, 272)
            assert torch.equal(y, forced[name]), name
        assert lcpp_ops.set_prefill_precision(17) == lcpp_ops.PREFILL_INTEGER                        # ignored
        assert lcpp_ops.set_prefill_precision(lcpp_ops.PREFILL_ROUNDED) == lcpp_ops.PREFILL_INTEGER
    finally:
        lcpp_ops.set_prefill_precision(lcpp_ops.PREFILL_ROUNDED)
    assert not torch.equal(forced["rounded"], forced["integer"])
    flag = ctypes.c_int(-1)
    assert lib.gsq_device_error_flag(ctypes.byref(flag)) == 0 and flag.value == 0


def test_environment_variable_sets_the_form():
    code = ("import gsq_b200, sys\nfrom gsq_b200 import lcpp_ops\n"
            "sys.exit(10 + lcpp_ops.set_prefill_precision(lcpp_ops.PREFILL_ROUNDED))")
    env = dict(os.environ, GSQ_PREFILL_PRECISION="split")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env["PYTHONPATH"] = os.pathsep.join([os.path.join(root, "vllm-gsqrco-exl3_b200"), root, env.get("PYTHONPATH", "")])
    assert subprocess.run([sys.executable, "-c", code], env=env).returncode == 10 + lcpp_ops.PREFILL_SPLIT
    env["GSQ_PREFILL_PRECISION"] = "nonsense"
    assert subprocess.run([sys.executable, "-c", code], env=env, stderr=subprocess.DEVNULL).returncode not in (10, 11, 12)


@pytest.mark.parametrize("rows,k,m", [(272, 5120, 700), (128, 512, 40), (1024, 1024, 1000)])
def test_two_cta_form_is_bit_identical(rows, k, m):
    """The same sums formed by pairs of CTAs (tcgen05 cta_group::2: 256 weight rows per instruction, each CTA decoding
    its 128 rows and copying its half of the tokens; an odd count of row tiles leaves a pair's second CTA without rows):
    the results of the rounded and the split form are those of the one-CTA kernels bit for bit. It measured slower
    than one CTA per item (the second half of the activation operand comes from the peer's shared memory) and is
    reached through the debug switch only."""
    raw, w, x, ref = _case(rows, k, m, 1.0, 300 + rows)
    assert torch.equal(_run(8, w, x, rows), _run(6, w, x, rows))
    assert torch.equal(_run(9, w, x, rows), _run(5, w, x, rows))
    flag = ctypes.c_int(-1)
    assert _cabi.lib.gsq_device_error_flag(ctypes.byref(flag)) == 0 and flag.value == 0


IQ4_XS, Q4_K = 23, 12


def _reference_q4k(raw, x):
    """The reference kernels' Q4_K arithmetic in float64: half d and half sum x per block, d * sc and dmin * m rounded
    to fp16 by its tile loader (mmq-load-tiles.cuh:775-780)."""
    dec = blocks.decode(raw, Q4_K)
    q, d, s = q8_1.quantize_mmq(x.numpy(), q8_1.LAYOUT_DS4)
    dh, sh = d.astype(np.float16).astype(np.float64), s.astype(np.float16).astype(np.float64)
    gs = (np.repeat(dec.d, 8, axis=1).astype(np.float16) * dec.isc.astype(np.float16)).astype(np.float64)
    mins = (np.repeat(dec.dmin, 8, axis=1).astype(np.float16) * dec.imin.astype(np.float16)).astype(np.float64)
    sums = product.block_sums(dec, q).astype(np.float64)
    return np.einsum("mns,ns,ms->mn", sums, gs, dh, optimize=True) - sh @ mins.T


@pytest.mark.parametrize("t", [IQ4_XS, Q4_K])
@pytest.mark.parametrize("rows,k,m,scale", [(128, 512, 256, 1.0), (202, 5120, 70, 1e-3), (300, 1024, 700, 3e4), (130, 17408, 300, 1.0)])
def test_gguf_order_types_on_fp16_operands(t, rows, k, m, scale):
    """IQ4_XS and Q4_K (GGUF order) on the same kernel, in its rounded form only.
    IQ4_XS: (ls - 32) * table value goes into the fp16 weight operand with one rounding (exact up to 2048; the odd
    products above, up to 4064, round to even), which by itself costs ~2e-4 of a row's norm.
    Q4_K: sc * q is exact; the minimum term rides along as 8 more columns of K per superblock (-(dmin / d) * m against
    half(sum x)), and 8 more give back what the products' rounding took from each slice in total, since quants of one
    sign would otherwise add those roundings up. The reference kernels round d * sc and dmin * m to fp16, this does
    not: about 2e-4 of the difference is theirs.
    Both stay within the 1e-3 bound; the split and integer settings take the int8 kernel's integer sums."""
    if t == Q4_K and scale > 100:
        scale = 30.0          # (the reference keeps Q4_K's sum of 32 activations as a half: it overflows beyond that)
    raw = synth.make_weight(t, rows, k, 40 + rows)
    w = torch.from_numpy(raw).to(DEV)
    xa = synth.make_activation(m, k, 41 + m).astype(np.float64) * scale
    xa[min(3, m - 1), :64] = 0.0
    if m > 100:
        xa[100, :] = 0.0
    xa[min(5, m - 1), 7] = 40.0 * scale
    x = synth.nudge_ties_torch(torch.from_numpy(xa.astype(np.float32)).to(torch.bfloat16)).float()
    if t == Q4_K:
        ref = _reference_q4k(raw, x)
    else:
        q, d, _ = q8_1.quantize_mmq(x.numpy(), q8_1.LAYOUT_D4)
        ref = product.product_q81(blocks.decode(raw, t), q, d)

    def run(form):
        old = _cabi.lib.gsq_debug_gemm_variant(form)
        old_mode = _cabi.lib.gsq_debug_mmv_mode(1)
        try:
            y = torch.ops._C_gguf.lcpp_mul_mat_q(w, x.to(DEV), t, rows)
            torch.cuda.synchronize()
        finally:
            _cabi.lib.gsq_debug_gemm_variant(old)
            _cabi.lib.gsq_debug_mmv_mode(old_mode)
        return y

    errs = {}
    for name, form, tol in (("rounded", 6, 1e-3), ("int8", 4, 2e-6)) + ((("split operands", 5, 1e-3),) if t == IQ4_XS else ()):
        got = run(form).cpu().numpy()
        assert np.isfinite(got).all(), name
        errs[name] = product.rel_err(got, ref)
        assert errs[name] <= tol, (name, errs)
        if m > 100:
            assert not got[100].any(), name
    print(f"type {t} {rows}x{k} m={m} scale {scale}:", {n: f"{e:.2e}" for n, e in errs.items()})
    if m >= 256:
        # the library's own choice: rounded by default; the split and integer settings = the int8 kernel
        assert torch.equal(run(0), run(6))
        for mode in (lcpp_ops.PREFILL_SPLIT, lcpp_ops.PREFILL_INTEGER):
            lcpp_ops.set_prefill_precision(mode)
            try:
                y = run(3)
            finally:
                lcpp_ops.set_prefill_precision(lcpp_ops.PREFILL_ROUNDED)
            assert torch.equal(y, run(4))


def test_q4_k_blocks_whose_minimum_dwarfs_their_scale():
    """Q4_K superblocks with d = 0, or dmin more than 64 times d: the kernel scales such a block by dmin / 64 instead of
    d (so that -(dmin / scale) * m stays inside fp16) and the weights then carry one more rounding."""
    rows, k, m = 128, 1024, 300
    raw = synth.make_weight(Q4_K, rows, k, 99).copy()
    blk = raw.reshape(rows, k // 256, 144)
    d16 = blk[:, :, 0:2].copy().view(np.float16)
    d16[::3, 0, 0] = 0.0                                   # d = 0 in the first superblock of every third row
    d16[1::3, 1, 0] = d16[1::3, 1, 0] / np.float16(512.0)  # d tiny against dmin in the second superblock of others
    blk[:, :, 0:2] = d16.view(np.uint8)
    w = torch.from_numpy(raw).to(DEV)
    x = synth.nudge_ties_torch(torch.from_numpy(synth.make_activation(m, k, 98)).to(torch.bfloat16)).float()
    ref = _reference_q4k(raw, x)
    old = _cabi.lib.gsq_debug_gemm_variant(6)
    try:
        y = torch.ops._C_gguf.lcpp_mul_mat_q(w, x.to(DEV), Q4_K, rows).cpu().numpy()
    finally:
        _cabi.lib.gsq_debug_gemm_variant(old)
    assert np.isfinite(y).all()
    assert product.rel_err(y, ref) <= 1e-3


@pytest.mark.parametrize("t,form,split", [(IQ3_S, 6, False), (IQ3_S, 5, True), (IQ4_XS, 6, False), (IQ4_XS, 5, True), (Q4_K, 6, False)])
@pytest.mark.parametrize("rows,k,m,scale", [(144, 1024, 300, 1.0), (128, 5120, 70, 1e-3), (272, 512, 513, 30.0)])
def test_kernels_follow_the_model_of_their_own_arithmetic(t, form, split, rows, k, m, scale):
    """The 1e-3 bound above is the distance to the reference's arithmetic. Against the CPU model of what these forms
    compute themselves (oracle/prefill_forms.py: the same roundings to fp16, sums in float64) the kernels agree at
    fp32 accuracy, which pins the operand layouts, the per-token scaling and Q4_K's extra columns exactly."""
    from oracle import prefill_forms

    raw = synth.make_weight(t, rows, k, 500 + rows)
    w = torch.from_numpy(raw).to(DEV)
    if t == IQ3_S:
        iq3_pack.pack_(w, IQ3_S)
    xa = synth.make_activation(m, k, 501 + m).astype(np.float64) * scale
    xa[3, :64] = 0.0
    xa[min(40, m - 1), :] = 0.0
    xa[5, 7] = 40.0 * scale
    x = synth.nudge_ties_torch(torch.from_numpy(xa.astype(np.float32)).to(torch.bfloat16)).float()
    want = prefill_forms.product(raw, t, x.numpy(), split=split)
    old = _cabi.lib.gsq_debug_gemm_variant(form)
    old_mode = _cabi.lib.gsq_debug_mmv_mode(1)
    try:
        op = torch.ops._C_gguf.lcpp_mul_mat_iq3_packed if t == IQ3_S else torch.ops._C_gguf.lcpp_mul_mat_q
        y = op(w, x.to(DEV), t, rows).cpu().numpy()
    finally:
        _cabi.lib.gsq_debug_gemm_variant(old)
        _cabi.lib.gsq_debug_mmv_mode(old_mode)
    err = product.rel_err(y, want)
    print(f"type {t} form {form} {rows}x{k} m={m} scale {scale}: {err:.2e}")
    assert err <= 3e-6, err
