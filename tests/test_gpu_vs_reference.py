"""GPU-vs-GPU parity with the reference's own CUDA kernels, rebuilt for sm_100a from the reference tree
(oracle/build_ref.py -> oracle/_ref/ref_C_gguf.so; skipped when that library was not built). The reference
library runs in a process of its own (oracle/ref_runner.py) because it defines the same torch op names.

  q8_1 bytes (both layouts)  bit exact, on inputs that INCLUDE rounding ties (no nudge): the quantisers
                             here use the same approximate-division instructions as the reference's
                             --use_fast_math build
  fp32 outputs               <= 1e-3 row-norm relative (the stated tolerance); measured ~1e-7 for the GEMV
                             and the GEMM, whose only difference from the reference is the fp32 summation order
"""

import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import gsq_b200  # noqa: F401
from gsq_b200 import synth
from gsq_b200.quantization import iq3_pack
from oracle import product

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF_SO = os.path.join(ROOT, "oracle", "_ref", "ref_C_gguf.so")
DEV = "cuda:0"
Q4_K, Q6_K, IQ3_S, IQ4_XS = 12, 14, 21, 23


def _x(m, k, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(m, k, generator=g)
    x[:, torch.randperm(k, generator=g)[: max(1, k // 256)]] *= 20
    return x.to(dtype)          # deliberately NOT tie-nudged


def run_reference(cases, tmp_path):
    if not os.path.exists(REF_SO):
        pytest.skip("oracle/_ref/ref_C_gguf.so not built")
    cin, cout = str(tmp_path / "cases.pt"), str(tmp_path / "results.pt")
    torch.save(cases, cin)
    p = subprocess.run([sys.executable, os.path.join(ROOT, "oracle", "ref_runner.py"), cin, cout], capture_output=True,
                       text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-3000:]
    return torch.load(cout)


def test_quantizers_bit_exact_including_ties(tmp_path):
    xs = [(_x(8, 5120, torch.float16, 1), IQ3_S), (_x(3, 17408, torch.bfloat16, 2), Q4_K), (_x(5, 1024, torch.float32, 3), IQ4_XS)]
    xs[0][0][0, :32] = 0                                     # an all-zero block
    xs[0][0][1, 32:64] = xs[0][0][1, 32:64].abs().max() / 2  # exact ties x = amax / 2
    cases = []
    for x, t in xs:
        for mmq in (False, True):
            cases.append({"op": "lcpp_quantize_q8_1", "args": [x, t, mmq, False]})
    res = run_reference(cases, tmp_path)
    i = 0
    for x, t in xs:
        for mmq in (False, True):
            mine = torch.ops._C_gguf.lcpp_quantize_q8_1(x.to(DEV), t, mmq, False).cpu()
            ref = res[i]["out"]
            i += 1
            assert mine.shape == ref.shape
            nbad = int((mine != ref).sum())
            assert nbad == 0, (str(x.dtype), t, mmq, nbad, mine.numel())


GEMV_CASES = [("Q4_K", Q4_K, "lcpp_mul_mat_vec_q"), ("IQ4_XS", IQ4_XS, "lcpp_mul_mat_vec_q"), ("Q6_K", Q6_K, "lcpp_mul_mat_vec_q"),
              ("IQ3_S", IQ3_S, "lcpp_mul_mat_vec_iq3"), ("Q4_K", Q4_K, "lcpp_mul_mat_vec_own")]


def test_gemv_outputs_match_reference_kernels(tmp_path):
    rows, k = 272, 5120
    cases, mine = [], []
    for name, t, op in GEMV_CASES:
        raw = torch.from_numpy(synth.make_weight(t, rows, k, 40 + t))
        for m in (1, 4, 8):
            x = _x(m, k, torch.float32, 50 + m)
            cases.append({"op": op, "args": [raw, x, t, rows]})
            w = raw.to(DEV)
            my_op = op
            if t == IQ3_S:
                iq3_pack.pack_(w, t)
                my_op = "lcpp_mul_mat_vec_iq3_mma_packed"
            mine.append(getattr(torch.ops._C_gguf, my_op)(w, x.to(DEV), t, rows).cpu())
    res = run_reference(cases, tmp_path)
    for c, y, r in zip(cases, mine, res):
        err = product.rel_err(y.numpy(), r["out"].double().numpy())
        assert err <= 1e-3, (c["op"], c["args"][2], err)
        assert err <= 1e-5, (c["op"], c["args"][2], err)     # in practice: fp32 summation order only


def test_gemm_outputs_match_reference_kernels(tmp_path):
    rows, k = 272, 5120
    cases, mine = [], []
    for name, t, op in (("Q4_K", Q4_K, "lcpp_mul_mat_q"), ("IQ4_XS", IQ4_XS, "lcpp_mul_mat_q"), ("IQ3_S", IQ3_S, "lcpp_mul_mat_q"),
                        ("Q4_K", Q4_K, "lcpp_mul_mat_mma_k"), ("IQ4_XS", IQ4_XS, "lcpp_mul_mat_mma_k")):
        raw = torch.from_numpy(synth.make_weight(t, rows, k, 60 + t))
        for m in (9, 33, 64) if op == "lcpp_mul_mat_mma_k" else (16, 130):
            x = _x(m, k, torch.float32, 70 + m)
            cases.append({"op": op, "args": [raw, x, t, rows]})
            w = raw.to(DEV)
            my_op = op
            if t == IQ3_S:
                iq3_pack.pack_(w, t)
                my_op = "lcpp_mul_mat_iq3_packed"
            mine.append(getattr(torch.ops._C_gguf, my_op)(w, x.to(DEV), t, rows).cpu())
    res = run_reference(cases, tmp_path)
    for c, y, r in zip(cases, mine, res):
        err = product.rel_err(y.numpy(), r["out"].double().numpy())
        assert err <= 1e-3, (c["op"], c["args"][2], c["args"][1].shape[0], err)


def test_packed_iq3_kernels_match_reference_packed_kernels(tmp_path):
    """The reference's packed IQ3_S kernels read the reference's own repack (tests/golden/iq3_ref_packed.npz,
    made by its iq3_pack.pack); the kernels here read this package's repack of the same raw blocks."""
    z = np.load(os.path.join(ROOT, "tests", "golden", "iq3_ref_packed.npz"))
    raw, ref_packed = torch.from_numpy(z["raw"]), torch.from_numpy(z["ref_packed"])
    rows, k = raw.shape[0], raw.shape[1] // 110 * 256
    w = raw.to(DEV)
    iq3_pack.pack_(w, IQ3_S)
    cases, mine = [], []
    for op, ms in (("lcpp_mul_mat_vec_iq3_mma_packed", (1, 5, 8, 32)), ("lcpp_mul_mat_iq3_packed", (16, 48, 130))):
        for m in ms:
            x = _x(m, k, torch.float32, 90 + m)
            cases.append({"op": op, "args": [ref_packed, x, IQ3_S, rows]})
            mine.append(getattr(torch.ops._C_gguf, op)(w, x.to(DEV), IQ3_S, rows).cpu())
    res = run_reference(cases, tmp_path)
    for c, y, r in zip(cases, mine, res):
        err = product.rel_err(y.numpy(), r["out"].double().numpy())
        assert err <= 1e-3, (c["op"], c["args"][1].shape[0], err)
