"""Boundary behaviour of the op layer on the GPU, restating what the reference checks about its own ops:

  * the very first op call of a fresh process may sit inside a CUDA-graph capture
    (tests/gpu/test_kernel_parity.py:655-698 of the reference: its occupancy caches used to be filled there);
  * nothing may depend on the contents of freshly allocated memory: the caching allocator is poisoned with
    0xFF before each op (tests/gpu/test_kernel_parity.py:280-286);
  * every op name of the routing table computes on the GPU, lcpp_mul_mat_vec_iq3_mma (GGUF-order IQ3_S at
    6..8 rows) included;
  * a shape the small-batch kernel declines is still served under the vec op names (up to their stated row
    limit) by the dp4a kernel, eight rows per launch.
"""

import os
import subprocess
import sys
import textwrap

import numpy as np
import pytest
import torch

import gsq_b200  # noqa: F401
from gsq_b200 import _cabi, synth
from gsq_b200.quantization import iq3_pack
from oracle import blocks, product, q8_1

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DEV = "cuda:0"
Q4_K, Q6_K, IQ3_S, IQ4_XS = 12, 14, 21, 23


def _x(m, k, dtype, seed):
    return synth.nudge_ties_torch(torch.from_numpy(synth.make_activation(m, k, seed)).to(dtype))


def _ref(raw, t, x):
    q, d, _ = q8_1.quantize_q8_1(x.float().numpy())
    return product.product_q81(blocks.decode(raw, t), q, d.astype(np.float32))


@pytest.mark.parametrize("m", [6, 8])
def test_vec_iq3_mma_op_on_gguf_order_weights(m):
    rows, k = 208, 5120
    raw = synth.make_weight(IQ3_S, rows, k, 70)
    x = _x(m, k, torch.float32, 71)
    y = torch.ops._C_gguf.lcpp_mul_mat_vec_iq3_mma(torch.from_numpy(raw).to(DEV), x.to(DEV), IQ3_S, rows)
    assert product.rel_err(y.cpu().numpy(), _ref(raw, IQ3_S, x)) <= 1e-5


_CAPTURE_FIRST = textwrap.dedent("""
    import sys
    sys.path[:0] = [{root!r}, {pkg!r}]
    import torch
    import gsq_b200
    from gsq_b200 import synth
    from gsq_b200.quantization import iq3_pack
    dev = "cuda:0"
    name, t, op, m, packed = {name!r}, {t}, {op!r}, {m}, {packed}
    rows, k = 256, 1024
    w = torch.from_numpy(synth.make_weight(t, rows, k, 5)).to(dev)
    if packed:
        iq3_pack.pack_(w, t)
    x = torch.from_numpy(synth.make_activation(m, k, 6)).to(torch.float16).to(dev)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):              # the first call of this op in the process is inside the capture
        y = getattr(torch.ops._C_gguf, op)(w, x, t, rows)
    g.replay()
    torch.cuda.synchronize()
    eager = getattr(torch.ops._C_gguf, op)(w, x, t, rows)
    torch.cuda.synchronize()
    assert torch.equal(y, eager), "graph replay differs from the eager call"
    assert torch.isfinite(y.float()).all() and float(y.float().abs().max()) > 0
    print("ok")
""")


@pytest.mark.parametrize("name,t,op,m,packed", [
    ("IQ3_S", IQ3_S, "lcpp_mul_mat_vec_iq3_mma_packed", 4, True),
    ("Q4_K", Q4_K, "lcpp_mul_mat_vec_q", 1, False),
    ("IQ4_XS", IQ4_XS, "lcpp_mul_mat_mma_k", 16, False),
    ("IQ4_XS", IQ4_XS, "lcpp_mul_mat_q", 200, False),
    ("IQ3_S", IQ3_S, "lcpp_mul_mat_iq3_packed", 130, True),
    ("IQ3_S", IQ3_S, "lcpp_mul_mat_iq3_packed", 512, True),
    ("IQ4_XS", IQ4_XS, "lcpp_mul_mat_q", 600, False),
    ("Q4_K", Q4_K, "lcpp_mul_mat_q", 600, False),
    ("Q6_K", Q6_K, "lcpp_mul_mat_vec_q", 3, False),
    ("Q6_K", Q6_K, "gsq_mul_mat_q6k_packed", 20, True),
])
def test_first_call_of_a_process_inside_a_capture(name, t, op, m, packed):
    code = _CAPTURE_FIRST.format(root=ROOT, pkg=os.path.join(ROOT, "vllm-gsqrco-exl3_b200"), name=name, t=t, op=op, m=m,
                                 packed=packed)
    p = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=300)
    assert p.returncode == 0 and "ok" in p.stdout, p.stderr[-2000:]


def _poison():
    """Fill what the caching allocator will hand out next with 0xFF (NaN as a float, -1 as an int)."""
    bufs = [torch.full((n,), 0xFF, dtype=torch.uint8, device=DEV) for n in (1 << 26, 1 << 22, 1 << 18, 1 << 14)]
    torch.cuda.synchronize()
    del bufs


@pytest.mark.parametrize("name,t,op,m,packed", [
    ("IQ3_S", IQ3_S, "lcpp_mul_mat_vec_iq3_mma_packed", 8, True),
    ("IQ3_S", IQ3_S, "lcpp_mul_mat_iq3_packed", 24, True),
    ("IQ3_S", IQ3_S, "lcpp_mul_mat_iq3_packed", 200, True),
    ("Q4_K", Q4_K, "lcpp_mul_mat_vec_own", 5, False),
    ("Q4_K", Q4_K, "lcpp_mul_mat_mma_k", 33, False),
    ("IQ4_XS", IQ4_XS, "lcpp_mul_mat_q", 70, False),
    ("Q6_K", Q6_K, "lcpp_mul_mat_q", 20, False),
])
def test_ops_do_not_read_uninitialised_memory(name, t, op, m, packed):
    rows, k = 272, 5120
    raw = synth.make_weight(t, rows, k, 80 + t)
    w = torch.from_numpy(raw).to(DEV)
    if packed:
        iq3_pack.pack_(w, t)
    x = _x(m, k, torch.float32, 81 + m).to(DEV)
    fn = getattr(torch.ops._C_gguf, op)
    clean = fn(w, x, t, rows).clone()
    _poison()
    dirty = fn(w, x, t, rows)
    assert torch.isfinite(dirty).all()
    assert torch.equal(clean, dirty)


def test_vec_op_serves_a_shape_the_small_batch_kernel_declines():
    """With one CTA per cluster the activations of 32 rows x 5120 columns do not fit beside the codebook, so the
    small-batch kernel declines; the packed vec op (up to 32 rows) must still answer."""
    rows, k, m = 208, 5120, 32
    raw = synth.make_weight(IQ3_S, rows, k, 90)
    w = torch.from_numpy(raw).to(DEV)
    iq3_pack.pack_(w, IQ3_S)
    x = _x(m, k, torch.float32, 91)
    old = _cabi.lib.gsq_debug_mmv_cluster_size(1)
    try:
        y = torch.ops._C_gguf.lcpp_mul_mat_vec_iq3_mma_packed(w, x.to(DEV), IQ3_S, rows)
    finally:
        _cabi.lib.gsq_debug_mmv_cluster_size(old)
    assert product.rel_err(y.cpu().numpy(), _ref(raw, IQ3_S, x)) <= 1e-5
