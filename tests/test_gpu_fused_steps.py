"""RMSNorm (+ residual add) -> q8_1 and SwiGLU -> q8_1 in one launch each (gsq_b200.fused): the activations against the
host model of vLLM's kernels (oracle/fused_steps.py), the q8_1 bytes bit for bit against the separate quantiser applied to
the activations the same call returned, and the bytes feeding a product."""

import numpy as np
import pytest
import torch

import gsq_b200  # noqa: F401
from gsq_b200 import fused, synth, tp
from oracle import blocks, fused_steps, product, q8_1

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _ulp_report(got, want):
    """(fraction of elements that differ, largest difference in units of the larger neighbour's spacing)."""
    g, w = got.float(), want.float()
    diff = (g != w)
    if not diff.any():
        return 0.0, 0.0
    spacing = torch.maximum(w.abs(), g.abs()) * {torch.bfloat16: 2.0 ** -7, torch.float16: 2.0 ** -10, torch.float32: 2.0 ** -23}[got.dtype]
    return float(diff.float().mean()), float(((g - w).abs() / spacing.clamp_min(1e-30))[diff].max())


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("m,k", [(1, 5120), (8, 5120), (33, 1024), (4, 17408)])
@pytest.mark.parametrize("with_residual", [False, True])
def test_rmsnorm_quantize(dtype, m, k, with_residual):
    g = torch.Generator().manual_seed(m * 7 + k)
    x = torch.randn(m, k, generator=g).to(dtype)
    w = (1.0 + 0.1 * torch.randn(k, generator=g)).to(dtype)
    r = torch.randn(m, k, generator=g).to(dtype) if with_residual else None
    want_y, want_r = fused_steps.rmsnorm(x, w, 1e-6, r)
    rd = r.to(DEV).clone() if with_residual else None
    xq, y = fused.rmsnorm_quantize_q8_1(x.to(DEV), w.to(DEV), 1e-6, rd, want_y=True)
    if with_residual:
        assert torch.equal(rd.cpu(), want_r)                       # x + residual, rounded once: exact
    frac, ulps = _ulp_report(y.cpu(), want_y)
    if dtype == torch.float32:      # nothing is rounded away: the fp32 sum order and rsqrt show in the last places
        assert ulps <= 4.0, (frac, ulps)
    else:
        assert frac <= 2e-3 and ulps <= 2.01, (frac, ulps)        # one place of X's type (the measure reads up to 2 at a binade edge), rarely
    # the q8_1 bytes are those of the separate quantiser on the very activations this call returned
    assert torch.equal(xq, torch.ops._C_gguf.lcpp_quantize_q8_1(y, 21, False, False))
    # and without y_out the same bytes
    rd2 = r.to(DEV).clone() if with_residual else None
    xq2, none = fused.rmsnorm_quantize_q8_1(x.to(DEV), w.to(DEV), 1e-6, rd2)
    assert none is None and torch.equal(xq, xq2)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("m,inter", [(1, 17408), (8, 2304), (40, 512)])
def test_silu_mul_quantize(dtype, m, inter):
    g = torch.Generator().manual_seed(m + inter)
    gu = (2.0 * torch.randn(m, 2 * inter, generator=g)).to(dtype)
    want = fused_steps.silu_mul(gu)
    xq, y = fused.silu_mul_quantize_q8_1(gu.to(DEV), want_y=True)
    frac, ulps = _ulp_report(y.cpu(), want)
    if dtype == torch.float32:
        assert ulps <= 4.0, (frac, ulps)
    else:
        assert frac <= 2e-3 and ulps <= 2.01, (frac, ulps)        # expf of the device against the host's in the last place
    with tp.relaxed_k():
        assert torch.equal(xq, torch.ops._C_gguf.lcpp_quantize_q8_1(y, 21, False, False))
    xq2, _ = fused.silu_mul_quantize_q8_1(gu.to(DEV))
    assert torch.equal(xq, xq2)


def test_fused_bytes_feed_a_product():
    """norm -> q8_1 -> product against the oracle's product on the oracle-side quantisation of the same activations."""
    m, k, rows = 4, 5120, 256
    g = torch.Generator().manual_seed(5)
    x = torch.randn(m, k, generator=g).to(torch.float16)
    w = torch.ones(k, dtype=torch.float16)
    xq, y = fused.rmsnorm_quantize_q8_1(x.to(DEV), w.to(DEV), 1e-6, None, want_y=True)
    raw = synth.make_weight(12, rows, k, 3)
    out = torch.ops._C_gguf.lcpp_mul_mat_vec_q(torch.from_numpy(raw).to(DEV), y, 12, rows, xq)
    q, d, _ = q8_1.quantize_q8_1(y.float().cpu().numpy())
    ref = product.product_q81(blocks.decode(raw, 12), q, d.astype(np.float32))
    assert product.rel_err(out.float().cpu().numpy(), ref) <= 2e-3
