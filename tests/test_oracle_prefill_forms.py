"""The CPU model of the fp16-operand prefill forms (oracle/prefill_forms.py) against the model of the reference
kernels' arithmetic (oracle/product.py): the forms stay inside the 1e-3 bound of this path, the split form at fp32
accuracy, on the inputs the GPU tests use (zero blocks, a zero token, an outlier channel, small and large scales)."""

import numpy as np
import pytest

from gsq_b200 import synth
from oracle import blocks, prefill_forms, product, q8_1

IQ3_S, IQ4_XS, Q4_K = 21, 23, 12


def _x(m, k, scale, seed):
    xa = synth.make_activation(m, k, seed).astype(np.float64) * scale
    xa[3, :64] = 0.0
    xa[min(20, m - 1), :] = 0.0
    xa[5, 7] = 40.0 * scale
    return q8_1.nudge_ties(xa.astype(np.float32).astype(np.float16).astype(np.float32)) if scale < 100 else xa.astype(np.float32)


def _reference(raw, t, x):
    dec = blocks.decode(raw, t)
    if t == Q4_K:
        q, d, s = q8_1.quantize_mmq(x, q8_1.LAYOUT_DS4)
        dh, sh = d.astype(np.float16).astype(np.float64), s.astype(np.float16).astype(np.float64)
        gs = (np.repeat(dec.d, 8, axis=1).astype(np.float16) * dec.isc.astype(np.float16)).astype(np.float64)
        mins = (np.repeat(dec.dmin, 8, axis=1).astype(np.float16) * dec.imin.astype(np.float16)).astype(np.float64)
        return np.einsum("mns,ns,ms->mn", product.block_sums(dec, q).astype(np.float64), gs, dh, optimize=True) - sh @ mins.T
    q, d, _ = q8_1.quantize_mmq(x, q8_1.LAYOUT_D4)
    return product.product_q81(dec, q, d)


@pytest.mark.parametrize("t,rows,k,m,scale", [(IQ3_S, 64, 1024, 40, 1.0), (IQ3_S, 48, 512, 33, 1e-3), (IQ3_S, 32, 512, 24, 3e4),
                                              (IQ4_XS, 64, 1024, 40, 1.0), (IQ4_XS, 40, 512, 24, 3e4),
                                              (Q4_K, 64, 1024, 40, 1.0), (Q4_K, 40, 512, 24, 30.0)])
def test_rounded_form_stays_inside_the_bound(t, rows, k, m, scale):
    raw = synth.make_weight(t, rows, k, 7 + rows)
    x = _x(m, k, scale, 8 + m)
    ref = _reference(raw, t, x)
    y = prefill_forms.product(raw, t, x)
    assert np.isfinite(y).all()
    err = product.rel_err(y, ref)
    assert err <= 1e-3, err
    assert not y[min(20, m - 1)].any()                    # a token of zeros
    if t != Q4_K:
        ys = prefill_forms.product(raw, t, x, split=True)
        errs = product.rel_err(ys, ref)
        assert errs <= (2e-6 if t == IQ3_S else 1e-3), errs


def test_operands_fit_fp16():
    """No scaled product reaches fp16's range whatever the activations' scale, and the pair hi + lo restores 22 bits."""
    for scale in (1e-30, 1e-3, 1.0, 3e4, 1e30):
        x = (synth.make_activation(9, 512, 3).astype(np.float64) * scale).astype(np.float32)
        hi, lo, inv_up, _, _ = prefill_forms.scaled_products(x, False)
        assert np.isfinite(hi.astype(np.float32)).all() and np.abs(hi.astype(np.float32)).max() <= 2.0 ** 14 * 1.001
        q, d, _ = q8_1.quantize_mmq(x, q8_1.LAYOUT_D4)
        exact = np.repeat(d.astype(np.float64), 32, axis=1) * q
        got = (hi.astype(np.float64) + lo.astype(np.float64)) * inv_up.astype(np.float64)[:, None]
        assert np.abs(got - exact).max() <= np.abs(exact).max() * 2.0 ** -20


def test_q4k_scale_rule():
    d = np.array([[1.0, 0.0, 1e-3, -2.0]], dtype=np.float32)
    dmin = np.array([[2.0, 0.5, 1.0, 1.0]], dtype=np.float32)
    s = prefill_forms.q4k_sigma(d, dmin)
    assert s[0, 0] == 1.0 and s[0, 1] == np.float32(0.5 / 64) and s[0, 2] == np.float32(1.0 / 64) and s[0, 3] == -2.0
    assert prefill_forms.q4k_sigma(np.zeros((1, 1), np.float32), np.zeros((1, 1), np.float32))[0, 0] == 1.0
