"""The oracle for the six low-bit types (Q2_K, IQ2_XXS, IQ2_XS, IQ2_S, IQ3_XXS, IQ1_M) against its pins: gguf-py
outputs on seeded blocks (committed), the record of the run against the reference's 48 real-row fixtures, and those
fixtures themselves when the reference tree is at hand (tests/fixtures/dequant/*.npz,
tests/cpu/test_dequant_fixtures.py:54-58)."""

import glob
import json
import os

import numpy as np
import pytest

from oracle import blocks_f1

NAMES = list(blocks_f1.TYPE_IDS)


@pytest.mark.parametrize("name", NAMES)
def test_dequant_matches_committed_gguf_py(golden_dir, name):
    z = np.load(os.path.join(golden_dir, "dequant_blocks_f1.npz"))
    mine = blocks_f1.dequantize(z[f"{name}_raw"], blocks_f1.TYPE_IDS[name])
    assert np.array_equal(mine.view(np.uint32), z[f"{name}_ref"].view(np.uint32))


def test_fixture_record_all_bit_exact(golden_dir):
    rec = json.load(open(os.path.join(golden_dir, "fixture_check_f1.json")))["fixtures"]
    assert len(rec) == 48
    assert all(r["oracle_bit_exact"] for r in rec)
    assert sorted({r["type"] for r in rec}) == [10, 16, 17, 18, 22, 29]


def test_reference_fixtures_when_present(reference_dir):
    if reference_dir is None:
        pytest.skip("reference tree not present")
    n = 0
    for f in sorted(glob.glob(os.path.join(reference_dir, "tests/fixtures/dequant/*.npz"))):
        z = np.load(f)
        t = int(z["ggml_type"])
        if t not in blocks_f1.BLOCK_BYTES:
            continue
        mine = blocks_f1.dequantize(z["raw"], t)[0]
        assert np.array_equal(mine.view(np.uint32), z["ref"].view(np.uint32)), f
        n += 1
    assert n == 48


@pytest.mark.parametrize("name", NAMES)
def test_product_model_close_to_full_product(name):
    """The integer model (truncating divisions of the reference's kernels included) stays within the quantisation
    error of dequantise-and-multiply; its group sums rebuild the dequantised weights where the format is linear."""
    from gsq_b200 import synth
    from oracle import product, q8_1

    t = blocks_f1.TYPE_IDS[name]
    raw = synth.make_weight(t, 24, 1024, 5)
    x = synth.make_activation(3, 1024, 6)
    q, d, _ = q8_1.quantize_q8_1(x)
    dec = blocks_f1.decode(raw, t)
    y = blocks_f1.product_q81(dec, q, d.astype(np.float32))
    full = blocks_f1.product_full(raw, t, x)
    assert product.rel_err(y, full) <= 3e-2
    s = blocks_f1.group_sums(dec, q)
    assert s.shape == (3, 24, 1024 // dec.g) and s.dtype == np.int32
