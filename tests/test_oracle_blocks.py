"""The block-decoding oracle against its pins: gguf-py outputs on seeded blocks (committed), the
record of the run against the reference's 36 real-row fixtures, and those fixtures themselves when
the reference tree is at hand (tests/fixtures/dequant/*.npz, tests/cpu/test_dequant_fixtures.py:54-58)."""

import glob
import json
import os

import numpy as np
import pytest

from oracle import blocks

NAMES = ["IQ3_S", "IQ4_XS", "Q4_K", "Q6_K"]


@pytest.mark.parametrize("name", NAMES)
def test_dequant_matches_committed_gguf_py(golden_dir, name):
    z = np.load(os.path.join(golden_dir, "dequant_blocks.npz"))
    mine = blocks.dequantize(z[f"{name}_raw"], blocks.TYPE_IDS[name])
    assert np.array_equal(mine.view(np.uint32), z[f"{name}_ref"].view(np.uint32))


def test_fixture_record_all_bit_exact(golden_dir):
    rec = json.load(open(os.path.join(golden_dir, "fixture_check.json")))["fixtures"]
    assert len(rec) == 36
    assert all(r["oracle_bit_exact"] for r in rec)
    assert sorted({r["type"] for r in rec}) == [12, 14, 21, 23]


def test_reference_fixtures_when_present(reference_dir):
    if reference_dir is None:
        pytest.skip("reference tree not present")
    n = 0
    for f in sorted(glob.glob(os.path.join(reference_dir, "tests/fixtures/dequant/*.npz"))):
        z = np.load(f)
        t = int(z["ggml_type"])
        if t not in blocks.BLOCK_BYTES:
            continue
        mine = blocks.dequantize(z["raw"], t)[0]
        assert np.array_equal(mine.view(np.uint32), z["ref"].view(np.uint32)), f
        n += 1
    assert n == 36


@pytest.mark.parametrize("name", NAMES)
def test_integer_decode_consistent_with_float(name):
    """w8, isc, d (and imin, dmin) rebuild the float dequantisation exactly in float64."""
    from gsq_b200 import synth

    t = blocks.TYPE_IDS[name]
    raw = synth.make_weight(t, 6, 768, 11)
    dec = blocks.decode(raw, t)
    gs = blocks.group_scales(dec)
    w = np.repeat(gs, dec.g, axis=1) * dec.w8.astype(np.float64)
    if dec.imin is not None:
        w -= np.repeat(np.repeat(dec.dmin.astype(np.float64), 8, axis=1) * dec.imin, 32, axis=1)
    ref = blocks.dequantize(raw, t).astype(np.float64)
    assert np.allclose(w, ref, rtol=1e-6, atol=1e-7)
    if name == "IQ3_S":
        assert np.all(np.abs(dec.w8) % 2 == 1) and np.abs(dec.w8).max() <= 15
        assert dec.isc.min() >= 1 and dec.isc.max() <= 31
    if name == "Q6_K":
        assert dec.w8.min() >= -32 and dec.w8.max() <= 31 and dec.g == 16
