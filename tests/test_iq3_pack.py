"""IQ3_S repack: the properties the reference pins for its own repack (tests/cpu/test_iq3_pack.py:26-77)
plus byte equality with the loop-form definition in oracle/iq3_layout.py."""

import glob
import os

import numpy as np
import pytest
import torch

from gsq_b200 import synth
from gsq_b200.quantization import iq3_pack
from oracle import iq3_layout

IQ3_S = 21


def test_matches_definition_and_round_trips():
    w = synth.make_weight(IQ3_S, 32, 1024, 5)
    p = iq3_pack.pack(torch.from_numpy(w), IQ3_S)
    assert np.array_equal(p.numpy(), iq3_layout.pack_ref(w))
    assert torch.equal(iq3_pack.unpack(p, IQ3_S), torch.from_numpy(w))
    assert not torch.equal(p, torch.from_numpy(w))


def test_round_trip_random_bytes():
    g = torch.Generator().manual_seed(1)
    w = torch.randint(0, 256, (64, 110 * 7), dtype=torch.uint8, generator=g)
    assert torch.equal(iq3_pack.unpack(iq3_pack.pack(w, IQ3_S), IQ3_S), w)


def test_round_trip_reference_rows(reference_dir):
    if reference_dir is None:
        pytest.skip("reference tree not present")
    rows = [np.load(f)["raw"] for f in sorted(glob.glob(os.path.join(reference_dir, "tests/fixtures/dequant/IQ3_S__*.npz")))]
    assert len(rows) == 9
    w = torch.from_numpy(np.stack((rows * 2)[:16]))
    assert torch.equal(iq3_pack.unpack(iq3_pack.pack(w, IQ3_S), IQ3_S), w)


def test_tile_locality():
    """Tile t of the packed bytes depends only on rows 16t..16t+15, and stays where they were."""
    w = torch.from_numpy(synth.make_weight(IQ3_S, 48, 512, 6))
    p = iq3_pack.pack(w, IQ3_S)
    w2 = w.clone()
    w2[16:32] = torch.from_numpy(synth.make_weight(IQ3_S, 16, 512, 7))
    p2 = iq3_pack.pack(w2, IQ3_S)
    assert torch.equal(p[:16], p2[:16]) and torch.equal(p[32:], p2[32:]) and not torch.equal(p[16:32], p2[16:32])
    assert torch.equal(iq3_pack.pack(w[16:32].clone(), IQ3_S), p[16:32])


def test_pack_in_place_on_view_inside_padded_buffer():
    rb = 110 * 4
    buf = torch.full((40, rb + 64), 0xAB, dtype=torch.uint8)
    w = torch.from_numpy(synth.make_weight(IQ3_S, 32, 1024, 8))
    flat = buf.view(-1)
    view = flat[: 32 * rb].view(32, rb)      # a run stored contiguously from the start of the buffer
    view.copy_(w)
    iq3_pack.pack_(view, IQ3_S)
    assert torch.equal(view, iq3_pack.pack(w, IQ3_S))
    assert (flat[32 * rb:] == 0xAB).all()


def test_rejects_bad_input():
    w = torch.zeros(24, 220, dtype=torch.uint8)
    with pytest.raises(AssertionError):
        iq3_pack.pack(w, IQ3_S)
    with pytest.raises(AssertionError):
        iq3_pack.pack(torch.zeros(16, 144, dtype=torch.uint8), 12)


# ---------------------------------------------------------------------------------------------
# Q6_K: the same functions, a byte permutation per 16-row tile (no counterpart in the reference; the properties
# are the ones it pins for IQ3_S)

Q6_K = 14


def test_q6k_matches_definition_and_round_trips():
    w = synth.make_weight(Q6_K, 32, 1024, 6)
    p = iq3_pack.pack(torch.from_numpy(w), Q6_K)
    assert np.array_equal(p.numpy(), iq3_layout.pack_q6k_ref(w))
    assert torch.equal(iq3_pack.unpack(p, Q6_K), torch.from_numpy(w))
    assert not torch.equal(p, torch.from_numpy(w))
    assert sorted(iq3_pack.q6k_record_source().tolist()) == list(range(3360))


def test_q6k_tile_locality_and_in_place_view():
    g = torch.Generator().manual_seed(2)
    w = torch.randint(0, 256, (48, 210 * 3), dtype=torch.uint8, generator=g)
    p = iq3_pack.pack(w, Q6_K)
    w2 = w.clone()
    w2[16:32] = torch.randint(0, 256, (16, 630), dtype=torch.uint8, generator=g)
    p2 = iq3_pack.pack(w2, Q6_K)
    assert torch.equal(p[:16], p2[:16]) and torch.equal(p[32:], p2[32:]) and not torch.equal(p[16:32], p2[16:32])
    wide = torch.zeros(64, 210 * 3, dtype=torch.uint8)
    wide[8:40].view(-1)[: 32 * 630].view(32, 630).copy_(w[:32])          # a run inside a wider buffer
    view = wide[8:40].view(-1)[: 32 * 630].view(32, 630)
    iq3_pack.pack_(view, Q6_K)
    assert torch.equal(view, p[:32]) and not wide[:8].any() and not wide[40:].any()
    with pytest.raises(AssertionError):
        iq3_pack.pack(w[:24], Q6_K)
