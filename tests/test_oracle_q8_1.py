"""The q8_1 oracle: layouts, summation order and the tie nudge (host only)."""

import numpy as np

from oracle import q8_1


def _x(m, k, seed, dtype=np.float16):
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((m, k)).astype(np.float32)
    x[:, rng.permutation(k)[: max(1, k // 256)]] *= 20
    return x.astype(dtype)


def test_q8_1_bytes_layout_and_values():
    x = _x(3, 512, 0, np.float32)
    buf = q8_1.q8_1_bytes(x)
    assert buf.dtype == np.uint8 and buf.size == 3 * 512 // 32 * 36
    q, d, s = q8_1.parse_q8_1_bytes(buf, 3, 512)
    amax = np.abs(x.reshape(3, 16, 32)).max(-1)
    assert np.array_equal(d, (amax / np.float32(127)).astype(np.float16))
    assert np.abs(q).max() == 127
    deq = q.reshape(3, 16, 32) * (amax / 127)[..., None]
    assert np.abs(deq - x.reshape(3, 16, 32)).max() <= (amax.max() / 127) * 0.5001


def test_zero_block_and_sum_order():
    x = np.zeros((1, 64), dtype=np.float32)
    x[0, 32:] = np.arange(32, dtype=np.float32) * 0.37 - 3
    q, d, s = q8_1.quantize_q8_1(x)
    assert np.all(q[0, :32] == 0) and d[0, 0] == 0 and s[0, 0] == 0
    v = x[0, 32:].copy()
    for h in (16, 8, 4, 2, 1):
        v = (v[:h] + v[h:2 * h]).astype(np.float32)
    assert s[0, 1] == np.float16(v[0])


def test_mmq_layouts():
    x = _x(5, 512, 1, np.float32)
    for layout in (q8_1.LAYOUT_D4, q8_1.LAYOUT_DS4):
        buf = q8_1.q8_1_mmq_bytes(x, layout)
        assert buf.size == 512 // 128 * 5 * 144
        b = buf.reshape(4, 5, 144)
        q, d, s = q8_1.quantize_mmq(x, layout)
        assert np.array_equal(b[2, 3, 16:].view(np.int8), q[3, 256:384])
        if layout == q8_1.LAYOUT_D4:
            assert np.array_equal(b[2, 3, :16].view(np.float32), d[3, 8:12])
        else:
            ds = b[2, 3, :16].view(np.float16).reshape(4, 2)
            assert np.array_equal(ds[:, 0], d[3, 8:12].astype(np.float16))
            assert np.array_equal(ds[:, 1], s[3, 8:12].astype(np.float16))
    # the two quantisers agree on the integers away from ties
    q0, _, _ = q8_1.quantize_q8_1(x)
    q1, _, _ = q8_1.quantize_mmq(x, q8_1.LAYOUT_D4)
    assert (q0 != q1).mean() < 1e-3


def test_nudge_removes_ties():
    x = _x(4, 1024, 2)
    x[0, 0] = np.float16(np.abs(x[0, :32].astype(np.float32)).max() / 2)   # a genuine tie candidate
    y = q8_1.nudge_ties(x)
    for qk in (32, 64):
        b = np.abs(y.astype(np.float32)).reshape(4, -1, qk)
        t = b * (np.float32(127) / b.max(-1, keepdims=True))
        assert not (np.abs(t - np.floor(t) - 0.5) < 1e-4).any()
    assert (x != y).mean() < 0.05
