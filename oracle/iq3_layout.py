"""CPU oracle (TEST INFRASTRUCTURE, not product code): the IQ3_S streaming layout, restated with
plain loops straight from its definition (csrc/gsq_repack.cu header comment).

The reference pins only the properties of its repack, not a byte layout
(tests/cpu/test_iq3_pack.py:26-77: round trip on real rows and random bytes, tile locality, in-place
packing of a view inside a wider buffer, rejection of rows % 16 != 0); the same properties are
checked for this layout, and `pack_ref` is an independent second formulation the product's two
implementations (torch ops on CPU, CUDA kernel on GPU) must agree with byte for byte.
"""

from __future__ import annotations

import numpy as np

BS, ROWS, REC = 110, 16, 1760


def pack_ref(w: np.ndarray) -> np.ndarray:
    rows, rb = w.shape
    assert rows % ROWS == 0 and rb % BS == 0
    nb = rb // BS
    out = np.zeros_like(w).reshape(-1)
    src = w.reshape(rows, nb, BS)
    for t in range(rows // ROWS):
        for j in range(nb):
            rec = np.zeros(REC, dtype=np.uint8)
            for lane in range(32):
                a, s = lane >> 3, lane & 7
                stream = 0
                sc = 0
                for i in range(4):
                    b = src[16 * t + a + 4 * i, j]
                    qh = int(b[66 + s])
                    for e in range(8):
                        f = int(b[2 + 8 * s + e]) | (((qh >> e) & 1) << 8)
                        stream |= f << (9 * (8 * i + e))
                    g = int.from_bytes(bytes(b[74 + 4 * s: 78 + 4 * s]), "little")
                    o = 0
                    for e in range(8):
                        for p in range(4):
                            o |= ((g >> (4 * e + p)) & 1) << (16 * (e >> 2) + 4 * p + (e & 3))
                    rec[1152 + 16 * lane + 4 * i: 1156 + 16 * lane + 4 * i] = np.frombuffer(o.to_bytes(4, "little"), np.uint8)
                    sc |= ((int(b[106 + (s >> 1)]) >> (4 * (s & 1))) & 15) << (4 * i)
                    if s == 0:
                        rec[1728 + 2 * (4 * a + i): 1730 + 2 * (4 * a + i)] = b[0:2]
                sb = np.frombuffer(stream.to_bytes(36, "little"), np.uint8)
                rec[16 * lane: 16 * lane + 16] = sb[0:16]
                rec[512 + 16 * lane: 528 + 16 * lane] = sb[16:32]
                rec[1024 + 4 * lane: 1028 + 4 * lane] = sb[32:36]
                rec[1664 + 2 * lane: 1666 + 2 * lane] = np.frombuffer(sc.to_bytes(2, "little"), np.uint8)
            off = t * ROWS * rb + j * REC
            out[off: off + REC] = rec
    return out.reshape(rows, rb)
