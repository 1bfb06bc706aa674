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
                g, tt = lane >> 2, lane & 3
                stream = 0
                sg = [0, 0, 0, 0]
                for s in range(8):
                    for h in range(2):
                        b = src[16 * t + g + 8 * h, j]
                        qh = int(b[66 + s])
                        sbits = int.from_bytes(bytes(b[74 + 4 * s: 78 + 4 * s]), "little")
                        for e in range(2):
                            f, e8 = 4 * s + 2 * h + e, 2 * tt + e
                            stream |= (int(b[2 + 8 * s + e8]) | (((qh >> e8) & 1) << 8)) << (9 * f)
                            fl = f & 7
                            for p in range(4):
                                sg[f >> 3] |= ((sbits >> (4 * e8 + p)) & 1) << (16 * (fl >> 2) + 4 * p + (fl & 3))
                sb = np.frombuffer(stream.to_bytes(36, "little"), np.uint8)
                rec[16 * lane: 16 * lane + 16] = sb[0:16]
                rec[512 + 16 * lane: 528 + 16 * lane] = sb[16:32]
                rec[1024 + 4 * lane: 1028 + 4 * lane] = sb[32:36]
                for q in range(4):
                    rec[1152 + 16 * lane + 4 * q: 1156 + 16 * lane + 4 * q] = np.frombuffer(sg[q].to_bytes(4, "little"), np.uint8)
            for g in range(8):
                for h in range(2):
                    b = src[16 * t + g + 8 * h, j]
                    rec[1664 + 8 * g + 4 * h: 1668 + 8 * g + 4 * h] = b[106:110]
                    rec[1728 + 4 * g + 2 * h: 1730 + 4 * g + 2 * h] = b[0:2]
            off = t * ROWS * rb + j * REC
            out[off: off + REC] = rec
    return out.reshape(rows, rb)


# ---------------------------------------------------------------------------------------------
# Q6_K streaming layout (csrc/gsq_repack.cu): a byte permutation inside each 16-row tile, one 3360-byte record per
# superblock. The reference does not repack Q6_K; the properties checked are the ones it checks for IQ3_S.

BS6, REC6 = 210, 3360


def pack_q6k_ref(w: np.ndarray) -> np.ndarray:
    rows, rb = w.shape
    assert rows % ROWS == 0 and rb % BS6 == 0
    nb = rb // BS6
    out = np.zeros_like(w).reshape(-1)
    src = w.reshape(rows, nb, BS6)
    for t in range(rows // ROWS):
        for j in range(nb):
            rec = np.zeros(REC6, dtype=np.uint8)
            for lane in range(32):
                g, tt = lane >> 2, lane & 3
                for h in range(2):
                    b = src[16 * t + g + 8 * h, j]
                    for n in range(2):
                        for qb in range(2):
                            for i in range(2):       # is
                                w8 = 4 * n + 2 * qb + i
                                o = 64 * lane + 32 * h + 4 * w8
                                rec[o: o + 4] = b[64 * n + 32 * qb + 16 * i + 4 * tt: 64 * n + 32 * qb + 16 * i + 4 * tt + 4]
                        for i in range(2):
                            w4 = 2 * n + i
                            o = 2048 + 32 * lane + 16 * h + 4 * w4
                            rec[o: o + 4] = b[128 + 32 * n + 16 * i + 4 * tt: 128 + 32 * n + 16 * i + 4 * tt + 4]
            for g in range(8):
                for h in range(2):
                    b = src[16 * t + g + 8 * h, j]
                    rec[3072 + 32 * g + 16 * h: 3088 + 32 * g + 16 * h] = b[192:208]
                    rec[3328 + 4 * g + 2 * h: 3330 + 4 * g + 2 * h] = b[208:210]
            off = t * ROWS * rb + j * REC6
            out[off: off + REC6] = rec
    return out.reshape(rows, rb)
