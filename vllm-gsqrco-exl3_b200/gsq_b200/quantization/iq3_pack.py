"""Lossless repack of IQ3_S weight bytes into the order the sm_100a kernels stream them.

Same role and interface as the reference's quantization/iq3_pack.py (pack_ / pack / unpack, ROWS = 16,
bijective, in place, tile t keeps the bytes of rows 16t..16t+15), a different layout: the reference's
is cut for mma.sync fragments, this one for 128-bit coalesced loads and a cheap register decode.
The layout is documented in csrc/gsq_repack.cu; in short, per 16-row x 256-column record (1760 B)
lane l = 8a + s owns slice s of rows a, a+4, a+8, a+12:

  [0,1152)     9 words per lane (split 4 + 4 + 1 over three planes): 32 nine-bit codebook indices,
               row i group e at bit 9(8i+e)
  [1152,1664)  4 words per lane: sign bits of row i, bit 16(e/4)+4p+e%4 = sign of value p of group e
  [1664,1728)  2 bytes per lane: nibble i = sub-scale of row i
  [1728,1760)  fp16 d of row a+4i at halfword 4a+i

CUDA tensors are repacked by gsq_iq3s_repack (one thread block per tile, staged in shared memory, no
scratch); CPU tensors by the torch-op formulation below, which also serves as the layout's
executable definition for the tests.
"""

from __future__ import annotations

import torch

from .. import _cabi

IQ3_S = 21
ROWS = 16  # rows per tile
BS = 110   # bytes per IQ3_S superblock
REC = ROWS * BS


def _check(w: torch.Tensor, weight_type: int) -> None:
    assert int(weight_type) == IQ3_S, weight_type
    assert w.dtype == torch.uint8 and w.dim() == 2, (w.shape, w.dtype)
    assert w.shape[0] % ROWS == 0 and w.shape[1] % BS == 0, w.shape


def _bits(x: torch.Tensor, n: int) -> torch.Tensor:
    """[..., n] the low n bits of an integer tensor, LSB first."""
    return (x.unsqueeze(-1) >> torch.arange(n, device=x.device)) & 1


def _pack_tiles(w: torch.Tensor) -> torch.Tensor:
    rows, rb = w.shape
    nb = rb // BS
    t = rows // ROWS
    # [tile, block, i, a, byte]: row = 4 i + a
    b = w.reshape(t, 4, 4, nb, BS).permute(0, 3, 1, 2, 4).to(torch.int64)
    qs = b[..., 2:66].reshape(t, nb, 4, 4, 8, 8)                      # i a s e
    qh = _bits(b[..., 66:74], 8)                                     # i a s e
    field = qs | (qh << 8)                                           # 9-bit index of (i, a, s, e)
    # 288-bit stream per lane (a, s): field (i, e) at bit 9 (8 i + e)
    fbits = _bits(field, 9).permute(0, 1, 3, 4, 2, 5, 6).reshape(t, nb, 32, 288)   # lane, bit
    words = (fbits.reshape(t, nb, 32, 9, 32) << torch.arange(32, device=w.device)).sum(-1)   # lane, word
    sg = b[..., 74:106].reshape(t, nb, 4, 4, 8, 4)                   # i a s byte
    sgbits = _bits(sg, 8).reshape(t, nb, 4, 4, 8, 2, 4, 4)           # i a s h e' p   (bit 4e+p of the slice word, e = 4h+e')
    spread = sgbits.permute(0, 1, 2, 3, 4, 5, 7, 6).reshape(t, nb, 4, 4, 8, 32)    # bit 16h + 4p + e'
    sgw = (spread << torch.arange(32, device=w.device)).sum(-1)      # i a s
    sgw = sgw.permute(0, 1, 3, 4, 2)                                 # a s i
    sc = b[..., 106:110]                                             # i a byte
    nib = torch.stack([sc & 15, sc >> 4], -1).reshape(t, nb, 4, 4, 8)               # i a s
    scw = (nib.permute(0, 1, 3, 4, 2) << (4 * torch.arange(4, device=w.device))).sum(-1)   # a s
    d = b[..., 0] | (b[..., 1] << 8)                                 # i a
    d = d.permute(0, 1, 3, 2)                                        # a i

    def le(x, nbytes):  # integer tensor -> little-endian bytes appended as a last axis
        return ((x.unsqueeze(-1) >> (8 * torch.arange(nbytes, device=w.device))) & 0xFF).to(torch.uint8)

    out = torch.empty(t, nb, REC, dtype=torch.uint8, device=w.device)
    out[..., 0:512] = le(words[..., 0:4], 4).reshape(t, nb, 512)
    out[..., 512:1024] = le(words[..., 4:8], 4).reshape(t, nb, 512)
    out[..., 1024:1152] = le(words[..., 8], 4).reshape(t, nb, 128)
    out[..., 1152:1664] = le(sgw, 4).reshape(t, nb, 512)
    out[..., 1664:1728] = le(scw, 2).reshape(t, nb, 64)
    out[..., 1728:1760] = le(d, 2).reshape(t, nb, 32)
    return out.reshape(rows, rb)


def _unpack_tiles(p: torch.Tensor) -> torch.Tensor:
    rows, rb = p.shape
    nb = rb // BS
    t = rows // ROWS
    r = p.reshape(t, nb, REC).to(torch.int64)

    def word(x, nbytes):  # [..., n * nbytes] bytes -> [..., n] little-endian integers
        x = x.reshape(*x.shape[:-1], -1, nbytes)
        return (x << (8 * torch.arange(nbytes, device=p.device))).sum(-1)

    words = torch.cat([word(r[..., 0:512], 4).reshape(t, nb, 32, 4), word(r[..., 512:1024], 4).reshape(t, nb, 32, 4),
                       word(r[..., 1024:1152], 4).reshape(t, nb, 32, 1)], -1)       # lane, 9
    fbits = _bits(words, 32).reshape(t, nb, 4, 8, 4, 8, 9)                          # a s i e bit
    field = (fbits << torch.arange(9, device=p.device)).sum(-1)                    # a s i e
    field = field.permute(0, 1, 4, 2, 3, 5)                                         # i a s e
    qs = field & 0xFF
    qh = ((field >> 8) << torch.arange(8, device=p.device)).sum(-1)                 # i a s
    sgw = word(r[..., 1152:1664], 4).reshape(t, nb, 4, 8, 4)                        # a s i
    sbits = _bits(sgw, 32).reshape(t, nb, 4, 8, 4, 2, 4, 4)                         # a s i h p e'
    gg = sbits.permute(0, 1, 2, 3, 4, 5, 7, 6).reshape(t, nb, 4, 8, 4, 4, 8)        # a s i byte bit (bit 4e+p)
    sg = (gg << torch.arange(8, device=p.device)).sum(-1)                           # a s i byte
    sg = sg.permute(0, 1, 4, 2, 3, 5)                                               # i a s byte
    scw = word(r[..., 1664:1728], 2).reshape(t, nb, 4, 8)                           # a s
    nib = (scw.unsqueeze(-1) >> (4 * torch.arange(4, device=p.device))) & 15        # a s i
    nib = nib.permute(0, 1, 4, 2, 3)                                                # i a s
    sc = nib[..., 0::2] | (nib[..., 1::2] << 4)                                     # i a byte
    d = word(r[..., 1728:1760], 2).reshape(t, nb, 4, 4).permute(0, 1, 3, 2)         # i a
    blocks = torch.cat([(d & 0xFF).unsqueeze(-1), (d >> 8).unsqueeze(-1), qs.reshape(t, nb, 4, 4, 64), qh,
                        sg.reshape(t, nb, 4, 4, 32), sc], -1)                       # i a 110
    return blocks.permute(0, 2, 3, 1, 4).reshape(rows, rb).to(torch.uint8)


def _cuda_repack(w: torch.Tensor, direction: int) -> None:
    if w.stride(1) != 1 or w.stride(0) != w.shape[1]:
        raise RuntimeError("iq3_pack: rows must be contiguous")
    if w.data_ptr() % 16 != 0:
        raise RuntimeError("iq3_pack: data must be 16-byte aligned")
    with torch.cuda.device(w.device):
        st = torch.cuda.current_stream(w.device).cuda_stream
        _cabi.check(_cabi.lib.gsq_iq3s_repack(w.data_ptr(), w.shape[0], w.shape[1], direction, st), "gsq_iq3s_repack")


def pack_(w: torch.Tensor, weight_type: int) -> None:
    """pack() in place."""
    _check(w, weight_type)
    if w.is_cuda:
        _cuda_repack(w, 0)
    else:
        w.copy_(_pack_tiles(w))


def pack(w: torch.Tensor, weight_type: int) -> torch.Tensor:
    """[rows, row_bytes] uint8 GGUF blocks (rows % 16 == 0) -> the packed bytes, same shape."""
    p = w.clone()
    pack_(p, weight_type)
    return p


def unpack(p: torch.Tensor, weight_type: int) -> torch.Tensor:
    """Inverse of pack: the GGUF block bytes."""
    _check(p, weight_type)
    if p.is_cuda:
        w = p.clone()
        _cuda_repack(w, 1)
        return w
    return _unpack_tiles(p)
