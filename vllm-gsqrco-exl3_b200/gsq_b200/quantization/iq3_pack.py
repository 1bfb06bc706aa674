"""Lossless repack of IQ3_S (and Q6_K) weight bytes into the order the sm_100a kernels stream them.

Same role and interface as the reference's quantization/iq3_pack.py (pack_ / pack / unpack, ROWS = 16,
bijective, in place, tile t keeps the bytes of rows 16t..16t+15), but a different bit layout inside a
record: this one is cut for 128-bit coalesced loads and a decode of shifts, one table load and one byte
permute per four values.
The layout is documented in csrc/gsq_repack.cu; in short, per 16-row x 256-column record (1760 B)
lane l = 4g + t owns rows g and g + 8 and, of every 32-value slice s, the 4-value groups 2t and 2t + 1;
its 32 fields are numbered f = 4s + 2h + e (row g + 8h, group 2t + e):

  [0,1152)     9 words per lane (split 4 + 4 + 1 over three planes): the 32 nine-bit codebook indices,
               field f at bit 9f
  [1152,1664)  4 words per lane: word f/8, bit 16((f%8)/4) + 4p + f%4 = sign of value p of field f
  [1664,1728)  8 bytes per g: the 4 sub-scale bytes of row g, then of row g + 8
  [1728,1760)  4 bytes per g: fp16 d of row g, then of row g + 8

CUDA tensors are repacked by gsq_iq3s_repack (one thread block per tile, staged in shared memory, no
scratch); CPU tensors by the torch-op formulation below, which also serves as the layout's
executable definition for the tests.

Q6_K (type 14; not repacked by the reference, whose vendored kernels read GGUF order): GGUF's 210-byte blocks
are only 2-byte aligned, so the same functions also take Q6_K and apply a byte permutation inside each 16-row
tile into 3360-byte records (csrc/gsq_repack.cu, `q6k_record_source` below): per lane its words of low
nibbles and of high parts, then the rows' sub-scales and d.
"""

from __future__ import annotations

import torch

from .. import _cabi

IQ3_S, Q6_K = 21, 14
ROWS = 16  # rows per tile
BS = 110   # bytes per IQ3_S superblock
REC = ROWS * BS
BS_Q6K = 210
REC_Q6K = ROWS * BS_Q6K
PACKABLE_TYPES = (IQ3_S, Q6_K)


def _check(w: torch.Tensor, weight_type: int) -> None:
    assert int(weight_type) in PACKABLE_TYPES, weight_type
    bs = BS if int(weight_type) == IQ3_S else BS_Q6K
    assert w.dtype == torch.uint8 and w.dim() == 2, (w.shape, w.dtype)
    assert w.shape[0] % ROWS == 0 and w.shape[1] % bs == 0, w.shape


def q6k_record_source() -> torch.Tensor:
    """int64 [3360]: byte o of a Q6_K record comes from byte (row * 210 + src) of the tile's 16 blocks of that
    superblock (row = row of the tile). The layout's definition, as in csrc/gsq_repack.cu."""
    o = torch.arange(REC_Q6K)
    row = torch.zeros_like(o)
    src = torch.zeros_like(o)
    m = o < 2048
    lane, w, b = o >> 6, (o & 63) >> 2, o & 3
    g, t, h, wi = lane >> 2, lane & 3, w >> 3, w & 7
    row = torch.where(m, g + 8 * h, row)
    src = torch.where(m, 64 * (wi >> 2) + 32 * ((wi >> 1) & 1) + 16 * (wi & 1) + 4 * t + b, src)
    m = (o >= 2048) & (o < 3072)
    q = o - 2048
    lane, w, b = q >> 5, (q & 31) >> 2, q & 3
    g, t, h, wi = lane >> 2, lane & 3, w >> 2, w & 3
    row = torch.where(m, g + 8 * h, row)
    src = torch.where(m, 128 + 32 * (wi >> 1) + 16 * (wi & 1) + 4 * t + b, src)
    m = (o >= 3072) & (o < 3328)
    q = o - 3072
    row = torch.where(m, (q >> 5) + 8 * ((q >> 4) & 1), row)
    src = torch.where(m, 192 + (q & 15), src)
    m = o >= 3328
    q = o - 3328
    row = torch.where(m, (q >> 2) + 8 * ((q >> 1) & 1), row)
    src = torch.where(m, 208 + (q & 1), src)
    return row * BS_Q6K + src


def _q6k_tiles(w: torch.Tensor, inverse: bool) -> torch.Tensor:
    rows, rb = w.shape
    nb, t = rb // BS_Q6K, rows // ROWS
    perm = q6k_record_source().to(w.device)
    if not inverse:
        blocks = w.reshape(t, ROWS, nb, BS_Q6K).permute(0, 2, 1, 3).reshape(t, nb, REC_Q6K)   # [tile, sb, row * 210 + byte]
        return blocks[..., perm].reshape(rows, rb)
    rec = w.reshape(t, nb, REC_Q6K)
    blocks = torch.empty_like(rec)
    blocks[..., perm] = rec
    return blocks.reshape(t, nb, ROWS, BS_Q6K).permute(0, 2, 1, 3).reshape(rows, rb)


def _bits(x: torch.Tensor, n: int) -> torch.Tensor:
    """[..., n] the low n bits of an integer tensor, LSB first."""
    return (x.unsqueeze(-1) >> torch.arange(n, device=x.device)) & 1


def _le(x: torch.Tensor, nbytes: int) -> torch.Tensor:
    """integer tensor -> its little-endian bytes as a new last axis"""
    return ((x.unsqueeze(-1) >> (8 * torch.arange(nbytes, device=x.device))) & 0xFF).to(torch.uint8)


def _word(x: torch.Tensor, nbytes: int) -> torch.Tensor:
    """[..., n * nbytes] bytes -> [..., n] little-endian integers"""
    x = x.reshape(*x.shape[:-1], -1, nbytes)
    return (x << (8 * torch.arange(nbytes, device=x.device))).sum(-1)


def _pack_tiles(w: torch.Tensor) -> torch.Tensor:
    rows, rb = w.shape
    nb = rb // BS
    t = rows // ROWS
    dev = w.device
    # [tile, block, h, g, byte]: row = 8 h + g
    b = w.reshape(t, 2, 8, nb, BS).permute(0, 3, 1, 2, 4).to(torch.int64)
    qs = b[..., 2:66].reshape(t, nb, 2, 8, 8, 4, 2)                   # h g s t e   (group 2t + e of slice s)
    qh = _bits(b[..., 66:74], 8).reshape(t, nb, 2, 8, 8, 4, 2)        # h g s t e
    field = (qs | (qh << 8)).permute(0, 1, 3, 5, 4, 2, 6)             # g t s h e: lane 4g + t, field 4s + 2h + e
    fbits = _bits(field.reshape(t, nb, 32, 32), 9).reshape(t, nb, 32, 288)
    words = (fbits.reshape(t, nb, 32, 9, 32) << torch.arange(32, device=dev)).sum(-1)     # lane, word
    # sign bits: GGUF bit 4 (2t + e) + p of the slice's 32-bit word
    sg = _bits(b[..., 74:106], 8).reshape(t, nb, 2, 8, 8, 4, 2, 4)    # h g s t e p
    sg = sg.permute(0, 1, 3, 5, 4, 2, 6, 7).reshape(t, nb, 32, 4, 2, 4, 4)     # lane, word f/8, (f%8)/4, f%4, p
    sgw = (sg.permute(0, 1, 2, 3, 4, 6, 5).reshape(t, nb, 32, 4, 32) << torch.arange(32, device=dev)).sum(-1)
    sc = b[..., 106:110].permute(0, 1, 3, 2, 4)                       # g h byte
    d = b[..., 0:2].permute(0, 1, 3, 2, 4)                            # g h byte
    out = torch.empty(t, nb, REC, dtype=torch.uint8, device=dev)
    out[..., 0:512] = _le(words[..., 0:4], 4).reshape(t, nb, 512)
    out[..., 512:1024] = _le(words[..., 4:8], 4).reshape(t, nb, 512)
    out[..., 1024:1152] = _le(words[..., 8], 4).reshape(t, nb, 128)
    out[..., 1152:1664] = _le(sgw, 4).reshape(t, nb, 512)
    out[..., 1664:1728] = sc.reshape(t, nb, 64).to(torch.uint8)
    out[..., 1728:1760] = d.reshape(t, nb, 32).to(torch.uint8)
    return out.reshape(rows, rb)


def _unpack_tiles(p: torch.Tensor) -> torch.Tensor:
    rows, rb = p.shape
    nb = rb // BS
    t = rows // ROWS
    dev = p.device
    r = p.reshape(t, nb, REC).to(torch.int64)
    words = torch.cat([_word(r[..., 0:512], 4).reshape(t, nb, 32, 4), _word(r[..., 512:1024], 4).reshape(t, nb, 32, 4),
                       _word(r[..., 1024:1152], 4).reshape(t, nb, 32, 1)], -1)      # lane, 9
    fbits = _bits(words, 32).reshape(t, nb, 32, 32, 9)                              # lane, field, bit
    field = (fbits << torch.arange(9, device=dev)).sum(-1).reshape(t, nb, 8, 4, 8, 2, 2)   # g t s h e
    field = field.permute(0, 1, 5, 2, 4, 3, 6).reshape(t, nb, 2, 8, 8, 8)           # h g s e8
    qs = field & 0xFF
    qh = ((field >> 8) << torch.arange(8, device=dev)).sum(-1)                      # h g s
    sgw = _word(r[..., 1152:1664], 4).reshape(t, nb, 32, 4)                         # lane, word
    sb = _bits(sgw, 32).reshape(t, nb, 8, 4, 4, 2, 4, 4)                            # g t word fh p fl
    sb = sb.permute(0, 1, 2, 3, 4, 5, 7, 6).reshape(t, nb, 8, 4, 8, 2, 2, 4)        # g t (f = s h e) p
    sb = sb.permute(0, 1, 5, 2, 4, 3, 6, 7).reshape(t, nb, 2, 8, 8, 4, 8)           # h g s byte bit (bit 4 e8 + p)
    sg = (sb << torch.arange(8, device=dev)).sum(-1)                                # h g s byte
    sc = r[..., 1664:1728].reshape(t, nb, 8, 2, 4).permute(0, 1, 3, 2, 4)           # h g byte
    d = r[..., 1728:1760].reshape(t, nb, 8, 2, 2).permute(0, 1, 3, 2, 4)            # h g byte
    blocks = torch.cat([d, qs.reshape(t, nb, 2, 8, 64), qh, sg.reshape(t, nb, 2, 8, 32), sc], -1)   # h g 110
    return blocks.permute(0, 2, 3, 1, 4).reshape(rows, rb).to(torch.uint8)


def _cuda_repack(w: torch.Tensor, direction: int, weight_type: int = IQ3_S) -> None:
    if w.stride(1) != 1 or w.stride(0) != w.shape[1]:
        raise RuntimeError("iq3_pack: rows must be contiguous")
    if w.data_ptr() % 16 != 0:
        raise RuntimeError("iq3_pack: data must be 16-byte aligned")
    with torch.cuda.device(w.device):
        st = torch.cuda.current_stream(w.device).cuda_stream
        if int(weight_type) == Q6_K:
            _cabi.check(_cabi.lib.gsq_q6k_repack(w.data_ptr(), w.shape[0], w.shape[1], direction, st), "gsq_q6k_repack")
        else:
            _cabi.check(_cabi.lib.gsq_iq3s_repack(w.data_ptr(), w.shape[0], w.shape[1], direction, st), "gsq_iq3s_repack")


def pack_(w: torch.Tensor, weight_type: int) -> None:
    """pack() in place."""
    _check(w, weight_type)
    if w.is_cuda:
        _cuda_repack(w, 0, weight_type)
    elif int(weight_type) == Q6_K:
        w.copy_(_q6k_tiles(w, False))
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
        _cuda_repack(w, 1, weight_type)
        return w
    if int(weight_type) == Q6_K:
        return _q6k_tiles(p, True)
    return _unpack_tiles(p)
