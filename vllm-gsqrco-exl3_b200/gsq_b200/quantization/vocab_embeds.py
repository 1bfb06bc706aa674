"""Quantised embedding look-up: the rows of a GGUF-quantised table selected by token ids, dequantised.

Mirrors the part of the reference's quantization/vocal_embeds.py that computes (79-98: `_apply_gguf_embedding` =
torch.index_select of the quantised rows + ops.ggml_dequantize; 186-194: GGUFEmbeddingMethod.embedding), on one CUDA
kernel (gsq_dequantize_rows) that gathers and dequantises in one pass. The module / parameter plumbing of vLLM's
VocabParallelEmbedding stays with the host framework.
"""

from __future__ import annotations

import torch

from .. import _cabi, ops

_DTYPES = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}


def apply_gguf_embedding(x: torch.Tensor, weight: torch.Tensor, weight_type: int, hidden_size: int,
                         dtype: torch.dtype | None = None) -> torch.Tensor:
    """x: integer token ids (any shape); weight: uint8 [vocab, row_bytes] in GGUF order (or the table itself for
    F32 / F16 / BF16); -> [*x.shape, hidden_size] in `dtype` (fp16 when None, as the reference's op)."""
    if weight_type in ops.UNQUANTIZED_TYPES:
        return torch.embedding(weight, x)
    if weight_type not in ops.LCPP_QUANT_TYPES:
        raise NotImplementedError(f"Unsupported GGUF quantization type: {weight_type}")
    dtype = dtype or torch.float16
    if dtype not in _DTYPES:
        raise RuntimeError("apply_gguf_embedding: dtype must be fp32, fp16 or bf16")
    if not (weight.is_cuda and weight.dtype == torch.uint8 and weight.dim() == 2 and weight.is_contiguous()):
        raise RuntimeError("apply_gguf_embedding: weight must be a contiguous CUDA uint8 [vocab, row_bytes] tensor")
    bs = _cabi.lib.gsq_type_block_bytes(int(weight_type))
    if bs <= 0 or weight.shape[1] % bs != 0 or weight.shape[1] // bs * 256 != hidden_size:
        raise RuntimeError(f"apply_gguf_embedding: row bytes {weight.shape[1]} do not hold {hidden_size} values of type {weight_type}")
    ids = x.reshape(-1).to(device=weight.device, dtype=torch.int64).contiguous()
    n = ids.numel()
    with torch.cuda.device(weight.device):
        out = torch.empty(n, hidden_size, dtype=dtype, device=weight.device)
        if n:
            _cabi.check(_cabi.lib.gsq_dequantize_rows(
                weight.data_ptr(), weight.shape[1], weight.shape[0], int(weight_type), ids.data_ptr(), n, hidden_size,
                out.data_ptr(), _DTYPES[dtype], hidden_size, torch.cuda.current_stream(weight.device).cuda_stream),
                "gsq_dequantize_rows")
    return out.view(*x.shape, hidden_size)


def dequantize(weight: torch.Tensor, weight_type: int, dtype: torch.dtype = torch.float16) -> torch.Tensor:
    """All rows of `weight`, dequantised (the reference's ops.ggml_dequantize on a whole tensor)."""
    bs = _cabi.lib.gsq_type_block_bytes(int(weight_type))
    k = weight.shape[1] // bs * 256
    with torch.cuda.device(weight.device):
        out = torch.empty(weight.shape[0], k, dtype=dtype, device=weight.device)
        if weight.shape[0]:
            _cabi.check(_cabi.lib.gsq_dequantize_rows(
                weight.data_ptr(), weight.shape[1], weight.shape[0], int(weight_type), None, weight.shape[0], k, out.data_ptr(),
                _DTYPES[dtype], k, torch.cuda.current_stream(weight.device).cuda_stream), "gsq_dequantize_rows")
    return out
