"""The element-wise step in front of a quantised linear fused with its q8_1 quantiser (gsq_rmsnorm_quantize_q8_1,
gsq_silu_mul_quantize_q8_1): what a decoder layer does between two linears, in one launch each.

The reference's layers run vLLM's RMSNorm / SiluAndMul modules and quantise inside apply()
(plugin/vllm_gguf_plugin/quantization/linear.py:527-570 -> _quantize_x_q8_1, 251-268); these functions return the
block_q8_1 bytes that the vec ops take as their `x_q8` argument (torch.ops._C_gguf.lcpp_mul_mat_vec_* and
torch.ops.vllm._fused_mul_mat_gguf), plus, on request, the activations themselves for the other consumers.
"""

from __future__ import annotations

import torch

from . import _cabi

_DTYPES = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}


def _stream(dev) -> int:
    return torch.cuda.current_stream(dev).cuda_stream


def rmsnorm_quantize_q8_1(x: torch.Tensor, weight: torch.Tensor, eps: float, residual: torch.Tensor | None = None,
                          want_y: bool = False):
    """-> (x_q8, y or None). x [m, k]; weight [k] in x's dtype; residual: None, or [m, k] contiguous, updated in place to
    x + residual before the norm (vLLM's fused_add_rms_norm). x_q8: uint8 [m * k/32 * 36]."""
    if not (x.is_cuda and x.dim() == 2 and x.stride(1) == 1 and x.dtype in _DTYPES and x.shape[1] % 32 == 0):
        raise RuntimeError("rmsnorm_quantize_q8_1: x must be a CUDA [m, k] tensor, unit inner stride, k % 32 == 0")
    m, k = x.shape
    if not (weight.shape == (k,) and weight.dtype == x.dtype and weight.device == x.device and weight.is_contiguous()):
        raise RuntimeError("rmsnorm_quantize_q8_1: weight must be [k] in x's dtype on x's device")
    if residual is not None and not (residual.shape == x.shape and residual.dtype == x.dtype and residual.is_contiguous()
                                     and residual.device == x.device):
        raise RuntimeError("rmsnorm_quantize_q8_1: residual must be contiguous and match x")
    with torch.cuda.device(x.device):
        xq = torch.empty(m * k // 32 * 36, dtype=torch.uint8, device=x.device)
        y = torch.empty(m, k, dtype=x.dtype, device=x.device) if want_y else None
        if m:
            _cabi.check(_cabi.lib.gsq_rmsnorm_quantize_q8_1(
                x.data_ptr(), _DTYPES[x.dtype], m, k, k if m == 1 else x.stride(0), residual.data_ptr() if residual is not None else None,
                weight.data_ptr(), float(eps), xq.data_ptr(), y.data_ptr() if want_y else None, _stream(x.device)),
                "gsq_rmsnorm_quantize_q8_1")
    return xq, y


def silu_mul_quantize_q8_1(gate_up: torch.Tensor, want_y: bool = False):
    """-> (x_q8, y or None). gate_up [m, 2 * inter], gate columns first; x_q8 of silu(gate) * up: uint8 [m * inter/32 * 36]."""
    if not (gate_up.is_cuda and gate_up.dim() == 2 and gate_up.stride(1) == 1 and gate_up.dtype in _DTYPES
            and gate_up.shape[1] % 64 == 0):
        raise RuntimeError("silu_mul_quantize_q8_1: gate_up must be a CUDA [m, 2 * inter] tensor, unit inner stride, inter % 32 == 0")
    m, inter = gate_up.shape[0], gate_up.shape[1] // 2
    with torch.cuda.device(gate_up.device):
        xq = torch.empty(m * inter // 32 * 36, dtype=torch.uint8, device=gate_up.device)
        y = torch.empty(m, inter, dtype=gate_up.dtype, device=gate_up.device) if want_y else None
        if m:
            _cabi.check(_cabi.lib.gsq_silu_mul_quantize_q8_1(
                gate_up.data_ptr(), _DTYPES[gate_up.dtype], m, inter, 2 * inter if m == 1 else gate_up.stride(0), xq.data_ptr(),
                y.data_ptr() if want_y else None, _stream(gate_up.device)), "gsq_silu_mul_quantize_q8_1")
    return xq, y
