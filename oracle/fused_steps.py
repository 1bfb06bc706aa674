"""CPU oracle (TEST INFRASTRUCTURE, not product code): the element-wise steps that stand in front of a quantised
linear, as vLLM's kernels compute them (csrc/layernorm_kernels.cu rms_norm / fused_add_rms_norm: the value scaled by
rsqrt(mean square + eps) is converted to the tensor's type before it is multiplied by the weight;
csrc/activation_kernels.cu silu_and_mul: silu in fp32, converted, multiplied by `up` in the tensor's type).

The reference runs those modules unchanged in front of GGUFLinearMethod.apply() (its layers are vLLM's). torch on the
host supplies the type conversions. The variance is summed in float64 here; the CUDA kernel sums in fp32 in a fixed
order, so a result can differ from this model in the last place of X's type where the scale lands on a rounding
boundary (the GPU test bounds how often, and checks the q8_1 bytes against the kernel's own activations bit for bit).

Only tests/, __graft_entry__.smoke() and bench.py's cpu_baseline / reference arm may import this package.
"""

from __future__ import annotations

import torch


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, residual: torch.Tensor | None = None):
    """-> (y, residual_out): x, weight, residual in one dtype (fp32 / fp16 / bf16), on the host."""
    dt = x.dtype
    z = x if residual is None else (x.float() + residual.float()).to(dt)
    zf = z.float()
    var = (zf.double() ** 2).sum(-1, keepdim=True) / x.shape[-1]
    rs = (1.0 / torch.sqrt(var + eps)).float()
    y = ((zf * rs).to(dt).float() * weight.float()).to(dt)
    return y, z


def silu_mul(gate_up: torch.Tensor):
    dt = gate_up.dtype
    inter = gate_up.shape[-1] // 2
    g, u = gate_up[..., :inter].float(), gate_up[..., inter:].float()
    act = (g / (1.0 + torch.exp(-g))).to(dt).float()
    return (act * u).to(dt)
