"""gsq_b200 -- B200 (sm_100a) kernels for the GGUF quantised-linear path of vllm_gguf_plugin.

Importing the package loads libgsq.so (raises if it has not been built) and registers
`torch.ops._C_gguf.lcpp_*`. `gsq_b200.quantization.linear` holds the linear method and the
Python-level custom ops (`torch.ops.vllm._fused_mul_mat_gguf`, `_quantize_x_q8_1`).
"""

from . import _cabi, lcpp_ops, ops  # noqa: F401

lcpp_ops.register()

__all__ = ["_cabi", "lcpp_ops", "ops"]
