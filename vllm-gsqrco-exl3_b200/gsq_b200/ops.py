"""Run-time switches of the quantised-linear path (plugin/vllm_gguf_plugin/ops.py:93-115 of the reference).

The reference turns its "Route L" on with VLLM_GGUF_LCPP=1 and falls back to stock kernels otherwise.
This package *is* that route and has nothing to fall back to, so LCPP_ENABLED is True unless the
variable is explicitly "0", in which case the linear method refuses to run instead of changing path.
"""

from __future__ import annotations

import os

GGML_TYPE_Q2_K, GGML_TYPE_Q4_K, GGML_TYPE_Q6_K = 10, 12, 14
GGML_TYPE_IQ2_XXS, GGML_TYPE_IQ2_XS, GGML_TYPE_IQ3_XXS = 16, 17, 18
GGML_TYPE_IQ3_S, GGML_TYPE_IQ2_S, GGML_TYPE_IQ4_XS, GGML_TYPE_IQ1_M = 21, 22, 23, 29
GGML_TYPE_F32, GGML_TYPE_F16, GGML_TYPE_BF16 = 0, 1, 30

LCPP_ENABLED = os.environ.get("VLLM_GGUF_LCPP", "1") != "0"
# types the reference's Route L accepts (ops.py:96-109) ...
LCPP_QUANT_TYPES = frozenset({
    GGML_TYPE_Q2_K, GGML_TYPE_Q4_K, GGML_TYPE_Q6_K, GGML_TYPE_IQ2_XXS, GGML_TYPE_IQ2_XS, GGML_TYPE_IQ2_S,
    GGML_TYPE_IQ3_XXS, GGML_TYPE_IQ3_S, GGML_TYPE_IQ4_XS, GGML_TYPE_IQ1_M,
})
# ... and the ones that have an sm_100a kernel here: all of them (tensor-core kernels for Q4_K, Q6_K, IQ3_S, IQ4_XS; the
# dp4a kernel of gsq_gemv_f1.cu for the rest)
B200_QUANT_TYPES = LCPP_QUANT_TYPES
UNQUANTIZED_TYPES = frozenset({GGML_TYPE_F32, GGML_TYPE_F16, GGML_TYPE_BF16})

# (values per block, bytes per block)
GGML_QUANT_SIZES = {
    GGML_TYPE_Q4_K: (256, 144), GGML_TYPE_Q6_K: (256, 210), GGML_TYPE_IQ3_S: (256, 110), GGML_TYPE_IQ4_XS: (256, 136),
    GGML_TYPE_Q2_K: (256, 84), GGML_TYPE_IQ2_XXS: (256, 66), GGML_TYPE_IQ2_XS: (256, 74), GGML_TYPE_IQ2_S: (256, 82),
    GGML_TYPE_IQ3_XXS: (256, 98), GGML_TYPE_IQ1_M: (256, 56),
    GGML_TYPE_F32: (1, 4), GGML_TYPE_F16: (1, 2), GGML_TYPE_BF16: (1, 2),
}
