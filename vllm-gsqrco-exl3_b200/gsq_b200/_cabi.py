"""ctypes binding of the C ABI declared in include/gsq.h (libgsq.so, built by build.py).

There is no fallback: if the library is missing, importing this module raises, and every op of
this package fails loudly instead of computing something elsewhere.
"""

from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libgsq.so")

OK, ERR_GUARD, ERR_CUDA, ERR_UNSUPPORTED, ERR_SCRATCH, ERR_TOO_LARGE, ERR_DEVICE = 0, -1, -2, -3, -4, -5, -6
F32, F16, BF16, DTYPE_OTHER = 0, 1, 2, 99
LAYOUT_D4, LAYOUT_DS4 = 0, 1
KERNEL_NONE, KERNEL_GEMV, KERNEL_GEMM, KERNEL_MMV, KERNEL_GEMM_PREFILL = 0, 1, 2, 3, 4

EXPORTS = (
    "gsq_strerror", "gsq_last_cuda_error", "gsq_abi_version", "gsq_type_block_bytes", "gsq_check_inputs",
    "gsq_device_init", "gsq_quantize_q8_1", "gsq_quantize_q8_1_mmq", "gsq_mul_mat_vec_q8",
    "gsq_debug_block_sums", "gsq_debug_force_direct_loads", "gsq_device_error_flag", "gsq_debug_force_cluster_size",
    "gsq_debug_swap_descriptor_strides", "gsq_debug_gemm_dump_sums", "gsq_debug_gemm_ksplit", "gsq_debug_gemm_variant", "gsq_debug_gemm_wait_hint", "gsq_q8_layout_for_type", "gsq_mul_mat_scratch_bytes", "gsq_mul_mat_q8", "gsq_iq3s_repack", "gsq_route", "gsq_linear_vec_static", "gsq_linear_vec_static_max_q8_bytes",
    "gsq_debug_mmv_mode", "gsq_debug_mmv_min_rows", "gsq_debug_mmv_cluster_size", "gsq_mul_mat_vec_max_rows",
    "gsq_debug_mmv_profile", "gsq_debug_mmv_max_rows", "gsq_debug_mmv_pdl", "gsq_debug_mmv_prefetch_first", "gsq_debug_mmv_chunking", "gsq_debug_mmv_trace",
    "gsq_linear", "gsq_linear_scratch_bytes", "gsq_debug_gemm_profile", "gsq_q6k_repack", "gsq_allreduce_sum", "gsq_allreduce_error_flag", "gsq_linear_allreduce", "gsq_peer_reduce_error_flag", "gsq_rmsnorm_quantize_q8_1", "gsq_silu_mul_quantize_q8_1", "gsq_dequantize_rows", "gsq_dequantize_bad_index_flag", "gsq_prefill_precision",
)


class PeerReduce(C.Structure):
    """gsq_peer_reduce (include/gsq.h)."""
    _fields_ = [("slots", C.c_void_p), ("flags", C.c_void_p), ("state", C.c_void_p), ("rank", C.c_int), ("world", C.c_int),
                ("slot_bytes", C.c_int64)]


class GuardArgs(C.Structure):
    _fields_ = [
        ("op", C.c_char_p),
        ("w_dim", C.c_int), ("w_is_uint8", C.c_int),
        ("w_size0", C.c_int64), ("w_size1", C.c_int64), ("w_stride0", C.c_int64), ("w_stride1", C.c_int64),
        ("w_addr", C.c_uint64),
        ("x_dim", C.c_int), ("x_dtype", C.c_int),
        ("x_size0", C.c_int64), ("x_size1", C.c_int64), ("x_stride0", C.c_int64), ("x_stride1", C.c_int64),
        ("row", C.c_int64), ("max_rows", C.c_int64),
        ("ggml_type", C.c_int),
        ("need_iq3", C.c_int), ("need_q4k_own", C.c_int), ("need_mma_k", C.c_int), ("is_mmq", C.c_int),
        ("packed", C.c_int),
        ("k_multiple", C.c_int),
        ("w_is_cuda", C.c_int), ("x_is_cuda", C.c_int), ("same_device", C.c_int),
    ]


def _load() -> C.CDLL:
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python vllm-gsqrco-exl3_b200/build.py` "
            "(nvcc, sm_100a). This package has no other compute path."
        )
    lib = C.CDLL(LIB_PATH)
    i64, vp, ci, sz = C.c_int64, C.c_void_p, C.c_int, C.c_size_t
    lib.gsq_strerror.restype = C.c_char_p
    lib.gsq_strerror.argtypes = [ci]
    lib.gsq_last_cuda_error.restype = ci
    lib.gsq_abi_version.restype = ci
    lib.gsq_type_block_bytes.restype = ci
    lib.gsq_type_block_bytes.argtypes = [ci]
    lib.gsq_check_inputs.restype = ci
    lib.gsq_check_inputs.argtypes = [C.POINTER(GuardArgs), C.POINTER(i64), C.c_char_p, sz]
    lib.gsq_device_init.restype = ci
    lib.gsq_device_init.argtypes = [ci]
    lib.gsq_quantize_q8_1.restype = ci
    lib.gsq_quantize_q8_1.argtypes = [vp, ci, i64, i64, i64, vp, vp]
    lib.gsq_quantize_q8_1_mmq.restype = ci
    lib.gsq_quantize_q8_1_mmq.argtypes = [vp, ci, i64, i64, i64, ci, vp, vp]
    lib.gsq_mul_mat_vec_q8.restype = ci
    lib.gsq_mul_mat_vec_q8.argtypes = [vp, i64, i64, ci, ci, vp, i64, i64, vp, ci, i64, vp]
    lib.gsq_debug_block_sums.restype = ci
    lib.gsq_debug_block_sums.argtypes = [vp, i64, i64, ci, ci, vp, i64, i64, vp, vp, vp]
    lib.gsq_debug_force_direct_loads.restype = ci
    lib.gsq_debug_force_direct_loads.argtypes = [ci]
    lib.gsq_debug_force_cluster_size.restype = ci
    lib.gsq_debug_force_cluster_size.argtypes = [ci]
    lib.gsq_debug_swap_descriptor_strides.restype = ci
    lib.gsq_debug_swap_descriptor_strides.argtypes = [ci]
    lib.gsq_debug_gemm_variant.restype = ci
    lib.gsq_debug_gemm_wait_hint.restype = ci
    lib.gsq_debug_gemm_wait_hint.argtypes = [ci]
    lib.gsq_debug_gemm_variant.argtypes = [ci]
    lib.gsq_debug_gemm_ksplit.restype = ci
    lib.gsq_debug_gemm_ksplit.argtypes = [ci]
    lib.gsq_debug_gemm_dump_sums.restype = ci
    lib.gsq_debug_gemm_dump_sums.argtypes = [vp]
    lib.gsq_device_error_flag.restype = ci
    lib.gsq_device_error_flag.argtypes = [C.POINTER(ci)]
    lib.gsq_q8_layout_for_type.restype = ci
    lib.gsq_q8_layout_for_type.argtypes = [ci]
    lib.gsq_mul_mat_scratch_bytes.restype = sz
    lib.gsq_mul_mat_scratch_bytes.argtypes = [i64, i64, i64, ci]
    lib.gsq_mul_mat_q8.restype = ci
    lib.gsq_mul_mat_q8.argtypes = [vp, i64, i64, ci, ci, vp, i64, i64, vp, ci, i64, vp, sz, vp]
    lib.gsq_linear_scratch_bytes.restype = sz
    lib.gsq_linear_scratch_bytes.argtypes = [i64, i64, i64, ci, ci]
    lib.gsq_prefill_precision.restype = ci
    lib.gsq_prefill_precision.argtypes = [ci]
    lib.gsq_linear.restype = ci
    lib.gsq_linear.argtypes = [vp, i64, i64, ci, ci, vp, ci, i64, i64, i64, vp, ci, i64, vp, sz, vp]
    lib.gsq_iq3s_repack.restype = ci
    lib.gsq_iq3s_repack.argtypes = [vp, i64, i64, ci, vp]
    lib.gsq_allreduce_sum.restype = ci
    lib.gsq_allreduce_sum.argtypes = [vp, vp, ci, ci, i64, ci, vp, vp, vp]
    lib.gsq_allreduce_error_flag.restype = ci
    lib.gsq_allreduce_error_flag.argtypes = [C.POINTER(ci)]
    lib.gsq_linear_allreduce.restype = ci
    lib.gsq_linear_allreduce.argtypes = [vp, i64, i64, ci, ci, vp, ci, i64, i64, i64, vp, ci, i64, vp, C.c_size_t,
                                         C.POINTER(PeerReduce), vp]
    lib.gsq_rmsnorm_quantize_q8_1.restype = ci
    lib.gsq_rmsnorm_quantize_q8_1.argtypes = [vp, ci, i64, i64, i64, vp, vp, C.c_float, vp, vp, vp]
    lib.gsq_silu_mul_quantize_q8_1.restype = ci
    lib.gsq_silu_mul_quantize_q8_1.argtypes = [vp, ci, i64, i64, i64, vp, vp, vp]
    lib.gsq_dequantize_rows.restype = ci
    lib.gsq_dequantize_rows.argtypes = [vp, i64, i64, ci, vp, i64, i64, vp, ci, i64, vp]
    lib.gsq_dequantize_bad_index_flag.restype = ci
    lib.gsq_dequantize_bad_index_flag.argtypes = [C.POINTER(ci)]
    lib.gsq_peer_reduce_error_flag.restype = ci
    lib.gsq_peer_reduce_error_flag.argtypes = [C.POINTER(ci)]
    lib.gsq_q6k_repack.restype = ci
    lib.gsq_q6k_repack.argtypes = [vp, i64, i64, ci, vp]
    lib.gsq_linear_vec_static.restype = ci
    lib.gsq_linear_vec_static.argtypes = [vp, i64, i64, ci, ci, vp, ci, i64, i64, i64, vp, ci, i64, vp]
    lib.gsq_linear_vec_static_max_q8_bytes.restype = i64
    lib.gsq_debug_gemm_profile.restype = ci
    lib.gsq_debug_gemm_profile.argtypes = [vp]
    lib.gsq_debug_mmv_profile.restype = ci
    lib.gsq_debug_mmv_profile.argtypes = [vp]
    for name in ("gsq_debug_mmv_mode", "gsq_debug_mmv_min_rows", "gsq_debug_mmv_max_rows", "gsq_debug_mmv_cluster_size", "gsq_debug_mmv_pdl", "gsq_debug_mmv_prefetch_first", "gsq_debug_mmv_chunking", "gsq_debug_mmv_trace"):
        getattr(lib, name).restype = ci
        getattr(lib, name).argtypes = [ci]
    lib.gsq_mul_mat_vec_max_rows.restype = ci
    lib.gsq_mul_mat_vec_max_rows.argtypes = [ci, ci]
    lib.gsq_route.restype = ci
    lib.gsq_route.argtypes = [i64, ci, i64, i64, ci]
    return lib


lib = _load()


def check(status: int, what: str) -> None:
    """Raise RuntimeError for a non-zero status of a launch entry point."""
    if status == OK:
        return
    msg = lib.gsq_strerror(status).decode()
    if status == ERR_CUDA:
        msg += f" (cudaError {lib.gsq_last_cuda_error()})"
    raise RuntimeError(f"{what}: {msg}")
