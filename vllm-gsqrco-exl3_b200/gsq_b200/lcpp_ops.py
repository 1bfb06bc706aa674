"""torch.ops._C_gguf.lcpp_* -- the reference's C++ op schemas, served by libgsq.so.

Schemas are those of plugin/vllm_gguf_plugin/csrc/lcpp_shim.cu:973-983, verbatim. As there, every
op is registered for CUDA and for CPU: on CPU every guard runs and the call then ends in
"... must be CUDA tensors" (lcpp_shim.cu:997-1008), which is how guards are tested without a GPU.

What runs underneath an op name (lcpp_shim.cu:753-909 `run`):
  * the ops that read block_q8_1 activations (`x_q8` argument; vec_q, vec_iq3, vec_iq3_mma,
    vec_own, vec_iq3_mma_packed) -> gsq_quantize_q8_1 (unless x_q8 is given) + gsq_mul_mat_vec_q8,
    as many activation rows per launch as the kernel for the type takes (8 or 48);
  * the ops that quantise X themselves (mul_mat_q, mma_k, iq3_packed) -> gsq_linear, which picks
    the activation layout together with the kernel (small-batch tensor-core kernel, tcgen05 GEMM).
Output and scratch come from torch's caching allocator on the current stream; the kernels write
X's dtype directly, so no cast kernel follows.
"""

from __future__ import annotations

import ctypes as C

import torch

from . import _cabi

_lib = _cabi.lib

IQ3_S, IQ3_XXS, Q4_K, Q6_K, IQ4_XS, IQ1_M = 21, 18, 12, 14, 23, 29
MMVQ_MAX_BATCH_SIZE = 8
MMA_K_MAX_COLS = 64
PACKED_VEC_MAX = 32

_SCHEMAS = {
    "lcpp_mul_mat_vec_q": "(Tensor W, Tensor X, int type, SymInt row, Tensor? x_q8=None) -> Tensor",
    "lcpp_mul_mat_q": "(Tensor W, Tensor X, int type, SymInt row) -> Tensor",
    "lcpp_mul_mat_vec_iq3": "(Tensor W, Tensor X, int type, SymInt row, Tensor? x_q8=None) -> Tensor",
    "lcpp_mul_mat_vec_iq3_mma": "(Tensor W, Tensor X, int type, SymInt row, Tensor? x_q8=None) -> Tensor",
    "lcpp_mul_mat_vec_own": "(Tensor W, Tensor X, int type, SymInt row, Tensor? x_q8=None) -> Tensor",
    "lcpp_mul_mat_mma_k": "(Tensor W, Tensor X, int type, SymInt row) -> Tensor",
    "lcpp_mul_mat_vec_iq3_mma_packed": "(Tensor W, Tensor X, int type, SymInt row, Tensor? x_q8=None) -> Tensor",
    "lcpp_mul_mat_iq3_packed": "(Tensor W, Tensor X, int type, SymInt row) -> Tensor",
    "lcpp_quantize_q8_1": "(Tensor X, int type, bool mmq, bool vendored) -> Tensor",
    # not in the reference: Q6_K repacked at load by this package (quantization/iq3_pack.py)
    "gsq_mul_mat_vec_q6k_packed": "(Tensor W, Tensor X, int type, SymInt row, Tensor? x_q8=None) -> Tensor",
    "gsq_mul_mat_q6k_packed": "(Tensor W, Tensor X, int type, SymInt row) -> Tensor",
}

# op -> (reads block_q8_1?, packed W?, IQ3 only?, Q4_K-own only?, mma_k types only?, is MMQ?, max X rows)
_OPS = {
    "lcpp_mul_mat_vec_q": dict(mmvq=True, max_rows=MMVQ_MAX_BATCH_SIZE),
    "lcpp_mul_mat_q": dict(mmvq=False, is_mmq=True, max_rows=0),
    "lcpp_mul_mat_vec_iq3": dict(mmvq=True, need_iq3=True, max_rows=MMVQ_MAX_BATCH_SIZE),
    "lcpp_mul_mat_vec_iq3_mma": dict(mmvq=True, need_iq3=True, max_rows=MMVQ_MAX_BATCH_SIZE),
    "lcpp_mul_mat_vec_own": dict(mmvq=True, need_q4k_own=True, max_rows=MMVQ_MAX_BATCH_SIZE),
    "lcpp_mul_mat_mma_k": dict(mmvq=False, need_mma_k=True, max_rows=MMA_K_MAX_COLS),
    "lcpp_mul_mat_vec_iq3_mma_packed": dict(mmvq=True, need_iq3=True, packed=True, max_rows=PACKED_VEC_MAX),
    "lcpp_mul_mat_iq3_packed": dict(mmvq=False, need_iq3=True, packed=True, max_rows=0),
    "gsq_mul_mat_vec_q6k_packed": dict(mmvq=True, need_q6k=True, packed=True, max_rows=MMVQ_MAX_BATCH_SIZE),
    "gsq_mul_mat_q6k_packed": dict(mmvq=False, need_q6k=True, packed=True, max_rows=0),
}

_DTYPES = {torch.float32: _cabi.F32, torch.float16: _cabi.F16, torch.bfloat16: _cabi.BF16}

# K granularity the guards demand: 512 as in the reference (MATRIX_ROW_PADDING); the tensor-parallel
# helpers lower it to 256 for K-sharded layers (gsq_b200.tp.relaxed_k).
_k_multiple = 512


# Where the next product writes its result, if set (see output_into): the kernels take any row stride, so a tensor-
# parallel runtime can have a shard's result land in its slot of a collective's buffer instead of copying it there.
_next_output: list = []


class output_into:
    """with output_into(t): the next op call of this module writes its [rows of X, row] result into `t` (same shape
    and dtype as it would have returned, unit inner stride, any row stride) and returns `t`."""

    def __init__(self, t: torch.Tensor):
        self.t = t

    def __enter__(self):
        _next_output.append(self.t)
        return self.t

    def __exit__(self, *a):
        if _next_output and _next_output[-1] is self.t:
            _next_output.pop()


# Set by tp.PeerAllReduce.fused(): the next self-quantising op call sums its result over the ranks inside its kernel
# (gsq_linear_allreduce) instead of returning this rank's partial.
_next_peer: list = []


class peer_reduce:
    """with peer_reduce(ctx): the next self-quantising op call of this module (lcpp_mul_mat_q, lcpp_mul_mat_mma_k,
    lcpp_mul_mat_iq3_packed, gsq_mul_mat_q6k_packed) is the product AND the sum of its result over the ranks of `ctx`
    (a _cabi.PeerReduce), one kernel. Raises if the shape is not one the small-batch kernel serves."""

    def __init__(self, ctx):
        self.ctx = ctx

    def __enter__(self):
        _next_peer.append(self.ctx)
        return self

    def __exit__(self, *a):
        if _next_peer and _next_peer[-1] is self.ctx:
            _next_peer.pop()


def _result(n: int, row: int, X: torch.Tensor) -> torch.Tensor:
    if _next_output:
        y = _next_output.pop()
        if y.shape != (n, row) or y.dtype != X.dtype or y.device != X.device or y.stride(1) != 1:
            raise RuntimeError("output_into: the tensor does not match the result's shape, dtype, device or inner stride")
        return y
    return torch.empty((n, row), dtype=X.dtype, device=X.device)


def set_k_multiple(v: int) -> int:
    global _k_multiple
    old, _k_multiple = _k_multiple, int(v)
    return old


PREFILL_ROUNDED, PREFILL_SPLIT, PREFILL_INTEGER = 0, 1, 2


def set_prefill_precision(mode: int) -> int:
    """How the prefill product of repacked IQ3_S is formed (gsq_prefill_precision): PREFILL_ROUNDED (default; within
    about 3e-4 of a row's norm of the reference kernels' result), PREFILL_SPLIT (about 1e-6), PREFILL_INTEGER (the
    reference's exact integer slice sums). Returns the previous mode. The environment variable GSQ_PREFILL_PRECISION
    (rounded / split / integer) sets it at import."""
    return int(_cabi.lib.gsq_prefill_precision(int(mode)))


def _stream(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def _guard(op: str, W: torch.Tensor, X: torch.Tensor, type_: int, row: int, spec: dict) -> int:
    a = _cabi.GuardArgs()
    a.op = op.encode()
    a.w_dim, a.x_dim = W.dim(), X.dim()
    a.w_is_uint8 = int(W.dtype == torch.uint8)
    if W.dim() == 2:
        a.w_size0, a.w_size1 = W.shape
        a.w_stride0, a.w_stride1 = W.stride()
    a.w_addr = W.data_ptr() if W.numel() else 0
    a.x_dtype = _DTYPES.get(X.dtype, _cabi.DTYPE_OTHER)
    if X.dim() == 2:
        a.x_size0, a.x_size1 = X.shape
        a.x_stride0, a.x_stride1 = X.stride()
    a.row, a.max_rows, a.ggml_type = int(row), spec.get("max_rows", 0), int(type_)
    a.need_iq3 = int(spec.get("need_iq3", False))
    a.need_q4k_own = int(spec.get("need_q4k_own", False))
    a.need_mma_k = int(spec.get("need_mma_k", False))
    a.is_mmq = int(spec.get("is_mmq", False))
    a.packed = int(spec.get("packed", False))
    a.k_multiple = _k_multiple
    a.w_is_cuda, a.x_is_cuda = int(W.is_cuda), int(X.is_cuda)
    a.same_device = int(W.device == X.device)
    k = C.c_int64(0)
    buf = C.create_string_buffer(512)
    if _lib.gsq_check_inputs(C.byref(a), C.byref(k), buf, len(buf)) != _cabi.OK:
        raise RuntimeError(buf.value.decode())
    return k.value


def quantize_q8_1_into(X: torch.Tensor, out: torch.Tensor) -> None:
    m, k = X.shape
    stride = k if m == 1 else X.stride(0)
    _cabi.check(_lib.gsq_quantize_q8_1(X.data_ptr(), _DTYPES[X.dtype], m, k, stride, out.data_ptr(), _stream(X.device)),
                "gsq_quantize_q8_1")


def quantize_q8_1_mmq_into(X: torch.Tensor, layout: int, out: torch.Tensor) -> None:
    m, k = X.shape
    stride = k if m == 1 else X.stride(0)
    _cabi.check(_lib.gsq_quantize_q8_1_mmq(X.data_ptr(), _DTYPES[X.dtype], m, k, stride, layout, out.data_ptr(),
                                           _stream(X.device)), "gsq_quantize_q8_1_mmq")


def _gemv(W, X, type_, row, x_q8, packed, y):
    """Rows of X, as many per call as the kernel for this type takes (8 or 48), reading block_q8_1."""
    n, k = X.shape
    per_row = k // 32 * 36
    st = _stream(X.device)
    step = _lib.gsq_mul_mat_vec_max_rows(type_, int(packed))
    for i in range(0, n, step):
        c = min(step, n - i)
        _cabi.check(
            _lib.gsq_mul_mat_vec_q8(W.data_ptr(), W.shape[1], row, type_, int(packed), x_q8.data_ptr() + i * per_row,
                                    c, k, y.data_ptr() + i * y.stride(0) * y.element_size(), _DTYPES[y.dtype],
                                    y.stride(0), st),
            "gsq_mul_mat_vec_q8")


def _run(op: str, W: torch.Tensor, X: torch.Tensor, type_: int, row: int, x_q8: torch.Tensor | None = None):
    spec = _OPS[op]
    if spec.get("need_q6k") and int(type_) != Q6_K:
        raise RuntimeError(f"{op}: Q6_K only, got type {type_}")
    k = _guard(op, W, X, type_, row, spec)
    n = X.shape[0]
    q8_bytes = n * k // 32 * 36
    if x_q8 is not None:
        if not (x_q8.dtype == torch.uint8 and x_q8.dim() == 1 and x_q8.stride(0) == 1 and x_q8.numel() >= q8_bytes):
            raise RuntimeError(f"{op}: x_q8 must be contiguous uint8 with at least {q8_bytes} bytes")
        if x_q8.data_ptr() % 16 != 0:
            raise RuntimeError(f"{op}: x_q8 must be 16-byte aligned")
        if not (x_q8.is_cuda and x_q8.device == X.device):
            raise RuntimeError(f"{op}: x_q8 must be on X's device")
    if n == 0:
        return X.new_empty((0, row))
    packed = bool(spec.get("packed", False))
    with torch.cuda.device(X.device):
        y = _result(n, row, X)
        if spec["mmvq"]:
            if x_q8 is None:
                x_q8 = torch.empty(q8_bytes, dtype=torch.uint8, device=X.device)
                quantize_q8_1_into(X, x_q8)
            _gemv(W, X, type_, row, x_q8, packed, y)
            return y
        # the ops that quantise X themselves: one library call (quantiser + kernel chosen together)
        sbytes = _lib.gsq_linear_scratch_bytes(row, n, k, type_, int(packed))
        scratch = torch.empty(max(sbytes, 1), dtype=torch.uint8, device=X.device)
        stride = k if n == 1 else X.stride(0)
        if _next_peer:
            ctx = _next_peer.pop()
            _cabi.check(
                _lib.gsq_linear_allreduce(W.data_ptr(), W.shape[1], row, type_, int(packed), X.data_ptr(), _DTYPES[X.dtype], n,
                                          k, stride, y.data_ptr(), _DTYPES[y.dtype], y.stride(0), scratch.data_ptr(), sbytes,
                                          C.byref(ctx), _stream(X.device)),
                "gsq_linear_allreduce")
            return y
        _cabi.check(
            _lib.gsq_linear(W.data_ptr(), W.shape[1], row, type_, int(packed), X.data_ptr(), _DTYPES[X.dtype], n, k, stride,
                            y.data_ptr(), _DTYPES[y.dtype], y.stride(0), scratch.data_ptr(), sbytes, _stream(X.device)),
            "gsq_linear")
        return y


def lcpp_quantize_q8_1(X: torch.Tensor, type_: int, mmq: bool, vendored: bool) -> torch.Tensor:
    """lcpp_shim.cu:949-971. `vendored` asked the reference for llama.cpp's own fp32 quantiser (a test
    hook); the arithmetic is the same, so it runs the same kernel under the same argument check."""
    ok = (_lib.gsq_type_block_bytes(int(type_)) > 0 and X.is_cuda and X.dim() == 2 and X.stride(1) == 1
          and X.shape[1] % _k_multiple == 0 and X.dtype in _DTYPES)
    if not ok:
        raise RuntimeError("lcpp_quantize_q8_1: bad arguments")
    n, k = X.shape
    if vendored and not (X.dtype == torch.float32 and (k if n == 1 else X.stride(0)) % 4 == 0):
        raise RuntimeError("vendored: fp32 X")
    with torch.cuda.device(X.device):
        if mmq:
            out = torch.empty(n * k // 128 * 144, dtype=torch.uint8, device=X.device)
            if n:
                quantize_q8_1_mmq_into(X, _lib.gsq_q8_layout_for_type(int(type_)), out)
        else:
            out = torch.empty(n * k // 32 * 36, dtype=torch.uint8, device=X.device)
            if n:
                quantize_q8_1_into(X, out)
    return out


def _make_impl(name):
    if "x_q8" in _SCHEMAS[name]:
        def impl(W, X, type, row, x_q8=None):
            return _run(name, W, X, int(type), int(row), x_q8)
    else:
        def impl(W, X, type, row):
            return _run(name, W, X, int(type), int(row))
    impl.__name__ = name
    return impl


def _make_fake(name):
    if "x_q8" in _SCHEMAS[name]:
        def fake(W, X, type, row, x_q8=None):
            return X.new_empty((X.shape[0], row))
    else:
        def fake(W, X, type, row):
            return X.new_empty((X.shape[0], row))
    return fake


_LIBRARY = None
registered: list[str] = []


def register() -> list[str]:
    """Define and implement the ops once per process. If another extension has already defined an op of
    this name in `_C_gguf` (the reference's own .so), that definition is left alone and the name is
    not in the returned list."""
    global _LIBRARY
    if _LIBRARY is not None:
        return registered
    import os

    want = os.environ.get("GSQ_PREFILL_PRECISION", "").strip().lower()
    if want:
        modes = {"rounded": PREFILL_ROUNDED, "split": PREFILL_SPLIT, "integer": PREFILL_INTEGER}
        if want not in modes:
            raise ValueError(f"GSQ_PREFILL_PRECISION={want!r}: expected one of {sorted(modes)}")
        set_prefill_precision(modes[want])
    _LIBRARY = torch.library.Library("_C_gguf", "FRAGMENT")
    for name, schema in _SCHEMAS.items():
        try:
            _LIBRARY.define(name + schema)
        except RuntimeError:
            continue
        if name == "lcpp_quantize_q8_1":
            _LIBRARY.impl(name, lcpp_quantize_q8_1, "CUDA")
            _LIBRARY.impl(name, lcpp_quantize_q8_1, "CPU")
            _LIBRARY._register_fake(name, lambda X, type, mmq, vendored: X.new_empty(
                (X.shape[0] * X.shape[1] // 128 * 144 if mmq else X.shape[0] * X.shape[1] // 32 * 36,), dtype=torch.uint8))
        else:
            impl = _make_impl(name)
            _LIBRARY.impl(name, impl, "CUDA")
            _LIBRARY.impl(name, impl, "CPU")
            _LIBRARY._register_fake(name, _make_fake(name))
        registered.append(name)
    return registered
