"""Input guards on CPU tensors: every guard runs, a clean call ends in "must be CUDA tensors"
(the scheme and the message fragments of the reference's tests/cpu/test_lcpp_guards.py:74-146)."""

import pytest
import torch

import gsq_b200  # noqa: F401  (registers torch.ops._C_gguf)

IQ3_S, IQ3_XXS, Q4_K, IQ1_M, IQ4_XS, IQ2_S, IQ1_S, Q6_K = 21, 18, 12, 29, 23, 22, 19, 14
TS = {IQ3_S: 110, IQ3_XXS: 98, Q4_K: 144, IQ4_XS: 136, IQ2_S: 82, IQ1_M: 56, Q6_K: 210}
K = 5120


def _w(rows, row_bytes, stride=None, offset=0, dtype=torch.uint8):
    stride = stride or row_bytes
    buf = torch.zeros(rows * stride + offset + 64, dtype=dtype)
    return buf[offset:offset + rows * stride].view(rows, stride)[:, :row_bytes]


def _case(op, type=IQ3_S, rows=256, row_bytes=None, n=4, k=K, row=None, **kw):
    rb = row_bytes if row_bytes is not None else K // 256 * TS.get(type, 110)
    return dict(op=op, type=type, rows=rows, row_bytes=rb, n=n, k=k, row=rows if row is None else row, **kw)


CASES = {}
for op in ("lcpp_mul_mat_vec_q", "lcpp_mul_mat_q"):
    n = 4 if op == "lcpp_mul_mat_vec_q" else 64
    for t in (IQ3_S, Q4_K, Q6_K, IQ4_XS):
        CASES[f"{op}-valid-{t}"] = (_case(op, t, n=n), "must be CUDA tensors")
        CASES[f"{op}-row_strided-{t}"] = (_case(op, t, n=n, stride=2 * K // 256 * TS[t]), "rows must be contiguous")
        CASES[f"{op}-w_narrow_view-{t}"] = (_case(op, t, n=n, stride=K // 256 * TS[t] + 256), "row stride")
    CASES[f"{op}-fp32_x"] = (_case(op, n=n, x_dtype="float32"), "must be CUDA tensors")
    CASES[f"{op}-iq1_s"] = (_case(op, IQ1_S, n=n), "unsupported ggml type")
    CASES[f"{op}-w_float"] = (_case(op, n=n, w_dtype="float32"), "W must be uint8")
    CASES[f"{op}-w_1d"] = (_case(op, n=n, w_1d=True), "must be 2-D")
    CASES[f"{op}-x_int"] = (_case(op, n=n, x_dtype="int32"), "X must be fp32, fp16 or bf16")
    CASES[f"{op}-row_bytes_not_blocks"] = (_case(op, n=n, row_bytes=2201), "not a multiple of the block size")
    CASES[f"{op}-k_not_512"] = (_case(op, n=n, row_bytes=110, k=256), "must be a multiple of 512")
    CASES[f"{op}-row_too_big"] = (_case(op, n=n, row=256 + 64), "out of range")
    CASES[f"{op}-row_zero"] = (_case(op, n=n, row=0), "out of range")
    CASES[f"{op}-w_transposed"] = (_case(op, n=n, rows=2200, row_bytes=256, w_t=True, row=256), "W inner stride")
    CASES[f"{op}-w_misaligned"] = (_case(op, n=n, w_offset=1), "16-byte aligned")
    CASES[f"{op}-k_mismatch"] = (_case(op, n=n, k=K // 2), "columns, W rows hold")
    CASES[f"{op}-x_noncontig"] = (_case(op, n=n, x_t=True), "X inner stride")
CASES["lcpp_mul_mat_vec_q-9_rows"] = (_case("lcpp_mul_mat_vec_q", n=9), "at most 8 rows")
CASES["lcpp_mul_mat_q-9_rows"] = (_case("lcpp_mul_mat_q", n=9), "must be CUDA tensors")
CASES["lcpp_mul_mat_q-1_row"] = (_case("lcpp_mul_mat_q", n=1), "must be CUDA tensors")
CASES["lcpp_mul_mat_vec_q-iq1_m"] = (_case("lcpp_mul_mat_vec_q", IQ1_M), "must be CUDA tensors")
CASES["lcpp_mul_mat_q-iq1_m"] = (_case("lcpp_mul_mat_q", IQ1_M, n=64), "no MMQ for IQ1_M")
for IQ3_OP in ("lcpp_mul_mat_vec_iq3", "lcpp_mul_mat_vec_iq3_mma", "lcpp_mul_mat_vec_iq3_mma_packed",
               "lcpp_mul_mat_iq3_packed"):
    packed = IQ3_OP.endswith("_packed")
    for t in (IQ3_S, IQ3_XXS):
        CASES[f"{IQ3_OP}-valid-{t}"] = (_case(IQ3_OP, t), "must be CUDA tensors")
        CASES[f"{IQ3_OP}-row_strided-{t}"] = (_case(IQ3_OP, t, stride=2 * K // 256 * TS[t]), "rows must be contiguous")
    CASES[f"{IQ3_OP}-q4_k"] = (_case(IQ3_OP, Q4_K), "IQ3_S or IQ3_XXS only")
    CASES[f"{IQ3_OP}-1_row"] = (_case(IQ3_OP, n=1), "must be CUDA tensors")
    if packed:
        CASES[f"{IQ3_OP}-32_rows"] = (_case(IQ3_OP, n=32), "must be CUDA tensors")
        if IQ3_OP == "lcpp_mul_mat_iq3_packed":
            CASES[f"{IQ3_OP}-2048_rows"] = (_case(IQ3_OP, n=2048), "must be CUDA tensors")
        else:
            CASES[f"{IQ3_OP}-33_rows"] = (_case(IQ3_OP, n=33), "at most 32 rows")
        CASES[f"{IQ3_OP}-row_not_16"] = (_case(IQ3_OP, row=200), "must be a multiple of 16")
    else:
        CASES[f"{IQ3_OP}-9_rows"] = (_case(IQ3_OP, n=9), "at most 8 rows")
    CASES[f"{IQ3_OP}-k_not_512"] = (_case(IQ3_OP, row_bytes=110, k=256), "must be a multiple of 512")
    CASES[f"{IQ3_OP}-w_misaligned"] = (_case(IQ3_OP, w_offset=1), "16-byte aligned")
    CASES[f"{IQ3_OP}-k_mismatch"] = (_case(IQ3_OP, k=K // 2), "columns, W rows hold")
OWN_OP = "lcpp_mul_mat_vec_own"
for t in (Q4_K, IQ2_S):
    CASES[f"{OWN_OP}-valid-{t}"] = (_case(OWN_OP, t), "must be CUDA tensors")
    CASES[f"{OWN_OP}-row_strided-{t}"] = (_case(OWN_OP, t, stride=2 * K // 256 * TS[t]), "rows must be contiguous")
CASES[f"{OWN_OP}-iq3_s"] = (_case(OWN_OP, IQ3_S), "Q4_K or IQ2_S only")
CASES[f"{OWN_OP}-iq4_xs"] = (_case(OWN_OP, IQ4_XS), "Q4_K or IQ2_S only")
CASES[f"{OWN_OP}-9_rows"] = (_case(OWN_OP, Q4_K, n=9), "at most 8 rows")
CASES[f"{OWN_OP}-k_not_512"] = (_case(OWN_OP, Q4_K, row_bytes=144, k=256), "must be a multiple of 512")
MMA_OP = "lcpp_mul_mat_mma_k"
for t in (Q4_K, IQ4_XS, IQ2_S):
    CASES[f"{MMA_OP}-valid-{t}"] = (_case(MMA_OP, t, n=16), "must be CUDA tensors")
CASES[f"{MMA_OP}-iq3_s"] = (_case(MMA_OP, IQ3_S, n=16), "Q4_K, IQ4_XS or IQ2_S only")
CASES[f"{MMA_OP}-64_rows"] = (_case(MMA_OP, Q4_K, n=64), "must be CUDA tensors")
CASES[f"{MMA_OP}-65_rows"] = (_case(MMA_OP, Q4_K, n=65), "at most 64 rows")
CASES[f"{MMA_OP}-k_mismatch"] = (_case(MMA_OP, Q4_K, n=16, k=K // 2), "columns, W rows hold")


def _run(c):
    W = _w(c["rows"], c["row_bytes"], c.get("stride"), c.get("w_offset", 0), getattr(torch, c.get("w_dtype", "uint8")))
    if c.get("w_t"):
        W = W.t()
    if c.get("w_1d"):
        W = W.reshape(-1)
    X = torch.zeros(c["n"], c["k"], dtype=getattr(torch, c.get("x_dtype", "bfloat16")))
    if c.get("x_t"):
        X = torch.zeros(c["k"], c["n"], dtype=X.dtype).t()
    try:
        getattr(torch.ops._C_gguf, c["op"])(W, X, c["type"], c["row"])
        return "no error"
    except RuntimeError as e:
        return str(e).splitlines()[0][:300]


def test_ops_registered_without_cuda_init():
    from gsq_b200 import lcpp_ops

    assert lcpp_ops.registered == list(lcpp_ops._SCHEMAS)
    for n in lcpp_ops._SCHEMAS:
        assert hasattr(torch.ops._C_gguf, n)
    assert torch.cuda.is_initialized() is False


@pytest.mark.parametrize("name", list(CASES))
def test_guard(name):
    got = _run(CASES[name][0])
    assert CASES[name][1] in got, got
    assert torch.cuda.is_initialized() is False


def test_relaxed_k_multiple_for_tensor_parallel_shards():
    from gsq_b200 import lcpp_ops

    c = _case("lcpp_mul_mat_vec_q", Q4_K, row_bytes=144 * 5, k=1280)
    assert "must be a multiple of 512" in _run(c)
    old = lcpp_ops.set_k_multiple(256)
    try:
        assert "must be CUDA tensors" in _run(c)
    finally:
        lcpp_ops.set_k_multiple(old)


def test_x_q8_guards():
    W = _w(256, K // 256 * 110)
    X = torch.zeros(4, K, dtype=torch.float16)
    with pytest.raises(RuntimeError, match="must be CUDA tensors"):
        torch.ops._C_gguf.lcpp_mul_mat_vec_q(W, X, IQ3_S, 256, torch.zeros(10, dtype=torch.uint8))
    with pytest.raises(RuntimeError, match="bad arguments"):
        torch.ops._C_gguf.lcpp_quantize_q8_1(X, IQ3_S, False, False)
