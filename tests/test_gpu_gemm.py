"""GPU parity of the tensor-core GEMM (gsq_mul_mat_q8, reached through the many-row torch ops): int32
slice sums bit exact, fp32 outputs within 1e-3 of the reference kernels' model (128-value q8_1 blocks:
d = 1 / (127 / amax) kept in fp32 for IQ3_S / IQ4_XS; Q4_K keeps half d and half sum x and rounds
d * sc, dmin * m to fp16), 16-bit outputs within the output rounding."""

import ctypes

import numpy as np
import pytest
import torch

import gsq_b200  # noqa: F401
from gsq_b200 import _cabi, synth
from gsq_b200.quantization import iq3_pack
from oracle import blocks, product, q8_1

pytestmark = pytest.mark.gpu
Q4_K, IQ3_S, IQ4_XS = 12, 21, 23
TYPES = {"IQ3_S": IQ3_S, "IQ4_XS": IQ4_XS, "Q4_K": Q4_K}
DEV = "cuda:0"


def _x(m, k, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(m, k, generator=g)
    x[:, torch.randperm(k, generator=g)[: max(1, k // 256)]] *= 20
    return synth.nudge_ties_torch(x.to(dtype))


def _weights(name, rows, k, seed):
    raw = synth.make_weight(TYPES[name], rows, k, seed)
    w = torch.from_numpy(raw).to(DEV)
    if name == "IQ3_S":
        iq3_pack.pack_(w, IQ3_S)
    return raw, w


def _reference(name, raw, x):
    """The reference kernels' arithmetic for the many-row path, in float64."""
    dec = blocks.decode(raw, TYPES[name])
    xf = x.float().numpy()
    if name == "Q4_K":
        q, d, s = q8_1.quantize_mmq(xf, q8_1.LAYOUT_DS4)
        dh, sh = d.astype(np.float16).astype(np.float64), s.astype(np.float16).astype(np.float64)
        # d * sc and dmin * m are rounded to fp16 by the tile loader (mmq-load-tiles.cuh:775-780)
        gs = (np.repeat(dec.d, 8, axis=1).astype(np.float16) * dec.isc.astype(np.float16)).astype(np.float64)
        mins = (np.repeat(dec.dmin, 8, axis=1).astype(np.float16) * dec.imin.astype(np.float16)).astype(np.float64)
        sums = product.block_sums(dec, q).astype(np.float64)
        return np.einsum("mns,ns,ms->mn", sums, gs, dh, optimize=True) - sh @ mins.T, q
    q, d, _ = q8_1.quantize_mmq(xf, q8_1.LAYOUT_D4)
    return product.product_q81(dec, q, d), q


def _op(name):
    return "lcpp_mul_mat_iq3_packed" if name == "IQ3_S" else "lcpp_mul_mat_q"


CASES = [("IQ3_S", 128, 512), ("IQ3_S", 272, 5120), ("IQ3_S", 48, 1024), ("Q4_K", 128, 512), ("Q4_K", 202, 5120),
         ("IQ4_XS", 128, 512), ("IQ4_XS", 202, 5120), ("IQ4_XS", 300, 17408)]


@pytest.fixture(params=["prefill", "prefill_split", "prefill_integer", "prefill_int8", "specialised", "lockstep", "default"],
                autouse=True)
def gemm_variant(request):
    """The tcgen05 GEMM kernels at every row count: the warp-specialised prefill GEMMs on operand-ordered activation
    tiles (weights decoded once per 256 tokens; for repacked IQ3_S "prefill" is the kernel with fp16 operands in its
    default form -- sub-scales and rounded activation products in the operands, sums over a superblock --,
    "prefill_split" the same with the products as fp16 pairs, "prefill_integer" the form with exact integer slice sums
    and "prefill_int8" the int8 kernel; IQ4_XS has the first two and the int8 kernel, Q4_K the first and the int8 kernel), the two older
    kernels on 128-value blocks (warp-specialised and all-warps-in-lockstep); and the library's own choice, which up
    to 48 rows is the register-operand kernel."""
    callspec = getattr(request.node, "callspec", None)
    name = callspec.params.get("name", "IQ3_S") if callspec is not None else "IQ3_S"
    if (request.param == "prefill_integer" and name != "IQ3_S") or (request.param == "prefill_split" and name == "Q4_K"):
        pytest.skip("the same kernel as 'prefill_int8' for this type")
    variant = {"prefill": 3, "prefill_split": 5, "prefill_integer": 7, "prefill_int8": 4, "specialised": 1, "lockstep": 2,
               "default": 0}[request.param]
    old = _cabi.lib.gsq_debug_gemm_variant(variant)
    old_mode = _cabi.lib.gsq_debug_mmv_mode(0 if request.param == "default" else 1)
    yield request.param
    _cabi.lib.gsq_debug_gemm_variant(old)
    _cabi.lib.gsq_debug_mmv_mode(old_mode)


@pytest.fixture(scope="module", autouse=True)
def descriptor_strides():
    """Settle which stride field of the shared-memory descriptor is which on the first case; a wrong
    guess gives garbage, not a fault (both place every access inside the tile)."""
    raw, w = _weights("Q4_K", 128, 512, 1)
    x = _x(64, 512, torch.float32, 2)
    ref, _ = _reference("Q4_K", raw, x)
    errs = {}
    for swap in (0, 1):
        _cabi.lib.gsq_debug_swap_descriptor_strides(swap)
        y = torch.ops._C_gguf.lcpp_mul_mat_q(w, x.to(DEV), Q4_K, 128)
        errs[swap] = product.rel_err(y.cpu().numpy(), ref)
    print("descriptor stride order errors:", errs)
    _cabi.lib.gsq_debug_swap_descriptor_strides(0)
    assert errs[0] <= 1e-3, errs
    yield


@pytest.mark.parametrize("name,rows,k", CASES)
@pytest.mark.parametrize("m", [9, 16, 24, 33, 48, 64, 65, 200, 300, 700])
def test_gemm_fp32_vs_reference_model(name, rows, k, m):
    raw, w = _weights(name, rows, k, 300 + rows)
    x = _x(m, k, torch.float32, 400 + m)
    y = getattr(torch.ops._C_gguf, _op(name))(w, x.to(DEV), TYPES[name], rows)
    assert y.shape == (m, rows) and y.dtype == torch.float32
    ref, _ = _reference(name, raw, x)
    err = product.rel_err(y.cpu().numpy(), ref)
    assert err <= 1e-3, err   # fp32 inputs are not tie-nudged: a few quants may round the other way (approximate reciprocal)
    full = product.product_full(raw, TYPES[name], x.float().numpy())
    assert product.rel_err(y.cpu().numpy(), full) <= (1.5e-1 if name == "Q4_K" else 3e-2)


@pytest.mark.parametrize("name", list(TYPES))
@pytest.mark.parametrize("dtype,tol", [(torch.float16, 1e-3), (torch.bfloat16, 5e-3)])
def test_gemm_16bit(name, dtype, tol):
    raw, w = _weights(name, 256, 1024, 7)
    x = _x(40, 1024, dtype, 8)
    y = getattr(torch.ops._C_gguf, _op(name))(w, x.to(DEV), TYPES[name], 256)
    assert y.dtype == dtype
    ref, _ = _reference(name, raw, x)
    assert product.rel_err(y.float().cpu().numpy(), ref) <= tol


@pytest.mark.parametrize("name,rows,k", [("IQ3_S", 144, 1024), ("Q4_K", 130, 512), ("IQ4_XS", 128, 1024)])
def test_gemm_int32_slice_sums_bit_exact(name, rows, k):
    m = 70
    raw, w = _weights(name, rows, k, 11)
    x = _x(m, k, torch.float16, 12)
    sums = torch.full((m, rows, k // 32), 0x7FFFFFFF, dtype=torch.int32, device=DEV)
    _cabi.lib.gsq_debug_gemm_dump_sums(ctypes.c_void_p(sums.data_ptr()))
    try:
        getattr(torch.ops._C_gguf, _op(name))(w, x.to(DEV), TYPES[name], rows)
        torch.cuda.synchronize()
    finally:
        _cabi.lib.gsq_debug_gemm_dump_sums(None)
    _, q = _reference(name, raw, x)
    want = product.block_sums(blocks.decode(raw, TYPES[name]), q)
    assert np.array_equal(sums.cpu().numpy(), want)


@pytest.mark.parametrize("ks", [1, 2, 4])
@pytest.mark.parametrize("name", list(TYPES))
def test_split_k_over_a_cluster(name, ks):
    """Few tiles: the superblocks of a tile are split over the CTAs of a cluster and summed in rank order."""
    raw, w = _weights(name, 256, 5120, 31)
    x = _x(20, 5120, torch.float32, 32)
    old = _cabi.lib.gsq_debug_gemm_ksplit(ks)
    try:
        y = getattr(torch.ops._C_gguf, _op(name))(w, x.to(DEV), TYPES[name], 256)
        y2 = getattr(torch.ops._C_gguf, _op(name))(w, x.to(DEV), TYPES[name], 256)
    finally:
        _cabi.lib.gsq_debug_gemm_ksplit(old)
    ref, _ = _reference(name, raw, x)
    assert product.rel_err(y.cpu().numpy(), ref) <= 1e-3
    assert torch.equal(y, y2)


def test_mma_k_op_and_graph_replay():
    raw, w = _weights("IQ4_XS", 256, 1024, 21)
    x = _x(24, 1024, torch.bfloat16, 22).to(DEV)
    eager = torch.ops._C_gguf.lcpp_mul_mat_mma_k(w, x, IQ4_XS, 256)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        out = torch.ops._C_gguf.lcpp_mul_mat_mma_k(w, x, IQ4_XS, 256)
    g.replay()
    torch.cuda.synchronize()
    assert torch.equal(out, eager)


def test_gemm_no_bounded_wait_gave_up():
    flag = ctypes.c_int(-1)
    assert _cabi.lib.gsq_device_error_flag(ctypes.byref(flag)) == 0
    assert flag.value == 0


@pytest.mark.parametrize("form", [6, 5, 7])
def test_prefill_waits_suspended_by_the_hardware_give_the_same_result(form):
    """The fp16-operand prefill GEMM (its rounded, split and integer forms) with its mbarrier waits in the time-limited
    try_wait form (gsq_debug_gemm_wait_hint) instead of polls with short sleeps: bit-identical results, no wait gives up."""
    raw, w = _weights("IQ3_S", 272, 5120, 77)
    x = _x(600, 5120, torch.bfloat16, 78).to(DEV)
    old_v = _cabi.lib.gsq_debug_gemm_variant(form)
    try:
        a = torch.ops._C_gguf.lcpp_mul_mat_iq3_packed(w, x, IQ3_S, 272)
        old_h = _cabi.lib.gsq_debug_gemm_wait_hint(2000)
        try:
            b = torch.ops._C_gguf.lcpp_mul_mat_iq3_packed(w, x, IQ3_S, 272)
        finally:
            _cabi.lib.gsq_debug_gemm_wait_hint(old_h)
        torch.cuda.synchronize()
    finally:
        _cabi.lib.gsq_debug_gemm_variant(old_v)
    assert torch.equal(a, b)
    flag = ctypes.c_int(-1)
    assert _cabi.lib.gsq_device_error_flag(ctypes.byref(flag)) == 0 and flag.value == 0
