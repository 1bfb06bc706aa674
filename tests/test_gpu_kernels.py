"""GPU parity: the CUDA path (through the torch ops, hence through the C ABI) against the CPU oracle
on the same seeded inputs. Acceptance follows the reference's metric (tests/gpu/_refs.py:94-99,
max over activation rows of ||y - ref|| / ||ref||):

  q8_1 bytes          bit exact on tie-free 16-bit inputs (int8 values always; the stored half d may
                      sit one half-ulp off on a few blocks because amax/127 is an approximate division
                      on the GPU, as in the reference's fast-math build)
  int32 slice sums    bit exact
  fp32 outputs        <= 1e-3 of the q8_1 model of the reference kernels, <= 1e-2 of dequant + matmul
  16-bit outputs      the same plus the output rounding: 1e-3 (fp16), 5e-3 (bf16)
"""

import numpy as np
import pytest
import torch

import gsq_b200  # noqa: F401
from gsq_b200 import _cabi, synth
from gsq_b200.quantization import iq3_pack, linear
from oracle import blocks, product, q8_1

pytestmark = pytest.mark.gpu

Q4_K, Q6_K, IQ3_S, IQ4_XS = 12, 14, 21, 23
TYPES = {"IQ3_S": IQ3_S, "IQ4_XS": IQ4_XS, "Q4_K": Q4_K, "Q6_K": Q6_K}
TOL = {torch.float32: 1e-3, torch.float16: 1e-3, torch.bfloat16: 5e-3}
DEV = "cuda:0"


def _x(m, k, dtype, seed, outliers=True):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(m, k, generator=g)
    if outliers:
        x[:, torch.randperm(k, generator=g)[: max(1, k // 256)]] *= 20
    return synth.nudge_ties_torch(x.to(dtype))


def _to_np(x):
    return x.float().cpu().numpy()


def _oracle_q8(x):
    return q8_1.quantize_q8_1(_to_np(x))


# ------------------------------------------------------------------------------------------ quantise

@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
@pytest.mark.parametrize("m,k", [(1, 5120), (8, 17408), (3, 512), (48, 1024)])
def test_quantize_q8_1_bytes(dtype, m, k):
    x = _x(m, k, dtype, 100 + m)
    got = torch.ops._C_gguf.lcpp_quantize_q8_1(x.to(DEV), IQ3_S, False, False).cpu().numpy()
    want = q8_1.q8_1_bytes(_to_np(x))
    assert got.shape == want.shape
    g, w = got.reshape(-1, 36), want.reshape(-1, 36)
    bad_q = int((g[:, 4:] != w[:, 4:]).sum())
    assert bad_q <= (0 if dtype != torch.float32 else 2), bad_q          # fp32 inputs are not tie-nudged
    gd, wd = g[:, 0:2].copy().view(np.uint16)[:, 0].astype(np.int32), w[:, 0:2].copy().view(np.uint16)[:, 0].astype(np.int32)
    assert np.abs(gd - wd).max() <= 1 and (gd != wd).mean() <= 2e-3
    assert np.array_equal(g[:, 2:4], w[:, 2:4])                           # half(sum x): same summation tree


def test_quantize_strided_and_zero_blocks():
    big = torch.randn(5, 1536, dtype=torch.float16)
    big[:, 1024:1056] = 0
    big = synth.nudge_ties_torch(big)
    x = big.to(DEV)[:, 512:1536]                                          # row stride 1536, 1024 columns
    got = torch.ops._C_gguf.lcpp_quantize_q8_1(x, Q4_K, False, False).cpu().numpy().reshape(-1, 36)
    want = q8_1.q8_1_bytes(_to_np(big[:, 512:1536])).reshape(-1, 36)
    assert np.array_equal(got[:, 4:], want[:, 4:]) and np.array_equal(got[:, 2:4], want[:, 2:4])
    zero_blocks = got.reshape(5, 32, 36)[:, 16]
    assert (zero_blocks == 0).all()


@pytest.mark.parametrize("wtype", [IQ3_S, Q4_K])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_quantize_mmq_layouts(wtype, dtype):
    m, k = 5, 1024
    x = _x(m, k, dtype, 7)
    layout = q8_1.LAYOUT_DS4 if wtype == Q4_K else q8_1.LAYOUT_D4
    got = torch.ops._C_gguf.lcpp_quantize_q8_1(x.to(DEV), wtype, True, False).cpu().numpy().reshape(k // 128, m, 144)
    want = q8_1.q8_1_mmq_bytes(_to_np(x), layout).reshape(k // 128, m, 144)
    assert np.array_equal(got[..., 16:], want[..., 16:])
    if layout == q8_1.LAYOUT_D4:
        gd, wd = got[..., :16].copy().view(np.float32), want[..., :16].copy().view(np.float32)
        assert np.allclose(gd, wd, rtol=5e-7, atol=0)                     # d = 1 / (127 / amax), both approximate
    else:
        gd, wd = got[..., :16].copy().view(np.float16).astype(np.float32), want[..., :16].copy().view(np.float16).astype(np.float32)
        assert np.allclose(gd, wd, rtol=2e-3, atol=1e-3)


# ------------------------------------------------------------------------------------------ products

def _weights(name, rows, k, seed, packed=False):
    raw = synth.make_weight(TYPES[name], rows, k, seed)
    w = torch.from_numpy(raw).to(DEV)
    if packed:
        iq3_pack.pack_(w, IQ3_S)
    return raw, w


def _op_for(name, packed):
    if name == "IQ3_S":
        return "lcpp_mul_mat_vec_iq3_mma_packed" if packed else "lcpp_mul_mat_vec_iq3"
    return "lcpp_mul_mat_vec_q"


CASES = [
    # name, rows, k, packed
    ("IQ3_S", 272, 5120, True), ("IQ3_S", 64, 512, True), ("IQ3_S", 208, 4608, True), ("IQ3_S", 48, 17408, True),
    ("IQ3_S", 202, 1024, False), ("IQ3_S", 37, 5120, False),
    ("Q4_K", 202, 5120, False), ("Q4_K", 64, 512, False), ("Q4_K", 129, 4608, False), ("Q4_K", 40, 17408, False),
    ("IQ4_XS", 202, 5120, False), ("IQ4_XS", 33, 512, False), ("IQ4_XS", 40, 17408, False),
    ("Q6_K", 202, 5120, False), ("Q6_K", 19, 512, False), ("Q6_K", 24, 17408, False),
]


@pytest.fixture(params=["staged", "direct", "tensor"])
def load_variant(request):
    """The kernels behind the vec ops: the dp4a GEMV with either weight-streaming variant (bulk copies into a
    shared-memory ring, direct loads), and the library's own choice, which is the register-operand tensor-core
    kernel for Q4_K and packed IQ3_S."""
    old = _cabi.lib.gsq_debug_force_direct_loads(int(request.param == "direct"))
    old_mode = _cabi.lib.gsq_debug_mmv_mode(0 if request.param == "tensor" else 1)
    old_min = _cabi.lib.gsq_debug_mmv_min_rows(1)
    yield request.param
    _cabi.lib.gsq_debug_force_direct_loads(old)
    _cabi.lib.gsq_debug_mmv_mode(old_mode)
    _cabi.lib.gsq_debug_mmv_min_rows(old_min)


def test_no_bounded_wait_gave_up():
    import ctypes

    flag = ctypes.c_int(-1)
    assert _cabi.lib.gsq_device_error_flag(ctypes.byref(flag)) == 0
    assert flag.value == 0


@pytest.mark.parametrize("name,rows,k,packed", CASES)
@pytest.mark.parametrize("m", [1, 2, 3, 4, 5, 8])
def test_gemv_fp32_vs_oracle(name, rows, k, packed, m, load_variant):
    raw, w = _weights(name, rows, k, 1000 + rows, packed)
    x = _x(m, k, torch.float32, 1200 + m)
    y = getattr(torch.ops._C_gguf, _op_for(name, packed))(w, x.to(DEV), TYPES[name], rows)
    assert y.shape == (m, rows) and y.dtype == torch.float32
    dec = blocks.decode(raw, TYPES[name])
    q, d, _ = _oracle_q8(x)
    ref = product.product_q81(dec, q, d.astype(np.float32))
    err = product.rel_err(y.cpu().numpy(), ref)
    assert err <= 1e-5, err        # same integers, fp32 accumulation: far inside the 1e-3 budget


@pytest.mark.parametrize("name", list(TYPES))
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_gemv_16bit_and_full_precision(name, dtype):
    rows, k, m = 256, 5120, 4
    raw, w = _weights(name, rows, k, 31, packed=(name == "IQ3_S"))
    x = _x(m, k, dtype, 32, outliers=False)
    y = getattr(torch.ops._C_gguf, _op_for(name, name == "IQ3_S"))(w, x.to(DEV), TYPES[name], rows)
    assert y.dtype == dtype
    dec = blocks.decode(raw, TYPES[name])
    q, d, _ = _oracle_q8(x)
    ref = product.product_q81(dec, q, d.astype(np.float32))
    assert product.rel_err(_to_np(y), ref) <= TOL[dtype]
    full = product.product_full(raw, TYPES[name], _to_np(x))
    assert product.rel_err(_to_np(y), full) <= 1e-2 + TOL[dtype]


@pytest.mark.parametrize("name,rows,k,packed", [c for c in CASES if c[2] <= 5120])
def test_int32_slice_sums_bit_exact(name, rows, k, packed):
    m = 3
    raw, w = _weights(name, rows, k, 77, packed)
    x = _x(m, k, torch.float16, 78)
    xq = torch.ops._C_gguf.lcpp_quantize_q8_1(x.to(DEV), TYPES[name], False, False)
    g = 16 if name == "Q6_K" else 32
    sums = torch.zeros(m, rows, k // g, dtype=torch.int32, device=DEV)
    scratch = torch.empty(rows, dtype=torch.float32, device=DEV)
    rc = _cabi.lib.gsq_debug_block_sums(w.data_ptr(), w.shape[1], rows, TYPES[name], int(packed), xq.data_ptr(), m, k,
                                        sums.data_ptr(), scratch.data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    dec = blocks.decode(raw, TYPES[name])
    q, _, _ = _oracle_q8(x)
    want = product.block_sums(dec, q)
    assert np.array_equal(sums.cpu().numpy(), want)


def test_shared_x_q8_gives_identical_result():
    raw, w = _weights("Q4_K", 128, 1024, 5)
    x = _x(4, 1024, torch.bfloat16, 6).to(DEV)
    xq = torch.ops._C_gguf.lcpp_quantize_q8_1(x, Q4_K, False, False)
    a = torch.ops._C_gguf.lcpp_mul_mat_vec_q(w, x, Q4_K, 128)
    b = torch.ops._C_gguf.lcpp_mul_mat_vec_q(w, x, Q4_K, 128, xq)
    assert torch.equal(a, b)


def test_row_argument_limits_output():
    raw, w = _weights("IQ4_XS", 96, 1024, 9)
    x = _x(2, 1024, torch.float32, 10).to(DEV)
    full = torch.ops._C_gguf.lcpp_mul_mat_vec_q(w, x, IQ4_XS, 96)
    part = torch.ops._C_gguf.lcpp_mul_mat_vec_q(w, x, IQ4_XS, 50)
    assert part.shape == (2, 50) and torch.equal(part, full[:, :50])


@pytest.mark.parametrize("name", ["Q6_K", "IQ3_S"])
@pytest.mark.parametrize("m", [9, 16, 33])
def test_many_rows_ops_on_the_gemv(name, m):
    """Q6_K and IQ3_S in GGUF order have no tensor-core kernel: the many-row op names run the dp4a kernel
    8 rows at a time on block_q8_1 activations."""
    rows, k = 256, 1024
    raw, w = _weights(name, rows, k, 50, False)
    x = _x(m, k, torch.float32, 51)
    y = torch.ops._C_gguf.lcpp_mul_mat_q(w, x.to(DEV), TYPES[name], rows)
    dec = blocks.decode(raw, TYPES[name])
    q, d, _ = _oracle_q8(x)
    ref = product.product_q81(dec, q, d.astype(np.float32))
    assert product.rel_err(y.cpu().numpy(), ref) <= 1e-5


# ------------------------------------------------------------------------------------------ repack

def test_repack_on_gpu_matches_host_definition():
    raw = synth.make_weight(IQ3_S, 64, 5120, 3)
    w = torch.from_numpy(raw)
    host = iq3_pack.pack(w, IQ3_S)
    dev = iq3_pack.pack(w.to(DEV), IQ3_S)
    assert torch.equal(dev.cpu(), host)
    assert torch.equal(iq3_pack.unpack(dev, IQ3_S).cpu(), w)
    big = torch.from_numpy(synth.make_weight(IQ3_S, 32, 17408, 4)).to(DEV)
    assert torch.equal(iq3_pack.unpack(iq3_pack.pack(big, IQ3_S), IQ3_S), big)


def test_packed_and_unpacked_kernels_agree():
    raw, w = _weights("IQ3_S", 128, 5120, 12)
    wp = iq3_pack.pack(w, IQ3_S)
    x = _x(4, 5120, torch.float32, 13).to(DEV)
    a = torch.ops._C_gguf.lcpp_mul_mat_vec_iq3(w, x, IQ3_S, 128)
    b = torch.ops._C_gguf.lcpp_mul_mat_vec_iq3_mma_packed(wp, x, IQ3_S, 128)
    assert product.rel_err(b.cpu().numpy(), a.cpu().numpy().astype(np.float64)) <= 1e-5


# ------------------------------------------------------------------------------------------ graphs, apply()

def test_cuda_graph_replay_bit_equal_to_eager():
    raw, w = _weights("IQ3_S", 256, 5120, 20, packed=True)
    x = _x(4, 5120, torch.bfloat16, 21).to(DEV)
    eager = torch.ops._C_gguf.lcpp_mul_mat_vec_iq3_mma_packed(w, x, IQ3_S, 256)
    torch.cuda.synchronize()
    static_x = x.clone()
    g = torch.cuda.CUDAGraph()
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        torch.ops._C_gguf.lcpp_mul_mat_vec_iq3_mma_packed(w, static_x, IQ3_S, 256)
    torch.cuda.current_stream().wait_stream(s)
    with torch.cuda.graph(g):
        out = torch.ops._C_gguf.lcpp_mul_mat_vec_iq3_mma_packed(w, static_x, IQ3_S, 256)
    g.replay()
    torch.cuda.synchronize()
    assert torch.equal(out, eager)
    x2 = _x(4, 5120, torch.bfloat16, 22).to(DEV)
    static_x.copy_(x2)
    g.replay()
    torch.cuda.synchronize()
    assert torch.equal(out, torch.ops._C_gguf.lcpp_mul_mat_vec_iq3_mma_packed(w, x2, IQ3_S, 256))


def _fused_layer(shards, k):
    """shards: list of (shard id, type name, rows). Returns (layer, method, raw dict)."""
    layer = torch.nn.Module()
    method = linear.GGUFLinearMethod(None)
    method.create_weights(layer, k, [r for _, _, r in shards], k, sum(r for _, _, r in shards), torch.bfloat16)
    raws = {}
    for i, (sid, name, rows) in enumerate(shards):
        raws[sid] = synth.make_weight(TYPES[name], rows, k, 900 + i)
        layer.weight.load_shard(torch.from_numpy(raws[sid]).to(DEV), sid)
        layer.weight_type.shard_weight_type[sid] = TYPES[name]
    layer.weight_type.weight_type = TYPES[shards[0][1]]
    method.process_weights_after_loading(layer)
    return layer, method, raws


@pytest.mark.parametrize("m", [1, 4, 8, 12])
def test_apply_mixed_type_fused_layer(m):
    k = 1024
    shards = [("q", "IQ3_S", 128), ("k", "Q4_K", 64), ("v", "Q4_K", 64)]
    layer, method, raws = _fused_layer(shards, k)
    assert layer.weight.iq3_packed and layer.weight.shape[0] == 256
    x = _x(m, k, torch.bfloat16, 40 + m)
    bias = torch.randn(256, dtype=torch.bfloat16, device=DEV)
    y = method.apply(layer, x.to(DEV), bias.clone())
    assert y.shape == (m, 256) and y.dtype == torch.bfloat16
    q, d, _ = _oracle_q8(x)
    refs = []
    for sid, name, rows in shards:
        dec = blocks.decode(raws[sid], TYPES[name])
        refs.append(product.product_q81(dec, q, d.astype(np.float32)))
    ref = np.concatenate(refs, axis=1) + bias.float().cpu().numpy()
    assert product.rel_err(_to_np(y), ref) <= 5e-3


def test_zz_no_bounded_wait_gave_up_after_all_tests():
    test_no_bounded_wait_gave_up()


def test_apply_single_type_and_unfused():
    k = 512
    layer, method, raws = _fused_layer([(0, "IQ3_S", 64), (1, "IQ3_S", 96)], k)
    x = _x(2, k, torch.float16, 60)
    y = method.apply(layer, x.to(DEV))
    q, d, _ = _oracle_q8(x)
    ref = np.concatenate([product.product_q81(blocks.decode(raws[i], IQ3_S), q, d.astype(np.float32)) for i in (0, 1)], axis=1)
    assert product.rel_err(_to_np(y), ref) <= 1e-3
    layer2 = torch.nn.Module()
    m2 = linear.GGUFLinearMethod(None)
    m2.create_weights(layer2, k, [80], k, 80, torch.float16)
    raw = synth.make_weight(IQ4_XS, 80, k, 61)
    layer2.weight.load_shard(torch.from_numpy(raw).to(DEV))
    layer2.weight_type.weight_type = IQ4_XS
    m2.process_weights_after_loading(layer2)
    y2 = m2.apply(layer2, x.to(DEV))
    ref2 = product.product_q81(blocks.decode(raw, IQ4_XS), q, d.astype(np.float32))
    assert product.rel_err(_to_np(y2), ref2) <= 1e-3


@pytest.mark.parametrize("name,packed", [("Q4_K", False), ("IQ3_S", True), ("IQ4_XS", False)])
@pytest.mark.parametrize("rows,k", [(2176, 5120), (640, 5120), (5120, 2048), (5120, 2304), (5120, 4352)])
def test_tensor_parallel_shard_shapes(name, packed, rows, k):
    """The shard shapes of 4- and 8-way tensor parallelism of the benchmark's layers (row shards of 17408 / 5120 rows,
    K shards of 8, 9 and 17 superblocks): the library's own choice of kernel against the other kernel behind the same
    op (dp4a GEMV, tcgen05 GEMM), at 1, 8 and 32 activation rows."""
    from gsq_b200 import lcpp_ops

    old_k = lcpp_ops.set_k_multiple(256)
    try:
        raw, w = _weights(name, rows, k, 900 + rows % 97 + k % 89, packed)
        many = {"Q4_K": "lcpp_mul_mat_q", "IQ4_XS": "lcpp_mul_mat_q", "IQ3_S": "lcpp_mul_mat_iq3_packed"}[name]
        for m in (1, 8, 32):
            x = _x(m, k, torch.float32, 950 + m).to(DEV)
            op = _op_for(name, packed) if m <= 8 else many
            y = getattr(torch.ops._C_gguf, op)(w, x, TYPES[name], rows)
            old = _cabi.lib.gsq_debug_mmv_mode(1)
            try:
                ref = getattr(torch.ops._C_gguf, op)(w, x, TYPES[name], rows)   # dp4a GEMV / tcgen05 GEMM
            finally:
                _cabi.lib.gsq_debug_mmv_mode(old)
            err = product.rel_err(y.cpu().numpy(), ref.double().cpu().numpy())
            assert err <= 1e-3, (name, rows, k, m, err)
    finally:
        lcpp_ops.set_k_multiple(old_k)


@pytest.mark.parametrize("m", [1, 3, 8, 24])
def test_chained_launches_do_not_depend_on_overlap(m):
    """Back-to-back products in one stream (quantiser -> product -> quantiser -> ..., each launched as a programmatic
    dependent of the one before, the products letting the next kernels start before they have finished): every
    result, the ones feeding the next product included, is bit-equal to the chain run with that overlap switched off."""
    k = 5120
    ws = []
    for name, packed, rows in (("IQ3_S", True, 5120), ("Q4_K", False, 5120), ("IQ4_XS", False, 5120), ("IQ3_S", True, 5120),
                               ("Q6_K", False, 5120)):
        ws.append((name, packed, rows, _weights(name, rows, k, 1300 + len(ws), packed)[1]))
    # fp32 results, and a start small enough that the fp16 block scales and block sums of the fifth quantisation still
    # fit: the synthetic weights gain 20x to 1000x per product, 1e7 over the first four (largest gain last)
    x0 = (_x(m, k, torch.float32, 1310 + m) * 3e-5).to(DEV)

    def chain():
        outs, x = [], x0
        for name, packed, rows, w in ws:
            op = linear._lcpp_op(m, TYPES[name], rows, k, packed)
            y = getattr(torch.ops._C_gguf, op)(w, x, TYPES[name], rows)
            outs.append(y)
            x = y  # the next product quantises this result (5120 -> 5120), with no other kernel in between
        torch.cuda.synchronize()
        return [o.clone() for o in outs]

    results = {}
    for mode in (0, 1, 2, 3):
        old = _cabi.lib.gsq_debug_mmv_pdl(mode)
        try:
            results[mode] = chain()
            results[(mode, "again")] = chain()
        finally:
            _cabi.lib.gsq_debug_mmv_pdl(old)
    for key, outs in results.items():
        for i, (a, b) in enumerate(zip(outs, results[0])):
            assert torch.isfinite(a).all()
            assert torch.equal(a, b), (key, i, ws[i][0])


@pytest.mark.parametrize("k", [2304, 4352])
@pytest.mark.parametrize("mmq", [False, True])
def test_quantize_op_on_tensor_parallel_k_shards(k, mmq):
    """The stand-alone quantise op follows the same relaxed K granularity as the products (K shards of 9 and 17
    superblocks are multiples of 256, not of 512) and its bytes feed a product to the same result."""
    from gsq_b200 import lcpp_ops

    x = _x(5, k, torch.float16, 1400 + k).to(DEV)
    with pytest.raises(RuntimeError, match="bad arguments"):
        torch.ops._C_gguf.lcpp_quantize_q8_1(x, Q4_K, mmq, False)
    old_k = lcpp_ops.set_k_multiple(256)
    try:
        xq = torch.ops._C_gguf.lcpp_quantize_q8_1(x, Q4_K, mmq, False)
        assert xq.numel() == (5 * k // 128 * 144 if mmq else 5 * k // 32 * 36)
        if not mmq:
            g, w = xq.cpu().numpy().reshape(-1, 36), q8_1.q8_1_bytes(_to_np(x)).reshape(-1, 36)
            assert np.array_equal(g[:, 2:], w[:, 2:])   # half(sum x) and the quants; d may differ by one fp16 step
            raw, w = _weights("Q4_K", 640, k, 1410, False)
            y0 = torch.ops._C_gguf.lcpp_mul_mat_vec_q(w, x, Q4_K, 640)
            y1 = torch.ops._C_gguf.lcpp_mul_mat_vec_q(w, x, Q4_K, 640, xq)
            assert torch.equal(y0, y1)
    finally:
        lcpp_ops.set_k_multiple(old_k)
