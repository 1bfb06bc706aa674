"""Q6_K repacked at load (a byte permutation per 16-row tile, quantization/iq3_pack.py) and served by the
register-operand tensor-core kernel at every row count: against the CPU oracle (int32 sums of every 16-value group
bit exact, fp32 outputs <= 1e-5 / 1e-3) and, through apply(), against the GGUF-order dp4a path."""

import ctypes

import numpy as np
import pytest
import torch

import gsq_b200  # noqa: F401
from gsq_b200 import _cabi, synth
from gsq_b200.quantization import iq3_pack, linear
from oracle import blocks, product, q8_1

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
Q6_K = 14


def _x(m, k, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(m, k, generator=g)
    x[:, torch.randperm(k, generator=g)[: max(1, k // 256)]] *= 20
    return synth.nudge_ties_torch(x.to(dtype))


def _ref(raw, x):
    q, d, _ = q8_1.quantize_q8_1(x.float().numpy())
    return product.product_q81(blocks.decode(raw, Q6_K), q, d.astype(np.float32)), q


def test_gpu_repack_matches_host_definition():
    raw = torch.from_numpy(synth.make_weight(Q6_K, 64, 5120, 3))
    host = iq3_pack.pack(raw, Q6_K)
    dev = iq3_pack.pack(raw.to(DEV), Q6_K)
    assert torch.equal(dev.cpu(), host)
    assert torch.equal(iq3_pack.unpack(dev, Q6_K).cpu(), raw)
    big = torch.from_numpy(synth.make_weight(Q6_K, 32, 17408, 4)).to(DEV)
    assert torch.equal(iq3_pack.unpack(iq3_pack.pack(big, Q6_K), Q6_K), big)


@pytest.mark.parametrize("rows,k", [(272, 5120), (64, 512), (208, 4608), (48, 17408)])
@pytest.mark.parametrize("m", [1, 2, 5, 8])
def test_vec_op_fp32_vs_oracle(rows, k, m):
    raw = synth.make_weight(Q6_K, rows, k, 100 + rows)
    w = iq3_pack.pack(torch.from_numpy(raw).to(DEV), Q6_K)
    x = _x(m, k, torch.float32, 110 + m)
    y = torch.ops._C_gguf.gsq_mul_mat_vec_q6k_packed(w, x.to(DEV), Q6_K, rows)
    ref, _ = _ref(raw, x)
    assert product.rel_err(y.cpu().numpy(), ref) <= 1e-5


@pytest.mark.parametrize("m", [9, 16, 24, 33, 48, 70, 130])
@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-3), (torch.bfloat16, 5e-3)])
def test_many_rows_op_vs_oracle(m, dtype, tol):
    rows, k = 272, 5120
    raw = synth.make_weight(Q6_K, rows, k, 120)
    w = iq3_pack.pack(torch.from_numpy(raw).to(DEV), Q6_K)
    x = _x(m, k, dtype, 130 + m)
    y = torch.ops._C_gguf.gsq_mul_mat_q6k_packed(w, x.to(DEV), Q6_K, rows)
    assert y.dtype == dtype and y.shape == (m, rows)
    ref, _ = _ref(raw, x)
    assert product.rel_err(y.float().cpu().numpy(), ref) <= tol


@pytest.mark.parametrize("m", [3, 20])
def test_group_sums_bit_exact(m):
    rows, k = 144, 1024
    raw = synth.make_weight(Q6_K, rows, k, 140)
    w = iq3_pack.pack(torch.from_numpy(raw).to(DEV), Q6_K)
    x = _x(m, k, torch.float16, 141 + m)
    sums = torch.full((m, rows, k // 16), 0x7FFFFFFF, dtype=torch.int32, device=DEV)
    _cabi.lib.gsq_debug_gemm_dump_sums(ctypes.c_void_p(sums.data_ptr()))
    try:
        torch.ops._C_gguf.gsq_mul_mat_q6k_packed(w, x.to(DEV), Q6_K, rows)
        torch.cuda.synchronize()
    finally:
        _cabi.lib.gsq_debug_gemm_dump_sums(None)
    q, _, _ = q8_1.quantize_mmq(x.float().numpy(), q8_1.LAYOUT_D4)
    want = product.block_sums(blocks.decode(raw, Q6_K), q)
    assert np.array_equal(sums.cpu().numpy(), want)


@pytest.mark.parametrize("m", [1, 8, 12, 60])
def test_apply_repacks_q6k_and_matches_gguf_order_path(m):
    k, rows = 1024, 256
    raw = synth.make_weight(Q6_K, rows, k, 150)

    def layer_with(pack):
        layer = torch.nn.Module()
        method = linear.GGUFLinearMethod(None)
        method.pack_iq3 = pack
        method.create_weights(layer, k, [rows], k, rows, torch.float16)
        layer.weight.load_shard(torch.from_numpy(raw).to(DEV))
        layer.weight_type.weight_type = Q6_K
        method.process_weights_after_loading(layer)
        return layer, method
    la, ma = layer_with(True)
    lb, mb = layer_with(False)
    assert la.weight.iq3_packed and not getattr(lb.weight, "iq3_packed", False)
    x = _x(m, k, torch.float16, 151 + m).to(DEV)
    ya, yb = ma.apply(la, x), mb.apply(lb, x)
    assert product.rel_err(ya.float().cpu().numpy(), yb.double().cpu().numpy()) <= 2e-3
    ref, _ = _ref(raw, x.cpu())
    assert product.rel_err(ya.float().cpu().numpy(), ref) <= 2e-3
