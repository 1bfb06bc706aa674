"""GPU parity of the low-bit types a model file mixes with the four main ones (Q2_K, IQ2_XXS, IQ2_XS, IQ2_S, IQ3_XXS,
IQ1_M; dp4a kernel on GGUF-order blocks): integer group sums bit exact against the integer oracle, fp32 results against
the float64 model of the reference's MMVQ arithmetic (truncating integer divisions included; oracle/blocks_f1.py),
against dequantise-and-multiply, through the routed torch ops at every row count, and -- when oracle/_ref is built --
against the reference's own CUDA kernels on the same bytes (<= 1e-3 of the row norm, tests/gpu/_refs.py:94-99)."""

import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import gsq_b200  # noqa: F401
from gsq_b200 import _cabi, synth
from gsq_b200.quantization import linear
from oracle import blocks_f1, product, q8_1

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF_SO = os.path.join(ROOT, "oracle", "_ref", "ref_C_gguf.so")
DEV = "cuda:0"
TYPES = blocks_f1.TYPE_IDS


def _x(m, k, dtype, seed):
    return synth.nudge_ties_torch(torch.from_numpy(synth.make_activation(m, k, seed)).to(dtype))


def _model(raw, t, x):
    q, d, _ = q8_1.quantize_q8_1(x.float().numpy())
    return blocks_f1.product_q81(blocks_f1.decode(raw, t), q, d.astype(np.float32)), q


@pytest.mark.parametrize("name", list(TYPES))
@pytest.mark.parametrize("rows,k", [(64, 512), (203, 5120), (48, 17408)])
@pytest.mark.parametrize("m", [1, 3, 8])
def test_vec_fp32_vs_model(name, rows, k, m):
    t = TYPES[name]
    raw = synth.make_weight(t, rows, k, 500 + t)
    x = _x(m, k, torch.float32, 600 + m)
    y = torch.ops._C_gguf.lcpp_mul_mat_vec_q(torch.from_numpy(raw).to(DEV), x.to(DEV), t, rows)
    assert y.shape == (m, rows) and y.dtype == torch.float32
    ref, _ = _model(raw, t, x)
    assert product.rel_err(y.cpu().numpy(), ref) <= 1e-5
    assert product.rel_err(y.cpu().numpy(), blocks_f1.product_full(raw, t, x.numpy())) <= 3e-2


@pytest.mark.parametrize("name", list(TYPES))
def test_integer_group_sums_bit_exact(name):
    t = TYPES[name]
    rows, k, m = 70, 1024, 3
    raw = synth.make_weight(t, rows, k, 700 + t)
    x = _x(m, k, torch.float16, 701).to(DEV)
    w = torch.from_numpy(raw).to(DEV)
    xq = torch.ops._C_gguf.lcpp_quantize_q8_1(x, t, False, False)
    dec = blocks_f1.decode(raw, t)
    sums = torch.zeros(m, rows, k // dec.g, dtype=torch.int32, device=DEV)
    scratch = torch.empty(rows, dtype=torch.float32, device=DEV)
    rc = _cabi.lib.gsq_debug_block_sums(w.data_ptr(), w.shape[1], rows, t, 0, xq.data_ptr(), m, k, sums.data_ptr(),
                                        scratch.data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    q, _, _ = q8_1.quantize_q8_1(x.float().cpu().numpy())
    assert np.array_equal(sums.cpu().numpy(), blocks_f1.group_sums(dec, q))


@pytest.mark.parametrize("name", list(TYPES))
@pytest.mark.parametrize("m,dtype,tol", [(1, torch.float16, 1e-3), (8, torch.bfloat16, 5e-3), (20, torch.float16, 1e-3),
                                         (70, torch.bfloat16, 5e-3)])
def test_routed_through_the_linear_method(name, m, dtype, tol):
    """Every row count through the reference's routing table (vec ops up to 8 rows, the self-quantising ops above:
    here both end in the dp4a kernel, eight rows per launch)."""
    t = TYPES[name]
    rows, k = 144, 5120
    raw = synth.make_weight(t, rows, k, 800 + t)
    x = _x(m, k, dtype, 801 + m)
    if name == "IQ1_M" and m > 32:   # the routing table has no op for IQ1_M above 32 rows (no MMQ for this type)
        with pytest.raises(NotImplementedError):
            linear.fused_mul_mat_gguf(x.to(DEV), torch.from_numpy(raw).to(DEV), t, None, False)
        return
    y = linear.fused_mul_mat_gguf(x.to(DEV), torch.from_numpy(raw).to(DEV), t, None, False)
    assert y.shape == (m, rows) and y.dtype == dtype
    ref, _ = _model(raw, t, x)
    assert product.rel_err(y.float().cpu().numpy(), ref) <= tol


@pytest.mark.parametrize("name", list(TYPES))
def test_against_reference_kernels(name, tmp_path):
    if not os.path.exists(REF_SO):
        pytest.skip("oracle/_ref/ref_C_gguf.so not built")
    t = TYPES[name]
    rows, k = 512, 5120
    raw = torch.from_numpy(synth.make_weight(t, rows, k, 900 + t))
    cases, mine = [], []
    for m in (1, 8):
        x = _x(m, k, torch.float32, 901 + m)
        cases.append({"op": "lcpp_mul_mat_vec_q", "args": [raw, x, t, rows, None]})
        mine.append(torch.ops._C_gguf.lcpp_mul_mat_vec_q(raw.to(DEV), x.to(DEV), t, rows).cpu())
    cin, cout = str(tmp_path / "cases.pt"), str(tmp_path / "results.pt")
    torch.save(cases, cin)
    p = subprocess.run([sys.executable, os.path.join(ROOT, "oracle", "ref_runner.py"), cin, cout], capture_output=True, text=True,
                       timeout=600)
    assert p.returncode == 0, p.stderr[-3000:]
    res = torch.load(cout)
    for y, r in zip(mine, res):
        assert product.rel_err(y.numpy(), r["out"].double().numpy()) <= 1e-3


@pytest.mark.parametrize("m", [1, 8, 20])
def test_apply_fused_layer_mixing_main_and_low_bit_types(m):
    """A fused layer as the model file has them: a repacked IQ3_S run beside IQ3_XXS (which stays in GGUF order here,
    though the layer carries the packed flag), IQ2_XS and Q2_K runs, through GGUFLinearMethod.apply()."""
    from oracle import blocks

    k = 1024
    main = {"IQ3_S": 21}
    shards = [("a", "IQ3_S", 128), ("b", "IQ3_XXS", 64), ("c", "IQ2_XS", 64), ("d", "Q2_K", 48)]
    layer = torch.nn.Module()
    method = linear.GGUFLinearMethod(None)
    method.create_weights(layer, k, [r for _, _, r in shards], k, sum(r for _, _, r in shards), torch.float16)
    raws = {}
    for i, (sid, name, rows) in enumerate(shards):
        t = main.get(name) or TYPES[name]
        raws[sid] = synth.make_weight(t, rows, k, 950 + i)
        layer.weight.load_shard(torch.from_numpy(raws[sid]).to(DEV), sid)
        layer.weight_type.shard_weight_type[sid] = t
    layer.weight_type.weight_type = 21
    method.process_weights_after_loading(layer)
    assert layer.weight.iq3_packed
    x = _x(m, k, torch.float16, 960 + m)
    y = method.apply(layer, x.to(DEV))
    q, d, _ = q8_1.quantize_q8_1(x.float().numpy())
    refs = []
    for sid, name, rows in shards:
        if name in main:
            refs.append(product.product_q81(blocks.decode(raws[sid], main[name]), q, d.astype(np.float32)))
        else:
            refs.append(blocks_f1.product_q81(blocks_f1.decode(raws[sid], TYPES[name]), q, d.astype(np.float32)))
    ref = np.concatenate(refs, axis=1)
    assert y.shape == ref.shape
    assert product.rel_err(y.float().cpu().numpy(), ref) <= 2e-3
