"""GGUF file -> tensors -> fused linear layer on the GPU (gsq_b200.gguf_load): a synthetic file written with gguf-py
(as the reference's kit/synth.py:91-108 does), read back byte for byte on the CPU; on the GPU, loaded, repacked and
multiplied against the oracle."""

import numpy as np
import pytest
import torch

from gsq_b200 import synth

K = 1024
TENSORS = [("blk.0.attn_q.weight", "IQ3_S", 256), ("blk.0.attn_k.weight", "Q4_K", 128), ("blk.0.attn_v.weight", "IQ2_XS", 64),
           ("output.weight", "Q6_K", 128)]
ALL = {**synth.TYPE_IDS, **synth.LOW_BIT_TYPE_IDS}


@pytest.fixture(scope="module")
def gguf_file(tmp_path_factory):
    gguf = pytest.importorskip("gguf")
    path = str(tmp_path_factory.mktemp("gguf") / "synthetic.gguf")
    w = gguf.GGUFWriter(path, "gsq-synthetic")
    raws = {}
    for i, (name, tname, rows) in enumerate(TENSORS):
        raws[name] = synth.make_weight(ALL[tname], rows, K, 600 + i)
        w.add_tensor(name, raws[name], raw_dtype=gguf.GGMLQuantizationType(ALL[tname]))
    w.add_tensor("norm.weight", np.ones(K, dtype=np.float32))
    w.write_header_to_file()
    w.write_kv_data_to_file()
    w.write_tensors_to_file()
    w.close()
    return path, raws


def test_tensors_round_trip(gguf_file):
    from gsq_b200 import gguf_load

    path, raws = gguf_file
    got = gguf_load.tensors(path)
    for name, tname, rows in TENSORS:
        tid, data = got[name]
        assert tid == ALL[tname] and data.dtype == np.uint8 and data.shape == raws[name].shape
        assert np.array_equal(data, raws[name])
    assert got["norm.weight"][0] == 0


@pytest.mark.gpu
@pytest.mark.parametrize("m", [1, 8, 20])
def test_load_fused_layer_and_apply(gguf_file, m):
    from gsq_b200 import gguf_load
    from oracle import blocks, blocks_f1, product, q8_1

    path, raws = gguf_file
    names = [n for n, _, _ in TENSORS[:3]]
    layer, method = gguf_load.load_linear(path, names, "cuda:0", torch.float16)
    assert layer.weight.iq3_packed and layer.weight.shape[0] == 448
    x = synth.nudge_ties_torch(torch.from_numpy(synth.make_activation(m, K, 610 + m)).half())
    y = method.apply(layer, x.to("cuda:0"))
    q, d, _ = q8_1.quantize_q8_1(x.float().numpy())
    refs = []
    for name, tname, rows in TENSORS[:3]:
        t = ALL[tname]
        if t in blocks.BLOCK_BYTES:
            refs.append(product.product_q81(blocks.decode(raws[name], t), q, d.astype(np.float32)))
        else:
            refs.append(blocks_f1.product_q81(blocks_f1.decode(raws[name], t), q, d.astype(np.float32)))
    assert product.rel_err(y.float().cpu().numpy(), np.concatenate(refs, axis=1)) <= 2e-3
    # a single repacked tensor, and its GGUF bytes back
    from gsq_b200.quantization import iq3_pack

    head, hm = gguf_load.load_linear(path, ["output.weight"], "cuda:0", torch.float16)
    yh = hm.apply(head, x.to("cuda:0"))
    ref = product.product_q81(blocks.decode(raws["output.weight"], 14), q, d.astype(np.float32))
    assert product.rel_err(yh.float().cpu().numpy(), ref) <= 2e-3
    back = iq3_pack.unpack(head.weight.data, 14) if head.weight.iq3_packed else head.weight.data
    assert np.array_equal(back.cpu().numpy(), raws["output.weight"])


def test_parallel_staging_copy():
    """The loader's host-side copy into its staging buffer: rows split over threads, byte for byte; small matrices
    take the plain copy."""
    from gsq_b200 import gguf_load

    rng = np.random.default_rng(5)
    for rows, rb in ((7, 110), (1000, 2200), (17408, 2200), (4099, 3997)):
        src = rng.integers(0, 256, size=(rows, rb), dtype=np.uint8)
        dst = np.zeros_like(src)
        gguf_load._parallel_copy(dst, src)
        assert np.array_equal(dst, src)
    big = rng.integers(0, 256, size=(20000, 1100), dtype=np.uint8)
    view = np.zeros((20000, 1100), dtype=np.uint8)
    gguf_load._parallel_copy(view, big[:, :1100])
    assert np.array_equal(view, big)
