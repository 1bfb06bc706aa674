"""Row gather + dequantisation (the quantised embedding look-up, gsq_dequantize_rows) for the ten types of the model
file: bit for bit against the oracles' fp32 dequantisation (themselves bit-exact on the reference's 84 real-row
fixtures), fp16 / bf16 outputs equal to that value rounded once, repeated and out-of-range indices."""

import ctypes

import numpy as np
import pytest
import torch

import gsq_b200  # noqa: F401
from gsq_b200 import _cabi, synth
from gsq_b200.quantization import vocab_embeds
from oracle import blocks, blocks_f1

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
ALL = {**synth.TYPE_IDS, **synth.LOW_BIT_TYPE_IDS}


def _oracle(raw, t):
    return blocks.dequantize(raw, t) if t in blocks.BLOCK_BYTES else blocks_f1.dequantize(raw, t)


@pytest.mark.parametrize("name", list(ALL))
def test_gather_bit_exact_fp32(name):
    t = ALL[name]
    vocab, k = 300, 5120
    raw = synth.make_weight(t, vocab, k, 40 + t)
    ids = torch.tensor([[0, 299, 7, 7], [150, 3, 298, 0]])
    y = vocab_embeds.apply_gguf_embedding(ids.to(DEV), torch.from_numpy(raw).to(DEV), t, k, torch.float32)
    assert y.shape == (2, 4, k) and y.dtype == torch.float32
    want = _oracle(raw, t)[ids.reshape(-1).numpy()].reshape(2, 4, k)
    assert np.array_equal(y.cpu().numpy().view(np.uint32), want.view(np.uint32))


@pytest.mark.parametrize("name", list(ALL))
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_whole_tensor_16bit_is_the_fp32_value_rounded_once(name, dtype):
    t = ALL[name]
    raw = synth.make_weight(t, 33, 1024, 50 + t)
    y = vocab_embeds.dequantize(torch.from_numpy(raw).to(DEV), t, dtype)
    want = torch.from_numpy(_oracle(raw, t)).to(dtype)
    assert torch.equal(y.cpu(), want)


def test_index_outside_the_table_is_flagged_and_reads_nothing():
    t = ALL["Q6_K"]
    raw = synth.make_weight(t, 16, 512, 9)
    ids = torch.tensor([3, 16, -1, 15], device=DEV)
    y = vocab_embeds.apply_gguf_embedding(ids, torch.from_numpy(raw).to(DEV), t, 512, torch.float32)
    torch.cuda.synchronize()
    flag = ctypes.c_int(0)
    assert _cabi.lib.gsq_dequantize_bad_index_flag(ctypes.byref(flag)) == 0 and flag.value == 1
    want = blocks.dequantize(raw, t)
    assert np.array_equal(y[0].cpu().numpy(), want[3]) and np.array_equal(y[3].cpu().numpy(), want[15])
    assert not y[1].any() and not y[2].any()
