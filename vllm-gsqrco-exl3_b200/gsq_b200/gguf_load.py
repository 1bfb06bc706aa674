"""GGUF file -> GPU weights of this package's linear method, repacked on the GPU.

The reference copies each tensor from the host into the layer's parameter (plugin/vllm_gguf_plugin/quantization/
params.py:75-99, through vLLM's weight loaders) and repacks the IQ3 runs afterwards with torch ops
(quantization/linear.py:425-457). Here the file is memory-mapped (gguf.GGUFReader), each tensor goes to the device
through one reused pinned staging buffer in chunks (so the host never holds a second copy of a large tensor and the
host-side fill of chunk i + 1 overlaps the transfer of chunk i), is placed into the layer's padded multi-shard buffer
on the device, and the IQ3_S / Q6_K runs are repacked in place by the CUDA repack kernels
(process_weights_after_loading -> gsq_iq3s_repack / gsq_q6k_repack). `unpack` still returns GGUF bytes for a consumer
that needs them.

Only what the linear path needs is here: tensor enumeration and fused-layer construction. Model architecture,
tokenizer and config handling of the reference's loader are not.
"""

from __future__ import annotations

import numpy as np
import torch

from . import ops
from .quantization import linear

_CHUNK = 64 << 20
_COPY_THREADS = 8
_pool = None


def _parallel_copy(dst: np.ndarray, src: np.ndarray) -> None:
    """dst[...] = src for row matrices, the rows split over a few threads: one thread copying out of the page cache
    reaches a fraction of what the staging buffer's transfer to the device can take (numpy's copy releases the GIL)."""
    global _pool
    rows = src.shape[0]
    if src.nbytes < (8 << 20) or rows < 2 * _COPY_THREADS:
        dst[...] = src
        return
    if _pool is None:
        from concurrent.futures import ThreadPoolExecutor

        _pool = ThreadPoolExecutor(max_workers=_COPY_THREADS, thread_name_prefix="gguf-stage")
    step = -(-rows // _COPY_THREADS)
    for f in [_pool.submit(np.copyto, dst[i:i + step], src[i:i + step]) for i in range(0, rows, step)]:
        f.result()


def tensors(path: str):
    """{name: (ggml type id, uint8 [rows, row_bytes] memory-mapped view)} of the quantised 2-D tensors of the file whose
    type this package serves, plus F32 / F16 / BF16 ones as (type id, array)."""
    import gguf

    out = {}
    for t in gguf.GGUFReader(path).tensors:
        tid = int(t.tensor_type)
        if tid in ops.LCPP_QUANT_TYPES:
            data = np.asarray(t.data)
            out[t.name] = (tid, data.reshape(data.shape[0], -1).view(np.uint8) if data.ndim == 2 else data.view(np.uint8))
        elif tid in ops.UNQUANTIZED_TYPES:
            out[t.name] = (tid, np.asarray(t.data))
    return out


class _Stager:
    """One pinned buffer, two halves used in turn: the copy of a chunk overlaps the placement of the one before."""

    def __init__(self, device):
        self.dev = torch.device(device)
        self.pin = torch.empty(2 * _CHUNK, dtype=torch.uint8).pin_memory()
        self.events = [torch.cuda.Event(), torch.cuda.Event()]
        self.turn = 0
        self.bytes = 0

    def to_device(self, src: np.ndarray, dst: torch.Tensor) -> None:
        """src: contiguous uint8 rows [r, row_bytes] on the host (memory-mapped); dst: [r, >= row_bytes] device view."""
        r, rb = src.shape
        per = max(1, _CHUNK // rb)
        for i in range(0, r, per):
            c = min(per, r - i)
            h = self.turn
            self.turn ^= 1
            self.events[h].synchronize()                       # the previous use of this half has been copied out
            stage = self.pin[h * _CHUNK: h * _CHUNK + c * rb].view(c, rb)
            _parallel_copy(stage.numpy(), src[i:i + c])
            dst[i:i + c, :rb].copy_(stage, non_blocking=True)
            self.events[h].record()
            self.bytes += c * rb


def load_linear(path_or_tensors, names: list[str], device="cuda:0", params_dtype=torch.bfloat16, stager: _Stager | None = None):
    """A fused linear layer from the named tensors of a GGUF file (one shard each, in this order: q/k/v, gate/up, or a
    single tensor): -> (layer, method) ready for method.apply(layer, x). All tensors must share K."""
    tens = tensors(path_or_tensors) if isinstance(path_or_tensors, str) else path_or_tensors
    metas = [tens[n] for n in names]
    bad = [n for n, (tid, _) in zip(names, metas) if tid not in ops.LCPP_QUANT_TYPES]
    if bad:
        raise ValueError(f"load_linear: {bad[0]} is not a quantised tensor of a served type")
    ks = {m[1].shape[1] // ops.GGML_QUANT_SIZES[m[0]][1] * ops.GGML_QUANT_SIZES[m[0]][0] for m in metas}
    if len(ks) != 1:
        raise ValueError(f"load_linear: tensors with different K: {sorted(ks)}")
    k = ks.pop()
    rows = [m[1].shape[0] for m in metas]
    stager = stager or _Stager(device)
    layer = torch.nn.Module()
    method = linear.GGUFLinearMethod(None)
    with torch.cuda.device(device):
        method.create_weights(layer, k, rows, k, sum(rows), params_dtype)
        fused = len(names) > 1
        for sid, (tid, data) in enumerate(metas):
            dev_rows = torch.empty(data.shape, dtype=torch.uint8, device=device)
            stager.to_device(data, dev_rows)
            layer.weight.load_shard(dev_rows, sid if fused else None)
            if fused:
                layer.weight_type.shard_weight_type[sid] = tid
        layer.weight_type.weight_type = metas[0][0]
        method.process_weights_after_loading(layer)          # pads, places, repacks IQ3_S / Q6_K runs on the GPU
        torch.cuda.synchronize()
    return layer, method
