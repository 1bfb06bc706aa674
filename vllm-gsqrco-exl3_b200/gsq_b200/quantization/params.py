"""Weight containers the linear method reads.

Only the attributes `GGUFLinearMethod` touches are modelled (the reference's
quantization/params.py:228-301, 353-416 also carries vLLM's loader plumbing, which stays with
vLLM): `weight.data` uint8 [rows, row_bytes]; `weight.shard_id` (ordered list), `weight.shard_id_map`,
`weight.data_container` (shards as loaded), `weight.shard_offset_map` {id: (start_row, end_row,
row_bytes)}, `weight.iq3_packed`; `weight_type.weight_type` (int) and `.shard_weight_type` {id: int}.
"""

from __future__ import annotations

import torch

_QKV_ORDER = ("q", "k", "v")


def _gguf_ordered_shard_ids(shard_id: list) -> list:
    """q, k, v in that order whatever order they were loaded in; numeric ids ascending."""
    if any(s in _QKV_ORDER for s in shard_id):
        return [s for s in _QKV_ORDER if s in shard_id]
    return sorted(shard_id)


class GGUFWeightParameter(torch.nn.Parameter):
    """uint8 GGUF block bytes plus the shard bookkeeping of a (possibly fused) linear layer."""

    def __new__(cls, data: torch.Tensor | None = None, **_):
        if data is None:
            data = torch.empty(0, dtype=torch.uint8)
        return torch.Tensor._make_subclass(cls, data, False)

    def __init__(self, data: torch.Tensor | None = None, **attrs):
        self.data_container: list[torch.Tensor] = []
        self.shard_id: list = []
        self.shard_id_map: dict = {}
        for k, v in attrs.items():
            setattr(self, k, v)

    def load_shard(self, loaded: torch.Tensor, shard_id=None) -> None:
        """Append one shard's bytes (uint8 [rows, row_bytes]); a layer without shards passes None."""
        assert loaded.dtype == torch.uint8 and loaded.dim() == 2
        if shard_id is None:
            self.data = loaded
            return
        self.shard_id_map[shard_id] = len(self.data_container)
        self.shard_id.append(shard_id)
        self.data_container.append(loaded)


class GGUFWeightTypeParameter(torch.nn.Parameter):
    """Scalar holder of the layer's ggml type id(s)."""

    def __new__(cls, weight_type: int = 0, **_):
        return torch.Tensor._make_subclass(cls, torch.empty(0, dtype=torch.uint8), False)

    def __init__(self, weight_type: int = 0, shard_weight_type: dict | None = None):
        self.weight_type = int(weight_type)
        self.shard_weight_type = dict(shard_weight_type or {})
