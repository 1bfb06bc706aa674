"""GGUF linear method on B200: the host side of the quantised-linear path.

Mirrors the public surface of the reference's plugin/vllm_gguf_plugin/quantization/linear.py -- the
same names, argument meaning and error behaviour -- so it can stand in for that module:

  _lcpp_op(n, weight_type, rows, k, packed)            linear.py:85-114   routing: op name or None
  _fused_mul_mat_gguf(x, weight, weight_type, x_q8, packed)   117-218     one product x @ W.T
  _quantize_x_q8_1(x, weight_types, weight_rows, packed)      251-268     shared q8_1 of x
  _shard_runs / _shard_weight                                  221-248     same-type runs of a fused weight
  GGUFLinearMethod.{create_weights, process_weights_after_loading, apply}  347-570
  torch.ops.vllm._fused_mul_mat_gguf / _quantize_x_q8_1       307-325     custom ops with fake impls

Differences, all deliberate: there is one route (the reference's "Route L"), no stock / Triton /
dequantise fallback, and only the four ggml types with an sm_100a kernel compute; a type outside
that set raises. The op names `_lcpp_op` returns are API (tests and `_quantize_x_q8_1` key on
them), so the table keeps the reference's thresholds; which kernel runs under a name is decided in
libgsq (gsq_route).
"""

from __future__ import annotations

import os
from itertools import groupby

import torch

from .. import lcpp_ops, ops
from . import iq3_pack
from .params import GGUFWeightParameter, GGUFWeightTypeParameter, _gguf_ordered_shard_ids

Q2_K, Q4_K, Q6_K = ops.GGML_TYPE_Q2_K, ops.GGML_TYPE_Q4_K, ops.GGML_TYPE_Q6_K
IQ2_S, IQ3_S, IQ3_XXS = ops.GGML_TYPE_IQ2_S, ops.GGML_TYPE_IQ3_S, ops.GGML_TYPE_IQ3_XXS
IQ4_XS, IQ1_M = ops.GGML_TYPE_IQ4_XS, ops.GGML_TYPE_IQ1_M

_IQ3_TYPES = (IQ3_S, IQ3_XXS)
_OWN_MIN_ROWS = {Q4_K: 3, IQ2_S: 1}          # fewest activation rows routed to lcpp_mul_mat_vec_own
_IQ1_M_MAX_ROWS = 32
_MMA_K_TYPES = (Q4_K, IQ4_XS, IQ2_S)
PACKED_VEC_MAX_ROWS = 8
# ops that quantise X themselves (128-value blocks); the others read apply()'s shared x_q8
_OWN_QUANTIZE_OPS = ("lcpp_mul_mat_q", "lcpp_mul_mat_mma_k", "lcpp_mul_mat_iq3_packed")
# in the reference these wrote X's dtype directly and the rest went through an fp32 dst; here every
# kernel writes X's dtype, the tuple is kept because callers import it
_X_DTYPE_OPS = ("lcpp_mul_mat_mma_k", "lcpp_mul_mat_iq3_packed", "lcpp_mul_mat_vec_iq3")
_FP32_DST_BUDGET = 256 << 20

_MMA_K_ON = os.environ.get("VLLM_GGUF_MMA_K", "1") != "0"
_IQ3_TILED_ON = os.environ.get("VLLM_GGUF_IQ3_TILED", "1") != "0"
_IQ1M_MMVQ_ON = os.environ.get("VLLM_GGUF_IQ1M_MMVQ", "1") != "0"


def _mma_k_wins(weight_type: int, n: int, rows: int, k: int) -> bool:
    """lcpp_mul_mat_mma_k's cell of the table: 9..32 activation rows, W above 2048 rows; IQ4_XS at
    17..32 rows only on W of at least 12288 x 5120 values."""
    if not _MMA_K_ON or weight_type not in _MMA_K_TYPES:
        return False
    if n < 9 or n > 32 or rows <= 2048:
        return False
    if weight_type == IQ4_XS and n > 16:
        return rows * k >= 12288 * 5120
    return True


def _lcpp_op(n: int, weight_type: int, rows: int, k: int, packed: bool = False) -> str | None:
    """Op name for n activation rows times a `weight_type` weight of `rows` x `k`, or None.
    packed: the layer's IQ3 runs are in iq3_pack's layout."""
    iq3 = weight_type in _IQ3_TYPES
    if iq3 and packed:
        vec = n <= PACKED_VEC_MAX_ROWS or not _IQ3_TILED_ON
        return "lcpp_mul_mat_vec_iq3_mma_packed" if vec else "lcpp_mul_mat_iq3_packed"
    if weight_type == IQ1_M:
        ok = n <= 8 or (n <= _IQ1_M_MAX_ROWS and _IQ1M_MMVQ_ON)
        return "lcpp_mul_mat_vec_q" if ok else None
    if n <= 8:
        if iq3:
            return "lcpp_mul_mat_vec_iq3" if n < 6 else "lcpp_mul_mat_vec_iq3_mma"
        if rows > 2048 and n >= _OWN_MIN_ROWS.get(weight_type, 9):
            return "lcpp_mul_mat_vec_own"
    if _mma_k_wins(weight_type, n, rows, k):
        return "lcpp_mul_mat_mma_k"
    return "lcpp_mul_mat_q" if n >= 8 else "lcpp_mul_mat_vec_q"


def _unquantized_gemm(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None = None) -> torch.Tensor:
    """x @ weight.T (+ bias) for an F32 / F16 / BF16 tensor of the file. Up to 8 activation rows times a weight of at
    most 128 rows run as a batched gemv, as in the reference (linear.py:281-291: the library GEMM picked for that shape
    is several times slower than reading the small weight once per row)."""
    if x.shape[0] <= 8 and weight.shape[0] <= 128 and bias is None:
        return torch.bmm(x.unsqueeze(1), weight.T.expand(x.shape[0], -1, -1)).squeeze(1)
    return torch.nn.functional.linear(x, weight, bias)


def _require_route() -> None:
    if not ops.LCPP_ENABLED:
        raise RuntimeError("VLLM_GGUF_LCPP=0: this package only implements that route and has no other path")


def _fused_mul_mat_gguf(
    x: torch.Tensor,
    weight: torch.Tensor,
    weight_type: int,
    x_q8: torch.Tensor | None = None,
    packed: bool = False,
) -> torch.Tensor:
    """x @ weight.T. x_q8: x already quantised by _quantize_x_q8_1 for this product and others on the
    same x; used if this product's op reads q8_1."""
    n, rows = x.shape[0], weight.shape[0]
    if n == 0:
        return torch.empty(0, rows, dtype=x.dtype, device=x.device)
    if weight_type in ops.UNQUANTIZED_TYPES:
        return _unquantized_gemm(x, weight)
    _require_route()
    if weight_type not in ops.LCPP_QUANT_TYPES:
        raise NotImplementedError(f"Unsupported GGUF quantization type: {weight_type}")
    # the layer's flag says its IQ3_S / Q6_K runs are repacked; this package leaves IQ3_XXS (which the reference
    # repacks too) in GGUF order, so such a run of a packed layer routes as unpacked
    packed = packed and weight_type in iq3_pack.PACKABLE_TYPES
    name = _lcpp_op(n, weight_type, rows, x.shape[1], packed)
    if name is None:
        raise NotImplementedError(f"no kernel for ggml type {weight_type} at {n} activation rows")
    if packed and weight_type == Q6_K:
        # this package also repacks Q6_K at load (_pack_iq3); its two ops keep the split of the table's names: the
        # vec op (reads the shared q8_1) where the table says lcpp_mul_mat_vec_q, the self-quantising one otherwise
        name = "gsq_mul_mat_vec_q6k_packed" if name == "lcpp_mul_mat_vec_q" else "gsq_mul_mat_q6k_packed"
    op = getattr(torch.ops._C_gguf, name)
    if name in _OWN_QUANTIZE_OPS or name == "gsq_mul_mat_q6k_packed":
        return op(weight, x, weight_type, rows)
    per_call = 32 if name == "lcpp_mul_mat_vec_iq3_mma_packed" else 8
    if n > per_call:  # VLLM_GGUF_IQ3_TILED=0, or IQ1_M above 8 rows: several calls of the vec op
        b = x.shape[1] // 32 * 36
        return torch.cat([
            op(weight, x[i:i + per_call], weight_type, rows, None if x_q8 is None else x_q8[i * b:(i + per_call) * b])
            for i in range(0, n, per_call)
        ])
    return op(weight, x, weight_type, rows, x_q8)


def _shard_weight(weight: torch.Tensor, start: int, end: int, size: int) -> torch.Tensor:
    """Rows start:end of a padded multi-shard weight as [rows, size] bytes. Runs of adjacent
    same-type shards are stored contiguously from the start of the run's first row
    (_create_padded_weight_param), so this is a view."""
    rows = end - start
    return weight[start:end].view(-1)[: rows * size].view(rows, size)


def _shard_runs(weight: torch.Tensor, shard_ids: list, weight_types: list[int]):
    """(bytes view, type) of each run of adjacent same-type shards: one product per run."""
    offsets = weight.shard_offset_map
    for wtype, run in groupby(zip(shard_ids, weight_types), key=lambda p: p[1]):
        ids = [i for i, _ in run]
        start, _, size = offsets[ids[0]]
        yield _shard_weight(weight, start, offsets[ids[-1]][1], size), wtype


def _quantize_x_q8_1_fake(x: torch.Tensor, weight_types: list[int], weight_rows: list[int],
                          packed: bool = False) -> torch.Tensor:
    return torch.empty(x.shape[0] * x.shape[1] // 32 * 36, dtype=torch.uint8, device=x.device)


def _quantize_x_q8_1(x: torch.Tensor, weight_types: list[int], weight_rows: list[int],
                     packed: bool = False) -> torch.Tensor:
    """x as block_q8_1 bytes, made once for all the listed products that read q8_1; when none does
    (their ops quantise for themselves), an unfilled buffer of the same size that nothing reads."""
    n, k = x.shape
    readers = [
        t for t, rows in zip(weight_types, weight_rows)
        if t in ops.LCPP_QUANT_TYPES and _lcpp_op(n, t, rows, k, packed) not in (None, *_OWN_QUANTIZE_OPS)
    ]
    if n and readers:
        return torch.ops._C_gguf.lcpp_quantize_q8_1(x, readers[0], False, False)
    return _quantize_x_q8_1_fake(x, weight_types, weight_rows)


def _fused_mul_mat_gguf_fake(x, weight, weight_type, x_q8=None, packed=False):
    return torch.empty(x.shape[0], weight.shape[0], dtype=x.dtype, device=x.device)


_VLLM_LIB = None


def _register_python_ops():
    """torch.ops.vllm._fused_mul_mat_gguf / _quantize_x_q8_1 with fake impls, as the reference does
    through vLLM's direct_register_custom_op. If the names are taken (vLLM's own GGUF module defines
    the first), the plain functions are used."""
    global _VLLM_LIB
    if _VLLM_LIB is not None:
        return
    _VLLM_LIB = torch.library.Library("vllm", "FRAGMENT")
    specs = [
        ("_fused_mul_mat_gguf",
         "(Tensor x, Tensor weight, int weight_type, Tensor? x_q8=None, bool packed=False) -> Tensor",
         _fused_mul_mat_gguf, _fused_mul_mat_gguf_fake),
        ("_quantize_x_q8_1", "(Tensor x, int[] weight_types, int[] weight_rows, bool packed=False) -> Tensor",
         _quantize_x_q8_1, _quantize_x_q8_1_fake),
    ]
    out = {}
    for name, schema, fn, fake in specs:
        try:
            _VLLM_LIB.define(name + schema)
            _VLLM_LIB.impl(name, fn, "CUDA")
            _VLLM_LIB.impl(name, fn, "CPU")
            _VLLM_LIB._register_fake(name, fake)
            out[name] = getattr(torch.ops.vllm, name)
        except RuntimeError:
            out[name] = fn
    return out


_py_ops = _register_python_ops()
fused_mul_mat_gguf = _py_ops["_fused_mul_mat_gguf"]
quantize_x_q8_1 = _py_ops["_quantize_x_q8_1"]


class GGUFLinearMethod:
    """Linear method for GGUF weights (create_weights / process_weights_after_loading / apply)."""

    # apply() sends IQ3_S weights to the packed kernels; False in subclasses that need GGUF bytes
    pack_iq3 = True

    def __init__(self, quant_config=None, layout=None) -> None:
        self.quant_config = quant_config
        self.layout = layout

    def create_weights(self, layer: torch.nn.Module, input_size_per_partition: int,
                       output_partition_sizes: list[int], input_size: int, output_size: int,
                       params_dtype: torch.dtype, **extra_weight_attrs):
        """Registers `weight` (uint8 bytes, filled by weight.load_shard) and `weight_type`."""
        del output_size
        self.params_dtype = params_dtype
        weight = GGUFWeightParameter(
            input_dim=1, output_dim=0,
            tensor_shape=(sum(output_partition_sizes), input_size_per_partition))
        weight_type = GGUFWeightTypeParameter()
        for k, v in extra_weight_attrs.items():
            if k != "weight_loader":
                setattr(weight, k, v)
        layer.register_parameter("weight", weight)
        layer.register_parameter("weight_type", weight_type)
        if self.layout is not None:
            weight.gguf_layout = self.layout
            weight.gguf_logical_input_size = input_size
            weight.gguf_weight_type_parameter = weight_type

    def process_weights_after_loading(self, layer: torch.nn.Module):
        _require_route()
        wt = layer.weight_type
        types = set(wt.shard_weight_type.values()) | {wt.weight_type}
        bad = [t for t in types if t not in ops.UNQUANTIZED_TYPES and t not in ops.B200_QUANT_TYPES]
        if bad:
            raise ValueError(f"Unsupported GGUF quantization type {bad[0]} in layer {layer}.")
        self._create_padded_weight_param(layer)
        if self.pack_iq3:
            self._pack_iq3(layer)

    def _pack_iq3(self, layer: torch.nn.Module) -> None:
        """Repack the layer's IQ3_S (and, in this package, Q6_K) products in place and set weight.iq3_packed. All
        or nothing per layer: only if every such run has a multiple of 16 rows and 16-byte aligned bytes."""
        weight = layer.weight
        if getattr(weight, "iq3_packed", False):
            return
        if hasattr(weight, "shard_offset_map"):
            types = layer.weight_type.shard_weight_type
            fallback = layer.weight_type.weight_type
            runs = list(_shard_runs(weight, weight.shard_id, [types.get(i, fallback) for i in weight.shard_id]))
        else:
            runs = [(weight.data, layer.weight_type.weight_type)]
        runs = [(w, t) for w, t in runs if t in iq3_pack.PACKABLE_TYPES]
        if not runs or any(w.shape[0] % iq3_pack.ROWS or w.data_ptr() % 16 for w, _ in runs):
            return
        for w, t in runs:
            iq3_pack.pack_(w, t)
        weight.iq3_packed = True

    def _create_padded_weight_param(self, layer: torch.nn.Module):
        """Fused layers: lay the shards out in one zeroed [sum rows, max row_bytes] buffer, each run
        of adjacent same-type shards contiguous from the start of its first shard's rows."""
        weight = layer.weight
        shards = weight.data_container
        if len(shards) <= 1:
            if len(shards) == 1 and weight.data.numel() == 0:
                weight.data = shards[0]
                only = weight.shard_id[0]
                layer.weight_type.weight_type = layer.weight_type.shard_weight_type.get(
                    only, layer.weight_type.weight_type)
                weight.data_container, weight.shard_id, weight.shard_id_map = [], [], {}
            return
        assert len({s.dtype for s in shards}) == 1, "data container has mixed dtypes"
        width = max(s.size(1) for s in shards)
        total = sum(s.size(0) for s in shards)
        padded = torch.zeros((total, width), dtype=shards[0].dtype, device=shards[0].device)
        flat = padded.view(-1)
        order = _gguf_ordered_shard_ids(weight.shard_id)
        types = layer.weight_type.shard_weight_type
        offsets: dict = {}
        row = run_row = 0
        run_type = None
        for sid in order:
            s = shards[weight.shard_id_map[sid]]
            n, size = s.shape
            wtype = types.get(sid, layer.weight_type.weight_type)
            if wtype != run_type:
                run_row, run_type = row, wtype
            at = run_row * width + (row - run_row) * size
            flat[at:at + n * size] = s.reshape(-1)
            offsets[sid] = (row, row + n, size)
            row += n
        new = GGUFWeightParameter(padded, input_dim=getattr(weight, "input_dim", 1),
                                  output_dim=getattr(weight, "output_dim", 0),
                                  tensor_shape=getattr(weight, "tensor_shape", None))
        new.shard_id = order
        new.shard_id_map = dict(weight.shard_id_map)
        new.shard_offset_map = offsets
        layer.register_parameter("weight", new)

    def apply(self, layer: torch.nn.Module, x: torch.Tensor, bias: torch.Tensor | None = None) -> torch.Tensor:
        if self.layout is not None:
            x = self.layout.input_to_gguf(x)
        weight = layer.weight
        shard_id = weight.shard_id
        packed = getattr(weight, "iq3_packed", False)
        if shard_id:
            shard_id = ["q", "k", "v"] if "q" in shard_id else shard_id
            fallback = layer.weight_type.weight_type
            types = [layer.weight_type.shard_weight_type.get(i, fallback) for i in shard_id]
            if len(set(types)) == 1:
                out = fused_mul_mat_gguf(x, weight, types[0], None, packed)
            else:
                runs = list(_shard_runs(weight, shard_id, types))
                x_q8 = quantize_x_q8_1(x, [t for _, t in runs], [w.shape[0] for w, _ in runs], packed)
                out = torch.cat([fused_mul_mat_gguf(x, w, t, x_q8, packed) for w, t in runs], dim=1)
        else:
            out = fused_mul_mat_gguf(x, weight, layer.weight_type.weight_type, None, packed)
        if bias is not None:
            out.add_(bias)
        return out


def register_compile_factor(registry: dict | None = None) -> bool:
    """VLLM_GGUF_LCPP changes the traced graph of apply() and the weight layout, so it has to key vLLM's torch.compile
    caches: the reference adds it to vllm.envs.environment_variables, which vLLM hashes into its compile factors
    (plugin/vllm_gguf_plugin/plugin.py:156-161). Same here; `registry` stands in for that dict in tests. Returns
    whether the entry is present afterwards."""
    import os

    if registry is None:
        try:
            import vllm.envs as envs

            registry = envs.environment_variables
        except Exception:  # no vLLM, or one without that registry
            return False
    registry.setdefault("VLLM_GGUF_LCPP", lambda: os.environ.get("VLLM_GGUF_LCPP"))
    return "VLLM_GGUF_LCPP" in registry


def _register_with_vllm() -> None:
    """Inside a vLLM process, make the class a LinearMethodBase and list it as weight-loader-v2 capable
    (the reference's decorator keys on the class name, linear.py:330, 347). Outside vLLM nothing is
    imported."""
    import sys

    if "vllm" not in sys.modules:
        return
    register_compile_factor()
    try:
        from vllm.model_executor.layers.linear import LinearMethodBase, register_weight_loader_v2_supported_method

        if LinearMethodBase not in GGUFLinearMethod.__bases__:
            GGUFLinearMethod.__bases__ = (LinearMethodBase,)
        register_weight_loader_v2_supported_method(GGUFLinearMethod)
    except Exception:  # vLLM present but with a different layout of these symbols
        pass


_register_with_vllm()
