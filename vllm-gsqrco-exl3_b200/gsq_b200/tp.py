"""Tensor-parallel sharding of GGUF weights for the quantised-linear path.

The reference narrows the loaded bytes evenly (quantization/params.py:228-301) and was only ever run at
TP = 1; its kernels demand K % 512 == 0 (lcpp_shim.cu:706-708), which K-shards of 5120 or 17408 columns
break at TP = 4 and 8. Here:

  * column-parallel layers (qkv, gate_up, lm_head) are cut along N in multiples of 16 rows (the IQ3_S
    repack tile), the last rank taking the remainder; outputs are all-gathered;
  * row-parallel layers (o_proj, down) are cut along K at superblock (256-column) granularity, the first
    (K/256) % world ranks taking one superblock more; fp32 partial outputs are summed (all-reduce).

`relaxed_k()` lowers the guards' K granularity from 512 to 256 for the duration of a block.
"""

from __future__ import annotations

import contextlib
from dataclasses import dataclass

from . import lcpp_ops

BLOCK_BYTES = {12: 144, 14: 210, 21: 110, 23: 136}


@dataclass(frozen=True)
class Shard:
    mode: str      # "N": rows [start, start + count) ; "K": superblocks [start, start + count)
    start: int
    count: int


def shard_plan(n: int, k: int, world: int, rank: int, mode: str | None = None) -> Shard:
    """This rank's shard of an [n, k] weight. mode None: K-shard when k > n (down-projection-like), else N."""
    if world == 1:
        return Shard("N", 0, n)
    if mode is None:
        mode = "K" if k > n else "N"
    if mode == "K":
        base, extra = divmod(k // 256, world)
        return Shard("K", rank * base + min(rank, extra), base + (1 if rank < extra else 0))
    per = n // world
    per -= per % 16
    start = rank * per
    return Shard("N", start, n - start if rank == world - 1 else per)


def matched_up_rows(k_down: int, world: int, rank: int) -> tuple[int, int]:
    """(first channel, channel count) of the gate / up projection that rank `rank` keeps so that its SwiGLU output
    is exactly the column range of its K-shard of the down projection (k_down columns, cut at 256 granularity, the
    first ranks one superblock more): at 8 ranks and 17408 columns {2304 x 4, 2048 x 4} channels, not 2176 each."""
    s = shard_plan(1, k_down, world, rank, "K")
    return s.start * 256, s.count * 256


def shard_bytes(raw, ggml_type: int, s: Shard):
    """Rows / superblock columns of a [rows, row_bytes] byte matrix (numpy array or torch tensor) for a shard."""
    if s.mode == "N":
        return raw[s.start:s.start + s.count]
    bs = BLOCK_BYTES[ggml_type]
    return raw[:, s.start * bs:(s.start + s.count) * bs]


def shard_activation(x, s: Shard):
    """Columns of X that a K-shard multiplies (a strided view, accepted as is by the ops)."""
    return x if s.mode == "N" else x[:, s.start * 256:(s.start + s.count) * 256]


@contextlib.contextmanager
def relaxed_k():
    old = lcpp_ops.set_k_multiple(256)
    try:
        yield
    finally:
        lcpp_ops.set_k_multiple(old)


def combine(y, s: Shard, n: int, k: int, world: int, group=None):
    """Collective after a sharded product: all-gather of [M, rows_r] along N, or all-reduce of partial [M, N]."""
    import torch
    import torch.distributed as dist

    if world == 1:
        return y
    if s.mode == "K":
        dist.all_reduce(y, group=group)
        return y
    parts = [torch.empty(y.shape[0], shard_plan(n, k, world, r, "N").count, dtype=y.dtype, device=y.device)
             for r in range(world)]
    dist.all_gather(parts, y.contiguous(), group=group)
    return torch.cat(parts, dim=1)


class PeerAllReduce:
    """Sum of K-sharded partial results over peer memory (gsq_allreduce_sum): `slots` partial buffers of `nbytes`
    each in symmetric memory (torch.distributed._symmetric_memory: the same allocation mapped into every rank of the
    group) plus the flag pad. Usage per reduction, the same sequence on every rank:

        part = ar.partial(i, (m, n), dtype)      # products write the rank's partial here (lcpp_ops.output_into)
        ar.reduce(i, out)                        # out[...] = sum over ranks, bit-identical on all of them

    with i alternating between slots from one reduction to the next. Launches one kernel on the current stream and
    nothing else, so it can be captured in a CUDA graph."""

    def __init__(self, nbytes: int, slots: int = 2, group=None):
        import torch
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm

        from . import _cabi

        assert slots >= 2
        group = group or dist.group.WORLD
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.dev = torch.device("cuda", torch.cuda.current_device())
        self.nbytes = (int(nbytes) + 255) // 256 * 256
        self.slots = slots
        total = slots * self.nbytes + 256
        self.buf = symm.empty(total, dtype=torch.uint8, device=self.dev)
        self.buf.zero_()
        self.handle = symm.rendezvous(self.buf, group)
        ptrs = [int(p) for p in self.handle.buffer_ptrs]
        self._bufs = [torch.tensor([p + i * self.nbytes for p in ptrs], dtype=torch.int64, device=self.dev) for i in range(slots)]
        self._flags = torch.tensor([p + slots * self.nbytes for p in ptrs], dtype=torch.int64, device=self.dev)
        self._state = torch.zeros(2, dtype=torch.int32, device=self.dev)
        self._lib, self._check = _cabi.lib, _cabi.check
        torch.cuda.synchronize()
        dist.barrier(group)      # every rank's pad is zero before anyone signals

    def fused(self, slot_bytes: int):
        """Resources of the sum fused into the product kernel (gsq_linear_allreduce): a second symmetric allocation of
        2 * world slots of `slot_bytes` plus `world` flag words per rank. Returns the context manager
        to wrap each K-sharded product call in: `with ar.fused(nbytes): y = op(W, X, type, rows)` -- y is the sum."""
        import torch
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm

        from . import _cabi, lcpp_ops

        if getattr(self, "_fused", None) is None or self._fused_slot < slot_bytes:
            sb = (int(slot_bytes) + 255) // 256 * 256
            total = 2 * self.world * sb + 256
            self._fbuf = symm.empty(total, dtype=torch.uint8, device=self.dev)
            self._fbuf.zero_()
            self._fhandle = symm.rendezvous(self._fbuf, dist.group.WORLD)
            ptrs = [int(p) for p in self._fhandle.buffer_ptrs]
            self._fslots = torch.tensor(ptrs, dtype=torch.int64, device=self.dev)
            self._fflags = torch.tensor([p + 2 * self.world * sb for p in ptrs], dtype=torch.int64, device=self.dev)
            self._fstate = torch.zeros(4, dtype=torch.int32, device=self.dev)
            ctx = _cabi.PeerReduce()
            ctx.slots, ctx.flags, ctx.state = self._fslots.data_ptr(), self._fflags.data_ptr(), self._fstate.data_ptr()
            ctx.rank, ctx.world, ctx.slot_bytes = self.rank, self.world, sb
            self._fused, self._fused_slot = ctx, sb
            torch.cuda.synchronize()
            dist.barrier()       # every rank's flags are zero before anyone signals
        return lcpp_ops.peer_reduce(self._fused)

    def partial(self, slot: int, shape, dtype):
        import torch

        n = 1
        for d in shape:
            n *= int(d)
        nb = n * torch.empty(0, dtype=dtype).element_size()
        assert nb <= self.nbytes, (nb, self.nbytes)
        return self.buf[slot * self.nbytes: slot * self.nbytes + nb].view(dtype).view(*shape)

    def reduce(self, slot: int, out) -> None:
        import torch

        dt = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}[out.dtype]
        assert out.is_contiguous() and out.numel() * out.element_size() <= self.nbytes
        st = torch.cuda.current_stream(self.dev).cuda_stream
        self._check(self._lib.gsq_allreduce_sum(self._bufs[slot].data_ptr(), self._flags.data_ptr(), self.rank, self.world,
                                                 out.numel(), dt, out.data_ptr(), self._state.data_ptr(), st),
                    "gsq_allreduce_sum")
