"""Tensor-parallel sharding on CPU: shard arithmetic for TP 2/4/8 (uneven K-shards included), equivalence
of sharded and unsharded products on the oracle, and the two collectives among gloo ranks (world size 2)."""

import os
import socket
import sys

import numpy as np
import pytest
import torch

from gsq_b200 import synth, tp
from oracle import blocks, product, q8_1


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("n,k", [(5120, 5120), (17408, 5120), (5120, 17408), (7168, 5120), (151936, 5120)])
def test_plans_cover_exactly(world, n, k):
    plans = [tp.shard_plan(n, k, world, r) for r in range(world)]
    mode = plans[0].mode
    assert all(p.mode == mode for p in plans)
    total = n if mode == "N" else k // 256
    pos = 0
    for p in plans:
        assert p.start == pos and p.count > 0
        pos += p.count
    assert pos == total
    if mode == "N":
        assert all(p.count % 16 == 0 for p in plans[:-1]) and all(p.start % 16 == 0 for p in plans)
    else:
        counts = [p.count for p in plans]
        assert max(counts) - min(counts) <= 1


def test_uneven_k_shards_of_the_two_k_sharded_layers():
    assert [tp.shard_plan(5120, 17408, 8, r).count for r in range(8)] == [9, 9, 9, 9, 8, 8, 8, 8]
    assert [tp.shard_plan(5120, 5120, 8, r, "K").count for r in range(8)] == [3, 3, 3, 3, 2, 2, 2, 2]


@pytest.mark.parametrize("world", [2, 4, 8])
def test_gate_up_channels_match_the_k_shards_of_down(world):
    """A rank's SwiGLU output must be exactly the columns its K-shard of the down projection multiplies: the gate /
    up channels are cut where down's superblocks are cut (uneven at 8 ranks: 2304 x 4, 2048 x 4), not evenly."""
    inter = 17408
    got = [tp.matched_up_rows(inter, world, r) for r in range(world)]
    assert got[0][0] == 0 and sum(c for _, c in got) == inter
    for r in range(world):
        s = tp.shard_plan(5120, inter, world, r, "K")
        assert got[r] == (s.start * 256, s.count * 256) and got[r][1] % 16 == 0
        if r:
            assert got[r][0] == got[r - 1][0] + got[r - 1][1]
    if world == 8:
        assert [c for _, c in got] == [2304] * 4 + [2048] * 4


@pytest.mark.parametrize("t", [21, 12])
@pytest.mark.parametrize("world", [2, 4, 8])
def test_sharded_products_equal_unsharded(t, world):
    n, k, m = 64, 2560, 3
    raw = synth.make_weight(t, n, k, 5)
    x = synth.make_activation(m, k, 6)
    q, d, _ = q8_1.quantize_q8_1(x)
    full = product.product_q81(blocks.decode(raw, t), q, d.astype(np.float32))
    ksum = np.zeros_like(full)
    for r in range(world):
        s = tp.shard_plan(n, k, world, r, "K")
        dec = blocks.decode(np.ascontiguousarray(tp.shard_bytes(raw, t, s)), t)
        cols = slice(s.start * 256, (s.start + s.count) * 256)
        ksum += product.product_q81(dec, q[:, cols], d[:, s.start * 8:(s.start + s.count) * 8].astype(np.float32))
    assert product.rel_err(ksum, full) <= 1e-12
    parts = []
    for r in range(world):
        s = tp.shard_plan(n, k, world, r, "N")
        if s.count:
            parts.append(product.product_q81(blocks.decode(tp.shard_bytes(raw, t, s), t), q, d.astype(np.float32)))
    assert np.array_equal(np.concatenate(parts, axis=1), full)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank, world, port, out):
    import torch.distributed as dist

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    n, k, m, t = 96, 1280, 2, 12
    raw = synth.make_weight(t, n, k, 9)
    x = synth.make_activation(m, k, 10)
    q, d, _ = q8_1.quantize_q8_1(x)
    res = {}
    for mode in ("N", "K"):
        s = tp.shard_plan(n, k, world, rank, mode)
        dec = blocks.decode(np.ascontiguousarray(tp.shard_bytes(raw, t, s)), t)
        if mode == "K":
            cols = slice(s.start * 256, (s.start + s.count) * 256)
            y = product.product_q81(dec, q[:, cols], d[:, s.start * 8:(s.start + s.count) * 8].astype(np.float32))
        else:
            y = product.product_q81(dec, q, d.astype(np.float32))
        res[mode] = tp.combine(torch.from_numpy(y), s, n, k, world).numpy()
    if rank == 0:
        full = product.product_q81(blocks.decode(raw, t), q, d.astype(np.float32))
        out.put({m_: float(product.rel_err(res[m_], full)) for m_ in res})
    dist.destroy_process_group()


def test_collectives_among_gloo_ranks():
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_rank_main, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    errs = out.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert errs["N"] == 0.0 and errs["K"] <= 1e-12
