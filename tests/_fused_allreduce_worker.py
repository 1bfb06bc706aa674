"""Worker of tests/test_gpu_peer_allreduce.py::test_product_fused_with_its_sum: one rank of a 2..4-GPU group (launched
with torch.distributed.run). K-sharded products whose kernel also sums the result over the ranks
(gsq_linear_allreduce through gsq_b200.tp.PeerAllReduce.fused) against the same products followed by a sum formed from
the gathered partials in rank order (bit for bit), eagerly and inside a CUDA graph."""
import ctypes
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path[:0] = [ROOT, os.path.join(ROOT, "vllm-gsqrco-exl3_b200")]


def main():
    rank, local, world = int(os.environ["RANK"]), int(os.environ["LOCAL_RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    import gsq_b200  # noqa: F401
    from gsq_b200 import _cabi, lcpp_ops, synth, tp
    from gsq_b200.quantization import iq3_pack

    ar = tp.PeerAllReduce(4096)
    ar.fused(48 * 5120 * 4)      # size the slots once for the largest result below
    cases = [("IQ3_S", 21, "lcpp_mul_mat_iq3_packed", 5120, 5120, True), ("IQ4_XS", 23, "lcpp_mul_mat_q", 5120, 17408, False),
             ("Q4_K", 12, "lcpp_mul_mat_q", 272, 5120, False)]
    checked = 0
    for name, t, opname, rows, k, packed in cases:
        sh = tp.shard_plan(rows, k, world, rank, "K")   # superblocks of this rank
        a0, cnt = sh.start, sh.count
        raw = synth.make_weight(t, rows, k, 31)           # the same full weight on every rank, then its K shard
        bs = synth.BLOCK_BYTES[t]
        w = torch.from_numpy(raw.reshape(rows, k // 256, bs)[:, a0:a0 + cnt].reshape(rows, cnt * bs).copy()).to(dev)
        if packed:
            iq3_pack.pack_(w, t)
        op = getattr(torch.ops._C_gguf, opname)
        for m, dtype in ((9, torch.bfloat16), (32, torch.bfloat16), (16, torch.float16), (48, torch.float32)):
            x = torch.from_numpy(synth.make_activation(m, k, 32 + m)).to(dtype)[:, a0 * 256:(a0 + cnt) * 256].contiguous().to(dev)
            with tp.relaxed_k():
                part = op(w, x, t, rows)                                     # this rank's partial
                gathered = [torch.empty_like(part) for _ in range(world)]
                dist.all_gather(gathered, part)
                want = torch.zeros(m, rows, dtype=torch.float32, device=dev)
                for p in gathered:                                           # rank order, fp32
                    want += p.float()
                want = want.to(dtype)
                for rep in range(3):                                         # both slot parities and back
                    with ar.fused(m * rows * 4):
                        y = op(w, x, t, rows)
                    torch.cuda.synchronize()
                    assert torch.equal(y, want), (name, m, str(dtype), rep, float((y.float() - want.float()).abs().max()))
                    checked += 1
    # inside a CUDA graph: four fused products in a row
    name, t, opname, rows, k, packed = cases[0]
    sh = tp.shard_plan(rows, k, world, rank, "K")
    a0, cnt = sh.start, sh.count
    raw = synth.make_weight(t, rows, k, 31)
    w = torch.from_numpy(raw.reshape(rows, k // 256, 110)[:, a0:a0 + cnt].reshape(rows, cnt * 110).copy()).to(dev)
    iq3_pack.pack_(w, t)
    x = torch.from_numpy(synth.make_activation(32, k, 77)).to(torch.bfloat16)[:, a0 * 256:(a0 + cnt) * 256].contiguous().to(dev)
    op = torch.ops._C_gguf.lcpp_mul_mat_iq3_packed
    outs = []

    def seq():
        outs.clear()
        with tp.relaxed_k():
            for _ in range(4):
                with ar.fused(32 * rows * 4):
                    outs.append(op(w, x, t, rows))
    seq()
    torch.cuda.synchronize()
    eager = [o.clone() for o in outs]
    dist.barrier()
    gph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(gph):
        seq()
    kept = list(outs)
    for _ in range(3):
        gph.replay()
    torch.cuda.synchronize()
    for a, b in zip(kept, eager):
        assert torch.equal(a, b)
    flag = ctypes.c_int(-1)
    assert _cabi.lib.gsq_peer_reduce_error_flag(ctypes.byref(flag)) == 0 and flag.value == 0
    del gph            # a graph holding captured kernels must go before the process group does
    dist.barrier()
    if rank == 0:
        print(f"fused product + sum ok: {checked} checks on {world} GPUs")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
