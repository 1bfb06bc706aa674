"""Worker of tests/test_gpu_peer_allreduce.py: one rank of a 2..4-GPU group (launched with torch.distributed.run).
Checks gsq_b200.tp.PeerAllReduce against a sum formed on the host in the same order, eagerly and inside a CUDA
graph, and prints the time per reduction beside NCCL's."""
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
    from gsq_b200 import tp

    def log(msg):
        if os.environ.get("GSQ_WORKER_LOG"):
            print(f"[rank {rank}] {msg}", file=sys.stderr, flush=True)
    m, n = 32, 5120
    log("setting up symmetric memory")
    ar = tp.PeerAllReduce(m * n * 4)
    log("set up")
    for dtype in (torch.bfloat16, torch.float16, torch.float32):
        for it in range(4):
            g = torch.Generator().manual_seed(100 * it + 7)
            parts = [torch.randn(m, n, generator=g).to(dtype) for _ in range(world)]      # every rank knows all partials
            slot = it % 2
            ar.partial(slot, (m, n), dtype).copy_(parts[rank].to(dev))
            out = torch.empty(m, n, dtype=dtype, device=dev)
            ar.reduce(slot, out)
            torch.cuda.synchronize()
            log(f"reduced {dtype} {it}")
            want = torch.zeros(m, n, dtype=torch.float32)
            for p in parts:                                                             # rank order, fp32
                want += p.float()
            assert torch.equal(out.cpu(), want.to(dtype)), (str(dtype), it, float((out.cpu().float() - want).abs().max()))
    # inside a CUDA graph: 8 reductions on alternating slots, each after a kernel that writes the partial
    dtype = torch.bfloat16
    src = [torch.randn(m, n, device=dev, dtype=dtype) for _ in range(8)]
    outs = [torch.empty(m, n, dtype=dtype, device=dev) for _ in range(8)]

    def seq():
        for i in range(8):
            ar.partial(i % 2, (m, n), dtype).copy_(src[i])
            ar.reduce(i % 2, outs[i])
    log("eager sequence")
    seq()
    torch.cuda.synchronize()
    eager = [o.clone() for o in outs]
    log("capture")
    dist.barrier()
    log("barrier passed")
    gph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(gph):
        seq()
    log("captured")
    for _ in range(3):
        gph.replay()
        torch.cuda.synchronize()
        log("replayed")
    for a, b in zip(eager, outs):
        assert torch.equal(a, b)
    dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(10):
        gph.replay()
    e1.record()
    torch.cuda.synchronize()
    t_peer = e0.elapsed_time(e1) * 1e3 / 80
    buf = torch.randn(m, n, device=dev, dtype=dtype)

    def nccl_seq():
        for i in range(8):
            buf.copy_(src[i])
            dist.all_reduce(buf)
    nccl_seq()
    torch.cuda.synchronize()
    dist.barrier()
    g2 = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g2):
        nccl_seq()
    for _ in range(3):
        g2.replay()
    torch.cuda.synchronize()
    dist.barrier()
    e0.record()
    for _ in range(10):
        g2.replay()
    e1.record()
    torch.cuda.synchronize()
    t_nccl = e0.elapsed_time(e1) * 1e3 / 80
    import ctypes
    from gsq_b200 import _cabi
    flag = ctypes.c_int(-1)
    assert _cabi.lib.gsq_allreduce_error_flag(ctypes.byref(flag)) == 0 and flag.value == 0
    if rank == 0:
        print(f"peer all-reduce ok: world {world}, [{m}, {n}] bf16: {t_peer:.1f} us per (copy + reduction) in a graph; "
              f"NCCL all_reduce {t_nccl:.1f} us", flush=True)
    log("releasing the graphs and the symmetric memory")
    del gph, g2, ar      # (a process group is not destroyed while graphs that hold its collectives are alive)
    import gc
    gc.collect()
    torch.cuda.synchronize()
    dist.barrier()
    log("destroying the process group")
    dist.destroy_process_group()
    log("exiting")


if __name__ == "__main__":
    main()
