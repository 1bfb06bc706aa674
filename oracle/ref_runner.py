"""Run the reference's own CUDA ops (oracle/_ref/ref_C_gguf.so, built by oracle/build_ref.py) on cases
prepared by a test, in a process of its own (TEST INFRASTRUCTURE; the library defines the same
torch.ops._C_gguf names as this repository, so the two never share a process).

    python oracle/ref_runner.py cases.pt results.pt

cases.pt: list of dicts {"op": name, "args": [tensors / ints / bools / None ...], "time": bool, "copies": int,
"no_out": bool}. Tensors are moved to cuda:0. results.pt: list of {"out": CPU tensor (None with no_out), "us": float
or None}. Timing (the method of the reference's kit/micro_gguf.py:164-195): one call per weight copy in one CUDA
graph, so that a copy is read again only after all the others, best of three replays.
"""

import os
import sys

import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def graph_us(fn, reps=10):
    reps = max(1, reps)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        fn()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for _ in range(reps):
            fn()
    best = 1e30
    for _ in range(3):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        g.replay()
        e1.record()
        torch.cuda.synchronize()
        best = min(best, e0.elapsed_time(e1) * 1e3 / reps)
    return best


def main():
    torch.ops.load_library(os.path.join(HERE, "_ref", "ref_C_gguf.so"))
    cases = torch.load(sys.argv[1])
    out = []
    on_device = {}   # a tensor shared by several cases is uploaded once
    for c in cases:
        args = []
        for a in c["args"]:
            if isinstance(a, torch.Tensor):
                key = (a.data_ptr(), tuple(a.shape), a.dtype)
                if key not in on_device:
                    if a.numel() > (1 << 24):
                        on_device.clear()
                        torch.cuda.empty_cache()
                    on_device[key] = a.to("cuda:0")
                a = on_device[key]
            args.append(a)
        op = getattr(torch.ops._C_gguf, c["op"])
        if c.get("copies"):  # timing on several copies of W so that L2 cannot serve it
            ws = [args[0]] + [args[0].clone() for _ in range(c["copies"] - 1)]
            i = [0]

            def fn():
                w = ws[i[0] % len(ws)]
                i[0] += 1
                return op(w, *args[1:])
        else:
            def fn():
                return op(*args)
        y = fn()
        torch.cuda.synchronize()
        us = graph_us(fn, c.get("copies") or 10) if c.get("time") else None
        out.append({"out": None if c.get("no_out") else y.cpu(), "us": us})
        del args, y
    torch.save(out, sys.argv[2])


if __name__ == "__main__":
    main()
