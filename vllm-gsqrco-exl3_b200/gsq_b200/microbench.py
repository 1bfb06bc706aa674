"""One cell of the kernel micro-benchmark: a (type, rows N, columns K, activation rows M) product on
seeded synthetic blocks, a few launches on distinct weight copies (the method of the reference's
kit/micro_gguf.py:164-195, without the graph: meant to be run under a profiler or for a quick number).

    python vllm-gsqrco-exl3_b200/gsq_b200/microbench.py --type Q4_K --n 17408 --k 5120 --m 1 --iters 3
"""

from __future__ import annotations

import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    import torch

    import gsq_b200  # noqa: F401
    from gsq_b200 import synth
    from gsq_b200.quantization import iq3_pack, linear

    ap = argparse.ArgumentParser()
    ap.add_argument("--type", default="Q4_K", choices=list(synth.TYPE_IDS))
    ap.add_argument("--n", type=int, default=17408)
    ap.add_argument("--k", type=int, default=5120)
    ap.add_argument("--m", type=int, default=1)
    ap.add_argument("--iters", type=int, default=3)
    ap.add_argument("--copies", type=int, default=4)
    ap.add_argument("--unpacked", action="store_true")
    ap.add_argument("--dtype", default="float16")
    a = ap.parse_args()
    dev = "cuda:0"
    t = synth.TYPE_IDS[a.type]
    w0 = torch.from_numpy(synth.make_weight(t, a.n, a.k, 1)).to(dev)
    packed = a.type == "IQ3_S" and not a.unpacked and a.n % 16 == 0
    if packed:
        iq3_pack.pack_(w0, t)
    ws = [w0] + [w0.clone() for _ in range(a.copies - 1)]
    x = synth.nudge_ties_torch(torch.from_numpy(synth.make_activation(a.m, a.k, 2)).to(getattr(torch, a.dtype))).to(dev)
    for i in range(2):
        linear.fused_mul_mat_gguf(x, ws[i % len(ws)], t, None, packed)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(a.iters):
        y = linear.fused_mul_mat_gguf(x, ws[(i + 2) % len(ws)], t, None, packed)
    e1.record()
    torch.cuda.synchronize()
    us = e0.elapsed_time(e1) * 1e3 / a.iters
    print(f"{a.type} {a.n}x{a.k} m={a.m} packed={packed}: {us:.1f} us per call (eager, incl. launch overhead), "
          f"{w0.numel() / us / 1e3:.0f} GB/s; op {linear._lcpp_op(a.m, t, a.n, a.k, packed)}; |y| {float(y.float().abs().mean()):.4f}")


if __name__ == "__main__":
    main()
