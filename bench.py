"""Benchmark of the quantised-linear hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (config.workload = "gemv_row_sweep"): the GEMV / small-GEMM row sweep -- Q4_K and IQ3_S
weights at (N, K) in {(5120, 5120), (17408, 5120), (5120, 17408)}, activation rows M in
{1, 2, 4, 8, 12, 16, 24, 32, 48}, fp16 activations ~ N(0,1) quantised to q8_1 on the device. One
step = one product for every (type, shape, M) cell (54 cells). The metric is weight GB/s: the GGUF
bytes of the weights each product has to read (N * K/256 * block bytes; activations and outputs are
not counted) divided by the time. Every cell cycles through enough distinct copies of its weight
that consecutive uses of one copy are more than 3 x L2 apart, so L2 cannot serve the weights.

  value     whole-job GB/s with weights and activations resident in HBM (quantise + product
            launches through torch.ops._C_gguf, CUDA events, max over ranks)
  e2e       the same sweep through GGUFLinearMethod.apply() with the activations in pinned host
            memory: host-to-device copy of X and device-to-host copy of Y inside the timed region
  roofline  the dp4a GEMV kernel alone (activations already quantised) on the M <= 8 cells: weight
            bytes per launch / mean launch time against the measured HBM copy bandwidth
  cpu_baseline  the oracle's restatement of the reference's CPU path (dequantise + fp32 matmul)
            on the host cores, on config 0 (IQ3_S 17408 x 5120, M = 1)

With --gpus N > 1 (one process per GPU under torchrun) the weights are tensor-parallel sharded:
along N for the (*, 5120) shapes with an all-gather of Y, along K (256-column granularity) for
(5120, 17408) with an all-reduce of the partial Y. Total work is fixed ("strong" scaling).

--impl reference times the reference's CPU implementation of the path (oracle port: gguf-py
dequantisation restated in numpy + torch fp32 matmul on all host threads) on a bounded sample.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
for p in (ROOT, os.path.join(ROOT, "vllm-gsqrco-exl3_b200")):
    if p not in sys.path:
        sys.path.insert(0, p)

SHAPES = [(5120, 5120), (17408, 5120), (5120, 17408)]
# DRAM bytes moved per weight byte by the small-batch kernel (profiles/mmv_iq3s_m8.txt: 38.384 MB read, the
# results staying in L2, for 38.298 MB of weights)
NCU_TRAFFIC_RATIO = 1.0023
TYPES = [("IQ3_S", 21), ("Q4_K", 12)]
ROWS = [1, 2, 4, 8, 12, 16, 24, 32, 48]
BLOCK_BYTES = {21: 110, 12: 144, 23: 136, 14: 210}
METRIC = "quant_gemv_weight_GBps_M1-48"


def weight_bytes(t: int, n: int, k: int) -> int:
    return n * (k // 256) * BLOCK_BYTES[t]


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            return json.load(open(p)), "measured"
        except Exception:
            pass
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}, "fallback"


class ClockSampler:
    """nvidia-smi clocks and throttle reasons while the timed region runs."""

    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.samples, self.stop, self.thread = index, [], threading.Event(), None

    def _run(self):
        while not self.stop.is_set():
            try:
                out = subprocess.run(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                      "-i", str(self.index)], capture_output=True, text=True, timeout=5).stdout
                f = [s.strip() for s in out.strip().split(",")]
                if len(f) >= 6:
                    self.samples.append(f)
            except Exception:
                pass
            self.stop.wait(0.2)

    def __enter__(self):
        self.thread = threading.Thread(target=self._run, daemon=True)
        self.thread.start()
        return self

    def __exit__(self, *a):
        self.stop.set()
        self.thread.join(timeout=6)

    def summary(self):
        sm = [int(s[0]) for s in self.samples if s[0].isdigit()]
        mx = [int(s[1]) for s in self.samples if s[1].isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({n for s in self.samples for n, v in zip(names, s[2:6]) if v.lower().startswith("active")})
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(self.samples)}


# --------------------------------------------------------------------------------------------------
# our arm

def shard_plan(n: int, k: int, world: int, rank: int):
    """(mode, start, count) of this rank's tensor-parallel shard (gsq_b200.tp.shard_plan)."""
    from gsq_b200 import tp

    p = tp.shard_plan(n, k, world, rank)
    return p.mode, p.start, p.count


def build_cells(dev, world, rank, l2_bytes):
    import numpy as np
    import torch

    from gsq_b200 import synth
    from gsq_b200.quantization import iq3_pack
    from gsq_b200.quantization.params import GGUFWeightParameter, GGUFWeightTypeParameter

    cells = {}
    for ti, (tname, t) in enumerate(TYPES):
        for si, (n, k) in enumerate(SHAPES):
            mode, a0, cnt = shard_plan(n, k, world, rank)
            raw = synth.make_weight(t, n, k, 1100 + 10 * ti + si)
            if mode == "N":
                raw = raw[a0:a0 + cnt]
                kk = k
            else:
                bs = BLOCK_BYTES[t]
                raw = np.ascontiguousarray(raw[:, a0 * bs:(a0 + cnt) * bs])
                kk = cnt * 256
            w0 = torch.from_numpy(raw).to(dev)
            packed = t == 21 and w0.shape[0] % 16 == 0
            if packed:
                iq3_pack.pack_(w0, t)
            full_bytes = weight_bytes(t, n, k)
            copies = max(2, -(-3 * l2_bytes // max(1, w0.numel())) + 1)
            ws = [w0] + [w0.clone() for _ in range(copies - 1)]
            layers = []
            for w in ws:  # one linear layer per weight copy, as GGUFLinearMethod.apply() expects it
                layer = torch.nn.Module()
                wp = GGUFWeightParameter(w)
                wp.iq3_packed = packed
                layer.register_parameter("weight", wp)
                layer.register_parameter("weight_type", GGUFWeightTypeParameter(t))
                layers.append(layer)
            cells[(tname, n, k)] = dict(t=t, n=n, k=k, kk=kk, mode=mode, a0=a0, cnt=cnt, ws=ws, layers=layers, packed=packed,
                                        bytes=full_bytes, local_rows=w0.shape[0], use=0)
    return cells


def make_inputs(dev, cells, dtype):
    import torch

    from gsq_b200 import synth

    xs = {}
    for (tname, n, k), c in cells.items():
        for m in ROWS:
            if (k, m) not in xs:
                x = torch.from_numpy(synth.make_activation(m, k, 1200 + m)).to(dtype)
                xs[(k, m)] = synth.nudge_ties_torch(x)
    return xs


def run_ours(args):
    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    assert world == args.gpus or world == 1, (world, args.gpus)
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    import gsq_b200  # noqa: F401
    from gsq_b200 import _cabi, lcpp_ops
    from gsq_b200.quantization import linear

    if world > 1:
        lcpp_ops.set_k_multiple(256)
    _cabi.check(_cabi.lib.gsq_device_init(local), "gsq_device_init")
    l2 = torch.cuda.get_device_properties(dev).L2_cache_size
    cells = build_cells(dev, world, rank, l2)
    xs_host = make_inputs(dev, cells, torch.float16)
    xs = {key: v.to(dev) for key, v in xs_host.items()}
    xs_pinned = {key: v.pin_memory() for key, v in xs_host.items()}
    order = [(key, m) for key in cells for m in ROWS]
    launches = {"n": 0}

    method = linear.GGUFLinearMethod(None)

    # Tensor parallel (world > 1): every product writes its shard's result into one of two flat buffers, and the
    # step ends with one all-gather (N-sharded cells: qkv / gate-up style) and one all-reduce (K-sharded cells:
    # o_proj / down style) over them -- the collectives of a step bucketed, as a TP runtime would.
    tp_slots, flat_n, flat_k, gath_n = {}, None, None, None
    if world > 1:
        off_n = off_k = 0
        for key, m in order:
            c = cells[key]
            if c["mode"] == "N":
                tp_slots[(key, m)] = ("N", off_n, m * c["local_rows"])
                off_n += m * c["local_rows"]
            else:
                tp_slots[(key, m)] = ("K", off_k, m * c["n"])
                off_k += m * c["n"]
        flat_n = torch.empty(max(off_n, 1), dtype=torch.float16, device=dev)
        flat_k = torch.empty(max(off_k, 1), dtype=torch.float16, device=dev)
        gath_n = torch.empty(world * flat_n.numel(), dtype=torch.float16, device=dev)

    def product(c, x, key_m=None):
        """One cell: GGUFLinearMethod.apply() on this rank's shard."""
        layer = c["layers"][c["use"] % len(c["layers"])]
        c["use"] += 1
        xl = x if c["mode"] == "N" else x[:, c["a0"] * 256:(c["a0"] + c["cnt"]) * 256]
        y = method.apply(layer, xl)
        m = x.shape[0]
        launches["n"] += 1 + (m + 7) // 8
        if world > 1 and key_m is not None:
            kind, off, cnt = tp_slots[key_m]
            tp_pending.append(((flat_n if kind == "N" else flat_k)[off:off + cnt].view_as(y), y))
        return y

    tp_pending = []   # (slot in a flat buffer, result): copied by one multi-tensor kernel at the end of a step

    def tp_flush():
        if tp_pending:
            torch._foreach_copy_([d for d, _ in tp_pending], [y for _, y in tp_pending])
            tp_pending.clear()

    def collectives():
        if world > 1:
            dist.all_gather_into_tensor(gath_n, flat_n)
            dist.all_reduce(flat_k)

    def compute():
        for key, m in order:
            product(cells[key], xs[(key[2], m)], (key, m))
        tp_flush()

    def step():
        compute()
        collectives()

    # End to end: uploads, products and downloads of a step are pipelined over three streams (upload stream ->
    # event per input -> product on the main stream -> event -> download stream), all inside the timed region.
    s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
    x_dev = [torch.empty_like(xs[(key[2], m)]) for key, m in order]

    def compute_e2e(outs):
        cur = torch.cuda.current_stream()
        s_in.wait_stream(cur)
        s_out.wait_stream(cur)
        ready = []
        with torch.cuda.stream(s_in):
            for i, (key, m) in enumerate(order):
                x_dev[i].copy_(xs_pinned[(key[2], m)], non_blocking=True)
                e = torch.cuda.Event()
                e.record(s_in)
                ready.append(e)
        keep = []   # results stay referenced until the streams have joined: their memory is not reused under a copy
        for i, (key, m) in enumerate(order):
            cur.wait_event(ready[i])
            y = product(cells[key], x_dev[i], (key, m))
            if world == 1:
                e = torch.cuda.Event()
                e.record(cur)
                s_out.wait_event(e)
                with torch.cuda.stream(s_out):
                    outs[i].copy_(y, non_blocking=True)
                keep.append(y)
        tp_flush()
        cur.wait_stream(s_in)
        cur.wait_stream(s_out)
        del keep

    def step_e2e(outs):
        compute_e2e(outs)
        if world > 1:  # the step's results are the two collective buffers
            collectives()
            outs[0][:gath_n.numel()].copy_(gath_n, non_blocking=True)
            outs[0][gath_n.numel():gath_n.numel() + flat_k.numel()].copy_(flat_k, non_blocking=True)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        barrier()
        ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    def capture(fn):
        """fn's launches as one CUDA graph (what vLLM does with the decode step it wraps around apply())."""
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            fn()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            fn()
        return g

    # The products (and, end to end, the copies) are replayed as one CUDA graph, as vLLM runs decode. NCCL
    # collectives stay outside the graph (captured together with the products they hung a 2-GPU run).
    use_graph = not args.eager
    for _ in range(max(3, args.warmup)):
        step()
    runner = step
    if use_graph:
        g_step = capture(compute)

        def runner():
            g_step.replay()
            collectives()
        for _ in range(3):
            runner()
    launches["n"] = 0
    step()                                      # count this step's launches once, untimed
    n_launch = launches["n"] * args.steps
    with ClockSampler(local) as clk:
        ms = timed(runner, args.steps)
    step_bytes = sum(cells[key]["bytes"] for key, _ in order)
    value = step_bytes * args.steps / (ms * 1e-3) / 1e9

    # end to end through GGUFLinearMethod.apply() with host buffers (pinned), copies inside the timed region
    if world == 1:
        outs = [torch.empty(m, cells[key]["n"], dtype=torch.float16).pin_memory() for key, m in order]
    else:
        outs = [torch.empty(gath_n.numel() + flat_k.numel(), dtype=torch.float16).pin_memory()]
    for _ in range(3):
        step_e2e(outs)
    ms_e2e_eager = timed(lambda: step_e2e(outs), args.steps)
    ms_e2e = ms_e2e_eager
    if use_graph:
        if world == 1:
            g_e2e = capture(lambda: step_e2e(outs))
            run_e2e = g_e2e.replay
        else:
            g_e2e = capture(lambda: compute_e2e(outs))

            def run_e2e():
                g_e2e.replay()
                collectives()
                outs[0][:gath_n.numel()].copy_(gath_n, non_blocking=True)
                outs[0][gath_n.numel():gath_n.numel() + flat_k.numel()].copy_(flat_k, non_blocking=True)
        for _ in range(3):
            run_e2e()
        ms_e2e = timed(run_e2e, args.steps)
    e2e = step_bytes * args.steps / (ms_e2e * 1e-3) / 1e9
    h2d = sum(m * key[2] * 2 for key, m in order)
    d2h = sum(m * cells[key]["n"] * 2 for key, m in order)

    # per-cell table and the GEMV kernel's roofline (this rank's shard; kernel alone, x already quantised).
    # Each cell: `reps` calls on successive weight copies in one graph, best of 3 replays.
    cell_rows, roof_bytes, roof_ms, roof_launches = [], 0, 0.0, 0
    peaks, peak_kind = measured_peaks()
    reps = 10

    def best_us(fn):
        if args.eager:
            for _ in range(3):
                fn()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(reps):
                fn()
            e1.record()
            torch.cuda.synchronize()
            return e0.elapsed_time(e1) * 1e3 / reps

        def many():
            for _ in range(reps):
                fn()
        g = capture(many)
        best = 1e30
        for _ in range(3):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            g.replay()
            e1.record()
            torch.cuda.synchronize()
            best = min(best, e0.elapsed_time(e1) * 1e3 / reps)
        return best

    for key, m in order:
        c = cells[key]
        x = xs[(key[2], m)]
        xl = x if c["mode"] == "N" else x[:, c["a0"] * 256:(c["a0"] + c["cnt"]) * 256].contiguous()
        us = best_us(lambda: product(c, x))
        row = {"type": key[0], "n": key[1], "k": key[2], "m": m, "us": round(us, 2),
               "GBps": round(c["bytes"] / us / 1e3, 1)}
        if m <= 8:
            xq = torch.ops._C_gguf.lcpp_quantize_q8_1(xl, c["t"], False, False)
            name = linear._lcpp_op(m, c["t"], c["local_rows"], c["kk"], c["packed"])
            op = getattr(torch.ops._C_gguf, name if name not in linear._OWN_QUANTIZE_OPS else "lcpp_mul_mat_vec_q")

            def kernel_only():
                w = c["ws"][c["use"] % len(c["ws"])]
                c["use"] += 1
                op(w, xl, c["t"], c["local_rows"], xq)
            kus = best_us(kernel_only)
            local_bytes = c["ws"][0].numel()
            row["kernel_us"] = round(kus, 2)
            row["kernel_GBps"] = round(local_bytes / kus / 1e3, 1)
            roof_bytes += local_bytes * reps
            roof_ms += kus * reps / 1e3
            roof_launches += reps
        cell_rows.append(row)

    if rank == 0:
        achieved = roof_bytes / (roof_ms * 1e-3) / 1e9 if roof_ms else None
        out = {
            "metric": METRIC, "value": round(value, 1), "unit": "GB/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(3, args.warmup), "ms_per_step": round(ms / args.steps, 4), "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "int8", "data": "synthetic",
            "config": {"workload": "gemv_row_sweep", "types": [t for t, _ in TYPES], "shapes": SHAPES, "rows": ROWS,
                       "x_dtype": "fp16", "l2_defeat": "weight copies cycled, > 3 x L2 between reuses",
                       "launch": ("cuda graph replay of one step" + (" + one all-gather and one all-reduce over the step's outputs"
                                                                    if world > 1 else "")) if use_graph else "eager",
                       "parallelism": "tp%d" % world if world > 1 else "single"},
            "clocks": clk.summary(),
            "e2e": {"value": round(e2e, 1), "unit": "GB/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "ms_per_step": round(ms_e2e / args.steps, 4),
                    "eager_ms_per_step": round(ms_e2e_eager / args.steps, 4),
                    "launch": ("cuda graph replay of apply() + copies, uploads / products / downloads on three streams"
                               + (", collectives and result copies eager" if world > 1 else ""))
                    if use_graph else "eager"},
            "gpu_launches": n_launch,
            "roofline": {"bound": "hbm", "achieved": round(achieved, 1) if achieved else None,
                         "peak": peaks["hbm_gbs"], "unit": "GB/s",
                         "frac": round(achieved / peaks["hbm_gbs"], 4) if achieved else None,
                         "traffic": int(roof_bytes // max(1, roof_launches) * NCU_TRAFFIC_RATIO), "peak_kind": peak_kind,
                         "traffic_source": "dram__bytes_read+write of one ncu capture of mmv_kernel (IQ3_S 17408x5120, "
                                           "8 rows) over its weight bytes, applied to the average launch",
                         "kernel": "mmv_kernel (2-8 rows, IQ3_S at 1 row) and gemv_kernel (Q4_K at 1 row)",
                         "bytes_per_launch": roof_bytes // max(1, roof_launches),
                         "avg_launch_us": round(roof_ms * 1e3 / max(1, roof_launches), 2)},
            "cells": cell_rows,
        }
        out["config"]["cells"] = len(order)
        if world == 1 and not args.no_extras:
            del cells, xs
            torch.cuda.empty_cache()
            out["prefill"] = extra_prefill(dev, capture)
            out["decode_stack"] = extra_decode_stack(dev, capture)
        if world == 1 and not args.no_cpu_baseline:
            out["cpu_baseline"] = cpu_baseline()
        print(json.dumps(out), flush=True)
    if world > 1:
        dist.destroy_process_group()



# --------------------------------------------------------------------------------------------------
# the other two quantities BASELINE.json's metric names, reported beside the headline (1 GPU)

def extra_prefill(dev, capture):
    """Prefill GEMM: M tokens x K=5120 -> N=17408 with IQ3_S weights, and M x K=17408 -> N=5120 with IQ4_XS;
    bf16 activations ~ N(0,1) with 0.1 % outliers x20. Algorithmic ops = 2 M N K."""
    import torch

    from gsq_b200 import synth
    from gsq_b200.quantization import iq3_pack, linear

    out = []
    for tname, t, n, k in (("IQ3_S", 21, 17408, 5120), ("IQ4_XS", 23, 5120, 17408)):
        w = torch.from_numpy(synth.make_weight(t, n, k, 1300)).to(dev)
        packed = t == 21
        if packed:
            iq3_pack.pack_(w, t)
        for m in (2048, 8192):
            x = torch.from_numpy(synth.make_activation(m, k, 1400 + m, outliers=1e-3)).to(torch.bfloat16).to(dev)
            fn = lambda: linear.fused_mul_mat_gguf(x, w, t, None, packed)
            for _ in range(2):
                fn()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(3):
                fn()
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1) / 3
            out.append({"type": tname, "m": m, "n": n, "k": k, "ms": round(ms, 3),
                        "int8_TOPS": round(2.0 * m * n * k / (ms * 1e-3) / 1e12, 1)})
            del x
        del w
    return out


def extra_decode_stack(dev, capture, layers=64):
    """64-layer dense decoder stack, linears only: per layer qkv IQ3_S 7168x5120, o_proj IQ3_S 5120x5120,
    gate_up IQ3_S 34816x5120, down IQ4_XS 5120x17408 (150,978,560 weight bytes per layer, distinct weights per
    layer so L2 cannot hold them); rows per step 4 / 8 / 16 / 32; one CUDA graph per step."""
    import torch

    from gsq_b200 import synth
    from gsq_b200.quantization import iq3_pack, linear

    shapes = [("qkv", 21, 7168, 5120), ("o", 21, 5120, 5120), ("gate_up", 21, 34816, 5120), ("down", 23, 5120, 17408)]
    base = {}
    for name, t, n, k in shapes:
        w = torch.from_numpy(synth.make_weight(t, n, k, 2000 + len(base))).to(dev)
        if t == 21:
            iq3_pack.pack_(w, t)
        base[name] = w
    # distinct bytes per layer: each layer's copy is the base tile rolled by a layer-dependent row count
    stack = [{name: torch.roll(base[name], shifts=16 * (l + 1), dims=0) if l else base[name] for name, *_ in shapes}
             for l in range(layers)]
    bytes_step = layers * sum(base[name].numel() for name, *_ in shapes)
    res = []
    for rows in (4, 8, 16, 32):
        x5 = torch.randn(rows, 5120, device=dev, dtype=torch.bfloat16)
        x17 = torch.randn(rows, 17408, device=dev, dtype=torch.bfloat16)

        def step():
            for lw in stack:
                linear.fused_mul_mat_gguf(x5, lw["qkv"], 21, None, True)
                linear.fused_mul_mat_gguf(x5, lw["o"], 21, None, True)
                linear.fused_mul_mat_gguf(x5, lw["gate_up"], 21, None, True)
                linear.fused_mul_mat_gguf(x17, lw["down"], 23, None, False)
        g = capture(step)
        best = 1e30
        for _ in range(3):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            g.replay()
            e1.record()
            torch.cuda.synchronize()
            best = min(best, e0.elapsed_time(e1))
        res.append({"rows": rows, "ms_per_step": round(best, 3), "GBps": round(bytes_step / best / 1e6, 1),
                    "floor_ms_at_measured_hbm": round(bytes_step / 6547.2e6, 3)})
    return {"layers": layers, "weight_bytes_per_step": bytes_step, "steps": res}

# --------------------------------------------------------------------------------------------------
# CPU baseline / reference arm (the only places bench.py executes oracle/)

def cpu_baseline(rows: int = 17408, k: int = 5120, m: int = 1):
    import numpy as np
    import torch

    from gsq_b200 import synth
    from oracle import product

    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    raw = synth.make_weight(21, rows, k, 1000)
    x = synth.make_activation(m, k, 1001)
    _, t_deq, t_mm = product.cpu_reference_linear(raw, 21, x, cores)
    gbs = raw.nbytes / (t_deq + t_mm) / 1e9
    return {"value": round(gbs, 4), "unit": "GB/s", "cores": cores, "kind": "port",
            "sample": f"config 0: IQ3_S {rows}x{k}, M={m}, one product (dequantise {t_deq:.2f} s in numpy, "
                      f"1 thread; fp32 matmul {t_mm:.3f} s, {cores} threads)"}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    steps = max(1, args.steps)
    vals = []
    for _ in range(max(0, min(args.warmup, 1))):
        cpu_baseline(rows=2048)
    t0 = time.perf_counter()
    for _ in range(steps):
        b = cpu_baseline(rows=4352)   # a quarter of config 0's rows per step keeps K steps within minutes
        vals.append(b["value"])
    dt = time.perf_counter() - t0
    v = statistics.mean(vals)
    b["value"] = round(v, 4)
    b["sample"] = "per step: IQ3_S 4352x5120 (a quarter of config 0), M=1; " + b["sample"].split(", one product ")[1]
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": round(v, 4), "unit": "GB/s", "n_gpus": args.gpus, "steps": steps,
        "warmup": min(args.warmup, 1), "ms_per_step": round(dt / steps * 1e3, 1), "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "gemv_row_sweep", "note": "CPU path of the reference: dequantise + fp32 matmul"},
        "cpu_baseline": b,
        "e2e": {"value": round(v, 4), "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true", help="skip the prefill-TOPS and decode-stack measurements")
    ap.add_argument("--eager", action="store_true", help="time eager launches instead of CUDA-graph replays")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
