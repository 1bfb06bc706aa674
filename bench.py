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

Before anything is timed every cell's output is compared once, on 64 sampled weight rows, with the CPU
oracle (`parity_checked`), and every cell's graph replay is compared bit for bit with the eager call
(`graph_exact`). `ref_kernels` times the reference's own CUDA kernels (oracle/_ref, built from the reference
tree for sm_100a; a process of its own) on the same cells by the same method.

--impl reference times the reference's CPU path (gguf-py dequantisation, which the reference's tests use as
their CPU model, + torch fp32 matmul on all host threads) on a bounded sample of the same workload.

--cell TYPE N K M runs one product a few times on distinct weight copies (for profilers).
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
            raw_host = raw
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
                                        bytes=full_bytes, local_rows=w0.shape[0], use=0, raw=raw_host)
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

    def product(c, x, key_m=None, sliced=False):
        """One cell: GGUFLinearMethod.apply() on this rank's shard. sliced: x is already the K-shard's columns."""
        layer = c["layers"][c["use"] % len(c["layers"])]
        c["use"] += 1
        xl = x if (c["mode"] == "N" or sliced) else x[:, c["a0"] * 256:(c["a0"] + c["cnt"]) * 256]
        m = x.shape[0]
        launches["n"] += 1 + (m + 7) // 8
        if world > 1 and key_m is not None:
            # the kernel writes the shard's result straight into its slot of the step's collective buffer
            kind, off, cnt = tp_slots[key_m]
            slot = (flat_n if kind == "N" else flat_k)[off:off + cnt].view(m, -1)
            with lcpp_ops.output_into(slot):
                return method.apply(layer, xl)
        return method.apply(layer, xl)

    def tp_flush():
        pass

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

    def x_slice(key, m, t):
        """The columns of the activation this rank needs: all of them for an N-shard, its K range for a K-shard."""
        c = cells[key]
        return t if c["mode"] == "N" else t[:, c["a0"] * 256:(c["a0"] + c["cnt"]) * 256]
    xs_pinned = {(key, m): x_slice(key, m, xs_host[(key[2], m)]).contiguous().pin_memory() for key, m in order}
    x_dev = [torch.empty_like(xs_pinned[(key, m)], device=dev) for key, m in order]

    def compute_e2e(outs):
        cur = torch.cuda.current_stream()
        s_in.wait_stream(cur)
        s_out.wait_stream(cur)
        ready = []
        with torch.cuda.stream(s_in):
            for i, (key, m) in enumerate(order):
                x_dev[i].copy_(xs_pinned[(key, m)], non_blocking=True)
                e = torch.cuda.Event()
                e.record(s_in)
                ready.append(e)
        keep = []   # results stay referenced until the streams have joined: their memory is not reused under a copy
        for i, (key, m) in enumerate(order):
            cur.wait_event(ready[i])
            y = product(cells[key], x_dev[i], (key, m), sliced=True)
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

    # Checker leg (untimed, before anything is measured): every cell's output against the CPU oracle on 64 sampled
    # weight rows, and every cell's graph replay against its eager call, bit for bit.
    parity, exact = {}, {}
    if world == 1 and not args.no_check:
        parity, exact = check_cells(cells, xs, xs_host, order, product, capture)

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
    h2d = sum(v.numel() * 2 for v in xs_pinned.values())
    d2h = sum(m * cells[key]["n"] * 2 for key, m in order)

    # per-cell table and the small-batch kernel's roofline (this rank's shard; kernel alone, x already quantised).
    # Each cell: one call per weight copy in one graph (a copy is read again only after all the others, more than
    # 3 x L2 later, also across replays), best of 3 replays.
    cell_rows, roof_bytes, roof_ms, roof_launches = [], 0, 0.0, 0
    peaks, peak_kind = measured_peaks()

    def best_us(fn, reps):
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
        reps = len(c["ws"])
        us = best_us(lambda: product(c, x), reps)
        row = {"type": key[0], "n": key[1], "k": key[2], "m": m, "us": round(us, 2),
               "GBps": round(c["bytes"] / us / 1e3, 1), "graph_exact": exact.get((key, m)),
               "parity_rel_err": parity.get((key, m))}
        if m <= 8:
            xq = torch.ops._C_gguf.lcpp_quantize_q8_1(xl, c["t"], False, False)
            name = linear._lcpp_op(m, c["t"], c["local_rows"], c["kk"], c["packed"])
            op = getattr(torch.ops._C_gguf, name if name not in linear._OWN_QUANTIZE_OPS else "lcpp_mul_mat_vec_q")

            def kernel_only():
                w = c["ws"][c["use"] % len(c["ws"])]
                c["use"] += 1
                op(w, xl, c["t"], c["local_rows"], xq)
            kus = best_us(kernel_only, reps)
            local_bytes = c["ws"][0].numel()
            row["kernel_us"] = round(kus, 2)
            row["kernel_GBps"] = round(local_bytes / kus / 1e3, 1)
            roof_bytes += local_bytes * reps
            roof_ms += kus * reps / 1e3
            roof_launches += reps
        cell_rows.append(row)

    tp_stack = None
    if world > 1 and not args.no_extras:
        del cells, xs
        torch.cuda.empty_cache()
        tp_stack = extra_tp_stack(dev, world, rank, capture)
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
        if parity:
            worst = max(parity.values())
            out["parity_checked"] = bool(worst <= PARITY_TOL)
            out["parity"] = {"against": "CPU oracle (oracle.product: exact int32 slice sums, q8_1 model of the reference "
                                        "kernels) on 64 sampled weight rows per cell", "cells": len(parity),
                             "max_rel_err": worst, "tolerance": PARITY_TOL}
            out["graph_exact"] = "%d/%d" % (sum(1 for v in exact.values() if v), len(exact))
        else:
            out["parity_checked"] = False
        if tp_stack is not None:
            out["tp_decode_stack"] = tp_stack
        raws = {key: c["raw"] for key, c in cells.items()} if world == 1 else {}
        if world == 1 and not args.no_extras:
            del cells, xs
            torch.cuda.empty_cache()
            out["prefill"] = extra_prefill(dev, capture, l2, not args.no_ref_kernels)
            out["decode_stack"] = extra_decode_stack(dev, capture)
            out["low_bit_types"] = extra_low_bit(dev, capture, l2)
            out["fused_steps"] = extra_fused_steps(dev, capture)
            out["embedding"] = extra_embedding(dev, capture)
            out["gguf_load"] = extra_gguf_load(dev)
        if world == 1 and not args.no_ref_kernels:
            out["ref_kernels"] = ref_kernels(cell_rows, raws, l2)
        if world == 1 and not args.no_cpu_baseline:
            out["cpu_baseline"] = cpu_baseline()
        print(json.dumps(out), flush=True)
    if world > 1:
        dist.destroy_process_group()



# --------------------------------------------------------------------------------------------------
# checker leg (untimed; the only part of the GPU arm that imports oracle/)

PARITY_TOL = 2e-3   # 1e-3 of the reference kernels' model + the fp16 rounding of the outputs


def check_cells(cells, xs, xs_host, order, product, capture):
    """({cell: rel_err vs the CPU oracle on 64 sampled weight rows}, {cell: graph replay == eager})."""
    import numpy as np
    import torch

    from gsq_b200.quantization import linear
    from oracle import blocks, product as oproduct, q8_1

    parity, exact, dec_cache = {}, {}, {}
    for key, m in order:
        c = cells[key]
        t, n, k = c["t"], c["n"], c["k"]
        if key not in dec_cache:
            rows = np.unique(np.concatenate([np.linspace(0, n - 1, 56).astype(np.int64), np.arange(n - 8, n)]))
            dec_cache[key] = (rows, blocks.decode(np.ascontiguousarray(c["raw"][rows]), t))
        rows, dec = dec_cache[key]
        x = xs[(k, m)]
        y = product(c, x)
        torch.cuda.synchronize()
        xf = xs_host[(k, m)].float().numpy()
        op = linear._lcpp_op(m, t, n, k, c["packed"])
        if op in linear._OWN_QUANTIZE_OPS:     # 128-value activation blocks; Q4_K's min term from the stored sums
            if t == 12:
                q, d, sm = q8_1.quantize_mmq(xf, q8_1.LAYOUT_DS4)
                ref = oproduct.product_xsum(dec, q, d.astype(np.float16).astype(np.float64),
                                            sm.astype(np.float16).astype(np.float64))
            else:
                q, d, _ = q8_1.quantize_mmq(xf, q8_1.LAYOUT_D4)
                ref = oproduct.product_q81(dec, q, d)
        else:
            q, d, _ = q8_1.quantize_q8_1(xf)
            ref = oproduct.product_q81(dec, q, d.astype(np.float32))
        got = y.float().cpu().numpy()[:, rows]
        parity[(key, m)] = round(oproduct.rel_err(got, ref), 7)
        # graph replay of the same call, on the same weight copy, bit for bit
        c["use"] -= 1
        holder = {}

        def once():
            holder["y"] = product(c, x)
        use0 = c["use"]
        g = capture(once)
        c["use"] = use0 + 1
        g.replay()
        torch.cuda.synchronize()
        exact[(key, m)] = bool(torch.equal(holder["y"], y))
        del g
    return parity, exact


def ref_kernels(cell_rows, raws, l2_bytes, types=None):
    """The reference's own CUDA kernels (oracle/_ref/ref_C_gguf.so, the routed op of each cell on GGUF-order bytes;
    for IQ3_S also its packed route, timed on the same bytes: same traffic, meaningless values) in a process of
    their own, timed like the cells above: one call per weight copy in one graph, best of 3 replays."""
    import tempfile

    import torch

    from gsq_b200.quantization import linear

    so = os.path.join(ROOT, "oracle", "_ref", "ref_C_gguf.so")
    if not os.path.exists(so):
        return {"unavailable": "oracle/_ref/ref_C_gguf.so not built (oracle/build_ref.py needs the reference tree)"}
    tens = {key: torch.from_numpy(r) for key, r in raws.items()}
    xs, cases, tags = {}, [], []
    for row in cell_rows:
        key = (row["type"], row["n"], row["k"])
        t = (types or dict(TYPES))[row["type"]]
        m, n, k = row["m"], row["n"], row["k"]
        if (k, m) not in xs:
            from gsq_b200 import synth
            xs[(k, m)] = torch.from_numpy(synth.make_activation(m, k, 1200 + m)).half()
        copies = max(2, -(-3 * l2_bytes // tens[key].numel()) + 1)
        for packed in ([False, True] if t == 21 else [False]):
            op = linear._lcpp_op(m, t, n, k, packed)
            a = [tens[key], xs[(k, m)], t, n] + ([] if op in linear._OWN_QUANTIZE_OPS else [None])
            cases.append({"op": op, "args": a, "time": True, "copies": copies, "no_out": True})
            tags.append((row, op, packed))
    with tempfile.TemporaryDirectory() as td:
        cin, cout = os.path.join(td, "cases.pt"), os.path.join(td, "res.pt")
        torch.save(cases, cin)
        del cases
        p = subprocess.run([sys.executable, os.path.join(ROOT, "oracle", "ref_runner.py"), cin, cout],
                           capture_output=True, text=True, timeout=1500)
        if p.returncode != 0:
            return {"unavailable": "reference kernels failed: " + p.stderr.strip().splitlines()[-1][:300]}
        res = torch.load(cout)
    best = {}
    for (row, op, packed), r in zip(tags, res):
        k = (row["type"], row["n"], row["k"], row["m"])
        if k not in best or r["us"] < best[k]["us"]:
            best[k] = {"us": r["us"], "op": op + (" (packed)" if packed else "")}
    out_cells, ahead = [], 0
    for row in cell_rows:
        b = best[(row["type"], row["n"], row["k"], row["m"])]
        sp = b["us"] / row["us"]
        ahead += sp >= 1.0
        out_cells.append({"type": row["type"], "n": row["n"], "k": row["k"], "m": row["m"], "ref_us": round(b["us"], 2),
                          "ref_op": b["op"], "us": row["us"], "speedup": round(sp, 3)})
    tot_ref = sum(c["ref_us"] for c in out_cells)
    tot = sum(c["us"] for c in out_cells)
    return {"what": "reference kernels rebuilt for sm_100a, same cells, quantise + product per call, graph replay, "
                    "weight copies cycled beyond 3 x L2; for IQ3_S the faster of its packed and unpacked routes",
            "cells_ahead": "%d/%d" % (ahead, len(out_cells)), "sum_ref_us": round(tot_ref, 1), "sum_us": round(tot, 1),
            "speedup_sum": round(tot_ref / tot, 3), "cells": out_cells}


# --------------------------------------------------------------------------------------------------
# the other two quantities BASELINE.json's metric names, reported beside the headline (1 GPU)

def int8_peak(dev):
    """Dense int8 tensor-core rate of this GPU as a library GEMM reaches it (torch._int_mm 8192^3, best of 5), the
    way the reference's kit/micro_gguf.py:134-161 measures its card: the measured denominator beside the nominal one."""
    import torch

    try:
        a = torch.randint(-127, 127, (8192, 8192), dtype=torch.int8, device=dev)
        b = torch.randint(-127, 127, (8192, 8192), dtype=torch.int8, device=dev)
        for _ in range(2):
            torch._int_mm(a, b)
        best = 1e30
        for _ in range(5):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            torch._int_mm(a, b)
            e1.record()
            torch.cuda.synchronize()
            best = min(best, e0.elapsed_time(e1))
        return round(2.0 * 8192 ** 3 / (best * 1e-3) / 1e12, 1)
    except Exception as e:  # noqa: BLE001
        return None


NOMINAL_INT8_TOPS = 4500.0


def extra_prefill(dev, capture, l2_bytes, with_ref=True):
    """Prefill GEMM: M tokens x K=5120 -> N=17408 with IQ3_S weights, M x K=17408 -> N=5120 with IQ4_XS (the two products
    of the prefill configuration), and M x K=5120 -> N=17408 with Q4_K;
    bf16 activations ~ N(0,1) with 0.1 % outliers x20, M in {2048, 8192, 16384}. Algorithmic ops = 2 M N K."""
    import torch

    from gsq_b200 import synth
    from gsq_b200.quantization import iq3_pack, linear

    peak = int8_peak(dev)
    rows = []
    from gsq_b200 import lcpp_ops

    def timed(fn):
        for _ in range(2):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(3):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / 3

    raws, ref_rows = {}, []
    for tname, t, n, k in (("IQ3_S", 21, 17408, 5120), ("IQ4_XS", 23, 5120, 17408), ("Q4_K", 12, 17408, 5120)):
        raws[(tname, n, k)] = synth.make_weight(t, n, k, 1300)
        w = torch.from_numpy(raws[(tname, n, k)]).to(dev)
        packed = t == 21
        if packed:
            iq3_pack.pack_(w, t)
        for m in (2048, 8192, 16384):
            x = torch.from_numpy(synth.make_activation(m, k, 1400 + m, outliers=1e-3)).to(torch.bfloat16).to(dev)
            fn = lambda: linear.fused_mul_mat_gguf(x, w, t, None, packed)
            ms = timed(fn)
            tops = 2.0 * m * n * k / (ms * 1e-3) / 1e12
            row = {"type": tname, "m": m, "n": n, "k": k, "ms": round(ms, 3), "int8_TOPS": round(tops, 1),
                   "frac_nominal": round(tops / NOMINAL_INT8_TOPS, 4),
                   "frac_measured": round(tops / peak, 4) if peak else None,
                   "frac_nominal_f16": round(tops / 2250.0, 4)}
            # the other forms of this product (gsq_prefill_precision), and how far the default is from the one that keeps
            # the reference's exact integer slice sums, relative to the result's norm (IQ4_XS, Q4_K: split = integer)
            row["form"] = "rounded (default)"
            xf = x.float() if m == 2048 else None        # fp32 in, fp32 out: no output rounding in the comparison
            cmp_fn = lambda: linear.fused_mul_mat_gguf(xf, w, t, None, packed)
            ys = {"rounded": cmp_fn()} if m == 2048 else {}
            for name, mode in ((("split", lcpp_ops.PREFILL_SPLIT),) if packed else ()) + (("integer", lcpp_ops.PREFILL_INTEGER),):
                lcpp_ops.set_prefill_precision(mode)
                try:
                    row[name + "_TOPS"] = round(2.0 * m * n * k / (timed(fn) * 1e-3) / 1e12, 1)
                    if m == 2048:
                        ys[name] = cmp_fn()
                finally:
                    lcpp_ops.set_prefill_precision(lcpp_ops.PREFILL_ROUNDED)
            if m == 2048:
                rel = lambda a, b: float(((ys[a] - ys[b]).norm() / ys[b].norm()).item())
                row["rounded_vs_integer"] = rel("rounded", "integer")
                if packed:
                    row["split_vs_integer"] = rel("split", "integer")
            del ys, xf
            rows.append(row)
            if m == 2048:
                ref_rows.append({"type": tname, "n": n, "k": k, "m": m, "us": round(ms * 1e3, 1)})
            del x
        del w
    torch.cuda.empty_cache()
    # the reference's own many-row kernels (its MMQ; for IQ3_S also its packed route) on the 2048-token cells
    ref = ref_kernels(ref_rows, raws, l2_bytes, {"IQ3_S": 21, "IQ4_XS": 23, "Q4_K": 12}) if with_ref else {"skipped": "--no-ref-kernels"}
    if "cells" in ref:
        ref["what"] = "reference kernels rebuilt for sm_100a on the 2048-token cells, quantise + product per call, graph replay"
        for c in ref["cells"]:
            c["ref_TOPS"] = round(2.0 * c["m"] * c["n"] * c["k"] / c["ref_us"] / 1e6, 1)
    return {"int8_peak_nominal_TOPS": NOMINAL_INT8_TOPS, "int8_peak_measured_TOPS": peak,
            "int8_peak_how": "torch._int_mm 8192^3, best of 5", "includes": "activation quantisation + GEMM per call",
            "operands": "ops = 2 M N K whatever the operand type; the default (rounded) and split forms run on fp16 tensor-core "
                        "operands (tcgen05 kind::f16, nominal dense peak 2250 TFLOP/s: frac_nominal_f16), the integer form of IQ4_XS and Q4_K on int8",
            "cells": rows, "ref_kernels": ref}


LOW_BIT_TYPES = [("Q2_K", 10), ("IQ2_XXS", 16), ("IQ2_XS", 17), ("IQ3_XXS", 18), ("IQ2_S", 22), ("IQ1_M", 29)]


def extra_low_bit(dev, capture, l2_bytes):
    """The six low-bit types the model file mixes with the main four (GGUF order, dp4a kernel): 17408 x 5120 at 1 and
    8 activation rows, quantise + product per call, one graph over weight copies cycled beyond 3 x L2, best of 3
    replays; and the reference's own kernel for the same cells (its stock MMVQ route) where oracle/_ref is built."""
    import torch

    from gsq_b200 import synth
    from gsq_b200.quantization import linear

    n, k = 17408, 5120
    rows, raws = [], {}
    for tname, t in LOW_BIT_TYPES:
        raw = synth.make_weight(t, n, k, 1700 + t)
        raws[(tname, n, k)] = raw
        w0 = torch.from_numpy(raw).to(dev)
        copies = max(2, -(-3 * l2_bytes // w0.numel()) + 1)
        ws = [w0] + [w0.clone() for _ in range(copies - 1)]
        for m in (1, 8):
            x = synth.nudge_ties_torch(torch.from_numpy(synth.make_activation(m, k, 1200 + m)).half()).to(dev)

            def many():
                for w in ws:
                    linear.fused_mul_mat_gguf(x, w, t, None, False)
            g = capture(many)
            best = 1e30
            for _ in range(3):
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                g.replay()
                e1.record()
                torch.cuda.synchronize()
                best = min(best, e0.elapsed_time(e1) * 1e3 / len(ws))
            rows.append({"type": tname, "n": n, "k": k, "m": m, "us": round(best, 2), "GBps": round(w0.numel() / best / 1e3, 1)})
            del g
        del ws, w0
        torch.cuda.empty_cache()
    ref = ref_kernels(rows, raws, l2_bytes, dict(LOW_BIT_TYPES))
    return {"what": "GGUF-order dp4a kernel, 8 activation rows per launch; weight GB/s = weight bytes / time", "cells": rows,
            "ref_kernels": {k2: v for k2, v in ref.items() if k2 != "cells"} if "cells" in ref else ref,
            "ref_cells": ref.get("cells")}


def extra_embedding(dev, capture):
    """Quantised embedding look-up: 2048 and 8 token ids into a [151936, 5120] table (Q6_K and IQ2_S, the two types the
    model file uses for it), bf16 output; one kernel gathers and dequantises (gsq_dequantize_rows)."""
    import torch

    from gsq_b200 import synth
    from gsq_b200.quantization import vocab_embeds

    vocab, k = 151936, 5120
    rows = []
    for tname, t in (("Q6_K", 14), ("IQ2_S", 22)):
        small = torch.from_numpy(synth.make_weight(t, 4096, k, 3300 + t)).to(dev)
        table = small.repeat(vocab // 4096 + 1, 1)[:vocab].contiguous()      # seeded blocks, tiled to the table's size
        del small
        for n in (8, 2048):
            ids = torch.randint(0, vocab, (n,), device=dev)
            fn = lambda: vocab_embeds.apply_gguf_embedding(ids, table, t, k, torch.bfloat16)
            g = capture(lambda: [fn() for _ in range(8)])
            best = 1e30
            for _ in range(3):
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                g.replay()
                e1.record()
                torch.cuda.synchronize()
                best = min(best, e0.elapsed_time(e1) * 1e3 / 8)
            del g
            moved = n * (table.shape[1] + k * 2)
            rows.append({"type": tname, "tokens": n, "us": round(best, 2), "GBps_read_plus_written": round(moved / best / 1e3, 1)})
        del table
        torch.cuda.empty_cache()
    return {"what": "ids -> [tokens, 5120] bf16 from a 151936-row quantised table, gather + dequantise in one kernel", "cells": rows}


def extra_gguf_load(dev):
    """GGUF file -> GPU layers (gsq_b200.gguf_load): a synthetic file of 8 IQ3_S [17408, 5120] and 2 Q6_K [16384, 5120]
    tensors written to the local temp directory, then loaded as single-tensor layers (memory-mapped read, pinned staging,
    device copy, in-place GPU repack); seconds and GB/s of file bytes."""
    import tempfile

    import numpy as np
    import torch

    try:
        import gguf
    except Exception as e:  # noqa: BLE001
        return {"unavailable": "gguf python package: " + str(e)[:100]}
    from gsq_b200 import gguf_load, synth

    with tempfile.TemporaryDirectory() as td:
        path = os.path.join(td, "synthetic.gguf")
        w = gguf.GGUFWriter(path, "gsq-synthetic")
        names, total = [], 0
        base3 = synth.make_weight(21, 17408, 5120, 3400)
        base6 = synth.make_weight(14, 16384, 5120, 3401)
        for i in range(8):
            names.append(f"blk.{i}.ffn_gate.weight")
            w.add_tensor(names[-1], np.roll(base3, 16 * i, axis=0), raw_dtype=gguf.GGMLQuantizationType(21))
            total += base3.nbytes
        for i in range(2):
            names.append(f"blk.{i}.attn_output.weight")
            w.add_tensor(names[-1], np.roll(base6, 16 * i, axis=0), raw_dtype=gguf.GGMLQuantizationType(14))
            total += base6.nbytes
        w.write_header_to_file()
        w.write_kv_data_to_file()
        w.write_tensors_to_file()
        w.close()
        tens = gguf_load.tensors(path)
        stager = gguf_load._Stager(dev)
        gguf_load.load_linear(tens, [names[0]], dev, torch.bfloat16, stager)      # warm-up: kernels, pinned buffer
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        layers = [gguf_load.load_linear(tens, [n], dev, torch.bfloat16, stager) for n in names]
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        packed = sum(1 for l, _ in layers if getattr(l.weight, "iq3_packed", False))
    return {"what": "10 tensors (8 IQ3_S 17408 x 5120, 2 Q6_K 16384 x 5120) from a GGUF file in the page cache to repacked GPU "
                    "layers", "file_bytes": total, "seconds": round(dt, 4), "GBps": round(total / dt / 1e9, 2), "layers_repacked": packed}


def extra_fused_steps(dev, capture):
    """The element-wise step in front of a quantised linear, separate (torch's RMSNorm arithmetic / silu * up as eager
    torch ops, then this library's q8_1 quantiser) against fused with the quantiser (gsq_b200.fused), each followed by
    the product that consumes the q8_1 bytes, 64 times in one CUDA graph; microseconds per (step + product)."""
    import torch

    from gsq_b200 import fused, synth
    from gsq_b200.quantization import iq3_pack

    H, I, eps = 5120, 17408, 1e-6
    out = []
    w_qkv = torch.from_numpy(synth.make_weight(21, 7168, H, 2100)).to(dev)
    iq3_pack.pack_(w_qkv, 21)
    w_down = torch.from_numpy(synth.make_weight(23, H, I, 2101)).to(dev)
    gamma = torch.ones(H, device=dev, dtype=torch.bfloat16)
    op_qkv = torch.ops._C_gguf.lcpp_mul_mat_vec_iq3_mma_packed
    op_down = torch.ops._C_gguf.lcpp_mul_mat_vec_q

    def timed(fn, reps=64):
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
        del g
        return round(best, 2)
    for m in (4, 8):
        x = torch.randn(m, H, device=dev, dtype=torch.bfloat16)
        res = torch.randn(m, H, device=dev, dtype=torch.bfloat16)
        gu = torch.randn(m, 2 * I, device=dev, dtype=torch.bfloat16)

        def norm_separate():
            z = x + res
            y = (z.float() * torch.rsqrt(z.float().pow(2).mean(-1, keepdim=True) + eps)).to(torch.bfloat16) * gamma
            xq = torch.ops._C_gguf.lcpp_quantize_q8_1(y, 21, False, False)
            op_qkv(w_qkv, y, 21, 7168, xq)

        def norm_fused():
            r = res.clone()
            xq, y = fused.rmsnorm_quantize_q8_1(x, gamma, eps, r, want_y=True)
            op_qkv(w_qkv, y, 21, 7168, xq)

        def act_separate():
            y = torch.nn.functional.silu(gu[:, :I]) * gu[:, I:]
            xq = torch.ops._C_gguf.lcpp_quantize_q8_1(y, 23, False, False)
            op_down(w_down, y, 23, H, xq)

        def act_fused():
            xq, y = fused.silu_mul_quantize_q8_1(gu, want_y=True)
            op_down(w_down, y, 23, H, xq)
        out.append({"rows": m, "add_rmsnorm_quantize_qkv_us": {"separate": timed(norm_separate), "fused": timed(norm_fused)},
                    "silu_mul_quantize_down_us": {"separate": timed(act_separate), "fused": timed(act_fused)}})
    return {"what": "residual add + RMSNorm -> q8_1 -> qkv product (IQ3_S 7168 x 5120) and SwiGLU -> q8_1 -> down product "
                    "(IQ4_XS 5120 x 17408); 'separate' = eager torch ops for the step + gsq quantiser, 'fused' = one gsq kernel "
                    "for step + quantiser (the fused norm also clones the residual per call)", "cells": out}


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
    hbm = measured_peaks()[0]["hbm_gbs"]
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
                    "floor_ms_at_measured_hbm": round(bytes_step / (hbm * 1e6), 3),
                    "frac_of_measured_hbm": round(bytes_step / best / 1e6 / hbm, 4)})
    # the same stack followed by the Q6_K output head 151936 x 5120 (the 1-GPU form of the tensor-parallel config)
    head = torch.from_numpy(synth.make_weight(14, 151936, 5120, 3000)).to(dev)
    iq3_pack.pack_(head, 14)    # repacked at load, as GGUFLinearMethod.process_weights_after_loading does
    res_head = []
    for rows in (32,):
        x5 = torch.randn(rows, 5120, device=dev, dtype=torch.bfloat16)
        x17 = torch.randn(rows, 17408, device=dev, dtype=torch.bfloat16)

        def step_head():
            for lw in stack:
                linear.fused_mul_mat_gguf(x5, lw["qkv"], 21, None, True)
                linear.fused_mul_mat_gguf(x5, lw["o"], 21, None, True)
                linear.fused_mul_mat_gguf(x5, lw["gate_up"], 21, None, True)
                linear.fused_mul_mat_gguf(x17, lw["down"], 23, None, False)
            linear.fused_mul_mat_gguf(x5, head, 14, None, True)
        g = capture(step_head)
        best = 1e30
        for _ in range(3):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            g.replay()
            e1.record()
            torch.cuda.synchronize()
            best = min(best, e0.elapsed_time(e1))
        b2 = bytes_step + head.numel()
        res_head.append({"rows": rows, "ms_per_step": round(best, 3), "GBps": round(b2 / best / 1e6, 1),
                         "floor_ms_at_measured_hbm": round(b2 / (hbm * 1e6), 3),
                         "frac_of_measured_hbm": round(b2 / best / 1e6 / hbm, 4)})
    return {"layers": layers, "weight_bytes_per_step": bytes_step, "steps": res,
            "with_q6k_output_head": {"weight_bytes_per_step": bytes_step + head.numel(), "steps": res_head}}

def extra_tp_stack(dev, world, rank, capture, layers=64, rows=32):
    """The 64-layer stack + Q6_K output head, tensor parallel over `world` GPUs, `rows` activation rows per step:
    qkv and gate_up cut along N (gate_up's channels matched to down's K-shards, so nothing is gathered between them),
    o_proj and down cut along K at 256-column granularity with an NCCL all-reduce of the partial [rows, 5120] results,
    the head cut along N with an all-gather of the logits. One CUDA graph per step, collectives inside it. Reported:
    the whole step, the products alone and the collectives alone (ms, max over ranks)."""
    import numpy as np
    import torch
    import torch.distributed as dist

    from gsq_b200 import lcpp_ops, synth, tp
    from gsq_b200.quantization import iq3_pack, linear

    H, I, QKV, V = 5120, 17408, 7168, 151936
    with tp.relaxed_k():
        p_qkv = tp.shard_plan(QKV, H, world, rank, "N")
        p_o = tp.shard_plan(H, H, world, rank, "K")
        up0, upc = tp.matched_up_rows(I, world, rank)
        p_down = tp.shard_plan(H, I, world, rank, "K")
        p_head = tp.shard_plan(V, H, world, rank, "N")

        def up(raw, t, pack):
            w = torch.from_numpy(np.ascontiguousarray(raw)).to(dev)
            if pack:
                iq3_pack.pack_(w, t)
            return w
        qkv = up(tp.shard_bytes(synth.make_weight(21, QKV, H, 2000), 21, p_qkv), 21, True)
        o = up(tp.shard_bytes(synth.make_weight(21, H, H, 2001), 21, p_o), 21, True)
        gu_full = synth.make_weight(21, 2 * I, H, 2002)
        gate_up = up(np.concatenate([gu_full[up0:up0 + upc], gu_full[I + up0:I + up0 + upc]]), 21, True)
        down = up(tp.shard_bytes(synth.make_weight(23, H, I, 2003), 23, p_down), 23, False)
        head = up(tp.shard_bytes(synth.make_weight(14, V, H, 3000), 14, p_head), 14, True)
        base = {"qkv": qkv, "o": o, "gate_up": gate_up, "down": down}
        stack = [{n: torch.roll(w, shifts=16 * (l + 1), dims=0) if l else w for n, w in base.items()} for l in range(layers)]
        local_bytes = layers * sum(w.numel() for w in base.values()) + head.numel()
        ko, kd = p_o.count * 256, p_down.count * 256
        x = torch.randn(rows, H, device=dev, dtype=torch.bfloat16)
        h1 = torch.empty(rows, H, device=dev, dtype=torch.bfloat16)      # o_proj partial -> all-reduce
        h2 = torch.empty(rows, H, device=dev, dtype=torch.bfloat16)      # down partial -> all-reduce
        logits_local = torch.empty(rows, p_head.count, device=dev, dtype=torch.bfloat16)
        # the head's N-shards are equal but for the last rank's remainder: the gather takes the largest, padded
        hmax = max(tp.shard_plan(V, H, world, r, "N").count for r in range(world))
        lg_in = torch.zeros(rows, hmax, device=dev, dtype=torch.bfloat16)
        lg_out = torch.empty(world, rows, hmax, device=dev, dtype=torch.bfloat16)

        r1 = torch.empty(rows, H, device=dev, dtype=torch.bfloat16)      # sums (peer variant: the partials are elsewhere)
        r2 = torch.empty(rows, H, device=dev, dtype=torch.bfloat16)

        def step_fused(peer):
            """o_proj and down as gsq_linear_allreduce: the product kernel itself pushes its partial to every rank, waits
            for the others' and writes the sum -- no collective call and no extra kernel for the two sums of a layer."""
            nb = rows * H * 2
            cur = x
            with tp.relaxed_k():
                for lw in stack:
                    a = linear.fused_mul_mat_gguf(cur, lw["qkv"], 21, None, True)
                    with peer.fused(nb), lcpp_ops.output_into(r1):
                        linear.fused_mul_mat_gguf(a[:, :ko], lw["o"], 21, None, True)
                    g = linear.fused_mul_mat_gguf(r1, lw["gate_up"], 21, None, True)
                    with peer.fused(nb), lcpp_ops.output_into(r2):
                        linear.fused_mul_mat_gguf(g[:, :kd], lw["down"], 23, None, False)
                    cur = r2
                with lcpp_ops.output_into(lg_in[:, :p_head.count]):
                    linear.fused_mul_mat_gguf(cur, head, 14, None, True)
            dist.all_gather_into_tensor(lg_out, lg_in)

        def step(products=True, collectives=True, peer=None):
            """peer: a tp.PeerAllReduce -- the partials of o_proj / down are written into its symmetric buffers and
            summed by one kernel per rank over peer memory instead of an NCCL all-reduce."""
            p1 = peer.partial(0, (rows, H), torch.bfloat16) if peer else h1
            p2 = peer.partial(1, (rows, H), torch.bfloat16) if peer else h2
            s1, s2 = (r1, r2) if peer else (h1, h2)
            cur = x
            for lw in stack:
                if products:
                    a = linear.fused_mul_mat_gguf(cur, lw["qkv"], 21, None, True)          # [rows, 7168 / world]
                    with lcpp_ops.output_into(p1):
                        linear.fused_mul_mat_gguf(a[:, :ko], lw["o"], 21, None, True)      # attention stub: its columns
                if collectives:
                    if peer:
                        peer.reduce(0, r1)
                    else:
                        dist.all_reduce(h1)
                if products:
                    g = linear.fused_mul_mat_gguf(s1, lw["gate_up"], 21, None, True)       # [rows, 2 * matched channels]
                    with lcpp_ops.output_into(p2):
                        linear.fused_mul_mat_gguf(g[:, :kd], lw["down"], 23, None, False)   # SwiGLU stub: gate's columns
                if collectives:
                    if peer:
                        peer.reduce(1, r2)
                    else:
                        dist.all_reduce(h2)
                cur = s2
            if products:
                with lcpp_ops.output_into(lg_in[:, :p_head.count]):
                    linear.fused_mul_mat_gguf(cur, head, 14, None, True)
            if collectives:
                dist.all_gather_into_tensor(lg_out, lg_in)

        def best_ms(fn):
            g = capture(fn)
            for _ in range(2):
                g.replay()
            torch.cuda.synchronize()
            dist.barrier()
            best = 1e30
            for _ in range(3):
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                g.replay()
                e1.record()
                torch.cuda.synchronize()
                best = min(best, e0.elapsed_time(e1))
                dist.barrier()
            del g        # (a graph that holds NCCL collectives must be gone before the process group is destroyed)
            t = torch.tensor([best], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            return float(t.item())
        total = best_ms(lambda: step(True, True))
        compute = best_ms(lambda: step(True, False))
        coll = best_ms(lambda: step(False, True))
        peer_res = None
        try:
            ar = tp.PeerAllReduce(rows * H * 2)
            p_total = best_ms(lambda: step(True, True, ar))
            p_coll = best_ms(lambda: step(False, True, ar))
            flag = __import__("ctypes").c_int(-1)
            _cabi_lib = __import__("gsq_b200")._cabi.lib
            _cabi_lib.gsq_allreduce_error_flag(__import__("ctypes").byref(flag))
            peer_res = {"ms_per_step": round(p_total, 3), "collectives_only_ms": round(p_coll, 3),
                        "collective_us_each": round(p_coll * 1e3 / (2 * layers + 1), 1), "wait_gave_up": int(flag.value),
                        "what": "the all-reduces replaced by gsq_allreduce_sum (one kernel per rank over symmetric "
                                "memory: flag exchange + peer loads); the logits' all-gather stays NCCL"}
            try:
                ar.fused(rows * H * 2)      # allocate before the capture
                f_total = best_ms(lambda: step_fused(ar))
                _cabi_lib.gsq_peer_reduce_error_flag(__import__("ctypes").byref(flag))
                peer_res["fused_into_the_product"] = {
                    "ms_per_step": round(f_total, 3), "wait_gave_up": int(flag.value),
                    "what": "o_proj and down through gsq_linear_allreduce: one kernel per rank forms the partial, stores it "
                            "into every rank's slot over peer pointers, waits for the others and sums in rank order"}
            except Exception as e:  # noqa: BLE001
                peer_res["fused_into_the_product"] = {"unavailable": str(e).splitlines()[0][:200]}
            del ar
        except Exception as e:  # noqa: BLE001  (symmetric memory unavailable: the NCCL variant stands alone)
            peer_res = {"unavailable": str(e).splitlines()[0][:200]}
        import gc
        gc.collect()
    full_bytes = layers * 150978560 + V * (H // 256) * 210
    return {"rows": rows, "layers": layers, "world": world, "ms_per_step": round(total, 3),
            "products_only_ms": round(compute, 3), "collectives_only_ms": round(coll, 3),
            "collectives_per_step": 2 * layers + 1,
            "collective_us_each": round(coll * 1e3 / (2 * layers + 1), 1),
            "weight_bytes_per_step_all_ranks": full_bytes, "weight_bytes_this_rank": local_bytes,
            "GBps_all_ranks": round(full_bytes / total / 1e6, 1),
            "peer_memory_allreduce": peer_res,
            "sharding": "qkv / gate_up / head along N (gate_up matched to down's K-shards), o_proj / down along K "
                        "(256-column granularity); all-reduce after o_proj and down, all-gather of the logits; "
                        "collectives captured in the step's CUDA graph"}


# --------------------------------------------------------------------------------------------------
# CPU baseline / reference arm (the only places bench.py executes oracle/)

def _synth_module():
    """gsq_b200/synth.py loaded by path: importing the package would load libgsq.so, which this arm never uses."""
    import importlib.util

    spec = importlib.util.spec_from_file_location(
        "gsq_synth_standalone", os.path.join(ROOT, "vllm-gsqrco-exl3_b200", "gsq_b200", "synth.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def _cpu_product(synth, t, rows, k, m, seed_w, seed_x, cores):
    """One product on the host the way the reference's CPU model does it (tests/gpu/_refs.py:33-37,
    tools/ggml_ref.py:48-56): dequantise W to fp32, then an fp32 matmul on all cores. -> (bytes, s_dequant, s_matmul)."""
    import numpy as np
    import torch

    raw = synth.make_weight(t, rows, k, seed_w)
    x = synth.make_activation(m, k, seed_x)
    t0 = time.perf_counter()
    try:
        import gguf

        w = gguf.quants.dequantize(raw, gguf.GGMLQuantizationType(t))
        kind = "reference"
    except ImportError:
        from oracle import blocks

        w = blocks.dequantize(raw, t)
        kind = "port"
    t1 = time.perf_counter()
    y = torch.from_numpy(np.asarray(x, dtype=np.float32)) @ torch.from_numpy(np.ascontiguousarray(w, dtype=np.float32)).T
    t2 = time.perf_counter()
    assert y.shape == (m, rows)
    return raw.nbytes, t1 - t0, t2 - t1, kind


def cpu_baseline(rows: int = 17408, k: int = 5120, m: int = 1):
    """The single-layer CPU-runnable configuration in full: IQ3_S 17408 x 5120, one fp32 activation row."""
    import torch

    synth = _synth_module()
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    nbytes, t_deq, t_mm, kind = _cpu_product(synth, 21, rows, k, m, 1000, 1001, cores)
    gbs = nbytes / (t_deq + t_mm) / 1e9
    return {"value": round(gbs, 4), "unit": "GB/s", "cores": cores, "kind": kind,
            "sample": f"IQ3_S {rows}x{k}, M={m}, one product: gguf-py dequantise {t_deq:.2f} s (numpy, 1 thread) + "
                      f"fp32 matmul {t_mm:.3f} s ({cores} threads); the reference's tools/ggml_ref.py needs "
                      f"libggml-base.so, absent here, and its tests pin gguf-py bit-identical to it"}


def run_reference(args):
    """The reference's CPU path on a bounded sample of the row sweep: per step the two corner cells (IQ3_S
    17408 x 5120 at 1 row, which is also the single-layer configuration in full, and Q4_K 5120 x 5120 at 48 rows)."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import torch

    synth = _synth_module()
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    steps = max(1, args.steps)
    sample = [(21, 17408, 5120, 1), (12, 5120, 5120, 48)]

    def one_step():
        b = s = 0.0
        kind = "reference"
        for t, n, k, m in sample:
            nb, t_deq, t_mm, kind = _cpu_product(synth, t, n, k, m, 1100, 1200 + m, cores)
            b += nb
            s += t_deq + t_mm
        return b, s, kind
    for _ in range(max(0, min(args.warmup, 1))):
        one_step()
    t0 = time.perf_counter()
    tot_b = tot_s = 0.0
    for _ in range(steps):
        b, sec, kind = one_step()
        tot_b += b
        tot_s += sec
    dt = time.perf_counter() - t0
    v = round(tot_b / tot_s / 1e9, 4)
    base = {"value": v, "unit": "GB/s", "cores": cores, "kind": kind,
            "sample": "per step 2 of the 54 cells: IQ3_S 17408x5120 M=1 and Q4_K 5120x5120 M=48; per product gguf-py "
                      "dequantise (numpy, 1 thread) + torch fp32 matmul (all threads)"}
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": v, "unit": "GB/s", "n_gpus": args.gpus, "steps": steps,
        "warmup": min(args.warmup, 1), "ms_per_step": round(dt / steps * 1e3, 1), "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "gemv_row_sweep", "types": [t for t, _ in TYPES], "shapes": SHAPES, "rows": ROWS,
                   "x_dtype": "fp16", "cells": len(TYPES) * len(SHAPES) * len(ROWS),
                   "note": "CPU path of the reference (dequantise + fp32 matmul) on a bounded sample of these cells"},
        "cpu_baseline": base,
        "e2e": {"value": v, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }), flush=True)


def run_cell(args):
    """One product (or the same product at several row counts: M may be a comma-separated list) a few times on distinct
    weight copies: eager for a profiler, or as a CUDA graph for a number without launch overhead."""
    import torch

    import gsq_b200  # noqa: F401
    from gsq_b200 import _cabi, synth
    from gsq_b200.quantization import iq3_pack, linear

    tname, n, k = args.cell[0], int(args.cell[1]), int(args.cell[2])
    ms = [int(v) for v in args.cell[3].split(",")]
    dev = "cuda:0"
    from gsq_b200 import lcpp_ops
    lcpp_ops.set_prefill_precision({"rounded": lcpp_ops.PREFILL_ROUNDED, "split": lcpp_ops.PREFILL_SPLIT,
                                    "integer": lcpp_ops.PREFILL_INTEGER}[args.precision])
    t = {**synth.TYPE_IDS, **synth.LOW_BIT_TYPE_IDS}[tname]
    w0 = torch.from_numpy(synth.make_weight(t, n, k, 1)).to(dev)
    packed = tname in ("IQ3_S", "Q6_K") and not args.unpacked and n % 16 == 0
    if packed:
        iq3_pack.pack_(w0, t)
    ws = [w0] + [w0.clone() for _ in range(15 if args.graph else 3)]
    for m in ms:
        dtype = torch.bfloat16 if m > 64 else torch.float16
        x = synth.nudge_ties_torch(torch.from_numpy(synth.make_activation(m, k, 2)).to(dtype)).to(dev)
        for kernel in (["default", "tcgen05"] if args.kernel == "both" else [args.kernel]):
            old = _cabi.lib.gsq_debug_mmv_mode(1 if kernel == "tcgen05" else 0)
            for i in range(2):
                y = linear.fused_mul_mat_gguf(x, ws[i % len(ws)], t, None, packed)
            torch.cuda.synchronize()
            if args.graph:
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g):
                    for w in ws:
                        linear.fused_mul_mat_gguf(x, w, t, None, packed)
                us = 1e30
                for _ in range(3):
                    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    e0.record()
                    g.replay()
                    e1.record()
                    torch.cuda.synchronize()
                    us = min(us, e0.elapsed_time(e1) * 1e3 / len(ws))
                del g
            else:
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                for i in range(args.iters):
                    y = linear.fused_mul_mat_gguf(x, ws[(i + 2) % len(ws)], t, None, packed)
                e1.record()
                torch.cuda.synchronize()
                us = e0.elapsed_time(e1) * 1e3 / args.iters
            _cabi.lib.gsq_debug_mmv_mode(old)
            how = "graph replay over 16 weight copies" if args.graph else "eager, with launch overhead"
            print(f"{tname} {n}x{k} m={m} packed={packed} kernel={kernel}: {us:.1f} us per call ({how}), "
                  f"{w0.numel() / us / 1e3:.0f} GB/s, {2.0 * m * n * k / us / 1e6:.1f} TOPS; op "
                  f"{linear._lcpp_op(m, t, n, k, packed)}; mean |y| {float(y.float().abs().mean()):.4f}", flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true", help="skip the prefill-TOPS and decode-stack measurements")
    ap.add_argument("--eager", action="store_true", help="time eager launches instead of CUDA-graph replays")
    ap.add_argument("--no-check", action="store_true", help="skip the untimed parity / graph-replay check of every cell")
    ap.add_argument("--no-ref-kernels", action="store_true", help="skip timing the reference's CUDA kernels (oracle/_ref)")
    ap.add_argument("--cell", nargs=4, metavar=("TYPE", "N", "K", "M"), help="run one product only (for profilers)")
    ap.add_argument("--iters", type=int, default=3)
    ap.add_argument("--unpacked", action="store_true", help="--cell: keep IQ3_S / Q6_K in GGUF order")
    ap.add_argument("--kernel", default="default", choices=["default", "tcgen05", "both"],
                    help="--cell: 'tcgen05' switches the register-operand small-batch kernel off, so that 9..48 rows run on "
                         "the tcgen05 GEMM instead; 'both' times one after the other")
    ap.add_argument("--precision", default="rounded", choices=["rounded", "split", "integer"],
                    help="--cell: form of the prefill product from 256 rows on (gsq_prefill_precision)")
    ap.add_argument("--graph", action="store_true", help="--cell: time a CUDA graph of the calls (no launch overhead), best of 3 replays")
    args = ap.parse_args()
    if args.cell:
        run_cell(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
