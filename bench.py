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
