#!/usr/bin/env python
"""Benchmark of the EXL3 decode hot path on B200.

Workload (benchmark configuration 1): the dense 27B-shaped decode stack at 4 bpw -- MLP
gate/up 5120->17408 (fp16 out), silu*up, down 17408->5120 (fp32 out), and the attention
projections q 5120->6144, k/v 5120->1024, o 6144->5120 -- for a batch of M fp16 token rows.
One "step" is one pass over one layer's seven trellis matrices; LAYERS distinct seeded layers
(> L2 in total) are cycled so that no step finds its weights in L2.

Metric: effective HBM GB/s on the algorithmic bytes of the pass (trellis + sign-scale vectors
+ activations in/out), value = bytes moved by all ranks / device time (CUDA events, max over
ranks).  `e2e` is the same metric through the host-buffer API: pinned host activations are
copied in and the results read back every step.  `roofline` is measured live for the dominant
kernel (the decode launch over the stacked gate and up projections).  `cpu_baseline` times the CPU oracle on a
bounded sample.  Extra records of the same line: the step at 8 and 32 rows, configuration 0 (one 5120x6144 linear
over a ring of 17 seeded copies), prefill (configuration 2), lm_head, MoE (configuration 3 / 4).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--m M] [--impl reference]
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

HIDDEN, INTER, QDIM, KVDIM = 5120, 17408, 6144, 1024
BITS, CB = 4, 2
# (name, K, N, fp32 out, input)
SHAPES = [("gate", HIDDEN, INTER, 0, "x"), ("up", HIDDEN, INTER, 0, "x"), ("down", INTER, HIDDEN, 1, "act"),
          ("q", HIDDEN, QDIM, 0, "xa"), ("k", HIDDEN, KVDIM, 0, "xa"), ("v", HIDDEN, KVDIM, 0, "xa"),
          ("o", QDIM, HIDDEN, 1, "attn")]
LAYERS = 4
METRIC = "exl3_gemv_eff_hbm_gbs"

# dram__bytes_read.sum + dram__bytes_write.sum of one decode launch over the stacked gate and up projections
# (2 x 5120x17408, 4 bpw, one row) from an ncu capture of this file's own step; valid for one row only.
NCU_TRAFFIC_GATE_UP_BYTES = 92_805_120   # 89.35 MB read + 3.46 MB written


def linear_bytes(k: int, n: int, m: int, fp32: int, bits: int = BITS) -> int:
    """Algorithmic bytes of one linear: trellis + suh + svh + x in + y out."""
    return k * n * bits // 8 + 2 * k + 2 * n + 2 * m * k + (4 if fp32 else 2) * m * n


def step_bytes(m: int) -> int:
    return sum(linear_bytes(k, n, m, f) for _, k, n, f, _ in SHAPES)


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        return float(json.load(open(p))["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


# ------------------------------------------------------------------ clocks

class ClockSampler:
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.idx = gpu_index
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.idx)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.strip().splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2]))
            except ValueError:
                continue
            for name, v in zip(names, f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


# ------------------------------------------------------------------ the workload on the GPU

class DecodeStack:
    """LAYERS layers of the seven 27B-shaped EXL3 linears, resident in HBM, with the host-side
    callers of berth_b200.engine (Exl3Linear / MlpLayer)."""

    def __init__(self, m: int, rank: int, share: "DecodeStack | None" = None):
        """m = token rows per step (buffers are sized for it); `share` = a stack whose weights (already in HBM) this
        one uses too."""
        import torch
        from berth_b200 import synth
        from berth_b200.engine import Exl3Linear, Gpu, MlpLayer, SlicedMultiLinear
        from berth_b200.kernels import OutDtype
        from berth_b200.kernels import Codebook
        self.torch = torch
        self.m = m
        self.gpu = Gpu(torch.cuda.current_device())
        dev = self.gpu.device
        f16, f32 = torch.float16, torch.float32
        # One pinned host block and one device block each for the step's inputs and for its results, so that the
        # end-to-end step is one copy in and one copy out (the tensors below are views into the device blocks).
        self.h2d_bytes = 2 * m * (HIDDEN + HIDDEN + QDIM)
        self.d2h_bytes = m * (4 * HIDDEN + 2 * QDIM + 4 * KVDIM + 4 * HIDDEN)
        self.h_in = torch.empty(self.h2d_bytes, dtype=torch.uint8).pin_memory()
        self.d_in = torch.empty(self.h2d_bytes, dtype=torch.uint8, device=dev)
        self.h_out = torch.empty(self.d2h_bytes, dtype=torch.uint8).pin_memory()
        self.d_out = torch.empty(self.d2h_bytes, dtype=torch.uint8, device=dev)

        def carve(block, specs):
            views, off = [], 0
            for rows, cols, dt in specs:
                nbytes = rows * cols * (2 if dt == f16 else 4)
                views.append(block[off:off + nbytes].view(dt).view(rows, cols))
                off += nbytes
            return views

        in_specs = [(m, HIDDEN, f16), (m, HIDDEN, f16), (m, QDIM, f16)]
        hx, hxa, hattn = carve(self.h_in, in_specs)
        hx.copy_(torch.from_numpy(synth.activations(1234, f"r{rank}.x", m, HIDDEN)))
        hxa.copy_(torch.from_numpy(synth.activations(1234, f"r{rank}.xa", m, HIDDEN)))
        hattn.copy_(torch.from_numpy(synth.activations(1234, f"r{rank}.attn", m, QDIM)))
        self.x, self.xa, self.attn = carve(self.d_in, in_specs)
        self.d_in.copy_(self.h_in)
        out_specs = [(m, HIDDEN, f32), (m, HIDDEN, f32), (m, QDIM, f16), (m, KVDIM, f16), (m, KVDIM, f16)]
        self.mlp_out, self.o, self.q, self.k, self.v = carve(self.d_out, out_specs)
        self.layers = []
        for l in range(LAYERS):
            lin = {}
            for name, k, n, _, _ in SHAPES:
                if share is not None:
                    src = share.layers[l][1][name]
                    w = {"trellis": src.trellis, "suh": src.suh, "svh": src.svh}
                else:
                    w = synth.linear_weights(synth.MASTER_SEED, f"r{rank}.layers.{l}.{name}", k, n, BITS, fan_in_gain=True)
                lin[name] = Exl3Linear(self.gpu, f"layers.{l}.{name}", w["trellis"], w["suh"], w["svh"], BITS,
                                       Codebook(CB), max_rows=m)
            mlp = MlpLayer(self.gpu, lin["gate"], lin["up"], lin["down"], max_rows=m)
            # q, k and v share their input: one sliced multi-linear launch, as in berth's attention layers
            # (berth_ops_mgemm; crates/berth-kernels/src/ops.rs:257-262)
            lin["qkv"] = SlicedMultiLinear(self.gpu, [lin["q"], lin["k"], lin["v"]], OutDtype.F16, max_rows=m,
                                           outputs=[self.q, self.k, self.v])
            self.layers.append((mlp, lin))
        # one row: gate+up (one stacked integer-path launch, rotation and finishing inside it), down (the same kernel, with
        # silu(gate) * up formed in its rotation) and o (one launch each), q/k/v (the same kernel over the three matrices,
        # one launch) = 4 launches.
        # two rows: the stacked launch, down and o on the fp16-path kernel (k_exl3_gemv + k_gemv_finish each), q/k/v = 6.
        # 3..4 rows: k_rotate_in_i8 per stacked matrix + the stacked launch, down and o with k_rotate_in + k_exl3_gemv +
        # k_gemv_finish each, q/k/v (one launch) = 10.
        # 5..16 rows: gate, up, down, o with three launches each (k_rotate_in + k_exl3_gemv + k_gemv_finish), q/k/v as one
        # sliced launch of the fp16-path kernel (k_rotate_in + k_exl3_gemv + k_gemv_finish) = 15.
        # above: the same with k_had128 + k_exl3_gemm_tc_splitk + k_sk_finish per linear, and k_silu_mul = 16.
        self.launches_per_step = 4 if m == 1 else (6 if m == 2 else (10 if m <= 4 else (15 if m <= 16 else 16)))

    def step(self, i: int) -> None:
        from berth_b200.kernels import OutDtype
        mlp, lin = self.layers[i % LAYERS]
        g, m = self.gpu, self.m
        mlp.forward_n(g, m, self.x, self.mlp_out)
        lin["qkv"].forward_n(g, m, self.xa)
        lin["o"].forward_n(g, m, self.attn, self.o, OutDtype.F32)

    def step_e2e(self, i: int) -> None:
        """Host buffers in, host buffers out: what a caller without device residency pays."""
        self.d_in.copy_(self.h_in, non_blocking=True)
        self.step(i)
        self.h_out.copy_(self.d_out, non_blocking=True)
        self.torch.cuda.current_stream().synchronize()

    def time_dominant_kernel(self, reps: int):
        """(average ms, algorithmic bytes, description) of the step's dominant launch, run back to back over the
        LAYERS distinct layers (357 MB of gate and up weights > L2) between two CUDA events: up to four rows the
        decode launch over the stacked gate and up projections, above the gate linear alone."""
        torch = self.torch
        from berth_b200 import kernels
        from berth_b200.kernels import OutDtype
        stacked = self.layers[0][0].gate_up is not None and self.m <= 4
        if stacked:
            calls = [(l[0].gate_up, l[0].gate_up_out) for l in self.layers]
            nbytes = 2 * linear_bytes(HIDDEN, INTER, self.m, 0) - 2 * self.m * HIDDEN   # the rows are read once
            what = "gate and up 2 x 5120x17408 as one stacked decode launch"
        else:
            calls = [(l[1][n], l[0].gate_out) for l in self.layers for n in ("gate", "up")]
            nbytes = linear_bytes(HIDDEN, INTER, self.m, 0)
            what = "gate/up 5120x17408"
        for lin, out in calls:
            lin.forward_n(self.gpu, self.m, self.x, out, OutDtype.F16)
        name = kernels.last_launch()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        for _ in range(reps):
            for lin, out in calls:
                lin.forward_n(self.gpu, self.m, self.x, out, OutDtype.F16)
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / (reps * len(calls)), nbytes, what, name

    def time_steps(self, steps: int, warmup: int) -> float:
        """ms per step, device timed."""
        torch = self.torch
        for i in range(warmup):
            self.step(i)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        for i in range(steps):
            self.step(i)
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / steps


def bench_rows(base: "DecodeStack", rank: int, m: int, steps: int) -> dict:
    """The same step at m rows on the weights of `base`: value and the dominant launch's roofline entry."""
    st = DecodeStack(m, rank, share=base)
    ms = st.time_steps(steps, 5)
    k_ms, k_bytes, what, name = st.time_dominant_kernel(max(4, steps // 8))
    peak, kind = peaks()
    sb = step_bytes(m)
    return {"m": m, "us_per_step": ms * 1e3, "value": sb / (ms * 1e-3) / 1e9, "unit": "GB/s", "bytes_per_step": sb,
            "frac_of_hbm_peak": sb / (ms * 1e-3) / 1e9 / peak, "gpu_launches_per_step": st.launches_per_step,
            "roofline": {"bound": "hbm", "achieved": k_bytes / (k_ms * 1e-3) / 1e9, "peak": peak, "unit": "GB/s",
                         "frac": k_bytes / (k_ms * 1e-3) / 1e9 / peak, "traffic": None, "kernel": name,
                         "launch": f"{what} m={m}: {k_bytes} algorithmic bytes in {k_ms * 1e3:.2f} us", "peak_kind": f"of {kind}"}}


def bench_decode_rate() -> dict:
    """Bare decode rate of an SM (berth_exl3_decode_rate): weights per clock per SM of the decode kernels' inner loops on
    tiles resident in shared memory, no global-memory traffic, per codebook and path at 4 bpw (and 3, 5, 6 bpw for MUL1),
    beside the rate the HBM roofline asks for at the clock seen during the run."""
    from berth_b200 import kernels
    from berth_b200.kernels import Codebook
    peak, kind = peaks()
    rec = {"workload": "bare_decode_rate", "warps": 16, "iters": 4096, "rates": []}
    paths = {0: "fp16 tensor path (mma.sync m16n8k16)", 1: "integer path, mma.sync m16n8k32", 2: "integer path, tcgen05.st into tensor memory"}
    for bits, cb, path in [(4, 0, 0), (4, 1, 0), (4, 2, 0), (4, 2, 1), (4, 2, 2), (3, 2, 0), (3, 2, 2), (5, 2, 0), (5, 2, 2), (6, 2, 0), (6, 2, 2)]:
        w, mhz = kernels.decode_rate(bits, Codebook(cb), path, 16, 4096)
        need = peak * 1e9 * 8 / bits / (148 * mhz * 1e6)      # weights per clock per SM at the measured HBM peak
        rec["rates"].append({"bits": bits, "codebook": ["3inst", "mcg", "mul1"][cb], "path": paths[path], "weights_per_clk_per_sm": round(w, 2),
                             "sm_mhz": round(mhz), "hbm_roofline_needs": round(need, 1), "ceiling_frac_of_hbm_peak": round(w / need, 3)})
    rec["peak_kind"] = f"of {kind}"
    names = ["2 mma.sync m16n8k16", "2 mma.sync m16n8k16 + 8 lop3", "2 mma.sync m16n8k16 + 8 imad", "8 lop3 + 8 imad",
             "2 mma.sync m16n8k32 (u8 x s8)", "2 mma.sync m16n8k32 + 8 lop3"]
    rec["pipe_probe_clk_per_bundle_per_scheduler"] = {n: round(kernels.pipe_probe(i), 2) for i, n in enumerate(names)}
    return rec


def bench_c0(rank: int, reps: int = 12) -> dict:
    """Configuration 0: one 5120 x 6144 linear, 4 bpw, one row, fp16 out, over a ring of 17 seeded weight copies
    (267 MB > L2); 17 * reps launches between two CUDA events, median of 5 repeats."""
    import torch
    from berth_b200 import synth
    from berth_b200.engine import Exl3Linear, Gpu
    from berth_b200.kernels import Codebook, OutDtype
    from berth_b200 import kernels
    K, N, ring = 5120, 6144, 17
    gpu = Gpu(torch.cuda.current_device())
    lins = []
    for i in range(ring):
        w = synth.linear_weights(synth.MASTER_SEED, f"r{rank}.c0.{i}", K, N, BITS)
        lins.append(Exl3Linear(gpu, f"c0.{i}", w["trellis"], w["suh"], w["svh"], BITS, Codebook(CB), max_rows=1))
    x = torch.from_numpy(synth.activations(1234, f"r{rank}.c0.x", 1, K)).to(gpu.device)
    c = torch.empty((1, N), dtype=torch.float16, device=gpu.device)
    for lin in lins:
        lin.forward_n(gpu, 1, x, c, OutDtype.F16)
    name = kernels.last_launch()
    times = []
    for _ in range(5):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        for _ in range(reps):
            for lin in lins:
                lin.forward_n(gpu, 1, x, c, OutDtype.F16)
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1) / (reps * ring))
    ms = statistics.median(times)
    nbytes = linear_bytes(K, N, 1, 0)
    peak, kind = peaks()
    return {"workload": "c0_single_linear_5120x6144_4bpw_m1", "us_per_launch": ms * 1e3, "launches_timed": reps * ring,
            "ring": f"{ring} seeded copies, {ring * K * N // 2 / 1e6:.0f} MB", "bytes_per_launch": nbytes,
            "roofline": {"bound": "hbm", "achieved": nbytes / (ms * 1e-3) / 1e9, "peak": peak, "unit": "GB/s",
                         "frac": nbytes / (ms * 1e-3) / 1e9 / peak, "traffic": None, "kernel": name, "peak_kind": f"of {kind}"}}


# ------------------------------------------------------------------ lm_head regime

def bench_lm_head(rank: int, reps: int = 10) -> dict:
    """berth's lm_head linear (6 bpw, 5120 -> 248320, one row; crates/berth-kernels/csrc/gemm_k6.cu:1-34): one
    decode launch over 953 MB of trellis, far larger than L2."""
    import torch
    from berth_b200 import synth
    from berth_b200.engine import Exl3Linear, Gpu
    from berth_b200.kernels import Codebook, OutDtype
    K, N, bits = HIDDEN, 248320, 6
    gpu = Gpu(torch.cuda.current_device())
    w = synth.linear_weights(synth.MASTER_SEED, f"r{rank}.lm_head", K, N, bits, fan_in_gain=True)
    lin = Exl3Linear(gpu, "lm_head", w["trellis"], w["suh"], w["svh"], bits, Codebook(CB), max_rows=1)
    x = torch.from_numpy(synth.activations(1234, f"r{rank}.lmh.x", 1, K)).to(gpu.device)
    out = torch.empty((1, N), dtype=torch.float32, device=gpu.device)
    for _ in range(3):
        lin.forward_n(gpu, 1, x, out, OutDtype.F32)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record()
    for _ in range(reps):
        lin.forward_n(gpu, 1, x, out, OutDtype.F32)
    e1.record()
    torch.cuda.synchronize()
    us = e0.elapsed_time(e1) * 1e3 / reps
    # the same launch with the greedy token taken in the finishing step and no logits written
    best = torch.zeros(1, dtype=torch.int64, device=gpu.device)
    for _ in range(3):
        lin.forward_argmax(gpu, 1, x, best)
    torch.cuda.synchronize()
    e0.record()
    for _ in range(reps):
        lin.forward_argmax(gpu, 1, x, best)
    e1.record()
    torch.cuda.synchronize()
    us_argmax = e0.elapsed_time(e1) * 1e3 / reps
    nbytes = linear_bytes(K, N, 1, 1, bits)
    pk, _ = peaks()
    return {"workload": "lm_head_6bpw_5120x248320_m1", "us": us, "gbs": nbytes / us / 1e3, "frac_of_hbm_peak": nbytes / us / 1e3 / pk,
            "bytes": nbytes, "us_with_argmax_no_logits": us_argmax}


# ------------------------------------------------------------------ configuration 2: prefill GEMM

PREFILL_M = 4096
# (name, K, N, bits, fp32 out): gate/up/q/o at 4 bpw, down at 5, k/v at 3 (a fixed mix of the three rates)
PREFILL_SHAPES = [("gate", HIDDEN, INTER, 4, 0), ("up", HIDDEN, INTER, 4, 0), ("down", INTER, HIDDEN, 5, 1),
                  ("q", HIDDEN, QDIM, 4, 0), ("k", HIDDEN, KVDIM, 3, 0), ("v", HIDDEN, KVDIM, 3, 0), ("o", QDIM, HIDDEN, 4, 1)]


def bench_prefill(rank: int, reps: int = 5) -> dict:
    """The seven 27B-shaped matrices at M = 4096 through berth_prefill_exl3_linear (rotation kernel +
    tcgen05 GEMM with in-kernel trellis decode).  Activations N(0,1) fp16 with 0.1 % x20 outliers."""
    import torch
    from berth_b200 import synth
    from berth_b200.kernels import Codebook, OutDtype, prefill_lin
    dev = torch.device("cuda", torch.cuda.current_device())
    up = lambda a: torch.from_numpy(np.ascontiguousarray(a).view(np.int16) if a.dtype == np.uint16 else np.ascontiguousarray(a)).to(dev)
    M = PREFILL_M
    xs = {k: up(synth.activations(1234, f"pf.x{k}", M, k, outlier_frac=0.001)) for k in (HIDDEN, INTER, QDIM)}
    scratch = torch.empty(16, dtype=torch.float16, device=dev)
    ahad = torch.empty(M * INTER, dtype=torch.float16, device=dev)
    runs, flops = [], 0
    for name, k, n, bits, f32 in PREFILL_SHAPES:
        w = synth.linear_weights(synth.MASTER_SEED, f"pf.{name}", k, n, bits, fan_in_gain=True)
        t, su, sv = up(w["trellis"]), up(w["suh"]), up(w["svh"])
        c = torch.empty((M, n), dtype=torch.float32 if f32 else torch.float16, device=dev)
        runs.append((xs[k], t, c, su, sv, k, n, bits, f32))
        flops += 2 * M * k * n

    def one_pass():
        for x, t, c, su, sv, k, n, bits, f32 in runs:
            prefill_lin.exl3_linear(x, t, c, su, ahad, sv, scratch, M, k, n, bits, Codebook(CB), OutDtype(f32))
    for _ in range(3):
        one_pass()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record()
    for _ in range(reps):
        one_pass()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / reps
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    peak = float(json.load(open(p))["bf16_tflops"]) if os.path.exists(p) else 1590.0
    tf = flops / ms / 1e9
    return {"workload": "c2_prefill_27b_shapes_m4096_mixed_3_4_5_bpw", "ms_per_pass": ms, "tflops": tf, "flops_per_pass": flops,
            "roofline": {"bound": "tensor", "achieved": tf, "peak": peak, "unit": "TFLOP/s", "frac": tf / peak,
                         "peak_kind": "of measured (burst)" if os.path.exists(p) else "of fallback", "traffic": None},
            "kernel": prefill_lin.last_launch()}


# ------------------------------------------------------------------ configuration 3: MoE layer

MOE = dict(hidden=2048, inter=512, n_experts=256, top_k=8, shared_inter=512)


def bench_moe(rank: int, world: int, steps: int = 20, tokens=(1, 64, 1024)) -> dict:
    """A3B MoE layer (256 experts + shared, top-8, 4 bpw) at 1, 64 and 1024 tokens in total.  One GPU: the
    fused berth_moe_layer.  N GPUs: experts sharded in blocks of 256/N, tokens split evenly, two NCCL
    all-to-alls per layer (expert parallelism); time = max over ranks."""
    import torch
    import torch.distributed as dist
    from berth_b200 import moe, synth
    dev = torch.device("cuda", torch.cuda.current_device())
    H, I, E, K, SI = MOE["hidden"], MOE["inter"], MOE["n_experts"], MOE["top_k"], MOE["shared_inter"]
    n_local = E // world
    # each rank builds only its own expert block (same seeds and names as the full layer)
    w = {"hidden": H, "inter": I, "n_experts": n_local, "top_k": K, "bits": BITS, "cb": CB, "shared_inter": SI,
         "w_router": synth.router_weight(1234, "c3.gate.weight", H, E), "router_bias": None}
    def stack(proj, k, n):
        ids = range(rank * n_local, (rank + 1) * n_local)
        t = np.stack([synth.trellis(1234, f"c3.experts.{proj}.{e}.trellis", k, n, BITS) for e in ids])
        su = np.stack([synth.sign_scale(1234, f"c3.experts.{proj}.{e}.suh", k) for e in ids])
        sv = np.stack([synth.sign_scale(1234, f"c3.experts.{proj}.{e}.svh", n, 1.0 / np.sqrt(k)) for e in ids])
        return t, su, sv
    w["gate_trellis"], w["gate_suh"], w["gate_svh"] = stack("gate_proj", H, I)
    w["up_trellis"], w["up_suh"], w["up_svh"] = stack("up_proj", H, I)
    w["down_trellis"], w["down_suh"], w["down_svh"] = stack("down_proj", I, H)
    for pname, (k, n) in (("gate", (H, SI)), ("up", (H, SI)), ("down", (SI, H))):
        lw = synth.linear_weights(1234, f"c3.shared_expert.{pname}_proj", k, n, BITS, fan_in_gain=True)
        w[f"sh_{pname}_trellis"], w[f"sh_{pname}_suh"], w[f"sh_{pname}_svh"] = lw["trellis"], lw["suh"], lw["svh"]
    out = {"workload": "c3_a3b_moe_layer_4bpw", "parallelism": "single" if world == 1 else f"ep{world}", "by_tokens": {}}
    if world == 1:
        layer = moe.MoeLayer(dev, w, 1024)
    else:
        # a rank may receive more rows than it sends (skewed routing): room for four times the mean
        stages = moe.GpuStages(dev, w, E, max_rows=4 * 1024 * K, max_rows_per_expert=1024)
        try:    # exchange by the kernels themselves over peer memory; NCCL all-to-alls if symmetric memory is not to be had
            layer = moe.P2pMoeLayer(stages, dist.group.WORLD, E, K, max_tokens=1024, max_rows=4 * 1024 * K)
            out["exchange"] = "peer-memory stores + flag barriers (no collective, no host sync)"
        except Exception as exc:   # noqa: BLE001 - any failure of the symmetric allocation
            layer = moe.EpMoeLayer(stages, dist.group.WORLD, E, K)
            out["exchange"] = f"NCCL all_to_all_single (symmetric memory unavailable: {type(exc).__name__})"
    # global batches (the batch is split over the ranks), then, on several GPUs, 1024 tokens on every rank
    cases = [(T, False) for T in tokens] + ([(1024 * world, True)] if world > 1 and 1024 in tokens else [])
    for T, weak in cases:
        t_loc = T // world if T >= world else (1 if rank < T else 0)    # tokens of this rank
        x = torch.from_numpy(synth.activations(1234, f"c3.x{T}.r{rank}", max(t_loc, 1), H)).to(dev)[:t_loc]
        if world == 1:
            o = torch.empty((T, H), dtype=torch.float32, device=dev)
            idx = torch.empty((T, K), dtype=torch.int32, device=dev)
            tw = torch.empty((T, K), dtype=torch.float32, device=dev)
            run = lambda: layer.forward(x, o, idx, tw)
        else:
            run = lambda: layer.forward(x)
        for _ in range(3):
            run()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            run()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / steps
        if world > 1:
            t = torch.tensor([ms], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t[0])
        total = (T // world) * world if T >= world else T
        rec = {"us_per_layer": ms * 1e3, "tokens_per_s": total / ms * 1e3}
        if world > 1 and isinstance(layer, moe.P2pMoeLayer):
            layer.profile = True
            run()
            torch.cuda.synchronize()
            ph = layer.phase_ms()
            layer.profile = False
            v = torch.tensor([ph["send"], ph["experts"], ph["combine"]], device=dev, dtype=torch.float64)
            dist.all_reduce(v, op=dist.ReduceOp.MAX)
            rec["phases_us_max_over_ranks"] = {"send": float(v[0]) * 1e3, "experts": float(v[1]) * 1e3, "combine": float(v[2]) * 1e3}
        if weak:
            out["tokens_1024_per_rank"] = dict(rec, total_tokens=total)
        else:
            out["by_tokens"][str(T)] = rec
    if world > 1:
        t_loc = 64 // world
        xc = torch.from_numpy(synth.activations(1234, f"c3.x64.r{rank}", max(t_loc, 1), H)).to(dev)[:t_loc]
        chk = ep_self_check(rank, layer, xc, None)
        if rank == 0:
            out["ep_check"] = chk
    return out


def _gpu_expert_stacks(dev, seed: int, n_local: int, H: int, I: int, with_shared: bool) -> dict:
    """Expert stacks of one layer generated on the device (uniform 16-bit codes, sign-scales of magnitude about 1 with the
    1/sqrt(fan_in) gain on the output side): seeded synthetic weights for the timing runs of configuration 4, where
    forty layers' worth (15 GiB over all ranks) would take minutes to generate on the host."""
    import torch
    g = torch.Generator(device=dev)
    g.manual_seed(seed)
    n = n_local + (1 if with_shared else 0)
    def stack(k, nn):
        t = torch.randint(-32768, 32768, (n, k // 16, nn // 16, 16 * BITS), dtype=torch.int16, device=dev, generator=g)
        sign = lambda m, gain: ((torch.randint(0, 2, (n, m), device=dev, generator=g).float() * 2 - 1)
                                * (1 + 0.05 * torch.randn((n, m), device=dev, generator=g)) * gain).half()
        return t, sign(k, 1.0), sign(nn, 1.0 / np.sqrt(k))
    w = {}
    for p, (k, nn) in (("gate", (H, I)), ("up", (H, I)), ("down", (I, H))):
        t, su, sv = stack(k, nn)
        w[f"{p}_trellis"], w[f"{p}_suh"], w[f"{p}_svh"] = t[:n_local], su[:n_local], sv[:n_local]
        if with_shared:
            w[f"sh_{p}_trellis"], w[f"sh_{p}_suh"], w[f"sh_{p}_svh"] = t[n_local], su[n_local], sv[n_local]
    return w


def bench_c4(rank: int, world: int, layers: int = 40, total_tokens: int = 8448, reps: int = 3) -> dict:
    """Configuration 4: a stack of `layers` MoE layers of configuration 3's shape, every layer with its own router and
    expert weights, 8448 tokens (8192 prefill + 256 decode) split evenly over the ranks, router bias = the log of a
    Zipf(s = 1.1) popularity over a seeded rank order (full strength).  The same token batch enters every layer (what
    lies between the MoE layers of a model is outside this path).  One GPU: berth_moe_layer.  Several: experts in
    contiguous blocks (the popularity order is a seeded permutation, so popular experts are spread over the blocks),
    exchange by peer-memory stores.  Reports the time per layer, the phases of the expert-parallel layer, the rows each
    rank received, the realised expert popularity beside the Zipf law, and an estimate of the exposed exchange time:
    layer time minus the same rank's routing, expert kernels and combine measured alone on the rows it received."""
    import torch
    import torch.distributed as dist
    from berth_b200 import kernels, moe, synth
    dev = torch.device("cuda", torch.cuda.current_device())
    H, I, E, K, SI = MOE["hidden"], MOE["inter"], MOE["n_experts"], MOE["top_k"], MOE["shared_inter"]
    n_local, T = E // world, total_tokens // world
    bias = synth.zipf_router_bias(1234, "c4.bias", E, s=1.1, strength=1.0)
    # Static expert placement for a known skew: experts are renumbered so that the contiguous blocks of the ranks hold
    # equal loads -- a relabelling of the router's columns, which leaves the layer's function unchanged.  The load of an
    # expert is taken from a calibration count (the router of layer 0 on the first rank's tokens, evaluated with numpy on
    # every rank alike); experts go, most loaded first, to the least loaded rank that still has a free place.
    x_cal = synth.activations(1234, f"c4.x.r0.of{world}", T, H).astype(np.float32)
    logit_cal = x_cal @ synth.router_weight(1234, "c4.0.gate.weight", H, E).astype(np.float32) + bias[None, :]
    cal = np.bincount(np.argsort(-logit_cal, axis=1, kind="stable")[:, :K].ravel(), minlength=E)
    by_load = np.argsort(-cal, kind="stable")
    load, held = np.zeros(world, np.int64), [[] for _ in range(world)]
    for e in by_load:
        r = min((q for q in range(world) if len(held[q]) < n_local), key=lambda q: (load[q], q))
        held[r].append(int(e))
        load[r] += int(cal[e])
    place = np.array([e for r in range(world) for e in held[r]], np.int64)
    bias = np.ascontiguousarray(bias[place])
    mk = []
    for l in range(layers):
        w = {"hidden": H, "inter": I, "n_experts": n_local, "top_k": K, "bits": BITS, "cb": CB, "shared_inter": SI,
             "w_router": np.ascontiguousarray(synth.router_weight(1234, f"c4.{l}.gate.weight", H, E)[:, place]), "router_bias": bias}
        w.update(_gpu_expert_stacks(dev, 77_000 + 1000 * l + rank, n_local, H, I, True))
        mk.append(w)
    x = torch.from_numpy(synth.activations(1234, f"c4.x.r{rank}.of{world}", T, H)).to(dev)
    rec = {"workload": "c4_40_layer_moe_stack_zipf", "layers": layers, "total_tokens": T * world, "tokens_per_rank": T,
           "router_bias": "ln(rank^-1.1) over a seeded rank order, strength 1.0", "expert_weights": "generated on the device, per layer",
           "placement": "greedy by calibrated load: most loaded expert first, to the least loaded rank with a free place"}
    if world == 1:
        lays = [moe.MoeLayer(dev, w, 1) for w in mk]
        lays[0]._alloc(T)
        for l in lays[1:]:
            l.workspace, l.max_tokens = lays[0].workspace, T      # the layers run one after the other: one workspace
        o = torch.empty((T, H), dtype=torch.float32, device=dev)
        idx = torch.empty((T, K), dtype=torch.int32, device=dev)
        tw = torch.empty((T, K), dtype=torch.float32, device=dev)
        run = lambda: [l.forward(x, o, idx, tw) for l in lays]
        counts_of = lambda: torch.bincount(idx.flatten().to(torch.int64), minlength=E)
    else:
        max_rows = T * world * K + T          # room for every routed row of the batch landing on one rank
        stages = moe.GpuStages(dev, mk[0], E, max_rows=max_rows, max_rows_per_expert=1024)
        mls = [stages.layer] + [moe.MoeLayer(dev, w, 1) for w in mk[1:]]
        layer = moe.P2pMoeLayer(stages, dist.group.WORLD, E, K, max_tokens=T, max_rows=max_rows)
        rec["exchange"] = "peer-memory stores + flag barriers"
        def run():
            for ml in mls:
                stages.layer = ml
                layer.forward(x)
        counts_of = lambda: layer._cnt.view(torch.int32).view(world, E).sum(0).to(torch.int64)
    for _ in range(2):
        run()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        run()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / (reps * layers)
    if world > 1:
        t = torch.tensor([ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t[0])
    rec.update(us_per_layer=ms * 1e3, ms_per_stack=ms * layers, tokens_per_s=T * world / ms * 1e3,
               device_status=kernels.device_status(torch.cuda.current_device()))
    # realised popularity of the last layer beside the law
    c = counts_of().float().cpu().numpy()
    order = np.argsort(-c)
    law = np.arange(1, E + 1, dtype=np.float64) ** -1.1
    law = law / law.sum() * c.sum()
    rec["popularity"] = {"rows_total": float(c.sum()), "top16_rows": [int(v) for v in c[order][:16]],
                         "zipf_1.1_top16_rows": [round(float(v), 1) for v in law[:16]],
                         "note": "a token selects an expert at most once, so an expert's rows saturate at the token count",
                         "rows_per_expert_max_over_mean": float(c.max() / max(c.mean(), 1.0))}
    if world > 1:
        per_rank = layer._cnt.view(torch.int32).view(world, world, n_local).sum(dim=(0, 2)).float().cpu().numpy()
        rec["rows_per_rank"] = [int(v) for v in per_rank]
        rec["rows_per_rank_max_over_mean"] = float(per_rank.max() / max(per_rank.mean(), 1.0))
        # phases of one layer (CUDA events inside forward), max over ranks
        # (ranks aligned first, three layers, the last one counts: a rank that enters late makes the others wait in "send")
        torch.cuda.synchronize()
        dist.barrier()
        layer.profile = True
        for ml in mls[-3:]:
            stages.layer = ml
            layer.forward(x)
        torch.cuda.synchronize()
        ph = layer.phase_ms()
        layer.profile = False
        # the same rank's compute measured alone on the rows it received: routing + sort, expert kernels, combine
        n_rows = int(per_rank[rank])
        keys = torch.repeat_interleave(torch.arange(n_local, dtype=torch.int32, device=dev),
                                       layer._cnt.view(torch.int32).view(world, E)[:, rank * n_local:(rank + 1) * n_local].sum(0).to(torch.int64))
        xr = layer._recv.view(torch.float16).view(-1, H)[:max(n_rows, 1)]
        def timed(fn, n=5):
            fn()
            torch.cuda.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(n):
                fn()
            b.record()
            torch.cuda.synchronize()
            return a.elapsed_time(b) / n
        def route_sort():
            idx_, _ = stages.route(x)
            stages.sort(idx_.flatten(), 0, E)
        t_route = timed(route_sort)
        def experts_alone():
            stages.sort(keys, 0, n_local, for_experts=True)
            stages.experts(xr[:n_rows])
        t_exp = timed(experts_alone) if n_rows > 0 else 0.0
        inv = torch.arange(T * K, dtype=torch.int32, device=dev)
        tw = torch.full((T, K), 1.0 / K, dtype=torch.float32, device=dev)
        t_comb = timed(lambda: stages.combine(layer.ret_rows[: T * K], inv, tw, None))
        v = torch.tensor([ph["send"], ph["experts"], ph["combine"], t_route, t_exp, t_comb], device=dev, dtype=torch.float64)
        dist.all_reduce(v, op=dist.ReduceOp.MAX)
        send, exps, comb, t_route, t_exp, t_comb = [float(q) * 1e3 for q in v]
        rec["phases_us_max_over_ranks"] = {"send": send, "experts": exps, "combine": comb}
        rec["compute_alone_us_max_over_ranks"] = {"route_and_sort": t_route, "expert_kernels_on_received_rows": t_exp, "combine": t_comb}
        rec["exposed_exchange_us"] = max(0.0, rec["us_per_layer"] - (t_route + t_exp + t_comb))
        rec["exposed_exchange_note"] = ("time per layer of the timed stack minus the layer's own kernels run alone on the rows this rank "
                                        "received (routing+sort, expert kernels, combine; max over ranks): count publication, three flag "
                                        "barriers (waiting for the busiest rank included), peer stores of rows and outputs")
    return rec


def ep_self_check(rank: int, layer, x, w_router, n_tokens: int = 4) -> dict:
    """Correctness evidence for the expert-parallel layer inside the bench run, without the CPU checker: the first tokens of
    rank 0 are evaluated expert by expert through the dense decode linear (berth_exl3_linear on weights regenerated from the
    same seeds: only the selected experts and the shared one), combined in fp64 on the host with the layer's routing weights,
    and compared with the layer's output.  The dense linear itself is compared with the checker by the test suite."""
    import torch
    from berth_b200 import kernels, synth
    from berth_b200.kernels import Codebook, OutDtype
    H, I, E, K = MOE["hidden"], MOE["inter"], MOE["n_experts"], MOE["top_k"]
    dev = x.device
    out, idx, tw = layer.forward(x)
    torch.cuda.synchronize()
    if rank != 0 or x.shape[0] == 0:
        return {}
    n = min(n_tokens, x.shape[0])
    idx_h, tw_h, out_h = idx[:n].cpu().numpy(), tw[:n].cpu().numpy().astype(np.float64), out[:n].cpu().numpy().astype(np.float64)
    to = lambda a: torch.from_numpy(np.ascontiguousarray(a).view(np.int16)).to(dev)
    def lin(xrow, lw, k, nn):
        c = torch.empty((1, nn), dtype=torch.float16, device=dev)
        ah = torch.empty((1, k), dtype=torch.float16, device=dev)
        kernels.exl3_linear(xrow, to(lw["trellis"]), c, to(lw["suh"]), ah, to(lw["svh"]), 1, k, nn, BITS, Codebook(CB), OutDtype.F16)
        return c
    def routed(proj, e, k, nn):     # the weights bench_moe gives expert e
        return {"trellis": synth.trellis(1234, f"c3.experts.{proj}.{e}.trellis", k, nn, BITS),
                "suh": synth.sign_scale(1234, f"c3.experts.{proj}.{e}.suh", k),
                "svh": synth.sign_scale(1234, f"c3.experts.{proj}.{e}.svh", nn, 1.0 / np.sqrt(k))}
    def shared(proj, k, nn):
        return synth.linear_weights(1234, f"c3.shared_expert.{proj}", k, nn, BITS, fan_in_gain=True)
    def mlp(xrow, get):
        g, u = lin(xrow, get("gate_proj", H, I), H, I), lin(xrow, get("up_proj", H, I), H, I)
        a = torch.empty_like(g)
        kernels.ops.silu_mul(g, u, a, I, 0.0)
        return lin(a, get("down_proj", I, H), I, H).double().cpu().numpy()[0]
    worst = 0.0
    for t in range(n):
        xrow = x[t:t + 1].contiguous()
        y = np.zeros(H)
        for s_ in range(K):
            e = int(idx_h[t, s_])
            y += tw_h[t, s_] * mlp(xrow, lambda proj, k, nn: routed(proj, e, k, nn))
        y += mlp(xrow, shared)
        worst = max(worst, float(np.abs(out_h[t] - y).max() / np.sqrt((y ** 2).mean())))
    return {"tokens_checked": n, "experts_per_token": K, "shared_expert": True, "max_abs_diff_over_row_rms": worst,
            "against": "the same tokens through the dense decode linear, expert by expert, combined in fp64 on the host"}


# ------------------------------------------------------------------ CPU arm

def cpu_pass(m: int, passes: int):
    """The CPU oracle (a restatement of the path; berth ships no CPU implementation) on `passes`
    full seven-matrix passes.  Returns (GB/s, seconds, threads)."""
    from berth_b200 import synth
    from oracle import exl3_oracle as orc
    orc.build()
    # all the host cores this process may use (a launcher that starts one rank per GPU sets OMP_NUM_THREADS=1)
    orc.set_num_threads(len(os.sched_getaffinity(0)))
    ws = {name: synth.linear_weights(synth.MASTER_SEED, f"cpu.{name}", k, n, BITS, fan_in_gain=True) for name, k, n, _, _ in SHAPES}
    x = {"x": synth.activations(1234, "cpu.x", m, HIDDEN), "xa": synth.activations(1234, "cpu.xa", m, HIDDEN),
         "attn": synth.activations(1234, "cpu.attn", m, QDIM)}
    t0 = time.perf_counter()
    for _ in range(passes):
        g, _ = orc.linear(x["x"], ws["gate"]["trellis"], ws["gate"]["suh"], ws["gate"]["svh"], HIDDEN, INTER, BITS, CB, False)
        u, _ = orc.linear(x["x"], ws["up"]["trellis"], ws["up"]["suh"], ws["up"]["svh"], HIDDEN, INTER, BITS, CB, False)
        act = orc.silu_mul(g, u)
        orc.linear(act, ws["down"]["trellis"], ws["down"]["suh"], ws["down"]["svh"], INTER, HIDDEN, BITS, CB, True)
        for name, k, n, f, src in SHAPES[3:]:
            orc.linear(x[src], ws[name]["trellis"], ws[name]["suh"], ws[name]["svh"], k, n, BITS, CB, bool(f))
    dt = time.perf_counter() - t0
    return step_bytes(m) * passes / dt / 1e9, dt, orc.num_threads()


def run_reference(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    m = args.m
    for _ in range(min(args.warmup, 1)):
        cpu_pass(m, 1)
    gbs, dt, threads = cpu_pass(m, args.steps)
    line = {
        "impl": "reference", "metric": METRIC, "value": gbs, "unit": "GB/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": min(args.warmup, 1), "ms_per_step": dt / args.steps * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "fp16 x trellis-u16, fp32 accumulate",
        "data": "synthetic",
        "config": {"workload": "c1_dense_27b_decode_stack_4bpw", "m": m, "bits": BITS, "codebook": "mul1",
                   "bytes_per_step": step_bytes(m)},
        "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": threads, "kind": "port",
                         "sample": f"{args.steps} full seven-matrix passes at m={m} (berth has no CPU path; "
                                   "this is the repo's CPU oracle, OpenMP)"},
        "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


# ------------------------------------------------------------------ main

def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--m", type=int, default=1, help="token rows per step (1, 8 or 32 in configuration 1)")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true", help="skip the prefill (configuration 2) and MoE (configuration 3) measurements")
    ap.add_argument("--only", default="all", choices=["all", "prefill", "moe", "lm_head", "c4", "decode_rate"],
                    help="run one of the extra measurements alone and print its record (for profiling; not the contract line)")
    ap.add_argument("--c4-layers", type=int, default=40, help="layers of the configuration-4 stack (0 = skip it)")
    ap.add_argument("--moe-tokens", type=int, nargs="*", default=[1, 64, 1024], help="token counts of the MoE measurement")
    args = ap.parse_args()
    if args.impl == "reference":
        if args.steps > 10:
            args.steps = 3
        run_reference(args)
        return

    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a GPU: berth_b200 has no CPU path")
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    warmup = max(args.warmup, 3)
    if args.only != "all":
        if args.only == "prefill":
            rec = bench_prefill(rank, reps=max(1, min(args.steps, 5)))
        elif args.only == "lm_head":
            rec = bench_lm_head(rank, reps=max(1, min(args.steps, 20)))
        elif args.only == "c4":
            rec = bench_c4(rank, world, layers=max(1, args.c4_layers))
        elif args.only == "decode_rate":
            rec = bench_decode_rate() if rank == 0 else None
        else:
            rec = bench_moe(rank, world, steps=args.steps, tokens=tuple(args.moe_tokens))
        if rank == 0:
            print(json.dumps(rec))
        if world > 1:
            dist.destroy_process_group()
        return

    stack = DecodeStack(args.m, rank)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-resident timing
    for i in range(warmup):
        stack.step(i)
    sampler = ClockSampler(local)
    barrier()
    if rank == 0:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for i in range(args.steps):
        stack.step(i)
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1)
    # ---- end to end with host buffers
    for i in range(3):
        stack.step_e2e(i)
    barrier()
    t0 = time.perf_counter()
    for i in range(args.steps):
        stack.step_e2e(i)
    barrier()
    e2e_ms = (time.perf_counter() - t0) * 1e3
    # ---- dominant kernel alone
    gate_ms, gate_bytes, gate_what, gate_name = stack.time_dominant_kernel(max(4, args.steps // 8))
    # nvidia-smi samples every 100 ms; a short timed region ends before the first sample, so the same
    # step loop is repeated for about 1.5 s under the sampler (same kernels, same clocks regime).
    t_end = time.perf_counter() + 1.5
    i = 0
    while time.perf_counter() < t_end:
        stack.step(i)
        i += 1
        if i % 64 == 0:
            torch.cuda.synchronize()
    torch.cuda.synchronize()
    clocks = sampler.stop() if rank == 0 else None
    if clocks is not None:
        clocks["window"] = "timed region + end-to-end region + 1.5 s repeat of the same step loop"
    extras = rank == 0 and not args.no_extras
    rows_extra = [bench_rows(stack, rank, mm, max(20, args.steps // 4)) for mm in (8, 32) if mm != args.m] if extras else None
    c0 = bench_c0(rank) if extras else None
    decode_rate = bench_decode_rate() if extras else None
    prefill = bench_prefill(rank) if (rank == 0 and not args.no_extras) else None
    lm_head = bench_lm_head(rank) if (rank == 0 and not args.no_extras) else None
    moe_res = None if args.no_extras else bench_moe(rank, world)
    c4 = None if (args.no_extras or args.c4_layers < 1) else bench_c4(rank, world, layers=args.c4_layers)

    if world > 1:
        t = torch.tensor([ms, e2e_ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, e2e_ms = float(t[0]), float(t[1])

    if rank == 0:
        sb = step_bytes(args.m)
        value = sb * args.steps * world / (ms * 1e-3) / 1e9
        e2e = sb * args.steps * world / (e2e_ms * 1e-3) / 1e9
        peak, peak_kind = peaks()
        achieved = gate_bytes / (gate_ms * 1e-3) / 1e9
        line = {
            "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps, "warmup": warmup,
            "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "fp16 x trellis-u16, fp32 accumulate", "data": "synthetic",
            "config": {"workload": "c1_dense_27b_decode_stack_4bpw", "m": args.m, "bits": BITS, "codebook": "mul1",
                       "bytes_per_step": sb, "layers_cycled": LAYERS,
                       "l2": f"{LAYERS} distinct layers ({LAYERS * sb / 1e6:.0f} MB) cycled; inputs larger than L2",
                       "qkv": "one launch over the three matrices, as berth's attention layers run them (berth_ops_mgemm; up to four rows the integer-path multi-matrix launch)",
                       "parallelism": "replicas" if world > 1 else "single"},
            "frac_of_hbm_peak": value / world / peak, "peak_kind": peak_kind,
            "tokens_per_s": args.m * args.steps * world / (ms * 1e-3),
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "traffic": NCU_TRAFFIC_GATE_UP_BYTES if args.m == 1 else None, "kernel": gate_name,
                         "launch": f"{gate_what} m={args.m}: {gate_bytes} algorithmic bytes in {gate_ms * 1e3:.2f} us",
                         "peak_kind": f"of {peak_kind}"},
            "e2e": {"value": e2e, "unit": "GB/s", "h2d_bytes_per_step": stack.h2d_bytes,
                    "d2h_bytes_per_step": stack.d2h_bytes, "ms_per_step": e2e_ms / args.steps},
            "gpu_launches": stack.launches_per_step * args.steps,
            "clocks": clocks,
            "rows": rows_extra, "c0": c0, "decode_rate": decode_rate,
            "prefill": prefill, "lm_head": lm_head,
            "moe": moe_res, "c4": c4,
        }
        if not args.no_cpu_baseline and world == 1:
            gbs, dt, threads = cpu_pass(args.m, 2)
            line["cpu_baseline"] = {"value": gbs, "unit": "GB/s", "cores": threads, "kind": "port",
                                    "sample": f"2 full seven-matrix passes at m={args.m}, {dt:.1f} s "
                                              "(the repo's CPU oracle; berth ships no CPU path)"}
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
