#!/usr/bin/env python
"""Benchmark of the batch-shared block-sparse activation GEMM on B200.

    python bench.py --gpus N --steps K --warmup W            # this repository's CUDA path
    python bench.py --impl reference --steps K --warmup W    # the reference's CPU torch path

Workload (synthetic, seeded): the Llama-2-7B down-projection, X fp16 [B, 11008] ~ Laplace(0,1),
W fp16 [4096, 11008] ~ N(0, 0.02^2), 172 blocks of 64 channels, batch-shared top-k masks keeping
34 / 62 / 83 blocks at B = 2 / 16 / 64 (block sparsity 0.803 / 0.638 / 0.520).  One "step" is the
three masked GEMMs B = 2, 16, 64.  The metric is the active-weight HBM bandwidth of a step:
(34 + 62 + 83) * 64 * 4096 * 2 bytes divided by the step time.

Timing: the K timed steps run as list launches (bas_list_*: 16 steps = 48 independent calls per
persistent launch, each call on one of 16 rotating weight copies so that a weight tile is never
found in L2), bracketed by CUDA events on the launching stream; the region is timed five times and
the median reported.  Activations and masks are resident before a launch.  The same calls as
single launches - pipelined several deep (ids and X declared stable), one call deep, and with no
promises, as the drop-in wrappers launch - are reported in per_batch beside the headline, with
dense cuBLAS timed the same way; `speedup_vs_cublas` is the like-for-like ratio (one call at a
time, cold L2, no promises).  With --gpus N every rank runs the same workload on its own GPU
(independent decode replicas, no collective on the data path); the sharded layer stack, which does
use collectives, is reported in `layer_stack` with a parity check against the unsharded product.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
PKG = ROOT / "towards-batched-activation-sparsity_b200"
for _p in (str(ROOT), str(PKG)):
    if _p not in sys.path:
        sys.path.insert(0, _p)

K_IN, N_OUT, NB = 11008, 4096, 172
BATCHES = (2, 16, 64)
N_KEEP = {2: 34, 16: 62, 64: 83}                     # round((1 - s) * 172), s = 0.803 / 0.638 / 0.520
SPARSITY = {2: 0.803, 16: 0.638, 64: 0.520}
SLAB_BYTES = 64 * N_OUT * 2                          # one active 64-row weight slab
STEP_BYTES = sum(N_KEEP.values()) * SLAB_BYTES       # algorithmic bytes of one step
ROTATE = 16                                          # weight copies cycled through (cold L2)
# dram__bytes_read.sum + dram__bytes_write.sum of one list launch of 16 steps (ncu; the command is in the
# summary under profiles/ named for the list kernel and this workload)
LIST_TRAFFIC_16_STEPS = 1_511_300_000
TRAFFIC_NOTE = ("ncu capture of one 16-step launch (python bench.py --profile-list 16), scaled by the steps of the timed launch: "
                "traffic grows in proportion to the calls walked")
METRIC = "block-sparse GEMM active-weight HBM bandwidth, down_proj, batch 2/16/64 (us & speedup vs cuBLAS in per_batch)"
WORKLOAD = ("llama2-7b down_proj X[B,11008] Laplace x W[4096,11008] N(0,0.02), B in {2,16,64}, "
            "batch-shared top-k block masks 34/62/83 of 172")


_STDOUT_FD = None


def _emit(line: dict) -> None:
    data = (json.dumps(line) + "\n").encode()
    if _STDOUT_FD is None:
        sys.stdout.write(data.decode())
        sys.stdout.flush()
    else:
        os.write(_STDOUT_FD, data)


def _peaks() -> dict:
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return {"hbm_gbs": float(d["hbm_gbs"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "source": "fallback"}


# ---------------------------------------------------------------------------------------------
# CPU leg: the reference's own CPU-runnable formulation, restated in oracle/
# ---------------------------------------------------------------------------------------------

def _cpu_inputs():
    import torch
    from oracle import bas_oracle as O

    w = torch.from_numpy(O.make_weight(N_OUT, K_IN, seed=0))
    xs = {b: torch.from_numpy(O.make_activations(b, K_IN, seed=1000 + b, dist="laplace")) for b in BATCHES}
    return w, xs


def _cpu_step(w, xs) -> None:
    from oracle import bas_oracle as O

    for b in BATCHES:
        ids = O.select_active_blocks_torch_cpu(xs[b].reshape(b, 1, K_IN), N_KEEP[b] / NB, O.SCORE_NORM)
        O.masked_linear_torch_cpu(xs[b], w, ids.numpy())


def _cpu_config1() -> dict:
    """The specification's CPU-runnable case: X [16, 4096] N(0,1), W [4096, 4096] N(0, 0.02), seed 0, the
    32 of 64 blocks with the largest batch-summed L2 norm; selection + masked linear on the host cores."""
    import torch
    from oracle import bas_oracle as O

    x = torch.from_numpy(O.make_activations(16, 4096, seed=0))
    w = torch.from_numpy(O.make_weight(4096, 4096, seed=0))
    def once():
        ids = O.select_active_blocks_torch_cpu(x.reshape(16, 1, 4096), 0.5, O.SCORE_NORM)
        return O.masked_linear_torch_cpu(x, w, ids.numpy())
    for _ in range(3):
        once()
    times = []
    for _ in range(20):
        t0 = time.perf_counter()
        once()
        times.append(time.perf_counter() - t0)
    med = statistics.median(times)
    return {"ms": round(med * 1e3, 4), "active_weight_gbs": round(32 * 64 * 4096 * 2 / med / 1e9, 2),
            "what": "X[16,4096] x W[4096,4096], 32 of 64 blocks kept by batch-summed block L2 norm, fp16 torch CPU"}


def cpu_baseline(max_seconds: float = 12.0, max_steps: int = 30) -> dict:
    """Time the reference's CPU path (selection + F.linear(x * blockmask, W), fp16) on all host cores."""
    import torch

    torch.set_num_threads(os.cpu_count() or 1)
    w, xs = _cpu_inputs()
    for _ in range(2):
        _cpu_step(w, xs)
    times = []
    t_end = time.perf_counter() + max_seconds
    while len(times) < max_steps and (time.perf_counter() < t_end or len(times) < 3):
        t0 = time.perf_counter()
        _cpu_step(w, xs)
        times.append(time.perf_counter() - t0)
    med = statistics.median(times)
    return {"value": STEP_BYTES / med / 1e9, "unit": "GB/s", "cores": torch.get_num_threads(), "kind": "port",
            "sample": f"{len(times)} steps of the same workload (selection + fp16 F.linear on the masked input, "
                      f"torch CPU), median {med * 1e3:.2f} ms per step",
            "ms_per_step": med * 1e3, "single_masked_linear": _cpu_config1()}


def run_reference(args) -> None:
    """--impl reference: the reference's CPU implementation of the path, timed on the host cores."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    import torch

    torch.set_num_threads(os.cpu_count() or 1)
    w, xs = _cpu_inputs()
    for _ in range(max(1, min(args.warmup, 3))):
        _cpu_step(w, xs)
    steps = max(1, min(args.steps, 40))                 # bounded sample: a step costs tens of ms on CPU
    t0 = time.perf_counter()
    for _ in range(steps):
        _cpu_step(w, xs)
    dt = (time.perf_counter() - t0) / steps
    val = STEP_BYTES / dt / 1e9
    line = {
        "impl": "reference", "metric": METRIC, "value": val, "unit": "GB/s", "n_gpus": args.gpus, "steps": steps,
        "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": {"workload": WORKLOAD, "path": "torch CPU: _select_active_blocks + F.linear(x*blockmask, W)"},
        "cpu_baseline": {"value": val, "unit": "GB/s", "cores": torch.get_num_threads(), "kind": "port",
                         "sample": f"{steps} steps of the same workload on the host cores"},
        "e2e": {"value": val, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    _emit(line)


# ---------------------------------------------------------------------------------------------
# GPU leg
# ---------------------------------------------------------------------------------------------

class ClockSampler:
    """nvidia-smi clocks and throttle reasons, sampled while the timed regions run."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, uuid: str):
        self.tmp = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.proc = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={uuid}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "50"], stdout=self.tmp, stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self) -> dict:
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        self.tmp.flush()
        rows = [r.split(", ") for r in Path(self.tmp.name).read_text().strip().splitlines() if r.strip()]
        os.unlink(self.tmp.name)
        sm, reasons = [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in rows:
            if len(r) < 7:
                continue
            try:
                sm.append(float(r[0]))
                out["sm_max_mhz"] = float(r[1])
            except ValueError:
                continue
            for name, v in zip(names, r[3:7]):
                if v.strip().lower() == "active":
                    reasons.add(name)
        if sm:
            out["sm_mhz"] = statistics.median(sm)
        out["reasons"] = sorted(reasons)
        out["samples"] = len(sm)
        return out


def _graph_time_us(torch, stream, build, calls_per_graph: int, reps: int, repeats: int = 3) -> float:
    """Median over `repeats` of: capture `build()` once, replay `reps` times between two events.
    Returns microseconds per call."""
    with torch.cuda.stream(stream):
        build()
        build()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=stream):
        build()
    torch.cuda.synchronize()
    vals = []
    for _ in range(repeats):
        with torch.cuda.stream(stream):
            g.replay()
            e0 = torch.cuda.Event(enable_timing=True)
            e1 = torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            for _ in range(reps):
                g.replay()
            e1.record(stream)
        torch.cuda.synchronize()
        vals.append(e0.elapsed_time(e1) * 1e3 / (reps * calls_per_graph))
    return float(statistics.median(vals))


def _layer_stack(torch, dist, dev, world, rank, stream, fuse=False, allreduce="nccl") -> dict:
    """The Llama-2-7B decode-step linear stack (32 layers x 7 masked projections, B = 16, sparsity
    0.638), column-/row-parallel over the ranks with the row-parallel sums by NCCL all-reduce or inside
    the contraction kernel: one CUDA graph per step where NCCL allows capture, timed by CUDA events,
    max over ranks.  Before timing, one step is checked against the unsharded product (fp32, first
    layer) and the masks are compared across the ranks.  On one GPU the step is also timed as ONE
    persistent launch over the list of its calls, with the model's dependencies and without."""
    from bas import tp

    stack = tp.DecodeLinearStack(32, 16, 0.638, dev, world, rank, fuse_shared_inputs=fuse, allreduce=allreduce)
    parity = stack.parity_check(layers=1)
    if not (parity["ids_equal"] and parity["max_err"] <= 2e-3):
        raise SystemExit(f"sharded stack disagrees with the unsharded product: {parity}")

    def meet():
        # Kernels that exchange partial sums wait inside the kernel for the other ranks (bounded, about a
        # second): the ranks line up before such launches, so that host-side work of different length
        # (graph capture, allocator trimming) on one rank is not mistaken for a rank that stays away.
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    def timed(step):
        meet()
        with torch.cuda.stream(stream):
            for _ in range(3):
                step()
        torch.cuda.synchronize()
        mode = "cuda graph"
        try:
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=stream):
                step()
            run = g.replay
        except Exception as exc:      # a collective that refuses capture: time eager launches instead
            mode = f"eager ({type(exc).__name__})"
            run = step
        meet()
        reps = 10
        with torch.cuda.stream(stream):
            run()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with torch.cuda.stream(stream):
            e0.record(stream)
            for _ in range(reps):
                run()
            e1.record(stream)
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / reps
        if world > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms, mode

    def gbs(ms):
        return round(stack.active_bytes / (ms * 1e-3) / 1e9, 1)

    ms, mode = timed(stack.step)
    extra = {}
    if world == 1 or allreduce == "in_kernel":
        # the whole step as one persistent launch per rank: the calls wait for one another as in the model;
        # on several ranks the row-parallel calls add their outputs over the ranks inside that launch ...
        lst = stack.make_list(dependencies=True)
        ms_dep, _ = timed(lst.run)
        status = lst.read_status()
        # ... and checked like the per-call step (the list wrote the same output buffers)
        par_l = stack.parity_check_outputs(layers=1)
        info = lst.info()
        lst.close()
        bad = int(status != 0 or not par_l["max_err"] <= 2e-3)
        if world > 1:
            t = torch.tensor([bad], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            bad = int(t.item())
        if bad and world == 1:
            raise SystemExit(f"one-launch stack: device status {status:#x}, parity {par_l}")
        if bad:
            # reported, not fatal: the per-call numbers of this line stand on their own
            print(f"one-launch stack (rank {rank} of {world}): device status {status:#x}, parity {par_l}", file=sys.stderr)
            extra["one_launch"] = {"error": f"device status {status:#x} on rank {rank}", "parity": par_l}
        else:
            extra["one_launch"] = {
                "ms_per_step": round(ms_dep, 4), "active_weight_gbs": gbs(ms_dep), "launches_per_step": 1,
                "max_err_vs_unsharded_fp32": round(par_l["max_err"], 6), "ctas": info["ctas"],
                "note": "bas_list_run: one persistent kernel per rank walks the step's calls; every call waits for the call "
                        "whose output its input is in the model (q/k/v <- down of the layer before, o <- v, gate/up <- o, "
                        "down <- up); on several ranks o and down add their outputs over the ranks inside the kernel"}
    if "one_launch" in extra and "error" not in extra["one_launch"]:
        # the same launch with every mask computed inside it from the activation it belongs to (what a decode step
        # has to do): a selection entry per distinct input, ranked by the calls that use it
        for o in [it[3] for it in stack.items]:
            o.zero_()
        lst = stack.make_list(dependencies=True, select=True)
        ms_sel, _ = timed(lst.run)
        status = lst.read_status()
        par_s = stack.parity_check_outputs(layers=1)
        lst.close()
        bad = int(status != 0 or not par_s["max_err"] <= 2e-3)
        if world > 1:
            t = torch.tensor([bad], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            bad = int(t.item())
        if bad and world == 1:
            raise SystemExit(f"one-launch stack with selection: device status {status:#x}, parity {par_s}")
        extra["one_launch"]["with_selection"] = (
            {"error": f"device status {status:#x} on rank {rank}", "parity": par_s} if bad else
            {"ms_per_step": round(ms_sel, 4), "max_err_vs_unsharded_fp32": round(par_s["max_err"], 6),
             "note": "masks computed inside the launch: one selection entry per distinct input (four per layer when q+k+v "
                     "and gate+up are stacked, seven otherwise: this stack generates an input per projection), each scored "
                     "when its input is complete; the outputs equal those of the precomputed masks"})
    if world > 1 and "one_launch" in extra and "error" not in extra["one_launch"].get("with_selection", {"error": 1}):
        # ... and with every rank scoring only its own K-shard of the row-parallel calls' inputs (what a chained
        # forward leaves a rank with): the block scores are exchanged inside the launch, one global top-k
        for o in [it[3] for it in stack.items]:
            o.zero_()
        lst = stack.make_list(dependencies=True, select=True, sharded_select=True)
        ms_sh, _ = timed(lst.run)
        status = lst.read_status()
        par_h = stack.parity_check_outputs(layers=1)
        lst.close()
        bad = int(status != 0 or not par_h["max_err"] <= 2e-3)
        t = torch.tensor([bad], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        extra["one_launch"]["with_sharded_selection"] = (
            {"error": f"device status {status:#x} on rank {rank}", "parity": par_h} if int(t.item()) else
            {"ms_per_step": round(ms_sh, 4), "max_err_vs_unsharded_fp32": round(par_h["max_err"], 6),
             "note": "as with_selection, but the entries of o and down see this rank's K-shard only and the ranks "
                     "exchange the block scores through the exchange area inside the launch"})
    if world == 1:
        lst = stack.make_list(dependencies=False)
        ms_free, _ = timed(lst.run)
        status = lst.read_status()
        lst.close()
        if status != 0:
            raise SystemExit(f"one-launch stack without dependencies: device status {status}")
        extra["one_launch"]["no_dependencies"] = {"ms_per_step": round(ms_free, 4), "active_weight_gbs": gbs(ms_free),
                                                   "note": "the same list with no call waiting for another"}
        if not fuse:
            # throughput probe: the same 224 single launches with every input declared stable
            stack.independent_calls = True
            ms_ind, _ = timed(stack.step)
            stack.independent_calls = False
            extra["independent_calls"] = {"ms_per_step": round(ms_ind, 4), "active_weight_gbs": gbs(ms_ind),
                                          "note": "single launches, every call declares ids and X stable; ms_per_step above "
                                                  "declares X stable only for k, v and up, which read what q / gate have read"}
    stack.close()
    return {**extra, "layers": 32, "linears_per_step": len(stack.items), "batch": 16, "sparsity": 0.638,
            "parallelism": f"tp{world}: column-parallel q/k/v/gate/up, row-parallel o/down + "
                           + ("all-reduce" if allreduce == "nccl" else "sum inside the contraction kernel"),
            "ms_per_step": round(ms, 4), "active_weight_gb_per_step": round(stack.active_bytes / 1e9, 3),
            "active_weight_gbs": gbs(ms), "launch": mode,
            "tp_parity": {"checked": parity["checked"], "max_err": round(parity["max_err"], 6), "ids_equal": parity["ids_equal"]}}


def _two_d_chain(torch, ops, O, dev, stream) -> dict:
    """up -> down of one Llama-2-7B layer (B = 16) with output-block sparsity: up computes only the 62 of 172
    intermediate blocks that down's mask keeps and writes them side by side, down reads that compact
    activation (the reference's 2-D kernels and compact chaining, kernels/...:2289-2894, 3411-3467), against the
    same pair with up computing all its columns.  One list launch per pair, eight rotating weight pairs (cold L2)."""
    batch, hidden, inter, rot = 16, 4096, 11008, 8
    k_up, k_down = 23, 62
    x = torch.from_numpy(O.make_activations(batch, hidden, seed=500)).to(dev)
    k_ids = torch.from_numpy(O.random_active_blocks(hidden // 64, k_up, seed=501)).to(dev)
    mid_ids = torch.from_numpy(O.random_active_blocks(inter // 64, k_down, seed=502)).to(dev)
    wu = ops.pack_weight(torch.from_numpy(O.make_weight(inter, hidden, seed=503)).to(dev))
    wd = ops.pack_weight(torch.from_numpy(O.make_weight(hidden, inter, seed=504)).to(dev))
    wus, wds = [wu.clone() for _ in range(rot)], [wd.clone() for _ in range(rot)]
    mid_full = torch.zeros(batch, inter, dtype=torch.float16, device=dev)
    mid_comp = torch.zeros(batch, k_down * 64, dtype=torch.float16, device=dev)
    y = torch.zeros(batch, hidden, dtype=torch.float16, device=dev)
    plain = [ops.GemmList([{"x": x, "packed": wus[i], "out": mid_full, "ids": k_ids},
                           {"x": mid_full, "packed": wds[i], "out": y, "ids": mid_ids, "depends_on": 0}]) for i in range(rot)]
    two_d = [ops.GemmList([{"x": x, "packed": wus[i], "out": mid_comp, "ids": k_ids, "n_ids": mid_ids, "out_compact": True, "n": inter},
                           {"x": mid_comp, "packed": wds[i], "out": y, "ids": mid_ids, "x_compact": True, "k": inter, "depends_on": 0}])
             for i in range(rot)]

    def run(lists):
        def go():
            for l in lists:
                l.run()
        return go

    us_plain = _graph_time_us(torch, stream, run(plain), rot, 20)
    y_plain = y.clone()
    us_2d = _graph_time_us(torch, stream, run(two_d), rot, 20)
    torch.cuda.synchronize()
    # the same blocks in the same order; the column tiles differ (64 wide against the even split), and with them
    # which of a CTA's accumulators a block's partial sum lands in: equal to fp32 rounding
    diff = float((y.float() - y_plain.float()).abs().max() / y_plain.float().abs().max().clamp_min(1e-30))
    if not diff <= 2e-3:
        raise SystemExit(f"2-D chain: differs from the plain pair by {diff}")
    for l in plain + two_d:
        if l.read_status() != 0:
            raise SystemExit("2-D chain: device status")
        l.close()
    bytes_plain = (k_up * inter + k_down * hidden) * 64 * 2
    bytes_2d = (k_up * k_down * 64 + k_down * hidden) * 64 * 2
    return {"batch": batch, "up_active_blocks": k_up, "down_active_blocks": k_down,
            "pair_us": round(us_plain, 3), "pair_2d_us": round(us_2d, 3), "speedup": round(us_plain / us_2d, 3),
            "weight_mb": round(bytes_plain / 1e6, 2), "weight_mb_2d": round(bytes_2d / 1e6, 2), "max_diff_vs_plain": round(diff, 6),
            "note": "one list launch of [up, down]; 2-D: up computes only the intermediate blocks that down keeps, "
                    "compact, and down reads the compact activation"}


def _sweep_gate_up(torch, ops, abi, O, dev, stream, peaks) -> dict:
    """The sparsity sweep of the specification on the gate/up shape: X [B, 4096] N(0,1), W [11008, 4096],
    B in {1..64}, block sparsity 0 .. 0.95 in steps of 0.05, top-k masks by block L2 norm; per point the
    masked GEMM as the drop-in wrappers launch it (single launches, no promises) against dense cuBLAS,
    both on 8 rotating weight copies (cold L2).  The reference's tuner walks the same grid
    (scripts/profile_kernel_configs.py:86-216).  Every point is also appended, as it is measured, to a
    JSON-lines file in the run's output folder."""
    k, n, nb, rot = 4096, 11008, 64, 8
    w = torch.from_numpy(O.make_weight(n, k, seed=3)).to(dev)
    packed = [ops.pack_weight(w) for _ in range(rot)]
    dense_wt = [w.t().contiguous() for _ in range(rot)]
    log = None
    try:
        (ROOT / "gpurun_out").mkdir(exist_ok=True)
        log = open(ROOT / "gpurun_out" / "sweep_gate_up.jsonl", "w")
    except OSError:
        log = None
    sparsities = [round(0.05 * i, 2) for i in range(20)]
    out = {"shape": "X[B,4096] x W[11008,4096], 64 blocks", "sparsity": sparsities, "per_batch": {},
           "protocol": "single launches with no promises vs torch.mm, 8 rotating weight copies (cold L2), CUDA-graph replays"}
    for b in (1, 2, 4, 8, 16, 32, 64):
        x = torch.from_numpy(O.make_activations(b, k, seed=300 + b)).to(dev)
        y = torch.zeros(b, n, dtype=torch.float16, device=dev)
        yd = torch.zeros(b, n, dtype=torch.float16, device=dev)

        def dense():
            for c in range(rot):
                torch.mm(x, dense_wt[c], out=yd)

        dense_us = _graph_time_us(torch, stream, dense, rot, 8, repeats=2)
        us_row, sp_row = [], []
        for sp in sparsities:
            n_keep = O.n_keep_from_density(1.0 - sp, nb)
            ids = ops.select_topk(x, n_keep, abi.SCORE_NORM)[0].clone()

            def sparse():
                for c in range(rot):
                    ops.gemm(x, packed[c], y, ids=ids)

            us = _graph_time_us(torch, stream, sparse, rot, 8, repeats=2)
            us_row.append(round(us, 2))
            sp_row.append(round(dense_us / us, 3))
            if log is not None:
                log.write(json.dumps({"batch": b, "sparsity": sp, "active_blocks": n_keep, "us": us, "dense_cublas_us": dense_us,
                                      "speedup": dense_us / us, "gbs": n_keep * 64 * n * 2 / us / 1e3}) + "\n")
                log.flush()
        first_win = next((sparsities[i] for i, v in enumerate(sp_row) if v >= 1.0), None)
        out["per_batch"][str(b)] = {"dense_cublas_us": round(dense_us, 2), "us": us_row, "speedup_vs_cublas": sp_row,
                                    "lowest_sparsity_faster_than_dense": first_win}
    if log is not None:
        log.close()
    del packed, dense_wt
    torch.cuda.empty_cache()
    return out


def _reference_triton(torch, O, dev, stream, xs, ids_by_batch) -> dict:
    """The reference's own Triton kernels (kernels/shared_mask_batched_triton_min_runtime.py:684-733,
    814-874, 1150-1216, 1898-1988, through its wrappers :1064-1454), JIT-compiled for this GPU from the
    copy under baseline/_ref and timed with the protocol of per_batch.no_promises_us: the best of the
    index-list and bitmap families with split-K 1, 2, 4, 8 per batch size."""
    import importlib.util

    path = ROOT / "baseline" / "_ref" / "kernels" / "shared_mask_batched_triton_min_runtime.py"
    if not path.exists():
        return {"unavailable": "baseline/_ref/kernels is not filled (python baseline/fill_ref.py)"}
    for key, val in (("TEAL_EXP_ENABLE_SPLIT_K_1D", "0"), ("TEAL_EXP_USE_RUN_COMPRESSED_METADATA", "0"),
                     ("TEAL_EXP_SORT_ACTIVE_BLOCKS", "0")):      # as the reference's scripts set them before importing
        os.environ.setdefault(key, val)
    try:
        spec = importlib.util.spec_from_file_location("reference_triton_kernels", path)
        ref = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(ref)
    except Exception as exc:
        return {"unavailable": f"import failed: {type(exc).__name__}: {exc}"[:200]}
    rot = 8
    ws = [torch.from_numpy(O.make_weight(N_OUT, K_IN, seed=0)).to(dev) for _ in range(rot)]
    out = {}
    for b in BATCHES:
        x3 = xs[b].reshape(b, 1, K_IN)
        y3 = torch.zeros(b, 1, N_OUT, dtype=torch.float16, device=dev)
        ids = ids_by_batch[b]
        bitmap = ref._build_active_k_bitmap(ids, NB, dev)
        tile = dict(tile_b=16 if b <= 16 else 32, tile_n=64, tile_warps=4, tile_stages=3)
        best, errors = None, []
        for kind, sk in [("bitmap", 1), ("naive", 1)] + [(f, kk) for kk in (2, 4, 8) for f in ("naive", "bitmap")]:
            def call(c, kind=kind, sk=sk):
                if kind == "naive":
                    ref._prepacked_block_sparse_gemm_from_active_blocks_splitk(
                        x3, ws[c], ids, y3, cache_prefix=f"bench{c}", num_split_k=sk, **tile)
                elif sk == 1:
                    ref._prepacked_block_sparse_gemm_from_active_blocks_bitmap_preload(
                        x3, ws[c], ids, y3, cache_prefix=f"bench{c}", total_k_blocks=NB, prebuilt_bitmap=bitmap)
                else:
                    ref._prepacked_block_sparse_gemm_from_active_blocks_bitmap_preload_splitk(
                        x3, ws[c], ids, y3, cache_prefix=f"bench{c}", total_k_blocks=NB, prebuilt_bitmap=bitmap,
                        num_split_k=sk, **tile)

            def chain():
                for c in range(rot):
                    call(c)

            try:
                us = _graph_time_us(torch, stream, chain, rot, 20, repeats=2)
            except Exception as exc:
                errors.append(f"{kind}/K{sk}: {type(exc).__name__}"[:60])
                torch.cuda.synchronize()
                continue
            if best is None or us < best[0]:
                best = (us, kind, sk)
        if best is None:
            out[str(b)] = {"unavailable": "; ".join(errors)[:200]}
        else:
            out[str(b)] = {"us": round(best[0], 2), "family": best[1], "split_k": best[2]}
    del ws
    torch.cuda.empty_cache()
    return out


def _thesis_protocol() -> dict:
    """The reference's own two-step kernel benchmark, both scripts unmodified against the drop-in
    module (bas/refscripts.py): mean kernel speed-up over dense per batch size over the thesis's 55
    per-step oracle schedules x 224 projections (one call replayed on one weight, as the thesis timed it)."""
    ref_root = ROOT / "baseline" / "_ref"
    if not (ref_root / "scripts" / "bench_perstep_actual_kernel_speedup.py").exists():
        return {"unavailable": "baseline/_ref/scripts is not filled (python baseline/fill_ref.py)"}
    from bas import refscripts

    try:
        with tempfile.TemporaryDirectory() as tmp:
            res = refscripts.run_thesis_protocol(ref_root, Path(tmp), batch_sizes=(2, 4, 8, 16, 32, 64), quiet=True)
    except Exception as exc:
        return {"unavailable": f"{type(exc).__name__}: {exc}"[:200]}
    return {"kernel_speedup_vs_dense": {str(r["batch_size"]): round(float(r["kernel_speedup"]), 3) for r in res["rows"]},
            "thesis_a100x": {"2": 1.948, "4": 1.945, "8": 1.761, "16": 1.602, "32": 1.405, "64": 1.203},
            "how": "scripts/profile_kernel_configs.py then scripts/bench_perstep_actual_kernel_speedup.py, unmodified"}


def run_gpu(args) -> None:
    import torch
    import torch.distributed as dist

    from bas import abi, launch_count, ops
    from oracle import bas_oracle as O      # input generation only: seeded synthetic tensors

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the CUDA path has no CPU fallback "
                         "(use --impl reference for the CPU reference leg)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("NCCL_DEBUG_FILE", "/tmp/nccl_debug.%h.%p")   # keep stdout to the one JSON line
        dist.init_process_group("nccl", device_id=dev)
    peaks = _peaks()
    stream = torch.cuda.Stream()

    # ---- resident inputs: weight copies, activations, masks ----
    w_host = O.make_weight(N_OUT, K_IN, seed=0)
    w = torch.from_numpy(w_host).to(dev)
    packed = [ops.pack_weight(w) for _ in range(ROTATE)]
    dense_wt = [w.t().contiguous() for _ in range(ROTATE)]       # the reference's dense operand layout
    xs, ids, outs, dense_outs = {}, {}, {}, {}
    for b in BATCHES:
        xs[b] = torch.from_numpy(O.make_activations(b, K_IN, seed=1000 + b, dist="laplace")).to(dev)
        sel, _ = ops.select_topk(xs[b], N_KEEP[b], abi.SCORE_NORM)
        ids[b] = sel.clone()
        outs[b] = torch.zeros(b, N_OUT, dtype=torch.float16, device=dev)
        dense_outs[b] = torch.zeros(b, N_OUT, dtype=torch.float16, device=dev)
    torch.cuda.synchronize()

    # correctness guard (torch fp32 on the GPU; not timed): a fast wrong kernel is not a result
    for b in BATCHES:
        ops.gemm(xs[b], packed[0], outs[b], ids=ids[b])
        mask = torch.zeros(NB, device=dev)
        mask[ids[b].long()] = 1
        ref = (xs[b].float() * mask.repeat_interleave(64)) @ w.float().t()
        err = ((outs[b].float() - ref).abs().max() / ref.abs().max()).item()
        if not err <= 2e-3:
            raise SystemExit(f"parity check failed at B={b}: max err ratio {err:.3e}")
    if ops.read_status(dev) != 0:
        raise SystemExit("device status word is not clean")

    # ---- the K timed steps: list launches of up to 16 steps (48 independent calls) each ----
    GS = 16

    def step_list(n_steps):
        calls = []
        for i in range(n_steps):
            for j, b in enumerate(BATCHES):
                calls.append({"x": xs[b], "packed": packed[(i * len(BATCHES) + j) % ROTATE], "out": outs[b], "ids": ids[b]})
        return ops.GemmList(calls, min_units=16)

    # up to 48 steps are one launch; longer runs are launches of 16 steps, the last one taking the remainder too
    if args.steps <= 3 * GS:
        n_full, rem = 0, args.steps
    else:
        n_full, rem = divmod(args.steps, GS)
        if rem:
            n_full, rem = n_full - 1, rem + GS
    lists = {n: step_list(n) for n in {GS if n_full else 0, rem} - {0}}
    with torch.cuda.stream(stream):
        for _ in range(max(args.warmup, 3)):
            for l in lists.values():
                l.run()
    torch.cuda.synchronize()
    for l in lists.values():
        if l.read_status() != 0:
            raise SystemExit("list launch reported a device flag")
    for b in BATCHES:       # the list wrote the same outputs as the guarded single calls
        mask = torch.zeros(NB, device=dev)
        mask[ids[b].long()] = 1
        ref = (xs[b].float() * mask.repeat_interleave(64)) @ w.float().t()
        err = ((outs[b].float() - ref).abs().max() / ref.abs().max()).item()
        if not err <= 2e-3:
            raise SystemExit(f"list launch: parity check failed at B={b}: max err ratio {err:.3e}")

    try:
        gpu_id = "GPU-" + str(torch.cuda.get_device_properties(dev).uuid).replace("GPU-", "")
    except AttributeError:
        gpu_id = str(local)
    sampler = ClockSampler(gpu_id)

    def region():
        n = 0
        for _ in range(n_full):
            lists[GS].run()
            n += 1
        if rem:
            lists[rem].run()
            n += 1
        return n

    region_ms = []
    launches = 0
    for _ in range(5):                                           # median of five timed regions of K steps
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        before = launch_count()
        with torch.cuda.stream(stream):
            e0.record(stream)
            region()
            e1.record(stream)
        torch.cuda.synchronize()
        launches = launch_count() - before
        ms = e0.elapsed_time(e1)
        if world > 1:
            dist.barrier()
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        region_ms.append(ms)
    ms_total = statistics.median(region_ms)
    ms_per_step = ms_total / args.steps
    value = world * STEP_BYTES / (ms_per_step * 1e-3) / 1e9
    # the dominant kernel: one list launch of GS steps (or of all K when K < 16), timed alone
    dom_steps = GS if n_full else rem
    dom_us = _graph_time_us(torch, stream, lists[dom_steps].run, 1, 20) if rank == 0 else 0.0
    list_info = lists[dom_steps].info()

    if args.headline_only:
        clocks = sampler.stop()
        if rank == 0:
            _emit({"metric": METRIC, "value": round(value, 2), "unit": "GB/s", "n_gpus": world, "steps": args.steps,
                   "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
                   "dtype": "f16", "data": "synthetic", "config": {"workload": WORKLOAD, "headline_only": True},
                   "roofline": {"bound": "hbm", "achieved": round(dom_steps * STEP_BYTES / (dom_us * 1e-6) / 1e9, 1),
                                "peak": peaks["hbm_gbs"], "unit": "GB/s", "launch_us": round(dom_us, 2)},
                   "gpu_launches": launches, "clocks": clocks})
        if world > 1:
            dist.destroy_process_group()
        return

    # ---- per-batch kernel time, dense cuBLAS, selection, fused chain (rank 0's GPU) ----
    per_batch = {}
    reps = 60
    for b in BATCHES:
        lb = ops.GemmList([{"x": xs[b], "packed": packed[c], "out": outs[b], "ids": ids[b]} for c in range(ROTATE)],
                          min_units=16)

        def sparse_cold(b=b):
            for c in range(ROTATE):
                ops.gemm(xs[b], packed[c], outs[b], ids=ids[b], ids_stable=True, x_stable=True, next_independent=True)

        def sparse_cold_ids_only(b=b):        # X may be the previous call's output: one call deep
            for c in range(ROTATE):
                ops.gemm(xs[b], packed[c], outs[b], ids=ids[b], ids_stable=True)

        def sparse_cold_plain(b=b):           # no promises: what the drop-in wrappers launch
            for c in range(ROTATE):
                ops.gemm(xs[b], packed[c], outs[b], ids=ids[b])

        def dense_cold(b=b):
            for c in range(ROTATE):
                torch.mm(xs[b], dense_wt[c], out=dense_outs[b])

        def sparse_hot(b=b):
            # one call per graph launch, as the reference's protocol replays it: graph launches do not
            # overlap, so the call runs alone and takes the one-deep grid
            ops.gemm(xs[b], packed[0], outs[b], ids=ids[b], ids_stable=True)

        def dense_hot(b=b):
            torch.mm(xs[b], dense_wt[0], out=dense_outs[b])

        us_list = _graph_time_us(torch, stream, lb.run, ROTATE, reps)
        lb.close()
        us = _graph_time_us(torch, stream, sparse_cold, ROTATE, reps)
        us_ids = _graph_time_us(torch, stream, sparse_cold_ids_only, ROTATE, reps)
        us_plain = _graph_time_us(torch, stream, sparse_cold_plain, ROTATE, reps)
        dus = _graph_time_us(torch, stream, dense_cold, ROTATE, reps)
        hus = _graph_time_us(torch, stream, sparse_hot, 1, 200)
        hdus = _graph_time_us(torch, stream, dense_hot, 1, 200)
        bytes_b = N_KEEP[b] * SLAB_BYTES
        gbs = bytes_b / (us_list * 1e-6) / 1e9
        per_batch[str(b)] = {
            "sparsity": SPARSITY[b], "active_blocks": N_KEEP[b], "active_weight_mb": round(bytes_b / 1e6, 2),
            "us": round(us_list, 3), "gbs": round(gbs, 1), "frac_of_measured_peak": round(gbs / peaks["hbm_gbs"], 4),
            "frac_of_8000": round(gbs / 8000.0, 4),
            "dense_cublas_us": round(dus, 3),
            "speedup_vs_cublas": round(dus / us_plain, 3),
            "no_promises_us": round(us_plain, 3), "no_promises_gbs": round(bytes_b / (us_plain * 1e-6) / 1e9, 1),
            "ids_stable_only_us": round(us_ids, 3), "ids_stable_only_speedup_vs_cublas": round(dus / us_ids, 3),
            "pipelined_single_launches_us": round(us, 3),
            "chain_throughput_vs_serial_cublas": round(dus / us_list, 3),
            "l2_resident_us": round(hus, 3), "l2_resident_dense_us": round(hdus, 3),
            "l2_resident_speedup": round(hdus / hus, 3),
            "note": "us: per call inside one list launch of 16 independent calls (cold L2); speedup_vs_cublas: "
                    "like for like, single launches with no promises against cuBLAS, both cold and one at a time; "
                    "chain_throughput_vs_serial_cublas: the list's period against serialised cuBLAS calls"}

    # per-step online selection fused ahead of the GEMM (B = 16, energy score, keep 36 %)
    b = 16
    x_steps = [torch.from_numpy(O.make_activations(b, K_IN, seed=100 + s, dist="laplace")).to(dev) for s in range(11)]
    n_keep4 = O.n_keep_from_density(0.36, NB)

    def select_only():
        for s in range(ROTATE):
            ops.select_topk(x_steps[s % 11], n_keep4, abi.SCORE_ENERGY)

    def chain():
        for s in range(ROTATE):
            sel, cnt = ops.select_topk(x_steps[s % 11], n_keep4, abi.SCORE_ENERGY)
            ops.gemm(x_steps[s % 11], packed[s], outs[b], ids=sel, count=cnt, k_host=n_keep4)

    # the same chain with the next step's selection overlapping this step's contraction: the steps
    # alternate between two id buffers and the selection declares its inputs stable
    sel_bufs = [(torch.empty(NB, dtype=torch.int32, device=dev), torch.zeros(1, dtype=torch.int32, device=dev))
                for _ in range(2)]

    def chain_overlapped():
        for s in range(ROTATE):
            ids_buf, cnt_buf = sel_bufs[s & 1]
            sel, cnt = ops.select_topk(x_steps[s % 11], n_keep4, abi.SCORE_ENERGY, ids_out=ids_buf, count_out=cnt_buf,
                                       inputs_stable=True)
            ops.gemm(x_steps[s % 11], packed[s], outs[b], ids=sel, count=cnt, k_host=n_keep4)

    def one_launch():
        for s in range(ROTATE):
            ops.select_gemm(x_steps[s % 11], packed[s], outs[b], n_keep4, abi.SCORE_ENERGY)

    # selection as an entry of the list launch: [score x, contraction that ranks the scores and runs with the kept
    # blocks] as ONE launch, against the same contraction alone in a launch of its own with the ids given
    fixed_ids = [ops.select_topk(x_steps[s % 11], n_keep4, abi.SCORE_ENERGY)[0][:n_keep4].clone() for s in range(ROTATE)]
    sel_lists = [ops.GemmList([{"select": x_steps[s % 11], "n_keep": n_keep4, "score_kind": abi.SCORE_ENERGY},
                               {"x": x_steps[s % 11], "packed": packed[s], "out": outs[b], "mask_from": 0}])
                 for s in range(ROTATE)]
    plain_lists = [ops.GemmList([{"x": x_steps[s % 11], "packed": packed[s], "out": outs[b], "ids": fixed_ids[s]}])
                   for s in range(ROTATE)]

    def list_select_gemm():
        for l in sel_lists:
            l.run()

    def list_gemm():
        for l in plain_lists:
            l.run()

    list_sel_us = _graph_time_us(torch, stream, list_select_gemm, ROTATE, reps)
    list_plain_us = _graph_time_us(torch, stream, list_gemm, ROTATE, reps)
    for l in sel_lists + plain_lists:
        if l.read_status() != 0:
            raise SystemExit("list launch with a selection entry: device status")
        l.close()
    sel_us = _graph_time_us(torch, stream, select_only, ROTATE, reps)
    chain_us = _graph_time_us(torch, stream, chain, ROTATE, reps)
    fused_us = _graph_time_us(torch, stream, one_launch, ROTATE, reps)
    overlapped_us = _graph_time_us(torch, stream, chain_overlapped, ROTATE, reps)
    # same mask and same sums from the one-launch form as from the oracle's ids (not timed)
    sel_ids, _ = ops.select_gemm(x_steps[3], packed[0], outs[b], n_keep4, abi.SCORE_ENERGY)
    torch.cuda.synchronize()
    want_ids = O.topk_ids(O.block_scores(x_steps[3].cpu().numpy(), abi.SCORE_ENERGY), n_keep4)
    if not np.array_equal(sel_ids[:n_keep4].cpu().numpy(), want_ids):
        raise SystemExit("in-kernel selection disagrees with the oracle's ids")
    online = {"batch": b, "keep_blocks": n_keep4, "select_us": round(sel_us, 3), "select_plus_gemm_us": round(chain_us, 3),
              "selection_inside_gemm_us": round(fused_us, 3),
              "select_plus_gemm_overlapped_us": round(overlapped_us, 3), "score": "energy",
              "list_select_plus_gemm_us": round(list_sel_us, 3), "list_gemm_alone_us": round(list_plain_us, 3),
              "note": "select_us: selection kernel alone; select_plus_gemm_us: two launches; "
                      "selection_inside_gemm_us: bas_select_gemm (one call; it selects inside the contraction "
                      "kernel only where that is the faster form, i.e. batches of a few rows); "
                      "list_select_plus_gemm_us: one list launch of a selection entry and the contraction that uses "
                      "its mask (fresh X, no promise), list_gemm_alone_us: the same contraction as a list launch of "
                      "its own with the ids given; "
                      "select_plus_gemm_overlapped_us: the two launches per step, with step i+1's selection "
                      "(BAS_SCORE_INPUTS_STABLE, alternating id buffers) scoring while step i's contraction runs"}

    # ---- rank 0 at N = 1: sparsity sweep on the gate/up shape, the reference's Triton kernels on this GPU,
    # and the reference's own two benchmark scripts against the drop-in ----
    sweep = ref_triton = thesis = None
    two_d = _two_d_chain(torch, ops, O, dev, stream) if world == 1 else None
    if world == 1 and not args.quick:
        sweep = _sweep_gate_up(torch, ops, abi, O, dev, stream, peaks)
        ref_triton = _reference_triton(torch, O, dev, stream, xs, ids)
        for bb in BATCHES:
            r = ref_triton.get(str(bb)) if isinstance(ref_triton, dict) else None
            if isinstance(r, dict) and "us" in r:
                per_batch[str(bb)]["reference_triton_us"] = r["us"]
                per_batch[str(bb)]["reference_triton_variant"] = f"{r['family']}, split-K {r['split_k']}"
                per_batch[str(bb)]["speedup_vs_reference_triton"] = round(r["us"] / per_batch[str(bb)]["no_promises_us"], 3)
        thesis = _thesis_protocol()
        torch.cuda.empty_cache()

    # ---- the sharded decode-step linear stack (all ranks take part) ----
    try:
        layer_stack = _layer_stack(torch, dist, dev, world, rank, stream)
        torch.cuda.empty_cache()
        # the same step with q/k/v and gate/up stacked into one masked GEMM each (they share their
        # input and mask in the model; here the q and gate inputs and masks stand for the group)
        stacked = _layer_stack(torch, dist, dev, world, rank, stream, fuse=True)
        keys = ("linears_per_step", "ms_per_step", "active_weight_gbs", "launch", "tp_parity", "one_launch")
        layer_stack["stacked_qkv_gateup"] = {k: stacked[k] for k in keys if k in stacked}
        if world > 1:
            # the same two steps with o/down summed over the ranks inside the contraction kernel
            # (fp32 partials read from the peers over NVLink) instead of by an NCCL all-reduce
            for name, fuse in (("in_kernel_sum", False), ("in_kernel_sum_stacked_qkv_gateup", True)):
                torch.cuda.empty_cache()
                try:
                    r = _layer_stack(torch, dist, dev, world, rank, stream, fuse=fuse, allreduce="in_kernel")
                    layer_stack[name] = {k: r[k] for k in keys if k in r}
                except Exception as exc:
                    layer_stack[name] = {"error": f"{type(exc).__name__}: {exc}"[:300]}
    except Exception as exc:
        layer_stack = {"error": f"{type(exc).__name__}: {exc}"[:300]}
    torch.cuda.empty_cache()

    # ---- end to end through the host-buffer operator: a step is one submission ----
    import ctypes
    calls = (abi.StepCall * len(BATCHES))()
    for c, bb in zip(calls, BATCHES):
        c.w_host, c.n, c.k, c.batch, c.n_keep, c.score_kind = w_host.ctypes.data, N_OUT, K_IN, bb, N_KEEP[bb], abi.SCORE_NORM
    E2E_DEPTH = 6
    hstep = ctypes.c_void_p()
    abi.check(abi.lib.bas_step_create(ctypes.byref(hstep), calls, len(BATCHES), E2E_DEPTH), "bas_step_create")
    # the step's inputs and results live in page-locked host memory, as a serving host keeps them; one
    # set of buffers per step in flight
    pinned = []

    def pinned_array(shape, dtype):
        t = torch.empty(shape, dtype=dtype, pin_memory=True)
        pinned.append(t)                # keeps the allocation alive
        return t.numpy()

    sets = []
    for _ in range(E2E_DEPTH):
        xh = [pinned_array((bb, K_IN), torch.float16) for bb in BATCHES]
        yh = [pinned_array((bb, N_OUT), torch.float16) for bb in BATCHES]
        ih = [np.full(NB, -1, np.int32) for bb in BATCHES]
        for arr, bb in zip(xh, BATCHES):
            arr[...] = O.make_activations(bb, K_IN, seed=1000 + bb, dist="laplace")
        ptrs = tuple((ctypes.c_void_p * len(BATCHES))(*[a.ctypes.data for a in group]) for group in (xh, yh, ih))
        sets.append((xh, yh, ih, ptrs))

    def e2e_run(n_steps):
        # keep E2E_DEPTH steps in flight: every step's uploads, kernels and downloads are inside the region
        for i in range(n_steps):
            if i >= E2E_DEPTH:
                abi.check(abi.lib.bas_step_wait(hstep), "bas_step_wait")
            px, py, pi = sets[i % E2E_DEPTH][3]
            abi.check(abi.lib.bas_step_submit(hstep, px, py, pi), "bas_step_submit")
        for _ in range(min(n_steps, E2E_DEPTH)):
            abi.check(abi.lib.bas_step_wait(hstep), "bas_step_wait")

    e2e_run(9)
    e2e_steps = max(60, min(args.steps, 600))
    if world > 1:
        dist.barrier()
    t0 = time.perf_counter()
    e2e_run(e2e_steps)
    e2e_dt = (time.perf_counter() - t0) / e2e_steps
    # one step alone, nothing else in flight: the latency of a step
    lat = []
    for _ in range(2 * E2E_DEPTH + 20):      # (a slot replays its captured step from its third use on)
        t1 = time.perf_counter()
        e2e_run(1)
        lat.append(time.perf_counter() - t1)
    lat = lat[-20:]
    if world > 1:
        t = torch.tensor([e2e_dt], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_dt = float(t.item())
    abi.lib.bas_step_destroy(hstep)
    # the bare transfers of a step - the three X up, the three Y down, both directions at once on two streams,
    # nothing else: what the host link allows for these sizes
    cs_up, cs_down = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
    xh_t = [torch.from_numpy(a) for a in sets[0][0]]
    yh_t = [torch.empty((bb, N_OUT), dtype=torch.float16, pin_memory=True) for bb in BATCHES]
    xd_t = [torch.empty(bb, K_IN, dtype=torch.float16, device=dev) for bb in BATCHES]
    yd_t = [torch.zeros(bb, N_OUT, dtype=torch.float16, device=dev) for bb in BATCHES]

    def copies(n):
        with torch.cuda.stream(cs_up):
            for _ in range(n):
                for d_, h_ in zip(xd_t, xh_t):
                    d_.copy_(h_, non_blocking=True)
        with torch.cuda.stream(cs_down):
            for _ in range(n):
                for h_, d_ in zip(yh_t, yd_t):
                    h_.copy_(d_, non_blocking=True)

    copies(20)
    torch.cuda.synchronize()
    t1 = time.perf_counter()
    copies(300)
    torch.cuda.synchronize()
    copies_ms = (time.perf_counter() - t1) / 300 * 1e3
    for xh, yh, ih, _ in sets:      # the e2e outputs are real results: same masks, same sums as the resident path
        for j, bb in enumerate(BATCHES):
            ops.gemm(xs[bb], packed[0], outs[bb], ids=ids[bb])
            torch.cuda.synchronize()
            d = np.abs(yh[j].astype(np.float32) - outs[bb].float().cpu().numpy()).max()
            same_ids = np.array_equal(ih[j][:N_KEEP[bb]], ids[bb].cpu().numpy())
            if not same_ids or not d <= 2e-3 * float(outs[bb].float().abs().max().item()):
                raise SystemExit(f"end-to-end result differs from the resident-input path at B={bb}: "
                                 f"ids equal {same_ids}, max |dy| {d:.3e}")
    e2e = {"value": world * STEP_BYTES / e2e_dt / 1e9, "unit": "GB/s",
           "h2d_bytes_per_step": sum(bb * K_IN * 2 for bb in BATCHES),
           "d2h_bytes_per_step": sum(bb * N_OUT * 2 + (NB + 1) * 4 for bb in BATCHES) + 16,
           "ms_per_step": e2e_dt * 1e3, "steps": e2e_steps, "steps_in_flight": E2E_DEPTH,
           "one_step_alone_ms": round(statistics.median(lat) * 1e3, 4),
           "transfers_alone_ms_per_step": round(copies_ms, 4),
           "api": "bas_step_submit / bas_step_wait: per step H2D of the three X from page-locked memory, three device-side "
                  "top-k selections, one list launch for the three GEMMs, D2H of the three Y, the ids and the status word"}

    clocks = sampler.stop()

    if rank == 0:
        list_bytes = dom_steps * STEP_BYTES
        achieved = list_bytes / (dom_us * 1e-6) / 1e9
        one_deep = {str(bb): {"us": per_batch[str(bb)]["no_promises_us"], "achieved": per_batch[str(bb)]["no_promises_gbs"],
                              "frac": round(per_batch[str(bb)]["no_promises_gbs"] / peaks["hbm_gbs"], 4)} for bb in BATCHES}
        roofline = {
            "bound": "hbm", "kernel": f"umma_list_kernel<64> over {dom_steps} steps = {dom_steps * len(BATCHES)} calls "
                                      f"(B = 2/16/64, 34/62/83 of 172 blocks), {list_info['ctas']} CTAs",
            "achieved": round(achieved, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
            "frac": round(achieved / peaks["hbm_gbs"], 4), "peak_source": peaks["source"] + " (stream copy, burst)",
            "algorithmic_bytes_per_launch": list_bytes, "launch_us": round(dom_us, 2),
            "duration": "CUDA events around replays of the one launch, on the launching stream",
            # dram__bytes_read.sum + dram__bytes_write.sum of one such launch (ncu, 16 steps), see TRAFFIC_NOTE
            "traffic": LIST_TRAFFIC_16_STEPS * dom_steps // 16 if LIST_TRAFFIC_16_STEPS else None,
            "traffic_note": TRAFFIC_NOTE,
            "one_call_deep_all": one_deep,
            "one_call_deep_note": "single launches with no promises (what the drop-in wrappers run), cold L2",
        }
        cpu = cpu_baseline() if world == 1 else None
        line = {
            "metric": METRIC, "value": round(value, 2), "unit": "GB/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": {"workload": WORKLOAD,
                       "step": "3 masked GEMMs (B=2,16,64); activations and masks are resident before the launch; the K steps "
                               "run as list launches of up to 16 steps (bas_list_run: one persistent kernel per launch walks "
                               "48 independent calls).  per_batch has the same calls as single launches with fewer promises",
                       "l2": f"cold: every call reads one of {ROTATE} rotating weight copies (1.4 GB in rotation)",
                       "parallelism": f"replicas x{world}" if world > 1 else "single GPU",
                       "timing": "CUDA events on the launch stream around the K steps, median of 5 regions, max over ranks",
                       "region_ms": [round(v, 4) for v in region_ms]},
            "per_batch": per_batch, "online_selection": online, "layer_stack": layer_stack, "two_d_chain": two_d, "sweep_gate_up": sweep,
            "reference_triton": ref_triton, "thesis_protocol": thesis, "roofline": roofline, "cpu_baseline": cpu,
            "e2e": e2e, "gpu_launches": launches, "clocks": clocks,
        }
        _emit(line)
    if world > 1:
        dist.destroy_process_group()


def run_profile_case(batch: int, family: int = 0, pipelined: bool = False) -> None:
    """A few eager launches of one batch size on 4 rotating weight copies (360 MB, larger than L2):
    the small case that profiler captures of the contraction kernels are taken on.  ``pipelined``:
    the masks are selected once, ahead, and the calls declare ids and X stable - the grid (one CTA per
    128-column range) that the benchmark's chains run."""
    import torch

    from bas import abi, ops
    from oracle import bas_oracle as O

    dev = torch.device("cuda", 0)
    w = torch.from_numpy(O.make_weight(N_OUT, K_IN, seed=0)).to(dev)
    packed = [ops.pack_weight(w) for _ in range(4)]
    nk = N_KEEP.get(batch, O.n_keep_from_density(0.36, NB))
    x = torch.from_numpy(O.make_activations(batch, K_IN, seed=1000 + batch, dist="laplace")).to(dev)
    out = torch.zeros(batch, N_OUT, dtype=torch.float16, device=dev)
    if pipelined:
        ids = ops.select_topk(x, nk, abi.SCORE_NORM)[0].clone()
        torch.cuda.synchronize()
        for i in range(8):
            ops.gemm(x, packed[i % 4], out, ids=ids, family=family, ids_stable=True, x_stable=True, next_independent=True)
    else:
        for i in range(8):
            ids, cnt = ops.select_topk(x, nk, abi.SCORE_NORM)
            ops.gemm(x, packed[i % 4], out, ids=ids, family=family)
    torch.cuda.synchronize()
    print(f"profile case B={batch} family={family} pipelined={pipelined}: 8 gemm launches, status {ops.read_status(dev)}")


def run_profile_list(steps: int) -> None:
    """Three eager list launches of `steps` benchmark steps each (16 rotating weight copies, 1.4 GB):
    the case that profiler captures of the list kernel are taken on."""
    import torch

    from bas import abi, ops
    from oracle import bas_oracle as O

    dev = torch.device("cuda", 0)
    w = torch.from_numpy(O.make_weight(N_OUT, K_IN, seed=0)).to(dev)
    packed = [ops.pack_weight(w) for _ in range(ROTATE)]
    xs = {b: torch.from_numpy(O.make_activations(b, K_IN, seed=1000 + b, dist="laplace")).to(dev) for b in BATCHES}
    ids = {b: ops.select_topk(xs[b], N_KEEP[b], abi.SCORE_NORM)[0].clone() for b in BATCHES}
    outs = {b: torch.zeros(b, N_OUT, dtype=torch.float16, device=dev) for b in BATCHES}
    calls = []
    for i in range(steps):
        for j, b in enumerate(BATCHES):
            calls.append({"x": xs[b], "packed": packed[(i * len(BATCHES) + j) % ROTATE], "out": outs[b], "ids": ids[b]})
    lst = ops.GemmList(calls, min_units=16)
    torch.cuda.synchronize()
    for _ in range(3):
        lst.run()
    torch.cuda.synchronize()
    print(f"profile list: 3 launches of {steps} steps ({len(calls)} calls, {steps * STEP_BYTES} algorithmic bytes each), "
          f"{lst.info()}, status {lst.read_status()}")


def run_profile_stack(layers: int) -> None:
    """Three eager launches of `layers` layers of the decode stack (B = 16, q+k+v and gate+up stacked) as ONE list
    with the model's dependencies and every mask computed inside the launch (selection entries): the case that
    profiler captures of the extended list kernel are taken on.  Four layers hold 0.8 GB of weights."""
    import torch

    from bas import tp

    dev = torch.device("cuda", 0)
    stack = tp.DecodeLinearStack(layers, 16, 0.638, dev, 1, 0, seed=5, fuse_shared_inputs=True)
    lst = stack.make_list(dependencies=True, select=True)
    torch.cuda.synchronize()
    for _ in range(3):
        lst.run()
    torch.cuda.synchronize()
    par = stack.parity_check_outputs(layers=1)
    print(f"profile stack: 3 launches of {layers} layers ({lst.n_calls} entries, {stack.active_bytes} active weight bytes each), "
          f"{lst.info()}, status {lst.read_status()}, parity {par}")


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=960)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="own", choices=["own", "reference"])
    ap.add_argument("--headline-only", action="store_true",
                    help="time the K steps only and print a short line (the case the profiler's launch list is taken on)")
    ap.add_argument("--quick", action="store_true",
                    help="skip the sparsity sweep, the reference's Triton kernels and the reference's scripts")
    ap.add_argument("--profile-case", type=int, default=0, metavar="B",
                    help="run only a few eager launches at batch B (for profiler captures) and exit")
    ap.add_argument("--profile-family", type=int, default=0, choices=[0, 1, 2],
                    help="kernel family of the profile case: 0 default, 1 CUDA-core kernel (batch <= 8), 2 tcgen05")
    ap.add_argument("--profile-list", type=int, default=0, metavar="STEPS",
                    help="run only three eager list launches of STEPS benchmark steps (for profiler captures) and exit")
    ap.add_argument("--profile-stack", type=int, default=0, metavar="LAYERS",
                    help="run only three eager launches of LAYERS layers of the decode stack as one list with selection "
                         "entries (for profiler captures) and exit")
    ap.add_argument("--profile-pipelined", action="store_true",
                    help="profile case: masks fixed ahead, calls declare ids and X stable (the benchmark's chains)")
    args = ap.parse_args()
    # stdout carries exactly one JSON line: libraries that chat on fd 1 (NCCL prints its version
    # there) are sent to stderr, and the line is written to the saved descriptor at the end.
    global _STDOUT_FD
    sys.stdout.flush()
    _STDOUT_FD = os.dup(1)
    os.dup2(2, 1)
    if args.profile_list:
        run_profile_list(args.profile_list)
    elif args.profile_stack:
        run_profile_stack(args.profile_stack)
    elif args.profile_case:
        run_profile_case(args.profile_case, args.profile_family, args.profile_pipelined)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_gpu(args)


if __name__ == "__main__":
    main()
