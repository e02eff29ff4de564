#!/usr/bin/env python
"""Benchmark of the batch-shared block-sparse activation GEMM on B200.

    python bench.py --gpus N --steps K --warmup W            # this repository's CUDA path
    python bench.py --impl reference --steps K --warmup W    # the reference's CPU torch path

Workload (synthetic, seeded): the Llama-2-7B down-projection, X fp16 [B, 11008] ~ Laplace(0,1),
W fp16 [4096, 11008] ~ N(0, 0.02^2), 172 blocks of 64 channels, batch-shared top-k masks keeping
34 / 62 / 83 blocks at B = 2 / 16 / 64 (block sparsity 0.803 / 0.638 / 0.520).  One "step" is the
three masked GEMMs B = 2, 16, 64.  The metric is the active-weight HBM bandwidth of a step:
(34 + 62 + 83) * 64 * 4096 * 2 bytes divided by the step time.

Timing: the K timed steps are CUDA-graph replays (16 steps per graph, each call on one of 16
rotating weight copies so that a weight tile is never found in L2), bracketed by CUDA events on the
launching stream.  Activations and masks are resident before a chain of calls starts and the calls
say so (ids and X declared stable), so consecutive, independent calls overlap on the GPU several
deep; each still stores its result only after the call before it has completed.  The same chains
with fewer promises (one call deep, as the drop-in wrappers launch) are reported in per_batch beside
the headline.  Per-batch microseconds, the dense cuBLAS baseline and the roofline figure come
from per-batch graphs timed the same way inside this program.  With --gpus N every rank runs the
same workload on its own GPU (independent decode replicas, no collective on the data path).
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
            "ms_per_step": med * 1e3}


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
    0.638), column-/row-parallel over the ranks with an NCCL all-reduce after o and down: one CUDA
    graph per step where NCCL allows capture, timed by CUDA events, max over ranks."""
    from bas import tp

    stack = tp.DecodeLinearStack(32, 16, 0.638, dev, world, rank, fuse_shared_inputs=fuse, allreduce=allreduce)
    def timed():
        with torch.cuda.stream(stream):
            for _ in range(3):
                stack.step()
        torch.cuda.synchronize()
        mode = "cuda graph"
        try:
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=stream):
                stack.step()
            run = g.replay
        except Exception as exc:      # a collective that refuses capture: time eager launches instead
            mode = f"eager ({type(exc).__name__})"
            run = stack.step
        torch.cuda.synchronize()
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

    ms, mode = timed()
    extra = {}
    if world == 1 and not fuse:
        # throughput probe: the same 224 calls with every input declared stable (they are: the stack's
        # inputs are generated ahead), i.e. no call depends on the one before it
        stack.independent_calls = True
        ms_ind, _ = timed()
        stack.independent_calls = False
        extra = {"independent_calls": {"ms_per_step": round(ms_ind, 4),
                                       "active_weight_gbs": round(stack.active_bytes / (ms_ind * 1e-3) / 1e9, 1),
                                       "note": "every call declares ids and X stable (a probe of the chain's throughput over "
                                               "the seven shapes); ms_per_step above declares X stable only for k, v and up, "
                                               "which in the model read what q / gate have already read"}}
    stack.close()
    return {**extra, "layers": 32, "linears_per_step": len(stack.items), "batch": 16, "sparsity": 0.638,
            "parallelism": f"tp{world}: column-parallel q/k/v/gate/up, row-parallel o/down + all-reduce",
            "ms_per_step": round(ms, 4), "active_weight_gb_per_step": round(stack.active_bytes / 1e9, 3),
            "active_weight_gbs": round(stack.active_bytes / (ms * 1e-3) / 1e9, 1), "launch": mode}


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

    counter = {"i": 0}

    def one_step():
        for b in BATCHES:
            c = counter["i"] % ROTATE
            counter["i"] += 1
            ops.gemm(xs[b], packed[c], outs[b], ids=ids[b], ids_stable=True, x_stable=True, next_independent=True)

    # ---- the K timed steps ----
    GS = 16                                                     # steps per captured graph
    def build_steps(n):
        def f():
            for _ in range(n):
                one_step()
        return f

    with torch.cuda.stream(stream):
        for _ in range(max(args.warmup, 3)):
            one_step()
    torch.cuda.synchronize()
    n_full, rem = divmod(args.steps, GS)
    graphs = {}
    for n in {GS if n_full else 0, rem} - {0}:
        counter["i"] = 0
        before = launch_count()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=stream):
            build_steps(n)()
        graphs[n] = (g, launch_count() - before)
    torch.cuda.synchronize()
    with torch.cuda.stream(stream):                              # warm the graphs themselves
        for n, (g, _) in graphs.items():
            g.replay()
    torch.cuda.synchronize()

    try:
        gpu_id = "GPU-" + str(torch.cuda.get_device_properties(dev).uuid).replace("GPU-", "")
    except AttributeError:
        gpu_id = str(local)
    sampler = ClockSampler(gpu_id)
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    launches = 0
    with torch.cuda.stream(stream):
        e0.record(stream)
        for _ in range(n_full):
            graphs[GS][0].replay()
            launches += graphs[GS][1]
        if rem:
            graphs[rem][0].replay()
            launches += graphs[rem][1]
        e1.record(stream)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    ms_total = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([ms_total], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_total = float(t.item())
    ms_per_step = ms_total / args.steps
    value = world * STEP_BYTES / (ms_per_step * 1e-3) / 1e9

    # ---- per-batch kernel time, dense cuBLAS, selection, fused chain (rank 0's GPU) ----
    per_batch = {}
    reps = 60
    for b in BATCHES:
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

        us = _graph_time_us(torch, stream, sparse_cold, ROTATE, reps)
        us_ids = _graph_time_us(torch, stream, sparse_cold_ids_only, ROTATE, reps)
        us_plain = _graph_time_us(torch, stream, sparse_cold_plain, ROTATE, reps)
        dus = _graph_time_us(torch, stream, dense_cold, ROTATE, reps)
        hus = _graph_time_us(torch, stream, sparse_hot, 1, 200)
        hdus = _graph_time_us(torch, stream, dense_hot, 1, 200)
        bytes_b = N_KEEP[b] * SLAB_BYTES
        gbs = bytes_b / (us * 1e-6) / 1e9
        per_batch[str(b)] = {
            "sparsity": SPARSITY[b], "active_blocks": N_KEEP[b], "active_weight_mb": round(bytes_b / 1e6, 2),
            "us": round(us, 3), "dense_cublas_us": round(dus, 3), "speedup_vs_cublas": round(dus / us, 3),
            "gbs": round(gbs, 1), "frac_of_measured_peak": round(gbs / peaks["hbm_gbs"], 4),
            "frac_of_8000": round(gbs / 8000.0, 4),
            "ids_stable_only_us": round(us_ids, 3), "ids_stable_only_speedup_vs_cublas": round(dus / us_ids, 3),
            "no_promises_us": round(us_plain, 3), "no_promises_speedup_vs_cublas": round(dus / us_plain, 3),
            "l2_resident_us": round(hus, 3), "l2_resident_dense_us": round(hdus, 3),
            "l2_resident_speedup": round(hdus / hus, 3),
        }

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
              "note": "select_us: selection kernel alone; select_plus_gemm_us: two launches; "
                      "selection_inside_gemm_us: bas_select_gemm (one call; it selects inside the contraction "
                      "kernel only where that is the faster form, i.e. batches of a few rows); "
                      "select_plus_gemm_overlapped_us: the two launches per step, with step i+1's selection "
                      "(BAS_SCORE_INPUTS_STABLE, alternating id buffers) scoring while step i's contraction runs"}

    # ---- the sharded decode-step linear stack (all ranks take part) ----
    try:
        layer_stack = _layer_stack(torch, dist, dev, world, rank, stream)
        torch.cuda.empty_cache()
        # the same step with q/k/v and gate/up stacked into one masked GEMM each (they share their
        # input and mask in the model; here the q and gate inputs and masks stand for the group)
        stacked = _layer_stack(torch, dist, dev, world, rank, stream, fuse=True)
        keys = ("linears_per_step", "ms_per_step", "active_weight_gbs", "launch")
        layer_stack["stacked_qkv_gateup"] = {k: stacked[k] for k in keys}
        if world > 1:
            # the same two steps with o/down summed over the ranks inside the contraction kernel
            # (fp32 partials read from the peers over NVLink) instead of by an NCCL all-reduce
            for name, fuse in (("in_kernel_sum", False), ("in_kernel_sum_stacked_qkv_gateup", True)):
                torch.cuda.empty_cache()
                try:
                    r = _layer_stack(torch, dist, dev, world, rank, stream, fuse=fuse, allreduce="in_kernel")
                    layer_stack[name] = {k: r[k] for k in keys}
                except Exception as exc:
                    layer_stack[name] = {"error": f"{type(exc).__name__}: {exc}"[:300]}
    except Exception as exc:
        layer_stack = {"error": f"{type(exc).__name__}: {exc}"[:300]}
    torch.cuda.empty_cache()

    # ---- end to end through the host-buffer operator (pinned staging inside the library) ----
    import ctypes
    handles = []
    E2E_COPIES = 4
    for _ in range(E2E_COPIES):
        h = ctypes.c_void_p()
        abi.check(abi.lib.bas_linear_create(ctypes.byref(h), w_host.ctypes.data, N_OUT, K_IN, 64), "bas_linear_create")
        handles.append(h)
    # the step's inputs and results live in page-locked host memory, as a serving host keeps them
    pinned = {}

    def pinned_array(key, shape, dtype):
        t = torch.empty(shape, dtype=dtype, pin_memory=True)
        pinned[key] = t                 # keeps the allocation alive
        return t.numpy()

    x_host, y_host = {}, {}
    for bb in BATCHES:
        x_host[bb] = pinned_array(("x", bb), (bb, K_IN), torch.float16)
        x_host[bb][...] = O.make_activations(bb, K_IN, seed=1000 + bb, dist="laplace")
        y_host[bb] = pinned_array(("y", bb), (bb, N_OUT), torch.float16)
    ids_host = {bb: np.full(NB, -1, np.int32) for bb in BATCHES}
    call = {"i": 0}

    def e2e_step():
        # the three calls of a step are independent: submit them on three handles (own streams, so the
        # copies of one overlap the kernels of another), then collect the three results
        used = []
        for bb in BATCHES:                            # smallest upload first (measured: 116 vs 127 us per step)
            h = handles[call["i"] % E2E_COPIES]
            call["i"] += 1
            abi.check(abi.lib.bas_linear_submit_host(h, x_host[bb].ctypes.data, bb, N_KEEP[bb], abi.SCORE_NORM,
                                                     y_host[bb].ctypes.data, ids_host[bb].ctypes.data),
                      "bas_linear_submit_host")
            used.append(h)
        for h in used:
            abi.check(abi.lib.bas_linear_wait(h), "bas_linear_wait")

    for _ in range(5):
        e2e_step()
    e2e_steps = max(20, min(args.steps, 500))
    if world > 1:
        dist.barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        e2e_step()
    e2e_dt = (time.perf_counter() - t0) / e2e_steps
    if world > 1:
        t = torch.tensor([e2e_dt], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_dt = float(t.item())
    for h in handles:
        abi.lib.bas_linear_destroy(h)
    for bb in BATCHES:      # the e2e outputs are real results: same masks, same sums as the resident path
        ops.gemm(xs[bb], packed[0], outs[bb], ids=ids[bb])
        torch.cuda.synchronize()
        d = np.abs(y_host[bb].astype(np.float32) - outs[bb].float().cpu().numpy()).max()
        same_ids = np.array_equal(ids_host[bb][:N_KEEP[bb]], ids[bb].cpu().numpy())
        if os.environ.get("BAS_BENCH_DEBUG"):
            mask = torch.zeros(NB, device=dev); mask[ids[bb].long()] = 1
            ref = ((xs[bb].float() * mask.repeat_interleave(64)) @ w.float().t()).cpu().numpy()
            print("debug B", bb, "e2e vs ref", np.abs(y_host[bb].astype(np.float32) - ref).max(),
                  "resident vs ref", np.abs(outs[bb].float().cpu().numpy() - ref).max(),
                  "x_host==xs", np.array_equal(x_host[bb], xs[bb].cpu().numpy()), file=sys.stderr)
        if not same_ids or not d <= 2e-3 * float(outs[bb].float().abs().max().item()):
            raise SystemExit(f"end-to-end result differs from the resident-input path at B={bb}: "
                             f"ids equal {same_ids}, max |dy| {d:.3e}")
    e2e = {"value": world * STEP_BYTES / e2e_dt / 1e9, "unit": "GB/s",
           "h2d_bytes_per_step": sum(bb * K_IN * 2 for bb in BATCHES),
           "d2h_bytes_per_step": sum(bb * N_OUT * 2 + N_KEEP[bb] * 4 for bb in BATCHES) + 3 * 4,
           "ms_per_step": e2e_dt * 1e3, "steps": e2e_steps,
           "api": "bas_linear_submit_host x3 + bas_linear_wait x3 per step: H2D X from pinned memory, device-side top-k selection, GEMM, D2H Y and ids, per call"}

    clocks = sampler.stop()

    if rank == 0:
        dom = per_batch["64"]
        roofline = {
            "bound": "hbm", "kernel": "umma_colsplit_kernel<64, false, false> (B=64, 83 of 172 blocks)",
            "achieved": dom["gbs"], "peak": peaks["hbm_gbs"], "unit": "GB/s",
            "frac": round(dom["gbs"] / peaks["hbm_gbs"], 4), "peak_source": peaks["source"],
            "algorithmic_bytes_per_launch": N_KEEP[64] * SLAB_BYTES, "traffic": None,
            "one_call_deep": {"achieved": round(N_KEEP[64] * SLAB_BYTES / (dom["ids_stable_only_us"] * 1e-6) / 1e9, 1),
                              "frac": round(N_KEEP[64] * SLAB_BYTES / (dom["ids_stable_only_us"] * 1e-6) / 1e9 / peaks["hbm_gbs"], 4),
                              "note": "the same call when X may be the previous kernel's output (launches do not "
                                      "overlap beyond a ring-full of weights): the 128-CTA cluster grid of "
                                      "profiles/umma_colsplit_down_proj_b64.md"},
            "duration": "timed region / launches: the chain's launches overlap (32 CTAs each, about four calls "
                        "resident), so this is the period of the chain, not the lifetime of one launch",
        }
        # dram__bytes_read.sum + dram__bytes_write.sum of one launch, from the ncu capture summarised in
        # profiles/umma_colsplit_pipelined_down_proj_b64.md (same workload and grid, one launch)
        roofline["traffic"] = 44_305_920
        cpu = cpu_baseline() if world == 1 else None
        line = {
            "metric": METRIC, "value": round(value, 2), "unit": "GB/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": {"workload": WORKLOAD,
                       "step": "3 masked GEMMs (B=2,16,64); activations and masks are resident before the chain of "
                               "calls starts and declared so (BAS_GEMM_IDS_STABLE | BAS_GEMM_X_STABLE | BAS_GEMM_NEXT_INDEPENDENT): independent "
                               "calls of a stream pipeline several deep, each waiting for its predecessor only "
                               "before it stores.  per_batch also has the same chains with only the masks declared "
                               "stable (ids_stable_only_*) and with nothing declared, as the drop-in wrappers "
                               "launch (no_promises_*): one call deep",
                       "l2": f"cold: every call reads one of {ROTATE} rotating weight copies (1.4 GB in rotation)",
                       "parallelism": f"replicas x{world}" if world > 1 else "single GPU",
                       "timing": "CUDA-graph replays of 16 steps, CUDA events on the launch stream, max over ranks"},
            "per_batch": per_batch, "online_selection": online, "layer_stack": layer_stack, "roofline": roofline, "cpu_baseline": cpu,
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


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=4000)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="own", choices=["own", "reference"])
    ap.add_argument("--profile-case", type=int, default=0, metavar="B",
                    help="run only a few eager launches at batch B (for profiler captures) and exit")
    ap.add_argument("--profile-family", type=int, default=0, choices=[0, 1, 2],
                    help="kernel family of the profile case: 0 default, 1 CUDA-core kernel (batch <= 8), 2 tcgen05")
    ap.add_argument("--profile-pipelined", action="store_true",
                    help="profile case: masks fixed ahead, calls declare ids and X stable (the benchmark's chains)")
    args = ap.parse_args()
    # stdout carries exactly one JSON line: libraries that chat on fd 1 (NCCL prints its version
    # there) are sent to stderr, and the line is written to the saved descriptor at the end.
    global _STDOUT_FD
    sys.stdout.flush()
    _STDOUT_FD = os.dup(1)
    os.dup2(2, 1)
    if args.profile_case:
        run_profile_case(args.profile_case, args.profile_family, args.profile_pipelined)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_gpu(args)


if __name__ == "__main__":
    main()
