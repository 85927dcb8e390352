#!/usr/bin/env python
"""Benchmark of the quantized MoE FFN hot path on B200.

    python bench.py --gpus N --steps K --warmup W [--streams R] [--impl reference]

Workload (N = 1): one Qwen3.6-35B-A3B-shaped MoE layer (hidden 2048, 256 routed experts, top-8,
expert intermediate 512, one sigmoid-gated shared expert; gate/up Q4_K, down Q6_K, router f32),
decode with R concurrent streams.  One step = one pass of the layer over one batch of R token
rows.  Weights are synthetic (random block payload, f16 scales ~ U[1e-4, 1e-3], router ~
N(0, 0.02)), activations ~ N(0, 1).  Steps rotate over LAYER_SETS independent weight sets so the
weights a step touches were evicted from L2 since their last use.

N > 1: every rank runs its own replica of the streams on its own GPU (token rows are independent;
no collective on the data path), timed between barriers, max over ranks.

The line printed by rank 0 follows the driver's contract; `roofline` is for the dominant kernel
(the gate/up dequant-GEMV), `cpu_baseline` is the CPU oracle (a restatement of the reference's
infr-cpu reference-mode arithmetic) timed on the host cores on a bounded sample.
"""
from __future__ import annotations

import argparse
import ctypes
import dataclasses
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

NE, N_EXPERT, N_USED, N_FF, SH_FF = 2048, 256, 8, 512, 512
LAYER_SETS = 16
X_POOL = 64
Q4K_ROW = NE // 256 * 144      # bytes of one gate/up row
Q6K_ROW = N_FF // 256 * 210    # bytes of one down row
EXPERT_BYTES = 2 * N_FF * Q4K_ROW + NE * Q6K_ROW  # 2 039 808
# DRAM bytes of one gate/up launch at 1 stream from the ncu capture summarised in
# profiles/decode_c1_r1.md (dram__bytes_read.sum + dram__bytes_write.sum)
GATEUP_TRAFFIC_R1 = 10_651_392


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=400)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--streams", type=int, default=1, help="concurrent decode streams (rows per step)")
    ap.add_argument("--workload", default="layer", choices=["layer", "stack", "prefill"],
                    help="layer: one MoE layer per step (the headline); stack: 40 such layers with RmsNorm and residual "
                         "add per step; prefill: one 4096-token chunk through one layer per step")
    ap.add_argument("--tokens", type=int, default=0, help="tokens of the prefill chunk (default 4096, or 8192 for --shape deepseek; "
                    "64 is the largest configuration's decode batch; a smaller chunk also suits profiler captures)")
    ap.add_argument("--shape", default="qwen", choices=["qwen", "deepseek"],
                    help="prefill workload only: the 256-expert Qwen3.6-35B-A3B layer, or the DeepSeek-V3-shaped one "
                         "(hidden 7168, intermediate 2048, sigmoid gating in 8 groups / 4 used, ungated shared expert)")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    return ap.parse_args()


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return json.load(f), "measured"
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}, "fallback"


class ClockSampler:
    """nvidia-smi clocks and throttle reasons sampled while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.f = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        try:
            self.p = subprocess.Popen(["nvidia-smi", "-i", str(gpu_index), f"--query-gpu={self.Q}",
                                       "--format=csv,noheader,nounits", "-lms", "100"],
                                      stdout=self.f, stderr=subprocess.DEVNULL)
        except OSError:
            self.p = None

    def stop(self):
        if self.p is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.p.terminate()
        try:
            self.p.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.p.kill()
        self.f.flush()
        self.f.seek(0)
        sm, mx, reasons = [], [], set()
        for line in self.f.read().splitlines():
            c = [v.strip() for v in line.split(",")]
            if len(c) < 8:
                continue
            try:
                sm.append(float(c[0]))
                mx.append(float(c[1]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), c[4:8]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        self.f.close()
        os.unlink(self.f.name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def distinct_experts(ids):
    import numpy as np
    return int(np.unique(ids).size)


# ---------------------------------------------------------------------------------------------
# reference arm: the CPU oracle on the host cores
# ---------------------------------------------------------------------------------------------

def cpu_layers(n_sets):
    from moe4all_b200 import synth
    return [synth.make_layer(1000 + i, NE, N_EXPERT, N_FF, sh_ff=SH_FF) for i in range(n_sets)]


def cpu_step(orc, L, x):
    return orc.moe_layer(x, L.router, L.gate, L.up, L.down, L.sh_gate, L.sh_up, L.sh_down, L.sh_gate_inp, SH_FF,
                         n_expert=N_EXPERT, n_used=N_USED, n_ff_exp=N_FF, threads=0)


def time_cpu(streams, steps, warmup, n_sets=2):
    """tok/s of the CPU oracle on `steps` steps of the same workload (all host threads)."""
    from moe4all_b200 import synth
    from oracle import oracle as orc
    layers = cpu_layers(n_sets)
    xs = [synth.activations(50 + i, streams, NE) for i in range(8)]
    for i in range(warmup):
        cpu_step(orc, layers[i % n_sets], xs[i % 8])
    t0 = time.perf_counter()
    for i in range(steps):
        cpu_step(orc, layers[i % n_sets], xs[i % 8])
    dt = time.perf_counter() - t0
    return streams * steps / dt, dt / steps, orc.hw_threads()


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    steps, warmup = args.steps, min(args.warmup, 5)
    # bound the run: the oracle takes a few ms per step
    steps = min(steps, 2000)
    toks, sec_per_step, cores = time_cpu(args.streams, steps, warmup)
    sample = f"{steps} steps of the same layer shape at {args.streams} stream(s), rotating over 2 weight sets"
    line = {
        "impl": "reference", "metric": "moe_layer_decode_tok_per_s", "value": toks, "unit": "tok/s",
        "n_gpus": args.gpus, "steps": steps, "warmup": warmup, "ms_per_step": sec_per_step * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(args.streams),
        "cpu_baseline": {"value": toks, "unit": "tok/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": toks, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "CPU restatement of infr-cpu reference mode (f32 dequant + 8-lane f32 dot); the reference's int8/VNNI production path is a different numeric regime and is not restated",
    }
    print(json.dumps(line))


def workload_config(streams):
    return {"workload": f"Qwen3.6-35B-A3B-shaped MoE layer decode, {streams} stream(s): hidden 2048, 256 experts top-8, "
                        f"intermediate 512, gated shared expert, gate/up Q4_K, down Q6_K",
            "streams": streams, "layer_sets": LAYER_SETS,
            "l2": f"steps rotate over {LAYER_SETS} weight sets of {N_EXPERT * EXPERT_BYTES >> 20} MiB each (inputs larger than L2)"}


# ---------------------------------------------------------------------------------------------
# our arm
# ---------------------------------------------------------------------------------------------

def run_ours(args):
    import numpy as np
    import torch
    import torch.distributed as dist

    from moe4all_b200 import CudaBackend, MoeFfn, build
    from moe4all_b200.devgen import DeviceLayer

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device(f"cuda:{local}"))
    torch.cuda.set_device(local)
    dev = f"cuda:{local}"
    build.build()
    be = CudaBackend(local)
    stream = torch.cuda.Stream()
    torch.cuda.set_stream(stream)
    be.set_stream(stream.cuda_stream)

    R, K, W = args.streams, args.steps, max(args.warmup, 3)
    layers = [DeviceLayer(be, 1000 * (rank + 1) + i, NE, N_EXPERT, N_FF, sh_ff=SH_FF, device=dev) for i in range(LAYER_SETS)]
    gen = torch.Generator(device=dev)
    gen.manual_seed(1234 + rank)
    x_dev = torch.randn(X_POOL, R, NE, generator=gen, device=dev)
    xb = [be.wrap_tensor(x_dev[i]) for i in range(X_POOL)]
    dst_t = torch.zeros(R, NE, device=dev)
    ids_t = torch.zeros(R, N_USED, dtype=torch.int32, device=dev)
    wts_t = torch.zeros(R, N_USED, device=dev)
    dst, ids, wts = be.wrap_tensor(dst_t), be.wrap_tensor(ids_t), be.wrap_tensor(wts_t)

    def op_for(step, xbuf=None, stages=0):
        b = layers[step % LAYER_SETS].b
        return MoeFfn(x=xbuf if xbuf is not None else xb[step % X_POOL], router=b["router"], gate_exps=b["gate"],
                      up_exps=b["up"], down_exps=b["down"], dst=dst, rows=R, ne=NE, n_expert=N_EXPERT,
                      n_used=N_USED, n_ff_exp=N_FF, ids_out=ids, wts_out=wts, sh_gate=b["sh_gate"],
                      sh_up=b["sh_up"], sh_down=b["sh_down"], sh_gate_inp=b["sh_gate_inp"], sh_ff=SH_FF, stages=stages)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-resident timing: K steps recorded once, replayed (the reference replays a
    # recorded decode step the same way); warm-up runs the same steps un-recorded ---------------
    for s in range(W):
        be.moe_ffn(op_for(s))
    be.sync()
    # distinct experts per step (for the byte count): routing of the first pass over the pool
    u_list = []
    for s in range(min(K, LAYER_SETS * 4)):
        be.moe_ffn(op_for(s))
        be.sync()
        u_list.append(distinct_experts(ids_t.cpu().numpy()))
    mean_u = sum(u_list) / len(u_list)

    chunk = min(K, 512)
    be.graph_begin()
    for s in range(chunk):
        be.moe_ffn(op_for(s))
    plan = be.graph_end()
    be.execute(plan)
    be.sync()

    sampler = ClockSampler(local)
    time.sleep(0.25)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    launches0 = be.launch_count()
    barrier()
    e0.record()
    done = 0
    while done + chunk <= K:
        be.execute(plan)
        done += chunk
    for s in range(done, K):
        be.moe_ffn(op_for(s))
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1)
    launches = be.launch_count() - launches0
    # keep the GPU busy a little longer so the sampler sees clocks under load
    t_end = time.time() + 0.6
    while time.time() < t_end:
        be.execute(plan)
        be.sync()
    clocks = sampler.stop()

    # ---- dominant kernel alone: the gate/up dequant-GEMV ------------------------------------------
    for s in range(LAYER_SETS):
        be.moe_ffn(op_for(s, stages=2))
    be.sync()
    n_k = 200
    e2, e3 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    # eager launches are host-bound at this size; replay them from a recording instead
    be.graph_begin()
    for s in range(n_k):
        be.moe_ffn(op_for(s, stages=2))
    kplan = be.graph_end()
    be.execute(kplan)
    be.sync()
    e2.record()
    be.execute(kplan)
    e3.record()
    torch.cuda.synchronize()
    gateup_us = e2.elapsed_time(e3) * 1e3 / n_k

    # ---- end to end through the C ABI with host buffers -------------------------------------------
    x_host = torch.randn(X_POOL, R, NE).pin_memory()
    out_host = torch.empty(R, NE).pin_memory()
    x_in_t = torch.empty(R, NE, device=dev)
    x_in = be.wrap_tensor(x_in_t)
    nbytes = R * NE * 4
    e2e_steps = min(K, 2000)

    # The result rows are small enough for the down kernel to write them straight into pinned host
    # memory (dst is a handle on that memory), which saves the separate copy; with many rows a
    # device buffer and a queued copy are faster.
    host_dst = be.wrap(out_host.data_ptr(), nbytes) if R <= 8 else None
    x_ptrs = [x_host[i].data_ptr() for i in range(X_POOL)]
    # compile once, execute per step: one recorded plan per weight set holding the host-to-device
    # copy of the step's input from a pinned staging buffer, the layer, and (past eight rows) the
    # device-to-host copy of the result (Backend::compile / Backend::execute,
    # crates/infr-core/src/backend.rs:907-908): one launch and one host wait per step
    stage_in = torch.empty(R, NE).pin_memory()
    plans = []
    for i in range(LAYER_SETS):
        be.graph_begin()
        be.upload_ptr_async(x_in, stage_in.data_ptr(), nbytes)
        if host_dst is not None:
            be.moe_ffn(dataclasses.replace(op_for(i, xbuf=x_in), dst=host_dst))
        else:
            be.moe_ffn(op_for(i, xbuf=x_in))
            be.download_ptr_async(dst, out_host.data_ptr(), nbytes)
        plans.append(be.graph_end())
    stage_ptr = stage_in.data_ptr()
    memmove = ctypes.memmove

    def e2e_step(s):
        # the step's result is in host memory when sync() returns
        memmove(stage_ptr, x_ptrs[s % X_POOL], nbytes)
        be.execute(plans[s % LAYER_SETS])
        be.sync()

    for s in range(W):
        e2e_step(s)
    barrier()
    t0 = time.perf_counter()
    for s in range(e2e_steps):
        e2e_step(s)
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0
    barrier()

    # ---- reduce over ranks -----------------------------------------------------------------------
    t = torch.tensor([ms, e2e_s], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, e2e_s = float(t[0]), float(t[1])
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    peaks, peak_kind = measured_peaks()
    tok_s = world * R * K / (ms * 1e-3)
    step_us = ms * 1e3 / K
    active_bytes = (mean_u + 1) * EXPERT_BYTES  # routed experts actually touched + the shared expert
    layer_gbs = active_bytes / (step_us * 1e-6) / 1e9
    # gate/up kernel: per launch it reads the gate and up rows of the step's (token, slot) pairs'
    # distinct experts and of the shared expert
    gateup_bytes = (mean_u + 1) * 2 * N_FF * Q4K_ROW
    gateup_gbs = gateup_bytes / (gateup_us * 1e-6) / 1e9
    line = {
        "metric": "moe_layer_decode_tok_per_s", "value": tok_s, "unit": "tok/s", "n_gpus": world, "steps": K,
        "warmup": W, "ms_per_step": ms / K, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic", "config": workload_config(R),
        "active_expert_gbs": layer_gbs * world,
        "layer": {"us_per_step": step_us, "active_expert_bytes": active_bytes, "distinct_routed_experts": mean_u,
                  "hbm_frac_of_" + peak_kind: layer_gbs / peaks["hbm_gbs"]},
        "roofline": {"bound": "hbm", "kernel": "k_decode_gateup", "achieved": gateup_gbs, "peak": peaks["hbm_gbs"],
                     "unit": "GB/s", "frac": gateup_gbs / peaks["hbm_gbs"], "peak_kind": peak_kind,
                     "us_per_launch": gateup_us, "algorithmic_bytes": gateup_bytes,
                     "traffic": GATEUP_TRAFFIC_R1 if R == 1 else None},
        "e2e": {"value": world * R * e2e_steps / e2e_s, "unit": "tok/s", "h2d_bytes_per_step": nbytes,
                "d2h_bytes_per_step": nbytes, "steps": e2e_steps},
        "gpu_launches": launches, "clocks": clocks,
    }
    if world == 1 and not args.no_cpu_baseline:
        cpu_steps = 400
        toks, sec_per_step, cores = time_cpu(R, cpu_steps, 3)
        line["cpu_baseline"] = {"value": toks, "unit": "tok/s", "cores": cores, "kind": "port",
                                "sample": f"{cpu_steps} steps of the same layer shape at {R} stream(s), 2 weight sets, all host threads"}
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def setup_dist():
    import torch
    import torch.distributed as dist
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device(f"cuda:{local}"))
    torch.cuda.set_device(local)
    return world, rank, local


def timed(torch, dist, world, fn, steps):
    """K calls of fn between barriers, CUDA events on the current stream, max over ranks (ms)."""
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for s in range(steps):
        fn(s)
    e1.record()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    t = torch.tensor([e0.elapsed_time(e1)], device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t[0])


def run_stack(args):
    """Config 3: 40 MoE sub-layers (RmsNorm eps 1e-6, MoE + shared expert, residual add), steady-state
    decode; one step = one token row per stream through all 40 layers, replayed from a recording."""
    import torch
    import torch.distributed as dist
    from moe4all_b200 import CudaBackend, build
    from moe4all_b200.devgen import DeviceLayer
    from moe4all_b200.stack import MoeStack

    world, rank, local = setup_dist()
    build.build()
    be = CudaBackend(local)
    stream = torch.cuda.Stream()
    torch.cuda.set_stream(stream)
    be.set_stream(stream.cuda_stream)
    R, K, W, NL = args.streams, args.steps, max(args.warmup, 3), 40
    dev = f"cuda:{local}"
    layers = [DeviceLayer(be, 5000 * (rank + 1) + i, NE, N_EXPERT, N_FF, sh_ff=SH_FF, device=dev) for i in range(NL)]
    nws = [torch.ones(NE, device=dev) for _ in range(NL)]
    st = MoeStack(be, layers, nws, R, NE, N_EXPERT, N_USED, N_FF, sh_ff=SH_FF)
    st.hidden.normal_()
    st.record()
    for _ in range(W):
        st.replay()
    be.sync()
    u = sum(len(torch.unique(st.ids[li])) for li in range(NL))
    sampler = ClockSampler(local)
    l0 = be.launch_count()
    ms = timed(torch, dist, world, lambda s: st.replay(), K)
    launches = be.launch_count() - l0
    clocks = sampler.stop()
    # end to end: the step's hidden rows come from pinned host memory and go back there, one wait per step
    nbytes = R * NE * 4
    x_host = torch.randn(8, R, NE).pin_memory()
    out_host = torch.empty(R, NE).pin_memory()
    hid = st.b_hidden
    e2e_steps = min(K, 200)

    def e2e_step(s):
        be.upload_ptr_async(hid, x_host[s % 8].data_ptr(), nbytes)
        st.replay()
        be.download_ptr_async(hid, out_host.data_ptr(), nbytes)
        be.sync()

    for s in range(3):
        e2e_step(s)
    if world > 1:
        dist.barrier()
    t0 = time.perf_counter()
    for s in range(e2e_steps):
        e2e_step(s)
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0
    if world > 1:
        t = torch.tensor([e2e_s], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_s = float(t[0])
    if rank == 0:
        peaks, kind = measured_peaks()
        active = (u + NL) * EXPERT_BYTES
        us = ms * 1e3 / K
        print(json.dumps({
            "metric": "moe_stack_decode_tok_per_s", "value": world * R * K / (ms * 1e-3), "unit": "tok/s", "n_gpus": world,
            "steps": K, "warmup": W, "ms_per_step": ms / K, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic",
            "config": {"workload": f"40 Qwen3.6-35B-A3B-shaped MoE FFN layers with RmsNorm and residual add, decode, {R} stream(s)",
                       "streams": R, "l2": "40 independent weight sets, 21 GB resident (inputs larger than L2)"},
            "active_expert_gbs": world * active / (us * 1e-6) / 1e9,
            "roofline": {"bound": "hbm", "kernel": "whole step", "achieved": active / (us * 1e-6) / 1e9, "peak": peaks["hbm_gbs"],
                         "unit": "GB/s", "frac": active / (us * 1e-6) / 1e9 / peaks["hbm_gbs"], "peak_kind": kind, "traffic": None},
            "e2e": {"value": world * R * e2e_steps / e2e_s, "unit": "tok/s", "h2d_bytes_per_step": nbytes,
                    "d2h_bytes_per_step": nbytes, "steps": e2e_steps},
            "gpu_launches": launches, "clocks": clocks}))
    if world > 1:
        dist.destroy_process_group()


def run_prefill(args):
    """Config 2: one 4096-token chunk through the layer, router biased Zipf(1.1) over experts.
    N = 1: the batched path of one device.  N > 1: tokens and experts sharded over the ranks,
    NCCL all-to-all dispatch and combine."""
    import torch
    import torch.distributed as dist
    from moe4all_b200 import CudaBackend, MoeFfn, build
    from moe4all_b200.devgen import DeviceLayer
    from moe4all_b200.ep import CudaExpertParallelLayer

    world, rank, local = setup_dist()
    build.build()
    be = CudaBackend(local)
    stream = torch.cuda.Stream()
    torch.cuda.set_stream(stream)
    be.set_stream(stream.cuda_stream)
    dev = f"cuda:{local}"
    deepseek = args.shape == "deepseek"
    ne, n_expert, n_used, n_ff, sh_ff = (7168, 256, 8, 2048, 2048) if deepseek else (NE, N_EXPERT, N_USED, N_FF, SH_FF)
    route_kw = dict(scale=2.5, gating=1, n_expert_groups=8, n_expert_groups_used=4) if deepseek else {}
    T, K, W = args.tokens or (8192 if deepseek else 4096), args.steps, max(args.warmup, 3)
    rows = T // world
    band = None if world == 1 else (rank * (n_expert // world), n_expert // world)
    L = DeviceLayer(be, 77, ne, n_expert, n_ff, sh_ff=sh_ff, gated_shared=not deepseek, device=dev, band=band)
    gen = torch.Generator(device=dev)
    if not deepseek:
        gen.manual_seed(9)
        zipf = -1.1 * torch.log((torch.randperm(n_expert, generator=gen, device=dev) + 1).float())
        L.t["router"][:-16].view(torch.float32).view(n_expert, ne)[:, ne - 1] = zipf
    gen.manual_seed(100 + rank)
    x = torch.randn(rows, ne, generator=gen, device=dev)
    dst = torch.empty_like(x)
    b = L.b
    if world == 1:
        rx = x.clone()
        if not deepseek:
            rx[:, ne - 1] = 1.0  # the bias column is read by the router only (separate router_x handle)
        op = MoeFfn(x=be.wrap_tensor(x), router_x=be.wrap_tensor(rx), router=b["router"], gate_exps=b["gate"], up_exps=b["up"],
                    down_exps=b["down"], dst=be.wrap_tensor(dst), rows=rows, ne=ne, n_expert=n_expert, n_used=n_used,
                    n_ff_exp=n_ff, sh_gate=b["sh_gate"], sh_up=b["sh_up"], sh_down=b["sh_down"], sh_gate_inp=b.get("sh_gate_inp"),
                    sh_ff=sh_ff, path=0 if T < 512 else 2, **route_kw)
        step = lambda s: be.moe_ffn(op)
    else:
        if not deepseek:
            x[:, ne - 1] = 1.0  # expert-parallel layer routes on x itself
        layer = CudaExpertParallelLayer(be, L, n_expert, n_used, n_ff, ne, **{("n_groups" if k == "n_expert_groups" else "n_groups_used" if k == "n_expert_groups_used" else k): v for k, v in route_kw.items()})
        step = lambda s: layer.forward(x, rows_equal=True)  # small calls take the fixed-shape exchange
    for s in range(W):
        step(s)
    sampler = ClockSampler(local)
    l0 = be.launch_count()
    ms = timed(torch, dist, world, step, K)
    launches = be.launch_count() - l0
    clocks = sampler.stop()
    # end to end: this rank's token rows come from pinned host memory and the results go back there
    # (copy-engine transfers at this size), one host wait per step
    nbytes = rows * ne * 4
    x_pin = x.cpu().pin_memory()
    out_pin = torch.empty(rows, ne).pin_memory()
    xb, db = be.wrap_tensor(x), be.wrap_tensor(dst)
    e2e_steps = min(K, 20)

    def e2e_step(s):
        be.upload_ptr_async(xb, x_pin.data_ptr(), nbytes)
        out = step(s)
        be.download_ptr_async(db if world == 1 else be.wrap_tensor(out), out_pin.data_ptr(), nbytes)
        be.sync()

    for s in range(2):
        e2e_step(s)
    if world > 1:
        dist.barrier()
    t0 = time.perf_counter()
    for s in range(e2e_steps):
        e2e_step(s)
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0
    if world > 1:
        tt = torch.tensor([e2e_s], device=dev, dtype=torch.float64)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        e2e_s = float(tt[0])
    if rank == 0:
        peaks, kind = measured_peaks()
        flops = 3 * 2 * T * n_used * ne * n_ff  # routed experts only (2*pairs*K*N per GEMM)
        tfl = flops / (ms / K * 1e-3) / 1e12
        print(json.dumps({
            "metric": "moe_prefill_routed_tflops", "value": tfl, "unit": "TFLOP/s", "n_gpus": world, "steps": K, "warmup": W,
            "ms_per_step": ms / K, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f16",
            "data": "synthetic", "tokens_per_s": T * K / (ms * 1e-3),
            "config": {"workload": (f"{T} tokens through one DeepSeek-V3-shaped MoE layer (hidden 7168, 256 experts top-8 in 8 groups / 4 used, "
                                    f"intermediate 2048, shared expert)" if deepseek else
                                    f"{T}-token prefill chunk through one Qwen3.6-35B-A3B-shaped MoE layer, Zipf(1.1) router bias"),
                       "parallelism": f"ep{world}" if world > 1 else "single",
                       "l2": f"{n_expert * (2 * n_ff * (ne // 256 * 144) + ne * (n_ff // 256 * 210)) >> 20} MiB expert banks (inputs larger than L2)"},
            "roofline": {"bound": "tensor", "kernel": "whole step (router + permute + grouped GEMMs + combine)", "achieved": tfl,
                         "peak": peaks["bf16_tflops"], "unit": "TFLOP/s", "frac": tfl / peaks["bf16_tflops"], "peak_kind": kind,
                         "traffic": None},
            "e2e": {"value": flops * e2e_steps / e2e_s / 1e12, "unit": "TFLOP/s", "h2d_bytes_per_step": nbytes,
                    "d2h_bytes_per_step": nbytes, "steps": e2e_steps},
            "gpu_launches": launches, "clocks": clocks}))
    if world > 1:
        dist.destroy_process_group()


def main():
    args = parse_args()
    if args.impl == "reference":
        run_reference(args)
    elif args.workload == "stack":
        run_stack(args)
    elif args.workload == "prefill":
        run_prefill(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
