#!/usr/bin/env python
"""Benchmark of the quantized MoE FFN hot path on B200.

    python bench.py --gpus N --steps K --warmup W [--streams R] [--workload layer|stack|prefill] [--impl reference]

Headline workload (`layer`): one Qwen3.6-35B-A3B-shaped MoE layer (hidden 2048, 256 routed experts,
top-8, expert intermediate 512, one sigmoid-gated shared expert; gate/up Q4_K, down Q6_K, router f32),
decode with R concurrent streams.  One step = one pass of the layer over one batch of R token rows.
Weights are synthetic (random block payload, f16 scales ~ U[1e-4, 1e-3], router ~ N(0, 0.02)),
activations ~ N(0, 1).  Steps rotate over `--layer-sets` independent weight sets so the weights a step
touches were evicted from L2 since their last use.  The K steps are recorded once and replayed
`--repeats` times; the reported time is the median replay (max over ranks).

N > 1: every rank runs its own replica of the streams on its own GPU (token rows are independent; no
collective on the decode data path).  The line's `prefill` sub-record is where the ranks work
together: the 4096-token chunk with experts sharded over the N ranks inside the library (NCCL
dispatch and combine), timed between barriers, max over ranks, with the per-phase breakdown and the
difference from the single-device result of the same rows.

The line printed by rank 0 follows the driver's contract.  `roofline` is the whole layer step on
active-expert bytes, with the three kernels' own times beside it; `prefill` and `stack` are the
other two halves of the metric (4096-token prefill chunk, TFLOP/s; 40-layer stack, tok/s);
`cpu_baseline` is the CPU oracle (a restatement of the reference's infr-cpu reference-mode
arithmetic) timed on the host cores on a bounded sample.  `e2e` is the same step with host buffers
through the C ABI: the rows start in pinned host memory and the result ends there, step after step,
as a host-paced plan (steps recorded and launched once, each released by a ticket the host writes);
`e2e.launch_per_step` is the same with one plan launch and one stream wait per step.
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
X_POOL = 64
Q4K_ROW = NE // 256 * 144      # bytes of one gate/up row
Q6K_ROW = N_FF // 256 * 210    # bytes of one down row
EXPERT_BYTES = 2 * N_FF * Q4K_ROW + NE * Q6K_ROW  # 2 039 808
# --banks: GGUF type numbers and (elements, bytes) per block of the formats an expert bank may have
BANK_TYPES = {"q4_0": 2, "q4_1": 3, "q5_0": 6, "q5_1": 7, "q8_0": 8, "q2k": 10, "q3k": 11, "q4k": 12, "q5k": 13, "q6k": 14, "iq4_nl": 20, "iq4_xs": 23, "mxfp4": 39, "nvfp4": 40, "q2_0": 42,
              "iq2_xs": 17, "iq2_s": 22, "iq3_xxs": 18, "iq3_s": 21}
BANK_BLOCK = {2: (32, 18), 3: (32, 20), 6: (32, 22), 7: (32, 24), 8: (32, 34), 10: (256, 84), 11: (256, 110), 12: (256, 144), 13: (256, 176),
              14: (256, 210), 20: (32, 18), 23: (256, 136), 39: (32, 17), 40: (64, 36), 42: (64, 18),
              17: (256, 74), 22: (256, 82), 18: (256, 98), 21: (256, 110)}
BANKS = (12, 12, 14)           # gate, up, down of the layer workload (set from --banks)


def set_banks(spec):
    """--banks gate,up,down: the layer workload's bank formats; the byte counts follow."""
    global BANKS, Q4K_ROW, Q6K_ROW, EXPERT_BYTES
    names = spec.lower().split(",")
    if len(names) != 3 or any(n not in BANK_TYPES for n in names):
        raise SystemExit(f"--banks wants gate,up,down out of {sorted(BANK_TYPES)}")
    BANKS = tuple(BANK_TYPES[n] for n in names)
    row = lambda dt, n: n // BANK_BLOCK[dt][0] * BANK_BLOCK[dt][1]
    Q4K_ROW, Q6K_ROW = (row(BANKS[0], NE) + row(BANKS[1], NE)) / 2, row(BANKS[2], N_FF)  # mean gate/up row, down row
    EXPERT_BYTES = int(2 * N_FF * Q4K_ROW + NE * Q6K_ROW)
    if BANKS != (12, 12, 14):
        global DTYPE
        DTYPE = DTYPE.replace("Q4_K / Q6_K codes", banks_name() + " codes")


def banks_tuned():
    return BANKS[0] == 12 and BANKS[1] == 12 and BANKS[2] in (12, 14)


def banks_name():
    inv = {v: k for k, v in BANK_TYPES.items()}
    pretty = {k: k.upper().replace("K", "_K") if k.endswith("k") else k.upper() for k in BANK_TYPES}
    g, u, d = (pretty[inv[b]] for b in BANKS)
    return f"gate/up {g}, down {d}" if g == u else f"gate {g}, up {u}, down {d}"
# DRAM bytes (dram__bytes_read.sum + dram__bytes_write.sum) of one launch of each kernel of the step at
# 1 stream, from an ncu capture of this workload: router, gate/up, down
NCU_TRAFFIC_R1 = {"k_router_small": 2_196_736, "k_decode_gateup": 10_651_392, "k_decode_down": 7_798_528}
DTYPE = "f32 accumulate; weights as stored (Q4_K / Q6_K codes), activations 16-bit fixed point (decode) or f16 (prefill)"


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=400)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--repeats", type=int, default=50, help="replays of the recorded K steps; the median is reported")
    ap.add_argument("--streams", type=int, default=1, help="concurrent decode streams (rows per step)")
    ap.add_argument("--layer-sets", type=int, default=16, help="independent weight sets the steps rotate over (0.5 GB each; "
                    "2 keeps a profiler capture under 2 GB resident)")
    ap.add_argument("--workload", default="layer", choices=["layer", "stack", "prefill"],
                    help="layer: one MoE layer per step (the headline, with the other two as sub-records); stack: 40 such "
                         "layers with RmsNorm and residual add per step; prefill: one 4096-token chunk through one layer per step")
    ap.add_argument("--tokens", type=int, default=0, help="tokens of the prefill chunk (default 4096, or 8192 for --shape deepseek; "
                    "64 is the largest configuration's decode batch; a smaller chunk also suits profiler captures)")
    ap.add_argument("--shape", default="qwen", choices=["qwen", "deepseek"],
                    help="prefill workload only: the 256-expert Qwen3.6-35B-A3B layer, or the DeepSeek-V3-shaped one "
                         "(hidden 7168, intermediate 2048, sigmoid gating in 8 groups / 4 used, ungated shared expert)")
    ap.add_argument("--banks", default="q4k,q4k,q6k", help="layer workload: formats of the gate, up and down banks "
                    "(q4_0, q4_1, q5_0, q5_1, q8_0, q2k ... q6k, iq4_nl, iq4_xs); the default is the configuration the metric is quoted on")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-subrecords", action="store_true", help="layer workload: skip the prefill and stack sub-records")
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
    return [synth.make_layer(1000 + i, NE, N_EXPERT, N_FF, sh_ff=SH_FF, dtypes=None if BANKS == (12, 12, 14) else BANKS)
            for i in range(n_sets)]


def cpu_step(orc, L, x, router_x=None):
    return orc.moe_layer(x, L.router, L.gate, L.up, L.down, L.sh_gate, L.sh_up, L.sh_down, L.sh_gate_inp, SH_FF,
                         n_expert=N_EXPERT, n_used=N_USED, n_ff_exp=N_FF, threads=0, router_x=router_x,
                         gate_dtype=L.gate_dtype, up_dtype=L.up_dtype, down_dtype=L.down_dtype)


def time_cpu(streams, steps, warmup, n_sets=2):
    """tok/s of the CPU oracle on `steps` steps of the layer workload (all host threads)."""
    from moe4all_b200 import synth
    from oracle import oracle as orc
    for dt in sorted(set(BANKS) & set(synth.CODEBOOKS)):
        orc.set_codebook(dt, synth.codebook(dt))
    layers = cpu_layers(n_sets)
    xs = [synth.activations(50 + i, streams, NE) for i in range(8)]
    for i in range(warmup):
        cpu_step(orc, layers[i % n_sets], xs[i % 8])
    t0 = time.perf_counter()
    for i in range(steps):
        cpu_step(orc, layers[i % n_sets], xs[i % 8])
    dt = time.perf_counter() - t0
    return streams * steps / dt, dt / steps, orc.hw_threads()


def reference_layer(args):
    steps, warmup = min(args.steps, 2000), min(args.warmup, 5)  # the oracle takes a few ms per step
    toks, sec_per_step, cores = time_cpu(args.streams, steps, warmup)
    sample = f"{steps} steps of the same layer shape at {args.streams} stream(s), rotating over 2 weight sets"
    return dict(metric="moe_layer_decode_tok_per_s", value=toks, unit="tok/s", steps=steps, warmup=warmup, ms_per_step=sec_per_step * 1e3,
                scaling="weak", config=workload_config(args.streams, args.layer_sets), cores=cores, sample=sample)


def reference_stack(args):
    """The 40-layer step on the CPU: 40 sub-layers per step, rotating over 2 weight sets (21 GB of host
    weights would take minutes to synthesise; the arithmetic per layer is the same)."""
    import numpy as np
    from moe4all_b200 import synth
    from oracle import oracle as orc
    R, NL = args.streams, 40
    layers = cpu_layers(2)
    nw = np.ones(NE, np.float32)
    steps, warmup = max(1, min(args.steps, 12 if R <= 4 else 2)), 1

    def step(h):
        for li in range(NL):
            hn = orc.rmsnorm(h, nw, 1e-6)
            h = orc.add(h, cpu_step(orc, layers[li % 2], hn).dst)
        return h

    h = synth.activations(7, R, NE)
    for _ in range(warmup):
        step(h)
    t0 = time.perf_counter()
    for _ in range(steps):
        step(h)
    dt = time.perf_counter() - t0
    return dict(metric="moe_stack_decode_tok_per_s", value=R * steps / dt, unit="tok/s", steps=steps, warmup=warmup,
                ms_per_step=dt / steps * 1e3, scaling="weak", config=stack_config(R), cores=orc.hw_threads(),
                sample=f"{steps} steps of 40 sub-layers at {R} stream(s), the 40 layers rotating over 2 weight sets")


def reference_prefill(args):
    """The prefill chunk on the CPU, on a token subset: rows are independent in the reference's f32 mode, so the
    time scales with the tokens; the subset keeps the run to seconds."""
    import numpy as np
    from moe4all_b200 import synth
    from oracle import oracle as orc
    if args.shape == "deepseek":
        return None
    T = args.tokens or 4096
    sub = max(64, T // 16)
    L = synth.make_layer(77, NE, N_EXPERT, N_FF, sh_ff=SH_FF)
    rng = np.random.default_rng(9)
    L.router[:, NE - 1] = -1.1 * np.log(rng.permutation(N_EXPERT) + 1.0)
    x = synth.activations(100, sub, NE)
    rx = x.copy()
    rx[:, NE - 1] = 1.0
    steps = max(1, min(args.steps, 3))
    cpu_step(orc, L, x, rx)
    t0 = time.perf_counter()
    for _ in range(steps):
        cpu_step(orc, L, x, rx)
    dt = (time.perf_counter() - t0) / steps
    flops = 3 * 2 * sub * N_USED * NE * N_FF
    return dict(metric="moe_prefill_routed_tflops", value=flops / dt / 1e12, unit="TFLOP/s", steps=steps, warmup=1, ms_per_step=dt * 1e3,
                scaling="strong", config=prefill_config(T, False, 1), cores=orc.hw_threads(),
                sample=f"{steps} passes over a {sub}-token subset (1/{T // sub}) of the {T}-token chunk, same Zipf(1.1) router bias; "
                       f"TFLOP/s counts the subset's routed FLOPs")


def run_reference(args):
    if int(os.environ.get("RANK", "0")) != 0:
        return
    rec = {"layer": reference_layer, "stack": reference_stack, "prefill": reference_prefill}[args.workload](args)
    if rec is None:
        print(json.dumps({"impl": "reference", "unavailable": "the CPU restatement is not timed on the DeepSeek-shaped prefill (hours of host time)"}))
        return
    cores, sample = rec.pop("cores"), rec.pop("sample")
    line = {"impl": "reference", **rec, "n_gpus": args.gpus, "higher_is_better": True, "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "cpu_baseline": {"value": rec["value"], "unit": rec["unit"], "cores": cores, "kind": "port", "sample": sample},
            "e2e": {"value": rec["value"], "unit": rec["unit"], "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "note": "CPU restatement of infr-cpu reference mode (f32 dequant + 8-lane f32 dot); the reference's int8/VNNI production path is a different numeric regime and is not restated"}
    print(json.dumps(line))


def workload_config(streams, layer_sets):
    return {"workload": f"Qwen3.6-35B-A3B-shaped MoE layer decode, {streams} stream(s): hidden 2048, 256 experts top-8, "
                        f"intermediate 512, gated shared expert, {banks_name()}",
            "streams": streams, "layer_sets": layer_sets,
            "l2": f"steps rotate over {layer_sets} weight sets of {N_EXPERT * EXPERT_BYTES >> 20} MiB each (inputs larger than L2)"}


def stack_config(R):
    return {"workload": f"40 Qwen3.6-35B-A3B-shaped MoE FFN layers with RmsNorm and residual add, decode, {R} stream(s)",
            "streams": R, "l2": "40 independent weight sets, 21 GB resident (inputs larger than L2)"}


def prefill_config(T, deepseek, world):
    ne, n_expert, n_ff = (7168, 256, 2048) if deepseek else (NE, N_EXPERT, N_FF)
    return {"workload": (f"{T} tokens through one DeepSeek-V3-shaped MoE layer (hidden 7168, 256 experts top-8 in 8 groups / 4 used, "
                         f"intermediate 2048, shared expert)" if deepseek else
                         f"{T}-token prefill chunk through one Qwen3.6-35B-A3B-shaped MoE layer, Zipf(1.1) router bias"),
            "parallelism": f"ep{world}" if world > 1 else "single",
            "l2": f"{n_expert * (2 * n_ff * (ne // 256 * 144) + ne * (n_ff // 256 * 210)) >> 20} MiB expert banks (inputs larger than L2)"}


# ---------------------------------------------------------------------------------------------
# our arm
# ---------------------------------------------------------------------------------------------

class Env:
    """One rank: device, stream, backend context, process group."""

    def __init__(self):
        import torch
        import torch.distributed as dist
        from moe4all_b200 import CudaBackend, DType, build
        self.torch, self.dist = torch, dist
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.local = int(os.environ.get("LOCAL_RANK", "0"))
        if self.world > 1:
            dist.init_process_group("nccl", device_id=torch.device(f"cuda:{self.local}"))
        torch.cuda.set_device(self.local)
        self.dev = f"cuda:{self.local}"
        build.build()
        self.be = CudaBackend(self.local)
        # --banks with a grid codebook format: the stand-in tables of synth.codebook (same shape and alphabet as
        # the real ones, which a host of the reference would hand over)
        from moe4all_b200 import synth as _synth
        for dt in sorted(set(BANKS) & set(_synth.CODEBOOKS)):
            self.be.set_codebook(DType(dt), _synth.codebook(dt))
        self.stream = torch.cuda.Stream()
        torch.cuda.set_stream(self.stream)
        self.be.set_stream(self.stream.cuda_stream)

    def barrier(self):
        if self.world > 1:
            self.dist.barrier()
        self.torch.cuda.synchronize()

    def max_over_ranks(self, *vals):
        t = self.torch.tensor(list(vals), device=self.dev, dtype=self.torch.float64)
        if self.world > 1:
            self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return [float(v) for v in t]

    def close(self):
        if self.world > 1:
            self.dist.destroy_process_group()


def timed_repeats(env, fn, repeats):
    """`repeats` calls of fn, each between CUDA events on the current stream, the whole between barriers;
    returns (median ms, all ms) of this rank."""
    torch = env.torch
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(repeats)]
    env.barrier()
    for a, b in ev:
        a.record()
        fn()
        b.record()
    env.barrier()
    ms = [a.elapsed_time(b) for a, b in ev]
    return statistics.median(ms), ms


def timed(env, fn, steps):
    """K calls of fn between barriers, CUDA events on the current stream, max over ranks (ms)."""
    torch = env.torch
    env.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for s in range(steps):
        fn(s)
    e1.record()
    env.barrier()
    return env.max_over_ranks(e0.elapsed_time(e1))[0]


def measure_stack(env, layers, R, steps, warmup, with_e2e=True):
    """Config 3: 40 MoE sub-layers (RmsNorm eps 1e-6, MoE + shared expert, residual add), steady-state
    decode; one step = one token row per stream through all 40 layers, replayed from a recording."""
    torch, be = env.torch, env.be
    from moe4all_b200.stack import MoeStack
    NL = len(layers)
    nws = [torch.ones(NE, device=env.dev) for _ in range(NL)]
    st = MoeStack(be, layers, nws, R, NE, N_EXPERT, N_USED, N_FF, sh_ff=SH_FF)
    st.hidden.normal_()
    st.record()
    for _ in range(warmup):
        st.replay()
    be.sync()
    u = sum(len(torch.unique(st.ids[li])) for li in range(NL))
    l0 = be.launch_count()
    ms = timed(env, lambda s: st.replay(), steps)
    launches = be.launch_count() - l0
    rec = {"streams": R, "steps": steps, "ms_per_step": ms / steps, "tok_per_s": env.world * R * steps / (ms * 1e-3), "gpu_launches": launches}
    peaks, kind = measured_peaks()
    active = (u + NL) * EXPERT_BYTES
    gbs = active / (ms / steps * 1e-3) / 1e9
    rec.update({"active_expert_bytes": active, "active_expert_gbs": gbs, "hbm_frac_of_" + kind: gbs / peaks["hbm_gbs"]})
    if with_e2e:
        # end to end: the step's hidden rows come from pinned host memory and go back there, one wait per step
        nbytes = R * NE * 4
        x_host = torch.randn(8, R, NE).pin_memory()
        out_host = torch.empty(R, NE).pin_memory()
        hid = st.b_hidden
        e2e_steps = min(steps, 200)

        def e2e_step(s):
            be.upload_ptr_async(hid, x_host[s % 8].data_ptr(), nbytes)
            st.replay()
            be.download_ptr_async(hid, out_host.data_ptr(), nbytes)
            be.sync()

        for s in range(3):
            e2e_step(s)
        env.barrier()
        t0 = time.perf_counter()
        for s in range(e2e_steps):
            e2e_step(s)
        torch.cuda.synchronize()
        e2e_s = env.max_over_ranks(time.perf_counter() - t0)[0]
        rec["e2e"] = {"value": env.world * R * e2e_steps / e2e_s, "unit": "tok/s", "h2d_bytes_per_step": nbytes,
                      "d2h_bytes_per_step": nbytes, "steps": e2e_steps}
    del st
    return rec


def prefill_dims(deepseek):
    dims = (7168, 256, 8, 2048, 2048) if deepseek else (NE, N_EXPERT, N_USED, N_FF, SH_FF)
    route_kw = dict(scale=2.5, gating=1, n_expert_groups=8, n_expert_groups_used=4) if deepseek else {}
    return dims, route_kw


def zipf_router(env, L, n_expert, ne):
    """Zipf(1.1) bias over a random permutation of the experts in the router's last column; a row whose last
    element is 1 picks it up."""
    torch = env.torch
    gen = torch.Generator(device=env.dev)
    gen.manual_seed(9)
    zipf = -1.1 * torch.log((torch.randperm(n_expert, generator=gen, device=env.dev) + 1).float())
    L.t["router"][:-16].view(torch.float32).view(n_expert, ne)[:, ne - 1] = zipf


def measure_prefill(env, T, deepseek, steps, warmup, with_e2e=True):
    """Config 2 (or the DeepSeek-shaped layer): one T-token chunk through the layer per step.  One GPU: the
    batched path.  N GPUs: tokens and experts sharded over the ranks inside the library (NCCL dispatch and
    combine), compared with the single-device result of this rank's rows."""
    torch, be, world, rank, dev = env.torch, env.be, env.world, env.rank, env.dev
    import numpy as np
    from moe4all_b200 import CudaBackend, MoeFfn
    from moe4all_b200.devgen import DeviceLayer
    from moe4all_b200.ep import LibraryExpertParallelLayer, join_communicator
    (ne, n_expert, n_used, n_ff, sh_ff), route_kw = prefill_dims(deepseek)
    rows = T // world
    gen = torch.Generator(device=dev)
    gen.manual_seed(100 + rank)
    x = torch.randn(rows, ne, generator=gen, device=dev)
    dst = torch.empty_like(x)
    full = None
    if world == 1 or not deepseek:  # the DeepSeek-shaped layer (7 GB) is only held whole on a single GPU
        full = DeviceLayer(be, 77, ne, n_expert, n_ff, sh_ff=sh_ff, gated_shared=not deepseek, device=dev)
        if not deepseek:
            zipf_router(env, full, n_expert, ne)

    def single_op(xt, dt, n):
        b = full.b
        rx = xt
        if not deepseek and world == 1:
            rx = xt.clone()
            rx[:, ne - 1] = 1.0  # the bias column is read by the router only (separate router_x handle)
        return MoeFfn(x=be.wrap_tensor(xt), router_x=be.wrap_tensor(rx), router=b["router"], gate_exps=b["gate"], up_exps=b["up"],
                      down_exps=b["down"], dst=be.wrap_tensor(dt), rows=n, ne=ne, n_expert=n_expert, n_used=n_used, n_ff_exp=n_ff,
                      sh_gate=b["sh_gate"], sh_up=b["sh_up"], sh_down=b["sh_down"], sh_gate_inp=b.get("sh_gate_inp"), sh_ff=sh_ff,
                      path=0 if T < 512 else 2, **route_kw)

    extra = {}
    if world == 1:
        op = single_op(x, dst, rows)
        step = lambda s: be.moe_ffn(op)
        sync_be = be
    else:
        if not deepseek:
            x[:, ne - 1] = 1.0  # the expert-parallel call routes on x itself
        el = n_expert // world
        be_ep = CudaBackend(env.local)
        be_ep.set_stream(env.stream.cuda_stream)
        join_communicator(be_ep)
        band = DeviceLayer(be_ep, 77, ne, n_expert, n_ff, sh_ff=sh_ff, gated_shared=not deepseek, device=dev, band=(rank * el, el))
        if not deepseek:
            zipf_router(env, band, n_expert, ne)
        layer = LibraryExpertParallelLayer(be_ep, band, n_expert, n_used, n_ff, ne, sh_ff=sh_ff, **route_kw)
        step = lambda s: layer.forward(x, out=dst)
        sync_be = be_ep
    for s in range(warmup):
        step(s)
    sync_be.sync()
    l0 = sync_be.launch_count()
    ms = timed(env, step, steps)
    launches = sync_be.launch_count() - l0
    if world > 1:
        # per-phase breakdown of the last call on every rank (the slowest rank per phase), and parity with
        # the single-device op on this rank's rows
        step(0)
        ph = sync_be.ep_last_phases()
        deltas = [ph[0]] + [b - a for a, b in zip(ph, ph[1:])]
        worst = env.max_over_ranks(*deltas)
        extra["ep_phases_ms"] = dict(zip(("route", "dispatch", "band_experts", "combine_exchange", "sum_and_shared"), worst))
        band_ms = env.torch.tensor([deltas[2]], device=dev, dtype=torch.float64)
        all_band = [torch.zeros_like(band_ms) for _ in range(world)]
        env.dist.all_gather(all_band, band_ms)
        extra["band_experts_ms_per_rank"] = [float(v) for v in all_band]
        if full is not None:
            # The comparison isolates the exchange: both sides keep the experts' raw rows in f32 for it (the
            # single-device call rounds the shared expert's rows to f16 with the routed ones, the band call
            # computes them apart), so what is left is the association of the sum over ranks.
            be.set_config(raw_rows_f32=1)
            sync_be.set_config(raw_rows_f32=1)
            step(0)
            sync_be.sync()
            ref = torch.empty_like(x)
            be.moe_ffn(single_op(x, ref, rows))
            be.sync()
            torch.cuda.synchronize()
            mag = float(ref.abs().max())
            extra["ep_parity_rel"] = env.max_over_ranks(float((dst - ref).abs().max()) / max(mag, 1e-3))[0]
            be.set_config(raw_rows_f32=0)
            sync_be.set_config(raw_rows_f32=0)
    flops = 3 * 2 * T * n_used * ne * n_ff  # routed experts only (2*pairs*K*N per GEMM)
    tfl = flops / (ms / steps * 1e-3) / 1e12
    peaks, kind = measured_peaks()
    rec = {"tokens": T, "n_gpus": world, "parallelism": f"ep{world}" if world > 1 else "single", "steps": steps, "ms_per_step": ms / steps,
           "routed_tflops": tfl, "tokens_per_s": T * steps / (ms * 1e-3),
           "tensor_frac_of_" + kind: tfl / (peaks["bf16_tflops"] * world), "gpu_launches": launches, **extra}
    if with_e2e:
        # end to end: this rank's token rows come from pinned host memory and the results go back there
        # (copy-engine transfers at this size), one host wait per step
        nbytes = rows * ne * 4
        x_pin = x.cpu().pin_memory()
        out_pin = torch.empty(rows, ne).pin_memory()
        xb, db = sync_be.wrap_tensor(x), sync_be.wrap_tensor(dst)
        e2e_steps = min(steps, 20)

        def e2e_step(s):
            sync_be.upload_ptr_async(xb, x_pin.data_ptr(), nbytes)
            step(s)
            sync_be.download_ptr_async(db, out_pin.data_ptr(), nbytes)
            sync_be.sync()

        for s in range(2):
            e2e_step(s)
        env.barrier()
        t0 = time.perf_counter()
        for s in range(e2e_steps):
            e2e_step(s)
        torch.cuda.synchronize()
        e2e_s = env.max_over_ranks(time.perf_counter() - t0)[0]
        rec["e2e"] = {"value": flops * e2e_steps / e2e_s / 1e12, "unit": "TFLOP/s", "h2d_bytes_per_step": nbytes,
                      "d2h_bytes_per_step": nbytes, "steps": e2e_steps}
    if world > 1:
        sync_be.ep_finalize()
        sync_be.close()
    return rec


def run_ours(args):
    import torch
    from moe4all_b200 import DType, MoeFfn
    from moe4all_b200.devgen import DeviceLayer

    env = Env()
    be, world, rank, dev = env.be, env.world, env.rank, env.dev
    R, K, W, SETS = args.streams, args.steps, max(args.warmup, 3), max(args.layer_sets, 1)
    subrecords = not args.no_subrecords and BANKS == (12, 12, 14)  # the sub-records are the default formats' configs
    # the stack sub-record needs 40 layers; the layer workload rotates over the first SETS of them
    n_layers = max(SETS, 40) if subrecords else SETS
    layers = [DeviceLayer(be, 1000 * (rank + 1) + i, NE, N_EXPERT, N_FF, sh_ff=SH_FF, device=dev, dtypes=BANKS) for i in range(n_layers)]
    gen = torch.Generator(device=dev)
    gen.manual_seed(1234 + rank)
    x_dev = torch.randn(X_POOL, R, NE, generator=gen, device=dev)
    xb = [be.wrap_tensor(x_dev[i]) for i in range(X_POOL)]
    dst_t = torch.zeros(R, NE, device=dev)
    ids_t = torch.zeros(R, N_USED, dtype=torch.int32, device=dev)
    wts_t = torch.zeros(R, N_USED, device=dev)
    dst, ids, wts = be.wrap_tensor(dst_t), be.wrap_tensor(ids_t), be.wrap_tensor(wts_t)

    def op_for(step, xbuf=None, stages=0):
        b = layers[step % SETS].b
        return MoeFfn(x=xbuf if xbuf is not None else xb[step % X_POOL], router=b["router"], gate_exps=b["gate"],
                      up_exps=b["up"], down_exps=b["down"], dst=dst, rows=R, ne=NE, n_expert=N_EXPERT,
                      n_used=N_USED, n_ff_exp=N_FF, ids_out=ids, wts_out=wts, sh_gate=b["sh_gate"],
                      sh_up=b["sh_up"], sh_down=b["sh_down"], sh_gate_inp=b["sh_gate_inp"], sh_ff=SH_FF, stages=stages,
                      gate_dtype=DType(BANKS[0]), up_dtype=DType(BANKS[1]), down_dtype=DType(BANKS[2]))

    # ---- device-resident timing: K steps recorded once, replayed (the reference replays a recorded decode
    # step the same way); warm-up runs the same steps un-recorded -----------------------------------
    for s in range(W):
        be.moe_ffn(op_for(s))
    be.sync()
    # distinct experts per step (for the byte count): routing of the first pass over the pool
    u_list = []
    for s in range(min(K, SETS * 4)):
        be.moe_ffn(op_for(s))
        be.sync()
        u_list.append(distinct_experts(ids_t.cpu().numpy()))
    mean_u = sum(u_list) / len(u_list)

    def record(n, stages=0):
        be.graph_begin()
        for s in range(n):
            be.moe_ffn(op_for(s, stages=stages))
        return be.graph_end()

    chunk = min(K, 512)
    plan = record(chunk)
    tail = record(K % chunk) if K % chunk else None
    be.execute(plan)
    be.sync()

    def k_steps():
        for _ in range(K // chunk):
            be.execute(plan)
        if tail is not None:
            be.execute(tail)

    sampler = ClockSampler(env.local)
    time.sleep(0.25)
    launches0 = be.launch_count()
    repeats = max(args.repeats, 1)
    ms, all_ms = timed_repeats(env, k_steps, repeats)
    launches = be.launch_count() - launches0
    # keep the GPU busy a little longer so the sampler sees clocks under load
    t_end = time.time() + 0.6
    while time.time() < t_end:
        be.execute(plan)
        be.sync()
    clocks = sampler.stop()

    # ---- the step's three kernels, each replayed alone (stage masks: 1 router + top-k, 2 gate/up, 4 down) ----
    kernel_us = {}
    n_k = 200
    # from n_expert / n_used rows on, the small-m path runs its expert-major kernels (the library's own rule)
    em = banks_tuned() and N_EXPERT <= R * N_USED and R * N_USED * 8 < N_EXPERT * 88
    router = "k_router_mid" if 8 < R <= 64 else "k_router_small"  # (beyond 64 rows: the batched router's three kernels)
    names = (router, "k_em_bucket + k_em_gateup", "k_em_down + k_em_combine") if em else \
            (router, "k_decode_gateup", "k_decode_down") if banks_tuned() else \
            (router, "k_anyfmt_gateup", "k_anyfmt_down")
    for name, mask in zip(names, (1, 2, 4)):
        for s in range(SETS):
            be.moe_ffn(op_for(s, stages=mask))
        be.sync()
        kplan = record(n_k, stages=mask)  # eager launches are host-bound at this size
        be.execute(kplan)
        be.sync()
        t, _ = timed_repeats(env, lambda: be.execute(kplan), 5)
        kernel_us[name] = t * 1e3 / n_k

    # ---- end to end through the C ABI with host buffers -------------------------------------------
    x_host = torch.randn(X_POOL, R, NE).pin_memory()
    out_host = torch.empty(R, NE).pin_memory()
    x_in_t = torch.empty(R, NE, device=dev)
    x_in = be.wrap_tensor(x_in_t)
    nbytes = R * NE * 4
    e2e_steps = max(min(K, 2000), 200)
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
    for i in range(SETS):
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
        be.execute(plans[s % SETS])
        be.sync()

    for s in range(W):
        e2e_step(s)
    env.barrier()
    t0 = time.perf_counter()
    for s in range(e2e_steps):
        e2e_step(s)
    torch.cuda.synchronize()
    launch_s = time.perf_counter() - t0  # one plan launch and one stream wait per step
    launch_steps = e2e_steps
    env.barrier()

    # The same steps as a host-paced plan: PACED steps recorded once and launched once; the host writes a
    # step's rows into the pinned staging buffer, rings the step's ticket and waits for the step's signal
    # (infr_cuda_host_step), so a token costs no launch and no stream wait.  Each step's fetch of the rows
    # (host to device) and the result written into pinned host memory (device to host) are inside the
    # timed region, as are the plan launches and the resets between them.
    PACED = 200
    e2e_steps = (e2e_steps + PACED - 1) // PACED * PACED
    be.graph_begin()
    for s in range(PACED):
        be.upload_ptr_gated(x_in, stage_ptr, nbytes, s + 1)
        if host_dst is not None:
            be.moe_ffn(dataclasses.replace(op_for(s, xbuf=x_in), dst=host_dst))
        else:
            be.moe_ffn(op_for(s, xbuf=x_in))
            be.download_ptr_async(dst, out_host.data_ptr(), nbytes)
        be.host_signal(s + 1)
    paced = be.graph_end()

    # the timed rounds go through one C call per round (infr_cuda_host_steps: per step rows in, ticket, wait);
    # a step's result is in pinned host memory (out_host) when its wait returns
    row_ptrs = [x_ptrs[s % X_POOL] for s in range(PACED)]

    def paced_round(check=False):
        be.host_reset()
        be.execute(paced)
        if check:
            for s in range(PACED):
                be.host_step(s + 1, stage_ptr, x_ptrs[s % X_POOL], nbytes)
                if s < 4:
                    want = paced_want[s]
                    paced_err[0] = max(paced_err[0], float((out_host - want).abs().max() / want.abs().max()))
        else:
            be.host_steps(1, stage_ptr, row_ptrs, nbytes)

    # the first steps of a round against the same steps launched one by one (same kernels: equal bits)
    paced_want, paced_err = [], [0.0]
    for s in range(4):
        memmove(stage_ptr, x_ptrs[s % X_POOL], nbytes)
        be.execute(plans[s % SETS])
        be.sync()
        paced_want.append(out_host.clone())
    paced_round(check=True)
    be.sync()
    env.barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps // PACED):
        paced_round()
    be.sync()
    e2e_s = time.perf_counter() - t0
    env.barrier()
    ms, e2e_s, launch_s = env.max_over_ranks(ms, e2e_s, launch_s)

    # ---- the other two halves of the metric --------------------------------------------------------
    sub = {}
    if subrecords:
        sub["stack"] = [measure_stack(env, layers[:40], r, 30 if r == 1 else 8, 3, with_e2e=False) for r in (1, 32)]
        sub["prefill"] = measure_prefill(env, 4096, False, 20, 3, with_e2e=False)

    if rank == 0:
        peaks, peak_kind = measured_peaks()
        tok_s = world * R * K / (ms * 1e-3)
        step_us = ms * 1e3 / K
        active_bytes = (mean_u + 1) * EXPERT_BYTES  # routed experts actually touched + the shared expert
        layer_gbs = active_bytes / (step_us * 1e-6) / 1e9
        kbytes = dict(zip(names, (N_EXPERT * NE * 4 + R * NE * 4, (mean_u + 1) * 2 * N_FF * Q4K_ROW, (mean_u + 1) * NE * Q6K_ROW)))
        kernels = [{"name": n, "us_alone": kernel_us[n], "algorithmic_bytes": kbytes[n],
                    "gbs_alone": kbytes[n] / (kernel_us[n] * 1e-6) / 1e9, "hbm_frac_alone": kbytes[n] / (kernel_us[n] * 1e-6) / 1e9 / peaks["hbm_gbs"],
                    "traffic": NCU_TRAFFIC_R1.get(n) if R == 1 and BANKS == (12, 12, 14) else None} for n in kernel_us]
        line = {
            "metric": "moe_layer_decode_tok_per_s", "value": tok_s, "unit": "tok/s", "n_gpus": world, "steps": K,
            "warmup": W, "repeats": repeats, "ms_per_step": ms / K, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": DTYPE, "data": "synthetic", "config": workload_config(R, SETS),
            "timing": f"median of {repeats} replays of the recorded {K} steps (this rank's replays: min {min(all_ms) / K * 1e3:.2f}, "
                      f"max {max(all_ms) / K * 1e3:.2f} us per step), max over ranks",
            "active_expert_gbs": layer_gbs * world,
            "roofline": {"bound": "hbm", "kernel": "layer step (router + gate/up + down)", "achieved": layer_gbs, "peak": peaks["hbm_gbs"],
                         "unit": "GB/s", "frac": layer_gbs / peaks["hbm_gbs"], "peak_kind": peak_kind, "us_per_step": step_us,
                         "algorithmic_bytes": active_bytes, "distinct_routed_experts": mean_u,
                         "traffic": sum(NCU_TRAFFIC_R1.values()) if R == 1 and BANKS == (12, 12, 14) else None, "kernels": kernels},
            "e2e": {"value": world * R * e2e_steps / e2e_s, "unit": "tok/s", "h2d_bytes_per_step": nbytes,
                    "d2h_bytes_per_step": nbytes, "steps": e2e_steps, "us_per_step": e2e_s / e2e_steps * 1e6,
                    "max_rel_diff_from_launch_per_step": paced_err[0],
                    "mode": f"host-paced plan: {PACED} steps recorded once, each released by a ticket in pinned host memory "
                            "(infr_cuda_host_steps: per step rows in, ticket, wait; the result is in pinned host memory when the wait returns); "
                            "plan launches and resets inside the timed region",
                    "launch_per_step": {"value": world * R * launch_steps / launch_s, "unit": "tok/s", "us_per_step": launch_s / launch_steps * 1e6,
                                        "mode": "one recorded plan launched and one stream wait per step"}},
            "gpu_launches": launches, "clocks": clocks, **sub,
        }
        if world == 1 and not args.no_cpu_baseline:
            cpu_steps = 400
            toks, sec_per_step, cores = time_cpu(R, cpu_steps, 3)
            line["cpu_baseline"] = {"value": toks, "unit": "tok/s", "cores": cores, "kind": "port",
                                    "sample": f"{cpu_steps} steps of the same layer shape at {R} stream(s), 2 weight sets, all host threads"}
        print(json.dumps(line))
    env.close()


def run_stack(args):
    from moe4all_b200.devgen import DeviceLayer
    env = Env()
    R, K, W = args.streams, args.steps, max(args.warmup, 3)
    layers = [DeviceLayer(env.be, 5000 * (env.rank + 1) + i, NE, N_EXPERT, N_FF, sh_ff=SH_FF, device=env.dev) for i in range(40)]
    sampler = ClockSampler(env.local)
    rec = measure_stack(env, layers, R, K, W)
    clocks = sampler.stop()
    if env.rank == 0:
        peaks, kind = measured_peaks()
        print(json.dumps({
            "metric": "moe_stack_decode_tok_per_s", "value": rec["tok_per_s"], "unit": "tok/s", "n_gpus": env.world,
            "steps": K, "warmup": W, "ms_per_step": rec["ms_per_step"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": DTYPE, "data": "synthetic", "config": stack_config(R),
            "active_expert_gbs": env.world * rec["active_expert_gbs"],
            "roofline": {"bound": "hbm", "kernel": "whole step", "achieved": rec["active_expert_gbs"], "peak": peaks["hbm_gbs"],
                         "unit": "GB/s", "frac": rec["active_expert_gbs"] / peaks["hbm_gbs"], "peak_kind": kind, "traffic": None},
            "e2e": rec["e2e"], "gpu_launches": rec["gpu_launches"], "clocks": clocks}))
    env.close()


def run_prefill(args):
    env = Env()
    deepseek = args.shape == "deepseek"
    T, K, W = args.tokens or (8192 if deepseek else 4096), args.steps, max(args.warmup, 3)
    sampler = ClockSampler(env.local)
    rec = measure_prefill(env, T, deepseek, K, W)
    clocks = sampler.stop()
    if env.rank == 0:
        peaks, kind = measured_peaks()
        extra = {k: rec[k] for k in ("ep_phases_ms", "band_experts_ms_per_rank", "ep_parity_rel") if k in rec}
        print(json.dumps({
            "metric": "moe_prefill_routed_tflops", "value": rec["routed_tflops"], "unit": "TFLOP/s", "n_gpus": env.world, "steps": K,
            "warmup": W, "ms_per_step": rec["ms_per_step"], "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": DTYPE, "data": "synthetic", "tokens_per_s": rec["tokens_per_s"], "config": prefill_config(T, deepseek, env.world),
            "roofline": {"bound": "tensor", "kernel": "whole step (router + permute + grouped GEMMs + combine)", "achieved": rec["routed_tflops"],
                         "peak": peaks["bf16_tflops"] * env.world, "unit": "TFLOP/s", "frac": rec["routed_tflops"] / (peaks["bf16_tflops"] * env.world),
                         "peak_kind": kind, "traffic": None},
            "e2e": rec["e2e"], "gpu_launches": rec["gpu_launches"], "clocks": clocks, **extra}))
    env.close()


def main():
    args = parse_args()
    set_banks(args.banks)
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
