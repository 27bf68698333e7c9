#!/usr/bin/env python
"""Benchmark of the routed-MoE layer (synthetic data, seeded).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl native|reference]
                    [--workload prefill8k|prefill512|decode|latent8k]

One step = one pass of the layer over one batch.  Default workload: layer-major
prefill of 8192 tokens with a Zipf-skewed router bias (the configuration the
headline metric is quoted on); at N > 1 the same 8192 tokens are split over the
ranks and the 896 experts are sharded expert-parallel (strong scaling).  The
one-token decode figure and its HBM roofline are reported in the same line
under "decode".  Rank 0 prints one JSON line.

--impl reference times the CPU restatement of the reference's host path
(oracle/) on the host cores, on a bounded sample of the same workload.
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

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

from moonshine_b200 import synth  # noqa: E402

METRIC = "routed_moe_layer_tokens_per_s"
UNIT = "tokens/s"
L2_BYTES = 126 * 1024 * 1024


def workload_config(name: str, args=None):
    if name == "prefill8k":
        cfg, tokens = synth.baseline_config(bias_mode="zipf"), 8192
    elif name == "prefill512":
        cfg, tokens = synth.baseline_config(), 512
    elif name == "decode":
        cfg, tokens = synth.baseline_config(), 1
    elif name == "latent8k":
        # the reference's real layer shape: experts on a latent vector of width 3584,
        # SiTU, Q8-128 static projections with f32 scales, routing scale 1
        cfg = synth.baseline_config(bias_mode="zipf", expert_hidden=3072, activation=synth.ACT_SITU,
                                    q8_block=128, q8_scale_type=synth.Q8_F32, route_scale=1.0)
        cfg["latent"] = 3584
        tokens = 8192
    else:
        raise SystemExit(f"unknown workload {name}")
    if args is not None:                      # reduced cases for profiler captures only
        if args.experts:
            cfg["experts"] = args.experts
        if args.tokens:
            tokens = args.tokens
    return cfg, tokens


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return {"hbm_gbs": p["hbm_gbs"], "bf16_tflops": p["bf16_tflops"],
                "bf16_tflops_sustained": p.get("bf16_tflops_sustained", p["bf16_tflops"]),
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0,
            "source": "fallback"}


# ------------------------------------------------------------------ clocks
class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.rows = []
        self.proc = None
        self.gpu_index = gpu_index

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-lms", "100", "-i", str(self.gpu_index)],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, sm_max, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            if len(r) < 9:
                continue
            try:
                sm.append(float(r[1]))
                sm_max.append(float(r[2]))
            except ValueError:
                continue
            for name, cell in zip(names, r[5:9]):
                if cell.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": max(sm_max) if sm_max else None,
                "samples": len(sm), "reasons": sorted(reasons)}


# ------------------------------------------------------------- CPU baseline
def cpu_baseline(cfg: dict, tokens: int, seed: int = 0, budget_s: float = 12.0) -> dict:
    """Times the CPU oracle on a bounded sample of the workload and extrapolates
    to tokens/s.  Prefill: `sample_experts` whole experts with the number of rows
    an average expert receives, plus router / shared expert / combine on
    `sample_tokens` tokens.  Decode: one token's 16 experts in full."""
    from oracle import k3_oracle as o
    d, i, e, k, s = cfg["hidden"], cfg["expert_hidden"], cfg["experts"], cfg["top_k"], cfg["shared_hidden"]
    cores = o.thread_count()
    rows_per_expert = max(1, round(tokens * k / e)) if tokens > 1 else 1
    sample_experts = 2 if tokens > 1 else k
    key = lambda tag: synth.stream_key(seed, tag)
    per13, per13s = i * d // 2, i * d // 32
    per2, per2s = d * i // 2, d * i // 32
    xs = synth.activations(seed, max(rows_per_expert, 8), d)
    t_expert = 0.0
    done_routes = 0
    t0 = time.perf_counter()
    for ex in range(sample_experts):
        w1p = synth.bytes_uniform(key(synth.TAG_W1P), per13, first=ex * per13)
        w1s = synth.bytes_uniform(key(synth.TAG_W1S), per13s, cfg["scale_low"], cfg["scale_span"], first=ex * per13s)
        w3p = synth.bytes_uniform(key(synth.TAG_W3P), per13, first=ex * per13)
        w3s = synth.bytes_uniform(key(synth.TAG_W3S), per13s, cfg["scale_low"], cfg["scale_span"], first=ex * per13s)
        w2p = synth.bytes_uniform(key(synth.TAG_W2P), per2, first=ex * per2)
        w2s = synth.bytes_uniform(key(synth.TAG_W2S), per2s, cfg["scale_low"], cfg["scale_span"], first=ex * per2s)
        xr = xs[:rows_per_expert]
        t = time.perf_counter()
        g = o.mxfp4_gemm(w1p, w1s, xr, i, d)
        u = o.mxfp4_gemm(w3p, w3s, xr, i, d)
        a = o.activation(g, u, cfg["activation"], cfg["beta"], cfg["linear_beta"])
        o.mxfp4_gemm(w2p, w2s, a, d, i)
        t_expert += time.perf_counter() - t
        done_routes += rows_per_expert
        if time.perf_counter() - t0 > budget_s and ex >= 1:
            break
    per_route = t_expert / done_routes
    # router + top-k + shared expert + combine on a token sample
    sample_tokens = 1 if tokens == 1 else 32
    w = synth.make_layer(cfg, seed, experts=False)
    xt = synth.activations(seed, sample_tokens, d)
    t = time.perf_counter()
    logits = o.bf16_gemm(w["router_weight"], xt, e, d)
    ids, wts = o.router_topk(logits, w["router_bias"], k, cfg["route_scale"])
    o.group_routes(ids, e)
    if s:
        sg = o.q8_gemm(w["shared_gate_q"], w["shared_gate_s"], xt, s, d, cfg["q8_block"], cfg["q8_scale_type"])
        su = o.q8_gemm(w["shared_up_q"], w["shared_up_s"], xt, s, d, cfg["q8_block"], cfg["q8_scale_type"])
        sa = o.activation(sg, su, cfg["activation"], cfg["beta"], cfg["linear_beta"])
        so = o.q8_gemm(w["shared_down_q"], w["shared_down_s"], sa, d, s, cfg["q8_block"], cfg["q8_scale_type"])
    fake = np.zeros((sample_tokens * k, d), np.uint16)
    routed = o.weighted_sum(fake, wts, sample_tokens, k, d)
    if s:
        o.add(routed, so)
    per_token_rest = (time.perf_counter() - t) / sample_tokens
    per_token = per_route * k + per_token_rest
    return {"value": 1.0 / per_token, "unit": UNIT, "cores": cores, "kind": "port",
            "sample": (f"{done_routes // rows_per_expert} experts x {rows_per_expert} rows "
                       f"(gate, up, activation, down) + router/top-k/dispatch/shared/combine on "
                       f"{sample_tokens} tokens; per-token time = 16 x per-route + rest; extrapolated"),
            "seconds": round(time.perf_counter() - t0, 2)}


# ------------------------------------------------------------ reference arm
def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cfg, tokens = workload_config(args.workload, args)
    values = []
    for step in range(args.warmup + args.steps):
        r = cpu_baseline(cfg, tokens, budget_s=6.0)
        if step >= args.warmup:
            values.append(r)
    value = statistics.mean(v["value"] for v in values)
    last = values[-1]
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * tokens / value,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic",
        "config": {"workload": args.workload, "tokens": tokens, "experts": cfg["experts"],
                   "top_k": cfg["top_k"], "hidden": cfg["hidden"],
                   "expert_hidden": cfg["expert_hidden"]},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": last["cores"], "kind": "port",
                         "sample": last["sample"]},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "CPU restatement of the reference's host MoE path (the reference's HIP build "
                "cannot run here); throughput extrapolated from a bounded sample",
    }
    print(json.dumps(line))


# DRAM bytes per launch measured with ncu on these workloads (one-pass metrics,
# summary kept under profiles/): prefill = gate/up (28.81 GB) + down (11.73 GB)
# launches of the grouped expert phase; decode = the five kernels of one token.
PREFILL_TRAFFIC_BYTES = 40.54e9
DECODE_TRAFFIC_BYTES = 435.6e6


# --------------------------------------------------------------- native arm
def launches_per_step(tokens: int, shared: bool) -> int:
    """Kernels of this library one layer pass launches (baseline shapes)."""
    if tokens == 1:
        return 5                                   # front, gate/up, down (+ combine) + shared gate/up, shared down
    route, shared_k, dispatch, combine = 2, (5 if shared else 0), 3, 1
    experts = 1 + 3 + 2                            # row split, 3 gathers, gate/up and down GEMMs
    return route + shared_k + dispatch + experts + combine


def time_decode(layer, cfg, torch, iters: int = 40):
    """One-token decode with a cold L2: distinct tokens round-robin and a buffer
    larger than L2 rewritten between iterations; each iteration timed by its own
    pair of events on the launching stream."""
    d = cfg["hidden"]
    xs = torch.from_numpy(synth.activations(7, 8, d).view(np.int16)).to(layer.device).view(torch.bfloat16)
    flush = torch.empty(2 * L2_BYTES, dtype=torch.uint8, device=layer.device)
    for i in range(5):
        layer.forward(xs[i % 8:i % 8 + 1])
    # every iteration has its own pair of events; the host does not wait inside the
    # loop, so launch overhead overlaps the previous iteration's flush and layer
    starts = [torch.cuda.Event(enable_timing=True) for _ in range(iters)]
    stops = [torch.cuda.Event(enable_timing=True) for _ in range(iters)]
    for i in range(iters):
        flush.fill_(i & 0xFF)
        starts[i].record()
        layer.forward(xs[i % 8:i % 8 + 1])
        stops[i].record()
    torch.cuda.synchronize()
    times = [a.elapsed_time(b) for a, b in zip(starts, stops)]
    ms = statistics.median(times)
    # per-kernel times from events the library records between its launches
    ph = layer.phase_times(xs[0:1], 10)
    kernels = {"front_ms": ph["router_ms"] + ph["shared_ms"], "gate_up_ms": ph["dispatch_ms"],
               "down_ms": ph["experts_ms"], "combine_ms": ph["combine_ms"],
               "note": "events between launches on the main stream; the shared expert runs beside them on a "
                       "side stream; front includes host launch latency after an idle device"}
    return ms, min(times), kernels


def run_latent(args, cfg, tokens, device, peaks, torch):
    """The latent-shape layer (k3_moe_latent_layer_forward): whole-step timing only."""
    from moonshine_b200.layer import LatentMoELayer
    latent = cfg.pop("latent")
    layer = LatentMoELayer(cfg, latent, seed=0, device=device, max_tokens=tokens)
    d, k, i, s, e = cfg["hidden"], cfg["top_k"], cfg["expert_hidden"], cfg["shared_hidden"], cfg["experts"]
    x = torch.from_numpy(synth.activations(0, tokens, d).view(np.int16).copy()).view(torch.bfloat16).to(device)
    for _ in range(max(args.warmup, 3)):
        layer.forward(x)
    torch.cuda.synchronize()
    sampler = ClockSampler(0)
    sampler.start()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(args.steps):
        layer.forward(x)
    stop.record()
    torch.cuda.synchronize()
    clocks = sampler.stop()
    ms = start.elapsed_time(stop) / args.steps
    flops = tokens * (k * 6 * i * latent + 4 * latent * d + 6 * s * d + 2 * e * d)
    achieved = flops / (ms * 1e-3) / 1e12
    print(json.dumps({
        "metric": METRIC, "value": tokens / (ms * 1e-3), "unit": UNIT, "n_gpus": 1, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": args.workload, "tokens": tokens, "experts": e, "top_k": k, "hidden": d,
                   "latent": latent, "expert_hidden": i, "shared_hidden": s, "router_bias": "zipf",
                   "l2": "inputs larger than L2"},
        "gpu_launches": (launches_per_step(tokens, bool(s)) + 4) * args.steps, "clocks": clocks,
        "roofline": {"bound": "tensor", "kernel": "whole layer pass", "achieved": achieved,
                     "peak": peaks["bf16_tflops_sustained"], "unit": "TFLOP/s",
                     "frac": achieved / peaks["bf16_tflops_sustained"], "traffic": None,
                     "peak_source": peaks["source"] + " bf16 sustained"},
        "e2e": None, "cpu_baseline": None}))


def run_native(args):
    import torch
    import torch.distributed as dist

    from moonshine_b200 import _native, ops
    from moonshine_b200.layer import MoELayer

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("launch with torch.distributed.run for --gpus > 1")
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: there is no CPU fallback for the native arm")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    _native.lib()                                   # fail loudly if the extension is missing
    if world > 1:
        dist.init_process_group("nccl", device_id=device)

    cfg, tokens = workload_config(args.workload, args)
    peaks = measured_peaks()
    d, k = cfg["hidden"], cfg["top_k"]
    flops = synth.prefill_flops_per_token(cfg)

    if "latent" in cfg:
        if world > 1:
            raise SystemExit("the latent workload runs on one GPU")
        return run_latent(args, cfg, tokens, device, peaks, torch)
    if world > 1:
        from moonshine_b200.ep import ExpertParallelLayer
        layer = ExpertParallelLayer(cfg, seed=0, device=device, tokens=tokens, pieces=args.ep_pieces)
        local_tokens = layer.local_tokens
    else:
        layer = MoELayer(cfg, None, seed=0, device=device, max_tokens=tokens)
        local_tokens = tokens
    x_host = torch.from_numpy(
        synth.activations(0, tokens, d)[rank * local_tokens:(rank + 1) * local_tokens].view(np.int16).copy()
    ).view(torch.bfloat16).pin_memory()
    x_dev = x_host.to(device)
    out_host = torch.empty_like(x_host).pin_memory()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup if args.lean else max(args.warmup, 3)):
        layer.forward(x_dev)
    barrier()

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    start.record()
    for _ in range(args.steps):
        layer.forward(x_dev)
    stop.record()
    barrier()
    ms_total = start.elapsed_time(stop)
    clocks = sampler.stop() if rank == 0 else None
    if world > 1:
        t = torch.tensor([ms_total], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_total = float(t.item())
    ms_step = ms_total / args.steps
    value = tokens / (ms_step * 1e-3)

    if args.lean:           # profiler capture: timed region only
        if rank == 0:
            print(json.dumps({"metric": METRIC, "value": value, "unit": UNIT, "ms_per_step": ms_step,
                              "config": {"workload": args.workload, "tokens": tokens,
                                         "experts": cfg["experts"]}, "lean": True}))
        if world > 1:
            dist.destroy_process_group()
        return

    # ---- end to end: pinned host input -> device -> layer -> pinned host output, every
    # step.  The three legs of consecutive steps overlap as in a serving loop: step i+1's
    # input is copied while step i computes and step i-1's output goes back; two buffers
    # per direction, ordering by events, all of it inside the timed region.
    copy_in, copy_out = torch.cuda.Stream(device), torch.cuda.Stream(device)
    main = torch.cuda.current_stream(device)
    x_in = [x_dev, torch.empty_like(x_dev)]
    out_hosts = [out_host, torch.empty_like(out_host).pin_memory()]
    in_ready = [torch.cuda.Event() for _ in range(args.steps)]
    computed = [torch.cuda.Event() for _ in range(args.steps)]
    returned = [torch.cuda.Event() for _ in range(args.steps)]
    barrier()
    start.record()
    copy_in.wait_stream(main)
    copy_out.wait_stream(main)
    for i in range(args.steps):
        with torch.cuda.stream(copy_in):
            if i >= 2:
                copy_in.wait_event(computed[i - 2])          # the buffer's previous reader is done
            x_in[i % 2].copy_(x_host, non_blocking=True)
            in_ready[i].record(copy_in)
        main.wait_event(in_ready[i])
        out = layer.forward(x_in[i % 2])
        computed[i].record(main)
        with torch.cuda.stream(copy_out):
            copy_out.wait_event(computed[i])
            if i >= 2:
                copy_out.wait_event(returned[i - 2])
            out.record_stream(copy_out)
            out_hosts[i % 2].copy_(out, non_blocking=True)
            returned[i].record(copy_out)
    main.wait_stream(copy_out)
    main.wait_stream(copy_in)
    stop.record()
    barrier()
    e2e_ms = start.elapsed_time(stop)
    if world > 1:
        t = torch.tensor([e2e_ms], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = float(t.item())
    e2e_value = tokens / (e2e_ms / args.steps * 1e-3)

    # ---- phase timing of the dominant kernel (grouped expert products), CUDA events on
    # the launching stream, same inputs, measured in this process after the timed region
    phases = layer.phase_times(x_dev, args.steps)
    experts_ms = phases["experts_ms"]
    if world > 1:
        t = torch.tensor([experts_ms], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        experts_ms = float(t.item())

    line = None
    if rank == 0:
        if tokens > 1:
            routed_flops = flops["routed"] * tokens / world     # per GPU when balanced
            achieved = routed_flops / (experts_ms * 1e-3) / 1e12
            weight_bytes = cfg["experts"] * (3 * cfg["hidden"] * cfg["expert_hidden"] // 2 * 17 // 16) / world
            roofline = {"bound": "tensor", "kernel": "grouped expert products (gate+up+act, down)",
                        "achieved": achieved, "peak": peaks["bf16_tflops_sustained"],
                        "unit": "TFLOP/s", "frac": achieved / peaks["bf16_tflops_sustained"],
                        "traffic": PREFILL_TRAFFIC_BYTES if args.workload == "prefill8k" and world == 1 else None,
                        "traffic_note": "DRAM read+write of the two grouped GEMM launches, ncu one-pass capture "
                                        "of this workload (summary under profiles/); algorithmic 26.2 GB",
                        "peak_source": peaks["source"] + " bf16 sustained",
                        "launch_ms": experts_ms,
                        "hbm_floor_gbs": weight_bytes / (experts_ms * 1e-3) / 1e9}
        else:
            nbytes = synth.decode_bytes_per_token(cfg)
            achieved = nbytes / (ms_step * 1e-3) / 1e9
            roofline = {"bound": "hbm", "kernel": "one-token layer", "achieved": achieved,
                        "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": achieved / peaks["hbm_gbs"],
                        "traffic": DECODE_TRAFFIC_BYTES, "peak_source": peaks["source"]}
        decode = None
        if world == 1:
            dcfg = synth.baseline_config()
            dlayer = layer if args.workload != "prefill8k" else MoELayer(dcfg, None, seed=0, device=device)
            if args.workload == "prefill8k":
                del layer
                torch.cuda.empty_cache()
            dms, dmin, dkernels = time_decode(dlayer, dcfg, torch)
            nbytes = synth.decode_bytes_per_token(dcfg)
            gbs = nbytes / (dms * 1e-3) / 1e9
            decode = {"tokens_per_s": 1e3 / dms, "ms_per_token": dms, "ms_min": dmin,
                      "roofline": {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm_gbs"],
                                   "unit": "GB/s", "frac": gbs / peaks["hbm_gbs"],
                                   "bytes_per_token": nbytes, "traffic": DECODE_TRAFFIC_BYTES,
                                   "peak_source": peaks["source"]},
                      "kernels_ms": dkernels,
                      "l2": "flushed between iterations (252 MiB buffer rewritten), 8 tokens round-robin",
                      "gpu_launches_per_token": launches_per_step(1, bool(dcfg["shared_hidden"]))}
        cpu = cpu_baseline(cfg, tokens) if world == 1 else None
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": args.workload, "tokens": tokens, "experts": cfg["experts"],
                       "top_k": k, "hidden": d, "expert_hidden": cfg["expert_hidden"],
                       "shared_hidden": cfg["shared_hidden"], "router_bias": cfg["bias_mode"],
                       "parallelism": (f"ep{world}" + (f" x {args.ep_pieces} pipelined row ranges" if args.ep_pieces > 1 else ""))
                       if world > 1 else "single",
                       "l2": "inputs larger than L2 (expert weights 20.96 GB per pass)"},
            "e2e": {"value": e2e_value, "unit": UNIT,
                    "h2d_bytes_per_step": local_tokens * d * 2 * world,
                    "d2h_bytes_per_step": local_tokens * d * 2 * world},
            "gpu_launches": launches_per_step(tokens, bool(cfg["shared_hidden"])) * args.steps,
            "clocks": clocks, "roofline": roofline, "phases_ms": phases, "decode": decode,
            "cpu_baseline": cpu,
        }
        print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="native", choices=["native", "reference"])
    ap.add_argument("--workload", default="prefill8k", choices=["prefill8k", "prefill512", "decode", "latent8k"])
    ap.add_argument("--lean", action="store_true", help="timed region only (for profiler captures)")
    ap.add_argument("--ep-pieces", type=int, default=1,
                    help="expert-parallel runs: row ranges per pass pipelined against each other")
    ap.add_argument("--experts", type=int, default=0, help="override the expert count (profiler captures)")
    ap.add_argument("--tokens", type=int, default=0, help="override the token count (profiler captures)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_native(args)


if __name__ == "__main__":
    main()
