#!/usr/bin/env python
"""GPTQ layers/sec on the DeepSeek-V3 routed-expert gate_proj shape (2048 x 7168, 4 bit, g128).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]
    python bench.py --single-layer --steps 1        (small untimed case for profiler captures)

One process per GPU (torchrun sets RANK/LOCAL_RANK/WORLD_SIZE for N > 1).  Routed experts
are expert-parallel: every rank quantizes its own experts and nothing crosses NVLink, so the
job is weak-scaled and `value` is (layers all ranks quantized) / (max-over-ranks time).

A step is one `GPTQ.quantize(4)` call on one expert's gate_proj whose Hessian is already
accumulated on the device: pre-step, scales, Hessian-inverse factor, column sweep, codes out.
Steps rotate over distinct experts (weight 29 MB + Hessian 205 MB each, larger than L2).

Printed JSON (one line, rank 0):
  value      layers/s with inputs resident in HBM
  e2e        layers/s through the public handle with HOST buffers: weight and calibration
             activations copied from pinned memory, Hessian accumulated, layer quantized,
             codes and scales copied back, every step
  roofline   the kernel that takes the largest share of a step, timed with CUDA events on
             its launching stream by the library's profiling hooks in a separate pass
  cpu_baseline  the CPU oracle (a port of the reference's torch path) on this box's cores
`--impl reference` times that CPU path alone, as the reference arm.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

R, C, TOKENS, GROUP, BITS = 2048, 7168, 4096, 128, 4
WORKLOAD = "deepseek_v3_routed_expert_gate_proj_2048x7168_bf16_g128 (one rank's expert shard, Hessian resident)"
METRIC = "GPTQ layers/sec (2048x7168, 4b g128)"


def _peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return dict(hbm=p["hbm_gbs"], tensor_burst=p["bf16_tflops"], tensor_sustained=p["bf16_tflops_sustained"],
                    source="measured")
    return dict(hbm=6650.0, tensor_burst=1590.0, tensor_sustained=1400.0, source="fallback")


class ClockSampler:
    """SM clock and throttle reasons of one GPU while the timed region runs, read through NVML
    (the source nvidia-smi prints) from a thread of this process.  NVML is initialised when the
    sampler is built, long before the timed region: starting nvidia-smi at that moment instead
    stalled the GPU's launches for up to half a second now and then."""

    REASONS = {0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown"}

    def __init__(self, index: int, period_s: float = 0.02):
        import threading
        self.result = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        self.samples, self.recording, self.period = [], False, period_s
        self.nvml = self.handle = None
        try:
            import pynvml
            pynvml.nvmlInit()
            props = torch.cuda.get_device_properties(index)
            try:
                self.handle = pynvml.nvmlDeviceGetHandleByUUID(("GPU-" + str(props.uuid)).encode())
            except Exception:
                self.handle = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.nvml = pynvml
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM))
        except Exception:
            self.nvml = None
            return
        self._stop = threading.Event()
        self.thread = threading.Thread(target=self._loop, daemon=True)
        self.thread.start()

    def _reasons(self) -> int:
        fn = getattr(self.nvml, "nvmlDeviceGetCurrentClocksEventReasons", None) or \
            self.nvml.nvmlDeviceGetCurrentClocksThrottleReasons
        return int(fn(self.handle))

    def _loop(self):
        while not self._stop.is_set():
            if self.recording:
                try:
                    self.samples.append((float(self.nvml.nvmlDeviceGetClockInfo(self.handle, self.nvml.NVML_CLOCK_SM)),
                                         self._reasons()))
                except Exception:
                    pass
            self._stop.wait(self.period)

    def __enter__(self):
        self.recording = True          # samples add up over several timed stretches
        return self

    def __exit__(self, *exc):
        self.recording = False
        if self.nvml is None or not self.samples:
            return
        mask = 0
        for _, r in self.samples:
            mask |= r
        self.result = {"sm_mhz": statistics.median(c for c, _ in self.samples), "sm_max_mhz": self.max_mhz,
                       "reasons": sorted(n for bit, n in self.REASONS.items() if mask & bit), "samples": len(self.samples)}

    def close(self):
        if self.nvml is not None:
            self._stop.set()
            self.thread.join(timeout=1)


def _dist():
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    return world, rank, local


# ---------------------------------------------------------------------------- reference arm / CPU baseline
def cpu_layers_per_s(steps: int, warmup: int, threads: int, dtype=torch.bfloat16):
    """The oracle's GPTQ.quantize on one 2048 x 7168 layer per step, Hessian pre-accumulated."""
    from moe_quant_b200 import synthetic
    from oracle import gptq_oracle as O

    torch.set_num_threads(threads)
    W = synthetic.layer_weight(R, C, 0, dtype)
    X = synthetic.activations(TOKENS, C, 0, dtype)
    t0 = time.perf_counter()
    H, _ = O.hessian_update(None, 0, X)
    t_h = time.perf_counter() - t0
    times = []
    for i in range(warmup + steps):
        Hc = H.clone()
        t0 = time.perf_counter()
        O.quantize_layer(W, Hc, bits=BITS, group_size=GROUP, rel_damp=1e-2, block_size=128)
        dt = time.perf_counter() - t0
        if i >= warmup:
            times.append(dt)
    total = sum(times)
    return steps / total, total / steps * 1e3, 2.0 * TOKENS * C * C / t_h / 1e12


def run_reference(args):
    world, rank, _ = _dist()
    if rank != 0:
        return
    cores = os.cpu_count() or 1
    steps, warmup = args.steps, args.warmup
    value, ms, h_tflops = cpu_layers_per_s(steps, warmup, cores)
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "layers/s", "n_gpus": args.gpus, "steps": steps,
        "warmup": warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "sample": "one full 2048x7168 layer per step, Hessian from 4096 tokens"},
        "cpu_baseline": {"value": value, "unit": "layers/s", "cores": cores, "kind": "port",
                         "sample": f"{steps} full layers after {warmup} warm-up, torch CPU oracle, {cores} threads"},
        "hessian_tflops_2nc2_cpu": h_tflops,
        "e2e": {"value": value, "unit": "layers/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


# ---------------------------------------------------------------------------- B200 arm
def run_b200(args):
    import torch.distributed as dist
    import torch.nn as nn

    from moe_quant_b200 import GPTQ, _lib, ops, quantize_many, synthetic

    world, rank, local = _dist()
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; this engine has no CPU path")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    steps, warmup = args.steps, max(args.warmup, 3)
    clocks = ClockSampler(local)         # NVML comes up here, not beside the timed region
    n_experts = 4
    seed = 1234 + 100 * rank

    # ---- this rank's experts: weights and Hessians resident in HBM (set-up, untimed)
    counts = synthetic.ragged_expert_counts(32 * 1024, 256, 8, seed)   # ragged top-8 routing of 32k tokens
    weights, hessians, tokens = [], [], []
    for e in range(n_experts):
        W = synthetic.layer_weight(R, C, seed + e, torch.bfloat16).to(dev)
        m = int(counts[(rank * n_experts + e) % 256].clamp(min=256, max=4 * TOKENS))
        g = torch.Generator(device=dev).manual_seed(seed + e)
        chan = torch.exp(torch.randn(C, generator=g, device=dev))
        X = (torch.randn(m, C, generator=g, device=dev) * chan).to(torch.bfloat16)
        H = torch.zeros(C, C, dtype=torch.float32, device=dev)
        ops.hessian_accum(H, X, 0.0, 2.0 / m)
        weights.append(W)
        hessians.append(H)
        tokens.append(m)
        del X

    def make_handles(n):
        hs = []
        for i in range(n):
            e = i % n_experts
            layer = nn.Linear(C, R, bias=False, dtype=torch.bfloat16, device="meta")
            layer.weight = nn.Parameter(weights[e], requires_grad=False)
            h = GPTQ(layer, GROUP, True, 1e-2, 128)
            h.H = hessians[e].clone()
            h.num_samples = tokens[e]
            hs.append(h)
        return hs

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- timed region: K quantize() calls, issued round-robin on `streams` CUDA streams
    # (independent experts: their kernel chains overlap on the GPU)
    n_streams = max(1, args.streams)
    # The warm-up is a whole pass of the same length with its results kept, then dropped: every
    # stream of the pool gets its workspace, and the caching allocator's per-stream pools hold
    # every block the timed pass will ask for.  A cudaMalloc inside the timed region goes
    # through the driver's global lock, which other jobs on a shared host can hold for tens of
    # milliseconds at a time.
    # Every step needs its own copy of a Hessian (quantize damps it in place) and keeps its
    # results: about 225 MB per step.  A step count that would not fit in memory is timed in
    # chunks (each bracketed by barrier + synchronize, their device times added up); the default
    # and anything up to a few hundred steps is one chunk.
    free_bytes, _total = torch.cuda.mem_get_info(dev)
    chunk = max(n_streams, min(steps, int(0.6 * free_bytes / 225e6)))
    warmup = max(warmup, min(steps, chunk))
    pre = make_handles(min(warmup, chunk))
    pre_results = quantize_many(pre, BITS, streams=n_streams)
    barrier()
    del pre, pre_results
    launches0 = _lib.lib().mq_launch_count()
    ms_total, done, issues = 0.0, 0, 0
    while done < steps:
        n = min(chunk, steps - done)
        handles = make_handles(n)
        barrier()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with clocks:
            ev0.record()
            results = quantize_many(handles, BITS, streams=n_streams)
            ev1.record()
            barrier()
        ms_total += ev0.elapsed_time(ev1)
        issues += sum(h.has_hessian_issues() for h in handles)
        done += n
        del handles, results
    clocks.close()
    launches = _lib.lib().mq_launch_count() - launches0
    steps_aux = min(steps, 48)             # the secondary rates below are measured on at most 48 steps
    # the same K calls one after the other on one stream (what a plain `for handle: quantize` loop gets)
    seq_pre = make_handles(steps_aux)      # same untimed pass first, for the same reason
    seq_pre_results = [h.quantize(BITS) for h in seq_pre]
    barrier()
    del seq_pre, seq_pre_results
    seq_handles = make_handles(steps_aux)
    barrier()
    s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s0.record()
    seq_results = [h.quantize(BITS) for h in seq_handles]
    s1.record()
    barrier()
    ms_single = s0.elapsed_time(s1)
    del seq_handles, seq_results
    fault = _lib.engine_fault()

    t = torch.tensor([ms_total], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_max = float(t.item())
    value = world * steps / (ms_max / 1e3)

    # ---- per-kernel pass (same work, events around every launch of the hot kernels), on one stream
    # directly after the one-stream pass: the library then sizes its grids as for a single caller
    prof_handles = make_handles(min(steps, 4))
    torch.cuda.synchronize()
    _lib.profile_begin()
    for h in prof_handles:
        h.quantize(BITS)
    prof = _lib.profile_end()
    del prof_handles
    peaks = _peaks()
    kinds = {k: v for k, v in prof.items() if v["launches"]}
    top = max(kinds, key=lambda k: kinds[k]["ms"]) if kinds else None
    roofline, shares = None, {}
    if top:
        tot = sum(v["ms"] for v in kinds.values())
        shares = {k: round(v["ms"] / tot, 4) for k, v in kinds.items()}
        v = kinds[top]
        if top in ("umma_gemm", "simt_gemm"):
            secs = v["ms"] / 1e3
            products = 6.0 if top == "umma_gemm" else 1.0     # bf16 products per fp32 product with three planes
            achieved = v["work"] * products / secs / 1e12
            # DRAM bytes per 128x128 output tile of a rank-128 update from the committed ncu capture
            # (141.1 MB for 1485 tiles, profiles/umma_panel_kernel_trailing_update_7168.md); traffic
            # grows with the tile count, so the average launch is scaled by its tiles
            tiles_per_launch = v["work2"] / v["launches"] / (2.0 * 128 * 128 * 128 * products)
            roofline = {"kernel": top, "bound": "tensor", "achieved": achieved, "peak": peaks["tensor_sustained"],
                        "unit": "TFLOP/s", "frac": achieved / peaks["tensor_sustained"],
                        "traffic": 95.0e3 * tiles_per_launch if top == "umma_gemm" else None,
                        "traffic_note": "bytes per average launch, scaled by tiles from an ncu capture of two large launches",
                        "fp32_equivalent_tflops": v["work"] / secs / 1e12,
                        "padded_tflops": v["work2"] / secs / 1e12,
                        "note": "algorithmic work of the split-bf16 GEMM: 2MNK on the kept tiles x 6 bf16 tensor products "
                                "per fp32 product (3 planes); fp32_equivalent_tflops counts each fp32 product once",
                        "avg_launch_us": v["ms"] / v["launches"] * 1e3, "launches_per_layer": v["launches"] / min(steps, 4),
                        "peak_source": peaks["source"] + " (sustained bf16)"}
        else:
            achieved = v["work"] / (v["ms"] / 1e3) / 1e9
            roofline = {"kernel": top, "bound": "hbm", "achieved": achieved, "peak": peaks["hbm"], "unit": "GB/s",
                        "frac": achieved / peaks["hbm"], "traffic": None, "avg_launch_us": v["ms"] / v["launches"] * 1e3,
                        "peak_source": peaks["source"]}

    # ---- gate_proj + up_proj of an expert share their input, hence their Hessian: quantized as a
    # tied pair they share one factorisation (quant.py --tie_gptq_handles; the reference factors twice)
    from moe_quant_b200 import quantize_tied
    n_pairs = max(2, steps_aux // 4)
    pair_pool = [torch.cuda.Stream(device=dev) for _ in range(min(n_streams, n_pairs))]

    def make_pairs(n):
        out = []
        for i in range(n):
            gate = make_handles(1)[0]
            gate.layer.weight = nn.Parameter(weights[i % n_experts], requires_grad=False)
            gate.H = hessians[i % n_experts].clone()
            up_layer = nn.Linear(C, R, bias=False, dtype=torch.bfloat16, device="meta")
            up_layer.weight = nn.Parameter(weights[(i + 1) % n_experts], requires_grad=False)
            out.append((gate, GPTQ(up_layer, GROUP, True, 1e-2, 128, tied_gptq_handle=gate)))
        return out

    def run_pairs(pairs):
        cur = torch.cuda.current_stream(dev)
        for st in pair_pool:
            st.wait_stream(cur)
        res = []
        for i, (g_h, u_h) in enumerate(pairs):
            with torch.cuda.stream(pair_pool[i % len(pair_pool)]):
                res.append(quantize_tied([g_h, u_h], BITS))
        for st in pair_pool:
            cur.wait_stream(st)
        return res

    pre_pairs = run_pairs(make_pairs(n_pairs))
    barrier()
    del pre_pairs
    pairs = make_pairs(n_pairs)
    barrier()
    p0, p1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    p0.record()
    pair_results = run_pairs(pairs)
    p1.record()
    barrier()
    tied_layers_per_s = 2 * n_pairs / (p0.elapsed_time(p1) / 1e3)
    del pairs, pair_results
    # ---- Hessian accumulation rate (the second half of the headline metric)
    g = torch.Generator(device=dev).manual_seed(seed)
    X = (torch.randn(TOKENS, C, generator=g, device=dev)).to(torch.bfloat16)
    Hs = torch.zeros(C, C, dtype=torch.float32, device=dev)
    for _ in range(3):
        ops.hessian_accum(Hs, X, 0.5, 1.0 / TOKENS)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(10):
        ops.hessian_accum(Hs, X, 0.5, 1.0 / TOKENS)
    e1.record()
    torch.cuda.synchronize()
    h_ms = e0.elapsed_time(e1) / 10
    del Hs

    # ---- end to end through the handle with host buffers
    Wh = [w.cpu().pin_memory() for w in weights]
    Xh = synthetic.activations(TOKENS, C, seed, torch.bfloat16).pin_memory()
    # one set of pinned result buffers per stream: steps on different streams overlap
    pool = [torch.cuda.Stream(device=dev) for _ in range(n_streams)]
    q_host = [torch.empty(R, C, dtype=torch.uint8).pin_memory() for _ in pool]
    s_host = [torch.empty(R, C // GROUP, dtype=torch.bfloat16).pin_memory() for _ in pool]
    h2d = Wh[0].numel() * 2 + Xh.numel() * 2
    d2h = q_host[0].numel() + s_host[0].numel() * 2

    def e2e_step(i):
        k = i % n_streams
        W = Wh[i % n_experts].to(dev, non_blocking=True)
        Xd = Xh.to(dev, non_blocking=True)
        layer = nn.Linear(C, R, bias=False, dtype=torch.bfloat16, device="meta")
        layer.weight = nn.Parameter(W, requires_grad=False)
        h = GPTQ(layer, GROUP, True, 1e-2, 128)
        h.update(Xd)
        q, s, _z = h.quantize(BITS)
        q_host[k].copy_(q, non_blocking=True)
        s_host[k].copy_(s, non_blocking=True)
        h.reset()

    def e2e_run(n):
        cur = torch.cuda.current_stream(dev)
        for st in pool:
            st.wait_stream(cur)
        for i in range(n):
            with torch.cuda.stream(pool[i % n_streams]):
                e2e_step(i)
        for st in pool:
            cur.wait_stream(st)

    e2e_steps = steps_aux
    e2e_run(max(e2e_steps, n_streams))
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    e2e_run(e2e_steps)
    e1.record()
    barrier()
    t = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    e2e_value = world * e2e_steps / (float(t.item()) / 1e3)

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        cores = os.cpu_count() or 1
        v, ms, _ = cpu_layers_per_s(2, 1, cores)
        cpu = {"value": v, "unit": "layers/s", "cores": cores, "kind": "port",
               "sample": f"2 full 2048x7168 layers after 1 warm-up ({ms:.0f} ms each), torch CPU oracle, {cores} threads"}

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": "layers/s", "n_gpus": world, "steps": steps, "warmup": warmup,
            "ms_per_step": ms_max / steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic",
            "config": {"workload": WORKLOAD, "experts_rotated": n_experts, "tokens_per_expert": tokens,
                       "l2": "inputs larger than L2: each step touches a different expert's 29 MB weight and 205 MB Hessian",
                       "parallelism": f"ep{world}", "streams": n_streams,
                       "single_stream_layers_per_s_per_gpu": steps_aux / (ms_single / 1e3),
                       "tied_gate_up_layers_per_s_per_gpu": tied_layers_per_s, "math": "tcgen05 split-bf16 x3 planes (6 products), fp32 TMEM accumulation"},
            "roofline": roofline, "kernel_time_shares": shares,
            "cpu_baseline": cpu,
            "e2e": {"value": e2e_value, "unit": "layers/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
            "gpu_launches": int(launches),
            "clocks": clocks.result,
            "hessian_accum": {"ms": h_ms, "tflops_2NC2": 2.0 * TOKENS * C * C / h_ms / 1e9,
                              "tflops_unique": TOKENS * C * (C + 1) / h_ms / 1e9, "tokens": TOKENS, "dtype": "bf16"},
            "hessian_issues": int(issues), "engine_fault": int(fault),
        }
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def run_single_layer(args):
    """The small case for profiler captures: one Hessian from 4096 bf16 tokens, one 2048 x 7168
    layer quantized `--steps` times on one stream (about 1 GB on the device), no timing."""
    from moe_quant_b200 import _lib, ops
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    g = torch.Generator(device="cuda").manual_seed(0)
    W = (0.02 * torch.randn(R, C, generator=g, device=dev)).to(torch.bfloat16)
    chan = torch.exp(torch.randn(C, generator=g, device=dev))
    X = (torch.randn(TOKENS, C, generator=g, device=dev) * chan).to(torch.bfloat16)
    H = torch.zeros(C, C, device=dev)
    ops.hessian_accum(H, X, 0.0, 2.0 / TOKENS)
    for _ in range(max(1, args.steps)):
        ops.quantize_layer([W], H.clone(), GROUP, BITS, 1e-2)
    torch.cuda.synchronize()
    print(json.dumps({"single_layer": True, "launches": int(_lib.lib().mq_launch_count()),
                      "engine_fault": int(_lib.engine_fault())}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=48)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--streams", type=int, default=8, help="CUDA streams the independent layers are spread over")
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--single-layer", action="store_true",
                    help="run one Hessian accumulation and --steps layers untimed (profiler captures)")
    args = ap.parse_args()
    if args.single_layer:
        run_single_layer(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_b200(args)


if __name__ == "__main__":
    main()
