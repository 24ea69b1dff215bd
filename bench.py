#!/usr/bin/env python
"""GPTQ layers/sec on the DeepSeek-V3 routed-expert gate_proj shape (2048 x 7168, 4 bit, g128).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]
    python bench.py --workload {all,headline,down_proj,mla,moe_layer}
    python bench.py --single-layer --steps 1        (small untimed case for profiler captures)

One process per GPU (torchrun sets RANK/LOCAL_RANK/WORLD_SIZE for N > 1).  Routed experts
are expert-parallel: every rank quantizes its own experts and nothing crosses NVLink, so the
job is weak-scaled and `value` is (layers all ranks quantized) / (max-over-ranks time).

A step is one `GPTQ.quantize(4)` call on one expert's gate_proj whose Hessian is already
accumulated on the device: pre-step, scales, Hessian-inverse factor, column sweep, codes out.
Steps rotate over distinct experts (weight 29 MB + Hessian 205 MB each, larger than L2).  The
pass of K steps is timed `--reps` times (default 5); `value` is K / (median pass time).

Printed JSON (one line, rank 0):
  value      layers/s with inputs resident in HBM
  e2e        layers/s through the public handles with HOST buffers: per expert the calibration
             activations and the gate_proj / up_proj weights are copied from pinned memory, the
             Hessian is accumulated, both layers are quantized, codes and scales copied back
  roofline   the tensor-core GEMMs take the largest share of a step; of that family the 512-deep
             update (nine tenths of a layer's flop), timed with CUDA events on its launching stream
             by the library's measurement hooks in a separate pass; the family's other member
             follows in roofline.others and every family's share in kernel_time_shares
  parity     code agreement of one sampled step with the CPU oracle on a slice of rows (untimed)
  cpu_baseline  the CPU oracle (a port of the reference's torch path) on this box's cores
  extra      the other named workloads (`--workload all`, the default): expert down_proj with the
             group-size sweep and packing, the five MLA projections, one rank's shard of a whole
             MoE layer including its ragged Hessian accumulation
`--impl reference` times the CPU path alone, as the reference arm.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

R, C, TOKENS, GROUP, BITS = 2048, 7168, 4096, 128, 4
WORKLOAD = "deepseek_v3_routed_expert_gate_proj_2048x7168_bf16_g128 (one rank's expert shard, Hessian resident)"
METRIC = "GPTQ layers/sec (2048x7168, 4b g128)"
# DRAM traffic of one 128 x 128 output tile of a 512-deep three-plane update (ncu, profiles/)
DEEP_DRAM_BYTES_PER_TILE = 103.0e3
CONFIG = {"workload": WORKLOAD, "rows": R, "cols": C, "bits": BITS, "group_size": GROUP, "rel_damp": 1e-2,
          "weight_dtype": "bf16", "calibration_tokens_mean": TOKENS}


def _peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return dict(hbm=p["hbm_gbs"], tensor_burst=p["bf16_tflops"], tensor_sustained=p["bf16_tflops_sustained"],
                    source="measured")
    return dict(hbm=6650.0, tensor_burst=1590.0, tensor_sustained=1400.0, source="fallback")


def layer_flop(rows: int, cols: int, block: int = 128) -> float:
    """fp32-equivalent flop of one GPTQ.quantize in the reference's formulation: potrf + potri +
    potrf are replaced by their useful part 2/3 C^3, plus the lazy and in-block updates."""
    return 2.0 / 3.0 * cols ** 3 + float(rows) * cols * (cols - block) + float(rows) * cols * (block - 1)


class ClockSampler:
    """SM clock and throttle reasons of one GPU while the timed region runs, read through NVML
    (the source nvidia-smi prints) from a thread of this process.  NVML is initialised when the
    sampler is built, long before the timed region: starting nvidia-smi at that moment instead
    stalled the GPU's launches for up to half a second now and then."""

    REASONS = {0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown"}

    def __init__(self, index: int, period_s: float = 0.01):
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
        "config": dict(CONFIG),
        "cpu_baseline": {"value": value, "unit": "layers/s", "cores": cores, "kind": "port",
                         "sample": f"{steps} full 2048x7168 layers after {warmup} warm-up, Hessian from {TOKENS} tokens "
                                   f"accumulated beforehand, torch CPU port of the reference path, {cores} threads"},
        "hessian_tflops_2nc2_cpu": h_tflops,
        "e2e": {"value": value, "unit": "layers/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


# ---------------------------------------------------------------------------- B200 arm
class Ctx:
    pass


def _event_pair():
    return torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)


def _randn_acts(tokens, cols, dtype, seed, dev):
    g = torch.Generator(device=dev).manual_seed(seed)
    chan = torch.exp(torch.randn(cols, generator=g, device=dev))
    return (torch.randn(tokens, cols, generator=g, device=dev) * chan).to(dtype)


def _randn_weight(rows, cols, dtype, seed, dev):
    g = torch.Generator(device=dev).manual_seed(seed)
    return (0.02 * torch.randn(rows, cols, generator=g, device=dev)).to(dtype)


def _linear(W):
    import torch.nn as nn
    layer = nn.Linear(W.shape[1], W.shape[0], bias=False, dtype=W.dtype, device="meta")
    layer.weight = nn.Parameter(W, requires_grad=False)
    return layer


def run_b200(args):
    import torch.distributed as dist

    from moe_quant_b200 import GPTQ, _lib, ops, quantize_many, synthetic

    world, rank, local = _dist()
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; this engine has no CPU path")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    cx = Ctx()
    cx.world, cx.rank, cx.dev, cx.dist = world, rank, dev, dist
    cx.steps, cx.warmup, cx.reps = args.steps, max(args.warmup, 3), max(1, args.reps)
    cx.n_streams = max(1, args.streams)
    cx.clocks = ClockSampler(local)         # NVML comes up here, not beside the timed region
    cx.peaks = _peaks()
    cx.seed = 1234 + 100 * rank
    cx.no_cpu_baseline = args.no_cpu_baseline
    n_experts = 4

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    cx.barrier = barrier

    def max_over_ranks(ms):
        t = torch.tensor([ms], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    cx.max_over_ranks = max_over_ranks

    # ---- this rank's experts: weights and Hessians resident in HBM (set-up, untimed)
    counts = synthetic.ragged_expert_counts(32 * 1024, 256, 8, cx.seed)   # ragged top-8 routing of 32k tokens
    weights, hessians, tokens = [], [], []
    for e in range(n_experts):
        W = synthetic.layer_weight(R, C, cx.seed + e, torch.bfloat16).to(dev)
        m = int(counts[(rank * n_experts + e) % 256].clamp(min=256, max=4 * TOKENS))
        X = _randn_acts(m, C, torch.bfloat16, cx.seed + e, dev)
        H = torch.zeros(C, C, dtype=torch.float32, device=dev)
        ops.hessian_accum(H, X, 0.0, 2.0 / m)
        weights.append(W)
        hessians.append(H)
        tokens.append(m)
        del X
    cx.weights, cx.hessians, cx.tokens, cx.n_experts = weights, hessians, tokens, n_experts

    def make_handles(n):
        hs = []
        for i in range(n):
            e = i % n_experts
            h = GPTQ(_linear(weights[e]), GROUP, True, 1e-2, 128)
            h.H = hessians[e].clone()
            h.num_samples = tokens[e]
            hs.append(h)
        return hs

    cx.make_handles = make_handles
    want = args.workload
    line = {}
    if want in ("all", "headline"):
        line = headline(cx)
    extra = {}
    if want in ("all", "down_proj") and rank == 0:
        extra["down_proj"] = _guarded(wl_down_proj, cx)
    if want in ("all", "moe_layer"):
        res = _guarded(wl_moe_layer, cx)        # no collective inside: a failure on one rank cannot hang the others
        total = cx.max_over_ranks(float(res.get("layer_ms_local", 0.0)))
        if "error" not in res and total > 0:
            res["layer_ms_max_over_ranks"] = total
            res["layers_per_s_all_ranks"] = world * res["layers_per_rank"] / (total / 1e3)
        extra["moe_layer"] = res
    if want in ("all", "mla"):
        extra["mla"] = wl_mla(cx)                 # collectives inside: every rank must take part, no guard
    cx.clocks.close()
    if rank == 0:
        if not line:
            line = {"metric": METRIC, "value": None, "unit": "layers/s", "n_gpus": world, "config": dict(CONFIG)}
        line["extra"] = extra
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def _guarded(fn, cx):
    try:
        return fn(cx)
    except Exception as exc:  # noqa: BLE001 - an extra workload must not take the headline down with it
        torch.cuda.synchronize()
        return {"error": f"{type(exc).__name__}: {exc}"[:300]}


def headline(cx):
    import torch.nn as nn

    from moe_quant_b200 import GPTQ, _lib, ops, quantize_many, quantize_tied, synthetic
    from moe_quant_b200.gptq import compact_launches

    dev, world, rank = cx.dev, cx.world, cx.rank
    steps, n_streams, barrier = cx.steps, cx.n_streams, cx.barrier
    make_handles = cx.make_handles

    # ---- timed region: K quantize() calls, issued round-robin on `streams` CUDA streams
    # (independent experts: their kernel chains overlap on the GPU).
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
    pre = make_handles(min(max(cx.warmup, steps), chunk))
    pre_results = quantize_many(pre, BITS, streams=n_streams)
    barrier()
    del pre, pre_results

    def timed_pass():
        ms_total, done, issues = 0.0, 0, 0
        while done < steps:
            n = min(chunk, steps - done)
            handles = make_handles(n)
            barrier()
            ev0, ev1 = _event_pair()
            with cx.clocks:
                ev0.record()
                results = quantize_many(handles, BITS, streams=n_streams)
                ev1.record()
                barrier()
            ms_total += ev0.elapsed_time(ev1)
            issues += sum(h.has_hessian_issues() for h in handles)
            done += n
            del handles, results
        return cx.max_over_ranks(ms_total), issues

    launches0 = _lib.lib().mq_launch_count()
    passes, issues = [], 0
    for _ in range(cx.reps):
        ms, bad = timed_pass()
        passes.append(ms)
        issues += bad
    launches = (_lib.lib().mq_launch_count() - launches0) // cx.reps
    ms_med = statistics.median(passes)
    value = world * steps / (ms_med / 1e3)

    steps_aux = min(steps, 48)             # the secondary rates below are measured on at most 48 steps
    # the same K calls one after the other on one stream (what a plain `for handle: quantize` loop gets)
    seq_pre = make_handles(steps_aux)      # same untimed pass first, for the same reason
    seq_pre_results = [h.quantize(BITS) for h in seq_pre]
    barrier()
    del seq_pre, seq_pre_results
    seq_ms = []
    for _ in range(min(cx.reps, 3)):
        seq_handles = make_handles(steps_aux)
        barrier()
        s0, s1 = _event_pair()
        s0.record()
        seq_results = [h.quantize(BITS) for h in seq_handles]
        s1.record()
        barrier()
        seq_ms.append(s0.elapsed_time(s1))
        del seq_handles, seq_results
    ms_single = statistics.median(seq_ms)
    fault = _lib.engine_fault()

    # ---- per-kernel pass (same work, events around every launch of the hot kernels), on one stream
    # directly after the one-stream pass: the library then sizes its grids as for a single caller
    n_prof = min(steps, 4)
    prof_handles = make_handles(n_prof)
    torch.cuda.synchronize()
    _lib.profile_begin()
    for h in prof_handles:
        h.quantize(BITS)
    prof = _lib.profile_end()
    del prof_handles
    peaks = cx.peaks
    kinds = {k: v for k, v in prof.items() if v["launches"]}
    top = max(kinds, key=lambda k: kinds[k]["ms"]) if kinds else None
    roofline, shares, per_layer_us = None, {}, {}
    if top:
        tot = sum(v["ms"] for v in kinds.values())
        shares = {k: round(v["ms"] / tot, 4) for k, v in kinds.items()}
        per_layer_us = {k: round(v["ms"] / n_prof * 1e3, 1) for k, v in kinds.items()}
        # The tensor-core GEMMs (rank-128 updates inside a 512-column super-block: umma_gemm; the
        # 512-deep updates behind it: umma_deep) are one family; when it has the largest share of the
        # kernel time the roofline is that of its member with the most work, the deep update (nine
        # tenths of a layer's flop, and the largest single share of a step once several layers run
        # side by side and the latency-bound kernels overlap).  The other members follow in
        # roofline["others"].
        family = {k: kinds[k] for k in ("umma_gemm", "umma_deep") if k in kinds}
        fam_ms = sum(v["ms"] for v in family.values())
        if family and fam_ms >= max(v["ms"] for k, v in kinds.items() if k not in family):
            top = max(family, key=lambda k: family[k]["work"])
        v = kinds[top]

        def tensor_line(kind, v):
            secs = v["ms"] / 1e3
            products = 1.0 if kind == "simt_gemm" else 6.0     # bf16 products per fp32 product with three planes
            achieved = v["work"] * products / secs / 1e12
            return {"kernel": kind, "bound": "tensor", "achieved": achieved, "peak": peaks["tensor_sustained"],
                    "unit": "TFLOP/s", "frac": achieved / peaks["tensor_sustained"],
                    "fp32_equivalent_tflops": v["work"] / secs / 1e12, "padded_tflops": v["work2"] / secs / 1e12,
                    "avg_launch_us": v["ms"] / v["launches"] * 1e3, "launches_per_layer": v["launches"] / n_prof,
                    "share_of_kernel_time": round(v["ms"] / tot, 4)}

        if top in ("umma_gemm", "umma_deep", "simt_gemm"):
            roofline = tensor_line(top, v)
            products = 1.0 if top == "simt_gemm" else 6.0
            out_tiles = v["work2"] / v["launches"] / (2.0 * 128 * 128 * products)   # output tiles x k per launch
            if top == "umma_deep":
                # DRAM bytes per 128 x 128 output tile of a 512-deep update, from an ncu capture of the
                # 6656 x 6656 x 512 upper-triangle update (profiles/): the C tile once in, once out, and
                # the operand slabs that miss the L2
                roofline["traffic"] = DEEP_DRAM_BYTES_PER_TILE * out_tiles / 512.0
                roofline["traffic_source"] = ("scaled by output tiles from an ncu capture of one 512-deep update "
                                              "(profiles/umma_stream_kernel_far_update.md), not measured in this run")
            elif top == "umma_gemm":
                roofline["traffic"] = 95.0e3 * out_tiles / 128.0
                roofline["traffic_source"] = ("scaled from an ncu capture (95 KB of DRAM traffic per 128x128 tile of a "
                                              "rank-128 update), not measured in this run")
            else:
                roofline["traffic"] = None
            roofline["note"] = ("algorithmic work of the split-bf16 GEMM: 2MNK on the kept tiles x 6 bf16 tensor products per "
                                "fp32 product (3 planes); fp32_equivalent_tflops counts each fp32 product once; timed on one "
                                "stream with full grids; chosen as the member of the tensor-GEMM family with the most work")
            roofline["peak_source"] = peaks["source"] + " (sustained bf16)"
            roofline["others"] = [tensor_line(k, kv) for k, kv in family.items() if k != top]
        else:
            achieved = v["work"] / (v["ms"] / 1e3) / 1e9
            roofline = {"kernel": top, "bound": "hbm", "achieved": achieved, "peak": peaks["hbm"], "unit": "GB/s",
                        "frac": achieved / peaks["hbm"], "traffic": None, "avg_launch_us": v["ms"] / v["launches"] * 1e3,
                        "peak_source": peaks["source"]}

    # ---- gate_proj + up_proj of an expert share their input, hence their Hessian: quantized as a
    # tied pair they share one factorisation (quant.py --tie_gptq_handles; the reference factors twice)
    weights, hessians, n_experts = cx.weights, cx.hessians, cx.n_experts
    n_pairs = max(2, steps_aux // 4)
    pair_pool = [torch.cuda.Stream(device=dev) for _ in range(min(n_streams, n_pairs))]

    def make_pairs(n):
        out = []
        for i in range(n):
            gate = make_handles(1)[0]
            gate.layer.weight = nn.Parameter(weights[i % n_experts], requires_grad=False)
            gate.H = hessians[i % n_experts].clone()
            up = GPTQ(_linear(weights[(i + 1) % n_experts]), GROUP, True, 1e-2, 128, tied_gptq_handle=gate)
            out.append((gate, up))
        return out

    def run_pairs(pairs):
        # quantize_many groups each up_proj with the gate_proj it is tied to: one factorisation per pair
        return quantize_many([h for pair in pairs for h in pair], BITS, streams=len(pair_pool))

    pre_pairs = run_pairs(make_pairs(n_pairs))
    barrier()
    del pre_pairs
    pairs = make_pairs(n_pairs)
    barrier()
    p0, p1 = _event_pair()
    p0.record()
    pair_results = run_pairs(pairs)
    p1.record()
    barrier()
    tied_layers_per_s = 2 * n_pairs / (p0.elapsed_time(p1) / 1e3)
    del pairs, pair_results

    # ---- Hessian accumulation rate (the second half of the headline metric), 16-bit and fp32 activations
    hess = {}
    for name, dt in (("bf16", torch.bfloat16), ("fp32", torch.float32)):
        X = _randn_acts(TOKENS, C, dt, cx.seed, dev)
        Hs = torch.zeros(C, C, dtype=torch.float32, device=dev)
        for _ in range(3):
            ops.hessian_accum(Hs, X, 0.5, 1.0 / TOKENS)
        torch.cuda.synchronize()
        e0, e1 = _event_pair()
        n_rep = 10
        e0.record()
        for _ in range(n_rep):
            ops.hessian_accum(Hs, X, 0.5, 1.0 / TOKENS)
        e1.record()
        torch.cuda.synchronize()
        h_ms = e0.elapsed_time(e1) / n_rep
        hess[name] = {"ms": h_ms, "tflops_2NC2": 2.0 * TOKENS * C * C / h_ms / 1e9,
                      "tflops_unique": TOKENS * C * (C + 1) / h_ms / 1e9, "tokens": TOKENS,
                      "products_per_fp32_product": 1 if dt != torch.float32 else 6}
        del Hs, X

    # ---- end to end through the handles with host buffers.  A step is one layer; layers come in
    # gate_proj/up_proj pairs of one expert, which see the same activations: X is uploaded once per
    # expert, the Hessian accumulated once, both layers quantized with one factorisation.
    Wh = [w.cpu().pin_memory() for w in weights]
    Xh = synthetic.activations(TOKENS, C, cx.seed, torch.bfloat16).pin_memory()
    pool = [torch.cuda.Stream(device=dev) for _ in range(n_streams)]
    q_host = [[torch.empty(R, C, dtype=torch.uint8).pin_memory() for _ in range(2)] for _ in pool]
    s_host = [[torch.empty(R, C // GROUP, dtype=torch.bfloat16).pin_memory() for _ in range(2)] for _ in pool]
    h2d_pair = 2 * Wh[0].numel() * 2 + Xh.numel() * 2
    d2h_pair = 2 * (q_host[0][0].numel() + s_host[0][0].numel() * 2)

    def e2e_pair(i):
        k = i % n_streams
        Wg = Wh[i % n_experts].to(dev, non_blocking=True)
        Wu = Wh[(i + 1) % n_experts].to(dev, non_blocking=True)
        Xd = Xh.to(dev, non_blocking=True)
        gate = GPTQ(_linear(Wg), GROUP, True, 1e-2, 128)
        up = GPTQ(_linear(Wu), GROUP, True, 1e-2, 128, tied_gptq_handle=gate)
        gate.update(Xd)
        with compact_launches(gate, n_streams > 1):   # several pairs are in flight on the other streams
            pair_res = quantize_tied([gate, up], BITS)
        for j, (q, s, _z) in enumerate(pair_res):
            q_host[k][j].copy_(q, non_blocking=True)
            s_host[k][j].copy_(s, non_blocking=True)
        gate.reset()
        up.reset()

    def e2e_run(n):
        cur = torch.cuda.current_stream(dev)
        for st in pool:
            st.wait_stream(cur)
        for i in range(n):
            with torch.cuda.stream(pool[i % n_streams]):
                e2e_pair(i)
        for st in pool:
            cur.wait_stream(st)

    e2e_pairs = max(n_streams, steps_aux // 2)
    e2e_run(e2e_pairs)
    barrier()
    e2e_ms = []
    for _ in range(min(cx.reps, 3)):
        e0, e1 = _event_pair()
        e0.record()
        e2e_run(e2e_pairs)
        e1.record()
        barrier()
        e2e_ms.append(cx.max_over_ranks(e0.elapsed_time(e1)))
    e2e_value = world * 2 * e2e_pairs / (statistics.median(e2e_ms) / 1e3)
    # the host link by itself, every rank copying at once: the ceiling of any end-to-end rate
    big = torch.empty(512 << 20, dtype=torch.uint8).pin_memory()
    dst = torch.empty_like(big, device=dev)
    dst.copy_(big, non_blocking=True)
    barrier()
    c0, c1 = _event_pair()
    c0.record()
    for _ in range(4):
        dst.copy_(big, non_blocking=True)
    c1.record()
    barrier()
    h2d_gbs = 4 * big.numel() / (cx.max_over_ranks(c0.elapsed_time(c1)) / 1e3) / 1e9
    del big, dst

    parity = _guarded(parity_sample, cx) if rank == 0 else None
    cpu = None
    if rank == 0 and world == 1 and not cx_no_cpu(cx):
        cores = os.cpu_count() or 1
        v, ms, _ = cpu_layers_per_s(2, 1, cores)
        cpu = {"value": v, "unit": "layers/s", "cores": cores, "kind": "port",
               "sample": f"2 full 2048x7168 layers after 1 warm-up ({ms:.0f} ms each), torch CPU oracle, {cores} threads"}

    config = dict(CONFIG)
    config.update({"experts_rotated": n_experts, "tokens_per_expert": cx.tokens,
                   "l2": "inputs larger than L2: each step touches a different expert's 29 MB weight and 205 MB Hessian",
                   "parallelism": f"ep{world}", "streams": n_streams, "timed_passes": cx.reps,
                   "untimed_pass_before": "one full pass of K steps (allocator and workspaces warm), then W >= 3 honoured",
                   "single_stream_layers_per_s_per_gpu": steps_aux / (ms_single / 1e3),
                   "tied_gate_up_layers_per_s_per_gpu": tied_layers_per_s,
                   "e2e_step": "one layer of a gate_proj/up_proj pair: X uploaded once per expert, one factorisation per pair",
                   "math": "tcgen05 split-bf16 x3 planes (6 products), fp32 TMEM accumulation"})
    return {
        "metric": METRIC, "value": value, "unit": "layers/s", "n_gpus": world, "steps": steps, "warmup": cx.warmup,
        "ms_per_step": ms_med / steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic", "config": config,
        "passes_ms": [round(p, 3) for p in passes],
        "spread": (max(passes) - min(passes)) / ms_med,
        "roofline": roofline, "kernel_time_shares": shares, "kernel_us_per_layer_one_stream": per_layer_us,
        "parity": parity, "cpu_baseline": cpu,
        "e2e": {"value": e2e_value, "unit": "layers/s", "h2d_bytes_per_step": h2d_pair // 2, "d2h_bytes_per_step": d2h_pair // 2,
                "h2d_gbs_per_rank_in_run": e2e_value / world * (h2d_pair / 2) / 1e9,
                "h2d_gbs_per_rank_link_alone": h2d_gbs, "passes_ms": [round(p, 3) for p in e2e_ms]},
        "gpu_launches": int(launches),
        "clocks": cx.clocks.result,
        "hessian_accum": hess,
        "hessian_issues": int(issues), "engine_fault": int(fault),
    }


def cx_no_cpu(cx):
    return getattr(cx, "no_cpu_baseline", False)


def parity_sample(cx):
    """Untimed: one of the benchmark's own experts (its ragged token count) quantized once, the
    first 128 rows compared with the CPU oracle fed with the same Hessian.  Beside the engine's
    figure stand the oracle's own distance from exact arithmetic on this Hessian (its fp32 route
    against the same route with the factor computed in fp64) and the engine's agreement with that
    exact-factor route.  (With far fewer tokens than input channels the
    damped Hessian is so ill conditioned that a code on a rounding boundary flips with the last
    bits of the factor, and one flip changes a third of the codes behind it in that row.)"""
    from oracle import gptq_oracle as O

    rows = 128
    h = cx.make_handles(1)[0]
    H_raw = h.H.clone()
    q, s, z = h.quantize(BITS)
    Wc = cx.weights[0][:rows].cpu()
    Hc = H_raw.cpu()
    want = O.quantize_layer(Wc, Hc.clone(), bits=BITS, group_size=GROUP, rel_damp=1e-2, block_size=128)
    got = O.dequantize_linear_weight(q[:rows].cpu(), s[:rows].cpu(), z[:rows].cpu()).float()
    ref = O.dequantize_linear_weight(want["qweight"], want["scale"], want["zero"]).float()
    out = {"rows": rows, "tokens": cx.tokens[0], "code_agreement": O.code_agreement(q[:rows].cpu(), want["qweight"]),
           "scales_equal": bool(torch.equal(s[:rows].cpu().float(), want["scale"].float())),
           "recon_error": O.reconstruction_error(Wc.float(), got, Hc),
           "recon_error_oracle": O.reconstruction_error(Wc.float(), ref, Hc)}
    if not cx_no_cpu(cx):
        Hp, Wf, _, _ = O.pre_step(Hc.clone(), Wc)
        Hd = Hp.double()
        Hd += 1e-2 * torch.diag(Hd).mean() * torch.eye(Hd.shape[0], dtype=torch.float64)
        U = torch.linalg.cholesky(torch.cholesky_inverse(torch.linalg.cholesky(Hd)), upper=True)
        U = (U / U.diag()[:, None]).float().contiguous()
        sc, zr, maxq = O.symmetric_grid(Wf, GROUP, BITS, Wc.dtype)
        Q = O.gptq_sweep(Wf.t().contiguous(), U, sc.repeat_interleave(GROUP, -1).t().contiguous(),
                         zr.repeat_interleave(GROUP, -1).t().contiguous(), maxq, Wc.dtype, 128)
        exact = Q.t().contiguous().to(torch.uint8)
        out["oracle_fp32_vs_exact_factor"] = O.code_agreement(exact, want["qweight"])
        out["code_agreement_with_exact_factor"] = O.code_agreement(q[:rows].cpu(), exact)
    return out


# ---------------------------------------------------------------------------- the other named workloads
def _time_layers(cx, build, n, streams):
    """layers/s of `n` independent handles made by build(i), spread over `streams` CUDA streams."""
    from moe_quant_b200 import quantize_many
    warm = quantize_many([build(i) for i in range(n)], BITS, streams=streams)
    torch.cuda.synchronize()
    del warm
    ms = []
    for _ in range(3):
        hs = [build(i) for i in range(n)]
        torch.cuda.synchronize()
        e0, e1 = _event_pair()
        e0.record()
        res = quantize_many(hs, BITS, streams=streams)
        e1.record()
        torch.cuda.synchronize()
        ms.append(e0.elapsed_time(e1))
        del hs, res
    return n / (statistics.median(ms) / 1e3), statistics.median(ms)


def wl_down_proj(cx):
    """Expert down_proj, 7168 x 2048 fp16, 8192 calibration tokens, group size 32 / 64 / 128 /
    per-channel, followed by the int4 -> int32 packing of the codes."""
    from moe_quant_b200 import GPTQ, ops
    dev = cx.dev
    rows, cols, toks = 7168, 2048, 8192
    W = _randn_weight(rows, cols, torch.float16, 77, dev)
    X = _randn_acts(toks, cols, torch.float16, 78, dev)
    H = torch.zeros(cols, cols, dtype=torch.float32, device=dev)
    ops.hessian_accum(H, X, 0.0, 2.0 / toks)
    out = {"shape": [rows, cols], "dtype": "fp16", "tokens": toks, "groups": {}}
    for g in (32, 64, 128, cols):
        def build(i, g=g):
            h = GPTQ(_linear(W), g, True, 1e-2, 128)
            h.H = H.clone()
            h.num_samples = toks
            return h
        many, _ = _time_layers(cx, build, 16, cx.n_streams)
        one, ms1 = _time_layers(cx, build, 4, 1)
        out["groups"][str(g)] = {"layers_per_s": many, "layers_per_s_one_stream": one,
                                 "fp32_equiv_tflops_one_stream": layer_flop(rows, cols) / (ms1 / 4 / 1e3) / 1e12}
    # quantize + separate packing pass against the sweep that writes the packed words itself (g = 128, one stream)
    def build128():
        h = GPTQ(_linear(W), 128, True, 1e-2, 128)
        h.H = H.clone()
        h.num_samples = toks
        return h

    def timed_layers(fn, n=6):
        fn(build128())
        torch.cuda.synchronize()
        hs = [build128() for _ in range(n)]
        torch.cuda.synchronize()
        e0, e1 = _event_pair()
        e0.record()
        keep = [fn(h) for h in hs]
        e1.record()
        torch.cuda.synchronize()
        del keep
        return e0.elapsed_time(e1) / n

    ms_two = timed_layers(lambda h: ops.pack_int4(h.quantize(BITS)[0]))
    ms_fused = timed_layers(lambda h: h.quantize_packed(BITS))
    out["quantize_then_pack_ms"] = ms_two
    out["quantize_packed_fused_ms"] = ms_fused

    # packing alone: 16 different code matrices (235 MB, larger than L2), one launch each, replayed
    # from a CUDA graph so that the device time is not the time Python needs to issue a launch
    from moe_quant_b200 import _lib
    codes = [torch.randint(0, 16, (rows, cols), dtype=torch.uint8, device=dev) for _ in range(16)]
    words = [torch.empty(rows, cols // 8, dtype=torch.int32, device=dev) for _ in range(16)]
    L = _lib.lib()

    def pack_all():
        st = _lib.stream_ptr(dev)
        for c, w in zip(codes, words):
            _lib.check(L.mq_pack_int4(c.data_ptr(), rows, cols, None, 0, w.data_ptr(), st))

    pack_all()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        pack_all()
    graph.replay()
    torch.cuda.synchronize()
    e0, e1 = _event_pair()
    e0.record()
    for _ in range(8):
        graph.replay()
    e1.record()
    torch.cuda.synchronize()
    us = e0.elapsed_time(e1) * 1e3 / (8 * 16)
    gbs = 1.5 * rows * cols / (us * 1e-6) / 1e9
    assert torch.equal(words[3], ops.pack_int4(codes[3]))
    out["pack"] = {"us_per_launch": us, "gbs": gbs, "bytes_per_launch": 1.5 * rows * cols,
                   "roofline": {"bound": "hbm", "achieved": gbs, "peak": cx.peaks["hbm"], "unit": "GB/s",
                                "frac": gbs / cx.peaks["hbm"], "peak_source": cx.peaks["source"]}}
    return out


def wl_moe_layer(cx):
    """One rank's shard of a whole MoE layer: 32 routed experts x {gate_proj, up_proj (tied to gate),
    down_proj}, ragged token counts (top-8 routing of 32 x 4096 tokens over 256 experts), Hessian
    accumulation included.  No collective: routed experts are expert-parallel."""
    from moe_quant_b200 import GPTQ, ops, quantize_many, quantize_tied, synthetic
    dev, rank = cx.dev, cx.rank
    n_exp, hidden, inter = 32, 7168, 2048
    counts = synthetic.ragged_expert_counts(32 * 4096, 256, 8, 99)
    mine = [int(counts[(rank * n_exp + e) % 256]) for e in range(n_exp)]
    Wg = [_randn_weight(inter, hidden, torch.bfloat16, 1000 + e, dev) for e in range(n_exp)]
    Wu = [_randn_weight(inter, hidden, torch.bfloat16, 2000 + e, dev) for e in range(n_exp)]
    Wd = [_randn_weight(hidden, inter, torch.bfloat16, 3000 + e, dev) for e in range(n_exp)]
    Xs = [_randn_acts(m, hidden, torch.bfloat16, 4000 + e, dev) for e, m in enumerate(mine)]
    Xd = [_randn_acts(m, inter, torch.bfloat16, 5000 + e, dev) for e, m in enumerate(mine)]
    pool = [torch.cuda.Stream(device=dev) for _ in range(cx.n_streams)]

    def one_pass():
        gates = [GPTQ(_linear(w), GROUP, True, 1e-2, 128) for w in Wg]
        ups = [GPTQ(_linear(w), GROUP, True, 1e-2, 128, tied_gptq_handle=g) for w, g in zip(Wu, gates)]
        downs = [GPTQ(_linear(w), GROUP, True, 1e-2, 128) for w in Wd]
        torch.cuda.synchronize()
        e0, e1, e2 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for e in range(n_exp):                       # the Hessian pass: what the forward hooks do
            gates[e].update(Xs[e])
            downs[e].update(Xd[e])
        e1.record()
        # every expert's layers in one call: gate/up pairs share a factorisation, pairs and down_proj
        # layers of different experts run side by side (what block_driver.quantize_block does)
        res = quantize_many([h for e in range(n_exp) for h in (gates[e], ups[e], downs[e])], BITS, streams=cx.n_streams)
        e2.record()
        torch.cuda.synchronize()
        issues = sum(h.has_hessian_issues() for h in gates + ups + downs)
        return e0.elapsed_time(e1), e1.elapsed_time(e2), issues

    one_pass()
    runs = [one_pass() for _ in range(2)]
    h_ms = statistics.median(r[0] for r in runs)
    q_ms = statistics.median(r[1] for r in runs)
    total = h_ms + q_ms
    flop_h = sum(m * hidden * (hidden + 1) + m * inter * (inter + 1) for m in mine)
    return {"experts_per_rank": n_exp, "layers_per_rank": 3 * n_exp, "tokens_per_expert_min_mean_max":
            [min(mine), sum(mine) / n_exp, max(mine)], "hessian_pass_ms": h_ms, "quantize_ms": q_ms,
            "layer_ms_local": total,
            "hessian_tflops_unique": flop_h / (h_ms / 1e3) / 1e12, "hessian_issues": int(runs[-1][2])}


def wl_mla(cx):
    """The five MLA projections of a block (shared layers: every rank holds a slice of the
    calibration tokens).  Per rank: Hessian accumulation from its tokens; then
    gptq.quantize_shared: Hessians reduced to owner ranks, owners quantize side by side, results
    broadcast.  With one GPU the five layers run on five streams."""
    from moe_quant_b200 import GPTQ
    from moe_quant_b200.gptq import quantize_shared, shared_layer_owners
    dev, rank, world = cx.dev, cx.rank, cx.world
    shapes = [("q_a_proj", 1536, 7168), ("q_b_proj", 24576, 1536), ("kv_a_proj_with_mqa", 576, 7168),
              ("kv_b_proj", 32768, 512), ("o_proj", 7168, 16384)]
    toks = 8192                                     # per rank
    Ws = [_randn_weight(r, c, torch.bfloat16, 600 + i, dev) for i, (_, r, c) in enumerate(shapes)]
    Xs = {c: _randn_acts(toks, c, torch.bfloat16, 700 + c + rank, dev) for c in sorted({c for _, _, c in shapes})}

    def handles():
        return [GPTQ(_linear(w), GROUP, True, 1e-2, 128, is_distributed=True) for w in Ws]

    def one_pass(shared: bool):
        hs = handles()
        cx.barrier()
        e0, e1, e2 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for h, (_, _, c) in zip(hs, shapes):
            h.update(Xs[c])
        e1.record()
        if shared:
            res = quantize_shared(hs, BITS, streams=5)
        else:
            res = [h.quantize(BITS) for h in hs]    # the reference's scheme: all-reduce, rank 0 works, broadcast
        e2.record()
        cx.barrier()
        bad = sum(h.has_hessian_issues() for h in hs)
        del res
        return e0.elapsed_time(e1), e1.elapsed_time(e2), bad

    one_pass(True)
    a = [one_pass(True) for _ in range(2)]
    one_pass(False)
    b = [one_pass(False) for _ in range(2)]
    own_ms = cx.max_over_ranks(statistics.median(r[1] for r in a))
    ref_ms = cx.max_over_ranks(statistics.median(r[1] for r in b))
    h_ms = cx.max_over_ranks(statistics.median(r[0] for r in a))
    # each projection alone on one stream (rank 0's GPU, no collective): the terms of the sum
    alone = {}
    if rank == 0:
        for (name, r, c), w in zip(shapes, Ws):
            ms = []
            for _ in range(3):
                h = GPTQ(_linear(w), GROUP, True, 1e-2, 128)
                h.update(Xs[c])
                torch.cuda.synchronize()
                e0, e1 = _event_pair()
                e0.record()
                h.quantize(BITS)
                e1.record()
                torch.cuda.synchronize()
                ms.append(e0.elapsed_time(e1))
            t = statistics.median(ms[1:])
            alone[name] = {"ms": t, "fp32_equiv_tflops": layer_flop(r, c) / (t / 1e3) / 1e12}
    cx.barrier()
    flop_h = sum(toks * c * (c + 1) for _, _, c in shapes)
    return {"tokens_per_rank": toks, "owners": shared_layer_owners(handles(), world),
            "hessian_pass_ms": h_ms, "hessian_tflops_unique_per_rank": flop_h / (h_ms / 1e3) / 1e12,
            "quantize_ms_owner_ranks": own_ms, "quantize_ms_rank0_scheme": ref_ms,
            "each_alone_one_stream": alone, "sum_alone_ms": sum(v["ms"] for v in alone.values()) if alone else None,
            "hessian_issues": int(a[-1][2])}


def run_single_layer(args):
    """The small case for profiler captures: one Hessian from 4096 bf16 tokens, one 2048 x 7168
    layer quantized `--steps` times on one stream (about 1 GB on the device), no timing."""
    from moe_quant_b200 import _lib, ops
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    W = _randn_weight(R, C, torch.bfloat16, 0, dev)
    X = _randn_acts(TOKENS, C, torch.bfloat16, 1, dev)
    H = torch.zeros(C, C, device=dev)
    ops.hessian_accum(H, X, 0.0, 2.0 / TOKENS)
    precision = ops.Precision(compact=bool(args.compact))   # --compact: the launch shapes quantize_many asks for
    for _ in range(max(1, args.steps)):
        ops.quantize_layer([W], H.clone(), GROUP, BITS, 1e-2, precision=precision)
    torch.cuda.synchronize()
    print(json.dumps({"single_layer": True, "launches": int(_lib.lib().mq_launch_count()),
                      "engine_fault": int(_lib.engine_fault())}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=48)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--reps", type=int, default=5, help="how many times the pass of K steps is timed (median reported)")
    ap.add_argument("--streams", type=int, default=8, help="CUDA streams the independent layers are spread over")
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="all", choices=["all", "headline", "down_proj", "mla", "moe_layer"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--single-layer", action="store_true",
                    help="run one Hessian accumulation and --steps layers untimed (profiler captures)")
    ap.add_argument("--compact", action="store_true", help="with --single-layer: the compact launch shapes of quantize_many")
    args = ap.parse_args()
    if args.single_layer:
        run_single_layer(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_b200(args)


if __name__ == "__main__":
    main()
