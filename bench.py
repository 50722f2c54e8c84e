#!/usr/bin/env python
"""MoE-layer throughput benchmark (tokens/s) with roofline, CPU baseline and per-configuration sub-records.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload decode4x44|cfg0|t64|prefill4096|ep_prefill16384|ep_decode512]
    python bench.py --impl reference ...     # the CPU restatement of the reference's path on the host cores

One "step" is one pass of the MoE block over one batch of synthetic tokens.  The headline workload is
  decode4x44  (default): the MTP-verify step, T=4 tokens through all 44 MoE layers (layers 2..45), an
               independent weight set per layer (55 GB resident), so nothing a step touches is L2-resident
               when it is touched again.
The default run also measures, after the headline and outside its timed region, the other configurations
as sub-records of the same JSON line (`configs`):
  cfg0         T=1 token, one layer per call (the T=1 logits order), cycling the 44 weight sets;
  t64          one 64-row block per call, the reference's prefill block size (src/model.cpp:53,257-271);
  prefill4096  T=4096 tokens through one layer, Zipf(1.2) routing: stage times, padding waste;
and under torchrun (N > 1, one rank per GPU, 256/N experts per GPU, every GPU home to its own tokens):
  ep_prefill16384  T=16384 tokens, one layer, uniform routing: exposed communication time;
  ep_decode512     (8 GPUs) T=512 tokens x 44 layers, Zipf(1.0): per-GPU load imbalance.
`--workload X` makes X the headline instead (no sub-records).
Rank 0 prints ONE JSON line.  `value` is device-timed (CUDA events) with inputs resident in HBM; `e2e` is the
same metric through the host-buffer C-ABI call, host<->device copies inside the timed region.  The event
pair brackets R repetitions of the K steps so that the timed region lasts about a second (clock samples
every 100 ms then cover it); ms_per_step is the total over K*R.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import re
import subprocess
import sys
import threading
import time

import numpy as np

import __graft_entry__ as entry

HIDDEN, INTER, EXPERTS, TOP = 2560, 1024, 256, 8
EXPERT_BYTES = 3 * (INTER * HIDDEN // 2 + INTER * HIDDEN // 16)        # 4,423,680: packed + scales, 3 matrices
ROUTER_BYTES = EXPERTS * HIDDEN * 2 + EXPERTS * 4                      # 1,311,744
FLOPS_PER_TOKEN = 2 * (TOP + 1) * 3 * INTER * HIDDEN                   # 141,557,760 (expert products, unpadded)
SEED = 20261125
LAYERS = 44
DTYPE = "nvfp4 x nvfp4 -> f32 -> bf16"
NVFP4_DENSE_SPEC_TFLOPS = 9000.0                                       # B200 dense FP4, vendor figure


def peaks():
    path = os.path.join(entry.ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return {"hbm_gbs": float(p["hbm_gbs"]), "bf16_tflops": float(p.get("bf16_tflops", 0.0)), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


def nvfp4_yardstick(torch):
    """Dense NVFP4 rate of this GPU measured with a LIBRARY block-scaled FP4 GEMM (torch._scaled_mm: E2M1 operands,
    E4M3 scales per 16 values, BF16 result; 8192^3, a burst of 20 calls after 5 warm-up calls).  A yardstick for the
    tensor-side denominator only - nothing of the product runs through it.  None if this torch build refuses."""
    try:
        m = n = k = 8192
        a = torch.randint(0, 255, (m, k // 2), dtype=torch.uint8, device="cuda").view(torch.float4_e2m1fn_x2)
        b = torch.randint(0, 255, (n, k // 2), dtype=torch.uint8, device="cuda").view(torch.float4_e2m1fn_x2)
        sa = torch.full((m * (k // 16),), 0x38, dtype=torch.uint8, device="cuda").view(torch.float8_e4m3fn)
        sb = torch.full((n * (k // 16),), 0x38, dtype=torch.uint8, device="cuda").view(torch.float8_e4m3fn)

        def run():
            return torch._scaled_mm(a, b.t(), scale_a=sa, scale_b=sb, out_dtype=torch.bfloat16)

        for _ in range(5):
            run()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        for _ in range(20):
            run()
        e1.record()
        torch.cuda.synchronize()
        return 2.0 * m * n * k * 20 / (e0.elapsed_time(e1) * 1e-3) / 1e12
    except Exception:                     # noqa: BLE001 - any refusal of the library call means "no yardstick"
        return None


def ncu_ratios() -> dict:
    """kernel -> (traffic / algorithmic bytes, tensor pipe %) from the table kept beside the ncu summaries."""
    out = {}
    path = os.path.join(entry.ROOT, "profiles", "ncu_ratios.md")
    if not os.path.exists(path):
        return out
    for line in open(path):
        cells = [c.strip() for c in line.strip().strip("|").split("|")]
        if len(cells) == 4 and re.fullmatch(r"[0-9.]+", cells[1] or "x"):
            out[cells[0]] = {"traffic_over_algorithmic": float(cells[1]), "tensor_pipe_pct": float(cells[2]),
                             "capture": cells[3]}
    return out


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while a region runs (read-only)."""

    QUERY = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.rows = []
        self.proc = None
        self.marks = []
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={index}", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.time(), line.strip()))

    def mark(self):
        self.marks.append(time.time())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        lo, hi = (self.marks + [0, 1e18])[:2] if len(self.marks) >= 2 else (0, 1e18)
        picked = [r for t, r in self.rows if lo <= t <= hi] or [r for _, r in self.rows]
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for row in picked:
            parts = [p.strip() for p in row.split(",")]
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except (ValueError, IndexError):
                continue
            for name, flag in zip(names, parts[3:7]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# --------------------------------------------------------------------------------------------
# workloads
# --------------------------------------------------------------------------------------------

WORKLOADS = {
    # name: (tokens per step on one GPU, layers per step, bias mode, zipf alpha)
    "decode4x44": (4, LAYERS, "normal", 0.0),
    "cfg0": (1, 1, "normal", 0.0),
    "t64": (64, 1, "normal", 0.0),
    "prefill4096": (4096, 1, "zipf", 1.2),
    "ep_prefill16384": (16384, 1, "zero", 0.0),
    "ep_decode512": (512, LAYERS, "zipf", 1.0),
}


def ep_mode(workload: str, world: int) -> str:
    """Orchestration bench.py picks for a workload at `world` GPUs (P92B_EP_EXCHANGE overrides)."""
    forced = os.environ.get("P92B_EP_EXCHANGE", "")
    if forced:
        return forced
    rows = ep_rows(workload, world)
    if rows <= 8 and world * rows <= 32:
        return "fused"
    if rows <= 128 and world * rows <= 1024:
        return "gathered"          # measured on the 512-token workload: 6.42 ms against 7.03 ms (bulk) at 128 rows per GPU,
    return "bulk"                  # 9.42 ms against 9.06 ms (bulk) at 256


def ep_rows(workload: str, world: int) -> int:
    """Home tokens per GPU: the decode step is weak-scaled (4 per GPU), the others split their batch."""
    tokens = WORKLOADS[workload][0]
    return tokens if workload == "decode4x44" else tokens // world


PARALLELISM = {
    "fused": "one kernel per GPU and layer, dispatch (all-gather) and combine by peer stores over NVLink inside the kernel",
    "gathered": "all-gather dispatch and direct placement of result rows by the library's own kernels (peer stores over "
                "NVLink, polled words), grouped tcgen05 products in between; no NCCL, no host sync",
    "bulk": "all-gather dispatch and direct placement of result rows by the library's own kernels (16-byte peer stores over "
            "NVLink, one flag per peer and exchange), permutation over the whole batch restricted to the local experts, "
            "grouped tcgen05 products; no NCCL, no host sync",
    "fixed": "NCCL all-to-all dispatch and combine, fixed-capacity blocks, no host sync",
    "exact": "NCCL all-to-all dispatch and combine, exact-size splits",
}


def workload_config(name: str, gpus: int) -> dict:
    tokens, layers, bias_mode, alpha = WORKLOADS[name]
    text = {
        "decode4x44": "decode MTP-verify: T=4 tokens x 44 MoE layers (hidden 2560, 256+1 experts, FFN 1024, top-8)",
        "cfg0": "single-token decode: T=1 token x 1 MoE layer per call, 44 weight sets cycled",
        "t64": "one prefill block of the reference: T=64 tokens x 1 MoE layer per call, 44 weight sets cycled",
        "prefill4096": "prefill chunk: T=4096 tokens x 1 MoE layer, Zipf(1.2) routing",
        "ep_prefill16384": "expert-parallel prefill: T=16384 tokens x 1 MoE layer, uniform routing (bias 0)",
        "ep_decode512": "batched serving decode: T=512 tokens (128 sequences x 4 MTP positions) x 44 MoE layers, Zipf(1.0) routing",
    }[name]
    routing = {"normal": "bias ~N(0,0.01)", "zero": "uniform (bias 0)", "zipf": f"zipf {alpha} (capped at 1/8)"}[bias_mode]
    cfg = {"workload": text, "tokens_per_step": tokens, "layers": layers, "routing": routing, "gpus": gpus,
           "l2": "inputs larger than L2: 44 distinct weight sets (55 GB) cycle" if name in ("decode4x44", "cfg0", "t64", "ep_decode512")
                 else "inputs larger than L2: 1.14 GB of weights per layer call (0.15-0.57 GB per GPU under expert parallelism, plus token rows)"}
    if gpus > 1:
        mode = ep_mode(name, gpus)
        rows = ep_rows(name, gpus)
        cfg["tokens_per_step"] = rows * gpus
        cfg["parallelism"] = f"ep{gpus}: {EXPERTS // gpus} experts per GPU, {rows} home tokens per GPU, {PARALLELISM[mode]}"
    return cfg


def host_inputs(layer: int, rows: int, bias_std: float, stream: int = 0):
    entry.load_package()
    from p92moe_b200 import synth

    return synth.host_router_inputs(SEED, layer, rows, bias_std=bias_std, stream=stream)


def as_u16(t) -> np.ndarray:
    import torch

    return t.contiguous().view(torch.int16).numpy().view(np.uint16)


# --------------------------------------------------------------------------------------------
# CPU arm: the CPU restatement of the reference's MoE forward on the host cores
# --------------------------------------------------------------------------------------------

class CpuLayer:
    """One synthetic layer on the host for the oracle.  Router weight, bias and token rows come from the same
    host generator the GPU arm uploads (synth.host_router_inputs), so both arms route identically; the NVFP4
    experts are drawn (N(0,0.02) -> BF16 -> the oracle's restatement of the offline quantiser) only when a
    token is routed to them, since expert weights do not influence routing."""

    def __init__(self, orc, layer: int, rows: int, bias_std: float = 0.01, bias=None):
        self.orc = orc
        router, host_bias, x = host_inputs(layer, rows, bias_std)
        self.router, self.x = as_u16(router), as_u16(x)
        self.bias = host_bias.numpy() if bias is None else np.ascontiguousarray(bias, dtype=np.float32)
        n = (EXPERTS + 1) * 3
        self.packed = np.empty((n, INTER * HIDDEN // 2), np.uint8)      # untouched pages stay virtual
        self.scales = np.empty((n, INTER * HIDDEN // 16), np.uint8)
        self.alpha = np.zeros(n, np.float32)
        self.have = set()
        self.layer = layer
        logits = orc.router_logits(self.x, self.router)
        ids, _, _ = orc.router_top8(logits, self.bias)
        for e in sorted(set(ids.reshape(-1).tolist()) | {EXPERTS}):
            self._draw(e)
        self.distinct = len(self.have) - 1

    def _draw(self, e: int):
        rng = np.random.default_rng([SEED, self.layer, 1000 + e])
        for kind in range(3):
            shape = (INTER, HIDDEN) if kind < 2 else (HIDDEN, INTER)
            w = self.orc.f32_to_bf16((rng.standard_normal(shape, dtype=np.float32) * np.float32(0.02)))
            p, s, a = self.orc.nvfp4_pack_weight(w)
            self.packed[e * 3 + kind] = p.reshape(-1)
            self.scales[e * 3 + kind] = s.reshape(-1)
            self.alpha[e * 3 + kind] = a
        self.have.add(e)

    def forward(self):
        return self.orc.moe_forward(self.x, self.router, self.bias, self.packed, self.scales, self.alpha, HIDDEN,
                                    INTER)


def cpu_threads(orc) -> int:
    """All host cores: torchrun exports OMP_NUM_THREADS=1, which would otherwise pin the oracle to one."""
    cores = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    orc.cpu().orc_set_threads(cores)
    return int(orc.cpu().orc_threads())


def run_cpu(workload: str, gpus: int, steps: int, warmup: int) -> dict:
    """Bounded sample of the workload on the host cores: decode-sized batches run whole on 2 of the 44 layers,
    the large batches run 16 of their tokens through one layer; tokens/s scales by layer count (every layer
    costs the same) and is per token whatever the sample size."""
    orc = entry.load_oracle()
    cores = cpu_threads(orc)
    tokens, total_layers, bias_mode, _ = WORKLOADS[workload]
    rows = tokens if workload == "decode4x44" and gpus == 1 else (tokens * gpus if workload == "decode4x44" else tokens)
    sample_rows = rows if rows <= 32 else 16
    sample_layers = min(2, total_layers)
    bias_std = 0.0 if bias_mode == "zero" else 0.01
    layers = [CpuLayer(orc, l, sample_rows, bias_std) for l in range(sample_layers)]
    for _ in range(warmup):
        layers[0].forward()
    t0 = time.perf_counter()
    for _ in range(steps):
        for layer in layers:
            layer.forward()
    dt = (time.perf_counter() - t0) / steps
    per_token_layer = dt / (sample_layers * sample_rows)
    step_time = per_token_layer * rows * total_layers
    return {"value": rows / step_time, "ms_per_step": step_time * 1e3, "cores": cores,
            "sample": f"{sample_rows} of {rows} tokens x {sample_layers} of {total_layers} layers per sample step, "
                      f"{steps} sample steps, scaled by token and layer count"
                      + ("" if bias_mode != "zipf" else "; routing bias ~N(0,0.01) instead of the fitted Zipf bias "
                                                            "(the CPU cost per token does not depend on which experts are hit)")}


def reference_arm(args) -> None:
    if int(os.environ.get("RANK", "0")) != 0:
        return
    steps = max(1, min(args.steps, 3))
    warmup = min(args.warmup, 1)
    r = run_cpu(args.workload, args.gpus, steps, warmup)
    line = {
        "impl": "reference", "metric": "moe_layer_tokens_per_s", "value": r["value"], "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": steps, "warmup": warmup, "ms_per_step": r["ms_per_step"],
        "higher_is_better": True, "scaling": "weak" if args.workload == "decode4x44" else "strong", "vs_baseline": None,
        "dtype": DTYPE, "data": "synthetic", "config": workload_config(args.workload, args.gpus),
        "cpu_baseline": {"value": r["value"], "unit": "tokens/s", "cores": r["cores"], "kind": "port",
                         "sample": r["sample"]},
        "e2e": {"value": r["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


# --------------------------------------------------------------------------------------------
# timing helpers
# --------------------------------------------------------------------------------------------

class Timer:
    """CUDA-event timing of `steps` x R calls of step(); R is chosen from one calibration pass so that the
    region lasts at least `min_seconds`.  Under torch.distributed the region is bracketed by a barrier and a
    device synchronisation on both sides and the result is the maximum over ranks."""

    def __init__(self, torch, dist=None):
        self.torch, self.dist = torch, dist

    def barrier(self):
        if self.dist is not None:
            self.dist.barrier()
        self.torch.cuda.synchronize()

    def max_over_ranks(self, value: float) -> float:
        if self.dist is None:
            return value
        t = self.torch.tensor([value], device="cuda", dtype=self.torch.float64)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t[0])

    def run(self, step, steps: int, min_seconds: float, sampler=None, max_repeats: int = 10000):
        torch = self.torch
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        self.barrier()
        a.record()
        step()
        b.record()
        self.barrier()
        estimate = self.max_over_ranks(a.elapsed_time(b)) * 1e-3
        repeats = int(min(max_repeats, max(1, math.ceil(min_seconds / max(estimate * steps, 1e-9)))))
        self.barrier()
        if sampler:
            sampler.mark()
        a.record()
        for _ in range(repeats * steps):
            step()
        b.record()
        self.barrier()
        if sampler:
            sampler.mark()
        return self.max_over_ranks(a.elapsed_time(b)) / (repeats * steps), repeats


def layer_bytes(distinct: float, rows: int) -> float:
    """Algorithmic bytes of one layer call: the experts hit (+ the shared one) once each, the router weight,
    the token rows in and out."""
    return (distinct + 1) * EXPERT_BYTES + ROUTER_BYTES + rows * HIDDEN * 2 * 2


# --------------------------------------------------------------------------------------------
# one GPU
# --------------------------------------------------------------------------------------------

class SingleGpu:
    def __init__(self, torch, pkg, synth, n_layers: int):
        self.torch, self.pkg, self.synth = torch, pkg, synth
        self.banks, self.routers, self.biases = [], [], []
        for l in range(n_layers):
            raw = synth.make_raw_layer_batched(SEED, l)
            self.banks.append(pkg.ExpertBank(raw.entries()))
            router, bias, _ = host_inputs(l, 1, 0.01)
            self.routers.append(router.cuda())
            self.biases.append(bias.cuda())
            del raw
        torch.cuda.synchronize()
        self.timer = Timer(torch)

    def inputs(self, rows: int, n_layers: int):
        return [host_inputs(l, rows, 0.01)[2].cuda() for l in range(n_layers)]

    def blocks(self, plan, biases=None):
        biases = biases or self.biases
        return [self.pkg.MoeBlock(b, r, c, plan) for b, r, c in zip(self.banks, self.routers, biases)]

    def distinct(self, plan, blocks, xs, outs, rows):
        d = []
        for b, x, o in zip(blocks, xs, outs):
            b.run_moe_rows(x, o, rows)
            d.append(int((plan.views(rows)["counts"] > 0).sum()))
        return float(np.mean(d))

    def decode_like(self, name: str, steps: int, warmup: int, min_seconds: float, sampler=None, e2e: bool = False) -> dict:
        """Workloads that run one small batch through the 44 weight sets: decode4x44 (a step = all 44 layers),
        cfg0 and t64 (a step = one layer call; the 44 sets cycle so nothing is L2-resident)."""
        torch, pkg = self.torch, self.pkg
        rows = WORKLOADS[name][0]
        n_layers = len(self.banks)
        per_call = name != "decode4x44"
        plan = pkg.MoePlan(max_rows=rows)
        blocks = self.blocks(plan)
        xs = self.inputs(rows, n_layers)
        outs = [torch.empty_like(x) for x in xs]
        cursor = [0]

        def step_all():
            for b, x, o in zip(blocks, xs, outs):
                b.run_moe_rows(x, o, rows)

        def step_one():
            i = cursor[0] % n_layers
            cursor[0] += 1
            blocks[i].run_moe_rows(xs[i], outs[i], rows)

        step = step_one if per_call else step_all
        for _ in range(warmup * (n_layers if per_call else 1)):
            step()
        inner = n_layers if per_call else 1            # a "step" of the per-call workloads is timed in whole cycles
        ms, repeats = self.timer.run(step, steps * inner, min_seconds, sampler)
        launches_per_call = plan.last_launches
        status = plan.status()
        d_mean = self.distinct(plan, blocks, xs, outs, rows)
        calls_per_step = 1 if per_call else n_layers
        us_per_call = ms * 1e3 / calls_per_step
        bytes_call = layer_bytes(d_mean, rows)
        pk = peaks()
        gbs = bytes_call / (us_per_call * 1e-6) / 1e9
        kernel = "moe_decode_kernel" if rows <= 16 else "expert_tc_kernel (gate/up + down of a %d-launch chain)" % launches_per_call
        ratio = ncu_ratios().get("moe_decode_kernel") if rows <= 16 else None
        rec = {
            "ms_per_step": ms, "value": rows / (ms * 1e-3), "unit": "tokens/s", "steps": steps * inner, "repeats": repeats,
            "us_per_layer_call": us_per_call, "gpu_launches": launches_per_call * calls_per_step * steps * inner * repeats,
            "launches_per_layer_call": launches_per_call, "status": status,
            "roofline": {"bound": "hbm", "kernel": kernel, "achieved": gbs, "peak": pk["hbm_gbs"], "unit": "GB/s",
                         "frac": gbs / pk["hbm_gbs"], "peak_source": pk["source"], "bytes_per_launch": bytes_call,
                         "us_per_launch": us_per_call, "distinct_routed_experts_mean": d_mean,
                         "traffic": bytes_call * ratio["traffic_over_algorithmic"] if ratio else None,
                         "traffic_source": (f"measured DRAM bytes / algorithmic bytes = {ratio['traffic_over_algorithmic']} in the ncu "
                                            f"capture {ratio['capture']}, applied to this run's algorithmic bytes") if ratio else None,
                         "timing": "one launch per layer call back to back on one stream: step time / calls (an event pair per "
                                   "launch would break the overlap of consecutive launches)"},
        }
        if rows > 8:
            # the multi-kernel pipeline: per-stage device times from event pairs inside the library
            plan.stage_timing(True)
            for _ in range(2 * n_layers):
                step_one()
            stage_ms, calls = plan.stage_times()
            plan.stage_timing(False)
            rec["stage_us"] = {k: v / calls * 1e3 for k, v in stage_ms.items()}
        if name == "cfg0":
            rec["target_us"] = 8.99
        if e2e:
            rec["e2e"] = self.e2e_decode(plan, blocks, xs, rows, steps)
        plan.close()
        return rec

    def e2e_decode(self, plan, blocks, xs, rows, steps) -> dict:
        torch = self.torch
        host_in = [x.cpu().pin_memory() for x in xs]
        host_out = [torch.empty_like(h).pin_memory() for h in host_in]
        for b, hi, ho in zip(blocks, host_in, host_out):
            b.run_moe_rows_host(hi, ho, rows)

        def one():
            for b, hi, ho in zip(blocks, host_in, host_out):
                b.run_moe_rows_host_async(hi, ho, rows)
            plan.host_flush()
            torch.cuda.current_stream().synchronize()

        one()
        t0 = time.perf_counter()
        one()
        estimate = time.perf_counter() - t0
        n = max(3, min(2000, math.ceil(0.5 / max(estimate, 1e-6))))
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(n):
            one()
        e2e_s = (time.perf_counter() - t0) / n
        t0 = time.perf_counter()
        for _ in range(max(3, n // 4)):
            for b, hi, ho in zip(blocks, host_in, host_out):
                b.run_moe_rows_host(hi, ho, rows)
        sync_s = (time.perf_counter() - t0) / max(3, n // 4)
        bytes_io = len(blocks) * rows * HIDDEN * 2
        return {"value": rows / e2e_s, "unit": "tokens/s", "h2d_bytes_per_step": bytes_io, "d2h_bytes_per_step": bytes_io,
                "ms_per_step": e2e_s * 1e3, "steps": n, "ms_per_step_sync_per_layer": sync_s * 1e3,
                "call": "p92b_moe_forward_host_async per layer (copies pipelined on the plan's streams), one flush + stream "
                        "synchronisation per step"}

    def prefill(self, name: str, steps: int, warmup: int, min_seconds: float, sampler=None, e2e: bool = False) -> dict:
        """Large batch through ONE layer (the first weight set): per-stage device times from event pairs inside the
        library, roofline of the dominant kernel, padding waste of the padded position space."""
        torch, pkg, synth = self.torch, self.pkg, self.synth
        rows, _, bias_mode, alpha = WORKLOADS[name]
        if bias_mode == "zipf":
            bias = synth.fit_zipf_bias(self.routers[0], alpha, SEED)[0].contiguous()
        elif bias_mode == "zero":
            bias = torch.zeros_like(self.biases[0])
        else:
            bias = self.biases[0]
        plan = pkg.MoePlan(max_rows=rows)
        block = pkg.MoeBlock(self.banks[0], self.routers[0], bias, plan)
        x = host_inputs(0, rows, 0.01)[2].cuda()
        out = torch.empty_like(x)

        def step():
            block.run_moe_rows(x, out, rows)

        for _ in range(warmup):
            step()
        ms, repeats = self.timer.run(step, steps, min_seconds, sampler)
        launches = plan.last_launches
        status = plan.status()
        counts = plan.views(rows)["counts"].cpu().numpy().astype(np.int64)
        plan.stage_timing(True)
        for _ in range(10):
            step()
        stage_ms, calls = plan.stage_times()
        plan.stage_timing(False)
        stage_us = {k: v / calls * 1e3 for k, v in stage_ms.items()}
        distinct = int((counts > 0).sum())
        real = rows * (TOP + 1)
        padded = int((np.ceil(counts / 128) * 128).sum() + math.ceil(rows / 128) * 128)
        tiles64 = int((np.ceil(counts / 64) * 64).sum() + math.ceil(rows / 64) * 64)
        pk = peaks()
        t_bytes = layer_bytes(distinct, rows) / (pk["hbm_gbs"] * 1e9)
        yardstick = nvfp4_yardstick(torch)
        nvfp4_peak = yardstick if yardstick else 4 * pk["bf16_tflops"]
        t_flops = rows * FLOPS_PER_TOKEN / (nvfp4_peak * 1e12)
        ratios = ncu_ratios()
        gu = ratios.get("expert_gu_pair_kernel")
        gu_bytes = (distinct + 1) * 2 * (EXPERT_BYTES // 3) + rows * (HIDDEN // 2 + HIDDEN // 16) + real * (INTER // 2 + INTER // 16)
        gu_us = stage_us["gate_up_swiglu"]
        gu_gbs = gu_bytes / (gu_us * 1e-6) / 1e9
        rec = {
            "ms_per_step": ms, "value": rows / (ms * 1e-3), "unit": "tokens/s", "steps": steps, "repeats": repeats,
            "gpu_launches": launches * steps * repeats, "launches_per_layer_call": launches, "status": status,
            "stage_us": stage_us, "distinct_routed_experts": distinct,
            "rows_per_expert": {"max": int(counts.max()), "mean": float(counts.mean()), "min": int(counts.min())},
            "padding_waste": {"padded_rows_over_real_rows": padded / real, "padded_rows": padded, "real_rows": real,
                              "mma_rows_over_real_rows_64_row_tiles": tiles64 / real,
                              "note": "every expert's rows start on a multiple of 128 padded positions (address space only); "
                                      "the products run on 64-row token tiles, whose last tile per expert is partly empty"},
            "roofline_layer": {"t_bytes_us": t_bytes * 1e6, "t_flops_us": t_flops * 1e6,
                               "frac_of_max": max(t_bytes, t_flops) / (ms * 1e-3),
                               "nvfp4_dense_peak_tflops": nvfp4_peak,
                               "nvfp4_peak_source": ("measured in this run: library block-scaled FP4 GEMM (torch._scaled_mm, 8192^3, "
                                                     "burst); vendor figure 9000") if yardstick else
                                                    ("4 x the measured dense BF16 rate of MEASURED_PEAKS.json (the library FP4 GEMM "
                                                     "was refused by this torch build); vendor figure 9000"),
                               "flops_per_token": FLOPS_PER_TOKEN, "tensor_pipe_pct_ncu": gu["tensor_pipe_pct"] if gu else None,
                               "tensor_pipe_capture": gu["capture"] if gu else None},
            "roofline": {"bound": "hbm", "kernel": "expert_gu_pair_kernel", "achieved": gu_gbs, "peak": pk["hbm_gbs"],
                         "unit": "GB/s", "frac": gu_gbs / pk["hbm_gbs"], "peak_source": pk["source"], "bytes_per_launch": gu_bytes,
                         "us_per_launch": gu_us, "traffic": gu_bytes * gu["traffic_over_algorithmic"] if gu else None,
                         "traffic_source": (f"measured DRAM bytes / algorithmic bytes = {gu['traffic_over_algorithmic']} in the ncu "
                                            f"capture {gu['capture']}, applied to this run's algorithmic bytes") if gu else None,
                         "timing": "event pair around the launch inside the library (p92b_plan_stage_timing)"},
        }
        if e2e:
            hi = x.cpu().pin_memory()
            ho = torch.empty_like(hi).pin_memory()
            block.run_moe_rows_host(hi, ho, rows)
            t0 = time.perf_counter()
            n = 0
            while time.perf_counter() - t0 < 0.5 or n < 3:
                block.run_moe_rows_host(hi, ho, rows)
                n += 1
            e2e_s = (time.perf_counter() - t0) / n
            io = rows * HIDDEN * 2
            rec["e2e"] = {"value": rows / e2e_s, "unit": "tokens/s", "h2d_bytes_per_step": io, "d2h_bytes_per_step": io,
                          "ms_per_step": e2e_s * 1e3, "steps": n, "call": "p92b_moe_forward_host (copies on the stream, synchronised on return)"}
        plan.close()
        return rec


def run_single_gpu(args, torch, pkg, synth, warmup, steps) -> None:
    headline = args.workload
    n_layers = args.layers or (1 if headline in ("prefill4096", "ep_prefill16384") else LAYERS)
    sampler = ClockSampler(int(os.environ.get("LOCAL_RANK", "0")))
    gpu = SingleGpu(torch, pkg, synth, n_layers)
    if headline in ("prefill4096", "ep_prefill16384"):
        rec = gpu.prefill(headline, steps, warmup, args.min_seconds, sampler, e2e=True)
    elif headline == "ep_decode512":
        rec = gpu_decode512_single(gpu, steps, warmup, args.min_seconds, sampler)
    else:
        rec = gpu.decode_like(headline, steps, warmup, args.min_seconds, sampler, e2e=True)
    clocks = sampler.stop()
    subs = {}
    if headline == "decode4x44" and not args.no_sub_records and n_layers == LAYERS:
        subs["cfg0"] = gpu.decode_like("cfg0", 5, 3, 0.3)
        subs["t64"] = gpu.decode_like("t64", 5, 3, 0.3)
        subs["prefill4096"] = gpu.prefill("prefill4096", 10, 3, 0.3)
        for name, sub in subs.items():
            sub["config"] = workload_config(name, 1)
    cpu = None
    if not args.no_cpu_baseline:
        r = run_cpu(headline, 1, 1, 1)
        cpu = {"value": r["value"], "unit": "tokens/s", "cores": r["cores"], "kind": "port", "sample": r["sample"]}
    status = max([rec["status"]] + [s["status"] for s in subs.values()])
    line = {
        "metric": "moe_layer_tokens_per_s", "value": rec["value"], "unit": "tokens/s", "n_gpus": 1, "steps": steps,
        "repeats": rec["repeats"], "warmup": warmup, "ms_per_step": rec["ms_per_step"], "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": DTYPE, "data": "synthetic",
        "config": workload_config(headline, 1), "clocks": clocks, "e2e": rec.get("e2e"),
        "gpu_launches": rec["gpu_launches"], "roofline": rec["roofline"], "cpu_baseline": cpu, "status": status,
        "timed_region": f"{steps} steps x {rec['repeats']} repetitions inside one CUDA-event pair",
    }
    for key in ("stage_us", "padding_waste", "roofline_layer", "us_per_layer_call", "launches_per_layer_call",
                "rows_per_expert"):
        if key in rec:
            line[key] = rec[key]
    if subs:
        line["configs"] = subs
    print(json.dumps(line))
    if status != 0:
        sys.exit(f"a kernel recorded status {status} (1: expert id out of range, 2: a bounded wait gave up)")


def gpu_decode512_single(gpu: "SingleGpu", steps, warmup, min_seconds, sampler) -> dict:
    """T=512 x 44 layers on one GPU (the single-GPU point of config 4): the multi-kernel pipeline per layer."""
    torch, pkg, synth = gpu.torch, gpu.pkg, gpu.synth
    rows = 512
    biases = [synth.fit_zipf_bias(r, 1.0, SEED + l)[0].contiguous() for l, r in enumerate(gpu.routers)]
    plan = pkg.MoePlan(max_rows=rows)
    blocks = gpu.blocks(plan, biases)
    xs = gpu.inputs(rows, len(blocks))
    outs = [torch.empty_like(x) for x in xs]

    def step():
        for b, x, o in zip(blocks, xs, outs):
            b.run_moe_rows(x, o, rows)

    for _ in range(warmup):
        step()
    ms, repeats = gpu.timer.run(step, steps, min_seconds, sampler)
    d_mean = gpu.distinct(plan, blocks, xs, outs, rows)
    pk = peaks()
    gbs = layer_bytes(d_mean, rows) * len(blocks) / (ms * 1e-3) / 1e9
    rec = {"ms_per_step": ms, "value": rows / (ms * 1e-3), "repeats": repeats, "status": plan.status(),
           "gpu_launches": plan.last_launches * len(blocks) * steps * repeats,
           "roofline": {"bound": "hbm", "kernel": "expert_tc_kernel chain", "achieved": gbs, "peak": pk["hbm_gbs"], "unit": "GB/s",
                        "frac": gbs / pk["hbm_gbs"], "peak_source": pk["source"], "traffic": None,
                        "distinct_routed_experts_mean": d_mean}}
    plan.close()
    return rec


# --------------------------------------------------------------------------------------------
# N GPUs, one rank each: expert parallel
# --------------------------------------------------------------------------------------------

class ExpertParallel:
    def __init__(self, torch, dist, pkg, synth, world, rank, n_layers):
        from p92moe_b200 import ep

        self.torch, self.dist, self.pkg, self.synth, self.ep = torch, dist, pkg, synth, ep
        self.world, self.rank = world, rank
        self.first, self.local = ep.shard_range(rank, world)
        self.banks, self.routers, self.biases = [], [], []
        for l in range(n_layers):
            raw = synth.make_raw_layer_batched(SEED, l)                  # same weights on every rank; keep the shard
            entries = raw.entries()
            shard = entries[self.first * 3:(self.first + self.local) * 3] + entries[EXPERTS * 3:]
            self.banks.append(pkg.ExpertBank(shard, first_expert=self.first, local_experts=self.local))
            router, bias, _ = host_inputs(l, 1, 0.01)
            self.routers.append(router.cuda())
            self.biases.append(bias.cuda())
            del raw, entries, shard
        torch.cuda.synchronize()
        self.timer = Timer(torch, dist)
        self.windows_ok = None

    def window_and_plan(self, rows, bulk=False):
        """One window and one plan serve all layers of a workload.  If the windows cannot be mapped into one
        another (no inter-process memory handles in this environment) every rank falls back to NCCL."""
        torch, dist = self.torch, self.dist
        ok, window, plan = 1, None, None
        try:
            window = self.ep.EpWindow(self.rank, self.world, rows, bulk=bulk)
            plan = self.pkg.MoePlan(max_rows=self.world * rows)
        except Exception as exc:                                 # noqa: BLE001 - any failure means "no peer windows"
            ok = 0
            if self.rank == 0:
                print(f"peer windows unavailable ({exc}); using the NCCL exchange", file=sys.stderr)
        agreed = torch.tensor([ok], device="cuda")
        dist.all_reduce(agreed, op=dist.ReduceOp.MIN)
        if int(agreed[0]) == 0:
            return None, None
        return window, plan

    def run(self, name: str, steps: int, warmup: int, min_seconds: float, sampler=None, e2e: bool = False) -> dict:
        torch, dist, ep, pkg, synth = self.torch, self.dist, self.ep, self.pkg, self.synth
        world, rank = self.world, self.rank
        rows = ep_rows(name, world)
        _, layers_wanted, bias_mode, alpha = WORKLOADS[name]
        n_layers = min(layers_wanted, len(self.banks))
        mode = ep_mode(name, world)
        window = plan = None
        if mode in ("fused", "gathered", "bulk"):
            window, plan = self.window_and_plan(rows, bulk=mode == "bulk")
            if window is None:
                mode = "fixed" if rows <= ep.FIXED_MAX_ROWS else "exact"
        biases = []
        for l in range(n_layers):
            if bias_mode == "zipf":
                biases.append(synth.fit_zipf_bias(self.routers[l], alpha, SEED + l)[0].contiguous())
            elif bias_mode == "zero":
                biases.append(torch.zeros_like(self.biases[l]))
            else:
                biases.append(self.biases[l])
        states = []
        if mode in ("fixed", "exact"):
            for l in range(n_layers):
                states.append(ep.EpRank(rank, world, self.banks[l], self.routers[l], biases[l], max_local_rows=rows,
                                        share_scratch_with=states[0] if states else None))
        xs = [host_inputs(l, rows, 0.01, stream=rank + 1)[2].cuda() for l in range(n_layers)]
        outs = [torch.empty_like(x) for x in xs]
        torch.cuda.synchronize()

        def forward(l, x, o):
            if mode == "fused":
                ep.forward_fused(window, plan, self.banks[l], self.routers[l], biases[l], x, o, rows)
            elif mode == "gathered":
                ep.forward_gathered(window, plan, self.banks[l], self.routers[l], biases[l], x, o, rows)
            elif mode == "bulk":
                ep.forward_bulk(window, plan, self.banks[l], self.routers[l], biases[l], x, o, rows)
            elif mode == "fixed":
                ep.forward_nccl_fixed(states[l], x, o, rows, 8 * rows)
            else:
                ep.forward_nccl(states[l], x, o, rows)

        def step():
            for l in range(n_layers):
                forward(l, xs[l], outs[l])

        # every rank has built its banks before anyone's kernels start polling a peer (their waits give up after ~1 s)
        self.timer.barrier()
        for _ in range(warmup):
            step()
        ms, repeats = self.timer.run(step, steps, min_seconds, sampler)
        own = mode in ("fused", "gathered", "bulk")
        count_plan = plan if own else states[-1].arrivals
        home_plan = plan if own else states[-1].home
        if own:
            launches = count_plan.last_launches
        else:    # the library's kernels of route + experts + combine, counted by the three plans they run on
            launches = states[-1].home.last_launches + states[-1].arrivals.last_launches + states[-1].shared.last_launches
        status = max(count_plan.status(), home_plan.status())
        step()
        torch.cuda.synchronize()
        local_counts = count_plan.device_counts()[self.first:self.first + self.local].clone()
        received = float(local_counts.sum())
        load = torch.tensor([received], device="cuda")
        loads = [torch.zeros_like(load) for _ in range(world)]
        dist.all_gather(loads, load)
        loads = [float(v[0]) for v in loads]
        st = torch.tensor([status], device="cuda")
        dist.all_reduce(st, op=dist.ReduceOp.MAX)
        status = int(st[0])
        distinct = float((local_counts > 0).sum())
        bytes_call = layer_bytes(distinct, rows)
        pk = peaks()
        gbs = bytes_call * n_layers / (ms * 1e-3) / 1e9
        rec = {
            "ms_per_step": ms, "value": world * rows / (ms * 1e-3), "unit": "tokens/s", "steps": steps, "repeats": repeats,
            "exchange": mode, "status": status, "launches_per_layer_call": launches,
            "gpu_launches": (launches * n_layers * steps * repeats) if launches else None,
            "us_per_layer_call": ms * 1e3 / n_layers,
            "roofline": {"bound": "hbm", "kernel": "moe_decode_ep_kernel (per-GPU shard)" if mode == "fused"
                         else "expert_tc_kernel (per-GPU shard)", "achieved": gbs, "peak": pk["hbm_gbs"], "unit": "GB/s",
                         "frac": gbs / pk["hbm_gbs"], "traffic": None, "peak_source": pk["source"],
                         "bytes_per_launch": bytes_call, "distinct_local_experts_last_layer": distinct,
                         "note": "per-GPU fraction of rank 0: its shard's bytes per layer over the step time"},
            "load_imbalance": {"rows_per_gpu_last_layer": loads, "max_over_mean": max(loads) / max(sum(loads) / world, 1e-9)},
        }
        if mode == "exact":
            rec["exposed_communication"] = self.exposed_communication(states, xs, outs, rows, n_layers, ms)
        if mode in ("bulk", "gathered"):
            # event pairs inside the library around the parts of the layer: the exchange parts hold the peer stores
            # AND the wait for the slowest peer, i.e. everything a GPU spends not computing
            plan.stage_timing(True)
            self.timer.barrier()
            for _ in range(5 if mode == "bulk" else 2):
                for l in range(n_layers):
                    forward(l, xs[l], outs[l])
            stage_ms, calls = plan.stage_times()
            plan.stage_timing(False)
            if mode == "bulk":
                names = ("router", "dispatch_exchange", "permute_and_placement", "unused", "gate_up_swiglu", "down",
                         "return_exchange_and_combine")
            else:
                names = ("router", "dispatch_exchange", "routing_lists_after_all_ids", "placement_after_all_rows",
                         "gate_up_swiglu", "down", "return_exchange_and_combine")
            per_call = [v / calls * 1e3 for v in stage_ms.values()]
            stage_us = {n: self.timer.max_over_ranks(v) for n, v in zip(names, per_call) if n != "unused"}
            exchange = stage_us["dispatch_exchange"] + stage_us["return_exchange_and_combine"]
            if mode == "gathered":
                exchange += stage_us["routing_lists_after_all_ids"]
            rec["stage_us_max_over_ranks"] = stage_us
            rec["exposed_communication"] = {
                "wall_ms_per_step": ms, "exchange_us_per_layer": exchange, "compute_us_per_layer": sum(stage_us.values()) - exchange,
                "exposed_ms": exchange * n_layers * 1e-3,
                "definition": "per layer, max over ranks: peer stores of the dispatch + wait for every peer's rows, and peer stores of "
                              "the results + wait for every peer's results + the slot-order combine; nothing overlaps them in this "
                              "orchestration (stage times with a stream synchronisation per call, so they add up to a little more "
                              "than the wall time)"}
        if e2e:
            rec["e2e"] = self.e2e(mode, window, plan, biases, forward, xs, outs, rows, n_layers)
        if window is not None:
            self.timer.barrier()
            window.close()
            plan.close()
        return rec

    def exposed_communication(self, states, xs, outs, rows, n_layers, wall_ms) -> dict:
        """The exact-split NCCL orchestration again with an event after each part: compute = route + experts +
        combine (the library's kernels), the rest of the layer is the two exchanges with their host synchronisation.
        Exposed communication = wall time of the step - the slowest rank's compute."""
        torch, dist, ep = self.torch, self.dist, self.ep
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(6)]
        compute_ms, exchange_ms = 0.0, 0.0
        reps = 3
        for _ in range(reps):
            for l in range(n_layers):
                state, x, out = states[l], xs[l], outs[l]
                self.timer.barrier()
                ev[0].record()
                send, counts = state.route(x, rows)
                ev[1].record()
                counts_by_dst = counts.view(state.world, state.local).contiguous()
                recv, recv_counts, send_sizes, recv_sizes = ep.exchange_dispatch(send, counts_by_dst)
                ev[2].record()
                down = state.experts(recv, recv_counts, recv.shape[0])
                ev[3].record()
                returned = ep.exchange_return(down, send_sizes, recv_sizes)
                ev[4].record()
                state.combine(x, returned, out, rows)
                ev[5].record()
                torch.cuda.synchronize()
                compute_ms += ev[0].elapsed_time(ev[1]) + ev[2].elapsed_time(ev[3]) + ev[4].elapsed_time(ev[5])
                exchange_ms += ev[1].elapsed_time(ev[2]) + ev[3].elapsed_time(ev[4])
        compute = self.timer.max_over_ranks(compute_ms / reps)
        exchange = self.timer.max_over_ranks(exchange_ms / reps)
        return {"wall_ms_per_step": wall_ms, "compute_ms_max_over_ranks": compute,
                "exposed_ms": max(0.0, wall_ms - compute), "exchange_ms_when_bracketed": exchange,
                "definition": "wall - max over ranks of (route + experts + combine kernels); nothing overlaps the exchanges in this orchestration"}

    def e2e(self, mode, window, plan, biases, forward, xs, outs, rows, n_layers) -> dict:
        torch, ep = self.torch, self.ep
        host_in = [x.cpu().pin_memory() for x in xs]
        host_out = [torch.empty_like(h).pin_memory() for h in host_in]
        dev_in = [torch.empty_like(x) for x in xs]

        if mode == "fused":
            def one():
                for l in range(n_layers):
                    ep.forward_fused_host_async(window, plan, self.banks[l], self.routers[l], biases[l], host_in[l],
                                                host_out[l], rows)
                plan.host_flush()
                torch.cuda.current_stream().synchronize()
            call = "p92b_ep_forward_fused_host_async per layer (copies pipelined on the plan's streams), one flush + stream synchronisation per step"
        else:
            def one():
                for l in range(n_layers):
                    dev_in[l].copy_(host_in[l], non_blocking=True)
                    forward(l, dev_in[l], outs[l])
                    host_out[l].copy_(outs[l], non_blocking=True)
                torch.cuda.current_stream().synchronize()
            call = "host rows copied in and out on the stream around the layer calls, one synchronisation per step"
        self.timer.barrier()
        one()
        n = 10 if n_layers > 1 else 5
        self.timer.barrier()
        t0 = time.perf_counter()
        for _ in range(n):
            one()
        e2e_s = self.timer.max_over_ranks((time.perf_counter() - t0) / n)
        io = n_layers * rows * HIDDEN * 2
        return {"value": self.world * rows / e2e_s, "unit": "tokens/s", "h2d_bytes_per_step": io, "d2h_bytes_per_step": io,
                "ms_per_step": e2e_s * 1e3, "steps": n, "call": call, "bytes_are": "per GPU"}


def run_expert_parallel(args, torch, dist, pkg, synth, world, rank, local_rank, warmup, steps) -> None:
    headline = args.workload
    n_layers = args.layers or (1 if headline in ("prefill4096", "ep_prefill16384") else LAYERS)
    sampler = ClockSampler(local_rank) if rank == 0 else None
    job = ExpertParallel(torch, dist, pkg, synth, world, rank, n_layers)
    rec = job.run(headline, steps, warmup, args.min_seconds, sampler, e2e=True)
    clocks = sampler.stop() if sampler else None
    subs = {}
    if headline == "decode4x44" and not args.no_sub_records and n_layers == LAYERS:
        subs["ep_prefill16384"] = job.run("ep_prefill16384", 10, 3, 0.3)
        if world == 8:
            subs["ep_decode512"] = job.run("ep_decode512", 3, 3, 0.3)
        for name, sub in subs.items():
            sub["config"] = workload_config(name, world)
    status = max([rec["status"]] + [s["status"] for s in subs.values()])
    if rank == 0:
        line = {
            "metric": "moe_layer_tokens_per_s", "value": rec["value"], "unit": "tokens/s", "n_gpus": world, "steps": steps,
            "repeats": rec["repeats"], "warmup": warmup, "ms_per_step": rec["ms_per_step"], "higher_is_better": True,
            "scaling": "weak" if headline == "decode4x44" else "strong", "exchange": rec["exchange"], "vs_baseline": None,
            "dtype": DTYPE, "data": "synthetic", "config": workload_config(headline, world), "clocks": clocks,
            "e2e": rec.get("e2e"), "gpu_launches": rec["gpu_launches"], "roofline": rec["roofline"],
            "load_imbalance": rec["load_imbalance"], "cpu_baseline": None, "status": status,
            "us_per_layer_call": rec["us_per_layer_call"],
            "timed_region": f"{steps} steps x {rec['repeats']} repetitions inside one CUDA-event pair, max over ranks",
        }
        if "exposed_communication" in rec:
            line["exposed_communication"] = rec["exposed_communication"]
        if subs:
            line["configs"] = subs
        print(json.dumps(line))
    if status != 0:
        sys.exit(f"a kernel recorded status {status} (1: expert id out of range, 2: a bounded wait gave up)")


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="decode4x44", choices=sorted(WORKLOADS))
    ap.add_argument("--layers", type=int, default=None, help="override the layer count (debugging and small ncu captures)")
    ap.add_argument("--min-seconds", type=float, default=1.0, help="lower bound of the headline's timed region")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-sub-records", action="store_true")
    args = ap.parse_args()
    if args.impl == "reference":
        reference_arm(args)
        return

    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    if world > 1:
        if os.environ.get("NCCL_DEBUG", "").upper() == "VERSION":
            os.environ["NCCL_DEBUG"] = "WARN"         # the version banner goes to stdout, where only the JSON line belongs
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    warmup = max(args.warmup, 3)
    steps = max(args.steps, 1)

    pkg = entry.load_package()
    pkg.load_library()
    from p92moe_b200 import synth

    if world > 1:
        run_expert_parallel(args, torch, dist, pkg, synth, world, rank, local_rank, warmup, steps)
        dist.destroy_process_group()
    else:
        run_single_gpu(args, torch, pkg, synth, warmup, steps)


if __name__ == "__main__":
    main()
