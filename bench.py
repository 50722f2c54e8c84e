#!/usr/bin/env python
"""MoE-layer throughput benchmark (tokens/s) with roofline and CPU baseline.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload decode4x44|prefill4096|ep_prefill16384|ep_decode512]
    python bench.py --impl reference ...     # the CPU restatement of the reference's path

One "step" is one pass of the MoE block over one batch of synthetic tokens:
  decode4x44  (default, N=1): the MTP-verify step, T=4 tokens through all 44 MoE layers
               (layers 2..45), an independent weight set per layer (55 GB resident), so
               nothing a step touches is L2-resident when it is touched again.
  prefill4096: T=4096 tokens through one MoE layer, Zipf(1.2)-skewed routing.
  ep_prefill16384, ep_decode512: the expert-parallel configurations (T=16384 x 1 layer, uniform routing;
               T=512 x 44 layers, Zipf(1.0)); on one GPU they run the single-GPU block at that size.
Under torchrun (N > 1, one rank per GPU) the step is expert-parallel: 256/N experts per GPU, every GPU home to
its own tokens (decode: 4 per GPU, weak scaling; the others split their T over the GPUs).  Small batches take
the kernels that do their own exchanges over NVLink, large ones NCCL all-to-alls; P92B_EP_EXCHANGE=
fused|gathered|fixed|exact overrides the choice.
Rank 0 prints ONE JSON line.  `value` is device-timed with inputs resident in HBM; `e2e` is
the same metric through the host-buffer C-ABI call, host<->device copies inside the timed region.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

import __graft_entry__ as entry

HIDDEN, INTER, EXPERTS, TOP = 2560, 1024, 256, 8
EXPERT_BYTES = 3 * (INTER * HIDDEN // 2 + INTER * HIDDEN // 16)        # 4,423,680: packed + scales, 3 matrices
ROUTER_BYTES = EXPERTS * HIDDEN * 2 + EXPERTS * 4                      # 1,311,744
SEED = 20261125
LAYERS = 44


def peaks():
    path = os.path.join(entry.ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return {"hbm_gbs": float(p["hbm_gbs"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while a region runs (read-only)."""

    QUERY = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.rows = []
        self.proc = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={index}", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        self.marks = []

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
# reference arm: the CPU restatement of the reference's MoE forward on the host cores
# --------------------------------------------------------------------------------------------

class CpuLayer:
    """Synthetic layer on the host for the oracle: router/bias/activations, and NVFP4 experts that are
    drawn (N(0,0.02) -> BF16 -> the oracle's own restatement of the offline quantiser) only when
    a token is routed to them, since the expert weights do not influence routing."""

    def __init__(self, orc, layer: int, rows: int):
        self.orc = orc
        rng = np.random.default_rng([SEED, layer])
        self.router = orc.f32_to_bf16((rng.standard_normal((EXPERTS, HIDDEN)) * 0.02).astype(np.float32))
        self.bias = (rng.standard_normal(EXPERTS) * 0.01).astype(np.float32)
        self.x = orc.f32_to_bf16(rng.standard_normal((rows, HIDDEN)).astype(np.float32))
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


def run_cpu(args, rows: int, sample_layers: int, total_layers: int, steps: int, warmup: int) -> dict:
    orc = entry.load_oracle()
    cores = orc.cpu().orc_threads()
    layers = [CpuLayer(orc, l, rows) for l in range(sample_layers)]
    for _ in range(warmup):
        layers[0].forward()
    t0 = time.perf_counter()
    for _ in range(steps):
        for layer in layers:
            layer.forward()
    dt = (time.perf_counter() - t0) / steps
    step_time = dt * total_layers / sample_layers
    return {"value": rows / step_time, "ms_per_step": step_time * 1e3, "cores": cores,
            "sample": f"{sample_layers} of {total_layers} layers x {rows} tokens per step, {steps} steps, scaled by layer count"}


def reference_arm(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    rows, total_layers = (4, LAYERS) if args.workload == "decode4x44" else (4096, 1)
    if args.workload == "decode4x44":
        sample_layers, sample_rows = 2, rows
    else:
        sample_layers, sample_rows = 1, 16          # 16 of the 4096 tokens, scaled by token count
    steps = max(1, min(args.steps, 3))
    r = run_cpu(args, sample_rows, sample_layers, total_layers, steps, min(args.warmup, 1))
    value = r["value"]                              # tokens/s is per token whatever the sample size
    line = {
        "impl": "reference", "metric": "moe_layer_tokens_per_s", "value": value, "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": steps, "warmup": min(args.warmup, 1), "ms_per_step": r["ms_per_step"],
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "nvfp4 x nvfp4 -> f32 -> bf16",
        "data": "synthetic", "config": workload_config(args.workload, args.gpus),
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": r["cores"], "kind": "port",
                         "sample": r["sample"]},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


def workload_config(name: str, gpus: int) -> dict:
    if name == "decode4x44":
        return {"workload": "decode MTP-verify: T=4 tokens x 44 MoE layers (hidden 2560, 256+1 experts, FFN 1024, top-8)",
                "tokens_per_step": 4, "layers": LAYERS, "routing": "bias ~N(0,0.01)", "gpus": gpus,
                "l2": "44 distinct weight sets (55 GB) cycle per step: inputs larger than L2"}
    if name == "ep_decode512":
        return {"workload": "batched serving decode: T=512 tokens (128 sequences x 4 MTP positions) x 44 MoE layers, "
                            "Zipf(1.0) routing", "tokens_per_step": 512, "layers": LAYERS,
                "routing": "zipf 1.0 (capped at 1/8)", "gpus": gpus,
                "l2": "44 distinct weight sets cycle per step: inputs larger than L2"}
    if name == "ep_prefill16384":
        return {"workload": "expert-parallel prefill: T=16384 tokens x 1 MoE layer, uniform routing (bias 0)",
                "tokens_per_step": 16384, "layers": 1, "routing": "uniform", "gpus": gpus,
                "l2": "0.57-1.14 GB of weights per GPU per step: inputs larger than L2"}
    return {"workload": "prefill chunk: T=4096 tokens x 1 MoE layer, Zipf(1.2) routing", "tokens_per_step": 4096,
            "layers": 1, "routing": "zipf 1.2 (capped at 1/8)", "gpus": gpus,
            "l2": "1.14 GB of weights per step: inputs larger than L2"}


# --------------------------------------------------------------------------------------------
# our arm
# --------------------------------------------------------------------------------------------

def run_expert_parallel(args, pkg, synth, world, rank, local_rank, warmup, steps) -> None:
    """N > 1: the same step, expert-parallel.  Every GPU is home to its own tokens (weak scaling:
    4 tokens per GPU for the decode step, 4096/N... tokens per GPU for the prefill workloads), the 256
    experts are sharded 256/N per GPU.  Small batches take the fused kernel (exchanges by peer stores
    inside it), larger ones two NCCL all-to-alls per layer; P92B_EP_EXCHANGE=fused|fixed|exact overrides."""
    import torch
    import torch.distributed as dist
    from p92moe_b200 import ep

    decode = args.workload == "decode4x44"
    if decode:
        rows, n_layers = 4, args.layers or LAYERS
    elif args.workload == "ep_prefill16384":
        rows, n_layers = 16384 // world, args.layers or 1
    elif args.workload == "ep_decode512":
        rows, n_layers = 512 // world, args.layers or LAYERS
    else:
        rows, n_layers = 4096 // world, args.layers or 1
    first, local = ep.shard_range(rank, world)
    mode = os.environ.get("P92B_EP_EXCHANGE", "")
    if not mode:
        mode = "fused" if rows <= ep.FUSED_MAX_ROWS and world * rows <= ep.FUSED_MAX_TOKENS else \
            "gathered" if rows <= ep.GATHERED_MAX_ROWS and world * rows <= ep.GATHERED_MAX_TOKENS else "exact"
    window = fused_plan = None
    if mode in ("fused", "gathered"):
        # one window and one plan serve all layers.  If the windows cannot be mapped into one another (no
        # inter-process memory handles in this environment), every rank falls back to the NCCL orchestration.
        ok = 1
        try:
            window = ep.EpWindow(rank, world, rows)
            fused_plan = pkg.MoePlan(max_rows=world * rows)
        except Exception as exc:                                 # noqa: BLE001 - any failure means "no peer windows"
            ok = 0
            if rank == 0:
                print(f"peer windows unavailable ({exc}); using the NCCL exchange", file=sys.stderr)
        agreed = torch.tensor([ok], device="cuda")
        dist.all_reduce(agreed, op=dist.ReduceOp.MIN)
        if int(agreed[0]) == 0:
            window = fused_plan = None
            mode = "fixed" if rows <= ep.FIXED_MAX_ROWS else "exact"
    banks, routers, states, xs = [], [], [], []
    for l in range(n_layers):
        raw = synth.make_raw_layer(SEED, l)                     # same weights on every rank; keep the shard
        entries = raw.entries()
        shard = entries[first * 3:(first + local) * 3] + entries[EXPERTS * 3:]
        banks.append(pkg.ExpertBank(shard, first_expert=first, local_experts=local))
        routers.append(synth.make_router(SEED, l, bias_std=0.0 if args.workload == "ep_prefill16384" else 0.01))
        if args.workload in ("ep_decode512", "prefill4096"):
            alpha = 1.0 if args.workload == "ep_decode512" else 1.2
            routers[-1] = (routers[-1][0], synth.fit_zipf_bias(routers[-1][0], alpha, SEED + l)[0].contiguous())
        if mode in ("fixed", "exact"):
            states.append(ep.EpRank(rank, world, banks[-1], routers[-1][0], routers[-1][1], max_local_rows=rows,
                                    share_scratch_with=states[0] if states else None))
        xs.append(synth.make_activations(SEED + 1000 * (rank + 1), l, rows))
        del raw, entries, shard
    outs = [torch.empty_like(x) for x in xs]
    torch.cuda.synchronize()

    def forward(l, x, o):
        if mode == "fused":
            ep.forward_fused(window, fused_plan, banks[l], routers[l][0], routers[l][1], x, o, rows)
        elif mode == "gathered":
            ep.forward_gathered(window, fused_plan, banks[l], routers[l][0], routers[l][1], x, o, rows)
        elif mode == "fixed":
            ep.forward_nccl_fixed(states[l], x, o, rows, 8 * rows)
        else:
            ep.forward_nccl(states[l], x, o, rows)

    def step():
        for l in range(n_layers):
            forward(l, xs[l], outs[l])

    def barrier():
        dist.barrier()
        torch.cuda.synchronize()

    for _ in range(warmup):
        step()
    sampler = ClockSampler(local_rank) if rank == 0 else None
    barrier()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if sampler:
        sampler.mark()
    start.record()
    for _ in range(steps):
        step()
    stop.record()
    barrier()
    if sampler:
        sampler.mark()
    t = torch.tensor([start.elapsed_time(stop)], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_per_step = float(t[0]) / steps
    value = world * rows / (ms_per_step * 1e-3)

    # end to end: pinned host rows in, host rows out, per layer
    host_in = [x.cpu().pin_memory() for x in xs]
    host_out = [torch.empty_like(h).pin_memory() for h in host_in]
    dev_in = [torch.empty_like(x) for x in xs]
    e2e_steps = max(2, min(steps, 10))
    barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        for l, (hi, di, o, ho) in enumerate(zip(host_in, dev_in, outs, host_out)):
            di.copy_(hi, non_blocking=True)
            forward(l, di, o)
            ho.copy_(o, non_blocking=True)
            torch.cuda.current_stream().synchronize()
    e2e_s = (time.perf_counter() - t0) / e2e_steps
    t = torch.tensor([e2e_s], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    e2e_s = float(t[0])
    bytes_io = n_layers * rows * HIDDEN * 2

    step()
    torch.cuda.synchronize()
    count_plans = [fused_plan] if mode in ("fused", "gathered") else [states[-1].arrivals]
    local_counts = [pl.device_counts()[first:first + local].clone() for pl in count_plans]
    received = [int(c.sum()) for c in local_counts]
    load = torch.tensor([float(np.mean(received))], device="cuda")     # rows arriving per layer
    loads = [torch.zeros_like(load) for _ in range(world)]
    dist.all_gather(loads, load)
    loads = [float(v[0]) for v in loads]
    distinct = float(np.mean([int((c > 0).sum()) for c in local_counts]))
    layer_bytes = (distinct + 1) * EXPERT_BYTES + ROUTER_BYTES + rows * HIDDEN * 2 * 2
    pk = peaks()
    gbs = layer_bytes * n_layers / (ms_per_step * 1e-3) / 1e9
    if rank == 0:
        line = {
            "metric": "moe_layer_tokens_per_s", "value": value, "unit": "tokens/s", "n_gpus": world, "steps": steps,
            "warmup": warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "weak" if decode else "strong", "exchange": mode, "vs_baseline": None, "dtype": "nvfp4 x nvfp4 -> f32 -> bf16",
            "data": "synthetic", "config": dict(workload_config(args.workload, world),
                                                parallelism=f"ep{world}: {local} experts per GPU, {rows} home tokens per GPU, "
                                                            + {"fused": "one kernel per GPU and layer, dispatch (all-gather) and combine by peer stores "
                                                                        "over NVLink inside the kernel",
                                                               "gathered": "all-gather dispatch and direct placement of result rows by the "
                                                                           "library's own kernels (peer stores over NVLink, polled words), "
                                                                           "grouped tcgen05 products in between; no NCCL, no host sync",
                                                               "fixed": "NCCL all-to-all dispatch and combine, fixed-capacity blocks, "
                                                                        "no host sync",
                                                               "exact": "NCCL all-to-all dispatch and combine, exact-size splits"}[mode]),
            "clocks": sampler.stop(),
            "e2e": {"value": world * rows / e2e_s, "unit": "tokens/s", "h2d_bytes_per_step": bytes_io,
                    "d2h_bytes_per_step": bytes_io, "ms_per_step": e2e_s * 1e3},
            "gpu_launches": steps * n_layers * {"fused": 1, "gathered": 11, "fixed": 16, "exact": 16}[mode],
            "roofline": {"bound": "hbm", "kernel": "moe_decode_ep_kernel (per-GPU shard)" if mode == "fused"
                         else "expert_tc_kernel (per-GPU shard)", "achieved": gbs,
                         "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": gbs / pk["hbm_gbs"], "traffic": None,
                         "peak_source": pk["source"], "bytes_per_launch": layer_bytes,
                         "distinct_local_experts_mean": distinct},
            "load_imbalance": {"rows_per_gpu_per_layer": loads, "max_over_mean": max(loads) / (sum(loads) / world)},
            "cpu_baseline": None,
        }
        print(json.dumps(line))


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="decode4x44", choices=["decode4x44", "prefill4096", "ep_prefill16384", "ep_decode512"])
    ap.add_argument("--layers", type=int, default=None, help="override the layer count (debugging only)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
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
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    warmup = max(args.warmup, 3)
    steps = max(args.steps, 1)

    pkg = entry.load_package()
    pkg.load_library()
    from p92moe_b200 import synth

    if world > 1:
        run_expert_parallel(args, pkg, synth, world, rank, local_rank, warmup, steps)
        dist.destroy_process_group()
        return
    decode = args.workload == "decode4x44"       # the fused kernel: any workload of up to 8 rows
    rows = {"decode4x44": 4, "prefill4096": 4096, "ep_prefill16384": 16384, "ep_decode512": 512}[args.workload]
    n_layers = args.layers or (LAYERS if args.workload in ("decode4x44", "ep_decode512") else 1)
    bias_mode, alpha = {"decode4x44": ("normal", 0.0), "prefill4096": ("zipf", 1.2), "ep_prefill16384": ("zero", 0.0),
                        "ep_decode512": ("zipf", 1.0)}[args.workload]
    layers = [synth.make_layer(SEED + rank, l, bias_mode=bias_mode, zipf_alpha=alpha) for l in range(n_layers)]
    xs = [synth.make_activations(SEED + rank, l, rows) for l in range(n_layers)]
    outs = [torch.empty_like(x) for x in xs]
    plan = pkg.MoePlan(max_rows=rows)
    blocks = [pkg.MoeBlock(L.bank, L.router_weight, L.bias, plan) for L in layers]
    torch.cuda.synchronize()

    def step():
        for b, x, o in zip(blocks, xs, outs):
            b.run_moe_rows(x, o, rows)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(warmup):
        step()
    sampler = ClockSampler(local_rank) if rank == 0 else None
    barrier()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if sampler:
        sampler.mark()
    start.record()
    for _ in range(steps):
        step()
    stop.record()
    barrier()
    if sampler:
        sampler.mark()
    ms = start.elapsed_time(stop)
    launches = plan.last_launches * n_layers * steps
    if world > 1:
        t = torch.tensor([ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t[0])
    ms_per_step = ms / steps
    value = world * rows / (ms_per_step * 1e-3)

    # ---- end to end through the host-buffer C-ABI call (pinned host tensors) -----------------
    host_in = [x.cpu().pin_memory() for x in xs]
    host_out = [torch.empty_like(h).pin_memory() for h in host_in]
    e2e_steps = max(3, min(steps, 50))
    for b, hi, ho in zip(blocks, host_in, host_out):
        b.run_moe_rows_host(hi, ho, rows)
    barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        # every layer: pinned rows in, block, rows out, all enqueued; the step ends when its last rows are on the host
        for b, hi, ho in zip(blocks, host_in, host_out):
            b.run_moe_rows_host_async(hi, ho, rows)
        plan.host_flush()
        torch.cuda.current_stream().synchronize()
    e2e_s = (time.perf_counter() - t0) / e2e_steps
    e2e_sync_s = None
    if decode:
        # the same with the synchronising call (one stream synchronisation per layer), for comparison
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            for b, hi, ho in zip(blocks, host_in, host_out):
                b.run_moe_rows_host(hi, ho, rows)
        e2e_sync_s = (time.perf_counter() - t0) / e2e_steps
    if world > 1:
        t = torch.tensor([e2e_s], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_s = float(t[0])
    bytes_io = n_layers * rows * HIDDEN * 2
    e2e = {"value": world * rows / e2e_s, "unit": "tokens/s", "h2d_bytes_per_step": bytes_io,
           "d2h_bytes_per_step": bytes_io, "ms_per_step": e2e_s * 1e3,
           "call": "p92b_moe_forward_host_async per layer (copies pipelined on the plan's streams), one flush + stream synchronisation per step"}
    if e2e_sync_s is not None:
        e2e["ms_per_step_sync_per_layer"] = e2e_sync_s * 1e3

    # ---- per-stage device times (event pairs inside the library) and the roofline -------------
    plan.stage_timing(True)
    distinct = []
    timed_steps = max(2, min(steps, 20))
    for i in range(timed_steps):
        for b, x, o in zip(blocks, xs, outs):
            b.run_moe_rows(x, o, rows)
            if i == 0:
                distinct.append(int((plan.views(rows)["counts"] > 0).sum()))
    stage_ms, calls = plan.stage_times()
    plan.stage_timing(False)
    stage_us = {k: v / calls * 1e3 for k, v in stage_ms.items()}
    d_mean = float(np.mean(distinct))
    layer_bytes = (d_mean + 1) * EXPERT_BYTES + ROUTER_BYTES + rows * HIDDEN * 2 * 2
    pk = peaks()
    if decode:
        # the whole block is one kernel (moe_decode_kernel): its algorithmic bytes are the layer's
        # (D+1 experts x 3 matrices packed + scales, the router weight, the token rows in and out).
        # The timed region launches exactly one kernel per layer back to back on one stream, so the
        # average launch duration is the CUDA-event step time over the layer count (an event pair
        # around every single launch would break the overlap of consecutive launches)
        kernel, k_bytes, k_us = "moe_decode_kernel", layer_bytes, ms_per_step * 1e3 / n_layers
    else:
        # dominant kernel of the multi-kernel path: gate/up + SwiGLU + re-quantise
        kernel = "expert_gu_pair_kernel" if rows > 32 else "expert_tc_kernel<0,N>"
        k_bytes = (d_mean + 1) * 2 * (EXPERT_BYTES // 3) + rows * (HIDDEN // 2 + HIDDEN // 16) + \
            9 * rows * (INTER // 2 + INTER // 16)
        k_us = stage_us["gate_up_swiglu"]
    k_gbs = k_bytes / (k_us * 1e-6) / 1e9
    # DRAM traffic per launch: one ncu capture of this kernel (profiles/) measured read + write bytes at
    # 1.02 x the algorithmic bytes of its launches (decode) / 1.12 x (prefill gate/up); traffic grows with
    # the experts hit exactly as the algorithmic bytes do, so the ratio is applied to this run's bytes
    traffic = k_bytes * (1.02 if decode else 1.12)
    roofline = {"bound": "hbm", "kernel": kernel, "achieved": k_gbs, "peak": pk["hbm_gbs"],
                "unit": "GB/s", "frac": k_gbs / pk["hbm_gbs"], "traffic": traffic,
                "traffic_source": "ncu capture of a 3-layer case, scaled by algorithmic bytes", "peak_source": pk["source"],
                "bytes_per_launch": k_bytes, "us_per_launch": k_us, "layer_bytes": layer_bytes,
                "layer_frac_of_hbm": layer_bytes * n_layers / (ms_per_step * 1e-3) / 1e9 / pk["hbm_gbs"],
                "distinct_routed_experts_mean": d_mean, "stage_us": stage_us}

    if rank == 0:
        clocks = sampler.stop()
        cpu = None
        if not args.no_cpu_baseline:
            r = run_cpu(args, 4 if decode else 16, 2 if decode else 1, n_layers, 1, 1)
            cpu = {"value": r["value"], "unit": "tokens/s", "cores": r["cores"], "kind": "port", "sample": r["sample"]}
        line = {
            "metric": "moe_layer_tokens_per_s", "value": value, "unit": "tokens/s", "n_gpus": world, "steps": steps,
            "warmup": warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "nvfp4 x nvfp4 -> f32 -> bf16", "data": "synthetic",
            "config": workload_config(args.workload, world), "clocks": clocks, "e2e": e2e,
            "gpu_launches": launches, "roofline": roofline, "cpu_baseline": cpu,
        }
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
