#!/usr/bin/env python3
"""Benchmark of the quantized linear-layer path.

Headline workload (`decode_gemv_layer_q4km`): one step = the seven projections of one synthetic decoder
layer (hidden 5120, 40 q / 8 kv heads x 128, FFN 27648; Q4_K_M mix: Q6_K for attn_v and ffn_down, Q4_K
elsewhere) run as dequant-fused GEMVs for M = 1, 2, 4 and 8 tokens, in the order and grouping a decode step
issues them: q | k | v in one launch, o_proj, gate | up in one launch, down_proj: 16 kernel launches, 312 MB
of weights streamed four times.  The metric is algorithmic GB/s: (weight bytes + M*K*2 + M*N*4) summed over
the 28 projections, divided by device time.  With --gpus N > 1 the layer is tensor-parallel (column-parallel
q/k/v/gate/up, row-parallel o/down with an all-reduce after each), total work fixed.

The same JSON line carries the other configurations of the metric as objects of their own, each with its
roofline: `skinny` (the layer at 8 / 16 / 32 / 64 tokens), `prefill` (NVFP4 GEMMs at 2048 tokens, one GPU) and
`prefill_layers` (NVFP4 linears of whole layers at 32768 tokens, tensor-parallel at every N).

  python bench.py [--gpus N] [--steps K] [--warmup W]          this library on the GPU(s)
  python bench.py --impl reference ...                          the CPU reference lane (oracle) on host cores
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
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

METRIC = "decode_gemv_algorithmic_bandwidth"
UNIT = "GB/s"
WORKLOAD = "decode_gemv_layer_q4km"
TOKEN_COUNTS = (1, 2, 4, 8)
SKINNY_TOKENS = (8, 16, 32, 64)
KQ_BYTES_PER_256 = {12: 144, 14: 210}

# DRAM bytes of one step's 16 launches on one GPU: dram__bytes_read.sum + dram__bytes_write.sum summed over the 160
# kernel nodes of a ten-step graph replay, divided by ten (ncu, one capture of `bench.py --steps 10 --no-autotune`
# with the kernels of the commit "Evict-first L2 policy on the weight stream"; the launch plans came from the cost
# model).  1.005 x the algorithmic bytes: every weight byte crosses the DRAM interface once.
MEASURED_STEP_TRAFFIC_BYTES = 1260822810


def layer_projections():
    from muser_b200 import synth
    return synth.LAYER_PROJECTIONS


def call_bytes(n_in, n_out, dtype, m, x_bytes=2):
    return n_out * (n_in // 256) * KQ_BYTES_PER_256[dtype] + m * n_in * x_bytes + m * n_out * 4


def step_bytes(x_bytes=2):
    return sum(call_bytes(k, n, dt, m, x_bytes) for (k, n, dt) in layer_projections().values() for m in TOKEN_COUNTS)


def workload_config(world: int) -> dict:
    """What is computed, identical for both arms (how each arm runs it is reported beside it, under `run`)."""
    return {"workload": WORKLOAD, "tokens": list(TOKEN_COUNTS), "projections": list(layer_projections()),
            "weights": "Q4_K_M mix, seeded N(0,0.02)", "activations": "bf16 N(0,1)",
            "l2": "inputs larger than L2 (312 MB of weights per pass, 126 MB L2)",
            "parallelism": f"tp{world}" if world > 1 else "single"}


def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return float(d["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.samples, self._stop, self._t = index, [], threading.Event(), None

    def _run(self):
        while not self._stop.is_set():
            try:
                out = subprocess.run(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                                      "-i", str(self.index)], capture_output=True, text=True, timeout=5).stdout.strip()
                if out:
                    self.samples.append([f.strip() for f in out.splitlines()[0].split(",")])
            except Exception:
                pass
            self._stop.wait(0.05)

    def __enter__(self):
        self._t = threading.Thread(target=self._run, daemon=True)
        self._t.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        self._t.join(timeout=10)

    def summary(self):
        mhz = [int(s[0]) for s in self.samples if s[0].isdigit()]
        mx = [int(s[1]) for s in self.samples if len(s) > 1 and s[1].isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({names[i] for s in self.samples for i in range(4) if len(s) > 2 + i and s[2 + i] == "Active"})
        return {"sm_mhz": int(statistics.median(mhz)) if mhz else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(self.samples),
                "window": "0.5 s of the same step replays right before the timed region, and the timed region"}


# ----------------------------------------------------------------------------------- reference arm
def run_reference(args):
    """The reference's CPU lane (weights::matmul restated in oracle/) on all host cores of this box."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import numpy as np
    import torch
    from muser_b200 import synth
    from oracle import oracle as O
    threads = O.host_threads()
    weights = {}
    for i, (name, (k, n, dt)) in enumerate(layer_projections().items()):
        raw = synth.quantize_kquant(synth.normal_weights(n, k, seed=0, stream=i), dt).numpy()
        weights[name] = O.TensorView(raw, dt, k, n)
    xs = {(name, m): synth.normal_activations(m, k, seed=0, stream=1000 + i).float().numpy()
          for i, (name, (k, n, dt)) in enumerate(layer_projections().items()) for m in TOKEN_COUNTS}
    bytes_per_step = step_bytes(2)  # same accounting as the GPU arm (the lane itself reads f32 activations)

    def step():
        for name in weights:
            for m in TOKEN_COUNTS:
                O.matmul(weights[name], xs[(name, m)], threads=threads)

    warmup = max(args.warmup, 3)
    for _ in range(warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    dt = time.perf_counter() - t0
    value = bytes_per_step * args.steps / dt / 1e9
    sample = "one full step: 7 projections x M in {1,2,4,8}, f32 activations, all host threads"
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": warmup, "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(args.gpus),
        "run": {"sample": sample, "note": "CPU restatement of weights::matmul (oracle/), not the GPU"},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }))


# ----------------------------------------------------------------------------------- GPU arm
def run_gpu(args):
    import numpy as np
    import torch
    import torch.distributed as dist
    from muser_b200 import operator as op
    from muser_b200 import synth, tp, workloads

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    plan = tp.ShardPlan(rank, world)
    ctx = op.Context(local_rank, workspace_bytes=256 << 20)
    kern = op.CudaKernels(ctx)
    collective = tp.Collective(ctx, rank, world) if world > 1 else None
    all_reduce = collective.all_reduce_sum if collective else None

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # weights: seeded N(0, 0.02), quantized on the device, repacked into this rank's shard
    projs = layer_projections()
    tokens_all = sorted(set(TOKEN_COUNTS) | set(SKINNY_TOKENS))
    layer = workloads.DecodeLayer(ctx, kern, plan, tokens_all, dev, all_reduce=all_reduce, autotune=not args.no_autotune,
                                  fuse_all_reduce=bool(collective and collective.oneshot and not args.no_fused_all_reduce))
    launches_per_step = layer.launches_per_pass * len(TOKEN_COUNTS)

    def step():
        for m in TOKEN_COUNTS:
            layer.run(m)

    warmup = max(args.warmup, 3)
    for _ in range(warmup):
        step()
    barrier()
    ctx.sync_status()

    # parity of the tensor-parallel path: sampled rows of the all-reduced row-parallel outputs against the CPU lane
    # on the UNSHARDED tensors (rank 0 checks; every rank's partial sums are in what it checks)
    tp_rel_l2 = None
    if world > 1 and not args.no_cpu:
        layer.run(8)
        torch.cuda.synchronize()
        if rank == 0:
            from oracle import oracle as O
            errs = {}
            for gi, name in ((1, "attn_o"), (3, "ffn_down")):
                k, n, dt = projs[name]
                rows = np.sort(np.random.default_rng(7).choice(n, 96, replace=False))
                sub = layer.views[name].raw.cpu().numpy().reshape(n, -1)[rows].copy()
                ref = O.matmul(O.TensorView(sub, dt, k, len(rows)), layer.full_input(gi, 8).float().cpu().numpy(), threads=O.host_threads())
                got = layer.y[(name, 8)][:, torch.from_numpy(rows).to(dev)].cpu().numpy()
                errs[name] = float(np.linalg.norm(got - ref) / np.linalg.norm(ref))
            tp_rel_l2 = errs
            if max(errs.values()) > 1e-3:
                print(f"tensor-parallel outputs differ from the CPU lane: {errs}", file=sys.stderr, flush=True)
                os._exit(3)
        barrier()

    # The launches of a step are microseconds each: replay them as one CUDA graph so that the device, not the
    # host's launch rate, is what gets timed.  (Capture falls back to plain launches if a collective refuses it.)
    run_step, graphed = step, False
    per_graph = 1  # steps per graph replay: the largest divisor of --steps up to 10, so that exactly --steps steps are timed
    if not args.no_graph:
        per_graph = max(d for d in range(1, 11) if args.steps % d == 0)

        def steps_chunk():
            for _ in range(per_graph):
                step()

        try:
            run_step, graphed = workloads.capture(steps_chunk), True
        except Exception as exc:  # pragma: no cover - depends on the collective in use
            print(f"graph capture unavailable ({type(exc).__name__}: {exc}); timing plain launches", file=sys.stderr)
            torch.cuda.synchronize()
            per_graph = 1
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local_rank) as clocks:
        # The timed region can be a few milliseconds, less than one nvidia-smi query: the sampler therefore also
        # covers ~0.5 s of the same replays immediately before it (same kernels, same load), all untimed.
        lead = time.time()
        while time.time() - lead < args.lead_seconds:
            for _ in range(10):
                run_step()
            torch.cuda.synchronize()
        barrier()
        start.record()
        for _ in range(args.steps // per_graph):
            run_step()
        stop.record()
        barrier()
    ms = start.elapsed_time(stop)
    if world > 1:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    ctx.sync_status()
    total_bytes = step_bytes(2) * args.steps
    value = total_bytes / (ms * 1e-3) / 1e9
    peak, peak_kind = measured_peaks()

    # per-launch device times (secondary detail): each launch of the step alone, rotating over enough copies of its
    # weights that they never sit in L2, replayed as a CUDA graph; without the collective
    detail = {}
    if rank == 0 and not args.no_detail:
        saved, layer.all_reduce = layer.all_reduce, None
        for gi, group in enumerate(layer.GROUPS):
            nbytes_w = sum(layer.views[n].raw.numel() for n in group) // world
            copies = [[op.Weight(ctx, layer.views[n], shard=plan.shard(n)) for n in group]
                      for _ in range(max(2, min(12, (300 << 20) // nbytes_w + 1)))]
            for m in TOKEN_COUNTS:
                us = workloads.rotating_call_seconds(lambda i: layer.launch_group(gi, m, copies[i]), len(copies)) * 1e6
                b = sum(workloads.kquant_call_bytes(layer.weights[n].n_in, layer.weights[n].n_out, projs[n][2], m) for n in group)
                detail[f"{'|'.join(group)}_m{m}"] = {"us": round(us, 2), "gbs": round(b / max(us, 1e-3) / 1e3, 1)}
            for c in copies:
                for w in c:
                    w.free()
        layer.all_reduce = saved
    if world > 1:
        barrier()

    # config 5: the same layer at the speculative-verify token counts
    skinny = None
    if not args.no_skinny:
        per_m = {}
        for m in SKINNY_TOKENS:
            run_m = workloads.capture(lambda: layer.run(m)) if graphed else (lambda: layer.run(m))
            for _ in range(3):
                run_m()
            barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(20):
                run_m()
            e1.record()
            barrier()
            t_ms = e0.elapsed_time(e1) / 20
            if world > 1:
                tt = torch.tensor([t_ms], device=dev)
                dist.all_reduce(tt, op=dist.ReduceOp.MAX)
                t_ms = float(tt.item())
            gbs, tfl = layer.pass_bytes(m) / (t_ms * 1e-3) / 1e9, layer.pass_flops(m) / (t_ms * 1e-3) / 1e12
            per_m[str(m)] = {"us": round(t_ms * 1e3, 2), "gbs": round(gbs, 1), "tflops": round(tfl, 2), "frac": round(gbs / (peak * world), 4)}
        ctx.sync_status()
        skinny = {"workload": "skinny_verify_layer_q4km", "tokens": list(SKINNY_TOKENS), "per_tokens": per_m,
                  "note": "one pass over the layer's 7 projections per token count (4 launches up to 16 tokens, 7 beyond); "
                          "GB/s over the algorithmic bytes (weights stream once per pass), TFLOP/s = 2 M N K",
                  "roofline": {"bound": "hbm", "unit": "GB/s", "peak": peak * world, "peak_kind": f"of {peak_kind}",
                               "achieved": per_m[str(SKINNY_TOKENS[0])]["gbs"], "frac": per_m[str(SKINNY_TOKENS[0])]["frac"],
                               "at_tokens": SKINNY_TOKENS[0]}}

    # end to end through the host-buffer entry point (weights::matmul's signature, the wait once per step): pinned
    # f32 host x in, f32 host y out, host<->device copies inside the timed region
    e2e = None
    if rank == 0 and world == 1 and not args.no_e2e:
        hx = {(gi, m): synth.normal_activations(m, layer.weights[group[0]].n_in, seed=0, stream=2000 + gi).float().pin_memory()
              for gi, group in enumerate(layer.GROUPS) for m in TOKEN_COUNTS}
        hy = {(name, m): torch.empty((m, layer.weights[name].n_out), dtype=torch.float32).pin_memory() for name in projs for m in TOKEN_COUNTS}
        # the step's call list, built once as a driver would: per token count the four launches of the decode step, each
        # group's projections reading one host x and writing their own host y
        calls = op.host_groups([([layer.weights[n] for n in group], hx[(gi, m)].data_ptr(), m, [hy[(n, m)].data_ptr() for n in group])
                                for m in TOKEN_COUNTS for gi, group in enumerate(layer.GROUPS)])
        stream = torch.cuda.current_stream().cuda_stream
        if args.host_output_mode is not None:
            from muser_b200._lib import TUNE_HOST_DIRECT_OUTPUT
            ctx.tuning_set(TUNE_HOST_DIRECT_OUTPUT, args.host_output_mode)

        def e2e_step():
            op.matmul_groups_enqueue(ctx, calls, stream)
            ctx.sync_status()  # the step's one wait; also folds device-side give-ups into an exception

        def timed(step_fn):
            for _ in range(3):
                step_fn()
            t0 = time.perf_counter()
            for _ in range(e2e_steps):
                step_fn()
            return time.perf_counter() - t0

        e2e_steps = max(3, min(args.steps, 50))
        dt_plain = timed(e2e_step)
        # the same call captured once into a CUDA graph (the counterpart of a pre-encoded command buffer): the copies
        # of x, the launches and the stores of y replay from the same pinned host buffers every step
        replay = workloads.capture(lambda: op.matmul_groups_enqueue(ctx, calls, torch.cuda.current_stream().cuda_stream))

        def e2e_graph_step():
            replay()
            ctx.sync_status()

        for h in hy.values():
            h.fill_(float("nan"))
        dt_e2e = timed(e2e_graph_step)
        name, m = "ffn_down", 8
        ref_dev = torch.empty((m, layer.weights[name].n_out), dtype=torch.float32, device=dev)
        kern.encode_quantized_matmul(layer.weights[name], hx[(3, m)].to(dev), ref_dev, m)
        e2e_check = float((hy[(name, m)] - ref_dev.cpu()).norm() / ref_dev.cpu().norm())
        dt_best = min(dt_e2e, dt_plain)  # both are the public call with host buffers; a user takes the faster way to issue it
        e2e = {"value": step_bytes(4) * e2e_steps / dt_best / 1e9, "unit": UNIT,
               "h2d_bytes_per_step": sum(m * layer.weights[group[0]].n_in * 4 for group in layer.GROUPS for m in TOKEN_COUNTS),
               "d2h_bytes_per_step": sum(m * layer.weights[name].n_out * 4 for name in projs for m in TOKEN_COUNTS),
               "ms_per_step": dt_best / e2e_steps * 1e3, "ms_per_step_graph_replay": dt_e2e / e2e_steps * 1e3,
               "ms_per_step_without_graph": dt_plain / e2e_steps * 1e3,
               "rel_l2_vs_device_call": e2e_check,
               "note": "muser_cuda_matmul_host_groups_enqueue (16 groups per step: pinned f32 host x copied up once per group on "
                       "a copy stream, one launch per group, each f32 y copied into its pinned host buffer on the copy stream "
                       "beside the next launches) + one muser_cuda_sync_status per step; wall clock around the steps; issued "
                       "anew every step (ms_per_step_without_graph) and captured once into a CUDA graph and replayed "
                       "(ms_per_step_graph_replay); value and ms_per_step are the faster of the two"}
    elif rank == 0 and world > 1:
        e2e = {"value": None, "unit": UNIT, "h2d_bytes_per_step": None, "d2h_bytes_per_step": None,
               "note": "not measured at N > 1: the host-buffer entry point runs one rank's shard without the all-reduce"}

    # second half of the metric: NVFP4 prefill GEMM, M = 2048, the same layer's shapes (N = 1 only); not part of `value`
    prefill = None
    if rank == 0 and world == 1 and not args.no_prefill:
        prefill = prefill_section(ctx, kern, op, synth, projs, dev, torch)

    # config 4: the NVFP4 linears of whole layers at 32768 tokens, tensor-parallel at every N
    prefill_layers = None
    if not args.no_prefill and args.prefill_layers > 0:
        M, L = args.prefill_tokens, args.prefill_layers
        pctx = op.Context(local_rank, workspace_bytes=workloads.PrefillLayer.workspace_bytes(M, world))
        pkern = op.CudaKernels(pctx)
        pcoll = tp.Collective(pctx, rank, world) if world > 1 else None
        pl = workloads.PrefillLayer(pctx, pkern, plan, M, dev, all_reduce=pcoll.all_reduce_sum if pcoll else None, chunks=args.chunks)
        pl.layer(pl.h)
        pctx.sync_status()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        pl.run(L)
        e1.record()
        barrier()
        pms = e0.elapsed_time(e1)
        if world > 1:
            tt = torch.tensor([pms], device=dev)
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
            pms = float(tt.item())
        pctx.sync_status()
        finite = bool(torch.isfinite(pl.h2.float()).all())
        tfl = pl.flops(L) / (pms * 1e-3) / 1e12
        peak_fp4 = (prefill or {}).get("roofline", {}).get("peak") or op.fp4_peak_tflops(pctx)
        prefill_layers = {"workload": "nvfp4_prefill_linears", "tokens": M, "layers": L, "of_layers": 52, "ms": round(pms, 2),
                          "ms_per_layer": round(pms / L, 3), "tflops": round(tfl, 1), "unit": "TFLOP/s", "parallelism": f"tp{world}" if world > 1 else "single",
                          "chunks": len(pl.bounds), "finite": finite,
                          "note": "input norms fused into the activation quantizer, SwiGLU into the gate/up GEMM, residuals into the o / down "
                                  "epilogues, attention excluded, all-reduce after o_proj and down_proj; every layer reuses one layer's weights "
                                  "(274 MB, larger than L2); whole-job TFLOP/s, max over ranks",
                          "roofline": {"bound": "tensor", "achieved": round(tfl, 1), "peak": round(peak_fp4 * world, 1), "unit": "TFLOP/s",
                                       "frac": round(tfl / (peak_fp4 * world), 4),
                                       "peak_kind": "measured here: muser_cuda_fp4_peak_probe (block-scaled FP4 MMAs, no memory traffic)"}}
        del pl
        pctx.close()

    # CPU lane on this box's host cores, bounded sample (N = 1 only)
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        from oracle import oracle as O
        threads = O.host_threads()
        name, m = "ffn_gate", 1
        k, n, dt = projs[name]
        ow = O.TensorView(layer.views[name].raw.cpu().numpy(), dt, k, n)
        x1 = layer.x[(2, m)]
        xin = x1.float().cpu().numpy()
        O.matmul(ow, xin, threads=threads)
        reps, t0 = 0, time.perf_counter()
        while time.perf_counter() - t0 < 10.0 and reps < 200:
            ref = O.matmul(ow, xin, threads=threads)
            reps += 1
        dt_cpu = (time.perf_counter() - t0) / reps
        y1 = torch.empty((m, n), dtype=torch.float32, device=dev)
        kern.encode_quantized_matmul(layer.weights[name], x1, y1, m)
        rel = float(np.linalg.norm(y1.cpu().numpy() - ref) / np.linalg.norm(ref))
        cpu = {"value": call_bytes(k, n, dt, m, 4) / dt_cpu / 1e9, "unit": UNIT, "cores": threads, "kind": "port",
               "sample": f"{name} (Q4_K {k}->{n}), M=1, {reps} repetitions of weights::matmul restated in C",
               "gpu_vs_cpu_rel_l2": rel}

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": warmup,
            "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic",
            "config": workload_config(world),
            "run": {"launch": f"CUDA graph replays of {per_graph} step(s) each" if graphed else "plain launches",
                    "schedule": "per token count: q|k|v grouped, o, gate|up grouped, down; one stream",
                    "collective": collective.kind if collective else None,
                    "row_parallel": ("projection kernel pushes its partial sums to the peers, a second kernel gathers" if layer.fuse_all_reduce
                                     else "projection, then all-reduce") if collective else None},
            "roofline": {"bound": "hbm", "achieved": value, "peak": peak * world, "unit": "GB/s", "frac": value / (peak * world),
                         "traffic": MEASURED_STEP_TRAFFIC_BYTES if world == 1 else None, "traffic_per": f"step ({launches_per_step} launches)",
                         "algorithmic_bytes_per_step": step_bytes(2), "peak_kind": f"of {peak_kind}",
                         "kernel": "kquant_decode_kernel (the 16 launches of a step; achieved = all their bytes / all their time)"},
            "cpu_baseline": cpu,
            "e2e": e2e,
            "gpu_launches": launches_per_step * args.steps,
            "clocks": clocks.summary(),
            "detail_us": detail,
            "skinny": skinny,
            "prefill": prefill,
            "prefill_layers": prefill_layers,
            "tp_rel_l2": tp_rel_l2,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        # Leave without tearing the process group down: ranks finish at different times, and a teardown that waits
        # for a peer that is already gone never returns.
        torch.cuda.synchronize()
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(0)


def prefill_section(ctx, kern, op, synth, projs, dev, torch):
    """NVFP4 GEMMs of the layer's shapes at 2048 tokens on one GPU, with the FP4 tensor peak measured in the same run."""
    from muser_b200._lib import NVFP4
    m = 2048
    peak_fp4 = op.fp4_peak_tflops(ctx)
    per, tot_fl, tot_s = {}, 0.0, 0.0
    for i, (name, (k, n, _)) in enumerate(projs.items()):
        wp, ws, s2 = synth.nvfp4_weight(synth.normal_weights(n, k, seed=0, stream=i, device=dev))
        xa = synth.normal_activations(m, k, seed=0, stream=3000 + i, device=dev)
        isi = synth.activation_input_scale_inv(xa)
        wq = op.Weight(ctx, op.TensorView(wp, NVFP4, k, n, ws, s2, isi))
        yq = torch.empty((m, n), dtype=torch.bfloat16, device=dev)
        xp, xs = kern.quantize_nvfp4_activation(xa, isi)
        for _ in range(3):
            kern.encode_nvfp4_prequant(wq, xp, xs, yq, m)
        e0, e1, e2 = (torch.cuda.Event(enable_timing=True) for _ in range(3))
        reps = 5
        e0.record()
        for _ in range(reps):
            kern.encode_nvfp4_prequant(wq, xp, xs, yq, m)
        e1.record()
        for _ in range(reps):
            kern.encode_nvfp4_matmul(wq, xa, yq, m)   # quantize + GEMM, as the operator is called
        e2.record()
        torch.cuda.synchronize()
        ctx.sync_status()
        t_gemm, t_full = e0.elapsed_time(e1) / reps * 1e-3, e1.elapsed_time(e2) / reps * 1e-3
        fl = 2.0 * m * n * k
        per[name] = {"gemm_tflops": round(fl / t_gemm / 1e12, 1), "with_quantize_tflops": round(fl / t_full / 1e12, 1)}
        tot_fl, tot_s = tot_fl + fl, tot_s + t_gemm
        wq.free()
        del wp, ws, xa, yq, xp, xs
    layer_tfl = tot_fl / tot_s / 1e12

    fused = {}
    try:
        def timed(fn, reps=5):
            for _ in range(2):
                fn()
            t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            t0.record()
            for _ in range(reps):
                fn()
            t1.record()
            torch.cuda.synchronize()
            ctx.sync_status()
            return t0.elapsed_time(t1) / reps * 1e-3

        names = list(projs)
        k_h = projs["attn_q"][0]
        xa = synth.normal_activations(m, k_h, seed=0, stream=3100, device=dev)
        isi = synth.activation_input_scale_inv(xa)
        xp, xs = kern.quantize_nvfp4_activation(xa, isi)
        n_f = projs["ffn_gate"][1]
        gu = [synth.nvfp4_weight(synth.normal_weights(n_f, k_h, seed=0, stream=names.index(nm), device=dev)) for nm in ("ffn_gate", "ffn_up")]
        w_g, w_u = (op.Weight(ctx, op.TensorView(p[0], NVFP4, k_h, n_f, p[1], p[2], isi)) for p in gu)
        y_f = torch.empty((m, n_f), dtype=torch.bfloat16, device=dev)
        t = timed(lambda: kern.encode_nvfp4_ffn_gate_up_silu_prequant(w_g, w_u, xp, xs, y_f, m))
        fused["ffn_gate|up+swiglu"] = {"gemm_tflops": round(2.0 * m * 2 * n_f * k_h / t / 1e12, 1)}
        w_g.free()
        w_u.free()
        # q | k | v on the same activations in one launch (muser_cuda_nvfp4_matmul_group_prequant)
        qkv = []
        for nm in ("attn_q", "attn_k", "attn_v"):
            n_p = projs[nm][1]
            p = synth.nvfp4_weight(synth.normal_weights(n_p, k_h, seed=0, stream=names.index(nm), device=dev))
            qkv.append((op.Weight(ctx, op.TensorView(p[0], NVFP4, k_h, n_p, p[1], p[2], isi)), torch.empty((m, n_p), dtype=torch.bfloat16, device=dev)))
        t = timed(lambda: kern.encode_nvfp4_group_prequant([w for w, _ in qkv], xp, xs, [y for _, y in qkv], m))
        fl_qkv = 2.0 * m * sum(projs[nm][1] for nm in ("attn_q", "attn_k", "attn_v")) * k_h
        fused["attn_q|k|v"] = {"gemm_tflops": round(fl_qkv / t / 1e12, 1)}
        # the layer as a caller would launch it: q | k | v grouped, the other four as measured above
        t_rest = sum(2.0 * m * projs[nm][0] * projs[nm][1] / (per[nm]["gemm_tflops"] * 1e12) for nm in ("attn_o", "ffn_gate", "ffn_up", "ffn_down"))
        fused["layer_with_q|k|v_grouped"] = {"gemm_tflops": round(tot_fl / (t + t_rest) / 1e12, 1)}
        for w, _ in qkv:
            w.free()
    except Exception as exc:  # the secondary section must never cost the headline line
        fused = {"error": f"{type(exc).__name__}: {exc}"}

    roofline = {"bound": "tensor", "achieved": round(layer_tfl, 1), "peak": round(peak_fp4, 1), "unit": "TFLOP/s",
                "frac": round(layer_tfl / peak_fp4, 4),
                "peak_kind": "measured here: muser_cuda_fp4_peak_probe (block-scaled FP4 MMAs, no memory traffic)"}
    grouped = fused.get("layer_with_q|k|v_grouped") if isinstance(fused, dict) else None
    if isinstance(grouped, dict) and "gemm_tflops" in grouped and peak_fp4 > 0:
        # the seven projections launched one by one are the figure above; a caller issues q | k | v as one launch
        roofline["frac_with_q|k|v_grouped"] = round(grouped["gemm_tflops"] / peak_fp4, 4)
    return {"workload": "nvfp4_prefill_gemm_layer_m2048", "unit": "TFLOP/s", "layer": round(layer_tfl, 1),
            "per_projection": per, "fused": fused, "roofline": roofline}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU-lane legs (baseline, tensor-parallel parity)")
    ap.add_argument("--no-detail", action="store_true", help="skip the per-launch timings")
    ap.add_argument("--no-skinny", action="store_true", help="skip the 8/16/32/64-token section")
    ap.add_argument("--no-prefill", action="store_true", help="skip the NVFP4 prefill sections")
    ap.add_argument("--prefill-layers", type=int, default=4, help="layers of the 52 that the prefill_layers section runs")
    ap.add_argument("--prefill-tokens", type=int, default=32768)
    ap.add_argument("--chunks", type=int, default=4, help="token chunks per row-parallel projection in prefill_layers (N > 1)")
    ap.add_argument("--no-graph", action="store_true", help="launch the step's kernels one by one instead of as a CUDA graph")
    ap.add_argument("--no-e2e", action="store_true", help="skip the end-to-end leg through host buffers")
    ap.add_argument("--host-output-mode", type=int, default=None, choices=[0, 1, 2],
                    help="e2e leg: how outputs reach the host buffers (MUSER_TUNE_HOST_DIRECT_OUTPUT); default: the library's")
    ap.add_argument("--no-fused-all-reduce", action="store_true", help="N > 1: projection, then all-reduce, as two calls")
    ap.add_argument("--no-autotune", action="store_true", help="launch plans from the cost model alone (no measuring at load time)")
    ap.add_argument("--lead-seconds", type=float, default=0.5, help="untimed replays under the clock sampler right before the timed region")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_gpu(args)


if __name__ == "__main__":
    main()
