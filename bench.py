#!/usr/bin/env python3
"""Benchmark of the quantized linear-layer path.

Headline workload (`decode_gemv_layer_q4km`): one step = the seven projections of one synthetic decoder
layer (hidden 5120, 40 q / 8 kv heads x 128, FFN 27648; Q4_K_M mix: Q6_K for attn_v and ffn_down, Q4_K
elsewhere) run as dequant-fused GEMVs for M = 1, 2, 4 and 8 tokens: 28 kernel launches, 312 MB of weights
streamed four times.  The metric is algorithmic GB/s: (weight bytes + M*K*2 + M*N*4) summed over the calls,
divided by device time.  With --gpus N > 1 the layer is tensor-parallel (column-parallel q/k/v/gate/up,
row-parallel o/down with an NCCL all-reduce after each), total work fixed.

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
KQ_BYTES_PER_256 = {12: 144, 14: 210}


def layer_projections():
    from muser_b200 import synth
    return synth.LAYER_PROJECTIONS


def call_bytes(n_in, n_out, dtype, m, x_bytes=2):
    return n_out * (n_in // 256) * KQ_BYTES_PER_256[dtype] + m * n_in * x_bytes + m * n_out * 4


def step_bytes(x_bytes=2):
    return sum(call_bytes(k, n, dt, m, x_bytes) for (k, n, dt) in layer_projections().values() for m in TOKEN_COUNTS)


def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return float(d["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


MEASURED_STEP_TRAFFIC_BYTES = 1262834688  # one GPU, one step, from the ncu capture named beside its use


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
    sample_tokens = TOKEN_COUNTS  # the whole step; the CPU lane finishes it in about a second on a server host
    weights = {}
    for i, (name, (k, n, dt)) in enumerate(layer_projections().items()):
        raw = synth.quantize_kquant(synth.normal_weights(n, k, seed=0, stream=i), dt).numpy()
        weights[name] = O.TensorView(raw, dt, k, n)
    xs = {(name, m): synth.normal_activations(m, k, seed=0, stream=1000 + i).float().numpy()
          for i, (name, (k, n, dt)) in enumerate(layer_projections().items()) for m in sample_tokens}
    bytes_per_step = step_bytes(2)  # same accounting as the GPU arm (the lane itself reads f32 activations)

    def step():
        for name in weights:
            for m in sample_tokens:
                O.matmul(weights[name], xs[(name, m)], threads=threads)

    for _ in range(min(args.warmup, 1)):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    dt = time.perf_counter() - t0
    value = bytes_per_step * args.steps / dt / 1e9
    sample = "one full step: 7 projections x M in {1,2,4,8}, f32 activations, all host threads"
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": min(args.warmup, 1), "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "sample": sample, "note": "CPU restatement of weights::matmul (oracle/), not the GPU"},
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
    from muser_b200 import synth, tp

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

    # weights: seeded N(0, 0.02), quantized on the device, repacked into this rank's shard
    projs = layer_projections()
    weights, views = {}, {}
    for i, (name, (k, n, dt)) in enumerate(projs.items()):
        raw = synth.quantize_kquant(synth.normal_weights(n, k, seed=0, stream=i, device=dev), dt)
        views[name] = op.TensorView(raw, dt, k, n)
        weights[name] = op.Weight(ctx, views[name], shard=plan.shard(name))
    x_dev, y_dev = {}, {}
    for i, (name, (k, n, dt)) in enumerate(projs.items()):
        for m in TOKEN_COUNTS:
            x = synth.normal_activations(m, k, seed=0, stream=1000 + i, device=dev)
            x_dev[(name, m)] = x[:, plan.input_slice(name, k)].contiguous()
            y_dev[(name, m)] = torch.empty((m, weights[name].n_out), dtype=torch.float32, device=dev)
    launches_per_step = len(projs) * len(TOKEN_COUNTS)

    # The projections of a layer that read the same input are independent: q | k | v, and gate | up.  They go to
    # parallel streams (one context each: a context's split-K scratch serves one stream at a time; weight handles are
    # shared), joined before o_proj and before down_proj, which is the order a decoder layer imposes.
    parallel = not args.serial
    side_ctx = [op.Context(local_rank, workspace_bytes=1 << 20) for _ in range(2)] if parallel else []
    side_kern = [op.CudaKernels(c) for c in side_ctx]
    side_stream = [torch.cuda.Stream() for _ in side_ctx]

    def launch(name, m, k):
        k.encode_quantized_matmul(weights[name], x_dev[(name, m)], y_dev[(name, m)], m)
        if plan.needs_all_reduce(name):
            tp.all_reduce_sum(y_dev[(name, m)])

    def step():
        if not parallel:
            for m in TOKEN_COUNTS:
                for name in projs:
                    launch(name, m, kern)
            return
        main = torch.cuda.current_stream()
        for m in TOKEN_COUNTS:
            for s_ in side_stream:
                s_.wait_stream(main)
            launch("attn_q", m, kern)
            with torch.cuda.stream(side_stream[0]):
                launch("attn_k", m, side_kern[0])
            with torch.cuda.stream(side_stream[1]):
                launch("attn_v", m, side_kern[1])
            for s_ in side_stream:
                main.wait_stream(s_)
            launch("attn_o", m, kern)
            side_stream[0].wait_stream(main)
            launch("ffn_gate", m, kern)
            with torch.cuda.stream(side_stream[0]):
                launch("ffn_up", m, side_kern[0])
            main.wait_stream(side_stream[0])
            launch("ffn_down", m, kern)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    warmup = max(args.warmup, 3)
    for _ in range(warmup):
        step()
    barrier()
    # The 28 launches of a step are microseconds each: replay them as one CUDA graph so that the device, not the
    # host's launch rate, is what gets timed.  (Capture falls back to plain launches if a collective refuses it.)
    run_step, graphed = step, False
    if not args.no_graph:
        try:
            graph = torch.cuda.CUDAGraph()
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                step()
                torch.cuda.synchronize()
                with torch.cuda.graph(graph, stream=side):
                    step()
            torch.cuda.synchronize()
            run_step, graphed = graph.replay, True
        except Exception as exc:  # pragma: no cover - depends on the NCCL build
            print(f"graph capture unavailable ({type(exc).__name__}: {exc}); timing plain launches", file=sys.stderr)
            torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local_rank) as clocks:
        # The timed region can be a few milliseconds, less than one nvidia-smi query: the sampler therefore also
        # covers ~0.5 s of the same replays immediately before it (same kernels, same load), all untimed.
        lead = time.time()
        while time.time() - lead < 0.5:
            for _ in range(10):
                run_step()
            torch.cuda.synchronize()
        barrier()
        start.record()
        for _ in range(args.steps):
            run_step()
        stop.record()
        barrier()
    ms = start.elapsed_time(stop)
    if world > 1:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    total_bytes = step_bytes(2) * args.steps
    value = total_bytes / (ms * 1e-3) / 1e9

    # per-call device times (secondary detail): each (projection, M) alone, launches rotating over enough copies of
    # the weight that it never sits in L2, replayed as a CUDA graph (the per-kernel harness's measurement)
    detail = {}
    if rank == 0 and not args.no_detail:
        from muser_b200 import microbench
        for name, (k, n, dt) in projs.items():
            ws = microbench.weight_copies(ctx, views[name].raw, dt, k, n, shard=plan.shard(name))
            for m in TOKEN_COUNTS:
                us = microbench.kquant_call_seconds(ctx, kern, ws, x_dev[(name, m)], y_dev[(name, m)], m) * 1e6
                kl, nl = weights[name].n_in, weights[name].n_out
                b = nl * ((kl + 255) // 256) * KQ_BYTES_PER_256[dt] + m * kl * 2 + m * nl * 4
                detail[f"{name}_m{m}"] = {"us": round(us, 2), "gbs": round(b / max(us, 1e-3) / 1e3, 1)}
            for w in ws:
                w.free()

    # end to end through the host-slice entry point (weights::matmul signature): f32 host x in, f32 host y out
    e2e = None
    if rank == 0:
        hx = {(name, m): synth.normal_activations(m, weights[name].n_in, seed=0, stream=2000).float().numpy()
              for name in projs for m in TOKEN_COUNTS}
        hy = {(name, m): np.empty((m, weights[name].n_out), dtype=np.float32) for name in projs for m in TOKEN_COUNTS}

        def e2e_step():
            for m in TOKEN_COUNTS:
                for name in projs:
                    op.matmul(ctx, weights[name], hx[(name, m)], m, hy[(name, m)])

        for _ in range(2):
            e2e_step()
        torch.cuda.synchronize()
        e2e_steps = max(3, min(args.steps, 20))
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            e2e_step()
        torch.cuda.synchronize()
        dt_e2e = time.perf_counter() - t0
        local_step_bytes = sum(
            weights[name].n_out * ((weights[name].n_in + 255) // 256) * KQ_BYTES_PER_256[projs[name][2]]
            + m * weights[name].n_in * 4 + m * weights[name].n_out * 4 for name in projs for m in TOKEN_COUNTS)
        e2e = {"value": local_step_bytes * e2e_steps / dt_e2e / 1e9, "unit": UNIT,
               "h2d_bytes_per_step": sum(m * weights[name].n_in * 4 for name in projs for m in TOKEN_COUNTS),
               "d2h_bytes_per_step": sum(m * weights[name].n_out * 4 for name in projs for m in TOKEN_COUNTS),
               "note": "muser_cuda_matmul_host per call: pinned staging, H2D of x, GEMV, D2H of y, synchronize"
                       + ("; rank 0's shard only" if world > 1 else "")}

    # second half of the metric: NVFP4 prefill GEMM, M = 2048, the same layer's shapes (N = 1 only); not part of `value`
    prefill = None
    if rank == 0 and world == 1 and not args.no_prefill:
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
        layer = tot_fl / tot_s / 1e12

        fused = {}
        try:
            # fused variants: q|k|v as one weight (rows concatenated, one quantized input), gate|up with SwiGLU in the epilogue
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
            parts = [synth.nvfp4_weight(synth.normal_weights(projs[nm][1], k_h, seed=0, stream=names.index(nm), device=dev))
                     for nm in ("attn_q", "attn_k", "attn_v")]
            n_qkv = sum(projs[nm][1] for nm in ("attn_q", "attn_k", "attn_v"))
            # one tensor scale for the concatenation: the synthetic weights share a distribution, so the first one's serves
            w_qkv = op.Weight(ctx, op.TensorView(torch.cat([p[0] for p in parts]), NVFP4, k_h, n_qkv,
                                                 torch.cat([p[1] for p in parts]), parts[0][2], isi))
            y_qkv = torch.empty((m, n_qkv), dtype=torch.bfloat16, device=dev)
            t = timed(lambda: kern.encode_nvfp4_prequant(w_qkv, xp, xs, y_qkv, m))
            fused["attn_q|k|v"] = {"gemm_tflops": round(2.0 * m * n_qkv * k_h / t / 1e12, 1)}
            w_qkv.free()
            n_f = projs["ffn_gate"][1]
            gu = [synth.nvfp4_weight(synth.normal_weights(n_f, k_h, seed=0, stream=names.index(nm), device=dev)) for nm in ("ffn_gate", "ffn_up")]
            w_g, w_u = (op.Weight(ctx, op.TensorView(p[0], NVFP4, k_h, n_f, p[1], p[2], isi)) for p in gu)
            y_f = torch.empty((m, n_f), dtype=torch.bfloat16, device=dev)
            t = timed(lambda: kern.encode_nvfp4_ffn_gate_up_silu_prequant(w_g, w_u, xp, xs, y_f, m))
            fused["ffn_gate|up+swiglu"] = {"gemm_tflops": round(2.0 * m * 2 * n_f * k_h / t / 1e12, 1)}
            w_g.free()
            w_u.free()
            del parts, gu, y_qkv, y_f, xa, xp, xs

        except Exception as exc:  # the secondary section must never cost the headline line
            fused = {"error": f"{type(exc).__name__}: {exc}"}

        prefill = {"workload": "nvfp4_prefill_gemm_layer_m2048", "unit": "TFLOP/s", "layer": round(layer, 1),
                   "per_projection": per, "fused": fused,
                   "roofline": {"bound": "tensor", "achieved": round(layer, 1), "peak": round(peak_fp4, 1), "unit": "TFLOP/s",
                                "frac": round(layer / peak_fp4, 4),
                                "peak_kind": "measured here: muser_cuda_fp4_peak_probe (block-scaled FP4 MMAs, no memory traffic)"}}

    # CPU lane on this box's host cores, bounded sample (N = 1 only)
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        from oracle import oracle as O
        threads = O.host_threads()
        name, m = "ffn_gate", 1
        k, n, dt = projs[name]
        ow = O.TensorView(views[name].raw.cpu().numpy(), dt, k, n)
        xin = x_dev[(name, m)].float().cpu().numpy()
        O.matmul(ow, xin, threads=threads)
        reps, t0 = 0, time.perf_counter()
        while time.perf_counter() - t0 < 10.0 and reps < 200:
            ref = O.matmul(ow, xin, threads=threads)
            reps += 1
        dt_cpu = (time.perf_counter() - t0) / reps
        kern.encode_quantized_matmul(weights[name], x_dev[(name, m)], y_dev[(name, m)], m)
        got = y_dev[(name, m)].cpu().numpy()
        rel = float(np.linalg.norm(got - ref) / np.linalg.norm(ref))
        cpu = {"value": call_bytes(k, n, dt, m, 4) / dt_cpu / 1e9, "unit": UNIT, "cores": threads, "kind": "port",
               "sample": f"{name} (Q4_K {k}->{n}), M=1, {reps} repetitions of weights::matmul restated in C",
               "gpu_vs_cpu_rel_l2": rel}

    if rank == 0:
        peak, peak_kind = measured_peaks()
        peak *= world
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": warmup,
            "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic",
            "config": {"workload": WORKLOAD, "tokens": list(TOKEN_COUNTS), "projections": list(projs),
                       "weights": "Q4_K_M mix, seeded N(0,0.02)", "activations": "bf16 N(0,1)",
                       "l2": "inputs larger than L2 (312 MB of weights per pass, 126 MB L2)",
                       "launch": "one CUDA graph replay per step" if graphed else "plain launches",
                       "schedule": "q|k|v and gate|up on parallel streams, joined before o and down" if parallel else "serial",
                       "parallelism": f"tp{world}" if world > 1 else "single"},
            "roofline": {"bound": "hbm", "achieved": value, "peak": peak, "unit": "GB/s", "frac": value / peak,
                         # DRAM bytes of one step's launches under ncu (dram__bytes_read.sum + dram__bytes_write.sum,
                         # profiles/bench_launch_list_decode_gemv_layer.md): 1.007 x the algorithmic bytes, no re-reads
                         "traffic": MEASURED_STEP_TRAFFIC_BYTES if world == 1 else None, "traffic_per": "step (28 launches)",
                         "algorithmic_bytes_per_step": step_bytes(2), "peak_kind": f"of {peak_kind}",
                         "kernel": "kquant_gemv_kernel / kquant_matmul_kernel / kquant_tc_kernel (the 28 launches of a step; achieved = all their bytes / all their time)"},
            "cpu_baseline": cpu,
            "e2e": e2e,
            "gpu_launches": launches_per_step * args.steps,
            "clocks": clocks.summary(),
            "detail_us": detail,
            "prefill": prefill,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        # Leave without tearing the process group down: ranks finish at different times (rank 0 alone runs the
        # detail, end-to-end and CPU legs), and a teardown that waits for a peer that is already gone never returns.
        torch.cuda.synchronize()
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(0)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU-lane baseline leg")
    ap.add_argument("--no-detail", action="store_true", help="skip the per-projection timings")
    ap.add_argument("--no-prefill", action="store_true", help="skip the NVFP4 prefill GEMM section")
    ap.add_argument("--serial", action="store_true", help="one stream: the 28 projections strictly one after another")
    ap.add_argument("--no-graph", action="store_true", help="launch the step's kernels one by one instead of as a CUDA graph")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_gpu(args)


if __name__ == "__main__":
    main()
