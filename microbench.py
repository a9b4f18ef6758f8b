"""Kernel microbenchmark of the quantized projections, in the spirit of the reference's `muser-m16-bench`
(crates/muser-bench/src/m16.rs:740-880): per shape and token count it prints milliseconds, GB/s over the
algorithmic bytes, TMAC/s, and (with --check) the differential against the CPU lane.

    python microbench.py kquant --proj ffn_gate,ffn_down --tokens 1,2,4,8 [--check] [--no-graph]
    python microbench.py groups --tokens 1,2,4,8          (the decode step's four launches: q|k|v, o, gate|up, down)
    python microbench.py lmhead --tokens 1,4,16           (202048-row Q5_K LM head with the fused greedy pick)
    python microbench.py nvfp4  --proj ffn_gate --tokens 2048 [--reps 5]
    python microbench.py peak
    python microbench.py layers --tokens 32768 --layers 52 [--chunks 4]      (torchrun for TP > 1)
    torchrun --nproc-per-node N microbench.py allreduce                      (the one-shot all-reduce beside NCCL)

Shapes are the projections of the synthetic layer in `synth.LAYER_PROJECTIONS`.  K-quant calls rotate over
enough weight copies to exceed L2 (126 MB) and are replayed as one CUDA graph unless --no-graph is given, so the
time is the device's, not the launch path's.  The ncu captures of single kernels wrap this harness.
"""
from __future__ import annotations

import argparse
import sys

import json
from pathlib import Path

import numpy as np
import torch

from muser_b200 import operator as op
from muser_b200 import synth, tp, workloads
from muser_b200.workloads import kquant_call_seconds, weight_copies

_PEAKS = Path(__file__).resolve().parent / "MEASURED_PEAKS.json"
HBM_PEAK_GBS = float(json.loads(_PEAKS.read_text())["hbm_gbs"]) if _PEAKS.exists() else 6650.0  # measured copy bandwidth, else the stated fallback


_time = workloads.time_calls


def run_groups(args) -> None:
    """The decode step's launches, each rotating over weight copies so that nothing is served from L2."""
    ctx = op.Context(0)
    kern = op.CudaKernels(ctx)
    layer = workloads.DecodeLayer(ctx, kern, tp.ShardPlan(0, 1), args.tokens, "cuda")
    print(f"{'launch':<28} {'tokens':>6} {'us':>9} {'GB/s':>9} {'%HBM':>6}")
    for gi, group in enumerate(layer.GROUPS):
        copies = [[op.Weight(ctx, layer.views[n]) for n in group] for _ in range(max(2, min(12, (300 << 20) // sum(layer.views[n].raw.numel() for n in group) + 1)))]
        for m in args.tokens:
            sec = workloads.rotating_call_seconds(lambda i: layer.launch_group(gi, m, copies[i]), len(copies), not args.no_graph, args.reps)
            nbytes = sum(workloads.kquant_call_bytes(*layer.projs[n], m) for n in group)
            print(f"{'|'.join(group):<28} {m:>6} {sec * 1e6:>9.2f} {nbytes / sec / 1e9:>9.1f} {nbytes / sec / 1e9 / HBM_PEAK_GBS * 100:>6.1f}", flush=True)
        for c in copies:
            for w in c:
                w.free()
    ctx.sync_status()


def run_kquant(args) -> None:
    ctx = op.Context(0)
    kern = op.CudaKernels(ctx)
    print(f"{'shape':<28} {'tokens':>6} {'us':>9} {'GB/s':>9} {'%HBM':>6} {'TFLOP/s':>8} {'rel_l2':>10}")
    for name in args.proj:
        k, n, dt = synth.LAYER_PROJECTIONS[name]
        raw = synth.quantize_kquant(synth.normal_weights(n, k, device="cuda"), dt)
        ws = weight_copies(ctx, raw, dt, k, n)
        for m in args.tokens:
            x = synth.normal_activations(m, k, device="cuda")
            y = torch.empty((m, n), dtype=torch.float32, device="cuda")
            sec = kquant_call_seconds(ctx, kern, ws, x, y, m, graph=not args.no_graph, reps=args.reps)
            nbytes = raw.numel() + m * k * 2 + m * n * 4
            rel = float("nan")
            if args.check:
                from oracle import oracle as O  # the checker, never the thing measured
                ref = O.matmul(O.TensorView(raw.cpu().numpy(), dt, k, n), x.float().cpu().numpy(), threads=O.host_threads())
                rel = float(np.linalg.norm(y.cpu().numpy() - ref) / np.linalg.norm(ref))
            print(f"{name + f' {k}->{n}':<28} {m:>6} {sec * 1e6:>9.2f} {nbytes / sec / 1e9:>9.1f} "
                  f"{nbytes / sec / 1e9 / HBM_PEAK_GBS * 100:>6.1f} {2 * m * n * k / sec / 1e12:>8.2f} {rel:>10.2e}", flush=True)
        for w in ws:
            w.free()


def run_lmhead(args) -> None:
    """The LM head of the real model's geometry (202048 rows x 5120, Q5_K: crates/muser-bench/src/m16.rs:195-201) with
    the greedy pick fused in, against the plain projection that writes the logits."""
    ctx = op.Context(0)
    kern = op.CudaKernels(ctx)
    n, k, dt = 202048, 5120, 13  # GgmlType::Q5_K
    raw = torch.cat([synth.quantize_kquant(synth.normal_weights(n // 8, k, seed=0, stream=90 + i, device="cuda"), dt) for i in range(8)])
    w = op.Weight(ctx, op.TensorView(raw, dt, k, n))
    nbytes_w = raw.numel()
    del raw
    print(f"{'LM head 5120->202048 Q5_K':<28} {'tokens':>6} {'pick us':>9} {'GB/s':>9} {'%HBM':>6} {'logits us':>10} {'same pick':>10}")
    for m in args.tokens:
        x = synth.normal_activations(m, k, device="cuda")
        y = torch.empty((m, n), dtype=torch.float32, device="cuda")
        res = {}
        t_pick = _time(lambda: res.__setitem__("r", kern.encode_lm_head_argmax(w, x, m, out_scale=0.5, softcap=30.0)), args.reps)
        t_full = _time(lambda: kern.encode_quantized_matmul(w, x, y, m, out_scale=0.5, softcap=30.0), args.reps)
        same = bool(torch.equal(res["r"][0].long(), torch.argmax(y, dim=1)))
        nbytes = nbytes_w + m * k * 2
        print(f"{'':<28} {m:>6} {t_pick * 1e6:>9.1f} {nbytes / t_pick / 1e9:>9.1f} {nbytes / t_pick / 1e9 / HBM_PEAK_GBS * 100:>6.1f} {t_full * 1e6:>10.1f} {str(same):>10}", flush=True)
    ctx.sync_status()


def run_nvfp4(args) -> None:
    ctx = op.Context(0, workspace_bytes=1 << 30)
    kern = op.CudaKernels(ctx)
    if args.form is not None:
        from muser_b200._lib import TUNE_NVFP4_PAIR
        ctx.tuning_set(TUNE_NVFP4_PAIR, args.form)
    print(f"{'shape':<28} {'tokens':>6} {'gemm us':>9} {'TFLOP/s':>9} {'quant us':>9} {'rel_l2':>10}")
    tot_f = tot_t = 0.0
    for name in args.proj:
        k, n, _ = synth.LAYER_PROJECTIONS[name]
        wp, wsc, s2 = synth.nvfp4_weight(synth.normal_weights(n, k, device="cuda"))
        for m in args.tokens:
            x = synth.normal_activations(m, k, device="cuda")
            isi = synth.activation_input_scale_inv(x)
            w = op.Weight(ctx, op.TensorView(wp, op.NVFP4, k, n, wsc, s2, isi))
            y = torch.empty((m, n), dtype=torch.float32 if args.check else torch.bfloat16, device="cuda")  # f32 for the comparison
            xp, xs = kern.quantize_nvfp4_activation(x, isi)
            for _ in range(2):
                kern.encode_nvfp4_prequant(w, xp, xs, y, m)
            t_gemm = _time(lambda: kern.encode_nvfp4_prequant(w, xp, xs, y, m), args.reps)
            t_quant = _time(lambda: kern.quantize_nvfp4_activation(x, isi), args.reps)
            ctx.sync_status()
            rel = float("nan")
            if args.check:
                from oracle import oracle as O
                rows = torch.randperm(m, generator=torch.Generator().manual_seed(0))[:32].cuda()
                ow = O.TensorView(wp.cpu().numpy(), O.NVFP4, k, n, wsc.cpu().numpy(), s2, isi)
                _, ref = O.matmul(ow, x[rows].float().cpu().numpy(), threads=O.host_threads(), return_pre_round=True)
                rel = float(np.linalg.norm(y[rows].float().cpu().numpy() - ref) / np.linalg.norm(ref))
            fl = 2.0 * m * n * k
            tot_f, tot_t = tot_f + fl, tot_t + t_gemm
            print(f"{name + f' {k}->{n}':<28} {m:>6} {t_gemm * 1e6:>9.1f} {fl / t_gemm / 1e12:>9.1f} {t_quant * 1e6:>9.1f} {rel:>10.2e}", flush=True)
            w.free()
    print(f"total: {tot_t * 1e6:.1f} us, {tot_f / tot_t / 1e12:.1f} TFLOP/s")


def run_allreduce(args) -> None:
    """The library's all-reduce beside NCCL's, per payload (torchrun, 2-8 ranks): device microseconds per call, 50
    calls replayed from a CUDA graph, the maximum over the ranks; then the tensor-parallel decode step with and
    without its all-reduces."""
    import os

    import torch.distributed as dist

    from muser_b200 import _lib
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    ctx = op.Context(local, workspace_bytes=1 << 20)
    kern = op.CudaKernels(ctx)
    coll = tp.Collective(ctx, rank, world)

    def timeit(fn, n=50, reps=5):
        replay = workloads.capture(lambda: [fn() for _ in range(n)])
        for _ in range(3):
            replay()
        torch.cuda.synchronize()
        dist.barrier()
        t = torch.tensor([workloads.time_calls(replay, reps) / n], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item()) * 1e6

    if rank == 0:
        print(f"{world} ranks; f32 payload: tokens x 5120 values\n{'tokens':>6} {'KiB':>7} {'one-shot us':>12} {'library NCCL us':>16} {'torch NCCL us':>14}", flush=True)
    for tokens in (args.tokens or [1, 8, 16, 64]):
        buf = torch.randn(tokens * 5120, device=dev)
        t1 = timeit(lambda: coll.all_reduce_sum(buf))
        ctx.tuning_set(_lib.TUNE_ONESHOT_MAX_BYTES, 0)
        t2 = timeit(lambda: coll.all_reduce_sum(buf))
        ctx.tuning_set(_lib.TUNE_ONESHOT_MAX_BYTES, 1536 << 10)
        t3 = timeit(lambda: dist.all_reduce(buf))
        if rank == 0:
            print(f"{tokens:>6} {tokens * 20:>7} {t1:>12.2f} {t2:>16.2f} {t3:>14.2f}", flush=True)
    layer = workloads.DecodeLayer(ctx, kern, tp.ShardPlan(rank, world), (1, 2, 4, 8), dev, all_reduce=coll.all_reduce_sum, fuse_all_reduce=True)
    step = lambda: [layer.run(m) for m in (1, 2, 4, 8)]
    t_fused = timeit(step, n=1, reps=50)
    layer.fuse_all_reduce = False
    t_sep = timeit(step, n=1, reps=50)
    layer.all_reduce = None
    t_none = timeit(step, n=1, reps=50)
    if rank == 0:
        print(f"decode step (M = 1, 2, 4, 8): {t_fused:.1f} us with the partial sums pushed by the projection kernels, {t_sep:.1f} us with "
              f"projection then all-reduce, {t_none:.1f} us without any all-reduce", flush=True)
    ctx.sync_status()
    torch.cuda.synchronize()
    os._exit(0)


def run_layers(args) -> None:
    """The linear layers of a prefill pass: `--layers` decoder layers x 7 NVFP4 projections at `--tokens` tokens
    (workloads.PrefillLayer), tensor-parallel over the ranks torchrun started, with one all-reduce after o_proj and
    one after down_proj."""
    import os

    import torch.distributed as dist

    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    M, L = args.tokens[0], args.layers
    ctx = op.Context(local, workspace_bytes=workloads.PrefillLayer.workspace_bytes(M, world))
    kern = op.CudaKernels(ctx)
    pl = workloads.PrefillLayer(ctx, kern, tp.ShardPlan(rank, world), M, f"cuda:{local}",
                                all_reduce=tp.all_reduce_sum if world > 1 else None, chunks=args.chunks)
    pl.layer(pl.h)
    ctx.sync_status()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    pl.run(L)
    e1.record()
    torch.cuda.synchronize()
    ms = torch.tensor([e0.elapsed_time(e1)], device=f"cuda:{local}")
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    ctx.sync_status()
    flops = pl.flops(L)
    if rank == 0:
        print(f"prefill linears: tokens {M}, layers {L}, TP {world}, chunks {len(pl.bounds)}: {ms.item():.1f} ms, "
              f"{flops / 1e15:.4f} PFLOP, {flops / (ms.item() * 1e-3) / 1e12:.1f} TFLOP/s whole job, "
              f"{flops / (ms.item() * 1e-3) / 1e12 / world:.1f} per GPU", flush=True)
    if world > 1:
        torch.cuda.synchronize()
        os._exit(0)  # skip the process-group teardown: the ranks finish at different times


def main(argv=None) -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("what", choices=["kquant", "groups", "lmhead", "nvfp4", "peak", "layers", "allreduce"])
    ap.add_argument("--layers", type=int, default=52)
    ap.add_argument("--chunks", type=int, default=4, help="token chunks per row-parallel projection (TP > 1)")
    ap.add_argument("--proj", type=lambda s: s.split(","), default=list(synth.LAYER_PROJECTIONS))
    ap.add_argument("--tokens", type=lambda s: [int(v) for v in s.split(",")], default=None)
    ap.add_argument("--reps", type=int, default=5)
    ap.add_argument("--check", action="store_true", help="compare with the CPU lane (oracle/)")
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--form", type=int, default=None, choices=[0, 1], help="nvfp4: 0 one CTA per tile, 1 pairs of SMs on one tile")
    args = ap.parse_args(argv)
    if args.what == "kquant":
        args.tokens = args.tokens or [1, 2, 4, 8]
        run_kquant(args)
    elif args.what == "groups":
        args.tokens = args.tokens or [1, 2, 4, 8]
        run_groups(args)
    elif args.what == "lmhead":
        args.tokens = args.tokens or [1, 2, 4, 8, 16]
        run_lmhead(args)
    elif args.what == "nvfp4":
        args.tokens = args.tokens or [2048]
        run_nvfp4(args)
    elif args.what == "allreduce":
        run_allreduce(args)
    elif args.what == "layers":
        args.tokens = args.tokens or [32768]
        run_layers(args)
    else:
        ctx = op.Context(0, workspace_bytes=32 << 20)
        print(f"dense block-scaled FP4 tensor peak: {op.fp4_peak_tflops(ctx):.1f} TFLOP/s")
        # the GEMM's per-slab instruction mix in isolation (one 128 x 256 x 256 slab per iteration and SM)
        mhz = int(getattr(torch.cuda.get_device_properties(0), "clock_rate", 1965000)) // 1000  # the device's maximum SM clock
        iters = 20000
        flops = 2.0 * 128 * 256 * 256 * iters * torch.cuda.get_device_properties(0).multi_processor_count
        print(f"{'per slab':<58} {'us/kernel':>10} {'ns/slab':>8} {'cycles@' + str(mhz):>11} {'TFLOP/s':>8}")
        rows = [(0, 0, False, "4 MMAs, zero operands"), (0, 0, True, "4 MMAs, random non-zero codes and scales"),
                (3, 0, True, "12 scale copies (32x128b.warpx4) alone"), (1, 0, True, "12 scale copies, then 4 MMAs"),
                (2, 0, True, "(3 scale copies, 1 MMA) x 4"), (4, 0, True, "6 scale copies of 128x256b alone"),
                (5, 0, True, "6 scale copies of 128x256b, then 4 MMAs"),
                (6, 54, True, "54 KiB of bulk loads from L2 alone"), (6, 36, True, "36 KiB of bulk loads from L2 alone"),
                (0, 54, True, "4 MMAs beside 54 KiB of loads"), (0, 36, True, "4 MMAs beside 36 KiB of loads"),
                (2, 54, True, "(3 copies, 1 MMA) x 4 beside 54 KiB of loads"), (1, 54, True, "12 copies, then 4 MMAs beside 54 KiB of loads")]
        for mode, kib, rnd, label in rows:
            us = op.fp4_pipe_probe_us(ctx, mode, iters, kib, rnd)
            tf = f"{flops / us / 1e6:8.0f}" if mode in (0, 1, 2, 5) else f"{'':>8}"
            print(f"{label:<58} {us:>10.1f} {us * 1e3 / iters:>8.1f} {us * mhz / iters:>11.0f} {tf}")
        for n in (16, 32, 64, 128, 256):
            print(f"tcgen05.mma kind::f16, 128 x {n:3d} x 16, back to back: {op.f16_mma_cycles(ctx, n):.1f} cycles per instruction")


if __name__ == "__main__":
    sys.exit(main())
