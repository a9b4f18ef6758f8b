"""Kernel microbenchmark of the quantized projections, in the spirit of the reference's `muser-m16-bench`
(crates/muser-bench/src/m16.rs:740-880): per shape and token count it prints milliseconds, GB/s over the
algorithmic bytes, TMAC/s, and (with --check) the differential against the CPU lane.

    python -m muser_b200.microbench kquant --proj ffn_gate,ffn_down --tokens 1,2,4,8 [--check] [--no-graph]
    python -m muser_b200.microbench nvfp4  --proj ffn_gate --tokens 2048 [--reps 5]
    python -m muser_b200.microbench peak

Shapes are the projections of the synthetic layer in `synth.LAYER_PROJECTIONS`.  K-quant calls rotate over
enough weight copies to exceed L2 (126 MB) and are replayed as one CUDA graph unless --no-graph is given, so the
time is the device's, not the launch path's.  This is also the harness the ncu captures under profiles/ wrap.
"""
from __future__ import annotations

import argparse
import sys

import numpy as np
import torch

from . import operator as op
from . import synth

HBM_PEAK_GBS = 6548.5  # measured copy bandwidth of this pool's B200s (MEASURED_PEAKS.json)


def _time(fn, reps: int) -> float:
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    fn()
    torch.cuda.synchronize()
    e0.record()
    for _ in range(reps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e-3 / reps


def run_kquant(args) -> None:
    ctx = op.Context(0)
    kern = op.CudaKernels(ctx)
    print(f"{'shape':<28} {'tokens':>6} {'us':>9} {'GB/s':>9} {'%HBM':>6} {'TMAC/s':>8} {'rel_l2':>10}")
    for name in args.proj:
        k, n, dt = synth.LAYER_PROJECTIONS[name]
        raw = synth.quantize_kquant(synth.normal_weights(n, k, device="cuda"), dt)
        copies = max(2, min(24, (300 << 20) // raw.numel() + 1))
        ws = [op.Weight(ctx, op.TensorView(raw, dt, k, n)) for _ in range(copies)]
        for m in args.tokens:
            x = synth.normal_activations(m, k, device="cuda")
            y = torch.empty((m, n), dtype=torch.float32, device="cuda")
            launches = max(20, copies)

            def run():
                for i in range(launches):
                    kern.encode_quantized_matmul(ws[i % copies], x, y, m)

            run()
            torch.cuda.synchronize()
            fn = run
            if not args.no_graph:
                g, side = torch.cuda.CUDAGraph(), torch.cuda.Stream()
                with torch.cuda.stream(side):
                    run()
                    torch.cuda.synchronize()
                    with torch.cuda.graph(g, stream=side):
                        run()
                torch.cuda.synchronize()
                fn = g.replay
            sec = _time(fn, args.reps) / launches
            nbytes = raw.numel() + m * k * 2 + m * n * 4
            rel = float("nan")
            if args.check:
                from oracle import oracle as O  # the checker, never the thing measured
                ref = O.matmul(O.TensorView(raw.cpu().numpy(), dt, k, n), x.float().cpu().numpy(), threads=O.host_threads())
                rel = float(np.linalg.norm(y.cpu().numpy() - ref) / np.linalg.norm(ref))
            print(f"{name + f' {k}->{n}':<28} {m:>6} {sec * 1e6:>9.2f} {nbytes / sec / 1e9:>9.1f} "
                  f"{nbytes / sec / 1e9 / HBM_PEAK_GBS * 100:>6.1f} {m * n * k / sec / 1e12:>8.2f} {rel:>10.2e}", flush=True)
        for w in ws:
            w.free()


def run_nvfp4(args) -> None:
    ctx = op.Context(0, workspace_bytes=1 << 30)
    kern = op.CudaKernels(ctx)
    print(f"{'shape':<28} {'tokens':>6} {'gemm us':>9} {'TFLOP/s':>9} {'quant us':>9} {'rel_l2':>10}")
    tot_f = tot_t = 0.0
    for name in args.proj:
        k, n, _ = synth.LAYER_PROJECTIONS[name]
        wp, wsc, s2 = synth.nvfp4_weight(synth.normal_weights(n, k, device="cuda"))
        for m in args.tokens:
            x = synth.normal_activations(m, k, device="cuda")
            isi = synth.activation_input_scale_inv(x)
            w = op.Weight(ctx, op.TensorView(wp, op.NVFP4, k, n, wsc, s2, isi))
            y = torch.empty((m, n), dtype=torch.bfloat16, device="cuda")
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


def main(argv=None) -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("what", choices=["kquant", "nvfp4", "peak"])
    ap.add_argument("--proj", type=lambda s: s.split(","), default=list(synth.LAYER_PROJECTIONS))
    ap.add_argument("--tokens", type=lambda s: [int(v) for v in s.split(",")], default=None)
    ap.add_argument("--reps", type=int, default=5)
    ap.add_argument("--check", action="store_true", help="compare with the CPU lane (oracle/)")
    ap.add_argument("--no-graph", action="store_true")
    args = ap.parse_args(argv)
    if args.what == "kquant":
        args.tokens = args.tokens or [1, 2, 4, 8]
        run_kquant(args)
    elif args.what == "nvfp4":
        args.tokens = args.tokens or [2048]
        run_nvfp4(args)
    else:
        ctx = op.Context(0)
        print(f"dense block-scaled FP4 tensor peak: {op.fp4_peak_tflops(ctx):.1f} TFLOP/s")


if __name__ == "__main__":
    sys.exit(main())
