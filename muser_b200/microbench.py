"""Kernel microbenchmark of the quantized projections, in the spirit of the reference's `muser-m16-bench`
(crates/muser-bench/src/m16.rs:740-880): per shape and token count it prints milliseconds, GB/s over the
algorithmic bytes, TMAC/s, and (with --check) the differential against the CPU lane.

    python -m muser_b200.microbench kquant --proj ffn_gate,ffn_down --tokens 1,2,4,8 [--check] [--no-graph]
    python -m muser_b200.microbench nvfp4  --proj ffn_gate --tokens 2048 [--reps 5]
    python -m muser_b200.microbench peak
    python -m muser_b200.microbench layers --tokens 32768 --layers 52 [--chunks 4]      (torchrun for TP > 1)

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


def kquant_call_seconds(ctx, kern, ws, x, y, m: int, graph: bool = True, reps: int = 5) -> float:
    """Device seconds of one K-quant projection call at `m` tokens: launches rotate over the weight copies `ws`
    (together larger than L2, so every launch streams its weights from HBM) and are replayed as one CUDA graph."""
    copies = len(ws)
    launches = max(20, copies)

    def run():
        for i in range(launches):
            kern.encode_quantized_matmul(ws[i % copies], x, y, m)

    run()
    torch.cuda.synchronize()
    fn = run
    if graph:
        g, side = torch.cuda.CUDAGraph(), torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            run()
            torch.cuda.synchronize()
            with torch.cuda.graph(g, stream=side):
                run()
        torch.cuda.synchronize()
        fn = g.replay
    return _time(fn, reps) / launches


def weight_copies(ctx, raw, dt: int, k: int, n: int, shard=None):
    """Enough repacked copies of one tensor to exceed L2 (126 MB) when launches rotate over them."""
    copies = max(2, min(24, (300 << 20) // raw.numel() + 1))
    return [op.Weight(ctx, op.TensorView(raw, dt, k, n), shard=shard) for _ in range(copies)]


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


def run_layers(args) -> None:
    """The linear layers of a prefill pass: `--layers` decoder layers x 7 NVFP4 projections at `--tokens` tokens, input
    norms fused into the activation quantizer, SwiGLU fused into the gate/up GEMM, residual adds fused into the o and
    down epilogues, attention left out (the q projection's output stands in for it), tensor-parallel over the ranks
    torchrun started with one all-reduce after o_proj and one after down_proj (chunked over tokens so that the
    GEMM of the next chunk runs under the all-reduce of the last).  All layers reuse one layer's weights: at
    274 MB they do not fit L2, so every layer still streams them from HBM."""
    import os

    import torch.distributed as dist

    from . import tp

    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    plan = tp.ShardPlan(rank, world)
    M, L, eps = args.tokens[0], args.layers, 1e-6
    dev = f"cuda:{local}"
    P = synth.LAYER_PROJECTIONS
    H, F = P["attn_q"][0], P["ffn_gate"][1]
    ctx = op.Context(local, workspace_bytes=(M + 128) * (F // world // 2 + F // world // 16 + 64) + (1 << 20))
    kern = op.CudaKernels(ctx)

    h = synth.normal_activations(M, H, device=dev)
    norm_w = [torch.ones(H, device=dev) + 0.1 * torch.randn(H, device=dev, generator=torch.Generator(dev).manual_seed(s)) for s in (1, 2)]

    def rms(x, w):
        xf = x.float()
        return xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * w

    # static input scales per projection input, fixed from this seeded data as a stored checkpoint would carry them
    sample = slice(0, min(M, 1024))
    isi_attn = synth.activation_input_scale_inv(rms(h[sample], norm_w[0]))
    isi_ffn = synth.activation_input_scale_inv(rms(h[sample], norm_w[1]))
    weights, dense = {}, {}
    for i, (name, (k, n, _)) in enumerate(P.items()):
        dense[name] = synth.normal_weights(n, k, seed=0, stream=i, device=dev)
    isi_o = synth.activation_input_scale_inv(rms(h[sample], norm_w[0]) @ dense["attn_q"].t())
    act = torch.nn.functional.silu(rms(h[sample], norm_w[1]) @ dense["ffn_gate"].t()) * (rms(h[sample], norm_w[1]) @ dense["ffn_up"].t())
    isi_down = synth.activation_input_scale_inv(act)
    isis = {"attn_q": isi_attn, "attn_k": isi_attn, "attn_v": isi_attn, "attn_o": isi_o, "ffn_gate": isi_ffn,
            "ffn_up": isi_ffn, "ffn_down": isi_down}
    for name, (k, n, _) in P.items():
        wp, wsc, s2 = synth.nvfp4_weight(dense[name])
        weights[name] = op.Weight(ctx, op.TensorView(wp, op.NVFP4, k, n, wsc, s2, isis[name]), shard=plan.shard(name))
    del dense, act
    Ql, KVl, Fl = P["attn_q"][1] // world, P["attn_k"][1] // world, F // world
    bf = dict(dtype=torch.bfloat16, device=dev)
    q, kk, vv = torch.empty((M, Ql), **bf), torch.empty((M, KVl), **bf), torch.empty((M, KVl), **bf)
    ffn_act, h1, h2 = torch.empty((M, Fl), **bf), torch.empty((M, H), **bf), torch.empty((M, H), **bf)
    xq = (torch.empty((M, H // 2), dtype=torch.uint8, device=dev),
          torch.empty((op._L.muser_cuda_nvfp4_swizzled_scale_bytes(M, H),), dtype=torch.uint8, device=dev))
    chunks = max(1, args.chunks if world > 1 else 1)
    step = (M + chunks - 1) // chunks // 128 * 128 or M
    bounds = [(a, min(M, a + step)) for a in range(0, M, step)]

    def row_parallel(name, x, res, out):
        """out = all_reduce(x @ W_shard^T) + res, in token chunks; the residual is added on rank 0's partial sum."""
        works = []
        for a, b in bounds:
            kern.encode_nvfp4_matmul(weights[name], x[a:b], out[a:b], b - a, residual=res[a:b] if rank == 0 else None)
            if world > 1:
                works.append(dist.all_reduce(out[a:b], async_op=True))
        for w in works:
            w.wait()

    def layer(x):
        kern.quantize_nvfp4_activation(x, isi_attn, norm_weight=norm_w[0], norm_eps=eps, out=xq)
        kern.encode_nvfp4_prequant(weights["attn_q"], xq[0], xq[1], q, M)
        kern.encode_nvfp4_prequant(weights["attn_k"], xq[0], xq[1], kk, M)
        kern.encode_nvfp4_prequant(weights["attn_v"], xq[0], xq[1], vv, M)
        row_parallel("attn_o", q, x, h1)
        kern.encode_ffn_gate_up_silu(weights["ffn_gate"], weights["ffn_up"], h1, ffn_act, M, norm_weight=norm_w[1], norm_eps=eps)
        row_parallel("ffn_down", ffn_act, h1, h2)
        return h2

    def run():
        x = h
        for _ in range(L):
            x = layer(x)  # h2 feeds the next layer; its values do not matter to the timing, only its shape
        return x

    layer(h)
    ctx.sync_status()
    if args.check and rank == 0:
        print("layer output finite:", bool(torch.isfinite(h2.float()).all()), flush=True)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    run()
    e1.record()
    torch.cuda.synchronize()
    ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    ctx.sync_status()
    macs = sum(k * n for k, n, _ in P.values())
    flops = 2.0 * M * macs * L
    if rank == 0:
        print(f"prefill linears: tokens {M}, layers {L}, TP {world}, chunks {len(bounds)}: {ms.item():.1f} ms, "
              f"{flops / 1e15:.4f} PFLOP, {flops / (ms.item() * 1e-3) / 1e12:.1f} TFLOP/s whole job, "
              f"{flops / (ms.item() * 1e-3) / 1e12 / world:.1f} per GPU", flush=True)
    if world > 1:
        torch.cuda.synchronize()
        os._exit(0)  # skip the process-group teardown, which has hung on this pool after the work was done


def main(argv=None) -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("what", choices=["kquant", "nvfp4", "peak", "layers"])
    ap.add_argument("--layers", type=int, default=52)
    ap.add_argument("--chunks", type=int, default=4, help="token chunks per row-parallel projection (TP > 1)")
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
    elif args.what == "layers":
        args.tokens = args.tokens or [32768]
        run_layers(args)
    else:
        ctx = op.Context(0)
        print(f"dense block-scaled FP4 tensor peak: {op.fp4_peak_tflops(ctx):.1f} TFLOP/s")
        for n in (16, 32, 64, 128, 256):
            print(f"tcgen05.mma kind::f16, 128 x {n:3d} x 16, back to back: {op.f16_mma_cycles(ctx, n):.1f} cycles per instruction")


if __name__ == "__main__":
    sys.exit(main())
