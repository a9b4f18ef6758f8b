"""The synthetic workloads that the benchmark, the kernel harness and the full-size tests share.

`DecodeLayer` is one decoder layer's K-quant projections as the decode step issues them: q | k | v in one grouped
launch, o_proj, gate | up in one grouped launch, down_proj (the order and the grouping of the reference's decode
driver, crates/muser-engine/src/decode.rs:5569-5598), optionally tensor-parallel.  `PrefillLayer` is the same layer in
NVFP4 as a prefill pass runs it: input norms fused into the activation quantizer, SwiGLU fused into the gate/up GEMM,
residual adds fused into the o and down epilogues, attention left out (the q projection's output stands in for it).
Nothing here checks results: the comparisons against the CPU lane live in tests/ and bench.py.
"""
from __future__ import annotations

import torch

from . import operator as op
from . import synth, tp

KQ_BYTES_PER_256 = {synth.Q4_K: 144, synth.Q6_K: 210}


def time_calls(fn, reps: int) -> float:
    """Device seconds per call of fn (CUDA events on the current stream, one untimed call first)."""
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    fn()
    torch.cuda.synchronize()
    e0.record()
    for _ in range(reps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e-3 / reps


def capture(fn):
    """fn's launches as one CUDA graph; returns its replay."""
    g, side = torch.cuda.CUDAGraph(), torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        fn()
        torch.cuda.synchronize()
        with torch.cuda.graph(g, stream=side):
            fn()
    torch.cuda.synchronize()
    return g.replay


def weight_copies(ctx, raw, dt: int, k: int, n: int, shard=None, budget: int = 300 << 20):
    """Enough repacked copies of one tensor to exceed L2 (126 MB) when launches rotate over them."""
    copies = max(2, min(24, budget // raw.numel() + 1))
    return [op.Weight(ctx, op.TensorView(raw, dt, k, n), shard=shard) for _ in range(copies)]


def rotating_call_seconds(launch, copies: int, graph: bool = True, reps: int = 5) -> float:
    """Device seconds of one launch(i), i rotating over `copies` weight copies (together larger than L2, so every
    launch streams its weights from HBM), replayed as one CUDA graph."""
    launches = max(20, copies)

    def run():
        for i in range(launches):
            launch(i % copies)

    run()
    torch.cuda.synchronize()
    fn = capture(run) if graph else run
    return time_calls(fn, reps) / launches


def kquant_call_seconds(ctx, kern, ws, x, y, m: int, graph: bool = True, reps: int = 5) -> float:
    return rotating_call_seconds(lambda i: kern.encode_quantized_matmul(ws[i], x, y, m), len(ws), graph, reps)


def kquant_call_bytes(n_in: int, n_out: int, dtype: int, m: int, x_bytes: int = 2) -> int:
    """Algorithmic bytes of one K-quant projection call: weights once, activations in, f32 outputs out."""
    return n_out * ((n_in + 255) // 256) * KQ_BYTES_PER_256[dtype] + m * n_in * x_bytes + m * n_out * 4


class DecodeLayer:
    """The seven K-quant projections of the synthetic layer, sharded for `plan`, with per-token-count inputs and
    outputs resident on the device.  `all_reduce(tensor)` sums a row-parallel projection's partial outputs."""

    GROUPS = (("attn_q", "attn_k", "attn_v"), ("attn_o",), ("ffn_gate", "ffn_up"), ("ffn_down",))

    def __init__(self, ctx, kern, plan: tp.ShardPlan, token_counts, device, all_reduce=None, seed: int = 0, autotune: bool = True,
                 fuse_all_reduce: bool = False):
        self.ctx, self.kern, self.plan, self.dev = ctx, kern, plan, device
        self.projs = synth.LAYER_PROJECTIONS
        self.all_reduce = all_reduce
        self.fuse_all_reduce = fuse_all_reduce
        self.views, self.weights, self.x, self.y = {}, {}, {}, {}
        for i, (name, (k, n, dt)) in enumerate(self.projs.items()):
            raw = synth.quantize_kquant(synth.normal_weights(n, k, seed=seed, stream=i, device=device), dt)
            self.views[name] = op.TensorView(raw, dt, k, n)
            self.weights[name] = op.Weight(ctx, self.views[name], shard=plan.shard(name))
        # one input per group: the projections of a group read the same activations
        for gi, group in enumerate(self.GROUPS):
            k = self.projs[group[0]][0]
            for m in token_counts:
                full = synth.normal_activations(m, k, seed=seed, stream=1000 + gi, device=device)
                self.x[(gi, m)] = full[:, plan.input_slice(group[0], k)].contiguous()
                for name in group:
                    self.y[(name, m)] = torch.empty((m, self.weights[name].n_out), dtype=torch.float32, device=device)
        self.launches_per_pass = len(self.GROUPS)
        if autotune:  # load-time: measured launch plans for the four launches of a pass
            for group in self.GROUPS:
                kern.autotune([self.weights[n] for n in group], max_tokens=min(16, max(token_counts)))

    def full_input(self, gi: int, m: int, seed: int = 0) -> torch.Tensor:
        """The unsharded activations that group gi reads at m tokens (what x[(gi, m)] is a column slice of)."""
        return synth.normal_activations(m, self.projs[self.GROUPS[gi][0]][0], seed=seed, stream=1000 + gi, device=self.dev)

    def launch_group(self, gi: int, m: int, weights=None) -> None:
        group = self.GROUPS[gi]
        ws = weights or [self.weights[n] for n in group]
        ys = [self.y[(n, m)] for n in group]
        reduce = self.all_reduce is not None and self.plan.needs_all_reduce(group[0])
        if len(group) == 1 or m > 16:
            for w, y in zip(ws, ys):
                # fused: the projection pushes its partial sums to the peers itself and the call completes the sum
                self.kern.encode_quantized_matmul(w, self.x[(gi, m)], y, m, all_reduce=reduce and self.fuse_all_reduce)
        else:
            self.kern.encode_quantized_matmul_group(ws, self.x[(gi, m)], ys, m)
        if reduce and not self.fuse_all_reduce:
            self.all_reduce(ys[0])

    def run(self, m: int) -> None:
        for gi in range(len(self.GROUPS)):
            self.launch_group(gi, m)

    def pass_bytes(self, m: int, x_bytes: int = 2) -> int:
        """Algorithmic bytes of one pass over the UNSHARDED layer at m tokens (whole-job accounting)."""
        return sum(kquant_call_bytes(k, n, dt, m, x_bytes) for (k, n, dt) in self.projs.values())

    def pass_flops(self, m: int) -> float:
        return 2.0 * m * sum(k * n for (k, n, _) in self.projs.values())


class PrefillLayer:
    """One layer's NVFP4 linears at `tokens` tokens (BASELINE config 4 runs 52 of them back to back; all layers
    reuse these weights, which at 274 MB do not fit L2, so every layer still streams them from HBM).

    act_dtype: dtype of the activations between the projections (bf16 in the benchmark; f32 in the parity test so
    that the CPU lane's composition can be followed without modelling bf16 roundings)."""

    def __init__(self, ctx, kern, plan: tp.ShardPlan, tokens: int, device, all_reduce=None, chunks: int = 1,
                 act_dtype=torch.bfloat16, eps: float = 1e-6, requant: bool = True):
        self.ctx, self.kern, self.plan, self.M, self.eps, self.dev = ctx, kern, plan, tokens, eps, device
        self.requant = requant  # silu(gate) * up leaves its GEMM as NVFP4 codes for down_proj (never as numbers)
        self.all_reduce = all_reduce
        P = self.P = synth.LAYER_PROJECTIONS
        H, F, world, M = P["attn_q"][0], P["ffn_gate"][1], plan.world, tokens
        self.h = synth.normal_activations(M, H, device=device).to(act_dtype)
        self.norm_w = [torch.ones(H, device=device) + 0.1 * torch.randn(H, device=device, generator=torch.Generator(device).manual_seed(s))
                       for s in (1, 2)]

        def rms(x, w):
            xf = x.float()
            return xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * w

        # static input scales per projection input, fixed from this seeded data as a stored checkpoint would carry them
        sample = slice(0, min(M, 1024))
        dense = {name: synth.normal_weights(n, k, seed=0, stream=i, device=device) for i, (name, (k, n, _)) in enumerate(P.items())}
        isi_attn = synth.activation_input_scale_inv(rms(self.h[sample], self.norm_w[0]))
        isi_ffn = synth.activation_input_scale_inv(rms(self.h[sample], self.norm_w[1]))
        isi_o = synth.activation_input_scale_inv(rms(self.h[sample], self.norm_w[0]) @ dense["attn_q"].t())
        act = torch.nn.functional.silu(rms(self.h[sample], self.norm_w[1]) @ dense["ffn_gate"].t()) * (rms(self.h[sample], self.norm_w[1]) @ dense["ffn_up"].t())
        isi_down = synth.activation_input_scale_inv(act)
        self.isi = {"attn_q": isi_attn, "attn_k": isi_attn, "attn_v": isi_attn, "attn_o": isi_o, "ffn_gate": isi_ffn,
                    "ffn_up": isi_ffn, "ffn_down": isi_down}
        self.stored, self.weights = {}, {}
        for name, (k, n, _) in P.items():
            wp, wsc, s2 = synth.nvfp4_weight(dense[name])
            self.stored[name] = (wp, wsc, s2)
            self.weights[name] = op.Weight(ctx, op.TensorView(wp, op.NVFP4, k, n, wsc, s2, self.isi[name]), shard=plan.shard(name))
        del dense, act
        Ql, KVl, Fl = P["attn_q"][1] // world, P["attn_k"][1] // world, F // world
        kw = dict(dtype=act_dtype, device=device)
        self.q, self.k, self.v = torch.empty((M, Ql), **kw), torch.empty((M, KVl), **kw), torch.empty((M, KVl), **kw)
        self.ffn_act, self.h1, self.h2 = torch.empty((M, Fl), **kw), torch.empty((M, H), **kw), torch.empty((M, H), **kw)
        self.xq = (torch.empty((M, H // 2), dtype=torch.uint8, device=device),
                   torch.empty((op._L.muser_cuda_nvfp4_swizzled_scale_bytes(M, H),), dtype=torch.uint8, device=device))
        self.fq = (torch.empty((M, Fl // 2), dtype=torch.uint8, device=device),
                   torch.empty((op._L.muser_cuda_nvfp4_swizzled_scale_bytes(M, Fl),), dtype=torch.uint8, device=device))
        self.Fl = Fl
        chunks = max(1, chunks if world > 1 else 1)
        step = (M + chunks - 1) // chunks // 128 * 128 or M
        self.bounds = [(a, min(M, a + step)) for a in range(0, M, step)]
        self.macs_per_token = sum(k * n for k, n, _ in P.values())

    @staticmethod
    def workspace_bytes(tokens: int, world: int) -> int:
        F = synth.LAYER_PROJECTIONS["ffn_gate"][1]
        return (tokens + 128) * (F // world // 2 + F // world // 16 + 64) + (1 << 20)

    def _row_parallel(self, name, x, res, out):
        """out = all_reduce(x @ W_shard^T) + res, in token chunks; the residual is added on rank 0's partial sum.
        x: activations, or (codes, swizzled scales) of activations quantized earlier."""
        for a, b in self.bounds:
            residual = res[a:b] if self.plan.rank == 0 else None
            if isinstance(x, tuple):
                chunk_bytes = (x[0].shape[1] * 2 + 63) // 64 * 512  # scale bytes per 128-row block
                self.kern.encode_nvfp4_prequant(self.weights[name], x[0][a:b], x[1][(a // 128) * chunk_bytes:], out[a:b], b - a, residual=residual)
            else:
                self.kern.encode_nvfp4_matmul(self.weights[name], x[a:b], out[a:b], b - a, residual=residual)
            if self.all_reduce is not None and self.plan.world > 1:
                self.all_reduce(out[a:b])

    def layer(self, x):
        k, W, M = self.kern, self.weights, self.M
        k.quantize_nvfp4_activation(x, self.isi["attn_q"], norm_weight=self.norm_w[0], norm_eps=self.eps, out=self.xq)
        # q | k | v read the same quantized activations: one launch over all their output tiles
        k.encode_nvfp4_group_prequant([W["attn_q"], W["attn_k"], W["attn_v"]], self.xq[0], self.xq[1], [self.q, self.k, self.v], M)
        self._row_parallel("attn_o", self.q, x, self.h1)
        if self.requant:
            k.quantize_nvfp4_activation(self.h1, self.isi["ffn_gate"], norm_weight=self.norm_w[1], norm_eps=self.eps, out=self.xq)
            k.encode_nvfp4_ffn_gate_up_silu_requant(W["ffn_gate"], W["ffn_up"], self.xq[0], self.xq[1], M, self.isi["ffn_down"],
                                                    out_packed=self.fq[0], out_scales=self.fq[1])
            self._row_parallel("ffn_down", self.fq, self.h1, self.h2)
        else:
            k.encode_ffn_gate_up_silu(W["ffn_gate"], W["ffn_up"], self.h1, self.ffn_act, M, norm_weight=self.norm_w[1], norm_eps=self.eps)
            self._row_parallel("ffn_down", self.ffn_act, self.h1, self.h2)
        return self.h2

    def run(self, layers: int):
        x = self.h
        for _ in range(layers):
            x = self.layer(x)  # h2 feeds the next layer; its values do not matter to the timing, only its shape
        return x

    def flops(self, layers: int) -> float:
        return 2.0 * self.M * self.macs_per_token * layers
