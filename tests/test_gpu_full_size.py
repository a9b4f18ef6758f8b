"""Parity at the benchmark's own sizes: every NVFP4 projection of the layer at 2048 tokens, the fused gate/up form at
27648 rows, one whole prefill layer at 32768 tokens, and the attention projections at the speculative-verify token
counts, each on sampled token rows (or output rows) against the CPU lane."""
import numpy as np
import pytest
import torch

from oracle import oracle as O
from tests import helpers as H

pytestmark = pytest.mark.gpu
REL_L2_TOL = 1e-3


@pytest.fixture(scope="module")
def gpu():
    from muser_b200 import operator as op
    ctx = op.Context(0, workspace_bytes=1 << 30)
    yield op, ctx, op.CudaKernels(ctx)
    ctx.close()


def _nvfp4_projection(op, ctx, name, tokens, seed_stream):
    from muser_b200 import synth
    n_in, n_out, _ = synth.LAYER_PROJECTIONS[name]
    packed, scales, scale2 = synth.nvfp4_weight(synth.normal_weights(n_out, n_in, seed=0, stream=seed_stream, device="cuda"))
    x = synth.normal_activations(tokens, n_in, seed=0, stream=3000 + seed_stream, device="cuda")
    isi = synth.activation_input_scale_inv(x)
    w = op.Weight(ctx, op.TensorView(packed, O.NVFP4, n_in, n_out, scales, scale2, isi))
    ow = O.TensorView(packed.cpu().numpy(), O.NVFP4, n_in, n_out, scales.cpu().numpy(), scale2, isi)
    return w, ow, x, n_in, n_out


@pytest.mark.parametrize("name", ["attn_q", "attn_o", "ffn_gate", "ffn_up", "ffn_down"])
def test_nvfp4_projection_at_2048_tokens(gpu, name):
    """BASELINE config 3: M = 2048 on the layer's own shapes; 64 sampled token rows x all outputs against the CPU
    lane's W4A4 dot (the value before its final f16 rounding), rel-L2 <= 1e-3."""
    op, ctx, k = gpu
    from muser_b200 import synth
    tokens = 2048
    w, ow, x, n_in, n_out = _nvfp4_projection(op, ctx, name, tokens, list(synth.LAYER_PROJECTIONS).index(name))
    y = torch.empty((tokens, n_out), dtype=torch.float32, device="cuda")
    k.encode_nvfp4_matmul(w, x, y, tokens)
    ctx.sync_status()
    rows = torch.randperm(tokens, generator=torch.Generator().manual_seed(1))[:64].cuda()
    _, ref = O.matmul(ow, x[rows].float().cpu().numpy(), threads=O.host_threads(), return_pre_round=True)
    assert H.rel_l2(y[rows].cpu().numpy(), ref) <= REL_L2_TOL, name
    w.free()


def test_nvfp4_fused_gate_up_silu_at_full_size(gpu):
    """The fused FFN front half at 27648 rows and 2048 tokens: silu(f16(gate)) * f16(up) on 64 sampled token rows."""
    op, ctx, k = gpu
    from muser_b200 import synth
    tokens, names = 2048, list(synth.LAYER_PROJECTIONS)
    n_in, n_out, _ = synth.LAYER_PROJECTIONS["ffn_gate"]
    x = synth.normal_activations(tokens, n_in, seed=0, stream=3100, device="cuda")
    isi = synth.activation_input_scale_inv(x)
    ws, ows = [], []
    for nm in ("ffn_gate", "ffn_up"):
        p, s, s2 = synth.nvfp4_weight(synth.normal_weights(n_out, n_in, seed=0, stream=names.index(nm), device="cuda"))
        ws.append(op.Weight(ctx, op.TensorView(p, O.NVFP4, n_in, n_out, s, s2, isi)))
        ows.append(O.TensorView(p.cpu().numpy(), O.NVFP4, n_in, n_out, s.cpu().numpy(), s2, isi))
    y = torch.empty((tokens, n_out), dtype=torch.float32, device="cuda")
    k.encode_ffn_gate_up_silu(ws[0], ws[1], x, y, tokens)
    ctx.sync_status()
    rows = torch.randperm(tokens, generator=torch.Generator().manual_seed(2))[:64].cuda()
    xs = x[rows].float().cpu().numpy()
    g = O.matmul(ows[0], xs, threads=O.host_threads())   # f16-rounded, as the W4A4 lane returns it
    u = O.matmul(ows[1], xs, threads=O.host_threads())
    assert H.rel_l2(y[rows].cpu().numpy(), O.silu_mul(g, u)) <= REL_L2_TOL
    for w in ws:
        w.free()


def test_one_prefill_layer_at_32768_tokens():
    """BASELINE config 4, one layer: norm -> quantize -> q / k / v, o + residual, norm -> gate | up + SwiGLU, down +
    residual at 32768 tokens, activations between the projections kept in f32 so that the CPU lane's composition can
    be followed step by step; 16 sampled token rows of q, of the attention-block output and of the layer output."""
    from muser_b200 import operator as op
    from muser_b200 import tp, workloads
    M = 32768
    ctx = op.Context(0, workspace_bytes=workloads.PrefillLayer.workspace_bytes(M, 1))
    k = op.CudaKernels(ctx)
    pl = workloads.PrefillLayer(ctx, k, tp.ShardPlan(0, 1), M, "cuda", act_dtype=torch.float32, requant=False)
    # first the form the benchmark runs: silu(gate) * up leaves its GEMM as NVFP4 codes.  With f32 activations in
    # between, the separate path quantizes exactly the numbers the fused epilogue holds, so the layer outputs must
    # carry the same bits.
    pl.requant = True
    h2_fused = pl.layer(pl.h).clone()
    pl.requant = False
    pl.layer(pl.h)
    ctx.sync_status()
    assert torch.equal(h2_fused.view(torch.int32), pl.h2.view(torch.int32))
    del h2_fused
    rows = torch.randperm(M, generator=torch.Generator().manual_seed(3))[:16].cuda()
    thr = O.host_threads()

    def lane(name, x):
        wp, wsc, s2 = pl.stored[name]
        kk, n, _ = pl.P[name]
        ow = O.TensorView(wp.cpu().numpy(), O.NVFP4, kk, n, wsc.cpu().numpy(), s2, pl.isi[name])
        return O.matmul(ow, x, threads=thr, return_pre_round=True)

    nw = [w.cpu().numpy() for w in pl.norm_w]
    h = pl.h[rows].float().cpu().numpy()
    xn = O.rms_norm_mul(h, pl.eps, nw[0])
    _, q = lane("attn_q", xn)
    assert H.rel_l2(pl.q[rows].cpu().numpy(), q) <= REL_L2_TOL
    # from here the CPU composition continues from the GPU's own intermediate, so that every stage is judged alone
    q_gpu = pl.q[rows].cpu().numpy()
    _, o = lane("attn_o", q_gpu)
    h1 = o + h
    assert H.rel_l2(pl.h1[rows].cpu().numpy(), h1) <= REL_L2_TOL
    h1_gpu = pl.h1[rows].cpu().numpy()
    xf = O.rms_norm_mul(h1_gpu, pl.eps, nw[1])
    g16, _ = lane("ffn_gate", xf)
    u16, _ = lane("ffn_up", xf)
    act = O.silu_mul(g16, u16)
    assert H.rel_l2(pl.ffn_act[rows].cpu().numpy(), act) <= REL_L2_TOL
    act_gpu = pl.ffn_act[rows].cpu().numpy()
    _, d = lane("ffn_down", act_gpu)
    assert H.rel_l2(pl.h2[rows].cpu().numpy(), d + h1_gpu) <= REL_L2_TOL
    del pl
    ctx.close()


@pytest.mark.parametrize("name", ["attn_q", "attn_k", "attn_v", "attn_o"])
def test_kquant_attention_projections_at_verify_token_counts(gpu, name):
    """BASELINE config 5 on the attention projections at full size: 16, 32 and 64 tokens, 96 sampled output rows
    (all rows for the 1024-row k and v) against the CPU lane."""
    op, ctx, k = gpu
    from muser_b200 import synth
    n_in, n_out, dtype = synth.LAYER_PROJECTIONS[name]
    raw = synth.quantize_kquant(synth.normal_weights(n_out, n_in, seed=0, stream=21, device="cuda"), dtype)
    w = op.Weight(ctx, op.TensorView(raw, dtype, n_in, n_out))
    rows = np.sort(np.random.default_rng(5).choice(n_out, 96, replace=False)) if n_out > 1024 else np.arange(n_out)
    ow = O.TensorView(raw.cpu().numpy().reshape(n_out, -1)[rows].copy(), dtype, n_in, len(rows))
    for tokens in (16, 32, 64):
        x = synth.normal_activations(tokens, n_in, seed=tokens, device="cuda")
        y = torch.full((tokens, n_out), float("nan"), dtype=torch.float32, device="cuda")
        k.encode_quantized_matmul(w, x, y, tokens)
        ctx.sync_status()
        ref = O.matmul(ow, x.float().cpu().numpy(), threads=O.host_threads())
        err = H.rel_l2(y[:, torch.from_numpy(rows).cuda()].cpu().numpy(), ref)
        assert err <= REL_L2_TOL, (name, tokens, err)
    w.free()


def test_host_enqueue_entry_point_matches_the_blocking_one(gpu):
    """muser_cuda_matmul_host_enqueue: several projections enqueued on pinned host buffers, one wait, against the
    blocking host entry point; and a step larger than the staging arena (the call then waits once by itself)."""
    op, ctx, k = gpu
    raw4 = H.lcg_weights(O.Q4_K, 300, 4, seed=5)
    raw6 = H.lcg_weights(O.Q6_K, 64, 4, seed=6)
    ws = [op.Weight(ctx, op.TensorView(raw4, O.Q4_K, 1024, 300)), op.Weight(ctx, op.TensorView(raw6, O.Q6_K, 1024, 64))]
    stream = torch.cuda.current_stream().cuda_stream
    calls = []
    for i, (w, n_out) in enumerate(zip(ws, (300, 64))):
        for tokens in (1, 5, 70):
            x = torch.from_numpy(H.lcg_activations(tokens * 1024, seed=10 * tokens + i).reshape(tokens, 1024)).pin_memory()
            y = torch.full((tokens, n_out), float("nan")).pin_memory()
            calls.append((w, x, y, tokens))
    for w, x, y, tokens in calls:
        op.matmul_enqueue(ctx, w, x.data_ptr(), tokens, y.data_ptr(), stream)
    ctx.sync_status()
    for w, x, y, tokens in calls:
        want = op.matmul(ctx, w, x.numpy(), tokens)
        assert H.rel_l2(y.numpy(), want) <= 1e-6, tokens
    big_w, big_ow = ws[0], O.TensorView(raw4, O.Q4_K, 1024, 300)
    x = torch.from_numpy(H.lcg_activations(64 * 1024, seed=3).reshape(64, 1024)).pin_memory()
    ys = [torch.empty((64, 300)).pin_memory() for _ in range(300)]   # 300 calls x ~340 KB of staging > 64 MiB
    for y in ys:
        op.matmul_enqueue(ctx, big_w, x.data_ptr(), 64, y.data_ptr(), stream)
    ctx.sync_status()
    want = O.matmul(big_ow, x.numpy(), threads=O.host_threads())
    assert H.rel_l2(ys[0].numpy(), want) <= REL_L2_TOL and torch.equal(ys[0], ys[-1])
    for w in ws:
        w.free()


def test_a_step_of_grouped_projections_through_host_buffers(gpu):
    """muser_cuda_matmul_host_groups_enqueue: a step's groups (q | k | v of mixed Q4_K / Q6_K, a single projection, a
    pair) in one call, outputs written by the kernels into pinned host buffers, or copied back where the caller's
    buffer is ordinary pageable memory; compared with the CPU lane and with the per-projection host entry."""
    op, ctx, k = gpu
    n_in = 1024
    shapes = [(O.Q4_K, 700), (O.Q4_K, 130), (O.Q6_K, 130), (O.Q4_K, 1024), (O.Q5_K, 333)]
    raws = [H.lcg_weights(dt, n, n_in // 256, seed=60 + i) for i, (dt, n) in enumerate(shapes)]
    ws = [op.Weight(ctx, op.TensorView(r, dt, n_in, n)) for r, (dt, n) in zip(raws, shapes)]
    stream = torch.cuda.current_stream().cuda_stream
    groups, expect = [], []
    for tokens in (1, 4, 8, 16):
        for members, pinned in (((0, 1, 2), True), ((3,), False), ((4,), True), ((0, 3), True)):
            x = torch.from_numpy(H.lcg_activations(tokens * n_in, seed=7 * tokens + len(members)).reshape(tokens, n_in)).pin_memory()
            ys = [torch.full((tokens, shapes[i][1]), float("nan")) for i in members]
            ys = [y.pin_memory() if pinned else y for y in ys]
            groups.append(([ws[i] for i in members], x.data_ptr(), tokens, [y.data_ptr() for y in ys]))
            expect.append((members, x, ys, tokens))
    calls = op.host_groups(groups)
    for _ in range(2):  # the list is reusable step after step
        op.matmul_groups_enqueue(ctx, calls, stream)
        ctx.sync_status()
    for members, x, ys, tokens in expect:
        for i, y in zip(members, ys):
            dt, n = shapes[i]
            want = O.matmul(O.TensorView(raws[i], dt, n_in, n), x.numpy(), threads=4)
            assert H.rel_l2(y.numpy(), want) <= REL_L2_TOL, (members, tokens)
            single = torch.empty_like(y).pin_memory()
            op.matmul_enqueue(ctx, ws[i], x.data_ptr(), tokens, single.data_ptr(), stream)
            ctx.sync_status()
            assert H.rel_l2(y.numpy(), single.numpy()) <= 1e-5
    bad = op.host_groups([([ws[0]], 0, 4, [0])])
    with pytest.raises(op.MuserCudaError) as e:
        op.matmul_groups_enqueue(ctx, bad, stream)
    assert e.value.status_name in ("BAD_ARG", "BAD_SHAPE")
    for w in ws:
        w.free()


def test_host_groups_call_replayed_from_a_cuda_graph(gpu):
    """The host-buffer step captured once and replayed: every replay reads the pinned inputs as they are then and
    rewrites the pinned outputs."""
    op, ctx, k = gpu
    from muser_b200 import workloads
    n_in = 1024
    raws = [H.lcg_weights(O.Q4_K, 300, 4, seed=90), H.lcg_weights(O.Q6_K, 200, 4, seed=91)]
    ws = [op.Weight(ctx, op.TensorView(raws[0], O.Q4_K, n_in, 300)), op.Weight(ctx, op.TensorView(raws[1], O.Q6_K, n_in, 200))]
    x = torch.from_numpy(H.lcg_activations(4 * n_in, seed=1).reshape(4, n_in)).pin_memory()
    ys = [torch.full((4, 300), float("nan")).pin_memory(), torch.full((4, 200), float("nan")).pin_memory()]
    calls = op.host_groups([(ws, x.data_ptr(), 4, [y.data_ptr() for y in ys]), ([ws[1]], x.data_ptr(), 4, [ys[1].data_ptr()])])
    op.matmul_groups_enqueue(ctx, calls, torch.cuda.current_stream().cuda_stream)
    ctx.sync_status()
    replay = workloads.capture(lambda: op.matmul_groups_enqueue(ctx, calls, torch.cuda.current_stream().cuda_stream))
    for seed in (2, 3):
        x.copy_(torch.from_numpy(H.lcg_activations(4 * n_in, seed=seed).reshape(4, n_in)))
        for y in ys:
            y.fill_(float("nan"))
        replay()
        ctx.sync_status()
        for raw, dt, n, y in ((raws[0], O.Q4_K, 300, ys[0]), (raws[1], O.Q6_K, 200, ys[1])):
            want = O.matmul(O.TensorView(raw, dt, n_in, n), x.numpy(), threads=4)
            assert H.rel_l2(y.numpy(), want) <= REL_L2_TOL, seed
    for w in ws:
        w.free()
