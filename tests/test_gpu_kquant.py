"""GPU parity of the K-quant path (through the C ABI) against the CPU oracle."""
import numpy as np
import pytest
import torch

from oracle import oracle as O
from tests import helpers as H

pytestmark = pytest.mark.gpu

REL_L2_TOL = 1e-3          # the stated bound: relative L2 against the f32-accumulating CPU lane
REF_REL, REF_ABS = 2e-4, 0.02  # the reference's own envelope for f32-order kernels (metal.rs:213)


@pytest.fixture(scope="module")
def gpu():
    from muser_b200 import operator as op
    ctx = op.Context(0)
    yield op, ctx, op.CudaKernels(ctx)
    ctx.close()


def fixtures(dtype):
    from muser_b200 import synth
    bs = O.BLOCK_BYTES[dtype]
    if dtype != O.Q5_K:   # the reference's closed-form rows exist for Q4_K and Q6_K
        closed = H.quant_rows(144, 64) if dtype == O.Q4_K else H.q6_rows(64)
        assert closed.shape[1] == bs
        yield "closed-form", closed, 256, 64
    yield "lcg-13x512", H.lcg_weights(dtype, 13, 2, seed=41 + dtype), 512, 13
    yield "lcg-37x1024", H.lcg_weights(dtype, 37, 4, seed=97 + dtype), 1024, 37
    if dtype != O.Q5_K:
        w = synth.normal_weights(48, 2048, seed=0, stream=dtype)
        yield "synthetic-48x2048", synth.quantize_kquant(w, dtype).numpy(), 2048, 48
    else:
        yield "lcg-300x2048", H.lcg_weights(dtype, 300, 8, seed=5), 2048, 300


@pytest.mark.parametrize("dtype", [O.Q4_K, O.Q5_K, O.Q6_K])
def test_dequantised_weights_are_bit_exact(gpu, dtype):
    op, ctx, k = gpu
    for name, raw, n_in, n_out in fixtures(dtype):
        w = op.Weight(ctx, op.TensorView(raw, dtype, n_in, n_out))
        got = k.dequant(w).cpu().numpy()
        want = O.dequant_blocks(dtype, raw).reshape(n_out, n_in)
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), name
        w.free()


FIXED_POINT = 2.0 ** -15   # decode kernel (up to 16 tokens): activations are 15-bit fixed point per 256-input tile


def fixed_point_magnitude(x, w_abs):
    """sum over 256-input tiles of amax(x, tile) * sum(|w|, tile): what the decode kernel's rounding of one activation
    (at most amax(tile) * 2^-15) can move an output by, per unit of FIXED_POINT."""
    tokens, n_in = x.shape
    amax = np.abs(x).reshape(tokens, n_in // 256, 256).max(axis=2).astype(np.float64)
    w_tile = w_abs.reshape(w_abs.shape[0], n_in // 256, 256).sum(axis=2)
    return amax @ w_tile.T


def check_close(got, want, name, magnitude=None):
    """Relative L2 is the gate.  Element-wise, the reference's envelope, widened where the dot product cancels
    by the activation fixed-point step times the tile-wise sum amax |w| (the decode kernel's documented error bound)."""
    assert H.rel_l2(got, want) <= REL_L2_TOL, (name, H.rel_l2(got, want))
    bound = np.maximum(REF_ABS, REF_REL * np.abs(want))
    if magnitude is not None:
        bound = np.maximum(bound, FIXED_POINT * magnitude)
    assert np.all(np.abs(got - want) <= bound), (name, float(np.max(np.abs(got - want) / bound)))


@pytest.mark.parametrize("dtype", [O.Q4_K, O.Q5_K, O.Q6_K])
@pytest.mark.parametrize("x_dtype", [torch.bfloat16, torch.float32])
def test_matmul_matches_cpu_lane(gpu, dtype, x_dtype):
    op, ctx, k = gpu
    for name, raw, n_in, n_out in fixtures(dtype):
        w = op.Weight(ctx, op.TensorView(raw, dtype, n_in, n_out))
        ow = O.TensorView(raw, dtype, n_in, n_out)
        w_abs = np.abs(O.dequant_blocks(dtype, raw).reshape(n_out, n_in)).astype(np.float64)
        for tokens in (1, 2, 3, 4, 8, 9, 16, 33, 64):
            x = torch.from_numpy(H.lcg_activations(tokens * n_in, seed=5 + tokens).reshape(tokens, n_in)).to(x_dtype)
            want = O.matmul(ow, x.float().numpy(), threads=4)
            y = torch.full((tokens, n_out), float("nan"), dtype=torch.float32, device="cuda")
            k.encode_quantized_matmul(w, x.cuda(), y, tokens)
            check_close(y.cpu().numpy(), want, (name, tokens), fixed_point_magnitude(x.float().numpy(), w_abs))
        w.free()


@pytest.mark.parametrize("dtype", [O.Q4_K, O.Q6_K])
def test_activations_beyond_the_f16_range(gpu, dtype):
    """bf16 and f32 activations can exceed f16's range (|x| > 65504).  The decode kernel (up to 16 tokens, and longer
    batches on weights below the tcgen05 kernel's row threshold) scales every 256-input tile by its own maximum, so
    such inputs cost nothing; the tcgen05 kernel (17-64 tokens) takes activations as f16 and clamps them: the stated
    range limit of that kernel, checked here so that it stays a clamp and never becomes inf or NaN."""
    from muser_b200._lib import TUNE_TC_MIN_ROWS
    op, ctx, k = gpu
    n_in, n_out = 1024, 1100
    raw = H.lcg_weights(dtype, n_out, n_in // 256, seed=71 + dtype)
    w = op.Weight(ctx, op.TensorView(raw, dtype, n_in, n_out))
    ow = O.TensorView(raw, dtype, n_in, n_out)
    for x_dtype in (torch.bfloat16, torch.float32):
        for tokens in (1, 4, 16, 24):
            x = torch.from_numpy(H.lcg_activations(tokens * n_in, seed=9 + tokens).reshape(tokens, n_in)).clone()
            x[0, 5], x[tokens - 1, 700], x[0, 300] = 3.0e5, -1.0e6, 7.0e4
            x = x.to(x_dtype)
            want = O.matmul(ow, x.float().numpy(), threads=4)
            y = torch.full((tokens, n_out), float("nan"), dtype=torch.float32, device="cuda")
            try:
                ctx.tuning_set(TUNE_TC_MIN_ROWS, 1 << 30)  # every token count through the decode kernel
                k.encode_quantized_matmul(w, x.cuda(), y, tokens)
                ctx.sync_status()
            finally:
                ctx.tuning_set(TUNE_TC_MIN_ROWS, 1024)
            assert H.rel_l2(y.cpu().numpy(), want) <= REL_L2_TOL, (x_dtype, tokens, H.rel_l2(y.cpu().numpy(), want))
        # the tcgen05 kernel on the same 24 tokens: finite, and equal to the CPU lane on the clamped activations
        tokens = 24
        y = torch.full((tokens, n_out), float("nan"), dtype=torch.float32, device="cuda")
        k.encode_quantized_matmul(w, x.cuda(), y, tokens)
        ctx.sync_status()
        assert torch.isfinite(y).all()
        want_clamped = O.matmul(ow, x.float().clamp(-65504.0, 65504.0).numpy(), threads=4)
        assert H.rel_l2(y.cpu().numpy(), want_clamped) <= REL_L2_TOL, (x_dtype, H.rel_l2(y.cpu().numpy(), want_clamped))
    w.free()


def test_epilogue_row_scale_residual_and_bf16_output(gpu):
    op, ctx, k = gpu
    raw = H.lcg_weights(O.Q4_K, 37, 2, seed=3)
    w = op.Weight(ctx, op.TensorView(raw, O.Q4_K, 512, 37))
    x = torch.from_numpy(H.lcg_activations(5 * 512, seed=8).reshape(5, 512)).to(torch.bfloat16)
    base = O.matmul(O.TensorView(raw, O.Q4_K, 512, 37), x.float().numpy())
    rs = torch.tensor([0.5, 2.0, 1.0, -1.5, 0.25], device="cuda")
    res = torch.from_numpy(H.lcg_activations(5 * 37, seed=2).reshape(5, 37)).cuda()
    y = torch.empty((5, 37), dtype=torch.float32, device="cuda")
    k.encode_quantized_matmul(w, x.cuda(), y, 5, row_scale=rs, residual=res)
    want = base * rs.cpu().numpy()[:, None] + res.cpu().numpy()
    assert H.rel_l2(y.cpu().numpy(), want) <= 1e-4
    yb = torch.empty((5, 37), dtype=torch.bfloat16, device="cuda")
    k.encode_quantized_matmul(w, x.cuda(), yb, 5)
    assert np.allclose(yb.float().cpu().numpy(), base, rtol=1e-2, atol=1e-2)


@pytest.mark.parametrize("dtype", [O.Q4_K, O.Q6_K])
def test_fused_gate_up_silu(gpu, dtype):
    op, ctx, k = gpu
    n_in, n_out = 1024, 37
    rg, ru = H.lcg_weights(dtype, n_out, 4, seed=21), H.lcg_weights(dtype, n_out, 4, seed=22)
    wg, wu = (op.Weight(ctx, op.TensorView(r, dtype, n_in, n_out)) for r in (rg, ru))
    for tokens in (1, 4, 11):
        x = torch.from_numpy(H.lcg_activations(tokens * n_in, seed=6).reshape(tokens, n_in) * 0.3).to(torch.bfloat16)
        g = O.matmul(O.TensorView(rg, dtype, n_in, n_out), x.float().numpy())
        u = O.matmul(O.TensorView(ru, dtype, n_in, n_out), x.float().numpy())
        want = O.silu_mul(g, u)
        y = torch.empty((tokens, n_out), dtype=torch.float32, device="cuda")
        k.encode_ffn_gate_up_silu(wg, wu, x.cuda(), y, tokens)
        assert H.rel_l2(y.cpu().numpy(), want) <= REL_L2_TOL


@pytest.mark.parametrize("dtype", [O.Q4_K, O.Q6_K])
@pytest.mark.parametrize("x_dtype", [torch.bfloat16, torch.float32])
def test_fused_input_rmsnorm(gpu, dtype, x_dtype):
    """rms_norm_mul (reference.rs:59-80) fused in front of the projection: the decode kernel norms while it stages
    the activations (bf16, few tokens), the skinny kernel behind a pass of its own; both against the CPU lane's
    norm followed by weights::matmul."""
    op, ctx, k = gpu
    n_in, n_out, eps = 1024, 37, 1e-6
    raw = H.lcg_weights(dtype, n_out, 4, seed=31)
    raw_up = H.lcg_weights(dtype, n_out, 4, seed=32)
    w, wu = (op.Weight(ctx, op.TensorView(r, dtype, n_in, n_out)) for r in (raw, raw_up))
    nw = torch.linspace(0.5, 1.5, n_in)
    for tokens in (1, 2, 5, 8, 19):
        x = torch.from_numpy(H.lcg_activations(tokens * n_in, seed=tokens).reshape(tokens, n_in) * 3.0).to(x_dtype)
        xn = O.rms_norm_mul(x.float().numpy(), eps, nw.numpy())
        want = O.matmul(O.TensorView(raw, dtype, n_in, n_out), xn)
        y = torch.empty((tokens, n_out), dtype=torch.float32, device="cuda")
        k.encode_quantized_matmul(w, x.cuda(), y, tokens, norm_weight=nw.cuda(), norm_eps=eps)
        assert H.rel_l2(y.cpu().numpy(), want) <= REL_L2_TOL, (tokens, H.rel_l2(y.cpu().numpy(), want))
        if tokens <= 16:
            want_ffn = O.silu_mul(want, O.matmul(O.TensorView(raw_up, dtype, n_in, n_out), xn))
            k.encode_ffn_gate_up_silu(w, wu, x.cuda(), y, tokens, norm_weight=nw.cuda(), norm_eps=eps)
            assert H.rel_l2(y.cpu().numpy(), want_ffn) <= REL_L2_TOL, tokens
    ctx.sync_status()
    # a K shard sees only part of the row: refused
    wk = op.Weight(ctx, op.TensorView(raw, dtype, n_in, n_out), shard=(0, 2, op.SHARD_K))
    with pytest.raises(op.MuserCudaError) as e:
        k.encode_quantized_matmul(wk, torch.zeros((1, n_in // 2), dtype=x_dtype, device="cuda"),
                                  torch.empty((1, n_out), dtype=torch.float32, device="cuda"), 1, norm_weight=nw.cuda())
    assert e.value.status_name == "BAD_SHAPE"


@pytest.mark.parametrize("dtype", [O.Q4_K, O.Q6_K])
@pytest.mark.parametrize("x_dtype", [torch.bfloat16, torch.float32])
def test_tensor_core_skinny_kernel(gpu, dtype, x_dtype):
    """The tcgen05 kernel (exact integer f16 operands, per-super-block drain) forced for every token count it serves,
    on shapes with a short last row block, one to many K slices, and the fused row scale / residual; then the same
    calls with that kernel switched off, which sends them through the decode kernel in chunks of 16 tokens."""
    op, ctx, k = gpu
    key = op.TUNE_TC_MIN_TOKENS_Q4_K if dtype == O.Q4_K else op.TUNE_TC_MIN_TOKENS_Q6_K
    shapes = [(512, 13, 2), (1024, 37, 4), (2048, 300, 8)]
    try:
        ctx.tuning_set(op.TUNE_TC_MIN_ROWS, 1)
        for threshold in (1, 65):
            ctx.tuning_set(key, threshold)
            for n_in, n_out, blocks in shapes:
                raw = H.lcg_weights(dtype, n_out, blocks, seed=n_out + dtype)
                w = op.Weight(ctx, op.TensorView(raw, dtype, n_in, n_out))
                for tokens in (3, 9, 16, 17, 40, 64):
                    x = torch.from_numpy(H.lcg_activations(tokens * n_in, seed=tokens).reshape(tokens, n_in)).to(x_dtype)
                    want = O.matmul(O.TensorView(raw, dtype, n_in, n_out), x.float().numpy(), threads=O.host_threads())
                    y = torch.full((tokens, n_out), float("nan"), dtype=torch.float32, device="cuda")
                    k.encode_quantized_matmul(w, x.cuda(), y, tokens)
                    ctx.sync_status()
                    err = H.rel_l2(y.cpu().numpy(), want)
                    assert err <= REL_L2_TOL, (threshold, n_in, n_out, tokens, err)
                rs = torch.linspace(0.5, 2.0, 5, device="cuda")
                res = torch.randn((5, n_out), device="cuda")
                x = torch.from_numpy(H.lcg_activations(5 * n_in, seed=3).reshape(5, n_in)).to(x_dtype)
                want = O.matmul(O.TensorView(raw, dtype, n_in, n_out), x.float().numpy())
                y = torch.empty((5, n_out), dtype=torch.float32, device="cuda")
                k.encode_quantized_matmul(w, x.cuda(), y, 5, row_scale=rs, residual=res)
                assert H.rel_l2(y.cpu().numpy(), want * rs.cpu().numpy()[:, None] + res.cpu().numpy()) <= REL_L2_TOL
                w.free()
    finally:
        ctx.tuning_set(op.TUNE_TC_MIN_TOKENS_Q4_K, 17)
        ctx.tuning_set(op.TUNE_TC_MIN_TOKENS_Q6_K, 17)
        ctx.tuning_set(op.TUNE_TC_MIN_ROWS, 1024)
    ctx.sync_status()


@pytest.mark.parametrize("dtype", [O.Q4_K, O.Q5_K, O.Q6_K])
def test_tensor_parallel_shards(gpu, dtype):
    """Row shards concatenate to the unsharded result exactly; K shards sum to it within tolerance."""
    op, ctx, k = gpu
    n_in, n_out, tokens = 1280, 64, 3   # 1280 / 4 = 320 inputs per K shard = 1.25 super-blocks
    raw = H.lcg_weights(dtype, n_out, n_in // 256, seed=77)
    x = torch.from_numpy(H.lcg_activations(tokens * n_in, seed=1).reshape(tokens, n_in)).to(torch.bfloat16).cuda()
    view = op.TensorView(raw, dtype, n_in, n_out)
    full = op.Weight(ctx, view)
    y_full = torch.empty((tokens, n_out), dtype=torch.float32, device="cuda")
    k.encode_quantized_matmul(full, x, y_full, tokens)
    want_deq = O.dequant_blocks(dtype, raw).reshape(n_out, n_in)
    world = 4
    parts, acc = [], torch.zeros_like(y_full)
    for rank in range(world):
        wr = op.Weight(ctx, view, shard=(rank, world, op.SHARD_ROWS))
        yr = torch.empty((tokens, n_out // world), dtype=torch.float32, device="cuda")
        k.encode_quantized_matmul(wr, x, yr, tokens)
        parts.append(yr)
        assert np.array_equal(k.dequant(wr).cpu().numpy(), want_deq[rank * 16:(rank + 1) * 16])
        wk = op.Weight(ctx, view, shard=(rank, world, op.SHARD_K))
        ks = n_in // world
        assert np.array_equal(k.dequant(wk).cpu().numpy(), want_deq[:, rank * ks:(rank + 1) * ks])
        yk = torch.empty((tokens, n_out), dtype=torch.float32, device="cuda")
        k.encode_quantized_matmul(wk, x[:, rank * ks:(rank + 1) * ks].contiguous(), yk, tokens)
        acc += yk
    assert torch.equal(torch.cat(parts, dim=1), y_full)
    # (a K shard cuts the 256-input tiles elsewhere, so its activations round on another fixed-point grid)
    assert H.rel_l2(acc.cpu().numpy(), y_full.cpu().numpy()) <= 1e-4
    # the same K shards (first tile starts before the shard's first input on odd ranks) through the tcgen05 kernel,
    # bf16 and f32 activations, against the CPU lane on the whole tensor
    ctx.tuning_set(op.TUNE_TC_MIN_ROWS, 1)
    key = op.TUNE_TC_MIN_TOKENS_Q4_K if dtype == O.Q4_K else op.TUNE_TC_MIN_TOKENS_Q6_K
    ctx.tuning_set(key, 1)
    try:
        ow = O.TensorView(raw, dtype, n_in, n_out)
        for x_dtype, toks in ((torch.bfloat16, 20), (torch.float32, 9)):
            xs = torch.from_numpy(H.lcg_activations(toks * n_in, seed=toks).reshape(toks, n_in)).to(x_dtype).cuda()
            want = O.matmul(ow, xs.float().cpu().numpy())
            acc = torch.zeros((toks, n_out), dtype=torch.float32, device="cuda")
            for rank in range(world):
                wk = op.Weight(ctx, view, shard=(rank, world, op.SHARD_K))
                yk = torch.empty((toks, n_out), dtype=torch.float32, device="cuda")
                k.encode_quantized_matmul(wk, xs[:, rank * ks:(rank + 1) * ks].contiguous(), yk, toks)
                acc += yk
            ctx.sync_status()
            assert H.rel_l2(acc.cpu().numpy(), want) <= REL_L2_TOL, x_dtype
    finally:
        ctx.tuning_set(op.TUNE_TC_MIN_ROWS, 1024)
        ctx.tuning_set(key, 17)


@pytest.mark.parametrize("dtype", [O.Q4_K, O.Q5_K, O.Q6_K])
def test_every_launch_plan_of_the_decode_kernel(gpu, dtype):
    """The decode kernel's plan forced through its tuning keys: few and many warps per CTA, one to ten K slices between
    CTAs (one slice: no scratch exchange; ten: one tile per slice), one to five K parts between the warps of a CTA
    (shared-memory meeting), both ring depths, every token-group variant, bf16 and f32 activations, against the CPU
    lane; a fixed plan must also give identical bits on a repeated call."""
    op, ctx, k = gpu
    n_in, n_out = 2560, 5000          # 10 K tiles, a short last row tile
    raw = H.lcg_weights(dtype, n_out, n_in // 256, seed=123 + dtype)
    ow = O.TensorView(raw, dtype, n_in, n_out)
    w = op.Weight(ctx, op.TensorView(raw, dtype, n_in, n_out))
    plans = [(0, 0, 0, 0), (2, 1, 2, 1), (6, 3, 4, 3), (12, 2, 2, 2), (14, 10, 2, 1), (16, 7, 4, 1), (20, 1, 2, 5), (16, 2, 2, 4), (10, 1, 2, 10)]
    try:
        for x_dtype in (torch.bfloat16, torch.float32):
            for tokens in (1, 2, 3, 4, 5, 8, 9, 12, 13, 16):
                x = torch.from_numpy(H.lcg_activations(tokens * n_in, seed=40 + tokens).reshape(tokens, n_in)).to(x_dtype).cuda()
                want = O.matmul(ow, x.float().cpu().numpy())
                for warps, ksplit, ring, wsplit in plans if tokens in (1, 4, 8, 13) else plans[:2]:
                    ctx.tuning_set(op.TUNE_DECODE_WARPS, warps)
                    ctx.tuning_set(op.TUNE_DECODE_KSPLIT, ksplit)
                    ctx.tuning_set(op.TUNE_DECODE_RING, ring)
                    ctx.tuning_set(op.TUNE_DECODE_WSPLIT, wsplit)
                    y = torch.full((tokens, n_out), float("nan"), dtype=torch.float32, device="cuda")
                    k.encode_quantized_matmul(w, x, y, tokens)
                    again = torch.empty_like(y)
                    k.encode_quantized_matmul(w, x, again, tokens)
                    ctx.sync_status()
                    assert torch.equal(y, again), (x_dtype, tokens, warps, ksplit, ring, wsplit)
                    assert H.rel_l2(y.cpu().numpy(), want) <= REL_L2_TOL, (x_dtype, tokens, warps, ksplit, ring, wsplit)
    finally:
        for key in (op.TUNE_DECODE_WARPS, op.TUNE_DECODE_KSPLIT, op.TUNE_DECODE_RING, op.TUNE_DECODE_WSPLIT):
            ctx.tuning_set(key, 0)
        w.free()


def test_grouped_projections_in_one_launch(gpu):
    """q | k | v of one hidden state in one launch (Q4_K, Q4_K and Q6_K rows of different counts), each with its own
    output dtype and epilogue, with and without the shared fused input norm: against the CPU lane and against the
    same projections launched one by one."""
    op, ctx, k = gpu
    n_in, eps = 1024, 1e-6
    shapes = [(O.Q4_K, 300), (O.Q4_K, 37), (O.Q6_K, 64), (O.Q6_K, 130)]
    raws = [H.lcg_weights(dt, n, n_in // 256, seed=70 + i) for i, (dt, n) in enumerate(shapes)]
    ws = [op.Weight(ctx, op.TensorView(r, dt, n_in, n)) for r, (dt, n) in zip(raws, shapes)]
    ows = [O.TensorView(r, dt, n_in, n) for r, (dt, n) in zip(raws, shapes)]
    nw = torch.linspace(0.5, 1.5, n_in)
    for tokens in (1, 3, 8, 16):
        x = torch.from_numpy(H.lcg_activations(tokens * n_in, seed=tokens).reshape(tokens, n_in) * 2.0).to(torch.bfloat16)
        res = torch.from_numpy(H.lcg_activations(tokens * 37, seed=2).reshape(tokens, 37)).cuda()
        rs = torch.linspace(0.5, 2.0, tokens, device="cuda")
        for normed in (False, True):
            norm = dict(norm_weight=nw.cuda(), norm_eps=eps) if normed else {}
            eps_list = [dict(norm), dict(norm, residual=res), dict(norm, row_scale=rs), dict(norm, out_scale=0.5)]
            xin = O.rms_norm_mul(x.float().numpy(), eps, nw.numpy()) if normed else x.float().numpy()
            for count in (4, 3, 1):
                ys = [torch.full((tokens, n), float("nan"), dtype=torch.bfloat16 if i == 3 else torch.float32, device="cuda")
                      for i, (_, n) in enumerate(shapes[:count])]
                k.encode_quantized_matmul_group(ws[:count], x.cuda(), ys, tokens, epilogues=eps_list[:count])
                ctx.sync_status()
                for i in range(count):
                    want = O.matmul(ows[i], xin)
                    if i == 1:
                        want = want + res.cpu().numpy()
                    if i == 2:
                        want = want * rs.cpu().numpy()[:, None]
                    if i == 3:
                        want = want * 0.5
                    tol = 4e-3 if i == 3 else REL_L2_TOL   # item 3 is stored as bf16
                    assert H.rel_l2(ys[i].float().cpu().numpy(), want) <= tol, (tokens, normed, count, i)
                    alone = torch.empty_like(ys[i])
                    k.encode_quantized_matmul(ws[i], x.cuda(), alone, tokens, **eps_list[i])
                    assert H.rel_l2(ys[i].float().cpu().numpy(), alone.float().cpu().numpy()) <= (1e-2 if i == 3 else 1e-5)
    # misuse
    x = torch.zeros((1, n_in), dtype=torch.bfloat16, device="cuda")
    ys = [torch.zeros((1, n), dtype=torch.float32, device="cuda") for _, n in shapes]
    other = op.Weight(ctx, op.TensorView(H.lcg_weights(O.Q4_K, 16, 2, seed=1), O.Q4_K, 512, 16))
    with pytest.raises(op.MuserCudaError) as e:
        k.encode_quantized_matmul_group([ws[0], other], x, [ys[0], torch.zeros((1, 16), device="cuda")], 1)
    assert e.value.status_name == "BAD_SHAPE"
    with pytest.raises(op.MuserCudaError) as e:
        k.encode_quantized_matmul_group(ws[:2], x, ys[:2], 1, epilogues=[dict(norm_weight=nw.cuda(), norm_eps=eps), None])
    assert e.value.status_name == "BAD_ARG"
    with pytest.raises(op.MuserCudaError) as e:
        k.encode_quantized_matmul_group(ws + ws[:1], x, ys + ys[:1], 1)
    assert e.value.status_name == "BAD_ARG"
    x17 = torch.zeros((17, n_in), dtype=torch.bfloat16, device="cuda")
    with pytest.raises(op.MuserCudaError) as e:
        k.encode_quantized_matmul_group(ws[:1], x17, [torch.zeros((17, 300), device="cuda")], 17)
    assert e.value.status_name == "BAD_SHAPE"
    for w in ws + [other]:
        w.free()


def test_measured_launch_plans_keep_the_results(gpu):
    """muser_cuda_decode_autotune replaces the cost model's launch plans with measured ones for a group, a single
    projection and a fused gate/up pair: results stay within tolerance of the CPU lane and repeat bit for bit."""
    op, ctx, k = gpu
    n_in = 2048
    shapes = [(O.Q4_K, 1100), (O.Q6_K, 260)]
    raws = [H.lcg_weights(dt, n, n_in // 256, seed=90 + i) for i, (dt, n) in enumerate(shapes)]
    ws = [op.Weight(ctx, op.TensorView(r, dt, n_in, n)) for r, (dt, n) in zip(raws, shapes)]
    ows = [O.TensorView(r, dt, n_in, n) for r, (dt, n) in zip(raws, shapes)]
    up = op.Weight(ctx, op.TensorView(H.lcg_weights(O.Q4_K, 1100, n_in // 256, seed=95), O.Q4_K, n_in, 1100))
    k.autotune(ws, max_tokens=16)
    k.autotune(ws[:1], max_tokens=6)
    k.autotune(ws[:1], up=up, max_tokens=4)
    ctx.sync_status()
    for tokens in (1, 3, 6, 11, 16):
        x = torch.from_numpy(H.lcg_activations(tokens * n_in, seed=tokens).reshape(tokens, n_in)).to(torch.bfloat16).cuda()
        ys = [torch.full((tokens, n), float("nan"), dtype=torch.float32, device="cuda") for _, n in shapes]
        again = [torch.empty_like(y) for y in ys]
        k.encode_quantized_matmul_group(ws, x, ys, tokens)
        k.encode_quantized_matmul_group(ws, x, again, tokens)
        alone = torch.empty_like(ys[0])
        k.encode_quantized_matmul(ws[0], x, alone, tokens)
        ctx.sync_status()
        for i in range(2):
            assert torch.equal(ys[i], again[i])
            assert H.rel_l2(ys[i].cpu().numpy(), O.matmul(ows[i], x.float().cpu().numpy(), threads=4)) <= REL_L2_TOL, (tokens, i)
        assert H.rel_l2(alone.cpu().numpy(), ys[0].cpu().numpy()) <= 1e-5
    with pytest.raises(op.MuserCudaError):
        k.autotune(ws, up=up)   # the fused pair form takes one gate weight
    for w in ws + [up]:
        w.free()


def test_config1_full_size_q4k_gemv(gpu):
    """y[1,27648] = x[1,5120] . W(Q4_K): every dequantised weight bit-exact, output within tolerance."""
    op, ctx, k = gpu
    from muser_b200 import synth
    n_in, n_out = 5120, 27648
    wf = synth.normal_weights(n_out, n_in, seed=0, stream=4, device="cuda")
    raw = synth.quantize_q4_k(wf)
    x = synth.normal_activations(1, n_in, seed=0, device="cuda")
    w = op.Weight(ctx, op.TensorView(raw, O.Q4_K, n_in, n_out))
    raw_h = raw.cpu().numpy()
    ow = O.TensorView(raw_h, O.Q4_K, n_in, n_out)
    deq = k.dequant(w)
    want = torch.from_numpy(O.dequant_tensor(ow))
    assert torch.equal(deq.cpu().view(torch.int32), want.view(torch.int32))
    y = torch.empty((1, n_out), dtype=torch.float32, device="cuda")
    k.encode_quantized_matmul(w, x, y, 1)
    ref = O.matmul(ow, x.float().cpu().numpy(), threads=O.host_threads())
    assert H.rel_l2(y.cpu().numpy(), ref) <= REL_L2_TOL
    # host-slice entry point (weights::matmul signature)
    yh = op.matmul(ctx, w, x.float().cpu().numpy(), 1)
    assert H.rel_l2(yh, ref) <= REL_L2_TOL
    # linearity at full size: W(2a + b) == 2 W a + W b up to rounding
    a, b = synth.normal_activations(2, n_in, seed=3, device="cuda")
    ab = torch.stack([a, b, (2 * a.float() + b.float()).to(torch.bfloat16)])
    y3 = torch.empty((3, n_out), dtype=torch.float32, device="cuda")
    k.encode_quantized_matmul(w, ab, y3, 3)
    lin = 2 * y3[0] + y3[1]
    exact = (2 * a.float() + b.float())
    y_exact = torch.empty((1, n_out), dtype=torch.float32, device="cuda")
    k.encode_quantized_matmul(w, exact.reshape(1, -1).contiguous(), y_exact, 1)
    assert H.rel_l2(lin.cpu().numpy(), y_exact[0].cpu().numpy()) <= 1e-4


@pytest.mark.parametrize("name", ["ffn_gate", "ffn_down"])
def test_layer_shapes_every_kernel_sampled_rows_and_determinism(gpu, name):
    """The layer's two big projections at full size, one token count per kernel variant and split-K regime (decode
    kernel with one to four token groups, tcgen05 kernel at 32 / 64 columns): 96 sampled output rows against the CPU
    lane, and bit-identical results when the same call runs twice (the K slices are summed in a fixed order)."""
    op, ctx, k = gpu
    from muser_b200 import synth
    n_in, n_out, dtype = synth.LAYER_PROJECTIONS[name]
    raw = synth.quantize_kquant(synth.normal_weights(n_out, n_in, seed=0, stream=11, device="cuda"), dtype)
    w = op.Weight(ctx, op.TensorView(raw, dtype, n_in, n_out))
    rows = np.sort(np.random.default_rng(5).choice(n_out, 96, replace=False))
    sub = raw.cpu().numpy().reshape(n_out, -1)[rows].copy()
    ow = O.TensorView(sub, dtype, n_in, len(rows))
    for tokens in (1, 2, 4, 8, 12, 16, 24, 64):
        x = synth.normal_activations(tokens, n_in, seed=tokens, device="cuda")
        y1 = torch.empty((tokens, n_out), dtype=torch.float32, device="cuda")
        y2 = torch.full_like(y1, float("nan"))
        k.encode_quantized_matmul(w, x, y1, tokens)
        k.encode_quantized_matmul(w, x, y2, tokens)
        ctx.sync_status()
        assert torch.equal(y1, y2), (name, tokens)
        ref = O.matmul(ow, x.float().cpu().numpy(), threads=O.host_threads())
        err = H.rel_l2(y1[:, torch.from_numpy(rows).cuda()].cpu().numpy(), ref)
        assert err <= REL_L2_TOL, (name, tokens, err)
    w.free()


@pytest.mark.parametrize("dtype", [O.Q4_K, O.Q6_K])
def test_host_slice_entry_point_repeated_calls(gpu, dtype):
    """weights::matmul's signature (host f32 slices in and out), called repeatedly through the context's one pinned
    staging area: every call must still see its own input and fill its own output."""
    op, ctx, k = gpu
    n_in, n_out = 1024, 80
    raw = H.lcg_weights(dtype, n_out, n_in // 256, seed=61)
    w = op.Weight(ctx, op.TensorView(raw, dtype, n_in, n_out))
    ow = O.TensorView(raw, dtype, n_in, n_out)
    for tokens in (1, 5, 70):  # 70: two chunks of at most 64 tokens
        for call in range(4):
            x = H.lcg_activations(tokens * n_in, seed=10 * tokens + call).reshape(tokens, n_in).astype(np.float32)
            y = op.matmul(ctx, w, x, tokens)
            assert H.rel_l2(y, O.matmul(ow, x)) <= REL_L2_TOL, (tokens, call)
    w.free()


@pytest.mark.parametrize("dtype", [O.Q4_K, O.Q5_K, O.Q6_K])
def test_lm_head_tail_and_selected_rows(gpu, dtype):
    """The LM-head end of the path (reference.rs:559-570, weights.rs:425-449): logit scale and tanh soft cap fused
    behind the projection in every K-quant kernel, and the projection restricted to a list of rows."""
    op, ctx, k = gpu
    n_in, n_out, cap = 1024, 300, 30.0
    raw = H.lcg_weights(dtype, n_out, n_in // 256, seed=55)
    ow = O.TensorView(raw, dtype, n_in, n_out)
    w = op.Weight(ctx, op.TensorView(raw, dtype, n_in, n_out))
    ctx.tuning_set(op.TUNE_TC_MIN_ROWS, 1)
    try:
        for tokens in (1, 3, 7, 20):  # decode kernel (one and two token groups), tcgen05 kernel
            x = torch.from_numpy(H.lcg_activations(tokens * n_in, seed=tokens).reshape(tokens, n_in)).to(torch.bfloat16)
            plain = O.matmul(ow, x.float().numpy())
            scale = float(15.0 / plain.std())  # scaled logits of std 15 against a cap of 30: both regimes of the tanh occur
            want = O.logit_tail(plain, scale, cap)
            assert np.abs(want).max() > 0.8 * cap and np.abs(want).min() < 0.1 * cap
            y = torch.empty((tokens, n_out), dtype=torch.float32, device="cuda")
            k.encode_quantized_matmul(w, x.cuda(), y, tokens, out_scale=scale, softcap=cap)
            assert H.rel_l2(y.cpu().numpy(), want) <= REL_L2_TOL, tokens
            k.encode_quantized_matmul(w, x.cuda(), y, tokens, out_scale=scale)
            assert H.rel_l2(y.cpu().numpy(), O.logit_tail(plain, scale, 0.0)) <= REL_L2_TOL
    finally:
        ctx.tuning_set(op.TUNE_TC_MIN_ROWS, 1024)
    rows = np.array([299, 0, 17, 17, 128, 255, 16], dtype=np.int32)
    for x_dtype in (torch.bfloat16, torch.float32):
        x = torch.from_numpy(H.lcg_activations(11 * n_in, seed=9).reshape(11, n_in)).to(x_dtype)
        y = torch.full((11, len(rows)), float("nan"), dtype=torch.float32, device="cuda")
        k.encode_quantized_matmul_rows(w, torch.from_numpy(rows).cuda(), x.cuda(), y, 11)
        want = O.matmul_rows(ow, x.float().numpy(), rows)
        assert np.array_equal(want, O.matmul(ow, x.float().numpy())[:, rows])
        assert H.rel_l2(y.cpu().numpy(), want) <= 1e-5, x_dtype
    bad = torch.tensor([5, n_out], dtype=torch.int32, device="cuda")  # an index past the last row reads nothing
    y = torch.zeros((1, 2), dtype=torch.float32, device="cuda")
    k.encode_quantized_matmul_rows(w, bad, torch.ones((1, n_in), dtype=torch.float32, device="cuda"), y, 1)
    assert torch.isfinite(y[0, 0]) and torch.isnan(y[0, 1])
    ctx.sync_status()


@pytest.mark.parametrize("dtype", [O.Q5_K, O.Q4_K, O.Q6_K])
def test_lm_head_with_the_greedy_pick_fused_in(gpu, dtype):
    """muser_cuda_lm_head_argmax: logits through the LM-head tail (reference.rs:559-570), then the index of the first
    maximum per token (api.rs:1842-1850).  The pick must equal a first-maximum scan of the logits the same call
    wrote, bit for bit; equal maxima must resolve to the lowest row wherever the rows sit in the grid; the CPU lane's
    logit at the picked row must be its maximum up to the kernel's error; NaN inputs raise the flag and never win."""
    op, ctx, k = gpu
    n_in, n_out = 1024, 20011
    raw = H.lcg_weights(dtype, n_out, n_in // 256, seed=81 + dtype).copy()
    scale, cap = 0.37, 30.0
    ow = O.TensorView(raw, dtype, n_in, n_out)
    for tokens in (1, 3, 8, 16):
        x = torch.from_numpy(H.lcg_activations(tokens * n_in, seed=31 + tokens).reshape(tokens, n_in)).to(torch.bfloat16)
        w = op.Weight(ctx, op.TensorView(raw, dtype, n_in, n_out))
        logits = torch.full((tokens, n_out), float("nan"), dtype=torch.float32, device="cuda")
        idx, val, bad = k.encode_lm_head_argmax(w, x.cuda(), tokens, logits=logits, out_scale=scale, softcap=cap)
        idx2, val2, _ = k.encode_lm_head_argmax(w, x.cuda(), tokens, out_scale=scale, softcap=cap)  # pick only; keys were reset
        ctx.sync_status()
        got = logits.cpu().numpy()
        first_max = np.array([int(np.flatnonzero(row == row.max())[0]) for row in got])
        assert np.array_equal(idx.cpu().numpy(), first_max), tokens
        assert np.array_equal(idx2.cpu().numpy(), first_max) and torch.equal(val, val2)
        assert np.array_equal(val.cpu().numpy().view(np.uint32), got[np.arange(tokens), first_max].view(np.uint32))
        assert not bad.cpu().numpy().any()
        want = O.logit_tail(O.matmul(ow, x.float().numpy(), threads=O.host_threads()), scale, cap)
        assert H.rel_l2(got, want) <= REL_L2_TOL
        picked = want[np.arange(tokens), first_max]
        assert np.all(want.max(axis=1) - picked <= 2e-3 * np.abs(want).max()), tokens
        w.free()
    # ties: the winning row of token 0 copied to an earlier and to a much later row -> the earliest of the three wins
    tokens = 4
    x = torch.from_numpy(H.lcg_activations(tokens * n_in, seed=77).reshape(tokens, n_in)).to(torch.bfloat16)
    w = op.Weight(ctx, op.TensorView(raw, dtype, n_in, n_out))
    idx, _, _ = k.encode_lm_head_argmax(w, x.cuda(), tokens)
    r0 = int(idx.cpu()[0])
    w.free()
    row_bytes = raw.size // n_out
    rows = raw.reshape(n_out, row_bytes)
    early, late = (5 if r0 != 5 else 6), (n_out - 3 if r0 != n_out - 3 else n_out - 4)
    tied = rows.copy()
    tied[early], tied[late] = rows[r0], rows[r0]
    w = op.Weight(ctx, op.TensorView(tied.reshape(-1), dtype, n_in, n_out))
    idx, _, bad = k.encode_lm_head_argmax(w, x.cuda(), tokens)
    assert int(idx.cpu()[0]) == min(early, r0) and not bad.cpu().numpy().any()
    # a NaN activation poisons token 1 only: flagged there, index 0 by the scalar scan's convention; the others keep their pick
    xn = x.clone()
    xn[1, 100] = float("nan")
    idx_n, _, bad_n = k.encode_lm_head_argmax(w, xn.cuda(), tokens)
    ctx.sync_status()
    assert bad_n.cpu().numpy().tolist() == [0, 1, 0, 0]
    assert idx_n.cpu().numpy()[[0, 2, 3]].tolist() == idx.cpu().numpy()[[0, 2, 3]].tolist()
    # misuse
    y = torch.empty((17, n_out), dtype=torch.float32, device="cuda")
    x17 = torch.zeros((17, n_in), dtype=torch.bfloat16, device="cuda")
    with pytest.raises(op.MuserCudaError) as e:
        k.encode_lm_head_argmax(w, x17, 17)
    assert e.value.status_name == "BAD_SHAPE"
    w.free()
    ws = op.Weight(ctx, op.TensorView(raw, dtype, n_in, n_out), shard=(0, 2, 2))  # a K shard: partial sums have no maximum
    with pytest.raises(op.MuserCudaError) as e:
        k.encode_lm_head_argmax(ws, x[:, :n_in // 2].contiguous().cuda(), tokens)
    assert e.value.status_name == "BAD_SHAPE"
    ws.free()


def test_misuse_returns_statuses(gpu):
    op, ctx, k = gpu
    raw = H.lcg_weights(O.Q4_K, 16, 1, seed=1)
    with pytest.raises(op.MuserCudaError) as e:
        op.Weight(ctx, op.TensorView(raw, 8, 256, 16))       # Q8_0: no projection kernel
    assert e.value.status_name == "UNSUPPORTED_DTYPE"
    with pytest.raises(op.MuserCudaError) as e:
        op.Weight(ctx, op.TensorView(raw[:, :100], O.Q4_K, 256, 16))
    assert e.value.status_name == "BAD_SHAPE"
    w = op.Weight(ctx, op.TensorView(raw, O.Q4_K, 256, 16))
    x = torch.zeros((65, 256), dtype=torch.bfloat16, device="cuda")
    y = torch.zeros((65, 16), dtype=torch.float32, device="cuda")
    with pytest.raises(op.MuserCudaError) as e:
        k.encode_quantized_matmul(w, x, y, 65)
    assert e.value.status_name == "BAD_SHAPE"
    with pytest.raises(op.MuserCudaError) as e:
        k.encode_quantized_matmul(w, x.flatten()[1:257], y, 1)   # 2 bytes off a 16-byte boundary
    assert e.value.status_name == "BAD_ALIGN"
    with pytest.raises(op.MuserCudaError) as e:
        op.Weight(ctx, op.TensorView(raw, O.Q4_K, 256, 16), shard=(0, 3, op.SHARD_ROWS))
    assert e.value.status_name == "BAD_SHAPE"


@pytest.mark.parametrize("tokens", [13, 16])
def test_repeated_calls_are_bit_identical(gpu, tokens):
    """The 16-token ffn_down projection runs with a ring of two tiles per warp and 14 K slices: the launch plan in
    which a refill of a ring slot that still had reads in flight showed up as one differing call in a few hundred
    (rows of one tile, every token).  800 calls must all carry the bits of the first."""
    op, ctx, k = gpu
    from muser_b200 import synth
    n_in, n_out, dtype = synth.LAYER_PROJECTIONS["ffn_down"]
    raw = synth.quantize_kquant(synth.normal_weights(n_out, n_in, seed=0, stream=11, device="cuda"), dtype)
    w = op.Weight(ctx, op.TensorView(raw, dtype, n_in, n_out))
    x = synth.normal_activations(tokens, n_in, seed=tokens, device="cuda")
    first = torch.empty((tokens, n_out), dtype=torch.float32, device="cuda")
    k.encode_quantized_matmul(w, x, first, tokens)
    ctx.sync_status()
    ys = [torch.full_like(first, float("nan")) for _ in range(16)]
    differing = 0
    for _ in range(50):
        for y in ys:
            k.encode_quantized_matmul(w, x, y, tokens)
        ctx.sync_status()
        differing += sum(0 if torch.equal(y, first) else 1 for y in ys)
    w.free()
    assert differing == 0, f"{differing} of 800 calls differ from the first"
