"""GPU parity of the NVFP4 path (quantizer, repack, block-scaled GEMM) against the CPU oracle and the
vectors produced by the reference's own Python code."""
import numpy as np
import pytest
import torch

from oracle import oracle as O
from tests import helpers as H

pytestmark = pytest.mark.gpu

REL_L2_TOL = 1e-3  # outputs: relative L2 against the CPU lane's value before its final f16 rounding


@pytest.fixture(scope="module")
def gpu():
    from muser_b200 import operator as op
    ctx = op.Context(0, workspace_bytes=64 << 20)
    yield op, ctx, op.CudaKernels(ctx)
    ctx.close()


def f16_bits_to_f32(a):
    return a.view(np.float16).astype(np.float32)


def test_activation_quantiser_is_bit_identical_to_reference_vectors(gpu, golden):
    op, ctx, k = gpu
    for tag in ("quant", "quant2", "w4a4"):
        key = f"{tag}_input_f16_bits" if tag != "w4a4" else "w4a4_activation_f16_bits"
        x = torch.from_numpy(f16_bits_to_f32(golden[key])).cuda()
        isi = float(golden[f"{tag}_global_scale"] if tag != "w4a4" else golden["w4a4_act_global"])
        packed, scales = k.quantize_nvfp4_activation(x, isi)
        want_packed = golden[f"{tag}_packed"] if tag != "w4a4" else golden["w4a4_act_packed"]
        assert np.array_equal(packed.cpu().numpy(), want_packed), tag
        rows, n_in = x.shape
        logical = op.unswizzle_scales(scales, rows, n_in).cpu().numpy()
        op_, os_ = O.quantize_nvfp4_activation(x.cpu().numpy(), isi)
        assert np.array_equal(logical, os_), tag
        if tag != "w4a4":  # the reference's own swizzled plane, byte for byte where rows exist
            ref = golden[f"{tag}_scales_swizzled"].reshape(-1)
            assert np.array_equal(scales.cpu().numpy()[: ref.size], ref), tag


@pytest.mark.parametrize("x_dtype", [torch.float32, torch.bfloat16])
def test_activation_quantiser_matches_oracle_on_random_and_edge_inputs(gpu, x_dtype):
    op, ctx, k = gpu
    g = torch.Generator().manual_seed(11)
    x = torch.randn((133, 320), generator=g) * torch.logspace(-6, 3, 320)[None, :]
    x[5, :16] = 0.0
    x[6, 16:32] = -0.0
    x[7, 32] = 70000.0      # beyond f16: rounds to inf, scale saturates
    x[8, 48:64] = 1e-8
    x = x.to(x_dtype)
    isi = 37.5
    packed, scales = k.quantize_nvfp4_activation(x.cuda(), isi)
    wp, ws = O.quantize_nvfp4_activation(x.float().numpy(), isi)
    assert np.array_equal(packed.cpu().numpy(), wp)
    assert np.array_equal(op.unswizzle_scales(scales, 133, 320).cpu().numpy(), ws)


def make_weight(op, ctx, n_out, n_in, seed, negative_scales=False):
    from muser_b200 import synth
    w = synth.normal_weights(n_out, n_in, seed=seed, stream=9)
    packed, scales, scale2 = synth.nvfp4_weight(w)
    packed, scales = packed.numpy().copy(), scales.numpy().copy()
    if negative_scales:
        scales[::3, ::5] |= 0x80  # signed E4M3 scale codes are legal in the stored format
    return packed, scales, scale2


def test_weight_repack_dequantises_bit_exactly(gpu, golden):
    op, ctx, k = gpu
    packed, scales, scale2 = make_weight(op, ctx, 37, 320, seed=2, negative_scales=True)
    w = op.Weight(ctx, op.TensorView(packed, O.NVFP4, 320, 37, scales, scale2, 100.0))
    got = k.dequant(w).cpu().numpy()
    want = O.dequant_nvfp4(packed, scales, scale2)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    # the reference Python decoder's vector
    w2 = op.Weight(ctx, op.TensorView(np.tile(golden["codec_packed"], (1, 1)), O.NVFP4, 128, 9,
                                      golden["codec_scales"], float(golden["codec_scale2"]), 1.0))
    got2 = k.dequant(w2).cpu().numpy()
    assert np.array_equal(got2.view(np.uint32), golden["codec_dequant"].view(np.uint32))
    bad = scales.copy()
    bad[3, 2] = 0x7F
    with pytest.raises(op.MuserCudaError) as e:
        op.Weight(ctx, op.TensorView(packed, O.NVFP4, 320, 37, bad, scale2, 100.0))
    assert e.value.status_name == "NAN_SCALE"


def test_w4a4_gemm_reproduces_the_reference_fixture(gpu, golden):
    """32 x 128 x 128 fixture of scripts/gx10/vllm/test_exact_fp4_mm.py, expected values computed by its numpy half."""
    op, ctx, k = gpu
    isi = float(golden["w4a4_act_global"])
    w = op.Weight(ctx, op.TensorView(golden["w4a4_w_packed"], O.NVFP4, 128, 128, golden["w4a4_w_scales_logical"],
                                     float(golden["w4a4_weight_scale2"]), isi))
    x = torch.from_numpy(f16_bits_to_f32(golden["w4a4_activation_f16_bits"])).cuda()
    y = torch.full((32, 128), float("nan"), dtype=torch.float16, device="cuda")
    k.encode_nvfp4_matmul(w, x, y, 32)
    ctx.sync_status()
    want = golden["w4a4_expected_f16_bits"].view(np.float16).astype(np.float32)
    got = y.float().cpu().numpy()
    assert H.rel_l2(got, want) <= REL_L2_TOL
    # the integer lane is exact; an f32-accumulating tensor core may differ by an f16 ulp on a few cells
    ulp = np.abs(got.astype(np.float16).view(np.int16).astype(np.int32) - want.astype(np.float16).view(np.int16).astype(np.int32))
    assert ulp.max() <= 1 and (ulp > 0).mean() < 0.02


@pytest.mark.parametrize("n_out,n_in,tokens", [(256, 256, 128), (37, 320, 7), (300, 1024, 130), (512, 2048, 300)])
def test_w4a4_gemm_matches_cpu_lane(gpu, n_out, n_in, tokens):
    op, ctx, k = gpu
    from muser_b200 import synth
    packed, scales, scale2 = make_weight(op, ctx, n_out, n_in, seed=n_out, negative_scales=True)
    x = synth.normal_activations(tokens, n_in, seed=4)
    isi = synth.activation_input_scale_inv(x)
    ow = O.TensorView(packed, O.NVFP4, n_in, n_out, scales, scale2, isi)
    ref_f16, ref_f32 = O.matmul(ow, x.float().numpy(), threads=O.host_threads(), return_pre_round=True)
    w = op.Weight(ctx, op.TensorView(packed, O.NVFP4, n_in, n_out, scales, scale2, isi))
    for y_dtype, ref in ((torch.float32, ref_f32), (torch.float16, ref_f16), (torch.bfloat16, ref_f32)):
        y = torch.full((tokens, n_out), float("nan"), dtype=y_dtype, device="cuda")
        k.encode_nvfp4_matmul(w, x.cuda(), y, tokens)
        ctx.sync_status()
        tol = REL_L2_TOL if y_dtype != torch.bfloat16 else 4e-3  # bf16 output rounding alone is 2^-9
        assert H.rel_l2(y.float().cpu().numpy(), ref) <= tol, (y_dtype, H.rel_l2(y.float().cpu().numpy(), ref))
    # prequantised entry point + fused row scale and residual
    xp, xs = k.quantize_nvfp4_activation(x.cuda(), isi)
    rs = torch.linspace(0.5, 1.5, tokens, device="cuda")
    res = torch.randn((tokens, n_out), device="cuda")
    y = torch.empty((tokens, n_out), dtype=torch.float32, device="cuda")
    k.encode_nvfp4_prequant(w, xp, xs, y, tokens, row_scale=rs, residual=res)
    ctx.sync_status()
    want = ref_f32 * rs.cpu().numpy()[:, None] + res.cpu().numpy()
    assert H.rel_l2(y.cpu().numpy(), want) <= REL_L2_TOL
    # LM-head tail (reference.rs:559-570) behind the GEMM
    big = float(1.0 / np.abs(ref_f32).max()) * 60.0
    k.encode_nvfp4_matmul(w, x.cuda(), y, tokens, out_scale=big, softcap=30.0)
    ctx.sync_status()
    assert H.rel_l2(y.cpu().numpy(), O.logit_tail(ref_f32, big, 30.0)) <= REL_L2_TOL


@pytest.mark.parametrize("n_out,n_in,tokens", [(128, 256, 128), (200, 320, 9), (700, 1024, 260)])
def test_fused_gate_up_silu_matches_cpu_lane(gpu, n_out, n_in, tokens):
    """silu_fast(gate) * up in one GEMM against the CPU lane's composition: two W4A4 matmuls (f16-rounded, as
    quant/nvfp4.rs:337 returns them), then x / (1 + exp(-x)) * up in f32 (reference.rs:511-513)."""
    op, ctx, k = gpu
    from muser_b200 import synth
    gp, gs, g2 = make_weight(op, ctx, n_out, n_in, seed=n_out + 1, negative_scales=True)
    up, us, u2 = make_weight(op, ctx, n_out, n_in, seed=n_out + 2)
    x = synth.normal_activations(tokens, n_in, seed=9)
    isi = synth.activation_input_scale_inv(x)
    xf = x.float().numpy()
    gate = O.matmul(O.TensorView(gp, O.NVFP4, n_in, n_out, gs, g2, isi), xf, threads=O.host_threads())
    upv = O.matmul(O.TensorView(up, O.NVFP4, n_in, n_out, us, u2, isi), xf, threads=O.host_threads())
    want = O.silu_mul(gate, upv)
    wg = op.Weight(ctx, op.TensorView(gp, O.NVFP4, n_in, n_out, gs, g2, isi))
    wu = op.Weight(ctx, op.TensorView(up, O.NVFP4, n_in, n_out, us, u2, isi))
    for y_dtype, tol in ((torch.float32, REL_L2_TOL), (torch.bfloat16, 4e-3)):
        y = torch.full((tokens, n_out), float("nan"), dtype=y_dtype, device="cuda")
        k.encode_ffn_gate_up_silu(wg, wu, x.cuda(), y, tokens)
        ctx.sync_status()
        assert H.rel_l2(y.float().cpu().numpy(), want) <= tol, (y_dtype, H.rel_l2(y.float().cpu().numpy(), want))
    xp, xs = k.quantize_nvfp4_activation(x.cuda(), isi)
    y2 = torch.empty((tokens, n_out), dtype=torch.float32, device="cuda")
    k.encode_nvfp4_ffn_gate_up_silu_prequant(wg, wu, xp, xs, y2, tokens)
    ctx.sync_status()
    assert H.rel_l2(y2.cpu().numpy(), want) <= REL_L2_TOL
    # the two weights must quantize their input alike
    other = op.Weight(ctx, op.TensorView(up, O.NVFP4, n_in, n_out, us, u2, isi * 2))
    with pytest.raises(op.MuserCudaError) as e:
        k.encode_ffn_gate_up_silu(wg, other, x.cuda(), y2, tokens)
    assert e.value.status_name == "BAD_ARG"


@pytest.mark.parametrize("n_out,n_in,tokens", [(256, 256, 256), (256, 256, 128), (300, 1024, 130), (512, 2048, 300),
                                               (768, 1088, 1024), (1000, 512, 640)])
def test_paired_sm_gemm_equals_the_single_sm_gemm(gpu, n_out, n_in, tokens):
    """The cta_group::2 form (pairs of SMs on 256-token tiles) adds the same products in the same order as the
    single-CTA form, so every output must carry the same bits; both are checked against the CPU lane as well.
    Covers a follower CTA without tokens (128, 130), an odd block count (300, 640), ragged K (1088 = 4.25 slabs),
    rows that do not fill a tile (300, 1000), the fused gate/up form, the LM-head tail, and residual + row scale."""
    from muser_b200 import synth
    from muser_b200._lib import TUNE_NVFP4_PAIR
    op, ctx, k = gpu
    packed, scales, scale2 = make_weight(op, ctx, n_out, n_in, seed=n_out + 3, negative_scales=True)
    up, us, u2 = make_weight(op, ctx, n_out, n_in, seed=n_out + 4)
    x = synth.normal_activations(tokens, n_in, seed=12)
    isi = synth.activation_input_scale_inv(x)
    w = op.Weight(ctx, op.TensorView(packed, O.NVFP4, n_in, n_out, scales, scale2, isi))
    wu = op.Weight(ctx, op.TensorView(up, O.NVFP4, n_in, n_out, us, u2, isi))
    xp, xs = k.quantize_nvfp4_activation(x.cuda(), isi)
    rs = torch.linspace(0.5, 1.5, tokens, device="cuda")
    res = torch.randn((tokens, n_out), device="cuda")
    out = {}
    try:
        for mode in (0, 1):
            ctx.tuning_set(TUNE_NVFP4_PAIR, mode)
            ys = [torch.full((tokens, n_out), float("nan"), dtype=dt, device="cuda")
                  for dt in (torch.float32, torch.float16, torch.bfloat16, torch.float32, torch.float32, torch.float32)]
            k.encode_nvfp4_prequant(w, xp, xs, ys[0], tokens)
            k.encode_nvfp4_prequant(w, xp, xs, ys[1], tokens)
            k.encode_nvfp4_prequant(w, xp, xs, ys[2], tokens, row_scale=rs)
            k.encode_nvfp4_prequant(w, xp, xs, ys[3], tokens, row_scale=rs, residual=res)
            k.encode_nvfp4_matmul(w, x.cuda(), ys[4], tokens, out_scale=3.0, softcap=30.0)
            k.encode_nvfp4_ffn_gate_up_silu_prequant(w, wu, xp, xs, ys[5], tokens)
            ctx.sync_status()
            out[mode] = [y.cpu() for y in ys]
    finally:
        ctx.tuning_set(TUNE_NVFP4_PAIR, 0)
    for i, (a, b) in enumerate(zip(out[0], out[1])):
        assert torch.equal(a.view(torch.int32 if a.dtype == torch.float32 else torch.int16),
                           b.view(torch.int32 if b.dtype == torch.float32 else torch.int16)), f"output {i} differs between the two kernels"
    ow = O.TensorView(packed, O.NVFP4, n_in, n_out, scales, scale2, isi)
    _, ref_f32 = O.matmul(ow, x.float().numpy(), threads=O.host_threads(), return_pre_round=True)
    assert H.rel_l2(out[1][0].numpy(), ref_f32) <= REL_L2_TOL


@pytest.mark.parametrize("n_out,n_in,tokens", [(128, 256, 128), (192, 320, 9), (704, 1024, 260), (2048, 512, 1000)])
def test_fused_gate_up_silu_leaves_as_nvfp4_activations(gpu, n_out, n_in, tokens):
    """muser_cuda_nvfp4_ffn_gate_up_silu_requant: codes and scale bytes must equal, byte for byte, what
    muser_cuda_quantize_nvfp4_activation makes of the fused call's f32 output (quant/nvfp4.rs:173-238 on
    silu_fast(f16(gate)) * f16(up)); the slots of rows past the last token in the last 128-row block are zero."""
    from muser_b200 import synth
    op, ctx, k = gpu
    gp, gs, g2 = make_weight(op, ctx, n_out, n_in, seed=n_out + 11, negative_scales=True)
    up, us, u2 = make_weight(op, ctx, n_out, n_in, seed=n_out + 12)
    x = synth.normal_activations(tokens, n_in, seed=19)
    isi = synth.activation_input_scale_inv(x)
    wg = op.Weight(ctx, op.TensorView(gp, O.NVFP4, n_in, n_out, gs, g2, isi))
    wu = op.Weight(ctx, op.TensorView(up, O.NVFP4, n_in, n_out, us, u2, isi))
    xp, xs = k.quantize_nvfp4_activation(x.cuda(), isi)
    y = torch.empty((tokens, n_out), dtype=torch.float32, device="cuda")
    k.encode_nvfp4_ffn_gate_up_silu_prequant(wg, wu, xp, xs, y, tokens)
    isi_next = synth.activation_input_scale_inv(y)
    want_p, want_s = k.quantize_nvfp4_activation(y, isi_next)
    got_s = torch.full_like(want_s, 0xAB)
    got_p, got_s = k.encode_nvfp4_ffn_gate_up_silu_requant(wg, wu, xp, xs, tokens, isi_next, out_scales=got_s)
    ctx.sync_status()
    assert torch.equal(got_p, want_p)
    assert np.array_equal(op.unswizzle_scales(got_s, tokens, n_out).cpu().numpy(), op.unswizzle_scales(want_s, tokens, n_out).cpu().numpy())
    pad = (tokens + 127) // 128 * 128
    if pad > tokens:
        assert not op.unswizzle_scales(got_s, pad, n_out)[tokens:].any()
    # and it feeds the down projection like any quantized activation
    dp, ds, d2 = make_weight(op, ctx, 96, n_out, seed=5)
    wd = op.Weight(ctx, op.TensorView(dp, O.NVFP4, n_out, 96, ds, d2, isi_next))
    a = torch.empty((tokens, 96), dtype=torch.float32, device="cuda")
    b = torch.empty_like(a)
    k.encode_nvfp4_prequant(wd, got_p, got_s, a, tokens)
    k.encode_nvfp4_matmul(wd, y, b, tokens)
    ctx.sync_status()
    assert torch.equal(a.view(torch.int32), b.view(torch.int32))
    with pytest.raises(op.MuserCudaError) as e:  # whole 64-value chunks only
        w40 = op.Weight(ctx, op.TensorView(gp[:40], O.NVFP4, n_in, 40, gs[:40], g2, isi))
        k.encode_nvfp4_ffn_gate_up_silu_requant(w40, w40, xp, xs, tokens, isi_next)
    assert e.value.status_name == "BAD_SHAPE"


@pytest.mark.parametrize("x_dtype", [torch.float32, torch.bfloat16])
def test_fused_input_rmsnorm(gpu, x_dtype):
    """rms_norm_mul (reference.rs:59-80) fused into the activation quantizer.  The block adds the squares as a tree
    where the CPU lane adds them front to back, so 1/rms can differ in its last bit: codes are compared by
    mismatch count (a value sitting on a rounding boundary may fall the other way), outputs by relative L2."""
    op, ctx, k = gpu
    from muser_b200 import synth
    n_out, n_in, tokens, eps = 200, 1024, 70, 1e-6
    packed, scales, scale2 = make_weight(op, ctx, n_out, n_in, seed=3)
    x = (synth.normal_activations(tokens, n_in, seed=12).float() * 2.5).to(x_dtype)
    nw = torch.linspace(0.25, 2.0, n_in)
    xn = O.rms_norm_mul(x.float().numpy(), eps, nw.numpy())
    isi = synth.activation_input_scale_inv(torch.from_numpy(xn))
    want_p, want_s = O.quantize_nvfp4_activation(xn, isi)
    got_p, got_s = k.quantize_nvfp4_activation(x.cuda(), isi, norm_weight=nw.cuda(), norm_eps=eps)
    got_p, got_s = got_p.cpu().numpy(), op.unswizzle_scales(got_s, tokens, n_in).cpu().numpy()
    differing = np.count_nonzero((got_p & 15) != (want_p & 15)) + np.count_nonzero((got_p >> 4) != (want_p >> 4))
    assert differing <= 1e-3 * tokens * n_in, differing
    assert np.count_nonzero(got_s != want_s) <= 1e-3 * want_s.size
    ow = O.TensorView(packed, O.NVFP4, n_in, n_out, scales, scale2, isi)
    _, ref = O.matmul(ow, xn, threads=O.host_threads(), return_pre_round=True)
    w = op.Weight(ctx, op.TensorView(packed, O.NVFP4, n_in, n_out, scales, scale2, isi))
    y = torch.empty((tokens, n_out), dtype=torch.float32, device="cuda")
    k.encode_nvfp4_matmul(w, x.cuda(), y, tokens, norm_weight=nw.cuda(), norm_eps=eps)
    ctx.sync_status()
    assert H.rel_l2(y.cpu().numpy(), ref) <= REL_L2_TOL
    # the fused FFN front half behind the same norm
    up_p, up_s, up_2 = make_weight(op, ctx, n_out, n_in, seed=4)
    wu = op.Weight(ctx, op.TensorView(up_p, O.NVFP4, n_in, n_out, up_s, up_2, isi))
    gate = O.matmul(ow, xn, threads=O.host_threads())
    upv = O.matmul(O.TensorView(up_p, O.NVFP4, n_in, n_out, up_s, up_2, isi), xn, threads=O.host_threads())
    k.encode_ffn_gate_up_silu(w, wu, x.cuda(), y, tokens, norm_weight=nw.cuda(), norm_eps=eps)
    ctx.sync_status()
    assert H.rel_l2(y.cpu().numpy(), O.silu_mul(gate, upv)) <= 2 * REL_L2_TOL  # f16 boundaries of both factors can flip


def test_nvfp4_tensor_parallel_shards(gpu):
    op, ctx, k = gpu
    from muser_b200 import synth
    n_out, n_in, tokens, world = 512, 1280, 40, 4   # 320 inputs per K shard: a ragged 256-value slab
    packed, scales, scale2 = make_weight(op, ctx, n_out, n_in, seed=5)
    x = synth.normal_activations(tokens, n_in, seed=6)
    isi = synth.activation_input_scale_inv(x)
    view = op.TensorView(packed, O.NVFP4, n_in, n_out, scales, scale2, isi)
    full = op.Weight(ctx, view)
    y_full = torch.empty((tokens, n_out), dtype=torch.float32, device="cuda")
    k.encode_nvfp4_matmul(full, x.cuda(), y_full, tokens)
    cols, acc = [], torch.zeros_like(y_full)
    for rank in range(world):
        wr = op.Weight(ctx, view, shard=(rank, world, op.SHARD_ROWS))
        yr = torch.empty((tokens, n_out // world), dtype=torch.float32, device="cuda")
        k.encode_nvfp4_matmul(wr, x.cuda(), yr, tokens)
        cols.append(yr)
        wk = op.Weight(ctx, view, shard=(rank, world, op.SHARD_K))
        ks = n_in // world
        yk = torch.empty((tokens, n_out), dtype=torch.float32, device="cuda")
        k.encode_nvfp4_matmul(wk, x[:, rank * ks:(rank + 1) * ks].contiguous().cuda(), yk, tokens)
        acc += yk
    ctx.sync_status()
    assert torch.equal(torch.cat(cols, dim=1), y_full)
    assert H.rel_l2(acc.cpu().numpy(), y_full.cpu().numpy()) <= 1e-5


def test_prefill_shape_sampled_rows(gpu):
    """M = 2048 on a real projection shape (attn_k: 5120 -> 1024), checked on 64 sampled token rows."""
    op, ctx, k = gpu
    from muser_b200 import synth
    n_in, n_out, tokens = 5120, 1024, 2048
    w_f = synth.normal_weights(n_out, n_in, seed=0, stream=2, device="cuda")
    packed, scales, scale2 = synth.nvfp4_weight(w_f)
    x = synth.normal_activations(tokens, n_in, seed=0, device="cuda")
    isi = synth.activation_input_scale_inv(x)
    w = op.Weight(ctx, op.TensorView(packed, O.NVFP4, n_in, n_out, scales, scale2, isi))
    y = torch.empty((tokens, n_out), dtype=torch.float32, device="cuda")
    k.encode_nvfp4_matmul(w, x, y, tokens)
    ctx.sync_status()
    rows = torch.randperm(tokens, generator=torch.Generator().manual_seed(0))[:64]
    ow = O.TensorView(packed.cpu().numpy(), O.NVFP4, n_in, n_out, scales.cpu().numpy(), scale2, isi)
    _, ref = O.matmul(ow, x[rows.cuda()].float().cpu().numpy(), threads=O.host_threads(), return_pre_round=True)
    assert H.rel_l2(y[rows.cuda()].cpu().numpy(), ref) <= REL_L2_TOL


def test_weight_only_lane_is_bit_identical(gpu, golden):
    """A weight without input_scale_inv takes the reference's weight-only lane (int8 activations per 256, exact
    integer contraction, f16 result).  First the reference's own fixture (7 tokens x 11 rows x 256 inputs: its Q8
    codes, scales and expected f16 bits were produced by the reference's Python), then larger shapes with several
    blocks, negative block scales, bf16 and f32 activations, against the CPU lane: equal bits everywhere."""
    op, ctx, k = gpu
    wp, ws, s2 = golden["a16_w_packed"], golden["a16_w_scales"], float(golden["a16_scale2"])
    x16 = torch.from_numpy(golden["a16_activation_f16_bits"].view(np.float16).astype(np.float32))
    w = op.Weight(ctx, op.TensorView(wp, O.NVFP4, 256, 11, ws, s2, None))
    y = torch.zeros((7, 11), dtype=torch.float16, device="cuda")
    k.encode_nvfp4_matmul(w, x16.cuda(), y, 7)
    ctx.sync_status()
    assert np.array_equal(y.cpu().numpy().view(np.uint16), golden["a16_expected_f16_bits"])
    w.free()
    for n_out, n_in, tokens, x_dtype in ((300, 1024, 19, torch.bfloat16), (37, 2560, 8, torch.float32), (130, 256, 1, torch.float32)):
        packed, scales, scale2 = make_weight(op, ctx, n_out, n_in, seed=n_out, negative_scales=True)
        w = op.Weight(ctx, op.TensorView(packed, O.NVFP4, n_in, n_out, scales, scale2, None))
        x = (torch.from_numpy(H.lcg_activations(tokens * n_in, seed=tokens).reshape(tokens, n_in)) * 3.0).to(x_dtype)
        x[0, :256] = 0.0   # a block of zeros is skipped
        want = O.matmul(O.TensorView(packed, O.NVFP4, n_in, n_out, scales, scale2, None), x.float().numpy(), threads=4)
        y = torch.full((tokens, n_out), float("nan"), dtype=torch.float32, device="cuda")
        k.encode_nvfp4_matmul(w, x.cuda(), y, tokens)
        ctx.sync_status()
        assert np.array_equal(y.cpu().numpy().view(np.uint32), want.astype(np.float32).view(np.uint32)), (n_out, n_in, tokens)
        w.free()


def test_workspace_and_dtype_misuse(gpu):
    op, ctx, k = gpu
    packed, scales, scale2 = make_weight(op, ctx, 64, 256, seed=1)
    w_only = op.Weight(ctx, op.TensorView(packed, O.NVFP4, 256, 64, scales, scale2, None))
    x = torch.zeros((4, 256), dtype=torch.bfloat16, device="cuda")
    y = torch.zeros((4, 64), dtype=torch.float32, device="cuda")
    k.encode_nvfp4_matmul(w_only, x, y, 4)   # no input_scale_inv: the weight-only lane serves it
    xp, xs = k.quantize_nvfp4_activation(x, 10.0)
    with pytest.raises(op.MuserCudaError) as e:
        k.encode_nvfp4_prequant(w_only, xp, xs, y, 4)   # pre-quantized activations are the W4A4 lane's
    assert e.value.status_name == "UNSUPPORTED_DTYPE"
    with pytest.raises(op.MuserCudaError) as e:
        k.encode_nvfp4_matmul(w_only, x, y, 4, residual=y)   # the weight-only lane fuses nothing
    assert e.value.status_name == "BAD_ARG"
    small = op.Context(0, workspace_bytes=1024)
    w = op.Weight(small, op.TensorView(packed, O.NVFP4, 256, 64, scales, scale2, 10.0))
    with pytest.raises(op.MuserCudaError) as e:
        op.CudaKernels(small).encode_nvfp4_matmul(w, x, y, 4)
    assert e.value.status_name == "WORKSPACE_TOO_SMALL"
    w.free()
    small.close()


@pytest.mark.parametrize("group_m", [1, 2, 3])
def test_raster_groups_do_not_change_the_outputs(gpu, group_m):
    """MUSER_TUNE_NVFP4_GROUP_M only reorders the output tiles (groups of token tiles; the last group short when the
    tile count is no multiple): every output must carry the same bits as with all token tiles in one group, in the
    plain, the fused gate/up and the quantized-output forms."""
    from muser_b200 import synth
    from muser_b200._lib import TUNE_NVFP4_GROUP_M
    op, ctx, k = gpu
    n_out, n_in, tokens = 768, 512, 900  # 8 token tiles (the last one ragged), 3 weight-row tiles
    packed, scales, scale2 = make_weight(op, ctx, n_out, n_in, seed=91, negative_scales=True)
    up, us, u2 = make_weight(op, ctx, n_out, n_in, seed=92)
    x = synth.normal_activations(tokens, n_in, seed=93)
    isi = synth.activation_input_scale_inv(x)
    w = op.Weight(ctx, op.TensorView(packed, O.NVFP4, n_in, n_out, scales, scale2, isi))
    wu = op.Weight(ctx, op.TensorView(up, O.NVFP4, n_in, n_out, us, u2, isi))
    xp, xs = k.quantize_nvfp4_activation(x.cuda(), isi)
    out = {}
    try:
        for gm in (0, group_m):
            ctx.tuning_set(TUNE_NVFP4_GROUP_M, gm)
            y = torch.full((tokens, n_out), float("nan"), dtype=torch.float32, device="cuda")
            y2 = torch.full((tokens, n_out), float("nan"), dtype=torch.float32, device="cuda")
            k.encode_nvfp4_prequant(w, xp, xs, y, tokens)
            k.encode_nvfp4_ffn_gate_up_silu_prequant(w, wu, xp, xs, y2, tokens)
            qp, qs = k.encode_nvfp4_ffn_gate_up_silu_requant(w, wu, xp, xs, tokens, 0.37)
            ctx.sync_status()
            out[gm] = [t.cpu() for t in (y, y2, qp, qs)]
    finally:
        ctx.tuning_set(TUNE_NVFP4_GROUP_M, 0)
    for i, (a, b) in enumerate(zip(out[0], out[group_m])):
        assert torch.equal(a.view(torch.int32) if a.dtype == torch.float32 else a, b.view(torch.int32) if b.dtype == torch.float32 else b), f"output {i}"
    assert not torch.isnan(out[group_m][0]).any()


@pytest.mark.parametrize("shapes,n_in,tokens", [((512, 256, 256), 512, 300), ((300, 128), 1088, 130), ((768, 256, 256, 1000), 256, 700)])
def test_grouped_projections_equal_the_single_calls(gpu, shapes, n_in, tokens):
    """muser_cuda_nvfp4_matmul_group_prequant (q | k | v in one launch): every output must carry the bits of
    muser_cuda_nvfp4_matmul_prequant on that weight alone; rows that do not fill a tile, ragged K and tokens, two to
    four projections.  Misuse (different n_in or input_scale_inv, one weight, five weights) is refused."""
    from muser_b200 import synth
    op, ctx, k = gpu
    x = synth.normal_activations(tokens, n_in, seed=31)
    isi = synth.activation_input_scale_inv(x)
    ws = []
    for i, n_out in enumerate(shapes):
        packed, scales, scale2 = make_weight(op, ctx, n_out, n_in, seed=200 + i, negative_scales=(i == 0))
        ws.append(op.Weight(ctx, op.TensorView(packed, O.NVFP4, n_in, n_out, scales, scale2, isi)))
    xp, xs = k.quantize_nvfp4_activation(x.cuda(), isi)
    for dt in (torch.float32, torch.bfloat16):
        alone = [torch.full((tokens, n), float("nan"), dtype=dt, device="cuda") for n in shapes]
        for w, y in zip(ws, alone):
            k.encode_nvfp4_prequant(w, xp, xs, y, tokens)
        grouped = [torch.full((tokens, n), float("nan"), dtype=dt, device="cuda") for n in shapes]
        k.encode_nvfp4_group_prequant(ws, xp, xs, grouped, tokens)
        ctx.sync_status()
        bits = torch.int32 if dt == torch.float32 else torch.int16
        for i, (a, b) in enumerate(zip(alone, grouped)):
            assert torch.equal(a.view(bits), b.view(bits)), f"projection {i} ({dt}) differs from the call on its own"
    # misuse
    other = make_weight(op, ctx, 256, n_in, seed=300)
    w_isi = op.Weight(ctx, op.TensorView(other[0], O.NVFP4, n_in, 256, other[1], other[2], isi * 2.0))
    y = torch.empty((tokens, 256), dtype=torch.float32, device="cuda")
    with pytest.raises(op.MuserCudaError):
        k.encode_nvfp4_group_prequant([ws[0], w_isi], xp, xs, [grouped[0], y], tokens)
    with pytest.raises(op.MuserCudaError):
        k.encode_nvfp4_group_prequant([ws[0]], xp, xs, [grouped[0]], tokens)
