"""GPU parity of the operations either side of the projections (sandwich-norm tail, attention gate, per-head norm)
against the CPU lane's composition in the oracle."""
import numpy as np
import pytest
import torch

from oracle import oracle as O
from tests import helpers as H

pytestmark = pytest.mark.gpu

REL_TOL = 2e-6  # f32 elementwise work; only the order of the sums of squares differs from the CPU lane


@pytest.fixture(scope="module")
def gpu():
    from muser_b200 import operator as op
    ctx = op.Context(0, workspace_bytes=1 << 20)
    yield op, ctx, op.CudaKernels(ctx)
    ctx.close()


def _rand(shape, seed, scale=1.0):
    return (torch.randn(shape, generator=torch.Generator().manual_seed(seed)) * scale).float()


@pytest.mark.parametrize("tokens,n", [(1, 5120), (8, 5120), (3, 260), (16, 27648)])
def test_sandwich_norm_tail(gpu, tokens, n):
    """hidden += rms_norm(src, 1e-8) * w1; output = rms_norm(hidden, 1e-5) * w2 (rmsnorm_batch_tail.metal:147-200)."""
    op, ctx, k = gpu
    hidden, src = _rand((tokens, n), 1), _rand((tokens, n), 2, 0.03)
    w1, w2 = 1.0 + 0.1 * _rand((n,), 3), 1.0 + 0.1 * _rand((n,), 4)
    want_h, want_o = O.norm_residual_norm(hidden.numpy(), src.numpy(), w1.numpy(), 1e-8, w2.numpy(), 1e-5)
    h, out = hidden.cuda(), torch.full((tokens, n), float("nan"), device="cuda")
    k.encode_fused_norm_residual_rms_norm(h, src.cuda(), w1.cuda(), 1e-8, out, w2.cuda(), 1e-5)
    ctx.sync_status()
    assert H.rel_l2(h.cpu().numpy(), want_h) <= REL_TOL and H.rel_l2(out.cpu().numpy(), want_o) <= REL_TOL
    assert np.max(np.abs(out.cpu().numpy() - want_o)) <= 1e-5 * np.max(np.abs(want_o))
    # without the second norm
    h2 = hidden.cuda()
    k.encode_fused_norm_residual_rms_norm(h2, src.cuda(), w1.cuda(), 1e-8)
    ctx.sync_status()
    assert torch.equal(h2, h)
    # tiny inputs: the post-norm's own epsilon (1e-8) matters, the pre-norm's (1e-5) would flatten them
    tiny = _rand((tokens, n), 5, 1e-4)
    want_h, _ = O.norm_residual_norm(np.zeros((tokens, n), np.float32), tiny.numpy(), w1.numpy(), 1e-8)
    h3 = torch.zeros((tokens, n), device="cuda")
    k.encode_fused_norm_residual_rms_norm(h3, tiny.cuda(), w1.cuda(), 1e-8)
    ctx.sync_status()
    assert H.rel_l2(h3.cpu().numpy(), want_h) <= REL_TOL


def test_sigmoid_gate(gpu):
    op, ctx, k = gpu
    x, gate = _rand((5, 5120), 7), _rand((5, 5120), 8, 4.0)
    gate[0, :4] = torch.tensor([-100.0, 100.0, 0.0, -0.0])
    want = O.sigmoid_gate(x.numpy(), gate.numpy())
    xd = x.cuda()
    k.encode_sigmoid_gate(xd, gate.cuda())
    ctx.sync_status()
    got = xd.cpu().numpy()
    assert H.rel_l2(got, want) <= REL_TOL and np.max(np.abs(got - want)) <= 2e-6 * np.max(np.abs(want))


@pytest.mark.parametrize("tokens,heads,head_dim", [(1, 40, 128), (8, 8, 128), (3, 5, 64), (2, 3, 256)])
def test_per_head_norm(gpu, tokens, heads, head_dim):
    """rms_norm_mul over head_dim-long pieces (reference.rs:384-393), weight a broadcast constant as in the model."""
    op, ctx, k = gpu
    x = _rand((tokens, heads * head_dim), 9, 3.0)
    w = torch.full((head_dim,), 0.0884) + 0.01 * _rand((head_dim,), 10)
    want = O.rms_norm_mul(x.numpy().reshape(-1, head_dim), 1e-5, w.numpy()).reshape(tokens, heads * head_dim)
    xd = x.cuda()
    k.encode_head_rms_norm(xd, w.cuda(), 1e-5, heads)
    ctx.sync_status()
    assert H.rel_l2(xd.cpu().numpy(), want) <= REL_TOL


def test_a_decoder_layers_non_attention_work_stays_on_the_device(gpu):
    """The calls in the order a decode step issues them (reference.rs:348-542, attention itself left out): attn_norm
    fused into q | k | v | gate, per-head norm of q and k, sigmoid gate, o_proj, post-norm + residual + ffn_norm,
    gate | up with SwiGLU, down, post-norm + residual; against the CPU lane's composition, K-quant weights."""
    op, ctx, k = gpu
    from muser_b200 import synth
    hdim, heads, kv_heads, hd, ffn, tokens = 1024, 8, 2, 128, 2048, 4
    shapes = {"q": (hdim, heads * hd, O.Q4_K), "k": (hdim, kv_heads * hd, O.Q4_K), "v": (hdim, kv_heads * hd, O.Q6_K),
              "gate": (hdim, heads * hd, O.Q4_K), "o": (heads * hd, hdim, O.Q4_K), "ffn_gate": (hdim, ffn, O.Q4_K),
              "ffn_up": (hdim, ffn, O.Q4_K), "ffn_down": (ffn, hdim, O.Q6_K)}
    raw = {n: synth.quantize_kquant(synth.normal_weights(o, i, seed=0, stream=40 + j), dt).numpy() for j, (n, (i, o, dt)) in enumerate(shapes.items())}
    ow = {n: O.TensorView(raw[n], dt, i, o) for n, (i, o, dt) in shapes.items()}
    w = {n: op.Weight(ctx, op.TensorView(raw[n], dt, i, o)) for n, (i, o, dt) in shapes.items()}
    nw = {n: (1.0 + 0.1 * _rand((hdim,), 20 + j)) for j, n in enumerate(("attn", "post_attn", "ffn", "post_ffn"))}
    qn, kn = torch.full((hd,), 0.0884), torch.ones(hd)
    hidden = _rand((tokens, hdim), 30)
    eps, eps_post = 1e-5, 1e-8
    # CPU lane
    x = O.rms_norm_mul(hidden.numpy(), eps, nw["attn"].numpy())
    mm = lambda name, a: O.matmul(ow[name], a, threads=4)
    q, kk, v, g = mm("q", x), mm("k", x), mm("v", x), mm("gate", x)
    q = O.rms_norm_mul(q.reshape(-1, hd), eps, qn.numpy()).reshape(tokens, -1)
    kk = O.rms_norm_mul(kk.reshape(-1, hd), eps, kn.numpy()).reshape(tokens, -1)
    attn = q  # attention itself is not on this path: its output is stood in for by q
    proj = mm("o", O.sigmoid_gate(attn, g))
    h1, y = O.norm_residual_norm(hidden.numpy(), proj, nw["post_attn"].numpy(), eps_post, nw["ffn"].numpy(), eps)
    down = mm("ffn_down", O.silu_mul(mm("ffn_gate", y), mm("ffn_up", y)))
    h2, _ = O.norm_residual_norm(h1, down, nw["post_ffn"].numpy(), eps_post)
    # device
    f32 = dict(dtype=torch.float32, device="cuda")
    hd_, outs = hidden.cuda(), {n: torch.empty((tokens, shapes[n][1]), **f32) for n in ("q", "k", "v", "gate")}
    norm = dict(norm_weight=nw["attn"].cuda(), norm_eps=eps)
    k.encode_quantized_matmul_group([w[n] for n in outs], hd_, list(outs.values()), tokens, epilogues=[norm] * 4)
    k.encode_head_rms_norm(outs["q"], qn.cuda(), eps, heads)
    k.encode_head_rms_norm(outs["k"], kn.cuda(), eps, kv_heads)
    k.encode_sigmoid_gate(outs["q"], outs["gate"])
    proj_d = torch.empty((tokens, hdim), **f32)
    k.encode_quantized_matmul(w["o"], outs["q"], proj_d, tokens)
    y_d = torch.empty((tokens, hdim), **f32)
    k.encode_fused_norm_residual_rms_norm(hd_, proj_d, nw["post_attn"].cuda(), eps_post, y_d, nw["ffn"].cuda(), eps)
    act = torch.empty((tokens, ffn), **f32)
    k.encode_ffn_gate_up_silu(w["ffn_gate"], w["ffn_up"], y_d, act, tokens)
    down_d = torch.empty((tokens, hdim), **f32)
    k.encode_quantized_matmul(w["ffn_down"], act, down_d, tokens)
    k.encode_fused_norm_residual_rms_norm(hd_, down_d, nw["post_ffn"].cuda(), eps_post)
    ctx.sync_status()
    assert H.rel_l2(outs["k"].cpu().numpy(), kk) <= 1e-3 and H.rel_l2(outs["v"].cpu().numpy(), v) <= 1e-3
    assert H.rel_l2(y_d.cpu().numpy(), y) <= 1e-3
    assert H.rel_l2(hd_.cpu().numpy(), h2) <= 1e-3, H.rel_l2(hd_.cpu().numpy(), h2)
    for ww in w.values():
        ww.free()
