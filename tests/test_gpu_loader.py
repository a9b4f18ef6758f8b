"""Model file -> repacked device images -> projections: the loader row next to the hot path, on a GPU."""
import struct

import numpy as np
import pytest
import torch

from oracle import oracle as O
from tests import helpers as H

pytestmark = pytest.mark.gpu


def test_gguf_file_to_device_projections(tmp_path):
    """A synthetic GGUF file with a Q4_K, a Q6_K and an NVFP4 (W4A4) projection: each tensor is loaded straight from
    the memory map into its repacked image and must decode bit-exactly and project within the stated tolerance."""
    from muser_b200 import gguf as G
    from muser_b200 import operator as op
    from muser_b200 import synth
    n_in, n_out = 1024, 48
    q4, q6 = H.lcg_weights(O.Q4_K, n_out, n_in // 256, seed=8), H.lcg_weights(O.Q6_K, n_out, n_in // 256, seed=9)
    wp, ws, scale2 = synth.nvfp4_weight(synth.normal_weights(n_out, n_in, seed=1, stream=3))
    x = synth.normal_activations(5, n_in, seed=2)
    isi = synth.activation_input_scale_inv(x)
    path = tmp_path / "layer.gguf"
    G.write_gguf(path, {
        "blk.0.attn_q.weight": (G.Q4_K, [n_in, n_out], q4),
        "blk.0.ffn_down.weight": (G.Q6_K, [n_in, n_out], q6),
        "blk.0.ffn_gate.weight": (G.NVFP4_E2M1, [n_in, n_out], wp.numpy()),
        "blk.0.ffn_gate.weight.nvfp4_scale": (G.F8_E4M3FN, [n_in // 16, n_out], ws.numpy()),
        "blk.0.ffn_gate.weight.nvfp4_scale2": (G.F32, [1], struct.pack("<f", scale2)),
        "blk.0.ffn_gate.weight.nvfp4_input_scale_inv": (G.F32, [1], struct.pack("<f", isi)),
    }, {"general.architecture": (8, "muse"), "muser.activation_precision": (8, "nvfp4")})
    weights = G.MuseWeights.open(path)
    ctx = op.Context(0)
    k = op.CudaKernels(ctx)
    for name, raw, dtype in (("blk.0.attn_q.weight", q4, O.Q4_K), ("blk.0.ffn_down.weight", q6, O.Q6_K)):
        w = weights.load(ctx, name)
        ow = O.TensorView(raw, dtype, n_in, n_out)
        assert np.array_equal(k.dequant(w).cpu().numpy().view(np.uint32), O.dequant_tensor(ow).view(np.uint32)), name
        y = torch.empty((5, n_out), dtype=torch.float32, device="cuda")
        k.encode_quantized_matmul(w, x.cuda(), y, 5)
        assert H.rel_l2(y.cpu().numpy(), O.matmul(ow, x.float().numpy())) <= 1e-3, name
        # a tensor-parallel shard loads from the same view
        ws_ = weights.load(ctx, name, shard=(1, 2, op.SHARD_ROWS))
        assert np.array_equal(k.dequant(ws_).cpu().numpy(), k.dequant(w).cpu().numpy()[n_out // 2:])
    w = weights.load(ctx, "blk.0.ffn_gate.weight")
    assert w.input_scale_inv == pytest.approx(isi)
    y = torch.empty((5, n_out), dtype=torch.float32, device="cuda")
    k.encode_nvfp4_matmul(w, x.cuda(), y, 5)
    ctx.sync_status()
    ow = O.TensorView(wp.numpy(), O.NVFP4, n_in, n_out, ws.numpy(), scale2, isi)
    _, ref = O.matmul(ow, x.float().numpy(), return_pre_round=True)
    assert H.rel_l2(y.cpu().numpy(), ref) <= 1e-3
    assert np.array_equal(k.dequant(w).cpu().numpy().view(np.uint32), O.dequant_nvfp4(wp.numpy(), ws.numpy(), scale2).view(np.uint32))
    weights.close()
    ctx.close()
