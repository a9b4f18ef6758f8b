"""The allocation-free NVFP4 entry point (muser_cuda_nvfp4_matmul_static) against the context-based one.

Some hosts of this library work out of arenas they sized once and cannot hand the backend an allocator, nor let
it take the device-wide lock that cudaMalloc / cudaFree hold while a step is in flight.  For them the quantized
activations pass through an array inside the library image instead of a context's workspace.  The kernels are the
same, so the two entry points must agree bit for bit; two calls in a row (the second smaller, over the first
call's leftovers in the shared array) check that nothing stale leaks into a result.

Collected last on purpose: a run that stops at the first failure has then already run every other test.
"""
import numpy as np
import pytest
import torch

from oracle import oracle as O
from tests import helpers as H

pytestmark = pytest.mark.gpu


def test_static_scratch_entry_point_matches_context_entry_point_twice():
    from muser_b200 import operator as op
    from muser_b200 import synth
    ctx = op.Context(0, workspace_bytes=16 << 20)
    k = op.CudaKernels(ctx)
    n_in, n_out = 1280, 300
    wq, ws, scale2 = synth.nvfp4_weight(synth.normal_weights(n_out, n_in, seed=3, stream=11))
    x_all = synth.normal_activations(128, n_in, seed=5)
    isi = synth.activation_input_scale_inv(x_all)
    w = op.Weight(ctx, op.TensorView(wq.numpy(), O.NVFP4, n_in, n_out, ws.numpy(), scale2, isi))
    ow = O.TensorView(wq.numpy(), O.NVFP4, n_in, n_out, ws.numpy(), scale2, isi)
    calls = 0
    for tokens, y_dtype in ((128, torch.float32), (37, torch.float16)):   # two calls in a row, the second smaller
        x = x_all[:tokens].contiguous().cuda()
        want = torch.full((tokens, n_out), float("nan"), dtype=y_dtype, device="cuda")
        k.encode_nvfp4_matmul(w, x, want, tokens)
        got = torch.full((tokens, n_out), float("nan"), dtype=y_dtype, device="cuda")
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]
        op.nvfp4_matmul_static(w, x, got, tokens)
        op.static_sync_status(0)   # synchronizes; raises if a bounded wait inside the call gave up
        if calls:                  # (the first call on a device may still load the kernels' code)
            assert torch.cuda.mem_get_info()[0] == free_before, "the static entry point must not allocate device memory"
        calls += 1
        assert torch.equal(got.view(torch.int16 if y_dtype == torch.float16 else torch.int32),
                           want.view(torch.int16 if y_dtype == torch.float16 else torch.int32))
        ref_f16, ref_f32 = O.matmul(ow, x.float().cpu().numpy(), threads=O.host_threads(), return_pre_round=True)
        ref = ref_f32 if y_dtype == torch.float32 else ref_f16
        assert H.rel_l2(got.float().cpu().numpy(), ref) <= 1e-3   # the tolerance of tests/test_gpu_nvfp4.py
    # sizes beyond the array are refused, with a message, before anything is launched
    big = torch.zeros((129, n_in), dtype=torch.bfloat16, device="cuda")
    out = torch.zeros((129, n_out), dtype=torch.float32, device="cuda")
    with pytest.raises(op.MuserCudaError) as e:
        op.nvfp4_matmul_static(w, big, out, 129)
    assert e.value.status_name == "WORKSPACE_TOO_SMALL" and "128" in str(e.value)
    w.free()
    ctx.close()
