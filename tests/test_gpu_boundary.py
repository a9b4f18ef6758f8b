"""Boundary behaviour of the C ABI on a GPU: per-device launch state, host threads, bounded-wait reporting."""
import threading

import numpy as np
import pytest
import torch

from oracle import oracle as O
from tests import helpers as H

pytestmark = pytest.mark.gpu


def _kquant_case(dtype, rows, blocks, seed):
    raw = H.lcg_weights(dtype, rows, blocks, seed=seed)
    return raw, O.TensorView(raw, dtype, blocks * 256, rows)


def test_two_contexts_from_two_host_threads():
    """Contexts are thread-compatible: two host threads, each with its own context and stream, run every kernel
    family at once (the launchers' cached plans and per-device attributes are shared state under a lock)."""
    from muser_b200 import operator as op
    raw4, ow4 = _kquant_case(O.Q4_K, 300, 8, 11)
    raw6, ow6 = _kquant_case(O.Q6_K, 2100, 4, 12)
    xs = {t: torch.from_numpy(H.lcg_activations(t * 4096, seed=3 + t).reshape(t, 4096)).to(torch.bfloat16) for t in (1, 4, 16)}
    want = {(name, t): O.matmul(ow, xs[t][:, :ow.n_in].float().numpy(), threads=4)
            for name, ow in (("q4", ow4), ("q6", ow6)) for t in xs}
    errors = []

    def worker(idx):
        try:
            torch.cuda.set_device(0)
            ctx = op.Context(0, workspace_bytes=1 << 20)
            k = op.CudaKernels(ctx)
            stream = torch.cuda.Stream()
            w4 = op.Weight(ctx, op.TensorView(raw4, O.Q4_K, ow4.n_in, ow4.n_out))
            w6 = op.Weight(ctx, op.TensorView(raw6, O.Q6_K, ow6.n_in, ow6.n_out))
            with torch.cuda.stream(stream):
                for rep in range(20):
                    for name, w, ow in (("q4", w4, ow4), ("q6", w6, ow6)):
                        for t, x in xs.items():
                            xd = x[:, :ow.n_in].contiguous().cuda()
                            y = torch.full((t, ow.n_out), float("nan"), dtype=torch.float32, device="cuda")
                            k.encode_quantized_matmul(w, xd, y, t)
                            stream.synchronize()
                            r = H.rel_l2(y.cpu().numpy(), want[(name, t)])
                            if not r <= 1e-3:
                                errors.append((idx, rep, name, t, r))
                ctx.sync_status()
            w4.free()
            w6.free()
            ctx.close()
        except Exception as exc:  # surfaced by the assert below
            errors.append((idx, repr(exc)))

    threads = [threading.Thread(target=worker, args=(i,)) for i in range(2)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert not errors, errors[:4]


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs in one process")
def test_two_devices_in_one_process():
    """One process, a context on each of two GPUs: kernels that need more than 48 KB of dynamic shared memory must
    launch on the second device too (that attribute is per device)."""
    from muser_b200 import operator as op
    from muser_b200 import synth
    raw, ow = _kquant_case(O.Q4_K, 2100, 8, 21)
    wq, ws, scale2 = synth.nvfp4_weight(synth.normal_weights(300, 1280, seed=3, stream=11))
    x_all = synth.normal_activations(64, 2048, seed=5)
    isi = synth.activation_input_scale_inv(x_all[:, :1280])
    ow_fp4 = O.TensorView(wq.numpy(), O.NVFP4, 1280, 300, ws.numpy(), scale2, isi)
    for dev in (0, 1):
        torch.cuda.set_device(dev)
        ctx = op.Context(dev, workspace_bytes=16 << 20)
        k = op.CudaKernels(ctx)
        w = op.Weight(ctx, op.TensorView(raw, O.Q4_K, ow.n_in, ow.n_out))
        for t in (1, 8, 16):
            x = x_all[:t].contiguous()
            y = torch.full((t, ow.n_out), float("nan"), dtype=torch.float32, device=f"cuda:{dev}")
            k.encode_quantized_matmul(w, x.to(f"cuda:{dev}"), y, t)
            assert H.rel_l2(y.cpu().numpy(), O.matmul(ow, x.float().numpy(), threads=4)) <= 1e-3, (dev, t)
        wf = op.Weight(ctx, op.TensorView(wq.numpy(), O.NVFP4, 1280, 300, ws.numpy(), scale2, isi))
        x = x_all[:64, :1280].contiguous()
        y = torch.full((64, 300), float("nan"), dtype=torch.float32, device=f"cuda:{dev}")
        k.encode_nvfp4_matmul(wf, x.to(f"cuda:{dev}"), y, 64)
        _, ref = O.matmul(ow_fp4, x.float().numpy(), threads=4, return_pre_round=True)
        assert H.rel_l2(y.cpu().numpy(), ref) <= 1e-3, dev
        ctx.sync_status()
        w.free()
        wf.free()
        ctx.close()
    torch.cuda.set_device(0)


def test_bounded_wait_expiry_is_reported_once_and_the_context_stays_usable():
    """A wait that runs out must come back as MUSER_CUDA_TIMEOUT from muser_cuda_sync_status, once, and leave the
    context healthy.  The expiry is made on purpose by a one-thread kernel that polls a barrier nobody arrives at
    a thousand times and then records its give-up code like the projection kernels do: no hang, no fault."""
    from muser_b200 import _lib
    from muser_b200 import operator as op
    ctx = op.Context(0, workspace_bytes=1 << 20)
    k = op.CudaKernels(ctx)
    ctx.sync_status()
    stream = torch.cuda.current_stream().cuda_stream
    ctx.check(_lib.lib.muser_cuda_wait_probe(ctx._h, 1000, stream))
    with pytest.raises(op.MuserCudaError) as e:
        ctx.sync_status()
    assert e.value.status_name == "TIMEOUT" and "901" in str(e.value)
    ctx.sync_status()  # cleared: the second read is clean
    raw, ow = _kquant_case(O.Q4_K, 37, 2, 5)
    w = op.Weight(ctx, op.TensorView(raw, O.Q4_K, 512, 37))
    x = torch.from_numpy(H.lcg_activations(2 * 512, seed=9).reshape(2, 512)).to(torch.bfloat16)
    y = torch.empty((2, 37), dtype=torch.float32, device="cuda")
    k.encode_quantized_matmul(w, x.cuda(), y, 2)
    ctx.sync_status()
    assert H.rel_l2(y.cpu().numpy(), O.matmul(ow, x.float().numpy())) <= 1e-3
    assert _lib.lib.muser_cuda_wait_probe(ctx._h, 0, stream) == 1  # BAD_ARG
    w.free()
    ctx.close()


def test_misuse_on_k_shards_is_refused():
    """softcap is not linear, so it cannot run on a K shard's partial sums (the ranks add them afterwards)."""
    from muser_b200 import operator as op
    ctx = op.Context(0, workspace_bytes=1 << 20)
    k = op.CudaKernels(ctx)
    raw, _ = _kquant_case(O.Q4_K, 37, 4, 6)
    w = op.Weight(ctx, op.TensorView(raw, O.Q4_K, 1024, 37), shard=(0, 2, op.SHARD_K))
    x = torch.zeros((1, 512), dtype=torch.bfloat16, device="cuda")
    y = torch.zeros((1, 37), dtype=torch.float32, device="cuda")
    with pytest.raises(op.MuserCudaError) as e:
        k.encode_quantized_matmul(w, x, y, 1, softcap=30.0)
    assert e.value.status_name == "BAD_SHAPE"
    k.encode_quantized_matmul(w, x, y, 1, out_scale=0.5)  # a plain scale is linear and stays allowed
    w.free()
    ctx.close()


def test_image_hash_is_deterministic_and_tells_shards_apart():
    """Repacking is deterministic: two repacks of one tensor (host and device source, two contexts) carry the same
    64-bit image digest; another tensor, another dtype and each tensor-parallel shard carry different ones."""
    from muser_b200 import operator as op
    from muser_b200 import synth
    from muser_b200._lib import NVFP4, SHARD_K, SHARD_ROWS
    ctx_a, ctx_b = op.Context(0, workspace_bytes=1 << 20), op.Context(0, workspace_bytes=1 << 20)
    try:
        raw, ow = _kquant_case(O.Q4_K, 512, 8, 21)
        view = op.TensorView(raw, O.Q4_K, ow.n_in, ow.n_out)
        h = [op.Weight(ctx_a, view).info().image_hash, op.Weight(ctx_b, view).info().image_hash,
             op.Weight(ctx_a, op.TensorView(torch.from_numpy(raw).cuda(), O.Q4_K, ow.n_in, ow.n_out)).info().image_hash]
        assert h[0] == h[1] == h[2] and h[0] != 0
        other, _ = _kquant_case(O.Q4_K, 512, 8, 22)
        assert op.Weight(ctx_a, op.TensorView(other, O.Q4_K, ow.n_in, ow.n_out)).info().image_hash != h[0]
        shards = {op.Weight(ctx_a, view, shard=(r, 2, axis)).info().image_hash for r in (0, 1) for axis in (SHARD_ROWS, SHARD_K)}
        assert len(shards) == 4 and h[0] not in shards
        raw6, ow6 = _kquant_case(O.Q6_K, 512, 8, 21)
        assert op.Weight(ctx_a, op.TensorView(raw6, O.Q6_K, ow6.n_in, ow6.n_out)).info().image_hash != h[0]
        wp, ws, s2 = synth.nvfp4_weight(synth.normal_weights(256, 512, seed=0, stream=1))
        n1 = op.Weight(ctx_a, op.TensorView(wp, NVFP4, 512, 256, ws, s2, 4.0)).info().image_hash
        n2 = op.Weight(ctx_b, op.TensorView(wp, NVFP4, 512, 256, ws, s2, 4.0)).info().image_hash
        n3 = op.Weight(ctx_a, op.TensorView(wp, NVFP4, 512, 256, ws, s2, 4.0), shard=(1, 2, SHARD_ROWS)).info().image_hash
        assert n1 == n2 and n1 != n3
    finally:
        ctx_a.close()
        ctx_b.close()
