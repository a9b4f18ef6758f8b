"""One rank of the two-GPU tensor-parallel test (started by tests/test_gpu_tp.py through torch.distributed.run).

Checks, through the C ABI only: the library's all-reduce (one-shot peer exchange and the NCCL path) against
torch.distributed's, plain and replayed from a CUDA graph; the tensor-parallel decode layer against the CPU lane on
the unsharded tensors; and that a wait which runs out (a peer that does not take part in one call, between steps) comes
back as MUSER_CUDA_TIMEOUT with the context still usable.  Prints TP_WORKER_OK on success."""
import os
import sys
from pathlib import Path

import numpy as np
import torch
import torch.distributed as dist

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))


def main():
    from muser_b200 import operator as op
    from muser_b200 import tp, workloads
    from oracle import oracle as O
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    ctx = op.Context(local, workspace_bytes=1 << 20)
    kern = op.CudaKernels(ctx)
    coll = tp.Collective(ctx, rank, world)
    assert coll.oneshot, "peer buffers were not mapped: " + (op._L.muser_cuda_last_error(ctx._h) or b"").decode()

    # 1. sums of several sizes (one CTA, several CTAs, a ragged tail, the largest one-shot payload, one past it -> NCCL)
    for count in (4, 5120, 5123, 8 * 5120, 65536, 393216, 393220, 1 << 20):
        g = torch.Generator(device=dev).manual_seed(100 * rank + count % 97)
        x = torch.randn(count, device=dev, generator=g)
        want = x.clone()
        dist.all_reduce(want)
        for _ in range(3):   # repeated calls walk both slots
            got = x.clone()
            coll.all_reduce_sum(got)
            ctx.sync_status()
            assert torch.allclose(got, want, rtol=1e-6, atol=1e-6), (count, float((got - want).abs().max()))
        gathered = [torch.empty_like(got) for _ in range(world)]
        dist.all_gather(gathered, got)
        assert all(torch.equal(gathered[0], t) for t in gathered), "ranks must end with identical bits"
    xb = torch.randn(4096, device=dev).to(torch.bfloat16)
    wb = xb.clone()
    dist.all_reduce(wb)
    coll.all_reduce_sum(xb)
    assert torch.allclose(xb.float(), wb.float(), rtol=2e-2, atol=2e-2)

    # 2. the same call replayed from a CUDA graph (nothing that changes per call is a launch argument)
    buf, src = torch.zeros(5120, device=dev), torch.randn(5120, device=dev)

    def step():
        buf.copy_(src)
        coll.all_reduce_sum(buf)

    replay = workloads.capture(step)
    want = src.clone()
    dist.all_reduce(want)
    for _ in range(5):
        replay()
    ctx.sync_status()
    assert torch.allclose(buf, want, rtol=1e-6, atol=1e-6)

    # 3. tensor-parallel decode layer against the CPU lane on the unsharded tensors
    plan = tp.ShardPlan(rank, world)
    layer = workloads.DecodeLayer(ctx, kern, plan, (1, 8), dev, all_reduce=coll.all_reduce_sum)
    for m in (1, 8):
        layer.run(m)
        ctx.sync_status()
        for gi, name in ((1, "attn_o"), (3, "ffn_down")):
            k, n, dt = layer.projs[name]
            rows = np.sort(np.random.default_rng(7).choice(n, 48, replace=False))
            sub = layer.views[name].raw.cpu().numpy().reshape(n, -1)[rows].copy()
            ref = O.matmul(O.TensorView(sub, dt, k, len(rows)), layer.full_input(gi, m).float().cpu().numpy(), threads=4)
            got = layer.y[(name, m)][:, torch.from_numpy(rows).to(dev)].cpu().numpy()
            err = float(np.linalg.norm(got - ref) / np.linalg.norm(ref))
            assert err <= 1e-3, (name, m, err)
        # a column-parallel projection: this rank's rows of the unsharded result
        k, n, dt = layer.projs["attn_k"]
        sl = plan.output_slice("attn_k", n)
        sub = layer.views["attn_k"].raw.cpu().numpy().reshape(n, -1)[sl].copy()
        ref = O.matmul(O.TensorView(sub, dt, k, sub.shape[0]), layer.full_input(0, m).float().cpu().numpy(), threads=4)
        got = layer.y[("attn_k", m)].cpu().numpy()
        assert float(np.linalg.norm(got - ref) / np.linalg.norm(ref)) <= 1e-3

    # 3b. the fused form: the row-parallel projection pushes its partial sums to the peers itself (all_reduce in its
    #     epilogue) and a small kernel gathers.  Same values in the same rank order as projection + all-reduce, so the
    #     outputs must carry the same bits, on every rank, also when replayed from a CUDA graph and when interleaved
    #     with plain all-reduces (the sequence numbers are shared).
    separate = {(n, m): layer.y[(n, m)].clone() for n in ("attn_o", "ffn_down") for m in (1, 8)}
    fused_layer = workloads.DecodeLayer(ctx, kern, plan, (1, 8), dev, all_reduce=coll.all_reduce_sum, fuse_all_reduce=True, autotune=False)
    for m in (1, 8):
        fused_layer.run(m)
        coll.all_reduce_sum(buf)          # a plain all-reduce in between
        fused_layer.run(m)
        ctx.sync_status()
        for n in ("attn_o", "ffn_down"):
            got = fused_layer.y[(n, m)]
            assert torch.equal(got.view(torch.int32), separate[(n, m)].view(torch.int32)), (n, m, float((got - separate[(n, m)]).abs().max()))
            gathered = [torch.empty_like(got) for _ in range(world)]
            dist.all_gather(gathered, got)
            assert all(torch.equal(gathered[0], t) for t in gathered)
    replay_layer = workloads.capture(lambda: fused_layer.run(8))
    for n in ("attn_o", "ffn_down"):
        fused_layer.y[(n, 8)].fill_(float("nan"))
    for _ in range(3):
        replay_layer()
    ctx.sync_status()
    for n in ("attn_o", "ffn_down"):
        assert torch.equal(fused_layer.y[(n, 8)].view(torch.int32), separate[(n, 8)].view(torch.int32)), n
    # bf16 outputs and more than 16 tokens fall back to projection + all-reduce inside the same call
    k_o, n_o, _ = layer.projs["attn_o"]
    xo = fused_layer.x[(1, 8)]
    yb = torch.empty((8, n_o), dtype=torch.bfloat16, device=dev)
    kern.encode_quantized_matmul(fused_layer.weights["attn_o"], xo, yb, 8, all_reduce=True)
    ctx.sync_status()
    assert torch.allclose(yb.float(), separate[("attn_o", 8)], rtol=2e-2, atol=2e-2 * float(separate[("attn_o", 8)].abs().max()))

    # 4. a wait that runs out: between steps, rank 1 sits one call out.  Rank 0's kernel gives up after about a second,
    #    records its code and returns; the host reads MUSER_CUDA_TIMEOUT; the context still computes.  (Nothing faults:
    #    both processes stay alive and every buffer stays mapped.)
    torch.cuda.synchronize()
    dist.barrier()
    if rank == 0:
        lonely = torch.ones(5120, device=dev)
        coll.all_reduce_sum(lonely)
        try:
            ctx.sync_status()
            raise AssertionError("the wait should have run out")
        except op.MuserCudaError as e:
            assert e.status_name == "TIMEOUT" and "401" in str(e), str(e)
        ctx.sync_status()   # reported once
        assert torch.equal(lonely, torch.ones(5120, device=dev)), "a give-up leaves the buffer as it was"
        layer.all_reduce = None
        layer.launch_group(0, 1)
        ctx.sync_status()
    torch.cuda.synchronize()
    dist.barrier()
    print("TP_WORKER_OK", flush=True)
    sys.stdout.flush()
    os._exit(0)   # (the communicator is out of step after part 4 by design; leave without a teardown that would use it)


if __name__ == "__main__":
    main()
