"""Host logic of the tensor-parallel split, on two CPU ranks over gloo (no GPU, no CUDA library calls).

Each rank dequantises the stored weights with the oracle, keeps the rows / inputs its ShardPlan assigns, multiplies
in f64, and the row-parallel partial sums meet in tp.all_reduce_sum.  The sharded layer must reproduce the
unsharded oracle result: column-parallel outputs exactly (they are the same dot products), row-parallel ones
to summation-order accuracy.
"""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from muser_b200 import synth, tp
from oracle import oracle as O

SHAPES = {"attn_q": (512, 64, O.Q4_K), "attn_v": (512, 32, O.Q6_K), "attn_o": (512, 48, O.Q4_K),
          "ffn_down": (1024, 32, O.Q6_K)}


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank: int, world: int, port: int, out_dir: str):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    plan = tp.ShardPlan(rank, world)
    results = {}
    for i, (name, (n_in, n_out, dtype)) in enumerate(SHAPES.items()):
        raw = synth.quantize_kquant(synth.normal_weights(n_out, n_in, seed=0, stream=i), dtype).numpy()
        w = O.dequant_blocks(dtype, raw).reshape(n_out, n_in).astype(np.float64)
        x = synth.normal_activations(3, n_in, seed=0, stream=100 + i).float().numpy().astype(np.float64)
        k_in, k_out = plan.local_shape(name, n_in, n_out, dtype)
        ws = w[plan.output_slice(name, n_out), plan.input_slice(name, n_in)]
        assert ws.shape == (k_out, k_in)
        y = torch.from_numpy(x[:, plan.input_slice(name, n_in)] @ ws.T)
        if plan.needs_all_reduce(name):
            tp.all_reduce_sum(y)
        else:  # column-parallel: gather the row slices to compare with the full result
            parts = [torch.empty_like(y) for _ in range(world)]
            dist.all_gather(parts, y)
            y = torch.cat(parts, dim=1)
        results[name] = y.numpy()
    if rank == 0:
        np.savez(os.path.join(out_dir, "tp.npz"), **results)
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_layer_matches_unsharded_oracle(tmp_path):
    world = 2
    mp.spawn(_rank_main, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    got = np.load(tmp_path / "tp.npz")
    for i, (name, (n_in, n_out, dtype)) in enumerate(SHAPES.items()):
        raw = synth.quantize_kquant(synth.normal_weights(n_out, n_in, seed=0, stream=i), dtype).numpy()
        x = synth.normal_activations(3, n_in, seed=0, stream=100 + i).float().numpy()
        want = O.matmul(O.TensorView(raw, dtype, n_in, n_out), x)
        rel = np.linalg.norm(got[name] - want) / np.linalg.norm(want)
        assert rel < 1e-5, (name, rel)


def test_shard_plan_geometry_and_refusals():
    plan = tp.ShardPlan(3, 8)
    assert plan.shard("attn_q") == (3, 8, tp.SHARD_ROWS) and plan.shard("ffn_down") == (3, 8, tp.SHARD_K)
    assert tp.ShardPlan(0, 1).shard("attn_q") is None
    # the synthetic layer at 8-way: whole heads per rank, K shards of 2.5 and 13.5 super-blocks
    assert plan.local_shape("attn_q", 5120, 5120, O.Q4_K) == (5120, 640)
    assert plan.local_shape("attn_k", 5120, 1024, O.Q4_K) == (5120, 128)
    assert plan.local_shape("attn_o", 5120, 5120, O.Q4_K) == (640, 5120)
    assert plan.local_shape("ffn_down", 27648, 5120, O.Q6_K) == (3456, 5120)
    assert plan.input_slice("ffn_down", 27648) == slice(3 * 3456, 4 * 3456)
    assert plan.output_slice("ffn_gate", 27648) == slice(3 * 3456, 4 * 3456)
    assert plan.needs_all_reduce("attn_o") and not plan.needs_all_reduce("ffn_up")
    with pytest.raises(ValueError):
        tp.ShardPlan(0, 3).local_shape("attn_q", 5120, 5120, O.Q4_K)      # 5120 rows / 3
    with pytest.raises(ValueError):
        tp.ShardPlan(0, 5).local_shape("attn_o", 5120 - 256, 5120, O.NVFP4)  # 972.8-element K shard
