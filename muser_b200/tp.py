"""Tensor-parallel split of one decoder layer's projections across the GPUs of one box.

The reference runs one accelerator and refuses tensor parallelism
(scripts/gx10/vllm/muser_vllm/connector.py:119-120); this module is new.  Output rows of a
projection are independent, so q, k, v, gate and up are column-parallel (each rank keeps
n_out / world rows, no communication); o_proj and down_proj consume those sharded
activations, so they are row-parallel (each rank keeps n_in / world inputs) and their partial
sums meet in one all-reduce per projection.  One process per GPU; NCCL through
torch.distributed on the box, gloo for the CPU tests of this host logic.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.distributed as dist

SHARD_NONE, SHARD_ROWS, SHARD_K = 0, 1, 2

# projection -> axis it is split on
LAYER_AXES = {
    "attn_q": SHARD_ROWS, "attn_k": SHARD_ROWS, "attn_v": SHARD_ROWS, "attn_o": SHARD_K,
    "ffn_gate": SHARD_ROWS, "ffn_up": SHARD_ROWS, "ffn_down": SHARD_K,
}
# granularity (elements) a K shard must respect per weight dtype: Q4_K sub-block, Q6_K sub-block, NVFP4 scale tile
K_GRANULARITY = {12: 32, 14: 16, 1000: 64}


@dataclass(frozen=True)
class ShardPlan:
    rank: int
    world: int

    def shard(self, name: str):
        """(rank, world, axis) for muser_cuda_weight_repack, or None when unsharded."""
        if self.world == 1:
            return None
        return (self.rank, self.world, LAYER_AXES[name])

    def local_shape(self, name: str, n_in: int, n_out: int, dtype: int) -> tuple[int, int]:
        """(n_in, n_out) of this rank's shard; raises when the split is not whole."""
        if self.world == 1:
            return n_in, n_out
        if LAYER_AXES[name] == SHARD_ROWS:
            if n_out % self.world:
                raise ValueError(f"{name}: n_out {n_out} is not divisible by {self.world}")
            return n_in, n_out // self.world
        if n_in % self.world or (n_in // self.world) % K_GRANULARITY[dtype]:
            raise ValueError(f"{name}: a K shard of {n_in}/{self.world} is not a whole number of sub-blocks")
        return n_in // self.world, n_out

    def input_slice(self, name: str, n_in: int) -> slice:
        """Which input features this rank's shard of `name` consumes."""
        if self.world == 1 or LAYER_AXES[name] == SHARD_ROWS:
            return slice(0, n_in)
        step = n_in // self.world
        return slice(self.rank * step, (self.rank + 1) * step)

    def output_slice(self, name: str, n_out: int) -> slice:
        if self.world == 1 or LAYER_AXES[name] == SHARD_K:
            return slice(0, n_out)
        step = n_out // self.world
        return slice(self.rank * step, (self.rank + 1) * step)

    def needs_all_reduce(self, name: str) -> bool:
        return self.world > 1 and LAYER_AXES[name] == SHARD_K


class Collective:
    """The library's own all-reduce for one context (muser_cuda_ctx_comm_init + muser_cuda_all_reduce): rank 0 makes
    the id, torch.distributed only carries its 128 bytes to the other ranks, and every later sum runs inside the
    library on the caller's stream: a one-shot exchange over peer memory for decode-sized payloads, NCCL above."""

    def __init__(self, ctx, rank: int, world: int, group=None):
        import ctypes as C

        from . import _lib
        self.ctx, self.rank, self.world, self._L = ctx, rank, world, _lib.lib
        ident = torch.zeros(128, dtype=torch.uint8)
        if rank == 0:
            buf = (C.c_uint8 * 128)()
            st = self._L.muser_cuda_comm_unique_id(buf, 128)
            if st != 0:
                raise _lib.MuserCudaError(st, (self._L.muser_cuda_last_error(None) or b"").decode())
            ident = torch.tensor(list(buf), dtype=torch.uint8)
        dev = torch.device("cuda", ctx.device)
        carrier = ident.to(dev) if dist.get_backend(group) == "nccl" else ident
        dist.broadcast(carrier, src=0, group=group)
        self._id = bytes(carrier.cpu().tolist())
        stream = torch.cuda.current_stream(dev).cuda_stream
        ctx.check(self._L.muser_cuda_ctx_comm_init(ctx._h, self._id, rank, world, stream))
        self.oneshot = bool(self._L.muser_cuda_ctx_comm_has_oneshot(ctx._h))
        self.kind = ("library: one-shot peer exchange up to 1.5 MiB of f32, ncclAllReduce above" if self.oneshot
                     else "library: ncclAllReduce (peer buffers could not be mapped)")

    def all_reduce_sum(self, partial: torch.Tensor) -> torch.Tensor:
        from .operator import _TORCH_DTYPE
        stream = torch.cuda.current_stream(partial.device).cuda_stream
        self.ctx.check(self._L.muser_cuda_all_reduce(self.ctx._h, partial.data_ptr(), partial.numel(), _TORCH_DTYPE[partial.dtype], stream))
        return partial


def all_reduce_sum(partial: torch.Tensor, group=None) -> torch.Tensor:
    """Sum the row-parallel partial outputs in place across ranks (NCCL over NVLink on the box)."""
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(partial, op=dist.ReduceOp.SUM, group=group)
    return partial
