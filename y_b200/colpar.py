"""Column-parallel (N-sharded) use of the FP8 GEMM across the GPUs of one node.

Rank r owns the weight columns [r*N_s, (r+1)*N_s) as a K-major e4m3 shard; the
activations are replicated and every rank runs the RMSNorm->e4m3 prologue itself
(cheaper than a broadcast). The data path has no collective. Two exchanges exist
around it: one scalar all-reduce(MAX) of the weight amax when the shards are
quantised, so the sharded result is bit-identical to the unsharded one, and an
optional all-gather of the bf16 output shards. Works on any torch.distributed
backend (NCCL on GPUs; gloo in the CPU tests of the host logic).
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def shard_range(n_total: int, world: int, rank: int, multiple: int = 16) -> tuple[int, int]:
    """Column range of `rank`. Shards are equal and a multiple of `multiple` columns
    (16 keeps rows of every shard 16-byte aligned for any element type)."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"bad rank {rank} of {world}")
    if n_total % world != 0:
        raise ValueError(f"N={n_total} does not divide over {world} ranks")
    n_s = n_total // world
    if n_s % multiple != 0:
        raise ValueError(f"shard width {n_s} is not a multiple of {multiple}")
    return rank * n_s, (rank + 1) * n_s


def agree_amax(local_amax: torch.Tensor, group=None) -> torch.Tensor:
    """Global max of the per-shard amax (in place); one scale for the whole weight."""
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(local_amax, op=dist.ReduceOp.MAX, group=group)
    return local_amax


def gather_columns(c_local: torch.Tensor, out: torch.Tensor | None = None, group=None) -> torch.Tensor:
    """All-gather of the output shards. Returns [world, M, N_s] (rank-major: the
    layout a contiguous all-gather produces; `assemble` gives row-major [M, N])."""
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    m, n_s = c_local.shape
    if out is None:
        out = torch.empty((world, m, n_s), dtype=c_local.dtype, device=c_local.device)
    if world == 1:
        out[0].copy_(c_local)
        return out
    if out.shape != (world, m, n_s):
        raise ValueError(f"gather buffer has shape {tuple(out.shape)}, want {(world, m, n_s)}")
    dist.all_gather_into_tensor(out.view(world * m, n_s), c_local.contiguous(), group=group)
    return out


def assemble(gathered: torch.Tensor) -> torch.Tensor:
    """[world, M, N_s] -> row-major [M, world * N_s]."""
    world, m, n_s = gathered.shape
    return gathered.permute(1, 0, 2).reshape(m, world * n_s)
