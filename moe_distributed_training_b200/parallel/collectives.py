"""Flat-buffer collectives used by the parameter sharding layer.

Two transports: `torch.distributed` (NCCL on GPUs, gloo on CPU; gloo has no
reduce-scatter, so it is stated as all-reduce + slice there) and, for CUDA
buffers that live in symmetric memory, this framework's own peer-memory kernels
(`parallel.symm`), which read the peers' buffers over NVLink directly and fuse
the scale / cast / accumulate that otherwise follow the collective.
"""
from __future__ import annotations


import torch
import torch.distributed as dist


def group_size(group) -> int:
    return dist.get_world_size(group) if (dist.is_available() and dist.is_initialized() and group is not None) else 1


def group_rank(group) -> int:
    return dist.get_rank(group) if (dist.is_available() and dist.is_initialized() and group is not None) else 0


def all_gather_flat(out_full: torch.Tensor, shard: torch.Tensor, group) -> None:
    """out_full[r*n:(r+1)*n] = shard of rank r."""
    ws = group_size(group)
    if ws == 1:
        if out_full.data_ptr() != shard.data_ptr():
            out_full.copy_(shard)
        return
    dist.all_gather_into_tensor(out_full, shard.contiguous(), group=group)


def reduce_scatter_flat(out_shard: torch.Tensor, full: torch.Tensor, group, scale: float = 1.0,
                        accumulate: bool = False) -> None:
    """out_shard (+)= scale * sum_r full_r[my slice]."""
    ws = group_size(group)
    n = out_shard.numel()
    if ws == 1:
        piece = full[:n]
    elif full.is_cuda:
        piece = torch.empty(n, dtype=full.dtype, device=full.device)
        dist.reduce_scatter_tensor(piece, full, op=dist.ReduceOp.SUM, group=group)
    else:
        tmp = full.clone()
        dist.all_reduce(tmp, group=group)
        r = group_rank(group)
        piece = tmp[r * n:(r + 1) * n]
    if accumulate:
        out_shard.add_(piece.to(out_shard.dtype), alpha=scale)
    else:
        out_shard.copy_(piece.to(out_shard.dtype) * scale if scale != 1.0 else piece)


def all_reduce_flat(buf: torch.Tensor, group, scale: float = 1.0) -> None:
    if group_size(group) > 1:
        dist.all_reduce(buf, group=group)
    if scale != 1.0:
        buf.mul_(scale)
