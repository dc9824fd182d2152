"""Global gradient norm and clipping for a model whose parameters are sharded three ways.

Dense flat shards are disjoint over the shard group, expert tensors are disjoint
over the expert-parallel group, router weights are replicated.  The reference
calls `accelerator.clip_grad_norm_` (train_accelerate_fsdp2.py:426-436), after the
optimizer step, so there it only logs; here the scale can be folded into the
fused optimizer step (`optimizer.grad_scale`) so that clipping costs no extra
pass over the gradients.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from ..parallel import collectives as coll


def global_grad_norm(model, shard_group=None, ep_group=None) -> torch.Tensor:
    dev = next(model.parameters()).device
    sq = torch.zeros(3, dtype=torch.float32, device=dev)  # dense shards, experts, replicated
    flat_ids = {id(p) for p in getattr(model, "_flat_shards", [])}
    from .. import ops
    native = dev.type == "cuda" and ops.get_backend() == "native"
    for p in model.parameters():
        if p.grad is None:
            continue
        slot = 0 if id(p) in flat_ids else (1 if getattr(p, "_is_expert_param", False) else 2)
        g = p.grad
        if native and g.is_contiguous() and g.dtype in (torch.bfloat16, torch.float32):
            # one vectorised pass that adds the sum of squares into the slot; no fp32 copy of the gradient
            ops._cuda().ext.sumsq(g, sq[slot:slot + 1])
        else:
            sq[slot] += g.float().pow(2).sum()
    if coll.group_size(shard_group) > 1:
        t = sq[0:1].clone(); dist.all_reduce(t, group=shard_group); sq[0] = t[0]
    if coll.group_size(ep_group) > 1:
        t = sq[1:2].clone(); dist.all_reduce(t, group=ep_group); sq[1] = t[0]
    return sq.sum().sqrt()


def clip_grad_norm_(model, max_norm: float, shard_group=None, ep_group=None, optimizer=None) -> torch.Tensor:
    norm = global_grad_norm(model, shard_group, ep_group)
    coef = (max_norm / (norm + 1e-6)).clamp(max=1.0)
    if optimizer is not None and hasattr(optimizer, "grad_scale"):
        optimizer.grad_scale = float(coef)  # one host read per optimizer step
    else:
        for p in model.parameters():
            if p.grad is not None:
                p.grad.mul_(coef.to(p.grad.dtype))
    return norm
