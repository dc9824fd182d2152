"""AdamW over flat shards and local expert tensors.

The reference builds `torch.optim.AdamW` on bf16 (sharded) parameters
(train_accelerate_fsdp2.py:320), so the moments are bf16 and there are no fp32
master weights.  This optimizer keeps that storage convention by default
(`state_dtype=None` -> parameter dtype), does the update math in fp32, and on
CUDA runs one multi-tensor kernel over all parameters per step.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..ops import reference


class FusedAdamW(torch.optim.Optimizer):
    def __init__(self, params, lr: float = 1e-5, betas=(0.9, 0.999), eps: float = 1e-8,
                 weight_decay: float = 0.01, state_dtype: Optional[torch.dtype] = None):
        defaults = dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay)
        super().__init__(params, defaults)
        self.state_dtype = state_dtype
        self.grad_scale = 1.0  # folded into the update (used by gradient clipping)

    @torch.no_grad()
    def step(self, closure=None):
        loss = closure() if closure is not None else None
        for group in self.param_groups:
            b1, b2 = group["betas"]
            ps, gs, ms, vs = [], [], [], []
            step = None
            for p in group["params"]:
                if p.grad is None:
                    continue
                st = self.state[p]
                if not st:
                    dt = self.state_dtype or p.dtype
                    st["step"] = 0
                    st["exp_avg"] = torch.zeros_like(p, dtype=dt)
                    st["exp_avg_sq"] = torch.zeros_like(p, dtype=dt)
                st["step"] += 1
                step = st["step"]
                ps.append(p.data); gs.append(p.grad); ms.append(st["exp_avg"]); vs.append(st["exp_avg_sq"])
            if not ps:
                continue
            from .. import ops as _ops
            if ps[0].is_cuda and _ops.get_backend() == "native":
                from ..ops import cuda_ops
                cuda_ops.adamw_multi(ps, gs, ms, vs, group["lr"], b1, b2, group["eps"],
                                     group["weight_decay"], step, self.grad_scale)
            else:
                for p, g, m, v in zip(ps, gs, ms, vs):
                    reference.adamw_step(p, g, m, v, group["lr"], b1, b2, group["eps"],
                                         group["weight_decay"], step, self.grad_scale)
        self.grad_scale = 1.0
        return loss
