"""Learned top-k router.

Behaviour of the reference's patched `LearnedRouter.forward`
(megablocks_utils/config_utils.py:255-284): linear -> softmax over all experts
-> top-k -> divide by the p-norm of the selected weights (p=1 when
`moe_normalize_expert_weights` is True) -> optional uniform assignment.
The parameter is named `layer.weight` so that the module path is
`router.layer.weight` (megablocks_utils/shard_moe_utils.py:23).
"""
from __future__ import annotations

import torch
import torch.nn as nn

from .. import ops
from ..config import MoEArguments


class LearnedRouter(nn.Module):
    def __init__(self, args: MoEArguments):
        super().__init__()
        self.args = args
        self.layer = nn.Linear(args.hidden_size, args.moe_num_experts, bias=False,
                               dtype=args.dtype, device=args.device)
        if self.layer.weight.device.type != "meta":
            nn.init.normal_(self.layer.weight, mean=0.0, std=args.init_std)

    def forward(self, x: torch.Tensor):
        x2d = x.reshape(-1, x.shape[-1])
        want_stats = self.args.moe_loss_weight > 0
        out = ops.router(
            x2d, self.layer.weight, self.args.moe_top_k,
            normalize=self.args.moe_normalize_expert_weights,
            jitter_eps=self.args.moe_jitter_eps, training=self.training, with_stats=want_stats)
        scores, weights, idx = out[:3]
        # per-expert slot counts and score sums of this call (only kept when the load-balancing loss is on)
        self.last_stats = out[3] if want_stats else None
        if self.args.uniform_expert_assignment:
            n = idx.numel()
            idx = (torch.arange(n, device=idx.device, dtype=torch.int32) % self.args.moe_num_experts).view_as(idx)
        return scores, weights, idx
