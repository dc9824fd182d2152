"""Expert parameter container and the grouped SwiGLU expert computation.

`SparseMLPv2` keeps the reference's parameter layout
(megablocks_utils/sparse_mlp2.py:22-36): `w1`, `w2`, `w3`, each
`[experts_per_rank * ffn_per_rank, hidden]`, expert-major on dim 0, with `w2`
stored transposed (megablocks_utils/shard_moe_utils.py:154-157).  The forward is
`(silu(x w1^T) * (x w3^T)) w2` per expert (megablocks_utils/sparse_mlp2.py:69-90),
computed here by one grouped-GEMM family on block-padded row groups instead of
block-sparse SDD/DSD products.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn

from .. import ops
from ..ops.reference import scale_gradient  # noqa: F401  (re-exported)
from ..config import MoEArguments


def experts_per_rank(args: MoEArguments) -> int:
    ep = args.expert_parallel_group.size() if (args.moe_expert_model_parallelism and args.expert_parallel_group is not None) else 1
    assert args.moe_num_experts % ep == 0, "number of experts must be divisible by the expert-parallel size"
    return args.moe_num_experts // ep


def features_per_rank(args: MoEArguments) -> int:
    assert args.ffn_hidden_size % args.tensor_parallel_size == 0
    return args.ffn_hidden_size // args.tensor_parallel_size


class SparseMLPv2(nn.Module):
    def __init__(self, args: MoEArguments):
        super().__init__()
        self.args = args
        self.experts_per_rank = experts_per_rank(args)
        self.features_per_rank = features_per_rank(args)
        rows = self.experts_per_rank * self.features_per_rank
        kw = dict(device=args.device, dtype=args.dtype)
        self.w1 = nn.Parameter(torch.empty(rows, args.hidden_size, **kw))
        self.w2 = nn.Parameter(torch.empty(rows, args.hidden_size, **kw))
        self.w3 = nn.Parameter(torch.empty(rows, args.hidden_size, **kw))
        if self.w1.device.type != "meta":
            for w in (self.w1, self.w2, self.w3):
                nn.init.normal_(w, mean=0.0, std=args.init_std)
        # Each expert sees the tokens of every expert-parallel peer, so its summed
        # gradient is divided by the EP size (megablocks_utils/sparse_mlp2.py:60-67).
        ep = args.expert_parallel_group.size() if (args.moe_expert_model_parallelism and args.expert_parallel_group is not None) else 1
        self.gradient_scale: Optional[float] = (1.0 / ep) if ep > 1 else None
        # name -> (A [E_l, in, r], B [E_l, r, out], r, alpha, hidden, ffn); filled by the LoRA wrapper
        self._lora_pointers: dict = {}

    def weight_views(self):
        E, Fr, H = self.experts_per_rank, self.features_per_rank, self.args.hidden_size
        return self.w1.view(E, Fr, H), self.w2.view(E, Fr, H), self.w3.view(E, Fr, H)

    def lora_views(self):
        if not self._lora_pointers:
            return None
        return {name: (A, B, alpha / r) for name, (A, B, r, alpha, _, _) in self._lora_pointers.items()}

    def call_args(self, xg: torch.Tensor):
        """(w1, w2, w3 views, LoRA dict, weight-gradient scale, direct-accumulation buffers) for one call."""
        w1, w2, w3 = self.weight_views()
        wgrad_out = None
        # (only for weights this module owns: when the experts are sharded like dense parameters the
        #  attributes are views of a gathered buffer and their gradients go through the flat reduction)
        if (xg.is_cuda and ops.get_backend() == "native" and torch.is_grad_enabled() and self.w1.requires_grad
                and isinstance(self.w1, nn.Parameter)):
            E, Fr, H = self.experts_per_rank, self.features_per_rank, self.args.hidden_size
            for w in (self.w1, self.w2, self.w3):
                if w.grad is None:
                    w.grad = torch.zeros_like(w)
            wgrad_out = tuple(w.grad.view(E, Fr, H) for w in (self.w1, self.w2, self.w3))
        return w1, w2, w3, self.lora_views(), self.gradient_scale or 1.0, wgrad_out

    def forward(self, xg: torch.Tensor, plan) -> torch.Tensor:
        """xg: block-padded expert-grouped rows [R, hidden]; returns rows of the same layout."""
        w1, w2, w3, lora, scale, wgrad_out = self.call_args(xg)
        return ops.grouped_swiglu_mlp(xg, w1, w2, w3, plan, lora, wgrad_scale=scale, wgrad_out=wgrad_out)
